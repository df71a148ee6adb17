// Mapped max / avg pooling, their adjoints, and resample gather / scatter.
//
// One launch covers the whole batch (the reference launches once per batch element,
// src/nn/cuda/mapped_max_pooling_layer.cu:31-35).  Element order follows the memory layout so
// that consecutive threads write consecutive addresses.  Semantics per element:
//   max pool   include/nn/common/mapped_max_pool.h:14-58   (+weighted :80-130)
//   max unpool include/nn/common/mapped_max_pool.h:61-78   (+weighted :132-169)
//   avg pool   include/nn/common/mapped_avg_pool.h:14-70   (+weighted :72-143)
//   resample   include/nn/common/resample.h:11-103
#include "common.cuh"

namespace mc {

enum { OP_GATHER = 0, OP_AVG = 1, OP_MAX = 2 };

// pool_fast.cu: bandwidth-oriented kernels for unweighted nearest (K in {1,4,7,9}) and single-tap
// bilinear maps; returns false when the generic kernel below has to take the call.
bool sample_fwd_fast(const mc_desc* d, int op, const void* x, const void* map, void* y, int64_t* idx,
                     cudaStream_t st, int* rc);

struct SampleArgs {
  const void* x;
  const void* map;
  const void* iw;
  void* y;
  int64_t* idx;
  int B, C, IH, IW, K, P, interp, layout;
  long npix_in, npix_out;
};

// Weighted sample of one tap: sum_i iw_i * interp(point i)   (include/core/resample.h:145-162)
template <typename T, typename CT, typename MT>
__device__ __forceinline__ CT sample_tap(const T* plane, long sp, const MT* m, const MT* wts, int P,
                                         int H, int W, int interp) {
  Tap<CT> t;
  if (P == 0) {
    decode_tap<MT, CT>(m[0], m[1], H, W, interp, t);
    return tap_gather<T, CT>(plane, sp, t);
  }
  CT acc = CT(0);
  for (int i = 0; i < P; ++i) {
    decode_tap<MT, CT>(m[2 * i], m[2 * i + 1], H, W, interp, t);
    acc = add_rn(acc, mul_rn((CT)wts[i], tap_gather<T, CT>(plane, sp, t)));
  }
  return acc;
}

template <typename T, int OP>
__global__ void __launch_bounds__(256) sample_fwd_kernel(SampleArgs a) {
  typedef typename Traits<T>::CT CT;
  typedef typename Traits<T>::MT MT;
  const T* x = (const T*)a.x;
  const MT* map = (const MT*)a.map;
  const MT* iw = (const MT*)a.iw;
  T* y = (T*)a.y;
  const Strides xs = make_strides(a.layout, a.C, a.npix_in);
  const Strides ys = make_strides(a.layout, a.C, a.npix_out);
  const long total = (long)a.B * a.C * a.npix_out;
  const int pp = a.P > 0 ? a.P : 1;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total;
       i += (long)gridDim.x * blockDim.x) {
    int b, c;
    long p;
    split_index(i, a.layout, a.C, a.npix_out, b, c, p);
    const T* plane = x + b * xs.b + c * xs.c;
    const long tap0 = p * a.K * pp;  // index of this location's first (tap, point)
    CT acc = OP == OP_MAX ? (CT)(-FLT_MAX) : CT(0);
    long best = -1;
    for (int k = 0; k < a.K; ++k) {
      const long e = tap0 + (long)k * pp;
      const CT v = sample_tap<T, CT, MT>(plane, xs.p, map + 2 * e, iw ? iw + e : nullptr, a.P,
                                         a.IH, a.IW, a.interp);
      if (OP == OP_MAX) {
        if (v > acc) { acc = v; best = 2 * e; }
      } else if (OP == OP_AVG) {
        acc = add_rn(acc, v);
      } else {
        acc = v;
      }
    }
    if (OP == OP_AVG) acc = div_rn(acc, (CT)a.K);
    const long o = b * ys.b + c * ys.c + p * ys.p;
    stv(y + o, acc);
    if (OP == OP_MAX) a.idx[o] = best;
  }
}

// ---- adjoints (scatter) ------------------------------------------------------------------

struct ScatterArgs {
  const void* g;       // values on the map grid (B, C, npix_grid)
  const int64_t* idx;  // max-unpool only
  const void* map;
  const void* iw;
  void* out;  // accumulation target in CT (B, C, npix_img), pre-zeroed
  int B, C, IH, IW, K, P, interp, layout;
  long npix_img, npix_grid;
};

template <typename CT, typename MT>
__device__ __forceinline__ void scatter_tap(CT* plane, long sp, const MT* m, const MT* wts, int P,
                                            int H, int W, int interp, CT value) {
  Tap<CT> t;
  if (P == 0) {
    decode_tap<MT, CT>(m[0], m[1], H, W, interp, t);
    tap_scatter<CT>(plane, sp, t, value);
    return;
  }
  for (int i = 0; i < P; ++i) {
    decode_tap<MT, CT>(m[2 * i], m[2 * i + 1], H, W, interp, t);
    tap_scatter<CT>(plane, sp, t, mul_rn((CT)wts[i], value));
  }
}

// OP_GATHER here means "adjoint of gather" (resample scatter, K = 1).
template <typename T, int OP>
__global__ void __launch_bounds__(256) sample_bwd_kernel(ScatterArgs a) {
  typedef typename Traits<T>::CT CT;
  typedef typename Traits<T>::MT MT;
  const T* g = (const T*)a.g;
  const MT* map = (const MT*)a.map;
  const MT* iw = (const MT*)a.iw;
  CT* out = (CT*)a.out;
  const Strides gs = make_strides(a.layout, a.C, a.npix_grid);
  const Strides os = make_strides(a.layout, a.C, a.npix_img);
  const long total = (long)a.B * a.C * a.npix_grid;
  const int pp = a.P > 0 ? a.P : 1;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total;
       i += (long)gridDim.x * blockDim.x) {
    int b, c;
    long p;
    split_index(i, a.layout, a.C, a.npix_grid, b, c, p);
    const long o = b * gs.b + c * gs.c + p * gs.p;
    CT* plane = out + b * os.b + c * os.c;
    CT v = (CT)ldv(g + o);
    if (OP == OP_MAX) {
      // the stored offset is read back as a 32-bit int (mapped_max_pool.h:72-73)
      const long off = (long)(int)a.idx[o];
      if (off < 0) continue;
      const long e = off / 2;  // (tap, point) index
      scatter_tap<CT, MT>(plane, os.p, map + off, iw ? iw + e : nullptr, a.P, a.IH, a.IW, a.interp,
                          v);
    } else {
      if (OP == OP_AVG) v = div_rn(v, (CT)a.K);
      const long tap0 = p * a.K * pp;
      for (int k = 0; k < a.K; ++k) {
        const long e = tap0 + (long)k * pp;
        scatter_tap<CT, MT>(plane, os.p, map + 2 * e, iw ? iw + e : nullptr, a.P, a.IH, a.IW,
                            a.interp, v);
      }
    }
  }
}

template <typename T>
__global__ void convert_from_f32_kernel(const float* src, T* dst, long n) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n;
       i += (long)gridDim.x * blockDim.x)
    stv(dst + i, src[i]);
}

static int check_desc(const mc_desc* d, bool need_k1) {
  if (!d) return MC_ERR_BAD_ARG;
  if (d->B <= 0 || d->C_in <= 0 || d->IH <= 0 || d->IW <= 0 || d->OH <= 0 || d->OW <= 0 ||
      d->K <= 0 || d->P < 0)
    return MC_ERR_BAD_ARG;
  if (d->dtype != MC_F32 && d->dtype != MC_F64 && d->dtype != MC_BF16) return MC_ERR_BAD_ARG;
  if (d->layout != MC_NCHW && d->layout != MC_NHWC) return MC_ERR_BAD_ARG;
  if ((long)d->IH * d->IW >= (1L << 31) || (long)d->OH * d->OW * d->K * (d->P ? d->P : 1) >= (1L << 30))
    return MC_ERR_TOO_LARGE;
  if (need_k1 && d->K != 1) return MC_ERR_BAD_ARG;
  return MC_OK;
}

template <int OP>
static int launch_fwd(const mc_desc* d, const void* x, const void* map, const void* iw, void* y,
                      int64_t* idx, cudaStream_t st) {
  SampleArgs a;
  a.x = x; a.map = map; a.iw = iw; a.y = y; a.idx = idx;
  a.B = d->B; a.C = d->C_in; a.IH = d->IH; a.IW = d->IW; a.K = d->K; a.P = d->P;
  a.interp = d->interp; a.layout = d->layout;
  a.npix_in = (long)d->IH * d->IW;
  a.npix_out = (long)d->OH * d->OW;
  int frc = MC_OK;
  if (sample_fwd_fast(d, OP, x, map, y, idx, st, &frc)) return frc;  // decode-once kernels
  const long total = (long)a.B * a.C * a.npix_out;
  const int grid = grid_for(total, 256);
  if (d->dtype == MC_F32) sample_fwd_kernel<float, OP><<<grid, 256, 0, st>>>(a), MC_COUNT(1);
  else if (d->dtype == MC_F64) sample_fwd_kernel<double, OP><<<grid, 256, 0, st>>>(a), MC_COUNT(1);
  else sample_fwd_kernel<bf16, OP><<<grid, 256, 0, st>>>(a), MC_COUNT(1);
  MC_CHECK_LAUNCH();
  return MC_OK;
}

template <int OP>
static int launch_bwd(const mc_desc* d, const void* g, const int64_t* idx, const void* map,
                      const void* iw, void* out, void* ws, size_t ws_bytes, cudaStream_t st) {
  ScatterArgs a;
  a.g = g; a.idx = idx; a.map = map; a.iw = iw;
  a.B = d->B; a.C = d->C_in; a.IH = d->IH; a.IW = d->IW; a.K = d->K; a.P = d->P;
  a.interp = d->interp; a.layout = d->layout;
  a.npix_img = (long)d->IH * d->IW;
  a.npix_grid = (long)d->OH * d->OW;
  const long nout = (long)a.B * a.C * a.npix_img;
  const long total = (long)a.B * a.C * a.npix_grid;
  const int grid = grid_for(total, 256);
  if (d->dtype == MC_BF16) {
    if (!ws || ws_bytes < (size_t)nout * sizeof(float)) return MC_ERR_WORKSPACE;
    a.out = ws;
    if (cudaMemsetAsync(ws, 0, nout * sizeof(float), st) != cudaSuccess) return MC_ERR_LAUNCH;
    sample_bwd_kernel<bf16, OP><<<grid, 256, 0, st>>>(a), MC_COUNT(1);
    MC_CHECK_LAUNCH();
    convert_from_f32_kernel<bf16><<<grid_for(nout, 256), 256, 0, st>>>((const float*)ws, (bf16*)out, nout), MC_COUNT(1);
  } else if (d->dtype == MC_F32) {
    a.out = out;
    if (cudaMemsetAsync(out, 0, nout * sizeof(float), st) != cudaSuccess) return MC_ERR_LAUNCH;
    sample_bwd_kernel<float, OP><<<grid, 256, 0, st>>>(a), MC_COUNT(1);
  } else {
    a.out = out;
    if (cudaMemsetAsync(out, 0, nout * sizeof(double), st) != cudaSuccess) return MC_ERR_LAUNCH;
    sample_bwd_kernel<double, OP><<<grid, 256, 0, st>>>(a), MC_COUNT(1);
  }
  MC_CHECK_LAUNCH();
  return MC_OK;
}

}  // namespace mc

using namespace mc;

extern "C" {

size_t mc_scatter_workspace_bytes(const mc_desc* d) {
  if (!d || d->dtype != MC_BF16) return 0;
  return (size_t)d->B * d->C_in * d->IH * d->IW * sizeof(float);
}

int mc_pool_max_fwd(const mc_desc* d, const void* x, const void* map, const void* iw, void* y,
                    int64_t* idx, void* stream) {
  int rc = check_desc(d, false);
  if (rc) return rc;
  if (!x || !map || !y || !idx || (d->P > 0 && !iw)) return MC_ERR_BAD_ARG;
  return launch_fwd<OP_MAX>(d, x, map, d->P ? iw : nullptr, y, idx, (cudaStream_t)stream);
}

int mc_pool_avg_fwd(const mc_desc* d, const void* x, const void* map, const void* iw, void* y,
                    void* stream) {
  int rc = check_desc(d, false);
  if (rc) return rc;
  if (!x || !map || !y || (d->P > 0 && !iw)) return MC_ERR_BAD_ARG;
  return launch_fwd<OP_AVG>(d, x, map, d->P ? iw : nullptr, y, nullptr, (cudaStream_t)stream);
}

int mc_resample_gather(const mc_desc* d, const void* x, const void* map, const void* iw, void* y,
                       void* stream) {
  int rc = check_desc(d, true);
  if (rc) return rc;
  if (!x || !map || !y || (d->P > 0 && !iw)) return MC_ERR_BAD_ARG;
  return launch_fwd<OP_GATHER>(d, x, map, d->P ? iw : nullptr, y, nullptr, (cudaStream_t)stream);
}

int mc_pool_max_bwd(const mc_desc* d, const void* gy, const int64_t* idx, const void* map,
                    const void* iw, void* gx, void* ws, size_t ws_bytes, void* stream) {
  int rc = check_desc(d, false);
  if (rc) return rc;
  if (!gy || !idx || !map || !gx || (d->P > 0 && !iw)) return MC_ERR_BAD_ARG;
  return launch_bwd<OP_MAX>(d, gy, idx, map, d->P ? iw : nullptr, gx, ws, ws_bytes,
                            (cudaStream_t)stream);
}

int mc_pool_avg_bwd(const mc_desc* d, const void* gy, const void* map, const void* iw, void* gx,
                    void* ws, size_t ws_bytes, void* stream) {
  int rc = check_desc(d, false);
  if (rc) return rc;
  if (!gy || !map || !gx || (d->P > 0 && !iw)) return MC_ERR_BAD_ARG;
  return launch_bwd<OP_AVG>(d, gy, nullptr, map, d->P ? iw : nullptr, gx, ws, ws_bytes,
                            (cudaStream_t)stream);
}

int mc_resample_scatter(const mc_desc* d, const void* x, const void* map, const void* iw, void* y,
                        void* ws, size_t ws_bytes, void* stream) {
  int rc = check_desc(d, true);
  if (rc) return rc;
  if (!x || !map || !y || (d->P > 0 && !iw)) return MC_ERR_BAD_ARG;
  return launch_bwd<OP_GATHER>(d, x, nullptr, map, d->P ? iw : nullptr, y, ws, ws_bytes,
                               (cudaStream_t)stream);
}

}  // extern "C"
