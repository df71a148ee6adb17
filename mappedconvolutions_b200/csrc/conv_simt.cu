// Generic (any dtype, any layout, weighted or not) mapped convolution kernels on the CUDA cores.
//
// These are the fp32 / fp64 paths (fp32 parity at 1e-5 rules out single-pass tensor-core math)
// and the fallback for shapes the tcgen05 path does not take.  No column buffer is
// materialised: each block interpolates a tile of the im2col matrix into shared memory and
// contracts it on the spot.  Row r = c_in * K + k of that matrix matches the reference's
// include/nn/common/mapped_im2col.h:31 and weight.view(C_out, C_in*K).
//
//   forward  : src/nn/cuda/mapped_convolution_layer.cu:16-73
//   dgrad    : src/nn/cuda/mapped_convolution_layer.cu:75-132   (col2im: mapped_im2col.h:45-78)
//   wgrad    : src/nn/cuda/mapped_convolution_layer.cu:134-193
#include "common.cuh"

namespace mc {

struct ConvArgs {
  const void* x;    // sampled image (B, Cin, IH*IW)            [fwd, wgrad]
  const void* gy;   // tensor on the map grid (B, Cout, OH*OW)  [dgrad, wgrad]
  const void* map;
  const void* iw;
  const void* w;     // (Cout, Cin*K)
  const void* bias;  // fwd: (Cout)
  int relu;          // fwd: clamp the result at zero after the bias
  void* out;         // fwd: y in T; dgrad: accumulation buffer in CT; wgrad: gw in CT
  int B, Cin, Cout, IH, IW, K, P, interp, layout;
  long npix_img, npix_grid;
  int R;  // Cin * K
  long pix_per_split;  // wgrad
};

template <typename T, typename CT, typename MT>
__device__ __forceinline__ CT conv_sample(const T* plane, long sp, const MT* map, const MT* iw,
                                          long e, int P, int H, int W, int interp) {
  Tap<CT> t;
  if (P == 0) {
    decode_tap<MT, CT>(map[2 * e], map[2 * e + 1], H, W, interp, t);
    return tap_gather<T, CT>(plane, sp, t);
  }
  CT acc = CT(0);
  for (int i = 0; i < P; ++i) {
    decode_tap<MT, CT>(map[2 * (e + i)], map[2 * (e + i) + 1], H, W, interp, t);
    acc = add_rn(acc, mul_rn((CT)iw[e + i], tap_gather<T, CT>(plane, sp, t)));
  }
  return acc;
}

constexpr int TP = 64;   // pixels per block tile
constexpr int TCO = 64;  // output channels per block tile
constexpr int RC = 32;   // im2col rows per shared-memory chunk

// ---- forward -----------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) conv_fwd_simt(ConvArgs a) {
  typedef typename Traits<T>::CT CT;
  typedef typename Traits<T>::MT MT;
  __shared__ CT col[RC][TP];
  __shared__ CT wsm[TCO][RC + 1];
  const T* x = (const T*)a.x;
  const T* w = (const T*)a.w;
  const MT* map = (const MT*)a.map;
  const MT* iw = (const MT*)a.iw;
  const Strides xs = make_strides(a.layout, a.Cin, a.npix_img);
  const Strides ys = make_strides(a.layout, a.Cout, a.npix_grid);
  const int tx = threadIdx.x % TP, ty = threadIdx.x / TP;
  const long total_pix = (long)a.B * a.npix_grid;
  const long g0 = (long)blockIdx.x * TP;
  const int co0 = blockIdx.y * TCO;
  const int pp = a.P > 0 ? a.P : 1;
  CT acc[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) acc[j] = CT(0);

  for (int r0 = 0; r0 < a.R; r0 += RC) {
    for (int i = threadIdx.x; i < RC * TP; i += 256) {
      const int r = i / TP, pl = i % TP;
      const int row = r0 + r;
      const long g = g0 + pl;
      CT v = CT(0);
      if (row < a.R && g < total_pix) {
        const int b = (int)(g / a.npix_grid);
        const long p = g % a.npix_grid;
        const int ci = row / a.K, k = row % a.K;
        v = conv_sample<T, CT, MT>(x + b * xs.b + ci * xs.c, xs.p, map, iw, (p * a.K + k) * pp, a.P,
                                   a.IH, a.IW, a.interp);
      }
      col[r][pl] = v;
    }
    for (int i = threadIdx.x; i < TCO * RC; i += 256) {
      const int c = i / RC, r = i % RC;
      wsm[c][r] = (co0 + c < a.Cout && r0 + r < a.R) ? (CT)ldv(w + (long)(co0 + c) * a.R + r0 + r)
                                                      : CT(0);
    }
    __syncthreads();
#pragma unroll 4
    for (int r = 0; r < RC; ++r) {
      const CT v = col[r][tx];
#pragma unroll
      for (int j = 0; j < 16; ++j) acc[j] += wsm[ty * 16 + j][r] * v;
    }
    __syncthreads();
  }
  const long g = g0 + tx;
  if (g >= total_pix) return;
  const int b = (int)(g / a.npix_grid);
  const long p = g % a.npix_grid;
  T* y = (T*)a.out;
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const int co = co0 + ty * 16 + j;
    if (co < a.Cout) {
      CT v = acc[j];
      if (a.bias) v += (CT)ldv((const T*)a.bias + co);
      if (a.relu && v < CT(0)) v = CT(0);
      stv(y + b * ys.b + co * ys.c + p * ys.p, v);
    }
  }
}

// ---- dgrad (col2im of W^T . gy, atomic scatter) -------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) conv_dgrad_simt(ConvArgs a) {
  typedef typename Traits<T>::CT CT;
  typedef typename Traits<T>::MT MT;
  constexpr int CC = 32;  // output-channel chunk
  __shared__ CT gsm[CC][TP];
  __shared__ CT wsm[CC][RC + 1];
  const T* gy = (const T*)a.gy;
  const T* w = (const T*)a.w;
  const MT* map = (const MT*)a.map;
  const MT* iw = (const MT*)a.iw;
  CT* out = (CT*)a.out;
  const Strides gs = make_strides(a.layout, a.Cout, a.npix_grid);
  const Strides os = make_strides(a.layout, a.Cin, a.npix_img);
  const int tx = threadIdx.x % TP, ty = threadIdx.x / TP;
  const long total_pix = (long)a.B * a.npix_grid;
  const long g0 = (long)blockIdx.x * TP;
  const int r0 = blockIdx.y * RC;
  const int pp = a.P > 0 ? a.P : 1;
  CT acc[RC / 4];
#pragma unroll
  for (int j = 0; j < RC / 4; ++j) acc[j] = CT(0);

  for (int c0 = 0; c0 < a.Cout; c0 += CC) {
    for (int i = threadIdx.x; i < CC * TP; i += 256) {
      const int c = i / TP, pl = i % TP;
      const long g = g0 + pl;
      CT v = CT(0);
      if (c0 + c < a.Cout && g < total_pix) {
        const int b = (int)(g / a.npix_grid);
        const long p = g % a.npix_grid;
        v = (CT)ldv(gy + b * gs.b + (c0 + c) * gs.c + p * gs.p);
      }
      gsm[c][pl] = v;
    }
    for (int i = threadIdx.x; i < CC * RC; i += 256) {
      const int c = i / RC, r = i % RC;
      wsm[c][r] = (c0 + c < a.Cout && r0 + r < a.R) ? (CT)ldv(w + (long)(c0 + c) * a.R + r0 + r)
                                                     : CT(0);
    }
    __syncthreads();
#pragma unroll 4
    for (int c = 0; c < CC; ++c) {
      const CT v = gsm[c][tx];
#pragma unroll
      for (int j = 0; j < RC / 4; ++j) acc[j] += wsm[c][ty + 4 * j] * v;
    }
    __syncthreads();
  }
  const long g = g0 + tx;
  if (g >= total_pix) return;
  const int b = (int)(g / a.npix_grid);
  const long p = g % a.npix_grid;
#pragma unroll
  for (int j = 0; j < RC / 4; ++j) {
    const int row = r0 + ty + 4 * j;
    if (row >= a.R) continue;
    const int ci = row / a.K, k = row % a.K;
    CT* plane = out + b * os.b + ci * os.c;
    const long e = (p * a.K + k) * pp;
    Tap<CT> t;
    if (a.P == 0) {
      decode_tap<MT, CT>(map[2 * e], map[2 * e + 1], a.IH, a.IW, a.interp, t);
      tap_scatter<CT>(plane, os.p, t, acc[j]);
    } else {
      for (int i = 0; i < a.P; ++i) {
        decode_tap<MT, CT>(map[2 * (e + i)], map[2 * (e + i) + 1], a.IH, a.IW, a.interp, t);
        tap_scatter<CT>(plane, os.p, t, mul_rn((CT)iw[e + i], acc[j]));
      }
    }
  }
}

// out[b, c, p] = bias[c] (or 0) in CT: the start value of the dgrad accumulation.
template <typename T, typename CT>
__global__ void fill_bias_kernel(CT* out, const T* bias, int layout, int C, long npix, long total) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total;
       i += (long)gridDim.x * blockDim.x) {
    int b, c;
    long p;
    split_index(i, layout, C, npix, b, c, p);
    out[i] = bias ? (CT)ldv(bias + c) : CT(0);
  }
}

__global__ void f32_to_bf16_kernel(const float* src, bf16* dst, long n) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n;
       i += (long)gridDim.x * blockDim.x)
    dst[i] = __float2bfloat16_rn(src[i]);
}

// ---- wgrad -------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) conv_wgrad_simt(ConvArgs a) {
  typedef typename Traits<T>::CT CT;
  typedef typename Traits<T>::MT MT;
  constexpr int PC = 16;  // pixels per chunk
  __shared__ CT gsm[PC][TCO + 1];
  __shared__ CT csm[PC][64 + 1];
  const T* x = (const T*)a.x;
  const T* gy = (const T*)a.gy;
  const MT* map = (const MT*)a.map;
  const MT* iw = (const MT*)a.iw;
  CT* gw = (CT*)a.out;
  const Strides xs = make_strides(a.layout, a.Cin, a.npix_img);
  const Strides gs = make_strides(a.layout, a.Cout, a.npix_grid);
  const int n_rt = (a.R + 63) / 64;
  const int co0 = (blockIdx.x / n_rt) * TCO;
  const int r0 = (blockIdx.x % n_rt) * 64;
  const long total_pix = (long)a.B * a.npix_grid;
  const long gbeg = (long)blockIdx.y * a.pix_per_split;
  long gend = gbeg + a.pix_per_split;
  if (gend > total_pix) gend = total_pix;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  const int pp = a.P > 0 ? a.P : 1;
  CT acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = CT(0);

  for (long g1 = gbeg; g1 < gend; g1 += PC) {
    for (int i = threadIdx.x; i < PC * 64; i += 256) {
      // layout-aware fill order: pixel-fastest for NCHW, channel-fastest for NHWC
      int pl, c;
      if (a.layout == MC_NHWC) { c = i % 64; pl = i / 64; } else { pl = i % PC; c = i / PC; }
      const long g = g1 + pl;
      CT gv = CT(0), cv = CT(0);
      if (g < gend) {
        const int b = (int)(g / a.npix_grid);
        const long p = g % a.npix_grid;
        if (co0 + c < a.Cout) gv = (CT)ldv(gy + b * gs.b + (co0 + c) * gs.c + p * gs.p);
        const int row = r0 + c;
        if (row < a.R) {
          const int ci = row / a.K, k = row % a.K;
          cv = conv_sample<T, CT, MT>(x + b * xs.b + ci * xs.c, xs.p, map, iw, (p * a.K + k) * pp,
                                      a.P, a.IH, a.IW, a.interp);
        }
      }
      gsm[pl][c] = gv;
      csm[pl][c] = cv;
    }
    __syncthreads();
#pragma unroll
    for (int q = 0; q < PC; ++q) {
      CT gv[4], cv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { gv[i] = gsm[q][tx * 4 + i]; cv[i] = csm[q][ty * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] += gv[i] * cv[j];
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int co = co0 + tx * 4 + i, row = r0 + ty * 4 + j;
      if (co < a.Cout && row < a.R) atomicAdd(gw + (long)co * a.R + row, acc[i][j]);
    }
}

// gb[c] = sum over batch and pixels of gy[b, c, p]
template <typename T, typename CT>
__global__ void __launch_bounds__(256) bias_grad_kernel(const T* gy, CT* gb, int layout, int B, int C,
                                                        long npix, long pix_per_split) {
  const int c = blockIdx.x;
  const Strides gs = make_strides(layout, C, npix);
  const long total = (long)B * npix;
  const long beg = (long)blockIdx.y * pix_per_split;
  long end = beg + pix_per_split;
  if (end > total) end = total;
  CT s = CT(0);
  for (long g = beg + threadIdx.x; g < end; g += 256) {
    const int b = (int)(g / npix);
    const long p = g % npix;
    s += (CT)ldv(gy + b * gs.b + c * gs.c + p * gs.p);
  }
  __shared__ CT red[256];
  red[threadIdx.x] = s;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) atomicAdd(gb + c, red[0]);
}

__device__ __forceinline__ float widen(float v) { return v; }
__device__ __forceinline__ double widen(double v) { return v; }
__device__ __forceinline__ float widen(bf16 v) { return __bfloat162float(v); }

// Channels-last variant: a thread owns one 16-byte group of channels and walks the pixels, so a
// warp reads whole rows; the partial sums of the threads that share a channel group are folded in
// shared memory.  NV = channels per 16 bytes.
template <typename T, typename CT, int NV>
__global__ void __launch_bounds__(256) bias_grad_cl_kernel(const T* __restrict__ gy, CT* gb, int C,
                                                           long total, long pix_per_block) {
  const int ng = C / NV;              // channel groups per pixel
  const int lanes = 256 / ng;         // pixels handled side by side (ng <= 256)
  const int cg = threadIdx.x % ng, pl = threadIdx.x / ng;
  const long beg = (long)blockIdx.x * pix_per_block;
  long end = beg + pix_per_block;
  if (end > total) end = total;
  CT s[NV];
#pragma unroll
  for (int j = 0; j < NV; ++j) s[j] = CT(0);
  if (pl < lanes) {
    for (long g = beg + pl; g < end; g += lanes) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(gy + g * C + cg * NV));
      const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
      for (int j = 0; j < NV; ++j) s[j] += (CT)widen(e[j]);
    }
  }
  extern __shared__ unsigned char red_raw[];
  CT* red = reinterpret_cast<CT*>(red_raw);  // [256][NV]
#pragma unroll
  for (int j = 0; j < NV; ++j) red[threadIdx.x * NV + j] = s[j];
  __syncthreads();
  for (int i = threadIdx.x; i < C; i += 256) {
    const int g = i / NV, j = i % NV;
    CT t = CT(0);
    for (int l = 0; l < lanes; ++l) t += red[(l * ng + g) * NV + j];
    atomicAdd(gb + i, t);
  }
}

// ---- host side ---------------------------------------------------------------------------

static int check_conv_desc(const mc_desc* d) {
  if (!d) return MC_ERR_BAD_ARG;
  if (d->B <= 0 || d->C_in <= 0 || d->C_out <= 0 || d->IH <= 0 || d->IW <= 0 || d->OH <= 0 ||
      d->OW <= 0 || d->K <= 0 || d->P < 0)
    return MC_ERR_BAD_ARG;
  if (d->dtype != MC_F32 && d->dtype != MC_F64 && d->dtype != MC_BF16) return MC_ERR_BAD_ARG;
  if (d->layout != MC_NCHW && d->layout != MC_NHWC) return MC_ERR_BAD_ARG;
  if ((long)d->IH * d->IW >= (1L << 31) ||
      (long)d->OH * d->OW * d->K * (d->P ? d->P : 1) >= (1L << 30) ||
      (long)d->C_in * d->K >= (1L << 24))
    return MC_ERR_TOO_LARGE;
  return MC_OK;
}

static ConvArgs make_args(const mc_desc* d) {
  ConvArgs a;
  a.x = a.gy = a.map = a.iw = a.w = a.bias = nullptr;
  a.relu = 0;
  a.out = nullptr;
  a.B = d->B; a.Cin = d->C_in; a.Cout = d->C_out; a.IH = d->IH; a.IW = d->IW; a.K = d->K;
  a.P = d->P; a.interp = d->interp; a.layout = d->layout;
  a.npix_img = (long)d->IH * d->IW;
  a.npix_grid = (long)d->OH * d->OW;
  a.R = d->C_in * d->K;
  a.pix_per_split = 0;
  return a;
}

int conv_fwd_simt_launch(const mc_desc* d, const void* x, const void* map, const void* iw,
                         const void* w, const void* bias, void* y, cudaStream_t st) {
  ConvArgs a = make_args(d);
  a.x = x; a.map = map; a.iw = d->P ? iw : nullptr; a.w = w; a.bias = bias; a.out = y;
  a.relu = (d->flags & MC_FLAG_RELU) ? 1 : 0;
  const long total_pix = (long)d->B * a.npix_grid;
  dim3 grid((unsigned)((total_pix + TP - 1) / TP), (unsigned)((d->C_out + TCO - 1) / TCO));
  if (d->dtype == MC_F32) conv_fwd_simt<float><<<grid, 256, 0, st>>>(a), MC_COUNT(1);
  else if (d->dtype == MC_F64) conv_fwd_simt<double><<<grid, 256, 0, st>>>(a), MC_COUNT(1);
  else conv_fwd_simt<bf16><<<grid, 256, 0, st>>>(a), MC_COUNT(1);
  MC_CHECK_LAUNCH();
  return MC_OK;
}

size_t conv_dgrad_simt_ws(const mc_desc* d) {
  return d->dtype == MC_BF16 ? (size_t)d->B * d->C_in * d->IH * d->IW * sizeof(float) : 0;
}

int conv_dgrad_simt_launch(const mc_desc* d, const void* gy, const void* map, const void* iw,
                           const void* w, const void* bias_out, void* gx, void* ws, size_t ws_bytes,
                           cudaStream_t st) {
  ConvArgs a = make_args(d);
  a.gy = gy; a.map = map; a.iw = d->P ? iw : nullptr; a.w = w;
  const long nout = (long)d->B * d->C_in * a.npix_img;
  const long total_pix = (long)d->B * a.npix_grid;
  dim3 grid((unsigned)((total_pix + TP - 1) / TP), (unsigned)((a.R + RC - 1) / RC));
  const int fgrid = grid_for(nout, 256);
  if (d->dtype == MC_F32) {
    a.out = gx;
    fill_bias_kernel<float, float><<<fgrid, 256, 0, st>>>((float*)gx, (const float*)bias_out, d->layout, d->C_in, a.npix_img, nout), MC_COUNT(1);
    conv_dgrad_simt<float><<<grid, 256, 0, st>>>(a), MC_COUNT(1);
  } else if (d->dtype == MC_F64) {
    a.out = gx;
    fill_bias_kernel<double, double><<<fgrid, 256, 0, st>>>((double*)gx, (const double*)bias_out, d->layout, d->C_in, a.npix_img, nout), MC_COUNT(1);
    conv_dgrad_simt<double><<<grid, 256, 0, st>>>(a), MC_COUNT(1);
  } else {
    if (!ws || ws_bytes < (size_t)nout * sizeof(float)) return MC_ERR_WORKSPACE;
    a.out = ws;
    fill_bias_kernel<bf16, float><<<fgrid, 256, 0, st>>>((float*)ws, (const bf16*)bias_out, d->layout, d->C_in, a.npix_img, nout), MC_COUNT(1);
    conv_dgrad_simt<bf16><<<grid, 256, 0, st>>>(a), MC_COUNT(1);
    f32_to_bf16_kernel<<<fgrid, 256, 0, st>>>((const float*)ws, (bf16*)gx, nout), MC_COUNT(1);
  }
  MC_CHECK_LAUNCH();
  return MC_OK;
}

int bias_grad_launch(const mc_desc* d, const void* gy, void* gb, cudaStream_t st) {
  const long npix = (long)d->OH * d->OW;
  const long total = (long)d->B * npix;
  long splits = (148L * 8 + d->C_out - 1) / d->C_out;
  if (splits > (total + 1023) / 1024) splits = (total + 1023) / 1024;
  if (splits < 1) splits = 1;
  const long pps = (total + splits - 1) / splits;
  dim3 grid((unsigned)d->C_out, (unsigned)splits);
  const size_t esz = d->dtype == MC_F64 ? 8 : 4;
  if (cudaMemsetAsync(gb, 0, d->C_out * esz, st) != cudaSuccess) return MC_ERR_LAUNCH;
  const int tsz = d->dtype == MC_F64 ? 8 : d->dtype == MC_F32 ? 4 : 2;
  const int nv = 16 / tsz;
  if (d->layout == MC_NHWC && d->C_out % nv == 0 && d->C_out / nv <= 256 &&
      (((uintptr_t)gy) & 15) == 0) {
    long blocks = (total + 4095) / 4096;
    if (blocks > 148 * 8) blocks = 148 * 8;
    if (blocks < 1) blocks = 1;
    const long ppb = (total + blocks - 1) / blocks;
    const size_t sm = 256 * 16 / tsz * esz;
    if (d->dtype == MC_F32) bias_grad_cl_kernel<float, float, 4><<<(unsigned)blocks, 256, sm, st>>>((const float*)gy, (float*)gb, d->C_out, total, ppb), MC_COUNT(1);
    else if (d->dtype == MC_F64) bias_grad_cl_kernel<double, double, 2><<<(unsigned)blocks, 256, sm, st>>>((const double*)gy, (double*)gb, d->C_out, total, ppb), MC_COUNT(1);
    else bias_grad_cl_kernel<bf16, float, 8><<<(unsigned)blocks, 256, sm, st>>>((const bf16*)gy, (float*)gb, d->C_out, total, ppb), MC_COUNT(1);
    MC_CHECK_LAUNCH();
    return MC_OK;
  }
  if (d->dtype == MC_F32) bias_grad_kernel<float, float><<<grid, 256, 0, st>>>((const float*)gy, (float*)gb, d->layout, d->B, d->C_out, npix, pps), MC_COUNT(1);
  else if (d->dtype == MC_F64) bias_grad_kernel<double, double><<<grid, 256, 0, st>>>((const double*)gy, (double*)gb, d->layout, d->B, d->C_out, npix, pps), MC_COUNT(1);
  else bias_grad_kernel<bf16, float><<<grid, 256, 0, st>>>((const bf16*)gy, (float*)gb, d->layout, d->B, d->C_out, npix, pps), MC_COUNT(1);
  MC_CHECK_LAUNCH();
  return MC_OK;
}

int conv_wgrad_simt_launch(const mc_desc* d, const void* gy, const void* x, const void* map,
                           const void* iw, void* gw, cudaStream_t st) {
  ConvArgs a = make_args(d);
  a.gy = gy; a.x = x; a.map = map; a.iw = d->P ? iw : nullptr; a.out = gw;
  const long total_pix = (long)d->B * a.npix_grid;
  const int tiles = ((d->C_out + TCO - 1) / TCO) * ((a.R + 63) / 64);
  long splits = (148L * 4 + tiles - 1) / tiles;
  if (splits > (total_pix + 63) / 64) splits = (total_pix + 63) / 64;
  if (splits < 1) splits = 1;
  a.pix_per_split = ((total_pix + splits - 1) / splits + 15) / 16 * 16;
  splits = (total_pix + a.pix_per_split - 1) / a.pix_per_split;
  const size_t esz = d->dtype == MC_F64 ? 8 : 4;
  if (cudaMemsetAsync(gw, 0, (size_t)d->C_out * a.R * esz, st) != cudaSuccess) return MC_ERR_LAUNCH;
  dim3 grid((unsigned)tiles, (unsigned)splits);
  if (d->dtype == MC_F32) conv_wgrad_simt<float><<<grid, 256, 0, st>>>(a), MC_COUNT(1);
  else if (d->dtype == MC_F64) conv_wgrad_simt<double><<<grid, 256, 0, st>>>(a), MC_COUNT(1);
  else conv_wgrad_simt<bf16><<<grid, 256, 0, st>>>(a), MC_COUNT(1);
  MC_CHECK_LAUNCH();
  return MC_OK;
}

int check_conv_desc_public(const mc_desc* d) { return check_conv_desc(d); }

}  // namespace mc
