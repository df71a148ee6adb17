// Bandwidth-oriented kernels for the gather-type ops (mapped max / avg pool, resample gather) on
// unweighted maps, float32 and bfloat16.
//
// The generic kernel decodes the sample map again for every (batch, channel) element.  Here the
// map entry of an output location is decoded ONCE into registers - up to NT (source pixel,
// weight) pairs - and reused for every channel and batch element:
//   * NCHW: one thread per output location walks over a group of (b, c) planes; tap 0 of a
//     one-ring map and the output are coalesced, the other taps are 4-byte gathers that live in
//     L1 / L2 (a plane is at most a few MB);
//   * NHWC: a group of lanes per output location reads every tap as one contiguous 16-byte-per-
//     lane run across channels and walks over the batch.
// Arithmetic is the same rounded sequence as the generic kernel, so results are bit-identical
// (include/nn/common/mapped_max_pool.h:14-58, mapped_avg_pool.h:14-42, resample.h:33-50 of the
// reference).
#include "common.cuh"

namespace mc {

enum { FOP_GATHER = 0, FOP_AVG = 1, FOP_MAX = 2 };

struct FastArgs {
  const void* x;
  const float* map;
  void* y;
  int64_t* idx;
  int B, C, IH, IW, K, interp;
  long npix_in, npix_out;
  int planes_per_block;
};

// Decoded entries of one output location.  NC = 1: K nearest taps (weight 1).  NC = 4: one
// bilinear / bispherical tap (K == 1).
template <int NT>
struct Entries {
  int off[NT];
  float w[NT];
};

template <int NT, int NC>
__device__ __forceinline__ void decode_entries(const FastArgs& a, long p, Entries<NT>& e) {
  if (NC == 1) {
#pragma unroll
    for (int k = 0; k < NT; ++k) {
      const float2 m = __ldg(reinterpret_cast<const float2*>(a.map) + p * NT + k);
      Tap<float> t;
      decode_tap<float, float>(m.x, m.y, a.IH, a.IW, 0, t);
      e.off[k] = t.off[0];
      e.w[k] = 1.f;
    }
  } else {
    const float2 m = __ldg(reinterpret_cast<const float2*>(a.map) + p);
    Tap<float> t;
    decode_tap<float, float>(m.x, m.y, a.IH, a.IW, a.interp, t);
#pragma unroll
    for (int i = 0; i < 4; ++i) { e.off[i] = t.off[i]; e.w[i] = t.w[i]; }
  }
}

// Combines the NT loaded values exactly like the generic kernel does.
template <int NT, int NC, int OP>
__device__ __forceinline__ float combine(const float (&v)[NT], const Entries<NT>& e, int K, int& best) {
  if (NC == 4) {
    float r = __fmul_rn(e.w[0], v[0]);
    r = __fadd_rn(r, __fmul_rn(e.w[1], v[1]));
    r = __fadd_rn(r, __fmul_rn(e.w[2], v[2]));
    r = __fadd_rn(r, __fmul_rn(e.w[3], v[3]));
    if (OP == FOP_AVG) r = div_by_const(__fadd_rn(0.f, r), (float)K, __frcp_rn((float)K));
    best = 0;
    return r;
  }
  if (OP == FOP_MAX) {
    float m = -FLT_MAX;
    best = -1;
#pragma unroll
    for (int k = 0; k < NT; ++k)
      if (v[k] > m) { m = v[k]; best = k; }
    return m;
  }
  if (OP == FOP_AVG) {
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < NT; ++k) s = __fadd_rn(s, v[k]);
    return div_by_const(s, (float)K, __frcp_rn((float)K));
  }
  best = 0;
  return v[0];
}

// ---- NCHW: thread per output location, loop over planes ------------------------------------------
template <typename T, int NT, int NC, int OP>
__global__ void __launch_bounds__(256) sample_planes_kernel(const FastArgs a) {
  const long p = blockIdx.x * 256L + threadIdx.x;
  if (p >= a.npix_out) return;
  Entries<NT> e;
  decode_entries<NT, NC>(a, p, e);
  const long nplanes = (long)a.B * a.C;
  const long pl0 = (long)blockIdx.y * a.planes_per_block;
  long pl1 = pl0 + a.planes_per_block;
  if (pl1 > nplanes) pl1 = nplanes;
  // (restrict: lets the loads of the next plane start before this plane's stores)
  const T* __restrict__ x = (const T*)a.x;
  T* __restrict__ y = (T*)a.y;
  int64_t* __restrict__ idx = a.idx;
#pragma unroll 2
  for (long pl = pl0; pl < pl1; ++pl) {
    const T* src = x + pl * a.npix_in;
    float v[NT];
#pragma unroll
    for (int k = 0; k < NT; ++k) v[k] = e.off[k] >= 0 ? (float)ldv(src + e.off[k]) : 0.f;
    int best;
    const float r = combine<NT, NC, OP>(v, e, a.K, best);
    stv(y + pl * a.npix_out + p, r);
    if (OP == FOP_MAX) idx[pl * a.npix_out + p] = best < 0 ? -1 : 2 * (p * NT + best);
  }
}

// ---- NHWC: LPP lanes per output location, 16 bytes per lane, loop over the batch -------------------
template <typename T> struct Vec16;
template <> struct Vec16<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void unpack(const uint4& u, float (&f)[4]) {
    f[0] = __uint_as_float(u.x); f[1] = __uint_as_float(u.y);
    f[2] = __uint_as_float(u.z); f[3] = __uint_as_float(u.w);
  }
  static __device__ __forceinline__ uint4 pack(const float (&f)[4]) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]),
                      __float_as_uint(f[3]));
  }
};
template <> struct Vec16<bf16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void unpack(const uint4& u, float (&f)[8]) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
  }
  static __device__ __forceinline__ uint4 pack(const float (&f)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
};

template <typename T, int NT, int NC, int OP>
__global__ void __launch_bounds__(256) sample_cl_kernel(const FastArgs a, int lpp_log2, int chunks) {
  constexpr int VN = Vec16<T>::N;
  const int lpp = 1 << lpp_log2;  // lanes per output location (C * sizeof(T) / 16 / chunks)
  const long gthread = blockIdx.x * 256L + threadIdx.x;
  const long p = gthread >> lpp_log2;
  const int lane = (int)(gthread & (lpp - 1));
  if (p >= a.npix_out) return;
  Entries<NT> e;
  decode_entries<NT, NC>(a, p, e);
  const T* x = (const T*)a.x;
  T* y = (T*)a.y;
  for (int b = blockIdx.y; b < a.B; b += gridDim.y) {
    for (int ch = 0; ch < chunks; ++ch) {
      const int c0 = (ch * lpp + lane) * VN;
      const T* src = x + (long)b * a.npix_in * a.C + c0;
      float v[NT][VN];
#pragma unroll
      for (int k = 0; k < NT; ++k) {
        uint4 u = make_uint4(0, 0, 0, 0);
        if (e.off[k] >= 0) u = __ldg(reinterpret_cast<const uint4*>(src + (long)e.off[k] * a.C));
        Vec16<T>::unpack(u, v[k]);
      }
      float r[VN];
      long bi[VN];
#pragma unroll
      for (int j = 0; j < VN; ++j) {
        float col[NT];
#pragma unroll
        for (int k = 0; k < NT; ++k) col[k] = v[k][j];
        int best;
        r[j] = combine<NT, NC, OP>(col, e, a.K, best);
        bi[j] = best < 0 ? -1 : 2 * (p * NT + best);
      }
      const long o = ((long)b * a.npix_out + p) * a.C + c0;
      *reinterpret_cast<uint4*>(y + o) = Vec16<T>::pack(r);
      if (OP == FOP_MAX) {
#pragma unroll
        for (int j = 0; j < VN; j += 2)
          *reinterpret_cast<longlong2*>(a.idx + o + j) = make_longlong2(bi[j], bi[j + 1]);
      }
    }
  }
}

template <typename T, int NT, int NC, int OP>
static int launch_fast(const mc_desc* d, FastArgs a, cudaStream_t st) {
  if (d->layout == MC_NCHW) {
    const long nplanes = (long)a.B * a.C;
    const long xblocks = (a.npix_out + 255) / 256;
    // enough blocks to fill the GPU several times over, at least 8 planes per block for reuse
    long ppb = nplanes * xblocks / (148L * 16);
    if (ppb < 8) ppb = 8;
    if (ppb > 64) ppb = 64;
    a.planes_per_block = (int)ppb;
    dim3 grid((unsigned)xblocks, (unsigned)((nplanes + ppb - 1) / ppb));
    if (grid.y > 65535) return MC_ERR_TOO_LARGE;
    sample_planes_kernel<T, NT, NC, OP><<<grid, 256, 0, st>>>(a), MC_COUNT(1);
  } else {
    const int row16 = a.C * (int)sizeof(T) / 16;  // 16-byte vectors per location
    int lpp_log2 = 0;
    while ((1 << (lpp_log2 + 1)) <= row16 && lpp_log2 < 5 && row16 % (1 << (lpp_log2 + 1)) == 0) ++lpp_log2;
    const int chunks = row16 >> lpp_log2;
    const long threads = a.npix_out << lpp_log2;
    const long xblocks = (threads + 255) / 256;
    int by = (int)((148L * 8 + xblocks - 1) / xblocks);
    if (by < 1) by = 1;
    if (by > a.B) by = a.B;
    dim3 grid((unsigned)xblocks, (unsigned)by);
    sample_cl_kernel<T, NT, NC, OP><<<grid, 256, 0, st>>>(a, lpp_log2, chunks), MC_COUNT(1);
  }
  return cudaGetLastError() == cudaSuccess ? MC_OK : MC_ERR_LAUNCH;
}

template <typename T, int OP>
static bool dispatch_nt(const mc_desc* d, const FastArgs& a, cudaStream_t st, int* rc) {
  const bool nearest = d->interp != 1 && d->interp != 2;
  if (nearest) {
    switch (d->K) {
      case 1: *rc = launch_fast<T, 1, 1, OP>(d, a, st); return true;
      case 4: *rc = launch_fast<T, 4, 1, OP>(d, a, st); return true;
      case 7: *rc = launch_fast<T, 7, 1, OP>(d, a, st); return true;
      case 9: *rc = launch_fast<T, 9, 1, OP>(d, a, st); return true;
      default: return false;
    }
  }
  if (d->K == 1 && OP != FOP_MAX) { *rc = launch_fast<T, 4, 4, OP>(d, a, st); return true; }
  return false;
}

// Returns true if a fast kernel took the call (its status is in *rc).
bool sample_fwd_fast(const mc_desc* d, int op, const void* x, const void* map, void* y, int64_t* idx,
                     cudaStream_t st, int* rc) {
  if (d->P != 0 || (d->dtype != MC_F32 && d->dtype != MC_BF16)) return false;
  const size_t esz = d->dtype == MC_F32 ? 4 : 2;
  if (d->layout == MC_NHWC) {
    if ((d->C_in * esz) % 16 != 0) return false;
    if ((((uintptr_t)x | (uintptr_t)y) & 15) || (idx && ((uintptr_t)idx & 15))) return false;
  }
  if (((uintptr_t)map & 7) != 0) return false;
  FastArgs a;
  a.x = x; a.map = (const float*)map; a.y = y; a.idx = idx;
  a.B = d->B; a.C = d->C_in; a.IH = d->IH; a.IW = d->IW; a.K = d->K; a.interp = d->interp;
  a.npix_in = (long)d->IH * d->IW;
  a.npix_out = (long)d->OH * d->OW;
  a.planes_per_block = 8;
  if (d->dtype == MC_F32) {
    if (op == FOP_MAX) return dispatch_nt<float, FOP_MAX>(d, a, st, rc);
    if (op == FOP_AVG) return dispatch_nt<float, FOP_AVG>(d, a, st, rc);
    return dispatch_nt<float, FOP_GATHER>(d, a, st, rc);
  }
  if (op == FOP_MAX) return dispatch_nt<bf16, FOP_MAX>(d, a, st, rc);
  if (op == FOP_AVG) return dispatch_nt<bf16, FOP_AVG>(d, a, st, rc);
  return dispatch_nt<bf16, FOP_GATHER>(d, a, st, rc);
}

}  // namespace mc

// ---- adjoints as gathers through the inverse map ---------------------------------------------------
// The reference scatters every grid value into the image with atomicAdd
// (include/nn/cuda/mapped_avg_pool.cuh:92-130, resample.cuh:14-52).  With the inverse map (for every
// image pixel the list of (grid location, weight) pairs that land on it, built once per map by
// mc_invmap_build) the same sums are formed by ONE thread per image pixel: no atomics, no
// zero-fill pass, coalesced stores, and results that repeat bit for bit.  The lists of the K taps
// of a pixel are adjacent in the CSR, so the pixel's entries are one contiguous range.
namespace mc {

struct InvGatherArgs {
  const void* g;     // values on the map grid (B, C, ngrid)
  void* out;         // image (B, C, npix), fully written
  const int* off;    // (npix * K + 1)
  const int2* ent;   // (grid location, weight bits)
  int B, C, K;
  long npix, ngrid;
  float inv_k;       // 1 / K, correctly rounded (average unpooling divides by K)
  int planes_per_block;
};

template <typename T, bool AVG>
__global__ void __launch_bounds__(256) inv_gather_planes_kernel(const InvGatherArgs a) {
  const long q = blockIdx.x * 256L + threadIdx.x;
  if (q >= a.npix) return;
  const int beg = __ldg(a.off + q * a.K), end = __ldg(a.off + (q + 1) * a.K);
  const long nplanes = (long)a.B * a.C;
  const long pl0 = (long)blockIdx.y * a.planes_per_block;
  long pl1 = pl0 + a.planes_per_block;
  if (pl1 > nplanes) pl1 = nplanes;
  const T* __restrict__ g = (const T*)a.g;
  T* __restrict__ out = (T*)a.out;
  // (Average unpooling only: the lists of a resample map are of mixed lengths, and the registers
  // of this path would cost the general loop its occupancy.)
  if (AVG && __all_sync(__activemask(), end - beg <= 2)) {
    // Every list of the warp has at most two entries (pooling maps): eight planes per trip, all
    // their loads issued before the first value is used.  The operations and their order are
    // those of the general loop below.  (A warp with longer lists takes the general loop as a
    // whole: running both paths side by side costs more than the batching gains.)
    constexpr int UP = 8;
    const int n = end - beg;
    const int2 e0 = n >= 1 ? __ldg(a.ent + beg) : make_int2(0, 0);
    const int2 e1 = n >= 2 ? __ldg(a.ent + beg + 1) : make_int2(0, 0);
    const float w0 = __int_as_float(e0.y), w1 = __int_as_float(e1.y);
    for (long pl = pl0; pl < pl1; pl += UP) {
      float v0[UP], v1[UP];
#pragma unroll
      for (int u = 0; u < UP; ++u) {
        v0[u] = v1[u] = 0.f;
        if (pl + u < pl1) {
          const T* src = g + (pl + u) * a.ngrid;
          if (n >= 1) v0[u] = (float)ldv(src + e0.x);
          if (n >= 2) v1[u] = (float)ldv(src + e1.x);
        }
      }
#pragma unroll
      for (int u = 0; u < UP; ++u) {
        if (pl + u >= pl1) break;
        float acc = 0.f;
        if (n >= 1) {
          const float t = AVG ? div_by_const(v0[u], (float)a.K, a.inv_k) : v0[u];
          acc = __fadd_rn(acc, __fmul_rn(w0, t));
        }
        if (n >= 2) {
          const float t = AVG ? div_by_const(v1[u], (float)a.K, a.inv_k) : v1[u];
          acc = __fadd_rn(acc, __fmul_rn(w1, t));
        }
        stv(out + (pl + u) * a.npix + q, acc);
      }
    }
    return;
  }
  // the common short lists stay in registers; longer ones are re-read per plane
  int2 e4[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) e4[i] = beg + i < end ? __ldg(a.ent + beg + i) : make_int2(0, 0);
  const int n4 = end - beg < 4 ? end - beg : 4;
  const bool longer = end - beg > 4;
  if (!AVG && __all_sync(__activemask(), !longer)) {
    // no list of the warp goes beyond the four entries held in registers: four planes per trip,
    // their loads issued together (same operations and order as the loop below)
    constexpr int UP = 4;
    for (long pl = pl0; pl < pl1; pl += UP) {
      float v[UP][4];
#pragma unroll
      for (int u = 0; u < UP; ++u) {
        const T* src = g + (pl + u) * a.ngrid;
#pragma unroll
        for (int i = 0; i < 4; ++i)
          v[u][i] = (i < n4 && pl + u < pl1) ? (float)ldv(src + e4[i].x) : 0.f;
      }
#pragma unroll
      for (int u = 0; u < UP; ++u) {
        if (pl + u >= pl1) break;
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (i < n4) acc = __fadd_rn(acc, __fmul_rn(__int_as_float(e4[i].y), v[u][i]));
        stv(out + (pl + u) * a.npix + q, acc);
      }
    }
    return;
  }
  // four planes per trip: their (independent) loads are in flight together
#pragma unroll 4
  for (long pl = pl0; pl < pl1; ++pl) {
    const T* src = g + pl * a.ngrid;
    float v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = i < n4 ? (float)ldv(src + e4[i].x) : 0.f;
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (i < n4) {
        float t = v[i];
        if (AVG) t = div_by_const(t, (float)a.K, a.inv_k);
        acc = __fadd_rn(acc, __fmul_rn(__int_as_float(e4[i].y), t));
      }
    }
    if (longer) {
      for (int e = beg + 4; e < end; ++e) {
        const int2 en = __ldg(a.ent + e);
        float t = (float)ldv(src + en.x);
        if (AVG) t = div_by_const(t, (float)a.K, a.inv_k);
        acc = __fadd_rn(acc, __fmul_rn(__int_as_float(en.y), t));
      }
    }
    stv(out + pl * a.npix + q, acc);
  }
}

template <typename T, bool AVG>
__global__ void __launch_bounds__(256) inv_gather_cl_kernel(const InvGatherArgs a, int lpp_log2,
                                                            int chunks) {
  constexpr int VN = Vec16<T>::N;
  const int lpp = 1 << lpp_log2;
  const long gthread = blockIdx.x * 256L + threadIdx.x;
  const long q = gthread >> lpp_log2;
  const int lane = (int)(gthread & (lpp - 1));
  if (q >= a.npix) return;
  const int beg = __ldg(a.off + q * a.K), end = __ldg(a.off + (q + 1) * a.K);
  const T* __restrict__ g = (const T*)a.g;
  T* __restrict__ out = (T*)a.out;
  if (chunks == 1 && __all_sync(__activemask(), end - beg <= 2)) {
    // Every list of the warp has one or two entries (pooling maps): the entries stay in registers
    // and four batch elements are in flight at once - one load per trip leaves the kernel waiting
    // on latency.  (A warp with longer lists takes the general loop as a whole.)
    constexpr int UB = 4;
    const int n = end - beg;
    const int2 e0 = n >= 1 ? __ldg(a.ent + beg) : make_int2(0, 0);
    const int2 e1 = n >= 2 ? __ldg(a.ent + beg + 1) : make_int2(0, 0);
    const float w0 = __int_as_float(e0.y), w1 = __int_as_float(e1.y);
    const int c0 = lane * VN;
    const long o0 = (long)e0.x * a.C + c0, o1 = (long)e1.x * a.C + c0;
    const long img_in = a.ngrid * a.C, img_out = a.npix * a.C;
    for (int b = blockIdx.y; b < a.B; b += UB * gridDim.y) {
      uint4 r0[UB], r1[UB];
#pragma unroll
      for (int u = 0; u < UB; ++u) {
        const int bb = b + u * gridDim.y;
        r0[u] = r1[u] = make_uint4(0, 0, 0, 0);
        if (bb < a.B) {
          const T* src = g + bb * img_in;
          if (n >= 1) r0[u] = __ldg(reinterpret_cast<const uint4*>(src + o0));
          if (n >= 2) r1[u] = __ldg(reinterpret_cast<const uint4*>(src + o1));
        }
      }
#pragma unroll
      for (int u = 0; u < UB; ++u) {
        const int bb = b + u * gridDim.y;
        if (bb >= a.B) break;
        float v0[VN], v1[VN], acc[VN];
        Vec16<T>::unpack(r0[u], v0);
        Vec16<T>::unpack(r1[u], v1);
#pragma unroll
        for (int j = 0; j < VN; ++j) {
          if (sizeof(T) == 2) {
            acc[j] = fmaf(w1, v1[j], w0 * v0[j]);
            if (AVG) acc[j] *= a.inv_k;
          } else {
            // the same operations in the same order as the general loop below
            const float t0 = AVG ? div_by_const(v0[j], (float)a.K, a.inv_k) : v0[j];
            acc[j] = __fadd_rn(0.f, __fmul_rn(w0, t0));
            if (n >= 2) {
              const float t1 = AVG ? div_by_const(v1[j], (float)a.K, a.inv_k) : v1[j];
              acc[j] = __fadd_rn(acc[j], __fmul_rn(w1, t1));
            }
          }
        }
        if (n == 0) {
#pragma unroll
          for (int j = 0; j < VN; ++j) acc[j] = 0.f;
        }
        *reinterpret_cast<uint4*>(out + bb * img_out + q * a.C + c0) = Vec16<T>::pack(acc);
      }
    }
    return;
  }
  for (int b = blockIdx.y; b < a.B; b += gridDim.y) {
    for (int ch = 0; ch < chunks; ++ch) {
      const int c0 = (ch * lpp + lane) * VN;
      const T* src = g + (long)b * a.ngrid * a.C + c0;
      float acc[VN];
#pragma unroll
      for (int j = 0; j < VN; ++j) acc[j] = 0.f;
      for (int e = beg; e < end; ++e) {
        const int2 en = __ldg(a.ent + e);
        const float w = __int_as_float(en.y);
        float v[VN];
        Vec16<T>::unpack(__ldg(reinterpret_cast<const uint4*>(src + (long)en.x * a.C)), v);
#pragma unroll
        for (int j = 0; j < VN; ++j) {
          if (sizeof(T) == 2) {
            // bf16: the reference has no such type to match bit for bit, and the kernel is bound
            // by its instruction count - one fma per value, the division by K once at the end
            acc[j] = fmaf(w, v[j], acc[j]);
          } else {
            const float t = AVG ? div_by_const(v[j], (float)a.K, a.inv_k) : v[j];
            acc[j] = __fadd_rn(acc[j], __fmul_rn(w, t));
          }
        }
      }
      if (sizeof(T) == 2 && AVG) {
#pragma unroll
        for (int j = 0; j < VN; ++j) acc[j] *= a.inv_k;
      }
      *reinterpret_cast<uint4*>(out + ((long)b * a.npix + q) * a.C + c0) = Vec16<T>::pack(acc);
    }
  }
}

template <typename T, bool AVG>
static int launch_inv_gather(const mc_desc* d, InvGatherArgs a, cudaStream_t st) {
  if (d->layout == MC_NCHW) {
    const long nplanes = (long)a.B * a.C;
    const long xblocks = (a.npix + 255) / 256;
    long ppb = nplanes * xblocks / (148L * 16);
    if (ppb < 4) ppb = 4;
    if (ppb > 64) ppb = 64;
    a.planes_per_block = (int)ppb;
    dim3 grid((unsigned)xblocks, (unsigned)((nplanes + ppb - 1) / ppb));
    if (grid.y > 65535) return MC_ERR_TOO_LARGE;
    inv_gather_planes_kernel<T, AVG><<<grid, 256, 0, st>>>(a), MC_COUNT(1);
  } else {
    const int row16 = a.C * (int)sizeof(T) / 16;
    int lpp_log2 = 0;
    while ((1 << (lpp_log2 + 1)) <= row16 && lpp_log2 < 5 && row16 % (1 << (lpp_log2 + 1)) == 0) ++lpp_log2;
    const int chunks = row16 >> lpp_log2;
    const long xblocks = ((a.npix << lpp_log2) + 255) / 256;
    int by = (int)((148L * 8 + xblocks - 1) / xblocks);
    if (by < 1) by = 1;
    if (by > a.B) by = a.B;
    dim3 grid((unsigned)xblocks, (unsigned)by);
    inv_gather_cl_kernel<T, AVG><<<grid, 256, 0, st>>>(a, lpp_log2, chunks), MC_COUNT(1);
  }
  return cudaGetLastError() == cudaSuccess ? MC_OK : MC_ERR_LAUNCH;
}

// inv: buffer built by mc_invmap_build for the same descriptor.  avg != 0: average unpooling
// (values divided by K first), else resample scatter.
int scatter_inv_launch(const mc_desc* d, const void* g, const void* inv, size_t inv_off_bytes,
                       void* out, int avg, cudaStream_t st) {
  if (d->P != 0 || (d->dtype != MC_F32 && d->dtype != MC_BF16)) return MC_ERR_UNSUPPORTED;
  const size_t esz = d->dtype == MC_F32 ? 4 : 2;
  if (d->layout == MC_NHWC && ((d->C_in * esz) % 16 != 0 || (((uintptr_t)g | (uintptr_t)out) & 15)))
    return MC_ERR_UNSUPPORTED;
  InvGatherArgs a;
  a.g = g; a.out = out;
  a.off = (const int*)inv;
  a.ent = (const int2*)((const uint8_t*)inv + inv_off_bytes);
  a.B = d->B; a.C = d->C_in; a.K = d->K;
  a.npix = (long)d->IH * d->IW;
  a.ngrid = (long)d->OH * d->OW;
  a.inv_k = 1.f / d->K;
  a.planes_per_block = 8;
  if (d->dtype == MC_F32)
    return avg ? launch_inv_gather<float, true>(d, a, st) : launch_inv_gather<float, false>(d, a, st);
  return avg ? launch_inv_gather<bf16, true>(d, a, st) : launch_inv_gather<bf16, false>(d, a, st);
}

// ---- input gradient of a convolution after the contraction -------------------------------------------
// gx[b, q, c] = sum over taps k, over the entries (p, w) of the inverse-map list (q, k), of
//               w * Z[b, p, k * C + c]      with Z[b, p, k * C + c] = sum_co gy[b, p, co] W[co, c, k]
// Z is the product of grad_output with the weights of every tap - one dense GEMM the caller runs -
// so what is gathered here are C_in-channel rows, each read exactly once; worth it when the layer
// has more output than input channels (the gather-in-the-GEMM form of mc_conv_dgrad_inv moves
// C_out-channel rows).  bf16, channels-last.  Thread = 8 channels of an input pixel; four rows of two
// images in flight per trip.
__global__ void __launch_bounds__(256) tap_gather_sum_kernel(const bf16* __restrict__ z, bf16* __restrict__ out,
                                                             const int* __restrict__ off,
                                                             const int2* __restrict__ ent, int B, int C, int K,
                                                             long npix, long ngrid, int lpp_log2) {
  constexpr int UB = 2;
  const long gthread = blockIdx.x * 256L + threadIdx.x;
  const long q = gthread >> lpp_log2;
  const int c0 = (int)(gthread & ((1 << lpp_log2) - 1)) * 8;
  if (q >= npix) return;
  const long zrow = (long)K * C, zimg = ngrid * zrow, oimg = npix * C;
  // The pixel's entries of all taps (one-ring and 3 x 3 maps: about K of them) are fetched first, so
  // that the row loads of a trip do not each wait for their list entry; rows beyond NE take the loop.
  constexpr int NE = 12;
  const int e0 = __ldg(off + q * K), e1 = __ldg(off + (q + 1) * K);
  long zo[NE];   // offset of the entry's row inside an image of z (its tap's block, this thread's channels)
  float zw[NE];
  {
    int k = 0, kend = __ldg(off + q * K + 1);
#pragma unroll
    for (int i = 0; i < NE; ++i) {
      const int e = e0 + i;
      zo[i] = 0; zw[i] = 0.f;
      if (e < e1) {
        while (e >= kend) { ++k; kend = __ldg(off + q * K + k + 1); }
        const int2 en = __ldg(ent + e);
        zo[i] = (long)en.x * zrow + k * C + c0;
        zw[i] = __int_as_float(en.y);
      }
    }
  }
  for (int b = blockIdx.y * UB; b < B; b += UB * gridDim.y) {
    float acc[UB][8];
#pragma unroll
    for (int u = 0; u < UB; ++u)
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[u][j] = 0.f;
    const bf16* zb = z + (long)b * zimg;
#pragma unroll
    for (int i0 = 0; i0 < NE; i0 += 4) {
      if (e0 + i0 >= e1) break;
      uint4 r[4][UB];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int u = 0; u < UB; ++u)
          r[i][u] = (e0 + i0 + i < e1 && b + u < B) ? __ldg(reinterpret_cast<const uint4*>(zb + zo[i0 + i] + u * zimg))
                                                   : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int u = 0; u < UB; ++u) {
          float v[8];
          Vec16<bf16>::unpack(r[i][u], v);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[u][j] = fmaf(zw[i0 + i], v[j], acc[u][j]);
        }
    }
    if (e1 - e0 > NE) {  // long lists
      int k = 0, kend = __ldg(off + q * K + 1);
      for (int e = e0 + NE; e < e1; ++e) {
        while (e >= kend) { ++k; kend = __ldg(off + q * K + k + 1); }
        const int2 en = __ldg(ent + e);
        const float w = __int_as_float(en.y);
        const bf16* zp = zb + (long)en.x * zrow + k * C + c0;
#pragma unroll
        for (int u = 0; u < UB; ++u) {
          if (b + u >= B) break;
          float v[8];
          Vec16<bf16>::unpack(__ldg(reinterpret_cast<const uint4*>(zp + u * zimg)), v);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[u][j] = fmaf(w, v[j], acc[u][j]);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < UB; ++u)
      if (b + u < B)
        *reinterpret_cast<uint4*>(out + (long)(b + u) * oimg + q * C + c0) = Vec16<bf16>::pack(acc[u]);
  }
}

// z (B, ngrid, K * C_in) bf16, gx (B, C_in, IH, IW) channels-last bf16, inv from mc_invmap_build.
int tap_gather_sum_launch(const mc_desc* d, const void* z, const void* inv, size_t inv_off_bytes, void* gx,
                          cudaStream_t st) {
  if (d->P != 0 || d->dtype != MC_BF16 || d->layout != MC_NHWC || d->C_in % 8 != 0) return MC_ERR_UNSUPPORTED;
  if ((((uintptr_t)z | (uintptr_t)gx | (uintptr_t)inv) & 15)) return MC_ERR_BAD_ARG;
  const int lanes = d->C_in / 8;
  int lpp_log2 = 0;
  while ((1 << lpp_log2) < lanes) ++lpp_log2;
  if ((1 << lpp_log2) != lanes) return MC_ERR_UNSUPPORTED;  // C_in / 8 a power of two
  const long npix = (long)d->IH * d->IW;
  const long xblocks = ((npix << lpp_log2) + 255) / 256;
  int by = (int)((148L * 8 + xblocks - 1) / xblocks);
  if (by < 1) by = 1;
  if (by > (d->B + 1) / 2) by = (d->B + 1) / 2;
  tap_gather_sum_kernel<<<dim3((unsigned)xblocks, (unsigned)by), 256, 0, st>>>(
      (const bf16*)z, (bf16*)gx, (const int*)inv, (const int2*)((const uint8_t*)inv + inv_off_bytes), d->B,
      d->C_in, d->K, npix, (long)d->OH * d->OW, lpp_log2), MC_COUNT(1);
  return cudaGetLastError() == cudaSuccess ? MC_OK : MC_ERR_LAUNCH;
}

}  // namespace mc
