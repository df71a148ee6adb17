// Shared device helpers: scalar traits, exact (non-contracted) arithmetic, and the sample-map
// tap decoder that every kernel uses.
//
// The tap decoder restates the per-sample semantics of the reference's
// include/core/interpolation.h:
//   nearest      :85-122  (llround = round half away from zero; zero outside the image)
//   bilinear     :125-180 (floor corner + 1; each corner valid iff inside; weights A*B, A*C, D*B, D*C)
//   bispherical  :183-238 (bilinear with the x coordinate wrapped, only y checked)
// Products and sums use the round-to-nearest intrinsics so that nvcc cannot contract them into
// FMAs: gather-type results are then bit-identical to the reference's host arithmetic.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

#include <atomic>

#include "mc_b200.h"

namespace mc {

typedef __nv_bfloat16 bf16;

template <typename T> struct Traits;
template <> struct Traits<float> { typedef float CT; typedef float MT; };
template <> struct Traits<double> { typedef double CT; typedef double MT; };
template <> struct Traits<bf16> { typedef float CT; typedef float MT; };

__device__ __forceinline__ float mul_rn(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ double mul_rn(double a, double b) { return __dmul_rn(a, b); }
__device__ __forceinline__ float add_rn(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ double add_rn(double a, double b) { return __dadd_rn(a, b); }
__device__ __forceinline__ float div_rn(float a, float b) { return __fdiv_rn(a, b); }
__device__ __forceinline__ double div_rn(double a, double b) { return __ddiv_rn(a, b); }

// v / k for a divisor that is the same for a whole kernel (a tap count), bit-identical to
// __fdiv_rn(v, k) at a fifth of its instructions.  rk = 1 / k correctly rounded (computed on the
// host).  q = RN(v * rk) is within an ulp of the quotient, the residual r = v - q * k is exact in
// one fma, and RN(q + r * rk) is then the correctly rounded quotient (Markstein's correction
// step), as long as nothing underflows or overflows on the way: magnitudes outside
// [1e-30, 1e30] take the ordinary division; zeros keep their sign.
__device__ __forceinline__ float div_by_const(float v, float k, float rk) {
  const float q = __fmul_rn(v, rk);
  const float r = __fmaf_rn(-q, k, v);
  float res = __fmaf_rn(r, rk, q);
  const float av = fabsf(v);
  if (!(av > 1e-30f && av < 1e30f)) res = av == 0.f ? v : __fdiv_rn(v, k);
  return res;
}

__device__ __forceinline__ float ldv(const float* p) { return __ldg(p); }
__device__ __forceinline__ double ldv(const double* p) { return __ldg(p); }
__device__ __forceinline__ float ldv(const bf16* p) {
  return __bfloat162float(__ushort_as_bfloat16(__ldg(reinterpret_cast<const unsigned short*>(p))));
}
__device__ __forceinline__ void stv(float* p, float v) { *p = v; }
__device__ __forceinline__ void stv(double* p, double v) { *p = v; }
__device__ __forceinline__ void stv(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float rnd_half_away(float v) { return roundf(v); }
__device__ __forceinline__ double rnd_half_away(double v) { return round(v); }
__device__ __forceinline__ float flr(float v) { return floorf(v); }
__device__ __forceinline__ double flr(double v) { return floor(v); }

// One decoded map sample: up to four source pixels (offset y*W+x inside one channel plane, or
// -1 for a corner that contributes zero) with their interpolation weights, in the reference's
// corner order (x1,y1), (x2,y1), (x1,y2), (x2,y2).
template <typename CT>
struct Tap {
  int off[4];
  CT w[4];
  int n;  // 1 for nearest, 4 otherwise
};

template <typename MT, typename CT>
__device__ __forceinline__ void decode_tap(MT x, MT y, int H, int W, int interp, Tap<CT>& t) {
  if (interp != 1 && interp != 2) {
    const MT xr = rnd_half_away(x), yr = rnd_half_away(y);
    const bool ok = xr >= MT(0) && xr <= MT(W - 1) && yr >= MT(0) && yr <= MT(H - 1);
    t.n = 1;
    t.off[0] = ok ? (int)yr * W + (int)xr : -1;
    t.w[0] = CT(1);
    return;
  }
  const MT xf = flr(x), yf = flr(y);
  const MT Bx = (xf + MT(1)) - x, Cx = x - xf;
  const MT Ay = (yf + MT(1)) - y, Dy = y - yf;
  t.n = 4;
  t.w[0] = (CT)mul_rn(Ay, Bx);
  t.w[1] = (CT)mul_rn(Ay, Cx);
  t.w[2] = (CT)mul_rn(Dy, Bx);
  t.w[3] = (CT)mul_rn(Dy, Cx);
  const bool y1ok = yf >= MT(0) && yf <= MT(H - 1);
  const bool y2ok = yf >= MT(-1) && yf <= MT(H - 2);
  const int y1 = y1ok ? (int)yf : 0, y2 = y2ok ? (int)yf + 1 : 0;
  int x1, x2;
  bool x1ok, x2ok;
  if (interp == 1) {
    x1ok = xf >= MT(0) && xf <= MT(W - 1);
    x2ok = xf >= MT(-1) && xf <= MT(W - 2);
    x1 = x1ok ? (int)xf : 0;
    x2 = x2ok ? (int)xf + 1 : 0;
  } else {
    // wrap: ((v % W) + W) % W on the integer corner (include/core/util.h:48-51)
    const bool fin = xf > MT(-1.0e18) && xf < MT(1.0e18);
    const long long xl = fin ? (long long)xf : 0;
    x1 = (int)(((xl % W) + W) % W);
    x2 = (int)((((xl + 1) % W) + W) % W);
    x1ok = x2ok = fin;
  }
  t.off[0] = (x1ok && y1ok) ? y1 * W + x1 : -1;
  t.off[1] = (x2ok && y1ok) ? y1 * W + x2 : -1;
  t.off[2] = (x1ok && y2ok) ? y2 * W + x1 : -1;
  t.off[3] = (x2ok && y2ok) ? y2 * W + x2 : -1;
}

// Interpolated value of one map sample read from one channel plane (pixel stride sp).
template <typename T, typename CT>
__device__ __forceinline__ CT tap_gather(const T* plane, long sp, const Tap<CT>& t) {
  if (t.n == 1) return t.off[0] >= 0 ? (CT)ldv(plane + (long)t.off[0] * sp) : CT(0);
  CT v[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] = t.off[i] >= 0 ? (CT)ldv(plane + (long)t.off[i] * sp) : CT(0);
  CT r = mul_rn(t.w[0], v[0]);
  r = add_rn(r, mul_rn(t.w[1], v[1]));
  r = add_rn(r, mul_rn(t.w[2], v[2]));
  r = add_rn(r, mul_rn(t.w[3], v[3]));
  return r;
}

// Adjoint of tap_gather: plane[corner] += weight * value (atomic).
template <typename CT>
__device__ __forceinline__ void tap_scatter(CT* plane, long sp, const Tap<CT>& t, CT value) {
  if (t.n == 1) {
    if (t.off[0] >= 0) atomicAdd(plane + (long)t.off[0] * sp, value);
    return;
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
    if (t.off[i] >= 0) atomicAdd(plane + (long)t.off[i] * sp, mul_rn(t.w[i], value));
}

// Strides (in elements) of a (B, C, H*W) activation in either layout.
struct Strides {
  long b, c, p;
};
__host__ __device__ inline Strides make_strides(int layout, int C, long npix) {
  Strides s;
  s.b = (long)C * npix;
  if (layout == MC_NHWC) { s.c = 1; s.p = C; } else { s.c = npix; s.p = 1; }
  return s;
}

// Splits a linear element index into (b, c, p) so that consecutive threads touch consecutive
// memory in the given layout.
__device__ __forceinline__ void split_index(long i, int layout, int C, long npix, int& b, int& c,
                                            long& p) {
  if (layout == MC_NHWC) {
    c = (int)(i % C);
    const long r = i / C;
    p = r % npix;
    b = (int)(r / npix);
  } else {
    p = i % npix;
    const long r = i / npix;
    c = (int)(r % C);
    b = (int)(r / C);
  }
}

inline int grid_for(long n, int block, int max_blocks = 148 * 32) {
  long g = (n + block - 1) / block;
  if (g > max_blocks) g = max_blocks;
  if (g < 1) g = 1;
  return (int)g;
}

// Number of kernels this library has launched in this process (diagnostic).
extern std::atomic<unsigned long long> g_launches;
#define MC_COUNT(n) (mc::g_launches.fetch_add((n), std::memory_order_relaxed))

#define MC_CHECK_LAUNCH()                                  \
  do {                                                     \
    if (cudaGetLastError() != cudaSuccess) return MC_ERR_LAUNCH; \
  } while (0)

}  // namespace mc
