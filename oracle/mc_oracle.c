/*
 * CPU oracle: a plain-C restatement of the reference's algorithm for the mapped-convolution hot
 * path (meder411/MappedConvolutions, package/ext_modules).
 *
 * THIS IS TEST INFRASTRUCTURE.  It is the checker that the CUDA kernels are compared against and
 * the "port" CPU baseline of the benchmark.  The product package never loads it.
 *
 * Parity pin: every function here except oracle_knn is checked against the reference's own CPU
 * extension (built from its sources by oracle/build_ref.py) on the reference's known-answer
 * inputs and on seeded random inputs; the resulting vectors are committed under tests/golden/.
 * oracle_knn restates include/util/cuda/knn.cuh (the reference has no CPU k-NN and no k-NN test);
 * it is pinned by vectors recorded from the reference's own CUDA kernels on a GPU
 * (tests/golden/knn_ref.npz) for M == k, the only case in which those kernels stay inside their
 * buffers (src/util/cuda/knn_layer.cu:22-27 against include/util/cuda/knn.cuh:112,169-170), and
 * PARITY UNPINNED for M > k.
 * oracle_voting_resample is pinned by the reference's CPU extension (tests/golden/extras.npz).
 * oracle_cube2rect restates include/util/cuda/cube2rect.cuh (CUDA only in the reference); it is
 * pinned by vectors recorded from the reference's CUDA kernel on a GPU
 * (tests/golden/cube2rect_ref.npz), up to the difference between the host's and the device's
 * sin / cos (tolerance in tests/test_extras.py).
 *
 * Build: gcc -O2 -fopenmp -ffp-contract=off -shared -fPIC mc_oracle.c -o libmc_oracle.so -lm
 */
#include <float.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define CAT_(a, b) a##b
#define CAT(a, b) CAT_(a, b)

#define T float
#define TMIN FLT_MIN
#define SUF(n) CAT(n, _f32)
#include "mc_oracle_impl.h"
#undef T
#undef TMIN
#undef SUF

#define T double
#define TMIN DBL_MIN
#define SUF(n) CAT(n, _f64)
#include "mc_oracle_impl.h"
#undef T
#undef TMIN
#undef SUF

/* k nearest neighbours, restating include/util/cuda/knn.cuh:
 *   :82-103  squared distance accumulated over the dimensions in order; nvcc contracts
 *            `ssd += tmp * tmp` into an fma, which is pinned here as s = fmaf(t, t, s), t = ref - query;
 *   :125-189 insertion into a sorted k-list with strict '<' == selection by (distance, index);
 *   :141,160,184 indices are 1-based;  :199-205 sqrt of the kept distances.
 * ref (B,D,M), query (B,D,N) -> idx (B,k,N) int64, dist (B,k,N). */
void oracle_knn(const float* ref, const float* query, int B, int D, int M, int N, int k,
                int64_t* idx, float* dist) {
  for (int b = 0; b < B; ++b) {
    const float* r = ref + (int64_t)b * D * M;
    const float* q = query + (int64_t)b * D * N;
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; ++n) {
      float bd[64];
      int bi[64];
      int cnt = 0;
      for (int m = 0; m < M; ++m) {
        float s = 0.f;
        for (int i = 0; i < D; ++i) {
          const float t = r[(int64_t)i * M + m] - q[(int64_t)i * N + n];
          s = fmaf(t, t, s);
        }
        if (cnt < k || s < bd[k - 1]) {
          int pos = cnt < k ? cnt : k - 1;
          while (pos > 0 && bd[pos - 1] > s) { bd[pos] = bd[pos - 1]; bi[pos] = bi[pos - 1]; --pos; }
          bd[pos] = s;
          bi[pos] = m;
          if (cnt < k) ++cnt;
        }
      }
      for (int j = 0; j < k; ++j) {
        idx[((int64_t)b * k + j) * N + n] = (int64_t)bi[j] + 1;
        dist[((int64_t)b * k + j) * N + n] = sqrtf(bd[j]);
      }
    }
  }
}


/* Voting resample, restating include/nn/common/resample.h:105-124 (one vote per input pixel),
 * include/core/interpolation.h:241-257 (Vote2D: votes outside the target image are dropped) and
 * src/nn/cpp/voting_resample_layer.cpp:8-38 (per image: zeroed vote table, then argmax over the
 * candidates - the first maximum, so the smallest label among equals and 0 for an empty pixel).
 * labels (B, C, IH, IW), map (IH, IW, 2) = (x, y) targets, out (B, C, OH, OW); all int64.
 * Labels outside [0, nc) are skipped (the reference writes outside its table for them).
 * resample.h:122 starts channel c's votes c * OH * OW entries into the image's (C, OH, OW, nc) table
 * (not c * OH * OW * nc), so the channels of an image with C > 1 overlap; restated as it is. */
void oracle_voting_resample(const int64_t* labels, const int64_t* map, int B, int C, int IH, int IW,
                            int OH, int OW, int nc, int64_t* out) {
#pragma omp parallel for schedule(static)
  for (int64_t b = 0; b < B; ++b) {
    int64_t* votes = (int64_t*)calloc((size_t)C * OH * OW * nc, sizeof(int64_t));
    for (int64_t c = 0; c < C; ++c) {
      const int64_t* in = labels + (b * C + c) * IH * IW;
      for (int64_t i = 0; i < (int64_t)IH * IW; ++i) {
        const int64_t x = map[2 * i], y = map[2 * i + 1], l = in[i];
        if (x < 0 || x > OW - 1 || y < 0 || y > OH - 1 || l < 0 || l >= nc) continue;
        votes[c * OH * OW + (y * OW + x) * nc + l] += 1;
      }
    }
    for (int64_t q = 0; q < (int64_t)C * OH * OW; ++q) {
      int64_t best = votes[q * nc], arg = 0;
      for (int k = 1; k < nc; ++k)
        if (votes[q * nc + k] > best) { best = votes[q * nc + k]; arg = k; }
      out[b * C * OH * OW + q] = arg;
    }
    free(votes);
  }
}

/* Cube map -> equirectangular image, restating Cube2RectKernel, include/util/cuda/cube2rect.cuh:15-62,
 * with the conversions of include/core/conversions.h:21-38 (pixel -> longitude / latitude -> unit
 * vector) and :66-135 (unit vector -> cube face and position on it: six tests in order, a later
 * hit replaces an earlier one) and the face sampling of include/core/interpolation.h:85-102
 * (nearest) and :17-33,124-154 (bilinear), which the kernel calls with the face's first column as
 * origin, cube_dim rows and the full 6 * cube_dim row as width.  cube (C, D, 6 D), rect (C, RH, RW). */
#define CUBE2RECT(NAME, T, SIN, COS, FABS, FLOOR)                                                     \
  void NAME(const T* cube, int C, int D, int RH, int RW, int interp, T* rect) {                       \
    const int64_t row = 6 * (int64_t)D, per = (int64_t)D * row, total = (int64_t)C * per;             \
    for (int64_t yr = 0; yr < RH; ++yr)                                                               \
      for (int64_t xr = 0; xr < RW; ++xr) {                                                           \
        const T lon = (T)(2 * M_PI * ((T)xr - (T)RW / 2) / (T)RW);                                    \
        const T lat = (T)(M_PI * ((T)yr - ((T)RH - 1) / 2) / ((T)RH - 1));                            \
        const T x = COS(lat) * SIN(lon), y = -SIN(lat), z = COS(lat) * COS(lon);                      \
        const T ax = FABS(x), ay = FABS(y), az = FABS(z);                                             \
        int64_t face = 0;                                                                             \
        T m = 1, uc = 0, vc = 0;                                                                      \
        if (x > 0 && ax >= ay && ax >= az) { m = ax; uc = -z; vc = -y; face = 3; }                    \
        if (!(x > 0) && ax >= ay && ax >= az) { m = ax; uc = z; vc = -y; face = 1; }                  \
        if (y > 0 && ay >= ax && ay >= az) { m = ay; uc = x; vc = z; face = 4; }                      \
        if (!(y > 0) && ay >= ax && ay >= az) { m = ay; uc = x; vc = -z; face = 5; }                  \
        if (z > 0 && az >= ax && az >= ay) { m = az; uc = x; vc = -y; face = 2; }                     \
        if (!(z > 0) && az >= ax && az >= ay) { m = az; uc = -x; vc = -y; face = 0; }                 \
        const T u = (T)0.5 * (uc / m + (T)1) * (T)(D - 1), v = (T)0.5 * (vc / m + (T)1) * (T)(D - 1); \
        for (int c = 0; c < C; ++c) {                                                                 \
          const int64_t base = (int64_t)c * per + face * D;                                           \
          T res;                                                                                      \
          if (interp == 0) {                                                                          \
            const int64_t xi = llround((double)u), yi = llround((double)v);                           \
            const int64_t f = base + yi * row + xi;                                                   \
            res = xi >= 0 && xi <= row - 1 && yi >= 0 && yi <= D - 1 && f < total ? cube[f] : (T)0;   \
          } else {                                                                                    \
            const int64_t x1 = (int64_t)FLOOR(u), y1 = (int64_t)FLOOR(v), x2 = x1 + 1, y2 = y1 + 1;   \
            const int x1v = x1 >= 0 && x1 <= row - 1, x2v = x2 >= 0 && x2 <= row - 1;                 \
            const int y1v = y1 >= 0 && y1 <= D - 1, y2v = y2 >= 0 && y2 <= D - 1;                     \
            const int64_t f11 = base + y1 * row + x1, f21 = base + y1 * row + x2;                     \
            const int64_t f12 = base + y2 * row + x1, f22 = base + y2 * row + x2;                     \
            const T d11 = x1v && y1v && f11 < total ? cube[f11] : (T)0;                               \
            const T d21 = x2v && y1v && f21 < total ? cube[f21] : (T)0;                               \
            const T d12 = x1v && y2v && f12 < total ? cube[f12] : (T)0;                               \
            const T d22 = x2v && y2v && f22 < total ? cube[f22] : (T)0;                               \
            const T a = (T)y2 - v, b = (T)x2 - u, cc = u - (T)x1, d = v - (T)y1;                      \
            res = a * b * d11 + a * cc * d21 + d * b * d12 + d * cc * d22;                            \
          }                                                                                           \
          rect[((int64_t)c * RH + yr) * RW + xr] = res;                                               \
        }                                                                                             \
      }                                                                                               \
  }
CUBE2RECT(oracle_cube2rect_f32, float, sinf, cosf, fabsf, floorf)
CUBE2RECT(oracle_cube2rect_f64, double, sin, cos, fabs, floor)
