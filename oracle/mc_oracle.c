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
 * oracle_knn: PARITY UNPINNED - the reference has no CPU k-NN, no k-NN test, and its CUDA k-NN
 * indexes a k x N buffer as an M x N matrix (src/util/cuda/knn_layer.cu:22-27 against
 * include/util/cuda/knn.cuh:112,169-170), so it cannot produce vectors.  It restates knn.cuh.
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
