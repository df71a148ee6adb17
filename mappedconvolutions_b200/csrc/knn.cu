// Brute-force k nearest neighbours without the N x M distance matrix.
//
// Each thread owns one query point and a sorted top-k list held in registers; reference points
// stream through shared memory in tiles that every thread of the block reads as a broadcast.
// Semantics restated from the reference's include/util/cuda/knn.cuh:
//   distance  :82-103   ssd over the dimensions in order, here pinned to s = fmaf(t, t, s) with
//                       t = ref_i - query_i starting from s = 0
//   selection :125-189  stable insertion, strict '<'  ==  order by (distance, index)
//   indices   :141,160,184  1-based
//   sqrt      :199-205
#include "common.cuh"

namespace mc {

template <int KMAX>
struct TopK {
  float d[KMAX];
  int i[KMAX];
  __device__ __forceinline__ void init() {
#pragma unroll
    for (int t = 0; t < KMAX; ++t) { d[t] = INFINITY; i[t] = -1; }
  }
  __device__ __forceinline__ void insert(float v, int j) {
    d[KMAX - 1] = v;
    i[KMAX - 1] = j;
#pragma unroll
    for (int t = KMAX - 1; t > 0; --t) {
      const bool sw = d[t] < d[t - 1];
      const float dt = d[t], dp = d[t - 1];
      const int it = i[t], ip = i[t - 1];
      d[t] = sw ? dp : dt; d[t - 1] = sw ? dt : dp;
      i[t] = sw ? ip : it; i[t - 1] = sw ? it : ip;
    }
  }
};

constexpr int KNN_THREADS = 256;
constexpr int KNN_TILE = 512;
constexpr int KNN_DMAX = 16;

// DT > 0: compile-time dimension; DT == 0: runtime dimension up to KNN_DMAX.
template <int DT, int KMAX>
__global__ void __launch_bounds__(KNN_THREADS) knn_kernel(const float* __restrict__ ref,
                                                          const float* __restrict__ query, int D,
                                                          int M, int N, int k,
                                                          int64_t* __restrict__ idx,
                                                          float* __restrict__ dist) {
  constexpr int DS = DT > 0 ? DT : KNN_DMAX;
  __shared__ float tile[DS][KNN_TILE];
  const int b = blockIdx.y;
  const float* rb = ref + (long)b * D * M;
  const float* qb = query + (long)b * D * N;
  const int n = blockIdx.x * KNN_THREADS + threadIdx.x;
  const bool live = n < N;
  float q[DS];
#pragma unroll
  for (int i = 0; i < DS; ++i) q[i] = (live && i < D) ? qb[(long)i * N + n] : 0.f;
  TopK<KMAX> top;
  top.init();

  for (int m0 = 0; m0 < M; m0 += KNN_TILE) {
    const int cnt = min(KNN_TILE, M - m0);
    __syncthreads();
    for (int t = threadIdx.x; t < DS * KNN_TILE; t += KNN_THREADS) {
      const int i = t / KNN_TILE, j = t % KNN_TILE;
      tile[i][j] = (i < D && j < cnt) ? rb[(long)i * M + m0 + j] : 0.f;
    }
    __syncthreads();
    if (live) {
#pragma unroll 4
      for (int j = 0; j < cnt; ++j) {
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < DS; ++i) {
          const float t = tile[i][j] - q[i];
          s = fmaf(t, t, s);
        }
        if (s < top.d[KMAX - 1]) top.insert(s, m0 + j);
      }
    }
  }
  if (!live) return;
#pragma unroll
  for (int t = 0; t < KMAX; ++t) {
    if (t < k) {
      const long o = ((long)b * k + t) * N + n;
      idx[o] = (int64_t)top.i[t] + 1;
      dist[o] = __fsqrt_rn(top.d[t]);
    }
  }
}

template <int DT>
static void knn_launch_big_k(const float* ref, const float* query, int B, int M, int N, int k,
                             int64_t* idx, float* dist, cudaStream_t st);

// D <= 4: reference points are staged as one float4 each, so that a pair costs one 16-byte
// broadcast load instead of D 4-byte ones (the shared-memory pipe, not the FMA pipe, was the limit).
constexpr int KNN2_THREADS = 256;
constexpr int KNN2_TILE = 1024;

template <int DT, int KMAX>
__global__ void __launch_bounds__(KNN2_THREADS) knn_small_d_kernel(const float* __restrict__ ref,
                                                                   const float* __restrict__ query,
                                                                   int M, int N, int k,
                                                                   int64_t* __restrict__ idx,
                                                                   float* __restrict__ dist) {
  __shared__ float4 tile[KNN2_TILE];
  const int b = blockIdx.y;
  const float* rb = ref + (long)b * DT * M;
  const float* qb = query + (long)b * DT * N;
  const int n = blockIdx.x * KNN2_THREADS + threadIdx.x;
  const bool live = n < N;
  float q[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int i = 0; i < DT; ++i)
    if (live) q[i] = qb[(long)i * N + n];
  TopK<KMAX> top;
  top.init();
  for (int m0 = 0; m0 < M; m0 += KNN2_TILE) {
    const int cnt = min(KNN2_TILE, M - m0);
    __syncthreads();
    for (int j = threadIdx.x; j < cnt; j += KNN2_THREADS) {
      float4 r = make_float4(0.f, 0.f, 0.f, 0.f);
      r.x = rb[m0 + j];
      if (DT > 1) r.y = rb[(long)M + m0 + j];
      if (DT > 2) r.z = rb[2L * M + m0 + j];
      if (DT > 3) r.w = rb[3L * M + m0 + j];
      tile[j] = r;
    }
    __syncthreads();
    if (live) {
#pragma unroll 8
      for (int j = 0; j < cnt; ++j) {
        const float4 r = tile[j];
        const float rr[4] = {r.x, r.y, r.z, r.w};
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < DT; ++i) {
          const float a = rr[i] - q[i];
          s = fmaf(a, a, s);
        }
        if (s < top.d[KMAX - 1]) top.insert(s, m0 + j);
      }
    }
  }
  if (!live) return;
#pragma unroll
  for (int t = 0; t < KMAX; ++t) {
    if (t < k) {
      const long o = ((long)b * k + t) * N + n;
      idx[o] = (int64_t)top.i[t] + 1;
      dist[o] = __fsqrt_rn(top.d[t]);
    }
  }
}

template <int DT>
static void knn_small_d_launch(const float* ref, const float* query, int B, int M, int N, int k,
                               int64_t* idx, float* dist, cudaStream_t st) {
  dim3 grid((unsigned)((N + KNN2_THREADS - 1) / KNN2_THREADS), (unsigned)B);
  if (k <= 8) knn_small_d_kernel<DT, 8><<<grid, KNN2_THREADS, 0, st>>>(ref, query, M, N, k, idx, dist), MC_COUNT(1);
  else if (k <= 16) knn_small_d_kernel<DT, 16><<<grid, KNN2_THREADS, 0, st>>>(ref, query, M, N, k, idx, dist), MC_COUNT(1);
  else knn_launch_big_k<DT>(ref, query, B, M, N, k, idx, dist, st);
}

template <int DT>
static void knn_launch_k(const float* ref, const float* query, int B, int D, int M, int N, int k,
                         int64_t* idx, float* dist, cudaStream_t st) {
  dim3 grid((unsigned)((N + KNN_THREADS - 1) / KNN_THREADS), (unsigned)B);
  if (k <= 8) knn_kernel<DT, 8><<<grid, KNN_THREADS, 0, st>>>(ref, query, D, M, N, k, idx, dist), MC_COUNT(1);
  else if (k <= 16) knn_kernel<DT, 16><<<grid, KNN_THREADS, 0, st>>>(ref, query, D, M, N, k, idx, dist), MC_COUNT(1);
  else knn_kernel<DT, 32><<<grid, KNN_THREADS, 0, st>>>(ref, query, D, M, N, k, idx, dist), MC_COUNT(1);
}

template <int DT>
static void knn_launch_big_k(const float* ref, const float* query, int B, int M, int N, int k,
                             int64_t* idx, float* dist, cudaStream_t st) {
  knn_launch_k<DT>(ref, query, B, DT, M, N, k, idx, dist, st);
}

}  // namespace mc

extern "C" int mc_knn(const float* ref, const float* query, int32_t B, int32_t D, int32_t M,
                      int32_t N, int32_t k, int64_t* idx, float* dist, void* stream) {
  using namespace mc;
  if (!ref || !query || !idx || !dist) return MC_ERR_BAD_ARG;
  if (B <= 0 || D <= 0 || M <= 0 || N <= 0 || k <= 0) return MC_ERR_BAD_ARG;
  if (k > 32 || D > KNN_DMAX || B > 65535) return MC_ERR_TOO_LARGE;
  if (k > M) return MC_ERR_BAD_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  switch (D) {
    case 1: knn_small_d_launch<1>(ref, query, B, M, N, k, idx, dist, st); break;
    case 2: knn_small_d_launch<2>(ref, query, B, M, N, k, idx, dist, st); break;
    case 3: knn_small_d_launch<3>(ref, query, B, M, N, k, idx, dist, st); break;
    case 4: knn_small_d_launch<4>(ref, query, B, M, N, k, idx, dist, st); break;
    default: knn_launch_k<0>(ref, query, B, D, M, N, k, idx, dist, st); break;
  }
  MC_CHECK_LAUNCH();
  return MC_OK;
}
