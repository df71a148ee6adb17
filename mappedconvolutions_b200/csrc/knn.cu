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

// D <= 4: reference points are staged per coordinate and visited two at a time with packed
// fp32 arithmetic (fma.rn.f32x2): difference and square-accumulate of a PAIR of references cost
// one instruction each per dimension.  Every lane of a packed operation is the same correctly
// rounded operation as its scalar form (r - q as fma(r, 1, -q), then s = fma(t, t, s) from 0), so
// distances - and with them the order of near ties - are bit-identical to the scalar kernel.
// Blocks of 128 threads, nine to an SM (56 registers): 170 496 resident queries, so that the
// 163 842 vertices of a level-7 icosphere run as ONE wave instead of one full wave and a sliver.
constexpr int KNN2_THREADS = 128;
constexpr int KNN2_BLOCKS_PER_SM = 9;
constexpr int KNN2_TILE = 1024;

__device__ __forceinline__ float2 fma2(const float2& a, const float2& b, const float2& c) {
  float2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;"
      : "=l"(reinterpret_cast<unsigned long long&>(d))
      : "l"(reinterpret_cast<const unsigned long long&>(a)),
        "l"(reinterpret_cast<const unsigned long long&>(b)),
        "l"(reinterpret_cast<const unsigned long long&>(c)));
  return d;
}

template <int DT, int KMAX>
__global__ void __launch_bounds__(KNN2_THREADS, KMAX <= 12 ? KNN2_BLOCKS_PER_SM : 8) knn_small_d_kernel(const float* __restrict__ ref,
                                                                   const float* __restrict__ query,
                                                                   int M, int N, int k,
                                                                   int64_t* __restrict__ idx,
                                                                   float* __restrict__ dist) {
  __shared__ __align__(16) float tile[DT][KNN2_TILE];
  const int b = blockIdx.y;
  const float* rb = ref + (long)b * DT * M;
  const float* qb = query + (long)b * DT * N;
  const int n = blockIdx.x * KNN2_THREADS + threadIdx.x;
  const bool live = n < N;
  float2 nq[DT];  // (-q_i, -q_i)
#pragma unroll
  for (int i = 0; i < DT; ++i) {
    const float v = live ? qb[(long)i * N + n] : 0.f;
    nq[i] = make_float2(-v, -v);
  }
  const float2 one = make_float2(1.f, 1.f), zero = make_float2(0.f, 0.f);
  TopK<KMAX> top;
  top.init();
  for (int m0 = 0; m0 < M; m0 += KNN2_TILE) {
    const int cnt = min(KNN2_TILE, M - m0);
    const int cnt2 = (cnt + 3) & ~3;  // the tail is padded with points at infinity
    __syncthreads();
    for (int j = threadIdx.x; j < cnt2; j += KNN2_THREADS) {
#pragma unroll
      for (int i = 0; i < DT; ++i) tile[i][j] = j < cnt ? rb[(long)i * M + m0 + j] : INFINITY;
    }
    __syncthreads();
    if (live) {
#pragma unroll 2
      for (int j = 0; j < cnt2; j += 4) {
        float2 s0 = zero, s1 = zero;
#pragma unroll
        for (int i = 0; i < DT; ++i) {
          const float4 r = *reinterpret_cast<const float4*>(&tile[i][j]);
          const float2 t0 = fma2(make_float2(r.x, r.y), one, nq[i]);  // r - q
          const float2 t1 = fma2(make_float2(r.z, r.w), one, nq[i]);
          s0 = fma2(t0, t0, s0);
          s1 = fma2(t1, t1, s1);
        }
        // one test for the four candidates; the list is rarely touched after the first few tiles
        if (fminf(fminf(s0.x, s0.y), fminf(s1.x, s1.y)) < top.d[KMAX - 1]) {
          if (s0.x < top.d[KMAX - 1]) top.insert(s0.x, m0 + j);
          if (s0.y < top.d[KMAX - 1]) top.insert(s0.y, m0 + j + 1);
          if (s1.x < top.d[KMAX - 1]) top.insert(s1.x, m0 + j + 2);
          if (s1.y < top.d[KMAX - 1]) top.insert(s1.y, m0 + j + 3);
        }
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
  else if (k <= 12) knn_small_d_kernel<DT, 12><<<grid, KNN2_THREADS, 0, st>>>(ref, query, M, N, k, idx, dist), MC_COUNT(1);
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
