// Tensor-core mapped convolution for bf16 channels-last activations: an implicit GEMM whose A
// operand never exists in global memory.
//
//   forward:  y[pixel, co] = sum_{tap, ci} A[pixel, (tap, ci)] * W[co, ci, tap] + bias[co]
//             A[pixel, (tap, ci)] = interp(x[., ci], map[pixel, tap])
//
// One persistent CTA per SM works on tiles of 128 output pixels:
//   * producer warps read the sample map, gather the (up to four) source pixels of every
//     (pixel, tap) as 16-byte channel vectors, blend them in fp32 and write the bf16 row straight
//     into a 128-byte-swizzled shared-memory stage (one stage = one tap = a 128 x 64 K-slice);
//   * one thread issues tcgen05.mma (M = 128, N = C_out, K = 16) from those stages against the
//     weight slices, which stay resident in shared memory, accumulating fp32 in tensor memory;
//   * four epilogue warps read the accumulators back with tcgen05.ld, add the bias and store bf16.
// Stages and the two accumulator buffers are handed over through mbarriers; every wait is bounded
// and raises a status word instead of spinning forever.
//
// Replaces the per-batch im2col + cublasSgemm + bias sequence of the reference's
// src/nn/cuda/mapped_convolution_layer.cu:39-70.
#include "common.cuh"
#include "tc_common.cuh"

namespace mc {
namespace tc {

constexpr int TILE_M = 128;
constexpr int STAGE_BYTES = TILE_M * 128;  // 128 rows x 64 bf16
constexpr int N_PRODUCER_WARPS = 16;
constexpr int N_EPI_WARPS = 4;
constexpr int FWD_THREADS = (1 + N_EPI_WARPS + N_PRODUCER_WARPS) * 32;

struct FwdArgs {
  const bf16* x;      // (B, IH*IW, Cin) channels-last
  const float* map;   // (OH*OW, K, 2)
  const uint4* wimg;  // weight slices in their shared-memory image
  const bf16* bias;   // may be null
  bf16* y;            // (B, OH*OW, NOUT) channels-last
  int Cin, IH, IW, OW, K, interp;
  int nsl;    // number of 64-wide K slices = K * Cin / 64
  int nst;    // pipeline stages
  long opix;  // OH*OW
  long mtot;  // B*OH*OW
  int tiles;
  int tile2d, tiles_x, tiles_per_img;
};

// Weight (Cout, Cin, K) -> nsl slices of [Cout rows][64 channels] bf16, each row 128 bytes with
// its 16-byte chunks XOR-swizzled by (row & 7): exactly what tcgen05.mma expects for a K-major
// operand with the 128-byte swizzle, so the kernel copies it into shared memory linearly.
// transpose = 1 builds the dgrad operand instead: rows are input channels, the 64-wide slices run
// over output channels (requires Cout % 64 == 0).
__global__ void weight_image_kernel(const bf16* __restrict__ w, uint16_t* __restrict__ img, int rows,
                                    int red, int K, int transpose, int Cin_w) {
  // rows: operand rows (N of the GEMM); red: reduction channels per tap (multiple of 64)
  const int cpb = red / 64;
  const long total = (long)K * cpb * rows * 64;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total;
       i += (long)gridDim.x * blockDim.x) {
    const int c = (int)(i % 64);
    const int n = (int)((i / 64) % rows);
    const int s = (int)(i / (64L * rows));
    const int tap = s / cpb, cb = s % cpb;
    const int r = cb * 64 + c;
    // forward: w[n][r][tap] with n = co, r = ci.   transpose: w[r][n][tap] with r = co, n = ci.
    const long src = transpose ? ((long)r * Cin_w + n) * K + tap : ((long)n * Cin_w + r) * K + tap;
    const long dst = (long)s * rows * 64 + (long)n * 64 + ((((c >> 3) ^ (n & 7)) << 3) | (c & 7));
    img[dst] = reinterpret_cast<const uint16_t*>(w)[src];
  }
}

__device__ __forceinline__ void tile_pixel(const FwdArgs& a, int tile, int r, long& gp, int& img,
                                           long& p, bool& valid) {
  if (a.tile2d) {
    img = tile / a.tiles_per_img;
    const int tt = tile % a.tiles_per_img;
    const int ty = tt / a.tiles_x, tx = tt % a.tiles_x;
    p = (long)(ty * 8 + (r >> 4)) * a.OW + tx * 16 + (r & 15);
    gp = (long)img * a.opix + p;
    valid = true;
  } else {
    gp = (long)tile * TILE_M + r;
    valid = gp < a.mtot;
    img = valid ? (int)(gp / a.opix) : 0;
    p = valid ? gp % a.opix : 0;
  }
}

template <int NOUT>
__global__ void __launch_bounds__(FWD_THREADS, 1) conv_fwd_tc_kernel(const FwdArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // carve-up (base is 1024-byte aligned by the runtime for dynamic shared memory of this size)
  uint8_t* sm = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* stages = sm;
  uint8_t* wsm = stages + (size_t)a.nst * STAGE_BYTES;
  float* bias_s = (float*)(wsm + (size_t)a.nsl * NOUT * 128);
  uint64_t* bars = (uint64_t*)(bias_s + NOUT);
  // bars: full[nst], empty[nst], tfull[2], tempty[2], drain
  uint32_t* misc = (uint32_t*)(bars + 2 * a.nst + 5);
  volatile int* abort_flag = (volatile int*)(misc + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t stage0 = smem_u32(stages), w0 = smem_u32(wsm);
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (a.nst + s); };
  auto tfull_bar = [&](int i) { return bar0 + 8u * (2 * a.nst + i); };
  auto tempty_bar = [&](int i) { return bar0 + 8u * (2 * a.nst + 2 + i); };
  const uint32_t drain_bar = bar0 + 8u * (2 * a.nst + 4);
  constexpr uint32_t TMEM_COLS = 2 * NOUT < 32 ? 32 : 2 * NOUT;

  if (threadIdx.x == 0) {
    for (int s = 0; s < a.nst; ++s) {
      mbar_init(full_bar(s), N_PRODUCER_WARPS * 32);
      mbar_init(empty_bar(s), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(tfull_bar(i), 1);
      mbar_init(tempty_bar(i), N_EPI_WARPS * 32);
    }
    mbar_init(drain_bar, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  // resident operands: weight slices and bias
  for (int i = threadIdx.x; i < a.nsl * NOUT * 8; i += FWD_THREADS)
    sts16(w0 + 16u * i, ldg16(a.wimg + i));
  for (int i = threadIdx.x; i < NOUT; i += FWD_THREADS)
    bias_s[i] = a.bias ? __bfloat162float(a.bias[i]) : 0.f;
  fence_proxy_async_smem();
  if (warp == 0) tmem_alloc(smem_u32(misc), TMEM_COLS);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *misc;

  if (warp == 0) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(TILE_M, NOUT, 0, 0);
      uint32_t n = 0, it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < a.tiles && ok; tile += gridDim.x, ++it) {
        const uint32_t acc = it & 1, aph = (it >> 1) & 1;
        ok = mbar_wait(tempty_bar(acc), aph ^ 1, abort_flag, 0x11);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + acc * NOUT;
        for (int s = 0; s < a.nsl; ++s, ++n) {
          const uint32_t st = n % a.nst, ph = (n / a.nst) & 1;
          ok = mbar_wait(full_bar(st), ph, abort_flag, 0x12);
          if (!ok) break;
          tc_fence_after_sync();
          const uint64_t adesc = make_desc_sw128(stage0 + st * STAGE_BYTES, 16, 1024);
          const uint64_t bdesc = make_desc_sw128(w0 + (uint32_t)s * NOUT * 128, 16, 1024);
#pragma unroll
          for (int j = 0; j < 4; ++j)  // four K = 16 steps inside the 64-wide slice: +32 bytes each
            mma_bf16_ss(tmem_d, adesc + 2 * j, bdesc + 2 * j, idesc, (s | j) != 0);
          mma_commit(empty_bar(st));  // frees the stage when these MMAs have read it
        }
        if (ok) mma_commit(tfull_bar(acc));
      }
      // make sure nothing of ours is still in flight before TMEM is released
      mma_commit(drain_bar);
      mbar_wait(drain_bar, 0, abort_flag, 0x13);
    }
    __syncwarp();
  } else if (warp <= N_EPI_WARPS) {
    // ------------------------------------------------------------------ epilogue
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const int r = q * 32 + lane;
    uint32_t it = 0;
    for (int tile = blockIdx.x; tile < a.tiles; tile += gridDim.x, ++it) {
      const uint32_t acc = it & 1, aph = (it >> 1) & 1;
      long gp, p;
      int img;
      bool valid;
      tile_pixel(a, tile, r, gp, img, p, valid);
      if (!mbar_wait(tfull_bar(acc), aph, abort_flag, 0x21)) break;
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + acc * NOUT;
      uint4* out = reinterpret_cast<uint4*>(a.y + gp * NOUT);
#pragma unroll
      for (int cc = 0; cc < NOUT / 32; ++cc) {
        uint32_t v[32];
        tmem_ld_32x32(taddr + cc * 32, v);
        tmem_ld_wait();
        if (cc == NOUT / 32 - 1) {
          // accumulator fully read: hand the buffer back before the global stores
          tc_fence_before_sync();
          mbar_arrive(tempty_bar(acc));
        }
        if (valid) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 o;
            const float* bs = bias_s + cc * 32 + j * 8;
            o.x = pack_bf16x2(__uint_as_float(v[j * 8 + 0]) + bs[0], __uint_as_float(v[j * 8 + 1]) + bs[1]);
            o.y = pack_bf16x2(__uint_as_float(v[j * 8 + 2]) + bs[2], __uint_as_float(v[j * 8 + 3]) + bs[3]);
            o.z = pack_bf16x2(__uint_as_float(v[j * 8 + 4]) + bs[4], __uint_as_float(v[j * 8 + 5]) + bs[5]);
            o.w = pack_bf16x2(__uint_as_float(v[j * 8 + 6]) + bs[6], __uint_as_float(v[j * 8 + 7]) + bs[7]);
            out[cc * 4 + j] = o;
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ producers
    const int pw = warp - 1 - N_EPI_WARPS;
    const int g = lane >> 3, lg = lane & 7;  // 8 lanes cover the 128 bytes of one row
    const int cpb = a.Cin / 64;
    const long ipix = (long)a.IH * a.IW;
    uint32_t n = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < a.tiles && ok; tile += gridDim.x) {
      for (int s = 0; s < a.nsl; ++s, ++n) {
        const uint32_t st = n % a.nst, ph = (n / a.nst) & 1;
        const int tap = s / cpb, cb = s % cpb;
        int okw = 1;
        if (lane == 0) okw = mbar_wait(empty_bar(st), ph ^ 1, abort_flag, 0x31) ? 1 : 0;
        okw = __shfl_sync(0xffffffffu, okw, 0);
        if (!okw) { ok = false; break; }
        const uint32_t sbase = stage0 + st * STAGE_BYTES;
        for (int r = pw * 4 + g; r < TILE_M; r += N_PRODUCER_WARPS * 4) {
          long gp, p;
          int img;
          bool valid;
          tile_pixel(a, tile, r, gp, img, p, valid);
          Tap<float> tp;
          tp.n = 0;
          if (valid) {
            const float2 m = __ldg(reinterpret_cast<const float2*>(a.map) + p * a.K + tap);
            decode_tap<float, float>(m.x, m.y, a.IH, a.IW, a.interp, tp);
          }
          const bf16* xb = a.x + ((long)img * ipix) * a.Cin + cb * 64 + lg * 8;
          uint4 v[4];
          float wv[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const bool on = i < tp.n && tp.off[i] >= 0 && tp.w[i] != 0.f;
            wv[i] = on ? tp.w[i] : 0.f;
            v[i] = on ? ldg16(xb + (long)tp.off[i] * a.Cin) : make_uint4(0, 0, 0, 0);
          }
          float acc[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            bf16x2_fma(v[i].x, wv[i], acc[0], acc[1]);
            bf16x2_fma(v[i].y, wv[i], acc[2], acc[3]);
            bf16x2_fma(v[i].z, wv[i], acc[4], acc[5]);
            bf16x2_fma(v[i].w, wv[i], acc[6], acc[7]);
          }
          uint4 o;
          o.x = pack_bf16x2(acc[0], acc[1]);
          o.y = pack_bf16x2(acc[2], acc[3]);
          o.z = pack_bf16x2(acc[4], acc[5]);
          o.w = pack_bf16x2(acc[6], acc[7]);
          sts16(sbase + r * 128 + ((lg ^ (r & 7)) << 4), o);
        }
        fence_proxy_async_smem();
        mbar_arrive(full_bar(st));
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

static int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
  }
  return n;
}

static size_t fwd_smem_bytes(int nst, int nsl, int nout) {
  return 1024 + (size_t)nst * STAGE_BYTES + (size_t)nsl * nout * 128 + nout * 4 +
         (2 * nst + 5) * 8 + 16;
}

// Number of pipeline stages that fit beside the resident weights (0 = does not fit).
static int fwd_stages(int nsl, int nout) {
  for (int nst = 8; nst >= 3; --nst)
    if (fwd_smem_bytes(nst, nsl, nout) <= 200 * 1024) return nst;
  return 0;
}

}  // namespace tc

using namespace tc;

bool conv_tc_fwd_supported(const mc_desc* d) {
  if (d->dtype != MC_BF16 || d->layout != MC_NHWC || d->P != 0) return false;
  if (d->C_in % 64 != 0 || d->C_out != 64) return false;
  const int nsl = d->K * (d->C_in / 64);
  return fwd_stages(nsl, d->C_out) > 0;
}

size_t conv_tc_fwd_ws(const mc_desc* d) {
  return (size_t)d->K * d->C_in * d->C_out * sizeof(bf16);
}

int conv_tc_fwd_launch(const mc_desc* d, const void* x, const void* map, const void* w,
                       const void* bias, void* y, void* ws, size_t ws_bytes, cudaStream_t st) {
  if (!ws || ws_bytes < conv_tc_fwd_ws(d)) return MC_ERR_WORKSPACE;
  if (((uintptr_t)x | (uintptr_t)y | (uintptr_t)ws | (uintptr_t)map) & 15) return MC_ERR_BAD_ARG;
  FwdArgs a;
  a.x = (const bf16*)x; a.map = (const float*)map; a.wimg = (const uint4*)ws;
  a.bias = (const bf16*)bias; a.y = (bf16*)y;
  a.Cin = d->C_in; a.IH = d->IH; a.IW = d->IW; a.OW = d->OW; a.K = d->K; a.interp = d->interp;
  a.nsl = d->K * (d->C_in / 64);
  a.nst = fwd_stages(a.nsl, d->C_out);
  a.opix = (long)d->OH * d->OW;
  a.mtot = (long)d->B * a.opix;
  a.tile2d = (d->OH % 8 == 0 && d->OW % 16 == 0) ? 1 : 0;
  a.tiles_x = d->OW / 16;
  a.tiles_per_img = (d->OH / 8) * (d->OW / 16);
  const long tiles = a.tile2d ? (long)d->B * a.tiles_per_img : (a.mtot + TILE_M - 1) / TILE_M;
  if (tiles >= (1L << 31)) return MC_ERR_TOO_LARGE;
  a.tiles = (int)tiles;
  const long nw = (long)d->K * d->C_in * d->C_out;
  weight_image_kernel<<<grid_for(nw, 256), 256, 0, st>>>((const bf16*)w, (uint16_t*)ws, d->C_out,
                                                         d->C_in, d->K, 0, d->C_in), MC_COUNT(1);
  const size_t smem = fwd_smem_bytes(a.nst, a.nsl, d->C_out);
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(conv_fwd_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             220 * 1024) != cudaSuccess)
      return MC_ERR_LAUNCH;
    attr_set = true;
  }
  const int grid = a.tiles < sm_count() ? a.tiles : sm_count();
  conv_fwd_tc_kernel<64><<<grid, FWD_THREADS, smem, st>>>(a), MC_COUNT(1);
  MC_CHECK_LAUNCH();
  return MC_OK;
}

bool conv_tc_dgrad_supported(const mc_desc*) { return false; }
size_t conv_tc_dgrad_ws(const mc_desc*) { return 0; }
int conv_tc_dgrad_launch(const mc_desc*, const void*, const void*, const void*, const void*, void*,
                         void*, size_t, cudaStream_t) { return MC_ERR_UNSUPPORTED; }
bool conv_tc_wgrad_supported(const mc_desc*) { return false; }
size_t conv_tc_wgrad_ws(const mc_desc*) { return 0; }
int conv_tc_wgrad_launch(const mc_desc*, const void*, const void*, const void*, void*, void*, void*,
                         size_t, cudaStream_t) { return MC_ERR_UNSUPPORTED; }

int device_status_read(cudaStream_t st, int reset) {
  int v = 0;
  if (cudaStreamSynchronize(st) != cudaSuccess) return MC_ERR_LAUNCH;
  if (cudaMemcpyFromSymbol(&v, tc::g_status, sizeof(int)) != cudaSuccess) return MC_ERR_LAUNCH;
  if (reset && v != 0) {
    const int z = 0;
    cudaMemcpyToSymbol(tc::g_status, &z, sizeof(int));
  }
  return v;
}

}  // namespace mc
