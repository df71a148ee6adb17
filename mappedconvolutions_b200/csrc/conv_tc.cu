// Tensor-core mapped convolution for bf16 channels-last activations: implicit GEMMs whose
// interpolated operand never exists in global memory.
//
//   forward: y[pix, co]  = sum_{tap, ci} A[pix, (tap, ci)] * W[co, ci, tap] + bias[co]
//            A[pix, (tap, ci)] = interp(x[., ci], map[pix, tap])
//   dgrad  : gx[q, ci]   = sum_{tap, co} G[q, (tap, co)] * W[co, ci, tap]
//            G[q, (tap, co)] = sum over the (pix, corner) pairs of tap that land on input pixel q
//                              of weight * gy[pix, co]        (gather through the inverse map;
//                              no atomics, deterministic)
//   wgrad  : gw[co, ci, tap] = sum_{pix} gy[pix, co] * A[pix, (tap, ci)]
//
// One persistent CTA per SM works on tiles of 128 pixels:
//   * producer warps build A (or G) rows: they read the sample map (or the inverse-map lists),
//     gather the source pixels as 16-byte channel vectors, blend them in fp32 and write the bf16
//     row into a 128-byte-swizzled shared-memory stage (one stage = 128 pixels x 64 channels of
//     one tap);
//   * one thread issues tcgen05.mma from those stages, accumulating fp32 in tensor memory;
//   * four warps read the accumulators back with tcgen05.ld (and, in wgrad, stream the gy tiles).
// The same stage bytes serve as a K-major operand (forward, dgrad: reduction over channels) and as
// an MN-major operand (wgrad: reduction over pixels).  Stages and accumulators are handed over
// through mbarriers; every wait is bounded and raises a status word instead of spinning forever.
//
// Replaces the per-batch im2col / col2im + cublasSgemm sequences of the reference's
// src/nn/cuda/mapped_convolution_layer.cu:39-70, :100-127, :155-190.
#include <cub/device/device_scan.cuh>

#include <atomic>
#include <mutex>
#include <set>
#include <utility>

#include "common.cuh"
#include "tc_common.cuh"

namespace mc {
namespace tc {

constexpr int TILE_M = 128;
constexpr int STAGE_BYTES = TILE_M * 128;  // 128 rows x 64 bf16
constexpr int N_PRODUCER_WARPS = 16;
constexpr int N_EPI_WARPS = 4;
constexpr int N_DEC_WARPS = 3;  // (24 warps in all: the register file is shared out per 4 warps) decode the sample map / inverse map of the NEXT tile
constexpr int FIRST_DEC_WARP = 1 + N_EPI_WARPS;
constexpr int FIRST_PROD_WARP = FIRST_DEC_WARP + N_DEC_WARPS;
constexpr int TC_THREADS = (FIRST_PROD_WARP + N_PRODUCER_WARPS) * 32;
constexpr size_t SMEM_LIMIT = 227 * 1024;  // the most a block may ask for
// forward / dgrad epilogue: every warp turns its 32 rows x 32 columns around in 2 KB of shared
// memory so that its global stores cover whole 64-byte row segments
constexpr size_t EPI_STAGING_BYTES = N_EPI_WARPS * 2048;

// How the pixels of the tiled domain are grouped into 128-row tiles.
struct Tiling {
  long npix;  // pixels per image of the tiled domain
  long mtot;  // batch * npix
  int W;      // width of the tiled domain
  int B;      // batch
  int tiles, tile2d, tiles_x, tiles_per_img;
};

// 2-D tiles are numbered batch-innermost: tile = spatial tile * B + image.  The CTAs that run at the
// same time then work on the same few spatial tiles of every image, so that a tile's slice of the
// tap table comes from DRAM once and from L2 for the other B - 1 images.
__host__ __device__ __forceinline__ int tile_img(const Tiling& t, int tile) { return tile % t.B; }
__host__ __device__ __forceinline__ int tile_spatial(const Tiling& t, int tile) { return tile / t.B; }

static bool make_tiling(Tiling& t, int B, int Hd, int Wd) {
  t.npix = (long)Hd * Wd;
  t.mtot = (long)B * t.npix;
  t.W = Wd;
  t.B = B;
  t.tile2d = (Hd % 8 == 0 && Wd % 16 == 0) ? 1 : 0;  // 8 x 16 pixel tiles keep the footprint small
  t.tiles_x = Wd / 16;
  t.tiles_per_img = (Hd / 8) * (Wd / 16);
  const long n = t.tile2d ? (long)B * t.tiles_per_img : (t.mtot + TILE_M - 1) / TILE_M;
  if (n >= (1L << 31)) return false;
  t.tiles = (int)n;
  return true;
}

__device__ __forceinline__ void tile_pixel(const Tiling& t, int tile, int r, long& gp, int& img,
                                           long& p, bool& valid) {
  if (t.tile2d) {
    img = tile_img(t, tile);
    const int tt = tile_spatial(t, tile);
    const int ty = tt / t.tiles_x, tx = tt % t.tiles_x;
    p = (long)(ty * 8 + (r >> 4)) * t.W + tx * 16 + (r & 15);
    gp = (long)img * t.npix + p;
    valid = true;
  } else {
    gp = (long)tile * TILE_M + r;
    valid = gp < t.mtot;
    img = valid ? (int)(gp / t.npix) : 0;
    p = valid ? gp % t.npix : 0;
  }
}

// One decoded (pixel, tap): up to four source pixels and their weights.  The same 32-byte record
// is used in shared memory and in the prebuilt global tables.
// Every off[] is a VALID pixel index: a corner that contributes nothing (outside the image, zero
// weight, list shorter than four) has weight 0 and points at a pixel that is read anyway, so the
// producers load unconditionally.  (A non-finite input value at such a pixel would therefore leak
// into the output as 0 * inf; inputs are expected to be finite.)
struct TapEnt {
  int off[4];  // source pixel index inside its image; off[3] may carry MORE_FLAG
  float w[4];
};

// What the producer warps gather from.
struct Source {
  const bf16* src;  // (B, spix, C) channels-last tensor that is gathered
  long spix;        // pixels per image of src
  int C;            // channels of src (multiple of 64)
  int SH, SW;       // size of the sampled image (map mode)
  int K, interp;
  const float* map;   // map mode: (npix, K, 2)
  const int* inv_off; // inverse-map mode: (npix * K + 1) list offsets
  const int2* inv_ent;  //                 (source pixel, weight bits) entries
  const TapEnt* tab;    // prebuilt table [pixel of the tiled domain][tap], or null
  const int* tab32;     // nearest maps: the same table as one int per entry (source pixel or -1)
  long src_elems;       // elements of src (batch * spix * C)
  int KC;      // K * C: length of the gathered (tap, channel) axis
  int packed;  // C is not a multiple of 64: a 64-wide slice holds elements tap * C + c of several
               // taps (map mode only).  2: the whole axis fits one slice and the row-per-thread
               // producer builds it straight from the global tap table
};

// Replace the inactive corners of a decoded tap by (some active pixel of the tap, weight 0).
__device__ __forceinline__ void seal_entry(int (&off)[4], float (&w)[4]) {
  int fb = 0;
#pragma unroll
  for (int i = 3; i >= 0; --i)
    if (off[i] >= 0 && w[i] != 0.f) fb = off[i];
#pragma unroll
  for (int i = 0; i < 4; ++i)
    if (off[i] < 0 || w[i] == 0.f) { off[i] = fb; w[i] = 0.f; }
}

struct GemmArgs {
  Source s;
  Tiling t;
  const uint4* wimg;  // fwd / dgrad: weight slices in their shared-memory image
  const bf16* bias;   // fwd / dgrad: per output channel, may be null
  bf16* y;            // fwd / dgrad: (B, npix, NOUT) channels-last
  const bf16* gy;     // wgrad: (B, npix, NOUT) channels-last
  float* gw;          // wgrad: (NOUT, Cin, K) fp32, accumulated atomically
  float* gb;          // wgrad: (NOUT) fp32 or null
  int nsl;            // 64-wide slices of the gathered operand = K * C / 64
  int nst;            // pipeline stages
  int ncol;           // channels of y / gy rows (a CTA works on a chunk of NOUT of them)
  int full_cnt;       // producer warps that arrive on a stage's "full" barrier
  int mtpg;           // wgrad: M = 128 gradient tiles per CTA (blockIdx.y picks the group)
  int relu;           // fwd: y = max(0, .) after the bias
};

__device__ __forceinline__ void blend4(const uint4& v, float w, float (&acc)[8]) {
  bf16x2_fma(v.x, w, acc[0], acc[1]);
  bf16x2_fma(v.y, w, acc[2], acc[3]);
  bf16x2_fma(v.z, w, acc[4], acc[5]);
  bf16x2_fma(v.w, w, acc[6], acc[7]);
}

// ---- producer ------------------------------------------------------------------------------------
// A group of 8 lanes builds one 128-byte row (pixel, tap, 64-channel block) of the gathered
// operand; lane lg owns channels [8 lg, 8 lg + 8).
//
// Map mode (forward, wgrad): the sample map of a tile is decoded ONCE per (pixel, tap) into a
// shared-memory table of (4 source pixels, 4 weights) entries - one coalesced pass over the
// tile's slice of the map by all producer threads - so that the per-row work is two shared loads,
// four predicated 16-byte global loads and the fp32 blend.  The table is double buffered; one
// named barrier per tile keeps the producer warps in step.
// Inverse-map mode (dgrad): every row walks its (source pixel, weight) list straight from global
// memory.


constexpr int N_DEC_THREADS = N_DEC_WARPS * 32;

// Set in off[3] of a table entry whose inverse-map list has more than four entries: the producer
// then walks the rest of the list from global memory (0.5 % of the lists of a gnomonic 3x3 map).
constexpr int MORE_FLAG = 1 << 30;

template <bool CSR>
__device__ __forceinline__ void decode_tile(const Source& s, const Tiling& t, int tile, TapEnt* tab,
                                            int ptid) {
  // per-tile constants (2-D tiles): image and the pixel of the tile's corner
  int img0 = 0, ty = 0, tx = 0;
  if (t.tile2d) {
    img0 = tile_img(t, tile);
    const int tt = tile_spatial(t, tile);
    ty = tt / t.tiles_x;
    tx = tt - ty * t.tiles_x;
  }
  const int n = TILE_M * s.K;
  // entry e = r * K + k; advancing e by the thread count advances (r, k) by fixed steps
  const int dr = N_DEC_THREADS / s.K, dk = N_DEC_THREADS - dr * s.K;
  int r = ptid / s.K, k = ptid - r * s.K;
  // Entries are handled U at a time so that the dependent global loads of a batch (map entry, or
  // list range and then list entries) are all in flight together instead of one after another.
  constexpr int U = 4;
  for (int e0 = ptid; e0 < n; e0 += U * N_DEC_THREADS) {
    long key[U];
    int ibase[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int e = e0 + u * N_DEC_THREADS;
      if (k >= s.K) { k -= s.K; ++r; }
      key[u] = -1;
      ibase[u] = 0;
      if (e < n) {
        long p;
        int img;
        bool valid = true;
        if (t.tile2d) {
          img = img0;
          p = (long)(ty * 8 + (r >> 4)) * t.W + tx * 16 + (r & 15);
        } else {
          const long gp = (long)tile * TILE_M + r;
          valid = gp < t.mtot;
          img = valid ? (int)(gp / t.npix) : 0;
          p = valid ? gp - (long)img * t.npix : 0;
        }
        if (valid) { key[u] = p * s.K + k; ibase[u] = img * (int)s.spix; }
      }
      r += dr;
      k += dk;
    }
    TapEnt ent[U];
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int i = 0; i < 4; ++i) { ent[u].off[i] = -1; ent[u].w[i] = 0.f; }
    if (CSR) {
      int beg[U], end[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        beg[u] = end[u] = 0;
        if (key[u] >= 0) { beg[u] = __ldg(s.inv_off + key[u]); end[u] = __ldg(s.inv_off + key[u] + 1); }
      }
      // the first four (grid pixel, weight) pairs of each list
      int2 en[U][4];
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int i = 0; i < 4; ++i)
          en[u][i] = beg[u] + i < end[u] ? __ldg(s.inv_ent + beg[u] + i) : make_int2(-1, 0);
#pragma unroll
      for (int u = 0; u < U; ++u) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if (en[u][i].x >= 0) {
            ent[u].off[i] = en[u][i].x;
            ent[u].w[i] = __int_as_float(en[u][i].y);
          }
        }
        if (end[u] - beg[u] > 4) ent[u].off[3] |= MORE_FLAG;
      }
    } else {
      float2 m[U];
#pragma unroll
      for (int u = 0; u < U; ++u)
        m[u] = key[u] >= 0 ? __ldg(reinterpret_cast<const float2*>(s.map) + key[u]) : make_float2(0.f, 0.f);
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (key[u] < 0) continue;
        Tap<float> tp;
        decode_tap<float, float>(m[u].x, m[u].y, s.SH, s.SW, s.interp, tp);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const bool on = i < tp.n && tp.off[i] >= 0 && tp.w[i] != 0.f;
          ent[u].off[i] = on ? tp.off[i] : -1;
          ent[u].w[i] = on ? tp.w[i] : 0.f;
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int e = e0 + u * N_DEC_THREADS;
      if (e >= n) continue;
      const int more = (ent[u].off[3] >= 0) ? (ent[u].off[3] & MORE_FLAG) : 0;
      if (more) ent[u].off[3] &= ~MORE_FLAG;
      seal_entry(ent[u].off, ent[u].w);
      ent[u].off[3] |= more;
      uint4* dst = reinterpret_cast<uint4*>(tab + e);
      dst[0] = make_uint4(ent[u].off[0], ent[u].off[1], ent[u].off[2], ent[u].off[3]);
      dst[1] = make_uint4(__float_as_uint(ent[u].w[0]), __float_as_uint(ent[u].w[1]),
                          __float_as_uint(ent[u].w[2]), __float_as_uint(ent[u].w[3]));
    }
  }
}

__device__ __forceinline__ uint4 pack8(const float (&acc)[8]) {
  uint4 o;
  o.x = pack_bf16x2(acc[0], acc[1]);
  o.y = pack_bf16x2(acc[2], acc[3]);
  o.z = pack_bf16x2(acc[4], acc[5]);
  o.w = pack_bf16x2(acc[6], acc[7]);
  return o;
}

// Loads of one row in flight: four source rows (16 bytes per lane each) and their weights.
struct RowLoad {
  uint4 v[4];
  float w[4];
  bool more;  // inverse-map mode: the list continues beyond these four
};

template <bool CSR>
__device__ __forceinline__ void issue_row(const TapEnt* ent, const bf16* sb, int C, RowLoad& L) {
  const uint4* e = reinterpret_cast<const uint4*>(ent);
  const uint4 o = e[0], w = e[1];
  int o3 = (int)o.w;
  L.more = false;
  if (CSR) {
    L.more = (o3 & MORE_FLAG) != 0;
    o3 &= ~MORE_FLAG;
  }
  L.w[0] = __uint_as_float(w.x); L.w[1] = __uint_as_float(w.y);
  L.w[2] = __uint_as_float(w.z); L.w[3] = __uint_as_float(w.w);
  L.v[0] = ldg16(sb + (long)(int)o.x * C);
  L.v[1] = ldg16(sb + (long)(int)o.y * C);
  L.v[2] = ldg16(sb + (long)(int)o.z * C);
  L.v[3] = ldg16(sb + (long)o3 * C);
}

__device__ __forceinline__ void blend_row(const RowLoad& L, float2 (&acc)[4]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) acc[j] = make_float2(0.f, 0.f);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 w2 = make_float2(L.w[i], L.w[i]);
    ffma2_bf16x2(acc[0], w2, L.v[i].x);
    ffma2_bf16x2(acc[1], w2, L.v[i].y);
    ffma2_bf16x2(acc[2], w2, L.v[i].z);
    ffma2_bf16x2(acc[3], w2, L.v[i].w);
  }
}

__device__ __forceinline__ uint4 pack_row(const float2 (&acc)[4]) {
  uint4 o;
  o.x = pack_bf16x2(acc[0].x, acc[0].y);
  o.y = pack_bf16x2(acc[1].x, acc[1].y);
  o.z = pack_bf16x2(acc[2].x, acc[2].y);
  o.w = pack_bf16x2(acc[3].x, acc[3].y);
  return o;
}

// Inverse-map mode, rare (0.5 % of the lists of a gnomonic 3x3 map): entries `first` and up of the
// list `key` = (input pixel, tap).  Runs after the row has been written: it re-reads the bf16 row
// from the stage, adds the remaining terms and writes it back, so that the hot loop keeps no state
// for it.  All arguments are scalars on purpose (no pointers to the kernel's structs, which would
// push them into local memory).
__device__ __noinline__ void add_list_tail(const int* __restrict__ inv_off,
                                           const int2* __restrict__ inv_ent, int C, long key,
                                           const bf16* base, uint32_t saddr, int first) {
  uint4 cur;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(cur.x), "=r"(cur.y), "=r"(cur.z), "=r"(cur.w)
               : "r"(saddr));
  float2 acc[4];
  acc[0] = make_float2(__uint_as_float(cur.x << 16), __uint_as_float(cur.x & 0xFFFF0000u));
  acc[1] = make_float2(__uint_as_float(cur.y << 16), __uint_as_float(cur.y & 0xFFFF0000u));
  acc[2] = make_float2(__uint_as_float(cur.z << 16), __uint_as_float(cur.z & 0xFFFF0000u));
  acc[3] = make_float2(__uint_as_float(cur.w << 16), __uint_as_float(cur.w & 0xFFFF0000u));
  const int end = __ldg(inv_off + key + 1);
  for (int e = __ldg(inv_off + key) + first; e < end; ++e) {
    const int2 en = __ldg(inv_ent + e);
    const uint4 v = ldg16(base + (long)en.x * C);
    const float w = __int_as_float(en.y);
    const float2 w2 = make_float2(w, w);
    ffma2_bf16x2(acc[0], w2, v.x);
    ffma2_bf16x2(acc[1], w2, v.y);
    ffma2_bf16x2(acc[2], w2, v.z);
    ffma2_bf16x2(acc[3], w2, v.w);
  }
  sts16(saddr, pack_row(acc));
}

// Pixel index inside its image of row r of a tile (0 for rows past the end of the batch).
__device__ __forceinline__ int tile_row_pixel(const Tiling& t, int tile, int r) {
  long gp, p;
  int img;
  bool valid;
  tile_pixel(t, tile, r, gp, img, p, valid);
  return valid ? (int)p : 0;
}

// Decoder warps: fill the table half of tile i while the producers gather tile i - 1.
// tab_full / tab_empty: two mbarriers each (one per table half) at tabbar0 + 8 i / + 16 + 8 i.
template <bool CSR>
__device__ __forceinline__ void decoder_loop(const Source& s, const Tiling& t, TapEnt* table,
                                             uint32_t tabbar0, volatile int* abort_flag, int dtid,
                                             int lane) {
  uint32_t it = 0;
  for (int tile = blockIdx.x; tile < t.tiles; tile += gridDim.x, ++it) {
    const uint32_t half = it & 1, ph = (it >> 1) & 1;
    int okw = 1;
    if (lane == 0) okw = mbar_wait(tabbar0 + 16 + 8 * half, ph ^ 1, abort_flag, 0x71) ? 1 : 0;
    okw = __shfl_sync(0xffffffffu, okw, 0);
    if (!okw) return;
    decode_tile<CSR>(s, t, tile, table + (size_t)half * TILE_M * s.K, dtid);
    __syncwarp();
    if (lane == 0) mbar_arrive(tabbar0 + 8 * half);
  }
}

// Prebuilt-table mode: one thread streams the table slice of tile i into its half with bulk
// copies (the copy engine signals the mbarrier with the byte count) while tile i - 1 is gathered.
__device__ __forceinline__ void loader_loop(const Source& s, const Tiling& t, uint32_t table0,
                                            uint32_t tabbar0, volatile int* abort_flag) {
  const uint32_t entb = (uint32_t)s.K * (uint32_t)sizeof(TapEnt);  // bytes per pixel
  uint32_t it = 0;
  for (int tile = blockIdx.x; tile < t.tiles; tile += gridDim.x, ++it) {
    const uint32_t half = it & 1, ph = (it >> 1) & 1;
    if (!mbar_wait(tabbar0 + 16 + 8 * half, ph ^ 1, abort_flag, 0x72)) return;
    const uint32_t dst0 = table0 + half * TILE_M * entb, bar = tabbar0 + 8 * half;
    if (t.tile2d) {
      const int tt = tile_spatial(t, tile);
      const int ty = tt / t.tiles_x, tx = tt - ty * t.tiles_x;
      mbar_expect_tx(bar, TILE_M * entb);
      for (int ry = 0; ry < 8; ++ry) {
        const long p0 = (long)(ty * 8 + ry) * t.W + tx * 16;
        bulk_g2s(dst0 + ry * 16 * entb, s.tab + p0 * s.K, 16 * entb, bar);
      }
    } else {
      // rows of the tile are consecutive pixels of the batch; a run ends at an image boundary
      long gp = (long)tile * TILE_M;
      long left = t.mtot - gp;
      if (left > TILE_M) left = TILE_M;
      mbar_expect_tx(bar, (uint32_t)left * entb);
      int r = 0;
      while (left > 0) {
        const long p = gp % t.npix;
        long len = t.npix - p;
        if (len > left) len = left;
        bulk_g2s(dst0 + r * entb, s.tab + p * s.K, (uint32_t)len * entb, bar);
        r += (int)len; gp += len; left -= len;
      }
    }
  }
}

// Producer warp (CSR = false: sample map; true: inverse map).  nslots ring slots are consumed per tile, of which the first nsl carry
// data (an odd slice count of the wgrad kernel is padded with a zero slice).  A group owns two rows
// of every stage; while it blends one of them the loads of the other are in flight.
template <bool CSR, bool PAD>
__device__ __forceinline__ void producer_loop_map(const Source& s, const Tiling& t, int nsl,
                                                  int nslots, int nst, uint32_t stage0,
                                                  uint32_t full0, uint32_t empty0, TapEnt* table,
                                                  uint32_t tabbar0, volatile int* abort_flag,
                                                  int pw, int lane, int code, int sl0 = 0) {
  const int g = lane >> 3, lg = lane & 7;
  const int cpb = s.C / 64;
  const int tap0 = sl0 / cpb, cb0 = sl0 - tap0 * cpb;  // first slice this CTA gathers
  const int r0 = pw * 4 + g, r1 = r0 + N_PRODUCER_WARPS * 4;  // the two rows of a stage this group owns
  const uint32_t so0 = r0 * 128 + ((lg ^ (r0 & 7)) << 4), so1 = r1 * 128 + ((lg ^ (r1 & 7)) << 4);
  const bf16* srcl = s.src + lg * 8;
  const uint4 zero = make_uint4(0, 0, 0, 0);
  uint32_t st = 0, ph = 0, it = 0;  // ring slot and its phase, advanced without divisions
  for (int tile = blockIdx.x; tile < t.tiles; tile += gridDim.x, ++it) {
    const TapEnt* tab = table + (size_t)(it & 1) * TILE_M * s.K;
    {  // wait until the decoder warps have filled this half of the table
      int okt = 1;
      if (lane == 0) okt = mbar_wait(tabbar0 + 8 * (it & 1), (it >> 1) & 1, abort_flag, code) ? 1 : 0;
      okt = __shfl_sync(0xffffffffu, okt, 0);
      if (!okt) return;
    }
    const TapEnt* t0 = tab + r0 * s.K;
    const TapEnt* t1 = tab + r1 * s.K;
    // source image of each of the two rows; a row beyond the end of the batch reads the K
    // all-zero-weight entries that follow the two table halves
    const bf16 *s0, *s1;
    if (t.tile2d) {
      s0 = s1 = srcl + (long)tile_img(t, tile) * s.spix * s.C;
    } else {
      const long g0 = (long)tile * TILE_M + r0, g1 = (long)tile * TILE_M + r1;
      const TapEnt* zero_ent = table + (size_t)2 * TILE_M * s.K;
      s0 = s1 = srcl;
      if (g0 < t.mtot) s0 = srcl + (g0 / t.npix) * s.spix * s.C; else t0 = zero_ent;
      if (g1 < t.mtot) s1 = srcl + (g1 / t.npix) * s.spix * s.C; else t1 = zero_ent;
    }
    const int p0 = CSR ? tile_row_pixel(t, tile, r0) : 0, p1 = CSR ? tile_row_pixel(t, tile, r1) : 0;
    RowLoad A, B;
    issue_row<CSR>(t0 + tap0, s0 + cb0 * 64, s.C, A);  // first slice
    int tap = tap0, cb = cb0;     // of the current slice
    for (int sl = 0; sl < nslots; ++sl) {
      const bool live = !PAD || sl < nsl;
      if (live) issue_row<CSR>(t1 + tap, s1 + cb * 64, s.C, B);
      int okw = 1;
      if (lane == 0) okw = mbar_wait(empty0 + 8u * st, ph ^ 1, abort_flag, code) ? 1 : 0;
      okw = __shfl_sync(0xffffffffu, okw, 0);
      if (!okw) return;
      const uint32_t sbase = stage0 + st * STAGE_BYTES;
      float2 acc[4];
      if (live) blend_row(A, acc);
      sts16(sbase + so0, live ? pack_row(acc) : zero);
      const bool more_a = CSR && A.more;
      const int tap_b = tap, cb_b = cb;
      if (++cb == cpb) { cb = 0; ++tap; }
      if (sl + 1 < nsl) issue_row<CSR>(t0 + tap, s0 + cb * 64, s.C, A);
      if (live) blend_row(B, acc);
      sts16(sbase + so1, live ? pack_row(acc) : zero);
      if (CSR) {
        if (more_a)
          add_list_tail(s.inv_off, s.inv_ent, s.C, (long)p0 * s.K + tap_b, s0 + cb_b * 64, sbase + so0, 4);
        if (B.more)
          add_list_tail(s.inv_off, s.inv_ent, s.C, (long)p1 * s.K + tap_b, s1 + cb_b * 64, sbase + so1, 4);
      }
      // every lane publishes its own writes to the async proxy; one arrival per warp
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(full0 + 8u * st);
      if (++st == (uint32_t)nst) { st = 0; ph ^= 1; }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(tabbar0 + 16 + 8 * (it & 1));  // this warp is done with the half
  }
}

// Producer warp for channel counts that are not a multiple of 64 (map mode).  The gathered axis is
// e = tap * C + c, cut into 64-element slices and zero-padded at the end; a lane owns 8 consecutive
// elements of a row.  With C % 8 == 0 those lie in one tap and are fetched as 16-byte vectors like
// in the regular producer, only with a tap of the lane's own; otherwise (e.g. the 3 input channels
// of a first layer) every element is gathered on its own.
__device__ __forceinline__ float gather_element(const TapEnt* ent, const bf16* sb, int C, int c) {
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int off = i == 3 ? (ent->off[3] & ~MORE_FLAG) : ent->off[i];
    const float v = __bfloat162float(__ldg(sb + (long)off * C + c));
    acc = fmaf(ent->w[i], v, acc);
  }
  return acc;
}

__device__ __forceinline__ uint4 gather_elements8(const TapEnt* trow, const bf16* sb, int C, int KC,
                                                  int e0) {
  float v[8];
  int k = e0 / C, c = e0 - k * C;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    v[j] = e0 + j < KC ? gather_element(trow + k, sb, C, c) : 0.f;
    if (++c == C) { c = 0; ++k; }
  }
  return pack8(v);
}

template <bool PAD>
__device__ __forceinline__ void producer_loop_packed(const Source& s, const Tiling& t, int nsl,
                                                     int nslots, int nst, uint32_t stage0,
                                                     uint32_t full0, uint32_t empty0, TapEnt* table,
                                                     uint32_t tabbar0, volatile int* abort_flag,
                                                     int pw, int lane, int code, int sl0 = 0) {
  const int g = lane >> 3, lg = lane & 7;
  const int C = s.C, KC = s.KC;
  const bool vec = (C & 7) == 0;
  const int r0 = pw * 4 + g, r1 = r0 + N_PRODUCER_WARPS * 4;
  const uint32_t so0 = r0 * 128 + ((lg ^ (r0 & 7)) << 4), so1 = r1 * 128 + ((lg ^ (r1 & 7)) << 4);
  const uint4 zero = make_uint4(0, 0, 0, 0);
  uint32_t st = 0, ph = 0, it = 0;
  for (int tile = blockIdx.x; tile < t.tiles; tile += gridDim.x, ++it) {
    const TapEnt* tab = table + (size_t)(it & 1) * TILE_M * s.K;
    {
      int okt = 1;
      if (lane == 0) okt = mbar_wait(tabbar0 + 8 * (it & 1), (it >> 1) & 1, abort_flag, code) ? 1 : 0;
      okt = __shfl_sync(0xffffffffu, okt, 0);
      if (!okt) return;
    }
    const TapEnt* t0 = tab + r0 * s.K;
    const TapEnt* t1 = tab + r1 * s.K;
    const bf16 *s0, *s1;
    if (t.tile2d) {
      s0 = s1 = s.src + (long)tile_img(t, tile) * s.spix * C;
    } else {
      const long g0 = (long)tile * TILE_M + r0, g1 = (long)tile * TILE_M + r1;
      // rows past the end of the batch: entries of tap 0..K-1 with zero weights
      const TapEnt* zero_ent = table + (size_t)2 * TILE_M * s.K;
      s0 = s1 = s.src;
      if (g0 < t.mtot) s0 = s.src + (g0 / t.npix) * s.spix * C; else t0 = zero_ent;
      if (g1 < t.mtot) s1 = s.src + (g1 / t.npix) * s.spix * C; else t1 = zero_ent;
    }
    int e0 = sl0 * 64 + lg * 8;
    for (int sl = 0; sl < nslots; ++sl, e0 += 64) {
      const bool live = (!PAD || sl < nsl) && e0 < KC;
      uint4 ra = zero, rb = zero;
      if (live) {
        if (vec) {
          const int k = e0 / C, c = e0 - k * C;
          RowLoad A, B;
          issue_row<false>(t0 + k, s0 + c, C, A);
          issue_row<false>(t1 + k, s1 + c, C, B);
          float2 acc[4];
          blend_row(A, acc);
          ra = pack_row(acc);
          blend_row(B, acc);
          rb = pack_row(acc);
        } else {
          ra = gather_elements8(t0, s0, C, KC, e0);
          rb = gather_elements8(t1, s1, C, KC, e0);
        }
      }
      int okw = 1;
      if (lane == 0) okw = mbar_wait(empty0 + 8u * st, ph ^ 1, abort_flag, code) ? 1 : 0;
      okw = __shfl_sync(0xffffffffu, okw, 0);
      if (!okw) return;
      const uint32_t sbase = stage0 + st * STAGE_BYTES;
      sts16(sbase + so0, ra);
      sts16(sbase + so1, rb);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(full0 + 8u * st);
      if (++st == (uint32_t)nst) { st = 0; ph ^= 1; }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(tabbar0 + 16 + 8 * (it & 1));
  }
}

// Producer for a gathered axis that fits ONE slice (K * C <= 64, e.g. a 3-channel first layer with
// 7 or 9 taps).  Such a layer is a stream of tiny tiles - one stage, one MMA group and one
// epilogue each - so the cost per tile is what matters: a thread builds a whole 128-byte row by
// itself (tap records read straight from the global table, which stays in L2; no shared-memory
// table, no idle lanes), four warps build a stage, and the four teams of four warps work on four
// consecutive ring slots at once.
constexpr int ROW_TEAMS = 4;

__device__ __forceinline__ void load_entry(const TapEnt* ent, int (&off)[4], float (&w)[4]) {
  const uint4 o = ldg16(ent), ww = ldg16(reinterpret_cast<const uint4*>(ent) + 1);
  off[0] = (int)o.x; off[1] = (int)o.y; off[2] = (int)o.z; off[3] = (int)o.w & ~MORE_FLAG;
  w[0] = __uint_as_float(ww.x); w[1] = __uint_as_float(ww.y);
  w[2] = __uint_as_float(ww.z); w[3] = __uint_as_float(ww.w);
}

__device__ __forceinline__ void gather_row_elements(const TapEnt* ent, const bf16* xb, int C, int K,
                                                    int KC, bool nearest, uint4 (&row)[8]) {
  int k = 0, c = 0;
  int off[4];
  float w[4];
  load_entry(ent, off, w);
#pragma unroll
  for (int ch = 0; ch < 8; ++ch) {
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = 0.f;
    if (ch * 8 < KC) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (ch * 8 + j < KC) {
          if (nearest) {
            v[j] = w[0] * __bfloat162float(__ldg(xb + (long)off[0] * C + c));
          } else {
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i)
              acc = fmaf(w[i], __bfloat162float(__ldg(xb + (long)off[i] * C + c)), acc);
            v[j] = acc;
          }
          if (++c == C) {
            c = 0;
            if (++k < K) load_entry(ent + k, off, w);
          }
        }
      }
    }
    row[ch] = pack8(v);
  }
}

// Nearest maps: one source pixel per tap.  The K (pixel, weight) pairs of the row are fetched
// first, all loads in flight together, and parked in the thread's private strip of shared memory;
// the element loop then reads them back with short shared loads, so that its global loads do not
// wait on one another.
__device__ __forceinline__ void gather_row_nearest(const TapEnt* ent, const bf16* xb, int C, int K,
                                                   int KC, uint2* mine, uint4 (&row)[8]) {
#pragma unroll 4
  for (int k = 0; k < K; ++k)
    mine[k] = make_uint2((uint32_t)__ldg(&ent[k].off[0]), __float_as_uint(__ldg(&ent[k].w[0])));
  int k = 0, c = 0;
  uint2 e = mine[0];
  // 24 elements (three 16-byte chunks) per pass, so that all loads of a typical row (21 or 27
  // elements) are in flight before the first of them is converted
#pragma unroll
  for (int pass = 0; pass < 3; ++pass) {
    constexpr int PE = 24;
    float v[PE];
#pragma unroll
    for (int j = 0; j < PE; ++j) v[j] = 0.f;
    if (pass * PE < KC) {
#pragma unroll
      for (int j = 0; j < PE; ++j) {
        if (pass * PE + j < 64 && pass * PE + j < KC) {
          v[j] = __uint_as_float(e.y) * __bfloat162float(__ldg(xb + (long)(int)e.x * C + c));
          if (++c == C) {
            c = 0;
            if (++k < K) e = mine[k];
          }
        }
      }
    }
#pragma unroll
    for (int q = 0; q < 3; ++q) {
      if (pass * 3 + q < 8) {
        uint4 o;
        o.x = pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]);
        o.y = pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]);
        o.z = pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]);
        o.w = pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]);
        row[pass * 3 + q] = o;
      }
    }
  }
}

// Nearest maps with 1, 3 or 4 channels (depth, RGB, RGB-D first layers), compact table.  A row is
// K pixels of C channels side by side.  What bounds this layer is the number of load instructions
// whose lanes all hit different cache lines (one line per lane and instruction goes through L1),
// so a pixel is fetched with as few loads as its alignment allows - two aligned 32-bit words for a
// 6-byte RGB pixel, one 64-bit word for four channels - and shifted into place in registers; the
// element loads of the generic path cost three to four times as many.
template <int C>
__device__ __forceinline__ void gather_row_nearest_c(const int* offs, const bf16* src, long pix0,
                                                     long src_elems, int K, uint4 (&row)[8]) {
  static_assert(C == 1 || C == 3 || C == 4, "unsupported channel count");
  constexpr int KMAX = 64 / C;
  constexpr int TPP = C == 1 ? 16 : 8;  // taps per pass (<= 16 registers of loads in flight)
  constexpr int NPASS = (KMAX + TPP - 1) / TPP;
  uint32_t wd[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) wd[i] = 0u;
  const uint32_t* xw = reinterpret_cast<const uint32_t*>(src);
  const uint16_t* xh = reinterpret_cast<const uint16_t*>(src);
#pragma unroll
  for (int pass = 0; pass < NPASS; ++pass) {
    if (pass * TPP < K) {
      uint32_t lo[TPP], hi[TPP], sh[TPP];
#pragma unroll
      for (int j = 0; j < TPP; ++j) {
        const int k = pass * TPP + j;
        lo[j] = hi[j] = sh[j] = 0u;
        if (k < KMAX && k < K) {
          const int off = offs[k];
          if (off >= 0) {
            const long g = (pix0 + off) * C;  // first element of the pixel
            if (C == 4) {
              const uint2 v = __ldg(reinterpret_cast<const uint2*>(xw + (g >> 1)));
              lo[j] = v.x; hi[j] = v.y;
            } else if (C == 3) {
              const long wi = g >> 1;
              sh[j] = (uint32_t)(g & 1) << 4;
              lo[j] = __ldg(xw + wi);
              // the second word may straddle the end of the tensor: then only its low half exists
              hi[j] = 2 * wi + 3 < src_elems ? __ldg(xw + wi + 1) : (uint32_t)__ldg(xh + 2 * wi + 2);
            } else {
              lo[j] = __ldg(xh + g);
            }
          }
        }
      }
#pragma unroll
      for (int j = 0; j < TPP; ++j) {
        const int k = pass * TPP + j;
        if (k < KMAX) {
          if (C == 4) {
            wd[2 * k] = lo[j]; wd[2 * k + 1] = hi[j];
          } else if (C == 3) {
            const uint32_t e01 = __funnelshift_r(lo[j], hi[j], sh[j]);
            const uint32_t e2 = (hi[j] >> sh[j]) & 0xFFFFu;
            const int P = 3 * k;  // element position in the row (compile-time after unrolling)
            if ((P & 1) == 0) {
              wd[P / 2] = e01;
              wd[P / 2 + 1] |= e2;
            } else {
              wd[(P - 1) / 2] |= e01 << 16;
              wd[(P + 1) / 2] = (e01 >> 16) | (e2 << 16);
            }
          } else {
            wd[k / 2] |= lo[j] << (16 * (k & 1));
          }
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) row[i] = make_uint4(wd[4 * i], wd[4 * i + 1], wd[4 * i + 2], wd[4 * i + 3]);
}

template <bool PAD>
__device__ __forceinline__ void producer_rowwise(const Source& s, const Tiling& t, int nsl, int nslots,
                                                 int nst, uint32_t stage0, uint32_t full0,
                                                 uint32_t empty0, TapEnt* table,
                                                 volatile int* abort_flag, int pw,
                                                 int lane, int code) {
  // the shared-memory tap table is not used in this mode; its space holds the threads' strips
  uint2* mine = reinterpret_cast<uint2*>(table) + (size_t)(pw * 32 + lane) * s.K;
  // compact-table mode: the warp's 32 x K offsets, [row][tap]
  int* wstrip = reinterpret_cast<int*>(table) + (size_t)pw * 32 * s.K;
  const bool compact = s.interp == 0 && s.tab32 != nullptr && (s.C == 1 || s.C == 3 || s.C == 4);
  constexpr int TW = N_PRODUCER_WARPS / ROW_TEAMS;  // warps per team: 4 x 32 threads = 128 rows
  const int team = pw / TW, r = (pw % TW) * 32 + lane;
  const uint32_t rowaddr = r * 128;
  const int rx = r & 7;
  // this team's ring slots: team, team + ROW_TEAMS, ... of the CTA's slot sequence
  int tile = blockIdx.x, sl = team;
  uint32_t st = team, ph = 0;
  while (sl >= nslots) { sl -= nslots; tile += gridDim.x; }
  while (tile < t.tiles) {
    uint4 row[8];
#pragma unroll
    for (int ch = 0; ch < 8; ++ch) row[ch] = make_uint4(0, 0, 0, 0);
    if (!PAD || sl < nsl) {
      long gp, p;
      int img;
      bool valid;
      tile_pixel(t, tile, r, gp, img, p, valid);
      if (compact) {
        // The 32 rows of a warp are consecutive pixels of one image unless the tile is a 2-D block
        // or crosses an image / the end: then their K x 32 table words are one contiguous run and
        // are fetched with coalesced loads; otherwise every lane fetches its own K words.
        const long p0 = __shfl_sync(0xffffffffu, p, 0);
        const bool run = __all_sync(0xffffffffu, valid && p == p0 + lane);
        __syncwarp();
        if (run) {
          const int* tw = s.tab32 + p0 * s.K;
          for (int i = lane; i < 32 * s.K; i += 32) wstrip[i] = __ldg(tw + i);
        } else {
          for (int k = 0; k < s.K; ++k) wstrip[lane * s.K + k] = valid ? __ldg(s.tab32 + p * s.K + k) : -1;
        }
        __syncwarp();
        const int* offs = wstrip + lane * s.K;
        const long pix0 = (long)img * s.spix;
        if (s.C == 3) gather_row_nearest_c<3>(offs, s.src, pix0, s.src_elems, s.K, row);
        else if (s.C == 4) gather_row_nearest_c<4>(offs, s.src, pix0, s.src_elems, s.K, row);
        else gather_row_nearest_c<1>(offs, s.src, pix0, s.src_elems, s.K, row);
      } else if (valid) {
        const TapEnt* ent = s.tab + p * s.K;
        const bf16* xb = s.src + (long)img * s.spix * s.C;
        if (s.interp == 0) gather_row_nearest(ent, xb, s.C, s.K, s.KC, mine, row);
        else gather_row_elements(ent, xb, s.C, s.K, s.KC, false, row);
      }
    }
    int okw = 1;
    if (lane == 0) okw = mbar_wait(empty0 + 8u * st, ph ^ 1, abort_flag, code) ? 1 : 0;
    okw = __shfl_sync(0xffffffffu, okw, 0);
    if (!okw) return;
    const uint32_t sbase = stage0 + st * STAGE_BYTES + rowaddr;
#pragma unroll
    for (int ch = 0; ch < 8; ++ch) sts16(sbase + ((ch ^ rx) << 4), row[ch]);
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) mbar_arrive(full0 + 8u * st);
    sl += ROW_TEAMS;
    while (sl >= nslots) { sl -= nslots; tile += gridDim.x; }
    st += ROW_TEAMS;
    if (st >= (uint32_t)nst) { st -= nst; ph ^= 1; }
  }
}

// Producer warp for nearest-neighbour maps: every (pixel, tap) reads ONE source pixel with weight 1
// (or nothing), so a row is a 128-byte copy.  There is no arithmetic to hide the load latency
// behind; instead the loads of the next COPY_AHEAD slices are kept in flight.  Inverse-map mode:
// the first list entry is copied, the (rare) further ones are added by add_list_tail.
constexpr int COPY_AHEAD = 4;
constexpr int COPY_AHEAD_CSR = 2;  // inverse-map mode keeps more state per row

struct CopyLoad {
  uint4 v;
  bool on, more;
};

template <bool CSR>
__device__ __forceinline__ void issue_copy(const TapEnt* ent, const bf16* sb, int C, CopyLoad& L) {
  const uint2 ow = *reinterpret_cast<const uint2*>(&ent->w[0]);  // weights of entries 0 and 1
  const int off = ent->off[0];
  L.on = ow.x != 0u;
  L.more = CSR && ow.y != 0u;
  L.v = ldg16(sb + (long)off * C);
  if (CSR && L.more)  // a second list entry (1.4 % of the lists of a one-ring map): warm L1 for it
    asm volatile("prefetch.global.L1 [%0];" ::"l"(sb + (long)ent->off[1] * C));
}

// Entries 1 and up of an inverse-map list whose first entry `row` is already loaded: entries 1-3
// from the table entry, the rest (MORE_FLAG) from the global list.  Accumulates in fp32.
__device__ __forceinline__ uint4 finish_list(const TapEnt* ent, const bf16* sb, int C, const uint4& row,
                                             const int* __restrict__ inv_off,
                                             const int2* __restrict__ inv_ent, long key) {
  float2 acc[4];
  acc[0] = make_float2(__uint_as_float(row.x << 16), __uint_as_float(row.x & 0xFFFF0000u));
  acc[1] = make_float2(__uint_as_float(row.y << 16), __uint_as_float(row.y & 0xFFFF0000u));
  acc[2] = make_float2(__uint_as_float(row.z << 16), __uint_as_float(row.z & 0xFFFF0000u));
  acc[3] = make_float2(__uint_as_float(row.w << 16), __uint_as_float(row.w & 0xFFFF0000u));
  const int o3 = ent->off[3];
#pragma unroll 1
  for (int i = 1; i < 4; ++i) {
    const float w = ent->w[i];
    if (w == 0.f) break;
    const int off = i == 3 ? (o3 & ~MORE_FLAG) : ent->off[i];
    const uint4 v = ldg16(sb + (long)off * C);
    const float2 w2 = make_float2(w, w);
    ffma2_bf16x2(acc[0], w2, v.x);
    ffma2_bf16x2(acc[1], w2, v.y);
    ffma2_bf16x2(acc[2], w2, v.z);
    ffma2_bf16x2(acc[3], w2, v.w);
  }
  if (o3 & MORE_FLAG) {
    const int end = __ldg(inv_off + key + 1);
#pragma unroll 1
    for (int e = __ldg(inv_off + key) + 4; e < end; ++e) {
      const int2 en = __ldg(inv_ent + e);
      const uint4 v = ldg16(sb + (long)en.x * C);
      const float w = __int_as_float(en.y);
      const float2 w2 = make_float2(w, w);
      ffma2_bf16x2(acc[0], w2, v.x);
      ffma2_bf16x2(acc[1], w2, v.y);
      ffma2_bf16x2(acc[2], w2, v.z);
      ffma2_bf16x2(acc[3], w2, v.w);
    }
  }
  return pack_row(acc);
}

template <bool CSR, bool PAD>
__device__ __forceinline__ void producer_loop_copy(const Source& s, const Tiling& t, int nsl,
                                                   int nslots, int nst, uint32_t stage0,
                                                   uint32_t full0, uint32_t empty0, TapEnt* table,
                                                   uint32_t tabbar0, volatile int* abort_flag,
                                                   int pw, int lane, int code, int sl0 = 0) {
  constexpr int AHEAD = CSR ? COPY_AHEAD_CSR : COPY_AHEAD;
  const int g = lane >> 3, lg = lane & 7;
  const int cpb = s.C / 64;
  const int tap0 = sl0 / cpb, cb0 = sl0 - tap0 * cpb;
  const int r0 = pw * 4 + g, r1 = r0 + N_PRODUCER_WARPS * 4;
  const uint32_t so0 = r0 * 128 + ((lg ^ (r0 & 7)) << 4), so1 = r1 * 128 + ((lg ^ (r1 & 7)) << 4);
  const bf16* srcl = s.src + lg * 8;
  const uint4 zero = make_uint4(0, 0, 0, 0);
  uint32_t st = 0, ph = 0, it = 0;
  for (int tile = blockIdx.x; tile < t.tiles; tile += gridDim.x, ++it) {
    const TapEnt* tab = table + (size_t)(it & 1) * TILE_M * s.K;
    {
      int okt = 1;
      if (lane == 0) okt = mbar_wait(tabbar0 + 8 * (it & 1), (it >> 1) & 1, abort_flag, code) ? 1 : 0;
      okt = __shfl_sync(0xffffffffu, okt, 0);
      if (!okt) return;
    }
    const TapEnt* t0 = tab + r0 * s.K;
    const TapEnt* t1 = tab + r1 * s.K;
    const bf16 *s0, *s1;
    if (t.tile2d) {
      s0 = s1 = srcl + (long)tile_img(t, tile) * s.spix * s.C;
    } else {
      const long g0 = (long)tile * TILE_M + r0, g1 = (long)tile * TILE_M + r1;
      const TapEnt* zero_ent = table + (size_t)2 * TILE_M * s.K;
      s0 = s1 = srcl;
      if (g0 < t.mtot) s0 = srcl + (g0 / t.npix) * s.spix * s.C; else t0 = zero_ent;
      if (g1 < t.mtot) s1 = srcl + (g1 / t.npix) * s.spix * s.C; else t1 = zero_ent;
    }
    const int p0 = CSR ? tile_row_pixel(t, tile, r0) : 0, p1 = CSR ? tile_row_pixel(t, tile, r1) : 0;
    CopyLoad A[AHEAD], B[AHEAD];
    int tap_i = tap0, cb_i = cb0;  // slice whose loads are issued next
    int tap_c = tap0, cb_c = cb0;  // slice that is stored next
#pragma unroll
    for (int u = 0; u < AHEAD; ++u) {
      if (u < nsl) {
        issue_copy<CSR>(t0 + tap_i, s0 + cb_i * 64, s.C, A[u]);
        issue_copy<CSR>(t1 + tap_i, s1 + cb_i * 64, s.C, B[u]);
        if (++cb_i == cpb) { cb_i = 0; ++tap_i; }
      }
    }
    for (int slb = 0; slb < nslots; slb += AHEAD) {
#pragma unroll
      for (int u = 0; u < AHEAD; ++u) {
        const int sl = slb + u;
        if (sl < nslots) {
          const bool live = !PAD || sl < nsl;
          int okw = 1;
          if (lane == 0) okw = mbar_wait(empty0 + 8u * st, ph ^ 1, abort_flag, code) ? 1 : 0;
          okw = __shfl_sync(0xffffffffu, okw, 0);
          if (!okw) return;
          const uint32_t sbase = stage0 + st * STAGE_BYTES;
          uint4 ra = live && A[u].on ? A[u].v : zero, rb = live && B[u].on ? B[u].v : zero;
          if (CSR && live) {
            if (A[u].more)
              ra = finish_list(t0 + tap_c, s0 + cb_c * 64, s.C, ra, s.inv_off, s.inv_ent, (long)p0 * s.K + tap_c);
            if (B[u].more)
              rb = finish_list(t1 + tap_c, s1 + cb_c * 64, s.C, rb, s.inv_off, s.inv_ent, (long)p1 * s.K + tap_c);
          }
          sts16(sbase + so0, ra);
          sts16(sbase + so1, rb);
          if (++cb_c == cpb) { cb_c = 0; ++tap_c; }
          if (sl + AHEAD < nsl) {
            issue_copy<CSR>(t0 + tap_i, s0 + cb_i * 64, s.C, A[u]);
            issue_copy<CSR>(t1 + tap_i, s1 + cb_i * 64, s.C, B[u]);
            if (++cb_i == cpb) { cb_i = 0; ++tap_i; }
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(full0 + 8u * st);
          if (++st == (uint32_t)nst) { st = 0; ph ^= 1; }
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(tabbar0 + 16 + 8 * (it & 1));  // this warp is done with the half
  }
}

// Shared-memory carve-up common to both kernels.
struct Smem {
  uint32_t stage0, extra0, bar0;
  uint8_t* extra;  // generic pointer to the region behind the stages
  float* fl;
  uint32_t* misc;
  volatile int* abort_flag;
};

__device__ __forceinline__ Smem carve(uint8_t* raw, int nst, size_t extra_bytes, int nfloat, int nbar) {
  uint8_t* sm = (uint8_t*)(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
  Smem s;
  uint8_t* extra = sm + (size_t)nst * STAGE_BYTES;
  s.fl = (float*)(extra + extra_bytes);
  uint64_t* bars = (uint64_t*)(s.fl + nfloat);
  s.misc = (uint32_t*)(bars + nbar);
  s.abort_flag = (volatile int*)(s.misc + 1);
  s.stage0 = smem_u32(sm);
  s.extra0 = smem_u32(extra);
  s.extra = extra;
  s.bar0 = smem_u32(bars);
  return s;
}

// Bytes of the double-buffered tap table of the map-mode producers.
// (two halves of TILE_M * K entries, then K entries with zero weights for rows past the end)
__host__ __device__ inline size_t tap_table_bytes(int K) {
  return ((size_t)2 * TILE_M * K + K) * sizeof(TapEnt);
}

static size_t smem_bytes(int nst, size_t extra_bytes, int nfloat, int nbar) {
  return 1024 + (size_t)nst * STAGE_BYTES + extra_bytes + (size_t)nfloat * 4 + (size_t)nbar * 8 + 16;
}

// ------------------------------------------------------------------------------------------------
// forward / dgrad:  D[128 pixels, NOUT] = gathered[128, nsl * 64] . Wimg^T
// ------------------------------------------------------------------------------------------------
// PRE: the tap table of the tiled domain was built beforehand in global memory (a.s.tab) and is
// streamed in by bulk copies; otherwise three warps decode the map / the inverse map in the kernel.
// WRES: all weight slices of the CTA's NOUT output channels stay in shared memory; otherwise the
// slice of every pipeline step is streamed in beside its stage by a bulk copy (needs PRE, whose
// idle decoder warps provide the thread that issues the copies).
// blockIdx.y selects the chunk of NOUT output channels.
template <int NOUT, bool CSR, bool PRE, bool WRES>
__global__ void __launch_bounds__(TC_THREADS, 1) conv_gemm_tc_kernel(const GemmArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const int nst = a.nst;
  const int co0 = blockIdx.y * NOUT;
  constexpr uint32_t WSLICE = NOUT * 128;  // bytes of one weight slice
  const size_t wbytes = (size_t)(WRES ? a.nsl : nst) * WSLICE;
  // bars: full[nst], empty[nst], tfull[2], tempty[2], drain, tab_full[2], tab_empty[2]
  const Smem sm = carve(smem_raw, nst, wbytes + tap_table_bytes(a.s.K) + EPI_STAGING_BYTES, NOUT,
                        2 * nst + 9);
  float* bias_s = sm.fl;
  volatile int* abort_flag = sm.abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t stage0 = sm.stage0, w0 = sm.extra0, bar0 = sm.bar0;
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (nst + s); };
  auto tfull_bar = [&](int i) { return bar0 + 8u * (2 * nst + i); };
  auto tempty_bar = [&](int i) { return bar0 + 8u * (2 * nst + 2 + i); };
  const uint32_t drain_bar = bar0 + 8u * (2 * nst + 4);
  const uint32_t tabbar0 = bar0 + 8u * (2 * nst + 5);
  constexpr uint32_t TMEM_COLS = 2 * NOUT < 32 ? 32 : 2 * NOUT;

  if (threadIdx.x == 0) {
    for (int s = 0; s < nst; ++s) {
      mbar_init(full_bar(s), a.full_cnt + (WRES ? 0 : 1));
      mbar_init(empty_bar(s), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(tfull_bar(i), 1);
      mbar_init(tempty_bar(i), N_EPI_WARPS);
    }
    mbar_init(drain_bar, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(tabbar0 + 8 * i, PRE ? 1 : N_DEC_WARPS);
      mbar_init(tabbar0 + 16 + 8 * i, N_PRODUCER_WARPS);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  // resident operands: weight slices and bias
  if (WRES) {
    for (int i = threadIdx.x; i < a.nsl * NOUT * 8; i += TC_THREADS) {
      const int sl = i / (NOUT * 8), j = i - sl * (NOUT * 8);
      sts16(w0 + 16u * i, ldg16(a.wimg + ((size_t)sl * a.ncol + co0) * 8 + j));
    }
  }
  for (int i = threadIdx.x; i < NOUT; i += TC_THREADS)
    bias_s[i] = a.bias ? __bfloat162float(a.bias[co0 + i]) : 0.f;
  fence_proxy_async_smem();
  {  // the K zero-weight entries behind the two table halves
    uint4* z = reinterpret_cast<uint4*>((TapEnt*)(sm.extra + wbytes) + (size_t)2 * TILE_M * a.s.K);
    for (int i = threadIdx.x; i < 2 * a.s.K; i += TC_THREADS) z[i] = make_uint4(0, 0, 0, 0);
  }
  if (warp == 0) tmem_alloc(smem_u32(sm.misc), TMEM_COLS);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *sm.misc;

  if (warp == 0) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(TILE_M, NOUT, 0, 0);
      uint32_t st = 0, ph = 0, it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < a.t.tiles && ok; tile += gridDim.x, ++it) {
        const uint32_t acc = it & 1, aph = (it >> 1) & 1;
        ok = mbar_wait(tempty_bar(acc), aph ^ 1, abort_flag, 0x11);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + acc * NOUT;
        for (int s = 0; s < a.nsl; ++s) {
          ok = mbar_wait(full_bar(st), ph, abort_flag, 0x12);
          if (!ok) break;
          tc_fence_after_sync();
          const uint64_t adesc = make_desc_sw128(stage0 + st * STAGE_BYTES, 16, 1024);
          const uint64_t bdesc = make_desc_sw128(w0 + (uint32_t)(WRES ? s : st) * WSLICE, 16, 1024);
#pragma unroll
          for (int j = 0; j < 4; ++j)  // four K = 16 steps inside the 64-wide slice: +32 bytes each
            mma_bf16_ss(tmem_d, adesc + 2 * j, bdesc + 2 * j, idesc, (s | j) != 0);
          mma_commit(empty_bar(st));  // frees the stage when these MMAs have read it
          if (++st == (uint32_t)nst) { st = 0; ph ^= 1; }
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
    // A lane reads its own row (TMEM lane) 32 columns at a time, adds the bias and packs to bf16.
    // Storing that directly would scatter 16-byte pieces over 32 rows per instruction; instead the
    // warp passes the 32 x 64-byte block through shared memory and stores 8 rows x 64 bytes per
    // instruction (lane -> row 8 i + lane / 4, 16-byte piece lane % 4).
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const uint32_t stg = w0 + (uint32_t)(wbytes + tap_table_bytes(a.s.K)) + (uint32_t)(warp - 1) * 2048u;
    const uint32_t wr_row = stg + lane * 64, wr_x = (lane >> 1) & 3;
    uint32_t rd_addr[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int row = 8 * i + (lane >> 2);
      rd_addr[i] = stg + row * 64 + (((lane & 3) ^ ((row >> 1) & 3)) << 4);
    }
    uint32_t it = 0;
    for (int tile = blockIdx.x; tile < a.t.tiles; tile += gridDim.x, ++it) {
      const uint32_t acc = it & 1, aph = (it >> 1) & 1;
      // where the four rows this lane stores live in global memory
      bf16* orow[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        long gp, p;
        int img;
        bool valid;
        tile_pixel(a.t, tile, q * 32 + 8 * i + (lane >> 2), gp, img, p, valid);
        orow[i] = valid ? a.y + gp * a.ncol + co0 + (lane & 3) * 8 : nullptr;
      }
      {
        int okt = 1;
        if (lane == 0) okt = mbar_wait(tfull_bar(acc), aph, abort_flag, 0x21) ? 1 : 0;
        okt = __shfl_sync(0xffffffffu, okt, 0);
        if (!okt) break;
      }
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + acc * NOUT;
#pragma unroll
      for (int cc = 0; cc < NOUT / 32; ++cc) {
        uint32_t v[32];
        tmem_ld_32x32(taddr + cc * 32, v);
        tmem_ld_wait();
        if (cc == NOUT / 32 - 1) {
          // accumulator fully read: hand the buffer back before the global stores
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(tempty_bar(acc));
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 o;
          const float* bs = bias_s + cc * 32 + j * 8;
          float f[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            f[e] = __uint_as_float(v[j * 8 + e]) + bs[e];
            if (a.relu) f[e] = fmaxf(f[e], 0.f);
          }
          o.x = pack_bf16x2(f[0], f[1]);
          o.y = pack_bf16x2(f[2], f[3]);
          o.z = pack_bf16x2(f[4], f[5]);
          o.w = pack_bf16x2(f[6], f[7]);
          sts16(wr_row + ((j ^ wr_x) << 4), o);
        }
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint4 o;
          asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(o.x), "=r"(o.y), "=r"(o.z), "=r"(o.w)
                       : "r"(rd_addr[i]));
          if (orow[i]) *reinterpret_cast<uint4*>(orow[i] + cc * 32) = o;
        }
        __syncwarp();  // the block is read out before the next one is written
      }
    }
  } else {
    // ------------------------------------------------------------------ producers
    if (warp < FIRST_PROD_WARP) {
      if (PRE) {
        if (warp == FIRST_DEC_WARP && lane == 0 && a.s.packed != 2)
          loader_loop(a.s, a.t, w0 + (uint32_t)wbytes, tabbar0, abort_flag);
        if (!WRES && warp == FIRST_DEC_WARP + 1 && lane == 0) {
          // weight streamer: slice s of every tile goes into the ring slot of pipeline step s
          uint32_t st = 0, ph = 0;
          bool ok = true;
          for (int tile = blockIdx.x; tile < a.t.tiles && ok; tile += gridDim.x) {
            for (int s = 0; s < a.nsl; ++s) {
              ok = mbar_wait(empty_bar(st), ph ^ 1, abort_flag, 0x73);
              if (!ok) break;
              mbar_expect_tx(full_bar(st), WSLICE);
              bulk_g2s(w0 + st * WSLICE, a.wimg + ((size_t)s * a.ncol + co0) * 8, WSLICE, full_bar(st));
              if (++st == (uint32_t)nst) { st = 0; ph ^= 1; }
            }
          }
        }
      } else {
        decoder_loop<CSR>(a.s, a.t, (TapEnt*)(sm.extra + wbytes), tabbar0, abort_flag,
                          (warp - FIRST_DEC_WARP) * 32 + lane, lane);
      }
    } else if (!CSR && PRE && a.s.packed == 2) {
      producer_rowwise<false>(a.s, a.t, a.nsl, a.nsl, nst, stage0, full_bar(0), empty_bar(0),
                              (TapEnt*)(sm.extra + wbytes), abort_flag, warp - FIRST_PROD_WARP, lane,
                              0x36);
    } else if (!CSR && a.s.packed) {
      producer_loop_packed<false>(a.s, a.t, a.nsl, a.nsl, nst, stage0, full_bar(0), empty_bar(0),
                                  (TapEnt*)(sm.extra + wbytes), tabbar0, abort_flag,
                                  warp - FIRST_PROD_WARP, lane, 0x35);
    } else if (a.s.interp == 0) {
      producer_loop_copy<CSR, false>(a.s, a.t, a.nsl, a.nsl, nst, stage0, full_bar(0), empty_bar(0),
                                     (TapEnt*)(sm.extra + wbytes), tabbar0, abort_flag,
                                     warp - FIRST_PROD_WARP, lane, CSR ? 0x33 : 0x34);
    } else {
      producer_loop_map<CSR, false>(a.s, a.t, a.nsl, a.nsl, nst, stage0, full_bar(0), empty_bar(0),
                             (TapEnt*)(sm.extra + wbytes), tabbar0, abort_flag,
                             warp - FIRST_PROD_WARP, lane, CSR ? 0x31 : 0x32);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------------------
// wgrad:  D_j[(slice 2j | slice 2j+1) x 64 channels, NOUT] += A_tile^T . gy_tile  over all tiles
// ------------------------------------------------------------------------------------------------
// The stage written by the producers, [pixel][64 channels] with the 128-byte swizzle, is read here
// as an MN-major A operand (M = channels, reduction = pixels); two consecutive stages (leading
// byte offset = STAGE_BYTES) make one M = 128 tile.  gy tiles [pixel][NOUT] are the MN-major B
// operand.  Every CTA keeps its partial sums in tensor memory for the whole kernel and adds them
// to gw with atomics at the end.
constexpr int GY_STAGES = 2;

template <int NOUT, bool PRE>
__global__ void __launch_bounds__(TC_THREADS, 1) conv_wgrad_tc_kernel(const GemmArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const int nst = a.nst;  // even
  constexpr uint32_t GYB = (NOUT / 64) * STAGE_BYTES;  // one gy tile: 128 pixels x NOUT channels
  // bars: full[nst], empty[nst], gfull[GY], gempty[GY], done
  const Smem sm = carve(smem_raw, nst, (size_t)GY_STAGES * GYB + tap_table_bytes(a.s.K), NOUT,
                        2 * nst + 2 * GY_STAGES + 5);
  float* gb_s = sm.fl;
  volatile int* abort_flag = sm.abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t stage0 = sm.stage0, gy0 = sm.extra0, bar0 = sm.bar0;
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (nst + s); };
  auto gfull_bar = [&](int i) { return bar0 + 8u * (2 * nst + i); };
  auto gempty_bar = [&](int i) { return bar0 + 8u * (2 * nst + GY_STAGES + i); };
  const uint32_t done_bar = bar0 + 8u * (2 * nst + 2 * GY_STAGES);
  const uint32_t tabbar0 = done_bar + 8u;
  // This CTA's share of the gradient: output channels [co0, co0 + NOUT) and the M = 128 tiles
  // [j0, j0 + nmt) of the (tap, input channel) axis, i.e. slices [sl0, sl0 + nsl).
  const int co0 = blockIdx.z * NOUT;
  const int j0 = blockIdx.y * a.mtpg;
  const int nmt_all = (a.nsl + 1) / 2;
  const int nmt = nmt_all - j0 < a.mtpg ? nmt_all - j0 : a.mtpg;
  const int sl0 = 2 * j0;
  const int nsl = a.nsl - sl0 < 2 * nmt ? a.nsl - sl0 : 2 * nmt;
  const int nsl_pad = nmt * 2;            // ring slots used per pixel tile
  const int ccols = a.mtpg * NOUT;
  const uint32_t tmem_cols = ccols <= 32 ? 32 : ccols <= 64 ? 64 : ccols <= 128 ? 128
                             : ccols <= 256 ? 256 : 512;

  if (threadIdx.x == 0) {
    for (int s = 0; s < nst; ++s) {
      mbar_init(full_bar(s), a.full_cnt);
      mbar_init(empty_bar(s), 1);
    }
    for (int i = 0; i < GY_STAGES; ++i) {
      mbar_init(gfull_bar(i), N_EPI_WARPS);
      mbar_init(gempty_bar(i), 1);
    }
    mbar_init(done_bar, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(tabbar0 + 8 * i, PRE ? 1 : N_DEC_WARPS);
      mbar_init(tabbar0 + 16 + 8 * i, N_PRODUCER_WARPS);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  for (int i = threadIdx.x; i < NOUT; i += TC_THREADS) gb_s[i] = 0.f;
  {  // the K zero-weight entries behind the two table halves
    uint4* z = reinterpret_cast<uint4*>((TapEnt*)(sm.extra + (size_t)GY_STAGES * GYB) +
                                        (size_t)2 * TILE_M * a.s.K);
    for (int i = threadIdx.x; i < 2 * a.s.K; i += TC_THREADS) z[i] = make_uint4(0, 0, 0, 0);
  }
  if (warp == 0) tmem_alloc(smem_u32(sm.misc), tmem_cols);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *sm.misc;

  if (warp == 0) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(TILE_M, NOUT, 1, 1);
      uint32_t it = 0, st = 0, ph = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < a.t.tiles && ok; tile += gridDim.x, ++it) {
        const uint32_t gs = it % GY_STAGES, gph = (it / GY_STAGES) & 1;
        ok = mbar_wait(gfull_bar(gs), gph, abort_flag, 0x41);
        if (!ok) break;
        const uint64_t bdesc = make_desc_sw128(gy0 + gs * GYB, STAGE_BYTES, 1024);
        for (int j = 0; j < nmt && ok; ++j) {
          // slots st and st + 1 (st is even) share the phase
          ok = mbar_wait(full_bar(st), ph, abort_flag, 0x42);
          if (ok) ok = mbar_wait(full_bar(st + 1), ph, abort_flag, 0x43);
          if (!ok) break;
          tc_fence_after_sync();
          const uint64_t adesc = make_desc_sw128(stage0 + st * STAGE_BYTES, STAGE_BYTES, 1024);
#pragma unroll
          for (int kk = 0; kk < TILE_M / 16; ++kk)  // 16 pixels per MMA: +2048 bytes each
            mma_bf16_ss(tmem_base + j * NOUT, adesc + 128 * kk, bdesc + 128 * kk, idesc,
                        (it | kk) != 0);
          mma_commit(empty_bar(st));
          mma_commit(empty_bar(st + 1));
          st += 2;
          if (st == (uint32_t)nst) { st = 0; ph ^= 1; }
        }
        if (ok) mma_commit(gempty_bar(gs));
      }
      mma_commit(done_bar);
    }
    __syncwarp();
  } else if (warp <= N_EPI_WARPS) {
    // ------------------------------------------------------------------ gy loader, then epilogue
    const int lw = warp - 1;
    const int g = lane >> 3, lg = lane & 7;
    float bsum[NOUT / 8];  // bias gradient: this lane's 8 channels of every 64-channel block
#pragma unroll
    for (int j = 0; j < NOUT / 8; ++j) bsum[j] = 0.f;
    uint32_t it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < a.t.tiles && ok; tile += gridDim.x, ++it) {
      const uint32_t gs = it % GY_STAGES, gph = (it / GY_STAGES) & 1;
      int okw = 1;
      if (lane == 0) okw = mbar_wait(gempty_bar(gs), gph ^ 1, abort_flag, 0x51) ? 1 : 0;
      okw = __shfl_sync(0xffffffffu, okw, 0);
      if (!okw) { ok = false; break; }
      const uint32_t sbase = gy0 + gs * GYB;
      if (nsl_pad <= 2 || (a.s.interp == 0 && a.s.C <= 64)) {
        // Few, cheap slices per tile (one-slice layers, 64-channel copies): the gy tile's load
        // latency is on the critical path, so all eight rows of a group are requested before the
        // first is stored.
#pragma unroll
        for (int nb = 0; nb < NOUT / 64; ++nb) {
          uint4 v[TILE_M / (N_EPI_WARPS * 4)];
#pragma unroll
          for (int i = 0; i < TILE_M / (N_EPI_WARPS * 4); ++i) {
            const int r = lw * 4 + g + i * (N_EPI_WARPS * 4);
            long gp, p;
            int img;
            bool valid;
            tile_pixel(a.t, tile, r, gp, img, p, valid);
            v[i] = valid ? ldcg16(a.gy + gp * a.ncol + co0 + nb * 64 + lg * 8)
                         : make_uint4(0, 0, 0, 0);
          }
#pragma unroll
          for (int i = 0; i < TILE_M / (N_EPI_WARPS * 4); ++i) {
            const int r = lw * 4 + g + i * (N_EPI_WARPS * 4);
            sts16(sbase + nb * STAGE_BYTES + r * 128 + ((lg ^ (r & 7)) << 4), v[i]);
            float* b8 = bsum + nb * 8;
            bf16x2_fma(v[i].x, 1.f, b8[0], b8[1]);
            bf16x2_fma(v[i].y, 1.f, b8[2], b8[3]);
            bf16x2_fma(v[i].z, 1.f, b8[4], b8[5]);
            bf16x2_fma(v[i].w, 1.f, b8[6], b8[7]);
          }
        }
      } else {
        // Otherwise the gy tile is far off the critical path; one row at a time keeps the loader
        // out of the producers' way (measured: bursts cost 5-10 % on the wide layers).
        for (int r = lw * 4 + g; r < TILE_M; r += N_EPI_WARPS * 4) {
          long gp, p;
          int img;
          bool valid;
          tile_pixel(a.t, tile, r, gp, img, p, valid);
#pragma unroll
          for (int nb = 0; nb < NOUT / 64; ++nb) {
            const uint4 v = valid ? ldcg16(a.gy + gp * a.ncol + co0 + nb * 64 + lg * 8)
                                  : make_uint4(0, 0, 0, 0);
            // N > 64: consecutive 64-channel blocks are separate swizzle atoms, STAGE_BYTES apart
            sts16(sbase + nb * STAGE_BYTES + r * 128 + ((lg ^ (r & 7)) << 4), v);
            float* b8 = bsum + nb * 8;
            bf16x2_fma(v.x, 1.f, b8[0], b8[1]);
            bf16x2_fma(v.y, 1.f, b8[2], b8[3]);
            bf16x2_fma(v.z, 1.f, b8[4], b8[5]);
            bf16x2_fma(v.w, 1.f, b8[6], b8[7]);
          }
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(gfull_bar(gs));
    }
    // bias gradient: lanes -> shared -> global
    const bool do_gb = a.gb != nullptr && blockIdx.y == 0;
    if (do_gb) {
#pragma unroll
      for (int nb = 0; nb < NOUT / 64; ++nb)
#pragma unroll
        for (int j = 0; j < 8; ++j) atomicAdd(gb_s + nb * 64 + lg * 8 + j, bsum[nb * 8 + j]);
    }
    asm volatile("bar.sync 1, %0;" ::"n"(N_EPI_WARPS * 32) : "memory");
    if (do_gb)
      for (int i = lw * 32 + lane; i < NOUT; i += N_EPI_WARPS * 32) atomicAdd(a.gb + co0 + i, gb_s[i]);
    // epilogue: partial weight gradient of this CTA
    if (ok && mbar_wait(done_bar, 0, abort_flag, 0x52, 1024)) {
      tc_fence_after_sync();
      const int q = warp & 3;
      const int m = q * 32 + lane;  // row of the M = 128 tile
      for (int j = 0; j < nmt; ++j) {
        const int e = (sl0 + 2 * j) * 64 + m;  // element tap * C + ci of the gathered axis
        const bool live = e < a.s.KC;
        const int tap = live ? e / a.s.C : 0, ci = live ? e - tap * a.s.C : 0;
#pragma unroll
        for (int cc = 0; cc < NOUT / 32; ++cc) {
          uint32_t v[32];
          tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + j * NOUT + cc * 32, v);
          tmem_ld_wait();
          if (live) {
#pragma unroll
            for (int c = 0; c < 32; ++c) {
              const int co = co0 + cc * 32 + c;
              atomicAdd(a.gw + ((long)co * a.s.C + ci) * a.s.K + tap, __uint_as_float(v[c]));
            }
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ producers
    if (warp < FIRST_PROD_WARP) {
      if (PRE) {
        if (warp == FIRST_DEC_WARP && lane == 0 && a.s.packed != 2)
          loader_loop(a.s, a.t, gy0 + (uint32_t)GY_STAGES * GYB, tabbar0, abort_flag);
      } else {
        decoder_loop<false>(a.s, a.t, (TapEnt*)(sm.extra + (size_t)GY_STAGES * GYB), tabbar0,
                            abort_flag, (warp - FIRST_DEC_WARP) * 32 + lane, lane);
      }
    } else if (PRE && a.s.packed == 2) {
      producer_rowwise<true>(a.s, a.t, nsl, nsl_pad, nst, stage0, full_bar(0), empty_bar(0),
                             (TapEnt*)(sm.extra + (size_t)GY_STAGES * GYB), abort_flag,
                             warp - FIRST_PROD_WARP, lane, 0x64);
    } else if (a.s.packed) {
      producer_loop_packed<true>(a.s, a.t, nsl, nsl_pad, nst, stage0, full_bar(0), empty_bar(0),
                                 (TapEnt*)(sm.extra + (size_t)GY_STAGES * GYB), tabbar0,
                                 abort_flag, warp - FIRST_PROD_WARP, lane, 0x63, sl0);
    } else if (a.s.interp == 0) {
      producer_loop_copy<false, true>(a.s, a.t, nsl, nsl_pad, nst, stage0, full_bar(0), empty_bar(0),
                                      (TapEnt*)(sm.extra + (size_t)GY_STAGES * GYB), tabbar0,
                                      abort_flag, warp - FIRST_PROD_WARP, lane, 0x62, sl0);
    } else {
      producer_loop_map<false, true>(a.s, a.t, nsl, nsl_pad, nst, stage0, full_bar(0), empty_bar(0),
                               (TapEnt*)(sm.extra + (size_t)GY_STAGES * GYB), tabbar0,
                               abort_flag, warp - FIRST_PROD_WARP, lane, 0x61, sl0);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    // all MMAs have completed once done_bar fired; if the epilogue gave up, wait for it here
    if (lane == 0) mbar_wait(done_bar, 0, abort_flag, 0x44);
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, tmem_cols);
  }
}

// ------------------------------------------------------------------------------------------------
// operand preparation
// ------------------------------------------------------------------------------------------------

// Weight (Cout, Cin, K) -> slices of [rows][64 channels] bf16, each row 128 bytes with its 16-byte
// chunks XOR-swizzled by (row & 7): exactly what tcgen05.mma expects for a K-major operand with
// the 128-byte swizzle, so the kernel copies it into shared memory linearly.
// transpose = 0 (forward): rows = output channels, slices run over (tap, input-channel block).
// transpose = 1 (dgrad)  : rows = input channels,  slices run over (tap, output-channel block).
// The reduction axis is e = tap * red + r, cut into 64-element slices and zero-padded at the end.
__global__ void weight_image_kernel(const bf16* __restrict__ w, uint16_t* __restrict__ img, int rows,
                                    int red, int K, int transpose, int Cin_w) {
  const int nsl = (K * red + 63) / 64;
  const long total = (long)nsl * rows * 64;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total;
       i += (long)gridDim.x * blockDim.x) {
    const int c = (int)(i % 64);
    const int n = (int)((i / 64) % rows);
    const int s = (int)(i / (64L * rows));
    const int e = s * 64 + c;
    const int tap = e / red, r = e - tap * red;
    const long src = transpose ? ((long)r * Cin_w + n) * K + tap : ((long)n * Cin_w + r) * K + tap;
    const long dst = (long)s * rows * 64 + (long)n * 64 + ((((c >> 3) ^ (n & 7)) << 3) | (c & 7));
    img[dst] = e < K * red ? reinterpret_cast<const uint16_t*>(w)[src] : (uint16_t)0;
  }
}

// ---- inverse map -------------------------------------------------------------------------------
// For every (input pixel q, tap k): the list of (grid pixel p, weight) pairs such that the forward
// sample of tap k at p reads q with that weight.  Built once per sample map; it turns the
// scatter-add of the reference's MappedCol2Im2D (include/nn/common/mapped_im2col.h:45-78) into a
// gather.  Layout of the buffer: int off[nkeys + 1], padded to 16 bytes, then int2 ent[].

struct InvArgs {
  const float* map;
  const float* iw;  // weighted maps: (ngrid, K, P) weights of the P points of every tap; else null
  int P;            // points per tap of a weighted map, 0 for a plain map
  int* cnt;  // pass 1: per-key counts; pass 2: per-key cursors
  const int* off;
  int2* ent;
  long ngrid;  // OH*OW
  int K, IH, IW, interp;
};

template <int PASS>
__global__ void invmap_pass_kernel(InvArgs a) {
  const long total = a.ngrid * a.K;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total;
       i += (long)gridDim.x * blockDim.x) {
    const long p = i / a.K;
    const int k = (int)(i % a.K);
    const int np = a.P > 0 ? a.P : 1;
    for (int pt = 0; pt < np; ++pt) {
      const float2 m = __ldg(reinterpret_cast<const float2*>(a.map) + i * np + pt);
      const float wp = a.P > 0 ? __ldg(a.iw + i * np + pt) : 1.f;
      Tap<float> tp;
      decode_tap<float, float>(m.x, m.y, a.IH, a.IW, a.interp, tp);
      for (int c = 0; c < tp.n; ++c) {
        const float wc = a.P > 0 ? __fmul_rn(wp, tp.w[c]) : tp.w[c];
        if (tp.off[c] < 0 || wc == 0.f) continue;
        const long key = (long)tp.off[c] * a.K + k;
        if (PASS == 1) {
          atomicAdd(a.cnt + key, 1);
        } else {
          const int pos = a.off[key] + atomicAdd(a.cnt + key, 1);
          a.ent[pos] = make_int2((int)p, __float_as_int(wc));
        }
      }
    }
  }
}

// Lists are filled in arrival order; sorting each by (grid pixel, weight bits) makes the sums, and
// so the whole backward pass, reproducible from run to run.
__global__ void invmap_sort_kernel(const int* __restrict__ off, int2* __restrict__ ent, long nkeys) {
  for (long key = blockIdx.x * (long)blockDim.x + threadIdx.x; key < nkeys;
       key += (long)gridDim.x * blockDim.x) {
    const int b = off[key], e = off[key + 1];
    for (int i = b + 1; i < e; ++i) {
      const int2 v = ent[i];
      int j = i - 1;
      while (j >= b && (ent[j].x > v.x || (ent[j].x == v.x && ent[j].y > v.y))) {
        ent[j + 1] = ent[j];
        --j;
      }
      ent[j + 1] = v;
    }
  }
}

// Forward tap table: TapEnt[(pixel of the map grid) * K + tap], offsets relative to the image.
__global__ void tapmap_build_kernel(const float* __restrict__ map, TapEnt* __restrict__ out,
                                    int* __restrict__ out32, long n, int SH, int SW, int interp) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    const float2 m = __ldg(reinterpret_cast<const float2*>(map) + i);
    Tap<float> tp;
    decode_tap<float, float>(m.x, m.y, SH, SW, interp, tp);
    int off[4];
    float w[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const bool on = c < tp.n && tp.off[c] >= 0 && tp.w[c] != 0.f;
      off[c] = on ? tp.off[c] : -1;
      w[c] = on ? tp.w[c] : 0.f;
    }
    if (out32) out32[i] = off[0];  // nearest: the one source pixel, -1 when the tap reads nothing
    seal_entry(off, w);
    uint4* dst = reinterpret_cast<uint4*>(out + i);
    dst[0] = make_uint4(off[0], off[1], off[2], off[3]);
    dst[1] = make_uint4(__float_as_uint(w[0]), __float_as_uint(w[1]), __float_as_uint(w[2]),
                        __float_as_uint(w[3]));
  }
}

// Tap table of a WEIGHTED map (include/core/resample.h:145-162: a tap is the sum over P points of
// weight x sample): the points' source pixels with weight = point weight x interpolation weight,
// packed into the four corners of a TapEnt.  The launcher guarantees P x (corners per point) <= 4,
// e.g. the three barycentric vertices of an icosphere tap with nearest sampling.
__global__ void tapmap_build_weighted_kernel(const float* __restrict__ map, const float* __restrict__ iw,
                                             int P, TapEnt* __restrict__ out, long n, int SH, int SW,
                                             int interp) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    int off[4] = {-1, -1, -1, -1};
    float w[4] = {0.f, 0.f, 0.f, 0.f};
    int nc = 0;
    for (int pt = 0; pt < P; ++pt) {
      const float2 m = __ldg(reinterpret_cast<const float2*>(map) + i * P + pt);
      const float wp = __ldg(iw + i * P + pt);
      Tap<float> tp;
      decode_tap<float, float>(m.x, m.y, SH, SW, interp, tp);
      for (int c = 0; c < tp.n; ++c) {
        const float wc = __fmul_rn(wp, tp.w[c]);
        if (tp.off[c] < 0 || wc == 0.f || nc >= 4) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (j == nc) { off[j] = tp.off[c]; w[j] = wc; }
        ++nc;
      }
    }
    seal_entry(off, w);
    uint4* dst = reinterpret_cast<uint4*>(out + i);
    dst[0] = make_uint4(off[0], off[1], off[2], off[3]);
    dst[1] = make_uint4(__float_as_uint(w[0]), __float_as_uint(w[1]), __float_as_uint(w[2]),
                        __float_as_uint(w[3]));
  }
}

// Inverse tap table: the first four entries of every (input pixel, tap) list in TapEnt form;
// MORE_FLAG marks the lists that go on.
__global__ void invtap_build_kernel(const int* __restrict__ off, const int2* __restrict__ ent,
                                    TapEnt* __restrict__ out, long nkeys) {
  for (long key = blockIdx.x * (long)blockDim.x + threadIdx.x; key < nkeys;
       key += (long)gridDim.x * blockDim.x) {
    const int b = off[key], e = off[key + 1];
    int o[4];
    float w[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      o[c] = -1;
      w[c] = 0.f;
      if (b + c < e) {
        const int2 en = ent[b + c];
        o[c] = en.x;
        w[c] = __int_as_float(en.y);
      }
    }
    seal_entry(o, w);
    if (e - b > 4) o[3] |= MORE_FLAG;
    uint4* dst = reinterpret_cast<uint4*>(out + key);
    dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[1] = make_uint4(__float_as_uint(w[0]), __float_as_uint(w[1]), __float_as_uint(w[2]),
                        __float_as_uint(w[3]));
  }
}

constexpr int MAX_DEVICES = 64;

// SM count of the current device (cached per device ordinal).
static int sm_count() {
  static std::atomic<int> cache[MAX_DEVICES];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return 148;
  int n = cache[dev].load(std::memory_order_relaxed);
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      return 148;  // not cached: asked again next time
    cache[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

// Pipeline stages that fit beside `extra` bytes of resident data (0 = does not fit).
static int pick_stages(size_t extra, int nfloat, int max_st, int min_st, bool even) {
  for (int nst = max_st; nst >= min_st; --nst) {
    if (even && (nst & 1)) continue;
    if (smem_bytes(nst, extra, nfloat, 2 * nst + 16) <= SMEM_LIMIT) return nst;
  }
  return 0;
}

// Opts a kernel in to the full dynamic shared memory of the SM.  The attribute belongs to the
// (device, kernel) pair, so it is set once per device the library is used on; a failure is not
// remembered (the next call tries again).
static bool allow_big_smem_ptr(const void* k) {
  static std::mutex mu;
  static std::set<std::pair<int, const void*>> done;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return false;
  std::lock_guard<std::mutex> g(mu);
  if (done.count({dev, k})) return true;
  if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_LIMIT) !=
      cudaSuccess)
    return false;
  done.insert({dev, k});
  return true;
}
template <typename Kern>
static bool allow_big_smem(Kern k) { return allow_big_smem_ptr(reinterpret_cast<const void*>(k)); }

static bool aligned16(const void* p) { return (((uintptr_t)p) & 15) == 0; }

}  // namespace tc

using namespace tc;

// ---- forward ---------------------------------------------------------------------------------------

// How a forward / dgrad GEMM with `ncol` output columns and `nsl` slices is run.
struct GemmPlan {
  int nout;   // columns per CTA: 64, 128 or 256 (ncol is a multiple of it)
  bool wres;  // weight slices resident in shared memory
  int nst;
  size_t extra;  // shared memory behind the stages: weights + tap table
};

static bool plan_gemm(int ncol, int nsl, int K, GemmPlan& p) {
  if (ncol <= 0 || ncol % 64 != 0) return false;
  // resident weights when they fit with a reasonable pipeline (needs ncol <= 256)
  if (ncol <= 256 && (ncol == 64 || ncol == 128 || ncol == 256)) {
    const size_t extra = (size_t)nsl * ncol * 128 + tap_table_bytes(K) + EPI_STAGING_BYTES;
    const int nst = pick_stages(extra, ncol, 8, 3, false);
    if (nst > 0) { p = {ncol, true, nst, extra}; return true; }
  }
  const int nout = ncol % 256 == 0 ? 256 : ncol % 128 == 0 ? 128 : 64;
  // streamed weights: every stage carries its weight slice
  for (int nst = 6; nst >= 3; --nst) {
    const size_t extra = (size_t)nst * nout * 128 + tap_table_bytes(K) + EPI_STAGING_BYTES;
    if (smem_bytes(nst, extra, nout, 2 * nst + 16) <= SMEM_LIMIT) {
      p = {nout, false, nst, extra};
      return true;
    }
  }
  return false;
}

// 64-element slices of the gathered (tap, input channel) axis of forward / wgrad
static int fwd_slices(const mc_desc* d) { return (int)(((long)d->K * d->C_in + 63) / 64); }

bool conv_tc_fwd_supported(const mc_desc* d) {
  if (d->dtype != MC_BF16 || d->layout != MC_NHWC || d->P != 0) return false;
  if ((long)d->K * d->C_in >= (1L << 24)) return false;
  GemmPlan p;
  return plan_gemm(d->C_out, fwd_slices(d), d->K, p);
}

// Streamed weights need the prebuilt tap table; when the caller passes the raw sample map the
// table is built into the workspace first.
// One-slice layers (K * C_in <= 64) use the row-per-thread producer, which reads the table from
// global memory.
static bool rowwise_shape(const mc_desc* d) { return d->C_in % 64 != 0 && (long)d->K * d->C_in <= 64; }

static bool fwd_needs_table(const mc_desc* d) {
  GemmPlan p;
  if (!plan_gemm(d->C_out, fwd_slices(d), d->K, p)) return false;
  return !p.wres || (rowwise_shape(d) && p.nst >= ROW_TEAMS);
}

size_t conv_tc_fwd_wimg_bytes(const mc_desc* d) {
  return ((size_t)fwd_slices(d) * 64 * d->C_out * sizeof(bf16) + 255) & ~(size_t)255;
}

size_t tapmap_bytes(const mc_desc* d);

size_t conv_tc_fwd_ws(const mc_desc* d) {
  return conv_tc_fwd_wimg_bytes(d) + (fwd_needs_table(d) ? tapmap_bytes(d) : 0);
}

template <int NOUT, bool CSR>
static int launch_gemm_n(const GemmArgs& a, const GemmPlan& p, bool pre, cudaStream_t st) {
  const size_t smem = smem_bytes(a.nst, p.extra, NOUT, 2 * a.nst + 9);
  const int ny = a.ncol / NOUT;
  int gx = sm_count() / ny;
  if (gx < 1) gx = 1;
  if (gx > a.t.tiles) gx = a.t.tiles;
  const dim3 grid(gx, ny);
  if (p.wres) {
    if (pre) {
      if (!allow_big_smem(conv_gemm_tc_kernel<NOUT, CSR, true, true>)) return MC_ERR_LAUNCH;
      conv_gemm_tc_kernel<NOUT, CSR, true, true><<<grid, TC_THREADS, smem, st>>>(a), MC_COUNT(1);
    } else {
      if (CSR) return MC_ERR_UNSUPPORTED;
      if (!allow_big_smem(conv_gemm_tc_kernel<NOUT, false, false, true>)) return MC_ERR_LAUNCH;
      conv_gemm_tc_kernel<NOUT, false, false, true><<<grid, TC_THREADS, smem, st>>>(a), MC_COUNT(1);
    }
  } else {
    if (!pre) return MC_ERR_UNSUPPORTED;
    if (!allow_big_smem(conv_gemm_tc_kernel<NOUT, CSR, true, false>)) return MC_ERR_LAUNCH;
    conv_gemm_tc_kernel<NOUT, CSR, true, false><<<grid, TC_THREADS, smem, st>>>(a), MC_COUNT(1);
  }
  MC_CHECK_LAUNCH();
  return MC_OK;
}

template <bool CSR>
static int launch_gemm(const GemmArgs& a, const GemmPlan& p, bool pre, cudaStream_t st) {
  switch (p.nout) {
    case 64: return launch_gemm_n<64, CSR>(a, p, pre, st);
    case 128: return launch_gemm_n<128, CSR>(a, p, pre, st);
    case 256: return launch_gemm_n<256, CSR>(a, p, pre, st);
  }
  return MC_ERR_UNSUPPORTED;
}

// Forward tap table of a sample map (one TapEnt per map entry).
// Nearest maps carry a second, compact form behind the records: one int per entry (the source
// pixel, or -1), which the row-per-thread producer reads with coalesced loads.
static bool tapmap_has_compact(const mc_desc* d) { return d->interp != 1 && d->interp != 2; }
static const int* tapmap_compact(const mc_desc* d, const void* tab) {
  if (!tab || !tapmap_has_compact(d)) return nullptr;
  return reinterpret_cast<const int*>((const uint8_t*)tab + (size_t)d->OH * d->OW * d->K * sizeof(TapEnt));
}

size_t tapmap_bytes(const mc_desc* d) {
  const size_t n = (size_t)d->OH * d->OW * d->K;
  return n * sizeof(TapEnt) + (tapmap_has_compact(d) ? ((n * sizeof(int) + 15) & ~(size_t)15) : 0);
}

int tapmap_build_launch(const mc_desc* d, const void* map, void* tab, cudaStream_t st) {
  if (!aligned16(map) || !aligned16(tab)) return MC_ERR_BAD_ARG;
  const long n = (long)d->OH * d->OW * d->K;
  tapmap_build_kernel<<<grid_for(n, 256), 256, 0, st>>>((const float*)map, (TapEnt*)tab,
                                                        const_cast<int*>(tapmap_compact(d, tab)), n,
                                                        d->IH, d->IW, d->interp), MC_COUNT(1);
  MC_CHECK_LAUNCH();
  return MC_OK;
}

// A weighted map whose taps fit a TapEnt (P points x corners per point <= 4) is "folded": its plans
// are built from (map, weights) and then used exactly like the plans of a plain bilinear map, under
// the descriptor this returns in *folded (P = 0, interp = bilinear: four weighted corners per tap).
bool weighted_fold(const mc_desc* d, mc_desc* folded) {
  if (d->P <= 0) return false;
  const int corners = (d->interp == 1 || d->interp == 2) ? 4 : 1;
  if (d->P * corners > 4) return false;
  *folded = *d;
  folded->P = 0;
  folded->interp = 1;
  return true;
}

int tapmap_build_weighted_launch(const mc_desc* d, const void* map, const void* iw, void* tab,
                                 cudaStream_t st) {
  if (!aligned16(map) || !aligned16(tab)) return MC_ERR_BAD_ARG;
  const long n = (long)d->OH * d->OW * d->K;
  tapmap_build_weighted_kernel<<<grid_for(n, 256), 256, 0, st>>>((const float*)map, (const float*)iw, d->P,
                                                                 (TapEnt*)tab, n, d->IH, d->IW, d->interp),
      MC_COUNT(1);
  MC_CHECK_LAUNCH();
  return MC_OK;
}

// map != null: the kernel decodes the map itself; tab != null: prebuilt table (tapmap_build_launch)
static int fwd_launch_impl(const mc_desc* d, const void* x, const void* map, const void* tab,
                           const void* w, const void* bias, void* y, void* ws, size_t ws_bytes,
                           cudaStream_t st) {
  if (!ws || ws_bytes < (tab ? (size_t)fwd_slices(d) * 64 * d->C_out * sizeof(bf16) : conv_tc_fwd_ws(d)))
    return MC_ERR_WORKSPACE;
  if (!aligned16(x) || !aligned16(y) || !aligned16(ws) || !aligned16(map) || !aligned16(tab))
    return MC_ERR_BAD_ARG;
  if ((long)d->B * d->IH * d->IW >= (1L << 30)) return MC_ERR_TOO_LARGE;
  GemmArgs a = {};
  a.s.src = (const bf16*)x; a.s.spix = (long)d->IH * d->IW; a.s.C = d->C_in;
  a.s.SH = d->IH; a.s.SW = d->IW; a.s.K = d->K; a.s.interp = d->interp;
  a.s.src_elems = (long)d->B * d->IH * d->IW * d->C_in;
  a.s.map = (const float*)map;
  a.s.tab = (const TapEnt*)tab;
  if (!make_tiling(a.t, d->B, d->OH, d->OW)) return MC_ERR_TOO_LARGE;
  a.wimg = (const uint4*)ws; a.bias = (const bf16*)bias; a.y = (bf16*)y;
  a.nsl = fwd_slices(d);
  a.s.KC = d->K * d->C_in;
  a.s.packed = d->C_in % 64 != 0;
  a.ncol = d->C_out;
  a.relu = (d->flags & MC_FLAG_RELU) ? 1 : 0;
  GemmPlan p;
  if (!plan_gemm(a.ncol, a.nsl, d->K, p)) return MC_ERR_UNSUPPORTED;
  a.nst = p.nst;
  const long nw = (long)a.nsl * 64 * d->C_out;
  weight_image_kernel<<<grid_for(nw, 256), 256, 0, st>>>((const bf16*)w, (uint16_t*)ws, d->C_out,
                                                         d->C_in, d->K, 0, d->C_in), MC_COUNT(1);
  if (!tab && fwd_needs_table(d)) {  // build the table behind the weight image
    void* t = (uint8_t*)ws + conv_tc_fwd_wimg_bytes(d);
    const int rc = tapmap_build_launch(d, map, t, st);
    if (rc) return rc;
    a.s.tab = (const TapEnt*)t;
  }
  a.full_cnt = N_PRODUCER_WARPS;
  if (a.s.tab && rowwise_shape(d) && p.nst >= ROW_TEAMS) {
    a.s.packed = 2;
    a.full_cnt = N_PRODUCER_WARPS / ROW_TEAMS;
    a.s.tab32 = tapmap_compact(d, a.s.tab);
  }
  return launch_gemm<false>(a, p, a.s.tab != nullptr, st);
}

int conv_tc_fwd_launch(const mc_desc* d, const void* x, const void* map, const void* w,
                       const void* bias, void* y, void* ws, size_t ws_bytes, cudaStream_t st) {
  return fwd_launch_impl(d, x, map, nullptr, w, bias, y, ws, ws_bytes, st);
}

int conv_tc_fwd_tab_launch(const mc_desc* d, const void* x, const void* tab, const void* w,
                           const void* bias, void* y, void* ws, size_t ws_bytes, cudaStream_t st) {
  return fwd_launch_impl(d, x, nullptr, tab, w, bias, y, ws, ws_bytes, st);
}

// ---- inverse map ---------------------------------------------------------------------------------------

static size_t inv_off_bytes(const mc_desc* d) {
  const size_t nkeys = (size_t)d->IH * d->IW * d->K;
  return ((nkeys + 1) * sizeof(int) + 15) & ~(size_t)15;
}
static size_t inv_max_entries(const mc_desc* d) {
  const size_t per = (d->interp == 1 || d->interp == 2) ? 4 : 1;
  return (size_t)d->OH * d->OW * d->K * per;
}

size_t invmap_off_bytes(const mc_desc* d) { return inv_off_bytes(d); }

bool invmap_supported(const mc_desc* d) {
  if (d->P != 0 || d->dtype == MC_F64) return false;
  return (size_t)d->IH * d->IW * d->K < (1u << 30) && inv_max_entries(d) < (1u << 31);
}
// layout: int off[nkeys + 1] | int2 ent[max entries] | TapEnt table[nkeys]   (each part 32-byte aligned)
static size_t inv_tab_offset(const mc_desc* d) {
  return (inv_off_bytes(d) + inv_max_entries(d) * sizeof(int2) + 31) & ~(size_t)31;
}
size_t invmap_bytes(const mc_desc* d) {
  return inv_tab_offset(d) + (size_t)d->IH * d->IW * d->K * sizeof(TapEnt);
}

static size_t scan_temp_bytes(size_t n) {
  size_t t = 0;
  cub::DeviceScan::ExclusiveSum(nullptr, t, (const int*)nullptr, (int*)nullptr, (int)n);
  return (t + 255) & ~(size_t)255;
}
size_t invmap_build_ws(const mc_desc* d) {
  const size_t nkeys = (size_t)d->IH * d->IW * d->K;
  return (((nkeys + 1) * sizeof(int) + 255) & ~(size_t)255) + scan_temp_bytes(nkeys + 1);
}

// iw != null: d_in is a weighted descriptor that folds (weighted_fold); the buffer then has the layout
// of the folded descriptor, which is the one the consumers are called with.
int invmap_build_launch(const mc_desc* d_in, const void* map, const void* iw, void* inv, void* ws,
                        size_t ws_bytes, cudaStream_t st) {
  mc_desc folded;
  const mc_desc* d = d_in;
  if (iw) {
    if (!weighted_fold(d_in, &folded)) return MC_ERR_UNSUPPORTED;
    d = &folded;
  }
  if (!invmap_supported(d)) return MC_ERR_UNSUPPORTED;
  if (!ws || ws_bytes < invmap_build_ws(d)) return MC_ERR_WORKSPACE;
  if (!aligned16(inv) || !aligned16(ws)) return MC_ERR_BAD_ARG;
  const size_t nkeys = (size_t)d->IH * d->IW * d->K;
  const size_t cnt_bytes = ((nkeys + 1) * sizeof(int) + 255) & ~(size_t)255;
  InvArgs a;
  a.map = (const float*)map;
  a.iw = (const float*)iw;
  a.P = iw ? d_in->P : 0;
  a.cnt = (int*)ws;
  a.off = (const int*)inv;
  a.ent = (int2*)((uint8_t*)inv + inv_off_bytes(d));
  a.ngrid = (long)d->OH * d->OW;
  a.K = d->K; a.IH = d->IH; a.IW = d->IW; a.interp = d_in->interp;
  if (cudaMemsetAsync(a.cnt, 0, (nkeys + 1) * sizeof(int), st) != cudaSuccess) return MC_ERR_LAUNCH;
  const int grid = grid_for(a.ngrid * a.K, 256);
  invmap_pass_kernel<1><<<grid, 256, 0, st>>>(a), MC_COUNT(1);
  size_t tb = ws_bytes - cnt_bytes;
  if (cub::DeviceScan::ExclusiveSum((uint8_t*)ws + cnt_bytes, tb, a.cnt, (int*)inv, (int)(nkeys + 1),
                                    st) != cudaSuccess)
    return MC_ERR_LAUNCH;
  if (cudaMemsetAsync(a.cnt, 0, (nkeys + 1) * sizeof(int), st) != cudaSuccess) return MC_ERR_LAUNCH;
  invmap_pass_kernel<2><<<grid, 256, 0, st>>>(a), MC_COUNT(1);
  invmap_sort_kernel<<<grid_for((long)nkeys, 256), 256, 0, st>>>(a.off, a.ent, (long)nkeys), MC_COUNT(1);
  invtap_build_kernel<<<grid_for((long)nkeys, 256), 256, 0, st>>>(
      a.off, a.ent, (TapEnt*)((uint8_t*)inv + inv_tab_offset(d)), (long)nkeys), MC_COUNT(1);
  MC_CHECK_LAUNCH();
  return MC_OK;
}

// ---- dgrad through the inverse map ---------------------------------------------------------------------

bool conv_tc_dgrad_supported(const mc_desc* d) {
  if (d->dtype != MC_BF16 || d->layout != MC_NHWC || d->P != 0) return false;
  if (d->C_out % 64 != 0) return false;
  if (!invmap_supported(d)) return false;
  GemmPlan p;
  return plan_gemm(d->C_in, d->K * (d->C_out / 64), d->K, p);
}

size_t conv_tc_dgrad_ws(const mc_desc* d) {
  return (size_t)d->K * d->C_in * d->C_out * sizeof(bf16);
}

int conv_tc_dgrad_launch(const mc_desc* d, const void* gy, const void* inv, const void* w,
                         const void* bias_out, void* gx, void* ws, size_t ws_bytes,
                         cudaStream_t st) {
  if (!ws || ws_bytes < conv_tc_dgrad_ws(d)) return MC_ERR_WORKSPACE;
  if (!aligned16(gy) || !aligned16(gx) || !aligned16(ws) || !aligned16(inv)) return MC_ERR_BAD_ARG;
  GemmArgs a = {};
  a.s.src = (const bf16*)gy; a.s.spix = (long)d->OH * d->OW; a.s.C = d->C_out;
  a.s.K = d->K; a.s.interp = d->interp;
  a.s.inv_off = (const int*)inv;
  a.s.inv_ent = (const int2*)((const uint8_t*)inv + inv_off_bytes(d));
  a.s.tab = (const TapEnt*)((const uint8_t*)inv + inv_tab_offset(d));
  if ((long)d->B * d->OH * d->OW >= (1L << 30)) return MC_ERR_TOO_LARGE;
  if (!make_tiling(a.t, d->B, d->IH, d->IW)) return MC_ERR_TOO_LARGE;
  a.wimg = (const uint4*)ws; a.bias = (const bf16*)bias_out; a.y = (bf16*)gx;
  a.nsl = d->K * (d->C_out / 64);
  a.ncol = d->C_in;
  a.relu = (bias_out && (d->flags & MC_FLAG_RELU)) ? 1 : 0;  // the transposed layer's forward
  GemmPlan p;
  if (!plan_gemm(a.ncol, a.nsl, d->K, p)) return MC_ERR_UNSUPPORTED;
  a.nst = p.nst;
  a.full_cnt = N_PRODUCER_WARPS;
  const long nw = (long)d->K * d->C_in * d->C_out;
  weight_image_kernel<<<grid_for(nw, 256), 256, 0, st>>>((const bf16*)w, (uint16_t*)ws, d->C_in,
                                                         d->C_out, d->K, 1, d->C_in), MC_COUNT(1);
  return launch_gemm<true>(a, p, true, st);
}

// ---- wgrad -----------------------------------------------------------------------------------------------

// How the weight gradient is split over CTAs: chunks of `nout` output channels (blockIdx.z) times
// groups of `mtpg` M = 128 tiles of the (tap, input channel) axis (blockIdx.y); mtpg * nout partial
// sums per pixel-tile row must fit the 512 TMEM columns.
struct WgradPlan {
  int nout, mtpg, groups, chunks, nst;
  size_t extra;
};

static bool plan_wgrad(const mc_desc* d, WgradPlan& p) {
  if (d->C_out % 64 != 0 || (long)d->K * d->C_in >= (1L << 24)) return false;
  const int nsl = fwd_slices(d);
  const int nmt = (nsl + 1) / 2;
  p.nout = d->C_out % 128 == 0 ? 128 : 64;
  p.chunks = d->C_out / p.nout;
  const int cap = 512 / p.nout;
  p.groups = (nmt + cap - 1) / cap;
  p.mtpg = (nmt + p.groups - 1) / p.groups;
  p.extra = (size_t)GY_STAGES * (p.nout / 64) * STAGE_BYTES + tap_table_bytes(d->K);
  p.nst = pick_stages(p.extra, p.nout, 10, 4, true);
  return p.nst > 0;
}

bool conv_tc_wgrad_supported(const mc_desc* d) {
  if (d->dtype != MC_BF16 || d->layout != MC_NHWC || d->P != 0) return false;
  WgradPlan p;
  return plan_wgrad(d, p);
}
size_t conv_tc_wgrad_ws(const mc_desc*) { return 0; }

template <int NOUT>
static int launch_wgrad_n(const GemmArgs& a, const WgradPlan& p, bool pre, cudaStream_t st) {
  const size_t smem = smem_bytes(a.nst, p.extra, NOUT, 2 * a.nst + 2 * GY_STAGES + 5);
  int gx = sm_count() / (p.groups * p.chunks);
  if (gx < 1) gx = 1;
  if (gx > a.t.tiles) gx = a.t.tiles;
  const dim3 grid(gx, p.groups, p.chunks);
  if (!allow_big_smem(conv_wgrad_tc_kernel<NOUT, false>) ||
      !allow_big_smem(conv_wgrad_tc_kernel<NOUT, true>))
    return MC_ERR_LAUNCH;
  if (pre) conv_wgrad_tc_kernel<NOUT, true><<<grid, TC_THREADS, smem, st>>>(a), MC_COUNT(1);
  else conv_wgrad_tc_kernel<NOUT, false><<<grid, TC_THREADS, smem, st>>>(a), MC_COUNT(1);
  MC_CHECK_LAUNCH();
  return MC_OK;
}

#include "conv_smallcin.cuh"

// ymask != null: grad_output is masked by (ymask > 0) on the way in (only the kernel for very few
// input channels can do that; MC_ERR_UNSUPPORTED otherwise)
static int wgrad_launch_impl(const mc_desc* d, const void* gy, const void* x, const void* map,
                             const void* tab, void* gw, void* gb, cudaStream_t st,
                             const void* ymask = nullptr) {
  if (ymask && !(tab && smallcin_wgrad_shape(d) && tapmap_compact(d, tab))) return MC_ERR_UNSUPPORTED;
  if (!aligned16(ymask)) return MC_ERR_BAD_ARG;
  if (!aligned16(gy) || !aligned16(x) || !aligned16(map) || !aligned16(tab)) return MC_ERR_BAD_ARG;
  if ((long)d->B * d->IH * d->IW >= (1L << 30)) return MC_ERR_TOO_LARGE;
  GemmArgs a = {};
  a.s.src = (const bf16*)x; a.s.spix = (long)d->IH * d->IW; a.s.C = d->C_in;
  a.s.SH = d->IH; a.s.SW = d->IW; a.s.K = d->K; a.s.interp = d->interp;
  a.s.src_elems = (long)d->B * d->IH * d->IW * d->C_in;
  a.s.map = (const float*)map;
  a.s.tab = (const TapEnt*)tab;
  if (!make_tiling(a.t, d->B, d->OH, d->OW)) return MC_ERR_TOO_LARGE;
  a.gy = (const bf16*)gy; a.gw = (float*)gw; a.gb = (float*)gb;
  a.nsl = fwd_slices(d);
  a.s.KC = d->K * d->C_in;
  a.s.packed = d->C_in % 64 != 0;
  a.ncol = d->C_out;
  WgradPlan p;
  if (!plan_wgrad(d, p)) return MC_ERR_UNSUPPORTED;
  a.nst = p.nst;
  a.mtpg = p.mtpg;
  a.full_cnt = N_PRODUCER_WARPS;
  if (tab && rowwise_shape(d) && p.nst >= ROW_TEAMS) {
    a.s.packed = 2;
    a.full_cnt = N_PRODUCER_WARPS / ROW_TEAMS;
    a.s.tab32 = tapmap_compact(d, tab);
  }
  if (cudaMemsetAsync(gw, 0, (size_t)d->C_out * d->C_in * d->K * sizeof(float), st) != cudaSuccess)
    return MC_ERR_LAUNCH;
  if (gb && cudaMemsetAsync(gb, 0, (size_t)d->C_out * sizeof(float), st) != cudaSuccess)
    return MC_ERR_LAUNCH;
  // very few input channels and a nearest map with its compact table: one pass over grad_output
  if (tab && smallcin_wgrad_shape(d) && tapmap_compact(d, tab))
    return smallcin_wgrad_launch(d, gy, ymask, x, tapmap_compact(d, tab), gw, gb, st);
  return p.nout == 128 ? launch_wgrad_n<128>(a, p, tab != nullptr, st)
                       : launch_wgrad_n<64>(a, p, tab != nullptr, st);
}

int conv_tc_wgrad_launch(const mc_desc* d, const void* gy, const void* x, const void* map, void* gw,
                         void* gb, void* ws, size_t ws_bytes, cudaStream_t st) {
  (void)ws; (void)ws_bytes;
  return wgrad_launch_impl(d, gy, x, map, nullptr, gw, gb, st);
}

int conv_tc_wgrad_tab_launch(const mc_desc* d, const void* gy, const void* x, const void* tab,
                             void* gw, void* gb, cudaStream_t st) {
  return wgrad_launch_impl(d, gy, x, nullptr, tab, gw, gb, st);
}

int conv_tc_wgrad_tab_relu_launch(const mc_desc* d, const void* gy, const void* y, const void* x,
                                  const void* tab, void* gw, void* gb, cudaStream_t st) {
  return wgrad_launch_impl(d, gy, x, nullptr, tab, gw, gb, st, y);
}

// ---- forward pass with library-owned scratch ---------------------------------------------------
// The tensor-core forward needs a small scratch buffer (the weights re-laid-out for the MMA
// unit).  mc_conv_fwd() takes it from the caller; this variant keeps it in a fixed array inside
// the library image instead, for callers that have no way to obtain device memory at call time.
constexpr size_t STATIC_SCRATCH_BYTES = 80 * 1024;
static __device__ __align__(256) unsigned char g_static_scratch[STATIC_SCRATCH_BYTES];
constexpr int STATIC_SCRATCH_MAX_DEVICES = 64;
// Device address of g_static_scratch for every device ordinal (the symbol itself is only a host
// stand-in; kernels must be given the address the runtime reports for the current device).
static void* g_static_scratch_addr[STATIC_SCRATCH_MAX_DEVICES] = {nullptr};

int check_conv_desc_public(const mc_desc* d);

extern "C" size_t mc_conv_fwd_static_scratch_limit(void) { return STATIC_SCRATCH_BYTES; }

extern "C" int mc_conv_fwd_static_scratch(const mc_desc* d, const void* x, const void* map,
                                          const void* w, const void* bias, void* y, void* stream) {
  int rc = check_conv_desc_public(d);
  if (rc) return rc;
  if (!x || !map || !w || !y) return MC_ERR_BAD_ARG;
  if (!conv_tc_fwd_supported(d)) return MC_ERR_UNSUPPORTED;
  if (conv_tc_fwd_ws(d) > STATIC_SCRATCH_BYTES) return MC_ERR_TOO_LARGE;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= STATIC_SCRATCH_MAX_DEVICES)
    return MC_ERR_LAUNCH;
  void* scratch = g_static_scratch_addr[dev];
  if (!scratch) {  // first call on this device: look the array's device address up once
    if (cudaGetSymbolAddress(&scratch, g_static_scratch) != cudaSuccess || !scratch)
      return MC_ERR_LAUNCH;
    g_static_scratch_addr[dev] = scratch;
  }
  return conv_tc_fwd_launch(d, x, map, w, bias, y, scratch, STATIC_SCRATCH_BYTES,
                            (cudaStream_t)stream);
}

// ---- self-test of the bounded waits ---------------------------------------------------------------
// One warp waits, with a limit of about a millisecond, on an mbarrier that nobody ever arrives at.
// The wait must give up, raise the block's abort flag and the device status word, and the kernel
// must return: the same path a tensor-core kernel takes if one of its roles stops answering.
constexpr int SELFTEST_STATUS = 0x7F1;
__global__ void wait_expiry_selftest_kernel(long long limit_cycles, int* observed) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag, wait_ok;
  if (threadIdx.x == 0) {
    tc::mbar_init(tc::smem_u32(&bar), 1);
    abort_flag = 0;
    tc::fence_barrier_init();
  }
  __syncthreads();
  if (threadIdx.x == 0)
    wait_ok = tc::mbar_wait(tc::smem_u32(&bar), 0, &abort_flag, SELFTEST_STATUS, 64, limit_cycles) ? 1 : 0;
  __syncthreads();
  // the other lanes see the abort flag, as the roles of a real kernel do
  if (threadIdx.x == 1 && observed) *observed = (abort_flag ? 2 : 0) | (wait_ok ? 1 : 0);
}

extern "C" int mc_selftest_wait_expiry(int32_t* observed_dev, void* stream) {
  wait_expiry_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(2000000LL, observed_dev), MC_COUNT(1);
  MC_CHECK_LAUNCH();
  return MC_OK;
}

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

#include "conv_rowinv.cuh"
