// Two utility ops of the reference's extension package that sit beside the layer path:
//
//   mc_cube2rect        cube map -> equirectangular image
//                       (replaces Cube2RectKernel / Cube2RectLauncher, include/util/cuda/cube2rect.cuh:15-82,
//                        and Cube2RectForward, src/util/cuda/cube2rect_layer.cu:11-29)
//   mc_voting_resample  label images scattered through an integer map, majority vote per target pixel
//                       (replaces ResampleToMap2DVotingLauncher, include/nn/cuda/resample.cuh:166-200,
//                        Vote2D, include/core/interpolation.h:241-257, and VotingResampleToMap,
//                        src/nn/cuda/voting_resample_layer.cu:10-38)
//
// Both are HBM-bound integer / gather work: one pass over the result (cube2rect) or over the input
// plus a vote table (voting), coalesced along the image rows.
#include "common.cuh"

namespace mc {

// ------------------------------------------------------------------------------------------------
// cube2rect.  One thread per pixel of the equirectangular image: the pixel's direction on the
// sphere, the cube face it leaves through and its position on that face are computed once and
// reused for every channel (the reference recomputes them per channel).  The arithmetic is spelled
// the way include/core/conversions.h:21-38,66-135 spells it, in the image's own type with the
// double-precision pi of <math.h>, so that the compiler rounds and contracts it the same way.
//
// The cube map is a (C, D, 6 D) image, faces side by side in the order -z, -x, +z, +x, +y, -y.
// The reference samples a face through its interpolation helpers with the face's first column as
// the origin and the whole 6 D row as the row length (cube2rect.cuh:46-62), so "inside" means
// 0 <= x < 6 D from the face's origin and 0 <= y < D: the right neighbour of a face's last column is
// the next face's first column.  It enters the result with weight zero (u <= D - 1); reads that
// would leave the tensor are replaced by zero here.
template <typename T>
__device__ __forceinline__ T cube_fetch(const T* __restrict__ ch, long flat, long count) {
  return flat >= 0 && flat < count ? ldv(ch + flat) : T(0);
}

template <typename T>
__global__ void __launch_bounds__(256) cube2rect_kernel(const T* __restrict__ cube, int C, long D, int RH, int RW,
                                                        int interp, T* __restrict__ rect) {
  const long pix = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (pix >= (long)RH * RW) return;
  const int64_t xr = pix % RW, yr = pix / RW;
  const int64_t width = RW, height = RH;
  const T lon = 2 * M_PI * (T(xr) - T(width) / 2) / T(width);
  const T lat = M_PI * (T(yr) - (T(height) - 1) / 2) / (T(height) - 1);
  const T x = cos(lat) * sin(lon);
  const T y = -sin(lat);
  const T z = cos(lat) * cos(lon);
  const T ax = fabs(x), ay = fabs(y), az = fabs(z);
  // Face selection: six tests in the reference's order, a later hit replaces an earlier one (that
  // decides directions that lie exactly on an edge or a corner of the cube).
  int64_t face = 0;
  T major = T(1), uc = T(0), vc = T(0);
  const bool xp = x > 0, yp = y > 0, zp = z > 0;
  const bool xmaj = ax >= ay && ax >= az, ymaj = ay >= ax && ay >= az, zmaj = az >= ax && az >= ay;
  if (xp && xmaj) { major = ax; uc = -z; vc = -y; face = 3; }
  if (!xp && xmaj) { major = ax; uc = z; vc = -y; face = 1; }
  if (yp && ymaj) { major = ay; uc = x; vc = z; face = 4; }
  if (!yp && ymaj) { major = ay; uc = x; vc = -z; face = 5; }
  if (zp && zmaj) { major = az; uc = x; vc = -y; face = 2; }
  if (!zp && zmaj) { major = az; uc = -x; vc = -y; face = 0; }
  T u = T(0.5) * (uc / major + T(1));
  T v = T(0.5) * (vc / major + T(1));
  u *= (D - 1);
  v *= (D - 1);

  const long row = 6 * D, per_channel = D * row, total = (long)C * per_channel;
  const long face0 = face * D;
  const long out_stride = (long)RH * RW;
  if (interp == 0) {
    const int64_t xi = llround(double(u)), yi = llround(double(v));
    const bool ok = xi >= 0 && xi <= row - 1 && yi >= 0 && yi <= D - 1;
    const long off = face0 + yi * row + xi;
    for (int c = 0; c < C; ++c) {
      const long flat = (long)c * per_channel + off;
      rect[(long)c * out_stride + pix] = ok ? cube_fetch(cube, flat, total) : T(0);
    }
  } else {
    const int64_t x1 = (int64_t)floor(u), y1 = (int64_t)floor(v);
    const int64_t x2 = x1 + 1, y2 = y1 + 1;
    const bool x1v = x1 >= 0 && x1 <= row - 1, x2v = x2 >= 0 && x2 <= row - 1;
    const bool y1v = y1 >= 0 && y1 <= D - 1, y2v = y2 >= 0 && y2 <= D - 1;
    const T wa = y2 - v, wb = x2 - u, wc = u - x1, wd = v - y1;
    for (int c = 0; c < C; ++c) {
      const long base = (long)c * per_channel + face0;
      const T d11 = x1v && y1v ? cube_fetch(cube, base + y1 * row + x1, total) : T(0);
      const T d21 = x2v && y1v ? cube_fetch(cube, base + y1 * row + x2, total) : T(0);
      const T d12 = x1v && y2v ? cube_fetch(cube, base + y2 * row + x1, total) : T(0);
      const T d22 = x2v && y2v ? cube_fetch(cube, base + y2 * row + x2, total) : T(0);
      const T p11 = wa * wb * d11;
      const T p21 = wa * wc * d21;
      const T p12 = wd * wb * d12;
      const T p22 = wd * wc * d22;
      rect[(long)c * out_stride + pix] = p11 + p21 + p12 + p22;
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Voting resample.  labels (B, C, IH, IW) int64, map (IH, IW, 2) int64 (x, y) target pixel of every
// source pixel.  Pass 1 counts, per target pixel and label, the source pixels that land there
// (32-bit counters: a count is at most IH * IW); pass 2 takes the label with the most votes, the
// smallest label among equals, 0 for a pixel nobody voted for (the first maximum, as
// torch.argmax over the candidate axis does in the reference).  Labels outside
// [0, num_candidates) do not vote (the reference would write outside its table).
// As in the reference (include/nn/common/resample.h:122) the votes of channel c of an image start
// c * OH * OW counters into the image's (C, OH, OW, candidates) table, not c * OH * OW * candidates:
// with more than one channel the channels' votes overlap, and the result is the argmax over that
// table, whatever it means; one channel - a label image - is unaffected.
__global__ void __launch_bounds__(256) vote_count_kernel(const int64_t* __restrict__ labels,
                                                         const int64_t* __restrict__ map, long planes, int C, int IH,
                                                         int IW, int OH, int OW, int NC, int* __restrict__ votes) {
  const long per_plane = (long)IH * IW;
  const long n = planes * per_plane;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    const long src = i % per_plane, plane = i / per_plane;
    const longlong2 xy = __ldg(reinterpret_cast<const longlong2*>(map) + src);
    const int64_t label = __ldg(labels + i);
    if (xy.x < 0 || xy.x > OW - 1 || xy.y < 0 || xy.y > OH - 1) continue;
    if (label < 0 || label >= NC) continue;
    const long image = plane / C, c = plane % C;
    atomicAdd(votes + (image * C * NC + c) * OH * OW + (xy.y * OW + xy.x) * NC + label, 1);
  }
}

__global__ void __launch_bounds__(256) vote_pick_kernel(const int* __restrict__ votes, long pixels, int NC,
                                                        int64_t* __restrict__ out) {
  for (long p = (long)blockIdx.x * blockDim.x + threadIdx.x; p < pixels; p += (long)gridDim.x * blockDim.x) {
    const int* v = votes + p * NC;
    int best = __ldg(v), arg = 0;
    for (int k = 1; k < NC; ++k) {
      const int c = __ldg(v + k);
      if (c > best) { best = c; arg = k; }
    }
    out[p] = arg;
  }
}

static int vote_grid(long n, int threads) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long want = (n + threads - 1) / threads;
  const long cap = (long)sms * 16;  // grid-stride loops: a few resident blocks per SM are enough
  return (int)(want < cap ? (want > 0 ? want : 1) : cap);
}

}  // namespace mc

extern "C" int mc_cube2rect(int32_t dtype, const void* cube, int32_t channels, int32_t cube_dim, int32_t rect_h,
                            int32_t rect_w, int32_t interp, void* rect, void* stream) {
  using namespace mc;
  if (!cube || !rect) return MC_ERR_BAD_ARG;
  if (channels <= 0 || cube_dim <= 0 || rect_h <= 0 || rect_w <= 0) return MC_ERR_BAD_ARG;
  if (interp != 0 && interp != 1) return MC_ERR_BAD_ARG;
  if (dtype != MC_F32 && dtype != MC_F64) return MC_ERR_UNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
  const long pixels = (long)rect_h * rect_w;
  const int threads = 256;
  const unsigned blocks = (unsigned)((pixels + threads - 1) / threads);
  if (dtype == MC_F32)
    cube2rect_kernel<float><<<blocks, threads, 0, st>>>((const float*)cube, channels, cube_dim, rect_h, rect_w,
                                                        interp, (float*)rect);
  else
    cube2rect_kernel<double><<<blocks, threads, 0, st>>>((const double*)cube, channels, cube_dim, rect_h, rect_w,
                                                         interp, (double*)rect);
  MC_COUNT(1);
  MC_CHECK_LAUNCH();
  return MC_OK;
}

extern "C" size_t mc_voting_resample_workspace(int32_t B, int32_t C, int32_t OH, int32_t OW, int32_t num_candidates) {
  if (B <= 0 || C <= 0 || OH <= 0 || OW <= 0 || num_candidates <= 0) return 0;
  return (size_t)B * C * OH * OW * num_candidates * sizeof(int);
}

extern "C" int mc_voting_resample(const int64_t* labels, const int64_t* map, int32_t B, int32_t C, int32_t IH,
                                  int32_t IW, int32_t OH, int32_t OW, int32_t num_candidates, void* ws,
                                  size_t ws_bytes, int64_t* out, void* stream) {
  using namespace mc;
  if (!labels || !map || !out) return MC_ERR_BAD_ARG;
  if (B <= 0 || C <= 0 || IH <= 0 || IW <= 0 || OH <= 0 || OW <= 0 || num_candidates <= 0) return MC_ERR_BAD_ARG;
  if ((uintptr_t)map & 15) return MC_ERR_BAD_ARG;
  const size_t need = mc_voting_resample_workspace(B, C, OH, OW, num_candidates);
  if (!ws || ws_bytes < need) return MC_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  if (cudaMemsetAsync(ws, 0, need, st) != cudaSuccess) return MC_ERR_LAUNCH;
  const long planes = (long)B * C;
  const long n_in = planes * IH * IW, n_out = planes * OH * OW;
  vote_count_kernel<<<vote_grid(n_in, 256), 256, 0, st>>>(labels, map, planes, C, IH, IW, OH, OW, num_candidates,
                                                         (int*)ws);
  vote_pick_kernel<<<vote_grid(n_out, 256), 256, 0, st>>>((const int*)ws, n_out, num_candidates, out);
  MC_COUNT(2);
  MC_CHECK_LAUNCH();
  return MC_OK;
}
