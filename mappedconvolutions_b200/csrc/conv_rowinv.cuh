// Mapped convolution for sample maps that are translation invariant along image rows - the maps
// of spherical kernels on equirectangular images (gnomonic, equirectangular, plain grids):
//
//     map[r, x, k] = (x + cx[r, k], cy[r, k])            x positions possibly wrapped into [0, W)
//
// Along a row every tap keeps its fractional position, so its bilinear weights are constants of
// the row and the interpolation can be folded into the weights once per call:
//
//     y[r, x, :] = sum over the row's slots (sy, dx) of  E[r, (sy, dx)] . X[sy, x + dx, :]
//     E[r, (sy, dx)] = sum over the (tap k, corner c) that read (sy, x + dx) of  w[r, k, c] * W[:, :, k]
//
// No interpolation is left in the data path.  The operand of the GEMM is a plain run of source
// pixels: a WINDOW of 128 * T + span consecutive pixels of source row sy is copied once into
// shared memory (TMA boxes, 128-byte swizzle) and serves every slot of that source row and every
// one of the T 128-pixel tiles of the unit - a slot only moves the START ADDRESS of the tcgen05
// operand by dx rows.  The reference interpolates every tap of every pixel
// (include/nn/common/mapped_im2col.h:12-42) and multiplies a K-times inflated column buffer
// (src/nn/cuda/mapped_convolution_layer.cu:39-70).
//
//   forward          result rows = rows of the map grid, source = x, E = sum w W_k
//   input gradient   result rows = rows of the sampled image, source = grad_output, the plan
//                    transposed (slot (r, -dx) for every forward slot (sy, dx) of row r) and E^T
//   weight gradient  per slot gE = sum over pixels of gy (x) X-window (conv_rowinv_wgrad kernel),
//                    then gw_k = sum over slots of w * gE
//
// Forward and input gradient work on PAIRS of adjacent result rows: the two rows read largely the
// same source rows, so one window serves both, and their effective weights sit side by side in an
// N = 128 MMA operand (a slot only one row reads has zeros for the other: 26.5 slots per pair against
// 2 x 20.8 at 512 x 1024 with a 3 x 3 gnomonic kernel).  Why N = 128: an M128 x N x K16 MMA takes
// max(48, N / 2) cycles (below N = 96 the 128 B/clk shared-memory fetch of A + B binds), and the ONE
// thread that issues needs ~45 cycles per instruction plus whatever else it executes - measured with
// the loops below stripped to bare issue.  So N = 64 MMAs can never run faster than their issuing
// thread; N = 128 halves the instructions per flop, and two threads (warps 0 and 7, two tiles of a
// unit each) issue side by side.
//
// A row's plan is the NOMINAL behaviour of its taps.  A few pixels deviate from it: a bilinear map
// whose positions are wrapped into [0, W) has, per tap and row, one pixel whose left corner is
// column W - 1 and whose right corner (column W) does not exist and reads as zero
// (include/core/interpolation.h:125-154), where a wrapped window reads column 0; and where a
// position sits within rounding of an integer the float32 map entry of single pixels can fall on
// the other side of it (or on W itself).  The planner therefore decodes EVERY map entry exactly as
// the general kernels do, compares it with the row's nominal corners and emits a list of
// corrections (result pixel, source pixel, tap, weight difference) for the pixels that differ by
// more than 1e-3 in a weight; the fix-up kernels below apply them after the main kernels.
//
// This header is part of conv_tc.cu's translation unit (one device status word, shared helpers).
#pragma once

#include <cuda.h>  // CUtensorMap (types only: the driver entry point is looked up at run time)

#include <algorithm>
#include <cmath>
#include <cstring>
#include <vector>

namespace mc {
namespace tc {

constexpr int RI_SPAN = 32;  // shifts 0..RI_SPAN of one source row share a window
constexpr int RI_MAX_WIN_PER_ROW = 64;
constexpr int RI_MAX_SLOT_PER_ROW = 128;
constexpr double RI_TOL = 1e-3;  // pixels: largest deviation from exact translation invariance
constexpr int RI_MODE_CLIP = 0, RI_MODE_WRAP = 1;
constexpr int RI_PLAN_MAGIC = 0x52495032;
constexpr int RI_WG_PAIRS = 8;  // M = 128 accumulators (two slots each) a weight-gradient unit holds

// ---- plan layout (a flat int32 buffer, identical on host and device) -------------------------------
struct RiDir {
  int rows, nwin, nslot, ncon, nskip, ngroup;
  int max_win_per_row, max_slot_per_row;
  // int offsets from the start of the plan
  int off_row;    // (rows + 1) first window of every result row
  int off_win;    // nwin x 4: source row, dx0 (first shift), first slot, nslots | span << 8 | mode << 16
  int off_slot;   // nslot: shift inside the window
  int off_coff;   // (nslot + 1) contributions of every slot
  int off_ctap;   // ncon taps
  int off_cw;     // ncon weights (float bits)
  int off_skip;   // nskip x 6 corrections: result row, result column, source row, source column, tap,
                  // weight difference (float bits; exact minus nominal)
  int off_group;  // (ngroup + 1): runs of corrections that apply to the same result pixel
  int nwgunit;    // weight-gradient work units: runs of windows of a row whose slot pairs fit TMEM
  int off_wgunit; // nwgunit x 4: row, first window, windows, first slot
};
struct RiHeader {
  int magic, total_ints;
  int OH, OW, IH, IW, K, interp;
  RiDir dir[2];   // 0: forward (result = map grid), 1: adjoint (result = sampled image)
  RiDir pair[2];  // the same two directions planned for PAIRS of adjacent result rows (2p, 2p + 1):
                  // rows = pairs; a slot is a (source row, shift) either row of the pair reads and has
                  // two contribution lists, off_coff[2 s] for row 2p and off_coff[2 s + 1] for row
                  // 2p + 1 (off_coff holds 2 nslot + 1 entries); no corrections, no weight-gradient units
};

// ---- analysis: is the map row invariant? --------------------------------------------------------------
// One block per row of the map grid.  out[(r * K + k) * 3 + {0, 1, 2}] = cx, cy, kind; kind is a
// bit mask: 1 = the x positions are x + cx as they stand, 2 = they are (x + cx) wrapped into [0, W)
// (a tap can be both, e.g. the centre tap of a kernel); 0 = not invariant.
__global__ void rowinv_analyse_kernel(const float* __restrict__ map, int OH, int OW, int K, int IW,
                                      double* __restrict__ out) {
  const int r = blockIdx.x;
  __shared__ double s_sum[2][32];
  __shared__ int s_bad[3][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  for (int k = 0; k < K; ++k) {
    const float2 mref = __ldg(reinterpret_cast<const float2*>(map) + ((long)r * OW + OW / 2) * K + k);
    const double ref = (double)mref.x - (double)(OW / 2), cy0 = (double)mref.y;
    double sum_d = 0.0, sum_y = 0.0;
    int bad_plain = 0, bad_wrap = 0, bad_y = 0;
    for (int x = threadIdx.x; x < OW; x += blockDim.x) {
      const float2 m = __ldg(reinterpret_cast<const float2*>(map) + ((long)r * OW + x) * K + k);
      const double d = (double)m.x - (double)x - ref;
      if (!(fabs(d) <= RI_TOL)) bad_plain = 1;
      double dw = fmod(d + IW * 0.5, (double)IW);
      if (dw < 0) dw += IW;
      dw -= IW * 0.5;
      if (!(fabs(dw) <= RI_TOL) || !(m.x >= 0.f && m.x < (float)IW)) bad_wrap = 1;
      if (!(fabs((double)m.y - cy0) <= RI_TOL)) bad_y = 1;
      sum_d += isfinite(dw) ? dw : 0.0;
      sum_y += isfinite(m.y) ? (double)m.y : 0.0;
    }
    for (int o = 16; o > 0; o >>= 1) {
      sum_d += __shfl_xor_sync(0xffffffffu, sum_d, o);
      sum_y += __shfl_xor_sync(0xffffffffu, sum_y, o);
      bad_plain |= __shfl_xor_sync(0xffffffffu, bad_plain, o);
      bad_wrap |= __shfl_xor_sync(0xffffffffu, bad_wrap, o);
      bad_y |= __shfl_xor_sync(0xffffffffu, bad_y, o);
    }
    __syncthreads();
    if (lane == 0) {
      s_sum[0][warp] = sum_d; s_sum[1][warp] = sum_y;
      s_bad[0][warp] = bad_plain; s_bad[1][warp] = bad_wrap; s_bad[2][warp] = bad_y;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      double sd = 0, sy = 0;
      int bp = 0, bw = 0, by = 0;
      for (int i = 0; i < nwarp; ++i) {
        sd += s_sum[0][i]; sy += s_sum[1][i];
        bp |= s_bad[0][i]; bw |= s_bad[1][i]; by |= s_bad[2][i];
      }
      int kind = 0;
      if (!by) kind = (!bp ? 1 : 0) | ((!bw && OW == IW) ? 2 : 0);
      double* o = out + ((long)r * K + k) * 3;
      o[0] = ref + sd / OW;
      o[1] = sy / OW;
      o[2] = (double)kind;
    }
  }
}

// ---- host-side planner ------------------------------------------------------------------------------------
struct RiCon {  // one (tap, corner) contribution
  int res_row, src_row, dx, mode, tap;
  float w;
};

struct RiFix {  // one correction: result pixel += dw * W_tap . source pixel
  int res_row, res_col, src_row, src_col, tap;
  float dw;
};

static void ri_emit_dir(std::vector<RiCon>& cons, std::vector<RiFix>& fixes, int rows,
                        std::vector<int>& plan, RiDir& d, bool& ok) {
  std::stable_sort(cons.begin(), cons.end(), [](const RiCon& a, const RiCon& b) {
    if (a.res_row != b.res_row) return a.res_row < b.res_row;
    if (a.mode != b.mode) return a.mode < b.mode;
    if (a.src_row != b.src_row) return a.src_row < b.src_row;
    if (a.dx != b.dx) return a.dx < b.dx;
    return a.tap < b.tap;
  });
  std::vector<int> row_off(rows + 1, 0), win, slot, coff, ctap, cw;
  int max_w = 0, max_s = 0;
  size_t i = 0;
  for (int r = 0; r < rows; ++r) {
    row_off[r] = (int)win.size() / 4;
    const int slot0 = (int)slot.size();
    while (i < cons.size() && cons[i].res_row == r) {
      // a new slot; a new window if the source row / mode changes or the shift leaves the span
      const RiCon& c = cons[i];
      bool new_win = win.size() / 4 == (size_t)row_off[r];
      if (!new_win) {
        const int* w = &win[win.size() - 4];
        new_win = w[0] != c.src_row || (w[3] >> 16) != c.mode || c.dx - w[1] > RI_SPAN;
      }
      if (new_win) {
        win.push_back(c.src_row); win.push_back(c.dx); win.push_back((int)slot.size());
        win.push_back(c.mode << 16);
      }
      int* w = &win[win.size() - 4];
      slot.push_back(c.dx - w[1]);
      w[3] = (w[3] & 0xFFFF0000) | ((c.dx - w[1]) << 8) | (((w[3] & 0xFF) + 1) & 0xFF);
      coff.push_back((int)ctap.size());
      size_t j = i;
      while (j < cons.size() && cons[j].res_row == r && cons[j].mode == c.mode &&
             cons[j].src_row == c.src_row && cons[j].dx == c.dx) {
        ctap.push_back(cons[j].tap);
        int bits;
        std::memcpy(&bits, &cons[j].w, 4);
        cw.push_back(bits);
        ++j;
      }
      i = j;
    }
    max_w = std::max(max_w, (int)win.size() / 4 - row_off[r]);
    max_s = std::max(max_s, (int)slot.size() - slot0);
  }
  row_off[rows] = (int)win.size() / 4;
  coff.push_back((int)ctap.size());
  if (max_w > RI_MAX_WIN_PER_ROW || max_s > RI_MAX_SLOT_PER_ROW) ok = false;
  // corrections, grouped by the result pixel they apply to
  std::stable_sort(fixes.begin(), fixes.end(), [](const RiFix& a, const RiFix& b) {
    if (a.res_row != b.res_row) return a.res_row < b.res_row;
    return a.res_col < b.res_col;
  });
  std::vector<int> skip, group;
  for (size_t e = 0; e < fixes.size(); ++e) {
    const RiFix& f = fixes[e];
    if (e == 0 || f.res_row != fixes[e - 1].res_row || f.res_col != fixes[e - 1].res_col)
      group.push_back((int)e);
    int bits;
    std::memcpy(&bits, &f.dw, 4);
    const int ent[6] = {f.res_row, f.res_col, f.src_row, f.src_col, f.tap, bits};
    skip.insert(skip.end(), ent, ent + 6);
  }
  group.push_back((int)fixes.size());
  d.rows = rows; d.nwin = (int)win.size() / 4; d.nslot = (int)slot.size(); d.ncon = (int)ctap.size();
  d.nskip = (int)fixes.size(); d.ngroup = (int)group.size() - 1;
  d.max_win_per_row = max_w; d.max_slot_per_row = max_s;
  auto put = [&plan](const std::vector<int>& v) {
    const int off = (int)plan.size();
    plan.insert(plan.end(), v.begin(), v.end());
    while (plan.size() % 4) plan.push_back(0);  // every array starts on a 16-byte boundary
    return off;
  };
  d.off_row = put(row_off); d.off_win = put(win); d.off_slot = put(slot); d.off_coff = put(coff);
  d.off_ctap = put(ctap); d.off_cw = put(cw); d.off_skip = put(skip); d.off_group = put(group);
  // weight-gradient units: consecutive windows of a row, as many as give at most RI_WG_PAIRS pairs
  // of slots (the slots of a window are paired up; an odd one out is paired with itself)
  struct WgUnit { int rec[4]; int pairs; };
  std::vector<WgUnit> units;
  for (int r = 0; r < rows; ++r) {
    int w = row_off[r];
    while (w < row_off[r + 1]) {
      int pairs = 0, w1 = w;
      while (w1 < row_off[r + 1]) {
        const int p = ((win[4 * w1 + 3] & 0xFF) + 1) / 2;
        if (w1 > w && pairs + p > RI_WG_PAIRS) break;
        pairs += p;
        ++w1;
      }
      if (pairs > RI_WG_PAIRS) ok = false;  // a single window with more than 16 slots
      units.push_back(WgUnit{{r, w, w1 - w, win[4 * w + 2]}, pairs});
      w = w1;
    }
  }
  // largest first: the kernel deals the units out to its blocks back and forth in this order, which
  // evens out the work of the blocks
  std::stable_sort(units.begin(), units.end(),
                   [](const WgUnit& p, const WgUnit& q) { return p.pairs > q.pairs; });
  std::vector<int> wg;
  for (const WgUnit& u : units) wg.insert(wg.end(), u.rec, u.rec + 4);
  d.nwgunit = (int)wg.size() / 4;
  d.off_wgunit = put(wg);
}

// The plan of one direction for pairs of adjacent result rows.  The forward / input-gradient
// kernel computes both rows of a pair with one MMA (N = 2 x 64 result channels): the rows share
// their windows, and a slot only one of them reads gets zero weights for the other.
static void ri_emit_pairs(std::vector<RiCon> cons, int rows, std::vector<int>& plan, RiDir& d,
                          bool& ok) {
  std::stable_sort(cons.begin(), cons.end(), [](const RiCon& a, const RiCon& b) {
    if ((a.res_row >> 1) != (b.res_row >> 1)) return (a.res_row >> 1) < (b.res_row >> 1);
    if (a.mode != b.mode) return a.mode < b.mode;
    if (a.src_row != b.src_row) return a.src_row < b.src_row;
    if (a.dx != b.dx) return a.dx < b.dx;
    if (a.res_row != b.res_row) return a.res_row < b.res_row;
    return a.tap < b.tap;
  });
  const int pairs = (rows + 1) / 2;
  std::vector<int> row_off(pairs + 1, 0), win, slot, coff, ctap, cw;
  int max_w = 0, max_s = 0;
  size_t i = 0;
  for (int p = 0; p < pairs; ++p) {
    row_off[p] = (int)win.size() / 4;
    const int slot0 = (int)slot.size();
    while (i < cons.size() && (cons[i].res_row >> 1) == p) {
      const RiCon c = cons[i];
      bool new_win = win.size() / 4 == (size_t)row_off[p];
      if (!new_win) {
        const int* w = &win[win.size() - 4];
        new_win = w[0] != c.src_row || (w[3] >> 16) != c.mode || c.dx - w[1] > RI_SPAN;
      }
      if (new_win) {
        win.push_back(c.src_row); win.push_back(c.dx); win.push_back((int)slot.size());
        win.push_back(c.mode << 16);
      }
      int* w = &win[win.size() - 4];
      slot.push_back(c.dx - w[1]);
      w[3] = (w[3] & 0xFFFF0000) | ((c.dx - w[1]) << 8) | (((w[3] & 0xFF) + 1) & 0xFF);
      for (int sub = 0; sub < 2; ++sub) {
        coff.push_back((int)ctap.size());
        while (i < cons.size() && cons[i].res_row == 2 * p + sub && cons[i].mode == c.mode &&
               cons[i].src_row == c.src_row && cons[i].dx == c.dx) {
          ctap.push_back(cons[i].tap);
          int bits;
          std::memcpy(&bits, &cons[i].w, 4);
          cw.push_back(bits);
          ++i;
        }
      }
    }
    max_w = std::max(max_w, (int)win.size() / 4 - row_off[p]);
    max_s = std::max(max_s, (int)slot.size() - slot0);
  }
  row_off[pairs] = (int)win.size() / 4;
  coff.push_back((int)ctap.size());
  if (max_w > RI_MAX_WIN_PER_ROW || max_s > RI_MAX_SLOT_PER_ROW) ok = false;
  std::memset(&d, 0, sizeof(d));
  d.rows = pairs; d.nwin = (int)win.size() / 4; d.nslot = (int)slot.size(); d.ncon = (int)ctap.size();
  d.max_win_per_row = max_w; d.max_slot_per_row = max_s;
  auto put = [&plan](const std::vector<int>& v) {
    const int off = (int)plan.size();
    plan.insert(plan.end(), v.begin(), v.end());
    while (plan.size() % 4) plan.push_back(0);
    return off;
  };
  d.off_row = put(row_off); d.off_win = put(win); d.off_slot = put(slot); d.off_coff = put(coff);
  d.off_ctap = put(ctap); d.off_cw = put(cw);
  d.off_skip = d.off_group = d.off_wgunit = (int)plan.size();
}

// One decoded map entry on the host: the (up to four) source pixels and weights the general kernels
// use for it (common.cuh decode_tap; include/core/interpolation.h:125-154, :183-210).
struct RiCorner {
  int row, col;
  float w;
};
static int ri_decode_exact(float x, float y, int H, int W, int interp, RiCorner (&out)[4]) {
  const float xf = floorf(x), yf = floorf(y);
  if (!std::isfinite(xf) || !std::isfinite(yf)) return 0;
  const float Bx = (xf + 1.f) - x, Cx = x - xf, Ay = (yf + 1.f) - y, Dy = y - yf;
  const float w4[4] = {Ay * Bx, Ay * Cx, Dy * Bx, Dy * Cx};
  int n = 0;
  for (int c = 0; c < 4; ++c) {
    const int oy = c >> 1, ox = c & 1;
    const double ry = (double)yf + oy, rx = (double)xf + ox;
    if (ry < 0 || ry > H - 1 || w4[c] == 0.f) continue;
    long col;
    if (interp == 1) {
      if (rx < 0 || rx > W - 1) continue;
      col = (long)rx;
    } else {
      if (!(fabs(rx) < 1e18)) continue;
      col = (((long)rx % W) + W) % W;
    }
    out[n].row = (int)ry; out[n].col = (int)col; out[n].w = w4[c];
    ++n;
  }
  return n;
}

// analysis: (OH, K, 3) doubles from rowinv_analyse_kernel; map: the (OH, OW, K, 2) sample map; both
// on the host.  Returns the plan as int32s (empty if the map does not qualify).
static std::vector<int> rowinv_assemble(const mc_desc* d, const double* analysis, const float* map) {
  const int OH = d->OH, OW = d->OW, IH = d->IH, IW = d->IW, K = d->K;
  std::vector<RiCon> fwd, adj;
  std::vector<RiFix> ffix, afix;
  // One addressing mode for the whole map where possible (windows are shared by the taps of a source
  // row only if they agree on it): wrap if some tap needs it, clip otherwise.  Single pixels where
  // the two differ are caught by the per-pixel comparison below.
  bool prefer_wrap = d->interp == 2;
  for (long i = 0; i < (long)OH * K; ++i) prefer_wrap |= (int)analysis[i * 3 + 2] == 2;
  for (int r = 0; r < OH; ++r) {
    for (int k = 0; k < K; ++k) {
      const double* a = analysis + ((long)r * K + k) * 3;
      const int kind = (int)a[2];
      if (kind == 0 || !std::isfinite(a[0]) || !std::isfinite(a[1]) || fabs(a[0]) > 1e7 ||
          fabs(a[1]) > 1e7)
        return {};
      // nominal corner weights in float32, from the row's position, with the reference's formulas
      // (include/core/interpolation.h:17-33: A = y2 - y, B = x2 - x, C = x - x1, D = y - y1)
      const float px = (float)a[0], py = (float)a[1];
      const float xf = floorf(px), yf = floorf(py);
      const float Bx = (xf + 1.f) - px, Cx = px - xf, Ay = (yf + 1.f) - py, Dy = py - yf;
      const float w4[4] = {Ay * Bx, Ay * Cx, Dy * Bx, Dy * Cx};
      const int mode = (d->interp == 2 || kind == 2 || (prefer_wrap && (kind & 2))) ? RI_MODE_WRAP
                                                                                     : RI_MODE_CLIP;
      RiCorner nom[4];  // col holds dx here
      int nn = 0;
      for (int c = 0; c < 4; ++c) {
        const int oy = c >> 1, ox = c & 1;
        const int sy = (int)yf + oy;
        if (sy < 0 || sy > IH - 1 || w4[c] == 0.f) continue;
        RiCon con;
        con.res_row = r; con.src_row = sy; con.dx = (int)xf + ox; con.mode = mode; con.tap = k;
        con.w = w4[c];
        fwd.push_back(con);
        RiCon t = con;
        t.res_row = sy; t.src_row = r; t.dx = -con.dx;
        adj.push_back(t);
        nom[nn].row = sy; nom[nn].col = con.dx; nom[nn].w = w4[c];
        ++nn;
      }
      // every pixel of the row against the nominal corners
      for (int x = 0; x < OW; ++x) {
        const float* m = map + (((long)r * OW + x) * K + k) * 2;
        RiCorner ex[4];
        const int ne = ri_decode_exact(m[0], m[1], IH, IW, d->interp, ex);
        RiCorner diff[8];
        int nd = 0;
        float worst = 0.f;
        for (int i = 0; i < ne; ++i) diff[nd++] = ex[i];
        for (int i = 0; i < nn; ++i) {
          long col = (long)x + nom[i].col;
          if (mode == RI_MODE_WRAP) col = ((col % IW) + IW) % IW;
          else if (col < 0 || col > IW - 1) continue;
          int j = 0;
          while (j < nd && !(diff[j].row == nom[i].row && diff[j].col == (int)col)) ++j;
          if (j == nd) { diff[nd].row = nom[i].row; diff[nd].col = (int)col; diff[nd].w = 0.f; ++nd; }
          diff[j].w -= nom[i].w;
        }
        for (int i = 0; i < nd; ++i) worst = std::max(worst, fabsf(diff[i].w));
        if (!(worst > 1e-3f)) continue;
        for (int i = 0; i < nd; ++i) {
          if (diff[i].w == 0.f) continue;
          ffix.push_back({r, x, diff[i].row, diff[i].col, k, diff[i].w});
          afix.push_back({diff[i].row, diff[i].col, r, x, k, diff[i].w});
        }
      }
    }
  }
  if (ffix.size() > (size_t)OH * 64) return {};  // more than a fringe: not what this path is for
  RiHeader h;
  std::memset(&h, 0, sizeof(h));
  h.magic = RI_PLAN_MAGIC;
  h.OH = OH; h.OW = OW; h.IH = IH; h.IW = IW; h.K = K; h.interp = d->interp;
  std::vector<int> plan((sizeof(RiHeader) + 3) / 4, 0);
  while (plan.size() % 4) plan.push_back(0);
  bool ok = true;
  ri_emit_pairs(fwd, OH, plan, h.pair[0], ok);
  ri_emit_pairs(adj, IH, plan, h.pair[1], ok);
  ri_emit_dir(fwd, ffix, OH, plan, h.dir[0], ok);
  ri_emit_dir(adj, afix, IH, plan, h.dir[1], ok);
  if (!ok) return {};
  h.total_ints = (int)plan.size();
  std::memcpy(plan.data(), &h, sizeof(h));
  return plan;
}

// ---- effective weights -------------------------------------------------------------------------------
// Wk[k][n][c]: the layer's weights with the tap outermost, n = result channel, c = source channel
// (transpose = 0: W[n, c, k]; transpose = 1: W[c, n, k]), so that the kernels below read whole
// 128-byte rows.
__global__ void rowinv_wk_kernel(const bf16* __restrict__ w, bf16* __restrict__ wk, int NR, int K,
                                 int Cin, int transpose) {
  const int total = K * NR * 64;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int c = i & 63, n = (i >> 6) % NR, k = i / (64 * NR);
    const int co = transpose ? c : n, ci = transpose ? n : c;
    wk[i] = w[((long)co * Cin + ci) * K + k];
  }
}

// E[slot] = sum over the slot's contributions of weight * Wk[tap], in the shared-memory image of a
// K-major MMA operand: NR rows (result channels) of 64 source channels, 128 bytes each, 16-byte
// chunks XOR-swizzled by (row & 7).  One thread per 16-byte chunk.
__global__ void __launch_bounds__(256) rowinv_weights_kernel(const bf16* __restrict__ wk,
                                                             const int* __restrict__ plan, RiDir d,
                                                             uint4* __restrict__ E, int NR) {
  const int s = blockIdx.x;
  const int b0 = __ldg(plan + d.off_coff + s), b1 = __ldg(plan + d.off_coff + s + 1);
  for (int i = threadIdx.x; i < NR * 8; i += 256) {
    const int n = i >> 3, ch = i & 7;
    float2 acc[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[j] = make_float2(0.f, 0.f);
    for (int e = b0; e < b1; ++e) {
      const float we = __int_as_float(__ldg(plan + d.off_cw + e));
      const uint4 v = ldg16(wk + ((long)__ldg(plan + d.off_ctap + e) * NR + n) * 64 + ch * 8);
      const float2 w2 = make_float2(we, we);
      ffma2_bf16x2(acc[0], w2, v.x);
      ffma2_bf16x2(acc[1], w2, v.y);
      ffma2_bf16x2(acc[2], w2, v.z);
      ffma2_bf16x2(acc[3], w2, v.w);
    }
    E[(size_t)s * NR * 8 + n * 8 + (ch ^ (n & 7))] = pack_row(acc);
  }
}

// ---- tensor map of the gathered tensor ---------------------------------------------------------------
// The windows of the forward / input-gradient kernel are fetched by the TMA unit: boxes of RI_BOX
// consecutive pixels of one image row, 64 channels each, written in the 128-byte swizzle the MMA
// operand wants.  (B * H, W, 64) view: a box that sticks out of the row's W pixels is filled with
// zeros there - exactly what a clipped window needs; the one box of a wrapped window that contains
// the seam is copied by cp.async instead.  Against cp.async for everything this takes the copies
// off the load/store path that the accumulator read-out's shared-memory traffic shares with them
// (measured: 50-60 cycles per shared-memory instruction of the read-out while cp.async bursts ran).
constexpr int RI_BOX = 32;
static bool ri_make_tensor_map(CUtensorMap* tm, const void* base, long rows, int W) {
  static std::atomic<void*> fn{nullptr};
  void* f = fn.load(std::memory_order_acquire);
  if (!f) {
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess || !f)
      return false;
    fn.store(f, std::memory_order_release);
  }
  using Encode = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                              CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                              CUtensorMapFloatOOBfill);
  const cuuint64_t dims[3] = {64, (cuuint64_t)W, (cuuint64_t)rows};
  const cuuint64_t strides[2] = {128, (cuuint64_t)W * 128};  // bytes, dimensions 1 and 2
  const cuuint32_t box[3] = {64, RI_BOX, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  return ((Encode)f)(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box,
                     estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
// One box: pixels [col, col + RI_BOX) of row `row` (col may be negative or reach past the row: zeros).
// The innermost coordinate (channel) is 0, as the 16-byte rule for it asks.
__device__ __forceinline__ void tma_load_box(uint32_t dst_smem, const CUtensorMap* tm, int col, int row,
                                             uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      :
      : "r"(dst_smem), "l"((uint64_t)tm), "r"(0), "r"(col), "r"(row), "r"(bar)
      : "memory");
}

// ---- main kernel: forward / input gradient ---------------------------------------------------------
struct RowInvArgs {
  const bf16* src;   // (B, SH, SW, 64) channels-last
  bf16* out;         // (B, RH, RW, NOUT)
  const bf16* bias;  // NOUT or null
  const int* plan;
  RiDir d;
  const uint4* E;  // [slot][NOUT x 128 B]
  int B, SH, SW, RH, RW;
  int tpu;         // 128-pixel tiles per unit
  int upr;         // units per (row, image): RW / (128 * tpu)
  long units;      // RH * B * upr
};

__device__ __forceinline__ void ri_unit(const RowInvArgs& a, long u, int& r, int& b, int& x0) {
  const int per_row = a.B * a.upr;
  r = (int)(u / per_row);
  const int rem = (int)(u - (long)r * per_row);
  b = rem / a.upr;
  x0 = (rem - b * a.upr) * a.tpu * TILE_M;
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

constexpr int RI_WIN_STAGES = 2;
// Warps of the forward / input-gradient kernel: 0 and 7 issue the MMAs, 1-4 and 20-23 read the accumulators
// out (each set two of a unit's four tiles; a warp reaches the 32 TMEM lanes given by its index
// modulo 4), 5 streams the effective weights, 6 writes the MMA thread's commands, 8 and 9 fetch
// windows (one warp per stage; 10-19 have no role).
constexpr int RI_LOADER_WARPS = 12;  // warps between the two read-out sets
constexpr int RI_ISSUERS = 2, RI_ISSUER2_WARP = FIRST_DEC_WARP + 2;
constexpr int RI_EPI2_FIRST = FIRST_PROD_WARP + RI_LOADER_WARPS;
constexpr int RI_EPI_WARPS = 2 * N_EPI_WARPS;
constexpr size_t RI_STAGING_BYTES = (size_t)RI_EPI_WARPS * 2048;
static_assert(RI_EPI2_FIRST % 4 == 0 && RI_EPI2_FIRST + N_EPI_WARPS == TC_THREADS / 32, "warp roles");
// Commands for the MMA thread, one per slot of a unit, written by a helper warp one unit ahead:
// x = low word of the A descriptor of the slot's first tile (window stage + shift);
// y = bit 0: first slot of a window - wait for the window stage (bit 1) in phase (bit 2);
//     bit 3: last slot of a window - hand the stage (bit 1) back afterwards.
constexpr int RI_CMD_SLOTS = RI_MAX_SLOT_PER_ROW + 2;
constexpr size_t RI_CMD_BYTES = (size_t)RI_CMD_SLOTS * 8;

template <int NOUT>
struct RiCfg {
  // NOUT = 128: two adjacent result rows of 64 channels each side by side in the accumulator (the
  // plan's pair directions); one accumulator set of 4 tiles x 128 columns fills tensor memory, so the
  // read-out of a unit and the MMAs of the next take turns.  NOUT = 64: one row, two sets of 4 x 64.
  static constexpr bool PAIR = NOUT == 128;
  static constexpr int TPU = 4;                                       // 128-pixel tiles per unit
  static constexpr int NACC = 512 / (TPU * NOUT);                     // accumulator sets in TMEM
  static constexpr uint32_t WIN_ROWS = TPU * TILE_M + RI_SPAN;
  static constexpr uint32_t WIN_BYTES = ((WIN_ROWS * 128 + 1023) / 1024) * 1024;
  static constexpr uint32_t E_BYTES = NOUT * 128;
  static constexpr int NE = NOUT == 64 ? 6 : (NOUT == 128 ? 4 : 2);  // E stages
  static constexpr int NBAR = 2 * RI_WIN_STAGES + 2 * NE + 11;
  static constexpr size_t SMEM = 1024 + (size_t)RI_WIN_STAGES * WIN_BYTES + (size_t)NE * E_BYTES +
                                 RI_STAGING_BYTES + NOUT * 4 + NBAR * 8 + 48 + 2 * RI_CMD_BYTES + 16;
};

template <int NOUT>
__global__ void __launch_bounds__(TC_THREADS, 1) conv_rowinv_tc_kernel(const RowInvArgs a,
                                                                       const __grid_constant__ CUtensorMap tmap) {
  using Cfg = RiCfg<NOUT>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* sm = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t win0 = smem_u32(sm);
  const uint32_t e0 = win0 + RI_WIN_STAGES * Cfg::WIN_BYTES;
  const uint32_t stg0 = e0 + Cfg::NE * Cfg::E_BYTES;
  uint8_t* tail = sm + RI_WIN_STAGES * Cfg::WIN_BYTES + Cfg::NE * Cfg::E_BYTES + RI_STAGING_BYTES;
  float* bias_s = (float*)tail;
  uint64_t* bars = (uint64_t*)(bias_s + NOUT);
  uint32_t* misc = (uint32_t*)(bars + Cfg::NBAR);
  volatile int* abort_flag = (volatile int*)(misc + 1);
  uint2* s_cmd = (uint2*)(((uintptr_t)(misc + 4) + 15) & ~(uintptr_t)15);  // two command lists
  volatile int* s_ns = (volatile int*)(misc + 2);                           // and their lengths
  const uint32_t bar0 = smem_u32(bars);
  auto wfull = [&](int s) { return bar0 + 8u * s; };
  auto wempty = [&](int s) { return bar0 + 8u * (RI_WIN_STAGES + s); };
  auto efull = [&](int s) { return bar0 + 8u * (2 * RI_WIN_STAGES + s); };
  auto eempty = [&](int s) { return bar0 + 8u * (2 * RI_WIN_STAGES + Cfg::NE + s); };
  auto tfull = [&](int i) { return bar0 + 8u * (2 * RI_WIN_STAGES + 2 * Cfg::NE + i); };
  auto tempty = [&](int i) { return bar0 + 8u * (2 * RI_WIN_STAGES + 2 * Cfg::NE + 2 + i); };
  const uint32_t drain_bar0 = bar0 + 8u * (2 * RI_WIN_STAGES + 2 * Cfg::NE + 9);
  auto cfull = [&](int i) { return bar0 + 8u * (2 * RI_WIN_STAGES + 2 * Cfg::NE + 5 + i); };
  auto cempty = [&](int i) { return bar0 + 8u * (2 * RI_WIN_STAGES + 2 * Cfg::NE + 7 + i); };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t TMEM_COLS = 512;
  const int* plan = a.plan;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) { mbar_init(cfull(i), 1); mbar_init(cempty(i), RI_ISSUERS); }
    for (int s = 0; s < RI_WIN_STAGES; ++s) { mbar_init(wfull(s), 1); mbar_init(wempty(s), RI_ISSUERS); }
    for (int s = 0; s < Cfg::NE; ++s) { mbar_init(efull(s), 1); mbar_init(eempty(s), RI_ISSUERS); }
    for (int i = 0; i < 2; ++i) { mbar_init(tfull(i), RI_ISSUERS); mbar_init(tempty(i), RI_EPI_WARPS); }
    mbar_init(drain_bar0, 1);
    mbar_init(drain_bar0 + 8u, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  for (int i = threadIdx.x; i < NOUT; i += TC_THREADS)
    bias_s[i] = a.bias ? __bfloat162float(a.bias[i & 63]) : 0.f;
  if (warp == 0) tmem_alloc(smem_u32(misc), TMEM_COLS);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *misc;

  if (warp == 0 || warp == RI_ISSUER2_WARP) {
    // ------------------------------------------------------------------ MMA issuers
    // A thread that issues MMAs spends more time between two of them than the tensor core takes
    // for one, so two threads issue: warp 0 for tiles 0 and 1 of a unit, warp RI_ISSUER2_WARP for
    // tiles 2 and 3 (accumulators of their own, so no order is needed between the two; every
    // hand-over barrier counts one commit from each).  They only walk a list of commands that a
    // helper warp prepares one unit ahead.
    constexpr uint32_t idesc = make_idesc_bf16(TILE_M, NOUT, 0, 0);
    const int issuer = warp == 0 ? 0 : 1;
    const uint32_t drain_bar = drain_bar0 + 8u * issuer;
    constexpr uint32_t DHI = desc_sw128_hi(1024);
    if (lane == 0) {
      const uint32_t blo0 = desc_sw128_lo(e0, 16);
      uint32_t it = 0, se = 0, pe = 0, blo = blo0;
      bool ok = true;
      for (long u = blockIdx.x; u < a.units && ok; u += gridDim.x, ++it) {
        const uint32_t cb = it & 1, cph = (it >> 1) & 1;
        ok = mbar_wait_spin(cfull(cb), cph, abort_flag, 0x80);
        const uint2* cmd = s_cmd + cb * RI_CMD_SLOTS;
        const int ns = s_ns[cb];
        const uint32_t acc = Cfg::NACC == 2 ? cb : 0u, aph = Cfg::NACC == 2 ? cph : cb;
        ok = ok && mbar_wait_spin(tempty(acc), aph ^ 1, abort_flag, 0x81);
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + acc * (Cfg::TPU * NOUT) + issuer * (Cfg::TPU / 2) * NOUT;
        const uint32_t aoff = issuer * (Cfg::TPU / 2) * (TILE_M * 128 / 16);
        uint32_t accum = 0;  // the first slot of a unit overwrites the accumulators
        uint2 nxt = cmd[0];
        for (int i = 0; i < ns && ok; ++i) {
          const uint2 cur = nxt;
          nxt = cmd[i + 1];  // (the list has a spare entry)
          const uint32_t stage = (cur.y >> 1) & 1;
          if (cur.y & 1) ok = mbar_wait_spin(wfull(stage), (cur.y >> 2) & 1, abort_flag, 0x82);
          ok = ok && mbar_wait_spin(efull(se), pe, abort_flag, 0x83);
          if (!ok) break;
          tc_fence_after_sync();
#pragma unroll
          for (int t = 0; t < Cfg::TPU / 2; ++t)
#pragma unroll
            for (int j = 0; j < 4; ++j)
              mma_bf16_ss_lo(tmem_d + t * NOUT, cur.x + aoff + t * (TILE_M * 128 / 16) + 2 * j, DHI, blo + 2 * j,
                             DHI, idesc, j ? 1u : accum);
          accum = 1;
          mma_commit(eempty(se));
          blo += Cfg::E_BYTES / 16;
          if (++se == (uint32_t)Cfg::NE) { se = 0; pe ^= 1; blo = blo0; }
          if (cur.y & 8) mma_commit(wempty(stage));
        }
        if (ok) {
          mma_commit(tfull(acc));
          mbar_arrive(cempty(cb));
        }
      }
    }
    if (lane == 0) {
      mma_commit(drain_bar);
      mbar_wait_spin(drain_bar, 0, abort_flag, 0x84);
    }
    __syncwarp();
  } else if (warp <= N_EPI_WARPS || warp >= RI_EPI2_FIRST) {
    // ------------------------------------------------------------------ epilogue
    // (the same accumulator read-out as conv_gemm_tc_kernel: TMEM -> registers -> + bias -> bf16 ->
    // a 32 x 64-byte block turned around in shared memory -> stores of 8 rows x 64 bytes)
    // Two sets of four warps: the first reads tiles 0 and 1 of a unit, the second tiles 2 and 3.
    const int q = warp & 3;
    const int eset = warp >= RI_EPI2_FIRST ? 1 : 0;
    const uint32_t stg = stg0 + (uint32_t)(eset ? N_EPI_WARPS + warp - RI_EPI2_FIRST : warp - 1) * 2048u;
    const uint32_t wr_row = stg + lane * 64, wr_x = (lane >> 1) & 3;
    uint32_t rd_addr[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int row = 8 * i + (lane >> 2);
      rd_addr[i] = stg + row * 64 + (((lane & 3) ^ ((row >> 1) & 3)) << 4);
    }
    uint32_t it = 0;
    for (long u = blockIdx.x; u < a.units; u += gridDim.x, ++it) {
      int r, b, x0;
      ri_unit(a, u, r, b, x0);
      const uint32_t acc = Cfg::NACC == 2 ? (it & 1) : 0u, aph = Cfg::NACC == 2 ? ((it >> 1) & 1) : (it & 1);
      const bool empty_row = __ldg(plan + a.d.off_row + r) == __ldg(plan + a.d.off_row + r + 1);
      {
        int okt = 1;
        if (lane == 0) okt = mbar_wait_spin(tfull(acc), aph, abort_flag, 0x85) ? 1 : 0;
        okt = __shfl_sync(0xffffffffu, okt, 0);
        if (!okt) break;
      }
      tc_fence_after_sync();
#pragma unroll
      for (int tt = 0; tt < Cfg::TPU / 2; ++tt) {
        const int t = eset * (Cfg::TPU / 2) + tt;
        bf16* orow[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const long gp = ((long)b * a.RH + (Cfg::PAIR ? 2 * r : r)) * a.RW + x0 + t * TILE_M + q * 32 + 8 * i +
                          (lane >> 2);
          orow[i] = a.out + gp * 64 + (lane & 3) * 8;
        }
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + acc * (Cfg::TPU * NOUT) + t * NOUT;
#pragma unroll
        for (int cc = 0; cc < NOUT / 32; ++cc) {
          uint32_t v[32];
          tmem_ld_32x32(taddr + cc * 32, v);
          tmem_ld_wait();
          if (tt == Cfg::TPU / 2 - 1 && cc == NOUT / 32 - 1) {
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty(acc));
          }
          if (empty_row) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = 0u;
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 o;
            const float* bs = bias_s + (cc & 1) * 32 + j * 8;
            o.x = pack_bf16x2(__uint_as_float(v[j * 8 + 0]) + bs[0], __uint_as_float(v[j * 8 + 1]) + bs[1]);
            o.y = pack_bf16x2(__uint_as_float(v[j * 8 + 2]) + bs[2], __uint_as_float(v[j * 8 + 3]) + bs[3]);
            o.z = pack_bf16x2(__uint_as_float(v[j * 8 + 4]) + bs[4], __uint_as_float(v[j * 8 + 5]) + bs[5]);
            o.w = pack_bf16x2(__uint_as_float(v[j * 8 + 6]) + bs[6], __uint_as_float(v[j * 8 + 7]) + bs[7]);
            sts16(wr_row + ((j ^ wr_x) << 4), o);
          }
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 o;
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(o.x), "=r"(o.y), "=r"(o.z), "=r"(o.w)
                         : "r"(rd_addr[i]));
            // (a pair's second row sits 64 accumulator columns and one image row further on)
            if (!Cfg::PAIR || cc < 2 || 2 * r + 1 < a.RH)
              *reinterpret_cast<uint4*>(orow[i] + (cc & 1) * 32 + (Cfg::PAIR && cc >= 2 ? (long)a.RW * 64 : 0L)) = o;
          }
          __syncwarp();
        }
      }
    }
  } else if (warp == FIRST_DEC_WARP) {
    // ------------------------------------------------------------------ E streamer
    if (lane == 0) {
      uint32_t se = 0, pe = 0;
      bool ok = true;
      for (long u = blockIdx.x; u < a.units && ok; u += gridDim.x) {
        int r, b, x0;
        ri_unit(a, u, r, b, x0);
        const int w0 = __ldg(plan + a.d.off_row + r), w1 = __ldg(plan + a.d.off_row + r + 1);
        if (w1 == w0) continue;
        const int4 wa = __ldg(reinterpret_cast<const int4*>(plan + a.d.off_win) + w0);
        const int4 wb = __ldg(reinterpret_cast<const int4*>(plan + a.d.off_win) + w1 - 1);
        const int s0 = wa.z, s1 = wb.z + (wb.w & 0xFF);
        for (int s = s0; s < s1; ++s) {
          ok = mbar_wait_spin(eempty(se), pe ^ 1, abort_flag, 0x86);
          if (!ok) break;
          mbar_expect_tx(efull(se), Cfg::E_BYTES);
          bulk_g2s(e0 + se * Cfg::E_BYTES, a.E + (size_t)s * (Cfg::E_BYTES / 16), Cfg::E_BYTES, efull(se));
          if (++se == (uint32_t)Cfg::NE) { se = 0; pe ^= 1; }
        }
      }
    }
  } else if (warp == FIRST_DEC_WARP + 1) {
    // ------------------------------------------------------------------ command writer
    // Turns the plan records of the block's next unit into the MMA thread's command list (lane =
    // window): descriptor words, which window stage a slot reads and when that stage changes hands.
    uint32_t it = 0, nw = 0;
    for (long u = blockIdx.x; u < a.units; u += gridDim.x, ++it) {
      int r, b, x0;
      ri_unit(a, u, r, b, x0);
      const uint32_t cb = it & 1, cph = (it >> 1) & 1;
      const int w0 = __ldg(plan + a.d.off_row + r), w1 = __ldg(plan + a.d.off_row + r + 1);
      const int sfirst = w1 > w0 ? __ldg(plan + a.d.off_win + 4 * w0 + 2) : 0;
      int okw = 1;
      if (lane == 0) okw = mbar_wait(cempty(cb), cph ^ 1, abort_flag, 0x88, 64) ? 1 : 0;
      okw = __shfl_sync(0xffffffffu, okw, 0);
      if (!okw) break;
      uint2* cmd = s_cmd + cb * RI_CMD_SLOTS;
      if (lane == 0 && w1 == w0) s_ns[cb] = 0;
      for (int w = w0 + lane; w < w1; w += 32) {
        const int4 wr = __ldg(reinterpret_cast<const int4*>(plan + a.d.off_win) + w);
        const int nsl = wr.w & 0xFF;
        const uint32_t nwg = nw + (uint32_t)(w - w0);
        const uint32_t stage = nwg % RI_WIN_STAGES, ph = (nwg / RI_WIN_STAGES) & 1;
        const uint32_t wlo = desc_sw128_lo(win0 + stage * Cfg::WIN_BYTES, 16);
        for (int sl = 0; sl < nsl; ++sl) {
          const uint32_t sh = (uint32_t)__ldg(plan + a.d.off_slot + wr.z + sl);
          const uint32_t fl = (stage << 1) | (sl == 0 ? (1u | (ph << 2)) : 0u) | (sl == nsl - 1 ? 8u : 0u);
          cmd[wr.z - sfirst + sl] = make_uint2(wlo + sh * 8u, fl);
        }
        if (w == w1 - 1) s_ns[cb] = wr.z + nsl - sfirst;
      }
      nw += (uint32_t)(w1 - w0);
      __syncwarp();
      if (lane == 0) mbar_arrive(cfull(cb));
    }
  } else if (warp >= FIRST_PROD_WARP && warp < RI_EPI2_FIRST) {
    // ------------------------------------------------------------------ window loaders
    // One warp per window stage (warp t copies the windows t, t + 2, ... of the block's window
    // sequence into stage t: a stage is always filled by the same warp, so a parity wait on its
    // barrier is unambiguous).  Lane 0 issues one TMA box per RI_BOX pixels; the box of a wrapped
    // window that contains the seam is copied by the warp with cp.async.  The stage's barrier gets
    // ONE arrival - after the warp's own copies have landed - which also announces the TMA bytes.
    const int team = warp - FIRST_PROD_WARP;
    if (team < RI_WIN_STAGES) {
      uint32_t nw = 0;   // windows of this block so far (every loader warp counts all of them)
      uint32_t mine = 0; // windows this warp has copied
      bool ok = true;
      for (long u = blockIdx.x; u < a.units && ok; u += gridDim.x) {
        int r, b, x0;
        ri_unit(a, u, r, b, x0);
        const int w0 = __ldg(plan + a.d.off_row + r), w1 = __ldg(plan + a.d.off_row + r + 1);
        for (int w = w0; w < w1; ++w, ++nw) {
          if ((int)(nw % RI_WIN_STAGES) != team) continue;
          const int4 wr = __ldg(reinterpret_cast<const int4*>(plan + a.d.off_win) + w);
          const uint32_t ws = team, wph = mine & 1;
          int okw = 1;
          if (lane == 0) okw = mbar_wait_spin(wempty(ws), wph ^ 1, abort_flag, 0x87) ? 1 : 0;
          okw = __shfl_sync(0xffffffffu, okw, 0);
          if (!okw) { ok = false; break; }
          const int span = (wr.w >> 8) & 0xFF, mode = wr.w >> 16;
          const int srow = b * a.SH + wr.x;
          const uint32_t sbase = win0 + ws * Cfg::WIN_BYTES;
          const int nbox = (Cfg::TPU * TILE_M + span + RI_BOX - 1) / RI_BOX;
          int c = x0 + wr.y;  // source column of the window's first pixel
          if (mode == RI_MODE_WRAP) { c %= a.SW; if (c < 0) c += a.SW; }
          uint32_t tma_bytes = 0;
          bool seam = false;
          for (int k = 0; k < nbox; ++k) {
            if (mode == RI_MODE_WRAP && c + RI_BOX > a.SW) {
              // the seam: pixel c + lane, wrapped; lane = row of the box, eight 16-byte chunks each
              int sc = c + lane;
              if (sc >= a.SW) sc -= a.SW;
              const bf16* sp = a.src + ((long)srow * a.SW + sc) * 64;
              const uint32_t dst = sbase + (uint32_t)(k * RI_BOX + lane) * 128u;
#pragma unroll
              for (int ch = 0; ch < 8; ++ch) cp_async16(dst + ((ch ^ (lane & 7)) << 4), sp + ch * 8, 16u);
              seam = true;
            } else {
              if (lane == 0) tma_load_box(sbase + (uint32_t)k * (RI_BOX * 128), &tmap, c, srow, wfull(ws));
              tma_bytes += RI_BOX * 128;
            }
            c += RI_BOX;
            if (mode == RI_MODE_WRAP && c >= a.SW) c -= a.SW;
          }
          if (seam) {
            cp_async_commit();
            cp_async_wait_all();
            fence_proxy_async_smem();
          }
          __syncwarp();
          if (lane == 0) {
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(wfull(ws)), "r"(tma_bytes)
                         : "memory");
          }
          ++mine;
        }
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

// ---- fix-up kernel: the planner's corrections for the pixels that deviate from their row's plan --------
// One block per group of corrections that share a result pixel, for every image of the batch:
// forward : y[b, row, col, n]   += sum_e dw_e sum_c W[n, c, k_e]  x[b, srow_e, scol_e, c]
// adjoint : gx[b, row, col, n]  += sum_e dw_e sum_c W[c, n, k_e] gy[b, srow_e, scol_e, c]
// Per correction that is a 64 x 64 by 64 x 8 product (W_k times the source pixel of eight images):
// 16 warp-level m16n8k16 MMAs (mma.sync - the tensor-core instruction for a product this small; a
// tcgen05 tile would be 128 rows).  Warp w of the block takes the corrections w, w + 4, ... of the
// group; the four partial results are added in a fixed order, so results repeat bit for bit.
constexpr int FIX_WARPS = 4, FIX_IMGS = 8;
__device__ __forceinline__ void mma_m16n8k16_bf16(float (&d)[4], const uint32_t (&a)[4],
                                                  const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__global__ void __launch_bounds__(32 * FIX_WARPS) rowinv_fix_kernel(
    const bf16* __restrict__ src, bf16* __restrict__ res, const bf16* __restrict__ wk,
    const int* __restrict__ plan, RiDir d, int B, int SH, int SW, int RH, int RW, int NR) {
  const int grp = blockIdx.x;
  const int e0 = __ldg(plan + d.off_group + grp), e1 = __ldg(plan + d.off_group + grp + 1);
  if (e0 >= e1) return;
  const int row = __ldg(plan + d.off_skip + 6 * e0), col = __ldg(plan + d.off_skip + 6 * e0 + 1);
  // fragment coordinates of mma.m16n8k16: g = row of A / column of B and D, t = pair of k / of columns
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  __shared__ float red[FIX_WARPS][4][4][32];  // [warp][m-tile][register][lane]
  for (int b0 = 0; b0 < B; b0 += FIX_IMGS) {
    float acc[4][4];
#pragma unroll
    for (int mt = 0; mt < 4; ++mt)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[mt][i] = 0.f;
    for (int e = e0 + warp; e < e1; e += FIX_WARPS) {
      const int* ent = plan + d.off_skip + 6 * e;
      const int srow = __ldg(ent + 2), scol = __ldg(ent + 3), k = __ldg(ent + 4);
      const float dw = __int_as_float(__ldg(ent + 5));
      // B operand (k = source channel, n = image): image b0 + g, channels 16 ks + 2 t (+ 8), two at a time
      const bool img = b0 + g < B;
      const uint32_t* xp = reinterpret_cast<const uint32_t*>(
          src + ((((long)(img ? b0 + g : 0)) * SH + srow) * SW + scol) * 64);
      uint32_t bfr[4][2];
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        bfr[ks][0] = img ? __ldg(xp + ks * 8 + t) : 0u;
        bfr[ks][1] = img ? __ldg(xp + ks * 8 + t + 4) : 0u;
      }
      // A operand: W_k[n][c], n = 16 mt + g (+ 8), c = 16 ks + 2 t (+ 8)
      const uint32_t* wp = reinterpret_cast<const uint32_t*>(wk + (long)k * NR * 64);
#pragma unroll
      for (int mt = 0; mt < 4; ++mt) {
        float tmp[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          uint32_t afr[4];
          afr[0] = __ldg(wp + (mt * 16 + g) * 32 + ks * 8 + t);
          afr[1] = __ldg(wp + (mt * 16 + g + 8) * 32 + ks * 8 + t);
          afr[2] = __ldg(wp + (mt * 16 + g) * 32 + ks * 8 + t + 4);
          afr[3] = __ldg(wp + (mt * 16 + g + 8) * 32 + ks * 8 + t + 4);
          mma_m16n8k16_bf16(tmp, afr, bfr[ks]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[mt][i] = fmaf(dw, tmp[i], acc[mt][i]);
      }
    }
#pragma unroll
    for (int mt = 0; mt < 4; ++mt)
#pragma unroll
      for (int i = 0; i < 4; ++i) red[warp][mt][i][lane] = acc[mt][i];
    __syncthreads();
    {
      // warp w finishes m-tile w: D[n][image], n = 16 w + g (+ 8 for registers 2, 3), image = 2 t (+ 1)
      const int mt = warp;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float sum = red[0][mt][i][lane];
#pragma unroll
        for (int w = 1; w < FIX_WARPS; ++w) sum += red[w][mt][i][lane];
        const int n = mt * 16 + g + (i >> 1) * 8, b = b0 + 2 * t + (i & 1);
        if (b < B) {
          bf16* rp = res + (((long)b * RH + row) * RW + col) * NR + n;
          *rp = __float2bfloat16_rn(__bfloat162float(*rp) + sum);
        }
      }
    }
    __syncthreads();
  }
}

// ---- weight gradient -------------------------------------------------------------------------------
// Per slot s = (row r, source row sy, shift dx):  gE[s][ci][co] = sum_{b, x} X[b, sy, x + dx, ci] gy[b, r, x, co],
// then gw[co, ci, k] = sum_s sum_{contributions (k, w) of s} w gE[s][ci][co]  (rowinv_wgrad_reduce_kernel).
// The X window [pixel][ci] is the MN-major A operand (M = ci); two slots of a window make one M = 128
// operand whose second half starts (shift_B - shift_A) rows after the first (the descriptor's
// leading byte offset); the gy chunk [pixel][co] is the MN-major B operand; the reduction runs
// over pixels, 16 per MMA.  A unit (a run of windows of one row with at most RI_WG_PAIRS pairs, for
// one part of the batch) keeps its pairs' accumulators in tensor memory while it streams the row of
// every image in chunks of 256 pixels.
constexpr int WG_TILES = 2;                                         // 128-pixel tiles per chunk
constexpr uint32_t WG_WIN_ROWS = WG_TILES * TILE_M + RI_SPAN;
constexpr uint32_t WG_WIN_BYTES = ((WG_WIN_ROWS * 128 + 1023) / 1024) * 1024;  // 36 864
constexpr uint32_t WG_GY_BYTES = WG_TILES * TILE_M * 128;           // 32 768
constexpr int WG_NW = 4, WG_NG = 2;                                 // window / gy stages
constexpr int WG_NBAR = 2 * WG_NW + 2 * WG_NG + 4;
constexpr int WG_ISSUERS = 2;  // threads (warps 0 and 5) that issue MMAs, each for every second pair of slots
constexpr size_t WG_SMEM = 1024 + (size_t)WG_NW * WG_WIN_BYTES + (size_t)WG_NG * WG_GY_BYTES +
                           WG_NBAR * 8 + 64 + WG_ISSUERS * (RI_MAX_WIN_PER_ROW * 16 + RI_MAX_SLOT_PER_ROW * 4 + 16);

struct RowInvWgArgs {
  const bf16* x;    // (B, SH, SW, 64)
  const bf16* gy;   // (B, RH, RW, 64)
  float* gE;        // [bsplit][nslot][64 ci][64 co]
  float* gb;        // 64 co, zero before the launch; null: no bias gradient in this launch
  const int* plan;
  RiDir d;
  int B, SH, SW, RH, RW;
  int bsplit;       // parts the batch is cut into (a unit works on one)
  long units;       // nwgunit * bsplit
};

__global__ void __launch_bounds__(TC_THREADS, 1) conv_rowinv_wgrad_kernel(const RowInvWgArgs a,
                                                                         const __grid_constant__ CUtensorMap tmap_x,
                                                                         const __grid_constant__ CUtensorMap tmap_gy) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* sm = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t win0 = smem_u32(sm);
  const uint32_t gy0 = win0 + WG_NW * WG_WIN_BYTES;
  uint64_t* bars = (uint64_t*)(sm + WG_NW * WG_WIN_BYTES + WG_NG * WG_GY_BYTES);
  uint32_t* misc = (uint32_t*)(bars + WG_NBAR);
  volatile int* abort_flag = (volatile int*)(misc + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Two threads issue the MMAs (a single one spends more time between two MMAs than the tensor core
  // takes for one): warp 0 takes the even pairs of slots of a unit, warp FIRST_DEC_WARP the odd ones.
  // Pairs have accumulators of their own, so the two need no order between them; every hand-over
  // barrier counts one commit from each.  Each has its copy of the unit's records.
  const int issuer = warp == 0 ? 0 : 1;
  int4* s_win = (int4*)(((uintptr_t)(misc + 4) + 15) & ~(uintptr_t)15) +
                issuer * (RI_MAX_WIN_PER_ROW + (RI_MAX_SLOT_PER_ROW * 4 + 16) / 16);
  int* s_shift = (int*)(s_win + RI_MAX_WIN_PER_ROW);
  const uint32_t bar0 = smem_u32(bars);
  auto wfull = [&](int s) { return bar0 + 8u * s; };
  auto wempty = [&](int s) { return bar0 + 8u * (WG_NW + s); };
  auto gfull = [&](int s) { return bar0 + 8u * (2 * WG_NW + s); };
  auto gempty = [&](int s) { return bar0 + 8u * (2 * WG_NW + WG_NG + s); };
  const uint32_t accfull = bar0 + 8u * (2 * WG_NW + 2 * WG_NG);
  const uint32_t accempty = accfull + 8u, drain_bar = accfull + 16u + 8u * issuer;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr int TEAMS = 2, TEAM_WARPS = N_PRODUCER_WARPS / TEAMS;
  const int* plan = a.plan;
  const int nchunk = a.RW / (WG_TILES * TILE_M);
  const int bper = (a.B + a.bsplit - 1) / a.bsplit;

  if (threadIdx.x == 0) {
    for (int s = 0; s < WG_NW; ++s) { mbar_init(wfull(s), 1); mbar_init(wempty(s), WG_ISSUERS); }
    for (int s = 0; s < WG_NG; ++s) { mbar_init(gfull(s), 1); mbar_init(gempty(s), WG_ISSUERS + N_EPI_WARPS); }
    mbar_init(accfull, WG_ISSUERS);
    mbar_init(accempty, N_EPI_WARPS);
    mbar_init(accfull + 16u, 1);
    mbar_init(accfull + 24u, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0) tmem_alloc(smem_u32(misc), TMEM_COLS);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *misc;

  // The i-th unit of this block: the units are dealt out back and forth (0 .. G-1, G-1 .. 0, ...)
  // in the planner's order, largest first; -1 after the last one.
  auto unit_at = [&](uint32_t i) -> long {
    const long G = gridDim.x;
    const long u = (long)i * G + ((i & 1) ? G - 1 - (long)blockIdx.x : (long)blockIdx.x);
    return u < a.units ? u : -1;  // a block without a unit in a round is in the last round
  };
  // unit u -> (unit record, batch part)
  auto unit_rec = [&](long u, int& part) {
    const int ui = (int)(u / a.bsplit);
    part = (int)(u - (long)ui * a.bsplit);
    return __ldg(reinterpret_cast<const int4*>(plan + a.d.off_wgunit) + ui);
  };

  if (warp == 0 || warp == FIRST_DEC_WARP) {
    // ------------------------------------------------------------------ MMA issuers
    constexpr uint32_t idesc = make_idesc_bf16(TILE_M, 64, 1, 1);
    constexpr uint32_t DHI = desc_sw128_hi(1024);
    uint32_t it = 0, nw = 0, ng = 0;
    int ok = 1;
    for (long u; ok && (u = unit_at(it)) >= 0; ++it) {
      int part;
      const int4 ur = unit_rec(u, part);
      __syncwarp();
      for (int i = lane; i < ur.z; i += 32)
        s_win[i] = __ldg(reinterpret_cast<const int4*>(plan + a.d.off_win) + ur.y + i);
      __syncwarp();
      // per pair of slots the low word of the A descriptor relative to the window's stage: start row of
      // the first slot (bytes >> 4) and, as leading byte offset, the distance to the second slot
      for (int w = lane; w < ur.z; w += 32) {
        const int4 wr = s_win[w];
        const int nsl = wr.w & 0xFF;
        for (int s = 0; s < nsl; s += 2) {
          const int shA = __ldg(plan + a.d.off_slot + wr.z + s);
          const int shB = s + 1 < nsl ? __ldg(plan + a.d.off_slot + wr.z + s + 1) : shA;
          s_shift[(wr.z - ur.w) + s] = shA * 8 + (((shB - shA) * 8) << 16);
        }
      }
      __syncwarp();
      if (lane == 0) {
        ok = mbar_wait(accempty, (it & 1) ^ 1, abort_flag, 0x91) ? 1 : 0;
        tc_fence_after_sync();
        const int b0 = part * bper, b1 = min(a.B, b0 + bper);
        uint32_t accum = 0;  // the first chunk of a unit overwrites the accumulators
        for (int b = b0; b < b1 && ok; ++b) {
          for (int ch = 0; ch < nchunk && ok; ++ch, ++ng) {
            const uint32_t gs = ng % WG_NG, gph = (ng / WG_NG) & 1;
            ok = mbar_wait(gfull(gs), gph, abort_flag, 0x92) ? 1 : 0;
            const uint32_t blo = desc_sw128_lo(gy0 + gs * WG_GY_BYTES, STAGE_BYTES);
            uint32_t tmem_d = tmem_base;
            int mine = issuer;  // 0: the next pair is this thread's
            for (int w = 0; w < ur.z && ok; ++w, ++nw) {
              const uint32_t ws = nw % WG_NW, wph = (nw / WG_NW) & 1;
              const int4 wr = s_win[w];
              const int nsl = wr.w & 0xFF, so = wr.z - ur.w;
              const uint32_t wlo = desc_sw128_lo(win0 + ws * WG_WIN_BYTES, 0);
              ok = mbar_wait(wfull(ws), wph, abort_flag, 0x93) ? 1 : 0;
              if (!ok) break;
              tc_fence_after_sync();
              for (int s = 0; s < nsl; s += 2, tmem_d += 64, mine ^= 1) {
                if (mine) continue;
                const uint32_t alo = wlo + (uint32_t)s_shift[so + s];
#pragma unroll
                for (int kk = 0; kk < WG_TILES * TILE_M / 16; ++kk)  // 16 pixels per MMA: +2048 bytes
                  mma_bf16_ss_lo(tmem_d, alo + 128 * kk, DHI, blo + 128 * kk, DHI, idesc, kk ? 1u : accum);
              }
              mma_commit(wempty(ws));
            }
            accum = 1;
            if (ok) mma_commit(gempty(gs));
          }
        }
        if (ok) mma_commit(accfull);
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
    }
    if (lane == 0) {
      mma_commit(drain_bar);
      mbar_wait(drain_bar, 0, abort_flag, 0x94);
    }
    __syncwarp();
  } else if (warp <= N_EPI_WARPS) {
    // ------------------------------------------------------------------ epilogue: accumulators -> gE
    // While a unit's MMAs run these warps have nothing to read out, so they add up the bias gradient
    // from the grad_output chunks that pass through shared memory anyway: in the unit that starts a
    // row (every chunk of a row's grad_output exactly once), thread = 8 channels x 16 pixels of a chunk.
    const int q = warp & 3;
    const int bcc = lane & 7, bpg = (warp - 1) * 4 + (lane >> 3);
    uint32_t it = 0, ng = 0;
    for (long u; (u = unit_at(it)) >= 0; ++it) {
      int part;
      const int4 ur = unit_rec(u, part);
      int okt = 1;
      {
        const bool sum_bias = a.gb != nullptr && ur.y == __ldg(plan + a.d.off_row + ur.x);
        float bs[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) bs[i] = 0.f;
        const int b0 = part * bper, b1 = min(a.B, b0 + bper);
        for (int c = 0; c < (b1 - b0) * nchunk && okt; ++c, ++ng) {
          const uint32_t gs = ng % WG_NG, gph = (ng / WG_NG) & 1;
          if (lane == 0) okt = mbar_wait(gfull(gs), gph, abort_flag, 0x98, 64) ? 1 : 0;
          okt = __shfl_sync(0xffffffffu, okt, 0);
          if (!okt) break;
          if (sum_bias) {
            const uint32_t base = gy0 + gs * WG_GY_BYTES;
#pragma unroll 4
            for (int j = bpg; j < WG_TILES * TILE_M; j += 16) {
              uint4 v;
              asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                           : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                           : "r"(base + j * 128 + ((bcc ^ (j & 7)) << 4)));
              const uint32_t p4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
              for (int t = 0; t < 4; ++t) {
                bs[2 * t] += __uint_as_float(p4[t] << 16);
                bs[2 * t + 1] += __uint_as_float(p4[t] & 0xFFFF0000u);
              }
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(gempty(gs));
        }
        if (!okt) break;
        if (sum_bias) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            bs[i] += __shfl_xor_sync(0xffffffffu, bs[i], 8);
            bs[i] += __shfl_xor_sync(0xffffffffu, bs[i], 16);
          }
          if (lane < 8) {
#pragma unroll
            for (int i = 0; i < 8; ++i) atomicAdd(a.gb + bcc * 8 + i, bs[i]);
          }
        }
      }
      if (lane == 0) okt = mbar_wait(accfull, it & 1, abort_flag, 0x95) ? 1 : 0;
      okt = __shfl_sync(0xffffffffu, okt, 0);
      if (!okt) break;
      tc_fence_after_sync();
      float* out = a.gE + (size_t)part * a.d.nslot * 4096;
      int pair = 0;
      for (int w = 0; w < ur.z; ++w) {
        const int4 wr = __ldg(reinterpret_cast<const int4*>(plan + a.d.off_win) + ur.y + w);
        const int nsl = wr.w & 0xFF;
        for (int s = 0; s < nsl; s += 2, ++pair) {
          // lanes 0-63 of the accumulator: slot s (row = ci); lanes 64-127: slot s + 1
          const int slot = wr.z + s + (q >> 1);
          const bool live = (q >> 1) == 0 || s + 1 < nsl;
          const int ci = (q & 1) * 32 + lane;
#pragma unroll
          for (int cc = 0; cc < 2; ++cc) {
            uint32_t v[32];
            tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + pair * 64 + cc * 32, v);
            tmem_ld_wait();
            if (live) {
              float4* dst = reinterpret_cast<float4*>(out + ((size_t)slot * 64 + ci) * 64 + cc * 32);
#pragma unroll
              for (int j = 0; j < 8; ++j)
                dst[j] = make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                     __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(accempty);
    }
  } else if (warp >= FIRST_PROD_WARP) {
    // ------------------------------------------------------------------ loaders
    // Items in the order the MMA threads consume them: per (image, chunk) the gy chunk, then the
    // unit's windows, fetched by the TMA unit in boxes of RI_BOX pixels (the seam box of a wrapped
    // window by cp.async).  Two warps work side by side, so two items are in flight.  A ring stage is
    // always filled by the same warp (stage index modulo 2): a warp waits for its stages in order, so
    // it can never be more than one phase ahead of the consumer - which is what a parity wait needs
    // to be unambiguous.  A stage's barrier gets one arrival, which also announces the TMA bytes.
    const int team = warp - FIRST_PROD_WARP;
    if (team < TEAMS) {
      uint32_t nw = 0, ng = 0, it = 0;
      bool ok = true;
      auto announce = [&](uint32_t bar, uint32_t bytes) {
        __syncwarp();
        if (lane == 0)
          asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
      };
      auto wait_empty = [&](uint32_t bar, uint32_t parity, int code) {
        int okw = 1;
        if (lane == 0) okw = mbar_wait(bar, parity, abort_flag, code) ? 1 : 0;
        return __shfl_sync(0xffffffffu, okw, 0) != 0;
      };
      for (long u; ok && (u = unit_at(it)) >= 0; ++it) {
        int part;
        const int4 ur = unit_rec(u, part);
        const int b0 = part * bper, b1 = min(a.B, b0 + bper);
        for (int b = b0; b < b1 && ok; ++b) {
          for (int ch = 0; ch < nchunk && ok; ++ch) {
            const int x0 = ch * WG_TILES * TILE_M;
            if ((int)(ng % TEAMS) == team) {  // the gy chunk
              const uint32_t gs = ng % WG_NG, gph = (ng / WG_NG) & 1;
              if (!wait_empty(gempty(gs), gph ^ 1, 0x96)) { ok = false; break; }
              const uint32_t dst = gy0 + gs * WG_GY_BYTES;
              if (lane == 0)
                for (int k = 0; k < WG_TILES * TILE_M / RI_BOX; ++k)
                  tma_load_box(dst + (uint32_t)k * (RI_BOX * 128), &tmap_gy, x0 + k * RI_BOX, b * a.RH + ur.x, gfull(gs));
              announce(gfull(gs), WG_GY_BYTES);
            }
            ++ng;
            for (int w = 0; w < ur.z; ++w, ++nw) {
              if ((int)(nw % TEAMS) != team) continue;
              const int4 wr = __ldg(reinterpret_cast<const int4*>(plan + a.d.off_win) + ur.y + w);
              const uint32_t ws = nw % WG_NW, wph = (nw / WG_NW) & 1;
              if (!wait_empty(wempty(ws), wph ^ 1, 0x97)) { ok = false; break; }
              const int span = (wr.w >> 8) & 0xFF, mode = wr.w >> 16;
              const int srow = b * a.SH + wr.x;
              const uint32_t sbase = win0 + ws * WG_WIN_BYTES;
              const int nbox = (WG_TILES * TILE_M + span + RI_BOX - 1) / RI_BOX;
              int c = x0 + wr.y;  // source column of the window's first pixel
              if (mode == RI_MODE_WRAP) { c %= a.SW; if (c < 0) c += a.SW; }
              uint32_t tma_bytes = 0;
              bool seam = false;
              for (int k = 0; k < nbox; ++k) {
                if (mode == RI_MODE_WRAP && c + RI_BOX > a.SW) {
                  int sc = c + lane;  // the seam: lane = row of the box
                  if (sc >= a.SW) sc -= a.SW;
                  const bf16* sp = a.x + ((long)srow * a.SW + sc) * 64;
                  const uint32_t dst = sbase + (uint32_t)(k * RI_BOX + lane) * 128u;
#pragma unroll
                  for (int cc = 0; cc < 8; ++cc) cp_async16(dst + ((cc ^ (lane & 7)) << 4), sp + cc * 8, 16u);
                  seam = true;
                } else {
                  if (lane == 0) tma_load_box(sbase + (uint32_t)k * (RI_BOX * 128), &tmap_x, c, srow, wfull(ws));
                  tma_bytes += RI_BOX * 128;
                }
                c += RI_BOX;
                if (mode == RI_MODE_WRAP && c >= a.SW) c -= a.SW;
              }
              if (seam) {
                cp_async_commit();
                cp_async_wait_all();
                fence_proxy_async_smem();
              }
              announce(wfull(ws), tma_bytes);
            }
          }
        }
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

// Weight gradient, second step.  Three kernels, no atomics, results repeat bit for bit:
//   rowinv_wgrad_reduce_kernel  P1[y][k][ci][co] = sum over the y-th chunk of slots, over the slot's
//                               contributions (k, w), of w * (sum over batch parts of gE[slot][ci][co])
//   rowinv_wgrad_fix_kernel     P2[k][y][ci][co] = the planner's corrections of tap k in the y-th chunk
//   rowinv_wgrad_final_kernel   gw[co][ci][k] = sum_y P1[y][k] + sum_y P2[k][y]
// In the first a thread owns four neighbouring co of one ci (one float4 of a slot's 64 x 64 block)
// and keeps the loads of the next U slots in flight while it works on the current ones.
constexpr int WGR_PARTS = 2;   // most parts the batch is cut into
constexpr int WGF_CHUNKS = 128;  // chunks the corrections are cut into
template <int PARTS, int TAPS, int U>
__global__ void __launch_bounds__(256, 2) rowinv_wgrad_reduce_kernel(const float4* __restrict__ gE,
                                                                     const int* __restrict__ plan, RiDir d,
                                                                     int K, float4* __restrict__ P1) {
  const int t = blockIdx.x * 256 + threadIdx.x;  // float4 of a slot: ci = t / 16, co = 4 (t % 16)
  const int per = (d.nslot + gridDim.y - 1) / gridDim.y;
  const int s0 = blockIdx.y * per, s1 = min(d.nslot, s0 + per);
  const size_t part_stride = (size_t)d.nslot * 1024;
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int k0 = 0; k0 < K; k0 += TAPS) {
    float4 acc[TAPS];
#pragma unroll
    for (int i = 0; i < TAPS; ++i) acc[i] = zero;
    float4 cur[U][PARTS], nxt[U][PARTS];
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int p = 0; p < PARTS; ++p)
        cur[u][p] = s0 + u < s1 ? __ldg(gE + p * part_stride + (size_t)(s0 + u) * 1024 + t) : zero;
    for (int s = s0; s < s1; s += U) {
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int p = 0; p < PARTS; ++p)
          nxt[u][p] = s + U + u < s1 ? __ldg(gE + p * part_stride + (size_t)(s + U + u) * 1024 + t) : zero;
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (s + u >= s1) break;
        float4 v = cur[u][0];
#pragma unroll
        for (int p = 1; p < PARTS; ++p) {
          v.x += cur[u][p].x; v.y += cur[u][p].y; v.z += cur[u][p].z; v.w += cur[u][p].w;
        }
        const int c0 = __ldg(plan + d.off_coff + s + u), c1 = __ldg(plan + d.off_coff + s + u + 1);
        for (int c = c0; c < c1; ++c) {
          const int k = __ldg(plan + d.off_ctap + c) - k0;
          const float wv = __int_as_float(__ldg(plan + d.off_cw + c));
#pragma unroll
          for (int i = 0; i < TAPS; ++i)
            if (i == k) {
              acc[i].x = fmaf(wv, v.x, acc[i].x); acc[i].y = fmaf(wv, v.y, acc[i].y);
              acc[i].z = fmaf(wv, v.z, acc[i].z); acc[i].w = fmaf(wv, v.w, acc[i].w);
            }
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int p = 0; p < PARTS; ++p) cur[u][p] = nxt[u][p];
    }
#pragma unroll
    for (int i = 0; i < TAPS; ++i)
      if (k0 + i < K) P1[((size_t)blockIdx.y * K + k0 + i) * 1024 + t] = acc[i];
  }
}

// The planner's corrections in the weight gradient:
// P2[k][y][ci][co] = sum_b dw gy[b, row, col, co] x[b, srow, scol, ci] over the corrections with tap k
// in chunk y.  blockIdx.x = tap, blockIdx.y = chunk: the block first lists the corrections of its chunk
// that belong to its tap (in order), then walks the list.  Per correction that is a 64 x B by B x 64
// product: warp w holds the 16 co x 64 ci block w of the result and issues 8 m16n8k16 MMAs per 16
// images (k = image).
constexpr int WGF_LIST = 128;
__global__ void __launch_bounds__(128) rowinv_wgrad_fix_kernel(const bf16* __restrict__ x,
                                                               const bf16* __restrict__ gy,
                                                               const int* __restrict__ plan, RiDir d,
                                                               int B, int SH, int SW, int RH, int RW,
                                                               float* __restrict__ P2) {
  __shared__ int s_list[WGF_LIST];
  __shared__ int s_cnt[5];
  const int k = blockIdx.x;
  const int per = (d.nskip + gridDim.y - 1) / gridDim.y;
  const int e0 = blockIdx.y * per, e1 = min(d.nskip, e0 + per);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const unsigned short* gy16 = reinterpret_cast<const unsigned short*>(gy);
  const unsigned short* x16 = reinterpret_cast<const unsigned short*>(x);
  const long gy_img = (long)RH * RW * 64, x_img = (long)SH * SW * 64;
  float acc[8][4];
#pragma unroll
  for (int nt = 0; nt < 8; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[nt][i] = 0.f;
  for (int base = e0; base < e1; base += WGF_LIST) {
    // ordered compaction of the entries with this block's tap
    const int e = base + threadIdx.x;
    const bool hit = e < e1 && __ldg(plan + d.off_skip + 6 * e + 4) == k;
    const unsigned m = __ballot_sync(0xffffffffu, hit);
    if (lane == 0) s_cnt[warp + 1] = __popc(m);
    __syncthreads();
    if (threadIdx.x == 0) {
      s_cnt[0] = 0;
      for (int w = 0; w < 4; ++w) s_cnt[w + 1] += s_cnt[w];
    }
    __syncthreads();
    if (hit) s_list[s_cnt[warp] + __popc(m & ((1u << lane) - 1))] = e;
    __syncthreads();
    const int n = s_cnt[4];
    for (int i = 0; i < n; ++i) {
      const int* ent = plan + d.off_skip + 6 * s_list[i];
      const int row = __ldg(ent), col = __ldg(ent + 1), srow = __ldg(ent + 2), scol = __ldg(ent + 3);
      const float dw = __int_as_float(__ldg(ent + 5));
      const unsigned short* gp = gy16 + ((long)row * RW + col) * 64 + warp * 16 + g;  // co = 16 w + g (+ 8)
      const unsigned short* xq = x16 + ((long)srow * SW + scol) * 64 + g;            // ci = 8 nt + g
      for (int b0 = 0; b0 < B; b0 += 16) {
        // images b0 + 2 t, + 1 (fragment registers 0, 1) and b0 + 2 t + 8, + 9 (registers 2, 3 / 1)
        const int ba = b0 + 2 * t;
        const bool v0 = ba < B, v1 = ba + 1 < B, v2 = ba + 8 < B, v3 = ba + 9 < B;
        auto pair = [](const unsigned short* p, long s0, bool on0, long s1, bool on1) -> uint32_t {
          const uint32_t lo = on0 ? (uint32_t)__ldg(p + s0) : 0u, hi = on1 ? (uint32_t)__ldg(p + s1) : 0u;
          return lo | (hi << 16);
        };
        uint32_t afr[4];
        afr[0] = pair(gp, ba * gy_img, v0, (ba + 1) * gy_img, v1);
        afr[1] = pair(gp + 8, ba * gy_img, v0, (ba + 1) * gy_img, v1);
        afr[2] = pair(gp, (ba + 8) * gy_img, v2, (ba + 9) * gy_img, v3);
        afr[3] = pair(gp + 8, (ba + 8) * gy_img, v2, (ba + 9) * gy_img, v3);
        uint32_t bfr[8][2];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
          bfr[nt][0] = pair(xq + nt * 8, ba * x_img, v0, (ba + 1) * x_img, v1);
          bfr[nt][1] = pair(xq + nt * 8, (ba + 8) * x_img, v2, (ba + 9) * x_img, v3);
        }
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
          float tmp[4] = {0.f, 0.f, 0.f, 0.f};
          mma_m16n8k16_bf16(tmp, afr, bfr[nt]);
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[nt][j] = fmaf(dw, tmp[j], acc[nt][j]);
        }
      }
    }
    __syncthreads();
  }
  // D[co][ci]: co = 16 w + g (+ 8 for registers 2, 3), ci = 8 nt + 2 t (+ 1 for registers 1, 3)
  float* out = P2 + ((size_t)k * gridDim.y + blockIdx.y) * 4096;
#pragma unroll
  for (int nt = 0; nt < 8; ++nt)
#pragma unroll
    for (int j = 0; j < 4; ++j)
      out[(nt * 8 + 2 * t + (j & 1)) * 64 + warp * 16 + g + (j >> 1) * 8] = acc[nt][j];
}

// gw[co][ci][k] = sum_y P1[y][k][ci][co] + sum_y P2[k][y][ci][co].  blockIdx.x = tap, blockIdx.y = 64
// elements (one ci); the block's four groups of threads share the terms, eight loads in flight each.
__global__ void __launch_bounds__(256) rowinv_wgrad_final_kernel(const float* __restrict__ P1, int Y1,
                                                                 const float* __restrict__ P2, int Y2,
                                                                 int K, int Cin, float* __restrict__ gw) {
  __shared__ float s_sum[4][64];
  const int k = blockIdx.x, e = blockIdx.y * 64 + (threadIdx.x & 63), grp = threadIdx.x >> 6;
  float acc = 0.f;
  for (int y0 = grp * 8; y0 < Y1 + Y2; y0 += 32) {
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int y = y0 + j;
      v[j] = y < Y1 ? __ldg(P1 + ((size_t)y * K + k) * 4096 + e)
                    : (y < Y1 + Y2 ? __ldg(P2 + ((size_t)k * Y2 + (y - Y1)) * 4096 + e) : 0.f);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) acc += v[j];
  }
  s_sum[grp][threadIdx.x & 63] = acc;
  __syncthreads();
  if (grp == 0) {
    const int l = threadIdx.x;
    const float r = (s_sum[0][l] + s_sum[1][l]) + (s_sum[2][l] + s_sum[3][l]);
    const int ci = e >> 6, co = e & 63;
    gw[((long)co * Cin + ci) * K + k] = r;
  }
}

static size_t rowinv_e_bytes(const RiDir& d, int NR) { return (size_t)d.nslot * NR * 128; }

template <int NOUT>
static int rowinv_launch_n(const RowInvArgs& a, cudaStream_t st) {
  using Cfg = RiCfg<NOUT>;
  static_assert(Cfg::SMEM <= SMEM_LIMIT, "row-invariant kernel does not fit shared memory");
  static_assert(Cfg::WIN_BYTES % (RI_BOX * 128) == 0 && (Cfg::TPU * TILE_M + RI_SPAN) % RI_BOX == 0, "window boxes");
  if (!allow_big_smem(conv_rowinv_tc_kernel<NOUT>)) return MC_ERR_LAUNCH;
  CUtensorMap tmap;
  if (!ri_make_tensor_map(&tmap, a.src, (long)a.B * a.SH, a.SW)) return MC_ERR_LAUNCH;
  const long g = a.units < sm_count() ? a.units : sm_count();
  conv_rowinv_tc_kernel<NOUT><<<(int)g, TC_THREADS, Cfg::SMEM, st>>>(a, tmap), MC_COUNT(1);
  MC_CHECK_LAUNCH();
  return MC_OK;
}

}  // namespace tc

using namespace tc;

// Shapes the row-invariant kernels take (the map itself is judged by the planner).
bool conv_rowinv_shape_ok(const mc_desc* d) {
  return d->dtype == MC_BF16 && d->layout == MC_NHWC && d->P == 0 && (d->interp == 1 || d->interp == 2) &&
         d->C_in == 64 && d->C_out == 64 && d->OW == d->IW && d->OW % TILE_M == 0 &&
         (d->OW / TILE_M) % RiCfg<128>::TPU == 0 && d->K <= 64 &&
         (long)d->B * std::max(d->OH, d->IH) * d->OW < (1L << 30);
}

size_t rowinv_analysis_bytes(const mc_desc* d) { return (size_t)d->OH * d->K * 3 * sizeof(double); }

int rowinv_analyse_launch(const mc_desc* d, const void* map, void* out, cudaStream_t st) {
  if (!aligned16(map) || !aligned16(out)) return MC_ERR_BAD_ARG;
  rowinv_analyse_kernel<<<d->OH, 256, 0, st>>>((const float*)map, d->OH, d->OW, d->K, d->IW,
                                               (double*)out), MC_COUNT(1);
  MC_CHECK_LAUNCH();
  return MC_OK;
}

// -> number of int32s of the plan (0: the map does not qualify); copies at most cap ints to out
long rowinv_assemble_host(const mc_desc* d, const double* analysis, const float* map, int* out,
                          long cap) {
  if (!conv_rowinv_shape_ok(d)) return 0;
  const std::vector<int> plan = rowinv_assemble(d, analysis, map);
  if (plan.empty()) return 0;
  if (out && cap >= (long)plan.size()) std::memcpy(out, plan.data(), plan.size() * sizeof(int));
  return (long)plan.size();
}

static bool rowinv_plan_matches(const mc_desc* d, const RiHeader* h) {
  return h && h->magic == RI_PLAN_MAGIC && h->OH == d->OH && h->OW == d->OW && h->IH == d->IH &&
         h->IW == d->IW && h->K == d->K && h->interp == d->interp;
}

// workspace of a call: the effective weights of every slot, then the tap-major weight copy
static size_t rowinv_wk_offset(const RiDir& D, int NR) { return (rowinv_e_bytes(D, NR) + 255) & ~(size_t)255; }
size_t rowinv_ws_bytes(const mc_desc* d, const void* plan_host, int dir) {
  const RiHeader* h = (const RiHeader*)plan_host;
  if (!rowinv_plan_matches(d, h)) return 0;
  return rowinv_wk_offset(h->pair[dir], 128) + (size_t)d->K * 64 * 64 * sizeof(bf16);
}

// dir 0: y = conv(x); dir 1: gx = conv^T(gy).  `src` is the tensor that is gathered from.
int rowinv_conv_launch(const mc_desc* d, int dir, const void* src, const void* plan_host,
                       const void* plan_dev, const void* w, const void* bias, void* res, void* ws,
                       size_t ws_bytes, cudaStream_t st) {
  if (!conv_rowinv_shape_ok(d) || (d->flags & MC_FLAG_RELU)) return MC_ERR_UNSUPPORTED;
  const RiHeader* h = (const RiHeader*)plan_host;
  if (!rowinv_plan_matches(d, h)) return MC_ERR_BAD_ARG;
  const RiDir& D = h->dir[dir];    // per row: the corrections
  const RiDir& P = h->pair[dir];   // per pair of rows: what the main kernel runs on
  if (!ws || ws_bytes < rowinv_ws_bytes(d, plan_host, dir)) return MC_ERR_WORKSPACE;
  if (!aligned16(src) || !aligned16(res) || !aligned16(ws) || !aligned16(plan_dev)) return MC_ERR_BAD_ARG;
  const int* plan = (const int*)plan_dev;
  bf16* wk = (bf16*)((uint8_t*)ws + rowinv_wk_offset(P, 128));
  rowinv_wk_kernel<<<grid_for((long)d->K * 64 * 64, 256), 256, 0, st>>>((const bf16*)w, wk, 64, d->K,
                                                                         d->C_in, dir), MC_COUNT(1);
  // a pair's slot has two lists of contributions, one per row: two consecutive 64 x 64 blocks, which
  // together are the N = 128 operand of the slot
  if (P.nslot > 0)
    rowinv_weights_kernel<<<2 * P.nslot, 256, 0, st>>>(wk, plan, P, (uint4*)ws, 64), MC_COUNT(1);
  RowInvArgs a;
  a.src = (const bf16*)src; a.out = (bf16*)res; a.bias = (const bf16*)bias;
  a.plan = plan; a.d = P; a.E = (const uint4*)ws;
  a.B = d->B;
  if (dir == 0) { a.SH = d->IH; a.SW = d->IW; a.RH = d->OH; a.RW = d->OW; }
  else { a.SH = d->OH; a.SW = d->OW; a.RH = d->IH; a.RW = d->IW; }
  a.tpu = RiCfg<128>::TPU;
  a.upr = a.RW / (TILE_M * a.tpu);
  a.units = (long)P.rows * a.B * a.upr;
  int rc = rowinv_launch_n<128>(a, st);
  if (rc) return rc;
  if (D.ngroup > 0) {
    rowinv_fix_kernel<<<D.ngroup, 32 * FIX_WARPS, 0, st>>>((const bf16*)src, (bf16*)res, wk, plan, D, d->B,
                                                                a.SH, a.SW, a.RH, a.RW, 64), MC_COUNT(1);
    MC_CHECK_LAUNCH();
  }
  return MC_OK;
}


int bias_grad_launch(const mc_desc*, const void*, void*, cudaStream_t);

// Parts the batch is cut into for the weight gradient: one when the units alone fill the device several
// times over, two otherwise (more, smaller units; twice the partial sums to add up afterwards).
static int rowinv_bsplit(const mc_desc* d, const RiDir& D) {
  return d->B >= 2 && D.nwgunit < 6 * sm_count() ? WGR_PARTS : 1;
}
// chunks the slots are cut into for the first reduction
static int rowinv_wgrad_chunks(const RiDir& D) { return std::max(1, std::min(D.nslot, sm_count())); }

// workspace of the weight gradient: gE [parts][nslot][64][64], P1 [chunks][K][64][64],
// P2 [K][WGF_CHUNKS][64][64], all float32
size_t rowinv_wgrad_ws_bytes(const mc_desc* d, const void* plan_host) {
  const RiHeader* h = (const RiHeader*)plan_host;
  if (!rowinv_plan_matches(d, h)) return 0;
  const RiDir& D = h->dir[0];
  return ((size_t)rowinv_bsplit(d, D) * D.nslot + (size_t)rowinv_wgrad_chunks(D) * d->K +
          (size_t)d->K * WGF_CHUNKS) * 4096 * sizeof(float);
}

template <int PARTS>
static void rowinv_wgrad_reduce_launch(const float4* gE, const int* plan, const RiDir& D, int K, int Y1,
                                       float4* P1, cudaStream_t st) {
  constexpr int U = PARTS == 1 ? 8 : 4;
  if (K <= 9)
    rowinv_wgrad_reduce_kernel<PARTS, 9, U><<<dim3(4, Y1), 256, 0, st>>>(gE, plan, D, K, P1), MC_COUNT(1);
  else
    rowinv_wgrad_reduce_kernel<PARTS, 16, U><<<dim3(4, Y1), 256, 0, st>>>(gE, plan, D, K, P1), MC_COUNT(1);
}

// gw (C_out, C_in, K) float32 and gb (C_out) float32 (may be null), fully overwritten.
int rowinv_wgrad_launch(const mc_desc* d, const void* gy, const void* x, const void* plan_host,
                        const void* plan_dev, void* gw, void* gb, void* ws, size_t ws_bytes,
                        cudaStream_t st) {
  if (!conv_rowinv_shape_ok(d)) return MC_ERR_UNSUPPORTED;
  const RiHeader* h = (const RiHeader*)plan_host;
  if (!rowinv_plan_matches(d, h)) return MC_ERR_BAD_ARG;
  const RiDir& D = h->dir[0];
  if (!ws || ws_bytes < rowinv_wgrad_ws_bytes(d, plan_host)) return MC_ERR_WORKSPACE;
  if (!aligned16(gy) || !aligned16(x) || !aligned16(ws) || !aligned16(plan_dev)) return MC_ERR_BAD_ARG;
  if (d->OW % (WG_TILES * TILE_M) != 0) return MC_ERR_UNSUPPORTED;
  const int* plan = (const int*)plan_dev;
  const int bsplit = rowinv_bsplit(d, D), Y1 = D.nwgunit > 0 ? rowinv_wgrad_chunks(D) : 0;
  float* gE = (float*)ws;
  float* P1 = gE + (size_t)bsplit * D.nslot * 4096;
  float* P2 = P1 + (size_t)rowinv_wgrad_chunks(D) * d->K * 4096;
  // the bias gradient comes out of the main kernel when every row of grad_output passes through it
  // (every row has a unit), otherwise from the stand-alone reduction
  bool bias_in_kernel = gb != nullptr && D.nwgunit > 0;
  if (bias_in_kernel) {
    const int* row_off = (const int*)plan_host + D.off_row;
    for (int r = 0; r < D.rows && bias_in_kernel; ++r) bias_in_kernel = row_off[r + 1] > row_off[r];
  }
  if (bias_in_kernel && cudaMemsetAsync(gb, 0, 64 * sizeof(float), st) != cudaSuccess) return MC_ERR_LAUNCH;
  if (D.nwgunit > 0) {
    RowInvWgArgs a;
    a.x = (const bf16*)x; a.gy = (const bf16*)gy; a.gE = gE; a.plan = plan; a.d = D;
    a.gb = bias_in_kernel ? (float*)gb : nullptr;
    a.B = d->B; a.SH = d->IH; a.SW = d->IW; a.RH = d->OH; a.RW = d->OW;
    a.bsplit = bsplit;
    a.units = (long)D.nwgunit * a.bsplit;
    if (!allow_big_smem(conv_rowinv_wgrad_kernel)) return MC_ERR_LAUNCH;
    const long g = a.units < sm_count() ? a.units : sm_count();
    CUtensorMap tmap_x, tmap_gy;
    if (!ri_make_tensor_map(&tmap_x, x, (long)d->B * d->IH, d->IW) ||
        !ri_make_tensor_map(&tmap_gy, gy, (long)d->B * d->OH, d->OW))
      return MC_ERR_LAUNCH;
    conv_rowinv_wgrad_kernel<<<(int)g, TC_THREADS, WG_SMEM, st>>>(a, tmap_x, tmap_gy), MC_COUNT(1);
    MC_CHECK_LAUNCH();
    if (bsplit == 1) rowinv_wgrad_reduce_launch<1>((const float4*)gE, plan, D, d->K, Y1, (float4*)P1, st);
    else rowinv_wgrad_reduce_launch<WGR_PARTS>((const float4*)gE, plan, D, d->K, Y1, (float4*)P1, st);
  }
  const int Y2 = D.nskip > 0 ? WGF_CHUNKS : 0;
  if (Y2 > 0)
    rowinv_wgrad_fix_kernel<<<dim3(d->K, Y2), 128, 0, st>>>((const bf16*)x, (const bf16*)gy, plan, D, d->B,
                                                            d->IH, d->IW, d->OH, d->OW, P2), MC_COUNT(1);
  rowinv_wgrad_final_kernel<<<dim3(d->K, 64), 256, 0, st>>>(P1, Y1, P2, Y2, d->K, d->C_in, (float*)gw),
      MC_COUNT(1);
  MC_CHECK_LAUNCH();
  if (gb && !bias_in_kernel) return bias_grad_launch(d, gy, gb, st);
  return MC_OK;
}

}  // namespace mc
