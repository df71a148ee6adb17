// Weight and bias gradient of a layer with very few input channels and a nearest map (the first
// layer of an encoder: 3 -> 64 channels, 7 taps), included by conv_tc.cu.
//
//   gw[co][ci][k] = sum_{b, p} gy[b, p, co] x[b, src(p, k), ci]        gb[co] = sum_{b, p} gy[b, p, co]
//   (MappedConvBackward's weight / bias part, src/nn/cuda/mapped_convolution_layer.cu:134-193)
//
// The whole (tap, channel) axis is K C_in <= 31 columns wide, so the product is tiny next to the
// one pass over grad_output it needs: the kernel is bound by HBM (algorithmic bytes: grad_output
// once - 128 bytes per pixel for 64 output channels; x and the compact tap table stay in L2).  A
// tcgen05 tile would be mostly padding; each warp instead multiplies 16 pixels at a time with
// warp-level MMAs (m16n8k16: m = output channel, n = (tap, channel) column, k = pixel) and keeps a
// 64 x 32 accumulator in registers for all the pixels it sees.  One extra column of ones gives the
// bias gradient.  Sixteen warps per SM each run a dependent chain per step (table entry -> x value
// -> MMA), so the step's loads are all issued up front, index arithmetic is 32-bit and nothing in
// the loop divides; grad_output rows are requested into L2 two steps ahead.
//
// Row r of m-tile mt holds output channel 8 (r % 8) + 2 mt + (r / 8): the eight channels a lane
// needs of a pixel are then neighbours, one 16-byte load, and the lanes of a warp read whole
// 128-byte rows.
constexpr int SCW_WARPS = 8;          // warps per block
constexpr int SCW_MAX_COLS = 32;      // (tap, channel) columns + the ones column, padded to 8s

__device__ __forceinline__ void scw_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

struct SmallCinArgs {
  const bf16* ymask; // MASK kernels: the layer's ReLU output (B, npix, C_out); grad_output counts where it is > 0
  const bf16* gy;    // (B, npix, C_out) channels-last
  const bf16* x;     // (B, spix, C_in) channels-last
  const int* tab32;  // (npix, K): source pixel of every (pixel, tap), -1 = reads nothing
  float* gw;         // (C_out, C_in, K), zero before the launch
  float* gb;         // (C_out), zero before the launch, or null
  long rows;         // B * npix
  int npix, spix, C_in, C_out, K;
};

// MASK: grad_output is the gradient behind a ReLU whose output is ymask - the activation's own
// gradient (grad_output where ymask > 0, else 0) is applied to the rows as they are loaded, which
// saves the separate pass that would write the masked tensor.
template <int NT, bool MASK>  // n-tiles of 8 columns: K * C_in + 1 <= 8 NT
__global__ void __launch_bounds__(32 * SCW_WARPS, 2) conv_wgrad_smallcin_kernel(const SmallCinArgs a) {
  __shared__ float s_acc[64][8 * NT + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int co0 = blockIdx.y * 64;  // this block's 64 output channels
  const int ncols = a.K * a.C_in;   // column ncols is the ones column
  for (int i = threadIdx.x; i < 64 * (8 * NT + 1); i += blockDim.x) (&s_acc[0][0])[i] = 0.f;
  __syncthreads();

  // the columns this lane gathers: n = 8 nt + g -> (tap, channel)
  int tap_n[NT], ci_n[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int n = 8 * nt + g;
    tap_n[nt] = n < ncols ? n / a.C_in : (n == ncols ? -1 : -2);  // -1: ones, -2: padding
    ci_n[nt] = n < ncols ? n % a.C_in : 0;
  }
  const unsigned short* x16 = reinterpret_cast<const unsigned short*>(a.x);
  float acc[4][NT][4];
#pragma unroll
  for (int mt = 0; mt < 4; ++mt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[mt][nt][j] = 0.f;

  // (all indices below fit 32 bits: the launcher checks rows * C_out / 64, npix * K and the size of x)
  const int nsteps = (int)((a.rows + 15) / 16);
  const int stride = (int)gridDim.x * SCW_WARPS;
  const int rows = (int)a.rows;
  int ks = (int)blockIdx.x * SCW_WARPS + warp;
  // (image, pixel) of the step's first row, carried from step to step instead of divided out
  int b0 = (int)(((long)ks * 16) / a.npix);
  int p0 = (int)((long)ks * 16 - (long)b0 * a.npix);
  const int adv = stride * 16, adv_b = adv / a.npix, adv_p = adv - adv_b * a.npix;
  for (; ks < nsteps; ks += stride) {
    // the lane's four pixels: rows r0 + 2 t, + 1, + 8, + 9 of the flattened (image, pixel) axis
    const int r0 = ks * 16;
    {
      // grad_output rows of this warp's step after next into L2 (the loads below go straight into
      // registers, so this is what keeps more than one step of DRAM traffic in flight per warp)
      const long rn = (long)r0 + 2L * adv + (lane >> 1);  // lane -> (row, half of its 128 bytes)
      if (rn < a.rows)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(a.gy + rn * a.C_out + co0 + (lane & 1) * 32));
    }
    const uint4* gyv = reinterpret_cast<const uint4*>(a.gy + (long)r0 * a.C_out + co0) + g;
    const uint4* ymv = reinterpret_cast<const uint4*>(a.ymask + (long)r0 * a.C_out + co0) + g;
    const int vstride = a.C_out / 8;  // uint4 per row
    uint4 v[4], ym[MASK ? 4 : 1];
    int src[NT][4];
    bool on[4];
    int xrow0[4];
    // every load of the step is issued before anything is used: rows past the end are clamped to a
    // valid address and zeroed afterwards, taps that read nothing likewise
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int j = 2 * t + (q & 1) + (q >> 1) * 8;
      on[q] = r0 + j < rows;
      const int jc = on[q] ? j : 0;
      v[q] = __ldg(gyv + jc * vstride);
      if (MASK) ym[q] = __ldg(ymv + jc * vstride);
      int p = p0 + jc, b = b0;
      if (p >= a.npix) { p -= a.npix; ++b; }  // (npix >= 16: at most one image boundary in a step)
      xrow0[q] = b * a.spix;
      const int* trow = a.tab32 + p * a.K;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) src[nt][q] = __ldg(trow + (tap_n[nt] >= 0 ? tap_n[nt] : 0));
    }
    uint32_t bv[NT][4];  // x values (16 bits each) of the four pixels, column 8 nt + g
#pragma unroll
    for (int q = 0; q < 4; ++q)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int sc = src[nt][q] > 0 ? src[nt][q] : 0;
        const uint32_t val = __ldg(x16 + (xrow0[q] + sc) * a.C_in + ci_n[nt]);
        bv[nt][q] = !on[q] ? 0u : tap_n[nt] >= 0 ? (src[nt][q] >= 0 ? val : 0u) : (tap_n[nt] == -1 ? 0x3F80u : 0u);
      }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      if (!on[q]) v[q] = make_uint4(0u, 0u, 0u, 0u);
      if (MASK) {  // 0xFFFF per bf16 of the output that is > 0
        const __nv_bfloat162 z2 = __float2bfloat162_rn(0.f);
        v[q].x &= __hgt2_mask(*reinterpret_cast<const __nv_bfloat162*>(&ym[q].x), z2);
        v[q].y &= __hgt2_mask(*reinterpret_cast<const __nv_bfloat162*>(&ym[q].y), z2);
        v[q].z &= __hgt2_mask(*reinterpret_cast<const __nv_bfloat162*>(&ym[q].z), z2);
        v[q].w &= __hgt2_mask(*reinterpret_cast<const __nv_bfloat162*>(&ym[q].w), z2);
      }
    }
    p0 += adv_p;
    b0 += adv_b;
    if (p0 >= a.npix) { p0 -= a.npix; ++b0; }
#pragma unroll
    for (int mt = 0; mt < 4; ++mt) {
      // word mt of a pixel's vector: channels 8 g + 2 mt (low half) and + 1 (high half)
      const uint32_t w0 = mt == 0 ? v[0].x : mt == 1 ? v[0].y : mt == 2 ? v[0].z : v[0].w;
      const uint32_t w1 = mt == 0 ? v[1].x : mt == 1 ? v[1].y : mt == 2 ? v[1].z : v[1].w;
      const uint32_t w2 = mt == 0 ? v[2].x : mt == 1 ? v[2].y : mt == 2 ? v[2].z : v[2].w;
      const uint32_t w3 = mt == 0 ? v[3].x : mt == 1 ? v[3].y : mt == 2 ? v[3].z : v[3].w;
      uint32_t afr[4];
      afr[0] = __byte_perm(w0, w1, 0x5410);  // row g     (channel 8 g + 2 mt),     pixels 2 t, 2 t + 1
      afr[1] = __byte_perm(w0, w1, 0x7632);  // row g + 8 (channel 8 g + 2 mt + 1), pixels 2 t, 2 t + 1
      afr[2] = __byte_perm(w2, w3, 0x5410);  // row g,     pixels 2 t + 8, 2 t + 9
      afr[3] = __byte_perm(w2, w3, 0x7632);  // row g + 8, pixels 2 t + 8, 2 t + 9
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
        scw_mma(acc[mt][nt], afr, bv[nt][0] | (bv[nt][1] << 16), bv[nt][2] | (bv[nt][3] << 16));
    }
  }

  // D[row][col]: row g (+ 8 for registers 2, 3) of m-tile mt, column 8 nt + 2 t (+ 1 for registers 1, 3)
#pragma unroll
  for (int mt = 0; mt < 4; ++mt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int j = 0; j < 4; ++j)
        atomicAdd(&s_acc[8 * g + 2 * mt + (j >> 1)][8 * nt + 2 * t + (j & 1)], acc[mt][nt][j]);
  __syncthreads();
  for (int i = threadIdx.x; i < 64 * (ncols + 1); i += blockDim.x) {
    const int co = i / (ncols + 1), n = i - co * (ncols + 1);
    const float val = s_acc[co][n];
    if (n < ncols) {
      const int tap = n / a.C_in, ci = n - tap * a.C_in;
      atomicAdd(a.gw + ((long)(co0 + co) * a.C_in + ci) * a.K + tap, val);
    } else if (a.gb) {
      atomicAdd(a.gb + co0 + co, val);
    }
  }
}

// Shapes this kernel takes: nearest map with a compact tap table, K * C_in + 1 <= 32 columns,
// output channels in blocks of 64, images of at least 16 pixels.
static bool smallcin_wgrad_shape(const mc_desc* d) {
  const long npix = (long)d->OH * d->OW, lim = 1L << 31;
  return d->interp != 1 && d->interp != 2 && d->C_in % 64 != 0 && (long)d->K * d->C_in + 1 <= SCW_MAX_COLS &&
         d->C_out % 64 == 0 && npix >= 16 && (long)d->B * npix + 16 < lim && npix * d->K < lim &&
         (long)d->B * d->IH * d->IW * d->C_in < lim;
}

static int smallcin_wgrad_launch(const mc_desc* d, const void* gy, const void* ymask, const void* x,
                                 const int* tab32, void* gw, void* gb, cudaStream_t st) {
  SmallCinArgs a;
  a.ymask = (const bf16*)(ymask ? ymask : gy);
  a.gy = (const bf16*)gy; a.x = (const bf16*)x; a.tab32 = tab32;
  a.gw = (float*)gw; a.gb = (float*)gb;
  a.npix = d->OH * d->OW; a.spix = d->IH * d->IW;
  a.rows = (long)d->B * a.npix;
  a.C_in = d->C_in; a.C_out = d->C_out; a.K = d->K;
  const int nt = (d->K * d->C_in + 1 + 7) / 8;
  const long nsteps = (a.rows + 15) / 16;
  long gx = 2L * sm_count();  // two blocks of eight warps per SM
  const long need = (nsteps + SCW_WARPS - 1) / SCW_WARPS;
  if (gx > need) gx = need;
  const dim3 grid((unsigned)gx, (unsigned)(d->C_out / 64));
  const int threads = 32 * SCW_WARPS;
  if (ymask) {
    switch (nt) {
      case 1: conv_wgrad_smallcin_kernel<1, true><<<grid, threads, 0, st>>>(a); break;
      case 2: conv_wgrad_smallcin_kernel<2, true><<<grid, threads, 0, st>>>(a); break;
      case 3: conv_wgrad_smallcin_kernel<3, true><<<grid, threads, 0, st>>>(a); break;
      default: conv_wgrad_smallcin_kernel<4, true><<<grid, threads, 0, st>>>(a); break;
    }
  } else {
    switch (nt) {
      case 1: conv_wgrad_smallcin_kernel<1, false><<<grid, threads, 0, st>>>(a); break;
      case 2: conv_wgrad_smallcin_kernel<2, false><<<grid, threads, 0, st>>>(a); break;
      case 3: conv_wgrad_smallcin_kernel<3, false><<<grid, threads, 0, st>>>(a); break;
      default: conv_wgrad_smallcin_kernel<4, false><<<grid, threads, 0, st>>>(a); break;
    }
  }
  MC_COUNT(1);
  MC_CHECK_LAUNCH();
  return MC_OK;
}
