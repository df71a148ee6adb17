/* Type-generic body of the CPU oracle; included once per scalar type by mc_oracle.c with
 *   T   = the scalar type,  SUF(name) = name##_f32 / name##_f64.
 * TEST INFRASTRUCTURE ONLY (see mc_oracle.c).  All tensors NCHW-contiguous.
 * Citations are paths inside the reference's package/ext_modules/. */

/* ---- per-sample interpolation: include/core/interpolation.h ------------------------------- */

/* Interpolate2DNearest :85-102, Interpolate2DBilinear :125-154 (+BilinearInterpolation :17-33),
 * Interpolate2DBispherical :183-210; dispatch core/resample.h:62-90 (unknown mode = nearest). */
static T SUF(interp)(const T* im, int64_t H, int64_t W, T x, T y, int mode) {
  if (mode != 1 && mode != 2) {
    const int64_t xi = llround((double)x), yi = llround((double)y);
    return (xi >= 0 && xi <= W - 1 && yi >= 0 && yi <= H - 1) ? im[yi * W + xi] : (T)0;
  }
  const int64_t x1 = (int64_t)floor((double)x), y1 = (int64_t)floor((double)y);
  const int64_t x2 = x1 + 1, y2 = y1 + 1;
  const int y1v = y1 >= 0 && y1 <= H - 1, y2v = y2 >= 0 && y2 <= H - 1;
  int x1v, x2v;
  int64_t xa, xb;
  if (mode == 1) {
    x1v = x1 >= 0 && x1 <= W - 1; x2v = x2 >= 0 && x2 <= W - 1; xa = x1; xb = x2;
  } else {
    x1v = x2v = 1; xa = ((x1 % W) + W) % W; xb = ((x2 % W) + W) % W;
  }
  const T d11 = (x1v && y1v) ? im[y1 * W + xa] : (T)0;
  const T d21 = (x2v && y1v) ? im[y1 * W + xb] : (T)0;
  const T d12 = (x1v && y2v) ? im[y2 * W + xa] : (T)0;
  const T d22 = (x2v && y2v) ? im[y2 * W + xb] : (T)0;
  const T A = (T)y2 - y, B = (T)x2 - x, C = x - (T)x1, D = y - (T)y1;
  const T t11 = A * B * d11, t21 = A * C * d21, t12 = D * B * d12, t22 = D * C * d22;
  return t11 + t21 + t12 + t22;
}

/* Extrapolate2D{Nearest,Bilinear,Bispherical} :105-122, :157-180, :213-238 (+BilinearExtrapolation
 * :36-53).  Serial here, so a plain += stands for atomic_add. */
static void SUF(extrap)(T* im, int64_t H, int64_t W, T x, T y, int mode, T v) {
  if (mode != 1 && mode != 2) {
    const int64_t xi = llround((double)x), yi = llround((double)y);
    if (xi >= 0 && xi <= W - 1 && yi >= 0 && yi <= H - 1) im[yi * W + xi] += v;
    return;
  }
  const int64_t x1 = (int64_t)floor((double)x), y1 = (int64_t)floor((double)y);
  const int64_t x2 = x1 + 1, y2 = y1 + 1;
  const int y1v = y1 >= 0 && y1 <= H - 1, y2v = y2 >= 0 && y2 <= H - 1;
  int x1v, x2v;
  int64_t xa, xb;
  if (mode == 1) {
    x1v = x1 >= 0 && x1 <= W - 1; x2v = x2 >= 0 && x2 <= W - 1; xa = x1; xb = x2;
  } else {
    x1v = x2v = 1; xa = ((x1 % W) + W) % W; xb = ((x2 % W) + W) % W;
  }
  const T A = (T)y2 - y, B = (T)x2 - x, C = x - (T)x1, D = y - (T)y1;
  if (x1v && y1v) im[y1 * W + xa] += A * B * v;
  if (x2v && y1v) im[y1 * W + xb] += A * C * v;
  if (x1v && y2v) im[y2 * W + xa] += D * B * v;
  if (x2v && y2v) im[y2 * W + xb] += D * C * v;
}

/* One tap, optionally a weighted sum over P points: core/resample.h:128-162.
 * m points at the tap's first (x, y) pair, w at its first weight (NULL / P = 0: single point). */
static T SUF(tap_get)(const T* im, int64_t H, int64_t W, const T* m, const T* w, int P, int mode) {
  if (P == 0) return SUF(interp)(im, H, W, m[0], m[1], mode);
  T acc = (T)0;
  for (int i = 0; i < P; ++i) acc += w[i] * SUF(interp)(im, H, W, m[2 * i], m[2 * i + 1], mode);
  return acc;
}
static void SUF(tap_put)(T* im, int64_t H, int64_t W, const T* m, const T* w, int P, int mode, T v) {
  if (P == 0) { SUF(extrap)(im, H, W, m[0], m[1], mode, v); return; }
  for (int i = 0; i < P; ++i) SUF(extrap)(im, H, W, m[2 * i], m[2 * i + 1], mode, w[i] * v);
}

/* ---- im2col / col2im for one batch element: include/nn/common/mapped_im2col.h:12-160 -------- */
/* col is (C*K, npix_grid), row c*K + k. */
static void SUF(im2col)(const T* im, const T* map, const T* iw, int C, int64_t H, int64_t W,
                        int64_t np, int K, int P, int mode, T* col) {
  const int pp = P ? P : 1;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < (int64_t)C * np; ++i) {
    const int64_t p = i % np, c = i / np;
    for (int k = 0; k < K; ++k) {
      const int64_t e = (p * K + k) * pp;
      col[(c * K + k) * np + p] =
          SUF(tap_get)(im + c * H * W, H, W, map + 2 * e, iw ? iw + e : 0, P, mode);
    }
  }
}
static void SUF(col2im)(const T* col, const T* map, const T* iw, int C, int64_t H, int64_t W,
                        int64_t np, int K, int P, int mode, T* im) {
  const int pp = P ? P : 1;
  /* channels are independent, so parallelising over c needs no atomics */
#pragma omp parallel for schedule(static)
  for (int64_t c = 0; c < C; ++c)
    for (int64_t p = 0; p < np; ++p)
      for (int k = 0; k < K; ++k) {
        const int64_t e = (p * K + k) * pp;
        SUF(tap_put)(im + c * H * W, H, W, map + 2 * e, iw ? iw + e : 0, P, mode,
                     col[(c * K + k) * np + p]);
      }
}

/* C(m,n) (+)= A(m,k) . B(k,n), optional transposes; plain loops standing in for at::mm. */
static void SUF(gemm)(int ta, int tb, int64_t m, int64_t n, int64_t k, const T* A, const T* B, T* C,
                      int accumulate) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < m; ++i) {
    T* c = C + i * n;
    if (!accumulate) for (int64_t j = 0; j < n; ++j) c[j] = (T)0;
    for (int64_t l = 0; l < k; ++l) {
      const T a = ta ? A[l * m + i] : A[i * k + l];
      if (!tb) {
        const T* b = B + l * n;
        for (int64_t j = 0; j < n; ++j) c[j] += a * b[j];
      } else {
        for (int64_t j = 0; j < n; ++j) c[j] += a * B[j * k + l];
      }
    }
  }
}

/* ---- mapped convolution: src/nn/cpp/mapped_convolution_layer.cpp:8-132 ---------------------- */
void SUF(oracle_conv_fwd)(const T* x, const T* map, const T* iw, const T* w, const T* bias, T* y,
                          int B, int Cin, int Cout, int IH, int IW, int OH, int OW, int K, int P,
                          int mode) {
  const int64_t np = (int64_t)OH * OW, R = (int64_t)Cin * K;
  T* col = (T*)malloc(sizeof(T) * R * np);
  for (int b = 0; b < B; ++b) {
    SUF(im2col)(x + (int64_t)b * Cin * IH * IW, map, iw, Cin, IH, IW, np, K, P, mode, col);
    T* yb = y + (int64_t)b * Cout * np;
    SUF(gemm)(0, 0, Cout, np, R, w, col, yb, 0);
    if (bias)
      for (int64_t c = 0; c < Cout; ++c)
        for (int64_t p = 0; p < np; ++p) yb[c * np + p] += bias[c];
  }
  free(col);
}

void SUF(oracle_conv_dgrad)(const T* gy, const T* map, const T* iw, const T* w, T* gx, int B,
                            int Cin, int Cout, int IH, int IW, int OH, int OW, int K, int P,
                            int mode) {
  const int64_t np = (int64_t)OH * OW, R = (int64_t)Cin * K;
  T* col = (T*)malloc(sizeof(T) * R * np);
  memset(gx, 0, sizeof(T) * (size_t)B * Cin * IH * IW);
  for (int b = 0; b < B; ++b) {
    SUF(gemm)(1, 0, R, np, Cout, w, gy + (int64_t)b * Cout * np, col, 0);
    SUF(col2im)(col, map, iw, Cin, IH, IW, np, K, P, mode, gx + (int64_t)b * Cin * IH * IW);
  }
  free(col);
}

void SUF(oracle_conv_wgrad)(const T* gy, const T* x, const T* map, const T* iw, T* gw, T* gb, int B,
                            int Cin, int Cout, int IH, int IW, int OH, int OW, int K, int P,
                            int mode) {
  const int64_t np = (int64_t)OH * OW, R = (int64_t)Cin * K;
  T* col = (T*)malloc(sizeof(T) * R * np);
  memset(gw, 0, sizeof(T) * (size_t)Cout * R);
  for (int b = 0; b < B; ++b) {
    SUF(im2col)(x + (int64_t)b * Cin * IH * IW, map, iw, Cin, IH, IW, np, K, P, mode, col);
    SUF(gemm)(0, 1, Cout, R, np, gy + (int64_t)b * Cout * np, col, gw, 1);
  }
  if (gb) /* grad_output.sum({0,2,3}): include/nn/layers/mapped_convolution_layer.h:113 */
    for (int c = 0; c < Cout; ++c) {
      T s = (T)0;
      for (int b = 0; b < B; ++b)
        for (int64_t p = 0; p < np; ++p) s += gy[((int64_t)b * Cout + c) * np + p];
      gb[c] = s;
    }
  free(col);
}

/* ---- mapped transposed convolution: src/nn/cpp/mapped_transposed_convolution_layer.cpp:8-131 --
 * x (B,Cin,H,W) on the map grid; w (Cin,Cout,K); output (B,Cout,OH,OW) is what the map points into. */
void SUF(oracle_tconv_fwd)(const T* x, const T* map, const T* iw, const T* w, const T* bias, T* y,
                           int B, int Cin, int Cout, int H, int W, int OH, int OW, int K, int P,
                           int mode) {
  const int64_t np = (int64_t)H * W, R = (int64_t)Cout * K, no = (int64_t)OH * OW;
  T* col = (T*)malloc(sizeof(T) * R * np);
  memset(y, 0, sizeof(T) * (size_t)B * Cout * no);
  for (int b = 0; b < B; ++b) {
    T* yb = y + (int64_t)b * Cout * no;
    SUF(gemm)(1, 0, R, np, Cin, w, x + (int64_t)b * Cin * np, col, 0);
    SUF(col2im)(col, map, iw, Cout, OH, OW, np, K, P, mode, yb);
    if (bias)
      for (int64_t c = 0; c < Cout; ++c)
        for (int64_t p = 0; p < no; ++p) yb[c * no + p] += bias[c];
  }
  free(col);
}

void SUF(oracle_tconv_dgrad)(const T* gy, const T* map, const T* iw, const T* w, T* gx, int B,
                             int Cin, int Cout, int H, int W, int OH, int OW, int K, int P,
                             int mode) {
  const int64_t np = (int64_t)H * W, R = (int64_t)Cout * K, no = (int64_t)OH * OW;
  T* col = (T*)malloc(sizeof(T) * R * np);
  for (int b = 0; b < B; ++b) {
    SUF(im2col)(gy + (int64_t)b * Cout * no, map, iw, Cout, OH, OW, np, K, P, mode, col);
    SUF(gemm)(0, 0, Cin, np, R, w, col, gx + (int64_t)b * Cin * np, 0);
  }
  free(col);
}

void SUF(oracle_tconv_wgrad)(const T* gy, const T* x, const T* map, const T* iw, T* gw, T* gb,
                             int B, int Cin, int Cout, int H, int W, int OH, int OW, int K, int P,
                             int mode) {
  const int64_t np = (int64_t)H * W, R = (int64_t)Cout * K, no = (int64_t)OH * OW;
  T* col = (T*)malloc(sizeof(T) * R * np);
  memset(gw, 0, sizeof(T) * (size_t)Cin * R);
  for (int b = 0; b < B; ++b) {
    SUF(im2col)(gy + (int64_t)b * Cout * no, map, iw, Cout, OH, OW, np, K, P, mode, col);
    SUF(gemm)(0, 1, Cin, R, np, x + (int64_t)b * Cin * np, col, gw, 1);
  }
  if (gb)
    for (int c = 0; c < Cout; ++c) {
      T s = (T)0;
      for (int b = 0; b < B; ++b)
        for (int64_t p = 0; p < no; ++p) s += gy[((int64_t)b * Cout + c) * no + p];
      gb[c] = s;
    }
  free(col);
}

/* ---- pooling: include/nn/common/mapped_max_pool.h, mapped_avg_pool.h --------------------------
 * cuda_init != 0 selects the start value of the reference's CUDA build (-FLT_MAX, :29); 0 selects
 * its CPU build (numeric_limits<T>::min(), the smallest positive normal, :31). */
void SUF(oracle_max_pool)(const T* x, const T* map, const T* iw, T* y, int64_t* idx, int B, int C,
                          int IH, int IW, int OH, int OW, int K, int P, int mode, int cuda_init) {
  const int64_t np = (int64_t)OH * OW, ni = (int64_t)IH * IW;
  const int pp = P ? P : 1;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < (int64_t)B * C * np; ++i) {
    const int64_t p = i % np, bc = i / np;
    T best = cuda_init ? (T)(-FLT_MAX) : (T)TMIN;
    int64_t bi = -1;
    for (int k = 0; k < K; ++k) {
      const int64_t e = (p * K + k) * pp;
      const T v = SUF(tap_get)(x + bc * ni, IH, IW, map + 2 * e, iw ? iw + e : 0, P, mode);
      if (v > best) { best = v; bi = 2 * e; }
    }
    y[i] = best;
    idx[i] = bi;
  }
}

void SUF(oracle_max_unpool)(const T* gy, const int64_t* idx, const T* map, const T* iw, T* gx, int B,
                            int C, int IH, int IW, int OH, int OW, int K, int P, int mode) {
  const int64_t np = (int64_t)OH * OW, ni = (int64_t)IH * IW;
  (void)K;
  memset(gx, 0, sizeof(T) * (size_t)B * C * ni);
#pragma omp parallel for schedule(static)
  for (int64_t bc = 0; bc < (int64_t)B * C; ++bc)
    for (int64_t p = 0; p < np; ++p) {
      const int64_t off = (int64_t)(int)idx[bc * np + p];
      if (off < 0) continue;
      SUF(tap_put)(gx + bc * ni, IH, IW, map + off, iw ? iw + off / 2 : 0, P, mode, gy[bc * np + p]);
    }
}

void SUF(oracle_avg_pool)(const T* x, const T* map, const T* iw, T* y, int B, int C, int IH, int IW,
                          int OH, int OW, int K, int P, int mode) {
  const int64_t np = (int64_t)OH * OW, ni = (int64_t)IH * IW;
  const int pp = P ? P : 1;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < (int64_t)B * C * np; ++i) {
    const int64_t p = i % np, bc = i / np;
    T acc = (T)0;
    for (int k = 0; k < K; ++k) {
      const int64_t e = (p * K + k) * pp;
      acc += SUF(tap_get)(x + bc * ni, IH, IW, map + 2 * e, iw ? iw + e : 0, P, mode);
    }
    y[i] = acc / K;
  }
}

void SUF(oracle_avg_unpool)(const T* gy, const T* map, const T* iw, T* gx, int B, int C, int IH,
                            int IW, int OH, int OW, int K, int P, int mode) {
  const int64_t np = (int64_t)OH * OW, ni = (int64_t)IH * IW;
  const int pp = P ? P : 1;
  memset(gx, 0, sizeof(T) * (size_t)B * C * ni);
#pragma omp parallel for schedule(static)
  for (int64_t bc = 0; bc < (int64_t)B * C; ++bc)
    for (int64_t p = 0; p < np; ++p) {
      const T v = gy[bc * np + p] / K;
      for (int k = 0; k < K; ++k) {
        const int64_t e = (p * K + k) * pp;
        SUF(tap_put)(gx + bc * ni, IH, IW, map + 2 * e, iw ? iw + e : 0, P, mode, v);
      }
    }
}

/* ---- resample: include/nn/common/resample.h:11-103 -------------------------------------------
 * gather : y (B,C,OH,OW)[p] = interp(x (B,C,IH,IW), map (OH,OW,[P,]2)[p])      ("Unresample")
 * scatter: y (B,C,IH,IW)   += extrap(x (B,C,OH,OW)[q], map (OH,OW,[P,]2)[q])   ("Resample") */
void SUF(oracle_resample_gather)(const T* x, const T* map, const T* iw, T* y, int B, int C, int IH,
                                 int IW, int OH, int OW, int P, int mode) {
  SUF(oracle_avg_pool)(x, map, iw, y, B, C, IH, IW, OH, OW, 1, P, mode);
}
void SUF(oracle_resample_scatter)(const T* x, const T* map, const T* iw, T* y, int B, int C, int IH,
                                  int IW, int OH, int OW, int P, int mode) {
  SUF(oracle_avg_unpool)(x, map, iw, y, B, C, IH, IW, OH, OW, 1, P, mode);
}
