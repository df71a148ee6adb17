// C-ABI entry points of the convolution family: argument checks and the choice between the
// tensor-core (tcgen05) kernels and the generic CUDA-core kernels.
#include "common.cuh"

namespace mc {
int check_conv_desc_public(const mc_desc* d);
int conv_fwd_simt_launch(const mc_desc*, const void*, const void*, const void*, const void*,
                         const void*, void*, cudaStream_t);
size_t conv_dgrad_simt_ws(const mc_desc*);
int conv_dgrad_simt_launch(const mc_desc*, const void*, const void*, const void*, const void*,
                           const void*, void*, void*, size_t, cudaStream_t);
int conv_wgrad_simt_launch(const mc_desc*, const void*, const void*, const void*, const void*, void*,
                           cudaStream_t);
int bias_grad_launch(const mc_desc*, const void*, void*, cudaStream_t);

// Tensor-core path (conv_tc.cu).  Each returns MC_ERR_UNSUPPORTED when the shape is not one it
// takes, in which case the generic kernel runs instead.
bool conv_tc_fwd_supported(const mc_desc*);
size_t conv_tc_fwd_ws(const mc_desc*);
int conv_tc_fwd_launch(const mc_desc*, const void*, const void*, const void*, const void*, void*,
                       void*, size_t, cudaStream_t);
int device_status_read(cudaStream_t, int);
bool conv_tc_dgrad_supported(const mc_desc*);
size_t conv_tc_dgrad_ws(const mc_desc*);
int conv_tc_dgrad_launch(const mc_desc*, const void*, const void*, const void*, const void*, void*,
                         void*, size_t, cudaStream_t);
size_t tapmap_bytes(const mc_desc*);
int tapmap_build_launch(const mc_desc*, const void*, void*, cudaStream_t);
int conv_tc_wgrad_tab_relu_launch(const mc_desc*, const void*, const void*, const void*, const void*, void*, void*,
                                  cudaStream_t);
int conv_tc_fwd_tab_launch(const mc_desc*, const void*, const void*, const void*, const void*, void*,
                           void*, size_t, cudaStream_t);
int conv_tc_wgrad_tab_launch(const mc_desc*, const void*, const void*, const void*, void*, void*,
                             cudaStream_t);
bool invmap_supported(const mc_desc*);
size_t invmap_off_bytes(const mc_desc*);
int scatter_inv_launch(const mc_desc*, const void*, const void*, size_t, void*, int, cudaStream_t);
int tap_gather_sum_launch(const mc_desc*, const void*, const void*, size_t, void*, cudaStream_t);
size_t invmap_bytes(const mc_desc*);
size_t invmap_build_ws(const mc_desc*);
int invmap_build_launch(const mc_desc*, const void*, const void*, void*, void*, size_t, cudaStream_t);
bool weighted_fold(const mc_desc*, mc_desc*);
int tapmap_build_weighted_launch(const mc_desc*, const void*, const void*, void*, cudaStream_t);
bool conv_tc_wgrad_supported(const mc_desc*);
size_t conv_tc_wgrad_ws(const mc_desc*);
int conv_tc_wgrad_launch(const mc_desc*, const void*, const void*, const void*, void*, void*, void*,
                         size_t, cudaStream_t);
bool conv_rowinv_shape_ok(const mc_desc*);
size_t rowinv_analysis_bytes(const mc_desc*);
int rowinv_analyse_launch(const mc_desc*, const void*, void*, cudaStream_t);
long rowinv_assemble_host(const mc_desc*, const double*, const float*, int*, long);
size_t rowinv_ws_bytes(const mc_desc*, const void*, int);
int rowinv_conv_launch(const mc_desc*, int, const void*, const void*, const void*, const void*,
                       const void*, void*, void*, size_t, cudaStream_t);
size_t rowinv_wgrad_ws_bytes(const mc_desc*, const void*);
int rowinv_wgrad_launch(const mc_desc*, const void*, const void*, const void*, const void*, void*,
                        void*, void*, size_t, cudaStream_t);
}  // namespace mc

namespace mc {
std::atomic<unsigned long long> g_launches{0};
}
using namespace mc;

extern "C" {

int mc_abi_version(void) { return 2; }

uint64_t mc_kernel_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

const char* mc_strerror(int code) {
  switch (code) {
    case MC_OK: return "ok";
    case MC_ERR_BAD_ARG: return "bad argument (null pointer, non-positive size or unknown enum)";
    case MC_ERR_UNSUPPORTED: return "unsupported configuration";
    case MC_ERR_WORKSPACE: return "workspace missing or too small";
    case MC_ERR_LAUNCH: return "CUDA launch or runtime error";
    case MC_ERR_DEVICE: return "device-side status word raised (bounded wait ran out)";
    case MC_ERR_TOO_LARGE: return "size beyond a fixed limit of this entry point";
    default: return "unknown error code";
  }
}

// ---- conv ----------------------------------------------------------------------------------

int mc_device_status(void* stream, int reset) {
  return device_status_read((cudaStream_t)stream, reset);
}

size_t mc_conv_fwd_workspace_bytes(const mc_desc* d) {
  if (!d || check_conv_desc_public(d)) return 0;
  return conv_tc_fwd_supported(d) ? conv_tc_fwd_ws(d) : 0;
}

int mc_conv_fwd(const mc_desc* d, const void* x, const void* map, const void* iw, const void* w,
                const void* bias, void* y, void* ws, size_t ws_bytes, void* stream) {
  int rc = check_conv_desc_public(d);
  if (rc) return rc;
  if (!x || !map || !w || !y || (d->P > 0 && !iw)) return MC_ERR_BAD_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  if (conv_tc_fwd_supported(d)) return conv_tc_fwd_launch(d, x, map, w, bias, y, ws, ws_bytes, st);
  return conv_fwd_simt_launch(d, x, map, iw, w, bias, y, st);
}

size_t mc_conv_dgrad_workspace_bytes(const mc_desc* d) {
  if (!d || check_conv_desc_public(d)) return 0;
  return conv_dgrad_simt_ws(d);
}

// ---- prebuilt forward tap table ------------------------------------------------------------------

size_t mc_tapmap_bytes(const mc_desc* d) {
  if (!d || check_conv_desc_public(d)) return 0;
  return (conv_tc_fwd_supported(d) || conv_tc_wgrad_supported(d)) ? tapmap_bytes(d) : 0;
}
int mc_tapmap_build(const mc_desc* d, const void* map, void* tapmap, size_t tapmap_bytes_, void* stream) {
  int rc = check_conv_desc_public(d);
  if (rc) return rc;
  if (!map || !tapmap) return MC_ERR_BAD_ARG;
  if (d->P != 0 || d->dtype == MC_F64) return MC_ERR_UNSUPPORTED;
  if (tapmap_bytes_ < tapmap_bytes(d)) return MC_ERR_WORKSPACE;
  return tapmap_build_launch(d, map, tapmap, (cudaStream_t)stream);
}
int mc_conv_fwd_tap(const mc_desc* d, const void* x, const void* tapmap, const void* w,
                    const void* bias, void* y, void* ws, size_t ws_bytes, void* stream) {
  int rc = check_conv_desc_public(d);
  if (rc) return rc;
  if (!x || !tapmap || !w || !y) return MC_ERR_BAD_ARG;
  if (!conv_tc_fwd_supported(d)) return MC_ERR_UNSUPPORTED;
  return conv_tc_fwd_tab_launch(d, x, tapmap, w, bias, y, ws, ws_bytes, (cudaStream_t)stream);
}
int mc_conv_wgrad_tap(const mc_desc* d, const void* gy, const void* x, const void* tapmap, void* gw,
                      void* gb, void* stream) {
  int rc = check_conv_desc_public(d);
  if (rc) return rc;
  if (!gy || !x || !tapmap || !gw) return MC_ERR_BAD_ARG;
  if (!conv_tc_wgrad_supported(d)) return MC_ERR_UNSUPPORTED;
  return conv_tc_wgrad_tab_launch(d, gy, x, tapmap, gw, gb, (cudaStream_t)stream);
}
int mc_conv_wgrad_tap_relu(const mc_desc* d, const void* gy, const void* y, const void* x, const void* tapmap,
                           void* gw, void* gb, void* stream) {
  int rc = check_conv_desc_public(d);
  if (rc) return rc;
  if (!gy || !y || !x || !tapmap || !gw) return MC_ERR_BAD_ARG;
  if (!conv_tc_wgrad_supported(d)) return MC_ERR_UNSUPPORTED;
  return conv_tc_wgrad_tab_relu_launch(d, gy, y, x, tapmap, gw, gb, (cudaStream_t)stream);
}

// ---- inverse map and the gather-form dgrad ---------------------------------------------------

size_t mc_invmap_bytes(const mc_desc* d) {
  if (!d || check_conv_desc_public(d) || !invmap_supported(d)) return 0;
  return invmap_bytes(d);
}
size_t mc_invmap_build_workspace_bytes(const mc_desc* d) {
  if (!d || check_conv_desc_public(d) || !invmap_supported(d)) return 0;
  return invmap_build_ws(d);
}
int mc_invmap_build(const mc_desc* d, const void* map, void* inv, size_t inv_bytes, void* ws,
                    size_t ws_bytes, void* stream) {
  int rc = check_conv_desc_public(d);
  if (rc) return rc;
  if (!map || !inv) return MC_ERR_BAD_ARG;
  if (!invmap_supported(d)) return MC_ERR_UNSUPPORTED;
  if (inv_bytes < invmap_bytes(d)) return MC_ERR_WORKSPACE;
  return invmap_build_launch(d, map, nullptr, inv, ws, ws_bytes, (cudaStream_t)stream);
}

// ---- plans of weighted maps ------------------------------------------------------------------------
int mc_weighted_plan_desc(const mc_desc* d, mc_desc* folded) {
  int rc = check_conv_desc_public(d);
  if (rc) return rc;
  if (!folded) return MC_ERR_BAD_ARG;
  if (d->dtype == MC_F64 || !weighted_fold(d, folded)) return MC_ERR_UNSUPPORTED;
  return MC_OK;
}
int mc_tapmap_build_weighted(const mc_desc* d, const void* map, const void* iw, void* tapmap,
                             size_t tapmap_bytes_, void* stream) {
  mc_desc f;
  int rc = mc_weighted_plan_desc(d, &f);
  if (rc) return rc;
  if (!map || !iw || !tapmap) return MC_ERR_BAD_ARG;
  if (mc_tapmap_bytes(&f) == 0) return MC_ERR_UNSUPPORTED;
  if (tapmap_bytes_ < tapmap_bytes(&f)) return MC_ERR_WORKSPACE;
  return tapmap_build_weighted_launch(d, map, iw, tapmap, (cudaStream_t)stream);
}
int mc_invmap_build_weighted(const mc_desc* d, const void* map, const void* iw, void* inv, size_t inv_bytes,
                             void* ws, size_t ws_bytes, void* stream) {
  mc_desc f;
  int rc = mc_weighted_plan_desc(d, &f);
  if (rc) return rc;
  if (!map || !iw || !inv) return MC_ERR_BAD_ARG;
  if (!invmap_supported(&f)) return MC_ERR_UNSUPPORTED;
  if (inv_bytes < invmap_bytes(&f)) return MC_ERR_WORKSPACE;
  return invmap_build_launch(d, map, iw, inv, ws, ws_bytes, (cudaStream_t)stream);
}
// adjoint ops (average unpooling, resample scatter) as gathers through the inverse map
static int scatter_inv_check(const mc_desc* d, const void* a, const void* b, const void* c) {
  if (!d || d->B <= 0 || d->C_in <= 0 || d->IH <= 0 || d->IW <= 0 || d->OH <= 0 || d->OW <= 0 ||
      d->K <= 0 || !a || !b || !c)
    return MC_ERR_BAD_ARG;
  mc_desc t = *d;
  t.C_out = t.C_in;
  int rc = check_conv_desc_public(&t);
  if (rc) return rc;
  return invmap_supported(&t) ? MC_OK : MC_ERR_UNSUPPORTED;
}
int mc_pool_avg_bwd_inv(const mc_desc* d, const void* gy, const void* inv, void* gx, void* stream) {
  int rc = scatter_inv_check(d, gy, inv, gx);
  if (rc) return rc;
  return scatter_inv_launch(d, gy, inv, invmap_off_bytes(d), gx, 1, (cudaStream_t)stream);
}
int mc_conv_dgrad_tapsum(const mc_desc* d, const void* z, const void* inv, void* gx, void* stream) {
  if (!d || !z || !inv || !gx) return MC_ERR_BAD_ARG;
  if (mc_invmap_bytes(d) == 0) return MC_ERR_UNSUPPORTED;
  return tap_gather_sum_launch(d, z, inv, invmap_off_bytes(d), gx, (cudaStream_t)stream);
}
int mc_resample_scatter_inv(const mc_desc* d, const void* x, const void* inv, void* y, void* stream) {
  int rc = scatter_inv_check(d, x, inv, y);
  if (rc) return rc;
  if (d->K != 1) return MC_ERR_BAD_ARG;
  return scatter_inv_launch(d, x, inv, invmap_off_bytes(d), y, 0, (cudaStream_t)stream);
}

int mc_conv_dgrad_inv_supported(const mc_desc* d) {
  return d && !check_conv_desc_public(d) && conv_tc_dgrad_supported(d) ? 1 : 0;
}
size_t mc_conv_dgrad_inv_workspace_bytes(const mc_desc* d) {
  return mc_conv_dgrad_inv_supported(d) ? conv_tc_dgrad_ws(d) : 0;
}
int mc_conv_dgrad_inv(const mc_desc* d, const void* gy, const void* inv, const void* w,
                      const void* bias_out, void* gx, void* ws, size_t ws_bytes, void* stream) {
  int rc = check_conv_desc_public(d);
  if (rc) return rc;
  if (!gy || !inv || !w || !gx) return MC_ERR_BAD_ARG;
  if (!conv_tc_dgrad_supported(d)) return MC_ERR_UNSUPPORTED;
  return conv_tc_dgrad_launch(d, gy, inv, w, bias_out, gx, ws, ws_bytes, (cudaStream_t)stream);
}

// ---- row-invariant maps --------------------------------------------------------------------------

size_t mc_rowplan_analysis_bytes(const mc_desc* d) {
  if (!d || check_conv_desc_public(d) || !conv_rowinv_shape_ok(d)) return 0;
  return rowinv_analysis_bytes(d);
}
int mc_rowplan_analyse(const mc_desc* d, const void* map, void* analysis, void* stream) {
  int rc = check_conv_desc_public(d);
  if (rc) return rc;
  if (!map || !analysis) return MC_ERR_BAD_ARG;
  if (!conv_rowinv_shape_ok(d)) return MC_ERR_UNSUPPORTED;
  return rowinv_analyse_launch(d, map, analysis, (cudaStream_t)stream);
}
int64_t mc_rowplan_assemble(const mc_desc* d, const double* analysis_host, const float* map_host,
                            int32_t* plan_host, int64_t capacity) {
  if (!d || check_conv_desc_public(d) || !analysis_host || !map_host) return 0;
  return rowinv_assemble_host(d, analysis_host, map_host, plan_host, capacity);
}
size_t mc_conv_rowplan_workspace_bytes(const mc_desc* d, const void* plan_host, int32_t dir) {
  if (!d || check_conv_desc_public(d) || !plan_host || dir < 0 || dir > 1) return 0;
  return rowinv_ws_bytes(d, plan_host, dir);
}
int mc_conv_fwd_rowplan(const mc_desc* d, const void* x, const void* plan_host, const void* plan_dev,
                        const void* w, const void* bias, void* y, void* ws, size_t ws_bytes,
                        void* stream) {
  int rc = check_conv_desc_public(d);
  if (rc) return rc;
  if (!x || !plan_host || !plan_dev || !w || !y) return MC_ERR_BAD_ARG;
  return rowinv_conv_launch(d, 0, x, plan_host, plan_dev, w, bias, y, ws, ws_bytes, (cudaStream_t)stream);
}
int mc_conv_dgrad_rowplan(const mc_desc* d, const void* gy, const void* plan_host,
                          const void* plan_dev, const void* w, const void* bias_out, void* gx,
                          void* ws, size_t ws_bytes, void* stream) {
  int rc = check_conv_desc_public(d);
  if (rc) return rc;
  if (!gy || !plan_host || !plan_dev || !w || !gx) return MC_ERR_BAD_ARG;
  return rowinv_conv_launch(d, 1, gy, plan_host, plan_dev, w, bias_out, gx, ws, ws_bytes,
                            (cudaStream_t)stream);
}

size_t mc_conv_wgrad_rowplan_workspace_bytes(const mc_desc* d, const void* plan_host) {
  if (!d || check_conv_desc_public(d) || !plan_host) return 0;
  return rowinv_wgrad_ws_bytes(d, plan_host);
}
int mc_conv_wgrad_rowplan(const mc_desc* d, const void* gy, const void* x, const void* plan_host,
                          const void* plan_dev, void* gw, void* gb, void* ws, size_t ws_bytes,
                          void* stream) {
  int rc = check_conv_desc_public(d);
  if (rc) return rc;
  if (!gy || !x || !plan_host || !plan_dev || !gw) return MC_ERR_BAD_ARG;
  return rowinv_wgrad_launch(d, gy, x, plan_host, plan_dev, gw, gb, ws, ws_bytes, (cudaStream_t)stream);
}

int mc_conv_dgrad(const mc_desc* d, const void* gy, const void* map, const void* iw, const void* w,
                  const void* bias_out, void* gx, void* ws, size_t ws_bytes, void* stream) {
  int rc = check_conv_desc_public(d);
  if (rc) return rc;
  if (!gy || !map || !w || !gx || (d->P > 0 && !iw)) return MC_ERR_BAD_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  return conv_dgrad_simt_launch(d, gy, map, iw, w, bias_out, gx, ws, ws_bytes, st);
}

size_t mc_conv_wgrad_workspace_bytes(const mc_desc* d) {
  if (!d) return 0;
  if (conv_tc_wgrad_supported(d)) return conv_tc_wgrad_ws(d);
  return 0;
}

int mc_conv_wgrad(const mc_desc* d, const void* gy, const void* x, const void* map, const void* iw,
                  void* gw, void* gb, void* ws, size_t ws_bytes, void* stream) {
  int rc = check_conv_desc_public(d);
  if (rc) return rc;
  if (!gy || !x || !map || !gw || (d->P > 0 && !iw)) return MC_ERR_BAD_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  if (conv_tc_wgrad_supported(d)) return conv_tc_wgrad_launch(d, gy, x, map, gw, gb, ws, ws_bytes, st);
  rc = conv_wgrad_simt_launch(d, gy, x, map, iw, gw, st);
  if (rc) return rc;
  if (gb) rc = bias_grad_launch(d, gy, gb, st);
  return rc;
}

int mc_bias_grad(const mc_desc* d, const void* gy, void* gb, void* stream) {
  int rc = check_conv_desc_public(d);
  if (rc) return rc;
  if (!gy || !gb) return MC_ERR_BAD_ARG;
  return bias_grad_launch(d, gy, gb, (cudaStream_t)stream);
}

// ---- transposed conv: the same three primitives with the roles of the tensors swapped --------
// (design note of the reference: src/nn/cuda/mapped_transposed_convolution_layer.cu:17-51)

static mc_desc swap_roles(const mc_desc* d) {
  mc_desc s = *d;
  s.C_in = d->C_out;  // the image that is sampled / scattered into has the layer's output channels
  s.C_out = d->C_in;  // the tensor living on the map grid has the layer's input channels
  return s;
}

size_t mc_tconv_workspace_bytes(const mc_desc* d) {
  if (!d) return 0;
  mc_desc s = swap_roles(d);
  size_t a = mc_conv_dgrad_workspace_bytes(&s), b = mc_conv_wgrad_workspace_bytes(&s);
  const size_t c = mc_conv_fwd_workspace_bytes(&s);  // the transposed layer's dgrad is a forward
  if (b > a) a = b;
  return c > a ? c : a;
}

int mc_tconv_fwd(const mc_desc* d, const void* x, const void* map, const void* iw, const void* w,
                 const void* bias, void* y, void* ws, size_t ws_bytes, void* stream) {
  if (!d) return MC_ERR_BAD_ARG;
  mc_desc s = swap_roles(d);
  // y = col2im(W.view(C_in, C_out*K)^T . x) + bias  == dgrad of a conv whose weight is W
  return mc_conv_dgrad(&s, x, map, iw, w, bias, y, ws, ws_bytes, stream);
}

int mc_tconv_dgrad(const mc_desc* d, const void* gy, const void* map, const void* iw,
                   const void* w, void* gx, void* ws, size_t ws_bytes, void* stream) {
  if (!d) return MC_ERR_BAD_ARG;
  mc_desc s = swap_roles(d);
  // gx = W.view(C_in, C_out*K) . im2col(gy)  == forward of that conv applied to gy, no bias
  return mc_conv_fwd(&s, gy, map, iw, w, nullptr, gx, ws, ws_bytes, stream);
}

int mc_tconv_wgrad(const mc_desc* d, const void* gy, const void* x, const void* map,
                   const void* iw, void* gw, void* gb, void* ws, size_t ws_bytes, void* stream) {
  if (!d) return MC_ERR_BAD_ARG;
  mc_desc s = swap_roles(d);
  // gw(C_in, C_out, K) = sum_b x_b . im2col(gy_b)^T : wgrad with x on the grid and gy sampled
  int rc = mc_conv_wgrad(&s, x, gy, map, iw, gw, nullptr, ws, ws_bytes, stream);
  if (rc || !gb) return rc;
  // bias gradient = gy summed over batch and pixels; gy lives on the (IH, IW) image here
  mc_desc b = *d;
  b.OH = d->IH; b.OW = d->IW;
  return bias_grad_launch(&b, gy, gb, (cudaStream_t)stream);
}

}  // extern "C"
