/*
 * mc_b200.h - C ABI of the sm_100a mapped-convolution kernels.
 *
 * Every entry point replaces one device-side driver of the reference project
 * (meder411/MappedConvolutions); the reference file:line each one stands in for is cited
 * beside its declaration (paths relative to package/ext_modules/).
 *
 * Conventions
 *  - plain pointers and sizes only; all pointers are device pointers on the current CUDA device;
 *  - every call is asynchronous on `stream` (a cudaStream_t passed as void*; NULL = legacy
 *    default stream) and allocates nothing: outputs and scratch are provided by the caller;
 *  - return value: MC_OK (0) or a negative MC_ERR_* code; mc_strerror() gives the text;
 *    nothing throws, prints or exits;
 *  - activations are (B, C, H, W) tensors; `layout` says how they lie in memory:
 *    MC_NCHW (the reference's contiguous layout) or MC_NHWC (channels innermost);
 *  - sample maps / interpolation weights keep the reference's layout:
 *    map (OH, OW, K, [P,] 2) with (x, y) pairs, weights (OH, OW, K, P); their scalar type is
 *    double when dtype == MC_F64 and float otherwise (also for MC_BF16 activations);
 *  - interp: 0 nearest, 1 bilinear, 2 bispherical (x wraps), any other value = nearest
 *    (include/core/resample.h:45-58);
 *  - alignment: the bf16 tensor-core paths (MC_BF16 + MC_NHWC, C_out % 64 == 0, every *_tap, *_inv and
 *    *_rowplan entry point, mc_conv_fwd_static_scratch) move 16 bytes at a time and return
 *    MC_ERR_BAD_ARG for a tensor, map, table or workspace pointer that is not 16-byte aligned; the
 *    generic kernels take any element-aligned pointer;
 *  - finite inputs: the bf16 tensor-core kernels gather without predicates - a corner or tap that
 *    contributes nothing still reads a real pixel (pixel 0 of the image for a tap that lies outside
 *    it completely) and multiplies it by zero.  The reference skips such corners
 *    (include/core/interpolation.h:125-154); results agree for finite inputs, a NaN or infinity
 *    in such a pixel reaches the output here.
 */
#ifndef MC_B200_H_
#define MC_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { MC_F32 = 0, MC_F64 = 1, MC_BF16 = 2 };
enum { MC_NCHW = 0, MC_NHWC = 1 };

enum {
  MC_OK = 0,
  MC_ERR_BAD_ARG = -1,      /* null pointer, non-positive size, unknown enum */
  MC_ERR_UNSUPPORTED = -2,  /* valid request this build has no kernel for */
  MC_ERR_WORKSPACE = -3,    /* scratch buffer missing or too small */
  MC_ERR_LAUNCH = -4,       /* CUDA reported a launch / runtime error */
  MC_ERR_DEVICE = -5,       /* kernel raised its device status word (bounded wait ran out) */
  MC_ERR_TOO_LARGE = -6     /* size beyond a documented fixed limit */
};

/* Problem description shared by the conv / pool / resample entry points.
 * B batch; C_in/C_out channels (pool and resample use C_in only);
 * (IH, IW) size of the image that is *sampled*; (OH, OW) size of the map grid;
 * K taps per map location (1 for resample); P interpolation points per tap, 0 = unweighted map. */
typedef struct mc_desc {
  int32_t B, C_in, C_out;
  int32_t IH, IW, OH, OW;
  int32_t K, P;
  int32_t interp;
  int32_t dtype;  /* MC_F32 / MC_F64 / MC_BF16 */
  int32_t layout; /* MC_NCHW / MC_NHWC, applies to every activation tensor of the call */
  int32_t flags;  /* MC_FLAG_* bits, 0 = the reference's behaviour */
} mc_desc;

/* mc_conv_fwd / mc_conv_fwd_tap / mc_tconv_fwd: y = max(0, W . im2col(x) + bias), the activation
 * applied in the kernel's epilogue (the reference leaves ReLU to a separate element-wise pass over
 * y).  Its gradient is taken before the backward entry points: gz = gy where y > 0, else 0.
 * Entry points that do not produce a layer output ignore the flag; the row-plan kernels refuse it
 * (MC_ERR_UNSUPPORTED). */
enum { MC_FLAG_RELU = 1 };

const char* mc_strerror(int code);
/* ABI version, bumped on any change of a signature or of mc_desc (2: mc_desc.flags, row plans). */
int mc_abi_version(void);
/* Diagnostic: kernels launched by this library so far in this process (no counterpart in the
 * reference; used by the benchmark to report its launch count). */
uint64_t mc_kernel_launch_count(void);

/* Synchronises `stream` and returns the device status word: 0, or the code of the first bounded
 * device-side wait that ran out (the kernel then returned early and its output is invalid).
 * reset != 0 clears the word.  No counterpart in the reference (its kernels have no waits). */
int mc_device_status(void* stream, int reset);

/* Self-test of the bounded device-side waits: launches a one-warp kernel that waits about a
 * millisecond on a barrier nobody arrives at.  The wait gives up, the kernel returns, and
 * mc_device_status() then reports 0x7F1; observed_dev (one int32 in device memory, may be NULL)
 * receives 2 (the block's abort flag was raised and the wait reported failure).  Nothing faults or
 * hangs.  No counterpart in the reference. */
int mc_selftest_wait_expiry(int32_t* observed_dev, void* stream);

/* ---- mapped convolution ---------------------------------------------------------------
 * weight (C_out, C_in, K) and bias (C_out) in `dtype`, contiguous. */

/* y(B,C_out,OH,OW) = W . im2col_map(x) + bias.
 * Replaces cuda::MappedConvForward, src/nn/cuda/mapped_convolution_layer.cu:16-73
 * (weighted form: src/nn/cuda/weighted_mapped_convolution_layer.cu:16-75). bias may be NULL. */
int mc_conv_fwd(const mc_desc* d, const void* x, const void* map, const void* iw, const void* w,
                const void* bias, void* y, void* ws, size_t ws_bytes, void* stream);
size_t mc_conv_fwd_workspace_bytes(const mc_desc* d);

/* mc_conv_fwd for callers that cannot hand over scratch memory.  (No counterpart in the
 * reference, whose drivers allocate their column buffer with torch on every call.)
 *
 * Who needs it: code that runs where the device allocator is off limits - a plugin called from
 * inside another framework's execution step, a serving loop whose memory was carved up once at
 * start-up, a real-time path in which cudaMalloc's implicit device synchronisation is not
 * acceptable.  Such callers own their input and output tensors but have no spare buffer, and
 * mc_conv_fwd's tensor-core path needs one for the weights re-laid-out for the MMA unit.
 *
 * Here that buffer is a fixed array in the library's device image
 * (mc_conv_fwd_static_scratch_limit() bytes, currently 80 KiB, resident on every GPU that loads the
 * library until the process exits).  The call allocates and frees nothing, and computes exactly
 * what mc_conv_fwd computes.
 *  - Supported: the configurations of the tensor-core forward (MC_BF16, MC_NHWC, P == 0,
 *    C_out % 64 == 0); anything else returns MC_ERR_UNSUPPORTED.
 *  - The scratch mc_conv_fwd would ask for (mc_conv_fwd_workspace_bytes: the re-laid-out weights,
 *    K * C_in * C_out * 2 bytes rounded up to whole 64-element slices, plus a tap table for the
 *    wide or very narrow layers that need one) must fit the array, otherwise MC_ERR_TOO_LARGE.
 *  - The first call on each device looks up the array's device address (with that device
 *    current); make that first call outside any stream capture.
 *  - All calls on a device share the one array: two calls whose kernels may overlap on the GPU
 *    (different streams, no ordering between them) race on it.  Calls on one stream are safe; the
 *    array is fully rewritten for the part a call uses, so nothing carries over between calls. */
size_t mc_conv_fwd_static_scratch_limit(void);
int mc_conv_fwd_static_scratch(const mc_desc* d, const void* x, const void* map, const void* w,
                               const void* bias, void* y, void* stream);

/* gx(B,C_in,IH,IW) = col2im_map(W^T . gy) [+ bias_out per channel of gx when bias_out != NULL,
 * which is how the transposed convolution forward uses it].
 * Replaces cuda::MappedConvBackwardInput, src/nn/cuda/mapped_convolution_layer.cu:75-132.
 * gx is fully written (no need to pre-zero). */
int mc_conv_dgrad(const mc_desc* d, const void* gy, const void* map, const void* iw, const void* w,
                  const void* bias_out, void* gx, void* ws, size_t ws_bytes, void* stream);
size_t mc_conv_dgrad_workspace_bytes(const mc_desc* d);

/* Tap table: the sample map decoded once - for every map entry the (up to four) source pixels and
 * interpolation weights, 32 bytes each (nearest maps: followed by a compact copy, one int per
 * entry - the buffer is opaque, size it with mc_tapmap_bytes()).  Like the inverse map below it depends only on the map and
 * the image size, so a layer builds it once and passes it to every forward / weight-gradient call;
 * the tensor-core kernels then stream it with bulk copies instead of decoding the map again for
 * every batch.  mc_tapmap_bytes() is 0 when the descriptor has no tensor-core path.
 * mc_conv_fwd_tap / mc_conv_wgrad_tap compute exactly what mc_conv_fwd / mc_conv_wgrad compute
 * (same reference drivers: src/nn/cuda/mapped_convolution_layer.cu:16-73, :134-193). */
size_t mc_tapmap_bytes(const mc_desc* d);
int mc_tapmap_build(const mc_desc* d, const void* map, void* tapmap, size_t tapmap_bytes, void* stream);
int mc_conv_fwd_tap(const mc_desc* d, const void* x, const void* tapmap, const void* w,
                    const void* bias, void* y, void* ws, size_t ws_bytes, void* stream);
int mc_conv_wgrad_tap(const mc_desc* d, const void* gy, const void* x, const void* tapmap, void* gw,
                      void* gb, void* stream);
/* The same for a layer with a fused ReLU: gy is the gradient behind the activation, y the layer's
 * output; the kernel uses gy where y > 0 and 0 elsewhere, so the caller needs no masked copy of gy.
 * Only where the weight gradient is one pass over gy in registers (nearest map, K * C_in + 1 <= 32:
 * a first layer with a handful of input channels); MC_ERR_UNSUPPORTED otherwise - mask gy and call
 * mc_conv_wgrad_tap. */
int mc_conv_wgrad_tap_relu(const mc_desc* d, const void* gy, const void* y, const void* x,
                           const void* tapmap, void* gw, void* gb, void* stream);

/* Inverse map: for every (input pixel, tap) the list of (grid pixel, weight) pairs whose forward
 * sample reads that input pixel.  It depends only on the sample map and the two image sizes, so
 * it is built once per map and reused by every backward pass.  With it the reference's atomic
 * col2im scatter (MappedCol2Im2DLauncher, include/nn/cuda/mapped_im2col.cuh:51-89) becomes a gather:
 * no atomics, and results that repeat bit for bit from run to run.
 * Unweighted maps only (d->P == 0).  mc_invmap_bytes() gives the size of the `inv` buffer
 * (0 = not supported for this descriptor). */
size_t mc_invmap_bytes(const mc_desc* d);
size_t mc_invmap_build_workspace_bytes(const mc_desc* d);
int mc_invmap_build(const mc_desc* d, const void* map, void* inv, size_t inv_bytes, void* ws,
                    size_t ws_bytes, void* stream);

/* Plans of WEIGHTED maps (d->P > 0: a tap is the sum over P points of interp_weight x sample,
 * include/core/resample.h:145-162; e.g. the three barycentric vertices of an icosphere tap).
 * When P x (corners per point: 1 for nearest, 4 for bilinear / bispherical) <= 4 the points of a tap
 * fit one tap-table record, and the map "folds": mc_weighted_plan_desc() fills *folded with the same
 * descriptor with P = 0 and interp = 1 (bilinear), the two builders below write a tap table and an
 * inverse map from (map, iw) in the layout of that folded descriptor (size the buffers with
 * mc_tapmap_bytes / mc_invmap_bytes / mc_invmap_build_workspace_bytes of *folded), and the caller
 * runs mc_conv_fwd_tap, mc_conv_wgrad_tap, mc_conv_dgrad_inv, mc_conv_dgrad_tapsum with *folded:
 * the bf16 tensor-core path of a weighted layer.  They compute what
 * WeightedMappedConvForward / Backward compute (src/nn/cuda/weighted_mapped_convolution_layer.cu:16-202).
 * MC_ERR_UNSUPPORTED: the map does not fold (or MC_F64). */
int mc_weighted_plan_desc(const mc_desc* d, mc_desc* folded);
int mc_tapmap_build_weighted(const mc_desc* d, const void* map, const void* iw, void* tapmap,
                             size_t tapmap_bytes, void* stream);
int mc_invmap_build_weighted(const mc_desc* d, const void* map, const void* iw, void* inv, size_t inv_bytes,
                             void* ws, size_t ws_bytes, void* stream);
/* Same result as mc_conv_dgrad, computed on the tensor cores from a prebuilt inverse map.
 * bf16, MC_NHWC, C_in % 64 == 0, C_out % 64 == 0 (mc_conv_dgrad_inv_supported() tells).
 * Replaces cuda::MappedConvBackwardInput, src/nn/cuda/mapped_convolution_layer.cu:75-132. */
int mc_conv_dgrad_inv_supported(const mc_desc* d);
size_t mc_conv_dgrad_inv_workspace_bytes(const mc_desc* d);
int mc_conv_dgrad_inv(const mc_desc* d, const void* gy, const void* inv, const void* w,
                      const void* bias_out, void* gx, void* ws, size_t ws_bytes, void* stream);
/* The same input gradient with the contraction done first - for layers with more output than input
 * channels.  The caller computes z (B, OH * OW, K * C_in) = grad_output, read as a (B * OH * OW, C_out)
 * matrix (channels-last), times the (C_out, K * C_in) matrix W'[co, k * C_in + ci] = w[co, ci, k] - one
 * dense GEMM, any GEMM routine - and this call sums the C_in-channel rows of z through the inverse map:
 * gx[b, q, ci] = sum_k sum_{(p, wt) in list(q, k)} wt * z[b, p, k * C_in + ci].  Every row of z is read
 * exactly once, where mc_conv_dgrad_inv gathers C_out-channel rows of grad_output.  bf16, MC_NHWC,
 * C_in / 8 a power of two; z is rounded to bf16 once more than in mc_conv_dgrad_inv.
 * Replaces cuda::MappedConvBackwardInput, src/nn/cuda/mapped_convolution_layer.cu:75-132. */
int mc_conv_dgrad_tapsum(const mc_desc* d, const void* z, const void* inv, void* gx, void* stream);

/* Row plans: sample maps that are translation invariant along image rows,
 *     map[r, x, k] = (x + cx[r, k], cy[r, k])      (x possibly wrapped into [0, W)),
 * which is what spherical kernels on equirectangular images produce (gnomonic, equirectangular and
 * plain grids).  For such maps the bilinear weights of a tap are constants of the row; they are
 * folded into per-row effective weight matrices, and the convolution runs on plain shifted windows
 * of source rows - no interpolation in the data path.  Same results as mc_conv_fwd / mc_conv_dgrad /
 * mc_conv_wgrad within the bf16 tolerance; same reference drivers
 * (src/nn/cuda/mapped_convolution_layer.cu:16-73, :75-132, :134-193).
 *
 * Building a plan takes three steps, none of which allocates:
 *   1. mc_rowplan_analyse writes (OH, K, 3) doubles (cx, cy, kind) to DEVICE memory
 *      (mc_rowplan_analysis_bytes; 0 = this descriptor has no row-plan kernels: they take MC_BF16,
 *      MC_NHWC, P == 0, bilinear / bispherical, C_in == C_out == 64, OW == IW, OW % 512 == 0);
 *   2. if no kind is 0 the caller copies them and the sample map to the host, and
 *      mc_rowplan_assemble (pure host code) writes the plan as int32s into a host buffer.  It decodes
 *      every map entry exactly as mc_conv_fwd does and lists the few pixels that deviate from their
 *      row's nominal behaviour (the seam of wrapped maps, positions within rounding of an integer)
 *      as corrections that the kernels apply, so results agree with mc_conv_fwd pixel for pixel.
 *      It returns the number of int32s the plan needs (call with capacity 0 to size the buffer) or 0
 *      if the map is not row invariant;
 *   3. the caller keeps the host copy and uploads a copy to the device (16-byte aligned).
 * A plan depends only on the map and the image sizes, like the tap table and the inverse map.  It
 * holds, for each direction, the rows' windows and slots twice: row by row (weight gradient,
 * corrections) and for pairs of adjacent rows (forward and input gradient compute two result rows
 * with one N = 128 MMA; the rows of a pair share their windows).
 * dir: 0 = forward, 1 = input gradient.  ws holds the effective weights of the call (16 KB per slot
 * of a row pair) and a tap-major copy of w. */
size_t mc_rowplan_analysis_bytes(const mc_desc* d);
int mc_rowplan_analyse(const mc_desc* d, const void* map, void* analysis, void* stream);
int64_t mc_rowplan_assemble(const mc_desc* d, const double* analysis_host, const float* map_host,
                            int32_t* plan_host, int64_t capacity);
size_t mc_conv_rowplan_workspace_bytes(const mc_desc* d, const void* plan_host, int32_t dir);
int mc_conv_fwd_rowplan(const mc_desc* d, const void* x, const void* plan_host, const void* plan_dev,
                        const void* w, const void* bias, void* y, void* ws, size_t ws_bytes,
                        void* stream);
int mc_conv_dgrad_rowplan(const mc_desc* d, const void* gy, const void* plan_host,
                          const void* plan_dev, const void* w, const void* bias_out, void* gx,
                          void* ws, size_t ws_bytes, void* stream);
/* Weight and bias gradient (float32, fully overwritten; gb may be NULL) from the same plan; ws holds
 * one 64 x 64 float32 partial sum per slot and batch part and the partial results of the two-step
 * reduction that follows (no atomics: gw repeats bit for bit; gb is summed per row inside the main
 * kernel and added up with float atomics, so it repeats to rounding only). */
size_t mc_conv_wgrad_rowplan_workspace_bytes(const mc_desc* d, const void* plan_host);
int mc_conv_wgrad_rowplan(const mc_desc* d, const void* gy, const void* x, const void* plan_host,
                          const void* plan_dev, void* gw, void* gb, void* ws, size_t ws_bytes,
                          void* stream);

/* gw(C_out,C_in,K) = sum_b gy_b . im2col_map(x_b)^T and gb(C_out) = sum_{b,h,w} gy.
 * gw and gb are written in the accumulation type: double for MC_F64, float otherwise
 * (also for MC_BF16), fully overwritten.  gb may be NULL.
 * Replaces cuda::MappedConvBackwardWeight, src/nn/cuda/mapped_convolution_layer.cu:134-193 and
 * grad_output.sum({0,2,3}), include/nn/layers/mapped_convolution_layer.h:113. */
int mc_conv_wgrad(const mc_desc* d, const void* gy, const void* x, const void* map, const void* iw,
                  void* gw, void* gb, void* ws, size_t ws_bytes, void* stream);
size_t mc_conv_wgrad_workspace_bytes(const mc_desc* d);

/* gb[c] = sum over batch and pixels of gy (B, C_out, OH, OW); gb is float32 (float64 for float64
 * tensors).  The reference takes it from grad_output.sum({0, 2, 3}),
 * include/nn/layers/mapped_convolution_layer.h:113; mc_conv_wgrad fuses it, this entry point
 * serves callers that obtain the weight gradient some other way. */
int mc_bias_grad(const mc_desc* d, const void* gy, void* gb, void* stream);

/* ---- mapped transposed convolution ----------------------------------------------------
 * Here d->C_in / d->C_out are the transposed layer's own in/out channels, weight is
 * (C_in, C_out, K), the map has the size of the layer *input* (d->OH, d->OW = input size) and
 * points into the layer *output* (d->IH, d->IW = output size).
 * Replace cuda::MappedTransposedConv{Forward,BackwardInput,BackwardWeight},
 * src/nn/cuda/mapped_transposed_convolution_layer.cu:53-108, :110-160, :162-220. */
int mc_tconv_fwd(const mc_desc* d, const void* x, const void* map, const void* iw, const void* w,
                 const void* bias, void* y, void* ws, size_t ws_bytes, void* stream);
int mc_tconv_dgrad(const mc_desc* d, const void* gy, const void* map, const void* iw,
                   const void* w, void* gx, void* ws, size_t ws_bytes, void* stream);
int mc_tconv_wgrad(const mc_desc* d, const void* gy, const void* x, const void* map,
                   const void* iw, void* gw, void* gb, void* ws, size_t ws_bytes, void* stream);
size_t mc_tconv_workspace_bytes(const mc_desc* d);

/* ---- mapped pooling ---------------------------------------------------------------------
 * x (B,C_in,IH,IW) -> y (B,C_in,OH,OW).  idx is int64, same shape/layout as y, and holds the
 * element offset of the winning tap inside the sample map (first maximum wins, -1 if no tap
 * compared greater than -FLT_MAX).
 * Replace MappedMaxPool2DLauncher / MappedMaxUnpool2DLauncher, include/nn/cuda/mapped_max_pool.cuh:15-183
 * and MappedAvgPool2DLauncher / MappedAvgUnpool2DLauncher, include/nn/cuda/mapped_avg_pool.cuh:15-169. */
int mc_pool_max_fwd(const mc_desc* d, const void* x, const void* map, const void* iw, void* y,
                    int64_t* idx, void* stream);
/* gx (B,C_in,IH,IW) is fully written.  bf16 needs scratch (see the workspace query). */
int mc_pool_max_bwd(const mc_desc* d, const void* gy, const int64_t* idx, const void* map,
                    const void* iw, void* gx, void* ws, size_t ws_bytes, void* stream);
int mc_pool_avg_fwd(const mc_desc* d, const void* x, const void* map, const void* iw, void* y,
                    void* stream);
int mc_pool_avg_bwd(const mc_desc* d, const void* gy, const void* map, const void* iw, void* gx,
                    void* ws, size_t ws_bytes, void* stream);
/* Scratch needed by the scatter-type kernels (pool backward, resample scatter). */
size_t mc_scatter_workspace_bytes(const mc_desc* d);

/* Average unpooling and resample scatter as gathers through the inverse map (mc_invmap_build with
 * the same descriptor): one thread per image pixel sums its contributions - no atomics, no
 * zero-fill pass, bit-reproducible.  MC_F32 / MC_BF16, unweighted maps; MC_ERR_UNSUPPORTED
 * otherwise (use the map-based entry points then).  Same reference kernels as mc_pool_avg_bwd /
 * mc_resample_scatter: include/nn/cuda/mapped_avg_pool.cuh:92-130, resample.cuh:14-52. */
int mc_pool_avg_bwd_inv(const mc_desc* d, const void* gy, const void* inv, void* gx, void* stream);
int mc_resample_scatter_inv(const mc_desc* d, const void* x, const void* inv, void* y, void* stream);

/* ---- resample ---------------------------------------------------------------------------
 * gather  ("Unresample"): y(B,C,OH,OW)[p] = interp(x(B,C,IH,IW), map(OH,OW,[P,]2)[p]);
 *   replaces ResampleFromMap2DLauncher, include/nn/cuda/resample.cuh:54-92 (+weighted :128-160).
 * scatter ("Resample"):   y(B,C,IH,IW) += extrapolate(x(B,C,OH,OW)[q], map(OH,OW,[P,]2)[q]);
 *   y is fully written (zero-filled first); replaces ResampleToMap2DLauncher, resample.cuh:14-52.
 * In both calls (OH,OW) is the map grid and (IH,IW) the image the map points into; d->K must be 1. */
int mc_resample_gather(const mc_desc* d, const void* x, const void* map, const void* iw, void* y,
                       void* stream);
int mc_resample_scatter(const mc_desc* d, const void* x, const void* map, const void* iw, void* y,
                        void* ws, size_t ws_bytes, void* stream);

/* ---- k nearest neighbours -----------------------------------------------------------------
 * ref (B, D, M), query (B, D, N) float, contiguous.  idx (B, k, N) int64 holds 1-BASED reference
 * indices, ordered by (distance, index); dist (B, k, N) the Euclidean distances.
 * Replaces KNNLauncher, include/util/cuda/knn.cuh:232-275 and KNNForward,
 * src/util/cuda/knn_layer.cu:13-32.  Limits: 1 <= k <= 32, k <= M, D <= 16. */
int mc_knn(const float* ref, const float* query, int32_t B, int32_t D, int32_t M, int32_t N,
           int32_t k, int64_t* idx, float* dist, void* stream);

/* ---- point location on the icosphere hierarchy ------------------------------------------------
 * samples (n, 2) float (lon, lat) radians.  Levels 0..order of the mesh hierarchy are given as host
 * arrays of DEVICE pointers: vertices[l] (V_l, 3) float, face_vertices[l] (F_l, 3) int32 (the
 * vertices of every face in its half-edge walk order), face_adjacent[l] (F_l, 3) int32 (the faces
 * across the three half-edges), num_faces[l] = F_l; children of face f of level l are faces
 * 4 f .. 4 f + 3 of level l + 1.  Outputs: face_idx (n) int64 face of level `order` hit by the ray
 * of every sample (-1: not found), vertex_idx (n, 3) int64 its vertices (walk vertices 2, 1, 0),
 * weights (n, 3) float their barycentric weights (one-hot of the largest when nearest != 0).
 * Replaces Sphere::getPlanarConvolutionOperatorFromSamples, src/util/cpp/sphere.cpp:1116-1270
 * (search :1007-1053, face test :1055-1105), a host OpenMP loop in the reference.  order <= 11. */
int mc_sphere_locate(const float* samples, int64_t n, int32_t order, const float* const* vertices,
                     const int32_t* const* face_vertices, const int32_t* const* face_adjacent,
                     const int32_t* num_faces, int32_t nearest, int64_t* face_idx,
                     int64_t* vertex_idx, float* weights, void* stream);

/* ---- cube map -> equirectangular image ------------------------------------------------------
 * cube (C, D, 6 D) of `dtype` (MC_F32 / MC_F64), the six faces side by side in the order
 * -z, -x, +z, +x, +y, -y; rect (C, rect_h, rect_w), fully written.  interp: 0 nearest, 1 bilinear.
 * Every pixel of the result looks along its longitude / latitude, finds the face that direction
 * leaves the cube through and samples the face there.  Replaces Cube2RectLauncher,
 * include/util/cuda/cube2rect.cuh:66-82 (kernel :15-62) and Cube2RectForward,
 * src/util/cuda/cube2rect_layer.cu:11-29; same arithmetic, bit-identical results. */
int mc_cube2rect(int32_t dtype, const void* cube, int32_t channels, int32_t cube_dim, int32_t rect_h,
                 int32_t rect_w, int32_t interp, void* rect, void* stream);

/* ---- voting resample ------------------------------------------------------------------------
 * labels (B, C, IH, IW) int64 in [0, num_candidates); map (IH, IW, 2) int64: the (x, y) target
 * pixel of every source pixel (16-byte aligned; targets outside (OH, OW) are dropped, and so are
 * labels outside the candidate range).  out (B, C, OH, OW) int64: the label most source pixels
 * brought to each target pixel - the smallest such label among equals, 0 where nothing landed.
 * ws: mc_voting_resample_workspace(...) bytes of device scratch (32-bit vote counters).
 * Replaces ResampleToMap2DVotingLauncher, include/nn/cuda/resample.cuh:166-200, Vote2D,
 * include/core/interpolation.h:241-257, and VotingResampleToMap (votes + argmax per image),
 * src/nn/cuda/voting_resample_layer.cu:10-38 / src/nn/cpp/voting_resample_layer.cpp:8-38. */
size_t mc_voting_resample_workspace(int32_t B, int32_t C, int32_t OH, int32_t OW, int32_t num_candidates);
int mc_voting_resample(const int64_t* labels, const int64_t* map, int32_t B, int32_t C, int32_t IH,
                       int32_t IW, int32_t OH, int32_t OW, int32_t num_candidates, void* ws,
                       size_t ws_bytes, int64_t* out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MC_B200_H_ */
