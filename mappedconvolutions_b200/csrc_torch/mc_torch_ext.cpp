// PyTorch C++ extension: the operator surface of the reference's pybind modules
// (_mapped_convolution_ext.<module>, package/ext_modules/src/*.cpp of the reference) bound to the
// sm_100a library through its C ABI (include/mc_b200.h).
//
// Function names, argument order and return values follow the reference's functions
// (include/nn/layers/*.h, include/util/layers/knn_layer.h); each binding cites the one it mirrors.
// As in the reference, outputs are freshly allocated and returned, and inputs must be contiguous
// and on one device.  Differences: tensors must be CUDA tensors (there is no CPU path), bfloat16
// activations are accepted (with a float32 sample map), and a 4-D activation may be channels_last,
// in which case the outputs are channels_last too.
//
// mappedconvolutions_b200/ops.py is the same host logic on ctypes; the tests use it to reach the
// C ABI without a compiler, and check the two against each other.
#include <algorithm>
#include <torch/extension.h>

#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>

#include <list>
#include <mutex>
#include <tuple>
#include <vector>

#include "mc_b200.h"

namespace {

using torch::Tensor;
using OptTensor = c10::optional<Tensor>;

void check(int rc) {
  TORCH_CHECK(rc == 0, "mc_b200: ", mc_strerror(rc), " (code ", rc, ")");
}

void* cur_stream() { return (void*)c10::cuda::getCurrentCUDAStream().stream(); }

c10::Device need_cuda(std::initializer_list<const Tensor*> ts) {
  c10::optional<c10::Device> dev;
  for (const Tensor* t : ts) {
    if (!t || !t->defined()) continue;
    TORCH_CHECK(t->is_cuda(), "mapped convolution ops are CUDA only: got a CPU tensor "
                              "(this build has no CPU path)");
    if (!dev) dev = t->device();
    else TORCH_CHECK(t->device() == *dev, "all tensors must be on the same device");
  }
  TORCH_CHECK(dev.has_value(), "no tensor given");
  return *dev;
}

const Tensor* opt(const OptTensor& t) { return t.has_value() ? &*t : nullptr; }
const void* ptr(const OptTensor& t) { return t.has_value() ? t->data_ptr() : nullptr; }

int layout_of(const Tensor& x) {
  if (x.is_contiguous()) return MC_NCHW;
  if (x.dim() == 4 && x.is_contiguous(at::MemoryFormat::ChannelsLast)) return MC_NHWC;
  TORCH_CHECK(false, "input must be contiguous");
}

Tensor as_layout(const Tensor& t, int layout) {
  return layout == MC_NHWC ? t.contiguous(at::MemoryFormat::ChannelsLast) : t.contiguous();
}

Tensor empty_in(at::IntArrayRef shape, const Tensor& like, int layout,
                c10::optional<at::ScalarType> dtype = c10::nullopt) {
  auto o = like.options().dtype(dtype.value_or(like.scalar_type()));
  return at::empty(shape, o, layout == MC_NHWC ? at::MemoryFormat::ChannelsLast
                                               : at::MemoryFormat::Contiguous);
}

void check_map(const Tensor& x, const Tensor& map, const OptTensor& iw) {
  const auto want = x.scalar_type() == at::kDouble ? at::kDouble : at::kFloat;
  if (map.scalar_type() != want) {
    TORCH_CHECK(!(x.scalar_type() == at::kBFloat16 && map.scalar_type() == at::kBFloat16),
                "sample map of a bfloat16 input must be float32");
    TORCH_CHECK(false, "sample map dtype ", map.scalar_type(), " does not match input dtype ",
                x.scalar_type());
  }
  TORCH_CHECK(map.is_contiguous(), "sample_map must be contiguous");
  if (iw.has_value()) {
    TORCH_CHECK(iw->scalar_type() == want, "interp_weights dtype must match the sample map");
    TORCH_CHECK(iw->is_contiguous(), "interp_weights must be contiguous");
  }
}

mc_desc make_desc(at::ScalarType dt, int layout, int64_t B, int64_t Cin, int64_t Cout, int64_t IH,
                  int64_t IW, int64_t OH, int64_t OW, int64_t K, int64_t P, int64_t interp) {
  mc_desc d{};
  d.B = (int32_t)B; d.C_in = (int32_t)Cin; d.C_out = (int32_t)Cout;
  d.IH = (int32_t)IH; d.IW = (int32_t)IW; d.OH = (int32_t)OH; d.OW = (int32_t)OW;
  d.K = (int32_t)K; d.P = (int32_t)P; d.interp = (int32_t)interp;
  if (dt == at::kFloat) d.dtype = MC_F32;
  else if (dt == at::kDouble) d.dtype = MC_F64;
  else if (dt == at::kBFloat16) d.dtype = MC_BF16;
  else TORCH_CHECK(false, "unsupported dtype ", dt, " (float32, float64, bfloat16)");
  d.layout = layout;
  return d;
}

int64_t n_interp(const OptTensor& iw) { return iw.has_value() ? iw->size(-1) : 0; }

// The C ABI takes raw pointers, so everything it would otherwise read past or misinterpret is
// checked here: parameter and gradient dtypes equal to the input's (the reference raises through
// weight.data<scalar_t>(), src/nn/cuda/mapped_convolution_layer.cu:57-65) and the shapes the
// descriptor is built from.  w0 / w1: the weight's first two dimensions.
void check_conv_args(const Tensor& input, const Tensor& sample_map, const Tensor& weight,
                     const Tensor& bias, int64_t w0, int64_t w1, int64_t n_bias, int64_t K,
                     const Tensor* grad_output = nullptr, at::IntArrayRef grad_shape = {}) {
  TORCH_CHECK(input.dim() == 4, "input must be 4-D (B, C, H, W)");
  TORCH_CHECK(sample_map.dim() >= 4 && sample_map.size(-1) == 2,
              "sample_map must be (OH, OW, K, 2) or (OH, OW, K, P, 2)");
  TORCH_CHECK(weight.scalar_type() == input.scalar_type(), "weight dtype ", weight.scalar_type(),
              " does not match input dtype ", input.scalar_type());
  TORCH_CHECK(bias.scalar_type() == input.scalar_type(), "bias dtype ", bias.scalar_type(),
              " does not match input dtype ", input.scalar_type());
  TORCH_CHECK(weight.dim() == 3 && weight.size(0) == w0 && weight.size(1) == w1 && weight.size(2) == K,
              "weight must have shape (", w0, ", ", w1, ", ", K, "), got ", weight.sizes());
  TORCH_CHECK(bias.numel() == n_bias, "bias must have ", n_bias, " elements, got ", bias.numel());
  TORCH_CHECK(sample_map.size(2) == K, "sample_map.size(2) = ", sample_map.size(2),
              " does not match kernel_size ", K);
  TORCH_CHECK(weight.is_contiguous() && bias.is_contiguous(), "weight and bias must be contiguous");
  if (grad_output) {
    TORCH_CHECK(grad_output->scalar_type() == input.scalar_type(), "grad_output dtype ",
                grad_output->scalar_type(), " does not match input dtype ", input.scalar_type());
    TORCH_CHECK(grad_output->sizes() == grad_shape, "grad_output must have shape ", grad_shape,
                ", got ", grad_output->sizes());
  }
}

// Scratch buffer of at least n bytes (undefined tensor for n == 0).
struct Scratch {
  Tensor t;
  void* p = nullptr;
  size_t n = 0;
};
Scratch scratch(size_t n, const c10::Device& dev) {
  Scratch s;
  if (n == 0) return s;
  s.t = at::empty({(int64_t)n}, at::TensorOptions().dtype(at::kByte).device(dev));
  s.p = s.t.data_ptr();
  s.n = n;
  return s;
}

// ---- per-map plans ----------------------------------------------------------------------------------
// The inverse map and the tap table depend only on the sample map tensor and the image sizes.  A
// layer is called with the same map tensor step after step, so the last few are kept, keyed by the
// tensor's identity and version counter (an in-place edit of the map invalidates its entry).
struct PlanKey {
  int kind;
  const void* data;
  int64_t version;
  std::vector<int64_t> shape;
  int IH, IW, interp, device;
  const void* iw_data = nullptr;  // plans of weighted maps: the interpolation-weight tensor as well
  int64_t iw_version = 0;
  bool operator==(const PlanKey& o) const {
    return kind == o.kind && data == o.data && version == o.version && shape == o.shape &&
           IH == o.IH && IW == o.IW && interp == o.interp && device == o.device &&
           iw_data == o.iw_data && iw_version == o.iw_version;
  }
};
struct PlanEntry {
  PlanKey key;
  c10::weak_intrusive_ptr<c10::TensorImpl> owner;
  c10::weak_intrusive_ptr<c10::TensorImpl> owner_iw;  // (the map again for plain maps)
  Tensor buf;
  Tensor aux;  // second buffer of the plan (row plans: the host copy)
};
std::list<PlanEntry>& plan_cache() {
  static std::list<PlanEntry> c;
  return c;
}
constexpr size_t PLAN_CACHE_SIZE = 8;

std::mutex& plan_mutex() {
  static std::mutex m;
  return m;
}

// The cache is shared by all threads of the process (one lock around lookup, build and insert).
// A plan is built on the caller's current stream, which is then synchronised once: later calls may
// read the cached buffer from any stream without further ordering.
// build() returns (device buffer, auxiliary buffer or an undefined tensor)
template <typename Build>
std::pair<Tensor, Tensor> cached_plan2(int kind, const mc_desc& d, const Tensor& map, Build build,
                                       const Tensor* iw = nullptr) {
  PlanKey key{kind, map.data_ptr(), (int64_t)map._version(), map.sizes().vec(), d.IH, d.IW, d.interp,
              (int)map.device().index()};
  const Tensor& second = iw ? *iw : map;
  if (iw) {
    key.iw_data = iw->data_ptr();
    key.iw_version = (int64_t)iw->_version();
  }
  std::lock_guard<std::mutex> lock(plan_mutex());
  auto& c = plan_cache();
  for (auto it = c.begin(); it != c.end(); ++it) {
    if (it->key == key && !it->owner.expired() &&
        it->owner.lock().get() == map.unsafeGetTensorImpl() && !it->owner_iw.expired() &&
        it->owner_iw.lock().get() == second.unsafeGetTensorImpl()) {
      if (it != c.begin()) c.splice(c.begin(), c, it);
      return {c.front().buf, c.front().aux};
    }
  }
  std::pair<Tensor, Tensor> p = build();
  c10::cuda::getCurrentCUDAStream().synchronize();
  c.push_front(PlanEntry{key, c10::weak_intrusive_ptr<c10::TensorImpl>(map.getIntrusivePtr()),
                         c10::weak_intrusive_ptr<c10::TensorImpl>(second.getIntrusivePtr()), p.first,
                         p.second});
  while (c.size() > PLAN_CACHE_SIZE) c.pop_back();
  return p;
}

template <typename Build>
Tensor cached_plan(int kind, const mc_desc& d, const Tensor& map, Build build, const Tensor* iw = nullptr) {
  return cached_plan2(kind, d, map, [&]() { return std::make_pair(build(), Tensor()); }, iw).first;
}

Tensor inverse_map(const mc_desc& d, const Tensor& map) {
  return cached_plan(0, d, map, [&]() {
    const size_t n = mc_invmap_bytes(&d);
    Tensor inv = at::empty({(int64_t)n}, at::TensorOptions().dtype(at::kByte).device(map.device()));
    Scratch ws = scratch(mc_invmap_build_workspace_bytes(&d), map.device());
    check(mc_invmap_build(&d, map.data_ptr(), inv.data_ptr(), n, ws.p, ws.n, cur_stream()));
    return inv;
  });
}

// Forward tap table (undefined tensor if the descriptor has no tensor-core path).
Tensor tap_map(const mc_desc& d, const Tensor& map) {
  const size_t n = mc_tapmap_bytes(&d);
  if (n == 0) return Tensor();
  return cached_plan(1, d, map, [&]() {
    Tensor tab = at::empty({(int64_t)n}, at::TensorOptions().dtype(at::kByte).device(map.device()));
    check(mc_tapmap_build(&d, map.data_ptr(), tab.data_ptr(), n, cur_stream()));
    return tab;
  });
}

// Weighted maps whose taps fit a tap-table record (mc_weighted_plan_desc: P points x corners per point
// <= 4, e.g. barycentric icosphere taps with nearest sampling) get the same two plans, built from
// (map, interp_weights); the calls that use them run under the folded descriptor *f.
bool weighted_folds(const mc_desc& d, const OptTensor& iw, mc_desc* f) {
  return iw.has_value() && iw->scalar_type() == at::kFloat && mc_weighted_plan_desc(&d, f) == MC_OK;
}

Tensor inverse_map_weighted(const mc_desc& d, const mc_desc& f, const Tensor& map, const Tensor& iw) {
  return cached_plan(3, d, map, [&]() {
    const size_t n = mc_invmap_bytes(&f);
    Tensor inv = at::empty({(int64_t)n}, at::TensorOptions().dtype(at::kByte).device(map.device()));
    Scratch ws = scratch(mc_invmap_build_workspace_bytes(&f), map.device());
    check(mc_invmap_build_weighted(&d, map.data_ptr(), iw.data_ptr(), inv.data_ptr(), n, ws.p, ws.n,
                                   cur_stream()));
    return inv;
  }, &iw);
}

Tensor tap_map_weighted(const mc_desc& d, const mc_desc& f, const Tensor& map, const Tensor& iw) {
  const size_t n = mc_tapmap_bytes(&f);
  if (n == 0) return Tensor();
  return cached_plan(4, d, map, [&]() {
    Tensor tab = at::empty({(int64_t)n}, at::TensorOptions().dtype(at::kByte).device(map.device()));
    check(mc_tapmap_build_weighted(&d, map.data_ptr(), iw.data_ptr(), tab.data_ptr(), n, cur_stream()));
    return tab;
  }, &iw);
}

// Row plan of a sample map that is translation invariant along image rows (spherical kernels on
// equirectangular images): (device copy, host copy), or undefined tensors if the descriptor has
// no row-plan kernels or the map does not qualify - which is remembered too, so that a map is
// analysed once.  Building it costs one pass over the map on the device, a copy of the map to the
// host and a host pass over it (0.3 s for a 512 x 1024 x 9 map); it depends only on the map.
bool g_row_plans = true;

std::pair<Tensor, Tensor> row_plan(const mc_desc& d, const Tensor& map) {
  if (!g_row_plans) return {Tensor(), Tensor()};
  const size_t na = mc_rowplan_analysis_bytes(&d);
  if (na == 0 || map.dim() != 4) return {Tensor(), Tensor()};
  auto p = cached_plan2(2, d, map, [&]() {
    Tensor ana = at::empty({(int64_t)(na / 8)}, at::TensorOptions().dtype(at::kDouble).device(map.device()));
    check(mc_rowplan_analyse(&d, map.data_ptr(), ana.data_ptr(), cur_stream()));
    Tensor ana_h = ana.cpu();
    const double* a = ana_h.data_ptr<double>();
    const Tensor none = at::empty({0}, at::TensorOptions().dtype(at::kInt));
    for (int64_t i = 0; i < (int64_t)(na / 24); ++i)
      if (a[3 * i + 2] == 0.0) return std::make_pair(none, none);
    Tensor map_h = map.cpu();
    const int64_t n = mc_rowplan_assemble(&d, a, map_h.data_ptr<float>(), nullptr, 0);
    if (n == 0) return std::make_pair(none, none);
    Tensor plan_h = at::empty({n}, at::TensorOptions().dtype(at::kInt));
    TORCH_CHECK(mc_rowplan_assemble(&d, a, map_h.data_ptr<float>(), plan_h.data_ptr<int32_t>(), n) == n,
                "row plan assembly changed its size");
    return std::make_pair(plan_h.to(map.device()), plan_h);
  });
  if (!p.first.defined() || p.first.numel() == 0) return {Tensor(), Tensor()};
  return p;
}

void clear_plan_cache() {
  std::lock_guard<std::mutex> lock(plan_mutex());
  plan_cache().clear();
}

// Kinds of the cached plans, most recently used first (0 inverse map, 1 tap table, 2 row plan,
// 3 / 4 inverse map / tap table of a weighted map): lets a test see which path a call took.
std::vector<int64_t> plan_cache_kinds() {
  std::lock_guard<std::mutex> lock(plan_mutex());
  std::vector<int64_t> kinds;
  for (const auto& e : plan_cache()) kinds.push_back(e.key.kind);
  return kinds;
}

Tensor channels_last(const Tensor& t) { return t.contiguous(at::MemoryFormat::ChannelsLast); }

// The tensor-core kernels read rows with 16-byte vector loads and bulk copies.  A view into a larger
// tensor (a batch slice, a map slice) can start on any element boundary: such a tensor is copied
// into a fresh allocation, which the caching allocator aligns to 512 bytes.
Tensor aligned16(const Tensor& t) {
  if ((reinterpret_cast<uintptr_t>(t.data_ptr()) & 15) == 0) return t;
  return t.clone(at::MemoryFormat::Preserve);
}

// bfloat16 tensors in the reference's NCHW layout: the tensor-core kernels want channels-last, and
// two extra layout passes cost far less than the generic kernels.  (A single-channel tensor is
// contiguous in both layouts at once and counts as NCHW: it is rerouted too, at no cost, and the
// result comes back in NCHW.  The rerouted call passes nhwc = true.)
bool via_channels_last(const Tensor& input, const OptTensor& iw, mc_desc d_nhwc) {
  if (input.scalar_type() != at::kBFloat16 || input.dim() != 4) return false;
  if (layout_of(input) != MC_NCHW) return false;
  d_nhwc.layout = MC_NHWC;
  if (iw.has_value()) {
    d_nhwc.P = (int32_t)iw->size(-1);
    mc_desc f;
    if (!weighted_folds(d_nhwc, iw, &f)) return false;
    d_nhwc = f;
  }
  return mc_conv_fwd_workspace_bytes(&d_nhwc) > 0;
}

// ---- convolution ---------------------------------------------------------------------------------------

// relu: y = max(0, conv + bias), applied in the kernel's epilogue (MC_FLAG_RELU)
Tensor conv_forward(const Tensor& input_in, const Tensor& sample_map_in, const OptTensor& iw,
                    const Tensor& weight, const Tensor& bias, int64_t K, int64_t interp,
                    bool nhwc = false, bool relu = false) {
  const Tensor input = aligned16(input_in), sample_map = aligned16(sample_map_in);
  TORCH_CHECK(input.dim() == 4 && weight.dim() == 3, "input must be 4-D, weight 3-D");
  check_conv_args(input, sample_map, weight, bias, weight.size(0), input.size(1), weight.size(0), K);
  const auto dev = need_cuda({&input, &sample_map, opt(iw), &weight, &bias});
  const int64_t B = input.size(0), Cin = input.size(1), IH = input.size(2), IW = input.size(3);
  const int64_t Cout = weight.size(0), OH = sample_map.size(0), OW = sample_map.size(1);
  if (!nhwc && via_channels_last(input, iw, make_desc(input.scalar_type(), MC_NHWC, B, Cin, Cout, IH,
                                                      IW, OH, OW, K, 0, interp)))
    return conv_forward(channels_last(input), sample_map, iw, weight, bias, K, interp, true,
                        relu).contiguous();
  const int layout = nhwc ? MC_NHWC : layout_of(input);
  check_map(input, sample_map, iw);
  TORCH_CHECK(weight.is_contiguous() && bias.is_contiguous(), "weight and bias must be contiguous");
  mc_desc d = make_desc(input.scalar_type(), layout, B, Cin, Cout, IH, IW, OH, OW, K, n_interp(iw),
                        interp);
  Tensor y = empty_in({B, Cout, OH, OW}, input, layout);
  c10::cuda::CUDAGuard guard(dev);
  if (!iw.has_value()) {
    auto rp = row_plan(d, sample_map);
    if (rp.first.defined()) {  // row-invariant map: shifted windows, no interpolation in the data path
      Scratch wsr = scratch(mc_conv_rowplan_workspace_bytes(&d, rp.second.data_ptr(), 0), dev);
      check(mc_conv_fwd_rowplan(&d, input.data_ptr(), rp.second.data_ptr(), rp.first.data_ptr(),
                                weight.data_ptr(), bias.data_ptr(), y.data_ptr(), wsr.p, wsr.n,
                                cur_stream()));
      // (these kernels correct single pixels after their epilogue, so the activation follows)
      return relu ? y.relu_() : y;
    }
  }
  if (relu) d.flags |= MC_FLAG_RELU;
  mc_desc f;
  if (weighted_folds(d, iw, &f) && mc_conv_fwd_workspace_bytes(&f) > 0) {
    // weighted map on the tensor cores: its points folded into the tap table (f keeps d's flags)
    Scratch wsf = scratch(mc_conv_fwd_workspace_bytes(&f), dev);
    Tensor tabw = tap_map_weighted(d, f, sample_map, *iw);
    if (tabw.defined()) {
      check(mc_conv_fwd_tap(&f, input.data_ptr(), tabw.data_ptr(), weight.data_ptr(), bias.data_ptr(),
                            y.data_ptr(), wsf.p, wsf.n, cur_stream()));
      return y;
    }
  }
  Scratch ws = scratch(mc_conv_fwd_workspace_bytes(&d), dev);
  Tensor tab = (ws.n && !iw.has_value()) ? tap_map(d, sample_map) : Tensor();
  if (tab.defined())  // tensor-core path with the map decoded once per map tensor
    check(mc_conv_fwd_tap(&d, input.data_ptr(), tab.data_ptr(), weight.data_ptr(), bias.data_ptr(),
                          y.data_ptr(), ws.p, ws.n, cur_stream()));
  else
    check(mc_conv_fwd(&d, input.data_ptr(), sample_map.data_ptr(), ptr(iw), weight.data_ptr(),
                      bias.data_ptr(), y.data_ptr(), ws.p, ws.n, cur_stream()));
  return y;
}

// Input gradient as GEMM + gather-sum (mc_conv_dgrad_tapsum) instead of gather-in-the-GEMM: when the
// layer has more output than input channels and the product z fits comfortably.
static bool contract_first(const mc_desc& d) {
  const int lanes = d.C_in / 8;
  // (also for square wide layers with a nearest map, where the gather inside the GEMM kernel runs at
  // half the forward's rate: 256 -> 256 channels 1.30 ms as a gather, 1.0 ms as GEMM + gather-sum)
  const bool wider = d.C_out > d.C_in || (d.C_out == d.C_in && d.C_in >= 128 && d.interp != 1 && d.interp != 2);
  return d.dtype == MC_BF16 && d.layout == MC_NHWC && d.P == 0 && wider && d.C_in % 8 == 0 &&
         (lanes & (lanes - 1)) == 0 &&
         (int64_t)d.B * d.OH * d.OW * d.K * d.C_in * 2 <= ((int64_t)8 << 30);
}

std::vector<Tensor> conv_backward(const Tensor& grad_output_in, const Tensor& sample_map_in,
                                  const OptTensor& iw, const Tensor& input_in, const Tensor& weight,
                                  const Tensor& bias, int64_t K, int64_t interp,
                                  bool need_input_grad, bool nhwc = false,
                                  bool need_weight_grad = true, const OptTensor& relu_output = c10::nullopt) {
  // relu_output: the layer's output behind a fused ReLU; grad_output is then the gradient behind the
  // activation.  Where the one kernel that can mask grad_output while it loads it does all the work
  // (weight gradient only, very few input channels) it is handed over; otherwise it is masked here.
  if (relu_output.has_value()) {
    TORCH_CHECK(relu_output->sizes() == grad_output_in.sizes() &&
                    relu_output->scalar_type() == grad_output_in.scalar_type(),
                "relu_output must have grad_output's shape and dtype");
    const bool fusable = !need_input_grad && need_weight_grad && !iw.has_value() &&
                         input_in.scalar_type() == at::kBFloat16 && input_in.dim() == 4 &&
                         layout_of(input_in) == MC_NHWC && layout_of(grad_output_in) == MC_NHWC &&
                         layout_of(*relu_output) == MC_NHWC;
    if (!fusable)
      return conv_backward(at::threshold_backward(grad_output_in, *relu_output, 0), sample_map_in, iw, input_in,
                           weight, bias, K, interp, need_input_grad, nhwc, need_weight_grad);
  }
  const Tensor input = aligned16(input_in), sample_map = aligned16(sample_map_in);
  TORCH_CHECK(input.dim() == 4 && weight.dim() == 3 && sample_map.dim() >= 4,
              "input must be 4-D, weight 3-D, the map (OH, OW, K, ..)");
  check_conv_args(input, sample_map, weight, bias, weight.size(0), input.size(1), weight.size(0), K,
                  &grad_output_in,
                  {input.size(0), weight.size(0), sample_map.size(0), sample_map.size(1)});
  const auto dev = need_cuda({&grad_output_in, &sample_map, opt(iw), &input, &weight, &bias});
  const int64_t B = input.size(0), Cin = input.size(1), IH = input.size(2), IW = input.size(3);
  const int64_t Cout = weight.size(0), OH = sample_map.size(0), OW = sample_map.size(1);
  if (!nhwc && via_channels_last(input, iw, make_desc(input.scalar_type(), MC_NHWC, B, Cin, Cout, IH,
                                                      IW, OH, OW, K, 0, interp))) {
    auto g = conv_backward(channels_last(grad_output_in), sample_map, iw,
                           channels_last(input), weight, bias, K, interp, need_input_grad, true,
                           need_weight_grad);
    if (g[0].defined()) g[0] = g[0].contiguous();
    return g;
  }
  const int layout = nhwc ? MC_NHWC : layout_of(input);
  const Tensor grad_output = aligned16(as_layout(grad_output_in, layout));
  check_map(input, sample_map, iw);
  const mc_desc d_map = make_desc(input.scalar_type(), layout, B, Cin, Cout, IH, IW, OH, OW, K,
                                  n_interp(iw), interp);
  // A weighted map that folds runs everything below under the folded descriptor, with plans built
  // from (map, interp_weights); any other weighted map has no plans and takes the plain entry points.
  mc_desc f;
  const bool folded = weighted_folds(d_map, iw, &f);
  const mc_desc d = folded ? f : d_map;
  const auto acc = input.scalar_type() == at::kDouble ? at::kDouble : at::kFloat;
  Tensor gx = need_input_grad ? empty_in(input.sizes(), input, layout) : Tensor();
  Tensor gw = at::empty(weight.sizes(), weight.options().dtype(acc));
  Tensor gb = at::empty({Cout}, weight.options().dtype(acc));
  c10::cuda::CUDAGuard guard(dev);
  auto rp = iw.has_value() ? std::pair<Tensor, Tensor>() : row_plan(d, sample_map);
  if (need_input_grad && rp.first.defined()) {
    Scratch wsr = scratch(mc_conv_rowplan_workspace_bytes(&d, rp.second.data_ptr(), 1), dev);
    check(mc_conv_dgrad_rowplan(&d, grad_output.data_ptr(), rp.second.data_ptr(), rp.first.data_ptr(),
                                weight.data_ptr(), nullptr, gx.data_ptr(), wsr.p, wsr.n, cur_stream()));
    need_input_grad = false;  // done
  }
  Tensor inv;
  if (need_input_grad && (folded || !iw.has_value()) && mc_conv_dgrad_inv_supported(&d))
    inv = folded ? inverse_map_weighted(d_map, f, sample_map, *iw) : inverse_map(d, sample_map);
  if (need_input_grad && inv.defined() && contract_first(d)) {
    // more output than input channels: contract with the weights first (one dense GEMM), then
    // gather-sum the narrow rows through the inverse map
    Tensor g2 = grad_output.permute({0, 2, 3, 1}).reshape({B * OH * OW, Cout});  // a view of channels-last
    Tensor wr = weight.permute({0, 2, 1}).reshape({Cout, K * Cin});
    Tensor z = at::matmul(g2, wr);
    check(mc_conv_dgrad_tapsum(&d, z.data_ptr(), inv.data_ptr(), gx.data_ptr(), cur_stream()));
    need_input_grad = false;  // done
  }
  const size_t n_dgrad = inv.defined() ? mc_conv_dgrad_inv_workspace_bytes(&d)
                                       : mc_conv_dgrad_workspace_bytes(&d_map);
  Scratch ws = scratch(std::max(n_dgrad, mc_conv_wgrad_workspace_bytes(&d_map)), dev);
  if (!need_input_grad) {
  } else if (inv.defined()) {
    check(mc_conv_dgrad_inv(&d, grad_output.data_ptr(), inv.data_ptr(), weight.data_ptr(), nullptr,
                            gx.data_ptr(), ws.p, ws.n, cur_stream()));
  } else {
    check(mc_conv_dgrad(&d_map, grad_output.data_ptr(), sample_map.data_ptr(), ptr(iw),
                        weight.data_ptr(), nullptr, gx.data_ptr(), ws.p, ws.n, cur_stream()));
  }
  if (!need_weight_grad) return {gx, Tensor(), Tensor()};
  if (rp.first.defined()) {  // row-invariant map: weight gradient from the same plan
    Scratch wsr = scratch(mc_conv_wgrad_rowplan_workspace_bytes(&d, rp.second.data_ptr()), dev);
    check(mc_conv_wgrad_rowplan(&d, grad_output.data_ptr(), input.data_ptr(), rp.second.data_ptr(),
                                rp.first.data_ptr(), gw.data_ptr(), gb.data_ptr(), wsr.p, wsr.n,
                                cur_stream()));
    return {gx, gw.to(weight.scalar_type()), gb.to(bias.scalar_type())};
  }
  Tensor tab = folded ? tap_map_weighted(d_map, f, sample_map, *iw)
                      : (iw.has_value() ? Tensor() : tap_map(d, sample_map));
  int rc = MC_ERR_UNSUPPORTED;
  if (relu_output.has_value()) {  // (weight gradient only, see above)
    const Tensor yr = aligned16(*relu_output);
    if (tab.defined())
      rc = mc_conv_wgrad_tap_relu(&d, grad_output.data_ptr(), yr.data_ptr(), input.data_ptr(), tab.data_ptr(),
                                  gw.data_ptr(), gb.data_ptr(), cur_stream());
    if (rc == MC_ERR_UNSUPPORTED)  // no kernel masks on the fly for this shape: mask first
      return conv_backward(at::threshold_backward(grad_output, yr, 0), sample_map, iw, input, weight, bias, K,
                           interp, false, nhwc, true);
    check(rc);
    return {gx, gw.to(weight.scalar_type()), gb.to(bias.scalar_type())};
  }
  if (tab.defined())  // weight / bias gradient on the tensor cores from the prebuilt table
    rc = mc_conv_wgrad_tap(&d, grad_output.data_ptr(), input.data_ptr(), tab.data_ptr(),
                           gw.data_ptr(), gb.data_ptr(), cur_stream());
  if (rc == MC_ERR_UNSUPPORTED)  // shapes only the generic kernels take
    rc = mc_conv_wgrad(&d_map, grad_output.data_ptr(), input.data_ptr(), sample_map.data_ptr(), ptr(iw),
                       gw.data_ptr(), gb.data_ptr(), ws.p, ws.n, cur_stream());
  check(rc);
  return {gx, gw.to(weight.scalar_type()), gb.to(bias.scalar_type())};
}

// ---- transposed convolution ------------------------------------------------------------------------------

Tensor tconv_forward(const Tensor& input_in, const Tensor& sample_map_in, const OptTensor& iw,
                     const Tensor& weight, const Tensor& bias, int64_t OHt, int64_t OWt, int64_t K,
                     int64_t interp, bool nhwc = false) {
  const Tensor input = aligned16(input_in), sample_map = aligned16(sample_map_in);
  TORCH_CHECK(input.dim() == 4 && weight.dim() == 3, "input must be 4-D, weight 3-D");
  check_conv_args(input, sample_map, weight, bias, input.size(1), weight.size(1), weight.size(1), K);
  TORCH_CHECK(sample_map.size(0) == input.size(2) && sample_map.size(1) == input.size(3),
              "the sample map of a transposed convolution has the size of the input");
  const auto dev = need_cuda({&input, &sample_map, opt(iw), &weight, &bias});
  const int64_t B = input.size(0), Cin = input.size(1), H = input.size(2), W = input.size(3);
  const int64_t Cout = weight.size(1);
  // the same layer seen as a convolution: the sampled image carries C_out channels, the grid C_in
  if (!nhwc && via_channels_last(input, iw, make_desc(input.scalar_type(), MC_NHWC, B, Cout, Cin, OHt,
                                                      OWt, H, W, K, 0, interp)))
    return tconv_forward(channels_last(input), sample_map, iw, weight, bias, OHt, OWt, K,
                         interp, true).contiguous();
  const int layout = nhwc ? MC_NHWC : layout_of(input);
  check_map(input, sample_map, iw);
  TORCH_CHECK(weight.is_contiguous() && bias.is_contiguous(), "weight and bias must be contiguous");
  const mc_desc d = make_desc(input.scalar_type(), layout, B, Cin, Cout, OHt, OWt, H, W, K,
                              n_interp(iw), interp);
  const mc_desc ds = make_desc(input.scalar_type(), layout, B, Cout, Cin, OHt, OWt, H, W, K,
                               n_interp(iw), interp);
  Tensor y = empty_in({B, Cout, OHt, OWt}, input, layout);
  c10::cuda::CUDAGuard guard(dev);
  mc_desc fs;
  const bool folded = weighted_folds(ds, iw, &fs);  // weighted map with plans (see conv_backward)
  const mc_desc dsu = folded ? fs : ds;
  if ((folded || !iw.has_value()) && mc_conv_dgrad_inv_supported(&dsu)) {
    // its input gradient IS this forward pass: the gather-form tensor-core dgrad serves
    Tensor inv = folded ? inverse_map_weighted(ds, fs, sample_map, *iw) : inverse_map(ds, sample_map);
    Scratch ws = scratch(mc_conv_dgrad_inv_workspace_bytes(&dsu), dev);
    check(mc_conv_dgrad_inv(&dsu, input.data_ptr(), inv.data_ptr(), weight.data_ptr(), bias.data_ptr(),
                            y.data_ptr(), ws.p, ws.n, cur_stream()));
    return y;
  }
  Scratch ws = scratch(mc_tconv_workspace_bytes(&d), dev);
  check(mc_tconv_fwd(&d, input.data_ptr(), sample_map.data_ptr(), ptr(iw), weight.data_ptr(),
                     bias.data_ptr(), y.data_ptr(), ws.p, ws.n, cur_stream()));
  return y;
}

std::vector<Tensor> tconv_backward(const Tensor& grad_output_in, const Tensor& sample_map_in,
                                   const OptTensor& iw, const Tensor& input_in, const Tensor& weight,
                                   const Tensor& bias, int64_t K, int64_t interp,
                                   bool nhwc = false) {
  const Tensor input = aligned16(input_in), sample_map = aligned16(sample_map_in);
  TORCH_CHECK(input.dim() == 4 && weight.dim() == 3 && grad_output_in.dim() == 4,
              "input and grad_output must be 4-D, weight 3-D");
  check_conv_args(input, sample_map, weight, bias, input.size(1), weight.size(1), weight.size(1), K,
                  &grad_output_in,
                  {input.size(0), weight.size(1), grad_output_in.size(2), grad_output_in.size(3)});
  TORCH_CHECK(sample_map.size(0) == input.size(2) && sample_map.size(1) == input.size(3),
              "the sample map of a transposed convolution has the size of the input");
  const auto dev = need_cuda({&grad_output_in, &sample_map, opt(iw), &input, &weight, &bias});
  const int64_t B = input.size(0), Cin = input.size(1), H = input.size(2), W = input.size(3);
  const int64_t Cout = weight.size(1);
  const int64_t OHt = grad_output_in.size(2), OWt = grad_output_in.size(3);
  if (!nhwc && via_channels_last(input, iw, make_desc(input.scalar_type(), MC_NHWC, B, Cout, Cin, OHt,
                                                      OWt, H, W, K, 0, interp))) {
    auto g = tconv_backward(channels_last(grad_output_in), sample_map, iw,
                            channels_last(input), weight, bias, K, interp, true);
    g[0] = g[0].contiguous();
    return g;
  }
  const int layout = nhwc ? MC_NHWC : layout_of(input);
  const Tensor grad_output = aligned16(as_layout(grad_output_in, layout));
  check_map(input, sample_map, iw);
  const mc_desc d = make_desc(input.scalar_type(), layout, B, Cin, Cout, OHt, OWt, H, W, K,
                              n_interp(iw), interp);
  const mc_desc ds = make_desc(input.scalar_type(), layout, B, Cout, Cin, OHt, OWt, H, W, K,
                               n_interp(iw), interp);
  const auto acc = input.scalar_type() == at::kDouble ? at::kDouble : at::kFloat;
  Tensor gx = empty_in(input.sizes(), input, layout);
  Tensor gw = at::empty(weight.sizes(), weight.options().dtype(acc));
  Tensor gb = at::empty({Cout}, weight.options().dtype(acc));
  c10::cuda::CUDAGuard guard(dev);
  mc_desc fs;
  const bool folded = weighted_folds(ds, iw, &fs);  // weighted map with plans (see conv_backward)
  const mc_desc dsu = folded ? fs : ds;
  Tensor tab = folded ? tap_map_weighted(ds, fs, sample_map, *iw)
                      : (iw.has_value() ? Tensor() : tap_map(ds, sample_map));
  if (tab.defined() && mc_conv_fwd_workspace_bytes(&dsu)) {
    // tensor-core path: input gradient = forward of the equivalent convolution applied to
    // grad_output; weight gradient = its weight gradient with the two tensors swapped
    Scratch ws = scratch(std::max(mc_conv_fwd_workspace_bytes(&dsu), mc_conv_wgrad_workspace_bytes(&ds)), dev);
    check(mc_conv_fwd_tap(&dsu, grad_output.data_ptr(), tab.data_ptr(), weight.data_ptr(), nullptr,
                          gx.data_ptr(), ws.p, ws.n, cur_stream()));
    int rc = mc_conv_wgrad_tap(&dsu, input.data_ptr(), grad_output.data_ptr(), tab.data_ptr(),
                               gw.data_ptr(), nullptr, cur_stream());
    if (rc == MC_ERR_UNSUPPORTED)
      rc = mc_conv_wgrad(&ds, input.data_ptr(), grad_output.data_ptr(), sample_map.data_ptr(),
                         ptr(iw), gw.data_ptr(), nullptr, ws.p, ws.n, cur_stream());
    check(rc);
    const mc_desc db = make_desc(input.scalar_type(), layout, B, Cout, Cout, OHt, OWt, OHt, OWt, 1, 0,
                                 interp);
    check(mc_bias_grad(&db, grad_output.data_ptr(), gb.data_ptr(), cur_stream()));
    return {gx, gw.to(weight.scalar_type()), gb.to(bias.scalar_type())};
  }
  Scratch ws = scratch(mc_tconv_workspace_bytes(&d), dev);
  check(mc_tconv_dgrad(&d, grad_output.data_ptr(), sample_map.data_ptr(), ptr(iw), weight.data_ptr(),
                       gx.data_ptr(), ws.p, ws.n, cur_stream()));
  check(mc_tconv_wgrad(&d, grad_output.data_ptr(), input.data_ptr(), sample_map.data_ptr(), ptr(iw),
                       gw.data_ptr(), gb.data_ptr(), ws.p, ws.n, cur_stream()));
  return {gx, gw.to(weight.scalar_type()), gb.to(bias.scalar_type())};
}

// ---- pooling ----------------------------------------------------------------------------------------------

// x lives on the image for forward, on the map grid for backward (then img gives the image size)
mc_desc pool_desc(const Tensor& x, const Tensor& map, const OptTensor& iw, int64_t K, int64_t interp,
                  int layout, int64_t IH = -1, int64_t IW = -1) {
  if (IH < 0) { IH = x.size(2); IW = x.size(3); }
  return make_desc(x.scalar_type(), layout, x.size(0), x.size(1), x.size(1), IH, IW, map.size(0),
                   map.size(1), K, n_interp(iw), interp);
}

std::vector<Tensor> max_pool(const Tensor& input, const Tensor& sample_map, const OptTensor& iw,
                             int64_t K, int64_t interp) {
  const auto dev = need_cuda({&input, &sample_map, opt(iw)});
  check_map(input, sample_map, iw);
  const int layout = layout_of(input);
  const mc_desc d = pool_desc(input, sample_map, iw, K, interp, layout);
  Tensor y = empty_in({d.B, d.C_in, d.OH, d.OW}, input, layout);
  Tensor idx = empty_in({d.B, d.C_in, d.OH, d.OW}, input, layout, at::kLong);
  c10::cuda::CUDAGuard guard(dev);
  check(mc_pool_max_fwd(&d, input.data_ptr(), sample_map.data_ptr(), ptr(iw), y.data_ptr(),
                        idx.data_ptr<int64_t>(), cur_stream()));
  return {y, idx};
}

Tensor max_unpool(const Tensor& grad_output_in, const Tensor& idx_mask, const Tensor& sample_map,
                  const OptTensor& iw, int64_t IH, int64_t IW, int64_t K, int64_t interp) {
  TORCH_CHECK(idx_mask.scalar_type() == at::kLong, "idx_mask must be int64, got ", idx_mask.scalar_type());
  TORCH_CHECK(idx_mask.sizes() == grad_output_in.sizes(), "idx_mask shape ", idx_mask.sizes(),
              " does not match grad_output shape ", grad_output_in.sizes());
  TORCH_CHECK(grad_output_in.dim() == 4 && sample_map.dim() >= 3 &&
                  grad_output_in.size(2) == sample_map.size(0) &&
                  grad_output_in.size(3) == sample_map.size(1),
              "grad_output must live on the map grid");
  const auto dev = need_cuda({&grad_output_in, &idx_mask, &sample_map, opt(iw)});
  const int layout = idx_mask.dim() == 4 ? layout_of(idx_mask) : MC_NCHW;
  const Tensor grad_output = as_layout(grad_output_in, layout);
  check_map(grad_output, sample_map, iw);
  const mc_desc d = pool_desc(grad_output, sample_map, iw, K, interp, layout, IH, IW);
  Tensor gx = empty_in({d.B, d.C_in, IH, IW}, grad_output, layout);
  c10::cuda::CUDAGuard guard(dev);
  Scratch ws = scratch(mc_scatter_workspace_bytes(&d), dev);
  check(mc_pool_max_bwd(&d, grad_output.data_ptr(), idx_mask.data_ptr<int64_t>(),
                        sample_map.data_ptr(), ptr(iw), gx.data_ptr(), ws.p, ws.n, cur_stream()));
  return gx;
}

Tensor avg_pool(const Tensor& input, const Tensor& sample_map, const OptTensor& iw, int64_t K,
                int64_t interp) {
  const auto dev = need_cuda({&input, &sample_map, opt(iw)});
  check_map(input, sample_map, iw);
  const int layout = layout_of(input);
  const mc_desc d = pool_desc(input, sample_map, iw, K, interp, layout);
  Tensor y = empty_in({d.B, d.C_in, d.OH, d.OW}, input, layout);
  c10::cuda::CUDAGuard guard(dev);
  check(mc_pool_avg_fwd(&d, input.data_ptr(), sample_map.data_ptr(), ptr(iw), y.data_ptr(),
                        cur_stream()));
  return y;
}

Tensor avg_unpool(const Tensor& grad_output, const Tensor& sample_map, const OptTensor& iw,
                  int64_t IH, int64_t IW, int64_t K, int64_t interp) {
  const auto dev = need_cuda({&grad_output, &sample_map, opt(iw)});
  const int layout = layout_of(grad_output);
  check_map(grad_output, sample_map, iw);
  const mc_desc d = pool_desc(grad_output, sample_map, iw, K, interp, layout, IH, IW);
  Tensor gx = empty_in({d.B, d.C_in, IH, IW}, grad_output, layout);
  c10::cuda::CUDAGuard guard(dev);
  int rc = MC_ERR_UNSUPPORTED;
  mc_desc f;
  if (weighted_folds(d, iw, &f) && mc_invmap_bytes(&f) > 0) {
    // weighted map whose points fit the inverse map's records: the same gather, under the folded descriptor
    Tensor inv = inverse_map_weighted(d, f, sample_map, *iw);
    rc = mc_pool_avg_bwd_inv(&f, grad_output.data_ptr(), inv.data_ptr(), gx.data_ptr(), cur_stream());
  } else if (!iw.has_value() && mc_invmap_bytes(&d) > 0) {
    // gather through the inverse map (built once per map tensor): no atomics
    Tensor inv = inverse_map(d, sample_map);
    rc = mc_pool_avg_bwd_inv(&d, grad_output.data_ptr(), inv.data_ptr(), gx.data_ptr(), cur_stream());
  }
  if (rc == MC_ERR_UNSUPPORTED) {
    Scratch ws = scratch(mc_scatter_workspace_bytes(&d), dev);
    rc = mc_pool_avg_bwd(&d, grad_output.data_ptr(), sample_map.data_ptr(), ptr(iw), gx.data_ptr(),
                         ws.p, ws.n, cur_stream());
  }
  check(rc);
  return gx;
}

// ---- resample ---------------------------------------------------------------------------------------------

Tensor resample_to(const Tensor& input, const Tensor& sample_map, const OptTensor& iw, int64_t OH,
                   int64_t OW, int64_t interp) {
  const auto dev = need_cuda({&input, &sample_map, opt(iw)});
  const int layout = layout_of(input);
  check_map(input, sample_map, iw);
  const int64_t B = input.size(0), C = input.size(1), H = input.size(2), W = input.size(3);
  const mc_desc d = make_desc(input.scalar_type(), layout, B, C, C, OH, OW, H, W, 1, n_interp(iw),
                              interp);
  Tensor y = empty_in({B, C, OH, OW}, input, layout);
  c10::cuda::CUDAGuard guard(dev);
  int rc = MC_ERR_UNSUPPORTED;
  mc_desc f;
  if (weighted_folds(d, iw, &f) && mc_invmap_bytes(&f) > 0) {
    Tensor inv = inverse_map_weighted(d, f, sample_map, *iw);
    rc = mc_resample_scatter_inv(&f, input.data_ptr(), inv.data_ptr(), y.data_ptr(), cur_stream());
  } else if (!iw.has_value() && mc_invmap_bytes(&d) > 0) {
    Tensor inv = inverse_map(d, sample_map);
    rc = mc_resample_scatter_inv(&d, input.data_ptr(), inv.data_ptr(), y.data_ptr(), cur_stream());
  }
  if (rc == MC_ERR_UNSUPPORTED) {
    Scratch ws = scratch(mc_scatter_workspace_bytes(&d), dev);
    rc = mc_resample_scatter(&d, input.data_ptr(), sample_map.data_ptr(), ptr(iw), y.data_ptr(), ws.p,
                             ws.n, cur_stream());
  }
  check(rc);
  return y;
}

Tensor resample_from(const Tensor& input, const Tensor& sample_map, const OptTensor& iw,
                     int64_t interp) {
  const auto dev = need_cuda({&input, &sample_map, opt(iw)});
  const int layout = layout_of(input);
  check_map(input, sample_map, iw);
  const int64_t B = input.size(0), C = input.size(1), H = input.size(2), W = input.size(3);
  const int64_t OH = sample_map.size(0), OW = sample_map.size(1);
  const mc_desc d = make_desc(input.scalar_type(), layout, B, C, C, H, W, OH, OW, 1, n_interp(iw),
                              interp);
  Tensor y = empty_in({B, C, OH, OW}, input, layout);
  c10::cuda::CUDAGuard guard(dev);
  check(mc_resample_gather(&d, input.data_ptr(), sample_map.data_ptr(), ptr(iw), y.data_ptr(),
                           cur_stream()));
  return y;
}

// ---- knn ----------------------------------------------------------------------------------------------------

std::vector<Tensor> knn_forward(const Tensor& ref, const Tensor& query, int64_t k) {
  const auto dev = need_cuda({&ref, &query});
  TORCH_CHECK(ref.is_contiguous() && query.is_contiguous(), "ref and query must be contiguous");
  TORCH_CHECK(ref.scalar_type() == at::kFloat && query.scalar_type() == at::kFloat,
              "knn works on float32 points");
  const int64_t B = ref.size(0), D = ref.size(1), M = ref.size(2), N = query.size(2);
  Tensor idx = at::empty({B, k, N}, ref.options().dtype(at::kLong));
  Tensor dist = at::empty({B, k, N}, ref.options());
  c10::cuda::CUDAGuard guard(dev);
  check(mc_knn(ref.data_ptr<float>(), query.data_ptr<float>(), (int32_t)B, (int32_t)D, (int32_t)M,
               (int32_t)N, (int32_t)k, idx.data_ptr<int64_t>(), dist.data_ptr<float>(), cur_stream()));
  return {idx, dist};
}

// ---- cube map -> equirectangular image, voting resample -----------------------------------------------

Tensor cube2rect(const Tensor& cubemap_in, int64_t rect_height, int64_t rect_width, int64_t interpolation) {
  const auto dev = need_cuda({&cubemap_in});
  TORCH_CHECK(cubemap_in.dim() == 3 && cubemap_in.size(2) == 6 * cubemap_in.size(1),
              "cubemap must be (channels, cube_dim, 6 * cube_dim)");
  TORCH_CHECK(cubemap_in.scalar_type() == at::kFloat || cubemap_in.scalar_type() == at::kDouble,
              "cube2rect works on float32 / float64 images");
  TORCH_CHECK(interpolation == 0 || interpolation == 1, "interpolation must be 0 (nearest) or 1 (bilinear)");
  const Tensor cubemap = cubemap_in.contiguous();
  Tensor rect = at::empty({cubemap.size(0), rect_height, rect_width}, cubemap.options());
  c10::cuda::CUDAGuard guard(dev);
  check(mc_cube2rect(cubemap.scalar_type() == at::kDouble ? MC_F64 : MC_F32, cubemap.data_ptr(),
                     (int32_t)cubemap.size(0), (int32_t)cubemap.size(1), (int32_t)rect_height, (int32_t)rect_width,
                     (int32_t)interpolation, rect.data_ptr(), cur_stream()));
  return rect;
}

Tensor voting_resample_to_map(const Tensor& input_in, const Tensor& map_in, int64_t oh, int64_t ow,
                              int64_t num_candidates) {
  const auto dev = need_cuda({&input_in, &map_in});
  TORCH_CHECK(input_in.scalar_type() == at::kLong && map_in.scalar_type() == at::kLong,
              "voting resample works on int64 labels and an int64 map");
  TORCH_CHECK(input_in.dim() == 4 && map_in.dim() == 3 && map_in.size(0) == input_in.size(2) &&
                  map_in.size(1) == input_in.size(3) && map_in.size(2) == 2,
              "input must be (B, C, IH, IW) and sample_map (IH, IW, 2)");
  TORCH_CHECK(num_candidates > 0, "num_candidates must be positive");
  const Tensor input = input_in.contiguous(), map = map_in.contiguous();
  const int64_t B = input.size(0), C = input.size(1), IH = input.size(2), IW = input.size(3);
  Tensor out = at::empty({B, C, oh, ow}, input.options());
  // (vote counters for a slice of the batch at a time: at most ~1 GiB of scratch)
  const int64_t per_image =
      (int64_t)mc_voting_resample_workspace(1, (int32_t)C, (int32_t)oh, (int32_t)ow, (int32_t)num_candidates);
  const int64_t step = std::max<int64_t>(1, std::min<int64_t>(B, (int64_t(1) << 30) / std::max<int64_t>(1, per_image)));
  Tensor ws = at::empty({per_image * step}, input.options().dtype(at::kByte));
  c10::cuda::CUDAGuard guard(dev);
  for (int64_t b0 = 0; b0 < B; b0 += step) {
    const int64_t nb = std::min(step, B - b0);
    check(mc_voting_resample(input.data_ptr<int64_t>() + b0 * C * IH * IW, map.data_ptr<int64_t>(), (int32_t)nb,
                             (int32_t)C, (int32_t)IH, (int32_t)IW, (int32_t)oh, (int32_t)ow,
                             (int32_t)num_candidates, ws.data_ptr(), (size_t)(per_image * nb),
                             out.data_ptr<int64_t>() + b0 * C * oh * ow, cur_stream()));
  }
  return out;
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  namespace py = pybind11;
  m.doc() = "mapped convolution ops on the sm_100a C-ABI library (reference pybind surface)";
  // MappedConvForward / Backward, include/nn/layers/mapped_convolution_layer.h:64-88, :90-135
  m.def("mapped_conv_forward",
        [](const Tensor& x, const Tensor& map, const Tensor& w, const Tensor& b, int64_t k, int64_t i,
           bool relu) { return conv_forward(x, map, c10::nullopt, w, b, k, i, false, relu); },
        py::arg("input"), py::arg("sample_map"), py::arg("weight"), py::arg("bias"),
        py::arg("kernel_size"), py::arg("interpolation"), py::arg("relu") = false);
  m.def("mapped_conv_backward",
        [](const Tensor& gy, const Tensor& map, const Tensor& x, const Tensor& w, const Tensor& b,
           int64_t k, int64_t i, bool need_input_grad, bool need_weight_grad,
           const c10::optional<Tensor>& relu_output) {
          return conv_backward(gy, map, c10::nullopt, x, w, b, k, i, need_input_grad, false,
                               need_weight_grad, relu_output);
        },
        py::arg("grad_output"), py::arg("sample_map"), py::arg("input"), py::arg("weight"),
        py::arg("bias"), py::arg("kernel_size"), py::arg("interpolation"),
        py::arg("need_input_grad") = true, py::arg("need_weight_grad") = true,
        py::arg("relu_output") = py::none());
  // include/nn/layers/weighted_mapped_convolution_layer.h:65-93, :95-150
  m.def("weighted_mapped_conv_forward",
        [](const Tensor& x, const Tensor& map, const Tensor& iw, const Tensor& w, const Tensor& b,
           int64_t k, int64_t i) { return conv_forward(x, map, iw, w, b, k, i); });
  m.def("weighted_mapped_conv_backward",
        [](const Tensor& gy, const Tensor& map, const Tensor& iw, const Tensor& x, const Tensor& w,
           const Tensor& b, int64_t k, int64_t i) {
          return conv_backward(gy, map, iw, x, w, b, k, i, true);
        });
  // include/nn/layers/mapped_transposed_convolution_layer.h:64-92, :94-143
  m.def("mapped_transposed_conv_forward",
        [](const Tensor& x, const Tensor& map, const Tensor& w, const Tensor& b, int64_t oh,
           int64_t ow, int64_t k, int64_t i) {
          return tconv_forward(x, map, c10::nullopt, w, b, oh, ow, k, i);
        });
  m.def("mapped_transposed_conv_backward",
        [](const Tensor& gy, const Tensor& map, const Tensor& x, const Tensor& w, const Tensor& b,
           int64_t k, int64_t i) { return tconv_backward(gy, map, c10::nullopt, x, w, b, k, i); });
  // include/nn/layers/weighted_mapped_transposed_convolution_layer.h:66-98, :100-155
  m.def("weighted_mapped_transposed_conv_forward",
        [](const Tensor& x, const Tensor& map, const Tensor& iw, const Tensor& w, const Tensor& b,
           int64_t oh, int64_t ow, int64_t k, int64_t i) {
          return tconv_forward(x, map, iw, w, b, oh, ow, k, i);
        });
  m.def("weighted_mapped_transposed_conv_backward",
        [](const Tensor& gy, const Tensor& map, const Tensor& iw, const Tensor& x, const Tensor& w,
           const Tensor& b, int64_t k, int64_t i) { return tconv_backward(gy, map, iw, x, w, b, k, i); });
  // include/nn/layers/mapped_max_pooling_layer.h:46-71, :73-98 and the weighted variants
  m.def("mapped_max_pool", [](const Tensor& x, const Tensor& map, int64_t k, int64_t i) {
    return max_pool(x, map, c10::nullopt, k, i);
  });
  m.def("mapped_max_unpool", [](const Tensor& gy, const Tensor& idx, const Tensor& map, int64_t ih,
                                int64_t iw_, int64_t k, int64_t i) {
    return max_unpool(gy, idx, map, c10::nullopt, ih, iw_, k, i);
  });
  m.def("weighted_mapped_max_pool",
        [](const Tensor& x, const Tensor& map, const Tensor& iw, int64_t k, int64_t i) {
          return max_pool(x, map, iw, k, i);
        });
  m.def("weighted_mapped_max_unpool",
        [](const Tensor& gy, const Tensor& idx, const Tensor& map, const Tensor& iw, int64_t ih,
           int64_t iw_, int64_t k, int64_t i) { return max_unpool(gy, idx, map, iw, ih, iw_, k, i); });
  // include/nn/layers/mapped_avg_pooling_layer.h:42-64, :66-88 and the weighted variants
  m.def("mapped_avg_pool", [](const Tensor& x, const Tensor& map, int64_t k, int64_t i) {
    return avg_pool(x, map, c10::nullopt, k, i);
  });
  m.def("mapped_avg_unpool", [](const Tensor& gy, const Tensor& map, int64_t ih, int64_t iw_,
                                int64_t k, int64_t i) {
    return avg_unpool(gy, map, c10::nullopt, ih, iw_, k, i);
  });
  m.def("weighted_mapped_avg_pool",
        [](const Tensor& x, const Tensor& map, const Tensor& iw, int64_t k, int64_t i) {
          return avg_pool(x, map, iw, k, i);
        });
  m.def("weighted_mapped_avg_unpool",
        [](const Tensor& gy, const Tensor& map, const Tensor& iw, int64_t ih, int64_t iw_, int64_t k,
           int64_t i) { return avg_unpool(gy, map, iw, ih, iw_, k, i); });
  // ResampleToMap (scatter) / ResampleFromMap (gather), include/nn/layers/resample_layer.h:38-80,
  // and include/nn/layers/weighted_resample_layer.h:49-103
  m.def("resample_to_map", [](const Tensor& x, const Tensor& map, int64_t oh, int64_t ow, int64_t i) {
    return resample_to(x, map, c10::nullopt, oh, ow, i);
  });
  m.def("resample_from_map", [](const Tensor& x, const Tensor& map, int64_t i) {
    return resample_from(x, map, c10::nullopt, i);
  });
  m.def("weighted_resample_to_map", [](const Tensor& x, const Tensor& map, const Tensor& iw,
                                       int64_t oh, int64_t ow, int64_t i) {
    return resample_to(x, map, iw, oh, ow, i);
  });
  m.def("weighted_resample_from_map",
        [](const Tensor& x, const Tensor& map, const Tensor& iw, int64_t i) {
          return resample_from(x, map, iw, i);
        });
  // KNNForward, include/util/layers/knn_layer.h:25-35 -> [idx (B,k,N) int64 1-based, dist]
  m.def("knn_forward", &knn_forward);
  // Cube2RectForward, include/util/layers/cube2rect_layer.h:14-45
  m.def("cube2rect", &cube2rect);
  // VotingResampleToMap, include/nn/layers/voting_resample_layer.h:34-58
  m.def("voting_resample_to_map", &voting_resample_to_map);
  m.def("clear_plan_cache", &clear_plan_cache);
  m.def("plan_cache_kinds", &plan_cache_kinds);
  // Row plans (the fast path for maps that are translation invariant along image rows) on / off;
  // returns the previous setting.  Off: every map takes the general kernels.
  m.def("set_row_plans", [](bool on) { const bool was = g_row_plans; g_row_plans = on; return was; });
  // Synchronises the current stream and returns the device status word (0 = every kernel ran to
  // completion; otherwise the code of the first bounded device-side wait that ran out, after which
  // the kernel returned early and its output is invalid).  reset clears the word.
  m.def("device_status", [](bool reset) { return mc_device_status(cur_stream(), reset ? 1 : 0); },
        py::arg("reset") = true);
  m.def("abi_version", []() { return mc_abi_version(); });
}
