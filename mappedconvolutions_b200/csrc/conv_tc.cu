// Tensor-core (tcgen05 + TMEM) mapped convolution kernels.  Placeholder: nothing supported yet.
#include "common.cuh"
namespace mc {
bool conv_tc_fwd_supported(const mc_desc*) { return false; }
int conv_tc_fwd_launch(const mc_desc*, const void*, const void*, const void*, const void*, void*,
                       cudaStream_t) { return MC_ERR_UNSUPPORTED; }
bool conv_tc_dgrad_supported(const mc_desc*) { return false; }
size_t conv_tc_dgrad_ws(const mc_desc*) { return 0; }
int conv_tc_dgrad_launch(const mc_desc*, const void*, const void*, const void*, const void*, void*,
                         void*, size_t, cudaStream_t) { return MC_ERR_UNSUPPORTED; }
bool conv_tc_wgrad_supported(const mc_desc*) { return false; }
size_t conv_tc_wgrad_ws(const mc_desc*) { return 0; }
int conv_tc_wgrad_launch(const mc_desc*, const void*, const void*, const void*, void*, void*, void*,
                         size_t, cudaStream_t) { return MC_ERR_UNSUPPORTED; }
}  // namespace mc
