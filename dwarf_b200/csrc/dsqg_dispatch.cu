// Chooses between the tensor-core kernels (bf16, D in {32,64}) and the generic CUDA-core
// kernels.  One decision per call, made on the host from the shape alone.
#include <atomic>

#include "dsqg_common.cuh"

namespace dsqg {

static std::atomic<int> g_path{0};   // 0 = automatic, 1 = always the generic kernels

cudaError_t launch_fwd(const FwdArgs& a, const Taps& t, int dtype, cudaStream_t s) {
    if (g_path.load() == 0 && mma_path_supported(dtype, a.D, t, a.scale_embed != nullptr))
        return launch_fwd_mma(a, t, s);
    return launch_fwd_generic(a, t, dtype, s);
}

cudaError_t launch_bwd(const BwdArgs& a, const Taps& t, int dtype, cudaStream_t s, int stages) {
    if (g_path.load() == 0 && mma_path_supported(dtype, a.D, t, a.scale_embed != nullptr))
        return launch_bwd_mma(a, t, s, stages);
    return launch_bwd_generic(a, t, dtype, s, stages);
}

}  // namespace dsqg

extern "C" int dsqg_set_kernel_path(int path) {
    if (path < 0 || path > 1) return DSQG_ERR_UNSUPPORTED;
    dsqg::g_path.store(path);
    return DSQG_OK;
}
