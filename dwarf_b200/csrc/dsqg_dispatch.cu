// Chooses between the tensor-core kernels (bf16; D in {32, 64} with or without scale_embed,
// D in {96, 128} without) and the generic CUDA-core kernels (everything else: fp32 storage,
// other head sizes, dense windows wider than the tensor-core kernels are built for).  One
// decision per call, made on the host from the shape alone.
#include <atomic>

#include "dsqg_common.cuh"

namespace dsqg {

// 0 = automatic, 1 = always the generic kernels, 2 = tensor-core kernels (same as automatic
// where they apply), 3 = persistent TMA variants wherever they exist.  The TMA variants are not
// chosen automatically: on B200 they measure 10-50 % slower than the plain tensor-core kernels,
// which need fewer registers and keep 20-24 warps resident per SM instead of 9-16.
static std::atomic<int> g_path{0};

cudaError_t launch_fwd(const FwdArgs& a, const Taps& t, int dtype, cudaStream_t s) {
    const int path = g_path.load();
    if (path == 3 && tma_fwd_supported(dtype, a.D, a.N, t, a.scale_embed != nullptr)) return launch_fwd_tma(a, t, s);
    if (path != 1 && mma_fwd_supported(dtype, a.D, t, a.scale_embed != nullptr)) return launch_fwd_mma(a, t, s);
    return launch_fwd_generic(a, t, dtype, s);
}

cudaError_t launch_bwd(const BwdArgs& a, const Taps& t, int dtype, cudaStream_t s, int stages) {
    const int path = g_path.load();
    if (path == 3 && tma_bwd_supported(dtype, a.D, a.N, t, a.scale_embed != nullptr)) return launch_bwd_tma(a, t, s, stages);
    if (path != 1 && mma_path_supported(dtype, a.D, t, a.scale_embed != nullptr))
        return launch_bwd_mma(a, t, s, stages);
    return launch_bwd_generic(a, t, dtype, s, stages);
}

}  // namespace dsqg

extern "C" int dsqg_set_kernel_path(int path) {
    if (path < 0 || path > 3) return DSQG_ERR_UNSUPPORTED;
    dsqg::g_path.store(path);
    return DSQG_OK;
}

extern "C" int dsqg_device_error(int reset) {
    int v = 0;
    int w = 0;
    if (dsqg::read_device_error_fwd_tma(&v, reset != 0) != cudaSuccess) return -1;
    if (dsqg::read_device_error_bwd_tma(&w, reset != 0) != cudaSuccess) return -1;
    return v ? v : w;
}
