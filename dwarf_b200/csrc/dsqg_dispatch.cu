// Chooses between the tensor-core kernels (bf16; D in {32, 64} with or without scale_embed,
// D in {96, 128} without) and the generic CUDA-core kernels (everything else: fp32 storage,
// other head sizes, dense windows wider than the tensor-core kernels are built for).  One
// decision per call, made on the host from the shape alone.
#include <atomic>

#include "dsqg_common.cuh"

namespace dsqg {

// 0 = automatic, 1 = always the generic kernels, 2 = the register-fed tensor-core kernels (what the
// automatic choice uses where they apply, except for the one case in umma_pays()), 3 = the forward with TMA-staged V wherever it applies
// (dsqg_staged.cu; not chosen automatically: it measures slower on B200), 4 = the forward with the
// dense window on tcgen05 / tensor memory wherever it applies (dsqg_umma.cu; not chosen automatically).
static std::atomic<int> g_path{0};

// Where the tcgen05 forward measures faster than the register-fed one: 128-byte rows (D = 64), no sparse
// taps, and enough 128-row tiles to keep one persistent block per SM busy (cfg2 shape, offsets 0..31:
// 46.4 us against 56.1 us on B200).
static bool umma_pays(const FwdArgs& a, const Taps& t, int dtype) {
    return a.D == 64 && t.n_sparse == 0 && !a.strided &&
           (long long)a.B * a.H * ((a.N + 127) / 128) >= 2 * 148 && umma_supported(dtype, a.D, t, a.scale_embed != nullptr);
}

cudaError_t launch_fwd(const FwdArgs& a, const Taps& t, int dtype, cudaStream_t s) {
    const int path = g_path.load();
    if (path == 0 && umma_pays(a, t, dtype)) return launch_fwd_umma(a, t, s);
    if (path == 4 && !a.strided && umma_supported(dtype, a.D, t, a.scale_embed != nullptr)) return launch_fwd_umma(a, t, s);
    if (path == 3 && staged_supported(dtype, a.D, t, a.scale_embed != nullptr)) return launch_fwd_staged(a, t, s);
    if (path != 1 && mma_fwd_supported(dtype, a.D, t, a.scale_embed != nullptr)) return launch_fwd_mma(a, t, s);
    return launch_fwd_generic(a, t, dtype, s);
}

cudaError_t launch_bwd(const BwdArgs& a, const Taps& t, int dtype, cudaStream_t s, int stages) {
    const int path = g_path.load();
    if (path != 1 && mma_path_supported(dtype, a.D, t, a.scale_embed != nullptr))
        return launch_bwd_mma(a, t, s, stages);
    return launch_bwd_generic(a, t, dtype, s, stages);
}

}  // namespace dsqg

extern "C" int dsqg_set_kernel_path(int path) {
    if (path < 0 || path > 4) return DSQG_ERR_UNSUPPORTED;
    dsqg::g_path.store(path);
    return DSQG_OK;
}

extern "C" int dsqg_device_error(int reset) {
    int v = 0, w = 0;
    if (dsqg::read_stage_error(&v, reset != 0) != cudaSuccess) return -1;
    if (dsqg::read_umma_error(&w, reset != 0) != cudaSuccess) return -1;
    return v ? v : w;
}

extern "C" int dsqg_test_wait_timeout(long long limit_cycles, void* stream) {
    if (limit_cycles < 1 || limit_cycles > 2000000000LL) return DSQG_ERR_UNSUPPORTED;
    return dsqg::launch_wait_timeout(limit_cycles, 0x7e57, static_cast<cudaStream_t>(stream)) == cudaSuccess ? DSQG_OK : DSQG_ERR_CUDA;
}
