// dsqg_bwd_static: the backward pass for callers that have no way to allocate device memory.
//
// Some hosts of this library cannot hand dsqg_bwd a scratch buffer: a serving process whose
// device memory was carved up completely at start-up, a plugin host that only lends the
// plugin the tensors of the current call, or code that runs where the CUDA allocator must
// not be entered.  For them the scratch lives in the library image itself: a fixed array in
// device global memory that every GPU holds from the moment it loads this library until
// the process exits.
#include <mutex>

#include "dsqg_common.cuh"

namespace dsqg {
namespace {

// The built-in scratch.  In host code this name is only a handle for the symbol, never a
// device address; the address of each device's copy comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_static_bwd_scratch[DSQG_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void* g_scratch_addr[kMaxDevices] = {nullptr};   // per device, filled on that device's first call

// Address of the current device's copy of the array (looked up once per device and kept for
// the life of the process: the entry point assumes the device's primary context and that the
// caller never calls cudaDeviceReset; a host that binds another context of the same device, or
// resets it, would be handed a stale address).
cudaError_t static_scratch(void** ptr) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!g_scratch_addr[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_bwd_scratch);   // resolves the symbol on the current device
        if (e != cudaSuccess) return e;
        g_scratch_addr[dev] = p;
    }
    *ptr = g_scratch_addr[dev];
    return cudaSuccess;
}

}  // namespace
}  // namespace dsqg

extern "C" int dsqg_bwd_static(const void* q, const void* k, const void* v,
                               const float* pos_bias, const float* scale_embed, const float* head_gain,
                               const int32_t* offsets, int J,
                               const void* out, const float* lse, const void* dout,
                               void* dq, void* dk, void* dv,
                               float* dpos_bias, float* dscale_embed, float* dhead_gain,
                               int B, int H, int N, int D, int dtype, void* stream) {
    const size_t need = dsqg_bwd_scratch_bytes(J, B, H, N, D, scale_embed != nullptr);
    if (need == 0) {
        // let the regular entry point name the argument error (it returns before using scratch)
        return dsqg_bwd(q, k, v, pos_bias, scale_embed, head_gain, offsets, J, out, lse, dout, dq, dk, dv,
                        dpos_bias, dscale_embed, dhead_gain, reinterpret_cast<void*>(256), 0, B, H, N, D, dtype, stream);
    }
    if (need > (size_t)DSQG_STATIC_SCRATCH_BYTES) return DSQG_ERR_STATIC_SCRATCH_EXCEEDED;
    void* scratch = nullptr;
    if (dsqg::static_scratch(&scratch) != cudaSuccess) return DSQG_ERR_CUDA;
    return dsqg_bwd(q, k, v, pos_bias, scale_embed, head_gain, offsets, J, out, lse, dout, dq, dk, dv,
                    dpos_bias, dscale_embed, dhead_gain, scratch, DSQG_STATIC_SCRATCH_BYTES, B, H, N, D, dtype, stream);
}
