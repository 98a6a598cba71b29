// Backward of the sigmoid gate that dsqg_fwd_strided folds into its epilogue.
//
// The forward wrote y = o * sigmoid(gate), o being the DSQG output (DWARF
// train/train_2048_condU.py:184-191: `out * torch.sigmoid(self.gate_proj(x))`).  Given dy this
// kernel forms, in one pass over the three tensors,
//   dout  = dy * sigmoid(gate)                    the gradient the DSQG backward consumes,
//   dgate = dy * o * s (1 - s) = dy * y * (1 - s) the gradient of the gate projection's output,
//   delta = sum_d dout * o = sum_d dy * y         per (batch, head, row): what the DSQG backward
//                                                 otherwise derives from its saved output,
// so the un-gated output o never has to be stored.  bf16 tensors, fp32 arithmetic.
#include "dsqg_common.cuh"

namespace dsqg {
namespace {

// one thread per (batch, row, head): D contiguous elements, 8 at a time
__global__ void __launch_bounds__(256)
gate_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ y,
                const __nv_bfloat16* __restrict__ gate, long long sb, long long sh, long long sn,
                __nv_bfloat16* __restrict__ dout, __nv_bfloat16* __restrict__ dgate, float* __restrict__ delta,
                int B, int H, int N, int D) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)B * N * H) return;
    const int h = (int)(idx % H);
    const long long bn = idx / H;
    const int n = (int)(bn % N), b = (int)(bn / N);
    const size_t off = (size_t)b * sb + (size_t)h * sh + (size_t)n * sn;
    float acc = 0.f;
    for (int c = 0; c < D; c += 8) {
        float g[8], d[8], o[8], go[8], gg[8];
        load8(gate + off + c, g); load8(dy + off + c, d); load8(y + off + c, o);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float s = __fdividef(1.f, 1.f + __expf(-g[i]));
            go[i] = d[i] * s;
            gg[i] = d[i] * o[i] * (1.f - s);
            acc = fmaf(d[i], o[i], acc);
        }
        store8(dout + off + c, go); store8(dgate + off + c, gg);
    }
    delta[((size_t)b * H + h) * N + n] = acc;
}

}  // namespace

cudaError_t launch_gate_bwd(const void* dy, const void* y, const void* gate, long long sb, long long sh, long long sn,
                            void* dout, void* dgate, float* delta, int B, int H, int N, int D, cudaStream_t s) {
    const long long total = (long long)B * N * H;
    gate_bwd_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(
        static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(y), static_cast<const __nv_bfloat16*>(gate),
        sb, sh, sn, static_cast<__nv_bfloat16*>(dout), static_cast<__nv_bfloat16*>(dgate), delta, B, H, N, D);
    return cudaGetLastError();
}

}  // namespace dsqg
