// Causal mean along the sequence: out[b,n,:] = (x[b,0,:] + ... + x[b,n,:]) / (n + 1).
//
// This is the pooling of the DWARF condU "interference" block, which feeds the K/V injection of
// its DSQG layer: `pool = xi.cumsum(dim=1) / counts` (train/train_2048_condU.py:289-292).  The
// reference runs a cumsum in the activation dtype and a divide; here one kernel reads x twice and
// writes the mean once, accumulating in fp32 whatever the storage type.
// REVERSE is its adjoint (the backward pass): out[b,n,:] = sum_{m >= n} x[b,m,:] / (m + 1).
//
// One thread block takes kGroups slices of 8 contiguous channels of one batch entry over the whole
// sequence, split into kChunks consecutive chunks of rows: every thread sums its chunk, the chunk
// sums are combined through shared memory, then every thread walks its chunk again with the
// running sum.  No scratch memory, no atomics, fixed order of additions.
#include "dsqg_common.cuh"

namespace dsqg {
namespace {

constexpr int kChunks = 32, kGroups = 8;

template <typename T, bool REVERSE>
__global__ void __launch_bounds__(kChunks * kGroups)
causal_mean_kernel(const T* __restrict__ x, T* __restrict__ out, int N, int D) {
    __shared__ float part[kChunks][kGroups][8];
    const int grp = threadIdx.x % kGroups, chunk = threadIdx.x / kGroups;
    const int d0 = (blockIdx.x * kGroups + grp) * 8;
    const bool active = d0 < D;
    const int len = (N + kChunks - 1) / kChunks;
    const int r0 = chunk * len, r1 = min(N, r0 + len);
    const T* xp = x + (size_t)blockIdx.y * N * D + d0;
    T* op = out + (size_t)blockIdx.y * N * D + d0;
    float s[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (active) {
        for (int r = r0; r < r1; ++r) {
            float v[8];
            load8(xp + (size_t)r * D, v);
            const float w = REVERSE ? 1.f / (float)(r + 1) : 1.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) s[i] = fmaf(v[i], w, s[i]);
        }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) part[chunk][grp][i] = s[i];
    __syncthreads();
    if (!active) return;
    // what lies before (forward) or after (reverse) this thread's chunk
    float run[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (REVERSE) {
        for (int c = kChunks - 1; c > chunk; --c)
#pragma unroll
            for (int i = 0; i < 8; ++i) run[i] += part[c][grp][i];
        for (int r = r1 - 1; r >= r0; --r) {
            float v[8], o[8];
            load8(xp + (size_t)r * D, v);
            const float w = 1.f / (float)(r + 1);
#pragma unroll
            for (int i = 0; i < 8; ++i) { run[i] = fmaf(v[i], w, run[i]); o[i] = run[i]; }
            store8(op + (size_t)r * D, o);
        }
    } else {
        for (int c = 0; c < chunk; ++c)
#pragma unroll
            for (int i = 0; i < 8; ++i) run[i] += part[c][grp][i];
        for (int r = r0; r < r1; ++r) {
            float v[8], o[8];
            load8(xp + (size_t)r * D, v);
            const float w = 1.f / (float)(r + 1);
#pragma unroll
            for (int i = 0; i < 8; ++i) { run[i] += v[i]; o[i] = run[i] * w; }
            store8(op + (size_t)r * D, o);
        }
    }
}

}  // namespace

cudaError_t launch_causal_mean(const void* x, void* out, int B, int N, int D, int dtype, bool reverse, cudaStream_t s) {
    dim3 grid((D / 8 + kGroups - 1) / kGroups, B);
    const int threads = kChunks * kGroups;
    if (dtype == DSQG_DTYPE_BF16) {
        auto xi = static_cast<const __nv_bfloat16*>(x); auto oi = static_cast<__nv_bfloat16*>(out);
        if (reverse) causal_mean_kernel<__nv_bfloat16, true><<<grid, threads, 0, s>>>(xi, oi, N, D);
        else causal_mean_kernel<__nv_bfloat16, false><<<grid, threads, 0, s>>>(xi, oi, N, D);
    } else {
        auto xi = static_cast<const float*>(x); auto oi = static_cast<float*>(out);
        if (reverse) causal_mean_kernel<float, true><<<grid, threads, 0, s>>>(xi, oi, N, D);
        else causal_mean_kernel<float, false><<<grid, threads, 0, s>>>(xi, oi, N, D);
    }
    return cudaGetLastError();
}

}  // namespace dsqg
