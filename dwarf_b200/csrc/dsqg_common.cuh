// Shared declarations for the DSQG CUDA sources (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "dsqg_b200.h"

namespace dsqg {

// The tap set, passed to every kernel by value (constant parameter space): no global
// state, so launches are re-entrant.  The leading run of consecutive offsets
// d_lo, d_lo+1, ..., d_lo+n_dense-1 is the dense window; sparse[] holds the rest.
struct Taps {
    int J;         // total number of taps
    int n_dense;   // taps 0 .. n_dense-1 are d_lo + j
    int d_lo;      // first (smallest) offset
    int n_sparse;  // J - n_dense
    int sparse[DSQG_MAX_TAPS];

    __host__ __device__ __forceinline__ int delta(int j) const {
        return j < n_dense ? d_lo + j : sparse[j - n_dense];
    }
};

struct FwdArgs {
    const void* q; const void* k; const void* v;
    const float* pos_bias; const float* scale_embed; const float* head_gain;
    void* out; float* lse;
    int B, H, N, D;
    float scale;   // 1/sqrt(D)
    // Strided addressing (tensor-core kernels only; strided == 0: everything is contiguous [B,H,N,D]).
    // Element strides of batch, head and row for q, k, v (in_*) and for out and gate (out_*); the D
    // elements of a row are contiguous.  gate (nullable, bf16, laid out like out): out *= sigmoid(gate).
    int strided;
    long long in_sb, in_sh, in_sn, out_sb, out_sh, out_sn;
    const void* gate;
};

struct BwdArgs {
    const void* q; const void* k; const void* v;
    const float* pos_bias; const float* scale_embed; const float* head_gain;
    const void* out; const float* lse; const void* dout;
    void* dq; void* dk; void* dv;
    float* dpos_bias; float* dscale_embed; float* dhead_gain;
    void* scratch; size_t scratch_bytes;
    // scratch carve-up (all fp32), filled in by carve_bwd_scratch() inside each launcher
    float* delta;      // [B*H*N] sum_d dout*out per row; the tensor-core kernels keep {lse*log2e, delta} pairs here ([B*H*N] float2)
    float* dpb_part;   // [n_tiles, J]
    float* dg_part;    // [n_tiles]
    float* dse_part;   // [n_dse_blocks, J, D] (only with scale_embed)
    float* qs_rows;    // [B*H*N, Jp] q.scale_embed[j] + pos_bias[j]/scale per row (tensor-core kernels with scale_embed)
    void* se_pre;      // tables of se_prep_kernel: split scale_embed, its dS.SE fragments, pos_bias/scale, offsets (same kernels)
    float* dse_tmp;    // [n_tiles, J, D] dscale_embed partial of every 64-row tile (same kernels)
    int n_tiles, tiles_per_bh, n_dse_blocks;
    int B, H, N, D;
    float scale;
    // Strided addressing as in FwdArgs: in_* for q, k, v, dq, dk, dv; out_* for out and dout.
    // delta_pre (nullable, [B,H,N] fp32): sum_d dout*out per row when an earlier kernel formed it.
    int strided;
    long long in_sb, in_sh, in_sn, out_sb, out_sh, out_sn;
    const float* delta_pre;
};

struct DecodeArgs {
    const void* q; const void* k_new; const void* v_new;
    void* k_ring; void* v_ring;
    const int32_t* head; const int32_t* fill;
    const float* pos_bias; const float* scale_embed; const float* head_gain;
    void* out;
    int S, H, D, R;
    float scale;
    int ring_stride;   // elements between two slots of a ring: D for separate K and V rings [S,H,R,D], 2 D for one ring [S,H,R,2,D]
};

// Launchers (defined in the .cu files; return a cudaError_t from the launch).
cudaError_t launch_fwd(const FwdArgs& a, const Taps& t, int dtype, cudaStream_t s);   // dispatcher
cudaError_t launch_bwd(const BwdArgs& a, const Taps& t, int dtype, cudaStream_t s, int stages);   // dispatcher
cudaError_t launch_fwd_generic(const FwdArgs& a, const Taps& t, int dtype, cudaStream_t s);
cudaError_t launch_bwd_generic(const BwdArgs& a, const Taps& t, int dtype, cudaStream_t s, int stages);
cudaError_t launch_reduce_params(const BwdArgs& a, int J, cudaStream_t s);
cudaError_t launch_decode(const DecodeArgs& a, const Taps& t, int dtype, cudaStream_t s, bool overlap);
cudaError_t launch_ring_prefill(const void* k, const void* v, void* k_ring, void* v_ring, int32_t* head, int32_t* fill,
                                int S, int H, int N, int D, int R, int dtype, cudaStream_t s, bool interleaved = false);

cudaError_t launch_causal_mean(const void* x, void* out, int B, int N, int D, int dtype, bool reverse, cudaStream_t s);
cudaError_t launch_gate_bwd(const void* dy, const void* y, const void* gate, long long sb, long long sh, long long sn,
                            void* dout, void* dgate, float* delta, int B, int H, int N, int D, cudaStream_t s);
cudaError_t launch_fwd_mma(const FwdArgs& a, const Taps& t, cudaStream_t s);
cudaError_t launch_bwd_mma(const BwdArgs& a, const Taps& t, cudaStream_t s, int stages);
bool mma_path_supported(int dtype, int D, const Taps& t, bool has_scale_embed);   // backward
bool mma_fwd_supported(int dtype, int D, const Taps& t, bool has_scale_embed);
// forward with TMA-staged V (dsqg_staged.cu)
bool staged_supported(int dtype, int D, const Taps& t, bool has_scale_embed);
cudaError_t launch_fwd_staged(const FwdArgs& a, const Taps& t, cudaStream_t s);
cudaError_t read_stage_error(int* value, bool reset);
cudaError_t launch_wait_timeout(long long limit_cycles, int site, cudaStream_t s);
// forward with the dense window on tcgen05 tensor cores and tensor memory (dsqg_umma.cu)
bool umma_supported(int dtype, int D, const Taps& t, bool has_scale_embed);
cudaError_t launch_fwd_umma(const FwdArgs& a, const Taps& t, cudaStream_t s);
cudaError_t read_umma_error(int* value, bool reset);

// Backward scratch layout: row statistics (8 bytes per row) | dpos_bias partials | dhead_gain partials | dscale_embed
// partials, each block rounded up to 256 bytes.  A "tile" is the set of rows whose partial
// sums one thread block produces; kernels differ in rows_per_tile, so each launcher carves
// for itself and the size query reserves room for the finest tiling in use.
constexpr int kMinRowsPerBwdTile = 64;
inline size_t round256(size_t bytes) { return (bytes + 255) / 256 * 256; }
inline size_t bwd_scratch_need(int rows_per_tile, int J, int B, int H, int N, int D, bool has_se) {
    const size_t tiles = (size_t)B * H * ((N + rows_per_tile - 1) / rows_per_tile);
    return round256((size_t)B * H * N * 8) + round256(tiles * J * 4) + round256(tiles * 4) +
           (has_se ? round256(tiles * J * D * 4) : 0);
}
// Tensor-core kernels with scale_embed: 64-row tiles, dscale_embed partials per group of
// kSeGroup consecutive tiles of a sequence, and the per-row table qs_rows[B*H*N][Jp], Jp = J rounded up to 8.
constexpr int kSeGroup = 8;
// split scale_embed | dS.SE fragments | pos_bias/scale per head [H][Jp] | dense-window offset table (<= 10 n-tiles)
inline size_t se_pre_bytes(int J, int D, int H) {
    const size_t Jp = (J + 7) / 8 * 8, JS = (J + 15) / 16 * 16;
    return 2 * Jp * D * 2 + (JS / 16) * (D / 8) * 32 * 8 + (size_t)H * Jp * 4 + 10 * 32 * 16;
}
inline size_t bwd_scratch_need_mma_se(int J, int B, int H, int N, int D) {
    const size_t tiles_bh = (N + kMinRowsPerBwdTile - 1) / kMinRowsPerBwdTile;
    const size_t tiles = (size_t)B * H * tiles_bh;
    const size_t clusters = (size_t)B * H * ((tiles_bh + kSeGroup - 1) / kSeGroup);
    const size_t Jp = (J + 7) / 8 * 8;
    return round256((size_t)B * H * N * 8) + round256(tiles * J * 4) + round256(tiles * 4) +
           round256(clusters * J * D * 4) + round256((size_t)B * H * N * Jp * 4) + round256(se_pre_bytes(J, D, H)) +
           round256(tiles * J * D * 4);
}
inline void carve_bwd_scratch_mma_se(BwdArgs& a, int J) {
    a.tiles_per_bh = (a.N + kMinRowsPerBwdTile - 1) / kMinRowsPerBwdTile;
    a.n_tiles = a.B * a.H * a.tiles_per_bh;
    a.n_dse_blocks = a.B * a.H * ((a.tiles_per_bh + kSeGroup - 1) / kSeGroup);
    const size_t Jp = (J + 7) / 8 * 8;
    char* p = static_cast<char*>(a.scratch);
    a.delta = reinterpret_cast<float*>(p);    p += round256((size_t)a.B * a.H * a.N * 8);
    a.dpb_part = reinterpret_cast<float*>(p); p += round256((size_t)a.n_tiles * J * 4);
    a.dg_part = reinterpret_cast<float*>(p);  p += round256((size_t)a.n_tiles * 4);
    a.dse_part = reinterpret_cast<float*>(p); p += round256((size_t)a.n_dse_blocks * J * a.D * 4);
    a.qs_rows = reinterpret_cast<float*>(p);  p += round256((size_t)a.B * a.H * a.N * Jp * 4);
    a.se_pre = p;                             p += round256(se_pre_bytes(J, a.D, a.H));
    a.dse_tmp = reinterpret_cast<float*>(p);
}
inline void carve_bwd_scratch(BwdArgs& a, int rows_per_tile, int J, bool has_se) {
    a.tiles_per_bh = (a.N + rows_per_tile - 1) / rows_per_tile;
    a.n_tiles = a.B * a.H * a.tiles_per_bh;
    a.n_dse_blocks = a.n_tiles;
    char* p = static_cast<char*>(a.scratch);
    a.delta = reinterpret_cast<float*>(p);    p += round256((size_t)a.B * a.H * a.N * 8);
    a.dpb_part = reinterpret_cast<float*>(p); p += round256((size_t)a.n_tiles * J * 4);
    a.dg_part = reinterpret_cast<float*>(p);  p += round256((size_t)a.n_tiles * 4);
    a.dse_part = has_se ? reinterpret_cast<float*>(p) : nullptr;
    a.qs_rows = nullptr;
    a.se_pre = nullptr;
    a.dse_tmp = nullptr;
}

// ---------------------------------------------------------------------------------
// Device helpers: 8-element row slices in fp32 registers, from bf16 or fp32 storage.
// ---------------------------------------------------------------------------------
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&x)[8]) {
    uint4 u = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        x[2 * i]     = __uint_as_float(w[i] << 16);
        x[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}
__device__ __forceinline__ void load8(const float* p, float (&x)[8]) {
    float4 a = *reinterpret_cast<const float4*>(p);
    float4 b = *reinterpret_cast<const float4*>(p + 4);
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
    x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&x)[8]) {
    uint4 u;
    u.x = pack_bf16x2(x[0], x[1]); u.y = pack_bf16x2(x[2], x[3]);
    u.z = pack_bf16x2(x[4], x[5]); u.w = pack_bf16x2(x[6], x[7]);
    *reinterpret_cast<uint4*>(p) = u;
}
__device__ __forceinline__ void store8(float* p, const float (&x)[8]) {
    *reinterpret_cast<float4*>(p)     = make_float4(x[0], x[1], x[2], x[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(x[4], x[5], x[6], x[7]);
}

// One output of the parameter-gradient reduction: the per-tile partial sums of dpos_bias[j,h]
// (idx < J*H), dhead_gain[h] (next H) or dscale_embed[j,d] (rest) are added by the
// kReduceThreads threads of a block in a fixed order (strided partial sums, then a fixed
// shared-memory tree), so the result is bitwise reproducible whichever kernel runs it.
constexpr int kReduceThreads = 128;
__device__ __forceinline__ void reduce_one_param(const BwdArgs& a, int J, int idx, float* red) {
    const int n_pb = J * a.H;
    const int per_h = a.B * a.tiles_per_bh;          // partials per (.., h): b-major, then tile
    float s = 0.f;
    float* dst = nullptr;
    if (idx < n_pb) {
        const int j = idx / a.H, h = idx - j * a.H;
        for (int i = threadIdx.x; i < per_h; i += kReduceThreads) {
            const int b = i / a.tiles_per_bh, c = i - b * a.tiles_per_bh;
            s += a.dpb_part[((size_t)(b * a.H + h) * a.tiles_per_bh + c) * J + j];
        }
        dst = a.dpos_bias + idx;
    } else if (idx < n_pb + a.H) {
        const int h = idx - n_pb;
        if (a.dhead_gain) {
            for (int i = threadIdx.x; i < per_h; i += kReduceThreads) {
                const int b = i / a.tiles_per_bh, c = i - b * a.tiles_per_bh;
                s += a.dg_part[(size_t)(b * a.H + h) * a.tiles_per_bh + c];
            }
            dst = a.dhead_gain + h;
        }
    } else if (a.dscale_embed && a.scale_embed) {
        const int e = idx - n_pb - a.H;
        for (int tl = threadIdx.x; tl < a.n_dse_blocks; tl += kReduceThreads)
            s += a.dse_part[(size_t)tl * J * a.D + e];
        dst = a.dscale_embed + e;
    }
    red[threadIdx.x] = s;
    __syncthreads();
    for (int o = kReduceThreads / 2; o > 0; o >>= 1) {
        if (threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
        __syncthreads();
    }
    if (threadIdx.x == 0 && dst) *dst = red[0];
    __syncthreads();
}

template <int WIDTH>
__device__ __forceinline__ float group_sum(float x) {
#pragma unroll
    for (int o = WIDTH / 2; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
}

}  // namespace dsqg
