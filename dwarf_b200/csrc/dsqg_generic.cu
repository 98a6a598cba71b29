// Generic DSQG kernels: any head dim D = 8k <= 128, any tap set, bf16 or fp32 storage,
// fp32 arithmetic on the CUDA cores.  These are the fp32-I/O instantiation (needed for
// the 1e-5 parity gate against the reference's fp32 PyTorch path) and the fall-back for
// shapes the tensor-core kernels do not cover.  Math follows the DWARF reference kernels
// kernels/dsqg_attention_v3.py:60-163 (forward), :198-275 (dQ, dpos_bias, dscale_embed),
// :282-352 (dK, dV), with the offset set as a runtime argument and the per-head output
// gain of train/train_2048_condU.py:187 fused in.
//
// Mapping: a group of TPR = next_pow2(D/8) lanes owns one row; every lane holds 8
// contiguous elements of the row in fp32 registers; dot products are reduced with
// xor-shuffles inside the group.  Global loads are 16/32-byte vectors and consecutive
// lanes read consecutive addresses, so each warp touches whole contiguous rows.
#include "dsqg_common.cuh"

namespace dsqg {

namespace {

constexpr int kThreads = 256;
constexpr int kRowsPerBwdTile = 512;   // rows handled by one dQ block (a multiple of every RPB)

template <typename T> struct Exp;
template <> struct Exp<float> { static __device__ __forceinline__ float f(float x) { return expf(x); } };
template <> struct Exp<__nv_bfloat16> { static __device__ __forceinline__ float f(float x) { return __expf(x); } };

template <typename T, int TPR>
__global__ void __launch_bounds__(kThreads)
fwd_generic_kernel(const FwdArgs a, const Taps t) {
    constexpr int RPB = kThreads / TPR;
    __shared__ float pb_s[DSQG_MAX_TAPS];
    const int bh = blockIdx.y, h = bh % a.H;
    const int g = threadIdx.x / TPR, li = threadIdx.x % TPR;
    const int d0 = li * 8;
    const bool active = d0 < a.D;
    const int n = blockIdx.x * RPB + g;
    const bool row_ok = n < a.N;
    for (int j = threadIdx.x; j < t.J; j += kThreads) pb_s[j] = a.pos_bias[j * a.H + h];
    __syncthreads();

    const T* qb = static_cast<const T*>(a.q) + (size_t)bh * a.N * a.D;
    const T* kb = static_cast<const T*>(a.k) + (size_t)bh * a.N * a.D;
    const T* vb = static_cast<const T*>(a.v) + (size_t)bh * a.N * a.D;
    const bool has_se = a.scale_embed != nullptr;

    float q[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (row_ok && active) load8(qb + (size_t)n * a.D + d0, q);
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    float m = -INFINITY, l = 0.f;

    for (int j = 0; j < t.J; ++j) {
        const int src = n - t.delta(j);
        const bool valid = row_ok && src >= 0;
        float kx[8] = {0, 0, 0, 0, 0, 0, 0, 0}, vx[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (valid && active) {
            load8(kb + (size_t)src * a.D + d0, kx);
            load8(vb + (size_t)src * a.D + d0, vx);
            if (has_se) {
                float se[8];
                load8(a.scale_embed + (size_t)j * a.D + d0, se);
#pragma unroll
                for (int i = 0; i < 8; ++i) kx[i] += se[i];
            }
        }
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) dot = fmaf(q[i], kx[i], dot);
        dot = group_sum<TPR>(dot);
        if (valid) {
            const float s = dot * a.scale + pb_s[j];
            const float mn = fmaxf(m, s);
            const float cor = Exp<T>::f(m - mn);   // m = -inf on the first valid tap -> 0
            const float p = Exp<T>::f(s - mn);
            l = l * cor + p;
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = acc[i] * cor + p * vx[i];
            m = mn;
        }
    }
    if (row_ok) {
        const float gain = a.head_gain ? a.head_gain[h] : 1.f;
        const float inv = l > 0.f ? gain / l : 0.f;
        if (active) {
            float o[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = acc[i] * inv;
            store8(static_cast<T*>(a.out) + ((size_t)bh * a.N + n) * a.D + d0, o);
        }
        if (li == 0) a.lse[(size_t)bh * a.N + n] = l > 0.f ? m + logf(l) : -INFINITY;
    }
}

// dQ + row-wise delta + partial sums of dpos_bias / dhead_gain / dscale_embed.
// One block owns kRowsPerBwdTile consecutive rows of one (b,h) and walks them RPB at a time.
// Dynamic shared memory: ds_s[RPB][J] | dg_s[RPB] | (q_s[RPB][D] | dse_acc[J*D] when SE).
template <typename T, int TPR>
__global__ void __launch_bounds__(kThreads)
bwd_dq_generic_kernel(const BwdArgs a, const Taps t) {
    constexpr int RPB = kThreads / TPR;
    extern __shared__ float smem[];
    __shared__ float pb_s[DSQG_MAX_TAPS];
    const int J = t.J, D = a.D;
    float* ds_s = smem;                  // [RPB][J]
    float* dg_s = ds_s + RPB * J;        // [RPB]
    float* q_s = dg_s + RPB;             // [RPB][D]
    float* dse_acc = q_s + RPB * D;      // [J*D]
    const bool has_se = a.scale_embed != nullptr;

    const int bh = blockIdx.y, h = bh % a.H;
    const int tile = bh * a.tiles_per_bh + blockIdx.x;
    const int row0 = blockIdx.x * kRowsPerBwdTile;
    const int row_end = min(a.N, row0 + kRowsPerBwdTile);
    const int g = threadIdx.x / TPR, li = threadIdx.x % TPR;
    const int d0 = li * 8;
    const bool active = d0 < D;

    for (int j = threadIdx.x; j < J; j += kThreads) pb_s[j] = a.pos_bias[j * a.H + h];
    if (has_se)
        for (int i = threadIdx.x; i < J * D; i += kThreads) dse_acc[i] = 0.f;
    __syncthreads();

    const size_t base = (size_t)bh * a.N * D;
    const T* qb = static_cast<const T*>(a.q) + base;
    const T* kb = static_cast<const T*>(a.k) + base;
    const T* vb = static_cast<const T*>(a.v) + base;
    const T* ob = static_cast<const T*>(a.out) + base;
    const T* dob = static_cast<const T*>(a.dout) + base;
    T* dqb = static_cast<T*>(a.dq) + base;
    const float gain = a.head_gain ? a.head_gain[h] : 1.f;

    float dpb_r = 0.f;   // thread j < J accumulates dpos_bias[j]
    float dg_r = 0.f;    // thread J accumulates sum_rows dout . o_pre

    for (int r0 = row0; r0 < row_end; r0 += RPB) {
        const int n = r0 + g;
        const bool row_ok = n < row_end;
        float q[8] = {0, 0, 0, 0, 0, 0, 0, 0}, dox[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        float delta = 0.f, lse_n = 0.f;
        if (row_ok && active) {
            float o[8];
            load8(qb + (size_t)n * D + d0, q);
            load8(dob + (size_t)n * D + d0, dox);
            load8(ob + (size_t)n * D + d0, o);
#pragma unroll
            for (int i = 0; i < 8; ++i) delta = fmaf(dox[i], o[i], delta);
        }
        delta = group_sum<TPR>(delta);
        if (row_ok) {
            lse_n = a.lse[(size_t)bh * a.N + n];
            if (li == 0) a.delta[(size_t)bh * a.N + n] = delta;
        }
        float dq[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        float dgrow = 0.f;
        for (int j = 0; j < J; ++j) {
            const int src = n - t.delta(j);
            const bool valid = row_ok && src >= 0;
            float kx[8] = {0, 0, 0, 0, 0, 0, 0, 0}, vx[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            if (valid && active) {
                load8(kb + (size_t)src * D + d0, kx);
                load8(vb + (size_t)src * D + d0, vx);
                if (has_se) {
                    float se[8];
                    load8(a.scale_embed + (size_t)j * D + d0, se);
#pragma unroll
                    for (int i = 0; i < 8; ++i) kx[i] += se[i];
                }
            }
            float dot_s = 0.f, dot_p = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) { dot_s = fmaf(q[i], kx[i], dot_s); dot_p = fmaf(dox[i], vx[i], dot_p); }
            dot_s = group_sum<TPR>(dot_s);
            dot_p = group_sum<TPR>(dot_p);
            float ds = 0.f;
            if (valid) {
                const float s = dot_s * a.scale + pb_s[j];
                const float p = Exp<T>::f(s - lse_n);
                ds = p * (gain * dot_p - delta);
                dgrow = fmaf(p, dot_p, dgrow);
                const float w = ds * a.scale;
#pragma unroll
                for (int i = 0; i < 8; ++i) dq[i] = fmaf(w, kx[i], dq[i]);
            }
            if (li == 0) ds_s[g * J + j] = ds;
        }
        if (row_ok && active) store8(dqb + (size_t)n * D + d0, dq);
        if (li == 0) dg_s[g] = row_ok ? dgrow : 0.f;
        if (has_se && active) {
#pragma unroll
            for (int i = 0; i < 8; ++i) q_s[g * D + d0 + i] = q[i];   // zeros for rows past the end
        }
        __syncthreads();
        if (threadIdx.x < J) {
            for (int r = 0; r < RPB; ++r) dpb_r += ds_s[r * J + threadIdx.x];
        } else if (threadIdx.x == J) {
            for (int r = 0; r < RPB; ++r) dg_r += dg_s[r];
        }
        if (has_se) {
            for (int idx = threadIdx.x; idx < J * D; idx += kThreads) {
                const int j = idx / D, d = idx - j * D;
                float acc = dse_acc[idx];
                for (int r = 0; r < RPB; ++r) acc = fmaf(ds_s[r * J + j], q_s[r * D + d], acc);
                dse_acc[idx] = acc;
            }
        }
        __syncthreads();
    }
    if (threadIdx.x < J) a.dpb_part[(size_t)tile * J + threadIdx.x] = dpb_r;
    else if (threadIdx.x == J) a.dg_part[tile] = dg_r;
    if (has_se)
        for (int idx = threadIdx.x; idx < J * D; idx += kThreads)
            a.dse_part[(size_t)tile * J * D + idx] = dse_acc[idx] * a.scale;
}

// dK, dV: the group owns key row m and visits the query rows m + delta_j that read it.
template <typename T, int TPR>
__global__ void __launch_bounds__(kThreads)
bwd_dkdv_generic_kernel(const BwdArgs a, const Taps t) {
    constexpr int RPB = kThreads / TPR;
    __shared__ float pb_s[DSQG_MAX_TAPS];
    const int J = t.J, D = a.D;
    const int bh = blockIdx.y, h = bh % a.H;
    const int g = threadIdx.x / TPR, li = threadIdx.x % TPR;
    const int d0 = li * 8;
    const bool active = d0 < D;
    const int m = blockIdx.x * RPB + g;
    const bool row_ok = m < a.N;
    for (int j = threadIdx.x; j < J; j += kThreads) pb_s[j] = a.pos_bias[j * a.H + h];
    __syncthreads();

    const size_t base = (size_t)bh * a.N * D;
    const T* qb = static_cast<const T*>(a.q) + base;
    const T* dob = static_cast<const T*>(a.dout) + base;
    const float* lse_b = a.lse + (size_t)bh * a.N;
    const float* delta_b = a.delta + (size_t)bh * a.N;
    const float gain = a.head_gain ? a.head_gain[h] : 1.f;
    const bool has_se = a.scale_embed != nullptr;

    float kx[8] = {0, 0, 0, 0, 0, 0, 0, 0}, vx[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (row_ok && active) {
        load8(static_cast<const T*>(a.k) + base + (size_t)m * D + d0, kx);
        load8(static_cast<const T*>(a.v) + base + (size_t)m * D + d0, vx);
    }
    float dk[8] = {0, 0, 0, 0, 0, 0, 0, 0}, dv[8] = {0, 0, 0, 0, 0, 0, 0, 0};

    for (int j = 0; j < J; ++j) {
        const int n = m + t.delta(j);
        const bool valid = row_ok && n < a.N;
        float qx[8] = {0, 0, 0, 0, 0, 0, 0, 0}, dox[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        float kk[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) kk[i] = kx[i];
        if (valid && active) {
            load8(qb + (size_t)n * D + d0, qx);
            load8(dob + (size_t)n * D + d0, dox);
            if (has_se) {
                float se[8];
                load8(a.scale_embed + (size_t)j * D + d0, se);
#pragma unroll
                for (int i = 0; i < 8; ++i) kk[i] += se[i];
            }
        }
        float dot_s = 0.f, dot_p = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) { dot_s = fmaf(qx[i], kk[i], dot_s); dot_p = fmaf(dox[i], vx[i], dot_p); }
        dot_s = group_sum<TPR>(dot_s);
        dot_p = group_sum<TPR>(dot_p);
        if (valid) {
            const float s = dot_s * a.scale + pb_s[j];
            const float p = Exp<T>::f(s - lse_b[n]);
            const float ds = p * (gain * dot_p - delta_b[n]);
            const float wv = p * gain, wk = ds * a.scale;
#pragma unroll
            for (int i = 0; i < 8; ++i) { dv[i] = fmaf(wv, dox[i], dv[i]); dk[i] = fmaf(wk, qx[i], dk[i]); }
        }
    }
    if (row_ok && active) {
        store8(static_cast<T*>(a.dk) + base + (size_t)m * D + d0, dk);
        store8(static_cast<T*>(a.dv) + base + (size_t)m * D + d0, dv);
    }
}

}  // namespace

// One block per output element; the partials are summed in a fixed order (per-thread strided
// partial sums, then a fixed shared-memory tree), so the result is bitwise reproducible.
__global__ void __launch_bounds__(kReduceThreads)
bwd_reduce_params_kernel(const BwdArgs a, const int J) {
    __shared__ float red[kReduceThreads];
    reduce_one_param(a, J, blockIdx.x, red);
}

cudaError_t launch_reduce_params(const BwdArgs& a, int J, cudaStream_t s) {
    const int total = J * a.H + a.H + ((a.dscale_embed && a.scale_embed) ? J * a.D : 0);
    bwd_reduce_params_kernel<<<total, kReduceThreads, 0, s>>>(a, J);
    return cudaGetLastError();
}

namespace {
template <typename T, int TPR>
cudaError_t fwd_launch(const FwdArgs& a, const Taps& t, cudaStream_t s) {
    constexpr int RPB = kThreads / TPR;
    dim3 grid((a.N + RPB - 1) / RPB, a.B * a.H);
    fwd_generic_kernel<T, TPR><<<grid, kThreads, 0, s>>>(a, t);
    return cudaGetLastError();
}

template <typename T, int TPR>
cudaError_t bwd_launch(BwdArgs a, const Taps& t, cudaStream_t s, int stages) {
    constexpr int RPB = kThreads / TPR;
    const bool has_se = a.scale_embed != nullptr;
    carve_bwd_scratch(a, kRowsPerBwdTile, t.J, has_se);
    size_t smem = sizeof(float) * ((size_t)RPB * t.J + RPB + (has_se ? (size_t)RPB * a.D + (size_t)t.J * a.D : 0));
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(bwd_dq_generic_kernel<T, TPR>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    cudaError_t e = cudaSuccess;
    if (stages & DSQG_BWD_STAGE_DQ) {
        dim3 grid_q(a.tiles_per_bh, a.B * a.H);
        bwd_dq_generic_kernel<T, TPR><<<grid_q, kThreads, smem, s>>>(a, t);
        if ((e = cudaGetLastError()) != cudaSuccess) return e;
    }
    if (stages & DSQG_BWD_STAGE_DKDV) {
        dim3 grid_k((a.N + RPB - 1) / RPB, a.B * a.H);
        bwd_dkdv_generic_kernel<T, TPR><<<grid_k, kThreads, 0, s>>>(a, t);
        if ((e = cudaGetLastError()) != cudaSuccess) return e;
    }
    if (stages & DSQG_BWD_STAGE_REDUCE) e = launch_reduce_params(a, t.J, s);
    return e;
}

}  // namespace

#define DSQG_DISPATCH_TPR(FN, T, ARGS, ...)                                   \
    do {                                                                      \
        const int chunks_ = (ARGS).D / 8;                                     \
        if (chunks_ <= 1) return FN<T, 1>(ARGS, __VA_ARGS__);                 \
        if (chunks_ <= 2) return FN<T, 2>(ARGS, __VA_ARGS__);                 \
        if (chunks_ <= 4) return FN<T, 4>(ARGS, __VA_ARGS__);                 \
        if (chunks_ <= 8) return FN<T, 8>(ARGS, __VA_ARGS__);                 \
        return FN<T, 16>(ARGS, __VA_ARGS__);                                  \
    } while (0)

cudaError_t launch_fwd_generic(const FwdArgs& a, const Taps& t, int dtype, cudaStream_t s) {
    if (dtype == DSQG_DTYPE_BF16) DSQG_DISPATCH_TPR(fwd_launch, __nv_bfloat16, a, t, s);
    DSQG_DISPATCH_TPR(fwd_launch, float, a, t, s);
}

cudaError_t launch_bwd_generic(const BwdArgs& a, const Taps& t, int dtype, cudaStream_t s, int stages) {
    if (dtype == DSQG_DTYPE_BF16) DSQG_DISPATCH_TPR(bwd_launch, __nv_bfloat16, a, t, s, stages);
    DSQG_DISPATCH_TPR(bwd_launch, float, a, t, s, stages);
}

}  // namespace dsqg
