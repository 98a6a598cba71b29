// Tensor-core DSQG kernels (bf16 storage, fp32 accumulate) for D in {32, 64}.
//
// One warp owns 16 consecutive rows of one (batch, head) sequence.  The dense window is a
// banded GEMM: the 16 query rows against the WB+16 key rows [g0-WB, g0+16) with
// mma.sync.m16n8k16; out-of-band entries are masked.  Every sparse tap pairs row n with row
// n-delta, i.e. it is the diagonal of a 16x16 tile: its scores come from two m16n8 MMAs per
// k-step, of which the thread with tig == g>>1 keeps the diagonal entries, and its value
// products use a diagonal A fragment.  The math is that of the DWARF reference kernels
// (kernels/dsqg_attention_v3.py:60-163 forward, :198-275 dQ, :282-352 dK/dV) without the
// scale_embed term (shapes with scale_embed use the generic kernels), with the per-head
// output gain of train/train_2048_condU.py:187 fused in.  See dsqg_mma.cuh for the
// fragment conventions.
#include "dsqg_mma.cuh"

namespace dsqg {
namespace {

constexpr int kMaxSparse = DSQG_MAX_TAPS;   // any number of sparse taps (they are processed in a loop)
constexpr int kWarps = 4;
constexpr int kRows = 16 * kWarps; // rows per CTA
constexpr int kStagePitch = kRows + 1;

struct Lane {
    int warp, lane, g, tig;
    bool owner;          // holds the diagonal entries of rows g and g+8
    int owner_lane;      // lane of this quad's owner
    __device__ Lane() {
        warp = threadIdx.x >> 5; lane = threadIdx.x & 31; g = lane >> 2; tig = lane & 3;
        owner = tig == (g >> 1);
        owner_lane = (lane & ~3) | (g >> 1);
    }
};

// ------------------------------------------------------------------------------ forward
// Online softmax: the dense window initialises the running maximum and denominator of each
// row, the sparse taps are then folded in one at a time (rescaling only when a maximum moves,
// which the distance prior makes rare).  Few live registers, so several CTAs stay resident.
template <int D> struct FwdOccupancy { static constexpr int ctas = D == 32 ? 5 : 3; };

template <int D, int WB>
__global__ void __launch_bounds__(kWarps * 32, FwdOccupancy<D>::ctas)
fwd_mma_kernel(const FwdArgs a, const Taps t) {
    constexpr int NT = (WB + 16) / 8;
    __shared__ float pb2_s[DSQG_MAX_TAPS];
    const Lane L;
    const int bh = blockIdx.y, h = bh % a.H, N = a.N;
    for (int j = threadIdx.x; j < t.J; j += kWarps * 32) pb2_s[j] = a.pos_bias[j * a.H + h] * kLog2e;
    __syncthreads();
    const int g0 = blockIdx.x * kRows + L.warp * 16;
    if (g0 >= N) return;
    const int g = L.g, tig = L.tig;
    const int row_lo = g0 + g, row_hi = row_lo + 8;
    const bool ok_lo = row_lo < N, ok_hi = row_hi < N;
    const size_t base = (size_t)bh * N * D;
    const __nv_bfloat16* qp = static_cast<const __nv_bfloat16*>(a.q) + base;
    const __nv_bfloat16* kp = static_cast<const __nv_bfloat16*>(a.k) + base;
    const __nv_bfloat16* vp = static_cast<const __nv_bfloat16*>(a.v) + base;
    const float c2 = a.scale * kLog2e;
    const int d_lo = t.d_lo, d_hi = t.d_lo + t.n_dense - 1, nd = t.n_dense, ns = t.n_sparse;
    const int kb0 = g0 - WB;

    RowFrag<D> qa, qb;
    load_row(qa, qp + (size_t)row_lo * D, tig, ok_lo);
    load_row(qb, qp + (size_t)row_hi * D, tig, ok_hi);

    // ---- dense window
    float S[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const int kr = kb0 + 8 * nt + g;
        RowFrag<D> kf;
        load_row(kf, kp + (size_t)kr * D, tig, kr >= 0 && kr < N);
        mma_rows_z(S[nt], qa, qb, kf);
    }
    float m_lo = kMinM, m_hi = kMinM;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int i = g + 8 * (r >> 1), c = 8 * nt + 2 * tig + (r & 1);
            const int delta = WB + i - c;
            const bool inband = delta >= d_lo && delta <= d_hi && kb0 + c >= 0;
            const float s = inband ? fmaf(S[nt][r], c2, pb2_s[inband ? delta - d_lo : 0]) : kNeg;
            S[nt][r] = s;
            if (r < 2) m_lo = fmaxf(m_lo, s); else m_hi = fmaxf(m_hi, s);
        }
    m_lo = quad_max(m_lo); m_hi = quad_max(m_hi);
    float l_lo = 0.f, l_hi = 0.f;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        S[nt][0] = ex2(S[nt][0] - m_lo); S[nt][1] = ex2(S[nt][1] - m_lo);
        S[nt][2] = ex2(S[nt][2] - m_hi); S[nt][3] = ex2(S[nt][3] - m_hi);
        l_lo += S[nt][0] + S[nt][1]; l_hi += S[nt][2] + S[nt][3];
    }
    float O[D / 8][4];
#pragma unroll
    for (int j = 0; j < D / 8; ++j) O[j][0] = O[j][1] = O[j][2] = O[j][3] = 0.f;
#pragma unroll
    for (int c = 0; c < NT / 2; ++c) {
        const int kr = kb0 + 16 * c + g;
        RowFrag<D> vf0, vf1, vt0, vt1;
        load_row(vf0, vp + (size_t)kr * D, tig, kr >= 0 && kr < N);
        load_row(vf1, vp + (size_t)(kr + 8) * D, tig, kr + 8 >= 0 && kr + 8 < N);
        transpose_frag(vt0, vf0); transpose_frag(vt1, vf1);
        mma_cols<D>(O, pack_bf16x2(S[2 * c][0], S[2 * c][1]), pack_bf16x2(S[2 * c][2], S[2 * c][3]),
                    pack_bf16x2(S[2 * c + 1][0], S[2 * c + 1][1]), pack_bf16x2(S[2 * c + 1][2], S[2 * c + 1][3]), vt0, vt1);
    }
    // ---- sparse taps, one at a time
#pragma unroll 1
    for (int si = 0; si < ns; ++si) {
        const int delta = t.sparse[si];
        if (g0 + 15 < delta) break;                       // taps ascend: no row of the tile reaches back that far
        const int kr0 = row_lo - delta, kr1 = row_hi - delta;
        const bool v0 = kr0 >= 0 && ok_lo, v1 = kr1 >= 0 && ok_hi;
        RowFrag<D> kf0, kf1, vf0, vf1;
        load_row(kf0, kp + (size_t)kr0 * D, tig, v0);
        load_row(kf1, kp + (size_t)kr1 * D, tig, v1);
        load_row(vf0, vp + (size_t)kr0 * D, tig, v0);
        load_row(vf1, vp + (size_t)kr1 * D, tig, v1);
        float s0[4], s1[4];
        mma_rows_z(s0, qa, qb, kf0);
        mma_rows_z(s1, qa, qb, kf1);
        const float pbv = pb2_s[nd + si];
        const float x0 = v0 ? fmaf((g & 1) ? s0[1] : s0[0], c2, pbv) : kNeg;
        const float x1 = v1 ? fmaf((g & 1) ? s1[3] : s1[2], c2, pbv) : kNeg;
        const float mn_lo = fmaxf(m_lo, __shfl_sync(0xffffffffu, x0, L.owner_lane));
        const float mn_hi = fmaxf(m_hi, __shfl_sync(0xffffffffu, x1, L.owner_lane));
        if (__any_sync(0xffffffffu, mn_lo > m_lo || mn_hi > m_hi)) {
            const float al_lo = ex2(m_lo - mn_lo), al_hi = ex2(m_hi - mn_hi);
            m_lo = mn_lo; m_hi = mn_hi;
            l_lo *= al_lo; l_hi *= al_hi;
#pragma unroll
            for (int j = 0; j < D / 8; ++j) { O[j][0] *= al_lo; O[j][1] *= al_lo; O[j][2] *= al_hi; O[j][3] *= al_hi; }
        }
        const float p0 = ex2(x0 - m_lo), p1 = ex2(x1 - m_hi);
        if (L.owner) { l_lo += p0; l_hi += p1; }
        RowFrag<D> vt0, vt1;
        transpose_frag(vt0, vf0); transpose_frag(vt1, vf1);
        uint32_t a0, a3;
        diag_frag(p0, p1, L.owner, g, a0, a3);
        mma_cols<D>(O, a0, 0u, 0u, a3, vt0, vt1);
    }
    l_lo = quad_sum(l_lo); l_hi = quad_sum(l_hi);
    const float gain = a.head_gain ? a.head_gain[h] : 1.f;
    __nv_bfloat16* op = static_cast<__nv_bfloat16*>(a.out) + base;
    store_acc_rows<D>(O, op + (size_t)row_lo * D, op + (size_t)row_hi * D, ok_lo, ok_hi,
                      l_lo > 0.f ? __fdividef(gain, l_lo) : 0.f, l_hi > 0.f ? __fdividef(gain, l_hi) : 0.f, tig);
    if (tig == 0) {
        if (ok_lo) a.lse[(size_t)bh * N + row_lo] = l_lo > 0.f ? (m_lo + __log2f(l_lo)) * kLn2 : -INFINITY;
        if (ok_hi) a.lse[(size_t)bh * N + row_hi] = l_hi > 0.f ? (m_hi + __log2f(l_hi)) * kLn2 : -INFINITY;
    }
}

// ------------------------------------------------------------------------------ backward: dQ
// Also writes delta[n] = sum_d dout*out for the dK/dV kernel and the per-CTA partial sums of
// dpos_bias (through a [J][rows] staging tile in shared memory, summed in a fixed order) and
// of dhead_gain.
// Resident CTAs per SM the backward kernels are compiled for (measured best on B200: the
// register budget that follows trades spills against warps in flight).
template <int D> struct BwdOccupancy { static constexpr int dq = D == 32 ? 6 : 4, dkdv = D == 32 ? 5 : 3; };

template <int D, int WB>
__global__ void __launch_bounds__(kWarps * 32, BwdOccupancy<D>::dq)
bwd_dq_mma_kernel(const BwdArgs a, const Taps t) {
    constexpr int NT = (WB + 16) / 8;
    extern __shared__ float stage[];                   // [J][kStagePitch] ds values, then [128] dgain terms
    __shared__ float pb2_s[DSQG_MAX_TAPS];
    const Lane L;
    const int bh = blockIdx.y, h = bh % a.H, N = a.N, J = t.J;
    float* dg_s = stage + J * kStagePitch;
    for (int j = threadIdx.x; j < J; j += kWarps * 32) pb2_s[j] = a.pos_bias[j * a.H + h] * kLog2e;
    for (int i = threadIdx.x; i < J * kStagePitch; i += kWarps * 32) stage[i] = 0.f;
    __syncthreads();
    const int g0 = blockIdx.x * kRows + L.warp * 16;
    const int g = L.g, tig = L.tig;
    float dgrow = 0.f;
    if (g0 < N) {
        const int row_lo = g0 + g, row_hi = row_lo + 8;
        const int rs_lo = L.warp * 16 + g, rs_hi = rs_lo + 8;        // row inside the CTA tile
        const bool ok_lo = row_lo < N, ok_hi = row_hi < N;
        const size_t base = (size_t)bh * N * D;
        const __nv_bfloat16* qp = static_cast<const __nv_bfloat16*>(a.q) + base;
        const __nv_bfloat16* kp = static_cast<const __nv_bfloat16*>(a.k) + base;
        const __nv_bfloat16* vp = static_cast<const __nv_bfloat16*>(a.v) + base;
        const __nv_bfloat16* op = static_cast<const __nv_bfloat16*>(a.out) + base;
        const __nv_bfloat16* dop = static_cast<const __nv_bfloat16*>(a.dout) + base;
        const float c2 = a.scale * kLog2e;
        const float gain = a.head_gain ? a.head_gain[h] : 1.f;
        const int d_lo = t.d_lo, d_hi = t.d_lo + t.n_dense - 1, nd = t.n_dense, ns = t.n_sparse;
        const int kb0 = g0 - WB;

        RowFrag<D> qa, qb, da, db;
        load_row(qa, qp + (size_t)row_lo * D, tig, ok_lo);
        load_row(qb, qp + (size_t)row_hi * D, tig, ok_hi);
        load_row(da, dop + (size_t)row_lo * D, tig, ok_lo);
        load_row(db, dop + (size_t)row_hi * D, tig, ok_hi);
        float delta_lo, delta_hi;
        {
            RowFrag<D> oa, ob;
            load_row(oa, op + (size_t)row_lo * D, tig, ok_lo);
            load_row(ob, op + (size_t)row_hi * D, tig, ok_hi);
            delta_lo = quad_sum(frag_dot(da, oa));
            delta_hi = quad_sum(frag_dot(db, ob));
        }
        float l2_lo = 0.f, l2_hi = 0.f;
        if (ok_lo) { const float x = a.lse[(size_t)bh * N + row_lo]; l2_lo = x == -INFINITY ? 0.f : x * kLog2e; }
        if (ok_hi) { const float x = a.lse[(size_t)bh * N + row_hi]; l2_hi = x == -INFINITY ? 0.f : x * kLog2e; }
        if (tig == 0) {
            if (ok_lo) a.delta[(size_t)bh * N + row_lo] = delta_lo;
            if (ok_hi) a.delta[(size_t)bh * N + row_hi] = delta_hi;
        }
        float dQ[D / 8][4];
#pragma unroll
        for (int j = 0; j < D / 8; ++j) dQ[j][0] = dQ[j][1] = dQ[j][2] = dQ[j][3] = 0.f;

#pragma unroll
        for (int c = 0; c < NT / 2; ++c) {
            RowFrag<D> kf[2];
            float ds[2][4];
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                const int nt = 2 * c + hf;
                const int kr = kb0 + 8 * nt + g;
                const bool kv = kr >= 0 && kr < N;
                RowFrag<D> vf;
                load_row(kf[hf], kp + (size_t)kr * D, tig, kv);
                load_row(vf, vp + (size_t)kr * D, tig, kv);
                float s[4], dp[4];
                mma_rows_z(s, qa, qb, kf[hf]);
                mma_rows_z(dp, da, db, vf);
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const int i = g + 8 * (r >> 1), cc = 8 * nt + 2 * tig + (r & 1);
                    const int delta = WB + i - cc;
                    const bool geom = delta >= d_lo && delta <= d_hi;
                    const bool inband = geom && kb0 + cc >= 0 && (r < 2 ? ok_lo : ok_hi);
                    const float p = inband ? ex2(fmaf(s[r], c2, pb2_s[inband ? delta - d_lo : 0]) - (r < 2 ? l2_lo : l2_hi)) : 0.f;
                    dgrow = fmaf(p, dp[r], dgrow);
                    const float x = p * (gain * dp[r] - (r < 2 ? delta_lo : delta_hi));
                    ds[hf][r] = x;
                    if (geom) stage[(delta - d_lo) * kStagePitch + (r < 2 ? rs_lo : rs_hi)] = x;
                }
            }
            RowFrag<D> kt0, kt1;
            transpose_frag(kt0, kf[0]); transpose_frag(kt1, kf[1]);
            mma_cols<D>(dQ, pack_bf16x2(ds[0][0], ds[0][1]), pack_bf16x2(ds[0][2], ds[0][3]),
                        pack_bf16x2(ds[1][0], ds[1][1]), pack_bf16x2(ds[1][2], ds[1][3]), kt0, kt1);
        }
#pragma unroll 1
        for (int si = 0; si < ns; ++si) {
            const int delta = t.sparse[si];
            if (g0 + 15 < delta) break;
            const int kr0 = row_lo - delta, kr1 = row_hi - delta;
            const bool v0 = kr0 >= 0 && ok_lo, v1 = kr1 >= 0 && ok_hi;
            RowFrag<D> kf0, kf1, vf0, vf1;
            load_row(kf0, kp + (size_t)kr0 * D, tig, v0);
            load_row(kf1, kp + (size_t)kr1 * D, tig, v1);
            load_row(vf0, vp + (size_t)kr0 * D, tig, v0);
            load_row(vf1, vp + (size_t)kr1 * D, tig, v1);
            float s0[4], s1[4], e0[4], e1[4];
            mma_rows_z(s0, qa, qb, kf0); mma_rows_z(s1, qa, qb, kf1);
            mma_rows_z(e0, da, db, vf0); mma_rows_z(e1, da, db, vf1);
            const float pbv = pb2_s[nd + si];
            const float sd0 = (g & 1) ? s0[1] : s0[0], sd1 = (g & 1) ? s1[3] : s1[2];
            const float dp0 = (g & 1) ? e0[1] : e0[0], dp1 = (g & 1) ? e1[3] : e1[2];
            const float p0 = v0 ? ex2(fmaf(sd0, c2, pbv) - l2_lo) : 0.f;
            const float p1 = v1 ? ex2(fmaf(sd1, c2, pbv) - l2_hi) : 0.f;
            const float x0 = p0 * (gain * dp0 - delta_lo), x1 = p1 * (gain * dp1 - delta_hi);
            if (L.owner) {
                dgrow = fmaf(p0, dp0, dgrow); dgrow = fmaf(p1, dp1, dgrow);
                stage[(nd + si) * kStagePitch + rs_lo] = x0;
                stage[(nd + si) * kStagePitch + rs_hi] = x1;
            }
            uint32_t a0, a3;
            diag_frag(x0, x1, L.owner, g, a0, a3);
            RowFrag<D> kt0, kt1;
            transpose_frag(kt0, kf0); transpose_frag(kt1, kf1);
            mma_cols<D>(dQ, a0, 0u, 0u, a3, kt0, kt1);
        }
        __nv_bfloat16* dqp = static_cast<__nv_bfloat16*>(a.dq) + base;
        store_acc_rows<D>(dQ, dqp + (size_t)row_lo * D, dqp + (size_t)row_hi * D, ok_lo, ok_hi, a.scale, a.scale, tig);
    }
    dg_s[threadIdx.x] = dgrow;
    __syncthreads();
    const int tile = bh * a.tiles_per_bh + blockIdx.x;
    if (threadIdx.x < J) {
        float s = 0.f;
        const float* row = stage + threadIdx.x * kStagePitch;
        for (int r = 0; r < kRows; ++r) s += row[r];
        a.dpb_part[(size_t)tile * J + threadIdx.x] = s;
    } else if (threadIdx.x == kWarps * 32 - 1) {
        float s = 0.f;
        for (int r = 0; r < kWarps * 32; ++r) s += dg_s[r];
        a.dg_part[tile] = s;
    }
}

// ------------------------------------------------------------------------------ backward: dK, dV
// The warp owns 16 key rows; the roles of rows and columns are swapped: S^T = K.Q^T over the
// query rows [m0, m0+16+WB) for the dense window and the diagonal of the tile at m0+delta for
// every sparse tap.  Key rows are owned by exactly one warp: no atomics.
template <int D, int WB>
__global__ void __launch_bounds__(kWarps * 32, BwdOccupancy<D>::dkdv)
bwd_dkdv_mma_kernel(const BwdArgs a, const Taps t) {
    constexpr int NT = (WB + 16) / 8;
    __shared__ float pb2_s[DSQG_MAX_TAPS];
    const Lane L;
    const int bh = blockIdx.y, h = bh % a.H, N = a.N;
    for (int j = threadIdx.x; j < t.J; j += kWarps * 32) pb2_s[j] = a.pos_bias[j * a.H + h] * kLog2e;
    __syncthreads();
    const int m0 = blockIdx.x * kRows + L.warp * 16;
    if (m0 >= N) return;
    const int g = L.g, tig = L.tig;
    const int row_lo = m0 + g, row_hi = row_lo + 8;
    const bool ok_lo = row_lo < N, ok_hi = row_hi < N;
    const size_t base = (size_t)bh * N * D;
    const __nv_bfloat16* qp = static_cast<const __nv_bfloat16*>(a.q) + base;
    const __nv_bfloat16* kp = static_cast<const __nv_bfloat16*>(a.k) + base;
    const __nv_bfloat16* vp = static_cast<const __nv_bfloat16*>(a.v) + base;
    const __nv_bfloat16* dop = static_cast<const __nv_bfloat16*>(a.dout) + base;
    const float* lse = a.lse + (size_t)bh * N;
    const float* dl = a.delta + (size_t)bh * N;
    const float c2 = a.scale * kLog2e;
    const float gain = a.head_gain ? a.head_gain[h] : 1.f;
    const int d_lo = t.d_lo, d_hi = t.d_lo + t.n_dense - 1, nd = t.n_dense, ns = t.n_sparse;

    RowFrag<D> ka, kb, va, vb;
    load_row(ka, kp + (size_t)row_lo * D, tig, ok_lo);
    load_row(kb, kp + (size_t)row_hi * D, tig, ok_hi);
    load_row(va, vp + (size_t)row_lo * D, tig, ok_lo);
    load_row(vb, vp + (size_t)row_hi * D, tig, ok_hi);
    float dK[D / 8][4], dV[D / 8][4];
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
        dK[j][0] = dK[j][1] = dK[j][2] = dK[j][3] = 0.f;
        dV[j][0] = dV[j][1] = dV[j][2] = dV[j][3] = 0.f;
    }

#pragma unroll
    for (int c = 0; c < NT / 2; ++c) {
        if (m0 + 16 * c >= N) break;                    // warp-uniform: no query rows left
        RowFrag<D> qf[2], df[2];
        float ds[2][4], pv[2][4];
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
            const int nt = 2 * c + hf;
            const int qr = m0 + 8 * nt + g;
            load_row(qf[hf], qp + (size_t)qr * D, tig, qr < N);
            load_row(df[hf], dop + (size_t)qr * D, tig, qr < N);
            float s[4], dp[4];
            mma_rows_z(s, ka, kb, qf[hf]);
            mma_rows_z(dp, va, vb, df[hf]);
            // this thread's two query columns of the n-tile
            const int qc = m0 + 8 * nt + 2 * tig;
            float l2c[2], dlc[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const bool qv = qc + e < N;
                const float x = qv ? lse[qc + e] : 0.f;
                l2c[e] = x == -INFINITY ? 0.f : x * kLog2e;
                dlc[e] = qv ? dl[qc + e] : 0.f;
            }
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int i = g + 8 * (r >> 1), cc = 8 * nt + 2 * tig + (r & 1);
                const int delta = cc - i;
                const bool inband = delta >= d_lo && delta <= d_hi && m0 + cc < N;
                const float p = inband ? ex2(fmaf(s[r], c2, pb2_s[inband ? delta - d_lo : 0]) - l2c[r & 1]) : 0.f;
                ds[hf][r] = p * (gain * dp[r] - dlc[r & 1]);
                pv[hf][r] = p * gain;
            }
        }
        RowFrag<D> t0, t1;
        transpose_frag(t0, df[0]); transpose_frag(t1, df[1]);
        mma_cols<D>(dV, pack_bf16x2(pv[0][0], pv[0][1]), pack_bf16x2(pv[0][2], pv[0][3]),
                    pack_bf16x2(pv[1][0], pv[1][1]), pack_bf16x2(pv[1][2], pv[1][3]), t0, t1);
        transpose_frag(t0, qf[0]); transpose_frag(t1, qf[1]);
        mma_cols<D>(dK, pack_bf16x2(ds[0][0], ds[0][1]), pack_bf16x2(ds[0][2], ds[0][3]),
                    pack_bf16x2(ds[1][0], ds[1][1]), pack_bf16x2(ds[1][2], ds[1][3]), t0, t1);
    }
#pragma unroll 1
    for (int si = 0; si < ns; ++si) {
        const int delta = t.sparse[si];
        if (m0 + delta >= N) break;                     // taps ascend: no query row reads these keys any more
        const int qr0 = row_lo + delta, qr1 = row_hi + delta;
        const bool v0 = qr0 < N, v1 = qr1 < N;
        RowFrag<D> qf0, qf1, df0, df1;
        load_row(qf0, qp + (size_t)qr0 * D, tig, v0);
        load_row(qf1, qp + (size_t)qr1 * D, tig, v1);
        load_row(df0, dop + (size_t)qr0 * D, tig, v0);
        load_row(df1, dop + (size_t)qr1 * D, tig, v1);
        float s0[4], s1[4], e0[4], e1[4];
        mma_rows_z(s0, ka, kb, qf0); mma_rows_z(s1, ka, kb, qf1);
        mma_rows_z(e0, va, vb, df0); mma_rows_z(e1, va, vb, df1);
        const float pbv = pb2_s[nd + si];
        const float sd0 = (g & 1) ? s0[1] : s0[0], sd1 = (g & 1) ? s1[3] : s1[2];
        const float dp0 = (g & 1) ? e0[1] : e0[0], dp1 = (g & 1) ? e1[3] : e1[2];
        float l0 = 0.f, l1 = 0.f, dl0 = 0.f, dl1 = 0.f;
        if (v0) { const float x = lse[qr0]; l0 = x == -INFINITY ? 0.f : x * kLog2e; dl0 = dl[qr0]; }
        if (v1) { const float x = lse[qr1]; l1 = x == -INFINITY ? 0.f : x * kLog2e; dl1 = dl[qr1]; }
        const float p0 = v0 ? ex2(fmaf(sd0, c2, pbv) - l0) : 0.f;
        const float p1 = v1 ? ex2(fmaf(sd1, c2, pbv) - l1) : 0.f;
        uint32_t a0, a3;
        RowFrag<D> t0, t1;
        diag_frag(p0 * gain, p1 * gain, L.owner, g, a0, a3);
        transpose_frag(t0, df0); transpose_frag(t1, df1);
        mma_cols<D>(dV, a0, 0u, 0u, a3, t0, t1);
        diag_frag(p0 * (gain * dp0 - dl0), p1 * (gain * dp1 - dl1), L.owner, g, a0, a3);
        transpose_frag(t0, qf0); transpose_frag(t1, qf1);
        mma_cols<D>(dK, a0, 0u, 0u, a3, t0, t1);
    }
    __nv_bfloat16* dkp = static_cast<__nv_bfloat16*>(a.dk) + base;
    __nv_bfloat16* dvp = static_cast<__nv_bfloat16*>(a.dv) + base;
    store_acc_rows<D>(dK, dkp + (size_t)row_lo * D, dkp + (size_t)row_hi * D, ok_lo, ok_hi, a.scale, a.scale, tig);
    store_acc_rows<D>(dV, dvp + (size_t)row_lo * D, dvp + (size_t)row_hi * D, ok_lo, ok_hi, 1.f, 1.f, tig);
}

template <int D, int WB>
cudaError_t fwd_launch_mma(const FwdArgs& a, const Taps& t, cudaStream_t s) {
    dim3 grid((a.N + kRows - 1) / kRows, a.B * a.H);
    fwd_mma_kernel<D, WB><<<grid, kWarps * 32, 0, s>>>(a, t);
    return cudaGetLastError();
}

template <int D, int WB>
cudaError_t bwd_launch_mma(BwdArgs a, const Taps& t, cudaStream_t s, int stages) {
    carve_bwd_scratch(a, kRows, t.J, false);
    dim3 grid((a.N + kRows - 1) / kRows, a.B * a.H);
    cudaError_t e = cudaSuccess;
    if (stages & DSQG_BWD_STAGE_DQ) {
        const size_t smem = sizeof(float) * ((size_t)t.J * kStagePitch + kWarps * 32);
        if (smem > 48 * 1024) {
            e = cudaFuncSetAttribute(bwd_dq_mma_kernel<D, WB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return e;
        }
        bwd_dq_mma_kernel<D, WB><<<grid, kWarps * 32, smem, s>>>(a, t);
        if ((e = cudaGetLastError()) != cudaSuccess) return e;
    }
    if (stages & DSQG_BWD_STAGE_DKDV) {
        bwd_dkdv_mma_kernel<D, WB><<<grid, kWarps * 32, 0, s>>>(a, t);
        if ((e = cudaGetLastError()) != cudaSuccess) return e;
    }
    if (stages & DSQG_BWD_STAGE_REDUCE) e = launch_reduce_params(a, t.J, s);
    return e;
}

int band_width(const Taps& t) {
    const int d_hi = t.d_lo + t.n_dense - 1;
    return d_hi <= 32 ? 32 : (d_hi <= 48 ? 48 : (d_hi <= 64 ? 64 : 0));
}

}  // namespace

bool mma_path_supported(int dtype, int D, const Taps& t, bool has_scale_embed) {
    return dtype == DSQG_DTYPE_BF16 && (D == 32 || D == 64) && !has_scale_embed &&
           t.n_sparse <= kMaxSparse && band_width(t) != 0;
}

#define DSQG_MMA_DISPATCH(FN, ...)                                             \
    do {                                                                       \
        const int wb_ = band_width(t);                                         \
        if (a.D == 32) {                                                       \
            if (wb_ == 32) return FN<32, 32>(__VA_ARGS__);                     \
            if (wb_ == 48) return FN<32, 48>(__VA_ARGS__);                     \
            return FN<32, 64>(__VA_ARGS__);                                    \
        }                                                                      \
        if (wb_ == 32) return FN<64, 32>(__VA_ARGS__);                         \
        if (wb_ == 48) return FN<64, 48>(__VA_ARGS__);                         \
        return FN<64, 64>(__VA_ARGS__);                                        \
    } while (0)

cudaError_t launch_fwd_mma(const FwdArgs& a, const Taps& t, cudaStream_t s) {
    DSQG_MMA_DISPATCH(fwd_launch_mma, a, t, s);
}

cudaError_t launch_bwd_mma(const BwdArgs& a, const Taps& t, cudaStream_t s, int stages) {
    DSQG_MMA_DISPATCH(bwd_launch_mma, a, t, s, stages);
}

}  // namespace dsqg
