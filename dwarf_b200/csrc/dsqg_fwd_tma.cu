// Persistent, TMA-fed DSQG forward kernel (bf16, D in {32, 64}, sparse taps multiples of 16).
//
// Work decomposition.  A "step" is 128 consecutive rows of one (batch, head) sequence; the
// flattened list of steps is cut into one contiguous range per CTA, so a CTA walks down a
// sequence and keeps the K/V rows it has already fetched.
//
// Shared memory.
//   * K ring and V ring: NR rows each (NR a power of two), filled 128 rows at a time by TMA.
//     Row R of the sequence lives in ring row R & (NR-1).  The ring holds rows
//     [r0 - (NR-256), r0 + 128) of the current step plus the 128 rows prefetched for the next
//     one, so the dense window and every sparse tap with delta <= NR-256 ("window taps") are
//     read from the ring: each K/V row is fetched from L2/HBM once per CTA, not once per tap.
//   * "far" taps (delta > NR-256) stream through a small ring of stages, each holding the
//     128-row K tile and V tile of one tap.
//
// Softmax.  The dense window initialises the running maximum / denominator of a row; sparse
// taps are then folded in group by group with the usual online-softmax rescaling.
//   * Q tiles are double buffered.
//
// Warp roles.  Warps 0..7 compute (16 rows each, tensor-core math as in dsqg_mma.cu); warp 8
// is the producer: one lane issues every TMA load and runs ahead of the consumers as far as
// the "empty" mbarriers allow.  All waits are bounded (dsqg_tma.cuh).
#include "dsqg_tma.cuh"

namespace dsqg {

namespace {

constexpr int kStepRows = 128;
constexpr int kConsumerWarps = 8;
constexpr int kThreadsTma = (kConsumerWarps + 1) * 32;
constexpr int kMaxSparseTma = 16;
constexpr int kMaxRingBlocks = 16;      // NR <= 2048 rows
constexpr int kMaxFarStages = 8;

struct FwdTmaPlan {
    int NR;              // ring rows (power of two, multiple of 128)
    int n_win;           // sparse taps 0 .. n_win-1 are read from the ring
    int n_far_stages;    // stages of the far-tap ring
    int steps_per_seq;   // ceil(N / 128)
    int total_steps;     // B*H*steps_per_seq
    int steps_per_cta;   // ceil(total_steps / gridDim.x)
};

// Shared-memory carve-up (byte offsets from the 1024-aligned base).
template <int D>
struct SmemLayout {
    static constexpr int kPitch = D * 2;
    static constexpr int kTile = kStepRows * kPitch;          // one 128-row tile
    int k_ring, v_ring, far, q, bars, pb, misc, total;
    __host__ __device__ SmemLayout(int NR, int n_far_stages) {
        k_ring = 0;
        v_ring = k_ring + NR * kPitch;
        far = v_ring + NR * kPitch;
        q = far + n_far_stages * 2 * kTile;
        bars = q + 2 * kTile;
        pb = bars + 8 * (2 * kMaxRingBlocks + 2 * kMaxFarStages + 4);
        misc = pb + 4 * DSQG_MAX_TAPS;
        total = misc + 64;
    }
};

struct Bars {           // addresses (shared-space u32) of the mbarriers
    uint32_t base;
    __device__ uint32_t win_full(int s) const { return base + 8 * s; }
    __device__ uint32_t win_empty(int s) const { return base + 8 * (kMaxRingBlocks + s); }
    __device__ uint32_t far_full(int s) const { return base + 8 * (2 * kMaxRingBlocks + s); }
    __device__ uint32_t far_empty(int s) const { return base + 8 * (2 * kMaxRingBlocks + kMaxFarStages + s); }
    __device__ uint32_t q_full(int s) const { return base + 8 * (2 * kMaxRingBlocks + 2 * kMaxFarStages + s); }
    __device__ uint32_t q_empty(int s) const { return base + 8 * (2 * kMaxRingBlocks + 2 * kMaxFarStages + 2 + s); }
};

// ------------------------------------------------------------------------------ producer
template <int D>
__device__ __forceinline__ void producer_loop(const FwdTmaPlan& plan, const Taps& t, const CUtensorMap* tm_q,
                              const CUtensorMap* tm_k, const CUtensorMap* tm_v, uint32_t smem_base,
                              const SmemLayout<D>& lay, const Bars& bars, volatile int* abort_flag,
                              int step_begin, int step_end) {
    constexpr int kTile = SmemLayout<D>::kTile;
    const int nrb = plan.NR / kStepRows;                  // ring blocks
    const int held = nrb - 1;                             // blocks a step needs (incl. its own)
    uint32_t win_empty_phase = 0xffffffffu;               // fresh barriers: the "previous" phase is complete
    uint32_t far_count = 0, q_count = 0;
    for (int s = step_begin; s < step_end; ++s) {
        const int bh = s / plan.steps_per_seq, sb = s - bh * plan.steps_per_seq;
        const int r0 = sb * kStepRows;
        const bool first = (s == step_begin) || sb == 0;
        // Q tile
        {
            const int st = q_count & 1;
            mbar_wait(bars.q_empty(st), ((q_count >> 1) & 1) ^ 1, abort_flag, 0x101);
            mbar_arrive_expect_tx(bars.q_full(st), kTile);
            tma_load_3d(smem_base + lay.q + st * kTile, tm_q, bars.q_full(st), 0, r0, bh);
            ++q_count;
        }
        // window blocks: all `held` blocks at the start of a sequence / of the CTA's range,
        // otherwise only the newest one
        for (int b = first ? sb - (held - 1) : sb; b <= sb; ++b) {
            const int slot = b & (nrb - 1);
            mbar_wait(bars.win_empty(slot), (win_empty_phase >> slot) & 1, abort_flag, 0x102);
            win_empty_phase ^= 1u << slot;
            mbar_arrive_expect_tx(bars.win_full(slot), 2 * kTile);
            tma_load_3d(smem_base + lay.k_ring + slot * kTile, tm_k, bars.win_full(slot), 0, b * kStepRows, bh);
            tma_load_3d(smem_base + lay.v_ring + slot * kTile, tm_v, bars.win_full(slot), 0, b * kStepRows, bh);
        }
        // far taps: one stage holds the K tile and the V tile of one tap
        for (int si = plan.n_win; si < t.n_sparse; ++si) {
            const int delta = t.sparse[si];
            if (r0 + kStepRows - 16 < delta) break;               // no row of this step reaches back that far
            const int st = far_count % plan.n_far_stages;
            mbar_wait(bars.far_empty(st), ((far_count / plan.n_far_stages) & 1) ^ 1, abort_flag, 0x103);
            mbar_arrive_expect_tx(bars.far_full(st), 2 * kTile);
            tma_load_3d(smem_base + lay.far + st * 2 * kTile, tm_k, bars.far_full(st), 0, r0 - delta, bh);
            tma_load_3d(smem_base + lay.far + st * 2 * kTile + kTile, tm_v, bars.far_full(st), 0, r0 - delta, bh);
            ++far_count;
        }
        if (*abort_flag) break;
    }
}


// Store rows g, g+8 of an accumulator tile; thread tig owns chunk_elem<D>(tig, c) + [0,8).
template <int D>
__device__ __forceinline__ void store_acc_rows_tma(const float (&acc)[D / 8][4], __nv_bfloat16* row_lo,
                                                   __nv_bfloat16* row_hi, bool ok_lo, bool ok_hi,
                                                   float s_lo, float s_hi, int tig) {
#pragma unroll
    for (int c = 0; c < D / 32; ++c) {
        uint4 lo, hi;
        lo.x = pack_bf16x2(acc[4 * c + 0][0] * s_lo, acc[4 * c + 0][1] * s_lo);
        lo.y = pack_bf16x2(acc[4 * c + 1][0] * s_lo, acc[4 * c + 1][1] * s_lo);
        lo.z = pack_bf16x2(acc[4 * c + 2][0] * s_lo, acc[4 * c + 2][1] * s_lo);
        lo.w = pack_bf16x2(acc[4 * c + 3][0] * s_lo, acc[4 * c + 3][1] * s_lo);
        hi.x = pack_bf16x2(acc[4 * c + 0][2] * s_hi, acc[4 * c + 0][3] * s_hi);
        hi.y = pack_bf16x2(acc[4 * c + 1][2] * s_hi, acc[4 * c + 1][3] * s_hi);
        hi.z = pack_bf16x2(acc[4 * c + 2][2] * s_hi, acc[4 * c + 2][3] * s_hi);
        hi.w = pack_bf16x2(acc[4 * c + 3][2] * s_hi, acc[4 * c + 3][3] * s_hi);
        if (ok_lo) *reinterpret_cast<uint4*>(row_lo + chunk_elem<D>(tig, c)) = lo;
        if (ok_hi) *reinterpret_cast<uint4*>(row_hi + chunk_elem<D>(tig, c)) = hi;
    }
}

// ------------------------------------------------------------------------------ consumers
// Running softmax state of the two rows (g, g+8) a thread works on, plus the output tile.
template <int D>
struct RowState {
    float m_lo, m_hi;          // running maxima (log2 units), never below kMinM
    float l_lo, l_hi;          // this thread's share of the denominators
    float O[D / 8][4];         // value accumulator, contiguous-d layout
};

// G sparse taps at once, branch-free: scores of the tile diagonals (two MMAs per k-step and
// tap), one online-softmax update for the group, then the value products with diagonal A
// fragments.  srcK[i] / srcV[i] are shared-memory addresses of the 8-row group that holds the
// key row of query row g (rows g+8: +8 rows).  ok[i] = false masks tap i (its addresses must
// still be readable).
template <int D, int G>
__device__ __forceinline__ void sparse_group(RowState<D>& st, const RowFrag<D>& qa, const RowFrag<D>& qb,
                                             const uint32_t (&srcK)[G], const uint32_t (&srcV)[G],
                                             const bool (&ok)[G], const float (&pb2)[G], float c2,
                                             const LaneOff<D>& lo, bool owner, int owner_lane, int g) {
    constexpr int kPitch = D * 2;
    float s_lo[G], s_hi[G];
    float gm_lo = kNeg, gm_hi = kNeg;
#pragma unroll
    for (int i = 0; i < G; ++i) {
        RowFrag<D> kf0, kf1;
        lds_frag<D>(kf0, srcK[i], lo);
        lds_frag<D>(kf1, srcK[i] + 8 * kPitch, lo);
        float s0[4], s1[4];
        mma_rows_z(s0, qa, qb, kf0);
        mma_rows_z(s1, qa, qb, kf1);
        s_lo[i] = ok[i] ? fmaf((g & 1) ? s0[1] : s0[0], c2, pb2[i]) : kNeg;
        s_hi[i] = ok[i] ? fmaf((g & 1) ? s1[3] : s1[2], c2, pb2[i]) : kNeg;
        gm_lo = fmaxf(gm_lo, s_lo[i]); gm_hi = fmaxf(gm_hi, s_hi[i]);
    }
    const float mn_lo = fmaxf(st.m_lo, __shfl_sync(0xffffffffu, gm_lo, owner_lane));
    const float mn_hi = fmaxf(st.m_hi, __shfl_sync(0xffffffffu, gm_hi, owner_lane));
    const float al_lo = ex2(st.m_lo - mn_lo), al_hi = ex2(st.m_hi - mn_hi);
    st.m_lo = mn_lo; st.m_hi = mn_hi;
    st.l_lo *= al_lo; st.l_hi *= al_hi;
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
        st.O[j][0] *= al_lo; st.O[j][1] *= al_lo; st.O[j][2] *= al_hi; st.O[j][3] *= al_hi;
    }
#pragma unroll
    for (int i = 0; i < G; ++i) {
        const float p0 = ex2(s_lo[i] - mn_lo), p1 = ex2(s_hi[i] - mn_hi);
        if (owner) { st.l_lo += p0; st.l_hi += p1; }
        RowFrag<D> vf0, vf1, vt0, vt1;
        lds_frag<D>(vf0, srcV[i], lo);
        lds_frag<D>(vf1, srcV[i] + 8 * kPitch, lo);
        transpose_frag(vt0, vf0); transpose_frag(vt1, vf1);
        uint32_t a0, a3;
        diag_frag(p0, p1, owner, g, a0, a3);
        mma_cols<D>(st.O, a0, 0u, 0u, a3, vt0, vt1);
    }
}

// Dense window of one 16-row tile: banded scores against ring rows [g0-WB, g0+16), softmax
// statistics initialised from it, P.V accumulated.
template <int D, int WB>
__device__ __forceinline__ void dense_window(RowState<D>& st, const RowFrag<D>& qa, const RowFrag<D>& qb,
                                             const float (&biasd)[(WB + 16) / 8][4], uint32_t k_ring, uint32_t v_ring,
                                             int g0, int ring_mask, float c2, const LaneOff<D>& lo, int tig) {
    constexpr int NT = (WB + 16) / 8;
    constexpr int kPitch = D * 2;
    float S[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        RowFrag<D> kf;
        lds_frag<D>(kf, k_ring + ((g0 - WB + 8 * nt) & ring_mask) * kPitch, lo);
        mma_rows_z(S[nt], qa, qb, kf);
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int r = 0; r < 4; ++r) S[nt][r] = fmaf(S[nt][r], c2, biasd[nt][r]);
    if (g0 < WB) {               // sequence start: keys before row 0 do not exist
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int r = 0; r < 4; ++r)
                if (g0 - WB + 8 * nt + 2 * tig + (r & 1) < 0) S[nt][r] = kNeg;
    }
    float m_lo = kMinM, m_hi = kMinM;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        m_lo = fmaxf(m_lo, fmaxf(S[nt][0], S[nt][1]));
        m_hi = fmaxf(m_hi, fmaxf(S[nt][2], S[nt][3]));
    }
    m_lo = quad_max(m_lo); m_hi = quad_max(m_hi);
    float l_lo = 0.f, l_hi = 0.f;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        S[nt][0] = ex2(S[nt][0] - m_lo); S[nt][1] = ex2(S[nt][1] - m_lo);
        S[nt][2] = ex2(S[nt][2] - m_hi); S[nt][3] = ex2(S[nt][3] - m_hi);
        l_lo += S[nt][0] + S[nt][1]; l_hi += S[nt][2] + S[nt][3];
    }
    st.m_lo = m_lo; st.m_hi = m_hi; st.l_lo = l_lo; st.l_hi = l_hi;
#pragma unroll
    for (int j = 0; j < D / 8; ++j) st.O[j][0] = st.O[j][1] = st.O[j][2] = st.O[j][3] = 0.f;
#pragma unroll
    for (int c = 0; c < NT / 2; ++c) {
        RowFrag<D> vf0, vf1, vt0, vt1;
        lds_frag<D>(vf0, v_ring + ((g0 - WB + 16 * c) & ring_mask) * kPitch, lo);
        lds_frag<D>(vf1, v_ring + ((g0 - WB + 16 * c + 8) & ring_mask) * kPitch, lo);
        transpose_frag(vt0, vf0); transpose_frag(vt1, vf1);
        mma_cols<D>(st.O, pack_bf16x2(S[2 * c][0], S[2 * c][1]), pack_bf16x2(S[2 * c][2], S[2 * c][3]),
                    pack_bf16x2(S[2 * c + 1][0], S[2 * c + 1][1]), pack_bf16x2(S[2 * c + 1][2], S[2 * c + 1][3]), vt0, vt1);
    }
}

constexpr int kGroup = 2;      // window taps processed per branch-free group

template <int D, int WB>
__device__ __forceinline__ void consumer_loop(const FwdArgs& a, const FwdTmaPlan& plan, const Taps& t, uint32_t smem_base,
                                              const SmemLayout<D>& lay, const Bars& bars, volatile int* abort_flag,
                                              int step_begin, int step_end) {
    constexpr int NT = (WB + 16) / 8;
    constexpr int kPitch = SmemLayout<D>::kPitch;
    constexpr int kTile = SmemLayout<D>::kTile;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tig = lane & 3;
    const bool owner = tig == (g >> 1);
    const int owner_lane = (lane & ~3) | (g >> 1);
    const LaneOff<D> lo = lane_offsets<D>(g, tig);
    const int N = a.N, H = a.H;
    const int nrb = plan.NR / kStepRows, held = nrb - 1, ring_mask = plan.NR - 1;
    const int d_lo = t.d_lo, d_hi = t.d_lo + t.n_dense - 1, nd = t.n_dense, ns = t.n_sparse, n_win = plan.n_win;
    const float c2 = a.scale * kLog2e;
    const uint32_t k_ring = smem_base + lay.k_ring, v_ring = smem_base + lay.v_ring;

    uint32_t win_full_phase = 0, far_count = 0, q_count = 0;
    float biasd[NT][4];
    int bias_h = -1;

#pragma unroll 1
    for (int s = step_begin; s < step_end; ++s) {
        const int bh = s / plan.steps_per_seq, sb = s - bh * plan.steps_per_seq;
        const int r0 = sb * kStepRows, h = bh % H;
        const bool first = (s == step_begin) || sb == 0;
        const bool last_of_seq = (s + 1 == step_end) || sb + 1 == plan.steps_per_seq;
        const int g0 = r0 + 16 * warp;
        const bool active = g0 < N;
        const int row_lo = g0 + g, row_hi = row_lo + 8;

        if (h != bias_h) {       // dense-window bias fragment of this head (Toeplitz: same for every tile)
            bias_h = h;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const int delta = WB + g + 8 * (r >> 1) - (8 * nt + 2 * tig + (r & 1));
                    biasd[nt][r] = (delta >= d_lo && delta <= d_hi) ? __ldg(a.pos_bias + (delta - d_lo) * H + h) * kLog2e : kNeg;
                }
        }
        // ---- Q fragments
        RowFrag<D> qa, qb;
        {
            const int st = q_count & 1;
            mbar_wait(bars.q_full(st), (q_count >> 1) & 1, abort_flag, 0x201);
            const uint32_t qt = smem_base + lay.q + st * kTile + warp * 16 * kPitch;
            lds_frag<D>(qa, qt, lo);
            lds_frag<D>(qb, qt + 8 * kPitch, lo);
            __syncwarp();
            if (lane == 0) mbar_arrive(bars.q_empty(st));
            ++q_count;
        }
        // ---- the ring blocks this step reads
#pragma unroll 1
        for (int b = first ? sb - (held - 1) : sb; b <= sb; ++b) {
            const int slot = b & (nrb - 1);
            mbar_wait(bars.win_full(slot), (win_full_phase >> slot) & 1, abort_flag, 0x202);
            win_full_phase ^= 1u << slot;
        }
        // number of sparse taps that reach back inside the sequence for this tile (taps ascend and
        // are multiples of 16, as is g0: a tap is valid for all 16 rows or for none)
        int nv = 0;
        while (nv < ns && t.sparse[nv] <= g0) ++nv;

        RowState<D> st;
        if (active) {
            dense_window<D, WB>(st, qa, qb, biasd, k_ring, v_ring, g0, ring_mask, c2, lo, tig);
            const int nvw = nv < n_win ? nv : n_win;
#pragma unroll 1
            for (int t0 = 0; t0 < nvw; t0 += kGroup) {
                uint32_t srcK[kGroup], srcV[kGroup];
                bool ok[kGroup];
                float pb2[kGroup];
#pragma unroll
                for (int i = 0; i < kGroup; ++i) {
                    ok[i] = t0 + i < nvw;
                    const int ti = ok[i] ? t0 + i : nvw - 1;
                    const uint32_t off = ((g0 - t.sparse[ti]) & ring_mask) * kPitch;
                    srcK[i] = k_ring + off; srcV[i] = v_ring + off;
                    pb2[i] = __ldg(a.pos_bias + (nd + ti) * H + h) * kLog2e;
                }
                sparse_group<D, kGroup>(st, qa, qb, srcK, srcV, ok, pb2, c2, lo, owner, owner_lane, g);
            }
        }
        // ---- far taps: streamed stages (every warp takes part in the barrier protocol)
#pragma unroll 1
        for (int si = n_win; si < ns; ++si) {
            const int delta = t.sparse[si];
            if (r0 + kStepRows - 16 < delta) break;                 // same test as the producer
            const int fs = far_count % plan.n_far_stages;
            mbar_wait(bars.far_full(fs), (far_count / plan.n_far_stages) & 1, abort_flag, 0x203);
            if (active && si < nv) {
                const uint32_t base = smem_base + lay.far + fs * 2 * kTile + warp * 16 * kPitch;
                const uint32_t srcK[1] = {base}, srcV[1] = {base + kTile};
                const bool ok[1] = {true};
                const float pb2[1] = {__ldg(a.pos_bias + (nd + si) * H + h) * kLog2e};
                sparse_group<D, 1>(st, qa, qb, srcK, srcV, ok, pb2, c2, lo, owner, owner_lane, g);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bars.far_empty(fs));
            ++far_count;
        }
        // ---- release the ring blocks that the next step does not need
        __syncwarp();
        if (lane == 0) {
            if (last_of_seq) {
                for (int b = sb - (held - 1); b <= sb; ++b) mbar_arrive(bars.win_empty(b & (nrb - 1)));
            } else {
                mbar_arrive(bars.win_empty((sb - (held - 1)) & (nrb - 1)));
            }
        }
        // ---- epilogue
        if (active) {
            const bool ok_lo = row_lo < N, ok_hi = row_hi < N;
            const float l_lo = quad_sum(st.l_lo), l_hi = quad_sum(st.l_hi);
            const float gain = a.head_gain ? __ldg(a.head_gain + h) : 1.f;
            __nv_bfloat16* op = static_cast<__nv_bfloat16*>(a.out) + (size_t)bh * N * D;
            store_acc_rows_tma<D>(st.O, op + (size_t)row_lo * D, op + (size_t)row_hi * D, ok_lo, ok_hi,
                                  l_lo > 0.f ? gain / l_lo : 0.f, l_hi > 0.f ? gain / l_hi : 0.f, tig);
            if (tig == 0) {
                if (ok_lo) a.lse[(size_t)bh * N + row_lo] = l_lo > 0.f ? (st.m_lo + log2f(l_lo)) * kLn2 : -INFINITY;
                if (ok_hi) a.lse[(size_t)bh * N + row_hi] = l_hi > 0.f ? (st.m_hi + log2f(l_hi)) * kLn2 : -INFINITY;
            }
        }
    }
}

template <int D, int WB>
__global__ void __launch_bounds__(kThreadsTma, 1)
fwd_tma_kernel(const FwdArgs a, const Taps t, const FwdTmaPlan plan,
               const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
               const __grid_constant__ CUtensorMap tm_v) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t smem_base = (raw + 1023u) & ~1023u;          // swizzled tiles want 1024-byte alignment
    uint8_t* gen_base = smem_raw + (smem_base - raw);
    const SmemLayout<D> lay(plan.NR, plan.n_far_stages);
    const Bars bars{smem_base + (uint32_t)lay.bars};
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + lay.misc);
    const int nrb = plan.NR / kStepRows;
    if (threadIdx.x == 0) {
        for (int i = 0; i < nrb; ++i) { mbar_init(bars.win_full(i), 1); mbar_init(bars.win_empty(i), kConsumerWarps); }
        for (int i = 0; i < plan.n_far_stages; ++i) { mbar_init(bars.far_full(i), 1); mbar_init(bars.far_empty(i), kConsumerWarps); }
        for (int i = 0; i < 2; ++i) { mbar_init(bars.q_full(i), 1); mbar_init(bars.q_empty(i), kConsumerWarps); }
        *abort_flag = 0;
        fence_mbar_init();
    }
    __syncthreads();
    const int step_begin = blockIdx.x * plan.steps_per_cta;
    const int step_end = min(plan.total_steps, step_begin + plan.steps_per_cta);
    if (step_begin >= step_end) return;
    if ((threadIdx.x >> 5) == kConsumerWarps) {
        if ((threadIdx.x & 31) == 0) {
            prefetch_tensormap(&tm_q); prefetch_tensormap(&tm_k); prefetch_tensormap(&tm_v);
            producer_loop<D>(plan, t, &tm_q, &tm_k, &tm_v, smem_base, lay, bars, abort_flag, step_begin, step_end);
        }
    } else {
        consumer_loop<D, WB>(a, plan, t, smem_base, lay, bars, abort_flag, step_begin, step_end);
    }
}

// ------------------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// [BH][N][D] bf16 tensor, box = 128 rows x D, swizzle matching the row pitch.
bool make_row_map(CUtensorMap* m, const void* ptr, int BH, int N, int D) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)N, (cuuint64_t)BH};
    cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)N * D * 2};
    cuuint32_t box[3] = {(cuuint32_t)D, (cuuint32_t)kStepRows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, D == 32 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
              CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int band_width_tma(const Taps& t) {
    const int d_hi = t.d_lo + t.n_dense - 1;
    return d_hi <= 32 ? 32 : (d_hi <= 48 ? 48 : (d_hi <= 64 ? 64 : 0));
}

template <int D, int WB>
cudaError_t fwd_launch_tma(const FwdArgs& a, const Taps& t, cudaStream_t stream) {
    int dev = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return e;
    FwdTmaPlan plan;
    plan.NR = D == 32 ? 1024 : 512;
    plan.n_far_stages = D == 32 ? 3 : 2;
    plan.n_win = 0;
    while (plan.n_win < t.n_sparse && t.sparse[plan.n_win] <= plan.NR - 2 * kStepRows) ++plan.n_win;
    plan.steps_per_seq = (a.N + kStepRows - 1) / kStepRows;
    plan.total_steps = a.B * a.H * plan.steps_per_seq;
    const int grid = plan.total_steps < sms ? plan.total_steps : sms;
    plan.steps_per_cta = (plan.total_steps + grid - 1) / grid;
    const SmemLayout<D> lay(plan.NR, plan.n_far_stages);
    const int smem = lay.total + 1024;
    CUtensorMap mq, mk, mv;
    if (!make_row_map(&mq, a.q, a.B * a.H, a.N, D) || !make_row_map(&mk, a.k, a.B * a.H, a.N, D) ||
        !make_row_map(&mv, a.v, a.B * a.H, a.N, D))
        return cudaErrorInvalidValue;
    if ((e = cudaFuncSetAttribute(fwd_tma_kernel<D, WB>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)) != cudaSuccess)
        return e;
    fwd_tma_kernel<D, WB><<<grid, kThreadsTma, smem, stream>>>(a, t, plan, mq, mk, mv);
    return cudaGetLastError();
}

}  // namespace

bool tma_fwd_supported(int dtype, int D, int N, const Taps& t, bool has_scale_embed) {
    if (dtype != DSQG_DTYPE_BF16 || (D != 32 && D != 64) || has_scale_embed) return false;
    if (t.n_sparse > kMaxSparseTma || band_width_tma(t) == 0 || N < 1) return false;
    for (int i = 0; i < t.n_sparse; ++i)
        if (t.sparse[i] % 16 != 0) return false;
    return encode_fn() != nullptr;
}

cudaError_t launch_fwd_tma(const FwdArgs& a, const Taps& t, cudaStream_t s) {
    const int wb = band_width_tma(t);
    if (a.D == 32) {
        if (wb == 32) return fwd_launch_tma<32, 32>(a, t, s);
        if (wb == 48) return fwd_launch_tma<32, 48>(a, t, s);
        return fwd_launch_tma<32, 64>(a, t, s);
    }
    if (wb == 32) return fwd_launch_tma<64, 32>(a, t, s);
    if (wb == 48) return fwd_launch_tma<64, 48>(a, t, s);
    return fwd_launch_tma<64, 64>(a, t, s);
}

cudaError_t read_device_error_fwd_tma(int* value, bool reset) {
    cudaError_t e = cudaMemcpyFromSymbol(value, g_device_error, sizeof(int));
    if (e == cudaSuccess && reset && *value != 0) {
        const int zero = 0;
        e = cudaMemcpyToSymbol(g_device_error, &zero, sizeof(int));
    }
    return e;
}

}  // namespace dsqg
