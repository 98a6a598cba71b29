// Persistent, TMA-fed DSQG forward kernel (bf16, D in {32, 64}, sparse taps multiples of 16).
//
// Row stream.  All (batch, head) sequences are padded to a whole number of 128-row blocks and
// laid end to end; block G of this stream is rows [128*sb, 128*sb+128) of sequence bh with
// G = bh*blocks_per_seq + sb.  A CTA owns a contiguous range of blocks and walks through it,
// so the K/V rows it fetched for one block are still in shared memory when later blocks of
// the same sequence look back at them.
//
// Shared memory.
//   * K ring and V ring of NRB blocks (NRB a power of two): stream block G lives in slot
//     (G - G_first) & (NRB-1).  A tile of block G may read blocks G-look .. G, i.e. the dense
//     window and every sparse tap with delta <= 128*look ("window taps"); the other
//     NRB-1-look slots let the producer fetch blocks ahead of the slowest warp.  Blocks that
//     belong to the previous sequence are simply never addressed: a tap that would reach
//     before row 0 is masked, and dense-window chunks before row 0 are skipped.
//   * "far" taps (delta beyond the window) stream through stages that hold the 128-row K
//     tile and V tile of one (block, tap) pair.
//   * Q tiles: a small ring of 128-row stages.
//
// Warps.  The last warp is the producer (one lane issues every TMA load, running ahead as far
// as the "empty" barriers allow).  The other W warps are consumers; 16-row tile T of the
// CTA's range is processed by consumer warp T mod W, so W need not divide 128.  All barrier
// phases are closed-form functions of the block number, so a warp may skip blocks.  Every
// wait is bounded (dsqg_tma.cuh).
//
// Softmax.  Online over groups: far taps, then the dense window, then the window taps.
#include <cstdlib>

#include "dsqg_tma.cuh"

namespace dsqg {
namespace {

constexpr int kBlockRows = 128;
constexpr int kTilesPerBlock = kBlockRows / 16;
constexpr int kMaxSparseTma = 16;
constexpr int kMaxRingBlocks = 16;
constexpr int kMaxFarStages = 8;
constexpr int kMaxQStages = 4;

struct FwdTmaPlan {
    int nrb;             // ring blocks (power of two)
    int look;            // blocks a tile may look back (window taps: delta <= 128*look); look <= nrb-2
    int n_win;           // sparse taps 0 .. n_win-1 are read from the ring
    int n_far;           // far taps per block (= n_sparse - n_win)
    int n_far_stages, n_q_stages;
    int blocks_per_seq;  // ceil(N / 128)
    int total_blocks;    // B*H*blocks_per_seq
    int blocks_per_cta;
    int consumers;       // W
};

template <int D>
struct SmemLayout {
    static constexpr int kPitch = D * 2;
    static constexpr int kTile = kBlockRows * kPitch;          // one 128-row tile
    int k_ring, v_ring, far, q, bars, misc, total;
    __host__ __device__ SmemLayout(int nrb, int n_far_stages, int n_q_stages) {
        k_ring = 0;
        v_ring = k_ring + nrb * kTile;
        far = v_ring + nrb * kTile;
        q = far + n_far_stages * 2 * kTile;
        bars = q + n_q_stages * kTile;
        misc = bars + 8 * (2 * kMaxRingBlocks + 2 * kMaxFarStages + 2 * kMaxQStages);
        total = misc + 64;
    }
};

struct Bars {           // shared-space addresses of the mbarriers
    uint32_t base;
    __device__ uint32_t win_full(int s) const { return base + 8 * s; }
    __device__ uint32_t win_empty(int s) const { return base + 8 * (kMaxRingBlocks + s); }
    __device__ uint32_t far_full(int s) const { return base + 8 * (2 * kMaxRingBlocks + s); }
    __device__ uint32_t far_empty(int s) const { return base + 8 * (2 * kMaxRingBlocks + kMaxFarStages + s); }
    __device__ uint32_t q_full(int s) const { return base + 8 * (2 * kMaxRingBlocks + 2 * kMaxFarStages + s); }
    __device__ uint32_t q_empty(int s) const { return base + 8 * (2 * kMaxRingBlocks + 2 * kMaxFarStages + kMaxQStages + s); }
};

// Relative block number r = G - (G_begin - look) >= 0 numbers every block the CTA ever loads:
// r = 0 .. look-1 are the look-back blocks fetched before the first own block.
//   ring slot = r & (nrb-1), fill number = r / nrb
// Own blocks are numbered j = G - G_begin = r - look:
//   Q stage = j % n_q_stages; far stage of (j, f) = (j*n_far + f) % n_far_stages.

// ------------------------------------------------------------------------------ producer
template <int D>
__device__ __forceinline__ void producer_loop(const FwdTmaPlan& plan, const Taps& t, const CUtensorMap* tm_q,
                                              const CUtensorMap* tm_k, const CUtensorMap* tm_v, uint32_t smem_base,
                                              const SmemLayout<D>& lay, const Bars& bars, volatile int* abort_flag,
                                              int g_begin, int g_end) {
    constexpr int kTile = SmemLayout<D>::kTile;
    const int nrb = plan.nrb, look = plan.look;
    const int n_blocks = g_end - g_begin;
#pragma unroll 1
    for (int r = 0; r < n_blocks + look; ++r) {
        int G = g_begin - look + r;
        if (G < 0) G = 0;                                   // never addressed by a consumer; keeps the protocol uniform
        const int bh = G / plan.blocks_per_seq, sb = G - bh * plan.blocks_per_seq;
        const int j = r - look;                             // own-block number (negative: look-back block)
        if (j >= 0) {                                       // Q tile of an own block
            const int qs = j % plan.n_q_stages, qn = j / plan.n_q_stages;
            mbar_wait(bars.q_empty(qs), (qn & 1) ^ 1, abort_flag, 0x101);
            mbar_arrive_expect_tx(bars.q_full(qs), kTile);
            tma_load_3d(smem_base + lay.q + qs * kTile, tm_q, bars.q_full(qs), 0, sb * kBlockRows, bh);
        }
        {
            const int slot = r & (nrb - 1), fill = r / nrb;
            mbar_wait(bars.win_empty(slot), (fill & 1) ^ 1, abort_flag, 0x102);
            mbar_arrive_expect_tx(bars.win_full(slot), 2 * kTile);
            tma_load_3d(smem_base + lay.k_ring + slot * kTile, tm_k, bars.win_full(slot), 0, sb * kBlockRows, bh);
            tma_load_3d(smem_base + lay.v_ring + slot * kTile, tm_v, bars.win_full(slot), 0, sb * kBlockRows, bh);
        }
        if (j >= 0) {
#pragma unroll 1
            for (int f = 0; f < plan.n_far; ++f) {
                const int seq = j * plan.n_far + f;
                const int fs = seq % plan.n_far_stages, fn = seq / plan.n_far_stages;
                const int row = sb * kBlockRows - t.sparse[plan.n_win + f];   // may be negative: zero-filled
                mbar_wait(bars.far_empty(fs), (fn & 1) ^ 1, abort_flag, 0x103);
                mbar_arrive_expect_tx(bars.far_full(fs), 2 * kTile);
                tma_load_3d(smem_base + lay.far + fs * 2 * kTile, tm_k, bars.far_full(fs), 0, row, bh);
                tma_load_3d(smem_base + lay.far + fs * 2 * kTile + kTile, tm_v, bars.far_full(fs), 0, row, bh);
            }
        }
        if (*abort_flag) break;
    }
}

// ------------------------------------------------------------------------------ tile math
// Running softmax state of the two rows (g, g+8) a thread works on, plus the output tile.
template <int D>
struct RowState {
    float m_lo, m_hi;          // running maxima (log2 units), never below kMinM
    float l_lo, l_hi;          // this thread's share of the denominators
    float O[D / 8][4];         // value accumulator: n-tile j, slot q <-> row g+8*(q>>1), element 8j+2tig+(q&1)
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
                                             const LaneOff<D>& lo, const ColOff<D>& co, bool owner, int owner_lane, int g) {
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
    // The running maxima rarely move once the dense window has been seen (the distance prior
    // makes far taps small), so the rescale is skipped unless some row of the warp needs it.
    if (__any_sync(0xffffffffu, mn_lo > st.m_lo || mn_hi > st.m_hi)) {
        const float al_lo = ex2(st.m_lo - mn_lo), al_hi = ex2(st.m_hi - mn_hi);
        st.m_lo = mn_lo; st.m_hi = mn_hi;
        st.l_lo *= al_lo; st.l_hi *= al_hi;
#pragma unroll
        for (int j = 0; j < D / 8; ++j) {
            st.O[j][0] *= al_lo; st.O[j][1] *= al_lo; st.O[j][2] *= al_hi; st.O[j][3] *= al_hi;
        }
    }
#pragma unroll
    for (int i = 0; i < G; ++i) {
        const float p0 = ex2(s_lo[i] - mn_lo), p1 = ex2(s_hi[i] - mn_hi);
        if (owner) { st.l_lo += p0; st.l_hi += p1; }
        ColFrag<D> vf;
        ldsm_cols<D>(vf, srcV[i], co);
        uint32_t a0, a3;
        diag_frag(p0, p1, owner, g, a0, a3);
        mma_colfrag<D>(st.O, a0, 0u, 0u, a3, vf);
    }
}

// Dense window of one 16-row tile (sequence rows g0.., ring rows gs..): banded scores against
// the WB+16 preceding/own key rows, folded
// into the running softmax state (merge = the state already holds taps), P.V accumulated.
template <int D, int WB>
__device__ __forceinline__ void dense_window(RowState<D>& st, const RowFrag<D>& qa, const RowFrag<D>& qb,
                                             const float (&biasd)[(WB + 16) / 8][4], uint32_t k_ring, uint32_t v_ring,
                                             int g0, int gs, int ring_mask, float c2, const LaneOff<D>& lo, const ColOff<D>& co, bool merge) {
    constexpr int NT = (WB + 16) / 8;
    constexpr int kPitch = D * 2;
    float S[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        RowFrag<D> kf;
        lds_frag<D>(kf, k_ring + ((gs - WB + 8 * nt) & ring_mask) * kPitch, lo);
        mma_rows_z(S[nt], qa, qb, kf);
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int r = 0; r < 4; ++r) S[nt][r] = fmaf(S[nt][r], c2, biasd[nt][r]);
    // sequence start: 16-key chunks that lie before row 0 do not exist (g0 and WB are multiples
    // of 16, so a chunk is either entirely valid or entirely absent); their ring rows hold
    // rows of the previous sequence and must not contribute
    const int c_first = g0 < WB ? (WB - g0) >> 4 : 0;
    if (c_first > 0) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
            if ((nt >> 1) < c_first) S[nt][0] = S[nt][1] = S[nt][2] = S[nt][3] = kNeg;
    }
    float m_lo = st.m_lo, m_hi = st.m_hi;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        m_lo = fmaxf(m_lo, fmaxf(S[nt][0], S[nt][1]));
        m_hi = fmaxf(m_hi, fmaxf(S[nt][2], S[nt][3]));
    }
    m_lo = quad_max(m_lo); m_hi = quad_max(m_hi);
    if (merge) {                 // warp-uniform: taps were already folded in before the window
        const float al_lo = ex2(st.m_lo - m_lo), al_hi = ex2(st.m_hi - m_hi);
        st.l_lo *= al_lo; st.l_hi *= al_hi;
#pragma unroll
        for (int j = 0; j < D / 8; ++j) {
            st.O[j][0] *= al_lo; st.O[j][1] *= al_lo; st.O[j][2] *= al_hi; st.O[j][3] *= al_hi;
        }
    }
    float l_lo = 0.f, l_hi = 0.f;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        S[nt][0] = ex2(S[nt][0] - m_lo); S[nt][1] = ex2(S[nt][1] - m_lo);
        S[nt][2] = ex2(S[nt][2] - m_hi); S[nt][3] = ex2(S[nt][3] - m_hi);
        l_lo += S[nt][0] + S[nt][1]; l_hi += S[nt][2] + S[nt][3];
    }
    st.m_lo = m_lo; st.m_hi = m_hi; st.l_lo += l_lo; st.l_hi += l_hi;
#pragma unroll
    for (int c = 0; c < NT / 2; ++c) {
        if (c < c_first) continue;
        ColFrag<D> vf;
        ldsm_cols<D>(vf, v_ring + ((gs - WB + 16 * c) & ring_mask) * kPitch, co);
        mma_colfrag<D>(st.O, pack_bf16x2(S[2 * c][0], S[2 * c][1]), pack_bf16x2(S[2 * c][2], S[2 * c][3]),
                       pack_bf16x2(S[2 * c + 1][0], S[2 * c + 1][1]), pack_bf16x2(S[2 * c + 1][2], S[2 * c + 1][3]), vf);
    }
}

constexpr int kGroup = 4;      // window taps processed per branch-free group

// ------------------------------------------------------------------------------ consumers
template <int D, int WB>
__device__ __forceinline__ void consumer_loop(const FwdArgs& a, const FwdTmaPlan& plan, const Taps& t, uint32_t smem_base,
                                              const SmemLayout<D>& lay, const Bars& bars, volatile int* abort_flag,
                                              int g_begin, int g_end) {
    constexpr int NT = (WB + 16) / 8;
    constexpr int kPitch = SmemLayout<D>::kPitch;
    constexpr int kTile = SmemLayout<D>::kTile;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tig = lane & 3;
    const bool owner = tig == (g >> 1);
    const int owner_lane = (lane & ~3) | (g >> 1);
    const LaneOff<D> lo = lane_offsets<D>(g, tig);
    const ColOff<D> co = col_offsets<D>(lane);
    const int N = a.N, H = a.H;
    const int nrb = plan.nrb, look = plan.look, ring_mask = nrb * kBlockRows - 1;
    const int d_lo = t.d_lo, d_hi = t.d_lo + t.n_dense - 1, nd = t.n_dense, ns = t.n_sparse, n_win = plan.n_win;
    const float c2 = a.scale * kLog2e;
    const uint32_t k_ring = smem_base + lay.k_ring, v_ring = smem_base + lay.v_ring;
    const uint32_t maskp = (uint32_t)ring_mask * kPitch | (kPitch - 1);
    const int n_tiles = (g_end - g_begin) * kTilesPerBlock;

    float biasd[NT][4];
    int bias_h = -1;
    // lane j keeps sparse tap j: its offset (pre-multiplied by the row pitch for ring addressing)
    // and, per head, its bias in log2 units; other lanes fetch them with a shuffle
    const int tap_delta = lane < ns ? t.sparse[lane < ns ? lane : 0] : 0x3fffffff;
    const uint32_t tap_deltap = (uint32_t)tap_delta * kPitch;
    float tap_pb2 = 0.f;
    int waited_r = 0;            // ring blocks [0, waited_r) have been waited for by this warp

#pragma unroll 1
    for (int T = warp; T < n_tiles; T += plan.consumers) {
        const int j = T >> 3, tib = T & 7;
        const int G = g_begin + j;
        const int bh = G / plan.blocks_per_seq, sb = G - bh * plan.blocks_per_seq;
        const int r = j + look;
        const int h = bh % H;
        const int g0 = sb * kBlockRows + 16 * tib;          // first row of the tile inside its sequence
        const int gs = r * kBlockRows + 16 * tib;           // the same row in ring coordinates
        const bool active = g0 < N;
        const int row_lo = g0 + g, row_hi = row_lo + 8;

        if (h != bias_h) {       // per-head constants: dense-window bias fragment (Toeplitz) and tap biases
            bias_h = h;
            tap_pb2 = lane < ns ? __ldg(a.pos_bias + (nd + lane) * H + h) * kLog2e : 0.f;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int delta = WB + g + 8 * (q >> 1) - (8 * nt + 2 * tig + (q & 1));
                    biasd[nt][q] = (delta >= d_lo && delta <= d_hi) ? __ldg(a.pos_bias + (delta - d_lo) * H + h) * kLog2e : kNeg;
                }
        }
        // ---- ring blocks up to the tile's own block (each block is waited for once per warp)
#pragma unroll 1
        for (; waited_r <= r; ++waited_r)
            mbar_wait(bars.win_full(waited_r & (nrb - 1)), (waited_r / nrb) & 1, abort_flag, 0x202);
        // ---- Q fragments
        RowFrag<D> qa, qb;
        {
            const int qs = j % plan.n_q_stages;
            mbar_wait(bars.q_full(qs), (j / plan.n_q_stages) & 1, abort_flag, 0x201);
            const uint32_t qt = smem_base + lay.q + qs * kTile + tib * 16 * kPitch;
            lds_frag<D>(qa, qt, lo);
            lds_frag<D>(qb, qt + 8 * kPitch, lo);
            __syncwarp();
            if (lane == 0) mbar_arrive(bars.q_empty(qs));
        }
        // number of sparse taps that stay inside the sequence for this tile (taps ascend and are
        // multiples of 16, as is g0: a tap is valid for all 16 rows or for none)
        const int nv = __popc(__ballot_sync(0xffffffffu, lane < ns && tap_delta <= g0));

        RowState<D> st;
        st.m_lo = st.m_hi = kMinM; st.l_lo = st.l_hi = 0.f;
#pragma unroll
        for (int jj = 0; jj < D / 8; ++jj) st.O[jj][0] = st.O[jj][1] = st.O[jj][2] = st.O[jj][3] = 0.f;
        // ---- far taps first, so that their stages are free again early
        bool merged = false;
#pragma unroll 1
        for (int f = 0; f < plan.n_far; ++f) {
            const int seq = j * plan.n_far + f;
            const int fs = seq % plan.n_far_stages;
            mbar_wait(bars.far_full(fs), (seq / plan.n_far_stages) & 1, abort_flag, 0x203);
            if (active && n_win + f < nv) {
                const uint32_t base = smem_base + lay.far + fs * 2 * kTile + tib * 16 * kPitch;
                const uint32_t srcK[1] = {base}, srcV[1] = {base + kTile};
                const bool ok[1] = {true};
                const float pb2[1] = {__shfl_sync(0xffffffffu, tap_pb2, n_win + f)};
                sparse_group<D, 1>(st, qa, qb, srcK, srcV, ok, pb2, c2, lo, co, owner, owner_lane, g);
                merged = true;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bars.far_empty(fs));
        }
        if (active) {
            dense_window<D, WB>(st, qa, qb, biasd, k_ring, v_ring, g0, gs, ring_mask, c2, lo, co, merged);
            const int nvw = nv < n_win ? nv : n_win;
            const uint32_t gsp = (uint32_t)gs * kPitch;
#pragma unroll 1
            for (int t0 = 0; t0 < nvw; t0 += kGroup) {
                uint32_t srcK[kGroup], srcV[kGroup];
                bool ok[kGroup];
                float pb2[kGroup];
#pragma unroll
                for (int i = 0; i < kGroup; ++i) {
                    ok[i] = t0 + i < nvw;
                    const int ti = ok[i] ? t0 + i : nvw - 1;
                    const uint32_t off = (gsp - __shfl_sync(0xffffffffu, tap_deltap, ti)) & maskp;
                    srcK[i] = k_ring + off; srcV[i] = v_ring + off;
                    pb2[i] = __shfl_sync(0xffffffffu, tap_pb2, ti);
                }
                sparse_group<D, kGroup>(st, qa, qb, srcK, srcV, ok, pb2, c2, lo, co, owner, owner_lane, g);
            }
        }
        // ---- this tile is done with every ring block it could read
        __syncwarp();
        if (lane == 0) {
#pragma unroll 1
            for (int b = r - look; b <= r; ++b) mbar_arrive(bars.win_empty(b & (nrb - 1)));
        }
        // ---- epilogue
        if (active) {
            const bool ok_lo = row_lo < N, ok_hi = row_hi < N;
            const float l_lo = quad_sum(st.l_lo), l_hi = quad_sum(st.l_hi);
            const float gain = a.head_gain ? __ldg(a.head_gain + h) : 1.f;
            __nv_bfloat16* op = static_cast<__nv_bfloat16*>(a.out) + (size_t)bh * N * D;
            store_acc_std<D>(st.O, op + (size_t)row_lo * D, op + (size_t)row_hi * D, ok_lo, ok_hi,
                             l_lo > 0.f ? __fdividef(gain, l_lo) : 0.f, l_hi > 0.f ? __fdividef(gain, l_hi) : 0.f, tig);
            if (tig == 0) {
                if (ok_lo) a.lse[(size_t)bh * N + row_lo] = l_lo > 0.f ? (st.m_lo + __log2f(l_lo)) * kLn2 : -INFINITY;
                if (ok_hi) a.lse[(size_t)bh * N + row_hi] = l_hi > 0.f ? (st.m_hi + __log2f(l_hi)) * kLn2 : -INFINITY;
            }
        }
    }
}

template <int D, int WB, int W>
__global__ void __launch_bounds__((W + 1) * 32, 1)
fwd_tma_kernel(const FwdArgs a, const Taps t, const FwdTmaPlan plan,
               const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
               const __grid_constant__ CUtensorMap tm_v) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t smem_base = (raw + 1023u) & ~1023u;          // swizzled tiles want 1024-byte alignment
    uint8_t* gen_base = smem_raw + (smem_base - raw);
    const SmemLayout<D> lay(plan.nrb, plan.n_far_stages, plan.n_q_stages);
    const Bars bars{smem_base + (uint32_t)lay.bars};
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + lay.misc);
    const int nrb = plan.nrb, look = plan.look;
    if (threadIdx.x == 0) {
        for (int i = 0; i < nrb; ++i) {
            mbar_init(bars.win_full(i), 1);
            mbar_init(bars.win_empty(i), (look + 1) * kTilesPerBlock);   // every tile of the blocks that can read it
        }
        for (int i = 0; i < plan.n_far_stages; ++i) { mbar_init(bars.far_full(i), 1); mbar_init(bars.far_empty(i), kTilesPerBlock); }
        for (int i = 0; i < plan.n_q_stages; ++i) { mbar_init(bars.q_full(i), 1); mbar_init(bars.q_empty(i), kTilesPerBlock); }
        *abort_flag = 0;
        fence_mbar_init();
        // look-back block b (b < look) is only read by the own blocks b+1 .. look of the first
        // `look` ones... i.e. by (b + 1) blocks instead of look + 1: make up for the missing tiles
        for (int b = 0; b < look; ++b)
            for (int k = 0; k < (look - b) * kTilesPerBlock; ++k) mbar_arrive(bars.win_empty(b & (nrb - 1)));
    }
    __syncthreads();
    const int g_begin = blockIdx.x * plan.blocks_per_cta;
    const int g_end = min(plan.total_blocks, g_begin + plan.blocks_per_cta);
    if (g_begin >= g_end) return;
    if ((threadIdx.x >> 5) == W) {
        if ((threadIdx.x & 31) == 0) {
            prefetch_tensormap(&tm_q); prefetch_tensormap(&tm_k); prefetch_tensormap(&tm_v);
            producer_loop<D>(plan, t, &tm_q, &tm_k, &tm_v, smem_base, lay, bars, abort_flag, g_begin, g_end);
        }
    } else {
        consumer_loop<D, WB>(a, plan, t, smem_base, lay, bars, abort_flag, g_begin, g_end);
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
    cuuint32_t box[3] = {(cuuint32_t)D, (cuuint32_t)kBlockRows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, D == 32 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
              CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int band_width_tma(const Taps& t) {
    const int d_hi = t.d_lo + t.n_dense - 1;
    return d_hi <= 32 ? 32 : (d_hi <= 48 ? 48 : (d_hi <= 64 ? 64 : 0));
}

constexpr int kSmemLimit = 227 * 1024;

template <int D, int WB, int W>
cudaError_t fwd_launch_tma(const FwdArgs& a, const Taps& t, cudaStream_t stream) {
    int dev = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return e;
    FwdTmaPlan plan;
    plan.consumers = W;
    plan.nrb = 8;                               // 8 x 128 rows of K and of V: 128 KB at D = 32
    if (D == 64) plan.nrb = 4;
    // Consumer warps run up to ~2 blocks apart, so the ring keeps nrb-1-look blocks of slack for
    // the producer to run ahead (measured best on B200: look = nrb-3 with 15 consumer warps).
    { const char* lk = getenv("DSQG_FWD_LOOK"); plan.look = lk ? atoi(lk) : plan.nrb - 3; }
    if (plan.look > plan.nrb - 2) plan.look = plan.nrb - 2;
    if (plan.look < 1) plan.look = 1;
    { const char* qs = getenv("DSQG_FWD_QSTAGES"); plan.n_q_stages = qs ? atoi(qs) : (D == 32 ? 3 : 2); }
    if (plan.n_q_stages < 2) plan.n_q_stages = 2;
    if (plan.n_q_stages > kMaxQStages) plan.n_q_stages = kMaxQStages;
    plan.n_win = 0;
    while (plan.n_win < t.n_sparse && t.sparse[plan.n_win] <= plan.look * kBlockRows) ++plan.n_win;
    plan.n_far = t.n_sparse - plan.n_win;
    // as many far stages as shared memory allows (at least 1 when there are far taps)
    plan.n_far_stages = plan.n_far > 0 ? 1 : 0;
    while (plan.n_far > 0 && plan.n_far_stages < kMaxFarStages && plan.n_far_stages < 2 * plan.n_far &&
           SmemLayout<D>(plan.nrb, plan.n_far_stages + 1, plan.n_q_stages).total + 1024 <= kSmemLimit)
        ++plan.n_far_stages;
    plan.blocks_per_seq = (a.N + kBlockRows - 1) / kBlockRows;
    plan.total_blocks = a.B * a.H * plan.blocks_per_seq;
    const int grid = plan.total_blocks < sms ? plan.total_blocks : sms;
    plan.blocks_per_cta = (plan.total_blocks + grid - 1) / grid;
    const SmemLayout<D> lay(plan.nrb, plan.n_far_stages, plan.n_q_stages);
    const int smem = lay.total + 1024;
    if (smem > kSmemLimit) return cudaErrorInvalidConfiguration;
    CUtensorMap mq, mk, mv;
    if (!make_row_map(&mq, a.q, a.B * a.H, a.N, D) || !make_row_map(&mk, a.k, a.B * a.H, a.N, D) ||
        !make_row_map(&mv, a.v, a.B * a.H, a.N, D))
        return cudaErrorInvalidValue;
    if ((e = cudaFuncSetAttribute(fwd_tma_kernel<D, WB, W>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)) != cudaSuccess)
        return e;
    fwd_tma_kernel<D, WB, W><<<grid, (W + 1) * 32, smem, stream>>>(a, t, plan, mq, mk, mv);
    return cudaGetLastError();
}

template <int D, int WB>
cudaError_t fwd_launch_tma_w(const FwdArgs& a, const Taps& t, cudaStream_t stream) {
    const char* w = getenv("DSQG_FWD_WARPS");
    const int W = w ? atoi(w) : (D == 32 ? 15 : 8);     // measured best on B200
    // at least 8 consumer warps: the 8 tiles of a block must sit on 8 different warps, or a warp
    // would wait for a stage that only its own later tile can release
    if (W == 8) return fwd_launch_tma<D, WB, 8>(a, t, stream);
    if (W == 11) return fwd_launch_tma<D, WB, 11>(a, t, stream);
    return fwd_launch_tma<D, WB, 15>(a, t, stream);
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
        if (wb == 32) return fwd_launch_tma_w<32, 32>(a, t, s);
        if (wb == 48) return fwd_launch_tma_w<32, 48>(a, t, s);
        return fwd_launch_tma_w<32, 64>(a, t, s);
    }
    if (wb == 32) return fwd_launch_tma_w<64, 32>(a, t, s);
    if (wb == 48) return fwd_launch_tma_w<64, 48>(a, t, s);
    return fwd_launch_tma_w<64, 64>(a, t, s);
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
