// Persistent, TMA-fed DSQG backward kernels (bf16, D in {32, 64}, sparse taps multiples of 16).
//
// Both kernels run on the pipeline of dsqg_pipe.cuh (row stream of 128-row blocks, one CTA per
// SM, ring of look-back / look-ahead blocks in shared memory, far-tap stages, producer warp +
// consumer warps taking 16-row tiles round-robin) and on the warp-level tensor-core math of
// dsqg_mma.cuh.  They follow the DWARF reference kernels kernels/dsqg_attention_v3.py:198-275
// (dQ, dpos_bias; delta = sum_d dout*out as in :170-191) and :282-352 (dK, dV), with the
// per-head output gain of train/train_2048_condU.py:187 folded in.
//
// dQ kernel (query-owned).  Ring/far: K and V; own stage: Q and dO.  Per tile:
//   delta from the saved output, p = exp2(s - lse), ds = p (gain dO.v - delta),
//   dQ += ds K (K re-read transposed with ldmatrix), and running sums of ds per offset
//   (dpos_bias) and of p dO.v (dhead_gain).  Those sums live in registers / a per-warp table
//   and are written out per (sequence, CTA, warp) when the warp moves to another sequence;
//   a second kernel adds them in a fixed order: no atomics, bitwise reproducible.
// dK/dV kernel (key-owned).  Ring/far: Q and dO (looking AHEAD: key row m is used by query
//   rows m + delta); own stage: K and V.  lse and delta of the query rows come from global
//   memory.  Key rows are owned by exactly one warp, so dK and dV need no atomics either.
#include <cstdlib>

#include "dsqg_pipe.cuh"

namespace dsqg {
namespace {

using namespace pipe;

constexpr int kMaxSparseTma = 16;
constexpr int kWarpScratchFloats = 256 + kMaxSparseTma * 8;   // per consumer warp: flush staging + sparse-tap sums

// rows g / g+8 of a global [N][D] slice in the fragment layout of the swizzled shared tiles
template <int D>
__device__ __forceinline__ void load_row_ce(RowFrag<D>& f, const __nv_bfloat16* row_ptr, int tig, bool valid) {
#pragma unroll
    for (int c = 0; c < D / 32; ++c) {
        uint4 u = make_uint4(0u, 0u, 0u, 0u);
        if (valid) u = __ldg(reinterpret_cast<const uint4*>(row_ptr + chunk_elem<D>(tig, c)));
        f.r[4 * c + 0] = u.x; f.r[4 * c + 1] = u.y; f.r[4 * c + 2] = u.z; f.r[4 * c + 3] = u.w;
    }
}

struct BwdTmaExtra {
    int* slot_bh;        // [n_slots] sequence (b*H+h) a partial slot belongs to, -1 = unused
    float* dpb_part;     // [n_slots][W][J]
    float* dg_part;      // [n_slots][W]
    int n_slots;
};

// Everything a thread needs to know about one row pair of a dQ tile.
struct RowPair {
    float l2_lo, l2_hi;        // lse in log2 units
    float dl_lo, dl_hi;        // delta
};

// ------------------------------------------------------------------------------ dQ: tile math
// G sparse taps of a dQ tile, branch-free.  sp_tab is this warp's [tap][8] table of ds sums; the
// entry (tap, g) is only ever touched by the lane that owns rows g and g+8.
template <int D, int G>
__device__ __forceinline__ void dq_sparse_group(float (&dQ)[D / 8][4], float& dgrow, float* sp_tab,
                                                const RowFrag<D>& qa, const RowFrag<D>& qb, const RowFrag<D>& da,
                                                const RowFrag<D>& db, const uint32_t (&srcK)[G], const uint32_t (&srcV)[G],
                                                const bool (&ok)[G], const float (&pb2)[G], const int (&ti)[G],
                                                const RowPair& rp, float c2, float gain, const LaneOff<D>& lo,
                                                const ColOff<D>& co, bool owner, int g) {
    constexpr int kPitch = D * 2;
#pragma unroll
    for (int i = 0; i < G; ++i) {
        RowFrag<D> kf0, kf1, vf0, vf1;
        lds_frag<D>(kf0, srcK[i], lo);
        lds_frag<D>(kf1, srcK[i] + 8 * kPitch, lo);
        lds_frag<D>(vf0, srcV[i], lo);
        lds_frag<D>(vf1, srcV[i] + 8 * kPitch, lo);
        float s0[4], s1[4], e0[4], e1[4];
        mma_rows_z(s0, qa, qb, kf0); mma_rows_z(s1, qa, qb, kf1);
        mma_rows_z(e0, da, db, vf0); mma_rows_z(e1, da, db, vf1);
        const float sd0 = (g & 1) ? s0[1] : s0[0], sd1 = (g & 1) ? s1[3] : s1[2];
        const float dp0 = (g & 1) ? e0[1] : e0[0], dp1 = (g & 1) ? e1[3] : e1[2];
        const float p0 = ok[i] ? ex2(fmaf(sd0, c2, pb2[i]) - rp.l2_lo) : 0.f;
        const float p1 = ok[i] ? ex2(fmaf(sd1, c2, pb2[i]) - rp.l2_hi) : 0.f;
        const float x0 = p0 * (gain * dp0 - rp.dl_lo), x1 = p1 * (gain * dp1 - rp.dl_hi);
        if (owner) {
            dgrow = fmaf(p0, dp0, dgrow); dgrow = fmaf(p1, dp1, dgrow);
            sp_tab[ti[i] * 8 + g] += x0 + x1;
        }
        uint32_t a0, a3;
        diag_frag(x0, x1, owner, g, a0, a3);
        ColFrag<D> kc;
        ldsm_cols<D>(kc, srcK[i], co);
        mma_colfrag<D>(dQ, a0, 0u, 0u, a3, kc);
    }
}

// Dense window of a dQ tile.  dpb_d mirrors the bias fragment: element (nt, q) always has the
// same offset delta, so the running sums of ds per offset stay in registers.
template <int D, int WB>
__device__ __forceinline__ void dq_dense(float (&dQ)[D / 8][4], float& dgrow, float (&dpb_d)[(WB + 16) / 8][4],
                                         const RowFrag<D>& qa, const RowFrag<D>& qb, const RowFrag<D>& da,
                                         const RowFrag<D>& db, const float (&biasd)[(WB + 16) / 8][4], uint32_t k_ring,
                                         uint32_t v_ring, int g0, int gs, int ring_mask, float c2, float gain,
                                         const RowPair& rp, const LaneOff<D>& lo, const ColOff<D>& co) {
    constexpr int NT = (WB + 16) / 8;
    constexpr int kPitch = D * 2;
    const int c_first = g0 < WB ? (WB - g0) >> 4 : 0;     // 16-key chunks before row 0 do not exist
#pragma unroll
    for (int c = 0; c < NT / 2; ++c) {
        if (c < c_first) continue;
        float ds[2][4];
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
            const int nt = 2 * c + hf;
            const uint32_t rb = ((gs - WB + 8 * nt) & ring_mask) * kPitch;
            RowFrag<D> kf, vf;
            lds_frag<D>(kf, k_ring + rb, lo);
            lds_frag<D>(vf, v_ring + rb, lo);
            float s[4], dp[4];
            mma_rows_z(s, qa, qb, kf);
            mma_rows_z(dp, da, db, vf);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float p = ex2(fmaf(s[q], c2, biasd[nt][q]) - (q < 2 ? rp.l2_lo : rp.l2_hi));   // out of band: exp2(-1e30) = 0
                const float x = p * (gain * dp[q] - (q < 2 ? rp.dl_lo : rp.dl_hi));
                dgrow = fmaf(p, dp[q], dgrow);
                dpb_d[nt][q] += x;
                ds[hf][q] = x;
            }
        }
        ColFrag<D> kc;
        ldsm_cols<D>(kc, k_ring + ((gs - WB + 16 * c) & ring_mask) * kPitch, co);
        mma_colfrag<D>(dQ, pack_bf16x2(ds[0][0], ds[0][1]), pack_bf16x2(ds[0][2], ds[0][3]),
                       pack_bf16x2(ds[1][0], ds[1][1]), pack_bf16x2(ds[1][2], ds[1][3]), kc);
    }
}

// Writes this warp's running sums for sequence `bh` to partial slot `slot` and clears them.
// Dense sums are regrouped by offset through a 256-float staging area (two n-tiles at a time):
// offset delta receives, from every row i of the tile, the element in column WB + i - delta.
template <int WB>
__device__ __forceinline__ void dq_flush(float (&dpb_d)[(WB + 16) / 8][4], float& dg, float* wscr, const BwdTmaExtra& x,
                                         int slot, int bh, int W, int J, int nd, int ns, int d_lo, int warp, int lane) {
    constexpr int NT = (WB + 16) / 8;
    float* stage = wscr;
    float* sp_tab = wscr + 256;
    float acc[3] = {0.f, 0.f, 0.f};                      // offsets lane, lane+32, lane+64 (n_dense <= 65)
#pragma unroll
    for (int pass = 0; pass < NT / 2; ++pass) {
#pragma unroll
        for (int s8 = 0; s8 < 8; ++s8) stage[s8 * 32 + lane] = dpb_d[2 * pass + (s8 >> 2)][s8 & 3];
        __syncwarp();
#pragma unroll
        for (int jj = 0; jj < 3; ++jj) {
            const int j = lane + 32 * jj;
            if (j < nd) {
                const int delta = d_lo + j;
                for (int i = 0; i < 16; ++i) {
                    const int c = WB + i - delta;
                    if (c >= 0 && (c >> 4) == pass)
                        acc[jj] += stage[(((c >> 3) & 1) * 4 + (i >> 3) * 2 + (c & 1)) * 32 + 4 * (i & 7) + ((c & 7) >> 1)];
                }
            }
        }
        __syncwarp();
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) dpb_d[nt][0] = dpb_d[nt][1] = dpb_d[nt][2] = dpb_d[nt][3] = 0.f;
    float* out = x.dpb_part + ((size_t)slot * W + warp) * J;
#pragma unroll
    for (int jj = 0; jj < 3; ++jj)
        if (lane + 32 * jj < nd) out[lane + 32 * jj] = acc[jj];
    if (lane < ns) {
        float s = 0.f;
        for (int gg = 0; gg < 8; ++gg) { s += sp_tab[lane * 8 + gg]; sp_tab[lane * 8 + gg] = 0.f; }
        out[nd + lane] = s;
    }
    float d = dg;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
    if (lane == 0) { x.dg_part[(size_t)slot * W + warp] = d; x.slot_bh[slot] = bh; }
    dg = 0.f;
    __syncwarp();
}

constexpr int kGroupBwd = 2;

// ------------------------------------------------------------------------------ dQ: consumer warps
template <int D, int WB>
__device__ __forceinline__ void dq_consumer_loop(const BwdArgs& a, const BwdTmaExtra& x, const Plan& plan, const Taps& t,
                                                 uint32_t smem_base, uint8_t* gen_base, const Smem<D, 2>& lay,
                                                 const Bars& bars, volatile int* abort_flag, int g_begin, int g_end) {
    constexpr int NT = (WB + 16) / 8;
    constexpr int kPitch = Smem<D, 2>::kPitch;
    constexpr int kTile = Smem<D, 2>::kTile;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tig = lane & 3;
    const bool owner = tig == (g >> 1);
    const LaneOff<D> lo = lane_offsets<D>(g, tig);
    const ColOff<D> co = col_offsets<D>(lane);
    const int N = a.N, H = a.H, J = t.J, W = plan.consumers;
    const int nrb = plan.nrb, look = plan.look, ring_mask = nrb * kBlockRows - 1;
    const int d_lo = t.d_lo, d_hi = t.d_lo + t.n_dense - 1, nd = t.n_dense, ns = t.n_sparse, n_win = plan.n_win;
    const float c2 = a.scale * kLog2e;
    const uint32_t k_ring = smem_base + lay.ring0, v_ring = smem_base + lay.ring1;
    const uint32_t maskp = (uint32_t)ring_mask * kPitch | (kPitch - 1);
    const int n_tiles = (g_end - g_begin) * kTilesPerBlock;
    float* wscr = reinterpret_cast<float*>(gen_base + lay.extra) + warp * kWarpScratchFloats;
    float* sp_tab = wscr + 256;
    for (int i = lane; i < kMaxSparseTma * 8; i += 32) sp_tab[i] = 0.f;
    __syncwarp();

    float biasd[NT][4], dpb_d[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) dpb_d[nt][0] = dpb_d[nt][1] = dpb_d[nt][2] = dpb_d[nt][3] = 0.f;
    float dg = 0.f, gain = 1.f;
    const int tap_delta = lane < ns ? t.sparse[lane < ns ? lane : 0] : 0x3fffffff;
    const uint32_t tap_deltap = (uint32_t)tap_delta * kPitch;
    float tap_pb2 = 0.f;
    int waited_r = 0;
    const int bh_first = g_begin / plan.blocks_per_seq, bh_last = (g_end - 1) / plan.blocks_per_seq;
    int cur_bh = bh_first - 1;                           // sequence whose sums are being accumulated

#pragma unroll 1
    for (int T = warp; T < n_tiles; T += W) {
        const int j = T >> 3, tib = T & 7;
        const int G = g_begin + j;
        const int bh = G / plan.blocks_per_seq, sb = G - bh * plan.blocks_per_seq;
        const int r = j + look;
        const int h = bh % H;
        const int g0 = sb * kBlockRows + 16 * tib, gs = r * kBlockRows + 16 * tib;
        const bool active = g0 < N;
        const int row_lo = g0 + g, row_hi = row_lo + 8;
        const bool ok_lo = row_lo < N, ok_hi = row_hi < N;

        if (bh != cur_bh) {
            // close every sequence up to bh-1 (a sequence this warp had no tile of gets zeros), then
            // load the per-head constants of the new one
            for (int b = cur_bh < bh_first ? bh_first : cur_bh; b < bh; ++b)
                dq_flush<WB>(dpb_d, dg, wscr, x, blockIdx.x + b, b, W, J, nd, ns, d_lo, warp, lane);
            cur_bh = bh;
            gain = a.head_gain ? __ldg(a.head_gain + h) : 1.f;
            tap_pb2 = lane < ns ? __ldg(a.pos_bias + (nd + lane) * H + h) * kLog2e : 0.f;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int delta = WB + g + 8 * (q >> 1) - (8 * nt + 2 * tig + (q & 1));
                    biasd[nt][q] = (delta >= d_lo && delta <= d_hi) ? __ldg(a.pos_bias + (delta - d_lo) * H + h) * kLog2e : kNeg;
                }
        }
#pragma unroll 1
        for (; waited_r <= r; ++waited_r)
            mbar_wait(bars.win_full(waited_r & (nrb - 1)), (waited_r / nrb) & 1, abort_flag, 0x212);
        // ---- Q and dO fragments of the tile, row statistics
        RowFrag<D> qa, qb, da, db;
        {
            const int os = j % plan.n_own_stages;
            mbar_wait(bars.own_full(os), (j / plan.n_own_stages) & 1, abort_flag, 0x211);
            const uint32_t qt = smem_base + lay.own + os * 2 * kTile + tib * 16 * kPitch;
            lds_frag<D>(qa, qt, lo);
            lds_frag<D>(qb, qt + 8 * kPitch, lo);
            lds_frag<D>(da, qt + kTile, lo);
            lds_frag<D>(db, qt + kTile + 8 * kPitch, lo);
            __syncwarp();
            if (lane == 0) mbar_arrive(bars.own_empty(os));
        }
        const size_t base = (size_t)bh * N * D;
        RowPair rp;
        {
            const __nv_bfloat16* op = static_cast<const __nv_bfloat16*>(a.out) + base;
            RowFrag<D> oa, ob;
            load_row_ce<D>(oa, op + (size_t)row_lo * D, tig, ok_lo);
            load_row_ce<D>(ob, op + (size_t)row_hi * D, tig, ok_hi);
            rp.dl_lo = quad_sum(frag_dot(da, oa));
            rp.dl_hi = quad_sum(frag_dot(db, ob));
            rp.l2_lo = 0.f; rp.l2_hi = 0.f;
            if (ok_lo) { const float v = __ldg(a.lse + (size_t)bh * N + row_lo); rp.l2_lo = v == -INFINITY ? 0.f : v * kLog2e; }
            if (ok_hi) { const float v = __ldg(a.lse + (size_t)bh * N + row_hi); rp.l2_hi = v == -INFINITY ? 0.f : v * kLog2e; }
            if (tig == 0) {
                if (ok_lo) a.delta[(size_t)bh * N + row_lo] = rp.dl_lo;
                if (ok_hi) a.delta[(size_t)bh * N + row_hi] = rp.dl_hi;
            }
        }
        const int nv = __popc(__ballot_sync(0xffffffffu, lane < ns && tap_delta <= g0));
        float dQ[D / 8][4];
#pragma unroll
        for (int jj = 0; jj < D / 8; ++jj) dQ[jj][0] = dQ[jj][1] = dQ[jj][2] = dQ[jj][3] = 0.f;
        float dgrow = 0.f;
        // ---- far taps
#pragma unroll 1
        for (int f = 0; f < plan.n_far; ++f) {
            const int seq = j * plan.n_far + f;
            const int fs = seq % plan.n_far_stages;
            mbar_wait(bars.far_full(fs), (seq / plan.n_far_stages) & 1, abort_flag, 0x213);
            if (active && n_win + f < nv) {
                const uint32_t fb = smem_base + lay.far + fs * 2 * kTile + tib * 16 * kPitch;
                const uint32_t srcK[1] = {fb}, srcV[1] = {fb + kTile};
                const bool ok[1] = {true};
                const float pb2[1] = {__shfl_sync(0xffffffffu, tap_pb2, n_win + f)};
                const int ti[1] = {n_win + f};
                dq_sparse_group<D, 1>(dQ, dgrow, sp_tab, qa, qb, da, db, srcK, srcV, ok, pb2, ti, rp, c2, gain, lo, co, owner, g);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bars.far_empty(fs));
        }
        if (active) {
            dq_dense<D, WB>(dQ, dgrow, dpb_d, qa, qb, da, db, biasd, k_ring, v_ring, g0, gs, ring_mask, c2, gain, rp, lo, co);
            const int nvw = nv < n_win ? nv : n_win;
            const uint32_t gsp = (uint32_t)gs * kPitch;
#pragma unroll 1
            for (int t0 = 0; t0 < nvw; t0 += kGroupBwd) {
                uint32_t srcK[kGroupBwd], srcV[kGroupBwd];
                bool ok[kGroupBwd];
                float pb2[kGroupBwd];
                int ti[kGroupBwd];
#pragma unroll
                for (int i = 0; i < kGroupBwd; ++i) {
                    ok[i] = t0 + i < nvw;
                    ti[i] = ok[i] ? t0 + i : nvw - 1;
                    const uint32_t off = (gsp - __shfl_sync(0xffffffffu, tap_deltap, ti[i])) & maskp;
                    srcK[i] = k_ring + off; srcV[i] = v_ring + off;
                    pb2[i] = __shfl_sync(0xffffffffu, tap_pb2, ti[i]);
                }
                dq_sparse_group<D, kGroupBwd>(dQ, dgrow, sp_tab, qa, qb, da, db, srcK, srcV, ok, pb2, ti, rp, c2, gain, lo, co, owner, g);
            }
        }
        dg += dgrow;
        __syncwarp();
        if (lane == 0) {
#pragma unroll 1
            for (int b = r - look; b <= r; ++b) mbar_arrive(bars.win_empty(b & (nrb - 1)));
        }
        if (active) {
            __nv_bfloat16* dqp = static_cast<__nv_bfloat16*>(a.dq) + base;
            store_acc_std<D>(dQ, dqp + (size_t)row_lo * D, dqp + (size_t)row_hi * D, ok_lo, ok_hi, a.scale, a.scale, tig);
        }
    }
    // close the remaining sequences of the CTA's range
    for (int b = cur_bh < bh_first ? bh_first : cur_bh; b <= bh_last; ++b)
        dq_flush<WB>(dpb_d, dg, wscr, x, blockIdx.x + b, b, W, J, nd, ns, d_lo, warp, lane);
}

// ------------------------------------------------------------------------------ dK/dV: tile math
constexpr float kBigL2 = 1.0e30f;          // lse stand-in for query rows that do not exist: exp2(x - 1e30) = 0
constexpr int kStatRows = 96;              // per-warp lse/delta window: 16 + WB rows, WB <= 64 (80 used)

// G sparse taps of a dK/dV tile, branch-free.  stat[i]: lanes 0-15 hold lse (log2 units) of query
// rows m0+delta+lane, lanes 16-31 hold delta of rows m0+delta+(lane-16).
template <int D, int G>
__device__ __forceinline__ void dkdv_sparse_group(float (&dK)[D / 8][4], float (&dV)[D / 8][4],
                                                  const RowFrag<D>& ka, const RowFrag<D>& kb, const RowFrag<D>& va,
                                                  const RowFrag<D>& vb, const uint32_t (&srcQ)[G], const uint32_t (&srcD)[G],
                                                  const bool (&ok)[G], const float (&pb2)[G], const float (&stat)[G],
                                                  float c2, float gain, const LaneOff<D>& lo, const ColOff<D>& co,
                                                  bool owner, int g) {
    constexpr int kPitch = D * 2;
#pragma unroll
    for (int i = 0; i < G; ++i) {
        RowFrag<D> qf0, qf1, df0, df1;
        lds_frag<D>(qf0, srcQ[i], lo);
        lds_frag<D>(qf1, srcQ[i] + 8 * kPitch, lo);
        lds_frag<D>(df0, srcD[i], lo);
        lds_frag<D>(df1, srcD[i] + 8 * kPitch, lo);
        float s0[4], s1[4], e0[4], e1[4];
        mma_rows_z(s0, ka, kb, qf0); mma_rows_z(s1, ka, kb, qf1);
        mma_rows_z(e0, va, vb, df0); mma_rows_z(e1, va, vb, df1);
        const float sd0 = (g & 1) ? s0[1] : s0[0], sd1 = (g & 1) ? s1[3] : s1[2];
        const float dp0 = (g & 1) ? e0[1] : e0[0], dp1 = (g & 1) ? e1[3] : e1[2];
        const float l0 = __shfl_sync(0xffffffffu, stat[i], g), l1 = __shfl_sync(0xffffffffu, stat[i], g + 8);
        const float d0 = __shfl_sync(0xffffffffu, stat[i], 16 + g), d1 = __shfl_sync(0xffffffffu, stat[i], 24 + g);
        const float p0 = ok[i] ? ex2(fmaf(sd0, c2, pb2[i]) - l0) : 0.f;
        const float p1 = ok[i] ? ex2(fmaf(sd1, c2, pb2[i]) - l1) : 0.f;
        uint32_t a0, a3;
        ColFrag<D> cf;
        diag_frag(p0 * gain, p1 * gain, owner, g, a0, a3);
        ldsm_cols<D>(cf, srcD[i], co);
        mma_colfrag<D>(dV, a0, 0u, 0u, a3, cf);
        diag_frag(p0 * (gain * dp0 - d0), p1 * (gain * dp1 - d1), owner, g, a0, a3);
        ldsm_cols<D>(cf, srcQ[i], co);
        mma_colfrag<D>(dK, a0, 0u, 0u, a3, cf);
    }
}

// Dense window of a dK/dV tile: keys m0..m0+15 against query rows m0 .. m0+16+WB-1 (ring rows gs..).
// stat_l2 / stat_dl: this warp's lse (log2 units, kBigL2 for rows >= N) and delta of those query rows.
template <int D, int WB>
__device__ __forceinline__ void dkdv_dense(float (&dK)[D / 8][4], float (&dV)[D / 8][4], const RowFrag<D>& ka,
                                           const RowFrag<D>& kb, const RowFrag<D>& va, const RowFrag<D>& vb,
                                           const float (&biast)[(WB + 16) / 8][4], uint32_t q_ring, uint32_t d_ring,
                                           const float* stat_l2, const float* stat_dl, int g0, int gs, int N,
                                           int ring_mask, float c2, float gain, const LaneOff<D>& lo,
                                           const ColOff<D>& co, int tig) {
    constexpr int NT = (WB + 16) / 8;
    constexpr int kPitch = D * 2;
#pragma unroll
    for (int c = 0; c < NT / 2; ++c) {
        if (g0 + 16 * c >= N) continue;                   // warp-uniform: no query rows left in this sequence
        float ds[2][4], pv[2][4];
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
            const int nt = 2 * c + hf;
            const uint32_t rb = ((gs + 8 * nt) & ring_mask) * kPitch;
            RowFrag<D> qf, df;
            lds_frag<D>(qf, q_ring + rb, lo);
            lds_frag<D>(df, d_ring + rb, lo);
            float s[4], dp[4];
            mma_rows_z(s, ka, kb, qf);
            mma_rows_z(dp, va, vb, df);
            const float2 l2c = *reinterpret_cast<const float2*>(stat_l2 + 8 * nt + 2 * tig);
            const float2 dlc = *reinterpret_cast<const float2*>(stat_dl + 8 * nt + 2 * tig);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float p = ex2(fmaf(s[q], c2, biast[nt][q]) - ((q & 1) ? l2c.y : l2c.x));
                ds[hf][q] = p * (gain * dp[q] - ((q & 1) ? dlc.y : dlc.x));
                pv[hf][q] = p * gain;
            }
        }
        const uint32_t cb = ((gs + 16 * c) & ring_mask) * kPitch;
        ColFrag<D> cf;
        ldsm_cols<D>(cf, d_ring + cb, co);
        mma_colfrag<D>(dV, pack_bf16x2(pv[0][0], pv[0][1]), pack_bf16x2(pv[0][2], pv[0][3]),
                       pack_bf16x2(pv[1][0], pv[1][1]), pack_bf16x2(pv[1][2], pv[1][3]), cf);
        ldsm_cols<D>(cf, q_ring + cb, co);
        mma_colfrag<D>(dK, pack_bf16x2(ds[0][0], ds[0][1]), pack_bf16x2(ds[0][2], ds[0][3]),
                       pack_bf16x2(ds[1][0], ds[1][1]), pack_bf16x2(ds[1][2], ds[1][3]), cf);
    }
}

// ------------------------------------------------------------------------------ dK/dV: consumer warps
template <int D, int WB>
__device__ __forceinline__ void dkdv_consumer_loop(const BwdArgs& a, const Plan& plan, const Taps& t, uint32_t smem_base,
                                                   uint8_t* gen_base, const Smem<D, 2>& lay, const Bars& bars,
                                                   volatile int* abort_flag, int g_begin, int g_end) {
    constexpr int NT = (WB + 16) / 8;
    constexpr int kPitch = Smem<D, 2>::kPitch;
    constexpr int kTile = Smem<D, 2>::kTile;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tig = lane & 3;
    const bool owner = tig == (g >> 1);
    const LaneOff<D> lo = lane_offsets<D>(g, tig);
    const ColOff<D> co = col_offsets<D>(lane);
    const int N = a.N, H = a.H, W = plan.consumers;
    const int nrb = plan.nrb, look = plan.look, ring_mask = nrb * kBlockRows - 1;
    const int d_lo = t.d_lo, d_hi = t.d_lo + t.n_dense - 1, nd = t.n_dense, ns = t.n_sparse, n_win = plan.n_win;
    const float c2 = a.scale * kLog2e;
    const uint32_t q_ring = smem_base + lay.ring0, d_ring = smem_base + lay.ring1;
    const uint32_t maskp = (uint32_t)ring_mask * kPitch | (kPitch - 1);
    const int n_tiles = (g_end - g_begin) * kTilesPerBlock;
    float* stat_l2 = reinterpret_cast<float*>(gen_base + lay.extra) + warp * 2 * kStatRows;
    float* stat_dl = stat_l2 + kStatRows;

    float biast[NT][4];
    int bias_h = -1;
    float gain = 1.f;
    const int tap_delta = lane < ns ? t.sparse[lane < ns ? lane : 0] : 0x3fffffff;
    const uint32_t tap_deltap = (uint32_t)tap_delta * kPitch;
    float tap_pb2 = 0.f;
    int waited_r = 0;

#pragma unroll 1
    for (int T = warp; T < n_tiles; T += W) {
        const int j = T >> 3, tib = T & 7;
        const int G = g_begin + j;
        const int bh = G / plan.blocks_per_seq, sb = G - bh * plan.blocks_per_seq;
        const int h = bh % H;
        const int g0 = sb * kBlockRows + 16 * tib, gs = j * kBlockRows + 16 * tib;   // own block = oldest ring block
        const bool active = g0 < N;
        const int row_lo = g0 + g, row_hi = row_lo + 8;
        const float* lse = a.lse + (size_t)bh * N;
        const float* dl = a.delta + (size_t)bh * N;

        if (h != bias_h) {
            bias_h = h;
            gain = a.head_gain ? __ldg(a.head_gain + h) : 1.f;
            tap_pb2 = lane < ns ? __ldg(a.pos_bias + (nd + lane) * H + h) * kLog2e : 0.f;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int delta = 8 * nt + 2 * tig + (q & 1) - (g + 8 * (q >> 1));      // query column - key row
                    biast[nt][q] = (delta >= d_lo && delta <= d_hi) ? __ldg(a.pos_bias + (delta - d_lo) * H + h) * kLog2e : kNeg;
                }
        }
#pragma unroll 1
        for (; waited_r <= j + look; ++waited_r)
            mbar_wait(bars.win_full(waited_r & (nrb - 1)), (waited_r / nrb) & 1, abort_flag, 0x222);
        // ---- K and V fragments of the tile
        RowFrag<D> ka, kb, va, vb;
        {
            const int os = j % plan.n_own_stages;
            mbar_wait(bars.own_full(os), (j / plan.n_own_stages) & 1, abort_flag, 0x221);
            const uint32_t kt = smem_base + lay.own + os * 2 * kTile + tib * 16 * kPitch;
            lds_frag<D>(ka, kt, lo);
            lds_frag<D>(kb, kt + 8 * kPitch, lo);
            lds_frag<D>(va, kt + kTile, lo);
            lds_frag<D>(vb, kt + kTile + 8 * kPitch, lo);
            __syncwarp();
            if (lane == 0) mbar_arrive(bars.own_empty(os));
        }
        // ---- lse / delta of the dense window's query rows into the warp's scratch
        __syncwarp();
#pragma unroll
        for (int i = lane; i < 16 + WB; i += 32) {
            const int n = g0 + i;
            const bool v = n < N;
            const float x = v ? __ldg(lse + n) : 0.f;
            stat_l2[i] = v ? (x == -INFINITY ? 0.f : x * kLog2e) : kBigL2;
            stat_dl[i] = v ? __ldg(dl + n) : 0.f;
        }
        __syncwarp();
        const int nv = __popc(__ballot_sync(0xffffffffu, lane < ns && g0 + tap_delta < N));
        float dK[D / 8][4], dV[D / 8][4];
#pragma unroll
        for (int jj = 0; jj < D / 8; ++jj) {
            dK[jj][0] = dK[jj][1] = dK[jj][2] = dK[jj][3] = 0.f;
            dV[jj][0] = dV[jj][1] = dV[jj][2] = dV[jj][3] = 0.f;
        }
        // ---- far taps
#pragma unroll 1
        for (int f = 0; f < plan.n_far; ++f) {
            const int seq = j * plan.n_far + f;
            const int fs = seq % plan.n_far_stages;
            mbar_wait(bars.far_full(fs), (seq / plan.n_far_stages) & 1, abort_flag, 0x223);
            if (active && n_win + f < nv) {
                const int delta = __shfl_sync(0xffffffffu, tap_delta, n_win + f);
                const int n = g0 + delta + (lane & 15);
                const bool v = n < N;
                float sv;
                if (lane < 16) { const float x = v ? __ldg(lse + n) : 0.f; sv = v ? (x == -INFINITY ? 0.f : x * kLog2e) : kBigL2; }
                else sv = v ? __ldg(dl + n) : 0.f;
                const uint32_t fb = smem_base + lay.far + fs * 2 * kTile + tib * 16 * kPitch;
                const uint32_t srcQ[1] = {fb}, srcD[1] = {fb + kTile};
                const bool ok[1] = {true};
                const float pb2[1] = {__shfl_sync(0xffffffffu, tap_pb2, n_win + f)};
                const float stat[1] = {sv};
                dkdv_sparse_group<D, 1>(dK, dV, ka, kb, va, vb, srcQ, srcD, ok, pb2, stat, c2, gain, lo, co, owner, g);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bars.far_empty(fs));
        }
        if (active) {
            dkdv_dense<D, WB>(dK, dV, ka, kb, va, vb, biast, q_ring, d_ring, stat_l2, stat_dl, g0, gs, N, ring_mask, c2, gain, lo, co, tig);
            const int nvw = nv < n_win ? nv : n_win;
            const uint32_t gsp = (uint32_t)gs * kPitch;
#pragma unroll 1
            for (int t0 = 0; t0 < nvw; t0 += kGroupBwd) {
                uint32_t srcQ[kGroupBwd], srcD[kGroupBwd];
                bool ok[kGroupBwd];
                float pb2[kGroupBwd], stat[kGroupBwd];
#pragma unroll
                for (int i = 0; i < kGroupBwd; ++i) {
                    ok[i] = t0 + i < nvw;
                    const int ti = ok[i] ? t0 + i : nvw - 1;
                    const uint32_t off = (gsp + __shfl_sync(0xffffffffu, tap_deltap, ti)) & maskp;
                    srcQ[i] = q_ring + off; srcD[i] = d_ring + off;
                    pb2[i] = __shfl_sync(0xffffffffu, tap_pb2, ti);
                    const int n = g0 + __shfl_sync(0xffffffffu, tap_delta, ti) + (lane & 15);
                    const bool v = n < N;
                    if (lane < 16) { const float x = v ? __ldg(lse + n) : 0.f; stat[i] = v ? (x == -INFINITY ? 0.f : x * kLog2e) : kBigL2; }
                    else stat[i] = v ? __ldg(dl + n) : 0.f;
                }
                dkdv_sparse_group<D, kGroupBwd>(dK, dV, ka, kb, va, vb, srcQ, srcD, ok, pb2, stat, c2, gain, lo, co, owner, g);
            }
        }
        __syncwarp();
        if (lane == 0) {
#pragma unroll 1
            for (int b = j; b <= j + look; ++b) mbar_arrive(bars.win_empty(b & (nrb - 1)));
        }
        if (active) {
            const size_t base = (size_t)bh * N * D;
            const bool ok_lo = row_lo < N, ok_hi = row_hi < N;
            __nv_bfloat16* dkp = static_cast<__nv_bfloat16*>(a.dk) + base;
            __nv_bfloat16* dvp = static_cast<__nv_bfloat16*>(a.dv) + base;
            store_acc_std<D>(dK, dkp + (size_t)row_lo * D, dkp + (size_t)row_hi * D, ok_lo, ok_hi, a.scale, a.scale, tig);
            store_acc_std<D>(dV, dvp + (size_t)row_lo * D, dvp + (size_t)row_hi * D, ok_lo, ok_hi, 1.f, 1.f, tig);
        }
    }
}

// ------------------------------------------------------------------------------ kernels
template <int D, int WB, int W>
__global__ void __launch_bounds__((W + 1) * 32, 1)
bwd_dq_tma_kernel(const BwdArgs a, const BwdTmaExtra x, const Taps t, const Plan plan,
                  const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                  const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t smem_base = (raw + 1023u) & ~1023u;
    uint8_t* gen_base = smem_raw + (smem_base - raw);
    const Smem<D, 2> lay(plan);
    const Bars bars{smem_base + (uint32_t)lay.bars};
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + lay.misc);
    if (threadIdx.x == 0) init_barriers(plan, bars, abort_flag);
    __syncthreads();
    const int g_begin = blockIdx.x * plan.blocks_per_cta;
    const int g_end = min(plan.total_blocks, g_begin + plan.blocks_per_cta);
    if (g_begin >= g_end) return;
    if ((threadIdx.x >> 5) == W) {
        if ((threadIdx.x & 31) == 0) {
            prefetch_tensormap(&tm_q); prefetch_tensormap(&tm_do); prefetch_tensormap(&tm_k); prefetch_tensormap(&tm_v);
            const CUtensorMap* const own[2] = {&tm_q, &tm_do};
            const CUtensorMap* const ring[2] = {&tm_k, &tm_v};
            producer_loop<D, 2, false>(plan, t, own, ring, smem_base, lay, bars, abort_flag, g_begin, g_end);
        }
    } else {
        dq_consumer_loop<D, WB>(a, x, plan, t, smem_base, gen_base, lay, bars, abort_flag, g_begin, g_end);
    }
}

template <int D, int WB, int W>
__global__ void __launch_bounds__((W + 1) * 32, 1)
bwd_dkdv_tma_kernel(const BwdArgs a, const Taps t, const Plan plan,
                    const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                    const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t smem_base = (raw + 1023u) & ~1023u;
    uint8_t* gen_base = smem_raw + (smem_base - raw);
    const Smem<D, 2> lay(plan);
    const Bars bars{smem_base + (uint32_t)lay.bars};
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + lay.misc);
    if (threadIdx.x == 0) init_barriers(plan, bars, abort_flag);
    __syncthreads();
    const int g_begin = blockIdx.x * plan.blocks_per_cta;
    const int g_end = min(plan.total_blocks, g_begin + plan.blocks_per_cta);
    if (g_begin >= g_end) return;
    if ((threadIdx.x >> 5) == W) {
        if ((threadIdx.x & 31) == 0) {
            prefetch_tensormap(&tm_q); prefetch_tensormap(&tm_do); prefetch_tensormap(&tm_k); prefetch_tensormap(&tm_v);
            const CUtensorMap* const own[2] = {&tm_k, &tm_v};
            const CUtensorMap* const ring[2] = {&tm_q, &tm_do};
            producer_loop<D, 2, true>(plan, t, own, ring, smem_base, lay, bars, abort_flag, g_begin, g_end);
        }
    } else {
        dkdv_consumer_loop<D, WB>(a, plan, t, smem_base, gen_base, lay, bars, abort_flag, g_begin, g_end);
    }
}

// Second stage of the parameter gradients: partials are indexed by (slot, warp); slot_bh names
// the sequence a slot belongs to.  One block per output element, fixed summation order.
constexpr int kSlotReduceThreads = 128;
__global__ void __launch_bounds__(kSlotReduceThreads)
bwd_reduce_slots_kernel(const BwdArgs a, const BwdTmaExtra x, const int J, const int W) {
    __shared__ float red[kSlotReduceThreads];
    const int idx = blockIdx.x;
    const bool is_gain = idx >= J * a.H;
    const int j = is_gain ? 0 : idx / a.H;
    const int h = is_gain ? idx - J * a.H : idx - j * a.H;
    float s = 0.f;
    for (int i = threadIdx.x; i < x.n_slots * W; i += kSlotReduceThreads) {
        const int bhv = x.slot_bh[i / W];
        if (bhv >= 0 && bhv % a.H == h) s += is_gain ? x.dg_part[i] : x.dpb_part[(size_t)i * J + j];
    }
    red[threadIdx.x] = s;
    __syncthreads();
    for (int o = kSlotReduceThreads / 2; o > 0; o >>= 1) {
        if (threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        if (!is_gain) a.dpos_bias[idx] = red[0];
        else if (a.dhead_gain) a.dhead_gain[h] = red[0];
    }
}

}  // namespace
namespace {
using namespace pipe;

constexpr int kMaxGrid = 512;

int env_int(const char* name, int dflt) {
    const char* v = getenv(name);
    return v ? atoi(v) : dflt;
}

// Shared-memory plan of one backward kernel; false if the configuration does not fit.
template <int D>
bool make_plan(Plan& p, const Taps& t, int B, int H, int N, int sms, int W, int extra_bytes, int look_override) {
    p.consumers = W;
    p.nrb = D == 32 ? 8 : 4;
    p.look = look_override > 0 ? look_override : (D == 32 ? p.nrb - 3 : p.nrb - 2);
    if (p.look > p.nrb - 2) p.look = p.nrb - 2;
    if (p.look < 1) p.look = 1;
    p.extra_bytes = extra_bytes;
    p.n_win = 0;
    while (p.n_win < t.n_sparse && t.sparse[p.n_win] <= p.look * kBlockRows) ++p.n_win;
    p.n_far = t.n_sparse - p.n_win;
    p.n_own_stages = 1;
    p.n_far_stages = p.n_far > 0 ? 1 : 0;
    if (Smem<D, 2>(p).total + 1024 > kSmemLimit) return false;
    // grow own stages to 2, then far stages, while shared memory allows
    p.n_own_stages = 2;
    if (Smem<D, 2>(p).total + 1024 > kSmemLimit) p.n_own_stages = 1;
    while (p.n_far > 0 && p.n_far_stages < kMaxFarStages && p.n_far_stages < 2 * p.n_far) {
        ++p.n_far_stages;
        if (Smem<D, 2>(p).total + 1024 > kSmemLimit) { --p.n_far_stages; break; }
    }
    p.blocks_per_seq = (N + kBlockRows - 1) / kBlockRows;
    p.total_blocks = B * H * p.blocks_per_seq;
    int grid = p.total_blocks < sms ? p.total_blocks : sms;
    if (grid > kMaxGrid) grid = kMaxGrid;
    p.blocks_per_cta = (p.total_blocks + grid - 1) / grid;
    return true;
}

template <int D, int WB, int W>
cudaError_t bwd_launch_tma(BwdArgs a, const Taps& t, cudaStream_t stream, int stages) {
    int dev = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return e;
    const int BH = a.B * a.H, J = t.J;
    Plan pq, pk;
    if (!make_plan<D>(pq, t, a.B, a.H, a.N, sms, W, W * kWarpScratchFloats * 4, env_int("DSQG_BWD_LOOK", 0)) ||
        !make_plan<D>(pk, t, a.B, a.H, a.N, sms, W, W * 2 * kStatRows * 4, env_int("DSQG_BWD_LOOK", 0)))
        return cudaErrorInvalidConfiguration;
    const int grid = (pq.total_blocks + pq.blocks_per_cta - 1) / pq.blocks_per_cta;
    // scratch: delta | slot_bh | dhead_gain partials | dpos_bias partials
    BwdTmaExtra x;
    x.n_slots = grid + BH;
    char* p = static_cast<char*>(a.scratch);
    a.delta = reinterpret_cast<float*>(p);        p += round256((size_t)BH * a.N * 4);
    x.slot_bh = reinterpret_cast<int*>(p);        p += round256((size_t)x.n_slots * 4);
    x.dg_part = reinterpret_cast<float*>(p);      p += round256((size_t)x.n_slots * W * 4);
    x.dpb_part = reinterpret_cast<float*>(p);     p += round256((size_t)x.n_slots * W * J * 4);
    if ((size_t)(p - static_cast<char*>(a.scratch)) > a.scratch_bytes) return cudaErrorInvalidValue;

    CUtensorMap mq, mk, mv, md;
    if (!make_row_map(&mq, a.q, BH, a.N, D) || !make_row_map(&mk, a.k, BH, a.N, D) ||
        !make_row_map(&mv, a.v, BH, a.N, D) || !make_row_map(&md, a.dout, BH, a.N, D))
        return cudaErrorInvalidValue;
    if (stages & DSQG_BWD_STAGE_DQ) {
        const int smem = Smem<D, 2>(pq).total + 1024;
        if ((e = cudaMemsetAsync(x.slot_bh, 0xff, (size_t)x.n_slots * 4, stream)) != cudaSuccess) return e;
        if ((e = cudaFuncSetAttribute(bwd_dq_tma_kernel<D, WB, W>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)) != cudaSuccess) return e;
        bwd_dq_tma_kernel<D, WB, W><<<grid, (W + 1) * 32, smem, stream>>>(a, x, t, pq, mq, md, mk, mv);
        if ((e = cudaGetLastError()) != cudaSuccess) return e;
    }
    if (stages & DSQG_BWD_STAGE_DKDV) {
        const int smem = Smem<D, 2>(pk).total + 1024;
        if ((e = cudaFuncSetAttribute(bwd_dkdv_tma_kernel<D, WB, W>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)) != cudaSuccess) return e;
        bwd_dkdv_tma_kernel<D, WB, W><<<grid, (W + 1) * 32, smem, stream>>>(a, t, pk, mk, mv, mq, md);
        if ((e = cudaGetLastError()) != cudaSuccess) return e;
    }
    if (stages & DSQG_BWD_STAGE_REDUCE) {
        bwd_reduce_slots_kernel<<<J * a.H + a.H, kSlotReduceThreads, 0, stream>>>(a, x, J, W);
        e = cudaGetLastError();
    }
    return e;
}

template <int D, int WB>
cudaError_t bwd_launch_tma_w(const BwdArgs& a, const Taps& t, cudaStream_t s, int stages) {
    const int W = env_int("DSQG_BWD_WARPS", 11);
    if (W == 8) return bwd_launch_tma<D, WB, 8>(a, t, s, stages);
    if (W == 15) return bwd_launch_tma<D, WB, 15>(a, t, s, stages);
    return bwd_launch_tma<D, WB, 11>(a, t, s, stages);
}
}  // namespace

size_t bwd_scratch_need_tma(int J, int B, int H, int N) {
    const size_t slots = (size_t)kMaxGrid + (size_t)B * H;
    return round256((size_t)B * H * N * 4) + round256(slots * 4) + round256(slots * 16 * 4) + round256(slots * 16 * J * 4);
}

bool tma_bwd_supported(int dtype, int D, int N, const Taps& t, bool has_scale_embed) {
    if (dtype != DSQG_DTYPE_BF16 || D != 32 || has_scale_embed) return false;     // D = 64 uses the non-TMA tensor-core kernels
    if (t.n_sparse > kMaxSparseTma || band_width(t) == 0 || N < 1) return false;
    for (int i = 0; i < t.n_sparse; ++i)
        if (t.sparse[i] % 16 != 0) return false;
    return encode_fn() != nullptr;
}

cudaError_t launch_bwd_tma(const BwdArgs& a, const Taps& t, cudaStream_t s, int stages) {
    const int wb = band_width(t);
    if (a.D == 32) {
        if (wb == 32) return bwd_launch_tma_w<32, 32>(a, t, s, stages);
        if (wb == 48) return bwd_launch_tma_w<32, 48>(a, t, s, stages);
        return bwd_launch_tma_w<32, 64>(a, t, s, stages);
    }
    if (wb == 32) return bwd_launch_tma_w<64, 32>(a, t, s, stages);
    if (wb == 48) return bwd_launch_tma_w<64, 48>(a, t, s, stages);
    return bwd_launch_tma_w<64, 64>(a, t, s, stages);
}

cudaError_t read_device_error_bwd_tma(int* value, bool reset) {
    cudaError_t e = cudaMemcpyFromSymbol(value, g_device_error, sizeof(int));
    if (e == cudaSuccess && reset && *value != 0) {
        const int zero = 0;
        e = cudaMemcpyToSymbol(g_device_error, &zero, sizeof(int));
    }
    return e;
}
}  // namespace dsqg
