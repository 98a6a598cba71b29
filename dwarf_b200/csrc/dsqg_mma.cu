// Tensor-core DSQG kernels (bf16 storage, fp32 accumulate) for D in {32, 64} (dense windows up
// to 64 wide) and D in {96, 128} (dense windows up to 32 wide).
//
// One warp owns 16 consecutive rows of one (batch, head) sequence.  The dense window is a
// banded GEMM: the 16 query rows against the WB+16 key rows [g0-WB, g0+16) with
// mma.sync.m16n8k16; out-of-band entries are masked.  Every sparse tap pairs row n with row
// n-delta, i.e. it is the diagonal of a 16x16 tile: its scores come from two m16n8 MMAs per
// k-step, of which the thread with tig == g>>1 keeps the diagonal entries; the products that
// follow (p.v, ds.k, ds.q, p.dO) scale row g of a tile the thread already holds as a row
// fragment, so they are plain fp32 FMAs on the thread's accumulators (no transposes, no tensor
// core: measured faster than a diagonal A fragment).  The math is that of the DWARF reference kernels
// (kernels/dsqg_attention_v3.py:60-163 forward, :198-275 dQ, :282-352 dK/dV), with the per-head
// output gain of train/train_2048_condU.py:187 fused in.  See dsqg_mma.cuh for the fragment
// conventions.  scale_embed (D <= 64): q.scale_embed[j] is computed per 16-row tile with
// split-bf16 MMAs into a shared-memory tile that also carries the position bias and replaces
// the start-value table; the dQ kernel adds dS.scale_embed (MMA, dS from its staging tile),
// produces dscale_embed partials per 64-row tile (dS^T.Q, MMA; dse_group_kernel adds groups of
// eight tiles) and leaves the per-row tile in global memory for the dK/dV kernel.
#include "dsqg_mma.cuh"
#include <mutex>
#include <type_traits>

namespace dsqg {
namespace {

constexpr int kMaxSparse = DSQG_MAX_TAPS;   // any number of sparse taps (they are processed in a loop)
constexpr int kWarps = 4;
constexpr int kRows = 16 * kWarps; // rows per CTA

// ------------------------------------------------------------------------------ forward
// Online softmax over the dense window, then over the sparse taps, with the per-element
// bookkeeping moved out of the tile loop:
//   * the band mask and the position bias of the dense window are the INITIAL VALUE of the score
//     accumulators (a per-lane table in shared memory, one 16-byte load per n-tile), so the
//     scores leave the MMAs already biased and masked (in units of 1/scale);
//   * interior tiles (all band rows inside the sequence) load with no predicates and constant
//     offsets from one pointer; a sparse tap whose 16 key rows all exist does the same;
//   * the running maximum only moves when a sparse score exceeds it by more than kSlack
//     (log2 units): p stays below 2^kSlack, which fp32 sums and bf16 probabilities absorb;
//   * lanes that do not own a diagonal entry subtract +1e30 instead of the maximum, so their
//     probability is exactly zero without a select.
// Shared-memory tables of the scale_embed variants (reference: kernels/dsqg_attention_v3.py:112-118,
// s_j += q.scale_embed[j] / sqrt(D)).  se_hi + se_lo are the bf16 halves of scale_embed (their sum
// carries 16 mantissa bits), pbs[j] = pos_bias[j,h] / scale, and qs (one tile per warp,
// [16][pitch] floats + one dump word holding the mask value) receives q.scale_embed[j] + pbs[j]
// for the warp's rows.  off[] maps dense-window accumulator slots to tile entries (or the dump).
struct SeTables {
    const __nv_bfloat16* se_hi; const __nv_bfloat16* se_lo;
    const float* pbs; const int4* off; float* qs;
    int Jp, pitch, nd;
};

// qs[row][j] = q[row].scale_embed[j] + pbs[j] for the 16 rows held as A fragments qa (rows g) / qb (rows g+8)
// GL: the tables (se_hi, se_lo, pbs) are in global memory (read-only path) instead of shared memory
// rows_lo / rows_hi (optional): global-memory rows (Jp floats each) that receive a copy of rows g / g+8
template <int D, bool GL>
__device__ __forceinline__ void build_qs_tile(const SeTables& se, const RowFrag<D>& qa, const RowFrag<D>& qb, int g, int tig,
                                              float* rows_lo = nullptr, float* rows_hi = nullptr) {
#pragma unroll 2
    for (int m = 0; m < se.Jp / 8; ++m) {
        const float2* pbp = reinterpret_cast<const float2*>(se.pbs + 8 * m + 2 * tig);
        const float2 pb2 = GL ? __ldg(pbp) : *pbp;
        float c[4] = {pb2.x, pb2.y, pb2.x, pb2.y};
        RowFrag<D> sf;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const uint4* src = reinterpret_cast<const uint4*>((half ? se.se_lo : se.se_hi) + (8 * m + g) * D + 8 * tig);
#pragma unroll
            for (int cc = 0; cc < D / 32; ++cc) {
                const uint4 u = GL ? __ldg(src + 4 * cc) : src[4 * cc];
                sf.r[4 * cc + 0] = u.x; sf.r[4 * cc + 1] = u.y; sf.r[4 * cc + 2] = u.z; sf.r[4 * cc + 3] = u.w;
            }
            mma_rows(c, qa, qb, sf);
        }
        *reinterpret_cast<float2*>(se.qs + g * se.pitch + 8 * m + 2 * tig) = make_float2(c[0], c[1]);
        *reinterpret_cast<float2*>(se.qs + (g + 8) * se.pitch + 8 * m + 2 * tig) = make_float2(c[2], c[3]);
        if (rows_lo) *reinterpret_cast<float2*>(rows_lo + 8 * m + 2 * tig) = make_float2(c[0], c[1]);
        if (rows_hi) *reinterpret_cast<float2*>(rows_hi + 8 * m + 2 * tig) = make_float2(c[2], c[3]);
    }
    __syncwarp();
}

template <int D, int WB, bool INTERIOR, int kTapGroup, bool SE, bool ST>
__device__ __forceinline__ void fwd_tile(const FwdArgs& a, const float4* init_s, const int2* tap_s, int ns,
                                         int bh, int h, int g0, const Lane& L, const SeTables& se) {
    constexpr int NT = (WB + 16) / 8;
    const int N = a.N, g = L.g, tig = L.tig;
    const int row_lo = g0 + g, row_hi = row_lo + 8;
    const bool ok_lo = INTERIOR || row_lo < N, ok_hi = INTERIOR || row_hi < N;
    const ptrdiff_t RS = ST ? (ptrdiff_t)a.in_sn : D, OS = ST ? (ptrdiff_t)a.out_sn : D;   // row strides of q/k/v and of out
    const size_t base = ST ? (size_t)(bh / a.H) * a.in_sb + (size_t)h * a.in_sh : (size_t)bh * N * D;
    const size_t obase = ST ? (size_t)(bh / a.H) * a.out_sb + (size_t)h * a.out_sh : base;
    const __nv_bfloat16* qp = static_cast<const __nv_bfloat16*>(a.q) + base;
    // per-thread pointers to this thread's chunk of row row_lo of K and V
    const __nv_bfloat16* kl = static_cast<const __nv_bfloat16*>(a.k) + base + (ptrdiff_t)row_lo * RS + 8 * tig;
    const __nv_bfloat16* vl = static_cast<const __nv_bfloat16*>(a.v) + base + (ptrdiff_t)row_lo * RS + 8 * tig;
    const float c2 = a.scale * kLog2e;
    const int kb0 = g0 - WB;

    RowFrag<D> qa, qb;
    load_row(qa, qp + (size_t)row_lo * RS, tig, ok_lo);
    load_row(qb, qp + (size_t)row_hi * RS, tig, ok_hi);
    if constexpr (SE) build_qs_tile<D, false>(se, qa, qb, g, tig);

    // ---- dense window: key row of n-tile nt for this thread is kb0 + 8 nt + g = row_lo - WB + 8 nt
    float S[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        if constexpr (SE) {
            const int4 qo = se.off[nt * 32 + L.lane];
            S[nt][0] = se.qs[qo.x]; S[nt][1] = se.qs[qo.y]; S[nt][2] = se.qs[qo.z]; S[nt][3] = se.qs[qo.w];
        } else {
            const float4 ini = init_s[nt * 32 + L.lane];
            S[nt][0] = ini.x; S[nt][1] = ini.y; S[nt][2] = ini.z; S[nt][3] = ini.w;
        }
        RowFrag<D> kf;
        if (INTERIOR) {
            load_row_at(kf, kl + (8 * nt - WB) * RS);
        } else {
            const int kr = kb0 + 8 * nt + g;
            load_row(kf, kl + (ptrdiff_t)(8 * nt - WB) * RS - 8 * tig, tig, kr >= 0 && kr < N);
        }
        mma_rows(S[nt], qa, qb, kf);
    }
    if (!INTERIOR && kb0 < 0) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int r = 0; r < 4; ++r)
                if (kb0 + 8 * nt + 2 * tig + (r & 1) < 0) S[nt][r] = kNeg;
    }
    float m_lo = kMinM, m_hi = kMinM;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        m_lo = fmaxf(m_lo, fmaxf(S[nt][0], S[nt][1]));
        m_hi = fmaxf(m_hi, fmaxf(S[nt][2], S[nt][3]));
    }
    m_lo = quad_max(m_lo) * c2; m_hi = quad_max(m_hi) * c2;          // log2 units from here on
    float l_lo = 0.f, l_hi = 0.f;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        S[nt][0] = ex2(fmaf(S[nt][0], c2, -m_lo)); S[nt][1] = ex2(fmaf(S[nt][1], c2, -m_lo));
        S[nt][2] = ex2(fmaf(S[nt][2], c2, -m_hi)); S[nt][3] = ex2(fmaf(S[nt][3], c2, -m_hi));
        l_lo += S[nt][0] + S[nt][1]; l_hi += S[nt][2] + S[nt][3];
    }
    float O[D / 8][4];
#pragma unroll
    for (int c = 0; c < NT / 2; ++c) {
        RowFrag<D> vf0, vf1, vt0, vt1;
        if (INTERIOR) {
            load_row_at(vf0, vl + (16 * c - WB) * RS);
            load_row_at(vf1, vl + (16 * c + 8 - WB) * RS);
        } else {
            const int kr = kb0 + 16 * c + g;
            load_row(vf0, vl + (ptrdiff_t)(16 * c - WB) * RS - 8 * tig, tig, kr >= 0 && kr < N);
            load_row(vf1, vl + (ptrdiff_t)(16 * c + 8 - WB) * RS - 8 * tig, tig, kr + 8 >= 0 && kr + 8 < N);
        }
        transpose_frag(vt0, vf0); transpose_frag(vt1, vf1);
        const uint32_t a0 = pack_bf16x2(S[2 * c][0], S[2 * c][1]), a1 = pack_bf16x2(S[2 * c][2], S[2 * c][3]);
        const uint32_t a2 = pack_bf16x2(S[2 * c + 1][0], S[2 * c + 1][1]), a3 = pack_bf16x2(S[2 * c + 1][2], S[2 * c + 1][3]);
        if (c == 0) {
#pragma unroll
            for (int j = 0; j < D / 8; ++j) mma16816_z(O[j], a0, a1, a2, a3, vt0.r[j], vt1.r[j]);
        } else {
            mma_cols<D>(O, a0, a1, a2, a3, vt0, vt1);
        }
    }
    // ---- sparse taps
    float ms_lo = L.owner ? m_lo : 1.0e30f, ms_hi = L.owner ? m_hi : 1.0e30f;   // what this lane subtracts
    // Folds G taps whose scores x0[i] (row g) and x1[i] (row g+8) are known into the running softmax.
    auto fold = [&](auto GC, const float (&x0)[decltype(GC)::value], const float (&x1)[decltype(GC)::value],
                    const RowFrag<D> (&vf0)[decltype(GC)::value], const RowFrag<D> (&vf1)[decltype(GC)::value]) {
        constexpr int G = decltype(GC)::value;
        float xm0 = x0[0], xm1 = x1[0];
#pragma unroll
        for (int i = 1; i < G; ++i) { xm0 = fmaxf(xm0, x0[i]); xm1 = fmaxf(xm1, x1[i]); }
        if (__any_sync(0xffffffffu, xm0 > ms_lo + kSlack || xm1 > ms_hi + kSlack)) {
            const float mn_lo = fmaxf(m_lo, __shfl_sync(0xffffffffu, xm0, L.owner_lane));
            const float mn_hi = fmaxf(m_hi, __shfl_sync(0xffffffffu, xm1, L.owner_lane));
            const float al_lo = ex2(m_lo - mn_lo), al_hi = ex2(m_hi - mn_hi);
            m_lo = mn_lo; m_hi = mn_hi;
            ms_lo = L.owner ? m_lo : 1.0e30f; ms_hi = L.owner ? m_hi : 1.0e30f;
            l_lo *= al_lo; l_hi *= al_hi;
#pragma unroll
            for (int j = 0; j < D / 8; ++j) { O[j][0] *= al_lo; O[j][1] *= al_lo; O[j][2] *= al_hi; O[j][3] *= al_hi; }
        }
#pragma unroll
        for (int i = 0; i < G; ++i) {
            const float p0 = ex2(x0[i] - ms_lo), p1 = ex2(x1[i] - ms_hi);   // exactly 0 on lanes that own no diagonal entry
            l_lo += p0; l_hi += p1;
            // P is diagonal: row g only needs its own value row, which this thread holds for the
            // same elements d as its accumulators
            diag_fma<D>(O, __shfl_sync(0xffffffffu, p0, L.owner_lane), __shfl_sync(0xffffffffu, p1, L.owner_lane),
                        vf0[i], vf1[i]);
        }
    };
    // G consecutive taps whose 16 key rows all exist: no predicates, loads of all G taps in flight together
    auto full_taps = [&](auto GC, int si) {
        constexpr int G = decltype(GC)::value;
        RowFrag<D> kf0[G], kf1[G], vf0[G], vf1[G];
        float pbv[G];
#pragma unroll
        for (int i = 0; i < G; ++i) {
            const int2 tp = tap_s[si + i];
            const ptrdiff_t off = (ptrdiff_t)tp.x * RS;
            pbv[i] = __int_as_float(tp.y);
            load_row_at(kf0[i], kl - off);
            load_row_at(kf1[i], kl - off + 8 * RS);
            load_row_at(vf0[i], vl - off);
            load_row_at(vf1[i], vl - off + 8 * RS);
        }
        float x0[G], x1[G];
#pragma unroll
        for (int i = 0; i < G; ++i) {
            float s0[4], s1[4];
            mma_rows_z(s0, qa, qb, kf0[i]);
            mma_rows_z(s1, qa, qb, kf1[i]);
            const float d0 = (g & 1) ? s0[1] : s0[0], d1 = (g & 1) ? s1[3] : s1[2];
            if constexpr (SE) {
                x0[i] = (d0 + se.qs[g * se.pitch + se.nd + si + i]) * c2;
                x1[i] = (d1 + se.qs[(g + 8) * se.pitch + se.nd + si + i]) * c2;
            } else {
                x0[i] = fmaf(d0, c2, pbv[i]);
                x1[i] = fmaf(d1, c2, pbv[i]);
            }
        }
        fold(GC, x0, x1, vf0, vf1);
    };
    // A tile that reaches past row N-1 may pair its missing rows with key rows that do not exist
    // either (past the end of the sequence, for the last (b,h) past the end of the tensor).  Their
    // scores land in lanes that own no diagonal entry and are meant to contribute exp(x - 1e30) = 0;
    // a NaN or Inf bit pattern there would make that NaN, so boundary tiles take the predicated path,
    // which reads zeros for those rows.
    // Only interior tiles load taps unpredicated (boundary tiles are the first WB rows, which the
    // usual tap sets do not reach from, and the last partial tile).
    int si = 0;
    if constexpr (INTERIOR)
        for (; si + kTapGroup <= ns && g0 >= tap_s[si + kTapGroup - 1].x; si += kTapGroup)
            full_taps(std::integral_constant<int, kTapGroup>(), si);
#pragma unroll 1
    for (; si < ns; ++si) {
        const int delta = tap_s[si].x;
        if (g0 + 15 < delta) break;                       // taps ascend: no row of the tile reaches back that far
        if (INTERIOR && g0 >= delta) {
            full_taps(std::integral_constant<int, 1>(), si);
        } else {                                          // some key rows lie outside the sequence
            const float pbv = __int_as_float(tap_s[si].y);
            const int kr0 = row_lo - delta, kr1 = row_hi - delta;
            const bool v0 = kr0 >= 0 && kr0 < N, v1 = kr1 >= 0 && kr1 < N;
            const ptrdiff_t off = (ptrdiff_t)delta * RS + 8 * tig;
            RowFrag<D> kf0, kf1, vf0[1], vf1[1];
            load_row(kf0, kl - off, tig, v0);
            load_row(kf1, kl - off + 8 * RS, tig, v1);
            load_row(vf0[0], vl - off, tig, v0);
            load_row(vf1[0], vl - off + 8 * RS, tig, v1);
            float s0[4], s1[4];
            mma_rows_z(s0, qa, qb, kf0);
            mma_rows_z(s1, qa, qb, kf1);
            const float d0 = (g & 1) ? s0[1] : s0[0], d1 = (g & 1) ? s1[3] : s1[2];
            const float y0 = SE ? (d0 + se.qs[g * se.pitch + se.nd + si]) * c2 : fmaf(d0, c2, pbv);
            const float y1 = SE ? (d1 + se.qs[(g + 8) * se.pitch + se.nd + si]) * c2 : fmaf(d1, c2, pbv);
            const float x0[1] = {v0 ? y0 : kNeg};
            const float x1[1] = {v1 ? y1 : kNeg};
            fold(std::integral_constant<int, 1>(), x0, x1, vf0, vf1);
        }
    }
    l_lo = quad_sum(l_lo); l_hi = quad_sum(l_hi);
    const float gain = a.head_gain ? a.head_gain[h] : 1.f;
    __nv_bfloat16* op = static_cast<__nv_bfloat16*>(a.out) + obase;
    const float sc_lo = l_lo > 0.f ? __fdividef(gain, l_lo) : 0.f, sc_hi = l_hi > 0.f ? __fdividef(gain, l_hi) : 0.f;
    if (ST && a.gate) {
        const __nv_bfloat16* gp = static_cast<const __nv_bfloat16*>(a.gate) + obase;
        store_acc_rows_gated<D>(O, op + (size_t)row_lo * OS, op + (size_t)row_hi * OS, gp + (size_t)row_lo * OS,
                                gp + (size_t)row_hi * OS, ok_lo, ok_hi, sc_lo, sc_hi, tig);
    } else {
        store_acc_rows<D>(O, op + (size_t)row_lo * OS, op + (size_t)row_hi * OS, ok_lo, ok_hi, sc_lo, sc_hi, tig);
    }
    if (tig == 0) {
        if (ok_lo) a.lse[(size_t)bh * N + row_lo] = l_lo > 0.f ? (m_lo + __log2f(l_lo)) * kLn2 : -INFINITY;
        if (ok_hi) a.lse[(size_t)bh * N + row_hi] = l_hi > 0.f ? (m_hi + __log2f(l_hi)) * kLn2 : -INFINITY;
    }
}

// Tuning per head dimension (measured on B200): warps per CTA, sparse taps folded together,
// resident CTAs per SM the register budget is set for.
template <int D> struct FwdTune {
    static constexpr int warps = 4, group = D <= 64 ? 2 : 1, ctas = D == 32 ? 5 : (D == 64 ? 4 : (D == 96 ? 3 : 2));
    static constexpr int group_se = D <= 64 ? 2 : 1, ctas_se = D == 32 ? 5 : 4;       // with scale_embed
};

// Fills the shared tables of the scale_embed variants (all threads of the CTA; the caller syncs).
// smem layout: se_hi [Jp][D] bf16 | se_lo [Jp][D] bf16 | pbs [Jp] f32 | off [NT*32] int4 | qs [warps][16*pitch+4] f32
template <int D, int WB, int W>
__device__ __forceinline__ SeTables fill_se_tables(unsigned char* smem, const float* scale_embed, const float* pos_bias,
                                                   const Taps& t, int H, int h, float scale, int warp, bool transposed) {
    constexpr int NT = (WB + 16) / 8;
    const int J = t.J, Jp = (J + 7) / 8 * 8, pitch = Jp + 2;
    __nv_bfloat16* se_hi = reinterpret_cast<__nv_bfloat16*>(smem);
    __nv_bfloat16* se_lo = se_hi + Jp * D;
    float* pbs = reinterpret_cast<float*>(se_lo + Jp * D);
    int4* off = reinterpret_cast<int4*>(pbs + Jp);
    float* qs = reinterpret_cast<float*>(off + NT * 32);
    for (int e = threadIdx.x; e < Jp * D / 2; e += W * 32) {
        const int j = (2 * e) / D;
        float2 x = make_float2(0.f, 0.f);
        if (j < J) x = *reinterpret_cast<const float2*>(scale_embed + 2 * e);
        const __nv_bfloat162 hi = __floats2bfloat162_rn(x.x, x.y);
        const __nv_bfloat162 lo = __floats2bfloat162_rn(x.x - __low2float(hi), x.y - __high2float(hi));
        reinterpret_cast<__nv_bfloat162*>(se_hi)[e] = hi;
        reinterpret_cast<__nv_bfloat162*>(se_lo)[e] = lo;
    }
    const float inv_scale = 1.f / scale;
    for (int j = threadIdx.x; j < Jp; j += W * 32) pbs[j] = j < J ? pos_bias[j * H + h] * inv_scale : 0.f;
    const int d_lo = t.d_lo, d_hi = t.d_lo + t.n_dense - 1;
    for (int e = threadIdx.x; e < NT * 32; e += W * 32) {
        const int nt = e >> 5, gg = (e & 31) >> 2, tt = e & 3;
        int o[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int i = gg + 8 * (r >> 1), cc = 8 * nt + 2 * tt + (r & 1);
            // forward / dQ: rows are queries, columns keys (delta = WB + i - cc); dK/dV: rows keys, columns queries
            const int delta = transposed ? cc - i : WB + i - cc;
            const int row = transposed ? cc : i;          // tile row = query index inside the tile
            o[r] = (delta >= d_lo && delta <= d_hi) ? row * pitch + (delta - d_lo) : 16 * pitch;
        }
        off[e] = make_int4(o[0], o[1], o[2], o[3]);
    }
    float* qs_w = qs + warp * (16 * pitch + 4);
    if ((threadIdx.x & 31) == 0) qs_w[16 * pitch] = kNeg;      // the dump entry: masked
    SeTables s;
    s.se_hi = se_hi; s.se_lo = se_lo; s.pbs = pbs; s.off = off; s.qs = qs_w;
    s.Jp = Jp; s.pitch = pitch; s.nd = t.n_dense;
    return s;
}
__host__ __device__ inline size_t se_tables_bytes(int J, int D, int NT, int warps, int tile_rows) {
    const int Jp = (J + 7) / 8 * 8;
    return (size_t)2 * Jp * D * 2 + (size_t)Jp * 4 + (size_t)NT * 32 * 16 + (size_t)warps * (tile_rows * (Jp + 2) + 4) * 4;
}

// ST: q, k, v and out are addressed through the element strides in FwdArgs (rows of D contiguous
// elements; any batch / head / row strides), e.g. the un-permuted output of a fused qkv projection
// and a token-major result; with a gate tensor the epilogue multiplies by sigmoid(gate).
template <int D, int WB, bool SE, bool ST>
__global__ void __launch_bounds__(FwdTune<D>::warps * 32, SE ? FwdTune<D>::ctas_se : FwdTune<D>::ctas)
fwd_mma_kernel(const FwdArgs a, const Taps t) {
    constexpr int W = FwdTune<D>::warps, G = SE ? FwdTune<D>::group_se : FwdTune<D>::group;
    constexpr int NT = (WB + 16) / 8;
    extern __shared__ __align__(16) unsigned char se_smem[];
    __shared__ float4 init_s[SE ? 1 : NT * 32];
    __shared__ int2 tap_s[DSQG_MAX_TAPS];
    const Lane L;
    const int bh = blockIdx.y, h = bh % a.H, N = a.N;
    SeTables se = {};
    if constexpr (SE) {
        se = fill_se_tables<D, WB, W>(se_smem, a.scale_embed, a.pos_bias, t, a.H, h, a.scale, L.warp, false);
    } else {
        const int d_lo = t.d_lo, d_hi = t.d_lo + t.n_dense - 1;
        const float inv_scale = 1.f / a.scale;
        for (int e = threadIdx.x; e < NT * 32; e += W * 32) {
            const int nt = e >> 5, gg = (e & 31) >> 2, tt = e & 3;
            float v[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int delta = WB + gg + 8 * (r >> 1) - (8 * nt + 2 * tt + (r & 1));
                v[r] = (delta >= d_lo && delta <= d_hi) ? a.pos_bias[(delta - d_lo) * a.H + h] * inv_scale : kNeg;
            }
            init_s[e] = make_float4(v[0], v[1], v[2], v[3]);
        }
    }
    for (int si = threadIdx.x; si < t.n_sparse; si += W * 32)
        tap_s[si] = make_int2(t.sparse[si], __float_as_int(a.pos_bias[(t.n_dense + si) * a.H + h] * kLog2e));
    __syncthreads();
    const int g0 = blockIdx.x * (16 * W) + L.warp * 16;
    if (g0 >= N) return;
    if (g0 >= WB && g0 + 16 <= N) fwd_tile<D, WB, true, G, SE, ST>(a, init_s, tap_s, t.n_sparse, bh, h, g0, L, se);
    else fwd_tile<D, WB, false, G, SE, ST>(a, init_s, tap_s, t.n_sparse, bh, h, g0, L, se);
}

// Tuning per head dimension (measured on B200): sparse taps whose loads are issued together and
// resident CTAs per SM the register budget is set for (spills against warps in flight).
template <int D> struct BwdTune {
    static constexpr int dq_group = D == 32 ? 2 : 1, dq_ctas = D == 32 ? 4 : (D == 64 ? 4 : 2);   // D = 32: 105.4 us against 107.5 with group 1 / 5 CTAs
    static constexpr int dq_group_se = 1, dq_ctas_se = D == 32 ? 5 : 4;      // with scale_embed: more shared memory and registers per CTA
    static constexpr int dkdv_group_se = D <= 64 ? 2 : 1, dkdv_ctas_se = D == 32 ? 4 : 3;
    static constexpr int dkdv_group = D <= 64 ? 2 : 1, dkdv_ctas = D == 32 ? 4 : (D == 64 ? 3 : 2);
};
constexpr int kStagePitch = kRows + 4;      // 68: no bank conflicts on the scattered writes; the column sums rotate their start
constexpr int kStagePitchSe = kRows + 4;    // 68 with scale_embed: rows are read back as 8-byte pairs by the dS MMAs
template <bool SE> struct StagePitch { static constexpr int v = SE ? kStagePitchSe : kStagePitch; };

// Extras of the dQ kernel with scale_embed.
//   seb:  scale_embed as B fragments of dS.SE (global memory, written by se_prep_kernel)
//   q_s:  the CTA's 64 query rows as bf16 in shared memory, row pitch 2D+16 bytes (conflict-free ldmatrix)
struct SeBwd {
    const uint2* seb; unsigned char* q_s;
    int JS;            // J rounded up to 16
};

template <int D, int WB, bool INTERIOR, int G, bool SE, bool ST>
__device__ __forceinline__ float dq_tile(const BwdArgs& a, const float4* init_s, const int4* soff_s, const int2* tap_s,
                                         float* stage_w, int nd, int ns, int bh, int h, int g0, const Lane& L,
                                         const SeTables& se, const SeBwd& sb) {
    constexpr int NT = (WB + 16) / 8;
    constexpr int SP = StagePitch<SE>::v;
    const int N = a.N, g = L.g, tig = L.tig;
    const int row_lo = g0 + g, row_hi = row_lo + 8;
    const bool ok_lo = INTERIOR || row_lo < N, ok_hi = INTERIOR || row_hi < N;
    const ptrdiff_t RS = ST ? (ptrdiff_t)a.in_sn : D, OS = ST ? (ptrdiff_t)a.out_sn : D;   // row strides of q/k/v/dq and of out/dout
    const size_t base = ST ? (size_t)(bh / a.H) * a.in_sb + (size_t)h * a.in_sh : (size_t)bh * N * D;
    const size_t obase = ST ? (size_t)(bh / a.H) * a.out_sb + (size_t)h * a.out_sh : base;
    const __nv_bfloat16* qp = static_cast<const __nv_bfloat16*>(a.q) + base;
    const __nv_bfloat16* op = static_cast<const __nv_bfloat16*>(a.out) + obase;
    const __nv_bfloat16* dop = static_cast<const __nv_bfloat16*>(a.dout) + obase;
    const __nv_bfloat16* kl = static_cast<const __nv_bfloat16*>(a.k) + base + (ptrdiff_t)row_lo * RS + 8 * tig;
    const __nv_bfloat16* vl = static_cast<const __nv_bfloat16*>(a.v) + base + (ptrdiff_t)row_lo * RS + 8 * tig;
    const float c2 = a.scale * kLog2e;
    const float gain = a.head_gain ? a.head_gain[h] : 1.f;
    const int kb0 = g0 - WB;
    float dgrow = 0.f;

    RowFrag<D> qa, qb, da, db;
    load_row(qa, qp + (size_t)row_lo * RS, tig, ok_lo);
    load_row(qb, qp + (size_t)row_hi * RS, tig, ok_hi);
    load_row(da, dop + (size_t)row_lo * OS, tig, ok_lo);
    load_row(db, dop + (size_t)row_hi * OS, tig, ok_hi);
    if constexpr (SE) {
        // the tile also goes to global memory for the dK/dV kernel (rows of this warp, Jp floats each)
        float* rows = a.qs_rows + ((size_t)bh * N + row_lo) * se.Jp;
        build_qs_tile<D, true>(se, qa, qb, g, tig, ok_lo ? rows : nullptr, ok_hi ? rows + 8 * se.Jp : nullptr);
        // and the query rows to shared memory for the CTA's dscale_embed partial
        unsigned char* qrow = sb.q_s + (size_t)(L.warp * 16 + g) * (2 * D + 16) + 16 * tig;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
            *reinterpret_cast<uint4*>(qrow + 64 * c) = make_uint4(qa.r[4 * c], qa.r[4 * c + 1], qa.r[4 * c + 2], qa.r[4 * c + 3]);
            *reinterpret_cast<uint4*>(qrow + 8 * (2 * D + 16) + 64 * c) = make_uint4(qb.r[4 * c], qb.r[4 * c + 1], qb.r[4 * c + 2], qb.r[4 * c + 3]);
        }
    }
    float delta_lo, delta_hi;
    if (ST && a.delta_pre) {       // sum_d dout*out was formed by an earlier kernel (gate backward)
        delta_lo = ok_lo ? a.delta_pre[(size_t)bh * N + row_lo] : 0.f;
        delta_hi = ok_hi ? a.delta_pre[(size_t)bh * N + row_hi] : 0.f;
    } else {
        RowFrag<D> oa, ob;
        load_row(oa, op + (size_t)row_lo * OS, tig, ok_lo);
        load_row(ob, op + (size_t)row_hi * OS, tig, ok_hi);
        delta_lo = quad_sum(frag_dot(da, oa));
        delta_hi = quad_sum(frag_dot(db, ob));
    }
    float l2_lo = 0.f, l2_hi = 0.f;
    if (ok_lo) { const float x = a.lse[(size_t)bh * N + row_lo]; l2_lo = x == -INFINITY ? 0.f : x * kLog2e; }
    if (ok_hi) { const float x = a.lse[(size_t)bh * N + row_hi]; l2_hi = x == -INFINITY ? 0.f : x * kLog2e; }
    if (tig == 0) {
        float2* rs = reinterpret_cast<float2*>(a.delta) + (size_t)bh * N;
        if (ok_lo) rs[row_lo] = make_float2(l2_lo, delta_lo);
        if (ok_hi) rs[row_hi] = make_float2(l2_hi, delta_hi);
    }
    float dQ[D / 8][4];
    const int stage_base = (WB + 15 + g - 2 * tig) * SP + g;      // plain kernel: see the dense loop

    // ---- dense window
#pragma unroll
    for (int c = 0; c < NT / 2; ++c) {
        RowFrag<D> kf[2];
        float ds[2][4];
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
            const int nt = 2 * c + hf;
            float4 ini;
            if constexpr (SE) {
                const int4 qo = __ldg(se.off + nt * 32 + L.lane);      // table in global memory (se_prep_kernel)
                ini = make_float4(se.qs[qo.x], se.qs[qo.y], se.qs[qo.z], se.qs[qo.w]);
            } else {
                ini = init_s[nt * 32 + L.lane];
            }
            int so_r[4];
            if constexpr (SE) {
                const int4 so = soff_s[nt * 32 + L.lane];
                so_r[0] = so.x; so_r[1] = so.y; so_r[2] = so.z; so_r[3] = so.w;
            } else {
                // plain kernel: staging row = delta + 15 for every delta a tile element can have
                // (-15 .. WB+15), so the address is a per-lane base plus a compile-time constant and
                // entries outside the dense window (exactly zero) land in rows nobody sums
#pragma unroll
                for (int r = 0; r < 4; ++r)
                    so_r[r] = stage_base + (8 * (r >> 1) - 8 * nt - (r & 1)) * SP + 8 * (r >> 1);
            }
            float s[4] = {ini.x, ini.y, ini.z, ini.w}, dp[4];
            RowFrag<D> vf;
            if (INTERIOR) {
                load_row_at(kf[hf], kl + (8 * nt - WB) * RS);
                load_row_at(vf, vl + (8 * nt - WB) * RS);
            } else {
                const int kr = kb0 + 8 * nt + g;
                const bool kv = kr >= 0 && kr < N;
                load_row(kf[hf], kl + (ptrdiff_t)(8 * nt - WB) * RS - 8 * tig, tig, kv);
                load_row(vf, vl + (ptrdiff_t)(8 * nt - WB) * RS - 8 * tig, tig, kv);
            }
            mma_rows(s, qa, qb, kf[hf]);
            mma_rows_z(dp, da, db, vf);
            if (!INTERIOR && kb0 < 0) {
#pragma unroll
                for (int r = 0; r < 4; ++r)
                    if (kb0 + 8 * nt + 2 * tig + (r & 1) < 0) s[r] = kNeg;
            }
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const float p = ex2(fmaf(s[r], c2, r < 2 ? -l2_lo : -l2_hi));
                dgrow = fmaf(p, dp[r], dgrow);
                const float x = p * fmaf(gain, dp[r], r < 2 ? -delta_lo : -delta_hi);
                ds[hf][r] = x;
                stage_w[so_r[r]] = x;
            }
        }
        RowFrag<D> kt0, kt1;
        transpose_frag(kt0, kf[0]); transpose_frag(kt1, kf[1]);
        const uint32_t a0 = pack_bf16x2(ds[0][0], ds[0][1]), a1 = pack_bf16x2(ds[0][2], ds[0][3]);
        const uint32_t a2 = pack_bf16x2(ds[1][0], ds[1][1]), a3 = pack_bf16x2(ds[1][2], ds[1][3]);
        if (c == 0) {
#pragma unroll
            for (int j = 0; j < D / 8; ++j) mma16816_z(dQ[j], a0, a1, a2, a3, kt0.r[j], kt1.r[j]);
        } else {
            mma_cols<D>(dQ, a0, a1, a2, a3, kt0, kt1);
        }
    }
    // ---- sparse taps
    const float ls_lo = L.owner ? l2_lo : 1.0e30f, ls_hi = L.owner ? l2_hi : 1.0e30f;   // p == 0 on lanes without a diagonal entry
    float* stage_sp = stage_w + (SE ? nd : WB + 31) * SP + g;     // plain kernel: after the WB+31 delta rows
    auto finish = [&](int si, float sd0, float sd1, float dp0, float dp1, float pbv, bool v0, bool v1,
                      const RowFrag<D>& kf0, const RowFrag<D>& kf1) {
        float p0, p1;
        if constexpr (SE) {
            p0 = v0 ? ex2((sd0 + se.qs[g * se.pitch + nd + si]) * c2 - ls_lo) : 0.f;
            p1 = v1 ? ex2((sd1 + se.qs[(g + 8) * se.pitch + nd + si]) * c2 - ls_hi) : 0.f;
        } else {
            p0 = v0 ? ex2(fmaf(sd0, c2, pbv) - ls_lo) : 0.f;
            p1 = v1 ? ex2(fmaf(sd1, c2, pbv) - ls_hi) : 0.f;
        }
        dgrow = fmaf(p0, dp0, dgrow); dgrow = fmaf(p1, dp1, dgrow);
        const float x0 = p0 * fmaf(gain, dp0, -delta_lo), x1 = p1 * fmaf(gain, dp1, -delta_hi);
        if (L.owner) { stage_sp[si * SP] = x0; stage_sp[si * SP + 8] = x1; }
        diag_fma<D>(dQ, __shfl_sync(0xffffffffu, x0, L.owner_lane), __shfl_sync(0xffffffffu, x1, L.owner_lane), kf0, kf1);
    };
    auto full_taps = [&](auto GC, int si) {
        constexpr int GG = decltype(GC)::value;
        RowFrag<D> kf0[GG], kf1[GG], vf0[GG], vf1[GG];
        float pbv[GG];
#pragma unroll
        for (int i = 0; i < GG; ++i) {
            const int2 tp = tap_s[si + i];
            const ptrdiff_t off = (ptrdiff_t)tp.x * RS;
            pbv[i] = __int_as_float(tp.y);
            load_row_at(kf0[i], kl - off);
            load_row_at(kf1[i], kl - off + 8 * RS);
            load_row_at(vf0[i], vl - off);
            load_row_at(vf1[i], vl - off + 8 * RS);
        }
#pragma unroll
        for (int i = 0; i < GG; ++i) {
            float s0[4], s1[4], e0[4], e1[4];
            mma_rows_z(s0, qa, qb, kf0[i]); mma_rows_z(s1, qa, qb, kf1[i]);
            mma_rows_z(e0, da, db, vf0[i]); mma_rows_z(e1, da, db, vf1[i]);
            finish(si + i, (g & 1) ? s0[1] : s0[0], (g & 1) ? s1[3] : s1[2], (g & 1) ? e0[1] : e0[0],
                   (g & 1) ? e1[3] : e1[2], pbv[i], true, true, kf0[i], kf1[i]);
        }
    };
    // as in the forward: only interior tiles load taps unpredicated, so no key row past the end is read
    int si = 0;
    if constexpr (INTERIOR)
        for (; si + G <= ns && g0 >= tap_s[si + G - 1].x; si += G) full_taps(std::integral_constant<int, G>(), si);
#pragma unroll 1
    for (; si < ns; ++si) {
        const int delta = tap_s[si].x;
        if (g0 + 15 < delta) break;
        if (INTERIOR && g0 >= delta) {
            full_taps(std::integral_constant<int, 1>(), si);
        } else {
            const float pbv = __int_as_float(tap_s[si].y);
            const bool v0 = row_lo >= delta && row_lo - delta < N, v1 = row_hi >= delta && row_hi - delta < N;
            const ptrdiff_t off = (ptrdiff_t)delta * RS + 8 * tig;
            RowFrag<D> kf0, kf1, vf0, vf1;
            load_row(kf0, kl - off, tig, v0);
            load_row(kf1, kl - off + 8 * RS, tig, v1);
            load_row(vf0, vl - off, tig, v0);
            load_row(vf1, vl - off + 8 * RS, tig, v1);
            float s0[4], s1[4], e0[4], e1[4];
            mma_rows_z(s0, qa, qb, kf0); mma_rows_z(s1, qa, qb, kf1);
            mma_rows_z(e0, da, db, vf0); mma_rows_z(e1, da, db, vf1);
            finish(si, (g & 1) ? s0[1] : s0[0], (g & 1) ? s1[3] : s1[2], (g & 1) ? e0[1] : e0[0],
                   (g & 1) ? e1[3] : e1[2], pbv, v0, v1, kf0, kf1);
        }
    }
    if (L.owner)                                          // taps no row of the tile reaches: zero entries
        for (; si < ns; ++si) { stage_sp[si * SP] = 0.f; stage_sp[si * SP + 8] = 0.f; }
    if constexpr (SE) {
        // dQ += dS.scale_embed: the warp's ds values are complete in its 16 staging columns
        __syncwarp();
#pragma unroll 1
        for (int kk = 0; kk < sb.JS / 16; ++kk) {
            const float* col = stage_w + (16 * kk + 2 * tig) * SP + g;
            const uint32_t a0 = pack_bf16x2(col[0], col[SP]), a1 = pack_bf16x2(col[8], col[SP + 8]);
            const uint32_t a2 = pack_bf16x2(col[8 * SP], col[9 * SP]), a3 = pack_bf16x2(col[8 * SP + 8], col[9 * SP + 8]);
#pragma unroll
            for (int jn = 0; jn < D / 8; ++jn) {
                const uint2 b = __ldg(sb.seb + (kk * (D / 8) + jn) * 32 + L.lane);
                mma16816(dQ[jn], a0, a1, a2, a3, b.x, b.y);
            }
        }
    }
    __nv_bfloat16* dqp = static_cast<__nv_bfloat16*>(a.dq) + base;
    store_acc_rows<D>(dQ, dqp + (size_t)row_lo * RS, dqp + (size_t)row_hi * RS, ok_lo, ok_hi, a.scale, a.scale, tig);
    return dgrow;
}

// One block, before the dQ kernel with scale_embed.  Writes, back to back:
//   scale_embed split into bf16 halves [2][Jp][D];
//   its B fragments for dQ += dS.scale_embed, [JS/16][D/8][32] x uint2, in the element order of the
//     dQ accumulators (n-tile jn, column g <-> d = 32 (jn/4) + 8 (g>>1) + 2 (jn%4) + (g&1)), rows j >= J zero;
//   pos_bias[j,h] / scale for every head, [H][Jp];
//   the offset table of the dense window into a per-warp tile of the given pitch, [NT*32] x int4
//     (16 * pitch = the dump entry that holds the mask value).
struct SePre {
    const __nv_bfloat16* se_hi; const __nv_bfloat16* se_lo; const uint2* seb; const float* pbs; const int4* off;
};
__host__ __device__ inline SePre se_pre_layout(const void* base, int J, int D, int H) {
    const int Jp = (J + 7) / 8 * 8, JS = (J + 15) / 16 * 16;
    SePre p;
    p.se_hi = static_cast<const __nv_bfloat16*>(base);
    p.se_lo = p.se_hi + Jp * D;
    p.seb = reinterpret_cast<const uint2*>(p.se_lo + Jp * D);
    p.pbs = reinterpret_cast<const float*>(p.seb + (JS / 16) * (D / 8) * 32);
    p.off = reinterpret_cast<const int4*>(p.pbs + H * Jp);
    return p;
}
template <int D>
__global__ void se_prep_kernel(const float* __restrict__ scale_embed, const float* __restrict__ pos_bias, float scale,
                               int J, int H, int d_lo, int n_dense, int WB, void* out) {
    const int Jp = (J + 7) / 8 * 8, JS = (J + 15) / 16 * 16;
    const SePre P = se_pre_layout(out, J, D, H);
    __nv_bfloat162* hi = reinterpret_cast<__nv_bfloat162*>(const_cast<__nv_bfloat16*>(P.se_hi));
    __nv_bfloat162* lo = reinterpret_cast<__nv_bfloat162*>(const_cast<__nv_bfloat16*>(P.se_lo));
    for (int e = threadIdx.x; e < Jp * D / 2; e += blockDim.x) {
        const int j = (2 * e) / D;
        float2 x = make_float2(0.f, 0.f);
        if (j < J) x = *reinterpret_cast<const float2*>(scale_embed + 2 * e);
        const __nv_bfloat162 h2 = __floats2bfloat162_rn(x.x, x.y);
        hi[e] = h2;
        lo[e] = __floats2bfloat162_rn(x.x - __low2float(h2), x.y - __high2float(h2));
    }
    uint2* seb = const_cast<uint2*>(P.seb);
    for (int e = threadIdx.x; e < (JS / 16) * (D / 8) * 32; e += blockDim.x) {
        const int ln = e & 31, jn = (e >> 5) % (D / 8), kk = (e >> 5) / (D / 8);
        const int gg = ln >> 2, tt = ln & 3;
        const int d = 32 * (jn / 4) + 8 * (gg >> 1) + 2 * (jn % 4) + (gg & 1);
        const int j0 = 16 * kk + 2 * tt;
        auto sev = [&](int j) { return j < J ? scale_embed[j * D + d] : 0.f; };
        seb[e] = make_uint2(pack_bf16x2(sev(j0), sev(j0 + 1)), pack_bf16x2(sev(j0 + 8), sev(j0 + 9)));
    }
    float* pbs = const_cast<float*>(P.pbs);
    const float inv_scale = 1.f / scale;
    for (int e = threadIdx.x; e < H * Jp; e += blockDim.x) {
        const int h = e / Jp, j = e - h * Jp;
        pbs[e] = j < J ? pos_bias[j * H + h] * inv_scale : 0.f;
    }
    int4* off = const_cast<int4*>(P.off);
    const int NT = (WB + 16) / 8, pitch = Jp + 2, d_hi = d_lo + n_dense - 1;
    for (int e = threadIdx.x; e < NT * 32; e += blockDim.x) {
        const int nt = e >> 5, gg = (e & 31) >> 2, tt = e & 3;
        int o[4];
        for (int r = 0; r < 4; ++r) {
            const int i = gg + 8 * (r >> 1), delta = WB + i - (8 * nt + 2 * tt + (r & 1));
            o[r] = (delta >= d_lo && delta <= d_hi) ? i * pitch + (delta - d_lo) : 16 * pitch;
        }
        off[e] = make_int4(o[0], o[1], o[2], o[3]);
    }
}

inline size_t dq_smem_bytes(int J, int n_sparse, int D, int NT, bool se) {
    // staging rows: with scale_embed one per tap (rounded up to the MMA shape) plus a dump row;
    // plain kernel one per delta a tile element can have (8 NT + 15 = WB + 31) plus the sparse taps
    const int rows = se ? (J + 15) / 16 * 16 + 1 : 8 * NT + 15 + n_sparse;
    size_t n = sizeof(float) * ((size_t)rows * (se ? kStagePitchSe : kStagePitch) + kWarps * 32);
    if (se) {
        n = (n + 15) / 16 * 16;
        n += (size_t)kWarps * (16 * ((J + 7) / 8 * 8 + 2) + 4) * 4;      // one q.scale_embed tile per warp
        n = (n + 15) / 16 * 16;
        n += (size_t)kRows * (2 * D + 16);
    }
    return n;
}

template <int D, int WB, int G, int CT, bool SE, bool ST>
__global__ void __launch_bounds__(kWarps * 32, CT)
bwd_dq_mma_kernel(const BwdArgs a, const Taps t) {
    constexpr int NT = (WB + 16) / 8;
    constexpr int SP = StagePitch<SE>::v;
    extern __shared__ __align__(16) float stage[];     // [JS + 1][SP] ds values, then [128] dgain terms, then the scale_embed extras
    __shared__ float4 init_s[SE ? 1 : NT * 32];
    __shared__ int4 soff_s[SE ? NT * 32 : 1];          // staging offsets per lane (scale_embed variant only)
    __shared__ int2 tap_s[DSQG_MAX_TAPS];
    const Lane L;
    const int bh = blockIdx.y, h = bh % a.H, N = a.N, J = t.J;
    const int JS = SE ? (J + 15) / 16 * 16 : J;         // scale_embed: staging rows (row JS is the dump for out-of-band entries)
    constexpr int kDeltaRows = WB + 31;                 // plain kernel: one staging row per delta -15 .. WB+15
    float* dg_s = stage + (SE ? JS + 1 : kDeltaRows + t.n_sparse) * SP;
    SeTables se = {};
    SeBwd sb = {};
    {
        const int d_lo = t.d_lo, d_hi = t.d_lo + t.n_dense - 1;
        const float inv_scale = 1.f / a.scale;
        for (int e = threadIdx.x; e < NT * 32; e += kWarps * 32) {
            const int nt = e >> 5, gg = (e & 31) >> 2, tt = e & 3;
            float v[4];
            int o[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int i = gg + 8 * (r >> 1);
                const int delta = WB + i - (8 * nt + 2 * tt + (r & 1));
                const bool inband = delta >= d_lo && delta <= d_hi;
                v[r] = (!SE && inband) ? a.pos_bias[(delta - d_lo) * a.H + h] * inv_scale : kNeg;
                o[r] = (inband ? delta - d_lo : JS) * SP + i;
            }
            if constexpr (!SE) init_s[e] = make_float4(v[0], v[1], v[2], v[3]);
            if constexpr (SE) soff_s[e] = make_int4(o[0], o[1], o[2], o[3]);
        }
        for (int si = threadIdx.x; si < t.n_sparse; si += kWarps * 32)
            tap_s[si] = make_int2(t.sparse[si], __float_as_int(a.pos_bias[(t.n_dense + si) * a.H + h] * kLog2e));
        if constexpr (SE) {
            // tables come from global memory (se_prep_kernel); shared memory only holds the per-warp
            // q.scale_embed tiles and the CTA's query rows
            const SePre P = se_pre_layout(a.se_pre, J, D, a.H);
            const int Jp = (J + 7) / 8 * 8, pitch = Jp + 2;
            unsigned char* p = reinterpret_cast<unsigned char*>(dg_s + kWarps * 32);
            p = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(p) + 15) & ~uintptr_t(15));
            float* qs_w = reinterpret_cast<float*>(p) + L.warp * (16 * pitch + 4);
            if (L.lane == 0) qs_w[16 * pitch] = kNeg;          // the dump entry: masked
            se.se_hi = P.se_hi; se.se_lo = P.se_lo; se.pbs = P.pbs + h * Jp; se.off = P.off; se.qs = qs_w;
            se.Jp = Jp; se.pitch = pitch; se.nd = t.n_dense;
            p += (size_t)kWarps * (16 * pitch + 4) * 4;
            p = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(p) + 15) & ~uintptr_t(15));
            sb.JS = JS;
            sb.seb = P.seb;
            sb.q_s = p;
            // staging rows J .. JS-1 take part in the dS MMAs: zero
            for (int e = threadIdx.x; e < (JS - J) * kRows; e += kWarps * 32)
                stage[(J + e / kRows) * SP + e % kRows] = 0.f;
        }
    }
    __syncthreads();
    const int g0 = blockIdx.x * kRows + L.warp * 16;
    float* stage_w = stage + L.warp * 16;
    float dgrow = 0.f;
    if (g0 >= N) {                                      // no rows: this warp's staging columns (and query rows) are zero
        if constexpr (SE) {
            for (int e = L.lane; e < J * 16; e += 32) stage_w[(e >> 4) * SP + (e & 15)] = 0.f;
        } else {                                        // the rows the column sums read: in-band deltas, then the sparse taps
            for (int e = L.lane; e < J * 16; e += 32) {
                const int j = e >> 4;
                stage_w[(j < t.n_dense ? t.d_lo + j + 15 : kDeltaRows + j - t.n_dense) * SP + (e & 15)] = 0.f;
            }
        }
        if constexpr (SE)
            for (int e = L.lane; e < 16 * (2 * D + 16) / 16; e += 32)
                reinterpret_cast<uint4*>(sb.q_s + (size_t)L.warp * 16 * (2 * D + 16))[e] = make_uint4(0u, 0u, 0u, 0u);
    } else if (g0 >= WB && g0 + 16 <= N) {
        dgrow = dq_tile<D, WB, true, G, SE, ST>(a, init_s, soff_s, tap_s, stage_w, t.n_dense, t.n_sparse, bh, h, g0, L, se, sb);
    } else {
        dgrow = dq_tile<D, WB, false, G, SE, ST>(a, init_s, soff_s, tap_s, stage_w, t.n_dense, t.n_sparse, bh, h, g0, L, se, sb);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dgrow += __shfl_xor_sync(0xffffffffu, dgrow, o);
    if (L.lane == 0) dg_s[L.warp] = dgrow;
    __syncthreads();
    const int tile = bh * a.tiles_per_bh + blockIdx.x;
    if constexpr (SE) {
        // CTA partial of dscale_embed = scale * dS^T[JS x 64] . Q[64 x D]; warp w takes n-tiles w, w+4, ...
        constexpr int QP = 2 * D + 16;
        const uint32_t q_base = static_cast<uint32_t>(__cvta_generic_to_shared(sb.q_s));
#pragma unroll 1
        for (int jn = L.warp; jn < D / 8; jn += kWarps) {
#pragma unroll 1
            for (int mt = 0; mt < JS / 16; ++mt) {
                float c[4];
#pragma unroll
                for (int kk = 0; kk < kRows / 16; ++kk) {
                    const float* r0 = stage + (16 * mt + L.g) * SP + 16 * kk + 2 * L.tig;
                    const float2 u0 = *reinterpret_cast<const float2*>(r0), u1 = *reinterpret_cast<const float2*>(r0 + 8 * SP);
                    const float2 u2 = *reinterpret_cast<const float2*>(r0 + 8), u3 = *reinterpret_cast<const float2*>(r0 + 8 * SP + 8);
                    uint32_t b0, b1;
                    const uint32_t addr = q_base + (16 * kk + (L.lane & 15)) * QP + 16 * jn;
                    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(addr));
                    const uint32_t a0 = pack_bf16x2(u0.x, u0.y), a1 = pack_bf16x2(u1.x, u1.y);
                    const uint32_t a2 = pack_bf16x2(u2.x, u2.y), a3 = pack_bf16x2(u3.x, u3.y);
                    if (kk == 0) mma16816_z(c, a0, a1, a2, a3, b0, b1); else mma16816(c, a0, a1, a2, a3, b0, b1);
                }
                // the tile's partial goes to global memory; dse_group_kernel adds the tiles of a group
                float* dst = a.dse_tmp + (size_t)tile * J * D + (16 * mt + L.g) * D + 8 * jn + 2 * L.tig;
                if (16 * mt + L.g < J) *reinterpret_cast<float2*>(dst) = make_float2(c[0] * a.scale, c[1] * a.scale);
                if (16 * mt + L.g + 8 < J) *reinterpret_cast<float2*>(dst + 8 * D) = make_float2(c[2] * a.scale, c[3] * a.scale);
            }
        }
    }
    // Column sums of the staging tile: two threads per tap (32 rows each, four independent partial
    // sums, fixed order), so the CTA's tail is a few dozen dependent additions instead of kRows.
    static_assert(kRows == 64 && kWarps == 4, "the column sums below split 64 rows over thread pairs");
    for (int j0 = 0; j0 < J; j0 += kWarps * 16) {
        const int j = j0 + (threadIdx.x >> 1), half = threadIdx.x & 1;
        float s = 0.f;
        if (j < J) {
            // pitch 68 puts rows j and j+8 (and the two halves) in the same banks: start each of the
            // four at a different column so that a warp's 32 reads fall into 32 banks
            const int jr = SE ? j : (j < t.n_dense ? t.d_lo + j + 15 : kDeltaRows + j - t.n_dense);   // staging row of tap j
            const float* row = stage + jr * SP + 32 * half;
            const int rot = ((jr >> 3) & 1) + 2 * half;
            float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
            for (int r = 0; r < 32; r += 4) {
                s0 += row[(r + rot) & 31]; s1 += row[(r + 1 + rot) & 31];
                s2 += row[(r + 2 + rot) & 31]; s3 += row[(r + 3 + rot) & 31];
            }
            s = (s0 + s1) + (s2 + s3);
        }
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        if (j < J && half == 0) a.dpb_part[(size_t)tile * J + j] = s;
    }
    if (threadIdx.x == 0) a.dg_part[tile] = (dg_s[0] + dg_s[1]) + (dg_s[2] + dg_s[3]);
}

// dscale_embed partials: one block per group of kSeGroup consecutive 64-row tiles of a sequence adds
// the tiles' partials (written by the dQ kernel) in tile order.
__global__ void __launch_bounds__(256)
dse_group_kernel(const float* __restrict__ tmp, float* __restrict__ part, int tiles_per_bh, int groups_bh, int JD) {
    const int bh = blockIdx.y, grp = blockIdx.x, first = grp * kSeGroup;
    const int members = tiles_per_bh - first < kSeGroup ? tiles_per_bh - first : kSeGroup;
    const float* src = tmp + ((size_t)bh * tiles_per_bh + first) * JD;
    float* out = part + ((size_t)bh * groups_bh + grp) * JD;
    for (int e = threadIdx.x; e < JD; e += 256) {
        float x[kSeGroup];
#pragma unroll
        for (int r = 0; r < kSeGroup; ++r) x[r] = r < members ? __ldg(src + (size_t)r * JD + e) : 0.f;
        float s = x[0];
#pragma unroll
        for (int r = 1; r < kSeGroup; ++r) s += x[r];
        out[e] = s;
    }
}

// ------------------------------------------------------------------------------ backward: dK, dV
// The warp owns 16 key rows; the roles of rows and columns are swapped: S^T = K.Q^T over the
// query rows [m0, m0+16+WB) for the dense window and the diagonal of the tile at m0+delta for
// every sparse tap.  Key rows are owned by exactly one warp: no atomics.  The per-query
// statistics {lse*log2(e), delta} of the CTA's dense query range sit in shared memory.
// With scale_embed the score accumulators of the dense window start from qsd, the CTA's copy of the
// dense part of qs_rows (row = query, nd + 1 columns, the last one holding the mask value), and a
// sparse tap adds the entry of its query row read from global memory.
template <int D, int WB, bool INTERIOR, int G, bool SE, bool ST>
__device__ __forceinline__ void dkdv_tile(const BwdArgs& a, const float4* init_s, const int2* tap_s, const float2* stat_w,
                                          int ns, int bh, int h, int m0, const Lane& L, const float* qsd_w,
                                          const int4* qoff, int nd, int Jp) {
    constexpr int NT = (WB + 16) / 8;
    const int N = a.N, g = L.g, tig = L.tig;
    const int row_lo = m0 + g, row_hi = row_lo + 8;
    const bool ok_lo = INTERIOR || row_lo < N, ok_hi = INTERIOR || row_hi < N;
    const ptrdiff_t RS = ST ? (ptrdiff_t)a.in_sn : D, OS = ST ? (ptrdiff_t)a.out_sn : D;   // row strides of q/k/v/dk/dv and of dout
    const size_t base = ST ? (size_t)(bh / a.H) * a.in_sb + (size_t)h * a.in_sh : (size_t)bh * N * D;
    const size_t obase = ST ? (size_t)(bh / a.H) * a.out_sb + (size_t)h * a.out_sh : base;
    const __nv_bfloat16* kp = static_cast<const __nv_bfloat16*>(a.k) + base;
    const __nv_bfloat16* vp = static_cast<const __nv_bfloat16*>(a.v) + base;
    const __nv_bfloat16* ql = static_cast<const __nv_bfloat16*>(a.q) + base + (ptrdiff_t)row_lo * RS + 8 * tig;
    const __nv_bfloat16* dl = static_cast<const __nv_bfloat16*>(a.dout) + obase + (ptrdiff_t)row_lo * OS + 8 * tig;
    const float2* rs = reinterpret_cast<const float2*>(a.delta) + (size_t)bh * N + row_lo;
    const float c2 = a.scale * kLog2e;
    const float gain = a.head_gain ? a.head_gain[h] : 1.f;

    RowFrag<D> ka, kb, va, vb;
    load_row(ka, kp + (size_t)row_lo * RS, tig, ok_lo);
    load_row(kb, kp + (size_t)row_hi * RS, tig, ok_hi);
    load_row(va, vp + (size_t)row_lo * RS, tig, ok_lo);
    load_row(vb, vp + (size_t)row_hi * RS, tig, ok_hi);
    float dK[D / 8][4], dV[D / 8][4];

    // ---- dense window: query row of n-tile nt for this thread is m0 + 8 nt + g
#pragma unroll
    for (int c = 0; c < NT / 2; ++c) {
        if (!INTERIOR && c > 0 && m0 + 16 * c >= N) break;   // warp-uniform: no query rows left
        RowFrag<D> qf[2], df[2];
        float ds[2][4], pv[2][4];
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
            const int nt = 2 * c + hf;
            float s[4], dp[4];
            if constexpr (SE) {
                const int4 qo = qoff[nt * 32 + L.lane];
                s[0] = qsd_w[qo.x]; s[1] = qsd_w[qo.y]; s[2] = qsd_w[qo.z]; s[3] = qsd_w[qo.w];
            } else {
                const float4 ini = init_s[nt * 32 + L.lane];
                s[0] = ini.x; s[1] = ini.y; s[2] = ini.z; s[3] = ini.w;
            }
            if (INTERIOR) {
                load_row_at(qf[hf], ql + 8 * nt * RS);
                load_row_at(df[hf], dl + 8 * nt * OS);
            } else {
                const bool qv = m0 + 8 * nt + g < N;
                load_row(qf[hf], ql + (ptrdiff_t)8 * nt * RS - 8 * tig, tig, qv);
                load_row(df[hf], dl + (ptrdiff_t)8 * nt * OS - 8 * tig, tig, qv);
            }
            mma_rows(s, ka, kb, qf[hf]);
            mma_rows_z(dp, va, vb, df[hf]);
            // statistics of this thread's two query columns: {l2, delta} x 2
            const float4 st = *reinterpret_cast<const float4*>(stat_w + 8 * nt + 2 * tig);
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const float p = ex2(fmaf(s[r], c2, (r & 1) ? -st.z : -st.x));
                ds[hf][r] = p * fmaf(gain, dp[r], (r & 1) ? -st.w : -st.y);
                pv[hf][r] = p * gain;
            }
        }
        RowFrag<D> t0, t1;
        transpose_frag(t0, df[0]); transpose_frag(t1, df[1]);
        const uint32_t b0 = pack_bf16x2(pv[0][0], pv[0][1]), b1 = pack_bf16x2(pv[0][2], pv[0][3]);
        const uint32_t b2 = pack_bf16x2(pv[1][0], pv[1][1]), b3 = pack_bf16x2(pv[1][2], pv[1][3]);
        const uint32_t a0 = pack_bf16x2(ds[0][0], ds[0][1]), a1 = pack_bf16x2(ds[0][2], ds[0][3]);
        const uint32_t a2 = pack_bf16x2(ds[1][0], ds[1][1]), a3 = pack_bf16x2(ds[1][2], ds[1][3]);
        if (c == 0) {
#pragma unroll
            for (int j = 0; j < D / 8; ++j) mma16816_z(dV[j], b0, b1, b2, b3, t0.r[j], t1.r[j]);
        } else {
            mma_cols<D>(dV, b0, b1, b2, b3, t0, t1);
        }
        transpose_frag(t0, qf[0]); transpose_frag(t1, qf[1]);
        if (c == 0) {
#pragma unroll
            for (int j = 0; j < D / 8; ++j) mma16816_z(dK[j], a0, a1, a2, a3, t0.r[j], t1.r[j]);
        } else {
            mma_cols<D>(dK, a0, a1, a2, a3, t0, t1);
        }
    }
    // ---- sparse taps
    const float* qs_r = SE ? a.qs_rows + ((size_t)bh * N + row_lo) * Jp + nd : nullptr;   // entry of tap si of query row row_lo + delta: qs_r[delta * Jp + si]
    // b0/b1: what is added to the raw score: the bias in log2 units (plain) or the qs_rows entry of
    // the query row, in units of 1/scale (scale_embed)
    auto finish = [&](float sd0, float sd1, float dp0, float dp1, float b0, float b1, float2 st0, float2 st1,
                      const RowFrag<D>& qf0, const RowFrag<D>& qf1, const RowFrag<D>& df0, const RowFrag<D>& df1) {
        const float y0 = SE ? (sd0 + b0) * c2 : fmaf(sd0, c2, b0), y1 = SE ? (sd1 + b1) * c2 : fmaf(sd1, c2, b1);
        const float p0 = ex2(y0 - st0.x), p1 = ex2(y1 - st1.x);
        const float w0 = p0 * gain, w1 = p1 * gain;
        const float x0 = p0 * fmaf(gain, dp0, -st0.y), x1 = p1 * fmaf(gain, dp1, -st1.y);
        diag_fma<D>(dV, __shfl_sync(0xffffffffu, w0, L.owner_lane), __shfl_sync(0xffffffffu, w1, L.owner_lane), df0, df1);
        diag_fma<D>(dK, __shfl_sync(0xffffffffu, x0, L.owner_lane), __shfl_sync(0xffffffffu, x1, L.owner_lane), qf0, qf1);
    };
    auto full_taps = [&](auto GC, int si) {
        constexpr int GG = decltype(GC)::value;
        RowFrag<D> qf0[GG], qf1[GG], df0[GG], df1[GG];
        float2 st0[GG], st1[GG];
        float b0[GG], b1[GG];
#pragma unroll
        for (int i = 0; i < GG; ++i) {
            const int2 tp = tap_s[si + i];
            const ptrdiff_t off = (ptrdiff_t)tp.x * RS, offd = (ptrdiff_t)tp.x * OS;
            if constexpr (SE) {
                b0[i] = __ldg(qs_r + (size_t)tp.x * Jp + si + i);
                b1[i] = __ldg(qs_r + (size_t)(tp.x + 8) * Jp + si + i);
            } else {
                b0[i] = b1[i] = __int_as_float(tp.y);
            }
            load_row_at(qf0[i], ql + off);
            load_row_at(qf1[i], ql + off + 8 * RS);
            load_row_at(df0[i], dl + offd);
            load_row_at(df1[i], dl + offd + 8 * OS);
            st0[i] = __ldg(rs + tp.x);
            st1[i] = __ldg(rs + tp.x + 8);
        }
#pragma unroll
        for (int i = 0; i < GG; ++i) {
            float s0[4], s1[4], e0[4], e1[4];
            mma_rows_z(s0, ka, kb, qf0[i]); mma_rows_z(s1, ka, kb, qf1[i]);
            mma_rows_z(e0, va, vb, df0[i]); mma_rows_z(e1, va, vb, df1[i]);
            finish((g & 1) ? s0[1] : s0[0], (g & 1) ? s1[3] : s1[2], (g & 1) ? e0[1] : e0[0], (g & 1) ? e1[3] : e1[2],
                   b0[i], b1[i], st0[i], st1[i], qf0[i], qf1[i], df0[i], df1[i]);
        }
    };
    int si = 0;
    for (; si + G <= ns && m0 + 16 + tap_s[si + G - 1].x <= N; si += G) full_taps(std::integral_constant<int, G>(), si);
#pragma unroll 1
    for (; si < ns; ++si) {
        const int delta = tap_s[si].x;
        if (m0 + delta >= N) break;                     // taps ascend: no query row reads these keys any more
        if (m0 + 16 + delta <= N) {
            full_taps(std::integral_constant<int, 1>(), si);
        } else {
            const bool v0 = row_lo + delta < N, v1 = row_hi + delta < N;
            float b0 = __int_as_float(tap_s[si].y), b1 = b0;
            if constexpr (SE) {
                b0 = v0 ? __ldg(qs_r + (size_t)delta * Jp + si) : 0.f;
                b1 = v1 ? __ldg(qs_r + (size_t)(delta + 8) * Jp + si) : 0.f;
            }
            const ptrdiff_t off = (ptrdiff_t)delta * RS - 8 * tig, offd = (ptrdiff_t)delta * OS - 8 * tig;
            RowFrag<D> qf0, qf1, df0, df1;
            load_row(qf0, ql + off, tig, v0);
            load_row(qf1, ql + off + 8 * RS, tig, v1);
            load_row(df0, dl + offd, tig, v0);
            load_row(df1, dl + offd + 8 * OS, tig, v1);
            const float2 st0 = v0 ? __ldg(rs + delta) : make_float2(0.f, 0.f);
            const float2 st1 = v1 ? __ldg(rs + delta + 8) : make_float2(0.f, 0.f);
            float s0[4], s1[4], e0[4], e1[4];
            mma_rows_z(s0, ka, kb, qf0); mma_rows_z(s1, ka, kb, qf1);
            mma_rows_z(e0, va, vb, df0); mma_rows_z(e1, va, vb, df1);
            finish((g & 1) ? s0[1] : s0[0], (g & 1) ? s1[3] : s1[2], (g & 1) ? e0[1] : e0[0], (g & 1) ? e1[3] : e1[2],
                   b0, b1, st0, st1, qf0, qf1, df0, df1);
        }
    }
    __nv_bfloat16* dkp = static_cast<__nv_bfloat16*>(a.dk) + base;
    __nv_bfloat16* dvp = static_cast<__nv_bfloat16*>(a.dv) + base;
    store_acc_rows<D>(dK, dkp + (size_t)row_lo * RS, dkp + (size_t)row_hi * RS, ok_lo, ok_hi, a.scale, a.scale, tig);
    store_acc_rows<D>(dV, dvp + (size_t)row_lo * RS, dvp + (size_t)row_hi * RS, ok_lo, ok_hi, 1.f, 1.f, tig);
}

inline size_t dkdv_smem_bytes(int n_dense, int WB, bool se) {
    return se ? (size_t)(kRows + WB) * (n_dense + 1) * 4 : 0;
}

template <int D, int WB, int G, int CT, bool SE, bool ST>
__global__ void __launch_bounds__(kWarps * 32, CT)
bwd_dkdv_mma_kernel(const BwdArgs a, const Taps t, const int n_reduce, const int reduce_stride) {
    constexpr int NT = (WB + 16) / 8;
    constexpr int kStat = kRows + WB;                  // query rows the CTA's dense windows touch
    extern __shared__ __align__(16) float qsd[];       // scale_embed: [kStat][n_dense + 1]
    __shared__ float4 init_s[NT * 32];                 // plain: score start values; scale_embed: int4 offsets into qsd
    __shared__ int2 tap_s[DSQG_MAX_TAPS];
    __shared__ __align__(16) float2 stat_s[kStat];
    const Lane L;
    const int bh = blockIdx.y, h = bh % a.H, N = a.N;
    // n_reduce CTAs (every reduce_stride-th one, so that no wave of CTAs is delayed as a whole)
    // also finish the parameter gradients: one output each, from the partial sums the dQ kernel
    // (an earlier launch on the stream) left in the scratch.
    static_assert(kWarps * 32 == kReduceThreads, "the fused reduction uses the CTA as one reduce block");
    const int cta = blockIdx.y * gridDim.x + blockIdx.x;
    if (cta % reduce_stride == 0 && cta / reduce_stride < n_reduce)
        reduce_one_param(a, t.J, cta / reduce_stride, reinterpret_cast<float*>(init_s));
    const int m_cta = blockIdx.x * kRows;
    const int nd = t.n_dense, ndp = nd + 1, Jp = (t.J + 7) / 8 * 8;
    {
        const int d_lo = t.d_lo, d_hi = t.d_lo + t.n_dense - 1;
        const float inv_scale = 1.f / a.scale;
        for (int e = threadIdx.x; e < NT * 32; e += kWarps * 32) {
            const int nt = e >> 5, gg = (e & 31) >> 2, tt = e & 3;
            float v[4];
            int o[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int cc = 8 * nt + 2 * tt + (r & 1);
                const int delta = cc - (gg + 8 * (r >> 1));
                const bool inband = delta >= d_lo && delta <= d_hi;
                v[r] = (!SE && inband) ? a.pos_bias[(delta - d_lo) * a.H + h] * inv_scale : kNeg;
                o[r] = cc * ndp + (inband ? delta - d_lo : nd);       // column nd of every row holds the mask value
            }
            if constexpr (SE) reinterpret_cast<int4*>(init_s)[e] = make_int4(o[0], o[1], o[2], o[3]);
            else init_s[e] = make_float4(v[0], v[1], v[2], v[3]);
        }
        for (int si = threadIdx.x; si < t.n_sparse; si += kWarps * 32)
            tap_s[si] = make_int2(t.sparse[si], __float_as_int(a.pos_bias[(t.n_dense + si) * a.H + h] * kLog2e));
        const float2* rs = reinterpret_cast<const float2*>(a.delta) + (size_t)bh * N;
        for (int i = threadIdx.x; i < kStat; i += kWarps * 32)
            stat_s[i] = m_cta + i < N ? rs[m_cta + i] : make_float2(0.f, 0.f);
        if constexpr (SE) {
            const float* src = a.qs_rows + ((size_t)bh * N + m_cta) * Jp;
            for (int r = threadIdx.x; r < kStat; r += kWarps * 32) qsd[r * ndp + nd] = kNeg;      // the mask column
            {
                // 16-byte loads for the first nd/4*4 columns: lane c4 < nd/4 of warp w takes rows w, w+4, ...;
                // eight rows per batch in flight
                const int per_row = nd / 4;
                constexpr int kBatch = 8;
                for (int c4 = L.lane; c4 < per_row; c4 += 32) {
#pragma unroll 1
                    for (int r0 = L.warp; r0 < kStat; r0 += kWarps * kBatch) {
                        float4 x[kBatch];
#pragma unroll
                        for (int u = 0; u < kBatch; ++u) {
                            const int r = r0 + kWarps * u;
                            x[u] = (r < kStat && m_cta + r < N) ? __ldg(reinterpret_cast<const float4*>(src + (size_t)r * Jp) + c4)
                                                                : make_float4(0.f, 0.f, 0.f, 0.f);
                        }
#pragma unroll
                        for (int u = 0; u < kBatch; ++u) {
                            const int r = r0 + kWarps * u;
                            if (r < kStat) {
                                float* dst = qsd + r * ndp + 4 * c4;
                                dst[0] = x[u].x; dst[1] = x[u].y; dst[2] = x[u].z; dst[3] = x[u].w;
                            }
                        }
                    }
                }
            }
            // the last nd % 4 columns, one element per thread
            const int rem = nd & 3, c_first = nd - rem;
            for (int e = threadIdx.x; e < kStat * rem; e += kWarps * 32) {
                const int r = e / rem, c = c_first + e - r * rem;
                qsd[r * ndp + c] = m_cta + r < N ? __ldg(src + (size_t)r * Jp + c) : 0.f;
            }
        }
    }
    __syncthreads();
    const int m0 = m_cta + L.warp * 16;
    if (m0 >= N) return;
    const float* qsd_w = qsd + L.warp * 16 * ndp;
    const int4* qoff = reinterpret_cast<const int4*>(init_s);
    if (m0 + 16 + WB <= N)
        dkdv_tile<D, WB, true, G, SE, ST>(a, init_s, tap_s, stat_s + L.warp * 16, t.n_sparse, bh, h, m0, L, qsd_w, qoff, nd, Jp);
    else
        dkdv_tile<D, WB, false, G, SE, ST>(a, init_s, tap_s, stat_s + L.warp * 16, t.n_sparse, bh, h, m0, L, qsd_w, qoff, nd, Jp);
}

// Raises a kernel's dynamic shared-memory limit to what this launch needs.  The attribute is set
// once per kernel and device for the largest size seen so far (`seen` is that kernel's record),
// not on every launch.
template <typename K>
cudaError_t ensure_dynamic_smem(K kernel, size_t bytes, int (&seen)[64]) {
    if (bytes <= 32 * 1024) return cudaSuccess;        // static shared memory counts against the 48 KB default as well
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    if (dev >= 0 && dev < 64 && seen[dev] >= (int)bytes) return cudaSuccess;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e == cudaSuccess && dev >= 0 && dev < 64) seen[dev] = (int)bytes;
    return e;
}

template <int D, int WB>
cudaError_t fwd_launch_mma(const FwdArgs& a, const Taps& t, cudaStream_t s) {
    constexpr int W = FwdTune<D>::warps, rows = 16 * W;
    dim3 grid((a.N + rows - 1) / rows, a.B * a.H);
    if (a.scale_embed) {
        if constexpr (D <= 64) {
            const size_t smem = se_tables_bytes(t.J, D, (WB + 16) / 8, W, 16);
            static int seen[64] = {0}, seen_st[64] = {0};
            cudaError_t e = a.strided ? ensure_dynamic_smem(fwd_mma_kernel<D, WB, true, true>, smem, seen_st)
                                      : ensure_dynamic_smem(fwd_mma_kernel<D, WB, true, false>, smem, seen);
            if (e != cudaSuccess) return e;
            if (a.strided) fwd_mma_kernel<D, WB, true, true><<<grid, W * 32, smem, s>>>(a, t);
            else fwd_mma_kernel<D, WB, true, false><<<grid, W * 32, smem, s>>>(a, t);
        } else {
            return cudaErrorInvalidValue;
        }
    } else if (a.strided) {
        fwd_mma_kernel<D, WB, false, true><<<grid, W * 32, 0, s>>>(a, t);
    } else {
        fwd_mma_kernel<D, WB, false, false><<<grid, W * 32, 0, s>>>(a, t);
    }
    return cudaGetLastError();
}

template <int D, int WB, bool SE, bool ST>
cudaError_t bwd_launch_mma_se(BwdArgs a, const Taps& t, cudaStream_t s, int stages) {
    using T = BwdTune<D>;
    constexpr int NT = (WB + 16) / 8;
    if constexpr (SE) carve_bwd_scratch_mma_se(a, t.J); else carve_bwd_scratch(a, kRows, t.J, false);
    dim3 grid((a.N + kRows - 1) / kRows, a.B * a.H);
    cudaError_t e = cudaSuccess;
    if (stages & DSQG_BWD_STAGE_DQ) {
        if constexpr (SE) {
            se_prep_kernel<D><<<1, 1024, 0, s>>>(a.scale_embed, a.pos_bias, a.scale, t.J, a.H, t.d_lo, t.n_dense, WB, a.se_pre);
            if ((e = cudaGetLastError()) != cudaSuccess) return e;
        }
        auto kern = bwd_dq_mma_kernel<D, WB, SE ? T::dq_group_se : T::dq_group, SE ? T::dq_ctas_se : T::dq_ctas, SE, ST>;
        const size_t smem = dq_smem_bytes(t.J, t.n_sparse, D, NT, SE);
        static int seen[64] = {0};
        if ((e = ensure_dynamic_smem(kern, smem, seen)) != cudaSuccess) return e;
        kern<<<grid, kWarps * 32, smem, s>>>(a, t);
        if ((e = cudaGetLastError()) != cudaSuccess) return e;
        if constexpr (SE) {
            const int groups_bh = (a.tiles_per_bh + kSeGroup - 1) / kSeGroup;
            dse_group_kernel<<<dim3(groups_bh, a.B * a.H), 256, 0, s>>>(a.dse_tmp, a.dse_part, a.tiles_per_bh, groups_bh, t.J * a.D);
            if ((e = cudaGetLastError()) != cudaSuccess) return e;
        }
    }
    // With both stages in one call the reduction rides on CTAs of the dK/dV kernel (same code,
    // same order of additions as the stand-alone kernel: bitwise equal results).
    const int n_out = t.J * a.H + a.H + (SE ? t.J * a.D : 0);
    const bool fuse = (stages & DSQG_BWD_STAGE_DKDV) && (stages & DSQG_BWD_STAGE_REDUCE) &&
                      (long long)grid.x * grid.y >= n_out;
    if (stages & DSQG_BWD_STAGE_DKDV) {
        auto kern = bwd_dkdv_mma_kernel<D, WB, SE ? T::dkdv_group_se : T::dkdv_group, SE ? T::dkdv_ctas_se : T::dkdv_ctas, SE, ST>;
        const size_t smem = dkdv_smem_bytes(t.n_dense, WB, SE);
        static int seen[64] = {0};
        if ((e = ensure_dynamic_smem(kern, smem, seen)) != cudaSuccess) return e;
        kern<<<grid, kWarps * 32, smem, s>>>(a, t, fuse ? n_out : 0, fuse ? (int)((long long)grid.x * grid.y / n_out) : 1);
        if ((e = cudaGetLastError()) != cudaSuccess) return e;
    }
    if ((stages & DSQG_BWD_STAGE_REDUCE) && !fuse) e = launch_reduce_params(a, t.J, s);
    return e;
}

template <int D, int WB>
cudaError_t bwd_launch_mma(const BwdArgs& a, const Taps& t, cudaStream_t s, int stages) {
    if (a.scale_embed) {
        if constexpr (D <= 64) {
            if (a.strided) return bwd_launch_mma_se<D, WB, true, true>(a, t, s, stages);
            return bwd_launch_mma_se<D, WB, true, false>(a, t, s, stages);
        } else {
            return cudaErrorInvalidValue;
        }
    }
    if (a.strided) return bwd_launch_mma_se<D, WB, false, true>(a, t, s, stages);
    return bwd_launch_mma_se<D, WB, false, false>(a, t, s, stages);
}

int band_width(const Taps& t) {
    const int d_hi = t.d_lo + t.n_dense - 1;
    return d_hi <= 32 ? 32 : (d_hi <= 48 ? 48 : (d_hi <= 64 ? 64 : 0));
}

}  // namespace

static bool mma_shape_supported(int dtype, int D, const Taps& t) {
    const int wb = band_width(t);
    return dtype == DSQG_DTYPE_BF16 && t.n_sparse <= kMaxSparse &&
           (((D == 32 || D == 64) && wb != 0) || ((D == 96 || D == 128) && wb == 32));
}
bool mma_fwd_supported(int dtype, int D, const Taps& t, bool has_scale_embed) {
    return mma_shape_supported(dtype, D, t) && (!has_scale_embed || D <= 64);
}
bool mma_path_supported(int dtype, int D, const Taps& t, bool has_scale_embed) {
    return mma_shape_supported(dtype, D, t) && (!has_scale_embed || D <= 64);
}

#define DSQG_MMA_DISPATCH(FN, ...)                                             \
    do {                                                                       \
        const int wb_ = band_width(t);                                         \
        if (a.D == 32) {                                                       \
            if (wb_ == 32) return FN<32, 32>(__VA_ARGS__);                     \
            if (wb_ == 48) return FN<32, 48>(__VA_ARGS__);                     \
            return FN<32, 64>(__VA_ARGS__);                                    \
        }                                                                      \
        if (a.D == 96) return FN<96, 32>(__VA_ARGS__);                         \
        if (a.D == 128) return FN<128, 32>(__VA_ARGS__);                       \
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
