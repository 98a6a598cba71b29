// Forward with TMA-staged V (bf16 storage, fp32 accumulate; D in {32, 64}; dense offsets within
// 0..32; up to 16 sparse taps).  Opt-in (kernel path 3): on B200 it measures slower than the
// register-fed kernels of dsqg_mma.cu (cfg1 forward 102 us against 75 us), so the automatic choice
// never takes it; it stays as the measured alternative and as the home of the copy-engine code.
//
// Math: DWARF reference kernels/dsqg_attention_v3.py:60-163, with the per-head output gain of
// train/train_2048_condU.py:187 fused in.
//
// A thread block owns 64 rows of one (batch, head) sequence, a warp 16 of them.
//   * K and Q are read straight from global memory as row fragments (scores contract over d, which
//     any consistent element order serves).  V, which the P.V products contract over ROWS, is
//     staged once per block by the copy engine (dsqg_stage.cuh: one fetch per block, taps that
//     overlap share rows) and read back transposed with ldmatrix;
//   * dense window: banded GEMM of the warp's 16 rows against the 48 band rows around them
//     (mma.sync m16n8k16), scores start from a table that holds bias and band mask;
//   * sparse taps: a tap pairs row r of the own tile with row r of a shifted tile, i.e. it needs
//     row-wise dot products.  They are formed as (own . partner) element-wise in bf16x2, summed
//     over d on the tensor core against a 0/1 selector that drops the sums of tap c into column
//     c of an accumulator tile: eight taps share one 16x8 tile, so the softmax arithmetic of the
//     sparse taps runs on full vectors, two MMAs per tap at D = 32;
//   * all scores of a row exist before the first exponential: exact row maximum, no rescaling;
//   * P.V of a sparse tap is an MMA with a diagonal A fragment built by one shuffle and two byte
//     permutes, B straight from ldmatrix.trans;
//   * the output leaves through shared memory and a copy-engine store (rows past N are clipped).
#include "dsqg_stage.cuh"

#include <mutex>

namespace dsqg {
namespace stg {

namespace {

constexpr int kWarps = kRows / 16;
constexpr int kThreads = kWarps * 32;
constexpr uint32_t kOnes = 0x3F803F80u;    // bf16x2 {1, 1}

// Shared-memory carve-up (byte offsets from a 1024-byte boundary).
//   y : staged partner tiles     stage : kRows x D output staging tiles (n_stage of them)     tab : tables
template <int D>
struct Smem {
    static constexpr int RB = 2 * D;
    int y, stage, tab, bars, misc, total;
    __host__ __device__ Smem(int rows, int n_stage, int tab_bytes) {
        y = 0;
        stage = y + rows * RB;
        tab = stage + n_stage * kRows * RB;
        bars = tab + ((tab_bytes + 15) & ~15);
        misc = bars + 8 * kMaxSeg;
        total = misc + 16;
    }
};

struct Maps { bool hf[8]; };   // head_first flag per tensor map of a launch

// Tables a block builds once (shared memory):
//   pbx[d + 48], d in [-48, 80): bias of dense offset d in units of 1/scale, a large negative number for every
//     d outside the dense window.  Entry (row i, band column c) of a 16 x 48 score tile has d = 32 + i - c, so
//     a lane's 24 start values sit at compile-time distances from pbx[48 + 32 + g - 2 tig];
//   taps[i] = {offset, bias / scale (float bits), byte offset of the tap's tile in the staged area, its segment};
//   tile_nv[w] = {taps that reach at least one row of warp w's tile, taps that reach all 16}.
constexpr int kPbxLo = 48, kPbxN = 128;
struct Tables {
    float pbx[kPbxN];
    int4 taps[kMaxTaps];
    int2 tile_nv[kWarps];
};

template <int D>
__device__ __forceinline__ void fill_tables(Tables* tb, const float* pos_bias, const Taps& t, const Plan& pl, int H, int h,
                                            float scale, int n0, int N) {
    const int d_lo = t.d_lo, d_hi = t.d_lo + t.n_dense - 1;
    const float inv_scale = 1.f / scale;
    for (int e = threadIdx.x; e < kPbxN; e += kThreads) {
        const int d = e - kPbxLo;
        tb->pbx[e] = (d >= d_lo && d <= d_hi) ? pos_bias[(d - d_lo) * H + h] * inv_scale : kNeg;
    }
    if (threadIdx.x < kMaxTaps) {
        const int i = threadIdx.x;
        tb->taps[i] = i < t.n_sparse
            ? make_int4(t.sparse[i], __float_as_int(pos_bias[(t.n_dense + i) * H + h] * inv_scale), pl.tap_row0[i] * 2 * D, pl.tap_seg[i])
            : make_int4(0x3fffffff, __float_as_int(kNeg), 0, 0);
    }
    if (threadIdx.x >= 32 && threadIdx.x < 32 + kWarps) {
        const int w = threadIdx.x - 32, g0 = n0 + 16 * w, reach = min(g0 + 15, N - 1);
        int nv = 0, nf = 0;
        for (int i = 0; i < t.n_sparse; ++i) { nv += t.sparse[i] <= reach; nf += t.sparse[i] <= g0; }
        tb->tile_nv[w] = make_int2(nv, nf);
    }
}

// Warp 0: lane i initialises and arms the barrier of segment i and issues box i.  n_reach = number of
// segments the block needs (segments are ordered by the smallest offset they serve); the others
// are neither copied nor waited for.
template <int D>
__device__ __forceinline__ void issue_copies(const Plan& pl, int lane, int n_reach, const Tma& ty, uint32_t sy,
                                             uint32_t bars, volatile int* abort_flag, int own0, int h, int b) {
    constexpr int RB = 2 * D;
    if (lane < n_reach) mbar_init(bars + 8 * lane, 1);
    if (lane == 0) *abort_flag = 0;
    fence_mbar_init();
    fence_proxy_async();
    __syncwarp();
    if (lane < n_reach) mbar_arrive_expect_tx(bars + 8 * lane, (uint32_t)pl.seg_boxes[lane] * kRows * RB);
    __syncwarp();
    if (lane < pl.n_box && pl.box_seg[lane] < n_reach)
        ty.load(sy + (uint32_t)pl.box_row0[lane] * RB, bars + 8 * pl.box_seg[lane], own0 + pl.box_rel[lane], h, b);
}

// ------------------------------------------------------------------------------ forward
// K and Q come straight from global memory as row fragments (scores contract over d, which any
// consistent element order serves); V, which the P.V products contract over ROWS, is staged by
// the copy engine and read back transposed with ldmatrix.  The copies are issued first and are
// only waited for after the scores and the softmax, so their latency is covered by the block's
// own arithmetic.  INTERIOR: every band row of the tile exists (loads without predicates).
struct FwdCtx {
    const Tables* tb; uint32_t sy, band_off, sstage, bars; unsigned char* stage; volatile int* abort_flag;
};

template <int D, bool INTERIOR>
__device__ __forceinline__ void fwd_tile(const FwdArgs& a, const FwdCtx& cx, const Tma& to, int bh, int b, int h, int g0,
                                         const Lane& L) {
    constexpr int RB = 2 * D, KS = D / 16;
    const int N = a.N, g = L.g, tig = L.tig;
    const int row_lo = g0 + g, row_hi = row_lo + 8;
    const float c2 = a.scale * kLog2e;
    const uint32_t tile_off = 16 * L.warp * RB;
    const size_t base = (size_t)bh * N * D;
    const __nv_bfloat16* qp = static_cast<const __nv_bfloat16*>(a.q) + base;
    // this thread's 16-byte chunk of row row_lo of K
    const __nv_bfloat16* kl = static_cast<const __nv_bfloat16*>(a.k) + base + (ptrdiff_t)row_lo * D + 8 * tig;
    const int2 nv = cx.tb->tile_nv[L.warp];
    const int n_valid = nv.x, n_full = nv.y;

    RowFrag<D> qa, qb;
    if (INTERIOR) {
        load_row_at(qa, qp + (size_t)row_lo * D + 8 * tig);
        load_row_at(qb, qp + (size_t)row_hi * D + 8 * tig);
    } else {
        load_row(qa, qp + (size_t)row_lo * D, tig, row_lo < N);
        load_row(qb, qp + (size_t)row_hi * D, tig, row_hi < N);
    }

    // ---- scores of the dense window: key row of n-tile nt for this thread is g0 - 32 + 8 nt + g
    float S[kNT][4];
    {
        const float* pb = cx.tb->pbx + kPbxLo + kWB + g - 2 * tig;
#pragma unroll
        for (int nt = 0; nt < kNT; ++nt) {
            S[nt][0] = pb[-8 * nt]; S[nt][1] = pb[-8 * nt - 1]; S[nt][2] = pb[8 - 8 * nt]; S[nt][3] = pb[7 - 8 * nt];
            RowFrag<D> kf;
            if (INTERIOR) {
                load_row_at(kf, kl + (8 * nt - kWB) * D);
            } else {
                const int kr = row_lo - kWB + 8 * nt;
                load_row(kf, kl + (ptrdiff_t)(8 * nt - kWB) * D - 8 * tig, tig, kr >= 0 && kr < N);
            }
            mma_rows(S[nt], qa, qb, kf);
        }
        if (!INTERIOR && g0 < kWB) {          // key rows before the sequence start
#pragma unroll
            for (int nt = 0; nt < kNT; ++nt)
#pragma unroll
                for (int r = 0; r < 4; ++r)
                    if (g0 - kWB + 8 * nt + 2 * tig + (r & 1) < 0) S[nt][r] = kNeg;
        }
    }

    // ---- scores of the sparse taps: tap 8 G + c lands in column c of T[G]
    float T[2][4];
#pragma unroll
    for (int G = 0; G < 2; ++G) {
        const int c0 = 8 * G + 2 * tig;
        const float i0 = __int_as_float(cx.tb->taps[c0].y), i1 = __int_as_float(cx.tb->taps[c0 + 1].y);
        T[G][0] = T[G][2] = c0 < n_valid ? i0 : kNeg;
        T[G][1] = T[G][3] = c0 + 1 < n_valid ? i1 : kNeg;
    }
    auto tap_score = [&](float (&acc)[4], float (&acc1)[4], int tp, int c, bool full) {
        const int dl = cx.tb->taps[tp].x;
        RowFrag<D> k0, k1;
        if (full) {
            load_row_at(k0, kl - (ptrdiff_t)dl * D);
            load_row_at(k1, kl - (ptrdiff_t)dl * D + 8 * D);
        } else {
            const int kr0 = row_lo - dl, kr1 = row_hi - dl;
            load_row(k0, kl - (ptrdiff_t)dl * D - 8 * tig, tig, kr0 >= 0 && kr0 < N);
            load_row(k1, kl - (ptrdiff_t)dl * D + 8 * D - 8 * tig, tig, kr1 >= 0 && kr1 < N);
        }
        const uint32_t sel = g == c ? kOnes : 0u;
#pragma unroll
        for (int kk = 0; kk < KS; ++kk) {
            const uint32_t h0 = mul_bf16x2(qa.r[2 * kk], k0.r[2 * kk]), h1 = mul_bf16x2(qb.r[2 * kk], k1.r[2 * kk]);
            const uint32_t h2 = mul_bf16x2(qa.r[2 * kk + 1], k0.r[2 * kk + 1]), h3 = mul_bf16x2(qb.r[2 * kk + 1], k1.r[2 * kk + 1]);
            if (kk & 1) mma16816(acc1, h0, h1, h2, h3, sel, sel); else mma16816(acc, h0, h1, h2, h3, sel, sel);
        }
    };
#pragma unroll
    for (int G = 0; G < 2; ++G) {
        float T1[4] = {0.f, 0.f, 0.f, 0.f};          // second accumulator: halves the dependent MMA chain
        const int n_fast = INTERIOR ? min(n_full - 8 * G, 8) : 0, cnt = min(n_valid - 8 * G, 8);
        int c = 0;
#pragma unroll 4
        for (; c < n_fast; ++c) tap_score(T[G], T1, 8 * G + c, c, true);
#pragma unroll 1
        for (; c < cnt; ++c) tap_score(T[G], T1, 8 * G + c, c, false);
#pragma unroll
        for (int r = 0; r < 4; ++r) T[G][r] += T1[r];
    }
    if (n_full < n_valid) {  // taps that reach only some rows of the tile
#pragma unroll
        for (int G = 0; G < 2; ++G)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int c = 8 * G + 2 * tig + e;
                const int dl = cx.tb->taps[c].x;
                if (c < n_valid && row_lo < dl) T[G][e] = kNeg;
                if (c < n_valid && row_hi < dl) T[G][2 + e] = kNeg;
            }
    }

    // ---- softmax over all taps of a row
    float m_lo = kMinM, m_hi = kMinM;
#pragma unroll
    for (int nt = 0; nt < kNT; ++nt) {
        m_lo = fmaxf(m_lo, fmaxf(S[nt][0], S[nt][1]));
        m_hi = fmaxf(m_hi, fmaxf(S[nt][2], S[nt][3]));
    }
#pragma unroll
    for (int G = 0; G < 2; ++G) {
        m_lo = fmaxf(m_lo, fmaxf(T[G][0], T[G][1]));
        m_hi = fmaxf(m_hi, fmaxf(T[G][2], T[G][3]));
    }
    m_lo = quad_max(m_lo) * c2; m_hi = quad_max(m_hi) * c2;          // log2 units from here on
    float l_lo = 0.f, l_hi = 0.f;
#pragma unroll
    for (int nt = 0; nt < kNT; ++nt) {
        S[nt][0] = ex2(fmaf(S[nt][0], c2, -m_lo)); S[nt][1] = ex2(fmaf(S[nt][1], c2, -m_lo));
        S[nt][2] = ex2(fmaf(S[nt][2], c2, -m_hi)); S[nt][3] = ex2(fmaf(S[nt][3], c2, -m_hi));
        l_lo += S[nt][0] + S[nt][1]; l_hi += S[nt][2] + S[nt][3];
    }
#pragma unroll
    for (int G = 0; G < 2; ++G) {
        T[G][0] = ex2(fmaf(T[G][0], c2, -m_lo)); T[G][1] = ex2(fmaf(T[G][1], c2, -m_lo));
        T[G][2] = ex2(fmaf(T[G][2], c2, -m_hi)); T[G][3] = ex2(fmaf(T[G][3], c2, -m_hi));
        l_lo += T[G][0] + T[G][1]; l_hi += T[G][2] + T[G][3];
    }

    // ---- O = P.V: dense window (V band rows 16 warp .. +47 of segment 0)
    const LaneAddr<D> la = lane_addr<D>(L.lane);
    mbar_wait(cx.bars, 0, cx.abort_flag, 0x201);
    float O[D / 8][4];
#pragma unroll
    for (int j = 0; j < D / 8; ++j) { O[j][0] = O[j][1] = O[j][2] = O[j][3] = 0.f; }
    const uint32_t vt = cx.sy + tile_off;
#pragma unroll
    for (int c = 0; c < kNT / 2; ++c) {
        const uint32_t a0 = pack_bf16x2(S[2 * c][0], S[2 * c][1]), a1 = pack_bf16x2(S[2 * c][2], S[2 * c][3]);
        const uint32_t a2 = pack_bf16x2(S[2 * c + 1][0], S[2 * c + 1][1]), a3 = pack_bf16x2(S[2 * c + 1][2], S[2 * c + 1][3]);
#pragma unroll
        for (int p = 0; p < KS; ++p) {
            uint32_t r[4];
            ldsm4t(r, vt + cx.band_off + c * 16 * RB + la.o[p]);
            mma16816(O[2 * p], a0, a1, a2, a3, r[0], r[1]);
            mma16816(O[2 * p + 1], a0, a1, a2, a3, r[2], r[3]);
        }
    }
    // ---- sparse taps: diag(p_tap) . V_tap
    uint32_t sel_lo, sel_hi;
    diag_selectors(g, tig, sel_lo, sel_hi);
    int cur = 0;
#pragma unroll
    for (int G = 0; G < 2; ++G) {
        const uint32_t w0 = pack_bf16x2(T[G][0], T[G][2]), w1 = pack_bf16x2(T[G][1], T[G][3]);
        const int cnt = min(n_valid - 8 * G, 8);
#pragma unroll 2
        for (int c = 0; c < cnt; ++c) {
            const int4 tp = cx.tb->taps[8 * G + c];
            if (tp.w != cur) { mbar_wait(cx.bars + 8 * tp.w, 0, cx.abort_flag, 0x202); cur = tp.w; }
            const uint32_t x = __shfl_sync(0xffffffffu, (c & 1) ? w1 : w0, (L.lane & ~3) | (c >> 1));
            diag_mma<D>(O, x, sel_lo, sel_hi, vt + tp.z, la);
        }
    }

    // ---- normalise, stage, store
    l_lo = quad_sum(l_lo); l_hi = quad_sum(l_hi);
    const float gain = a.head_gain ? a.head_gain[h] : 1.f;
    stage_acc<D>(cx.stage + tile_off, O, l_lo > 0.f ? __fdividef(gain, l_lo) : 0.f,
                 l_hi > 0.f ? __fdividef(gain, l_hi) : 0.f, g, tig);
    fence_proxy_async();
    __syncwarp();
    if (L.lane == 0) { to.store(cx.sstage + tile_off, g0, h, b); tma_store_commit(); }
    if (tig == 0) {
        if (INTERIOR || row_lo < N) a.lse[(size_t)bh * N + row_lo] = l_lo > 0.f ? (m_lo + __log2f(l_lo)) * kLn2 : -INFINITY;
        if (INTERIOR || row_hi < N) a.lse[(size_t)bh * N + row_hi] = l_hi > 0.f ? (m_hi + __log2f(l_hi)) * kLn2 : -INFINITY;
    }
    if (L.lane == 0) tma_store_wait_read();
}

template <int D>
__global__ void __launch_bounds__(kThreads, D == 32 ? 4 : 2)
fwd_staged_kernel(const FwdArgs a, const Taps t, const Plan pl, const Maps mf,
                  const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_o) {
    constexpr int RB = 2 * D;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const Smem<D> lay(pl.rows, 1, sizeof(Tables));
    const uint32_t sb = smem_u32(smem);
    Tables* tb = reinterpret_cast<Tables*>(smem + lay.tab);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + lay.misc);
    const uint32_t bars = sb + lay.bars;

    const Lane L;
    const int N = a.N, bh = blockIdx.y, b = bh / a.H, h = bh - b * a.H, n0 = blockIdx.x * kRows;
    const int n_last = min(n0 + kRows, N) - 1;
    const Tma tv{&map_v, mf.hf[0]}, to{&map_o, mf.hf[1]};
    int n_reach = 0;
    for (int i = 0; i < pl.n_seg; ++i) n_reach += pl.seg_reach[i] <= n_last;

    if (L.warp == 0) issue_copies<D>(pl, L.lane, n_reach, tv, sb + lay.y, bars, abort_flag, n0, h, b);
    fill_tables<D>(tb, a.pos_bias, t, pl, a.H, h, a.scale, n0, N);
    __syncthreads();     // tables and barrier initialisation visible to every warp

    const int g0 = n0 + 16 * L.warp;
    if (g0 < N) {
        FwdCtx cx;
        cx.tb = tb; cx.sy = sb + lay.y; cx.band_off = pl.band_row0 * RB; cx.sstage = sb + lay.stage; cx.bars = bars;
        cx.stage = smem + lay.stage; cx.abort_flag = abort_flag;
        if (g0 >= kWB && g0 + 16 <= N) fwd_tile<D, true>(a, cx, to, bh, b, h, g0, L);
        else fwd_tile<D, false>(a, cx, to, bh, b, h, g0, L);
    }
    // no copy of this block may still be in flight when its shared memory is released
    if (threadIdx.x == 0)
        for (int i = 0; i < n_reach; ++i) mbar_wait(bars + 8 * i, 0, abort_flag, 0x203);
}

// One thread waits on a barrier that nothing ever signals, with the given cycle limit: the wait
// gives up, records `site` in the error word and the kernel returns.  Used by the test of the
// bounded-wait path; no copy is in flight, nothing can hang.
__global__ void wait_timeout_kernel(long long limit_cycles, int site) {
    __shared__ __align__(8) unsigned long long bar;
    __shared__ int abort_flag;
    const uint32_t b = smem_u32(&bar);
    mbar_init(b, 1);
    abort_flag = 0;
    fence_mbar_init();
    mbar_wait(b, 0, &abort_flag, site, limit_cycles);
}

// ------------------------------------------------------------------------------ host side
}  // namespace

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
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

// bf16 tensor addressed as [batch][head][row][D] through element strides sb, sh, sn (rows of D
// contiguous elements).  The two middle dimensions are ordered by stride; *head_first tells the
// kernel which order the coordinates take.  box_rows consecutive rows of one head per copy.
bool make_map(CUtensorMap* m, bool* head_first, const void* ptr, int B, int H, int N, int D,
              long long sb, long long sh, long long sn, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const bool hf = sh < sn;
    *head_first = hf;
    cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)(hf ? H : N), (cuuint64_t)(hf ? N : H), (cuuint64_t)B};
    cuuint64_t strides[3] = {(cuuint64_t)(hf ? sh : sn) * 2, (cuuint64_t)(hf ? sn : sh) * 2, (cuuint64_t)sb * 2};
    cuuint32_t box[4] = {(cuuint32_t)D, hf ? 1u : (cuuint32_t)box_rows, hf ? (cuuint32_t)box_rows : 1u, 1u};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, D == 32 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
              CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool tensor_map_encoder_available() { return encode_fn() != nullptr; }

namespace {

// cudaFuncSetAttribute once per kernel and device is enough; `done` is that kernel's flag word.
template <typename K>
cudaError_t ensure_smem(K kernel, int bytes, unsigned long long* done) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    if (dev < 64 && (*done >> dev) & 1ull) return cudaSuccess;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
    if (e == cudaSuccess && dev < 64) *done |= 1ull << dev;
    (void)bytes;
    return e;
}

template <int D>
cudaError_t fwd_launch(const FwdArgs& a, const Taps& t, const Plan& pl, cudaStream_t s) {
    const Smem<D> lay(pl.rows, 1, sizeof(Tables));
    const int smem = lay.total + 1024;
    if (smem > kSmemLimit) return cudaErrorInvalidConfiguration;
    const long long sn = a.D, sh = (long long)a.N * a.D, sbt = (long long)a.H * a.N * a.D;
    CUtensorMap mv, mo;
    Maps mf = {};
    if (!make_map(&mv, &mf.hf[0], a.v, a.B, a.H, a.N, D, sbt, sh, sn, kRows) ||
        !make_map(&mo, &mf.hf[1], a.out, a.B, a.H, a.N, D, sbt, sh, sn, 16))
        return cudaErrorInvalidValue;
    static unsigned long long done = 0;
    cudaError_t e = ensure_smem(fwd_staged_kernel<D>, smem, &done);
    if (e != cudaSuccess) return e;
    dim3 grid((a.N + kRows - 1) / kRows, a.B * a.H);
    fwd_staged_kernel<D><<<grid, kThreads, smem, s>>>(a, t, pl, mf, mv, mo);
    return cudaGetLastError();
}

}  // namespace
}  // namespace stg

bool staged_supported(int dtype, int D, const Taps& t, bool has_scale_embed) {
    if (dtype != DSQG_DTYPE_BF16 || (D != 32 && D != 64) || has_scale_embed) return false;
    stg::Plan pl;
    if (!stg::build_plan(t, false, &pl)) return false;
    // two staged tensors of pl.rows rows at most, staging tiles, tables
    if ((size_t)2 * pl.rows * 2 * D + 2 * stg::kRows * 2 * D + 8192 > (size_t)stg::kSmemLimit) return false;
    return stg::encode_fn() != nullptr;
}

cudaError_t launch_fwd_staged(const FwdArgs& a, const Taps& t, cudaStream_t s) {
    stg::Plan pl;
    if (!stg::build_plan(t, false, &pl)) return cudaErrorInvalidValue;
    return a.D == 32 ? stg::fwd_launch<32>(a, t, pl, s) : stg::fwd_launch<64>(a, t, pl, s);
}

cudaError_t launch_wait_timeout(long long limit_cycles, int site, cudaStream_t s) {
    stg::wait_timeout_kernel<<<1, 1, 0, s>>>(limit_cycles, site);
    return cudaGetLastError();
}

cudaError_t read_stage_error(int* value, bool reset) {
    cudaError_t e = cudaMemcpyFromSymbol(value, stg::g_stage_error, sizeof(int));
    if (e == cudaSuccess && reset && *value != 0) {
        const int zero = 0;
        e = cudaMemcpyToSymbol(stg::g_stage_error, &zero, sizeof(int));
    }
    return e;
}

}  // namespace dsqg
