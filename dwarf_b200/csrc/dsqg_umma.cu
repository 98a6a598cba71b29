// DSQG forward with the dense window on the 5th-generation tensor cores (tcgen05.mma, accumulators
// in tensor memory, operands staged by the copy engine), bf16, D = 32 or 64, sm_100a.  Kernel path 4
// (dsqg_set_kernel_path(4)); not chosen automatically.
//
// Reference math: kernels/dsqg_attention_v3.py:60-163 (scores, bias, causal mask, softmax over the
// taps, weighted sum of the value rows) without scale_embed.
//
// One persistent thread block per SM walks a contiguous range of 128-row tiles, three tiles in flight
// (tile j uses tensor-memory slot j % 3, a 160-column third of the SM's 512 columns, softmax group
// j % 3, and one of the Q / K-band / V-band buffers in shared memory):
//   copy warp (one lane):  Q[128 x D], the key band K[n0-32, n0+128) and the value band of a tile into
//       a free buffer (cp.async.bulk.tensor; rows outside the sequence arrive as zeros);
//   S warp (one lane):     S = Q . Kband^T   (tcgen05.mma M 128, N 160, K 16 per step) -> slot columns [0, 160)
//   softmax group (4 warps, one thread per query row = tensor-memory lane): reads its row's 64-column
//       window of S (tcgen05.ld), adds the bias / mask table, takes the row maximum and the
//       exponentials, writes P as bf16 pairs over S (tcgen05.st: the A operand of the second product;
//       zero outside the row's window), [runs the sparse taps, see Half / fold_tap], reads O, scales by
//       gain / sum and stores the row;
//   O warp (one lane):     O = P . Vband     (M 128, N D, K 16 per step, A from tensor memory, B MN-major
//       from shared memory) -> the last D columns of the slot, dead once S has been read.
// Every hand-over is an mbarrier: copies -> S warp (full), tcgen05.commit -> softmax (S ready), softmax ->
// O warp (P written), commit -> softmax (O ready) and -> copy warp (buffer free), softmax -> S warp (O read).
// Row r of warp w (r = 32 w + l) needs band columns c = r + 32 - delta, delta = 0..32, i.e.
// c - 32 w in [l, l + 32]: a window of 64 columns per warp holds them, and the bias/mask table
// Bm[l][c - 32 w] (pos_bias[delta, h] * log2 e inside the window, "minus infinity" outside) is
// the same for every warp and tile of a head.
//
// Every wait on a barrier is bounded (stg::mbar_wait): a wait that gives up sets the block's
// abort flag and the device error word, every other wait of the block returns at once, tensor
// memory is released and the kernel ends.
#include <cuda.h>
#include <cuda_bf16.h>

#include <mutex>

#include "dsqg_common.cuh"
#include "dsqg_stage.cuh"

namespace dsqg {
namespace umma {

using namespace stg;

constexpr int kTM = 128;                 // query rows per tile (= tensor-memory lanes)
constexpr int kBand = kTM + kWB;         // key rows of the dense window of a tile: 160
constexpr int kThreads = 480;            // 3 softmax groups of 4 warps + two MMA issuer warps + copy warp
constexpr int kTmemCols = 512;           // three slots of 160 columns
constexpr int kBmPitch = 68;             // floats per row of the bias/mask table (64 + 4: conflict-free float4 reads)

// ---- tcgen05 / tensor memory
__device__ __forceinline__ void tmem_alloc(uint32_t slot, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// D[tmem] (+)= A[smem] . B[smem], bf16 operands, fp32 accumulation; issued by one thread.
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// The same with A read from tensor memory (bf16 pairs per 32-bit column, lane = row).
__device__ __forceinline__ void umma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// 16 consecutive 32-bit columns of this thread's tensor-memory lane.
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// The barrier gets one arrival when every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Non-blocking test of a barrier phase (try_wait may suspend the thread for a while before it answers).
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}

// 32 consecutive fp32 columns of this thread's tensor-memory lane.
__device__ __forceinline__ void tmem_ld32(float (&v)[32], uint32_t taddr) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory operand descriptor: 128-byte-swizzled (layout 2) or 64-byte-swizzled (layout 4)
// tile whose 8-row groups are `sbo` bytes apart.  The leading-dimension offset is not used by the
// swizzled layouts of one atom width; bits 46-47 carry the descriptor version of this architecture.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t sbo, uint32_t layout) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(sbo >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)layout << 61);
}
// Instruction descriptor: fp32 accumulator, bf16 A and B, A K-major, B K-major or MN-major.
__host__ __device__ constexpr uint32_t instr_desc(int M, int N, bool b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(N >> 3) << 17) |
           ((uint32_t)(M >> 4) << 24);
}

constexpr int kSlots = 3;                // tiles in flight per thread block = softmax warp groups = tensor-memory slots
constexpr int kMaxBufs = 2 * kSlots;     // Q / K-band / V-band buffers in shared memory: six at D = 32, three at D = 64
constexpr int kSlotCols = 160;           // tensor-memory columns per slot: S [0,160), then P over [0,80) and O over [128,160)

constexpr int kMaxSparse = 16;           // sparse taps a tile can take (kernel path 4)

// SP: the offset set has sparse taps; the softmax warps then also run them (register-fed MMAs on row
// fragments read from global memory) and hand their partial results to the row threads through a
// per-warp scratch tile.
template <int D, bool SP>
struct Layout {
    static constexpr int bufs = D == 32 ? (SP ? 4 : kMaxBufs) : kSlots;
    static constexpr int row_bytes = 2 * D;                       // 64 / 128: one swizzle atom wide
    static constexpr int swizzle = D == 32 ? 4 : 2;               // descriptor layout code: 64-byte / 128-byte swizzle
    static constexpr int sbo = 8 * row_bytes;                     // distance of 8-row groups
    static constexpr int o_col = kSlotCols - D;                   // O occupies the last D columns of a slot (P ends at 80)
    static constexpr int q_bytes = kTM * row_bytes;               // 8 / 16 KB
    static constexpr int band_bytes = kBand * row_bytes;          // 10 / 20 KB
    static constexpr int buf_bytes = q_bytes + 2 * band_bytes;    // 28 / 56 KB: Q | K band | V band
    static constexpr int bm0 = bufs * buf_bytes;
    static constexpr int bm_bytes = 32 * kBmPitch * 4 + kMaxSparse * 8;      // bias/mask table | sparse taps {offset, bias}
    static constexpr int sp_pitch = D + 4;                        // floats per scratch row: D partial sums, maximum, sum
    static constexpr int sp_bytes = SP ? 32 * sp_pitch * 4 : 0;   // per softmax warp
    static constexpr int sp0 = bm0 + kSlots * bm_bytes;
    static constexpr int bars0 = sp0 + 4 * kSlots * sp_bytes;
    static constexpr int total = bars0 + 256;
};

// State of one 16-row half of a warp's rows during the sparse taps (rows g and g+8 per lane).
template <int D>
struct Half {
    RowFrag<D> qa, qb;
    float m_lo, m_hi, ms_lo, ms_hi, l_lo, l_hi;
    float O[D / 8][4];
};

// One sparse tap into the running softmax of a half: x0 / x1 are the scores of rows g / g+8 (valid on
// the lane that owns the diagonal entry), vf0 / vf1 the value rows they weight.
template <int D>
__device__ __forceinline__ void fold_tap(Half<D>& hf, const Lane& L, float x0, float x1, const RowFrag<D>& vf0,
                                         const RowFrag<D>& vf1) {
    if (__any_sync(0xffffffffu, x0 > hf.ms_lo + kSlack || x1 > hf.ms_hi + kSlack)) {
        const float mn_lo = fmaxf(hf.m_lo, __shfl_sync(0xffffffffu, x0, L.owner_lane));
        const float mn_hi = fmaxf(hf.m_hi, __shfl_sync(0xffffffffu, x1, L.owner_lane));
        const float al_lo = ex2(hf.m_lo - mn_lo), al_hi = ex2(hf.m_hi - mn_hi);
        hf.m_lo = mn_lo; hf.m_hi = mn_hi;
        hf.ms_lo = L.owner ? mn_lo : 1.0e30f; hf.ms_hi = L.owner ? mn_hi : 1.0e30f;
        hf.l_lo *= al_lo; hf.l_hi *= al_hi;
#pragma unroll
        for (int j = 0; j < D / 8; ++j) { hf.O[j][0] *= al_lo; hf.O[j][1] *= al_lo; hf.O[j][2] *= al_hi; hf.O[j][3] *= al_hi; }
    }
    const float p0 = ex2(x0 - hf.ms_lo), p1 = ex2(x1 - hf.ms_hi);       // exactly 0 on lanes that own no diagonal entry
    hf.l_lo += p0; hf.l_hi += p1;
    diag_fma<D>(hf.O, __shfl_sync(0xffffffffu, p0, L.owner_lane), __shfl_sync(0xffffffffu, p1, L.owner_lane), vf0, vf1);
}

// barrier slots (8 bytes each) behind the tables
enum { kBarFull = 0, kBarEmpty = kBarFull + kMaxBufs, kBarS = kBarEmpty + kMaxBufs, kBarP = kBarS + kSlots,
       kBarO = kBarP + kSlots, kBarORead = kBarO + kSlots, kNumBars = kBarORead + kSlots };

template <int D, bool SP>
__global__ void __launch_bounds__(kThreads, 1)
fwd_umma_kernel(const FwdArgs a, const Taps t, int tiles_per_seq, int n_tiles,
                const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v) {
    static_assert(D == 32 || D == 64, "a row is one 64-byte or 128-byte swizzle atom");
    static_assert(!SP || D == 32, "the scratch tiles of the sparse taps fit next to the operand buffers at D = 32 only");
    using Lay = Layout<D, SP>;
    constexpr int kBufs = Lay::bufs, kOCol = Lay::o_col;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t sb = smem_u32(smem);
    const uint32_t bars = sb + Lay::bars0;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + Lay::bars0 + 8 * kNumBars);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + Lay::bars0 + 8 * kNumBars + 8);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int N = a.N, H = a.H;
    const long long tile_lo = (long long)blockIdx.x * n_tiles / gridDim.x;
    const long long tile_hi = (long long)(blockIdx.x + 1) * n_tiles / gridDim.x;
    const int my_tiles = (int)(tile_hi - tile_lo);
    constexpr int kProducerWarp = 4 * kSlots, kOWarp = kProducerWarp + 1, kCopyWarp = kProducerWarp + 2;

    // ---- one-time setup: barriers, tensor memory
    if (tid == 0) {
        *abort_flag = 0;
        for (int i = 0; i < kBufs; ++i) { mbar_init(bars + 8 * (kBarFull + i), 1); mbar_init(bars + 8 * (kBarEmpty + i), 1); }
        for (int i = 0; i < kSlots; ++i) {
            mbar_init(bars + 8 * (kBarS + i), 1); mbar_init(bars + 8 * (kBarP + i), kTM);
            mbar_init(bars + 8 * (kBarO + i), 1); mbar_init(bars + 8 * (kBarORead + i), kTM);
        }
        fence_mbar_init();
    }
    if (warp == kProducerWarp) {
        if (lane == 0) { prefetch_tensormap(&map_q); prefetch_tensormap(&map_k); prefetch_tensormap(&map_v); }
        __syncwarp();
        tmem_alloc(smem_u32(tmem_slot), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == kCopyWarp) {
        // ================================================================= copies: Q, key band, value band of tile j -> buffer j % 6
        if (lane == 0) {
            int bh = (int)(tile_lo / tiles_per_seq), nt = (int)(tile_lo % tiles_per_seq);
            int b = bh / H, h = bh % H, j = 0;
            for (; j < my_tiles; ++j) {
                const int buf = j % kBufs;
                // the buffer comes back when O of the tile six before this one has completed
                if (j >= kBufs && !mbar_wait(bars + 8 * (kBarEmpty + buf), ((j - kBufs) / kBufs) & 1, abort_flag, 0x401)) break;
                const uint32_t bar = bars + 8 * (kBarFull + buf), dst = sb + buf * Lay::buf_bytes;
                const int n0 = nt * kTM;
                mbar_arrive_expect_tx(bar, Lay::buf_bytes);
                tma_load(dst, &map_q, bar, n0, h, b);
                tma_load(dst + Lay::q_bytes, &map_k, bar, n0 - kWB, h, b);
                tma_load(dst + Lay::q_bytes + Lay::band_bytes, &map_v, bar, n0 - kWB, h, b);
                if (++nt == tiles_per_seq) { nt = 0; if (++h == H) { h = 0; ++b; } }
            }
            // after an abort: no copy of this block may be in flight when its shared memory is released
            if (*abort_flag)
                for (int i = j > kBufs ? j - kBufs : 0; i < j; ++i) mbar_wait(bars + 8 * (kBarFull + i % kBufs), (i / kBufs) & 1, abort_flag, 0x404);
        }
        __syncwarp();
    } else if (warp == kProducerWarp) {
        // ================================================================= issuer of S(j) = Q(j) . Kband(j)^T
        // S(j) needs its operands in shared memory and its slot back from tile j - 3 (O read by the softmax group).
        if (lane == 0) {
            constexpr uint32_t kIdS = instr_desc(kTM, kBand, false);
            const uint64_t desc0 = smem_desc(sb, Lay::sbo, Lay::swizzle);       // tiles differ in the start-address field only (16-byte units)
            for (int j = 0; j < my_tiles; ++j) {
                const int slot = j % kSlots, buf = j % kBufs;
                if (!mbar_wait(bars + 8 * (kBarFull + buf), (j / kBufs) & 1, abort_flag, 0x402)) break;
                if (j >= kSlots && !mbar_wait(bars + 8 * (kBarORead + slot), ((j - kSlots) / kSlots) & 1, abort_flag, 0x405)) break;
                tc_fence_after();
                const uint64_t dq = desc0 + (uint32_t)((buf * Lay::buf_bytes) >> 4), dk = dq + (uint32_t)(Lay::q_bytes >> 4);
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk)
                    umma_bf16(tmem + kSlotCols * slot, dq + 2 * kk, dk + 2 * kk, kIdS, kk > 0);
                umma_commit(bars + 8 * (kBarS + slot));
            }
        }
        __syncwarp();
    } else if (warp == kOWarp) {
        // ================================================================= issuer of O(j) = P(j) . Vband(j)
        // P: 16 bf16 = 8 columns of tensor memory per step.  The second commit hands the shared-memory buffer back.
        if (lane == 0) {
            constexpr uint32_t kIdO = instr_desc(kTM, D, true);
            const uint64_t desc0 = smem_desc(sb, Lay::sbo, Lay::swizzle);
            for (int j = 0; j < my_tiles; ++j) {
                const int slot = j % kSlots, buf = j % kBufs;
                if (!mbar_wait(bars + 8 * (kBarP + slot), (j / kSlots) & 1, abort_flag, 0x403)) break;
                tc_fence_after();
                const uint32_t tS = tmem + kSlotCols * slot;
                const uint64_t dv = desc0 + (uint32_t)((buf * Lay::buf_bytes + Lay::q_bytes + Lay::band_bytes) >> 4);
#pragma unroll
                for (int kk = 0; kk < kBand / 16; ++kk)
                    umma_bf16_ts(tS + kOCol, tS + 8 * kk, dv + (uint32_t)((kk * 16 * Lay::row_bytes) >> 4), kIdO, kk > 0);
                umma_commit(bars + 8 * (kBarO + slot));
                umma_commit(bars + 8 * (kBarEmpty + buf));
            }
        }
        __syncwarp();
    } else {
        // ================================================================= softmax groups: thread = query row
        const int grp = warp >> 2, wq = warp & 3, r = tid & (kTM - 1), l = lane;
        float* Bm = reinterpret_cast<float*>(smem + Lay::bm0 + grp * Lay::bm_bytes);
        int2* tap_s = reinterpret_cast<int2*>(smem + Lay::bm0 + grp * Lay::bm_bytes + 32 * kBmPitch * 4);
        float* scratch = reinterpret_cast<float*>(smem + Lay::sp0 + warp * Lay::sp_bytes);
        const uint32_t tS = tmem + kSlotCols * grp + ((uint32_t)(32 * wq) << 16);
        const float c2 = a.scale * kLog2e;
        const int d_lo = t.d_lo, d_hi = t.d_lo + t.n_dense - 1;
        int cur_h = -1;
        for (int j = grp, k = 0; j < my_tiles; j += kSlots, ++k) {
            const long long tile = tile_lo + j;
            const int bh = (int)(tile / tiles_per_seq), n0 = (int)(tile % tiles_per_seq) * kTM;
            const int h = bh % H, n = n0 + r;
            if (h != cur_h) {
                asm volatile("bar.sync %0, 128;" ::"r"(1 + grp) : "memory");
            for (int e = r; e < 32 * 64; e += kTM) {
                    const int ll = e >> 6, cc = e & 63, delta = ll + 32 - cc;
                    Bm[ll * kBmPitch + cc] = (delta >= d_lo && delta <= d_hi) ? a.pos_bias[(delta - d_lo) * H + h] * kLog2e : kNeg;
                }
                if (SP && r < t.n_sparse)
                    tap_s[r] = make_int2(t.sparse[r], __float_as_int(a.pos_bias[(t.n_dense + r) * H + h] * kLog2e));
                asm volatile("bar.sync %0, 128;" ::"r"(1 + grp) : "memory");
                cur_h = h;
            }
            if (!__all_sync(0xffffffffu, mbar_wait(bars + 8 * (kBarS + grp), k & 1, abort_flag, 0x411))) break;
            tc_fence_after();
            float z[64];
            {
                float x0[32], x1[32];
                tmem_ld32(x0, tS + 32 * wq);
                tmem_ld32(x1, tS + 32 * wq + 32);
                tmem_wait_ld();
                const float4* brow = reinterpret_cast<const float4*>(Bm + l * kBmPitch);
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const float4 b0 = brow[c], b1 = brow[8 + c];
                    z[4 * c + 0] = fmaf(x0[4 * c + 0], c2, b0.x); z[4 * c + 1] = fmaf(x0[4 * c + 1], c2, b0.y);
                    z[4 * c + 2] = fmaf(x0[4 * c + 2], c2, b0.z); z[4 * c + 3] = fmaf(x0[4 * c + 3], c2, b0.w);
                    z[32 + 4 * c + 0] = fmaf(x1[4 * c + 0], c2, b1.x); z[32 + 4 * c + 1] = fmaf(x1[4 * c + 1], c2, b1.y);
                    z[32 + 4 * c + 2] = fmaf(x1[4 * c + 2], c2, b1.z); z[32 + 4 * c + 3] = fmaf(x1[4 * c + 3], c2, b1.w);
                }
            }
            if (n0 == 0 && wq == 0) {            // band columns 0..31 of the first tile are key rows -32..-1
#pragma unroll
                for (int c = 0; c < 32; ++c) z[c] = kNeg;
            }
            float m4[4] = {kNeg, kNeg, kNeg, kNeg};
#pragma unroll
            for (int c = 0; c < 64; c += 4) {
                m4[0] = fmaxf(m4[0], z[c]); m4[1] = fmaxf(m4[1], z[c + 1]);
                m4[2] = fmaxf(m4[2], z[c + 2]); m4[3] = fmaxf(m4[3], z[c + 3]);
            }
            const float m_raw = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
            const float m = m_raw < kMinM ? 0.f : m_raw;      // a row without a valid tap: every p becomes 0
            // P (bf16 pairs) replaces S in tensor memory: band column c sits in 32-bit column c / 2, so the
            // row's window is columns 16 wq .. 16 wq + 31 of the 80; the other 48 are zeroed
            float s4[4] = {0.f, 0.f, 0.f, 0.f};
            uint32_t pw[2][16];
#pragma unroll
            for (int c = 0; c < 32; ++c) {
                const float p0 = ex2(z[2 * c] - m), p1 = ex2(z[2 * c + 1] - m);
                s4[c & 3] += p0 + p1;
                pw[c >> 4][c & 15] = pack_bf16x2(p0, p1);
            }
            const float lsum = (s4[0] + s4[1]) + (s4[2] + s4[3]);
            {
                const uint32_t zero[16] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
#pragma unroll
                for (int ch = 0; ch < kBand / 32; ++ch) {
                    if (ch == wq) tmem_st16(tS + 16 * ch, pw[0]);
                    else if (ch == wq + 1) tmem_st16(tS + 16 * ch, pw[1]);
                    else tmem_st16(tS + 16 * ch, zero);
                }
            }
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(bars + 8 * (kBarP + grp));

            if constexpr (SP) {
                // ---- sparse taps of the warp's two 16-row halves while the tensor cores form O: the default
                // kernels' scheme (dsqg_mma.cu): Q and the tap's key rows as row fragments, the 16 x 16 score
                // tile by mma.sync, its diagonal into an online softmax, P.V as a diagonal update.  The
                // running maximum of a row starts at its dense-window maximum.
                const Lane L;
                const size_t seq = (size_t)bh * N * D;
                const __nv_bfloat16* qg = static_cast<const __nv_bfloat16*>(a.q) + seq;
                const __nv_bfloat16* kg = static_cast<const __nv_bfloat16*>(a.k) + seq + 8 * L.tig;
                const __nv_bfloat16* vg = static_cast<const __nv_bfloat16*>(a.v) + seq + 8 * L.tig;
                const int gw = n0 + 32 * wq;                  // first row of the warp
                Half<D> hs[2];
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    const int row_lo = gw + 16 * hh + L.g, row_hi = row_lo + 8;
                    load_row(hs[hh].qa, qg + (size_t)row_lo * D, L.tig, row_lo < N);
                    load_row(hs[hh].qb, qg + (size_t)row_hi * D, L.tig, row_hi < N);
                    hs[hh].m_lo = fmaxf(__shfl_sync(0xffffffffu, m_raw, 16 * hh + L.g), kMinM);
                    hs[hh].m_hi = fmaxf(__shfl_sync(0xffffffffu, m_raw, 16 * hh + L.g + 8), kMinM);
                    hs[hh].ms_lo = L.owner ? hs[hh].m_lo : 1.0e30f; hs[hh].ms_hi = L.owner ? hs[hh].m_hi : 1.0e30f;
                    hs[hh].l_lo = 0.f; hs[hh].l_hi = 0.f;
#pragma unroll
                    for (int jj = 0; jj < D / 8; ++jj) { hs[hh].O[jj][0] = 0.f; hs[hh].O[jj][1] = 0.f; hs[hh].O[jj][2] = 0.f; hs[hh].O[jj][3] = 0.f; }
                }
                const int ns = t.n_sparse;
#pragma unroll 1
                for (int si = 0; si < ns; ++si) {
                    const int2 tp = tap_s[si];
                    const int delta = tp.x;
                    const float pbv = __int_as_float(tp.y);
                    if (gw + 31 < delta) break;                  // taps ascend: no row of the warp reaches back that far
                    if (gw >= delta && gw + 32 <= N) {
                        // all 32 key rows exist: no predicates, the eight row loads in flight together
                        const __nv_bfloat16* kp = kg + (ptrdiff_t)(gw + L.g - delta) * D;
                        const __nv_bfloat16* vp = vg + (ptrdiff_t)(gw + L.g - delta) * D;
                        RowFrag<D> kf[4], vf[4];
#pragma unroll
                        for (int q4 = 0; q4 < 4; ++q4) { load_row_at(kf[q4], kp + 8 * q4 * D); load_row_at(vf[q4], vp + 8 * q4 * D); }
#pragma unroll
                        for (int hh = 0; hh < 2; ++hh) {
                            float s0[4], s1[4];
                            mma_rows_z(s0, hs[hh].qa, hs[hh].qb, kf[2 * hh]);
                            mma_rows_z(s1, hs[hh].qa, hs[hh].qb, kf[2 * hh + 1]);
                            const float d0 = (L.g & 1) ? s0[1] : s0[0], d1 = (L.g & 1) ? s1[3] : s1[2];
                            fold_tap(hs[hh], L, fmaf(d0, c2, pbv), fmaf(d1, c2, pbv), vf[2 * hh], vf[2 * hh + 1]);
                        }
                    } else {
#pragma unroll
                        for (int hh = 0; hh < 2; ++hh) {
                            const int g0 = gw + 16 * hh;
                            if (g0 + 15 < delta || g0 >= N) continue;
                            const int kr0 = g0 + L.g - delta, kr1 = kr0 + 8;
                            const bool v0 = kr0 >= 0 && kr0 < N, v1 = kr1 >= 0 && kr1 < N;
                            RowFrag<D> kf0, kf1, vf0, vf1;
                            load_row(kf0, kg + (ptrdiff_t)kr0 * D - 8 * L.tig, L.tig, v0);
                            load_row(kf1, kg + (ptrdiff_t)kr1 * D - 8 * L.tig, L.tig, v1);
                            load_row(vf0, vg + (ptrdiff_t)kr0 * D - 8 * L.tig, L.tig, v0);
                            load_row(vf1, vg + (ptrdiff_t)kr1 * D - 8 * L.tig, L.tig, v1);
                            float s0[4], s1[4];
                            mma_rows_z(s0, hs[hh].qa, hs[hh].qb, kf0);
                            mma_rows_z(s1, hs[hh].qa, hs[hh].qb, kf1);
                            const float d0 = (L.g & 1) ? s0[1] : s0[0], d1 = (L.g & 1) ? s1[3] : s1[2];
                            fold_tap(hs[hh], L, v0 ? fmaf(d0, c2, pbv) : kNeg, v1 ? fmaf(d1, c2, pbv) : kNeg, vf0, vf1);
                        }
                    }
                }
                // partial sums, maximum and sum of each row to the row's thread through the warp's scratch tile
                // (accumulator tile 4 c + i, columns 2 tig, 2 tig + 1 = elements 32 c + 8 tig + 2 i, + 1)
                __syncwarp();
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    float* lo = scratch + (16 * hh + L.g) * Lay::sp_pitch;
                    float* hi = lo + 8 * Lay::sp_pitch;
#pragma unroll
                    for (int jj = 0; jj < D / 8; ++jj) {
                        const int col = 32 * (jj >> 2) + 8 * L.tig + 2 * (jj & 3);
                        *reinterpret_cast<float2*>(lo + col) = make_float2(hs[hh].O[jj][0], hs[hh].O[jj][1]);
                        *reinterpret_cast<float2*>(hi + col) = make_float2(hs[hh].O[jj][2], hs[hh].O[jj][3]);
                    }
                    const float sl = quad_sum(hs[hh].l_lo), sh = quad_sum(hs[hh].l_hi);
                    if (L.tig == 0) {
                        *reinterpret_cast<float2*>(lo + D) = make_float2(hs[hh].m_lo, sl);
                        *reinterpret_cast<float2*>(hi + D) = make_float2(hs[hh].m_hi, sh);
                    }
                }
                __syncwarp();
            }

            if (!__all_sync(0xffffffffu, mbar_wait(bars + 8 * (kBarO + grp), k & 1, abort_flag, 0x412))) break;
            tc_fence_after();
            float o[D];
#pragma unroll
            for (int c = 0; c < D / 32; ++c) tmem_ld32(*reinterpret_cast<float(*)[32]>(o + 32 * c), tS + kOCol + 32 * c);
            tmem_wait_ld();
            tc_fence_before();
            mbar_arrive(bars + 8 * (kBarORead + grp));       // the slot may take the next tile's S
            float m_out = m, l_out = lsum;
            if constexpr (SP) {
                // this row's sparse partials: weights relative to ms >= the dense maximum
                const float* row = scratch + l * Lay::sp_pitch;
                const float2 st = *reinterpret_cast<const float2*>(row + D);
                const float ad = lsum > 0.f ? ex2(m - st.x) : 0.f;
#pragma unroll
                for (int c = 0; c < D / 4; ++c) {
                    const float4 sp4 = *reinterpret_cast<const float4*>(row + 4 * c);
                    o[4 * c + 0] = fmaf(o[4 * c + 0], ad, sp4.x); o[4 * c + 1] = fmaf(o[4 * c + 1], ad, sp4.y);
                    o[4 * c + 2] = fmaf(o[4 * c + 2], ad, sp4.z); o[4 * c + 3] = fmaf(o[4 * c + 3], ad, sp4.w);
                }
                m_out = st.x; l_out = fmaf(lsum, ad, st.y);
            }
            if (n < N) {
                const float gain = a.head_gain ? a.head_gain[h] : 1.f;
                const float sc = l_out > 0.f ? __fdividef(gain, l_out) : 0.f;
                uint4* dst = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(a.out) + ((size_t)bh * N + n) * D);
#pragma unroll
                for (int c = 0; c < D / 8; ++c)
                    dst[c] = make_uint4(pack_bf16x2(o[8 * c] * sc, o[8 * c + 1] * sc), pack_bf16x2(o[8 * c + 2] * sc, o[8 * c + 3] * sc),
                                        pack_bf16x2(o[8 * c + 4] * sc, o[8 * c + 5] * sc), pack_bf16x2(o[8 * c + 6] * sc, o[8 * c + 7] * sc));
                a.lse[(size_t)bh * N + n] = l_out > 0.f ? (m_out + __log2f(l_out)) * kLn2 : -INFINITY;
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == kProducerWarp) tmem_dealloc(tmem, kTmemCols);
}

}  // namespace umma

cudaError_t read_umma_error(int* value, bool reset) {
    cudaError_t e = cudaMemcpyFromSymbol(value, stg::g_stage_error, sizeof(int));
    if (e == cudaSuccess && reset && *value != 0) {
        const int zero = 0;
        e = cudaMemcpyToSymbol(stg::g_stage_error, &zero, sizeof(int));
    }
    return e;
}

bool umma_supported(int dtype, int D, const Taps& t, bool has_scale_embed) {
    return dtype == DSQG_DTYPE_BF16 && (D == 32 || (D == 64 && t.n_sparse == 0)) && !has_scale_embed &&
           t.n_sparse <= umma::kMaxSparse &&
           t.d_lo + t.n_dense - 1 <= stg::kWB && stg::tensor_map_encoder_available();
}

namespace umma {
template <int D, bool SP>
cudaError_t fwd_launch(const FwdArgs& a, const Taps& t, cudaStream_t s) {
    const long long sn = D, sh = (long long)a.N * D, sbt = (long long)a.H * a.N * D;
    CUtensorMap mq, mk, mv;
    bool hf = false;
    if (!stg::make_map(&mq, &hf, a.q, a.B, a.H, a.N, D, sbt, sh, sn, kTM) || hf ||
        !stg::make_map(&mk, &hf, a.k, a.B, a.H, a.N, D, sbt, sh, sn, kBand) || hf ||
        !stg::make_map(&mv, &hf, a.v, a.B, a.H, a.N, D, sbt, sh, sn, kBand) || hf)
        return cudaErrorInvalidValue;
    const int smem = Layout<D, SP>::total + 1024;
    int dev = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    static std::mutex mu;
    static int attr_done[64] = {0}, sm_count[64] = {0};
    {
        std::lock_guard<std::mutex> lock(mu);
        if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
        if (!attr_done[dev]) {
            if ((e = cudaFuncSetAttribute(fwd_umma_kernel<D, SP>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)) != cudaSuccess) return e;
            if ((e = cudaDeviceGetAttribute(&sm_count[dev], cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return e;
            attr_done[dev] = 1;
        }
        sms = sm_count[dev];
    }
    const int tiles_per_seq = (a.N + kTM - 1) / kTM;
    const long long n_tiles = (long long)a.B * a.H * tiles_per_seq;
    if (n_tiles > 0x7fffffffLL) return cudaErrorInvalidValue;
    const int grid = (int)(n_tiles < (long long)sms ? n_tiles : (long long)sms);
    fwd_umma_kernel<D, SP><<<grid, kThreads, smem, s>>>(a, t, tiles_per_seq, (int)n_tiles, mq, mk, mv);
    return cudaGetLastError();
}
}  // namespace umma

cudaError_t launch_fwd_umma(const FwdArgs& a, const Taps& t, cudaStream_t s) {
    if (a.strided) return cudaErrorInvalidValue;
    if (a.D == 32) return t.n_sparse ? umma::fwd_launch<32, true>(a, t, s) : umma::fwd_launch<32, false>(a, t, s);
    if (a.D == 64 && t.n_sparse == 0) return umma::fwd_launch<64, false>(a, t, s);
    return cudaErrorInvalidValue;
}

}  // namespace dsqg
