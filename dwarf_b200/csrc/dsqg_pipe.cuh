// Producer/consumer pipeline shared by the persistent backward kernels (sm_100a).
//
// Row stream, ring, stages and barrier numbering are those of the forward kernel
// (dsqg_fwd_tma.cu), generalised in two ways:
//   * an "own" stage holds NOWN 128-row tiles of the block being worked on (dQ: Q and dO;
//     dK/dV: K and V), the ring and the far stages hold two tensors (dQ: K,V; dK/dV: Q,dO);
//   * AHEAD = false: a tile of own block j looks BACK over ring blocks (dQ, like the forward);
//     AHEAD = true : it looks AHEAD (dK/dV: key row m is read by query rows m+delta).
// In both cases own block j needs ring blocks r = j .. j+look, with
//   AHEAD = false: ring block r is stream block G_begin - look + r  (own block = newest, r = j+look)
//   AHEAD = true : ring block r is stream block G_begin + r         (own block = oldest, r = j)
// so waits, releases and phases are identical; only the block mapping and the sign of the
// tap offset differ.
#pragma once

#include "dsqg_tma.cuh"

namespace dsqg {
namespace pipe {

constexpr int kBlockRows = 128;
constexpr int kTilesPerBlock = kBlockRows / 16;
constexpr int kMaxRingBlocks = 16;
constexpr int kMaxFarStages = 8;
constexpr int kMaxOwnStages = 4;
constexpr int kSmemLimit = 227 * 1024;

struct Plan {
    int nrb;             // ring blocks (power of two)
    int look;            // ring blocks a tile reads besides its own (window taps: delta <= 128*look)
    int n_win, n_far;    // sparse taps served by the ring / by far stages
    int n_far_stages, n_own_stages;
    int blocks_per_seq, total_blocks, blocks_per_cta;
    int consumers;
    int extra_bytes;     // kernel-specific shared memory after the barriers
};

template <int D, int NOWN>
struct Smem {
    static constexpr int kPitch = D * 2;
    static constexpr int kTile = kBlockRows * kPitch;
    int ring0, ring1, far, own, bars, misc, extra, total;
    __host__ __device__ Smem(const Plan& p) {
        ring0 = 0;
        ring1 = ring0 + p.nrb * kTile;
        far = ring1 + p.nrb * kTile;
        own = far + p.n_far_stages * 2 * kTile;
        bars = own + p.n_own_stages * NOWN * kTile;
        misc = bars + 8 * (2 * kMaxRingBlocks + 2 * kMaxFarStages + 2 * kMaxOwnStages);
        extra = misc + 64;
        total = extra + p.extra_bytes;
    }
};

struct Bars {
    uint32_t base;
    __device__ uint32_t win_full(int s) const { return base + 8 * s; }
    __device__ uint32_t win_empty(int s) const { return base + 8 * (kMaxRingBlocks + s); }
    __device__ uint32_t far_full(int s) const { return base + 8 * (2 * kMaxRingBlocks + s); }
    __device__ uint32_t far_empty(int s) const { return base + 8 * (2 * kMaxRingBlocks + kMaxFarStages + s); }
    __device__ uint32_t own_full(int s) const { return base + 8 * (2 * kMaxRingBlocks + 2 * kMaxFarStages + s); }
    __device__ uint32_t own_empty(int s) const { return base + 8 * (2 * kMaxRingBlocks + 2 * kMaxFarStages + kMaxOwnStages + s); }
};

// One thread: barrier initialisation, including the make-up arrivals for the first `look`
// ring blocks (block r < look is only read by own blocks 0 .. r, not by look+1 of them).
__device__ __forceinline__ void init_barriers(const Plan& p, const Bars& bars, volatile int* abort_flag) {
    for (int i = 0; i < p.nrb; ++i) {
        mbar_init(bars.win_full(i), 1);
        mbar_init(bars.win_empty(i), (p.look + 1) * kTilesPerBlock);
    }
    for (int i = 0; i < p.n_far_stages; ++i) { mbar_init(bars.far_full(i), 1); mbar_init(bars.far_empty(i), kTilesPerBlock); }
    for (int i = 0; i < p.n_own_stages; ++i) { mbar_init(bars.own_full(i), 1); mbar_init(bars.own_empty(i), kTilesPerBlock); }
    *abort_flag = 0;
    fence_mbar_init();
    for (int b = 0; b < p.look; ++b)
        for (int k = 0; k < (p.look - b) * kTilesPerBlock; ++k) mbar_arrive(bars.win_empty(b & (p.nrb - 1)));
}

// The producer thread.  own_maps[NOWN]: tensors of the own stage; ring_maps[2]: ring and far tensors.
template <int D, int NOWN, bool AHEAD>
__device__ __forceinline__ void producer_loop(const Plan& p, const Taps& t, const CUtensorMap* const (&own_maps)[NOWN],
                                              const CUtensorMap* const (&ring_maps)[2], uint32_t smem_base,
                                              const Smem<D, NOWN>& lay, const Bars& bars, volatile int* abort_flag,
                                              int g_begin, int g_end) {
    constexpr int kTile = Smem<D, NOWN>::kTile;
    const int nrb = p.nrb, look = p.look;
    const int n_blocks = g_end - g_begin;
    const int last_block = p.total_blocks - 1;
#pragma unroll 1
    for (int r = 0; r < n_blocks + look; ++r) {
        // ring block r (blocks outside the stream are replaced by a valid one: their rows are never used)
        int G = AHEAD ? g_begin + r : g_begin - look + r;
        G = G < 0 ? 0 : (G > last_block ? last_block : G);
        {
            const int bh = G / p.blocks_per_seq, sb = G - bh * p.blocks_per_seq;
            const int slot = r & (nrb - 1), fill = r / nrb;
            mbar_wait(bars.win_empty(slot), (fill & 1) ^ 1, abort_flag, 0x102);
            mbar_arrive_expect_tx(bars.win_full(slot), 2 * kTile);
            tma_load_3d(smem_base + lay.ring0 + slot * kTile, ring_maps[0], bars.win_full(slot), 0, sb * kBlockRows, bh);
            tma_load_3d(smem_base + lay.ring1 + slot * kTile, ring_maps[1], bars.win_full(slot), 0, sb * kBlockRows, bh);
        }
        const int j = r - look;                              // own block whose ring window is now complete
        if (j >= 0) {
            const int Go = g_begin + j;
            const int bh = Go / p.blocks_per_seq, sb = Go - bh * p.blocks_per_seq;
            const int os = j % p.n_own_stages, on = j / p.n_own_stages;
            mbar_wait(bars.own_empty(os), (on & 1) ^ 1, abort_flag, 0x101);
            mbar_arrive_expect_tx(bars.own_full(os), NOWN * kTile);
#pragma unroll
            for (int i = 0; i < NOWN; ++i)
                tma_load_3d(smem_base + lay.own + (os * NOWN + i) * kTile, own_maps[i], bars.own_full(os), 0, sb * kBlockRows, bh);
#pragma unroll 1
            for (int f = 0; f < p.n_far; ++f) {
                const int seq = j * p.n_far + f;
                const int fs = seq % p.n_far_stages, fn = seq / p.n_far_stages;
                const int delta = t.sparse[p.n_win + f];
                const int row = sb * kBlockRows + (AHEAD ? delta : -delta);   // outside [0,N): zero-filled
                mbar_wait(bars.far_empty(fs), (fn & 1) ^ 1, abort_flag, 0x103);
                mbar_arrive_expect_tx(bars.far_full(fs), 2 * kTile);
                tma_load_3d(smem_base + lay.far + fs * 2 * kTile, ring_maps[0], bars.far_full(fs), 0, row, bh);
                tma_load_3d(smem_base + lay.far + fs * 2 * kTile + kTile, ring_maps[1], bars.far_full(fs), 0, row, bh);
            }
        }
        if (*abort_flag) break;
    }
}

// ------------------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            ptr = nullptr;
        return reinterpret_cast<EncodeTiledFn>(ptr);
    }();
    return fn;
}

// [BH][N][D] bf16 tensor, box = 128 rows x D, swizzle matching the row pitch.
inline bool make_row_map(CUtensorMap* m, const void* ptr, int BH, int N, int D) {
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

inline int band_width(const Taps& t) {
    const int d_hi = t.d_lo + t.n_dense - 1;
    return d_hi <= 32 ? 32 : (d_hi <= 48 ? 48 : (d_hi <= 64 ? 64 : 0));
}

}  // namespace pipe
}  // namespace dsqg
