// TMA (cp.async.bulk.tensor) and mbarrier helpers for the persistent DSQG kernels (sm_100a).
//
// Only plain per-CTA tensor loads are used: every CTA fetches its own tiles from its own
// GPU's memory into its own shared memory.  Every wait is bounded: after kWaitCycleLimit SM
// cycles the waiter raises the CTA's abort flag and a device-wide error word, and from then on
// all waits in the CTA fall through so that the kernel returns instead of hanging.
#pragma once

#include <cuda.h>

#include "dsqg_mma.cuh"

namespace dsqg {

constexpr long long kWaitCycleLimit = 200000000LL;   // ~0.1 s of SM clock before a wait gives up

// Error word of this translation unit (one copy per .cu file that includes this header; the
// host ORs them together in dsqg_device_error()).  0 = ok; otherwise (kernel id << 8) | wait-site
// id of the first wait that gave up.
static __device__ int g_device_error = 0;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}

// Bounded wait.  `abort_flag` lives in shared memory; once set, every wait returns at once.
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int site) {
    if (mbar_try_wait(bar, parity)) return;
    const long long t0 = clock64();
    for (uint32_t it = 0;; ++it) {
        if (mbar_try_wait(bar, parity)) return;
        if (*abort_flag) return;
        if (it > 64) {
            __nanosleep(64);
            if (clock64() - t0 > kWaitCycleLimit) break;
        }
    }
    *abort_flag = 1;
    atomicCAS(&g_device_error, 0, site);
}

// 3-D tiled load: coordinates are (x = element in row, y = row, z = batch*head slice).
// x is always 0 here (whole rows), which satisfies the 16-byte start rule; rows outside
// [0, N) are filled with zeros by the copy engine.
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "r"(z)
        : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// --------------------------------------------------------------------------------------
// Row fragments out of a TMA-swizzled tile.  A tile is `rows` x D bf16, row pitch D*2 bytes,
// written with SWIZZLE_64B (D = 32) or SWIZZLE_128B (D = 64): the 16-byte chunk index of a
// row is XORed with (row>>1)&3 resp. row&7.  Tiles start on 1024-byte boundaries and every
// 16-row warp tile starts on a multiple of 8 rows, so the XOR term only depends on the lane.
//   D = 32: thread tig owns chunk tig             (elements 8*tig + [0,8))
//   D = 64: thread tig owns chunks 2*tig, 2*tig+1 (elements 16*tig + [0,16))
// --------------------------------------------------------------------------------------
template <int D> struct LaneOff { uint32_t o[D / 32]; };

template <int D>
__device__ __forceinline__ LaneOff<D> lane_offsets(int g, int tig) {
    LaneOff<D> l;
    if (D == 32) {
        l.o[0] = g * 64 + ((tig ^ ((g >> 1) & 3)) << 4);
    } else {
        l.o[0] = g * 128 + (((2 * tig) ^ g) << 4);
        l.o[D / 32 - 1] = g * 128 + (((2 * tig + 1) ^ g) << 4);
    }
    return l;
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

// rows g (plus `row8` * 8) of the 8-row group that starts at byte address `group_base`
template <int D>
__device__ __forceinline__ void lds_frag(RowFrag<D>& f, uint32_t group_base, const LaneOff<D>& lo) {
#pragma unroll
    for (int c = 0; c < D / 32; ++c) {
        const uint4 u = lds128(group_base + lo.o[c]);
        f.r[4 * c + 0] = u.x; f.r[4 * c + 1] = u.y; f.r[4 * c + 2] = u.z; f.r[4 * c + 3] = u.w;
    }
}

// --------------------------------------------------------------------------------------
// Transposed B fragments straight from a swizzled tile: ldmatrix.x4.trans on a 16-row x 16-element
// patch gives, for the two 8-column n-tiles of the patch, the registers {b0 (rows 0-7), b1 (rows
// 8-15)} of a product that contracts over the 16 rows.  Lane l addresses row (l&7) + 8*((l>>3)&1)
// and 16-byte chunk 2*patch + (l>>4).  The accumulator of such a product has the standard layout:
// n-tile j, slot r  <->  row g + 8*(r>>1), element 8*j + 2*tig + (r&1).
// --------------------------------------------------------------------------------------
template <int D> struct ColOff { uint32_t o[D / 16]; };
template <int D> struct ColFrag { uint32_t b0[D / 8], b1[D / 8]; };

template <int D>
__device__ __forceinline__ ColOff<D> col_offsets(int lane) {
    ColOff<D> c;
    const int row = (lane & 7) + 8 * ((lane >> 3) & 1), hi = lane >> 4;
    const int swz = D == 32 ? (row >> 1) & 3 : row & 7;
#pragma unroll
    for (int p = 0; p < D / 16; ++p) c.o[p] = row * (D * 2) + (((2 * p + hi) ^ swz) << 4);
    return c;
}

// tile_base: shared address of row 0 of the 16-row tile (a multiple of 8 rows inside a TMA tile)
template <int D>
__device__ __forceinline__ void ldsm_cols(ColFrag<D>& f, uint32_t tile_base, const ColOff<D>& co) {
#pragma unroll
    for (int p = 0; p < D / 16; ++p)
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(f.b0[2 * p]), "=r"(f.b1[2 * p]), "=r"(f.b0[2 * p + 1]), "=r"(f.b1[2 * p + 1])
                     : "r"(tile_base + co.o[p]));
}

template <int D>
__device__ __forceinline__ void mma_colfrag(float (&acc)[D / 8][4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                            const ColFrag<D>& f) {
#pragma unroll
    for (int j = 0; j < D / 8; ++j) mma16816(acc[j], a0, a1, a2, a3, f.b0[j], f.b1[j]);
}

// Store rows g, g+8 of a standard-layout accumulator as bf16 pairs, scaled per row.
template <int D>
__device__ __forceinline__ void store_acc_std(const float (&acc)[D / 8][4], __nv_bfloat16* row_lo, __nv_bfloat16* row_hi,
                                              bool ok_lo, bool ok_hi, float s_lo, float s_hi, int tig) {
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
        if (ok_lo) *reinterpret_cast<uint32_t*>(row_lo + 8 * j + 2 * tig) = pack_bf16x2(acc[j][0] * s_lo, acc[j][1] * s_lo);
        if (ok_hi) *reinterpret_cast<uint32_t*>(row_hi + 8 * j + 2 * tig) = pack_bf16x2(acc[j][2] * s_hi, acc[j][3] * s_hi);
    }
}

// element offset of this thread's chunk c inside a row (matches lane_offsets)
template <int D>
__device__ __forceinline__ int chunk_elem(int tig, int c) { return D == 32 ? 8 * tig : 16 * tig + 8 * c; }

}  // namespace dsqg
