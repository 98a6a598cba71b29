// TMA (cp.async.bulk.tensor) and mbarrier helpers for the persistent DSQG kernels (sm_100a).
//
// Only plain per-CTA tensor loads are used: every CTA fetches its own tiles from its own
// GPU's memory into its own shared memory.  Every wait is bounded: after kSpinLimit failed
// polls the waiter raises the CTA's abort flag and a device-wide error word, and from then on
// all waits in the CTA fall through so that the kernel returns instead of hanging.
#pragma once

#include <cuda.h>

#include "dsqg_mma.cuh"

namespace dsqg {

constexpr uint32_t kSpinLimit = 1u << 22;   // polls (each with a short sleep) before giving up

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
    for (uint32_t it = 0; it < kSpinLimit; ++it) {
        if (mbar_try_wait(bar, parity)) return;
        if (*abort_flag) return;
        if (it > 64) __nanosleep(64);
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

// element offset of this thread's chunk c inside a row (matches lane_offsets)
template <int D>
__device__ __forceinline__ int chunk_elem(int tig, int c) { return D == 32 ? 8 * tig : 16 * tig + 8 * c; }

}  // namespace dsqg
