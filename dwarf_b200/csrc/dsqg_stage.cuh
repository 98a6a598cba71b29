// Staging layer of the TMA-fed DSQG forward (bf16, sm_100a): what a thread block copies into
// shared memory, how the copies are issued and waited for, and how warps read MMA fragments
// out of the swizzled tiles.
//
// A thread block owns kRows = 64 consecutive rows of one (batch, head) sequence ("own rows").
// What it needs from the other side of the attention ("partner rows": value rows n - delta for a
// query row n; the plan also covers the mirrored case, rows m + delta for a key row m) is fetched
// ONCE per block by the copy engine (cp.async.bulk.tensor, plain per-block loads from this GPU's
// own memory, every block fetching for itself):
//   * the dense window of all 64 rows is one contiguous band of 64 + 32 partner rows;
//   * every sparse tap is a 64-row tile shifted by its offset; taps whose tiles overlap or touch
//     the band or each other are merged into one contiguous "segment", so a partner row that
//     several taps share is fetched once (offsets 48 ... 256 of the usual sets join the band:
//     320 rows instead of 96 + 6 x 64).
// A segment is copied as 64-row boxes and has its own mbarrier; all copies of a block are issued
// by warp 0 at block start (one box per lane).  Rows outside [0, N) are zero-filled by the copy
// engine.  Every wait on a barrier is bounded (see mbar_wait).
#pragma once

#include <cuda.h>

#include "dsqg_mma.cuh"

namespace dsqg {
namespace stg {

constexpr int kRows = 64;            // own rows per thread block = rows per copy box
constexpr int kWB = 32;              // dense offsets served: 0 .. kWB
constexpr int kNT = (kWB + 16) / 8;  // 8-row n-tiles of the band a 16-row tile touches
constexpr int kMaxSeg = 18;
constexpr int kMaxBox = 32;
constexpr int kMaxTaps = 16;         // sparse taps (two groups of eight score columns)
constexpr int kSmemLimit = 227 * 1024;
constexpr long long kWaitCycleLimit = 200000000LL;   // ~0.1 s of SM clock before a wait gives up

// What a block stages, computed on the host from the tap set (identical for every block).
// Rows are counted in "tile rows": row r of the staged area of a tensor sits at byte r * 2D.
struct Plan {
    int n_seg;                 // segments; segment 0 always holds the band
    int n_box;                 // copy boxes (kRows rows each) over all segments
    int rows;                  // tile rows per tensor (a multiple of kRows)
    int band_row0;             // tile row of the band's first partner row
    int seg_reach[kMaxSeg];    // smallest offset the segment serves (0 for segment 0)
    int seg_boxes[kMaxSeg];    // its length in boxes
    int box_rel[kMaxBox];      // first partner row of the box, relative to the block's first own row
    short box_row0[kMaxBox];   // its first tile row
    short box_seg[kMaxBox];    // its segment
    short tap_row0[kMaxTaps];  // tile row of the tap's first partner row (a multiple of 8)
    short tap_seg[kMaxTaps];   // segment that holds it (non-decreasing in the tap index)
};

// ahead = false: partner rows lie BEFORE the own rows (forward, dQ: key row n - delta);
// ahead = true : partner rows lie AFTER them (dK/dV: query row m + delta).
// Returns false when the tap set does not fit this path.
inline bool build_plan(const Taps& t, bool ahead, Plan* p) {
    if (t.n_sparse > kMaxTaps || t.d_lo + t.n_dense - 1 > kWB) return false;
    *p = Plan{};
    int lo[kMaxSeg], hi[kMaxSeg], start[kMaxTaps];
    int ns = 1;
    lo[0] = ahead ? 0 : -kWB;
    hi[0] = lo[0] + kRows + kWB;
    p->seg_reach[0] = 0;
    for (int i = 0; i < t.n_sparse; ++i) {
        const int s = ahead ? t.sparse[i] : -t.sparse[i], e = s + kRows;
        start[i] = s;
        int& l = lo[ns - 1];
        int& h = hi[ns - 1];
        const int grow = (s < l ? l - s : 0) + (e > h ? e - h : 0);
        const bool aligned = ((s - l) % 8 + 8) % 8 == 0;
        const bool touches = e >= l && s <= h;
        if (aligned && touches && grow <= kRows) {
            if (s < l) l = s;
            if (e > h) h = e;
        } else {
            if (ns == kMaxSeg) return false;
            lo[ns] = s; hi[ns] = e;
            p->seg_reach[ns] = t.sparse[i];
            ++ns;
        }
        p->tap_seg[i] = (short)(ns - 1);
    }
    p->n_seg = ns;
    int row = 0, nb = 0;
    int seg_row0[kMaxSeg];
    for (int i = 0; i < ns; ++i) {
        seg_row0[i] = row;
        p->seg_boxes[i] = (hi[i] - lo[i] + kRows - 1) / kRows;
        for (int b = 0; b < p->seg_boxes[i]; ++b) {
            if (nb == kMaxBox) return false;
            p->box_rel[nb] = lo[i] + b * kRows;
            p->box_row0[nb] = (short)(row + b * kRows);
            p->box_seg[nb] = (short)i;
            ++nb;
        }
        row += p->seg_boxes[i] * kRows;
    }
    p->n_box = nb;
    p->rows = row;
    p->band_row0 = (ahead ? 0 : -kWB) - lo[0];
    if (p->band_row0 % 8 != 0) return false;
    for (int i = 0; i < t.n_sparse; ++i) {
        const int sg = p->tap_seg[i];
        p->tap_row0[i] = (short)(seg_row0[sg] + start[i] - lo[sg]);
    }
    return true;
}

// Host side (dsqg_staged.cu): a bf16 tensor addressed as [batch][head][row][D] through element
// strides sb, sh, sn (rows of D contiguous elements) as a 4-D tiled tensor map whose box is
// box_rows consecutive rows of one head, written with the 64-byte (D = 32) or 128-byte swizzle.
// The two middle dimensions are ordered by stride; *head_first tells the kernel which order the
// coordinates take.  false when the driver's encoder is missing or refuses the shape.
bool make_map(CUtensorMap* m, bool* head_first, const void* ptr, int B, int H, int N, int D,
              long long sb, long long sh, long long sn, int box_rows);
bool tensor_map_encoder_available();

// ------------------------------------------------------------------------------ device side
#ifdef __CUDACC__

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

// Error word of this translation unit (the host ORs the copies together in dsqg_device_error()):
// 0 = ok, else the id of the first wait that gave up.
static __device__ int g_stage_error = 0;

// Bounded wait.  `abort_flag` lives in shared memory; once set, every wait of the block returns
// at once, so the kernel ends instead of hanging.  Returns false when the wait gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int site,
                                          long long limit = kWaitCycleLimit) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t it = 0;; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (it > 64) {
            __nanosleep(40);
            if (clock64() - t0 > limit) break;
        }
    }
    *abort_flag = 1;
    atomicCAS(&g_stage_error, 0, site);
    return false;
}

// 4-D tiled copies.  Coordinates are (element in row = 0, c1, c2, batch); c1/c2 are (row, head)
// or (head, row), whichever order keeps the tensor's strides ascending (see make_map).  The
// innermost coordinate is always 0, which satisfies the 16-byte start rule of the copy engine.
__device__ __forceinline__ void tma_load(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
__device__ __forceinline__ void tma_store(const CUtensorMap* map, uint32_t src, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
        ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// A tensor as the copy engine sees it, plus the order of its middle coordinates.
struct Tma {
    const CUtensorMap* map;
    bool head_first;           // coordinates are (0, head, row, batch) instead of (0, row, head, batch)
    __device__ __forceinline__ void load(uint32_t dst, uint32_t bar, int row, int h, int b) const {
        if (head_first) tma_load(dst, map, bar, h, row, b); else tma_load(dst, map, bar, row, h, b);
    }
    __device__ __forceinline__ void store(uint32_t src, int row, int h, int b) const {
        if (head_first) tma_store(map, src, h, row, b); else tma_store(map, src, row, h, b);
    }
};

// ------------------------------------------------------------------------------------------
// Fragments out of a swizzled tile.  A tile row is D bf16 = 2D bytes; the copy engine writes
// with SWIZZLE_64B (D = 32) or SWIZZLE_128B (D = 64): the 16-byte chunk index of a row is XORed
// with (row >> 1) & 3 resp. row & 7, rows counted from a 1024-byte boundary.  Every 16-row group
// a warp reads starts on a multiple of 8 tile rows, so the XOR term depends on the lane only.
//
// One ldmatrix.x4 reads a 16-row x 16-element patch as four 8x8 matrices; lane l supplies the
// address of row (l & 7) + 8 * ((l >> 3) & 1), chunk 2p + (l >> 4).  The four registers are
//   r0 = rows 0-7 / chunk 2p,  r1 = rows 8-15 / chunk 2p,  r2 = rows 0-7 / chunk 2p+1,  r3 = rows 8-15 / chunk 2p+1
// which is, without .trans,
//   the A fragment {a0,a1,a2,a3} of k-step p when the 16 rows are the M rows, and
//   the B fragments of k-step p of two n-tiles when the rows are N columns: n-tile 0 = {r0,r2}, n-tile 1 = {r1,r3};
// and with .trans the B fragments of a product that contracts over the 16 rows:
//   n-tile 2p = {r0,r1}, n-tile 2p+1 = {r2,r3}.
// ------------------------------------------------------------------------------------------
template <int D> struct LaneAddr { uint32_t o[D / 16]; };

template <int D>
__device__ __forceinline__ LaneAddr<D> lane_addr(int lane) {
    LaneAddr<D> a;
    const int row = (lane & 7) + 8 * ((lane >> 3) & 1), hi = lane >> 4;
    const int swz = D == 32 ? (row >> 1) & 3 : row & 7;
#pragma unroll
    for (int p = 0; p < D / 16; ++p) a.o[p] = row * (2 * D) + (((2 * p + hi) ^ swz) << 4);
    return a;
}
__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm4t(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

// acc[16 x D] += diag(w) . T, where T is the 16-row group at `group_base` and w holds one weight
// per row: lane (g, tig) passes the packed pair {w[g], w[g+8]} (bf16x2) of the quad member that
// owns the tap's column; sel_lo / sel_hi are this lane's byte-permute selectors (diag_selectors).
template <int D>
__device__ __forceinline__ void diag_mma(float (&acc)[D / 8][4], uint32_t packed, uint32_t sel_lo, uint32_t sel_hi,
                                         uint32_t group_base, const LaneAddr<D>& la) {
    const uint32_t a0 = __byte_perm(packed, 0u, sel_lo), a3 = __byte_perm(packed, 0u, sel_hi);
#pragma unroll
    for (int p = 0; p < D / 16; ++p) {
        uint32_t r[4];
        ldsm4t(r, group_base + la.o[p]);
        mma16816(acc[2 * p], a0, 0u, 0u, a3, r[0], r[1]);
        mma16816(acc[2 * p + 1], a0, 0u, 0u, a3, r[2], r[3]);
    }
}
// The diagonal A fragment has A[g][g] in register a0 and A[g+8][g+8] in a3 of the lane with
// tig == g >> 1, at half-word g & 1; every other entry is zero.
__device__ __forceinline__ void diag_selectors(int g, int tig, uint32_t& sel_lo, uint32_t& sel_hi) {
    const bool owner = tig == (g >> 1);
    sel_lo = !owner ? 0x4444u : ((g & 1) ? 0x1044u : 0x4410u);
    sel_hi = !owner ? 0x4444u : ((g & 1) ? 0x3244u : 0x4432u);
}

// Writes rows g and g+8 of a 16 x D accumulator tile as bf16 into a swizzled 16-row group (the
// layout a copy-engine store with the same swizzle mode expects).  Free of bank conflicts.
template <int D>
__device__ __forceinline__ void stage_acc(unsigned char* group, const float (&acc)[D / 8][4], float s_lo, float s_hi,
                                          int g, int tig) {
    const int swz_lo = D == 32 ? (g >> 1) & 3 : g & 7;     // rows g and g+8 have the same XOR term
    unsigned char* lo = group + g * (2 * D) + 4 * tig;
    unsigned char* hi = lo + 8 * (2 * D);
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
        const int off = (j ^ swz_lo) << 4;
        *reinterpret_cast<uint32_t*>(lo + off) = pack_bf16x2(acc[j][0] * s_lo, acc[j][1] * s_lo);
        *reinterpret_cast<uint32_t*>(hi + off) = pack_bf16x2(acc[j][2] * s_hi, acc[j][3] * s_hi);
    }
}

#endif  // __CUDACC__

}  // namespace stg
}  // namespace dsqg
