// Warp-level building blocks of the tensor-core DSQG kernels (bf16, sm_100a).
//
// Fragment convention used by every kernel in dsqg_mma*.cu
// --------------------------------------------------------
// lane = 4*g + tig  (g = 0..7, tig = 0..3).  A warp owns a tile of 16 rows.
// A row of D bf16 elements is split into 16-byte chunks; thread tig reads chunk tig of
// every 64-byte group, i.e. elements  d = 32*c + 8*tig + [0,8)  for c = 0 .. D/32-1.
// Those 8*D/32 elements are the thread's share of the contraction dimension for BOTH
// operands of  mma.sync.m16n8k16  (the instruction assigns k-indices {2tig,2tig+1,2tig+8,
// 2tig+9} of every k-step to thread tig in the A and in the B fragment alike, so any fixed
// assignment of physical d to k-index is legal as long as A and B agree).  Hence
//   * a "row fragment" (RowFrag) is loaded with one 16-byte load per 32 elements of D,
//   * the same RowFrag serves as A operand (rows g, g+8 of the warp tile) or as B operand
//     (row g of an 8-row n-tile) of a product that contracts over d,
//   * movmatrix(.trans) turns a RowFrag into the B operand of a product that contracts over
//     ROWS (P.V, dS.K, ...); the accumulator column n of such a product maps to
//     d = 32*c + 8*(n>>1) + 2*j + (n&1), so thread tig ends up owning the contiguous elements
//     d = 32*c + 8*tig + [0,8) of rows g and g+8: one 16-byte store per chunk.
#pragma once

#include "dsqg_common.cuh"

namespace dsqg {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kNeg = -1.0e30f;   // finite "minus infinity": masked scores
constexpr float kMinM = -1.0e29f;  // floor of the running row maximum: exp2(kNeg - kMinM) == 0

template <int D> struct RowFrag { uint32_t r[D / 8]; };   // D/32 chunks x 4 registers

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// 16-byte chunks of one row; zero-filled when !valid (the pointer is not dereferenced then).
template <int D>
__device__ __forceinline__ void load_row(RowFrag<D>& f, const __nv_bfloat16* row_ptr, int tig, bool valid) {
#pragma unroll
    for (int c = 0; c < D / 32; ++c) {
        uint4 u = make_uint4(0u, 0u, 0u, 0u);
        if (valid) u = __ldg(reinterpret_cast<const uint4*>(row_ptr + 32 * c + 8 * tig));
        f.r[4 * c + 0] = u.x; f.r[4 * c + 1] = u.y; f.r[4 * c + 2] = u.z; f.r[4 * c + 3] = u.w;
    }
}

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// d = A.B with a zero accumulator input (no register initialisation needed)
__device__ __forceinline__ void mma16816_z(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                           uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}

// c = A.B (overwrites c), contraction over d as in mma_rows
template <int D>
__device__ __forceinline__ void mma_rows_z(float (&c)[4], const RowFrag<D>& a_lo, const RowFrag<D>& a_hi,
                                           const RowFrag<D>& b) {
    mma16816_z(c, a_lo.r[0], a_hi.r[0], a_lo.r[1], a_hi.r[1], b.r[0], b.r[1]);
#pragma unroll
    for (int kk = 1; kk < D / 16; ++kk)
        mma16816(c, a_lo.r[2 * kk], a_hi.r[2 * kk], a_lo.r[2 * kk + 1], a_hi.r[2 * kk + 1], b.r[2 * kk], b.r[2 * kk + 1]);
}

// C[16 x 8] += A(rows g / g+8 = a_lo / a_hi)[16 x D] . B(row g = b)[8 x D]^T   (contracts over d)
template <int D>
__device__ __forceinline__ void mma_rows(float (&c)[4], const RowFrag<D>& a_lo, const RowFrag<D>& a_hi,
                                         const RowFrag<D>& b) {
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk)
        mma16816(c, a_lo.r[2 * kk], a_hi.r[2 * kk], a_lo.r[2 * kk + 1], a_hi.r[2 * kk + 1], b.r[2 * kk], b.r[2 * kk + 1]);
}

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
    uint32_t y;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
    return y;
}

template <int D>
__device__ __forceinline__ void transpose_frag(RowFrag<D>& t, const RowFrag<D>& f) {
#pragma unroll
    for (int j = 0; j < D / 8; ++j) t.r[j] = movmatrix_trans(f.r[j]);
}

// acc[16 x D] += A[16 x 16] . B[16 x D]  where the 16 contraction rows are the rows of the two
// transposed row fragments (rows 0..7 = t_lo, rows 8..15 = t_hi).  acc[j] is n-tile j.
template <int D>
__device__ __forceinline__ void mma_cols(float (&acc)[D / 8][4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         const RowFrag<D>& t_lo, const RowFrag<D>& t_hi) {
#pragma unroll
    for (int j = 0; j < D / 8; ++j) mma16816(acc[j], a0, a1, a2, a3, t_lo.r[j], t_hi.r[j]);
}

__device__ __forceinline__ float quad_max(float x) {
    x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 1));
    return fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 2));
}
__device__ __forceinline__ float quad_sum(float x) {
    x += __shfl_xor_sync(0xffffffffu, x, 1);
    return x + __shfl_xor_sync(0xffffffffu, x, 2);
}

// Diagonal A fragment: A[g][g] = x_lo, A[g+8][g+8] = x_hi, zero elsewhere.  Only the thread
// with tig == g>>1 holds non-zeros (element g&1 of its a0a1 / a6a7 registers).
__device__ __forceinline__ void diag_frag(float x_lo, float x_hi, bool owner, int g, uint32_t& a0, uint32_t& a3) {
    const uint32_t lo = owner ? (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(x_lo)) : 0u;
    const uint32_t hi = owner ? (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(x_hi)) : 0u;
    const int sh = (g & 1) * 16;
    a0 = lo << sh;
    a3 = hi << sh;
}

// Store rows g and g+8 of an accumulator tile (contiguous-d layout) as bf16, scaled per row.
template <int D>
__device__ __forceinline__ void store_acc_rows(const float (&acc)[D / 8][4], __nv_bfloat16* row_lo, __nv_bfloat16* row_hi,
                                               bool ok_lo, bool ok_hi, float s_lo, float s_hi, int tig) {
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
        if (ok_lo) *reinterpret_cast<uint4*>(row_lo + 32 * c + 8 * tig) = lo;
        if (ok_hi) *reinterpret_cast<uint4*>(row_hi + 32 * c + 8 * tig) = hi;
    }
}

// As store_acc_rows, with every element multiplied by sigmoid(gate) of the same position (gate rows
// are bf16 in the layout of the output rows): the sigmoid gate of the attention block folded into
// the epilogue (DWARF train/train_2048_condU.py:190-191).
template <int D>
__device__ __forceinline__ void store_acc_rows_gated(const float (&acc)[D / 8][4], __nv_bfloat16* row_lo, __nv_bfloat16* row_hi,
                                                     const __nv_bfloat16* gate_lo, const __nv_bfloat16* gate_hi,
                                                     bool ok_lo, bool ok_hi, float s_lo, float s_hi, int tig) {
    auto sig2 = [](uint32_t u, float& a, float& b) {
        a = __fdividef(1.f, 1.f + __expf(-__uint_as_float(u << 16)));
        b = __fdividef(1.f, 1.f + __expf(-__uint_as_float(u & 0xffff0000u)));
    };
#pragma unroll
    for (int c = 0; c < D / 32; ++c) {
        uint4 gl = make_uint4(0u, 0u, 0u, 0u), gh = gl;
        if (ok_lo) gl = __ldg(reinterpret_cast<const uint4*>(gate_lo + 32 * c + 8 * tig));
        if (ok_hi) gh = __ldg(reinterpret_cast<const uint4*>(gate_hi + 32 * c + 8 * tig));
        const uint32_t gls[4] = {gl.x, gl.y, gl.z, gl.w}, ghs[4] = {gh.x, gh.y, gh.z, gh.w};
        uint32_t lo[4], hi[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float a0, a1, b0, b1;
            sig2(gls[j], a0, a1); sig2(ghs[j], b0, b1);
            lo[j] = pack_bf16x2(acc[4 * c + j][0] * s_lo * a0, acc[4 * c + j][1] * s_lo * a1);
            hi[j] = pack_bf16x2(acc[4 * c + j][2] * s_hi * b0, acc[4 * c + j][3] * s_hi * b1);
        }
        if (ok_lo) *reinterpret_cast<uint4*>(row_lo + 32 * c + 8 * tig) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
        if (ok_hi) *reinterpret_cast<uint4*>(row_hi + 32 * c + 8 * tig) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
    }
}

// Partial dot product of two row fragments over this thread's elements (fp32).
template <int D>
__device__ __forceinline__ float frag_dot(const RowFrag<D>& a, const RowFrag<D>& b) {
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
        s = fmaf(__uint_as_float(a.r[j] << 16), __uint_as_float(b.r[j] << 16), s);
        s = fmaf(__uint_as_float(a.r[j] & 0xffff0000u), __uint_as_float(b.r[j] & 0xffff0000u), s);
    }
    return s;
}

// Lane roles inside a 16-row tile held as MMA fragments (rows g and g+8 per lane).
struct Lane {
    int warp, lane, g, tig;
    bool owner;          // holds the diagonal entries of rows g and g+8
    int owner_lane;      // lane of this quad's owner
    __device__ Lane() {
        warp = threadIdx.x >> 5; lane = threadIdx.x & 31; g = lane >> 2; tig = lane & 3;
        owner = tig == (g >> 1);
        owner_lane = (lane & ~3) | (g >> 1);
    }
};

// acc(rows g / g+8) += x_lo * f_lo, x_hi * f_hi for this thread's elements: the diagonal form of
// "A.B with A = diag(x)" -- row g of the product only needs row g of B, which the thread holds
// as a row fragment for exactly the elements d its accumulators cover.
template <int D>
__device__ __forceinline__ void diag_fma(float (&acc)[D / 8][4], float x_lo, float x_hi, const RowFrag<D>& f_lo,
                                         const RowFrag<D>& f_hi) {
    // packed fp32 FMA (fma.rn.f32x2, sm_100): one instruction updates the two accumulators a row has
    // in an n-tile; measured 1 % off the step against scalar FMAs (cfg1: 284.8 against 287.6 us)
    unsigned long long xl, xh;
    asm("mov.b64 %0, {%1, %1};" : "=l"(xl) : "f"(x_lo));
    asm("mov.b64 %0, {%1, %1};" : "=l"(xh) : "f"(x_hi));
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
        const uint32_t u0 = f_lo.r[j], u1 = f_hi.r[j];
        unsigned long long v0, v1, c0, c1;
        asm("mov.b64 %0, {%1, %2};" : "=l"(v0) : "r"(u0 << 16), "r"(u0 & 0xffff0000u));
        asm("mov.b64 %0, {%1, %2};" : "=l"(v1) : "r"(u1 << 16), "r"(u1 & 0xffff0000u));
        asm("mov.b64 %0, {%1, %2};" : "=l"(c0) : "f"(acc[j][0]), "f"(acc[j][1]));
        asm("mov.b64 %0, {%1, %2};" : "=l"(c1) : "f"(acc[j][2]), "f"(acc[j][3]));
        asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(c0) : "l"(xl), "l"(v0));
        asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(c1) : "l"(xh), "l"(v1));
        asm("mov.b64 {%0, %1}, %2;" : "=f"(acc[j][0]), "=f"(acc[j][1]) : "l"(c0));
        asm("mov.b64 {%0, %1}, %2;" : "=f"(acc[j][2]), "=f"(acc[j][3]) : "l"(c1));
    }
}

// The running maximum of the online softmax only moves when a score exceeds it by more than this
// (log2 units): probabilities stay below 2^kSlack, which fp32 sums and bf16 values absorb.
constexpr float kSlack = 16.f;

template <int D>
__device__ __forceinline__ void load_row_at(RowFrag<D>& f, const __nv_bfloat16* p) {
#pragma unroll
    for (int c = 0; c < D / 32; ++c) {
        const uint4 u = __ldg(reinterpret_cast<const uint4*>(p + 32 * c));
        f.r[4 * c + 0] = u.x; f.r[4 * c + 1] = u.y; f.r[4 * c + 2] = u.z; f.r[4 * c + 3] = u.w;
    }
}

}  // namespace dsqg
