// Single-token DSQG decode over a circular K/V ring buffer.
//
// The DWARF reference describes this cache only in prose (README.md:175-179): because the
// tap set is fixed, a layer needs the last max(delta)+1 keys/values and nothing else.
// One warp serves one (sequence, head) pair: it stores the new k, v in slot head[s], then
// each group of TPR lanes reads one tap row (slot (head - delta_j) mod R) per round, keeps
// an online-softmax state over the taps it saw, and the groups are merged with shuffles.
// Pure streaming: 2*J rows of D elements are read per (sequence, head) and nothing is reused.
#include "dsqg_common.cuh"
#include <type_traits>

namespace dsqg {
namespace {

constexpr int kWarpsPerBlock = 4;     // 2 warps per CTA measured within 1 % of this

// Raw 8-element slices as loaded from memory; conversion happens after every load of the step
// has been issued, so one (sequence, head) pair costs a single memory round trip.
template <typename T> struct Raw8;
template <> struct Raw8<__nv_bfloat16> {
    uint4 u;
    __device__ __forceinline__ void load(const __nv_bfloat16* p) { u = *reinterpret_cast<const uint4*>(p); }
    __device__ __forceinline__ void zero() { u = make_uint4(0u, 0u, 0u, 0u); }
    __device__ __forceinline__ void get(float (&x)[8]) const {
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) { x[2 * i] = __uint_as_float(w[i] << 16); x[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
    }
};
template <> struct Raw8<float> {
    float4 a, b;
    __device__ __forceinline__ void load(const float* p) { a = *reinterpret_cast<const float4*>(p); b = *reinterpret_cast<const float4*>(p + 4); }
    __device__ __forceinline__ void zero() { a = make_float4(0.f, 0.f, 0.f, 0.f); b = a; }
    __device__ __forceinline__ void get(float (&x)[8]) const {
        x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
    }
};

// Online-softmax state of one lane group over the taps it has seen: running maximum m, sum l and
// the 8 output elements this lane owns.
struct TapState {
    float m = -INFINITY, l = 0.f;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
};

// Folds tap j (key slice kx, value slice vx of this lane) into the state.  All lanes of the warp
// must call it (the dot product is summed over the lane group with shuffles); `valid` says
// whether the tap exists for this sequence.
template <int TPR>
__device__ __forceinline__ void fold_tap(TapState& st, const DecodeArgs& a, int j, int h, int d0, bool valid, bool active,
                                         const float (&qx)[8], float (&kx)[8], const float (&vx)[8]) {
    if (a.scale_embed != nullptr && valid && active) {
        float se[8];
        load8(a.scale_embed + (size_t)j * a.D + d0, se);
#pragma unroll
        for (int i = 0; i < 8; ++i) kx[i] += se[i];
    }
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) dot = fmaf(qx[i], kx[i], dot);
    dot = group_sum<TPR>(dot);
    if (valid) {
        const float sc = dot * a.scale + a.pos_bias[j * a.H + h];
        const float mn = fmaxf(st.m, sc);
        const float cor = __expf(st.m - mn), p = __expf(sc - mn);
        st.l = st.l * cor + p;
#pragma unroll
        for (int i = 0; i < 8; ++i) st.acc[i] = st.acc[i] * cor + p * vx[i];
        st.m = mn;
    }
}

// Merges the 32/TPR lane-group states of the warp and stores gain * acc / l from lane group 0.
template <typename T, int TPR>
__device__ __forceinline__ void merge_and_store(TapState& st, const DecodeArgs& a, int sh, int h, int d0, bool writer) {
#pragma unroll
    for (int o = TPR; o < 32; o <<= 1) {
        const float m2 = __shfl_xor_sync(0xffffffffu, st.m, o);
        const float l2 = __shfl_xor_sync(0xffffffffu, st.l, o);
        const float mn = fmaxf(st.m, m2);
        const float c1 = (st.m == -INFINITY) ? 0.f : __expf(st.m - mn);
        const float c2 = (m2 == -INFINITY) ? 0.f : __expf(m2 - mn);
        st.l = st.l * c1 + l2 * c2;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float a2 = __shfl_xor_sync(0xffffffffu, st.acc[i], o);
            st.acc[i] = st.acc[i] * c1 + a2 * c2;
        }
        st.m = mn;
    }
    if (writer) {
        const float gain = a.head_gain ? a.head_gain[h] : 1.f;
        const float inv = st.l > 0.f ? gain / st.l : 0.f;
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = st.acc[i] * inv;
        store8(static_cast<T*>(a.out) + (size_t)sh * a.D + d0, o);
    }
}

// All K and V rows of up to ROUNDS taps per lane group are requested before any is used
// (2*ROUNDS independent 16/32-byte loads per lane): one memory round trip per pass.
template <typename T, int TPR, int ROUNDS>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
decode_kernel(const DecodeArgs a, const Taps t) {
    constexpr int GROUPS = 32 / TPR;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sh = blockIdx.x * kWarpsPerBlock + warp;      // (sequence, head) pair
    if (sh >= a.S * a.H) return;                            // whole warp leaves together
    const int s = sh / a.H, h = sh - s * a.H;
    const int g = lane / TPR, li = lane % TPR;
    const int d0 = li * 8, D = a.D;
    const bool active = d0 < D;

    const int head = a.head[s];
    const int fill = a.fill ? a.fill[s] : a.R;
    const T* q = static_cast<const T*>(a.q) + (size_t)sh * D;
    const T* kn = static_cast<const T*>(a.k_new) + (size_t)sh * D;
    const T* vn = static_cast<const T*>(a.v_new) + (size_t)sh * D;
    const int RS = a.ring_stride;                           // elements between two slots of a ring: D, or 2 D when K and V interleave
    T* kr = static_cast<T*>(a.k_ring) + (size_t)sh * a.R * RS;
    T* vr = static_cast<T*>(a.v_ring) + (size_t)sh * a.R * RS;

    float qx[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (active) load8(q + d0, qx);
    if (g == 0 && active) {          // store the new token in the ring (bf16->fp32->bf16 is exact)
        float t8[8];
        load8(kn + d0, t8); store8(kr + (size_t)head * RS + d0, t8);
        load8(vn + d0, t8); store8(vr + (size_t)head * RS + d0, t8);
    }
    TapState st;
    const int rounds = (t.J + GROUPS - 1) / GROUPS;
#pragma unroll 1
    for (int r0 = 0; r0 < rounds; r0 += ROUNDS) {         // one pass for the usual tap counts
        // ---- request the rows of up to ROUNDS taps per lane group
        Raw8<T> kraw[ROUNDS], vraw[ROUNDS];
#pragma unroll
        for (int r = 0; r < ROUNDS; ++r) {
            const int j = (r0 + r) * GROUPS + g;
            const int delta = j < t.J ? t.delta(j) : 0;
            int slot = head - delta;
            if (slot < 0) slot += a.R;
            kraw[r].zero(); vraw[r].zero();
            if (j < t.J && delta < fill && active) {
                // taps with delta == 0 read k_new / v_new directly, so nothing depends on the ring
                // store above becoming visible inside the kernel
                kraw[r].load(delta == 0 ? kn + d0 : kr + (size_t)slot * RS + d0);
                vraw[r].load(delta == 0 ? vn + d0 : vr + (size_t)slot * RS + d0);
            }
        }
        // ---- scores and online softmax over this lane group's taps
#pragma unroll
        for (int r = 0; r < ROUNDS; ++r) {
            const int j = (r0 + r) * GROUPS + g;
            const bool valid = j < t.J && t.delta(j < t.J ? j : 0) < fill;
            float kx[8], vx[8];
            kraw[r].get(kx); vraw[r].get(vx);
            fold_tap<TPR>(st, a, j, h, d0, valid, active, qx, kx, vx);
        }
    }
    merge_and_store<T, TPR>(st, a, sh, h, d0, g == 0 && active);
}

// ---- single-pass variant for bf16 rings --------------------------------------------------
// Every K row of the step is copied asynchronously into shared memory (cp.async, 16 bytes per
// lane, no register held while the copy is in flight), the first VSM rounds of V rows likewise,
// and the remaining V rows are loaded into registers.  All 2*J row requests of a (sequence, head)
// pair are therefore in flight together and the pair costs one memory round trip after head[s],
// at a register count that keeps every warp of the benchmark shape resident.  Each lane reads
// back only the 16 bytes it requested itself, so no barrier is needed after the wait.
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
    const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" :: "r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;\n" ::: "memory"); }

//
// PDL = true is the overlapped form (programmatic dependent launch): the kernel lets the next
// kernel of the stream start at once, and itself reads only head, fill and the ring rows of taps
// with delta > 0 before it waits for the kernels ahead of it; q, k_new, v_new are read and the
// ring and out are written after that wait.  The ring gather of one layer then overlaps the tail
// of whatever runs before it.
template <int TPR, int ROUNDS, int VSM, int CTAS, bool PDL>
__global__ void __launch_bounds__(kWarpsPerBlock * 32, CTAS)
decode_1pass_kernel(const DecodeArgs a, const Taps t) {
    if constexpr (PDL) asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    using T = __nv_bfloat16;
    constexpr int GROUPS = 32 / TPR;
    constexpr int VREG = ROUNDS - VSM;
    __shared__ uint4 k_sm[kWarpsPerBlock][ROUNDS][32];
    __shared__ uint4 v_sm[kWarpsPerBlock][VSM > 0 ? VSM : 1][32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sh = blockIdx.x * kWarpsPerBlock + warp;
    if (sh >= a.S * a.H) return;
    const int s = sh / a.H, h = sh - s * a.H;
    const int g = lane / TPR, li = lane % TPR;
    const int d0 = li * 8, D = a.D;
    const bool active = d0 < D;

    const int head = a.head[s];
    const int fill = a.fill ? a.fill[s] : a.R;
    const T* kn = static_cast<const T*>(a.k_new) + (size_t)sh * D;
    const T* vn = static_cast<const T*>(a.v_new) + (size_t)sh * D;
    const int RS = a.ring_stride;
    T* kr = static_cast<T*>(a.k_ring) + (size_t)sh * a.R * RS;
    T* vr = static_cast<T*>(a.v_ring) + (size_t)sh * a.R * RS;

    // ---- request every row of the step
    Raw8<T> vraw[VREG > 0 ? VREG : 1];
    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
    for (int r = 0; r < ROUNDS; ++r) {
        const int j = r * GROUPS + g;
        const int delta = j < t.J ? t.delta(j) : 0;
        int slot = head - delta;
        if (slot < 0) slot += a.R;
        const bool on = j < t.J && delta < fill && active;
        if (PDL && j == 0 && delta == 0) continue;       // the new token itself: after the wait
        // the tap with delta == 0 reads k_new / v_new, so nothing waits for the ring store below
        const T* ksrc = delta == 0 ? kn + d0 : kr + (size_t)slot * RS + d0;
        const T* vsrc = delta == 0 ? vn + d0 : vr + (size_t)slot * RS + d0;
        if (on) cp_async16(&k_sm[warp][r][lane], ksrc); else k_sm[warp][r][lane] = zero4;
        if (r < VSM) {
            if (on) cp_async16(&v_sm[warp][r][lane], vsrc); else v_sm[warp][r][lane] = zero4;
        } else {
            vraw[r - VSM].zero();
            if (on) vraw[r - VSM].load(vsrc);
        }
    }
    if constexpr (PDL) {
        asm volatile("griddepcontrol.wait;\n" ::: "memory");
        if (g == 0 && t.delta(0) == 0) {                 // offsets ascend: only tap 0 can be delta 0
            const bool on = fill > 0 && active;
            if (on) cp_async16(&k_sm[warp][0][lane], kn + d0); else k_sm[warp][0][lane] = zero4;
            if (VSM > 0) {
                if (on) cp_async16(&v_sm[warp][0][lane], vn + d0); else v_sm[warp][0][lane] = zero4;
            } else {
                vraw[0].zero();
                if (on) vraw[0].load(vn + d0);
            }
        }
    }
    float qx[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (active) load8(static_cast<const T*>(a.q) + (size_t)sh * D + d0, qx);
    if (g == 0 && active) {          // store the new token in the ring
        *reinterpret_cast<uint4*>(kr + (size_t)head * RS + d0) = *reinterpret_cast<const uint4*>(kn + d0);
        *reinterpret_cast<uint4*>(vr + (size_t)head * RS + d0) = *reinterpret_cast<const uint4*>(vn + d0);
    }
    cp_async_wait_all();

    // ---- scores and online softmax over this lane group's taps
    TapState st;
#pragma unroll
    for (int r = 0; r < ROUNDS; ++r) {
        const int j = r * GROUPS + g;
        const bool valid = j < t.J && t.delta(j < t.J ? j : 0) < fill;
        float kx[8], vx[8];
        Raw8<T> kk; kk.u = k_sm[warp][r][lane]; kk.get(kx);
        if (r < VSM) { Raw8<T> vv; vv.u = v_sm[warp][r][lane]; vv.get(vx); }
        else vraw[r - VSM].get(vx);
        fold_tap<TPR>(st, a, j, h, d0, valid, active, qx, kx, vx);
    }
    merge_and_store<T, TPR>(st, a, sh, h, d0, g == 0 && active);
}

template <int TPR, int ROUNDS, int VSM, int CTAS>
cudaError_t decode_launch_1pass(const DecodeArgs& a, const Taps& t, cudaStream_t s, bool overlap) {
    const int pairs = a.S * a.H;
    const unsigned blocks = (pairs + kWarpsPerBlock - 1) / kWarpsPerBlock;
    if (!overlap) {
        decode_1pass_kernel<TPR, ROUNDS, VSM, CTAS, false><<<blocks, kWarpsPerBlock * 32, 0, s>>>(a, t);
        return cudaGetLastError();
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(blocks); cfg.blockDim = dim3(kWarpsPerBlock * 32); cfg.dynamicSmemBytes = 0; cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, decode_1pass_kernel<TPR, ROUNDS, VSM, CTAS, true>, a, t);
}

template <typename T, int TPR, int ROUNDS>
cudaError_t decode_launch_r(const DecodeArgs& a, const Taps& t, cudaStream_t s) {
    const int pairs = a.S * a.H;
    decode_kernel<T, TPR, ROUNDS><<<(pairs + kWarpsPerBlock - 1) / kWarpsPerBlock, kWarpsPerBlock * 32, 0, s>>>(a, t);
    return cudaGetLastError();
}

template <typename T, int TPR>
cudaError_t decode_launch(const DecodeArgs& a, const Taps& t, cudaStream_t s, bool overlap) {
    const int rounds = (t.J + 32 / TPR - 1) / (32 / TPR);
    if constexpr (std::is_same<T, __nv_bfloat16>::value) {
        // bf16 rings, up to 12 rounds: single-pass kernel.  K rows plus four rounds of V rows in
        // shared memory leave 80 registers (6 CTAs per SM); measured 9.95 us per launch on the
        // benchmark shape against 14.4 us for two register passes, 15.1 us with all of V in
        // registers (5 CTAs per SM) and 15.7 us with all of V in shared memory (4 CTAs per SM).
        if (rounds <= 6) return decode_launch_1pass<TPR, 6, 0, 24 / kWarpsPerBlock>(a, t, s, overlap);
        if (rounds <= 12) return decode_launch_1pass<TPR, 12, 4, 24 / kWarpsPerBlock>(a, t, s, overlap);
    }
    // Other cases (fp32 rings, more than 12 rounds): register passes of 6 rounds (96 registers),
    // launched as an ordinary kernel (the overlapped form is a hint, not a requirement).
    return decode_launch_r<T, TPR, 6>(a, t, s);
}
}  // namespace

#define DSQG_DECODE_TPR(T)                                              \
    do {                                                                \
        const int chunks_ = a.D / 8;                                    \
        if (chunks_ <= 1) return decode_launch<T, 1>(a, t, s, overlap);          \
        if (chunks_ <= 2) return decode_launch<T, 2>(a, t, s, overlap);          \
        if (chunks_ <= 4) return decode_launch<T, 4>(a, t, s, overlap);          \
        if (chunks_ <= 8) return decode_launch<T, 8>(a, t, s, overlap);          \
        return decode_launch<T, 16>(a, t, s, overlap);                           \
    } while (0)

// Ring prefill: copies the last min(N, R) positions of K and V from the training layout
// [S,H,N,D] into the rings [S,H,R,D] so that position p lands in slot p mod R, and sets
// head[s] = (N-1) mod R, fill[s] = min(N, R).  One 16-byte chunk per thread.
// ring_chunks: 16-byte chunks between two slots of a ring (chunks_per_row, or twice that when K and V interleave).
__global__ void ring_prefill_kernel(const uint4* __restrict__ k, const uint4* __restrict__ v, uint4* k_ring, uint4* v_ring,
                                    int32_t* head, int32_t* fill, int SH, int H, int N, int R, int chunks_per_row,
                                    int ring_chunks) {
    const int keep = N < R ? N : R;
    const long long total = (long long)SH * keep * chunks_per_row;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int c = (int)(i % chunks_per_row);
        const long long rowi = i / chunks_per_row;
        const int j = (int)(rowi % keep);
        const int sh = (int)(rowi / keep);
        const int p = N - keep + j;                       // position in the sequence
        const int slot = p % R;
        const long long src = ((long long)sh * N + p) * chunks_per_row + c;
        const long long dst = ((long long)sh * R + slot) * ring_chunks + c;
        k_ring[dst] = k[src];
        v_ring[dst] = v[src];
    }
    const int tid = blockIdx.x * blockDim.x + threadIdx.x;
    if (tid < SH / H) { head[tid] = (N - 1) % R; fill[tid] = keep; }
}

cudaError_t launch_ring_prefill(const void* k, const void* v, void* k_ring, void* v_ring, int32_t* head, int32_t* fill,
                                int S, int H, int N, int D, int R, int dtype, cudaStream_t s, bool interleaved) {
    const int chunks = D * (dtype == DSQG_DTYPE_BF16 ? 2 : 4) / 16;
    const long long total = (long long)S * H * (N < R ? N : R) * chunks;
    long long blocks = (total + 255) / 256;
    if (blocks < (S + 255) / 256) blocks = (S + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    ring_prefill_kernel<<<(int)blocks, 256, 0, s>>>(static_cast<const uint4*>(k), static_cast<const uint4*>(v),
                                                  static_cast<uint4*>(k_ring), static_cast<uint4*>(v_ring), head, fill,
                                                  S * H, H, N, R, chunks, interleaved ? 2 * chunks : chunks);
    return cudaGetLastError();
}

cudaError_t launch_decode(const DecodeArgs& a, const Taps& t, int dtype, cudaStream_t s, bool overlap) {
    if (dtype == DSQG_DTYPE_BF16) DSQG_DECODE_TPR(__nv_bfloat16);
    DSQG_DECODE_TPR(float);
}

}  // namespace dsqg
