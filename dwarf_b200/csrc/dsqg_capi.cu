// C ABI of libdsqg_b200.so: argument validation on the host, then dispatch to the
// sm_100a kernels.  Declarations and the reference interfaces they replace are in
// include/dsqg_b200.h.  Nothing here allocates or throws; the little state the library keeps
// between calls (kernel-path knob, error word, built-in scratch) lives in other files.
#include <cmath>
#include <cstdio>
#include <cstring>

#include <nvtx3/nvToolsExt.h>

#include "dsqg_common.cuh"

namespace dsqg {

// NVTX range around the launches of one entry point (visible in Nsight timelines; a no-op when no
// tool is attached).
struct NvtxRange {
    explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
    ~NvtxRange() { nvtxRangePop(); }
};

static thread_local char g_cuda_err[256] = "";

static int cuda_fail(cudaError_t e) {
    snprintf(g_cuda_err, sizeof(g_cuda_err), "%s: %s", cudaGetErrorName(e), cudaGetErrorString(e));
    return DSQG_ERR_CUDA;
}

static inline bool misaligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) != 0; }

// Validates the offsets and splits them into the dense run and the sparse taps.
static int build_taps(const int32_t* offsets, int J, Taps* t) {
    if (!offsets) return DSQG_ERR_NULL_POINTER;
    if (J < 1 || J > DSQG_MAX_TAPS) return DSQG_ERR_BAD_SHAPE;
    if (offsets[0] < 0) return DSQG_ERR_BAD_OFFSETS;
    for (int j = 1; j < J; ++j)
        if (offsets[j] <= offsets[j - 1]) return DSQG_ERR_BAD_OFFSETS;
    memset(t, 0, sizeof(*t));
    t->J = J;
    t->d_lo = offsets[0];
    int nd = 1;
    while (nd < J && offsets[nd] == offsets[nd - 1] + 1) ++nd;
    t->n_dense = nd;
    t->n_sparse = J - nd;
    for (int j = nd; j < J; ++j) t->sparse[j - nd] = offsets[j];
    return DSQG_OK;
}

static int check_shape(int B, int H, int N, int D, int dtype) {
    if (dtype != DSQG_DTYPE_BF16 && dtype != DSQG_DTYPE_F32) return DSQG_ERR_BAD_DTYPE;
    if (B < 1 || H < 1 || N < 1 || D < 8 || D > 128 || (D % 8) != 0) return DSQG_ERR_BAD_SHAPE;
    if ((long long)B * H > 0x7fffffffLL / 2 || (long long)B * H * N > 0x7fffffffLL) return DSQG_ERR_BAD_SHAPE;
    return DSQG_OK;
}

// Forward and backward launch one grid row per (batch, head) pair: B*H is bounded by the grid's y extent.
static int check_op_shape(int B, int H, int N, int D, int dtype) {
    const int rc = check_shape(B, H, N, D, dtype);
    if (rc) return rc;
    return (long long)B * H > 65535 ? DSQG_ERR_BAD_SHAPE : DSQG_OK;
}

}  // namespace dsqg

using namespace dsqg;

extern "C" {

const char* dsqg_status_str(int status) {
    switch (status) {
        case DSQG_OK: return "ok";
        case DSQG_ERR_NULL_POINTER: return "a required pointer is NULL";
        case DSQG_ERR_BAD_SHAPE: return "shape out of range (need B,H,N >= 1; B*H <= 65535 for forward/backward; D a multiple of 8 in [8,128]; 1 <= J <= 128)";
        case DSQG_ERR_BAD_OFFSETS: return "offsets must be non-negative and strictly ascending (and < R for decode)";
        case DSQG_ERR_BAD_DTYPE: return "dtype must be DSQG_DTYPE_BF16 (0) or DSQG_DTYPE_F32 (1)";
        case DSQG_ERR_MISALIGNED: return "tensor pointers must be 16-byte aligned";
        case DSQG_ERR_SCRATCH_TOO_SMALL: return "scratch buffer smaller than dsqg_bwd_scratch_bytes()";
        case DSQG_ERR_CUDA: return "CUDA error (see dsqg_last_cuda_error)";
        case DSQG_ERR_UNSUPPORTED: return "no kernel for this configuration";
        case DSQG_ERR_STATIC_SCRATCH_EXCEEDED:
            return "dsqg_bwd_static: this problem needs more scratch than the built-in DSQG_STATIC_SCRATCH_BYTES; "
                   "use dsqg_bwd with a caller-allocated buffer";
        default: return "unknown status";
    }
}

const char* dsqg_last_cuda_error(void) { return g_cuda_err; }

int dsqg_version(void) { return 100; }

int dsqg_tensor_core_path(int dtype, int D, const int32_t* offsets, int J, int has_scale_embed) {
    Taps t;
    if (check_shape(1, 1, 1, D, dtype) || build_taps(offsets, J, &t)) return 0;
    return mma_fwd_supported(dtype, D, t, has_scale_embed != 0) && mma_path_supported(dtype, D, t, has_scale_embed != 0) ? 1 : 0;
}

static inline bool bad_strides(const dsqg_strides* s) {
    return s->batch < 0 || s->head < 0 || s->row < 0 || (s->batch % 8) || (s->head % 8) || (s->row % 8);
}

// scale <= 0 selects the operator's own 1/sqrt(D); in_st / out_st == NULL: contiguous [B,H,N,D]
static int fwd_impl(const void* q, const void* k, const void* v,
                    const float* pos_bias, const float* scale_embed, const float* head_gain,
                    const int32_t* offsets, int J, void* out, float* lse,
                    int B, int H, int N, int D, int dtype, void* stream, float scale,
                    const dsqg_strides* in_st = nullptr, const dsqg_strides* out_st = nullptr, const void* gate = nullptr) {
    if (!q || !k || !v || !pos_bias || !out || !lse) return DSQG_ERR_NULL_POINTER;
    int rc = check_op_shape(B, H, N, D, dtype);
    if (rc) return rc;
    Taps t;
    rc = build_taps(offsets, J, &t);
    if (rc) return rc;
    if (misaligned16(q) || misaligned16(k) || misaligned16(v) || misaligned16(out) ||
        (scale_embed && misaligned16(scale_embed)))
        return DSQG_ERR_MISALIGNED;
    FwdArgs a;
    a.q = q; a.k = k; a.v = v; a.pos_bias = pos_bias; a.scale_embed = scale_embed;
    a.head_gain = head_gain; a.out = out; a.lse = lse;
    a.B = B; a.H = H; a.N = N; a.D = D;
    a.scale = scale > 0.f ? scale : 1.0f / sqrtf((float)D);
    a.strided = 0; a.gate = nullptr;
    a.in_sb = a.in_sh = a.in_sn = a.out_sb = a.out_sh = a.out_sn = 0;
    NvtxRange range(in_st ? "dsqg_fwd_strided" : "dsqg_fwd");
    if (in_st) {
        // strided tensors exist for the tensor-core kernels only
        if (!out_st) return DSQG_ERR_NULL_POINTER;
        if (bad_strides(in_st) || bad_strides(out_st) || (gate && misaligned16(gate))) return DSQG_ERR_MISALIGNED;
        if (!mma_fwd_supported(dtype, D, t, scale_embed != nullptr)) return DSQG_ERR_UNSUPPORTED;
        a.strided = 1; a.gate = gate;
        a.in_sb = in_st->batch; a.in_sh = in_st->head; a.in_sn = in_st->row;
        a.out_sb = out_st->batch; a.out_sh = out_st->head; a.out_sn = out_st->row;
        cudaError_t e = launch_fwd_mma(a, t, static_cast<cudaStream_t>(stream));
        return e == cudaSuccess ? DSQG_OK : cuda_fail(e);
    }
    cudaError_t e = launch_fwd(a, t, dtype, static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? DSQG_OK : cuda_fail(e);
}

int dsqg_fwd(const void* q, const void* k, const void* v,
             const float* pos_bias, const float* scale_embed, const float* head_gain,
             const int32_t* offsets, int J, void* out, float* lse,
             int B, int H, int N, int D, int dtype, void* stream) {
    return fwd_impl(q, k, v, pos_bias, scale_embed, head_gain, offsets, J, out, lse, B, H, N, D, dtype, stream, 0.f);
}

int dsqg_fwd_scaled(const void* q, const void* k, const void* v,
                    const float* pos_bias, const float* scale_embed, const float* head_gain,
                    const int32_t* offsets, int J, void* out, float* lse,
                    int B, int H, int N, int D, int dtype, void* stream, float scale) {
    if (!(scale > 0.f) || !(scale < 3.0e38f)) return DSQG_ERR_UNSUPPORTED;
    return fwd_impl(q, k, v, pos_bias, scale_embed, head_gain, offsets, J, out, lse, B, H, N, D, dtype, stream, scale);
}

int dsqg_fwd_strided(const void* q, const void* k, const void* v, const dsqg_strides* qkv_strides,
                     const float* pos_bias, const float* head_gain, const int32_t* offsets, int J,
                     void* out, const dsqg_strides* out_strides, const void* gate, float* lse,
                     int B, int H, int N, int D, int dtype, void* stream, float scale) {
    if (!qkv_strides || !out_strides) return DSQG_ERR_NULL_POINTER;
    if (scale > 3.0e38f) return DSQG_ERR_UNSUPPORTED;
    return fwd_impl(q, k, v, pos_bias, nullptr, head_gain, offsets, J, out, lse, B, H, N, D, dtype, stream, scale,
                    qkv_strides, out_strides, gate);
}

size_t dsqg_bwd_scratch_bytes(int J, int B, int H, int N, int D, int has_scale_embed) {
    if (J < 1 || J > DSQG_MAX_TAPS || check_op_shape(B, H, N, D, DSQG_DTYPE_BF16)) return 0;
    // every kernel family tiles at kMinRowsPerBwdTile rows or coarser; with scale_embed the larger of
    // the generic kernels' need (512-row partials) and the tensor-core kernels' need (per-row table,
    // per-tile and per-group partials, prepared tables) is reported
    size_t need = bwd_scratch_need(kMinRowsPerBwdTile, J, B, H, N, D, false);
    if (!has_scale_embed) return need;
    need += bwd_scratch_need(512, J, B, H, N, D, true);
    const size_t mma_se = bwd_scratch_need_mma_se(J, B, H, N, D);
    return mma_se > need ? mma_se : need;
}

int dsqg_bwd(const void* q, const void* k, const void* v,
             const float* pos_bias, const float* scale_embed, const float* head_gain,
             const int32_t* offsets, int J,
             const void* out, const float* lse, const void* dout,
             void* dq, void* dk, void* dv,
             float* dpos_bias, float* dscale_embed, float* dhead_gain,
             void* scratch, size_t scratch_bytes,
             int B, int H, int N, int D, int dtype, void* stream) {
    return dsqg_bwd_stages(q, k, v, pos_bias, scale_embed, head_gain, offsets, J, out, lse, dout,
                           dq, dk, dv, dpos_bias, dscale_embed, dhead_gain, scratch, scratch_bytes,
                           B, H, N, D, dtype, stream, DSQG_BWD_STAGE_ALL);
}

static int bwd_impl(const void* q, const void* k, const void* v,
                    const float* pos_bias, const float* scale_embed, const float* head_gain,
                    const int32_t* offsets, int J,
                    const void* out, const float* lse, const void* dout,
                    void* dq, void* dk, void* dv,
                    float* dpos_bias, float* dscale_embed, float* dhead_gain,
                    void* scratch, size_t scratch_bytes,
                    int B, int H, int N, int D, int dtype, void* stream, int stages, float scale,
                    const dsqg_strides* in_st = nullptr, const dsqg_strides* out_st = nullptr,
                    const float* delta_pre = nullptr);

int dsqg_bwd_stages(const void* q, const void* k, const void* v,
                    const float* pos_bias, const float* scale_embed, const float* head_gain,
                    const int32_t* offsets, int J,
                    const void* out, const float* lse, const void* dout,
                    void* dq, void* dk, void* dv,
                    float* dpos_bias, float* dscale_embed, float* dhead_gain,
                    void* scratch, size_t scratch_bytes,
                    int B, int H, int N, int D, int dtype, void* stream, int stages) {
    return bwd_impl(q, k, v, pos_bias, scale_embed, head_gain, offsets, J, out, lse, dout, dq, dk, dv,
                    dpos_bias, dscale_embed, dhead_gain, scratch, scratch_bytes, B, H, N, D, dtype, stream, stages, 0.f);
}

int dsqg_bwd_scaled(const void* q, const void* k, const void* v,
                    const float* pos_bias, const float* scale_embed, const float* head_gain,
                    const int32_t* offsets, int J,
                    const void* out, const float* lse, const void* dout,
                    void* dq, void* dk, void* dv,
                    float* dpos_bias, float* dscale_embed, float* dhead_gain,
                    void* scratch, size_t scratch_bytes,
                    int B, int H, int N, int D, int dtype, void* stream, float scale) {
    if (!(scale > 0.f) || !(scale < 3.0e38f)) return DSQG_ERR_UNSUPPORTED;
    return bwd_impl(q, k, v, pos_bias, scale_embed, head_gain, offsets, J, out, lse, dout, dq, dk, dv,
                    dpos_bias, dscale_embed, dhead_gain, scratch, scratch_bytes, B, H, N, D, dtype, stream,
                    DSQG_BWD_STAGE_ALL, scale);
}

static int bwd_impl(const void* q, const void* k, const void* v,
                    const float* pos_bias, const float* scale_embed, const float* head_gain,
                    const int32_t* offsets, int J,
                    const void* out, const float* lse, const void* dout,
                    void* dq, void* dk, void* dv,
                    float* dpos_bias, float* dscale_embed, float* dhead_gain,
                    void* scratch, size_t scratch_bytes,
                    int B, int H, int N, int D, int dtype, void* stream, int stages, float scale,
                    const dsqg_strides* in_st, const dsqg_strides* out_st, const float* delta_pre) {
    if (stages < 1 || stages > DSQG_BWD_STAGE_ALL) return DSQG_ERR_UNSUPPORTED;
    if (!q || !k || !v || !pos_bias || !out || !lse || !dout || !dq || !dk || !dv || !dpos_bias || !scratch)
        return DSQG_ERR_NULL_POINTER;
    if (scale_embed && !dscale_embed) return DSQG_ERR_NULL_POINTER;
    if (head_gain && !dhead_gain) return DSQG_ERR_NULL_POINTER;
    int rc = check_op_shape(B, H, N, D, dtype);
    if (rc) return rc;
    Taps t;
    rc = build_taps(offsets, J, &t);
    if (rc) return rc;
    if (misaligned16(q) || misaligned16(k) || misaligned16(v) || misaligned16(out) || misaligned16(dout) ||
        misaligned16(dq) || misaligned16(dk) || misaligned16(dv) || misaligned16(scratch) ||
        (scale_embed && misaligned16(scale_embed)))
        return DSQG_ERR_MISALIGNED;
    if (scratch_bytes < dsqg_bwd_scratch_bytes(J, B, H, N, D, scale_embed != nullptr))
        return DSQG_ERR_SCRATCH_TOO_SMALL;

    BwdArgs a;
    a.q = q; a.k = k; a.v = v; a.pos_bias = pos_bias; a.scale_embed = scale_embed; a.head_gain = head_gain;
    a.out = out; a.lse = lse; a.dout = dout; a.dq = dq; a.dk = dk; a.dv = dv;
    a.dpos_bias = dpos_bias; a.dscale_embed = dscale_embed; a.dhead_gain = head_gain ? dhead_gain : nullptr;
    a.scratch = scratch; a.scratch_bytes = scratch_bytes;
    a.delta = a.dpb_part = a.dg_part = a.dse_part = nullptr;
    a.n_tiles = a.tiles_per_bh = a.n_dse_blocks = 0;
    a.B = B; a.H = H; a.N = N; a.D = D;
    a.scale = scale > 0.f ? scale : 1.0f / sqrtf((float)D);
    a.strided = 0; a.delta_pre = nullptr;
    a.in_sb = a.in_sh = a.in_sn = a.out_sb = a.out_sh = a.out_sn = 0;
    NvtxRange range(in_st ? "dsqg_bwd_strided" : "dsqg_bwd");
    if (in_st) {
        if (!out_st) return DSQG_ERR_NULL_POINTER;
        if (bad_strides(in_st) || bad_strides(out_st)) return DSQG_ERR_MISALIGNED;
        if (!mma_path_supported(dtype, D, t, scale_embed != nullptr)) return DSQG_ERR_UNSUPPORTED;
        a.strided = 1; a.delta_pre = delta_pre;
        a.in_sb = in_st->batch; a.in_sh = in_st->head; a.in_sn = in_st->row;
        a.out_sb = out_st->batch; a.out_sh = out_st->head; a.out_sn = out_st->row;
        cudaError_t e = launch_bwd_mma(a, t, static_cast<cudaStream_t>(stream), stages);
        return e == cudaSuccess ? DSQG_OK : cuda_fail(e);
    }
    cudaError_t e = launch_bwd(a, t, dtype, static_cast<cudaStream_t>(stream), stages);
    return e == cudaSuccess ? DSQG_OK : cuda_fail(e);
}

int dsqg_bwd_strided(const void* q, const void* k, const void* v, const dsqg_strides* qkv_strides,
                     const float* pos_bias, const float* head_gain, const int32_t* offsets, int J,
                     const void* out, const float* lse, const void* dout, const dsqg_strides* out_strides,
                     const float* delta_pre,
                     void* dq, void* dk, void* dv, float* dpos_bias, float* dhead_gain,
                     void* scratch, size_t scratch_bytes,
                     int B, int H, int N, int D, int dtype, void* stream, float scale) {
    if (!qkv_strides || !out_strides) return DSQG_ERR_NULL_POINTER;
    if (scale > 3.0e38f) return DSQG_ERR_UNSUPPORTED;
    return bwd_impl(q, k, v, pos_bias, nullptr, head_gain, offsets, J, out, lse, dout, dq, dk, dv,
                    dpos_bias, nullptr, dhead_gain, scratch, scratch_bytes, B, H, N, D, dtype, stream,
                    DSQG_BWD_STAGE_ALL, scale, qkv_strides, out_strides, delta_pre);
}

int dsqg_fwd_strided_se(const void* q, const void* k, const void* v, const dsqg_strides* qkv_strides,
                        const float* pos_bias, const float* scale_embed, const float* head_gain,
                        const int32_t* offsets, int J,
                        void* out, const dsqg_strides* out_strides, const void* gate, float* lse,
                        int B, int H, int N, int D, int dtype, void* stream, float scale) {
    if (!qkv_strides || !out_strides || !scale_embed) return DSQG_ERR_NULL_POINTER;
    if (scale > 3.0e38f) return DSQG_ERR_UNSUPPORTED;
    return fwd_impl(q, k, v, pos_bias, scale_embed, head_gain, offsets, J, out, lse, B, H, N, D, dtype, stream, scale,
                    qkv_strides, out_strides, gate);
}

int dsqg_bwd_strided_se(const void* q, const void* k, const void* v, const dsqg_strides* qkv_strides,
                        const float* pos_bias, const float* scale_embed, const float* head_gain,
                        const int32_t* offsets, int J,
                        const void* out, const float* lse, const void* dout, const dsqg_strides* out_strides,
                        const float* delta_pre,
                        void* dq, void* dk, void* dv, float* dpos_bias, float* dscale_embed, float* dhead_gain,
                        void* scratch, size_t scratch_bytes,
                        int B, int H, int N, int D, int dtype, void* stream, float scale) {
    if (!qkv_strides || !out_strides || !scale_embed) return DSQG_ERR_NULL_POINTER;
    if (scale > 3.0e38f) return DSQG_ERR_UNSUPPORTED;
    return bwd_impl(q, k, v, pos_bias, scale_embed, head_gain, offsets, J, out, lse, dout, dq, dk, dv,
                    dpos_bias, dscale_embed, dhead_gain, scratch, scratch_bytes, B, H, N, D, dtype, stream,
                    DSQG_BWD_STAGE_ALL, scale, qkv_strides, out_strides, delta_pre);
}

int dsqg_gate_bwd(const void* dy, const void* y, const void* gate, const dsqg_strides* strides,
                  void* dout, void* dgate, float* delta, int B, int H, int N, int D, void* stream) {
    if (!dy || !y || !gate || !strides || !dout || !dgate || !delta) return DSQG_ERR_NULL_POINTER;
    int rc = check_op_shape(B, H, N, D, DSQG_DTYPE_BF16);
    if (rc) return rc;
    if (bad_strides(strides) || misaligned16(dy) || misaligned16(y) || misaligned16(gate) || misaligned16(dout) ||
        misaligned16(dgate))
        return DSQG_ERR_MISALIGNED;
    cudaError_t e = launch_gate_bwd(dy, y, gate, strides->batch, strides->head, strides->row, dout, dgate, delta,
                                    B, H, N, D, static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? DSQG_OK : cuda_fail(e);
}

static int decode_impl(const void* q, const void* k_new, const void* v_new,
                       void* k_ring, void* v_ring, const int32_t* head, const int32_t* fill,
                       const float* pos_bias, const float* scale_embed, const float* head_gain,
                       const int32_t* offsets, int J, int R,
                       void* out, int S, int H, int D, int dtype, void* stream, bool overlap, bool interleaved = false) {
    if (!q || !k_new || !v_new || !k_ring || !v_ring || !head || !pos_bias || !out) return DSQG_ERR_NULL_POINTER;
    int rc = check_shape(S, H, 1, D, dtype);
    if (rc) return rc;
    if (R < 1 || (long long)S * H * R * (interleaved ? 2 : 1) > 0x7fffffffLL) return DSQG_ERR_BAD_SHAPE;
    Taps t;
    rc = build_taps(offsets, J, &t);
    if (rc) return rc;
    if (offsets[J - 1] >= R) return DSQG_ERR_BAD_OFFSETS;
    if (misaligned16(q) || misaligned16(k_new) || misaligned16(v_new) || misaligned16(k_ring) ||
        misaligned16(v_ring) || misaligned16(out) || (scale_embed && misaligned16(scale_embed)))
        return DSQG_ERR_MISALIGNED;
    DecodeArgs a;
    a.q = q; a.k_new = k_new; a.v_new = v_new; a.k_ring = k_ring; a.v_ring = v_ring;
    a.head = head; a.fill = fill; a.pos_bias = pos_bias; a.scale_embed = scale_embed;
    a.head_gain = head_gain; a.out = out; a.S = S; a.H = H; a.D = D; a.R = R;
    a.scale = 1.0f / sqrtf((float)D);
    a.ring_stride = interleaved ? 2 * D : D;
    NvtxRange range(interleaved ? "dsqg_decode_kv" : "dsqg_decode");
    cudaError_t e = launch_decode(a, t, dtype, static_cast<cudaStream_t>(stream), overlap);
    return e == cudaSuccess ? DSQG_OK : cuda_fail(e);
}

int dsqg_decode(const void* q, const void* k_new, const void* v_new,
                void* k_ring, void* v_ring, const int32_t* head, const int32_t* fill,
                const float* pos_bias, const float* scale_embed, const float* head_gain,
                const int32_t* offsets, int J, int R,
                void* out, int S, int H, int D, int dtype, void* stream) {
    return decode_impl(q, k_new, v_new, k_ring, v_ring, head, fill, pos_bias, scale_embed, head_gain,
                       offsets, J, R, out, S, H, D, dtype, stream, false);
}

int dsqg_decode_overlapped(const void* q, const void* k_new, const void* v_new,
                           void* k_ring, void* v_ring, const int32_t* head, const int32_t* fill,
                           const float* pos_bias, const float* scale_embed, const float* head_gain,
                           const int32_t* offsets, int J, int R,
                           void* out, int S, int H, int D, int dtype, void* stream) {
    return decode_impl(q, k_new, v_new, k_ring, v_ring, head, fill, pos_bias, scale_embed, head_gain,
                       offsets, J, R, out, S, H, D, dtype, stream, true);
}

int dsqg_causal_mean(const void* x, void* out, int B, int N, int D, int dtype, int reverse, void* stream) {
    if (!x || !out) return DSQG_ERR_NULL_POINTER;
    if (dtype != DSQG_DTYPE_BF16 && dtype != DSQG_DTYPE_F32) return DSQG_ERR_BAD_DTYPE;
    if (B < 1 || N < 1 || D < 8 || (D % 8) != 0 || B > 65535 || (long long)B * N * D > 0x7fffffffffLL) return DSQG_ERR_BAD_SHAPE;
    if (misaligned16(x) || misaligned16(out)) return DSQG_ERR_MISALIGNED;
    cudaError_t e = launch_causal_mean(x, out, B, N, D, dtype, reverse != 0, static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? DSQG_OK : cuda_fail(e);
}

int dsqg_decode_kv(const void* q, const void* k_new, const void* v_new, void* kv_ring,
                   const int32_t* head, const int32_t* fill,
                   const float* pos_bias, const float* scale_embed, const float* head_gain,
                   const int32_t* offsets, int J, int R,
                   void* out, int S, int H, int D, int dtype, void* stream, int overlapped) {
    if (!kv_ring) return DSQG_ERR_NULL_POINTER;
    if (check_shape(S, H, 1, D, dtype)) return check_shape(S, H, 1, D, dtype);
    char* v_ring = static_cast<char*>(kv_ring) + (size_t)D * (dtype == DSQG_DTYPE_BF16 ? 2 : 4);
    return decode_impl(q, k_new, v_new, kv_ring, v_ring, head, fill, pos_bias, scale_embed, head_gain,
                       offsets, J, R, out, S, H, D, dtype, stream, overlapped != 0, true);
}

int dsqg_ring_prefill_kv(const void* k, const void* v, void* kv_ring,
                         int32_t* head, int32_t* fill, int S, int H, int N, int D, int R, int dtype, void* stream) {
    if (!k || !v || !kv_ring || !head || !fill) return DSQG_ERR_NULL_POINTER;
    int rc = check_shape(S, H, N, D, dtype);
    if (rc) return rc;
    if (R < 1 || (long long)S * H * R * 2 > 0x7fffffffLL) return DSQG_ERR_BAD_SHAPE;
    if (misaligned16(k) || misaligned16(v) || misaligned16(kv_ring)) return DSQG_ERR_MISALIGNED;
    char* v_ring = static_cast<char*>(kv_ring) + (size_t)D * (dtype == DSQG_DTYPE_BF16 ? 2 : 4);
    cudaError_t e = launch_ring_prefill(k, v, kv_ring, v_ring, head, fill, S, H, N, D, R, dtype,
                                        static_cast<cudaStream_t>(stream), true);
    return e == cudaSuccess ? DSQG_OK : cuda_fail(e);
}

int dsqg_ring_prefill(const void* k, const void* v, void* k_ring, void* v_ring,
                      int32_t* head, int32_t* fill, int S, int H, int N, int D, int R, int dtype, void* stream) {
    if (!k || !v || !k_ring || !v_ring || !head || !fill) return DSQG_ERR_NULL_POINTER;
    int rc = check_shape(S, H, N, D, dtype);
    if (rc) return rc;
    if (R < 1 || (long long)S * H * R > 0x7fffffffLL) return DSQG_ERR_BAD_SHAPE;
    if (misaligned16(k) || misaligned16(v) || misaligned16(k_ring) || misaligned16(v_ring)) return DSQG_ERR_MISALIGNED;
    cudaError_t e = launch_ring_prefill(k, v, k_ring, v_ring, head, fill, S, H, N, D, R, dtype, static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? DSQG_OK : cuda_fail(e);
}

}  // extern "C"
