/* dsqg_b200.h -- C ABI of the B200-native DSQG attention library (libdsqg_b200.so).
 *
 * DSQG = Dyadic Sparse Q-K Gather attention, the hot operator of Lanerra/DWARF: for
 * every query row n of every (batch, head) pair, score a fixed ascending set of J causal
 * offsets delta_j,
 *
 *     s_j = q[n].k[n-delta_j] / sqrt(D) + pos_bias[j,h] (+ q[n].scale_embed[j] / sqrt(D)),
 *     s_j = -inf where n - delta_j < 0,
 *     out[n] = head_gain[h] * sum_j softmax_j(s)_j * v[n-delta_j].
 *
 * Conventions shared by every entry point
 *   - q, k, v, out, dout, dq, dk, dv: DEVICE pointers, contiguous [B,H,N,D], element type
 *     selected by `dtype` (DSQG_DTYPE_BF16 or DSQG_DTYPE_F32), 16-byte aligned.
 *   - pos_bias [J,H], scale_embed [J,D] (nullable), head_gain [H] (nullable), lse [B,H,N]:
 *     DEVICE pointers to fp32.
 *   - offsets: HOST pointer to J int32 values, strictly ascending, >= 0.  The leading run
 *     of consecutive integers is treated as the dense window, the rest as sparse taps.
 *   - stream: a cudaStream_t passed as void* (NULL = legacy default stream).
 *   - The caller owns every buffer; the library allocates nothing.  The only state it keeps
 *     between calls is named where it is declared: the kernel-path knob
 *     (dsqg_set_kernel_path), the device error word (dsqg_device_error), the built-in scratch
 *     of dsqg_bwd_static with its per-device address cache, and per-kernel "attribute set"
 *     flags.  The caller makes the device current (cudaSetDevice) before calling.
 *   - Every function returns DSQG_OK (0) or a negative dsqg_status; nothing throws, traps
 *     or aborts.  Argument errors are detected on the host before any launch.
 *   - D must be a multiple of 8, 8 <= D <= 128; J <= DSQG_MAX_TAPS.
 */
#ifndef DSQG_B200_H
#define DSQG_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DSQG_MAX_TAPS 128

typedef enum {
    DSQG_OK = 0,
    DSQG_ERR_NULL_POINTER = -1,   /* a required pointer is NULL */
    DSQG_ERR_BAD_SHAPE = -2,      /* B,H,N,D,J,R,S out of the supported range (B*H <= 65535 for fwd/bwd) */
    DSQG_ERR_BAD_OFFSETS = -3,    /* offsets not strictly ascending / negative */
    DSQG_ERR_BAD_DTYPE = -4,      /* dtype is neither DSQG_DTYPE_BF16 nor DSQG_DTYPE_F32 */
    DSQG_ERR_MISALIGNED = -5,     /* a tensor pointer is not 16-byte aligned */
    DSQG_ERR_SCRATCH_TOO_SMALL = -6,
    DSQG_ERR_CUDA = -7,           /* a CUDA runtime/driver call failed (see dsqg_last_cuda_error) */
    DSQG_ERR_UNSUPPORTED = -8,    /* valid request that this build has no kernel for */
    DSQG_ERR_STATIC_SCRATCH_EXCEEDED = -9  /* dsqg_bwd_static: problem needs more than DSQG_STATIC_SCRATCH_BYTES */
} dsqg_status;

enum { DSQG_DTYPE_BF16 = 0, DSQG_DTYPE_F32 = 1 };

/* Human-readable text for a status code.  Never NULL. */
const char* dsqg_status_str(int status);

/* Text of the last CUDA error seen by the calling thread inside this library ("" if none). */
const char* dsqg_last_cuda_error(void);

/* Library version, major*10000 + minor*100 + patch. */
int dsqg_version(void);

/* Testing knob with no counterpart in the reference: 0 = choose kernels automatically
 * (default), 1 = always use the generic CUDA-core kernels, 2 = the tensor-core kernels (what the
 * automatic choice uses where they apply), 3 = the forward with TMA-staged V wherever it applies
 * (not chosen automatically: it measures slower on B200), 4 = the forward whose dense window runs
 * on tcgen05 tensor cores with accumulators in tensor memory (bf16, no scale_embed, dense window
 * within offsets 0..32; D = 32 with up to 16 sparse taps, D = 64 without sparse taps; every other
 * call goes to the automatic choice; chosen automatically only where it measures faster: D = 64,
 * no sparse taps, at least 296 tiles of 128 rows).  Process-wide state. */
int dsqg_set_kernel_path(int path);

/* Device-side error word of the current device (no counterpart in the reference).  The
 * kernels that wait on shared-memory barriers for the copy engine or the tensor cores (kernel paths 3 and 4) bound every
 * such wait; a wait that runs out records its site id here and the kernel returns with
 * unspecified output instead of hanging.  0 = no error, -1 = the word could not be read.
 * Synchronises the device.  reset != 0 clears the word after reading. */
int dsqg_device_error(int reset);

/* Test hook for the bounded wait (no counterpart in the reference): launches one thread that
 * waits, for at most limit_cycles SM cycles (1 .. 2e9), on a barrier nothing signals.  The wait
 * gives up, dsqg_device_error() then reports site 0x7e57, and the kernel returns: nothing is
 * in flight, nothing hangs or faults. */
int dsqg_test_wait_timeout(long long limit_cycles, void* stream);

/* Forward.
 * Replaces: _DSQGFn.forward / _DSQGFnV3.forward + the _fwd/_fwd_v3 kernels
 *   (DWARF kernels/dsqg_attention_v2.py:337-363, kernels/dsqg_attention_v3.py:359-387,
 *   :60-163) and the native precedent dsqg_forward_cuda
 *   (kernels/dsqg_cuda/dsqg_cuda_kernel.cu:496-519); the `* if_gain` of
 *   train/train_2048_condU.py:187 is fused into the epilogue through head_gain.
 * Writes out [B,H,N,D] (dtype) and lse [B,H,N] fp32 (natural log of the softmax
 * denominator, as the reference saves it).  A row with no valid tap gets out = 0 and
 * lse = -inf. */
int dsqg_fwd(const void* q, const void* k, const void* v,
             const float* pos_bias, const float* scale_embed, const float* head_gain,
             const int32_t* offsets, int J,
             void* out, float* lse,
             int B, int H, int N, int D, int dtype, void* stream);

/* Bytes of device scratch dsqg_bwd needs for this problem (0 on invalid arguments). */
size_t dsqg_bwd_scratch_bytes(int J, int B, int H, int N, int D, int has_scale_embed);

/* Backward.
 * Replaces: _DSQGFn.backward / _DSQGFnV3.backward and their three kernels _compute_D,
 *   _bwd_dq, _bwd_dkdv (kernels/dsqg_attention_v3.py:170-352, :389-442) and
 *   dsqg_backward_cuda (kernels/dsqg_cuda/dsqg_cuda_kernel.cu:582-609).
 * Inputs: the forward's inputs, its out and lse, and the upstream gradient dout.
 * Writes dq, dk, dv (dtype), dpos_bias [J,H] fp32, and, when the matching input is
 * given, dscale_embed [J,D] fp32 and dhead_gain [H] fp32.  Parameter gradients are
 * produced by per-block partial sums in `scratch` followed by a fixed-order reduction:
 * no atomics, bitwise reproducible from run to run. */
int dsqg_bwd(const void* q, const void* k, const void* v,
             const float* pos_bias, const float* scale_embed, const float* head_gain,
             const int32_t* offsets, int J,
             const void* out, const float* lse, const void* dout,
             void* dq, void* dk, void* dv,
             float* dpos_bias, float* dscale_embed, float* dhead_gain,
             void* scratch, size_t scratch_bytes,
             int B, int H, int N, int D, int dtype, void* stream);

/* Backward without a caller-supplied scratch buffer.  No counterpart in the reference (its
 * extensions allocate through PyTorch); it exists for callers that cannot allocate device
 * memory at all -- e.g. a server that hands all of its device memory to a fixed arena at
 * start-up, or a plugin host that lends the plugin nothing but the tensors of the call.
 * Same arguments and results as dsqg_bwd minus scratch/scratch_bytes; the scratch is a
 * DSQG_STATIC_SCRATCH_BYTES array built into the library (each GPU that loads the library
 * holds those bytes until the process exits).  The call allocates and frees nothing.
 *   - Problems with dsqg_bwd_scratch_bytes(...) > DSQG_STATIC_SCRATCH_BYTES are refused with
 *     DSQG_ERR_STATIC_SCRATCH_EXCEEDED before anything is launched.
 *   - The first call on each device looks up that device's copy of the array (the device must
 *     be current, as for every entry point); make that first call outside any stream capture.
 *     The address is kept until the process exits: use the device's primary context (what the
 *     CUDA runtime gives you) and do not call cudaDeviceReset while the library is loaded.
 *   - All calls on a device share the one array and it keeps whatever the last call left; the
 *     kernels overwrite every word they later read, so nothing has to be cleared.  Two calls
 *     that may run on the GPU at the same time (different streams) race on it: serialise them. */
#define DSQG_STATIC_SCRATCH_BYTES (8u << 20)
int dsqg_bwd_static(const void* q, const void* k, const void* v,
                    const float* pos_bias, const float* scale_embed, const float* head_gain,
                    const int32_t* offsets, int J,
                    const void* out, const float* lse, const void* dout,
                    void* dq, void* dk, void* dv,
                    float* dpos_bias, float* dscale_embed, float* dhead_gain,
                    int B, int H, int N, int D, int dtype, void* stream);

/* dsqg_bwd restricted to some of its kernels: a profiling aid with no counterpart in the
 * reference.  `stages` is a bit mask: DSQG_BWD_STAGE_DQ (dQ, delta and the parameter-gradient
 * partials), DSQG_BWD_STAGE_DKDV (dK, dV; needs the delta a previous DQ stage left in the same
 * scratch), DSQG_BWD_STAGE_REDUCE (fixed-order reduction of the partials into dpos_bias,
 * dscale_embed, dhead_gain).  Running the three stages one after the other on one stream with
 * the same scratch is exactly dsqg_bwd. */
#define DSQG_BWD_STAGE_DQ 1
#define DSQG_BWD_STAGE_DKDV 2
#define DSQG_BWD_STAGE_REDUCE 4
#define DSQG_BWD_STAGE_ALL 7
int dsqg_bwd_stages(const void* q, const void* k, const void* v,
                    const float* pos_bias, const float* scale_embed, const float* head_gain,
                    const int32_t* offsets, int J,
                    const void* out, const float* lse, const void* dout,
                    void* dq, void* dk, void* dv,
                    float* dpos_bias, float* dscale_embed, float* dhead_gain,
                    void* scratch, size_t scratch_bytes,
                    int B, int H, int N, int D, int dtype, void* stream, int stages);

/* 1 if dsqg_fwd and dsqg_bwd run the tensor-core kernels for this dtype, head dimension, offset
 * set and use of scale_embed, 0 if they run the CUDA-core kernels (or the arguments are invalid).
 * Replaces: nothing (the reference has one kernel family); a host uses it to decide whether
 * zero-padding the head dimension (dsqg_fwd_scaled) pays.  No launch, no device access. */
int dsqg_tensor_core_path(int dtype, int D, const int32_t* offsets, int J, int has_scale_embed);

/* dsqg_fwd / dsqg_bwd with the score scale given by the caller instead of 1/sqrt(D):
 *     s_j = scale * q[n].(k[n-delta_j] [+ scale_embed[j]]) + pos_bias[j,h].
 * Replaces: the power-of-two padding of the head dimension inside the reference's kernels
 *   (BLOCK_HD = next_power_of_2(HD) with masked lanes, kernels/dsqg_attention_v2.py:344): a host
 *   that zero-pads q, k, v (and scale_embed, dout) from HD = 80 to 96 columns calls these with
 *   D = 96 and scale = 1/sqrt(80), gets the tensor-core kernels, and drops the padded columns of
 *   the results (they are exactly zero).  scale must be positive and finite
 *   (DSQG_ERR_UNSUPPORTED otherwise).  Everything else as dsqg_fwd / dsqg_bwd. */
int dsqg_fwd_scaled(const void* q, const void* k, const void* v,
                    const float* pos_bias, const float* scale_embed, const float* head_gain,
                    const int32_t* offsets, int J, void* out, float* lse,
                    int B, int H, int N, int D, int dtype, void* stream, float scale);
int dsqg_bwd_scaled(const void* q, const void* k, const void* v,
                    const float* pos_bias, const float* scale_embed, const float* head_gain,
                    const int32_t* offsets, int J,
                    const void* out, const float* lse, const void* dout,
                    void* dq, void* dk, void* dv,
                    float* dpos_bias, float* dscale_embed, float* dhead_gain,
                    void* scratch, size_t scratch_bytes,
                    int B, int H, int N, int D, int dtype, void* stream, float scale);

/* Strided tensors: the caller's layouts instead of contiguous [B,H,N,D] copies.
 * Replaces: the three transposing copies a DWARF attention module makes before the op and the
 *   permute + gate multiply after it -- `view(B,N,H,HD).permute(0,2,1,3).contiguous()` on each of
 *   q, k, v (train/train_2048_condU.py:171-175, kernels/dsqg_attention_v2.py:462-467), then
 *   `out.permute(0,2,1,3).reshape(B,N,D)` and `* torch.sigmoid(self.gate_proj(x))`
 *   (train/train_2048_condU.py:189-191) -- and the autograd backward of those PyTorch ops.
 * A dsqg_strides gives the ELEMENT strides of the batch, head and row index of a tensor whose D
 * elements per (batch, head, row) are contiguous; all three must be multiples of 8 (16 bytes).
 *   qkv_strides: layout shared by q, k, v (and by dq, dk, dv in the backward).  For the output of a
 *     fused qkv projection, [B,N,3*H*D] seen as [B,N,3,H,D]: {N*3*H*D, D, 3*H*D}, with q, k, v
 *     pointing at elements 0, H*D and 2*H*D of that buffer.
 *   out_strides: layout shared by out, gate (and by dout in the backward).  Token-major
 *     [B,N,H*D]: {N*H*D, D, H*D}.
 *   gate (dsqg_fwd_strided, nullable): bf16 tensor laid out like out; the kernel writes
 *     out * sigmoid(gate).  With a gate, dsqg_gate_bwd turns the gradient dy of that product into
 *     the dout, dgate and delta ([B,H,N] fp32 = sum_d dy*y) that dsqg_bwd_strided takes; y is the
 *     forward's (gated) output, which is also what dsqg_bwd_strided gets as `out`.  Without a gate
 *     pass delta_pre = NULL and the forward's output and its gradient as out and dout.
 * lse, dpos_bias, dhead_gain, scratch (dsqg_bwd_scratch_bytes(..., 0)) are as in dsqg_fwd / dsqg_bwd.
 * bf16 only, and only shapes the tensor-core kernels take
 * (dsqg_tensor_core_path(...) == 1): DSQG_ERR_UNSUPPORTED otherwise, so that a caller can fall
 * back to the copies.  scale <= 0 selects 1/sqrt(D). */
typedef struct { long long batch, head, row; } dsqg_strides;
int dsqg_fwd_strided(const void* q, const void* k, const void* v, const dsqg_strides* qkv_strides,
                     const float* pos_bias, const float* head_gain, const int32_t* offsets, int J,
                     void* out, const dsqg_strides* out_strides, const void* gate, float* lse,
                     int B, int H, int N, int D, int dtype, void* stream, float scale);
int dsqg_bwd_strided(const void* q, const void* k, const void* v, const dsqg_strides* qkv_strides,
                     const float* pos_bias, const float* head_gain, const int32_t* offsets, int J,
                     const void* out, const float* lse, const void* dout, const dsqg_strides* out_strides,
                     const float* delta_pre,
                     void* dq, void* dk, void* dv, float* dpos_bias, float* dhead_gain,
                     void* scratch, size_t scratch_bytes,
                     int B, int H, int N, int D, int dtype, void* stream, float scale);
/* The same two entries with the reference's scale_embed term (dsqg_attention_v3,
 * kernels/dsqg_attention_v3.py:112-118; the op of DSQGAttentionQW, train/train_2048_condU.py:184):
 * scale_embed [J,D] fp32 is required, dscale_embed [J,D] fp32 receives its gradient, the scratch
 * size is dsqg_bwd_scratch_bytes(..., 1), D <= 64. */
int dsqg_fwd_strided_se(const void* q, const void* k, const void* v, const dsqg_strides* qkv_strides,
                        const float* pos_bias, const float* scale_embed, const float* head_gain,
                        const int32_t* offsets, int J,
                        void* out, const dsqg_strides* out_strides, const void* gate, float* lse,
                        int B, int H, int N, int D, int dtype, void* stream, float scale);
int dsqg_bwd_strided_se(const void* q, const void* k, const void* v, const dsqg_strides* qkv_strides,
                        const float* pos_bias, const float* scale_embed, const float* head_gain,
                        const int32_t* offsets, int J,
                        const void* out, const float* lse, const void* dout, const dsqg_strides* out_strides,
                        const float* delta_pre,
                        void* dq, void* dk, void* dv, float* dpos_bias, float* dscale_embed, float* dhead_gain,
                        void* scratch, size_t scratch_bytes,
                        int B, int H, int N, int D, int dtype, void* stream, float scale);
int dsqg_gate_bwd(const void* dy, const void* y, const void* gate, const dsqg_strides* strides,
                  void* dout, void* dgate, float* delta, int B, int H, int N, int D, void* stream);

/* Causal mean along the sequence of a contiguous [B,N,D] tensor (bf16 or fp32, D a multiple of 8):
 *   reverse == 0:  out[b,n,:] = (x[b,0,:] + ... + x[b,n,:]) / (n + 1)
 *   reverse != 0:  out[b,n,:] = sum_{m >= n} x[b,m,:] / (m + 1)        (the adjoint: its backward pass)
 * Replaces: the pooling of the condU "interference" block that feeds the K/V injection of its DSQG
 *   layer, `pool = xi.cumsum(dim=1) / counts` (DWARF train/train_2048_condU.py:289-292), and the
 *   autograd backward of those two PyTorch ops.  fp32 accumulation, fixed order of additions, no
 *   scratch memory; out may not alias x. */
int dsqg_causal_mean(const void* x, void* out, int B, int N, int D, int dtype, int reverse, void* stream);

/* Single-token decode over a circular K/V ring buffer.
 * Replaces: nothing executable -- the reference only describes the O(1) cache in prose
 *   (DWARF README.md:175-179; generate() in train/train_2048_condU.py:463-487 re-runs the
 *   whole prefix).  Semantics are those of dsqg_fwd's last row on the time-ordered ring.
 * q, k_new, v_new, out: [S,H,D]; k_ring, v_ring: [S,H,R,D] (updated in place: the new
 * k, v are stored in slot head[s] before the taps are read); head: DEVICE int32 [S],
 * 0 <= head[s] < R; fill: DEVICE int32 [S] = number of valid tokens in the ring counting
 * the new one, or NULL for a full ring.  Tap j reads slot (head - delta_j) mod R and is
 * valid iff delta_j < fill[s].  Requires max(offsets) < R. */
int dsqg_decode(const void* q, const void* k_new, const void* v_new,
                void* k_ring, void* v_ring, const int32_t* head, const int32_t* fill,
                const float* pos_bias, const float* scale_embed, const float* head_gain,
                const int32_t* offsets, int J, int R,
                void* out, int S, int H, int D, int dtype, void* stream);

/* dsqg_decode / dsqg_ring_prefill over ONE ring per layer that holds the key and the value of a slot
 * side by side: kv_ring [S,H,R,2,D] (slot-major; element 0 of the pair is the key row, element 1 the
 * value row).  A tap is then one contiguous read of 2*D elements and a step touches half as many
 * memory pages as with two separate rings.  Same semantics, arguments and results as dsqg_decode
 * (overlapped != 0: as dsqg_decode_overlapped) and dsqg_ring_prefill otherwise.
 * Replaces: nothing executable (see dsqg_decode). */
int dsqg_decode_kv(const void* q, const void* k_new, const void* v_new, void* kv_ring,
                   const int32_t* head, const int32_t* fill,
                   const float* pos_bias, const float* scale_embed, const float* head_gain,
                   const int32_t* offsets, int J, int R,
                   void* out, int S, int H, int D, int dtype, void* stream, int overlapped);
int dsqg_ring_prefill_kv(const void* k, const void* v, void* kv_ring,
                         int32_t* head, int32_t* fill, int S, int H, int N, int D, int R, int dtype, void* stream);

/* dsqg_decode launched so that it overlaps the kernel ahead of it in the stream (programmatic
 * dependent launch).  Same arguments and results as dsqg_decode.
 * Replaces: nothing executable (see dsqg_decode).
 * The kernel starts while the previous kernel of the stream may still be running and, before it
 * waits for that kernel, reads head, fill and the ring rows of every tap with delta > 0; q, k_new,
 * v_new are read, and the rings and out written, only after the wait.  The caller therefore
 * promises that the kernel launched just before this call on the same stream writes none of
 * head, fill, k_ring, v_ring of THIS call (true for a stack of layers that each own their rings
 * and share one write head advanced once per token, after some other kernel).  It also lets the
 * kernel launched after it start early if that kernel was launched in the same way; an ordinary
 * kernel after it waits as usual.  bf16 rings with at most 12 taps per lane group (J <= 48 at
 * D = 64, J <= 96 at D = 32) take this form; other cases run exactly as dsqg_decode. */
int dsqg_decode_overlapped(const void* q, const void* k_new, const void* v_new,
                           void* k_ring, void* v_ring, const int32_t* head, const int32_t* fill,
                           const float* pos_bias, const float* scale_embed, const float* head_gain,
                           const int32_t* offsets, int J, int R,
                           void* out, int S, int H, int D, int dtype, void* stream);

/* Fills the decode rings from a training-layout prefix.
 * Replaces: nothing executable (the reference has no cache; its generate() re-runs the whole
 *   prefix, DWARF train/train_2048_condU.py:463-487).
 * k, v: [S,H,N,D]; k_ring, v_ring: [S,H,R,D].  Position p of every sequence is copied to slot
 * p mod R for the last min(N,R) positions; head[s] = (N-1) mod R and fill[s] = min(N,R) are
 * written (DEVICE int32 [S]).  The next token then goes to slot (head+1) mod R with fill+1
 * (capped at R), which is what dsqg_decode expects. */
int dsqg_ring_prefill(const void* k, const void* v, void* k_ring, void* v_ring,
                      int32_t* head, int32_t* fill, int S, int H, int N, int D, int R, int dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* DSQG_B200_H */
