/*
 * btp_sm100.h - C ABI of libbtp_sm100.so: block two-pass (BTP) sliding-window
 * recurrence, forward and backward, hand-written for NVIDIA B200 (sm_100a).
 *
 * These entry points are what a foreign-function binding for the reference's
 * native extension `spear._btp` would bind.  They replace
 *   forward (coeff, x, y, checkpoint, k, wpb)             csrc/btp/_bindings.cu:76-150
 *   backward(coeff, x, dy, checkpoint, dx, dA, k, wpb)    csrc/btp/_bindings.cu:152-229
 * and the launchers behind them (csrc/btp/btp-forward.cu:462-527,
 * csrc/btp/btp-backwards.cu:811-884).
 *
 * Contract shared by every entry point
 *  - All tensor pointers are DEVICE pointers on the current CUDA device, dense
 *    and contiguous:  x, y, dy, dx : [B, H, 16, L]   coeff, dA : [B, H, L]
 *    checkpoint : [B, H, L/16, 16] float (slot j = carry into block j+1).
 *  - L is a multiple of 16.  Pointers are 16-byte aligned.
 *  - The library never allocates, frees or synchronises; it enqueues one kernel
 *    on `stream` (a cudaStream_t passed as void*; NULL = the legacy default
 *    stream) and returns.  Every element of y, dx and dA is written.
 *  - Return value: BTP_OK or a negative BTP_ERR_* code; nothing is printed and
 *    the process is never aborted.  btp_sm100_status_string() names a code and
 *    btp_sm100_last_error() gives the detail recorded by the calling thread's
 *    most recent failing call.
 *  - Calls are re-entrant and thread-safe.
 *  - Stream order is kept: a kernel never reads or writes memory before all earlier work in `stream` has
 *    completed.  (The forward and backward kernels are launched with programmatic stream serialization, so
 *    their launch may be processed while the previous kernel still runs; they wait for it before touching
 *    memory.  Set BTP_SM100_PDL=0 in the environment for plain launches.)
 */
#ifndef BTP_SM100_H_
#define BTP_SM100_H_

#ifdef __cplusplus
extern "C" {
#endif

#define BTP_SM100_ABI_VERSION 4

/* status codes */
#define BTP_OK 0
#define BTP_ERR_NULL_POINTER (-1)
#define BTP_ERR_BAD_SHAPE (-2)      /* B, H, L <= 0, L % 16 != 0, or sizes beyond int32 tile counts */
#define BTP_ERR_BAD_ORDER (-3)      /* k not in {1, 2} */
#define BTP_ERR_BAD_DTYPE (-4)
#define BTP_ERR_MISALIGNED (-5)     /* a pointer is not 16-byte aligned */
#define BTP_ERR_CUDA (-6)           /* a CUDA runtime / driver call failed; see btp_sm100_last_error() */
#define BTP_ERR_UNSUPPORTED_DEVICE (-7) /* current device is not compute capability 10.x */
#define BTP_ERR_DEVICE_TIMEOUT (-8) /* a bounded wait inside a kernel gave up (btp_sm100_device_status) */
#define BTP_ERR_TOO_LARGE (-9)      /* problem exceeds the built-in scratch of btp_sm100_forward_noalloc */

/* dtype tags.  x and dx are 16-bit: bfloat16 unless the call says float16 (the reference takes both,
 * csrc/btp/_bindings.cu:29-31).  A call says float16 activations through its coefficient tag: BTP_DTYPE_F16 (a
 * float16 coefficient), or BTP_DTYPE_F32 / BTP_DTYPE_F32_LOG or'ed with BTP_ACT_F16.  y and dy are float32 or the
 * activations' own 16-bit type. */
#define BTP_DTYPE_BF16 0        /* x, y, dy, dx, coeff */
#define BTP_DTYPE_F32 1         /* y, dy;  coeff given in linear space as float */
#define BTP_DTYPE_F32_LOG 2     /* coeff only: natural log of the coefficient, float (superset of the reference) */
#define BTP_DTYPE_F16 3         /* x, y, dy, dx, coeff as float16 */
#define BTP_ACT_F16 0x10        /* flag on a float coefficient tag: the activations are float16 */

/*
 * Forward:  y = btp(coeff, x).
 * Replaces spear._btp.forward (csrc/btp/_bindings.cu:76-150 -> btp-forward.cu:85-457).
 *   coeff        [B,H,L]      coeff_dtype: BTP_DTYPE_BF16 | BTP_DTYPE_F16 | BTP_DTYPE_F32 | BTP_DTYPE_F32_LOG (see the tags)
 *   x            [B,H,16,L]   bf16 (float16 when the coefficient tag says so)
 *   y            [B,H,16,L]   out_dtype: x's type | BTP_DTYPE_F32
 *   checkpoint   [B,H,L/16,16] float, or NULL.  When given and k == 2, slot j < L/16-1 receives the
 *                block-local last token of block j, exactly the tensor the reference's forward
 *                saves (btp-forward.cu:369-373).  The backward below does not need it.
 *   k            2 = local pass + one-hop carry, 1 = local pass only (interface.py:164-188)
 */
int btp_sm100_forward(const void* coeff, const void* x, void* y, float* checkpoint,
                      int B, int H, int L, int k, int coeff_dtype, int out_dtype, void* stream);

/*
 * Backward:  (dx, dA) for upstream gradient dy.
 * Replaces spear._btp.backward (csrc/btp/_bindings.cu:152-229 -> btp-backwards.cu:165-808).
 *   dy           [B,H,16,L]   dy_dtype: x's type | BTP_DTYPE_F32
 *   checkpoint   accepted for signature compatibility and ignored (may be NULL): the carry is
 *                recomputed from x and coeff, which costs no extra memory traffic.
 *   dx           [B,H,16,L]   x's type
 *   dA           [B,H,L]      float, gradient w.r.t. the linear coefficient (w.r.t. the log
 *                coefficient when coeff_dtype == BTP_DTYPE_F32_LOG)
 */
int btp_sm100_backward(const void* coeff, const void* x, const void* dy, const float* checkpoint,
                       void* dx, float* dA, int B, int H, int L, int k,
                       int coeff_dtype, int dy_dtype, void* stream);

/*
 * Forward that also produces the carry checkpoint, but keeps it in memory that is part of the library
 * image instead of memory the caller has to provide.
 * No counterpart in the reference (there the Python wrapper allocates the checkpoint with torch.empty,
 * spear/ops/btp/interface.py:142).
 *
 * Who this is for: callers that want the reference's forward behaviour (y plus the per-block carry
 * record) but are not in a position to allocate device memory for the record at call time - a serving
 * process whose whole device memory was handed to an arena at start-up, code running under a framework
 * allocator it must not bypass, a plugin that only ever receives its input and output buffers.  They pass
 * coeff, x and y exactly as for btp_sm100_forward and nothing else.
 *
 * The record goes to a fixed array of BTP_SM100_NOALLOC_MAX_HEAD_TOKENS floats (4 MiB) that every GPU
 * holds from the moment it loads the library until the process exits.  The call returns
 * BTP_ERR_TOO_LARGE when B*H*L exceeds that number; use btp_sm100_forward with your own buffer then.
 * (With k == 1 there is no carry and no record: the array is not touched and the limit does not apply.)
 * The entry point itself never calls cudaMalloc, cudaFree or any other allocating routine.
 *
 * First call on each device: it looks up the device address of the array (one cudaGetSymbolAddress with
 * that device current) and keeps it; make this first call outside any stream capture.
 * The array is shared by all calls and keeps the contents of the last one.  Nothing in it has to start
 * at zero (every slot that is ever read is written by the same launch), but two calls whose kernels
 * overlap on the GPU (different streams) write the same slots and race: serialise them.
 */
#define BTP_SM100_NOALLOC_MAX_HEAD_TOKENS (1 << 20)
int btp_sm100_forward_noalloc(const void* coeff, const void* x, void* y, int B, int H, int L, int k,
                              int coeff_dtype, int out_dtype, void* stream);

/*
 * Copies the first n_floats of the record that btp_sm100_forward_noalloc keeps inside the library into `dst`
 * (device memory of the caller, current device), in stream order.  No counterpart in the reference.  The layout
 * is the checkpoint's, [B, H, L/16, 16] of the last btp_sm100_forward_noalloc call with k == 2 on this device; a
 * caller that wants the record (the reference's backward reads it, btp-backwards.cu:374-378) fetches it here, and
 * the tests use it to check that the kernel really wrote to this device's copy of the array.  Allocates nothing.
 */
int btp_sm100_noalloc_read_record(float* dst, long long n_floats, void* stream);

/*
 * Gated forward in token-major layout: the Phalanx layer's glue fused around the op.
 * Replaces, in one kernel, spear/nn/phalanx/swr.py:216-219 (a = sigmoid(A_logits), X = sigmoid(B_logits) * V),
 * the two transposing copies of spear/ops/btp/interface.py:186-187, spear._btp.forward, and
 * swr.py:320-323 (y * C + V and the permute back to [B, L, H*16]).
 *   a_logits  [B, L, H]      bf16, row pitch ld_a elements (>= H)
 *   b_logits  [B, L, H*16]   bf16, row pitch ld_b   \  pitches are multiples of 8 elements, bases 16-byte aligned;
 *   c, v      [B, L, H*16]   bf16, pitches ld_c, ld_v } the four inputs may be column slices of one wide
 *   out       [B, L, H*16]   bf16, pitch ld_out      /  projection output
 *   H % 4 == 0, L % 16 == 0, k as in btp_sm100_forward.
 *   kv_heads  number of key/value heads, a divisor of H.  With kv_heads < H, b_logits and c are
 *             [B, L, kv_heads*16] and head h uses the columns of key/value head h / (H / kv_heads), as KVRepeat
 *             does (spear/nn/phalanx/swr.py:96-103, 209-214) - read in place, nothing is repeated in memory.
 * out = btp(sigmoid(a_logits), sigmoid(b_logits) * v) * c + v, with the decay rounded to bf16 as the layer does.
 */
int btp_sm100_gated_forward(const void* a_logits, const void* b_logits, const void* c, const void* v, void* out,
                            int B, int L, int H, int kv_heads, long long ld_a, long long ld_b, long long ld_c,
                            long long ld_v, long long ld_out, int k, void* stream);

/*
 * Backward of btp_sm100_gated_forward, token-major throughout.  Replaces autograd through
 * spear/nn/phalanx/swr.py:216-219 and 320-323, the transposing copies (interface.py:186-187, 154) and
 * spear._btp.backward.  Everything the forward computed is recomputed from the four inputs.
 *   dout                      [B, L, H*16] bf16  gradient of `out`
 *   da_logits                 [B, L, H]    bf16  (pitch a multiple of 4 elements, base 8-byte aligned)
 *   db_logits, dc, dv         [B, L, H*16] bf16
 * Pitches (elements) follow the pointers in the same order; constraints as for the forward.
 * With kv_heads < H, b_logits and c are [B, L, kv_heads*16] (read in place, as in the forward).  db_logits and
 * dc are then [B, L, H*16 / r]: the kernel sums the gradients of runs of r neighbouring heads that share a
 * key/value head - r = 4 when the group size H / kv_heads is a multiple of 4, r = 2 when it is 2, r = 1
 * otherwise.  For groups of 2 and 4 that is the gradient of the key/value head itself, [B, L, kv_heads*16];
 * for larger or odd groups the caller adds up the group / r partial sums per key/value head (columns
 * [kv][group / r][16]; autograd does the whole sum for KVRepeat).
 */
int btp_sm100_gated_backward(const void* a_logits, const void* b_logits, const void* c, const void* v, const void* dout,
                             void* da_logits, void* db_logits, void* dc, void* dv, int B, int L, int H, int kv_heads,
                             long long ld_a, long long ld_b, long long ld_c, long long ld_v, long long ld_do,
                             long long ld_da, long long ld_db, long long ld_dc, long long ld_dv, int k, void* stream);

/*
 * One decode step of the streaming form of the recurrence, all of it in one launch.
 * Replaces the tensor-op body of step_jagged (spear/nn/phalanx/inference.py:177-266).
 *   a_t                      [n_heads]      gate of the new token (its natural log when gate_is_log)
 *   x_t, c_t, v_t, y_t       [n_heads,16]   n_heads = B*H, rows contiguous
 *   h_loc, c_prev_loc        [n_heads,16]   state going in (JagState.h_loc, .c_prev_loc)
 *   r_pref                   [n_heads]      state going in: running gate product of the current block, or its
 *                                           log when r_is_log; NULL stands for an empty block (1, or log 1)
 *   h_loc_out, r_pref_out    state coming out, separate buffers (the reference returns a new state object and
 *                            leaves the old one valid); passing the input pointers updates in place
 *   c_prev_loc_out           written only when block_complete (the step with in-block index 15); may be NULL
 *                            otherwise - c_prev_loc carries over unchanged
 *   dtype                    storage of the [n_heads,16] tensors, gate_dtype that of a_t and r_pref:
 *                            BTP_DTYPE_BF16 | BTP_DTYPE_F32.  Arithmetic is fp32; one rounding on the store.
 *   y = (h + r * c_prev_loc) * c_t + v_t  with  h = a * h_loc + x_t,  r = a * r_pref
 *   (log space: r = exp(r_pref + log(max(a, tiny)))).
 */
int btp_sm100_decode_step(const void* a_t, const void* x_t, const void* c_t, const void* v_t, void* y_t,
                          const void* h_loc, const void* r_pref, const void* c_prev_loc, void* h_loc_out,
                          void* r_pref_out, void* c_prev_loc_out, long long n_heads, int block_complete,
                          int gate_is_log, int r_is_log, int dtype, int gate_dtype, void* stream);

/*
 * Hand-off state after a prompt of L tokens (any L >= 1), one launch.
 * Replaces the state extraction at the end of parallel_jagged (spear/nn/phalanx/inference.py:333-358), which
 * there falls out of two nested Python loops over the whole prompt; the state only depends on the last
 * (possibly partial) 16-token block and the complete block before it.
 *   a   [n_heads, L]      gates (log gates when gate_is_log), contiguous
 *   x   [n_heads, 16, L]  driving term, contiguous
 *   h_loc, c_prev_loc [n_heads,16], r_pref [n_heads]: outputs (r_pref always in linear space, as the reference's)
 */
int btp_sm100_prefill_state(const void* a, const void* x, void* h_loc, void* r_pref, void* c_prev_loc, long long n_heads,
                            int L, int gate_is_log, int dtype, int gate_dtype, void* stream);

/* Name of a status code ("BTP_OK", "BTP_ERR_BAD_SHAPE", ...).  Never NULL. */
const char* btp_sm100_status_string(int status);

/* Detail text of the calling thread's most recent failing call ("" if none).  Never NULL. */
const char* btp_sm100_last_error(void);

/*
 * Synchronises `stream` and reads the device-side error word that the kernels set when one of
 * their bounded waits gives up.  Returns BTP_OK, BTP_ERR_DEVICE_TIMEOUT or BTP_ERR_CUDA.
 * `detail`, if not NULL, receives 4 words: {code, blockIdx.x, warp, chunk}.  The word is cleared.
 * Not on the hot path: the forward/backward calls themselves never synchronise.
 */
int btp_sm100_device_status(void* stream, unsigned int* detail);

/*
 * How long a wait inside a kernel may last before the kernel gives up, records the error word that
 * btp_sm100_device_status reports, lets its copies in flight land and returns (default 2 s; 0 restores the
 * default).  Applies to every launch that follows, process-wide.  Returns the previous
 * value.  No counterpart in the reference, whose kernels wait on cluster barriers without a bound
 * (csrc/btp/btp-forward.cu:340-347).
 */
unsigned long long btp_sm100_set_wait_limit(unsigned long long ns);

/*
 * How the forward kernel gets the carry across a seam, i.e. where the stretch of a sequence one warp works on ends
 * and another warp's begins (sequences longer than 256 tokens; the result is the same to rounding either way):
 *   BTP_SEAM_RECOMPUTE (default)  the warp on the right re-reads the one 16-token block to its left and recomputes
 *                                 the 16 numbers; no warp ever waits for another.
 *   BTP_SEAM_HANDOFF              the warp on the left hands the 16 numbers over through distributed shared memory
 *                                 inside a thread-block cluster, which is what the reference does between the CTAs
 *                                 of its cluster (csrc/btp/btp-forward.cu:276-335, csrc/btp/btp_common.h:56-64).
 *                                 Taken for k = 2, a 16-bit y without checkpoint, L a multiple of 128 and 2 ... 32
 *                                 stretches per sequence (a power of two); every other call recomputes.
 * Applies to every forward launch that follows, process-wide.  Returns the previous mode; any other value of
 * `mode` changes nothing and returns the current mode.
 */
#define BTP_SEAM_RECOMPUTE 0
#define BTP_SEAM_HANDOFF 1
int btp_sm100_set_seam_mode(int mode);

/*
 * Launch shape of the last btp_sm100_forward / btp_sm100_backward kernel the CALLING THREAD launched: the number of
 * CTAs and the thread-block cluster size (1 unless BTP_SEAM_HANDOFF applied).  Either pointer may be NULL.  A
 * diagnostic with no counterpart in the reference; the hand-off's grid is one wave of resident clusters, which is
 * fewer CTAs than the device holds without clusters.
 */
void btp_sm100_last_launch(int* grid, int* cluster);

/*
 * Test hook for the give-up path, no counterpart in the reference: the NEXT forward or backward launch makes
 * warp 0 of block 0 expect `bytes` more bytes on its first load barrier than its loads deliver, so that this
 * one wait runs out.  The kernel then behaves as documented for a timeout: it returns normally, the chunks of
 * that warp stay unwritten, btp_sm100_device_status reports BTP_ERR_DEVICE_TIMEOUT once.  Nothing faults or
 * hangs; combine it with a short btp_sm100_set_wait_limit so that the test takes milliseconds.
 */
void btp_sm100_test_expect_missing_bytes(unsigned int bytes);

/* Number of kernels this library has launched in this process (all threads). */
unsigned long long btp_sm100_launch_count(void);

/* ABI version of the loaded library (BTP_SM100_ABI_VERSION at build time). */
int btp_sm100_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* BTP_SM100_H_ */
