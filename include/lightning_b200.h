/*
 * C ABI of liblightning_b200.so: Lightning Attention-2 forward/backward and SimpleRMSNorm
 * forward/backward for NVIDIA B200 (sm_100a).
 *
 * Conventions
 *  - Every pointer is a CUDA device pointer owned by the caller unless stated otherwise; the
 *    library never allocates or frees device memory (its only allocation is 256 bytes of pinned host
 *    memory per device for lab200_last_status).
 *  - `stream` is a cudaStream_t passed as void*; all work is enqueued on it and the calls return
 *    without synchronising (except lab200_read_status).
 *  - Return value 0 means the work was enqueued; any other value is an error code
 *    (lab200_error_string) and nothing was enqueued.
 *  - Tensors are contiguous row-major. q, k: (b, h, n, d); v, o: (b, h, n, e).
 *    `slopes` holds h fp32 decay rates (one per head, shared by the batch) or is NULL for no decay.
 *  - dtype codes: LAB200_F32, LAB200_F16, LAB200_BF16. Attention supports F16 and BF16 with
 *    d, e multiples of 16, d <= 256; SRMSNorm supports all three.
 *
 * The entry points replace the device side of the reference's torch.autograd.Functions; the
 * reference file:line each one stands in for is given beside it (paths inside
 * OpenNLPLab/lightning-attention).
 */
#ifndef LIGHTNING_B200_H_
#define LIGHTNING_B200_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LAB200_F32 0
#define LAB200_F16 1
#define LAB200_BF16 2
/* Layout flag, OR-ed into the dtype argument of the attention entry points (lab200_la_generic*, lab200_la2_fwd*,
 * lab200_la2_bwd, lab200_la2_dkdv): every 16-bit tensor of the call is (b, n, h, dim) contiguous - what the projection GEMMs around the
 * op produce and consume (examples/module/tnl_attn.py:56-64 rearranges to (b, h, n, d) and back) - instead of
 * (b, h, n, dim). States stay (bh, dv, dk). Needs bh = b * h with whole batches and dk <= 128. */
#define LAB200_LAYOUT_BNHD 0x100

#define LAB200_OK 0
#define LAB200_ERR_SHAPE 1       /* unsupported or inconsistent sizes */
#define LAB200_ERR_DTYPE 2       /* unsupported dtype code */
#define LAB200_ERR_WORKSPACE 3   /* workspace missing or too small */
#define LAB200_ERR_CUDA 4        /* a CUDA runtime call or launch failed */
#define LAB200_ERR_DRIVER 5      /* the driver lacks cuTensorMapEncodeTiled or refused the tensor map */
#define LAB200_ERR_ALIGN 6       /* a pointer is not 16-byte aligned */
#define LAB200_ERR_SCRATCH_LIMIT 7 /* lab200_la2_fwd_static: the problem needs more than the built-in scratch */

/* Size of the scratch array built into the library for lab200_la2_fwd_static. */
#define LAB200_STATIC_SCRATCH_BYTES (16 * 1024 * 1024)
#define LAB200_ERR_WAIT_INPUT 101 /* device side: a bounded barrier wait ran out (see lab200_read_status) */
#define LAB200_ERR_WAIT_MMA1 102
#define LAB200_ERR_WAIT_MMA2 103

/* Library version, major * 10000 + minor * 100 + patch. */
int lab200_version(void);

/* Number of CUDA kernels this library has launched in this process so far (all entry points,
 * all streams). Bookkeeping for benchmarks; no counterpart in the reference. */
long long lab200_launch_count(void);

/* Profiling aid, off by default: while `device_buffer` is non-NULL, the CTA that handles (batch*head 0,
 * slice 0, chunk 0) of every attention block kernel writes clock64() stamps for each of its first `blocks`
 * 128-token blocks into device_buffer[block * 16 + slot]. Slots 0-5 (serial kernel): block start, inputs landed,
 * first MMA group done, masked tile stored, second MMA group done, epilogue done. Slots 0-11 (pipelined kernel):
 * MMA issuer (0 inputs landed, 1 S and X issued, 2 P ready, 3 PC and D issued), mask group (4 S ready, 5 P stored,
 * 6 Bm scaled), state/output group (7 PC and D done, 8 D consumed, 9 state published, 10 accumulators released,
 * 11 output rows stored). The buffer must hold blocks * 16 64-bit words. Pass NULL to switch it off. No
 * counterpart in the reference. */
void lab200_la_debug_trace(long long* device_buffer, int blocks);

/* Static, human-readable text for an error code. */
const char* lab200_error_string(int code);

/* Number of sequence chunks the library would pick for this problem on the current device when
 * `chunks` = 0 is passed to the calls below (1 = one serial sweep per (batch, head)). */
int lab200_la_plan_chunks(int bh, int n, int dk, int dv);

/* Bytes of workspace the attention calls below need for the given sizes; `chunks` as passed to
 * the call (0 = automatic). Always at least 256 (a status block lives in front). */
size_t lab200_la_workspace_bytes(int bh, int n, int dk, int dv, int chunks);

/*
 * The generic decayed causal product that all four attention results are instances of:
 *   reverse = 0:  out_t = sum_{j<=t} lambda^(t-j) (a_t . bm_j) c_j
 *   reverse = 1:  out_t = sum_{j>=t} lambda^(j-t) (a_t . bm_j) c_j
 * a, bm: (bh, n, dk); c, out: (bh, n, dv); lambda = exp(-slopes[bh % h]).
 * state_in / state_out: optional (bh, dv, dk) fp32 running state entering / leaving the sequence
 * (the transposed d x e "KV" matrix of lightning_attn2.py:55,84), for sequence-parallel chaining and prefill/decode.
 * Forward time: state_out is the state entering token n for any n (a ragged last block is decayed to token n, not to
 * the end of its 128-token tile). Reverse time: chaining requires n to be a multiple of 128.
 * state_only != 0 computes only state_out (a, out may be NULL).
 * chunks: 0 = automatic, otherwise the number of sequence chunks processed by independent CTAs.
 * Stands in for _fwd_kernel (lightning_attn2.py:8-85), _bwd_intra_kernel (:88-183) and
 * _bwd_inter_kernel (:186-395), which are the four role assignments of this product.
 */
int lab200_la_generic(const void* a, const void* bm, const void* c, const float* slopes, void* out,
                      const float* state_in, float* state_out, void* workspace, size_t workspace_bytes,
                      int bh, int h, int n, int dk, int dv, int reverse, int state_only, int chunks,
                      int dtype, void* stream);

/*
 * Second half of a two-step use of lab200_la_generic, for callers that learn `state_in` only after the local states
 * are known (sequence parallelism): step 1 is lab200_la_generic(..., state_only = 1) with a `state_out` buffer, which
 * leaves the per-chunk states of the sequence (from a zero initial state) in `workspace`; step 2 is this call with the
 * SAME bm, c, sizes, reverse, chunks and workspace: it adds the decayed `state_in` (may be NULL) to those states and runs
 * only the block loop, so bm and c are not read a second time for states. No counterpart in the reference.
 */
int lab200_la_generic_resume(const void* a, const void* bm, const void* c, const float* slopes, void* out,
                             const float* state_in, void* workspace, size_t workspace_bytes, int bh, int h,
                             int n, int dk, int dv, int reverse, int chunks, int dtype, void* stream);

/*
 * lab200_la_generic_resume for the product with Bm and C exchanged (dk == dv only). The states a product keeps per
 * chunk are sum lambda^.. bm_t^T c_t laid out (dv, dk); exchanging bm and c transposes them, which is how dk and dv
 * (and forward and dq) are related. `workspace` must come from a call - state-only, full or resumed - on (c, bm) with the
 * same sizes, reverse and chunks; its states are transposed in place (the workspace then belongs to THIS product) and only
 * the block loop runs. rebase != 0: those states started from a zero initial state and the decayed `state_in` is added;
 * rebase == 0: they already include the incoming state. `state_in` ((bh, dv, dk), this product's layout) must be given
 * either way when there is an incoming state: a sequence that is not cut into chunks uses it directly.
 * No counterpart in the reference.
 */
int lab200_la_generic_resume_swapped(const void* a, const void* bm, const void* c, const float* slopes, void* out,
                                     const float* state_in, void* workspace, size_t workspace_bytes, int bh,
                                     int h, int n, int dk, int dv, int reverse, int chunks, int rebase, int dtype,
                                     void* stream);

/*
 * Sequence parallelism: the state entering this rank's shard from the all-gathered shard states.
 * gathered: (ranks, bh, x, y) fp32, entry r = the state shard r contributes from a zero initial state
 * (lab200_la_generic state_out, x = dv, y = dk); every shard holds `shard_tokens` tokens.
 *   reverse == 0:  out = sum_{r < rank} lambda^((rank-1-r) shard_tokens) gathered[r]
 *   reverse != 0:  out = sum_{r > rank} lambda^((r-rank-1) shard_tokens) gathered[r]
 * out: (bh, x, y) and/or out_t: (bh, y, x), the same state transposed (for the product with Bm and C exchanged);
 * either may be NULL. One launch, no workspace. No counterpart in the reference (it is single-GPU).
 */
int lab200_la_combine_states(const float* gathered, const float* slopes, float* out, float* out_t, int ranks,
                             int rank, int bh, int h, int x, int y, long long shard_tokens, int reverse,
                             void* stream);

/*
 * One decode step of the recurrence for every (batch, head) pair, for inference after a prefill with
 * lab200_la_generic(..., state_out):   o = q (S + k^T v),   S <- lambda (S + k^T v).
 * q, k: (bh, dk); v, o: (bh, dv), 16-bit; state: (bh, dv, dk) fp32, updated in place - the state entering the token,
 * i.e. sum_{j<t} lambda^(t-j) k_j^T v_j transposed, exactly what state_out of a forward-time call holds.
 * dk a multiple of 16. One launch, no workspace. No counterpart in the reference (it has no inference path).
 */
int lab200_la_decode_step(const void* q, const void* k, const void* v, const float* slopes, float* state, void* o,
                          int bh, int h, int dk, int dv, int dtype, void* stream);

/* o = LightningAttention2.forward(q, k, v, s): lightning_attn2.py:400-434 (with slopes) and
 * lightning_attn2_no_decay.py:368-400 (slopes = NULL). */
int lab200_la2_fwd(const void* q, const void* k, const void* v, const float* slopes, void* o,
                   void* workspace, size_t workspace_bytes, int b, int h, int n, int d, int e,
                   int chunks, int dtype, void* stream);

/*
 * lab200_la2_fwd for callers that cannot hand over a workspace. It has no counterpart in the reference.
 *
 * Who needs it: code that runs where device memory cannot be obtained at call time -- a plugin whose host
 * passes it only the input and output buffers and offers no allocator, or a serving loop that must not call
 * cudaMalloc because that call synchronises the whole device and may fail once memory is fully committed to
 * other tenants. For them the scratch (status word + per-chunk states) is a fixed array of
 * LAB200_STATIC_SCRATCH_BYTES (16 MiB) inside the library's device image. The price: every GPU that loads the
 * library carries those 16 MiB until the process exits, whether or not this entry point is ever called.
 *
 * Behaviour: same result as lab200_la2_fwd with the same `chunks`. The call allocates and frees nothing.
 * Problems whose workspace (lab200_la_workspace_bytes(b*h, n, d, e, chunks)) exceeds the array are refused with
 * LAB200_ERR_SCRATCH_LIMIT before anything is enqueued; pass chunks = 1 to need only the status word.
 * The first call on each device looks up the array's device address (a host-side runtime query, done once per
 * device with that device current); make that first call outside any stream capture.
 * All calls on a device share the one array: calls whose GPU execution may overlap (different streams, or
 * different host threads on different streams) race on it and must be serialised by the caller.
 */
int lab200_la2_fwd_static(const void* q, const void* k, const void* v, const float* slopes, void* o,
                          int b, int h, int n, int d, int e, int chunks, int dtype, void* stream);

/* dq, dk, dv = LightningAttention2.backward(do): lightning_attn2.py:437-504 and
 * lightning_attn2_no_decay.py:403-468. dq is one forward-time launch of the generic product, dk and dv come out of one
 * fused reverse-time sweep (d, e <= 128; two generic launches otherwise).
 * Workspace size: lab200_la2_bwd_workspace_bytes(b, h, n, d, e, chunks). */
int lab200_la2_bwd(const void* q, const void* k, const void* v, const float* slopes, const void* dout,
                   void* dq, void* dk, void* dv, void* workspace, size_t workspace_bytes, int b, int h,
                   int n, int d, int e, int chunks, int dtype, void* stream);

/* Bytes of workspace lab200_la2_bwd needs: the largest need of the three products it runs ((dk, dv) = (e, d) for dq
 * and for dk/dv, (d, e) for dv on the unfused path), each with its own chunk plan when `chunks` = 0. */
size_t lab200_la2_bwd_workspace_bytes(int b, int h, int n, int d, int e, int chunks);

/*
 * dk and dv of the same backward pass in ONE reverse-time sweep that reads q, k, v, do once and writes dk, dv (6 tensor
 * passes instead of the 8 that two generic launches move); d, e <= 128. Same results as the dk, dv of lab200_la2_bwd.
 * Stands in for the dk/dv halves of _bwd_intra_kernel (lightning_attn2.py:156-162) and for the reverse sweep of
 * _bwd_inter_kernel (:335-395).
 * state_in: optional (b*h, d, e) fp32 reverse-time state sum_t lambda^t q_t^T do_t entering the sequence from tokens
 * after its end (sequence parallelism; needs n % 128 == 0), or NULL.
 * chunks: 0 = automatic, otherwise the number of sequence chunks processed by independent CTAs; with more than one chunk
 * the call first computes the state entering every chunk (a state-only pass over do and q and a scan).
 * resume != 0: `workspace` already holds those per-chunk states from lab200_la_generic(NULL, do, q, ..., dk = e, dv = d,
 * reverse = 1, state_only = 1, same chunks) with a zero initial state; the decayed `state_in` is added and the state-only
 * pass is skipped (the two-step protocol of lab200_la_generic_resume).
 * Workspace: lab200_la_workspace_bytes(b*h, n, e, d, chunks).
 */
int lab200_la2_dkdv(const void* q, const void* k, const void* v, const float* slopes, const void* dout,
                    void* dk, void* dv, const float* state_in, void* workspace, size_t workspace_bytes, int b,
                    int h, int n, int d, int e, int chunks, int resume, int dtype, void* stream);

/* Synchronises `stream` and returns the device-side status word of the last attention call that
 * used `workspace` (0, or one of LAB200_ERR_WAIT_*). Negative: the copy itself failed. */
int lab200_read_status(const void* workspace, void* stream);

/*
 * Status without a host synchronisation. After the last launch of every attention call that takes a workspace the
 * library enqueues a 4-byte copy of the call's status word into a ring (64 slots per device) of pinned host memory,
 * which it allocates with cudaHostAlloc on the first such call on a device (make that call outside stream capture).
 * lab200_last_status() looks through the ring of the current device and returns - and clears - the first non-zero word
 * (a LAB200_ERR_WAIT_* code: a bounded wait of an EARLIER call ran out and that call's outputs are invalid), or 0.
 * It never blocks; the report is at least one call late (the copy runs behind the kernels) and a word that is not
 * collected within 64 later calls is overwritten. The Python operators call it before every launch and raise.
 * No counterpart in the reference (its kernels have no waits that can run out).
 */
int lab200_last_status(void);

/* lab200_read_status for the scratch array built into the library (lab200_la2_fwd_static has no workspace argument
 * to read it from): synchronises `stream` and returns the status word of the last static call on the current device.
 * Allocates nothing. */
int lab200_static_status(void* stream);

/* Test hook for the error path: one tiny kernel waits - with the bounded wait of the block kernels and a budget of
 * `budget_cycles` SM clocks (at most 1e8) - on a barrier nothing arrives on, so the wait runs out and the kernel writes
 * LAB200_ERR_WAIT_INPUT into the workspace's status word and returns; the call then posts the word like every attention
 * call does. No copy, tensor memory or MMA is in flight in that kernel. No counterpart in the reference. */
int lab200_debug_wait_expiry(void* workspace, size_t workspace_bytes, long long budget_cycles, void* stream);

/* y = x * rsqrt(mean(x^2, last dim) + eps), rstd saved per row: _SrmsNorm.forward /
 * srms_norm_fw, srmsnorm.py:12-33, 78-122. x, y: (M, N); rstd: (M) fp32. N * sizeof(elem) <= 65536. */
int lab200_srmsnorm_fwd(const void* x, void* y, float* rstd, long long M, int N, float eps, int dtype,
                        void* stream);

/* dx for the above: _SrmsNorm.backward / srms_norm_bwd_dx_fused, srmsnorm.py:38-74, 125-175. */
int lab200_srmsnorm_bwd(const void* x, const void* dy, const float* rstd, void* dx, long long M, int N,
                        int dtype, void* stream);

/*
 * SimpleRMSNorm followed by a sigmoid gate in one pass, the epilogue of the reference's example caller
 * (examples/module/tnl_attn.py:66-69: norm, sigmoid(gate), multiply - with this repo's SimpleRMSNorm as the norm):
 *   forward : y = x * rstd * sigmoid(gate)
 *   backward: dx and dgate from dy (see csrc/srmsnorm_kernels.cuh)
 * x, gate, y, dy, dx, dgate: (M, N) row-major of one dtype; rstd: (M) fp32. Rows must be vectorisable: N a multiple of
 * 8 (16-bit) or 4 (fp32) and at most 16384 / 8192 elements, pointers 16-byte aligned; LAB200_ERR_SHAPE / _ALIGN otherwise
 * (compose lab200_srmsnorm_* with element-wise kernels then). No counterpart kernel in the reference.
 */
int lab200_srmsnorm_gate_fwd(const void* x, const void* gate, void* y, float* rstd, long long M, int N, float eps,
                             int dtype, void* stream);
int lab200_srmsnorm_gate_bwd(const void* x, const void* gate, const void* dy, const float* rstd, void* dx,
                             void* dgate, long long M, int N, int dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* LIGHTNING_B200_H_ */
