/*
 * webgpt_b200 — C ABI of the B200 (sm_100a) implementation of WebGPT's GPT-2 forward path.
 *
 * Every entry point names the piece of the reference (0hq/WebGPT) it stands in for, as
 * file:line inside that project. The reference drives a WebGPU device from JavaScript; a
 * Node N-API addon (or any FFI) binds these functions one to one.
 *
 * Conventions
 *  - All functions return a status code (WGPT_OK or a negative WGPT_ERR_*); nothing throws or
 *    aborts across this boundary. wgpt_last_error() returns the message of the calling
 *    thread's most recent failure.
 *  - Device memory is passed as plain device addresses (void* / float* obtained from
 *    wgpt_buffer_create or from any other CUDA allocation of the same device). Host memory is
 *    named *_host.
 *  - All work of a device is ordered on that device's stream. Calls that return data to the
 *    host wait for it; every other call only enqueues.
 *  - Matrices are row-major f32. "W[K,N]" is the reference's matmul weight layout
 *    (instructions.js:219-224: B is [K,N], N contiguous).
 *  - A handle may be used from one host thread at a time. Different devices may be driven
 *    from different threads concurrently.
 *  - There is no CPU fallback: a shape a kernel does not support returns
 *    WGPT_ERR_UNSUPPORTED or WGPT_ERR_SHAPE.
 */
#ifndef WEBGPT_B200_H
#define WEBGPT_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define WGPT_ABI_VERSION 1

enum {
  WGPT_OK = 0,
  WGPT_ERR_SHAPE = -1,       /* a dimension violates a precondition (the reference throws) */
  WGPT_ERR_ALIGN = -2,       /* a device address is not 16-byte aligned */
  WGPT_ERR_OOM = -3,         /* device or host allocation failed */
  WGPT_ERR_CUDA = -4,        /* a CUDA call failed; the message carries the CUDA error */
  WGPT_ERR_TIMEOUT = -5,     /* a bounded device-side wait gave up */
  WGPT_ERR_STATE = -6,       /* call not valid in the handle's current state */
  WGPT_ERR_UNSUPPORTED = -7, /* valid in the reference, not implemented by these kernels */
  WGPT_ERR_ARG = -8          /* null pointer, bad enum value, id out of range */
};

/* Arithmetic used by matrix products with more than 8 rows (prefill, batched decode, wgpt_matmul_nk; wgpt_matmul and
 * wgpt_attention on reference-layout weights from 32 rows on, through a transposed copy of the weight in the
 * workspace). Products with up to 8 rows always run in FP32 on the CUDA cores. A new device starts in
 * WGPT_PRECISION_TF32X3. */
enum {
  WGPT_PRECISION_FP32 = 0,   /* FP32 FMA on the CUDA cores */
  WGPT_PRECISION_TF32X3 = 1, /* tensor cores, three TF32 products per FP32 product (error 1e-6..2e-5, growing with K) */
  WGPT_PRECISION_TF32 = 2    /* tensor cores, single TF32 product (error ~1e-3) */
};

typedef struct wgpt_device wgpt_device;
typedef struct wgpt_model wgpt_model;
typedef struct wgpt_session wgpt_session;

int32_t wgpt_abi_version(void);
const char *wgpt_last_error(void);

/* ---- device: GPT.initialize requestAdapter/requestDevice + initializeOperations
 *      (model.js:27-30, globals.js:13-15); destroyOperations (globals.js:25-27). */
int32_t wgpt_device_create(int32_t ordinal, wgpt_device **out);
int32_t wgpt_device_destroy(wgpt_device *dev);
int32_t wgpt_device_synchronize(wgpt_device *dev);
int32_t wgpt_device_set_precision(wgpt_device *dev, int32_t mode);
/* Number of kernels this library has launched on the device since creation. */
int32_t wgpt_device_launch_count(wgpt_device *dev, uint64_t *count);
/* Free and total device memory in bytes as the driver reports them (the reference reads its budget from
 * device.limits, instructions.js:75-80). Lets a caller check that a call allocated nothing. */
int32_t wgpt_device_mem_info(wgpt_device *dev, uint64_t *free_bytes, uint64_t *total_bytes);

/* ---- buffers: Block.initBuffer / GPT.initTensor (instructions.js:67-81, model.js:490-500),
 *      queue copies (model.js:253-255), mapAsync read-back (model.js:261-263). */
int32_t wgpt_buffer_create(wgpt_device *dev, uint64_t bytes, void **dptr);
int32_t wgpt_buffer_destroy(wgpt_device *dev, void *dptr);
int32_t wgpt_buffer_write(wgpt_device *dev, void *dst, uint64_t dst_offset, const void *src_host, uint64_t bytes);
int32_t wgpt_buffer_read(wgpt_device *dev, const void *src, uint64_t src_offset, void *dst_host, uint64_t bytes);
int32_t wgpt_buffer_copy(wgpt_device *dev, const void *src, uint64_t src_offset, void *dst, uint64_t dst_offset,
                         uint64_t bytes);
/* Page-locked host memory for inputs/outputs of the calls below (optional; any host memory works). */
int32_t wgpt_host_alloc(uint64_t bytes, void **ptr_host);
int32_t wgpt_host_free(void *ptr_host);

/* ---- timing on the device's stream (the reference times run() with performance.now(),
 *      model.js:72-79). elapsed waits for the second event. */
int32_t wgpt_event_create(wgpt_device *dev, void **event);
int32_t wgpt_event_record(wgpt_device *dev, void *event);
int32_t wgpt_event_elapsed_ms(wgpt_device *dev, void *start, void *stop, float *ms);
int32_t wgpt_event_destroy(wgpt_device *dev, void *event);

/* ---- pass-list replay: the reference encodes its whole pass list into one command buffer and submits it once
 *      (model.js:245-257). Between wgpt_graph_begin and wgpt_graph_end the per-operator calls below are recorded
 *      instead of executed; wgpt_graph_launch replays the recording (a CUDA graph) with one submission. Only the
 *      enqueue-only calls may be recorded (the per-operator entry points and wgpt_buffer_copy); buffers must stay
 *      alive and in place; run the same calls once before recording so that library workspaces have their size. */
typedef struct wgpt_graph wgpt_graph;
int32_t wgpt_graph_begin(wgpt_device *dev);
int32_t wgpt_graph_end(wgpt_device *dev, wgpt_graph **out);
int32_t wgpt_graph_launch(wgpt_device *dev, wgpt_graph *graph);
int32_t wgpt_graph_destroy(wgpt_device *dev, wgpt_graph *graph);

/* ---- per-operator entry points: one per instruction class of instructions.js ----
 * Parameter buffers (weights, bias, gamma, beta, scales) are treated as constants of the model: a kernel may read
 * them before the operation enqueued just ahead of it has finished. Fill them with wgpt_buffer_write /
 * wgpt_buffer_copy (copies are fully ordered), or call wgpt_device_synchronize between an operator that writes such
 * a buffer and the operator that uses it as a parameter. Inputs and outputs carry no such restriction. */

/* FastMatMulBlock.newInstance(rows, cols, shared, input, weights, bias) (instructions.js:157-177),
 * kernel fastMatMul (:179-319): out[rows,cols] = in[rows,shared] . W[shared,cols] + bias[cols].
 * bias may be NULL. Requires cols % 8 == 0 (:158) and shared % 4 == 0. */
int32_t wgpt_matmul(wgpt_device *dev, int32_t rows, int32_t cols, int32_t shared, const float *in, const float *W,
                    const float *bias, float *out);

/* FastMatMulBlock (instructions.js:157-319) with the weight stored transposed, Wt[cols, shared] (each output
 * column's weights contiguous) - the layout the model path keeps after its load-time re-layout
 * (model.js:362,456-468 re-lay-out at load too). Up to 8 rows stream the weights in FP32; more rows use the
 * device's precision mode (wgpt_device_set_precision): tensor cores for TF32 / 3xTF32. Same preconditions as
 * wgpt_matmul. */
int32_t wgpt_matmul_nk(wgpt_device *dev, int32_t rows, int32_t cols, int32_t shared, const float *in, const float *Wt,
                       const float *bias, float *out);

/* Waits for the device's stream and reports an error a kernel flagged on the device since the last check
 * (WGPT_ERR_TIMEOUT: a bounded device-side wait gave up; WGPT_ERR_ARG: a token id was out of range). The
 * model-level calls do this themselves; the per-operator calls only enqueue. */
int32_t wgpt_device_check(wgpt_device *dev);

/* Diagnostic, no counterpart in the reference: runs a one-thread kernel whose bounded mbarrier wait (the wait every
 * bulk-copy kernel of this library uses) cannot complete within `polls` polls because the barrier is armed for more
 * bytes than the first copy delivers. The kernel then takes the library's expiry path: it sets the device error
 * word, supplies the missing bytes, completes a second bounded wait and returns. *first_wait_completed is 0 when
 * the wait ran out (expected), *drain_wait_completed 1 when the drain succeeded. The next wgpt_device_check
 * reports WGPT_ERR_TIMEOUT once and clears it; the device stays usable. Nothing faults and nothing waits without
 * a limit. polls in 1..1024. */
int32_t wgpt_device_probe_wait_expiry(wgpt_device *dev, uint32_t polls, int32_t *first_wait_completed,
                                      int32_t *drain_wait_completed);

/* No counterpart in the reference. The same product as wgpt_matmul for 1..8 rows, for callers that must not
 * trigger a device allocation: an inference server that has handed all of HBM to its own arena and treats any
 * later cudaMalloc as a budget violation, a latency-critical decode loop (cudaMalloc can serialise against every
 * stream of the device), or a plugin host that forbids driver allocations once it is serving. wgpt_matmul may
 * grow a library-owned workspace for its split-K partial sums; this entry point keeps them in an array compiled
 * into the library (WGPT_STATIC_SCRATCH_FLOATS floats = 8 MiB per GPU that loads the library, held until
 * exit) and calls no allocating routine.
 *  - Limits: rows <= 8 and (K slices) * rows * cols <= WGPT_STATIC_SCRATCH_FLOATS, otherwise WGPT_ERR_SHAPE
 *    (rows * cols above the array size is always refused; the K split is the one wgpt_matmul uses, a few hundred
 *    slices at most for very long shared dimensions). All other preconditions are those of wgpt_matmul.
 *  - The first call on each device looks up the array's device address; make that first call outside any
 *    stream capture. The CUDA runtime loads a library's device code, this array included, when the library is
 *    first used on a GPU, and that load takes device memory: the "allocates nothing" guarantee holds from the
 *    second call on (make one warm-up call per GPU at start-up).
 *  - All calls on one GPU share the array (it keeps the previous call's partial sums; every call overwrites all
 *    it reads, nothing needs clearing). Calls on the same wgpt_device are stream-ordered and safe; calls that
 *    can overlap on one GPU (two wgpt_device handles on the same ordinal) race on it. */
#define WGPT_STATIC_SCRATCH_FLOATS 2097152
int32_t wgpt_matmul_static(wgpt_device *dev, int32_t rows, int32_t cols, int32_t shared, const float *in,
                           const float *W, const float *bias, float *out);

/* ResidualBlock.newInstance(rows, cols, outputBuf, residualBuf) (instructions.js:336-356; kernel :358-384).
 * cols % 4 == 0 (:337). out may alias a or b. */
int32_t wgpt_residual(wgpt_device *dev, int32_t rows, int32_t cols, const float *a, const float *b, float *out);

/* LayerNormBlock.newInstance(rows, cols, input, gamma, beta) (instructions.js:409-448; kernels :451-550).
 * eps = 1e-5 inside the square root. cols % 4 == 0 (:410). */
int32_t wgpt_layernorm(wgpt_device *dev, int32_t rows, int32_t cols, const float *in, const float *gamma,
                       const float *beta, float *out);

/* SoftmaxBlock.newInstance(rows, cols, input) (instructions.js:567-588; kernel :593-666), row softmax. */
int32_t wgpt_softmax(wgpt_device *dev, int32_t rows, int32_t cols, const float *in, float *out);

/* GeluBlock.newInstance(rows, cols, input) (instructions.js:683-703; kernel :705-748). cols % 4 == 0 (:684). */
int32_t wgpt_gelu(wgpt_device *dev, int32_t rows, int32_t cols, const float *in, float *out);

/* EmbedBlock.newInstance(idx, seq_length, n_embd, ...) (instructions.js:790-827):
 * out[t,:] = wte[idx[t],:] + wpe[t,:]. idx lives on the device (u32). Ids >= vocab_size give
 * WGPT_ERR_ARG after the kernel has run (the offending row is left zero). */
int32_t wgpt_embed(wgpt_device *dev, const uint32_t *idx, int32_t seq_length, int32_t n_embd, int32_t vocab_size,
                   const float *wte, const float *wpe, float *out);

/* DeEmbedBlock.newInstance(n_embd, vocab_size, ..., seq_length, ...) (instructions.js:844-888; kernel :890-952):
 * logits[v] = x[seq_length-1,:] . wte[v,:]. wte is the untransposed [vocab, n_embd] table: the
 * reference's transposed, padded chunks (model.js:346-364) exist only to fit WebGPU binding limits. */
int32_t wgpt_deembed(wgpt_device *dev, int32_t n_embd, int32_t vocab_size, int32_t seq_length, const float *x,
                     const float *wte, float *logits);

/* AttentionBlock.newFusedInstance(seq_length, n_embd, scale, n_head, head_size, input, qW, qB, kW, kB, vW, vB,
 * linearW, linearB) (instructions.js:985-1099; kernels :1101-1214): causal self-attention over one window,
 * out[seq_length, n_embd]. Weights are [n_embd, n_embd] in the W[K,N] layout. head_size must be one of
 * 4, 8, 16, 32, 64, 128 and n_head * head_size == n_embd. */
int32_t wgpt_attention(wgpt_device *dev, int32_t seq_length, int32_t n_embd, float scale, int32_t n_head,
                       int32_t head_size, const float *in, const float *qW, const float *qB, const float *kW,
                       const float *kB, const float *vW, const float *vB, const float *linW, const float *linB,
                       float *out);

/* int8 weight-only dequant-GEMM, the prototype of other/int8-gemm.js:117-229:
 * out[M,N] = A[M,K] . (f32(q[K,N]) * scale[N]); Bq holds q packed four per 32-bit word along N,
 * byte j of word w in row k = column 4w+j (:36-42), unpacked with sign extension (:126-131).
 * scale is per output column (the prototype's header asks for vector-wise scales, :4). N % 8 == 0, K % 4 == 0. */
int32_t wgpt_int8_matmul(wgpt_device *dev, int32_t M, int32_t K, int32_t N, const float *A, const uint32_t *Bq,
                         const float *scale, float *out);

/* The prototype's load step for a weight that is used many times (it uploads the packed matrix once and then
 * dispatches against it, other/int8-gemm.js:101-113): the handle owns a copy of Bq [K, N/4] and scale [N] (both
 * device memory) and, when K % 16 == 0, a re-laid-out copy with each output column's codes contiguous, which the
 * kernels stream with 128-bit loads. wgpt_int8_matmul_w computes what wgpt_int8_matmul computes, out[M,N] =
 * A[M,K] . (f32(q) * scale[n]): up to 4 rows in one weight-streaming kernel, more than 16 rows on the tensor cores
 * (device precision mode), otherwise through wgpt_int8_matmul. */
typedef struct wgpt_int8_weight wgpt_int8_weight;
int32_t wgpt_int8_weight_create(wgpt_device *dev, int32_t K, int32_t N, const uint32_t *Bq, const float *scale,
                                wgpt_int8_weight **out);
int32_t wgpt_int8_weight_destroy(wgpt_int8_weight *weight);
int32_t wgpt_int8_matmul_w(wgpt_device *dev, int32_t M, const wgpt_int8_weight *weight, const float *A, float *out);

/* quantizeMatrix (other/int8-gemm.js:25-46) on the device: W is the row-major f32 [K, N] weight; Bq_out receives
 * [K, N/4] words, byte j of word w in row k = round(W[k, 4w+j] / absmax * 127) & 0xff with the JavaScript
 * arithmetic (double precision, Math.round halves toward +infinity, :36-42); scale_out[n] = absmax / 127.
 * per_column != 0 takes absmax per output column (the vector-wise scales the prototype's header asks for, :4),
 * per_column == 0 over the whole matrix as the prototype does (:29-33). A zero column packs zeros with scale 0.
 * Feeds wgpt_int8_matmul directly. N % 4 == 0. All pointers are device memory. */
int32_t wgpt_int8_quantize(wgpt_device *dev, int32_t K, int32_t N, int32_t per_column, const float *W,
                           uint32_t *Bq_out, float *scale_out);

/* ---- model level: class GPT of model.js ---- */

/* params_gpt.json fields (model.js:289-322). bias is informational (model.js:322). */
typedef struct wgpt_params {
  int32_t n_layer, n_head, n_embd, n_ctx, vocab_size, bias;
} wgpt_params;

/* GPT.loadParameters checks (model.js:294-297): n_embd % 4, n_embd % n_head, head_size % 4. */
int32_t wgpt_model_create(wgpt_device *dev, const wgpt_params *params, wgpt_model **out);
/* GPT.loadEmbeddings/loadLayer/fetchAndInitTensor (model.js:339-500): name is the state-dict key of the
 * on-disk file "<name>_gpt.bin" (e.g. "transformer.h.0.attn.c_attn.weight"), data the raw f32 contents in
 * the on-disk layout ([in,out] for matmul weights), count its number of floats. The device copy is
 * re-laid-out for the kernels, as the reference re-lays-out at load (model.js:362,456-468). */
int32_t wgpt_model_set_tensor(wgpt_model *model, const char *name, const float *data_host, uint64_t count);
/* Verifies every tensor was supplied; after this the model is read-only. */
int32_t wgpt_model_finalize(wgpt_model *model);
/* GPT.unloadBuffers (model.js:502-505). */
int32_t wgpt_model_destroy(wgpt_model *model);

/* A session holds the KV cache and activations of n_seq independent sequences of equal length. */
int32_t wgpt_session_create(wgpt_model *model, int32_t n_seq, wgpt_session **out);
int32_t wgpt_session_destroy(wgpt_session *session);
int32_t wgpt_session_reset(wgpt_session *session);
int32_t wgpt_session_length(wgpt_session *session, int32_t *length);

/* Appends n_tok tokens to every sequence (ids_host is [n_seq, n_tok]) and, if logits_host is not NULL,
 * returns the vocab logits of each sequence's newest position ([n_seq, vocab_size]). */
int32_t wgpt_session_forward(wgpt_session *session, const uint32_t *ids_host, int32_t n_tok, float *logits_host);

/* GPT.run(idx) (model.js:104-268): forward pass over the whole window idx[0..n), returns the vocab logits
 * of the last position. The session (n_seq == 1) is reset first; it then holds the window's KV cache. */
int32_t wgpt_model_run(wgpt_session *session, const uint32_t *idx_host, int32_t n, float *logits_host);

/* GPT.generate with top_k = 1 (model.js:53-102, globals.js:47-74): feeds prompts_host [n_seq, n_prompt],
 * then produces n_new greedy tokens per sequence into new_ids_host [n_seq, n_new]; arg-max, lowest index on
 * ties. While a sequence fits in n_ctx every step reuses the KV cache; once the window would slide
 * (model.js:69) each step recomputes the slid window, as the reference does. */
int32_t wgpt_generate_greedy(wgpt_session *session, const uint32_t *prompts_host, int32_t n_prompt, int32_t n_new,
                             uint32_t *new_ids_host);

/* GPT.generate for independent sequences spread over several GPUs (each sequence has its own ids, cache and
 * logits; GPT.run has no cross-sequence state, model.js:104-268): sessions[i] is a session of n_seq_i sequences on
 * its own device (one wgpt_device + wgpt_model per GPU, weights replicated). prompts_host is
 * [sum of n_seq_i, n_prompt] in session order, new_ids_host [sum of n_seq_i, n_new] likewise. One host thread per
 * session runs wgpt_generate_greedy on its block; all are joined before the call returns. Nothing is exchanged
 * between devices. Two sessions must not share a wgpt_device handle. */
int32_t wgpt_generate_greedy_sharded(wgpt_session **sessions, int32_t n_sessions, const uint32_t *prompts_host,
                                     int32_t n_prompt, int32_t n_new, uint32_t *new_ids_host);

/* The three stages of wgpt_generate_greedy as separate calls, for callers that keep prompts resident or want to
 * overlap: set_prompts uploads [n_seq, n_prompt] ids; generate only enqueues the whole greedy loop (no copy and,
 * while n_prompt + n_new <= n_ctx, no host synchronisation) and may be repeated to regenerate from the same
 * prompts; get_new_ids waits and copies the [n_seq, n_new] result to the host. */
int32_t wgpt_session_set_prompts(wgpt_session *session, const uint32_t *prompts_host, int32_t n_prompt);
int32_t wgpt_session_generate(wgpt_session *session, int32_t n_new);
int32_t wgpt_session_get_new_ids(wgpt_session *session, int32_t n_new, uint32_t *new_ids_host);

/* GPT.generate with top_k > 1 (model.js:53-102): after each forward pass the reference reads the logits back
 * and runs selectTopK -> cpuSoftmax(temperature) -> sampleFromDistribution on the CPU (model.js:81-83,
 * globals.js:47-74). Here that chain runs on the device between decode steps, so nothing is read back per token.
 * The reference draws Math.random() inside sampleFromDistribution (globals.js:48); these calls take the uniform
 * numbers from the caller instead: uniforms_host is [n_new, n_seq] doubles in [0,1), number [i, q] deciding token
 * i of sequence q. Same arithmetic as the reference: stable descending order (lowest index first among equal
 * logits), exp((v - max) / temperature) in double precision, left-to-right sums, first index whose running sum
 * exceeds the uniform number, else the last. top_k is limited to WGPT_MAX_TOP_K (the reference's page allows
 * 1..100). wgpt_session_generate_sample is the enqueue-only stage, like wgpt_session_generate. */
#define WGPT_MAX_TOP_K 128
int32_t wgpt_generate_sample(wgpt_session *session, const uint32_t *prompts_host, int32_t n_prompt, int32_t n_new,
                             int32_t top_k, double temperature, const double *uniforms_host,
                             uint32_t *new_ids_host);
int32_t wgpt_session_generate_sample(wgpt_session *session, int32_t n_new, int32_t top_k, double temperature,
                                     const double *uniforms_host);

/* The sampling step alone, on device buffers: one pick per row of logits [n_rows, V] with uniforms [n_rows]
 * (doubles) into ids_out [n_rows] (globals.js:47-74 as above). */
int32_t wgpt_sample_topk(wgpt_device *dev, const float *logits, int32_t n_rows, int32_t V, int32_t top_k,
                         double temperature, const double *uniforms, uint32_t *ids_out);

/* GPT.externalBuffer tap (model.js:18,211-222): copies the residual stream before ln_f of the most recent
 * forward ([rows, n_embd], rows = n_seq * tokens of that call) into dst (device memory). */
int32_t wgpt_session_tap(wgpt_session *session, float *dst, uint64_t max_floats, uint64_t *floats_written);

/* Visuals.render (visuals.js:213-236) without a canvas: the fragment shader fsMain / hdrColorMapping
 * (visuals.js:104-135) applied to the buffer the model's externalBuffer tap fills ([n_ctx, n_embd] floats,
 * model.js:211-222), one pixel per element, into rgba_out (device memory, n_ctx * n_embd * 4 bytes, RGBA8). */
int32_t wgpt_visuals_render(wgpt_device *dev, const float *embeddings, int32_t n_ctx, int32_t n_embd,
                            uint8_t *rgba_out);

#ifdef __cplusplus
}
#endif
#endif
