/*
 * qmk_b200.h -- C ABI of the B200 (sm_100a) decode megakernel library, libqmk_b200.so.
 *
 * This is the drop-in boundary for the `--route mk` decode path of QiMeng-MegaKernel.
 * The reference binds one pybind11 function per model,
 *     mk(instructions, hidden_states, q_post_rope, k_cache, v_cache, attn_out,
 *        attn_lse_intermediates, attn_out_intermediates, silu_out, logits,
 *        attn_norm_weights, qkv_weights, rope_cos, rope_sin, o_proj_weights,
 *        mlp_norm_weights, up_proj_weights, gate_proj_weights, down_proj_weights,
 *        head_norm_weights, head_weights, barriers, pos_id, attn_scale, rms_norm_eps)
 * (qimeng_megakernel/models/LLM/llama/llama3_2__1b/A100/single_batch/decode_kernel/pybind.cpp:11-39,
 *  mk.h:8-31, host launcher mk.cu:97-198).  Here the same tensors are passed once as raw
 * device pointers (weights at create time, per-request state at bind time) and each decode
 * step is one call that launches one persistent kernel.  No torch / pybind types cross
 * this boundary; every entry point returns 0 or a negative qmk_error code.
 *
 * The library owns its scheduler: there is no `instructions` tensor and no `barriers`
 * tensor to zero between steps (the reference's STATIC_MEGAKERNEL contract,
 * qimeng_megakernel/models/LLM/decode.py:609-642, 688-689, 1383-1384).
 *
 * Threading: a handle is not thread-safe.  One handle per (device, request stream).
 */
#ifndef QMK_B200_H
#define QMK_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define QMK_ABI_VERSION 5

/* Error codes (negative).  qmk_strerror() gives the text. */
enum qmk_error {
  QMK_OK = 0,
  QMK_ERR_INVALID_ARG = -1,      /* null pointer, bad size, misaligned pointer            */
  QMK_ERR_UNSUPPORTED_MODEL = -2, /* descriptor does not match a compiled specialisation   */
  QMK_ERR_CUDA = -3,             /* a CUDA runtime call failed (see qmk_last_cuda_error)  */
  QMK_ERR_DEVICE = -4,           /* not an sm_100 device, or too few SMs / shared memory  */
  QMK_ERR_NOT_BOUND = -5,        /* decode called before qmk_bind_state                   */
  QMK_ERR_POSITION = -6,         /* pos_id outside the bound KV cache or RoPE table       */
  QMK_ERR_DEVICE_TIMEOUT = -7,   /* a bounded device-side wait expired (see qmk_status)   */
  QMK_ERR_OOM = -8,              /* scratch allocation failed                             */
  QMK_ERR_SCRATCH_TOO_LARGE = -9 /* qmk_decode_step_static: the model needs more than the fixed scratch array */
};

/* Architecture families (selects epilogue variants). */
enum qmk_arch {
  QMK_ARCH_LLAMA = 0,           /* RMSNorm -> QKV -> interleaved RoPE -> GQA -> SwiGLU    */
  QMK_ARCH_QWEN3 = 1,           /* the same with a per-head RMSNorm on Q and K before RoPE
                                   (qimeng_megakernel/models/LLM/qwen/qwen3__0_6b/A100/single_batch/
                                   decode_schedule/fused/operations.py:52-120)             */
  QMK_ARCH_MOE = 2              /* the Llama attention block with a mixture-of-experts MLP: router (fp32 softmax over
                                   all experts, top-k, no renormalisation) and per-expert SwiGLU, no shared expert
                                   (qimeng_megakernel/models/LLM/qwen/qwen1_5_moe_a2_7b/A100/single_batch/
                                   decode_schedule/fused/operations.py:175-240 with the shared branch absent);
                                   batched kernel only */
};

/*
 * Model descriptor.  Mirrors LlamaConfig / Qwen3Config of the reference
 * (.../A100/single_batch/decode_schedule/model_config.py:4-17).  Two kernels serve it:
 *   - the batch-1 kernel, compiled for the Llama-3.2-1B layer shape (hidden 2048, intermediate 8192,
 *     32 / 8 heads of 64), any num_layers and vocab_size;
 *   - the batched kernel, runtime shapes: hidden_size and intermediate_size multiples of 64
 *     (hidden_size <= 8192), head_dim 64 or 128, query heads per kv head 1, 2 or 4, batch 1..64.
 * qmk_create picks by descriptor, qmk_bind_state by batch (see qmk_set_kernel_variant).
 */
typedef struct qmk_model_desc {
  int32_t abi_version;       /* QMK_ABI_VERSION */
  int32_t arch;              /* enum qmk_arch */
  int32_t num_layers;
  int32_t hidden_size;
  int32_t intermediate_size;
  int32_t num_attention_heads;
  int32_t num_key_value_heads;
  int32_t head_dim;
  int32_t vocab_size;
  int32_t rope_rows;         /* rows of rope_cos / rope_sin (max positions)                */
  float rms_norm_eps;
  float attn_scale;          /* 1/sqrt(head_dim), as the reference passes it (mk_kernel.py:61) */
  float qk_norm_eps;         /* QMK_ARCH_QWEN3: eps of the per-head Q/K norm (0 = rms_norm_eps)     */
  int32_t num_experts;           /* QMK_ARCH_MOE: 8..128 experts (else 0)                            */
  int32_t num_experts_per_tok;   /* QMK_ARCH_MOE: 1..16                                              */
  int32_t moe_intermediate_size; /* QMK_ARCH_MOE: expert intermediate size, a multiple of 64         */
  int32_t ep_world;              /* QMK_ARCH_MOE: expert-parallel ranks (0 or 1 = off; 2, 4, 8; divides num_experts):
                                    this handle holds num_experts / ep_world experts, expert_gate_up / expert_down are
                                    [L, num_experts / ep_world, ...]; everything else is replicated             */
  int32_t ep_rank;               /* this handle's rank: it holds experts [ep_rank, ep_rank + 1) * num_experts / ep_world */
  int32_t tp_world;              /* QMK_ARCH_LLAMA / QMK_ARCH_QWEN3: tensor-parallel ranks (0 or 1 = off; 2, 4, 8).  The
                                    descriptor then describes this rank's SLICE: num_attention_heads, num_key_value_heads,
                                    intermediate_size and vocab_size are the whole model's divided by tp_world, the weight
                                    tensors are the matching slices (Q/K/V rows of its heads, O-proj columns of its heads,
                                    up/gate rows and down-proj columns of its intermediate units, LM-head rows of its
                                    vocabulary slice), hidden_size and the norms are whole.  The partial sums of the O-proj
                                    and down-proj phases are exchanged like the expert tiles (qmk_ep_export /
                                    qmk_ep_connect); the arg-max runs over all ranks' vocabulary slices.  logits is this
                                    rank's [B, vocab_size] slice                                                   */
  int32_t tp_rank;               /* this handle's rank; its LM-head rows are global rows tp_rank * vocab_size ...   */
  int32_t embed_rows;            /* rows of embed_tokens (0 = vocab_size): the whole vocabulary under tensor parallelism */
} qmk_model_desc;

/*
 * Weights: device pointers, bf16 row-major unless noted, layouts exactly as the reference's
 * Globals (decode_schedule/globs.py:13-24):
 *   attn_norm [L,H]  qkv [L,(NH+2*NKV)*HD,H] (Q and K rows interleaved per head,
 *   qimeng_megakernel/models/LLM/llama/preprocess.py:57-83)  o_proj [L,H,NH*HD]
 *   mlp_norm [L,H]  up/gate [L,I,H]  down [L,H,I]  lm_head_norm [H]  lm_head [V,H]
 *   rope_cos/rope_sin [rope_rows,HD] fp32, interleaved (preprocess.py:31-44)
 *   embed_tokens [V,H] (may alias lm_head; only read in token-input mode).
 * All matrix pointers must be 16-byte aligned.  The library never frees them.
 */
typedef struct qmk_weight_ptrs {
  const void* attn_norm;
  const void* qkv;
  const void* o_proj;
  const void* mlp_norm;
  const void* up_proj;
  const void* gate_proj;
  const void* down_proj;
  const void* lm_head_norm;
  const void* lm_head;
  const void* embed_tokens;
  const float* rope_cos;
  const float* rope_sin;
  const void* q_norm;        /* QMK_ARCH_QWEN3: [L, HD] bf16, interleaved order; else NULL */
  const void* k_norm;        /* QMK_ARCH_QWEN3: [L, HD] bf16, interleaved order; else NULL */
  /* QMK_ARCH_MOE (layouts of the reference's MoE Globals, globs.py:30-34; up_proj / gate_proj / down_proj unused): */
  const void* router;            /* [L, E, H] bf16                                     */
  const void* expert_gate_up;    /* [L, E, 2 * Ie, H] bf16, gate rows then up rows     */
  const void* expert_down;       /* [L, E, H, Ie] bf16                                 */
} qmk_weight_ptrs;

/*
 * Per-request state: device pointers borrowed until the next qmk_bind_state / qmk_destroy
 * (the reference re-allocates the KV cache between requests, decode.py:587-591, so binding
 * is separate from creation).  bf16 unless noted:
 *   hidden_states [B,H]  q_post_rope [B,NH*HD]  attn_out [B,NH*HD]  silu_out [B,I]  logits [B,V]
 *   (the leading B is absent / 1 for a single sequence, as in the reference's Globals)
 *   k_cache / v_cache [L, batch, kv_seq_len, NKV, HD] (K stored in the interleaved layout)
 *   next_token: optional int64[B]; receives argmax(logits) per row (lowest index on ties).
 *   token_in:   optional int64[B]; when non-null the step reads embed_tokens[token_in[b]]
 *               instead of hidden_states as the layer-0 input (may alias next_token for a
 *               device-resident greedy loop).
 *   out_tokens: optional int64[B, out_tokens_len]; when non-null the step also stores the argmax of
 *               row b at out_tokens[b, pos_b + 1] (the reference's output_tokens, decode.py:1391-1395).
 */
typedef struct qmk_state_ptrs {
  void* hidden_states;
  void* q_post_rope;
  void* k_cache;
  void* v_cache;
  void* attn_out;
  void* silu_out;
  void* logits;
  int64_t* next_token;
  const int64_t* token_in;
  int64_t* out_tokens;
  int64_t out_tokens_len;
  int32_t batch;             /* B: 1..64 sequences decoded per step */
  int32_t kv_seq_len;        /* S: allocated positions per sequence */
  const int32_t* position_ids;   /* optional int32[B]: position of each row (the reference's multi-batch
                                    position_ids); NULL = every row at the pos_id of the call */
  const uint8_t* active_mask;    /* optional uint8[B]: 0 = the row is finished: no KV write, zero attention
                                    output and projections, logits -1e9 (row_active in the reference's
                                    fused operations.py:226-317); NULL = all rows active */
  const int32_t* kv_slots;       /* optional int32[B]: the sequence of the KV cache that row b attends to and appends
                                    its K / V row to; NULL = row b owns sequence b.  With it the rows of one step may be
                                    consecutive positions of the same sequence -- a row attends to every earlier
                                    position, also to those written by other rows of the same step -- which is how a
                                    prompt is prefilled 64 tokens per launch (the reference's fused prefill is a
                                    PyTorch pass, llama/llama3_2__1b/A100/fused_prefill.py:185-335); batched kernel only */
  int32_t kv_batch;              /* sequences in k_cache / v_cache when kv_slots is given (0 = batch) */
} qmk_state_ptrs;

/* Device-side status record, filled when a bounded wait expires. */
typedef struct qmk_status {
  int32_t code;      /* 0 = healthy; 1 = dependency wait expired; 2 = weight-copy wait expired;
                        3 = activation-staging wait expired; 4 = (batched kernel) an active row's position was
                        outside the KV cache or the RoPE table: that row was treated as inactive, `seen` is the
                        position, `expected` the limit, `detail` the row; qmk_poll_status returns QMK_ERR_POSITION */
  int32_t sm;        /* CTA (one per SM) that reported */
  int32_t warp;
  int32_t phase;     /* global phase index: layer*5 + {0 qkv,1 attn,2 oproj,3 upgate,4 down}; 5*L = lm head */
  uint32_t seen;
  uint32_t expected;
  int32_t detail;
  int32_t reserved;
} qmk_status;

typedef struct qmk_handle qmk_handle;

/* Phase kinds inside one layer; phase index = layer * QMK_PHASES_PER_LAYER + kind, LM head last.
 * (QMK_ARCH_MOE has six phases per layer: QKV, attention, O-proj, router, expert up/gate, expert down.) */
#define QMK_PHASES_PER_LAYER 5
#define QMK_PHASE_QKV 0
#define QMK_PHASE_ATTN 1
#define QMK_PHASE_OPROJ 2
#define QMK_PHASE_UPGATE 3
#define QMK_PHASE_DOWN 4

/* Replaces get_mk()/module load (decode_schedule/mk_kernel.py:40-53): validates the descriptor
 * and the device, allocates library-owned scratch (dependency counters, split-KV partials,
 * status words) on `device`. */
int qmk_create(const qmk_model_desc* desc, const qmk_weight_ptrs* weights, int device, qmk_handle** out);

/* Replaces the per-call tensor marshalling of call_mk (mk_kernel.py:56-94). */
int qmk_bind_state(qmk_handle* h, const qmk_state_ptrs* state);

/* Replaces one mk(...) launch (mk.cu:97-198): one persistent kernel on `cuda_stream`
 * (a cudaStream_t; 0 = legacy default stream like the A100 reference, mk.cu:191).
 * Asynchronous; pos_id is the position of the token being fed (KV length becomes pos_id+1). */
int qmk_decode_step(qmk_handle* h, int32_t pos_id, void* cuda_stream);

/* Per-op isolation, the counterpart of the reference's run_instructions() with a filtered
 * instruction list (mk_kernel.py:97-111; verifier barrier pre-fill, verifier/common/barrier_fill.py:67-147):
 * runs phases [phase_begin, phase_end).  mode 0: one launch per phase, ordered by the stream,
 * no device-side dependency waits.  mode 1: one persistent launch with dependency counters. */
int qmk_run_phases(qmk_handle* h, int32_t pos_id, int32_t phase_begin, int32_t phase_end, int32_t mode,
                   void* cuda_stream);

/* Greedy decode with HOST token buffers (the end-to-end form of FusedGenerator.generate_greedy_fast,
 * decode.py:1340-1435): for i in [0,n_steps): copies host_tokens[first_pos+i] to the device, runs one
 * step at position first_pos+i, copies the argmax back into host_tokens[first_pos+i+1] before the
 * next step.  If teacher_forced != 0 the device never reads a generated token: inputs always come
 * from host_tokens as given and the argmax is written to host_argmax[i] instead.
 * Synchronous on `cuda_stream`. */
int qmk_generate_host(qmk_handle* h, int64_t* host_tokens, int64_t host_tokens_len, int32_t first_pos,
                      int32_t n_steps, int32_t teacher_forced, int64_t* host_argmax, void* cuda_stream);

/* Device-resident run of n_steps greedy steps from position first_pos (the second half of generate_greedy_fast,
 * decode.py:1340-1435, with the token loop on the device): step 0 reads state.token_in, every later step the arg-max of
 * the step before; each step writes next_token and, when bound, out_tokens[pos + 1].  Needs token_in and embed_tokens.
 * Batch-1 kernel: ONE persistent launch runs all n_steps -- the token crosses from the last phase of a step to the first
 * phase of the next as a tagged word, and every warp's weight stream runs on across the step boundary.  Batched kernel:
 * the same run as n_steps launches (token_in must alias next_token; per-row position_ids are not advanced, so they must
 * be null).  1 <= n_steps <= 4096; positions first_pos .. first_pos + n_steps - 1 must lie inside the KV cache and the
 * RoPE tables.  Asynchronous on `cuda_stream`. */
int qmk_generate_device(qmk_handle* h, int32_t first_pos, int32_t n_steps, void* cuda_stream);

/* Reads the device status record (synchronises the stream it was last launched on). */
int qmk_poll_status(qmk_handle* h, qmk_status* out);

/* Device-side wait budget in SM clock cycles (default 2e9, about one second). */
int qmk_set_timeout_cycles(qmk_handle* h, int64_t cycles);

/* Launch mode.  on (default): cooperative launch, the driver guarantees that all CTAs are co-resident
 * (they wait on one another) or fails the launch.  off: plain launch, for a GPU the caller knows to be
 * otherwise idle; the bounded waits still turn a missing CTA into QMK_ERR_DEVICE_TIMEOUT. */
int qmk_set_cooperative_launch(qmk_handle* h, int32_t on);

/* Debug knob used by the failure-detection test: when set, qmk_run_phases(mode 1) also waits for the
 * dependency of its first phase, which nothing publishes, so the bounded wait must expire. */
int qmk_set_wait_first_dependency(qmk_handle* h, int32_t on);

/* Which kernel serves the handle.  0 (default): the batch-1 kernel when the descriptor has its compiled
 * shape and one sequence is bound, else the batched kernel.  1: always the batched kernel (any batch,
 * also 1).  The batched kernel implements qmk_decode_step, qmk_run_phases, qmk_generate_host (batch 1),
 * qmk_poll_status, the wait-first knob and qmk_set_trace (slots 0 dependency satisfied, 1 first accumulator of the
 * phase complete, 2 epilogue warps enter, 5 the CTA arrives at the phase's counter). */
int qmk_set_kernel_variant(qmk_handle* h, int32_t variant);

/* Optional device timeline (the counterpart of the reference's ENABLE_PROFILING clock64 buffer,
 * qimeng_megakernel/models/LLM/llama/llama3_2__1b/A100/multi_batch/decode_kernel/profiling.cuh:7-35, selected
 * at run time instead of compile time).  device_buffer: uint64 [CTAs, phases, W], W = 8 words for the batch-1 kernel
 * (globaltimer nanoseconds: 0 dependency satisfied, 1 activations staged, 2 first worker enters, 5 first worker
 * leaves, 6 last worker leaves) and 16 for the batched kernel (stamps and cycle sums, listed in
 * csrc/qmk_batch_kernel.cuh).  NULL switches tracing off. */
int qmk_set_trace(qmk_handle* h, void* device_buffer, int64_t bytes);

/* Algorithmic HBM bytes of one decode step at KV length pos_id+1 (weights + KV read + KV write). */
int64_t qmk_step_bytes(const qmk_handle* h, int32_t pos_id);

/* QMK_ARCH_MOE: number of distinct experts the last layer's router selected in the last step (synchronises the
 * stream of the last launch); the bytes of a MoE step depend on it.  0 for other architectures. */
int qmk_last_expert_count(qmk_handle* h, int32_t* out);

/* QMK_ARCH_MOE: what the last router phase selected (the reference keeps it in Globals.expert_indices /
 * expert_weights, qwen1_5_moe_a2_7b/.../decode_schedule/globs.py:41-42, for one row): `count` distinct experts of the
 * step, their indices ascending in experts[0..count), and weights[slot * 64 + row] = router probability of row `row`
 * for experts[slot], 0 where the row did not select it.  experts: int32[num_experts], weights: float[num_experts * 64]
 * (host memory).  Synchronises the stream of the last launch. */
int qmk_last_expert_routing(qmk_handle* h, int32_t* count, int32_t* experts, float* weights);

/* Expert parallelism over the GPUs of one box (no counterpart in the reference, which has no distributed code; the
 * math that is split is its routed accumulate, qwen1_5_moe_a2_7b/.../fused/operations.py:220-268).  One process per GPU,
 * one handle each, created with ep_world / ep_rank in the descriptor.  qmk_ep_export allocates this rank's exchange
 * buffer and writes its 64-byte inter-process memory handle; the caller gathers the handles of all ranks (over
 * torch.distributed or any other channel) and passes them, in rank order, to qmk_ep_connect, which maps the peers'
 * buffers.  From then on every decode step of every rank must be launched in the same order on all ranks: inside the
 * expert down-projection each rank stores its partial tiles into the peers' buffers and adds up what it receives, in rank
 * order.  A peer that never shows up ends the bounded wait with QMK_ERR_DEVICE_TIMEOUT. */
int qmk_ep_export(qmk_handle* h, void* ipc_handle_out);
int qmk_ep_connect(qmk_handle* h, const void* ipc_handles);

/* QMK_ARCH_MOE: distinct experts read, summed over every router phase (layer and step) since the counter was last
 * reset: each one stands for 3 * hidden_size * moe_intermediate_size bf16 weights streamed from HBM, which is what a
 * benchmark needs to turn a timed run into achieved bytes.  Synchronises the stream of the last launch. */
int qmk_expert_reads(qmk_handle* h, int64_t* total, int32_t reset);

/* Number of kernels the library has launched through this handle. */
int64_t qmk_launch_count(const qmk_handle* h);

/* Launch geometry actually used: CTAs (= SMs), threads per CTA, dynamic shared memory bytes. */
int qmk_launch_geometry(const qmk_handle* h, int32_t* ctas, int32_t* threads, int32_t* smem_bytes);

/* No counterpart in the reference.  One decode step for callers that must not allocate device memory
 * (a serving loop whose memory belongs to a framework's pool allocator, an embedder with a fixed memory
 * budget, code running where an allocation would synchronise the device): same kernel as qmk_decode_step,
 * but the library's scratch (hand-off words, split-KV records, status) lives in a file-scope __device__
 * array of QMK_STATIC_SCRATCH_MAX_BYTES inside the library image instead of a cudaMalloc'ed block, and
 * there is no handle: descriptor, weights and state are passed on every call.  Calls no cudaMalloc /
 * cudaFree / allocating routine.  Every GPU that loads the library holds the array until exit.  All calls
 * on a device share it: run them on one stream, one after the other (overlapping calls race); what must
 * start at zero is cleared by each call.  The first call on a device does the set-up (symbol address,
 * kernel attribute): make it outside any stream capture.  A model whose scratch would not fit returns
 * QMK_ERR_SCRATCH_TOO_LARGE; a state with position_ids or active_mask (which the batch-1 kernel does not
 * have) returns QMK_ERR_INVALID_ARG.  Asynchronous on `cuda_stream`; not thread-safe. */
#define QMK_STATIC_SCRATCH_MAX_BYTES (2u << 20)
int qmk_decode_step_static(const qmk_model_desc* desc, const qmk_weight_ptrs* weights, const qmk_state_ptrs* state,
                           int32_t pos_id, int device, void* cuda_stream);

/* Companions of qmk_decode_step_static (no counterparts in the reference either; none of them allocates).
 * qmk_static_poll_status: synchronises the stream of the last static launch on `device` and copies the
 * status record out of the fixed array.  The record of an expired wait is sticky: later static calls do
 * not clear it, so the failure is still there when the caller gets round to polling.  When it is non-zero
 * the whole array is cleared and QMK_ERR_DEVICE_TIMEOUT is returned; results of the failed launch and of
 * launches queued behind it must be discarded.
 * qmk_static_set_timeout_cycles: the wait budget of static launches on `device` (0 = default 2e9 cycles).
 * qmk_static_set_wait_first_dependency: the failure-detection knob of qmk_set_wait_first_dependency for
 * the static path (the first phase waits for words nothing writes).
 * qmk_static_last_cuda_error: text behind the last QMK_ERR_CUDA of a static entry point. */
int qmk_static_poll_status(int device, qmk_status* out);
int qmk_static_set_timeout_cycles(int device, int64_t cycles);
int qmk_static_set_wait_first_dependency(int device, int32_t on);
const char* qmk_static_last_cuda_error(void);

void qmk_destroy(qmk_handle* h);
const char* qmk_strerror(int code);
const char* qmk_last_cuda_error(const qmk_handle* h);
int qmk_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* QMK_B200_H */
