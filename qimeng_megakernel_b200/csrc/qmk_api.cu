// Host side of libqmk_b200.so: the C ABI declared in include/qmk_b200.h.
// Plain CUDA runtime, no torch / pybind types.  The reference's host launcher is
// qimeng_megakernel/models/LLM/llama/llama3_2__1b/A100/single_batch/decode_kernel/mk.cu:97-198
// (fills a globals POD from tensors, sets the dynamic shared-memory limit, launches, prints errors);
// here errors are returned, the stream is explicit and scratch is owned by the handle.
#include <cuda_runtime.h>
#include <math.h>
#include <stdio.h>
#include <string.h>

#include <new>

#include "../../include/qmk_b200.h"
#include "qmk_batch_host.h"
#include "qmk_megakernel.cuh"

using namespace qmk;
using Shape = ShapeLlama1B;

struct qmk_handle {
  qmk_model_desc desc;
  qmk_weight_ptrs w;
  qmk_state_ptrs st;
  bool bound;
  int device;
  int n_sm;
  unsigned launch_seq;
  int cooperative;
  long long timeout_cycles;
  int wait_first;
  long long launches;
  cudaStream_t last_stream;
  char cuda_err[256];
  // scratch (one allocation)
  unsigned char* scratch;
  size_t scratch_bytes;
  unsigned long long* part_rec;
  uint32_t* t_hid_o;
  uint32_t* t_hid_d;
  uint32_t* t_q;
  uint32_t* t_attn;
  uint32_t* t_silu;
  unsigned* tickets;
  unsigned long long* argmax_key;
  unsigned* status;
  long long* d_tok;   // [2]: token fed, token produced (host-buffer generate path)
  unsigned long long* trace;
  // which kernels can serve this handle
  bool tuned_shape;        // the descriptor has the compiled shape of the batch-1 kernel
  int variant;             // 0: batch-1 kernel when possible; 1: always the batched kernel
  qmk_batch_ctx* bctx;     // batched kernel: tensor maps + scratch (created on first need)
  int last_kernel;         // 0 batch-1 kernel, 1 batched kernel: whose status record the next poll reads
};

// The batch-1 kernel has neither per-row positions nor an active mask: a state that carries either goes to the
// batched kernel, so that the same state behaves the same under both kernel variants.
static bool use_batched(const qmk_handle* h) {
  return !h->tuned_shape || h->variant == 1 ||
         (h->bound && (h->st.batch != 1 || h->st.position_ids != nullptr || h->st.active_mask != nullptr ||
                       h->st.kv_slots != nullptr));
}

static int ensure_bctx(qmk_handle* h) {
  if (h->bctx) return QMK_OK;
  return qmkb_create(&h->desc, &h->w, h->n_sm, &h->bctx, h->cuda_err, sizeof(h->cuda_err));
}

static int cuda_fail(qmk_handle* h, cudaError_t e, const char* what) {
  if (h) snprintf(h->cuda_err, sizeof(h->cuda_err), "%s: %s", what, cudaGetErrorString(e));
  return QMK_ERR_CUDA;
}
#define QMK_CUDA(h, call)                                   \
  do {                                                      \
    cudaError_t e__ = (call);                               \
    if (e__ != cudaSuccess) return cuda_fail(h, e__, #call); \
  } while (0)

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

extern "C" int qmk_abi_version(void) { return QMK_ABI_VERSION; }

extern "C" const char* qmk_strerror(int code) {
  switch (code) {
    case QMK_OK: return "ok";
    case QMK_ERR_INVALID_ARG: return "invalid argument (null or misaligned pointer, bad size)";
    case QMK_ERR_UNSUPPORTED_MODEL: return "model descriptor matches no compiled specialisation";
    case QMK_ERR_CUDA: return "CUDA runtime call failed";
    case QMK_ERR_DEVICE: return "device is not sm_100 or lacks SMs / shared memory";
    case QMK_ERR_NOT_BOUND: return "no request state bound (call qmk_bind_state)";
    case QMK_ERR_POSITION: return "position outside the bound KV cache or RoPE table";
    case QMK_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait expired";
    case QMK_ERR_OOM: return "scratch allocation failed";
    case QMK_ERR_SCRATCH_TOO_LARGE: return "model needs more scratch than the fixed array of qmk_decode_step_static";
    default: return "unknown error";
  }
}

extern "C" const char* qmk_last_cuda_error(const qmk_handle* h) { return h ? h->cuda_err : ""; }

static int reset_scratch(qmk_handle* h, cudaStream_t s) {
  // everything but the status record, which sits last and is cleared only after it has been read
  QMK_CUDA(h, cudaMemsetAsync(h->scratch, 0, (size_t)((unsigned char*)h->status - h->scratch), s));
  return QMK_OK;
}

extern "C" int qmk_create(const qmk_model_desc* d, const qmk_weight_ptrs* w, int device, qmk_handle** out) {
  if (!d || !w || !out) return QMK_ERR_INVALID_ARG;
  *out = nullptr;
  if (d->abi_version != QMK_ABI_VERSION) return QMK_ERR_INVALID_ARG;
  const bool tuned = d->arch == QMK_ARCH_LLAMA && d->hidden_size == Shape::H && d->intermediate_size == Shape::I &&
                     d->num_attention_heads == Shape::NH && d->num_key_value_heads == Shape::NKV &&
                     d->head_dim == Shape::HD;
  if (!tuned && qmkb_supported(d) != QMK_OK) return QMK_ERR_UNSUPPORTED_MODEL;
  if (d->num_layers < 0 || d->num_layers > 1024 || d->vocab_size < 1 || d->rope_rows < 1) return QMK_ERR_INVALID_ARG;
  if (!(d->rms_norm_eps > 0.f) || !(d->attn_scale > 0.f)) return QMK_ERR_INVALID_ARG;
  const bool moe = d->arch == QMK_ARCH_MOE;
  const void* ptrs[] = {w->attn_norm, w->qkv, w->o_proj, w->mlp_norm, moe ? w->router : w->up_proj,
                        moe ? w->expert_gate_up : w->gate_proj, moe ? w->expert_down : w->down_proj,
                        w->lm_head_norm, w->lm_head, w->rope_cos, w->rope_sin};
  for (const void* p : ptrs)
    if (!p || !aligned16(p)) return QMK_ERR_INVALID_ARG;
  if (w->embed_tokens && !aligned16(w->embed_tokens)) return QMK_ERR_INVALID_ARG;
  if (d->arch == QMK_ARCH_QWEN3 && (!w->q_norm || !w->k_norm)) return QMK_ERR_INVALID_ARG;

  qmk_handle* h = new (std::nothrow) qmk_handle();
  if (!h) return QMK_ERR_OOM;
  memset(h, 0, sizeof(*h));
  h->desc = *d;
  h->w = *w;
  h->device = device;
  h->timeout_cycles = 2000000000ll;
  h->cooperative = 1;
  h->tuned_shape = tuned;
  int rc = QMK_OK;
  do {
    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) { rc = cuda_fail(h, e, "cudaSetDevice"); break; }
    cudaDeviceProp prop;
    e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess) { rc = cuda_fail(h, e, "cudaGetDeviceProperties"); break; }
    int bsmem = 0;
    qmkb_geometry(nullptr, nullptr, nullptr, &bsmem);
    if (prop.major != 10 || (int)prop.sharedMemPerBlockOptin < SmemLayout<Shape>::kTotal ||
        (int)prop.sharedMemPerBlockOptin < bsmem ||
        prop.multiProcessorCount < 1 || !prop.cooperativeLaunch) {
      rc = QMK_ERR_DEVICE;
      break;
    }
    h->n_sm = prop.multiProcessorCount;
    {
      // the device splits work with 32-bit arithmetic: (worker + 1) * units must fit
      const unsigned long long nwt = (unsigned long long)h->n_sm * kWorkers;
      const unsigned long long units = d->vocab_size > Shape::I ? d->vocab_size : Shape::I;
      if ((nwt + 1) * units >= (1ull << 32)) { rc = QMK_ERR_INVALID_ARG; break; }
    }
    e = cudaFuncSetAttribute(qmk_decode_kernel<Shape>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             SmemLayout<Shape>::kTotal);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(qmk_decode_kernel<ShapeLlama1BSteps>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             SmemLayout<Shape>::kTotal);
    if (e != cudaSuccess) { rc = cuda_fail(h, e, "cudaFuncSetAttribute"); break; }
    const size_t b_part = align_up((size_t)Shape::NH * kMaxSplits * (Shape::HD + 2) * 8, 256);
    const size_t b_hid = align_up((size_t)Shape::H * 4, 256);
    const size_t b_q = align_up((size_t)(Shape::QDIM + 2 * Shape::NKV * Shape::HD) * 4, 256);
    const size_t b_attn = align_up((size_t)Shape::QDIM * 4, 256);
    const size_t b_silu = align_up((size_t)Shape::I * 4, 256);
    const size_t b_tickets = 512, b_argmax = 256, b_status = 256, b_tok = 256;
    h->scratch_bytes = b_part + 2 * b_hid + b_q + b_attn + b_silu + b_tickets + b_argmax + b_tok + b_status;
    e = cudaMalloc((void**)&h->scratch, h->scratch_bytes);
    if (e != cudaSuccess) { rc = QMK_ERR_OOM; cuda_fail(h, e, "cudaMalloc"); break; }
    unsigned char* q = h->scratch;
    h->part_rec = (unsigned long long*)q; q += b_part;
    h->t_hid_o = (uint32_t*)q; q += b_hid;
    h->t_hid_d = (uint32_t*)q; q += b_hid;
    h->t_q = (uint32_t*)q; q += b_q;
    h->t_attn = (uint32_t*)q; q += b_attn;
    h->t_silu = (uint32_t*)q; q += b_silu;
    h->tickets = (unsigned*)q; q += b_tickets;
    h->argmax_key = (unsigned long long*)q; q += b_argmax;
    h->d_tok = (long long*)q; q += b_tok;
    h->status = (unsigned*)q;
    e = cudaMemset(h->scratch, 0, h->scratch_bytes);
    if (e != cudaSuccess) { rc = cuda_fail(h, e, "cudaMemset"); break; }
    if (!tuned) rc = ensure_bctx(h);
  } while (0);
  if (rc != QMK_OK) {
    if (h->scratch) cudaFree(h->scratch);
    qmkb_destroy(h->bctx);
    delete h;
    return rc;
  }
  *out = h;
  return QMK_OK;
}

extern "C" void qmk_destroy(qmk_handle* h) {
  if (!h) return;
  cudaSetDevice(h->device);
  if (h->scratch) cudaFree(h->scratch);
  qmkb_destroy(h->bctx);
  delete h;
}

extern "C" int qmk_bind_state(qmk_handle* h, const qmk_state_ptrs* s) {
  if (!h || !s) return QMK_ERR_INVALID_ARG;
  if (s->batch < 1 || s->batch > 64 || s->kv_seq_len < 1) return QMK_ERR_INVALID_ARG;
  void* ptrs[] = {s->hidden_states, s->q_post_rope, s->k_cache, s->v_cache, s->attn_out, s->silu_out, s->logits};
  for (void* p : ptrs)
    if (!p || !aligned16(p)) return QMK_ERR_INVALID_ARG;
  if (s->token_in && !h->w.embed_tokens) return QMK_ERR_INVALID_ARG;
  if (s->out_tokens && s->out_tokens_len < 1) return QMK_ERR_INVALID_ARG;
  if (s->kv_batch < 0 || (s->kv_slots == nullptr && s->kv_batch != 0 && s->kv_batch != s->batch)) return QMK_ERR_INVALID_ARG;
  h->st = *s;
  h->bound = true;
  if (use_batched(h)) {
    QMK_CUDA(h, cudaSetDevice(h->device));
    return ensure_bctx(h);
  }
  return QMK_OK;
}

static int batched_launch(qmk_handle* h, int pos, int phase_begin, int phase_end, int wait_first, cudaStream_t stream) {
  int rc = ensure_bctx(h);
  if (rc) return rc;
  qmkb_launch_args a;
  a.pos = pos;
  a.phase_begin = phase_begin;
  a.phase_end = phase_end;
  a.wait_first = wait_first;
  a.cooperative = h->cooperative;
  a.timeout_cycles = h->timeout_cycles;
  a.trace = h->trace;
  rc = qmkb_launch(h->bctx, &h->st, &a, stream, h->cuda_err, sizeof(h->cuda_err));
  if (rc) return rc;
  h->launches++;
  h->last_stream = stream;
  h->last_kernel = 1;
  return QMK_OK;
}

static void fill_params(const qmk_handle* h, Params& p, int pos) {
  memset(&p, 0, sizeof(p));
  const qmk_weight_ptrs& w = h->w;
  const qmk_state_ptrs& s = h->st;
  p.attn_norm = (const uint16_t*)w.attn_norm;
  p.qkv = (const uint16_t*)w.qkv;
  p.o_proj = (const uint16_t*)w.o_proj;
  p.mlp_norm = (const uint16_t*)w.mlp_norm;
  p.up = (const uint16_t*)w.up_proj;
  p.gate = (const uint16_t*)w.gate_proj;
  p.down = (const uint16_t*)w.down_proj;
  p.lm_norm = (const uint16_t*)w.lm_head_norm;
  p.lm_head = (const uint16_t*)w.lm_head;
  p.embed = (const uint16_t*)w.embed_tokens;
  p.rope_cos = w.rope_cos;
  p.rope_sin = w.rope_sin;
  p.hidden = (uint16_t*)s.hidden_states;
  p.q_post_rope = (uint16_t*)s.q_post_rope;
  p.k_cache = (uint16_t*)s.k_cache;
  p.v_cache = (uint16_t*)s.v_cache;
  p.attn_out = (uint16_t*)s.attn_out;
  p.silu_out = (uint16_t*)s.silu_out;
  p.logits = (uint16_t*)s.logits;
  p.next_token = (long long*)s.next_token;
  p.token_in = (const long long*)s.token_in;
  p.out_tokens = (long long*)s.out_tokens;
  p.out_tokens_len = s.out_tokens_len;
  p.kv_seq_stride = (long long)Shape::NKV * Shape::HD;
  p.kv_layer_stride = (long long)(s.kv_batch > 0 ? s.kv_batch : s.batch) * s.kv_seq_len * p.kv_seq_stride;
  p.part_rec = h->part_rec;
  p.t_hid_o = h->t_hid_o;
  p.t_hid_d = h->t_hid_d;
  p.t_q = h->t_q;
  p.t_attn = h->t_attn;
  p.t_silu = h->t_silu;
  p.tickets = h->tickets;
  p.argmax_key = h->argmax_key;
  p.status = h->status;
  p.trace = h->trace;
  p.num_layers = h->desc.num_layers;
  p.vocab = h->desc.vocab_size;
  p.pos = pos;
  p.eps = h->desc.rms_norm_eps;
  p.scale_log2e = h->desc.attn_scale * 1.4426950408889634f;
  p.timeout_cycles = h->timeout_cycles;
  p.wait_first = 0;
  p.n_steps = 1;
  p.tok_word = (unsigned long long*)(h->d_tok + 8);   // (d_tok[0..1] are qmk_generate_host's token buffers)
}

static int launch(qmk_handle* h, Params& p, cudaStream_t stream) {
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((unsigned)h->n_sm);
  cfg.blockDim = dim3(kLaunchThreads);
  cfg.dynamicSmemBytes = SmemLayout<Shape>::kTotal;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;   // all CTAs co-resident: they wait on one another
  attr[0].val.cooperative = h->cooperative;
  p.stream_end = p.phase_end + (p.n_steps > 1 ? (p.n_steps - 1) * num_phases(p.num_layers) : 0);
  p.launch_seq = h->launch_seq + 1;   // number of the launch's first step; every step takes one
  h->launch_seq += (unsigned)(p.n_steps > 0 ? p.n_steps : 1);
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (p.n_steps > 1) QMK_CUDA(h, cudaLaunchKernelEx(&cfg, qmk_decode_kernel<ShapeLlama1BSteps>, p));   // the multi-step instance
  else QMK_CUDA(h, cudaLaunchKernelEx(&cfg, qmk_decode_kernel<Shape>, p));
  h->launches++;
  h->last_stream = stream;
  h->last_kernel = 0;
  return QMK_OK;
}

static int check_step_args(const qmk_handle* h, int pos) {
  if (!h) return QMK_ERR_INVALID_ARG;
  if (!h->bound) return QMK_ERR_NOT_BOUND;
  if (pos < 0 || pos >= h->st.kv_seq_len || pos >= h->desc.rope_rows) return QMK_ERR_POSITION;
  return QMK_OK;
}

static int step_with(qmk_handle* h, Params& p, cudaStream_t stream) {
  if (h->launch_seq >= (1u << 23)) {   // record tags are launch_seq * 256 + phase: restart from a zeroed scratch
    int rc = reset_scratch(h, stream);
    if (rc) return rc;
    h->launch_seq = 0;
  }
  p.phase_begin = 0;
  p.phase_end = num_phases(p.num_layers);
  p.sync = 1;
  return launch(h, p, stream);
}

extern "C" int qmk_decode_step(qmk_handle* h, int32_t pos_id, void* cuda_stream) {
  int rc = check_step_args(h, pos_id);
  if (rc) return rc;
  QMK_CUDA(h, cudaSetDevice(h->device));
  if (use_batched(h)) return batched_launch(h, pos_id, 0, qmkb_num_phases(&h->desc), 0, (cudaStream_t)cuda_stream);
  Params p;
  fill_params(h, p, pos_id);
  return step_with(h, p, (cudaStream_t)cuda_stream);
}

extern "C" int qmk_generate_device(qmk_handle* h, int32_t first_pos, int32_t n_steps, void* cuda_stream) {
  if (!h || n_steps < 1 || n_steps > 4096 || first_pos < 0) return QMK_ERR_INVALID_ARG;
  int rc = check_step_args(h, first_pos + n_steps - 1);
  if (rc) return rc;
  // the steps feed themselves: the first one reads token_in, the others the arg-max of the step before
  if (!h->st.token_in || !h->w.embed_tokens) return QMK_ERR_INVALID_ARG;
  QMK_CUDA(h, cudaSetDevice(h->device));
  cudaStream_t stream = (cudaStream_t)cuda_stream;
  if (use_batched(h)) {
    // the batched kernel runs one step per launch: the same run as n launches (token_in must alias next_token, as in
    // the device-resident loop of the host mirror)
    if (n_steps > 1 && ((const void*)h->st.token_in != (const void*)h->st.next_token || h->st.position_ids != nullptr))
      return QMK_ERR_INVALID_ARG;   // (per-row positions are advanced by the caller between steps)
    for (int i = 0; i < n_steps; ++i) {
      rc = batched_launch(h, first_pos + i, 0, qmkb_num_phases(&h->desc), 0, stream);
      if (rc) return rc;
    }
    return QMK_OK;
  }
  Params p;
  fill_params(h, p, first_pos);
  p.n_steps = n_steps;
  return step_with(h, p, stream);
}

extern "C" int qmk_run_phases(qmk_handle* h, int32_t pos_id, int32_t phase_begin, int32_t phase_end, int32_t mode,
                              void* cuda_stream) {
  int rc = check_step_args(h, pos_id);
  if (rc) return rc;
  const int nph = use_batched(h) ? qmkb_num_phases(&h->desc) : num_phases(h->desc.num_layers);
  if (phase_begin < 0 || phase_end > nph || phase_begin > phase_end || (mode != 0 && mode != 1))
    return QMK_ERR_INVALID_ARG;
  QMK_CUDA(h, cudaSetDevice(h->device));
  cudaStream_t stream = (cudaStream_t)cuda_stream;
  if (use_batched(h)) {
    if (mode == 0) {
      for (int ph = phase_begin; ph < phase_end; ++ph) {
        rc = batched_launch(h, pos_id, ph, ph + 1, 0, stream);
        if (rc) return rc;
      }
      return QMK_OK;
    }
    if (phase_begin == phase_end) return QMK_OK;
    return batched_launch(h, pos_id, phase_begin, phase_end, h->wait_first, stream);
  }
  Params p;
  fill_params(h, p, pos_id);
  if (mode == 0) {
    for (int ph = phase_begin; ph < phase_end; ++ph) {
      p.phase_begin = ph;
      p.phase_end = ph + 1;
      p.sync = 0;
      rc = launch(h, p, stream);
      if (rc) return rc;
    }
    return QMK_OK;
  }
  if (phase_begin == phase_end) return QMK_OK;
  // Tags are unique per launch, so a sub-range needs no clean-up.  The failure-detection knob waits
  // for words nothing writes: zero the scratch first so that no stale tag can match by accident.
  if (h->wait_first) {
    rc = reset_scratch(h, stream);
    if (rc) return rc;
  }
  p.phase_begin = phase_begin;
  p.phase_end = phase_end;
  p.sync = 1;
  p.wait_first = h->wait_first;
  return launch(h, p, stream);
}

extern "C" int qmk_generate_host(qmk_handle* h, int64_t* host_tokens, int64_t host_tokens_len, int32_t first_pos,
                                 int32_t n_steps, int32_t teacher_forced, int64_t* host_argmax,
                                 void* cuda_stream) {
  if (!h || !host_tokens || n_steps < 0 || first_pos < 0) return QMK_ERR_INVALID_ARG;
  if (!h->w.embed_tokens) return QMK_ERR_INVALID_ARG;
  if (teacher_forced && !host_argmax) return QMK_ERR_INVALID_ARG;
  const long long need = (long long)first_pos + n_steps + (teacher_forced ? 0 : 1);
  if (need > host_tokens_len) return QMK_ERR_INVALID_ARG;
  if (n_steps == 0) return QMK_OK;
  int rc = check_step_args(h, first_pos + n_steps - 1);
  if (rc) return rc;
  QMK_CUDA(h, cudaSetDevice(h->device));
  cudaStream_t stream = (cudaStream_t)cuda_stream;
  if (h->st.batch != 1) return QMK_ERR_INVALID_ARG;
  const bool batched = use_batched(h);
  const qmk_state_ptrs saved = h->st;
  for (int i = 0; i < n_steps; ++i) {
    const int pos = first_pos + i;
    QMK_CUDA(h, cudaMemcpyAsync(h->d_tok, host_tokens + pos, sizeof(int64_t), cudaMemcpyHostToDevice, stream));
    if (batched) {
      h->st.token_in = (const int64_t*)h->d_tok;
      h->st.next_token = (int64_t*)(h->d_tok + 1);
      h->st.out_tokens = nullptr;
      h->st.position_ids = nullptr;
      rc = batched_launch(h, pos, 0, qmkb_num_phases(&h->desc), 0, stream);
      h->st = saved;
    } else {
      Params p;
      fill_params(h, p, pos);
      p.token_in = h->d_tok;
      p.next_token = h->d_tok + 1;
      p.out_tokens = nullptr;
      rc = step_with(h, p, stream);
    }
    if (rc) return rc;
    int64_t* dst = teacher_forced ? host_argmax + i : host_tokens + pos + 1;
    QMK_CUDA(h, cudaMemcpyAsync(dst, h->d_tok + 1, sizeof(int64_t), cudaMemcpyDeviceToHost, stream));
    QMK_CUDA(h, cudaStreamSynchronize(stream));
  }
  return QMK_OK;
}

extern "C" int qmk_poll_status(qmk_handle* h, qmk_status* out) {
  if (!h || !out) return QMK_ERR_INVALID_ARG;
  QMK_CUDA(h, cudaSetDevice(h->device));
  QMK_CUDA(h, cudaStreamSynchronize(h->last_stream));
  unsigned words[8];
  unsigned* status = (h->last_kernel == 1 && h->bctx) ? qmkb_status_ptr(h->bctx) : h->status;
  QMK_CUDA(h, cudaMemcpy(words, status, sizeof(words), cudaMemcpyDeviceToHost));
  out->code = (int32_t)words[kStCode];
  out->sm = (int32_t)words[kStSm];
  out->warp = (int32_t)words[kStWarp];
  out->phase = (int32_t)words[kStPhase];
  out->seen = words[kStSeen];
  out->expected = words[kStExpected];
  out->detail = (int32_t)words[kStDetail];
  out->reserved = 0;
  if (out->code == kErrRowPosition) {
    // no wait expired: a row's position was out of range, the row was switched off and the step completed
    QMK_CUDA(h, cudaMemsetAsync(status, 0, 32, h->last_stream));
    QMK_CUDA(h, cudaStreamSynchronize(h->last_stream));
    return QMK_ERR_POSITION;
  }
  if (out->code != 0) {
    // The aborted launch left half-written tagged words: start over from a clean slate.
    int rc = reset_scratch(h, h->last_stream);
    if (rc) return rc;
    if (h->bctx) {
      rc = qmkb_reset(h->bctx, h->last_stream);
      if (rc) return rc;
    }
    QMK_CUDA(h, cudaMemsetAsync(h->status, 0, 32, h->last_stream));
    QMK_CUDA(h, cudaStreamSynchronize(h->last_stream));
    return QMK_ERR_DEVICE_TIMEOUT;
  }
  return QMK_OK;
}

extern "C" int qmk_set_timeout_cycles(qmk_handle* h, int64_t cycles) {
  if (!h || cycles < 1000) return QMK_ERR_INVALID_ARG;
  h->timeout_cycles = cycles;
  return QMK_OK;
}

extern "C" int qmk_set_trace(qmk_handle* h, void* device_buffer, int64_t bytes) {
  if (!h) return QMK_ERR_INVALID_ARG;
  if (device_buffer == nullptr) { h->trace = nullptr; return QMK_OK; }
  const int64_t need = (int64_t)h->n_sm * (use_batched(h) ? qmkb_num_phases(&h->desc) * 2 : num_phases(h->desc.num_layers)) * 8 * 8;   // 16 words per (CTA, phase) in the batched kernel, 8 in the batch-1 kernel
  if (bytes < need || (reinterpret_cast<uintptr_t>(device_buffer) & 7u)) return QMK_ERR_INVALID_ARG;
  h->trace = (unsigned long long*)device_buffer;
  return QMK_OK;
}

extern "C" int qmk_set_kernel_variant(qmk_handle* h, int32_t variant) {
  if (!h || (variant != 0 && variant != 1)) return QMK_ERR_INVALID_ARG;
  h->variant = variant;
  if (use_batched(h)) {
    QMK_CUDA(h, cudaSetDevice(h->device));
    return ensure_bctx(h);
  }
  return QMK_OK;
}

extern "C" int qmk_set_cooperative_launch(qmk_handle* h, int32_t on) {
  if (!h) return QMK_ERR_INVALID_ARG;
  h->cooperative = on ? 1 : 0;
  return QMK_OK;
}

extern "C" int qmk_set_wait_first_dependency(qmk_handle* h, int32_t on) {
  if (!h) return QMK_ERR_INVALID_ARG;
  h->wait_first = on ? 1 : 0;
  return QMK_OK;
}

extern "C" int64_t qmk_step_bytes(const qmk_handle* h, int32_t pos_id) {
  if (!h) return 0;
  const qmk_model_desc& d = h->desc;
  const long long H = d.hidden_size, I = d.intermediate_size;
  const long long QKV = (long long)(d.num_attention_heads + 2 * d.num_key_value_heads) * d.head_dim;
  const long long QD = (long long)d.num_attention_heads * d.head_dim;
  long long per_layer = 2 * (QKV * H + H * QD + 2 * I * H + H * I);
  if (d.arch == QMK_ARCH_MOE) {
    // experts touched by a step: at most one distinct set of top-k per row (an upper bound; the kernel reads the
    // distinct experts only, which for near-uniform routing is min(E, about B * k))
    const long long Bq = h->bound ? h->st.batch : 1;
    long long touched = Bq * d.num_experts_per_tok;
    if (touched > d.num_experts) touched = d.num_experts;
    per_layer = 2 * (QKV * H + H * QD + (long long)d.num_experts * H + touched * 3 * H * d.moe_intermediate_size);
  }
  const long long lm = 2ll * d.vocab_size * H;
  const long long kv_row = 2ll * d.num_key_value_heads * d.head_dim * 2;   // K and V, bf16
  const long long T = (long long)pos_id + 1;
  const long long B = h->bound ? h->st.batch : 1;   // every row at pos_id: weights once, KV per sequence
  return d.num_layers * per_layer + lm + B * (d.num_layers * kv_row * T + d.num_layers * kv_row);
}

extern "C" int qmk_last_expert_count(qmk_handle* h, int32_t* out) {
  if (!h || !out) return QMK_ERR_INVALID_ARG;
  *out = 0;
  if (!h->bctx || !qmkb_expert_count_ptr(h->bctx)) return QMK_OK;
  QMK_CUDA(h, cudaSetDevice(h->device));
  QMK_CUDA(h, cudaStreamSynchronize(h->last_stream));
  QMK_CUDA(h, cudaMemcpy(out, qmkb_expert_count_ptr(h->bctx), sizeof(int32_t), cudaMemcpyDeviceToHost));
  return QMK_OK;
}

extern "C" int qmk_last_expert_routing(qmk_handle* h, int32_t* count, int32_t* experts, float* weights) {
  if (!h || !count || !experts || !weights) return QMK_ERR_INVALID_ARG;
  *count = 0;
  if (!h->bctx || !qmkb_expert_count_ptr(h->bctx)) return QMK_OK;
  QMK_CUDA(h, cudaSetDevice(h->device));
  QMK_CUDA(h, cudaStreamSynchronize(h->last_stream));
  const int E = h->desc.num_experts;
  QMK_CUDA(h, cudaMemcpy(count, qmkb_expert_count_ptr(h->bctx), sizeof(int32_t), cudaMemcpyDeviceToHost));
  QMK_CUDA(h, cudaMemcpy(experts, qmkb_expert_list_ptr(h->bctx), sizeof(int32_t) * E, cudaMemcpyDeviceToHost));
  QMK_CUDA(h, cudaMemcpy(weights, qmkb_expert_weight_ptr(h->bctx), sizeof(float) * E * 64, cudaMemcpyDeviceToHost));
  return QMK_OK;
}

extern "C" int qmk_ep_export(qmk_handle* h, void* ipc_handle_out) {
  if (!h || !ipc_handle_out) return QMK_ERR_INVALID_ARG;
  QMK_CUDA(h, cudaSetDevice(h->device));
  int rc = ensure_bctx(h);
  if (rc) return rc;
  return qmkb_ep_export(h->bctx, ipc_handle_out, h->cuda_err, sizeof(h->cuda_err));
}

extern "C" int qmk_ep_connect(qmk_handle* h, const void* ipc_handles) {
  if (!h || !ipc_handles || !h->bctx) return QMK_ERR_INVALID_ARG;
  QMK_CUDA(h, cudaSetDevice(h->device));
  return qmkb_ep_connect(h->bctx, ipc_handles, h->cuda_err, sizeof(h->cuda_err));
}

extern "C" int qmk_expert_reads(qmk_handle* h, int64_t* total, int32_t reset) {
  if (!h || !total) return QMK_ERR_INVALID_ARG;
  *total = 0;
  if (!h->bctx || !qmkb_expert_reads_ptr(h->bctx)) return QMK_OK;
  QMK_CUDA(h, cudaSetDevice(h->device));
  QMK_CUDA(h, cudaStreamSynchronize(h->last_stream));
  unsigned long long v = 0;
  QMK_CUDA(h, cudaMemcpy(&v, qmkb_expert_reads_ptr(h->bctx), sizeof(v), cudaMemcpyDeviceToHost));
  *total = (int64_t)v;
  if (reset) QMK_CUDA(h, cudaMemset(qmkb_expert_reads_ptr(h->bctx), 0, sizeof(v)));
  return QMK_OK;
}

extern "C" int64_t qmk_launch_count(const qmk_handle* h) { return h ? h->launches : 0; }

extern "C" int qmk_launch_geometry(const qmk_handle* h, int32_t* ctas, int32_t* threads, int32_t* smem_bytes) {
  if (!h) return QMK_ERR_INVALID_ARG;
  if (use_batched(h) && h->bctx) {
    qmkb_geometry(h->bctx, ctas, threads, smem_bytes);
    return QMK_OK;
  }
  if (ctas) *ctas = h->n_sm;
  if (threads) *threads = kLaunchThreads;
  if (smem_bytes) *smem_bytes = SmemLayout<Shape>::kTotal;
  return QMK_OK;
}
