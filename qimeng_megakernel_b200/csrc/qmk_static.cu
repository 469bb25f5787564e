// qmk_decode_step_static: one decode step for callers that must not allocate device memory.
//
// Who needs this: code that runs where cudaMalloc is off limits -- a serving loop whose memory is
// owned entirely by a framework's pool allocator and audited for stray driver allocations, a step that
// is issued from inside a region where allocation would synchronise the device, or an embedder that
// hands this library a fixed memory budget.  The handle-based entry points allocate their scratch
// (hand-off words, split-KV records, status) with cudaMalloc in qmk_create; this one keeps the same
// scratch in a file-scope __device__ array instead, so the library image itself carries it.
//
// Consequences the caller must know:
//  * every GPU that loads the library holds kStaticScratchBytes (2 MiB) of device memory until exit;
//  * all calls on a device share that one array.  Its contents survive from call to call; the words
//    that must start at zero (arg-max key, LM-head ticket) are cleared at the start of every call, the
//    tagged words need no clearing because each call uses fresh tags;
//  * the status record of a bounded wait that expired also lives in the array and is NOT cleared by
//    later calls: it stays until qmk_static_poll_status reads it (and then clears the whole array), so
//    a failure cannot be lost behind steps that were queued after it;
//  * two calls that overlap on the same GPU (two streams, two threads) race on the array: issue them
//    on one stream, one after the other;
//  * the first call on a device performs the set-up (symbol address, kernel attribute, device
//    properties).  Make that first call outside any stream capture.
//  * no cudaMalloc, cudaFree or allocating library routine is called, ever.
#include <cuda_runtime.h>
#include <stdio.h>
#include <string.h>

#include "../../include/qmk_b200.h"
#include "qmk_megakernel.cuh"

using namespace qmk;
using Shape = ShapeLlama1B;

namespace {

constexpr size_t kStaticScratchBytes = QMK_STATIC_SCRATCH_MAX_BYTES;   // the stated maximum: 2 MiB per GPU
constexpr int kMaxDevices = 64;

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

struct StaticLayout {   // byte offsets inside the array (each 256-aligned)
  size_t part_rec, t_hid_o, t_hid_d, t_q, t_attn, t_silu, tickets, argmax, status, total;
};

size_t align256(size_t v) { return (v + 255) / 256 * 256; }

// Scratch a model of this descriptor needs; the compiled shape fixes everything but the head geometry.
StaticLayout layout_for(const qmk_model_desc& d) {
  StaticLayout l;
  size_t o = 0;
  l.part_rec = o; o += align256((size_t)d.num_attention_heads * kMaxSplits * (d.head_dim + 2) * 8);
  l.t_hid_o = o;  o += align256((size_t)d.hidden_size * 4);
  l.t_hid_d = o;  o += align256((size_t)d.hidden_size * 4);
  l.t_q = o;      o += align256((size_t)(d.num_attention_heads + 2 * d.num_key_value_heads) * d.head_dim * 4);
  l.t_attn = o;   o += align256((size_t)d.num_attention_heads * d.head_dim * 4);
  l.t_silu = o;   o += align256((size_t)d.intermediate_size * 4);
  l.tickets = o;  o += 512;
  l.argmax = o;   o += 256;
  l.status = o;   o += 256;
  l.total = o;
  return l;
}

struct DeviceSetup {
  bool ready;
  unsigned char* scratch;   // DEVICE address of g_static_scratch on this device (from cudaGetSymbolAddress)
  int n_sm;
  unsigned launch_seq;
  long long timeout_cycles;   // device-side wait budget (qmk_static_set_timeout_cycles), 0 = default
  int wait_first;             // failure-detection knob (qmk_static_set_wait_first_dependency)
  cudaStream_t last_stream;   // stream of the last launch: what qmk_static_poll_status synchronises
  size_t status_off;          // offset of the status record used by the last launch
  bool launched;
};
constexpr long long kDefaultTimeoutCycles = 2000000000ll;
DeviceSetup g_setup[kMaxDevices];
char g_static_err[256];

int fail(cudaError_t e, const char* what) {
  snprintf(g_static_err, sizeof(g_static_err), "%s: %s", what, cudaGetErrorString(e));
  return QMK_ERR_CUDA;
}

// Once per device, with that device current.  The array's name is only a host-side stand-in for the
// symbol: the address a kernel may use comes from cudaGetSymbolAddress.
int setup_device(int device) {
  DeviceSetup& s = g_setup[device];
  if (s.ready) return QMK_OK;
  cudaDeviceProp prop;
  cudaError_t e = cudaGetDeviceProperties(&prop, device);
  if (e != cudaSuccess) return fail(e, "cudaGetDeviceProperties");
  if (prop.major != 10 || (int)prop.sharedMemPerBlockOptin < SmemLayout<Shape>::kTotal || !prop.cooperativeLaunch)
    return QMK_ERR_DEVICE;
  void* ptr = nullptr;
  e = cudaGetSymbolAddress(&ptr, g_static_scratch);
  if (e != cudaSuccess) return fail(e, "cudaGetSymbolAddress(g_static_scratch)");
  if (ptr == nullptr) return QMK_ERR_CUDA;
  e = cudaFuncSetAttribute(qmk_decode_kernel<Shape>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           SmemLayout<Shape>::kTotal);
  if (e != cudaSuccess) return fail(e, "cudaFuncSetAttribute");
  s.scratch = static_cast<unsigned char*>(ptr);
  s.n_sm = prop.multiProcessorCount;
  s.launch_seq = 0;
  s.ready = true;
  return QMK_OK;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

extern "C" int qmk_decode_step_static(const qmk_model_desc* d, const qmk_weight_ptrs* w, const qmk_state_ptrs* st,
                                      int32_t pos_id, int device, void* cuda_stream) {
  if (!d || !w || !st) return QMK_ERR_INVALID_ARG;
  if (device < 0 || device >= kMaxDevices) return QMK_ERR_INVALID_ARG;
  if (d->abi_version != QMK_ABI_VERSION) return QMK_ERR_INVALID_ARG;
  if (d->num_layers < 0 || d->num_layers > 255 || d->vocab_size < 1 || d->rope_rows < 1) return QMK_ERR_INVALID_ARG;
  if (d->num_attention_heads < 1 || d->head_dim < 1 || d->hidden_size < 1 || d->intermediate_size < 1 ||
      d->num_key_value_heads < 1)
    return QMK_ERR_INVALID_ARG;
  // size check first: a model whose scratch does not fit the fixed array is refused with its own code
  const StaticLayout lay = layout_for(*d);
  if (lay.total > kStaticScratchBytes) return QMK_ERR_SCRATCH_TOO_LARGE;
  if (d->arch != QMK_ARCH_LLAMA || d->hidden_size != Shape::H || d->intermediate_size != Shape::I ||
      d->num_attention_heads != Shape::NH || d->num_key_value_heads != Shape::NKV || d->head_dim != Shape::HD)
    return QMK_ERR_UNSUPPORTED_MODEL;
  if (!(d->rms_norm_eps > 0.f) || !(d->attn_scale > 0.f)) return QMK_ERR_INVALID_ARG;
  const void* wp[] = {w->attn_norm, w->qkv, w->o_proj, w->mlp_norm, w->up_proj, w->gate_proj,
                      w->down_proj, w->lm_head_norm, w->lm_head, w->rope_cos, w->rope_sin};
  for (const void* p : wp)
    if (!p || !aligned16(p)) return QMK_ERR_INVALID_ARG;
  void* sp[] = {st->hidden_states, st->q_post_rope, st->k_cache, st->v_cache, st->attn_out, st->silu_out, st->logits};
  for (void* p : sp)
    if (!p || !aligned16(p)) return QMK_ERR_INVALID_ARG;
  if (st->batch != 1 || st->kv_seq_len < 1) return QMK_ERR_INVALID_ARG;
  // the batch-1 kernel has neither per-row positions nor an active mask: refuse rather than ignore them
  if (st->position_ids != nullptr || st->active_mask != nullptr || st->kv_slots != nullptr) return QMK_ERR_INVALID_ARG;
  if (st->token_in && !w->embed_tokens) return QMK_ERR_INVALID_ARG;
  if (pos_id < 0 || pos_id >= st->kv_seq_len || pos_id >= d->rope_rows) return QMK_ERR_POSITION;

  cudaError_t e = cudaSetDevice(device);
  if (e != cudaSuccess) return fail(e, "cudaSetDevice");
  int rc = setup_device(device);     // first call on this device only; keep it outside stream capture
  if (rc != QMK_OK) return rc;
  DeviceSetup& dev = g_setup[device];
  {
    const unsigned long long nwt = (unsigned long long)dev.n_sm * kWorkers;
    const unsigned long long units = d->vocab_size > Shape::I ? d->vocab_size : Shape::I;
    if ((nwt + 1) * units >= (1ull << 32)) return QMK_ERR_INVALID_ARG;
  }
  cudaStream_t stream = (cudaStream_t)cuda_stream;
  // what must start at zero: LM-head ticket and arg-max key (contiguous).  The status record behind them is left
  // alone: a record written by an earlier call stays until qmk_static_poll_status has read it.
  e = cudaMemsetAsync(dev.scratch + lay.tickets, 0, lay.status - lay.tickets, stream);
  if (e != cudaSuccess) return fail(e, "cudaMemsetAsync");

  Params p;
  memset(&p, 0, sizeof(p));
  p.attn_norm = (const uint16_t*)w->attn_norm;
  p.qkv = (const uint16_t*)w->qkv;
  p.o_proj = (const uint16_t*)w->o_proj;
  p.mlp_norm = (const uint16_t*)w->mlp_norm;
  p.up = (const uint16_t*)w->up_proj;
  p.gate = (const uint16_t*)w->gate_proj;
  p.down = (const uint16_t*)w->down_proj;
  p.lm_norm = (const uint16_t*)w->lm_head_norm;
  p.lm_head = (const uint16_t*)w->lm_head;
  p.embed = (const uint16_t*)w->embed_tokens;
  p.rope_cos = w->rope_cos;
  p.rope_sin = w->rope_sin;
  p.hidden = (uint16_t*)st->hidden_states;
  p.q_post_rope = (uint16_t*)st->q_post_rope;
  p.k_cache = (uint16_t*)st->k_cache;
  p.v_cache = (uint16_t*)st->v_cache;
  p.attn_out = (uint16_t*)st->attn_out;
  p.silu_out = (uint16_t*)st->silu_out;
  p.logits = (uint16_t*)st->logits;
  p.next_token = (long long*)st->next_token;
  p.token_in = (const long long*)st->token_in;
  p.out_tokens = (long long*)st->out_tokens;
  p.out_tokens_len = st->out_tokens_len;
  p.kv_seq_stride = (long long)Shape::NKV * Shape::HD;
  p.kv_layer_stride = (long long)(st->kv_batch > 0 ? st->kv_batch : st->batch) * st->kv_seq_len * p.kv_seq_stride;
  p.part_rec = (unsigned long long*)(dev.scratch + lay.part_rec);
  p.t_hid_o = (uint32_t*)(dev.scratch + lay.t_hid_o);
  p.t_hid_d = (uint32_t*)(dev.scratch + lay.t_hid_d);
  p.t_q = (uint32_t*)(dev.scratch + lay.t_q);
  p.t_attn = (uint32_t*)(dev.scratch + lay.t_attn);
  p.t_silu = (uint32_t*)(dev.scratch + lay.t_silu);
  p.tickets = (unsigned*)(dev.scratch + lay.tickets);
  p.argmax_key = (unsigned long long*)(dev.scratch + lay.argmax);
  p.tok_word = (unsigned long long*)(dev.scratch + lay.argmax + 64);
  p.n_steps = 1;
  p.status = (unsigned*)(dev.scratch + lay.status);
  p.trace = nullptr;
  p.num_layers = d->num_layers;
  p.vocab = d->vocab_size;
  p.pos = pos_id;
  p.phase_begin = 0;
  p.phase_end = num_phases(d->num_layers);
  p.sync = 1;
  p.wait_first = dev.wait_first;
  if (dev.wait_first) {   // the first phase will wait for words nothing writes: no stale tag may match by accident
    e = cudaMemsetAsync(dev.scratch, 0, lay.tickets, stream);
    if (e != cudaSuccess) return fail(e, "cudaMemsetAsync");
  }
  if (dev.launch_seq >= (1u << 23)) {   // tags would wrap: start over on a cleared array
    e = cudaMemsetAsync(dev.scratch, 0, lay.status, stream);
    if (e != cudaSuccess) return fail(e, "cudaMemsetAsync");
    dev.launch_seq = 0;
  }
  p.stream_end = p.phase_end;
  p.launch_seq = ++dev.launch_seq;
  p.eps = d->rms_norm_eps;
  p.scale_log2e = d->attn_scale * 1.4426950408889634f;
  p.timeout_cycles = dev.timeout_cycles > 0 ? dev.timeout_cycles : kDefaultTimeoutCycles;

  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((unsigned)dev.n_sm);
  cfg.blockDim = dim3(kLaunchThreads);
  cfg.dynamicSmemBytes = SmemLayout<Shape>::kTotal;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, qmk_decode_kernel<Shape>, p);
  if (e != cudaSuccess) return fail(e, "cudaLaunchKernelEx");
  dev.last_stream = stream;
  dev.status_off = lay.status;
  dev.launched = true;
  return QMK_OK;
}

// Reads the status record that qmk_decode_step_static launches leave in the static array: synchronises the stream of
// the last launch on `device`, copies the 32-byte record to the host (a cudaMemcpy into the caller's struct: nothing
// is allocated).  A non-zero record means a bounded wait expired in some launch since the last poll: the whole array
// is then cleared (half-written hand-off words of the aborted launch must not survive) and QMK_ERR_DEVICE_TIMEOUT is
// returned; the outputs of that launch and of launches queued behind it are not to be trusted.
extern "C" int qmk_static_poll_status(int device, qmk_status* out) {
  if (!out || device < 0 || device >= kMaxDevices) return QMK_ERR_INVALID_ARG;
  memset(out, 0, sizeof(*out));
  DeviceSetup& dev = g_setup[device];
  if (!dev.ready || !dev.launched) return QMK_OK;   // nothing was ever launched on this device
  cudaError_t e = cudaSetDevice(device);
  if (e != cudaSuccess) return fail(e, "cudaSetDevice");
  e = cudaStreamSynchronize(dev.last_stream);
  if (e != cudaSuccess) return fail(e, "cudaStreamSynchronize");
  unsigned words[8];
  e = cudaMemcpy(words, dev.scratch + dev.status_off, sizeof(words), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return fail(e, "cudaMemcpy(status)");
  out->code = (int32_t)words[kStCode];
  out->sm = (int32_t)words[kStSm];
  out->warp = (int32_t)words[kStWarp];
  out->phase = (int32_t)words[kStPhase];
  out->seen = words[kStSeen];
  out->expected = words[kStExpected];
  out->detail = (int32_t)words[kStDetail];
  if (out->code != 0) {
    e = cudaMemsetAsync(dev.scratch, 0, kStaticScratchBytes, dev.last_stream);
    if (e != cudaSuccess) return fail(e, "cudaMemsetAsync");
    e = cudaStreamSynchronize(dev.last_stream);
    if (e != cudaSuccess) return fail(e, "cudaStreamSynchronize");
    return QMK_ERR_DEVICE_TIMEOUT;
  }
  return QMK_OK;
}

// Wait budget of the static entry point's launches on `device`, in SM clock cycles (0 restores the default, 2e9).
extern "C" int qmk_static_set_timeout_cycles(int device, int64_t cycles) {
  if (device < 0 || device >= kMaxDevices || (cycles != 0 && cycles < 1000)) return QMK_ERR_INVALID_ARG;
  g_setup[device].timeout_cycles = cycles;
  return QMK_OK;
}

// Failure-detection knob, the counterpart of qmk_set_wait_first_dependency: while set, the first phase of every
// static launch on `device` also waits for hand-off words that nothing writes, so its bounded wait must expire.
extern "C" int qmk_static_set_wait_first_dependency(int device, int32_t on) {
  if (device < 0 || device >= kMaxDevices) return QMK_ERR_INVALID_ARG;
  g_setup[device].wait_first = on ? 1 : 0;
  return QMK_OK;
}

// Text of the last CUDA runtime error seen by the static entry points (QMK_ERR_CUDA), empty if none.
extern "C" const char* qmk_static_last_cuda_error(void) { return g_static_err; }
