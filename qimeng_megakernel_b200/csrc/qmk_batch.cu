// Host side of the batched decode kernel: tensor maps of the weight matrices, scratch, launch.
// The reference's multi-batch launcher fills a globals POD from torch tensors and launches one kernel per
// step (qimeng_megakernel/models/LLM/llama/llama3_2__1b/A100/multi_batch/decode_kernel/mk.cu); here the
// descriptor is plain data, scratch is owned by the context and errors are returned.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <new>

#include "qmk_batch_host.h"
#include "qmk_batch_kernel.cuh"

using namespace qmkb;

struct qmk_batch_ctx {
  qmk_model_desc desc;
  qmk_weight_ptrs w;
  int n_sm;
  TensorMaps maps;
  unsigned char* scratch;
  size_t scratch_bytes;
  // regions of the scratch
  long long* ws;
  float* ss;
  float* attn_part;
  int* moe_ne;
  unsigned long long* moe_ne_sum;
  int* moe_elist;
  float* moe_w;
  unsigned char* ximg;
  unsigned char* eimg;
  unsigned char* aimg;
  unsigned char* simg;
  unsigned* img_done;
  size_t img_bytes;       // ximg, aimg and simg are one range
  int img_batch;          // batch size the images were last used with
  unsigned char* zero_begin;   // [phase_done | tile_tickets | attn_tickets | argmax_key]: zeroed before every launch
  size_t zero_bytes;
  unsigned* phase_done;
  unsigned* tile_tickets;
  unsigned* attn_tickets;
  unsigned long long* argmax_key;
  unsigned* status;
  unsigned epoch;
  // expert parallelism
  unsigned char* ep_local;       // this rank's exchange buffer (data, then flags)
  size_t ep_data_bytes, ep_flag_bytes, ep_key_bytes, ep_bytes;
  void* ep_peer[8];              // every rank's buffer as mapped here (own = ep_local); null until connected
  bool ep_connected;
};

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
static int fail(char* err, size_t n, const char* what, cudaError_t e) {
  if (err && n) snprintf(err, n, "%s: %s", what, cudaGetErrorString(e));
  return QMK_ERR_CUDA;
}

int qmkb_supported(const qmk_model_desc* d) {
  const int H = d->hidden_size, I = d->intermediate_size, NH = d->num_attention_heads, NKV = d->num_key_value_heads,
            HD = d->head_dim;
  if (d->arch != QMK_ARCH_LLAMA && d->arch != QMK_ARCH_QWEN3 && d->arch != QMK_ARCH_MOE) return QMK_ERR_UNSUPPORTED_MODEL;
  if (d->arch == QMK_ARCH_MOE) {
    if (d->num_experts < 8 || d->num_experts > kTileRows || d->num_experts_per_tok < 1 || d->num_experts_per_tok > 16 ||
        d->num_experts_per_tok > d->num_experts || d->moe_intermediate_size < kBlockK ||
        d->moe_intermediate_size % kBlockK != 0)
      return QMK_ERR_UNSUPPORTED_MODEL;
  }
  if (d->ep_world > 1) {
    if (d->arch != QMK_ARCH_MOE || (d->ep_world != 2 && d->ep_world != 4 && d->ep_world != 8) ||
        d->num_experts % d->ep_world != 0 || d->ep_rank < 0 || d->ep_rank >= d->ep_world)
      return QMK_ERR_UNSUPPORTED_MODEL;
  }
  if (d->tp_world > 1) {
    if (d->arch == QMK_ARCH_MOE || (d->tp_world != 2 && d->tp_world != 4 && d->tp_world != 8) || d->tp_rank < 0 ||
        d->tp_rank >= d->tp_world || d->embed_rows < d->vocab_size * d->tp_world)
      return QMK_ERR_UNSUPPORTED_MODEL;
  }
  if (HD != 64 && HD != 128) return QMK_ERR_UNSUPPORTED_MODEL;
  if (NH < 1 || NKV < 1 || NH % NKV != 0) return QMK_ERR_UNSUPPORTED_MODEL;
  const int gq = NH / NKV;
  if (gq != 1 && gq != 2 && gq != 4) return QMK_ERR_UNSUPPORTED_MODEL;
  if (H < kBlockK || H % kBlockK != 0 || H > 8192) return QMK_ERR_UNSUPPORTED_MODEL;
  if (d->arch != QMK_ARCH_MOE && (I < kBlockK || I % kBlockK != 0)) return QMK_ERR_UNSUPPORTED_MODEL;
  if ((NH * HD) % kBlockK != 0 || NKV > 64) return QMK_ERR_UNSUPPORTED_MODEL;
  return QMK_OK;
}

int qmkb_num_phases(const qmk_model_desc* d) { return (d->arch == QMK_ARCH_MOE ? 6 : 5) * d->num_layers + 1; }

typedef CUresult (*encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// bf16 matrix [layers, rows, k] row-major -> 3-D map {k, rows, layers}, box {64, box_rows, 1}, 128-byte swizzle,
// rows past the end read as zero.
static int make_map(encode_fn enc, CUtensorMap* m, const void* base, long long k, long long rows, long long layers,
                    int box_rows) {
  const cuuint64_t dims[3] = {(cuuint64_t)k, (cuuint64_t)rows, (cuuint64_t)(layers > 0 ? layers : 1)};
  const cuuint64_t strides[2] = {(cuuint64_t)k * 2, (cuuint64_t)k * 2 * (cuuint64_t)rows};
  const cuuint32_t box[3] = {(cuuint32_t)kBlockK, (cuuint32_t)box_rows, 1};
  const cuuint32_t es[3] = {1, 1, 1};
  const CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, es,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

int qmkb_create(const qmk_model_desc* d, const qmk_weight_ptrs* w, int n_sm, qmk_batch_ctx** out, char* err, size_t errlen) {
  *out = nullptr;
  int rc = qmkb_supported(d);
  if (rc) return rc;
  if (d->arch == QMK_ARCH_QWEN3 && (!w->q_norm || !w->k_norm)) return QMK_ERR_INVALID_ARG;
  if (d->arch == QMK_ARCH_MOE && (!w->router || !w->expert_gate_up || !w->expert_down)) return QMK_ERR_INVALID_ARG;
  qmk_batch_ctx* c = new (std::nothrow) qmk_batch_ctx();
  if (!c) return QMK_ERR_OOM;
  memset(c, 0, sizeof(*c));
  c->desc = *d;
  c->w = *w;
  c->n_sm = n_sm;
  const int H = d->hidden_size, I = d->intermediate_size, NH = d->num_attention_heads, NKV = d->num_key_value_heads,
            HD = d->head_dim, L = d->num_layers, V = d->vocab_size;
  const int QKV = (NH + 2 * NKV) * HD, QD = NH * HD;
  do {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess || !fn || qres != cudaDriverEntryPointSuccess) {
      rc = fail(err, errlen, "cudaGetDriverEntryPoint(cuTensorMapEncodeTiled)", e);
      break;
    }
    encode_fn enc = (encode_fn)fn;
    int bad = 0;
    const bool moe = d->arch == QMK_ARCH_MOE;
    const int E = moe ? d->num_experts : 0, Ie = moe ? d->moe_intermediate_size : 0;
    const int El = d->ep_world > 1 ? E / d->ep_world : E;   // experts this rank holds
    if (L > 0) {
      bad |= make_map(enc, &c->maps.qkv, w->qkv, H, QKV, L, kTileRows);
      bad |= make_map(enc, &c->maps.o_proj, w->o_proj, QD, H, L, kTileRows);
      if (moe) {
        bad |= make_map(enc, &c->maps.router, w->router, H, E, L, kTileRows);
        bad |= make_map(enc, &c->maps.egu, w->expert_gate_up, H, 2 * Ie, (long long)L * El, kTileRows / 2);
        bad |= make_map(enc, &c->maps.edown, w->expert_down, Ie, H, (long long)L * El, kTileRows);
      } else {
        bad |= make_map(enc, &c->maps.up, w->up_proj, H, I, L, kTileRows / 2);
        bad |= make_map(enc, &c->maps.gate, w->gate_proj, H, I, L, kTileRows / 2);
        bad |= make_map(enc, &c->maps.down, w->down_proj, I, H, L, kTileRows);
      }
    }
    bad |= make_map(enc, &c->maps.lm_head, w->lm_head, H, V, 1, kTileRows);
    if (bad) {
      if (err && errlen) snprintf(err, errlen, "cuTensorMapEncodeTiled failed (CUresult %d)", bad);
      rc = QMK_ERR_CUDA;
      break;
    }
    e = cudaFuncSetAttribute(plain::qmk_batch_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(traced::qmk_batch_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget);
    if (e != cudaSuccess) { rc = fail(err, errlen, "cudaFuncSetAttribute", e); break; }

    int max_tiles = (V + kTileRows - 1) / kTileRows;
    const int t_upgate = moe ? E * (Ie / (kTileRows / 2)) : (I + kTileRows / 2 - 1) / (kTileRows / 2), t_qkv = (QKV + kTileRows - 1) / kTileRows;
    if (t_upgate > max_tiles) max_tiles = t_upgate;
    if (t_qkv > max_tiles) max_tiles = t_qkv;
    if ((H + kTileRows - 1) / kTileRows > max_tiles) max_tiles = (H + kTileRows - 1) / kTileRows;
    const int gq = NH / NKV;
    const size_t b_ws = align_up((size_t)n_sm * kTileRows * kMaxBatch * 8, 256);
    const size_t b_ss = align_up((size_t)((H + kTileRows - 1) / kTileRows) * kMaxBatch * 4, 256);
    const size_t b_part = align_up(((size_t)n_sm * 8 + (size_t)kMaxBatch * NKV) * gq * (HD + 2) * 4, 256);
    const size_t b_done = align_up((size_t)(6 * L + 1 + 2) * 4, 256);
    const size_t b_moe = moe ? align_up(256 + (size_t)E * 4, 256) + align_up((size_t)E * kMaxBatch * 4, 256) +
                                   align_up((size_t)E * kMaxBatch * Ie * 2, 256) +
                                   0 : 0;
    const size_t b_img = align_up((size_t)H * kMaxBatch * 2, 256) + align_up((size_t)NH * HD * kMaxBatch * 2, 256) +
                         (moe ? 0 : align_up((size_t)I * kMaxBatch * 2, 256));
    const size_t b_tt = align_up((size_t)max_tiles * 4, 256);
    const size_t b_at = align_up((size_t)kMaxBatch * NKV * 4, 256);
    const size_t b_am = align_up((size_t)kMaxBatch * 8, 256);
    const size_t b_status = 256;
    c->scratch_bytes = b_ws + b_ss + b_part + b_moe + b_img + 2 * b_done + b_tt + b_at + b_am + b_status;
    e = cudaMalloc((void**)&c->scratch, c->scratch_bytes);
    if (e != cudaSuccess) { rc = QMK_ERR_OOM; fail(err, errlen, "cudaMalloc", e); break; }
    unsigned char* q = c->scratch;
    c->ws = (long long*)q; q += b_ws;
    c->ss = (float*)q; q += b_ss;
    c->attn_part = (float*)q; q += b_part;
    if (moe) {
      c->moe_ne = (int*)q; c->moe_ne_sum = (unsigned long long*)(q + 64); c->moe_elist = (int*)(q + 256); q += align_up(256 + (size_t)E * 4, 256);
      c->moe_w = (float*)q; q += align_up((size_t)E * kMaxBatch * 4, 256);
      c->eimg = q; q += align_up((size_t)E * kMaxBatch * Ie * 2, 256);
    }
    c->ximg = q; c->img_bytes = b_img; c->img_batch = 0;
    q += align_up((size_t)H * kMaxBatch * 2, 256);
    c->aimg = q; q += align_up((size_t)NH * HD * kMaxBatch * 2, 256);
    c->simg = q; if (!moe) q += align_up((size_t)I * kMaxBatch * 2, 256);
    c->zero_begin = q;
    c->phase_done = (unsigned*)q; q += b_done;
    c->img_done = (unsigned*)q; q += b_done;
    c->tile_tickets = (unsigned*)q; q += b_tt;
    c->attn_tickets = (unsigned*)q; q += b_at;
    c->argmax_key = (unsigned long long*)q; q += b_am;
    c->zero_bytes = (size_t)(q - c->zero_begin);
    c->status = (unsigned*)q;
    e = cudaMemset(c->scratch, 0, c->scratch_bytes);
    if (e != cudaSuccess) { rc = fail(err, errlen, "cudaMemset", e); break; }
  } while (0);
  if (rc != QMK_OK) {
    if (c->scratch) cudaFree(c->scratch);
    delete c;
    return rc;
  }
  *out = c;
  return QMK_OK;
}

static int exchange_world(const qmk_model_desc& d) { return d.ep_world > 1 ? d.ep_world : (d.tp_world > 1 ? d.tp_world : 1); }
static int exchange_rank(const qmk_model_desc& d) { return d.ep_world > 1 ? d.ep_rank : (d.tp_world > 1 ? d.tp_rank : 0); }

int qmkb_ep_export(qmk_batch_ctx* c, void* ipc_handle_out, char* err, size_t errlen) {
  const qmk_model_desc& d = c->desc;
  const int xw = exchange_world(d);
  if (xw <= 1 || !ipc_handle_out) return QMK_ERR_INVALID_ARG;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the ABI documents a 64-byte handle");
  if (!c->ep_local) {
    const size_t tiles = (size_t)((d.hidden_size + kTileRows - 1) / kTileRows);
    // [2 buffers][source rank][tile][128][64] floats | [2][source][tile] flags | [source][64] arg-max keys | [source] key flags
    c->ep_data_bytes = align_up((size_t)2 * xw * tiles * kTileRows * kMaxBatch * 4, 256);
    c->ep_flag_bytes = align_up((size_t)2 * xw * tiles * 4, 256);
    c->ep_key_bytes = align_up((size_t)xw * kMaxBatch * 8, 256);
    c->ep_bytes = c->ep_data_bytes + c->ep_flag_bytes + c->ep_key_bytes + 256;
    cudaError_t e = cudaMalloc((void**)&c->ep_local, c->ep_bytes);
    if (e != cudaSuccess) { fail(err, errlen, "cudaMalloc(exchange buffer)", e); return QMK_ERR_OOM; }
    e = cudaMemset(c->ep_local, 0, c->ep_bytes);
    if (e != cudaSuccess) return fail(err, errlen, "cudaMemset", e);
  }
  cudaIpcMemHandle_t hnd;
  const cudaError_t e = cudaIpcGetMemHandle(&hnd, c->ep_local);
  if (e != cudaSuccess) return fail(err, errlen, "cudaIpcGetMemHandle", e);
  memcpy(ipc_handle_out, &hnd, sizeof(hnd));
  return QMK_OK;
}

int qmkb_ep_connect(qmk_batch_ctx* c, const void* ipc_handles, char* err, size_t errlen) {
  const qmk_model_desc& d = c->desc;
  const int xw = exchange_world(d), xr = exchange_rank(d);
  if (xw <= 1 || !ipc_handles || !c->ep_local) return QMK_ERR_INVALID_ARG;
  if (c->ep_connected) return QMK_OK;
  for (int r = 0; r < xw; ++r) {
    if (r == xr) { c->ep_peer[r] = c->ep_local; continue; }
    cudaIpcMemHandle_t hnd;
    memcpy(&hnd, (const unsigned char*)ipc_handles + (size_t)r * sizeof(hnd), sizeof(hnd));
    const cudaError_t e = cudaIpcOpenMemHandle(&c->ep_peer[r], hnd, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return fail(err, errlen, "cudaIpcOpenMemHandle", e);
  }
  c->ep_connected = true;
  return QMK_OK;
}

void qmkb_destroy(qmk_batch_ctx* c) {
  if (!c) return;
  if (c->ep_connected)
    for (int r = 0; r < exchange_world(c->desc); ++r)
      if (r != exchange_rank(c->desc) && c->ep_peer[r]) cudaIpcCloseMemHandle(c->ep_peer[r]);
  if (c->ep_local) cudaFree(c->ep_local);
  if (c->scratch) cudaFree(c->scratch);
  delete c;
}

unsigned* qmkb_status_ptr(qmk_batch_ctx* c) { return c->status; }
const int* qmkb_expert_count_ptr(const qmk_batch_ctx* c) { return c->moe_ne; }
const int* qmkb_expert_list_ptr(const qmk_batch_ctx* c) { return c->moe_elist; }
unsigned long long* qmkb_expert_reads_ptr(const qmk_batch_ctx* c) { return c->moe_ne_sum; }
const float* qmkb_expert_weight_ptr(const qmk_batch_ctx* c) { return c->moe_w; }
size_t qmkb_scratch_bytes(const qmk_batch_ctx* c) { return c->scratch_bytes; }

int qmkb_reset(qmk_batch_ctx* c, cudaStream_t stream) {
  const cudaError_t e = cudaMemsetAsync(c->scratch, 0, c->scratch_bytes, stream);
  return e == cudaSuccess ? QMK_OK : QMK_ERR_CUDA;
}

void qmkb_geometry(const qmk_batch_ctx* c, int* ctas, int* threads, int* smem_bytes) {
  if (ctas && c) *ctas = c->n_sm;
  if (threads) *threads = kBatchThreads;
  if (smem_bytes) *smem_bytes = kSmemBudget;   // upper bound; a launch asks for smem_plan(Bpad).total
}

int qmkb_launch(qmk_batch_ctx* c, const qmk_state_ptrs* st, const qmkb_launch_args* a, cudaStream_t stream, char* err,
                size_t errlen) {
  const qmk_model_desc& d = c->desc;
  BParams p;
  memset(&p, 0, sizeof(p));
  p.attn_norm = (const uint16_t*)c->w.attn_norm;
  p.mlp_norm = (const uint16_t*)c->w.mlp_norm;
  p.lm_norm = (const uint16_t*)c->w.lm_head_norm;
  p.q_norm = d.arch == QMK_ARCH_QWEN3 ? (const uint16_t*)c->w.q_norm : nullptr;
  p.k_norm = d.arch == QMK_ARCH_QWEN3 ? (const uint16_t*)c->w.k_norm : nullptr;
  p.embed = (const uint16_t*)c->w.embed_tokens;
  p.rope_cos = c->w.rope_cos;
  p.rope_sin = c->w.rope_sin;
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
  p.position_ids = st->position_ids;
  p.active_mask = st->active_mask;
  p.kv_seq_stride = (long long)d.num_key_value_heads * d.head_dim;
  p.kv_batch_stride = (long long)st->kv_seq_len * p.kv_seq_stride;
  p.kv_slots = st->kv_slots;
  p.kv_batch = st->kv_batch > 0 ? st->kv_batch : st->batch;
  p.kv_layer_stride = (long long)p.kv_batch * p.kv_batch_stride;
  p.ws = c->ws;
  p.tile_tickets = c->tile_tickets;
  p.ss = c->ss;
  p.attn_part = c->attn_part;
  p.attn_tickets = c->attn_tickets;
  p.argmax_key = c->argmax_key;
  p.phase_done = c->phase_done;
  p.status = c->status;
  p.moe_ne = c->moe_ne;
  p.moe_elist = c->moe_elist;
  p.moe_ne_sum = c->moe_ne_sum;
  p.moe_w = c->moe_w;
  p.ximg = c->ximg;
  p.eimg = c->eimg;
  p.aimg = c->aimg;
  p.simg = c->simg;
  p.img_done = c->img_done;
  // (measured choices: the pre-pass pays from 32 padded sequences on and, in the LM head, when a CTA walks the k-blocks at
  // least twice; O-proj / down-proj read the images their producers left)
  p.pre_bpad = 32;
  p.pre_lm_units = 2 * (d.hidden_size / kBlockK);
  p.dense_img = 1;
  const bool moe = d.arch == QMK_ARCH_MOE;
  p.E = moe ? d.num_experts : 0;
  p.topk = moe ? d.num_experts_per_tok : 0;
  p.Ie = moe ? d.moe_intermediate_size : 0;
  p.ppl = moe ? 6 : 5;
  p.trace = a->trace;
  p.epoch = ++c->epoch;
  p.ep_world = moe && d.ep_world > 1 ? d.ep_world : 1;
  p.ep_rank = p.ep_world > 1 ? d.ep_rank : 0;
  p.x_world = exchange_world(d);
  p.x_rank = exchange_rank(d);
  p.x_per_layer = d.tp_world > 1 ? 2 : 1;
  p.vocab_offset = d.tp_world > 1 ? d.tp_rank * d.vocab_size : 0;
  p.embed_rows = d.embed_rows > 0 ? d.embed_rows : d.vocab_size;
  if (p.x_world > 1) {
    if (!c->ep_connected) {
      if (err && errlen) snprintf(err, errlen, "model parallelism: qmk_ep_connect has not been called");
      return QMK_ERR_NOT_BOUND;
    }
    for (int r = 0; r < p.x_world; ++r) {
      unsigned char* base = (unsigned char*)c->ep_peer[r];
      p.ep_buf[r] = (float*)base;
      p.ep_flag[r] = (unsigned*)(base + c->ep_data_bytes);
      p.ep_key[r] = (unsigned long long*)(base + c->ep_data_bytes + c->ep_flag_bytes);
      p.ep_kflag[r] = (unsigned*)(base + c->ep_data_bytes + c->ep_flag_bytes + c->ep_key_bytes);
    }
  }
  p.H = d.hidden_size;
  p.I = d.intermediate_size;
  p.NH = d.num_attention_heads;
  p.NKV = d.num_key_value_heads;
  p.HD = d.head_dim;
  p.QKV_ROWS = (p.NH + 2 * p.NKV) * p.HD;
  p.QDIM = p.NH * p.HD;
  p.num_layers = d.num_layers;
  p.vocab = d.vocab_size;
  p.B = st->batch;
  p.Bpad = (st->batch + 15) / 16 * 16;
  const SmemPlan plan = smem_plan(p.Bpad);
  p.stages = plan.stages;
  p.stage_bytes = plan.stage_bytes;
  p.off_stages = plan.off_stages;
  p.exch_stride = plan.exch_stride;
  p.pos = a->pos;
  p.pos_limit = st->kv_seq_len < d.rope_rows ? st->kv_seq_len : d.rope_rows;
  p.phase_begin = a->phase_begin;
  p.phase_end = a->phase_end;
  p.wait_first = a->wait_first;
  p.eps = d.rms_norm_eps;
  p.qk_eps = d.qk_norm_eps > 0.f ? d.qk_norm_eps : d.rms_norm_eps;
  p.scale_log2e = d.attn_scale * 1.4426950408889634f;
  p.timeout_cycles = a->timeout_cycles;
  // The first phase of the launch, when it starts with an RMSNorm, needs the sums of squares of the residual
  // stream: computed by a prologue (with the embedding of token_in when the step starts at phase 0).
  if (a->phase_begin < a->phase_end) {
    const int k0 = phase_kind(p, a->phase_begin);
    if (phase_normed(k0))
      p.prologue = (a->phase_begin == 0 && st->token_in != nullptr) ? 2 : 1;
  }
  if (a->wait_first) p.prologue = 0;

  cudaError_t e = cudaMemsetAsync(c->zero_begin, 0, c->zero_bytes, stream);
  if (e != cudaSuccess) return fail(err, errlen, "cudaMemsetAsync", e);
  if (c->img_batch != st->batch) {   // the images' layout follows the padded batch, and rows from B up must read as zero
    e = cudaMemsetAsync(c->ximg, 0, c->img_bytes, stream);
    if (e != cudaSuccess) return fail(err, errlen, "cudaMemsetAsync", e);
    c->img_batch = st->batch;
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((unsigned)c->n_sm);
  cfg.blockDim = dim3(kBatchThreads);
  cfg.dynamicSmemBytes = (size_t)plan.total;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;   // all CTAs co-resident: they wait on one another
  attr[0].val.cooperative = a->cooperative;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  // (the kernel without the timeline's code unless a trace buffer is attached)
  e = p.trace != nullptr ? cudaLaunchKernelEx(&cfg, traced::qmk_batch_kernel, p, c->maps)
                         : cudaLaunchKernelEx(&cfg, plain::qmk_batch_kernel, p, c->maps);
  if (e != cudaSuccess) return fail(err, errlen, "cudaLaunchKernelEx(qmk_batch_kernel)", e);
  return QMK_OK;
}
