// Static on-device schedule of the decode megakernel: phases, per-worker work ranges and the
// weight-chunk stream.  Everything here is pure integer arithmetic shared by host and device
// (the host uses it for validation and for the CPU simulation of the schedule in the tests).
//
// The reference builds per-SM instruction queues on the host for every request
// (qimeng_megakernel/models/LLM/llama/llama3_2__1b/A100/single_batch/decode_schedule/instructions/scheduler.py:164-361)
// and ships them as an int32 tensor.  Here every worker warp derives its own work from
// (phase, worker id) with the closed-form splits below, so nothing is built or uploaded.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define QMK_HD __host__ __device__ __forceinline__
#else
#define QMK_HD inline
#endif

namespace qmk {

// One weight chunk = 2048 contiguous bf16 = 4 KiB: the unit of every bulk copy and ring slot.
constexpr int kChunkElems = 2048;
constexpr int kChunkBytes = kChunkElems * 2;

enum PhaseKind : int { kQkv = 0, kAttn = 1, kOproj = 2, kUpGate = 3, kDown = 4, kLmHead = 5 };
constexpr int kPhasesPerLayer = 5;
constexpr int kCounterShards = 32;        // dependency counter shards per phase (one per controller lane)
constexpr int kCounterStrideWords = 32;   // each shard in its own 128-byte line
constexpr int kAttnBlockKeys = 32;        // keys per attention block (one per lane)
constexpr int kMaxSplits = 64;            // upper bound on split-KV partials per head

// Llama-3.2-1B family shape (decode_schedule/model_config.py:4-17).
struct ShapeLlama1B {
  static constexpr int H = 2048;     // hidden
  static constexpr int I = 8192;     // SwiGLU intermediate
  static constexpr int NH = 32;      // query heads
  static constexpr int NKV = 8;      // key/value heads
  static constexpr int HD = 64;      // head dim
  static constexpr int QKV_ROWS = (NH + 2 * NKV) * HD;
  static constexpr int QDIM = NH * HD;
  static constexpr int GQA = NH / NKV;
};

QMK_HD int phase_kind(int ph, int num_layers) {
  return ph >= num_layers * kPhasesPerLayer ? (int)kLmHead : ph % kPhasesPerLayer;
}
QMK_HD int phase_layer(int ph) { return ph / kPhasesPerLayer; }
QMK_HD int num_phases(int num_layers) { return num_layers * kPhasesPerLayer + 1; }

// Even contiguous split of `units` over `parts`: part g owns [lo, hi).
QMK_HD void split_range(int units, int parts, int g, int& lo, int& hi) {
  lo = (int)(((long long)g * units) / parts);
  hi = (int)(((long long)(g + 1) * units) / parts);
}

// Work units of a streaming phase for worker g of nwt: units are row pairs (QKV: RoPE pairs),
// rows (O-proj, down-proj, LM head) or up/gate row pairs (SwiGLU).
template <class S>
QMK_HD int phase_units(int kind, int vocab) {
  switch (kind) {
    case kQkv: return S::QKV_ROWS / 2;
    case kOproj: return S::H;
    case kUpGate: return S::I;
    case kDown: return S::H;
    case kLmHead: return vocab;
    default: return 0;
  }
}
template <class S>
QMK_HD int chunks_per_unit(int kind) {
  switch (kind) {
    case kQkv: return 2;
    case kOproj: return S::QDIM / kChunkElems;
    case kUpGate: return 2;
    case kDown: return S::I / kChunkElems;
    case kLmHead: return 1;
    default: return 0;
  }
}

// Chunk range [c0, c1) of worker g in a phase of this kind (empty for attention).
template <class S>
QMK_HD void phase_chunk_range(int kind, int vocab, int g, int nwt, int& c0, int& c1) {
  if (kind == kAttn) { c0 = c1 = 0; return; }
  int u0, u1;
  split_range(phase_units<S>(kind, vocab), nwt, g, u0, u1);
  const int cpu = chunks_per_unit<S>(kind);
  c0 = u0 * cpu;
  c1 = u1 * cpu;
}

struct WeightBases {
  const uint16_t* qkv;
  const uint16_t* o_proj;
  const uint16_t* up;
  const uint16_t* gate;
  const uint16_t* down;
  const uint16_t* lm_head;
};

// Address of chunk c of (kind, layer).  Chunk numbering follows consumption order inside a unit:
// QKV: chunk = row (rows 2u, 2u+1); SwiGLU: chunk 2u = up row u, 2u+1 = gate row u;
// down-proj: chunk = row * (I/2048) + k-slice; O-proj / LM head: chunk = row.
template <class S>
QMK_HD const uint16_t* chunk_ptr(const WeightBases& w, int kind, int layer, int c) {
  switch (kind) {
    case kQkv: return w.qkv + ((size_t)layer * S::QKV_ROWS + c) * S::H;
    case kOproj: return w.o_proj + (size_t)layer * S::H * S::QDIM + (size_t)c * kChunkElems;
    case kUpGate: return ((c & 1) ? w.gate : w.up) + ((size_t)layer * S::I + (c >> 1)) * S::H;
    case kDown: return w.down + (size_t)layer * S::H * S::I + (size_t)c * kChunkElems;
    default: return w.lm_head + (size_t)c * S::H;
  }
}

// Split-KV plan for KV length T (= pos+1): blocks of 32 keys, `bps` blocks per partial, P partials.
// The reference picks P = min(16, SMs / kv_heads) regardless of length
// (.../instructions/scheduler.py:85-94); here P follows the length so that short contexts
// skip the merge entirely (P = 1) and long ones keep each partial at a few blocks.
QMK_HD void attn_plan(int T, int& bps, int& P) {
  const int nblk = (T + kAttnBlockKeys - 1) / kAttnBlockKeys;
  bps = (nblk + kMaxSplits - 1) / kMaxSplits;
  if (bps < 1) bps = 1;
  P = (nblk + bps - 1) / bps;
  if (P < 1) P = 1;
}

// How many publishers of a phase land on counter shard `shard`.
// Streaming phases: every worker publishes once (shard = g % 32).
// Attention: one publish per (kv head) merge (shard = kv_head % 32).
QMK_HD unsigned shard_contrib(int n_publishers, int shard) {
  return n_publishers > shard ? (unsigned)((n_publishers - shard + kCounterShards - 1) / kCounterShards) : 0u;
}

}  // namespace qmk
