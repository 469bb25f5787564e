// Static on-device schedule of the decode megakernel: phases, per-worker work ranges and the
// weight-tile stream.  Everything here is pure integer / pointer arithmetic shared by host and device:
// the device uses it to drive its bulk copies, the host tests replay it on the CPU and check that the
// streams of all workers cover every weight byte exactly once, in the order the phases consume them.
//
// The reference builds per-SM instruction queues on the host for every request
// (qimeng_megakernel/models/LLM/llama/llama3_2__1b/A100/single_batch/decode_schedule/instructions/scheduler.py:164-361)
// and ships them as an int32 tensor.  Here every worker warp derives its own work from
// (phase, worker id) with the closed-form splits below, so nothing is built or uploaded.
#pragma once
#include <stddef.h>
#include <stdint.h>

#if defined(__CUDACC__)
#define QMK_HD __host__ __device__ __forceinline__
#else
#define QMK_HD inline
#endif

namespace qmk {

// One weight chunk = 2048 contiguous bf16 = 4 KiB = one row (or one k-slice of a row).
constexpr int kChunkElems = 2048;
constexpr int kChunkBytes = kChunkElems * 2;

enum PhaseKind : int { kQkv = 0, kAttn = 1, kOproj = 2, kUpGate = 3, kDown = 4, kLmHead = 5 };
constexpr int kPhasesPerLayer = 5;
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
  static constexpr bool kMulti = false;   // kernel instance for launches of one decode step
};
// The same shape, compiled for launches that run several decode steps (the token loop inside the kernel).  A separate
// instance because the kernel has no register to spare: the few extra values of the multi-step form cost the one-step
// form 2 % when compiled in.
struct ShapeLlama1BSteps : ShapeLlama1B {
  static constexpr bool kMulti = true;
};

QMK_HD int phase_kind(int ph, int num_layers) {
  return ph >= num_layers * kPhasesPerLayer ? (int)kLmHead : ph % kPhasesPerLayer;
}
QMK_HD int phase_layer(int ph) { return ph / kPhasesPerLayer; }
QMK_HD int num_phases(int num_layers) { return num_layers * kPhasesPerLayer + 1; }

// Even contiguous split of `units` over `parts`: part g owns [lo, hi).  32-bit arithmetic:
// (g + 1) * units must stay below 2^32 (checked by the host when a handle is created).
QMK_HD void split_range_u32(unsigned units, unsigned parts, unsigned g, int& lo, int& hi) {
  lo = (int)((g * units) / parts);
  hi = (int)(((g + 1u) * units) / parts);
}

// Split-KV plan for KV length T (= pos+1).  Blocks of 32 keys; a warp takes `bpw` consecutive blocks, the eight
// warps of a CTA one CTA-part of 8*bpw blocks of one kv head, merged inside the CTA through shared memory;
// Pc CTA-parts per kv head (<= kMaxCtaParts) are merged through global records by one merge unit per query head.
// The reference picks P = min(16, SMs / kv_heads) partials regardless of length
// (.../instructions/scheduler.py:85-94); here short contexts (T <= 256) have Pc = 1 and no second merge at all.
constexpr int kAttnWarps = 8;
constexpr int kMaxCtaParts = 8;
QMK_HD void attn_plan(int T, int& bpw, int& Pc) {
  const int nblk = (T + kAttnBlockKeys - 1) / kAttnBlockKeys;
  bpw = (nblk + kAttnWarps * kMaxCtaParts - 1) / (kAttnWarps * kMaxCtaParts);
  if (bpw < 1) bpw = 1;
  Pc = (nblk + kAttnWarps * bpw - 1) / (kAttnWarps * bpw);
  if (Pc < 1) Pc = 1;
}

// ------------------------------------------------------------------------------------------
// The weight stream of a worker is a sequence of TILES.  A tile is what one tensor-pipe product
// consumes: two 4-KiB chunks (or one, for an odd last row) that meet the same activations.  It
// occupies one 8-KiB ring slot and is fetched by one 8-KiB bulk copy when its two chunks are
// adjacent in memory, else by two 4-KiB copies:
//   QKV      rows (2u, 2u+1) of one RoPE pair                                          one copy
//   O-proj   rows (r, r+1)                                                              one copy
//   LM head  rows (r, r+1)                                                              one copy
//   up/gate  (up row u, gate row u)                                                     two copies
//   down     (row a, k-slice j), (row a+1, k-slice j), j = 0..I/2048-1 per row pair     two copies
// ------------------------------------------------------------------------------------------
struct StreamBases {
  const unsigned char* qkv;
  const unsigned char* o_proj;
  const unsigned char* up;
  const unsigned char* gate;
  const unsigned char* down;
  const unsigned char* lm_head;
};

struct Tile {
  const unsigned char* a;   // first chunk (or both, when bytes_a == 8192)
  const unsigned char* b;   // second chunk when it is not adjacent, else null
  uint32_t bytes_a;
};

template <class S>
struct TileCursor {
  // this worker's item ranges per streaming kind: identical for every layer, so the divisions of the
  // even split are done once per launch.
  int q0, q1;              // QKV units (RoPE pairs)
  int r0, r1;              // rows of the residual phases (O-proj and down-proj share the split)
  int u0, u1;              // SwiGLU units
  int l0, l1;              // LM head rows
  // position in the stream
  int ph, kind;            // phase being issued (in a launch of several steps: step * num_phases + phase) and its kind
  int left;                // tiles left in that phase
  int sub;                 // down-proj: k-slice of the next tile
  int rows_left;           // rows (O-proj / LM / down) still to be covered, to spot the odd last row
  const unsigned char* p0; // next source (first chunk)
  const unsigned char* p1; // up/gate: gate row

  QMK_HD void init(int g, int nwt, int vocab, int phase_begin) {
    split_range_u32(S::QKV_ROWS / 2, nwt, g, q0, q1);
    split_range_u32(S::H, nwt, g, r0, r1);
    split_range_u32(S::I, nwt, g, u0, u1);
    split_range_u32((unsigned)vocab, nwt, g, l0, l1);
    ph = phase_begin;
    kind = left = sub = rows_left = 0;
    p0 = p1 = nullptr;
  }

  // Number of tiles of this worker in a phase of kind k.
  QMK_HD int tiles(int k) const {
    switch (k) {
      case kQkv: return q1 - q0;
      case kOproj: return (r1 - r0 + 1) >> 1;
      case kUpGate: return u1 - u0;
      case kDown: return ((r1 - r0 + 1) >> 1) * (S::I / kChunkElems);
      case kLmHead: return (l1 - l0 + 1) >> 1;
      default: return 0;
    }
  }

  // Position on the first phase >= ph in which this worker streams weights; set its first sources.
  QMK_HD void seek(const StreamBases& w, int num_layers, int phase_end) {
    // (phase_end may lie beyond one step's phases: a launch of n whole steps streams phases [0, n * num_phases), the
    // same matrices again in every step)
    const int np = num_phases(num_layers);
    while (ph < phase_end) {
      int lp = ph;
      if constexpr (S::kMulti) lp = ph < np ? ph : ph % np;
      const int layer = lp / kPhasesPerLayer;
      const int k = layer >= num_layers ? (int)kLmHead : lp - layer * kPhasesPerLayer;
      const int n = tiles(k);
      if (n > 0) {
        kind = k;
        left = n;
        sub = 0;
        const size_t row_b = (size_t)kChunkBytes;
        switch (k) {
          case kQkv: p0 = w.qkv + ((size_t)layer * S::QKV_ROWS + 2 * (size_t)q0) * row_b; break;
          case kOproj:
            p0 = w.o_proj + ((size_t)layer * S::H + r0) * row_b;
            rows_left = r1 - r0;
            break;
          case kUpGate:
            p0 = w.up + ((size_t)layer * S::I + u0) * row_b;
            p1 = w.gate + ((size_t)layer * S::I + u0) * row_b;
            break;
          case kDown:
            p0 = w.down + ((size_t)layer * S::H + r0) * (size_t)S::I * 2;
            rows_left = r1 - r0;
            break;
          default:
            p0 = w.lm_head + (size_t)l0 * row_b;
            rows_left = l1 - l0;
            break;
        }
        return;
      }
      ++ph;
    }
  }

  QMK_HD bool done(int phase_end) const { return ph >= phase_end; }

  // The next tile of the stream; advances the cursor (and seeks the next phase when this one ends).
  QMK_HD Tile next(const StreamBases& w, int num_layers, int phase_end) {
    constexpr int kSlices = S::I / kChunkElems;
    Tile t;
    t.a = p0;
    t.b = nullptr;
    t.bytes_a = 2 * kChunkBytes;
    switch (kind) {
      case kQkv:
        p0 += 2 * kChunkBytes;
        break;
      case kUpGate:
        t.bytes_a = kChunkBytes;
        t.b = p1;
        p0 += kChunkBytes;
        p1 += kChunkBytes;
        break;
      case kDown:
        t.bytes_a = kChunkBytes;
        t.a += (size_t)sub * kChunkBytes;
        if (rows_left > 1) t.b = t.a + (size_t)S::I * 2;
        if (++sub == kSlices) {
          sub = 0;
          p0 += 2 * (size_t)S::I * 2;
          rows_left -= 2;
        }
        break;
      default:   // O-proj, LM head
        if (rows_left < 2) t.bytes_a = kChunkBytes;
        rows_left -= 2;
        p0 += 2 * kChunkBytes;
        break;
    }
    if (--left == 0) {
      ++ph;
      seek(w, num_layers, phase_end);
    }
    return t;
  }
};

}  // namespace qmk
