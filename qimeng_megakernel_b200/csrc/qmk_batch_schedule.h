// Static schedule of the batched decode kernel: pure integer arithmetic shared by every role of the device
// code and by the host tests, which replay it on the CPU.
//
// The reference deals 16-row output blocks to SMs on the host for every request and ships the result as an
// instruction tensor (qimeng_megakernel/models/LLM/llama/llama3_2__1b/A100/single_batch/decode_schedule/
// instructions/scheduler.py:138-152, 164-361).  Here a phase is cut into (row tile, k-block) units and every
// CTA derives its contiguous unit range in closed form.
#pragma once
#include "qmk_batch_params.h"

#if defined(__CUDACC__)
#define QMKB_HD __host__ __device__ __forceinline__
#else
#define QMKB_HD inline
#endif

namespace qmkb {

struct PhaseDims {
  int N;        // output rows (SwiGLU: units)
  int K;        // contraction length
  int T;        // row tiles
  int KB;       // k-blocks
  int rows;     // output rows (units) per tile
};
QMKB_HD int phase_kind(const BParams& p, int ph) {
  if (ph >= p.ppl * p.num_layers) return (int)kLmHead;
  const int i = ph % p.ppl;
  if (p.ppl == 6 && i >= 3) return i == 3 ? (int)kRouter : (i == 4 ? (int)kEUpGate : (int)kEDown);
  return i;
}
QMKB_HD int phase_layer(const BParams& p, int ph) { return ph >= p.ppl * p.num_layers ? 0 : ph / p.ppl; }
QMKB_HD int num_phases(const BParams& p) { return p.ppl * p.num_layers + 1; }
QMKB_HD bool phase_normed(int kind) {
  return kind == kQkv || kind == kUpGate || kind == kLmHead || kind == kRouter || kind == kEUpGate;
}
// ne: number of distinct experts selected in this step (expert phases only; known once the layer's router is done)
QMKB_HD PhaseDims phase_dims(const BParams& p, int kind, int ne = 0) {
  PhaseDims d;
  switch (kind) {
    case kQkv: d.N = p.QKV_ROWS; d.K = p.H; d.rows = kTileRows; break;
    case kOproj: d.N = p.H; d.K = p.QDIM; d.rows = kTileRows; break;
    case kUpGate: d.N = p.I; d.K = p.H; d.rows = kTileRows / 2; break;   // 64 up rows + the 64 gate rows of the same units
    case kDown: d.N = p.H; d.K = p.I; d.rows = kTileRows; break;
    case kRouter: d.N = p.E; d.K = p.H; d.rows = kTileRows; break;       // one tile (E <= 128)
    case kEUpGate: d.N = ne * p.Ie; d.K = p.H; d.rows = kTileRows / 2; break;   // 64 gate rows + 64 up rows of one expert
    case kEDown: d.N = p.H; d.K = ne * p.Ie; d.rows = kTileRows; break;  // one GEMM over the k-blocks of all selected experts
    default: d.N = p.vocab; d.K = p.H; d.rows = kTileRows; break;
  }
  d.T = (d.N + d.rows - 1) / d.rows;
  d.KB = d.K / kBlockK;
  return d;
}
// CTAs that share a phase's units: all of them; the router's single tile has only K / 64 units and gives one to each of
// as many CTAs (measured: 37 us per router phase with eight units on each of four CTAs, whose stagers then pay a round
// trip per pair of units; one unit per CTA is 2-3 % of the whole mixture-of-experts step faster, the 32 partial tiles
// meeting in the tile's fixed-point accumulator).
QMKB_HD int phase_ctas(int kind, int U, int G) {
  if (kind != kRouter) return G;
  return U < 1 ? 1 : (U < G ? U : G);
}

// Units [lo, hi) of CTA c out of G, for U units (none for c >= G).
QMKB_HD void unit_range(int U, int G, int c, int& lo, int& hi) {
  if (c >= G) { lo = hi = 0; return; }
  lo = (int)(((long long)c * U) / G);
  hi = (int)(((long long)(c + 1) * U) / G);
}
// The CTA that owns unit u.
QMKB_HD int unit_owner(int U, int G, int u) { return (int)((((long long)u + 1) * G - 1) / U); }

// Number of segments (= CTAs with units) of row tile t.  With fewer units than CTAs every CTA owns at most one
// unit and the owners of consecutive units are not consecutive CTAs: then a tile has KB one-unit segments.
QMKB_HD int tile_segments(int U, int G, int KB, int t) {
  if (U < G) return KB;
  return unit_owner(U, G, (t + 1) * KB - 1) - unit_owner(U, G, t * KB) + 1;
}

// Split-KV plan: keys per item `ck` (a multiple of 32) and items per (sequence, kv head) `nch`, for the longest
// context Tmax, `seqs` = sequences x kv heads and NW attention warps: enough items to occupy every warp, at most
// kMaxSplits per (sequence, kv head); seqs * nch <= NW + seqs.  The reference picks min(16, SMs / kv_heads)
// partials whatever the length (.../instructions/scheduler.py:85-94).
QMKB_HD void attn_plan(int Tmax, int seqs, int NW, int& ck, int& nch) {
  ck = (int)(((long long)Tmax * seqs + NW - 1) / NW);
  const int floor_ck = (Tmax + kMaxSplits - 1) / kMaxSplits;
  if (ck < floor_ck) ck = floor_ck;
  ck = (ck + 31) & ~31;
  if (ck < 32) ck = 32;
  nch = (Tmax + ck - 1) / ck;
}

}  // namespace qmkb
