// Batched decode megakernel for sm_100a: B sequences per step, runtime model shape.
//
// One persistent CTA per SM, ten warps with fixed roles:
//   warp 0      producer   one lane streams the CTA's weight tiles (TMA tensor copies, 128-byte swizzle)
//   warp 1      issuer     one lane issues tcgen05.mma (M = 128 weight rows, N = padded batch, K = 16)
//   warps 2-5   epilogue   read accumulators from tensor memory, finish the phase's arithmetic
//   warps 6-9   stagers    build the activation operand ([batch, 64] bf16, RMSNorm applied) in shared memory
// In the attention phase warps 2-9 are eight attention workers: one (sequence, kv head, key range) item per warp, scores
// and P.V on the tensor pipe with warp-level mma.sync (the query heads of the kv head are the rows of a 16 x 8 tile).
//
// Every projection is a stream-K GEMM  out[b, n] = sum_k X[b, k] * W[n, k]:  the (row tile, k-block)
// units of a phase, 128 x 64 weights = 16 KiB each, are dealt to the CTAs as equal contiguous ranges,
// so every SM streams the same number of bytes whatever the matrix shape.  A maximal run of units of
// one row tile is a SEGMENT, accumulated in tensor memory.  A segment that covers the whole K is
// finished by its CTA.  A tile that is split over several CTAs is finished by the CTA that owns its first
// unit (its range ends inside the tile, so it gets there last): the others add their partial tiles to the
// tile's fixed-point accumulator at L2 (64-bit integer reductions, nothing returned) and count themselves
// in with one release; the owner waits for the count, takes the sum out and adds its own part in the same
// fixed point, so the result does not depend on the order of arrival and a step gives the same bits every
// time.  The reference splits K in the
// down-projection only and adds the partials with bf16 compare-and-swap in arrival order
// (qimeng_megakernel/models/LLM/llama/llama3_2__1b/A100/single_batch/decode_kernel/down_proj_gemv_residual.cu:39-52).
//
// Phases are separated by grid-wide arrival counters (one per phase, zeroed by the host before the
// launch); the weight stream runs ahead across them.  What each phase computes, rounding points
// included, follows the reference's fused PyTorch ops for [B, H] state
// (.../A100/single_batch/decode_schedule/fused/operations.py:126-321; per-row positions and the active
// mask as in decode_pos_id / row_active there; Qwen3's per-head Q/K RMSNorm:
// qimeng_megakernel/models/LLM/qwen/qwen3__0_6b/A100/single_batch/decode_schedule/fused/operations.py:52-120).
//
// Every wait is bounded.  A wait that expires records a status, raises the CTA's abort word; from then
// on every wait in the CTA returns at once, work is skipped, the barriers inside the CTA are still
// executed (trip counts do not depend on data), and all roles meet at the common exit where copies in
// flight are waited for and the tensor memory is freed.
#pragma once
#include <cuda.h>

#include "qmk_batch_params.h"
#include "qmk_batch_schedule.h"
#include "qmk_device.cuh"
#include "qmk_params.h"

namespace qmkb {

using namespace qmk;

constexpr int kStages = 8;                              // ring slots (a power of two: slot and parity of unit n are n & 7, (n >> 3) & 1;
                                                        // more slots were measured to change nothing)
constexpr int kMaxStages = kStages, kMinStages = kStages;
constexpr int kABytes = kTileRows * kBlockK * 2;        // 16 KiB of weights per unit
constexpr int kNumWarps = 10;
constexpr int kBatchThreads = kNumWarps * 32;
constexpr int kEpiWarp0 = 2, kStgWarp0 = 6;
constexpr int kBarEpi = 1, kBarStg = 2, kBarAttn = 3;   // named barriers (0 is __syncthreads)
constexpr int kTraceSlots = 16;                         // 64-bit words per (CTA, phase) of the optional timeline
constexpr int kSmemBudget = 227 * 1024;                 // dynamic shared memory a CTA may ask for on sm_100

// Shared memory: a fixed header, then the fp32 exchange tile [128][Bpad + 1], then the ring on a 1024-byte boundary
// (128-byte-swizzle atoms).  A ring slot holds 16 KiB of weights and Bpad * 128 bytes of activations, so small
// batches get more slots: more weight bytes in flight per SM.
struct Smem {
  static constexpr int kOffBars = 0;                                          // mbarriers
  //   full[kMaxStages] (unused)[kMaxStages] empty[kMaxStages / 2] ... acc_full[2] acc_empty[2]
  // A slot's `full` barrier collects both operands of a unit: the producer's arrive with the weight bytes expected, and
  // the 32 arrivals of the stager warp (after its stores, or with the bytes of its bulk copy expected).  `empty` is per
  // PAIR of slots: the issuer commits once per two units, and a slot is refilled when its pair has been consumed.
  static constexpr int kNumBars = 3 * kMaxStages + 4;
  static constexpr int kOffRs = kOffBars + kNumBars * 8;                      // float [64]  rsqrt factors
  static constexpr int kOffHs = kOffRs + kMaxBatch * 4;                       // float [2][64] scratch of the prologue
  static constexpr int kOffPos = kOffHs + 2 * kMaxBatch * 4;                  // int [64]
  static constexpr int kOffAct = kOffPos + kMaxBatch * 4;                     // int [64]
  static constexpr int kOffSlot = kOffAct + kMaxBatch * 4;                    // int [64]  KV-cache sequence of every row
  static constexpr int kOffCtl = kOffSlot + kMaxBatch * 4;                    // control words
  static constexpr int kOffExch = 2048;
  static_assert(kOffCtl + 64 <= kOffExch, "header overflows");
};
struct SmemPlan { int off_stages, stage_bytes, stages, exch_stride, total; };
__host__ __device__ inline SmemPlan smem_plan(int Bpad) {
  SmemPlan s;
  s.exch_stride = Bpad + 1;
  s.off_stages = (Smem::kOffExch + kTileRows * s.exch_stride * 4 + 1023) / 1024 * 1024;
  s.stage_bytes = kABytes + Bpad * kBlockK * 2;
  s.stages = kStages;
  s.total = s.off_stages + s.stages * s.stage_bytes;   // 227 KiB exactly at Bpad = 64; the base must be 1024-aligned
  return s;
}
// control words: [0] abort  [1] tensor-memory base  [2] Tmax  [3] flag of the epilogue group  [4] flag of the stagers
// [5] flag of the attention group  [7] / [8] number of selected experts as read by the stagers / the epilogue group
// [10..13] router epilogue: experts listed by each of its four warps
constexpr int kCAbort = 0, kCTmem = 1, kCTmax = 2, kCFlagEpi = 3, kCFlagStg = 4, kCFlagAttn = 5, kCNeStg = 7, kCNeEpi = 8,
              kCRouterCnt = 10;   // [10..13] listed experts per epilogue warp

struct TensorMaps {
  CUtensorMap qkv, o_proj, up, gate, down, lm_head;   // 3-D {k, row, layer}; box {64, 128 (up/gate: 64), 1}
  // MoE: router {H, E, L} box 128 rows; expert gate|up {H, 2 * Ie, L * E} box 64 rows; expert down {Ie, H, L * E} box 128
  CUtensorMap router, egu, edown;
};

namespace plain {
constexpr bool kTraceOn = false;
#include "qmk_batch_device.cuh"
}  // namespace plain

namespace traced {
constexpr bool kTraceOn = true;
#include "qmk_batch_device.cuh"
}  // namespace traced

}  // namespace qmkb
