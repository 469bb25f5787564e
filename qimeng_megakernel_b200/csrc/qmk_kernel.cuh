// The persistent decode megakernel for sm_100a: one CTA per SM, eight independent worker warps
// plus one controller warp per CTA.
//
//  * Worker warps own a private ring of 4-KiB shared-memory slots.  Lane 0 streams the warp's
//    weight chunks into the ring with cp.async.bulk (TMA engine, mbarrier byte completion); the
//    stream is one static sequence that runs across phase and layer boundaries, so the next
//    phase's weights are already in flight while the warp waits for its activations.
//  * The controller warp of each CTA waits for the previous phase's dependency counters (32
//    shards, one per lane, ld.acquire.gpu), stages the phase's activation vector into shared
//    memory (fusing RMSNorm where the phase starts with one) and releases the workers through a
//    shared-memory flag.
//  * Workers publish a phase with one red.release.gpu per warp on a sharded counter.  Counters are
//    never reset: the target of step n is (n+1) * publishers.
//
// What each phase computes follows the reference's fused PyTorch ops, including their bf16
// rounding points (qimeng_megakernel/models/LLM/llama/llama3_2__1b/A100/single_batch/
// decode_schedule/fused/operations.py:126-321); the CUDA phases they correspond to in the
// reference are decode_kernel/{rms_qkv_gemv_rope,decode_attention_splitkv,decode_attention_reduction,
// oproj_gemv_residual,rms_upgate_gemv_silu,down_proj_gemv_residual,rms_lm_head}.cu.
#pragma once
#include "qmk_device.cuh"
#include "qmk_params.h"
#include "qmk_schedule.h"

namespace qmk {

constexpr int kWorkers = 8;            // worker warps per CTA
constexpr int kSlots = 6;              // ring slots per worker warp
constexpr int kThreads = (kWorkers + 1) * 32;
constexpr unsigned kAbortFlag = 0xffffffffu;

template <class S>
struct SmemLayout {
  static constexpr int kRingBytes = kWorkers * kSlots * kChunkBytes;
  static constexpr int kActSmall = S::H * 2;                        // bf16 activation vector
  static constexpr int kActBigA = S::I * 2;                         // silu_out (bf16)
  static constexpr int kActBigB = S::QDIM * 4;                      // q in fp32 for attention
  static constexpr int kActBig = kActBigA > kActBigB ? kActBigA : kActBigB;
  static constexpr int kOffRing = 0;
  static constexpr int kOffActA = kOffRing + kRingBytes;
  static constexpr int kOffActB = kOffActA + kActSmall;
  static constexpr int kOffActD = kOffActB + kActSmall;
  static constexpr int kOffBars = kOffActD + kActBig;                // kWorkers*kSlots u64
  static constexpr int kOffCtl = kOffBars + kWorkers * kSlots * 8;   // control words
  static constexpr int kTotal = kOffCtl + 64;
};
// control words (u32 index from kOffCtl): 0 staged, 1 lm_arrive, 2..3 cta argmax key (u64)

__device__ __forceinline__ void report_error(const Params& p, int code, int warp, int phase, unsigned seen,
                                             unsigned expected, int detail) {
  if (atomicCAS(&p.status[kStCode], 0u, (unsigned)code) == 0u) {
    p.status[kStSm] = blockIdx.x;
    p.status[kStWarp] = warp;
    p.status[kStPhase] = phase;
    p.status[kStSeen] = seen;
    p.status[kStExpected] = expected;
    p.status[kStDetail] = detail;
    __threadfence();
  }
}

// ------------------------------------------------------------------------------------------
// Worker state: ring + issue cursor.  All fields are warp-uniform.
// ------------------------------------------------------------------------------------------
template <class S>
struct Worker {
  int lane, w, g, nwt;
  uint32_t ring;       // shared address of this warp's first slot
  uint32_t bars;       // shared address of this warp's first mbarrier
  uint32_t ctl;        // shared address of the control words
  unsigned n_issued, n_consumed;
  int i_ph, i_c, i_cend;   // issue cursor: phase, next chunk, end chunk
  int staged_seen;         // highest staged value observed
  bool aborted;
  uint64_t policy;
  WeightBases wb;
};

template <class S>
__device__ __forceinline__ void cursor_seek(Worker<S>& s, const Params& p) {
  while (s.i_ph < p.phase_end) {
    const int kind = phase_kind(s.i_ph, p.num_layers);
    int c0, c1;
    phase_chunk_range<S>(kind, p.vocab, s.g, s.nwt, c0, c1);
    if (c0 < c1) {
      s.i_c = c0;
      s.i_cend = c1;
      return;
    }
    ++s.i_ph;
  }
}

// Issue the next chunk of the stream into slot (n_issued % kSlots), if any is left.
template <class S>
__device__ __forceinline__ void issue_one(Worker<S>& s, const Params& p) {
  if (s.aborted || s.i_ph >= p.phase_end) return;
  const int kind = phase_kind(s.i_ph, p.num_layers);
  const uint16_t* src = chunk_ptr<S>(s.wb, kind, phase_layer(s.i_ph), s.i_c);
  const unsigned slot = s.n_issued % kSlots;
  if (s.lane == 0) {
    const uint32_t bar = s.bars + slot * 8;
    mbar_expect_tx(bar, kChunkBytes);
    bulk_g2s(s.ring + slot * kChunkBytes, src, kChunkBytes, bar, s.policy);
  }
  ++s.n_issued;
  if (++s.i_c == s.i_cend) {
    ++s.i_ph;
    cursor_seek(s, p);
  }
}

// Bounded wait for chunk n of this warp's stream.  Returns false (and flags the error) on expiry.
template <class S>
__device__ __forceinline__ bool wait_chunk(Worker<S>& s, const Params& p, unsigned n, int phase) {
  const uint32_t bar = s.bars + (n % kSlots) * 8;
  const uint32_t parity = (n / kSlots) & 1u;
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (unsigned it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 255u) == 0u && clock64() - t0 > p.timeout_cycles) {
      if (s.lane == 0) report_error(p, kErrCopyWait, s.w, phase, n, s.n_issued, (int)(n % kSlots));
      return false;
    }
  }
}

// Next chunk in consumption order: returns the slot's generic shared pointer (as uint4*).
template <class S>
__device__ __forceinline__ const uint4* acquire_chunk(Worker<S>& s, const Params& p, unsigned char* smem,
                                                      int phase) {
  if (!s.aborted && !wait_chunk(s, p, s.n_consumed, phase)) s.aborted = true;
  const unsigned slot = s.n_consumed % kSlots;
  return reinterpret_cast<const uint4*>(smem + SmemLayout<S>::kOffRing +
                                        (s.w * kSlots + slot) * kChunkBytes);
}
// All lanes are done reading the slot: hand it back to the copy engine with the next chunk.
template <class S>
__device__ __forceinline__ void release_chunk(Worker<S>& s, const Params& p) {
  __syncwarp();
  if (s.aborted) return;
  ++s.n_consumed;
  issue_one(s, p);
}

// Wait until the controller has staged the activations of `phase` (staged >= phase+1).
template <class S>
__device__ __forceinline__ bool wait_staged(Worker<S>& s, const Params& p, int phase) {
  if (s.aborted) return false;
  if (s.staged_seen > phase && s.staged_seen != (int)kAbortFlag) return true;
  unsigned v = 0;
  if (s.lane == 0) {
    const long long t0 = clock64();
    for (unsigned it = 0;; ++it) {
      v = ld_acquire_cta_shared(s.ctl);
      if (v == kAbortFlag || v >= (unsigned)(phase + 1)) break;
      if ((it & 1023u) == 1023u && clock64() - t0 > 4 * p.timeout_cycles) {   // outlasts the controller's own wait
        report_error(p, kErrStageWait, s.w, phase, v, (unsigned)(phase + 1), 0);
        v = kAbortFlag;
        break;
      }
    }
  }
  v = __shfl_sync(kFullMask, v, 0);
  if (v == kAbortFlag) {
    s.aborted = true;
    return false;
  }
  s.staged_seen = (int)v;
  return true;
}

// Publish this warp's share of `phase` (all of its global stores precede the release).
template <class S>
__device__ __forceinline__ void publish(const Worker<S>& s, const Params& p, int phase, int shard) {
  __syncwarp();
  if (p.sync && !s.aborted && s.lane == 0) {
    __threadfence();
    red_release_gpu_add(p.counters + ((size_t)phase * kCounterShards + shard) * kCounterStrideWords, 1u);
  }
}

// Which small activation buffer (A or B) a phase uses: they alternate along the phase sequence.
__device__ __forceinline__ int small_buf_index(int phase, int num_layers) {
  const int kind = phase_kind(phase, num_layers);
  const int l = phase_layer(phase);
  int idx;
  if (kind == kLmHead) idx = num_layers * 3;
  else idx = l * 3 + (kind == kQkv ? 0 : (kind == kOproj ? 1 : 2));
  return idx & 1;
}

// Load this lane's 64 activation values of a 2048-element bf16 vector staged in shared memory:
// element k = j*256 + lane*8 + e  ->  x[j*8 + e]  (the same positions the lane reads in a weight chunk).
__device__ __forceinline__ void load_x64(float (&x)[64], const unsigned char* act, int lane) {
  const uint4* v = reinterpret_cast<const uint4*>(act);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint4 q = v[j * 32 + lane];
    x[j * 8 + 0] = bf_lo(q.x); x[j * 8 + 1] = bf_hi(q.x);
    x[j * 8 + 2] = bf_lo(q.y); x[j * 8 + 3] = bf_hi(q.y);
    x[j * 8 + 4] = bf_lo(q.z); x[j * 8 + 5] = bf_hi(q.z);
    x[j * 8 + 6] = bf_lo(q.w); x[j * 8 + 7] = bf_hi(q.w);
  }
}

// Per-lane partial dot product of one 4-KiB weight chunk with the lane's 64 activations.
__device__ __forceinline__ float dot_chunk(const uint4* slot, const float (&x)[64], int lane) {
  float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f, a4 = 0.f, a5 = 0.f, a6 = 0.f, a7 = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint4 q = slot[j * 32 + lane];
    a0 = fmaf(bf_lo(q.x), x[j * 8 + 0], a0);
    a1 = fmaf(bf_hi(q.x), x[j * 8 + 1], a1);
    a2 = fmaf(bf_lo(q.y), x[j * 8 + 2], a2);
    a3 = fmaf(bf_hi(q.y), x[j * 8 + 3], a3);
    a4 = fmaf(bf_lo(q.z), x[j * 8 + 4], a4);
    a5 = fmaf(bf_hi(q.z), x[j * 8 + 5], a5);
    a6 = fmaf(bf_lo(q.w), x[j * 8 + 6], a6);
    a7 = fmaf(bf_hi(q.w), x[j * 8 + 7], a7);
  }
  return ((a0 + a1) + (a2 + a3)) + ((a4 + a5) + (a6 + a7));
}

}  // namespace qmk

#include "qmk_phases.cuh"
