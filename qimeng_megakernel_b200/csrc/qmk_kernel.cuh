// Core of the persistent decode megakernel for sm_100a: one CTA per SM, eight identical worker warps.
//
//  * Weight stream.  Every warp owns a private ring of 4-KiB shared-memory slots.  Lane 0 streams
//    the warp's weight chunks into it with cp.async.bulk (TMA engine, mbarrier byte completion); the
//    stream is one static sequence that runs across phase and layer boundaries, so the next phases'
//    weights are in flight while the warp waits for activations.
//  * Hand-off between phases without fences or counters.  Every activation word that crosses SMs is
//    written as ONE 32-bit store {bf16 value, 16-bit tag of (step, phase)}.  A consumer polls the
//    data itself until every word carries the expected tag (the idea of NCCL's LL protocol).  The
//    eight warps of a CTA each fetch one eighth of the vector ("cooperative staging"), drop it in
//    shared memory, raise a per-warp flag and then wait for the other seven.
//  * The residual stream never goes through memory on the critical path: the warp that owns row r
//    in the O-projection owns it in the down-projection and in every later layer, so hidden[r]
//    stays in a register of that warp.
//
// What each phase computes follows the reference's fused PyTorch ops, including their bf16
// rounding points (qimeng_megakernel/models/LLM/llama/llama3_2__1b/A100/single_batch/
// decode_schedule/fused/operations.py:126-321); the CUDA phases they correspond to in the
// reference are decode_kernel/{rms_qkv_gemv_rope,decode_attention_splitkv,decode_attention_reduction,
// oproj_gemv_residual,rms_upgate_gemv_silu,down_proj_gemv_residual,rms_lm_head}.cu, whose
// cross-SM protocol is counters + acquire spins (decode_kernel/utils.cuh:266-328).
#pragma once
#include "qmk_device.cuh"
#include "qmk_params.h"
#include "qmk_schedule.h"

namespace qmk {

#ifndef QMK_WORKERS
#define QMK_WORKERS 8
#endif
#ifndef QMK_SLOTS
#define QMK_SLOTS 6
#endif
constexpr int kWorkers = QMK_WORKERS;  // warps per CTA (all of them stream weights)
constexpr int kSlots = QMK_SLOTS;      // ring slots per warp
constexpr int kThreads = kWorkers * 32;
constexpr unsigned kAbortFlag = 0xffffffffu;
static_assert(kWorkers <= 8, "the staging flags are polled by lanes 0..7");

template <class S>
struct SmemLayout {
  static constexpr int kRingBytes = kWorkers * kSlots * kChunkBytes;
  static constexpr int kActSmall = S::H * 2;                                  // bf16 activation vector
  static constexpr int kActBigA = S::I * 2;                                   // silu_out (bf16)
  static constexpr int kActBigB = S::QDIM * 4 + 2 * S::NKV * S::HD * 2;       // q fp32 + new K/V rows bf16
  static constexpr int kActBig = kActBigA > kActBigB ? kActBigA : kActBigB;
  static constexpr int kOffRing = 0;
  static constexpr int kOffActA = kOffRing + kRingBytes;
  static constexpr int kOffActB = kOffActA + kActSmall;
  static constexpr int kOffActD = kOffActB + kActSmall;
  static constexpr int kOffBars = kOffActD + kActBig;                // kWorkers*kSlots u64
  static constexpr int kOffCtl = kOffBars + kWorkers * kSlots * 8;   // control words (128 B)
  static constexpr int kOffRope = kOffCtl + 128;                     // cos[HD], sin[HD] of this step's position
  static constexpr int kTotal = kOffRope + S::HD * 8;
};
// control block, 32-bit words from kOffCtl:
//   [0..7]   part_done[w]: last phase (+1) whose staging part warp w has written; kAbortFlag = abort
//   [8]      lm_arrive     [10..11] CTA arg-max key (u64)
//   [16..23] sum-of-squares partials, buffer A     [24..31] buffer B
constexpr int kCtlLmArrive = 8, kCtlKey = 10, kCtlSumSq = 16;

__device__ __noinline__ void report_error(const Params& p, int code, int warp, int phase, unsigned seen,
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

// Optional timeline: slot of (CTA, phase).  Warp 0 writes: 2 enters the phase (globaltimer ns),
// 5 leaves it (ns); cycles spent 3 polling its staging part, 4 waiting for the other warps' parts,
// 6 in the streaming loop + epilogue, 7 in the whole phase.
__device__ __forceinline__ void trace_put(const Params& p, int ph, int slot, unsigned long long v, int lane) {
  if (p.trace != nullptr && lane == 0) p.trace[((size_t)blockIdx.x * num_phases(p.num_layers) + ph) * 8 + slot] = v;
}

// Tag of (step, phase): 1..65535, consecutive phases get consecutive tags, so a stale word (written
// at most one step earlier) can never carry the tag a reader waits for.  0 = never written.
__device__ __forceinline__ unsigned phase_tag(const Params& p, int ph) {
  return (p.epoch * (unsigned)num_phases(p.num_layers) + (unsigned)ph) % 65535u + 1u;
}

// ------------------------------------------------------------------------------------------
// Worker state: ring + issue cursor.  All fields are warp-uniform except `res`.
// ------------------------------------------------------------------------------------------
template <class S>
struct Worker {
  int lane, w, g, nwt;
  uint32_t ring;       // shared address of this warp's first slot
  uint32_t bars;       // shared address of this warp's first mbarrier
  uint32_t ctl;        // shared address of the control words
  unsigned n_issued, n_acquired;
  unsigned i_slot;         // slot the next issue goes into
  unsigned c_slot, c_par;  // slot and mbarrier parity of the next chunk to consume
  int i_ph, i_kind, i_layer, i_c, i_cend;   // issue cursor: phase, its kind / layer, next chunk, end chunk
  // This worker's chunk range per streaming kind: identical for every layer, so the 32-bit
  // divisions of the even split are done once per launch.
  int q0, q1, o0, o1, u0, u1, d0, d1, l0, l1;
  float res;               // residual stream value of row (first row of this warp + lane), bf16-exact
  bool res_valid;
  bool aborted;
  uint64_t policy;
  WeightBases wb;
};

__device__ __forceinline__ void split_range_u32(unsigned units, unsigned parts, unsigned g, int& lo, int& hi) {
  lo = (int)((g * units) / parts);            // (g + 1) * units < 2^32 is checked on the host
  hi = (int)(((g + 1u) * units) / parts);
}

template <class S>
__device__ __forceinline__ void init_ranges(Worker<S>& s, const Params& p) {
  int a, b;
  split_range_u32(S::QKV_ROWS / 2, s.nwt, s.g, a, b); s.q0 = 2 * a; s.q1 = 2 * b;
  split_range_u32(S::H, s.nwt, s.g, a, b); s.o0 = a * (S::QDIM / kChunkElems); s.o1 = b * (S::QDIM / kChunkElems);
  split_range_u32(S::I, s.nwt, s.g, a, b); s.u0 = 2 * a; s.u1 = 2 * b;
  split_range_u32(S::H, s.nwt, s.g, a, b); s.d0 = a * (S::I / kChunkElems); s.d1 = b * (S::I / kChunkElems);
  split_range_u32((unsigned)p.vocab, s.nwt, s.g, a, b); s.l0 = a; s.l1 = b;
}

template <class S>
__device__ __forceinline__ void kind_range(const Worker<S>& s, int kind, int& c0, int& c1) {
  switch (kind) {
    case kQkv: c0 = s.q0; c1 = s.q1; break;
    case kOproj: c0 = s.o0; c1 = s.o1; break;
    case kUpGate: c0 = s.u0; c1 = s.u1; break;
    case kDown: c0 = s.d0; c1 = s.d1; break;
    case kLmHead: c0 = s.l0; c1 = s.l1; break;
    default: c0 = c1 = 0; break;
  }
}

// Down-projection rows are consumed two at a time, k-slice by k-slice, so that both chunks of a pair
// meet the same activations: order (row a, slice 0), (row b, slice 0), (row a, slice 1), ...; an odd
// last row goes alone.  Maps the t-th chunk of this worker's down-proj stream to row * slices + slice.
template <class S>
__device__ __forceinline__ int down_canonical(int t, int d0, int d1) {
  constexpr int kSlices = S::I / kChunkElems;
  const int r0 = d0 / kSlices, nrows = (d1 - d0) / kSlices;
  const int pair = t / (2 * kSlices), tt = t % (2 * kSlices);
  int row = 2 * pair, slice;
  if (row + 1 < nrows) {
    slice = tt >> 1;
    row += tt & 1;
  } else {
    slice = tt;
  }
  return (r0 + row) * kSlices + slice;
}

// Position the issue cursor on the first phase >= i_ph in which this worker streams weights.
template <class S>
__device__ __forceinline__ void cursor_seek(Worker<S>& s, const Params& p) {
  while (s.i_ph < p.phase_end) {
    const int layer = s.i_ph / kPhasesPerLayer;
    s.i_kind = layer >= p.num_layers ? (int)kLmHead : s.i_ph - layer * kPhasesPerLayer;
    s.i_layer = layer;
    kind_range(s, s.i_kind, s.i_c, s.i_cend);
    if (s.i_c < s.i_cend) return;
    ++s.i_ph;
  }
}

// Issue the next chunk of the stream into the oldest free slot, if any chunk is left.
template <class S>
__device__ __forceinline__ void issue_one(Worker<S>& s, const Params& p) {
  if (s.aborted || s.i_ph >= p.phase_end) return;
  if (s.lane == 0) {
    const int c = s.i_kind == kDown ? down_canonical<S>(s.i_c - s.d0, s.d0, s.d1) : s.i_c;
    const uint16_t* src = chunk_ptr<S>(s.wb, s.i_kind, s.i_layer, c);
    const uint32_t bar = s.bars + s.i_slot * 8;
    mbar_expect_tx(bar, kChunkBytes);
    bulk_g2s(s.ring + s.i_slot * kChunkBytes, src, kChunkBytes, bar, s.policy);
  }
  ++s.n_issued;
  s.i_slot = (s.i_slot + 1 == kSlots) ? 0u : s.i_slot + 1;
  if (++s.i_c == s.i_cend) {
    ++s.i_ph;
    cursor_seek(s, p);
  }
}

// Bounded wait on one ring slot.  Returns false (and flags the error) on expiry.  The spin with its
// deadline is a separate, non-inlined function: it runs only when the data is not there yet.
__device__ __noinline__ bool wait_slot_slow(const Params& p, uint32_t bar, uint32_t parity, int warp, int phase,
                                            unsigned acquired, unsigned issued, int slot, int lane) {
  const long long t0 = clock64();
  for (unsigned it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 255u) == 0u && clock64() - t0 > p.timeout_cycles) {
      if (lane == 0) report_error(p, kErrCopyWait, warp, phase, acquired, issued, slot);
      return false;
    }
  }
}

// Next chunk in consumption order: waits for it, advances the consume cursor and returns the slot's
// shared address.  The slot stays owned by the warp until release_chunks().
template <class S>
__device__ __forceinline__ uint32_t acquire_chunk(Worker<S>& s, const Params& p, int phase) {
  const unsigned slot = s.c_slot;
  if (!s.aborted) {
    const uint32_t bar = s.bars + slot * 8;
    if (!mbar_try_wait(bar, s.c_par) &&
        !wait_slot_slow(p, bar, s.c_par, s.w, phase, s.n_acquired, s.n_issued, (int)slot, s.lane))
      s.aborted = true;
    ++s.n_acquired;
    if (++s.c_slot == kSlots) {
      s.c_slot = 0;
      s.c_par ^= 1u;
    }
  }
  return s.ring + slot * kChunkBytes;
}
// All lanes are done reading the `n` oldest acquired slots: refill them with the next chunks.
template <class S>
__device__ __forceinline__ void release_chunks(Worker<S>& s, const Params& p, int n) {
  __syncwarp();
  for (int i = 0; i < n; ++i) issue_one(s, p);
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

// ------------------------------------------------------------------------------------------
// GEMV core.  One 4-KiB chunk is 2048 consecutive weights of one output row.  View it as 8
// "pseudo-rows": pseudo-row r holds the 16-byte pieces r, r+8, r+16, ... of the chunk (256 weights).
// The dot product of the chunk with its 2048 activations is the sum over r of
// (pseudo-row r) . (the same pieces of the activation vector), i.e. the diagonal of an 8x8 product.
// A warp computes that product on the tensor pipe for TWO chunks at once with mma.m16n8k16:
// A rows 0-7 = pseudo-rows of chunk 0, rows 8-15 = pseudo-rows of chunk 1, B column n = activation
// pieces of pseudo-row n, 16 k-steps of 16 weights.  Products of bf16 are exact in fp32 and the
// accumulation is fp32, so the arithmetic is the same as an fp32 FMA chain in a different order.
// Eight consecutive pseudo-rows of one piece index are 128 contiguous bytes: ldmatrix reads them
// without bank conflicts, and the B fragments are plain 32-bit words x32[32*i + lane].
// (tcgen05 tiles pay off only when the batch makes the projection a real matrix product.)
// ------------------------------------------------------------------------------------------
struct XFrag {
  uint32_t b[32];   // b[2t], b[2t+1]: B fragment of k-step t
};

__device__ __forceinline__ void load_xfrag(XFrag& xf, const unsigned char* act_bf16, int lane) {
  const uint32_t* v = reinterpret_cast<const uint32_t*>(act_bf16);
#pragma unroll
  for (int i = 0; i < 32; ++i) xf.b[i] = v[32 * i + lane];
}

// The same, applying RMSNorm on the way: y = bf16(g * bf16(x * rstd))  (_rms_norm, operations.py:126-131).
__device__ __forceinline__ void load_xfrag_normed(XFrag& xf, const unsigned char* act_bf16, const uint32_t (&gains)[32],
                                                  float rstd, int lane) {
  const uint32_t* v = reinterpret_cast<const uint32_t*>(act_bf16);
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const uint32_t x = v[32 * i + lane], g = gains[i];
    xf.b[i] = pack_bf16x2(bf_lo(g) * bf16_round(bf_lo(x) * rstd), bf_hi(g) * bf16_round(bf_hi(x) * rstd));
  }
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&a)[4], uint32_t saddr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3])
               : "r"(saddr));
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Accumulate the 16x8 product of two chunks (shared addresses slot0 / slot1) into cc.
__device__ __forceinline__ void mma_chunk_pair(float (&cc)[4], uint32_t slot0, uint32_t slot1, const XFrag& xf,
                                               int lane) {
  // ldmatrix row address of this lane: matrices 0/2 come from chunk 0, 1/3 from chunk 1;
  // matrices 2/3 are the second piece (k 8..15) of the k-step.
  const uint32_t addr = ((lane & 8) ? slot1 : slot0) + ((((lane >> 4) << 3) + (lane & 7)) << 4);
  float c[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) c[i][j] = 0.f;
#pragma unroll
  for (int t = 0; t < 16; ++t) {
    uint32_t a[4];
    ldmatrix_x4(a, addr + t * 256);
    mma_bf16_16816(c[t & 3], a, xf.b[2 * t], xf.b[2 * t + 1]);
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) cc[j] += (c[0][j] + c[1][j]) + (c[2][j] + c[3][j]);
}

// Diagonal of the accumulated product -> the two dot products, summed over the warp.
__device__ __forceinline__ void diag_reduce(const float (&cc)[4], int lane, float& s0, float& s1) {
  const int r = lane >> 2, q2 = (lane & 3) * 2;
  s0 = r == q2 ? cc[0] : (r == q2 + 1 ? cc[1] : 0.f);
  s1 = r == q2 ? cc[2] : (r == q2 + 1 ? cc[3] : 0.f);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    s0 += __shfl_xor_sync(kFullMask, s0, o);
    s1 += __shfl_xor_sync(kFullMask, s1, o);
  }
}

}  // namespace qmk

#include "qmk_staging.cuh"
#include "qmk_phases.cuh"
