// Core of the persistent decode megakernel for sm_100a: one CTA per SM, eight identical worker warps.
//
//  * Weight stream.  Every warp owns a private ring of 8-KiB shared-memory slots.  Lane 0 streams
//    the warp's weight tiles into it with cp.async.bulk (TMA engine, mbarrier byte completion); the
//    stream is one static sequence that runs across phase and layer boundaries, so the next phases'
//    weights are in flight while the warp waits for activations.
//  * Hand-off between phases without fences or counters.  Every activation word that crosses SMs is
//    written as ONE 32-bit store {bf16 value, 16-bit tag of (step, phase)}.  A consumer polls the
//    data itself until every word carries the expected tag (the idea of NCCL's LL protocol).  The
//    eight warps of a CTA each fetch one eighth of the vector ("cooperative staging"), drop it in
//    shared memory and meet at a CTA barrier.  A warp pushes its tagged stores out with a fence that
//    nothing waits for.
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

constexpr int kWorkers = 8;            // warps per CTA (all of them stream weights)
constexpr int kSlots = 2;              // ring slots (8 KiB tiles) per warp (a third slot made every hand-off slower)
constexpr int kThreads = kWorkers * 32;
constexpr unsigned kAbortFlag = 0xffffffffu;


template <class S>
struct SmemLayout {
  static constexpr int kRingBytes = kWorkers * kSlots * 2 * kChunkBytes;
  static constexpr int kActSmall = S::H * 2;                                  // bf16 activation vector
  static constexpr int kActBigA = S::I * 2;                                   // silu_out (bf16)
  static constexpr int kActBigB = S::QDIM * 4 + 2 * S::NKV * S::HD * 2;       // q fp32 + new K/V rows bf16
  static constexpr int kActBig = kActBigA > kActBigB ? kActBigA : kActBigB;
  // first attention block of every warp (K and V rows of 32 keys, 8 KiB), copied in ahead of the attention phase
  static constexpr bool kKvStage = true;
  static constexpr int kKvStageBytes = kWorkers * 16 * 512;
  static constexpr int kOffRing = 0;
  static constexpr int kOffKvStage = kOffRing + kRingBytes;
  static constexpr int kOffActA = kOffKvStage + kKvStageBytes;
  static constexpr int kOffActB = kOffActA + kActSmall;
  static constexpr int kOffActD = kOffActB + kActSmall;
  static constexpr int kOffBars = kOffActD + kActBig;                // kWorkers*kSlots u64
  static constexpr int kOffCtl = kOffBars + kWorkers * kSlots * 8;   // control words (128 B)
  static constexpr int kOffRope = kOffCtl + 128;                     // cos[HD], sin[HD] of this step's position
  static constexpr int kOffPos = kOffRope + S::HD * 8;               // position of the step the CTA is in (one int)
  static constexpr int kTotal = kOffPos + 16;
};
// control block, 32-bit words from kOffCtl:
//   [0] abort word (non-zero: a warp of this CTA gave up)   [8] lm_arrive   [10..11] CTA arg-max key (u64)
//   [16..23] sum-of-squares partials, buffer A     [24..31] buffer B
constexpr int kCtlAbort = 0, kCtlTmem = 4, kCtlLmArrive = 8, kCtlKey = 10, kCtlSumSq = 16;

static __device__ __noinline__ void report_error(const Params& p, int code, int warp, int phase, unsigned seen,
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

// Optional timeline (qmk_set_trace): eight 64-bit slots per (CTA, phase), written by warp 0 unless noted.
//   2 enters the phase, 5 leaves it (globaltimer ns); 3 cycles until its input was staged; 6 cycles from there to
//   the end of the phase.  Streaming phases: 1 / 0 latest / (inverted) earliest end of the streaming loop over the
//   CTA's warps (ns), 4 longest loop of a warp (cycles).  Attention, compute CTAs: 0 staged, 1 own partial done,
//   4 all partials in shared memory, 7 outputs pushed out (ns).  First phase of the launch: 3 (inverted) entry and
//   7 exit of the CTA (ns).
__device__ __forceinline__ void trace_put(const Params& p, int ph, int slot, unsigned long long v, int lane) {
  if (p.trace != nullptr && lane == 0) p.trace[((size_t)blockIdx.x * num_phases(p.num_layers) + ph) * 8 + slot] = v;
}

// Tag of (launch, phase): 1..65535, consecutive phases and launches get consecutive tags, so a stale
// word (every tagged word is rewritten by every full step) cannot carry the tag a reader waits for.
// 0 = never written.
// gph: the phase counted over the steps of the launch (step * num_phases + phase; launch_seq numbers the launch's first
// step, every step takes one number, so consecutive launches continue the same sequence).
__device__ __forceinline__ unsigned phase_tag(const Params& p, int gph) {
  return (p.launch_seq * (unsigned)num_phases(p.num_layers) + (unsigned)gph) % 65535u + 1u;
}

// ------------------------------------------------------------------------------------------
// Worker state: tile ring + issue cursor (qmk_schedule.h).  All fields are warp-uniform except `res`.
// ------------------------------------------------------------------------------------------
template <class S>
struct Worker {
  int lane, w, g, nwt;
  uint32_t ring;       // shared address of this warp's first slot
  uint32_t bars;       // shared address of this warp's first mbarrier
  uint32_t ctl;        // shared address of the control words
  unsigned n_issued, n_acquired;
  unsigned i_slot;         // slot the next issue goes into
  unsigned c_slot, c_par;  // slot and mbarrier parity of the next tile to consume
  TileCursor<S> cur;       // where the weight stream is; also holds this worker's item ranges
  uint32_t tmem;           // tensor-memory address of this warp's parking space (its lane quarter, its column half)
  unsigned t_head, t_count;   // oldest parked tile and number of parked tiles (FIFO, all older than the ring's tiles)
  StreamBases wb;
  float res;               // residual stream value of row (cur.r0 + lane), bf16-exact
  bool res_valid;
  bool aborted;            // this warp gave up (bounded wait expired)
  bool cta_abort;          // the whole CTA leaves the phase loop
  uint64_t policy;
};

// Position of the decode step the CTA is in: written by warp 0 with the step's RoPE row (kernel entry, and the first phase
// of every later step of a multi-step launch), read after a CTA barrier of the same step.
template <class S>
__device__ __forceinline__ int step_pos(const Params& p, const unsigned char* smem) {
  if constexpr (S::kMulti) return *reinterpret_cast<const volatile int*>(smem + SmemLayout<S>::kOffPos);
  else return p.pos;
}

// Issue the next tile of the stream into the oldest free slot, if any tile is left: one 8-KiB bulk
// copy, or two 4-KiB copies completing on the same mbarrier.
template <class S>
__device__ __forceinline__ void issue_one(Worker<S>& s, const Params& p) {
  const int end = S::kMulti ? p.stream_end : p.phase_end;
  if (s.aborted || s.cur.done(end)) return;
  const Tile t = s.cur.next(s.wb, p.num_layers, end);
  if (s.lane == 0) {
    const uint32_t bar = s.bars + s.i_slot * 8;
    const uint32_t dst = s.ring + s.i_slot * (2 * kChunkBytes);
    mbar_expect_tx(bar, t.bytes_a + (t.b != nullptr ? (uint32_t)kChunkBytes : 0u));
    bulk_g2s(dst, t.a, t.bytes_a, bar, s.policy);
    if (t.b != nullptr) bulk_g2s(dst + kChunkBytes, t.b, kChunkBytes, bar, s.policy);
  }
  ++s.n_issued;
  s.i_slot = (s.i_slot + 1 == kSlots) ? 0u : s.i_slot + 1;
}

// Bounded wait on one ring slot.  Returns false (and flags the error) on expiry.  The spin with its
// deadline is a separate, non-inlined function: it runs only when the data is not there yet.
static __device__ __noinline__ bool wait_slot_slow(const Params& p, uint32_t bar, uint32_t parity, int warp, int phase,
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

// Next tile in consumption order: waits for it, advances the consume cursor and returns the slot's
// shared address.  The slot stays owned by the warp until release_tile().
template <class S>
__device__ __forceinline__ uint32_t acquire_tile(Worker<S>& s, const Params& p, int phase) {
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
  return s.ring + slot * (2 * kChunkBytes);
}
// All lanes are done reading the oldest acquired slot: refill it with the next tile.
template <class S>
__device__ __forceinline__ void release_tile(Worker<S>& s, const Params& p) {
  __syncwarp();
  issue_one(s, p);
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
  const uint32_t addr = ((lane & 8) ? slot1 : slot0) + ((((lane >> 4) << 3) + (lane & 7)) << 4);   // = ldmatrix_lane_addr
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

// ------------------------------------------------------------------------------------------
// Tensor-memory parking.  The ring holds 24 KiB per warp, i.e. all rings together hold about 4 us of
// HBM streaming; whenever the workers wait for activations longer than that (the attention chain
// between QKV and the O-projection takes about 10 us) the rings are full and HBM idles.  The
// tensor memory of the SM (256 KiB, unused by mma.sync) more than doubles the depth: a warp that
// is polling moves landed tiles from its ring into its TMEM share (32 lanes x 256 columns = 4 tiles)
// and refills the freed slots, so the weight stream keeps running through the wait.  A tile is parked
// as the very registers ldmatrix produces for the product (tcgen05.st) and comes back with
// tcgen05.ld, so the product is bit-identical whichever way a tile took.  Parked tiles are older
// than every tile in the ring: consume them first.
// ------------------------------------------------------------------------------------------
constexpr int kTSlots = 4;
constexpr int kTileCols = 2 * kChunkBytes / (32 * 4);   // 32-bit columns one tile takes in a 32-lane quarter
static_assert(kTSlots * kTileCols * (kWorkers / 4) <= 512, "parking space exceeds the tensor memory");

// A tile moves to and from tensor memory in pieces of kPieceSteps k-steps (4 registers per k-step).
constexpr int kPieceSteps = 2;
__device__ __forceinline__ void tmem_st_piece(uint32_t taddr, const uint32_t (&r)[16]) { tmem_st16(taddr, r); }
__device__ __forceinline__ void tmem_st_piece(uint32_t taddr, const uint32_t (&r)[8]) { tmem_st8(taddr, r); }
__device__ __forceinline__ void tmem_ld_piece(uint32_t (&r)[16], uint32_t taddr) { tmem_ld16(r, taddr); }
__device__ __forceinline__ void tmem_ld_piece(uint32_t (&r)[8], uint32_t taddr) { tmem_ld8(r, taddr); }

__device__ __forceinline__ uint32_t ldmatrix_lane_addr(uint32_t slot0, uint32_t slot1, int lane) {
  // matrices 0/2 come from chunk 0, 1/3 from chunk 1; matrices 2/3 are the second piece (k 8..15) of the k-step.
  return ((lane & 8) ? slot1 : slot0) + ((((lane >> 4) << 3) + (lane & 7)) << 4);
}

// Move the oldest landed tile of the ring into tensor memory, if there is one and room for it.
template <class S>
__device__ __forceinline__ void park_one(Worker<S>& s, const Params& p) {
  if (kTSlots == 0 || s.aborted || s.t_count == (unsigned)kTSlots || s.n_acquired == s.n_issued) return;
  const unsigned slot = s.c_slot;
  if (!mbar_try_wait(s.bars + slot * 8, s.c_par)) return;
  const uint32_t src = s.ring + slot * (2 * kChunkBytes);
  const uint32_t addr = ldmatrix_lane_addr(src, src + kChunkBytes, s.lane);
  unsigned tail = s.t_head + s.t_count;
  if (tail >= (unsigned)kTSlots) tail -= kTSlots;
  const uint32_t dst = s.tmem + tail * kTileCols;
#pragma unroll
  for (int q = 0; q < 16 / kPieceSteps; ++q) {
    uint32_t r[4 * kPieceSteps];
#pragma unroll
    for (int t = 0; t < kPieceSteps; ++t) {
      uint32_t a[4];
      ldmatrix_x4(a, addr + (kPieceSteps * q + t) * 256);
#pragma unroll
      for (int j = 0; j < 4; ++j) r[4 * t + j] = a[j];
    }
    tmem_st_piece(dst + q * 4 * kPieceSteps, r);
  }
  tmem_wait_st();
  ++s.t_count;
  ++s.n_acquired;
  if (++s.c_slot == kSlots) {
    s.c_slot = 0;
    s.c_par ^= 1u;
  }
  release_tile(s, p);
}

// The next tile of the stream times the activations in xf, accumulated into cc: from tensor memory
// when tiles are parked there, else from the ring (waits for the copy, refills the slot).
// two = false: the tile holds a single row (its second half is not read from the ring).
template <class S>
__device__ __forceinline__ void consume_tile(Worker<S>& s, const Params& p, int ph, float (&cc)[4], const XFrag& xf,
                                             bool two) {
  if (kTSlots > 0 && s.t_count > 0) {
    const uint32_t src = s.tmem + s.t_head * kTileCols;
    float c[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) c[i][j] = 0.f;
#pragma unroll
    for (int q = 0; q < 16 / kPieceSteps; ++q) {
      uint32_t r[4 * kPieceSteps];
      tmem_ld_piece(r, src + q * 4 * kPieceSteps);
      tmem_wait_ld();
#pragma unroll
      for (int t = 0; t < kPieceSteps; ++t) {
        const int ks = kPieceSteps * q + t;   // k-step: same accumulator and order as mma_chunk_pair
        const uint32_t a[4] = {r[4 * t], r[4 * t + 1], r[4 * t + 2], r[4 * t + 3]};
        mma_bf16_16816(c[ks & 3], a, xf.b[2 * ks], xf.b[2 * ks + 1]);
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) cc[j] += (c[0][j] + c[1][j]) + (c[2][j] + c[3][j]);
    --s.t_count;
    if (++s.t_head == (unsigned)kTSlots) s.t_head = 0;
    return;
  }
  const uint32_t t0 = acquire_tile(s, p, ph);
  mma_chunk_pair(cc, t0, two ? t0 + kChunkBytes : t0, xf, s.lane);
  release_tile(s, p);
}

}  // namespace qmk

#include "qmk_staging.cuh"
#include "qmk_phases.cuh"
