// Batched decode megakernel for sm_100a: B sequences per step, runtime model shape.
//
// One persistent CTA per SM, ten warps with fixed roles:
//   warp 0      producer   one lane streams the CTA's weight tiles (TMA tensor copies, 128-byte swizzle)
//   warp 1      issuer     one lane issues tcgen05.mma (M = 128 weight rows, N = padded batch, K = 16)
//   warps 2-5   epilogue   read accumulators from tensor memory, finish the phase's arithmetic
//   warps 6-9   stagers    build the activation operand ([batch, 64] bf16, RMSNorm applied) in shared memory
// In the attention phase warps 2-9 are eight attention workers.
//
// Every projection is a stream-K GEMM  out[b, n] = sum_k X[b, k] * W[n, k]:  the (row tile, k-block)
// units of a phase, 128 x 64 weights = 16 KiB each, are dealt to the CTAs as equal contiguous ranges,
// so every SM streams the same number of bytes whatever the matrix shape.  A maximal run of units of
// one row tile is a SEGMENT, accumulated in tensor memory.  A segment that covers the whole K is
// finished by its CTA.  Otherwise the CTA that holds the tile's last units FINISHES the tile: the other
// CTAs write their partial tiles as self-validating records {fp32, tag} and go on; the finisher adds the
// records to its own accumulator in a fixed order (ascending CTA), so a step gives the same bits every
// time.  A CTA works through its range head segment first (a partial somebody waits for), whole tiles
// next, tail segment last (qmk_batch_schedule.h).  The reference splits K in the down-projection only
// and adds the partials with bf16 compare-and-swap in arrival order
// (qimeng_megakernel/models/LLM/llama/llama3_2__1b/A100/single_batch/decode_kernel/down_proj_gemv_residual.cu:39-52).
//
// Phases hand data to one another without counters or fences: every activation that crosses SMs is a
// 32-bit word {bf16, 16-bit tag of (launch, producing phase)}, every fp32 value a 64-bit record
// {fp32, 32-bit tag}; consumers poll the data itself (the idea of NCCL's LL protocol, as in the batch-1
// kernel).  The reference's cross-SM protocol is counters with acquire spins (decode_kernel/utils.cuh:266-328).
// The weight stream runs ahead across phase boundaries.  What each phase computes, rounding points
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
constexpr int kSmemBudget = 227 * 1024;                 // dynamic shared memory a CTA may ask for on sm_100

// Shared memory: a fixed header, then the fp32 exchange tile [128][Bpad + 1], then the ring on a 1024-byte boundary
// (128-byte-swizzle atoms).  A ring slot holds 16 KiB of weights and Bpad * 128 bytes of activations, so small
// batches get more slots: more weight bytes in flight per SM.
struct Smem {
  static constexpr int kOffBars = 0;                                          // mbarriers
  //   a_full[kMaxStages] b_full[kMaxStages] empty[kMaxStages] acc_full[2] acc_empty[2]
  static constexpr int kNumBars = 3 * kMaxStages + 4;
  static constexpr int kOffRs = kOffBars + kNumBars * 8;                      // float [64]  rsqrt factors
  static constexpr int kOffHs = kOffRs + kMaxBatch * 4;                       // float [2][64] scratch of the prologue
  static constexpr int kOffPos = kOffHs + 2 * kMaxBatch * 4;                  // int [64]
  static constexpr int kOffAct = kOffPos + kMaxBatch * 4;                     // int [64]
  static constexpr int kOffCtl = kOffAct + kMaxBatch * 4;                     // control words
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
constexpr int kCAbort = 0, kCTmem = 1, kCTmax = 2, kCFlagEpi = 3, kCFlagStg = 4, kCFlagAttn = 5, kCNeStg = 7, kCNeEpi = 8;

struct TensorMaps {
  CUtensorMap qkv, o_proj, up, gate, down, lm_head;   // 3-D {k, row, layer}; box {64, 128 (up/gate: 64), 1}
  // MoE: router {H, E, L} box 128 rows; expert gate|up {H, 2 * Ie, L * E} box 64 rows; expert down {Ie, H, L * E} box 128
  CUtensorMap router, egu, edown;
};

// ------------------------------------------------------------------------------------------------
// small device helpers
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void named_bar(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ void mbar_arrive1(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar,
                                            uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%2, %3, %4}], [%5], %6;" ::"r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// Shared-memory operand descriptor: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_sw128(uint32_t saddr) {
  return (uint64_t)((saddr >> 4) & 0x3fffu) | ((uint64_t)1 << 16) | ((uint64_t)(1024u >> 4) << 32) | (1ull << 46) |
         (2ull << 61);
}
// D (f32, tensor memory) = A (bf16, K-major) x B (bf16, K-major), M = 128: the accumulator is overwritten.
__device__ __forceinline__ void mma_bf16_set(uint32_t d_tmem, uint64_t da, uint64_t db, uint32_t idesc) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.u32 p, 0, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(da), "l"(db), "r"(idesc)
      : "memory");
}
// D += A x B.
__device__ __forceinline__ void mma_bf16_add(uint32_t d_tmem, uint64_t da, uint64_t db, uint32_t idesc) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.eq.u32 p, 0, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(da), "l"(db), "r"(idesc)
      : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}


static __device__ __noinline__ void report(const BParams& p, int code, int warp, int phase, unsigned seen, unsigned expected,
                                           int detail) {
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

// Every wait that gives up -- its own budget ran out (why 1) or it found that another CTA had reported (why 2) -- leaves
// a line in the wait log (the first 64 do): what a launch was waiting for when it stopped, for the host to print.
static __device__ __noinline__ void log_wait(const BParams& p, int warp, int phase, int detail, unsigned seen,
                                             unsigned expected, unsigned why) {
  if ((threadIdx.x & 31u) != 0u && detail != 16) return;   // one line per warp is enough (detail 16: every thread waits alone)
  const unsigned i = atomicAdd(p.wait_log, 1u);
  if (i < 64u) {
    unsigned* e = p.wait_log + 1 + i * 8;
    e[0] = blockIdx.x; e[1] = (unsigned)warp; e[2] = (unsigned)phase; e[3] = (unsigned)detail;
    e[4] = seen; e[5] = expected; e[6] = why; e[7] = 0u;
  }
}

// Optional timeline (qmk_set_trace), eight 64-bit slots per (CTA, phase), globaltimer ns: 0 the stagers (attention:
// the first worker) have the phase's input, 1 the CTA's first accumulator of the phase is complete, 2 the epilogue group
// enters the phase, 5 the CTA's last output of the phase is written.  Cycle sums over the phase's units: 3 / 4 the issuer
// waiting for the weights / the activations of a unit; 6 / 7 stager warp 0 waiting for a free slot / filling.
__device__ __forceinline__ void trace_put(const BParams& p, int ph, int slot) {
  if (p.trace != nullptr) p.trace[((size_t)blockIdx.x * (size_t)num_phases(p) + ph) * 8 + slot] = globaltimer_ns();
}
__device__ __forceinline__ void trace_val(const BParams& p, int ph, int slot, unsigned long long v) {
  if (p.trace != nullptr) p.trace[((size_t)blockIdx.x * (size_t)num_phases(p) + ph) * 8 + slot] = v;
}

struct Ctx {
  const BParams* p;
  unsigned char* smem;
  volatile unsigned* ctl;
  uint32_t bars;     // shared address of the mbarriers
  int warp, lane;
  __device__ __forceinline__ uint32_t a_full(int s) const { return bars + s * 8; }
  __device__ __forceinline__ uint32_t b_full(int s) const { return bars + (kMaxStages + s) * 8; }
  __device__ __forceinline__ uint32_t empty(int s) const { return bars + (2 * kMaxStages + s) * 8; }
  __device__ __forceinline__ uint32_t acc_full(int b) const { return bars + (3 * kMaxStages + b) * 8; }
  __device__ __forceinline__ uint32_t acc_empty(int b) const { return bars + (3 * kMaxStages + 2 + b) * 8; }
  __device__ __forceinline__ bool aborted() const { return ctl[kCAbort] != 0u; }
};

// Bounded wait on an mbarrier phase.  False when the budget expired or the CTA is aborting.
static __device__ __noinline__ bool mbar_wait_slow(const Ctx& c, uint32_t bar, uint32_t parity, int phase, int detail) {
  if (c.ctl[kCAbort] != 0u) return false;
  const long long t0 = clock64();
  for (unsigned it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 63u) == 0u) {
      if (c.ctl[kCAbort] != 0u) return false;
      // (twice the budget of a data wait: these waits sit downstream of one, which should be the one to report)
      if (clock64() - t0 > 2 * c.p->timeout_cycles) {
        log_wait(*c.p, c.warp, phase, detail, parity, bar, 1u);
        report(*c.p, kErrCopyWait, c.warp, phase, parity, bar, detail);
        c.ctl[kCAbort] = 1u;
        return false;
      }
    }
  }
}
__device__ __forceinline__ bool mbar_wait(const Ctx& c, uint32_t bar, uint32_t parity, int phase, int detail) {
  return mbar_try_wait(bar, parity) || mbar_wait_slow(c, bar, parity, phase, detail);
}

// Bounded wait until `*counter` reaches `target` (the LM head's arrivals, before the tokens are written out).
static __device__ __noinline__ bool counter_wait(const Ctx& c, const unsigned* counter, unsigned target, int phase) {
  if (c.ctl[kCAbort] != 0u) return false;
  const long long t0 = clock64();
  for (unsigned it = 1;; ++it) {
    unsigned v = ld_relaxed_gpu(counter);
    if (v >= target) {
      v = ld_acquire_gpu(counter);
      return true;
    }
    if ((it & 15u) == 0u) {
      if (c.ctl[kCAbort] != 0u) return false;
      if (clock64() - t0 > c.p->timeout_cycles) {
        report(*c.p, kErrCounterWait, c.warp, phase, v, target, 0);
        c.ctl[kCAbort] = 1u;
        return false;
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// tags and self-validating data
// ------------------------------------------------------------------------------------------------
// 16-bit tag of the bf16 words phase `ph` of this launch writes; ph = phase_begin - 1 (possibly -1) is the prologue.
// A consumer whose producing phase lies before the launch's first phase reads what the prologue tagged.
__device__ __forceinline__ unsigned tag16(const BParams& p, int src_ph) {
  if (src_ph < p.phase_begin) src_ph = p.phase_begin - 1;
  return (p.epoch * (unsigned)(num_phases(p) + 1) + (unsigned)(src_ph + 1)) % 65535u + 1u;
}
// 32-bit tag of the fp32 records (never 0; the host restarts the epoch on a cleared scratch before it could wrap).
__device__ __forceinline__ unsigned tag32(const BParams& p, int src_ph) {
  if (src_ph < p.phase_begin) src_ph = p.phase_begin - 1;
  return p.epoch * 8192u + (unsigned)(src_ph + 2);
}
__device__ __forceinline__ unsigned long long make_rec(float v, unsigned tag) {
  return (unsigned long long)__float_as_uint(v) | ((unsigned long long)tag << 32);
}
__device__ __forceinline__ bool rec_ok(unsigned long long r, unsigned tag) { return (unsigned)(r >> 32) == tag; }
__device__ __forceinline__ float rec_val(unsigned long long r) { return __uint_as_float((unsigned)r); }

// Loads that are repeated until the data is there: L2 only, never merged or hoisted by the compiler.
__device__ __forceinline__ uint4 poll_ld_u4(const void* ptr) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(ptr) : "memory");
  return v;
}
__device__ __forceinline__ ulonglong2 poll_ld_rec2(const void* ptr) {
  ulonglong2 v;
  asm volatile("ld.global.cg.v2.u64 {%0,%1}, [%2];" : "=l"(v.x), "=l"(v.y) : "l"(ptr) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long poll_ld_rec(const void* ptr) {
  unsigned long long v;
  asm volatile("ld.global.cg.u64 %0, [%1];" : "=l"(v) : "l"(ptr) : "memory");
  return v;
}
__device__ __forceinline__ void st_rec2(void* ptr, unsigned long long a, unsigned long long b) {
  asm volatile("st.global.v2.u64 [%0], {%1,%2};" ::"l"(ptr), "l"(a), "l"(b) : "memory");
}
__device__ __forceinline__ void st_rec(void* ptr, unsigned long long a) {
  asm volatile("st.global.u64 [%0], %1;" ::"l"(ptr), "l"(a) : "memory");
}
// four tagged words carry `tagw` (= tag << 16) in their upper halves
__device__ __forceinline__ bool tags4_ok(const uint4& v, unsigned tagw) {
  return (((v.x ^ tagw) | (v.y ^ tagw) | (v.z ^ tagw) | (v.w ^ tagw)) & 0xffff0000u) == 0u;
}
// 8 tagged words (two 16-byte pieces) -> 8 bf16 packed in 16 bytes
__device__ __forceinline__ uint4 untag8(const uint4& a, const uint4& b) {
  return make_uint4((a.x & 0xffffu) | (a.y << 16), (a.z & 0xffffu) | (a.w << 16), (b.x & 0xffffu) | (b.y << 16),
                    (b.z & 0xffffu) | (b.w << 16));
}
// 8 packed bf16 -> two 16-byte pieces of tagged words
__device__ __forceinline__ void tag8(const uint4& v, unsigned tagw, uint4& a, uint4& b) {
  a = make_uint4((v.x & 0xffffu) | tagw, (v.x >> 16) | tagw, (v.y & 0xffffu) | tagw, (v.y >> 16) | tagw);
  b = make_uint4((v.z & 0xffffu) | tagw, (v.z >> 16) | tagw, (v.w & 0xffffu) | tagw, (v.w >> 16) | tagw);
}
__device__ __forceinline__ void st_tagged8(uint32_t* dst, const uint4& v, unsigned tagw) {
  uint4 a, b;
  tag8(v, tagw, a, b);
  reinterpret_cast<uint4*>(dst)[0] = a;
  reinterpret_cast<uint4*>(dst)[1] = b;
}

// The slow side of a data poll (non-inlined: runs only when the data is not there yet): checks the CTA's abort word,
// the device-wide status word (another CTA gave up: whoever waits for its output would wait in vain) and the budget.
// Returns true when the caller must give up.
static __device__ __noinline__ bool poll_expired(const Ctx& c, long long t0, int phase, unsigned seen, unsigned expected,
                                                 int detail) {
  if (c.ctl[kCAbort] != 0u) return true;
  const unsigned code = ld_relaxed_gpu(c.p->status + kStCode);
  if (code != 0u && code != (unsigned)kErrRowPosition) {   // (a switched-off row is reported but stops nothing)
    log_wait(*c.p, c.warp, phase, detail, seen, expected, 2u);
    c.ctl[kCAbort] = 1u;
    return true;
  }
  if (clock64() - t0 > c.p->timeout_cycles) {
    log_wait(*c.p, c.warp, phase, detail, seen, expected, 1u);
    report(*c.p, kErrCounterWait, c.warp, phase, seen, expected, detail);
    c.ctl[kCAbort] = 1u;
    return true;
  }
  return false;
}

// Number of distinct experts of this step, for the two expert phases of a MoE layer: the router phase's finisher
// publishes {count, tag} after the expert list and the router weights are written and fenced (one thread calls this;
// 0 after a wait that gave up).  A router phase that ran in an earlier launch is taken on stream order.
static __device__ __noinline__ int expert_count(const Ctx& c, int ph) {
  const BParams& p = *c.p;
  const int rph = phase_layer(p, ph) * p.ppl + 3;
  if (rph < p.phase_begin) return *reinterpret_cast<const volatile int*>(p.moe_ne);
  if (c.ctl[kCAbort] != 0u) return 0;
  const unsigned tag = tag32(p, rph);
  const long long t0 = clock64();
  for (unsigned it = 1;; ++it) {
    const unsigned long long r = poll_ld_rec(p.moe_ne_rec);
    if (rec_ok(r, tag)) {
      __threadfence();   // (acquire side of the router's fence: the list and the weights are read after this)
      return (int)(unsigned)r;
    }
    if ((it & 15u) == 0u && poll_expired(c, t0, ph, (unsigned)(r >> 32), tag, 7)) return 0;
  }
}
__device__ __forceinline__ bool is_expert_kind(int kind) { return kind == kEUpGate || kind == kEDown; }

// ------------------------------------------------------------------------------------------------
// producer (one thread)
// ------------------------------------------------------------------------------------------------
static __device__ __noinline__ void producer(const Ctx& c, const TensorMaps& maps, unsigned& n_issued) {
  const BParams& p = *c.p;
  const uint32_t stages = smem_u32(c.smem + p.off_stages);
  const uint64_t policy = l2_policy_evict_first();
  const int G = (int)gridDim.x, cta = (int)blockIdx.x;
  unsigned n = 0;
#pragma unroll 1
  for (int ph = p.phase_begin; ph < p.phase_end; ++ph) {
    const int kind = phase_kind(p, ph);
    if (kind == kAttn) continue;
    const int layer = phase_layer(p, ph);
    const int ne = is_expert_kind(kind) ? expert_count(c, ph) : 0;
    const PhaseDims d = phase_dims(p, kind, ne);
    int lo, hi;
    unit_range(d.T * d.KB, phase_ctas(kind, d.T * d.KB, G), cta, lo, hi);
    const UnitRuns R = unit_runs(lo, hi, d.KB);
    const CUtensorMap* map = kind == kQkv ? &maps.qkv : kind == kOproj ? &maps.o_proj : kind == kUpGate ? &maps.up
                           : kind == kDown ? &maps.down : kind == kRouter ? &maps.router : &maps.lm_head;
    const int per = p.Ie > 0 ? p.Ie / kBlockK : 1;   // 64-row tiles (k-blocks) of one expert
    int zslot = -1, zval = 0;   // expert phases: the selected expert's index is fetched when the slot changes
    auto expert_z = [&](int slot) {
      if (slot != zslot) { zslot = slot; zval = layer * p.E + __ldcg(p.moe_elist + slot); }
      return zval;
    };
#pragma unroll 1
    for (int r = 0; r < 3; ++r) {
      int t = d.KB > 0 ? R.lo[r] / d.KB : 0, kb = R.lo[r] - t * d.KB;
#pragma unroll 1
      for (int u = R.lo[r]; u < R.hi[r]; ++u, ++n) {
        const int s = (int)(n & (unsigned)(kStages - 1));
        if (n >= (unsigned)kStages && !mbar_wait(c, c.empty(s), ((n / (unsigned)kStages) - 1u) & 1u, ph, 1)) {
          n_issued = n;
          return;
        }
        const uint32_t dst = stages + s * p.stage_bytes;
        mbar_expect_tx(c.a_full(s), (uint32_t)kABytes);
        if (kind == kUpGate) {
          tma_load_3d(dst, map, kb * kBlockK, t * (kTileRows / 2), layer, c.a_full(s), policy);
          tma_load_3d(dst + kABytes / 2, &maps.gate, kb * kBlockK, t * (kTileRows / 2), layer, c.a_full(s), policy);
        } else if (kind == kEUpGate) {   // tile t = (selected expert t / per, 64 gate rows + 64 up rows of that expert)
          const int z = expert_z(t / per), lt = t % per;
          tma_load_3d(dst, &maps.egu, kb * kBlockK, lt * (kTileRows / 2), z, c.a_full(s), policy);
          tma_load_3d(dst + kABytes / 2, &maps.egu, kb * kBlockK, p.Ie + lt * (kTileRows / 2), z, c.a_full(s), policy);
        } else if (kind == kEDown) {     // k-block kb = (selected expert kb / per, its k-block kb % per)
          const int z = expert_z(kb / per);
          tma_load_3d(dst, &maps.edown, (kb % per) * kBlockK, t * kTileRows, z, c.a_full(s), policy);
        } else {
          tma_load_3d(dst, map, kb * kBlockK, t * kTileRows, layer, c.a_full(s), policy);
        }
        if (++kb == d.KB) { kb = 0; ++t; }
      }
    }
  }
  n_issued = n;
}

// ------------------------------------------------------------------------------------------------
// issuer (one thread)
// ------------------------------------------------------------------------------------------------
static __device__ __noinline__ void issuer(const Ctx& c, uint32_t tmem) {
  const BParams& p = *c.p;
  const uint32_t stages = smem_u32(c.smem + p.off_stages);
  const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (((uint32_t)p.Bpad >> 3) << 17) | ((128u >> 4) << 24);
  const int G = (int)gridDim.x, cta = (int)blockIdx.x;
  unsigned n = 0, sg = 0;
  const bool tr = p.trace != nullptr;
#pragma unroll 1
  for (int ph = p.phase_begin; ph < p.phase_end; ++ph) {
    const int kind = phase_kind(p, ph);
    if (kind == kAttn) continue;
    const PhaseDims d = phase_dims(p, kind, is_expert_kind(kind) ? expert_count(c, ph) : 0);
    int lo, hi;
    unit_range(d.T * d.KB, phase_ctas(kind, d.T * d.KB, G), cta, lo, hi);
    const UnitRuns R = unit_runs(lo, hi, d.KB);
    long long w_a = 0, w_b = 0;
#pragma unroll 1
    for (int r = 0; r < 3; ++r) {
      int kb = d.KB > 0 ? R.lo[r] % d.KB : 0;
      bool seg_start = true;
#pragma unroll 1
      for (int u = R.lo[r]; u < R.hi[r]; ++u, ++n) {
        const unsigned buf = sg & 1u;
        if (seg_start && sg >= 2u && !mbar_wait(c, c.acc_empty(buf), ((sg >> 1) - 1u) & 1u, ph, 2)) return;
        const int s = (int)(n & (unsigned)(kStages - 1));
        const unsigned par = (n / (unsigned)kStages) & 1u;
        const long long t0 = tr ? clock64() : 0;
        if (!mbar_wait(c, c.a_full(s), par, ph, 3)) return;
        const long long t1 = tr ? clock64() : 0;
        if (!mbar_wait(c, c.b_full(s), par, ph, 4)) return;
        w_a += t1 - t0;
        w_b += (tr ? clock64() : 0) - t1;
        tmem_fence_after_sync();
        const uint64_t da = desc_sw128(stages + s * p.stage_bytes), db = desc_sw128(stages + s * p.stage_bytes + kABytes);
        const uint32_t dcol = tmem + buf * (uint32_t)p.Bpad;
        // (k-step k reads 32 bytes further along K: the start-address field grows by 2)
        if (seg_start) mma_bf16_set(dcol, da, db, idesc);
        else mma_bf16_add(dcol, da, db, idesc);
#pragma unroll
        for (int k = 1; k < kBlockK / 16; ++k) mma_bf16_add(dcol, da + 2u * k, db + 2u * k, idesc);
        mma_commit(c.empty(s));
        seg_start = false;
        if (++kb == d.KB || u + 1 == R.hi[r]) {
          mma_commit(c.acc_full(buf));
          ++sg;
          kb = kb == d.KB ? 0 : kb;
          seg_start = true;
        }
      }
    }
    trace_val(p, ph, 3, (unsigned long long)w_a);
    trace_val(p, ph, 4, (unsigned long long)w_b);
  }
}

// ------------------------------------------------------------------------------------------------
// stagers (128 threads): activation operand of every unit
// ------------------------------------------------------------------------------------------------
// What a phase's activation operand is read from: tagged words [row, K] (expert down-projection: [slot, row, Ie]).
struct StageSrc {
  const uint32_t* words;     // tagged source
  unsigned tagw;             // expected tag << 16
  bool checked;              // false: the producer ran in an earlier launch, the words are taken on stream order
  const uint16_t* gain;      // RMSNorm gain of the phase, or null
  const float* wsc;          // expert down-projection: router weight of (slot, row)
  int per;                   // expert down-projection: k-blocks per expert (0 otherwise)
};

// Stages the activation operand of the CTA's units of one phase: `total` units in the order of the runs R, at ring
// positions n, n + 1, ...  Ring positions are dealt to the four warps in groups of D by position, not by unit:
// group g = position / D belongs to warp g % 4, so a warp always fills the same ring slots, lap after lap, and the wait
// for a slot's previous occupant to be consumed (an mbarrier parity wait, which cannot tell a phase from the one two
// laps before it) is never more than one lap ahead of the wait the same warp made for that slot before.  A lane owns the
// 16-byte piece `chunk` of the 128-byte k-block row of the batch rows row0, row0 + 4, ...; the rows are taken in PASSES
// passes of NPL rows so that the 2 * D * NPL loads of a pass (tagged words are twice the size of the bf16 they carry)
// fit the registers; all loads of a pass are issued before the first is used and repeated until every word carries the
// tag.
template <int NPL, int PASSES, int D, bool EXPERT>
static __device__ __noinline__ void stage_units(const Ctx& c, int ph, const PhaseDims& d, const UnitRuns& R, int total, int st,
                                                unsigned n, const StageSrc& src, const float* rs) {
  static_assert(kStages % (4 * D) == 0, "every warp must own whole ring slots");
  const BParams& p = *c.p;
  const int sw = st >> 5, lane = st & 31;
  const int chunk = lane & 7;         // 16-byte piece inside the 128-byte k-block row
  const int row0 = lane >> 3;         // first batch row of this lane (then +4, +8, ...)
  long long w_slot = 0, w_fill = 0;
  const bool tr = p.trace != nullptr;
  const int la = R.hi[0] - R.lo[0], lab = la + R.hi[1] - R.lo[1];
  auto unit_at = [&](int i) { return i < la ? R.lo[0] + i : (i < lab ? R.lo[1] + (i - la) : R.lo[2] + (i - lab)); };
  // first group of this warp at or after ring position n
  unsigned g0 = n / (unsigned)D;
  g0 += ((unsigned)sw + 4u - (g0 & 3u)) & 3u;
  bool first_group = true;
#pragma unroll 1
  for (unsigned g = g0; g * (unsigned)D < n + (unsigned)total; g += 4u) {
    const int base = (int)(g * (unsigned)D) - (int)n;   // index of the group's first position in the phase's unit sequence (may be < 0)
    bool slot_ok[D];
#pragma unroll
    for (int j = 0; j < D; ++j) slot_ok[j] = false;
#pragma unroll 1
    for (int q = 0; q < PASSES; ++q) {
      uint4 va[D][NPL], vb[D][NPL];
      int off[D][NPL];   // word offset of the lane's piece in the source, -1: nothing to fetch (row or unit past the end)
      float sc[EXPERT ? D : 1][EXPERT ? NPL : 1];
      uint4 g4[D];
#pragma unroll
      for (int j = 0; j < D; ++j) {
        const bool have = base + j >= 0 && base + j < total;
        const int kbu = have ? unit_at(base + j) % d.KB : 0;
        const int k0 = kbu * kBlockK + chunk * 8;
        g4[j] = make_uint4(0, 0, 0, 0);
        if (src.gain != nullptr && have) g4[j] = __ldg(reinterpret_cast<const uint4*>(src.gain + k0));
#pragma unroll
        for (int i = 0; i < NPL; ++i) {
          const int r = row0 + 4 * (q * NPL + i);
          off[j][i] = -1;
          if (EXPERT) sc[EXPERT ? j : 0][EXPERT ? i : 0] = 0.f;
          if (have && r < p.B) {
            if (EXPERT) {
              const int slot = kbu / src.per;
              off[j][i] = (slot * kMaxBatch + r) * p.Ie + (kbu % src.per) * kBlockK + chunk * 8;
              sc[EXPERT ? j : 0][EXPERT ? i : 0] = ldcg_f32(src.wsc + slot * kMaxBatch + r);
            } else {
              off[j][i] = r * d.K + k0;
            }
          }
        }
      }
      // fetch until every word of the pass carries the tag
      const long long tp0 = clock64();
      for (unsigned it = 1;; ++it) {
        bool ok = true;
#pragma unroll
        for (int j = 0; j < D; ++j)
#pragma unroll
          for (int i = 0; i < NPL; ++i) {
            va[j][i] = vb[j][i] = make_uint4(0, 0, 0, 0);
            if (off[j][i] >= 0) {
              va[j][i] = poll_ld_u4(src.words + off[j][i]);
              vb[j][i] = poll_ld_u4(src.words + off[j][i] + 4);
            }
          }
        if (src.checked) {
#pragma unroll
          for (int j = 0; j < D; ++j)
#pragma unroll
            for (int i = 0; i < NPL; ++i)
              if (off[j][i] >= 0) ok = ok && tags4_ok(va[j][i], src.tagw) && tags4_ok(vb[j][i], src.tagw);
        }
        if (__all_sync(kFullMask, ok)) break;
        if ((it & 7u) == 0u && __any_sync(kFullMask, poll_expired(c, tp0, ph, va[0][0].x >> 16, src.tagw >> 16, 5))) return;
      }
      if (q == 0 && first_group && base <= 0 && (st & 31) == 0) trace_put(p, ph, 0);
      first_group = false;
#pragma unroll
      for (int j = 0; j < D; ++j) {
        if (base + j < 0 || base + j >= total) continue;
        const unsigned nu = g * (unsigned)D + (unsigned)j;
        const int s = (int)(nu & (unsigned)(kStages - 1));
        const long long t0 = tr ? clock64() : 0;
        if (q == 0) slot_ok[j] = nu < (unsigned)kStages || mbar_wait(c, c.empty(s), ((nu / (unsigned)kStages) - 1u) & 1u, ph, 5);
        const long long t1 = tr ? clock64() : 0;
        w_slot += t1 - t0;
        if (!slot_ok[j]) continue;
        unsigned char* dst = c.smem + p.off_stages + s * p.stage_bytes + kABytes;
        const uint32_t* gw = reinterpret_cast<const uint32_t*>(&g4[j]);
#pragma unroll
        for (int i = 0; i < NPL; ++i) {
          const int r = row0 + 4 * (q * NPL + i);
          uint4 v = untag8(va[j][i], vb[j][i]);
          uint32_t* w = reinterpret_cast<uint32_t*>(&v);
          if (src.gain != nullptr && r < p.B) {
            const float f = rs[r];
#pragma unroll
            for (int x = 0; x < 4; ++x) {
              const float a = bf16_round(bf_lo(w[x]) * f) * bf_lo(gw[x]);
              const float b = bf16_round(bf_hi(w[x]) * f) * bf_hi(gw[x]);
              w[x] = pack_bf16x2(a, b);
            }
          } else if (EXPERT) {
            const float f = sc[EXPERT ? j : 0][EXPERT ? i : 0];
#pragma unroll
            for (int x = 0; x < 4; ++x) w[x] = pack_bf16x2(bf_lo(w[x]) * f, bf_hi(w[x]) * f);
          }
          *reinterpret_cast<uint4*>(dst + r * 128 + ((chunk ^ (r & 7)) << 4)) = v;
        }
        if (q == PASSES - 1) {
          fence_async_smem();
          mbar_arrive1(c.b_full(s));
        }
        if (tr) w_fill += clock64() - t1;
      }
    }
  }
  if (st == 0) {
    trace_val(p, ph, 6, (unsigned long long)w_slot);
    trace_val(p, ph, 7, (unsigned long long)w_fill);
  }
}

// Reciprocal RMS of every row of the residual stream: the producing residual phase left one record {sum of squares,
// tag} per (row tile, row); thread st < B adds its row's records in tile order (sixteen per round trip).
__device__ __forceinline__ void stage_rs(const Ctx& c, int ph, int st, unsigned tag, float* rs) {
  const BParams& p = *c.p;
  if (st >= p.Bpad) return;
  if (st >= p.B) { rs[st] = 0.f; return; }
  float tot = 0.f;
  const int nt = (p.H + kTileRows - 1) / kTileRows;
  const long long t0 = clock64();
  for (int tb = 0; tb < nt; tb += 16) {
    unsigned long long v[16];
    for (unsigned it = 1;; ++it) {
      bool ok = true;
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] = tb + j < nt ? poll_ld_rec(p.ss_rec + (size_t)(tb + j) * kMaxBatch + st) : 0ull;
#pragma unroll
      for (int j = 0; j < 16; ++j) ok = ok && (tb + j >= nt || rec_ok(v[j], tag));
      if (ok) break;
      if ((it & 7u) == 0u && poll_expired(c, t0, ph, (unsigned)(v[0] >> 32), tag, 6)) { rs[st] = 0.f; return; }
    }
#pragma unroll
    for (int j = 0; j < 16; ++j) tot += tb + j < nt ? rec_val(v[j]) : 0.f;
  }
  rs[st] = rsqrtf(tot / (float)p.H + p.eps);
}

static __device__ __noinline__ void stage_phase(const Ctx& c, int ph, int kind, int st, unsigned& n) {
  // st: thread index inside the stager group, 0..127
  const BParams& p = *c.p;
  const int layer = phase_layer(p, ph);
  named_bar(kBarStg, 128);   // every stager is done with the phase before: its rs factors and control word are free
  if (is_expert_kind(kind)) {
    if (st == 0) c.ctl[kCNeStg] = (unsigned)expert_count(c, ph);
    named_bar(kBarStg, 128);
  }
  const PhaseDims d = phase_dims(p, kind, is_expert_kind(kind) ? (int)c.ctl[kCNeStg] : 0);
  int lo, hi;
  unit_range(d.T * d.KB, phase_ctas(kind, d.T * d.KB, (int)gridDim.x), (int)blockIdx.x, lo, hi);
  const bool normed = phase_normed(kind);
  float* rs = reinterpret_cast<float*>(c.smem + Smem::kOffRs);
  if (hi > lo) {
    if (normed) stage_rs(c, ph, st, tag32(p, hidden_source(kind, ph)), rs);
    named_bar(kBarStg, 128);
    StageSrc src;
    const int sph = normed ? hidden_source(kind, ph) : ph - 1;
    src.words = kind == kOproj ? p.t_attn : kind == kDown ? p.t_silu : kind == kEDown ? p.t_esilu : p.t_hid;
    src.tagw = tag16(p, sph) << 16;
    src.checked = !(kind == kEDown && sph < p.phase_begin);
    src.gain = !normed ? nullptr
             : kind == kQkv ? p.attn_norm + (size_t)layer * p.H
             : kind == kLmHead ? p.lm_norm : p.mlp_norm + (size_t)layer * p.H;
    src.wsc = kind == kEDown ? p.moe_w : nullptr;
    src.per = kind == kEDown ? p.Ie / kBlockK : 0;
    const UnitRuns R = unit_runs(lo, hi, d.KB);
    const int total = hi - lo;
    if (kind == kEDown) {
      switch (p.Bpad) {
        case 16: stage_units<4, 1, 2, true>(c, ph, d, R, total, st, n, src, rs); break;
        case 32: stage_units<8, 1, 1, true>(c, ph, d, R, total, st, n, src, rs); break;
        case 48: stage_units<6, 2, 1, true>(c, ph, d, R, total, st, n, src, rs); break;
        default: stage_units<8, 2, 1, true>(c, ph, d, R, total, st, n, src, rs); break;
      }
    } else {
      switch (p.Bpad) {
        case 16: stage_units<4, 1, 2, false>(c, ph, d, R, total, st, n, src, rs); break;
        case 32: stage_units<8, 1, 1, false>(c, ph, d, R, total, st, n, src, rs); break;
        case 48: stage_units<6, 2, 1, false>(c, ph, d, R, total, st, n, src, rs); break;
        default: stage_units<8, 2, 1, false>(c, ph, d, R, total, st, n, src, rs); break;
      }
    }
  }
  n += (unsigned)(hi - lo);
}

}  // namespace qmkb

#include "qmk_batch_epilogue.cuh"
#include "qmk_batch_attention.cuh"

namespace qmkb {

// ------------------------------------------------------------------------------------------------
// prologue / finalize (epilogue group)
// ------------------------------------------------------------------------------------------------
// Copies `n` bf16 (a multiple of 8) into tagged words.
__device__ __forceinline__ void tag_row(uint32_t* dst, const uint16_t* src, int n, unsigned tagw, int e) {
  for (int i = e; i < n / 8; i += 128) st_tagged8(dst + i * 8, ldcg_u4(src + i * 8), tagw);
}

static __device__ __noinline__ void prologue(const Ctx& c, int e) {
  // What the first phase of the launch reads comes from the caller's buffers: rows b = cta, cta + G, ... are copied into
  // the tagged scratch under the tag of "the phase before the first" -- the residual stream (optionally the embedding
  // row of token_in[b]) with its sum of squares, and, when the launch starts in the middle of a layer, the first
  // phase's own input (q and this position's K / V row, the attention output, or the SwiGLU output).
  const BParams& p = *c.p;
  float* red = reinterpret_cast<float*>(c.smem + Smem::kOffHs);
  const int* pos_s = reinterpret_cast<const int*>(c.smem + Smem::kOffPos);
  const int* act_s = reinterpret_cast<const int*>(c.smem + Smem::kOffAct);
  const int nt = (p.H + kTileRows - 1) / kTileRows;
  const unsigned tagw = tag16(p, p.phase_begin - 1) << 16;
  const unsigned rtag = tag32(p, p.phase_begin - 1);
  const int kind0 = phase_kind(p, p.phase_begin), layer0 = phase_layer(p, p.phase_begin);
  for (int b = (int)blockIdx.x; b < p.B; b += (int)gridDim.x) {
    uint16_t* h = p.hidden + (size_t)b * p.H;
    const uint16_t* src = h;
    if (p.prologue == 2) {   // (a token id outside the vocabulary is clamped, as the batch-1 kernel does)
      long long tok = p.token_in[b];
      tok = tok < 0 ? 0 : (tok >= p.vocab ? (long long)p.vocab - 1 : tok);
      src = p.embed + (size_t)tok * p.H;
    }
    float s = 0.f;
    for (int i = e; i < p.H / 8; i += 128) {
      const uint4 v = ldcg_u4(src + i * 8);
      if (p.prologue == 2) reinterpret_cast<uint4*>(h)[i] = v;
      st_tagged8(p.t_hid + (size_t)b * p.H + i * 8, v, tagw);
      const uint32_t* w = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) s += bf_lo(w[j]) * bf_lo(w[j]) + bf_hi(w[j]) * bf_hi(w[j]);
    }
    s = warp_sum(s);
    if (c.lane == 0) red[e >> 5] = s;
    named_bar(kBarEpi, 128);
    if (e < nt) st_rec(p.ss_rec + (size_t)e * kMaxBatch + b, make_rec(e == 0 ? red[0] + red[1] + red[2] + red[3] : 0.f, rtag));
    named_bar(kBarEpi, 128);
    if (kind0 == kAttn) {
      tag_row(p.t_q + (size_t)b * p.QDIM, p.q_post_rope + (size_t)b * p.QDIM, p.QDIM, tagw, e);
      if (act_s[b]) {
        const int kdim = p.NKV * p.HD;
        const size_t row = (size_t)layer0 * p.kv_layer_stride + (size_t)b * p.kv_batch_stride + (size_t)pos_s[b] * p.kv_seq_stride;
        tag_row(p.t_kv + ((size_t)b * 2 + 0) * kdim, p.k_cache + row, kdim, tagw, e);
        tag_row(p.t_kv + ((size_t)b * 2 + 1) * kdim, p.v_cache + row, kdim, tagw, e);
      }
    } else if (kind0 == kOproj) {
      tag_row(p.t_attn + (size_t)b * p.QDIM, p.attn_out + (size_t)b * p.QDIM, p.QDIM, tagw, e);
    } else if (kind0 == kDown) {
      tag_row(p.t_silu + (size_t)b * p.I, p.silu_out + (size_t)b * p.I, p.I, tagw, e);
    }
  }
  __threadfence();   // (push the tagged words out; nothing waits for this fence)
}

__device__ __forceinline__ void finalize(const Ctx& c, int e) {
  // CTA 0, after every CTA has finished the LM head: tokens out
  const BParams& p = *c.p;
  const int lm = p.ppl * p.num_layers;
  if (e == 0) c.ctl[kCFlagEpi] = counter_wait(c, p.phase_done + 1 + lm, gridDim.x, lm) ? 1u : 0u;
  named_bar(kBarEpi, 128);
  if (c.ctl[kCFlagEpi] != 0u && e < p.B) {
    const int* pos_s = reinterpret_cast<const int*>(c.smem + Smem::kOffPos);
    const unsigned long long win = __ldcg(p.argmax_key + e);
    const long long tok = (long long)(0xffffffffu - (unsigned)(win & 0xffffffffull));
    if (p.next_token) p.next_token[e] = tok;
    if (p.out_tokens && pos_s[e] >= 0 && (long long)pos_s[e] + 1 < p.out_tokens_len)
      p.out_tokens[(size_t)e * p.out_tokens_len + pos_s[e] + 1] = tok;
  }
}

// ------------------------------------------------------------------------------------------------
// kernel
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kBatchThreads, 1)
qmk_batch_kernel(const __grid_constant__ BParams p, const __grid_constant__ TensorMaps maps) {
  extern __shared__ __align__(1024) unsigned char smem[];
  if ((smem_u32(smem) & 1023u) != 0u) {   // the swizzle atoms need a 1024-byte aligned ring (true without static shared memory)
    if (threadIdx.x == 0) report(p, kErrStageWait, 0, p.phase_begin, smem_u32(smem), 1024u, 9);
    return;
  }
  Ctx c;
  c.p = &p;
  c.smem = smem;
  c.ctl = reinterpret_cast<volatile unsigned*>(smem + Smem::kOffCtl);
  c.bars = smem_u32(smem + Smem::kOffBars);
  c.warp = threadIdx.x >> 5;
  c.lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(c.a_full(s), 1);
      mbar_init(c.b_full(s), 32);
      mbar_init(c.empty(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(c.acc_full(b), 1);
      mbar_init(c.acc_empty(b), 128);
    }
    fence_barrier_init();
    for (int i = 0; i < 16; ++i) c.ctl[i] = 0u;
  }
  if (threadIdx.x < kMaxBatch) {
    const int b = threadIdx.x;
    int* pos_s = reinterpret_cast<int*>(smem + Smem::kOffPos);
    int* act_s = reinterpret_cast<int*>(smem + Smem::kOffAct);
    int pos = b < p.B ? (p.position_ids ? p.position_ids[b] : p.pos) : 0;
    int act = b < p.B ? (p.active_mask ? (int)p.active_mask[b] : 1) : 0;
    // An active row whose position lies outside the KV cache or the RoPE table would read and write out of bounds:
    // it is switched off (no KV write, zero projections, like a finished row) and the launch reports it.
    if (act != 0 && (pos < 0 || pos >= p.pos_limit)) {
      if (blockIdx.x == 0) report(p, kErrRowPosition, 0, p.phase_begin, (unsigned)pos, (unsigned)p.pos_limit, b);
      act = 0;
      pos = -1;
    }
    pos_s[b] = pos;
    act_s[b] = act;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const int* pos_s = reinterpret_cast<const int*>(smem + Smem::kOffPos);
    const int* act_s = reinterpret_cast<const int*>(smem + Smem::kOffAct);
    int tmax = 1;
    for (int b = 0; b < p.B; ++b)
      if (act_s[b]) tmax = max(tmax, pos_s[b] + 1);
    c.ctl[kCTmax] = (unsigned)tmax;
  }
  if (c.warp == 0) {
    tmem_alloc(smem_u32(smem + Smem::kOffCtl + kCTmem * 4), 128);
    tmem_fence_before_sync();
  }
  __syncthreads();
  tmem_fence_after_sync();
  const uint32_t tmem = c.ctl[kCTmem];
  unsigned n_issued = 0;

  if (c.warp == 0) {
    if (c.lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&maps.qkv) : "memory");
      producer(c, maps, n_issued);
    }
  } else if (c.warp == 1) {
    if (c.lane == 0) issuer(c, tmem);
  } else {
    const bool epi = c.warp < kStgWarp0;
    const int gi = (c.warp - (epi ? kEpiWarp0 : kStgWarp0)) * 32 + c.lane;   // index inside the group of 128
    unsigned n = 0, sg = 0;
    if (epi && p.prologue != 0) prologue(c, gi);
#pragma unroll 1
    for (int ph = p.phase_begin; ph < p.phase_end; ++ph) {
      const int kind = phase_kind(p, ph);
      if (kind == kAttn) {
        attention_phase(c, ph, c.warp - kEpiWarp0);
      } else if (epi) {
        if (gi == 0) trace_put(p, ph, 2);
        epilogue_phase(c, ph, kind, tmem, gi, sg);
        if (gi == 0) trace_put(p, ph, 5);
        if (kind == kLmHead) {   // the tokens are written once every CTA's logits and arg-max keys are out
          __threadfence();
          named_bar(kBarEpi, 128);
          if (gi == 0 && !c.aborted()) red_release_gpu_add(p.phase_done + 1 + ph, 1u);
        }
      } else {
        stage_phase(c, ph, kind, gi, n);
      }
    }
    if (epi && blockIdx.x == 0 && p.phase_end == num_phases(p)) finalize(c, gi);
  }
  __syncwarp();
  tmem_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && c.aborted()) {
    // leave no tensor copy in flight into this CTA's shared memory: wait (bounded) for the last fills
    const unsigned first = n_issued > (unsigned)kStages ? n_issued - (unsigned)kStages : 0u;
    for (unsigned m = first; m < n_issued; ++m) {
      const long long t0 = clock64();
      while (!mbar_try_wait(c.a_full((int)(m & (unsigned)(kStages - 1))), (m / (unsigned)kStages) & 1u)) {
        if (clock64() - t0 > p.timeout_cycles) break;
      }
    }
  }
  __syncthreads();
  if (c.warp == 0) {
    tmem_fence_after_sync();
    tmem_dealloc(tmem, 128);
  }
}

}  // namespace qmkb
