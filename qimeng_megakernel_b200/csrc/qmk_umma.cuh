// Weight streaming on the 5th-generation tensor cores (tcgen05.mma, accumulators in tensor memory).
// Included by qmk_megakernel.cuh.
//
// Roles in a CTA (one CTA per SM): eight worker warps (staging of activations, attention, epilogues),
// one producer warp and one issuer warp (one lane of each runs).
//
//  * Producer: walks the CTA's static stream of GROUPS (16 row chunks of 4 KiB, qmk_schedule.h) and
//    copies each group with cp.async.bulk into one of three 64-KiB ring slots, across phase and
//    layer boundaries, as far ahead as the ring allows.
//  * Issuer: for every landed slot issues sixteen tcgen05.mma (M = 128, N = 16, K = 16, bf16 -> fp32).
//    The weights stay exactly as the bulk copy laid them down (plain rows).  Read through a
//    no-swizzle K-major descriptor, 128 contiguous bytes are one 8 x 16-byte "core matrix": its 8 rows
//    are eight consecutive 16-byte PIECES of one weight row.  With the stride between 8-row groups set
//    to 4 KiB, row 8*s + i of the A operand is piece i of slot s; the B operand is the activation vector
//    read the same way (row j = piece j).  Then D[8*s + i][j] accumulates piece_i(w_s) . piece_j(x) over
//    the whole row, and the dot product of slot s with x is the trace sum_i D[8*s + i][i].
//    Only 1/8 of the products are used; the tensor pipe has nothing else to do in a batch-1 decode.
//  * Workers: lane 8*s' + i of a warp's quarter of tensor memory holds row 8*s + i of D.  The thread
//    takes column i of its row (tcgen05.ld), three shuffles add the eight threads of a slot, and the
//    phase's epilogue runs on that value.  Even groups of a phase go to warps 0-3, odd ones to 4-7.
//
// Every wait is bounded; a wait that expires records a status, raises the CTA's abort words and all
// roles fall through to the common exit, where the tensor memory is freed.
#pragma once

namespace qmk {

constexpr int kUSlots = 3;                        // 64-KiB ring slots
constexpr int kDBufs = 4;                         // accumulator buffers in tensor memory
constexpr int kDCols = 16;                        // 32-bit columns per accumulator buffer (N = 16)
constexpr int kTmemCols = 64;                     // allocation: a power of two >= kDBufs * kDCols
constexpr int kCtrlWarps = 2;
constexpr int kLaunchThreads = kThreads + 32 * kCtrlWarps;
static_assert(kUSlots * kGroupBytes <= kWorkers * kSlots * 2 * kChunkBytes, "ring region too small");
static_assert(kDBufs * kDCols <= kTmemCols, "accumulators exceed the tensor-memory allocation");
// mbarriers (64-bit each, from SmemLayout::kOffBars)
constexpr int kBarFull = 0;                       // [kUSlots]  bytes of a slot landed        (producer -> issuer)
constexpr int kBarFree = kBarFull + kUSlots;      // [kUSlots]  products of a slot complete   (issuer -> producer)
constexpr int kBarDReady = kBarFree + kUSlots;    // [kDBufs]   accumulator complete          (issuer -> workers)
constexpr int kBarDFree = kBarDReady + kDBufs;    // [kDBufs]   accumulator read, 4 arrivals  (workers -> issuer)
constexpr int kBarXReady = kBarDFree + kDBufs;    // [1]        activations of a phase staged (workers -> issuer)
constexpr int kNumBars = kBarXReady + 1;
static_assert(kNumBars <= kWorkers * kSlots, "mbarrier region too small");
// second abort word, written by the control warps only (the workers' own word must not change between
// the worker barriers, see cta_sync)
constexpr int kCtlCtrlAbort = 5;

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Shared-memory matrix descriptor, K-major, no swizzle: lbo = bytes between the two core matrices of a
// k-step, sbo = bytes between 8-row groups.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  return (uint64_t)((saddr >> 4) & 0x3fffu) | ((uint64_t)((lbo >> 4) & 0x3fffu) << 16) |
         ((uint64_t)((sbo >> 4) & 0x3fffu) << 32) | (1ull << 46);
}
// D (f32) [+]= A (bf16, K-major) x B (bf16, K-major); M = 128, N = 16.
constexpr uint32_t kUmmaIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((16u >> 3) << 17) | ((128u >> 4) << 24);
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t da, uint64_t db, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(da), "l"(db), "r"(kUmmaIdesc), "r"(accumulate), "r"(0), "r"(0), "r"(0), "r"(0)
      : "memory");
}
// The same with the accumulate flag fixed to "add": no predicate to compute per instruction.
__device__ __forceinline__ void umma_bf16_add(uint32_t d_tmem, uint64_t da, uint64_t db) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.eq.u32 p, 0, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%4, %5, %6, %7}, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(da), "l"(db), "r"(kUmmaIdesc), "r"(0), "r"(0), "r"(0), "r"(0)
      : "memory");
}
// The mbarrier gets one arrival when every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_alloc_cols(uint32_t smem_dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_cols(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

// Bounded wait on an mbarrier phase; gives up when the budget expires or one of the CTA's abort words is set.
static __device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, long long budget, const volatile unsigned* ctl) {
  const long long t0 = clock64();
  for (unsigned it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 31u) == 0u && (ctl[kCtlAbort] != 0u || ctl[kCtlCtrlAbort] != 0u || clock64() - t0 > budget)) return false;
  }
}
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, const Params& p, const volatile unsigned* ctl) {
  return mbar_try_wait(bar, parity) || mbar_wait_slow(bar, parity, p.timeout_cycles, ctl);
}

__device__ __forceinline__ StreamBases stream_bases(const Params& p) {
  StreamBases b;
  b.qkv = reinterpret_cast<const unsigned char*>(p.qkv);
  b.o_proj = reinterpret_cast<const unsigned char*>(p.o_proj);
  b.up = reinterpret_cast<const unsigned char*>(p.up);
  b.gate = reinterpret_cast<const unsigned char*>(p.gate);
  b.down = reinterpret_cast<const unsigned char*>(p.down);
  b.lm_head = reinterpret_cast<const unsigned char*>(p.lm_head);
  return b;
}

// A control thread gives up: record why (first error wins), tell everyone.
__device__ __forceinline__ void ctrl_fail(const Params& p, volatile unsigned* ctl, int code, int warp, int ph, unsigned a, unsigned b) {
  if (ctl[kCtlAbort] == 0u && ctl[kCtlCtrlAbort] == 0u) report_error(p, code, warp, ph, a, b, 0);
  ctl[kCtlCtrlAbort] = 1u;
}

// ---- producer: one thread ---------------------------------------------------------------------
template <class S>
__device__ __forceinline__ void umma_producer(const Params& p, unsigned char* smem) {
  using L = SmemLayout<S>;
  constexpr int kSlices = S::I / kChunkElems;
  volatile unsigned* ctl = reinterpret_cast<volatile unsigned*>(smem + L::kOffCtl);
  const uint32_t ring = smem_u32(smem + L::kOffRing), bars = smem_u32(smem + L::kOffBars);
  const StreamBases wb = stream_bases(p);
  const uint64_t policy = l2_policy_evict_first();
  CtaRanges<S> R;
  R.init((int)blockIdx.x, (int)gridDim.x, p.vocab);
  unsigned n = 0;   // ring slots filled so far
  bool ok = true;
#pragma unroll 1
  for (int ph = p.phase_begin; ph < p.phase_end && ok; ++ph) {
    const int kind = phase_kind(ph, p.num_layers);
    if (kind == kAttn) continue;
    const int layer = phase_layer(ph), ng = R.groups(kind), nsl = kind == kDown ? kSlices : 1;
#pragma unroll 1
    for (int g = 0; g < ng && ok; ++g) {
#pragma unroll 1
      for (int j = 0; j < nsl; ++j, ++n) {
        const unsigned slot = n % kUSlots, use = n / kUSlots;
        if (use > 0 && !mbar_wait_bounded(bars + (kBarFree + slot) * 8, (use - 1) & 1u, p, ctl)) {
          ctrl_fail(p, ctl, kErrCopyWait, kWorkers, ph, n, slot);
          ok = false;
          break;
        }
        const uint32_t full = bars + (kBarFull + slot) * 8, dst = ring + slot * kGroupBytes;
        mbar_expect_tx(full, (uint32_t)(R.group_slots(kind, g) * kChunkBytes));
        for_each_group_copy<S>(wb, R, layer, kind, g, j, [&](uint32_t off, const unsigned char* src, uint32_t bytes) {
          bulk_g2s(dst + off, src, bytes, full, policy);
        });
      }
    }
  }
  if (!ok || ctl[kCtlAbort] != 0u || ctl[kCtlCtrlAbort] != 0u) {
    // leave no bulk copy in flight into this CTA's shared memory: wait (bounded) for the last fills
    const unsigned first = n > (unsigned)kUSlots ? n - kUSlots : 0u;
    for (unsigned m = first; m < n; ++m) {
      const uint32_t full = bars + (kBarFull + m % kUSlots) * 8;
      const long long t0 = clock64();
      while (!mbar_try_wait(full, (m / kUSlots) & 1u)) {
        if (clock64() - t0 > p.timeout_cycles) break;
      }
    }
  }
}

// ---- issuer: one thread -----------------------------------------------------------------------
template <class S>
__device__ __forceinline__ void umma_issuer(const Params& p, unsigned char* smem, uint32_t tmem) {
  using L = SmemLayout<S>;
  constexpr int kSlices = S::I / kChunkElems;
  volatile unsigned* ctl = reinterpret_cast<volatile unsigned*>(smem + L::kOffCtl);
  const uint32_t ring = smem_u32(smem + L::kOffRing), bars = smem_u32(smem + L::kOffBars);
  CtaRanges<S> R;
  R.init((int)blockIdx.x, (int)gridDim.x, p.vocab);
  unsigned n = 0, gcount = 0, sp = 0;   // slots consumed, groups issued, streaming phases entered
#pragma unroll 1
  for (int ph = p.phase_begin; ph < p.phase_end; ++ph) {
    const int kind = phase_kind(ph, p.num_layers);
    if (kind == kAttn) continue;
    // the workers have staged this phase's activations
    long long c_x = clock64(), c_full = 0, c_dfree = 0;
    if (!mbar_wait_bounded(bars + kBarXReady * 8, sp & 1u, p, ctl)) {
      ctrl_fail(p, ctl, kErrStageWait, kWorkers + 1, ph, sp, 0u);
      return;
    }
    ++sp;
    c_x = clock64() - c_x;
    const uint32_t x = smem_u32(smem + (kind == kDown ? L::kOffActD
                                                      : (small_buf_index(ph, p.num_layers) ? L::kOffActB : L::kOffActA)));
    const int ng = R.groups(kind), nsl = kind == kDown ? kSlices : 1;
#pragma unroll 1
    for (int g = 0; g < ng; ++g, ++gcount) {
      const unsigned b = gcount % kDBufs, duse = gcount / kDBufs;
      long long c0 = clock64();
      if (duse > 0 && !mbar_wait_bounded(bars + (kBarDFree + b) * 8, (duse - 1) & 1u, p, ctl)) {
        ctrl_fail(p, ctl, kErrStageWait, kWorkers + 1, ph, gcount, b);
        return;
      }
      const uint32_t d = tmem + b * kDCols;
      c_dfree += clock64() - c0;
#pragma unroll 1
      for (int j = 0; j < nsl; ++j, ++n) {
        const unsigned slot = n % kUSlots;
        c0 = clock64();
        if (!mbar_wait_bounded(bars + (kBarFull + slot) * 8, (n / kUSlots) & 1u, p, ctl)) {
          ctrl_fail(p, ctl, kErrCopyWait, kWorkers + 1, ph, n, slot);
          return;
        }
        c_full += clock64() - c0;
        tmem_fence_after_sync();
        const uint32_t a0 = ring + slot * kGroupBytes, x0 = x + j * kChunkBytes;
        // k-step s reads 256 bytes further into every chunk: the start-address field (16-byte units) grows by 16
        const uint64_t da = umma_desc(a0, 128, kChunkBytes), db = umma_desc(x0, 128, 128);
        umma_bf16(d, da, db, j != 0 ? 1u : 0u);
#pragma unroll
        for (int s = 1; s < kChunkBytes / 256; ++s) umma_bf16_add(d, da + 16u * s, db + 16u * s);
        umma_commit(bars + (kBarFree + slot) * 8);
      }
      umma_commit(bars + (kBarDReady + b) * 8);
    }
    if (p.trace != nullptr) {   // cycles the issuer waited in this phase: for the activations, the copies, a free accumulator
      unsigned long long* t = p.trace + ((size_t)blockIdx.x * num_phases(p.num_layers) + ph) * 8;
      t[0] = (unsigned long long)c_x;
      t[1] = (unsigned long long)c_full;
      t[4] = (unsigned long long)c_dfree;
    }
  }
}

// ---- workers ----------------------------------------------------------------------------------
// Value of this thread's slot of accumulator buffer b: valid in the lanes with lane % 8 == 0
// (slot 4 * (warp % 4) + lane / 8 of the group).  Returns false when the wait gave up.
template <class S>
__device__ __forceinline__ bool group_result(Worker<S>& s, const Params& p, unsigned char* smem, unsigned gc, float& v) {
  using L = SmemLayout<S>;
  const volatile unsigned* ctl = reinterpret_cast<const volatile unsigned*>(smem + L::kOffCtl);
  const uint32_t bars = smem_u32(smem + L::kOffBars);
  const unsigned b = gc % kDBufs;
  // (the answer must be the same in all lanes: the tensor-memory load below is warp-collective)
  if (!__all_sync(kFullMask, mbar_wait_bounded(bars + (kBarDReady + b) * 8, (gc / kDBufs) & 1u, p, ctl))) return false;
  tmem_fence_after_sync();
  uint32_t r[8];
  tmem_ld8(r, s.tmem + b * kDCols);
  tmem_wait_ld();
  tmem_fence_before_sync();
  if (s.lane == 0) mbar_arrive(bars + (kBarDFree + b) * 8);
  const int i = s.lane & 7;
  uint32_t pick = r[0];
#pragma unroll
  for (int j = 1; j < 8; ++j) pick = i == j ? r[j] : pick;
  v = __uint_as_float(pick);
  v += __shfl_xor_sync(kFullMask, v, 1);
  v += __shfl_xor_sync(kFullMask, v, 2);
  v += __shfl_xor_sync(kFullMask, v, 4);
  return true;
}

template <class S>
__device__ __forceinline__ void phase_stream(Worker<S>& s, const Params& p, unsigned char* smem, int ph, int kind,
                                             const CtaRanges<S>& R) {
  using L = SmemLayout<S>;
  const int layer = phase_layer(ph);
  const bool tagged = p.sync && (ph > p.phase_begin || p.wait_first);
  const unsigned tag_in = phase_tag(p, ph - 1);
  const unsigned tagw = phase_tag(p, ph) << 16;
  const bool normed = kind == kQkv || kind == kUpGate || kind == kLmHead;
  const int sbuf = small_buf_index(ph, p.num_layers);
  unsigned char* act = smem + (kind == kDown ? L::kOffActD : (sbuf ? L::kOffActB : L::kOffActA));
  float* sumsq = reinterpret_cast<float*>(smem + L::kOffCtl) + kCtlSumSq + sbuf * 8;
  const long long tq0 = clock64();

  // ---- stage this warp's eighth of the phase input (qmk_staging.cuh), then hand it to the issuer
  if (kind == kDown) {
    Part<S::I> part;
    if (!s.aborted) {
      if (fetch_part<S::I>(s, p, p.t_silu, p.silu_out, tagged, tag_in, ph, part)) store_part(part, act, s.w, s.lane);
      else flag_abort(s, smem);
    }
  } else {
    Part<S::H> part;
    uint2 gains[Part<S::H>::NPL];
    if (normed) {   // the gains do not depend on the step: fetch them before polling for the activations
      const uint16_t* gsrc = kind == kQkv ? p.attn_norm + (size_t)layer * S::H
                                          : (kind == kUpGate ? p.mlp_norm + (size_t)layer * S::H : p.lm_norm);
      const uint2* g2 = reinterpret_cast<const uint2*>(gsrc + s.w * Part<S::H>::kElems);
#pragma unroll
      for (int j = 0; j < Part<S::H>::NPL; ++j) gains[j] = __ldg(g2 + j * 32 + s.lane);
    }
    const uint32_t* tsrc = kind == kOproj ? p.t_attn : (kind == kUpGate ? p.t_hid_o : p.t_hid_d);
    const uint16_t* psrc = kind == kOproj ? p.attn_out
                                          : (kind == kQkv || (kind == kLmHead && p.num_layers == 0)
                                                 ? residual_src<S>(p, layer) : p.hidden);
    if (!s.aborted && !fetch_part<S::H>(s, p, tsrc, psrc, tagged, tag_in, ph, part)) flag_abort(s, smem);
    if (normed) {
      const float ss = s.aborted ? 0.f : part_sumsq(part);
      if (s.lane == 0) sumsq[s.w] = ss;
      cta_sync(s, smem);
      if (s.cta_abort) return;
      float tot = 0.f;
#pragma unroll
      for (int j = 0; j < kWorkers; ++j) tot += sumsq[j];
      normalise_part(part, gains, rsqrtf(tot * (1.0f / S::H) + p.eps));
    }
    if (!s.aborted) store_part(part, act, s.w, s.lane);
  }
  fence_proxy_async_smem();   // the tensor core reads the activations through the async proxy
  cta_sync(s, smem);
  if (s.cta_abort) return;
  if (s.w == 0 && s.lane == 0) mbar_arrive(smem_u32(smem + L::kOffBars) + kBarXReady * 8);
  const long long tq1 = clock64();
  if (kind == kQkv && !s.aborted) prefetch_attn_rows<S>(p, smem, layer, s.w, s.lane);

  // ---- epilogues of this CTA's groups
  const int ng = R.groups(kind), nslots = R.slots(kind);
  const bool pairs = kind == kQkv || kind == kUpGate;
  const uint16_t* res = kind == kOproj ? residual_src<S>(p, layer) : p.hidden;
  uint32_t* tres = kind == kOproj ? p.t_hid_o : p.t_hid_d;
  unsigned long long best = 0ull;
#pragma unroll 1
  for (int g = (s.w >> 2); g < ng && !s.aborted; g += 2) {
    float v = 0.f;
    const long long cw = clock64();
    if (g < 2 && s.w == 0) trace_put(p, ph, 7, 0ull, s.lane);
    if (!group_result(s, p, smem, s.groups_done + (unsigned)g, v)) {
      s.aborted = true;
      break;
    }
    if (g < 2 && s.w == 0) trace_put(p, ph, 7, (unsigned long long)(clock64() - cw), s.lane);
    const int sidx = g * kGroupRows + 4 * (s.w & 3) + (s.lane >> 3);   // slot of this thread in the phase
    const float partner = __shfl_down_sync(kFullMask, v, 8);           // the odd slot of a pair
    if (pairs) {
      if ((s.lane & 15) == 0 && sidx + 1 < nslots) {
        if (kind == kQkv) {
          epilogue_qkv<S>(p, smem, layer, R.a0 + (sidx >> 1), v, partner, tagw);
        } else {
          const int item = R.u0 + (sidx >> 1);
          const unsigned short bits = epilogue_silu(v, partner);
          p.silu_out[item] = bits;
          if (p.sync) st_handoff(p.t_silu + item, (uint32_t)bits | tagw);
        }
      }
    } else if ((s.lane & 7) == 0 && sidx < nslots) {
      if (kind == kLmHead) {
        const int row = R.l0 + sidx;
        const unsigned short bits = f32_to_bf16_bits(v);
        p.logits[row] = bits;
        const unsigned long long key = argmax_key(bits, row);
        best = key > best ? key : best;
      } else {
        // residual value of this thread's row: kept in a register from phase to phase for the
        // first group (the same thread owns the row in O-proj and down-proj of every layer)
        const int row = R.r0 + sidx;
        const float old = (g == 0 && s.res_valid) ? s.res : bf16_bits_to_f32(ldcg_u16(res + row));
        const unsigned short bits = f32_to_bf16_bits(old + bf16_round(v));
        p.hidden[row] = bits;
        if (p.sync) st_handoff(tres + row, (uint32_t)bits | tagw);
        if (g == 0) s.res = bf16_bits_to_f32(bits);
      }
    }
  }
  if (kind == kOproj || kind == kDown) s.res_valid = true;
  if (s.aborted) flag_abort(s, smem);
  s.groups_done += (unsigned)ng;
  // Push this warp's tagged stores out now (nothing waits for the fence itself; without it the stores
  // linger behind the polling loads and every consumer sees them about a microsecond later).
  flush_handoff();
  if (s.w == 0) {
    trace_put(p, ph, 3, (unsigned long long)(tq1 - tq0), s.lane);
    trace_put(p, ph, 6, (unsigned long long)(clock64() - tq1), s.lane);
  }
  if (kind != kLmHead) return;

  // LM head: warp -> CTA -> grid arg-max.  Every warp arrives, also those without rows.
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(kFullMask, best, o);
    best = other > best ? other : best;
  }
  if (s.lane == 0 && !s.aborted) {
    unsigned* ctl = reinterpret_cast<unsigned*>(smem + L::kOffCtl);
    unsigned long long* cta_key = reinterpret_cast<unsigned long long*>(ctl + kCtlKey);
    atomicMax(cta_key, best);
    __threadfence();
    if (atomicAdd(ctl + kCtlLmArrive, 1u) == (unsigned)(kWorkers - 1)) {
      const unsigned long long k = atomicMax(cta_key, 0ull);
      atomicMax(p.argmax_key, k);
      __threadfence();
      unsigned* lm_ticket = p.tickets + 64;
      if (atomicAdd(lm_ticket, 1u) == gridDim.x - 1) {
        __threadfence();
        const unsigned long long win = atomicMax(p.argmax_key, 0ull);
        const long long tok = (long long)(0xffffffffu - (unsigned)(win & 0xffffffffull));
        if (p.next_token) *p.next_token = tok;
        if (p.out_tokens && (long long)p.pos + 1 < p.out_tokens_len) p.out_tokens[p.pos + 1] = tok;
        *p.argmax_key = 0ull;
        *lm_ticket = 0u;
        __threadfence();
      }
    }
  }
}

}  // namespace qmk

#include "qmk_attention.cuh"

namespace qmk {

template <class S>
__device__ __forceinline__ void worker_main(const Params& p, unsigned char* smem, int w, int lane, uint32_t tmem) {
  Worker<S> s;
  s.lane = lane;
  s.w = w;
  s.nwt = (int)gridDim.x * kWorkers;
  s.g = (int)blockIdx.x * kWorkers + w;
  s.res = 0.f;
  s.res_valid = false;
  s.aborted = false;
  s.cta_abort = false;
  s.groups_done = 0;
  s.tmem = tmem + ((uint32_t)(32 * (w & 3)) << 16);
  CtaRanges<S> R;
  R.init((int)blockIdx.x, (int)gridDim.x, p.vocab);
#pragma unroll 1
  for (int ph = p.phase_begin; ph < p.phase_end && !s.cta_abort; ++ph) {
    if (w == 0) trace_put(p, ph, 2, globaltimer_ns(), lane);
    const int kind = phase_kind(ph, p.num_layers);
    if (kind == kAttn) {
      const unsigned f = phase_attn_call<S>(p, smem, ph, lane, w, s.aborted ? 1u : 0u);
      s.aborted = (f & 1u) != 0u;
      s.cta_abort = (f & 2u) != 0u;
    }
    else phase_stream(s, p, smem, ph, kind, R);
    if (w == 0) trace_put(p, ph, 5, globaltimer_ns(), lane);
  }
}

template <class S>
__global__ void __launch_bounds__(kLaunchThreads, 1) qmk_decode_kernel(const __grid_constant__ Params p) {
  extern __shared__ __align__(128) unsigned char smem[];
  using L = SmemLayout<S>;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned long long t_entry = globaltimer_ns();
  unsigned* ctl = reinterpret_cast<unsigned*>(smem + L::kOffCtl);
  if (threadIdx.x == 0) {
    const uint32_t bars = smem_u32(smem + L::kOffBars);
    for (int i = 0; i < kNumBars; ++i) mbar_init(bars + i * 8, (i >= kBarDFree && i < kBarDFree + kDBufs) ? 4u : 1u);
    fence_barrier_init();
  }
  if (warp == 0) {
    ctl[lane] = 0u;                                    // flags, arrival count, arg-max key, partial sums
    // cos / sin of this step's position: read by the QKV epilogues of every layer.
    float* rope = reinterpret_cast<float*>(smem + L::kOffRope);
    for (int i = lane; i < S::HD; i += 32) {
      rope[i] = __ldg(p.rope_cos + (size_t)p.pos * S::HD + i);
      rope[S::HD + i] = __ldg(p.rope_sin + (size_t)p.pos * S::HD + i);
    }
  }
  __syncthreads();   // (the control words are zeroed before the allocation writes its address among them)
  if (warp == 0) {
    tmem_alloc_cols(smem_u32(ctl + kCtlTmem), kTmemCols);
    tmem_fence_before_sync();
  }
  __syncthreads();
  tmem_fence_after_sync();
  const uint32_t tmem = reinterpret_cast<const volatile uint32_t*>(ctl)[kCtlTmem];
  if (warp < kWorkers) {
    worker_main<S>(p, smem, warp, lane, tmem);
  } else if (lane == 0) {
    if (warp == kWorkers) umma_producer<S>(p, smem);
    else umma_issuer<S>(p, smem, tmem);
  }
  __syncwarp();
  if (p.trace != nullptr && lane == 0 && warp < kWorkers) {   // kernel entry / exit of this CTA, kept in the slots of the first phase
    unsigned long long* t = p.trace + ((size_t)blockIdx.x * num_phases(p.num_layers) + p.phase_begin) * 8;
    atomicMax(t + 3, ~t_entry);
    atomicMax(t + 7, globaltimer_ns());
  }
  // every role is done with the tensor memory (the issuer's last commit was waited for by the workers,
  // or the CTA is aborting): the allocating warp frees it
  tmem_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tmem_fence_after_sync();
    tmem_dealloc_cols(tmem, kTmemCols);
  }
}

}  // namespace qmk
