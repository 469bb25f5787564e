// Device code of the batched decode megakernel (roles, epilogues, attention, the kernel itself).
//
// NOT a stand-alone header: qmk_batch_kernel.cuh includes this file TWICE, inside namespace qmkb::plain with
// kTraceOn = false and inside qmkb::traced with kTraceOn = true, so that the library holds the kernel without any of the
// optional timeline's code (the kernel sits at its register cap: with the trace code compiled in but switched off it was
// measured 3.5-4 % slower) and, for qmk_set_trace, the kernel with it.

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
// Split-K partial tiles meet in a FIXED-POINT accumulator at L2.  fp32 additions in arrival order would make the last bit
// of a sum depend on timing; 64-bit integer additions are associative, so the sum of the partials -- each rounded once to
// a multiple of 2^-36, finer than fp32 resolves above 2^-12 -- is the same whatever order they arrive in, and two runs
// of a step give the same bits.
constexpr float kFixScale = 68719476736.0f;              // 2^36
constexpr float kFixInv = 1.0f / 68719476736.0f;       // (a power of two: the product is exact)
__device__ __forceinline__ long long to_fixed(float v) { return __float2ll_rn(v * kFixScale); }
__device__ __forceinline__ void red_add_s64(long long* addr, long long v) {
  asm volatile("red.relaxed.gpu.global.add.u64 [%0], %1;" ::"l"(addr), "l"(v) : "memory");
}
// Reads an accumulator and leaves zero for its next user, in one operation at L2.  (Plain loads followed by stores of
// zero were measured equal.)
__device__ __forceinline__ long long exch_zero_s64(long long* addr) {
  long long old;
  asm volatile("atom.relaxed.gpu.global.exch.b64 %0, [%1], %2;" : "=l"(old) : "l"(addr), "l"(0ll) : "memory");
  return old;
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

// Optional timeline (qmk_set_trace), sixteen 64-bit slots per (CTA, phase), globaltimer ns: 0 the phase's dependency is
// satisfied (stagers / attention), 1 the CTA's first accumulator of the phase is complete, 2 the epilogue group enters
// the phase, 5 the CTA arrives at the phase's counter.  Cycle sums over the phase's units: 3 / 4 the issuer waiting for
// the weights / the activations of a unit; 6 / 7 stager warp 0 waiting for a free slot / from there to its arrival 8 the issuer
// waiting for a free accumulator, 9 issuing a unit's four MMAs, 10 the commits.  The CTA's LAST tile part: 11 stamp of its
// accumulator complete, then cycle counts: 12 part read out of tensor memory, 13 count released (owner: all parts counted),
// 14 sum read back, 15 tile epilogue (14 / 15 only on the CTA that finishes the tile).  (Stamps inside the epilogue
// path were measured to cost a fifth of the step at 64 rows when compiled into the untraced kernel: it sits at its
// register cap, so they exist in the traced build only.)
__device__ __forceinline__ void trace_put(const BParams& p, int ph, int slot) {
  if ((kTraceOn && p.trace != nullptr)) p.trace[((size_t)blockIdx.x * (size_t)num_phases(p) + ph) * kTraceSlots + slot] = globaltimer_ns();
}

__device__ __forceinline__ void trace_val(const BParams& p, int ph, int slot, unsigned long long v) {
  if ((kTraceOn && p.trace != nullptr)) p.trace[((size_t)blockIdx.x * (size_t)num_phases(p) + ph) * kTraceSlots + slot] = v;
}

// Byte offset of the 16-byte piece that holds (batch row b, column col) in an activation image: k-block col / 64, then
// [Bpad rows][128 bytes] with the eight 16-byte pieces of a row swizzled by the row, as the tensor core reads a ring slot.
__device__ __forceinline__ size_t img_piece(int Bpad, int b, int col) {
  return (size_t)(col >> 6) * (size_t)(Bpad * 128) + (size_t)(b * 128 + ((((col & 63) >> 3) ^ (b & 7)) << 4));
}

struct Ctx {
  const BParams* p;
  unsigned char* smem;
  volatile unsigned* ctl;
  uint32_t bars;     // shared address of the mbarriers
  int warp, lane;
  __device__ __forceinline__ uint32_t a_full(int s) const { return bars + s * 8; }
  __device__ __forceinline__ uint32_t b_full(int s) const { return bars + s * 8; }   // (the same barrier)
  __device__ __forceinline__ uint32_t empty(int s) const { return bars + (2 * kMaxStages + (s >> 1)) * 8; }
  __device__ __forceinline__ uint32_t acc_full(int b) const { return bars + (3 * kMaxStages + b) * 8; }
  __device__ __forceinline__ uint32_t acc_empty(int b) const { return bars + (3 * kMaxStages + 2 + b) * 8; }
  __device__ __forceinline__ bool aborted() const { return ctl[kCAbort] != 0u; }
};

// A try_wait that lets the hardware park the thread for up to `ns` nanoseconds (it returns at once when the phase
// completes).  Without the hint the issuing and the producing thread spin through a phase's tail and take issue slots
// from the epilogue warps on their schedulers: 2 % of the step.
__device__ __forceinline__ uint32_t mbar_try_wait_parked(uint32_t bar, uint32_t parity, uint32_t ns) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(ns)
      : "memory");
  return ok;
}

// Bounded wait on an mbarrier phase.  False when the budget expired or the CTA is aborting.
static __device__ __noinline__ bool mbar_wait_slow(const Ctx& c, uint32_t bar, uint32_t parity, int phase, int detail) {
  if (c.ctl[kCAbort] != 0u) return false;
  const long long t0 = clock64();
  for (unsigned it = 1;; ++it) {
    if (mbar_try_wait_parked(bar, parity, 4000u)) return true;
    if ((it & 63u) == 0u) {
      if (c.ctl[kCAbort] != 0u) return false;
      // (twice the budget of a dependency wait: these waits sit downstream of one, which should be the one to report)
      if (clock64() - t0 > 2 * c.p->timeout_cycles) {
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

// Bounded wait until `*counter` reaches `target` (arrivals of all CTAs at the end of a phase).
static __device__ __noinline__ bool counter_wait(const Ctx& c, const unsigned* counter, unsigned target, int phase) {
  if (c.ctl[kCAbort] != 0u) return false;
  const long long t0 = clock64();
  for (unsigned it = 1;; ++it) {
    // Polled with relaxed loads, one acquire load at the end: acquire loads in a tight loop from
    // three threads of a CTA slowed the warps of the same SM that were still working (the router's epilogue took 60 us
    // with them, 20 us without).
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

// Number of distinct experts of this step, for the two expert phases of a MoE layer: valid once every CTA has finished
// the layer's router phase (one thread calls this; 0 after a wait that gave up).
static __device__ __noinline__ int expert_count(const Ctx& c, int ph) {
  const BParams& p = *c.p;
  const int rph = phase_layer(p, ph) * p.ppl + 3;
  if (rph >= p.phase_begin && !counter_wait(c, p.phase_done + 1 + rph, gridDim.x, ph)) return 0;
  return (int)ld_acquire_gpu(reinterpret_cast<const unsigned*>(p.moe_ne));
}
__device__ __forceinline__ bool is_expert_kind(int kind) { return kind == kEUpGate || kind == kEDown; }

// ------------------------------------------------------------------------------------------------
// producer (one thread)
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void producer(const Ctx& c, const TensorMaps& maps, unsigned& n_issued) {
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
    const CUtensorMap* map = kind == kQkv ? &maps.qkv : kind == kOproj ? &maps.o_proj : kind == kUpGate ? &maps.up
                           : kind == kDown ? &maps.down : kind == kRouter ? &maps.router : &maps.lm_head;
    const int per = p.Ie > 0 ? p.Ie / kBlockK : 1;   // 64-row tiles (k-blocks) of one expert
    int t = d.KB > 0 ? lo / d.KB : 0, kb = lo - t * d.KB;
    int zslot = -1, zval = 0;   // expert phases: the selected expert's index is fetched when the slot changes
    auto expert_z = [&](int slot) {
      if (slot != zslot) { zslot = slot; zval = layer * (p.E / p.ep_world) + __ldcg(p.moe_elist + slot); }   // (E / ep_world experts per layer on this rank)
      return zval;
    };
#pragma unroll 1
    for (int u = lo; u < hi; ++u, ++n) {
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
  n_issued = n;
}

// ------------------------------------------------------------------------------------------------
// issuer (one thread)
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void issuer(const Ctx& c, uint32_t tmem) {
  const BParams& p = *c.p;
  const uint32_t stages = smem_u32(c.smem + p.off_stages);
  const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (((uint32_t)p.Bpad >> 3) << 17) | ((128u >> 4) << 24);
  const int G = (int)gridDim.x, cta = (int)blockIdx.x;
  unsigned n = 0, sg = 0;
  const bool tr = (kTraceOn && p.trace != nullptr);
#pragma unroll 1
  for (int ph = p.phase_begin; ph < p.phase_end; ++ph) {
    const int kind = phase_kind(p, ph);
    if (kind == kAttn) continue;
    const PhaseDims d = phase_dims(p, kind, is_expert_kind(kind) ? expert_count(c, ph) : 0);
    int lo, hi;
    unit_range(d.T * d.KB, phase_ctas(kind, d.T * d.KB, G), cta, lo, hi);
    int kb = d.KB > 0 ? lo % d.KB : 0;
    bool seg_start = true;
    long long w_a = 0, w_b = 0, w_acc = 0, w_mma = 0, w_commit = 0;
#pragma unroll 1
    for (int u = lo; u < hi; ++u, ++n) {
      const unsigned buf = sg & 1u;
      const long long ta = tr ? clock64() : 0;
      if (seg_start && sg >= 2u && !mbar_wait(c, c.acc_empty(buf), ((sg >> 1) - 1u) & 1u, ph, 2)) return;
      const int s = (int)(n & (unsigned)(kStages - 1));
      const unsigned par = (n / (unsigned)kStages) & 1u;
      const long long t0 = tr ? clock64() : 0;
      w_acc += t0 - ta;
      if (!mbar_wait(c, c.a_full(s), par, ph, 3)) return;
      const long long t1 = tr ? clock64() : 0;
      w_a += t1 - t0;
      const long long t2 = tr ? clock64() : 0;
      w_b += t2 - t1;
      tmem_fence_after_sync();
      const uint64_t da = desc_sw128(stages + s * p.stage_bytes), db = desc_sw128(stages + s * p.stage_bytes + kABytes);
      const uint32_t dcol = tmem + buf * (uint32_t)p.Bpad;
      // (k-step k reads 32 bytes further along K: the start-address field grows by 2)
      if (seg_start) mma_bf16_set(dcol, da, db, idesc);
      else mma_bf16_add(dcol, da, db, idesc);
#pragma unroll
      for (int k = 1; k < kBlockK / 16; ++k) mma_bf16_add(dcol, da + 2u * k, db + 2u * k, idesc);
      const long long t3 = tr ? clock64() : 0;
      if (n & 1u) mma_commit(c.empty(s));   // frees this slot and the one before it
      seg_start = false;
      if (++kb == d.KB || u + 1 == hi) {
        mma_commit(c.acc_full(buf));
        ++sg;
        kb = kb == d.KB ? 0 : kb;
        seg_start = true;
      }
      if (tr) { const long long t4 = clock64(); w_mma += t3 - t2; w_commit += t4 - t3; }
    }
    trace_val(p, ph, 3, (unsigned long long)w_a);
    trace_val(p, ph, 4, (unsigned long long)w_b);
    trace_val(p, ph, 8, (unsigned long long)w_acc);
    trace_val(p, ph, 9, (unsigned long long)w_mma);
    trace_val(p, ph, 10, (unsigned long long)w_commit);
  }
}

// ------------------------------------------------------------------------------------------------
// stagers (128 threads): activation operand of every unit
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ bool phase_dependency(const Ctx& c, int ph, bool& needed) {
  // what must have finished before phase ph reads its input: the phase before it, or the prologue
  const BParams& p = *c.p;
  needed = true;
  if (ph > p.phase_begin) return counter_wait(c, p.phase_done + ph, gridDim.x, ph);          // counter of phase ph - 1
  if (p.prologue != 0) return counter_wait(c, p.phase_done + 0, gridDim.x, ph);
  if (p.wait_first) return counter_wait(c, p.phase_done + (ph > 0 ? ph : num_phases(p) + 1), gridDim.x, ph);
  needed = false;
  return true;
}

// Stages the activation operand of units [lo, hi).  A warp takes D consecutive units at a time (the four warps
// round-robin over groups of D) and a lane has NPL 16-byte pieces per unit: all D * NPL <= 16 loads of a group are
// issued before the first is used, so that a warp pays one L2 round trip per group, not per unit or per piece.
// 5 * D - 1 must stay below twice the number of ring slots: a warp that got two laps of the ring ahead of the tensor core would take an
// old completion of a stage's mbarrier (same parity) for the one it waits for.
template <int NPL, int D>
__device__ __forceinline__ void stage_units(const Ctx& c, int ph, const PhaseDims& d, int lo, int hi, int st, unsigned n,
                                            const uint16_t* src, const uint16_t* gain, float* rs,
                                            unsigned char* img = nullptr) {
  // gain != nullptr: a normalised phase.  The rsqrt factors rs[Bpad] are computed here, by the threads st < Bpad from the
  // previous phase's partial sums of squares, AFTER every warp has issued the loads of its first group: one L2 round
  // trip for both.  All 128 stager threads call this function then (it contains one barrier of the group).
  // img != nullptr (router phase): the staged block of every unit is also stored, in the same swizzled layout, as
  // k-block u % KB of a global image [KB][Bpad * 128 bytes] that the expert up/gate phase fetches with bulk copies
  static_assert(4 * D + D - 1 < 2 * kMinStages, "a stager warp could run two ring laps ahead");
  const BParams& p = *c.p;
  const int sw = st >> 5, lane = st & 31;
  const int chunk = lane & 7;         // 16-byte piece inside the 128-byte k-block row
  const int row0 = lane >> 3;         // first batch row of this lane (then +4, +8, ...)
  long long w_slot = 0, w_fill = 0;
  const bool tr = (kTraceOn && p.trace != nullptr);
  bool need_rs = gain != nullptr;
  auto compute_rs = [&]() {
    if (st < p.Bpad) {
      float tot = 0.f;
      const int nt = (p.H + kTileRows - 1) / kTileRows;
      for (int t0 = 0; t0 < nt; t0 += 16) {   // sixteen partial sums per round trip, added in tile order
        float x[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) x[j] = t0 + j < nt ? ldcg_f32(p.ss + (t0 + j) * kMaxBatch + st) : 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) tot += x[j];
      }
      rs[st] = rsqrtf(tot / (float)p.H + p.eps);
    }
    named_bar(kBarStg, 128);
  };
#pragma unroll 1
  for (int base = lo + sw * D; base < hi; base += 4 * D) {
    uint4 v[D][NPL];
    uint4 g4[D];
#pragma unroll
    for (int j = 0; j < D; ++j) {
      const int u = base + j;
      const int kbu = u < hi ? u % d.KB : 0;
      const int k0 = kbu * kBlockK + chunk * 8;
      g4[j] = make_uint4(0, 0, 0, 0);
      if (gain != nullptr && u < hi) g4[j] = __ldg(reinterpret_cast<const uint4*>(gain + k0));
#pragma unroll
      for (int i = 0; i < NPL; ++i) {
        const int r = row0 + 4 * i;
        v[j][i] = make_uint4(0, 0, 0, 0);
        if (u < hi && r < p.B) v[j][i] = ldcg_u4(src + (size_t)r * d.K + k0);
      }
    }
    if (need_rs) {   // (first group of this warp: its loads are in flight)
      need_rs = false;
      compute_rs();
    }
#pragma unroll
    for (int j = 0; j < D; ++j) {
      const int u = base + j;
      if (u >= hi) break;
      const unsigned nu = n + (unsigned)(u - lo);
      const int s = (int)(nu & (unsigned)(kStages - 1));
      const long long t0 = tr ? clock64() : 0;
      const bool ok = nu < (unsigned)kStages || mbar_wait(c, c.empty(s), ((nu / (unsigned)kStages) - 1u) & 1u, ph, 5);
      const long long t1 = tr ? clock64() : 0;
      w_slot += t1 - t0;
      if (!ok) continue;
      unsigned char* dst = c.smem + p.off_stages + s * p.stage_bytes + kABytes;
      unsigned char* gdst = img != nullptr ? img + (size_t)(u % d.KB) * (size_t)(p.Bpad * 128) : nullptr;
      const uint32_t* gw = reinterpret_cast<const uint32_t*>(&g4[j]);
#pragma unroll
      for (int i = 0; i < NPL; ++i) {
        const int r = row0 + 4 * i;
        if (gain != nullptr && r < p.B) {
          const float f = rs[r];
          uint32_t* w = reinterpret_cast<uint32_t*>(&v[j][i]);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float a = bf16_round(bf_lo(w[q]) * f) * bf_lo(gw[q]);
            const float b = bf16_round(bf_hi(w[q]) * f) * bf_hi(gw[q]);
            w[q] = pack_bf16x2(a, b);
          }
        }
        const int off = r * 128 + ((chunk ^ (r & 7)) << 4);
        *reinterpret_cast<uint4*>(dst + off) = v[j][i];
        if (gdst != nullptr) *reinterpret_cast<uint4*>(gdst + off) = v[j][i];
      }
      if (gdst != nullptr) __threadfence();   // the image is read by other CTAs once this phase's counter is complete
      fence_async_smem();
      mbar_arrive1(c.b_full(s));
      if (tr) w_fill += clock64() - t1;
    }
  }
  if (need_rs) compute_rs();   // a warp without units in this phase still takes part in the barrier
  if (st == 0) {
    trace_val(p, ph, 6, (unsigned long long)w_slot);
    trace_val(p, ph, 7, (unsigned long long)w_fill);
  }
}

// Activation operand of units [lo, hi) from a global image [KB][Bpad * 128 bytes] that already has the layout of a ring
// slot's activation half: one bulk copy per unit, issued by lane 0 of the warp that owns the unit (units are dealt to the
// four warps round-robin), completing on the slot's b_full barrier together with the 32 arrivals of the warp.
__device__ __forceinline__ void stage_images(const Ctx& c, int ph, const PhaseDims& d, int lo, int hi, int st, unsigned n,
                                             const unsigned char* img) {
  const BParams& p = *c.p;
  const int sw = st >> 5, lane = st & 31;
  const uint32_t bytes = (uint32_t)p.Bpad * 128u;
  // the image was written with ordinary stores by other CTAs (seen through the phase counter): order them before this
  // thread's bulk copies, which read through the async proxy
  asm volatile("fence.proxy.async;" ::: "memory");
  long long w_slot = 0;
  const bool tr = (kTraceOn && p.trace != nullptr);
#pragma unroll 1
  for (int u = lo + sw; u < hi; u += 4) {
    const unsigned nu = n + (unsigned)(u - lo);
    const int s = (int)(nu & (unsigned)(kStages - 1));
    const long long t0 = tr ? clock64() : 0;
    const bool ok = nu < (unsigned)kStages || mbar_wait(c, c.empty(s), ((nu / (unsigned)kStages) - 1u) & 1u, ph, 5);
    if (tr) w_slot += clock64() - t0;
    if (!ok) continue;
    if (lane == 0) {
      const uint32_t dst = smem_u32(c.smem + p.off_stages + s * p.stage_bytes + kABytes);
      const unsigned char* g = img + (size_t)(u % d.KB) * bytes;
      asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(c.b_full(s)), "r"(bytes) : "memory");
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                   "l"(g), "r"(bytes), "r"(c.b_full(s))
                   : "memory");
    }
    __syncwarp();
    mbar_arrive1(c.b_full(s));
  }
  if (st == 0) {
    trace_val(p, ph, 6, (unsigned long long)w_slot);
  }
}

__device__ __forceinline__ void stage_phase(const Ctx& c, int ph, int kind, int st, unsigned& n) {
  // st: thread index inside the stager group, 0..127
  const BParams& p = *c.p;
  const int layer = phase_layer(p, ph);
  if (st == 0) {
    bool needed;
    const bool ok = phase_dependency(c, ph, needed);
    (void)ok;
    if (is_expert_kind(kind)) c.ctl[kCNeStg] = (unsigned)expert_count(c, ph);
    trace_put(p, ph, 0);
  }
  named_bar(kBarStg, 128);
  const PhaseDims d = phase_dims(p, kind, is_expert_kind(kind) ? (int)c.ctl[kCNeStg] : 0);
  int lo, hi;
  unit_range(d.T * d.KB, phase_ctas(kind, d.T * d.KB, (int)gridDim.x), (int)blockIdx.x, lo, hi);
  // Where the operand comes from.  Expert phases: images (the normalised residual stream stored by the router phase's
  // stagers; SiLU(gate) * up times the router weight stored by the expert up/gate epilogue).  O-proj and down-proj: the
  // image the attention / up-gate phase stored beside its plain output, when that phase ran in this launch.  Normalised
  // phases with enough work per k-block (wide batches; the LM head when a CTA walks the k-blocks more than once): an
  // image built by a pre-pass, CTA i normalising k-block i, behind one more grid-wide counter.  Else: staged per unit.
  const bool expert = is_expert_kind(kind);
  const bool plain_img = (kind == kOproj || kind == kDown) && ph > p.phase_begin && p.dense_img != 0;
  const bool normed = phase_normed(kind) && !expert;
  const int KBx = p.H / kBlockK;
  const bool pre = normed && kind != kRouter && p.H % kBlockK == 0 &&
                   (kind == kLmHead ? (d.T * d.KB) / (int)gridDim.x >= p.pre_lm_units : p.Bpad >= p.pre_bpad);   // (the same on every CTA)
  float* rs = reinterpret_cast<float*>(c.smem + Smem::kOffRs);
  const uint16_t* src = kind == kOproj ? p.attn_out : kind == kDown ? p.silu_out : p.hidden;
  const uint16_t* gain = kind == kQkv ? p.attn_norm + (size_t)layer * p.H
                       : kind == kLmHead ? p.lm_norm : p.mlp_norm + (size_t)layer * p.H;
  if (pre) {
    // CTA i normalises k-block i (only these CTAs need the rsqrt factors, computed while the block's rows are in flight);
    // every CTA, also one without units in this phase, then waits for all k-blocks.
    const int chunk = st & 7;
    bool need_rs = true;
    for (int kb = (int)blockIdx.x; kb < KBx; kb += (int)gridDim.x) {
      const int k0 = kb * kBlockK + chunk * 8;
      const uint4 g4 = __ldg(reinterpret_cast<const uint4*>(gain + k0));
      const uint32_t* gw = reinterpret_cast<const uint32_t*>(&g4);
      uint4 v[kMaxBatch / 16];
#pragma unroll
      for (int i = 0; i < kMaxBatch / 16; ++i) {
        const int r = (st >> 3) + 16 * i;
        v[i] = make_uint4(0, 0, 0, 0);
        if (r < p.B) v[i] = ldcg_u4(src + (size_t)r * p.H + k0);
      }
      if (need_rs) {
        need_rs = false;
        if (st < p.Bpad) {
          float tot = 0.f;
          const int nt = (p.H + kTileRows - 1) / kTileRows;
          for (int t0 = 0; t0 < nt; t0 += 16) {   // sixteen partial sums per round trip, added in tile order
            float x[16];
#pragma unroll
            for (int j2 = 0; j2 < 16; ++j2) x[j2] = t0 + j2 < nt ? ldcg_f32(p.ss + (t0 + j2) * kMaxBatch + st) : 0.f;
#pragma unroll
            for (int j2 = 0; j2 < 16; ++j2) tot += x[j2];
          }
          rs[st] = rsqrtf(tot / (float)p.H + p.eps);
        }
        named_bar(kBarStg, 128);
      }
#pragma unroll
      for (int i = 0; i < kMaxBatch / 16; ++i) {
        const int r = (st >> 3) + 16 * i;
        if (r < p.Bpad) {
          if (r < p.B) {
            const float f = rs[r];
            uint32_t* w = reinterpret_cast<uint32_t*>(&v[i]);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float a = bf16_round(bf_lo(w[q]) * f) * bf_lo(gw[q]);
              const float b = bf16_round(bf_hi(w[q]) * f) * bf_hi(gw[q]);
              w[q] = pack_bf16x2(a, b);
            }
          }
          *reinterpret_cast<uint4*>(p.ximg + img_piece(p.Bpad, r, k0)) = v[i];
        }
      }
      named_bar(kBarStg, 128);   // the group's stores, then one release on the count (cumulative over the barrier)
      if (st == 0) red_release_gpu_add(p.img_done + ph, 1u);
    }
    if (st == 0) counter_wait(c, p.img_done + ph, (unsigned)KBx, ph);
    named_bar(kBarStg, 128);
  }
  const uint16_t* gn = normed ? gain : nullptr;
  if (expert || plain_img || pre) {
    if (hi > lo) {
      const unsigned char* img = kind == kEDown ? p.eimg : kind == kOproj ? p.aimg : kind == kDown ? p.simg : p.ximg;
      stage_images(c, ph, d, lo, hi, st, n, img);
    }
  } else if (hi > lo || gn != nullptr) {   // (a normalised phase: every stager thread takes part in the rsqrt barrier)
    unsigned char* img = kind == kRouter ? p.ximg : nullptr;
    switch (p.Bpad) {
      case 16: stage_units<4, 2>(c, ph, d, lo, hi, st, n, src, gn, rs, img); break;
      case 32: stage_units<8, 2>(c, ph, d, lo, hi, st, n, src, gn, rs, img); break;
      case 48: stage_units<12, 1>(c, ph, d, lo, hi, st, n, src, gn, rs, img); break;
      default: stage_units<16, 1>(c, ph, d, lo, hi, st, n, src, gn, rs, img); break;
    }
  }
  n += (unsigned)(hi - lo);
}

// ------------------------------------------------------------------------------------------------
// epilogues (128 threads, e = thread index in the group) on the fp32 tile exch[128][65]
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ unsigned short silu_mul(float up, float gate) {
  // fused_mlp_upgate (operations.py:265-282): both products rounded to bf16, SiLU rounded, product rounded
  // (the quotient is rounded to bf16 right away: the approximate division differs from the exact one in the last fp32
  // bits only, and unlike it is branch-free, so eight of these interleave in the epilogue; the reference builds its kernels
  // with --use_fast_math: .../A100/multi_batch/decode_kernel/Makefile:39)
  const float g = bf16_round(gate);
  const float sl = bf16_round(__fdividef(g, 1.0f + __expf(-g)));
  return f32_to_bf16_bits(sl * bf16_round(up));
}
__device__ __forceinline__ unsigned long long argmax_key(unsigned short bits, int row) {
  return ((unsigned long long)float_ordered_bits(bf16_bits_to_f32(bits)) << 32) | (0xffffffffu - (unsigned)row);
}

// Expert parallelism: the finished partial tile of this rank (exch, row tile t of the expert down-projection) is stored
// into this rank's slot of every peer's exchange buffer, a flag with the tag of (launch, layer) follows after a
// system-scope fence, then the flags of the other ranks are awaited in THIS rank's buffer (bounded) and the slots are added
// in rank order -- the same order on every rank, so all ranks hold the same bits afterwards.  128 threads, e = tile row.
static __device__ __noinline__ void ep_exchange(const Ctx& c, int ph, int t, int e, int which) {
  const BParams& p = *c.p;
  float* exch = reinterpret_cast<float*>(c.smem + Smem::kOffExch);
  const int W = p.x_world, me = p.x_rank, layer = phase_layer(p, ph);
  const int T = (p.H + kTileRows - 1) / kTileRows;
  // Exchanges are numbered over the launches (all ranks launch in lockstep); the number is the flag's tag and its low
  // bit picks one of two buffers, so a rank that runs one exchange ahead never overwrites a tile a peer still reads.
  const unsigned seq = (p.epoch * (unsigned)p.num_layers + (unsigned)layer) * (unsigned)p.x_per_layer + (unsigned)which;
  const unsigned tag = seq + 1u;
  const int par = (int)(seq & 1u);
  const size_t tile_f = (size_t)kTileRows * p.Bpad;
  const size_t fidx = (size_t)(par * W + me) * T + t;                  // my slot in a peer's buffer
  for (int d = 0; d < W; ++d) {
    if (d == me) continue;
    float4* dst = reinterpret_cast<float4*>(p.ep_buf[d] + fidx * tile_f + (size_t)e * p.Bpad);
    for (int q = 0; q < p.Bpad / 4; ++q)
      dst[q] = make_float4(exch[e * p.exch_stride + 4 * q], exch[e * p.exch_stride + 4 * q + 1],
                           exch[e * p.exch_stride + 4 * q + 2], exch[e * p.exch_stride + 4 * q + 3]);
  }
  // (no fence per thread: the barrier orders the group's peer stores before the publishing thread's release at system
  // scope, which is cumulative over what the barrier made visible to it)
  named_bar(kBarEpi, 128);
  if (e < W && e != me) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.ep_flag[e] + fidx), "r"(tag) : "memory");
    // wait for rank e's tile in my own buffer
    const unsigned* flag = p.ep_flag[me] + (size_t)(par * W + e) * T + t;
    const long long t0 = clock64();
    for (unsigned it = 1;; ++it) {
      unsigned v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
      if (v == tag) break;
      if ((it & 15u) == 0u) {
        if (c.ctl[kCAbort] != 0u) break;
        if (clock64() - t0 > c.p->timeout_cycles) {
          report(p, kErrCounterWait, c.warp, ph, v, tag, 32 + e);
          c.ctl[kCAbort] = 1u;
          break;
        }
      }
    }
  }
  named_bar(kBarEpi, 128);
  if (c.ctl[kCAbort] == 0u) {
    for (int q = 0; q < p.Bpad / 4; ++q) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int s = 0; s < W; ++s) {
        float4 v;
        if (s == me) {
          v = make_float4(exch[e * p.exch_stride + 4 * q], exch[e * p.exch_stride + 4 * q + 1],
                          exch[e * p.exch_stride + 4 * q + 2], exch[e * p.exch_stride + 4 * q + 3]);
        } else {
          v = __ldcg(reinterpret_cast<const float4*>(p.ep_buf[me] + ((size_t)(par * W + s) * T + t) * tile_f +
                                                     (size_t)e * p.Bpad) + q);
        }
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
      exch[e * p.exch_stride + 4 * q] = acc.x; exch[e * p.exch_stride + 4 * q + 1] = acc.y;
      exch[e * p.exch_stride + 4 * q + 2] = acc.z; exch[e * p.exch_stride + 4 * q + 3] = acc.w;
    }
  }
  named_bar(kBarEpi, 128);
}

__device__ __forceinline__ void epilogue_tile(const Ctx& c, int ph, int kind, int t, int e) {
  const BParams& p = *c.p;
  float* exch = reinterpret_cast<float*>(c.smem + Smem::kOffExch);
  const int* pos_s = reinterpret_cast<const int*>(c.smem + Smem::kOffPos);
  const int* act_s = reinterpret_cast<const int*>(c.smem + Smem::kOffAct);
  const int* slot_s = reinterpret_cast<const int*>(c.smem + Smem::kOffSlot);
  const int layer = phase_layer(p, ph);
  const int B = p.B;
  switch (kind) {
    case kQkv: {
      // A thread owns (sequence b, eight consecutive rows): four RoPE pairs of one head of Q, K or V.  Everything it
      // reads or writes in global memory is a 16-byte piece; lanes 0-15 / 16-31 of a warp hold the sixteen row
      // groups of one sequence, so the per-head sums of squares of the Q/K norm are warp shuffles.
      const int rg = e & 15;
      const int row = t * kTileRows + rg * 8;
      const int kdim = p.NKV * p.HD;
      const bool in_range = row < p.QKV_ROWS;
      const bool is_v = row >= p.QDIM + kdim;
      const bool is_k = !is_v && row >= p.QDIM;
      const int d0 = row % p.HD;
      const uint16_t* nw = (is_v || !in_range) ? nullptr : (is_k ? p.k_norm : p.q_norm);
      float wn[8];
      if (nw != nullptr) {
        const uint4 w4 = __ldg(reinterpret_cast<const uint4*>(nw + (size_t)layer * p.HD + d0));
        const uint32_t* ww = reinterpret_cast<const uint32_t*>(&w4);
#pragma unroll
        for (int j = 0; j < 4; ++j) { wn[2 * j] = bf_lo(ww[j]); wn[2 * j + 1] = bf_hi(ww[j]); }
      }
      const int nit = (B + 7) / 8;
#pragma unroll 1
      for (int i = 0; i < nit; ++i) {
        const int b = (e >> 4) + 8 * i;
        const bool live = in_range && b < B && act_s[b] != 0;
        const int bb = b < B ? b : 0;
        const int pos = pos_s[bb];
        float x[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] = bf16_round(exch[(rg * 8 + j) * p.exch_stride + bb]);
        if (p.q_norm != nullptr) {
          // _per_head_rms_norm (Qwen3 operations.py:52-63) on the bf16-rounded projection, fp32 until the end
          float ssq = 0.f;
#pragma unroll
          for (int j = 0; j < 8; ++j) ssq += x[j] * x[j];
          const int lanes = p.HD / 8;   // row groups per head: 8 or 16
          for (int o = 1; o < lanes; o <<= 1) ssq += __shfl_xor_sync(kFullMask, ssq, o);
          if (nw != nullptr) {
            const float f = rsqrtf(ssq / (float)p.HD + p.qk_eps);
#pragma unroll
            for (int j = 0; j < 8; ++j) x[j] = bf16_round(wn[j] * (x[j] * f));
          }
        }
        if (!live) continue;
        uint4 o4;
        if (is_v) {
          o4.x = pack_bf16x2(x[0], x[1]); o4.y = pack_bf16x2(x[2], x[3]);
          o4.z = pack_bf16x2(x[4], x[5]); o4.w = pack_bf16x2(x[6], x[7]);
        } else {
          const float4* cp = reinterpret_cast<const float4*>(p.rope_cos + (size_t)pos * p.HD + d0);
          const float4* sp = reinterpret_cast<const float4*>(p.rope_sin + (size_t)pos * p.HD + d0);
          const float4 c0 = __ldg(cp), c1 = __ldg(cp + 1), s0 = __ldg(sp), s1 = __ldg(sp + 1);
          const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
          const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
          float y[8];
#pragma unroll
          for (int j = 0; j < 8; j += 2) {   // pair (2m, 2m+1): rotate_half gives (-odd, even)
            y[j] = x[j] * cs[j] - x[j + 1] * sn[j];
            y[j + 1] = x[j + 1] * cs[j + 1] + x[j] * sn[j + 1];
          }
          o4.x = pack_bf16x2(y[0], y[1]); o4.y = pack_bf16x2(y[2], y[3]);
          o4.z = pack_bf16x2(y[4], y[5]); o4.w = pack_bf16x2(y[6], y[7]);
        }
        if (!is_k && !is_v) {
          *reinterpret_cast<uint4*>(p.q_post_rope + (size_t)b * p.QDIM + row) = o4;
        } else {
          const int col = is_k ? row - p.QDIM : row - p.QDIM - kdim;
          uint16_t* cache = is_k ? p.k_cache : p.v_cache;
          *reinterpret_cast<uint4*>(cache + (size_t)layer * p.kv_layer_stride + (size_t)slot_s[b] * p.kv_batch_stride +
                                    (size_t)pos * p.kv_seq_stride + col) = o4;
        }
      }
      break;
    }
    case kRouter: {
      // fused_router (qwen1_5_moe_a2_7b/.../fused/operations.py:175-194): fp32 softmax over all experts, the k largest
      // probabilities as they are (no renormalisation), lowest index first on equal values.  Column b of the tile is
      // overwritten by row b's selection (probability, 0 elsewhere); then the distinct experts of the step are listed
      // in ascending order and every (selected expert, row) gets its weight for the expert down-projection.
      const int E = p.E;
      // tpr consecutive lanes share a row: each takes the experts x = q, q + tpr, ...; maxima, sums and the k winners
      // are combined with shuffles.  A winner is marked by negating its (positive) exponential in place.  Every pass
      // reads its values eight at a time before it uses them: one shared-memory latency per eight, not per value.
      const int lg = p.Bpad <= 16 ? 3 : (p.Bpad <= 32 ? 2 : 1), tpr = 1 << lg;
      const int b = e >> lg, q = e & (tpr - 1);
      const bool rowok = b < p.Bpad;
      const int bb = rowok ? b : 0;
      const bool act = b < B && act_s[bb] != 0;
      const int stride = p.exch_stride;
      float* col = exch + bb;
      float mx = -INFINITY;
      for (int x0 = q; x0 < E; x0 += 8 * tpr) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) { const int x = x0 + u * tpr; v[u] = x < E ? col[x * stride] : -INFINITY; }
#pragma unroll
        for (int u = 0; u < 8; ++u) mx = fmaxf(mx, v[u]);
      }
      for (int o = 1; o < tpr; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(kFullMask, mx, o));
      float sum = 0.f;
      for (int x0 = q; x0 < E; x0 += 8 * tpr) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) { const int x = x0 + u * tpr; v[u] = x < E ? __expf(col[x * stride] - mx) : 0.f; }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int x = x0 + u * tpr;
          if (rowok && x < E) col[x * stride] = v[u];
          sum += v[u];
        }
      }
      for (int o = 1; o < tpr; o <<= 1) sum += __shfl_xor_sync(kFullMask, sum, o);
      const float inv = 1.0f / sum;
      for (int j = 0; j < p.topk; ++j) {
        float best = -1.f;
        int bi = E;
        for (int x0 = q; x0 < E; x0 += 8 * tpr) {
          float v[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) { const int x = x0 + u * tpr; v[u] = x < E ? (rowok ? col[x * stride] : 0.f) : -2.f; }
#pragma unroll
          for (int u = 0; u < 8; ++u)
            if (v[u] > best) { best = v[u]; bi = x0 + u * tpr; }
        }
        for (int o = 1; o < tpr; o <<= 1) {
          const float ob = __shfl_xor_sync(kFullMask, best, o);
          const int oi = __shfl_xor_sync(kFullMask, bi, o);
          if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
        }
        if (rowok && bi < E && (bi & (tpr - 1)) == q) col[bi * stride] = -best;
      }
      if (rowok)
        for (int x0 = q; x0 < E; x0 += 8 * tpr) {
          float v[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) { const int x = x0 + u * tpr; v[u] = x < E ? col[x * stride] : 0.f; }
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int x = x0 + u * tpr;
            if (x < E) col[x * stride] = (act && v[u] < 0.f) ? -v[u] * inv : 0.f;
          }
        }
      named_bar(kBarEpi, 128);
      // The distinct experts of the step in ascending order: thread x looks at expert x, slots come from a ballot per warp
      // and the warps' counts.  (Expert parallelism: only the experts this rank holds are listed, under their local index;
      // every rank runs the same router on the same rows, so the ranks' lists together are the step's selection.)
      int* slot_of = reinterpret_cast<int*>(c.smem + Smem::kOffHs);   // [128] (the prologue's scratch, free now)
      const int per_rank = p.ep_world > 1 ? E / p.ep_world : E;
      const int e_lo = p.ep_world > 1 ? p.ep_rank * per_rank : 0;
      bool any = false;
      if (e < E && e >= e_lo && e < e_lo + per_rank) {
        const float* row = exch + e * stride;
        for (int b0 = 0; b0 < B; b0 += 8) {
          float v[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) v[u] = b0 + u < B ? row[b0 + u] : 0.f;
#pragma unroll
          for (int u = 0; u < 8; ++u) any |= v[u] > 0.f;
        }
      }
      const unsigned ballot = __ballot_sync(kFullMask, any);
      if (c.lane == 0) c.ctl[kCRouterCnt + (e >> 5)] = (unsigned)__popc(ballot);
      named_bar(kBarEpi, 128);
      int before = 0, total = 0;
      for (int w = 0; w < 4; ++w) {
        const int cw = (int)c.ctl[kCRouterCnt + w];
        before += w < (e >> 5) ? cw : 0;
        total += cw;
      }
      const int slot = any ? before + __popc(ballot & ((1u << c.lane) - 1u)) : -1;
      slot_of[e] = slot;
      if (any) p.moe_elist[slot] = e - e_lo;
      if (e == 0) {
        *p.moe_ne = total;
        atomicAdd(p.moe_ne_sum, (unsigned long long)total);
      }
      named_bar(kBarEpi, 128);
      // router weight of every (listed expert, row), zero for rows that did not select it: all threads, row-contiguous stores
      for (int i0 = e; i0 < E * kMaxBatch; i0 += 128 * 4) {
        float v[4];
        int sl[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int i = i0 + u * 128, x = i >> 6, bc = i & (kMaxBatch - 1);
          sl[u] = i < E * kMaxBatch ? slot_of[x] : -1;
          v[u] = (sl[u] >= 0 && bc < B) ? exch[x * stride + bc] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int i = i0 + u * 128;
          if (sl[u] >= 0) p.moe_w[sl[u] * kMaxBatch + (i & (kMaxBatch - 1))] = v[u];
        }
      }
      break;
    }
    case kEUpGate: {
      // fused_routed_expert_upgate (operations.py:197-219): gate and up rounded to bf16 (a bf16 linear), SiLU(gate) * up
      // in fp32, one rounding.  Tile rows 0..63 are gate rows, 64..127 the up rows of the same units of one expert.
      // The result goes out as the activation operand of the expert down-projection: times the row's router weight
      // (rounded to bf16 again: the weight rides in the operand), as k-block (slot, lt) of the image [slot * per + lt]
      // [Bpad rows][128 bytes, 16-byte pieces swizzled by the row], rows from B up zeroed.
      const int per = p.Ie / kBlockK;
      const int slot = t / per, lt = t % per;
      const int u = e & 63, half = e >> 6;
      float* wrow = reinterpret_cast<float*>(c.smem + Smem::kOffHs);   // [64] router weights of this expert's rows
      if (e < kMaxBatch) wrow[e] = ldcg_f32(p.moe_w + slot * kMaxBatch + e);
      named_bar(kBarEpi, 128);
      const int b0 = half * (p.Bpad / 2), b1 = b0 + p.Bpad / 2;
      unsigned char* blk = p.eimg + (size_t)(slot * per + lt) * (size_t)(p.Bpad * 128);
      // (eight rows at a time, loads / arithmetic / stores in separate passes: the four epilogue warps have a scheduler
      // each to themselves, so independent chains side by side are the only way to hide instruction latency)
      const float* grow = exch + u * p.exch_stride;
      const float* urow = exch + (64 + u) * p.exch_stride;
      for (int bb = b0; bb < b1; bb += 8) {
        float g[8], up[8], w[8];
        bool on[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const int b = bb + k;
          on[k] = (b < B) & (act_s[b] != 0);     // (no short circuit: a branch per row would serialise the loads)
          g[k] = grow[b];
          up[k] = urow[b];
          w[k] = wrow[b];
        }
        unsigned short bits[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float gr = bf16_round(g[k]);
          const float v = on[k] ? bf16_round(__fdividef(gr, 1.0f + __expf(-gr)) * bf16_round(up[k])) * w[k] : 0.f;
          bits[k] = f32_to_bf16_bits(v);
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const int b = bb + k;
          *reinterpret_cast<unsigned short*>(blk + b * 128 + (((u >> 3) ^ (b & 7)) << 4) + (u & 7) * 2) = bits[k];
        }
      }
      break;
    }
    case kOproj:
    case kEDown:
    case kDown: {
      // hidden[b, row] = bf16(hidden + bf16(projection)), zero projection for inactive rows
      // (fused_oproj_gemv_residual / fused_mlp_down_residual, operations.py:251-262, 285-295).
      // Same (sequence, eight rows) ownership: one 16-byte load and store of the residual stream per item, all loads
      // issued first; the sums of squares for the next RMSNorm are reduced over the sixteen row groups by shuffles.
      // model parallelism: the tile holds this rank's partial sums (its experts, or its slice of the K dimension);
      // exch := sum over the ranks' tiles, in rank order on every rank
      if (p.x_world > 1 && (kind == kEDown || p.x_per_layer == 2)) ep_exchange(c, ph, t, e, kind == kDown ? 1 : 0);
      const int rg = e & 15;
      const int row = t * kTileRows + rg * 8;
      const bool in_range = row < p.H;
      const int nit = (B + 7) / 8;
      uint4 oldv[kMaxBatch / 8];
#pragma unroll
      for (int i = 0; i < kMaxBatch / 8; ++i) {
        const int b = (e >> 4) + 8 * i;
        oldv[i] = (i < nit && in_range && b < B) ? ldcg_u4(p.hidden + (size_t)b * p.H + row) : make_uint4(0, 0, 0, 0);
      }
      if (nit == 1) {
        // up to eight sequences: one item per thread (the four-item pass below would carry three empty ones: measured
        // 4.0 us against 2.8 us for this path)
        const int b = e >> 4;
        const int bb = b < B ? b : 0;
        const bool act = (b < B) & (act_s[bb] != 0);
        const uint32_t* ow = reinterpret_cast<const uint32_t*>(&oldv[0]);
        float nv[8], s0 = 0.f, s1 = 0.f;
#pragma unroll
        for (int j = 0; j < 8; j += 2) {
          const float a0 = exch[(rg * 8 + j) * p.exch_stride + bb], a1 = exch[(rg * 8 + j + 1) * p.exch_stride + bb];
          nv[j] = bf16_round(bf_lo(ow[j >> 1]) + bf16_round(act ? a0 : 0.f));
          nv[j + 1] = bf16_round(bf_hi(ow[j >> 1]) + bf16_round(act ? a1 : 0.f));
          s0 += nv[j] * nv[j];
          s1 += nv[j + 1] * nv[j + 1];
        }
        float sq = 0.f;
        if (in_range && b < B) {
          uint4 o4;
          o4.x = pack_bf16x2(nv[0], nv[1]); o4.y = pack_bf16x2(nv[2], nv[3]);
          o4.z = pack_bf16x2(nv[4], nv[5]); o4.w = pack_bf16x2(nv[6], nv[7]);
          *reinterpret_cast<uint4*>(p.hidden + (size_t)b * p.H + row) = o4;
          sq = s0 + s1;
        }
#pragma unroll
        for (int o = 1; o < 16; o <<= 1) sq += __shfl_xor_sync(kFullMask, sq, o);
        if (rg == 0 && b < B) p.ss[t * kMaxBatch + b] = sq;
        break;
      }
      // four items at a time, every pass over all four before the next pass (independent chains side by side: see
      // kEUpGate); items past the batch carry zeros through the arithmetic and are not stored
#pragma unroll
      for (int i0 = 0; i0 < kMaxBatch / 8; i0 += 4) {
        if (i0 < nit) {
          float add[4][8];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int b = (e >> 4) + 8 * (i0 + k);
            const int bb = b < B ? b : 0;
            const bool act = (b < B) & (act_s[bb] != 0);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float v = exch[(rg * 8 + j) * p.exch_stride + bb];
              add[k][j] = act ? v : 0.f;
            }
          }
          float sq[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int b = (e >> 4) + 8 * (i0 + k);
            const uint32_t* ow = reinterpret_cast<const uint32_t*>(&oldv[i0 + k]);
            float nv[8];
            float s0 = 0.f, s1 = 0.f;
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
              nv[j] = bf16_round(bf_lo(ow[j >> 1]) + bf16_round(add[k][j]));
              nv[j + 1] = bf16_round(bf_hi(ow[j >> 1]) + bf16_round(add[k][j + 1]));
              s0 += nv[j] * nv[j];
              s1 += nv[j + 1] * nv[j + 1];
            }
            sq[k] = 0.f;
            if (in_range && b < B) {
              uint4 o4;
              o4.x = pack_bf16x2(nv[0], nv[1]); o4.y = pack_bf16x2(nv[2], nv[3]);
              o4.z = pack_bf16x2(nv[4], nv[5]); o4.w = pack_bf16x2(nv[6], nv[7]);
              *reinterpret_cast<uint4*>(p.hidden + (size_t)b * p.H + row) = o4;
              sq[k] = s0 + s1;
            }
          }
          // The four sums over the sixteen row groups with five shuffles instead of sixteen (a shuffle costs the
          // epilogue warp ~0.1 us here): lanes 8 apart swap two of the four sums, lanes 4 apart one of the remaining
          // two, then the four lanes that hold the same item add up.  Item 2 * (bit 3 of rg) + (bit 2 of rg) ends in
          // the lane.
          {
            const bool h8 = (rg & 8) != 0, h4 = (rg & 4) != 0;
            float k0 = h8 ? sq[2] : sq[0], k1 = h8 ? sq[3] : sq[1];
            const float s0 = h8 ? sq[0] : sq[2], s1 = h8 ? sq[1] : sq[3];
            k0 += __shfl_xor_sync(kFullMask, s0, 8);
            k1 += __shfl_xor_sync(kFullMask, s1, 8);
            float kk = h4 ? k1 : k0;
            const float ss = h4 ? k0 : k1;
            kk += __shfl_xor_sync(kFullMask, ss, 4);
            kk += __shfl_xor_sync(kFullMask, kk, 2);
            kk += __shfl_xor_sync(kFullMask, kk, 1);
            const int b = (e >> 4) + 8 * (i0 + (h8 ? 2 : 0) + (h4 ? 1 : 0));
            if ((rg & 3) == 0 && b < B) p.ss[t * kMaxBatch + b] = kk;
          }
        }
      }
      break;
    }
    case kUpGate: {
      const int u = e & 63, half = e >> 6;
      const int unit = t * (kTileRows / 2) + u;
      if (unit < p.I) {
        const int b0 = half * (p.Bpad / 2), b1 = b0 + p.Bpad / 2;
        const float* grow = exch + u * p.exch_stride;
        const float* urow = exch + (64 + u) * p.exch_stride;
        for (int bb = b0; bb < b1 && bb < B; bb += 8) {   // eight rows at a time: loads, arithmetic, stores (see kEUpGate)
          float g[8], up[8];
          bool on[8];
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const int b = bb + k;
            on[k] = (b < B) & (act_s[b] != 0);
            g[k] = grow[b];
            up[k] = urow[b];
          }
          unsigned short bits[8];
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const unsigned short v = silu_mul(g[k], up[k]);
            bits[k] = on[k] ? v : (unsigned short)0;
          }
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const int b = bb + k;
            if (b < B) {
              p.silu_out[(size_t)b * p.I + unit] = bits[k];
              *reinterpret_cast<unsigned short*>(p.simg + img_piece(p.Bpad, b, unit) + (unit & 7) * 2) = bits[k];
            }
          }
        }
      }
      break;
    }
    default: {   // LM head: logits and the per-row arg-max (lowest index on ties)
      const int nrow = min(kTileRows, p.vocab - t * kTileRows);
      if (p.vocab % 8 == 0 && (reinterpret_cast<unsigned long long>(p.logits) & 15ull) == 0ull) {
        // a thread owns (sequence b, eight consecutive vocabulary rows): one 16-byte store per item, as in the residual
        // epilogue (the tile's rows end on a multiple of eight)
        const int rg = e & 15, r0 = rg * 8;
        const int nit = (B + 7) / 8;
        if (r0 < nrow) {
#pragma unroll 2
          for (int i = 0; i < nit; ++i) {
            const int b = (e >> 4) + 8 * i;
            const int bb = b < B ? b : 0;
            const bool on = (b < B) & (act_s[bb] != 0);
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = exch[(r0 + j) * p.exch_stride + bb];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = on ? v[j] : -1e9f;
            uint4 o4;
            o4.x = pack_bf16x2(v[0], v[1]); o4.y = pack_bf16x2(v[2], v[3]);
            o4.z = pack_bf16x2(v[4], v[5]); o4.w = pack_bf16x2(v[6], v[7]);
            if (b < B) *reinterpret_cast<uint4*>(p.logits + (size_t)b * p.vocab + t * kTileRows + r0) = o4;
          }
        }
      } else {
        const int row = t * kTileRows + e;
        if (row < p.vocab) {
          const float* lrow = exch + e * p.exch_stride;
          for (int bb = 0; bb < B; bb += 8) {      // eight rows at a time: loads, then stores
            unsigned short bits[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const int b = bb + k;
              const float v = lrow[b];            // (b < Bpad: the padded batch is a multiple of 16)
              bits[k] = f32_to_bf16_bits(((b < B) & (act_s[b] != 0)) ? v : -1e9f);
            }
#pragma unroll
            for (int k = 0; k < 8; ++k)
              if (bb + k < B) p.logits[(size_t)(bb + k) * p.vocab + row] = bits[k];
          }
        }
      }
      {
        // arg-max: all 128 threads, 8 / 4 / 2 of them per sequence (a share of the tile's rows each, four independent
        // maxima side by side; the key holds the row, so the maximum of the maxima is the scan's result)
        const int lg = p.Bpad <= 16 ? 3 : (p.Bpad <= 32 ? 2 : 1);
        const int nb = kTileRows >> lg;              // sequences side by side = rows per thread: 16 / 32 / 64
        const int b = e & (nb - 1), part = e >> (7 - lg);
        if (b < B) {
          unsigned long long bst[4] = {0ull, 0ull, 0ull, 0ull};
          const bool on = act_s[b] != 0;
          const float* col = exch + b;
          const int r_lo = part * nb, r_hi = min(nrow, r_lo + nb);
          for (int r0 = r_lo; r0 < r_hi; r0 += 4) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const int r = r0 + k;
              const float x = col[min(r, r_hi - 1) * p.exch_stride];
              const float v = on ? x : -1e9f;
              const unsigned long long key = argmax_key(f32_to_bf16_bits(v), p.vocab_offset + t * kTileRows + r);
              bst[k] = (r < r_hi && key > bst[k]) ? key : bst[k];
            }
          }
          unsigned long long best = bst[0] > bst[1] ? bst[0] : bst[1];
          const unsigned long long b23 = bst[2] > bst[3] ? bst[2] : bst[3];
          best = best > b23 ? best : b23;
          if (r_lo < nrow) atomicMax(p.argmax_key + b, best);
        }
      }
      break;
    }
  }
}

__device__ __forceinline__ void epilogue_phase(const Ctx& c, int ph, int kind, uint32_t tmem, int e, unsigned& sg) {
  // e: thread index in the epilogue group; the warp's lane quarter of tensor memory is (warp % 4)
  const BParams& p = *c.p;
  const int cta = (int)blockIdx.x;
  int ne = 0;
  if (is_expert_kind(kind)) {
    if (e == 0) c.ctl[kCNeEpi] = (unsigned)expert_count(c, ph);
    named_bar(kBarEpi, 128);
    ne = (int)c.ctl[kCNeEpi];
  }
  const PhaseDims d = phase_dims(p, kind, ne);
  const int U = d.T * d.KB;
  if (U == 0) {
    // Expert parallelism, no selected expert on this rank: the other ranks still wait for this rank's partial tiles, and
    // the residual stream still has to be updated from theirs: zero tiles, dealt to the CTAs, take the usual way out.
    if (kind == kEDown && p.x_world > 1) {
      float* ex = reinterpret_cast<float*>(c.smem + Smem::kOffExch);
      for (int t = cta; t < d.T; t += (int)gridDim.x) {
        for (int j = 0; j < p.Bpad; ++j) ex[e * p.exch_stride + j] = 0.f;
        named_bar(kBarEpi, 128);
        epilogue_tile(c, ph, kind, t, e);
        named_bar(kBarEpi, 128);
      }
    }
    return;
  }
  const int G = phase_ctas(kind, U, (int)gridDim.x);   // CTAs that share this phase's units
  int lo, hi;
  unit_range(U, G, cta, lo, hi);
  float* exch = reinterpret_cast<float*>(c.smem + Smem::kOffExch);
  const int quarter = c.warp & 3;
  const int r = quarter * 32 + c.lane;           // accumulator row (= tile row) of this thread
  const int nchunk = p.Bpad / 16;
  int u = lo;
#pragma unroll 1
  while (u < hi) {
    const int t = u / d.KB, kb_lo = u - t * d.KB;
    const int u_end = min(hi, (t + 1) * d.KB);
    const bool full = kb_lo == 0 && u_end == (t + 1) * d.KB;
    // A tile that is split over several CTAs is finished by the CTA that owns its FIRST unit: that CTA's range ends inside
    // the tile, so it reaches the tile last, when the others (whose ranges start with the tile's later units) have long
    // added their parts.  The others add their partial tile to the tile's fixed-point accumulator at L2 and count
    // themselves in with one release (no ticket to wait for); the owner keeps its own part in shared memory, waits for
    // the count, takes the sum out (leaving zero for the accumulator's next user, a phase later) and adds its own part in
    // the same fixed point: the result is the integer sum of all parts, whatever the order.
    const bool owner = kb_lo == 0 && !full;
    const unsigned buf = sg & 1u;
    const bool ok = __all_sync(kFullMask, mbar_wait(c, c.acc_full(buf), (sg >> 1) & 1u, ph, 6));
    if (e == 0 && u == lo) trace_put(p, ph, 1);
    // (cycle counts, not stamps: a read of the global timer costs about a microsecond, five of them distorted the tail)
    const bool stamp = kTraceOn && e == 0 && u_end == hi && p.trace != nullptr;
    long long tk = stamp ? clock64() : 0;
    if (stamp) trace_put(p, ph, 11);
    // accumulator of a split tile: the slot of the owner (a CTA owns the first unit of at most one split tile, so the
    // slot is the tile's alone)
    const int c_first = unit_owner(U, G, t * d.KB);
    long long* slot = p.ws + (size_t)c_first * (size_t)(kTileRows * p.Bpad);
    if (ok) {
      tmem_fence_after_sync();
#pragma unroll 1
      for (int ch = 0; ch < nchunk; ++ch) {
        uint32_t v[16];
        tmem_ld16(v, tmem + ((uint32_t)(quarter * 32) << 16) + buf * (uint32_t)p.Bpad + ch * 16);
        tmem_wait_ld();
        if (full || owner) {
#pragma unroll
          for (int j = 0; j < 16; ++j) exch[r * p.exch_stride + ch * 16 + j] = __uint_as_float(v[j]);
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) red_add_s64(slot + (size_t)(ch * 16 + j) * kTileRows + r, to_fixed(__uint_as_float(v[j])));
        }
      }
      tmem_fence_before_sync();
      mbar_arrive1(c.acc_empty(buf));
    }
    ++sg;
    // (no fence per thread: the barrier orders the group's additions before thread 0's release on the tile's count,
    // which is cumulative over what the barrier made visible to it)
    named_bar(kBarEpi, 128);
    if (stamp) { const long long n = clock64(); trace_val(p, ph, 12, (unsigned long long)(n - tk)); tk = n; }   // part read out of tensor memory
    if (e == 0) {
      unsigned fin = 0u;
      if (ok && !c.aborted()) {
        if (full) {
          fin = 1u;
        } else if (owner) {
          const unsigned others = (unsigned)tile_segments(U, G, d.KB, t) - 1u;
          if (counter_wait(c, p.tile_tickets + t, others, ph)) {
            p.tile_tickets[t] = 0u;
            fin = 1u;
          }
        } else {
          red_release_gpu_add(p.tile_tickets + t, 1u);
        }
      }
      c.ctl[kCFlagEpi] = fin;
      if (stamp) { const long long n = clock64(); trace_val(p, ph, 13, (unsigned long long)(n - tk)); tk = n; }   // count released, or (owner) all parts counted
    }
    named_bar(kBarEpi, 128);
    const bool run = c.ctl[kCFlagEpi] != 0u;
    if (run && !full) {
      float* o = exch + r * p.exch_stride;
#pragma unroll 1
      for (int ch = 0; ch < nchunk; ++ch) {
        long long x[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) x[j] = exch_zero_s64(slot + (size_t)(ch * 16 + j) * kTileRows + r);
#pragma unroll
        for (int j = 0; j < 16; ++j) o[ch * 16 + j] = __ll2float_rn(x[j] + to_fixed(o[ch * 16 + j])) * kFixInv;   // (no fp64: its rate made this loop the read-back's cost)
      }
    }
    named_bar(kBarEpi, 128);           // the tile is complete in shared memory (or nobody runs)
    if (stamp && run) { const long long n = clock64(); trace_val(p, ph, 14, (unsigned long long)(n - tk)); tk = n; }   // sum read back (split tiles)
    if (run) epilogue_tile(c, ph, kind, t, e);
    named_bar(kBarEpi, 128);           // the exchange tile is free again
    if (stamp && run) trace_val(p, ph, 15, (unsigned long long)(clock64() - tk));                             // tile epilogue
    u = u_end;
  }
}

// ------------------------------------------------------------------------------------------------
// attention: eight workers per CTA, one (sequence, kv head, key range) item per warp at a time
// ------------------------------------------------------------------------------------------------
// The key loop runs on the tensor pipe (mma.sync; a warp-level product of 16 x 8 tiles is the right size for one
// query row of GQ <= 8 heads against a block of keys).  g = lane / 4, t = lane % 4.
//   scores  S[head][key] = q . k : m16n8k16 bf16, A = q (row = query head of the group; rows past the group and rows
//     8..15 are zero), B = K.  n-tile j holds keys 8j..8j+7 (column g = key 8j + g).  The contraction index may be
//     permuted freely as long as q and K agree, so lane (g, t) takes the 16-byte pieces t, 4 + t, 8 + t, ... of its
//     key's row and the same pieces of q: every piece feeds two k-steps (words x,y and z,w).
//     Result: lane (g, t) holds S[head g][keys 8j + 2t, 8j + 2t + 1].
//   output  O[head][dim] = sum_key P V : m16n8k8 tf32 (P rounded to tf32, the sum l taken over the same rounded values;
//     V is bf16 and exact), A = P, B = V.  k-step ks contracts keys 8ks..8ks+7 in the order (k = t -> key 8ks + 2t,
//     k = t + 4 -> key 8ks + 2t + 1): the probabilities the lane already holds.  n-tile jn column g is dim
//     (HD / 8) g + jn, so lane (g, t) loads dims (HD / 8) g .. + HD / 8 of keys 8ks + 2t and 8ks + 2t + 1.
//     Result: lane (g, t) holds O[head g][dims (HD / 4) t + jn] (c0 of n-tile jn) and [(HD / 4) t + HD / 8 + jn] (c1).
// A block is 32 keys at head_dim 64 (16 row pieces of K and 16 of V per lane) and 8 keys at 128 (4 and 4).  The K pieces
// of the next block are requested as soon as the scores of this one exist, its V pieces after the P V products.
__device__ __forceinline__ void mma_qk(float (&c)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_pv(float (&c)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t word_of(const uint4& v, int i) {
  return i == 0 ? v.x : (i == 1 ? v.y : (i == 2 ? v.z : v.w));
}

template <int HD, int GQ>
__device__ __forceinline__ void attention_items(const Ctx& c, int layer, int aw, int trace_ph) {
  const BParams& p = *c.p;
  static_assert(HD == 64 || HD == 128, "row pieces are laid out for head_dim 64 and 128");
  static_assert(GQ <= 8, "one mma row per query head of the group");
  constexpr int LPR = HD / 8;          // 16-byte pieces per K/V row
  constexpr int QP = HD / 32;          // K pieces per key per lane (two k-steps each)
  constexpr int VP = HD / 64;          // V pieces per key per lane
  constexpr int NT = HD == 64 ? 4 : 1; // n-tiles (8 keys each) per block (measured: two n-tiles at head_dim 128 spill)
  constexpr int BK = NT * 8;           // keys per block
  constexpr int NJ = HD / 8;           // n-tiles of the output
  constexpr int DPT = HD / 4;          // output dims per lane
  const int lane = c.lane;
  const int g = lane >> 2, t = lane & 3;
  const int* pos_s = reinterpret_cast<const int*>(c.smem + Smem::kOffPos);
  const int* act_s = reinterpret_cast<const int*>(c.smem + Smem::kOffAct);
  const int* slot_s = reinterpret_cast<const int*>(c.smem + Smem::kOffSlot);
  const int NW = (int)gridDim.x * 8, gw = (int)blockIdx.x * 8 + aw;
  const int Tmax = (int)c.ctl[kCTmax];
  const int seqs = p.B * p.NKV;
  int ck, nch;
  attn_plan(Tmax, seqs, NW, ck, nch);
  const int items = seqs * nch;
  constexpr int REC = GQ * (HD + 2);
#pragma unroll 1
  for (int item = gw; item < items; item += NW) {
    const int ch = item % nch, sq = item / nch;
    const int kvh = sq % p.NKV, b = sq / p.NKV;
    const int T = pos_s[b] + 1;
    const int nsplit = (T + ck - 1) / ck;
    uint16_t* outp = p.attn_out + (size_t)b * p.QDIM + (size_t)kvh * GQ * HD;
    if (!act_s[b]) {   // fused_decode_attention zeroes the output of an inactive row (operations.py:226-231)
      if (ch == 0)
        for (int i = lane; i < GQ * HD / 8; i += 32) {
          reinterpret_cast<uint4*>(outp)[i] = make_uint4(0, 0, 0, 0);
          *reinterpret_cast<uint4*>(p.aimg + img_piece(p.Bpad, b, kvh * GQ * HD + i * 8)) = make_uint4(0, 0, 0, 0);
        }
      continue;
    }
    if (ch >= nsplit) continue;
    const int k_lo = ch * ck, k_hi = min(T, k_lo + ck);
    // q pieces of head g: the same pieces of the row as the lane's K pieces
    uint4 q[QP];
#pragma unroll
    for (int h = 0; h < QP; ++h) q[h] = make_uint4(0u, 0u, 0u, 0u);
    if (g < GQ) {
      const uint16_t* qrow = p.q_post_rope + (size_t)b * p.QDIM + (size_t)(kvh * GQ + g) * HD;
#pragma unroll
      for (int h = 0; h < QP; ++h) q[h] = ldcg_u4(qrow + (4 * h + t) * 8);
    }
    const size_t base = (size_t)layer * p.kv_layer_stride + (size_t)slot_s[b] * p.kv_batch_stride + (size_t)kvh * HD;
    // rows past the end of the range are clamped to its last row (their probability is 0)
    uint4 kk[NT][QP], vv[NT][2][VP];
    auto load_k = [&](int kb) {
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        const uint16_t* row = p.k_cache + base + (size_t)min(kb + 8 * j + g, k_hi - 1) * p.kv_seq_stride;
#pragma unroll
        for (int h = 0; h < QP; ++h) kk[j][h] = ldcg_u4(row + (4 * h + t) * 8);
      }
    };
    auto load_v = [&](int kb) {
#pragma unroll
      for (int ks = 0; ks < NT; ++ks)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const uint16_t* row = p.v_cache + base + (size_t)min(kb + 8 * ks + 2 * t + e, k_hi - 1) * p.kv_seq_stride;
#pragma unroll
          for (int h = 0; h < VP; ++h) vv[ks][e][h] = ldcg_u4(row + g * LPR + h * 8);
        }
    };
    float m = -INFINITY, l = 0.f, o0[NJ], o1[NJ];
#pragma unroll
    for (int i = 0; i < NJ; ++i) o0[i] = o1[i] = 0.f;
    const long long tq0 = (kTraceOn && p.trace != nullptr) ? clock64() : 0;
    load_k(k_lo);
    load_v(k_lo);
#pragma unroll 1
    for (int kb = k_lo; kb < k_hi; kb += BK) {
      float sc0[NT], sc1[NT];
      float bmax = -INFINITY;
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        float cc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int h = 0; h < QP; ++h) {
          mma_qk(cc, q[h].x, q[h].y, kk[j][h].x, kk[j][h].y);
          mma_qk(cc, q[h].z, q[h].w, kk[j][h].z, kk[j][h].w);
        }
        const int key = kb + 8 * j + 2 * t;
        sc0[j] = key < k_hi ? cc[0] * p.scale_log2e : -INFINITY;
        sc1[j] = key + 1 < k_hi ? cc[1] * p.scale_log2e : -INFINITY;
        bmax = fmaxf(bmax, fmaxf(sc0[j], sc1[j]));
      }
      if (kb + BK < k_hi) load_k(kb + BK);
      bmax = fmaxf(bmax, __shfl_xor_sync(kFullMask, bmax, 1));
      bmax = fmaxf(bmax, __shfl_xor_sync(kFullMask, bmax, 2));
      const float m_new = fmaxf(m, bmax);          // finite: key kb of the block is always valid
      const float corr = exp2f(m - m_new);
      m = m_new;
      l *= corr;
#pragma unroll
      for (int i = 0; i < NJ; ++i) {
        o0[i] *= corr;
        o1[i] *= corr;
      }
#pragma unroll
      for (int ks = 0; ks < NT; ++ks) {
        const uint32_t a0 = (__float_as_uint(exp2f(sc0[ks] - m_new)) + 0x1000u) & 0xffffe000u;
        const uint32_t a2 = (__float_as_uint(exp2f(sc1[ks] - m_new)) + 0x1000u) & 0xffffe000u;
        l += __uint_as_float(a0) + __uint_as_float(a2);
#pragma unroll
        for (int jn = 0; jn < NJ; ++jn) {
          const uint32_t wa = word_of(vv[ks][0][jn >> 3], (jn >> 1) & 3), wb = word_of(vv[ks][1][jn >> 3], (jn >> 1) & 3);
          const uint32_t b0 = (jn & 1) ? (wa & 0xffff0000u) : (wa << 16);
          const uint32_t b1 = (jn & 1) ? (wb & 0xffff0000u) : (wb << 16);
          float cc[4] = {o0[jn], o1[jn], 0.f, 0.f};
          mma_pv(cc, a0, a2, b0, b1);
          o0[jn] = cc[0];
          o1[jn] = cc[1];
        }
      }
      if (kb + BK < k_hi) load_v(kb + BK);
    }
    l += __shfl_xor_sync(kFullMask, l, 1);
    l += __shfl_xor_sync(kFullMask, l, 2);
    if (kTraceOn && p.trace != nullptr && aw == 0 && lane == 0) {   // timeline: cycles of this warp's key loop, keys it walked
      trace_val(p, trace_ph, 3, (unsigned long long)(clock64() - tq0));
      trace_val(p, trace_ph, 4, (unsigned long long)(k_hi - k_lo));
    }
    // lane (g, t) with g < GQ now holds dims DPT t .. DPT t + DPT of head g: o0 the first NJ of them, o1 the rest
    if (nsplit == 1) {
      if (g < GQ) {
        const float inv = 1.0f / l;
#pragma unroll
        for (int i = 0; i < DPT / 8; ++i) {
          const float* src = i < NJ / 8 ? o0 + i * 8 : o1 + (i - NJ / 8) * 8;
          uint4 o4;
          o4.x = pack_bf16x2(src[0] * inv, src[1] * inv);
          o4.y = pack_bf16x2(src[2] * inv, src[3] * inv);
          o4.z = pack_bf16x2(src[4] * inv, src[5] * inv);
          o4.w = pack_bf16x2(src[6] * inv, src[7] * inv);
          *reinterpret_cast<uint4*>(outp + g * HD + DPT * t + i * 8) = o4;
          *reinterpret_cast<uint4*>(p.aimg + img_piece(p.Bpad, b, (kvh * GQ + g) * HD + DPT * t + i * 8)) = o4;
        }
      }
      continue;
    }
    float* rec = p.attn_part + (size_t)item * REC;
    if (g < GQ) {
      // (HD + 2) * 4 bytes per head record keeps 8-byte alignment only: write as float2 pairs
      float2* d2 = reinterpret_cast<float2*>(rec + g * (HD + 2) + DPT * t);
#pragma unroll
      for (int i = 0; i < NJ / 2; ++i) {
        d2[i] = make_float2(o0[2 * i], o0[2 * i + 1]);
        d2[NJ / 2 + i] = make_float2(o1[2 * i], o1[2 * i + 1]);
      }
      if (t == 0) *reinterpret_cast<float2*>(rec + g * (HD + 2) + HD) = make_float2(m, l);
    }
    // (no fence per lane: the warp barrier orders the lanes' record stores before lane 0's acquire-release ticket, and
    // the second one orders lane 0's acquire before the other lanes' reads of the records)
    __syncwarp();
    unsigned last = 0u;
    if (lane == 0) {
      const unsigned old = atom_add_acq_rel_gpu(p.attn_tickets + sq, 1u);
      last = old == (unsigned)(nsplit - 1) ? 1u : 0u;
      if (last) p.attn_tickets[sq] = 0u;
    }
    last = __shfl_sync(kFullMask, last, 0);
    if (!last) continue;
    __syncwarp();
    // merge the nsplit records of this (sequence, kv head): every lane takes (head, 8 dims) pieces and folds the
    // records in split order (loads of four records in flight)
    const float* recs = p.attn_part + (size_t)(sq * nch) * REC;
    for (int piece = lane; piece < GQ * LPR; piece += 32) {
      const int g = piece / LPR, dd = piece % LPR;
      float M = -INFINITY, L = 0.f, o[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
      for (int s = 0; s < nsplit; ++s) {
        const float* rr = recs + (size_t)s * REC + g * (HD + 2);
        const float2 ml = ldcg_f2(rr + HD);
        float2 a[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) a[j] = ldcg_f2(rr + dd * 8 + 2 * j);
        const float mn = fmaxf(M, ml.x);
        const float c0 = exp2f(M - mn), c1 = exp2f(ml.x - mn);
        L = L * c0 + ml.y * c1;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          o[2 * j] = o[2 * j] * c0 + a[j].x * c1;
          o[2 * j + 1] = o[2 * j + 1] * c0 + a[j].y * c1;
        }
        M = mn;
      }
      const float inv = 1.0f / L;
      uint4 o4;
      o4.x = pack_bf16x2(o[0] * inv, o[1] * inv);
      o4.y = pack_bf16x2(o[2] * inv, o[3] * inv);
      o4.z = pack_bf16x2(o[4] * inv, o[5] * inv);
      o4.w = pack_bf16x2(o[6] * inv, o[7] * inv);
      *reinterpret_cast<uint4*>(outp + g * HD + dd * 8) = o4;
      *reinterpret_cast<uint4*>(p.aimg + img_piece(p.Bpad, b, (kvh * GQ + g) * HD + dd * 8)) = o4;
    }
  }
}

__device__ __forceinline__ void attention_phase(const Ctx& c, int ph, int aw) {
  const BParams& p = *c.p;
  if (aw == 0 && c.lane == 0) {
    bool needed;
    const bool ok = phase_dependency(c, ph, needed);
    c.ctl[kCFlagAttn] = ok ? 1u : 0u;
    trace_put(p, ph, 0);
  }
  named_bar(kBarAttn, 256);
  if (c.ctl[kCFlagAttn] != 0u) {
    const int layer = phase_layer(p, ph), gq = p.NH / p.NKV;
    if (p.HD == 64) {
      if (gq == 4) attention_items<64, 4>(c, layer, aw, ph);
      else if (gq == 2) attention_items<64, 2>(c, layer, aw, ph);
      else attention_items<64, 1>(c, layer, aw, ph);
    } else {
      if (gq == 4) attention_items<128, 4>(c, layer, aw, ph);
      else if (gq == 2) attention_items<128, 2>(c, layer, aw, ph);
      else attention_items<128, 1>(c, layer, aw, ph);
    }
  }
  named_bar(kBarAttn, 256);   // the workers' stores, then one release on the phase counter
  if (aw == 0 && c.lane == 0 && !c.aborted()) {
    red_release_gpu_add(p.phase_done + 1 + ph, 1u);
    trace_put(p, ph, 5);
  }
}

// ------------------------------------------------------------------------------------------------
// prologue / finalize (epilogue group)
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void prologue(const Ctx& c, int e) {
  // rows b = cta, cta + G, ...: optional embedding of token_in[b], then the sum of squares of hidden[b]
  const BParams& p = *c.p;
  float* red = reinterpret_cast<float*>(c.smem + Smem::kOffHs);
  const int nt = (p.H + kTileRows - 1) / kTileRows;
  for (int b = (int)blockIdx.x; b < p.B; b += (int)gridDim.x) {
    uint16_t* h = p.hidden + (size_t)b * p.H;
    const uint16_t* src = h;
    if (p.prologue == 2) {   // (a token id outside the vocabulary is clamped, as the batch-1 kernel does)
      long long tok = p.token_in[b];
      tok = tok < 0 ? 0 : (tok >= p.embed_rows ? (long long)p.embed_rows - 1 : tok);
      src = p.embed + (size_t)tok * p.H;
    }
    float s = 0.f;
    for (int i = e; i < p.H / 8; i += 128) {
      const uint4 v = ldcg_u4(src + i * 8);
      if (p.prologue == 2) reinterpret_cast<uint4*>(h)[i] = v;
      const uint32_t* w = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) s += bf_lo(w[j]) * bf_lo(w[j]) + bf_hi(w[j]) * bf_hi(w[j]);
    }
    s = warp_sum(s);
    if (c.lane == 0) red[e >> 5] = s;
    named_bar(kBarEpi, 128);
    if (e < nt) p.ss[e * kMaxBatch + b] = e == 0 ? red[0] + red[1] + red[2] + red[3] : 0.f;
    named_bar(kBarEpi, 128);
  }
  __threadfence();
  named_bar(kBarEpi, 128);
  if (e == 0) red_release_gpu_add(p.phase_done + 0, 1u);
}

__device__ __forceinline__ void finalize(const Ctx& c, int e) {
  // CTA 0, after every CTA has finished the LM head: tokens out
  const BParams& p = *c.p;
  const int lm = p.ppl * p.num_layers;
  if (e == 0) c.ctl[kCFlagEpi] = counter_wait(c, p.phase_done + 1 + lm, gridDim.x, lm) ? 1u : 0u;
  named_bar(kBarEpi, 128);
  if (p.x_world > 1 && p.x_per_layer == 2) {
    // Tensor parallelism: every rank holds a slice of the vocabulary and the arg-max key of its slice (the key carries the
    // global row).  Keys go to the peers' buffers like the partial tiles do: store, flag, bounded wait on the local flags.
    const int W = p.x_world, me = p.x_rank;
    const unsigned tag = p.epoch;
    if (c.ctl[kCFlagEpi] != 0u) {
      if (e < p.B) {
        const unsigned long long mine = __ldcg(p.argmax_key + e);
        for (int d = 0; d < W; ++d)
          if (d != me) p.ep_key[d][me * kMaxBatch + e] = mine;
      }
      __threadfence_system();
      named_bar(kBarEpi, 128);
      if (e < W && e != me) {
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.ep_kflag[e] + me), "r"(tag) : "memory");
        const unsigned* flag = p.ep_kflag[me] + e;
        const long long t0 = clock64();
        for (unsigned it = 1;; ++it) {
          unsigned v;
          asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
          if (v == tag) break;
          if ((it & 15u) == 0u) {
            if (c.ctl[kCAbort] != 0u) break;
            if (clock64() - t0 > c.p->timeout_cycles) {
              report(p, kErrCounterWait, c.warp, lm, v, tag, 48 + e);
              c.ctl[kCAbort] = 1u;
              break;
            }
          }
        }
      }
      named_bar(kBarEpi, 128);
      if (c.ctl[kCAbort] == 0u && e < p.B) {
        unsigned long long best = __ldcg(p.argmax_key + e);
        for (int s = 0; s < W; ++s) {
          if (s == me) continue;
          const unsigned long long k = __ldcg(p.ep_key[me] + s * kMaxBatch + e);
          best = k > best ? k : best;
        }
        p.argmax_key[e] = best;
      }
      named_bar(kBarEpi, 128);
      if (c.ctl[kCAbort] != 0u) return;
    }
  }
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
      mbar_init(c.a_full(s), 33);
      if ((s & 1) == 0) mbar_init(c.empty(s), 1);
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
    // (the same goes for a row that names a sequence the KV cache does not have)
    int slot = b < p.B ? (p.kv_slots ? p.kv_slots[b] : b) : 0;
    if (act != 0 && (pos < 0 || pos >= p.pos_limit || slot < 0 || slot >= p.kv_batch)) {
      if (blockIdx.x == 0) report(p, kErrRowPosition, 0, p.phase_begin, (unsigned)pos, (unsigned)p.pos_limit, b);
      act = 0;
      pos = -1;
    }
    if (slot < 0 || slot >= p.kv_batch) slot = 0;
    pos_s[b] = pos;
    act_s[b] = act;
    reinterpret_cast<int*>(smem + Smem::kOffSlot)[b] = slot;
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
        named_bar(kBarEpi, 128);           // the group's stores, then thread 0's release on the phase counter
        if (gi == 0 && !c.aborted()) {
          red_release_gpu_add(p.phase_done + 1 + ph, 1u);
          trace_put(p, ph, 5);
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
      // (a slot's barrier also counts the stagers' arrivals, which an aborting CTA may never make: a short bound, a bulk
      // copy lands within microseconds)
      while (!mbar_try_wait(c.a_full((int)(m & (unsigned)(kStages - 1))), (m / (unsigned)kStages) & 1u)) {
        if (clock64() - t0 > 400000) break;
      }
    }
  }
  __syncthreads();
  if (c.warp == 0) {
    tmem_fence_after_sync();
    tmem_dealloc(tmem, 128);
  }
}

