// Kernel entry of the decode megakernel: per-warp set-up, the phase loop, the abort drain.
#pragma once
#include "qmk_kernel.cuh"


namespace qmk {

constexpr int kLaunchThreads = kThreads;

template <class S>
__device__ __forceinline__ void worker_main(const Params& p, unsigned char* smem, int w, int lane) {
  using L = SmemLayout<S>;
  Worker<S> s;
  s.lane = lane;
  s.w = w;
  s.nwt = (int)gridDim.x * kWorkers;
  s.g = (int)blockIdx.x * kWorkers + w;
  s.ring = smem_u32(smem + L::kOffRing + w * kSlots * 2 * kChunkBytes);
  s.bars = smem_u32(smem + L::kOffBars + w * kSlots * 8);
  s.ctl = smem_u32(smem + L::kOffCtl);
  s.n_issued = s.n_acquired = 0;
  s.t_head = s.t_count = 0;
  // this warp's parking space: lanes of its quarter (warp rank mod 4), first or second half of the columns
  s.tmem = reinterpret_cast<const volatile uint32_t*>(smem + L::kOffCtl)[kCtlTmem] + ((uint32_t)(32 * (w & 3)) << 16) +
           (uint32_t)((w >> 2) * kTSlots * kTileCols);
  s.i_slot = s.c_slot = s.c_par = 0;
  s.res = 0.f;
  s.res_valid = false;
  s.aborted = false;
  s.cta_abort = false;
  s.policy = l2_policy_evict_first();
  s.wb.qkv = reinterpret_cast<const unsigned char*>(p.qkv);
  s.wb.o_proj = reinterpret_cast<const unsigned char*>(p.o_proj);
  s.wb.up = reinterpret_cast<const unsigned char*>(p.up);
  s.wb.gate = reinterpret_cast<const unsigned char*>(p.gate);
  s.wb.down = reinterpret_cast<const unsigned char*>(p.down);
  s.wb.lm_head = reinterpret_cast<const unsigned char*>(p.lm_head);
  s.cur.init(s.g, s.nwt, p.vocab, p.phase_begin);
  s.cur.seek(s.wb, p.num_layers, S::kMulti ? p.stream_end : p.phase_end);
#pragma unroll 1
  for (int i = 0; i < kSlots; ++i) issue_one(s, p);

  // A launch runs n_steps decode steps (one unless the caller asked for a device-resident run of several): ONE loop over
  // the launch's phases, step after step (a loop around the phase loop costs the streaming code five registers it does
  // not have).  The weight stream of this warp runs on across the step boundary, so the first tiles of the next step are
  // in the ring and in tensor memory while the step's token is still being decided.
  const int np = num_phases(p.num_layers);
#pragma unroll 1
  for (int gph = p.phase_begin; gph < (S::kMulti ? p.stream_end : p.phase_end) && !s.cta_abort; ++gph) {
    int ph = gph;
    if (S::kMulti && gph >= np) {          // a later step of the launch
      ph = gph % np;
      if (ph == 0) {
        s.res_valid = false;   // the residual stream restarts from the new token's embedding row
        if (w == 0) {
          // cos / sin of the new position.  Every warp of the CTA has left the last QKV epilogue of the step before (it
          // passed the CTA barriers of the later phases with this warp), and reads the table only after the barrier of
          // this step's first staging.
          float* rope = reinterpret_cast<float*>(smem + SmemLayout<S>::kOffRope);
          const int pos = p.pos + gph / np;
          if (lane == 0) *reinterpret_cast<volatile int*>(smem + SmemLayout<S>::kOffPos) = pos;
          for (int i = lane; i < S::HD; i += 32) {
            rope[i] = __ldg(p.rope_cos + (size_t)pos * S::HD + i);
            rope[S::HD + i] = __ldg(p.rope_sin + (size_t)pos * S::HD + i);
          }
        }
      }
    }
    if (w == 0) trace_put(p, ph, 2, globaltimer_ns(), lane);
    const int kind = phase_kind(ph, p.num_layers);
    if (kind == kAttn) {
      const unsigned f = phase_attn_call<S>(p, smem, ph, lane, w, s.aborted ? 1u : 0u, gph);
      s.aborted = (f & 1u) != 0u;
      s.cta_abort = (f & 2u) != 0u;
    }
    else phase_stream(s, p, smem, ph, kind, gph);
    if (w == 0) {
      trace_put(p, ph, 5, globaltimer_ns(), lane);
    }
  }
  if (s.n_acquired != s.n_issued) {
    // (only after an abort)  Leave no bulk copy in flight into this CTA's shared memory: wait (bounded) for each one.
    for (unsigned n = s.n_acquired; n < s.n_issued; ++n) {
      const uint32_t bar = s.bars + (n % kSlots) * 8;
      const long long t0 = clock64();
      while (!mbar_try_wait(bar, (n / kSlots) & 1u)) {
        if (clock64() - t0 > p.timeout_cycles) break;
      }
    }
  }
}

template <class S>
__global__ void __launch_bounds__(kThreads, 1) qmk_decode_kernel(const __grid_constant__ Params p) {
  extern __shared__ __align__(128) unsigned char smem[];
  using L = SmemLayout<S>;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned long long t_entry = globaltimer_ns();
  if (lane == 0) {
    for (int i = 0; i < kSlots; ++i) mbar_init(smem_u32(smem + L::kOffBars + (warp * kSlots + i) * 8), 1);
  }
  if (warp == 0) {
    unsigned* ctl = reinterpret_cast<unsigned*>(smem + L::kOffCtl);
    ctl[lane] = 0u;                                    // flags, arrival count, arg-max key, partial sums
    // cos / sin of this step's position: read by the QKV epilogues of every layer.
    float* rope = reinterpret_cast<float*>(smem + L::kOffRope);
    if (lane == 0) *reinterpret_cast<volatile int*>(smem + L::kOffPos) = p.pos;
    for (int i = lane; i < S::HD; i += 32) {
      rope[i] = __ldg(p.rope_cos + (size_t)p.pos * S::HD + i);
      rope[S::HD + i] = __ldg(p.rope_sin + (size_t)p.pos * S::HD + i);
    }
  }
  if (lane == 0) fence_barrier_init();
  __syncthreads();   // (the control words are zeroed before the allocation writes its address among them)
  if (kTSlots > 0 && warp == 0) {
    tmem_alloc_512(smem_u32(smem + L::kOffCtl + kCtlTmem * 4));
    tmem_fence_before_sync();
  }
  __syncthreads();
  tmem_fence_after_sync();
  worker_main<S>(p, smem, warp, lane);
  if (kTSlots > 0) {   // every warp is done with its tensor-memory share: the allocating warp frees it
    tmem_fence_before_sync();
    __syncthreads();
    if (warp == 0) {
      tmem_fence_after_sync();
      tmem_dealloc_512(reinterpret_cast<const volatile uint32_t*>(smem + L::kOffCtl)[kCtlTmem]);
    }
  }
  if (p.trace != nullptr && lane == 0) {   // kernel entry / exit of this CTA, kept in the slots of the first phase
    unsigned long long* t = p.trace + ((size_t)blockIdx.x * num_phases(p.num_layers) + p.phase_begin) * 8;
    atomicMax(t + 3, ~t_entry);
    atomicMax(t + 7, globaltimer_ns());
  }
}

}  // namespace qmk
