// Controller warp and the kernel entry of the decode megakernel.
#pragma once
#include "qmk_kernel.cuh"

namespace qmk {

// Optional timeline: slot of (CTA, phase) <- globaltimer.  Slots: 0 dependency satisfied, 1 activations
// staged (controller); 2 worker 0 enters the phase, 5 worker 0 leaves it, 6 last worker leaves it.
__device__ __forceinline__ void trace_stamp(const Params& p, int ph, int slot, int lane) {
  if (p.trace != nullptr && lane == 0)
    p.trace[((size_t)blockIdx.x * num_phases(p.num_layers) + ph) * 8 + slot] = globaltimer_ns();
}

// Wait until every publisher of phase `dep` has arrived for this step.  Lane i watches shard i.
template <class S>
__device__ __forceinline__ bool poll_dependency(const Params& p, int dep, int ph, int lane, int nwt) {
  const int kind = phase_kind(dep, p.num_layers);
  const int n_pub = (kind == kAttn) ? S::NKV : nwt;
  const unsigned target = (p.epoch + 1u) * shard_contrib(n_pub, lane);
  const unsigned* c = p.counters + ((size_t)dep * kCounterShards + lane) * kCounterStrideWords;
  const long long t0 = clock64();
  for (unsigned it = 0;; ++it) {
    const unsigned v = ld_acquire_gpu(c);
    const bool ok = (int)(v - target) >= 0;
    if (__all_sync(kFullMask, ok)) return true;
    if ((it & 63u) == 63u) {
      const unsigned st = ld_relaxed_gpu(p.status + kStCode);
      const bool expired = clock64() - t0 > p.timeout_cycles;
      if (__any_sync(kFullMask, st != 0u || expired)) {
        if (st == 0u && expired && !ok) report_error(p, kErrCounterWait, kWorkers, ph, v, target, lane);
        return false;
      }
    }
  }
}

// RMSNorm of the residual stream into a bf16 shared-memory vector:
// y = bf16(w * bf16(x * rsqrt(mean(x^2) + eps)))   (_rms_norm, fused/operations.py:126-131).
template <class S>
__device__ __forceinline__ void stage_rmsnorm(const uint16_t* src, const uint16_t* weight, float eps,
                                              unsigned char* dst, int lane) {
  constexpr int N4 = S::H / 8 / 32;   // uint4 per lane
  uint4 v[N4];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < N4; ++j) {
    v[j] = ldcg_u4(reinterpret_cast<const uint4*>(src) + j * 32 + lane);
    const uint32_t u[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float a = bf_lo(u[e]), b = bf_hi(u[e]);
      ss = fmaf(a, a, ss);
      ss = fmaf(b, b, ss);
    }
  }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss * (1.0f / S::H) + eps);
  uint4* out = reinterpret_cast<uint4*>(dst);
#pragma unroll
  for (int j = 0; j < N4; ++j) {
    const uint4 wv = __ldg(reinterpret_cast<const uint4*>(weight) + j * 32 + lane);
    const uint32_t u[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
    const uint32_t wu[4] = {wv.x, wv.y, wv.z, wv.w};
    uint32_t o[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float a = bf16_round(bf_lo(u[e]) * rstd), b = bf16_round(bf_hi(u[e]) * rstd);
      o[e] = pack_bf16x2(bf_lo(wu[e]) * a, bf_hi(wu[e]) * b);
    }
    out[j * 32 + lane] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

__device__ __forceinline__ void stage_copy(const uint16_t* src, unsigned char* dst, int n_elems, int lane) {
  uint4* out = reinterpret_cast<uint4*>(dst);
  const int n4 = n_elems / 8;
  for (int i = lane; i < n4; i += 32) out[i] = ldcg_u4(reinterpret_cast<const uint4*>(src) + i);
}

__device__ __forceinline__ void stage_bf16_to_f32(const uint16_t* src, unsigned char* dst, int n_elems, int lane) {
  float4* out = reinterpret_cast<float4*>(dst);
  const int n4 = n_elems / 8;
  for (int i = lane; i < n4; i += 32) {
    const uint4 q = ldcg_u4(reinterpret_cast<const uint4*>(src) + i);
    out[2 * i] = make_float4(bf_lo(q.x), bf_hi(q.x), bf_lo(q.y), bf_hi(q.y));
    out[2 * i + 1] = make_float4(bf_lo(q.z), bf_hi(q.z), bf_lo(q.w), bf_hi(q.w));
  }
}

template <class S>
__device__ __forceinline__ void controller(const Params& p, unsigned char* smem, int lane) {
  using L = SmemLayout<S>;
  const uint32_t ctl = smem_u32(smem + L::kOffCtl);
  const int nwt = (int)gridDim.x * kWorkers;
  for (int ph = p.phase_begin; ph < p.phase_end; ++ph) {
    const int kind = phase_kind(ph, p.num_layers);
    const int layer = phase_layer(ph);
    if (p.sync && ph > 0 && (ph > p.phase_begin || p.wait_first)) {
      if (!poll_dependency<S>(p, ph - 1, ph, lane, nwt)) {
        __syncwarp();
        if (lane == 0) st_release_cta_shared(ctl, kAbortFlag);
        return;
      }
    }
    trace_stamp(p, ph, 0, lane);
    unsigned char* small = smem + (small_buf_index(ph, p.num_layers) ? L::kOffActB : L::kOffActA);
    switch (kind) {
      case kQkv:
        stage_rmsnorm<S>(residual_src<S>(p, layer), p.attn_norm + (size_t)layer * S::H, p.eps, small, lane);
        break;
      case kAttn: {
        int bps, P;
        attn_plan(p.pos + 1, bps, P);
        if ((int)blockIdx.x < S::NKV * P) stage_bf16_to_f32(p.q_post_rope, smem + L::kOffActD, S::QDIM, lane);
        break;
      }
      case kOproj:
        stage_copy(p.attn_out, small, S::QDIM, lane);
        break;
      case kUpGate:
        stage_rmsnorm<S>(p.hidden, p.mlp_norm + (size_t)layer * S::H, p.eps, small, lane);
        break;
      case kDown:
        stage_copy(p.silu_out, smem + L::kOffActD, S::I, lane);
        break;
      default:
        stage_rmsnorm<S>(p.num_layers == 0 ? residual_src<S>(p, 0) : p.hidden, p.lm_norm, p.eps, small, lane);
        break;
    }
    __syncwarp();
    if (lane == 0) st_release_cta_shared(ctl, (unsigned)(ph + 1));
    trace_stamp(p, ph, 1, lane);
  }
}

template <class S>
__device__ __forceinline__ void worker_main(const Params& p, unsigned char* smem, int w, int lane) {
  using L = SmemLayout<S>;
  Worker<S> s;
  s.lane = lane;
  s.w = w;
  s.nwt = (int)gridDim.x * kWorkers;
  s.g = (int)blockIdx.x * kWorkers + w;
  s.ring = smem_u32(smem + L::kOffRing + w * kSlots * kChunkBytes);
  s.bars = smem_u32(smem + L::kOffBars + w * kSlots * 8);
  s.ctl = smem_u32(smem + L::kOffCtl);
  s.n_issued = s.n_consumed = 0;
  s.i_ph = p.phase_begin;
  s.i_c = s.i_cend = 0;
  s.staged_seen = 0;
  s.aborted = false;
  s.policy = l2_policy_evict_first();
  s.wb.qkv = p.qkv;
  s.wb.o_proj = p.o_proj;
  s.wb.up = p.up;
  s.wb.gate = p.gate;
  s.wb.down = p.down;
  s.wb.lm_head = p.lm_head;
  cursor_seek(s, p);
#pragma unroll 1
  for (int i = 0; i < kSlots; ++i) issue_one(s, p);

#pragma unroll 1
  for (int ph = p.phase_begin; ph < p.phase_end && !s.aborted; ++ph) {
    if (w == 0) trace_stamp(p, ph, 2, lane);
    switch (phase_kind(ph, p.num_layers)) {
      case kQkv: phase_qkv(s, p, smem, ph); break;
      case kAttn: phase_attn(s, p, smem, ph); break;
      case kOproj: phase_oproj(s, p, smem, ph); break;
      case kUpGate: phase_upgate(s, p, smem, ph); break;
      case kDown: phase_down(s, p, smem, ph); break;
      default: phase_lm_head(s, p, smem, ph); break;
    }
    if (w == 0) trace_stamp(p, ph, 5, lane);
    if (w == kWorkers - 1) trace_stamp(p, ph, 6, lane);
  }
  if (s.aborted) {
    // Leave no bulk copy in flight into this CTA's shared memory: wait (bounded) for each.
    for (unsigned n = s.n_consumed; n < s.n_issued; ++n) {
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
  if (lane == 0) {
    if (warp < kWorkers) {
      for (int i = 0; i < kSlots; ++i) mbar_init(smem_u32(smem + L::kOffBars + (warp * kSlots + i) * 8), 1);
    } else {
      unsigned* ctl = reinterpret_cast<unsigned*>(smem + L::kOffCtl);
      ctl[0] = 0u;
      ctl[1] = 0u;
      ctl[2] = 0u;
      ctl[3] = 0u;
    }
    fence_barrier_init();
  }
  __syncthreads();
  if (warp < kWorkers) worker_main<S>(p, smem, warp, lane);
  else controller<S>(p, smem, lane);
}

}  // namespace qmk
