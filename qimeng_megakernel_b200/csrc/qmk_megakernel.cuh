// Controller warp and the kernel entry of the decode megakernel.
#pragma once
#include "qmk_kernel.cuh"

namespace qmk {

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
struct NormWeights {
  uint4 w[S::H / 8 / 32];
};
// The gains do not depend on the step: fetch them before the dependency wait.
template <class S>
__device__ __forceinline__ void load_norm_weights(NormWeights<S>& nw, const uint16_t* weight, int lane) {
#pragma unroll
  for (int j = 0; j < S::H / 8 / 32; ++j) nw.w[j] = __ldg(reinterpret_cast<const uint4*>(weight) + j * 32 + lane);
}

template <class S>
__device__ __forceinline__ void stage_rmsnorm(const uint16_t* src, const NormWeights<S>& nw, float eps,
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
    const uint4 wv = nw.w[j];
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
  const int n4 = n_elems / 8;          // a multiple of 256: eight independent loads per lane per round
  for (int base = 0; base < n4; base += 256) {
    uint4 t[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) t[j] = ldcg_u4(reinterpret_cast<const uint4*>(src) + base + j * 32 + lane);
#pragma unroll
    for (int j = 0; j < 8; ++j) out[base + j * 32 + lane] = t[j];
  }
}

__device__ __forceinline__ void stage_bf16_to_f32(const uint16_t* src, unsigned char* dst, int n_elems, int lane) {
  float4* out = reinterpret_cast<float4*>(dst);
  const int n4 = n_elems / 8;
  for (int base = 0; base < n4; base += 256) {
    uint4 t[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) t[j] = ldcg_u4(reinterpret_cast<const uint4*>(src) + base + j * 32 + lane);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int i = base + j * 32 + lane;
      out[2 * i] = make_float4(bf_lo(t[j].x), bf_hi(t[j].x), bf_lo(t[j].y), bf_hi(t[j].y));
      out[2 * i + 1] = make_float4(bf_lo(t[j].z), bf_hi(t[j].z), bf_lo(t[j].w), bf_hi(t[j].w));
    }
  }
}

template <class S>
__device__ __forceinline__ void controller(const Params& p, unsigned char* smem, int lane) {
  using L = SmemLayout<S>;
  const uint32_t ctl = smem_u32(smem + L::kOffCtl);
  const int nwt = (int)gridDim.x * kWorkers;
  // cos / sin of this step's position: read by the QKV epilogues of every layer.
  {
    float* rope = reinterpret_cast<float*>(smem + L::kOffRope);
    for (int i = lane; i < S::HD; i += 32) {
      rope[i] = __ldg(p.rope_cos + (size_t)p.pos * S::HD + i);
      rope[S::HD + i] = __ldg(p.rope_sin + (size_t)p.pos * S::HD + i);
    }
  }
  for (int ph = p.phase_begin; ph < p.phase_end; ++ph) {
    const int kind = phase_kind(ph, p.num_layers);
    const int layer = phase_layer(ph);
    NormWeights<S> nw;
    const bool normed = kind == kQkv || kind == kUpGate || kind == kLmHead;
    if (normed) {
      const uint16_t* gains = kind == kQkv ? p.attn_norm + (size_t)layer * S::H
                                           : (kind == kUpGate ? p.mlp_norm + (size_t)layer * S::H : p.lm_norm);
      load_norm_weights<S>(nw, gains, lane);
    }
    if (p.sync && ph > 0 && (ph > p.phase_begin || p.wait_first)) {
      if (!poll_dependency<S>(p, ph - 1, ph, lane, nwt)) {
        __syncwarp();
        if (lane == 0) st_release_cta_shared(ctl, kAbortFlag);
        return;
      }
    }
    trace_stamp(p, ph, 0, lane);
    unsigned char* small = smem + (small_buf_index(ph, p.num_layers) ? L::kOffActB : L::kOffActA);
    if (normed) {
      const bool from_token = kind == kQkv || (kind == kLmHead && p.num_layers == 0);
      stage_rmsnorm<S>(from_token ? residual_src<S>(p, layer) : p.hidden, nw, p.eps, small, lane);
    } else if (kind == kAttn) {
      int bps, P;
      attn_plan(p.pos + 1, bps, P);
      if ((int)blockIdx.x < S::NKV * P) stage_bf16_to_f32(p.q_post_rope, smem + L::kOffActD, S::QDIM, lane);
    } else if (kind == kOproj) {
      stage_copy(p.attn_out, small, S::QDIM, lane);
    } else {
      stage_copy(p.silu_out, smem + L::kOffActD, S::I, lane);
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
  s.n_issued = s.n_acquired = 0;
  s.i_slot = s.c_slot = s.c_par = 0;
  s.i_ph = p.phase_begin;
  s.i_kind = s.i_layer = s.i_c = s.i_cend = 0;
  init_ranges(s, p);
  s.staged_seen = 0;
  s.aborted = false;
  s.trace_first = false;
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
    s.cyc_wait = s.cyc_issue = s.cyc_stage = 0;
    const long long tph = clock64();
    const int kind = phase_kind(ph, p.num_layers);
#ifndef QMK_NO_ATTN
    if (kind == kAttn) phase_attn(s, p, smem, ph);
    else
#endif
    phase_stream(s, p, smem, ph, kind);
    if (w == 0) trace_stamp(p, ph, 5, lane);
  }
  if (s.aborted) {
    // Leave no bulk copy in flight into this CTA's shared memory: wait (bounded) for each.
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
