// Split-KV GQA decode attention with a cross-SM log-sum-exp merge.  Included by qmk_phases.cuh.
//
// Math: fused_decode_attention (decode_schedule/fused/operations.py:218-248) -- softmax(q.k/sqrt(d)) v
// in fp32 over keys 0..pos, output rounded to bf16.  Partials keep a running maximum in the log2
// domain and are merged with exp2, as the reference's split / reduction kernels do
// (decode_kernel/decode_attention_splitkv.cu:265-281, 355-381; decode_attention_reduction.cu:212-251).
// Unlike the reference there is no separate reduction instruction: the last partial of a kv head
// to arrive (atomic ticket) performs the merge, which saves one cross-SM hand-off per layer.
#pragma once

namespace qmk {

template <class S>
__device__ __forceinline__ void attn_unit(Worker<S>& s, const Params& p, const unsigned char* smem, int ph,
                                          int kvh, int part, int bps, int P) {
  constexpr int HD = S::HD, GQA = S::GQA;
  constexpr int DPL = HD / 32;          // output dims per lane
  constexpr int KV4 = HD / 8;           // uint4 per K row
  static_assert(DPL == 2 || DPL == 4, "head_dim must be 64 or 128");
  const int layer = phase_layer(ph);
  const int T = p.pos + 1;
  const int k0 = part * bps * kAttnBlockKeys;
  int k1 = k0 + bps * kAttnBlockKeys;
  if (k1 > T) k1 = T;
  const uint16_t* kbase = p.k_cache + (size_t)layer * p.kv_layer_stride + (size_t)kvh * HD;
  const uint16_t* vbase = p.v_cache + (size_t)layer * p.kv_layer_stride + (size_t)kvh * HD + s.lane * DPL;
  const float4* q4 = reinterpret_cast<const float4*>(smem + SmemLayout<S>::kOffActD) + (size_t)kvh * GQA * (HD / 4);

  float m[GQA], l[GQA], acc[GQA][DPL];
#pragma unroll
  for (int h = 0; h < GQA; ++h) {
    m[h] = -INFINITY;
    l[h] = 0.f;
#pragma unroll
    for (int d = 0; d < DPL; ++d) acc[h][d] = 0.f;
  }

  for (int kb = k0; kb < k1; kb += kAttnBlockKeys) {
    const int key = kb + s.lane;
    const bool valid = key < k1;
    const int kc = valid ? key : (k1 - 1);
    uint4 kreg[KV4];
    {
      const uint4* kp = reinterpret_cast<const uint4*>(kbase + (size_t)kc * p.kv_seq_stride);
#pragma unroll
      for (int i = 0; i < KV4; ++i) kreg[i] = ldcg_u4(kp + i);
    }
    float pr[GQA];
#pragma unroll
    for (int h = 0; h < GQA; ++h) {
      const float4* qh = q4 + h * (HD / 4);
      float s0 = 0.f, s1 = 0.f;
#pragma unroll
      for (int i = 0; i < KV4; ++i) {
        const float4 qa = qh[2 * i], qb = qh[2 * i + 1];
        const uint4 kk = kreg[i];
        s0 = fmaf(bf_lo(kk.x), qa.x, s0);
        s1 = fmaf(bf_hi(kk.x), qa.y, s1);
        s0 = fmaf(bf_lo(kk.y), qa.z, s0);
        s1 = fmaf(bf_hi(kk.y), qa.w, s1);
        s0 = fmaf(bf_lo(kk.z), qb.x, s0);
        s1 = fmaf(bf_hi(kk.z), qb.y, s1);
        s0 = fmaf(bf_lo(kk.w), qb.z, s0);
        s1 = fmaf(bf_hi(kk.w), qb.w, s1);
      }
      const float sc = valid ? (s0 + s1) * p.scale_log2e : -INFINITY;
      const float m_new = fmaxf(m[h], warp_max(sc));
      const float corr = exp2f(m[h] - m_new);
      pr[h] = valid ? exp2f(sc - m_new) : 0.f;
      l[h] = l[h] * corr + pr[h];
#pragma unroll
      for (int d = 0; d < DPL; ++d) acc[h][d] *= corr;
      m[h] = m_new;
    }
    // P.V: lane = output dims.  Rows past the end are clamped and carry probability 0.
#pragma unroll 1
    for (int j0 = 0; j0 < kAttnBlockKeys; j0 += 8) {
      if (kb + j0 >= k1) break;
      uint32_t vreg[8][DPL / 2];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        int kj = kb + j0 + j;
        if (kj > k1 - 1) kj = k1 - 1;
        const uint16_t* vp = vbase + (size_t)kj * p.kv_seq_stride;
        if (DPL == 2) {
          vreg[j][0] = ldcg_u32(vp);
        } else {
          const uint2 t = __ldcg(reinterpret_cast<const uint2*>(vp));
          vreg[j][0] = t.x;
          vreg[j][DPL / 2 - 1] = t.y;
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
#pragma unroll
        for (int h = 0; h < GQA; ++h) {
          const float pj = __shfl_sync(kFullMask, pr[h], j0 + j);
#pragma unroll
          for (int d2 = 0; d2 < DPL / 2; ++d2) {
            acc[h][2 * d2] = fmaf(pj, bf_lo(vreg[j][d2]), acc[h][2 * d2]);
            acc[h][2 * d2 + 1] = fmaf(pj, bf_hi(vreg[j][d2]), acc[h][2 * d2 + 1]);
          }
        }
      }
    }
  }
#pragma unroll
  for (int h = 0; h < GQA; ++h) l[h] = warp_sum(l[h]);

  if (P == 1) {
#pragma unroll
    for (int h = 0; h < GQA; ++h) {
      const float inv = 1.0f / l[h];
      uint16_t* dst = p.attn_out + (size_t)(kvh * GQA + h) * HD + s.lane * DPL;
#pragma unroll
      for (int d2 = 0; d2 < DPL / 2; ++d2)
        reinterpret_cast<uint32_t*>(dst)[d2] = pack_bf16x2(acc[h][2 * d2] * inv, acc[h][2 * d2 + 1] * inv);
    }
    publish(s, p, ph, kvh % kCounterShards);
    return;
  }

  // Store the un-normalised partial, then take a ticket; the last arrival merges.
#pragma unroll
  for (int h = 0; h < GQA; ++h) {
    const int head = kvh * GQA + h;
    float* po = p.part_o + ((size_t)head * kMaxSplits + part) * HD + s.lane * DPL;
#pragma unroll
    for (int d2 = 0; d2 < DPL / 2; ++d2)
      reinterpret_cast<float2*>(po)[d2] = make_float2(acc[h][2 * d2], acc[h][2 * d2 + 1]);
    if (s.lane == 0) {
      float* ml = p.part_ml + ((size_t)head * kMaxSplits + part) * 2;
      *reinterpret_cast<float2*>(ml) = make_float2(m[h], l[h]);
    }
  }
  // Release the partial (all lanes' stores are ordered before lane 0's atomic by the __syncwarp),
  // take a ticket; only the last arrival goes on, and its atomic acquires the other partials.
  __syncwarp();
  unsigned ticket = 0;
  if (s.lane == 0) ticket = atom_add_acq_rel_gpu(p.tickets + kvh, 1u);
  ticket = __shfl_sync(kFullMask, ticket, 0);
  if (ticket != (unsigned)(P - 1)) return;

  // Merge all GQA heads at once so that the loads of the whole merge overlap: first every (max, sum)
  // pair (lane = partial, two rounds cover kMaxSplits = 64), then the partial outputs four at a time.
  float w_lo[GQA], w_hi[GQA], inv[GQA];
  {
    float2 t_lo[GQA], t_hi[GQA];
#pragma unroll
    for (int h = 0; h < GQA; ++h) {
      const float* mlb = p.part_ml + (size_t)(kvh * GQA + h) * kMaxSplits * 2;
      t_lo[h] = s.lane < P ? ldcg_f2(mlb + 2 * s.lane) : make_float2(-INFINITY, 0.f);
      t_hi[h] = s.lane + 32 < P ? ldcg_f2(mlb + 2 * (s.lane + 32)) : make_float2(-INFINITY, 0.f);
    }
#pragma unroll
    for (int h = 0; h < GQA; ++h) {
      const float M = warp_max(fmaxf(t_lo[h].x, t_hi[h].x));
      w_lo[h] = exp2f(t_lo[h].x - M);
      w_hi[h] = exp2f(t_hi[h].x - M);
      inv[h] = 1.0f / warp_sum(w_lo[h] * t_lo[h].y + w_hi[h] * t_hi[h].y);
    }
  }
  float num[GQA][DPL];
#pragma unroll
  for (int h = 0; h < GQA; ++h)
#pragma unroll
    for (int d = 0; d < DPL; ++d) num[h][d] = 0.f;
  const float* pob = p.part_o + (size_t)kvh * GQA * kMaxSplits * HD + s.lane * DPL;
  for (int q0 = 0; q0 < P; q0 += 4) {
    float2 t[4][GQA][DPL / 2];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int q = (q0 + j) < P ? (q0 + j) : (P - 1);
#pragma unroll
      for (int h = 0; h < GQA; ++h)
#pragma unroll
        for (int d2 = 0; d2 < DPL / 2; ++d2)
          t[j][h][d2] = ldcg_f2(pob + ((size_t)h * kMaxSplits + q) * HD + 2 * d2);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int q = q0 + j;
#pragma unroll
      for (int h = 0; h < GQA; ++h) {
        float wq = __shfl_sync(kFullMask, q < 32 ? w_lo[h] : w_hi[h], q & 31);
        if (q >= P) wq = 0.f;
#pragma unroll
        for (int d2 = 0; d2 < DPL / 2; ++d2) {
          num[h][2 * d2] = fmaf(wq, t[j][h][d2].x, num[h][2 * d2]);
          num[h][2 * d2 + 1] = fmaf(wq, t[j][h][d2].y, num[h][2 * d2 + 1]);
        }
      }
    }
  }
#pragma unroll
  for (int h = 0; h < GQA; ++h) {
    uint16_t* dst = p.attn_out + (size_t)(kvh * GQA + h) * HD + s.lane * DPL;
#pragma unroll
    for (int d2 = 0; d2 < DPL / 2; ++d2)
      reinterpret_cast<uint32_t*>(dst)[d2] = pack_bf16x2(num[h][2 * d2] * inv[h], num[h][2 * d2 + 1] * inv[h]);
  }
  if (s.lane == 0) p.tickets[kvh] = 0u;   // self-reset: every partial of this step has arrived
  publish(s, p, ph, kvh % kCounterShards);
}

// ---- phase 1: attention.  Units (kv head, partial) are dealt round-robin over SMs first.
template <class S>
__device__ __forceinline__ void phase_attn(Worker<S>& s, const Params& p, unsigned char* smem, int ph) {
  int bps, P;
  attn_plan(p.pos + 1, bps, P);
  const int n_units = S::NKV * P;
  const int first = s.w * (int)gridDim.x + (int)blockIdx.x;
  if (first >= n_units) return;
  if (!wait_staged(s, p, ph)) return;
  for (int u = first; u < n_units && !s.aborted; u += s.nwt) attn_unit(s, p, smem, ph, u / P, u % P, bps, P);
}

}  // namespace qmk
