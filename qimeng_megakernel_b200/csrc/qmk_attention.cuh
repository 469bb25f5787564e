// Split-KV GQA decode attention with a cross-SM log-sum-exp merge.  Included by qmk_phases.cuh.
//
// Math: fused_decode_attention (decode_schedule/fused/operations.py:218-248) -- softmax(q.k/sqrt(d)) v
// in fp32 over keys 0..pos, output rounded to bf16.  Partials keep a running maximum in the log2
// domain and are merged with exp2, as the reference's split / reduction kernels do
// (decode_kernel/decode_attention_splitkv.cu:265-281, 355-381; decode_attention_reduction.cu:212-251).
// Unlike the reference there is no separate reduction instruction: the last partial of a kv head
// to arrive (atomic ticket) performs the merge, which saves one cross-SM hand-off per layer.
// The heads of a GQA group are processed by a rolled loop whose per-head state rotates through
// fixed registers, so the code is emitted once instead of once per head.
#pragma once

namespace qmk {

template <int N>
__device__ __forceinline__ void rotate(float (&a)[N]) {
  const float t = a[0];
#pragma unroll
  for (int i = 0; i + 1 < N; ++i) a[i] = a[i + 1];
  a[N - 1] = t;
}

// Stage this warp's part of q (fp32) and of the new K / V rows (bf16) into the big activation buffer.
template <class S>
__device__ __forceinline__ bool stage_attn_part(const Params& p, unsigned char* smem, bool tagged, unsigned tag,
                                                int warp, int lane, int ph) {
  using L = SmemLayout<S>;
  constexpr int kQPart = S::QDIM / kWorkers;                 // q elements per warp
  constexpr int kKvPart = 2 * S::NKV * S::HD / kWorkers;     // new K+V elements per warp
  static_assert(kQPart % 128 == 0 && kKvPart % 128 == 0, "parts must be whole rounds of tagged uint4");
  constexpr int NQ = kQPart / 128, NKV4 = kKvPart / 128;
  float4* qdst = reinterpret_cast<float4*>(smem + L::kOffActD);
  unsigned char* kvdst = smem + L::kOffActD + S::QDIM * 4;
  if (tagged) {
    // one poll loop over both ranges (q words, then K/V words, contiguous in the scratch)
    const unsigned tagw = tag << 16;
    const uint4* qsrc = reinterpret_cast<const uint4*>(p.t_q + warp * kQPart) + lane;
    const uint4* kvsrc = reinterpret_cast<const uint4*>(p.t_q + S::QDIM + warp * kKvPart) + lane;
    uint4 vq[NQ], vk[NKV4];
    const long long t0 = clock64();
    for (unsigned it = 0;; ++it) {
      bool ok = true;
#pragma unroll
      for (int j = 0; j < NQ; ++j) {
        vq[j] = ldcg_u4(qsrc + j * 32);
        ok = ok && tags_ok(vq[j], tagw);
      }
#pragma unroll
      for (int j = 0; j < NKV4; ++j) {
        vk[j] = ldcg_u4(kvsrc + j * 32);
        ok = ok && tags_ok(vk[j], tagw);
      }
      if (__all_sync(kFullMask, ok)) break;
      if ((it & 15u) == 15u) {
        const bool expired = clock64() - t0 > p.timeout_cycles;
        const unsigned st = ld_relaxed_gpu(p.status + kStCode);
        if (__any_sync(kFullMask, expired || st != 0u)) {
          if (!ok && st == 0u) report_error(p, kErrCounterWait, warp, ph, vq[0].x >> 16, tag, lane);
          return false;
        }
      }
    }
#pragma unroll
    for (int j = 0; j < NQ; ++j) {
      const uint2 b = untag4(vq[j]);
      qdst[(warp * kQPart) / 4 + j * 32 + lane] = make_float4(bf_lo(b.x), bf_hi(b.x), bf_lo(b.y), bf_hi(b.y));
    }
#pragma unroll
    for (int j = 0; j < NKV4; ++j)
      *reinterpret_cast<uint2*>(kvdst + (size_t)(warp * kKvPart + (j * 32 + lane) * 4) * 2) = untag4(vk[j]);
  } else {
    const uint2* qsrc = reinterpret_cast<const uint2*>(p.q_post_rope + warp * kQPart);
#pragma unroll
    for (int j = 0; j < NQ; ++j) {
      const uint2 b = __ldcg(qsrc + j * 32 + lane);
      qdst[(warp * kQPart) / 4 + j * 32 + lane] = make_float4(bf_lo(b.x), bf_hi(b.x), bf_lo(b.y), bf_hi(b.y));
    }
  }
  return true;
}

template <class S>
__device__ __forceinline__ void attn_unit(Worker<S>& s, const Params& p, const unsigned char* smem, int ph,
                                          int kvh, int part, int bps, int P, bool staged_kv, unsigned tagw) {
  using L = SmemLayout<S>;
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
  const unsigned char* knew = smem + L::kOffActD + S::QDIM * 4 + (size_t)kvh * HD * 2;
  const unsigned char* vnew = knew + (size_t)S::NKV * HD * 2 + s.lane * DPL * 2;
  const float4* q4 = reinterpret_cast<const float4*>(smem + L::kOffActD) + (size_t)kvh * GQA * (HD / 4);

  float m[GQA], l[GQA], acc0[GQA], acc1[GQA], acc2[GQA], acc3[GQA];
#pragma unroll
  for (int h = 0; h < GQA; ++h) {
    m[h] = -INFINITY;
    l[h] = acc0[h] = acc1[h] = acc2[h] = acc3[h] = 0.f;
  }

#pragma unroll 1
  for (int kb = k0; kb < k1; kb += kAttnBlockKeys) {
    const int key = kb + s.lane;
    const bool valid = key < k1;
    const int kc = valid ? key : (k1 - 1);
    uint4 kreg[KV4];
    if (staged_kv && kc == p.pos) {
#pragma unroll
      for (int i = 0; i < KV4; ++i) kreg[i] = reinterpret_cast<const uint4*>(knew)[i];
    } else {
      const uint4* kp = reinterpret_cast<const uint4*>(kbase + (size_t)kc * p.kv_seq_stride);
#pragma unroll
      for (int i = 0; i < KV4; ++i) kreg[i] = ldcg_u4(kp + i);
    }
    // V rows of the block, lane = output dims; rows past the end are clamped and carry probability 0.
    uint32_t vreg[kAttnBlockKeys][DPL / 2];
#pragma unroll
    for (int j = 0; j < kAttnBlockKeys; ++j) {
      int kj = kb + j;
      if (kj > k1 - 1) kj = k1 - 1;
      if (staged_kv && kj == p.pos) {
#pragma unroll
        for (int d2 = 0; d2 < DPL / 2; ++d2) vreg[j][d2] = reinterpret_cast<const uint32_t*>(vnew)[d2];
      } else {
        const uint16_t* vp = vbase + (size_t)kj * p.kv_seq_stride;
        if (DPL == 2) {
          vreg[j][0] = ldcg_u32(vp);
        } else {
          const uint2 t = __ldcg(reinterpret_cast<const uint2*>(vp));
          vreg[j][0] = t.x;
          vreg[j][DPL / 2 - 1] = t.y;
        }
      }
    }
#pragma unroll 1
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
      const float m_new = fmaxf(m[0], warp_max(sc));
      const float corr = exp2f(m[0] - m_new);
      const float pr = valid ? exp2f(sc - m_new) : 0.f;
      l[0] = l[0] * corr + pr;
      m[0] = m_new;
      float a0 = acc0[0] * corr, a1 = acc1[0] * corr, a2 = acc2[0] * corr, a3 = acc3[0] * corr;
#pragma unroll
      for (int j = 0; j < kAttnBlockKeys; ++j) {
        const float pj = __shfl_sync(kFullMask, pr, j);
        a0 = fmaf(pj, bf_lo(vreg[j][0]), a0);
        a1 = fmaf(pj, bf_hi(vreg[j][0]), a1);
        if (DPL == 4) {
          a2 = fmaf(pj, bf_lo(vreg[j][DPL / 2 - 1]), a2);
          a3 = fmaf(pj, bf_hi(vreg[j][DPL / 2 - 1]), a3);
        }
      }
      acc0[0] = a0; acc1[0] = a1; acc2[0] = a2; acc3[0] = a3;
      rotate(m); rotate(l); rotate(acc0); rotate(acc1); rotate(acc2); rotate(acc3);
    }
  }
#pragma unroll
  for (int h = 0; h < GQA; ++h) l[h] = warp_sum(l[h]);

  if (P == 1) {
#pragma unroll
    for (int h = 0; h < GQA; ++h) {
      const float inv = 1.0f / l[h];
      const int e = (kvh * GQA + h) * HD + s.lane * DPL;
      const uint32_t w0 = pack_bf16x2(acc0[h] * inv, acc1[h] * inv);
      *reinterpret_cast<uint32_t*>(p.attn_out + e) = w0;
      if (p.sync) *reinterpret_cast<uint2*>(p.t_attn + e) = make_uint2((w0 & 0xffffu) | tagw, (w0 >> 16) | tagw);
      if (DPL == 4) {
        const uint32_t w1 = pack_bf16x2(acc2[h] * inv, acc3[h] * inv);
        *reinterpret_cast<uint32_t*>(p.attn_out + e + 2) = w1;
        if (p.sync) *reinterpret_cast<uint2*>(p.t_attn + e + 2) = make_uint2((w1 & 0xffffu) | tagw, (w1 >> 16) | tagw);
      }
    }
    return;
  }

  // Store the un-normalised partial, then take a ticket; the last arrival merges.
#pragma unroll
  for (int h = 0; h < GQA; ++h) {
    const int head = kvh * GQA + h;
    float* po = p.part_o + ((size_t)head * kMaxSplits + part) * HD + s.lane * DPL;
    *reinterpret_cast<float2*>(po) = make_float2(acc0[h], acc1[h]);
    if (DPL == 4) *reinterpret_cast<float2*>(po + 2) = make_float2(acc2[h], acc3[h]);
    if (s.lane == 0) *reinterpret_cast<float2*>(p.part_ml + ((size_t)head * kMaxSplits + part) * 2) = make_float2(m[h], l[h]);
  }
  // Release the partial (all lanes' stores are ordered before lane 0's atomic by the __syncwarp),
  // take a ticket; only the last arrival goes on, and its atomic acquires the other partials.
  __syncwarp();
  unsigned* ticket_word = p.tickets + (layer & 1) * 32 + kvh;
  unsigned ticket = 0;
  if (s.lane == 0) ticket = atom_add_acq_rel_gpu(ticket_word, 1u);
  ticket = __shfl_sync(kFullMask, ticket, 0);
  if (ticket != (unsigned)(P - 1)) return;
  if (s.lane == 0) atomicExch(ticket_word, 0u);   // every partial of this step has arrived

  // Merge: the warp's lanes are divided among the heads of the group, each lane owns DPM output dims
  // of one head and walks the partials with a running maximum (one pass, loads four partials ahead).
  constexpr int LPH = 32 / GQA;                // lanes per head
  constexpr int DPM = HD / LPH;                // dims per lane (multiple of 4)
  static_assert(DPM % 4 == 0, "merge lanes read float4");
  const int head = kvh * GQA + s.lane / LPH;
  const int d0 = (s.lane % LPH) * DPM;
  const float* mlb = p.part_ml + (size_t)head * kMaxSplits * 2;
  const float* pob = p.part_o + (size_t)head * kMaxSplits * HD + d0;
  float M = -INFINITY, den = 0.f, num[DPM];
#pragma unroll
  for (int d = 0; d < DPM; ++d) num[d] = 0.f;
#pragma unroll 1
  for (int q0 = 0; q0 < P; q0 += 4) {
    float2 ml[4];
    float4 t[4][DPM / 4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int q = (q0 + j) < P ? (q0 + j) : (P - 1);
      ml[j] = ldcg_f2(mlb + 2 * q);
#pragma unroll
      for (int d4 = 0; d4 < DPM / 4; ++d4) t[j][d4] = __ldcg(reinterpret_cast<const float4*>(pob + (size_t)q * HD) + d4);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (q0 + j < P) {
        const float M_new = fmaxf(M, ml[j].x);
        const float corr = exp2f(M - M_new), wq = exp2f(ml[j].x - M_new);
        den = den * corr + wq * ml[j].y;
#pragma unroll
        for (int d4 = 0; d4 < DPM / 4; ++d4) {
          num[4 * d4 + 0] = fmaf(wq, t[j][d4].x, num[4 * d4 + 0] * corr);
          num[4 * d4 + 1] = fmaf(wq, t[j][d4].y, num[4 * d4 + 1] * corr);
          num[4 * d4 + 2] = fmaf(wq, t[j][d4].z, num[4 * d4 + 2] * corr);
          num[4 * d4 + 3] = fmaf(wq, t[j][d4].w, num[4 * d4 + 3] * corr);
        }
        M = M_new;
      }
    }
  }
  const float inv = 1.0f / den;
  const int e = head * HD + d0;
#pragma unroll
  for (int d = 0; d < DPM; d += 2) {
    const uint32_t w = pack_bf16x2(num[d] * inv, num[d + 1] * inv);
    *reinterpret_cast<uint32_t*>(p.attn_out + e + d) = w;
    if (p.sync) *reinterpret_cast<uint2*>(p.t_attn + e + d) = make_uint2((w & 0xffffu) | tagw, (w >> 16) | tagw);
  }
}

// ---- phase 1: attention.  Units (kv head, partial) are dealt round-robin over SMs first.
template <class S>
__device__ __forceinline__ void phase_attn(Worker<S>& s, const Params& p, unsigned char* smem, int ph) {
  int bps, P;
  attn_plan(p.pos + 1, bps, P);
  const int n_units = S::NKV * P;
  if ((int)blockIdx.x >= n_units) return;          // no unit lands on this CTA: nothing to stage
  const bool tagged = p.sync && (ph > p.phase_begin || p.wait_first);
  const long long tq0 = clock64();
  if (!stage_attn_part<S>(p, smem, tagged, phase_tag(p, ph - 1), s.w, s.lane, ph)) s.aborted = true;
  raise_part_flag(s.ctl, s.w, s.lane, s.aborted ? kAbortFlag : (unsigned)(ph + 1));
  const long long tq1 = clock64();
  const int first = s.w * (int)gridDim.x + (int)blockIdx.x;
  if (first < n_units && !s.aborted) {
    if (!wait_parts(p, s.ctl, s.w, s.lane, ph)) s.aborted = true;
    const long long tq2 = clock64();
    const unsigned tagw = phase_tag(p, ph) << 16;
    for (int u = first; u < n_units && !s.aborted; u += s.nwt) attn_unit(s, p, smem, ph, u / P, u % P, bps, P, tagged, tagw);
    if (s.w == 0) {
      trace_put(p, ph, 3, (unsigned long long)(tq1 - tq0), s.lane);
      trace_put(p, ph, 4, (unsigned long long)(tq2 - tq1), s.lane);
      trace_put(p, ph, 6, (unsigned long long)(clock64() - tq2), s.lane);
    }
  }
}

}  // namespace qmk
