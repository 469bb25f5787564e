// Split-KV GQA decode attention with a cross-SM log-sum-exp merge.  Included by qmk_phases.cuh.
//
// Math: fused_decode_attention (decode_schedule/fused/operations.py:218-248) -- softmax(q.k/sqrt(d)) v
// in fp32 over keys 0..pos, output rounded to bf16.  Partials keep a running maximum in the log2
// domain and are merged with exp2, as the reference's split / reduction kernels do
// (decode_kernel/decode_attention_splitkv.cu:265-281, 355-381; decode_attention_reduction.cu:212-251).
//
// Differences from the reference's two instructions (split, then reduction behind a counter):
//  * a unit fetches the K / V rows of its first block BEFORE it waits for this step's q: old keys do
//    not depend on the step, so their HBM latency hides behind the QKV phase's tail;
//  * this step's own K / V row never goes through the cache on the critical path: it is staged from
//    the tagged scratch next to q;
//  * a compute unit is one kv head x one block of keys; the heads of its GQA group are processed by a
//    rolled loop whose per-head state rotates through fixed registers (code emitted once, not per head);
//  * partials are written as self-validating records (every 64-bit word = {fp32 value, 32-bit tag}),
//    and one merge unit per head, on an otherwise idle warp, polls those records from the start of the
//    phase: no atomic, no separate reduction phase, and no fence in front of the merge.
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
__device__ __forceinline__ bool stage_attn_part(Worker<S>& s, const Params& p, unsigned char* smem, bool tagged,
                                                unsigned tag, int ph) {
  const int warp = s.w, lane = s.lane;
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
      if ((it & 15u) == 15u && poll_give_up(p, t0, ok, vq[0].x >> 16, tag, warp, ph, lane)) return false;
      poll_backoff(s, p, it);
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

// One block of 32 keys of one kv head: lane = key for K (a whole row per lane), lane = output dims for V.
template <class S>
struct KvBlock {
  static constexpr int KV4 = S::HD / 8;     // uint4 per K row
  static constexpr int DPL = S::HD / 32;    // V dims per lane
  uint4 k[KV4];
  uint32_t v[kAttnBlockKeys][DPL / 2];
};

// Rows come from the cache in global memory; rows past the end of the range are clamped to its last
// row (they get probability 0).  With `skip_pos` the row of this step's own position is not fetched
// (its slot keeps whatever it held): patch_new_row() fills it from shared memory after the staging.
template <class S>
__device__ __forceinline__ void load_kv_block(KvBlock<S>& b, const Params& p, int layer, int kvh, int kb, int k1,
                                              int lane) {
  constexpr int HD = S::HD, DPL = KvBlock<S>::DPL;
  const uint16_t* kbase = p.k_cache + (size_t)layer * p.kv_layer_stride + (size_t)kvh * HD;
  const uint16_t* vbase = p.v_cache + (size_t)layer * p.kv_layer_stride + (size_t)kvh * HD + lane * DPL;
  int kc = kb + lane;
  if (kc > k1 - 1) kc = k1 - 1;
  const uint4* kp = reinterpret_cast<const uint4*>(kbase + (size_t)kc * p.kv_seq_stride);
#pragma unroll
  for (int i = 0; i < KvBlock<S>::KV4; ++i) b.k[i] = ldcg_u4(kp + i);
#pragma unroll
  for (int j = 0; j < kAttnBlockKeys; ++j) {
    int kj = kb + j;
    if (kj > k1 - 1) kj = k1 - 1;
    const uint16_t* vp = vbase + (size_t)kj * p.kv_seq_stride;
    if (DPL == 2) {
      b.v[j][0] = ldcg_u32(vp);
    } else {
      const uint2 t = __ldcg(reinterpret_cast<const uint2*>(vp));
      b.v[j][0] = t.x;
      b.v[j][DPL / 2 - 1] = t.y;
    }
  }
}

// Overwrite the row of position `pos` (if it falls in this block, clamped copies included) with the
// K / V row staged in shared memory.
template <class S>
__device__ __forceinline__ void patch_new_row(KvBlock<S>& b, const unsigned char* smem, int kvh, int kb, int k1, int pos,
                                              int lane) {
  using L = SmemLayout<S>;
  constexpr int HD = S::HD, DPL = KvBlock<S>::DPL;
  if (pos < kb || pos >= kb + kAttnBlockKeys || pos != k1 - 1) return;   // the new row is always the last key
  const unsigned char* knew = smem + L::kOffActD + S::QDIM * 4 + (size_t)kvh * HD * 2;
  const unsigned char* vnew = knew + (size_t)S::NKV * HD * 2 + lane * DPL * 2;
  if (kb + lane >= pos) {
#pragma unroll
    for (int i = 0; i < KvBlock<S>::KV4; ++i) b.k[i] = reinterpret_cast<const uint4*>(knew)[i];
  }
#pragma unroll
  for (int j = 0; j < kAttnBlockKeys; ++j) {
    if (kb + j >= pos) {
#pragma unroll
      for (int d2 = 0; d2 < DPL / 2; ++d2) b.v[j][d2] = reinterpret_cast<const uint32_t*>(vnew)[d2];
    }
  }
}

// Partial record of (head, part): HD words of un-normalised output, then running max (log2 domain)
// and sum; every 64-bit word is {fp32 bits, tag}.
template <class S>
__device__ __forceinline__ unsigned long long* part_record(const Params& p, int head, int part) {
  return p.part_rec + ((size_t)head * kMaxSplits + part) * (S::HD + 2);
}

// ---- compute unit: one kv head (all query heads of its group) x one range of keys --------------
template <class S>
__device__ __forceinline__ void attn_unit(Worker<S>& s, const Params& p, unsigned char* smem, int ph, int kvh,
                                          int part, int bps, int P, bool staged_kv, unsigned tagw, KvBlock<S>& blk,
                                          bool blk_loaded) {
  using L = SmemLayout<S>;
  constexpr int HD = S::HD, GQA = S::GQA, DPL = KvBlock<S>::DPL, KV4 = KvBlock<S>::KV4;
  static_assert(DPL == 2 || DPL == 4, "head_dim must be 64 or 128");
  const int layer = phase_layer(ph);
  const int T = p.pos + 1;
  const int k0 = part * bps * kAttnBlockKeys;
  int k1 = k0 + bps * kAttnBlockKeys;
  if (k1 > T) k1 = T;
  const float4* q4 = reinterpret_cast<const float4*>(smem + L::kOffActD) + (size_t)kvh * GQA * (HD / 4);

  float m[GQA], l[GQA], acc0[GQA], acc1[GQA], acc2[GQA], acc3[GQA];
#pragma unroll
  for (int h = 0; h < GQA; ++h) {
    m[h] = -INFINITY;
    l[h] = acc0[h] = acc1[h] = acc2[h] = acc3[h] = 0.f;
  }

#pragma unroll 1
  for (int kb = k0; kb < k1; kb += kAttnBlockKeys) {
    if (!(blk_loaded && kb == k0)) load_kv_block(blk, p, layer, kvh, kb, k1, s.lane);
    if (staged_kv) patch_new_row(blk, smem, kvh, kb, k1, p.pos, s.lane);
    const bool valid = kb + s.lane < k1;
#pragma unroll 1
    for (int h = 0; h < GQA; ++h) {
      const float4* qh = q4 + h * (HD / 4);
      float s0 = 0.f, s1 = 0.f;
#pragma unroll
      for (int i = 0; i < KV4; ++i) {
        const float4 qa = qh[2 * i], qb = qh[2 * i + 1];
        const uint4 kk = blk.k[i];
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
        a0 = fmaf(pj, bf_lo(blk.v[j][0]), a0);
        a1 = fmaf(pj, bf_hi(blk.v[j][0]), a1);
        if (DPL == 4) {
          a2 = fmaf(pj, bf_lo(blk.v[j][DPL / 2 - 1]), a2);
          a3 = fmaf(pj, bf_hi(blk.v[j][DPL / 2 - 1]), a3);
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
      if (p.sync) st_handoff(p.t_attn + e, make_uint2((w0 & 0xffffu) | tagw, (w0 >> 16) | tagw));
      if (DPL == 4) {
        const uint32_t w1 = pack_bf16x2(acc2[h] * inv, acc3[h] * inv);
        *reinterpret_cast<uint32_t*>(p.attn_out + e + 2) = w1;
        if (p.sync) st_handoff(p.t_attn + e + 2, make_uint2((w1 & 0xffffu) | tagw, (w1 >> 16) | tagw));
      }
    }
    flush_handoff();
    return;
  }

  // ---- publish the partial as a self-validating record
  const unsigned rtag = p.launch_seq * 256u + (unsigned)(ph & 255) + 1u;
#pragma unroll
  for (int h = 0; h < GQA; ++h) {
    unsigned long long* rec = part_record<S>(p, kvh * GQA + h, part);
    uint4* dst = reinterpret_cast<uint4*>(rec + s.lane * DPL);
    st_handoff(dst, make_uint4(__float_as_uint(acc0[h]), rtag, __float_as_uint(acc1[h]), rtag));
    if (DPL == 4) st_handoff(dst + 1, make_uint4(__float_as_uint(acc2[h]), rtag, __float_as_uint(acc3[h]), rtag));
    if (s.lane == 0)
      st_handoff(rec + HD, make_uint4(__float_as_uint(m[h]), rtag, __float_as_uint(l[h]), rtag));
  }

  flush_handoff();     // push the records out
}



// ---- merge unit: one query head; polls the P partial records of that head (eight at a time, all
// loads in flight together), merges them with a running maximum and writes attn_out.
template <class S>
__device__ __forceinline__ void attn_merge(Worker<S>& s, const Params& p, int ph, int head, int P, unsigned tagw) {
  constexpr int HD = S::HD, DPL = KvBlock<S>::DPL;
  constexpr int kBatch = 8;
  const unsigned rtag = p.launch_seq * 256u + (unsigned)(ph & 255) + 1u;
  float M = -INFINITY, den = 0.f, num[DPL];
#pragma unroll
  for (int d = 0; d < DPL; ++d) num[d] = 0.f;
#pragma unroll 1
  for (int q0 = 0; q0 < P; q0 += kBatch) {
    uint4 ta[kBatch][DPL / 2], tm[kBatch];
    const long long t0 = clock64();
    for (unsigned it = 0;; ++it) {
      bool ok = true;
#pragma unroll
      for (int j = 0; j < kBatch; ++j) {
        const int q = (q0 + j) < P ? (q0 + j) : (P - 1);
        const unsigned long long* rec = part_record<S>(p, head, q);
        tm[j] = ldcg_u4(rec + HD);
        ok = ok && tm[j].y == rtag && tm[j].w == rtag;
#pragma unroll
        for (int d2 = 0; d2 < DPL / 2; ++d2) {
          ta[j][d2] = ldcg_u4(rec + s.lane * DPL + 2 * d2);
          ok = ok && ta[j][d2].y == rtag && ta[j][d2].w == rtag;
        }
      }
      if (__all_sync(kFullMask, ok)) break;
      if ((it & 15u) == 15u && poll_give_up(p, t0, ok, tm[0].y, rtag, s.w, ph, s.lane)) {
        s.aborted = true;
        return;
      }
      poll_pause(it);
    }
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      if (q0 + j < P) {
        const float mq = __uint_as_float(tm[j].x), lq = __uint_as_float(tm[j].z);
        const float M_new = fmaxf(M, mq);
        const float corr = exp2f(M - M_new), wq = exp2f(mq - M_new);
        den = den * corr + wq * lq;
#pragma unroll
        for (int d2 = 0; d2 < DPL / 2; ++d2) {
          num[2 * d2] = fmaf(wq, __uint_as_float(ta[j][d2].x), num[2 * d2] * corr);
          num[2 * d2 + 1] = fmaf(wq, __uint_as_float(ta[j][d2].z), num[2 * d2 + 1] * corr);
        }
        M = M_new;
      }
    }
  }
  const float inv = 1.0f / den;
  const int e = head * HD + s.lane * DPL;
#pragma unroll
  for (int d = 0; d < DPL; d += 2) {
    const uint32_t w = pack_bf16x2(num[d] * inv, num[d + 1] * inv);
    *reinterpret_cast<uint32_t*>(p.attn_out + e + d) = w;
    if (p.sync) st_handoff(p.t_attn + e + d, make_uint2((w & 0xffffu) | tagw, (w >> 16) | tagw));
  }
  flush_handoff();
}

// ---- phase 1: attention.  Compute units (kv head, part) come first, then (when P > 1) one merge unit per
// head; units are dealt round-robin over SMs first, so a merge unit usually lands on a warp that has
// nothing else to do and polls from the start of the phase.  In any warp's own sequence the merge unit
// is the last one, so it never waits for work queued behind it.
template <class S>
__device__ __forceinline__ void phase_attn(Worker<S>& s, const Params& p, unsigned char* smem, int ph) {
  int bps, P;
  attn_plan(p.pos + 1, bps, P);
  const int n_compute = S::NKV * P;
  const int n_units = n_compute + (P > 1 ? S::NH : 0);
  if ((int)blockIdx.x >= n_units) return;          // no unit lands on this CTA: nothing to stage
  const bool tagged = p.sync && (ph > p.phase_begin || p.wait_first);
  const long long tq0 = clock64();
  const int first = s.w * (int)gridDim.x + (int)blockIdx.x;
  const bool has_unit = first < n_units && !s.aborted;
  KvBlock<S> blk;
  if (has_unit && first < n_compute) {   // old keys do not depend on this step: fetch them before waiting for q
    const int part = first % P, k0 = part * bps * kAttnBlockKeys;
    int k1 = k0 + bps * kAttnBlockKeys;
    if (k1 > p.pos + 1) k1 = p.pos + 1;
    load_kv_block(blk, p, phase_layer(ph), first / P, k0, k1, s.lane);
  }
  if (!s.aborted && !stage_attn_part<S>(s, p, smem, tagged, phase_tag(p, ph - 1), ph)) flag_abort(s, smem);
  cta_sync(s, smem);
  if (s.cta_abort) return;
  const long long tq1 = clock64();
  if (s.w == 0) trace_put(p, ph, 0, globaltimer_ns(), s.lane);
  if (has_unit) {
    const unsigned tagw = phase_tag(p, ph) << 16;
    for (int u = first; u < n_units && !s.aborted; u += s.nwt) {
      if (u < n_compute) attn_unit(s, p, smem, ph, u / P, u % P, bps, P, tagged, tagw, blk, u == first);
      else attn_merge(s, p, ph, u - n_compute, P, tagw);
    }
    if (s.aborted) flag_abort(s, smem);
  }
  if (s.w == 0) {
    trace_put(p, ph, 3, (unsigned long long)(tq1 - tq0), s.lane);
    trace_put(p, ph, 6, (unsigned long long)(clock64() - tq1), s.lane);
    trace_put(p, ph, 7, globaltimer_ns(), s.lane);
  }
}

}  // namespace qmk
