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

// Stage this warp's part of q and of the new K / V rows (all bf16) into the big activation buffer:
// q at its start, the K row then the V row from byte QDIM * 4 on.
template <class S>
__device__ __forceinline__ bool stage_attn_part(Worker<S>& s, const Params& p, unsigned char* smem, bool tagged,
                                                unsigned tag, int ph) {
  const int warp = s.w, lane = s.lane;
  using L = SmemLayout<S>;
  constexpr int kQPart = S::QDIM / kWorkers;                 // q elements per warp
  constexpr int kKvPart = 2 * S::NKV * S::HD / kWorkers;     // new K+V elements per warp
  static_assert(kQPart % 128 == 0 && kKvPart % 128 == 0, "parts must be whole rounds of tagged uint4");
  constexpr int NQ = kQPart / 128, NKV4 = kKvPart / 128;
  unsigned char* qdst = smem + L::kOffActD;
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
      // (no tile parking here: a compute warp already holds its K / V block in registers)
    }
#pragma unroll
    for (int j = 0; j < NQ; ++j)
      *reinterpret_cast<uint2*>(qdst + (size_t)(warp * kQPart + (j * 32 + lane) * 4) * 2) = untag4(vq[j]);
#pragma unroll
    for (int j = 0; j < NKV4; ++j)
      *reinterpret_cast<uint2*>(kvdst + (size_t)(warp * kKvPart + (j * 32 + lane) * 4) * 2) = untag4(vk[j]);
  } else {
    const uint2* qsrc = reinterpret_cast<const uint2*>(p.q_post_rope + warp * kQPart);
#pragma unroll
    for (int j = 0; j < NQ; ++j)
      *reinterpret_cast<uint2*>(qdst + (size_t)(warp * kQPart + (j * 32 + lane) * 4) * 2) = __ldcg(qsrc + j * 32 + lane);
  }
  return true;
}

// ---- attention on the tensor pipe (head_dim 64, up to 8 query heads per kv head) ----------------
// One block = 32 keys of one kv head.  g = lane / 4, t = lane % 4.
//   scores  S[head][key] = q . k  : mma.m16n8k16 bf16, A = q (row = query head of the group, rows past the
//     group are zero), B = K.  n-tile j holds keys 8j..8j+7 (column g = key 8j + g).  The contraction index may be
//     permuted freely as long as q and K agree, so lane (g, t) simply takes the 32-bit words 4t..4t+3 and
//     16+4t..16+4t+3 of its key's row (two 16-byte loads) and the same words of q: k-step s uses words
//     (4t+2s, 4t+2s+1) of the first half (s = 0, 1) or of the second half (s = 2, 3).
//     Result: lane (g, t) holds S[head g][keys 8j+2t, 8j+2t+1], j = 0..3.
//   output  O[head][dim] = sum_key P V : mma.m16n8k8 tf32 (P in tf32: 2^-11 relative; V exact), A = P, B = V.
//     k-step ks contracts keys 8ks..8ks+7 in the order (k = t -> key 8ks+2t, k = t+4 -> key 8ks+2t+1): exactly the
//     probabilities the lane already holds, no shuffles.  n-tile jn column g is dim 8g + jn, so lane (g, t) loads
//     dims 8g..8g+7 (16 bytes) of keys 8ks+2t and 8ks+2t+1.
//     Result: lane (g, t) holds O[head g][dims 16t + jn] (c0 of n-tile jn) and [16t + 8 + jn] (c1).
template <class S>
struct KvBlock {
  uint4 k[4][2];    // [n-tile j][half]: words 4t..4t+3 / 16+4t..16+4t+3 of key 8j+g
  uint4 v[4][2];    // [k-step ks][key 8ks+2t / 8ks+2t+1]: dims 8g..8g+7
};

// Rows come from the cache in global memory; rows past the end of the range are clamped to its last row
// (they get probability 0).
template <class S>
__device__ __forceinline__ void load_kv_block(KvBlock<S>& b, const Params& p, int layer, int kvh, int kb, int k1,
                                              int lane) {
  static_assert(S::HD == 64, "the tensor-pipe attention is laid out for head_dim 64");
  const uint64_t keep = l2_policy_evict_last();
#pragma unroll
  for (int i = 0; i < 8; ++i) b.k[i >> 1][i & 1] = ld_keep_u4(kv_piece<S>(p, layer, kvh, kb, k1, lane, i), keep);
#pragma unroll
  for (int i = 8; i < 16; ++i) b.v[(i - 8) >> 1][i & 1] = ld_keep_u4(kv_piece<S>(p, layer, kvh, kb, k1, lane, i), keep);
}
// The block that prefetch_attn_rows copied into shared memory during the QKV phase of this launch.
template <class S>
__device__ __forceinline__ void take_staged_kv_block(KvBlock<S>& b, const unsigned char* smem, int w, int lane) {
  using L = SmemLayout<S>;
  cp_async_wait_all();
  const uint4* src = reinterpret_cast<const uint4*>(smem + L::kOffKvStage + w * 16 * 512) + lane;
#pragma unroll
  for (int i = 0; i < 8; ++i) b.k[i >> 1][i & 1] = src[i * 32];
#pragma unroll
  for (int i = 8; i < 16; ++i) b.v[(i - 8) >> 1][i & 1] = src[i * 32];
}

// Overwrite the row of position `pos` (if it falls in this block, clamped copies included) with the
// K / V row staged in shared memory.
template <class S>
__device__ __forceinline__ void patch_new_row(KvBlock<S>& b, const unsigned char* smem, int kvh, int kb, int k1, int pos,
                                              int lane) {
  using L = SmemLayout<S>;
  if (pos < kb || pos >= kb + kAttnBlockKeys || pos != k1 - 1) return;   // the new row is always the last key
  const int g = lane >> 2, t = lane & 3;
  const uint4* knew = reinterpret_cast<const uint4*>(smem + L::kOffActD + S::QDIM * 4 + (size_t)kvh * S::HD * 2);
  const uint4* vnew = reinterpret_cast<const uint4*>(smem + L::kOffActD + S::QDIM * 4 + (size_t)(S::NKV + kvh) * S::HD * 2);
#pragma unroll
  for (int j = 0; j < 4; ++j)
    if (kb + 8 * j + g >= pos) {
      b.k[j][0] = knew[t];
      b.k[j][1] = knew[4 + t];
    }
#pragma unroll
  for (int ks = 0; ks < 4; ++ks)
#pragma unroll
    for (int e = 0; e < 2; ++e)
      if (kb + 8 * ks + 2 * t + e >= pos) b.v[ks][e] = vnew[g];
}

// Partial record of (head, part): HD words of un-normalised output, then running max (log2 domain)
// and sum; every 64-bit word is {fp32 bits, tag}.
template <class S>
__device__ __forceinline__ unsigned long long* part_record(const Params& p, int head, int part) {
  return p.part_rec + ((size_t)head * kMaxSplits + part) * (S::HD + 2);
}

__device__ __forceinline__ void mma_tf32_1688(float (&c)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
  // rows 8..15 of A are zero (a1 = a3 = 0)
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t word_of(const uint4& v, int i) {
  return i == 0 ? v.x : (i == 1 ? v.y : (i == 2 ? v.z : v.w));
}

// ---- a warp's share of a compute unit: keys [k0, k1) of one kv head, all query heads of its group.
// Returns the un-normalised partial in registers: lane (g, t) with g < GQA holds head g's running max m (log2
// domain), sum l, and O[16t + jn] in o0[jn], O[16t + 8 + jn] in o1[jn].
struct AttnPartial {
  float m, l, o0[8], o1[8];
};

template <class S>
__device__ __forceinline__ void attn_blocks(const Params& p, unsigned char* smem, int layer, int kvh, int k0, int k1,
                                            bool staged_kv, bool first_in_smem, KvBlock<S>& blk, int w, int lane,
                                            AttnPartial& out, int pos) {
  using L = SmemLayout<S>;
  constexpr int HD = S::HD, GQA = S::GQA;
  static_assert(GQA <= 8, "one mma row per query head of the group");
  const int g = lane >> 2, t = lane & 3;
  // q fragments of head g: the same words of the row as the lane's K words (rows past the group are zero)
  uint4 qa = make_uint4(0u, 0u, 0u, 0u), qb = qa;
  if (g < GQA) {
    const uint4* qrow = reinterpret_cast<const uint4*>(smem + L::kOffActD + (size_t)(kvh * GQA + g) * HD * 2);
    qa = qrow[t];
    qb = qrow[4 + t];
  }
  float m = -INFINITY, l = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) out.o0[i] = out.o1[i] = 0.f;

#pragma unroll 1
  for (int kb = k0; kb < k1; kb += kAttnBlockKeys) {
    if (kb == k0 && first_in_smem) take_staged_kv_block(blk, smem, w, lane);
    else load_kv_block(blk, p, layer, kvh, kb, k1, lane);
    if (staged_kv) patch_new_row(blk, smem, kvh, kb, k1, pos, lane);
    // scores
    float sc0[4], sc1[4];
    float bmax = -INFINITY;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float c[4] = {0.f, 0.f, 0.f, 0.f};
      {
        const uint32_t a[4] = {qa.x, 0u, qa.y, 0u};
        mma_bf16_16816(c, a, blk.k[j][0].x, blk.k[j][0].y);
      }
      {
        const uint32_t a[4] = {qa.z, 0u, qa.w, 0u};
        mma_bf16_16816(c, a, blk.k[j][0].z, blk.k[j][0].w);
      }
      {
        const uint32_t a[4] = {qb.x, 0u, qb.y, 0u};
        mma_bf16_16816(c, a, blk.k[j][1].x, blk.k[j][1].y);
      }
      {
        const uint32_t a[4] = {qb.z, 0u, qb.w, 0u};
        mma_bf16_16816(c, a, blk.k[j][1].z, blk.k[j][1].w);
      }
      const int key = kb + 8 * j + 2 * t;
      sc0[j] = key < k1 ? c[0] * p.scale_log2e : -INFINITY;
      sc1[j] = key + 1 < k1 ? c[1] * p.scale_log2e : -INFINITY;
      bmax = fmaxf(bmax, fmaxf(sc0[j], sc1[j]));
    }
    bmax = fmaxf(bmax, __shfl_xor_sync(kFullMask, bmax, 1));
    bmax = fmaxf(bmax, __shfl_xor_sync(kFullMask, bmax, 2));
    const float m_new = fmaxf(m, bmax);          // finite: key kb of the block is always valid
    const float corr = exp2f(m - m_new);
    m = m_new;
    l *= corr;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      out.o0[i] *= corr;
      out.o1[i] *= corr;
    }
    // probabilities -> output
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      const float p0 = exp2f(sc0[ks] - m_new), p1 = exp2f(sc1[ks] - m_new);
      l += p0 + p1;
      const uint32_t a0 = __float_as_uint(p0), a2 = __float_as_uint(p1);
      const uint4 va = blk.v[ks][0], vb = blk.v[ks][1];
#pragma unroll
      for (int jn = 0; jn < 8; ++jn) {
        const uint32_t wa = word_of(va, jn >> 1), wb = word_of(vb, jn >> 1);
        const uint32_t b0 = (jn & 1) ? (wa & 0xffff0000u) : (wa << 16);
        const uint32_t b1 = (jn & 1) ? (wb & 0xffff0000u) : (wb << 16);
        float c[4] = {out.o0[jn], out.o1[jn], 0.f, 0.f};
        mma_tf32_1688(c, a0, a2, b0, b1);
        out.o0[jn] = c[0];
        out.o1[jn] = c[1];
      }
    }
  }
  l += __shfl_xor_sync(kFullMask, l, 1);
  l += __shfl_xor_sync(kFullMask, l, 2);
  out.m = m;
  out.l = l;
}

// ---- merge unit: one query head; polls the P partial records of that head (eight at a time, all
// loads in flight together), merges them with a running maximum and writes attn_out.
template <class S>
__device__ __forceinline__ void attn_merge(Worker<S>& s, const Params& p, int ph, int gph, int head, int P, unsigned tagw) {
  constexpr int HD = S::HD, DPL = S::HD / 32;
  constexpr int kBatch = 8;
  const unsigned rtag = p.launch_seq * (unsigned)num_phases(p.num_layers) + (unsigned)gph + 1u;   // unique per (step, phase)
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
}

// ---- phase 1: attention.  CTA c < NKV * Pc computes CTA-part (kv head c / Pc, part c % Pc): warp w takes
// blocks (part * 8 + w) * bpw .. + bpw, the eight partials meet in shared memory (the x buffers of the
// neighbouring phases are free during this one) and 256 threads merge them, one (query head, dim) each.
// Pc == 1 (T <= 256): that is attn_out.  Otherwise the merged partial is a record, and merge unit m (query head m)
// on warp 0 of CTA NKV * Pc + m polls the Pc records of its head.
template <class S>
__device__ __forceinline__ void phase_attn(Worker<S>& s, const Params& p, unsigned char* smem, int ph, int gph) {
  using L = SmemLayout<S>;
  constexpr int HD = S::HD, GQA = S::GQA;
  static_assert(GQA * HD == kThreads, "the in-CTA merge gives every thread one (head, dim)");
  static_assert(kWorkers == kAttnWarps, "attn_plan counts eight compute warps per CTA");
  static_assert(kWorkers * GQA * HD * 4 <= 2 * L::kActSmall && L::kOffActB == L::kOffActA + L::kActSmall,
                "the partial outputs use both small activation buffers");
  int bpw, Pc;
  const int T = step_pos<S>(p, smem) + 1;
  attn_plan(T, bpw, Pc);
  const int cta = (int)blockIdx.x;
  const int n_compute = S::NKV * Pc;
  const int n_merge = Pc > 1 ? S::NH : 0;
  const unsigned tagw = phase_tag(p, gph) << 16;
  if (cta >= n_compute) {   // no staging, no barrier on these CTAs
    if (cta < n_compute + n_merge && s.w == 0 && !s.aborted) {
      const long long tq1 = clock64();
      attn_merge(s, p, ph, gph, cta - n_compute, Pc, tagw);
      trace_put(p, ph, 6, (unsigned long long)(clock64() - tq1), s.lane);
    }
    return;
  }
  const bool tagged = p.sync && (ph > p.phase_begin || p.wait_first);
  const long long tq0 = clock64();
  const int kvh = cta / Pc, part = cta % Pc;
  const int k0 = (part * kAttnWarps + s.w) * bpw * kAttnBlockKeys;
  int k1 = k0 + bpw * kAttnBlockKeys;
  if (k1 > T) k1 = T;
  const int kend = (part + 1) * kAttnWarps * bpw * kAttnBlockKeys;           // end of the CTA-part
  const int part_keys = (kend < T ? kend : T) - part * kAttnWarps * bpw * kAttnBlockKeys;
  const int n_active = (part_keys + bpw * kAttnBlockKeys - 1) / (bpw * kAttnBlockKeys);   // warps that have keys
  const bool has = k0 < T && !s.aborted;
  KvBlock<S> blk;   // (its first rows have been on their way since the QKV phase started: prefetch_attn_rows)
  if (!s.aborted && !stage_attn_part<S>(s, p, smem, tagged, phase_tag(p, gph - 1), ph)) flag_abort(s, smem);
  cta_sync(s, smem);
  if (s.cta_abort) return;
  const long long tq1 = clock64();
  if (s.w == 0) trace_put(p, ph, 0, globaltimer_ns(), s.lane);

  float* opart = reinterpret_cast<float*>(smem + L::kOffActA);              // [warp][head of the group][HD]
  float* mlpart = reinterpret_cast<float*>(smem + L::kOffActD + S::QDIM * 2);   // [warp][head][m, l] (behind the bf16 q)
  if (has) {
    AttnPartial r;
    attn_blocks<S>(p, smem, phase_layer(ph), kvh, k0, k1, tagged, L::kKvStage && gph > p.phase_begin, blk, s.w, s.lane, r,
                   T - 1);
    const int g = s.lane >> 2, t = s.lane & 3;
    if (g < GQA) {
      float4* dst = reinterpret_cast<float4*>(opart + ((size_t)(s.w * GQA + g) * HD + 16 * t));
      dst[0] = make_float4(r.o0[0], r.o0[1], r.o0[2], r.o0[3]);
      dst[1] = make_float4(r.o0[4], r.o0[5], r.o0[6], r.o0[7]);
      dst[2] = make_float4(r.o1[0], r.o1[1], r.o1[2], r.o1[3]);
      dst[3] = make_float4(r.o1[4], r.o1[5], r.o1[6], r.o1[7]);
      if (t == 0) *reinterpret_cast<float2*>(mlpart + (size_t)(s.w * GQA + g) * 2) = make_float2(r.m, r.l);
    }
  }
  if (s.w == 0) trace_put(p, ph, 1, globaltimer_ns(), s.lane);
  cta_sync(s, smem);
  if (s.cta_abort) return;
  if (s.w == 0) trace_put(p, ph, 4, globaltimer_ns(), s.lane);
  {
    // merge over the warps that had keys: thread = (head h of the group, dim d)
    const int tid = s.w * 32 + s.lane, h = tid / HD, d = tid % HD;
    float M = -INFINITY;
    for (int w = 0; w < n_active; ++w) M = fmaxf(M, mlpart[(w * GQA + h) * 2]);
    float num = 0.f, den = 0.f;
    for (int w = 0; w < n_active; ++w) {
      const float wgt = exp2f(mlpart[(w * GQA + h) * 2] - M);
      den = fmaf(wgt, mlpart[(w * GQA + h) * 2 + 1], den);
      num = fmaf(wgt, opart[(size_t)(w * GQA + h) * HD + d], num);
    }
    const int head = kvh * GQA + h;
    if (Pc == 1) {
      const unsigned short bits = f32_to_bf16_bits(num / den);
      p.attn_out[head * HD + d] = bits;
      if (p.sync) st_handoff(p.t_attn + head * HD + d, (uint32_t)bits | tagw);
    } else {
      const unsigned rtag = p.launch_seq * (unsigned)num_phases(p.num_layers) + (unsigned)gph + 1u;
      unsigned long long* rec = part_record<S>(p, head, part);
      st_handoff(reinterpret_cast<uint32_t*>(rec + d), make_uint2(__float_as_uint(num), rtag));
      if (d == 0) st_handoff(reinterpret_cast<uint4*>(rec + HD), make_uint4(__float_as_uint(M), rtag, __float_as_uint(den), rtag));
    }
  }
  if (s.w == 0) {
    trace_put(p, ph, 3, (unsigned long long)(tq1 - tq0), s.lane);
    trace_put(p, ph, 6, (unsigned long long)(clock64() - tq1), s.lane);
    trace_put(p, ph, 7, globaltimer_ns(), s.lane);
  }
}

// The attention phase as a real function call: its register allocation (a K / V block is 64 registers) stays
// out of the streaming loop's, and the other way round.  Takes and returns the two abort flags of the warp.
template <class S>
static __device__ __noinline__ unsigned phase_attn_call(const Params& p, unsigned char* smem, int ph, int lane, int w,
                                                        unsigned aborted, int gph) {
  Worker<S> s;
  s.lane = lane;
  s.w = w;
  s.nwt = (int)gridDim.x * kWorkers;
  s.g = (int)blockIdx.x * kWorkers + w;
  s.aborted = aborted != 0u;
  s.cta_abort = false;
  phase_attn(s, p, smem, ph, gph);
  return (s.aborted ? 1u : 0u) | (s.cta_abort ? 2u : 0u);
}

}  // namespace qmk
