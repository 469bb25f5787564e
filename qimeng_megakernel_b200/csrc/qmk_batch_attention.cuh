// Attention phase of the batched decode kernel: eight workers (warps) per CTA, one (sequence, kv head, key range) item
// per warp at a time.  Included by qmk_batch_kernel.cuh.
//
// fused_decode_attention of the reference (fused/operations.py:218-248) for [B, ...] state with per-row positions; its
// CUDA phases are decode_attention_splitkv.cu / decode_attention_reduction.cu (log2-domain softmax, partials merged by
// their log-sum-exp).  Here the inputs are polled as tagged words (q and this step's K / V row come from the QKV phase's
// scratch, older rows from the cache), scores and P.V run in fp32 on the CUDA cores, and when a (sequence, kv head) is
// split over several key ranges every range leaves a self-validating record {acc, max, sum}; the warp that owns the
// last range folds all of them in range order.
#pragma once

namespace qmkb {

template <int HD, int GQ>
static __device__ __noinline__ void attention_items(const Ctx& c, int ph, int layer, int aw) {
  const BParams& p = *c.p;
  constexpr int LPR = HD / 8;          // lanes per K/V row (16 bytes each)
  constexpr int KPL = 32 / LPR;        // keys per load instruction
  const int lane = c.lane;
  const int sub = lane / LPR, dl = lane % LPR;
  const int* pos_s = reinterpret_cast<const int*>(c.smem + Smem::kOffPos);
  const int* act_s = reinterpret_cast<const int*>(c.smem + Smem::kOffAct);
  const int NW = (int)gridDim.x * 8, gw = (int)blockIdx.x * 8 + aw;
  const int Tmax = (int)c.ctl[kCTmax];
  const int seqs = p.B * p.NKV;
  const int kdim = p.NKV * HD;
  int ck, nch;
  attn_plan(Tmax, seqs, NW, ck, nch);
  const int items = seqs * nch;
  constexpr int REC = GQ * (HD + 2);
  const unsigned in_tagw = tag16(p, ph - 1) << 16, out_tagw = tag16(p, ph) << 16;
  const unsigned rtag = tag32(p, ph);
  bool first_item = true;
#pragma unroll 1
  for (int item = gw; item < items; item += NW) {
    const int ch = item % nch, sq = item / nch;
    const int kvh = sq % p.NKV, b = sq / p.NKV;
    const int T = pos_s[b] + 1;
    const int nsplit = (T + ck - 1) / ck;
    uint16_t* outp = p.attn_out + (size_t)b * p.QDIM + (size_t)kvh * GQ * HD;
    uint32_t* toutp = p.t_attn + (size_t)b * p.QDIM + (size_t)kvh * GQ * HD;
    if (!act_s[b]) {   // fused_decode_attention zeroes the output of an inactive row (operations.py:226-231)
      if (ch == 0)
        for (int i = lane; i < GQ * HD / 8; i += 32) {
          reinterpret_cast<uint4*>(outp)[i] = make_uint4(0, 0, 0, 0);
          st_tagged8(toutp + i * 8, make_uint4(0, 0, 0, 0), out_tagw);
        }
      continue;
    }
    if (ch >= nsplit) continue;
    const int k_lo = ch * ck, k_hi = min(T, k_lo + ck);
    bool alive = true;
    float q[GQ][8], acc[GQ][8], m[GQ], l[GQ];
    // q of the group's heads and, for the range that holds it, this step's own K / V row (key T - 1) come from the QKV
    // phase's tagged words: all pieces are fetched together and again until every word carries the tag
    uint4 kcur = make_uint4(0, 0, 0, 0), vcur = make_uint4(0, 0, 0, 0);
    {
      const uint32_t* qsrc = p.t_q + (size_t)b * p.QDIM + (size_t)(kvh * GQ) * HD + dl * 8;
      const uint32_t* ksrc = p.t_kv + ((size_t)b * 2 + 0) * kdim + (size_t)kvh * HD + dl * 8;
      const uint32_t* vsrc = ksrc + kdim;
      const bool own_row = k_hi == T;
      uint4 qa[GQ], qb[GQ], ka2 = make_uint4(in_tagw, in_tagw, in_tagw, in_tagw), kb3 = ka2, va2 = ka2, vb3 = ka2;
      const long long t0 = clock64();
      for (unsigned it = 1;; ++it) {
#pragma unroll
        for (int g = 0; g < GQ; ++g) { qa[g] = poll_ld_u4(qsrc + g * HD); qb[g] = poll_ld_u4(qsrc + g * HD + 4); }
        if (own_row) { ka2 = poll_ld_u4(ksrc); kb3 = poll_ld_u4(ksrc + 4); va2 = poll_ld_u4(vsrc); vb3 = poll_ld_u4(vsrc + 4); }
        bool ok = tags4_ok(ka2, in_tagw) && tags4_ok(kb3, in_tagw) && tags4_ok(va2, in_tagw) && tags4_ok(vb3, in_tagw);
#pragma unroll
        for (int g = 0; g < GQ; ++g) ok = ok && tags4_ok(qa[g], in_tagw) && tags4_ok(qb[g], in_tagw);
        if (ok) break;
        if ((it & 7u) == 0u && poll_expired(c, t0, ph, qa[0].x >> 16, in_tagw >> 16, 9)) { alive = false; break; }
      }
      kcur = untag8(ka2, kb3);
      vcur = untag8(va2, vb3);
#pragma unroll
      for (int g = 0; g < GQ; ++g) {
        const uint4 qv = untag8(qa[g], qb[g]);
        const uint32_t* w = reinterpret_cast<const uint32_t*>(&qv);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          q[g][2 * j] = bf_lo(w[j]) * p.scale_log2e;
          q[g][2 * j + 1] = bf_hi(w[j]) * p.scale_log2e;
        }
        m[g] = -INFINITY;
        l[g] = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[g][j] = 0.f;
      }
    }
    if (!__all_sync(kFullMask, alive)) return;
    if (first_item && aw == 0 && lane == 0) trace_put(p, ph, 0);
    first_item = false;
    const size_t base = (size_t)layer * p.kv_layer_stride + (size_t)b * p.kv_batch_stride + (size_t)kvh * HD + dl * 8;
    // one key for every lane group of LPR lanes: score by shuffles, online softmax in the log2 domain
    auto use_key = [&](const uint4& kq, const uint4& vq, bool valid) {
      const uint32_t* kw = reinterpret_cast<const uint32_t*>(&kq);
      const uint32_t* vw = reinterpret_cast<const uint32_t*>(&vq);
      float kf[8], vf[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        kf[2 * j] = bf_lo(kw[j]); kf[2 * j + 1] = bf_hi(kw[j]);
        vf[2 * j] = bf_lo(vw[j]); vf[2 * j + 1] = bf_hi(vw[j]);
      }
#pragma unroll
      for (int g = 0; g < GQ; ++g) {
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) s += q[g][j] * kf[j];
#pragma unroll
        for (int o = 1; o < LPR; o <<= 1) s += __shfl_xor_sync(kFullMask, s, o);
        if (valid) {
          const float mn = fmaxf(m[g], s);
          const float corr = exp2f(m[g] - mn);     // 0 when m was -inf
          const float pe = exp2f(s - mn);
          l[g] = l[g] * corr + pe;
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[g][j] = acc[g][j] * corr + pe * vf[j];
          m[g] = mn;
        }
      }
    };
    // this step's own row first (its registers are free afterwards), then the rows of the cache
    if (k_hi == T) use_key(kcur, vcur, sub == 0);
    const int k_end = min(k_hi, T - 1);
    // Cache keys are taken in half-blocks of NLD row pieces per lane (16 keys at head_dim 64, 8 at 128), double-buffered
    // in registers: the loads of the next half-block are in flight while this one is multiplied.
    constexpr int NLD = 4;
    constexpr int KBK = NLD * KPL;
    auto load_block = [&](uint4 (&kk)[NLD], uint4 (&vv)[NLD], int ks) {
#pragma unroll
      for (int i = 0; i < NLD; ++i) {
        const int k = ks + i * KPL + sub;
        kk[i] = k < k_end ? ldcg_u4(p.k_cache + base + (size_t)k * p.kv_seq_stride) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int i = 0; i < NLD; ++i) {
        const int k = ks + i * KPL + sub;
        vv[i] = k < k_end ? ldcg_u4(p.v_cache + base + (size_t)k * p.kv_seq_stride) : make_uint4(0, 0, 0, 0);
      }
    };
    auto use_block = [&](const uint4 (&kk)[NLD], const uint4 (&vv)[NLD], int ks) {
#pragma unroll
      for (int i = 0; i < NLD; ++i) use_key(kk[i], vv[i], ks + i * KPL + sub < k_end);
    };
    uint4 ka[NLD], va[NLD], kb2[NLD], vb2[NLD];
    load_block(ka, va, k_lo);
#pragma unroll 1
    for (int k0 = k_lo; k0 < k_end; k0 += 2 * KBK) {
      load_block(kb2, vb2, k0 + KBK);          // (past the end: nothing is loaded, nothing is used)
      use_block(ka, va, k0);
      load_block(ka, va, k0 + 2 * KBK);
      use_block(kb2, vb2, k0 + KBK);
    }
    // merge the KPL key sub-streams (lanes with equal dl)
#pragma unroll
    for (int o = LPR; o < 32; o <<= 1) {
#pragma unroll
      for (int g = 0; g < GQ; ++g) {
        const float mo = __shfl_xor_sync(kFullMask, m[g], o);
        const float lo_ = __shfl_xor_sync(kFullMask, l[g], o);
        const float mn = fmaxf(m[g], mo);
        const float ca = mn == -INFINITY ? 0.f : exp2f(m[g] - mn);
        const float cb = mn == -INFINITY ? 0.f : exp2f(mo - mn);
        l[g] = l[g] * ca + lo_ * cb;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float ao = __shfl_xor_sync(kFullMask, acc[g][j], o);
          acc[g][j] = acc[g][j] * ca + ao * cb;
        }
        m[g] = mn;
      }
    }
    if (nsplit == 1) {
      if (sub == 0) {
#pragma unroll
        for (int g = 0; g < GQ; ++g) {
          const float inv = 1.0f / l[g];
          uint4 o4;
          o4.x = pack_bf16x2(acc[g][0] * inv, acc[g][1] * inv);
          o4.y = pack_bf16x2(acc[g][2] * inv, acc[g][3] * inv);
          o4.z = pack_bf16x2(acc[g][4] * inv, acc[g][5] * inv);
          o4.w = pack_bf16x2(acc[g][6] * inv, acc[g][7] * inv);
          st_tagged8(toutp + g * HD + dl * 8, o4, out_tagw);
          *reinterpret_cast<uint4*>(outp + g * HD + dl * 8) = o4;
        }
      }
      __threadfence();   // (push the tagged words out; nothing waits for this fence)
      continue;
    }
    // this range's record: {acc[HD], max, sum} per query head, every value with the tag
    unsigned long long* rec = p.attn_rec + (size_t)item * REC;
    if (sub == 0) {
#pragma unroll
      for (int g = 0; g < GQ; ++g) {
        unsigned long long* dst = rec + g * (HD + 2) + dl * 8;
#pragma unroll
        for (int j = 0; j < 4; ++j) st_rec2(dst + 2 * j, make_rec(acc[g][2 * j], rtag), make_rec(acc[g][2 * j + 1], rtag));
        if (dl == 0) st_rec2(rec + g * (HD + 2) + HD, make_rec(m[g], rtag), make_rec(l[g], rtag));
      }
    }
    __threadfence();     // (push the records out; nothing waits for this fence)
    if (ch != nsplit - 1) continue;
    // The owner of the last range folds the nsplit records of this (sequence, kv head) in range order: every lane takes
    // (head, 8 dims) pieces; the records of range s + 1 are in flight while range s is folded.
    const unsigned long long* recs = p.attn_rec + (size_t)(sq * nch) * REC;
    const long long t0 = clock64();
    for (int piece = lane; piece < GQ * LPR; piece += 32) {
      const int g = piece / LPR, dd = piece % LPR;
      float M = -INFINITY, L = 0.f, o[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      auto fetch = [&](ulonglong2 (&v)[5], int s) {
        const unsigned long long* rr = recs + (size_t)s * REC + g * (HD + 2);
        v[4] = poll_ld_rec2(rr + HD);
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = poll_ld_rec2(rr + dd * 8 + 2 * j);
      };
      auto fold = [&](ulonglong2 (&v)[5], int s) {
        for (unsigned it = 1; alive; ++it) {
          bool ok = true;
#pragma unroll
          for (int j = 0; j < 5; ++j) ok = ok && rec_ok(v[j].x, rtag) && rec_ok(v[j].y, rtag);
          if (ok) break;
          if ((it & 7u) == 0u && poll_expired(c, t0, ph, (unsigned)(v[4].x >> 32), rtag, 10)) { alive = false; break; }
          fetch(v, s);
        }
        const float ms = rec_val(v[4].x), ls = rec_val(v[4].y);
        const float mn = fmaxf(M, ms);
        const float c0 = exp2f(M - mn), c1 = exp2f(ms - mn);
        L = L * c0 + ls * c1;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          o[2 * j] = o[2 * j] * c0 + rec_val(v[j].x) * c1;
          o[2 * j + 1] = o[2 * j + 1] * c0 + rec_val(v[j].y) * c1;
        }
        M = mn;
      };
      ulonglong2 ra[5], rb[5];
      fetch(ra, 0);
#pragma unroll 1
      for (int s = 0; s < nsplit && alive; s += 2) {
        if (s + 1 < nsplit) fetch(rb, s + 1);
        fold(ra, s);
        if (s + 1 < nsplit) {
          if (s + 2 < nsplit) fetch(ra, s + 2);
          fold(rb, s + 1);
        }
      }
      if (alive) {
        const float inv = 1.0f / L;
        uint4 o4;
        o4.x = pack_bf16x2(o[0] * inv, o[1] * inv);
        o4.y = pack_bf16x2(o[2] * inv, o[3] * inv);
        o4.z = pack_bf16x2(o[4] * inv, o[5] * inv);
        o4.w = pack_bf16x2(o[6] * inv, o[7] * inv);
        st_tagged8(toutp + g * HD + dd * 8, o4, out_tagw);
        *reinterpret_cast<uint4*>(outp + g * HD + dd * 8) = o4;
      }
    }
    __threadfence();
    if (!__all_sync(kFullMask, alive)) return;
  }
}

static __device__ __noinline__ void attention_phase(const Ctx& c, int ph, int aw) {
  const BParams& p = *c.p;
  if (!c.aborted()) {
    const int layer = phase_layer(p, ph), gq = p.NH / p.NKV;
    if (p.HD == 64) {
      if (gq == 4) attention_items<64, 4>(c, ph, layer, aw);
      else if (gq == 2) attention_items<64, 2>(c, ph, layer, aw);
      else attention_items<64, 1>(c, ph, layer, aw);
    } else {
      if (gq == 4) attention_items<128, 4>(c, ph, layer, aw);
      else if (gq == 2) attention_items<128, 2>(c, ph, layer, aw);
      else attention_items<128, 1>(c, ph, layer, aw);
    }
  }
  if (aw == 0 && c.lane == 0) trace_put(p, ph, 5);
}

}  // namespace qmkb
