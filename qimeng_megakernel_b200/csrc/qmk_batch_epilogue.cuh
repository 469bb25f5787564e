// Epilogues of the batched decode kernel: what happens to a finished accumulator tile [128 weight rows][batch].
// Included by qmk_batch_kernel.cuh.  The arithmetic of every case follows the reference's fused PyTorch ops (cited per
// case); outputs go to the caller's bf16 buffers AND, tagged, to the scratch the next phase polls.
#pragma once

namespace qmkb {

__device__ __forceinline__ unsigned short silu_mul(float up, float gate) {
  // fused_mlp_upgate (operations.py:265-282): both products rounded to bf16, SiLU rounded, product rounded
  const float g = bf16_round(gate);
  const float sl = bf16_round(g / (1.0f + __expf(-g)));
  return f32_to_bf16_bits(sl * bf16_round(up));
}
__device__ __forceinline__ unsigned long long argmax_key(unsigned short bits, int row) {
  return ((unsigned long long)float_ordered_bits(bf16_bits_to_f32(bits)) << 32) | (0xffffffffu - (unsigned)row);
}

// 128 threads (e = thread index in the epilogue group) on the fp32 tile exch[128][Bpad + 1] of row tile t.
__device__ __forceinline__ void epilogue_tile(const Ctx& c, int ph, int kind, int t, int e) {
  const BParams& p = *c.p;
  float* exch = reinterpret_cast<float*>(c.smem + Smem::kOffExch);
  const int* pos_s = reinterpret_cast<const int*>(c.smem + Smem::kOffPos);
  const int* act_s = reinterpret_cast<const int*>(c.smem + Smem::kOffAct);
  const int layer = phase_layer(p, ph);
  const int B = p.B;
  const unsigned tagw = tag16(p, ph) << 16;
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
        const bool live = in_range && b < B && act_s[b < B ? b : 0] != 0;
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
          st_tagged8(p.t_q + (size_t)b * p.QDIM + row, o4, tagw);
          *reinterpret_cast<uint4*>(p.q_post_rope + (size_t)b * p.QDIM + row) = o4;
        } else {
          const int col = is_k ? row - p.QDIM : row - p.QDIM - kdim;
          st_tagged8(p.t_kv + ((size_t)b * 2 + (is_v ? 1 : 0)) * kdim + col, o4, tagw);
          uint16_t* cache = is_k ? p.k_cache : p.v_cache;
          *reinterpret_cast<uint4*>(cache + (size_t)layer * p.kv_layer_stride + (size_t)b * p.kv_batch_stride +
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
      // are combined with shuffles.  A winner is marked by negating its (positive) exponential in place.
      const int tpr = p.Bpad <= 16 ? 8 : (p.Bpad <= 32 ? 4 : 2);
      const int b = e / tpr, q = e % tpr;
      const bool rowok = b < p.Bpad;
      const int bb = rowok ? b : 0;
      const bool act = b < B && act_s[bb] != 0;
      float mx = -INFINITY;
      for (int x = q; x < E; x += tpr) mx = fmaxf(mx, exch[x * p.exch_stride + bb]);
      for (int o = 1; o < tpr; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(kFullMask, mx, o));
      float sum = 0.f;
      for (int x = q; x < E; x += tpr) {
        const float pe = __expf(exch[x * p.exch_stride + bb] - mx);
        if (rowok) exch[x * p.exch_stride + bb] = pe;
        sum += pe;
      }
      for (int o = 1; o < tpr; o <<= 1) sum += __shfl_xor_sync(kFullMask, sum, o);
      const float inv = 1.0f / sum;
      for (int j = 0; j < p.topk; ++j) {
        float best = -1.f;
        int bi = E;
        for (int x = q; x < E; x += tpr) {
          const float v = rowok ? exch[x * p.exch_stride + bb] : 0.f;
          if (v > best) { best = v; bi = x; }
        }
        for (int o = 1; o < tpr; o <<= 1) {
          const float ob = __shfl_xor_sync(kFullMask, best, o);
          const int oi = __shfl_xor_sync(kFullMask, bi, o);
          if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
        }
        if (rowok && bi < E && bi % tpr == q) exch[bi * p.exch_stride + bb] = -best;
      }
      if (rowok)
        for (int x = q; x < E; x += tpr) {
          const float v = exch[x * p.exch_stride + bb];
          exch[x * p.exch_stride + bb] = (act && v < 0.f) ? -v * inv : 0.f;
        }
      named_bar(kBarEpi, 128);
      int* slot_of = reinterpret_cast<int*>(c.smem + Smem::kOffHs);   // [128] (free scratch of the header)
      if (e < E) {
        bool any = false;
        for (int b2 = 0; b2 < B; ++b2) any |= exch[e * p.exch_stride + b2] > 0.f;
        slot_of[e] = any ? 1 : 0;
      }
      named_bar(kBarEpi, 128);
      if (e == 0) {
        int n = 0;
        for (int x = 0; x < E; ++x) {
          if (slot_of[x]) { p.moe_elist[n] = x; slot_of[x] = n++; } else slot_of[x] = -1;
        }
        *p.moe_ne = n;
        atomicAdd(p.moe_ne_sum, (unsigned long long)n);
      }
      named_bar(kBarEpi, 128);
      if (e < E && slot_of[e] >= 0)
        for (int b2 = 0; b2 < kMaxBatch; ++b2) p.moe_w[slot_of[e] * kMaxBatch + b2] = b2 < B ? exch[e * p.exch_stride + b2] : 0.f;
      // the list and the weights are out: fence, then ONE record {count, tag} tells the expert phases of every CTA
      __threadfence();
      named_bar(kBarEpi, 128);
      if (e == 0) st_rec(p.moe_ne_rec, (unsigned long long)(unsigned)*reinterpret_cast<volatile int*>(p.moe_ne) |
                                           ((unsigned long long)tag32(p, ph) << 32));
      break;
    }
    case kEUpGate: {
      // fused_routed_expert_upgate (operations.py:197-219): gate and up rounded to bf16 (a bf16 linear), SiLU(gate) * up
      // in fp32, one rounding.  Tile rows 0..63 are gate rows, 64..127 the up rows of the same units of one expert.
      const int per = p.Ie / kBlockK;
      const int slot = t / per, lt = t % per;
      const int u = e & 63, half = e >> 6;
      const int b0 = half * (p.Bpad / 2), b1 = b0 + p.Bpad / 2;
      for (int b = b0; b < b1 && b < B; ++b) {
        const float g = bf16_round(exch[u * p.exch_stride + b]), up = bf16_round(exch[(64 + u) * p.exch_stride + b]);
        const float v = act_s[b] ? (g / (1.0f + __expf(-g))) * up : 0.f;
        p.t_esilu[((size_t)slot * kMaxBatch + b) * p.Ie + lt * (kTileRows / 2) + u] = (uint32_t)f32_to_bf16_bits(v) | tagw;
      }
      break;
    }
    case kOproj:
    case kEDown:
    case kDown: {
      // hidden[b, row] = bf16(hidden + bf16(projection)), zero projection for inactive rows
      // (fused_oproj_gemv_residual / fused_mlp_down_residual, operations.py:251-262, 285-295).
      // Same (sequence, eight rows) ownership.  The old residual value comes from the tagged words the residual phase
      // before left (this very CTA wrote them: the same CTA finishes row tile t in every residual phase); the sums of
      // squares for the next RMSNorm are reduced over the sixteen row groups by shuffles and leave as one record.
      const int rg = e & 15;
      const int row = t * kTileRows + rg * 8;
      const bool in_range = row < p.H;
      const int nit = (B + 7) / 8;
      const unsigned oldtagw = tag16(p, hidden_source(kind, ph)) << 16;
      const unsigned rtag = tag32(p, ph);
      const long long t0 = clock64();
#pragma unroll 1
      for (int i0 = 0; i0 < nit; i0 += 4) {
        uint4 oa[4], ob[4];
        for (unsigned it = 1;; ++it) {
          bool ok = true;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int b = (e >> 4) + 8 * (i0 + i);
            oa[i] = ob[i] = make_uint4(oldtagw, oldtagw, oldtagw, oldtagw);
            if (i0 + i < nit && in_range && b < B) {
              const uint32_t* src = p.t_hid + (size_t)b * p.H + row;
              oa[i] = poll_ld_u4(src);
              ob[i] = poll_ld_u4(src + 4);
            }
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) ok = ok && tags4_ok(oa[i], oldtagw) && tags4_ok(ob[i], oldtagw);
          if (__all_sync(kFullMask, ok)) break;
          if ((it & 7u) == 0u && __any_sync(kFullMask, poll_expired(c, t0, ph, oa[0].x >> 16, oldtagw >> 16, 8))) break;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if (i0 + i < nit) {
            const int b = (e >> 4) + 8 * (i0 + i);
            const int bb = b < B ? b : 0;
            const bool act = b < B && act_s[bb] != 0;
            const uint4 ov = untag8(oa[i], ob[i]);
            const uint32_t* ow = reinterpret_cast<const uint32_t*>(&ov);
            float nv[8], sq = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float old = (j & 1) ? bf_hi(ow[j >> 1]) : bf_lo(ow[j >> 1]);
              const float add = act ? bf16_round(exch[(rg * 8 + j) * p.exch_stride + bb]) : 0.f;
              nv[j] = bf16_round(old + add);
              sq += nv[j] * nv[j];
            }
            if (in_range && b < B) {
              uint4 o4;
              o4.x = pack_bf16x2(nv[0], nv[1]); o4.y = pack_bf16x2(nv[2], nv[3]);
              o4.z = pack_bf16x2(nv[4], nv[5]); o4.w = pack_bf16x2(nv[6], nv[7]);
              st_tagged8(p.t_hid + (size_t)b * p.H + row, o4, tagw);
              *reinterpret_cast<uint4*>(p.hidden + (size_t)b * p.H + row) = o4;
            } else {
              sq = 0.f;
            }
#pragma unroll
            for (int o = 1; o < 16; o <<= 1) sq += __shfl_xor_sync(kFullMask, sq, o);
            if (rg == 0 && b < B) st_rec(p.ss_rec + (size_t)t * kMaxBatch + b, make_rec(sq, rtag));
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
        for (int b = b0; b < b1 && b < B; ++b) {
          const unsigned short bits =
              act_s[b] ? silu_mul(exch[u * p.exch_stride + b], exch[(64 + u) * p.exch_stride + b]) : (unsigned short)0;
          p.t_silu[(size_t)b * p.I + unit] = (uint32_t)bits | tagw;
          p.silu_out[(size_t)b * p.I + unit] = bits;
        }
      }
      break;
    }
    default: {   // LM head: logits and the per-row arg-max (lowest index on ties)
      const int row = t * kTileRows + e;
      if (row < p.vocab) {
        for (int b = 0; b < B; ++b) {
          const float v = act_s[b] ? exch[e * p.exch_stride + b] : -1e9f;
          p.logits[(size_t)b * p.vocab + row] = f32_to_bf16_bits(v);
        }
      }
      if (e < B) {
        unsigned long long best = 0ull;
        const int nrow = min(kTileRows, p.vocab - t * kTileRows);
        for (int r = 0; r < nrow; ++r) {
          const float v = act_s[e] ? exch[r * p.exch_stride + e] : -1e9f;
          const unsigned long long key = argmax_key(f32_to_bf16_bits(v), t * kTileRows + r);
          best = key > best ? key : best;
        }
        atomicMax(p.argmax_key + e, best);
      }
      break;
    }
  }
}

// Split-K partial tiles meet in a fixed-point accumulator at L2.  fp32 additions in arrival order would make the last
// bit of a sum depend on timing; 64-bit integer additions are associative, so the sum of the partials -- each rounded
// once to a multiple of 2^-36, finer than fp32 resolves above 2^-12 -- is the same whatever order they arrive in.
constexpr float kFixScale = 68719476736.0f;              // 2^36
constexpr double kFixInv = 1.0 / 68719476736.0;
__device__ __forceinline__ long long to_fixed(float v) { return __float2ll_rn(v * kFixScale); }
__device__ __forceinline__ void red_add_s64(long long* addr, long long v) {
  asm volatile("red.relaxed.gpu.global.add.u64 [%0], %1;" ::"l"(addr), "l"(v) : "memory");
}
__device__ __forceinline__ long long exch_zero_s64(long long* addr) {
  long long old;
  asm volatile("atom.relaxed.gpu.global.exch.b64 %0, [%1], %2;" : "=l"(old) : "l"(addr), "l"(0ll) : "memory");
  return old;
}

static __device__ __noinline__ void epilogue_phase(const Ctx& c, int ph, int kind, uint32_t tmem, int e, unsigned& sg) {
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
  if (U == 0) return;
  const int G = phase_ctas(kind, U, (int)gridDim.x);   // CTAs that share this phase's units
  int lo, hi;
  unit_range(U, G, cta, lo, hi);
  const UnitRuns R = unit_runs(lo, hi, d.KB);
  float* exch = reinterpret_cast<float*>(c.smem + Smem::kOffExch);
  const int quarter = c.warp & 3;
  const int r = quarter * 32 + c.lane;           // accumulator row (= tile row) of this thread
  const int nchunk = p.Bpad / 16;
  // accumulators of split tiles: one slot per (area, finishing CTA) -- a CTA finishes at most one split tile per phase
  const size_t slot_elems = (size_t)kTileRows * p.Bpad;
  const int area = gemm_ordinal(p, ph) & 1;
  long long* acc_area = reinterpret_cast<long long*>(p.part_rec) + (size_t)area * gridDim.x * slot_elems;
  unsigned* cnt_area = p.part_cnt + (size_t)area * gridDim.x;
  bool first_acc = true;
#pragma unroll 1
  for (int run = 0; run < 3; ++run) {
    int u = R.lo[run];
#pragma unroll 1
    while (u < R.hi[run]) {
      const int t = u / d.KB;
      const int u_end = min(R.hi[run], (t + 1) * d.KB);
      const bool first = seg_first(u, d.KB), last = seg_last(u_end, d.KB);
      const unsigned buf = sg & 1u;
      const bool ok = __all_sync(kFullMask, mbar_wait(c, c.acc_full(buf), (sg >> 1) & 1u, ph, 6));
      if (e == 0 && first_acc) trace_put(p, ph, 1);
      first_acc = false;
      const int fin_cta = unit_owner(U, G, (t + 1) * d.KB - 1);   // the CTA that finishes tile t
      if (ok) {
        tmem_fence_after_sync();
#pragma unroll 1
        for (int ch = 0; ch < nchunk; ++ch) {
          uint32_t v[16];
          tmem_ld16(v, tmem + ((uint32_t)(quarter * 32) << 16) + buf * (uint32_t)p.Bpad + ch * 16);
          tmem_wait_ld();
          if (last) {     // this CTA finishes the tile: its accumulator goes to the exchange tile
#pragma unroll
            for (int j = 0; j < 16; ++j) exch[r * p.exch_stride + ch * 16 + j] = __uint_as_float(v[j]);
          } else {        // a contribution: added to the tile's fixed-point accumulator at L2, nothing returned
            long long* slot = acc_area + (size_t)fin_cta * slot_elems;
#pragma unroll
            for (int j = 0; j < 16; ++j) red_add_s64(slot + (size_t)(ch * 16 + j) * kTileRows + r, to_fixed(__uint_as_float(v[j])));
          }
        }
        tmem_fence_before_sync();
        mbar_arrive1(c.acc_empty(buf));
        if (!last) {      // every warp announces its quarter once its additions are performed
          __threadfence();
          __syncwarp();
          if (c.lane == 0) red_release_gpu_add(cnt_area + fin_cta, 1u);
        }
      }
      ++sg;
      if (last) {
        bool good = ok;
        if (good && !first) {
          // wait for the 4 * (segments - 1) announcements, then take the sum out of the accumulator (leaving zero for its
          // next user) and add this CTA's own partial, all in fixed point
          const unsigned want = 4u * (unsigned)(tile_segments(U, G, d.KB, t) - 1);
          const long long t0 = clock64();
          for (unsigned it = 1;; ++it) {
            const unsigned have = ld_relaxed_gpu(cnt_area + cta);
            if (have >= want) { (void)ld_acquire_gpu(cnt_area + cta); break; }
            if ((it & 15u) == 0u && poll_expired(c, t0, ph, have, want, 16)) { good = false; break; }
          }
          good = __all_sync(kFullMask, good);
          if (good) {
            long long* slot = acc_area + (size_t)cta * slot_elems;
#pragma unroll 1
            for (int ch = 0; ch < nchunk; ++ch) {
              long long got[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) got[j] = exch_zero_s64(slot + (size_t)(ch * 16 + j) * kTileRows + r);
              float* o = exch + r * p.exch_stride + ch * 16;
#pragma unroll
              for (int j = 0; j < 16; ++j) o[j] = (float)((double)(got[j] + to_fixed(o[j])) * kFixInv);
            }
          }
        }
        // one thread decides for the group whether the tile's epilogue runs (a wait may have given up in one warp only)
        if (!good) c.ctl[kCAbort] = 1u;
        named_bar(kBarEpi, 128);
        if (e == 0) {
          c.ctl[kCFlagEpi] = c.aborted() ? 0u : 1u;
          if (!first) atomicExch(cnt_area + cta, 0u);   // (every warp has seen the count: ready for the slot's next user)
        }
        named_bar(kBarEpi, 128);
        if (c.ctl[kCFlagEpi] != 0u) {
          epilogue_tile(c, ph, kind, t, e);   // (any barrier inside is executed by all 128 threads)
          if (kind != kLmHead) __threadfence();   // push the tagged outputs out; nothing waits for this fence
        }
        named_bar(kBarEpi, 128);           // the exchange tile is free again
      }
      u = u_end;
    }
  }
}

}  // namespace qmkb
