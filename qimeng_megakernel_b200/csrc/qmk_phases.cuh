// Worker-side phase bodies of the decode megakernel.  Included by qmk_kernel.cuh.
//
// All weight-streaming phases (QKV, O-proj, up/gate, down, LM head) share ONE instance of the hot
// loop (acquire tile -> tensor-pipe product -> release) and differ only in their epilogue;
// keeping a single copy keeps the persistent kernel's code footprint small.
#pragma once

namespace qmk {

// Residual stream input of a layer: hidden_states, or the embedding row of *token_in for layer 0
// when the step is fed a token id (the reference does `hidden_states.copy_(embed[ids])` on the
// host side, qimeng_megakernel/models/LLM/decode.py:1376-1377).
template <class S>
__device__ __forceinline__ const uint16_t* residual_src(Worker<S>& s, const Params& p, int layer, int ph, bool wait, int gph) {
  const int step = (S::kMulti && layer == 0) ? gph / num_phases(p.num_layers) : 0;
  if (layer == 0 && (p.token_in != nullptr || step > 0)) {
    // (wait: the QKV phase, which is the first to need the token of a later step; the O-projection reads the word the
    // QKV phase of the same step has already seen)
    long long tok = step == 0 ? __ldcg(p.token_in)
                  : (wait ? wait_token(p, p.launch_seq + (unsigned)step, s.w, ph, s.lane)
                          : (long long)(unsigned)(__ldcg(p.tok_word) & 0xffffffffull));
    if (tok < 0 && step > 0) return nullptr;
    if (tok < 0) tok = 0;
    if (tok >= p.vocab) tok = p.vocab - 1;
    return p.embed + (size_t)tok * S::H;
  }
  return p.hidden;
}

__device__ __forceinline__ unsigned long long argmax_key(unsigned short bits, int row) {
  return ((unsigned long long)float_ordered_bits(bf16_bits_to_f32(bits)) << 32) | (0xffffffffu - (unsigned)row);
}

// ---- epilogues: lane i of a batch holds the fp32 sums of the batch's i-th item -------------------

// QKV item = one RoPE pair (rows 2u, 2u+1).  fused_rms_qkvproj_gemv_rope (operations.py:151-215):
// the GEMV result is rounded to bf16 (einsum on bf16 tensors), the rotation is fp32 with separately
// rounded products, the result is rounded to bf16 and written to q_post_rope / the KV cache row and,
// tagged, to the scratch the attention phase of this step reads.
template <class S>
__device__ __forceinline__ void epilogue_qkv(const Params& p, const unsigned char* smem, int layer, int unit,
                                             float a, float b, unsigned tagw, int pos) {
  const float* rope = reinterpret_cast<const float*>(smem + SmemLayout<S>::kOffRope);
  const int row = 2 * unit;
  a = bf16_round(a);
  b = bf16_round(b);
  constexpr int kStart = S::NH * S::HD;
  constexpr int vStart = kStart + S::NKV * S::HD;
  uint32_t packed;
  uint16_t* dst;
  uint32_t* tdst;
  if (row < vStart) {
    const int d = row % S::HD;
    const float c0 = rope[d], c1 = rope[d + 1], s0 = rope[S::HD + d], s1 = rope[S::HD + d + 1];
    const float o0 = __fadd_rn(__fmul_rn(a, c0), __fmul_rn(-b, s0));
    const float o1 = __fadd_rn(__fmul_rn(b, c1), __fmul_rn(a, s1));
    packed = pack_bf16x2(o0, o1);
    if (row < kStart) {
      dst = p.q_post_rope + row;
      tdst = p.t_q + row;
    } else {
      dst = p.k_cache + (size_t)layer * p.kv_layer_stride + (size_t)pos * p.kv_seq_stride + (row - kStart);
      tdst = p.t_q + S::QDIM + (row - kStart);
    }
  } else {
    packed = pack_bf16x2(a, b);
    dst = p.v_cache + (size_t)layer * p.kv_layer_stride + (size_t)pos * p.kv_seq_stride + (row - vStart);
    tdst = p.t_q + S::QDIM + S::NKV * S::HD + (row - vStart);
  }
  if (row < kStart) *reinterpret_cast<uint32_t*>(dst) = packed;
  else st_keep_u32(dst, packed, l2_policy_evict_last());   // a KV-cache row: keep it in L2 for the coming steps
  if (p.sync) st_handoff(tdst, make_uint2((packed & 0xffffu) | tagw, (packed >> 16) | tagw));
}

// SwiGLU item = (up row u, gate row u).  fused_mlp_upgate (operations.py:265-282): up and gate rounded
// to bf16, silu(gate) rounded to bf16, product rounded to bf16.
__device__ __forceinline__ unsigned short epilogue_silu(float up, float gate) {
  const float g = bf16_round(gate);
  const float sl = bf16_round(g / (1.0f + __expf(-g)));
  return f32_to_bf16_bits(sl * bf16_round(up));
}

// ---- the streaming phase -----------------------------------------------------------------------
// An item is what one lane of the epilogue owns: a QKV RoPE pair or SwiGLU unit (one tile each), or a
// row of O-proj / LM head (two rows per tile) or of down-proj (two rows per I/2048 tiles, one tile
// per k-slice, each slice against its own 2048 activations).
// Residual phases (fused_oproj_gemv_residual, operations.py:251-262; fused_mlp_down_residual, 285-295):
// hidden[r] = bf16(hidden[r] + bf16(W[r,:] . x)).  One warp owns a whole down-proj row, so its K
// reduction has a fixed order (the reference adds four split-K partials with bf16 CAS in arrival
// order, decode_kernel/down_proj_gemv_residual.cu:39-52, 225-234).
// LM head (fused_rms_lmhead_gemv, operations.py:303-321) also keeps the arg-max of the bf16 logits,
// lowest index on ties, replacing `logits.argmax()` of the host loop (decode.py:1391-1395).
template <class S>
__device__ __forceinline__ void phase_stream(Worker<S>& s, const Params& p, unsigned char* smem, int ph, int kind, int gph) {
  using L = SmemLayout<S>;
  constexpr int kSlices = S::I / kChunkElems;
  static_assert(S::QDIM == kChunkElems && S::H == kChunkElems, "rows of QKV/O/up/gate/LM must be one chunk");
  const int layer = phase_layer(ph);
  const bool tagged = p.sync && (ph > p.phase_begin || p.wait_first);
  const unsigned tag_in = phase_tag(p, gph - 1);
  const unsigned tagw = phase_tag(p, gph) << 16;
  const bool normed = kind == kQkv || kind == kUpGate || kind == kLmHead;
  const int sbuf = small_buf_index(ph, p.num_layers);
  unsigned char* act = smem + (kind == kDown ? L::kOffActD : (sbuf ? L::kOffActB : L::kOffActA));
  float* sumsq = reinterpret_cast<float*>(smem + L::kOffCtl) + kCtlSumSq + sbuf * 8;
  const long long tq0 = clock64();

  // ---- stage this warp's eighth of the phase input (see qmk_staging.cuh)
  if (kind == kDown) {
    Part<S::I> part;
    if (!s.aborted) {
      if (fetch_part<S::I>(s, p, p.t_silu, p.silu_out, tagged, tag_in, ph, part)) store_part(part, act, s.w, s.lane);
      else flag_abort(s, smem);
    }
    cta_sync(s, smem);
  } else {
    Part<S::H> part;
    uint2 gains[Part<S::H>::NPL];
    if (normed) {   // the gains do not depend on the step: fetch them before polling for the activations
      const uint16_t* gsrc = kind == kQkv ? p.attn_norm + (size_t)layer * S::H
                                          : (kind == kUpGate ? p.mlp_norm + (size_t)layer * S::H : p.lm_norm);
      const uint2* g2 = reinterpret_cast<const uint2*>(gsrc + s.w * Part<S::H>::kElems);
#pragma unroll
      for (int j = 0; j < Part<S::H>::NPL; ++j) gains[j] = __ldg(g2 + j * 32 + s.lane);
    }
    const uint32_t* tsrc = kind == kOproj ? p.t_attn : (kind == kUpGate ? p.t_hid_o : p.t_hid_d);
    const uint16_t* psrc = kind == kOproj ? p.attn_out
                                          : (kind == kQkv || (kind == kLmHead && p.num_layers == 0)
                                                 ? residual_src<S>(s, p, layer, ph, true, gph) : p.hidden);
    if (!s.aborted && (psrc == nullptr || !fetch_part<S::H>(s, p, tsrc, psrc, tagged, tag_in, ph, part))) flag_abort(s, smem);
    if (normed) {
      const float ss = s.aborted ? 0.f : part_sumsq(part);
      if (s.lane == 0) sumsq[s.w] = ss;
      cta_sync(s, smem);
      if (s.cta_abort) return;
      float tot = 0.f;
#pragma unroll
      for (int j = 0; j < kWorkers; ++j) tot += sumsq[j];
      normalise_part(part, gains, rsqrtf(tot * (1.0f / S::H) + p.eps));
    }
    if (!s.aborted) store_part(part, act, s.w, s.lane);
    cta_sync(s, smem);
  }
  if (s.cta_abort) return;
  const long long tq1 = clock64();
  // (after the poll, not before it: loads that a warp issues behind these copies wait for them)
  // First K/V block of the coming attention phase -> shared memory.  Issued from the up/gate phase of the layer before
  // (the staging area is free from the end of that layer's attention on, and the copy then has ten microseconds to
  // land); the first layer of a launch does it in its own QKV phase.
  if (!s.aborted) {
    if (kind == kUpGate && layer + 1 < p.num_layers && ph + 3 < p.phase_end)
      prefetch_attn_rows<S>(p, smem, layer + 1, s.w, s.lane, step_pos<S>(p, smem));
    if (kind == kQkv && (layer == 0 || ph - 2 < p.phase_begin)) prefetch_attn_rows<S>(p, smem, layer, s.w, s.lane, step_pos<S>(p, smem));
  }

  int i0, i1;
  switch (kind) {
    case kQkv: i0 = s.cur.q0; i1 = s.cur.q1; break;
    case kUpGate: i0 = s.cur.u0; i1 = s.cur.u1; break;
    case kLmHead: i0 = s.cur.l0; i1 = s.cur.l1; break;
    default: i0 = s.cur.r0; i1 = s.cur.r1; break;
  }
  const bool unit_tiles = kind == kQkv || kind == kUpGate;   // one item per tile (else two rows per tile)
  const int nsl = kind == kDown ? kSlices : 1;
  unsigned long long best = 0ull;
  if (i0 < i1 && !s.aborted) {
    XFrag xf;
    if (nsl == 1) load_xfrag(xf, act, s.lane);
    const bool residual = kind == kOproj || kind == kDown;
    const uint16_t* res = kind == kOproj ? residual_src<S>(s, p, layer, ph, false, gph) : p.hidden;
    uint32_t* tres = kind == kOproj ? p.t_hid_o : p.t_hid_d;
#pragma unroll 1
    for (int ib = i0; ib < i1 && !s.aborted; ib += 32) {
      const int nb = (i1 - ib) < 32 ? (i1 - ib) : 32;
      // residual value of this lane's row: kept in a register from phase to phase for the first
      // 32 rows of the warp, re-read (this thread wrote it) for any further rows.
      float old = 0.f;
      if (residual && s.lane < nb) {
        if (ib == i0 && s.res_valid) old = s.res;
        else old = bf16_bits_to_f32(ldcg_u16(res + ib + s.lane));
      }
      float va = 0.f, vb = 0.f;
      const int step = unit_tiles ? 1 : 2;
#pragma unroll 1
      for (int i = 0; i < nb; i += step) {
        float cc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
        for (int k = 0; k < nsl; ++k) {
          if (nsl > 1) load_xfrag(xf, act + k * kChunkBytes, s.lane);
          consume_tile(s, p, ph, cc, xf, unit_tiles || (i + 1 < nb));
        }
        float sa, sb;
        diag_reduce(cc, s.lane, sa, sb);
        if (s.lane == i) {
          va = sa;
          vb = sb;
        }
        if (!unit_tiles && s.lane == i + 1) va = sb;
      }
      if (s.aborted) flag_abort(s, smem);
      if (s.lane < nb && !s.aborted) {
        const int item = ib + s.lane;
        switch (kind) {
          case kQkv: epilogue_qkv<S>(p, smem, layer, item, va, vb, tagw, step_pos<S>(p, smem)); break;
          case kUpGate: {
            const unsigned short bits = epilogue_silu(va, vb);
            p.silu_out[item] = bits;
            if (p.sync) st_handoff(p.t_silu + item, (uint32_t)bits | tagw);
            break;
          }
          case kLmHead: {
            const unsigned short bits = f32_to_bf16_bits(va);
            p.logits[item] = bits;
            const unsigned long long key = argmax_key(bits, item);
            best = key > best ? key : best;
            break;
          }
          default: {
            const unsigned short bits = f32_to_bf16_bits(old + bf16_round(va));
            p.hidden[item] = bits;
            if (p.sync) st_handoff(tres + item, (uint32_t)bits | tagw);
            if (ib == i0) s.res = bf16_bits_to_f32(bits);
            break;
          }
        }
      }
      if (residual && ib == i0) s.res_valid = true;
    }
  }
  if (s.w == 0) {
    trace_put(p, ph, 3, (unsigned long long)(tq1 - tq0), s.lane);
    trace_put(p, ph, 6, (unsigned long long)(clock64() - tq1), s.lane);
  }
  if (p.trace != nullptr && s.lane == 0) {   // per CTA: earliest and latest end of the streaming loop over its warps
    unsigned long long* t = p.trace + ((size_t)blockIdx.x * num_phases(p.num_layers) + ph) * 8;
    const unsigned long long now = globaltimer_ns();
    atomicMax(t + 1, now);
    atomicMax(t + 0, ~now);
    atomicMax(t + 4, (unsigned long long)(clock64() - tq1));
  }
  if (kind != kLmHead) return;

  // LM head: warp -> CTA -> grid arg-max.  Every warp arrives, also those without rows.
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(kFullMask, best, o);
    best = other > best ? other : best;
  }
  if (s.lane == 0 && !s.aborted) {
    unsigned* ctl = reinterpret_cast<unsigned*>(smem + L::kOffCtl);
    unsigned long long* cta_key = reinterpret_cast<unsigned long long*>(ctl + kCtlKey);
    atomicMax(cta_key, best);
    __threadfence();
    if (atomicAdd(ctl + kCtlLmArrive, 1u) == (unsigned)(kWorkers - 1)) {
      unsigned long long k;
      if constexpr (S::kMulti) {   // both words are left zero for the launch's next step
        k = atomicExch(cta_key, 0ull);
        ctl[kCtlLmArrive] = 0u;
      } else {
        k = atomicMax(cta_key, 0ull);
      }
      atomicMax(p.argmax_key, k);
      __threadfence();
      unsigned* lm_ticket = p.tickets + 64;
      if (atomicAdd(lm_ticket, 1u) == gridDim.x - 1) {
        __threadfence();
        const unsigned long long win = atomicMax(p.argmax_key, 0ull);
        const long long tok = (long long)(0xffffffffu - (unsigned)(win & 0xffffffffull));
        if (p.next_token) *p.next_token = tok;
        const int step = S::kMulti ? gph / num_phases(p.num_layers) : 0;
        const long long at = (long long)p.pos + step + 1;
        if (p.out_tokens && at < p.out_tokens_len) p.out_tokens[at] = tok;
        *p.argmax_key = 0ull;
        *lm_ticket = 0u;
        __threadfence();
        // the token hand-off to the launch's next step, after the resets it must not overtake
        if constexpr (S::kMulti)
          st_handoff(reinterpret_cast<uint32_t*>(p.tok_word), make_uint2((unsigned)tok, p.launch_seq + (unsigned)step + 1u));
      }
    }
  }
}

}  // namespace qmk

#include "qmk_attention.cuh"
