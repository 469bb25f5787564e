// Worker-side phase bodies of the decode megakernel.  Included by qmk_kernel.cuh.
#pragma once

namespace qmk {

// Residual stream input of a layer: hidden_states, or the embedding row of *token_in for layer 0
// when the step is fed a token id (the reference does `hidden_states.copy_(embed[ids])` on the
// host side, qimeng_megakernel/models/LLM/decode.py:1376-1377).
template <class S>
__device__ __forceinline__ const uint16_t* residual_src(const Params& p, int layer) {
  if (layer == 0 && p.token_in != nullptr) {
    long long tok = __ldcg(p.token_in);
    if (tok < 0) tok = 0;
    if (tok >= p.vocab) tok = p.vocab - 1;
    return p.embed + (size_t)tok * S::H;
  }
  return p.hidden;
}

// ---- phase 0: RMSNorm -> QKV GEMV -> interleaved RoPE -> q_post_rope / KV cache append ----
// fused_rms_qkvproj_gemv_rope (operations.py:151-215).  Unit = two adjacent output rows
// (one RoPE pair).  The GEMV result is rounded to bf16 before the rotation, like the einsum
// on bf16 tensors in the reference; the rotation itself is fp32 with separately rounded products.
template <class S>
__device__ __forceinline__ void phase_qkv(Worker<S>& s, const Params& p, unsigned char* smem, int ph) {
  const int layer = phase_layer(ph);
  int u0, u1;
  split_range(S::QKV_ROWS / 2, s.nwt, s.g, u0, u1);
  if (u0 < u1 && wait_staged(s, p, ph)) {
    float x[64];
    const int buf = small_buf_index(ph, p.num_layers);
    load_x64(x, smem + (buf ? SmemLayout<S>::kOffActB : SmemLayout<S>::kOffActA), s.lane);
    for (int u = u0; u < u1 && !s.aborted; ++u) {
      const uint4* c0 = acquire_chunk(s, p, smem, ph);
      float a = warp_sum(dot_chunk(c0, x, s.lane));
      release_chunk(s, p);
      const uint4* c1 = acquire_chunk(s, p, smem, ph);
      float b = warp_sum(dot_chunk(c1, x, s.lane));
      release_chunk(s, p);
      if (s.lane == 0 && !s.aborted) {
        const int row = 2 * u;
        a = bf16_round(a);
        b = bf16_round(b);
        constexpr int kStart = S::NH * S::HD;
        constexpr int vStart = kStart + S::NKV * S::HD;
        if (row < vStart) {
          const int d = row % S::HD;
          const float* cs = p.rope_cos + (size_t)p.pos * S::HD + d;
          const float* sn = p.rope_sin + (size_t)p.pos * S::HD + d;
          const float o0 = __fadd_rn(__fmul_rn(a, cs[0]), __fmul_rn(-b, sn[0]));
          const float o1 = __fadd_rn(__fmul_rn(b, cs[1]), __fmul_rn(a, sn[1]));
          const uint32_t packed = pack_bf16x2(o0, o1);
          if (row < kStart) {
            *reinterpret_cast<uint32_t*>(p.q_post_rope + row) = packed;
          } else {
            uint16_t* dst = p.k_cache + (size_t)layer * p.kv_layer_stride + (size_t)p.pos * p.kv_seq_stride +
                            (row - kStart);
            *reinterpret_cast<uint32_t*>(dst) = packed;
          }
        } else {
          uint16_t* dst = p.v_cache + (size_t)layer * p.kv_layer_stride + (size_t)p.pos * p.kv_seq_stride +
                          (row - vStart);
          *reinterpret_cast<uint32_t*>(dst) = pack_bf16x2(a, b);
        }
      }
    }
  }
  publish(s, p, ph, s.g % kCounterShards);
}

// ---- phase 2: O-projection GEMV + residual.  fused_oproj_gemv_residual (operations.py:251-262):
// hidden[r] = bf16(hidden[r] + bf16(W_o[r,:] . attn_out)).
template <class S>
__device__ __forceinline__ void phase_oproj(Worker<S>& s, const Params& p, unsigned char* smem, int ph) {
  static_assert(S::QDIM == kChunkElems, "O-proj row must be one chunk");
  const int layer = phase_layer(ph);
  int r0, r1;
  split_range(S::H, s.nwt, s.g, r0, r1);
  if (r0 < r1 && wait_staged(s, p, ph)) {
    float x[64];
    const int buf = small_buf_index(ph, p.num_layers);
    load_x64(x, smem + (buf ? SmemLayout<S>::kOffActB : SmemLayout<S>::kOffActA), s.lane);
    const uint16_t* res = residual_src<S>(p, layer);
    for (int r = r0; r < r1 && !s.aborted; ++r) {
      const uint4* c = acquire_chunk(s, p, smem, ph);
      const float acc = warp_sum(dot_chunk(c, x, s.lane));
      release_chunk(s, p);
      if (s.lane == 0 && !s.aborted) {
        const float old = bf16_bits_to_f32(ldcg_u16(res + r));
        p.hidden[r] = f32_to_bf16_bits(old + bf16_round(acc));
      }
    }
  }
  publish(s, p, ph, s.g % kCounterShards);
}

// ---- phase 3: RMSNorm -> up / gate GEMV -> SiLU(gate) * up.  fused_mlp_upgate (operations.py:265-282).
// Rounding points of the reference: up and gate to bf16, silu(gate) to bf16, product to bf16.
template <class S>
__device__ __forceinline__ void phase_upgate(Worker<S>& s, const Params& p, unsigned char* smem, int ph) {
  static_assert(S::H == kChunkElems, "hidden row must be one chunk");
  int u0, u1;
  split_range(S::I, s.nwt, s.g, u0, u1);
  if (u0 < u1 && wait_staged(s, p, ph)) {
    float x[64];
    const int buf = small_buf_index(ph, p.num_layers);
    load_x64(x, smem + (buf ? SmemLayout<S>::kOffActB : SmemLayout<S>::kOffActA), s.lane);
    for (int u = u0; u < u1 && !s.aborted; ++u) {
      const uint4* cu = acquire_chunk(s, p, smem, ph);
      const float up = warp_sum(dot_chunk(cu, x, s.lane));
      release_chunk(s, p);
      const uint4* cg = acquire_chunk(s, p, smem, ph);
      const float gt = warp_sum(dot_chunk(cg, x, s.lane));
      release_chunk(s, p);
      if (s.lane == 0 && !s.aborted) {
        const float g = bf16_round(gt);
        const float sl = bf16_round(g / (1.0f + __expf(-g)));
        p.silu_out[u] = f32_to_bf16_bits(sl * bf16_round(up));
      }
    }
  }
  publish(s, p, ph, s.g % kCounterShards);
}

// ---- phase 4: down-projection GEMV + residual.  fused_mlp_down_residual (operations.py:285-295).
// A row is I/2048 consecutive chunks; one warp owns the whole row, so the K reduction has a fixed
// order (the reference's kernel adds four split-K partials with bf16 CAS in arrival order,
// decode_kernel/down_proj_gemv_residual.cu:39-52, 225-234).
template <class S>
__device__ __forceinline__ void phase_down(Worker<S>& s, const Params& p, unsigned char* smem, int ph) {
  constexpr int kSlices = S::I / kChunkElems;
  int r0, r1;
  split_range(S::H, s.nwt, s.g, r0, r1);
  if (r0 < r1 && wait_staged(s, p, ph)) {
    for (int r = r0; r < r1 && !s.aborted; ++r) {
      float acc = 0.f;
#pragma unroll 1
      for (int k = 0; k < kSlices; ++k) {
        float x[64];
        load_x64(x, smem + SmemLayout<S>::kOffActD + k * kChunkBytes, s.lane);
        const uint4* c = acquire_chunk(s, p, smem, ph);
        acc += dot_chunk(c, x, s.lane);
        release_chunk(s, p);
      }
      acc = warp_sum(acc);
      if (s.lane == 0 && !s.aborted) {
        const float old = bf16_bits_to_f32(ldcg_u16(p.hidden + r));
        p.hidden[r] = f32_to_bf16_bits(old + bf16_round(acc));
      }
    }
  }
  publish(s, p, ph, s.g % kCounterShards);
}

// ---- last phase: RMSNorm -> LM head GEMV -> logits (+ fused argmax).  fused_rms_lmhead_gemv
// (operations.py:303-321); the argmax replaces `logits.argmax()` of the host loop (decode.py:1391-1395):
// maximum of the bf16-rounded logits, lowest index on ties.
template <class S>
__device__ __forceinline__ void phase_lm_head(Worker<S>& s, const Params& p, unsigned char* smem, int ph) {
  int r0, r1;
  split_range(p.vocab, s.nwt, s.g, r0, r1);
  unsigned long long best = 0ull;
  if (r0 < r1 && wait_staged(s, p, ph)) {
    float x[64];
    const int buf = small_buf_index(ph, p.num_layers);
    load_x64(x, smem + (buf ? SmemLayout<S>::kOffActB : SmemLayout<S>::kOffActA), s.lane);
    unsigned short mine = 0;
    for (int r = r0; r < r1 && !s.aborted; ++r) {
      const uint4* c = acquire_chunk(s, p, smem, ph);
      const float acc = warp_sum(dot_chunk(c, x, s.lane));
      release_chunk(s, p);
      const unsigned short bits = f32_to_bf16_bits(acc);
      const unsigned long long key =
          ((unsigned long long)float_ordered_bits(bf16_bits_to_f32(bits)) << 32) | (0xffffffffu - (unsigned)r);
      best = key > best ? key : best;
      const int i = r - r0;
      if ((i & 31) == s.lane) mine = bits;
      if ((i & 31) == 31 || r == r1 - 1) {
        const int base = r0 + (i & ~31);
        if (base + s.lane <= r) p.logits[base + s.lane] = mine;
      }
    }
  }
  // CTA-level then grid-level argmax; every worker arrives, also those without rows.
  __syncwarp();
  if (s.lane == 0 && !s.aborted) {
    unsigned long long* cta_key = reinterpret_cast<unsigned long long*>(smem + SmemLayout<S>::kOffCtl + 8);
    unsigned* arrive = reinterpret_cast<unsigned*>(smem + SmemLayout<S>::kOffCtl + 4);
    atomicMax(cta_key, best);
    __threadfence();
    if (atomicAdd(arrive, 1u) == (unsigned)(kWorkers - 1)) {
      const unsigned long long k = atomicMax(cta_key, 0ull);
      atomicMax(p.argmax_key, k);
      __threadfence();
      unsigned* lm_ticket = p.tickets + 64;
      if (atomicAdd(lm_ticket, 1u) == gridDim.x - 1) {
        __threadfence();
        const unsigned long long win = atomicMax(p.argmax_key, 0ull);
        const long long tok = (long long)(0xffffffffu - (unsigned)(win & 0xffffffffull));
        if (p.next_token) *p.next_token = tok;
        if (p.out_tokens && (long long)p.pos + 1 < p.out_tokens_len) p.out_tokens[p.pos + 1] = tok;
        *p.argmax_key = 0ull;
        *lm_ticket = 0u;
        __threadfence();
      }
    }
  }
}

}  // namespace qmk

#include "qmk_attention.cuh"
