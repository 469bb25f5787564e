// Cooperative staging of a phase's activation vector into shared memory.  Included by qmk_kernel.cuh.
//
// The producers of a vector (other SMs, earlier phase of the same step) store every element as one
// 32-bit word {low: bf16 value, high: tag of (step, phase)}.  Each of the CTA's warps polls one
// eighth of the words until all carry the expected tag; after a CTA barrier the warp normalises its
// eighth (when the phase starts with RMSNorm) and writes bf16 to shared memory; after a second
// barrier every warp reads the whole vector.  When the launch runs a single phase on stream order
// (or for the first phase of a launch) the plain bf16 buffers are read instead of the tagged words.
#pragma once

namespace qmk {

__device__ __forceinline__ bool tags_ok(const uint4& v, unsigned tagw) {
  return (((v.x ^ tagw) | (v.y ^ tagw) | (v.z ^ tagw) | (v.w ^ tagw)) & 0xffff0000u) == 0u;
}

// Non-inlined tail of a tagged poll: checks the deadline and the global status word.
// Returns true when the poll must give up.
static __device__ __noinline__ bool poll_give_up(const Params& p, long long t0, bool ok, unsigned seen_tag, unsigned tag,
                                          int warp, int ph, int lane) {
  const bool expired = clock64() - t0 > p.timeout_cycles;
  const unsigned st = ld_relaxed_gpu(p.status + kStCode);
  if (__any_sync(kFullMask, expired || st != 0u)) {
    if (!ok && st == 0u) report_error(p, kErrCounterWait, warp, ph, seen_tag, tag, lane);
    return true;
  }
  return false;
}

// While a poll waits, keep the weight stream moving (tensor-memory parking, qmk_kernel.cuh).  A pause between two
// polls only adds latency; the polling traffic itself does not disturb the weight stream (both measured on B200).
template <class S>
__device__ __forceinline__ void poll_backoff(Worker<S>& s, const Params& p, unsigned it) {
  park_one(s, p);
}

// Poll NPL uint4 per lane (4 tagged words each) starting at word `word0` until every word carries `tag`.
template <int NPL, class S>
__device__ __forceinline__ bool poll_tagged(Worker<S>& s, const Params& p, const uint32_t* tsrc, int word0, unsigned tag,
                                            int ph, uint4 (&v)[NPL]) {
  const int lane = s.lane, warp = s.w;
  const unsigned tagw = tag << 16;
  const uint4* src = reinterpret_cast<const uint4*>(tsrc + word0) + lane;
  const long long t0 = clock64();
  for (unsigned it = 0;; ++it) {
    bool ok = true;
#pragma unroll
    for (int j = 0; j < NPL; ++j) v[j] = ldcg_u4(src + j * 32);
    if (it > 0) poll_backoff(s, p, it);   // while the loads are in flight
#pragma unroll
    for (int j = 0; j < NPL; ++j) ok = ok && tags_ok(v[j], tagw);
    if (__all_sync(kFullMask, ok)) return true;
    if ((it & 15u) == 15u && poll_give_up(p, t0, ok, v[0].x >> 16, tag, warp, ph, lane)) return false;
  }
}

// Steps after the first of a multi-step launch: the token fed to the step is the arg-max of the step before, handed over
// as one 64-bit word {token id, tag}; every warp polls it (bounded) before it reads its part of the embedding row.
// Returns -1 when the wait gave up.  A real call with plain arguments: the poll's code and registers stay out of the
// streaming loop (inlined, with the tensor-memory parking that the other polls do while they wait, it cost the whole
// kernel 4 %); the wait is a microsecond per step.
static __device__ __noinline__ long long wait_token(const Params& p, unsigned want, int warp, int ph, int lane) {
  const long long t0 = clock64();
  for (unsigned it = 0;; ++it) {
    const unsigned long long w = __ldcg(p.tok_word);
    const bool ok = (unsigned)(w >> 32) == want;
    if (__all_sync(kFullMask, ok)) return (long long)(unsigned)(w & 0xffffffffull);
    if ((it & 15u) == 15u && poll_give_up(p, t0, ok, (unsigned)(w >> 32), want, warp, ph, lane)) return -1;
  }
}

// 4 tagged words -> 4 bf16 packed in 8 bytes.
__device__ __forceinline__ uint2 untag4(const uint4& v) {
  return make_uint2((v.x & 0xffffu) | (v.y << 16), (v.z & 0xffffu) | (v.w << 16));
}
__device__ __forceinline__ float sumsq4(const uint2& b) {
  const float a0 = bf_lo(b.x), a1 = bf_hi(b.x), a2 = bf_lo(b.y), a3 = bf_hi(b.y);
  return fmaf(a0, a0, fmaf(a1, a1, fmaf(a2, a2, a3 * a3)));
}

// Fetch this warp's part of an N-element vector into registers: v[j] holds elements
// e0 + (j*32 + lane)*4 .. +3 as packed bf16.  tsrc: tagged words (polled when `tagged`), psrc: plain bf16.
template <int N>
struct Part {
  static constexpr int kElems = N / kWorkers;      // elements per warp
  static constexpr int NPL = kElems / 128;         // 4-element groups per lane
  static_assert(kElems % 128 == 0, "a warp's part must be whole rounds of 32 lanes x 4 elements");
  uint2 v[NPL];
};

template <int N, class S>
__device__ __forceinline__ bool fetch_part(Worker<S>& s, const Params& p, const uint32_t* tsrc, const uint16_t* psrc,
                                           bool tagged, unsigned tag, int ph, Part<N>& part) {
  const int lane = s.lane;
  const int e0 = s.w * Part<N>::kElems;
  if (tagged) {
    uint4 t[Part<N>::NPL];
    if (!poll_tagged<Part<N>::NPL>(s, p, tsrc, e0, tag, ph, t)) return false;
#pragma unroll
    for (int j = 0; j < Part<N>::NPL; ++j) part.v[j] = untag4(t[j]);
  } else {
    const uint2* src = reinterpret_cast<const uint2*>(psrc + e0);
#pragma unroll
    for (int j = 0; j < Part<N>::NPL; ++j) part.v[j] = __ldcg(src + j * 32 + lane);
  }
  return true;
}

template <int N>
__device__ __forceinline__ void store_part(const Part<N>& part, unsigned char* dst, int warp, int lane) {
  const int e0 = warp * Part<N>::kElems;
#pragma unroll
  for (int j = 0; j < Part<N>::NPL; ++j)
    *reinterpret_cast<uint2*>(dst + (size_t)(e0 + (j * 32 + lane) * 4) * 2) = part.v[j];
}

template <int N>
__device__ __forceinline__ float part_sumsq(const Part<N>& part) {
  float acc = 0.f;
#pragma unroll
  for (int j = 0; j < Part<N>::NPL; ++j) acc += sumsq4(part.v[j]);
  return warp_sum(acc);
}

// RMSNorm of the part in registers: y = bf16(g * bf16(x * rstd))  (_rms_norm, fused/operations.py:126-131).
template <int N>
__device__ __forceinline__ void normalise_part(Part<N>& part, const uint2 (&gains)[Part<N>::NPL], float rstd) {
#pragma unroll
  for (int j = 0; j < Part<N>::NPL; ++j) {
    const uint2 x = part.v[j], g = gains[j];
    part.v[j].x = pack_bf16x2(bf_lo(g.x) * bf16_round(bf_lo(x.x) * rstd), bf_hi(g.x) * bf16_round(bf_hi(x.x) * rstd));
    part.v[j].y = pack_bf16x2(bf_lo(g.y) * bf16_round(bf_lo(x.y) * rstd), bf_hi(g.y) * bf16_round(bf_hi(x.y) * rstd));
  }
}

// The 16 x 16 bytes of K and V rows that lane (g = lane / 4, t = lane % 4) needs of the 32-key block starting at kb
// (layout of the tensor-pipe attention, qmk_attention.cuh): i < 8: K, key kb + 8*(i/2) + g, words 4t.. (i even) or
// 16+4t.. (i odd); i >= 8: V, key kb + 8*((i-8)/2) + 2t + (i&1), dims 8g..8g+7.  Keys past k1-1 are clamped.
template <class S>
__device__ __forceinline__ const uint4* kv_piece(const Params& p, int layer, int kvh, int kb, int k1, int lane, int i) {
  const int g = lane >> 2, t = lane & 3;
  const size_t base = (size_t)layer * p.kv_layer_stride + (size_t)kvh * S::HD;
  if (i < 8) {
    int kc = kb + 8 * (i >> 1) + g;
    if (kc > k1 - 1) kc = k1 - 1;
    return reinterpret_cast<const uint4*>(p.k_cache + base + (size_t)kc * p.kv_seq_stride) + ((i & 1) ? 4 + t : t);
  }
  int kc = kb + 8 * ((i - 8) >> 1) + 2 * t + (i & 1);
  if (kc > k1 - 1) kc = k1 - 1;
  return reinterpret_cast<const uint4*>(p.v_cache + base + (size_t)kc * p.kv_seq_stride) + g;
}

// Early fetch for the attention phase that follows a QKV phase.  The KV-cache rows a warp will read there were last
// touched a whole step (2.5 GB of weight traffic) ago; fetched only once q is there, they take 3-5 us under the
// weight stream's load (measured), all of it on the critical path.  So every warp that will have keys (same plan as
// phase_attn) starts copying its first block into shared memory (cp.async: no registers held) when the QKV phase
// starts; each lane copies exactly the pieces it will read back itself, so its own wait_group is all the
// synchronisation needed.  Without room in shared memory the rows are only pulled into L2.
template <class S>
__device__ __forceinline__ void prefetch_attn_rows(const Params& p, unsigned char* smem, int layer, int w, int lane, int pos) {
  using L = SmemLayout<S>;
  int bpw, Pc;
  const int T = pos + 1;
  attn_plan(T, bpw, Pc);
  const int cta = (int)blockIdx.x;
  if (cta >= S::NKV * Pc) return;
  const int kvh = cta / Pc, part = cta % Pc;
  const int k0 = (part * kAttnWarps + w) * bpw * kAttnBlockKeys;
  if (k0 >= T) return;
  int k1 = k0 + bpw * kAttnBlockKeys;
  if (k1 > T) k1 = T;
  if (L::kKvStage) {
    const uint64_t keep = l2_policy_evict_last();
    const uint32_t dst = smem_u32(smem + L::kOffKvStage) + (uint32_t)(w * 16 * 512 + lane * 16);
#pragma unroll
    for (int i = 0; i < 16; ++i) cp_async_keep_16(dst + i * 512, kv_piece<S>(p, layer, kvh, k0, k1, lane, i), keep);
    cp_async_commit();
  } else {
    const size_t base = (size_t)layer * p.kv_layer_stride + (size_t)kvh * S::HD;
    int kc = k0 + lane;
    if (kc > k1 - 1) kc = k1 - 1;
    prefetch_l2_keep(p.k_cache + base + (size_t)kc * p.kv_seq_stride);
    prefetch_l2_keep(p.v_cache + base + (size_t)kc * p.kv_seq_stride);
  }
}

// CTA barrier followed by a look at the CTA's abort word.  Every warp of the CTA executes the same
// sequence of these (also warps that have given up), so a bounded wait that expires in one warp
// never leaves the others stuck at a barrier.
template <class S>
__device__ __forceinline__ void cta_sync(Worker<S>& s, const unsigned char* smem) {
  __syncthreads();
  if (reinterpret_cast<const volatile unsigned*>(smem + SmemLayout<S>::kOffCtl)[kCtlAbort] != 0u) s.cta_abort = true;
}
template <class S>
__device__ __forceinline__ void flag_abort(Worker<S>& s, unsigned char* smem) {
  s.aborted = true;
  if (s.lane == 0) reinterpret_cast<volatile unsigned*>(smem + SmemLayout<S>::kOffCtl)[kCtlAbort] = 1u;
}

}  // namespace qmk
