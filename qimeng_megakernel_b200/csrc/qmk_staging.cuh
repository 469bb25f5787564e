// Cooperative staging of a phase's activation vector into shared memory.  Included by qmk_kernel.cuh.
//
// The producers of a vector (other SMs, earlier phase of the same step) store every element as one
// 32-bit word {low: bf16 value, high: tag of (step, phase)}.  Each of the CTA's warps polls one
// eighth of the words until all carry the expected tag, writes the bf16 values to shared memory,
// raises part_done[warp] and later waits for the other warps' flags.  When the launch runs a single
// phase on stream order (or for the first phase of a launch) the plain bf16 buffers are read instead.
#pragma once

namespace qmk {

__device__ __forceinline__ bool tags_ok(const uint4& v, unsigned tagw) {
  return (((v.x ^ tagw) | (v.y ^ tagw) | (v.z ^ tagw) | (v.w ^ tagw)) & 0xffff0000u) == 0u;
}

// Poll NPL uint4 per lane (4 tagged words each) starting at word `word0` until every word carries `tag`.
template <int NPL>
__device__ __forceinline__ bool poll_tagged(const Params& p, const uint32_t* tsrc, int word0, unsigned tag, int lane,
                                            int warp, int ph, uint4 (&v)[NPL]) {
  const unsigned tagw = tag << 16;
  const uint4* src = reinterpret_cast<const uint4*>(tsrc + word0) + lane;
  const long long t0 = clock64();
  for (unsigned it = 0;; ++it) {
    bool ok = true;
#pragma unroll
    for (int j = 0; j < NPL; ++j) {
      v[j] = ldcg_u4(src + j * 32);
      ok = ok && tags_ok(v[j], tagw);
    }
    if (__all_sync(kFullMask, ok)) return true;
    if ((it & 15u) == 15u) {
      const bool expired = clock64() - t0 > p.timeout_cycles;
      const unsigned st = ld_relaxed_gpu(p.status + kStCode);
      if (__any_sync(kFullMask, expired || st != 0u)) {
        if (!ok && st == 0u) report_error(p, kErrCounterWait, warp, ph, v[0].x >> 16, tag, lane);
        return false;
      }
    }
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

// This warp's part of an N-element vector -> bf16 in shared memory at dst.  Returns the part's sum of
// squares (warp-reduced) through `ss`.  tsrc: tagged words (used when `tagged`), psrc: plain bf16.
template <int N>
__device__ __forceinline__ bool stage_part_bf16(const Params& p, const uint32_t* tsrc, const uint16_t* psrc, bool tagged,
                                                unsigned tag, unsigned char* dst, int warp, int lane, int ph,
                                                float& ss) {
  constexpr int kPart = N / kWorkers;              // elements per warp
  static_assert(kPart % 128 == 0, "a warp's part must be whole uint4 rounds of tagged words");
  constexpr int NPL = kPart / 128;                 // uint4 of tagged words per lane
  const int e0 = warp * kPart;
  float acc = 0.f;
  if (tagged) {
    uint4 v[NPL];
    if (!poll_tagged<NPL>(p, tsrc, e0, tag, lane, warp, ph, v)) return false;
#pragma unroll
    for (int j = 0; j < NPL; ++j) {
      const uint2 b = untag4(v[j]);
      acc += sumsq4(b);
      *reinterpret_cast<uint2*>(dst + (size_t)(e0 + (j * 32 + lane) * 4) * 2) = b;
    }
  } else {
    const uint2* src = reinterpret_cast<const uint2*>(psrc + e0);
#pragma unroll
    for (int j = 0; j < NPL; ++j) {
      const uint2 b = __ldcg(src + j * 32 + lane);
      acc += sumsq4(b);
      *reinterpret_cast<uint2*>(dst + (size_t)(e0 + (j * 32 + lane) * 4) * 2) = b;
    }
  }
  ss = warp_sum(acc);
  return true;
}

// Raise this warp's staging flag for `ph` (its shared-memory writes are ordered before it).
__device__ __forceinline__ void raise_part_flag(uint32_t ctl, int warp, int lane, unsigned value) {
  __syncwarp();
  if (lane == 0) st_release_cta_shared(ctl + warp * 4, value);
}

// Wait until every warp of the CTA has staged its part of `ph`.
__device__ __noinline__ bool wait_parts(const Params& p, uint32_t ctl, int warp, int lane, int ph) {
  const unsigned want = (unsigned)(ph + 1);
  const long long t0 = clock64();
  for (unsigned it = 0;; ++it) {
    unsigned v = want;
    if (lane < kWorkers) v = ld_acquire_cta_shared(ctl + lane * 4);
    const bool aborted = __any_sync(kFullMask, v == kAbortFlag);
    if (aborted) return false;
    if (__all_sync(kFullMask, v >= want)) return true;
    if ((it & 255u) == 255u && clock64() - t0 > 4 * p.timeout_cycles) {   // outlasts the pollers' own deadline
      if (lane == 0) report_error(p, kErrStageWait, warp, ph, v, want, 0);
      return false;
    }
  }
}

}  // namespace qmk
