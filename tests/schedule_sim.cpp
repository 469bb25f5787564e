// CPU replay of the megakernel's weight-tile schedule (qimeng_megakernel_b200/csrc/qmk_schedule.h).
// For a grid of `nsm` CTAs x `warps` workers it walks every worker's TileCursor through all phases and
// checks that (1) within each phase every 4-KiB chunk of the phase's weight matrix is fetched exactly
// once, (2) a worker's tiles come in phase order and their count per phase is what the consumer loop
// expects, (3) every copy is 16-byte aligned and inside its matrix.  Exit code 0 = all good.
#include <cstdio>
#include <cstdlib>
#include <map>
#include <vector>

#include "qmk_schedule.h"

using namespace qmk;
using S = ShapeLlama1B;

static int fail(const char* what, int a = 0, int b = 0, int c = 0) {
  std::fprintf(stderr, "FAIL: %s (%d, %d, %d)\n", what, a, b, c);
  return 1;
}

int run(int nsm, int warps, int layers, int vocab, int phase_begin, int phase_end) {
  const int nwt = nsm * warps;
  // virtual address space: matrices far apart, 4-KiB aligned
  const size_t GB = 1ull << 30;
  StreamBases w;
  unsigned char* base = reinterpret_cast<unsigned char*>(0x100000000ull);
  w.qkv = base;
  w.o_proj = base + 8 * GB;
  w.up = base + 16 * GB;
  w.gate = base + 32 * GB;
  w.down = base + 48 * GB;
  w.lm_head = base + 64 * GB;
  struct Mat { const unsigned char* b; size_t bytes; };
  auto mat = [&](int kind, int layer, int which) -> Mat {
    switch (kind) {
      case kQkv: return {w.qkv + (size_t)layer * S::QKV_ROWS * kChunkBytes, (size_t)S::QKV_ROWS * kChunkBytes};
      case kOproj: return {w.o_proj + (size_t)layer * S::H * kChunkBytes, (size_t)S::H * kChunkBytes};
      case kUpGate: return {(which ? w.gate : w.up) + (size_t)layer * S::I * kChunkBytes, (size_t)S::I * kChunkBytes};
      case kDown: return {w.down + (size_t)layer * S::H * S::I * 2, (size_t)S::H * S::I * 2};
      default: return {w.lm_head, (size_t)vocab * kChunkBytes};
    }
  };
  const int nph = num_phases(layers);
  if (phase_end > nph) phase_end = nph;
  // coverage counters per (phase) -> chunk index -> count ; up/gate use two maps
  std::vector<std::map<size_t, int>> cover(nph * 2);
  for (int g = 0; g < nwt; ++g) {
    TileCursor<S> cur;
    cur.init(g, nwt, vocab, phase_begin);
    cur.seek(w, layers, phase_end);
    int last_ph = -1;
    std::vector<int> count(nph, 0);
    while (!cur.done(phase_end)) {
      const int ph = cur.ph, kind = cur.kind;
      if (ph < last_ph) return fail("phase order", g, ph, last_ph);
      last_ph = ph;
      if (kind != phase_kind(ph, layers)) return fail("kind mismatch", g, ph, kind);
      const int expect_tiles = cur.tiles(kind);
      const Tile t = cur.next(w, layers, phase_end);
      ++count[ph];
      if (count[ph] > expect_tiles) return fail("too many tiles", g, ph, count[ph]);
      const int layer = phase_layer(ph);
      auto account = [&](const unsigned char* p, uint32_t bytes, int which) -> int {
        if ((reinterpret_cast<uintptr_t>(p) & 15u) || (bytes & 15u)) return fail("alignment", g, ph);
        const Mat m = mat(kind, layer, which);
        if (p < m.b || p + bytes > m.b + m.bytes) return fail("outside matrix", g, ph, which);
        for (uint32_t o = 0; o < bytes; o += kChunkBytes) cover[ph * 2 + which][(size_t)(p + o - m.b) / kChunkBytes]++;
        return 0;
      };
      if (account(t.a, t.bytes_a, 0)) return 1;
      if (t.b && account(t.b, kChunkBytes, kind == kUpGate ? 1 : 0)) return 1;
      if (kind == kUpGate && (t.b == nullptr || t.bytes_a != (uint32_t)kChunkBytes)) return fail("up/gate tile shape", g, ph);
      if (kind == kQkv && (t.b != nullptr || t.bytes_a != 2u * kChunkBytes)) return fail("qkv tile shape", g, ph);
    }
    // the consumer loop of a phase takes exactly tiles(kind) tiles
    TileCursor<S> ref;
    ref.init(g, nwt, vocab, phase_begin);
    for (int ph = phase_begin; ph < phase_end; ++ph) {
      const int kind = phase_kind(ph, layers);
      const int want = kind == kAttn ? 0 : ref.tiles(kind);
      if (count[ph] != want) return fail("tile count", g, ph, count[ph]);
    }
  }
  for (int ph = phase_begin; ph < phase_end; ++ph) {
    const int kind = phase_kind(ph, layers), layer = phase_layer(ph);
    if (kind == kAttn) continue;
    for (int which = 0; which < (kind == kUpGate ? 2 : 1); ++which) {
      const Mat m = mat(kind, layer, which);
      const size_t chunks = m.bytes / kChunkBytes;
      const auto& c = cover[ph * 2 + which];
      if (c.size() != chunks) return fail("coverage size", ph, (int)c.size(), (int)chunks);
      for (const auto& kv : c)
        if (kv.second != 1) return fail("chunk fetched more than once", ph, (int)kv.first, kv.second);
    }
  }
  return 0;
}

// attn_plan: the CTA-parts cover every block exactly once, fit the grid, and a merge needs at most one batch.
int run_attn_plan() {
  for (int T = 1; T <= 70000; T += (T < 3000 ? 1 : 977)) {
    int bpw, Pc;
    attn_plan(T, bpw, Pc);
    const int nblk = (T + kAttnBlockKeys - 1) / kAttnBlockKeys;
    if (bpw < 1 || Pc < 1 || Pc > kMaxCtaParts) return fail("attn plan range", T, bpw, Pc);
    if (Pc * kAttnWarps * bpw < nblk) return fail("attn plan does not cover the keys", T, bpw, Pc);
    if ((Pc - 1) * kAttnWarps * bpw >= nblk) return fail("attn plan has an empty part", T, bpw, Pc);
    if (T <= kAttnWarps * kAttnBlockKeys && Pc != 1) return fail("short context needs no second merge", T, bpw, Pc);
  }
  return 0;
}

// A launch of several steps: every worker's stream is its one-step stream, repeated, and ends after the last step.
int run_multi_step(int nsm, int warps, int layers, int vocab, int steps) {
  using S = ShapeLlama1BSteps;   // (the cursor of the multi-step kernel instance)
  StreamBases w;
  unsigned char* base = reinterpret_cast<unsigned char*>(uintptr_t(1) << 40);
  w.qkv = base; w.o_proj = base + (size_t(1) << 36); w.up = base + (size_t(2) << 36); w.gate = base + (size_t(3) << 36);
  w.down = base + (size_t(4) << 36); w.lm_head = base + (size_t(5) << 36);
  const int nwt = nsm * warps, nph = num_phases(layers);
  for (int g = 0; g < nwt; ++g) {
    std::vector<Tile> one;
    TileCursor<S> a;
    a.init(g, nwt, vocab, 0);
    a.seek(w, layers, nph);
    while (!a.done(nph)) one.push_back(a.next(w, layers, nph));
    TileCursor<S> b;
    const int end = steps * nph;      // the stream of a launch of `steps` whole steps ends here
    b.init(g, nwt, vocab, 0);
    b.seek(w, layers, end);
    size_t n = 0;
    while (!b.done(end)) {
      if (one.empty()) return fail("a worker without tiles streams in a multi-step launch", g, 0);
      const Tile t = b.next(w, layers, end), &r = one[n % one.size()];
      if (t.a != r.a || t.b != r.b || t.bytes_a != r.bytes_a) return fail("multi-step stream differs from the repeated step", g, (int)n);
      ++n;
      if (n > one.size() * (size_t)steps) return fail("multi-step stream does not end", g, (int)n);
    }
    if (n != one.size() * (size_t)steps) return fail("multi-step stream length", g, (int)n, (int)(one.size() * steps));
  }
  return 0;
}

int main() {
  struct Case { int nsm, warps, layers, vocab, pb, pe; };
  const Case cases[] = {
      {148, 8, 2, 128256, 0, 1 << 30}, {148, 8, 1, 4096, 0, 1 << 30}, {132, 8, 2, 4097, 0, 1 << 30},
      {8, 8, 1, 1000, 0, 1 << 30},     {1, 8, 1, 37, 0, 1 << 30},      {148, 8, 3, 151936, 5, 11},
      {3, 8, 0, 50304, 0, 1},          {148, 8, 2, 1, 0, 1 << 30},
  };
  for (const Case& c : cases) {
    if (run(c.nsm, c.warps, c.layers, c.vocab, c.pb, c.pe)) {
      std::fprintf(stderr, "case nsm=%d warps=%d layers=%d vocab=%d [%d,%d)\n", c.nsm, c.warps, c.layers, c.vocab, c.pb, c.pe);
      return 1;
    }
  }
  if (run_attn_plan()) return 1;
  if (run_multi_step(148, 8, 2, 128256, 3) || run_multi_step(4, 8, 1, 37, 5) || run_multi_step(148, 8, 0, 4096, 2)) return 1;
  std::puts("schedule ok");
  return 0;
}
