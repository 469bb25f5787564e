// CPU replay of the batched kernel's schedule (qimeng_megakernel_b200/csrc/qmk_batch_schedule.h): for several
// model shapes and grid sizes, walks every CTA's unit range of every phase kind exactly as the device roles do
// and checks that (1) every (row tile, k-block) unit is owned by exactly one CTA, and unit_owner agrees;
// (2) a CTA has at most two partial segments per phase, and no two split tiles of a phase share the CTA that owns
// their first unit, which is what the tile's accumulator slot is keyed on;
// (3) the partial segments of a tile are exactly the CTAs unit_owner(first unit) .. unit_owner(last unit), which
// is what the tile's ticket counts and what the last arriver sums; (4) the split-KV plan keeps its bounds.
#include <cstdio>
#include <algorithm>
#include <map>
#include <set>
#include <vector>

#include "qmk_batch_schedule.h"

using namespace qmkb;

static int fail(const char* what, int a = 0, int b = 0, int c = 0) {
  std::fprintf(stderr, "FAIL: %s (%d, %d, %d)\n", what, a, b, c);
  return 1;
}

static int check_phase(const BParams& p, int kind, int G) {
  const PhaseDims d = phase_dims(p, kind);
  if (d.K % kBlockK != 0 || d.T < 1 || d.KB < 1) return fail("dims", kind, d.K, d.T);
  const int U = d.T * d.KB;
  std::vector<int> owner(U, -1);
  std::map<int, std::vector<int>> partial_of_tile;   // tile -> CTAs with a partial segment
  for (int c = 0; c < G; ++c) {
    int lo, hi;
    unit_range(U, G, c, lo, hi);
    if (lo < 0 || hi > U || lo > hi) return fail("range", c, lo, hi);
    std::set<int> slots_used;
    int u = lo;
    while (u < hi) {   // the segment walk of epilogue_phase
      const int t = u / d.KB, kb_lo = u - t * d.KB;
      const int u_end = hi < (t + 1) * d.KB ? hi : (t + 1) * d.KB;
      const bool full = kb_lo == 0 && u_end == (t + 1) * d.KB;
      for (int x = u; x < u_end; ++x) {
        if (owner[x] != -1) return fail("unit owned twice", x, owner[x], c);
        owner[x] = c;
        if (unit_owner(U, G, x) != c) return fail("unit_owner disagrees", x, unit_owner(U, G, x), c);
      }
      if (!full) {
        const int which = t == lo / d.KB ? 0 : 1;
        if (!slots_used.insert(which).second) return fail("scratch slot used twice in a phase", c, t, which);
        partial_of_tile[t].push_back(c);
      }
      u = u_end;
    }
  }
  for (int x = 0; x < U; ++x)
    if (owner[x] == -1) return fail("unit not owned", x, kind, G);
  std::set<int> acc_slots;
  for (auto& kv : partial_of_tile) {
    const int t = kv.first;
    if (!acc_slots.insert(unit_owner(U, G, t * d.KB)).second) return fail("accumulator slot shared by two split tiles", t, kind, G);
    const int c_first = unit_owner(U, G, t * d.KB), c_last = unit_owner(U, G, (t + 1) * d.KB - 1);
    if ((int)kv.second.size() != tile_segments(U, G, d.KB, t))
      return fail("ticket count", t, (int)kv.second.size(), tile_segments(U, G, d.KB, t));
    // the last arriver walks CTAs c_first..c_last, skips those without units, and must meet exactly the writers
    int i = 0;
    for (int cc = c_first; cc <= c_last; ++cc) {
      int clo, chi;
      unit_range(U, G, cc, clo, chi);
      if (clo == chi) continue;
      if (i >= (int)kv.second.size() || kv.second[i] != cc) return fail("reader meets another CTA than the writers", t, cc, i);
      ++i;
      const int which = t == clo / d.KB ? 0 : 1;
      // writer side: tile t is the CTA's first tile iff it contains unit clo
      if ((which == 0) != (clo >= t * d.KB && clo < (t + 1) * d.KB)) return fail("slot choice", t, cc, which);
    }
    if (i != (int)kv.second.size()) return fail("reader misses a writer", t, i, (int)kv.second.size());
  }
  return 0;
}

int main() {
  struct Shape { int H, I, NH, NKV, HD, V; };
  const Shape shapes[] = {{2048, 8192, 32, 8, 64, 128256}, {1024, 3072, 16, 8, 128, 151936}, {2048, 1024, 16, 16, 128, 50304},
                          {320, 704, 4, 2, 64, 1000}, {256, 512, 2, 2, 128, 777}, {64, 64, 1, 1, 64, 1}};
  const int grids[] = {148, 132, 1, 7, 296};
  for (const Shape& s : shapes)
    for (int G : grids) {
      BParams p{};
      p.H = s.H; p.I = s.I; p.NH = s.NH; p.NKV = s.NKV; p.HD = s.HD; p.vocab = s.V;
      p.QKV_ROWS = (s.NH + 2 * s.NKV) * s.HD;
      p.QDIM = s.NH * s.HD;
      for (int kind : {kQkv, kOproj, kUpGate, kDown, kLmHead})
        if (int rc = check_phase(p, kind, G)) return rc;
    }
  for (int Tmax : {1, 31, 32, 33, 500, 2048, 8192, 100000})
    for (int seqs : {1, 8, 16, 64, 512, 1024})
      for (int NW : {8, 1184}) {
        int ck, nch;
        attn_plan(Tmax, seqs, NW, ck, nch);
        if (ck < 32 || ck % 32 != 0) return fail("ck", Tmax, seqs, ck);
        if (nch < 1 || nch > kMaxSplits || (long long)nch * ck < Tmax) return fail("nch", Tmax, seqs, nch);
        if ((long long)seqs * nch > (long long)NW + seqs && nch > 1) return fail("items bound", Tmax, seqs, nch);
      }
  // The attention key loop's walk over a key range (csrc/qmk_batch_device.cuh, attention_items): blocks of 32 keys at
  // head_dim 64 and 8 at 128; lane (g, t) scores keys kb + 8j + 2t and + 1 of n-tile j, loads K rows kb + 8j + g and V rows
  // kb + 8ks + 2t (+ 1), clamped to the last row of the range.  Every key of the range must be scored exactly once, and
  // no load may leave the range.
  for (int hd : {64, 128})
    for (int k_lo : {0, 32, 96})
      for (int len : {1, 2, 7, 8, 9, 31, 32, 33, 64, 100, 160}) {
        const int k_hi = k_lo + len, NT = hd == 64 ? 4 : 1, BK = NT * 8;
        std::map<int, int> scored;
        for (int kb = k_lo; kb < k_hi; kb += BK)
          for (int lane = 0; lane < 32; ++lane) {
            const int g = lane >> 2, t = lane & 3;
            for (int j = 0; j < NT; ++j) {
              const int krow = std::min(kb + 8 * j + g, k_hi - 1);
              if (krow < k_lo || krow >= k_hi) return fail("K row leaves the range", hd, k_lo, krow);
              for (int e = 0; e < 2; ++e) {
                const int vrow = std::min(kb + 8 * j + 2 * t + e, k_hi - 1);
                if (vrow < k_lo || vrow >= k_hi) return fail("V row leaves the range", hd, k_lo, vrow);
                const int key = kb + 8 * j + 2 * t + e;
                if (g == 0 && key < k_hi) ++scored[key];      // (the four lanes t of a head hold the block's 8 NT scores)
              }
            }
          }
        if ((int)scored.size() != len) return fail("keys scored", hd, k_lo, (int)scored.size());
        for (const auto& kv : scored)
          if (kv.second != 1 || kv.first < k_lo) return fail("key scored twice", hd, kv.first, kv.second);
      }
  std::printf("batch schedule ok\n");
  return 0;
}
