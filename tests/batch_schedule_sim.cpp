// CPU replay of the batched kernel's schedule (qimeng_megakernel_b200/csrc/qmk_batch_schedule.h): for several
// model shapes and grid sizes, walks every CTA's unit runs of every phase kind exactly as the device roles do
// and checks that (1) every (row tile, k-block) unit is owned by exactly one CTA and appears exactly once in its runs,
// and unit_owner agrees; (2) a CTA has at most one contributing and at most one finishing partial segment per phase
// (a contributor writes ONE slot, keyed on the CTA); (3) every tile has exactly one segment that holds its last unit
// (the finisher), and the contributors the finisher enumerates with tile_contributor are exactly the CTAs that wrote a
// contributing segment of that tile, in ascending order; (4) the split-KV plan keeps its bounds.
#include <algorithm>
#include <cstdio>
#include <map>
#include <set>
#include <vector>

#include "qmk_batch_schedule.h"

using namespace qmkb;

static int fail(const char* what, int a = 0, int b = 0, int c = 0) {
  std::fprintf(stderr, "FAIL: %s (%d, %d, %d)\n", what, a, b, c);
  return 1;
}

static int check_phase(const BParams& p, int kind, int Gall, int ne = 0) {
  const PhaseDims d = phase_dims(p, kind, ne);
  if (d.K % kBlockK != 0 || d.T < 1 || d.KB < 1) return fail("dims", kind, d.K, d.T);
  const int U = d.T * d.KB;
  const int G = phase_ctas(kind, U, Gall);   // CTAs that share the phase's units (the others have none)
  std::vector<int> owner(U, -1);
  std::map<int, std::vector<int>> contrib_of_tile;   // tile -> CTAs with a contributing segment, in CTA order
  std::map<int, int> finisher_of_tile;               // tile -> CTA that holds its last unit
  for (int c = 0; c < G; ++c) {
    int lo, hi;
    unit_range(U, G, c, lo, hi);
    if (lo < 0 || hi > U || lo > hi) return fail("range", c, lo, hi);
    const UnitRuns R = unit_runs(lo, hi, d.KB);
    int n_contrib = 0, n_finish_partial = 0, seen = 0;
    for (int r = 0; r < 3; ++r) {
      if (R.lo[r] > R.hi[r] || (R.lo[r] < R.hi[r] && (R.lo[r] < lo || R.hi[r] > hi))) return fail("run bounds", c, r, kind);
      int u = R.lo[r];
      while (u < R.hi[r]) {   // the segment walk of the device roles
        const int t = u / d.KB;
        const int u_end = R.hi[r] < (t + 1) * d.KB ? R.hi[r] : (t + 1) * d.KB;
        for (int x = u; x < u_end; ++x) {
          if (owner[x] != -1) return fail("unit owned twice", x, owner[x], c);
          owner[x] = c;
          ++seen;
          if (unit_owner(U, G, x) != c) return fail("unit_owner disagrees", x, unit_owner(U, G, x), c);
        }
        const bool first = seg_first(u, d.KB), last = seg_last(u_end, d.KB);
        if (last) {
          if (finisher_of_tile.count(t)) return fail("two finishers", t, c, kind);
          finisher_of_tile[t] = c;
          if (!first) ++n_finish_partial;
          if (r == 0 && R.hi[1] > R.lo[1]) return fail("a finishing segment must not come first when other runs follow", c, t, kind);
        } else {
          ++n_contrib;
          contrib_of_tile[t].push_back(c);
          if (r != 0) return fail("a contributing segment must be the first run", c, r, kind);
        }
        u = u_end;
      }
    }
    if (seen != hi - lo) return fail("runs do not cover the range", c, seen, hi - lo);
    if (n_contrib > 1 || n_finish_partial > 1) return fail("more than one partial segment of a kind", c, n_contrib, n_finish_partial);
  }
  for (int x = 0; x < U; ++x)
    if (owner[x] == -1) return fail("unit not owned", x, kind, G);
  for (int t = 0; t < d.T; ++t) {
    if (!finisher_of_tile.count(t)) return fail("tile without finisher", t, kind, G);
    if (finisher_of_tile[t] != unit_owner(U, G, (t + 1) * d.KB - 1)) return fail("finisher is not the owner of the last unit", t, kind, G);
    const std::vector<int>& cs = contrib_of_tile[t];
    if ((int)cs.size() != tile_segments(U, G, d.KB, t) - 1) return fail("contributor count", t, (int)cs.size(), tile_segments(U, G, d.KB, t));
    std::vector<int> sorted(cs.begin(), cs.end());
    std::sort(sorted.begin(), sorted.end());
    for (int j = 0; j < (int)sorted.size(); ++j)
      if (tile_contributor(U, G, d.KB, t, j) != sorted[j]) return fail("tile_contributor disagrees", t, j, sorted[j]);
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
      if (s.H == 2048 && s.I == 1024) {   // the mixture-of-experts shape: router tile and the two expert phases
        p.E = 64; p.Ie = 1024; p.ppl = 6; p.topk = 8;
        if (int rc = check_phase(p, kRouter, G)) return rc;
        for (int ne : {1, 8, 33, 64})
          for (int kind : {kEUpGate, kEDown})
            if (int rc = check_phase(p, kind, G, ne)) return rc;
      }
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
  std::printf("batch schedule ok\n");
  return 0;
}
