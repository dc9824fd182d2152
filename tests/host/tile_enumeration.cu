// Host-side check of the GEMM kernels' tile enumeration (no GPU needed): for random problems, the tiles that
// get_tile / get_pair_tile hand out must cover every (128-row block, column block) of the output exactly once, stay
// inside one row group, and report the right group.  Built and run by tests/test_tile_enumeration.py.
#include <stdio.h>
#include <stdlib.h>
#include <vector>

#include "../../csrc/gemm_sm100.cu"

using namespace mdt;

// (defined in csrc/comm.cu, which this host program does not link)
extern "C" unsigned long long mdt_peer_wait_limit_ns(void) { return 0; }

static unsigned long long rng_state = 88172645463325252ull;
static int rnd(int n) {
  rng_state ^= rng_state << 13; rng_state ^= rng_state >> 7; rng_state ^= rng_state << 17;
  return (int)(rng_state % (unsigned long long)n);
}

template <int BN_OUT>
static int check(const GemmParams& p, bool pair, const std::vector<int>& offs) {
  const int rows = p.mode == 1 ? offs[p.G] : p.M;
  const int mb = (rows + BM - 1) / BM, nb = (p.N + BN_OUT - 1) / BN_OUT;
  const int groups = p.mode == 2 ? p.G : 1;
  std::vector<int> seen((size_t)groups * mb * nb, 0);
  int bad = 0;
  for (int t = 0;; ++t) {
    int g, m0, n0, second = 0, nkb;
    if (pair) {
      PairTile o;
      if (!get_pair_tile<BN_OUT>(p, t, o)) break;
      g = o.g; m0 = o.m0; n0 = o.n0; second = o.second_ok; nkb = o.num_kb;
    } else {
      Tile o;
      if (!get_tile<BN_OUT>(p, t, o)) break;
      g = o.g; m0 = o.m0; n0 = o.n0; nkb = o.num_kb;
    }
    if (t > 4 * (int)seen.size() + 16) { printf("enumeration does not end\n"); return 1; }
    if (m0 % BM != 0 || n0 % BN_OUT != 0 || n0 >= p.N) { ++bad; continue; }
    for (int h = 0; h < (pair ? 2 : 1); ++h) {
      const int mm = m0 + h * BM;
      if (pair && h == 1 && (!second || mm >= rows)) continue;      // idle half: nothing is stored
      if (mm >= rows) { ++bad; continue; }
      if (p.mode == 1) {
        if (!(offs[g] <= mm && mm + BM <= offs[g + 1])) ++bad;        // the block lies inside the reported group
      }
      if (p.mode == 2) {
        const int want_kb = (offs.empty() ? p.K : offs[g + 1] - offs[g]);
        if (nkb != (want_kb + BK - 1) / BK) ++bad;
      }
      seen[((size_t)(p.mode == 2 ? g : 0) * mb + mm / BM) * nb + n0 / BN_OUT] += 1;
    }
  }
  for (size_t i = 0; i < seen.size(); ++i) {
    // row-grouped problems: blocks of empty padding between groups do not exist (groups are multiples of 128 rows)
    if (seen[i] != 1) ++bad;
  }
  return bad;
}

// The work lists of all CTAs together (get_work, 128-row kernel): every k block of every tile exactly once; whole
// tiles in one piece; a shared tile's pieces come from exactly `contributors` CTAs; at most two pieces per CTA.
template <int BN_OUT>
static int check_work(const GemmParams& p, int num_ctas, const std::vector<int>& offs) {
  const int rows = p.mode == 1 ? offs[p.G] : p.M;
  const int mb = (rows + BM - 1) / BM, nb = (p.N + BN_OUT - 1) / BN_OUT;
  const int kbt = (p.K + BK - 1) / BK + (p.K_l + BK - 1) / BK;
  std::vector<int> covered((size_t)mb * nb * kbt, 0), pieces_of_tile((size_t)mb * nb, 0), claimed((size_t)mb * nb, 0);
  int bad = 0;
  for (int cta = 0; cta < num_ctas; ++cta) {
    int pieces = 0;
    for (int it = 0;; ++it) {
      Work w;
      if (!get_work<BN_OUT>(p, cta, num_ctas, it, w)) break;
      if (it > mb * nb + 4) { printf("work list does not end\n"); return 1; }
      const size_t tile = (size_t)(w.t.m0 / BM) * nb + w.t.n0 / BN_OUT;
      if (w.kb0 < 0 || w.kb1 > kbt || w.kb0 >= w.kb1) { ++bad; continue; }
      for (int kb = w.kb0; kb < w.kb1; ++kb) covered[tile * kbt + kb] += 1;
      if (w.split >= 0) {
        ++pieces;
        pieces_of_tile[tile] += 1;
        if (claimed[tile] != 0 && claimed[tile] != w.contributors) ++bad;
        claimed[tile] = w.contributors;
        if (w.split >= num_ctas) ++bad;                 // the workspace has one tile per CTA
      } else if (w.kb0 != 0 || w.kb1 != kbt) {
        ++bad;                                          // a tile that is not shared is computed whole
      }
    }
    if (pieces > 2) ++bad;
  }
  for (size_t i = 0; i < covered.size(); ++i) if (covered[i] != 1) ++bad;
  for (size_t i = 0; i < claimed.size(); ++i) if (claimed[i] != 0 && claimed[i] != pieces_of_tile[i]) ++bad;
  return bad;
}

int main() {
  int failures = 0, cases = 0;
  for (int it = 0; it < 300; ++it) {
    GemmParams p;
    memset(&p, 0, sizeof(p));
    p.mode = it % 2;
    p.N = 8 * (1 + rnd(600));
    p.K = 8 * (1 + rnd(2000));
    p.K_l = (rnd(3) == 0) ? 16 : 0;
    p.sk_ws = reinterpret_cast<float*>(0x10);           // any non-null value: only tested against NULL
    std::vector<int> offs;
    if (p.mode == 0) {
      p.M = 1 + rnd(3000); p.G = 1;
    } else {
      p.G = 1 + rnd(8);
      offs.push_back(0);
      for (int g = 0; g < p.G; ++g) offs.push_back(offs.back() + BM * rnd(6));
      p.M = offs[p.G];
      p.offsets = offs.data();
    }
    const int ctas[3] = {148, 132, 7};
    for (int c = 0; c < 3; ++c) {
      const int b1 = check_work<256>(p, ctas[c], offs), b2 = check_work<128>(p, ctas[c], offs);
      ++cases;
      if (b1 || b2) {
        ++failures;
        printf("work lists: mode %d M %d N %d K %d K_l %d G %d ctas %d: %d / %d errors\n", p.mode, p.M, p.N, p.K, p.K_l, p.G, ctas[c], b1, b2);
      }
    }
  }
  for (int it = 0; it < 400; ++it) {
    GemmParams p;
    memset(&p, 0, sizeof(p));
    p.mode = it % 3;
    p.N = 8 * (1 + rnd(200));
    p.K = 8 * (1 + rnd(300));
    p.K_l = (rnd(3) == 0) ? 16 : 0;
    std::vector<int> offs;
    if (p.mode == 0) {
      p.M = 1 + rnd(3000); p.G = 1;
    } else if (p.mode == 1) {
      p.G = 1 + rnd(8);
      offs.push_back(0);
      for (int g = 0; g < p.G; ++g) offs.push_back(offs.back() + BM * rnd(6));   // groups of 0..5 blocks
      p.M = offs[p.G];
      p.offsets = offs.data();
    } else {
      p.G = 1 + rnd(4);
      p.M = 8 * (1 + rnd(150));
      if (rnd(2)) {
        offs.push_back(0);
        for (int g = 0; g < p.G; ++g) offs.push_back(offs.back() + BM * rnd(5));
        p.offsets = offs.data();
      } else {
        p.G = 1;
      }
    }
    for (int pair = 0; pair < 2; ++pair) {
      const int b1 = check<256>(p, pair != 0, offs);
      const int b2 = check<128>(p, pair != 0, offs);
      ++cases;
      if (b1 || b2) {
        ++failures;
        printf("mode %d pair %d M %d N %d K %d G %d: %d / %d bad tiles\n", p.mode, pair, p.M, p.N, p.K, p.G, b1, b2);
      }
    }
  }
  printf("%d cases, %d failures\n", cases, failures);
  return failures ? 1 : 0;
}
