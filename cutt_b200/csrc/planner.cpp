// Plan builder (host only).  See planner.h.
#include "planner.h"
#include "cost_model_data.h"
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <set>

namespace cuttb {

static inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Test aid: build every tile with 64-bit row offsets, so that the kernel variant which tensors of
// 2^32 elements and more select is also exercised by small problems.
static bool g_forceWideOffsets = false;
void debug_force_wide_offsets(bool on) { g_forceWideOffsets = on; }

bool canonicalize(int rank, const int64_t* d, const int64_t* is, const int64_t* os, int elt,
                  int peerDim, Problem& P) {
  struct Dim { int64_t d, is, os; bool peer; };
  std::vector<Dim> v;
  int64_t vol = 1;
  for (int i = 0; i < rank; i++) {
    vol *= d[i];
    if (d[i] == 1 && i != peerDim) continue;
    v.push_back({d[i], is[i], os[i], i == peerDim});
  }
  std::stable_sort(v.begin(), v.end(), [](const Dim& a, const Dim& b) { return a.is < b.is; });
  // fuse neighbours that are contiguous on both sides (the rule of reduceRanks,
  // src/cuttplan.cpp:63-126, stated on strides)
  std::vector<Dim> f;
  for (const Dim& x : v) {
    if (!f.empty()) {
      Dim& b = f.back();
      if (!b.peer && !x.peer && x.is == b.is * b.d && x.os == b.os * b.d) {
        b.d *= x.d;
        continue;
      }
    }
    f.push_back(x);
  }
  if (f.empty()) f.push_back({1, 1, 1, false});
  if ((int)f.size() > kMaxDims) return false;
  P = Problem();
  P.rank = (int)f.size();
  P.elt = elt;
  P.volume = vol;
  P.inElems = vol;
  P.peerDim = -1;
  for (int i = 0; i < P.rank; i++) {
    P.d[i] = f[i].d;
    P.is[i] = f[i].is;
    P.os[i] = f[i].os;
    if (f[i].peer) P.peerDim = i;
  }
  P.identity = (P.rank == 1 && P.is[0] == 1 && P.os[0] == 1 && P.peerDim < 0);
  return true;
}

bool problem_from_cutt(int rank, const int* dim, const int* perm, int elt, Problem& P) {
  std::vector<int64_t> d(rank), is(rank), os(rank);
  int64_t acc = 1;
  for (int i = 0; i < rank; i++) { d[i] = dim[i]; is[i] = acc; acc *= dim[i]; }
  acc = 1;
  for (int k = 0; k < rank; k++) { os[perm[k]] = acc; acc *= dim[perm[k]]; }
  return canonicalize(rank, d.data(), is.data(), os.data(), elt, -1, P);
}

bool problem_from_cutt_ext(int rank, const int* dim, const int* perm, int eltBytes, Problem& P) {
  if (eltBytes == 4 || eltBytes == 8) return problem_from_cutt(rank, dim, perm, eltBytes, P);
  if (eltBytes != 1 && eltBytes != 2 && eltBytes != 16) return false;
  std::vector<int64_t> d(rank + 1), is(rank + 1), os(rank + 1);
  int64_t acc = 1;
  for (int i = 0; i < rank; i++) { d[i + 1] = dim[i]; is[i + 1] = acc; acc *= dim[i]; }
  acc = 1;
  for (int k = 0; k < rank; k++) { os[perm[k] + 1] = acc; acc *= dim[perm[k]]; }
  if (eltBytes == 16) {
    // an unpermuted innermost dimension of two 8-byte words
    d[0] = 2; is[0] = 1; os[0] = 1;
    for (int i = 1; i <= rank; i++) { is[i] *= 2; os[i] *= 2; }
    return canonicalize(rank + 1, d.data(), is.data(), os.data(), 8, -1, P);
  }
  if (!canonicalize(rank, d.data() + 1, is.data() + 1, os.data() + 1, eltBytes, -1, P)) return false;
  if (P.identity || P.is[0] != 1 || P.os[0] != 1) return true;
  for (int unit = 8; unit >= 4; unit /= 2) {
    const int f = unit / eltBytes;  // elements per unit
    if (P.d[0] % f) continue;
    // every other stride is a multiple of the leading extent, hence of f
    Problem Q = P;
    Q.d[0] /= f;
    for (int j = 1; j < Q.rank; j++) { Q.is[j] /= f; Q.os[j] /= f; }
    return canonicalize(Q.rank, Q.d, Q.is, Q.os, unit, -1, P);
  }
  return true;
}

bool problem_from_cutt_chunk(int rank, const int* dim, const int* perm, int elt, int chunk, Problem& P) {
  if (rank < 1 || chunk < 1 || chunk > dim[rank - 1]) return false;
  std::vector<int64_t> d(rank), is(rank), os(rank);
  int64_t acc = 1;
  for (int i = 0; i < rank; i++) { d[i] = i == rank - 1 ? chunk : dim[i]; is[i] = acc; acc *= d[i]; }
  acc = 1;
  for (int k = 0; k < rank; k++) { os[perm[k]] = acc; acc *= dim[perm[k]]; }
  if (!canonicalize(rank, d.data(), is.data(), os.data(), elt, -1, P)) return false;
  // one contiguous block on both sides only if the slab is also contiguous in the output
  return true;
}

bool problem_from_cutt_sharded(int rank, const int* dim, const int* perm, int elt, int world, int me,
                               Problem& P, ShardInfo& info) {
  info = ShardInfo();
  if (rank < 2 || rank > 31 || world < 1 || world > kMaxPeers || me < 0 || me >= world) return false;
  const int last = rank - 1;
  const int s = perm[last];  // input dimension that is slowest in the output
  if (dim[last] % world != 0 || dim[s] % world != 0) return false;
  for (int i = 0; i < rank; i++) info.localDim[i] = dim[i];
  info.localDim[last] = dim[last] / world;
  info.localVolume = 1;
  for (int i = 0; i < rank; i++) info.localVolume *= info.localDim[i];
  if (s == last) {
    info.mode = 0;
    return problem_from_cutt(rank, info.localDim, perm, elt, P);
  }
  info.mode = 1;
  // input strides of the local slab; output strides of one output slab (extent dim[s]/world last)
  std::vector<int64_t> is(rank), os(rank);
  int64_t acc = 1;
  for (int i = 0; i < rank; i++) { is[i] = acc; acc *= info.localDim[i]; }
  acc = 1;
  for (int k = 0; k < rank; k++) {
    os[perm[k]] = acc;
    acc *= (perm[k] == s) ? dim[s] / world : dim[perm[k]];
  }
  // dimensions: all input dims with dim[s] cut to its inner part, plus the peer dimension
  std::vector<int64_t> d2, is2, os2;
  int peer = -1;
  for (int i = 0; i < rank; i++) {
    if (i == s) {
      d2.push_back(dim[s] / world); is2.push_back(is[s]); os2.push_back(os[s]);
      peer = (int)d2.size();
      d2.push_back(world); is2.push_back(is[s] * (dim[s] / world)); os2.push_back(0);
    } else {
      d2.push_back(info.localDim[i]); is2.push_back(is[i]); os2.push_back(os[i]);
    }
  }
  if (!canonicalize((int)d2.size(), d2.data(), is2.data(), os2.data(), elt, peer, P)) return false;
  // this GPU's slab of input dimension `last` lands at this offset of every output slab
  P.outBase = (int64_t)me * info.localDim[last] * os[last];
  P.peerRot = me;
  P.identity = false;
  return true;
}

// chunk of about `want` elements out of d, with equal-sized chunks except possibly the last;
// chunks are rounded up to a multiple of `mult` (vector width) when that is small against them
static int64_t balanced_chunk(int64_t d, int64_t want, int64_t mult = 1) {
  if (want >= d) return d;
  if (want < 1) want = 1;
  int64_t n = ceil_div(d, want);
  int64_t c = ceil_div(d, n);
  if (mult > 1 && c >= 2 * mult) c = ceil_div(c, mult) * mult;
  return c < d ? c : d;
}

static uint32_t ilog2_exact(uint32_t x) { uint32_t l = 0; while ((1u << l) < x) l++; return l; }

// thread split of a side: tq threads along the run, nthreads/tq along the rows,
// minimising the number of loop trips of the busiest thread.
static void choose_thread_split(Side& S, uint32_t nthreads) {
  uint32_t vpr = (uint32_t)ceil_div(S.run, S.vec);
  uint64_t best = ~0ull;
  uint32_t bestTq = 1;
  for (uint32_t tq = 1; tq <= nthreads; tq *= 2) {
    uint32_t tr = nthreads / tq;
    uint64_t trips = (uint64_t)ceil_div(S.nrows, tr) * (uint64_t)ceil_div(vpr, tq);
    // prefer wider tq on ties: neighbouring lanes then touch neighbouring addresses
    if (trips < best || (trips == best && tq <= 32)) { best = trips; bestTq = tq; }
  }
  S.tq = bestTq;
  S.tqShift = ilog2_exact(bestTq);
}

bool build_tile(const Problem& P, const TileParams& tp, const DeviceInfo& dev, Candidate& out,
                std::set<std::string>* seenExtents) {
  const int r = P.rank;
  const int elt = P.elt;
  if (r < 1 || r > kMaxDims) return false;
  int64_t t[kMaxDims];
  for (int j = 0; j < r; j++) t[j] = 1;

  // output order
  int oo[kMaxDims];
  for (int j = 0; j < r; j++) oo[j] = j;
  // (the peer dimension has no output stride: it goes last and never joins a run)
  std::stable_sort(oo, oo + r, [&](int a, int b) {
    if ((a == P.peerDim) != (b == P.peerDim)) return b == P.peerDim;
    return P.os[a] < P.os[b];
  });

  const int64_t tin = std::max<int64_t>(1, tp.tinBytes / elt);
  const int64_t tout = std::max<int64_t>(1, tp.toutBytes / elt);
  const int64_t vtarget = std::max<int64_t>(1, tp.vtargetBytes / elt);
  const int64_t kMaxChunk = 32768;

  // 1. input run: leading dimensions in input order
  {
    int64_t cum = 1, expect = 1;
    for (int j = 0; j < r; j++) {
      if (P.is[j] != expect || j == P.peerDim || cum * 4 >= tin * 3) break;
      int64_t want = ceil_div(tin, cum);
      if (P.d[j] <= want + want / 2 && P.d[j] <= kMaxChunk) {
        t[j] = P.d[j]; cum *= P.d[j]; expect *= P.d[j];
      } else {
        t[j] = balanced_chunk(P.d[j], std::min(want, kMaxChunk), 16 / elt);
        break;
      }
    }
  }
  // 2. output run: leading dimensions in output order
  {
    int64_t cum = 1, expect = 1;
    for (int k = 0; k < r; k++) {
      int j = oo[k];
      if (P.os[j] != expect || j == P.peerDim) break;
      if (t[j] == P.d[j]) { cum *= P.d[j]; expect *= P.d[j]; continue; }
      if (t[j] > 1) break;  // already chunked by the input run: the output run ends here
      if (cum * 4 >= tout * 3) break;
      int64_t want = ceil_div(tout, cum);
      if (P.d[j] <= want + want / 2 && P.d[j] <= kMaxChunk) {
        t[j] = P.d[j]; cum *= P.d[j]; expect *= P.d[j];
      } else {
        t[j] = balanced_chunk(P.d[j], std::min(want, kMaxChunk), 16 / elt);
        break;
      }
    }
  }
  // 3. grow the tile towards the target volume
  auto volume = [&]() { int64_t v = 1; for (int j = 0; j < r; j++) v *= t[j]; return v; };
  auto num_chunked = [&]() { int n = 0; for (int j = 0; j < r; j++) if (t[j] > 1 && t[j] < P.d[j]) n++; return n; };
  for (int guard = 0; guard < 2 * kMaxDims; guard++) {
    int64_t V = volume();
    if (V >= vtarget) break;
    int pick = -1;
    // prefer enlarging a dimension that is already chunked? No: a new row dimension keeps
    // both runs at their target; take the first non-full dimension in the chosen order.
    for (int k = 0; k < r && pick < 0; k++) {
      int j = tp.extend == 0 ? oo[k] : k;
      if (j == P.peerDim) continue;
      if (t[j] < P.d[j]) {
        if (t[j] == 1 && num_chunked() >= 2) continue;  // would create a third chunked dimension
        pick = j;
      }
    }
    if (pick < 0) break;
    int64_t want = ceil_div(vtarget * t[pick], V);
    int64_t nt = balanced_chunk(P.d[pick], std::min(want, kMaxChunk), 16 / elt);
    if (nt <= t[pick]) break;
    t[pick] = nt;
    if (nt < P.d[pick]) break;  // chunked: the target is met (or the chunk limit was hit)
  }
  if (num_chunked() > 2) return false;
  if (seenExtents) {
    // everything below depends only on the extents and these options
    std::string key;
    char kb[64];
    for (int j = 0; j < r; j++) { snprintf(kb, sizeof kb, "%lld,", (long long)t[j]); key += kb; }
    snprintf(kb, sizeof kb, "|%d%d%d%d%d%d%d%d%d%d", tp.nthreads, tp.stages, tp.maxVecBytes, tp.maxVBytes, tp.loopOrder,
             tp.cutInRun, tp.allowAof, tp.groupIn * 16 + tp.groupOut, tp.oneTilePerBlock, tp.peerOrder);
    key += kb;
    if (!seenExtents->insert(key).second) return false;
  }

  // 4. derive descriptor
  TileDesc& D = out.desc;
  memset(&D, 0, sizeof(D));
  D.elt = elt;
  D.nthreads = tp.nthreads;
  D.stages = tp.stages;
  D.peerLoopDim = -1;
  D.inBase = P.inBase;
  D.outBase = P.outBase;

  // partial slots
  int slotOf[kMaxDims];
  int nslots = 0;
  for (int j = 0; j < r; j++) {
    slotOf[j] = -1;
    if (t[j] > 1 && t[j] < P.d[j] && P.d[j] % t[j] != 0) {
      if (nslots == 2) return false;
      slotOf[j] = nslots++;
    }
  }

  // run membership
  bool inRun[kMaxDims] = {false}, outRun[kMaxDims] = {false};
  int inRunLast = -1, outRunLast = -1;
  {
    int64_t expect = 1;
    for (int j = 0; j < r; j++) {
      if (P.is[j] != expect || t[j] == 1 || j == P.peerDim) break;
      if (tp.cutInRun && j > 0 && j == oo[0]) break;
      inRun[j] = true; inRunLast = j;
      if (t[j] < P.d[j]) break;
      expect *= P.d[j];
    }
  }
  int outRunOrder[kMaxDims], nOutRun = 0;
  {
    int64_t expect = 1;
    for (int k = 0; k < r; k++) {
      int j = oo[k];
      if (P.os[j] != expect || t[j] == 1 || j == P.peerDim) break;
      outRun[j] = true; outRunLast = j; outRunOrder[nOutRun++] = j;
      if (t[j] < P.d[j]) break;
      expect *= P.d[j];
    }
  }

  // vector widths (elements per access)
  auto side_vec = [&](bool input) -> uint32_t {
    const bool* inrun = input ? inRun : outRun;
    int last = input ? inRunLast : outRunLast;
    for (int W = std::min(16, tp.maxVecBytes) / elt; W > 1; W /= 2) {
      bool ok = true;
      if (last < 0) { ok = false; }
      else {
        int64_t prefix = 1;
        for (int j = 0; j < r; j++) if (inrun[j] && j != last) prefix *= t[j];
        // every valid run length must be a multiple of W
        if (prefix % W != 0) {
          if (t[last] % W != 0) ok = false;
          if (t[last] < P.d[last] && P.d[last] % W != 0) ok = false;
        }
      }
      for (int j = 0; j < r && ok; j++) {
        int64_t gs = input ? P.is[j] : P.os[j];
        if (inrun[j]) {
          // chunk steps along the run's last dimension
          if (j == last && t[j] < P.d[j] && (gs * t[j]) % W != 0) ok = false;
          continue;
        }
        if (P.d[j] > 1 && gs % W != 0 && !(j == P.peerDim && !input)) ok = false;
      }
      if ((input ? P.inBase : P.outBase) % W != 0) ok = false;
      if (ok) return (uint32_t)W;
    }
    return 1;
  };
  uint32_t win = side_vec(true);
  const uint32_t wout = side_vec(false);

  // 64-bit row offsets are needed when a tile spans 2^32 elements or more on either side
  bool wide = false;
  {
    int64_t spanIn = 1, spanOut = 1;
    for (int j = 0; j < r; j++) { spanIn += (t[j] - 1) * P.is[j]; spanOut += (t[j] - 1) * P.os[j]; }
    wide = spanIn >= (1ll << 32) || spanOut >= (1ll << 32) || g_forceWideOffsets;
  }

  // register blocking of the output side along dimension 0
  uint32_t V = 1;
  if (!wide && r > 0 && t[0] > 1 && inRun[0] && !outRun[0] && P.is[0] == 1) {
    for (int v = std::min(16, tp.maxVBytes) / elt; v > 1; v /= 2) {
      if (t[0] % v == 0 && P.d[0] % v == 0) { V = (uint32_t)v; break; }
    }
  }
  // aligned over-fetch: misaligned input rows are still fetched with 16-byte copies
  const uint32_t VE = 16u / elt;
  bool aof = false;
  if (tp.allowAof && !wide && win < VE && inRunLast >= 0 && P.is[0] == 1 && tp.maxVecBytes >= 16) {
    int64_t run = 1;
    for (int j = 0; j < r; j++) if (inRun[j]) run *= t[j];
    if (run >= 2 * (int64_t)VE) {
      // rows keep their alignment to the widest legal plain vector (winOrig elements), so every
      // displacement is a multiple of it and register blocking up to that width stays possible
      const uint32_t winOrig = win;
      aof = true;
      win = VE;
      while (V > winOrig) V /= 2;
      if (V < 1) V = 1;
    }
  }
  D.aof = aof ? 1 : 0;
  D.inElems = P.inElems;
  D.vblk = V;
  D.vstep = P.os[0];

  // shared-memory strides (elements): input order; rows aligned to A elements; the
  // dimension that starts the output run gets an odd stride (in units of A) and a skew
  const int64_t A = std::max(win, V);
  Skew skewOf[kMaxDims];
  for (int j = 0; j < r; j++) { skewOf[j].shift = 0; skewOf[j].mask = 0; skewOf[j].unitB = 0; }
  int64_t ss[kMaxDims];
  {
    int p0 = nOutRun > 0 ? outRunOrder[0] : -1;
    int64_t s = 1;
    bool slackDone = false;
    for (int j = 0; j < r; j++) {
      if (t[j] == 1) { ss[j] = 0; continue; }
      if (!inRun[j]) {
        if (aof && !slackDone) { s += VE - 1; slackDone = true; }  // room for the row's displacement
        if (j == p0) {
          // lanes per shared-memory wavefront for one output-side access
          uint32_t G = 128u / (V * elt);
          if (wout > 1 && t[j] > (int64_t)G) {
            skewOf[j].shift = ilog2_exact(G);
            skewOf[j].mask = wout - 1;
            skewOf[j].unitB = (uint32_t)(A * elt);
            s += (int64_t)(wout - 1) * A;  // room for the skew inside every row's pitch
          }
          s = ceil_div(s, A) * A;
          while (((s / A) & 1) == 0) s += A;
        } else {
          s = ceil_div(s, A) * A;
        }
      }
      ss[j] = s;
      s = s * t[j];
    }
    int64_t elems = 1 + (aof ? 2 * (int64_t)VE : 0);
    for (int j = 0; j < r; j++)
      if (t[j] > 1) elems += (t[j] - 1) * ss[j] + (skewOf[j].mask ? (int64_t)skewOf[j].mask * A : 0);
    if (elems > (int64_t)dev.maxSmemPerBlock / elt) return false;
    D.tileElems = (uint32_t)elems;
    D.stageBytes = (uint32_t)((elems * elt + 15) / 16 * 16);
  }

  // sides
  auto fill_side = [&](Side& S, bool input) -> bool {
    const bool* inrun = input ? inRun : outRun;
    int last = input ? inRunLast : outRunLast;
    int64_t run = 1, prefix = 1;
    for (int j = 0; j < r; j++) if (inrun[j]) { run *= t[j]; if (j != last) prefix *= t[j]; }
    if (run > 16384) return false;
    S.run = (uint32_t)run;
    S.runPrefix = (uint32_t)prefix;
    S.runSlot = last >= 0 ? slotOf[last] : -1;
    S.vec = input ? win : wout;
    S.nRowDims = 0;
    int64_t nrows = 1;
    for (int j = 0; j < r; j++) {
      if (t[j] == 1 || inrun[j]) continue;
      RowDim& R = S.rowDim[S.nRowDims++];
      const int64_t blk = (!input && j == 0) ? V : 1;
      R.ext = (uint32_t)(t[j] / blk);
      R.div = make_fastdiv(R.ext);
      R.sstrideB = (uint32_t)(ss[j] * blk * elt);
      R.gstride = (input ? P.is[j] : P.os[j]) * blk;
      R.slot = slotOf[j];
      R.cmul = (uint32_t)blk;
      R.skew = skewOf[j];
      R.ishift = (aof && !input && !inRun[j]) ? (uint32_t)(P.is[j] % VE) : 0;
      nrows *= R.ext;
    }
    if (nrows > 8192) return false;
    S.nrows = (uint32_t)nrows;
    choose_thread_split(S, tp.nthreads);
    return true;
  };
  if (!fill_side(D.in, true)) return false;
  if (!fill_side(D.out, false)) return false;
  D.wide = wide ? 1 : 0;

  // gather description of the output run
  D.nOutRunDims = 0;
  for (int k = 0; k < nOutRun; k++) {
    int j = outRunOrder[k];
    RunDim& R = D.outRunDim[D.nOutRunDims++];
    R.div = make_fastdiv((uint32_t)t[j]);
    R.sstrideB = (uint32_t)(ss[j] * elt);
    R.skew = skewOf[j];
    R.ishift = (aof && !inRun[j]) ? (uint32_t)(P.is[j] % VE) : 0;
  }
  if (D.nOutRunDims == 0) {
    D.outRunDim[0].div = make_fastdiv(1);
    D.outRunDim[0].sstrideB = 0;
    D.outRunDim[0].skew = skewOf[0];
    D.outRunDim[0].skew.mask = 0;
    D.outRunDim[0].ishift = 0;
    D.nOutRunDims = 1;
  }
  D.smemGatherContig = 0;
  if (wout > 1 && nOutRun > 0 && V == 1 && !aof) {
    int j0 = outRunOrder[0];
    bool ok = ss[j0] == 1 && t[j0] % wout == 0 && skewOf[j0].mask == 0;
    for (int j = 0; j < r && ok; j++)
      if (j != j0 && t[j] > 1 && (ss[j] % wout != 0 || (skewOf[j].unitB / elt) % wout != 0)) ok = false;
    D.smemGatherContig = ok ? 1 : 0;
  }
  D.tableBytes = table_layout(D).total;
  if (D.tableBytes > 64 * 1024) return false;

  // loop dimensions (digits of the tile index, fastest first)
  {
    int order[kMaxDims];
    for (int k = 0; k < r; k++) order[k] = tp.loopOrder == 0 ? k : oo[k];
    const bool balanced = tp.peerOrder == 1 && P.peerDim >= 0;
    if (balanced) {  // the destination GPU becomes the fastest digit
      int n = 0;
      order[n++] = P.peerDim;
      for (int k = 0; k < r; k++) {
        const int j = tp.loopOrder == 0 ? k : oo[k];
        if (j != P.peerDim) order[n++] = j;
      }
    }
    D.peerRot = balanced ? (uint32_t)P.peerRot : 0u;
    // optional inner groups along the chunked dimensions of the two runs
    int splitDim[2] = {-1, -1};
    int64_t splitS[2] = {1, 1};
    if (tp.groupIn > 1 && inRunLast >= 0 && t[inRunLast] < P.d[inRunLast] && inRunLast != P.peerDim &&
        ceil_div(P.d[inRunLast], t[inRunLast]) >= 2 * tp.groupIn) {
      splitDim[0] = inRunLast; splitS[0] = tp.groupIn;
    }
    if (tp.groupOut > 1 && outRunLast >= 0 && t[outRunLast] < P.d[outRunLast] && outRunLast != P.peerDim &&
        outRunLast != splitDim[0] && ceil_div(P.d[outRunLast], t[outRunLast]) >= 2 * tp.groupOut) {
      splitDim[1] = outRunLast; splitS[1] = tp.groupOut;
    }
    int64_t ntiles = 1;
    D.nLoopDims = 0;
    auto push = [&](int j, int64_t n, int64_t mul, uint32_t part, uint32_t which) {
      LoopDim& L = D.loop[D.nLoopDims];
      L.n = (uint32_t)n;
      L.div = make_fastdiv((uint32_t)n);
      L.t = (uint32_t)t[j];
      L.d = (uint32_t)P.d[j];
      L.slot = part == 0 ? slotOf[j] : -1;
      L.part = part;
      L.which = which;
      L.mul = (uint32_t)mul;
      L.istep = P.is[j] * t[j] * mul;
      L.ostep = P.os[j] * t[j] * mul;
      if (j == P.peerDim) D.peerLoopDim = (int32_t)D.nLoopDims;
      D.nLoopDims++;
      ntiles *= n;
    };
    for (int w = 0; w < 2; w++) {
      D.split[w].used = 0;
      if (splitDim[w] < 0) continue;
      int j = splitDim[w];
      D.split[w].used = 1;
      D.split[w].n = (uint32_t)ceil_div(P.d[j], t[j]);
      D.split[w].t = (uint32_t)t[j];
      D.split[w].d = (uint32_t)P.d[j];
      D.split[w].slot = slotOf[j];
      push(j, splitS[w], 1, 1, (uint32_t)w);
    }
    for (int k = 0; k < r; k++) {
      int j = order[k];
      int64_t n = ceil_div(P.d[j], t[j]);
      if (n <= 1) continue;
      int w = j == splitDim[0] ? 0 : (j == splitDim[1] ? 1 : -1);
      if (w >= 0) push(j, ceil_div(n, splitS[w]), splitS[w], 2, (uint32_t)w);
      else push(j, n, 1, 0, 0);
      if (ntiles >= (1ll << 31)) return false;
    }
    D.numTiles = (uint32_t)ntiles;
  }
  for (int j = 0; j < r; j++) if (P.d[j] >= (1ll << 32)) return false;

  out.method = kMethodTiles;
  out.params = tp;
  out.smemBytes = (int)(D.tableBytes + D.stages * D.stageBytes);
  if (out.smemBytes > dev.maxSmemPerBlock) return false;
  int bps = std::min(dev.smemPerSM / (out.smemBytes + 1024), dev.maxThreadsPerSM / tp.nthreads);
  bps = std::max(1, std::min(bps, 32));
  out.blocksPerSM = bps;
  out.gridBlocks = tp.oneTilePerBlock ? (int)D.numTiles
                                      : (int)std::min<int64_t>(D.numTiles, (int64_t)dev.numSM * bps);

  char buf[512];
  std::string ts;
  for (int j = 0; j < r; j++) { snprintf(buf, sizeof buf, "%s%lld", j ? "," : "", (long long)t[j]); ts += buf; }
  snprintf(buf, sizeof buf, "tiles t=[%s] in=%ux%u/w%u%s out=%ux%u/w%u V%u%s smem=%d st=%d lo=%d nt=%d",
           ts.c_str(), D.in.nrows, D.in.run, D.in.vec, D.aof ? "a" : "", D.out.nrows, D.out.run, D.out.vec, D.vblk,
           D.wide ? " wide" : "", out.smemBytes, D.stages, tp.loopOrder, tp.nthreads);
  if (D.split[0].used || D.split[1].used) {
    snprintf(buf + strlen(buf), sizeof buf - strlen(buf), " g=%d/%d", D.split[0].used ? tp.groupIn : 1,
             D.split[1].used ? tp.groupOut : 1);
  }
  if (tp.oneTilePerBlock) snprintf(buf + strlen(buf), sizeof buf - strlen(buf), " 1tpb");
  if (D.peerLoopDim >= 0 && tp.peerOrder == 1) snprintf(buf + strlen(buf), sizeof buf - strlen(buf), " peers-first");
  out.label = buf;

  // features of the cost model
  {
    float* f = out.feat;
    for (int i = 0; i < kNumFeatures; i++) f[i] = 0.f;
    auto lg = [](double x) { return (float)std::log2(x < 1.0 ? 1.0 : x); };
    int nslot = 0;
    for (int j = 0; j < r; j++) if (slotOf[j] >= 0) nslot++;
    // distance (bytes) between consecutive rows of each side = stride of its first row dimension
    double inRowStride = 0, outRowStride = 0;
    bool inAligned = true, outAligned = true;  // every run starts on a 32-byte sector boundary
    for (int j = 0; j < r; j++) {
      if (P.d[j] <= 1) continue;
      if (!inRun[j]) { if (t[j] > 1 && inRowStride == 0) inRowStride = (double)P.is[j] * elt; if ((P.is[j] * elt) % 32) inAligned = false; }
      else if (j == inRunLast && t[j] < P.d[j] && (P.is[j] * t[j] * elt) % 32) inAligned = false;
      if (j == P.peerDim) continue;
      if (!outRun[j]) { if (t[j] > 1 && outRowStride == 0) outRowStride = (double)P.os[j] * elt; if ((P.os[j] * elt) % 32) outAligned = false; }
      else if (j == outRunLast && t[j] < P.d[j] && (P.os[j] * t[j] * elt) % 32) outAligned = false;
    }
    f[0] = (float)elt;
    f[1] = lg((double)D.in.run * elt);
    f[2] = lg((double)D.out.run * elt);
    f[3] = (float)(D.in.vec * elt);
    f[4] = (float)(D.out.vec * elt);
    f[5] = (float)(D.vblk * elt);
    f[6] = lg(D.in.nrows);
    f[7] = lg((double)D.out.nrows * D.vblk);
    f[8] = lg((double)D.tileElems * elt);
    f[9] = (float)out.smemBytes / 1024.f;
    f[10] = (float)tp.nthreads / 256.f;
    f[11] = (float)tp.loopOrder;
    f[12] = D.split[0].used ? (float)tp.groupIn : 1.f;
    f[13] = D.split[1].used ? (float)tp.groupOut : 1.f;
    f[14] = (float)out.blocksPerSM;
    f[15] = lg(D.numTiles);
    f[16] = (float)std::min(64.0, (double)D.numTiles / ((double)dev.numSM * out.blocksPerSM));
    f[17] = D.in.nRowDims <= 1 ? 1.f : 0.f;
    f[18] = D.out.nRowDims <= 1 ? 1.f : 0.f;
    f[19] = (float)D.smemGatherContig;
    f[20] = (r > 0 && t[0] == P.d[0]) ? 1.f : 0.f;
    f[21] = inAligned ? 1.f : 0.f;
    f[22] = outAligned ? 1.f : 0.f;
    f[23] = lg((double)P.volume * elt);
    f[24] = (float)nslot;
    f[25] = lg(D.in.tq);
    f[26] = lg(D.out.tq);
    f[27] = (float)D.nLoopDims;
    f[28] = lg(inRowStride);
    f[29] = lg(outRowStride);
    f[30] = (float)D.wide + 2.f * (float)tp.oneTilePerBlock;
    f[31] = (float)D.aof;
  }
  out.cost = model_cost(P, out, dev);
  return true;
}

// Closed-form estimate (no measurements behind it); kept as a cross-check and for devices the
// fitted model was not trained on.
double analytic_cost(const Problem& P, const Candidate& c, const DeviceInfo& dev) {
  const TileDesc& D = c.desc;
  const double bytes = 2.0 * (double)P.volume * P.elt;
  const double rin = (double)D.in.run * P.elt, rout = (double)D.out.run * P.elt;
  // DRAM/L2 sector over-fetch at both ends of every run
  double fin = rin / (rin + 32.0), fout = rout / (rout + 32.0);
  // instruction pressure: work items per element on both sides
  double ipe = 1.0 / D.in.vec + 1.0 / D.out.vec + (D.smemGatherContig ? 0.0 : 1.0);
  double finstr = 1.0 / (1.0 + 0.04 * ipe);
  // fixed per-tile overhead
  double vol = (double)D.in.run * D.in.nrows;
  double ftile = vol / (vol + 384.0);
  // bytes in flight per SM
  double inflight = (double)c.blocksPerSM * D.stageBytes;
  double focc = std::min(1.0, inflight / 49152.0);
  // tail quantisation
  double waves = std::ceil((double)D.numTiles / c.gridBlocks);
  double fwave = (double)D.numTiles / (waves * c.gridBlocks);
  fwave = 0.5 + 0.5 * fwave;
  double eff = fin * fout * finstr * ftile * (0.5 + 0.5 * focc) * fwave;
  return bytes / (dev.hbmGBs * 1e9 * eff) + 4e-6;
}

// Fitted model: gradient-boosted regression trees over the candidate's feature vector, trained
// on B200 timings of every candidate of the benchmark shapes (cutt_b200/cost_model/).  Predicts
// the fraction of the copy bandwidth the candidate reaches.
static double predicted_efficiency(const float* f) {
  using namespace cost_model;
  double s = kInit;
  for (int t = 0; t < kTrees; t++) {
    int n = kRoot[t];
    while (kFeat[n] >= 0) n = f[kFeat[n]] <= kThr[n] ? kLeft[n] : kRight[n];
    s += kVal[n];
  }
  return s;
}

double model_cost(const Problem& P, const Candidate& c, const DeviceInfo& dev) {
  static_assert(cost_model::kFeatures == kNumFeatures, "regenerate cost_model_data.h");
  const double bytes = 2.0 * (double)P.volume * P.elt;
  double eff = predicted_efficiency(c.feat);
  if (eff < 0.02) eff = 0.02;
  const double stream = bytes / (cost_model::kRefGBs * 1e9 * eff);
  if (bytes < 64e6) {
    // Tensors far smaller than the training shapes are latency bound: what counts is how many
    // tiles are in flight at once and how long one block needs for its tile.  Constants fitted
    // to B200 timings of every candidate of 20 shapes between 0.3 and 48 MB (launch floor
    // 4.5 us; 0.5 us per tile plus 80 MB/s per thread; 0.6 us for the two-stage prologue).
    const TileDesc& D = c.desc;
    const double conc = std::min((double)D.numTiles, (double)dev.numSM * std::max(1, c.blocksPerSM));
    const double waves = std::ceil((double)D.numTiles / conc);
    const double tileBytes = bytes / (double)D.numTiles;   // read + written
    const double perTile = 0.5e-6 + tileBytes / ((double)D.nthreads * 80e6) + (D.stages >= 2 ? 0.6e-6 : 0.0);
    return 4.5e-6 + std::max(stream, waves * perTile);
  }
  return stream + 4e-6;
}

bool build_rowcopy(const Problem& P, const DeviceInfo& dev, Candidate& out) {
  if (P.rank < 2 || P.rank > kMaxDims || P.peerDim >= 0 || P.inBase != 0 || P.outBase != 0) return false;
  if (P.is[0] != 1 || P.os[0] != 1) return false;
  const int elt = P.elt;
  const int64_t L = P.d[0];
  const uint32_t VE = 16u / elt;
  if (L * elt < 64 || L >= (1ll << 31)) return false;
  int64_t nrows = 1;
  for (int j = 1; j < P.rank; j++) { if (P.d[j] >= (1ll << 32)) return false; nrows *= P.d[j]; }
  const int64_t slots = L / VE + 2;
  const int64_t segs = ceil_div(slots, 32 * kRowCopyUnroll);
  if (nrows * segs >= (1ll << 31)) return false;
  out = Candidate();
  out.method = kMethodRowCopy;
  RowCopyDesc& R = out.rc;
  memset(&R, 0, sizeof R);
  R.elt = elt;
  R.nd = P.rank - 1;
  R.rowLen = (uint32_t)L;
  R.segsPerRow = (uint32_t)segs;
  R.numItems = (uint32_t)(nrows * segs);
  R.inBytes = (uint64_t)P.inElems * elt;
  R.segDiv = make_fastdiv((uint32_t)segs);
  bool aligned = true;
  for (int j = 1; j < P.rank; j++) {
    R.div[j - 1] = make_fastdiv((uint32_t)P.d[j]);
    R.is[j - 1] = P.is[j];
    R.os[j - 1] = P.os[j];
    if (P.is[j] % VE || P.os[j] % VE) aligned = false;
  }
  // measured on B200: 0.85-0.89 of the copy bandwidth when the lanes of a work item are all
  // busy (rows of 0.5 K elements and more), proportionally less for rows that leave lanes idle
  (void)aligned;
  if (L * elt < 512) return false;
  double eff = 0.86 * (double)slots / (double)(segs * 32 * kRowCopyUnroll);
  out.cost = 2.0 * (double)P.volume * elt / (dev.hbmGBs * 1e9 * eff) + 4e-6;
  char buf[128];
  snprintf(buf, sizeof buf, "rowcopy rows=%lldx%lld %s", (long long)nrows, (long long)L, aligned ? "aligned" : "misaligned");
  out.label = buf;
  out.gridBlocks = 0;
  return true;
}

bool build_tma(const Problem& P, const TileParams& tp, const DeviceInfo& dev, Candidate& out) {
  const int r = P.rank;
  const int elt = P.elt;
  if (elt != 4 && elt != 8) return false;
  if (r < 2 || r > 5 || P.peerDim >= 0 || P.inBase != 0 || P.outBase != 0 || P.identity) return false;
  if (P.is[0] != 1) return false;
  int p = 0;
  for (int j = 1; j < r; j++) if (P.os[j] < P.os[p]) p = j;
  if (p == 0 || P.os[p] != 1) return false;
  const int64_t VE = 16 / elt;
  for (int j = 0; j < r; j++) {
    if (P.d[j] >= (1ll << 31)) return false;
    if (j >= 1 && (P.is[j] % VE != 0 || P.is[j] * elt >= (1ll << 40))) return false;
    if (j != p && P.os[j] % VE != 0) return false;
  }
  if (P.d[0] % VE != 0 || P.d[p] % VE != 0) return false;
  const uint32_t ta = tp.tinBytes / elt, tb = tp.toutBytes / elt;
  if (ta == 0 || (ta * elt) % 128 != 0 || ta * elt > 512) return false;
  if (tb == 0 || tb % (8 * VE) != 0 || tb > 256) return false;
  if (tp.stages < 1 || tp.stages > kTmaMaxStages) return false;
  if (tp.nthreads != 128 && tp.nthreads != 256) return false;
  // tiles far larger than the tensor along either dimension would be mostly padding
  if (P.d[0] * elt < 64 || P.d[p] < (int64_t)tb / 4) return false;

  out = Candidate();
  out.method = kMethodTma;
  out.params = tp;
  TmaDesc& D = out.tma;
  memset(&D, 0, sizeof D);
  D.elt = elt;
  D.ta = ta;
  D.tb = tb;
  D.nboxes = ta * elt / 128;
  D.cbShift = ilog2_exact(ta * elt / 64);
  if ((1u << D.cbShift) != ta * elt / 64) return false;
  D.stages = tp.stages;
  D.nthreads = tp.nthreads;
  D.order = tp.loopOrder ? 1 : 0;
  D.d0 = (uint32_t)P.d[0];
  D.dp = (uint32_t)P.d[p];
  D.nA = (uint32_t)ceil_div(P.d[0], ta);
  D.nB = (uint32_t)ceil_div(P.d[p], tb);
  D.divA = make_fastdiv(D.nA);
  D.divB = make_fastdiv(D.nB);
  D.os0 = P.os[0];
  TmaMapRecipe& R = out.tmaMap;
  memset(&R, 0, sizeof R);
  for (int i = 0; i < 5; i++) { R.dims[i] = 1; R.box[i] = 1; }
  // the tensor map lists the dimensions in input order (ascending strides); dimension p sits at
  // slot p, the loop dimensions fill the other slots in order
  for (int j = 0; j < r; j++) {
    R.dims[j] = (uint64_t)P.d[j];
    if (j >= 1) R.strideBytes[j - 1] = (uint64_t)P.is[j] * elt;
  }
  for (int j = r; j < 5; j++) R.strideBytes[j - 1] = R.strideBytes[j - 2] * R.dims[j - 1];
  R.box[0] = 128 / elt;
  R.box[p] = tb;
  D.pSlot = (uint32_t)p;
  int64_t ntiles = (int64_t)D.nA * D.nB;
  D.nOuter = 0;
  for (int j = 1; j < r; j++) {
    if (j == p) continue;
    const uint32_t k = D.nOuter++;
    D.nO[k] = (uint32_t)P.d[j];
    D.divO[k] = make_fastdiv(D.nO[k]);
    D.osO[k] = P.os[j];
    ntiles *= P.d[j];
    if (ntiles >= (1ll << 31)) return false;
  }
  for (uint32_t k = D.nOuter; k < 3; k++) { D.nO[k] = 1; D.divO[k] = make_fastdiv(1); D.osO[k] = 0; }
  D.numTiles = (uint32_t)ntiles;
  out.smemBytes = (int)(D.stages * ta * tb * elt + 1024);
  if (out.smemBytes > dev.maxSmemPerBlock - 1024) return false;   // (room for the kernel's static shared memory)
  int bps = std::min(dev.smemPerSM / (out.smemBytes + 1024), dev.maxThreadsPerSM / tp.nthreads);
  bps = std::max(1, std::min(bps, 16));
  out.blocksPerSM = bps;
  out.gridBlocks = tp.stages == 1 ? (int)ntiles : (int)std::min<int64_t>(ntiles, (int64_t)dev.numSM * bps);
  // Estimate: the copy rate, reduced by the share of each tile that lies outside the tensor and,
  // for tensors too small to give every SM a few tiles, by the idle SMs.  Measured on B200: in its
  // one-tile-per-block form this kernel runs within 1-2 % of the best cp.async tile plan (a ring of
  // stages in a persistent block: 15 % behind), so the estimate sits just below the fitted model's
  // typical value for those and cuttPlanMeasure decides.
  const double util = ((double)P.d[0] / ((double)D.nA * ta)) * ((double)P.d[p] / ((double)D.nB * tb));
  const double fill = std::min(1.0, (double)ntiles / ((double)dev.numSM * 2.0));
  const double eff = 0.93 * util * (0.25 + 0.75 * fill);
  out.cost = 2.0 * (double)P.volume * elt / (dev.hbmGBs * 1e9 * eff) + 5e-6;
  char buf[160];
  snprintf(buf, sizeof buf, "tma t=%ux%u boxes=%u st=%u lo=%u nt=%u smem=%d tiles=%u", ta, tb, D.nboxes, D.stages,
           D.order, D.nthreads, out.smemBytes, D.numTiles);
  out.label = buf;
  return true;
}

bool build_t2d(const Problem& P, const TileParams& tp, const DeviceInfo& dev, Candidate& out) {
  const int r = P.rank;
  const int elt = P.elt;
  if (elt != 4 && elt != 8 && elt != 2 && elt != 1) return false;
  if (r < 2 || r > kT2dMaxOuter + 2 || P.peerDim >= 0 || P.identity) return false;
  if (P.is[0] != 1) return false;
  int p = 0;
  for (int j = 1; j < r; j++) if (P.os[j] < P.os[p]) p = j;
  if (p == 0 || P.os[p] != 1) return false;
  for (int j = 0; j < r; j++) if (P.d[j] >= (1ll << 31)) return false;
  // widest accesses the strides allow (the pointers are checked when the plan is executed)
  auto width = [&](bool input) -> uint32_t {
    for (int64_t w = std::min(16, tp.maxVecBytes) / elt; w > 1; w /= 2) {
      bool ok = (input ? P.inBase : P.outBase) % w == 0 && P.d[input ? 0 : p] % w == 0;
      for (int j = 0; j < r && ok; j++) {
        if (input ? j == 0 : j == p) continue;
        if ((input ? P.is[j] : P.os[j]) % w != 0) ok = false;
      }
      if (ok) return (uint32_t)(w * elt);
    }
    return (uint32_t)elt;
  };
  const uint32_t ta = tp.tinBytes / elt, tb = tp.toutBytes / elt;
  if (ta * elt != 128 && ta * elt != 256) return false;
  if (elt >= 4 ? (tb != 32 && tb != 64) : (tb != 32 && tb != 64 && tb != 128 && tb != 256)) return false;
  if (elt == 1 && tb < 64) return false;   // an item of the byte transpose is 16 rows, a warp pass 64
  if (tp.nthreads != 128 && tp.nthreads != 256) return false;
  if (P.d[0] * elt < 64 || P.d[p] < 16) return false;   // tiles would be mostly padding
  out = Candidate();
  out.method = kMethodT2d;
  out.params = tp;
  T2dDesc& D = out.t2d;
  memset(&D, 0, sizeof D);
  D.elt = elt;
  D.ta = ta;
  D.tb = tb;
  D.nboxes = ta * elt / 128;
  D.nthreads = tp.nthreads;
  // The widest plain accesses the strides allow (16, 8 or 4 bytes per side).  extend = 1 selects
  // the shift / shear modes instead: 16-byte aligned accesses whatever the alignment of rows and
  // buffers.  Measured on B200 they cost 1.5 warp instructions per element and run at 4.0-5.3 TB/s,
  // below the 8-byte modes (6.0 TB/s), so they serve as the form a plan falls back to when its
  // buffers turn out not to be aligned for its access width, not as a first choice.
  D.loadMode = width(true);
  D.storeMode = width(false);
  if (tp.extend) D.loadMode = D.storeMode = 1;
  // 1- and 2-byte elements: cp.async moves at least 4 bytes; the register transposes write 16-byte
  // or (tiles of whole 64-row passes) 8-byte vectors
  if (elt < 4 && (tp.extend || D.loadMode < 4 || (D.storeMode != 16 && !(D.storeMode == 8 && tb % 64 == 0))))
    return false;
  if (elt < 4) {
    // lane map 1 needs whole warp passes of 64 (2-byte) / 128 (1-byte) rows
    const uint32_t pass = elt == 2 ? 64u : 128u;
    const char* lm = getenv("CUTT_SMALL_LANEMAP");   // tuning aid
    D.laneMap = (tb % pass == 0 && !(lm && lm[0] == '0')) ? 1u : 0u;
  }
  D.padTop = D.storeMode == 1 ? kT2dPadTop : 0;
  D.rowsLoad = tb + (D.storeMode == 1 ? 16 / elt - 1 : 0);
  D.rowsAlloc = D.storeMode == 1 ? tb + kT2dPadTop + kT2dPadBottom : tb;
  D.divRows = make_fastdiv(D.rowsLoad);
  D.uprShift = ilog2_exact(D.nboxes * 8u * (16u / (D.loadMode == 1 ? 16u : D.loadMode)));
  D.inElems = P.inElems;
  if (tp.loopOrder < 0 || tp.loopOrder > 3) return false;
  D.order = (uint32_t)tp.loopOrder;
  D.d0 = (uint32_t)P.d[0];
  D.dp = (uint32_t)P.d[p];
  D.nA = (uint32_t)ceil_div(P.d[0], ta);
  D.nB = (uint32_t)ceil_div(P.d[p], tb);
  D.divA = make_fastdiv(D.nA);
  D.divB = make_fastdiv(D.nB);
  D.nBand = (uint32_t)ceil_div(D.order == 2 ? D.nA : D.nB, 4);
  D.divBand = make_fastdiv(D.nBand ? D.nBand : 1);
  if (D.order >= 2 && (D.order == 2 ? D.nA : D.nB) < 8) return false;   // bands need a few tiles across
  D.isP = P.is[p];
  D.os0 = P.os[0];
  D.inBase = P.inBase;
  D.outBase = P.outBase;
  int64_t ntiles = D.order == 2 ? (int64_t)D.nBand * 4 * D.nB : (D.order == 3 ? (int64_t)D.nBand * 4 * D.nA : (int64_t)D.nA * D.nB);
  for (int j = 1; j < r; j++) {
    if (j == p) continue;
    const uint32_t k = D.nOuter++;
    D.nO[k] = (uint32_t)P.d[j];
    D.divO[k] = make_fastdiv(D.nO[k]);
    D.isO[k] = P.is[j];
    D.osO[k] = P.os[j];
    ntiles *= P.d[j];
    if (ntiles >= (1ll << 31)) return false;
  }
  D.numTiles = (uint32_t)ntiles;
  out.smemBytes = (int)(D.nboxes * D.rowsAlloc * 128);
  int bps = std::min(dev.smemPerSM / (out.smemBytes + 1024), dev.maxThreadsPerSM / tp.nthreads);
  out.blocksPerSM = std::max(1, std::min(bps, 32));
  out.gridBlocks = (int)ntiles;
  // Estimate: the copy rate, reduced by the share of each tile that lies outside the tensor, by
  // narrow accesses, and for tensors too small to give every SM a few tiles by the idle SMs.
  const double util = ((double)P.d[0] / ((double)D.nA * ta)) * ((double)P.d[p] / ((double)D.nB * tb));
  const double fill = std::min(1.0, (double)ntiles / ((double)dev.numSM * 4.0));
  auto side = [](uint32_t mode) { return mode == 16 ? 1.0 : (mode == 8 ? 0.97 : (mode == 1 ? 0.8 : 0.75)); };
  const double narrow = side(D.loadMode) * side(D.storeMode);
  double eff = 0.93 * util * narrow * (0.25 + 0.75 * fill);
  if (elt >= 4 && fill >= 1.0) {
    // Among the shapes of one tensor the estimate above cannot tell tile orders, thread counts and
    // tile shapes apart, and cuttPlanMeasure times only the first few of the family: put the forms
    // that won most often first (best candidate per tensor over seven large shapes on B200: 256-byte x
    // 64-row tiles in six, tile order 2 in four and order 1 in two, 256 threads in five)
    if (ta * elt == 256 && tb == 64) eff *= 1.004;
    if (D.order == 2) eff *= 1.003; else if (D.order == 1) eff *= 1.002;
    if (tp.nthreads == 256 && ta * elt * tb >= 16384) eff *= 1.001;
  }
  out.cost = 2.0 * (double)P.volume * elt / (dev.hbmGBs * 1e9 * eff) + 5e-6;
  char buf[160];
  char li[16], lo[16];
  if (D.loadMode == 1) snprintf(li, sizeof li, "shift"); else snprintf(li, sizeof li, "w%u", D.loadMode / elt);
  if (D.storeMode == 1) snprintf(lo, sizeof lo, "shear"); else snprintf(lo, sizeof lo, "w%u", D.storeMode / elt);
  snprintf(buf, sizeof buf, "t2d t=%ux%u in/%s out/%s lo=%u nt=%u smem=%d tiles=%u", ta, tb, li, lo, D.order, D.nthreads,
           out.smemBytes, D.numTiles);
  out.label = buf;
  return true;
}

bool build_t2d_small(const Problem& P, const DeviceInfo& dev, Candidate& out) {
  if (P.elt != 2 && P.elt != 1) return false;
  TileParams tp;
  // Tall tiles: with elements this small the runs written per output row are only as long as the
  // tile is high.  Measured on B200 with lane map 1 (GB/s; 1-byte (28000,28000)/(1,0) and
  // (1024,64,16384)/(2,1,0), 2-byte (20000,20000)/(1,0) and (1024,64,8192)/(2,1,0); tile = bytes
  // along dimension 0 x rows):
  //   256 x 128: 6027 5935 | 6102 6019     128 x 256: 5893 5887 | 6023 5924
  //   128 x 128: 5208 5161 | 6066 5987     256 x 64:  4750 5000 (lane map 0) | 6155 6010
  // (lane map 0, a store instruction writing 64 instead of 128 contiguous bytes per output row:
  // 256 x 128: 4982 5313 | 5357 5460).  128 threads throughout (256 threads: 4-15 % slower); tile
  // order 0 the same as 1.
  int p = 0;
  for (int j = 1; j < P.rank; j++) if (P.os[j] < P.os[p]) p = j;
  const int64_t dp = P.d[p];
  const uint32_t rows = dp >= 112 ? 128u : 64u;
  tp.tinBytes = 256;
  tp.toutBytes = rows * P.elt;
  tp.stages = 1;
  tp.nthreads = 128;
  tp.loopOrder = 1;
  if (const char* v = getenv("CUTT_SMALL_TILE")) {   // tuning aid: "bytes along dimension 0,rows,threads"
    unsigned a = 0, b = 0, n = 0;
    if (sscanf(v, "%u,%u,%u", &a, &b, &n) == 3) { tp.tinBytes = a; tp.toutBytes = b * P.elt; tp.nthreads = (int)n; }
  }
  if (build_t2d(P, tp, dev, out)) return true;
  tp.tinBytes = tp.tinBytes == 128 ? 256 : 128;
  if (build_t2d(P, tp, dev, out)) return true;
  tp.tinBytes = 128;
  tp.toutBytes = 64 * P.elt;
  return build_t2d(P, tp, dev, out);
}

std::vector<Candidate> enumerate_candidates(const Problem& P, const DeviceInfo& dev) {
  std::vector<Candidate> res;
  if (P.identity) {
    // measured on B200: the driver's D2D copy reaches 6.5 TB/s, the copy kernel 5.9 TB/s
    Candidate m;
    m.method = kMethodMemcpy;
    m.label = "memcpy";
    m.cost = 2.0 * P.volume * P.elt / (dev.hbmGBs * 1e9);
    res.push_back(m);
    Candidate c = m;
    c.method = kMethodCopy;
    c.label = "copy";
    c.cost = m.cost * 1.1;
    res.push_back(c);
    return res;
  }
  std::set<std::string> seen, seenExt;
  // first dimension of the output order (the peer dimension has no output stride)
  int oo0 = -1;
  for (int j = 0; j < P.rank; j++)
    if (j != P.peerDim && (oo0 < 0 || P.os[j] < P.os[oo0])) oo0 = j;
  const uint32_t runs[] = {128, 256, 512, 1024, 2048};
  // small tensors need small tiles to give every SM something to do
  const bool small = (double)P.volume * P.elt < 64e6;
  std::vector<uint32_t> vols = {8192, 16384, 32768, 65536};
  if (small) { vols.insert(vols.begin(), 4096); vols.insert(vols.begin(), 2048); }
  const int groups[][2] = {{1, 1}, {2, 1}, {4, 1}, {1, 4}, {2, 4}};
  for (uint32_t tinB : runs)
    for (uint32_t toutB : runs)
      for (uint32_t vB : vols)
        for (int ext = 0; ext < 2; ext++)
          for (int lo = 0; lo < 2; lo++)
            for (const auto& g : groups)
              for (int nt = 256; nt <= 512; nt *= 2)
                for (int aofpo = 3; aofpo >= 0; aofpo--) {
                  // all-to-all plans come in both destination orders (TileParams::peerOrder)
                  const int aof = aofpo & 1, po = aofpo >> 1;
                  if (po && P.peerDim < 0) continue;
                  TileParams tp;
                  tp.tinBytes = tinB; tp.toutBytes = toutB; tp.vtargetBytes = vB;
                  tp.extend = ext; tp.loopOrder = lo;
                  tp.groupIn = g[0]; tp.groupOut = g[1];
                  tp.nthreads = nt;
                  tp.allowAof = aof;
                  tp.peerOrder = po;
                  Candidate c;
                  if (!build_tile(P, tp, dev, c, &seenExt)) continue;
                  // same tile with the input run cut in front of the output's first dimension
                  if (P.rank > 1 && oo0 > 0 && c.desc.in.nrows * (uint64_t)c.desc.in.run > 0) {
                    TileParams tc = tp;
                    tc.cutInRun = 1;
                    Candidate cc;
                    if (build_tile(P, tc, dev, cc, &seenExt) && cc.label != c.label &&
                        !(nt == 512 && cc.smemBytes < 40 * 1024) && seen.insert(cc.label).second)
                      res.push_back(cc);
                  }
                  if (nt == 512 && c.smemBytes < 40 * 1024) continue;  // small tiles: more blocks instead
                  // 4-byte element-wise loads never beat the aligned over-fetch of the same tile
                  if (!aof && P.elt == 4 && c.desc.in.vec == 1 && c.desc.in.run >= 8) continue;
                  if (!seen.insert(c.label).second) continue;
                  res.push_back(c);
                }
  // small tiles, one per thread block, single stage: the hardware block scheduler replaces the
  // persistent loop and many blocks per SM hide each other's phases
  {
    const uint32_t sruns[] = {128, 256, 512};
    const uint32_t svols[] = {4096, 8192, 16384};
    for (uint32_t tinB : sruns)
      for (uint32_t toutB : sruns)
        for (uint32_t vB : svols)
          for (int lo = 0; lo < 2; lo++)
            for (int nt = 128; nt <= 256; nt *= 2)
              for (int aofpo = 3; aofpo >= 0; aofpo--) {
                const int aof = aofpo & 1, po = aofpo >> 1;
                if (po && P.peerDim < 0) continue;
                TileParams tp;
                tp.tinBytes = tinB; tp.toutBytes = toutB; tp.vtargetBytes = vB;
                tp.loopOrder = lo; tp.nthreads = nt; tp.stages = 1; tp.oneTilePerBlock = 1; tp.allowAof = aof;
                tp.peerOrder = po;
                Candidate c;
                if (!build_tile(P, tp, dev, c, &seenExt)) continue;
                if (c.smemBytes > 24 * 1024) continue;
                if (!aof && P.elt == 4 && c.desc.in.vec == 1 && c.desc.in.run >= 8) continue;
                if (!seen.insert(c.label).second) continue;
                res.push_back(c);
              }
  }
  {
    Candidate rc;
    if (build_rowcopy(P, dev, rc)) res.push_back(rc);
  }
  // two-dimensional tiles with swizzled shared memory, loaded by cp.async (any alignment) or by the
  // copy engine through a tensor map (strides that are multiples of 16 bytes only): one tile per
  // block, a few tile shapes, both tile orders
  {
    const uint32_t ta[] = {128, 256}, tbE[] = {32, 64};
    for (uint32_t a : ta)
      for (uint32_t b : tbE)
        for (int lo = 0; lo < 4; lo++)
          for (int nt = 128; nt <= 256; nt *= 2) {
            if (nt == 256 && a * b <= 128 * 32) continue;   // 4 KB tiles: 128 threads are enough
            TileParams tp;
            tp.tinBytes = a; tp.toutBytes = b * (uint32_t)P.elt; tp.loopOrder = lo; tp.nthreads = nt;
            tp.stages = 1;
            Candidate c;
            // (rows on 4-byte boundaries: measured 3.6-4.1 TB/s against 4.4-5.7 TB/s for the general
            // kernel's over-fetching loads - not worth a measurement slot)
            if (build_t2d(P, tp, dev, c) && c.t2d.loadMode >= 8 && c.t2d.storeMode >= 8) res.push_back(c);
            if (lo < 2 && dev.tmaLoads && build_tma(P, tp, dev, c)) res.push_back(c);
          }
  }
  std::stable_sort(res.begin(), res.end(), [](const Candidate& a, const Candidate& b) { return a.cost < b.cost; });
  return res;
}

std::string describe(const Problem& P, const Candidate& c) {
  char buf[2048];
  std::string dims, iss, oss;
  for (int j = 0; j < P.rank; j++) {
    snprintf(buf, sizeof buf, "%s%lld", j ? "," : "", (long long)P.d[j]); dims += buf;
    snprintf(buf, sizeof buf, "%s%lld", j ? "," : "", (long long)P.is[j]); iss += buf;
    snprintf(buf, sizeof buf, "%s%lld", j ? "," : "", (long long)P.os[j]); oss += buf;
  }
  snprintf(buf, sizeof buf,
           "{\"method\": %d, \"label\": \"%s\", \"fused_dims\": [%s], \"istride\": [%s], \"ostride\": [%s], "
           "\"elt\": %d, \"num_tiles\": %u, \"grid\": %d, \"smem\": %d, \"model_us\": %.2f, \"feat\": [",
           (int)c.method, c.label.c_str(), dims.c_str(), iss.c_str(), oss.c_str(), P.elt,
           c.method == kMethodTiles ? c.desc.numTiles
                                    : (c.method == kMethodTma ? c.tma.numTiles : (c.method == kMethodT2d ? c.t2d.numTiles : 0u)),
           c.gridBlocks,
           c.smemBytes, c.cost * 1e6);
  std::string res = buf;
  for (int i = 0; i < kNumFeatures; i++) {
    snprintf(buf, sizeof buf, "%s%.4g", i ? "," : "", c.method == kMethodTiles ? (double)c.feat[i] : 0.0);
    res += buf;
  }
  res += "]}";
  return res;
}

}  // namespace cuttb
