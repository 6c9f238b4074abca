// Host-side plan interpreter.  TEST ONLY: built into its own shared library
// (libcutt_hostcheck.so), never linked into libcutt.  It executes a tile descriptor on
// host arrays by calling, for every block, tile and thread index in turn, the very same
// per-thread phase functions the CUDA kernel calls, so the planner and the index
// arithmetic are checked against the CPU oracle without a GPU.
#include <cstdio>
#include <cstring>
#include <vector>
#define CUTT_HOSTCHECK_BOUNDS 1
#include "permute_tile_impl.h"
#include "planner.h"
#include "small_elt_impl.h"

using namespace cuttb;

// Mirrors permute_tiles_kernel for an emulated grid of `grid` blocks, one block after the
// other: same shared-memory layout (tables, the two context slots, the stage buffers), same
// order of decode / load / store steps per block.  Threads of a block run one after the
// other inside each step, so data races are not modelled, layout overlaps are.
// Output base pointers per destination GPU (host emulation of PeerPtrs); null = single output.
static unsigned char* const* g_peerOuts = nullptr;

template <int ELT, int WIN, int WOUT, int V, bool WIDE, bool AOF>
static void run_desc(const TileDesc& D, const unsigned char* in, unsigned char* out) {
  const uint32_t G = D.numTiles < 3 ? D.numTiles : 3;
  std::vector<unsigned char> smem(D.tableBytes + D.stages * D.stageBytes);
  host_bounds().s0 = smem.data() + D.tableBytes;
  host_bounds().s1 = smem.data() + smem.size();
  for (uint32_t block = 0; block < G; block++) {
    memset(smem.data(), 0xEE, smem.size());
    TileCtx* ctxs = reinterpret_cast<TileCtx*>(smem.data() + table_layout(D).ctx);
    uint32_t tile = block;
    decode_tile(D, tile, ctxs[0]);
    if (tile + G < D.numTiles) decode_tile(D, tile + G, ctxs[1]);
    for (uint32_t tid = 0; tid < D.nthreads; tid++) build_tables<WIDE>(D, smem.data(), tid, D.nthreads);
    const Tables<WIDE> T = make_tables<WIDE>(D, smem.data());
    unsigned char* stage0 = smem.data() + D.tableBytes;
    TileCtx cur = ctxs[0], nxt = cur;
    auto load = [&](const TileCtx& c, unsigned char* st) {
      if (!c.valid) return;
      for (uint32_t tid = 0; tid < D.nthreads; tid++) tile_load<ELT, WIN, WIDE, AOF>(D, c, T, st, in, tid);
    };
    auto store = [&](const TileCtx& c, unsigned char* st) {
      if (!c.valid) return;
      unsigned char* o = (D.peerLoopDim >= 0 && g_peerOuts) ? g_peerOuts[c.peer] : out;
      for (uint32_t tid = 0; tid < D.nthreads; tid++) tile_store<ELT, WOUT, V, WIDE, AOF>(D, c, T, st, in, o, tid);
    };
    if (D.stages >= 2) {
      load(cur, stage0);
      uint32_t st = 0;
      for (uint32_t it = 0; tile < D.numTiles; tile += G, it++) {
        if (tile + G < D.numTiles) {
          nxt = ctxs[(it + 1) & 1];
          load(nxt, stage0 + (st ^ 1u) * D.stageBytes);
        }
        if (tile + 2 * (uint64_t)G < D.numTiles) decode_tile(D, tile + 2 * G, ctxs[it & 1]);
        store(cur, stage0 + st * D.stageBytes);
        cur = nxt;
        st ^= 1u;
      }
    } else {
      for (uint32_t it = 0; tile < D.numTiles; tile += G, it++) {
        if (it > 0) cur = ctxs[it & 1];
        load(cur, stage0);
        if (tile + 2 * (uint64_t)G < D.numTiles) decode_tile(D, tile + 2 * G, ctxs[it & 1]);
        store(cur, stage0);
      }
    }
  }
}

static int dispatch(const TileDesc& D, const unsigned char* in, unsigned char* out);

// Every global and shared access of the phases is range- and alignment-checked; accesses
// that fail are skipped and counted, and the run then reports code 9.
static int dispatch_checked(const TileDesc& D, const unsigned char* in, unsigned char* out, size_t bytes) {
  HostBounds& b = host_bounds();
  b.gin0 = in; b.gin1 = in + bytes; b.gout0 = out; b.gout1 = out + bytes; b.violations = 0;
  int rc = dispatch(D, in, out);
  if (rc == 0 && b.violations) { fprintf(stderr, "hostcheck: %lld out-of-range or misaligned accesses\n", b.violations); return 9; }
  return rc;
}

static int dispatch(const TileDesc& D, const unsigned char* in, unsigned char* out) {
  if (D.aof) {
    if (D.wide || D.vblk > 2) return 4;
#define ACASE(E, A, B, V) if (D.elt == E && D.in.vec == A && D.out.vec == B && D.vblk == V) { run_desc<E, A, B, V, false, true>(D, in, out); return 0; }
    ACASE(4, 4, 1, 1) ACASE(4, 4, 2, 1) ACASE(4, 4, 4, 1) ACASE(8, 2, 1, 1) ACASE(8, 2, 2, 1)
    ACASE(4, 4, 1, 2) ACASE(4, 4, 2, 2) ACASE(4, 4, 4, 2)
#undef ACASE
    return 4;
  }
#define CASE(E, A, B, V) \
  if (D.elt == E && D.in.vec == A && D.out.vec == B && D.vblk == V) { \
    if (D.wide) { if (V != 1) return 4; run_desc<E, A, B, 1, true, false>(D, in, out); } \
    else run_desc<E, A, B, V, false, false>(D, in, out); \
    return 0; }
#define CASES_V(E, A, B) CASE(E, A, B, 1) CASE(E, A, B, 2) CASE(E, A, B, 4)
  CASES_V(4, 1, 1) CASES_V(4, 1, 2) CASES_V(4, 1, 4) CASES_V(4, 2, 1) CASES_V(4, 2, 2) CASES_V(4, 2, 4)
  CASES_V(4, 4, 1) CASES_V(4, 4, 2) CASES_V(4, 4, 4)
  CASE(8, 1, 1, 1) CASE(8, 1, 1, 2) CASE(8, 1, 2, 1) CASE(8, 1, 2, 2)
  CASE(8, 2, 1, 1) CASE(8, 2, 1, 2) CASE(8, 2, 2, 1) CASE(8, 2, 2, 2)
#undef CASES_V
#undef CASE
  return 4;
}

// Row-copy method: every work item, every lane, with all accesses range- and alignment-checked.
static int run_rowcopy(const RowCopyDesc& R, const unsigned char* in, unsigned char* out, size_t bytes) {
  rowcopy_bounds().in0 = in; rowcopy_bounds().in1 = in + bytes;
  rowcopy_bounds().out0 = out; rowcopy_bounds().out1 = out + bytes;
  rowcopy_violations() = 0;
  for (uint32_t item = 0; item < R.numItems; item++)
    for (uint32_t lane = 0; lane < 32; lane++) {
      if (R.elt == 4) rowcopy_item<4>(R, in, out, item, lane);
      else rowcopy_item<8>(R, in, out, item, lane);
    }
  if (rowcopy_violations()) { fprintf(stderr, "hostcheck: %lld bad row-copy accesses\n", rowcopy_violations()); return 9; }
  return 0;
}

// Small-element method: every tile, every thread, both phases, all accesses range-checked.
static int run_small(const SmallDesc& plan, const unsigned char* in, unsigned char* out) {
  SmallDesc S = plan;   // as the launcher: 32-bit accesses only on 4-byte aligned buffers
  if ((uintptr_t)in % 4) S.packLoad = 0;
  if ((uintptr_t)out % 4) S.packStore = 0;
  std::vector<uint32_t> smemWords(S.smemBytes / 4 + 1);
  unsigned char* smemBase = reinterpret_cast<unsigned char*>(smemWords.data());
  small_violations() = 0;
  for (uint32_t tile = 0; tile < S.numTiles; tile++) {
    const SmallOrigin o = small_origin(S, tile);
    for (uint32_t tid = 0; tid < (uint32_t)kSmallThreads; tid++) {
      if (S.elt == 1) small_load<1>(S, o, in, smemBase, tid, kSmallThreads);
      else small_load<2>(S, o, in, smemBase, tid, kSmallThreads);
    }
    for (uint32_t tid = 0; tid < (uint32_t)kSmallThreads; tid++) {
      if (S.elt == 1) small_store<1>(S, o, out, smemBase, tid, kSmallThreads);
      else small_store<2>(S, o, out, smemBase, tid, kSmallThreads);
    }
  }
  if (small_violations()) { fprintf(stderr, "hostcheck: %lld bad small-element accesses\n", small_violations()); return 9; }
  return 0;
}

// Tensor-map transpose: the box loads are emulated as the copy engine performs them (128-byte rows,
// 16-byte chunk c of row r at chunk position c ^ (r & 7), zeros outside the tensor); the store
// phase is the device code.
static int run_tma(const Candidate& c, const unsigned char* in, unsigned char* out, size_t bytes,
                   unsigned char* outLo = nullptr, unsigned char* outHi = nullptr) {
  const TmaDesc& D = c.tma;
  const TmaMapRecipe& R = c.tmaMap;
  HostBounds& b = host_bounds();
  b.gin0 = in; b.gin1 = in + bytes; b.violations = 0;
  b.gout0 = outLo ? outLo : out; b.gout1 = outHi ? outHi : out + bytes;
  const uint32_t elt = D.elt, V = 16 / elt;
  const size_t stageBytes = (size_t)D.ta * D.tb * elt;
  std::vector<unsigned char> raw(stageBytes + 1024 + 16);
  unsigned char* stage = raw.data() + (1024 - ((uintptr_t)raw.data() & 1023)) % 1024;
  b.s0 = stage; b.s1 = stage + stageBytes;
  for (uint32_t tile = 0; tile < D.numTiles; tile++) {
    TmaTile t;
    tma_decode(D, tile, t);
    memset(stage, 0xEE, stageBytes);
    for (uint32_t k = 0; k < D.nboxes; k++)
      for (uint32_t row = 0; row < D.tb; row++)
        for (uint32_t chunk = 0; chunk < 8; chunk++)
          for (uint32_t e = 0; e < V; e++) {
            int b0, b1, b2, b3, b4;
            tma_box_coords(D, t, k, b0, b1, b2, b3, b4);
            uint64_t x[5] = {(uint64_t)b0 + chunk * V + e, (uint64_t)b1, (uint64_t)b2, (uint64_t)b3, (uint64_t)b4};
            x[D.pSlot] += row;
            unsigned char* dst = stage + k * (D.tb * 128) + row * 128 + ((chunk ^ (row & 7u)) << 4) + e * elt;
            bool inside = true;
            for (int i = 0; i < 5; i++) inside = inside && x[i] < R.dims[i];
            if (!inside) { memset(dst, 0, elt); continue; }
            size_t off = (size_t)x[0] * elt;
            for (int i = 1; i < 5; i++) off += (size_t)x[i] * R.strideBytes[i - 1];
            if (off + elt > bytes) return 9;
            memcpy(dst, in + off, elt);
          }
    const uint32_t nItems = tma_items_per_tile(D);
    for (uint32_t it = 0; it < nItems; it++) {
      if (elt == 4) tma_store_item<4>(D, t, stage, out, it);
      else tma_store_item<8>(D, t, stage, out, it);
    }
  }
  return b.violations ? 9 : 0;
}

// Two-dimensional tile method: load units and store items are the device code; every global and
// shared access is range- and alignment-checked.
template <int ELT, int LOAD, int STORE>
static void run_t2d_typed(const T2dDesc& D, const unsigned char* in, unsigned char* out, unsigned char* stage) {
  for (uint32_t tile = 0; tile < D.numTiles; tile++) {
    T2dTile t;
    if (!t2d_decode(D, tile, t)) continue;
    memset(stage, 0xEE, (size_t)D.nboxes * D.rowsAlloc * 128);
    const uint32_t nUnits = t2d_load_units(D), nItems = t2d_store_items(D);
    // as the kernel: per-thread phases for the plain modes, unit / item loops for shift and shear
    if constexpr (LOAD == 1) {
      for (uint32_t u = 0; u < nUnits; u++) t2d_load_shift<ELT>(D, t, stage, in, u);
    } else {
      for (uint32_t tid = 0; tid < D.nthreads; tid++) t2d_load_rows<ELT, (LOAD == 1 ? 16 : LOAD)>(D, t, stage, in, tid);
    }
    if constexpr (ELT == 2) {
      for (uint32_t tid = 0; tid < D.nthreads; tid++) t2d_store_rows_e2(D, t, stage, out, tid);
    } else if constexpr (ELT == 1) {
      for (uint32_t tid = 0; tid < D.nthreads; tid++) t2d_store_rows_e1(D, t, stage, out, tid);
    } else if constexpr (STORE == 1) {
      for (uint32_t it = 0; it < nItems; it++) t2d_store_shear<ELT>(D, t, stage, out, it);
    } else {
      for (uint32_t tid = 0; tid < D.nthreads; tid++) t2d_store_rows<ELT, (STORE == 1 ? 16 : STORE)>(D, t, stage, out, tid);
    }
  }
}

static int run_t2d(const Candidate& c, const unsigned char* in, size_t inBytes, unsigned char* out,
                   unsigned char* outLo, unsigned char* outHi) {
  T2dDesc D = c.t2d;
  const uintptr_t ai = D.loadMode == 1 ? D.elt : D.loadMode, ao = D.storeMode == 1 ? D.elt : D.storeMode;
  if ((uintptr_t)in % ai || (uintptr_t)out % ao) return 7;
  D.inMis = (uint32_t)(((uintptr_t)in / D.elt) % (16 / D.elt));     // as the launcher does
  D.outMis = (uint32_t)(((uintptr_t)out / D.elt) % (16 / D.elt));
  HostBounds& b = host_bounds();
  b.gin0 = in; b.gin1 = in + inBytes; b.gout0 = outLo; b.gout1 = outHi; b.violations = 0;
  const size_t smem = (size_t)D.nboxes * D.rowsAlloc * 128;
  std::vector<unsigned char> raw(smem + 256);
  unsigned char* stage = raw.data() + (128 - ((uintptr_t)raw.data() & 127)) % 128;
  b.s0 = stage; b.s1 = stage + smem;
#define T2D_CASE(E, A, B) if (D.elt == E && D.loadMode == A && D.storeMode == B) { run_t2d_typed<E, A, B>(D, in, out, stage); return b.violations ? 9 : 0; }
#define T2D_ROW(E, A) T2D_CASE(E, A, 16) T2D_CASE(E, A, 1) T2D_CASE(E, A, 8)
  T2D_ROW(4, 16) T2D_ROW(4, 1) T2D_ROW(4, 8) T2D_ROW(4, 4)
  T2D_CASE(4, 16, 4) T2D_CASE(4, 1, 4) T2D_CASE(4, 8, 4) T2D_CASE(4, 4, 4)
  T2D_ROW(8, 16) T2D_ROW(8, 1) T2D_ROW(8, 8)
  T2D_CASE(2, 16, 16) T2D_CASE(2, 8, 16) T2D_CASE(2, 4, 16)
  T2D_CASE(1, 16, 16) T2D_CASE(1, 8, 16) T2D_CASE(1, 4, 16)
  T2D_CASE(2, 16, 8) T2D_CASE(2, 8, 8) T2D_CASE(2, 4, 8)
  T2D_CASE(1, 16, 8) T2D_CASE(1, 8, 8) T2D_CASE(1, 4, 8)
#undef T2D_ROW
#undef T2D_CASE
  return 4;
}

static DeviceInfo g_dev;

// Candidate list of the last problem asked for (tests run candidate 0, 1, 2, ... of one problem
// in a row; enumerating is the expensive part).
static bool g_candidatesStale = false;
static const std::vector<Candidate>& candidates_of(const Problem& P) {
  static Problem last;
  static std::vector<Candidate> list;
  static bool have = false;
  if (g_candidatesStale) { have = false; g_candidatesStale = false; }
  bool same = have && last.rank == P.rank && last.elt == P.elt && last.peerDim == P.peerDim &&
              last.inBase == P.inBase && last.outBase == P.outBase && last.inElems == P.inElems;
  for (int j = 0; same && j < P.rank; j++)
    same = last.d[j] == P.d[j] && last.is[j] == P.is[j] && last.os[j] == P.os[j];
  if (!same) {
    list = enumerate_candidates(P, g_dev);
    last = P;
    have = true;
  }
  return list;
}

extern "C" {

// Number of candidates the planner enumerates for a cuTT-style problem (0 on invalid input).
int cutt_hostcheck_num_candidates(int rank, const int* dim, const int* perm, int elt) {
  Problem P;
  if (!problem_from_cutt(rank, dim, perm, elt, P)) return 0;
  return (int)candidates_of(P).size();
}

// JSON description (label, model estimate, features) of candidate `index` without executing it.
int cutt_hostcheck_describe(int rank, const int* dim, const int* perm, int elt, int index, char* label, int labelLen) {
  Problem P;
  if (!problem_from_cutt(rank, dim, perm, elt, P)) return 2;
  const std::vector<Candidate>& cands = candidates_of(P);
  if (index < 0 || index >= (int)cands.size()) return 3;
  if (!label || labelLen <= 0) return 4;
  snprintf(label, labelLen, "%s", describe(P, cands[index]).c_str());
  return 0;
}

// Executes candidate `index` on host memory.  Returns 0 on success; `label` receives the
// JSON description of the candidate.  Copy candidates are executed as a memcpy.
int cutt_hostcheck_run(int rank, const int* dim, const int* perm, int elt, int index,
                       const void* in, void* out, char* label, int labelLen) {
  Problem P;
  if (!problem_from_cutt(rank, dim, perm, elt, P)) return 2;
  const std::vector<Candidate>& cands = candidates_of(P);
  if (index < 0 || index >= (int)cands.size()) return 3;
  const Candidate& c = cands[index];
  if (label && labelLen > 0) snprintf(label, labelLen, "%s", describe(P, c).c_str());
  if (c.method == kMethodCopy || c.method == kMethodMemcpy) {
    memcpy(out, in, (size_t)P.volume * elt);
    return 0;
  }
  if (c.method == kMethodRowCopy) return run_rowcopy(c.rc, (const unsigned char*)in, (unsigned char*)out, (size_t)P.volume * elt);
  if (c.method == kMethodTma) return run_tma(c, (const unsigned char*)in, (unsigned char*)out, (size_t)P.volume * elt);
  if (c.method == kMethodT2d)
    return run_t2d(c, (const unsigned char*)in, (size_t)P.volume * elt, (unsigned char*)out, (unsigned char*)out,
                   (unsigned char*)out + (size_t)P.volume * elt);
  return dispatch_checked(c.desc, (const unsigned char*)in, (unsigned char*)out, (size_t)P.volume * elt);
}

// Two-dimensional tile method with explicit parameters (tile bytes along dimension 0, tile extent
// along dimension p, threads, tile order, widest access in bytes).  Returns 2 when the problem is
// outside the method's class.
int cutt_hostcheck_run_t2d(int rank, const int* dim, const int* perm, int elt, unsigned taBytes, unsigned tbElems,
                           int nthreads, int order, int maxVecBytes, int forceShift, const void* in, void* out,
                           char* label, int labelLen) {
  Problem P;
  if (!problem_from_cutt(rank, dim, perm, elt, P)) return 2;
  TileParams tp;
  tp.tinBytes = taBytes; tp.toutBytes = tbElems * elt; tp.stages = 1; tp.nthreads = nthreads; tp.loopOrder = order;
  tp.maxVecBytes = maxVecBytes;
  tp.extend = forceShift;
  Candidate c;
  if (!build_t2d(P, tp, g_dev, c)) return 2;
  if (label && labelLen > 0) snprintf(label, labelLen, "%s", describe(P, c).c_str());
  return run_t2d(c, (const unsigned char*)in, (size_t)P.volume * elt, (unsigned char*)out, (unsigned char*)out,
                 (unsigned char*)out + (size_t)P.volume * elt);
}

// Tensor-map transpose with explicit parameters (tile bytes along the two dimensions, stages,
// threads, tile order).  Returns 2 when the problem is outside the method's class.
int cutt_hostcheck_run_tma(int rank, const int* dim, const int* perm, int elt, unsigned taBytes, unsigned tbBytes,
                           int stages, int nthreads, int order, const void* in, void* out, char* label, int labelLen) {
  Problem P;
  if (!problem_from_cutt(rank, dim, perm, elt, P)) return 2;
  TileParams tp;
  tp.tinBytes = taBytes; tp.toutBytes = tbBytes; tp.stages = stages; tp.nthreads = nthreads; tp.loopOrder = order;
  Candidate c;
  if (!build_tma(P, tp, g_dev, c)) return 2;
  if (label && labelLen > 0) snprintf(label, labelLen, "%s", describe(P, c).c_str());
  return run_tma(c, (const unsigned char*)in, (unsigned char*)out, (size_t)P.volume * elt);
}

// Extension element sizes (1, 2, 16 bytes besides 4 and 8): the problem as the library re-states
// it, then candidate `index` of the planner or the small-element method.  `label` receives
// "memcpy", "small ..." or the candidate's description.  Returns 0 on success, 3 when `index`
// is past the end of the candidate list.
int cutt_hostcheck_run_ext(int rank, const int* dim, const int* perm, int eltBytes, int index,
                           const void* in, void* out, char* label, int labelLen) {
  Problem P;
  if (!problem_from_cutt_ext(rank, dim, perm, eltBytes, P)) return 2;
  size_t bytes = (size_t)eltBytes;
  for (int i = 0; i < rank; i++) bytes *= (size_t)dim[i];
  if ((size_t)P.volume * P.elt != bytes) return 6;
  if (P.identity) {
    if (index > 0) return 3;
    if (label && labelLen > 0) snprintf(label, labelLen, "memcpy");
    memcpy(out, in, bytes);
    return 0;
  }
  if (P.elt < 4) {
    if (index > 0) return 3;
    {   // as the library: 2-byte elements on aligned rows take the swizzled two-dimensional tiles
      Candidate c;
      if (build_t2d_small(P, g_dev, c) && (uintptr_t)in % c.t2d.loadMode == 0 && (uintptr_t)out % c.t2d.storeMode == 0) {
        if (label && labelLen > 0) snprintf(label, labelLen, "%s", c.label.c_str());
        return run_t2d(c, (const unsigned char*)in, bytes, (unsigned char*)out, (unsigned char*)out, (unsigned char*)out + bytes);
      }
    }
    SmallDesc S;
    if (!build_small(P, S)) return 5;
    if (label && labelLen > 0)
      snprintf(label, labelLen, "small t=%ux%u%s%s%s tiles=%u", 1u << S.logTA, 1u << S.logTB,
               S.storeAlongB ? "" : " rows", S.packLoad ? " ld32" : "", S.packStore ? " st32" : "", S.numTiles);
    return run_small(S, (const unsigned char*)in, (unsigned char*)out);
  }
  const std::vector<Candidate>& cands = candidates_of(P);
  if (index < 0 || index >= (int)cands.size()) return 3;
  const Candidate& c = cands[index];
  if (label && labelLen > 0) snprintf(label, labelLen, "%s", describe(P, c).c_str());
  if (c.method == kMethodCopy || c.method == kMethodMemcpy) { memcpy(out, in, bytes); return 0; }
  if (c.method == kMethodRowCopy) return run_rowcopy(c.rc, (const unsigned char*)in, (unsigned char*)out, bytes);
  if (c.method == kMethodTma) return run_tma(c, (const unsigned char*)in, (unsigned char*)out, bytes);
  if (c.method == kMethodT2d)
    return run_t2d(c, (const unsigned char*)in, bytes, (unsigned char*)out, (unsigned char*)out, (unsigned char*)out + bytes);
  return dispatch_checked(c.desc, (const unsigned char*)in, (unsigned char*)out, bytes);
}

// Same, for an explicit parameter choice (used to force odd tile shapes in tests).
int cutt_hostcheck_run_params(int rank, const int* dim, const int* perm, int elt,
                              unsigned tinBytes, unsigned toutBytes, unsigned vtargetBytes,
                              int extend, int loopOrder, int maxVecBytes, int maxVBytes, int nthreads,
                              int groupIn, int groupOut,
                              const void* in, void* out, char* label, int labelLen) {
  Problem P;
  if (!problem_from_cutt(rank, dim, perm, elt, P)) return 2;
  if (P.identity) { memcpy(out, in, (size_t)P.volume * elt); return 0; }
  TileParams tp;
  tp.tinBytes = tinBytes; tp.toutBytes = toutBytes; tp.vtargetBytes = vtargetBytes;
  tp.extend = extend; tp.loopOrder = loopOrder; tp.maxVecBytes = maxVecBytes; tp.maxVBytes = maxVBytes; tp.nthreads = nthreads;
  tp.groupIn = groupIn; tp.groupOut = groupOut;
  Candidate c;
  if (!build_tile(P, tp, g_dev, c)) return 5;
  if (label && labelLen > 0) snprintf(label, labelLen, "%s", describe(P, c).c_str());
  return dispatch_checked(c.desc, (const unsigned char*)in, (unsigned char*)out, (size_t)P.volume * elt);
}

// Sharded permutation, rank `me` of `world`: `in` is the local input slab, `outs[h]` the output
// slab of GPU h (all of them host arrays here).  Returns the mode (0 slab, 1 all-to-all) or a
// negative code.  Candidate `index` of the enumeration is executed.
int cutt_hostcheck_run_sharded(int rank, const int* dim, const int* perm, int elt, int world, int me,
                               int index, const void* in, void* const* outs, char* label, int labelLen) {
  Problem P;
  ShardInfo info;
  if (!problem_from_cutt_sharded(rank, dim, perm, elt, world, me, P, info)) return -2;
  const std::vector<Candidate>& cands = candidates_of(P);
  if (cands.empty()) return -3;
  if (index < 0) index = 0;
  index %= (int)cands.size();
  const Candidate& c = cands[index];
  if (label && labelLen > 0) snprintf(label, labelLen, "%s", describe(P, c).c_str());
  const size_t bytes = (size_t)info.localVolume * elt;
  if (c.method != kMethodTiles) {   // slab mode only: an ordinary local problem
    if (info.mode != 0) return -4;
    unsigned char* o = (unsigned char*)outs[me];
    int rc = 0;
    if (c.method == kMethodCopy || c.method == kMethodMemcpy) memcpy(o, in, bytes);
    else if (c.method == kMethodRowCopy) rc = run_rowcopy(c.rc, (const unsigned char*)in, o, bytes);
    else if (c.method == kMethodTma) rc = run_tma(c, (const unsigned char*)in, o, bytes);
    else if (c.method == kMethodT2d) rc = run_t2d(c, (const unsigned char*)in, bytes, o, o, o + bytes);
    else rc = 4;
    return rc ? -5 : 0;
  }
  HostBounds& b = host_bounds();
  b.gin0 = (const unsigned char*)in; b.gin1 = b.gin0 + bytes; b.violations = 0;
  // outputs: accept any address inside any destination slab
  const unsigned char* lo = (const unsigned char*)outs[0];
  const unsigned char* hi = lo + bytes;
  for (int h = 0; h < world; h++) {
    const unsigned char* p = (const unsigned char*)outs[h];
    if (p < lo) lo = p;
    if (p + bytes > hi) hi = p + bytes;
  }
  b.gout0 = lo; b.gout1 = hi;
  g_peerOuts = (unsigned char* const*)outs;
  int rc = dispatch(c.desc, (const unsigned char*)in, (unsigned char*)outs[info.mode == 0 ? me : 0]);
  g_peerOuts = nullptr;
  if (rc) return -5;
  if (b.violations) return -9;
  return info.mode;
}

// The host-buffer pipeline cuts the input into slabs along its slowest dimension and permutes
// each slab straight into the full output (strided).  This runs that decomposition on the host:
// `nslab` slabs, candidate `index` of each slab's enumeration.
int cutt_hostcheck_run_chunked(int rank, const int* dim, const int* perm, int elt, int nslab, int index,
                               const void* in, void* out) {
  const int last = rank - 1;
  const int dlast = dim[last];
  if (nslab < 1) return 2;
  const int chunk = (dlast + nslab - 1) / nslab;
  size_t isLast = 1, osLast = 1;
  for (int i = 0; i < last; i++) isLast *= (size_t)dim[i];
  for (int k = 0; k < rank && perm[k] != last; k++) osLast *= (size_t)dim[perm[k]];
  size_t total = (size_t)elt;
  for (int i = 0; i < rank; i++) total *= (size_t)dim[i];
  for (int c0 = 0; c0 < dlast; c0 += chunk) {
    const int ext = c0 + chunk <= dlast ? chunk : dlast - c0;
    Problem P;
    if (!problem_from_cutt_chunk(rank, dim, perm, elt, ext, P)) return 2;
    const unsigned char* pin = (const unsigned char*)in + (size_t)c0 * isLast * elt;
    unsigned char* pout = (unsigned char*)out + (size_t)c0 * osLast * elt;
    const std::vector<Candidate>& cands = candidates_of(P);
    if (cands.empty()) return 3;
    Candidate c = cands[(size_t)index % cands.size()];
    if (c.method == kMethodTiles) {
      // what the library does at execute time: pointers that are not aligned for the plan's
      // vector widths take the element-wise variant of the same tile
      const TileDesc& D = c.desc;
      const bool inOk = D.aof ? ((uintptr_t)pin % (D.vblk * D.elt) == 0) : ((uintptr_t)pin % (D.in.vec * D.elt) == 0);
      const bool outOk = (uintptr_t)pout % (D.out.vec * D.elt) == 0;
      if (!inOk || !outOk) {
        TileParams tp = c.params;
        tp.maxVecBytes = elt; tp.maxVBytes = elt; tp.allowAof = 0;
        Candidate f;
        if (!build_tile(P, tp, g_dev, f)) return 6;
        c = f;
      }
    }
    if (c.method == kMethodCopy || c.method == kMethodMemcpy) {
      memcpy(pout, pin, (size_t)P.volume * elt);
    } else if (c.method == kMethodT2d) {
      const uintptr_t ai = c.t2d.loadMode == 1 ? elt : c.t2d.loadMode, ao = c.t2d.storeMode == 1 ? elt : c.t2d.storeMode;
      if ((uintptr_t)pin % ai || (uintptr_t)pout % ao) {   // as the library: the modes that take any address
        TileParams tp = c.params;
        tp.maxVecBytes = 16;
        tp.extend = 1;
        Candidate f;
        if (!build_t2d(P, tp, g_dev, f)) return 6;
        c = f;
      }
      if (run_t2d(c, pin, (size_t)P.volume * elt, pout, (unsigned char*)out, (unsigned char*)out + total)) return 9;
    } else if (c.method == kMethodTma) {
      if ((uintptr_t)pin % 16 || (uintptr_t)pout % 16) return 7;   // (the library would take its fallback tile)
      if (run_tma(c, pin, pout, (size_t)P.volume * elt, (unsigned char*)out, (unsigned char*)out + total)) return 9;
    } else if (c.method == kMethodRowCopy) {
      rowcopy_bounds().in0 = pin; rowcopy_bounds().in1 = pin + (size_t)P.volume * elt;
      rowcopy_bounds().out0 = (unsigned char*)out; rowcopy_bounds().out1 = (unsigned char*)out + total;
      rowcopy_violations() = 0;
      for (uint32_t item = 0; item < c.rc.numItems; item++)
        for (uint32_t lane = 0; lane < 32; lane++) {
          if (elt == 4) rowcopy_item<4>(c.rc, pin, pout, item, lane);
          else rowcopy_item<8>(c.rc, pin, pout, item, lane);
        }
      if (rowcopy_violations()) return 9;
    } else {
      HostBounds& b = host_bounds();
      b.gin0 = pin; b.gin1 = pin + (size_t)P.volume * elt;
      b.gout0 = (unsigned char*)out; b.gout1 = (unsigned char*)out + total;
      b.violations = 0;
      if (dispatch(c.desc, pin, pout)) return 4;
      if (b.violations) return 9;
    }
  }
  return 0;
}

// Exhaustive-ish self check of the division helper: returns the number of mismatches.
long long cutt_hostcheck_fastdiv(unsigned d, unsigned long long nmax, unsigned long long step) {
  FastDiv f = make_fastdiv(d);
  long long bad = 0;
  for (unsigned long long n = 0; n <= nmax; n += step) if (fdiv((uint32_t)n, f) != (uint32_t)n / d) bad++;
  const uint32_t edge[] = {0u, 1u, d - 1, d, d + 1, 0x7fffffffu, 0x80000000u, 0xfffffffeu, 0xffffffffu};
  for (uint32_t n : edge) if (fdiv(n, f) != n / d) bad++;
  return bad;
}

// Builds every tile with 64-bit row offsets from now on (on != 0) or as the planner decides.
void cutt_hostcheck_force_wide(int on) {
  debug_force_wide_offsets(on != 0);
  g_candidatesStale = true;
}

}  // extern "C"
