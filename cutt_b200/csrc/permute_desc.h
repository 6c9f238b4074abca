// Plan descriptor of the tiled permutation kernels, and the index arithmetic that
// host code (planner, host-side plan interpreter used by the CPU tests) and device
// code (the kernels) share.  Everything here is plain data + inline functions.
//
// Model.  A permutation is a strided copy: element with coordinates c[0..r) lives at
// in[sum c_j * istride_j] and goes to out[sum c_j * ostride_j].  A *tile* gives every
// dimension an extent t_j <= d_j.  Dimensions with t_j < d_j are also *loop*
// dimensions: the tile grid has ceil(d_j / t_j) positions along them.  On each side
// (input, output) the tile's elements form `nrows` contiguous *runs* of `run`
// elements in global memory; the run is made of the leading dimensions in that
// side's stride order, the rows enumerate the remaining tile dimensions.  In shared
// memory the tile is kept in input order (a run of the input side is contiguous),
// padded and skewed so that the gather performed by the output side spreads over banks.
//
// Output side register blocking: when the fastest input dimension (dimension 0) is a
// row dimension of the output side, rows are handled in groups of V along it.  A thread
// then reads W vectors of V elements from shared memory (V consecutive along dimension 0,
// for W consecutive positions of the output run) and writes V vectors of W elements to
// global memory; the V x W transpose happens in registers.
//
// Aligned over-fetch (aof): when input rows do not start on 16-byte boundaries, each row is
// still fetched with 16-byte cp.async from the enclosing aligned range (a few elements of the
// neighbouring rows come along and are ignored; vectors that would leave the buffer are replaced
// by element copies).  The row then sits in shared memory displaced by its misalignment
// `shift = (address / elt) mod (16 / elt)`; the store side recomputes that shift from the tile
// origin and from per-row / per-position residues carried in the low bits of the table offsets.
//
// At most two dimensions may have 1 < t_j < d_j with d_j not a multiple of t_j
// ("partial" dimensions, slots 0 and 1); the last tile along such a dimension is
// short, which is handled by comparing coordinates with the remaining extent.
//
// This replaces the TensorConv/TensorConvInOut tables and the Mm/Mk/Mmk/Mbar
// decomposition of the reference (src/cuttTypes.h:30-44, src/cuttplan.cpp:817-1046):
// those are built on the host and copied to the device per plan; here the descriptor
// travels as a kernel argument and the per-row tables are rebuilt in shared memory by
// each thread block, so a plan owns no device memory.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define CUTT_HD __host__ __device__ __forceinline__
#else
#define CUTT_HD inline
#endif

namespace cuttb {

constexpr int kMaxDims = 16;     // maximum rank after fusion handled by the tiled kernels
constexpr int kMaxPeers = 8;     // GPUs addressable by one multi-GPU launch

// Exact unsigned division of any 32-bit n by a fixed divisor d >= 1
// (multiply-high + shifts; Granlund & Montgomery, "Division by invariant integers").
struct FastDiv {
  uint32_t mul;
  uint32_t sh1;
  uint32_t sh2;
  uint32_t d;
};

inline FastDiv make_fastdiv(uint32_t d) {
  FastDiv f;
  f.d = d;
  uint32_t l = 0;
  while ((1ull << l) < d) l++;
  f.mul = (uint32_t)((((1ull << l) - d) << 32) / d + 1);
  f.sh1 = l < 1 ? l : 1;
  f.sh2 = l == 0 ? 0 : l - 1;
  return f;
}

CUTT_HD uint32_t mulhi_u32(uint32_t a, uint32_t b) {
#if defined(__CUDA_ARCH__)
  return __umulhi(a, b);
#else
  return (uint32_t)(((uint64_t)a * b) >> 32);
#endif
}

CUTT_HD uint32_t fdiv(uint32_t n, const FastDiv& f) {
  uint32_t t = mulhi_u32(f.mul, n);
  return (t + ((n - t) >> f.sh1)) >> f.sh2;
}

// Row-table entries (built per thread block in shared memory).  goff: global offset of
// the run start relative to the tile origin, in elements; soffB: shared-memory offset of
// the row base in bytes.  The narrow form is used when every goff fits 32 bits.
struct RowEntN {
  uint32_t goff;
  uint32_t soffB;
};
struct __attribute__((aligned(16))) RowEntW {
  int64_t goff;
  uint32_t soffB;
  uint32_t pad_;
};
template <bool WIDE> struct RowEntSel { typedef RowEntN type; };
template <> struct RowEntSel<true> { typedef RowEntW type; };

// Coordinates of a row along the two partial dimensions (elements; 0 if not applicable).
struct RowCoord {
  uint16_t c0;
  uint16_t c1;
};

// Skew of a dimension's shared-memory placement: position c is moved by
// ((c >> shift) & mask) * unitB bytes so that lanes that are W positions apart do not
// meet in the same bank group.
struct Skew {
  uint32_t shift;
  uint32_t mask;   // 0: no skew
  uint32_t unitB;
};

// A tile dimension that enumerates rows of one side.
struct RowDim {
  uint32_t ext;      // positions along this dimension within the tile
  uint32_t sstrideB; // shared-memory stride per position (bytes)
  int64_t gstride;   // global stride per position on this side (elements)
  int32_t slot;      // partial slot (0/1) this dimension feeds, or -1
  uint32_t cmul;     // elements per position (V for the register-blocked dimension, else 1)
  Skew skew;
  uint32_t ishift;   // aligned over-fetch mode: input stride of this dimension modulo the vector
                     // width (elements) if the dimension selects input rows, else 0
  FastDiv div;       // division by ext (row-table construction)
};

// A dimension inside the output side's run: turns a position along the run into a
// shared-memory offset (the gather).
struct RunDim {
  FastDiv div;       // division by the tile extent
  uint32_t sstrideB; // shared-memory stride (bytes)
  Skew skew;
  uint32_t ishift;   // as RowDim::ishift
  uint32_t pad_[3];
};

struct Side {
  uint32_t run;        // elements per run in a full tile
  uint32_t runPrefix;  // run length = runPrefix * (extent of the run's last dimension)
  int32_t runSlot;     // partial slot that shortens the run in the last tile, or -1
  uint32_t nrows;      // rows (output side: row groups of V) per tile
  uint32_t nRowDims;
  uint32_t vec;        // elements per global memory access on this side (1, 2 or 4)
  uint32_t tq;         // threads along the run (power of two, <= block size)
  uint32_t tqShift;    // log2(tq)
  RowDim rowDim[kMaxDims];
};

// One digit of the tile index.  A dimension normally contributes one digit ("whole").  The
// chunked dimension of a run may be split into an inner digit (a small group of neighbouring
// tiles, placed first so that blocks running at the same time touch neighbouring memory) and
// an outer digit; positions past the end of the dimension are skipped.
struct LoopDim {
  FastDiv div;      // division by n
  uint32_t n;       // positions of this digit
  uint32_t t;       // tile extent
  uint32_t d;       // full extent
  int32_t slot;     // partial slot fed by this dimension, or -1 (whole digits only)
  uint32_t part;    // 0 whole, 1 inner digit, 2 outer digit of a split dimension
  uint32_t which;   // split dimension index (0/1) for part != 0
  uint32_t mul;     // tile positions per step of this digit (group size for an outer digit, else 1)
  uint32_t pad_;
  int64_t istep;    // input offset per step (istride * t * mul)
  int64_t ostep;    // output offset per step; unused for the peer dimension
};

struct SplitDim {
  uint32_t used;
  uint32_t n;       // tile positions along the dimension
  uint32_t t;
  uint32_t d;
  int32_t slot;
  uint32_t pad_[3];
};

struct TileDesc {
  uint32_t elt;         // element size in bytes (4 or 8)
  uint32_t nthreads;    // threads per block
  uint32_t numTiles;
  uint32_t nLoopDims;
  uint32_t nOutRunDims;
  uint32_t tileElems;   // shared-memory elements per stage (with padding)
  uint32_t stageBytes;  // bytes per stage, rounded up to 16
  uint32_t tableBytes;  // bytes of all tables in front of the stages, rounded up to 16
  uint32_t stages;      // shared-memory stages (1 or 2)
  uint32_t smemGatherContig; // 1 if `out.vec` consecutive run positions are contiguous and aligned in smem
  uint32_t vblk;        // V: rows of the output side handled together along dimension 0 (1, 2 or 4)
  uint32_t wide;        // 1: 64-bit row offsets
  int32_t peerLoopDim;  // loop dimension whose coordinate selects the destination GPU, or -1
  uint32_t aof;         // 1: aligned over-fetch loads (see below)
  uint32_t peerRot;     // added (modulo the GPU count) to the peer digit of the tile index: GPU r
                        // starts with destination r, so that at any moment the GPUs of a job write
                        // to different destinations instead of all to the same one
  uint32_t pad0_;
  int64_t inElems;      // elements of the input buffer (bounds of the over-fetch)
  int64_t vstep;        // output offset between the V rows of a group (elements)
  int64_t inBase;       // element offset added to the input pointer
  int64_t outBase;      // element offset added to the output pointer
  Side in;
  Side out;
  RunDim outRunDim[kMaxDims];
  LoopDim loop[kMaxDims + 2];
  SplitDim split[2];
};

constexpr uint32_t kTileCtxBytes = 48;  // sizeof(TileCtx), checked below

// Shared-memory layout in front of the stage buffers.
struct TableLayout {
  uint32_t tabIn, tabOut, coordIn, coordOut, qtab, ctx, total;
};
CUTT_HD TableLayout table_layout(const TileDesc& D) {
  TableLayout L;
  const uint32_t esz = D.wide ? (uint32_t)sizeof(RowEntW) : (uint32_t)sizeof(RowEntN);
  L.tabIn = 0;
  L.tabOut = L.tabIn + D.in.nrows * esz;
  L.coordIn = L.tabOut + D.out.nrows * esz;
  L.coordOut = L.coordIn + D.in.nrows * (uint32_t)sizeof(RowCoord);
  L.qtab = (L.coordOut + D.out.nrows * (uint32_t)sizeof(RowCoord) + 15u) & ~15u;
  L.ctx = (L.qtab + D.out.run * 4u + 15u) & ~15u;
  L.total = L.ctx + 2u * kTileCtxBytes;  // two per-tile contexts, written by one thread, read by all
  return L;
}

// Per-tile context derived from the tile index.
struct __attribute__((aligned(16))) TileCtx {
  int64_t inOff;
  int64_t outOff;
  uint32_t rem0;     // remaining extent along partial slot 0 (huge if the tile is not short)
  uint32_t rem1;     // same for slot 1
  uint32_t peer;
  uint32_t partial;  // 1 if the tile is short along a partial dimension
  uint32_t valid;    // 0: the tile index falls past the end of a split dimension (nothing to do)
  uint32_t pad_;
};

static_assert(sizeof(TileCtx) == kTileCtxBytes, "table_layout reserves kTileCtxBytes per context");

CUTT_HD void set_rem(TileCtx& c, int32_t slot, uint32_t left, uint32_t t) {
  if (slot >= 0 && left < t) {
    c.partial = 1;
    if (slot == 0) c.rem0 = left; else c.rem1 = left;
  }
}

CUTT_HD void decode_tile(const TileDesc& D, uint32_t tile, TileCtx& c) {
  c.inOff = D.inBase;
  c.outOff = D.outBase;
  c.rem0 = 0xffffffffu;
  c.rem1 = 0xffffffffu;
  c.peer = 0;
  c.partial = 0;
  c.valid = 1;
  c.pad_ = 0;
  uint32_t id = tile;
  uint32_t pos0 = 0, pos1 = 0;
  for (uint32_t k = 0; k < D.nLoopDims; k++) {
    const LoopDim& L = D.loop[k];
    uint32_t q = fdiv(id, L.div);
    uint32_t cc = id - q * L.n;
    id = q;
    if ((int32_t)k == D.peerLoopDim) {
      cc += D.peerRot;
      if (cc >= L.n) cc -= L.n;
      c.peer = cc;
    } else {
      c.outOff += (int64_t)cc * L.ostep;
    }
    c.inOff += (int64_t)cc * L.istep;
    if (L.part == 0) {
      set_rem(c, L.slot, L.d - cc * L.t, L.t);
    } else if (L.which == 0) {
      pos0 += cc * L.mul;
    } else {
      pos1 += cc * L.mul;
    }
  }
  if (D.split[0].used) {
    const SplitDim& S = D.split[0];
    if (pos0 >= S.n) c.valid = 0;
    else set_rem(c, S.slot, S.d - pos0 * S.t, S.t);
  }
  if (D.split[1].used) {
    const SplitDim& S = D.split[1];
    if (pos1 >= S.n) c.valid = 0;
    else set_rem(c, S.slot, S.d - pos1 * S.t, S.t);
  }
}

CUTT_HD uint32_t skew_bytes(const Skew& s, uint32_t pos) {
  return ((pos >> s.shift) & s.mask) * s.unitB;
}

// Row `r` of one side: mixed-radix decode over the side's row dimensions.
CUTT_HD void make_row(const Side& S, uint32_t r, int64_t& goff, uint32_t& soffB, RowCoord& rc) {
  goff = 0;
  soffB = 0;
  rc.c0 = 0;
  rc.c1 = 0;
  uint32_t resid = 0;
  for (uint32_t k = 0; k < S.nRowDims; k++) {
    const RowDim& R = S.rowDim[k];
    const uint32_t nr = fdiv(r, R.div);
    uint32_t cc = r - nr * R.ext;
    r = nr;
    goff += (int64_t)cc * R.gstride;
    soffB += cc * R.sstrideB + skew_bytes(R.skew, cc);
    resid += cc * R.ishift;
    if (R.slot == 0) rc.c0 = (uint16_t)(cc * R.cmul);
    if (R.slot == 1) rc.c1 = (uint16_t)(cc * R.cmul);
  }
  soffB |= resid & 3u;  // zero unless the side uses aligned over-fetch residues
}

// Valid run length of a side in the tile described by `c`.
CUTT_HD uint32_t run_valid(const Side& S, const TileCtx& c) {
  if (S.runSlot < 0) return S.run;
  uint32_t rem = S.runSlot == 0 ? c.rem0 : c.rem1;
  if (rem == 0xffffffffu) return S.run;
  uint32_t v = S.runPrefix * rem;
  return v < S.run ? v : S.run;
}

// Shared-memory byte offset of position q along the output side's run.
CUTT_HD uint32_t out_run_soff(const TileDesc& D, uint32_t q) {
  uint32_t s = 0, resid = 0;
  for (uint32_t k = 0; k + 1 < D.nOutRunDims; k++) {
    const RunDim& R = D.outRunDim[k];
    uint32_t nq = fdiv(q, R.div);
    uint32_t cc = q - nq * R.div.d;
    s += cc * R.sstrideB + skew_bytes(R.skew, cc);
    resid += cc * R.ishift;
    q = nq;
  }
  const RunDim& R = D.outRunDim[D.nOutRunDims - 1];  // the last run dimension needs no modulo
  resid += q * R.ishift;
  return (s + q * R.sstrideB + skew_bytes(R.skew, q)) | (resid & 3u);
}

// Fills the shared-memory tables; thread `tid` of `nthreads` does its share.
template <bool WIDE>
CUTT_HD void build_tables(const TileDesc& D, unsigned char* tables, uint32_t tid, uint32_t nthreads) {
  typedef typename RowEntSel<WIDE>::type Ent;
  const TableLayout L = table_layout(D);
  Ent* tabIn = reinterpret_cast<Ent*>(tables + L.tabIn);
  Ent* tabOut = reinterpret_cast<Ent*>(tables + L.tabOut);
  RowCoord* coIn = reinterpret_cast<RowCoord*>(tables + L.coordIn);
  RowCoord* coOut = reinterpret_cast<RowCoord*>(tables + L.coordOut);
  uint32_t* qtab = reinterpret_cast<uint32_t*>(tables + L.qtab);
  // a side with at most one row dimension computes its row offsets by multiplication and never
  // reads its tables
  if (D.in.nRowDims > 1)
  for (uint32_t r = tid; r < D.in.nrows; r += nthreads) {
    int64_t g; uint32_t s; RowCoord rc;
    make_row(D.in, r, g, s, rc);
    tabIn[r].goff = (decltype(tabIn[r].goff))g;
    tabIn[r].soffB = s;
    coIn[r] = rc;
  }
  if (D.out.nRowDims > 1)
  for (uint32_t r = tid; r < D.out.nrows; r += nthreads) {
    int64_t g; uint32_t s; RowCoord rc;
    make_row(D.out, r, g, s, rc);
    tabOut[r].goff = (decltype(tabOut[r].goff))g;
    tabOut[r].soffB = s;
    coOut[r] = rc;
  }
  for (uint32_t q = tid; q < D.out.run; q += nthreads) qtab[q] = out_run_soff(D, q);
}

}  // namespace cuttb
