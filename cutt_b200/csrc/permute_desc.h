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
// with padding so that the gather performed by the output side spreads over banks.
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

// One entry of a side's row table (built per thread block in shared memory).
struct __attribute__((aligned(16))) RowEnt {
  int64_t goff;     // global offset of the run start, relative to the tile origin (elements)
  uint32_t soff;    // shared-memory offset of the row base (elements)
  uint16_t c0;      // coordinate of this row along partial dimension slot 0 (0 if none)
  uint16_t c1;      // same for slot 1
};

// A tile dimension that enumerates rows of one side.
struct RowDim {
  uint32_t ext;     // tile extent
  uint32_t sstride; // shared-memory stride (elements)
  int64_t gstride;  // global stride on this side (elements)
  int32_t slot;     // partial slot (0/1) this dimension feeds, or -1
  int32_t pad_;
};

// A dimension inside the output side's run: needed to turn a position along the run
// into a shared-memory offset (the gather).
struct RunDim {
  FastDiv div;      // division by ext
  uint32_t sstride; // shared-memory stride (elements)
  uint32_t pad_;
};

struct Side {
  uint32_t run;        // elements per run in a full tile
  uint32_t runPrefix;  // run length = runPrefix * (extent of the run's last dimension)
  int32_t runSlot;     // partial slot that shortens the run in the last tile, or -1
  uint32_t nrows;      // rows per tile
  uint32_t nRowDims;
  uint32_t vec;        // elements per memory access on this side (1, 2 or 4)
  uint32_t tq;         // threads along the run (power of two, <= block size)
  uint32_t tqShift;    // log2(tq)
  RowDim rowDim[kMaxDims];
};

struct LoopDim {
  FastDiv div;      // division by n
  uint32_t n;       // tiles along this dimension
  uint32_t t;       // tile extent
  uint32_t d;       // full extent
  int32_t slot;     // partial slot fed by this dimension, or -1
  int64_t istep;    // input offset per tile step (istride * t)
  int64_t ostep;    // output offset per tile step (ostride * t); unused for the peer dimension
};

struct TileDesc {
  uint32_t elt;         // element size in bytes (4 or 8)
  uint32_t nthreads;    // threads per block
  uint32_t numTiles;
  uint32_t nLoopDims;
  uint32_t nOutRunDims;
  uint32_t tileElems;   // shared-memory elements per stage (with padding)
  uint32_t stageBytes;  // bytes per stage, rounded up to 16
  uint32_t tableBytes;  // bytes of the two row tables
  uint32_t stages;      // shared-memory stages (1 or 2)
  uint32_t smemGatherContig; // 1 if `out.vec` consecutive run positions are contiguous and aligned in smem
  int32_t peerLoopDim;  // loop dimension whose coordinate selects the destination GPU, or -1
  uint32_t pad_;
  int64_t inBase;       // element offset added to the input pointer
  int64_t outBase;      // element offset added to the output pointer
  Side in;
  Side out;
  RunDim outRunDim[kMaxDims];
  LoopDim loop[kMaxDims];
};

// Per-tile context derived from the tile index.
struct TileCtx {
  int64_t inOff;
  int64_t outOff;
  uint32_t rem0;     // remaining extent along partial slot 0 (huge if the tile is not short)
  uint32_t rem1;     // same for slot 1
  uint32_t peer;
};

CUTT_HD void decode_tile(const TileDesc& D, uint32_t tile, TileCtx& c) {
  c.inOff = D.inBase;
  c.outOff = D.outBase;
  c.rem0 = 0xffffffffu;
  c.rem1 = 0xffffffffu;
  c.peer = 0;
  uint32_t id = tile;
  for (uint32_t k = 0; k < D.nLoopDims; k++) {
    const LoopDim& L = D.loop[k];
    uint32_t q = fdiv(id, L.div);
    uint32_t cc = id - q * L.n;
    id = q;
    c.inOff += (int64_t)cc * L.istep;
    if ((int32_t)k == D.peerLoopDim) c.peer = cc;
    else c.outOff += (int64_t)cc * L.ostep;
    if (L.slot >= 0) {
      uint32_t left = L.d - cc * L.t;
      left = left < L.t ? left : L.t;
      if (L.slot == 0) c.rem0 = left; else c.rem1 = left;
    }
  }
}

// Row `r` of one side: mixed-radix decode over the side's row dimensions.
CUTT_HD RowEnt make_row(const Side& S, uint32_t r) {
  RowEnt e;
  e.goff = 0;
  e.soff = 0;
  e.c0 = 0;
  e.c1 = 0;
  for (uint32_t k = 0; k < S.nRowDims; k++) {
    const RowDim& R = S.rowDim[k];
    uint32_t cc = r % R.ext;
    r /= R.ext;
    e.goff += (int64_t)cc * R.gstride;
    e.soff += cc * R.sstride;
    if (R.slot == 0) e.c0 = (uint16_t)cc;
    if (R.slot == 1) e.c1 = (uint16_t)cc;
  }
  return e;
}

// Valid run length of a side in the tile described by `c`.
CUTT_HD uint32_t run_valid(const Side& S, const TileCtx& c) {
  if (S.runSlot < 0) return S.run;
  uint32_t v = S.runPrefix * (S.runSlot == 0 ? c.rem0 : c.rem1);
  return v < S.run ? v : S.run;
}

// Shared-memory offset of position q along the output side's run.
CUTT_HD uint32_t out_run_soff(const TileDesc& D, uint32_t q) {
  uint32_t s = 0;
  for (uint32_t k = 0; k + 1 < D.nOutRunDims; k++) {
    const RunDim& R = D.outRunDim[k];
    uint32_t nq = fdiv(q, R.div);
    s += (q - nq * R.div.d) * R.sstride;
    q = nq;
  }
  // the last run dimension needs no modulo
  return s + q * D.outRunDim[D.nOutRunDims - 1].sstride;
}

}  // namespace cuttb
