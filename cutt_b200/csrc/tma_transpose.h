// Tensor-map (TMA) transpose: descriptor and the per-thread store phase, shared by the device
// kernel (tma_transpose.cu) and the host-side plan interpreter used by the CPU tests.
//
// Problem class.  Canonical problems (planner.h) of fused rank 2-5 whose input dimension 0 is
// contiguous and whose output-fastest dimension p is another dimension, with every stride on
// both sides a multiple of 16 bytes - the class for which a tensor map over the input is legal
// and the output can be written with aligned 16-byte stores.  A tile is ta elements along
// dimension 0 by tb elements along dimension p; all other dimensions are loop dimensions.
// It replaces what the reference does for this class with transposeTiled
// (src/cuttkernel.cu:123-222: 32x32 tiles, one element per thread and access).
//
// Load.  One elected thread issues, per tile, `nboxes` box loads (cp.async.bulk.tensor.5d, box =
// 128 bytes along dimension 0 by tb rows along dimension p) that complete on an mbarrier; the
// copy engine writes each box into shared memory in the 128-byte swizzle mode: 16-byte chunk c
// of row r lands at chunk position c ^ (r & 7).  Elements outside the tensor are filled with
// zeros by the engine, so edge tiles need no special load code.
//
// Store.  An item is one 16-byte chunk (V = 16/elt elements along dimension 0) of W = 16/elt
// consecutive rows: W shared-memory vector loads, a V x W transpose in registers, V global
// 16-byte stores (one per output row).  Lane l of a warp takes chunk (l & 3) of row group
// (l >> 2): per store instruction a warp writes 4 output rows x 128 contiguous bytes, and the
// two row groups met by a quarter warp are four rows apart, which the swizzle maps to disjoint
// bank groups - shared-memory reads are conflict free.
#pragma once
#include "permute_desc.h"
#include "permute_tile_impl.h"

namespace cuttb {

constexpr int kTmaMaxStages = 8;
constexpr uint32_t kTmaBoxBytes = 128;   // bytes of one box row = swizzle span

struct TmaDesc {
  uint32_t elt;        // 4 or 8
  uint32_t ta;         // tile extent along dimension 0 (elements); ta * elt is a multiple of 128
  uint32_t tb;         // tile extent along dimension p (elements); a multiple of 8 * (16 / elt)
  uint32_t nboxes;     // ta * elt / 128
  uint32_t cbShift;    // log2(ta * elt / 64): blocks of four chunks along dimension 0
  uint32_t stages;
  uint32_t nthreads;
  uint32_t numTiles;
  uint32_t order;      // tile index runs fastest along 0: dimension 0, 1: dimension p
  uint32_t d0, dp;     // extents of the two tile dimensions
  uint32_t nA, nB;     // tiles along dimension 0 / dimension p
  uint32_t nOuter;     // loop dimensions beside the two tile dimensions (0..3)
  uint32_t nO[3];
  uint32_t pSlot;      // position (1..4) of dimension p among the tensor map's dimensions
  FastDiv divA, divB, divO[3];
  int64_t os0;         // output stride of dimension 0 (elements)
  int64_t osO[3];      // output strides of the loop dimensions
};

// What cuTensorMapEncodeTiled needs for the input tensor (host side only): the problem's
// dimensions in input order (ascending strides, as for any dense tensor); the box is 128 bytes
// along dimension 0, tb along dimension p (slot pSlot) and 1 elsewhere; unused trailing dimensions
// have extent 1.
struct TmaMapRecipe {
  uint64_t dims[5];
  uint64_t strideBytes[4];   // strides of dimensions 1..4
  uint32_t box[5];
};

struct TmaTile {
  uint32_t c0, cp;     // coordinates of the tile origin along dimension 0 / p
  uint32_t co[3];      // coordinates along the loop dimensions
  uint32_t pad_;
  int64_t outOff;      // output offset of the tile origin (elements)
};

CUTT_HD void tma_decode(const TmaDesc& D, uint32_t tile, TmaTile& t) {
  uint32_t id = tile, a, b;
  if (D.order == 0) {
    uint32_t q = fdiv(id, D.divA); a = id - q * D.nA; id = q;
    q = fdiv(id, D.divB); b = id - q * D.nB; id = q;
  } else {
    uint32_t q = fdiv(id, D.divB); b = id - q * D.nB; id = q;
    q = fdiv(id, D.divA); a = id - q * D.nA; id = q;
  }
  t.c0 = a * D.ta;
  t.cp = b * D.tb;
  t.pad_ = 0;
  t.outOff = (int64_t)t.c0 * D.os0 + (int64_t)t.cp;
  // unused loop dimensions have extent 1 (coordinate 0, stride 0): three fixed steps, no loop
#pragma unroll
  for (int k = 0; k < 3; k++) {
    const uint32_t q = fdiv(id, D.divO[k]);
    const uint32_t c = id - q * D.nO[k];
    id = q;
    t.co[k] = c;
    t.outOff += (int64_t)c * D.osO[k];
  }
}

// Coordinates of box k of tile t in the order of the tensor map's dimensions: dimension 0, then
// the loop dimensions with dimension p inserted at slot pSlot.
CUTT_HD void tma_box_coords(const TmaDesc& D, const TmaTile& t, uint32_t k, int& c0, int& c1, int& c2, int& c3, int& c4) {
  const uint32_t p = D.pSlot;
  c0 = (int)(t.c0 + k * (kTmaBoxBytes / D.elt));
  c1 = (int)(p == 1 ? t.cp : t.co[0]);
  c2 = (int)(p == 1 ? t.co[0] : (p == 2 ? t.cp : t.co[1]));
  c3 = (int)(p <= 2 ? t.co[1] : (p == 3 ? t.cp : t.co[2]));
  c4 = (int)(p == 4 ? t.cp : t.co[2]);
}

CUTT_HD uint32_t tma_items_per_tile(const TmaDesc& D) {
  return (D.ta * D.elt / 16u) * (D.tb / (16u / D.elt));
}

// Shared-memory byte offset (within a stage) of 16-byte chunk `chunk` (counted along dimension 0
// over the whole tile) of row `row`.
CUTT_HD uint32_t tma_smem_offset(const TmaDesc& D, uint32_t chunk, uint32_t row) {
  const uint32_t box = chunk >> 3, cib = chunk & 7u;
  return box * (D.tb * kTmaBoxBytes) + row * kTmaBoxBytes + ((cib ^ (row & 7u)) << 4);
}

// Item `it` of the tile in `stage`: W rows x one chunk -> V output rows x 16 bytes.
template <int ELT>
CUTT_HD void tma_store_item(const TmaDesc& D, const TmaTile& t, sptr_t stage, unsigned char* gout, uint32_t it) {
  constexpr int W = 16 / ELT;   // rows per item = elements per 16-byte global store
  constexpr int V = 16 / ELT;   // elements per 16-byte shared-memory vector = output rows per item
  constexpr int EW = ELT / 4;   // 32-bit words per element
  const uint32_t c4 = it & 3u, g = (it >> 2) & 7u, rest = it >> 5;
  const uint32_t cb = rest & ((1u << D.cbShift) - 1u), gb = rest >> D.cbShift;
  const uint32_t chunk = cb * 4u + c4;
  // 8-byte elements: items are two rows high, so neighbouring groups would be two rows apart and
  // the swizzle would map them to the same banks; swapping the low two bits of the group number
  // puts the two groups of a quarter warp four rows apart
  const uint32_t gg = (ELT == 8) ? ((g & 4u) | ((g & 1u) << 1) | ((g >> 1) & 1u)) : g;
  const uint32_t row0 = (gb * 8u + gg) * (uint32_t)W;
  const uint32_t r0 = t.c0 + chunk * (uint32_t)V;   // dimension-0 coordinate of the first output row
  if (r0 >= D.d0 || t.cp + row0 >= D.dp) return;    // extents are multiples of V and W: whole vectors
  uint32_t x[W][4];
#pragma unroll
  for (int i = 0; i < W; i++) lds<16>(x[i], stage + tma_smem_offset(D, chunk, row0 + (uint32_t)i));
  unsigned char* g0 = gout + (t.outOff + (int64_t)(chunk * (uint32_t)V) * D.os0 + (int64_t)row0) * ELT;
  const int64_t os0B = D.os0 * ELT;
#pragma unroll
  for (int j = 0; j < V; j++) {
    uint32_t y[4];
#pragma unroll
    for (int i = 0; i < W; i++) {
#pragma unroll
      for (int w = 0; w < EW; w++) y[i * EW + w] = x[i][j * EW + w];
    }
    stg<16>(g0, y);
    g0 += os0B;
  }
}

}  // namespace cuttb
