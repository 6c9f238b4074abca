// Two-dimensional tile transpose with swizzled shared memory ("t2d"): descriptor and the per-thread
// load / store steps, shared by the device kernel (tile2d.cu) and the host-side plan interpreter.
//
// Problem class.  Canonical problems (planner.h) whose input dimension 0 is contiguous and whose
// output-fastest dimension p is another dimension; any alignment, up to six loop dimensions.  A tile
// is ta elements along dimension 0 by tb elements along dimension p, one tile per thread block.
// This is the case the reference serves with transposeTiled (src/cuttkernel.cu:123-222) and the
// general tiled kernel of this library with a descriptor-driven code path; here the tile shape is
// fixed enough for the index arithmetic to collapse to shifts and masks, which is what the
// instruction-bound 4-byte cases need.
//
// Shared memory holds the tile as rows of 128 bytes along dimension 0 (nboxes row blocks side by
// side), row r of a block at r * 128, its 16-byte chunk c at chunk position c ^ (r & 7) - the
// layout the tensor-map kernel gets from the copy engine (tma_transpose.h).
//
// Load: cp.async of WIB bytes (16, 8 or 4: what the alignment of the input rows allows), consecutive
// lanes along a row.  Store: an item is one 16-byte chunk (V = 16/elt elements along dimension 0) of
// wo = WOB/elt consecutive rows: wo shared-memory vector loads, a register transpose, V global
// stores of WOB bytes (16, 8 or 4: what the alignment of the output rows allows).  The lanes of a
// warp are spread over WOB/4 chunks and 128/WOB row groups, so every store instruction writes 128
// contiguous bytes of each output row it touches, and the row groups met by a quarter warp differ
// in the row bits the swizzle uses: shared-memory reads are conflict free.
#pragma once
#include "permute_desc.h"
#include "permute_tile_impl.h"

namespace cuttb {

constexpr int kT2dMaxOuter = 6;

struct T2dDesc {
  uint32_t elt;        // 4 or 8
  uint32_t ta;         // tile extent along dimension 0 (elements); ta * elt is a multiple of 128
  uint32_t tb;         // tile extent along dimension p (elements): 32 or 64
  uint32_t tbShift;    // log2(tb)
  uint32_t nboxes;     // ta * elt / 128
  uint32_t nthreads;
  uint32_t wiB, woB;   // bytes per access on the input / output side
  uint32_t numTiles;
  uint32_t order;      // tile index runs fastest along 0: dimension 0, 1: dimension p
  uint32_t d0, dp;
  uint32_t nA, nB;
  uint32_t nOuter;
  uint32_t nO[kT2dMaxOuter];
  uint32_t pad_;
  FastDiv divA, divB, divO[kT2dMaxOuter];
  int64_t isP;         // input stride of dimension p (elements)
  int64_t os0;         // output stride of dimension 0 (elements)
  int64_t isO[kT2dMaxOuter], osO[kT2dMaxOuter];
  int64_t inBase, outBase;
};

struct T2dTile {
  uint32_t c0, cp;
  int64_t inOff, outOff;   // offsets of the tile origin (elements)
};

CUTT_HD void t2d_decode(const T2dDesc& D, uint32_t tile, T2dTile& t) {
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
  t.inOff = D.inBase + (int64_t)t.c0 + (int64_t)t.cp * D.isP;
  t.outOff = D.outBase + (int64_t)t.c0 * D.os0 + (int64_t)t.cp;
  for (uint32_t k = 0; k < D.nOuter; k++) {
    const uint32_t q = fdiv(id, D.divO[k]);
    const uint32_t c = id - q * D.nO[k];
    id = q;
    t.inOff += (int64_t)c * D.isO[k];
    t.outOff += (int64_t)c * D.osO[k];
  }
}

CUTT_HD uint32_t t2d_load_units(const T2dDesc& D) { return D.ta * D.tb * D.elt / D.wiB; }
CUTT_HD uint32_t t2d_store_items(const T2dDesc& D) { return (D.ta * D.elt / 16u) * (D.tb * D.elt / D.woB); }

// Load unit u: WIB bytes of one tile row.
template <int ELT, int WIB>
CUTT_HD void t2d_load_unit(const T2dDesc& D, const T2dTile& t, sptr_t stage, const unsigned char* gin, uint32_t u) {
  constexpr uint32_t UPR = 128u / WIB;            // units per 128-byte row
  const uint32_t q = u & (UPR - 1u);
  const uint32_t rr = u / UPR;
  const uint32_t r = rr & (D.tb - 1u);
  const uint32_t k = rr >> D.tbShift;             // row block (128 bytes of dimension 0 each)
  const uint32_t e0 = k * (128u / ELT) + q * (WIB / ELT);
  if (t.c0 + e0 >= D.d0 || t.cp + r >= D.dp) return;   // (extents are multiples of the access width)
  const unsigned char* g = gin + (t.inOff + (int64_t)e0 + (int64_t)r * D.isP) * ELT;
  const uint32_t byteInRow = q * WIB;
  const uint32_t s = k * (D.tb * 128u) + r * 128u + (((byteInRow >> 4) ^ (r & 7u)) << 4) + (byteInRow & 15u);
  copy_g2s<WIB>(stage + s, g);
}

// Store item `it`: wo rows x one 16-byte chunk -> V output rows x WOB bytes.
template <int ELT, int WOB>
CUTT_HD void t2d_store_item(const T2dDesc& D, const T2dTile& t, sptr_t stage, unsigned char* gout, uint32_t it) {
  constexpr int WO = WOB / ELT;          // rows per item = elements per global store
  constexpr int V = 16 / ELT;            // elements per shared-memory vector = output rows per item
  constexpr int EW = ELT / 4;            // 32-bit words per element
  constexpr uint32_t NC = WOB / 4;       // chunks the lanes of a warp spread over
  constexpr uint32_t NG = 128u / WOB;    // row groups the lanes of a warp spread over
  const uint32_t cl = it & (NC - 1u);
  uint32_t g = (it / NC) & (NG - 1u);
  const uint32_t rest = it >> 5;
  const uint32_t cblocks = (D.ta * ELT / 16u) / NC;     // a power of two
  const uint32_t cb = rest & (cblocks - 1u);
  const uint32_t gb = rest / cblocks;
  // 8-byte elements: an item is only WOB/8 rows high, half of what keeps neighbouring groups apart
  // in the swizzle's row bits; rotating the low three bits of the group number restores that
  if (ELT == 8) g = (g & ~7u) | ((g << 1) & 6u) | ((g >> 2) & 1u);
  const uint32_t chunk = cb * NC + cl;
  const uint32_t row0 = (gb * NG + g) * (uint32_t)WO;
  const uint32_t r0 = t.c0 + chunk * (uint32_t)V;
  if (r0 >= D.d0 || t.cp + row0 >= D.dp) return;
  const uint32_t box = chunk >> 3, cib = chunk & 7u;
  uint32_t x[WO][4];
#pragma unroll
  for (int i = 0; i < WO; i++) {
    const uint32_t row = row0 + (uint32_t)i;
    lds<16>(x[i], stage + box * (D.tb * 128u) + row * 128u + ((cib ^ (row & 7u)) << 4));
  }
  unsigned char* g0 = gout + (t.outOff + (int64_t)(chunk * (uint32_t)V) * D.os0 + (int64_t)row0) * ELT;
  const int64_t os0B = D.os0 * ELT;
#pragma unroll
  for (int j = 0; j < V; j++) {
    if (r0 + (uint32_t)j < D.d0) {
      uint32_t y[WO * EW];
#pragma unroll
      for (int i = 0; i < WO; i++) {
#pragma unroll
        for (int w = 0; w < EW; w++) y[i * EW + w] = x[i][j * EW + w];
      }
      stg<WOB>(g0, y);
    }
    g0 += os0B;
  }
}

}  // namespace cuttb
