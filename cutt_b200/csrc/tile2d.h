// Two-dimensional tile transpose with swizzled shared memory ("t2d"): descriptor and the per-thread
// load / store steps, shared by the device kernel (tile2d.cu) and the host-side plan interpreter.
//
// Problem class.  Canonical problems (planner.h) whose input dimension 0 is contiguous and whose
// output-fastest dimension p is another dimension; any alignment, up to six loop dimensions.  A tile
// is ta elements along dimension 0 by tb elements along dimension p, one tile per thread block.
// This is the case the reference serves with transposeTiled (src/cuttkernel.cu:123-222) and the
// general tiled kernel of this library with a descriptor-driven code path; here the tile shape is
// fixed enough for the index arithmetic to collapse to shifts and masks.
//
// Shared memory holds the tile as rows of 128 bytes along dimension 0 (nboxes row blocks side by
// side); 16-byte chunk c of shared-memory row s sits at chunk position c ^ (s & 7) - the layout the
// tensor-map kernel gets from the copy engine (tma_transpose.h).  Tile row q (a position along
// dimension p, relative to the tile origin) is shared-memory row q + padTop.
//
// Every global access is 16 bytes wide and 16-byte aligned, whatever the alignment of the rows:
//
// Load modes.  16: the input rows start on 16-byte boundaries: cp.async of 16 bytes.  1 ("shift"):
// they do not: for each 16-byte chunk of the tile the two aligned vectors that cover it are loaded
// (ld.global.v4), the chunk is cut out of them in registers and stored to shared memory; only the
// first and last vector of the whole buffer are read element by element.  8 and 4: cp.async of 8 or
// 4 bytes (kept as the plain alternative for rows on 8- or 4-byte boundaries).
//
// Store modes.  An item is one 16-byte chunk of shared memory (V = 16/elt elements along dimension
// 0, i.e. V output rows) over a few consecutive rows.  16: the output rows start on 16-byte
// boundaries: V shared vector loads (V = W rows), a V x W register transpose, V global stores of 16
// bytes.  1 ("shear"): they do not: output row c is misaligned by mo(c) elements, and the tile is
// sheared accordingly - for row c it covers positions [cp - mo(c), cp + tb - mo(c)) instead of
// [cp, cp + tb), so that every vector it writes is aligned; neighbouring tiles along p shear the
// same way and leave no gap.  An item then reads 2V-1 rows (the V windows of its V output rows lie
// within them), and the loads bring V-1 extra rows above the tile.  Only the first and last vector
// of an output row are written element by element.  8 and 4: narrower stores on V x (8/elt) or
// V x (4/elt) blocks.
//
// The lanes of a warp are spread over 4 chunks and 8 row groups (modes 16 and 1), so every store
// instruction writes 128 contiguous bytes of each output row it touches, and the row groups met by
// a quarter warp differ in the row bits the swizzle uses: shared-memory reads are conflict free.
//
// 1- and 2-byte elements (extension entry points; cp.async loads of 16, 8 or 4 bytes, stores of 16 or
// 8 bytes, no shift / shear): a chunk holds 16 / 8 elements, so an item is 16 / 8 rows (store mode 16)
// or 8 / 4 rows (store mode 8) of one chunk, transposed in registers with byte permutes
// (t2d_store_rows_e1*, t2d_store_rows_e2*).  Row groups this tall agree in the row bits the swizzle
// uses; where a quarter warp meets two or four of them, the later groups read their rows in rotated
// order - which changes exactly those bits - and undo the rotation on the output words.
#pragma once
#include "permute_desc.h"
#include "permute_tile_impl.h"

namespace cuttb {

constexpr int kT2dMaxOuter = 6;
constexpr uint32_t kT2dPadTop = 4;      // shared-memory rows in front of tile row 0 (sheared stores)
constexpr uint32_t kT2dPadBottom = 4;   // and behind the last one (never loaded, keeps reads in range)

struct T2dDesc {
  uint32_t elt;        // 4 or 8; 1 or 2 for the extension entry points
  uint32_t ta;         // tile extent along dimension 0 (elements); ta * elt is a multiple of 128
  uint32_t tb;         // tile extent along dimension p (elements): 32 or 64; up to 256 for 1- and 2-byte elements
  uint32_t nboxes;     // ta * elt / 128
  uint32_t nthreads;
  uint32_t loadMode;   // 16, 8, 4 or 1 (see above)
  uint32_t storeMode;  // 16, 8, 4 or 1
  uint32_t padTop;     // kT2dPadTop for sheared stores, else 0
  uint32_t rowsLoad;   // rows loaded per tile: tb, plus 16/elt - 1 rows above it for sheared stores
  uint32_t rowsAlloc;  // shared-memory rows per row block
  uint32_t uprShift;   // log2(load units per tile row)
  uint32_t inMis;      // (input buffer address / elt) mod (16/elt); set when the kernel is launched
  uint32_t outMis;     // same for the output buffer
  uint32_t numTiles;
  uint32_t laneMap;    // 1- and 2-byte elements: 0 = a quarter warp takes the 8 chunks of one row (a store
                       // instruction writes 64 contiguous bytes per output row), 1 = 4 chunks x 8 row
                       // groups per warp with the odd groups walking their rows from the middle (128 bytes)
  uint32_t order;      // tile index runs fastest along 0: dimension 0, 1: dimension p; 2 / 3: as 1 / 0,
                       // but in bands of four tiles across the other dimension (blocks that run at the
                       // same time then share lines on BOTH sides); tile indices past the end of a
                       // band are empty
  uint32_t d0, dp;
  uint32_t nA, nB;
  uint32_t nOuter;
  uint32_t nO[kT2dMaxOuter];
  uint32_t nBand;      // orders 2 / 3: bands of four tiles along dimension 0 / p
  FastDiv divA, divB, divBand, divRows, divO[kT2dMaxOuter];
  int64_t isP;         // input stride of dimension p (elements)
  int64_t os0;         // output stride of dimension 0 (elements)
  int64_t isO[kT2dMaxOuter], osO[kT2dMaxOuter];
  int64_t inBase, outBase;
  int64_t inElems;     // elements of the input buffer (the over-fetching loads stay inside it)
};

struct T2dTile {
  uint32_t c0, cp;
  int64_t inOff, outOff;   // offsets of the tile origin (elements)
};

// false: the tile index names no tile (bands of the orders 2 and 3 are padded to a multiple of four)
CUTT_HD bool t2d_decode(const T2dDesc& D, uint32_t tile, T2dTile& t) {
  uint32_t id = tile, a, b;
  if (D.order == 0) {
    uint32_t q = fdiv(id, D.divA); a = id - q * D.nA; id = q;
    q = fdiv(id, D.divB); b = id - q * D.nB; id = q;
  } else if (D.order == 1) {
    uint32_t q = fdiv(id, D.divB); b = id - q * D.nB; id = q;
    q = fdiv(id, D.divA); a = id - q * D.nA; id = q;
  } else if (D.order == 2) {   // four tiles along dimension 0, then along p, then the bands of dimension 0
    const uint32_t lo = id & 3u; id >>= 2;
    uint32_t q = fdiv(id, D.divB); b = id - q * D.nB; id = q;
    q = fdiv(id, D.divBand); a = (id - q * D.nBand) * 4u + lo; id = q;
    if (a >= D.nA) return false;
  } else {                     // four tiles along p, then along dimension 0, then the bands of p
    const uint32_t lo = id & 3u; id >>= 2;
    uint32_t q = fdiv(id, D.divA); a = id - q * D.nA; id = q;
    q = fdiv(id, D.divBand); b = (id - q * D.nBand) * 4u + lo; id = q;
    if (b >= D.nB) return false;
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
  return true;
}

// Shared-memory byte offset of chunk c8 (0..7) of shared-memory row `srow` in row block k.
CUTT_HD uint32_t t2d_smem_offset(const T2dDesc& D, uint32_t k, uint32_t srow, uint32_t c8) {
  return k * (D.rowsAlloc * 128u) + srow * 128u + ((c8 ^ (srow & 7u)) << 4);
}

CUTT_HD uint32_t t2d_load_units(const T2dDesc& D) {
  const uint32_t perRow = 128u / (D.loadMode == 1u ? 16u : D.loadMode);
  return D.nboxes * D.rowsLoad * perRow;
}

// Row block k, tile row q (may be negative: rows above the tile) and unit-in-row of load unit u.
CUTT_HD void t2d_unit_decode(const T2dDesc& D, uint32_t u, uint32_t upr, uint32_t& k, int32_t& q, uint32_t& x) {
  x = u & (upr - 1u);
  const uint32_t rr = u / upr;
  k = fdiv(rr, D.divRows);
  q = (int32_t)(rr - k * D.rowsLoad) - (int32_t)(D.rowsLoad - D.tb);
}

// cp.async load unit: WIB bytes (16, 8 or 4) of one tile row; rows and buffer aligned to WIB.
template <int ELT, int WIB>
CUTT_HD void t2d_load_unit(const T2dDesc& D, const T2dTile& t, sptr_t stage, const unsigned char* gin, uint32_t u) {
  constexpr uint32_t UPR = 128u / WIB;
  uint32_t k, x;
  int32_t q;
  t2d_unit_decode(D, u, UPR, k, q, x);
  const uint32_t e0 = k * (128u / ELT) + x * (WIB / ELT);
  const int64_t pos = (int64_t)t.cp + q;
  if (t.c0 + e0 >= D.d0 || pos < 0 || pos >= (int64_t)D.dp) return;   // (extents are multiples of the access width)
  const unsigned char* g = gin + (t.inOff + (int64_t)e0 + (int64_t)q * D.isP) * ELT;
  const uint32_t byteInRow = x * WIB;
  copy_g2s<WIB>(stage + t2d_smem_offset(D, k, (uint32_t)(q + (int32_t)D.padTop), byteInRow >> 4) + (byteInRow & 15u), g);
}

// The cp.async load phase of one thread: a thread keeps its place along dimension 0 and walks down
// the rows of the tile, so everything but one pointer addition and the swizzled shared-memory offset
// is computed once.
template <int ELT, int WIB>
CUTT_HD void t2d_load_rows(const T2dDesc& D, const T2dTile& t, sptr_t stage, const unsigned char* gin, uint32_t tid) {
  constexpr uint32_t UPC = 16u / WIB;                   // units per 16-byte chunk
  const uint32_t ux = tid & ((1u << D.uprShift) - 1u);  // unit along the tile row
  const uint32_t ry = tid >> D.uprShift;                // first row of this thread
  const uint32_t rstep = D.nthreads >> D.uprShift;      // rows per pass (a power of two)
  const uint32_t e0 = ux * (WIB / ELT);
  if (t.c0 + e0 >= D.d0) return;                        // (extents are multiples of the access width)
  const uint32_t chunk = ux / UPC;
  const uint32_t c8 = chunk & 7u;
  const uint32_t sbase = (chunk >> 3) * (D.rowsAlloc * 128u) + (ux & (UPC - 1u)) * WIB;
  const uint32_t pad = D.rowsLoad - D.tb;               // rows loaded above the tile
  // rows whose position cp + rl - pad lies inside [0, dp)
  const uint32_t rlo = t.cp >= pad ? 0u : pad - t.cp;
  uint32_t rhi = D.dp - t.cp + pad;
  if (rhi > D.rowsLoad) rhi = D.rowsLoad;
  uint32_t rl = ry;
  while (rl < rlo) rl += rstep;
  const unsigned char* g = gin + (t.inOff + (int64_t)e0 + ((int64_t)rl - (int64_t)pad) * D.isP) * ELT;
  const int64_t gstep = (int64_t)rstep * D.isP * ELT;
  const uint32_t sdelta = D.padTop - pad;
  for (; rl < rhi; rl += rstep, g += gstep) {
    const uint32_t srow = rl + sdelta;
    copy_g2s<WIB>(stage + sbase + srow * 128u + ((c8 ^ (srow & 7u)) << 4), g);
  }
}

// global -> registers / registers -> shared, 16 bytes (plain loads and stores; range-checked on the host)
CUTT_HD void t2d_ldg16(uint32_t* dst, const unsigned char* g) {
#if defined(__CUDA_ARCH__)
  const uint4 v = *reinterpret_cast<const uint4*>(g);
  dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
#else
  CUTT_CHECK_RANGE(g, 16, host_bounds().gin0, host_bounds().gin1);
  memcpy(dst, g, 16);
#endif
}
template <int ELT>
CUTT_HD void t2d_ldg_elem(uint32_t* dst, const unsigned char* g) {
#if defined(__CUDA_ARCH__)
  if (ELT == 4) dst[0] = *reinterpret_cast<const uint32_t*>(g);
  else { const uint2 v = *reinterpret_cast<const uint2*>(g); dst[0] = v.x; dst[1] = v.y; }
#else
  CUTT_CHECK_RANGE(g, ELT, host_bounds().gin0, host_bounds().gin1);
  memcpy(dst, g, ELT);
#endif
}
CUTT_HD void t2d_sts16(sptr_t s, const uint32_t* w) {
#if defined(__CUDA_ARCH__)
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};\n" ::"r"(s), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
#else
  CUTT_CHECK_RANGE(s, 16, host_bounds().s0, host_bounds().s1);
  memcpy(s, w, 16);
#endif
}

// "Shift" load unit: one 16-byte chunk of the tile, cut out of the two aligned vectors that cover it.
// In two steps, so that a thread can have the global loads of several units in flight before it
// needs the data of the first: fetch (global -> registers; returns false if the unit lies outside
// the tensor) and commit (cut the chunk out, registers -> shared).
template <int ELT>
CUTT_HD bool t2d_shift_fetch(const T2dDesc& D, const T2dTile& t, const unsigned char* gin, uint32_t u, uint32_t* w,
                             uint32_t& m, uint32_t& soff) {
  constexpr int VE = 16 / ELT;
  constexpr int EW = ELT / 4;
  uint32_t k, c8;
  int32_t q;
  t2d_unit_decode(D, u, 8u, k, q, c8);
  const uint32_t e0 = k * (128u / ELT) + c8 * (uint32_t)VE;
  const int64_t pos = (int64_t)t.cp + q;
  if (t.c0 + e0 >= D.d0 || pos < 0 || pos >= (int64_t)D.dp) return false;
  const int64_t ge = t.inOff + (int64_t)e0 + (int64_t)q * D.isP;   // first element of the chunk in the buffer
  m = (uint32_t)((ge + (int64_t)D.inMis) & (int64_t)(VE - 1));
  soff = t2d_smem_offset(D, k, (uint32_t)(q + (int32_t)D.padTop), c8);
  const int64_t gl = ge - (int64_t)m;                              // first element of the aligned vector below it
#pragma unroll
  for (int i = 0; i < 8; i++) w[i] = 0u;
  if (gl >= 0 && gl + 2 * VE <= D.inElems) {
    t2d_ldg16(w, gin + gl * ELT);
    if (m) t2d_ldg16(w + 4, gin + (gl + VE) * ELT);
  } else {
    // first or last vector of the buffer: the chunk's own elements, one by one, placed where the
    // aligned loads would have put them
#pragma unroll
    for (int e = 0; e < 2 * VE; e++) {
      const int64_t idx = gl + e;
      if (e >= (int)m && e < (int)m + VE && idx >= 0 && idx < D.inElems) t2d_ldg_elem<ELT>(w + e * EW, gin + idx * ELT);
    }
  }
  return true;
}

template <int ELT>
CUTT_HD void t2d_shift_commit(sptr_t sdst, const uint32_t* w, uint32_t m) {
  uint32_t o[4];
  if (ELT == 4) {
    uint32_t s[6];
#pragma unroll
    for (int i = 0; i < 6; i++) s[i] = (m & 2u) ? w[i + 2] : w[i];
#pragma unroll
    for (int i = 0; i < 4; i++) o[i] = (m & 1u) ? s[i + 1] : s[i];
  } else {
#pragma unroll
    for (int i = 0; i < 4; i++) o[i] = m ? w[i + 2] : w[i];
  }
  t2d_sts16(sdst, o);
}

template <int ELT>
CUTT_HD void t2d_load_shift(const T2dDesc& D, const T2dTile& t, sptr_t stage, const unsigned char* gin, uint32_t u) {
  uint32_t w[8], m, soff;
  if (t2d_shift_fetch<ELT>(D, t, gin, u, w, m, soff)) t2d_shift_commit<ELT>(stage + soff, w, m);
}

CUTT_HD uint32_t t2d_store_items(const T2dDesc& D) {
  const uint32_t chunks = D.ta * D.elt / 16u;
  if (D.storeMode == 1u) {
    const uint32_t nv = D.tb / (16u / D.elt) + 1u;        // vectors per output row, one more in the last tile
    return chunks * ((nv + 7u) & ~7u);
  }
  return chunks * (D.tb * D.elt / D.storeMode);
}

// Store item for output rows on WOB-byte boundaries: wo rows x one 16-byte chunk -> V output rows x WOB bytes.
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
  uint32_t x[WO][4];
#pragma unroll
  for (int i = 0; i < WO; i++)
    lds<16>(x[i], stage + t2d_smem_offset(D, chunk >> 3, row0 + (uint32_t)i + D.padTop, chunk & 7u));
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

// The plain store phase of one thread: the lane's chunk and row group are fixed, the warp walks
// over the blocks of 32 items.
template <int ELT, int WOB>
CUTT_HD void t2d_store_rows(const T2dDesc& D, const T2dTile& t, sptr_t stage, unsigned char* gout, uint32_t tid) {
  constexpr uint32_t NC = WOB / 4, NG = 128u / WOB;
  const uint32_t lane = tid & 31u;
  const uint32_t nblocks = ((D.ta * ELT / 16u) / NC) * (D.tb * ELT / 128u);
  for (uint32_t ib = tid >> 5; ib < nblocks; ib += D.nthreads >> 5) t2d_store_item<ELT, WOB>(D, t, stage, gout, ib * 32u + lane);
  (void)NG;
}

// 2-byte elements (the extension entry points): a 16-byte chunk holds 8 elements, i.e. 8 output rows,
// so an item is 8 rows x one chunk: 8 shared vector loads, an 8 x 8 transpose of 16-bit values with
// one byte-permute per output word, 8 global stores of 16 bytes.  The 8 lanes of a quarter warp take
// the 8 chunks of one shared-memory row (conflict free), the 4 quarters take 4 row groups: every
// store instruction writes 8 output rows x 64 contiguous bytes.  Output rows must start on 16-byte
// boundaries (store mode 16).
CUTT_HD uint32_t t2d_pack16(uint32_t a, uint32_t b, bool high) {
#if defined(__CUDA_ARCH__)
  return high ? __byte_perm(a, b, 0x7632) : __byte_perm(a, b, 0x5410);
#else
  return high ? ((a >> 16) | (b & 0xffff0000u)) : ((a & 0xffffu) | (b << 16));
#endif
}

// Lane map 1 for 2-byte elements.  A warp pass covers 4 chunks (half a shared-memory row) x 8 groups
// of 8 rows, so each store instruction writes 4 output rows x 128 contiguous bytes.  The two groups
// met by a quarter warp would read the same banks (their rows agree in the bits the swizzle uses);
// the odd group therefore reads its rows in the order 4,5,6,7,0,1,2,3, which flips swizzle bit 2, and
// un-rotates the four output words with selects before it stores.
CUTT_HD void t2d_store_rows_e2_wide(const T2dDesc& D, const T2dTile& t, sptr_t stage, unsigned char* gout, uint32_t tid) {
  const uint32_t lane = tid & 31u;
  const uint32_t cl = lane & 3u, g = lane >> 2;
  const uint32_t rot = (g & 1u) * 4u;
  const uint32_t nhalf = D.nboxes * 2u;                  // blocks of 4 chunks along dimension 0
  const uint32_t nblocks = nhalf * (D.tb >> 6);          // x blocks of 8 groups x 8 rows
  const int64_t os0B = D.os0 * 2;
  for (uint32_t ib = tid >> 5; ib < nblocks; ib += D.nthreads >> 5) {
    const uint32_t hb = ib & (nhalf - 1u), rb = ib / nhalf;
    const uint32_t k = hb >> 1, c8 = (hb & 1u) * 4u + cl;
    const uint32_t row0 = (rb * 8u + g) * 8u;
    const uint32_t r0 = t.c0 + (k * 8u + c8) * 8u;
    if (r0 >= D.d0 || t.cp + row0 >= D.dp) continue;     // (dp is a multiple of 8: whole vectors)
    uint32_t x[8][4];
#pragma unroll
    for (int i = 0; i < 8; i++)
      lds<16>(x[i], stage + t2d_smem_offset(D, k, row0 + (((uint32_t)i + rot) & 7u) + D.padTop, c8));
    unsigned char* g0 = gout + (t.outOff + (int64_t)((k * 8u + c8) * 8u) * D.os0 + (int64_t)row0) * 2;
#pragma unroll
    for (int j = 0; j < 8; j++) {
      if (r0 + (uint32_t)j < D.d0) {
        uint32_t z[4], y[4];
#pragma unroll
        for (int w = 0; w < 4; w++) z[w] = t2d_pack16(x[2 * w][j >> 1], x[2 * w + 1][j >> 1], (j & 1) != 0);
        // register pair w holds rows 2w + rot, 2w + rot + 1 (mod 8): output word w is pair w ^ 2 for the odd groups
#pragma unroll
        for (int w = 0; w < 4; w++) y[w] = rot ? z[w ^ 2] : z[w];
        stg<16>(g0, y);
      }
      g0 += os0B;
    }
  }
}

// 2-byte elements whose output rows start on 8-byte boundaries only (store mode 8): an item is one chunk
// (8 output rows) x 4 rows, written with 8-byte stores.  A warp pass covers 2 chunks x 16 groups of 4
// rows, so each store instruction still writes 128 contiguous bytes per output row.  The four groups
// met by a quarter warp lie 4 rows apart; groups 2 and 3 would repeat the swizzle bits of groups 0 and
// 1, so they read their rows in the order 2,3,0,1 (which flips swizzle bit 1) and swap the two
// output words back.
CUTT_HD void t2d_store_rows_e2_w8(const T2dDesc& D, const T2dTile& t, sptr_t stage, unsigned char* gout, uint32_t tid) {
  const uint32_t lane = tid & 31u;
  const uint32_t cl = lane & 1u, g = lane >> 1;
  const uint32_t rot = g & 2u;
  const uint32_t npair = D.nboxes * 4u;                  // blocks of 2 chunks along dimension 0
  const uint32_t nblocks = npair * (D.tb >> 6);          // x blocks of 16 groups x 4 rows
  const int64_t os0B = D.os0 * 2;
  for (uint32_t ib = tid >> 5; ib < nblocks; ib += D.nthreads >> 5) {
    const uint32_t pb = ib & (npair - 1u), rb = ib / npair;
    const uint32_t k = pb >> 2, c8 = (pb & 3u) * 2u + cl;
    const uint32_t row0 = (rb * 16u + g) * 4u;
    const uint32_t r0 = t.c0 + (k * 8u + c8) * 8u;
    if (r0 >= D.d0 || t.cp + row0 >= D.dp) continue;     // (dp is a multiple of 4: whole vectors)
    uint32_t x[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
      lds<16>(x[i], stage + t2d_smem_offset(D, k, row0 + (((uint32_t)i + rot) & 3u) + D.padTop, c8));
    unsigned char* g0 = gout + (t.outOff + (int64_t)((k * 8u + c8) * 8u) * D.os0 + (int64_t)row0) * 2;
#pragma unroll
    for (int j = 0; j < 8; j++) {
      if (r0 + (uint32_t)j < D.d0) {
        const uint32_t z0 = t2d_pack16(x[0][j >> 1], x[1][j >> 1], (j & 1) != 0);
        const uint32_t z1 = t2d_pack16(x[2][j >> 1], x[3][j >> 1], (j & 1) != 0);
        uint32_t y[2];
        y[0] = rot ? z1 : z0;
        y[1] = rot ? z0 : z1;
        stg<8>(g0, y);
      }
      g0 += os0B;
    }
  }
}

CUTT_HD void t2d_store_rows_e2(const T2dDesc& D, const T2dTile& t, sptr_t stage, unsigned char* gout, uint32_t tid) {
  if (D.storeMode == 8u) { t2d_store_rows_e2_w8(D, t, stage, gout, tid); return; }
  if (D.laneMap == 1u) { t2d_store_rows_e2_wide(D, t, stage, gout, tid); return; }
  const uint32_t lane = tid & 31u;
  const uint32_t cl = lane & 7u, g = lane >> 3;
  const uint32_t gblocks = D.tb >> 5;                    // blocks of 4 groups x 8 rows
  const uint32_t nblocks = D.nboxes * gblocks;
  const int64_t os0B = D.os0 * 2;
  for (uint32_t ib = tid >> 5; ib < nblocks; ib += D.nthreads >> 5) {
    const uint32_t cb = ib & (D.nboxes - 1u);            // (nboxes is 1 or 2)
    const uint32_t gb = ib / D.nboxes;
    const uint32_t chunk = cb * 8u + cl;
    const uint32_t row0 = (gb * 4u + g) * 8u;
    const uint32_t r0 = t.c0 + chunk * 8u;
    if (r0 >= D.d0 || t.cp + row0 >= D.dp) continue;     // (dp is a multiple of 8: whole vectors)
    uint32_t x[8][4];
#pragma unroll
    for (int i = 0; i < 8; i++) lds<16>(x[i], stage + t2d_smem_offset(D, cb, row0 + (uint32_t)i + D.padTop, cl));
    unsigned char* g0 = gout + (t.outOff + (int64_t)(chunk * 8u) * D.os0 + (int64_t)row0) * 2;
#pragma unroll
    for (int j = 0; j < 8; j++) {
      if (r0 + (uint32_t)j < D.d0) {
        uint32_t y[4];
#pragma unroll
        for (int w = 0; w < 4; w++) y[w] = t2d_pack16(x[2 * w][j >> 1], x[2 * w + 1][j >> 1], (j & 1) != 0);
        stg<16>(g0, y);
      }
      g0 += os0B;
    }
  }
}

// 1-byte elements: a chunk holds 16 elements, i.e. 16 output rows, so an item is 16 rows x one chunk:
// 16 shared vector loads, a 16 x 16 transpose of bytes (sixteen 4 x 4 blocks, eight byte-permutes
// each), 16 global stores of 16 bytes.  Lanes as for 2-byte elements: the quarter warp takes the 8
// chunks of one shared-memory row, the 4 quarters take 4 groups of 16 rows.
CUTT_HD uint32_t t2d_prmt(uint32_t a, uint32_t b, uint32_t sel) {
#if defined(__CUDA_ARCH__)
  return __byte_perm(a, b, sel);
#else
  const uint64_t v = ((uint64_t)b << 32) | a;
  uint32_t r = 0;
  for (int i = 0; i < 4; i++) r |= (uint32_t)((v >> (8u * ((sel >> (4 * i)) & 7u))) & 0xffu) << (8 * i);
  return r;
#endif
}

// Lane map 1 for 1-byte elements: 4 chunks x 8 groups of 16 rows per warp pass (128 rows); the odd
// groups read their rows in the order 4..15,0..3 and un-rotate the four output words.
CUTT_HD void t2d_store_rows_e1_wide(const T2dDesc& D, const T2dTile& t, sptr_t stage, unsigned char* gout, uint32_t tid) {
  const uint32_t lane = tid & 31u;
  const uint32_t cl = lane & 3u, g = lane >> 2;
  const uint32_t rot = (g & 1u) * 4u;
  const uint32_t nhalf = D.nboxes * 2u;
  const uint32_t nblocks = nhalf * (D.tb >> 7);          // x blocks of 8 groups x 16 rows
  for (uint32_t ib = tid >> 5; ib < nblocks; ib += D.nthreads >> 5) {
    const uint32_t hb = ib & (nhalf - 1u), rb = ib / nhalf;
    const uint32_t k = hb >> 1, c8 = (hb & 1u) * 4u + cl;
    const uint32_t row0 = (rb * 8u + g) * 16u;
    const uint32_t r0 = t.c0 + (k * 8u + c8) * 16u;
    if (r0 >= D.d0 || t.cp + row0 >= D.dp) continue;     // (dp is a multiple of 16: whole vectors)
    uint32_t x[16][4];
#pragma unroll
    for (int i = 0; i < 16; i++)
      lds<16>(x[i], stage + t2d_smem_offset(D, k, row0 + (((uint32_t)i + rot) & 15u) + D.padTop, c8));
    unsigned char* g0 = gout + (t.outOff + (int64_t)((k * 8u + c8) * 16u) * D.os0 + (int64_t)row0);
#pragma unroll
    for (int jw = 0; jw < 4; jw++) {
      uint32_t o[4][4];
#pragma unroll
      for (int w = 0; w < 4; w++) {
        const uint32_t a = x[4 * w][jw], b = x[4 * w + 1][jw], c = x[4 * w + 2][jw], d = x[4 * w + 3][jw];
        const uint32_t ab01 = t2d_prmt(a, b, 0x5140), cd01 = t2d_prmt(c, d, 0x5140);
        const uint32_t ab23 = t2d_prmt(a, b, 0x7362), cd23 = t2d_prmt(c, d, 0x7362);
        o[0][w] = t2d_prmt(ab01, cd01, 0x5410);
        o[1][w] = t2d_prmt(ab01, cd01, 0x7632);
        o[2][w] = t2d_prmt(ab23, cd23, 0x5410);
        o[3][w] = t2d_prmt(ab23, cd23, 0x7632);
      }
#pragma unroll
      for (int jj = 0; jj < 4; jj++) {
        if (r0 + (uint32_t)(jw * 4 + jj) < D.d0) {
          // register quad w holds rows 4w + rot .. (mod 16): output word w is quad w - 1 for the odd groups
          uint32_t y[4];
#pragma unroll
          for (int w = 0; w < 4; w++) y[w] = rot ? o[jj][(w + 3) & 3] : o[jj][w];
          stg<16>(g0, y);
        }
        g0 += D.os0;
      }
    }
  }
}

// 1-byte elements whose output rows start on 8-byte boundaries only (store mode 8): an item is one chunk
// (16 output rows) x 8 rows, written with 8-byte stores; 4 chunks x 8 groups of 8 rows per warp pass (a
// store instruction writes 64 contiguous bytes per output row); the odd groups read their rows in the
// order 4..7,0..3 and swap the two output words back.
CUTT_HD void t2d_store_rows_e1_w8(const T2dDesc& D, const T2dTile& t, sptr_t stage, unsigned char* gout, uint32_t tid) {
  const uint32_t lane = tid & 31u;
  const uint32_t cl = lane & 3u, g = lane >> 2;
  const uint32_t rot = (g & 1u) * 4u;
  const uint32_t nhalf = D.nboxes * 2u;
  const uint32_t nblocks = nhalf * (D.tb >> 6);          // x blocks of 8 groups x 8 rows
  for (uint32_t ib = tid >> 5; ib < nblocks; ib += D.nthreads >> 5) {
    const uint32_t hb = ib & (nhalf - 1u), rb = ib / nhalf;
    const uint32_t k = hb >> 1, c8 = (hb & 1u) * 4u + cl;
    const uint32_t row0 = (rb * 8u + g) * 8u;
    const uint32_t r0 = t.c0 + (k * 8u + c8) * 16u;
    if (r0 >= D.d0 || t.cp + row0 >= D.dp) continue;     // (dp is a multiple of 8: whole vectors)
    uint32_t x[8][4];
#pragma unroll
    for (int i = 0; i < 8; i++)
      lds<16>(x[i], stage + t2d_smem_offset(D, k, row0 + (((uint32_t)i + rot) & 7u) + D.padTop, c8));
    unsigned char* g0 = gout + (t.outOff + (int64_t)((k * 8u + c8) * 16u) * D.os0 + (int64_t)row0);
#pragma unroll
    for (int jw = 0; jw < 4; jw++) {
      uint32_t o[4][2];
#pragma unroll
      for (int w = 0; w < 2; w++) {
        const uint32_t a = x[4 * w][jw], b = x[4 * w + 1][jw], c = x[4 * w + 2][jw], d = x[4 * w + 3][jw];
        const uint32_t ab01 = t2d_prmt(a, b, 0x5140), cd01 = t2d_prmt(c, d, 0x5140);
        const uint32_t ab23 = t2d_prmt(a, b, 0x7362), cd23 = t2d_prmt(c, d, 0x7362);
        o[0][w] = t2d_prmt(ab01, cd01, 0x5410);
        o[1][w] = t2d_prmt(ab01, cd01, 0x7632);
        o[2][w] = t2d_prmt(ab23, cd23, 0x5410);
        o[3][w] = t2d_prmt(ab23, cd23, 0x7632);
      }
#pragma unroll
      for (int jj = 0; jj < 4; jj++) {
        if (r0 + (uint32_t)(jw * 4 + jj) < D.d0) {
          uint32_t y[2];
          y[0] = rot ? o[jj][1] : o[jj][0];
          y[1] = rot ? o[jj][0] : o[jj][1];
          stg<8>(g0, y);
        }
        g0 += D.os0;
      }
    }
  }
}

CUTT_HD void t2d_store_rows_e1(const T2dDesc& D, const T2dTile& t, sptr_t stage, unsigned char* gout, uint32_t tid) {
  if (D.storeMode == 8u) { t2d_store_rows_e1_w8(D, t, stage, gout, tid); return; }
  if (D.laneMap == 1u) { t2d_store_rows_e1_wide(D, t, stage, gout, tid); return; }
  const uint32_t lane = tid & 31u;
  const uint32_t cl = lane & 7u, g = lane >> 3;
  const uint32_t gblocks = D.tb >> 6;                    // blocks of 4 groups x 16 rows
  const uint32_t nblocks = D.nboxes * gblocks;
  for (uint32_t ib = tid >> 5; ib < nblocks; ib += D.nthreads >> 5) {
    const uint32_t cb = ib & (D.nboxes - 1u);            // (nboxes is 1 or 2)
    const uint32_t gb = ib / D.nboxes;
    const uint32_t chunk = cb * 8u + cl;
    const uint32_t row0 = (gb * 4u + g) * 16u;
    const uint32_t r0 = t.c0 + chunk * 16u;
    if (r0 >= D.d0 || t.cp + row0 >= D.dp) continue;     // (dp is a multiple of 16: whole vectors)
    uint32_t x[16][4];
#pragma unroll
    for (int i = 0; i < 16; i++) lds<16>(x[i], stage + t2d_smem_offset(D, cb, row0 + (uint32_t)i + D.padTop, cl));
    unsigned char* g0 = gout + (t.outOff + (int64_t)(chunk * 16u) * D.os0 + (int64_t)row0);
#pragma unroll
    for (int jw = 0; jw < 4; jw++) {        // word jw of the chunk: output rows 4 jw .. 4 jw + 3
      uint32_t o[4][4];
#pragma unroll
      for (int w = 0; w < 4; w++) {         // rows 4 w .. 4 w + 3 of the item: one 4 x 4 block of bytes
        const uint32_t a = x[4 * w][jw], b = x[4 * w + 1][jw], c = x[4 * w + 2][jw], d = x[4 * w + 3][jw];
        const uint32_t ab01 = t2d_prmt(a, b, 0x5140), cd01 = t2d_prmt(c, d, 0x5140);
        const uint32_t ab23 = t2d_prmt(a, b, 0x7362), cd23 = t2d_prmt(c, d, 0x7362);
        o[0][w] = t2d_prmt(ab01, cd01, 0x5410);
        o[1][w] = t2d_prmt(ab01, cd01, 0x7632);
        o[2][w] = t2d_prmt(ab23, cd23, 0x5410);
        o[3][w] = t2d_prmt(ab23, cd23, 0x7632);
      }
#pragma unroll
      for (int jj = 0; jj < 4; jj++) {
        if (r0 + (uint32_t)(jw * 4 + jj) < D.d0) stg<16>(g0, o[jj]);
        g0 += D.os0;
      }
    }
  }
}

// One output row of a sheared item whose misalignment is MO elements: the aligned vector holds the
// elements of shared rows (V-1) - MO + i, i < V.  pos0: position along p of its first element.
template <int ELT, int MO>
CUTT_HD void t2d_shear_row(const uint32_t (*x)[4], int j, unsigned char* g, int64_t pos0, int64_t dp) {
  constexpr int VE = 16 / ELT;
  constexpr int EW = ELT / 4;
  uint32_t y[4];
#pragma unroll
  for (int i = 0; i < VE; i++) {
#pragma unroll
    for (int w = 0; w < EW; w++) y[i * EW + w] = x[(VE - 1) - MO + i][j * EW + w];
  }
  if (pos0 >= 0 && pos0 + VE <= dp) {
    stg<16>(g, y);
  } else {   // first or last vector of an output row: only the elements inside it
#pragma unroll
    for (int i = 0; i < VE; i++)
      if (pos0 + i >= 0 && pos0 + i < dp) stg<ELT>(g + i * ELT, y + i * EW);
  }
}

// "Shear" store item: one chunk (V output rows) x one aligned vector per output row.
template <int ELT>
CUTT_HD void t2d_store_shear(const T2dDesc& D, const T2dTile& t, sptr_t stage, unsigned char* gout, uint32_t it) {
  constexpr int VE = 16 / ELT;
  constexpr int NR = 2 * VE - 1;         // shared-memory rows an item reads
  const uint32_t cl = it & 3u;
  uint32_t g = (it >> 2) & 7u;
  const uint32_t rest = it >> 5;
  const uint32_t cblocks = (D.ta * ELT / 16u) / 4u;
  const uint32_t cb = rest & (cblocks - 1u);
  const uint32_t gb = rest / cblocks;
  if (ELT == 8) g = ((g << 1) & 6u) | ((g >> 2) & 1u);   // (see t2d_store_item)
  const uint32_t chunk = cb * 4u + cl;
  const uint32_t kv = gb * 8u + g;                       // vector index along p within the sheared tile
  const uint32_t nvFull = D.tb / (uint32_t)VE;
  const bool lastTile = t.cp + D.tb >= D.dp;
  if (kv > nvFull || (kv == nvFull && !lastTile)) return;
  const uint32_t r0 = t.c0 + chunk * (uint32_t)VE;
  if (r0 >= D.d0) return;
  const int32_t qb = (int32_t)(kv * (uint32_t)VE) - (VE - 1);   // tile row held by x[0]
  if ((int64_t)t.cp + qb >= (int64_t)D.dp) return;
  uint32_t x[NR][4];
#pragma unroll
  for (int r = 0; r < NR; r++)
    lds<16>(x[r], stage + t2d_smem_offset(D, chunk >> 3, (uint32_t)(qb + r + (int32_t)D.padTop), chunk & 7u));
#pragma unroll
  for (int j = 0; j < VE; j++) {
    if (r0 + (uint32_t)j >= D.d0) continue;
    const int64_t rowOff = t.outOff + (int64_t)(chunk * (uint32_t)VE + (uint32_t)j) * D.os0;   // element (c, cp)
    const uint32_t mo = (uint32_t)((rowOff + (int64_t)D.outMis) & (int64_t)(VE - 1));
    const int64_t pos0 = (int64_t)t.cp + (int64_t)(kv * (uint32_t)VE) - (int64_t)mo;
    if (pos0 >= (int64_t)D.dp) continue;
    if (kv == nvFull && mo == 0u) continue;
    unsigned char* gp = gout + (rowOff + (int64_t)(kv * (uint32_t)VE) - (int64_t)mo) * ELT;
    // (mo is the same for every lane of the warp: no divergence)
    if (mo == 0u) t2d_shear_row<ELT, 0>(x, j, gp, pos0, (int64_t)D.dp);
    else if (mo == 1u) t2d_shear_row<ELT, 1>(x, j, gp, pos0, (int64_t)D.dp);
    else if (ELT == 4 && mo == 2u) t2d_shear_row<ELT, (ELT == 4 ? 2 : 0)>(x, j, gp, pos0, (int64_t)D.dp);
    else if (ELT == 4) t2d_shear_row<ELT, (ELT == 4 ? 3 : 0)>(x, j, gp, pos0, (int64_t)D.dp);
  }
}

}  // namespace cuttb
