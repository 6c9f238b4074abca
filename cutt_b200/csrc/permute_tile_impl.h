// Per-thread phases of the tiled permutation kernel.  The same functions run on the
// device (inside permute_tiles_kernel, one call per thread) and on the host (inside
// the plan interpreter that the CPU tests use to check descriptors without a GPU):
// only the copy primitives differ.
//
// Phase "load":  global input  -> shared tile (contiguous runs, shared memory in input order)
// Phase "store": shared tile   -> global output (contiguous runs of the output, gathered
//                from shared memory through the output run's offset table, V x W blocks
//                transposed in registers)
//
// Role in the reference: these two phases are what transposePacked / transposePackedSplit /
// transposeTiled / transposeTiledCopy (src/cuttkernel.cu:38-426) do between their two
// __syncthreads, generalised to one code path with explicit strides.
#pragma once
#include "permute_desc.h"
#include <string.h>

namespace cuttb {

// Shared-memory address: a 32-bit shared-window address on the device, a pointer on the host.
#if defined(__CUDA_ARCH__)
typedef uint32_t sptr_t;
#else
typedef unsigned char* sptr_t;
#endif

// Host-side interpreter only: address ranges that every access is checked against.
#if !defined(__CUDA_ARCH__) && defined(CUTT_HOSTCHECK_BOUNDS)
struct HostBounds {
  const unsigned char *gin0, *gin1, *gout0, *gout1, *s0, *s1;
  long long violations;
};
inline HostBounds& host_bounds() { static thread_local HostBounds b = {}; return b; }
#define CUTT_CHECK_RANGE(p, n, lo, hi) \
  do { if ((const unsigned char*)(p) < (lo) || (const unsigned char*)(p) + (n) > (hi) || ((uintptr_t)(p) % (n)) != 0) { host_bounds().violations++; return; } } while (0)
#else
#define CUTT_CHECK_RANGE(p, n, lo, hi) do { } while (0)
#endif

// global -> shared, BYTES in {4, 8, 16}; asynchronous on the device.
template <int BYTES>
CUTT_HD void copy_g2s(sptr_t sdst, const unsigned char* gsrc) {
#if defined(__CUDA_ARCH__)
  if (BYTES == 16) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(sdst), "l"(gsrc) : "memory");
  } else {
    asm volatile("cp.async.ca.shared.global [%0], [%1], %2;\n" ::"r"(sdst), "l"(gsrc), "n"(BYTES) : "memory");
  }
#else
  CUTT_CHECK_RANGE(gsrc, BYTES, host_bounds().gin0, host_bounds().gin1);
  CUTT_CHECK_RANGE(sdst, BYTES, host_bounds().s0, host_bounds().s1);
  memcpy(sdst, gsrc, BYTES);
#endif
}

// shared -> registers: BYTES/4 32-bit words
template <int BYTES>
CUTT_HD void lds(uint32_t* dst, sptr_t ssrc) {
#if defined(__CUDA_ARCH__)
  if (BYTES == 4) {
    asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(dst[0]) : "r"(ssrc));
  } else if (BYTES == 8) {
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];\n" : "=r"(dst[0]), "=r"(dst[1]) : "r"(ssrc));
  } else {
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];\n"
                 : "=r"(dst[0]), "=r"(dst[1]), "=r"(dst[2]), "=r"(dst[3]) : "r"(ssrc));
  }
#else
  CUTT_CHECK_RANGE(ssrc, BYTES, host_bounds().s0, host_bounds().s1);
  memcpy(dst, ssrc, BYTES);
#endif
}

// registers -> global
template <int BYTES>
CUTT_HD void stg(unsigned char* gdst, const uint32_t* src) {
#if defined(__CUDA_ARCH__)
  if (BYTES == 4) *reinterpret_cast<uint32_t*>(gdst) = src[0];
  else if (BYTES == 8) *reinterpret_cast<uint2*>(gdst) = make_uint2(src[0], src[1]);
  else *reinterpret_cast<uint4*>(gdst) = make_uint4(src[0], src[1], src[2], src[3]);
#else
  CUTT_CHECK_RANGE(gdst, BYTES, host_bounds().gout0, host_bounds().gout1);
  memcpy(gdst, src, BYTES);
#endif
}

// Pointers to the shared-memory tables (computed once per thread block).
template <bool WIDE>
struct Tables {
  typedef typename RowEntSel<WIDE>::type Ent;
  const Ent* tabIn;
  const Ent* tabOut;
  const RowCoord* coIn;
  const RowCoord* coOut;
  const uint32_t* qtab;
};

template <bool WIDE>
CUTT_HD Tables<WIDE> make_tables(const TileDesc& D, const unsigned char* tables) {
  typedef typename RowEntSel<WIDE>::type Ent;
  const TableLayout L = table_layout(D);
  Tables<WIDE> T;
  T.tabIn = reinterpret_cast<const Ent*>(tables + L.tabIn);
  T.tabOut = reinterpret_cast<const Ent*>(tables + L.tabOut);
  T.coIn = reinterpret_cast<const RowCoord*>(tables + L.coordIn);
  T.coOut = reinterpret_cast<const RowCoord*>(tables + L.coordOut);
  T.qtab = reinterpret_cast<const uint32_t*>(tables + L.qtab);
  return T;
}

// Rows of a side with at most one row dimension need no table: offsets are multiples of
// the row index and a short tile simply has fewer rows.
CUTT_HD uint32_t single_dim_rows(const Side& S, const TileCtx& c) {
  uint32_t nr = S.nrows;
  if (S.nRowDims == 1 && S.rowDim[0].slot >= 0) {
    const uint32_t rem = S.rowDim[0].slot == 0 ? c.rem0 : c.rem1;
    if (rem != 0xffffffffu) {
      const uint32_t cm = S.rowDim[0].cmul;
      const uint32_t v = (rem + cm - 1) / cm;
      nr = v < nr ? v : nr;
    }
  }
  return nr;
}

template <int ELT, int W, bool WIDE, bool PARTIAL>
CUTT_HD void tile_load_impl(const TileDesc& D, const TileCtx& c, const Tables<WIDE>& T,
                            sptr_t sbuf, const unsigned char* gin, uint32_t tid) {
  typedef typename RowEntSel<WIDE>::type Ent;
  const Side& S = D.in;
  const uint32_t tq = tid & (S.tq - 1);
  const uint32_t tr = tid >> S.tqShift;
  const uint32_t Tr = D.nthreads >> S.tqShift;
  const uint32_t valid = PARTIAL ? run_valid(S, c) : S.run;
  const uint32_t q0 = tq * W;
  if (q0 >= valid) return;
  const uint32_t qstep = S.tq * W;
  const uint32_t qstepB = qstep * ELT;
  const unsigned char* gbase = gin + (c.inOff + q0) * ELT;
  const sptr_t sbase = sbuf + q0 * ELT;
  if (S.nRowDims <= 1) {
    const RowDim& R = S.rowDim[0];
    const uint32_t nr = PARTIAL ? single_dim_rows(S, c) : S.nrows;
    const int64_t gstepB = S.nRowDims ? R.gstride * (int64_t)(Tr * ELT) : 0;
    const unsigned char* g0 = gbase + (S.nRowDims ? R.gstride * (int64_t)(tr * ELT) : 0);
    const bool skewed = S.nRowDims && R.skew.mask != 0;
#pragma unroll 4
    for (uint32_t row = tr; row < nr; row += Tr) {
      sptr_t s = sbase + row * R.sstrideB;
      if (skewed) s += skew_bytes(R.skew, row);
      const unsigned char* g = g0;
      copy_g2s<ELT * W>(s, g);
      for (uint32_t q = q0 + qstep; q < valid; q += qstep) {
        g += qstepB;
        s += qstepB;
        copy_g2s<ELT * W>(s, g);
      }
      g0 += gstepB;
    }
    return;
  }
  for (uint32_t row = tr; row < S.nrows; row += Tr) {
    if (PARTIAL) {
      const RowCoord rc = T.coIn[row];
      if (!(rc.c0 < c.rem0 && rc.c1 < c.rem1)) continue;
    }
    const Ent e = T.tabIn[row];
    const unsigned char* g = gbase + (WIDE ? (int64_t)e.goff * ELT : (int64_t)((uint64_t)(uint32_t)e.goff * ELT));
    sptr_t s = sbase + e.soffB;
    copy_g2s<ELT * W>(s, g);
    for (uint32_t q = q0 + qstep; q < valid; q += qstep) {
      g += qstepB;
      s += qstepB;
      copy_g2s<ELT * W>(s, g);
    }
  }
}

// Aligned over-fetch load of one input row (see permute_desc.h): 16-byte copies from the
// aligned range that encloses the row; at the ends of the buffer element copies of the row's
// own elements only.
template <int ELT>
CUTT_HD void aof_row(sptr_t srow, const unsigned char* grow, uint32_t valid, uint32_t tq, uint32_t Tq,
                     const unsigned char* lo, const unsigned char* hi) {
  constexpr uint32_t VE = 16 / ELT;
  const uint32_t sh = (uint32_t)(((uintptr_t)grow / ELT) & (VE - 1));
  const unsigned char* gal = grow - sh * ELT;
  const uint32_t nvec = (sh + valid + VE - 1) / VE;
  if (gal >= lo && gal + 16u * (size_t)nvec <= hi) {
    // the whole aligned range lies inside the buffer (every row but the first and last few)
    for (uint32_t v = tq; v < nvec; v += Tq) copy_g2s<16>(srow + 16u * v, gal + 16u * (size_t)v);
    return;
  }
  for (uint32_t v = tq; v < nvec; v += Tq) {
    const unsigned char* src = gal + 16u * v;
    if (src >= lo && src + 16 <= hi) {
      copy_g2s<16>(srow + 16u * v, src);
    } else {
      for (uint32_t e = 0; e < VE; e++) {
        const uint32_t pos = v * VE + e;  // position relative to the aligned start
        if (pos >= sh && pos < sh + valid) copy_g2s<ELT>(srow + pos * ELT, gal + (size_t)pos * ELT);
      }
    }
  }
}

template <int ELT, bool WIDE, bool PARTIAL>
CUTT_HD void tile_load_aof(const TileDesc& D, const TileCtx& c, const Tables<WIDE>& T,
                           sptr_t sbuf, const unsigned char* gin, uint32_t tid) {
  typedef typename RowEntSel<WIDE>::type Ent;
  const Side& S = D.in;
  const uint32_t tq = tid & (S.tq - 1);
  const uint32_t tr = tid >> S.tqShift;
  const uint32_t Tr = D.nthreads >> S.tqShift;
  const uint32_t valid = PARTIAL ? run_valid(S, c) : S.run;
  const unsigned char* lo = gin;
  const unsigned char* hi = gin + D.inElems * ELT;
  const unsigned char* gbase = gin + c.inOff * ELT;
  if (S.nRowDims <= 1) {
    const RowDim& R = S.rowDim[0];
    const uint32_t nr = PARTIAL ? single_dim_rows(S, c) : S.nrows;
    const int64_t gstepB = S.nRowDims ? R.gstride * (int64_t)(Tr * ELT) : 0;
    const unsigned char* g0 = gbase + (S.nRowDims ? R.gstride * (int64_t)(tr * ELT) : 0);
    const bool skewed = S.nRowDims && R.skew.mask != 0;
    // Strides are positive, so rows 0 and nr-1 bound the tile: when both lie inside the buffer with
    // a vector to spare on either side, no row of the tile needs the per-row range test.
    const unsigned char* lastRow = gbase + (S.nRowDims && nr ? R.gstride * (int64_t)((nr - 1) * ELT) : 0);
    if ((uintptr_t)gbase >= (uintptr_t)lo + 16 && (uintptr_t)lastRow + (size_t)valid * ELT + 16 <= (uintptr_t)hi) {
      constexpr uint32_t VE = 16 / ELT;
      for (uint32_t row = tr; row < nr; row += Tr) {
        sptr_t s = sbuf + row * R.sstrideB;
        if (skewed) s += skew_bytes(R.skew, row);
        const uint32_t sh = (uint32_t)(((uintptr_t)g0 / ELT) & (VE - 1));
        const unsigned char* gal = g0 - sh * ELT;
        const uint32_t nvec = (sh + valid + VE - 1) / VE;
        for (uint32_t v = tq; v < nvec; v += S.tq) copy_g2s<16>(s + 16u * v, gal + 16u * (size_t)v);
        g0 += gstepB;
      }
      return;
    }
    for (uint32_t row = tr; row < nr; row += Tr) {
      sptr_t s = sbuf + row * R.sstrideB;
      if (skewed) s += skew_bytes(R.skew, row);
      aof_row<ELT>(s, g0, valid, tq, S.tq, lo, hi);
      g0 += gstepB;
    }
    return;
  }
  for (uint32_t row = tr; row < S.nrows; row += Tr) {
    if (PARTIAL) {
      const RowCoord rc = T.coIn[row];
      if (!(rc.c0 < c.rem0 && rc.c1 < c.rem1)) continue;
    }
    const Ent e = T.tabIn[row];
    const unsigned char* g = gbase + (WIDE ? (int64_t)e.goff * ELT : (int64_t)((uint64_t)(uint32_t)e.goff * ELT));
    aof_row<ELT>(sbuf + e.soffB, g, valid, tq, S.tq, lo, hi);
  }
}

// Store side of the aligned over-fetch mode: scalar shared loads at
// base + row offset + position offset + ((A + row residue + position residue) mod VE) * ELT,
// where A is the misalignment of the tile origin and the residues travel in the low two bits
// of the offsets.
template <int ELT, int W, int V, bool WIDE, bool PARTIAL>
CUTT_HD void tile_store_aof(const TileDesc& D, const TileCtx& c, const Tables<WIDE>& T,
                            sptr_t sbuf, const unsigned char* gin, unsigned char* gout, uint32_t tid) {
  typedef typename RowEntSel<WIDE>::type Ent;
  constexpr int EW = ELT / 4;
  constexpr uint32_t VE = 16 / ELT;
  const Side& S = D.out;
  const uint32_t tq = tid & (S.tq - 1);
  const uint32_t tr = tid >> S.tqShift;
  const uint32_t Tr = D.nthreads >> S.tqShift;
  const uint32_t valid = PARTIAL ? run_valid(S, c) : S.run;
  const uint32_t qstep = S.tq * W;
  const uint32_t A = (uint32_t)((((uintptr_t)gin / ELT) + (uint64_t)c.inOff) & (VE - 1));
  const int64_t vstepB = D.vstep * ELT;
  unsigned char* gbase = gout + c.outOff * ELT;
  const bool single = S.nRowDims <= 1;
  const RowDim& R = S.rowDim[0];
  const uint32_t nr = single ? (PARTIAL ? single_dim_rows(S, c) : S.nrows) : S.nrows;
  const int64_t gstepB = (single && S.nRowDims) ? R.gstride * (int64_t)(Tr * ELT) : 0;
  const int64_t g0off = (single && S.nRowDims) ? R.gstride * (int64_t)(tr * ELT) : 0;
  const bool skewed = single && S.nRowDims && R.skew.mask != 0;
  for (uint32_t q = tq * W; q < valid; q += qstep) {
    uint32_t so[W], qr[W];
#pragma unroll
    for (int i = 0; i < W; i++) {
      const uint32_t v = T.qtab[q + i];
      so[i] = v & ~3u;
      qr[i] = A + (v & 3u);
    }
    unsigned char* gq = gbase + (size_t)q * ELT;
    unsigned char* g = gq + g0off;
    if (single && ((Tr * R.ishift) & (VE - 1)) == 0) {
      // the row residue is the same for every row this thread visits: fold it into the
      // position offsets once
      const uint32_t rres0 = tr * R.ishift;
      uint32_t sofs[W];
#pragma unroll
      for (int i = 0; i < W; i++) sofs[i] = so[i] + ((qr[i] + rres0) & (VE - 1)) * ELT;
#pragma unroll 2
      for (uint32_t row = tr; row < nr; row += Tr) {
        uint32_t soff = row * R.sstrideB;
        if (skewed) soff += skew_bytes(R.skew, row);
        uint32_t x[W][V * EW];
#pragma unroll
        for (int i = 0; i < W; i++) lds<ELT * V>(x[i], sbuf + soff + sofs[i]);
        unsigned char* gg = g;
#pragma unroll
        for (int j = 0; j < V; j++) {
          uint32_t y[W * EW];
#pragma unroll
          for (int i = 0; i < W; i++) {
#pragma unroll
            for (int w = 0; w < EW; w++) y[i * EW + w] = x[i][j * EW + w];
          }
          stg<ELT * W>(gg, y);
          gg += vstepB;
        }
        g += gstepB;
      }
      continue;
    }
#pragma unroll 2
    for (uint32_t row = tr; row < nr; row += Tr) {
      uint32_t soff, rres;
      if (single) {
        soff = row * R.sstrideB;
        if (skewed) soff += skew_bytes(R.skew, row);
        rres = row * R.ishift;
      } else {
        if (PARTIAL) {
          const RowCoord rc = T.coOut[row];
          if (!(rc.c0 < c.rem0 && rc.c1 < c.rem1)) continue;
        }
        const Ent e = T.tabOut[row];
        soff = e.soffB & ~3u;
        rres = e.soffB & 3u;
        g = gq + (WIDE ? (int64_t)e.goff * ELT : (int64_t)((uint64_t)(uint32_t)e.goff * ELT));
      }
      // V consecutive elements along dimension 0 stay one aligned shared vector because every
      // displacement is a multiple of V in this mode (the planner guarantees it)
      uint32_t x[W][V * EW];
#pragma unroll
      for (int i = 0; i < W; i++)
        lds<ELT * V>(x[i], sbuf + soff + so[i] + ((qr[i] + rres) & (VE - 1)) * ELT);
      unsigned char* gg = g;
#pragma unroll
      for (int j = 0; j < V; j++) {
        uint32_t y[W * EW];
#pragma unroll
        for (int i = 0; i < W; i++) {
#pragma unroll
          for (int w = 0; w < EW; w++) y[i * EW + w] = x[i][j * EW + w];
        }
        stg<ELT * W>(gg, y);
        gg += vstepB;
      }
      if (single) g += gstepB;
    }
  }
}

// One (row group, run position) item of the store side: W shared-memory vectors of V
// elements in, V global vectors of W elements out.
template <int ELT, int W, int V>
CUTT_HD void store_item(sptr_t sb, const uint32_t* so, bool contig, unsigned char* g, int64_t vstepB) {
  constexpr int EW = ELT / 4;  // 32-bit words per element
  if (contig) {
    uint32_t x[W * EW];
    lds<ELT * W>(x, sb + so[0]);
    stg<ELT * W>(g, x);
  } else {
    uint32_t x[W][V * EW];
#pragma unroll
    for (int i = 0; i < W; i++) lds<ELT * V>(x[i], sb + so[i]);
#pragma unroll
    for (int j = 0; j < V; j++) {
      uint32_t y[W * EW];
#pragma unroll
      for (int i = 0; i < W; i++) {
#pragma unroll
        for (int w = 0; w < EW; w++) y[i * EW + w] = x[i][j * EW + w];
      }
      stg<ELT * W>(g, y);
      g += vstepB;
    }
  }
}

template <int ELT, int W, int V, bool WIDE, bool PARTIAL>
CUTT_HD void tile_store_impl(const TileDesc& D, const TileCtx& c, const Tables<WIDE>& T,
                             sptr_t sbuf, unsigned char* gout, uint32_t tid) {
  typedef typename RowEntSel<WIDE>::type Ent;
  const Side& S = D.out;
  const uint32_t tq = tid & (S.tq - 1);
  const uint32_t tr = tid >> S.tqShift;
  const uint32_t Tr = D.nthreads >> S.tqShift;
  const uint32_t valid = PARTIAL ? run_valid(S, c) : S.run;
  const uint32_t qstep = S.tq * W;
  const bool contig = (W > 1) && (V == 1) && D.smemGatherContig;
  const int64_t vstepB = D.vstep * ELT;
  unsigned char* gbase = gout + c.outOff * ELT;
  const bool single = S.nRowDims <= 1;
  const RowDim& R = S.rowDim[0];
  const uint32_t nr = single ? (PARTIAL ? single_dim_rows(S, c) : S.nrows) : S.nrows;
  const int64_t gstepB = (single && S.nRowDims) ? R.gstride * (int64_t)(Tr * ELT) : 0;
  const int64_t g0off = (single && S.nRowDims) ? R.gstride * (int64_t)(tr * ELT) : 0;
  const bool skewed = single && S.nRowDims && R.skew.mask != 0;
  for (uint32_t q = tq * W; q < valid; q += qstep) {
    uint32_t so[W];
#pragma unroll
    for (int i = 0; i < W; i++) so[i] = T.qtab[q + i];
    unsigned char* gq = gbase + (size_t)q * ELT;
    if (single) {
      unsigned char* g = gq + g0off;
#pragma unroll 2
      for (uint32_t row = tr; row < nr; row += Tr) {
        sptr_t sb = sbuf + row * R.sstrideB;
        if (skewed) sb += skew_bytes(R.skew, row);
        store_item<ELT, W, V>(sb, so, contig, g, vstepB);
        g += gstepB;
      }
    } else {
#pragma unroll 2
      for (uint32_t row = tr; row < nr; row += Tr) {
        if (PARTIAL) {
          const RowCoord rc = T.coOut[row];
          if (!(rc.c0 < c.rem0 && rc.c1 < c.rem1)) continue;
        }
        const Ent e = T.tabOut[row];
        unsigned char* g = gq + (WIDE ? (int64_t)e.goff * ELT : (int64_t)((uint64_t)(uint32_t)e.goff * ELT));
        store_item<ELT, W, V>(sbuf + e.soffB, so, contig, g, vstepB);
      }
    }
  }
}

template <int ELT, int W, bool WIDE, bool AOF>
CUTT_HD void tile_load(const TileDesc& D, const TileCtx& c, const Tables<WIDE>& T,
                       sptr_t sbuf, const unsigned char* gin, uint32_t tid) {
  if (AOF) {
    if (c.partial) tile_load_aof<ELT, WIDE, true>(D, c, T, sbuf, gin, tid);
    else tile_load_aof<ELT, WIDE, false>(D, c, T, sbuf, gin, tid);
  } else {
    if (c.partial) tile_load_impl<ELT, W, WIDE, true>(D, c, T, sbuf, gin, tid);
    else tile_load_impl<ELT, W, WIDE, false>(D, c, T, sbuf, gin, tid);
  }
}

template <int ELT, int W, int V, bool WIDE, bool AOF>
CUTT_HD void tile_store(const TileDesc& D, const TileCtx& c, const Tables<WIDE>& T,
                        sptr_t sbuf, const unsigned char* gin, unsigned char* gout, uint32_t tid) {
  if (AOF) {
    if (c.partial) tile_store_aof<ELT, W, V, WIDE, true>(D, c, T, sbuf, gin, gout, tid);
    else tile_store_aof<ELT, W, V, WIDE, false>(D, c, T, sbuf, gin, gout, tid);
  } else {
    if (c.partial) tile_store_impl<ELT, W, V, WIDE, true>(D, c, T, sbuf, gout, tid);
    else tile_store_impl<ELT, W, V, WIDE, false>(D, c, T, sbuf, gout, tid);
  }
}

}  // namespace cuttb
