// Strided row copy: permutations that keep the fastest dimension (after fusion) are copies of
// contiguous rows between two different row orders.  When the rows start on 16-byte boundaries
// on both sides the tiled kernel already moves them with 16-byte accesses; this path is for rows
// that do NOT (odd row lengths), where it still issues only 16-byte aligned loads and stores:
// for every aligned 16-byte vector of the OUTPUT row it loads the two aligned input vectors that
// cover it, shifts in registers and stores once.  Heads and tails (fewer than one vector per row
// end) are copied element-wise.  No shared memory, no barriers.
//
// Role in the reference: transposeTiledCopy (src/cuttkernel.cu:356-426), which moves 32-element
// row pieces with scalar accesses.
//
// The per-lane body below is shared by the CUDA kernel and by the host interpreter of the CPU
// tests (which checks every access against the buffer bounds).
#pragma once
#include "permute_desc.h"
#include <string.h>

namespace cuttb {

constexpr int kRowCopyUnroll = 4;   // vector slots per lane and work item

struct RowCopyDesc {
  uint32_t elt;          // 4 or 8
  uint32_t nd;           // dimensions that enumerate the rows
  uint32_t rowLen;       // elements per row
  uint32_t segsPerRow;   // work items per row; an item is 32 * kRowCopyUnroll vector slots
  uint32_t numItems;     // rows * segsPerRow
  uint32_t pad_;
  uint64_t inBytes;      // size of the input buffer (bounds of the aligned loads)
  FastDiv segDiv;        // division by segsPerRow
  FastDiv div[kMaxDims]; // division by the extents of the row dimensions (input order)
  int64_t is[kMaxDims];  // input stride of each row dimension (elements)
  int64_t os[kMaxDims];  // output stride
};

#if !defined(__CUDA_ARCH__) && defined(CUTT_HOSTCHECK_BOUNDS)
struct HostBounds;
#define ROWCOPY_CHECK(p, n, lo, hi, al) \
  do { if ((const unsigned char*)(p) < (lo) || (const unsigned char*)(p) + (n) > (hi) || ((uintptr_t)(p) % (al)) != 0) { rowcopy_violations()++; return; } } while (0)
inline long long& rowcopy_violations() { static thread_local long long v = 0; return v; }
struct RowCopyBounds { const unsigned char *in0, *in1, *out0, *out1; };
inline RowCopyBounds& rowcopy_bounds() { static thread_local RowCopyBounds b = {}; return b; }
#endif

struct Vec16 { uint32_t w[4]; };

CUTT_HD void rc_load16(Vec16& v, const unsigned char* p) {
#if defined(__CUDA_ARCH__)
  const uint4 t = __ldg(reinterpret_cast<const uint4*>(p));
  v.w[0] = t.x; v.w[1] = t.y; v.w[2] = t.z; v.w[3] = t.w;
#else
#if defined(CUTT_HOSTCHECK_BOUNDS)
  ROWCOPY_CHECK(p, 16, rowcopy_bounds().in0, rowcopy_bounds().in1, 16);
#endif
  memcpy(v.w, p, 16);
#endif
}

CUTT_HD void rc_store16(unsigned char* p, const uint32_t* w) {
#if defined(__CUDA_ARCH__)
  *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
#else
#if defined(CUTT_HOSTCHECK_BOUNDS)
  ROWCOPY_CHECK(p, 16, rowcopy_bounds().out0, rowcopy_bounds().out1, 16);
#endif
  memcpy(p, w, 16);
#endif
}

template <int ELT>
CUTT_HD void rc_copy_elems(unsigned char* dst, const unsigned char* src, uint32_t n) {
  for (uint32_t e = 0; e < n; e++) {
#if defined(__CUDA_ARCH__)
    if (ELT == 4) reinterpret_cast<uint32_t*>(dst)[e] = reinterpret_cast<const uint32_t*>(src)[e];
    else reinterpret_cast<uint2*>(dst)[e] = reinterpret_cast<const uint2*>(src)[e];
#else
#if defined(CUTT_HOSTCHECK_BOUNDS)
    ROWCOPY_CHECK(src + (size_t)e * ELT, ELT, rowcopy_bounds().in0, rowcopy_bounds().in1, ELT);
    ROWCOPY_CHECK(dst + (size_t)e * ELT, ELT, rowcopy_bounds().out0, rowcopy_bounds().out1, ELT);
#endif
    memcpy(dst + (size_t)e * ELT, src + (size_t)e * ELT, ELT);
#endif
  }
}

// One lane's share of one work item.
template <int ELT>
CUTT_HD void rowcopy_item(const RowCopyDesc& D, const unsigned char* in, unsigned char* out,
                          uint32_t item, uint32_t lane) {
  constexpr uint32_t VE = 16 / ELT;
  constexpr int U = kRowCopyUnroll;
  // row and segment of this item
  const uint32_t row0 = fdiv(item, D.segDiv);
  const uint32_t seg = item - row0 * D.segsPerRow;
  int64_t ioff = 0, ooff = 0;
  uint32_t r = row0;
  for (uint32_t k = 0; k < D.nd; k++) {
    const uint32_t q = fdiv(r, D.div[k]);
    const uint32_t c = r - q * D.div[k].d;
    r = q;
    ioff += (int64_t)c * D.is[k];
    ooff += (int64_t)c * D.os[k];
  }
  const unsigned char* gin = in + ioff * ELT;
  unsigned char* gout = out + ooff * ELT;
  const uint32_t L = D.rowLen;
  // output alignment decides head / body / tail
  uint32_t h = (VE - (uint32_t)(((uintptr_t)gout / ELT) & (VE - 1))) & (VE - 1);
  if (h > L) h = L;
  const uint32_t nv = (L - h) / VE;
  const uint32_t tail0 = h + nv * VE;
  // misalignment of the input vector that feeds an aligned output vector (same for the whole row)
  const uint32_t delta = (uint32_t)((((uintptr_t)gin / ELT) + h) & (VE - 1));
  const unsigned char* inEnd = in + D.inBytes;

  Vec16 v0[U], v1[U];
  uint32_t kind[U];  // 0 nothing, 1 vector from registers, 2 vector copied element-wise already
#pragma unroll
  for (int u = 0; u < U; u++) {
    const uint32_t s = (seg * U + u) * 32 + lane;  // slot: 0 head, 1..nv body, nv+1 tail
    kind[u] = 0;
    if (s == 0) {
      if (h) rc_copy_elems<ELT>(gout, gin, h);
    } else if (s <= nv) {
      const uint32_t e0 = h + (s - 1) * VE;
      const unsigned char* src = gin + (size_t)e0 * ELT;
      const unsigned char* a = src - delta * ELT;
      const bool twoVecs = delta != 0;
      if (a >= in && a + (twoVecs ? 32 : 16) <= inEnd) {
        rc_load16(v0[u], a);
        if (twoVecs) rc_load16(v1[u], a + 16);
        kind[u] = 1;
      } else {
        rc_copy_elems<ELT>(gout + (size_t)e0 * ELT, src, VE);  // at the very ends of the buffer
        kind[u] = 2;
      }
    } else if (s == nv + 1) {
      if (tail0 < L) rc_copy_elems<ELT>(gout + (size_t)tail0 * ELT, gin + (size_t)tail0 * ELT, L - tail0);
    }
  }
  const uint32_t dw = delta * (ELT / 4);  // shift in 32-bit words
#pragma unroll
  for (int u = 0; u < U; u++) {
    if (kind[u] != 1) continue;
    const uint32_t s = (seg * U + u) * 32 + lane;
    const uint32_t e0 = h + (s - 1) * VE;
    uint32_t w[4];
    const uint32_t* a = v0[u].w;
    const uint32_t* b = v1[u].w;
    switch (dw) {  // uniform over the row, hence over the warp
      case 0: w[0] = a[0]; w[1] = a[1]; w[2] = a[2]; w[3] = a[3]; break;
      case 1: w[0] = a[1]; w[1] = a[2]; w[2] = a[3]; w[3] = b[0]; break;
      case 2: w[0] = a[2]; w[1] = a[3]; w[2] = b[0]; w[3] = b[1]; break;
      default: w[0] = a[3]; w[1] = b[0]; w[2] = b[1]; w[3] = b[2]; break;
    }
    rc_store16(gout + (size_t)e0 * ELT, w);
  }
}

}  // namespace cuttb
