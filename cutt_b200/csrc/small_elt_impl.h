// Permutations of 1- and 2-byte elements (extension entry points; the reference handles 4- and
// 8-byte elements only, src/cutt.cpp:62).
//
// When the leading run of the tensor is kept and its byte length is a multiple of 4, such a
// problem is re-stated in 4- or 8-byte units and goes through the ordinary planner.  This file
// covers what is left: the elements really have to be moved one by one.
//
// A tile spans two dimensions: A, the fastest input dimension, and B, the fastest output
// dimension (the second-fastest output dimension when A is fastest on both sides).  One thread
// block moves one tile: lanes run along A while loading into shared memory, along B (or A again)
// while storing, so that both sides issue contiguous warp accesses.  All remaining dimensions
// are enumerated by the tile index.  Role in the reference: transposeTiled
// (src/cuttkernel.cu:38-118), which does the same for 32x32 tiles of 4/8-byte elements.
//
// The per-thread bodies are shared by the CUDA kernel and by the host interpreter of the CPU
// tests (which checks every access against the buffer bounds).
#pragma once
#include <string.h>
#include "permute_desc.h"
#include "planner.h"

namespace cuttb {

constexpr int kSmallThreads = 256;
constexpr uint32_t kSmallTileElems = 4096;   // elements per tile (when the extents allow)

struct SmallDesc {
  uint32_t elt;          // 1 or 2 bytes
  uint32_t nloop;        // dimensions enumerated by the tile index besides A and B
  uint32_t logTA;        // tile extent along A = 1 << logTA
  uint32_t logTB;
  uint32_t pitch;        // shared-memory row pitch (elements); rows run along A
  uint32_t storeAlongB;  // 1: B is the fastest output dimension, lanes store along B
  uint32_t numTiles;
  uint32_t smemBytes;
  uint32_t packLoad;     // 1: the strides allow 4-byte global loads (buffer 4-byte aligned)
  uint32_t packStore;    // 1: the same for the stores
  uint64_t dA, dB;       // extents
  int64_t isB;           // input stride of B (A has input stride 1), elements
  int64_t osA, osB;      // output strides
  uint64_t volume;       // elements of each buffer
  FastDiv tilesA, tilesB;        // divisions by the number of tiles along A and B
  FastDiv loopDiv[kMaxDims];     // divisions by the extents of the remaining dimensions
  int64_t loopIs[kMaxDims];
  int64_t loopOs[kMaxDims];
};

template <int ELT> struct SmallType;
template <> struct SmallType<1> { typedef uint8_t type; };
template <> struct SmallType<2> { typedef uint16_t type; };

// Range check of the host interpreter; always true in the library.
#if !defined(__CUDA_ARCH__) && defined(CUTT_HOSTCHECK_BOUNDS)
inline long long& small_violations() { static thread_local long long v = 0; return v; }
inline bool small_ok(uint64_t idx, uint64_t n) {
  if (idx < n) return true;
  small_violations()++;
  return false;
}
#else
CUTT_HD bool small_ok(uint64_t, uint64_t) { return true; }
#endif

// Alignment check of the host interpreter (a misaligned 32-bit access faults on the device).
#if !defined(__CUDA_ARCH__) && defined(CUTT_HOSTCHECK_BOUNDS)
inline bool small_aligned4(const void* p) {
  if (((uintptr_t)p & 3) == 0) return true;
  small_violations()++;
  return false;
}
#else
CUTT_HD bool small_aligned4(const void*) { return true; }
#endif

CUTT_HD uint32_t small_ldg32(const void* p) {
#if defined(__CUDA_ARCH__)
  return __ldg(reinterpret_cast<const uint32_t*>(p));
#else
  uint32_t w;
  memcpy(&w, p, 4);
  return w;
#endif
}

struct SmallOrigin {
  uint64_t a0, b0;     // coordinates of the tile's first element along A and B
  int64_t ioff, ooff;  // offsets of that element in the two buffers (elements)
};

CUTT_HD SmallOrigin small_origin(const SmallDesc& D, uint32_t tile) {
  SmallOrigin o;
  uint32_t q = fdiv(tile, D.tilesA);
  const uint32_t ta = tile - q * D.tilesA.d;
  uint32_t r = fdiv(q, D.tilesB);
  const uint32_t tb = q - r * D.tilesB.d;
  o.a0 = (uint64_t)ta << D.logTA;
  o.b0 = (uint64_t)tb << D.logTB;
  o.ioff = (int64_t)o.a0 + (int64_t)o.b0 * D.isB;
  o.ooff = (int64_t)o.a0 * D.osA + (int64_t)o.b0 * D.osB;
  for (uint32_t k = 0; k < D.nloop; k++) {
    const uint32_t qq = fdiv(r, D.loopDiv[k]);
    const uint32_t c = r - qq * D.loopDiv[k].d;
    r = qq;
    o.ioff += (int64_t)c * D.loopIs[k];
    o.ooff += (int64_t)c * D.loopOs[k];
  }
  return o;
}

// Global -> shared, lanes along A.
template <int ELT>
CUTT_HD void small_load(const SmallDesc& D, const SmallOrigin& o, const unsigned char* in,
                        unsigned char* smem, uint32_t tid, uint32_t nthreads) {
  typedef typename SmallType<ELT>::type T;
  const T* g = reinterpret_cast<const T*>(in);
  T* s = reinterpret_cast<T*>(smem);
  const uint64_t ra = D.dA - o.a0, rb = D.dB - o.b0;
  const uint32_t TA = 1u << D.logTA, TB = 1u << D.logTB;
  const uint32_t extA = ra < TA ? (uint32_t)ra : TA;
  const uint32_t extB = rb < TB ? (uint32_t)rb : TB;
  const uint32_t n = TA << D.logTB;
  if (D.packLoad) {
    // one 32-bit word (K elements along A) per step; the ragged end of a row element by element
    constexpr uint32_t K = 4 / ELT, LK = ELT == 2 ? 1 : 2;
    const uint32_t logWA = D.logTA - LK;
#if defined(__CUDA_ARCH__)
#pragma unroll 4
#endif
    for (uint32_t i = tid; i < (n >> LK); i += nthreads) {
      const uint32_t a = (i & ((1u << logWA) - 1)) << LK, b = i >> logWA;
      if (a >= extA || b >= extB) continue;
      const int64_t gi = o.ioff + (int64_t)a + (int64_t)b * D.isB;
      const uint32_t si = b * D.pitch + a;
      if (a + K <= extA) {
        if (small_ok((uint64_t)gi + K - 1, D.volume) && small_ok((uint64_t)(si + K) * ELT - 1, D.smemBytes) &&
            small_aligned4(g + gi) && small_aligned4(s + si))
          *reinterpret_cast<uint32_t*>(s + si) = small_ldg32(g + gi);
      } else {
        for (uint32_t k = 0; a + k < extA; k++)
          if (small_ok((uint64_t)gi + k, D.volume) && small_ok((uint64_t)(si + k) * ELT, D.smemBytes)) s[si + k] = g[gi + k];
      }
    }
    return;
  }
#if defined(__CUDA_ARCH__)
#pragma unroll 8
#endif
  for (uint32_t i = tid; i < n; i += nthreads) {
    const uint32_t a = i & (TA - 1), b = i >> D.logTA;
    if (a < extA && b < extB) {
      const int64_t gi = o.ioff + (int64_t)a + (int64_t)b * D.isB;
      const uint32_t si = b * D.pitch + a;
      if (small_ok((uint64_t)gi, D.volume) && small_ok((uint64_t)si * ELT, D.smemBytes)) s[si] = g[gi];
    }
  }
}

// Shared -> global, lanes along B when B is the fastest output dimension, else along A.
template <int ELT>
CUTT_HD void small_store(const SmallDesc& D, const SmallOrigin& o, unsigned char* out,
                         const unsigned char* smem, uint32_t tid, uint32_t nthreads) {
  typedef typename SmallType<ELT>::type T;
  T* g = reinterpret_cast<T*>(out);
  const T* s = reinterpret_cast<const T*>(smem);
  const uint64_t ra = D.dA - o.a0, rb = D.dB - o.b0;
  const uint32_t TA = 1u << D.logTA, TB = 1u << D.logTB;
  const uint32_t extA = ra < TA ? (uint32_t)ra : TA;
  const uint32_t extB = rb < TB ? (uint32_t)rb : TB;
  const uint32_t n = TA << D.logTB;
  if (D.packStore) {
    constexpr uint32_t K = 4 / ELT, LK = ELT == 2 ? 1 : 2;
#if defined(__CUDA_ARCH__)
#pragma unroll 4
#endif
    for (uint32_t i = tid; i < (n >> LK); i += nthreads) {
      if (D.storeAlongB) {
        // K neighbouring lanes take the K columns that share one shared-memory word (a broadcast,
        // not a bank conflict); each gathers K rows of its column into one output word
        const uint32_t da = i & (K - 1);
        const uint32_t b = ((i >> LK) & ((TB >> LK) - 1)) << LK;
        const uint32_t a = ((i >> D.logTB) << LK) + da;
        if (a >= extA || b >= extB) continue;
        const int64_t gi = o.ooff + (int64_t)a * D.osA + (int64_t)b;
        const uint32_t si = b * D.pitch + a;
        if (b + K <= extB) {
          uint32_t w = 0;
          bool ok = small_ok((uint64_t)gi + K - 1, D.volume) && small_aligned4(g + gi);
          for (uint32_t k = 0; k < K; k++) {
            if (!small_ok((uint64_t)(si + k * D.pitch) * ELT, D.smemBytes)) { ok = false; break; }
            w |= (uint32_t)s[si + k * D.pitch] << (8 * ELT * k);
          }
          if (ok) *reinterpret_cast<uint32_t*>(g + gi) = w;
        } else {
          for (uint32_t k = 0; b + k < extB; k++)
            if (small_ok((uint64_t)gi + k, D.volume) && small_ok((uint64_t)(si + k * D.pitch) * ELT, D.smemBytes))
              g[gi + k] = s[si + k * D.pitch];
        }
      } else {
        const uint32_t logWA = D.logTA - LK;
        const uint32_t a = (i & ((1u << logWA) - 1)) << LK, b = i >> logWA;
        if (a >= extA || b >= extB) continue;
        const int64_t gi = o.ooff + (int64_t)a + (int64_t)b * D.osB;
        const uint32_t si = b * D.pitch + a;
        if (a + K <= extA) {
          if (small_ok((uint64_t)gi + K - 1, D.volume) && small_ok((uint64_t)(si + K) * ELT - 1, D.smemBytes) &&
              small_aligned4(g + gi) && small_aligned4(s + si))
            *reinterpret_cast<uint32_t*>(g + gi) = *reinterpret_cast<const uint32_t*>(s + si);
        } else {
          for (uint32_t k = 0; a + k < extA; k++)
            if (small_ok((uint64_t)gi + k, D.volume) && small_ok((uint64_t)(si + k) * ELT, D.smemBytes)) g[gi + k] = s[si + k];
        }
      }
    }
    return;
  }
#if defined(__CUDA_ARCH__)
#pragma unroll 8
#endif
  for (uint32_t i = tid; i < n; i += nthreads) {
    uint32_t a, b;
    if (D.storeAlongB) { b = i & (TB - 1); a = i >> D.logTB; }
    else { a = i & (TA - 1); b = i >> D.logTA; }
    if (a < extA && b < extB) {
      const int64_t gi = o.ooff + (int64_t)a * D.osA + (int64_t)b * D.osB;
      const uint32_t si = b * D.pitch + a;
      if (small_ok((uint64_t)gi, D.volume) && small_ok((uint64_t)si * ELT, D.smemBytes)) g[gi] = s[si];
    }
  }
}

inline uint32_t small_log2_ceil(uint64_t x) {
  uint32_t l = 0;
  while ((1ull << l) < x) l++;
  return l;
}

// Describes a fused problem with 1- or 2-byte elements for the kernel above.  False when the
// problem is a plain copy, or has more tiles than one launch can index.
inline bool build_small(const Problem& P, SmallDesc& D) {
  if ((P.elt != 1 && P.elt != 2) || P.rank < 2 || P.identity || P.peerDim >= 0) return false;
  if (P.is[0] != 1 || P.inBase != 0 || P.outBase != 0) return false;
  memset(&D, 0, sizeof D);
  D.elt = (uint32_t)P.elt;
  const int A = 0;
  int B = -1;
  for (int j = 1; j < P.rank; j++)
    if (B < 0 || P.os[j] < P.os[B]) B = j;    // fastest output dimension apart from A
  D.storeAlongB = P.os[A] == 1 ? 0u : 1u;
  if (D.storeAlongB && P.os[B] != 1) return false;
  D.dA = (uint64_t)P.d[A];
  D.dB = (uint64_t)P.d[B];
  D.isB = P.is[B];
  D.osA = P.os[A];
  D.osB = P.os[B];
  D.volume = (uint64_t)P.volume;
  const uint64_t capA = D.storeAlongB ? 64 : 256;
  D.logTA = small_log2_ceil(D.dA < capA ? D.dA : capA);
  const uint64_t roomB = kSmallTileElems >> D.logTA;
  D.logTB = small_log2_ceil(D.dB < roomB ? D.dB : roomB);
  // an odd number of 32-bit words per row keeps the column-wise reads of the store phase on
  // distinct banks
  const uint32_t rowWords = (((1u << D.logTA) * D.elt + 3) / 4) | 1u;
  D.pitch = rowWords * 4 / D.elt;
  D.smemBytes = (D.pitch << D.logTB) * D.elt;
  const uint64_t nA = (D.dA + (1ull << D.logTA) - 1) >> D.logTA;
  const uint64_t nB = (D.dB + (1ull << D.logTB) - 1) >> D.logTB;
  uint64_t tiles = nA * nB;
  if (nA >= (1ull << 31) || nB >= (1ull << 31) || tiles >= (1ull << 31)) return false;
  D.tilesA = make_fastdiv((uint32_t)nA);
  D.tilesB = make_fastdiv((uint32_t)nB);
  for (int j = 1; j < P.rank; j++) {
    if (j == B) continue;
    if ((uint64_t)P.d[j] >= (1ull << 31)) return false;
    tiles *= (uint64_t)P.d[j];
    if (tiles >= (1ull << 31)) return false;
    D.loopDiv[D.nloop] = make_fastdiv((uint32_t)P.d[j]);
    D.loopIs[D.nloop] = P.is[j];
    D.loopOs[D.nloop] = P.os[j];
    D.nloop++;
  }
  D.numTiles = (uint32_t)tiles;
  // 4-byte accesses need every row of a tile to start on a 4-byte boundary
  const int64_t K = 4 / P.elt;
  bool inOk = D.logTA >= (P.elt == 2 ? 1u : 2u) && D.isB % K == 0;
  bool outOk = D.storeAlongB ? (D.logTB >= (P.elt == 2 ? 1u : 2u) && D.logTA >= (P.elt == 2 ? 1u : 2u) && D.osA % K == 0)
                             : (D.logTA >= (P.elt == 2 ? 1u : 2u) && D.osB % K == 0);
  for (uint32_t k = 0; k < D.nloop; k++) {
    if (D.loopIs[k] % K) inOk = false;
    if (D.loopOs[k] % K) outOk = false;
  }
  D.packLoad = inOk ? 1u : 0u;
  D.packStore = outOk ? 1u : 0u;
  return true;
}

}  // namespace cuttb
