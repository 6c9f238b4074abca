// Per-thread phases of the tiled permutation kernel.  The same functions run on the
// device (inside permute_tiles_kernel, one call per thread) and on the host (inside
// the plan interpreter that the CPU tests use to check descriptors without a GPU):
// only the three copy primitives differ.
//
// Phase "load":  global input  -> shared tile (contiguous runs, shared memory in input order)
// Phase "store": shared tile   -> global output (contiguous runs of the output, gathered
//                from shared memory through the output run's strides)
//
// Role in the reference: these two phases are what transposePacked / transposePackedSplit /
// transposeTiled / transposeTiledCopy (src/cuttkernel.cu:38-426) do between their two
// __syncthreads, generalised to one code path with explicit strides.
#pragma once
#include "permute_desc.h"
#include <string.h>

namespace cuttb {

template <int BYTES> struct VecT;
template <> struct VecT<4>  { uint32_t w[1]; };
template <> struct VecT<8>  { uint32_t w[2]; };
template <> struct VecT<16> { uint32_t w[4]; };

// global -> shared, BYTES in {4, 8, 16}; asynchronous on the device.
template <int BYTES>
CUTT_HD void copy_g2s(unsigned char* sdst, const unsigned char* gsrc) {
#if defined(__CUDA_ARCH__)
  unsigned int saddr = (unsigned int)__cvta_generic_to_shared(sdst);
  if (BYTES == 16) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(saddr), "l"(gsrc) : "memory");
  } else {
    asm volatile("cp.async.ca.shared.global [%0], [%1], %2;\n" ::"r"(saddr), "l"(gsrc), "n"(BYTES) : "memory");
  }
#else
  memcpy(sdst, gsrc, BYTES);
#endif
}

template <int BYTES>
CUTT_HD void lds(void* dst, const unsigned char* ssrc) {
#if defined(__CUDA_ARCH__)
  if (BYTES == 4) *(uint32_t*)dst = *(const uint32_t*)ssrc;
  else if (BYTES == 8) *(uint2*)dst = *(const uint2*)ssrc;
  else *(uint4*)dst = *(const uint4*)ssrc;
#else
  memcpy(dst, ssrc, BYTES);
#endif
}

template <int BYTES>
CUTT_HD void stg(unsigned char* gdst, const void* src) {
#if defined(__CUDA_ARCH__)
  if (BYTES == 4) *(uint32_t*)gdst = *(const uint32_t*)src;
  else if (BYTES == 8) *(uint2*)gdst = *(const uint2*)src;
  else *(uint4*)gdst = *(const uint4*)src;
#else
  memcpy(gdst, src, BYTES);
#endif
}

template <int ELT, int W>
CUTT_HD void tile_load(const TileDesc& D, const TileCtx& c, const RowEnt* tab,
                       unsigned char* sbuf, const unsigned char* gin, uint32_t tid) {
  const Side& S = D.in;
  const uint32_t tq = tid & (S.tq - 1);
  const uint32_t tr = tid >> S.tqShift;
  const uint32_t Tr = D.nthreads >> S.tqShift;
  const uint32_t valid = run_valid(S, c);
  const uint32_t rem0 = c.rem0, rem1 = c.rem1;
  const unsigned char* gbase = gin + c.inOff * ELT;
  const uint32_t qstep = S.tq * W;
  for (uint32_t row = tr; row < S.nrows; row += Tr) {
    const RowEnt e = tab[row];
    if (e.c0 < rem0 && e.c1 < rem1) {
      const unsigned char* g = gbase + e.goff * ELT;
      unsigned char* s = sbuf + (size_t)e.soff * ELT;
      for (uint32_t q = tq * W; q < valid; q += qstep)
        copy_g2s<ELT * W>(s + (size_t)q * ELT, g + (size_t)q * ELT);
    }
  }
}

template <int ELT, int W>
CUTT_HD void tile_store(const TileDesc& D, const TileCtx& c, const RowEnt* tab,
                        const unsigned char* sbuf, unsigned char* gout, uint32_t tid) {
  const Side& S = D.out;
  const uint32_t tq = tid & (S.tq - 1);
  const uint32_t tr = tid >> S.tqShift;
  const uint32_t Tr = D.nthreads >> S.tqShift;
  const uint32_t valid = run_valid(S, c);
  const uint32_t rem0 = c.rem0, rem1 = c.rem1;
  unsigned char* gbase = gout + c.outOff * ELT;
  const uint32_t qstep = S.tq * W;
  for (uint32_t q = tq * W; q < valid; q += qstep) {
    uint32_t so[W];
    so[0] = out_run_soff(D, q);
    if (W > 1) {
      if (D.smemGatherContig) {
#pragma unroll
        for (int i = 1; i < W; i++) so[i] = so[0] + i;
      } else {
#pragma unroll
        for (int i = 1; i < W; i++) so[i] = out_run_soff(D, q + i);
      }
    }
    unsigned char* gq = gbase + (size_t)q * ELT;
#pragma unroll 4
    for (uint32_t row = tr; row < S.nrows; row += Tr) {
      const RowEnt e = tab[row];
      if (e.c0 < rem0 && e.c1 < rem1) {
        VecT<ELT * W> v;
        if (W > 1 && D.smemGatherContig) {
          lds<ELT * W>(&v, sbuf + (size_t)(e.soff + so[0]) * ELT);
        } else {
#pragma unroll
          for (int i = 0; i < W; i++)
            lds<ELT>(&v.w[i * (ELT / 4)], sbuf + (size_t)(e.soff + so[i]) * ELT);
        }
        stg<ELT * W>(gq + e.goff * ELT, &v);
      }
    }
  }
}

}  // namespace cuttb
