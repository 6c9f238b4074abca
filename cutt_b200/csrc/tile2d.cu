// Two-dimensional tile transpose kernel for sm_100a (see tile2d.h): one tile per thread block,
// 16-byte global accesses on both sides whatever the alignment of the rows, 128-byte-swizzled
// shared memory, register-transposed stores.
#include <map>
#include <mutex>
#include "kernels.h"
#include "tile2d.h"

namespace cuttb {

template <int ELT, int LOAD, int STORE>
__global__ void __launch_bounds__(256)
tile2d_kernel(const __grid_constant__ T2dDesc D, const unsigned char* __restrict__ in, unsigned char* __restrict__ out) {
  extern __shared__ __align__(128) unsigned char t2d_smem[];
  const uint32_t tid = threadIdx.x;
  if (blockIdx.x >= D.numTiles) return;
  T2dTile t;
  if (!t2d_decode(D, blockIdx.x, t)) return;
  const uint32_t stage = (uint32_t)__cvta_generic_to_shared(t2d_smem);
  const uint32_t nUnits = t2d_load_units(D);
  if constexpr (LOAD == 1) {
    // four units per thread at a time: eight global loads in flight before the first is consumed
    constexpr int B = 4;
    for (uint32_t u0 = tid; u0 < nUnits; u0 += B * blockDim.x) {
      uint32_t w[B][8], m[B], soff[B];
      bool ok[B];
#pragma unroll
      for (int b = 0; b < B; b++) {
        const uint32_t u = u0 + (uint32_t)b * blockDim.x;
        ok[b] = u < nUnits && t2d_shift_fetch<ELT>(D, t, in, u, w[b], m[b], soff[b]);
      }
#pragma unroll
      for (int b = 0; b < B; b++)
        if (ok[b]) t2d_shift_commit<ELT>(stage + soff[b], w[b], m[b]);
    }
  } else {
    t2d_load_rows<ELT, (LOAD == 1 ? 16 : LOAD)>(D, t, stage, in, tid);
    asm volatile("cp.async.commit_group;\n" ::: "memory");
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
  }
  __syncthreads();
  const uint32_t nItems = t2d_store_items(D);
  if constexpr (STORE == 1) {
    for (uint32_t it = tid; it < nItems; it += blockDim.x) t2d_store_shear<ELT>(D, t, stage, out, it);
  } else if constexpr (ELT == 2) {
    t2d_store_rows_e2(D, t, stage, out, tid);
  } else if constexpr (ELT == 1) {
    t2d_store_rows_e1(D, t, stage, out, tid);
  } else {
    t2d_store_rows<ELT, (STORE == 1 ? 16 : STORE)>(D, t, stage, out, tid);
  }
}

typedef void (*T2dKernel)(const T2dDesc, const unsigned char*, unsigned char*);

static T2dKernel pick_t2d(const T2dDesc& D) {
#define T2D_CASE(E, A, B) if (D.elt == E && D.loadMode == A && D.storeMode == B) return tile2d_kernel<E, A, B>;
#define T2D_ROW(E, A) T2D_CASE(E, A, 16) T2D_CASE(E, A, 1) T2D_CASE(E, A, 8)
  T2D_ROW(4, 16) T2D_ROW(4, 1) T2D_ROW(4, 8) T2D_ROW(4, 4)
  T2D_CASE(4, 16, 4) T2D_CASE(4, 1, 4) T2D_CASE(4, 8, 4) T2D_CASE(4, 4, 4)
  T2D_ROW(8, 16) T2D_ROW(8, 1) T2D_ROW(8, 8)
  T2D_CASE(2, 16, 16) T2D_CASE(2, 8, 16) T2D_CASE(2, 4, 16)   // 2- and 1-byte elements: extension entry points
  T2D_CASE(1, 16, 16) T2D_CASE(1, 8, 16) T2D_CASE(1, 4, 16)
  T2D_CASE(2, 16, 8) T2D_CASE(2, 8, 8) T2D_CASE(2, 4, 8)
  T2D_CASE(1, 16, 8) T2D_CASE(1, 8, 8) T2D_CASE(1, 4, 8)
#undef T2D_ROW
#undef T2D_CASE
  return nullptr;
}

size_t t2d_smem_bytes(const T2dDesc& D) { return (size_t)D.nboxes * D.rowsAlloc * 128u; }

int t2d_blocks_per_sm(const T2dDesc& D) {
  T2dKernel k = pick_t2d(D);
  if (!k) return -1;
  int nb = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, (const void*)k, (int)D.nthreads, t2d_smem_bytes(D)) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  return nb;
}

// The cp.async load modes and the plain store modes need buffers aligned to their access width; the
// shift and shear modes take any element-aligned buffer (the misalignment travels in the descriptor).
bool t2d_pointers_aligned(const T2dDesc& D, const void* in, const void* out) {
  const uintptr_t ai = D.loadMode == 1 ? D.elt : D.loadMode, ao = D.storeMode == 1 ? D.elt : D.storeMode;
  return (uintptr_t)in % ai == 0 && (uintptr_t)out % ao == 0;
}

cudaError_t launch_t2d(const T2dDesc& desc, const void* in, void* out, cudaStream_t stream) {
  T2dKernel k = pick_t2d(desc);
  if (!k) return cudaErrorInvalidValue;
  T2dDesc D = desc;
  const uintptr_t ve = 16 / D.elt;
  D.inMis = (uint32_t)(((uintptr_t)in / D.elt) % ve);
  D.outMis = (uint32_t)(((uintptr_t)out / D.elt) % ve);
  k<<<D.numTiles, D.nthreads, t2d_smem_bytes(D), stream>>>(D, (const unsigned char*)in, (unsigned char*)out);
  count_launch();
  return cudaGetLastError();
}

}  // namespace cuttb
