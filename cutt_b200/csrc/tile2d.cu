// Two-dimensional tile transpose kernel for sm_100a (see tile2d.h): one tile per thread block,
// cp.async loads into 128-byte-swizzled shared memory, register-transposed stores.
#include <map>
#include <mutex>
#include "kernels.h"
#include "tile2d.h"

namespace cuttb {

template <int ELT, int WIB, int WOB>
__global__ void __launch_bounds__(256)
tile2d_kernel(const __grid_constant__ T2dDesc D, const unsigned char* __restrict__ in, unsigned char* __restrict__ out) {
  extern __shared__ __align__(1024) unsigned char t2d_smem[];
  const uint32_t tid = threadIdx.x;
  if (blockIdx.x >= D.numTiles) return;
  T2dTile t;
  t2d_decode(D, blockIdx.x, t);
  const uint32_t stage = (uint32_t)__cvta_generic_to_shared(t2d_smem);
  const uint32_t nUnits = t2d_load_units(D);
  for (uint32_t u = tid; u < nUnits; u += blockDim.x) t2d_load_unit<ELT, WIB>(D, t, stage, in, u);
  asm volatile("cp.async.commit_group;\n" ::: "memory");
  asm volatile("cp.async.wait_group 0;\n" ::: "memory");
  __syncthreads();
  const uint32_t nItems = t2d_store_items(D);
  for (uint32_t it = tid; it < nItems; it += blockDim.x) t2d_store_item<ELT, WOB>(D, t, stage, out, it);
}

typedef void (*T2dKernel)(const T2dDesc, const unsigned char*, unsigned char*);

static T2dKernel pick_t2d(const T2dDesc& D) {
#define T2D_CASE(E, A, B) if (D.elt == E && D.wiB == A && D.woB == B) return tile2d_kernel<E, A, B>;
  T2D_CASE(4, 4, 4) T2D_CASE(4, 4, 8) T2D_CASE(4, 4, 16)
  T2D_CASE(4, 8, 4) T2D_CASE(4, 8, 8) T2D_CASE(4, 8, 16)
  T2D_CASE(4, 16, 4) T2D_CASE(4, 16, 8) T2D_CASE(4, 16, 16)
  T2D_CASE(8, 8, 8) T2D_CASE(8, 8, 16) T2D_CASE(8, 16, 8) T2D_CASE(8, 16, 16)
#undef T2D_CASE
  return nullptr;
}

size_t t2d_smem_bytes(const T2dDesc& D) { return (size_t)D.ta * D.tb * D.elt; }

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

bool t2d_pointers_aligned(const T2dDesc& D, const void* in, const void* out) {
  return (uintptr_t)in % D.wiB == 0 && (uintptr_t)out % D.woB == 0;
}

cudaError_t launch_t2d(const T2dDesc& D, const void* in, void* out, cudaStream_t stream) {
  T2dKernel k = pick_t2d(D);
  if (!k) return cudaErrorInvalidValue;
  k<<<D.numTiles, D.nthreads, t2d_smem_bytes(D), stream>>>(D, (const unsigned char*)in, (unsigned char*)out);
  count_launch();
  return cudaGetLastError();
}

}  // namespace cuttb
