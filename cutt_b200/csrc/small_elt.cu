// Kernel and launcher for permutations of 1- and 2-byte elements (small_elt_impl.h).
#include "kernels.h"
#include "small_elt_impl.h"
#include <stdint.h>

namespace cuttb {

template <int ELT>
__global__ void __launch_bounds__(kSmallThreads)
small_elt_kernel(const __grid_constant__ SmallDesc D, const unsigned char* __restrict__ in,
                 unsigned char* __restrict__ out) {
  extern __shared__ __align__(16) unsigned char smem[];
  const uint32_t tile = blockIdx.x;
  if (tile >= D.numTiles) return;
  const SmallOrigin o = small_origin(D, tile);
  small_load<ELT>(D, o, in, smem, threadIdx.x, blockDim.x);
  __syncthreads();
  small_store<ELT>(D, o, out, smem, threadIdx.x, blockDim.x);
}

cudaError_t launch_small(const SmallDesc& plan, const void* in, void* out, cudaStream_t stream) {
  if (plan.numTiles == 0 || plan.smemBytes > 48 * 1024) return cudaErrorInvalidValue;
  // 32-bit accesses only on buffers that are 4-byte aligned themselves
  SmallDesc d = plan;
  if ((uintptr_t)in % 4) d.packLoad = 0;
  if ((uintptr_t)out % 4) d.packStore = 0;
  if (d.elt == 1)
    small_elt_kernel<1><<<d.numTiles, kSmallThreads, d.smemBytes, stream>>>(
        d, (const unsigned char*)in, (unsigned char*)out);
  else if (d.elt == 2)
    small_elt_kernel<2><<<d.numTiles, kSmallThreads, d.smemBytes, stream>>>(
        d, (const unsigned char*)in, (unsigned char*)out);
  else
    return cudaErrorInvalidValue;
  count_launch();
  return cudaGetLastError();
}

}  // namespace cuttb
