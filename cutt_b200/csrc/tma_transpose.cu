// Tensor-map (TMA) transpose kernel for sm_100a: see tma_transpose.h for the problem class, the
// shared-memory layout and the store phase.
//
// A persistent grid walks the tile space.  Per thread block a ring of `stages` shared-memory
// buffers is filled by box loads that one thread issues `stages` tiles ahead
// (cp.async.bulk.tensor.5d, no cluster forms: every tensor map covers memory of this GPU only);
// each buffer has an mbarrier that the copy engine completes with the byte count of the boxes.
// All waits on the barriers are bounded: after kTmaSpinLimit failed polls (each may sleep up to about
// a microsecond) a thread raises the
// block's abort flag, the block stops after the current tile, thread 0 gives the loads still in
// flight their (bounded) chance to land, counts the event in the status word and returns.
//
// The tensor map is encoded on the host at launch time (cuTensorMapEncodeTiled, looked up through
// cudaGetDriverEntryPoint so that the library keeps linking against the CUDA runtime alone) and
// travels as a __grid_constant__ kernel parameter.
#include <cuda.h>
#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <map>
#include "kernels.h"
#include "tma_transpose.h"

namespace cuttb {

constexpr uint32_t kTmaSpinLimit = 1u << 20;   // polls of a barrier before giving up
constexpr uint32_t kTmaPollHintNs = 1000;      // a poll may suspend the thread for up to about this long

__device__ __forceinline__ uint32_t tma_shared_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void tma_mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void tma_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool tma_mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      "  .reg .pred p;\n"
      "  mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
      "  selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok) : "r"(bar), "r"(parity), "r"(kTmaPollHintNs) : "memory");
  return ok != 0;
}
// (the suspend-time hint lets a waiting thread sleep inside the poll instead of spinning through
// issue slots that the other blocks of the SM need: measured 1.7 -> 1.1 warp instructions per
// element on the fp64 matrix transpose)
__device__ __forceinline__ bool tma_mbar_wait_bounded(uint32_t bar, uint32_t parity) {
  for (uint32_t spin = 0; spin < kTmaSpinLimit; spin++)
    if (tma_mbar_try_wait(bar, parity)) return true;
  return false;
}

// One box: coordinates are element indices along the five dimensions of the tensor map.
__device__ __forceinline__ void tma_load_box(uint32_t dst, const CUtensorMap* tm, uint32_t bar, int c0, int c1, int c2,
                                             int c3, int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];\n"
      ::"r"(dst), "l"(tm), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
      : "memory");
}

template <int ELT>
__global__ void __launch_bounds__(256)
tma_transpose_kernel(const __grid_constant__ CUtensorMap tm, const __grid_constant__ TmaDesc D,
                     unsigned char* __restrict__ out, unsigned int* __restrict__ status) {
  extern __shared__ unsigned char tma_smem_raw[];
  __shared__ __align__(8) unsigned long long full[kTmaMaxStages];
  __shared__ uint32_t abortFlag;
  const uint32_t tid = threadIdx.x;
  const uint32_t G = gridDim.x;
  const uint32_t first = blockIdx.x;
  if (first >= D.numTiles) return;
  const uint32_t nlocal = (D.numTiles - first + G - 1) / G;
  const uint32_t S = D.stages;
  const uint32_t stageBytes = D.ta * D.tb * ELT;
  // the swizzle pattern is a function of the shared-memory address: stage buffers start on
  // 1024-byte boundaries (8 rows of 128 bytes)
  const uint32_t sbase = (tma_shared_addr(tma_smem_raw) + 1023u) & ~1023u;
  const uint32_t bar0 = tma_shared_addr(full);
  if (tid == 0) {
    for (uint32_t s = 0; s < S; s++) tma_mbar_init(bar0 + 8u * s, 1);
    abortFlag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  __syncthreads();

  auto issue = [&](uint32_t i) {   // thread 0: loads of this block's i-th tile
    TmaTile t;
    tma_decode(D, first + i * G, t);
    const uint32_t s = i % S;
    const uint32_t bar = bar0 + 8u * s;
    tma_mbar_expect_tx(bar, stageBytes);
    for (uint32_t k = 0; k < D.nboxes; k++) {
      int c0, c1, c2, c3, c4;
      tma_box_coords(D, t, k, c0, c1, c2, c3, c4);
      tma_load_box(sbase + s * stageBytes + k * (D.tb * kTmaBoxBytes), &tm, bar, c0, c1, c2, c3, c4);
    }
  };

  uint32_t issued = 0;
  if (tid == 0)
    for (; issued < S && issued < nlocal; issued++) issue(issued);

  const uint32_t nItems = tma_items_per_tile(D);
  uint32_t i = 0;
  bool aborted = false;
  for (; i < nlocal; i++) {
    const uint32_t s = i % S;
    const bool ok = tma_mbar_wait_bounded(bar0 + 8u * s, (i / S) & 1u);
    if (!ok) abortFlag = 1;   // every writer writes the same value
    if (ok) {
      TmaTile t;
      tma_decode(D, first + i * G, t);
      const uint32_t stage = sbase + s * stageBytes;
      for (uint32_t it = tid; it < nItems; it += blockDim.x) tma_store_item<ELT>(D, t, stage, out, it);
    }
    __syncthreads();   // everybody is done reading stage s (and has seen or set the abort flag)
    if (abortFlag) { aborted = true; break; }
    if (tid == 0 && i + S < nlocal) { issue(i + S); issued = i + S + 1; }
  }
  if (aborted && tid == 0) {
    atomicAdd(status, 1u);
    // loads i .. issued-1 may still be in flight: nothing may land in this block's shared memory
    // after the block has exited
    for (uint32_t j = i; j < issued; j++) tma_mbar_wait_bounded(bar0 + 8u * (j % S), (j / S) & 1u);
  }
}

// ---------------------------------------------------------------------------------------
// host side

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qr) == cudaSuccess &&
        qr == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)sym;
    else
      cudaGetLastError();
  });
  return fn;
}

bool tma_supported() { return encode_fn() != nullptr; }

size_t tma_smem_bytes(const TmaDesc& D) {
  return (size_t)D.stages * D.ta * D.tb * D.elt + 1024;   // + slack for the 1024-byte alignment
}

static const void* tma_kernel(const TmaDesc& D) {
  return D.elt == 4 ? (const void*)tma_transpose_kernel<4> : (const void*)tma_transpose_kernel<8>;
}

static std::mutex g_tmaAttrMutex;
static std::map<std::pair<int, const void*>, bool> g_tmaAttr;

static cudaError_t tma_ensure_smem(const void* k) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  std::lock_guard<std::mutex> lk(g_tmaAttrMutex);
  auto key = std::make_pair(dev, k);
  if (g_tmaAttr.count(key)) return cudaSuccess;
  int maxOptin = 0;
  e = cudaDeviceGetAttribute(&maxOptin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  if (e != cudaSuccess) return e;
  // the kernel also has a little static shared memory (barriers, abort flag): the dynamic part
  // may take what is left of the per-block limit
  cudaFuncAttributes fa;
  e = cudaFuncGetAttributes(&fa, k);
  if (e != cudaSuccess) return e;
  e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, maxOptin - (int)fa.sharedSizeBytes);
  if (e != cudaSuccess) {
    if (getenv("CUTT_VERBOSE")) fprintf(stderr, "[cutt] tma shared-memory attribute: %s\n", cudaGetErrorString(e));
    return e;
  }
  g_tmaAttr[key] = true;
  return cudaSuccess;
}

int tma_blocks_per_sm(const TmaDesc& D) {
  const void* k = tma_kernel(D);
  if (!tma_supported() || tma_ensure_smem(k) != cudaSuccess) return -1;
  int nb = 0;
  const cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, k, (int)D.nthreads, tma_smem_bytes(D));
  if (e != cudaSuccess) {
    if (getenv("CUTT_VERBOSE")) fprintf(stderr, "[cutt] tma occupancy query failed: %s\n", cudaGetErrorString(e));
    cudaGetLastError();
    return -1;
  }
  if (nb <= 0 && getenv("CUTT_VERBOSE")) fprintf(stderr, "[cutt] tma kernel does not fit: %zu bytes of shared memory\n", tma_smem_bytes(D));
  return nb;
}

static bool tma_encode(const TmaDesc& D, const TmaMapRecipe& R, const void* in, CUtensorMap& tm);

// The driver accepts this problem's tensor map (checked once, when a plan adopts the candidate; the
// encoder looks at the numbers only, so any 16-byte aligned address will do).
bool tma_map_encodable(const TmaDesc& D, const TmaMapRecipe& R) {
  CUtensorMap tm;
  return tma_encode(D, R, reinterpret_cast<const void*>((uintptr_t)1 << 20), tm);
}

static bool tma_encode(const TmaDesc& D, const TmaMapRecipe& R, const void* in, CUtensorMap& tm) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return false;
  cuuint64_t dims[5], strides[4];
  cuuint32_t box[5], estr[5];
  for (int i = 0; i < 5; i++) { dims[i] = R.dims[i]; box[i] = R.box[i]; estr[i] = 1; }
  for (int i = 0; i < 4; i++) strides[i] = R.strideBytes[i];
  const CUresult r = enc(&tm, D.elt == 4 ? CU_TENSOR_MAP_DATA_TYPE_UINT32 : CU_TENSOR_MAP_DATA_TYPE_UINT64, 5,
                         const_cast<void*>(in), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS && getenv("CUTT_VERBOSE"))
    fprintf(stderr, "[cutt] cuTensorMapEncodeTiled failed with code %d: dims %llu %llu %llu %llu %llu strides %llu %llu %llu %llu "
            "box %u %u %u %u %u\n", (int)r, (unsigned long long)dims[0], (unsigned long long)dims[1],
            (unsigned long long)dims[2], (unsigned long long)dims[3], (unsigned long long)dims[4],
            (unsigned long long)strides[0], (unsigned long long)strides[1], (unsigned long long)strides[2],
            (unsigned long long)strides[3], box[0], box[1], box[2], box[3], box[4]);
  return r == CUDA_SUCCESS;
}

cudaError_t launch_tma(const TmaDesc& D, const TmaMapRecipe& R, int gridBlocks, const void* in, void* out,
                       cudaStream_t stream) {
  if (!tma_supported()) return cudaErrorNotSupported;
  if ((uintptr_t)in % 16 || (uintptr_t)out % 16) return cudaErrorInvalidValue;
  CUtensorMap tm;
  if (!tma_encode(D, R, in, tm)) return cudaErrorInvalidValue;
  const void* k = tma_kernel(D);
  cudaError_t e = tma_ensure_smem(k);
  if (e != cudaSuccess) return e;
  unsigned int* st = bulk_copy_status_word();
  if (!st) return cudaErrorMemoryAllocation;
  if (D.elt == 4)
    tma_transpose_kernel<4><<<gridBlocks, D.nthreads, tma_smem_bytes(D), stream>>>(tm, D, (unsigned char*)out, st);
  else
    tma_transpose_kernel<8><<<gridBlocks, D.nthreads, tma_smem_bytes(D), stream>>>(tm, D, (unsigned char*)out, st);
  count_launch();
  return cudaGetLastError();
}

}  // namespace cuttb
