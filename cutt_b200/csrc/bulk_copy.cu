// Contiguous copy through the bulk asynchronous copy engine (TMA without a tensor map):
// global -> shared with cp.async.bulk + mbarrier transaction counts, shared -> global with
// cp.async.bulk bulk groups.  One thread per block drives a ring of 32 KB stages; no thread
// touches the data.  Used for identity permutations (the reference's Trivial method,
// src/cuttkernel.cu:846-851, calls cudaMemcpyAsync) when both buffers are 16-byte aligned.
//
// Every wait on an mbarrier is bounded: after kBulkSpinLimit failed polls the block counts a
// timeout in a status word in global memory, drains what it has in flight (bounded again) and
// returns, so a lost completion can never hang the device.  The status word is the only global
// memory the kernel uses besides its input and output.
#include "kernels.h"
#include <cstdio>
#include <map>
#include <mutex>

namespace cuttb {

constexpr uint32_t kBulkChunk = 32u * 1024u;   // bytes per stage
constexpr int kBulkStages = 4;                 // 128 KB of shared memory per block
constexpr uint32_t kBulkSpinLimit = 1u << 22;  // polls of a barrier before giving up

__device__ __forceinline__ uint32_t shared_addr(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      "  .reg .pred p;\n"
      "  mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "  selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}

// false if the barrier did not complete the awaited phase within the poll limit
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
  for (uint32_t spin = 0; spin < kBulkSpinLimit; spin++)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}

__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

__device__ __forceinline__ void bulk_s2g(void* dst, uint32_t src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;\n"
               ::"l"(dst), "r"(src), "r"(bytes) : "memory");
}

__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;\n" ::: "memory"); }
// all committed stores have finished READING shared memory
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory"); }
// all committed stores are complete
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;\n" ::: "memory"); }

// The copy pipeline of one thread block (its thread 0).  nbytes: multiple of 16; in/out: 16-byte
// aligned.  A barrier wait that runs out is reported in status[blockIdx.x] (PER_BLOCK: one word
// per block, set to 1) or counted in status[0].
template <bool PER_BLOCK>
__device__ __forceinline__ void bulk_copy_block(const unsigned char* __restrict__ in, unsigned char* __restrict__ out,
                                                unsigned long long nbytes, unsigned int* __restrict__ status) {
  extern __shared__ __align__(128) unsigned char stages[];
  __shared__ __align__(8) unsigned long long full[kBulkStages];
  if (threadIdx.x != 0) return;  // the copy engine does the work; one thread issues and waits

  const uint32_t bar0 = shared_addr(full);
  const uint32_t st0 = shared_addr(stages);
  for (int s = 0; s < kBulkStages; s++) mbar_init(bar0 + 8u * s, 1);
  // make the initialised barriers visible to the asynchronous proxy before it signals them
  asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");

  const unsigned long long nchunks = (nbytes + kBulkChunk - 1) / kBulkChunk;
  const unsigned long long first = blockIdx.x, stride = gridDim.x;
  if (first >= nchunks) return;
  const unsigned long long nlocal = (nchunks - first + stride - 1) / stride;

  auto load = [&](unsigned long long i) {
    const unsigned long long off = (first + i * stride) * kBulkChunk;
    const unsigned long long rem = nbytes - off;
    const uint32_t bytes = rem < kBulkChunk ? (uint32_t)rem : kBulkChunk;
    const uint32_t s = (uint32_t)(i % kBulkStages);
    mbar_expect_tx(bar0 + 8u * s, bytes);
    bulk_g2s(st0 + s * kBulkChunk, in + off, bytes, bar0 + 8u * s);
  };

  unsigned long long issued = 0;
  for (; issued < nlocal && issued < (unsigned long long)kBulkStages; issued++) load(issued);

  bool failed = false;
  unsigned long long i = 0;
  for (; i < nlocal; i++) {
    const uint32_t s = (uint32_t)(i % kBulkStages);
    const uint32_t parity = (uint32_t)((i / kBulkStages) & 1ull);
    if (!mbar_wait_bounded(bar0 + 8u * s, parity)) { failed = true; break; }
    const unsigned long long off = (first + i * stride) * kBulkChunk;
    const unsigned long long rem = nbytes - off;
    const uint32_t bytes = rem < kBulkChunk ? (uint32_t)rem : kBulkChunk;
    bulk_s2g(out + off, st0 + s * kBulkChunk, bytes);
    bulk_commit();
    if (issued < nlocal) {
      bulk_wait_read_all();  // the stage may be overwritten once the store has read it
      load(issued);
      issued++;
    }
  }
  if (failed) {
    if (PER_BLOCK) status[blockIdx.x] = 1u;
    else atomicAdd(status, 1u);
    // loads i .. issued-1 may still be in flight: give each its (bounded) chance to land so that
    // nothing is written into this block's shared memory after it has exited
    for (unsigned long long j = i; j < issued; j++)
      mbar_wait_bounded(bar0 + 8u * (uint32_t)(j % kBulkStages), (uint32_t)((j / kBulkStages) & 1ull));
  }
  bulk_wait_all();
}

__global__ void __launch_bounds__(32, 1)
bulk_copy_kernel(const unsigned char* __restrict__ in, unsigned char* __restrict__ out,
                 unsigned long long nbytes, unsigned int* __restrict__ status) {
  bulk_copy_block<false>(in, out, nbytes, status);
}

// Per-device status word (timeouts observed by bulk_copy_kernel), allocated on first use.
static std::mutex g_statusMutex;
static std::map<int, unsigned int*> g_statusWord;

static unsigned int* status_word(int dev) {
  std::lock_guard<std::mutex> lk(g_statusMutex);
  auto it = g_statusWord.find(dev);
  if (it != g_statusWord.end()) return it->second;
  unsigned int* p = nullptr;
  if (cudaMalloc(&p, 256) != cudaSuccess) { cudaGetLastError(); return nullptr; }
  if (cudaMemset(p, 0, 256) != cudaSuccess) { cudaGetLastError(); cudaFree(p); return nullptr; }
  g_statusWord[dev] = p;
  return p;
}

unsigned int* bulk_copy_status_word() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
  return status_word(dev);
}

bool bulk_copy_usable(const void* in, const void* out, size_t bytes) {
  return ((uintptr_t)in % 16 == 0) && ((uintptr_t)out % 16 == 0) && bytes >= (size_t)kBulkChunk;
}

cudaError_t launch_bulk_copy_with_status(const void* in, void* out, size_t bytes16, int numSM,
                                         unsigned int* status, cudaStream_t stream) {
  static std::mutex attrMutex;
  static std::map<int, bool> attrSet;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  const int smem = kBulkStages * (int)kBulkChunk;
  {
    std::lock_guard<std::mutex> lk(attrMutex);
    if (!attrSet[dev]) {
      e = cudaFuncSetAttribute((const void*)bulk_copy_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (e != cudaSuccess) return e;
      attrSet[dev] = true;
    }
  }
  const unsigned long long nchunks = (bytes16 + kBulkChunk - 1) / kBulkChunk;
  int grid = (int)(nchunks < (unsigned long long)numSM ? nchunks : (unsigned long long)numSM);
  if (grid < 1) return cudaSuccess;
  bulk_copy_kernel<<<grid, 32, smem, stream>>>((const unsigned char*)in, (unsigned char*)out,
                                               (unsigned long long)bytes16, status);
  return cudaGetLastError();
}

cudaError_t launch_bulk_copy(const void* in, void* out, size_t bytes16, int numSM, cudaStream_t stream) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  unsigned int* st = status_word(dev);
  if (!st) return cudaErrorMemoryAllocation;
  return launch_bulk_copy_with_status(in, out, bytes16, numSM, st, stream);
}

// Timeouts counted on the current device since the library was loaded.  Waits for all work on the
// device first (cudaDeviceSynchronize: a plain blocking copy would not wait for streams created
// with cudaStreamNonBlocking).
int bulk_copy_timeouts() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  unsigned int* st = nullptr;
  {
    std::lock_guard<std::mutex> lk(g_statusMutex);
    auto it = g_statusWord.find(dev);
    if (it == g_statusWord.end()) return 0;
    st = it->second;
  }
  unsigned int v = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  if (cudaMemcpy(&v, st, sizeof v, cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  return (int)v;
}

// ---------------------------------------------------------------------------------------
// Copy entry point for callers that must not allocate device memory.
//
// Some hosts cannot call cudaMalloc when they need a copy: they have handed the whole device
// to a memory manager of their own, or they sit in a latency-critical loop where the
// device-wide synchronisation an allocation implies is not acceptable.  For them the status
// words of the copy kernel live in a fixed array inside the library image instead of an
// allocation: kNoAllocMaxBlocks words (1 KB), present on every GPU that loads the library
// until the process exits.
//
// The array below is a device symbol.  Its name is only a stand-in on the host side - handing
// it to a kernel as if it were a pointer would make the kernel use the wrong memory - so the
// device address is looked up once per device with cudaGetSymbolAddress (device current, return
// code checked) and that address is what the kernel receives.
constexpr int kNoAllocMaxBlocks = 256;                       // thread blocks one launch may use
constexpr unsigned long long kNoAllocMaxBytes = 1ull << 40;  // largest copy accepted (1 TiB)

static __device__ __align__(256) unsigned int g_noalloc_status[kNoAllocMaxBlocks];

// Same pipeline as bulk_copy_kernel; block b reports in status[b] (1 = a barrier wait ran out).
__global__ void __launch_bounds__(32, 1)
bulk_copy_noalloc_kernel(const unsigned char* __restrict__ in, unsigned char* __restrict__ out,
                         unsigned long long nbytes, unsigned int* __restrict__ status) {
  bulk_copy_block<true>(in, out, nbytes, status);
}

struct NoAllocDevice {
  unsigned int* status = nullptr;  // device address of g_noalloc_status on this device
  int numSM = 0;
};
static std::mutex g_noallocMutex;
static std::map<int, NoAllocDevice> g_noallocDevices;

// One-time set-up for the current device: symbol address, SM count, shared-memory limit of the
// kernel.  None of these allocate.
static cudaError_t noalloc_setup(int dev, NoAllocDevice& out) {
  std::lock_guard<std::mutex> lk(g_noallocMutex);
  auto it = g_noallocDevices.find(dev);
  if (it != g_noallocDevices.end()) { out = it->second; return cudaSuccess; }
  NoAllocDevice d;
  void* p = nullptr;
  cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_status);
  if (e != cudaSuccess) return e;
  d.status = static_cast<unsigned int*>(p);
  e = cudaDeviceGetAttribute(&d.numSM, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return e;
  e = cudaFuncSetAttribute((const void*)bulk_copy_noalloc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           kBulkStages * (int)kBulkChunk);
  if (e != cudaSuccess) return e;
  g_noallocDevices[dev] = d;
  out = d;
  return cudaSuccess;
}

}  // namespace cuttb

extern "C" {

// Declared in include/cutt_c.h.  0 success, 2 invalid parameter (null or misaligned pointers, size
// not a multiple of 16, size over the limit), 4 a CUDA call failed.  The launch uses one thread
// block per SM but never more than the array has status words (the kernel strides over the
// chunks, so a smaller grid only means more chunks per block).
int cutt_c_copy_noalloc(const void* src, void* dst, size_t bytes, void* stream) {
  using namespace cuttb;
  if (!src || !dst || src == dst) return 2;
  if ((uintptr_t)src % 16 || (uintptr_t)dst % 16 || bytes % 16) return 2;
  if (bytes == 0) return 0;
  if ((unsigned long long)bytes > kNoAllocMaxBytes) {
    fprintf(stderr, "cutt_c_copy_noalloc: %zu bytes exceed the limit of %llu bytes per call\n", bytes, kNoAllocMaxBytes);
    return 2;
  }
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 4;
  NoAllocDevice d;
  if (noalloc_setup(dev, d) != cudaSuccess) { cudaGetLastError(); return 4; }
  const unsigned long long nchunks = ((unsigned long long)bytes + kBulkChunk - 1) / kBulkChunk;
  unsigned long long want = nchunks < (unsigned long long)d.numSM ? nchunks : (unsigned long long)d.numSM;
  if (want > (unsigned long long)kNoAllocMaxBlocks) want = kNoAllocMaxBlocks;
  const int grid = (int)want;
  cudaStream_t st = (cudaStream_t)stream;
  // the array keeps what earlier calls left (a larger launch may have set words this one does not
  // use): the whole array starts at zero for every call
  if (cudaMemsetAsync(d.status, 0, sizeof(unsigned int) * kNoAllocMaxBlocks, st) != cudaSuccess) { cudaGetLastError(); return 4; }
  bulk_copy_noalloc_kernel<<<grid, 32, kBulkStages * (int)kBulkChunk, st>>>(
      (const unsigned char*)src, (unsigned char*)dst, (unsigned long long)bytes, d.status);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

// Thread blocks whose barrier wait ran out during the most recent cutt_c_copy_noalloc on the
// current device (0 in a healthy run).  Waits for all work on the device, whatever stream it is on
// (cudaDeviceSynchronize), before reading the words; -1 on error or before the first call.
int cutt_c_copy_noalloc_timeouts(void) {
  using namespace cuttb;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  NoAllocDevice d;
  {
    std::lock_guard<std::mutex> lk(g_noallocMutex);
    auto it = g_noallocDevices.find(dev);
    if (it == g_noallocDevices.end()) return -1;
    d = it->second;
  }
  unsigned int host[kNoAllocMaxBlocks];
  if (cudaDeviceSynchronize() != cudaSuccess) { cudaGetLastError(); return -1; }
  if (cudaMemcpy(host, d.status, sizeof host, cudaMemcpyDeviceToHost) != cudaSuccess) { cudaGetLastError(); return -1; }
  int n = 0;
  for (int b = 0; b < kNoAllocMaxBlocks; b++) n += host[b] ? 1 : 0;
  return n;
}

}  // extern "C"
