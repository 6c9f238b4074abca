// sm_100a kernels of the permutation path.
//
//  permute_tiles_kernel  the general kernel: a persistent grid walks the tile space; each
//                        tile is staged global -> shared with cp.async (4/8/16-byte, two
//                        stages so the next tile's loads overlap this tile's stores) and
//                        written back as contiguous runs of the output.  It covers what the
//                        reference does with four kernels (Tiled, TiledCopy, Packed,
//                        PackedSplit; src/cuttkernel.cu:38-426).
//  copy_kernel           identity permutations (the reference's Trivial method,
//                        src/cuttkernel.cu:846-851, uses cudaMemcpyAsync).
//  naive_kernel          one thread per output element, any rank; fallback and cross-check.
#include "kernels.h"
#include <atomic>
#include <mutex>
#include <map>
#include <tuple>
#include "permute_tile_impl.h"

namespace cuttb {

static std::atomic<unsigned long long> g_launches{0};
unsigned long long launch_count() { return g_launches.load(); }
void count_launch() { g_launches++; }

__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

template <int ELT, int WIN, int WOUT, int V, bool WIDE, bool AOF>
__global__ void __launch_bounds__(512)
permute_tiles_kernel(const __grid_constant__ TileDesc D, const unsigned char* __restrict__ in,
                     const __grid_constant__ PeerPtrs outs) {
  extern __shared__ __align__(16) unsigned char smem[];
  const uint32_t tid = threadIdx.x;
  const uint32_t G = gridDim.x;
  uint32_t tile = blockIdx.x;
  if (tile >= D.numTiles) return;
  // Per-tile contexts are decoded by one thread, two tiles ahead, and read by everybody
  // after the barriers that separate the phases.
  TileCtx* ctxs = reinterpret_cast<TileCtx*>(smem + table_layout(D).ctx);
  if (tid == 0) {
    decode_tile(D, tile, ctxs[0]);
    if (tile + G < D.numTiles) decode_tile(D, tile + G, ctxs[1]);
  }
  build_tables<WIDE>(D, smem, tid, blockDim.x);
  __syncthreads();
  const Tables<WIDE> T = make_tables<WIDE>(D, smem);
  const uint32_t stage0 = (uint32_t)__cvta_generic_to_shared(smem) + D.tableBytes;

  TileCtx cur = ctxs[0];
  TileCtx nxt = cur;
  if (D.stages >= 2) {
    if (cur.valid) tile_load<ELT, WIN, WIDE, AOF>(D, cur, T, stage0, in, tid);
    cp_async_commit();
    uint32_t s = 0;
    for (uint32_t it = 0; tile < D.numTiles; tile += G, it++) {
      if (tile + G < D.numTiles) {
        nxt = ctxs[(it + 1) & 1];
        if (nxt.valid) tile_load<ELT, WIN, WIDE, AOF>(D, nxt, T, stage0 + (s ^ 1u) * D.stageBytes, in, tid);
      }
      cp_async_commit();
      cp_async_wait<1>();
      __syncthreads();
      // Slot it&1 held this tile's context.  Every thread copied it to registers before the
      // barrier above (at the top of the previous iteration, or in the prologue), and nobody
      // reads the slot again before the barrier below, so thread 0 may overwrite it here.
      if (tid == 0 && tile + 2 * (uint64_t)G < D.numTiles) decode_tile(D, tile + 2 * G, ctxs[it & 1]);
      unsigned char* o = D.peerLoopDim >= 0 ? outs.p[cur.peer] : outs.p[0];
      if (cur.valid) tile_store<ELT, WOUT, V, WIDE, AOF>(D, cur, T, stage0 + s * D.stageBytes, in, o, tid);
      __syncthreads();
      cur = nxt;
      s ^= 1u;
    }
  } else {
    for (uint32_t it = 0; tile < D.numTiles; tile += G, it++) {
      if (it > 0) cur = ctxs[it & 1];
      if (cur.valid) tile_load<ELT, WIN, WIDE, AOF>(D, cur, T, stage0, in, tid);
      cp_async_commit();
      cp_async_wait<0>();
      __syncthreads();
      // every thread has read slot it&1 (this tile) before the barrier above
      if (tid == 0 && tile + 2 * (uint64_t)G < D.numTiles) decode_tile(D, tile + 2 * G, ctxs[it & 1]);
      unsigned char* o = D.peerLoopDim >= 0 ? outs.p[cur.peer] : outs.p[0];
      if (cur.valid) tile_store<ELT, WOUT, V, WIDE, AOF>(D, cur, T, stage0, in, o, tid);
      __syncthreads();
    }
  }
}

static_assert(sizeof(TileDesc) + sizeof(void*) + sizeof(PeerPtrs) <= 4096,
              "kernel parameters must fit the 4 KB parameter space");

typedef void (*TilesKernel)(const TileDesc, const unsigned char*, const PeerPtrs);

static TilesKernel pick_tiles_kernel(const TileDesc& D) {
  const int elt = D.elt, win = D.in.vec, wout = D.out.vec, v = D.vblk;
  if (D.aof) {  // aligned over-fetch: 16-byte loads, no register blocking, 32-bit offsets
    if (D.wide || v > 2) return nullptr;
    if (elt == 4 && win == 4 && v == 2) {  // rows 8-byte aligned: 8-byte register blocking still works
      if (wout == 1) return permute_tiles_kernel<4, 4, 1, 2, false, true>;
      if (wout == 2) return permute_tiles_kernel<4, 4, 2, 2, false, true>;
      if (wout == 4) return permute_tiles_kernel<4, 4, 4, 2, false, true>;
    }
    if (v != 1) return nullptr;
    if (elt == 4 && win == 4) {
      if (wout == 1) return permute_tiles_kernel<4, 4, 1, 1, false, true>;
      if (wout == 2) return permute_tiles_kernel<4, 4, 2, 1, false, true>;
      if (wout == 4) return permute_tiles_kernel<4, 4, 4, 1, false, true>;
    }
    if (elt == 8 && win == 2) {
      if (wout == 1) return permute_tiles_kernel<8, 2, 1, 1, false, true>;
      if (wout == 2) return permute_tiles_kernel<8, 2, 2, 1, false, true>;
    }
    return nullptr;
  }
#define CASE(E, A, B, VV) \
  if (elt == E && win == A && wout == B && v == VV) { \
    if (D.wide) return VV == 1 ? permute_tiles_kernel<E, A, B, 1, true, false> : nullptr; \
    return permute_tiles_kernel<E, A, B, VV, false, false>; }
#define CASES_V(E, A, B) CASE(E, A, B, 1) CASE(E, A, B, 2) CASE(E, A, B, 4)
  CASES_V(4, 1, 1) CASES_V(4, 1, 2) CASES_V(4, 1, 4) CASES_V(4, 2, 1) CASES_V(4, 2, 2) CASES_V(4, 2, 4)
  CASES_V(4, 4, 1) CASES_V(4, 4, 2) CASES_V(4, 4, 4)
  CASE(8, 1, 1, 1) CASE(8, 1, 1, 2) CASE(8, 1, 2, 1) CASE(8, 1, 2, 2)
  CASE(8, 2, 1, 1) CASE(8, 2, 1, 2) CASE(8, 2, 2, 1) CASE(8, 2, 2, 2)
#undef CASES_V
#undef CASE
  return nullptr;
}

// Largest dynamic shared-memory size configured so far per (device, kernel).
static std::mutex g_attrMutex;
static std::map<std::pair<int, const void*>, int> g_smemAttr;

static cudaError_t ensure_smem(TilesKernel k, int bytes) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  std::lock_guard<std::mutex> lk(g_attrMutex);
  auto key = std::make_pair(dev, (const void*)k);
  auto it = g_smemAttr.find(key);
  if (it != g_smemAttr.end() && it->second >= bytes) return cudaSuccess;
  // raise to the device maximum once: later plans never need to touch the attribute again
  int maxOptin = 0;
  e = cudaDeviceGetAttribute(&maxOptin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  if (e != cudaSuccess) return e;
  if (bytes > maxOptin) return cudaErrorInvalidValue;
  e = cudaFuncSetAttribute((const void*)k, cudaFuncAttributeMaxDynamicSharedMemorySize, maxOptin);
  if (e != cudaSuccess) return e;
  g_smemAttr[key] = maxOptin;
  return cudaSuccess;
}

int tiles_blocks_per_sm(const Candidate& c) {
  const TileDesc& D = c.desc;
  TilesKernel k = pick_tiles_kernel(D);
  if (!k) return -1;
  if (ensure_smem(k, c.smemBytes) != cudaSuccess) return -1;
  int nb = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, (const void*)k, (int)D.nthreads,
                                                    (size_t)c.smemBytes) != cudaSuccess)
    return -1;
  return nb;
}

bool tiles_pointers_aligned(const Candidate& c, const void* in, const void* out) {
  const TileDesc& D = c.desc;
  // aligned over-fetch reads whatever alignment the input has, but register blocking of width V on
  // the store side relies on every row displacement being a multiple of V elements
  const bool inOk = D.aof ? ((uintptr_t)in % (D.vblk * D.elt) == 0) : ((uintptr_t)in % (D.in.vec * D.elt) == 0);
  return inOk && ((uintptr_t)out % (D.out.vec * D.elt) == 0);
}

cudaError_t launch_tiles(const Candidate& c, int gridBlocks, const void* in, const PeerPtrs& outs,
                         cudaStream_t stream) {
  const TileDesc& D = c.desc;
  TilesKernel k = pick_tiles_kernel(D);
  if (!k) return cudaErrorInvalidValue;
  cudaError_t e = ensure_smem(k, c.smemBytes);
  if (e != cudaSuccess) return e;
  k<<<gridBlocks, D.nthreads, c.smemBytes, stream>>>(D, (const unsigned char*)in, outs);
  g_launches++;
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------
// contiguous copy
template <typename V, int UNROLL>
__global__ void __launch_bounds__(256)
copy_kernel(const V* __restrict__ in, V* __restrict__ out, size_t n) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  // full groups of UNROLL accesses per thread keep several loads in flight
  for (; i + (UNROLL - 1) * stride < n; i += UNROLL * stride) {
    V v[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; u++) v[u] = __ldcs(in + i + u * stride);
#pragma unroll
    for (int u = 0; u < UNROLL; u++) __stcs(out + i + u * stride, v[u]);
  }
  for (; i < n; i += stride) out[i] = in[i];
}

cudaError_t launch_copy(const void* in, void* out, size_t bytes, int numSM, cudaStream_t stream) {
  if (bytes == 0) return cudaSuccess;
  const int threads = 256;
  // Buffers that miss a 16-byte boundary by the same number of 4-byte words: a few words bring both
  // to the boundary, the rest goes the aligned way (measured: the word kernel alone reaches 2.3 TB/s
  // on such buffers, five sectors per 128-byte warp access and 16 bytes in flight per thread).
  {
    const uintptr_t mi = (uintptr_t)in & 15u, mo = (uintptr_t)out & 15u;
    if (mi != 0 && mi == mo && mi % 4 == 0 && bytes > 64) {
      const size_t head = 16 - mi;
      copy_kernel<uint32_t, 4><<<1, 32, 0, stream>>>((const uint32_t*)in, (uint32_t*)out, head / 4);
      g_launches++;
      cudaError_t e = cudaGetLastError();
      if (e != cudaSuccess) return e;
      return launch_copy((const unsigned char*)in + head, (unsigned char*)out + head, bytes - head, numSM, stream);
    }
  }
  const bool al16 = ((uintptr_t)in % 16 == 0) && ((uintptr_t)out % 16 == 0);
  size_t body = al16 ? bytes / 16 : 0;  // 16-byte words
  if (body && bulk_copy_usable(in, out, bytes)) {
    // large aligned copies go through the bulk copy engine
    cudaError_t e = launch_bulk_copy(in, out, body * 16, numSM, stream);
    if (e != cudaSuccess) return e;
    g_launches++;
  } else if (body) {
    size_t want = (body + threads * 4 - 1) / (threads * 4);
    int grid = (int)(want < (size_t)numSM * 8 ? want : (size_t)numSM * 8);
    copy_kernel<uint4, 4><<<grid, threads, 0, stream>>>((const uint4*)in, (uint4*)out, body);
    g_launches++;
  }
  size_t done = body * 16;
  if (done < bytes) {  // tail (or everything, for pointers that are only 4-byte aligned)
    size_t words = (bytes - done) / 4;
    size_t want = (words + threads * 4 - 1) / (threads * 4);
    int grid = (int)(want < (size_t)numSM * 8 ? want : (size_t)numSM * 8);
    if (grid < 1) grid = 1;
    copy_kernel<uint32_t, 4><<<grid, threads, 0, stream>>>(
        (const uint32_t*)((const unsigned char*)in + done), (uint32_t*)((unsigned char*)out + done), words);
    g_launches++;
  }
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------
// strided row copy (rowcopy_impl.h): one warp per work item, grid-stride
template <int ELT>
__global__ void __launch_bounds__(256)
rowcopy_kernel(const __grid_constant__ RowCopyDesc D, const unsigned char* __restrict__ in,
               unsigned char* __restrict__ out) {
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t wpb = blockDim.x >> 5;
  const uint32_t stride = gridDim.x * wpb;
  for (uint32_t item = blockIdx.x * wpb + (threadIdx.x >> 5); item < D.numItems; item += stride)
    rowcopy_item<ELT>(D, in, out, item, lane);
}

cudaError_t launch_rowcopy(const RowCopyDesc& d, int numSM, const void* in, void* out, cudaStream_t stream) {
  const int threads = 256;
  int nb = 0;
  const void* k = d.elt == 4 ? (const void*)rowcopy_kernel<4> : (const void*)rowcopy_kernel<8>;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, k, threads, 0) != cudaSuccess || nb < 1) nb = 4;
  long long want = ((long long)d.numItems + (threads / 32) - 1) / (threads / 32);
  long long grid = (long long)numSM * nb;
  if (grid > want) grid = want;
  if (grid < 1) grid = 1;
  if (d.elt == 4) rowcopy_kernel<4><<<(int)grid, threads, 0, stream>>>(d, (const unsigned char*)in, (unsigned char*)out);
  else rowcopy_kernel<8><<<(int)grid, threads, 0, stream>>>(d, (const unsigned char*)in, (unsigned char*)out);
  g_launches++;
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------
// one thread per output element
template <typename T>
__global__ void __launch_bounds__(256)
naive_kernel(const __grid_constant__ NaiveDesc d, const T* __restrict__ in, T* __restrict__ out) {
  const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
  for (unsigned long long o = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; o < d.volume;
       o += stride) {
    unsigned long long rem = o, src = 0;
    for (int k = 0; k < d.rank; k++) {
      unsigned long long q = rem / d.odim[k];
      src += (rem - q * d.odim[k]) * d.istride[k];
      rem = q;
    }
    out[o] = in[src];
  }
}

// the same with 32-bit indices (volume < 2^31, so neither an offset nor the loop counter wraps)
template <typename T>
__global__ void __launch_bounds__(256)
naive32_kernel(const __grid_constant__ NaiveDesc d, const T* __restrict__ in, T* __restrict__ out) {
  const uint32_t n = (uint32_t)d.volume;
  const uint32_t stride = gridDim.x * blockDim.x;
  for (uint32_t o = blockIdx.x * blockDim.x + threadIdx.x; o < n; o += stride) {
    uint32_t rem = o, src = 0;
    for (int k = 0; k < d.rank; k++) {
      const uint32_t q = fdiv(rem, d.div[k]);
      src += (rem - q * (uint32_t)d.odim[k]) * (uint32_t)d.istride[k];
      rem = q;
    }
    out[o] = in[src];
  }
}

cudaError_t launch_naive(const NaiveDesc& d, int numSM, const void* in, void* out, cudaStream_t stream) {
  const int threads = 256;
  unsigned long long want = (d.volume + threads - 1) / threads;
  const unsigned long long cap = (unsigned long long)(numSM > 0 ? numSM : 1) * 16;
  int grid = (int)(want < cap ? want : cap);
  if (grid < 1) grid = 1;
  if (d.narrow) {
    if (d.elt == 4) naive32_kernel<uint32_t><<<grid, threads, 0, stream>>>(d, (const uint32_t*)in, (uint32_t*)out);
    else if (d.elt == 2) naive32_kernel<uint16_t><<<grid, threads, 0, stream>>>(d, (const uint16_t*)in, (uint16_t*)out);
    else if (d.elt == 1) naive32_kernel<uint8_t><<<grid, threads, 0, stream>>>(d, (const uint8_t*)in, (uint8_t*)out);
    else naive32_kernel<unsigned long long><<<grid, threads, 0, stream>>>(d, (const unsigned long long*)in, (unsigned long long*)out);
    g_launches++;
    return cudaGetLastError();
  }
  if (d.elt == 4) naive_kernel<uint32_t><<<grid, threads, 0, stream>>>(d, (const uint32_t*)in, (uint32_t*)out);
  else if (d.elt == 2) naive_kernel<uint16_t><<<grid, threads, 0, stream>>>(d, (const uint16_t*)in, (uint16_t*)out);
  else if (d.elt == 1) naive_kernel<uint8_t><<<grid, threads, 0, stream>>>(d, (const uint8_t*)in, (uint8_t*)out);
  else naive_kernel<unsigned long long><<<grid, threads, 0, stream>>>(d, (const unsigned long long*)in, (unsigned long long*)out);
  g_launches++;
  return cudaGetLastError();
}

}  // namespace cuttb
