// Launch interface of the sm_100a permutation kernels (kernels.cu).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include "planner.h"

namespace cuttb {

struct PeerPtrs {
  unsigned char* p[kMaxPeers];
};

// One thread per output element; any rank up to 32.  Fallback, cross-check, and the quickest way
// through tensors of a few hundred kilobytes, whose time is launch and one memory round trip.
struct NaiveDesc {
  int rank;
  int elt;
  unsigned long long volume;
  unsigned long long odim[32];     // extents in output order
  unsigned long long istride[32];  // input stride of the k-th output dimension
  int narrow;                      // volume < 2^31: 32-bit indices, divisions by multiplication
  FastDiv div[32];                 // of odim[k]
};

// Resident blocks per SM of the tiled kernel for this candidate (also raises the kernel's
// dynamic shared-memory limit).  <= 0 on error.
int tiles_blocks_per_sm(const Candidate& c);

// Effective vector widths the kernel can use with these pointers (elements).
bool tiles_pointers_aligned(const Candidate& c, const void* in, const void* out);

cudaError_t launch_tiles(const Candidate& c, int gridBlocks, const void* in, const PeerPtrs& outs,
                         cudaStream_t stream);
cudaError_t launch_copy(const void* in, void* out, size_t bytes, int numSM, cudaStream_t stream);
cudaError_t launch_naive(const NaiveDesc& d, int numSM, const void* in, void* out, cudaStream_t stream);

// Bulk-copy-engine copy (bulk_copy.cu): both pointers 16-byte aligned, bytes16 a multiple of 16.
bool bulk_copy_usable(const void* in, const void* out, size_t bytes);
cudaError_t launch_bulk_copy(const void* in, void* out, size_t bytes16, int numSM, cudaStream_t stream);
cudaError_t launch_bulk_copy_with_status(const void* in, void* out, size_t bytes16, int numSM,
                                         unsigned int* status, cudaStream_t stream);
int bulk_copy_timeouts();
// Device word of the current device in which kernels count bounded waits that ran out (allocated
// on first use; null if that fails).
unsigned int* bulk_copy_status_word();

// Tensor-map (TMA) transpose (tma_transpose.cu, tma_transpose.h).
bool tma_supported();                       // the driver exports cuTensorMapEncodeTiled
int tma_blocks_per_sm(const TmaDesc& D);    // resident blocks per SM (<= 0 on error)
bool tma_map_encodable(const TmaDesc& D, const TmaMapRecipe& R);
cudaError_t launch_tma(const TmaDesc& D, const TmaMapRecipe& R, int gridBlocks, const void* in, void* out,
                       cudaStream_t stream);
cudaError_t launch_rowcopy(const RowCopyDesc& d, int numSM, const void* in, void* out, cudaStream_t stream);

// Two-dimensional tile transpose with swizzled shared memory (tile2d.cu, tile2d.h).
int t2d_blocks_per_sm(const T2dDesc& D);
bool t2d_pointers_aligned(const T2dDesc& D, const void* in, const void* out);
cudaError_t launch_t2d(const T2dDesc& D, const void* in, void* out, cudaStream_t stream);

// Permutation of 1- or 2-byte elements, one tile per block (small_elt.cu).
struct SmallDesc;
cudaError_t launch_small(const SmallDesc& d, const void* in, void* out, cudaStream_t stream);

// Number of kernel launches issued by this library since load (for benchmarks' accounting).
unsigned long long launch_count();
void count_launch();

}  // namespace cuttb
