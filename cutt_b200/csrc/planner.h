// Plan builder: canonical form of a permutation, candidate tile enumeration, cost model.
// Pure host C++ (no CUDA calls) so that it is unit-tested without a GPU.
//
// Replaces reduceRanks (src/cuttplan.cpp:63-126), TensorSplit and the five
// create*Plans enumerators (src/cuttplan.cpp:172-698) and the MWP-CWP cycle model
// (src/cuttGpuModel.cpp) of the reference.
#pragma once
#include <stdint.h>
#include <set>
#include <string>
#include <vector>
#include "permute_desc.h"
#include "rowcopy_impl.h"
#include "tma_transpose.h"
#include "tile2d.h"

namespace cuttb {

struct DeviceInfo {
  int numSM = 148;
  int maxSmemPerBlock = 227 * 1024;  // opt-in dynamic shared memory per block
  int smemPerSM = 228 * 1024;
  int maxThreadsPerSM = 2048;
  double hbmGBs = 6500.0;            // attainable copy bandwidth used by the cost model
  bool tmaLoads = true;              // tensor-map loads available (the driver exports the encoder)
};

// A permutation as a strided copy, dimensions sorted by input stride, fused.
struct Problem {
  int rank = 0;
  int elt = 4;
  int64_t d[kMaxDims];
  int64_t is[kMaxDims];
  int64_t os[kMaxDims];
  int64_t inBase = 0, outBase = 0;
  int peerDim = -1;   // canonical dimension whose coordinate selects the destination GPU
  int peerRot = 0;    // this GPU's rank: first destination of the balanced tile order (TileParams::peerOrder)
  int64_t volume = 0;
  int64_t inElems = 0;  // elements of the input buffer this problem reads from
  bool identity = false;  // one contiguous run on both sides: a plain copy
};

// rank, dims, strides (elements). Drops unit dims, sorts by input stride, fuses runs that
// are contiguous on both sides.  peerDim (index into the given dims, or -1) is never fused.
// Returns false if the fused rank exceeds kMaxDims.
bool canonicalize(int rank, const int64_t* d, const int64_t* is, const int64_t* os, int elt,
                  int peerDim, Problem& P);

// cuTT convention (dim[0] fastest, outDim[i] = dim[perm[i]]) -> Problem.
bool problem_from_cutt(int rank, const int* dim, const int* perm, int elt, Problem& P);

// The same for element sizes 1, 2, 4, 8 and 16 bytes (extension entry points).  16-byte elements
// become pairs of 8-byte words.  1- and 2-byte elements are re-stated in 8- or 4-byte units when
// the fastest dimension stays fastest and its byte length allows; otherwise P.elt stays 1 or 2.
bool problem_from_cutt_ext(int rank, const int* dim, const int* perm, int eltBytes, Problem& P);

// A tensor sharded over `world` GPUs of one box: the input along its slowest dimension, the
// output along ITS slowest dimension (= input dimension perm[rank-1]), both in equal parts.
struct ShardInfo {
  int mode = -1;            // 0 slab: each GPU permutes its own slab, no communication
                            // 1 all-to-all: each GPU writes pieces of every GPU's output slab
                            // -1 not shardable this way (extents not divisible)
  int64_t localVolume = 0;  // elements of one input slab (= one output slab)
  int localDim[32];         // extents of the local input slab (mode 0: a plain cuTT problem)
};

// Builds rank `me`'s part of the sharded permutation as a strided-copy Problem.  In mode 1 the
// Problem carries a peer dimension: its coordinate names the GPU whose output slab is written.
bool problem_from_cutt_sharded(int rank, const int* dim, const int* perm, int elt, int world, int me,
                               Problem& P, ShardInfo& info);

// A slab of the input along its slowest dimension (extent `chunk` instead of dim[rank-1]) permuted
// INTO the full output tensor: input strides of the slab, output strides of the whole tensor.
// Used to pipeline host transfers with the kernel.
bool problem_from_cutt_chunk(int rank, const int* dim, const int* perm, int elt, int chunk, Problem& P);

enum Method : int {
  kMethodCopy = 0,     // identity after fusion: contiguous copy kernel
  kMethodMemcpy = 1,   // identity: cudaMemcpyAsync device-to-device
  kMethodTiles = 2,    // tiled permutation kernel (cp.async staged)
  kMethodNaive = 3,    // one thread per output element (fallback for rank > kMaxDims, debug)
  kMethodRowCopy = 4,  // strided copy of contiguous rows with register shifting (rowcopy_impl.h)
  kMethodSmall = 5,    // 1- and 2-byte elements moved one by one (small_elt_impl.h)
  kMethodTma = 6,      // tensor-map box loads into swizzled shared memory (tma_transpose.h)
  kMethodT2d = 7,      // two-dimensional tiles, cp.async loads into swizzled shared memory (tile2d.h)
};

struct TileParams {
  uint32_t tinBytes = 256;     // target bytes per input run
  uint32_t toutBytes = 256;    // target bytes per output run
  uint32_t vtargetBytes = 16384;  // target tile volume
  int extend = 0;              // which dimension grows when the tile is below target: 0 next in output order, 1 next in input order
  int nthreads = 256;
  int stages = 2;
  int maxVecBytes = 16;        // widest global access
  int maxVBytes = 16;          // widest shared-memory vector of the register-blocked store side
  int cutInRun = 0;            // end the input run before the dimension that starts the output run, so that
                               // dimension gets a padded (bank-conflict-free) shared-memory stride
  int oneTilePerBlock = 0;     // launch one block per tile (no persistent loop); for small tiles
  int allowAof = 1;            // aligned over-fetch loads when input rows are not 16-byte aligned
  int loopOrder = 0;           // tile index runs fastest along 0: input order, 1: output order
  int groupIn = 1;             // neighbouring tiles along the input run's chunked dimension taken first
  int groupOut = 1;            // then this many along the output run's chunked dimension
  int peerOrder = 0;           // multi-GPU all-to-all plans: 0 = the destination GPU is one more digit of
                               // the tile index at its place in the loop order (every GPU works through
                               // destination 0, then 1, ...: all GPUs write to the same destination at the
                               // same time); 1 = the destination is the FASTEST digit and GPU r starts
                               // with destination r, so the blocks of one GPU spread their stores over
                               // all destinations and no destination receives from everybody at once
};

constexpr int kNumFeatures = 32;

struct Candidate {
  Method method = kMethodTiles;
  float feat[kNumFeatures] = {0};  // inputs of the cost model (see candidate_features in planner.cpp)
  TileParams params;
  TileDesc desc;
  RowCopyDesc rc;              // kMethodRowCopy only
  TmaDesc tma;                 // kMethodTma only
  TmaMapRecipe tmaMap;         // kMethodTma only
  T2dDesc t2d;                 // kMethodT2d only
  int smemBytes = 0;
  int blocksPerSM = 1;
  int gridBlocks = 0;
  double cost = 0.0;           // model estimate, seconds
  std::string label;           // short human-readable description
};

// Builds the descriptor for one parameter choice; false if it is illegal
// (too much shared memory, more than two partial dimensions, ...).  With `seenExtents`, also
// false when the same tile extents and launch options were already built (enumeration dedup).
bool build_tile(const Problem& P, const TileParams& tp, const DeviceInfo& dev, Candidate& out,
                std::set<std::string>* seenExtents = nullptr);

// Tensor-map transpose candidate (tma_transpose.h): tile of taBytes along dimension 0 by tbElems
// along the output's fastest dimension; false if the problem is outside the class (strides not
// multiples of 16 bytes, fused rank above 5, fastest dimension kept, ...).  The parameters travel
// in a TileParams so that the plan cache stores them like any other choice:
// tinBytes = bytes along dimension 0, toutBytes = bytes along dimension p, stages, nthreads,
// loopOrder = which of the two varies fastest in the tile index.
bool build_tma(const Problem& P, const TileParams& tp, const DeviceInfo& dev, Candidate& out);

// Two-dimensional tile candidate (tile2d.h): tinBytes = tile bytes along dimension 0 (128 or 256),
// toutBytes = tile extent along the output's fastest dimension times the element size (32 or 64
// elements), nthreads 128 or 256, loopOrder = which of the two runs fastest in the tile order,
// maxVecBytes < 16 selects the plain narrow access modes, extend = 1 forces the shift / shear modes
// (any buffer alignment).  False outside the class.
bool build_t2d(const Problem& P, const TileParams& tp, const DeviceInfo& dev, Candidate& out);

// The tile2d candidate the extension entry points use for 2-byte elements (rows of the output on
// 16-byte boundaries, rows of the input on at least 4-byte boundaries); false if not applicable.
bool build_t2d_small(const Problem& P, const DeviceInfo& dev, Candidate& out);

// Row-copy candidate for problems whose fastest dimension is kept; false if not applicable.
bool build_rowcopy(const Problem& P, const DeviceInfo& dev, Candidate& out);

// All distinct candidates for a problem, cheapest model cost first.
std::vector<Candidate> enumerate_candidates(const Problem& P, const DeviceInfo& dev);

// Model estimate (seconds) for a tiles candidate (fitted model; closed form for small tensors).
double analytic_cost(const Problem& P, const Candidate& c, const DeviceInfo& dev);
double model_cost(const Problem& P, const Candidate& c, const DeviceInfo& dev);

// Test aid: while on, every tile is built with 64-bit row offsets (the kernel variant that tiles
// spanning 2^32 elements and more need).  Not thread-safe; meant for test processes only.
void debug_force_wide_offsets(bool on);

// One-line JSON description (used by tests and by CUTT_VERBOSE).
std::string describe(const Problem& P, const Candidate& c);

}  // namespace cuttb
