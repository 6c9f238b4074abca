/*
 * cutt_c.h - C ABI of the transpose library, for FFI users (ctypes, cgo, JNI, ...).
 *
 * The original cuTT exports only C++-mangled symbols (src/cutt.h:25-103 has no extern "C").
 * Each function below is the unmangled twin of one of them and has identical semantics;
 * result codes are the cuttResult values as plain ints (0 = CUTT_SUCCESS ... 5).
 * Streams are passed as void* (a cudaStream_t).  All data pointers are DEVICE pointers
 * unless a name says "host".
 */
#ifndef CUTT_C_H
#define CUTT_C_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* cuttPlan (src/cutt.h:57-58, src/cutt.cpp:84-184). */
int cutt_c_plan(unsigned int* handle, int rank, const int* dim, const int* permutation,
                size_t sizeofType, void* stream);

/* cuttPlanMeasure (src/cutt.h:75-76, src/cutt.cpp:186-284). Overwrites odata. */
int cutt_c_plan_measure(unsigned int* handle, int rank, const int* dim, const int* permutation,
                        size_t sizeofType, void* stream, void* idata, void* odata);

/* Element sizes 1, 2 and 16 bytes besides 4 and 8.  No counterpart in the original library, which
 * rejects them (src/cutt.cpp:62); every other rule of cuttPlan / cuttPlanMeasure applies
 * unchanged.  The handles are executed and destroyed with cutt_c_execute / cutt_c_destroy (or
 * cuttExecute / cuttDestroy).  Buffers must be aligned for the element type (16-byte elements:
 * 8 bytes suffice); otherwise execution returns CUTT_INVALID_PARAMETER.
 * 16-byte elements move as pairs of 8-byte words through the ordinary plans.  1- and 2-byte
 * elements do so in 4- or 8-byte units when the fastest dimension stays fastest and its byte
 * length is a multiple of 4.  When the elements really move one by one: tensors whose output rows
 * start on 16- or 8-byte and whose input rows start on at least 4-byte boundaries take swizzled
 * shared-memory tiles with a register transpose of 16 x 16 bytes or 8 x 8 half-words (16- or 8-byte
 * stores); all other cases, and buffers that are not aligned for the plan's access widths, an
 * element-wise tiled kernel. */
int cutt_c_plan_ext(unsigned int* handle, int rank, const int* dim, const int* permutation,
                    size_t sizeofType, void* stream);
int cutt_c_plan_measure_ext(unsigned int* handle, int rank, const int* dim, const int* permutation,
                            size_t sizeofType, void* stream, void* idata, void* odata);

/* cuttExecute (src/cutt.h:101, src/cutt.cpp:296-310). */
int cutt_c_execute(unsigned int handle, void* idata, void* odata);

/* cuttDestroy (src/cutt.h:87, src/cutt.cpp:286-294). */
int cutt_c_destroy(unsigned int handle);

/*
 * The functions below have no counterpart in the original library.
 */

/* Writes a one-line JSON description of the plan (method, tile, grid, model estimate). */
int cutt_c_plan_describe(unsigned int handle, char* buf, size_t len);

/* Number of candidate implementations the planner enumerates for this problem on the
 * current device, cheapest model estimate first (0 on invalid input). */
int cutt_c_num_candidates(int rank, const int* dim, const int* permutation, size_t sizeofType);

/* Plan that uses candidate number `index` of that list (benchmark sweeps, tests). */
int cutt_c_plan_candidate(unsigned int* handle, int rank, const int* dim, const int* permutation,
                          size_t sizeofType, void* stream, int index);

/* Plan with an explicit tile parameter choice (tests; see TileParams in planner.h).
 * method: 2 = tiled kernel, 3 = one-thread-per-element kernel, 4 = strided row copy (fastest
 * dimension kept), 0 = copy kernel (identity only), 1 = cudaMemcpyAsync (identity only),
 * 6 = tensor-map (TMA) transpose: tinBytes = tile bytes along the input's fastest dimension (128,
 * 256 or 512), toutBytes = tile bytes along the output's fastest dimension (a multiple of 128, at
 * most 256 elements), stages 2-8, nthreads 128 or 256, loopOrder = which of the two runs fastest
 * in the tile order; CUTT_INVALID_PARAMETER when a stride of the problem is not a multiple of 16
 * bytes, its fused rank exceeds 5 or the fastest dimension does not move. */
int cutt_c_plan_params(unsigned int* handle, int rank, const int* dim, const int* permutation,
                       size_t sizeofType, void* stream, int method, unsigned tinBytes,
                       unsigned toutBytes, unsigned vtargetBytes, int extend, int loopOrder,
                       int maxVecBytes, int maxVBytes, int nthreads, int stages);

/* Convenience for callers holding HOST buffers: plans (cost model, cached), copies hin to the
 * device, executes, copies the result to hout, and synchronises.  Scratch device buffers are
 * owned by the library and reused between calls. */
int cutt_c_transpose_host(int rank, const int* dim, const int* permutation, size_t sizeofType,
                          const void* hin, void* hout);

/* Kernel launches issued by the library since it was loaded. */
unsigned long long cutt_c_launch_count(void);

/* The copy kernel used for identity permutations waits on hardware barriers with a poll limit;
 * this returns how many such waits have run out on the current device since the library was
 * loaded (0 in a healthy run; waits for all work on the device first; -1 on error). */
int cutt_c_copy_timeouts(void);

/*
 * Device-to-device copy of `bytes` bytes that allocates nothing (no counterpart in the original
 * library, whose identity case calls cudaMemcpyAsync).
 *
 * Meant for hosts that cannot allocate device memory at the moment they need the copy - the
 * device's memory belongs to their own memory manager, or they run in a loop where the
 * device-wide synchronisation of an allocation is not tolerable.  The kernel is the bulk-copy
 * kernel used for identity permutations; the status words it needs are a fixed 1 KB array inside
 * the library image (256 words, one per thread block: a launch uses one block per SM and at most
 * 256 blocks), which every GPU that loads the library holds until the process exits.
 *
 * Rules: src and dst are device pointers aligned to 16 bytes, bytes is a multiple of 16 and at
 * most 2^40; anything else returns CUTT_INVALID_PARAMETER (2) with a message on stderr for the
 * two size limits.  The first call on a device looks up the array's device address and sets the
 * kernel's shared-memory limit; make that first call before any stream capture begins.  All
 * calls share the one array and each call clears it on its stream before its kernel runs, so two
 * calls whose kernels overlap on the GPU (different streams) race on it: issue them on one stream
 * or order them with events.  The copy is asynchronous on `stream`.
 */
int cutt_c_copy_noalloc(const void* src, void* dst, size_t bytes, void* stream);

/* Thread blocks whose hardware-barrier wait ran out during the most recent cutt_c_copy_noalloc on
 * the current device (0 in a healthy run; -1 before the first call or on error).  Waits for all
 * work on the device, on every stream, before it reads the status words. */
int cutt_c_copy_noalloc_timeouts(void);

/* Test aid: while on (on != 0) every tiled plan is built with 64-bit row offsets, the kernel
 * variant that otherwise only tiles spanning 2^32 elements or more select.  Affects plans made
 * afterwards; meant for test processes, not thread-safe against concurrent planning. */
void cutt_c_debug_force_wide(int on);

/* Empties the plan cache (the cuttPlanMeasure winners). */
void cutt_c_clear_plan_cache(void);

/* Writes / reads the plan cache as a text file, so that winners measured in one process are
 * reused by cuttPlan and cuttPlanMeasure in the next.  Keys include the device ordinal.
 * Loading accepts only files with this format's version header and skips entries whose fields are
 * out of range; a loaded entry is a hint that cuttPlan re-validates against the problem (a copy
 * method is never used for a non-identity permutation).  cuttPlanMeasure served from the cache
 * times nothing but still overwrites odata and synchronises the device, like the original
 * (src/cutt.cpp:240-250). */
int cutt_c_plan_cache_save(const char* path);
int cutt_c_plan_cache_load(const char* path);
int cutt_c_plan_cache_size(void);

const char* cutt_c_version(void);

#ifdef __cplusplus
}
#endif
#endif /* CUTT_C_H */
