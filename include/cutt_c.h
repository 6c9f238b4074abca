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
 * dimension kept), 0 = copy kernel (identity only), 1 = cudaMemcpyAsync (identity only). */
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
 * loaded (0 in a healthy run; synchronises the device; -1 on error). */
int cutt_c_copy_timeouts(void);

/* Empties the plan cache (the cuttPlanMeasure winners). */
void cutt_c_clear_plan_cache(void);

/* Writes / reads the plan cache as a text file, so that winners measured in one process are
 * reused by cuttPlan and cuttPlanMeasure in the next.  Keys include the device ordinal. */
int cutt_c_plan_cache_save(const char* path);
int cutt_c_plan_cache_load(const char* path);
int cutt_c_plan_cache_size(void);

const char* cutt_c_version(void);

#ifdef __cplusplus
}
#endif
#endif /* CUTT_C_H */
