// extern "C" doorway into the ORIGINAL cuTT library, for the test-suite and the benchmark's
// reference leg only.  The original exports C++-mangled symbols (its src/cutt.h has no
// extern "C"); this shim is compiled together with the unmodified original sources (see
// build_ref.py) and forwards to them so that ctypes can call the real thing.
#include "cutt.h"  // the original header, found through -I<reference>/src

extern "C" {
int ref_cutt_plan(unsigned int* h, int rank, int* dim, int* perm, size_t elt, void* stream) {
  return (int)cuttPlan(h, rank, dim, perm, elt, (cudaStream_t)stream);
}
int ref_cutt_plan_measure(unsigned int* h, int rank, int* dim, int* perm, size_t elt, void* stream,
                          void* idata, void* odata) {
  return (int)cuttPlanMeasure(h, rank, dim, perm, elt, (cudaStream_t)stream, idata, odata);
}
int ref_cutt_execute(unsigned int h, void* idata, void* odata) { return (int)cuttExecute(h, idata, odata); }
int ref_cutt_destroy(unsigned int h) { return (int)cuttDestroy(h); }
}
