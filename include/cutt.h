/*
 * cutt.h - tensor transpose (permutation) plans for CUDA devices.
 *
 * Source-compatible with the public header of cuTT 1.1 (ap-hynninen/cutt, src/cutt.h:25-103):
 * same type names, same enumerators in the same order, same four functions with the same
 * C++ signatures (and therefore the same mangled symbols), so host code written against the
 * original header compiles and links against this library's libcutt.a unchanged.
 *
 * Conventions (original README.md:94-97): dim[0] is the fastest-varying dimension; the output
 * tensor has dimensions outDim[i] = dim[permutation[i]]; element size is 4 or 8 bytes; the
 * operation is out of place.  A plan belongs to the device that was current when it was made
 * and launches on the stream it was made with.
 */
#ifndef CUTT_H
#define CUTT_H

#include <cuda_runtime.h>

/* Opaque plan identifier. */
typedef unsigned int cuttHandle;

/* Status codes (values 0..5, fixed order). */
typedef enum cuttResult_t {
  CUTT_SUCCESS,            /* no error */
  CUTT_INVALID_PLAN,       /* the handle names no live plan */
  CUTT_INVALID_PARAMETER,  /* bad rank, dimension, permutation, element size or buffer */
  CUTT_INVALID_DEVICE,     /* the current device is not the plan's device */
  CUTT_INTERNAL_ERROR,     /* a CUDA call or an internal step failed */
  CUTT_UNDEFINED_ERROR,    /* anything else */
} cuttResult;

/*
 * Build a plan with the built-in cost model.
 *   handle       receives the plan identifier
 *   rank         number of dimensions (>= 2)
 *   dim          extents, dim[0] fastest (each >= 2)
 *   permutation  permutation[i] is the input dimension that becomes output dimension i
 *   sizeofType   element size in bytes: 4 or 8
 *   stream       stream the plan will execute on (0 for the default stream)
 */
cuttResult cuttPlan(cuttHandle* handle, int rank, int* dim, int* permutation, size_t sizeofType,
  cudaStream_t stream);

/*
 * Build a plan by timing candidate implementations on the device.  idata and odata are
 * device buffers of prod(dim) elements; odata is overwritten and the device is synchronised.
 */
cuttResult cuttPlanMeasure(cuttHandle* handle, int rank, int* dim, int* permutation, size_t sizeofType,
  cudaStream_t stream, void* idata, void* odata);

/* Release a plan. */
cuttResult cuttDestroy(cuttHandle handle);

/* Enqueue the permutation idata -> odata on the plan's stream (asynchronous, out of place). */
cuttResult cuttExecute(cuttHandle handle, void* idata, void* odata);

#endif /* CUTT_H */
