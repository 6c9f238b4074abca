// A host program written against the ORIGINAL cuTT interface only (cutt.h, four functions,
// device pointers), as in the usage example of the original README (README.md:78-120).
// It is compiled with g++ and linked with  -lcutt -lcudart  exactly like a user of the original
// libcutt.a would do; nothing in it knows about this repository's extensions.
//
// Exit code 0: the transposed tensor equals a host nested-loop permutation bit for bit.
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>
#include "cutt.h"

#define CUDA_OK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { \
  fprintf(stderr, "CUDA error %s at line %d\n", cudaGetErrorString(e_), __LINE__); return 2; } } while (0)
#define CUTT_OK(x) do { cuttResult r_ = (x); if (r_ != CUTT_SUCCESS) { \
  fprintf(stderr, "cuTT error %d at line %d\n", (int)r_, __LINE__); return 3; } } while (0)

template <typename T>
static int run(std::vector<int> dim, std::vector<int> perm, bool measure) {
  const int rank = (int)dim.size();
  size_t vol = 1;
  for (int d : dim) vol *= (size_t)d;
  std::vector<T> hin(vol), hout(vol), ref(vol);
  unsigned long long s = 88172645463325252ull;
  for (size_t i = 0; i < vol; i++) { s ^= s << 13; s ^= s >> 7; s ^= s << 17; hin[i] = (T)s; }
  // host nested loop: out[o] = in[sum_k coord_k * instride(perm[k])]
  std::vector<size_t> is(rank), od(rank), ois(rank);
  size_t acc = 1;
  for (int i = 0; i < rank; i++) { is[i] = acc; acc *= dim[i]; }
  for (int k = 0; k < rank; k++) { od[k] = dim[perm[k]]; ois[k] = is[perm[k]]; }
  for (size_t o = 0; o < vol; o++) {
    size_t rem = o, src = 0;
    for (int k = 0; k < rank; k++) { src += (rem % od[k]) * ois[k]; rem /= od[k]; }
    ref[o] = hin[src];
  }
  T *din = nullptr, *dout = nullptr;
  CUDA_OK(cudaMalloc(&din, vol * sizeof(T)));
  CUDA_OK(cudaMalloc(&dout, vol * sizeof(T)));
  CUDA_OK(cudaMemcpy(din, hin.data(), vol * sizeof(T), cudaMemcpyHostToDevice));
  cudaStream_t stream;
  CUDA_OK(cudaStreamCreate(&stream));
  cuttHandle plan;
  if (measure) CUTT_OK(cuttPlanMeasure(&plan, rank, dim.data(), perm.data(), sizeof(T), stream, din, dout));
  else CUTT_OK(cuttPlan(&plan, rank, dim.data(), perm.data(), sizeof(T), stream));
  CUDA_OK(cudaMemset(dout, 0xFF, vol * sizeof(T)));
  CUTT_OK(cuttExecute(plan, din, dout));
  CUDA_OK(cudaStreamSynchronize(stream));
  CUTT_OK(cuttDestroy(plan));
  if (cuttDestroy(plan) != CUTT_INVALID_PLAN) return 4;
  CUDA_OK(cudaMemcpy(hout.data(), dout, vol * sizeof(T), cudaMemcpyDeviceToHost));
  CUDA_OK(cudaFree(din));
  CUDA_OK(cudaFree(dout));
  CUDA_OK(cudaStreamDestroy(stream));
  if (memcmp(hout.data(), ref.data(), vol * sizeof(T)) != 0) { fprintf(stderr, "mismatch\n"); return 1; }
  return 0;
}

int main() {
  int rc;
  // the README example of the original library, both ways of planning, both element sizes
  if ((rc = run<double>({31, 549, 2, 3}, {3, 0, 2, 1}, false))) return rc;
  if ((rc = run<double>({31, 549, 2, 3}, {3, 0, 2, 1}, true))) return rc;
  if ((rc = run<float>({31, 549, 2, 3}, {3, 0, 2, 1}, false))) return rc;
  if ((rc = run<float>({43, 67}, {1, 0}, true))) return rc;
  if ((rc = run<double>({24, 32, 16, 36, 9}, {4, 1, 3, 2, 0}, false))) return rc;
  if ((rc = run<float>({2, 5, 9, 12}, {0, 1, 2, 3}, false))) return rc;  // identity
  // invalid input is rejected with the original codes
  int dim[2] = {4, 1}, perm[2] = {1, 0};
  cuttHandle h;
  if (cuttPlan(&h, 2, dim, perm, 4, 0) != CUTT_INVALID_PARAMETER) return 5;
  printf("drop-in example ok\n");
  return 0;
}
