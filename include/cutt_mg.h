/*
 * cutt_mg.h - multi-GPU extension of the transpose library (one box, up to 8 GPUs).
 *
 * NOTHING in this header has a counterpart in the original cuTT, which is single-GPU
 * (no peer access, NCCL or MPI anywhere in its tree); cutt.h is unchanged by it.
 *
 * Model.  A tensor (dim[0] fastest, cuTT conventions) is sharded over `world` GPUs:
 *   - the INPUT along its slowest dimension dim[rank-1]: GPU g holds the contiguous slab with
 *     that extent divided by world;
 *   - the OUTPUT along ITS slowest dimension (input dimension permutation[rank-1]), same way.
 * Two modes follow from the permutation:
 *   mode 0 "slab":        permutation[rank-1] == rank-1.  Every GPU permutes its own slab; there
 *                          is no communication and cutt_mg_execute only touches local memory.
 *   mode 1 "all-to-all":  the sharded dimension moves.  Every GPU reads its local slab and STORES
 *                          each tile straight into the output slab of the GPU that owns it
 *                          (peer-to-peer stores over NVLink from inside the transpose kernel; no
 *                          NCCL, no staging copy, loads are local only).
 * Both extents must be divisible by world, otherwise planning returns CUTT_INVALID_PARAMETER.
 *
 * Process model: one rank per GPU.  Ranks may be threads or processes.  With processes, each
 * rank exports its output slab with cutt_mg_ipc_export, the tokens travel through any
 * host channel (torch.distributed, MPI, a pipe), and cutt_mg_ipc_open maps a peer's slab.  The
 * buffer may sit anywhere inside a larger allocation (pooling allocators): the token records its
 * offset and cutt_mg_ipc_open returns the address of the buffer itself.
 * Within one process cudaDeviceEnablePeerAccess (or cutt_mg_enable_peer_access) is enough.
 *
 * Completion: cutt_mg_execute is asynchronous on the plan's stream.  A rank's output slab is
 * complete when EVERY rank's kernel has finished, so callers synchronise their stream and then
 * meet at a host barrier before reading the output (and before the next execute overwrites a
 * buffer that peers may still be writing).  The library never spins on device flags.
 *
 * Result codes are cuttResult values as ints.
 */
#ifndef CUTT_MG_H
#define CUTT_MG_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CUTT_MG_MAX_WORLD 8
#define CUTT_MG_IPC_BYTES 80   /* CUDA IPC handle (64) + offset of the buffer inside its allocation (8) + reserved (8) */

/* Plan for rank `me` of `world` on the current device.  dim/permutation describe the GLOBAL
 * tensor.  The handle lives in the same table as cuttPlan's (destroy with cuttDestroy /
 * cutt_c_destroy). */
int cutt_mg_plan(unsigned int* handle, int rank, const int* dim, const int* permutation,
                 size_t sizeofType, void* stream, int world, int me);

/* As above, choosing the implementation by timing candidates.  idata: local input slab;
 * odata[h], h < world: output slab of rank h as addressable from this device (odata[me] local).
 * Overwrites the output slabs.  All ranks should call it at the same time (the timings include
 * the peers' traffic). */
int cutt_mg_plan_measure(unsigned int* handle, int rank, const int* dim, const int* permutation,
                         size_t sizeofType, void* stream, int world, int me, void* idata,
                         void* const* odata);

/* Candidate implementations the planner enumerates for rank `me`'s part, cheapest model estimate
 * first (0 on invalid input), and a plan that uses candidate number `index` of that list.  The
 * list depends on the problem only, so every rank sees the same list: a job can time candidate
 * 0, 1, 2, ... on all ranks AT THE SAME TIME (barrier, execute, barrier), take the slowest rank's
 * time and so choose one plan for the whole job, which is what an all-to-all needs - a plan's
 * speed depends on what the other GPUs are sending meanwhile.  cutt_mg_plan_measure, in
 * contrast, lets each rank time its candidates on its own. */
int cutt_mg_num_candidates(int rank, const int* dim, const int* permutation, size_t sizeofType,
                           int world, int me);
int cutt_mg_plan_candidate(unsigned int* handle, int rank, const int* dim, const int* permutation,
                           size_t sizeofType, void* stream, int world, int me, int index);

/* 0 slab, 1 all-to-all; negative: not a multi-GPU plan. */
int cutt_mg_mode(unsigned int handle);

/* Elements of one slab (input and output slabs have the same volume). */
long long cutt_mg_local_volume(unsigned int handle);

/* Enqueue this rank's part.  odata as in cutt_mg_plan_measure (only odata[me] is used in mode 0). */
int cutt_mg_execute(unsigned int handle, void* idata, void* const* odata);

/* Inter-process sharing of a device buffer (wraps the CUDA IPC calls). */
int cutt_mg_ipc_export(void* devptr, unsigned char token[CUTT_MG_IPC_BYTES]);
int cutt_mg_ipc_open(const unsigned char token[CUTT_MG_IPC_BYTES], void** devptr);
int cutt_mg_ipc_close(void* devptr);

/* Single-process helper: enables peer access from the current device to devices 0..world-1. */
int cutt_mg_enable_peer_access(int world);

#ifdef __cplusplus
}
#endif
#endif /* CUTT_MG_H */
