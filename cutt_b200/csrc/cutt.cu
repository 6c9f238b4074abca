// Public API: cuttPlan / cuttPlanMeasure / cuttExecute / cuttDestroy (C++ symbols of
// include/cutt.h) and their extern "C" twins (include/cutt_c.h).
//
// Behaviour follows src/cutt.cpp of the original library:
//   validation rules                         src/cutt.cpp:59-82
//   handles 0,1,2,... consumed once the input is valid, even if planning fails later   :96-97
//   cuttPlanMeasure rejects idata == odata, overwrites odata, synchronises the device   :193,240-250
//   cuttExecute: unknown handle -> INVALID_PLAN, idata == odata -> INVALID_PARAMETER,
//                other current device -> INVALID_DEVICE                                 :296-308
// Differences (supersets): CUDA failures return CUTT_INTERNAL_ERROR instead of exiting the
// process; the handle table and the plan cache are guarded by a mutex; plans own no device
// memory; measured winners are remembered in an LRU plan cache that cuttPlan consults.
#include "../../include/cutt.h"
#include "../../include/cutt_c.h"
#include "../../include/cutt_mg.h"

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <list>
#include <memory>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "kernels.h"
#include <algorithm>
#include "planner.h"
#include "small_elt_impl.h"

using namespace cuttb;

namespace {

struct Plan {
  int device = 0;
  cudaStream_t stream = 0;
  int elt = 4;
  size_t bytes = 0;
  Method method = kMethodTiles;
  Problem prob;
  Candidate cand;          // tiled candidate in use
  int grid = 0;
  bool haveFallback = false;
  Candidate fallback;      // same tile with element-sized accesses, for unaligned pointers
  int fallbackGrid = 0;
  NaiveDesc naive{};
  int numSM = 0;           // set from the device when the plan is made
  std::string note;
  // multi-GPU plans (cutt_mg.h)
  int mgWorld = 0;
  int mgMe = 0;
  int mgMode = -1;
  long long mgLocalVolume = 0;
  // plans of the extension entry points (element sizes 1, 2, 16)
  int extBytes = 0;        // the caller's element size; 0 for ordinary plans
  SmallDesc small{};       // kMethodSmall
  bool extSmallFallback = false;   // 2-byte tile2d plans: `small` is filled and serves unaligned buffers
};

struct CachedChoice {
  Method method;
  TileParams params;
};

// LRU map: problem key -> choice found by measurement.
class PlanCache {
 public:
  explicit PlanCache(size_t cap) : cap_(cap) {}
  bool get(const std::string& k, CachedChoice& out) {
    auto it = map_.find(k);
    if (it == map_.end()) return false;
    order_.splice(order_.begin(), order_, it->second);
    out = it->second->second;
    return true;
  }
  void put(const std::string& k, const CachedChoice& c) {
    auto it = map_.find(k);
    if (it != map_.end()) {
      it->second->second = c;
      order_.splice(order_.begin(), order_, it->second);
      return;
    }
    order_.emplace_front(k, c);
    map_[k] = order_.begin();
    while (map_.size() > cap_) {
      map_.erase(order_.back().first);
      order_.pop_back();
    }
  }
  void clear() { map_.clear(); order_.clear(); }
  size_t size() const { return map_.size(); }
  // least recently used first, so that re-inserting in this order restores the recency order
  template <typename F> void for_each_oldest_first(F f) const {
    for (auto it = order_.rbegin(); it != order_.rend(); ++it) f(it->first, it->second);
  }

 private:
  size_t cap_;
  std::list<std::pair<std::string, CachedChoice>> order_;
  std::unordered_map<std::string, std::list<std::pair<std::string, CachedChoice>>::iterator> map_;
};

std::mutex g_mutex;
// Plans are shared: cuttExecute copies the pointer under the lock and keeps the plan alive while it
// launches, so a concurrent cuttDestroy cannot free it under the launch.
std::unordered_map<cuttHandle, std::shared_ptr<Plan>> g_plans;
cuttHandle g_nextHandle = 0;
std::unordered_map<int, DeviceInfo> g_devices;

size_t env_size(const char* name, size_t dflt) {
  const char* v = getenv(name);
  if (!v || !*v) return dflt;
  long long x = atoll(v);
  return x > 0 ? (size_t)x : dflt;
}
bool env_flag(const char* name) {
  const char* v = getenv(name);
  return v && *v && strcmp(v, "0") != 0;
}

PlanCache& plan_cache() {
  static PlanCache cache(env_size("CUTT_PLAN_CACHE_SIZE", 4096));
  return cache;
}

bool device_info(int& dev, DeviceInfo& info) {
  if (cudaGetDevice(&dev) != cudaSuccess) return false;
  auto it = g_devices.find(dev);
  if (it != g_devices.end()) { info = it->second; return true; }
  int v = 0;
  DeviceInfo d;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return false;
  d.numSM = v;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) return false;
  d.maxSmemPerBlock = v;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev) != cudaSuccess) return false;
  d.smemPerSM = v;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrMaxThreadsPerMultiProcessor, dev) != cudaSuccess) return false;
  d.maxThreadsPerSM = v;
  d.tmaLoads = tma_supported() && !env_flag("CUTT_NO_TMA");
  g_devices[dev] = d;
  info = d;
  return true;
}

// src/cutt.cpp:59-82
cuttResult check_input(int rank, const int* dim, const int* perm, size_t elt, bool ext = false) {
  if (elt != 4 && elt != 8 && !(ext && (elt == 1 || elt == 2 || elt == 16))) return CUTT_INVALID_PARAMETER;
  if (rank <= 1) return CUTT_INVALID_PARAMETER;
  if (!dim || !perm) return CUTT_INVALID_PARAMETER;
  for (int i = 0; i < rank; i++)
    if (dim[i] <= 1) return CUTT_INVALID_PARAMETER;
  std::vector<char> seen(rank, 0);
  for (int i = 0; i < rank; i++) {
    if (perm[i] < 0 || perm[i] >= rank || seen[perm[i]]) return CUTT_INVALID_PARAMETER;
    seen[perm[i]] = 1;
  }
  return CUTT_SUCCESS;
}

std::string problem_key(int dev, int rank, const int* dim, const int* perm, size_t elt) {
  std::string k = std::to_string(dev) + "/" + std::to_string(elt) + "/";
  for (int i = 0; i < rank; i++) k += std::to_string(dim[i]) + ",";
  k += "/";
  for (int i = 0; i < rank; i++) k += std::to_string(perm[i]) + ",";
  return k;
}

void fill_naive(Plan& p, int rank, const int* dim, const int* perm) {
  NaiveDesc& n = p.naive;
  memset(&n, 0, sizeof n);
  n.rank = rank;
  n.elt = p.elt;
  unsigned long long is[32], acc = 1;
  for (int i = 0; i < rank; i++) { is[i] = acc; acc *= (unsigned long long)dim[i]; }
  n.volume = acc;
  for (int k = 0; k < rank; k++) { n.odim[k] = dim[perm[k]]; n.istride[k] = is[perm[k]]; }
  n.narrow = acc < (1ull << 31) ? 1 : 0;
  if (n.narrow)
    for (int k = 0; k < rank; k++) n.div[k] = make_fastdiv((uint32_t)n.odim[k]);
}

// Occupancy-based grid for a tiled candidate; false if the kernel cannot be configured.
bool finalize_tiles(const DeviceInfo& dev, Candidate& c, int& grid) {
  int nb = tiles_blocks_per_sm(c);
  if (nb <= 0) return false;
  c.blocksPerSM = nb;
  long long g = (long long)dev.numSM * nb;
  if (g > (long long)c.desc.numTiles || c.params.oneTilePerBlock) g = c.desc.numTiles;
  grid = (int)g;
  c.gridBlocks = grid;
  return true;
}

cudaError_t run_plan(const Plan& p, const void* in, void* out, cudaStream_t stream,
                     void* const* peers = nullptr) {
  if (p.mgMode == 1) {
    // all-to-all: the kernel picks the destination slab per tile; element-aligned fallback
    // when any of the slabs is not aligned for the plan's vector width
    if (p.method != kMethodTiles || !peers) return cudaErrorInvalidValue;
    PeerPtrs pp;
    bool aligned = true;
    for (int i = 0; i < kMaxPeers; i++) {
      pp.p[i] = (unsigned char*)peers[i < p.mgWorld ? i : 0];
      aligned = aligned && tiles_pointers_aligned(p.cand, in, pp.p[i]);
    }
    if (aligned) return launch_tiles(p.cand, p.grid, in, pp, stream);
    if (p.haveFallback) return launch_tiles(p.fallback, p.fallbackGrid, in, pp, stream);
    return cudaErrorInvalidValue;
  }
  if (p.extBytes && p.method != kMethodMemcpy && p.method != kMethodSmall &&
      ((uintptr_t)in % p.elt || (uintptr_t)out % p.elt)) {
    // a re-stated problem moves 4- or 8-byte units; buffers aligned for the caller's smaller
    // type only are permuted element by element
    return launch_naive(p.naive, p.numSM, in, out, stream);
  }
  switch (p.method) {
    case kMethodSmall:
      return launch_small(p.small, in, out, stream);
    case kMethodMemcpy:
      return cudaMemcpyAsync(out, in, p.bytes, cudaMemcpyDeviceToDevice, stream);
    case kMethodCopy:
      return launch_copy(in, out, p.bytes, p.numSM, stream);
    case kMethodNaive:
      return launch_naive(p.naive, p.numSM, in, out, stream);
    case kMethodRowCopy:
      if ((uintptr_t)in % p.elt || (uintptr_t)out % p.elt) return cudaErrorInvalidValue;
      return launch_rowcopy(p.cand.rc, p.numSM, in, out, stream);
    case kMethodT2d: {
      if (t2d_pointers_aligned(p.cand.t2d, in, out)) return launch_t2d(p.cand.t2d, in, out, stream);
      if (p.extBytes && p.elt < 4) return p.extSmallFallback ? launch_small(p.small, in, out, stream)
                                                             : launch_naive(p.naive, p.numSM, in, out, stream);
      if (p.haveFallback) {   // the same tile with element-sized accesses
        if (p.fallback.method == kMethodT2d) return launch_t2d(p.fallback.t2d, in, out, stream);
        PeerPtrs pp;
        for (int i = 0; i < kMaxPeers; i++) pp.p[i] = (unsigned char*)out;
        return launch_tiles(p.fallback, p.fallbackGrid, in, pp, stream);
      }
      if (p.mgMode >= 1) return cudaErrorInvalidValue;
      return launch_naive(p.naive, p.numSM, in, out, stream);
    }
    case kMethodTma: {
      // tensor maps and 16-byte stores need 16-byte aligned buffers; others take the tiled kernel
      // with element-sized accesses
      if ((uintptr_t)in % 16 == 0 && (uintptr_t)out % 16 == 0)
        return launch_tma(p.cand.tma, p.cand.tmaMap, p.grid, in, out, stream);
      if (p.haveFallback) {
        PeerPtrs pp;
        for (int i = 0; i < kMaxPeers; i++) pp.p[i] = (unsigned char*)out;
        return launch_tiles(p.fallback, p.fallbackGrid, in, pp, stream);
      }
      if (p.mgMode >= 1) return cudaErrorInvalidValue;   // (no element-wise description of these)
      return launch_naive(p.naive, p.numSM, in, out, stream);
    }
    case kMethodTiles: {
      PeerPtrs pp;
      for (int i = 0; i < kMaxPeers; i++) pp.p[i] = (unsigned char*)out;
      if (tiles_pointers_aligned(p.cand, in, out)) return launch_tiles(p.cand, p.grid, in, pp, stream);
      if (p.haveFallback) return launch_tiles(p.fallback, p.fallbackGrid, in, pp, stream);
      if (p.mgMode >= 1) return cudaErrorInvalidValue;
      return launch_naive(p.naive, p.numSM, in, out, stream);
    }
  }
  return cudaErrorInvalidValue;
}

// Label of a plan that is not described by a tiled candidate.
std::string plain_label(const Plan& p) {
  if (p.method == kMethodNaive) return "naive";
  if (p.method == kMethodCopy) return "copy";
  if (p.method == kMethodMemcpy) return "memcpy";
  if (p.method == kMethodSmall) {
    char buf[96];
    snprintf(buf, sizeof buf, "small t=%ux%u%s%s%s tiles=%u", 1u << p.small.logTA, 1u << p.small.logTB,
             p.small.storeAlongB ? "" : " rows", p.small.packLoad ? " ld32" : "",
             p.small.packStore ? " st32" : "", p.small.numTiles);
    return buf;
  }
  return "?";
}

// Completes a plan around a chosen candidate (grid sizes, unaligned-pointer fallback).
bool adopt_candidate(Plan& p, const DeviceInfo& dev, const Candidate& c) {
  p.method = c.method;
  p.cand = c;
  if (c.method == kMethodT2d) {
    const int nb = t2d_blocks_per_sm(p.cand.t2d);
    if (nb <= 0) return false;
    p.cand.blocksPerSM = nb;
    p.grid = (int)c.t2d.numTiles;
    p.cand.gridBlocks = p.grid;
    p.haveFallback = false;
    if (c.t2d.loadMode != 1 || c.t2d.storeMode != 1) {
      // buffers that are not aligned for this plan's access modes: the same tile in the modes that
      // take any element-aligned address
      TileParams tp = c.params;
      tp.maxVecBytes = 16;
      tp.extend = 1;
      Candidate f;
      if (build_t2d(p.prob, tp, dev, f) && t2d_blocks_per_sm(f.t2d) > 0) {
        p.fallback = f;
        p.fallbackGrid = (int)f.t2d.numTiles;
        p.haveFallback = true;
      }
    }
    return true;
  }
  if (c.method == kMethodTma) {
    const int nb = tma_blocks_per_sm(p.cand.tma);
    if (nb <= 0 || !tma_map_encodable(p.cand.tma, p.cand.tmaMap)) return false;
    p.cand.blocksPerSM = nb;
    long long g = (long long)dev.numSM * nb;
    // a single stage means one tile per block: the hardware block scheduler replaces the ring
    if (g > (long long)c.tma.numTiles || c.tma.stages == 1) g = c.tma.numTiles;
    p.grid = (int)g;
    p.cand.gridBlocks = p.grid;
    // buffers that are not 16-byte aligned: a default tile with element-sized accesses
    p.haveFallback = false;
    TileParams tp;
    tp.maxVecBytes = p.elt;
    tp.maxVBytes = p.elt;
    tp.allowAof = 0;
    Candidate f;
    if (build_tile(p.prob, tp, dev, f) && finalize_tiles(dev, f, p.fallbackGrid)) {
      p.fallback = f;
      p.haveFallback = true;
    }
    return true;
  }
  if (c.method != kMethodTiles) return true;
  if (!finalize_tiles(dev, p.cand, p.grid)) return false;
  p.haveFallback = false;
  if (p.cand.desc.in.vec > 1 || p.cand.desc.out.vec > 1) {
    TileParams tp = c.params;
    tp.maxVecBytes = p.elt;
    tp.maxVBytes = p.elt;
    tp.allowAof = 0;
    Candidate f;
    if (build_tile(p.prob, tp, dev, f) && finalize_tiles(dev, f, p.fallbackGrid)) {
      p.fallback = f;
      p.haveFallback = true;
    }
  }
  return true;
}

// The candidate list of the last problem enumerated (sweeps ask for candidate 0, 1, 2, ... of the
// same problem in a row).
std::string g_enumKey;
std::vector<Candidate> g_enumList;
const std::vector<Candidate>& enumerate_cached(const std::string& key, const Problem& P, const DeviceInfo& dev) {
  if (key != g_enumKey || g_enumList.empty()) {
    g_enumList = enumerate_candidates(P, dev);
    g_enumKey = key;
  }
  return g_enumList;
}

enum PlanMode { kByModel, kByMeasure, kByIndex, kByParams };

// Largest tensor (bytes per side) for which the element-per-thread kernel is a candidate of
// cuttPlan; cuttPlanMeasure, which times it, lets it compete up to eight times that.
constexpr size_t kNaiveCandidateBytes = (size_t)1 << 20;

struct PlanRequest {
  PlanMode mode = kByModel;
  void* idata = nullptr;
  void* odata = nullptr;
  int chunkLast = 0;           // > 0: plan for a slab of this extent along the last dimension,
                               // written into the full output tensor (host pipeline)
  int world = 0;               // > 0: multi-GPU plan for rank `me`
  int me = 0;
  void* const* peers = nullptr;  // output slabs per rank (measure mode)
  int index = 0;
  int method = kMethodTiles;
  TileParams params;
  bool ext = false;            // extension entry point: element sizes 1, 2 and 16 as well
};

// Values a tile parameter set may take (what the enumerator and the test entry point produce);
// anything else in a persisted plan cache is a damaged or foreign entry.
bool valid_tile_params(const TileParams& t, Method method = kMethodTiles) {
  auto one_of = [](int v, std::initializer_list<int> ok) {
    for (int x : ok) if (v == x) return true;
    return false;
  };
  if (method == kMethodTma ? (t.stages < 1 || t.stages > kTmaMaxStages) : (t.stages != 1 && t.stages != 2)) return false;
  return one_of(t.nthreads, {64, 128, 256, 512}) &&
         one_of(t.maxVecBytes, {4, 8, 16}) && one_of(t.maxVBytes, {4, 8, 16}) &&
         one_of(t.extend, {0, 1}) && one_of(t.loopOrder, {0, 1, 2, 3}) && one_of(t.groupIn, {1, 2, 4}) &&
         one_of(t.groupOut, {1, 2, 4}) && one_of(t.cutInRun, {0, 1}) && one_of(t.allowAof, {0, 1}) &&
         one_of(t.oneTilePerBlock, {0, 1}) && one_of(t.peerOrder, {0, 1}) && t.tinBytes >= 4 && t.tinBytes <= (1u << 16) &&
         t.toutBytes >= 4 && t.toutBytes <= (1u << 16) && t.vtargetBytes >= 4 && t.vtargetBytes <= (1u << 20);
}

// With `internalOut` the plan is handed to the caller instead of entering the public handle table
// (no handle number is consumed): plans the library makes for its own use.
cuttResult make_plan(cuttHandle* handle, int rank, const int* dim, const int* perm, size_t elt,
                     cudaStream_t stream, const PlanRequest& req,
                     std::shared_ptr<Plan>* internalOut = nullptr) {
  cuttResult chk = check_input(rank, dim, perm, elt, req.ext);
  if (chk != CUTT_SUCCESS) return chk;
  if (!handle && !internalOut) return CUTT_INVALID_PARAMETER;
  const bool extSize = req.ext && elt != 4 && elt != 8;
  if (extSize && (rank > 31 || req.world > 0 || req.chunkLast > 0 ||
                  (req.mode != kByModel && req.mode != kByMeasure)))
    return CUTT_INVALID_PARAMETER;
  if (req.mode == kByMeasure && req.idata == req.odata) return CUTT_INVALID_PARAMETER;

  std::unique_lock<std::mutex> lk(g_mutex);
  if (!internalOut) {
    *handle = g_nextHandle++;
    if (g_plans.count(*handle)) return CUTT_INTERNAL_ERROR;
  }

  int devId = 0;
  DeviceInfo dev;
  if (!device_info(devId, dev)) return CUTT_INTERNAL_ERROR;

  std::shared_ptr<Plan> p(new Plan);
  p->device = devId;
  p->stream = stream;
  p->elt = (int)elt;
  p->numSM = dev.numSM;
  if (rank > 32) return CUTT_INVALID_PARAMETER;
  const bool verbose = env_flag("CUTT_VERBOSE");
  bool ok = false;
  bool canon = false;
  std::string key = problem_key(devId, rank, dim, perm, elt);
  if (req.world > 0) {
    ShardInfo info;
    if (!problem_from_cutt_sharded(rank, dim, perm, (int)elt, req.world, req.me, p->prob, info))
      return CUTT_INVALID_PARAMETER;
    canon = true;
    p->mgWorld = req.world;
    p->mgMe = req.me;
    p->mgMode = info.mode;
    p->mgLocalVolume = info.localVolume;
    p->bytes = (size_t)info.localVolume * elt;
    if (info.mode == 0) fill_naive(*p, rank, info.localDim, perm);
    key += "/mg" + std::to_string(req.world) + "." + std::to_string(req.me);
  } else if (req.chunkLast > 0) {
    if (!problem_from_cutt_chunk(rank, dim, perm, (int)elt, req.chunkLast, p->prob)) return CUTT_INVALID_PARAMETER;
    canon = true;
    p->bytes = (size_t)p->prob.volume * elt;
    p->mgMode = 2;  // no element-wise fallback: the output is a strided part of a larger tensor
    key += "/chunk" + std::to_string(req.chunkLast);
  } else if (extSize) {
    size_t vol = 1;
    for (int i = 0; i < rank; i++) vol *= (size_t)dim[i];
    p->bytes = vol * elt;
    p->extBytes = (int)elt;
    // the element-wise kernel works on the caller's element type (16 bytes: two 8-byte words)
    if (elt == 16) {
      int d2[32], p2[32];
      d2[0] = 2; p2[0] = 0;
      for (int i = 0; i < rank; i++) { d2[i + 1] = dim[i]; p2[i + 1] = perm[i] + 1; }
      p->elt = 8;
      fill_naive(*p, rank + 1, d2, p2);
    } else {
      p->elt = (int)elt;
      fill_naive(*p, rank, dim, perm);
    }
    canon = problem_from_cutt_ext(rank, dim, perm, (int)elt, p->prob);
    if (canon) p->elt = p->prob.elt;
    key += "/ext";
  } else {
    size_t vol = 1;
    for (int i = 0; i < rank; i++) vol *= (size_t)dim[i];
    p->bytes = vol * elt;
    fill_naive(*p, rank, dim, perm);
    canon = problem_from_cutt(rank, dim, perm, (int)elt, p->prob);
  }
  void* const* peers = req.peers;
  void* measureOut = req.odata;
  if (req.world > 0 && req.mode == kByMeasure) {
    if (!peers) return CUTT_INVALID_PARAMETER;
    measureOut = peers[req.me];
    if (req.idata == measureOut) return CUTT_INVALID_PARAMETER;
  }

  if (!canon) {
    p->method = kMethodNaive;  // fused rank beyond the tiled kernel's limit
    ok = true;
  } else if (extSize && p->prob.identity) {
    p->method = kMethodMemcpy;
    ok = true;
  } else if (extSize && p->prob.elt < 4) {
    // 2-byte elements whose output rows start on 16-byte boundaries: swizzled two-dimensional tiles
    // with an 8 x 8 register transpose; everything else: the element-wise tiled kernel, which is
    // also what such a plan falls back to on buffers that are not aligned for it
    const bool haveSmall = build_small(p->prob, p->small);
    Candidate c;
    if (build_t2d_small(p->prob, dev, c) && adopt_candidate(*p, dev, c)) {
      p->extSmallFallback = haveSmall;
    } else {
      p->method = haveSmall ? kMethodSmall : kMethodNaive;
    }
    ok = true;
  } else if (p->mgMode == 1 && req.mode != kByModel && req.mode != kByMeasure && req.mode != kByIndex) {
    return CUTT_INVALID_PARAMETER;
  } else if (req.mode == kByParams) {
    if (req.method == kMethodNaive) { p->method = kMethodNaive; ok = true; }
    else if (req.method == kMethodRowCopy) {
      Candidate c;
      if (!build_rowcopy(p->prob, dev, c)) return CUTT_INVALID_PARAMETER;
      ok = adopt_candidate(*p, dev, c);
    }
    else if (req.method == kMethodT2d) {
      Candidate c;
      if (!build_t2d(p->prob, req.params, dev, c)) return CUTT_INVALID_PARAMETER;
      ok = adopt_candidate(*p, dev, c);
    }
    else if (req.method == kMethodTma) {
      Candidate c;
      if (!dev.tmaLoads || !build_tma(p->prob, req.params, dev, c)) return CUTT_INVALID_PARAMETER;
      ok = adopt_candidate(*p, dev, c);
    }
    else if (req.method == kMethodCopy || req.method == kMethodMemcpy) {
      if (!p->prob.identity) return CUTT_INVALID_PARAMETER;
      p->method = (Method)req.method; ok = true;
    } else {
      if (p->prob.identity) return CUTT_INVALID_PARAMETER;
      Candidate c;
      if (!build_tile(p->prob, req.params, dev, c)) return CUTT_INVALID_PARAMETER;
      ok = adopt_candidate(*p, dev, c);
    }
  } else {
    // (a copy: the cached list may be replaced by another thread while this one measures)
    std::vector<Candidate> cands = enumerate_cached(key, p->prob, dev);
    if (!cands.empty() && req.world == 0 && req.chunkLast == 0 && !extSize && !p->prob.identity &&
        (req.mode == kByModel || req.mode == kByMeasure) &&
        p->bytes <= (req.mode == kByMeasure ? 8 * kNaiveCandidateBytes : kNaiveCandidateBytes) &&
        !env_flag("CUTT_NO_NAIVE_CANDIDATE")) {
      // tensors this small stay in the L2 cache and their time is launch plus one round trip to
      // memory: one thread per element, no shared-memory stage, competes (measured on B200 over
      // thirty shapes of 0.1-1 MB: 3.5-3.6 us per launch, the rate at which launches issue, against
      // 4.0-6.2 us for the model's first tiled plan; (31,549,2,3) perm (3,0,2,1): 3.6 against 6.2)
      Candidate nv;
      nv.method = kMethodNaive;
      nv.label = "naive";
      nv.cost = 4.0e-6 + 2.0 * (double)p->bytes / 1.5e12;
      size_t at = 0;
      while (at < cands.size() && cands[at].cost <= nv.cost) at++;
      cands.insert(cands.begin() + at, nv);
    }
    if (cands.empty()) {
      if (p->mgMode >= 1) return CUTT_INTERNAL_ERROR;  // no element-wise fallback for these
      p->method = kMethodNaive;
      ok = true;
    } else if (req.mode == kByIndex) {
      if (req.index < 0 || req.index >= (int)cands.size()) return CUTT_INVALID_PARAMETER;
      ok = adopt_candidate(*p, dev, cands[req.index]);
    } else {
      CachedChoice cc;
      bool hit = plan_cache().get(key, cc);
      if (hit) {
        // An entry is only a hint (the cache may come from a file): it is used when it describes
        // a legal plan for THIS problem, and ignored - the model or the measurement decides -
        // otherwise.  Copy methods are legal for identity permutations only.
        if (cc.method == kMethodTiles) {
          Candidate c;
          ok = !p->prob.identity && valid_tile_params(cc.params) && build_tile(p->prob, cc.params, dev, c) &&
               adopt_candidate(*p, dev, c);
        } else if (cc.method == kMethodRowCopy) {
          Candidate c;
          ok = build_rowcopy(p->prob, dev, c) && adopt_candidate(*p, dev, c);
        } else if (cc.method == kMethodT2d) {
          Candidate c;
          ok = valid_tile_params(cc.params, kMethodT2d) && build_t2d(p->prob, cc.params, dev, c) &&
               adopt_candidate(*p, dev, c);
        } else if (cc.method == kMethodTma) {
          Candidate c;
          ok = dev.tmaLoads && valid_tile_params(cc.params, kMethodTma) && build_tma(p->prob, cc.params, dev, c) &&
               adopt_candidate(*p, dev, c);
        } else if (cc.method == kMethodCopy || cc.method == kMethodMemcpy) {
          ok = p->prob.identity;
          if (ok) p->method = cc.method;
        } else if (cc.method == kMethodNaive) {
          ok = req.world == 0 && req.chunkLast == 0 && !extSize && !p->prob.identity &&
               p->bytes <= 8 * kNaiveCandidateBytes;
          if (ok) p->method = kMethodNaive;
        }
        if (ok) p->note = "cache";
        if (ok && req.mode == kByMeasure) {
          // nothing is timed, but the visible effects of cuttPlanMeasure stay those of
          // src/cutt.cpp:240-250: odata is overwritten and the device is synchronised
          if (cudaMemsetAsync(measureOut, 0xFF, p->bytes, stream) != cudaSuccess ||
              cudaDeviceSynchronize() != cudaSuccess) {
            cudaGetLastError();
            return CUTT_INTERNAL_ERROR;
          }
        }
      }
      if (!ok && req.mode == kByModel) {
        for (size_t i = 0; i < cands.size() && !ok; i++) ok = adopt_candidate(*p, dev, cands[i]);
        if (ok) p->note = "model";
      }
      if (!ok && req.mode == kByMeasure) {
        // Time the most promising candidates on the device (src/cutt.cpp:236-258 times every
        // candidate once, cold, on stream 0; here: one warm-up and the best of three runs on
        // the plan's stream, after the same memset + device synchronisation).
        lk.unlock();
        const size_t topk = env_size("CUTT_MEASURE_TOPK", 48);
        cudaEvent_t e0, e1;
        if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess)
          return CUTT_INTERNAL_ERROR;
        if (cudaMemsetAsync(measureOut, 0xFF, p->bytes, stream) != cudaSuccess ||
            cudaDeviceSynchronize() != cudaSuccess) {
          cudaEventDestroy(e0); cudaEventDestroy(e1);
          return CUTT_INTERNAL_ERROR;
        }
        double best = 1e30, bestFirst = 1e30;
        int bestIdx = -1;
        std::vector<std::pair<double, int>> scored;   // (score, candidate) of fully timed candidates
        Plan trial = *p;
        size_t nT2d = 0, nTma = 0;
        const size_t familyQuota = env_size("CUTT_MEASURE_FAMILY", 8);
        for (size_t i = 0; i < cands.size(); i++) {
          // beyond the model's best `topk`, only methods of another kind still get their turn; the
          // two swizzled-tile families are timed up to a quota each (their estimates are coarse, so
          // they do not compete for the tiled kernel's slots)
          if (i >= topk && cands[i].method == kMethodTiles) continue;
          if (cands[i].method == kMethodT2d && nT2d++ >= familyQuota) continue;
          if (cands[i].method == kMethodTma && nTma++ >= familyQuota) continue;
          if (!adopt_candidate(trial, dev, cands[i])) continue;
          bool fail = false;
          double tmin = 1e30;
          // The first run doubles as warm-up; clearly slower candidates are dropped after it.
          // The score is the SLOWER of the two runs that follow: some plans alternate between
          // a fast and a much slower mode from launch to launch, and the best of three would
          // rank them by the mode a caller only sees half of the time.
          double first = 1e30, warm = 0.0;
          for (int rep = 0; rep < 3 && !fail; rep++) {
            // launches of a few microseconds are timed eight at a time
            const int batch = (rep > 0 && first < 0.05) ? 8 : 1;
            cudaEventRecord(e0, stream);
            for (int b = 0; b < batch && !fail; b++)
              fail = run_plan(trial, req.idata, measureOut, stream, peers) != cudaSuccess;
            cudaEventRecord(e1, stream);
            if (cudaEventSynchronize(e1) != cudaSuccess) fail = true;
            float ms = 0.f;
            if (fail || cudaEventElapsedTime(&ms, e0, e1) != cudaSuccess) { fail = true; break; }
            ms /= (float)batch;
            if (rep == 0) {
              first = ms;
              // like with like: first run against the best plan's first run
              if (first > 1.2 * bestFirst && first > best) break;
            } else if (ms > warm) {
              warm = ms;
            }
          }
          tmin = warm > 0.0 ? warm : first;
          if (fail) { cudaGetLastError(); continue; }
          if (verbose) fprintf(stderr, "[cutt] measure %2zu %8.4f ms  %s\n", i, tmin, cands[i].label.c_str());
          if (warm > 0.0) scored.push_back(std::make_pair(tmin, (int)i));
          if (tmin < best) { best = tmin; bestIdx = (int)i; bestFirst = first; }
        }
        // Play-off: candidates within 3 % of the winner (at most four) are timed seven more
        // times each, alternating, and ranked by their median - two runs cannot separate them.
        std::sort(scored.begin(), scored.end());
        while (scored.size() > 4 || (!scored.empty() && scored.back().first > 1.03 * scored.front().first))
          scored.pop_back();
        if (scored.size() >= 2) {
          std::vector<std::vector<float>> t(scored.size());
          bool fail = false;
          for (int round = 0; round < 7 && !fail; round++) {
            for (size_t k = 0; k < scored.size() && !fail; k++) {
              if (!adopt_candidate(trial, dev, cands[scored[k].second])) { fail = true; break; }
              const int batch = scored[k].first < 0.05 ? 8 : 1;
              cudaEventRecord(e0, stream);
              for (int b = 0; b < batch && !fail; b++)
                fail = run_plan(trial, req.idata, measureOut, stream, peers) != cudaSuccess;
              cudaEventRecord(e1, stream);
              float ms = 0.f;
              if (cudaEventSynchronize(e1) != cudaSuccess || fail ||
                  cudaEventElapsedTime(&ms, e0, e1) != cudaSuccess) { fail = true; break; }
              t[k].push_back(ms / (float)batch);
            }
          }
          if (fail) {
            cudaGetLastError();
          } else {
            double bestMed = 1e30;
            std::vector<double> med(scored.size());
            for (size_t k = 0; k < scored.size(); k++) {
              std::sort(t[k].begin(), t[k].end());
              med[k] = t[k][t[k].size() / 2];
              if (verbose) fprintf(stderr, "[cutt] play-off %2d median %8.4f ms\n", scored[k].second, med[k]);
              if (med[k] < bestMed) bestMed = med[k];
            }
            // medians within 0.5 % are a tie: the cost model's order decides
            bestIdx = -1;
            for (size_t k = 0; k < scored.size(); k++)
              if (med[k] <= 1.005 * bestMed && (bestIdx < 0 || scored[k].second < bestIdx)) bestIdx = scored[k].second;
          }
        }
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
        lk.lock();
        if (bestIdx >= 0) {
          ok = adopt_candidate(*p, dev, cands[bestIdx]);
          if (ok) {
            CachedChoice w;
            w.method = cands[bestIdx].method;
            w.params = cands[bestIdx].params;
            plan_cache().put(key, w);
            p->note = "measured";
          }
        }
      }
    }
  }
  if (!ok) return CUTT_INTERNAL_ERROR;
  if (verbose) {
    Candidate shown = p->cand;
    shown.method = p->method;
    if (p->method != kMethodTiles && p->method != kMethodRowCopy && p->method != kMethodTma && p->method != kMethodT2d)
      shown.label = plain_label(*p);
    fprintf(stderr, "[cutt] plan %u (%s): %s\n", *handle, p->note.c_str(),
            canon ? describe(p->prob, shown).c_str() : "naive (rank too high after fusion)");
  }
  if (internalOut) *internalOut = p;
  else g_plans[*handle] = p;
  return CUTT_SUCCESS;
}

}  // namespace

// ---------------------------------------------------------------------------------------
// C++ API (include/cutt.h)

cuttResult cuttPlan(cuttHandle* handle, int rank, int* dim, int* permutation, size_t sizeofType,
                    cudaStream_t stream) {
  PlanRequest req;
  req.mode = kByModel;
  return make_plan(handle, rank, dim, permutation, sizeofType, stream, req);
}

cuttResult cuttPlanMeasure(cuttHandle* handle, int rank, int* dim, int* permutation, size_t sizeofType,
                           cudaStream_t stream, void* idata, void* odata) {
  PlanRequest req;
  req.mode = kByMeasure;
  req.idata = idata;
  req.odata = odata;
  return make_plan(handle, rank, dim, permutation, sizeofType, stream, req);
}

cuttResult cuttDestroy(cuttHandle handle) {
  std::lock_guard<std::mutex> lk(g_mutex);
  auto it = g_plans.find(handle);
  if (it == g_plans.end()) return CUTT_INVALID_PLAN;
  g_plans.erase(it);
  return CUTT_SUCCESS;
}

cuttResult cuttExecute(cuttHandle handle, void* idata, void* odata) {
  std::shared_ptr<Plan> p;
  {
    std::lock_guard<std::mutex> lk(g_mutex);
    auto it = g_plans.find(handle);
    if (it == g_plans.end()) return CUTT_INVALID_PLAN;
    p = it->second;
  }
  if (idata == odata) return CUTT_INVALID_PARAMETER;
  if (p->mgMode == 1) return CUTT_INVALID_PARAMETER;  // needs the peers' slabs: cutt_mg_execute
  if (p->extBytes) {  // buffers must be aligned for the caller's element type (at most 8 bytes)
    const uintptr_t need = p->extBytes > 8 ? 8 : p->extBytes;
    if ((uintptr_t)idata % need || (uintptr_t)odata % need) return CUTT_INVALID_PARAMETER;
  }
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return CUTT_INTERNAL_ERROR;
  if (dev != p->device) return CUTT_INVALID_DEVICE;
  return run_plan(*p, idata, odata, p->stream) == cudaSuccess ? CUTT_SUCCESS : CUTT_INTERNAL_ERROR;
}

// ---------------------------------------------------------------------------------------
// Host-buffer pipeline state (cutt_c_transpose_host), one per device: scratch buffers (grown on
// demand, kept), three streams, events and the plans of recent problems.  The plans are the
// library's own: they never enter the public handle table, and the least recently used one is
// dropped beyond kHostPlanLimit.
namespace {

struct HostPipe {
  void* dIn = nullptr;
  void* dOut = nullptr;
  size_t cap = 0;
  cudaStream_t sUp = nullptr, sRun = nullptr, sDown = nullptr;
  std::vector<cudaEvent_t> evUp, evRun;
  std::list<std::pair<std::string, std::shared_ptr<Plan>>> plans;  // most recently used first
};
constexpr size_t kHostPlanLimit = 64;
std::mutex g_hostMutex;
std::unordered_map<int, HostPipe> g_hostPipes;

// Error exit of the pipeline: nothing may still be reading or writing the caller's host buffers
// when the call returns.
int host_pipe_fail(HostPipe& hp, int code) {
  if (hp.sUp) cudaStreamSynchronize(hp.sUp);
  if (hp.sRun) cudaStreamSynchronize(hp.sRun);
  if (hp.sDown) cudaStreamSynchronize(hp.sDown);
  cudaGetLastError();
  return code;
}

}  // namespace

// ---------------------------------------------------------------------------------------
// C ABI (include/cutt_c.h)

extern "C" {

int cutt_c_plan(unsigned int* handle, int rank, const int* dim, const int* permutation,
                size_t sizeofType, void* stream) {
  PlanRequest req;
  return (int)make_plan(handle, rank, dim, permutation, sizeofType, (cudaStream_t)stream, req);
}

int cutt_c_plan_measure(unsigned int* handle, int rank, const int* dim, const int* permutation,
                        size_t sizeofType, void* stream, void* idata, void* odata) {
  PlanRequest req;
  req.mode = kByMeasure;
  req.idata = idata;
  req.odata = odata;
  return (int)make_plan(handle, rank, dim, permutation, sizeofType, (cudaStream_t)stream, req);
}

int cutt_c_plan_ext(unsigned int* handle, int rank, const int* dim, const int* permutation,
                    size_t sizeofType, void* stream) {
  PlanRequest req;
  req.ext = true;
  return (int)make_plan(handle, rank, dim, permutation, sizeofType, (cudaStream_t)stream, req);
}

int cutt_c_plan_measure_ext(unsigned int* handle, int rank, const int* dim, const int* permutation,
                            size_t sizeofType, void* stream, void* idata, void* odata) {
  PlanRequest req;
  req.ext = true;
  req.mode = kByMeasure;
  req.idata = idata;
  req.odata = odata;
  return (int)make_plan(handle, rank, dim, permutation, sizeofType, (cudaStream_t)stream, req);
}

int cutt_c_execute(unsigned int handle, void* idata, void* odata) {
  return (int)cuttExecute(handle, idata, odata);
}

int cutt_c_destroy(unsigned int handle) { return (int)cuttDestroy(handle); }

int cutt_c_plan_describe(unsigned int handle, char* buf, size_t len) {
  std::lock_guard<std::mutex> lk(g_mutex);
  auto it = g_plans.find(handle);
  if (it == g_plans.end()) return CUTT_INVALID_PLAN;
  if (!buf || !len) return CUTT_INVALID_PARAMETER;
  const Plan& p = *it->second;
  Candidate shown = p.cand;
  shown.method = p.method;
  if (p.method != kMethodTiles && p.method != kMethodRowCopy && p.method != kMethodTma && p.method != kMethodT2d)
    shown.label = plain_label(p);
  snprintf(buf, len, "%s", describe(p.prob, shown).c_str());
  return CUTT_SUCCESS;
}

int cutt_c_num_candidates(int rank, const int* dim, const int* permutation, size_t sizeofType) {
  if (check_input(rank, dim, permutation, sizeofType) != CUTT_SUCCESS) return 0;
  std::lock_guard<std::mutex> lk(g_mutex);
  int devId;
  DeviceInfo dev;
  if (!device_info(devId, dev)) return 0;
  Problem P;
  if (!problem_from_cutt(rank, dim, permutation, (int)sizeofType, P)) return 0;
  return (int)enumerate_cached(problem_key(devId, rank, dim, permutation, sizeofType), P, dev).size();
}

int cutt_c_plan_candidate(unsigned int* handle, int rank, const int* dim, const int* permutation,
                          size_t sizeofType, void* stream, int index) {
  PlanRequest req;
  req.mode = kByIndex;
  req.index = index;
  return (int)make_plan(handle, rank, dim, permutation, sizeofType, (cudaStream_t)stream, req);
}

int cutt_c_plan_params(unsigned int* handle, int rank, const int* dim, const int* permutation,
                       size_t sizeofType, void* stream, int method, unsigned tinBytes,
                       unsigned toutBytes, unsigned vtargetBytes, int extend, int loopOrder,
                       int maxVecBytes, int maxVBytes, int nthreads, int stages) {
  PlanRequest req;
  req.mode = kByParams;
  req.method = method;
  req.params.tinBytes = tinBytes;
  req.params.toutBytes = toutBytes;
  req.params.vtargetBytes = vtargetBytes;
  req.params.extend = extend;
  req.params.loopOrder = loopOrder;
  req.params.maxVecBytes = maxVecBytes;
  req.params.maxVBytes = maxVBytes;
  if (nthreads != 64 && nthreads != 128 && nthreads != 256 && nthreads != 512) return CUTT_INVALID_PARAMETER;
  if (method == kMethodTma ? (stages < 1 || stages > kTmaMaxStages) : (stages != 1 && stages != 2))
    return CUTT_INVALID_PARAMETER;
  req.params.nthreads = nthreads;
  req.params.stages = stages;
  return (int)make_plan(handle, rank, dim, permutation, sizeofType, (cudaStream_t)stream, req);
}

int cutt_c_transpose_host(int rank, const int* dim, const int* permutation, size_t sizeofType,
                          const void* hin, void* hout) {
  // Calls are serialised.  Large tensors are cut into slabs along the slowest input dimension so
  // that the upload of slab k+1, the kernel of slab k and the download of slab k-1 overlap (PCIe
  // is full duplex); each slab is permuted straight into its strided place in the device output,
  // which is downloaded with a 2-D copy.
  if (check_input(rank, dim, permutation, sizeofType) != CUTT_SUCCESS) return CUTT_INVALID_PARAMETER;
  if (!hin || !hout) return CUTT_INVALID_PARAMETER;
  std::lock_guard<std::mutex> lk(g_hostMutex);
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return CUTT_INTERNAL_ERROR;
  HostPipe& hp = g_hostPipes[dev];
  size_t bytes = sizeofType;
  for (int i = 0; i < rank; i++) bytes *= (size_t)dim[i];
  if (bytes > hp.cap) {
    if (hp.dIn) cudaFree(hp.dIn);
    if (hp.dOut) cudaFree(hp.dOut);
    hp.dIn = hp.dOut = nullptr;
    hp.cap = 0;
    if (cudaMalloc(&hp.dIn, bytes) != cudaSuccess || cudaMalloc(&hp.dOut, bytes) != cudaSuccess) {
      if (hp.dIn) cudaFree(hp.dIn);
      hp.dIn = hp.dOut = nullptr;
      cudaGetLastError();
      return CUTT_INTERNAL_ERROR;
    }
    hp.cap = bytes;
  }
  if (!hp.sDown) {
    if ((!hp.sUp && cudaStreamCreateWithFlags(&hp.sUp, cudaStreamNonBlocking) != cudaSuccess) ||
        (!hp.sRun && cudaStreamCreateWithFlags(&hp.sRun, cudaStreamNonBlocking) != cudaSuccess) ||
        cudaStreamCreateWithFlags(&hp.sDown, cudaStreamNonBlocking) != cudaSuccess) {
      cudaGetLastError();
      return CUTT_INTERNAL_ERROR;
    }
  }
  const int last = rank - 1;
  const int dlast = dim[last];
  int nslab = 1;
  if (bytes >= (size_t)64 << 20) nslab = dlast < 8 ? dlast : 8;
  if (bytes >= (size_t)512 << 20 && dlast >= 256) {
    // measured on B200 hosts (PCIe 5 x16, 0.8 and 1.6 GB tensors): 6-9 slabs are fastest; every
    // slab beyond that costs about 1 ms, fewer leave a long unoverlapped head and tail
    const size_t n = bytes / ((size_t)160 << 20);
    nslab = n < 6 ? 6 : (n > 8 ? 8 : (int)n);
  }
  // strides of the slowest input dimension on both sides (elements)
  size_t isLast = 1, osLast = 1;
  for (int i = 0; i < last; i++) isLast *= (size_t)dim[i];
  for (int k = 0; k < rank && permutation[k] != last; k++) osLast *= (size_t)dim[permutation[k]];
  const size_t pitch = osLast * (size_t)dlast * sizeofType;   // distance between the pieces of a slab's output
  const size_t height = bytes / pitch;
  if (height == 1 && bytes >= (size_t)1 << 30) {
    // the slowest dimension stays slowest: every slab's output is one contiguous piece, a slab
    // costs next to nothing, and what is left outside the overlap is one slab's upload and
    // kernel (measured, 4.3 GB tensor: 8 slabs 96.6 ms, 16 slabs 91.8 ms, 32 slabs 90.0 ms)
    const size_t n = bytes / ((size_t)128 << 20);
    const int cap = dlast < 32 ? dlast : 32;
    nslab = n > (size_t)cap ? cap : (int)n;
  }
  {
    const size_t forced = env_size("CUTT_HOST_SLABS", 0);     // tuning aid
    if (forced >= 1 && (int)forced <= dlast) nslab = (int)forced;
  }
  if (nslab > 1 && height > 1 && pitch >= ((size_t)1 << 31)) nslab = 1;  // beyond what a 2-D copy can describe
  int chunk = (dlast + nslab - 1) / nslab;
  if (nslab > 1 && chunk >= 32) chunk = (chunk + 15) / 16 * 16;  // keeps slab offsets 16-byte aligned
  nslab = (dlast + chunk - 1) / chunk;
  while ((int)hp.evUp.size() < nslab) {
    cudaEvent_t a, b;
    if (cudaEventCreateWithFlags(&a, cudaEventDisableTiming) != cudaSuccess) { cudaGetLastError(); return CUTT_INTERNAL_ERROR; }
    if (cudaEventCreateWithFlags(&b, cudaEventDisableTiming) != cudaSuccess) {
      cudaEventDestroy(a);
      cudaGetLastError();
      return CUTT_INTERNAL_ERROR;
    }
    hp.evUp.push_back(a);
    hp.evRun.push_back(b);
  }
  auto plan_for = [&](int extent, std::shared_ptr<Plan>& out) -> cuttResult {
    const std::string key = problem_key(dev, rank, dim, permutation, sizeofType) + "/host" + std::to_string(extent);
    for (auto it = hp.plans.begin(); it != hp.plans.end(); ++it) {
      if (it->first != key) continue;
      out = it->second;
      hp.plans.splice(hp.plans.begin(), hp.plans, it);
      return CUTT_SUCCESS;
    }
    PlanRequest req;
    if (extent != dlast) req.chunkLast = extent;
    cuttResult r = make_plan(nullptr, rank, dim, permutation, sizeofType, hp.sRun, req, &out);
    if (r != CUTT_SUCCESS) return r;
    hp.plans.emplace_front(key, out);
    while (hp.plans.size() > kHostPlanLimit) hp.plans.pop_back();
    return CUTT_SUCCESS;
  };
  for (int k = 0; k < nslab; k++) {
    const int c0 = k * chunk;
    const int ext = (c0 + chunk <= dlast) ? chunk : dlast - c0;
    std::shared_ptr<Plan> p;
    cuttResult r = plan_for(ext, p);
    if (r != CUTT_SUCCESS) return host_pipe_fail(hp, r);
    const size_t inOff = (size_t)c0 * isLast * sizeofType;
    const size_t inBytes = (size_t)ext * isLast * sizeofType;
    const size_t outOff = (size_t)c0 * osLast * sizeofType;
    const size_t width = (size_t)ext * osLast * sizeofType;
    if (cudaMemcpyAsync((char*)hp.dIn + inOff, (const char*)hin + inOff, inBytes, cudaMemcpyHostToDevice, hp.sUp) != cudaSuccess ||
        cudaEventRecord(hp.evUp[k], hp.sUp) != cudaSuccess || cudaStreamWaitEvent(hp.sRun, hp.evUp[k], 0) != cudaSuccess)
      return host_pipe_fail(hp, CUTT_INTERNAL_ERROR);
    if (run_plan(*p, (char*)hp.dIn + inOff, (char*)hp.dOut + outOff, hp.sRun) != cudaSuccess)
      return host_pipe_fail(hp, CUTT_INTERNAL_ERROR);
    if (cudaEventRecord(hp.evRun[k], hp.sRun) != cudaSuccess || cudaStreamWaitEvent(hp.sDown, hp.evRun[k], 0) != cudaSuccess)
      return host_pipe_fail(hp, CUTT_INTERNAL_ERROR);
    cudaError_t e;
    if (nslab == 1) e = cudaMemcpyAsync(hout, hp.dOut, bytes, cudaMemcpyDeviceToHost, hp.sDown);
    else if (height == 1) e = cudaMemcpyAsync((char*)hout + outOff, (char*)hp.dOut + outOff, width, cudaMemcpyDeviceToHost, hp.sDown);
    else e = cudaMemcpy2DAsync((char*)hout + outOff, pitch, (char*)hp.dOut + outOff, pitch, width, height,
                               cudaMemcpyDeviceToHost, hp.sDown);
    if (e != cudaSuccess) return host_pipe_fail(hp, CUTT_INTERNAL_ERROR);
  }
  if (cudaStreamSynchronize(hp.sDown) != cudaSuccess) return host_pipe_fail(hp, CUTT_INTERNAL_ERROR);
  return CUTT_SUCCESS;
}

// ---- multi-GPU extension (include/cutt_mg.h) ----

int cutt_mg_plan(unsigned int* handle, int rank, const int* dim, const int* permutation,
                 size_t sizeofType, void* stream, int world, int me) {
  if (world < 1 || world > CUTT_MG_MAX_WORLD || me < 0 || me >= world) return CUTT_INVALID_PARAMETER;
  PlanRequest req;
  req.world = world;
  req.me = me;
  return (int)make_plan(handle, rank, dim, permutation, sizeofType, (cudaStream_t)stream, req);
}

int cutt_mg_plan_measure(unsigned int* handle, int rank, const int* dim, const int* permutation,
                         size_t sizeofType, void* stream, int world, int me, void* idata,
                         void* const* odata) {
  if (world < 1 || world > CUTT_MG_MAX_WORLD || me < 0 || me >= world) return CUTT_INVALID_PARAMETER;
  if (!idata || !odata) return CUTT_INVALID_PARAMETER;
  PlanRequest req;
  req.mode = kByMeasure;
  req.world = world;
  req.me = me;
  req.idata = idata;
  req.peers = odata;
  return (int)make_plan(handle, rank, dim, permutation, sizeofType, (cudaStream_t)stream, req);
}

int cutt_mg_num_candidates(int rank, const int* dim, const int* permutation, size_t sizeofType,
                           int world, int me) {
  if (world < 1 || world > CUTT_MG_MAX_WORLD || me < 0 || me >= world) return 0;
  if (check_input(rank, dim, permutation, sizeofType) != CUTT_SUCCESS) return 0;
  std::lock_guard<std::mutex> lk(g_mutex);
  int devId;
  DeviceInfo dev;
  if (!device_info(devId, dev)) return 0;
  Problem P;
  ShardInfo info;
  if (!problem_from_cutt_sharded(rank, dim, permutation, (int)sizeofType, world, me, P, info)) return 0;
  const std::string key = problem_key(devId, rank, dim, permutation, sizeofType) + "/mg" + std::to_string(world) +
                          "." + std::to_string(me);
  return (int)enumerate_cached(key, P, dev).size();
}

int cutt_mg_plan_candidate(unsigned int* handle, int rank, const int* dim, const int* permutation,
                           size_t sizeofType, void* stream, int world, int me, int index) {
  if (world < 1 || world > CUTT_MG_MAX_WORLD || me < 0 || me >= world) return CUTT_INVALID_PARAMETER;
  PlanRequest req;
  req.mode = kByIndex;
  req.world = world;
  req.me = me;
  req.index = index;
  return (int)make_plan(handle, rank, dim, permutation, sizeofType, (cudaStream_t)stream, req);
}

int cutt_mg_mode(unsigned int handle) {
  std::lock_guard<std::mutex> lk(g_mutex);
  auto it = g_plans.find(handle);
  if (it == g_plans.end() || it->second->mgWorld == 0) return -1;
  return it->second->mgMode;
}

long long cutt_mg_local_volume(unsigned int handle) {
  std::lock_guard<std::mutex> lk(g_mutex);
  auto it = g_plans.find(handle);
  if (it == g_plans.end() || it->second->mgWorld == 0) return -1;
  return it->second->mgLocalVolume;
}

int cutt_mg_execute(unsigned int handle, void* idata, void* const* odata) {
  std::shared_ptr<Plan> p;
  {
    std::lock_guard<std::mutex> lk(g_mutex);
    auto it = g_plans.find(handle);
    if (it == g_plans.end()) return CUTT_INVALID_PLAN;
    p = it->second;
  }
  if (p->mgWorld == 0 || !odata || !idata) return CUTT_INVALID_PARAMETER;
  for (int h = 0; h < p->mgWorld; h++)
    if (!odata[h] || odata[h] == idata) return CUTT_INVALID_PARAMETER;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return CUTT_INTERNAL_ERROR;
  if (dev != p->device) return CUTT_INVALID_DEVICE;
  return run_plan(*p, idata, odata[p->mgMe], p->stream, odata) == cudaSuccess ? CUTT_SUCCESS
                                                                              : CUTT_INTERNAL_ERROR;
}

// Base address of the allocation that contains p (driver entry point looked up at run time so
// that the library keeps linking with the CUDA runtime alone).
static bool allocation_base(void* p, unsigned long long& base) {
  typedef int (*GetRange)(unsigned long long*, size_t*, unsigned long long);
  static GetRange fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qr;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &sym, cudaEnableDefault, &qr) == cudaSuccess &&
        qr == cudaDriverEntryPointSuccess)
      fn = (GetRange)sym;
    else
      cudaGetLastError();
  }
  if (!fn) return false;
  size_t size = 0;
  return fn(&base, &size, (unsigned long long)(uintptr_t)p) == 0;
}

static std::mutex g_ipcMutex;
static std::unordered_map<void*, void*> g_ipcBases;  // mapped buffer address -> mapped allocation base

int cutt_mg_ipc_export(void* devptr, unsigned char token[CUTT_MG_IPC_BYTES]) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "token layout");
  if (!devptr || !token) return CUTT_INVALID_PARAMETER;
  unsigned long long base = 0;
  if (!allocation_base(devptr, base)) return CUTT_INTERNAL_ERROR;
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, (void*)(uintptr_t)base) != cudaSuccess) { cudaGetLastError(); return CUTT_INTERNAL_ERROR; }
  memset(token, 0, CUTT_MG_IPC_BYTES);
  memcpy(token, &h, sizeof h);
  unsigned long long off = (unsigned long long)(uintptr_t)devptr - base;
  memcpy(token + 64, &off, sizeof off);
  return CUTT_SUCCESS;
}

int cutt_mg_ipc_open(const unsigned char token[CUTT_MG_IPC_BYTES], void** devptr) {
  if (!devptr || !token) return CUTT_INVALID_PARAMETER;
  cudaIpcMemHandle_t h;
  memcpy(&h, token, sizeof h);
  unsigned long long off = 0;
  memcpy(&off, token + 64, sizeof off);
  void* base = nullptr;
  if (cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
    cudaGetLastError();
    return CUTT_INTERNAL_ERROR;
  }
  *devptr = (unsigned char*)base + off;
  std::lock_guard<std::mutex> lk(g_ipcMutex);
  g_ipcBases[*devptr] = base;
  return CUTT_SUCCESS;
}

int cutt_mg_ipc_close(void* devptr) {
  if (!devptr) return CUTT_INVALID_PARAMETER;
  void* base = nullptr;
  {
    std::lock_guard<std::mutex> lk(g_ipcMutex);
    auto it = g_ipcBases.find(devptr);
    if (it == g_ipcBases.end()) return CUTT_INVALID_PARAMETER;
    base = it->second;
    g_ipcBases.erase(it);
  }
  return cudaIpcCloseMemHandle(base) == cudaSuccess ? CUTT_SUCCESS : CUTT_INTERNAL_ERROR;
}

int cutt_mg_enable_peer_access(int world) {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaGetDeviceCount(&n) != cudaSuccess) return CUTT_INTERNAL_ERROR;
  if (world < 1 || world > n) return CUTT_INVALID_PARAMETER;
  for (int d = 0; d < world; d++) {
    if (d == dev) continue;
    int can = 0;
    if (cudaDeviceCanAccessPeer(&can, dev, d) != cudaSuccess || !can) return CUTT_INVALID_DEVICE;
    cudaError_t e = cudaDeviceEnablePeerAccess(d, 0);
    if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); return CUTT_INTERNAL_ERROR; }
    cudaGetLastError();
  }
  return CUTT_SUCCESS;
}

unsigned long long cutt_c_launch_count(void) { return launch_count(); }

int cutt_c_copy_timeouts(void) { return bulk_copy_timeouts(); }

void cutt_c_debug_force_wide(int on) {
  std::lock_guard<std::mutex> lk(g_mutex);
  debug_force_wide_offsets(on != 0);
  g_enumKey.clear();   // candidate lists built so far no longer apply
  g_enumList.clear();
}

void cutt_c_clear_plan_cache(void) {
  std::lock_guard<std::mutex> lk(g_mutex);
  plan_cache().clear();
}

static const char kPlanCacheHeader[] = "# cutt-b200 plan cache v4";

// One line per entry: key, method and the tile parameters of the measured winner.
int cutt_c_plan_cache_save(const char* path) {
  if (!path) return CUTT_INVALID_PARAMETER;
  std::lock_guard<std::mutex> lk(g_mutex);
  FILE* f = fopen(path, "w");
  if (!f) return CUTT_INTERNAL_ERROR;
  fprintf(f, "%s\n", kPlanCacheHeader);
  plan_cache().for_each_oldest_first([&](const std::string& k, const CachedChoice& c) {
    const TileParams& t = c.params;
    fprintf(f, "%s %d %u %u %u %d %d %d %d %d %d %d %d %d %d %d %d\n", k.c_str(), (int)c.method, t.tinBytes, t.toutBytes,
            t.vtargetBytes, t.extend, t.nthreads, t.stages, t.maxVecBytes, t.maxVBytes, t.loopOrder,
            t.groupIn, t.groupOut, t.cutInRun, t.allowAof, t.oneTilePerBlock, t.peerOrder);
  });
  fclose(f);
  return CUTT_SUCCESS;
}

// Only files written by cutt_c_plan_cache_save of this format version are accepted (first line =
// the version header); lines whose method or tile parameters are out of range are skipped.  What
// is loaded is still only a hint: cuttPlan re-validates every entry against the problem it is
// asked to plan before using it.
int cutt_c_plan_cache_load(const char* path) {
  if (!path) return CUTT_INVALID_PARAMETER;
  std::lock_guard<std::mutex> lk(g_mutex);
  FILE* f = fopen(path, "r");
  if (!f) return CUTT_INVALID_PARAMETER;
  char line[1024];
  const size_t hl = strlen(kPlanCacheHeader);
  if (!fgets(line, sizeof line, f) || strncmp(line, kPlanCacheHeader, hl) != 0 ||
      (line[hl] != '\n' && line[hl] != '\r' && line[hl] != '\0')) {
    fclose(f);
    return CUTT_INVALID_PARAMETER;
  }
  int n = 0;
  while (fgets(line, sizeof line, f)) {
    if (line[0] == '#') continue;
    char key[512];
    int method;
    CachedChoice c;
    TileParams& t = c.params;
    if (sscanf(line, "%511s %d %u %u %u %d %d %d %d %d %d %d %d %d %d %d %d", key, &method, &t.tinBytes, &t.toutBytes,
               &t.vtargetBytes, &t.extend, &t.nthreads, &t.stages, &t.maxVecBytes, &t.maxVBytes,
               &t.loopOrder, &t.groupIn, &t.groupOut, &t.cutInRun, &t.allowAof, &t.oneTilePerBlock,
               &t.peerOrder) != 17)
      continue;
    // winners are tiled plans, row copies, the element-per-thread kernel (small tensors) or, for
    // identity permutations, the two copy methods
    if (method != kMethodTiles && method != kMethodRowCopy && method != kMethodCopy && method != kMethodMemcpy &&
        method != kMethodTma && method != kMethodT2d && method != kMethodNaive)
      continue;
    if ((method == kMethodTiles || method == kMethodTma || method == kMethodT2d) && !valid_tile_params(t, (Method)method))
      continue;
    c.method = (Method)method;
    plan_cache().put(key, c);
    n++;
  }
  fclose(f);
  return n > 0 ? CUTT_SUCCESS : CUTT_INVALID_PARAMETER;
}

int cutt_c_plan_cache_size(void) {
  std::lock_guard<std::mutex> lk(g_mutex);
  return (int)plan_cache().size();
}

const char* cutt_c_version(void) { return "cutt-b200 0.1 (sm_100a)"; }

}  // extern "C"
