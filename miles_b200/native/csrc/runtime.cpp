// Native runtime pieces with a C ABI (loaded through ctypes; no torch or CUDA headers needed to build):
//   * BlockAllocator  — KV-cache block free list with reference counts (shared prefixes), O(1) alloc/release.
//   * VmmArena        — a CUDA virtual-memory arena with tagged pause/resume: allocations keep their virtual
//                       addresses while their physical pages are released (optionally saved to host) and mapped
//                       again later.  This is what lets a colocated trainer and rollout engine hand the GPU back and
//                       forth without invalidating pointers captured in CUDA graphs or peer mappings.
//                       The CUDA driver is loaded with dlopen at first use so the library builds and loads on
//                       machines without a GPU.
//   * LeastLoadRouter — request → worker choice (least active requests, round robin, consistent hashing).
#include <dlfcn.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <map>
#include <mutex>
#include <string>
#include <vector>

extern "C" {

// ------------------------------------------------------------------------------------------------
// BlockAllocator
// ------------------------------------------------------------------------------------------------
struct BlockAllocator {
  std::vector<int32_t> free_list;
  std::vector<int32_t> refcnt;
  std::mutex mu;
};

void* mbrt_alloc_create(int32_t num_blocks) {
  auto* a = new BlockAllocator();
  a->refcnt.assign(num_blocks, 0);
  a->free_list.reserve(num_blocks);
  for (int32_t b = num_blocks - 1; b >= 0; --b) a->free_list.push_back(b);
  return a;
}
void mbrt_alloc_destroy(void* h) { delete static_cast<BlockAllocator*>(h); }
int32_t mbrt_alloc_num_free(void* h) {
  auto* a = static_cast<BlockAllocator*>(h);
  std::lock_guard<std::mutex> g(a->mu);
  return static_cast<int32_t>(a->free_list.size());
}
// returns 0 on success (out[0..n) filled), −1 when fewer than n blocks are free (nothing allocated)
int32_t mbrt_alloc_take(void* h, int32_t n, int32_t* out) {
  auto* a = static_cast<BlockAllocator*>(h);
  std::lock_guard<std::mutex> g(a->mu);
  if (static_cast<size_t>(n) > a->free_list.size()) return -1;
  for (int32_t i = 0; i < n; ++i) {
    out[i] = a->free_list.back();
    a->free_list.pop_back();
    a->refcnt[out[i]] = 1;
  }
  return 0;
}
void mbrt_alloc_share(void* h, const int32_t* blocks, int32_t n) {
  auto* a = static_cast<BlockAllocator*>(h);
  std::lock_guard<std::mutex> g(a->mu);
  for (int32_t i = 0; i < n; ++i) a->refcnt[blocks[i]] += 1;
}
// returns the number of blocks that became free, or −1 on a double release
int32_t mbrt_alloc_release(void* h, const int32_t* blocks, int32_t n) {
  auto* a = static_cast<BlockAllocator*>(h);
  std::lock_guard<std::mutex> g(a->mu);
  int32_t freed = 0;
  for (int32_t i = 0; i < n; ++i) {
    int32_t& r = a->refcnt[blocks[i]];
    if (r <= 0) return -1;
    if (--r == 0) {
      a->free_list.push_back(blocks[i]);
      ++freed;
    }
  }
  return freed;
}
void mbrt_alloc_reset(void* h) {
  auto* a = static_cast<BlockAllocator*>(h);
  std::lock_guard<std::mutex> g(a->mu);
  const int32_t n = static_cast<int32_t>(a->refcnt.size());
  std::fill(a->refcnt.begin(), a->refcnt.end(), 0);
  a->free_list.clear();
  for (int32_t b = n - 1; b >= 0; --b) a->free_list.push_back(b);
}

// ------------------------------------------------------------------------------------------------
// CUDA driver entry points (resolved lazily)
// ------------------------------------------------------------------------------------------------
typedef int CUresult;
typedef unsigned long long CUdeviceptr;
typedef unsigned long long CUmemGenericAllocationHandle;
struct CUmemLocation { int type; int id; };
struct CUmemAllocationProp {
  int type; int requestedHandleTypes; CUmemLocation location; void* win32HandleMetaData;
  struct { unsigned char compressionType; unsigned char gpuDirectRDMACapable; unsigned short usage; unsigned char reserved[4]; } allocFlags;
};
struct CUmemAccessDesc { CUmemLocation location; int flags; };

struct Driver {
  void* lib = nullptr;
  CUresult (*cuInit)(unsigned) = nullptr;
  CUresult (*cuMemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, int) = nullptr;
  CUresult (*cuMemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*cuMemAddressFree)(CUdeviceptr, size_t) = nullptr;
  CUresult (*cuMemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
  CUresult (*cuMemRelease)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*cuMemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*cuMemUnmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*cuMemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  CUresult (*cuMemcpyDtoH)(void*, CUdeviceptr, size_t) = nullptr;
  CUresult (*cuMemcpyHtoD)(CUdeviceptr, const void*, size_t) = nullptr;
  CUresult (*cuCtxSynchronize)() = nullptr;
  CUresult (*cuMemHostAlloc)(void**, size_t, unsigned) = nullptr;
  CUresult (*cuMemFreeHost)(void*) = nullptr;
  bool ok = false;
};

static Driver& driver() {
  static Driver d;
  static std::once_flag once;
  std::call_once(once, [] {
    d.lib = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
    if (!d.lib) return;
#define LOAD(name, sym) *reinterpret_cast<void**>(&d.name) = dlsym(d.lib, sym)
    LOAD(cuInit, "cuInit");
    LOAD(cuMemGetAllocationGranularity, "cuMemGetAllocationGranularity");
    LOAD(cuMemAddressReserve, "cuMemAddressReserve");
    LOAD(cuMemAddressFree, "cuMemAddressFree");
    LOAD(cuMemCreate, "cuMemCreate");
    LOAD(cuMemRelease, "cuMemRelease");
    LOAD(cuMemMap, "cuMemMap");
    LOAD(cuMemUnmap, "cuMemUnmap");
    LOAD(cuMemSetAccess, "cuMemSetAccess");
    LOAD(cuMemcpyDtoH, "cuMemcpyDtoH_v2");
    LOAD(cuMemcpyHtoD, "cuMemcpyHtoD_v2");
    LOAD(cuCtxSynchronize, "cuCtxSynchronize");
    LOAD(cuMemHostAlloc, "cuMemHostAlloc");
    LOAD(cuMemFreeHost, "cuMemFreeHost");
#undef LOAD
    d.ok = d.cuInit && d.cuMemCreate && d.cuMemMap && d.cuMemAddressReserve && d.cuMemSetAccess && d.cuMemUnmap &&
           d.cuMemRelease && d.cuMemGetAllocationGranularity && d.cuMemcpyDtoH && d.cuMemcpyHtoD;
    if (d.ok) d.ok = d.cuInit(0) == 0;
  });
  return d;
}

int32_t mbrt_driver_available() { return driver().ok ? 1 : 0; }

// ------------------------------------------------------------------------------------------------
// VmmArena
// ------------------------------------------------------------------------------------------------
struct Region {
  CUdeviceptr va = 0;
  size_t size = 0;
  CUmemGenericAllocationHandle handle = 0;
  bool mapped = false;
  std::string tag;
  void* host_copy = nullptr;
  bool host_pinned = false;      // the saved copy lives in page-locked memory (copies run at PCIe rate)
};

static void* host_alloc(Region& r) {
  Driver& d = driver();
  void* p = nullptr;
  if (d.cuMemHostAlloc && d.cuMemFreeHost && d.cuMemHostAlloc(&p, r.size, 0) == 0 && p) {
    r.host_pinned = true;
    return p;
  }
  r.host_pinned = false;
  return malloc(r.size);
}

static void host_free(Region& r) {
  if (!r.host_copy) return;
  if (r.host_pinned) driver().cuMemFreeHost(r.host_copy);
  else free(r.host_copy);
  r.host_copy = nullptr;
}

struct VmmArena {
  int device = 0;
  size_t granularity = 2 << 20;
  std::map<CUdeviceptr, Region> regions;
  std::mutex mu;
  size_t mapped_bytes = 0;
};

static CUmemAllocationProp make_prop(int device) {
  CUmemAllocationProp p;
  memset(&p, 0, sizeof(p));
  p.type = 1;           // CU_MEM_ALLOCATION_TYPE_PINNED
  p.location.type = 1;  // CU_MEM_LOCATION_TYPE_DEVICE
  p.location.id = device;
  return p;
}

static int map_region(VmmArena* a, Region& r) {
  Driver& d = driver();
  CUmemAllocationProp p = make_prop(a->device);
  if (d.cuMemCreate(&r.handle, r.size, &p, 0) != 0) return -2;
  if (d.cuMemMap(r.va, r.size, 0, r.handle, 0) != 0) { d.cuMemRelease(r.handle); return -3; }
  CUmemAccessDesc acc;
  acc.location.type = 1;
  acc.location.id = a->device;
  acc.flags = 3;  // read/write
  if (d.cuMemSetAccess(r.va, r.size, &acc, 1) != 0) return -4;
  r.mapped = true;
  a->mapped_bytes += r.size;
  return 0;
}

void* mbrt_arena_create(int32_t device) {
  Driver& d = driver();
  if (!d.ok) return nullptr;
  auto* a = new VmmArena();
  a->device = device;
  CUmemAllocationProp p = make_prop(device);
  size_t g = 0;
  if (d.cuMemGetAllocationGranularity(&g, &p, 0) == 0 && g > 0) a->granularity = g;
  return a;
}

// Allocate `bytes` under `tag`; returns the device address (0 on failure).
uint64_t mbrt_arena_malloc(void* h, uint64_t bytes, const char* tag) {
  auto* a = static_cast<VmmArena*>(h);
  Driver& d = driver();
  std::lock_guard<std::mutex> g(a->mu);
  Region r;
  r.size = (bytes + a->granularity - 1) / a->granularity * a->granularity;
  r.tag = tag ? tag : "";
  if (d.cuMemAddressReserve(&r.va, r.size, a->granularity, 0, 0) != 0) return 0;
  if (map_region(a, r) != 0) { d.cuMemAddressFree(r.va, r.size); return 0; }
  a->regions[r.va] = r;
  return r.va;
}

int32_t mbrt_arena_free(void* h, uint64_t ptr) {
  auto* a = static_cast<VmmArena*>(h);
  Driver& d = driver();
  std::lock_guard<std::mutex> g(a->mu);
  auto it = a->regions.find(ptr);
  if (it == a->regions.end()) return -1;
  Region& r = it->second;
  if (r.mapped) {
    d.cuMemUnmap(r.va, r.size);
    d.cuMemRelease(r.handle);
    a->mapped_bytes -= r.size;
  }
  host_free(r);
  d.cuMemAddressFree(r.va, r.size);
  a->regions.erase(it);
  return 0;
}

// Release the physical memory of every region with this tag (all regions when tag is empty).
// keep_contents != 0 saves the bytes to host memory first and restores them on resume.
int64_t mbrt_arena_pause(void* h, const char* tag, int32_t keep_contents) {
  auto* a = static_cast<VmmArena*>(h);
  Driver& d = driver();
  std::lock_guard<std::mutex> g(a->mu);
  if (d.cuCtxSynchronize) d.cuCtxSynchronize();
  int64_t released = 0;
  for (auto& kv : a->regions) {
    Region& r = kv.second;
    if (!r.mapped || (tag && tag[0] && r.tag != tag)) continue;
    if (keep_contents) {
      r.host_copy = host_alloc(r);
      if (!r.host_copy || d.cuMemcpyDtoH(r.host_copy, r.va, r.size) != 0) return -1;
    }
    d.cuMemUnmap(r.va, r.size);
    d.cuMemRelease(r.handle);
    r.mapped = false;
    a->mapped_bytes -= r.size;
    released += static_cast<int64_t>(r.size);
  }
  return released;
}

int64_t mbrt_arena_resume(void* h, const char* tag) {
  auto* a = static_cast<VmmArena*>(h);
  Driver& d = driver();
  std::lock_guard<std::mutex> g(a->mu);
  int64_t restored = 0;
  for (auto& kv : a->regions) {
    Region& r = kv.second;
    if (r.mapped || (tag && tag[0] && r.tag != tag)) continue;
    if (map_region(a, r) != 0) return -1;
    if (r.host_copy) {
      if (d.cuMemcpyHtoD(r.va, r.host_copy, r.size) != 0) return -2;
      host_free(r);
    }
    restored += static_cast<int64_t>(r.size);
  }
  return restored;
}

uint64_t mbrt_arena_mapped_bytes(void* h) { return static_cast<VmmArena*>(h)->mapped_bytes; }

void mbrt_arena_destroy(void* h) {
  auto* a = static_cast<VmmArena*>(h);
  std::vector<CUdeviceptr> ptrs;
  for (auto& kv : a->regions) ptrs.push_back(kv.first);
  for (auto p : ptrs) mbrt_arena_free(h, p);
  delete a;
}

// ------------------------------------------------------------------------------------------------
// Router core: pick a worker for a request
// ------------------------------------------------------------------------------------------------
struct Router {
  std::vector<int32_t> active;
  std::vector<uint8_t> healthy;
  uint64_t rr = 0;
  std::mutex mu;
};

void* mbrt_router_create(int32_t workers) {
  auto* r = new Router();
  r->active.assign(workers, 0);
  r->healthy.assign(workers, 1);
  return r;
}
void mbrt_router_destroy(void* h) { delete static_cast<Router*>(h); }
int32_t mbrt_router_add_worker(void* h) {
  auto* r = static_cast<Router*>(h);
  std::lock_guard<std::mutex> g(r->mu);
  r->active.push_back(0);
  r->healthy.push_back(1);
  return static_cast<int32_t>(r->active.size()) - 1;
}
void mbrt_router_set_health(void* h, int32_t w, int32_t ok) {
  auto* r = static_cast<Router*>(h);
  std::lock_guard<std::mutex> g(r->mu);
  if (w >= 0 && w < static_cast<int32_t>(r->healthy.size())) r->healthy[w] = ok ? 1 : 0;
}
static uint64_t fnv1a(const char* s) {
  uint64_t x = 1469598103934665603ull;
  for (; s && *s; ++s) { x ^= static_cast<unsigned char>(*s); x *= 1099511628211ull; }
  return x;
}
// policy: 0 least-active, 1 round-robin, 2 consistent hashing on `key`, 3 random (hash of counter).
// Returns the worker index (its active count is incremented) or −1 if no healthy worker exists.
int32_t mbrt_router_pick(void* h, int32_t policy, const char* key) {
  auto* r = static_cast<Router*>(h);
  std::lock_guard<std::mutex> g(r->mu);
  const int32_t n = static_cast<int32_t>(r->active.size());
  std::vector<int32_t> ok;
  for (int32_t i = 0; i < n; ++i) if (r->healthy[i]) ok.push_back(i);
  if (ok.empty()) return -1;
  int32_t pick;
  if (policy == 1) {
    pick = ok[r->rr++ % ok.size()];
  } else if (policy == 2 && key && key[0]) {
    pick = ok[fnv1a(key) % ok.size()];
  } else if (policy == 3) {
    uint64_t x = ++r->rr * 0x9E3779B97F4A7C15ull;
    x ^= x >> 29;
    pick = ok[x % ok.size()];
  } else {
    pick = ok[0];
    for (int32_t i : ok) if (r->active[i] < r->active[pick]) pick = i;
  }
  r->active[pick] += 1;
  return pick;
}
void mbrt_router_done(void* h, int32_t w) {
  auto* r = static_cast<Router*>(h);
  std::lock_guard<std::mutex> g(r->mu);
  if (w >= 0 && w < static_cast<int32_t>(r->active.size()) && r->active[w] > 0) r->active[w] -= 1;
}
int32_t mbrt_router_active(void* h, int32_t w) {
  auto* r = static_cast<Router*>(h);
  std::lock_guard<std::mutex> g(r->mu);
  return (w >= 0 && w < static_cast<int32_t>(r->active.size())) ? r->active[w] : -1;
}

}  // extern "C"
