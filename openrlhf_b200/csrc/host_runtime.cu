// Host-side native runtime pieces of the rollout engine (no device code in this file):
//
//  * PagePool  - reference-counted KV page allocator (free list, prefix sharing between the n samples of a prompt);
//                the role vLLM's block manager plays for the reference (openrlhf/trainer/ray/vllm_engine.py:63-64).
//  * admit     - continuous-batching admission: how many queued requests fit into the free rows and pages.
//  * VmmArena  - a virtual address range whose physical backing can be released and re-created without changing the
//                address (cuMemAddressReserve / cuMemCreate / cuMemMap / cuMemUnmap): sleep / wake of the KV cache
//                keeps every captured CUDA graph valid. Counterpart of vLLM's sleep mode as the reference drives it
//                (openrlhf/trainer/ray/vllm_engine.py:138-153). Driver entry points are resolved at run time, so the
//                library has no link-time dependency on libcuda.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <vector>

namespace {

struct PagePool {
  std::vector<int> free_list;
  std::vector<int> ref;
  std::mutex mu;
};

template <typename Fn>
Fn driver_fn(const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
    return nullptr;
  return reinterpret_cast<Fn>(p);
}

struct VmmArena {
  CUdeviceptr va = 0;
  size_t size = 0;        // reserved (and mapped) bytes, multiple of the granularity
  size_t gran = 0;
  int device = 0;
  bool mapped = false;
  CUmemGenericAllocationHandle handle = 0;
};

typedef CUresult (*GranFn)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
typedef CUresult (*ReserveFn)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
typedef CUresult (*CreateFn)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
typedef CUresult (*MapFn)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
typedef CUresult (*AccessFn)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
typedef CUresult (*UnmapFn)(CUdeviceptr, size_t);
typedef CUresult (*ReleaseFn)(CUmemGenericAllocationHandle);
typedef CUresult (*FreeVaFn)(CUdeviceptr, size_t);

CUmemAllocationProp props_for(int device) {
  CUmemAllocationProp prop = {};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  return prop;
}

}  // namespace

// ---------------------------------------------------------------------------------------------- page pool
extern "C" void* b200_pool_create(int num_pages) {
  PagePool* p = new PagePool();
  p->ref.assign(num_pages, 0);
  p->free_list.reserve(num_pages);
  for (int i = num_pages - 1; i >= 0; --i) p->free_list.push_back(i);
  return p;
}
extern "C" void b200_pool_destroy(void* h) { delete static_cast<PagePool*>(h); }
extern "C" int b200_pool_num_free(void* h) {
  PagePool* p = static_cast<PagePool*>(h);
  std::lock_guard<std::mutex> g(p->mu);
  return (int)p->free_list.size();
}
// Returns the page index, or -1 when the pool is exhausted.
extern "C" int b200_pool_alloc(void* h) {
  PagePool* p = static_cast<PagePool*>(h);
  std::lock_guard<std::mutex> g(p->mu);
  if (p->free_list.empty()) return -1;
  int page = p->free_list.back();
  p->free_list.pop_back();
  p->ref[page] = 1;
  return page;
}
// Allocates n pages at once into out[]; all-or-nothing. Returns 0 or -1.
extern "C" int b200_pool_alloc_many(void* h, int n, int* out) {
  PagePool* p = static_cast<PagePool*>(h);
  std::lock_guard<std::mutex> g(p->mu);
  if ((int)p->free_list.size() < n) return -1;
  for (int i = 0; i < n; ++i) {
    out[i] = p->free_list.back();
    p->free_list.pop_back();
    p->ref[out[i]] = 1;
  }
  return 0;
}
extern "C" int b200_pool_share(void* h, int page) {
  PagePool* p = static_cast<PagePool*>(h);
  std::lock_guard<std::mutex> g(p->mu);
  if (page < 0 || page >= (int)p->ref.size() || p->ref[page] <= 0) return -1;
  return ++p->ref[page];
}
// Returns the remaining reference count, or -1 on a double free / bad index.
extern "C" int b200_pool_free(void* h, int page) {
  PagePool* p = static_cast<PagePool*>(h);
  std::lock_guard<std::mutex> g(p->mu);
  if (page < 0 || page >= (int)p->ref.size() || p->ref[page] <= 0) return -1;
  if (--p->ref[page] == 0) p->free_list.push_back(page);
  return p->ref[page];
}

// Continuous-batching admission in queue order: request i needs n[i] rows and
// n[i] * ((prompt[i] + max_new[i]) / page + 1) pages (upper bound without prefix sharing). Stops at the first request
// that does not fit (no reordering, so long requests are not starved). Returns the number admitted.
extern "C" int b200_admit(const int* prompt_len, const int* max_new, const int* n, int count, int free_rows,
                          int free_pages, int page_size, int reserve_pages) {
  int admitted = 0;
  for (int i = 0; i < count; ++i) {
    const long long pages = (long long)n[i] * ((prompt_len[i] + max_new[i]) / page_size + 1);
    if (n[i] > free_rows || pages + reserve_pages > free_pages) break;
    free_rows -= n[i];
    free_pages -= (int)pages;
    ++admitted;
  }
  return admitted;
}

// ---------------------------------------------------------------------------------------------- VMM arena
// Reserve `bytes` (rounded up to the allocation granularity) of virtual address space on `device` and back it with
// physical memory. Returns a handle or null; *out_ptr / *out_size receive the address and the rounded size.
extern "C" void* b200_arena_create(size_t bytes, int device, unsigned long long* out_ptr, size_t* out_size) {
  auto gran_fn = driver_fn<GranFn>("cuMemGetAllocationGranularity");
  auto reserve = driver_fn<ReserveFn>("cuMemAddressReserve");
  if (!gran_fn || !reserve) return nullptr;
  cudaFree(0);  // make sure the primary context exists
  CUmemAllocationProp prop = props_for(device);
  size_t gran = 0;
  if (gran_fn(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS || gran == 0) return nullptr;
  VmmArena* a = new VmmArena();
  a->gran = gran;
  a->device = device;
  a->size = (bytes + gran - 1) / gran * gran;
  if (reserve(&a->va, a->size, gran, 0, 0) != CUDA_SUCCESS) {
    delete a;
    return nullptr;
  }
  if (out_ptr) *out_ptr = (unsigned long long)a->va;
  if (out_size) *out_size = a->size;
  return a;
}
// Back the range with physical memory (no-op when already mapped). Returns 0 on success.
extern "C" int b200_arena_map(void* h) {
  VmmArena* a = static_cast<VmmArena*>(h);
  if (a->mapped) return 0;
  auto create = driver_fn<CreateFn>("cuMemCreate");
  auto map = driver_fn<MapFn>("cuMemMap");
  auto access = driver_fn<AccessFn>("cuMemSetAccess");
  auto release = driver_fn<ReleaseFn>("cuMemRelease");
  if (!create || !map || !access || !release) return -1;
  CUmemAllocationProp prop = props_for(a->device);
  if (create(&a->handle, a->size, &prop, 0) != CUDA_SUCCESS) return -2;
  if (map(a->va, a->size, 0, a->handle, 0) != CUDA_SUCCESS) {
    release(a->handle);
    return -3;
  }
  CUmemAccessDesc desc = {};
  desc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  desc.location.id = a->device;
  desc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  if (access(a->va, a->size, &desc, 1) != CUDA_SUCCESS) return -4;
  a->mapped = true;
  return 0;
}
// Release the physical memory, keep the address range. The caller synchronises the device first.
extern "C" int b200_arena_unmap(void* h) {
  VmmArena* a = static_cast<VmmArena*>(h);
  if (!a->mapped) return 0;
  auto unmap = driver_fn<UnmapFn>("cuMemUnmap");
  auto release = driver_fn<ReleaseFn>("cuMemRelease");
  if (!unmap || !release) return -1;
  if (unmap(a->va, a->size) != CUDA_SUCCESS) return -2;
  if (release(a->handle) != CUDA_SUCCESS) return -3;
  a->mapped = false;
  return 0;
}
extern "C" int b200_arena_is_mapped(void* h) { return static_cast<VmmArena*>(h)->mapped ? 1 : 0; }
extern "C" int b200_arena_destroy(void* h) {
  VmmArena* a = static_cast<VmmArena*>(h);
  int rc = b200_arena_unmap(h);
  auto free_va = driver_fn<FreeVaFn>("cuMemAddressFree");
  if (free_va) free_va(a->va, a->size);
  delete a;
  return rc;
}
