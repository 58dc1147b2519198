// Symmetric-memory allocator on the CUDA virtual-memory-management API: physical allocations that can be exported as file
// descriptors, imported and mapped by peer processes (one per GPU), and bound to an NVSwitch multicast object so that one
// `multimem` store / load-reduce reaches every rank's copy.  The driver entry points are looked up through the runtime
// (no link against libcuda).  Every call returns 0 on success or a CUresult / errno-style code; nothing here launches a
// kernel or waits on the device.
//
//   owner:  id = mmb_vmm_create(dev, bytes)        fd = mmb_vmm_export_fd(id)         ... send fd to the peers ...
//   peer:   id = mmb_vmm_import_fd(fd, bytes, dev)  ptr = mmb_vmm_ptr(id)             (mapped read / write for `dev`)
//   NVLS:   rank 0: mc = mmb_mc_create(n_dev, bytes), fd = mmb_mc_export_fd(mc); others: mc = mmb_mc_import_fd(fd, n_dev, bytes)
//           every rank: mmb_mc_add_device(mc, dev); (barrier); mmb_mc_bind(mc, id); va = mmb_mc_map(mc, dev)
#include <cuda.h>
#include <cuda_runtime.h>
#include <unistd.h>

#include <mutex>
#include <unordered_map>

#include "api_vmm.h"

#define MMB_API extern "C" __attribute__((visibility("default")))

namespace {

template <typename F>
F entry(const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) return nullptr;
  return reinterpret_cast<F>(p);
}

struct Api {
  CUresult (*memCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
  CUresult (*memRelease)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*addrReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*addrFree)(CUdeviceptr, size_t) = nullptr;
  CUresult (*memMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*memUnmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*setAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  CUresult (*exportH)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long) = nullptr;
  CUresult (*importH)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType) = nullptr;
  CUresult (*granularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
  CUresult (*mcCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*) = nullptr;
  CUresult (*mcAddDevice)(CUmemGenericAllocationHandle, CUdevice) = nullptr;
  CUresult (*mcBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long) = nullptr;
  CUresult (*mcGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags) = nullptr;
  CUresult (*mcUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t) = nullptr;
  bool ok = false, mc_ok = false;
};

Api& api() {
  static Api a;
  static std::once_flag once;
  std::call_once(once, [] {
    a.memCreate = entry<decltype(a.memCreate)>("cuMemCreate");
    a.memRelease = entry<decltype(a.memRelease)>("cuMemRelease");
    a.addrReserve = entry<decltype(a.addrReserve)>("cuMemAddressReserve");
    a.addrFree = entry<decltype(a.addrFree)>("cuMemAddressFree");
    a.memMap = entry<decltype(a.memMap)>("cuMemMap");
    a.memUnmap = entry<decltype(a.memUnmap)>("cuMemUnmap");
    a.setAccess = entry<decltype(a.setAccess)>("cuMemSetAccess");
    a.exportH = entry<decltype(a.exportH)>("cuMemExportToShareableHandle");
    a.importH = entry<decltype(a.importH)>("cuMemImportFromShareableHandle");
    a.granularity = entry<decltype(a.granularity)>("cuMemGetAllocationGranularity");
    a.mcCreate = entry<decltype(a.mcCreate)>("cuMulticastCreate");
    a.mcAddDevice = entry<decltype(a.mcAddDevice)>("cuMulticastAddDevice");
    a.mcBindMem = entry<decltype(a.mcBindMem)>("cuMulticastBindMem");
    a.mcGranularity = entry<decltype(a.mcGranularity)>("cuMulticastGetGranularity");
    a.mcUnbind = entry<decltype(a.mcUnbind)>("cuMulticastUnbind");
    a.ok = a.memCreate && a.memRelease && a.addrReserve && a.addrFree && a.memMap && a.memUnmap && a.setAccess && a.exportH && a.importH &&
           a.granularity;
    a.mc_ok = a.ok && a.mcCreate && a.mcAddDevice && a.mcBindMem && a.mcGranularity && a.mcUnbind;
  });
  return a;
}

struct Block {
  CUmemGenericAllocationHandle h = 0;
  CUdeviceptr va = 0;
  size_t size = 0;
  int dev = 0;
  bool multicast = false;
  bool mapped = false;
};

std::mutex g_mu;
std::unordered_map<long long, Block> g_blocks;
long long g_next = 1;

CUmemAllocationProp prop_for(int dev) {
  CUmemAllocationProp p{};
  p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  p.location.id = dev;
  p.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return p;
}

int map_block(Block& b, int dev, size_t align) {
  Api& a = api();
  CUresult r = a.addrReserve(&b.va, b.size, align, 0, 0);
  if (r != CUDA_SUCCESS) return (int)r;
  r = a.memMap(b.va, b.size, 0, b.h, 0);
  if (r != CUDA_SUCCESS) {
    a.addrFree(b.va, b.size);
    b.va = 0;
    return (int)r;
  }
  CUmemAccessDesc acc{};
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = dev;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  r = a.setAccess(b.va, b.size, &acc, 1);
  if (r != CUDA_SUCCESS) {
    a.memUnmap(b.va, b.size);
    a.addrFree(b.va, b.size);
    b.va = 0;
    return (int)r;
  }
  b.mapped = true;
  return 0;
}

long long put(const Block& b) {
  std::lock_guard<std::mutex> lk(g_mu);
  const long long id = g_next++;
  g_blocks[id] = b;
  return id;
}

bool get(long long id, Block* out) {
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_blocks.find(id);
  if (it == g_blocks.end()) return false;
  *out = it->second;
  return true;
}

}  // namespace

MMB_API int mmb_vmm_available(void) { return api().ok ? (api().mc_ok ? 2 : 1) : 0; }

MMB_API long long mmb_vmm_granularity(int dev) {
  Api& a = api();
  if (!a.ok) return -1;
  cudaSetDevice(dev);
  cudaFree(nullptr);
  CUmemAllocationProp p = prop_for(dev);
  size_t g = 0;
  if (a.granularity(&g, &p, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS) return -1;
  return (long long)g;
}

// New physical allocation on `dev`, mapped read / write for `dev`.  `bytes` is rounded up to the allocation granularity.
// Returns an id > 0, or the negated error code.
MMB_API long long mmb_vmm_create(int dev, long long bytes) {
  Api& a = api();
  if (!a.ok || bytes <= 0) return -1;
  cudaSetDevice(dev);
  cudaFree(nullptr);      // makes sure the primary context exists
  const long long g = mmb_vmm_granularity(dev);
  if (g <= 0) return -2;
  Block b;
  b.dev = dev;
  b.size = (size_t)((bytes + g - 1) / g * g);
  CUmemAllocationProp p = prop_for(dev);
  CUresult r = a.memCreate(&b.h, b.size, &p, 0);
  if (r != CUDA_SUCCESS) return -(long long)r;
  const int e = map_block(b, dev, (size_t)g);
  if (e) {
    a.memRelease(b.h);
    return -(long long)e;
  }
  return put(b);
}

MMB_API int mmb_vmm_export_fd(long long id) {
  Block b;
  if (!get(id, &b)) return -1;
  int fd = -1;
  CUresult r = api().exportH(&fd, b.h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  return r == CUDA_SUCCESS ? fd : -(int)r;
}

// Maps an allocation exported by another process (or this one) for device `dev`.  The descriptor stays owned by the caller.
MMB_API long long mmb_vmm_import_fd(int fd, long long bytes, int dev) {
  Api& a = api();
  if (!a.ok || fd < 0 || bytes <= 0) return -1;
  cudaSetDevice(dev);
  cudaFree(nullptr);
  const long long g = mmb_vmm_granularity(dev);
  if (g <= 0) return -2;
  Block b;
  b.dev = dev;
  b.size = (size_t)((bytes + g - 1) / g * g);
  CUresult r = a.importH(&b.h, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  if (r != CUDA_SUCCESS) return -(long long)r;
  const int e = map_block(b, dev, (size_t)g);
  if (e) {
    a.memRelease(b.h);
    return -(long long)e;
  }
  return put(b);
}

MMB_API long long mmb_vmm_ptr(long long id) {
  Block b;
  return get(id, &b) ? (long long)b.va : 0;
}

MMB_API long long mmb_vmm_size(long long id) {
  Block b;
  return get(id, &b) ? (long long)b.size : 0;
}

MMB_API int mmb_vmm_free(long long id) {
  Block b;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_blocks.find(id);
    if (it == g_blocks.end()) return -1;
    b = it->second;
    g_blocks.erase(it);
  }
  Api& a = api();
  if (b.mapped && b.va) {
    a.memUnmap(b.va, b.size);
    a.addrFree(b.va, b.size);
  }
  if (b.h) a.memRelease(b.h);
  return 0;
}

// ---- NVSwitch multicast objects
static CUmulticastObjectProp mc_prop(int n_dev, size_t size) {
  CUmulticastObjectProp p{};
  p.numDevices = (unsigned)n_dev;
  p.size = size;
  p.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return p;
}

MMB_API long long mmb_mc_granularity(int n_dev, long long bytes) {
  Api& a = api();
  if (!a.mc_ok) return -1;
  CUmulticastObjectProp p = mc_prop(n_dev, (size_t)bytes);
  size_t g = 0;
  if (a.mcGranularity(&g, &p, CU_MULTICAST_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS) return -1;
  return (long long)g;
}

MMB_API long long mmb_mc_create(int n_dev, long long bytes) {
  Api& a = api();
  if (!a.mc_ok || bytes <= 0) return -1;
  cudaFree(nullptr);
  const long long g = mmb_mc_granularity(n_dev, bytes);
  if (g <= 0) return -2;
  Block b;
  b.multicast = true;
  b.size = (size_t)((bytes + g - 1) / g * g);
  CUmulticastObjectProp p = mc_prop(n_dev, b.size);
  CUresult r = a.mcCreate(&b.h, &p);
  if (r != CUDA_SUCCESS) return -(long long)r;
  return put(b);
}

MMB_API int mmb_mc_export_fd(long long id) { return mmb_vmm_export_fd(id); }

MMB_API long long mmb_mc_import_fd(int fd, int n_dev, long long bytes) {
  Api& a = api();
  if (!a.mc_ok || fd < 0) return -1;
  cudaFree(nullptr);
  const long long g = mmb_mc_granularity(n_dev, bytes);
  if (g <= 0) return -2;
  Block b;
  b.multicast = true;
  b.size = (size_t)((bytes + g - 1) / g * g);
  CUresult r = a.importH(&b.h, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  if (r != CUDA_SUCCESS) return -(long long)r;
  return put(b);
}

MMB_API int mmb_mc_add_device(long long mc, int dev) {
  Block b;
  if (!get(mc, &b) || !b.multicast) return -1;
  CUdevice d = 0;
  cudaSetDevice(dev);
  cudaFree(nullptr);
  d = (CUdevice)dev;
  return (int)api().mcAddDevice(b.h, d);
}

// Binds the whole physical allocation `mem` at offset 0 of the multicast object (after every device was added).
MMB_API int mmb_mc_bind(long long mc, long long mem) {
  Block m, b;
  if (!get(mc, &m) || !m.multicast || !get(mem, &b) || b.multicast || b.size > m.size) return -1;
  return (int)api().mcBindMem(m.h, 0, b.h, 0, b.size, 0);
}

// Maps the multicast object for `dev`; the returned address is the `multimem` view of all bound copies (0 on failure).
MMB_API long long mmb_mc_map(long long mc, int dev) {
  Block m;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_blocks.find(mc);
    if (it == g_blocks.end() || !it->second.multicast) return 0;
    if (it->second.mapped) return (long long)it->second.va;
    m = it->second;
  }
  cudaSetDevice(dev);
  const long long g = mmb_mc_granularity(1, (long long)m.size);
  m.dev = dev;
  if (map_block(m, dev, (size_t)(g > 0 ? g : (2 << 20)))) return 0;
  std::lock_guard<std::mutex> lk(g_mu);
  g_blocks[mc] = m;
  return (long long)m.va;
}

MMB_API int mmb_mc_unbind(long long mc, int dev, long long mem) {
  Block m, b;
  if (!get(mc, &m) || !m.multicast || !get(mem, &b)) return -1;
  return (int)api().mcUnbind(m.h, (CUdevice)dev, 0, b.size);
}

MMB_API void mmb_close_fd(int fd) {
  if (fd >= 0) close(fd);
}
