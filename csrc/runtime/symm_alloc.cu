#include "symm_alloc.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>

namespace sar {
namespace {

// Driver entry points, looked up once through the runtime.
struct Driver {
  bool tried = false, ok = false;
  decltype(&cuDeviceGet) DeviceGet = nullptr;
  decltype(&cuDeviceGetAttribute) DeviceGetAttribute = nullptr;
  decltype(&cuGetErrorString) GetErrorString = nullptr;
  decltype(&cuMemCreate) MemCreate = nullptr;
  decltype(&cuMemRelease) MemRelease = nullptr;
  decltype(&cuMemAddressReserve) MemAddressReserve = nullptr;
  decltype(&cuMemAddressFree) MemAddressFree = nullptr;
  decltype(&cuMemMap) MemMap = nullptr;
  decltype(&cuMemUnmap) MemUnmap = nullptr;
  decltype(&cuMemSetAccess) MemSetAccess = nullptr;
  decltype(&cuMemGetAllocationGranularity) MemGetAllocationGranularity = nullptr;
  decltype(&cuMulticastCreate) MulticastCreate = nullptr;
  decltype(&cuMulticastAddDevice) MulticastAddDevice = nullptr;
  decltype(&cuMulticastBindMem) MulticastBindMem = nullptr;
  decltype(&cuMulticastUnbind) MulticastUnbind = nullptr;
  decltype(&cuMulticastGetGranularity) MulticastGetGranularity = nullptr;
};

template <typename F>
bool lookup(F& fn, const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || !p) {
    cudaGetLastError();
    return false;
  }
  fn = reinterpret_cast<F>(p);
  return true;
}

Driver& driver() {
  static Driver d;
  if (d.tried) return d;
  d.tried = true;
  d.ok = lookup(d.DeviceGet, "cuDeviceGet") && lookup(d.DeviceGetAttribute, "cuDeviceGetAttribute") &&
         lookup(d.GetErrorString, "cuGetErrorString") && lookup(d.MemCreate, "cuMemCreate") &&
         lookup(d.MemRelease, "cuMemRelease") && lookup(d.MemAddressReserve, "cuMemAddressReserve") &&
         lookup(d.MemAddressFree, "cuMemAddressFree") && lookup(d.MemMap, "cuMemMap") && lookup(d.MemUnmap, "cuMemUnmap") &&
         lookup(d.MemSetAccess, "cuMemSetAccess") && lookup(d.MemGetAllocationGranularity, "cuMemGetAllocationGranularity") &&
         lookup(d.MulticastCreate, "cuMulticastCreate") && lookup(d.MulticastAddDevice, "cuMulticastAddDevice") &&
         lookup(d.MulticastBindMem, "cuMulticastBindMem") && lookup(d.MulticastUnbind, "cuMulticastUnbind") &&
         lookup(d.MulticastGetGranularity, "cuMulticastGetGranularity");
  return d;
}

int fail(char* err, int errlen, const char* what, CUresult r) {
  if (err && errlen > 0) {
    const char* s = nullptr;
    Driver& d = driver();
    if (d.GetErrorString) d.GetErrorString(r, &s);
    snprintf(err, (size_t)errlen, "%s: %s (CUresult %d)", what, s ? s : "?", (int)r);
  }
  return 1;
}
int fail_msg(char* err, int errlen, const char* msg) {
  if (err && errlen > 0) snprintf(err, (size_t)errlen, "%s", msg);
  return 1;
}

size_t round_up(size_t x, size_t g) { return (x + g - 1) / g * g; }
int popcount(uint32_t x) { int c = 0; while (x) { c += x & 1; x >>= 1; } return c; }

int alloc_plain(SymmAlloc* a, char* err, int errlen) {
  for (int r = 0; r < a->n; ++r) {
    cudaError_t e = cudaSetDevice(a->dev[r]);
    if (e == cudaSuccess) e = cudaMalloc(&a->uc[r], a->bytes < 16 ? 16 : a->bytes);
    if (e != cudaSuccess) {
      if (err && errlen > 0) snprintf(err, (size_t)errlen, "cudaMalloc of %zu bytes on device %d: %s", a->bytes, a->dev[r], cudaGetErrorString(e));
      symm_free(a);
      return 1;
    }
  }
  a->mapped = a->bytes;
  return 0;
}

#define DRV(call, what)                                   \
  do {                                                    \
    CUresult r_ = (call);                                 \
    if (r_ != CUDA_SUCCESS) {                             \
      fail(err, errlen, what, r_);                        \
      symm_free(a);                                       \
      return 1;                                           \
    }                                                     \
  } while (0)

int alloc_multicast(SymmAlloc* a, uint32_t sub_members, char* err, int errlen) {
  Driver& d = driver();
  const int n = a->n;
  for (int r = 0; r < n; ++r)
    for (int q = 0; q < r; ++q)
      if (a->dev[r] == a->dev[q]) return fail_msg(err, errlen, "multicast needs one device per rank");
  CUdevice cudev[SAR_MAX_RANKS];
  for (int r = 0; r < n; ++r) {
    if (cudaSetDevice(a->dev[r]) != cudaSuccess || cudaFree(nullptr) != cudaSuccess)   // the primary context exists
      return fail_msg(err, errlen, "cannot initialise a device");
    CUresult rc = d.DeviceGet(&cudev[r], a->dev[r]);
    if (rc != CUDA_SUCCESS) return fail(err, errlen, "cuDeviceGet", rc);
  }
  a->vmm = true;
  a->members[0] = n >= 32 ? 0xffffffffu : ((1u << n) - 1u);
  a->members[1] = sub_members & a->members[0];
  if (a->members[1] == a->members[0] || popcount(a->members[1]) < 2) a->members[1] = 0;

  // sizes: a multiple of the allocation granularity and of every group's multicast granularity
  size_t gran = 0;
  CUmemAllocationProp prop;
  memset(&prop, 0, sizeof prop);
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = cudev[0];
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_NONE;
  DRV(d.MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED), "cuMemGetAllocationGranularity");
  CUmulticastObjectProp mcprop[2];
  for (int g = 0; g < 2; ++g) {
    memset(&mcprop[g], 0, sizeof mcprop[g]);
    if (!a->members[g]) continue;
    mcprop[g].numDevices = (unsigned)popcount(a->members[g]);
    mcprop[g].handleTypes = CU_MEM_HANDLE_TYPE_NONE;
    mcprop[g].size = round_up(a->bytes < 16 ? 16 : a->bytes, gran);
    size_t mg = 0;
    DRV(d.MulticastGetGranularity(&mg, &mcprop[g], CU_MULTICAST_GRANULARITY_RECOMMENDED), "cuMulticastGetGranularity");
    if (mg > gran) gran = round_up(mg, gran);
  }
  a->mapped = round_up(a->bytes < 16 ? 16 : a->bytes, gran);

  // the multicast objects and their devices (every device must be added before memory is bound)
  for (int g = 0; g < 2; ++g) {
    if (!a->members[g]) continue;
    mcprop[g].size = a->mapped;
    CUmemGenericAllocationHandle h = 0;
    DRV(d.MulticastCreate(&h, &mcprop[g]), "cuMulticastCreate");
    a->mc_handle[g] = (unsigned long long)h;
    for (int r = 0; r < n; ++r)
      if (a->members[g] >> r & 1) DRV(d.MulticastAddDevice(h, cudev[r]), "cuMulticastAddDevice");
  }

  // the buffers: physical memory on each device, mapped once and readable/writable by every device
  CUmemAccessDesc access[SAR_MAX_RANKS];
  for (int r = 0; r < n; ++r) {
    access[r].location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    access[r].location.id = cudev[r];
    access[r].flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  }
  for (int r = 0; r < n; ++r) {
    prop.location.id = cudev[r];
    CUmemGenericAllocationHandle h = 0;
    DRV(d.MemCreate(&h, a->mapped, &prop, 0), "cuMemCreate");
    a->mem_handle[r] = (unsigned long long)h;
    CUdeviceptr va = 0;
    DRV(d.MemAddressReserve(&va, a->mapped, gran, 0, 0), "cuMemAddressReserve");
    a->uc[r] = (void*)va;
    CUresult rc = d.MemMap(va, a->mapped, 0, h, 0);
    if (rc != CUDA_SUCCESS) {
      d.MemAddressFree(va, a->mapped);
      a->uc[r] = nullptr;
      fail(err, errlen, "cuMemMap", rc);
      symm_free(a);
      return 1;
    }
    DRV(d.MemSetAccess(va, a->mapped, access, (size_t)n), "cuMemSetAccess");
  }

  // bind the buffers, then give every member its own mapping of the object
  for (int g = 0; g < 2; ++g) {
    if (!a->members[g]) continue;
    const CUmemGenericAllocationHandle mch = (CUmemGenericAllocationHandle)a->mc_handle[g];
    for (int r = 0; r < n; ++r) {
      if (!(a->members[g] >> r & 1)) continue;
      CUresult rc = d.MulticastBindMem(mch, 0, (CUmemGenericAllocationHandle)a->mem_handle[r], 0, a->mapped, 0);
      if (rc != CUDA_SUCCESS) {
        if (g == 1) {   // the second group is an extra: go on without it
          for (int q = 0; q < n; ++q)
            if (a->bound[1][q]) { d.MulticastUnbind(mch, cudev[q], 0, a->mapped); a->bound[1][q] = false; }
          d.MemRelease(mch);
          a->mc_handle[1] = 0; a->members[1] = 0;
          break;
        }
        fail(err, errlen, "cuMulticastBindMem", rc);
        symm_free(a);
        return 1;
      }
      a->bound[g][r] = true;
    }
    if (!a->members[g]) continue;
    for (int r = 0; r < n; ++r) {
      if (!(a->members[g] >> r & 1)) continue;
      CUdeviceptr va = 0;
      DRV(d.MemAddressReserve(&va, a->mapped, gran, 0, 0), "cuMemAddressReserve (multicast)");
      a->mc[g][r] = (void*)va;
      CUresult rc = d.MemMap(va, a->mapped, 0, mch, 0);
      if (rc != CUDA_SUCCESS) {
        d.MemAddressFree(va, a->mapped);
        a->mc[g][r] = nullptr;
        fail(err, errlen, "cuMemMap (multicast)", rc);
        symm_free(a);
        return 1;
      }
      DRV(d.MemSetAccess(va, a->mapped, &access[r], 1), "cuMemSetAccess (multicast)");
    }
  }
  return 0;
}
#undef DRV

}  // namespace

bool multicast_supported(int n, const int* devices) {
  Driver& d = driver();
  if (!d.ok) return false;
  for (int r = 0; r < n; ++r) {
    CUdevice dev;
    int v = 0;
    if (cudaSetDevice(devices[r]) != cudaSuccess || cudaFree(nullptr) != cudaSuccess) { cudaGetLastError(); return false; }
    if (d.DeviceGet(&dev, devices[r]) != CUDA_SUCCESS) return false;
    if (d.DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) != CUDA_SUCCESS || !v) return false;
  }
  return true;
}

int symm_alloc(SymmAlloc* a, int n, const int* devices, size_t bytes, int mode, uint32_t sub_members, char* err, int errlen) {
  *a = SymmAlloc();
  if (n < 1 || n > SAR_MAX_RANKS) return fail_msg(err, errlen, "rank count out of range");
  a->n = n; a->bytes = bytes;
  for (int r = 0; r < n; ++r) a->dev[r] = devices[r];
  if (mode == SYMM_PLAIN) return alloc_plain(a, err, errlen);
  if (!multicast_supported(n, devices)) {
    if (mode == SYMM_TRY_MULTICAST) return alloc_plain(a, err, errlen);
    return fail_msg(err, errlen, "NVLink multicast is not offered by the devices or the driver");
  }
  char why[256] = "";
  if (alloc_multicast(a, sub_members, why, (int)sizeof why) == 0) return 0;
  if (mode == SYMM_TRY_MULTICAST) {
    *a = SymmAlloc();
    a->n = n; a->bytes = bytes;
    for (int r = 0; r < n; ++r) a->dev[r] = devices[r];
    return alloc_plain(a, err, errlen);
  }
  return fail_msg(err, errlen, why);
}

void symm_free(SymmAlloc* a) {
  if (!a || a->n == 0) return;
  for (int r = 0; r < a->n; ++r) { cudaSetDevice(a->dev[r]); cudaDeviceSynchronize(); }
  if (!a->vmm) {
    for (int r = 0; r < a->n; ++r)
      if (a->uc[r]) { cudaSetDevice(a->dev[r]); cudaFree(a->uc[r]); }
    *a = SymmAlloc();
    return;
  }
  Driver& d = driver();
  for (int g = 0; g < 2; ++g) {
    for (int r = 0; r < a->n; ++r) {
      if (!a->mc[g][r]) continue;
      d.MemUnmap((CUdeviceptr)a->mc[g][r], a->mapped);
      d.MemAddressFree((CUdeviceptr)a->mc[g][r], a->mapped);
    }
    if (!a->mc_handle[g]) continue;
    for (int r = 0; r < a->n; ++r) {
      if (!a->bound[g][r]) continue;
      CUdevice dev;
      if (d.DeviceGet(&dev, a->dev[r]) == CUDA_SUCCESS) d.MulticastUnbind((CUmemGenericAllocationHandle)a->mc_handle[g], dev, 0, a->mapped);
    }
    d.MemRelease((CUmemGenericAllocationHandle)a->mc_handle[g]);
  }
  for (int r = 0; r < a->n; ++r) {
    if (a->uc[r]) {
      d.MemUnmap((CUdeviceptr)a->uc[r], a->mapped);
      d.MemAddressFree((CUdeviceptr)a->uc[r], a->mapped);
    }
    if (a->mem_handle[r]) d.MemRelease((CUmemGenericAllocationHandle)a->mem_handle[r]);
  }
  *a = SymmAlloc();
}

}  // namespace sar
