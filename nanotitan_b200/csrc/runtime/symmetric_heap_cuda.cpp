// `nt::symm::cuda_driver()`: the symmetric heap's driver table filled from the CUDA driver.  Entry points are
// resolved at run time (cudaGetDriverEntryPoint), so the library links without libcuda.
#include <cuda.h>
#include <cuda_runtime.h>

#include <stdexcept>
#include <string>

#include "symmetric_heap.h"

namespace nt::symm {
namespace {

template <typename Fn>
Fn entry(const char* name) {
  void* ptr = nullptr;
  cudaDriverEntryPointQueryResult res;
  cudaError_t err = cudaGetDriverEntryPoint(name, &ptr, cudaEnableDefault, &res);
  if (err != cudaSuccess || ptr == nullptr || res != cudaDriverEntryPointSuccess)
    throw std::runtime_error(std::string("symmetric heap: the driver has no ") + name);
  return reinterpret_cast<Fn>(ptr);
}

#define NT_DRV(name) static auto fn_##name = entry<decltype(&name)>(#name)

void check(CUresult r, const char* what) {
  if (r == CUDA_SUCCESS) return;
  NT_DRV(cuGetErrorString);
  const char* text = nullptr;
  fn_cuGetErrorString(r, &text);
  throw std::runtime_error(std::string("symmetric heap: ") + what + " failed: " + (text ? text : "unknown error") + " (" +
                           std::to_string(static_cast<int>(r)) + ")");
}

CUdevice device_of(int ordinal) {
  NT_DRV(cuDeviceGet);
  CUdevice dev = 0;
  check(fn_cuDeviceGet(&dev, ordinal), "cuDeviceGet");
  return dev;
}

CUmemAllocationProp memory_prop(int device) {
  CUmemAllocationProp prop{};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

CUmulticastObjectProp multicast_prop(int n_devices, size_t bytes) {
  CUmulticastObjectProp prop{};
  prop.numDevices = static_cast<unsigned>(n_devices);
  prop.size = bytes;
  prop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

DriverApi make() {
  DriverApi api;
  api.granularity = [](int device, int multicast_devices) -> size_t {
    size_t g = 0;
    if (multicast_devices > 0) {
      NT_DRV(cuMulticastGetGranularity);
      CUmulticastObjectProp prop = multicast_prop(multicast_devices, size_t(2) << 20);
      check(fn_cuMulticastGetGranularity(&g, &prop, CU_MULTICAST_GRANULARITY_RECOMMENDED), "cuMulticastGetGranularity");
    } else {
      NT_DRV(cuMemGetAllocationGranularity);
      CUmemAllocationProp prop = memory_prop(device);
      check(fn_cuMemGetAllocationGranularity(&g, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED), "cuMemGetAllocationGranularity");
    }
    return g;
  };
  api.multicast_supported = [](int device) -> bool {
    NT_DRV(cuDeviceGetAttribute);
    int yes = 0;
    check(fn_cuDeviceGetAttribute(&yes, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, device_of(device)), "cuDeviceGetAttribute");
    return yes != 0;
  };
  api.create = [](int device, size_t bytes) -> Handle {
    NT_DRV(cuMemCreate);
    CUmemAllocationProp prop = memory_prop(device);
    CUmemGenericAllocationHandle h = 0;
    check(fn_cuMemCreate(&h, bytes, &prop, 0), "cuMemCreate");
    return h;
  };
  api.export_fd = [](Handle h) -> int {
    NT_DRV(cuMemExportToShareableHandle);
    int fd = -1;
    check(fn_cuMemExportToShareableHandle(&fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0), "cuMemExportToShareableHandle");
    return fd;
  };
  api.import_fd = [](int fd) -> Handle {
    NT_DRV(cuMemImportFromShareableHandle);
    CUmemGenericAllocationHandle h = 0;
    check(fn_cuMemImportFromShareableHandle(&h, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                                            CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR),
          "cuMemImportFromShareableHandle");
    return h;
  };
  api.release = [](Handle h) {
    NT_DRV(cuMemRelease);
    check(fn_cuMemRelease(h), "cuMemRelease");
  };
  api.reserve = [](size_t bytes, size_t alignment) -> Address {
    NT_DRV(cuMemAddressReserve);
    CUdeviceptr p = 0;
    check(fn_cuMemAddressReserve(&p, bytes, alignment, 0, 0), "cuMemAddressReserve");
    return p;
  };
  api.unreserve = [](Address a, size_t bytes) {
    NT_DRV(cuMemAddressFree);
    check(fn_cuMemAddressFree(a, bytes), "cuMemAddressFree");
  };
  api.map = [](Address a, size_t bytes, Handle h, int device) {
    NT_DRV(cuMemMap);
    NT_DRV(cuMemSetAccess);
    NT_DRV(cuMemUnmap);
    check(fn_cuMemMap(a, bytes, 0, h, 0), "cuMemMap");
    CUmemAccessDesc access{};
    access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    access.location.id = device;
    access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    CUresult r = fn_cuMemSetAccess(a, bytes, &access, 1);
    if (r != CUDA_SUCCESS) {
      fn_cuMemUnmap(a, bytes);
      check(r, "cuMemSetAccess");
    }
  };
  api.unmap = [](Address a, size_t bytes) {
    NT_DRV(cuMemUnmap);
    check(fn_cuMemUnmap(a, bytes), "cuMemUnmap");
  };
  api.multicast_create = [](int n_devices, size_t bytes) -> Handle {
    NT_DRV(cuMulticastCreate);
    CUmulticastObjectProp prop = multicast_prop(n_devices, bytes);
    CUmemGenericAllocationHandle h = 0;
    check(fn_cuMulticastCreate(&h, &prop), "cuMulticastCreate");
    return h;
  };
  api.multicast_add_device = [](Handle mc, int device) {
    NT_DRV(cuMulticastAddDevice);
    check(fn_cuMulticastAddDevice(mc, device_of(device)), "cuMulticastAddDevice");
  };
  api.multicast_bind = [](Handle mc, Handle memory, size_t bytes) {
    NT_DRV(cuMulticastBindMem);
    check(fn_cuMulticastBindMem(mc, 0, memory, 0, bytes, 0), "cuMulticastBindMem");
  };
  api.multicast_unbind = [](Handle mc, int device, size_t bytes) {
    NT_DRV(cuMulticastUnbind);
    check(fn_cuMulticastUnbind(mc, device_of(device), 0, bytes), "cuMulticastUnbind");
  };
  return api;
}

}  // namespace

const DriverApi& cuda_driver() {
  static const DriverApi api = make();
  return api;
}

}  // namespace nt::symm
