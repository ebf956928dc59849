// Host side of the NVLink multicast region (see multicast.h): CUDA virtual memory management plus the multicast
// object calls, reached through cudaGetDriverEntryPoint so that nothing links against the driver library.
#include "multicast.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <stdexcept>

namespace sky {
namespace {

template <typename Fn>
Fn driver_fn(const char* name) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn) {
        cudaGetLastError();
        throw std::runtime_error(std::string("driver entry point not found: ") + name);
    }
    return reinterpret_cast<Fn>(fn);
}

struct Driver {
    CUresult (*GetErrorString)(CUresult, const char**);
    CUresult (*DeviceGet)(CUdevice*, int);
    CUresult (*DeviceGetAttribute)(int*, CUdevice_attribute, CUdevice);
    CUresult (*MulticastGetGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags);
    CUresult (*MulticastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*);
    CUresult (*MulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice);
    CUresult (*MulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long);
    CUresult (*MulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t);
    CUresult (*MemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
    CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
    CUresult (*MemRelease)(CUmemGenericAllocationHandle);
    CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
    CUresult (*MemAddressFree)(CUdeviceptr, size_t);
    CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
    CUresult (*MemUnmap)(CUdeviceptr, size_t);
    CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);

    Driver() {
        GetErrorString = driver_fn<decltype(GetErrorString)>("cuGetErrorString");
        DeviceGet = driver_fn<decltype(DeviceGet)>("cuDeviceGet");
        DeviceGetAttribute = driver_fn<decltype(DeviceGetAttribute)>("cuDeviceGetAttribute");
        MulticastGetGranularity = driver_fn<decltype(MulticastGetGranularity)>("cuMulticastGetGranularity");
        MulticastCreate = driver_fn<decltype(MulticastCreate)>("cuMulticastCreate");
        MulticastAddDevice = driver_fn<decltype(MulticastAddDevice)>("cuMulticastAddDevice");
        MulticastBindMem = driver_fn<decltype(MulticastBindMem)>("cuMulticastBindMem");
        MulticastUnbind = driver_fn<decltype(MulticastUnbind)>("cuMulticastUnbind");
        MemGetAllocationGranularity = driver_fn<decltype(MemGetAllocationGranularity)>("cuMemGetAllocationGranularity");
        MemCreate = driver_fn<decltype(MemCreate)>("cuMemCreate");
        MemRelease = driver_fn<decltype(MemRelease)>("cuMemRelease");
        MemAddressReserve = driver_fn<decltype(MemAddressReserve)>("cuMemAddressReserve");
        MemAddressFree = driver_fn<decltype(MemAddressFree)>("cuMemAddressFree");
        MemMap = driver_fn<decltype(MemMap)>("cuMemMap");
        MemUnmap = driver_fn<decltype(MemUnmap)>("cuMemUnmap");
        MemSetAccess = driver_fn<decltype(MemSetAccess)>("cuMemSetAccess");
    }
};

Driver& drv() {
    static Driver d;
    return d;
}

void check(CUresult r, const char* what) {
    if (r == CUDA_SUCCESS) return;
    const char* s = nullptr;
    drv().GetErrorString(r, &s);
    throw std::runtime_error(std::string(what) + " failed: " + (s ? s : "unknown driver error") + " (" + std::to_string((int)r) + ")");
}

CUdevice cu_device(int ordinal) {
    // The runtime's primary context must exist before the driver calls below touch the device.
    if (cudaSetDevice(ordinal) != cudaSuccess || cudaFree(nullptr) != cudaSuccess) {
        cudaGetLastError();
        throw std::runtime_error("cannot open device " + std::to_string(ordinal));
    }
    CUdevice d;
    check(drv().DeviceGet(&d, ordinal), "cuDeviceGet");
    return d;
}

}  // namespace

bool multicast_supported(int device, std::string* why) {
    try {
        int prev = 0;
        cudaGetDevice(&prev);
        CUdevice d = cu_device(device);
        cudaSetDevice(prev);
        int ok = 0;
        check(drv().DeviceGetAttribute(&ok, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, d), "cuDeviceGetAttribute(MULTICAST_SUPPORTED)");
        if (!ok && why) *why = "device reports no multicast support";
        return ok != 0;
    } catch (const std::exception& e) {
        if (why) *why = e.what();
        return false;
    }
}

MulticastRegion* multicast_create(const std::vector<int>& devices, size_t bytes) {
    if (devices.size() < 2) throw std::runtime_error("a multicast team needs at least two devices");
    if (bytes == 0) throw std::runtime_error("a multicast region needs a size");
    int prev = 0;
    cudaGetDevice(&prev);
    auto* r = new MulticastRegion();
    r->devices = devices;
    const size_t n = devices.size();
    r->mem_handles.assign(n, 0);
    r->unicast.assign(n, 0);
    r->bound.assign(n, 0);
    try {
        Driver& D = drv();
        std::vector<CUdevice> cu(n);
        for (size_t i = 0; i < n; ++i) {
            std::string why;
            if (!multicast_supported(devices[i], &why)) throw std::runtime_error("device " + std::to_string(devices[i]) + ": " + why);
            cu[i] = cu_device(devices[i]);
        }
        CUmulticastObjectProp mp = {};
        mp.numDevices = (unsigned)n;
        mp.size = bytes;
        mp.handleTypes = 0;
        size_t gran = 0;
        check(D.MulticastGetGranularity(&gran, &mp, CU_MULTICAST_GRANULARITY_MINIMUM), "cuMulticastGetGranularity");
        CUmemAllocationProp ap = {};
        ap.type = CU_MEM_ALLOCATION_TYPE_PINNED;
        ap.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
        for (size_t i = 0; i < n; ++i) {
            ap.location.id = cu[i];
            size_t g = 0;
            check(D.MemGetAllocationGranularity(&g, &ap, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED), "cuMemGetAllocationGranularity");
            gran = std::max(gran, g);
        }
        r->granularity = gran;
        r->bytes = (bytes + gran - 1) / gran * gran;
        mp.size = r->bytes;
        CUmemGenericAllocationHandle mc = 0;
        check(D.MulticastCreate(&mc, &mp), "cuMulticastCreate");
        r->mc_handle = mc;
        for (size_t i = 0; i < n; ++i) check(D.MulticastAddDevice(mc, cu[i]), "cuMulticastAddDevice");   // all members before any bind
        std::vector<CUmemAccessDesc> access(n);
        for (size_t i = 0; i < n; ++i) {
            access[i].location.type = CU_MEM_LOCATION_TYPE_DEVICE;
            access[i].location.id = cu[i];
            access[i].flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
        }
        for (size_t i = 0; i < n; ++i) {
            ap.location.id = cu[i];
            CUmemGenericAllocationHandle h = 0;
            check(D.MemCreate(&h, r->bytes, &ap, 0), "cuMemCreate");
            r->mem_handles[i] = h;
            check(D.MulticastBindMem(mc, 0, h, 0, r->bytes, 0), "cuMulticastBindMem");
            r->bound[i] = 1;
            CUdeviceptr va = 0;
            check(D.MemAddressReserve(&va, r->bytes, gran, 0, 0), "cuMemAddressReserve");
            r->unicast[i] = va;
            check(D.MemMap(va, r->bytes, 0, h, 0), "cuMemMap");
            check(D.MemSetAccess(va, r->bytes, access.data(), n), "cuMemSetAccess");
        }
        CUdeviceptr mva = 0;
        check(D.MemAddressReserve(&mva, r->bytes, gran, 0, 0), "cuMemAddressReserve(multicast)");
        r->multicast = mva;
        check(D.MemMap(mva, r->bytes, 0, mc, 0), "cuMemMap(multicast)");
        check(D.MemSetAccess(mva, r->bytes, access.data(), n), "cuMemSetAccess(multicast)");
    } catch (...) {
        multicast_destroy(r);
        cudaSetDevice(prev);
        throw;
    }
    cudaSetDevice(prev);
    return r;
}

void multicast_destroy(MulticastRegion* r) {
    if (!r) return;
    int prev = 0;
    cudaGetDevice(&prev);
    for (int d : r->devices) {
        if (cudaSetDevice(d) == cudaSuccess) cudaDeviceSynchronize();     // nothing of ours may still be storing into the region
    }
    cudaGetLastError();
    cudaSetDevice(prev);
    try {
        Driver& D = drv();
        if (r->multicast) {
            D.MemUnmap(r->multicast, r->bytes);
            D.MemAddressFree(r->multicast, r->bytes);
        }
        for (size_t i = 0; i < r->devices.size(); ++i) {
            if (r->bound[i]) {
                CUdevice d;
                if (D.DeviceGet(&d, r->devices[i]) == CUDA_SUCCESS) D.MulticastUnbind(r->mc_handle, d, 0, r->bytes);
            }
            if (r->unicast[i]) {
                D.MemUnmap(r->unicast[i], r->bytes);
                D.MemAddressFree(r->unicast[i], r->bytes);
            }
            if (r->mem_handles[i]) D.MemRelease(r->mem_handles[i]);
        }
        if (r->mc_handle) D.MemRelease(r->mc_handle);
    } catch (...) {
    }
    delete r;
}

}  // namespace sky
