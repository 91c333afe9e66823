// Making one rank's device buffer addressable in another rank's process (one process per
// GPU): thin wrappers over the CUDA IPC calls, used to set up the peer-mapped output
// buffers and flag arrays of the head gather. Setup-time code, nothing here is on a hot path.
#include <cuda.h>

#include <mutex>

#include "common.cuh"

namespace rfx {

using AddressRangeFn = CUresult (*)(CUdeviceptr*, size_t*, CUdeviceptr);

static AddressRangeFn address_range_fn() {
    static AddressRangeFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<AddressRangeFn>(p);
    });
    return fn;
}

}  // namespace rfx

extern "C" int rfx_peer_export(const void* device_ptr, RfxPeerHandle* out) {
    using namespace rfx;
    const char* name = "rfx_peer_export";
    RFX_REQUIRE(device_ptr && out, "%s: null pointer", name);
    int st = check_device();
    if (st != RFX_SUCCESS) return st;
    static_assert(sizeof(cudaIpcMemHandle_t) == sizeof(out->handle), "handle size");
    // The IPC handle names a whole allocation: find its base and keep the offset.
    AddressRangeFn range = address_range_fn();
    if (!range) return fail(RFX_CUDA_ERROR, "%s: cuMemGetAddressRange is not available", name);
    CUdeviceptr base = 0;
    size_t size = 0;
    CUresult r = range(&base, &size, (CUdeviceptr)(uintptr_t)device_ptr);
    if (r != CUDA_SUCCESS) return fail(RFX_CUDA_ERROR, "%s: cuMemGetAddressRange failed (%d)", name, (int)r);
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, (void*)(uintptr_t)base);
    if (e != cudaSuccess) return fail(RFX_CUDA_ERROR, "%s: cudaIpcGetMemHandle: %s", name, cudaGetErrorString(e));
    memcpy(out->handle, &h, sizeof(h));
    out->offset = (int64_t)((uintptr_t)device_ptr - (uintptr_t)base);
    return RFX_SUCCESS;
}

extern "C" int rfx_peer_open(const RfxPeerHandle* h, void** mapped, void** mapped_base) {
    using namespace rfx;
    const char* name = "rfx_peer_open";
    RFX_REQUIRE(h && mapped && mapped_base, "%s: null pointer", name);
    int st = check_device();
    if (st != RFX_SUCCESS) return st;
    cudaIpcMemHandle_t ih;
    memcpy(&ih, h->handle, sizeof(ih));
    void* base = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&base, ih, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return fail(RFX_CUDA_ERROR, "%s: cudaIpcOpenMemHandle: %s", name, cudaGetErrorString(e));
    *mapped_base = base;
    *mapped = (char*)base + h->offset;
    return RFX_SUCCESS;
}

extern "C" int rfx_peer_close(void* mapped_base) {
    using namespace rfx;
    if (!mapped_base) return RFX_SUCCESS;
    cudaError_t e = cudaIpcCloseMemHandle(mapped_base);
    if (e != cudaSuccess) return fail(RFX_CUDA_ERROR, "rfx_peer_close: cudaIpcCloseMemHandle: %s", cudaGetErrorString(e));
    return RFX_SUCCESS;
}
