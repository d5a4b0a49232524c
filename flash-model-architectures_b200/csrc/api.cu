// Library-wide helpers of libxma_b200: status names, ABI version, cached device properties.
#include <stdio.h>
#include <string.h>

#include <mutex>

#include "common.cuh"

namespace xma {

int sm_count() {
    constexpr int kMaxDevices = 64;
    static int cached[kMaxDevices];
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
    std::lock_guard<std::mutex> lock(mu);
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

}  // namespace xma

extern "C" {

const char* xma_status_string(int status) {
    switch (status) {
        case XMA_OK: return "ok";
        case XMA_ERR_BAD_ARG: return "bad argument (null or misaligned pointer, negative or inconsistent size)";
        case XMA_ERR_UNSUPPORTED: return "shape or dtype not supported by the sm_100a kernels";
        case XMA_ERR_LAUNCH: return "CUDA launch failed";
        case XMA_ERR_DRIVER: return "tensor-map encode / driver entry point failed";
        case XMA_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait ran out";
        case XMA_ERR_SCRATCH_TOO_SMALL:
            return "the problem needs more scratch memory than the library's built-in buffer holds "
                   "(use the variant that takes a caller-provided workspace)";
        default:
            if (status >= 1000) {
                static thread_local char text[96];
                snprintf(text, sizeof(text), "CUDA runtime error %d (%s)", status - 1000,
                         cudaGetErrorName(static_cast<cudaError_t>(status - 1000)));
                return text;
            }
            return "unknown status";
    }
}

int xma_abi_version(void) { return 2; }

int xma_ipc_get_handle(const void* allocation_base, void* handle64) {
    if (allocation_base == nullptr || handle64 == nullptr) return XMA_ERR_BAD_ARG;
    cudaIpcMemHandle_t handle;
    const cudaError_t err = cudaIpcGetMemHandle(&handle, const_cast<void*>(allocation_base));
    if (err != cudaSuccess) {
        cudaGetLastError();
        return 1000 + static_cast<int>(err);
    }
    memcpy(handle64, &handle, sizeof(handle));
    return XMA_OK;
}

int xma_ipc_open_handle(const void* handle64, void** device_ptr) {
    if (handle64 == nullptr || device_ptr == nullptr) return XMA_ERR_BAD_ARG;
    cudaIpcMemHandle_t handle;
    static_assert(sizeof(handle) == 64, "cudaIpcMemHandle_t is 64 bytes");
    memcpy(&handle, handle64, sizeof(handle));
    // Opened with the CALLER's device current: the runtime then maps the owner's allocation for this
    // device and switches peer access on, so this device's kernels can load and store through it.
    const cudaError_t err = cudaIpcOpenMemHandle(device_ptr, handle, cudaIpcMemLazyEnablePeerAccess);
    if (err != cudaSuccess) {
        cudaGetLastError();
        return 1000 + static_cast<int>(err);  // xma_status_string reports the CUDA error number
    }
    return XMA_OK;
}

int xma_ipc_close_handle(void* device_ptr) {
    if (device_ptr == nullptr) return XMA_ERR_BAD_ARG;
    const cudaError_t err = cudaIpcCloseMemHandle(device_ptr);
    if (err != cudaSuccess) {
        cudaGetLastError();
        return 1000 + static_cast<int>(err);
    }
    return XMA_OK;
}

}  // extern "C"
