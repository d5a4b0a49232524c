// Library-wide helpers of libxma_b200: status names, ABI version, cached device properties.
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
        default: return "unknown status";
    }
}

int xma_abi_version(void) { return 1; }

}  // extern "C"
