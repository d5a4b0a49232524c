// Shared device/host helpers for libxma_b200 (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "xma_b200.h"

namespace xma {

constexpr int kDtypeBF16 = 0;
constexpr int kDtypeF16 = 1;
constexpr int kDtypeF32 = 2;

constexpr int kMaxExperts = 1024;

inline int dtype_size(int dtype) { return dtype == kDtypeF32 ? 4 : 2; }

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Number of SMs of the current device, cached per device.
int sm_count();

// Launch-error check used after every kernel launch.
inline int launch_status() { return cudaGetLastError() == cudaSuccess ? XMA_OK : XMA_ERR_LAUNCH; }

template <typename T>
struct Elem;
template <>
struct Elem<__nv_bfloat16> {
    static __device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
    static __device__ __forceinline__ __nv_bfloat16 from_float(float v) { return __float2bfloat16_rn(v); }
};
template <>
struct Elem<__half> {
    static __device__ __forceinline__ float to_float(__half v) { return __half2float(v); }
    static __device__ __forceinline__ __half from_float(float v) { return __float2half_rn(v); }
};
template <>
struct Elem<float> {
    static __device__ __forceinline__ float to_float(float v) { return v; }
    static __device__ __forceinline__ float from_float(float v) { return v; }
};

// 16 bytes of elements of type T.
template <typename T>
struct alignas(16) Vec16 {
    static constexpr int kCount = 16 / sizeof(T);
    T v[kCount];
};

template <typename T>
__device__ __forceinline__ Vec16<T> load16(const T* p) {
    Vec16<T> r;
    *reinterpret_cast<uint4*>(&r) = __ldg(reinterpret_cast<const uint4*>(p));
    return r;
}

template <typename T>
__device__ __forceinline__ void store16(T* p, const Vec16<T>& r) {
    *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(&r);
}

}  // namespace xma
