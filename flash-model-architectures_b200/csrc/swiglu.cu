// Stand-alone packed swiglu (forward and backward) for callers that use the activation outside the
// fused MoE path. HBM-bound elementwise kernels: 16-byte accesses when the half width allows it.
#include "common.cuh"

namespace xma {

constexpr int kSwigluThreads = 256;

__device__ __forceinline__ float sigmoid_f32(float x) { return 1.f / (1.f + expf(-x)); }

// x [rows, 2*half] = [up | gate]; y [rows, half] = up * silu(gate)
template <typename T, bool kVec>
__global__ void __launch_bounds__(kSwigluThreads)
swiglu_packed_forward_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t rows, int64_t half) {
    constexpr int kPer = kVec ? Vec16<T>::kCount : 1;
    const int64_t per_row = half / kPer;
    const int64_t total = rows * per_row;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t r = i / per_row, c = (i - r * per_row) * kPer;
        const T* up = x + r * 2 * half + c;
        const T* gate = up + half;
        if (kVec) {
            const Vec16<T> u = load16(up), g = load16(gate);
            Vec16<T> o;
#pragma unroll
            for (int j = 0; j < Vec16<T>::kCount; ++j) {
                const float gf = Elem<T>::to_float(g.v[j]);
                o.v[j] = Elem<T>::from_float(Elem<T>::to_float(u.v[j]) * gf * sigmoid_f32(gf));
            }
            store16(y + r * half + c, o);
        } else {
            const float gf = Elem<T>::to_float(*gate);
            y[r * half + c] = Elem<T>::from_float(Elem<T>::to_float(*up) * gf * sigmoid_f32(gf));
        }
    }
}

// dx = [du | dg], du = dy * silu(g), dg = dy * u * (s + g s (1 - s))
template <typename T, bool kVec>
__global__ void __launch_bounds__(kSwigluThreads)
swiglu_packed_backward_kernel(const T* __restrict__ x, const T* __restrict__ dy, T* __restrict__ dx, int64_t rows,
                              int64_t half) {
    constexpr int kPer = kVec ? Vec16<T>::kCount : 1;
    const int64_t per_row = half / kPer;
    const int64_t total = rows * per_row;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t r = i / per_row, c = (i - r * per_row) * kPer;
        const int64_t up_off = r * 2 * half + c;
        if (kVec) {
            const Vec16<T> u = load16(x + up_off), g = load16(x + up_off + half), d = load16(dy + r * half + c);
            Vec16<T> du, dg;
#pragma unroll
            for (int j = 0; j < Vec16<T>::kCount; ++j) {
                const float gf = Elem<T>::to_float(g.v[j]), uf = Elem<T>::to_float(u.v[j]), df = Elem<T>::to_float(d.v[j]);
                const float s = sigmoid_f32(gf), silu = gf * s;
                du.v[j] = Elem<T>::from_float(df * silu);
                dg.v[j] = Elem<T>::from_float(df * uf * (s + silu * (1.f - s)));
            }
            store16(dx + up_off, du);
            store16(dx + up_off + half, dg);
        } else {
            const float gf = Elem<T>::to_float(x[up_off + half]), uf = Elem<T>::to_float(x[up_off]);
            const float df = Elem<T>::to_float(dy[r * half + c]);
            const float s = sigmoid_f32(gf), silu = gf * s;
            dx[up_off] = Elem<T>::from_float(df * silu);
            dx[up_off + half] = Elem<T>::from_float(df * uf * (s + silu * (1.f - s)));
        }
    }
}

// Unpacked form: gate and up are separate tensors of `count` elements; y = up * silu(gate).
template <typename T, bool kVec>
__global__ void __launch_bounds__(kSwigluThreads)
swiglu_forward_kernel(const T* __restrict__ gate, const T* __restrict__ up, T* __restrict__ y, int64_t count) {
    constexpr int kPer = kVec ? Vec16<T>::kCount : 1;
    const int64_t total = count / kPer;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        if (kVec) {
            const Vec16<T> g = load16(gate + i * kPer), u = load16(up + i * kPer);
            Vec16<T> o;
#pragma unroll
            for (int j = 0; j < Vec16<T>::kCount; ++j) {
                const float gf = Elem<T>::to_float(g.v[j]);
                o.v[j] = Elem<T>::from_float(Elem<T>::to_float(u.v[j]) * gf * sigmoid_f32(gf));
            }
            store16(y + i * kPer, o);
        } else {
            const float gf = Elem<T>::to_float(gate[i]);
            y[i] = Elem<T>::from_float(Elem<T>::to_float(up[i]) * gf * sigmoid_f32(gf));
        }
    }
}

// dgate = dy * up * (s + gate s (1 - s)), dup = dy * silu(gate), s = sigmoid(gate)
template <typename T, bool kVec>
__global__ void __launch_bounds__(kSwigluThreads)
swiglu_backward_kernel(const T* __restrict__ gate, const T* __restrict__ up, const T* __restrict__ dy,
                       T* __restrict__ dgate, T* __restrict__ dup, int64_t count) {
    constexpr int kPer = kVec ? Vec16<T>::kCount : 1;
    const int64_t total = count / kPer;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        if (kVec) {
            const Vec16<T> g = load16(gate + i * kPer), u = load16(up + i * kPer), d = load16(dy + i * kPer);
            Vec16<T> og, ou;
#pragma unroll
            for (int j = 0; j < Vec16<T>::kCount; ++j) {
                const float gf = Elem<T>::to_float(g.v[j]), uf = Elem<T>::to_float(u.v[j]), df = Elem<T>::to_float(d.v[j]);
                const float sg = sigmoid_f32(gf), silu = gf * sg;
                ou.v[j] = Elem<T>::from_float(df * silu);
                og.v[j] = Elem<T>::from_float(df * uf * (sg + silu * (1.f - sg)));
            }
            store16(dgate + i * kPer, og);
            store16(dup + i * kPer, ou);
        } else {
            const float gf = Elem<T>::to_float(gate[i]), uf = Elem<T>::to_float(up[i]), df = Elem<T>::to_float(dy[i]);
            const float sg = sigmoid_f32(gf), silu = gf * sg;
            dup[i] = Elem<T>::from_float(df * silu);
            dgate[i] = Elem<T>::from_float(df * uf * (sg + silu * (1.f - sg)));
        }
    }
}

inline unsigned swiglu_grid(int64_t work) {
    int64_t blocks = ceil_div(work > 0 ? work : 1, kSwigluThreads);
    const int64_t max_blocks = static_cast<int64_t>(sm_count()) * 16;
    return static_cast<unsigned>(blocks > max_blocks ? max_blocks : blocks);
}

template <typename T>
int launch_swiglu_fwd(const void* x, void* y, int64_t rows, int64_t half, cudaStream_t s) {
    const bool vec = half % Vec16<T>::kCount == 0 && aligned16(x) && aligned16(y);
    if (vec)
        swiglu_packed_forward_kernel<T, true><<<swiglu_grid(rows * half / Vec16<T>::kCount), kSwigluThreads, 0, s>>>(
            static_cast<const T*>(x), static_cast<T*>(y), rows, half);
    else
        swiglu_packed_forward_kernel<T, false><<<swiglu_grid(rows * half), kSwigluThreads, 0, s>>>(
            static_cast<const T*>(x), static_cast<T*>(y), rows, half);
    return launch_status();
}

template <typename T>
int launch_swiglu_bwd(const void* x, const void* dy, void* dx, int64_t rows, int64_t half, cudaStream_t s) {
    const bool vec = half % Vec16<T>::kCount == 0 && aligned16(x) && aligned16(dy) && aligned16(dx);
    if (vec)
        swiglu_packed_backward_kernel<T, true><<<swiglu_grid(rows * half / Vec16<T>::kCount), kSwigluThreads, 0, s>>>(
            static_cast<const T*>(x), static_cast<const T*>(dy), static_cast<T*>(dx), rows, half);
    else
        swiglu_packed_backward_kernel<T, false><<<swiglu_grid(rows * half), kSwigluThreads, 0, s>>>(
            static_cast<const T*>(x), static_cast<const T*>(dy), static_cast<T*>(dx), rows, half);
    return launch_status();
}

template <typename T>
int launch_swiglu_flat_fwd(const void* gate, const void* up, void* y, int64_t count, cudaStream_t s) {
    const bool vec = count % Vec16<T>::kCount == 0 && aligned16(gate) && aligned16(up) && aligned16(y);
    if (vec)
        swiglu_forward_kernel<T, true><<<swiglu_grid(count / Vec16<T>::kCount), kSwigluThreads, 0, s>>>(
            static_cast<const T*>(gate), static_cast<const T*>(up), static_cast<T*>(y), count);
    else
        swiglu_forward_kernel<T, false><<<swiglu_grid(count), kSwigluThreads, 0, s>>>(
            static_cast<const T*>(gate), static_cast<const T*>(up), static_cast<T*>(y), count);
    return launch_status();
}

template <typename T>
int launch_swiglu_flat_bwd(const void* gate, const void* up, const void* dy, void* dgate, void* dup, int64_t count,
                           cudaStream_t s) {
    const bool vec = count % Vec16<T>::kCount == 0 && aligned16(gate) && aligned16(up) && aligned16(dy) &&
                     aligned16(dgate) && aligned16(dup);
    if (vec)
        swiglu_backward_kernel<T, true><<<swiglu_grid(count / Vec16<T>::kCount), kSwigluThreads, 0, s>>>(
            static_cast<const T*>(gate), static_cast<const T*>(up), static_cast<const T*>(dy), static_cast<T*>(dgate),
            static_cast<T*>(dup), count);
    else
        swiglu_backward_kernel<T, false><<<swiglu_grid(count), kSwigluThreads, 0, s>>>(
            static_cast<const T*>(gate), static_cast<const T*>(up), static_cast<const T*>(dy), static_cast<T*>(dgate),
            static_cast<T*>(dup), count);
    return launch_status();
}

}  // namespace xma

extern "C" {

int xma_swiglu_forward(const void* gate, const void* up, int32_t dtype, int64_t count, void* y, void* stream) {
    if (count < 0) return XMA_ERR_BAD_ARG;
    if (count == 0) return XMA_OK;
    if (!gate || !up || !y) return XMA_ERR_BAD_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case xma::kDtypeBF16: return xma::launch_swiglu_flat_fwd<__nv_bfloat16>(gate, up, y, count, s);
        case xma::kDtypeF16: return xma::launch_swiglu_flat_fwd<__half>(gate, up, y, count, s);
        case xma::kDtypeF32: return xma::launch_swiglu_flat_fwd<float>(gate, up, y, count, s);
        default: return XMA_ERR_UNSUPPORTED;
    }
}

int xma_swiglu_backward(const void* gate, const void* up, const void* dy, int32_t dtype, int64_t count, void* dgate,
                        void* dup, void* stream) {
    if (count < 0) return XMA_ERR_BAD_ARG;
    if (count == 0) return XMA_OK;
    if (!gate || !up || !dy || !dgate || !dup) return XMA_ERR_BAD_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case xma::kDtypeBF16: return xma::launch_swiglu_flat_bwd<__nv_bfloat16>(gate, up, dy, dgate, dup, count, s);
        case xma::kDtypeF16: return xma::launch_swiglu_flat_bwd<__half>(gate, up, dy, dgate, dup, count, s);
        case xma::kDtypeF32: return xma::launch_swiglu_flat_bwd<float>(gate, up, dy, dgate, dup, count, s);
        default: return XMA_ERR_UNSUPPORTED;
    }
}

int xma_swiglu_packed_forward(const void* x, int32_t dtype, int64_t rows, int64_t half, void* y, void* stream) {
    if (rows < 0 || half <= 0) return XMA_ERR_BAD_ARG;
    if (rows == 0) return XMA_OK;
    if (!x || !y) return XMA_ERR_BAD_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case xma::kDtypeBF16: return xma::launch_swiglu_fwd<__nv_bfloat16>(x, y, rows, half, s);
        case xma::kDtypeF16: return xma::launch_swiglu_fwd<__half>(x, y, rows, half, s);
        case xma::kDtypeF32: return xma::launch_swiglu_fwd<float>(x, y, rows, half, s);
        default: return XMA_ERR_UNSUPPORTED;
    }
}

int xma_swiglu_packed_backward(const void* x, const void* dy, int32_t dtype, int64_t rows, int64_t half, void* dx,
                               void* stream) {
    if (rows < 0 || half <= 0) return XMA_ERR_BAD_ARG;
    if (rows == 0) return XMA_OK;
    if (!x || !dy || !dx) return XMA_ERR_BAD_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case xma::kDtypeBF16: return xma::launch_swiglu_bwd<__nv_bfloat16>(x, dy, dx, rows, half, s);
        case xma::kDtypeF16: return xma::launch_swiglu_bwd<__half>(x, dy, dx, rows, half, s);
        case xma::kDtypeF32: return xma::launch_swiglu_bwd<float>(x, dy, dx, rows, half, s);
        default: return XMA_ERR_UNSUPPORTED;
    }
}

}  // extern "C"
