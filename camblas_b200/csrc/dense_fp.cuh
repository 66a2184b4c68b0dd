/*
 * Elementwise and reduction kernels of the FP32 / FP64 layer compositions
 * (affine, two-layer perceptron forward and backward, single-head attention).
 * The products themselves run on the CUDA-core GEMM of gemm_simt.cuh; none of
 * this is on the BF16/FP8 hot path, so the kernels are plain: coalesced, one
 * pass where possible, sums in a fixed order so that results repeat bit for bit.
 *
 * Semantics follow the reference's entry points (camblas_cuda.h:70-99;
 * backend.cu:870-911, fusion.cuh:95-156, 204-263); all arrays are row-major.
 */
#pragma once

#include <cuda_runtime.h>
#include <math_constants.h>

namespace dense
{

/* out[r][c] = act(out[r][c] + bias[c]) over a contiguous rows x columns array. */
template <typename T>
__global__ void add_bias(T *out, const T *bias, long long count, int columns, int relu)
{
    const long long stride = 1ll * gridDim.x * blockDim.x;
    for (long long i = 1ll * blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride) {
        T value = out[i] + bias[i % columns];
        out[i] = relu && value < T(0) ? T(0) : value;
    }
}

template <typename T> __device__ __forceinline__ T exponential_of(T value);
template <> __device__ __forceinline__ float exponential_of<float>(float value)
{
    return expf(value);
}
template <> __device__ __forceinline__ double exponential_of<double>(double value)
{
    return exp(value);
}

/* Largest / summed value over the 256 threads of a CTA; every thread gets it. */
template <typename T, bool Largest> __device__ T over_cta(T value, T *lanes)
{
    for (int offset = 16; offset; offset >>= 1) {
        const T other = __shfl_xor_sync(0xffffffffu, value, offset);
        value = Largest ? (other > value ? other : value) : value + other;
    }
    const int warp = threadIdx.x >> 5;
    if ((threadIdx.x & 31) == 0)
        lanes[warp] = value;
    __syncthreads();
    T total = lanes[0];
    for (int w = 1; w < int(blockDim.x >> 5); ++w)
        total = Largest ? (lanes[w] > total ? lanes[w] : total) : total + lanes[w];
    __syncthreads();
    return total;
}

/* One CTA per row: row = softmax(scale * row), with the row's maximum
 * subtracted before the exponential. */
template <typename T> __global__ void softmax_scaled(T *scores, int columns, T scale)
{
    __shared__ T lanes[8];
    T *row = scores + static_cast<size_t>(blockIdx.x) * columns;
    T largest = -T(CUDART_INF);
    for (int c = threadIdx.x; c < columns; c += blockDim.x) {
        const T value = row[c] * scale;
        largest = value > largest ? value : largest;
    }
    largest = over_cta<T, true>(largest, lanes);
    T sum = T(0);
    for (int c = threadIdx.x; c < columns; c += blockDim.x) {
        const T value = exponential_of<T>(row[c] * scale - largest);
        row[c] = value;
        sum += value;
    }
    sum = over_cta<T, false>(sum, lanes);
    for (int c = threadIdx.x; c < columns; c += blockDim.x)
        row[c] /= sum;
}

/* sums[c] = sum over the rows of values[r][c], rows in ascending order; one
 * thread per column. With Gate, values[r][c] is first set to zero wherever
 * gate[r][c] <= 0 (the derivative of ReLU), in place. sums may be NULL. */
template <typename T, bool Gate>
__global__ void column_sums(T *values, const T *gate, int rows, int columns, T *sums)
{
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= columns)
        return;
    T sum = T(0);
    for (int r = 0; r < rows; ++r) {
        const size_t at = static_cast<size_t>(r) * columns + c;
        T value = values[at];
        if (Gate && gate[at] <= T(0)) {
            value = T(0);
            values[at] = value;
        }
        sum += value;
    }
    if (sums != nullptr)
        sums[c] = sum;
}

} // namespace dense
