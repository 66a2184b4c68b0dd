/*
 * Residual add + RMS normalisation and the small elementwise kernels beside
 * it. These are bound by HBM traffic: every row is read once (twice from L2 for
 * the second pass) and every result written once.
 *
 * Arithmetic order. The reference normalises a row with 512 threads, four
 * running sums per thread over columns 4t+o+2048i, a shared-memory halving tree
 * down to one warp and a shuffle tree whose direction is selectable
 * (inference_fusion.cuh:136-191). rms_row_kernel below performs exactly that
 * sequence of FP32 roundings - products and sums are rounded separately, never
 * fused - for one row per CTA, so a batch of rows gives, row by row, the bits
 * the reference's single-row kernel gives. Loads are 8- or 16-byte vectors.
 */
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace rms
{

template <typename T> struct Storage;
template <> struct Storage<float> {
    static __device__ __forceinline__ float load(const float *p, long long i) { return p[i]; }
    static __device__ __forceinline__ float round(float v) { return v; }
    static __device__ __forceinline__ void store(float *p, long long i, float v) { p[i] = v; }
    static __device__ __forceinline__ void load4(const float *p, long long i, float (&v)[4])
    {
        float4 q = *reinterpret_cast<const float4 *>(p + i);
        v[0] = q.x, v[1] = q.y, v[2] = q.z, v[3] = q.w;
    }
    static __device__ __forceinline__ void store4(float *p, long long i, const float (&v)[4])
    {
        *reinterpret_cast<float4 *>(p + i) = make_float4(v[0], v[1], v[2], v[3]);
    }
};
template <> struct Storage<__nv_bfloat16> {
    static __device__ __forceinline__ float load(const __nv_bfloat16 *p, long long i)
    {
        return __bfloat162float(p[i]);
    }
    static __device__ __forceinline__ float round(float v)
    {
        return __bfloat162float(__float2bfloat16_rn(v));
    }
    static __device__ __forceinline__ void store(__nv_bfloat16 *p, long long i, float v)
    {
        p[i] = __float2bfloat16_rn(v);
    }
    static __device__ __forceinline__ void load4(const __nv_bfloat16 *p, long long i, float (&v)[4])
    {
        uint2 q = *reinterpret_cast<const uint2 *>(p + i);
        v[0] = __uint_as_float(q.x << 16), v[1] = __uint_as_float(q.x & 0xffff0000u);
        v[2] = __uint_as_float(q.y << 16), v[3] = __uint_as_float(q.y & 0xffff0000u);
    }
    static __device__ __forceinline__ void store4(__nv_bfloat16 *p, long long i,
                                                  const float (&v)[4])
    {
        __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
        uint2 q;
        q.x = *reinterpret_cast<uint32_t *>(&a), q.y = *reinterpret_cast<uint32_t *>(&b);
        *reinterpret_cast<uint2 *>(p + i) = q;
    }
};

constexpr int kRowThreads = 512;

/* One row per CTA. Vector: every pointer is aligned for four-element vector
 * access and width % 4 == 0 (always true for the row width, checked by the
 * caller for the pointers); otherwise the scalar accessors are used. */
template <typename T, typename W, bool Add, bool Vector>
__global__ void __launch_bounds__(kRowThreads)
    rms_row_kernel(int width, float epsilon, const T *input, const T *residual, const W *weight,
                   T *added, T *output, bool round_before_weight, bool descending)
{
    __shared__ float tree[kRowThreads];
    __shared__ float scale_slot;
    const long long base = static_cast<long long>(blockIdx.x) * width;
    input += base;
    output += base;
    if (Add) {
        residual += base;
        added += base;
    }
    const int t = threadIdx.x;
    float sums[4] = {0.f, 0.f, 0.f, 0.f};
    for (int column = t * 4; column < width; column += kRowThreads * 4) {
        float v[4];
        if (Vector) {
            Storage<T>::load4(input, column, v);
            if (Add) {
                float r[4];
                Storage<T>::load4(residual, column, r);
#pragma unroll
                for (int o = 0; o < 4; ++o)
                    v[o] = Storage<T>::round(__fadd_rn(v[o], r[o]));
                Storage<T>::store4(added, column, v);
            }
        } else {
#pragma unroll
            for (int o = 0; o < 4; ++o) {
                v[o] = Storage<T>::load(input, column + o);
                if (Add) {
                    v[o] = Storage<T>::round(
                        __fadd_rn(v[o], Storage<T>::load(residual, column + o)));
                    Storage<T>::store(added, column + o, v[o]);
                }
            }
        }
#pragma unroll
        for (int o = 0; o < 4; ++o)
            sums[o] = __fadd_rn(sums[o], __fmul_rn(v[o], v[o]));
    }
    float sum = __fadd_rn(__fadd_rn(__fadd_rn(sums[0], sums[1]), sums[2]), sums[3]);
    tree[t] = sum;
    for (int offset = kRowThreads / 2; offset >= 32; offset >>= 1) {
        __syncthreads();
        if (t < offset) {
            sum = __fadd_rn(sum, tree[t + offset]);
            tree[t] = sum;
        }
    }
    __syncthreads();
    if (t < 32) {
        if (descending) {
            for (int offset = 16; offset; offset >>= 1)
                sum = __fadd_rn(sum, __shfl_down_sync(0xffffffffu, sum, offset));
        } else {
            for (int offset = 1; offset < 32; offset <<= 1)
                sum = __fadd_rn(sum, __shfl_down_sync(0xffffffffu, sum, offset));
        }
        if (t == 0)
            scale_slot = rsqrtf(__fadd_rn(__fmul_rn(sum, 1.f / static_cast<float>(width)), epsilon));
    }
    __syncthreads();
    const float scale = scale_slot;
    /* Second pass: the sum x+r is recomputed rather than re-read so that the
     * pass does not depend on the visibility of this CTA's own stores. */
    for (int column = t * 4; column < width; column += kRowThreads * 4) {
        float v[4], g[4];
        if (Vector) {
            Storage<T>::load4(input, column, v);
            if (Add) {
                float r[4];
                Storage<T>::load4(residual, column, r);
#pragma unroll
                for (int o = 0; o < 4; ++o)
                    v[o] = Storage<T>::round(__fadd_rn(v[o], r[o]));
            }
            Storage<W>::load4(weight, column, g);
        } else {
#pragma unroll
            for (int o = 0; o < 4; ++o) {
                v[o] = Storage<T>::load(input, column + o);
                if (Add)
                    v[o] = Storage<T>::round(
                        __fadd_rn(v[o], Storage<T>::load(residual, column + o)));
                g[o] = Storage<W>::load(weight, column + o);
            }
        }
#pragma unroll
        for (int o = 0; o < 4; ++o) {
            float normalised = __fmul_rn(v[o], scale);
            if (round_before_weight)
                normalised = Storage<T>::round(normalised);
            v[o] = __fmul_rn(normalised, g[o]);
        }
        if (Vector) {
            Storage<T>::store4(output, column, v);
        } else {
#pragma unroll
            for (int o = 0; o < 4; ++o)
                Storage<T>::store(output, column + o, v[o]);
        }
    }
}

/* Rows of any width, in the order of the reference's multi-row kernel
 * (inference_fusion.cuh:53-86): 256 threads, thread t sums columns t+256i in
 * sequence, a descending shuffle tree per warp, then the eight warp sums through
 * the same tree; scale = rsqrt(sum/width + eps). */
template <typename T>
__global__ void __launch_bounds__(256) rms_rows_kernel(int rows, int width, float epsilon,
                                                       const T *input, const T *weight, T *output)
{
    __shared__ float warp_sums[8];
    for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
        const T *source = input + row * width;
        float sum = 0.f;
        for (int column = threadIdx.x; column < width; column += 256) {
            float value = Storage<T>::load(source, column);
            sum = __fadd_rn(sum, __fmul_rn(value, value));
        }
        for (int offset = 16; offset; offset >>= 1)
            sum = __fadd_rn(sum, __shfl_down_sync(0xffffffffu, sum, offset));
        if ((threadIdx.x & 31) == 0)
            warp_sums[threadIdx.x >> 5] = sum;
        __syncthreads();
        if (threadIdx.x < 32) {
            sum = threadIdx.x < 8 ? warp_sums[threadIdx.x] : 0.f;
            for (int offset = 16; offset; offset >>= 1)
                sum = __fadd_rn(sum, __shfl_down_sync(0xffffffffu, sum, offset));
            if (threadIdx.x == 0)
                warp_sums[0] = rsqrtf(sum / static_cast<float>(width) + epsilon);
        }
        __syncthreads();
        const float scale = warp_sums[0];
        for (int column = threadIdx.x; column < width; column += 256) {
            float normalised = Storage<T>::round(__fmul_rn(Storage<T>::load(source, column), scale));
            Storage<T>::store(output, row * width + column,
                              __fmul_rn(normalised, Storage<T>::load(weight, column)));
        }
        __syncthreads();
    }
}

__global__ void square_kernel(size_t count, const __nv_bfloat16 *input, float *output)
{
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < count;
         i += size_t(gridDim.x) * blockDim.x) {
        float value = __bfloat162float(input[i]);
        output[i] = __fmul_rn(value, value);
    }
}

template <typename T>
__global__ void scale_kernel(size_t count, int width, float epsilon, const T *input,
                             const T *weight, const float *means, T *output)
{
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < count;
         i += size_t(gridDim.x) * blockDim.x) {
        float scale = rsqrtf(__fadd_rn(means[i / width], epsilon));
        float normalised = Storage<T>::round(__fmul_rn(Storage<T>::load(input, i), scale));
        Storage<T>::store(output, i, __fmul_rn(normalised, Storage<T>::load(weight, i % width)));
    }
}

/* SiLU(gate) rounded to storage, then times up (inference_fusion.cuh:19-29). */
template <typename T>
__global__ void silu_multiply_kernel(size_t count, const T *gate, const T *up, T *output)
{
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < count;
         i += size_t(gridDim.x) * blockDim.x) {
        float g = Storage<T>::load(gate, i);
        float activated = Storage<T>::round(g / (1.f + expf(-g)));
        Storage<T>::store(output, i, activated * Storage<T>::load(up, i));
    }
}

/* SiLU(gate)*up with optional clip and per-row routing factor; one rounding
 * (inference_fusion.cuh:31-51). Comparisons, not fmin/fmax, so NaNs survive. */
template <typename T>
__global__ void swiglu_kernel(size_t count, int width, float limit, const T *gate, const T *up,
                              const float *routing, T *output)
{
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < count;
         i += size_t(gridDim.x) * blockDim.x) {
        float g = Storage<T>::load(gate, i), u = Storage<T>::load(up, i);
        if (limit > 0.f) {
            g = g > limit ? limit : g;
            u = u > limit ? limit : u;
            u = u < -limit ? -limit : u;
        }
        float value = __fmul_rn(g / (1.f + expf(-g)), u);
        if (routing != nullptr)
            value = __fmul_rn(routing[i / width], value);
        Storage<T>::store(output, i, value);
    }
}

} // namespace rms
