/*
 * Residual add + RMS normalisation and the elementwise kernels beside it. All
 * of them are bound by HBM traffic, so they are built around three rules: every
 * byte is read from global memory once, accesses are 8- or 16-byte vectors that
 * a warp issues as whole 128-byte lines, and a thread has all the loads of its
 * row in flight before it uses the first of them.
 *
 * Arithmetic order. Results are meant to agree with the reference bit for bit
 * wherever the device functions involved (rsqrtf, expf) agree, so the order of
 * the FP32 roundings is the reference's and products and sums are rounded
 * separately (__fmul_rn/__fadd_rn, never contracted):
 *   - single-row normalisation (inference_fusion.cuh:136-191): 512 threads, four
 *     running sums per thread over columns 4t+o+2048i, a shared-memory halving
 *     tree down to one warp, a shuffle tree whose direction is selectable;
 *   - multi-row normalisation (inference_fusion.cuh:53-86): 256 threads, thread
 *     t adds columns t+256i in sequence, a descending shuffle tree per warp, then
 *     the eight warp sums through the same tree.
 * How the data reaches the threads is this library's own: rows_in_registers
 * keeps a row's values in registers between the sum and the scaling pass,
 * rows_staged brings a row into shared memory with 16-byte loads and lets the
 * threads pick their strided columns from there.
 */
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace rms
{

/* Storage type <-> FP32, scalar and as the widest vector a thread moves:
 * kLanes elements in 16 bytes. */
template <typename T> struct Storage;
template <> struct Storage<float> {
    static constexpr int kLanes = 4;
    using Raw4 = float4; /* four elements as they are stored */
    static __device__ __forceinline__ Raw4 load_raw4(const float *p, long long i)
    {
        return *reinterpret_cast<const float4 *>(p + i);
    }
    static __device__ __forceinline__ void store_raw4(float *p, long long i, Raw4 q)
    {
        *reinterpret_cast<float4 *>(p + i) = q;
    }
    static __device__ __forceinline__ void unpack4(Raw4 q, float (&v)[4])
    {
        v[0] = q.x, v[1] = q.y, v[2] = q.z, v[3] = q.w;
    }
    static __device__ __forceinline__ Raw4 pack4(const float (&v)[4])
    {
        return make_float4(v[0], v[1], v[2], v[3]);
    }
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
    static __device__ __forceinline__ void load16(const float *p, long long i, float (&v)[4])
    {
        load4(p, i, v);
    }
    static __device__ __forceinline__ void store16(float *p, long long i, const float (&v)[4])
    {
        store4(p, i, v);
    }
};
template <> struct Storage<__nv_bfloat16> {
    static constexpr int kLanes = 8;
    using Raw4 = uint2;
    static __device__ __forceinline__ Raw4 load_raw4(const __nv_bfloat16 *p, long long i)
    {
        return *reinterpret_cast<const uint2 *>(p + i);
    }
    static __device__ __forceinline__ void store_raw4(__nv_bfloat16 *p, long long i, Raw4 q)
    {
        *reinterpret_cast<uint2 *>(p + i) = q;
    }
    static __device__ __forceinline__ void unpack4(Raw4 q, float (&v)[4])
    {
        v[0] = __uint_as_float(q.x << 16), v[1] = __uint_as_float(q.x & 0xffff0000u);
        v[2] = __uint_as_float(q.y << 16), v[3] = __uint_as_float(q.y & 0xffff0000u);
    }
    static __device__ __forceinline__ Raw4 pack4(const float (&v)[4])
    {
        __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
        return make_uint2(*reinterpret_cast<uint32_t *>(&a), *reinterpret_cast<uint32_t *>(&b));
    }
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
    static __device__ __forceinline__ float low(uint32_t word) { return __uint_as_float(word << 16); }
    static __device__ __forceinline__ float high(uint32_t word)
    {
        return __uint_as_float(word & 0xffff0000u);
    }
    static __device__ __forceinline__ uint32_t pack(float a, float b)
    {
        __nv_bfloat162 pair = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t *>(&pair);
    }
    static __device__ __forceinline__ void load4(const __nv_bfloat16 *p, long long i, float (&v)[4])
    {
        uint2 q = *reinterpret_cast<const uint2 *>(p + i);
        v[0] = low(q.x), v[1] = high(q.x), v[2] = low(q.y), v[3] = high(q.y);
    }
    static __device__ __forceinline__ void store4(__nv_bfloat16 *p, long long i,
                                                  const float (&v)[4])
    {
        *reinterpret_cast<uint2 *>(p + i) = make_uint2(pack(v[0], v[1]), pack(v[2], v[3]));
    }
    static __device__ __forceinline__ void load16(const __nv_bfloat16 *p, long long i,
                                                  float (&v)[8])
    {
        uint4 q = *reinterpret_cast<const uint4 *>(p + i);
        v[0] = low(q.x), v[1] = high(q.x), v[2] = low(q.y), v[3] = high(q.y);
        v[4] = low(q.z), v[5] = high(q.z), v[6] = low(q.w), v[7] = high(q.w);
    }
    static __device__ __forceinline__ void store16(__nv_bfloat16 *p, long long i,
                                                   const float (&v)[8])
    {
        *reinterpret_cast<uint4 *>(p + i) = make_uint4(pack(v[0], v[1]), pack(v[2], v[3]),
                                                       pack(v[4], v[5]), pack(v[6], v[7]));
    }
};

/* Row pitches in elements of the four row-structured buffers of the single-row
 * order kernels (a contiguous matrix has all four equal to the width). */
struct RowPitch {
    long long input, residual, added, output;
};

constexpr int kRowThreads = 512;
constexpr int kRowSpan = kRowThreads * 4; /* columns one sweep of the 512 threads covers */

/* Sum of the 512 per-thread values in the single-row order: halving tree in
 * shared memory down to 32, then a shuffle tree (descending: offsets 16..1,
 * ascending: 1..16). Returns the total in thread 0 only. */
__device__ __forceinline__ float row_tree_sum(float sum, float *tree, int t, bool descending)
{
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
    }
    return sum;
}

/* One row per CTA, the row held in registers in its stored form: Sweeps
 * four-element vectors per thread (width <= Sweeps * 2048, width % 4 == 0, all
 * pointers aligned for four-element vectors). The loads of input and residual
 * are all issued before the first value is used, the weight loads before the
 * reduction tree so that they arrive while it runs; the sums run over the
 * values in the order 4t+o+2048i; the scaling pass unpacks the registers again,
 * so input and residual are read exactly once and nothing depends on this
 * CTA's own stores. Keeping the stored form (two registers per four BF16
 * values; rnd(x+r) is exactly representable) is what lets four CTAs share an
 * SM - with the row unpacked to FP32 only two fit and the kernel ran a quarter
 * slower on rows streamed from HBM. */
template <typename T, int Sweeps>
constexpr int rows_in_registers_ctas()
{
    return (sizeof(T) == 2 && Sweeps <= 4) ? 4 : (sizeof(T) * Sweeps <= 16 ? 2 : 1);
}

template <typename T, typename W, bool Add, int Sweeps>
__global__ void __launch_bounds__(kRowThreads, rows_in_registers_ctas<T, Sweeps>())
    rows_in_registers(int width, RowPitch pitch, float epsilon, const T *__restrict__ input,
                      const T *__restrict__ residual, const W *__restrict__ weight,
                      T *__restrict__ added, T *__restrict__ output, bool round_before_weight,
                      bool descending)
{
    __shared__ float tree[kRowThreads];
    __shared__ float scale_slot;
    const long long row = blockIdx.x;
    input += row * pitch.input, output += row * pitch.output;
    if (Add)
        residual += row * pitch.residual, added += row * pitch.added;
    const int t = threadIdx.x;
    typename Storage<T>::Raw4 kept[Sweeps], other[Sweeps];
#pragma unroll
    for (int i = 0; i < Sweeps; ++i) {
        const int column = i * kRowSpan + t * 4;
        if (column < width) {
            kept[i] = Storage<T>::load_raw4(input, column);
            if (Add)
                other[i] = Storage<T>::load_raw4(residual, column);
        }
    }
    float sums[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < Sweeps; ++i) {
        const int column = i * kRowSpan + t * 4;
        if (column < width) {
            float v[4];
            Storage<T>::unpack4(kept[i], v);
            if (Add) {
                float r[4];
                Storage<T>::unpack4(other[i], r);
#pragma unroll
                for (int o = 0; o < 4; ++o)
                    v[o] = Storage<T>::round(__fadd_rn(v[o], r[o]));
                kept[i] = Storage<T>::pack4(v);
                Storage<T>::store_raw4(added, column, kept[i]);
            }
#pragma unroll
            for (int o = 0; o < 4; ++o)
                sums[o] = __fadd_rn(sums[o], __fmul_rn(v[o], v[o]));
        }
    }
    typename Storage<W>::Raw4 gamma[Sweeps];
#pragma unroll
    for (int i = 0; i < Sweeps; ++i) {
        const int column = i * kRowSpan + t * 4;
        if (column < width)
            gamma[i] = Storage<W>::load_raw4(weight, column);
    }
    float sum = __fadd_rn(__fadd_rn(__fadd_rn(sums[0], sums[1]), sums[2]), sums[3]);
    sum = row_tree_sum(sum, tree, t, descending);
    if (t == 0)
        scale_slot = rsqrtf(__fadd_rn(__fmul_rn(sum, 1.f / static_cast<float>(width)), epsilon));
    __syncthreads();
    const float scale = scale_slot;
#pragma unroll
    for (int i = 0; i < Sweeps; ++i) {
        const int column = i * kRowSpan + t * 4;
        if (column < width) {
            float v[4], g[4];
            Storage<T>::unpack4(kept[i], v);
            Storage<W>::unpack4(gamma[i], g);
#pragma unroll
            for (int o = 0; o < 4; ++o) {
                float normalised = __fmul_rn(v[o], scale);
                if (round_before_weight)
                    normalised = Storage<T>::round(normalised);
                v[o] = __fmul_rn(normalised, g[o]);
            }
            Storage<T>::store_raw4(output, column, Storage<T>::pack4(v));
        }
    }
}

/* The same arithmetic for rows that do not fit the register kernel (wider than
 * 16384 columns), whose pointers are not aligned for vector access, or whose
 * output is the input (in place): two sweeps over global memory, the second one
 * re-forming x+r instead of reading back this CTA's own stores, and every
 * element read before it is overwritten. Vector selects four-element vector
 * access. */
template <typename T, typename W, bool Add, bool Vector>
__global__ void __launch_bounds__(kRowThreads)
    rows_two_sweeps(int width, RowPitch pitch, float epsilon, const T *input, const T *residual,
                    const W *weight, T *added, T *output, bool round_before_weight, bool descending)
{
    __shared__ float tree[kRowThreads];
    __shared__ float scale_slot;
    const long long row = blockIdx.x;
    input += row * pitch.input, output += row * pitch.output;
    if (Add)
        residual += row * pitch.residual, added += row * pitch.added;
    constexpr long long base = 0;
    const int t = threadIdx.x;
    auto fetch = [&](int column, float (&v)[4]) {
        if (Vector) {
            Storage<T>::load4(input + base, column, v);
            if (Add) {
                float r[4];
                Storage<T>::load4(residual + base, column, r);
#pragma unroll
                for (int o = 0; o < 4; ++o)
                    v[o] = Storage<T>::round(__fadd_rn(v[o], r[o]));
            }
        } else {
#pragma unroll
            for (int o = 0; o < 4; ++o) {
                v[o] = Storage<T>::load(input + base, column + o);
                if (Add)
                    v[o] = Storage<T>::round(
                        __fadd_rn(v[o], Storage<T>::load(residual + base, column + o)));
            }
        }
    };
    float sums[4] = {0.f, 0.f, 0.f, 0.f};
    for (int column = t * 4; column < width; column += kRowSpan) {
        float v[4];
        fetch(column, v);
        if (Add) {
            if (Vector) {
                Storage<T>::store4(added + base, column, v);
            } else {
#pragma unroll
                for (int o = 0; o < 4; ++o)
                    Storage<T>::store(added + base, column + o, v[o]);
            }
        }
#pragma unroll
        for (int o = 0; o < 4; ++o)
            sums[o] = __fadd_rn(sums[o], __fmul_rn(v[o], v[o]));
    }
    float sum = __fadd_rn(__fadd_rn(__fadd_rn(sums[0], sums[1]), sums[2]), sums[3]);
    sum = row_tree_sum(sum, tree, t, descending);
    if (t == 0)
        scale_slot = rsqrtf(__fadd_rn(__fmul_rn(sum, 1.f / static_cast<float>(width)), epsilon));
    __syncthreads();
    const float scale = scale_slot;
    for (int column = t * 4; column < width; column += kRowSpan) {
        float v[4], g[4];
        fetch(column, v);
        if (Vector) {
            Storage<W>::load4(weight, column, g);
        } else {
#pragma unroll
            for (int o = 0; o < 4; ++o)
                g[o] = Storage<W>::load(weight, column + o);
        }
#pragma unroll
        for (int o = 0; o < 4; ++o) {
            float normalised = __fmul_rn(v[o], scale);
            if (round_before_weight)
                normalised = Storage<T>::round(normalised);
            v[o] = __fmul_rn(normalised, g[o]);
        }
        if (Vector) {
            Storage<T>::store4(output + base, column, v);
        } else {
#pragma unroll
            for (int o = 0; o < 4; ++o)
                Storage<T>::store(output + base, column + o, v[o]);
        }
    }
}

constexpr int kStagedThreads = 256;

/* Sum over the 256 threads in the multi-row order: descending shuffle tree per
 * warp, the eight warp sums through the same tree. Every thread gets the total. */
__device__ __forceinline__ float staged_tree_sum(float sum, float *warp_sums)
{
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
            warp_sums[8] = sum;
    }
    __syncthreads();
    return warp_sums[8];
}

/* Rows of any width, multi-row order. With Staged the row is brought into
 * dynamic shared memory by 16-byte loads (width a multiple of the vector
 * length, pointers 16-byte aligned, row fits in `width * sizeof(T)` bytes of
 * shared memory), each thread then takes its columns t+256i from there, and the
 * scaling pass reads shared memory and writes 16-byte vectors: one global read
 * of the row instead of two strided ones. A CTA that works through several rows
 * fetches the next row into registers (up to kPrefetch vectors per thread, i.e.
 * rows of up to 16 KB) while it reduces and scales the current one, so that its
 * share of the memory system does not idle during the two passes. Without
 * Staged both passes read global memory element by element. The output may be
 * the input: a row is complete in shared memory (or each element read) before
 * it is overwritten, and the row fetched ahead is a different row. */
constexpr int kPrefetch = 4;

template <typename T, bool Staged>
__global__ void __launch_bounds__(kStagedThreads)
    rows_staged(int rows, int width, float epsilon, const T *input, const T *weight, T *output)
{
    extern __shared__ __align__(16) uint8_t staged_bytes[];
    __shared__ float warp_sums[9];
    T *row_copy = reinterpret_cast<T *>(staged_bytes);
    constexpr int kLanes = Storage<T>::kLanes;
    const int t = threadIdx.x;
    const bool ahead = Staged && width <= kPrefetch * kStagedThreads * kLanes;
    uint4 next[kPrefetch];
    auto fetch = [&](long long row) {
        const T *source = input + row * width;
#pragma unroll
        for (int i = 0; i < kPrefetch; ++i) {
            const int column = (i * kStagedThreads + t) * kLanes;
            if (column < width)
                next[i] = *reinterpret_cast<const uint4 *>(source + column);
        }
    };
    if (ahead && blockIdx.x < rows)
        fetch(blockIdx.x);
    for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
        const T *source = input + row * width;
        float sum = 0.f;
        if (Staged) {
            if (ahead) {
#pragma unroll
                for (int i = 0; i < kPrefetch; ++i) {
                    const int column = (i * kStagedThreads + t) * kLanes;
                    if (column < width)
                        *reinterpret_cast<uint4 *>(row_copy + column) = next[i];
                }
                if (row + gridDim.x < rows)
                    fetch(row + gridDim.x);
            } else {
                for (int column = t * kLanes; column < width; column += kStagedThreads * kLanes)
                    *reinterpret_cast<uint4 *>(row_copy + column) =
                        *reinterpret_cast<const uint4 *>(source + column);
            }
            __syncthreads();
            for (int column = t; column < width; column += kStagedThreads) {
                const float value = Storage<T>::load(row_copy, column);
                sum = __fadd_rn(sum, __fmul_rn(value, value));
            }
        } else {
            for (int column = t; column < width; column += kStagedThreads) {
                const float value = Storage<T>::load(source, column);
                sum = __fadd_rn(sum, __fmul_rn(value, value));
            }
        }
        sum = staged_tree_sum(sum, warp_sums);
        const float scale = rsqrtf(sum / static_cast<float>(width) + epsilon);
        if (Staged) {
            for (int column = t * kLanes; column < width; column += kStagedThreads * kLanes) {
                float v[kLanes], g[kLanes];
                Storage<T>::load16(row_copy, column, v);
                Storage<T>::load16(weight, column, g);
#pragma unroll
                for (int o = 0; o < kLanes; ++o)
                    v[o] = __fmul_rn(Storage<T>::round(__fmul_rn(v[o], scale)), g[o]);
                Storage<T>::store16(output, row * width + column, v);
            }
        } else {
            for (int column = t; column < width; column += kStagedThreads) {
                const float normalised =
                    Storage<T>::round(__fmul_rn(Storage<T>::load(source, column), scale));
                Storage<T>::store(output, row * width + column,
                                  __fmul_rn(normalised, Storage<T>::load(weight, column)));
            }
        }
        __syncthreads(); /* the row copy and warp_sums are reused by the next row */
    }
}

/* ---- elementwise kernels -------------------------------------------------------
 * Each works on 16-byte vectors (eight BF16 or four FP32) over the leading
 * `vectors * kLanes` elements and finishes the remaining elements one by one;
 * the host passes vectors = 0 when a pointer is not 16-byte aligned. A thread
 * takes kBatch vectors per step, a grid stride apart, and loads all of their
 * operands before it computes and stores any of them, so that several memory
 * requests per thread are in flight whatever the compiler can prove about
 * aliasing. Outputs may be one of the inputs: a thread reads its vectors
 * before it writes those same vectors. `width`-dependent kernels are
 * vectorised only when width is a multiple of the vector length, so that a
 * vector never crosses a row. SiLU costs an exponential and an IEEE division
 * per element in the reference's expression, which is kept so that the bits
 * agree; on B200 that arithmetic is within a factor of two of the memory time,
 * so these kernels do not reach the copy bandwidth. */
constexpr int kBatch = 4; /* square and scale: plain streaming */
constexpr int kBatchSilu = 1; /* the SiLU kernels are bound by instruction issue (about forty
                                 instructions per element): more resident threads beat more
                                 loads per thread, measured 0.78 against 0.70 of the copy rate */

/* output[i] = input[i]^2 in FP32 (the per-element squares the multi-kernel RMS
 * path of the reference averages, backend.cu:1442-1454). */
__global__ void __launch_bounds__(256)
    square_kernel(size_t count, size_t vectors, const __nv_bfloat16 *input, float *output)
{
    const size_t stride = size_t(gridDim.x) * blockDim.x;
    const size_t first = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    for (size_t vector = first; vector < vectors; vector += kBatch * stride) {
        uint4 raw[kBatch];
#pragma unroll
        for (int b = 0; b < kBatch; ++b)
            if (vector + b * stride < vectors)
                raw[b] = *reinterpret_cast<const uint4 *>(input + (vector + b * stride) * 8);
#pragma unroll
        for (int b = 0; b < kBatch; ++b)
            if (vector + b * stride < vectors) {
                const uint32_t words[4] = {raw[b].x, raw[b].y, raw[b].z, raw[b].w};
                float v[8];
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    v[2 * w] = Storage<__nv_bfloat16>::low(words[w]);
                    v[2 * w + 1] = Storage<__nv_bfloat16>::high(words[w]);
                }
                float4 *target = reinterpret_cast<float4 *>(output + (vector + b * stride) * 8);
                target[0] = make_float4(__fmul_rn(v[0], v[0]), __fmul_rn(v[1], v[1]),
                                        __fmul_rn(v[2], v[2]), __fmul_rn(v[3], v[3]));
                target[1] = make_float4(__fmul_rn(v[4], v[4]), __fmul_rn(v[5], v[5]),
                                        __fmul_rn(v[6], v[6]), __fmul_rn(v[7], v[7]));
            }
    }
    for (size_t i = vectors * 8 + first; i < count; i += stride) {
        const float value = __bfloat162float(input[i]);
        output[i] = __fmul_rn(value, value);
    }
}

/* Sixteen bytes of T as FP32 values and back. */
template <typename T> __device__ __forceinline__ void unpack16(uint4 raw, float (&v)[Storage<T>::kLanes]);
template <> __device__ __forceinline__ void unpack16<float>(uint4 raw, float (&v)[4])
{
    v[0] = __uint_as_float(raw.x), v[1] = __uint_as_float(raw.y);
    v[2] = __uint_as_float(raw.z), v[3] = __uint_as_float(raw.w);
}
template <> __device__ __forceinline__ void unpack16<__nv_bfloat16>(uint4 raw, float (&v)[8])
{
    using S = Storage<__nv_bfloat16>;
    v[0] = S::low(raw.x), v[1] = S::high(raw.x), v[2] = S::low(raw.y), v[3] = S::high(raw.y);
    v[4] = S::low(raw.z), v[5] = S::high(raw.z), v[6] = S::low(raw.w), v[7] = S::high(raw.w);
}
template <typename T> __device__ __forceinline__ uint4 pack16(const float (&v)[Storage<T>::kLanes]);
template <> __device__ __forceinline__ uint4 pack16<float>(const float (&v)[4])
{
    return make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]),
                      __float_as_uint(v[3]));
}
template <> __device__ __forceinline__ uint4 pack16<__nv_bfloat16>(const float (&v)[8])
{
    using S = Storage<__nv_bfloat16>;
    return make_uint4(S::pack(v[0], v[1]), S::pack(v[2], v[3]), S::pack(v[4], v[5]),
                      S::pack(v[6], v[7]));
}

/* The batched loop shared by the two-operand kernels: for every vector of this
 * thread, element(a, b, index of the vector's first element) -> result values
 * written over a. */
template <typename T, typename Element>
__device__ __forceinline__ void for_each_vector(size_t vectors, const T *left, const T *right,
                                                T *output, Element element)
{
    constexpr int kLanes = Storage<T>::kLanes;
    constexpr int kBatch = kBatchSilu;
    const size_t stride = size_t(gridDim.x) * blockDim.x;
    const size_t first = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    for (size_t vector = first; vector < vectors; vector += kBatch * stride) {
        uint4 a[kBatch], b[kBatch];
#pragma unroll
        for (int s = 0; s < kBatch; ++s)
            if (vector + s * stride < vectors) {
                a[s] = *reinterpret_cast<const uint4 *>(left + (vector + s * stride) * kLanes);
                b[s] = *reinterpret_cast<const uint4 *>(right + (vector + s * stride) * kLanes);
            }
#pragma unroll
        for (int s = 0; s < kBatch; ++s)
            if (vector + s * stride < vectors) {
                float x[kLanes], y[kLanes];
                unpack16<T>(a[s], x);
                unpack16<T>(b[s], y);
                element(x, y, (vector + s * stride) * kLanes);
                *reinterpret_cast<uint4 *>(output + (vector + s * stride) * kLanes) = pack16<T>(x);
            }
    }
}

/* output = rnd(rnd(input * rsqrt(means[row] + eps)) * weight[column]) with a
 * mean of squares per row supplied by the caller (backend.cu:1456-1475). */
template <typename T>
__global__ void __launch_bounds__(256)
    scale_kernel(size_t count, size_t vectors, int width, float epsilon, const T *input,
                 const T *weight, const float *means, T *output)
{
    constexpr int kLanes = Storage<T>::kLanes;
    const size_t stride = size_t(gridDim.x) * blockDim.x;
    const size_t first = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    for (size_t vector = first; vector < vectors; vector += kBatch * stride) {
        uint4 a[kBatch], b[kBatch];
        float scale[kBatch];
#pragma unroll
        for (int s = 0; s < kBatch; ++s)
            if (vector + s * stride < vectors) {
                const size_t i = (vector + s * stride) * kLanes;
                const size_t row = i / width;
                a[s] = *reinterpret_cast<const uint4 *>(input + i);
                b[s] = *reinterpret_cast<const uint4 *>(weight + (i - row * width));
                scale[s] = means[row];
            }
#pragma unroll
        for (int s = 0; s < kBatch; ++s)
            if (vector + s * stride < vectors) {
                float v[kLanes], g[kLanes];
                unpack16<T>(a[s], v);
                unpack16<T>(b[s], g);
                const float factor = rsqrtf(__fadd_rn(scale[s], epsilon));
#pragma unroll
                for (int o = 0; o < kLanes; ++o)
                    v[o] = __fmul_rn(Storage<T>::round(__fmul_rn(v[o], factor)), g[o]);
                *reinterpret_cast<uint4 *>(output + (vector + s * stride) * kLanes) = pack16<T>(v);
            }
    }
    for (size_t i = vectors * kLanes + first; i < count; i += stride) {
        const float factor = rsqrtf(__fadd_rn(means[i / width], epsilon));
        const float normalised = Storage<T>::round(__fmul_rn(Storage<T>::load(input, i), factor));
        Storage<T>::store(output, i, __fmul_rn(normalised, Storage<T>::load(weight, i % width)));
    }
}

/* SiLU(g) = g / (1 + exp(-g)), the expression of inference_fusion.cuh:19-29. */
__device__ __forceinline__ float silu(float g)
{
    return g / (1.f + expf(-g));
}

/* output = rnd(rnd(SiLU(gate)) * up). */
template <typename T>
__global__ void __launch_bounds__(256)
    silu_multiply_kernel(size_t count, size_t vectors, const T *gate, const T *up, T *output)
{
    constexpr int kLanes = Storage<T>::kLanes;
    for_each_vector<T>(vectors, gate, up, output,
                       [](float (&g)[kLanes], const float (&u)[kLanes], size_t) {
#pragma unroll
                           for (int o = 0; o < kLanes; ++o)
                               g[o] = Storage<T>::round(silu(g[o])) * u[o];
                       });
    const size_t stride = size_t(gridDim.x) * blockDim.x;
    const size_t first = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    for (size_t i = vectors * kLanes + first; i < count; i += stride) {
        const float activated = Storage<T>::round(silu(Storage<T>::load(gate, i)));
        Storage<T>::store(output, i, activated * Storage<T>::load(up, i));
    }
}

/* One element of the clipped, routed SwiGLU (inference_fusion.cuh:31-51): gate
 * clipped from above, up from both sides (comparisons rather than fmin/fmax, so
 * that NaNs pass through), SiLU(gate) * up, times the row's routing factor, one
 * rounding by the caller. */
__device__ __forceinline__ float swiglu_element(float g, float u, float limit, bool routed,
                                                float factor)
{
    if (limit > 0.f) {
        g = g > limit ? limit : g;
        u = u > limit ? limit : u;
        u = u < -limit ? -limit : u;
    }
    float value = __fmul_rn(silu(g), u);
    if (routed)
        value = __fmul_rn(factor, value);
    return value;
}

template <typename T>
__global__ void __launch_bounds__(256)
    swiglu_kernel(size_t count, size_t vectors, int width, float limit, const T *gate, const T *up,
                  const float *routing, T *output)
{
    constexpr int kLanes = Storage<T>::kLanes;
    const bool routed = routing != nullptr;
    for_each_vector<T>(vectors, gate, up, output,
                       [&](float (&g)[kLanes], const float (&u)[kLanes], size_t index) {
                           const float factor = routed ? routing[index / width] : 1.f;
#pragma unroll
                           for (int o = 0; o < kLanes; ++o)
                               g[o] = swiglu_element(g[o], u[o], limit, routed, factor);
                       });
    const size_t stride = size_t(gridDim.x) * blockDim.x;
    const size_t first = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    for (size_t i = vectors * kLanes + first; i < count; i += stride)
        Storage<T>::store(output, i,
                          swiglu_element(Storage<T>::load(gate, i), Storage<T>::load(up, i), limit,
                                         routed, routed ? routing[i / width] : 1.f));
}

} // namespace rms
