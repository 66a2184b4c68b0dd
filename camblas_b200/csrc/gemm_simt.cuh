/*
 * FP32 and FP64 GEMM on the CUDA cores: camblas_cuda_sgemm / camblas_cuda_dgemm.
 *
 * The reference sends these to cuBLAS, cuBLASLt or its Strassen levels
 * (src/cuda/backend.cu:786-866). They are not on the BF16/FP8 path this library
 * is built around - B200 has no FP32 tensor-core mode that keeps FP32 products
 * (TF32 is excluded by the reference's own contract) - so this is a plain,
 * correct, reasonably tiled kernel that completes the ABI: column-major
 * C = alpha op(A) op(B) + beta C, all four transpose pairs, any leading
 * dimensions, accumulation in the storage type in ascending k per thread.
 * A 128 x 64 tile of C per CTA of 256 threads, an 8 x 4 register block per
 * thread, 16-deep K slices staged in shared memory (two buffers: the next slice
 * is fetched into registers while the current one is multiplied). Every policy
 * value multiplies classically.
 */
#pragma once

#include <cuda_runtime.h>

namespace simt
{

constexpr int kTileM = 128, kTileN = 64;
/* K slice depth: 16 for FP32, 8 for FP64 (the two buffers fit the 48 KB of static shared memory) */
template <typename T> constexpr int depth_of = sizeof(T) == 8 ? 8 : 16;

template <typename T> struct Task {
    int m, n, k;
    bool ta, tb;
    long long lda, ldb, ldc;
    T alpha, beta;
    const T *a, *b;
    T *c;
};

template <typename T> __global__ void __launch_bounds__(256) gemm_simt(const Task<T> task)
{
    constexpr int kDepth = depth_of<T>;
    constexpr int kMovesA = kTileM * kDepth / 256, kMovesB = kTileN * kDepth / 256;
    __shared__ T as[2][kDepth][kTileM + 4];
    __shared__ T bs[2][kDepth][kTileN + 4];
    const int i0 = blockIdx.x * kTileM, j0 = blockIdx.y * kTileN;
    const int ti = threadIdx.x & 15, tj = threadIdx.x >> 4; /* 16 x 16 threads */
    T acc[8][4] = {};
    /* each thread moves kMovesA elements of the A slice and kMovesB of the B slice */
    T a_next[kMovesA], b_next[kMovesB];
    auto fetch = [&](int l0) {
#pragma unroll
        for (int u = 0; u < kMovesA; ++u) {
            const int index = threadIdx.x + 256 * u; /* over kTileM * kDepth */
            /* walk the contiguous direction of op(A) with consecutive threads */
            const int i = task.ta ? index / kDepth : index % kTileM;
            const int l = task.ta ? index % kDepth : index / kTileM;
            T value = T(0);
            if (i0 + i < task.m && l0 + l < task.k)
                value = task.ta ? task.a[(l0 + l) + (i0 + i) * task.lda]
                                : task.a[(i0 + i) + (l0 + l) * task.lda];
            a_next[u] = value;
        }
#pragma unroll
        for (int u = 0; u < kMovesB; ++u) {
            const int index = threadIdx.x + 256 * u; /* over kTileN * kDepth */
            const int j = task.tb ? index % kTileN : index / kDepth;
            const int l = task.tb ? index / kTileN : index % kDepth;
            T value = T(0);
            if (j0 + j < task.n && l0 + l < task.k)
                value = task.tb ? task.b[(j0 + j) + (l0 + l) * task.ldb]
                                : task.b[(l0 + l) + (j0 + j) * task.ldb];
            b_next[u] = value;
        }
    };
    auto stage = [&](int buffer) {
#pragma unroll
        for (int u = 0; u < kMovesA; ++u) {
            const int index = threadIdx.x + 256 * u;
            const int i = task.ta ? index / kDepth : index % kTileM;
            const int l = task.ta ? index % kDepth : index / kTileM;
            as[buffer][l][i] = a_next[u];
        }
#pragma unroll
        for (int u = 0; u < kMovesB; ++u) {
            const int index = threadIdx.x + 256 * u;
            const int j = task.tb ? index % kTileN : index / kDepth;
            const int l = task.tb ? index / kTileN : index % kDepth;
            bs[buffer][l][j] = b_next[u];
        }
    };
    fetch(0);
    stage(0);
    __syncthreads();
    int buffer = 0;
    for (int l0 = 0; l0 < task.k; l0 += kDepth) {
        const bool more = l0 + kDepth < task.k;
        if (more)
            fetch(l0 + kDepth);
#pragma unroll
        for (int l = 0; l < kDepth; ++l) {
            T av[8], bv[4];
#pragma unroll
            for (int u = 0; u < 8; ++u)
                av[u] = as[buffer][l][ti + 16 * u];
#pragma unroll
            for (int w = 0; w < 4; ++w)
                bv[w] = bs[buffer][l][tj + 16 * w];
#pragma unroll
            for (int u = 0; u < 8; ++u)
#pragma unroll
                for (int w = 0; w < 4; ++w)
                    acc[u][w] += av[u] * bv[w];
        }
        if (more) {
            stage(buffer ^ 1);
            __syncthreads();
            buffer ^= 1;
        }
    }
#pragma unroll
    for (int u = 0; u < 8; ++u)
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const int i = i0 + ti + 16 * u, j = j0 + tj + 16 * w;
            if (i < task.m && j < task.n) {
                T value = task.alpha * acc[u][w];
                if (task.beta != T(0))
                    value += task.beta * task.c[i + j * task.ldc];
                task.c[i + j * task.ldc] = value;
            }
        }
}

/* C = beta * C over the m x n window (beta == 0 writes zeros without reading). */
template <typename T> __global__ void scale_window(int m, int n, T beta, T *c, long long ldc)
{
    const long long index = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (index >= static_cast<long long>(m) * n)
        return;
    const long long at = index % m + (index / m) * ldc;
    c[at] = beta == T(0) ? T(0) : beta * c[at];
}

} // namespace simt
