/*
 * CUDA-core BF16 GEMM for operands the tensor-core pipeline cannot take:
 * pointers or leading dimensions that are not 16-byte aligned (TMA needs
 * both), and tiny products. Column-major C = alpha op(A) op(B) + beta C, any
 * transpose pair, any leading dimension, FP32 accumulation in ascending k.
 * A 64x64 tile of C per CTA, a 4x4 register block per thread, operands staged
 * in shared memory as FP32 with every element bounds-checked.
 */
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace generic
{

constexpr int kTile = 64;
constexpr int kDepth = 16;

struct Task {
    int m, n, k;
    bool ta, tb;
    long long lda, ldb, ldc;
    float alpha, beta;
    const __nv_bfloat16 *a, *b;
    __nv_bfloat16 *c;
    const __nv_bfloat16 *bias; /* per row of C (index i), may be NULL */
    const __nv_bfloat16 *addend;
    long long ld_add;
};

__global__ void __launch_bounds__(256) gemm_bf16_generic(const Task task)
{
    __shared__ float as[kDepth][kTile + 1];
    __shared__ float bs[kDepth][kTile + 1];
    const int i0 = blockIdx.x * kTile, j0 = blockIdx.y * kTile;
    const int ti = threadIdx.x & 15, tj = threadIdx.x >> 4;
    float acc[4][4] = {};
    for (int l0 = 0; l0 < task.k; l0 += kDepth) {
        for (int index = threadIdx.x; index < kTile * kDepth; index += 256) {
            /* op(A)[i,l]: 'N' -> a[i + l*lda], 'T' -> a[l + i*lda]; walk the
             * contiguous direction with consecutive threads */
            int i = task.ta ? index / kDepth : index % kTile;
            int l = task.ta ? index % kDepth : index / kTile;
            float value = 0.f;
            if (i0 + i < task.m && l0 + l < task.k)
                value = __bfloat162float(task.ta ? task.a[(l0 + l) + (i0 + i) * task.lda]
                                                 : task.a[(i0 + i) + (l0 + l) * task.lda]);
            as[l][i] = value;
            /* op(B)[l,j]: 'N' -> b[l + j*ldb], 'T' -> b[j + l*ldb] */
            int j = task.tb ? index % kTile : index / kDepth;
            int lb = task.tb ? index / kTile : index % kDepth;
            value = 0.f;
            if (j0 + j < task.n && l0 + lb < task.k)
                value = __bfloat162float(task.tb ? task.b[(j0 + j) + (l0 + lb) * task.ldb]
                                                 : task.b[(l0 + lb) + (j0 + j) * task.ldb]);
            bs[lb][j] = value;
        }
        __syncthreads();
#pragma unroll
        for (int l = 0; l < kDepth; ++l) {
            float av[4], bv[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                av[u] = as[l][ti + 16 * u];
                bv[u] = bs[l][tj + 16 * u];
            }
#pragma unroll
            for (int u = 0; u < 4; ++u)
#pragma unroll
                for (int w = 0; w < 4; ++w)
                    acc[u][w] = fmaf(av[u], bv[w], acc[u][w]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            int i = i0 + ti + 16 * u, j = j0 + tj + 16 * w;
            if (i < task.m && j < task.n) {
                float value = task.alpha * acc[u][w];
                if (task.bias != nullptr)
                    value += __bfloat162float(task.bias[i]);
                if (task.beta != 0.f)
                    value = fmaf(task.beta, __bfloat162float(task.addend[i + j * task.ld_add]),
                                 value);
                task.c[i + j * task.ldc] = __float2bfloat16_rn(value);
            }
        }
}

/* C = beta * C over the m x n window (beta == 0 writes zeros without reading). */
__global__ void scale_window(int m, int n, float beta, __nv_bfloat16 *c, long long ldc)
{
    long long index = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (index >= static_cast<long long>(m) * n)
        return;
    long long at = index % m + (index / m) * ldc;
    c[at] = __float2bfloat16_rn(beta == 0.f ? 0.f : beta * __bfloat162float(c[at]));
}

} // namespace generic
