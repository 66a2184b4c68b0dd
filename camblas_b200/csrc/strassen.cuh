/*
 * One level of Strassen for BF16 squares (policy CAMBLAS_CUDA_STRASSEN).
 *
 * The reference applies Strassen to FP32/FP64 'N','N' squares only
 * (backend.cu:442-551, camblas_cuda.h:64-66); this is the same seven-product
 * schedule for BF16 storage:
 *   left  planes  a11+a22, a21+a22, a11, a22, a11+a12, a21-a11, a12-a22
 *   right planes  b11+b22, b11, b12-b22, b21-b11, b22, b11+b12, b21+b22
 * (backend.cu:128-144). The plane sums are rounded to BF16 because they feed the
 * BF16 tensor-core kernel; the seven half-size products are one batched launch
 * of that kernel with FP32 output planes; the quadrants are recombined in FP32
 * in the reference's association order, c11 = ((p1+p4)-p5)+p7, c12 = p3+p5,
 * c21 = p2+p4, c22 = ((p1-p2)+p3)+p6 (backend.cu:163), scaled by alpha, joined
 * with beta*C and rounded once.
 *
 * Range guard. The reference checks every packed input against
 * sqrt(max/(64 n max(1,|alpha|))) and, after a host synchronisation, falls back
 * to the classical product (backend.cu:490-526). Here the pack kernel raises a
 * device flag instead; the batched product and the recombination skip their
 * work when it is set, and a classical launch that runs only when it is set
 * follows - no host synchronisation, so the sequence can be captured in a CUDA
 * graph. Fall-backs are counted in pinned host memory (counter slot 5).
 */
#pragma once

#include "dispatch_bf16.cuh"

#include <cfloat>
#include <cmath>

namespace strassen
{

__global__ void __launch_bounds__(256)
    pack_planes(int h, const __nv_bfloat16 *a, long long lda, const __nv_bfloat16 *b, long long ldb,
                __nv_bfloat16 *left, __nv_bfloat16 *right, float limit, unsigned *unsafe)
{
    const long long plane = static_cast<long long>(h) * h;
    const long long index = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (index >= plane)
        return;
    const int row = static_cast<int>(index % h), column = static_cast<int>(index / h);
    float q[8];
    q[0] = __bfloat162float(a[row + column * lda]);
    q[1] = __bfloat162float(a[row + (column + h) * lda]);
    q[2] = __bfloat162float(a[row + h + column * lda]);
    q[3] = __bfloat162float(a[row + h + (column + h) * lda]);
    q[4] = __bfloat162float(b[row + column * ldb]);
    q[5] = __bfloat162float(b[row + (column + h) * ldb]);
    q[6] = __bfloat162float(b[row + h + column * ldb]);
    q[7] = __bfloat162float(b[row + h + (column + h) * ldb]);
    bool bad = false;
#pragma unroll
    for (int i = 0; i < 8; ++i)
        bad |= !(fabsf(q[i]) <= limit);
    if (__any_sync(__activemask(), bad) && (threadIdx.x & 31) == 0)
        atomicOr(unsafe, 1u);
    const float a11 = q[0], a12 = q[1], a21 = q[2], a22 = q[3];
    const float b11 = q[4], b12 = q[5], b21 = q[6], b22 = q[7];
    /* plane p, element (row, column) at (p*h + column)*h + row */
    const float l[7] = {a11 + a22, a21 + a22, a11, a22, a11 + a12, a21 - a11, a12 - a22};
    const float r[7] = {b11 + b22, b11, b12 - b22, b21 - b11, b22, b11 + b12, b21 + b22};
#pragma unroll
    for (int p = 0; p < 7; ++p) {
        left[p * plane + index] = __float2bfloat16_rn(l[p]);
        right[p * plane + index] = __float2bfloat16_rn(r[p]);
    }
}

/* products[p][j][i] holds (L_p R_p)[i,j]; C is column-major with pitch ldc. */
__global__ void __launch_bounds__(256)
    recombine(int h, float alpha, float beta, const float *products, __nv_bfloat16 *c, long long ldc,
              const unsigned *unsafe, unsigned long long *guard_hits)
{
    if (*unsafe != 0) {
        if (blockIdx.x == 0 && threadIdx.x == 0)
            atomicAdd(guard_hits, 1ull);
        return;
    }
    const long long plane = static_cast<long long>(h) * h;
    const long long index = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (index >= plane)
        return;
    const int i = static_cast<int>(index % h), j = static_cast<int>(index / h);
    float p[7];
#pragma unroll
    for (int s = 0; s < 7; ++s)
        p[s] = products[s * plane + index]; /* (s*h + j)*h + i */
    const float quadrant[4] = {((p[0] + p[3]) - p[4]) + p[6], p[2] + p[4], p[1] + p[3],
                               ((p[0] - p[1]) + p[2]) + p[5]};
    const long long where[4] = {i + j * ldc, i + (j + h) * ldc, i + h + j * ldc,
                                i + h + (j + h) * ldc};
#pragma unroll
    for (int s = 0; s < 4; ++s) {
        float value = alpha * quadrant[s];
        if (beta != 0.f)
            value = fmaf(beta, __bfloat162float(c[where[s]]), value);
        c[where[s]] = __float2bfloat16_rn(value);
    }
}

/* 'N','N' squares whose halves tile evenly (n a multiple of 512), operands the
 * tensor-core kernel can read directly, a finite alpha. */
inline bool eligible(camblas_cuda_context *, const host::Product &x)
{
    return !x.ta && !x.tb && x.m == x.n && x.n == x.k && x.n >= 512 && x.n % 512 == 0 &&
           host::tensor_operands_ok(x) && host::rows_store_ok(x) && std::isfinite(x.alpha) &&
           x.bias == nullptr && x.addend == x.c;
}

inline int run(camblas_cuda_context *context, const host::Product &x)
{
    using namespace sm100;
    const int n = x.n, h = n / 2;
    const size_t plane = size_t(h) * h;
    const size_t bytes = plane * 7 * (2 + 2 + 4);
    int status = host::reserve_scratch(context, bytes);
    if (status != 0) {
        /* No room for the planes: multiply classically and count it, as the
         * reference does when its Strassen workspace cannot be had
         * (backend.cu:490-526). The failed allocation left no CUDA error behind. */
        context->counts[5]++;
        context->error[0] = 0;
        return host::run_product(context, x);
    }
    auto *left = static_cast<__nv_bfloat16 *>(context->scratch);
    auto *right = left + 7 * plane;
    auto *products = reinterpret_cast<float *>(right + 7 * plane);
    unsigned *flag = context->status + 1;
    cudaError_t error = cudaMemsetAsync(flag, 0, sizeof(unsigned), context->stream);
    if (error != cudaSuccess)
        return host::fail(context, "range flag reset", error);
    const float limit =
        sqrtf(FLT_MAX / (64.f * float(n) * fmaxf(1.f, fabsf(x.alpha))));
    const unsigned blocks = unsigned((plane + 255) / 256);
    pack_planes<<<blocks, 256, 0, context->stream>>>(h, x.a, x.lda, x.b, x.ldb, left, right, limit,
                                                     flag);
    status = host::launched(context, "Strassen packing");
    if (status != 0)
        return status;

    GemmTask task{};
    task.rows = h, task.cols = h, task.depth = h;
    task.r_blocks = h / 128, task.c_blocks = h / 256;
    task.k_blocks = h / 64;
    task.split = 1, task.k_blocks_per_split = task.k_blocks;
    task.panel = task.r_blocks < 8 ? task.r_blocks : 8;
    task.alpha = 1.f, task.beta = 0.f;
    task.status = context->status;
    task.cut0 = task.cut1 = h;
    task.batch = 7, task.batch_p = h, task.batch_q = h;
    task.out_float = products, task.ld_out = h;
    task.skip_if_set = flag;
    CUtensorMap p, q;
    const auto bf16 = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    /* P = right planes: row j of plane b is contiguous along l (K-major), planes stacked by rows.
     * Q = left planes: line l of plane b is contiguous along i (MN-major), planes stacked along K. */
    bool ok = host::encode_2d(context, &p, bf16, 2, right, h, 7ull * h, size_t(h) * 2, 64, 128) &&
              host::encode_2d(context, &q, bf16, 2, left, h, 7ull * h, size_t(h) * 2, 64, 64);
    if (!ok)
        return host::fail(context, "tensor map encoding", 1);
    host::launch_tensor<256, 4, kStoreFloat, kMajorK, kMajorMN>(context, p, q, p, p, p, task);
    status = host::launched(context, "Strassen batched product");
    if (status != 0)
        return status;
    recombine<<<blocks, 256, 0, context->stream>>>(h, x.alpha, x.beta, products, x.c, x.ldc, flag,
                                                   context->guard_hits_device);
    status = host::launched(context, "Strassen recombination");
    if (status != 0)
        return status;
    context->counts[1]++;
    /* classical product that runs only when the guard fired */
    host::Product fallback = x;
    fallback.run_if_set = flag;
    return host::run_tensor_rows(context, fallback);
}

} // namespace strassen
