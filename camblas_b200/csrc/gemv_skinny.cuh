/*
 * Weight-streaming kernel for a handful of tokens (1..4): out[t,o] =
 * sum_k x[t,k] * w[o,k]. The product is bound by reading w once from HBM, so
 * the kernel is organised around 128-bit coalesced loads of weight rows:
 *   - a CTA of eight warps owns RowsPerWarp*8 consecutive weight rows and one
 *     K split; the token slice of that split is staged once in shared memory;
 *   - each lane reads 16 bytes (8 BF16) of each of its RowsPerWarp rows per
 *     step, consecutive lanes reading consecutive 16-byte pieces, and keeps
 *     RowsPerWarp x Tokens FP32 accumulators;
 *   - lanes are combined by warp shuffles; with one split the result is
 *     scaled and rounded in place, otherwise FP32 partials go to scratch
 *     [split][token][output] and are summed in split order by
 *     skinny_reduce (no floating-point atomics, so results are repeatable).
 * The design follows the reference's FP32 decode kernel (two rows per block,
 * float4 streaming, shuffle plus shared-memory reduce, decode_float.cuh:2-41)
 * but is written for BF16 and several tokens.
 */
#pragma once

#include "sm100_primitives.cuh"

namespace skinny
{

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;

struct Task {
    int outputs, tokens, depth; /* weight rows, token count, K */
    long long ldw, ldx;         /* row strides of w and x in elements */
    int split, depth_per_split; /* depth_per_split is a multiple of 8 */
    float alpha, beta;
    const __nv_bfloat16 *w, *x;
    __nv_bfloat16 *out; /* out[t*ld_out + o] */
    long long ld_out;
    const __nv_bfloat16 *addend; /* addend[t*ld_add + o], read when beta != 0 */
    long long ld_add;
    const __nv_bfloat16 *bias; /* per output, may be NULL */
    float *partial;            /* [split][tokens][outputs] when split > 1 */
};

__device__ __forceinline__ uint4 load_stream(const void *pointer)
{
    uint4 value;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(value.x), "=r"(value.y), "=r"(value.z), "=r"(value.w)
                 : "l"(pointer));
    return value;
}

template <int Tokens, int RowsPerWarp>
__global__ void __launch_bounds__(kThreads) skinny_gemv(const Task task)
{
    extern __shared__ __align__(16) uint8_t shared[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int part = blockIdx.y;
    const int k0 = part * task.depth_per_split;
    const int k1 = min(task.depth, k0 + task.depth_per_split);
    const int span = k1 - k0;        /* multiple of 8 except possibly at the tail */
    const int vectors = span >> 3;   /* whole 16-byte pieces */
    const int span8 = (span + 7) & ~7;

    const int row0 = (blockIdx.x * kWarps + warp) * RowsPerWarp;
    const bool active = row0 < task.outputs; /* warps beyond the last row only help staging */
    const __nv_bfloat16 *rows[RowsPerWarp];
#pragma unroll
    for (int r = 0; r < RowsPerWarp; ++r)
        rows[r] = task.w + static_cast<long long>(min(row0 + r, task.outputs - 1)) * task.ldw + k0;

    /* The first batch of weight loads is issued before the tokens are staged,
     * so that the HBM latency of a short row runs under the staging and its
     * barrier instead of after them. */
    constexpr int kUnroll = RowsPerWarp >= 4 ? 2 : 4;
    uint4 wv[kUnroll][RowsPerWarp];
    int v = lane;
    const bool ahead = active && v + (kUnroll - 1) * 32 < vectors;
    if (ahead) {
#pragma unroll
        for (int u = 0; u < kUnroll; ++u)
#pragma unroll
            for (int r = 0; r < RowsPerWarp; ++r)
                wv[u][r] = load_stream(rows[r] + (v + u * 32) * 8);
    }

    /* Stage the token slice: [Tokens][span8] BF16, zero padded. */
    __nv_bfloat16 *xs = reinterpret_cast<__nv_bfloat16 *>(shared);
    for (int t = 0; t < Tokens; ++t) {
        const __nv_bfloat16 *source = task.x + t * task.ldx + k0;
        for (int i = threadIdx.x; i < span8; i += kThreads)
            xs[t * span8 + i] = (t < task.tokens && i < span) ? source[i] : __float2bfloat16(0.f);
    }
    __syncthreads();
    if (!active)
        return;

    float acc[RowsPerWarp][Tokens];
#pragma unroll
    for (int r = 0; r < RowsPerWarp; ++r)
#pragma unroll
        for (int t = 0; t < Tokens; ++t)
            acc[r][t] = 0.f;

    auto multiply = [&](int at) {
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
#pragma unroll
            for (int t = 0; t < Tokens; ++t) {
                uint4 xv = *reinterpret_cast<const uint4 *>(xs + t * span8 + (at + u * 32) * 8);
                const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
                for (int r = 0; r < RowsPerWarp; ++r) {
                    const uint32_t ww[4] = {wv[u][r].x, wv[u][r].y, wv[u][r].z, wv[u][r].w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        acc[r][t] = fmaf(sm100::bf16_low(ww[i]), sm100::bf16_low(xw[i]), acc[r][t]);
                        acc[r][t] =
                            fmaf(sm100::bf16_high(ww[i]), sm100::bf16_high(xw[i]), acc[r][t]);
                    }
                }
            }
        }
    };
    if (ahead) {
        multiply(v);
        v += kUnroll * 32;
    }
    for (; v + (kUnroll - 1) * 32 < vectors; v += kUnroll * 32) {
#pragma unroll
        for (int u = 0; u < kUnroll; ++u)
#pragma unroll
            for (int r = 0; r < RowsPerWarp; ++r)
                wv[u][r] = load_stream(rows[r] + (v + u * 32) * 8);
        multiply(v);
    }
    for (; v < vectors; v += 32) {
#pragma unroll
        for (int r = 0; r < RowsPerWarp; ++r) {
            uint4 wq = load_stream(rows[r] + v * 8);
            const uint32_t ww[4] = {wq.x, wq.y, wq.z, wq.w};
#pragma unroll
            for (int t = 0; t < Tokens; ++t) {
                uint4 xv = *reinterpret_cast<const uint4 *>(xs + t * span8 + v * 8);
                const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    acc[r][t] = fmaf(sm100::bf16_low(ww[i]), sm100::bf16_low(xw[i]), acc[r][t]);
                    acc[r][t] = fmaf(sm100::bf16_high(ww[i]), sm100::bf16_high(xw[i]), acc[r][t]);
                }
            }
        }
    }
    /* ragged tail of fewer than eight elements */
    for (int i = vectors * 8 + lane; i < span; i += 32) {
#pragma unroll
        for (int r = 0; r < RowsPerWarp; ++r) {
            float wf = __bfloat162float(rows[r][i]);
#pragma unroll
            for (int t = 0; t < Tokens; ++t)
                acc[r][t] = fmaf(wf, __bfloat162float(xs[t * span8 + i]), acc[r][t]);
        }
    }

#pragma unroll
    for (int r = 0; r < RowsPerWarp; ++r)
#pragma unroll
        for (int t = 0; t < Tokens; ++t) {
            float value = acc[r][t];
#pragma unroll
            for (int offset = 16; offset; offset >>= 1)
                value += __shfl_xor_sync(0xffffffffu, value, offset);
            acc[r][t] = value;
        }

    if (lane == 0) {
#pragma unroll
        for (int r = 0; r < RowsPerWarp; ++r) {
            const int o = row0 + r;
            if (o >= task.outputs)
                break;
#pragma unroll
            for (int t = 0; t < Tokens; ++t) {
                if (t >= task.tokens)
                    break;
                if (task.split > 1) {
                    task.partial[(static_cast<long long>(part) * task.tokens + t) * task.outputs +
                                 o] = acc[r][t];
                } else {
                    float value = task.alpha * acc[r][t];
                    if (task.bias != nullptr)
                        value += __bfloat162float(task.bias[o]);
                    if (task.beta != 0.f)
                        value = fmaf(task.beta, __bfloat162float(task.addend[t * task.ld_add + o]),
                                     value);
                    task.out[t * task.ld_out + o] = __float2bfloat16_rn(value);
                }
            }
        }
    }
}

/* out[t,o] = rnd(alpha * (p_0 + p_1 + ... in split order) + bias + beta*addend) */
__global__ void skinny_reduce(const Task task)
{
    const int o = blockIdx.x * blockDim.x + threadIdx.x;
    const int t = blockIdx.y;
    if (o >= task.outputs)
        return;
    float sum = 0.f;
    for (int s = 0; s < task.split; ++s)
        sum += task.partial[(static_cast<long long>(s) * task.tokens + t) * task.outputs + o];
    float value = task.alpha * sum;
    if (task.bias != nullptr)
        value += __bfloat162float(task.bias[o]);
    if (task.beta != 0.f)
        value = fmaf(task.beta, __bfloat162float(task.addend[t * task.ld_add + o]), value);
    task.out[t * task.ld_out + o] = __float2bfloat16_rn(value);
}

} // namespace skinny
