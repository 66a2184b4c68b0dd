/*
 * Block-scaled FP8 / FP4 products with power-of-two (E8M0) scales and the
 * expert routing beside them: camblas_cuda_quantized_matmul,
 * camblas_cuda_grouped_quantized_matmul, camblas_cuda_route_groups,
 * camblas_cuda_reduce_groups.
 *
 * The reference multiplies 32-deep K blocks with mma.sync, scales each block
 * sum by the two power-of-two factors and adds the blocks in ascending order in
 * FP32; every warp re-reads its operands from global memory for each block
 * (src/cuda/quantized.cuh:22-156). Here the arithmetic is moved in front of the
 * tensor cores instead: because the scales are powers of two, an E4M3 or E2M1
 * value times its block scale is exactly a BF16 number (four significant bits,
 * BF16's exponent range), so both operands are rewritten once as BF16 images
 * with the scales folded in, and the product is the library's ordinary tcgen05
 * BF16 GEMM with FP32 accumulation. Every term a*w that the reference adds is
 * formed exactly in both schemes; the results differ only by the order in which
 * FP32 sums are rounded (rel-L2 far inside the 2e-2 FP8 bound). The price is
 * one pass over the operands (reads N*K, writes 2*N*K bytes for the weight) per
 * call, which the caller of a static weight pays again on every call because
 * the ABI has no place to keep a prepared weight.
 *
 * Layouts (reference include/camblas_cuda.h:122-176): input E4M3 [rows, inner],
 * input scales E8M0 [rows, inner/activation_block]; FP8 weight E4M3
 * [outputs, inner] with scales E8M0 [ceil(outputs/32), inner/32] (one per
 * 32 x 32 block); packed weight E2M1, two values per byte, low nibble first,
 * [outputs, inner/2] with scales E8M0 [outputs, inner/32]; BF16 output
 * [rows, outputs].
 */
#pragma once

#include "context.cuh"
#include "dispatch_bf16.cuh"

#include <cuda_fp8.h>

namespace quant
{

/* E8M0 byte -> FP32 factor: 2^(v-127); 0 is 2^-127 (an FP32 denormal), 255 NaN. */
__device__ __forceinline__ float power_of_two(uint32_t byte)
{
    if (byte == 255u)
        return __uint_as_float(0x7fc00000u);
    return __uint_as_float(byte == 0u ? 0x00400000u : byte << 23);
}

__device__ __forceinline__ float e4m3_value(uint32_t byte)
{
    __half_raw half = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(byte), __NV_E4M3);
    return __half2float(*reinterpret_cast<__half *>(&half));
}

/* E2M1 nibble: sign, two exponent bits, one mantissa bit: 0, 0.5, 1, 1.5, 2, 3, 4, 6. */
__device__ __forceinline__ float e2m1_value(uint32_t nibble)
{
    const uint32_t magnitude = nibble & 7u;
    const float table = magnitude < 2u ? 0.5f * magnitude
                                       : __uint_as_float(((magnitude >> 1) + 126u) << 23) *
                                             (1.f + 0.5f * (magnitude & 1u));
    return (nibble & 8u) ? -table : table;
}

__device__ __forceinline__ uint32_t pack_pair(float low, float high)
{
    __nv_bfloat162 pair = __floats2bfloat162_rn(low, high);
    return *reinterpret_cast<uint32_t *>(&pair);
}

struct Images {
    int groups;         /* batches (1 for the plain product) */
    int weight_groups;  /* entries of metadata (grouped form) */
    int rows, outputs, inner, activation_block;
    const uint8_t *input, *input_scale;
    const uint8_t *weight, *weight_scale; /* plain form */
    const uint64_t *metadata;             /* grouped form: [weight_groups][2] addresses */
    const int32_t *active, *counts;       /* grouped form: [groups] */
    __nv_bfloat16 *input_image;           /* [groups][rows][inner] */
    __nv_bfloat16 *weight_image;          /* [groups][outputs][inner] */
};

/* BF16 image of the activations: sixteen bytes in, thirty-two out per thread.
 * Rows at or beyond the batch's (clipped) count and batches without a valid
 * weight group become zeros, which makes their output rows zeros. */
__global__ void __launch_bounds__(256) input_image_kernel(const Images task)
{
    const long long per_row = task.inner >> 4;
    const long long total = 1ll * task.groups * task.rows * per_row;
    const int scale_blocks = task.inner / task.activation_block;
    for (long long item = 1ll * blockIdx.x * blockDim.x + threadIdx.x; item < total;
         item += 1ll * gridDim.x * blockDim.x) {
        const long long row = item / per_row; /* over all batches */
        const int column = static_cast<int>(item - row * per_row) << 4;
        bool live = true;
        if (task.active != nullptr) {
            const int batch = static_cast<int>(row / task.rows);
            const int within = static_cast<int>(row - 1ll * batch * task.rows);
            const int selected = task.active[batch];
            const int count = max(0, min(task.rows, task.counts[batch]));
            live = selected >= 0 && selected < task.weight_groups && within < count;
        }
        uint4 out[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
        if (live) {
            const uint4 raw = *reinterpret_cast<const uint4 *>(task.input + row * task.inner + column);
            const float factor =
                power_of_two(task.input_scale[row * scale_blocks + column / task.activation_block]);
            const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
            uint32_t packed[8];
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                packed[2 * w] = pack_pair(e4m3_value(words[w] & 255u) * factor,
                                          e4m3_value((words[w] >> 8) & 255u) * factor);
                packed[2 * w + 1] = pack_pair(e4m3_value((words[w] >> 16) & 255u) * factor,
                                              e4m3_value(words[w] >> 24) * factor);
            }
            out[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            out[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
        }
        uint4 *target = reinterpret_cast<uint4 *>(task.input_image + row * task.inner + column);
        target[0] = out[0];
        target[1] = out[1];
    }
}

/* BF16 image of the weight of every batch: a thread rewrites sixteen
 * consecutive values of one weight row (half a scale block). */
template <bool Packed> __global__ void __launch_bounds__(256) weight_image_kernel(const Images task)
{
    const long long per_row = task.inner >> 4;
    const long long per_batch = 1ll * task.outputs * per_row;
    const long long total = task.groups * per_batch;
    const int blocks = task.inner >> 5;
    for (long long item = 1ll * blockIdx.x * blockDim.x + threadIdx.x; item < total;
         item += 1ll * gridDim.x * blockDim.x) {
        const int batch = static_cast<int>(item / per_batch);
        const long long local = item - batch * per_batch;
        const int row = static_cast<int>(local / per_row);
        const int column = static_cast<int>(local - row * per_row) << 4;
        const uint8_t *weight = task.weight, *scales = task.weight_scale;
        bool live = true;
        if (task.active != nullptr) {
            const int selected = task.active[batch];
            live = selected >= 0 && selected < task.weight_groups;
            if (live) {
                weight = reinterpret_cast<const uint8_t *>(task.metadata[2ll * selected]);
                scales = reinterpret_cast<const uint8_t *>(task.metadata[2ll * selected + 1]);
            }
        }
        uint32_t packed[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (live) {
            const int block = column >> 5;
            const float factor =
                power_of_two(scales[(Packed ? 1ll * row : 1ll * (row >> 5)) * blocks + block]);
            if (Packed) {
                const uint2 raw = *reinterpret_cast<const uint2 *>(
                    weight + 1ll * row * (task.inner >> 1) + (column >> 1));
                const uint32_t words[2] = {raw.x, raw.y};
#pragma unroll
                for (int w = 0; w < 2; ++w)
#pragma unroll
                    for (int pair = 0; pair < 4; ++pair) {
                        const uint32_t byte = (words[w] >> (8 * pair)) & 255u;
                        packed[4 * w + pair] = pack_pair(e2m1_value(byte & 15u) * factor,
                                                         e2m1_value(byte >> 4) * factor);
                    }
            } else {
                const uint4 raw =
                    *reinterpret_cast<const uint4 *>(weight + 1ll * row * task.inner + column);
                const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    packed[2 * w] = pack_pair(e4m3_value(words[w] & 255u) * factor,
                                              e4m3_value((words[w] >> 8) & 255u) * factor);
                    packed[2 * w + 1] = pack_pair(e4m3_value((words[w] >> 16) & 255u) * factor,
                                                  e4m3_value(words[w] >> 24) * factor);
                }
            }
        }
        uint4 *target = reinterpret_cast<uint4 *>(task.weight_image + batch * per_batch * 16 +
                                                  1ll * row * task.inner + column);
        target[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        target[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
    }
}

inline unsigned grid_for(const camblas_cuda_context *context, long long items)
{
    const long long blocks = (items + 255) / 256;
    const long long limit = 1ll * context->sm_count * 16;
    return unsigned(blocks < 1 ? 1 : (blocks < limit ? blocks : limit));
}

/* Both images, then one BF16 product per batch. */
inline int run(camblas_cuda_context *context, bool packed, Images task, __nv_bfloat16 *output)
{
    const size_t input_elements = size_t(task.groups) * task.rows * task.inner;
    const size_t weight_elements = size_t(task.groups) * task.outputs * task.inner;
    const size_t input_bytes = (input_elements * 2 + 255) & ~size_t(255);
    int status = host::reserve_operands(context, input_bytes + weight_elements * 2);
    if (status != 0)
        return status;
    task.input_image = static_cast<__nv_bfloat16 *>(context->operands);
    task.weight_image = reinterpret_cast<__nv_bfloat16 *>(static_cast<uint8_t *>(context->operands) +
                                                          input_bytes);
    input_image_kernel<<<grid_for(context, input_elements / 16), 256, 0, context->stream>>>(task);
    status = host::launched(context, "quantized input image");
    if (status != 0)
        return status;
    if (packed)
        weight_image_kernel<true>
            <<<grid_for(context, weight_elements / 16), 256, 0, context->stream>>>(task);
    else
        weight_image_kernel<false>
            <<<grid_for(context, weight_elements / 16), 256, 0, context->stream>>>(task);
    status = host::launched(context, "quantized weight image");
    for (int batch = 0; status == 0 && batch < task.groups; ++batch) {
        host::Product p{};
        p.ta = true, p.tb = false, p.m = task.outputs, p.n = task.rows, p.k = task.inner;
        p.alpha = 1.f, p.beta = 0.f;
        p.a = task.weight_image + size_t(batch) * task.outputs * task.inner, p.lda = task.inner;
        p.b = task.input_image + size_t(batch) * task.rows * task.inner, p.ldb = task.inner;
        p.c = output + size_t(batch) * task.rows * task.outputs, p.ldc = task.outputs;
        p.addend = nullptr, p.ld_add = 0;
        p.cut0 = p.cut1 = task.outputs;
        status = host::run_product(context, p);
    }
    return status;
}

/* ---- routing ------------------------------------------------------------------- */

/* group_of[slot] = first group whose active id equals the slot's local expert id,
 * or -1 (ids below first_expert or not below INT_MAX are ignored; duplicate
 * active ids select their first group). */
__global__ void __launch_bounds__(256)
    match_groups_kernel(int slots_count, int first_expert, int groups, const int64_t *experts,
                        const int32_t *active, int32_t *group_of, bool stage)
{
    /* the active ids are searched once per slot: keep them in shared memory when they fit */
    extern __shared__ int32_t staged_ids[];
    const int32_t *active_copy = active;
    if (stage) {
        for (int g = threadIdx.x; g < groups; g += blockDim.x)
            staged_ids[g] = active[g];
        __syncthreads();
        active_copy = staged_ids;
    }
    for (long long slot = 1ll * blockIdx.x * blockDim.x + threadIdx.x; slot < slots_count;
         slot += 1ll * gridDim.x * blockDim.x) {
        const int64_t expert = experts[slot];
        int found = -1;
        if (expert >= first_expert && expert < INT_MAX) {
            const int local = static_cast<int>(expert) - first_expert;
            for (int g = 0; g < groups; ++g)
                if (active_copy[g] == local) {
                    found = g;
                    break;
                }
        }
        group_of[slot] = found;
    }
}

/* One CTA per group walks the slots in ascending order and numbers its own:
 * row r of group g is the r-th slot (by index) routed to g. The reference
 * numbers them with an atomic counter, i.e. in whatever order its threads
 * happen to run (routing.cuh:2-24); here the layout is the same from run to
 * run. counts[g] is the number of slots routed to g, also beyond `rows`;
 * slots without a row keep -1 in `reverse`. */
__global__ void __launch_bounds__(256)
    number_groups_kernel(int slots_count, int rows, const int32_t *group_of, int32_t *counts,
                         int32_t *slots, int32_t *reverse)
{
    __shared__ int warp_totals[8];
    __shared__ int base;
    const int group = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0)
        base = 0;
    __syncthreads();
    for (int start = 0; start < slots_count; start += 256) {
        const int slot = start + threadIdx.x;
        const bool mine = slot < slots_count && group_of[slot] == group;
        const unsigned ballot = __ballot_sync(0xffffffffu, mine);
        if (lane == 0)
            warp_totals[warp] = __popc(ballot);
        __syncthreads();
        int before = base + __popc(ballot & ((1u << lane) - 1u));
        for (int w = 0; w < warp; ++w)
            before += warp_totals[w];
        if (mine && before < rows) {
            slots[1ll * group * rows + before] = slot;
            reverse[slot] = group * rows + before;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            int total = 0;
            for (int w = 0; w < 8; ++w)
                total += warp_totals[w];
            base += total;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0)
        counts[group] = base;
}

/* output[token][column] = sum over the token's choices, in ascending
 * (expert id, choice index) order, of input[reverse[token][choice]][column],
 * FP32 adds of BF16 values (routing.cuh:26-60). One CTA per token: the order
 * is worked out once, then the threads stream eight columns at a time. */
__global__ void __launch_bounds__(256)
    reduce_groups_kernel(int choices, int width, int grouped_rows, const int64_t *experts,
                         const int32_t *reverse, const __nv_bfloat16 *input, float *output,
                         bool vector)
{
    __shared__ int ordered_rows[64];
    __shared__ int ordered_count;
    const long long token = blockIdx.x;
    if (threadIdx.x == 0) {
        /* selection sort over at most 64 choices; invalid experts never enter */
        int taken = 0;
        long long previous = -1;
        int previous_choice = -1;
        for (int step = 0; step < choices; ++step) {
            long long smallest = INT_MAX;
            int selected = -1;
            for (int top = 0; top < choices; ++top) {
                const long long expert = experts[token * choices + top];
                const bool valid = expert >= 0 && expert < INT_MAX;
                const bool after = expert > previous || (expert == previous && top > previous_choice);
                if (valid && after && (expert < smallest || (expert == smallest && selected < 0))) {
                    smallest = expert;
                    selected = top;
                }
            }
            if (selected < 0)
                break;
            const int row = reverse[token * choices + selected];
            if (row >= 0 && row < grouped_rows)
                ordered_rows[taken++] = row;
            previous = smallest;
            previous_choice = selected;
        }
        ordered_count = taken;
    }
    __syncthreads();
    const int count = ordered_count;
    float *target = output + token * width;
    if (vector) {
        for (int column = threadIdx.x * 8; column < width; column += blockDim.x * 8) {
            float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int i = 0; i < count; ++i) {
                const uint4 raw = *reinterpret_cast<const uint4 *>(
                    input + 1ll * ordered_rows[i] * width + column);
                const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    sum[2 * w] = __fadd_rn(sum[2 * w], __uint_as_float(words[w] << 16));
                    sum[2 * w + 1] = __fadd_rn(sum[2 * w + 1], __uint_as_float(words[w] & 0xffff0000u));
                }
            }
            reinterpret_cast<float4 *>(target + column)[0] = make_float4(sum[0], sum[1], sum[2], sum[3]);
            reinterpret_cast<float4 *>(target + column)[1] = make_float4(sum[4], sum[5], sum[6], sum[7]);
        }
    } else {
        for (int column = threadIdx.x; column < width; column += blockDim.x) {
            float sum = 0.f;
            for (int i = 0; i < count; ++i)
                sum = __fadd_rn(sum, __bfloat162float(input[1ll * ordered_rows[i] * width + column]));
            target[column] = sum;
        }
    }
}

} // namespace quant

/* ---- extern "C" ------------------------------------------------------------------ */

namespace quant
{
inline bool dimensions_bad(int packed, int rows, int outputs, int inner, int activation_block)
{
    const bool block_ok = activation_block == 32 || (packed == 1 && activation_block == 128);
    return (packed != 0 && packed != 1) || rows < 0 || rows > 65535 || outputs < 8 || outputs % 8 ||
           inner < 32 || inner % 32 || !block_ok || inner % activation_block;
}
} // namespace quant

extern "C" int camblas_cuda_quantized_matmul(camblas_cuda_context *context, int packed, int rows,
                                             int outputs, int inner, int activation_block,
                                             const void *input, const void *input_scale,
                                             const void *weight, const void *weight_scale,
                                             void *output)
{
    return host::guarded(context, [&] {
        if (quant::dimensions_bad(packed, rows, outputs, inner, activation_block))
            return host::fail(context, "invalid quantized matrix dimensions", 1);
        if (rows == 0)
            return 0;
        const void *read[4] = {input, input_scale, weight, weight_scale};
        bool bad = !output || (uintptr_t(output) & 1);
        for (const void *pointer : read)
            bad = bad || !pointer || pointer == output;
        if (bad || (uintptr_t(input) & 3) || (uintptr_t(weight) & (packed ? 1 : 3)))
            return host::fail(context, "invalid quantized matrix buffers", 1);
        /* the image kernels move sixteen input bytes (eight packed bytes) at a time */
        if ((uintptr_t(input) & 15) || (uintptr_t(weight) & (packed ? 7 : 15)))
            return host::fail(context, "quantized operands must be 16-byte aligned", 1);
        quant::Images task{};
        task.groups = 1, task.weight_groups = 1;
        task.rows = rows, task.outputs = outputs, task.inner = inner;
        task.activation_block = activation_block;
        task.input = static_cast<const uint8_t *>(input);
        task.input_scale = static_cast<const uint8_t *>(input_scale);
        task.weight = static_cast<const uint8_t *>(weight);
        task.weight_scale = static_cast<const uint8_t *>(weight_scale);
        context->counts[0]++;
        return quant::run(context, packed == 1, task, static_cast<__nv_bfloat16 *>(output));
    });
}

extern "C" int camblas_cuda_grouped_quantized_matmul(camblas_cuda_context *context, int packed,
                                                     int groups, int weight_groups, int rows,
                                                     int outputs, int inner, int activation_block,
                                                     const void *input, const void *input_scale,
                                                     const void *metadata, const void *active,
                                                     const void *counts, void *output)
{
    return host::guarded(context, [&] {
        if (quant::dimensions_bad(packed, rows, outputs, inner, activation_block) || groups < 0 ||
            groups > 65535 || weight_groups < 1 || weight_groups > 65535 ||
            uint64_t(groups) * uint64_t(rows) > SIZE_MAX / (uint64_t(outputs) * 2))
            return host::fail(context, "invalid grouped matrix dimensions", 1);
        if (groups == 0 || rows == 0)
            return 0;
        const void *read[5] = {input, input_scale, metadata, active, counts};
        bool bad = !output || (uintptr_t(output) & 1);
        for (const void *pointer : read)
            bad = bad || !pointer || pointer == output;
        if (bad || (uintptr_t(input) & 15) || (uintptr_t(metadata) & 7) || (uintptr_t(active) & 3) ||
            (uintptr_t(counts) & 3))
            return host::fail(context, "invalid grouped matrix buffers", 1);
        quant::Images task{};
        task.groups = groups, task.weight_groups = weight_groups;
        task.rows = rows, task.outputs = outputs, task.inner = inner;
        task.activation_block = activation_block;
        task.input = static_cast<const uint8_t *>(input);
        task.input_scale = static_cast<const uint8_t *>(input_scale);
        task.metadata = static_cast<const uint64_t *>(metadata);
        task.active = static_cast<const int32_t *>(active);
        task.counts = static_cast<const int32_t *>(counts);
        context->counts[0] += uint64_t(groups);
        return quant::run(context, packed == 1, task, static_cast<__nv_bfloat16 *>(output));
    });
}

extern "C" int camblas_cuda_route_groups(camblas_cuda_context *context, int tokens, int choices,
                                         int first_expert, int groups, int rows,
                                         const void *experts, const void *active, void *counts,
                                         void *slots, void *reverse)
{
    return host::guarded(context, [&] {
        const bool sizes_ok = tokens >= 0 && choices >= 1 && choices <= 64 && first_expert >= 0 &&
                              groups >= 1 && groups <= 65535 && rows >= 1 && rows <= 65535 &&
                              int64_t(tokens) * choices <= INT_MAX &&
                              int64_t(groups) * rows <= INT_MAX;
        const void *all[5] = {experts, active, counts, slots, reverse};
        bool distinct = true;
        for (int i = 0; i < 5; ++i)
            for (int j = i + 1; j < 5; ++j)
                distinct = distinct && (all[i] == nullptr || all[i] != all[j]);
        const bool present = counts && slots && active && (tokens == 0 || (experts && reverse));
        const bool aligned = !(uintptr_t(experts) & 7) && !(uintptr_t(active) & 3) &&
                             !(uintptr_t(counts) & 3) && !(uintptr_t(slots) & 3) &&
                             !(uintptr_t(reverse) & 3);
        if (!sizes_ok || !present || !distinct || !aligned)
            return host::fail(context, "invalid routing dimensions or buffers", 1);
        const int slots_count = tokens * choices;
        int status = host::reserve_scratch(context, size_t(slots_count ? slots_count : 1) * 4);
        if (status != 0)
            return status;
        cudaError_t error = cudaMemsetAsync(counts, 0, size_t(groups) * 4, context->stream);
        if (error == cudaSuccess)
            error = cudaMemsetAsync(slots, 255, size_t(groups) * rows * 4, context->stream);
        if (error == cudaSuccess && tokens)
            error = cudaMemsetAsync(reverse, 255, size_t(slots_count) * 4, context->stream);
        if (error != cudaSuccess)
            return host::fail(context, "routing initialisation", error);
        if (tokens == 0)
            return 0;
        int32_t *group_of = static_cast<int32_t *>(context->scratch);
        const bool stage = groups <= 8192;
        quant::match_groups_kernel<<<quant::grid_for(context, slots_count), 256,
                                     stage ? size_t(groups) * 4 : 0, context->stream>>>(
            slots_count, first_expert, groups, static_cast<const int64_t *>(experts),
            static_cast<const int32_t *>(active), group_of, stage);
        status = host::launched(context, "expert matching");
        if (status != 0)
            return status;
        quant::number_groups_kernel<<<groups, 256, 0, context->stream>>>(
            slots_count, rows, group_of, static_cast<int32_t *>(counts),
            static_cast<int32_t *>(slots), static_cast<int32_t *>(reverse));
        return host::launched(context, "expert routing");
    });
}

extern "C" int camblas_cuda_reduce_groups(camblas_cuda_context *context, int tokens, int choices,
                                          int width, int grouped_rows, const void *experts,
                                          const void *reverse, const void *input, void *output)
{
    return host::guarded(context, [&] {
        const bool sizes_ok = tokens >= 0 && choices >= 1 && choices <= 64 && width >= 1 &&
                              grouped_rows >= 0 && int64_t(tokens) * choices <= INT_MAX;
        const bool present = (grouped_rows == 0 || input) && (tokens == 0 || (experts && reverse && output));
        const bool aligned = !(uintptr_t(experts) & 7) && !(uintptr_t(reverse) & 3) &&
                             !(uintptr_t(input) & 1) && !(uintptr_t(output) & 3);
        const bool distinct = tokens == 0 || (output != experts && output != reverse && output != input);
        if (!sizes_ok || !present || !aligned || !distinct)
            return host::fail(context, "invalid grouped reduction arguments", 1);
        if (tokens == 0)
            return 0;
        const bool vector = width % 8 == 0 && !(uintptr_t(input) & 15) && !(uintptr_t(output) & 15);
        quant::reduce_groups_kernel<<<tokens, 256, 0, context->stream>>>(
            choices, width, grouped_rows, static_cast<const int64_t *>(experts),
            static_cast<const int32_t *>(reverse), static_cast<const __nv_bfloat16 *>(input),
            static_cast<float *>(output), vector);
        return host::launched(context, "grouped reduction");
    });
}
