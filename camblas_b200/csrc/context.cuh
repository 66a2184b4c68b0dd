/*
 * Context object behind the C ABI: device, stream, policy, scratch arena with
 * the reference's capture rules, device status word, launch counters, error
 * text. It holds no vendor-library handle.
 */
#pragma once

#include "../../include/camblas_cuda.h"

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <exception>
#include <new>
#include <vector>

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

/* Tuning and test switches of a context. They are read from the environment
 * once, when the context is created (names in parentheses), and changed
 * afterwards only through camblas_cuda_set_option; no entry point on the call
 * path looks at the environment. */
struct ContextOptions {
    int pair_tail = 0;     /* "pair_tail" (CAMBLAS_B200_PAIR_MODE=plain|sk): 0 cost model, 1 whole
                              tiles only, 2 always split the last wave by K */
    int pair_width = 0;    /* "pair_width" (CAMBLAS_B200_PAIR_MODE=width=<n>): forced tile width of
                              the two-SM kernel, 0 = fixed 256/128-column tiles */
    int push_width = 0;    /* "push_width" (CAMBLAS_B200_PUSH_WIDTH): tile width of the peer-memory
                              row-parallel product, 0 = by shape */
    int fp8_rows = 0;      /* "fp8_rows" (CAMBLAS_B200_FP8_ROWS=four|single): which many-row FP8
                              kernel; all give the same bits. 0 by size; 1, 2 the older
                              128 x 128 forms; 3 / 4 256-column tiles on one / two SMs; 5 the
                              current 128 x 128 form whatever the size */
    int fp8_swapped_rows = 16; /* "fp8_swapped_rows": most token rows the weight-streaming
                                  (swapped, split-K) FP8 modes take, 0 to 128; above it
                                  the row tiling with its K ranges (measured on four
                                  shapes: equal at 17 rows, 5-25 % faster from 33) */
    int cluster_split = 1; /* "cluster_split": K split inside a thread-block cluster: 0 never,
                              1 for row tiles (65 rows and more), 2 also for few-token tiles */
    int bf16_strassen = 0; /* "bf16_strassen" (CAMBLAS_B200_BF16_STRASSEN=1): let policy STRASSEN
                              run one Strassen level on BF16 squares */
    int peer_wait_ms = 5000; /* "peer_wait_ms": how long a kernel waits for another GPU's flag */
};

/* One cached tensor map: the arguments it was encoded from and the result. */
struct TensorMapEntry {
    const void *base = nullptr;
    uint64_t extent0 = 0, extent1 = 0, pitch = 0;
    uint32_t box0 = 0, box1 = 0;
    int type = -1;
    CUtensorMap map;
};

struct camblas_cuda_context {
    int device = 0;
    int algorithm = CAMBLAS_CUDA_AUTO;
    int forced_family = 0;
    int sm_count = 0;
    cudaStream_t stream = nullptr;
    void *scratch = nullptr;
    size_t scratch_bytes = 0;
    bool scratch_captured = false;
    /* second arena, same rules: operands that an entry point rewrites before it
     * multiplies (the BF16 images of block-scaled FP8/FP4 matrices), kept apart
     * from `scratch` because the GEMM that follows uses that one from offset 0 */
    void *operands = nullptr;
    size_t operands_bytes = 0;
    bool operands_captured = false;
    std::vector<void *> retired;
    unsigned *status = nullptr; /* device words: [0] written by bounded waits that gave up,
                                   [1] Strassen range-guard flag of the call in flight */
    unsigned long long *guard_hits = nullptr;        /* pinned host counter of guard fall-backs */
    unsigned long long *guard_hits_device = nullptr; /* the same word as the device sees it */
    EncodeTiledFn encode = nullptr;
    ContextOptions options;
    /* Direct-mapped cache of encoded tensor maps: a serving loop presents the
     * same (pointer, shape) pairs call after call, and a hit costs a 128-byte
     * copy instead of a driver call. */
    static constexpr int kMapSlots = 128;
    TensorMapEntry maps[kMapSlots];
    uint64_t map_hits = 0, map_misses = 0;
    /* clusters of each cluster-split kernel the device keeps resident, by kernel
     * slot and cluster size (0 not asked yet, -1 none) */
    int cluster_capacity[5][9] = {};
    int fp8_cluster_capacity[9] = {}; /* the same for the FP8 row kernel, by cluster size */
    std::atomic<uint64_t> counts[8] = {};
    std::atomic<uint64_t> kernel_launches{0}; /* every kernel this context put on its stream */
    char error[256] = "";
};

namespace host
{

inline thread_local char creation_error[256] = "";

/* Record "<what> failed (status <code>)" and turn the code into a negative
 * status, as the reference does (backend.cu:81-86). */
inline int fail(camblas_cuda_context *context, const char *what, int code)
{
    char *message = context ? context->error : creation_error;
    std::snprintf(message, 256, "%s failed (status %d)", what, code);
    return code > 0 ? -code : -1;
}

/* Run `work` with `device` current and put the caller's device back afterwards,
 * whichever way `work` ends. False, with `error` set and `work` not run, when
 * the device could not be made current. */
template <typename Work> bool on_device(int device, cudaError_t &error, Work work)
{
    int home = -1;
    error = cudaGetDevice(&home);
    const bool move = error == cudaSuccess && home != device;
    if (move)
        error = cudaSetDevice(device);
    if (error != cudaSuccess)
        return false;
    try {
        work();
    } catch (...) {
        if (move)
            cudaSetDevice(home);
        throw;
    }
    if (move)
        cudaSetDevice(home);
    return true;
}

/* Status and message for the exception in flight (call from a catch block).
 * The C ABI lets none out: -2 for an allocation failure, -1 otherwise, the
 * codes of the reference's entry points (backend.cu:913-951). */
inline int exception_status(camblas_cuda_context *context) noexcept
{
    try {
        throw;
    } catch (const std::bad_alloc &) {
        return fail(context, "host allocation", 2);
    } catch (const std::exception &error) {
        std::snprintf(context->error, sizeof(context->error), "host exception: %s", error.what());
    } catch (...) {
        return fail(context, "unexpected host exception", 1);
    }
    return -1;
}

/* Every entry point that takes a context runs through here: on the context's
 * device, with the caller's device restored and host exceptions turned into a
 * status. */
template <typename Function> int guarded(camblas_cuda_context *context, Function function)
{
    if (!context)
        return fail(nullptr, "missing context", 1);
    int status = 0;
    cudaError_t error = cudaSuccess;
    const bool ran = on_device(context->device, error, [&] {
        try {
            status = function();
        } catch (...) {
            status = exception_status(context);
        }
    });
    return ran ? status : fail(context, "activate device", error);
}

inline int launched(camblas_cuda_context *context, const char *what)
{
    cudaError_t error = cudaGetLastError();
    if (context && error == cudaSuccess)
        context->kernel_launches.fetch_add(1, std::memory_order_relaxed);
    return error == cudaSuccess ? 0 : fail(context, what, error);
}

/* Make an arena at least `required` bytes. During stream capture growth is
 * refused and the arena is marked as recorded; a recorded arena is retired, not
 * freed, when it later grows, so replayed graphs keep valid addresses (the rules
 * of the reference's workspace, backend.cu:397-434). */
inline int reserve_arena(camblas_cuda_context *context, void *&base, size_t &bytes, bool &recorded,
                         size_t required, const char *what)
{
    cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
    cudaError_t error = cudaStreamIsCapturing(context->stream, &capture);
    if (error != cudaSuccess)
        return fail(context, "scratch capture status", error);
    const bool capturing = capture != cudaStreamCaptureStatusNone;
    if (required <= bytes) {
        recorded = recorded || capturing;
        return 0;
    }
    if (capturing)
        return fail(context, "warm up scratch storage before CUDA graph capture", 1);
    /* the stream may still be using the old block */
    error = cudaStreamSynchronize(context->stream);
    if (error != cudaSuccess)
        return fail(context, "scratch synchronisation", error);
    constexpr size_t granule = size_t(1) << 20;
    const size_t rounded = (required + granule - 1) / granule * granule;
    void *fresh = nullptr;
    error = cudaMalloc(&fresh, rounded);
    if (error != cudaSuccess) {
        cudaGetLastError();
        return fail(context, what, error);
    }
    if (base != nullptr) {
        if (recorded)
            context->retired.push_back(base);
        else
            cudaFree(base);
    }
    base = fresh, bytes = rounded, recorded = false;
    return 0;
}

inline int reserve_scratch(camblas_cuda_context *context, size_t required)
{
    return reserve_arena(context, context->scratch, context->scratch_bytes,
                         context->scratch_captured, required, "scratch allocation");
}

inline int reserve_operands(camblas_cuda_context *context, size_t required)
{
    return reserve_arena(context, context->operands, context->operands_bytes,
                         context->operands_captured, required, "operand image allocation");
}

/* 2-D tensor map over a row-major [extent1][extent0] array of `element_bytes`
 * elements with row pitch `pitch_bytes`, 128-byte swizzle. */
inline bool encode_2d(camblas_cuda_context *context, CUtensorMap *map, CUtensorMapDataType type,
                      int element_bytes, const void *base, uint64_t extent0, uint64_t extent1,
                      uint64_t pitch_bytes, uint32_t box0, uint32_t box1)
{
    cuuint64_t dims[2] = {extent0, extent1};
    /* A single row never uses the pitch; keep it legal (multiple of 16). */
    if (extent1 == 1)
        pitch_bytes = (extent0 * element_bytes + 15) & ~uint64_t(15);
    uint64_t hash = reinterpret_cast<uintptr_t>(base) >> 4;
    hash = (hash ^ (extent0 * 0x9e3779b97f4a7c15ull) ^ (extent1 * 0xc2b2ae3d27d4eb4full) ^
            (pitch_bytes << 7) ^ (uint64_t(box0) << 20) ^ (uint64_t(box1) << 40) ^ uint64_t(type)) *
           0xff51afd7ed558ccdull;
    TensorMapEntry &entry = context->maps[(hash >> 40) % camblas_cuda_context::kMapSlots];
    if (entry.base == base && entry.extent0 == extent0 && entry.extent1 == extent1 &&
        entry.pitch == pitch_bytes && entry.box0 == box0 && entry.box1 == box1 &&
        entry.type == int(type)) {
        *map = entry.map;
        ++context->map_hits;
        return true;
    }
    cuuint64_t strides[1] = {pitch_bytes};
    cuuint32_t box[2] = {box0, box1};
    cuuint32_t element_strides[2] = {1, 1};
    CUresult result = context->encode(map, type, 2, const_cast<void *>(base), dims, strides, box,
                                      element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (result != CUDA_SUCCESS)
        return false;
    ++context->map_misses;
    entry.base = base, entry.extent0 = extent0, entry.extent1 = extent1, entry.pitch = pitch_bytes;
    entry.box0 = box0, entry.box1 = box1, entry.type = int(type);
    entry.map = *map;
    return true;
}

inline bool aligned16(const void *pointer)
{
    return (reinterpret_cast<uintptr_t>(pointer) & 15) == 0;
}

} // namespace host
