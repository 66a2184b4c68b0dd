/*
 * extern "C" surface of libcamblas_cuda.so for B200. Argument checks and
 * status/error behaviour mirror the reference's wrappers
 * (src/cuda/backend.cu:954-1535, src/cuda/bfloat16.cuh:11-57); the device work
 * is in the headers included below. There is no CPU or vendor-library route:
 * a call either launches one of these kernels or fails with a message.
 */
#include "context.cuh"
#include "dispatch_bf16.cuh"
#include "fp8_block.cuh"
#include "fp8_block_wide.cuh"
#include "gemm_simt.cuh"
#include "dense_fp.cuh"
#include "quantized.cuh"
#include "rms_norm.cuh"
#include "row_parallel.cuh"
#include "static_scratch.cuh"

#include <algorithm>
#include <cmath>
#include <cstdlib>

using host::fail;
using host::guarded;
using host::launched;

namespace
{
int prepare_rms_kernels(); /* defined with the RMS wrappers below */

/* The environment is consulted here, once per context, and nowhere else. */
void options_from_environment(ContextOptions &options)
{
    if (const char *text = std::getenv("CAMBLAS_B200_PAIR_MODE")) {
        if (std::strcmp(text, "plain") == 0)
            options.pair_tail = 1;
        else if (std::strcmp(text, "sk") == 0)
            options.pair_tail = 2;
        else if (std::strncmp(text, "width=", 6) == 0)
            options.pair_width = std::atoi(text + 6);
    }
    if (const char *text = std::getenv("CAMBLAS_B200_PUSH_WIDTH"))
        options.push_width = std::atoi(text);
    if (const char *text = std::getenv("CAMBLAS_B200_FP8_ROWS"))
        options.fp8_rows = std::strcmp(text, "four") == 0 ? 1 : (std::strcmp(text, "single") == 0 ? 2 : 0);
    if (const char *text = std::getenv("CAMBLAS_B200_BF16_STRASSEN"))
        options.bf16_strassen = std::atoi(text) != 0;
}
} // namespace

namespace
{
/* The body of camblas_cuda_create, with `device` current. */
int create_here(int device, void *stream, camblas_cuda_context **out)
{
    auto *context = new (std::nothrow) camblas_cuda_context;
    if (!context)
        return fail(nullptr, "context allocation", 2);
    context->device = device;
    context->stream = static_cast<cudaStream_t>(stream);
    options_from_environment(context->options);
    cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
    int status = int(cudaStreamIsCapturing(context->stream, &capture));
    const char *what = "stream capture status";
    if (status == 0 && capture != cudaStreamCaptureStatusNone) {
        what = "context creation during CUDA graph capture";
        status = 1;
    }
    cudaDeviceProp properties{};
    if (status == 0) {
        what = "device properties";
        status = int(cudaGetDeviceProperties(&properties, device));
    }
    if (status == 0 && properties.major != 10) {
        what = "B200 build on a device that is not compute capability 10.x";
        status = 1;
    }
    if (status == 0) {
        context->sm_count = properties.multiProcessorCount;
        what = "tensor map encoder lookup";
        void *entry = nullptr;
        cudaDriverEntryPointQueryResult query;
        status = int(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault,
                                             &query));
        if (status == 0 && (query != cudaDriverEntryPointSuccess || entry == nullptr))
            status = 1;
        context->encode = reinterpret_cast<EncodeTiledFn>(entry);
    }
    if (status == 0) {
        what = "status word allocation";
        status = int(cudaMalloc(reinterpret_cast<void **>(&context->status), 2 * sizeof(unsigned)));
    }
    if (status == 0) {
        what = "status word initialisation";
        status = int(cudaMemsetAsync(context->status, 0, 2 * sizeof(unsigned), context->stream));
    }
    if (status == 0) {
        what = "guard counter allocation";
        status = int(cudaHostAlloc(reinterpret_cast<void **>(&context->guard_hits),
                                   sizeof(unsigned long long), cudaHostAllocMapped));
        if (status == 0) {
            *context->guard_hits = 0;
            status = int(cudaHostGetDevicePointer(
                reinterpret_cast<void **>(&context->guard_hits_device), context->guard_hits, 0));
        }
    }
    if (status == 0) {
        what = "kernel attributes";
        status = host::prepare_kernels() | fp8::prepare_kernels() | fp8::prepare_wide_kernels() |
                 prepare_rms_kernels();
    }
    if (status != 0) {
        cudaGetLastError();
        int result = fail(nullptr, what, status);
        char keep[256];
        std::memcpy(keep, host::creation_error, sizeof(keep));
        camblas_cuda_destroy(context);
        std::memcpy(host::creation_error, keep, sizeof(keep));
        return result;
    }
    *out = context;
    return 0;
}

/* The body of camblas_cuda_destroy, with the context's device current. */
int destroy_here(camblas_cuda_context *context)
{
    cudaError_t error = cudaStreamSynchronize(context->stream);
    if (context->scratch)
        cudaFree(context->scratch);
    if (context->operands)
        cudaFree(context->operands);
    for (void *allocation : context->retired)
        cudaFree(allocation);
    if (context->status)
        cudaFree(context->status);
    if (context->guard_hits)
        cudaFreeHost(context->guard_hits);
    delete context;
    return error == cudaSuccess ? 0 : fail(nullptr, "stream completion during destruction", error);
}
} // namespace

extern "C" int camblas_cuda_create(int device, void *stream, camblas_cuda_context **out)
{
    if (!out)
        return fail(nullptr, "missing context output", 1);
    *out = nullptr;
    int status = 0;
    cudaError_t error = cudaSuccess;
    if (!host::on_device(device, error, [&] { status = create_here(device, stream, out); }))
        return fail(nullptr, "activate device", error);
    return status;
}

extern "C" int camblas_cuda_destroy(camblas_cuda_context *context)
{
    if (!context)
        return 0;
    int status = 0;
    cudaError_t error = cudaSuccess;
    if (!host::on_device(context->device, error, [&] { status = destroy_here(context); }))
        return fail(context, "activate device for destruction", error);
    return status;
}

extern "C" const char *camblas_cuda_error(const camblas_cuda_context *context)
{
    return context ? context->error : host::creation_error;
}

extern "C" int camblas_cuda_set_algorithm(camblas_cuda_context *context, int algorithm)
{
    if (!context || algorithm < CAMBLAS_CUDA_AUTO || algorithm > CAMBLAS_CUDA_STRASSEN_FOUR)
        return fail(context, "invalid algorithm", 1);
    context->algorithm = algorithm;
    return 0;
}

extern "C" int camblas_cuda_force_kernel(camblas_cuda_context *context, int family)
{
    if (!context || family < 0 || family > 5)
        return fail(context, "invalid kernel family", 1);
    context->forced_family = family;
    return 0;
}

extern "C" int camblas_cuda_set_option(camblas_cuda_context *context, const char *name, int value)
{
    if (!context || !name)
        return fail(context, "missing context or option name", 1);
    ContextOptions &options = context->options;
    struct Known {
        const char *name;
        int *slot;
        int low, high;
    } const known[] = {
        {"pair_tail", &options.pair_tail, 0, 2},
        {"pair_width", &options.pair_width, 0, 256},
        {"push_width", &options.push_width, 0, 256},
        {"fp8_rows", &options.fp8_rows, 0, 5},
        {"fp8_swapped_rows", &options.fp8_swapped_rows, 0, 128},
        {"cluster_split", &options.cluster_split, 0, 2},
        {"bf16_strassen", &options.bf16_strassen, 0, 1},
        {"peer_wait_ms", &options.peer_wait_ms, 1, 60000},
    };
    for (const Known &entry : known)
        if (std::strcmp(name, entry.name) == 0) {
            if (value < entry.low || value > entry.high ||
                (entry.slot == &options.pair_width && value % 16 != 0) ||
                (entry.slot == &options.push_width && value != 0 && value != 128 && value != 256))
                return fail(context, "option value out of range", 1);
            *entry.slot = value;
            return 0;
        }
    return fail(context, "unknown option", 1);
}

extern "C" int camblas_cuda_stats(const camblas_cuda_context *context, uint64_t *counts, int length)
{
    if (!context || !counts || (length != 6 && length != 8))
        return fail(nullptr, "invalid stats output", 1);
    for (int i = 0; i < length; ++i)
        counts[i] = context->counts[i].load(std::memory_order_relaxed);
    /* guard fall-backs are decided on the device and counted in pinned host memory */
    if (context->guard_hits)
        counts[5] += *static_cast<volatile unsigned long long *>(context->guard_hits);
    return 0;
}

extern "C" int camblas_cuda_reset_stats(camblas_cuda_context *context)
{
    if (!context)
        return fail(nullptr, "missing context", 1);
    for (auto &count : context->counts)
        count.store(0, std::memory_order_relaxed);
    if (context->guard_hits)
        *static_cast<volatile unsigned long long *>(context->guard_hits) = 0;
    return 0;
}

extern "C" int camblas_cuda_kernel_launches(const camblas_cuda_context *context, uint64_t *count)
{
    if (!context || !count)
        return fail(nullptr, "invalid launch count output", 1);
    *count = context->kernel_launches.load(std::memory_order_relaxed);
    return 0;
}

extern "C" int camblas_cuda_device_status(camblas_cuda_context *context, unsigned *status)
{
    return guarded(context, [&] {
        if (!status)
            return fail(context, "missing status output", 1);
        cudaError_t error = cudaMemcpyAsync(status, context->status, sizeof(unsigned),
                                            cudaMemcpyDeviceToHost, context->stream);
        if (error == cudaSuccess)
            error = cudaMemsetAsync(context->status, 0, sizeof(unsigned), context->stream);
        if (error == cudaSuccess)
            error = cudaStreamSynchronize(context->stream);

        return error == cudaSuccess ? 0 : fail(context, "device status read", error);
    });
}

/* ---- BF16 GEMM ---- */

extern "C" int camblas_cuda_bgemm(camblas_cuda_context *context, char trans_a, char trans_b, int m,
                                  int n, int k, float alpha, const void *a, int lda, const void *b,
                                  int ldb, float beta, void *c, int ldc)
{
    return guarded(context, [&] {
        bool na = trans_a == 'N' || trans_a == 'n', ta = trans_a == 'T' || trans_a == 't';
        bool nb = trans_b == 'N' || trans_b == 'n', tb = trans_b == 'T' || trans_b == 't';
        if ((!na && !ta) || (!nb && !tb) || m < 0 || n < 0 || k < 0 || lda < 1 || ldb < 1 ||
            ldc < 1)
            return fail(context, "invalid BF16 GEMM arguments", 1);
        if (m == 0 || n == 0)
            return 0;
        if (!c || lda < std::max(1, na ? m : k) || ldb < std::max(1, nb ? k : n) || ldc < m)
            return fail(context, "invalid BF16 pointer or leading dimension", 1);
        auto *out = static_cast<__nv_bfloat16 *>(c);
        if (alpha == 0 || k == 0) {
            if (beta == 1)
                return 0;
            generic::scale_window<<<unsigned((size_t(m) * n + 255) / 256), 256, 0,
                                    context->stream>>>(m, n, beta, out, ldc);
            return launched(context, "scale BF16 output");
        }
        if (!a || !b || a == c || b == c)
            return fail(context, "missing or aliased BF16 GEMM operand", 1);
        host::Product x{};
        x.ta = ta, x.tb = tb, x.m = m, x.n = n, x.k = k;
        x.alpha = alpha, x.beta = beta;
        x.a = static_cast<const __nv_bfloat16 *>(a), x.lda = lda;
        x.b = static_cast<const __nv_bfloat16 *>(b), x.ldb = ldb;
        x.c = out, x.ldc = ldc;
        x.addend = out, x.ld_add = ldc;
        x.cut0 = x.cut1 = m;
        if (context->algorithm == CAMBLAS_CUDA_STRASSEN && context->options.bf16_strassen &&
            strassen::eligible(context, x))
            return strassen::run(context, x);
        return host::run_product(context, x);
    });
}

extern "C" int camblas_cuda_linear_bf16(camblas_cuda_context *context, int rows, int inner,
                                        int outputs, const void *x, int ldx, const void *w, int ldw,
                                        const void *bias, const void *residual, int ldr, void *out,
                                        int ldo)
{
    return guarded(context, [&] {
        if (rows < 0 || inner < 1 || outputs < 0 || ldx < inner || ldw < inner || ldo < outputs ||
            (residual && ldr < outputs))
            return fail(context, "invalid BF16 linear dimensions", 1);
        if (rows == 0 || outputs == 0)
            return 0;
        if (!x || !w || !out || out == x || out == w)
            return fail(context, "missing or aliased BF16 linear operand", 1);
        host::Product p{};
        p.ta = true, p.tb = false, p.m = outputs, p.n = rows, p.k = inner;
        p.alpha = 1.f, p.beta = residual ? 1.f : 0.f;
        p.a = static_cast<const __nv_bfloat16 *>(w), p.lda = ldw;
        p.b = static_cast<const __nv_bfloat16 *>(x), p.ldb = ldx;
        p.c = static_cast<__nv_bfloat16 *>(out), p.ldc = ldo;
        p.addend = static_cast<const __nv_bfloat16 *>(residual), p.ld_add = ldr;
        p.bias = static_cast<const __nv_bfloat16 *>(bias);
        p.cut0 = p.cut1 = outputs;
        return host::run_product(context, p);
    });
}

extern "C" int camblas_cuda_qkv_linear_bf16(camblas_cuda_context *context, int rows, int inner,
                                            int q_out, int k_out, int v_out, const void *x, int ldx,
                                            const void *w, int ldw, void *q, int ldq, void *k,
                                            int ldk, void *v, int ldv)
{
    return guarded(context, [&] {
        if (rows < 0 || inner < 1 || q_out < 1 || k_out < 1 || v_out < 1 || ldx < inner ||
            ldw < inner || ldq < q_out || ldk < k_out || ldv < v_out ||
            long(q_out) + k_out + v_out > INT_MAX)
            return fail(context, "invalid packed projection dimensions", 1);
        if (rows == 0)
            return 0;
        if (!x || !w || !q || !k || !v || q == k || q == v || k == v)
            return fail(context, "missing or aliased packed projection operand", 1);
        host::Product p{};
        p.ta = true, p.tb = false, p.m = q_out + k_out + v_out, p.n = rows, p.k = inner;
        p.alpha = 1.f, p.beta = 0.f;
        p.a = static_cast<const __nv_bfloat16 *>(w), p.lda = ldw;
        p.b = static_cast<const __nv_bfloat16 *>(x), p.ldb = ldx;
        p.c = static_cast<__nv_bfloat16 *>(q), p.ldc = ldq;
        p.c1 = static_cast<__nv_bfloat16 *>(k), p.ldc1 = ldk;
        p.c2 = static_cast<__nv_bfloat16 *>(v), p.ldc2 = ldv;
        p.addend = nullptr, p.ld_add = 0;
        p.cut0 = q_out, p.cut1 = q_out + k_out;
        return host::run_product(context, p);
    });
}

extern "C" int camblas_cuda_gate_up_swiglu_bf16(camblas_cuda_context *context, int rows, int inner,
                                                int intermediate, const void *x, int ldx,
                                                const void *w, int ldw, void *out, int ldo)
{
    return guarded(context, [&] {
        if (rows < 0 || inner < 1 || intermediate < 0 || ldx < inner || ldw < inner ||
            ldo < intermediate || intermediate > INT_MAX / 2)
            return fail(context, "invalid gate_up SwiGLU dimensions", 1);
        if (rows == 0 || intermediate == 0)
            return 0;
        if (!x || !w || !out || out == x || out == w)
            return fail(context, "missing or aliased gate_up SwiGLU operand", 1);
        if (intermediate % 128 != 0)
            return fail(context, "gate_up SwiGLU needs an intermediate width that is a multiple of 128",
                        1);
        if (ldx % 8 != 0 || ldw % 8 != 0 || ldo % 8 != 0 || !host::aligned16(x) ||
            !host::aligned16(w) || !host::aligned16(out))
            return fail(context, "gate_up SwiGLU needs 16-byte aligned rows (multiples of 8 elements)",
                        1);
        return host::run_gate_up_swiglu(context, rows, inner, intermediate,
                                        static_cast<const __nv_bfloat16 *>(x), ldx,
                                        static_cast<const __nv_bfloat16 *>(w), ldw,
                                        static_cast<__nv_bfloat16 *>(out), ldo);
    });
}

extern "C" int camblas_cuda_gate_up_swiglu_fp8(camblas_cuda_context *context, int rows, int inner,
                                               int intermediate, const void *x, int ldx,
                                               const void *w, int ldw, void *q, float *scale)
{
    return guarded(context, [&] {
        if (rows < 0 || inner < 1 || intermediate < 0 || ldx < inner || ldw < inner ||
            intermediate > INT_MAX / 2)
            return fail(context, "invalid gate_up SwiGLU dimensions", 1);
        if (rows == 0 || intermediate == 0)
            return 0;
        if (!x || !w || !q || !scale || q == x || q == w)
            return fail(context, "missing or aliased gate_up SwiGLU operand", 1);
        if (intermediate % 128 != 0)
            return fail(context, "gate_up SwiGLU needs an intermediate width that is a multiple of 128",
                        1);
        if (ldx % 8 != 0 || ldw % 8 != 0 || !host::aligned16(x) || !host::aligned16(w) ||
            !host::aligned16(q) || (uintptr_t(scale) & 3))
            return fail(context, "gate_up SwiGLU needs 16-byte aligned rows (multiples of 8 elements)",
                        1);
        return host::run_gate_up_swiglu(context, rows, inner, intermediate,
                                        static_cast<const __nv_bfloat16 *>(x), ldx,
                                        static_cast<const __nv_bfloat16 *>(w), ldw, nullptr, 0,
                                        static_cast<uint8_t *>(q), scale);
    });
}

/* ---- RMS normalisation ---- */

namespace
{
constexpr int kStagedLimitBytes = 160 * 1024; /* widest row rows_staged keeps in shared memory */

int prepare_rms_kernels()
{
    return int(cudaFuncSetAttribute(rms::rows_staged<float, true>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    kStagedLimitBytes)) |
           int(cudaFuncSetAttribute(rms::rows_staged<__nv_bfloat16, true>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    kStagedLimitBytes));
}

template <typename T, typename W, bool Add, int Sweeps>
void launch_in_registers(camblas_cuda_context *context, int rows, int width, rms::RowPitch pitch,
                         float epsilon, const T *in, const T *res, const W *gamma, T *sum, T *out,
                         bool round_before_weight, bool descending)
{
    rms::rows_in_registers<T, W, Add, Sweeps><<<rows, rms::kRowThreads, 0, context->stream>>>(
        width, pitch, epsilon, in, res, gamma, sum, out, round_before_weight, descending);
}

/* Single-row order for `rows` rows, one CTA each. Rows of up to 16384 columns
 * with vector-aligned pointers stay in registers between the two passes. */
template <typename T, typename W, bool Add>
int launch_rms_rows(camblas_cuda_context *context, int rows, int width, float epsilon,
                    const void *input, const void *residual, const void *weight, void *added,
                    void *output, bool round_before_weight, bool descending, bool in_place = false,
                    const rms::RowPitch *pitches = nullptr)
{
    constexpr uintptr_t mask = sizeof(T) * 4 - 1, weight_mask = sizeof(W) * 4 - 1;
    const rms::RowPitch pitch = pitches ? *pitches : rms::RowPitch{width, width, width, width};
    const bool pitches_ok = rows == 1 || (pitch.input % 4 == 0 && pitch.output % 4 == 0 &&
                                          (!Add || (pitch.residual % 4 == 0 && pitch.added % 4 == 0)));
    const bool vector = width % 4 == 0 && pitches_ok && !(uintptr_t(input) & mask) &&
                        !(uintptr_t(output) & mask) && !(uintptr_t(weight) & weight_mask) &&
                        (!Add || (!(uintptr_t(residual) & mask) && !(uintptr_t(added) & mask)));
    auto *in = static_cast<const T *>(input);
    auto *res = static_cast<const T *>(residual);
    auto *gamma = static_cast<const W *>(weight);
    auto *sum = static_cast<T *>(added);
    auto *out = static_cast<T *>(output);
    /* the register kernel declares its pointers restrict: not for in-place calls */
    const int sweeps = in_place ? 9 : (width + rms::kRowSpan - 1) / rms::kRowSpan;
    if (vector && sweeps <= 1)
        launch_in_registers<T, W, Add, 1>(context, rows, width, pitch, epsilon, in, res, gamma, sum, out,
                                          round_before_weight, descending);
    else if (vector && sweeps <= 2)
        launch_in_registers<T, W, Add, 2>(context, rows, width, pitch, epsilon, in, res, gamma, sum, out,
                                          round_before_weight, descending);
    else if (vector && sweeps <= 4)
        launch_in_registers<T, W, Add, 4>(context, rows, width, pitch, epsilon, in, res, gamma, sum, out,
                                          round_before_weight, descending);
    else if (vector && sweeps <= 8)
        launch_in_registers<T, W, Add, 8>(context, rows, width, pitch, epsilon, in, res, gamma, sum, out,
                                          round_before_weight, descending);
    else if (vector)
        rms::rows_two_sweeps<T, W, Add, true><<<rows, rms::kRowThreads, 0, context->stream>>>(
            width, pitch, epsilon, in, res, gamma, sum, out, round_before_weight, descending);
    else
        rms::rows_two_sweeps<T, W, Add, false><<<rows, rms::kRowThreads, 0, context->stream>>>(
            width, pitch, epsilon, in, res, gamma, sum, out, round_before_weight, descending);
    return launched(context, Add ? "residual RMS normalisation" : "RMS normalisation");
}

/* Multi-row order for rows of any width. */
template <typename T>
int launch_rms_any(camblas_cuda_context *context, int rows, int width, float epsilon,
                   const void *input, const void *weight, void *output)
{
    constexpr int lanes = rms::Storage<T>::kLanes;
    const size_t row_bytes = size_t(width) * sizeof(T);
    const bool staged = width % lanes == 0 && host::aligned16(input) && host::aligned16(weight) &&
                        host::aligned16(output) && row_bytes <= size_t(kStagedLimitBytes);
    const int grid = std::min(rows, context->sm_count * 8);
    auto *in = static_cast<const T *>(input);
    auto *gamma = static_cast<const T *>(weight);
    auto *out = static_cast<T *>(output);
    if (staged)
        rms::rows_staged<T, true><<<grid, rms::kStagedThreads, row_bytes, context->stream>>>(
            rows, width, epsilon, in, gamma, out);
    else
        rms::rows_staged<T, false><<<grid, rms::kStagedThreads, 0, context->stream>>>(
            rows, width, epsilon, in, gamma, out);
    return launched(context, "RMS normalisation");
}

bool decode_width(int width)
{
    return width >= 2048 && width <= 65536 && width % 4 == 0;
}

/* Launch geometry of the elementwise kernels: how many leading 16-byte vectors
 * the kernel may take (none unless every pointer is 16-byte aligned and, for
 * row-structured operands, rows are whole vectors) and a grid that gives every
 * SM a few CTAs without exceeding the work. */
struct Elementwise {
    size_t vectors;
    unsigned blocks;
};

Elementwise elementwise_plan(const camblas_cuda_context *context, uint64_t count, int lanes,
                             bool aligned, int width = 0)
{
    Elementwise plan{};
    if (aligned && (width == 0 || width % lanes == 0))
        plan.vectors = size_t(count / uint64_t(lanes));
    const uint64_t items = std::max<uint64_t>(plan.vectors, count - plan.vectors * lanes);
    plan.blocks = unsigned(std::min<uint64_t>((items + 255) / 256, uint64_t(context->sm_count) * 16));
    if (plan.blocks == 0)
        plan.blocks = 1;
    return plan;
}
} // namespace

extern "C" int camblas_cuda_rms_norm(camblas_cuda_context *context, int dtype, int rows, int width,
                                     float epsilon, const void *input, const void *weight,
                                     void *output)
{
    return guarded(context, [&] {
        if ((dtype != 0 && dtype != 2) || rows < 0 || width < 0 || !std::isfinite(epsilon) ||
            epsilon < 0)
            return fail(context, "invalid RMS normalisation dimensions, dtype or epsilon", 1);
        if (!rows || !width)
            return 0;
        if (!input || !weight || !output || output == weight)
            return fail(context, "invalid RMS normalisation operands", 1);
        /* a single long row takes the single-row order, as in the reference
         * (inference_fusion.cuh:194-207); the output may be the input there */
        if (rows == 1 && decode_width(width)) {
            const bool in_place = output == input;
            if (dtype == 0)
                return launch_rms_rows<float, float, false>(context, 1, width, epsilon, input,
                                                            nullptr, weight, nullptr, output, true,
                                                            false, in_place);
            return launch_rms_rows<__nv_bfloat16, __nv_bfloat16, false>(
                context, 1, width, epsilon, input, nullptr, weight, nullptr, output, true, false,
                in_place);
        }
        if (dtype == 0)
            return launch_rms_any<float>(context, rows, width, epsilon, input, weight, output);
        return launch_rms_any<__nv_bfloat16>(context, rows, width, epsilon, input, weight, output);
    });
}

extern "C" int camblas_cuda_rms_norm_decode(camblas_cuda_context *context, int dtype,
                                            int weight_dtype, int width, float epsilon,
                                            int round_before_weight, int descending,
                                            const void *input, const void *weight, void *output)
{
    return guarded(context, [&] {
        const bool types_ok = (dtype == 0 || dtype == 2) && (weight_dtype == 0 || weight_dtype == 2) &&
                              !(dtype == 0 && weight_dtype != 0);
        const bool flags_ok = (round_before_weight == 0 || round_before_weight == 1) &&
                              (descending == 0 || descending == 1);
        const bool values_ok = decode_width(width) && std::isfinite(epsilon) && epsilon >= 0;
        const uintptr_t element = dtype == 0 ? 4 : 2, weight_element = weight_dtype == 0 ? 4 : 2;
        const bool operands_ok = input && weight && output && output != input && output != weight &&
                                 uintptr_t(input) % element == 0 &&
                                 uintptr_t(output) % element == 0 &&
                                 uintptr_t(weight) % weight_element == 0;
        if (!types_ok || !flags_ok || !values_ok || !operands_ok)
            return fail(context, "invalid decode RMS arguments", 1);
        if (dtype == 0)
            return launch_rms_rows<float, float, false>(context, 1, width, epsilon, input, nullptr,
                                                        weight, nullptr, output,
                                                        round_before_weight, descending);
        if (weight_dtype == 0)
            return launch_rms_rows<__nv_bfloat16, float, false>(context, 1, width, epsilon, input,
                                                                nullptr, weight, nullptr, output,
                                                                round_before_weight, descending);
        return launch_rms_rows<__nv_bfloat16, __nv_bfloat16, false>(
            context, 1, width, epsilon, input, nullptr, weight, nullptr, output,
            round_before_weight, descending);
    });
}

namespace
{
int add_rms(camblas_cuda_context *context, int dtype, int rows, int width, float epsilon,
            const void *input, const void *residual, const void *weight, void *added, void *output,
            const rms::RowPitch *pitches = nullptr)
{
    if (dtype == 0)
        return launch_rms_rows<float, float, true>(context, rows, width, epsilon, input, residual,
                                                   weight, added, output, true, false, false,
                                                   pitches);
    return launch_rms_rows<__nv_bfloat16, __nv_bfloat16, true>(
        context, rows, width, epsilon, input, residual, weight, added, output, true, false, false,
        pitches);
}

/* the five buffers of the residual form must all be present and pairwise distinct
 * where one is written (reference backend.cu:1404-1408) */
bool add_rms_operands_bad(const void *input, const void *residual, const void *weight, void *added,
                          void *output)
{
    const void *read[3] = {input, residual, weight};
    if (!added || !output || added == output)
        return true;
    for (const void *pointer : read)
        if (!pointer || pointer == added || pointer == output)
            return true;
    return false;
}
} // namespace

extern "C" int camblas_cuda_add_rms_norm(camblas_cuda_context *context, int dtype, int width,
                                         float epsilon, const void *input, const void *residual,
                                         const void *weight, void *added, void *output)
{
    return guarded(context, [&] {
        if ((dtype != 0 && dtype != 2) || !decode_width(width) || !std::isfinite(epsilon) ||
            epsilon < 0 || add_rms_operands_bad(input, residual, weight, added, output))
            return fail(context, "invalid residual RMS arguments", 1);
        return add_rms(context, dtype, 1, width, epsilon, input, residual, weight, added, output);
    });
}

extern "C" int camblas_cuda_add_rms_norm_rows(camblas_cuda_context *context, int dtype, int rows,
                                              int width, float epsilon, const void *input,
                                              const void *residual, const void *weight,
                                              void *added, void *output)
{
    return guarded(context, [&] {
        if ((dtype != 0 && dtype != 2) || rows < 0 || width < 4 || width > 65536 || width % 4 ||
            !std::isfinite(epsilon) || epsilon < 0)
            return fail(context, "invalid residual RMS rows arguments", 1);
        if (rows == 0)
            return 0;
        if (add_rms_operands_bad(input, residual, weight, added, output))
            return fail(context, "invalid residual RMS rows operands", 1);
        return add_rms(context, dtype, rows, width, epsilon, input, residual, weight, added,
                       output);
    });
}

extern "C" int camblas_cuda_add_rms_norm_strided(camblas_cuda_context *context, int dtype, int rows,
                                                 int width, float epsilon, const void *input,
                                                 long long ld_input, const void *residual,
                                                 long long ld_residual, const void *weight,
                                                 void *added, long long ld_added, void *output,
                                                 long long ld_output)
{
    return guarded(context, [&] {
        if ((dtype != 0 && dtype != 2) || rows < 0 || width < 4 || width > 65536 || width % 4 ||
            !std::isfinite(epsilon) || epsilon < 0 || ld_input < width || ld_residual < width ||
            ld_added < width || ld_output < width)
            return fail(context, "invalid residual RMS rows arguments", 1);
        if (rows == 0)
            return 0;
        if (add_rms_operands_bad(input, residual, weight, added, output))
            return fail(context, "invalid residual RMS rows operands", 1);
        const rms::RowPitch pitch{ld_input, ld_residual, ld_added, ld_output};
        return add_rms(context, dtype, rows, width, epsilon, input, residual, weight, added, output,
                       &pitch);
    });
}

extern "C" int camblas_cuda_bfloat16_square(camblas_cuda_context *context, uint64_t count,
                                            const void *input, float *output)
{
    return guarded(context, [&] {
        if (!count)
            return 0;
        if (!input || !output || count > SIZE_MAX / sizeof(float))
            return fail(context, "invalid BF16 square operands", 1);
        const Elementwise plan = elementwise_plan(
            context, count, 8, host::aligned16(input) && host::aligned16(output));
        rms::square_kernel<<<plan.blocks, 256, 0, context->stream>>>(
            size_t(count), plan.vectors, static_cast<const __nv_bfloat16 *>(input), output);
        return launched(context, "BF16 squares");
    });
}

extern "C" int camblas_cuda_rms_scale(camblas_cuda_context *context, int dtype, uint64_t count,
                                      int width, float epsilon, const void *input,
                                      const void *weight, const float *means, void *output)
{
    return guarded(context, [&] {
        if ((dtype != 0 && dtype != 2) || width < 0 || !std::isfinite(epsilon) || epsilon < 0)
            return fail(context, "invalid RMS scale dimensions, dtype or epsilon", 1);
        if (!count)
            return 0;
        if (!width || count % width || count > SIZE_MAX / sizeof(float) || !input || !weight ||
            !means || !output || output == weight)
            return fail(context, "invalid RMS scale operands", 1);
        const bool aligned =
            host::aligned16(input) && host::aligned16(weight) && host::aligned16(output);
        const Elementwise plan =
            elementwise_plan(context, count, dtype == 0 ? 4 : 8, aligned, width);
        if (dtype == 0)
            rms::scale_kernel<float><<<plan.blocks, 256, 0, context->stream>>>(
                size_t(count), plan.vectors, width, epsilon, static_cast<const float *>(input),
                static_cast<const float *>(weight), means, static_cast<float *>(output));
        else
            rms::scale_kernel<__nv_bfloat16><<<plan.blocks, 256, 0, context->stream>>>(
                size_t(count), plan.vectors, width, epsilon,
                static_cast<const __nv_bfloat16 *>(input),
                static_cast<const __nv_bfloat16 *>(weight), means,
                static_cast<__nv_bfloat16 *>(output));
        return launched(context, "RMS scaling");
    });
}

extern "C" int camblas_cuda_silu_multiply(camblas_cuda_context *context, int dtype, uint64_t count,
                                          const void *gate, const void *up, void *output)
{
    return guarded(context, [&] {
        if (dtype != 0 && dtype != 2)
            return fail(context, "invalid SiLU multiply dtype", 1);
        if (!count)
            return 0;
        if (!gate || !up || !output)
            return fail(context, "missing SiLU multiply operand", 1);
        const bool aligned = host::aligned16(gate) && host::aligned16(up) && host::aligned16(output);
        const Elementwise plan = elementwise_plan(context, count, dtype == 0 ? 4 : 8, aligned);
        if (dtype == 0)
            rms::silu_multiply_kernel<float><<<plan.blocks, 256, 0, context->stream>>>(
                size_t(count), plan.vectors, static_cast<const float *>(gate),
                static_cast<const float *>(up), static_cast<float *>(output));
        else
            rms::silu_multiply_kernel<__nv_bfloat16><<<plan.blocks, 256, 0, context->stream>>>(
                size_t(count), plan.vectors, static_cast<const __nv_bfloat16 *>(gate),
                static_cast<const __nv_bfloat16 *>(up), static_cast<__nv_bfloat16 *>(output));
        return launched(context, "SiLU multiply");
    });
}

extern "C" int camblas_cuda_swiglu(camblas_cuda_context *context, int dtype, uint64_t count,
                                   int width, float limit, const void *gate, const void *up,
                                   const float *routing, void *output)
{
    return guarded(context, [&] {
        if ((dtype != 0 && dtype != 2) || width < 1 || !(limit >= 0) || !std::isfinite(limit) ||
            count % uint64_t(width))
            return fail(context, "invalid SwiGLU dimensions, dtype or limit", 1);
        if (!count)
            return 0;
        if (!gate || !up || !output || static_cast<const void *>(routing) == output)
            return fail(context, "invalid SwiGLU operands", 1);
        const bool aligned = host::aligned16(gate) && host::aligned16(up) && host::aligned16(output);
        const Elementwise plan =
            elementwise_plan(context, count, dtype == 0 ? 4 : 8, aligned, routing ? width : 0);
        if (dtype == 0)
            rms::swiglu_kernel<float><<<plan.blocks, 256, 0, context->stream>>>(
                size_t(count), plan.vectors, width, limit, static_cast<const float *>(gate),
                static_cast<const float *>(up), routing, static_cast<float *>(output));
        else
            rms::swiglu_kernel<__nv_bfloat16><<<plan.blocks, 256, 0, context->stream>>>(
                size_t(count), plan.vectors, width, limit, static_cast<const __nv_bfloat16 *>(gate),
                static_cast<const __nv_bfloat16 *>(up), routing,
                static_cast<__nv_bfloat16 *>(output));
        return launched(context, "SwiGLU");
    });
}

/* ---- exported for link compatibility only ---- */

namespace
{
/* FP32 / FP64 GEMM with the argument rules of the reference's gemm<T>
 * (backend.cu:786-806). */
template <typename T>
int simt_gemm(camblas_cuda_context *context, char trans_a, char trans_b, int m, int n, int k, T alpha,
              const T *a, int lda, const T *b, int ldb, T beta, T *c, int ldc)
{
    return guarded(context, [&] {
        const bool na = trans_a == 'N' || trans_a == 'n', ta = trans_a == 'T' || trans_a == 't';
        const bool nb = trans_b == 'N' || trans_b == 'n', tb = trans_b == 'T' || trans_b == 't';
        if ((!na && !ta) || (!nb && !tb) || m < 0 || n < 0 || k < 0 || lda < 1 || ldb < 1 || ldc < 1)
            return fail(context, "invalid GEMM arguments", 1);
        if (m == 0 || n == 0)
            return 0;
        if (!c || lda < std::max(1, na ? m : k) || ldb < std::max(1, nb ? k : n) || ldc < m)
            return fail(context, "invalid device pointer or leading dimension", 1);
        if (alpha == T(0) || k == 0) {
            if (beta == T(1))
                return 0;
            simt::scale_window<T><<<unsigned((size_t(m) * n + 255) / 256), 256, 0, context->stream>>>(
                m, n, beta, c, ldc);
            return launched(context, "scale output");
        }
        if (!a || !b || a == c || b == c)
            return fail(context, "missing or aliased GEMM operand", 1);
        simt::Task<T> task{};
        task.m = m, task.n = n, task.k = k;
        task.ta = ta, task.tb = tb;
        task.lda = lda, task.ldb = ldb, task.ldc = ldc;
        task.alpha = alpha, task.beta = beta;
        task.a = a, task.b = b, task.c = c;
        dim3 grid((m + simt::kTileM - 1) / simt::kTileM, (n + simt::kTileN - 1) / simt::kTileN);
        if (grid.y > 65535)
            return fail(context, "GEMM column count", 1);
        context->counts[0]++;
        simt::gemm_simt<T><<<grid, 256, 0, context->stream>>>(task);
        return launched(context, "classical GEMM");
    });
}
} // namespace

extern "C" int camblas_cuda_sgemm(camblas_cuda_context *context, char trans_a, char trans_b, int m,
                                  int n, int k, float alpha, const float *a, int lda, const float *b,
                                  int ldb, float beta, float *c, int ldc)
{
    return simt_gemm<float>(context, trans_a, trans_b, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc);
}
extern "C" int camblas_cuda_dgemm(camblas_cuda_context *context, char trans_a, char trans_b, int m,
                                  int n, int k, double alpha, const double *a, int lda,
                                  const double *b, int ldb, double beta, double *c, int ldc)
{
    return simt_gemm<double>(context, trans_a, trans_b, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc);
}
namespace
{
/* ---- FP32 / FP64 layer compositions on the CUDA-core GEMM -----------------------
 * Row-major operands; a row-major product X . W is the column-major product
 * W . X of the same buffers, which is how the GEMM is called. */

/* out[rows][columns] = act(x[rows][inner] . w[inner][columns] + bias[columns]) */
template <typename T>
int affine_layer(camblas_cuda_context *context, int rows, int inner, int columns, const T *x, const T *w,
                 const T *bias, bool relu, T *out)
{
    return guarded(context, [&] {
        if (rows < 0 || inner < 0 || columns < 0)
            return fail(context, "invalid affine dimensions", 1);
        if (rows == 0 || columns == 0)
            return 0;
        if (!out || !bias || (inner > 0 && (!x || !w)))
            return fail(context, "missing affine operand", 1);
        context->counts[3]++;
        int status = simt_gemm<T>(context, 'N', 'N', columns, rows, inner, T(1), w, std::max(1, columns), x,
                                  std::max(1, inner), T(0), out, columns);
        if (status != 0)
            return status;
        const long long count = 1ll * rows * columns;
        dense::add_bias<T><<<unsigned(std::min<long long>((count + 255) / 256, 65535)), 256, 0,
                             context->stream>>>(out, bias, count, columns, relu ? 1 : 0);
        return launched(context, "bias and activation");
    });
}

/* out[queries][values] = softmax(scale q . k^T) . v; the scores live in the
 * context's scratch arena between the two products. */
template <typename T>
int attention_layer(camblas_cuda_context *context, int queries, int keys, int depth, int values, T scale,
                    const T *q, const T *k, const T *v, T *out)
{
    return guarded(context, [&] {
        if (queries < 0 || keys < 0 || depth < 0 || values < 0)
            return fail(context, "invalid attention dimensions", 1);
        if (queries == 0 || values == 0)
            return 0;
        if (!out || (depth > 0 && !q) || (keys > 0 && depth > 0 && !k) || (keys > 0 && !v))
            return fail(context, "missing attention operand", 1);
        if (keys > 0 && size_t(queries) > SIZE_MAX / sizeof(T) / size_t(keys))
            return fail(context, "attention scratch size overflow", 2);
        context->counts[6]++;
        int status = host::reserve_scratch(context, std::max<size_t>(16, size_t(queries) * keys * sizeof(T)));
        if (status != 0)
            return status;
        T *scores = static_cast<T *>(context->scratch);
        status = simt_gemm<T>(context, 'T', 'N', keys, queries, depth, T(1), k, std::max(1, depth), q,
                              std::max(1, depth), T(0), scores, std::max(1, keys));
        if (status != 0)
            return status;
        if (keys > 0) {
            dense::softmax_scaled<T><<<unsigned(queries), 256, 0, context->stream>>>(scores, keys, scale);
            status = launched(context, "attention softmax");
            if (status != 0)
                return status;
        }
        return simt_gemm<T>(context, 'N', 'N', values, queries, keys, T(1), v, std::max(1, values), scores,
                            std::max(1, keys), T(0), out, std::max(1, values));
    });
}

/* First derivatives of out = relu(x . w1 + b1) . w2 + b2 with respect to
 * whatever is requested (non-NULL): dw2 = h^T . g, db2 = column sums of g,
 * dh = (g . w2^T) where h > 0, db1 = column sums of dh, dw1 = x^T . dh,
 * dx = dh . w1^T. */
template <typename T>
int perceptron_backward(camblas_cuda_context *context, int rows, int inputs, int hidden, int outputs,
                        const T *x, const T *w1, const T *w2, const T *h, const T *g, T *dh, T *dx, T *dw1,
                        T *db1, T *dw2, T *db2)
{
    return guarded(context, [&] {
        if (rows < 0 || inputs < 0 || hidden < 0 || outputs < 0)
            return fail(context, "invalid backward dimensions", 1);
        const bool first_layer = dx || dw1 || db1;
        if ((rows > 0 && outputs > 0 && !g) || (rows > 0 && hidden > 0 && first_layer && (!dh || !h)))
            return fail(context, "missing backward operand", 1);
        context->counts[7]++;
        int status = 0;
        if (dw2) {
            status = simt_gemm<T>(context, 'N', 'T', outputs, hidden, rows, T(1), g, std::max(1, outputs), h,
                                  std::max(1, hidden), T(0), dw2, std::max(1, outputs));
            if (status != 0)
                return status;
        }
        if (db2 && outputs > 0) {
            dense::column_sums<T, false><<<unsigned((outputs + 127) / 128), 128, 0, context->stream>>>(
                const_cast<T *>(g), nullptr, rows, outputs, db2);
            status = launched(context, "output bias gradient");
            if (status != 0)
                return status;
        }
        if (!first_layer)
            return 0;
        status = simt_gemm<T>(context, 'T', 'N', hidden, rows, outputs, T(1), w2, std::max(1, outputs), g,
                              std::max(1, outputs), T(0), dh, std::max(1, hidden));
        if (status != 0)
            return status;
        if (hidden > 0) {
            dense::column_sums<T, true><<<unsigned((hidden + 127) / 128), 128, 0, context->stream>>>(
                dh, h, rows, hidden, db1);
            status = launched(context, "hidden gradient gate");
            if (status != 0)
                return status;
        }
        if (dw1) {
            status = simt_gemm<T>(context, 'N', 'T', hidden, inputs, rows, T(1), dh, std::max(1, hidden), x,
                                  std::max(1, inputs), T(0), dw1, std::max(1, hidden));
            if (status != 0)
                return status;
        }
        if (dx)
            status = simt_gemm<T>(context, 'T', 'N', inputs, rows, hidden, T(1), w1, std::max(1, hidden), dh,
                                  std::max(1, hidden), T(0), dx, std::max(1, inputs));
        return status;
    });
}
} // namespace

/* Replaces camblas_cuda_affine (camblas_cuda.h:73-75; backend.cu:870-911, 1086-1101). */
extern "C" int camblas_cuda_affine(camblas_cuda_context *context, int dtype, int rows, int inner,
                                   int columns, const void *x, const void *weight, const void *bias,
                                   int relu, void *output)
{
    if (dtype == 0)
        return affine_layer<float>(context, rows, inner, columns, static_cast<const float *>(x),
                                   static_cast<const float *>(weight), static_cast<const float *>(bias),
                                   relu != 0, static_cast<float *>(output));
    if (dtype == 1)
        return affine_layer<double>(context, rows, inner, columns, static_cast<const double *>(x),
                                    static_cast<const double *>(weight), static_cast<const double *>(bias),
                                    relu != 0, static_cast<double *>(output));
    return fail(context, "unsupported affine dtype", 1);
}

/* Replaces camblas_cuda_mlp (camblas_cuda.h:76-78; backend.cu:1103-1117): two affine
 * layers, ReLU after the first, whose output the caller keeps for the backward pass. */
extern "C" int camblas_cuda_mlp(camblas_cuda_context *context, int dtype, int rows, int inputs,
                                int hidden, int outputs, const void *x, const void *w1, const void *b1,
                                const void *w2, const void *b2, void *hidden_output, void *output)
{
    int status = camblas_cuda_affine(context, dtype, rows, inputs, hidden, x, w1, b1, 1, hidden_output);
    if (status != 0)
        return status;
    return camblas_cuda_affine(context, dtype, rows, hidden, outputs, hidden_output, w2, b2, 0, output);
}

/* Replaces camblas_cuda_attention (camblas_cuda.h:80-85; backend.cu:1495-1510). */
extern "C" int camblas_cuda_attention(camblas_cuda_context *context, int dtype, int queries, int keys,
                                      int depth, int values, double scale, const void *q,
                                      const void *k, const void *v, void *output)
{
    if (dtype == 0)
        return attention_layer<float>(context, queries, keys, depth, values, float(scale),
                                      static_cast<const float *>(q), static_cast<const float *>(k),
                                      static_cast<const float *>(v), static_cast<float *>(output));
    if (dtype == 1)
        return attention_layer<double>(context, queries, keys, depth, values, scale,
                                       static_cast<const double *>(q), static_cast<const double *>(k),
                                       static_cast<const double *>(v), static_cast<double *>(output));
    return fail(context, "unsupported attention dtype", 1);
}

/* Replaces camblas_cuda_mlp_backward (camblas_cuda.h:87-99; backend.cu:1512-1535). */
extern "C" int camblas_cuda_mlp_backward(camblas_cuda_context *context, int dtype, int rows, int inputs,
                                         int hidden, int outputs, const void *x, const void *w1,
                                         const void *w2, const void *h, const void *grad, void *dh,
                                         void *dx, void *dw1, void *db1, void *dw2, void *db2)
{
    if (dtype == 0)
        return perceptron_backward<float>(
            context, rows, inputs, hidden, outputs, static_cast<const float *>(x),
            static_cast<const float *>(w1), static_cast<const float *>(w2), static_cast<const float *>(h),
            static_cast<const float *>(grad), static_cast<float *>(dh), static_cast<float *>(dx),
            static_cast<float *>(dw1), static_cast<float *>(db1), static_cast<float *>(dw2),
            static_cast<float *>(db2));
    if (dtype == 1)
        return perceptron_backward<double>(
            context, rows, inputs, hidden, outputs, static_cast<const double *>(x),
            static_cast<const double *>(w1), static_cast<const double *>(w2),
            static_cast<const double *>(h), static_cast<const double *>(grad), static_cast<double *>(dh),
            static_cast<double *>(dx), static_cast<double *>(dw1), static_cast<double *>(db1),
            static_cast<double *>(dw2), static_cast<double *>(db2));
    return fail(context, "unsupported backward dtype", 1);
}
