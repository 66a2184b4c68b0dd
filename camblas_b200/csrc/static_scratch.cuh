/*
 * camblas_cuda_linear_bf16_static: a few-token BF16 linear layer that never
 * allocates.
 *
 * Who needs it. The ordinary entry points grow a per-context scratch arena
 * with cudaMalloc the first time a K split needs it, and a context itself is
 * created with cudaMalloc. Some callers cannot do either at the point where
 * they need the product: serving processes that hand all device memory to their
 * own pool at start-up and forbid later driver allocations, and real-time paths
 * where the latency of an allocation is not acceptable. This entry point takes no context and touches no allocator: the
 * FP32 partial sums of the K split live in a fixed array that is part of the
 * library image, so every GPU that loads the library holds those 8 MiB until
 * the process exits.
 *
 * How the address is obtained. In host code the array's name is only a
 * stand-in for the device symbol, not a device address. The first call on each
 * device, with that device current, asks the runtime for the real address with
 * cudaGetSymbolAddress and caches it per device; later calls reuse it. That
 * first call should therefore be made before any stream capture begins. The
 * look-up is guarded by a once-flag per device, so host threads may make their
 * first calls concurrently; each of them sees a complete entry.
 *
 * Sharing. All calls on a device share the one array and it keeps whatever
 * the previous call left. Nothing in it has to start at zero: every partial
 * that the reduction reads is written by the product kernel of the same call
 * first. Two calls whose kernels overlap on the GPU (different streams without
 * an ordering between them) race on the array; order them.
 */
#pragma once

#include "context.cuh"
#include "gemv_skinny.cuh"

#include <mutex>

namespace static_scratch
{

constexpr size_t kScratchBytes = size_t(8) << 20; /* 8 MiB of FP32 partial sums */
constexpr int kMaxDevices = 64;

static __device__ __align__(256) float partial_sums[kScratchBytes / sizeof(float)];

struct DeviceSetup {
    std::once_flag once;
    float *scratch = nullptr; /* device address of partial_sums on this device */
    int sm_count = 0;
    int lookup = 0; /* cudaError_t of the look-up, 0 when it succeeded */
};
static DeviceSetup device_setup[kMaxDevices];

/* Look up the device address of the array once per device (current device).
 * std::call_once orders the writes of the first caller before every other
 * caller's reads, so no thread can see a half-filled entry. A failed look-up
 * is remembered and reported by every later call on that device. */
inline int setup(int device, DeviceSetup **out)
{
    if (device < 0 || device >= kMaxDevices)
        return host::fail(nullptr, "static scratch device index", 1);
    DeviceSetup &entry = device_setup[device];
    std::call_once(entry.once, [&entry, device] {
        float *address = nullptr;
        cudaError_t error =
            cudaGetSymbolAddress(reinterpret_cast<void **>(&address), partial_sums);
        if (error == cudaSuccess && address == nullptr)
            error = cudaErrorInvalidSymbol;
        if (error == cudaSuccess)
            error = cudaDeviceGetAttribute(&entry.sm_count, cudaDevAttrMultiProcessorCount, device);
        entry.scratch = address;
        entry.lookup = int(error);
    });
    if (entry.lookup != 0 || entry.scratch == nullptr || entry.sm_count < 1)
        return host::fail(nullptr, "static scratch address lookup", entry.lookup ? entry.lookup : 1);
    *out = &entry;
    return 0;
}

template <int Tokens>
int launch(const DeviceSetup &entry, cudaStream_t stream, skinny::Task &task)
{
    /* same geometry rules as the context-based skinny path */
    const int sms = entry.sm_count;
    int rows_per_warp = 4;
    while (rows_per_warp > 1 &&
           (task.outputs + rows_per_warp * skinny::kWarps - 1) / (rows_per_warp * skinny::kWarps) <
               2 * sms)
        rows_per_warp >>= 1;
    const int row_blocks =
        (task.outputs + rows_per_warp * skinny::kWarps - 1) / (rows_per_warp * skinny::kWarps);
    int split = (task.depth + 4095) / 4096;
    while (1ll * row_blocks * split < 2ll * sms && task.depth / (split * 2) >= 512)
        split *= 2;
    const int per = ((task.depth + split - 1) / split + 7) & ~7;
    split = (task.depth + per - 1) / per;
    task.split = split, task.depth_per_split = per;
    if (split > 1) {
        const size_t bytes = size_t(split) * task.tokens * task.outputs * sizeof(float);
        if (bytes > kScratchBytes) {
            std::snprintf(host::creation_error, sizeof(host::creation_error),
                          "static scratch too small: this product needs %zu bytes of partial sums, "
                          "the fixed array holds %zu",
                          bytes, kScratchBytes);
            return -1;
        }
        task.partial = entry.scratch;
    }
    const size_t shared = size_t(Tokens) * per * sizeof(__nv_bfloat16);
    dim3 grid(row_blocks, split);
    if (rows_per_warp == 4)
        skinny::skinny_gemv<Tokens, 4><<<grid, skinny::kThreads, shared, stream>>>(task);
    else if (rows_per_warp == 2)
        skinny::skinny_gemv<Tokens, 2><<<grid, skinny::kThreads, shared, stream>>>(task);
    else
        skinny::skinny_gemv<Tokens, 1><<<grid, skinny::kThreads, shared, stream>>>(task);
    int status = host::launched(nullptr, "static-scratch skinny product");
    if (status != 0 || split == 1)
        return status;
    dim3 reduce_grid((task.outputs + 255) / 256, task.tokens);
    skinny::skinny_reduce<<<reduce_grid, 256, 0, stream>>>(task);
    return host::launched(nullptr, "static-scratch split reduction");
}

} // namespace static_scratch

extern "C" int camblas_cuda_linear_bf16_static(void *stream, int rows, int inner, int outputs,
                                               const void *x, int ldx, const void *w, int ldw,
                                               void *out, int ldo)
{
    if (rows < 0 || rows > 4 || inner < 1 || outputs < 0 || ldx < inner || ldw < inner ||
        ldo < outputs)
        return host::fail(nullptr, "invalid static-scratch linear dimensions (1 to 4 token rows)", 1);
    if (rows == 0 || outputs == 0)
        return 0;
    if (!x || !w || !out || out == x || out == w)
        return host::fail(nullptr, "missing or aliased static-scratch linear operand", 1);
    if (!host::aligned16(w) || ldw % 8 != 0)
        return host::fail(nullptr, "static-scratch linear needs 16-byte aligned weight rows", 1);
    int device = -1;
    cudaError_t error = cudaGetDevice(&device);
    if (error != cudaSuccess)
        return host::fail(nullptr, "current device query", int(error));
    static_scratch::DeviceSetup *entry = nullptr;
    int status = static_scratch::setup(device, &entry);
    if (status != 0)
        return status;
    skinny::Task task{};
    task.outputs = outputs, task.tokens = rows, task.depth = inner;
    task.ldw = ldw, task.ldx = ldx;
    task.alpha = 1.f, task.beta = 0.f;
    task.w = static_cast<const __nv_bfloat16 *>(w);
    task.x = static_cast<const __nv_bfloat16 *>(x);
    task.out = static_cast<__nv_bfloat16 *>(out);
    task.ld_out = ldo;
    cudaStream_t launch_stream = static_cast<cudaStream_t>(stream);
    switch (rows) {
    case 1:
        return static_scratch::launch<1>(*entry, launch_stream, task);
    case 2:
        return static_scratch::launch<2>(*entry, launch_stream, task);
    default:
        return static_scratch::launch<4>(*entry, launch_stream, task);
    }
}
