#pragma once
#include "context.cuh"
namespace fp8 { inline int prepare_kernels() { return 0; } }
namespace strassen {
inline bool eligible(camblas_cuda_context *, const host::Product &) { return false; }
inline int run(camblas_cuda_context *context, const host::Product &) { return host::fail(context, "strassen", 1); }
}
extern "C" int camblas_cuda_fp8_quantize_rows(camblas_cuda_context *context, int, int, const void *, int, void *, float *) { return host::unavailable(context, "camblas_cuda_fp8_quantize_rows"); }
extern "C" int camblas_cuda_fp8_block_gemm(camblas_cuda_context *context, int, int, int, const void *, const float *, const void *, const float *, void *, int) { return host::unavailable(context, "camblas_cuda_fp8_block_gemm"); }
extern "C" int camblas_cuda_fp8_decode_supported(const camblas_cuda_context *) { return 0; }
extern "C" int camblas_cuda_fp8_decode(camblas_cuda_context *context, int, int, const void *, const float *, const void *, const float *, int, int, int, void *, size_t, void *) { return host::unavailable(context, "camblas_cuda_fp8_decode"); }
extern "C" size_t camblas_cuda_fp8_workspace_size(int, int, int) { return 0; }
extern "C" int camblas_cuda_fp8_linear(camblas_cuda_context *context, int, int, const void *, const void *, const float *, int, int, void *, size_t, void *) { return host::unavailable(context, "camblas_cuda_fp8_linear"); }
