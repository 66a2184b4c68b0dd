/*
 * Host-side choice of the BF16 kernel family and launch geometry. The table is
 * static: the same shape always gets the same kernel, tile and K split, so the
 * first call is as fast as the hundredth and results are repeatable (the
 * reference times up to twelve library candidates on first use,
 * backend.cu:719-779).
 *
 * In BLAS terms C[m,n] (column-major) = op(A)[m,k] op(B)[k,n]. Written from
 * the torch side, A is the weight [outputs,inner] ('T'), B the activations
 * [tokens,inner] ('N'), and C the row-major [tokens,outputs] result. The
 * kernels see a row-major D[n,m] with row pitch ldc:
 *   family 3 (tcgen05)          P = op(B) rows (tokens), Q = op(A) rows (outputs)
 *   family 4 (tcgen05, swapped) P = op(A) rows (outputs), Q = op(B) rows (tokens),
 *                               D^T stored, optional split-K through scratch
 *   family 2 (skinny)           up to four tokens, CUDA cores, split-K
 *   family 5 (tcgen05, two SMs) as family 3 with 256-row tiles computed by CTA pairs
 *   family 1 (generic)          anything else
 */
#pragma once

#include "context.cuh"
#include "gemm_bf16_cluster.cuh"
#include "gemm_bf16_pair.cuh"
#include "gemm_bf16_tcgen05.cuh"
#include "gemm_generic.cuh"
#include "gemv_skinny.cuh"

#include <algorithm>
#include <cstdlib>
#include <cstring>

namespace host
{

enum Family : int {
    kAuto = 0,
    kGeneric = 1,
    kSkinny = 2,
    kTensor = 3,
    kTensorSwapped = 4,
    kTensorPair = 5
};

struct Product {
    bool ta, tb;
    int m, n, k;
    float alpha, beta;
    const __nv_bfloat16 *a, *b;
    long long lda, ldb;
    __nv_bfloat16 *c;
    long long ldc;
    const __nv_bfloat16 *addend; /* beta term, indexed like c */
    long long ld_add;
    const __nv_bfloat16 *bias; /* per BLAS row i (output feature), may be NULL */
    /* packed projection: BLAS rows [0,cut0) -> c, [cut0,cut1) -> c1, [cut1,m) -> c2 */
    int cut0, cut1;
    __nv_bfloat16 *c1, *c2;
    long long ldc1, ldc2;
    /* device word: when non-NULL the tensor-core row kernel runs only if it is non-zero */
    const unsigned *run_if_set;
};

template <int BN, int Stages, int Mode, int PMajor = sm100::kMajorK, int QMajor = sm100::kMajorK>
int prepare_kernel()
{
    return int(cudaFuncSetAttribute(sm100::gemm_bf16_tcgen05<BN, Stages, Mode, PMajor, QMajor>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    sm100::GemmSmem<BN, Stages, Mode>::kTotal));
}

template <int PMajor, int QMajor> int prepare_row_kernels()
{
    return prepare_kernel<256, 4, sm100::kStoreRows, PMajor, QMajor>() |
           prepare_kernel<128, 6, sm100::kStoreRows, PMajor, QMajor>() |
           prepare_kernel<64, 8, sm100::kStoreRows, PMajor, QMajor>();
}

template <int PMajor, int QMajor> int prepare_pair_kernels()
{
    using namespace sm100;
    int status = int(cudaFuncSetAttribute(gemm_bf16_pair<256, 3, PMajor, QMajor, 2>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          PairSmem<256, 3, 2>::kTotal));
    status |= int(cudaFuncSetAttribute(gemm_bf16_pair<128, 4, PMajor, QMajor, 2>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       PairSmem<128, 4, 2>::kTotal));
    if constexpr (QMajor == kMajorK)
        status |= int(cudaFuncSetAttribute(gemm_bf16_pair<0, 3, PMajor, QMajor, 2>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           PairSmem<256, 3, 2>::kTotal));
    return status;
}

template <int BN, int Stages, int Mode> int prepare_cluster_kernel()
{
    return int(cudaFuncSetAttribute(sm100::gemm_bf16_cluster<BN, Stages, Mode>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    sm100::GemmSmem<BN, Stages, sm100::kStoreColumns>::kTotal));
}

inline int prepare_kernels()
{
    using namespace sm100;
    int status = prepare_row_kernels<kMajorK, kMajorK>();
    status |= prepare_cluster_kernel<256, 4, kStoreRows>();
    status |= prepare_cluster_kernel<128, 6, kStoreRows>();
    status |= prepare_cluster_kernel<16, 8, kStoreColumns>();
    status |= prepare_cluster_kernel<32, 8, kStoreColumns>();
    status |= prepare_cluster_kernel<64, 8, kStoreColumns>();
    status |= prepare_pair_kernels<kMajorK, kMajorK>();
    status |= prepare_pair_kernels<kMajorK, kMajorMN>();
    status |= prepare_pair_kernels<kMajorMN, kMajorK>();
    status |= prepare_pair_kernels<kMajorMN, kMajorMN>();
    status |= int(cudaFuncSetAttribute(gemm_bf16_pair<256, 3, kMajorK, kMajorK, 2, kEpiPush>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       PairSmem<256, 3, 2>::kTotal));
    status |= int(cudaFuncSetAttribute(gemm_bf16_pair<128, 4, kMajorK, kMajorK, 2, kEpiPush>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       PairSmem<128, 4, 2>::kTotal));
    status |= int(cudaFuncSetAttribute(gemm_bf16_pair<256, 3, kMajorK, kMajorK, 2, kEpiSwiglu>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       PairSmem<256, 3, 2>::kTotal));
    status |= int(cudaFuncSetAttribute(gemm_bf16_pair<256, 3, kMajorK, kMajorK, 2, kEpiSwigluQuant>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       PairSmem<256, 3, 2>::kTotal));
    status |= prepare_row_kernels<kMajorK, kMajorMN>();
    status |= prepare_row_kernels<kMajorMN, kMajorK>();
    status |= prepare_row_kernels<kMajorMN, kMajorMN>();
    status |= prepare_kernel<256, 4, kStoreFloat, kMajorK, kMajorMN>();
    status |= prepare_kernel<16, 8, sm100::kStoreColumns>();
    status |= prepare_kernel<32, 8, sm100::kStoreColumns>();
    status |= prepare_kernel<64, 8, sm100::kStoreColumns>();
    status |= prepare_kernel<16, 8, sm100::kStorePartial>();
    status |= prepare_kernel<32, 8, sm100::kStorePartial>();
    status |= prepare_kernel<64, 8, sm100::kStorePartial>();
    return status;
}

template <int BN, int Stages, int Mode, int PMajor = sm100::kMajorK, int QMajor = sm100::kMajorK>
void launch_tensor(camblas_cuda_context *context, const CUtensorMap &p, const CUtensorMap &q,
                   const CUtensorMap &d0, const CUtensorMap &d1, const CUtensorMap &d2,
                   const sm100::GemmTask &task)
{
    long long units = sm100::unit_count(task);
    int grid = (units < context->sm_count && task.sk_cols == 0) ? int(units) : context->sm_count;
    sm100::gemm_bf16_tcgen05<BN, Stages, Mode, PMajor, QMajor>
        <<<grid, sm100::kThreads, sm100::GemmSmem<BN, Stages, Mode>::kTotal, context->stream>>>(
            p, q, d0, d1, d2, task);
}

template <int PMajor, int QMajor>
void launch_rows(camblas_cuda_context *context, int bn, const CUtensorMap &p, const CUtensorMap &q,
                 const CUtensorMap &d0, const CUtensorMap &d1, const CUtensorMap &d2,
                 const sm100::GemmTask &task)
{
    if (bn == 256)
        launch_tensor<256, 4, sm100::kStoreRows, PMajor, QMajor>(context, p, q, d0, d1, d2, task);
    else if (bn == 128)
        launch_tensor<128, 6, sm100::kStoreRows, PMajor, QMajor>(context, p, q, d0, d1, d2, task);
    else
        launch_tensor<64, 8, sm100::kStoreRows, PMajor, QMajor>(context, p, q, d0, d1, d2, task);
}

/* Operands the TMA pipeline can take: 16-byte aligned base and row pitch. */
inline bool tensor_operands_ok(const Product &x)
{
    return aligned16(x.a) && aligned16(x.b) && x.lda % 8 == 0 &&
           (x.ldb % 8 == 0 || (x.n == 1 && !x.tb));
}

/* The few-token kernels take only the layout a linear layer produces. */
inline bool swapped_operands_ok(const Product &x)
{
    return x.ta && !x.tb && tensor_operands_ok(x);
}

inline bool rows_store_ok(const Product &x)
{
    if (!aligned16(x.c) || x.ldc % 8 != 0)
        return false;
    if (x.cut0 < x.m)
        return aligned16(x.c1) && aligned16(x.c2) && x.ldc1 % 8 == 0 && x.ldc2 % 8 == 0;
    return true;
}

/* Smallest K split whose work units fill the SMs evenly; the split costs
 * 8 bytes of scratch traffic per partial element, so smaller is better. */
inline int choose_split(int tiles, int k_blocks, int sms)
{
    int limit = k_blocks / 8 < 1 ? 1 : (k_blocks / 8 > 32 ? 32 : k_blocks / 8);
    int best = 1;
    double best_score = 0;
    for (int split = 1; split <= limit; ++split) {
        long long units = 1ll * tiles * split;
        long long waves = (units + sms - 1) / sms;
        double fill = double(units) / double(waves * sms);
        double score = fill - 0.01 * split;
        if (score > best_score + 1e-9) {
            best_score = score;
            best = split;
        }
    }
    return best;
}

/* ---- K split inside a cluster (gemm_bf16_cluster.cuh) ---- */

template <int BN, int Stages, int Mode>
cudaLaunchConfig_t cluster_config(camblas_cuda_context *context, int tiles, int parts,
                                  cudaLaunchAttribute *attribute)
{
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(unsigned(tiles) * unsigned(parts));
    config.blockDim = dim3(sm100::kThreads);
    config.dynamicSmemBytes = sm100::GemmSmem<BN, Stages, sm100::kStoreColumns>::kTotal;
    config.stream = context->stream;
    attribute[0].id = cudaLaunchAttributeClusterDimension;
    attribute[0].val.clusterDim.x = unsigned(parts);
    attribute[0].val.clusterDim.y = 1;
    attribute[0].val.clusterDim.z = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    return config;
}

/* How many clusters of `parts` CTAs of this kernel the device runs at once (a
 * cluster lives inside one GPC, so this is less than SMs / parts); asked once
 * per kernel and size, kept in the context. */
template <int BN, int Stages, int Mode>
int resident_clusters(camblas_cuda_context *context, int slot, int parts)
{
    int &cached = context->cluster_capacity[slot][parts];
    if (cached == 0) {
        cudaLaunchAttribute attribute[1];
        cudaLaunchConfig_t config = cluster_config<BN, Stages, Mode>(context, 1, parts, attribute);
        int clusters = 0;
        cudaError_t error = cudaOccupancyMaxActiveClusters(
            &clusters, sm100::gemm_bf16_cluster<BN, Stages, Mode>, &config);
        if (error != cudaSuccess) {
            cudaGetLastError();
            clusters = 0;
        }
        cached = clusters > 0 ? clusters : -1;
    }
    return cached > 0 ? cached : 0;
}

/* Largest cluster size (2..8) whose clusters for all `tiles` are resident
 * together and whose K ranges keep at least four K blocks; 0 when the tiles
 * would still occupy less than half of the SMs, or when switched off. */
template <int BN, int Stages, int Mode>
int choose_cluster_parts(camblas_cuda_context *context, int slot, int tiles, int k_blocks)
{
    if (context->options.cluster_split == 0)
        return 0;
    for (int parts = 8; parts >= 2; --parts) {
        if (k_blocks / parts < 4 || 1ll * tiles * parts > context->sm_count)
            continue;
        if (resident_clusters<BN, Stages, Mode>(context, slot, parts) < tiles)
            continue;
        return 2 * tiles * parts >= context->sm_count ? parts : 0;
    }
    return 0;
}

template <int BN, int Stages, int Mode>
int launch_cluster(camblas_cuda_context *context, int tiles, int parts, const CUtensorMap &p,
                   const CUtensorMap &q, const sm100::GemmTask &task)
{
    cudaLaunchAttribute attribute[1];
    cudaLaunchConfig_t config = cluster_config<BN, Stages, Mode>(context, tiles, parts, attribute);
    cudaError_t error =
        cudaLaunchKernelEx(&config, sm100::gemm_bf16_cluster<BN, Stages, Mode>, p, q, task);
    if (error != cudaSuccess)
        return fail(context, "cluster split-K tcgen05 BF16 GEMM", error);
    context->kernel_launches.fetch_add(1, std::memory_order_relaxed);
    return 0;
}

/* Whether a K split pays at all. The split buys a better fill of the SMs and
 * costs a second launch plus a write and a read of `split` FP32 copies of the
 * result. Rough microseconds for a weight-streaming tile of 128 rows by `bn`
 * token columns whose K blocks are 128 bytes deep: a CTA alone takes about
 * 0.29 us per block (measured: 64 tiles of the Llama down projection without a
 * split stream at 3.6 TB/s); with every SM streaming, HBM (6.5 TB/s) allows one
 * block per SM every 148 * bytes / 6.5 MB us. When the tiles alone already give
 * most SMs work (N = 24576: 192 tiles), not splitting wins even though the fill
 * is worse: measured 22 against 31 us for 64 tokens. The model is rough, so the
 * unsplit form has to win by a quarter to be taken. */
inline int split_if_it_pays(int split, int tiles, int k_blocks, int sms, int tokens, int outputs,
                            int bn)
{
    if (split <= 1)
        return 1;
    const double step_bytes = 128.0 * 128 + 128.0 * bn;
    auto main_us = [&](int parts) {
        const long long units = 1ll * tiles * parts;
        const double waves = double((units + sms - 1) / sms);
        const double busy = double(units < sms ? units : sms);
        const double step = std::max(0.29, busy * step_bytes / 6.5e6);
        return waves * ((k_blocks + parts - 1) / parts) * step;
    };
    const double reduce_us = 3.0 + 2.0 * split * double(tokens) * outputs * 4 / 3.0e6;
    return 1.25 * main_us(1) <= main_us(split) + reduce_us ? 1 : split;
}

/* The same estimate over every candidate split, with the step of a CTA that
 * streams alone taken from its bytes (69 GB/s per CTA: 0.36 us for a 64-token
 * step, measured on the K/4 shard of the down projection). Returns the cheapest. */
inline int cheapest_split(int tiles, int k_blocks, int sms, int tokens, int outputs, int bn)
{
    const double step_bytes = 128.0 * 128 + 128.0 * bn;
    const double alone = std::max(0.29, step_bytes / 69.0e3);
    const int limit = k_blocks / 8 < 1 ? 1 : (k_blocks / 8 > 32 ? 32 : k_blocks / 8);
    int best = 1;
    double best_us = 1e30;
    for (int parts = 1; parts <= limit; ++parts) {
        const long long units = 1ll * tiles * parts;
        const double waves = double((units + sms - 1) / sms);
        const double busy = double(units < sms ? units : sms);
        const double step = std::max(alone, busy * step_bytes / 6.5e6);
        double us = waves * ((k_blocks + parts - 1) / parts) * step;
        if (parts > 1)
            us += 3.0 + 2.0 * parts * double(tokens) * outputs * 4 / 3.0e6;
        if (us < best_us - 1e-9)
            best_us = us, best = parts;
    }
    return best;
}

inline int run_tensor_rows(camblas_cuda_context *context, const Product &x)
{
    sm100::GemmTask task{};
    task.rows = x.n, task.cols = x.m, task.depth = x.k;
    task.r_blocks = (x.n + 127) / 128;
    task.k_blocks = (x.k + 63) / 64;
    task.split = 1, task.k_blocks_per_split = task.k_blocks;
    task.alpha = x.alpha, task.beta = x.beta;
    task.out = x.c, task.ld_out = x.ldc;
    task.addend = x.addend, task.ld_add = x.ld_add;
    task.bias = x.bias;
    task.status = context->status;
    task.cut0 = x.cut0, task.cut1 = x.cut1;
    task.batch = 1;
    task.run_if_set = x.run_if_set;
    bool packed = x.cut0 < x.m;
    /* Tile width: 256 columns unless the product is narrower. When the tiles do
     * not fill the SMs evenly, the last partial wave is spread over all SMs by
     * K range (stream-K) if the idle time it recovers outweighs the second pass
     * over the partial sums. Rates are rough steady-state figures of this kernel
     * on a B200; only their ratio matters. */
    const int sms = context->sm_count;
    int bn = x.m <= 64 ? 64 : (x.m <= 128 ? 128 : 256);
    if (packed && (x.cut0 % bn != 0 || x.cut1 % bn != 0)) {
        bn = 128;
        if (x.cut0 % bn != 0 || x.cut1 % bn != 0)
            return fail(context, "packed projection widths must be multiples of 128", 1);
    }
    task.c_blocks = (x.m + bn - 1) / bn;
    task.panel = task.r_blocks < 8 ? task.r_blocks : 8;
    /* Few tiles and a long K in the layout of a linear layer: one cluster per
     * tile, K split over its CTAs, sums through distributed shared memory: one
     * launch, no scratch, 2-5 % faster than the stream-K pieces on the QKV shards
     * of tensor-parallel ranks (23.1 against 23.8 us at 512 x 8192 -> 1280). Both
     * forms pull the same 126 MB through L2 for that product, which is what
     * bounds them. */
    if (x.ta && !x.tb && x.run_if_set == nullptr && bn >= 128 && task.k_blocks >= 16) {
        /* This kernel stores eight columns at a time and looks up the output of each,
         * so a packed projection needs cuts on multiples of eight only, not on tile
         * boundaries: 256-column tiles pull a quarter fewer bytes through L2 than
         * 128-column ones (the QKV shard of a rank at tensor-parallel 8 is 1024 +
         * 128 + 128 columns). */
        int wide = bn;
        if (packed && x.m > 128 && x.cut0 % 8 == 0 && x.cut1 % 8 == 0)
            wide = 256;
        const int c_blocks = (x.m + wide - 1) / wide;
        const int tiles = task.r_blocks * c_blocks;
        const int parts = wide == 256 ? choose_cluster_parts<256, 4, sm100::kStoreRows>(
                                            context, 0, tiles, task.k_blocks)
                                      : choose_cluster_parts<128, 6, sm100::kStoreRows>(
                                            context, 1, tiles, task.k_blocks);
        if (parts >= 2) {
            task.c_blocks = c_blocks;
            task.out1 = x.c1, task.out2 = x.c2;
            task.ld_out1 = x.ldc1, task.ld_out2 = x.ldc2;
            CUtensorMap p, q;
            const auto bf16 = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
            if (!encode_2d(context, &p, bf16, 2, x.b, x.k, x.n, x.ldb * 2, 64, 128) ||
                !encode_2d(context, &q, bf16, 2, x.a, x.k, x.m, x.lda * 2, 64, wide))
                return fail(context, "tensor map encoding", 1);
            return wide == 256
                       ? launch_cluster<256, 4, sm100::kStoreRows>(context, tiles, parts, p, q, task)
                       : launch_cluster<128, 6, sm100::kStoreRows>(context, tiles, parts, p, q, task);
        }
    }
    if (task.r_blocks <= 8 && sms / task.r_blocks >= 2) {
        const int teams = sms / task.r_blocks;
        const int rest = task.c_blocks % teams;
        const double tile_us = 2.0 * 128 * bn * x.k / (1.35e15 / 148.0 / 1e6);
        const double recovered = (1.0 - double(rest) / teams) * tile_us;
        const double second_pass =
            3.0 + double(rest + teams) * task.r_blocks * 128 * bn * 8 / 5.0e6;
        if (rest != 0 && task.k_blocks >= 16 && x.run_if_set == nullptr &&
            recovered > second_pass) {
            task.dp_cols = task.c_blocks - rest, task.sk_cols = rest;
            int status = reserve_scratch(context, size_t(2) * sms * 128 * bn * sizeof(float));
            if (status != 0)
                return status;
            task.sk_partial = static_cast<float *>(context->scratch);
        }
    }

    CUtensorMap p, q, d0, d1, d2;
    const auto bf16 = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    /* P = op(B): 'N' stores row j contiguous along k (K-major); 'T' stores b[j + l*ldb]
     * (MN-major, 64 x 64 boxes). Q = op(A): 'T' is K-major, 'N' is a[i + l*lda]. */
    bool ok = x.tb ? encode_2d(context, &p, bf16, 2, x.b, x.n, x.k, x.ldb * 2, 64, 64)
                   : encode_2d(context, &p, bf16, 2, x.b, x.k, x.n, x.ldb * 2, 64, 128);
    ok = ok && (x.ta ? encode_2d(context, &q, bf16, 2, x.a, x.k, x.m, x.lda * 2, 64, bn)
                     : encode_2d(context, &q, bf16, 2, x.a, x.m, x.k, x.lda * 2, 64, 64));
    if (packed) {
        ok = ok &&
             encode_2d(context, &d0, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x.c, x.cut0, x.n,
                       x.ldc * 2, 64, 32) &&
             encode_2d(context, &d1, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x.c1, x.cut1 - x.cut0,
                       x.n, x.ldc1 * 2, 64, 32) &&
             encode_2d(context, &d2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x.c2, x.m - x.cut1, x.n,
                       x.ldc2 * 2, 64, 32);
    } else {
        ok = ok && encode_2d(context, &d0, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x.c, x.m, x.n,
                             x.ldc * 2, 64, 32);
        d1 = d0, d2 = d0;
    }
    if (!ok)
        return fail(context, "tensor map encoding", 1);
    using namespace sm100;
    if (!x.tb && x.ta)
        launch_rows<kMajorK, kMajorK>(context, bn, p, q, d0, d1, d2, task);
    else if (!x.tb && !x.ta)
        launch_rows<kMajorK, kMajorMN>(context, bn, p, q, d0, d1, d2, task);
    else if (x.tb && x.ta)
        launch_rows<kMajorMN, kMajorK>(context, bn, p, q, d0, d1, d2, task);
    else
        launch_rows<kMajorMN, kMajorMN>(context, bn, p, q, d0, d1, d2, task);
    int status = launched(context, "tcgen05 BF16 GEMM");
    if (status != 0 || task.sk_cols == 0)
        return status;
    dim3 grid(task.sk_cols, 128 * bn / 8 / 256, task.r_blocks);
    if (bn == 256)
        sm100::sk_fixup<256><<<grid, 256, 0, context->stream>>>(task, sms, x.c1, x.ldc1, x.c2,
                                                                x.ldc2);
    else if (bn == 128)
        sm100::sk_fixup<128><<<grid, 256, 0, context->stream>>>(task, sms, x.c1, x.ldc1, x.c2,
                                                                x.ldc2);
    else
        sm100::sk_fixup<64><<<grid, 256, 0, context->stream>>>(task, sms, x.c1, x.ldc1, x.c2,
                                                               x.ldc2);
    return launched(context, "stream-K fix-up");
}

template <int BN, int Stages, int PMajor, int QMajor, int Sub = 1, int Epi = sm100::kEpiStore>
cudaError_t launch_pair(camblas_cuda_context *context, int pairs, const CUtensorMap &p,
                        const CUtensorMap &q, const CUtensorMap &d0, const CUtensorMap &d1,
                        const CUtensorMap &d2, const sm100::GemmTask &task)
{
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(2 * pairs);
    config.blockDim = dim3(sm100::kThreads);
    config.dynamicSmemBytes = sm100::PairSmem<(BN ? BN : 256), Stages, Sub>::kTotal;
    config.stream = context->stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeClusterDimension;
    attribute[0].val.clusterDim.x = 2;
    attribute[0].val.clusterDim.y = 1;
    attribute[0].val.clusterDim.z = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, sm100::gemm_bf16_pair<BN, Stages, PMajor, QMajor, Sub, Epi>,
                              p, q, d0, d1, d2, task);
}

template <int PMajor, int QMajor>
cudaError_t launch_pair_width(camblas_cuda_context *context, int bn, int pairs, const CUtensorMap &p,
                              const CUtensorMap &q, const CUtensorMap &d0, const CUtensorMap &d1,
                              const CUtensorMap &d2, const sm100::GemmTask &task)
{
    if (task.width != 0) {
        if constexpr (QMajor == sm100::kMajorK)
            return launch_pair<0, 3, PMajor, QMajor, 2>(context, pairs, p, q, d0, d1, d2, task);
        else
            return cudaErrorInvalidValue;
    }
    /* two 64-deep K blocks per stage: half as many barrier round trips per flop
     * as one block per stage, measured 3-7 % faster on B200 */
    if (bn == 256)
        return launch_pair<256, 3, PMajor, QMajor, 2>(context, pairs, p, q, d0, d1, d2, task);
    return launch_pair<128, 4, PMajor, QMajor, 2>(context, pairs, p, q, d0, d1, d2, task);
}

/* Two-SM tiles: 256 token rows x bn outputs per CTA pair. */
inline int run_tensor_pair(camblas_cuda_context *context, const Product &x)
{
    sm100::GemmTask task{};
    task.rows = x.n, task.cols = x.m, task.depth = x.k;
    task.r_blocks = (x.n + 255) / 256;
    task.k_blocks = (x.k + 63) / 64;
    task.split = 1, task.k_blocks_per_split = task.k_blocks;
    task.alpha = x.alpha, task.beta = x.beta;
    task.out = x.c, task.ld_out = x.ldc;
    task.addend = x.addend, task.ld_add = x.ld_add;
    task.bias = x.bias;
    task.status = context->status;
    task.cut0 = x.cut0, task.cut1 = x.cut1;
    task.batch = 1;
    task.run_if_set = x.run_if_set;
    const bool packed = x.cut0 < x.m;
    const int pairs_max = context->sm_count / 2;
    task.out1 = x.c1, task.out2 = x.c2;
    task.ld_out1 = x.ldc1, task.ld_out2 = x.ldc2;
    /* Tile width. With a K-major weight the width may be any multiple of 16:
     * take the one whose tile count fills whole waves of CTA pairs best (wide
     * tiles are a little more efficient per flop, hence the weight on width).
     * The alternative for 256-column tiles is the stream-K tail. Costs are in
     * microseconds from rough steady-state rates; only their order matters. */
    const double pair_flops_per_us = 2 * 1.45e15 / 148.0 / 1e6;
    /* A K block costs the longer of its MMA time (two cycles per tile column)
     * and the time to bring its operands in (16 KB of P plus 64 bytes per column
     * at about 65 bytes per cycle and SM), so narrow tiles are bound by loads. */
    auto tile_us = [&](int width) {
        const double cycles = std::max(2.0 * width, (16384.0 + 64.0 * width) / 65.0);
        return 2.0 * 256 * 256 * x.k / pair_flops_per_us * cycles / 512.0;
    };
    /* tuning aids of the context: whole tiles only, always split the tail, forced width */
    const bool tail_plain = context->options.pair_tail == 1, tail_split = context->options.pair_tail == 2;
    int bn = x.m <= 128 ? 128 : 256;
    double best = 1e30;
    int best_width = 0;
    const int forced_width = context->options.pair_width;
    /* Measured on B200, tiles narrower than 256 columns are bound by operand
     * loads and never beat 256-column tiles with or without the stream-K tail on
     * the Llama shapes, so a run-time width is used only on request. */
    if (forced_width != 0 && x.ta && x.m > 128 &&
        (!packed || (x.cut0 % 16 == 0 && x.cut1 % 16 == 0))) {
        for (int width = 128; width <= 256; width += 16) {
            if (forced_width != 0 && width != forced_width)
                continue;
            long long tiles = 1ll * task.r_blocks * ((x.m + width - 1) / width);
            double cost = double((tiles + pairs_max - 1) / pairs_max) * tile_us(width);
            if (cost < best - 1e-9)
                best = cost, best_width = width;
        }
    }
    if (packed && best_width == 0 && (x.cut0 % bn != 0 || x.cut1 % bn != 0)) {
        bn = 128;
        if (x.cut0 % bn != 0 || x.cut1 % bn != 0)
            return fail(context, "packed projection widths must be multiples of 128", 1);
    }
    bool stream_k = false;
    if (task.r_blocks <= 8 && pairs_max / task.r_blocks >= 2 && task.k_blocks >= 16 &&
        x.run_if_set == nullptr && !(packed && (x.cut0 % bn != 0 || x.cut1 % bn != 0))) {
        const int columns = (x.m + bn - 1) / bn;
        const int teams = pairs_max / task.r_blocks;
        const int rest = columns % teams;
        /* a long tail (most teams busy anyway) gains less than the second pass costs */
        if (rest != 0 && (2 * rest <= teams || tail_split)) {
            const double second_pass =
                6.0 + double(rest + teams) * task.r_blocks * 256 * bn * 8 / 5.0e6;
            const double cost = (double(columns) / teams) * tile_us(bn) + second_pass;
            const double plain = double((columns + teams - 1) / teams) * tile_us(bn);
            if ((cost < plain && cost < best && forced_width == 0 && !tail_plain) || tail_split) {
                stream_k = true;
                best_width = 0;
            }
        }
    }
    /* One exception, measured: when the 256-column tiles fit in a single wave that
     * leaves pairs idle, the product takes as long as one tile, and a tile's time
     * falls with its width (512 x 8192 -> 5120, 40 tiles on 74 pairs: 46.6 us at
     * 256 columns, 44.1 at 208, 42.4 at 144 with 72 tiles). Take the narrowest width
     * from 144 columns that still needs one wave only; with a second wave every
     * narrower width loses (-> 10240: 73.8 us at 256, 81 and more below). */
    if (!stream_k && forced_width == 0 && bn == 256 && x.ta && x.run_if_set == nullptr &&
        (!packed || (x.cut0 % 16 == 0 && x.cut1 % 16 == 0)) &&
        1ll * task.r_blocks * ((x.m + 255) / 256) <= pairs_max) {
        for (int width = 144; width < 256; width += 16)
            if (1ll * task.r_blocks * ((x.m + width - 1) / width) <= pairs_max) {
                best_width = width, best = 0.0;
                break;
            }
    }
    if (best_width != 0) {
        const long long tiles = 1ll * task.r_blocks * ((x.m + bn - 1) / bn);
        const double plain = double((tiles + pairs_max - 1) / pairs_max) * tile_us(bn);
        if (plain <= best && forced_width == 0)
            best_width = 0; /* the fixed-width kernel does as well */
    }
    if (best_width != 0)
        bn = best_width, task.width = best_width;
    task.c_blocks = (x.m + bn - 1) / bn;
    task.panel = task.r_blocks < 8 ? task.r_blocks : 8;
    if (stream_k) {
        const int teams = pairs_max / task.r_blocks;
        const int rest = task.c_blocks % teams;
        task.dp_cols = task.c_blocks - rest, task.sk_cols = rest;
        int status = reserve_scratch(context, size_t(4) * pairs_max * 128 * bn * sizeof(float));
        if (status != 0)
            return status;
        task.sk_partial = static_cast<float *>(context->scratch);
    }
    long long units = 1ll * task.r_blocks * task.c_blocks;
    int pairs = (units < pairs_max && task.sk_cols == 0) ? int(units) : pairs_max;

    CUtensorMap p, q, d0, d1, d2;
    const auto bf16 = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    bool ok = x.tb ? encode_2d(context, &p, bf16, 2, x.b, x.n, x.k, x.ldb * 2, 64, 64)
                   : encode_2d(context, &p, bf16, 2, x.b, x.k, x.n, x.ldb * 2, 64, 128);
    ok = ok && (x.ta ? encode_2d(context, &q, bf16, 2, x.a, x.k, x.m, x.lda * 2, 64, bn / 2)
                     : encode_2d(context, &q, bf16, 2, x.a, x.m, x.k, x.lda * 2, 64, 64));
    if (packed) {
        ok = ok && encode_2d(context, &d0, bf16, 2, x.c, x.cut0, x.n, x.ldc * 2, 64, 32) &&
             encode_2d(context, &d1, bf16, 2, x.c1, x.cut1 - x.cut0, x.n, x.ldc1 * 2, 64, 32) &&
             encode_2d(context, &d2, bf16, 2, x.c2, x.m - x.cut1, x.n, x.ldc2 * 2, 64, 32);
    } else {
        ok = ok && encode_2d(context, &d0, bf16, 2, x.c, x.m, x.n, x.ldc * 2, 64, 32);
        d1 = d0, d2 = d0;
    }
    if (!ok)
        return fail(context, "tensor map encoding", 1);
    using namespace sm100;
    cudaError_t error;
    if (!x.tb && x.ta)
        error = launch_pair_width<kMajorK, kMajorK>(context, bn, pairs, p, q, d0, d1, d2, task);
    else if (!x.tb && !x.ta)
        error = launch_pair_width<kMajorK, kMajorMN>(context, bn, pairs, p, q, d0, d1, d2, task);
    else if (x.tb && x.ta)
        error = launch_pair_width<kMajorMN, kMajorK>(context, bn, pairs, p, q, d0, d1, d2, task);
    else
        error = launch_pair_width<kMajorMN, kMajorMN>(context, bn, pairs, p, q, d0, d1, d2, task);
    if (error != cudaSuccess)
        return fail(context, "two-SM tcgen05 BF16 GEMM", error);
    context->kernel_launches.fetch_add(1, std::memory_order_relaxed);
    if (task.sk_cols == 0)
        return 0;
    dim3 grid(task.sk_cols, 256 * bn / 8 / 256, task.r_blocks);
    if (bn == 256)
        sm100::sk_fixup_pair<256><<<grid, 256, 0, context->stream>>>(task, pairs, x.c1, x.ldc1,
                                                                     x.c2, x.ldc2);
    else
        sm100::sk_fixup_pair<128><<<grid, 256, 0, context->stream>>>(task, pairs, x.c1, x.ldc1,
                                                                     x.c2, x.ldc2);
    return launched(context, "stream-K fix-up");
}

/* out[rows, intermediate] = SiLU(x . Wg^T) * (x . Wu^T) in one pass over a weight
 * whose gate and up rows are interleaved in blocks of 128 (rows [256j, 256j+128)
 * gate features 128j.., rows [256j+128, 256j+256) the matching up features), so
 * that every 256-column tile of the two-SM kernel holds both halves of 128
 * outputs. Whole tiles apply SwiGLU in the epilogue; a stream-K tail does it in
 * its second pass. */
inline int run_gate_up_swiglu(camblas_cuda_context *context, int rows, int inner, int intermediate,
                              const __nv_bfloat16 *x, long long ldx, const __nv_bfloat16 *w,
                              long long ldw, __nv_bfloat16 *out, long long ldo,
                              uint8_t *quant_out = nullptr, float *quant_scale = nullptr)
{
    /* with quant_out the result leaves as E4M3 [rows, intermediate] plus FP32
     * scales [rows, intermediate / 128] and `out` is not written */
    const bool quantise = quant_out != nullptr;
    sm100::GemmTask task{};
    const int packed = 2 * intermediate;
    task.rows = rows, task.cols = packed, task.depth = inner;
    task.r_blocks = (rows + 255) / 256;
    task.c_blocks = packed / 256;
    task.k_blocks = (inner + 63) / 64;
    task.split = 1, task.k_blocks_per_split = task.k_blocks;
    task.alpha = 1.f, task.beta = 0.f;
    task.out = out, task.ld_out = ldo;
    task.status = context->status;
    task.cut0 = task.cut1 = packed;
    task.batch = 1;
    task.panel = task.r_blocks < 8 ? task.r_blocks : 8;
    task.quant_out = quant_out, task.ld_quant = intermediate;
    task.quant_scale = quant_scale, task.quant_groups = intermediate / 128;
    const int pairs_max = context->sm_count / 2;
    if (task.r_blocks <= 8 && pairs_max / task.r_blocks >= 2 && task.k_blocks >= 16) {
        /* the policy of run_tensor_pair for 256-column tiles */
        const int teams = pairs_max / task.r_blocks;
        const int rest = task.c_blocks % teams;
        const double tile = 2.0 * 256 * 256 * inner / (2 * 1.45e15 / 148.0 / 1e6);
        const double second_pass = 6.0 + double(rest + teams) * task.r_blocks * 256 * 256 * 8 / 5.0e6;
        if (rest != 0 && 2 * rest <= teams &&
            (double(task.c_blocks) / teams) * tile + second_pass <
                double((task.c_blocks + teams - 1) / teams) * tile) {
            task.dp_cols = task.c_blocks - rest, task.sk_cols = rest;
            int status = reserve_scratch(context, size_t(4) * pairs_max * 128 * 256 * sizeof(float));
            if (status != 0)
                return status;
            task.sk_partial = static_cast<float *>(context->scratch);
        }
    }
    const long long units = 1ll * task.r_blocks * task.c_blocks;
    const int pairs = (units < pairs_max && task.sk_cols == 0) ? int(units) : pairs_max;
    CUtensorMap p, q, d;
    const auto bf16 = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    bool ok = encode_2d(context, &p, bf16, 2, x, inner, rows, uint64_t(ldx) * 2, 64, 128) &&
              encode_2d(context, &q, bf16, 2, w, inner, packed, uint64_t(ldw) * 2, 64, 128);
    if (quantise)
        d = q; /* the kernel only prefetches its output map in this mode */
    else
        ok = ok && encode_2d(context, &d, bf16, 2, out, intermediate, rows, uint64_t(ldo) * 2, 64, 32);
    if (!ok)
        return fail(context, "tensor map encoding", 1);
    using namespace sm100;
    cudaError_t error =
        quantise ? launch_pair<256, 3, kMajorK, kMajorK, 2, kEpiSwigluQuant>(context, pairs, p, q, d,
                                                                         d, d, task)
                 : launch_pair<256, 3, kMajorK, kMajorK, 2, kEpiSwiglu>(context, pairs, p, q, d, d, d,
                                                                    task);
    if (error != cudaSuccess)
        return fail(context, "two-SM tcgen05 gate_up GEMM with SwiGLU", error);
    context->kernel_launches.fetch_add(1, std::memory_order_relaxed);
    if (task.sk_cols == 0)
        return 0;
    dim3 grid(task.sk_cols, 16, task.r_blocks);
    if (quantise)
        sm100::sk_fixup_pair_swiglu<true><<<grid, 256, 0, context->stream>>>(task, pairs);
    else
        sm100::sk_fixup_pair_swiglu<false><<<grid, 256, 0, context->stream>>>(task, pairs);
    return launched(context, "stream-K fix-up with SwiGLU");
}

inline int run_tensor_swapped(camblas_cuda_context *context, const Product &x)
{
    sm100::GemmTask task{};
    task.rows = x.m, task.cols = x.n, task.depth = x.k;
    task.r_blocks = (x.m + 127) / 128;
    int bn = x.n <= 16 ? 16 : (x.n <= 32 ? 32 : 64);
    task.c_blocks = (x.n + bn - 1) / bn;
    task.k_blocks = (x.k + 63) / 64;
    /* A few tiles more than whole waves (448 tiles of the Llama gate_up on 148 SMs:
     * three waves and four tiles) would leave all but those few SMs idle for a
     * whole tile's time, and splitting every tile's K to even that out costs a
     * pass over `split` copies of the result. The leftover output rows are
     * multiplied as a product of their own instead, which with so few tiles
     * splits its K over all SMs: 181 -> 156 us at 64 tokens, 159 -> 153 at 32, 154 -> 150
     * at 16. Up to eight tokens the partial sums are so small that splitting every
     * tile is cheaper than the two extra launches (144 against 148 us at two tokens). */
    const int sms = context->sm_count;
    const int leftover = task.c_blocks == 1 ? task.r_blocks % sms : 0;
    if (x.n > 8 && task.r_blocks > sms && leftover != 0 && 4 * leftover <= sms && task.k_blocks >= 32) {
        const int whole = (task.r_blocks - leftover) * 128; /* output features of the whole waves */
        Product head = x, tail = x;
        head.m = whole, head.cut0 = head.cut1 = whole;
        tail.m = x.m - whole, tail.cut0 = tail.cut1 = tail.m;
        tail.a = x.a + whole * x.lda; /* 'T' operand: a block of weight rows */
        tail.c = x.c + whole;
        if (x.addend != nullptr)
            tail.addend = x.addend + whole;
        if (x.bias != nullptr)
            tail.bias = x.bias + whole;
        int status = run_tensor_swapped(context, head);
        return status != 0 ? status : run_tensor_swapped(context, tail);
    }
    task.split = choose_split(task.r_blocks * task.c_blocks, task.k_blocks, context->sm_count);
    task.split = split_if_it_pays(task.split, task.r_blocks * task.c_blocks, task.k_blocks,
                                  context->sm_count, x.n, x.m, bn);
    /* where that estimate declines the split it had been offered, a smaller split may
     * still pay (64 tokens on a K/4 shard of the down projection: 64 tiles unsplit
     * 39.7 us, cut in two 27.9 us) */
    if (task.split == 1)
        task.split = cheapest_split(task.r_blocks * task.c_blocks, task.k_blocks, context->sm_count, x.n,
                                    x.m, bn);
    task.k_blocks_per_split = (task.k_blocks + task.split - 1) / task.split;
    task.split = (task.k_blocks + task.k_blocks_per_split - 1) / task.k_blocks_per_split;
    task.panel = task.r_blocks < 8 ? task.r_blocks : 8;
    task.alpha = x.alpha, task.beta = x.beta;
    task.out = x.c, task.ld_out = x.ldc;
    task.addend = x.addend, task.ld_add = x.ld_add;
    task.bias = x.bias;
    task.status = context->status;
    task.cut0 = task.cut1 = x.m;
    task.batch = 1;
    if (task.split > 1 && context->options.cluster_split == 2) {
        /* The split inside a cluster needs neither scratch nor a second launch, but
         * for few tokens the partial sums are small and the second launch is a
         * programmatic dependent: measured on the Llama down projection it is 1-3 %
         * slower than the scratch route (16 tokens 78.4 against 77.5 us), so it is
         * taken here only on request. */
        const int tiles = task.r_blocks * task.c_blocks;
        int parts = 0;
        if (bn == 16)
            parts = choose_cluster_parts<16, 8, sm100::kStoreColumns>(context, 2, tiles, task.k_blocks);
        else if (bn == 32)
            parts = choose_cluster_parts<32, 8, sm100::kStoreColumns>(context, 3, tiles, task.k_blocks);
        else
            parts = choose_cluster_parts<64, 8, sm100::kStoreColumns>(context, 4, tiles, task.k_blocks);
        if (parts >= 2) {
            task.split = 1, task.k_blocks_per_split = task.k_blocks;
            CUtensorMap p, q;
            const auto bf16 = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
            if (!encode_2d(context, &p, bf16, 2, x.a, x.k, x.m, x.lda * 2, 64, 128) ||
                !encode_2d(context, &q, bf16, 2, x.b, x.k, x.n, x.ldb * 2, 64, bn))
                return fail(context, "tensor map encoding", 1);
            if (bn == 16)
                return launch_cluster<16, 8, sm100::kStoreColumns>(context, tiles, parts, p, q, task);
            if (bn == 32)
                return launch_cluster<32, 8, sm100::kStoreColumns>(context, tiles, parts, p, q, task);
            return launch_cluster<64, 8, sm100::kStoreColumns>(context, tiles, parts, p, q, task);
        }
    }
    long long plane = 1ll * task.r_blocks * 128;
    if (task.split > 1) {
        size_t bytes = size_t(task.split) * x.n * plane * sizeof(float);
        int status = reserve_scratch(context, bytes);
        if (status != 0)
            return status;
        task.partial = static_cast<float *>(context->scratch);
    }
    CUtensorMap p, q;
    bool ok = encode_2d(context, &p, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x.a, x.k, x.m, x.lda * 2,
                        64, 128) &&
              encode_2d(context, &q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x.b, x.k, x.n, x.ldb * 2,
                        64, bn);
    if (!ok)
        return fail(context, "tensor map encoding", 1);
    if (task.split > 1) {
        if (bn == 16)
            launch_tensor<16, 8, sm100::kStorePartial>(context, p, q, p, p, p, task);
        else if (bn == 32)
            launch_tensor<32, 8, sm100::kStorePartial>(context, p, q, p, p, p, task);
        else
            launch_tensor<64, 8, sm100::kStorePartial>(context, p, q, p, p, p, task);
        int status = launched(context, "tcgen05 split-K BF16 GEMM");
        if (status != 0)
            return status;
        cudaError_t error = sm100::launch_split_reduce(context->stream, x.m, x.n, task.split, plane,
                                                       x.alpha, x.beta, task.partial, x.addend,
                                                       x.ld_add, x.bias, x.c, x.ldc);
        if (error != cudaSuccess)
            return fail(context, "split-K reduction", error);
        context->kernel_launches.fetch_add(1, std::memory_order_relaxed);
        return 0;
    }
    if (bn == 16)
        launch_tensor<16, 8, sm100::kStoreColumns>(context, p, q, p, p, p, task);
    else if (bn == 32)
        launch_tensor<32, 8, sm100::kStoreColumns>(context, p, q, p, p, p, task);
    else
        launch_tensor<64, 8, sm100::kStoreColumns>(context, p, q, p, p, p, task);
    return launched(context, "tcgen05 swapped BF16 GEMM");
}

template <int Tokens> int launch_skinny(camblas_cuda_context *context, skinny::Task &task)
{
    /* rows per warp: more rows amortise the token reads, fewer rows give more
     * CTAs; keep at least two CTAs per SM when the matrix allows it */
    int sms = context->sm_count;
    int rows_per_warp = 4;
    while (rows_per_warp > 1 &&
           (task.outputs + rows_per_warp * skinny::kWarps - 1) / (rows_per_warp * skinny::kWarps) <
               2 * sms)
        rows_per_warp >>= 1;
    int row_blocks =
        (task.outputs + rows_per_warp * skinny::kWarps - 1) / (rows_per_warp * skinny::kWarps);
    /* K split: slices of at most 4096 elements (the staged tokens must fit in
     * shared memory) and enough CTAs for four per SM */
    int split = (task.depth + 4095) / 4096;
    while (1ll * row_blocks * split < 2ll * sms && task.depth / (split * 2) >= 512)
        split *= 2;
    int per = ((task.depth + split - 1) / split + 7) & ~7;
    split = (task.depth + per - 1) / per;
    task.split = split, task.depth_per_split = per;
    if (split > 1) {
        size_t bytes = size_t(split) * task.tokens * task.outputs * sizeof(float);
        int status = reserve_scratch(context, bytes);
        if (status != 0)
            return status;
        task.partial = static_cast<float *>(context->scratch);
    }
    size_t shared = size_t(Tokens) * per * sizeof(__nv_bfloat16);
    dim3 grid(row_blocks, split);
    if (rows_per_warp == 4)
        skinny::skinny_gemv<Tokens, 4><<<grid, skinny::kThreads, shared, context->stream>>>(task);
    else if (rows_per_warp == 2)
        skinny::skinny_gemv<Tokens, 2><<<grid, skinny::kThreads, shared, context->stream>>>(task);
    else
        skinny::skinny_gemv<Tokens, 1><<<grid, skinny::kThreads, shared, context->stream>>>(task);
    int status = launched(context, "skinny BF16 GEMV");
    if (status != 0 || split == 1)
        return status;
    dim3 reduce_grid((task.outputs + 255) / 256, task.tokens);
    skinny::skinny_reduce<<<reduce_grid, 256, 0, context->stream>>>(task);
    return launched(context, "skinny split-K reduction");
}

inline int run_skinny(camblas_cuda_context *context, const Product &x)
{
    skinny::Task task{};
    task.outputs = x.m, task.tokens = x.n, task.depth = x.k;
    task.ldw = x.lda, task.ldx = x.ldb;
    task.alpha = x.alpha, task.beta = x.beta;
    task.w = x.a, task.x = x.b;
    task.out = x.c, task.ld_out = x.ldc;
    task.addend = x.addend, task.ld_add = x.ld_add;
    task.bias = x.bias;
    switch (x.n) {
    case 1:
        return launch_skinny<1>(context, task);
    case 2:
        return launch_skinny<2>(context, task);
    case 3:
    case 4:
        return launch_skinny<4>(context, task);
    }
    return fail(context, "skinny kernel token count", 1);
}

inline int run_generic(camblas_cuda_context *context, const Product &x)
{
    generic::Task task{};
    task.m = x.m, task.n = x.n, task.k = x.k;
    task.ta = x.ta, task.tb = x.tb;
    task.lda = x.lda, task.ldb = x.ldb, task.ldc = x.ldc;
    task.alpha = x.alpha, task.beta = x.beta;
    task.a = x.a, task.b = x.b, task.c = x.c;
    task.bias = x.bias, task.addend = x.addend, task.ld_add = x.ld_add;
    dim3 grid((x.m + 63) / 64, (x.n + 63) / 64);
    if (grid.y > 65535)
        return fail(context, "generic GEMM column count", 1);
    generic::gemm_bf16_generic<<<grid, 256, 0, context->stream>>>(task);
    return launched(context, "generic BF16 GEMM");
}

/* Route one product. Packed projections (cut0 < m) are split into three
 * products unless the tensor-core row store takes them in one launch. */
inline int run_product(camblas_cuda_context *context, const Product &x)
{
    bool packed = x.cut0 < x.m;
    bool tensor = tensor_operands_ok(x) && rows_store_ok(x);
    bool swapped = swapped_operands_ok(x);
    bool skinny_ok = x.ta && !x.tb && aligned16(x.a) && x.lda % 8 == 0 && x.n <= 4;
    int family = context->forced_family;
    if (family == kAuto) {
        /* one token streams best on CUDA cores; from two tokens on the swapped
         * tensor-core kernel stays at HBM speed while the FMA loop would not */
        if (skinny_ok && (x.n == 1 || !swapped))
            family = kSkinny;
        else if (swapped && x.n <= 64)
            family = kTensorSwapped;
        else if (tensor) {
            /* Two-SM tiles from 129 token rows on, except when there are so few of
             * them (at most 30 tiles of 256 x 256 for 74 CTA pairs, up to 1024 rows)
             * that the one-SM kernel's 128-row tiles and its stream-K teams spread
             * the work better: measured 5-9 % faster on such shapes. */
            const long long pair_tiles = ((x.n + 255) / 256) * ((x.m + 255) / 256);
            family = x.n <= 128 || (x.n <= 1024 && pair_tiles <= 30) ? kTensor : kTensorPair;
        }
        else
            family = kGeneric;
    } else {
        bool possible = family == kGeneric || (family == kSkinny && skinny_ok) ||
                        (family == kTensorSwapped && swapped) ||
                        ((family == kTensor || family == kTensorPair) && tensor);
        if (!possible)
            return fail(context, "forced kernel family cannot take these operands", 1);
    }
    /* One launch serves a packed projection only on the tensor-core row kernels and
     * only when the three outputs start on tile boundaries (multiples of 128
     * columns; of 16 with a forced run-time width); any other packed projection is
     * three independent products, each dispatched on its own, which is what the
     * reference computes (torch_bindings.cpp:725-736). */
    const bool cuts_on_tiles =
        (x.cut0 % 128 == 0 && x.cut1 % 128 == 0) ||
        (family == kTensorPair && context->options.pair_width != 0 && x.ta && x.m > 128 &&
         x.cut0 % 16 == 0 && x.cut1 % 16 == 0);
    if (packed && ((family != kTensor && family != kTensorPair) || !cuts_on_tiles)) {
        Product part = x;
        part.cut0 = part.cut1 = 0;
        const int starts[4] = {0, x.cut0, x.cut1, x.m};
        __nv_bfloat16 *outs[3] = {x.c, x.c1, x.c2};
        const long long lds[3] = {x.ldc, x.ldc1, x.ldc2};
        for (int i = 0; i < 3; ++i) {
            part.m = starts[i + 1] - starts[i];
            if (part.m == 0)
                continue;
            part.a = x.a + starts[i] * x.lda; /* 'T' operand: row block of the weight */
            part.c = outs[i], part.ldc = lds[i];
            part.cut0 = part.cut1 = part.m;
            part.addend = part.c, part.ld_add = part.ldc;
            int status = run_product(context, part);
            if (status != 0)
                return status;
        }
        return 0;
    }
    context->counts[context->algorithm == CAMBLAS_CUDA_LT ? 4 : 0]++;
    switch (family) {
    case kSkinny:
        return run_skinny(context, x);
    case kTensorSwapped:
        return run_tensor_swapped(context, x);
    case kTensor:
        return run_tensor_rows(context, x);
    case kTensorPair:
        return run_tensor_pair(context, x);
    default:
        return run_generic(context, x);
    }
}

} // namespace host
