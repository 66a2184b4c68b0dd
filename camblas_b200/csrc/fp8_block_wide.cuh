/*
 * FP8 E4M3 block-scaled GEMM for many token rows with 256-column tiles.
 *
 * What bounds the 128 x 128 tiles of fp8_block_rows is neither the operand feed
 * nor the promotion but the one thread that issues the MMAs. Measured on B200
 * with a stand-alone loop: a kind::f8f6f4 MMA of M = 128, N = 128, K = 32 keeps
 * the tensor pipe busy for 64 cycles, N = 256 for 128 cycles; issuing one costs
 * the thread some 55 cycles and every tcgen05.commit about 100 more, and the
 * pipe only stays busy while the thread runs ahead of it. A 128-deep K block of
 * a 128 x 128 tile is four 64-cycle MMAs, a commit for the accumulator and half
 * a commit for the stage, plus two barrier waits: about 600 cycles of issue for
 * 256 cycles of arithmetic (with the operand loads removed altogether the kernel
 * took the same 199 us; with the promotion removed, 185 us). So here every MMA
 * is N = 256 wide, a K block costs four of them and ONE commit, and the stage
 * is handed back to the producer by a promotion warp, not by a second commit:
 *
 *   Pair = false  one CTA per 128-row x 256-column tile.
 *   Pair = true   two CTAs of a cluster per 256-row x 256-column tile with
 *                 tcgen05.mma.cta_group::2: one thread issues for both SMs, the
 *                 commit arrives on both CTAs' barriers at once (multicast),
 *                 every CTA stages its own 128 token rows and 128 of the weight
 *                 rows: half the issue work and half the operand bytes per flop.
 *
 * The scales (FP32 per 1 x 128 activation block and per 128 x 128 weight block)
 * make every K block a fresh accumulation that is promoted in registers,
 *     acc = fma(block sum, a_scale[row, g] * w_scale[band, g], acc)   g ascending,
 * with one rounding at the end - the same arithmetic as fp8_block_rows, bit for
 * bit. Two 256-column accumulator buffers alternate, each with an issuing thread
 * of its own (warps 1 and 2: even and odd K blocks), because even this K block
 * costs one thread some 1 100 cycles (two barrier polls 500, four MMAs and a
 * commit 500) against 512 cycles of MMA. Eight promotion warps per CTA: two per
 * quarter of the tensor-memory lanes, one for each 128-column weight band of the
 * tile, 128 running sums per thread. They take 232 registers (setmaxnreg), which
 * the producer and issuer warps give up. The recurring waits poll without
 * suspending (mbarrier.test_wait) and a warp hands the buffer back as soon as
 * its second load has landed, before the additions. What is left (about 950
 * cycles per K block, 55 % of the pipe): the promotion warps are busy three
 * quarters of the time, their tensor-memory loads taking several times longer
 * next to running MMAs than alone.
 */
#pragma once

#include "fp8_block.cuh"
#include "gemm_bf16_pair.cuh"

namespace fp8
{

constexpr int kWideThreads = 384; /* warps 0-3: producer, MMA issuer, two spare; 4-11: promotion */
constexpr int kWideColumns = 256;
constexpr int kWideBuffers = 2;
constexpr int kWideScaleAhead = 4; /* K blocks whose scales are in flight ahead of the promotion */
constexpr int kWidePromotionRegisters = 232, kWideOtherRegisters = 40;

template <bool Pair> struct WideSmem {
    static constexpr int kStages = Pair ? 6 : 4;
    static constexpr int kPBytes = 128 * 128;                   /* 128 token rows x 128 B */
    static constexpr int kQBytes = (Pair ? 128 : 256) * 128;    /* this CTA's weight rows */
    static constexpr int kStageBytes = kPBytes + kQBytes;
    static constexpr int kStaging = 8 * 4096; /* one 32 x 64 BF16 slab per promotion warp */
    static constexpr int kTotal = kStages * kStageBytes + kStaging + 512 + 1024;
};

__device__ __forceinline__ void umma_f8_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                             uint32_t idesc, uint32_t accumulate)
{
    asm volatile("{\n"
                 ".reg .pred p;\n"
                 "setp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
                 "}\n" ::"r"(tmem_d),
                 "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
                 : "memory");
}

/* Arrival on a barrier of the other CTA that orders nothing but itself: the
 * tensor-memory loads it follows have completed (tcgen05.wait::ld), and a
 * release at cluster scope would wait for this warp's unrelated stores. */
__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint32_t cluster_address)
{
    asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_address)
                 : "memory");
}

template <int Registers> __device__ __forceinline__ void registers_grow()
{
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(Registers));
}

template <int Registers> __device__ __forceinline__ void registers_shrink()
{
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(Registers));
}

/* task: rows = token rows, cols = outputs, r_blocks counts tiles of 128 (256 in
 * the pair form) token rows, c_blocks tiles of 256 columns; p_scale per token
 * row, q_scale per 128-row weight band; split is 1. The pair form is launched in
 * clusters of two, one tile per cluster at a time. */
template <bool Pair>
__global__ void __launch_bounds__(kWideThreads, 1)
    fp8_block_wide(const __grid_constant__ CUtensorMap map_p,
                   const __grid_constant__ CUtensorMap map_q,
                   const __grid_constant__ CUtensorMap map_d, const BlockTask task)
{
    using namespace sm100;
    using Layout = WideSmem<Pair>;
    constexpr int kStages = Layout::kStages;
    constexpr int kTileRows = Pair ? 256 : 128;

    extern __shared__ uint8_t raw_smem[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) &
                                                ~static_cast<uintptr_t>(1023));
    uint8_t *staging = smem + kStages * Layout::kStageBytes;
    uint64_t *full = reinterpret_cast<uint64_t *>(staging + Layout::kStaging);
    uint64_t *empty = full + kStages;
    uint64_t *tmem_full = empty + kStages;
    uint64_t *tmem_empty = tmem_full + kWideBuffers;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tmem_empty + kWideBuffers);
    volatile uint32_t *abort = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint32_t rank = 0;
    if constexpr (Pair)
        rank = cluster_rank();
    const bool leader = rank == 0;
    const int worker = Pair ? int(blockIdx.x >> 1) : int(blockIdx.x);
    const int workers = Pair ? int(gridDim.x >> 1) : int(gridDim.x);
    const int tiles = task.r_blocks * task.c_blocks;
    const int groups = task.k_blocks;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int s = 0; s < kWideBuffers; ++s) {
            mbar_init(&tmem_full[s], 1);
            mbar_init(&tmem_empty[s], Pair ? 16 : 8); /* every promotion warp of every CTA */
        }
        *abort = 0;
        fence_barrier_init();
        prefetch_tensormap(&map_p);
        prefetch_tensormap(&map_q);
        prefetch_tensormap(&map_d);
    }
    if (warp == 1) {
        if constexpr (Pair) {
            tmem_alloc_pair(tmem_slot, 512);
            tmem_relinquish_pair();
        } else {
            tmem_alloc(tmem_slot, 512);
            tmem_relinquish();
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if constexpr (Pair)
        cluster_sync();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    /* tile -> (row block, column tile): column tiles in turn inside panels of row blocks */
    auto locate = [&](int tile, int &rb, int &cb) {
        const int per_panel = task.panel * task.c_blocks;
        const int panel = tile / per_panel;
        const int local = tile - panel * per_panel;
        const int height = min(task.panel, task.r_blocks - panel * task.panel);
        cb = local / height;
        rb = panel * task.panel + local - cb * height;
    };

    if (warp < 4) {
        registers_shrink<kWideOtherRegisters>();
        if (warp == 0 && lane == 0) {
            /* ---- producer ---- */
            const uint64_t keep = policy_evict_last();
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (int tile = worker; ok && tile < tiles; tile += workers) {
                int rb, cb;
                locate(tile, rb, cb);
                const int p_row = rb * kTileRows + int(rank) * 128;
                for (int kb = 0; kb < groups; ++kb) {
                    if (!mbar_wait(&empty[stage], phase ^ 1, abort)) {
                        report(task.status, abort, kRoleProducer);
                        ok = false;
                        break;
                    }
                    uint8_t *p_tile = smem + stage * Layout::kStageBytes;
                    uint8_t *q_tile = p_tile + Layout::kPBytes;
                    if constexpr (Pair) {
                        /* both CTAs' bytes are counted on the leader's barrier; of the
                         * tile's 256 weight rows this CTA stages 128 */
                        const uint32_t barrier = map_to_rank(smem_u32(&full[stage]), 0);
                        if (leader)
                            mbar_arrive_expect_tx(&full[stage], 2 * Layout::kStageBytes);
                        tma_load_2d_pair(p_tile, &map_p, barrier, kb * kBlockDepth, p_row, keep);
                        tma_load_2d_pair(q_tile, &map_q, barrier, kb * kBlockDepth,
                                         cb * kWideColumns + int(rank) * 128, keep);
                    } else {
                        mbar_arrive_expect_tx(&full[stage], Layout::kStageBytes);
                        tma_load_2d_hint(p_tile, &map_p, &full[stage], kb * kBlockDepth, p_row, keep);
                        for (int half = 0; half < 2; ++half)
                            tma_load_2d_hint(q_tile + half * 128 * 128, &map_q, &full[stage],
                                             kb * kBlockDepth, cb * kWideColumns + half * 128, keep);
                    }
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
            if (!ok) /* loads in flight must land before the CTA may leave */
                for (int wait = 0; wait < 64; ++wait)
                    __nanosleep(1000);
        } else if ((warp == 1 || warp == 2) && lane == 0 && leader) {
            /* ---- two MMA issuers: warp 1 takes the even K blocks (accumulator buffer
             * 0), warp 2 the odd ones (buffer 1). Timed inside the kernel, one thread
             * needs about 1 100 cycles per K block - two barrier polls (500), four
             * MMAs and a commit (500), the loop - against 512 cycles of MMA; with two
             * threads, each has two blocks' time for it. The blocks use different
             * accumulators and different operand stages, so their MMAs need no order
             * between them. */
            constexpr uint32_t idesc = make_idesc(0, kTileRows, kWideColumns, 0, 0); /* E4M3 x E4M3 */
            const uint32_t buffer = warp - 1;
            const uint32_t tmem_d = tmem_base + buffer * kWideColumns;
            const int total = ((tiles - worker + workers - 1) / workers) * groups;
            for (int block = int(buffer); block < total; block += 2) {
                const uint32_t use = uint32_t(block) >> 1;
                const uint32_t stage = uint32_t(block) % kStages, phase = (uint32_t(block) / kStages) & 1;
                if (!mbar_wait_polling(&tmem_empty[buffer], (use & 1) ^ 1, abort)) {
                    report(task.status, abort, kRoleMmaTmemEmpty);
                    break;
                }
                if (!mbar_wait_polling(&full[stage], phase, abort)) {
                    report(task.status, abort, kRoleMma);
                    break;
                }
                tcgen05_fence_after();
                const uint32_t p_address = smem_u32(smem + stage * Layout::kStageBytes);
                const uint64_t desc_p = desc_kmajor_sw128(p_address);
                const uint64_t desc_q = desc_kmajor_sw128(p_address + Layout::kPBytes);
                if constexpr (Pair) {
                    umma_f8_pair(tmem_d, desc_p, desc_q, idesc, 0u);
                    umma_f8_pair(tmem_d, desc_p + 2, desc_q + 2, idesc, 1u);
                    umma_f8_pair(tmem_d, desc_p + 4, desc_q + 4, idesc, 1u);
                    umma_f8_pair(tmem_d, desc_p + 6, desc_q + 6, idesc, 1u);
                    umma_commit_both(smem_u32(&tmem_full[buffer]));
                } else {
                    umma_f8(tmem_d, desc_p, desc_q, idesc, 0u);
                    umma_f8(tmem_d, desc_p + 2, desc_q + 2, idesc, 1u);
                    umma_f8(tmem_d, desc_p + 4, desc_q + 4, idesc, 1u);
                    umma_f8(tmem_d, desc_p + 6, desc_q + 6, idesc, 1u);
                    umma_commit(&tmem_full[buffer]);
                }
            }
        }
    } else {
        /* ---- promotion: 32 rows x one band of 128 columns per warp ---- */
        registers_grow<kWidePromotionRegisters>();
        const int quarter = warp & 3;     /* tensor-memory lanes 32*quarter .. +31 */
        const int half = (warp - 4) >> 2; /* columns 128*half .. +127 of the tile */
        uint8_t *slab = staging + (warp - 4) * 4096;
        uint32_t release = smem_u32(&tmem_empty[0]);
        if constexpr (Pair)
            release = map_to_rank(release, 0);
        uint32_t block = 0, stage = 0;
        bool ok = true;
        for (int tile = worker; ok && tile < tiles; tile += workers) {
            int rb, cb;
            locate(tile, rb, cb);
            const int row0 = rb * kTileRows + int(rank) * 128 + quarter * 32;
            const int row = row0 + lane;
            const int col0 = cb * kWideColumns + half * 128;
            const int band = min(2 * cb + half, (task.cols + 127) / 128 - 1);
            const float *row_scale =
                task.p_scale + static_cast<long long>(min(row, task.rows - 1)) * groups;
            const float *band_scale = task.q_scale + static_cast<long long>(band) * groups;
            float acc[128];
#pragma unroll
            for (int i = 0; i < 128; ++i)
                acc[i] = 0.f;
            /* the scales of the next kWideScaleAhead K blocks are in flight */
            float own[kWideScaleAhead], weight[kWideScaleAhead];
#pragma unroll
            for (int j = 0; j < kWideScaleAhead; ++j) {
                const int at = min(j, groups - 1);
                own[j] = row_scale[at];
                weight[j] = band_scale[at];
            }
            for (int kb_group = 0; ok && kb_group < groups; kb_group += kWideScaleAhead) {
#pragma unroll
                for (int j = 0; j < kWideScaleAhead; ++j) {
                    const int kb = kb_group + j;
                    if (kb >= groups)
                        break;
                    const uint32_t buffer = block & 1, use = block >> 1;
                    ++block;
                    const float scale = __fmul_rn(own[j], weight[j]);
                    if (kb + kWideScaleAhead < groups) {
                        own[j] = row_scale[kb + kWideScaleAhead];
                        weight[j] = band_scale[kb + kWideScaleAhead];
                    }
                    if (!mbar_wait_polling(&tmem_full[buffer], use & 1, abort)) {
                        report(task.status, abort, kRoleEpilogueFull);
                        ok = false;
                        break;
                    }
                    tcgen05_fence_after();
                    /* the block's MMAs are done, so its operand stage is free: the
                     * first promotion warp says so, which spares the issuer a commit */
                    if (warp == 4 && lane == 0)
                        mbar_arrive(&empty[stage]);
                    if (++stage == kStages)
                        stage = 0;
                    const uint32_t taddr = tmem_base + buffer * kWideColumns + half * 128 +
                                           (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll
                    for (int chunk = 0; chunk < 2; ++chunk) {
                        uint32_t piece[64];
                        tmem_ld_32x64(taddr + chunk * 64, piece);
                        tmem_ld_wait();
                        if (chunk == 1) {
                            /* the buffer is in registers: hand it back before the additions */
                            tcgen05_fence_before();
                            __syncwarp();
                            if (lane == 0) {
                                if constexpr (Pair)
                                    mbar_arrive_cluster_relaxed(release + buffer * 8);
                                else
                                    mbar_arrive(&tmem_empty[buffer]);
                            }
                        }
#pragma unroll
                        for (int i = 0; i < 64; ++i)
                            acc[chunk * 64 + i] =
                                fmaf(__uint_as_float(piece[i]), scale, acc[chunk * 64 + i]);
                    }
                }
            }
            if (!ok)
                break;
            if (col0 < task.cols && row0 < task.rows) {
                /* 32 rows x 128 columns: two swizzled 4 KB slabs, one TMA store each */
#pragma unroll
                for (int part = 0; part < 2; ++part) {
                    if (lane == 0)
                        tma_store_wait_read<0>();
                    __syncwarp();
                    const uint32_t base = smem_u32(slab) + lane * 128;
#pragma unroll
                    for (int piece = 0; piece < 8; ++piece) {
                        const float *v = acc + part * 64 + piece * 8;
                        st_shared_v4(base + ((piece ^ (lane & 7)) << 4), pack_bf16(v[0], v[1]),
                                     pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]),
                                     pack_bf16(v[6], v[7]));
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0 && col0 + part * 64 < task.cols) {
                        tma_store_2d(&map_d, slab, col0 + part * 64, row0);
                        tma_store_commit();
                    }
                }
            }
        }
        if (lane == 0)
            tma_store_wait_all<0>();
        __syncwarp();
    }

    tcgen05_fence_before();
    __syncthreads();
    if constexpr (Pair)
        cluster_sync();
    if (warp == 1) {
        tcgen05_fence_after();
        if constexpr (Pair)
            tmem_dealloc_pair(tmem_base, 512);
        else
            tmem_dealloc(tmem_base, 512);
    }
}

inline int prepare_wide_kernels()
{
    cudaError_t error = cudaFuncSetAttribute(fp8_block_wide<false>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             WideSmem<false>::kTotal);
    if (error == cudaSuccess)
        error = cudaFuncSetAttribute(fp8_block_wide<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     WideSmem<true>::kTotal);
    return int(error);
}

/* Many token rows on 256-column tiles; `pair` selects the two-SM form. */
inline int block_gemm_wide(camblas_cuda_context *context, bool pair, int rows, int outputs, int inner,
                           const void *q, const float *q_scale, const void *w, const float *w_scale,
                           void *out, int ldo)
{
    using host::encode_2d;
    const int tile_rows = pair ? 256 : 128;
    BlockTask task{};
    task.rows = rows, task.cols = outputs, task.depth = inner;
    task.r_blocks = (rows + tile_rows - 1) / tile_rows;
    task.c_blocks = (outputs + kWideColumns - 1) / kWideColumns;
    task.k_blocks = inner / 128;
    task.split = 1, task.k_blocks_per_split = task.k_blocks;
    task.panel = task.r_blocks < 8 ? task.r_blocks : 8;
    task.p_scale = q_scale, task.q_scale = w_scale;
    task.out = static_cast<__nv_bfloat16 *>(out);
    task.ld_out = ldo;
    task.status = context->status;
    CUtensorMap p, qm, d;
    const auto type = CU_TENSOR_MAP_DATA_TYPE_UINT8;
    bool ok = encode_2d(context, &p, type, 1, q, inner, rows, inner, 128, 128) &&
              encode_2d(context, &qm, type, 1, w, inner, outputs, inner, 128, 128) &&
              encode_2d(context, &d, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, out, outputs, rows,
                        size_t(ldo) * 2, 64, 32);
    if (!ok)
        return host::fail(context, "tensor map encoding", 1);
    const int tiles = task.r_blocks * task.c_blocks;
    cudaLaunchConfig_t config = {};
    config.blockDim = dim3(kWideThreads);
    config.stream = context->stream;
    cudaLaunchAttribute attribute[1];
    cudaError_t error;
    if (pair) {
        const int pairs = std::min(tiles, context->sm_count / 2);
        config.gridDim = dim3(2 * pairs);
        config.dynamicSmemBytes = WideSmem<true>::kTotal;
        attribute[0].id = cudaLaunchAttributeClusterDimension;
        attribute[0].val.clusterDim.x = 2;
        attribute[0].val.clusterDim.y = 1;
        attribute[0].val.clusterDim.z = 1;
        config.attrs = attribute;
        config.numAttrs = 1;
        error = cudaLaunchKernelEx(&config, fp8_block_wide<true>, p, qm, d, task);
    } else {
        config.gridDim = dim3(std::min(tiles, context->sm_count));
        config.dynamicSmemBytes = WideSmem<false>::kTotal;
        error = cudaLaunchKernelEx(&config, fp8_block_wide<false>, p, qm, d, task);
    }
    if (error != cudaSuccess)
        return host::fail(context, "tcgen05 FP8 block GEMM on 256-column tiles", error);
    context->kernel_launches.fetch_add(1, std::memory_order_relaxed);
    return 0;
}

} // namespace fp8
