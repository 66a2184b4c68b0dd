/*
 * FP8 E4M3 w8a8 kernels.
 *
 * 1. quantize_rows_kernel: BF16 rows -> E4M3 with one FP32 scale per 128
 *    elements (amax/448), the activation-quantise prologue.
 * 2. fp8_block_gemm: block-scaled GEMM on the tensor cores (tcgen05.mma
 *    kind::f8f6f4, FP32 accumulation in TMEM). The scales are FP32 amax/448
 *    values, one per 1x128 activation block and per 128x128 weight block, so
 *    they cannot ride on the hardware's E8M0 block-scaled MMA. Instead every
 *    128-deep K block is a fresh accumulation into one of two TMEM buffers and
 *    the epilogue warps promote it into FP32 registers while the next block is
 *    being multiplied: acc = fma(block, a_scale*w_scale, acc), blocks in
 *    ascending K order - the recurrence of the reference's block-128 decode
 *    kernel (camblas/_hopper.py:118-126, 168-182), applied to every row.
 *    For more than 128 token rows fp8_block_rows (eight promotion warps, four
 *    accumulator buffers) replaces the row mode of this kernel; what bounds
 *    it is written there.
 *    Store modes as in the BF16 kernel: token rows on TMEM lanes with a TMA
 *    store, or operands swapped for up to 128 tokens (64 per column block),
 *    optionally with a K split through FP32 scratch and an ordered reduction.
 * 3. fp8_token_kernel: the reference ABI's single-token block-32 product
 *    (src/cuda/fp8_decode.cuh:74-165) on CUDA cores: 16-byte weight loads,
 *    per-block FP32 dot products, then sum = fma(rnd(dot*sw), sx, sum) in
 *    ascending block order; optional power-of-two BF16->E4M3 quantiser first
 *    (fp8_decode.cuh:60-72).
 */
#pragma once

#include "context.cuh"
#include "dispatch_bf16.cuh"
#include "gemm_bf16_tcgen05.cuh"

#include <algorithm>
#include <cuda_fp8.h>

namespace fp8
{

using sm100::GemmSmem;
using sm100::kStoreColumns;
using sm100::kStorePartial;
using sm100::kStoreRows;

/* ---- 1. activation quantiser ------------------------------------------------ */

/* One warp per 128-element group; lane l owns elements 4l..4l+3. */
__global__ void __launch_bounds__(256) quantize_rows_kernel(int rows, int inner, long long ldx,
                                                            const __nv_bfloat16 *x, uint8_t *q,
                                                            float *scale)
{
    const int groups = inner >> 7;
    const long long total = static_cast<long long>(rows) * groups;
    const int lane = threadIdx.x & 31;
    for (long long group = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
         group < total; group += (static_cast<long long>(gridDim.x) * blockDim.x) >> 5) {
        const long long row = group / groups;
        const int g = static_cast<int>(group - row * groups);
        const __nv_bfloat16 *source = x + row * ldx + g * 128 + lane * 4;
        uint2 packed = *reinterpret_cast<const uint2 *>(source);
        float v[4] = {sm100::bf16_low(packed.x), sm100::bf16_high(packed.x),
                      sm100::bf16_low(packed.y), sm100::bf16_high(packed.y)};
        float local = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
        /* non-negative floats order like their bit patterns */
        float maximum = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(local)));
        maximum = fmaxf(maximum, 1e-10f);
        if (lane == 0)
            scale[group] = __fmul_rn(maximum, 1.0f / 448.0f);
        const float inverse = __fdiv_rn(448.0f, maximum);
        uint32_t bytes = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float value = fminf(fmaxf(__fmul_rn(v[i], inverse), -448.f), 448.f);
            bytes |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(value, __NV_SATFINITE, __NV_E4M3))
                     << (8 * i);
        }
        *reinterpret_cast<uint32_t *>(q + row * inner + g * 128 + lane * 4) = bytes;
    }
}

/* ---- 2. block-scaled tensor-core GEMM ---------------------------------------- */

struct BlockTask {
    int rows, cols, depth;  /* P rows, Q rows, K (multiple of 128) */
    int r_blocks, c_blocks; /* 128-row and BN-row tiles */
    int k_blocks;           /* K / 128 */
    int split, k_blocks_per_split;
    int panel;
    const float *p_scale, *q_scale; /* kStoreRows: P per row [rows][G], Q per band [ceil/128][G];
                                       swapped modes: P per band, Q per row */
    __nv_bfloat16 *out;
    long long ld_out;
    float *partial; /* kStorePartial: [split][cols][r_blocks*128] */
    unsigned *status;
};

constexpr int kBlockDepth = 128; /* bytes = E4M3 elements per stage row */
constexpr int kSwappedRowLimit = 128; /* most token rows the swapped (weight-streaming) modes take */

/* Swapped modes: every epilogue warp keeps the scale products a_scale * w_scale
 * of the next kScaleChunk K blocks for the BN token columns of its tile in a
 * table of its own ([block][column], rows padded by one float so that the
 * fill is free of bank conflicts). Fetching them block by block put an L2 round
 * trip (about a microsecond) in front of every 128-deep K block, which is all a
 * few-token tile costs otherwise. */
constexpr int kScaleChunk = 16;

/* Dynamic shared memory of fp8_block_gemm: the BF16 kernel's layout plus, in the
 * swapped modes, the scale tables of the four epilogue warps. */
template <int BN, int Stages, int Mode> constexpr int block_smem_bytes()
{
    return GemmSmem<BN, Stages, Mode>::kTotal + 256 +
           (Mode == kStoreRows ? 0 : 4 * kScaleChunk * (BN + 1) * 4);
}

template <int BN, int Stages, int Mode>
__global__ void __launch_bounds__(sm100::kThreads, 1)
    fp8_block_gemm(const __grid_constant__ CUtensorMap map_p,
                   const __grid_constant__ CUtensorMap map_q,
                   const __grid_constant__ CUtensorMap map_d, const BlockTask task)
{
    using namespace sm100;
    using Layout = GemmSmem<BN, Stages, Mode>; /* 128 B rows: same byte layout as BF16 x 64 */
    /* Accumulator buffers in tensor memory, one per K block in flight. The swapped
     * modes have narrow tiles and take eight, so that the MMA issuer runs up to
     * seven K blocks ahead of the promotion warps: with two, every 128-deep block
     * paid a round trip MMA -> barrier -> promotion warp -> barrier -> MMA, about a
     * microsecond for a multiplication of a few hundred cycles. */
    constexpr int kBuffers = Mode == kStoreRows ? 2 : 8;
    constexpr uint32_t kTmemColumns = BN * kBuffers < 32 ? 32 : BN * kBuffers;
    static_assert(kTmemColumns <= 512 && (kTmemColumns & (kTmemColumns - 1)) == 0, "TMEM size");
    static_assert(Mode != kStoreRows || BN == 128, "row store: one 128-column weight band per tile");

    extern __shared__ uint8_t raw_smem[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) &
                                                ~static_cast<uintptr_t>(1023));
    uint8_t *staging = smem + Stages * Layout::kStageBytes;
    uint64_t *full = reinterpret_cast<uint64_t *>(staging + Layout::kStaging);
    uint64_t *empty = full + Stages;
    uint64_t *tmem_full = empty + Stages;
    uint64_t *tmem_empty = tmem_full + kBuffers;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tmem_empty + kBuffers);
    volatile uint32_t *abort = tmem_slot + 1;
    static_assert((2 * Stages + 2 * kBuffers + 1) * 8 <= 512, "barrier area");
    /* swapped modes: the scale tables of the epilogue warps, behind the barrier area
     * (512 bytes: the 256 of the BF16 layout plus 256 counted in block_smem_bytes) */
    float *scale_area = reinterpret_cast<float *>(full) + 128;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int units = task.r_blocks * task.c_blocks * task.split;
    const int groups = task.k_blocks;
    if constexpr (Mode == kStorePartial) {
        /* the reduction that follows may become resident now; it waits for this
         * grid's completion itself (griddepcontrol.wait) */
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    }

    if (threadIdx.x == 0) {
        for (int s = 0; s < Stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int s = 0; s < kBuffers; ++s) {
            mbar_init(&tmem_full[s], 1);
            mbar_init(&tmem_empty[s], 4);
        }
        *abort = 0;
        fence_barrier_init();
        prefetch_tensormap(&map_p);
        prefetch_tensormap(&map_q);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, kTmemColumns);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    auto decode = [&](int unit, int &rb, int &cb, int &part) {
        part = unit % task.split;
        int tile = unit / task.split;
        int per_panel = task.panel * task.c_blocks;
        int panel = tile / per_panel;
        int local = tile - panel * per_panel;
        int height = min(task.panel, task.r_blocks - panel * task.panel);
        cb = local / height;
        rb = panel * task.panel + local - cb * height;
    };

    if (warp == 0) {
        if (lane == 0) {
            const uint64_t keep = policy_evict_last(), stream = policy_evict_first();
            const bool weights_are_q = Mode == kStoreRows;
            const uint64_t policy_p = weights_are_q ? keep : stream;
            const uint64_t policy_q = weights_are_q ? stream : keep;
            uint32_t stage = 0, phase = 0, armed = 0, armed_parity = 0;
            bool ok = true;
            for (int unit = blockIdx.x; ok && unit < units; unit += gridDim.x) {
                int rb, cb, part;
                decode(unit, rb, cb, part);
                int kb0 = part * task.k_blocks_per_split;
                int kb1 = min(task.k_blocks, kb0 + task.k_blocks_per_split);
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait(&empty[stage], phase ^ 1, abort)) {
                        report(task.status, abort, kRoleProducer);
                        ok = false;
                        break;
                    }
                    uint8_t *p_tile = smem + stage * Layout::kStageBytes;
                    mbar_arrive_expect_tx(&full[stage], Layout::kStageBytes);
                    tma_load_2d_hint(p_tile, &map_p, &full[stage], kb * kBlockDepth, rb * kBlockR,
                                     policy_p);
                    tma_load_2d_hint(p_tile + Layout::kPBytes, &map_q, &full[stage],
                                     kb * kBlockDepth, cb * BN, policy_q);
                    armed |= 1u << stage;
                    armed_parity = (armed_parity & ~(1u << stage)) | (phase << stage);
                    if (++stage == Stages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
            if (!ok)
                for (uint32_t s = 0; s < Stages; ++s)
                    if (armed & (1u << s))
                        for (uint32_t spin = 0; spin < (1u << 16); ++spin)
                            if (mbar_try_wait(&full[s], (armed_parity >> s) & 1))
                                break;
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(0, kBlockR, BN, 0, 0); /* E4M3 x E4M3 */
            uint32_t stage = 0, phase = 0, block = 0;
            bool ok = true;
            for (int unit = blockIdx.x; ok && unit < units; unit += gridDim.x) {
                int part = unit % task.split;
                int kb0 = part * task.k_blocks_per_split;
                int kb1 = min(task.k_blocks, kb0 + task.k_blocks_per_split);
                for (int kb = kb0; kb < kb1; ++kb, ++block) {
                    uint32_t buffer = block % kBuffers, use = block / kBuffers;
                    /* This one thread's instruction stream bounds the kernel when the
                     * tiles are narrow: it polls instead of suspending, and commits once
                     * per block; the stage goes back to the producer from the first
                     * promotion warp, which sees the same completion. */
                    if (!mbar_wait_polling(&tmem_empty[buffer], (use & 1) ^ 1, abort)) {
                        report(task.status, abort, kRoleMmaTmemEmpty);
                        ok = false;
                        break;
                    }
                    if (!mbar_wait_polling(&full[stage], phase, abort)) {
                        report(task.status, abort, kRoleMma);
                        ok = false;
                        break;
                    }
                    tcgen05_fence_after();
                    uint32_t p_address = smem_u32(smem + stage * Layout::kStageBytes);
                    uint64_t desc_p = desc_kmajor_sw128(p_address);
                    uint64_t desc_q = desc_kmajor_sw128(p_address + Layout::kPBytes);
                    uint32_t tmem_d = tmem_base + buffer * BN;
#pragma unroll
                    for (int k = 0; k < kBlockDepth / 32; ++k) /* 32 E4M3 = 32 bytes per MMA */
                        umma_f8(tmem_d, desc_p + 2 * k, desc_q + 2 * k, idesc, k > 0 ? 1u : 0u);
                    umma_commit(&tmem_full[buffer]);
                    if (++stage == Stages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
    } else {
        const int quarter = warp & 3;
        uint8_t *slab = staging + (warp - 2) * 8192;
        uint32_t block = 0, slab_use = 0;
        bool ok = true;
        for (int unit = blockIdx.x; ok && unit < units; unit += gridDim.x) {
            int rb, cb, part;
            decode(unit, rb, cb, part);
            const int kb0 = part * task.k_blocks_per_split;
            const int kb1 = min(task.k_blocks, kb0 + task.k_blocks_per_split);
            const int row = rb * kBlockR + quarter * 32 + lane;
            const int col0 = cb * BN;
            float acc[BN];
#pragma unroll
            for (int i = 0; i < BN; ++i)
                acc[i] = 0.f;
            /* scale sources: one value per thread (lane side) and one per tile or column */
            const float *lane_scale;
            if (Mode == kStoreRows)
                lane_scale = task.p_scale + static_cast<long long>(min(row, task.rows - 1)) * groups;
            else
                lane_scale = task.p_scale + static_cast<long long>(rb) * groups;
            float *const table = scale_area + (warp - 2) * kScaleChunk * (BN + 1);
            for (int kb = kb0; kb < kb1; ++kb, ++block) {
                const uint32_t buffer = block % kBuffers, use = block / kBuffers;
                float own = 0.f, band = 1.f;
                if (Mode == kStoreRows) {
                    own = lane_scale[kb];
                    band = task.q_scale[static_cast<long long>(cb) * groups + kb];
                }
                const int slot = (kb - kb0) % kScaleChunk;
                if (Mode != kStoreRows && slot == 0) {
                    /* Refill this warp's table with the products for blocks kb .. kb+count-1.
                     * Element e of the chunk is (column e / 16, block e % 16), so that
                     * neighbouring lanes fetch neighbouring floats of one scale row. A
                     * lane has sixteen loads in flight before it uses the first: issued one
                     * by one, each refill paid an L2 round trip per element. */
                    __syncwarp(); /* every lane is done with the previous chunk */
                    const int count = min(kScaleChunk, kb1 - kb);
                    constexpr int kInFlight = 16;
                    static_assert(kScaleChunk == 16, "element index split by shifts");
                    for (int e0 = lane; e0 < kScaleChunk * BN; e0 += 32 * kInFlight) {
                        float token_side[kInFlight], weight_side[kInFlight];
#pragma unroll
                        for (int u = 0; u < kInFlight; ++u) {
                            const int e = e0 + u * 32, i = e >> 4, j = e & 15;
                            if (e < kScaleChunk * BN && j < count) {
                                const int c = min(col0 + i, task.cols - 1);
                                token_side[u] =
                                    task.q_scale[static_cast<long long>(c) * groups + kb + j];
                                weight_side[u] = lane_scale[kb + j];
                            }
                        }
#pragma unroll
                        for (int u = 0; u < kInFlight; ++u) {
                            const int e = e0 + u * 32, i = e >> 4, j = e & 15;
                            if (e < kScaleChunk * BN && j < count)
                                table[j * (BN + 1) + i] = __fmul_rn(token_side[u], weight_side[u]);
                        }
                    }
                    __syncwarp();
                }
                const float *column_scale = table + slot * (BN + 1);
                if (!mbar_wait(&tmem_full[buffer], use & 1, abort)) {
                    report(task.status, abort, kRoleEpilogueFull);
                    ok = false;
                    break;
                }
                tcgen05_fence_after();
                /* the block's products are complete, so its operand stage is free */
                if (warp == 2 && lane == 0)
                    mbar_arrive(&empty[block % Stages]);
                const uint32_t taddr =
                    tmem_base + buffer * BN + (static_cast<uint32_t>(quarter * 32) << 16);
                constexpr int kPiece = BN >= 64 ? 64 : (BN >= 32 ? 32 : 16);
#pragma unroll
                for (int chunk = 0; chunk < BN / kPiece; ++chunk) {
                    uint32_t piece[kPiece];
                    if constexpr (kPiece == 64)
                        tmem_ld_32x64(taddr + chunk * kPiece, piece);
                    else if constexpr (kPiece == 32)
                        tmem_ld_32x32(taddr + chunk * kPiece, piece);
                    else
                        tmem_ld_32x16(taddr + chunk * kPiece, piece);
                    tmem_ld_wait();
                    if (chunk == BN / kPiece - 1) {
                        tcgen05_fence_before();
                        __syncwarp();
                        if (lane == 0)
                            mbar_arrive(&tmem_empty[buffer]);
                    }
                    if constexpr (Mode == kStoreRows) {
                        const float s = __fmul_rn(own, band);
#pragma unroll
                        for (int i = 0; i < kPiece; ++i)
                            acc[chunk * kPiece + i] =
                                fmaf(__uint_as_float(piece[i]), s, acc[chunk * kPiece + i]);
                    } else {
#pragma unroll
                        for (int i = 0; i < kPiece; ++i)
                            acc[chunk * kPiece + i] =
                                fmaf(__uint_as_float(piece[i]), column_scale[chunk * kPiece + i],
                                     acc[chunk * kPiece + i]);
                    }
                }
            }
            if (!ok)
                break;
            if constexpr (Mode == kStoreRows) {
#pragma unroll
                for (int chunk = 0; chunk < BN / 64; ++chunk) {
                    uint8_t *buffer_smem = slab + (slab_use & 1) * 4096;
                    if (lane == 0)
                        tma_store_wait_read<1>();
                    __syncwarp();
#pragma unroll
                    for (int piece = 0; piece < 8; ++piece) {
                        const float *v = acc + chunk * 64 + piece * 8;
                        uint4 packed;
                        packed.x = pack_bf16(v[0], v[1]);
                        packed.y = pack_bf16(v[2], v[3]);
                        packed.z = pack_bf16(v[4], v[5]);
                        packed.w = pack_bf16(v[6], v[7]);
                        *reinterpret_cast<uint4 *>(buffer_smem + lane * 128 +
                                                   ((piece ^ (lane & 7)) << 4)) = packed;
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_2d(&map_d, buffer_smem, col0 + chunk * 64,
                                     rb * kBlockR + quarter * 32);
                        tma_store_commit();
                    }
                    ++slab_use;
                }
            } else if constexpr (Mode == kStorePartial) {
                const long long plane = static_cast<long long>(task.r_blocks) * kBlockR;
                float *target =
                    task.partial + (static_cast<long long>(part) * task.cols + col0) * plane + row;
#pragma unroll
                for (int i = 0; i < BN; ++i)
                    if (col0 + i < task.cols)
                        target[i * plane] = acc[i];
            } else {
                if (row < task.rows) {
#pragma unroll
                    for (int i = 0; i < BN; ++i)
                        if (col0 + i < task.cols)
                            task.out[static_cast<long long>(col0 + i) * task.ld_out + row] =
                                __float2bfloat16_rn(acc[i]);
                }
            }
        }
        if constexpr (Mode == kStoreRows) {
            if (lane == 0)
                tma_store_wait_all<0>();
            __syncwarp();
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, kTmemColumns);
    }
}

/* ---- 2b. many token rows: eight promotion warps, four accumulator buffers ------ */

/* Row mode on 128 x 128 tiles, taken when 128 x 256 tiles (fp8_block_wide.cuh)
 * would leave SMs without one. Two warps share each quarter of the tensor-memory
 * lanes and take 64 columns each (64 accumulator registers, one 64-column load,
 * 64 FMAs per K block), so every scheduler has two promotion warps to
 * interleave, and the accumulator ring has four 128-column buffers (all 512
 * tensor-memory columns); a pipeline stage holds two K blocks. The arithmetic:
 * acc = fma(block sum, a_scale * w_scale, acc) in ascending K order, one
 * rounding at the end; every form of the kernel gives the same bits.
 *
 * What bounds it is the instruction stream of the thread that issues the MMAs,
 * not the operand feed and not the promotion (with the loads removed the kernel
 * took the same time, with the promotion removed 7 % less): issuing an MMA
 * costs the thread some 55-100 cycles and a commit about 100, against 64 cycles
 * that an M = 128, N = 128, K = 32 MMA occupies the pipe. Hence: the stage is
 * handed back by a promotion warp instead of a second commit, the recurring
 * waits poll without suspending, and two threads issue (even and odd K blocks,
 * buffers 0/2 and 1/3): 185 -> 146 us at 4096 x 4096 x 7168. */
constexpr int kRowsThreads = 352; /* producer, MMA issuer, eight promotion warps, second issuer */
constexpr int kRowsBuffers = 4;

constexpr int kRowsInboxPitch = 128 + sm100::kInboxPad; /* floats per row of the cluster form's inbox */

template <int Stages, int Sub = 1, bool Cluster = false> struct RowsSmem {
    static constexpr int kBlockBytes = 2 * 128 * 128;    /* 128 rows x 128 B of each operand */
    static constexpr int kStageBytes = Sub * kBlockBytes; /* Sub K blocks per stage */
    /* one 32 x 128 B slab per promotion warp; in the cluster form the inbox instead:
     * FP32 [K range][owned row][pitch], at most 128 + 7 rows in all */
    static constexpr int kStaging =
        Cluster ? ((128 + 8) * kRowsInboxPitch * 4 + 1023) / 1024 * 1024 : 8 * 4096;
    static constexpr int kTotal = Stages * kStageBytes + kStaging + 256 + 1024;
};

template <int Stages, int Sub = 1, bool Cluster = false>
__global__ void __launch_bounds__(kRowsThreads, 1)
    fp8_block_rows(const __grid_constant__ CUtensorMap map_p,
                   const __grid_constant__ CUtensorMap map_q,
                   const __grid_constant__ CUtensorMap map_d, const BlockTask task)
{
    using namespace sm100;
    using Layout = RowsSmem<Stages, Sub, Cluster>;
    constexpr int BN = 128;
    constexpr uint32_t kTmemColumns = kRowsBuffers * BN;

    extern __shared__ uint8_t raw_smem[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) &
                                                ~static_cast<uintptr_t>(1023));
    uint8_t *staging = smem + Stages * Layout::kStageBytes;
    uint64_t *full = reinterpret_cast<uint64_t *>(staging + Layout::kStaging);
    uint64_t *empty = full + Stages;
    uint64_t *tmem_full = empty + Stages;
    uint64_t *tmem_empty = tmem_full + kRowsBuffers;
    uint64_t *inbox_full = tmem_empty + kRowsBuffers; /* Cluster: every warp of every CTA delivered */
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(inbox_full + 1);
    volatile uint32_t *abort = tmem_slot + 1;
    /* Cluster: FP32 sums delivered by the CTAs of the cluster, [K range][owned row][kPitch];
     * memory of its own, so a CTA that is done early delivers while the others multiply */
    constexpr int kPitch = kRowsInboxPitch;
    float *inbox = reinterpret_cast<float *>(staging);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    bool cluster_waited = false; /* Cluster: this thread has waited on the set-up barrier */
    /* a unit is a tile, or one of `split` contiguous K ranges of a tile when the
     * tiles alone would leave most SMs idle; consecutive units are the K ranges
     * of one tile. Cluster: the grid has one CTA per unit and a cluster is the
     * `split` units of one tile. */
    const int units = task.r_blocks * task.c_blocks * task.split;
    const int groups = task.k_blocks;
    if (!Cluster && task.split > 1) {
        /* the reduction over the K ranges may become resident now; it waits for
         * this grid's completion itself */
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    }

    if (threadIdx.x == 0) {
        for (int s = 0; s < Stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int s = 0; s < kRowsBuffers; ++s) {
            mbar_init(&tmem_full[s], 1);
            mbar_init(&tmem_empty[s], 8);
        }
        if (Cluster) {
            /* completed by the bytes of the bulk copies alone: every CTA of the
             * cluster sends all the rows this one owns, 512 bytes each */
            const int parts = task.split, part = static_cast<int>(cluster_rank());
            const int owned = cluster_first_row(part + 1, parts) - cluster_first_row(part, parts);
            mbar_init(inbox_full, 1);
            mbar_arrive_expect_tx(inbox_full, uint32_t(owned) * 512u * uint32_t(parts));
        }
        *abort = 0;
        fence_barrier_init();
        prefetch_tensormap(&map_p);
        prefetch_tensormap(&map_q);
        prefetch_tensormap(&map_d);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, kTmemColumns);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    /* every CTA's inbox barrier must exist before a remote arrival: arrive here, wait
     * only in front of the first remote access, after the multiplication */
    if (Cluster)
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    auto range = [&](int unit, int &kb0, int &kb1) {
        const int part = unit % task.split;
        kb0 = part * task.k_blocks_per_split;
        kb1 = min(groups, kb0 + task.k_blocks_per_split);
    };
    auto decode = [&](int unit, int &rb, int &cb) {
        const int tile = unit / task.split;
        int per_panel = task.panel * task.c_blocks;
        int panel = tile / per_panel;
        int local = tile - panel * per_panel;
        int height = min(task.panel, task.r_blocks - panel * task.panel);
        cb = local / height;
        rb = panel * task.panel + local - cb * height;
    };

    if (warp == 0) {
        if (lane == 0) {
            /* activations are re-read by every column tile, weights by the row
             * tiles of one panel: keep both in L2 */
            const uint64_t keep = policy_evict_last();
            uint32_t stage = 0, phase = 0, armed = 0, armed_parity = 0;
            bool ok = true;
            for (int unit = blockIdx.x; ok && unit < units; unit += gridDim.x) {
                int rb, cb, kb0, kb1;
                decode(unit, rb, cb);
                range(unit, kb0, kb1);
                for (int kb = kb0; kb < kb1; kb += Sub) {
                    if (!mbar_wait(&empty[stage], phase ^ 1, abort)) {
                        report(task.status, abort, kRoleProducer);
                        ok = false;
                        break;
                    }
                    /* a stage holds up to Sub K blocks; the last of a range may hold fewer */
                    const int blocks = min(Sub, kb1 - kb);
                    mbar_arrive_expect_tx(&full[stage], blocks * Layout::kBlockBytes);
                    for (int sub = 0; sub < blocks; ++sub) {
                        uint8_t *p_tile =
                            smem + stage * Layout::kStageBytes + sub * Layout::kBlockBytes;
                        tma_load_2d_hint(p_tile, &map_p, &full[stage], (kb + sub) * kBlockDepth,
                                         rb * kBlockR, keep);
                        tma_load_2d_hint(p_tile + 128 * 128, &map_q, &full[stage],
                                         (kb + sub) * kBlockDepth, cb * BN, keep);
                    }
                    armed |= 1u << stage;
                    armed_parity = (armed_parity & ~(1u << stage)) | (phase << stage);
                    if (++stage == Stages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
            if (!ok)
                for (uint32_t s = 0; s < Stages; ++s)
                    if (armed & (1u << s))
                        for (uint32_t spin = 0; spin < (1u << 16); ++spin)
                            if (mbar_try_wait(&full[s], (armed_parity >> s) & 1))
                                break;
        }
    } else if (warp == 1 || warp == 10) {
        if (lane == 0) {
            /* Two issuing threads, the even K blocks on warp 1 and the odd ones on warp
             * 10: four 64-cycle MMAs, a commit and two barrier polls cost one thread
             * several times the 256 cycles the MMAs take (fp8_block_wide.cuh). The
             * blocks go to different accumulator buffers, so they need no order. */
            const uint32_t mine = warp == 1 ? 0u : 1u;
            constexpr uint32_t idesc = make_idesc(0, kBlockR, BN, 0, 0); /* E4M3 x E4M3 */
            uint32_t stage = 0, phase = 0, block = 0;
            bool ok = true;
            for (int unit = blockIdx.x; ok && unit < units; unit += gridDim.x) {
                int kb0, kb1;
                range(unit, kb0, kb1);
                for (int kb = kb0; ok && kb < kb1; kb += Sub) {
                    if (!mbar_wait(&full[stage], phase, abort)) {
                        report(task.status, abort, kRoleMma);
                        ok = false;
                        break;
                    }
                    const int blocks = min(Sub, kb1 - kb);
                    for (int sub = 0; sub < blocks; ++sub, ++block) {
                        if ((block & 1u) != mine)
                            continue;
                        const uint32_t buffer = block % kRowsBuffers, use = block / kRowsBuffers;
                        if (!mbar_wait_polling(&tmem_empty[buffer], (use & 1) ^ 1, abort)) {
                            report(task.status, abort, kRoleMmaTmemEmpty);
                            ok = false;
                            break;
                        }
                        tcgen05_fence_after();
                        const uint32_t p_address = smem_u32(smem + stage * Layout::kStageBytes +
                                                            sub * Layout::kBlockBytes);
                        const uint64_t desc_p = desc_kmajor_sw128(p_address);
                        const uint64_t desc_q = desc_kmajor_sw128(p_address + 128 * 128);
                        const uint32_t tmem_d = tmem_base + buffer * BN;
#pragma unroll
                        for (int k = 0; k < kBlockDepth / 32; ++k) /* 32 E4M3 = 32 bytes per MMA */
                            umma_f8(tmem_d, desc_p + 2 * k, desc_q + 2 * k, idesc, k > 0 ? 1u : 0u);
                        umma_commit(&tmem_full[buffer]);
                    }
                    if (!ok)
                        break;
                    /* no commit for the stage: the first promotion warp hands it back
                     * once it has seen the stage's last block complete (a commit
                     * costs this thread about a hundred cycles, and this thread's
                     * instruction stream is what the tensor pipe waits for) */
                    if (++stage == Stages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
    } else {
        const int quarter = warp & 3;       /* tensor-memory lanes 32*quarter .. +31 */
        const int half = (warp - 2) >> 2;   /* columns 64*half .. +63 of the tile */
        uint8_t *slab = staging + (warp - 2) * 4096;
        uint32_t block = 0, stage = 0;
        for (int unit = blockIdx.x; unit < units; unit += gridDim.x) {
            int rb, cb, kb0, kb1;
            decode(unit, rb, cb);
            range(unit, kb0, kb1);
            const int row = rb * kBlockR + quarter * 32 + lane;
            float acc[64];
#pragma unroll
            for (int i = 0; i < 64; ++i)
                acc[i] = 0.f;
            const float *lane_scale =
                task.p_scale + static_cast<long long>(min(row, task.rows - 1)) * groups;
            const float *band_scale = task.q_scale + static_cast<long long>(cb) * groups;
            float own = lane_scale[kb0], band = band_scale[kb0];
            bool ok = true;
            for (int kb = kb0; kb < kb1; ++kb, ++block) {
                const uint32_t buffer = block % kRowsBuffers, use = block / kRowsBuffers;
                const float s = __fmul_rn(own, band);
                if (kb + 1 < kb1) { /* next block's scales travel while this one is added */
                    own = lane_scale[kb + 1];
                    band = band_scale[kb + 1];
                }
                if (!mbar_wait_polling(&tmem_full[buffer], use & 1, abort)) {
                    report(task.status, abort, kRoleEpilogueFull);
                    ok = false;
                    break;
                }
                tcgen05_fence_after();
                /* the last block of a stage is done: its operands may be overwritten */
                if (((kb - kb0) % Sub) == Sub - 1 || kb == kb1 - 1) {
                    if (warp == 2 && lane == 0)
                        mbar_arrive(&empty[stage]);
                    if (++stage == Stages)
                        stage = 0;
                }
                uint32_t piece[64];
                tmem_ld_32x64(tmem_base + buffer * BN + half * 64 +
                                  (static_cast<uint32_t>(quarter * 32) << 16),
                              piece);
                tmem_ld_wait();
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0)
                    mbar_arrive(&tmem_empty[buffer]);
#pragma unroll
                for (int i = 0; i < 64; ++i)
                    acc[i] = fmaf(__uint_as_float(piece[i]), s, acc[i]);
            }
            if (!ok)
                break;
            if constexpr (Cluster) {
                /* The K ranges of this tile sit in the CTAs of this cluster. Each thread
                 * puts its row of 64 sums into this CTA's operand ring (idle: the thread
                 * has seen the last block complete) and sends it with one bulk copy
                 * through distributed shared memory to the CTA that owns the row (tile
                 * row i belongs to CTA i * parts / 128), slot `part` of its inbox; the
                 * copy's bytes complete the owner's barrier. Stores of 16 bytes per
                 * lane straight into the other CTA took 2.6 us for the 64 KB of a CTA
                 * and their fence 1.1 us more. The owner adds the slots in K-range
                 * order, as fp8_rows_reduce does, so the bits are those of the
                 * two-launch form with the same ranges. The cluster barrier below was
                 * arrived at by every thread of the cluster during set-up, so it cannot
                 * hang; the wait for the bytes is bounded. */
                const int parts = task.split, part = unit % parts;
                const int rows_owned_max = (kBlockR + parts - 1) / parts;
                asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
                cluster_waited = true;
                {
                    const int tile_row = quarter * 32 + lane;
                    const int owner = (tile_row * parts) / kBlockR;
                    const int local_row = tile_row - cluster_first_row(owner, parts);
                    /* 272-byte pitch: 16-byte aligned rows, no bank conflicts between lanes */
                    const uint32_t mine = smem_u32(smem) + ((warp - 2) * 32 + lane) * 272;
#pragma unroll
                    for (int i = 0; i < 64; i += 4)
                        st_shared_v4(mine + i * 4, __float_as_uint(acc[i]), __float_as_uint(acc[i + 1]),
                                     __float_as_uint(acc[i + 2]), __float_as_uint(acc[i + 3]));
                    fence_proxy_async_smem();
                    const uint32_t target = map_to_rank(
                        smem_u32(inbox + (part * rows_owned_max + local_row) * kPitch + half * 64),
                        owner);
                    const uint32_t barrier = map_to_rank(smem_u32(inbox_full), owner);
                    asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes "
                                 "[%0], [%1], 256, [%2];" ::"r"(target),
                                 "r"(mine), "r"(barrier)
                                 : "memory");
                }
                if (!mbar_wait(inbox_full, 0, abort)) {
                    report(task.status, abort, kRoleDrain);
                    break;
                }
                const int first = cluster_first_row(part, parts);
                const int owned = cluster_first_row(part + 1, parts) - first;
                const int thread = (warp - 2) * 32 + lane; /* 0..255 */
                constexpr int kVectors = BN / 8;
                for (int item = thread; item < owned * kVectors; item += 256) {
                    const int local_row = item / kVectors, c8 = (item - local_row * kVectors) * 8;
                    const int out_row = rb * kBlockR + first + local_row, col = cb * BN + c8;
                    if (out_row >= task.rows || col >= task.cols)
                        continue;
                    float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                    for (int s = 0; s < parts; ++s) {
                        const float4 *source = reinterpret_cast<const float4 *>(
                            inbox + (s * rows_owned_max + local_row) * kPitch + c8);
                        const float4 low = source[0], high = source[1];
                        sum[0] += low.x, sum[1] += low.y, sum[2] += low.z, sum[3] += low.w;
                        sum[4] += high.x, sum[5] += high.y, sum[6] += high.z, sum[7] += high.w;
                    }
                    /* the row tiling is only taken with a 16-byte aligned output whose
                     * width and pitch are multiples of eight */
                    uint4 packed;
                    packed.x = pack_bf16(sum[0], sum[1]);
                    packed.y = pack_bf16(sum[2], sum[3]);
                    packed.z = pack_bf16(sum[4], sum[5]);
                    packed.w = pack_bf16(sum[6], sum[7]);
                    *reinterpret_cast<uint4 *>(task.out + static_cast<long long>(out_row) * task.ld_out +
                                               col) = packed;
                }
                continue;
            } else if (task.split > 1) {
                /* FP32 sums of this K range: [range][row][column], 256 contiguous
                 * bytes per thread; fp8_rows_reduce adds the ranges in order */
                if (row < task.rows) {
                    float *target = task.partial +
                                    (static_cast<long long>(unit % task.split) * task.rows + row) *
                                        task.cols +
                                    cb * BN + half * 64;
#pragma unroll
                    for (int i = 0; i < 64; i += 4)
                        if (cb * BN + half * 64 + i < task.cols)
                            *reinterpret_cast<float4 *>(target + i) =
                                make_float4(acc[i], acc[i + 1], acc[i + 2], acc[i + 3]);
                }
                continue;
            }
            /* this warp's 32 rows x 64 columns: one swizzled 4 KB slab, one TMA store */
            if (lane == 0)
                tma_store_wait_read<0>();
            __syncwarp();
            const uint32_t base = smem_u32(slab) + lane * 128;
#pragma unroll
            for (int piece = 0; piece < 8; ++piece) {
                const float *v = acc + piece * 8;
                st_shared_v4(base + ((piece ^ (lane & 7)) << 4), pack_bf16(v[0], v[1]),
                             pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                tma_store_2d(&map_d, slab, cb * BN + half * 64, rb * kBlockR + quarter * 32);
                tma_store_commit();
            }
        }
        if (lane == 0)
            tma_store_wait_all<0>();
        __syncwarp();
    }

    tcgen05_fence_before();
    __syncthreads();
    if (Cluster) {
        /* The copies out of this CTA's shared memory are known to be complete only
         * when their owners' barriers are: no CTA leaves before every CTA is past
         * its inbox. Every thread of the cluster gets here, whatever gave up before. */
        if (!cluster_waited)
            asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
        asm volatile("barrier.cluster.arrive.release;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
    }
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, kTmemColumns);
    }
}

/* out[row][column] = rnd(sum over the K ranges, in order, of partial[range][row][column]);
 * four columns per thread (cols is a multiple of eight). Launched as a
 * programmatic dependent of fp8_block_rows. */
__global__ void __launch_bounds__(256)
    fp8_rows_reduce(int rows, int cols, int split, const float *partial, __nv_bfloat16 *out,
                    long long ld_out)
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const long long quads = static_cast<long long>(rows) * (cols >> 2);
    const long long plane = static_cast<long long>(rows) * cols;
    for (long long quad = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; quad < quads;
         quad += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long row = quad / (cols >> 2);
        const int column = static_cast<int>(quad - row * (cols >> 2)) << 2;
        const float *source = partial + row * cols + column;
        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s0 = 0; s0 < split; s0 += 8) {
            float4 v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (s0 + i < split)
                    v[i] = __ldcg(reinterpret_cast<const float4 *>(source + (s0 + i) * plane));
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (s0 + i < split)
                    sum.x += v[i].x, sum.y += v[i].y, sum.z += v[i].z, sum.w += v[i].w;
        }
        uint2 packed;
        packed.x = sm100::pack_bf16(sum.x, sum.y);
        packed.y = sm100::pack_bf16(sum.z, sum.w);
        *reinterpret_cast<uint2 *>(out + row * ld_out + column) = packed;
    }
}

/* ---- 3. single token, block-32 scales (reference ABI) ------------------------- */

__device__ __forceinline__ float e4m3_to_float(uint32_t byte)
{
    __half_raw half = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(byte), __NV_E4M3);
    return __half2float(*reinterpret_cast<__half *>(&half));
}

/* Power-of-two block-32 quantiser of one BF16 token; one warp per block
 * (arithmetic of fp8_decode.cuh:60-72). */
__device__ __forceinline__ uint8_t quantise_pow2(float value, float &scale)
{
    unsigned magnitude = __float_as_uint(fmaxf(fabsf(value), 1.e-10f));
    float maximum = __uint_as_float(__reduce_max_sync(0xffffffffu, magnitude));
    unsigned bits = __float_as_uint(__fmul_rn(maximum, 1.f / 448.f));
    int exponent = int((bits >> 23) & 255) - 127 + int((bits & 0x7fffff) != 0);
    scale = __uint_as_float(unsigned(exponent + 127) << 23);
    float multiplier = __uint_as_float(unsigned(127 - exponent) << 23);
    return __nv_cvt_float_to_fp8(fminf(__fmul_rn(value, multiplier), 448.f), __NV_SATFINITE,
                                 __NV_E4M3);
}

/* One warp per output row. Lane l owns the 16 bytes [16l, 16l+16) of every
 * 512-byte stretch of the row, so two neighbouring lanes hold one 32-element
 * block; after each stretch the sixteen block sums are folded into the running
 * sum in block order by every lane alike. */
template <bool Quantise>
__global__ void __launch_bounds__(256)
    fp8_token_kernel(int outputs, int inner, const void *input, const float *sx, int sx_stride,
                     const uint8_t *w, const float *sw, int sw_row, int sw_col,
                     __nv_bfloat16 *out)
{
    extern __shared__ __align__(16) uint8_t shared[];
    uint8_t *xq = shared;                                       /* [inner] */
    float *xs = reinterpret_cast<float *>(shared + inner);      /* [inner/32] */
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int groups = inner >> 5;
    if (Quantise) {
        const __nv_bfloat16 *x = static_cast<const __nv_bfloat16 *>(input);
        for (int g = warp; g < groups; g += 8) {
            float scale;
            uint8_t byte = quantise_pow2(__bfloat162float(x[g * 32 + lane]), scale);
            xq[g * 32 + lane] = byte;
            if (lane == 0)
                xs[g] = scale;
        }
    } else {
        const uint8_t *x = static_cast<const uint8_t *>(input);
        for (int i = threadIdx.x; i < inner; i += 256)
            xq[i] = x[i];
        for (int g = threadIdx.x; g < groups; g += 256)
            xs[g] = sx[static_cast<long long>(g) * sx_stride];
    }
    __syncthreads();
    const int row = blockIdx.x * 8 + warp;
    if (row >= outputs)
        return;
    const uint8_t *weights = w + static_cast<long long>(row) * inner;
    const float *row_scale = sw + static_cast<long long>(row >> 5) * sw_row;
    float sum = 0.f;
    for (int base = 0; base < inner; base += 512) {
        const int offset = base + lane * 16;
        float dot = 0.f;
        if (offset < inner) {
            /* inner is a multiple of 32, so a lane's 16 bytes are all inside or all outside */
            uint4 wv, xv = *reinterpret_cast<const uint4 *>(xq + offset);
            if ((reinterpret_cast<uintptr_t>(weights + offset) & 15) == 0) {
                wv = *reinterpret_cast<const uint4 *>(weights + offset);
            } else {
                const uint32_t *words = reinterpret_cast<const uint32_t *>(weights + offset);
                wv = make_uint4(words[0], words[1], words[2], words[3]);
            }
            const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w}, xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int b = 0; b < 4; ++b)
                    dot = fmaf(e4m3_to_float((ww[i] >> (8 * b)) & 255),
                               e4m3_to_float((xw[i] >> (8 * b)) & 255), dot);
        }
        dot += __shfl_xor_sync(0xffffffffu, dot, 1);
        const int g = (base >> 5) + (lane >> 1);
        float scaled = 0.f, xscale = 0.f;
        if (g < groups) {
            scaled = __fmul_rn(dot, row_scale[static_cast<long long>(g) * sw_col]);
            xscale = xs[g];
        }
        const int live = min(16, groups - (base >> 5));
        for (int j = 0; j < live; ++j)
            sum = fmaf(__shfl_sync(0xffffffffu, scaled, 2 * j),
                       __shfl_sync(0xffffffffu, xscale, 2 * j), sum);
    }
    if (lane == 0)
        out[row] = __float2bfloat16_rn(sum);
}

/* ---- host side ----------------------------------------------------------------- */

template <int BN, int Stages, int Mode> int prepare_kernel()
{
    return int(cudaFuncSetAttribute(fp8_block_gemm<BN, Stages, Mode>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    block_smem_bytes<BN, Stages, Mode>()));
}

inline int prepare_kernels()
{
    int status = prepare_kernel<128, 6, kStoreRows>();
    status |= int(cudaFuncSetAttribute(fp8_block_rows<6>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       RowsSmem<6>::kTotal));
    status |= int(cudaFuncSetAttribute(fp8_block_rows<3, 2>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       RowsSmem<3, 2>::kTotal));
    status |= int(cudaFuncSetAttribute(fp8_block_rows<4, 1, true>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       RowsSmem<4, 1, true>::kTotal));

    status |= prepare_kernel<16, 8, kStoreColumns>();
    status |= prepare_kernel<32, 8, kStoreColumns>();
    status |= prepare_kernel<64, 8, kStoreColumns>();
    status |= prepare_kernel<16, 8, kStorePartial>();
    status |= prepare_kernel<32, 8, kStorePartial>();
    status |= prepare_kernel<64, 8, kStorePartial>();
    status |= int(cudaFuncSetAttribute(fp8_token_kernel<false>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, 16384));
    status |= int(cudaFuncSetAttribute(fp8_token_kernel<true>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, 16384));
    return status;
}

/* Launch shape of the row kernel whose K ranges are the CTAs of a cluster. */
inline cudaLaunchConfig_t rows_cluster_config(camblas_cuda_context *context, int tiles, int parts,
                                              cudaLaunchAttribute *attribute)
{
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(unsigned(tiles) * unsigned(parts));
    config.blockDim = dim3(kRowsThreads);
    config.dynamicSmemBytes = RowsSmem<4, 1, true>::kTotal;
    config.stream = context->stream;
    attribute[0].id = cudaLaunchAttributeClusterDimension;
    attribute[0].val.clusterDim.x = unsigned(parts);
    attribute[0].val.clusterDim.y = 1;
    attribute[0].val.clusterDim.z = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    return config;
}

/* Number of K ranges (2..8, at most `wanted`) for which the clusters of all
 * `tiles` are resident together and no range is empty; 0 when there is none or
 * the cluster form is switched off. The device is asked once per cluster size. */
inline int rows_cluster_parts(camblas_cuda_context *context, int tiles, int k_blocks, int wanted)
{
    if (context->options.cluster_split == 0)
        return 0;
    for (int parts = std::min(wanted, 8); parts >= 2; --parts) {
        const int per = (k_blocks + parts - 1) / parts;
        if ((k_blocks + per - 1) / per != parts || 1ll * tiles * parts > context->sm_count)
            continue;
        int &cached = context->fp8_cluster_capacity[parts];
        if (cached == 0) {
            cudaLaunchAttribute attribute[1];
            cudaLaunchConfig_t config = rows_cluster_config(context, 1, parts, attribute);
            int clusters = 0;
            if (cudaOccupancyMaxActiveClusters(&clusters, fp8_block_rows<4, 1, true>, &config) !=
                cudaSuccess) {
                cudaGetLastError();
                clusters = 0;
            }
            cached = clusters > 0 ? clusters : -1;
        }
        if (cached >= tiles)
            return parts;
    }
    return 0;
}

template <int BN, int Stages, int Mode>
void launch_block(camblas_cuda_context *context, const CUtensorMap &p, const CUtensorMap &q,
                  const CUtensorMap &d, const BlockTask &task)
{
    int units = task.r_blocks * task.c_blocks * task.split;
    int grid = units < context->sm_count ? units : context->sm_count;
    fp8_block_gemm<BN, Stages, Mode>
        <<<grid, sm100::kThreads, block_smem_bytes<BN, Stages, Mode>(), context->stream>>>(p, q, d,
                                                                                         task);
}

/* 256-column tiles for many token rows (fp8_block_wide.cuh) */
inline int block_gemm_wide(camblas_cuda_context *context, bool pair, int rows, int outputs, int inner,
                           const void *q, const float *q_scale, const void *w, const float *w_scale,
                           void *out, int ldo);

inline int block_gemm(camblas_cuda_context *context, int rows, int outputs, int inner,
                      const void *q, const float *q_scale, const void *w, const float *w_scale,
                      void *out, int ldo)
{
    using host::encode_2d;
    BlockTask task{};
    task.depth = inner;
    task.k_blocks = inner / 128;
    task.out = static_cast<__nv_bfloat16 *>(out);
    task.ld_out = ldo;
    task.status = context->status;
    CUtensorMap p, qm, d;
    const auto type = CU_TENSOR_MAP_DATA_TYPE_UINT8;
    /* Few token rows: the product is bound by streaming the weights, and the
     * swapped kernel puts them on the 128-row side with the tokens on a 16, 32 or
     * 64 column side and the K range split over the SMs. The row tiling needs an
     * output it can store through a tensor map; without one, up to 128 rows stay
     * here whatever the limit. */
    const bool storable = host::aligned16(out) && ldo % 8 == 0 && outputs % 8 == 0;
    const bool swapped =
        rows <= context->options.fp8_swapped_rows || (rows <= kSwappedRowLimit && !storable);
    /* Many token rows: 128 x 256 tiles with N = 256 MMAs (fp8_block_wide.cuh) as soon
     * as they give every SM a tile; measured 27-44 % faster than the 128 x 128 tiles
     * at 4096 rows (same bits), slower when they leave SMs idle (512 x 4096: 64
     * tiles, 38 against 31 us). "fp8_rows" 3 / 4 force the one-SM / two-SM form. */
    if (!swapped) {
        const long long wide_tiles = 1ll * ((rows + 127) / 128) * ((outputs + 255) / 256);
        const int variant = context->options.fp8_rows;
        if (variant == 3 || variant == 4 || (variant == 0 && wide_tiles >= context->sm_count))
            return block_gemm_wide(context, variant == 4, rows, outputs, inner, q, q_scale, w, w_scale,
                                   out, ldo);
    }
    if (!swapped) {
        task.rows = rows, task.cols = outputs;
        task.r_blocks = (rows + 127) / 128, task.c_blocks = (outputs + 127) / 128;
        task.split = 1, task.k_blocks_per_split = task.k_blocks;
        /* few tiles and a long K: cut K into ranges, one unit each, summed by a
         * second launch (the tiles of M = 128, N = 4096 alone fill 32 of 148 SMs:
         * 22 against 30 us). With half the SMs busy or a short K the second launch
         * costs more than it recovers (N = 7168, K = 2048: 15.6 against 12.1 us). */
        const int tiles = task.r_blocks * task.c_blocks;
        int cluster_parts = 0;
        if ((context->options.fp8_rows == 0 || context->options.fp8_rows == 5) &&
            3 * tiles <= context->sm_count && task.k_blocks >= 32 &&
            outputs % 4 == 0) {
            int split = host::choose_split(tiles, task.k_blocks * 2, context->sm_count);
            /* The K ranges as the CTAs of a cluster, added through distributed shared
             * memory, when the device keeps all the clusters resident: no scratch
             * round trip and no second launch. Its time does not depend on the
             * number of rows, the two-launch form's does (N = 4096, K = 7168, 32 to
             * 128 rows: 14.9 us against 14.3, 15.8, 18.4, 21.4 us; the forms cross
             * between 64 and 96 rows on every shape measured). A cluster has at
             * most eight CTAs, so with very few tiles the scratch form has several
             * times as many CTAs and stays ahead (N = 512, K = 16384: 14.6 against
             * 10.5-14.5 us). */
            if (context->options.fp8_rows == 0 && rows >= 80) {
                cluster_parts = rows_cluster_parts(context, tiles, task.k_blocks, split);
                if (5 * cluster_parts < 2 * split)
                    cluster_parts = 0;
            }
            if (cluster_parts > 0)
                split = cluster_parts;
            task.k_blocks_per_split = (task.k_blocks + split - 1) / split;
            task.split = (task.k_blocks + task.k_blocks_per_split - 1) / task.k_blocks_per_split;
            if (task.split > 1 && cluster_parts == 0) {
                int status = host::reserve_scratch(context,
                                                   size_t(task.split) * rows * outputs * sizeof(float));
                if (status != 0)
                    return status;
                task.partial = static_cast<float *>(context->scratch);
            }
        }
        task.panel = task.r_blocks < 8 ? task.r_blocks : 8;
        task.p_scale = q_scale, task.q_scale = w_scale;
        bool ok = encode_2d(context, &p, type, 1, q, inner, rows, inner, 128, 128) &&
                  encode_2d(context, &qm, type, 1, w, inner, outputs, inner, 128, 128) &&
                  encode_2d(context, &d, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, out, outputs, rows,
                            size_t(ldo) * 2, 64, 32);
        if (!ok)
            return host::fail(context, "tensor map encoding", 1);
        const int variant = context->options.fp8_rows; /* tuning aid: 1 four warps, 2 one block per stage */
        if (cluster_parts > 0) {
            cudaLaunchAttribute attribute[1];
            cudaLaunchConfig_t config = rows_cluster_config(context, tiles, cluster_parts, attribute);
            cudaError_t error =
                cudaLaunchKernelEx(&config, fp8_block_rows<4, 1, true>, p, qm, d, task);
            if (error != cudaSuccess)
                return host::fail(context, "tcgen05 FP8 block GEMM, K ranges in a cluster", error);
            context->kernel_launches.fetch_add(1, std::memory_order_relaxed);
            return 0;
        }
        if (variant == 1) {
            launch_block<128, 6, kStoreRows>(context, p, qm, d, task);
        } else {
            const int units = task.r_blocks * task.c_blocks * task.split;
            const int grid = units < context->sm_count ? units : context->sm_count;
            /* two K blocks per stage: 5 % faster than one (fewer barrier round trips) */
            if (variant == 2)
                fp8_block_rows<6><<<grid, kRowsThreads, RowsSmem<6>::kTotal, context->stream>>>(
                    p, qm, d, task);
            else
                fp8_block_rows<3, 2><<<grid, kRowsThreads, RowsSmem<3, 2>::kTotal, context->stream>>>(
                    p, qm, d, task);
        }
        int status = host::launched(context, "tcgen05 FP8 block GEMM");
        if (status != 0 || task.split == 1)
            return status;
        cudaLaunchConfig_t config = {};
        const long long quads = 1ll * rows * (outputs / 4);
        config.gridDim = dim3(unsigned(std::min<long long>((quads + 255) / 256, 4ll * context->sm_count)));
        config.blockDim = dim3(256);
        config.stream = context->stream;
        cudaLaunchAttribute attribute[1];
        attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attribute[0].val.programmaticStreamSerializationAllowed = 1;
        config.attrs = attribute;
        config.numAttrs = 1;
        cudaError_t error =
            cudaLaunchKernelEx(&config, fp8_rows_reduce, rows, outputs, task.split,
                               static_cast<const float *>(task.partial), task.out, (long long)ldo);
        if (error != cudaSuccess)
            return host::fail(context, "FP8 K-range reduction", error);
        context->kernel_launches.fetch_add(1, std::memory_order_relaxed);
        return 0;
    }
    /* few tokens: weights on the 128-row side, tokens on the narrow side */
    task.rows = outputs, task.cols = rows;
    task.r_blocks = (outputs + 127) / 128;
    int bn = rows <= 16 ? 16 : (rows <= 32 ? 32 : 64);
    task.c_blocks = (rows + bn - 1) / bn;
    task.split = host::choose_split(task.r_blocks * task.c_blocks, task.k_blocks * 2,
                                    context->sm_count);
    task.split = host::split_if_it_pays(task.split, task.r_blocks * task.c_blocks, task.k_blocks,
                                        context->sm_count, rows, outputs, bn);
    task.k_blocks_per_split = (task.k_blocks + task.split - 1) / task.split;
    task.split = (task.k_blocks + task.k_blocks_per_split - 1) / task.k_blocks_per_split;
    task.panel = task.r_blocks < 8 ? task.r_blocks : 8;
    task.p_scale = w_scale, task.q_scale = q_scale;
    long long plane = 1ll * task.r_blocks * 128;
    if (task.split > 1) {
        int status = host::reserve_scratch(context, size_t(task.split) * rows * plane * 4);
        if (status != 0)
            return status;
        task.partial = static_cast<float *>(context->scratch);
    }
    bool ok = encode_2d(context, &p, type, 1, w, inner, outputs, inner, 128, 128) &&
              encode_2d(context, &qm, type, 1, q, inner, rows, inner, 128, bn);
    if (!ok)
        return host::fail(context, "tensor map encoding", 1);
    if (task.split > 1) {
        if (bn == 16)
            launch_block<16, 8, kStorePartial>(context, p, qm, p, task);
        else if (bn == 32)
            launch_block<32, 8, kStorePartial>(context, p, qm, p, task);
        else
            launch_block<64, 8, kStorePartial>(context, p, qm, p, task);
        int status = host::launched(context, "tcgen05 FP8 split-K block GEMM");
        if (status != 0)
            return status;
        cudaError_t error = sm100::launch_split_reduce(context->stream, outputs, rows, task.split,
                                                       plane, 1.f, 0.f, task.partial, nullptr, 0,
                                                       nullptr, task.out, ldo);
        if (error != cudaSuccess)
            return host::fail(context, "FP8 split-K reduction", error);
        context->kernel_launches.fetch_add(1, std::memory_order_relaxed);
        return 0;
    }
    if (bn == 16)
        launch_block<16, 8, kStoreColumns>(context, p, qm, p, task);
    else if (bn == 32)
        launch_block<32, 8, kStoreColumns>(context, p, qm, p, task);
    else
        launch_block<64, 8, kStoreColumns>(context, p, qm, p, task);
    return host::launched(context, "tcgen05 FP8 swapped block GEMM");
}

} // namespace fp8

/* ---- extern "C" ------------------------------------------------------------------ */

extern "C" int camblas_cuda_fp8_quantize_rows(camblas_cuda_context *context, int rows, int inner,
                                              const void *x, int ldx, void *q, float *scale)
{
    return host::guarded(context, [&] {
        if (rows < 0 || inner < 128 || inner % 128 || ldx < inner || ldx % 4)
            return host::fail(context, "invalid FP8 quantise dimensions", 1);
        if (rows == 0)
            return 0;
        if (!x || !q || !scale || (uintptr_t(x) & 7) || (uintptr_t(q) & 3) || x == q)
            return host::fail(context, "invalid FP8 quantise operands", 1);
        long long groups = 1ll * rows * (inner / 128);
        unsigned blocks = unsigned(std::min<long long>((groups + 7) / 8, 148 * 16));
        fp8::quantize_rows_kernel<<<blocks, 256, 0, context->stream>>>(
            rows, inner, ldx, static_cast<const __nv_bfloat16 *>(x), static_cast<uint8_t *>(q),
            scale);
        return host::launched(context, "FP8 row quantisation");
    });
}

extern "C" int camblas_cuda_fp8_block_gemm(camblas_cuda_context *context, int rows, int outputs,
                                           int inner, const void *q, const float *q_scale,
                                           const void *w, const float *w_scale, void *out, int ldo)
{
    return host::guarded(context, [&] {
        if (rows < 0 || outputs < 0 || inner < 128 || inner % 128 || ldo < outputs)
            return host::fail(context, "invalid FP8 block GEMM dimensions", 1);
        if (rows == 0 || outputs == 0)
            return 0;
        if (!q || !q_scale || !w || !w_scale || !out || out == q || out == w)
            return host::fail(context, "missing or aliased FP8 block GEMM operand", 1);
        if (!host::aligned16(q) || !host::aligned16(w) ||
            (rows > fp8::kSwappedRowLimit && (!host::aligned16(out) || ldo % 8 || outputs % 8)))
            return host::fail(context, "FP8 block GEMM operands must be 16-byte aligned", 1);
        context->counts[0]++;
        return fp8::block_gemm(context, rows, outputs, inner, q, q_scale, w, w_scale, out, ldo);
    });
}

extern "C" int camblas_cuda_fp8_decode_supported(const camblas_cuda_context *context)
{
    return context ? 1 : 0;
}

extern "C" size_t camblas_cuda_fp8_workspace_size(int, int, int)
{
    return 0;
}

namespace fp8
{
inline int token_arguments_bad(int outputs, int inner, const void *input, const void *weight,
                               const float *weight_scale, int row_stride, int column_stride,
                               const void *output)
{
    return outputs < 16 || outputs % 16 || inner < 32 || inner > 8192 || inner % 32 || !input ||
           !weight || !weight_scale || !output || row_stride < 1 || column_stride < 1 ||
           (uintptr_t(input) & 3) || (uintptr_t(weight) & 3) || (uintptr_t(weight_scale) & 3) ||
           (uintptr_t(output) & 1) || output == input || output == weight ||
           output == static_cast<const void *>(weight_scale);
}
} // namespace fp8

extern "C" int camblas_cuda_fp8_decode(camblas_cuda_context *context, int outputs, int inner,
                                       const void *input, const float *input_scale,
                                       const void *weight, const float *weight_scale,
                                       int input_scale_stride, int weight_scale_row_stride,
                                       int weight_scale_column_stride, void *workspace,
                                       size_t workspace_bytes, void *output)
{
    return host::guarded(context, [&] {
        (void)workspace;
        (void)workspace_bytes;
        if (fp8::token_arguments_bad(outputs, inner, input, weight, weight_scale,
                                     weight_scale_row_stride, weight_scale_column_stride, output) ||
            !input_scale || input_scale_stride < 1 || (uintptr_t(input_scale) & 3))
            return host::fail(context, "invalid FP8 decode arguments", 1);
        size_t shared = size_t(inner) + size_t(inner / 32) * sizeof(float);
        fp8::fp8_token_kernel<false><<<(outputs + 7) / 8, 256, shared, context->stream>>>(
            outputs, inner, input, input_scale, input_scale_stride,
            static_cast<const uint8_t *>(weight), weight_scale, weight_scale_row_stride,
            weight_scale_column_stride, static_cast<__nv_bfloat16 *>(output));
        return host::launched(context, "FP8 decode");
    });
}

extern "C" int camblas_cuda_fp8_linear(camblas_cuda_context *context, int outputs, int inner,
                                       const void *input, const void *weight,
                                       const float *weight_scale, int weight_scale_row_stride,
                                       int weight_scale_column_stride, void *workspace,
                                       size_t workspace_bytes, void *output)
{
    return host::guarded(context, [&] {
        (void)workspace;
        (void)workspace_bytes;
        if (fp8::token_arguments_bad(outputs, inner, input, weight, weight_scale,
                                     weight_scale_row_stride, weight_scale_column_stride, output))
            return host::fail(context, "invalid FP8 linear arguments", 1);
        size_t shared = size_t(inner) + size_t(inner / 32) * sizeof(float);
        fp8::fp8_token_kernel<true><<<(outputs + 7) / 8, 256, shared, context->stream>>>(
            outputs, inner, input, nullptr, 1, static_cast<const uint8_t *>(weight), weight_scale,
            weight_scale_row_stride, weight_scale_column_stride,
            static_cast<__nv_bfloat16 *>(output));
        return host::launched(context, "FP8 linear");
    });
}

/* One-level Strassen for BF16 squares lives in strassen.cuh. */
#include "strassen.cuh"
