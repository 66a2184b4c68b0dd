/*
 * BF16 GEMM on the fifth-generation tensor cores: D[R,C] = P[R,K] . Q[C,K]^T
 * with FP32 accumulation in tensor memory.
 *
 * One persistent CTA per SM, six warps with fixed roles:
 *   warp 0      TMA producer: streams 128 x 64 tiles of P and BN x 64 tiles of Q
 *               into a ring of 128-byte-swizzled shared-memory stages.
 *   warp 1      MMA issuer: one thread issues tcgen05.mma (M=128, N=BN, K=16)
 *               four times per stage and commits the stage back to the producer;
 *               accumulators alternate between two TMEM buffers so the epilogue
 *               of one tile overlaps the main loop of the next.
 *   warps 2-5   epilogue: tcgen05.ld of the accumulator quarter the warp owns,
 *               alpha/beta/bias/addend in FP32, one rounding to BF16, then
 *                 kStoreRows     swizzled staging + TMA store (row-major D),
 *                 kStoreColumns  lane-contiguous stores of D^T (operands swapped:
 *                                P = weights, Q = tokens, for few tokens),
 *                 kStorePartial  FP32 partial sums of one K split into scratch.
 * Every barrier wait is bounded; a wait that gives up records its role in the
 * status word, raises a CTA-wide abort flag and all roles drain and return.
 */
#pragma once

#include "sm100_primitives.cuh"

namespace sm100
{

enum StoreMode : int { kStoreRows = 0, kStoreColumns = 1, kStorePartial = 2, kStoreFloat = 3 };
/* Operand storage: kMajorK = rows contiguous along K (a 64-wide K slice of a row
 * is one 128-byte swizzled line); kMajorMN = contiguous along the row index (a
 * 64-row slice of one K index is one line; a tile is a sequence of 64 x 64
 * boxes of 8 KB). */
enum OperandMajor : int { kMajorK = 0, kMajorMN = 1 };

struct GemmTask {
    int rows, cols, depth;         /* R, C, K */
    int r_blocks, c_blocks;        /* tiles along R (128) and C (BN) */
    int k_blocks;                  /* ceil(K / 64) */
    int split, k_blocks_per_split; /* K partition (1 = whole K per tile) */
    int panel;                     /* row blocks per rasterisation panel */
    float alpha, beta;
    __nv_bfloat16 *out;
    long long ld_out;
    const __nv_bfloat16 *addend; /* indexed like out; read only when beta != 0 */
    long long ld_add;
    const __nv_bfloat16 *bias; /* per column (kStoreRows) or per row (kStoreColumns) */
    float *partial;            /* kStorePartial: [split][cols][r_blocks*128] */
    unsigned *status;
    /* Optional second and third outputs for a packed projection: columns
     * [0,cut0) go to out, [cut0,cut1) to out1, [cut1,cols) to out2. cut0 and
     * cut1 are multiples of BN; cut0 == cols disables the feature. */
    int cut0, cut1;
    __nv_bfloat16 *out1, *out2; /* second and third output of a packed projection */
    long long ld_out1, ld_out2;
    int width; /* tile width of the two-SM kernel when it is chosen at run time */
    /* Batch of independent products over stacked operands (batch >= 1): product
     * b reads P rows (K-major) or P K indices (MN-major) offset by b*batch_p,
     * likewise Q by b*batch_q, and writes FP32 plane b of out_float. */
    int batch, batch_p, batch_q;
    float *out_float; /* kStoreFloat: [batch][rows][ld_out] */
    /* Stream-K tail (kStoreRows, at most eight row blocks). CTAs form teams of
     * r_blocks members, member i owning row block i, so that the members of a
     * team walk the same weight tiles at the same time and share them through
     * L2. The first dp_cols column blocks are processed whole, column block c by
     * team c mod teams. The (column block, K block) iterations of the remaining
     * sk_cols column blocks (fewer than there are teams) are cut into equal
     * contiguous ranges, one per team; a range touches at most two column
     * blocks, and each piece leaves its raw FP32 sums in slot 2*cta + piece of
     * sk_partial ([slot][128][BN]). sk_fixup then adds the pieces of every tile
     * in K order and applies the epilogue. sk_cols == 0 switches this off. */
    int dp_cols, sk_cols;
    float *sk_partial;
    const unsigned *skip_if_set; /* when non-NULL and *skip_if_set != 0 the kernel does nothing */
    const unsigned *run_if_set;  /* when non-NULL and *run_if_set == 0 the kernel does nothing */
    /* Row-parallel product whose partial sums go to other GPUs (Push variant of
     * the two-SM kernel, push_world >= 1). The epilogue scales the tile by alpha
     * and, instead of storing it to `out`, writes it as BF16 into the staging
     * area of the GPU that owns the tile's column block (owner = column block
     * mod push_world): push_staging[owner] is the slot that GPU keeps for this
     * rank, in this process's address space, laid out slab by slab (see
     * epilogue_push). An epilogue warp covers a 32-row slab of the tile; when
     * its copies are complete it adds one to word `unit` of push_arrive[owner],
     * unit = (row block * c_blocks + column block) * 8 + slab. */
    int push_world;
    __nv_bfloat16 *push_staging[8];
    unsigned *push_arrive[8];
    /* SwiGLU epilogue that also quantises (kEpiSwigluQuant): the 128 outputs a
     * tile holds for one row are one 1 x 128 quantisation group, written as E4M3
     * bytes to quant_out[row * ld_quant + column] with their FP32 scale
     * (max(amax, 1e-10) / 448) in quant_scale[row * quant_groups + column / 128]. */
    uint8_t *quant_out;
    long long ld_quant;
    float *quant_scale;
    int quant_groups;
};

constexpr int kBlockR = 128;
constexpr int kBlockK = 64;
constexpr int kUmmaK = 16;
constexpr int kThreads = 192;
constexpr int kStagingBytes = 4 * 2 * 4096; /* 4 warps x 2 buffers x (32 rows x 128 B) */

template <int BN, int Stages, int Mode> struct GemmSmem {
    static constexpr int kPBytes = kBlockR * kBlockK * 2;
    static constexpr int kQBytes = BN * kBlockK * 2;
    static constexpr int kStageBytes = kPBytes + kQBytes;
    static constexpr int kStaging = Mode == kStoreRows ? kStagingBytes : 0;
    static constexpr int kBarrierBytes = 256;
    static constexpr int kTotal = Stages * kStageBytes + kStaging + kBarrierBytes + 1024;
};

__device__ __forceinline__ void report(unsigned *status, volatile uint32_t *abort, unsigned role)
{
    if (!*abort) {
        *abort = 1;
        atomicCAS(status, 0u, role | (blockIdx.x << 4));
    }
}

__device__ __forceinline__ void locate_tile(const GemmTask &task, int tile, int &rb, int &cb,
                                            int &batch)
{
    const int per_batch = task.r_blocks * task.c_blocks;
    batch = tile / per_batch;
    tile -= batch * per_batch;
    int per_panel = task.panel * task.c_blocks;
    int panel = tile / per_panel;
    int local = tile - panel * per_panel;
    int height = min(task.panel, task.r_blocks - panel * task.panel);
    cb = local / height;
    rb = panel * task.panel + local - cb * height;
}

/* One piece of work of a CTA: a tile, a K-block range and, for a stream-K
 * piece, the slot its partial sums go to (slot < 0: the piece owns the whole K
 * of its tile or is one of the uniform splits of the few-token modes). */
struct Unit {
    int rb, cb, part, batch, kb0, kb1, slot;
};

/* The item-th piece of work of worker `worker` out of `workers` (a worker is a
 * CTA, or a pair of CTAs in the two-SM kernel); false when it has no more. */
__device__ __forceinline__ bool fetch_unit(const GemmTask &task, int item, int worker, int workers,
                                           Unit &u)
{
    int tile;
    u.slot = -1;
    if (task.sk_cols == 0) {
        const long long unit = worker + static_cast<long long>(item) * workers;
        if (unit >= 1ll * task.r_blocks * task.c_blocks * task.split * task.batch)
            return false;
        u.part = static_cast<int>(unit % task.split);
        tile = static_cast<int>(unit / task.split);
        u.kb0 = u.part * task.k_blocks_per_split;
        u.kb1 = min(task.k_blocks, u.kb0 + task.k_blocks_per_split);
        locate_tile(task, tile, u.rb, u.cb, u.batch);
        return true;
    }
    const int teams = workers / task.r_blocks, team = worker / task.r_blocks;
    if (team >= teams)
        return false;
    u.rb = worker - team * task.r_blocks;
    u.part = 0, u.batch = 0;
    const int whole = task.dp_cols > team ? (task.dp_cols - team + teams - 1) / teams : 0;
    if (item < whole) {
        u.cb = team + item * teams;
        u.kb0 = 0, u.kb1 = task.k_blocks;
        return true;
    }
    const int piece = item - whole;
    if (piece > 1)
        return false;
    const long long total = 1ll * task.sk_cols * task.k_blocks;
    const long long begin = team * total / teams, end = (team + 1) * total / teams;
    if (begin >= end)
        return false;
    const long long first = begin / task.k_blocks;
    const long long cut = min(end, (first + 1) * task.k_blocks);
    if (piece == 0) {
        u.cb = task.dp_cols + static_cast<int>(first);
        u.kb0 = static_cast<int>(begin - first * task.k_blocks);
        u.kb1 = static_cast<int>(cut - first * task.k_blocks);
    } else {
        if (end <= cut)
            return false;
        u.cb = task.dp_cols + static_cast<int>(first) + 1;
        u.kb0 = 0;
        u.kb1 = static_cast<int>(end - cut);
    }
    u.slot = 2 * worker + piece;
    return true;
}

__host__ __device__ inline long long unit_count(const GemmTask &task)
{
    return 1ll * task.r_blocks * task.c_blocks * task.split * task.batch;
}

/* Layout of a stream-K partial slot (128 accumulator rows x BN columns of raw
 * FP32 sums): 32-column chunks, chunk-major, each chunk [128 rows][32 floats]
 * with the eight 16-byte pieces of a row XOR-swizzled by (row & 7). A warp's 32
 * rows of one chunk are therefore 4 KB of contiguous global memory, which it
 * stages in shared memory (same swizzle, conflict-free) and writes with one bulk
 * copy; per-lane stores of 128-byte row pieces would cost eight times the
 * memory transactions. Float offset of the piece holding columns c..c+3: */
__device__ __forceinline__ int partial_offset(int r, int c)
{
    return (c >> 5) * 4096 + r * 32 + ((((c & 31) >> 2) ^ (r & 7)) << 2);
}

/* Epilogue of a stream-K piece: the raw FP32 sums of this warp's 32 accumulator
 * rows to rows quarter*32.. of the 128-row partial slot, one 4 KB bulk copy per
 * 32-column chunk through the warp's two staging buffers. `release` is called
 * once every lane of the warp has read the last column of the accumulator. */
template <int BN, typename Release>
__device__ __forceinline__ void epilogue_partial(float *slot, uint32_t taddr, int quarter, int lane,
                                                 uint8_t *slab, uint32_t &slab_use, bool roomy,
                                                 Release release)
{
    constexpr int kChunks = BN / 32;
    static_assert(kChunks % 2 == 0, "chunks are processed in pairs");
    /* with `roomy` the caller passes BN/32 buffers and none is reused */
    auto store = [&](int chunk, const uint32_t (&acc)[32]) {
        uint8_t *buffer_smem = slab + (roomy ? chunk : (slab_use & 1)) * 4096;
        if (!roomy) {
            /* the bulk copy that last read this buffer must be done */
            if (lane == 0)
                tma_store_wait_read<1>();
            __syncwarp();
        }
        const uint32_t base = smem_u32(buffer_smem) + lane * 128;
#pragma unroll
        for (int piece = 0; piece < 8; ++piece)
            st_shared_v4(base + ((piece ^ (lane & 7)) << 4), acc[piece * 4], acc[piece * 4 + 1],
                         acc[piece * 4 + 2], acc[piece * 4 + 3]);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
            bulk_store(slot + chunk * 4096 + quarter * 1024, buffer_smem, 4096);
            tma_store_commit();
        }
        ++slab_use;
    };
    /* The tensor-memory load of the next chunk is in flight while this one is
     * staged; its latency would otherwise be paid once per chunk. */
    uint32_t even[32], odd[32];
    tmem_ld_32x32(taddr, even);
#pragma unroll 1
    for (int chunk = 0; chunk < kChunks; chunk += 2) {
        tmem_ld_wait();
        tmem_ld_32x32(taddr + (chunk + 1) * 32, odd);
        store(chunk, even);
        tmem_ld_wait();
        if (chunk + 2 < kChunks)
            tmem_ld_32x32(taddr + (chunk + 2) * 32, even);
        else
            release();
        store(chunk + 1, odd);
    }
}

/* Adds, in ascending K order, the stream-K pieces of the tile in stream-K
 * column block `sk_col` for row r (0..127 of its 128-row slot) and columns
 * c8..c8+7. slot_of(team, piece) is the 128-row slot that team's piece went to.
 * Loads are issued four pieces at a time so that their latencies overlap. */
template <int BN, typename SlotOf>
__device__ __forceinline__ void sum_pieces(const GemmTask &task, int teams, int sk_col, int r,
                                           int c8, SlotOf slot_of, float (&sum)[8])
{
    const long long total = 1ll * task.sk_cols * task.k_blocks;
    const long long tile_begin = 1ll * sk_col * task.k_blocks, tile_end = tile_begin + task.k_blocks;
    /* start of team t's range; 32-bit division when the products are small enough */
    const bool narrow = total * teams < 0x7fffffffll;
    auto range_begin = [&](int t) -> long long {
        return narrow ? static_cast<long long>(static_cast<unsigned>(t) * static_cast<unsigned>(total) /
                                               static_cast<unsigned>(teams))
                      : t * total / teams;
    };
    int team = narrow ? static_cast<int>(static_cast<unsigned>(tile_begin) *
                                         static_cast<unsigned>(teams) / static_cast<unsigned>(total))
                      : static_cast<int>(tile_begin * teams / total);
    team = team > 0 ? team - 1 : 0;
    const int low_offset = partial_offset(r, c8), high_offset = partial_offset(r, c8 + 4);
    bool more = true;
    long long end = range_begin(team);
    while (more) {
        const float *source[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            source[j] = nullptr;
            while (more && source[j] == nullptr) {
                if (team >= teams) {
                    more = false;
                    break;
                }
                const long long begin = end;
                end = range_begin(team + 1);
                if (begin >= tile_end) {
                    more = false;
                    break;
                }
                if (end > tile_begin && begin < end) {
                    /* a team's first piece lies in the column block its range starts in */
                    const int piece = begin < tile_begin ? 1 : 0;
                    source[j] = task.sk_partial + slot_of(team, piece) * (128ll * BN);
                }
                ++team;
            }
        }
        float4 low[4], high[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (source[j] != nullptr) {
                low[j] = *reinterpret_cast<const float4 *>(source[j] + low_offset);
                high[j] = *reinterpret_cast<const float4 *>(source[j] + high_offset);
            }
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (source[j] != nullptr) {
                sum[0] += low[j].x, sum[1] += low[j].y, sum[2] += low[j].z, sum[3] += low[j].w;
                sum[4] += high[j].x, sum[5] += high[j].y, sum[6] += high[j].z, sum[7] += high[j].w;
            }
    }
}

/* Rounds 64 accumulator columns of this thread's row (alpha applied; bias and
 * beta*addend when present) to BF16 and writes them as eight 16-byte pieces to
 * row `lane` of a 128-byte-swizzled 32 x 128 B staging buffer. The common case
 * without bias and addend has its own straight-line code: with the tests of the
 * general case inside the unrolled loop the block ran 2.5 times slower. */
__device__ __forceinline__ void stage_row64(const GemmTask &task, const uint32_t (&acc)[2][32],
                                            int row, int cbase, int lane, uint8_t *buffer_smem)
{
    const float alpha = task.alpha;
    const uint32_t base = smem_u32(buffer_smem) + lane * 128;
    if (task.bias == nullptr && task.beta == 0.f) {
#pragma unroll
        for (int piece = 0; piece < 8; ++piece) {
            const uint32_t *a = &acc[piece >> 2][(piece & 3) * 8];
            st_shared_v4(base + ((piece ^ (lane & 7)) << 4),
                         pack_bf16(alpha * __uint_as_float(a[0]), alpha * __uint_as_float(a[1])),
                         pack_bf16(alpha * __uint_as_float(a[2]), alpha * __uint_as_float(a[3])),
                         pack_bf16(alpha * __uint_as_float(a[4]), alpha * __uint_as_float(a[5])),
                         pack_bf16(alpha * __uint_as_float(a[6]), alpha * __uint_as_float(a[7])));
        }
        return;
    }
    const bool has_bias = task.bias != nullptr;
    const bool has_addend = task.beta != 0.f && row < task.rows;
    const float beta = task.beta;
    const __nv_bfloat16 *addend_row =
        has_addend ? task.addend + static_cast<long long>(row) * task.ld_add : nullptr;
#pragma unroll
    for (int piece = 0; piece < 8; ++piece) {
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
            v[i] = alpha * __uint_as_float(acc[piece >> 2][(piece & 3) * 8 + i]);
        const int c = cbase + piece * 8;
        if (has_bias) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (c + i < task.cols)
                    v[i] += __bfloat162float(task.bias[c + i]);
        }
        if (has_addend) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (c + i < task.cols)
                    v[i] = fmaf(beta, __bfloat162float(addend_row[c + i]), v[i]);
        }
        st_shared_v4(base + ((piece ^ (lane & 7)) << 4), pack_bf16(v[0], v[1]),
                     pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
    }
}

/* Epilogue of a whole tile, token rows on TMEM lanes: alpha, bias and
 * beta*addend in FP32, one rounding, 64-column slabs staged with the 128-byte
 * swizzle and written with TMA stores (which clip rows and columns beyond the
 * matrix). `row` is this thread's row, `store_row` the first row of the warp's
 * slab. Normally `slab` is the warp's pair of 4 KB buffers, used in turn; a
 * buffer is reused only after the TMA store that read it two slabs ago is done,
 * and since such a store takes about 0.7 us from issue to that point, the
 * second half of a tile waits for the first. With `roomy` the caller passes
 * BN/64 buffers (the CTA's last tile borrows the operand ring, which is idle by
 * then) and no slab waits. */
template <int BN, typename Release>
__device__ __forceinline__ void epilogue_rows(const GemmTask &task, const CUtensorMap *map_d,
                                              uint32_t taddr, int row, int store_row, int col0,
                                              int col_shift, int lane, uint8_t *slab,
                                              uint32_t &slab_use, bool roomy, Release release)
{
    constexpr int kChunks = BN / 64;
    auto store = [&](int chunk, const uint32_t (&acc)[2][32]) {
        uint8_t *buffer_smem = slab + (roomy ? chunk : (slab_use & 1)) * 4096;
        if (!roomy) {
            /* the TMA store that last read this buffer must be done */
            if (lane == 0)
                tma_store_wait_read<1>();
            __syncwarp();
        }
        const int cbase = col0 + chunk * 64;
        stage_row64(task, acc, row, cbase, lane, buffer_smem);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
            tma_store_2d(map_d, buffer_smem, cbase - col_shift, store_row);
            tma_store_commit();
        }
        ++slab_use;
    };
    auto load = [&](int chunk, uint32_t (&acc)[2][32]) {
        tmem_ld_32x32(taddr + chunk * 64, acc[0]);
        tmem_ld_32x32(taddr + chunk * 64 + 32, acc[1]);
    };
    if constexpr (kChunks == 1) {
        uint32_t acc[2][32];
        load(0, acc);
        tmem_ld_wait();
        release();
        store(0, acc);
    } else {
        /* The tensor-memory load of the next slab is in flight while this one is
         * rounded and staged. */
        static_assert(kChunks % 2 == 0, "slabs are processed in pairs");
        uint32_t even[2][32], odd[2][32];
        load(0, even);
#pragma unroll 1
        for (int chunk = 0; chunk < kChunks; chunk += 2) {
            tmem_ld_wait();
            load(chunk + 1, odd);
            store(chunk, even);
            tmem_ld_wait();
            if (chunk + 2 < kChunks)
                load(chunk + 2, even);
            else
                release();
            store(chunk + 1, odd);
        }
    }
}

/* SiLU(gate) * up with the roundings of the two-step path it replaces (a BF16
 * GEMM output followed by the reference's silu_multiply,
 * inference_fusion.cuh:19-29): gate and up are first rounded to BF16 as the
 * GEMM would have stored them, SiLU(gate) is rounded, the product is rounded. */
__device__ __forceinline__ float swiglu_value(float gate_sum, float up_sum)
{
    const float g = __bfloat162float(__float2bfloat16_rn(gate_sum));
    const float u = __bfloat162float(__float2bfloat16_rn(up_sum));
    const float activated = __bfloat162float(__float2bfloat16_rn(g / (1.f + expf(-g))));
    return activated * u;
}

/* Epilogue of a 256-column tile whose first 128 columns are gate features and
 * whose last 128 the matching up features (the weight was interleaved that
 * way): writes the 128 columns SiLU(gate) * up of the tile to `map_out` at
 * column out_col0. Two 64-column slabs, each needing the gate and the up
 * accumulators of its columns; staging and TMA store as in epilogue_rows. */
template <typename Release>
__device__ __forceinline__ void epilogue_swiglu(const GemmTask &task, const CUtensorMap *map_out,
                                                uint32_t taddr, int store_row, int out_col0, int lane,
                                                uint8_t *slab, uint32_t &slab_use, bool roomy,
                                                Release release)
{
    const float alpha = task.alpha;
#pragma unroll 1
    for (int chunk = 0; chunk < 2; ++chunk) {
        uint32_t gate[2][32], up[2][32];
        tmem_ld_32x32(taddr + chunk * 64, gate[0]);
        tmem_ld_32x32(taddr + chunk * 64 + 32, gate[1]);
        tmem_ld_32x32(taddr + 128 + chunk * 64, up[0]);
        tmem_ld_32x32(taddr + 128 + chunk * 64 + 32, up[1]);
        tmem_ld_wait();
        if (chunk == 1)
            release();
        uint8_t *buffer_smem = slab + (roomy ? chunk : (slab_use & 1)) * 4096;
        if (!roomy) {
            if (lane == 0)
                tma_store_wait_read<1>();
            __syncwarp();
        }
        const uint32_t base = smem_u32(buffer_smem) + lane * 128;
#pragma unroll
        for (int piece = 0; piece < 8; ++piece) {
            const uint32_t *g = &gate[piece >> 2][(piece & 3) * 8];
            const uint32_t *u = &up[piece >> 2][(piece & 3) * 8];
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i)
                v[i] = swiglu_value(alpha * __uint_as_float(g[i]), alpha * __uint_as_float(u[i]));
            st_shared_v4(base + ((piece ^ (lane & 7)) << 4), pack_bf16(v[0], v[1]),
                         pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
            tma_store_2d(map_out, buffer_smem, out_col0 + chunk * 64, store_row);
            tma_store_commit();
        }
        ++slab_use;
    }
}

/* E4M3 byte of value * inverse, clamped to the finite range: the conversion of
 * the activation quantiser (fp8::quantize_rows_kernel). */
__device__ __forceinline__ uint32_t quantise_e4m3(float value, float inverse)
{
    const float scaled = fminf(fmaxf(__fmul_rn(value, inverse), -448.f), 448.f);
    uint16_t pair;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(pair) : "f"(0.f), "f"(scaled));
    return pair & 255u;
}

/* SwiGLU epilogue that hands the down projection its FP8 input directly: the
 * 128 outputs SiLU(gate) * up of this thread's row (one quantisation group) are
 * rounded to BF16 exactly as epilogue_swiglu would store them, their largest
 * magnitude gives the group's scale, and the E4M3 bytes and the scale are
 * written instead of the BF16 values - what fp8::quantize_rows_kernel would
 * produce from the BF16 tensor, without that tensor ever reaching memory.
 * Four passes of 32 columns keep the registers in hand: 64 packed BF16 pairs
 * stay live next to one pass of gate and up accumulators. */
template <typename Release>
__device__ __forceinline__ void epilogue_swiglu_quant(const GemmTask &task, uint32_t taddr, int row,
                                                      int out_col0, Release release)
{
    const float alpha = task.alpha;
    uint32_t kept[64]; /* the row's 128 outputs as BF16 pairs */
    float largest = 0.f;
#pragma unroll
    for (int pass = 0; pass < 4; ++pass) {
        uint32_t gate[32], up[32];
        tmem_ld_32x32(taddr + pass * 32, gate);
        tmem_ld_32x32(taddr + 128 + pass * 32, up);
        tmem_ld_wait();
        if (pass == 3)
            release();
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
            const float low = swiglu_value(alpha * __uint_as_float(gate[i]), alpha * __uint_as_float(up[i]));
            const float high =
                swiglu_value(alpha * __uint_as_float(gate[i + 1]), alpha * __uint_as_float(up[i + 1]));
            const uint32_t pair = pack_bf16(low, high);
            kept[pass * 16 + i / 2] = pair;
            largest = fmaxf(largest, fmaxf(fabsf(bf16_low(pair)), fabsf(bf16_high(pair))));
        }
    }
    if (row >= task.rows)
        return;
    const float maximum = fmaxf(largest, 1e-10f);
    task.quant_scale[static_cast<long long>(row) * task.quant_groups + (out_col0 >> 7)] =
        __fmul_rn(maximum, 1.0f / 448.0f);
    const float inverse = __fdiv_rn(448.0f, maximum);
    uint4 *target =
        reinterpret_cast<uint4 *>(task.quant_out + static_cast<long long>(row) * task.ld_quant + out_col0);
#pragma unroll
    for (int piece = 0; piece < 8; ++piece) {
        uint32_t words[4];
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const uint32_t first = kept[piece * 8 + w * 2], second = kept[piece * 8 + w * 2 + 1];
            words[w] = quantise_e4m3(bf16_low(first), inverse) |
                       (quantise_e4m3(bf16_high(first), inverse) << 8) |
                       (quantise_e4m3(bf16_low(second), inverse) << 16) |
                       (quantise_e4m3(bf16_high(second), inverse) << 24);
        }
        target[piece] = make_uint4(words[0], words[1], words[2], words[3]);
    }
}

/* Push variant of the row epilogue for a product whose K range is split over
 * GPUs: alpha*acc rounded to BF16 (bias and addend are applied once, by the GPU
 * that sums the partials) and sent to the owner's staging slot. The slot is
 * laid out by slab, not by matrix row: slab `unit` (32 rows x BN columns) is
 * BN/64 consecutive 4 KB chunks, each [32 rows][128 bytes] with the 16-byte
 * pieces of a row XOR-swizzled by (row & 7) - exactly the warp's staging buffer.
 * A chunk therefore leaves as ONE 4 KB bulk copy from shared memory to the
 * owner's memory: large NVLink writes issued by one thread, instead of 128-byte
 * row segments stored by all lanes. When the warp's copies are complete a
 * system-scope release add tells the owner that the slab is there. Rows and
 * columns beyond the matrix carry zeros (their operands were zero-filled).
 * `slab`/`roomy` as in epilogue_rows. */
template <int BN, typename Release>
__device__ __forceinline__ void epilogue_push(const GemmTask &task, uint32_t taddr, int owner,
                                              int unit, int lane, uint8_t *slab,
                                              uint32_t &slab_use, bool roomy, Release release)
{
    constexpr int kChunks = BN / 64;
    static_assert(kChunks % 2 == 0, "slabs are processed in pairs");
    __nv_bfloat16 *destination =
        task.push_staging[owner] + static_cast<long long>(unit) * (32 * BN);
    const float alpha = task.alpha;
    auto send = [&](int chunk, const uint32_t (&acc)[2][32]) {
        uint8_t *buffer_smem = slab + (roomy ? chunk : (slab_use & 1)) * 4096;
        if (!roomy) {
            if (lane == 0)
                tma_store_wait_read<1>();
            __syncwarp();
        }
        const uint32_t base = smem_u32(buffer_smem) + lane * 128;
#pragma unroll
        for (int piece = 0; piece < 8; ++piece) {
            const uint32_t *a = &acc[piece >> 2][(piece & 3) * 8];
            st_shared_v4(base + ((piece ^ (lane & 7)) << 4),
                         pack_bf16(alpha * __uint_as_float(a[0]), alpha * __uint_as_float(a[1])),
                         pack_bf16(alpha * __uint_as_float(a[2]), alpha * __uint_as_float(a[3])),
                         pack_bf16(alpha * __uint_as_float(a[4]), alpha * __uint_as_float(a[5])),
                         pack_bf16(alpha * __uint_as_float(a[6]), alpha * __uint_as_float(a[7])));
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
            bulk_store(destination + chunk * 2048, buffer_smem, 4096);
            tma_store_commit();
        }
        ++slab_use;
    };
    auto load = [&](int chunk, uint32_t (&acc)[2][32]) {
        tmem_ld_32x32(taddr + chunk * 64, acc[0]);
        tmem_ld_32x32(taddr + chunk * 64 + 32, acc[1]);
    };
    uint32_t even[2][32], odd[2][32];
    load(0, even);
#pragma unroll 1
    for (int chunk = 0; chunk < kChunks; chunk += 2) {
        tmem_ld_wait();
        load(chunk + 1, odd);
        send(chunk, even);
        tmem_ld_wait();
        if (chunk + 2 < kChunks)
            load(chunk + 2, even);
        else
            release();
        send(chunk + 1, odd);
    }
    if (lane == 0) {
        tma_store_wait_all<0>(); /* the copies have been written, not only read */
        __threadfence_system();
        flag_add_release_system(task.push_arrive[owner] + unit, 1u);
    }
    __syncwarp();
}

/* alpha*acc + bias + beta*addend for eight consecutive columns of one row. */
__device__ __forceinline__ void finish8(const GemmTask &task, int row, int c, const uint32_t *acc,
                                        float (&v)[8])
{
#pragma unroll
    for (int i = 0; i < 8; ++i)
        v[i] = task.alpha * __uint_as_float(acc[i]);
    if (task.bias != nullptr) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (c + i < task.cols)
                v[i] += __bfloat162float(task.bias[c + i]);
    }
    if (task.beta != 0.f && row < task.rows) {
        const __nv_bfloat16 *source = task.addend + static_cast<long long>(row) * task.ld_add + c;
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (c + i < task.cols)
                v[i] = fmaf(task.beta, __bfloat162float(source[i]), v[i]);
    }
}

/* Store sixteen consecutive columns of one row straight from registers,
 * choosing the output of a packed projection by column. Used for the ragged
 * right edge of a tile whose width is not a multiple of 64 and for slabs that
 * straddle two outputs; cut points are multiples of 16, so a group of sixteen
 * never does. */
__device__ __forceinline__ void store_direct16(const GemmTask &task, int row, int c,
                                               const uint32_t *acc)
{
    if (row >= task.rows || c >= task.cols)
        return;
    __nv_bfloat16 *out = task.out;
    long long ld = task.ld_out;
    int shift = 0, limit = min(task.cols, task.cut0);
    if (c >= task.cut0) {
        const bool third = c >= task.cut1;
        out = third ? task.out2 : task.out1;
        ld = third ? task.ld_out2 : task.ld_out1;
        shift = third ? task.cut1 : task.cut0;
        limit = third ? task.cols : task.cut1;
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        float v[8];
        const int cc = c + half * 8;
        finish8(task, row, cc, acc + half * 8, v);
        __nv_bfloat16 *target = out + static_cast<long long>(row) * ld + (cc - shift);
        if (cc + 8 <= limit) {
            uint4 packed;
            packed.x = pack_bf16(v[0], v[1]);
            packed.y = pack_bf16(v[2], v[3]);
            packed.z = pack_bf16(v[4], v[5]);
            packed.w = pack_bf16(v[6], v[7]);
            *reinterpret_cast<uint4 *>(target) = packed;
        } else {
            for (int i = 0; i < 8 && cc + i < limit; ++i)
                target[i] = __float2bfloat16_rn(v[i]);
        }
    }
}

/* Epilogue of a whole tile whose width (a multiple of 16 up to 256) is chosen
 * at run time. Full 64-column slabs that lie in one output go through the
 * swizzled staging buffers and TMA stores like epilogue_rows; a slab that
 * straddles two outputs of a packed projection and the ragged right edge are
 * stored straight from registers. */
template <typename Release>
__device__ __forceinline__ void
epilogue_rows_dynamic(const GemmTask &task, const CUtensorMap *map0, const CUtensorMap *map1,
                      const CUtensorMap *map2, uint32_t taddr, int row, int store_row, int col0,
                      int width, int lane, uint8_t *slab, uint32_t &slab_use, Release release)
{
    const int full = width >> 6, tail = (width & 63) >> 4;
#pragma unroll 1
    for (int chunk = 0; chunk < full; ++chunk) {
        uint32_t acc[2][32];
        tmem_ld_32x32(taddr + chunk * 64, acc[0]);
        tmem_ld_32x32(taddr + chunk * 64 + 32, acc[1]);
        tmem_ld_wait();
        if (chunk == full - 1 && tail == 0)
            release();
        const int cbase = col0 + chunk * 64;
        if (cbase >= task.cols)
            continue; /* a slab wholly beyond the last column of the matrix */
        const bool straddles = (cbase < task.cut0 && task.cut0 < cbase + 64) ||
                               (cbase < task.cut1 && task.cut1 < cbase + 64);
        if (straddles) {
#pragma unroll
            for (int g = 0; g < 4; ++g)
                store_direct16(task, row, cbase + g * 16, &acc[g >> 1][(g & 1) * 16]);
            continue;
        }
        const CUtensorMap *map_d = map0;
        int col_shift = 0;
        if (cbase >= task.cut0) {
            const bool third = cbase >= task.cut1;
            map_d = third ? map2 : map1;
            col_shift = third ? task.cut1 : task.cut0;
        }
        uint8_t *buffer_smem = slab + (slab_use & 1) * 4096;
        if (lane == 0)
            tma_store_wait_read<1>();
        __syncwarp();
        stage_row64(task, acc, row, cbase, lane, buffer_smem);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
            tma_store_2d(map_d, buffer_smem, cbase - col_shift, store_row);
            tma_store_commit();
        }
        ++slab_use;
    }
#pragma unroll 1
    for (int g = 0; g < tail; ++g) {
        uint32_t acc[16];
        tmem_ld_32x16(taddr + full * 64 + g * 16, acc);
        tmem_ld_wait();
        if (g == tail - 1)
            release();
        store_direct16(task, row, col0 + full * 64 + g * 16, acc);
    }
}

template <int BN, int Stages, int Mode, int PMajor = kMajorK, int QMajor = kMajorK>
__global__ void __launch_bounds__(kThreads, 1)
    gemm_bf16_tcgen05(const __grid_constant__ CUtensorMap map_p,
                      const __grid_constant__ CUtensorMap map_q,
                      const __grid_constant__ CUtensorMap map_d0,
                      const __grid_constant__ CUtensorMap map_d1,
                      const __grid_constant__ CUtensorMap map_d2, const GemmTask task)
{
    using Layout = GemmSmem<BN, Stages, Mode>;
    constexpr uint32_t kTmemColumns = BN * 2 < 32 ? 32 : BN * 2;
    static_assert((kTmemColumns & (kTmemColumns - 1)) == 0 && kTmemColumns <= 512, "TMEM size");
    static_assert(BN % 16 == 0 && BN >= 16 && BN <= 256, "UMMA N");
    static_assert(Mode != kStoreRows || BN % 64 == 0, "row store works on 64-column slabs");
    static_assert(QMajor == kMajorK || BN % 64 == 0, "MN-major tiles are made of 64-row boxes");

    extern __shared__ uint8_t raw_smem[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) &
                                                ~static_cast<uintptr_t>(1023));
    uint8_t *staging = smem + Stages * Layout::kStageBytes;
    uint64_t *full = reinterpret_cast<uint64_t *>(staging + Layout::kStaging);
    uint64_t *empty = full + Stages;
    uint64_t *tmem_full = empty + Stages;
    uint64_t *tmem_empty = tmem_full + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tmem_empty + 2);
    volatile uint32_t *abort = tmem_slot + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    if constexpr (Mode == kStorePartial) {
        /* the reduction that follows may become resident now; it waits for this
         * grid's completion itself (griddepcontrol.wait) */
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    }
    if (task.skip_if_set != nullptr && *task.skip_if_set != 0)
        return;
    if (task.run_if_set != nullptr && *task.run_if_set == 0)
        return;

    if (threadIdx.x == 0) {
        for (int s = 0; s < Stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&tmem_full[s], 1);
            mbar_init(&tmem_empty[s], 4);
        }
        *abort = 0;
        fence_barrier_init();
        prefetch_tensormap(&map_p);
        prefetch_tensormap(&map_q);
        if (Mode == kStoreRows)
            prefetch_tensormap(&map_d0);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, kTmemColumns);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            /* ---- producer ---- */
            const uint64_t keep = policy_evict_last();
            const uint64_t stream = policy_evict_first();
            /* The operand that is re-read by many tiles stays in L2; the one
             * that is read once per panel is streamed. With few row blocks the
             * column operand (weights) is the streamed one. */
            const uint64_t policy_p = task.r_blocks <= task.panel ? keep : stream;
            const uint64_t policy_q = task.r_blocks <= task.panel ? stream : keep;
            uint32_t stage = 0, phase = 0;
            uint32_t armed = 0, armed_parity = 0;
            bool ok = true;
            Unit u;
            for (int item = 0; ok && fetch_unit(task, item, blockIdx.x, gridDim.x, u); ++item) {
                const int rb = u.rb, cb = u.cb;
                const int p_shift = u.batch * task.batch_p, q_shift = u.batch * task.batch_q;
                for (int kb = u.kb0; kb < u.kb1; ++kb) {
                    if (!mbar_wait(&empty[stage], phase ^ 1, abort)) {
                        report(task.status, abort, kRoleProducer);
                        ok = false;
                        break;
                    }
                    uint8_t *p_tile = smem + stage * Layout::kStageBytes;
                    uint8_t *q_tile = p_tile + Layout::kPBytes;
                    mbar_arrive_expect_tx(&full[stage], Layout::kStageBytes);
                    if constexpr (PMajor == kMajorK) {
                        tma_load_2d_hint(p_tile, &map_p, &full[stage], kb * kBlockK,
                                         rb * kBlockR + p_shift, policy_p);
                    } else {
#pragma unroll
                        for (int g = 0; g < kBlockR / 64; ++g)
                            tma_load_2d_hint(p_tile + g * 8192, &map_p, &full[stage],
                                             rb * kBlockR + g * 64, kb * kBlockK + p_shift,
                                             policy_p);
                    }
                    if constexpr (QMajor == kMajorK) {
                        tma_load_2d_hint(q_tile, &map_q, &full[stage], kb * kBlockK,
                                         cb * BN + q_shift, policy_q);
                    } else {
#pragma unroll
                        for (int g = 0; g < BN / 64; ++g)
                            tma_load_2d_hint(q_tile + g * 8192, &map_q, &full[stage],
                                             cb * BN + g * 64, kb * kBlockK + q_shift, policy_q);
                    }
                    armed |= 1u << stage;
                    armed_parity = (armed_parity & ~(1u << stage)) | (phase << stage);
                    if (++stage == Stages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
            if (!ok) {
                /* Let copies already in flight land before the CTA retires. */
                for (uint32_t s = 0; s < Stages; ++s)
                    if (armed & (1u << s))
                        for (uint32_t spin = 0; spin < (1u << 16); ++spin)
                            if (mbar_try_wait(&full[s], (armed_parity >> s) & 1))
                                break;
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            /* ---- MMA issuer ---- */
            constexpr uint32_t idesc = make_idesc(1, kBlockR, BN, PMajor, QMajor);
            uint32_t stage = 0, phase = 0;
            uint32_t local = 0;
            bool ok = true;
            Unit u;
            for (int item = 0; ok && fetch_unit(task, item, blockIdx.x, gridDim.x, u); ++item, ++local) {
                const int kb0 = u.kb0, kb1 = u.kb1;
                uint32_t buffer = local & 1, use = local >> 1;
                if (!mbar_wait(&tmem_empty[buffer], (use & 1) ^ 1, abort)) {
                    report(task.status, abort, kRoleMmaTmemEmpty);
                    break;
                }
                tcgen05_fence_after();
                uint32_t tmem_d = tmem_base + buffer * BN;
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait_polling(&full[stage], phase, abort)) {
                        report(task.status, abort, kRoleMma);
                        ok = false;
                        break;
                    }
                    tcgen05_fence_after();
                    const uint32_t p_address = smem_u32(smem + stage * Layout::kStageBytes);
                    const uint32_t q_address = p_address + Layout::kPBytes;
#pragma unroll
                    for (int k = 0; k < kBlockK / kUmmaK; ++k) {
                        /* K-major: 16 BF16 along K are 32 bytes further in the same
                         * swizzled lines. MN-major: 16 K indices are 16 lines = 2048 bytes. */
                        const uint64_t desc_p = PMajor == kMajorK
                                                    ? desc_kmajor_sw128(p_address) + 2 * k
                                                    : desc_mnmajor_sw128(p_address + k * 2048, 8192);
                        const uint64_t desc_q = QMajor == kMajorK
                                                    ? desc_kmajor_sw128(q_address) + 2 * k
                                                    : desc_mnmajor_sw128(q_address + k * 2048, 8192);
                        umma_f16(tmem_d, desc_p, desc_q, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(&empty[stage]);
                    if (++stage == Stages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (ok)
                    umma_commit(&tmem_full[buffer]);
            }
        }
    } else {
        /* ---- epilogue ---- */
        const int quarter = warp & 3;
        uint8_t *slab = staging + (warp - 2) * 8192;
        uint32_t local = 0;
        uint32_t slab_use = 0;
        Unit u;
        for (int item = 0; fetch_unit(task, item, blockIdx.x, gridDim.x, u); ++item, ++local) {
            const int rb = u.rb, cb = u.cb, part = u.part, batch = u.batch;
            uint32_t buffer = local & 1, use = local >> 1;
            if (!mbar_wait(&tmem_full[buffer], use & 1, abort)) {
                report(task.status, abort, kRoleEpilogueFull);
                break;
            }
            tcgen05_fence_after();
            const uint32_t taddr = tmem_base + buffer * BN + (static_cast<uint32_t>(quarter * 32) << 16);
            const int row = rb * kBlockR + quarter * 32 + lane;
            const int col0 = cb * BN;

            auto release = [&]() {
                /* accumulator fully read: hand the TMEM buffer back */
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0)
                    mbar_arrive(&tmem_empty[buffer]);
            };
            if constexpr (Mode == kStoreRows) {
              if (u.slot >= 0) {
                float *slot = task.sk_partial + static_cast<long long>(u.slot) * kBlockR * BN;
                epilogue_partial<BN>(slot, taddr, quarter, lane, slab, slab_use, false, release);
              } else {
                const CUtensorMap *map_d = &map_d0;
                int col_shift = 0;
                if (col0 >= task.cut0) {
                    bool third = col0 >= task.cut1;
                    map_d = third ? &map_d2 : &map_d1;
                    col_shift = third ? task.cut1 : task.cut0;
                }
                epilogue_rows<BN>(task, map_d, taddr, row, rb * kBlockR + quarter * 32, col0,
                                  col_shift, lane, slab, slab_use, false, release);
              }
            } else if constexpr (Mode == kStoreFloat) {
                /* FP32 plane of a batched product: this thread owns one row and
                 * writes 32 consecutive floats per piece (128 bytes). */
                float *plane = task.out_float +
                               static_cast<long long>(batch) * task.rows * task.ld_out +
                               static_cast<long long>(row) * task.ld_out;
#pragma unroll 1
                for (int chunk = 0; chunk < BN / 32; ++chunk) {
                    uint32_t acc[32];
                    tmem_ld_32x32(taddr + chunk * 32, acc);
                    tmem_ld_wait();
                    if (chunk == BN / 32 - 1) {
                        tcgen05_fence_before();
                        __syncwarp();
                        if (lane == 0)
                            mbar_arrive(&tmem_empty[buffer]);
                    }
                    const int cbase = col0 + chunk * 32;
                    if (row < task.rows) {
#pragma unroll
                        for (int i = 0; i < 32; i += 4)
                            if (cbase + i < task.cols)
                                *reinterpret_cast<float4 *>(plane + cbase + i) = make_float4(
                                    __uint_as_float(acc[i]), __uint_as_float(acc[i + 1]),
                                    __uint_as_float(acc[i + 2]), __uint_as_float(acc[i + 3]));
                    }
                }
            } else {
                /* Operands are swapped: this thread owns output feature `row`,
                 * the registers run over tokens col0 + i. */
                constexpr int kPiece = BN >= 32 ? 32 : 16;
#pragma unroll 1
                for (int chunk = 0; chunk < BN / kPiece; ++chunk) {
                    uint32_t acc[kPiece];
                    if constexpr (kPiece == 32)
                        tmem_ld_32x32(taddr + chunk * kPiece, acc);
                    else
                        tmem_ld_32x16(taddr + chunk * kPiece, acc);
                    tmem_ld_wait();
                    if (chunk == BN / kPiece - 1) {
                        tcgen05_fence_before();
                        __syncwarp();
                        if (lane == 0)
                            mbar_arrive(&tmem_empty[buffer]);
                    }
                    const int cbase = col0 + chunk * kPiece;
                    if constexpr (Mode == kStorePartial) {
                        const long long plane =
                            static_cast<long long>(task.r_blocks) * kBlockR;
                        float *target = task.partial +
                                        (static_cast<long long>(part) * task.cols + cbase) * plane +
                                        row;
#pragma unroll
                        for (int i = 0; i < kPiece; ++i)
                            if (cbase + i < task.cols)
                                target[i * plane] = __uint_as_float(acc[i]);
                    } else {
                        if (row < task.rows) {
                            float bias =
                                task.bias != nullptr ? __bfloat162float(task.bias[row]) : 0.f;
#pragma unroll
                            for (int i = 0; i < kPiece; ++i) {
                                if (cbase + i < task.cols) {
                                    float v = task.alpha * __uint_as_float(acc[i]) + bias;
                                    long long at = static_cast<long long>(cbase + i);
                                    if (task.beta != 0.f)
                                        v = fmaf(task.beta,
                                                 __bfloat162float(
                                                     task.addend[at * task.ld_add + row]),
                                                 v);
                                    task.out[at * task.ld_out + row] = __float2bfloat16_rn(v);
                                }
                            }
                        }
                    }
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

/* Ordered reduction of the K splits written by kStorePartial:
 * out[c*ld_out + r] = rnd(alpha * sum_s partial[s][c][r] + beta*addend + bias[r]).
 * Launched as a programmatic dependent of the product kernel (which releases
 * its dependents when it starts), so that this grid is already resident when the
 * product ends and only the wait below separates them; the loads of eight
 * splits are in flight at a time and are added in ascending split order. */
__global__ void __launch_bounds__(256)
    gemm_split_reduce(int rows, int cols, int split, long long plane, float alpha, float beta,
                      const float *partial, const __nv_bfloat16 *addend, long long ld_add,
                      const __nv_bfloat16 *bias, __nv_bfloat16 *out, long long ld_out)
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    const int c = blockIdx.y;
    if (r >= rows)
        return;
    const float *source = partial + static_cast<long long>(c) * plane + r;
    const long long step = static_cast<long long>(cols) * plane;
    float sum = 0.f;
    int s = 0;
    for (; s + 8 <= split; s += 8) {
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
            v[i] = __ldcg(source + (s + i) * step);
#pragma unroll
        for (int i = 0; i < 8; ++i)
            sum += v[i];
    }
    for (; s < split; ++s)
        sum += __ldcg(source + s * step);
    float v = alpha * sum;
    if (bias != nullptr)
        v += __bfloat162float(bias[r]);
    if (beta != 0.f)
        v = fmaf(beta, __bfloat162float(addend[c * ld_add + r]), v);
    out[c * ld_out + r] = __float2bfloat16_rn(v);
}

/* Launch gemm_split_reduce behind a product kernel on `stream` with programmatic
 * stream serialization. */
inline cudaError_t launch_split_reduce(cudaStream_t stream, int rows, int cols, int split,
                                       long long plane, float alpha, float beta,
                                       const float *partial, const __nv_bfloat16 *addend,
                                       long long ld_add, const __nv_bfloat16 *bias,
                                       __nv_bfloat16 *out, long long ld_out)
{
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3((rows + 255) / 256, cols);
    config.blockDim = dim3(256);
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, gemm_split_reduce, rows, cols, split, plane, alpha, beta,
                              partial, addend, ld_add, bias, out, ld_out);
}

/* Second pass of the stream-K tail: add the pieces of every stream-K tile in
 * ascending K order, apply alpha, bias and beta*addend, round once, store BF16.
 * One thread per eight consecutive columns; blockIdx.x is the stream-K column
 * block, blockIdx.z the row block, `grid` the number of CTAs the product kernel
 * ran with. out1/out2 are the extra outputs of a packed projection (columns
 * from cut0 and cut1 on). */
template <int BN>
__global__ void __launch_bounds__(256)
    sk_fixup(const GemmTask task, int grid, __nv_bfloat16 *out1, long long ld1,
             __nv_bfloat16 *out2, long long ld2)
{
    const int vector = blockIdx.y * 256 + threadIdx.x;
    const int r = vector / (BN / 8), c8 = (vector % (BN / 8)) * 8;
    const int rb = blockIdx.z, cb = task.dp_cols + blockIdx.x;
    const int row = rb * kBlockR + r, col = cb * BN + c8;
    if (row >= task.rows || col >= task.cols)
        return;
    float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    sum_pieces<BN>(
        task, grid / task.r_blocks, blockIdx.x, r, c8,
        [&](int team, int piece) { return 2ll * (team * task.r_blocks + rb) + piece; }, sum);
    __nv_bfloat16 *out = task.out;
    long long ld = task.ld_out;
    int shift = 0, limit = min(task.cols, task.cut0);
    if (col >= task.cut0) {
        const bool third = col >= task.cut1;
        out = third ? out2 : out1;
        ld = third ? ld2 : ld1;
        shift = third ? task.cut1 : task.cut0;
        limit = third ? task.cols : task.cut1;
    }
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        v[i] = task.alpha * sum[i];
        if (col + i < task.cols) {
            if (task.bias != nullptr)
                v[i] += __bfloat162float(task.bias[col + i]);
            if (task.beta != 0.f)
                v[i] = fmaf(task.beta,
                            __bfloat162float(
                                task.addend[static_cast<long long>(row) * task.ld_add + col + i]),
                            v[i]);
        }
    }
    __nv_bfloat16 *target = out + static_cast<long long>(row) * ld + (col - shift);
    if (col + 8 <= limit) {
        uint4 packed;
        packed.x = pack_bf16(v[0], v[1]);
        packed.y = pack_bf16(v[2], v[3]);
        packed.z = pack_bf16(v[4], v[5]);
        packed.w = pack_bf16(v[6], v[7]);
        *reinterpret_cast<uint4 *>(target) = packed;
    } else {
        for (int i = 0; i < 8 && col + i < limit; ++i)
            target[i] = __float2bfloat16_rn(v[i]);
    }
}

} // namespace sm100
