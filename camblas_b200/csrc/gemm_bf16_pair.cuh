/*
 * BF16 GEMM with two-SM tensor-core instructions (tcgen05.mma.cta_group::2).
 *
 * Two CTAs on neighbouring SMs form a cluster and compute one 256 x BN tile of
 * D[R,C] = P[R,K] . Q[C,K]^T together: each CTA stages its own 128 rows of P and
 * its own BN/2 rows of Q, the leader CTA (cluster rank 0) issues one MMA of
 * shape M=256, N=BN, K=16 that reads both CTAs' shared memory, and each CTA
 * receives its 128 accumulator rows in its own tensor memory. Compared with the
 * one-SM kernel this halves the Q bytes every SM pulls from L2 and keeps in
 * shared memory per multiply (32 KB instead of 48 KB per 64-deep K block at
 * BN=256), which is what that kernel is short of. The ring holds six K blocks
 * (192 KB); with Sub=2 a stage is two of them, so that every barrier round
 * trip, expect_tx and pair of commits covers eight MMAs instead of four.
 *
 * Roles per CTA (192 threads): warp 0 = TMA producer for this CTA's halves
 * (every CTA fetches its own bytes; no load is shared between CTAs), warp 1 =
 * MMA issuer in the leader and idle in the peer, warps 2-5 = epilogue for this
 * CTA's 128 rows.
 *
 * Barriers. Every CTA has the same barrier objects at the same shared-memory
 * offsets; the ones that synchronise the pair live in the leader:
 *   full[s]        leader: one arrival (leader's producer, which also posts the
 *                  byte count of BOTH CTAs' loads) + the bytes of both CTAs'
 *                  TMA loads (the peer's loads name the leader's barrier);
 *   empty[s]       one per CTA, arrived by two tcgen05.commit of the leader,
 *                  one to its own barrier and one to the peer's;
 *   tmem_full[b]   one per CTA, same mechanism;
 *   tmem_empty[b]  leader: eight arrivals, four epilogue warps of each CTA (the
 *                  peer's arrive remotely).
 * Waits are bounded as in the one-SM kernel. The two CTAs meet at a cluster
 * barrier after set-up and before tear-down so that neither touches the other's
 * shared memory outside that window.
 */
#pragma once

#include "gemm_bf16_tcgen05.cuh"

namespace sm100
{

__device__ __forceinline__ uint32_t cluster_rank()
{
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    return rank;
}

__device__ __forceinline__ void cluster_sync()
{
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

/* Shared-memory address of the same object in the CTA of rank `rank`. */
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local_address, uint32_t rank)
{
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_address), "r"(rank));
    return remote;
}

__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_address)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_address)
                 : "memory");
}

/* TMA load whose completion bytes are counted on a barrier that may live in the
 * other CTA of the pair (address in the cluster's shared window). */
__device__ __forceinline__ void tma_load_2d_pair(void *smem, const CUtensorMap *map,
                                                 uint32_t barrier_cluster_address, int x, int y,
                                                 uint64_t policy)
{
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
                 ".L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;" ::"r"(smem_u32(smem)),
                 "l"(map), "r"(barrier_cluster_address), "r"(x), "r"(y), "l"(policy)
                 : "memory");
}

__device__ __forceinline__ void tmem_alloc_pair(uint32_t *smem_result, uint32_t columns)
{
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(smem_result)),
                 "r"(columns)
                 : "memory");
}

__device__ __forceinline__ void tmem_relinquish_pair()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc_pair(uint32_t address, uint32_t columns)
{
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(address), "r"(columns)
                 : "memory");
}

__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                              uint32_t idesc, uint32_t accumulate)
{
    asm volatile("{\n"
                 ".reg .pred p;\n"
                 "setp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
                 "}\n" ::"r"(tmem_d),
                 "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
                 : "memory");
}

/* Arrive on a barrier (cluster shared address, this CTA's or the peer's) once
 * every MMA issued so far by this thread is done. */
__device__ __forceinline__ void umma_commit_pair(uint32_t barrier_cluster_address)
{
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     barrier_cluster_address)
                 : "memory");
}

/* One commit that arrives on the barrier at the same shared-memory offset in both
 * CTAs of the pair. */
__device__ __forceinline__ void umma_commit_both(uint32_t barrier)
{
    const uint16_t both = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
                 "[%0], %1;" ::"r"(barrier),
                 "h"(both)
                 : "memory");
}

constexpr int kPairRows = 256;
/* What the epilogue of the two-SM kernel does with a finished tile. */
constexpr int kEpiStore = 0;  /* alpha, bias, addend, one rounding, TMA store */
constexpr int kEpiPush = 1;   /* BF16 partial tile to the GPU that owns it (row_parallel.cuh) */
constexpr int kEpiSwiglu = 2; /* tile = 128 gate + 128 up columns: SiLU(gate) * up */
constexpr int kEpiSwigluQuant = 3; /* the same, written as E4M3 with 1 x 128 scales */


template <int BN, int Stages, int Sub = 1> struct PairSmem {
    static constexpr int kPBytes = kBlockR * kBlockK * 2;      /* this CTA's 128 rows of P */
    static constexpr int kQBytes = (BN / 2) * kBlockK * 2;     /* this CTA's half of the Q tile */
    static constexpr int kBlockBytes = kPBytes + kQBytes;      /* one 64-deep K block */
    static constexpr int kStageBytes = Sub * kBlockBytes;      /* Sub K blocks per stage */
    static constexpr int kTotal = Stages * kStageBytes + kStagingBytes + 256 + 1024;
};

/* task.r_blocks counts 256-row blocks here; everything else as in GemmTask.
 * BNT is the tile width, or 0 when the width comes from task.width at run time
 * (any multiple of 16 from 64 to 256; Q must then be K-major and the stage
 * layout and TMEM buffers are those of the 256-column tile). */
template <int BNT, int Stages, int PMajor = kMajorK, int QMajor = kMajorK, int Sub = 1,
          int Epi = kEpiStore>
__global__ void __launch_bounds__(kThreads, 1)
    gemm_bf16_pair(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q,
                   const __grid_constant__ CUtensorMap map_d0,
                   const __grid_constant__ CUtensorMap map_d1,
                   const __grid_constant__ CUtensorMap map_d2, const GemmTask task)
{
    constexpr bool kDynamic = BNT == 0;
    constexpr int kLayoutWidth = kDynamic ? 256 : BNT;
    using Layout = PairSmem<kLayoutWidth, Stages, Sub>;
    constexpr uint32_t kTmemColumns = kLayoutWidth * 2;
    static_assert(BNT == 256 || BNT == 128 || BNT == 0, "pair tiles: 256, 128 or run-time width");
    static_assert(!kDynamic || QMajor == kMajorK, "run-time width needs a K-major Q operand");
    constexpr bool Push = Epi == kEpiPush;
    static_assert(Epi == kEpiStore || !kDynamic, "the special epilogues work on fixed-width tiles");
    static_assert((Epi != kEpiSwiglu && Epi != kEpiSwigluQuant) || (BNT == 256 && QMajor == kMajorK),
                  "the SwiGLU epilogue pairs 128 gate with 128 up columns of a K-major weight");
    const int BN = kDynamic ? task.width : BNT;
    const int kHalf = BN / 2;
    const uint32_t stage_bytes = Layout::kPBytes + kHalf * kBlockK * 2; /* bytes one CTA loads */

    extern __shared__ uint8_t raw_smem[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) &
                                                ~static_cast<uintptr_t>(1023));
    uint8_t *staging = smem + Stages * Layout::kStageBytes;
    uint64_t *full = reinterpret_cast<uint64_t *>(staging + kStagingBytes);
    uint64_t *empty = full + Stages;
    uint64_t *tmem_full = empty + Stages;
    uint64_t *tmem_empty = tmem_full + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tmem_empty + 2);
    volatile uint32_t *abort = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if constexpr (Push) {
        /* The kernel that sums the pushed tiles is launched as a programmatic
         * dependent: it may become resident as soon as every CTA here has run
         * this, and then waits on flags, not on this kernel's completion. */
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    }
    const uint32_t rank = cluster_rank();
    const bool leader = rank == 0;
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < Stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&tmem_full[s], 1);
            mbar_init(&tmem_empty[s], 8);
        }
        *abort = 0;
        fence_barrier_init();
        prefetch_tensormap(&map_p);
        prefetch_tensormap(&map_q);
        prefetch_tensormap(&map_d0);
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, kTmemColumns);
        tmem_relinquish_pair();
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            /* ---- producer: this CTA's rows of P and its half of the Q tile ---- */
            const uint64_t keep = policy_evict_last(), stream = policy_evict_first();
            /* Both operands are re-read by other CTAs through L2 (the weight tile by
             * the other row blocks, the token tile by every column tile); measured
             * on B200, asking L2 to keep both is as good as or better than marking
             * the weights as streamed. */
            const uint64_t policy_p = keep, policy_q = keep;
            (void)stream;
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            Unit u;
            for (int item = 0; ok && fetch_unit(task, item, pair, pairs, u); ++item) {
                const int p_row = u.rb * kPairRows + rank * kBlockR;
                const int q_row = u.cb * BN + rank * kHalf;
                for (int kb = u.kb0; kb < u.kb1; kb += Sub) {
                    if (!mbar_wait_polling(&empty[stage], phase ^ 1, abort)) {
                        report(task.status, abort, kRoleProducer);
                        ok = false;
                        break;
                    }
                    const uint32_t barrier = map_to_rank(smem_u32(&full[stage]), 0);
                    /* a stage holds up to Sub 64-deep K blocks; the last stage of a
                     * piece of work may hold fewer */
                    const int blocks = min(Sub, u.kb1 - kb);
                    if (leader)
                        mbar_arrive_expect_tx(&full[stage], 2 * blocks * stage_bytes);
                    for (int sub = 0; sub < blocks; ++sub) {
                        uint8_t *p_tile =
                            smem + stage * Layout::kStageBytes + sub * Layout::kBlockBytes;
                        uint8_t *q_tile = p_tile + Layout::kPBytes;
                        const int k0 = (kb + sub) * kBlockK;
                        if constexpr (PMajor == kMajorK) {
                            tma_load_2d_pair(p_tile, &map_p, barrier, k0, p_row, policy_p);
                        } else {
#pragma unroll
                            for (int g = 0; g < kBlockR / 64; ++g)
                                tma_load_2d_pair(p_tile + g * 8192, &map_p, barrier, p_row + g * 64,
                                                 k0, policy_p);
                        }
                        if constexpr (QMajor == kMajorK) {
                            tma_load_2d_pair(q_tile, &map_q, barrier, k0, q_row, policy_q);
                        } else {
                            for (int g = 0; g < kHalf / 64; ++g)
                                tma_load_2d_pair(q_tile + g * 8192, &map_q, barrier, q_row + g * 64,
                                                 k0, policy_q);
                        }
                    }
                    if (++stage == Stages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
            if (!ok) {
                /* let copies already in flight land before the pair retires */
                for (int wait = 0; wait < 64; ++wait)
                    __nanosleep(1000);
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && leader) {
            /* ---- MMA issuer (leader only) ---- */
            const uint32_t idesc = make_idesc(1, kPairRows, BN, PMajor, QMajor);
            uint32_t stage = 0, phase = 0, local = 0;
            bool ok = true;
            Unit u;
            for (int item = 0; ok && fetch_unit(task, item, pair, pairs, u); ++item, ++local) {
                const uint32_t buffer = local & 1, use = local >> 1;
                if (!mbar_wait(&tmem_empty[buffer], (use & 1) ^ 1, abort)) {
                    report(task.status, abort, kRoleMmaTmemEmpty);
                    break;
                }
                tcgen05_fence_after();
                const uint32_t tmem_d = tmem_base + buffer * kLayoutWidth;
                for (int kb = u.kb0; kb < u.kb1; kb += Sub) {
                    /* polled, not suspended: measured against the suspending wait in one
                     * process, alternating, the polling form was level or up to 5 % faster
                     * on the Llama projections and their shards */
                    if (!mbar_wait_polling(&full[stage], phase, abort)) {
                        report(task.status, abort, kRoleMma);
                        ok = false;
                        break;
                    }
                    tcgen05_fence_after();
                    const int blocks = min(Sub, u.kb1 - kb);
                    for (int sub = 0; sub < blocks; ++sub) {
                    const uint32_t p_address =
                        smem_u32(smem + stage * Layout::kStageBytes + sub * Layout::kBlockBytes);
                    const uint32_t q_address = p_address + Layout::kPBytes;
#pragma unroll
                    for (int k = 0; k < kBlockK / kUmmaK; ++k) {
                        const uint64_t desc_p = PMajor == kMajorK
                                                    ? desc_kmajor_sw128(p_address) + 2 * k
                                                    : desc_mnmajor_sw128(p_address + k * 2048, 8192);
                        const uint64_t desc_q = QMajor == kMajorK
                                                    ? desc_kmajor_sw128(q_address) + 2 * k
                                                    : desc_mnmajor_sw128(q_address + k * 2048, 8192);
                        umma_f16_pair(tmem_d, desc_p, desc_q, idesc,
                                      (kb > u.kb0 || k > 0 || sub > 0) ? 1u : 0u);
                    }
                    }
                    /* free the stage in both CTAs: one commit that arrives on both
                     * barriers (a commit costs this thread about a hundred cycles, and
                     * with eight MMAs and two commits per stage its instruction stream,
                     * not the operand feed, was what held the tensor pipe at 82 %) */
                    umma_commit_both(smem_u32(&empty[stage]));
                    if (++stage == Stages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (ok)
                    umma_commit_both(smem_u32(&tmem_full[buffer]));
            }
        }
    } else {
        /* ---- epilogue: this CTA's 128 accumulator rows ---- */
        const int quarter = warp & 3;
        uint8_t *const own_slab = staging + (warp - 2) * 8192;
        /* For the CTA's last piece of work the operand ring is idle once the
         * accumulator is complete (all loads landed, all MMAs read them), so the
         * epilogue borrows it: one 4 KB buffer per slab, none reused. */
        uint8_t *const ring_slab = smem + (warp - 2) * (kLayoutWidth / 32) * 4096;
        static_assert(4 * (kLayoutWidth / 32) * 4096 <= Stages * Layout::kStageBytes,
                      "borrowed staging fits in the operand ring");
        uint32_t local = 0, slab_use = 0;
        Unit u, following;
        bool more = fetch_unit(task, 0, pair, pairs, u);
        for (int item = 0; more; ++item, ++local, u = following) {
            more = fetch_unit(task, item + 1, pair, pairs, following);
            const bool roomy = !more;
            uint8_t *slab = roomy ? ring_slab : own_slab;
            const uint32_t buffer = local & 1, use = local >> 1;
            if (!mbar_wait(&tmem_full[buffer], use & 1, abort)) {
                report(task.status, abort, kRoleEpilogueFull);
                break;
            }
            tcgen05_fence_after();
            const uint32_t taddr =
                tmem_base + buffer * kLayoutWidth + (static_cast<uint32_t>(quarter * 32) << 16);
            const int row0 = u.rb * kPairRows + rank * kBlockR + quarter * 32;
            const int col0 = u.cb * BN;
            auto release = [&]() {
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0)
                    mbar_arrive_cluster(map_to_rank(smem_u32(&tmem_empty[buffer]), 0));
            };
            if constexpr (Epi == kEpiSwiglu || Epi == kEpiSwigluQuant) {
                if (u.slot >= 0) {
                    float *slot = task.sk_partial +
                                  (static_cast<long long>(u.slot) * 2 + rank) * kBlockR * BNT;
                    epilogue_partial<kLayoutWidth>(slot, taddr, quarter, lane, slab, slab_use, roomy,
                                                   release);
                } else if constexpr (Epi == kEpiSwigluQuant) {
                    epilogue_swiglu_quant(task, taddr, row0 + lane, u.cb * 128, release);
                } else {
                    epilogue_swiglu(task, &map_d0, taddr, row0, u.cb * 128, lane, slab, slab_use,
                                    roomy, release);
                }
            } else if constexpr (Push) {
                /* partial sums of a K range split over GPUs: to the tile's owner */
                const int unit = ((u.rb * task.c_blocks + u.cb) * 2 + static_cast<int>(rank)) * 4 +
                                 quarter;
                epilogue_push<kLayoutWidth>(task, taddr, u.cb % task.push_world, unit, lane, slab,
                                            slab_use, roomy, release);
            } else if constexpr (kDynamic) {
                epilogue_rows_dynamic(task, &map_d0, &map_d1, &map_d2, taddr, row0 + lane, row0, col0,
                                      BN, lane, own_slab, slab_use, release);
            } else if (u.slot >= 0) {
                float *slot = task.sk_partial +
                              (static_cast<long long>(u.slot) * 2 + rank) * kBlockR * BNT;
                epilogue_partial<kLayoutWidth>(slot, taddr, quarter, lane, slab, slab_use, roomy,
                                               release);
            } else {
                const CUtensorMap *map_d = &map_d0;
                int col_shift = 0;
                if (col0 >= task.cut0) {
                    const bool third = col0 >= task.cut1;
                    map_d = third ? &map_d2 : &map_d1;
                    col_shift = third ? task.cut1 : task.cut0;
                }
                epilogue_rows<kLayoutWidth>(task, map_d, taddr, row0 + lane, row0, col0, col_shift,
                                            lane, slab, slab_use, roomy, release);
            }
        }
        if (lane == 0)
            tma_store_wait_all<0>();
        __syncwarp();
    }

    tcgen05_fence_before();
    __syncthreads();
    cluster_sync();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc_pair(tmem_base, kTmemColumns);
    }
}

/* Second pass of the stream-K tail of the pair kernel: like sk_fixup, with
 * 256-row tiles whose two 128-row halves were written by the two CTAs of a
 * pair (slot = (2*pair + piece)*2 + half). blockIdx.z = 256-row block. */
template <int BN>
__global__ void __launch_bounds__(256)
    sk_fixup_pair(const GemmTask task, int pairs, __nv_bfloat16 *out1, long long ld1,
                  __nv_bfloat16 *out2, long long ld2)
{
    const int vector = blockIdx.y * 256 + threadIdx.x;
    const int r = vector / (BN / 8), c8 = (vector % (BN / 8)) * 8; /* r in [0, 256) */
    const int rb = blockIdx.z, cb = task.dp_cols + blockIdx.x;
    const int row = rb * kPairRows + r, col = cb * BN + c8;
    if (row >= task.rows || col >= task.cols)
        return;
    float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    sum_pieces<BN>(
        task, pairs / task.r_blocks, blockIdx.x, r & 127, c8,
        [&](int team, int piece) {
            return (2ll * (team * task.r_blocks + rb) + piece) * 2 + (r >> 7);
        },
        sum);
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

/* Second pass of the stream-K tail for SwiGLU tiles (256 packed columns = 128
 * gate + 128 up): one thread per eight output columns adds the pieces of its
 * gate columns and of the matching up columns in ascending K order and stores
 * SiLU(gate) * up. grid = (stream-K column blocks, 16, 256-row blocks). */
template <bool Quantise>
__global__ void __launch_bounds__(256) sk_fixup_pair_swiglu(const GemmTask task, int pairs)
{
    const int vector = blockIdx.y * 256 + threadIdx.x;
    const int r = vector >> 4, c8 = (vector & 15) * 8; /* r in [0, 256), c8 in [0, 128) */
    const int rb = blockIdx.z, cb = task.dp_cols + blockIdx.x;
    const int row = rb * kPairRows + r, col = cb * 128 + c8; /* output column */
    const bool live = row < task.rows && cb * 256 + c8 < task.cols;
    if (!Quantise && !live)
        return;
    float gate[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    float up[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    auto slot_of = [&](int team, int piece) {
        return (2ll * (team * task.r_blocks + rb) + piece) * 2 + (r >> 7);
    };
    if (live) {
        sum_pieces<256>(task, pairs / task.r_blocks, blockIdx.x, r & 127, c8, slot_of, gate);
        sum_pieces<256>(task, pairs / task.r_blocks, blockIdx.x, r & 127, 128 + c8, slot_of, up);
    }
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
        v[i] = swiglu_value(task.alpha * gate[i], task.alpha * up[i]);
    uint4 packed;
    packed.x = pack_bf16(v[0], v[1]);
    packed.y = pack_bf16(v[2], v[3]);
    packed.z = pack_bf16(v[4], v[5]);
    packed.w = pack_bf16(v[6], v[7]);
    if constexpr (!Quantise) {
        *reinterpret_cast<uint4 *>(task.out + static_cast<long long>(row) * task.ld_out + col) = packed;
    } else {
        /* sixteen neighbouring threads hold the 128 outputs of one row: their
         * largest magnitude (of the BF16-rounded values) is the group's */
        const uint32_t words[4] = {packed.x, packed.y, packed.z, packed.w};
        float largest = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w)
            largest = fmaxf(largest, fmaxf(fabsf(bf16_low(words[w])), fabsf(bf16_high(words[w]))));
#pragma unroll
        for (int offset = 1; offset < 16; offset <<= 1)
            largest = fmaxf(largest, __shfl_xor_sync(0xffffffffu, largest, offset));
        if (!live)
            return;
        const float maximum = fmaxf(largest, 1e-10f);
        if ((vector & 15) == 0)
            task.quant_scale[static_cast<long long>(row) * task.quant_groups + cb] =
                __fmul_rn(maximum, 1.0f / 448.0f);
        const float inverse = __fdiv_rn(448.0f, maximum);
        uint2 bytes;
        bytes.x = quantise_e4m3(bf16_low(words[0]), inverse) |
                  (quantise_e4m3(bf16_high(words[0]), inverse) << 8) |
                  (quantise_e4m3(bf16_low(words[1]), inverse) << 16) |
                  (quantise_e4m3(bf16_high(words[1]), inverse) << 24);
        bytes.y = quantise_e4m3(bf16_low(words[2]), inverse) |
                  (quantise_e4m3(bf16_high(words[2]), inverse) << 8) |
                  (quantise_e4m3(bf16_low(words[3]), inverse) << 16) |
                  (quantise_e4m3(bf16_high(words[3]), inverse) << 24);
        *reinterpret_cast<uint2 *>(task.quant_out + static_cast<long long>(row) * task.ld_quant + col) =
            bytes;
    }
}

} // namespace sm100
