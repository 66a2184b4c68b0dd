/*
 * BF16 GEMM for products with few tiles and a long K: the K range of every tile
 * is split over the CTAs of a thread-block cluster and the partial accumulators
 * are added through distributed shared memory.
 *
 * The other kernels of this library handle "fewer tiles than SMs" by writing
 * FP32 partial sums to global scratch and adding them in a second launch
 * (kStorePartial + gemm_split_reduce, the stream-K pieces + sk_fixup). For the
 * shapes where that matters - a few token rows against a Llama-sized weight,
 * the QKV shard of a rank at tensor-parallel 4 or 8 - the second launch and the
 * scratch round trip cost as much as the multiplication. Here a cluster of S
 * CTAs (2..8) owns one 128 x BN tile: CTA p multiplies K range p into its own
 * tensor memory exactly as gemm_bf16_tcgen05 does (TMA producer warp, MMA
 * issuer warp, four epilogue warps), and then
 *   1. every epilogue warp copies its 32 accumulator rows from tensor memory
 *      into the CTA's own operand ring (idle once its last MMA is complete);
 *   2. the cluster meets at a hardware barrier (release / acquire);
 *   3. every CTA reads the rows it OWNS (row i of the tile belongs to CTA
 *      i*S/128) out of all S rings with ld.shared::cluster, whole 512-byte
 *      stretches per warp and all S loads of a value in flight together, adds
 *      them in K order in FP32, applies alpha, bias and beta*addend, rounds
 *      once and stores its rows;
 *   4. a second cluster barrier keeps every ring alive until all have read it.
 * An earlier form pushed: each lane stored its accumulator row, 16 bytes at a
 * time, into the owner's ring, and the owner added from there. A timeline taken
 * inside that kernel on the QKV shard of a rank at tensor-parallel 8 (512 x
 * 8192 -> 1280, six CTAs per tile, 21 us in all) showed 6 us for the stores
 * into the other CTAs, 0.9 us for their fence and 2.7 us for the additions
 * against 8 us for the multiplication itself.
 *
 * The sums are added in ascending K order by exactly one CTA per row, so results
 * are repeatable. Every thread of the cluster reaches both barriers whatever its
 * bounded waits did before (nothing returns early), so they cannot hang.
 *
 * Mode kStoreRows: D[R,C] row-major (tokens on the tile rows), optional second
 * and third outputs of a packed projection. Mode kStoreColumns: operands
 * swapped (weights on the tile rows, up to 64 tokens on the columns), D^T stored.
 */
#pragma once

#include "gemm_bf16_pair.cuh"

namespace sm100
{

__device__ __forceinline__ uint32_t cluster_size()
{
    uint32_t size;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(size));
    return size;
}

__device__ __forceinline__ float4 ld_cluster_v4(uint32_t cluster_address)
{
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "r"(cluster_address)
                 : "memory");
    return v;
}

__device__ __forceinline__ float ld_cluster_f32(uint32_t cluster_address)
{
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(cluster_address) : "memory");
    return v;
}

constexpr int kInboxPad = 4; /* floats added to a row of FP32 sums in shared memory: keeps 16-byte alignment, spreads banks */

/* First tile row owned by CTA `part` of `parts`: rows are dealt out in
 * contiguous, nearly equal ranges. */
__host__ __device__ constexpr int cluster_first_row(int part, int parts)
{
    return (part * kBlockR + parts - 1) / parts;
}

template <int BN, int Stages, int Mode>
__global__ void __launch_bounds__(kThreads, 1)
    gemm_bf16_cluster(const __grid_constant__ CUtensorMap map_p,
                      const __grid_constant__ CUtensorMap map_q, const GemmTask task)
{
    static_assert(Mode == kStoreRows || Mode == kStoreColumns, "cluster split: rows or swapped");
    using Layout = GemmSmem<BN, Stages, kStoreColumns>; /* ring + barriers, no staging buffers */
    constexpr uint32_t kTmemColumns = BN < 32 ? 32 : BN;
    /* FP32 sums of this CTA's K range over the ring. Rows: [tile row][kPitch], a
     * row is read by its owner in 16-byte pieces. Swapped: [token][kColPitch], the
     * output features of a token are contiguous in memory, so they are here. */
    constexpr int kPitch = BN + kInboxPad;
    constexpr int kColPitch = kBlockR + kInboxPad;
    static_assert(kBlockR * kPitch * 4 <= Stages * Layout::kStageBytes &&
                      BN * kColPitch * 4 <= Stages * Layout::kStageBytes,
                  "the sums fit in the operand ring");

    extern __shared__ uint8_t raw_smem[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) &
                                                ~static_cast<uintptr_t>(1023));
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + Stages * Layout::kStageBytes);
    uint64_t *empty = full + Stages;
    uint64_t *tmem_full = empty + Stages;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tmem_full + 1);
    volatile uint32_t *abort = tmem_slot + 1;
    const uint32_t sums = smem_u32(smem);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int parts = static_cast<int>(cluster_size());
    const int part = static_cast<int>(cluster_rank());
    int rb, cb, batch;
    locate_tile(task, blockIdx.x / parts, rb, cb, batch);
    const int per_part = (task.k_blocks + parts - 1) / parts;
    const int kb0 = min(task.k_blocks, part * per_part), kb1 = min(task.k_blocks, kb0 + per_part);

    if (threadIdx.x == 0) {
        for (int s = 0; s < Stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(tmem_full, 1);
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

    if (warp == 0) {
        if (lane == 0) {
            /* ---- producer: this CTA's K range of the tile ---- */
            const uint64_t keep = policy_evict_last(), stream = policy_evict_first();
            /* swapped: P is the weight, read once; rows: Q is the weight */
            const uint64_t policy_p = Mode == kStoreColumns ? stream : keep;
            const uint64_t policy_q = Mode == kStoreColumns ? keep : stream;
            uint32_t stage = 0, phase = 0;
            for (int kb = kb0; kb < kb1; ++kb) {
                if (!mbar_wait(&empty[stage], phase ^ 1, abort)) {
                    report(task.status, abort, kRoleProducer);
                    break;
                }
                uint8_t *p_tile = smem + stage * Layout::kStageBytes;
                mbar_arrive_expect_tx(&full[stage], Layout::kStageBytes);
                tma_load_2d_hint(p_tile, &map_p, &full[stage], kb * kBlockK, rb * kBlockR, policy_p);
                tma_load_2d_hint(p_tile + Layout::kPBytes, &map_q, &full[stage], kb * kBlockK, cb * BN,
                                 policy_q);
                if (++stage == Stages) {
                    stage = 0;
                    phase ^= 1;
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            /* ---- MMA issuer ---- */
            constexpr uint32_t idesc = make_idesc(1, kBlockR, BN, kMajorK, kMajorK);
            uint32_t stage = 0, phase = 0;
            bool ok = true;
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
                for (int k = 0; k < kBlockK / kUmmaK; ++k)
                    umma_f16(tmem_base, desc_kmajor_sw128(p_address) + 2 * k,
                             desc_kmajor_sw128(q_address) + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
                umma_commit(&empty[stage]);
                if (++stage == Stages) {
                    stage = 0;
                    phase ^= 1;
                }
            }
            if (ok) {
                if (kb1 > kb0)
                    umma_commit(tmem_full);
                else
                    mbar_arrive(tmem_full); /* an empty K range: nothing to wait for */
            }
        }
    } else {
        /* ---- epilogue warps, step 1: the accumulators into this CTA's ring ---- */
        const int quarter = warp & 3;
        const bool ok = mbar_wait(tmem_full, 0, abort);
        if (!ok)
            report(task.status, abort, kRoleEpilogueFull);
        tcgen05_fence_after();
        if (ok) {
            const int row = quarter * 32 + lane; /* row of the tile */
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
            constexpr int kPiece = BN >= 32 ? 32 : 16;
#pragma unroll 1
            for (int chunk = 0; chunk < BN / kPiece; ++chunk) {
                uint32_t acc[kPiece];
                if (kb1 > kb0) {
                    if constexpr (kPiece == 32)
                        tmem_ld_32x32(taddr + chunk * kPiece, acc);
                    else
                        tmem_ld_32x16(taddr + chunk * kPiece, acc);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int i = 0; i < kPiece; ++i)
                        acc[i] = 0u;
                }
                if constexpr (Mode == kStoreRows) {
                    const uint32_t target = sums + (row * kPitch + chunk * kPiece) * 4;
#pragma unroll
                    for (int i = 0; i < kPiece; i += 4)
                        st_shared_v4(target + i * 4, acc[i], acc[i + 1], acc[i + 2], acc[i + 3]);
                } else {
#pragma unroll
                    for (int i = 0; i < kPiece; ++i)
                        asm volatile("st.shared.b32 [%0], %1;" ::"r"(
                                         sums + ((chunk * kPiece + i) * kColPitch + row) * 4),
                                     "r"(acc[i])
                                     : "memory");
                }
            }
        }
    }

    /* step 2: every ring holds its CTA's sums (or the CTA has given up and said so) */
    tcgen05_fence_before();
    __syncthreads();
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");

    if (*abort == 0) {
        /* step 3: add the sums of the owned rows in K order and store them. All six
         * warps take part: a load from another CTA's ring takes most of a
         * microsecond, so what counts is how many are in flight. */
        const int first = cluster_first_row(part, parts);
        const int owned = cluster_first_row(part + 1, parts) - first;
        const int thread = threadIdx.x; /* 0..191 */
        if constexpr (Mode == kStoreRows) {
            /* four consecutive columns per thread and item, four items in flight: every
             * load instruction of a warp reads 512 contiguous bytes of one ring */
            constexpr int kQuads = BN / 4;
            constexpr int kInFlight = 4;
            const int total = owned * kQuads;
            for (int item0 = thread; item0 < total; item0 += kInFlight * kThreads) {
                float4 piece[kInFlight][8];
                int rows_of[kInFlight], cols_of[kInFlight];
                bool live[kInFlight];
#pragma unroll
                for (int u = 0; u < kInFlight; ++u) {
                    const int item = item0 + u * kThreads;
                    const int local_row = item / kQuads, c4 = (item - local_row * kQuads) * 4;
                    rows_of[u] = rb * kBlockR + first + local_row, cols_of[u] = cb * BN + c4;
                    live[u] = item < total && rows_of[u] < task.rows && cols_of[u] < task.cols;
                    const uint32_t local = sums + ((first + local_row) * kPitch + c4) * 4;
#pragma unroll
                    for (int s = 0; s < 8; ++s)
                        if (s < parts && live[u])
                            piece[u][s] = ld_cluster_v4(map_to_rank(local, s));
                }
#pragma unroll
                for (int u = 0; u < kInFlight; ++u) {
                    if (!live[u])
                        continue;
                    const int row = rows_of[u], col = cols_of[u];
                    float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int s = 0; s < 8; ++s)
                        if (s < parts)
                            sum[0] += piece[u][s].x, sum[1] += piece[u][s].y, sum[2] += piece[u][s].z,
                                sum[3] += piece[u][s].w;
                    __nv_bfloat16 *out = task.out;
                    long long ld = task.ld_out;
                    int shift = 0, limit = min(task.cols, task.cut0);
                    if (col >= task.cut0) {
                        const bool third = col >= task.cut1;
                        out = third ? task.out2 : task.out1;
                        ld = third ? task.ld_out2 : task.ld_out1;
                        shift = third ? task.cut1 : task.cut0;
                        limit = third ? task.cols : task.cut1;
                    }
                    float v[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        v[i] = task.alpha * sum[i];
                        if (col + i < task.cols) {
                            if (task.bias != nullptr)
                                v[i] += __bfloat162float(task.bias[col + i]);
                            if (task.beta != 0.f)
                                v[i] = fmaf(task.beta,
                                            __bfloat162float(
                                                task.addend[static_cast<long long>(row) * task.ld_add +
                                                            col + i]),
                                            v[i]);
                        }
                    }
                    __nv_bfloat16 *target = out + static_cast<long long>(row) * ld + (col - shift);
                    if (col + 4 <= limit && (reinterpret_cast<uintptr_t>(target) & 7) == 0) {
                        uint2 packed;
                        packed.x = pack_bf16(v[0], v[1]);
                        packed.y = pack_bf16(v[2], v[3]);
                        *reinterpret_cast<uint2 *>(target) = packed;
                    } else {
                        for (int i = 0; i < 4 && col + i < limit; ++i)
                            target[i] = __float2bfloat16_rn(v[i]);
                    }
                }
            }
        } else {
            /* swapped: tile rows are output features (contiguous in memory), tile
             * columns are tokens; consecutive threads take consecutive features */
            for (int item = thread; item < owned * BN; item += kThreads) {
                const int token = item / owned, local_row = item - token * owned;
                const int feature = rb * kBlockR + first + local_row, column = cb * BN + token;
                if (feature >= task.rows || column >= task.cols)
                    continue;
                const uint32_t local = sums + (token * kColPitch + first + local_row) * 4;
                float piece[8];
#pragma unroll
                for (int s = 0; s < 8; ++s)
                    if (s < parts)
                        piece[s] = ld_cluster_f32(map_to_rank(local, s));
                float sum = 0.f;
#pragma unroll
                for (int s = 0; s < 8; ++s)
                    if (s < parts)
                        sum += piece[s];
                float v = task.alpha * sum;
                if (task.bias != nullptr)
                    v += __bfloat162float(task.bias[feature]);
                const long long at = static_cast<long long>(column);
                if (task.beta != 0.f)
                    v = fmaf(task.beta, __bfloat162float(task.addend[at * task.ld_add + feature]), v);
                task.out[at * task.ld_out + feature] = __float2bfloat16_rn(v);
            }
        }
    }

    /* step 4: nobody leaves while another CTA may still be reading its ring (the
     * lanes of a warp leave the loops above after different numbers of items, so
     * this is the form that does not ask for a converged warp) */
    asm volatile("barrier.cluster.arrive.release;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, kTmemColumns);
    }
}

} // namespace sm100
