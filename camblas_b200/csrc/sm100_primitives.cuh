/*
 * Thin inline-PTX wrappers for the Blackwell (sm_100a) data path: mbarriers,
 * TMA tensor copies, tensor memory (TMEM) management and tcgen05 MMA issue.
 * Everything here is single-CTA (cta_group::1); every copy has exactly one
 * destination CTA.
 */
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace sm100
{

/* Bounds of one barrier wait: a poll count and, because a poll of
 * mbarrier.try_wait may itself block for a hardware-defined slice, a wall-clock
 * limit of two seconds. A healthy pipeline needs microseconds. */
constexpr uint32_t kSpinLimit = 1u << 24;
constexpr unsigned long long kWaitLimitNs = 2000000000ull;
/* Waits on another GPU allow for the skew between processes: five seconds unless
 * the context's "peer_wait_ms" option says otherwise (the limit travels as a
 * kernel argument). */
constexpr unsigned long long kPeerWaitLimitNs = 5000000000ull;

__device__ __forceinline__ unsigned long long global_timer_ns()
{
    unsigned long long now;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
    return now;
}

/* Status codes written to the context status word when a bounded wait gives up. */
enum StatusRole : unsigned {
    kRoleProducer = 1,
    kRoleMma = 2,
    kRoleEpilogueFull = 3,
    kRoleMmaTmemEmpty = 4,
    kRoleDrain = 5,
    kRolePeerArrive = 6,    /* partial sums of another GPU did not arrive */
    kRolePeerDelivered = 7, /* reduced tiles of another GPU did not arrive */
};

/* Flag words shared between GPUs: system-scope release add and acquire load. */
__device__ __forceinline__ void flag_add_release_system(unsigned *word, unsigned value)
{
    asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(word), "r"(value) : "memory");
}

__device__ __forceinline__ unsigned flag_load_acquire_system(const unsigned *word)
{
    unsigned value;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(value) : "l"(word) : "memory");
    return value;
}

__device__ __forceinline__ void flag_store_relaxed_system(unsigned *word, unsigned value)
{
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(word), "r"(value) : "memory");
}

/* Poll a flag word until it reaches `target`; gives up after `limit_ns`. */
__device__ __forceinline__ bool flag_wait_system(const unsigned *word, unsigned target,
                                                 unsigned long long limit_ns = kPeerWaitLimitNs);

__device__ __forceinline__ uint32_t smem_u32(const void *pointer)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(pointer));
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void fence_barrier_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async_smem()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity)
{
    uint32_t done;
    asm volatile("{\n"
                 ".reg .pred p;\n"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
                 "selp.u32 %0, 1, 0, p;\n"
                 "}\n"
                 : "=r"(done)
                 : "r"(smem_u32(bar)), "r"(parity)
                 : "memory");
    return done != 0;
}

/* Bounded wait. Returns false when the limit ran out or another role already
 * raised the CTA-wide abort flag; the caller then leaves its loop. */
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile uint32_t *abort)
{
    unsigned long long started = 0;
    for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
        if (mbar_try_wait(bar, parity))
            return true;
        if ((spin & 255u) == 255u) {
            if (*abort)
                return false;
            const unsigned long long now = global_timer_ns();
            if (started == 0)
                started = now;
            else if (now - started > kWaitLimitNs)
                return false;
        }
    }
    return false;
}

/* The same bounded wait with a poll that never suspends the thread
 * (mbarrier.test_wait): for hand-overs that recur every few hundred cycles,
 * where the time a suspended try_wait takes to resume is the cost that counts. */
__device__ __forceinline__ bool mbar_test_wait(uint64_t *bar, uint32_t parity)
{
    uint32_t done;
    asm volatile("{\n"
                 ".reg .pred p;\n"
                 "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
                 "selp.u32 %0, 1, 0, p;\n"
                 "}\n"
                 : "=r"(done)
                 : "r"(smem_u32(bar)), "r"(parity)
                 : "memory");
    return done != 0;
}

__device__ __forceinline__ bool mbar_wait_polling(uint64_t *bar, uint32_t parity,
                                                  volatile uint32_t *abort)
{
    unsigned long long started = 0;
    for (uint32_t spin = 0; spin < (kSpinLimit << 4); ++spin) {
        if (mbar_test_wait(bar, parity))
            return true;
        if ((spin & 4095u) == 4095u) {
            if (*abort)
                return false;
            const unsigned long long now = global_timer_ns();
            if (started == 0)
                started = now;
            else if (now - started > kWaitLimitNs)
                return false;
        }
    }
    return false;
}

__device__ __forceinline__ bool flag_wait_system(const unsigned *word, unsigned target,
                                                 unsigned long long limit_ns)
{
    unsigned long long started = 0;
    /* the poll count alone bounds the loop even if the timer misbehaves */
    for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
        if (flag_load_acquire_system(word) >= target)
            return true;
        if ((spin & 63u) == 63u) {
            const unsigned long long now = global_timer_ns();
            if (started == 0)
                started = now;
            else if (now - started > limit_ns)
                return false;
        }
    }
    return false;
}

/* 2-D tiled TMA load global -> shared, completion counted on an mbarrier. */
__device__ __forceinline__ void tma_load_2d(void *smem, const CUtensorMap *map, uint64_t *bar,
                                            int x, int y)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes "
                 "[%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(smem)),
                 "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
                 : "memory");
}

__device__ __forceinline__ void tma_load_2d_hint(void *smem, const CUtensorMap *map, uint64_t *bar,
                                                 int x, int y, uint64_t policy)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
                 ".L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;" ::"r"(smem_u32(smem)),
                 "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y), "l"(policy)
                 : "memory");
}

/* 2-D tiled TMA store shared -> global (bulk async group). */
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, const void *smem, int x, int y)
{
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::
                     "l"(map),
                 "r"(smem_u32(smem)), "r"(x), "r"(y)
                 : "memory");
}

/* Untiled bulk copy shared -> global of `bytes` contiguous bytes (both addresses
 * 16-byte aligned, bytes a multiple of 16); joins the same bulk groups as the
 * tensor stores. */
__device__ __forceinline__ void bulk_store(void *global, const void *smem, uint32_t bytes)
{
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(global),
                 "r"(smem_u32(smem)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void tma_store_commit()
{
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

template <int Pending> __device__ __forceinline__ void tma_store_wait_read()
{
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(Pending) : "memory");
}

template <int Pending> __device__ __forceinline__ void tma_store_wait_all()
{
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(Pending) : "memory");
}

__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap *map)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

__device__ __forceinline__ uint64_t policy_evict_first()
{
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}

__device__ __forceinline__ uint64_t policy_evict_last()
{
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}

/* ---- tensor memory ---- */

/* Whole-warp call. Writes the TMEM base address of `columns` columns (power of
 * two, 32..512) to *smem_result. */
__device__ __forceinline__ void tmem_alloc(uint32_t *smem_result, uint32_t columns)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(smem_result)),
                 "r"(columns)
                 : "memory");
}

__device__ __forceinline__ void tmem_relinquish()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t address, uint32_t columns)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(address),
                 "r"(columns)
                 : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before()
{
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tcgen05_fence_after()
{
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

/* D[tmem] (+)= A[smem] . B[smem]; BF16/FP16 operands, FP32 accumulator. */
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                         uint32_t idesc, uint32_t accumulate)
{
    asm volatile("{\n"
                 ".reg .pred p;\n"
                 "setp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
                 "}\n" ::"r"(tmem_d),
                 "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
                 : "memory");
}

/* Same for 8-bit float operands (E4M3/E5M2), FP32 accumulator. */
__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                        uint32_t idesc, uint32_t accumulate)
{
    asm volatile("{\n"
                 ".reg .pred p;\n"
                 "setp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
                 "}\n" ::"r"(tmem_d),
                 "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
                 : "memory");
}

/* Arrive on an mbarrier once every MMA issued so far by this thread is done. */
__device__ __forceinline__ void umma_commit(uint64_t *bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::
                     "r"(smem_u32(bar))
                 : "memory");
}

/* 32 lanes x 32 consecutive FP32 columns: thread t of the warp receives lane
 * (lane base of the warp's quarter + t), register i receives column + i. */
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, "
                 "[%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]),
                   "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]),
                   "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]),
                   "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),
                   "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr)
                 : "memory");
}

/* 32 lanes x 64 consecutive FP32 columns in one instruction. */
__device__ __forceinline__ void tmem_ld_32x64(uint32_t taddr, uint32_t (&r)[64])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x64.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
                 : "r"(taddr)
                 : "memory");
}

__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]),
                   "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]),
                   "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr)
                 : "memory");
}

__device__ __forceinline__ void tmem_ld_wait()
{
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

/* ---- descriptors ---- */

/* Shared-memory matrix descriptor for a K-major operand tile whose rows are
 * 128 bytes long and stored with the 128-byte swizzle (what a TMA box of
 * 64 BF16 or 128 FP8 columns produces): eight-row groups are 1024 bytes apart.
 * Field positions: start address >> 4 in bits 0-13, leading byte offset >> 4
 * in 16-29 (unused for this layout), stride byte offset >> 4 in 32-45,
 * descriptor version 1 in 46-47, swizzle mode 2 (128 B) in 61-63. */
__device__ __forceinline__ uint64_t desc_kmajor_sw128(uint32_t smem_address)
{
    uint64_t desc = 0;
    desc |= static_cast<uint64_t>((smem_address & 0x3ffffu) >> 4);
    desc |= static_cast<uint64_t>(1) << 16;
    desc |= static_cast<uint64_t>(1024 >> 4) << 32;
    desc |= static_cast<uint64_t>(1) << 46;
    desc |= static_cast<uint64_t>(2) << 61;
    return desc;
}

/* Descriptor for an MN-major operand tile: 64 BF16 consecutive along M/N form
 * one 128-byte swizzled row per K index, eight K indices form a 1024-byte atom
 * (stride offset), the next 64 M/N elements start `mn_group_bytes` further
 * (leading offset). */
__device__ __forceinline__ uint64_t desc_mnmajor_sw128(uint32_t smem_address,
                                                       uint32_t mn_group_bytes)
{
    uint64_t desc = 0;
    desc |= static_cast<uint64_t>((smem_address & 0x3ffffu) >> 4);
    desc |= static_cast<uint64_t>((mn_group_bytes >> 4) & 0x3fffu) << 16;
    desc |= static_cast<uint64_t>(1024 >> 4) << 32;
    desc |= static_cast<uint64_t>(1) << 46;
    desc |= static_cast<uint64_t>(2) << 61;
    return desc;
}

/* Instruction descriptor of tcgen05.mma kind::f16 / kind::f8f6f4 with FP32
 * accumulation. Bits: 4-5 accumulator format (1 = F32), 7-9 A format, 10-12 B
 * format (kind::f16: 1 = BF16; kind::f8f6f4: 0 = E4M3), 15 A major, 16 B major
 * (0 = K-major, 1 = MN-major), 17-22 N >> 3, 24-28 M >> 4. */
__host__ __device__ constexpr uint32_t make_idesc(uint32_t format, uint32_t m, uint32_t n,
                                                  uint32_t a_mn_major, uint32_t b_mn_major)
{
    return (1u << 4) | (format << 7) | (format << 10) | (a_mn_major << 15) | (b_mn_major << 16) |
           ((n >> 3) << 17) | ((m >> 4) << 24);
}

/* 16-byte store to shared memory through its 32-bit shared-window address. */
__device__ __forceinline__ void st_shared_v4(uint32_t address, uint32_t x, uint32_t y, uint32_t z,
                                             uint32_t w)
{
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(address), "r"(x), "r"(y), "r"(z),
                 "r"(w)
                 : "memory");
}

__device__ __forceinline__ uint32_t pack_bf16(float low, float high)
{
    __nv_bfloat162 pair = __floats2bfloat162_rn(low, high);
    return *reinterpret_cast<uint32_t *>(&pair);
}

__device__ __forceinline__ float bf16_low(uint32_t packed)
{
    return __uint_as_float(packed << 16);
}

__device__ __forceinline__ float bf16_high(uint32_t packed)
{
    return __uint_as_float(packed & 0xffff0000u);
}

} // namespace sm100
