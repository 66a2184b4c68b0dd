/*
 * Row-parallel BF16 linear layer with the sum over GPUs done through peer
 * memory: y = sum_r x[:, K_r] . W[:, K_r]^T (+ bias + residual), one process
 * per GPU, every GPU ends with the full [rows][outputs] result.
 *
 * The reference has no multi-GPU code; in its published runs the sum is the
 * all-reduce that SGLang's RowParallelLinear issues after the hooked F.linear
 * (camblas/sglang.py:250-285). Here the product and the exchange are one
 * sequence of three launches per GPU on one stream:
 *
 *   1. gemm_bf16_pair<.., Push>: the two-SM tcgen05 product of this GPU's K
 *      range. Its epilogue does not store a local result: every 256 x BN tile
 *      is sent, rounded to BF16, straight into the staging slot that the OWNER
 *      of the tile's column block keeps for this GPU (owner = column block mod
 *      world) as 4 KB bulk copies from shared memory over NVLink, 32-row slab
 *      by slab, each slab followed by a system-scope release add on the
 *      owner's arrival word for it. Tiles leave as they finish, so the
 *      transfer of early tiles overlaps the multiplication of later ones.
 *   2. peer_reduce_broadcast, launched as a programmatic dependent so that it
 *      is resident before the product ends: on the owner, one CTA per 64-column
 *      piece of a slab (256 CTAs per GPU for the benchmark's down projection at
 *      eight ranks, so that every SM issues loads and peer stores) waits
 *      (bounded) until all `world` partial slabs are there, adds the partials in
 *      rank order in FP32, adds bias and residual, rounds once and writes its
 *      piece into the result buffer of EVERY GPU; the last CTA to have read a
 *      slab clears its arrival word; then each adds one to every GPU's
 *      delivery counter.
 *   3. the wait (bounded) until this GPU's delivery counter has reached the
 *      number of slabs of the whole matrix: done by the CTA of launch 2 that
 *      finishes last, or by the small kernel peer_wait_delivered when the
 *      phases are issued separately or this GPU owns no tile.
 *
 * Because every slab is summed by exactly one GPU in a fixed order, all GPUs
 * hold bit-identical results and repeated calls give identical bits.
 *
 * Memory. Each GPU owns one region laid out as
 *   [result: capacity BF16][staging: world slots of capacity BF16][flag words]
 * obtained from camblas_cuda_peer_alloc and made visible to the other
 * processes with CUDA IPC handles (camblas_cuda_peer_open). `capacity` bounds
 * rows * outputs of a call, both rounded up to multiples of 256 (staging holds
 * whole tiles). Flag words are cleared by their consumer, so the
 * region is ready for the next call when phase 3 has run; nothing depends on
 * a call count.
 *
 * Why reuse is safe without a barrier between calls: GPU A starts call i+1
 * only after its phase 3 of call i, i.e. after every owner B has delivered all
 * of B's slabs to A. B delivers a slab after it has read the slab's partials
 * and cleared its arrival word, so A's next pushes can neither overwrite
 * partials that B still needs nor be counted into call i. Deliveries of call
 * i+1 into A's result buffer need A's own pushes of call i+1, which A's stream
 * orders after whatever A enqueued to read the result of call i.
 *
 * Every wait is bounded (five seconds to allow for skew between processes);
 * when one expires the kernel records role | cta << 4 in the context status
 * word and returns. After such a failure the flag words are undefined:
 * camblas_cuda_peer_reset on every GPU, with a host barrier around it, makes the
 * region usable again.
 *
 * The phases can be run separately (`phases` bit mask). That is how the
 * single-GPU tests drive several emulated ranks in turn: all phase-1 launches,
 * then all phase-2 launches, then all phase-3 launches, so that no kernel ever
 * waits for one that has not been launched.
 */
#pragma once

#include "dispatch_bf16.cuh"

namespace peer
{

constexpr int kMaxWorld = 8;
constexpr int kFlagWords = 65536; /* word 0: delivery counter; word 1: CTAs of the reduction
                                     done; words 64..: one arrival word per slab, then one
                                     word per slab counting the CTAs that have read it, then
                                     one word per tile counting its finished slabs */
constexpr int kFlagHeader = 64;
constexpr int kMaxUnits = 24576; /* slabs of the tile path: two words each from kFlagHeader on */
/* The rest of the flag words belongs to the all-reduce of small tensors: one
 * call counter per 2048-element chunk of the flagged-line exchange (the last
 * kLineChunks words), and before them three words per chunk (arrived, consumed,
 * pending) for tensors too large for that exchange. */
constexpr int kSmallChunkElements = 2048; /* 256 threads x 8 BF16 */
constexpr long long kLineMaxElements = 64 * 8192; /* 1 MiB of BF16: 64 token rows of 8192 */
constexpr int kLineChunks = int(kLineMaxElements / kSmallChunkElements);
constexpr int kLineBase = kFlagWords - kLineChunks;
constexpr int kTileBase = kFlagHeader + 2 * kMaxUnits; /* one word per tile: its finished slabs */
constexpr int kSmallBase = kTileBase + kMaxUnits / 8;
constexpr int kSmallChunks = (kLineBase - kSmallBase) / 3;
/* A flagged line is 16 bytes: two 8-byte halves of 4 payload bytes and a 4-byte
 * flag each. One rank's tensor takes at most kLineSlotLines of them. */
constexpr size_t kLinesPerChunk = 2 * 256;
constexpr size_t kLineSlotLines = size_t(kLineChunks) * kLinesPerChunk;

inline size_t slot_bytes(size_t capacity)
{
    return (capacity * sizeof(__nv_bfloat16) + 255) & ~size_t(255);
}

/* Two buffers of one slot per rank, directly behind the flag words. */
inline size_t line_bytes(int world)
{
    return 2 * size_t(world) * kLineSlotLines * sizeof(uint4);
}

inline size_t region_bytes(int world, size_t capacity)
{
    return slot_bytes(capacity) * (1 + size_t(world)) + size_t(kFlagWords) * sizeof(unsigned) +
           line_bytes(world);
}

struct Region {
    __nv_bfloat16 *result;
    __nv_bfloat16 *staging; /* slot s at staging + s * slot_elements */
    unsigned *flags;
    uint4 *lines; /* [buffer][rank][kLineSlotLines] */
    size_t slot_elements;
};

inline Region carve(void *memory, int world, size_t capacity)
{
    Region region;
    uint8_t *base = static_cast<uint8_t *>(memory);
    region.slot_elements = slot_bytes(capacity) / sizeof(__nv_bfloat16);
    region.result = reinterpret_cast<__nv_bfloat16 *>(base);
    region.staging = reinterpret_cast<__nv_bfloat16 *>(base + slot_bytes(capacity));
    region.flags = reinterpret_cast<unsigned *>(base + slot_bytes(capacity) * (1 + size_t(world)));
    region.lines = reinterpret_cast<uint4 *>(region.flags + kFlagWords);
    return region;
}

struct ReduceTask {
    int rank, world;
    int rows, cols;
    int r_blocks, c_blocks, width; /* 256-row blocks, column blocks of `width` */
    const __nv_bfloat16 *staging;  /* this GPU's staging slots */
    long long slot_elements;
    unsigned *arrive;              /* this GPU's arrival words */
    const __nv_bfloat16 *bias;     /* per column, may be NULL */
    const __nv_bfloat16 *residual; /* [rows][ld_residual], may be NULL */
    long long ld_residual;
    __nv_bfloat16 *result[kMaxWorld]; /* every GPU's result buffer */
    unsigned *delivered[kMaxWorld];   /* every GPU's delivery counter */
    unsigned *status;
    unsigned long long wait_ns; /* how long a wait on another GPU's flag may last */
};

__device__ __forceinline__ void accumulate8(float (&sum)[8], const uint4 &packed)
{
    const uint32_t words[4] = {packed.x, packed.y, packed.z, packed.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        sum[2 * i] += __uint_as_float(words[i] << 16);
        sum[2 * i + 1] += __uint_as_float(words[i] & 0xffff0000u);
    }
}

/* Waits until `expected` tiles have been delivered to this GPU, then clears the counter. */
__device__ __forceinline__ void wait_delivered(unsigned *delivered, unsigned expected,
                                               unsigned *status, unsigned long long wait_ns)
{
    if (sm100::flag_wait_system(delivered, expected, wait_ns))
        sm100::flag_store_relaxed_system(delivered, 0u);
    else
        atomicCAS(status, 0u, unsigned(sm100::kRolePeerDelivered));
}

/* grid = (column blocks this GPU owns, 8 * r_blocks, 1..width / 64); 256 threads.
 * The CTAs of a slab (32 rows of one owned tile) share its 64-column pieces - in
 * the staging layout (see sm100::epilogue_push) a piece is one contiguous 4 KB
 * chunk per rank. The host picks their number so that the launch has some 256
 * CTAs: with eight ranks a GPU owns few slabs and needs four CTAs on each to keep
 * its NVLink ports busy; with two ranks one CTA per slab is right, because the
 * CTAs become resident while the product kernel still runs (programmatic
 * dependent launch) and every one of them polls a flag, which a thousand of them
 * did at the product's expense (tp2 step 0.368 -> 0.391 ms). A CTA
 * waits for the slab's `world` partial copies, adds them in rank
 * order (one 16-byte piece per thread, all ranks' loads in flight together),
 * applies bias and residual, rounds once and writes the piece, now as ordinary
 * matrix rows (eight threads store 128 contiguous bytes of a row), into every
 * GPU's result. The CTAs of a slab count themselves on the slab's second flag
 * word; the last one clears both words, so the next call finds them zero, and
 * counts the slab on the tile's word. The CTA that completes a tile announces
 * it to every GPU with one system-scope addition per GPU: a delivery counter
 * takes one addition per tile from its owner, not one per CTA (thousands of
 * remote additions to one word serialise and cost tens of microseconds). The
 * counts are chained by fences, so the announcement is ordered after the stores
 * of every CTA of the tile. With `wait_inline` the CTA that
 * finishes last also waits for the deliveries to this GPU, which saves the
 * launch of peer_wait_delivered. */
__global__ void __launch_bounds__(256)
    peer_reduce_broadcast(const ReduceTask task, unsigned expected, int wait_inline)
{
    __shared__ int failed;
    const int cb = task.rank + blockIdx.x * task.world;
    const int rb = blockIdx.y >> 3, slab = blockIdx.y & 7;
    const int chunks = gridDim.z; /* CTAs that share this slab */
    const int unit = (rb * task.c_blocks + cb) * 8 + slab;
    unsigned *const arrived = task.arrive + unit;
    unsigned *const readers = task.arrive + kMaxUnits + unit;
    unsigned *const slabs_done = task.arrive + 2 * kMaxUnits + (rb * task.c_blocks + cb);
    __shared__ int announce;
    if (threadIdx.x == 0) {
        announce = 0;
        const bool ok = sm100::flag_wait_system(arrived, unsigned(task.world), task.wait_ns);
        if (!ok)
            atomicCAS(task.status, 0u, sm100::kRolePeerArrive | (blockIdx.x << 4));
        failed = ok ? 0 : 1;
    }
    __syncthreads();
    if (!failed) {
        const int r = threadIdx.x >> 3, piece = threadIdx.x & 7;
        const int row = rb * 256 + slab * 32 + r;
        /* the slab's 64-column pieces are dealt out to the CTAs of the slab in turn */
        for (int chunk = blockIdx.z; chunk < task.width / 64; chunk += chunks) {
            const int c = cb * task.width + chunk * 64 + piece * 8;
            const long long offset = static_cast<long long>(unit) * (32 * task.width) + chunk * 2048 +
                                     r * 64 + ((piece ^ (r & 7)) << 3);
            uint4 part[kMaxWorld];
#pragma unroll
            for (int s = 0; s < kMaxWorld; ++s)
                if (s < task.world)
                    part[s] = __ldcg(reinterpret_cast<const uint4 *>(
                        task.staging + s * task.slot_elements + offset));
            if (row < task.rows && c < task.cols) {
                float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int s = 0; s < kMaxWorld; ++s)
                    if (s < task.world)
                        accumulate8(sum, part[s]);
                if (task.bias != nullptr)
                    accumulate8(sum, *reinterpret_cast<const uint4 *>(task.bias + c));
                if (task.residual != nullptr)
                    accumulate8(sum,
                                *reinterpret_cast<const uint4 *>(
                                    task.residual + static_cast<long long>(row) * task.ld_residual + c));
                uint4 packed;
                packed.x = sm100::pack_bf16(sum[0], sum[1]);
                packed.y = sm100::pack_bf16(sum[2], sum[3]);
                packed.z = sm100::pack_bf16(sum[4], sum[5]);
                packed.w = sm100::pack_bf16(sum[6], sum[7]);
                const long long target_offset = static_cast<long long>(row) * task.cols + c;
                /* start with the next GPU so that the owners do not all write to the same one */
                for (int hop = 1; hop <= task.world; ++hop) {
                    int target = task.rank + hop;
                    if (target >= task.world)
                        target -= task.world;
                    *reinterpret_cast<uint4 *>(task.result[target] + target_offset) = packed;
                }
            }
        }
        __threadfence_system();
    }
    __syncthreads();
    if (!failed && threadIdx.x == 0) {
        /* the partials of this slab have been read by this CTA; the last reader
         * hands the two words back as zeros */
        if (atomicAdd(readers, 1u) == unsigned(chunks) - 1u) {
            sm100::flag_store_relaxed_system(readers, 0u);
            sm100::flag_store_relaxed_system(arrived, 0u);
            if (atomicAdd(slabs_done, 1u) == 7u) {
                *slabs_done = 0u;
                announce = 1;
            }
        }
        __threadfence_system();
    }
    __syncthreads();
    if (announce && threadIdx.x < task.world)
        sm100::flag_add_release_system(task.delivered[threadIdx.x], 1u);
    if (wait_inline && threadIdx.x == 0) {
        /* word 1 of this GPU's flags counts the CTAs of this launch that are done */
        unsigned *ticket = task.delivered[task.rank] + 1;
        const unsigned done = atomicAdd(ticket, 1u);
        if (done == gridDim.x * gridDim.y * gridDim.z - 1) {
            *ticket = 0;
            wait_delivered(task.delivered[task.rank], expected, task.status, task.wait_ns);
        }
    }
    /* This kernel is launched as a programmatic dependent of the product kernel
     * and may otherwise finish before it: on the success path every push of the
     * product has landed by now (the arrivals say so), but after an expired wait
     * the product could still be writing into other GPUs' staging while the
     * stream moves on to camblas_cuda_peer_reset or the next call. Waiting for the
     * preceding grid here makes "this launch is complete" imply "the product is
     * complete" in every case; it is free when the product has already ended and
     * does nothing when the launch had no programmatic dependency. The product
     * kernel waits on nothing that this kernel provides, so no cycle can form. */
    if (threadIdx.x == 0)
        asm volatile("griddepcontrol.wait;" ::: "memory");
}

/* One thread: wait until `expected` slabs have been delivered to this GPU. */
__global__ void peer_wait_delivered(unsigned *delivered, unsigned expected, unsigned *status,
                                    unsigned long long wait_ns)
{
    if (threadIdx.x == 0)
        wait_delivered(delivered, expected, status, wait_ns);
}

/* ---- all-reduce of a BF16 tensor through the peer regions, counted arrivals -----
 *
 * Used for tensors beyond the 1 MiB that the flagged-line exchange further down
 * takes. A one-shot exchange: every rank stores its tensor into slot `rank` of
 * EVERY GPU's staging area (16-byte stores over NVLink), tells each GPU so, waits
 * until all `world` tensors have arrived in its own staging area, adds them in
 * rank order in FP32, rounds once and writes its own copy of the sum. All ranks
 * add the same values in the same order, so they hold the same bits.
 *
 * The work is cut into chunks of 2048 elements, one CTA each, and every chunk
 * synchronises on its own three flag words of the region, so no CTA depends on
 * another CTA of its own GPU and nothing spans the grid:
 *   arrived[c]   raised by each rank (release, system scope) once its copy of
 *                chunk c is in this GPU's staging; the summing CTA waits for
 *                `world` of them and clears the word;
 *   consumed[c]  raised on every GPU by each rank once it has summed chunk c and
 *                so no longer reads the copies it was sent; before a rank
 *                overwrites its slot on its peers in the next call it waits until
 *                its own word has reached `world`, and clears it;
 *   pending[c]   local: whether a previous call left a `consumed` count to wait
 *                for (zero after camblas_cuda_peer_alloc / peer_reset).
 * Waits are bounded like the others; after one expires the words are undefined
 * until camblas_cuda_peer_reset. `phases` 1 (wait consumed, store, announce) and
 * 2 (wait arrived, add, announce consumed) can be issued separately so that one
 * process can drive several ranks on one GPU in turn without any kernel waiting
 * for an unlaunched one. */
struct SmallTask {
    int rank, world;
    long long elements; /* multiple of 8 */
    const __nv_bfloat16 *input;
    __nv_bfloat16 *output;
    __nv_bfloat16 *slot_at[kMaxWorld]; /* this rank's slot in every GPU's staging */
    unsigned *flags_at[kMaxWorld];     /* every GPU's small-path words */
    const __nv_bfloat16 *staging;      /* this GPU's staging slots */
    long long slot_elements;
    unsigned *flags;                   /* this GPU's small-path words */
    unsigned *status;
    unsigned long long wait_ns;
};

__global__ void __launch_bounds__(256) peer_small_allreduce(const SmallTask task, int phases)
{
    __shared__ int failed;
    const int chunk = blockIdx.x;
    const long long element = static_cast<long long>(chunk) * kSmallChunkElements + threadIdx.x * 8;
    const bool live = element < task.elements;
    unsigned *const arrived = task.flags + chunk;
    unsigned *const consumed = task.flags + kSmallChunks + chunk;
    unsigned *const pending = task.flags + 2 * kSmallChunks + chunk;
    if (threadIdx.x == 0)
        failed = 0;
    __syncthreads();
    if (phases & 1) {
        if (threadIdx.x == 0 && *pending != 0u) {
            /* the peers must be done with what this rank sent them last time */
            if (sm100::flag_wait_system(consumed, unsigned(task.world), task.wait_ns)) {
                sm100::flag_store_relaxed_system(consumed, 0u);
                *pending = 0u;
            } else {
                atomicCAS(task.status, 0u, sm100::kRolePeerDelivered | (blockIdx.x << 4));
                failed = 1;
            }
        }
        __syncthreads();
        if (failed)
            return;
        if (live) {
            const uint4 mine = *reinterpret_cast<const uint4 *>(task.input + element);
            for (int hop = 0; hop < task.world; ++hop) {
                int target = task.rank + 1 + hop; /* peers first, own copy last */
                if (target >= task.world)
                    target -= task.world;
                *reinterpret_cast<uint4 *>(task.slot_at[target] + element) = mine;
            }
        }
        __threadfence_system();
        __syncthreads();
        if (threadIdx.x < task.world)
            sm100::flag_add_release_system(task.flags_at[threadIdx.x] + chunk, 1u);
    }
    if (phases & 2) {
        if (threadIdx.x == 0) {
            if (sm100::flag_wait_system(arrived, unsigned(task.world), task.wait_ns)) {
                sm100::flag_store_relaxed_system(arrived, 0u);
            } else {
                atomicCAS(task.status, 0u, sm100::kRolePeerArrive | (blockIdx.x << 4));
                failed = 1;
            }
        }
        __syncthreads();
        if (failed)
            return;
        if (live) {
            uint4 part[kMaxWorld];
#pragma unroll
            for (int s = 0; s < kMaxWorld; ++s)
                if (s < task.world)
                    part[s] = __ldcg(reinterpret_cast<const uint4 *>(
                        task.staging + s * task.slot_elements + element));
            float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int s = 0; s < kMaxWorld; ++s)
                if (s < task.world)
                    accumulate8(sum, part[s]);
            uint4 packed;
            packed.x = sm100::pack_bf16(sum[0], sum[1]);
            packed.y = sm100::pack_bf16(sum[2], sum[3]);
            packed.z = sm100::pack_bf16(sum[4], sum[5]);
            packed.w = sm100::pack_bf16(sum[6], sum[7]);
            *reinterpret_cast<uint4 *>(task.output + element) = packed;
        }
        __syncthreads(); /* every thread has its operands in registers */
        if (threadIdx.x < task.world)
            sm100::flag_add_release_system(task.flags_at[threadIdx.x] + kSmallChunks + chunk, 1u);
        if (threadIdx.x == 0)
            *pending = 1u;
    }
}

/* ---- all-reduce of at most 1 MiB of BF16 through flagged lines ------------------
 *
 * The exchange above needs three trips over NVLink per call (stores and their
 * fence, the arrival count, the consumed count). For the tensors of decoding that
 * latency is the whole cost, so up to kLineMaxElements take this route instead,
 * which needs one: every 8 bytes of payload travel as a 16-byte line
 * {4 bytes, flag, 4 bytes, flag}, each 8-byte half written by one store
 * instruction so that payload and flag become visible together. The receiver
 * polls the lines themselves until both flags show the number of the current
 * call; there is no fence, no separate flag word and no acknowledgement.
 *
 * Call numbers. Word kLineBase + c of a GPU's flag words counts the calls that
 * have used chunk c; every rank makes the same calls, so the ranks agree on it
 * without talking. The flag of a call is that count plus one, cycling through
 * 1 .. 2^32 - 2 (never zero, which is what a cleared line holds; the cycle length
 * is even so that consecutive calls always differ in the lowest bit).
 *
 * Reuse. The lowest bit of the flag selects one of two line buffers. Rank A
 * writes call n + 2 into the buffer of call n only after it finished call n + 1,
 * for which it needed B's lines of call n + 1, which B's stream sent only after
 * B's kernel of call n had finished reading. So nothing is overwritten while it
 * is still being read, provided the calls of one rank run in stream order.
 *
 * Stale lines. A sender always writes all 512 lines of a chunk (zero payload
 * beyond the tensor's end), so every line of a chunk carries the flag of the
 * latest call that used its buffer and an older number cannot be mistaken for the
 * current one. The line area is written by nothing else and is cleared by
 * camblas_cuda_peer_alloc and camblas_cuda_peer_reset.
 *
 * The sum is formed like above: FP32, rank order (the rank's own tensor comes
 * from `input`, not through memory), one rounding. Waits are bounded; `phases`
 * 1 (send) and 2 (receive, add, count the call) can be issued separately. */
struct LineTask {
    int rank, world;
    long long elements; /* multiple of 8 */
    const __nv_bfloat16 *input;
    __nv_bfloat16 *output;
    uint4 *slot_at[kMaxWorld]; /* this rank's slot of buffer 0 in every GPU's line area */
    const uint4 *lines;        /* this GPU's line area */
    unsigned *calls;           /* this GPU's call counters, one per chunk */
    unsigned *status;
    unsigned long long wait_ns;
};

__device__ __forceinline__ void store_line(uint4 *line, unsigned low, unsigned high, unsigned flag)
{
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(line), "r"(low),
                 "r"(flag), "r"(high), "r"(flag)
                 : "memory");
}

__device__ __forceinline__ uint4 load_line(const uint4 *line)
{
    uint4 value;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(value.x), "=r"(value.y), "=r"(value.z), "=r"(value.w)
                 : "l"(line)
                 : "memory");
    return value;
}

__global__ void __launch_bounds__(256) peer_lines_allreduce(const LineTask task, int phases)
{
    const int chunk = blockIdx.x;
    const long long element = static_cast<long long>(chunk) * kSmallChunkElements + threadIdx.x * 8;
    const bool live = element < task.elements;
    const unsigned flag = task.calls[chunk] + 1u;
    const size_t buffer = size_t(flag & 1u) * size_t(task.world) * kLineSlotLines;
    const size_t first = size_t(chunk) * kLinesPerChunk + threadIdx.x; /* second line 256 further */
    const uint4 mine =
        live ? *reinterpret_cast<const uint4 *>(task.input + element) : make_uint4(0u, 0u, 0u, 0u);
    if (phases & 1) {
        for (int hop = 1; hop < task.world; ++hop) {
            int target = task.rank + hop;
            if (target >= task.world)
                target -= task.world;
            uint4 *const slot = task.slot_at[target] + buffer + first;
            store_line(slot, mine.x, mine.y, flag);
            store_line(slot + 256, mine.z, mine.w, flag);
        }
    }
    if (phases & 2) {
        if (live) {
            const uint4 *const inbox = task.lines + buffer + first;
            uint4 part[kMaxWorld];
            bool complete = false;
            unsigned long long started = 0;
            for (uint32_t spin = 0; spin < sm100::kSpinLimit && !complete; ++spin) {
                uint4 low[kMaxWorld], high[kMaxWorld];
#pragma unroll
                for (int s = 0; s < kMaxWorld; ++s)
                    if (s < task.world && s != task.rank) {
                        low[s] = load_line(inbox + size_t(s) * kLineSlotLines);
                        high[s] = load_line(inbox + size_t(s) * kLineSlotLines + 256);
                    }
                complete = true;
#pragma unroll
                for (int s = 0; s < kMaxWorld; ++s)
                    if (s < task.world && s != task.rank) {
                        complete = complete && low[s].y == flag && low[s].w == flag &&
                                   high[s].y == flag && high[s].w == flag;
                        part[s] = make_uint4(low[s].x, low[s].z, high[s].x, high[s].z);
                    }
                if (!complete && (spin & 63u) == 63u) {
                    const unsigned long long now = sm100::global_timer_ns();
                    if (started == 0)
                        started = now;
                    else if (now - started > task.wait_ns)
                        break;
                }
            }
            if (complete) {
                float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int s = 0; s < kMaxWorld; ++s)
                    if (s < task.world)
                        accumulate8(sum, s == task.rank ? mine : part[s]);
                uint4 packed;
                packed.x = sm100::pack_bf16(sum[0], sum[1]);
                packed.y = sm100::pack_bf16(sum[2], sum[3]);
                packed.z = sm100::pack_bf16(sum[4], sum[5]);
                packed.w = sm100::pack_bf16(sum[6], sum[7]);
                *reinterpret_cast<uint4 *>(task.output + element) = packed;
            } else {
                atomicCAS(task.status, 0u, sm100::kRolePeerArrive | (blockIdx.x << 4));
            }
        }
        __syncthreads(); /* every thread has read the counter */
        if (threadIdx.x == 0)
            task.calls[chunk] = flag == 0xFFFFFFFEu ? 0u : flag;
    }
}

/* ---- the same through flagged lines in two steps, for four ranks and more ----------
 *
 * One shot sends every rank's whole tensor to every peer: 2 x (world - 1) x bytes
 * of lines leave each GPU, 14 MB for a 1 MB tensor on eight ranks (27 us). With
 * four ranks or more and enough data it is cheaper to cut the tensor into
 * `world` slices: every rank sends slice o to rank o, which adds the `world`
 * copies of its slice in rank order (same FP32 order and single rounding as the
 * one-shot form, so the same bits) and sends the sum to every rank: two trips,
 * but 2 x 2 x (world - 1) / world x bytes of lines per GPU, a quarter at eight
 * ranks. The host takes this form where the one-shot form would send more than
 * about 1.75 MB of payload per GPU. CTA c serves elements [2048 c, 2048 c + 2048) of EVERY slice. The
 * first step uses the lines of chunk c of a slot, the second those of chunk
 * kLineChunks / 2 + c, each with the call counter of its own chunk, so a line
 * position always carries numbers of one counter whichever form wrote it last.
 * `phases`: 1 send the slices, 2 add my slice and send the sum, 4 collect the
 * sums and count the call. */
constexpr int kLineHalf = kLineChunks / 2;

struct SliceTask {
    LineTask base;
    long long slice; /* elements per slice, a multiple of 8; at most kLineHalf chunks */
};

/* Polls the two lines of every rank but `skip` until they carry `flag`; false when
 * the limit ran out. part[s] holds the 16 payload bytes of rank s. */
__device__ __forceinline__ bool collect_lines(const uint4 *inbox, int world, int skip, unsigned flag,
                                              unsigned long long wait_ns, uint4 (&part)[kMaxWorld])
{
    unsigned long long started = 0;
    for (uint32_t spin = 0; spin < sm100::kSpinLimit; ++spin) {
        uint4 low[kMaxWorld], high[kMaxWorld];
#pragma unroll
        for (int s = 0; s < kMaxWorld; ++s)
            if (s < world && s != skip) {
                low[s] = load_line(inbox + size_t(s) * kLineSlotLines);
                high[s] = load_line(inbox + size_t(s) * kLineSlotLines + 256);
            }
        bool complete = true;
#pragma unroll
        for (int s = 0; s < kMaxWorld; ++s)
            if (s < world && s != skip) {
                complete = complete && low[s].y == flag && low[s].w == flag && high[s].y == flag &&
                           high[s].w == flag;
                part[s] = make_uint4(low[s].x, low[s].z, high[s].x, high[s].z);
            }
        if (complete)
            return true;
        if ((spin & 63u) == 63u) {
            const unsigned long long now = sm100::global_timer_ns();
            if (started == 0)
                started = now;
            else if (now - started > wait_ns)
                return false;
        }
    }
    return false;
}

__global__ void __launch_bounds__(256) peer_lines_allreduce_sliced(const SliceTask sliced, int phases)
{
    const LineTask &task = sliced.base;
    const int chunk = blockIdx.x;
    const long long local = static_cast<long long>(chunk) * kSmallChunkElements + threadIdx.x * 8;
    const bool in_slice = local < sliced.slice;
    const unsigned flag_a = task.calls[chunk] + 1u, flag_b = task.calls[kLineHalf + chunk] + 1u;
    const size_t buffer_a = size_t(flag_a & 1u) * size_t(task.world) * kLineSlotLines;
    const size_t buffer_b = size_t(flag_b & 1u) * size_t(task.world) * kLineSlotLines;
    const size_t first_a = size_t(chunk) * kLinesPerChunk + threadIdx.x;
    const size_t first_b = size_t(kLineHalf + chunk) * kLinesPerChunk + threadIdx.x;
    auto of_slice = [&](int owner) { return static_cast<long long>(owner) * sliced.slice + local; };
    auto read_input = [&](int owner) {
        const long long element = of_slice(owner);
        return in_slice && element < task.elements
                   ? *reinterpret_cast<const uint4 *>(task.input + element)
                   : make_uint4(0u, 0u, 0u, 0u);
    };
    if (phases & 1) {
        for (int hop = 1; hop < task.world; ++hop) {
            int owner = task.rank + hop;
            if (owner >= task.world)
                owner -= task.world;
            const uint4 piece = read_input(owner);
            uint4 *const slot = task.slot_at[owner] + buffer_a + first_a;
            store_line(slot, piece.x, piece.y, flag_a);
            store_line(slot + 256, piece.z, piece.w, flag_a);
        }
    }
    bool failed = false;
    if (phases & 2) {
        /* my slice: the other ranks' copies arrive in my line area, mine comes from `input` */
        uint4 part[kMaxWorld];
        const uint4 mine = read_input(task.rank);
        if (collect_lines(task.lines + buffer_a + first_a, task.world, task.rank, flag_a, task.wait_ns,
                          part)) {
            float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int s = 0; s < kMaxWorld; ++s)
                if (s < task.world)
                    accumulate8(sum, s == task.rank ? mine : part[s]);
            uint4 packed;
            packed.x = sm100::pack_bf16(sum[0], sum[1]);
            packed.y = sm100::pack_bf16(sum[2], sum[3]);
            packed.z = sm100::pack_bf16(sum[4], sum[5]);
            packed.w = sm100::pack_bf16(sum[6], sum[7]);
            for (int hop = 1; hop < task.world; ++hop) {
                int target = task.rank + hop;
                if (target >= task.world)
                    target -= task.world;
                uint4 *const slot = task.slot_at[target] + buffer_b + first_b;
                store_line(slot, packed.x, packed.y, flag_b);
                store_line(slot + 256, packed.z, packed.w, flag_b);
            }
            const long long element = of_slice(task.rank);
            if (in_slice && element < task.elements)
                *reinterpret_cast<uint4 *>(task.output + element) = packed;
        } else {
            failed = true;
        }
    }
    if (phases & 4) {
        uint4 part[kMaxWorld];
        if (collect_lines(task.lines + buffer_b + first_b, task.world, task.rank, flag_b, task.wait_ns,
                          part)) {
#pragma unroll
            for (int s = 0; s < kMaxWorld; ++s)
                if (s < task.world && s != task.rank) {
                    const long long element = of_slice(s);
                    if (in_slice && element < task.elements)
                        *reinterpret_cast<uint4 *>(task.output + element) = part[s];
                }
        } else {
            failed = true;
        }
        __syncthreads(); /* every thread has read the counters */
        if (threadIdx.x == 0) {
            task.calls[chunk] = flag_a == 0xFFFFFFFEu ? 0u : flag_a;
            task.calls[kLineHalf + chunk] = flag_b == 0xFFFFFFFEu ? 0u : flag_b;
        }
    }
    if (failed)
        atomicCAS(task.status, 0u, sm100::kRolePeerArrive | (blockIdx.x << 4));
}

struct Call {
    int rank, world;
    size_t capacity;
    void *const *memory;
    int phases;
    int rows, inner, outputs;
    const __nv_bfloat16 *x, *w, *bias, *residual;
    int ldx, ldw, ldr;
};

inline int run(camblas_cuda_context *context, const Call &call)
{
    using namespace host;
    Region regions[kMaxWorld];
    for (int r = 0; r < call.world; ++r)
        regions[r] = carve(call.memory[r], call.world, call.capacity);
    const Region &own = regions[call.rank];

    int bn = call.outputs <= 128 ? 128 : 256;
    if (context->options.push_width == 128)
        bn = 128;
    const int r_blocks = (call.rows + 255) / 256;
    const int c_blocks = (call.outputs + bn - 1) / bn;
    const long long units = 1ll * r_blocks * c_blocks * 8;
    if (units > kMaxUnits)
        return fail(context, "row-parallel product has more slabs than the region has flag words", 1);
    /* staging holds whole tiles */
    if (size_t(r_blocks) * 256 * size_t(c_blocks) * bn > own.slot_elements)
        return fail(context,
                    "row-parallel result exceeds the peer region capacity (rows and outputs count "
                    "rounded up to multiples of 256)",
                    1);

    if (call.phases & 1) {
        sm100::GemmTask task{};
        task.rows = call.rows, task.cols = call.outputs, task.depth = call.inner;
        task.r_blocks = r_blocks, task.c_blocks = c_blocks;
        task.k_blocks = (call.inner + 63) / 64;
        task.split = 1, task.k_blocks_per_split = task.k_blocks;
        task.alpha = 1.f, task.beta = 0.f;
        task.status = context->status;
        task.cut0 = task.cut1 = call.outputs;
        task.batch = 1;
        task.panel = r_blocks < 8 ? r_blocks : 8;
        task.push_world = call.world;
        for (int r = 0; r < call.world; ++r) {
            task.push_staging[r] = regions[r].staging + size_t(call.rank) * regions[r].slot_elements;
            task.push_arrive[r] = regions[r].flags + kFlagHeader;
        }
        const int pairs_max = context->sm_count / 2;
        const long long tiles = 1ll * r_blocks * c_blocks;
        const int pairs = tiles < pairs_max ? int(tiles) : pairs_max;
        CUtensorMap p, q;
        const auto bf16 = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
        bool ok = encode_2d(context, &p, bf16, 2, call.x, call.inner, call.rows,
                            uint64_t(call.ldx) * 2, 64, 128) &&
                  encode_2d(context, &q, bf16, 2, call.w, call.inner, call.outputs,
                            uint64_t(call.ldw) * 2, 64, bn / 2);
        if (!ok)
            return fail(context, "tensor map encoding", 1);
        using namespace sm100;
        /* the kernel only prefetches its output maps in this mode; any valid map will do */
        cudaError_t error =
            bn == 256 ? launch_pair<256, 3, kMajorK, kMajorK, 2, kEpiPush>(context, pairs, p, q, q, q, q,
                                                                       task)
                      : launch_pair<128, 4, kMajorK, kMajorK, 2, kEpiPush>(context, pairs, p, q, q, q, q,
                                                                       task);
        if (error != cudaSuccess)
            return fail(context, "two-SM tcgen05 BF16 GEMM with peer push", error);
        context->kernel_launches.fetch_add(1, std::memory_order_relaxed);
    }
    bool wait_inline = false;
    if (call.phases & 2) {
        const int owned = (c_blocks - call.rank + call.world - 1) / call.world;
        if (owned > 0) {
            ReduceTask task{};
            task.rank = call.rank, task.world = call.world;
            task.rows = call.rows, task.cols = call.outputs;
            task.r_blocks = r_blocks, task.c_blocks = c_blocks, task.width = bn;
            task.staging = own.staging;
            task.slot_elements = static_cast<long long>(own.slot_elements);
            task.arrive = own.flags + kFlagHeader;
            task.bias = call.bias;
            task.residual = call.residual, task.ld_residual = call.ldr;
            for (int r = 0; r < call.world; ++r) {
                task.result[r] = regions[r].result;
                task.delivered[r] = regions[r].flags;
            }
            task.status = context->status;
            task.wait_ns = 1000000ull * unsigned(context->options.peer_wait_ms);
            /* Launched as a programmatic dependent of the product kernel: its CTAs
             * may become resident while that kernel still runs (it says so at its
             * start) and wait on the arrival words, not on the kernel boundary. */
            cudaLaunchConfig_t config = {};
            const int slabs = owned * 8 * r_blocks;
            const int share = std::max(1, std::min(bn / 64, 256 / slabs));
            config.gridDim = dim3(owned, 8 * r_blocks, share == 3 ? 2 : share);
            config.blockDim = dim3(256);
            config.stream = context->stream;
            cudaLaunchAttribute attribute[1];
            attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attribute[0].val.programmaticStreamSerializationAllowed = 1;
            config.attrs = attribute;
            config.numAttrs = 1;
            wait_inline = (call.phases & 4) != 0;
            cudaError_t error = cudaLaunchKernelEx(&config, peer_reduce_broadcast, task,
                                                   unsigned(units / 8), int(wait_inline));
            if (error != cudaSuccess)
                return fail(context, "peer reduction and broadcast", error);
            context->kernel_launches.fetch_add(1, std::memory_order_relaxed);
        }
    }
    if ((call.phases & 4) && !wait_inline) {
        peer_wait_delivered<<<1, 32, 0, context->stream>>>(
            own.flags, unsigned(units / 8), context->status,
            1000000ull * unsigned(context->options.peer_wait_ms));
        return launched(context, "peer delivery wait");
    }
    return 0;
}

} // namespace peer

extern "C" size_t camblas_cuda_peer_bytes(int world, size_t capacity)
{
    if (world < 1 || world > peer::kMaxWorld || capacity == 0)
        return 0;
    return peer::region_bytes(world, capacity);
}

extern "C" int camblas_cuda_peer_alloc(camblas_cuda_context *context, size_t bytes, void **memory,
                                       void *handle)
{
    return host::guarded(context, [&] {
        if (!memory || bytes == 0)
            return host::fail(context, "missing peer allocation output or size", 1);
        void *pointer = nullptr;
        cudaError_t error = cudaMalloc(&pointer, bytes);
        if (error != cudaSuccess) {
            cudaGetLastError();
            return host::fail(context, "peer region allocation", error);
        }
        error = cudaMemset(pointer, 0, bytes);
        if (error == cudaSuccess && handle != nullptr) {
            cudaIpcMemHandle_t exported;
            error = cudaIpcGetMemHandle(&exported, pointer);
            if (error == cudaSuccess)
                std::memcpy(handle, &exported, sizeof(exported));
        }
        if (error != cudaSuccess) {
            cudaGetLastError();
            cudaFree(pointer);
            return host::fail(context, "peer region export", error);
        }
        *memory = pointer;
        return 0;
    });
}

extern "C" int camblas_cuda_peer_open(camblas_cuda_context *context, const void *handle,
                                      void **memory)
{
    return host::guarded(context, [&] {
        if (!memory || !handle)
            return host::fail(context, "missing peer handle or output", 1);
        cudaIpcMemHandle_t imported;
        std::memcpy(&imported, handle, sizeof(imported));
        void *pointer = nullptr;
        cudaError_t error =
            cudaIpcOpenMemHandle(&pointer, imported, cudaIpcMemLazyEnablePeerAccess);
        if (error != cudaSuccess) {
            cudaGetLastError();
            return host::fail(context, "peer region import", error);
        }
        *memory = pointer;
        return 0;
    });
}

extern "C" int camblas_cuda_peer_close(camblas_cuda_context *context, void *memory)
{
    return host::guarded(context, [&] {
        if (!memory)
            return 0;
        cudaError_t error = cudaStreamSynchronize(context->stream);
        if (error == cudaSuccess)
            error = cudaIpcCloseMemHandle(memory);
        return error == cudaSuccess ? 0 : host::fail(context, "peer region close", error);
    });
}

extern "C" int camblas_cuda_peer_free(camblas_cuda_context *context, void *memory)
{
    return host::guarded(context, [&] {
        if (!memory)
            return 0;
        cudaError_t error = cudaStreamSynchronize(context->stream);
        if (error == cudaSuccess)
            error = cudaFree(memory);
        return error == cudaSuccess ? 0 : host::fail(context, "peer region release", error);
    });
}

extern "C" int camblas_cuda_peer_reset(camblas_cuda_context *context, void *memory, int world,
                                       size_t capacity)
{
    return host::guarded(context, [&] {
        if (!memory || world < 1 || world > peer::kMaxWorld || capacity == 0)
            return host::fail(context, "invalid peer region description", 1);
        peer::Region region = peer::carve(memory, world, capacity);
        /* the flagged lines lie directly behind the flag words */
        cudaError_t error = cudaMemsetAsync(
            region.flags, 0, size_t(peer::kFlagWords) * 4 + peer::line_bytes(world), context->stream);
        return error == cudaSuccess ? 0 : host::fail(context, "peer flag reset", error);
    });
}

extern "C" int camblas_cuda_peer_allreduce_bf16(camblas_cuda_context *context, int rank, int world,
                                                size_t capacity, void *const *memory, int phases,
                                                size_t count, const void *input, void *output)
{
    return host::guarded(context, [&] {
        if (world < 1 || world > peer::kMaxWorld || rank < 0 || rank >= world || !memory ||
            capacity == 0 || (phases & ~7) != 0 || phases == 0)
            return host::fail(context, "invalid all-reduce group description", 1);
        for (int r = 0; r < world; ++r)
            if (!memory[r])
                return host::fail(context, "missing peer region", 1);
        if (count == 0)
            return 0;
        if (!input || !output || count % 8 != 0 || !host::aligned16(input) || !host::aligned16(output))
            return host::fail(context,
                              "peer all-reduce needs 16-byte aligned BF16 buffers of a multiple of 8 elements",
                              1);
        const size_t chunks = (count + peer::kSmallChunkElements - 1) / peer::kSmallChunkElements;
        if (count > capacity || chunks > size_t(peer::kSmallChunks))
            return host::fail(context,
                              "peer all-reduce exceeds the region capacity or 8.8 million elements", 1);
        if (count <= size_t(peer::kLineMaxElements)) {
            peer::LineTask task{};
            task.rank = rank, task.world = world;
            task.elements = static_cast<long long>(count);
            task.input = static_cast<const __nv_bfloat16 *>(input);
            task.output = static_cast<__nv_bfloat16 *>(output);
            for (int r = 0; r < world; ++r) {
                const peer::Region region = peer::carve(memory[r], world, capacity);
                task.slot_at[r] = region.lines + size_t(rank) * peer::kLineSlotLines;
                if (r == rank) {
                    task.lines = region.lines;
                    task.calls = region.flags + peer::kLineBase;
                }
            }
            task.status = context->status;
            task.wait_ns = 1000000ull * unsigned(context->options.peer_wait_ms);
            /* Two steps over slices where the one-shot form would send more than about
             * 1.75 MB of payload per GPU (measured on four ranks: 1 MB 13.9 -> 10.8 us,
             * 512 KB level, 128-256 KB 6-7 -> 8-9 us: the second trip costs some 3 us);
             * `phases` 3 means all of it. */
            if (world >= 4 && count * sizeof(__nv_bfloat16) * size_t(world - 1) >= 1792 * 1024) {
                peer::SliceTask sliced{};
                sliced.base = task;
                sliced.slice = static_cast<long long>((count / size_t(world) + 7) / 8 * 8);
                if (sliced.slice * world < static_cast<long long>(count))
                    sliced.slice += 8;
                const size_t slice_chunks =
                    (size_t(sliced.slice) + peer::kSmallChunkElements - 1) / peer::kSmallChunkElements;
                peer::peer_lines_allreduce_sliced<<<unsigned(slice_chunks), 256, 0, context->stream>>>(
                    sliced, phases == 3 ? 7 : phases);
                return host::launched(context, "peer all-reduce through flagged lines, sliced");
            }
            if ((phases & 3) == 0)
                return 0; /* the third phase exists only in the sliced form */
            peer::peer_lines_allreduce<<<unsigned(chunks), 256, 0, context->stream>>>(task, phases & 3);
            return host::launched(context, "peer all-reduce through flagged lines");
        }
        peer::SmallTask task{};
        task.rank = rank, task.world = world;
        task.elements = static_cast<long long>(count);
        task.input = static_cast<const __nv_bfloat16 *>(input);
        task.output = static_cast<__nv_bfloat16 *>(output);
        for (int r = 0; r < world; ++r) {
            const peer::Region region = peer::carve(memory[r], world, capacity);
            task.slot_at[r] = region.staging + size_t(rank) * region.slot_elements;
            task.flags_at[r] = region.flags + peer::kSmallBase;
            if (r == rank) {
                task.staging = region.staging;
                task.slot_elements = static_cast<long long>(region.slot_elements);
                task.flags = region.flags + peer::kSmallBase;
            }
        }
        task.status = context->status;
        task.wait_ns = 1000000ull * unsigned(context->options.peer_wait_ms);
        peer::peer_small_allreduce<<<unsigned(chunks), 256, 0, context->stream>>>(task, phases);
        return host::launched(context, "peer all-reduce");
    });
}

extern "C" int camblas_cuda_linear_bf16_allreduce(camblas_cuda_context *context, int rank, int world,
                                                  size_t capacity, void *const *memory, int phases,
                                                  int rows, int inner, int outputs, const void *x,
                                                  int ldx, const void *w, int ldw, const void *bias,
                                                  const void *residual, int ldr)
{
    return host::guarded(context, [&] {
        if (world < 1 || world > peer::kMaxWorld || rank < 0 || rank >= world || !memory ||
            capacity == 0 || (phases & ~7) != 0 || phases == 0)
            return host::fail(context, "invalid row-parallel group description", 1);
        for (int r = 0; r < world; ++r)
            if (!memory[r])
                return host::fail(context, "missing peer region", 1);
        if (rows < 0 || inner < 1 || outputs < 0 || ldx < inner || ldw < inner ||
            (residual && ldr < outputs))
            return host::fail(context, "invalid row-parallel linear dimensions", 1);
        if (rows == 0 || outputs == 0)
            return 0;
        if (size_t(rows) * size_t(outputs) > capacity)
            return host::fail(context, "row-parallel result exceeds the peer region capacity", 1);
        if (outputs % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0 || (residual && ldr % 8 != 0) ||
            !host::aligned16(x) || !host::aligned16(w) || (bias && !host::aligned16(bias)) ||
            (residual && !host::aligned16(residual)))
            return host::fail(context,
                              "row-parallel linear needs 16-byte aligned rows (multiples of 8 elements)",
                              1);
        if (!x || !w)
            return host::fail(context, "missing row-parallel linear operand", 1);
        peer::Call call{};
        call.rank = rank, call.world = world, call.capacity = capacity, call.memory = memory;
        call.phases = phases;
        call.rows = rows, call.inner = inner, call.outputs = outputs;
        call.x = static_cast<const __nv_bfloat16 *>(x), call.ldx = ldx;
        call.w = static_cast<const __nv_bfloat16 *>(w), call.ldw = ldw;
        call.bias = static_cast<const __nv_bfloat16 *>(bias);
        call.residual = static_cast<const __nv_bfloat16 *>(residual), call.ldr = ldr;
        return peer::run(context, call);
    });
}
