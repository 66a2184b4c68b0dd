/*
 * C ABI of libcamblas_cuda.so, B200 (sm_100a) build.
 *
 * Every function of the reference header include/camblas_cuda.h is declared
 * here with the same name, argument list and status convention, so a caller
 * compiled against the reference links against this library unchanged. Each
 * declaration cites the reference declaration and implementation it stands in
 * for. The FP32 / FP64 entry points outside the BF16/FP8 GEMM path (sgemm, dgemm,
 * affine, MLP, attention, MLP backward) run on a tiled CUDA-core GEMM of this
 * library; nothing here falls back to a CPU or to a vendor GEMM library.
 *
 * Conventions shared by all entry points
 *   status      0 on success, negative on failure; the text of the last
 *               failure is camblas_cuda_error(context) (creation failures are
 *               kept per host thread and read with a NULL context).
 *   memory      all operand, output and workspace pointers are device memory
 *               of the context's device, owned by the caller, and must stay
 *               alive until the context stream has drained. Outputs never
 *               alias inputs unless a function says otherwise.
 *   execution   work is enqueued on the context stream and returns without
 *               waiting. The calling thread's current device is restored.
 *   threading   a context serves one host thread and one stream; it is not
 *               usable after fork().
 *   capture     scratch-using operations must be run once on the stream before
 *               that stream is captured into a CUDA graph; growth of scratch is
 *               refused during capture, and scratch addresses recorded by a
 *               capture stay valid until camblas_cuda_destroy().
 */
#ifndef CAMBLAS_CUDA_H
#define CAMBLAS_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct camblas_cuda_context camblas_cuda_context;

/* Multiplication policies; values match reference include/camblas_cuda.h:14-23.
 * AUTO, CLASSICAL and LT all select the tcgen05 GEMM (LT has no separate
 * library route here). For BF16 the reference runs the classical library GEMM
 * under every policy, the Strassen ones included (camblas_cuda.h:64-66;
 * bfloat16.cuh has no Strassen branch), and so does this library by default:
 * STRASSEN, the multi-level values and SYMMETRIC are accepted and computed
 * classically. A one-level BF16 Strassen exists as a deliberate extension
 * behind the context option "bf16_strassen" (camblas_cuda_set_option): with it
 * set, STRASSEN on 'N','N' squares whose order is a multiple of 512 multiplies
 * seven half-size products of BF16-rounded operand sums, which costs accuracy
 * (measured rel-L2 against FP64 2-5 times the classical kernel's on uniform
 * [-1,1] inputs) and gives different bits than the classical kernel. */
enum camblas_cuda_algorithm {
    CAMBLAS_CUDA_AUTO = 0,
    CAMBLAS_CUDA_CLASSICAL = 1,
    CAMBLAS_CUDA_STRASSEN = 2,
    CAMBLAS_CUDA_LT = 3,
    CAMBLAS_CUDA_SYMMETRIC = 4,
    CAMBLAS_CUDA_STRASSEN_TWO = 5,
    CAMBLAS_CUDA_STRASSEN_THREE = 6,
    CAMBLAS_CUDA_STRASSEN_FOUR = 7
};

/* ---- context lifetime -------------------------------------------------- */

/* Replaces camblas_cuda_create (camblas_cuda.h:39; backend.cu:954-1015).
 * stream is a cudaStream_t passed as void* (NULL = legacy default stream).
 * The context owns a scratch arena, a device status word and eight launch
 * counters; it holds no vendor-library handle. Must not be called while the
 * stream is being captured. */
int camblas_cuda_create(int device, void *stream, camblas_cuda_context **out);
/* Replaces camblas_cuda_destroy (camblas_cuda.h:40; backend.cu:1017-1042).
 * Waits for the stream, then frees every allocation the context ever made.
 * NULL is accepted. */
int camblas_cuda_destroy(camblas_cuda_context *context);
/* Replaces camblas_cuda_error (camblas_cuda.h:41; backend.cu:1044-1047). */
const char *camblas_cuda_error(const camblas_cuda_context *context);
/* Replaces camblas_cuda_set_algorithm (camblas_cuda.h:42; backend.cu:1049-1055). */
int camblas_cuda_set_algorithm(camblas_cuda_context *context, int algorithm);
/* Replace camblas_cuda_stats / reset_stats (camblas_cuda.h:211-215;
 * backend.cu:1477-1493). Slots: 0 classical GEMM launches (tcgen05, skinny and
 * generic kernels), 1 Strassen, 2 Gram (always 0), 3 affine layers, 4 LT
 * policy launches, 5 guarded classical fall-backs, 6 attention calls, 7 MLP
 * backward calls. length is 6 or 8. */
int camblas_cuda_stats(const camblas_cuda_context *context, uint64_t *counts, int length);
int camblas_cuda_reset_stats(camblas_cuda_context *context);

/* ---- BF16 GEMM --------------------------------------------------------- */

/* Replaces camblas_cuda_bgemm (camblas_cuda.h:67-72; backend.cu:1075-1084;
 * bfloat16.cuh:11-57). C = alpha op(A) op(B) + beta C over column-major BF16
 * storage with FP32 accumulation and FP32 scalars, one rounding to BF16.
 * trans_* is 'N'/'n' or 'T'/'t'. m==0 or n==0 succeeds without touching memory.
 * alpha==0 or k==0 scales C by beta without reading A or B (which may then be
 * NULL); beta==0 overwrites C without reading it, so NaNs in C do not survive.
 * lda/ldb/ldc must cover the stored rows; A==C or B==C is rejected. Elements
 * of C beyond row m of each column are left untouched. */
int camblas_cuda_bgemm(camblas_cuda_context *context, char trans_a, char trans_b, int m, int n,
                       int k, float alpha, const void *a, int lda, const void *b, int ldb,
                       float beta, void *c, int ldc);

/* No counterpart in the reference ABI (its torch binding issues bgemm and a
 * separate add, torch_bindings.cpp:244-270, and materialises addmm's bias,
 * torch_backend.cuh:59-71). Row-major linear layer with the epilogue fused:
 *   out[rows,outputs] = x[rows,inner] . w[outputs,inner]^T (+ bias[outputs])
 *                       (+ residual[rows,outputs])
 * ldx/ldw/ldo/ldr are row strides in elements; bias and residual may be NULL.
 * out may equal residual; it must not overlap x or w. */
int camblas_cuda_linear_bf16(camblas_cuda_context *context, int rows, int inner, int outputs,
                             const void *x, int ldx, const void *w, int ldw, const void *bias,
                             const void *residual, int ldr, void *out, int ldo);

/* No counterpart in the reference ABI (qkv_linear_public runs three GEMMs,
 * torch_bindings.cpp:725-736). One launch over a weight that stores the q, k
 * and v projections as consecutive row blocks [q_out+k_out+v_out, inner]; the
 * three results go to three distinct row-major outputs with their own row
 * strides. */
int camblas_cuda_qkv_linear_bf16(camblas_cuda_context *context, int rows, int inner, int q_out,
                                 int k_out, int v_out, const void *x, int ldx, const void *w,
                                 int ldw, void *q, int ldq, void *k, int ldk, void *v, int ldv);

/* Has no counterpart in the reference. A linear layer for one to four token
 * rows, out[rows,outputs] = x[rows,inner] . w[outputs,inner]^T (row strides
 * ldx/ldw/ldo in elements, BF16, FP32 accumulation, one rounding), for callers
 * that may not allocate device memory when they need the product: processes
 * whose own memory pool owns the whole device and forbids later driver
 * allocations, and latency-bound paths that cannot absorb an allocation. It takes a cudaStream_t (as void*) instead of a context,
 * runs on the calling thread's current device, and calls no allocator: the FP32
 * partial sums of its K split live in a fixed 8 MiB array inside the library
 * image (held by every GPU that loads the library until the process exits).
 * A product whose partial sums (K splits x rows x outputs x 4 bytes) exceed
 * 8 MiB is rejected with -1 and a message that names both sizes. Weight rows
 * must be 16-byte aligned (w aligned, ldw a multiple of 8). The first call on
 * each device looks up the array's device address; make that call before any
 * stream capture. All calls on a device share the array: it needs no clearing
 * (every partial is written before it is read), but two calls that overlap on
 * the GPU race on it - keep them ordered. Host threads may call it
 * concurrently (the per-device look-up runs once, under a once-flag; the
 * failure text is per thread), but each thread is responsible for ordering its
 * GPU work against the others' as above. Failure text is read with
 * camblas_cuda_error(NULL). */
int camblas_cuda_linear_bf16_static(void *stream, int rows, int inner, int outputs, const void *x,
                                    int ldx, const void *w, int ldw, void *out, int ldo);

/* No counterpart in the reference ABI: there the MLP's first half is a GEMM that
 * writes [rows, 2*intermediate] and camblas_cuda_silu_multiply
 * (camblas_cuda.h:115-121; inference_fusion.cuh:19-29) that reads it back.
 * This entry point does both in one pass: out[rows, intermediate] =
 * rnd(rnd(SiLU(rnd(x . Wg^T))) * rnd(x . Wu^T)), the roundings of the two-step
 * path, so the result equals silu_multiply applied to the BF16 GEMM outputs.
 * `w` is [2*intermediate, inner] with gate and up rows interleaved in blocks of
 * 128: rows [256j, 256j+128) are gate features [128j, 128j+128), rows
 * [256j+128, 256j+256) the up features of the same indices (a one-time
 * permutation of the packed [gate; up] weight). intermediate must be a
 * multiple of 128; x, w, out 16-byte aligned, ldx, ldw, ldo multiples of 8.
 * May grow the context's scratch on first use (not during stream capture). */
int camblas_cuda_gate_up_swiglu_bf16(camblas_cuda_context *context, int rows, int inner,
                                     int intermediate, const void *x, int ldx, const void *w,
                                     int ldw, void *out, int ldo);

/* No counterpart in the reference ABI. camblas_cuda_gate_up_swiglu_bf16 whose
 * result leaves as the FP8 input of the down projection: q[rows, intermediate]
 * (E4M3, contiguous) and scale[rows, intermediate/128] (FP32) are exactly what
 * camblas_cuda_fp8_quantize_rows produces from the BF16 result of
 * camblas_cuda_gate_up_swiglu_bf16 - every 128 outputs that a GEMM tile holds
 * for a row are one quantisation group - without that BF16 tensor being written
 * or read. The reference quantises the activated product in the prologue of its
 * block-128 kernel (camblas/_hopper.py:66-98). Same weight layout and
 * requirements as camblas_cuda_gate_up_swiglu_bf16; q 16-byte aligned. */
int camblas_cuda_gate_up_swiglu_fp8(camblas_cuda_context *context, int rows, int inner,
                                    int intermediate, const void *x, int ldx, const void *w,
                                    int ldw, void *q, float *scale);

/* ---- row-parallel linear layer over several GPUs ------------------------ */

/* None of the following has a counterpart in the reference, which has no
 * multi-GPU code: in its published runs the sum over tensor-parallel ranks is
 * the all-reduce SGLang issues after the hooked F.linear (sglang.py:250-285).
 *
 * One process per GPU. Every GPU owns one *peer region*,
 *   [result: capacity BF16][staging: world slots of capacity BF16][flag words],
 * of camblas_cuda_peer_bytes(world, capacity) bytes, where capacity bounds
 * rows * outputs of any later call, each rounded up to a multiple of 256. camblas_cuda_peer_alloc allocates and
 * clears it and, when `handle` is not NULL, writes a 64-byte CUDA IPC handle
 * that another process on the same machine passes to camblas_cuda_peer_open to
 * map the region into its own address space (the caller carries the bytes
 * between processes). camblas_cuda_peer_close unmaps an opened region,
 * camblas_cuda_peer_free releases an allocated one; both synchronise the
 * context's stream first. The regions must outlive all work that uses them. */
size_t camblas_cuda_peer_bytes(int world, size_t capacity);
int camblas_cuda_peer_alloc(camblas_cuda_context *context, size_t bytes, void **memory,
                            void *handle);
int camblas_cuda_peer_open(camblas_cuda_context *context, const void *handle, void **memory);
int camblas_cuda_peer_close(camblas_cuda_context *context, void *memory);
int camblas_cuda_peer_free(camblas_cuda_context *context, void *memory);
/* Clears the flag words of this GPU's own region on the context's stream. Only
 * needed after a call failed with a device status; all GPUs must be idle (host
 * barrier before and after). */
int camblas_cuda_peer_reset(camblas_cuda_context *context, void *memory, int world,
                            size_t capacity);

/* result[rows,outputs] = sum over ranks of x_r[rows,inner] . w_r[outputs,inner]^T
 * (+ bias[outputs] + residual[rows,outputs]), BF16 with FP32 accumulation, where
 * rank r holds the r-th slice of the inner dimension of both operands (inner is
 * the slice's depth). memory[r] is rank r's peer region as mapped in this
 * process (memory[rank] the region this process allocated); the full result
 * appears at the start of memory[rank] with row stride `outputs` on every rank,
 * bit-identical on all of them. All ranks must make the same sequence of calls
 * with the same rows and outputs. bias and residual are read on every rank from
 * its own copies (they must be equal); they are added once, in FP32, before the
 * single rounding of the sum of the BF16-rounded partial products.
 *
 * Launches on the context's stream, asynchronous: (1) the two-SM tcgen05
 * product whose epilogue sends each tile straight into the staging slot of
 * the GPU that owns the tile (owner = column block mod world) over NVLink and
 * raises that GPU's arrival word, tile by tile while later tiles are still
 * being multiplied; (2) on the owner, a kernel that waits for the `world`
 * partials of each 32-row slab, adds them in rank order, applies bias and
 * residual and writes the finished slab into every GPU's result; (3) a wait
 * until every slab has been delivered to this GPU (part of launch 2 when both
 * are requested together). `phases` is a bit mask of the steps to issue, 7 in
 * production; the parts exist so that a single
 * process can drive several ranks on one GPU in turn (all of 1, then all of 2,
 * then all of 4), where no kernel may wait for one that has not been launched.
 * Waits inside the kernels give up after five seconds (option "peer_wait_ms"
 * of camblas_cuda_set_option) and record a device
 * status (camblas_cuda_device_status), after which camblas_cuda_peer_reset is
 * needed. The result may be overwritten by the next call: consume it with work
 * enqueued on the same stream before that call. rows * outputs, each rounded up
 * to a multiple of 256, <= capacity; outputs, ldx, ldw and ldr multiples of 8; x, w, bias, residual 16-byte
 * aligned; world <= 8. */
int camblas_cuda_linear_bf16_allreduce(camblas_cuda_context *context, int rank, int world,
                                       size_t capacity, void *const *memory, int phases, int rows,
                                       int inner, int outputs, const void *x, int ldx,
                                       const void *w, int ldw, const void *bias,
                                       const void *residual, int ldr);

/* No counterpart in the reference (SGLang's all-reduce follows the hooked
 * F.linear there). Sum of one BF16 tensor of `count` elements per rank over
 * the ranks of a peer-region group, for the small results of decoding (a few
 * token rows): output = rnd(input_0 + input_1 + ... in rank order, FP32), the
 * same bits on every rank. One kernel per rank on the context's stream, no
 * collective library and no second launch. Up to 524 288 elements (1 MiB) every
 * 8 bytes travel to each peer as a 16-byte line that carries the call's number
 * beside the payload, the receiver polls the lines until the number is the
 * current one (bounded, "peer_wait_ms"), and the exchange costs one trip over
 * NVLink; the calls of one rank must then run in stream order, because two line
 * buffers alternate. With four ranks or more, where that would send more than
 * about 1.75 MB per GPU, the tensor goes in two such trips over `world` slices
 * (every rank adds one slice and sends the sum to all), with the same bits. Larger tensors are stored into this rank's staging slot on
 * every GPU, announced and acknowledged through counted flag words per chunk of
 * 2048 elements. All ranks must make the same sequence of calls with the same
 * count. count is a multiple of 8, at most min(capacity, 8 867 840); input and
 * output 16-byte
 * aligned, output may be input. `phases` is 3 in production (everything); 1
 * (send), 2 (receive and add; in the two-trip form also send the sum) and 4
 * (two-trip form: collect the sums; otherwise nothing) exist so that one process
 * can drive several ranks on one GPU in turn. After a wait has expired (device status) the region needs
 * camblas_cuda_peer_reset. */
int camblas_cuda_peer_allreduce_bf16(camblas_cuda_context *context, int rank, int world,
                                     size_t capacity, void *const *memory, int phases,
                                     size_t count, const void *input, void *output);

/* ---- residual add + RMS normalisation ---------------------------------- */

/* Replaces camblas_cuda_rms_norm (camblas_cuda.h:171-175; backend.cu:1423-1440).
 * dtype 0 FP32, 2 BF16. out = rnd(rnd(x * rsqrt(mean(x^2)+eps)) * weight). */
int camblas_cuda_rms_norm(camblas_cuda_context *context, int dtype, int rows, int width,
                          float epsilon, const void *input, const void *weight, void *output);
/* Replaces camblas_cuda_rms_norm_decode (camblas_cuda.h:176-183;
 * backend.cu:1363-1396): one row, width 2048..65536 divisible by four, with the
 * 512-thread four-accumulator reduction order of inference_fusion.cuh:136-191. */
int camblas_cuda_rms_norm_decode(camblas_cuda_context *context, int dtype, int weight_dtype,
                                 int width, float epsilon, int round_before_weight, int descending,
                                 const void *input, const void *weight, void *output);
/* Replaces camblas_cuda_add_rms_norm (camblas_cuda.h:184-189; backend.cu:1398-1421):
 * one row; added = rnd(input+residual); output = rnd(rnd(added*s)*weight). */
int camblas_cuda_add_rms_norm(camblas_cuda_context *context, int dtype, int width, float epsilon,
                              const void *input, const void *residual, const void *weight,
                              void *added, void *output);
/* No counterpart in the reference ABI (it handles one row per call and its
 * torch binding falls back to separate add and RMS kernels for more rows,
 * torch_bindings.cpp:686-690). Same arithmetic as camblas_cuda_add_rms_norm for
 * rows >= 1 contiguous rows; width is a positive multiple of 8 up to 65536. */
int camblas_cuda_add_rms_norm_rows(camblas_cuda_context *context, int dtype, int rows, int width,
                                   float epsilon, const void *input, const void *residual,
                                   const void *weight, void *added, void *output);
/* No counterpart in the reference ABI. camblas_cuda_add_rms_norm_rows for rows
 * that are not packed back to back: row i of input, residual, added and output
 * starts ld_input, ld_residual, ld_added and ld_output elements after row i-1
 * (each >= width), so that column slices and interleaved buffers are
 * normalised where they lie instead of being copied first. Same arithmetic,
 * same bits. The rows of `added` and `output` must not overlap any row read. */
int camblas_cuda_add_rms_norm_strided(camblas_cuda_context *context, int dtype, int rows, int width,
                                      float epsilon, const void *input, long long ld_input,
                                      const void *residual, long long ld_residual,
                                      const void *weight, void *added, long long ld_added,
                                      void *output, long long ld_output);
/* Replace camblas_cuda_bfloat16_square / rms_scale (camblas_cuda.h:190-198;
 * backend.cu:1442-1475). */
int camblas_cuda_bfloat16_square(camblas_cuda_context *context, uint64_t count, const void *input,
                                 float *output);
int camblas_cuda_rms_scale(camblas_cuda_context *context, int dtype, uint64_t count, int width,
                           float epsilon, const void *input, const void *weight, const float *means,
                           void *output);

/* ---- FP8 E4M3 w8a8 ------------------------------------------------------ */

/* No counterpart in the reference ABI; the arithmetic is the quantiser of the
 * reference's block-128 decode kernel (camblas/_hopper.py:82-98). For every
 * 128-element group of each row: scale = max(amax,1e-10)/448 (FP32),
 * q = e4m3_satfinite(clamp(x * (448/max(amax,1e-10)), -448, 448)).
 * x is BF16 [rows,inner] with row stride ldx; q is E4M3 [rows,inner]
 * contiguous; scale is FP32 [rows, inner/128] contiguous. inner % 128 == 0. */
int camblas_cuda_fp8_quantize_rows(camblas_cuda_context *context, int rows, int inner,
                                   const void *x, int ldx, void *q, float *scale);
/* No counterpart in the reference ABI for rows > 1 (the reference's block-128
 * product is single-token, camblas/_hopper.py:13-182). Row-major
 *   out[rows,outputs] = sum over 128-deep K blocks g, in ascending g, of
 *        fma(dot_g(q[r,:], w[o,:]), q_scale[r,g] * w_scale[o/128,g], acc)
 * with E4M3 q [rows,inner], E4M3 w [outputs,inner], FP32 q_scale
 * [rows,inner/128], FP32 w_scale [ceil(outputs/128), inner/128], BF16 out with
 * row stride ldo, one rounding at the end. inner % 128 == 0; outputs % 8 == 0. */
int camblas_cuda_fp8_block_gemm(camblas_cuda_context *context, int rows, int outputs, int inner,
                                const void *q, const float *q_scale, const void *w,
                                const float *w_scale, void *out, int ldo);

/* Replace camblas_cuda_fp8_decode_supported / fp8_decode / fp8_workspace_size /
 * fp8_linear (camblas_cuda.h:137-163; backend.cu:1193-1256; fp8_decode.cuh):
 * single-token block-32 E4M3 product with FP32 scales and ordered FP32
 * accumulation; fp8_linear quantises a BF16 token with power-of-two block-32
 * scales first. inner is a multiple of 32 in [32,8192], outputs a positive
 * multiple of 16. The workspace query always returns 0 in this build. */
int camblas_cuda_fp8_decode_supported(const camblas_cuda_context *context);
int camblas_cuda_fp8_decode(camblas_cuda_context *context, int outputs, int inner,
                            const void *input, const float *input_scale, const void *weight,
                            const float *weight_scale, int input_scale_stride,
                            int weight_scale_row_stride, int weight_scale_column_stride,
                            void *workspace, size_t workspace_bytes, void *output);
size_t camblas_cuda_fp8_workspace_size(int quantise, int outputs, int inner);
int camblas_cuda_fp8_linear(camblas_cuda_context *context, int outputs, int inner,
                            const void *input, const void *weight, const float *weight_scale,
                            int weight_scale_row_stride, int weight_scale_column_stride,
                            void *workspace, size_t workspace_bytes, void *output);

/* ---- elementwise --------------------------------------------------------- */

/* Replace camblas_cuda_silu_multiply / swiglu (camblas_cuda.h:107-121;
 * inference_fusion.cuh:19-51). dtype 0 FP32, 2 BF16. */
int camblas_cuda_silu_multiply(camblas_cuda_context *context, int dtype, uint64_t count,
                               const void *gate, const void *up, void *output);
int camblas_cuda_swiglu(camblas_cuda_context *context, int dtype, uint64_t count, int width,
                        float limit, const void *gate, const void *up, const float *routing,
                        void *output);

/* ---- diagnostics ---------------------------------------------------------- */

/* No counterpart in the reference ABI. Copies the device status word of the
 * context to *status after waiting for the stream: 0 when every bounded wait
 * inside the pipelined kernels completed; otherwise a code naming the wait that
 * gave up (role in bits 0-3, CTA index above). Clears the word. */
int camblas_cuda_device_status(camblas_cuda_context *context, unsigned *status);
/* No counterpart in the reference ABI. Number of CUDA kernels this context has
 * enqueued since it was created (every launch, including reduction and fix-up
 * passes; graph replays are not counted). */
int camblas_cuda_kernel_launches(const camblas_cuda_context *context, uint64_t *count);
/* No counterpart in the reference ABI. Sets one tuning or test switch of the
 * context by name; returns -1 for an unknown name or a value out of range.
 * Every switch starts from the environment variable in parentheses, which is
 * read once when the context is created; no call on the hot path reads the
 * environment.
 *   "pair_tail"      0 cost model, 1 whole tiles only, 2 always split the last
 *                    wave of the two-SM BF16 kernel by K
 *                    (CAMBLAS_B200_PAIR_MODE=plain|sk)
 *   "pair_width"     forced tile width of the two-SM kernel, a multiple of 16 up
 *                    to 256, 0 = off (CAMBLAS_B200_PAIR_MODE=width=<n>)
 *   "push_width"     0, 128 or 256: tile width of the peer-memory row-parallel
 *                    product (CAMBLAS_B200_PUSH_WIDTH)
 *   "fp8_rows"       which many-row FP8 kernel, all with the same bits: 0 by size,
 *                    1 four-warp, 2 one-block-per-stage, 5 current 128 x 128
 *                    tiles, 3 / 4 128 x 256 tiles on one SM / 256 x 256 on two
 *                    (CAMBLAS_B200_FP8_ROWS=four|single)
 *   "fp8_swapped_rows" 0..128: most token rows for which the FP8 block GEMM
 *                    puts the weights on the 128-row side of the tiles and
 *                    the tokens on a 16 to 64 column side (default 16; an
 *                    output that is not 16-byte aligned, or whose ldo is not
 *                    a multiple of 8, stays there up to 128 rows)
 *   "cluster_split"  K split inside a thread-block cluster with the partial
 *                    sums added through distributed shared memory: 0 never,
 *                    1 for products of 65 token rows and more with few tiles
 *                    (default), 2 also for the few-token kernels
 *   "bf16_strassen"  1 lets policy STRASSEN run one Strassen level on BF16
 *                    squares (CAMBLAS_B200_BF16_STRASSEN)
 *   "peer_wait_ms"   1..60000, how long a kernel of the row-parallel layer waits
 *                    for another GPU's flag before it gives up (default 5000) */
int camblas_cuda_set_option(camblas_cuda_context *context, const char *name, int value);
/* No counterpart in the reference ABI. Chooses the BF16 kernel family for the
 * next calls on this context: 0 automatic, 1 generic CUDA-core kernel,
 * 2 skinny weight-streaming kernel, 3 tcgen05 kernel, 4 tcgen05 with swapped
 * operands and split-K, 5 tcgen05 kernel with two-SM (CTA pair) tiles. A forced family that cannot take the operands fails
 * with status -1 instead of silently using another one. For tests. */
int camblas_cuda_force_kernel(camblas_cuda_context *context, int family);

/* ---- block-scaled products with power-of-two scales, expert routing ------- */

/* Replaces camblas_cuda_quantized_matmul (camblas_cuda.h:122-135;
 * backend.cu:1165-1191; quantized.cuh:22-177). output[rows,outputs] (BF16) =
 * input . weight^T with FP32 accumulation, where input is E4M3 [rows,inner]
 * with E8M0 scales [rows, inner/activation_block] and weight is E4M3
 * [outputs,inner] with E8M0 scales [ceil(outputs/32), inner/32] (packed = 0,
 * activation_block 32) or packed E2M1, two values per byte, low nibble first,
 * [outputs, inner/2] with E8M0 scales [outputs, inner/32] (packed = 1,
 * activation_block 32 or 128). An E8M0 byte v is 2^(v-127), 0 is 2^-127, 255
 * NaN. Where the reference scales and adds 32-deep block sums in order, this
 * library folds the scales into exact BF16 images of both operands (context
 * operand arena, grown on first use, not during stream capture) and multiplies
 * them on the tensor cores: every term is exact in both, only the order of the
 * FP32 additions differs. rows <= 65535; outputs a positive multiple of 8; inner
 * a positive multiple of 32 and of activation_block. input and weight 16-byte
 * aligned (8 for a packed weight); all five buffers distinct. */
int camblas_cuda_quantized_matmul(camblas_cuda_context *context, int packed, int rows, int outputs,
                                  int inner, int activation_block, const void *input,
                                  const void *input_scale, const void *weight,
                                  const void *weight_scale, void *output);
/* Replaces camblas_cuda_grouped_quantized_matmul (camblas_cuda.h:165-176;
 * backend.cu:1258-1304). input [groups,rows,inner], input scales
 * [groups,rows,inner/activation_block], output BF16 [groups,rows,outputs].
 * metadata is device uint64 [weight_groups][2]: the device addresses of each
 * expert's weight and weight-scale storage in the layouts above (16-byte
 * aligned). active and counts are device int32 [groups]: batch b is multiplied
 * with expert active[b] for its first min(max(counts[b],0),rows) rows; every
 * other row of the output, and every row of a batch whose active[b] is not in
 * [0, weight_groups), is zero. One product launch per batch after two image
 * kernels over all batches; needs groups * (rows + outputs) * inner * 2 bytes of
 * the context's operand arena. */
int camblas_cuda_grouped_quantized_matmul(camblas_cuda_context *context, int packed, int groups,
                                          int weight_groups, int rows, int outputs, int inner,
                                          int activation_block, const void *input,
                                          const void *input_scale, const void *metadata,
                                          const void *active, const void *counts, void *output);
/* Replaces camblas_cuda_route_groups (camblas_cuda.h:177-185;
 * backend.cu:1306-1338; routing.cuh:2-24). experts is device int64
 * [tokens,choices]; slot s = token*choices+choice is routed to the first group
 * g with active[g] == experts[s] - first_expert (ids below first_expert or not
 * below INT_MAX are ignored). counts[g] = slots routed to g (may exceed rows);
 * slots[g][r] = the r-th such slot in ascending slot order for r < rows, else
 * -1; reverse[s] = g*rows + r, or -1 for slots without a row. The reference
 * numbers rows in the order its atomics happen to complete; this numbering is
 * the same on every run. Uses 4 bytes of context scratch per slot. */
int camblas_cuda_route_groups(camblas_cuda_context *context, int tokens, int choices,
                              int first_expert, int groups, int rows, const void *experts,
                              const void *active, void *counts, void *slots, void *reverse);
/* Replaces camblas_cuda_reduce_groups (camblas_cuda.h:186-192;
 * backend.cu:1340-1361; routing.cuh:26-60). output[t][c] (FP32) = sum over the
 * choices of token t, in ascending (expert id, choice index) order, of the BF16
 * value input[reverse[t][choice]][c]; invalid expert ids and reverse rows
 * outside [0, grouped_rows) are skipped. Same additions in the same order as
 * the reference, so the same bits. choices 1..64. */
int camblas_cuda_reduce_groups(camblas_cuda_context *context, int tokens, int choices, int width,
                               int grouped_rows, const void *experts, const void *reverse,
                               const void *input, void *output);

/* ---- FP32 / FP64 GEMM ----------------------------------------------------- */

/* Replace camblas_cuda_sgemm / camblas_cuda_dgemm (camblas_cuda.h:57-62;
 * backend.cu:786-866, 1057-1073). Column-major C = alpha op(A) op(B) + beta C
 * in the storage type, argument rules as for camblas_cuda_bgemm. Off the
 * BF16/FP8 path: a tiled CUDA-core kernel (B200 has no tensor-core mode that
 * keeps FP32 products, and the reference keeps TF32 off); every policy value
 * multiplies classically, no Strassen levels, no Gram shortcut. */
int camblas_cuda_sgemm(camblas_cuda_context *context, char trans_a, char trans_b, int m, int n,
                       int k, float alpha, const float *a, int lda, const float *b, int ldb,
                       float beta, float *c, int ldc);
int camblas_cuda_dgemm(camblas_cuda_context *context, char trans_a, char trans_b, int m, int n,
                       int k, double alpha, const double *a, int lda, const double *b, int ldb,
                       double beta, double *c, int ldc);

/* ---- FP32 / FP64 layer compositions (off the BF16/FP8 GEMM path) ----------- */
/* dtype 0 FP32, 1 FP64; all arrays row-major, contiguous, caller-owned; every
 * product runs on the CUDA-core GEMM above, sums in a fixed order.
 * Replace camblas_cuda_affine / _mlp (camblas_cuda.h:70-78; backend.cu:870-911,
 * 1086-1117): output = x . weight + bias, ReLU on request; the MLP is two such
 * layers with ReLU after the first, whose activations are returned in
 * hidden_output. camblas_cuda_attention (camblas_cuda.h:80-85; fusion.cuh:95-156):
 * softmax(scale q k^T) v for one head, no mask; the scores live in the context's
 * scratch arena. camblas_cuda_mlp_backward (camblas_cuda.h:87-99;
 * fusion.cuh:204-263): every non-NULL gradient is filled; grad_hidden is
 * rows x hidden caller scratch, required when dx, dw1 or db1 is requested. */
int camblas_cuda_affine(camblas_cuda_context *context, int dtype, int rows, int inner, int columns,
                        const void *x, const void *weight, const void *bias, int relu,
                        void *output);
int camblas_cuda_mlp(camblas_cuda_context *context, int dtype, int rows, int inputs, int hidden,
                     int outputs, const void *x, const void *w1, const void *b1, const void *w2,
                     const void *b2, void *hidden_output, void *output);
int camblas_cuda_attention(camblas_cuda_context *context, int dtype, int queries, int keys,
                           int depth, int values, double scale, const void *q, const void *k,
                           const void *v, void *output);
int camblas_cuda_mlp_backward(camblas_cuda_context *context, int dtype, int rows, int inputs,
                              int hidden, int outputs, const void *x, const void *w1,
                              const void *w2, const void *hidden_output, const void *grad_output,
                              void *grad_hidden, void *dx, void *dw1, void *db1, void *dw2,
                              void *db2);

#ifdef __cplusplus
}
#endif
#endif
