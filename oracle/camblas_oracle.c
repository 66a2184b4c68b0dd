/*
 * CPU restatement of the reference arithmetic for the CUDA GEMM path.
 *
 * TEST INFRASTRUCTURE ONLY. Nothing in the shipped library or package calls
 * this file; it exists so that the tests, the smoke check and the CPU leg of
 * the benchmark can compare the CUDA kernels against plain C that follows the
 * reference's algorithms line by line. Each function names the reference code
 * it restates. Parity pins: the golden vectors of the reference's own tests
 * (tests/test_bfloat16.py:94-121, tests/test_quantized.py:160-216,
 * tests/test_inference_fusion.py:106-110, tests/test_float_gemv.py:69-90) and
 * the reference's own cblas_sgemm compiled from its sources (oracle/_ref).
 * Not pinned by any runnable reference code: the block-128 FP8 product for more
 * than one token (the reference has no such kernel) - see oracle_fp8_block_gemm.
 *
 * Build: make -C oracle   (gcc -O2 -ffp-contract=off: no fused multiply-adds
 * are introduced behind the code's back; where the reference fuses, fmaf() is
 * written out).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

/* ---- storage formats ---------------------------------------------------- */

static float bf16_to_float(uint16_t bits)
{
    uint32_t word = (uint32_t)bits << 16;
    float value;
    memcpy(&value, &word, sizeof value);
    return value;
}

/* Round-to-nearest-even FP32 -> BF16, NaN kept quiet (__float2bfloat16_rn). */
static uint16_t float_to_bf16(float value)
{
    uint32_t word;
    memcpy(&word, &value, sizeof word);
    if ((word & 0x7fffffffu) > 0x7f800000u)
        return 0x7fff;
    word += 0x7fffu + ((word >> 16) & 1u);
    return (uint16_t)(word >> 16);
}

static float round_bf16(float value)
{
    return bf16_to_float(float_to_bf16(value));
}

/* E4M3 ("fn" variant: no infinities, 0x7f/0xff are NaN, largest finite 448). */
static float e4m3_to_float(uint8_t bits)
{
    int sign = bits >> 7, exponent = (bits >> 3) & 15, mantissa = bits & 7;
    float value;
    if (exponent == 15 && mantissa == 7)
        return NAN;
    if (exponent == 0)
        value = ldexpf((float)mantissa, -9);
    else
        value = ldexpf((float)(8 + mantissa), exponent - 10);
    return sign ? -value : value;
}

/* FP32 -> E4M3, round to nearest even, finite saturation (the conversion
 * __nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3) performs). */
static uint8_t float_to_e4m3(float value)
{
    uint8_t sign = signbit(value) ? 0x80 : 0;
    float magnitude = fabsf(value);
    if (isnan(value))
        return (uint8_t)(sign | 0x7f);
    if (magnitude >= 448.f)
        return (uint8_t)(sign | 0x7e);
    if (magnitude < ldexpf(1.f, -6)) {
        /* subnormal: multiples of 2^-9, ties to even */
        float scaled = magnitude * 512.f;
        int quantum = (int)rintf(scaled);
        return (uint8_t)(sign | quantum); /* quantum 8 is the smallest normal, 0x08 */
    }
    int exponent;
    float fraction = frexpf(magnitude, &exponent); /* magnitude = fraction * 2^exponent, [0.5,1) */
    int scaled = (int)rintf(fraction * 16.f);      /* 8..16, ties to even */
    if (scaled == 16) {
        scaled = 8;
        exponent += 1;
    }
    int biased = exponent - 1 + 7;
    if (biased > 15 || (biased == 15 && scaled - 8 == 7))
        return (uint8_t)(sign | 0x7e);
    return (uint8_t)(sign | (biased << 3) | (scaled - 8));
}

uint16_t oracle_float_to_bf16(float value) { return float_to_bf16(value); }
float oracle_bf16_to_float(uint16_t bits) { return bf16_to_float(bits); }
uint8_t oracle_float_to_e4m3(float value) { return float_to_e4m3(value); }
float oracle_e4m3_to_float(uint8_t bits) { return e4m3_to_float(bits); }

/* ---- FP32 GEMM: the reference's portable kernel ------------------------- */

/*
 * Column-major C = alpha op(A) op(B) + beta C as the reference's scalar tile
 * function computes it (src/scalar.c:223-255): C is scaled by beta first
 * (beta==0 stores zeros without reading), then every element receives
 * alpha * acc where acc sums a*b in FP32 for l = 0..k-1 in order, each product
 * rounded before the add.
 */
void oracle_sgemm(char trans_a, char trans_b, int m, int n, int k, float alpha, const float *a,
                  int lda, const float *b, int ldb, float beta, float *c, int ldc)
{
    for (int j = 0; j < n; ++j)
        for (int i = 0; i < m; ++i) {
            float *cell = c + i + (size_t)j * ldc;
            if (beta == 0.f)
                *cell = 0.f;
            else if (beta != 1.f)
                *cell *= beta;
        }
    if (alpha == 0.f || k == 0)
        return;
    for (int j = 0; j < n; ++j)
        for (int i = 0; i < m; ++i) {
            float acc = 0.f;
            for (int l = 0; l < k; ++l) {
                float av = trans_a == 'N' ? a[i + (size_t)l * lda] : a[l + (size_t)i * lda];
                float bv = trans_b == 'N' ? b[l + (size_t)j * ldb] : b[j + (size_t)l * ldb];
                acc += av * bv;
            }
            c[i + (size_t)j * ldc] += alpha * acc;
        }
}

/*
 * BF16 GEMM contract of camblas_cuda_bgemm (src/cuda/bfloat16.cuh:11-57):
 * BF16 operands, FP32 accumulation and scalars, result alpha*sum + beta*C
 * rounded once to BF16; alpha==0 or k==0 scales C by beta without reading A/B
 * and beta==0 writes zeros without reading C (bfloat16.cuh:2-9, 24-32). The
 * accumulation order inside the reference is the vendor library's; this
 * restatement sums in ascending l like oracle_sgemm and adds beta*C last.
 */
void oracle_bgemm(char trans_a, char trans_b, int m, int n, int k, float alpha, const uint16_t *a,
                  int lda, const uint16_t *b, int ldb, float beta, uint16_t *c, int ldc)
{
    for (int j = 0; j < n; ++j)
        for (int i = 0; i < m; ++i) {
            uint16_t *cell = c + i + (size_t)j * ldc;
            if (alpha == 0.f || k == 0) {
                if (beta != 1.f)
                    *cell = float_to_bf16(beta == 0.f ? 0.f : beta * bf16_to_float(*cell));
                continue;
            }
            float acc = 0.f;
            for (int l = 0; l < k; ++l) {
                uint16_t av = trans_a == 'N' ? a[i + (size_t)l * lda] : a[l + (size_t)i * lda];
                uint16_t bv = trans_b == 'N' ? b[l + (size_t)j * ldb] : b[j + (size_t)l * ldb];
                acc += bf16_to_float(av) * bf16_to_float(bv);
            }
            float value = alpha * acc;
            if (beta != 0.f)
                value = fmaf(beta, bf16_to_float(*cell), value);
            *cell = float_to_bf16(value);
        }
}

/* Row-major linear with fused epilogue: out = x w^T + bias + residual, one
 * rounding (the arithmetic camblas_cuda_linear_bf16 documents). */
void oracle_linear_bf16(int rows, int inner, int outputs, const uint16_t *x, int ldx,
                        const uint16_t *w, int ldw, const uint16_t *bias, const uint16_t *residual,
                        int ldr, uint16_t *out, int ldo)
{
    for (int r = 0; r < rows; ++r)
        for (int o = 0; o < outputs; ++o) {
            float acc = 0.f;
            for (int l = 0; l < inner; ++l)
                acc += bf16_to_float(x[(size_t)r * ldx + l]) * bf16_to_float(w[(size_t)o * ldw + l]);
            if (bias)
                acc += bf16_to_float(bias[o]);
            if (residual)
                acc = fmaf(1.f, bf16_to_float(residual[(size_t)r * ldr + o]), acc);
            out[(size_t)r * ldo + o] = float_to_bf16(acc);
        }
}

/* ---- RMS normalisation --------------------------------------------------- */

/*
 * One row in the order of the reference's 512-thread kernel
 * (src/cuda/inference_fusion.cuh:136-191): thread t keeps four sums over
 * columns 4t+o+2048i; they are added 0,1,2,3; a halving tree over the 512
 * partials down to 32; then a shuffle-down tree with offsets 1,2,4,8,16
 * (ascending) or 16,8,4,2,1 (descending); scale = rsqrt(sum*(1/width)+eps).
 * Shuffles are modelled on 32 lanes, all updated at once; a lane whose source
 * is beyond lane 31 receives its own value, as __shfl_down_sync does.
 * added = rnd(x+r); out = rnd(rnd?(added*scale) * weight).
 * bf16 != 0: storage is BF16 (weight FP32 when weight_fp32), else FP32.
 * rsqrtf on the device is an approximation with <= 2 ulp error; this file uses
 * 1/sqrt in double rounded to float, so scale may differ by an ulp - the tests
 * compare `added` bit-exactly and `out` within one BF16 ulp.
 */
void oracle_rms_row(int bf16, int weight_fp32, int width, float epsilon, int round_before_weight,
                    int descending, const void *input, const void *residual, const void *weight,
                    void *added, void *output)
{
    static float partial[512];
    for (int t = 0; t < 512; ++t) {
        float sums[4] = {0, 0, 0, 0};
        for (int column = t * 4; column < width; column += 2048)
            for (int o = 0; o < 4; ++o) {
                float value;
                if (bf16) {
                    value = bf16_to_float(((const uint16_t *)input)[column + o]);
                    if (residual)
                        value = round_bf16(
                            value + bf16_to_float(((const uint16_t *)residual)[column + o]));
                } else {
                    value = ((const float *)input)[column + o];
                    if (residual)
                        value = value + ((const float *)residual)[column + o];
                }
                float square = value * value;
                sums[o] = sums[o] + square;
            }
        float sum = sums[0];
        for (int o = 1; o < 4; ++o)
            sum = sum + sums[o];
        partial[t] = sum;
    }
    for (int offset = 256; offset >= 32; offset /= 2)
        for (int t = 0; t < offset; ++t)
            partial[t] = partial[t] + partial[t + offset];
    float lanes[32];
    memcpy(lanes, partial, sizeof lanes);
    if (descending) {
        for (int offset = 16; offset; offset /= 2) {
            float next[32];
            for (int i = 0; i < 32; ++i)
                next[i] = lanes[i] + (i + offset < 32 ? lanes[i + offset] : lanes[i]);
            memcpy(lanes, next, sizeof next);
        }
    } else {
        for (int offset = 1; offset < 32; offset *= 2) {
            float next[32];
            for (int i = 0; i < 32; ++i)
                next[i] = lanes[i] + (i + offset < 32 ? lanes[i + offset] : lanes[i]);
            memcpy(lanes, next, sizeof next);
        }
    }
    float mean = lanes[0] * (1.f / (float)width);
    float shifted = mean + epsilon;
    float scale = (float)(1.0 / sqrt((double)shifted));
    for (int column = 0; column < width; ++column) {
        float value, gamma;
        if (bf16) {
            value = bf16_to_float(((const uint16_t *)input)[column]);
            if (residual) {
                value = round_bf16(value + bf16_to_float(((const uint16_t *)residual)[column]));
                ((uint16_t *)added)[column] = float_to_bf16(value);
            }
            gamma = weight_fp32 ? ((const float *)weight)[column]
                                : bf16_to_float(((const uint16_t *)weight)[column]);
        } else {
            value = ((const float *)input)[column];
            if (residual) {
                value = value + ((const float *)residual)[column];
                ((float *)added)[column] = value;
            }
            gamma = ((const float *)weight)[column];
        }
        float normalised = value * scale;
        if (round_before_weight && bf16)
            normalised = round_bf16(normalised);
        float result = normalised * gamma;
        if (bf16)
            ((uint16_t *)output)[column] = float_to_bf16(result);
        else
            ((float *)output)[column] = result;
    }
}

/* Rows of the single-row arithmetic above (camblas_cuda_add_rms_norm_rows and
 * camblas_cuda_add_rms_norm; reference backend.cu:1398-1421). */
void oracle_add_rms_norm_rows(int bf16, int rows, int width, float epsilon, const void *input,
                              const void *residual, const void *weight, void *added, void *output)
{
    size_t element = bf16 ? 2 : 4;
    for (int row = 0; row < rows; ++row) {
        size_t offset = (size_t)row * width * element;
        oracle_rms_row(bf16, 0, width, epsilon, 1, 0, (const char *)input + offset,
                       (const char *)residual + offset, weight, (char *)added + offset,
                       (char *)output + offset);
    }
}

/* Multi-row RMS norm in the order of the reference's 256-thread kernel
 * (src/cuda/inference_fusion.cuh:53-86). */
void oracle_rms_norm_rows(int bf16, int rows, int width, float epsilon, const void *input,
                          const void *weight, void *output)
{
    for (int row = 0; row < rows; ++row) {
        float thread_sum[256];
        for (int t = 0; t < 256; ++t) {
            float sum = 0.f;
            for (int column = t; column < width; column += 256) {
                float value = bf16 ? bf16_to_float(((const uint16_t *)input)[(size_t)row * width + column])
                                   : ((const float *)input)[(size_t)row * width + column];
                float square = value * value;
                sum = sum + square;
            }
            thread_sum[t] = sum;
        }
        float warp_sum[32] = {0};
        for (int w = 0; w < 8; ++w) {
            float lanes[32];
            memcpy(lanes, thread_sum + 32 * w, sizeof lanes);
            for (int offset = 16; offset; offset /= 2) {
                float next[32];
                for (int i = 0; i < 32; ++i)
                    next[i] = lanes[i] + (i + offset < 32 ? lanes[i + offset] : lanes[i]);
                memcpy(lanes, next, sizeof next);
            }
            warp_sum[w] = lanes[0];
        }
        for (int offset = 16; offset; offset /= 2) {
            float next[32];
            for (int i = 0; i < 32; ++i)
                next[i] = warp_sum[i] + (i + offset < 32 ? warp_sum[i + offset] : warp_sum[i]);
            memcpy(warp_sum, next, sizeof next);
        }
        float shifted = warp_sum[0] / (float)width + epsilon;
        float scale = (float)(1.0 / sqrt((double)shifted));
        for (int column = 0; column < width; ++column) {
            size_t at = (size_t)row * width + column;
            if (bf16) {
                float normalised = round_bf16(bf16_to_float(((const uint16_t *)input)[at]) * scale);
                ((uint16_t *)output)[at] =
                    float_to_bf16(normalised * bf16_to_float(((const uint16_t *)weight)[column]));
            } else {
                float normalised = ((const float *)input)[at] * scale;
                ((float *)output)[at] = normalised * ((const float *)weight)[column];
            }
        }
    }
}

/* ---- SiLU * up ------------------------------------------------------------ */

/* inference_fusion.cuh:19-29: rnd(rnd(g/(1+exp(-g))) * u). expf here is libm's;
 * the device's differs by at most 2 ulp, so tests allow one BF16 ulp. */
void oracle_silu_multiply_bf16(size_t count, const uint16_t *gate, const uint16_t *up,
                               uint16_t *output)
{
    for (size_t i = 0; i < count; ++i) {
        float g = bf16_to_float(gate[i]);
        float activated = round_bf16(g / (1.f + expf(-g)));
        output[i] = float_to_bf16(activated * bf16_to_float(up[i]));
    }
}

/* inference_fusion.cuh:31-51. */
void oracle_swiglu_bf16(size_t count, int width, float limit, const uint16_t *gate,
                        const uint16_t *up, const float *routing, uint16_t *output)
{
    for (size_t i = 0; i < count; ++i) {
        float g = bf16_to_float(gate[i]), u = bf16_to_float(up[i]);
        if (limit > 0) {
            if (g > limit)
                g = limit;
            if (u > limit)
                u = limit;
            if (u < -limit)
                u = -limit;
        }
        float value = (g / (1.f + expf(-g))) * u;
        if (routing)
            value = routing[i / width] * value;
        output[i] = float_to_bf16(value);
    }
}

/* ---- FP8 block-128 (w8a8) -------------------------------------------------- */

/*
 * Activation quantiser of the reference's block-128 decode kernel
 * (camblas/_hopper.py:82-98): per 128 elements amax = max(|x|) floored at
 * 1e-10, scale = amax * (1/448), q = e4m3(clamp(x * (448/amax), -448, 448)).
 * The reference forms 448/amax with the GPU's approximate division; this
 * restatement and the CUDA kernel both use the correctly rounded quotient, so
 * the two agree bit for bit with each other.
 */
void oracle_fp8_quantize_rows(int rows, int inner, const uint16_t *x, int ldx, uint8_t *q,
                              float *scale)
{
    int groups = inner / 128;
    for (int r = 0; r < rows; ++r)
        for (int g = 0; g < groups; ++g) {
            const uint16_t *source = x + (size_t)r * ldx + g * 128;
            float maximum = 1e-10f;
            for (int i = 0; i < 128; ++i)
                maximum = fmaxf(maximum, fabsf(bf16_to_float(source[i])));
            scale[(size_t)r * groups + g] = maximum * (1.0f / 448.0f);
            float inverse = 448.0f / maximum;
            for (int i = 0; i < 128; ++i) {
                float value = bf16_to_float(source[i]) * inverse;
                value = fminf(fmaxf(value, -448.f), 448.f);
                q[(size_t)r * inner + g * 128 + i] = float_to_e4m3(value);
            }
        }
}

/* Weight quantiser for the tests: 128x128 blocks, scale = max(amax,1e-10)/448
 * (the checkpoint format the reference consumes, camblas/_hopper.py:229-232). */
void oracle_fp8_quantize_weight(int outputs, int inner, const uint16_t *w, uint8_t *q, float *scale)
{
    int groups = inner / 128, bands = (outputs + 127) / 128;
    for (int band = 0; band < bands; ++band)
        for (int g = 0; g < groups; ++g) {
            int last = band * 128 + 128 < outputs ? band * 128 + 128 : outputs;
            float maximum = 1e-10f;
            for (int o = band * 128; o < last; ++o)
                for (int i = 0; i < 128; ++i)
                    maximum = fmaxf(maximum, fabsf(bf16_to_float(w[(size_t)o * inner + g * 128 + i])));
            scale[(size_t)band * groups + g] = maximum * (1.0f / 448.0f);
            float inverse = 448.0f / maximum;
            for (int o = band * 128; o < last; ++o)
                for (int i = 0; i < 128; ++i) {
                    float value = bf16_to_float(w[(size_t)o * inner + g * 128 + i]) * inverse;
                    value = fminf(fmaxf(value, -448.f), 448.f);
                    q[(size_t)o * inner + g * 128 + i] = float_to_e4m3(value);
                }
        }
}

/*
 * Block-128 product (camblas/_hopper.py:118-126 products, :168-182 reduction):
 * every 128-deep block is a fresh tensor-core accumulation; the blocks are then
 * combined in ascending order as acc = fma(dot, a_scale*w_scale, acc) and the
 * result is rounded once to BF16. The 128 products of a block are exact in
 * binary64, so dot is formed exactly and rounded to FP32; the tensor core's own
 * in-block rounding is not specified and may differ in the last FP32 bits.
 * The reference implements this for one token; the same recurrence is applied
 * to every row here. PARITY UNPINNED for rows > 1: no reference kernel or test
 * exists to run against.
 */
void oracle_fp8_block_gemm(int rows, int outputs, int inner, const uint8_t *q, const float *q_scale,
                           const uint8_t *w, const float *w_scale, uint16_t *out, int ldo)
{
    int groups = inner / 128;
    static float table[256];
    for (int i = 0; i < 256; ++i)
        table[i] = e4m3_to_float((uint8_t)i);
    for (int r = 0; r < rows; ++r)
        for (int o = 0; o < outputs; ++o) {
            float acc = 0.f;
            for (int g = 0; g < groups; ++g) {
                double dot = 0.0;
                const uint8_t *qa = q + (size_t)r * inner + g * 128;
                const uint8_t *wa = w + (size_t)o * inner + g * 128;
                for (int i = 0; i < 128; ++i)
                    dot += (double)table[qa[i]] * (double)table[wa[i]];
                float scale = q_scale[(size_t)r * groups + g] * w_scale[(size_t)(o / 128) * groups + g];
                acc = fmaf((float)dot, scale, acc);
            }
            out[(size_t)r * ldo + o] = float_to_bf16(acc);
        }
}

/* Dequantise to FP32 for the check the benchmark definition names: the
 * reference's FP32 CPU GEMM on the dequantised operands. */
void oracle_fp8_dequantize(int rows, int inner, int block_rows, const uint8_t *q, const float *scale,
                           float *out)
{
    int groups = inner / 128;
    for (int r = 0; r < rows; ++r)
        for (int i = 0; i < inner; ++i)
            out[(size_t)r * inner + i] =
                e4m3_to_float(q[(size_t)r * inner + i]) * scale[(size_t)(r / block_rows) * groups + i / 128];
}

/* ---- FP8 block-32 single token --------------------------------------------- */

/* Power-of-two activation quantiser (src/cuda/fp8_decode.cuh:60-72): per 32
 * elements, amax floored at 1e-10, e = ceil(log2(amax/448)) taken from the
 * FP32 bits of amax*(1/448), scale = 2^e, q = e4m3(min(x*2^-e, 448)). */
void oracle_fp8_quantize_block32(int inner, const uint16_t *x, uint8_t *q, float *scale)
{
    for (int g = 0; g < inner / 32; ++g) {
        float maximum = 1e-10f;
        for (int i = 0; i < 32; ++i)
            maximum = fmaxf(maximum, fabsf(bf16_to_float(x[g * 32 + i])));
        float ratio = maximum * (1.f / 448.f);
        uint32_t bits;
        memcpy(&bits, &ratio, sizeof bits);
        int exponent = (int)((bits >> 23) & 255) - 127 + ((bits & 0x7fffff) != 0);
        scale[g] = ldexpf(1.f, exponent);
        float multiplier = ldexpf(1.f, -exponent);
        for (int i = 0; i < 32; ++i)
            q[g * 32 + i] = float_to_e4m3(fminf(bf16_to_float(x[g * 32 + i]) * multiplier, 448.f));
    }
}

/* Single-token block-32 product (src/cuda/fp8_decode.cuh:148-165):
 * sum = fma(rnd(dot_g * sw[o/32][g]), sx[g], sum) for g ascending; BF16 out.
 * dot_g is exact (32 products) and rounded to FP32. */
void oracle_fp8_decode(int outputs, int inner, const uint8_t *x, const float *sx, int sx_stride,
                       const uint8_t *w, const float *sw, int sw_row, int sw_col, uint16_t *out)
{
    for (int o = 0; o < outputs; ++o) {
        float sum = 0.f;
        for (int g = 0; g < inner / 32; ++g) {
            double dot = 0.0;
            for (int i = 0; i < 32; ++i)
                dot += (double)e4m3_to_float(x[g * 32 + i]) *
                       (double)e4m3_to_float(w[(size_t)o * inner + g * 32 + i]);
            float scaled = (float)dot * sw[(size_t)(o / 32) * sw_row + (size_t)g * sw_col];
            sum = fmaf(scaled, sx[(size_t)g * sx_stride], sum);
        }
        out[o] = float_to_bf16(sum);
    }
}

/* ---- one-level Strassen ----------------------------------------------------- */

/*
 * Column-major even squares, 'N','N' (src/cuda/backend.cu:128-166): seven
 * half-size products of the packed planes
 *   left  : a11+a22, a21+a22, a11, a22, a11+a12, a21-a11, a12-a22
 *   right : b11+b22, b11, b12-b22, b21-b11, b22, b11+b12, b21+b22
 * recombined as c11 = ((p1+p4)-p5)+p7, c12 = p3+p5, c21 = p2+p4,
 * c22 = ((p1-p2)+p3)+p6, then C = alpha*c + beta*C. For BF16 the packed planes
 * are rounded to BF16 (they feed the BF16 tensor-core kernel), products are
 * kept in FP32, the recombination is FP32 and the result is rounded once.
 */
void oracle_strassen_bf16(int n, float alpha, const uint16_t *a, int lda, const uint16_t *b,
                          int ldb, float beta, uint16_t *c, int ldc, float *work)
{
    int h = n / 2;
    size_t plane = (size_t)h * h;
    float *left = work, *right = work + 7 * plane, *product = work + 14 * plane;
    for (int col = 0; col < h; ++col)
        for (int row = 0; row < h; ++row) {
            size_t at = row + (size_t)col * h;
            float a11 = bf16_to_float(a[row + (size_t)col * lda]);
            float a12 = bf16_to_float(a[row + (size_t)(col + h) * lda]);
            float a21 = bf16_to_float(a[row + h + (size_t)col * lda]);
            float a22 = bf16_to_float(a[row + h + (size_t)(col + h) * lda]);
            float b11 = bf16_to_float(b[row + (size_t)col * ldb]);
            float b12 = bf16_to_float(b[row + (size_t)(col + h) * ldb]);
            float b21 = bf16_to_float(b[row + h + (size_t)col * ldb]);
            float b22 = bf16_to_float(b[row + h + (size_t)(col + h) * ldb]);
            left[at] = round_bf16(a11 + a22);
            left[plane + at] = round_bf16(a21 + a22);
            left[2 * plane + at] = a11;
            left[3 * plane + at] = a22;
            left[4 * plane + at] = round_bf16(a11 + a12);
            left[5 * plane + at] = round_bf16(a21 - a11);
            left[6 * plane + at] = round_bf16(a12 - a22);
            right[at] = round_bf16(b11 + b22);
            right[plane + at] = b11;
            right[2 * plane + at] = round_bf16(b12 - b22);
            right[3 * plane + at] = round_bf16(b21 - b11);
            right[4 * plane + at] = b22;
            right[5 * plane + at] = round_bf16(b11 + b12);
            right[6 * plane + at] = round_bf16(b21 + b22);
        }
    for (int p = 0; p < 7; ++p)
        oracle_sgemm('N', 'N', h, h, h, 1.f, left + p * plane, h, right + p * plane, h, 0.f,
                     product + p * plane, h);
    for (int col = 0; col < h; ++col)
        for (int row = 0; row < h; ++row) {
            size_t at = row + (size_t)col * h;
            float p1 = product[at], p2 = product[plane + at], p3 = product[2 * plane + at];
            float p4 = product[3 * plane + at], p5 = product[4 * plane + at];
            float p6 = product[5 * plane + at], p7 = product[6 * plane + at];
            float q[4] = {((p1 + p4) - p5) + p7, p3 + p5, p2 + p4, ((p1 - p2) + p3) + p6};
            size_t where[4] = {row + (size_t)col * ldc, row + (size_t)(col + h) * ldc,
                               row + h + (size_t)col * ldc, row + h + (size_t)(col + h) * ldc};
            for (int i = 0; i < 4; ++i) {
                float value = alpha * q[i];
                if (beta != 0.f)
                    value = fmaf(beta, bf16_to_float(c[where[i]]), value);
                c[where[i]] = float_to_bf16(value);
            }
        }
}
