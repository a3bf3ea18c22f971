/*
 * TEST INFRASTRUCTURE ONLY — CPU oracle for the blockwise KV quantiser.
 *
 * PARITY UNPINNED: the reference delegates this arithmetic to the third-party
 * bitsandbytes shared library (pinned 0.45.0 in crates/bitsandbytes-sys/build.rs:17-19),
 * which is neither vendored in the reference tree nor installed here, and no reference
 * test pins a single code or scale (crates/hyprstream/src/runtime/kv_cache.rs:2277-2330
 * checks shapes only).  This file therefore states a written specification that honours
 * everything the reference does pin, and chooses — and flags — the rest.
 *
 * Pinned by the reference (followed exactly):
 *   - a block is `blocksize` consecutive elements of the flattened [T, Hkv, D] tensor
 *     (kv_cache.rs:704 QUANT_BLOCKSIZE = 64; bitsandbytes-sys/src/lib.rs:104-105)
 *   - one absmax = max|x| per block (lib.rs:89, QuantState::absmax)
 *   - 8-bit codebook code[i] = (i - 127) / 127 evaluated in f32 (lib.rs:108-111)
 *   - NF4 and FP4 16-entry codebooks (lib.rs:131-148, 152-169)
 *   - 4-bit output occupies (n + 1) / 2 bytes (lib.rs:189-197)
 *   - dequantised value = code[idx] * absmax[block] (kv_cache.rs:871-957 call sites)
 *
 * Chosen here (assumptions, each flagged where used):
 *   A1  normalise by multiplying with the f32 reciprocal 1/absmax (not by dividing)
 *   A2  nearest codeword via f32 midpoints; a value exactly on a midpoint takes the LOWER index
 *   A3  4-bit packing: even-indexed element in the HIGH nibble
 *   A4  an all-zero block stores absmax 0 and the codeword index of the value 0
 *   A5  the 4-bit entry points use the built-in table; no `code` pointer is consulted
 *   A6  f16-scale mode (the 2-byte scales of the ragged-decode and long-context workloads): absmax is rounded to f16 (nearest even,
 *       saturating at 65504) BEFORE it is used to normalise, so codes and the stored scale
 *       stay self-consistent
 * NaN/Inf inputs are outside the contract.
 *
 * Build: see oracle/Makefile (gcc -O2 -ffp-contract=off: no FMA contraction, the
 * arithmetic below is meant literally, one IEEE-754 binary32 rounding per operation).
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

#define HSQ_INT8 1
#define HSQ_NF4 2
#define HSQ_FP4 3

/* lib.rs:131-148 (the published NF4 quantiles) */
static const float k_nf4[16] = {
    -1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f,
    -0.28444138169288635f, -0.18477343022823334f, -0.09105003625154495f, 0.0f,
    0.07958029955625534f, 0.16093020141124725f, 0.24611230945587158f, 0.33791524171829224f,
    0.44070982933044434f, 0.5626170039176941f, 0.7229568362236023f, 1.0f};

/* lib.rs:152-169 (the reference's own FP4 table: unsigned, ascending) */
static const float k_fp4[16] = {0.0f,  0.0625f, 0.125f, 0.1875f, 0.25f,  0.3125f, 0.375f, 0.4375f,
                                0.5f,  0.5625f, 0.625f, 0.6875f, 0.75f,  0.8125f, 0.875f, 1.0f};

/* Fill `table` with the codebook of `kind`; returns its length (256 or 16), 0 on bad kind. */
int hsq_codebook(int kind, float *table) {
    if (kind == HSQ_INT8) {
        for (int i = 0; i < 256; ++i) table[i] = ((float)i - 127.0f) / 127.0f; /* lib.rs:110 */
        return 256;
    }
    if (kind == HSQ_NF4) { memcpy(table, k_nf4, sizeof k_nf4); return 16; }
    if (kind == HSQ_FP4) { memcpy(table, k_fp4, sizeof k_fp4); return 16; }
    return 0;
}

/* f32 midpoints between neighbouring codewords (A2). */
int hsq_midpoints(int kind, float *mid) {
    float t[256];
    int n = hsq_codebook(kind, t);
    for (int i = 0; i + 1 < n; ++i) {
        volatile float s = t[i] + t[i + 1];
        mid[i] = 0.5f * s;
    }
    return n > 0 ? n - 1 : 0;
}

/* binary32 -> binary16 bits, round to nearest even, saturating at 65504 (A6). */
uint16_t hsq_f32_to_f16_sat(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t mag = x & 0x7fffffffu;
    if (mag >= 0x477ff000u) return (uint16_t)(sign | 0x7bffu); /* >= 65520 rounds past max: saturate */
    if (mag < 0x33000001u) return (uint16_t)sign;               /* <= 2^-25: rounds to zero */
    int32_t exp = (int32_t)(mag >> 23) - 127;
    uint32_t man = (mag & 0x7fffffu) | 0x800000u;
    uint32_t shift, half, res;
    if (exp < -14) { /* subnormal half */
        shift = (uint32_t)(13 + (-14 - exp));
        res = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1u);
        half = 1u << (shift - 1);
        if (rem > half || (rem == half && (res & 1u))) res++;
        return (uint16_t)(sign | res);
    }
    res = ((uint32_t)(exp + 15) << 10) | ((man >> 13) & 0x3ffu);
    uint32_t rem = man & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (res & 1u))) res++;
    return (uint16_t)(sign | res);
}

float hsq_f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu, man = h & 0x3ffu, x;
    if (exp == 0) {
        if (man == 0) x = sign;
        else {
            int e = -1;
            do { man <<= 1; e++; } while (!(man & 0x400u));
            x = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31) x = sign | 0x7f800000u | (man << 13);
    else x = sign | ((exp - 15 + 127) << 23) | (man << 13);
    float f;
    memcpy(&f, &x, 4);
    return f;
}

/* bf16 bits <-> f32 (round to nearest even), used by callers that hold bf16 data. */
float hsq_bf16_to_f32(uint16_t b) {
    uint32_t x = (uint32_t)b << 16;
    float f;
    memcpy(&f, &x, 4);
    return f;
}
uint16_t hsq_f32_to_bf16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    if ((x & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((x >> 16) | 0x40u);
    x += 0x7fffu + ((x >> 16) & 1u);
    return (uint16_t)(x >> 16);
}

/*
 * Blockwise quantise `n` f32 values (bf16/fp16 inputs are widened exactly by the caller).
 *   kind       HSQ_INT8 | HSQ_NF4 | HSQ_FP4
 *   blocksize  elements per block (reference: 64)
 *   scale_f16  0: absmax stored as f32 in absmax_f32[]  (reference layout)
 *              1: absmax rounded to f16, bits in absmax_f16[] (A6)
 *   codes      n bytes (8-bit) or (n+1)/2 bytes (4-bit, A3)
 * Mirrors the geometry of QuantizedTensor::from_tensor (kv_cache.rs:741-865).
 * Returns 0, or -1 on bad arguments.
 */
int hsq_quantize_blockwise(int kind, const float *x, int64_t n, int blocksize, int scale_f16,
                           uint8_t *codes, float *absmax_f32, uint16_t *absmax_f16) {
    float table[256], mid[255];
    int ncode = hsq_codebook(kind, table);
    if (ncode == 0 || blocksize <= 0 || n < 0) return -1;
    int nmid = hsq_midpoints(kind, mid);
    int zero_code = 0;
    for (int i = 0; i < ncode; ++i)
        if (table[i] == 0.0f) zero_code = i; /* A4 */
    int four_bit = (ncode == 16);
    if (four_bit) memset(codes, 0, (size_t)((n + 1) / 2));
    int64_t nblocks = (n + blocksize - 1) / blocksize;
    for (int64_t b = 0; b < nblocks; ++b) {
        int64_t lo = b * blocksize, hi = lo + blocksize < n ? lo + blocksize : n;
        float amax = 0.0f;
        for (int64_t i = lo; i < hi; ++i) amax = fmaxf(amax, fabsf(x[i]));
        float a = amax;
        if (scale_f16) {
            uint16_t hb = hsq_f32_to_f16_sat(amax);
            absmax_f16[b] = hb;
            a = hsq_f16_to_f32(hb);
        } else {
            absmax_f32[b] = amax;
        }
        volatile float inv = (a == 0.0f) ? 0.0f : 1.0f / a; /* A1 */
        for (int64_t i = lo; i < hi; ++i) {
            int c;
            if (a == 0.0f) {
                c = zero_code; /* A4 */
            } else {
                volatile float y = x[i] * inv; /* A1: one rounding */
                c = 0;
                for (int j = 0; j < nmid; ++j) c += (y > mid[j]); /* A2 */
            }
            if (four_bit) {
                if ((i & 1) == 0) codes[i >> 1] |= (uint8_t)(c << 4); /* A3 */
                else codes[i >> 1] |= (uint8_t)c;
            } else {
                codes[i] = (uint8_t)c;
            }
        }
    }
    return 0;
}

/*
 * Dequantise: out[i] = table[code_i] * absmax[block(i)], one f32 rounding
 * (QuantizedTensor::to_tensor, kv_cache.rs:871-957).  The caller narrows to bf16/fp16.
 */
int hsq_dequantize_blockwise(int kind, const uint8_t *codes, int64_t n, int blocksize, int scale_f16,
                             const float *absmax_f32, const uint16_t *absmax_f16, float *out) {
    float table[256];
    int ncode = hsq_codebook(kind, table);
    if (ncode == 0 || blocksize <= 0 || n < 0) return -1;
    int four_bit = (ncode == 16);
    for (int64_t i = 0; i < n; ++i) {
        int64_t b = i / blocksize;
        float a = scale_f16 ? hsq_f16_to_f32(absmax_f16[b]) : absmax_f32[b];
        int c = four_bit ? (((i & 1) == 0) ? (codes[i >> 1] >> 4) : (codes[i >> 1] & 0xf)) : codes[i];
        volatile float v = table[c] * a;
        out[i] = v;
    }
    return 0;
}
