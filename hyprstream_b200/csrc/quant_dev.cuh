// Device-side pieces of the blockwise quantiser and of the bf16 rotary embedding, shared by the quantiser / cache-write
// kernels (quant.cu) and by the decode kernel that writes a step's new token itself (decode_tc.cu).  One definition, so
// that every writer produces the same codes and scales bit for bit.
#pragma once
#include <cuda_bf16.h>

#include "hs_common.cuh"

namespace hs {

__device__ __forceinline__ float code8(int i) { return __fdiv_rn(static_cast<float>(i) - 127.0f, 127.0f); }
__device__ __forceinline__ float mid8(int j) { return __fmul_rn(0.5f, __fadd_rn(code8(j), code8(j + 1))); }

// Index of y in the 8-bit linear codebook.  The candidate round(y*127)+127 is exact unless y*127 sits
// within 1e-3 of a half-integer; only then are the true f32 midpoints consulted (smid: the 255 midpoints in shared
// memory, so the rare path costs two loads and not four divisions for every lane of the warp).
// (rounding by the magic-number add: t + 1.5 * 2^23 is round-to-nearest-even of t in the low mantissa bits for |t| < 2^22 -
// the same integer rintf gives - at full rate, where rintf and the float -> int conversion run on the quarter-rate pipe)
__device__ __forceinline__ int index_int8(float y, const float *smid) {
    float t = __fmul_rn(y, 127.0f);
    const float tm = __fadd_rn(t, 12582912.0f);
    const float r = __fadd_rn(tm, -12582912.0f);
    int c = max(0, min(255, __float_as_int(tm) - 0x4B400000 + 127));
    if (fabsf(t - r) > 0.499f) {  // within 1e-3 of a half-integer
        if (c > 0 && !(y > smid[c - 1])) c--;
        else if (c < 255 && y > smid[c]) c++;
    }
    return c;
}

// The same index with the midpoints worked out on the spot (two IEEE divisions, on the rare tie path only): for a caller
// that has no table in shared memory.  mid8 is the function the table is filled from, so the results are identical.
__device__ __forceinline__ int index_int8_direct(float y) {
    float t = __fmul_rn(y, 127.0f);
    const float tm = __fadd_rn(t, 12582912.0f);
    const float r = __fadd_rn(tm, -12582912.0f);
    int c = max(0, min(255, __float_as_int(tm) - 0x4B400000 + 127));
    if (fabsf(t - r) > 0.499f) {
        if (c > 0 && !(y > mid8(c - 1))) c--;
        else if (c < 255 && y > mid8(c)) c++;
    }
    return c;
}

// Index of y in a 16-entry ascending codebook whose 15 midpoints are in shared memory.
__device__ __forceinline__ int index_4bit(float y, const float *smid) {
    int c = 0;
#pragma unroll
    for (int j = 0; j < 15; ++j) c += (y > smid[j]) ? 1 : 0;
    return c;
}

// smid: 256 floats; the block has at least 255 threads
__device__ __forceinline__ void fill_midpoints(int kind, float *smid) {
    if (kind == HS_KV_INT8) {
        if (threadIdx.x < 255) smid[threadIdx.x] = mid8(threadIdx.x);
    } else if (threadIdx.x < 15) {
        const float *t = kind == HS_KV_NF4 ? c_nf4 : c_fp4;
        smid[threadIdx.x] = __fmul_rn(0.5f, __fadd_rn(t[threadIdx.x], t[threadIdx.x + 1]));
    }
}

__device__ __forceinline__ float f16_sat_round(float a) {
    // nearest-even to f16, saturating: anything that would round past 65504 stays 65504
    return a >= 65520.0f ? 65504.0f : __half2float(__float2half_rn(a));
}

// Quantise the 8 values of this thread; `tpb` consecutive lanes (a power of two <= 32) share a block.
// Returns the stored scale (already rounded in f16 mode); codes[] receives 8 indices.
template <int KIND, int N>
__device__ __forceinline__ float quantize_n(const float (&x)[N], int tpb, int scale_dtype, const float *smid,
                                            int (&codes)[N]) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < N; ++i) amax = fmaxf(amax, fabsf(x[i]));
    for (int o = 1; o < tpb; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    float a = scale_dtype == HS_SCALE_F16 ? f16_sat_round(amax) : amax;
    if (a == 0.0f) {
        const int zc = KIND == HS_KV_INT8 ? 127 : (KIND == HS_KV_NF4 ? 7 : 0);
#pragma unroll
        for (int i = 0; i < N; ++i) codes[i] = zc;
        return a;
    }
    float inv = __fdiv_rn(1.0f, a);
#pragma unroll
    for (int i = 0; i < N; ++i) {
        float y = __fmul_rn(x[i], inv);
        codes[i] = KIND == HS_KV_INT8 ? (smid != nullptr ? index_int8(y, smid) : index_int8_direct(y)) : index_4bit(y, smid);
    }
    return a;
}
template <int KIND>
__device__ __forceinline__ float quantize8(const float (&x)[8], int tpb, int scale_dtype, const float *smid, int (&codes)[8]) {
    return quantize_n<KIND, 8>(x, tpb, scale_dtype, smid, codes);
}

__device__ __forceinline__ void store_scale(void *p, int64_t idx, int scale_dtype, float a) {
    if (scale_dtype == HS_SCALE_F16) reinterpret_cast<__half *>(p)[idx] = __float2half_rn(a);
    else reinterpret_cast<float *>(p)[idx] = a;
}

__device__ __forceinline__ float load_elem(const void *src, int dtype, int64_t i) {
    if (dtype == HS_DTYPE_BF16) return bf16_bits_to_f32(reinterpret_cast<const uint16_t *>(src)[i]);
    if (dtype == HS_DTYPE_F16) return __half2float(reinterpret_cast<const __half *>(src)[i]);
    return reinterpret_cast<const float *>(src)[i];
}

__device__ __forceinline__ void unpack8_bf16(const uint4 &w, float (&x)[8]) {
    x[0] = bf16lo(w.x); x[1] = bf16hi(w.x); x[2] = bf16lo(w.y); x[3] = bf16hi(w.y);
    x[4] = bf16lo(w.z); x[5] = bf16hi(w.z); x[6] = bf16lo(w.w); x[7] = bf16hi(w.w);
}

template <int KIND>
__device__ __forceinline__ void store_codes8(uint8_t *codes, int64_t e0, int64_t n, const int (&c)[8], bool full) {
    if (KIND == HS_KV_INT8) {
        if (full) {
            uint2 w;
            w.x = c[0] | (c[1] << 8) | (c[2] << 16) | (c[3] << 24);
            w.y = c[4] | (c[5] << 8) | (c[6] << 16) | (c[7] << 24);
            *reinterpret_cast<uint2 *>(codes + e0) = w;
        } else {
            for (int i = 0; i < 8 && e0 + i < n; ++i) codes[e0 + i] = static_cast<uint8_t>(c[i]);
        }
    } else {
        if (full) {
            uint32_t w = ((c[0] << 4) | c[1]) | (((c[2] << 4) | c[3]) << 8) | (((c[4] << 4) | c[5]) << 16) |
                         (((c[6] << 4) | c[7]) << 24);
            *reinterpret_cast<uint32_t *>(codes + (e0 >> 1)) = w;
        } else {
            for (int i = 0; i < 8 && e0 + i < n; i += 2) {
                int lo = (e0 + i + 1 < n) ? c[i + 1] : 0;
                codes[(e0 + i) >> 1] = static_cast<uint8_t>((c[i] << 4) | lo);
            }
        }
    }
}

// ---- RoPE ------------------------------------------------------------------------------------------
// Rotated value of element d of a row, given the row's unrotated elements `own` (at d) and `partner`
// (at d +- rotary_dim/2).  Every product, difference and sum is rounded to bf16 (rope.rs:243-244).
__device__ __forceinline__ float rope_elem(float own, float partner, float s, float c, bool first_half) {
    if (first_half) return bf16_round(bf16_round(own * c) - bf16_round(partner * s));  // x1*cos - x2*sin
    return bf16_round(bf16_round(partner * s) + bf16_round(own * c));                 // x1*sin + x2*cos
}

// Loads the 8 bf16 elements [d0, d0+8) of a row, rotated when sin != NULL.  The rotation runs on packed bf16 pairs: a product
// of two bf16 values is exact in fp32, so mul.rn.bf16x2 rounds it once exactly as "multiply in fp32, round to bf16" does, and
// the difference / sum of two bf16 values rounds to the same bf16 either way - three instructions per pair instead of the
// unpack, three roundings and two multiplies per element of rope_elem (which stays for callers that hold fp32 values).
__device__ __forceinline__ void load_row8_rope(const uint16_t *row, int d0, const uint16_t *sin, const uint16_t *cos,
                                               int pos, int rotary_dim, float (&x)[8]) {
    uint4 ow = *reinterpret_cast<const uint4 *>(row + d0);
    if (sin != nullptr && d0 < rotary_dim) {
        const int half = rotary_dim >> 1;
        const bool first = d0 < half;
        const uint4 pw = *reinterpret_cast<const uint4 *>(row + (first ? d0 + half : d0 - half));
        const int j0 = first ? d0 : d0 - half;
        const uint16_t *srow = sin + static_cast<int64_t>(pos) * half + j0;
        const uint16_t *crow = cos + static_cast<int64_t>(pos) * half + j0;
        uint32_t sw[4], cw[4];
        if (((reinterpret_cast<uintptr_t>(srow) | reinterpret_cast<uintptr_t>(crow)) & 15u) == 0) {
            const uint4 s4 = *reinterpret_cast<const uint4 *>(srow), c4 = *reinterpret_cast<const uint4 *>(crow);
            sw[0] = s4.x; sw[1] = s4.y; sw[2] = s4.z; sw[3] = s4.w;
            cw[0] = c4.x; cw[1] = c4.y; cw[2] = c4.z; cw[3] = c4.w;
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                sw[i] = static_cast<uint32_t>(srow[2 * i]) | (static_cast<uint32_t>(srow[2 * i + 1]) << 16);
                cw[i] = static_cast<uint32_t>(crow[2 * i]) | (static_cast<uint32_t>(crow[2 * i + 1]) << 16);
            }
        }
        uint32_t o[4] = {ow.x, ow.y, ow.z, ow.w};
        const uint32_t pp[4] = {pw.x, pw.y, pw.z, pw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __nv_bfloat162 own = *reinterpret_cast<const __nv_bfloat162 *>(&o[i]), par = *reinterpret_cast<const __nv_bfloat162 *>(&pp[i]);
            const __nv_bfloat162 s2 = *reinterpret_cast<const __nv_bfloat162 *>(&sw[i]), c2 = *reinterpret_cast<const __nv_bfloat162 *>(&cw[i]);
            const __nv_bfloat162 oc = __hmul2(own, c2), ps = __hmul2(par, s2);
            const __nv_bfloat162 r = first ? __hsub2(oc, ps) : __hadd2(ps, oc);  // x1*cos - x2*sin | x1*sin + x2*cos
            o[i] = *reinterpret_cast<const uint32_t *>(&r);
        }
        ow = make_uint4(o[0], o[1], o[2], o[3]);
    }
    unpack8_bf16(ow, x);
}

}  // namespace hs
