// Per-head RMS norm of q or k fused with the (partial) rotary embedding and, for Qwen3.5's doubled q projection, the
// split of the output gate: the steps between the q/k/v projections and the cache / attention call in
// Qwen3_5FullAttention::forward (architectures/qwen3_5.rs:963-990, apply_qknorm :1077-1091) and, with the plain weight,
// LlamaAttention's optional QK-norm (architectures/llama.rs:929-992 before rope at :598-602).
//
//   n   = bf16( x * rsqrt(mean(x^2) + eps) * (w or 1 + w) )          fp32 inside, one rounding to the model dtype
//   out = rope(n) on the first rotary_dim dims (half-split; every product, difference and sum rounded to bf16,
//         runtime/rope.rs:206-248), the remaining dims passed through
//   gate_out = x[head_dim : 2 head_dim] copied out of the strided projection output (qwen3_5.rs:965-967)
//
// One pass over HBM: head_dim/8 lanes hold one (token, head) row, 8 elements each; the row's sum of squares and the
// rotation partners travel by shuffles.  Input rows may be strided (the query half of a [.., 2 head_dim] projection);
// outputs are dense [n_tokens, n_heads, head_dim].
#include <cuda_bf16.h>

#include "hs_common.cuh"

namespace hs {

constexpr int kNormThreads = 256;


// LPR: lanes per row = head_dim / 8
template <int LPR>
__global__ void __launch_bounds__(kNormThreads)
qk_norm_rope_kernel(const uint16_t *__restrict__ x, int64_t token_stride, int64_t head_stride, uint16_t *__restrict__ out,
                    uint16_t *__restrict__ gate_out, const float *__restrict__ weight, float eps, int plus_one,
                    const uint16_t *__restrict__ sin, const uint16_t *__restrict__ cos, const int32_t *__restrict__ positions,
                    int n_positions, int rotary_dim, int64_t n_tokens, int n_heads, int *__restrict__ err) {
    constexpr int D = LPR * 8;
    const int64_t row = (static_cast<int64_t>(blockIdx.x) * kNormThreads + threadIdx.x) / LPR;  // (token, head)
    const int l = threadIdx.x % LPR, d0 = l * 8;
    const bool live = row < n_tokens * n_heads;  // dead lanes still take part in the shuffles
    int64_t tok = 0;
    int h = 0;
    if (live) {
        if (row <= 0x7fffffffLL) {  // (a 64-bit division is several dozen instructions)
            const unsigned r32 = static_cast<unsigned>(row), t32 = r32 / static_cast<unsigned>(n_heads);
            tok = t32;
            h = static_cast<int>(r32 - t32 * static_cast<unsigned>(n_heads));
        } else {
            tok = row / n_heads;
            h = static_cast<int>(row % n_heads);
        }
    }
    const uint16_t *src = x + tok * token_stride + h * head_stride;
    const uint4 w4 = live ? *reinterpret_cast<const uint4 *>(src + d0) : make_uint4(0u, 0u, 0u, 0u);
    if (gate_out != nullptr && live)
        *reinterpret_cast<uint4 *>(gate_out + row * D + d0) = *reinterpret_cast<const uint4 *>(src + D + d0);
    // n: the normed row as bf16 pairs (one packed conversion per pair = the one rounding to the model dtype)
    uint32_t n[4] = {w4.x, w4.y, w4.z, w4.w};
    if (weight != nullptr) {
        const float v[8] = {bf16lo(w4.x), bf16hi(w4.x), bf16lo(w4.y), bf16hi(w4.y), bf16lo(w4.z), bf16hi(w4.z), bf16lo(w4.w), bf16hi(w4.w)};
        float ss = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) ss = fmaf(v[i], v[i], ss);
#pragma unroll
        for (int off = 1; off < LPR; off <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
        const float rrms = rsqrtf(ss * (1.0f / D) + eps);
        const float4 w0 = *reinterpret_cast<const float4 *>(weight + d0), w1 = *reinterpret_cast<const float4 *>(weight + d0 + 4);
        const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
        const float add = plus_one ? 1.0f : 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) n[i] = pack_bf16(v[2 * i] * rrms * (wv[2 * i] + add), v[2 * i + 1] * rrms * (wv[2 * i + 1] + add));
    }
    if (sin != nullptr) {
        const int half = rotary_dim >> 1;
        const int pos = live ? positions[tok] : 0;
        const bool in_table = pos >= 0 && pos < n_positions;
        if (live && !in_table && l == 0) atomicOr(err, HS_DEVERR_ROPE_RANGE);  // recorded; the row is left unrotated
        const bool rot = d0 < rotary_dim, first = d0 < half;
        // the partner chunk (d0 +- half) sits half/8 lanes away in the same row
        const int partner_lane = (threadIdx.x & 31) + (first ? half / 8 : -(half / 8));
        uint32_t p[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) p[i] = __shfl_sync(0xffffffffu, n[i], rot ? partner_lane : (threadIdx.x & 31));
        if (rot && in_table && live) {
            // In packed bf16 arithmetic: the product of two bf16 values is exact in fp32, so mul.rn.bf16x2 rounds it once exactly as
            // "multiply in fp32, round to bf16" does, and the difference / sum of two bf16 values rounds to the same bf16 either way
            // (runtime/rope.rs:206-248 rounds every product, difference and sum to bf16).
            const int j0 = first ? d0 : d0 - half;
            const uint4 s4 = *reinterpret_cast<const uint4 *>(sin + static_cast<int64_t>(pos) * half + j0);
            const uint4 c4 = *reinterpret_cast<const uint4 *>(cos + static_cast<int64_t>(pos) * half + j0);
            const uint32_t sw[4] = {s4.x, s4.y, s4.z, s4.w}, cw[4] = {c4.x, c4.y, c4.z, c4.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const __nv_bfloat162 own = *reinterpret_cast<const __nv_bfloat162 *>(&n[i]), par = *reinterpret_cast<const __nv_bfloat162 *>(&p[i]);
                const __nv_bfloat162 s2 = *reinterpret_cast<const __nv_bfloat162 *>(&sw[i]), c2 = *reinterpret_cast<const __nv_bfloat162 *>(&cw[i]);
                const __nv_bfloat162 oc = __hmul2(own, c2), ps = __hmul2(par, s2);
                const __nv_bfloat162 r = first ? __hsub2(oc, ps) : __hadd2(ps, oc);  // x1*cos - x2*sin | x1*sin + x2*cos
                n[i] = *reinterpret_cast<const uint32_t *>(&r);
            }
        }
    }
    if (live) *reinterpret_cast<uint4 *>(out + row * D + d0) = make_uint4(n[0], n[1], n[2], n[3]);
}

}  // namespace hs

using namespace hs;

extern "C" {

int32_t hs_qk_norm_rope(const void *x, int64_t token_stride, int64_t head_stride, void *out, void *gate_out,
                        const float *norm_weight, float eps, int32_t weight_plus_one, const void *sin, const void *cos,
                        const int32_t *positions, int32_t n_positions, int32_t rotary_dim, int64_t n_tokens, int32_t n_heads,
                        int32_t head_dim, hs_stream_t stream) {
    if (int32_t st = check_device()) return st;
    if (n_tokens < 0 || n_heads <= 0) return fail(HS_ERR_ARG, "hs_qk_norm_rope: bad sizes");
    if (head_dim != 64 && head_dim != 128 && head_dim != 256) return fail(HS_ERR_UNSUPPORTED, "hs_qk_norm_rope: head_dim %d (supported: 64, 128, 256)", head_dim);
    if (n_tokens == 0) return HS_OK;
    if (!x || !out) return fail(HS_ERR_ARG, "hs_qk_norm_rope: NULL pointer");
    if (x == out || x == gate_out) return fail(HS_ERR_ARG, "hs_qk_norm_rope: out of place only");
    if (token_stride < static_cast<int64_t>(n_heads - 1) * head_stride + head_dim * (gate_out ? 2 : 1))
        return fail(HS_ERR_ARG, "hs_qk_norm_rope: rows overlap (token_stride %lld, head_stride %lld)", (long long)token_stride, (long long)head_stride);
    if (head_stride < head_dim * (gate_out ? 2 : 1)) return fail(HS_ERR_ARG, "hs_qk_norm_rope: head_stride %lld too small", (long long)head_stride);
    if (token_stride % 8 != 0 || head_stride % 8 != 0 || !aligned(x, 16) || !aligned(out, 16) || (gate_out && !aligned(gate_out, 16)) ||
        (norm_weight && !aligned(norm_weight, 16)))
        return fail(HS_ERR_ARG, "hs_qk_norm_rope: pointers must be 16-byte aligned and strides multiples of 8 elements");
    if (sin != nullptr) {
        if (!cos || !positions) return fail(HS_ERR_ARG, "hs_qk_norm_rope: sin given without cos / positions");
        if (rotary_dim <= 0 || rotary_dim % 16 != 0 || rotary_dim > head_dim || n_positions <= 0)
            return fail(HS_ERR_UNSUPPORTED, "hs_qk_norm_rope: rotary_dim must be a positive multiple of 16 <= head_dim");
        if (!aligned(sin, 16) || !aligned(cos, 16)) return fail(HS_ERR_ARG, "hs_qk_norm_rope: sin / cos tables must be 16-byte aligned");
    }
    int *err = device_error_word();
    if (!err) return fail(HS_ERR_DEVICE, "hs_qk_norm_rope: device error word unavailable");
    const int lpr = head_dim / 8;
    const int64_t threads = n_tokens * n_heads * lpr;
    const int64_t blocks = (threads + kNormThreads - 1) / kNormThreads;
    if (blocks > 0x7fffffffLL) return fail(HS_ERR_ARG, "hs_qk_norm_rope: too many rows");
    cudaStream_t s = as_stream(stream);
#define HS_QKN(L)                                                                                                                   \
    qk_norm_rope_kernel<L><<<static_cast<unsigned>(blocks), kNormThreads, 0, s>>>(                                                  \
        reinterpret_cast<const uint16_t *>(x), token_stride, head_stride, reinterpret_cast<uint16_t *>(out),                        \
        reinterpret_cast<uint16_t *>(gate_out), norm_weight, eps, weight_plus_one, reinterpret_cast<const uint16_t *>(sin),         \
        reinterpret_cast<const uint16_t *>(cos), positions, n_positions, rotary_dim, n_tokens, n_heads, err)
    prof_begin(s);
    if (lpr == 32) HS_QKN(32); else if (lpr == 16) HS_QKN(16); else HS_QKN(8);
    prof_end(s);
#undef HS_QKN
    return check_launch("hs_qk_norm_rope");
}

}  // extern "C"
