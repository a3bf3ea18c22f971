// Blockwise KV quantiser for sm_100a: flat quantise / dequantise, RoPE, quantise-on-write into a
// (paged) cache view, and the gather-dequantise compatibility read.
//
// Arithmetic contract (bit-exact with the CPU specification used by the parity tests):
//   absmax = max|x| over the block in f32; in f16-scale mode it is rounded to f16 (nearest even,
//   saturating at 65504) before use;  y = x * (1/absmax), one IEEE rounding each;
//   index = number of f32 codeword midpoints 0.5*(c[j]+c[j+1]) strictly below y;
//   an all-zero block stores absmax 0 and the index of the codeword 0;
//   4-bit codes pack the even element into the high nibble.
// Codebooks and block geometry follow bitsandbytes-sys/src/lib.rs:104-181 and
// crates/hyprstream/src/runtime/kv_cache.rs:704,741-957.
//
// All kernels here are HBM-streaming: one thread owns 8 consecutive elements (one 16-byte bf16
// load, one 8-byte int8 store), a block's absmax is reduced with warp shuffles, nothing is staged.
#include "hs_common.cuh"
#include "quant_dev.cuh"

namespace hs {

constexpr int kQThreads = 256;
#ifndef HS_KV_WRITE_WIDE
#define HS_KV_WRITE_WIDE 16
#endif
constexpr int kWriteElems = 64;  // elements per thread of the quantise-on-write kernel (as 8- or 16-element chunks)

// ---- flat quantise ----------------------------------------------------------------------------
template <int KIND>
__global__ void __launch_bounds__(kQThreads) quantize_flat_kernel(const void *__restrict__ src, int dtype, int64_t n,
                                                                  int block, int scale_dtype, uint8_t *__restrict__ codes,
                                                                  void *__restrict__ absmax, int vec_ok) {
    __shared__ float smid[256];
    fill_midpoints(KIND, smid);
    __syncthreads();
    const int64_t chunk = static_cast<int64_t>(blockIdx.x) * kQThreads + threadIdx.x;
    const int64_t e0 = chunk * 8;
    float x[8];
    const bool full = e0 + 8 <= n;
    if (full && vec_ok && dtype == HS_DTYPE_BF16) {
        unpack8_bf16(*reinterpret_cast<const uint4 *>(reinterpret_cast<const uint16_t *>(src) + e0), x);
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = (e0 + i < n) ? load_elem(src, dtype, e0 + i) : 0.0f;
    }
    int c[8];
    const int tpb = block / 8;
    float a = quantize8<KIND>(x, tpb, scale_dtype, smid, c);
    if (e0 < n) {
        if ((chunk % tpb) == 0) store_scale(absmax, e0 / block, scale_dtype, a);
        store_codes8<KIND>(codes, e0, n, c, full);
    }
}

// ---- flat dequantise ----------------------------------------------------------------------------
__device__ __forceinline__ float table_value(int kind, int c, const float *stab) {
    return kind == HS_KV_INT8 ? code8(c) : stab[c];
}

__device__ __forceinline__ void store_elem(void *out, int dtype, int64_t i, float v) {
    if (dtype == HS_DTYPE_BF16) reinterpret_cast<uint16_t *>(out)[i] = f32_to_bf16_bits(v);
    else if (dtype == HS_DTYPE_F16) reinterpret_cast<__half *>(out)[i] = __float2half_rn(v);
    else reinterpret_cast<float *>(out)[i] = v;
}

__global__ void __launch_bounds__(kQThreads) dequantize_flat_kernel(int kind, const uint8_t *__restrict__ codes,
                                                                    const void *__restrict__ absmax, int64_t n, int block,
                                                                    int scale_dtype, void *__restrict__ out, int dtype) {
    __shared__ float stab[16];
    if (kind != HS_KV_INT8 && threadIdx.x < 16) stab[threadIdx.x] = kind == HS_KV_NF4 ? c_nf4[threadIdx.x] : c_fp4[threadIdx.x];
    __syncthreads();
    const int64_t e0 = (static_cast<int64_t>(blockIdx.x) * kQThreads + threadIdx.x) * 8;
    if (e0 >= n) return;
    const float a = load_scale(absmax, e0 / block, scale_dtype);
    for (int i = 0; i < 8 && e0 + i < n; ++i) {
        int64_t e = e0 + i;
        int c = kind == HS_KV_INT8 ? codes[e] : ((e & 1) ? (codes[e >> 1] & 0xf) : (codes[e >> 1] >> 4));
        store_elem(out, dtype, e, __fmul_rn(table_value(kind, c, stab), a));
    }
}

// ---- RoPE (device helpers in quant_dev.cuh) ------------------------------------------------------------
__global__ void __launch_bounds__(kQThreads) rope_kernel(const uint16_t *__restrict__ x, uint16_t *__restrict__ out,
                                                         const uint16_t *__restrict__ sin, const uint16_t *__restrict__ cos,
                                                         const int32_t *__restrict__ positions, int64_t n_rows, int n_heads,
                                                         int head_dim, int rotary_dim, int n_positions, int *__restrict__ err) {
    const int cpr = head_dim / 8;  // chunks per (row, head)
    const int64_t chunk = static_cast<int64_t>(blockIdx.x) * kQThreads + threadIdx.x;
    const int64_t total = n_rows * n_heads * cpr;
    if (chunk >= total) return;
    const int d0 = static_cast<int>(chunk % cpr) * 8;
    const int64_t rh = chunk / cpr;
    const int64_t r = rh / n_heads;
    float v[8];
    const int pos = positions[r];
    const bool in_table = pos >= 0 && pos < n_positions;
    if (!in_table) atomicOr(err, HS_DEVERR_ROPE_RANGE);  // recorded; the row is copied unrotated
    load_row8_rope(x + rh * head_dim, d0, in_table ? sin : nullptr, cos, in_table ? pos : 0, rotary_dim, v);
    uint4 w;
    w.x = pack_bf16(v[0], v[1]); w.y = pack_bf16(v[2], v[3]); w.z = pack_bf16(v[4], v[5]); w.w = pack_bf16(v[6], v[7]);
    *reinterpret_cast<uint4 *>(out + rh * head_dim + d0) = w;
}

// Optional per-head RMS norm of K fused into quantise-on-write (weight == NULL: off).
struct KNormArgs {
    const float *weight;  // f32 [head_dim]
    float eps;
    int plus_one;         // multiply by (1 + w) instead of w
    uint16_t *k_out;      // optional bf16 [n_seqs, n_tokens, n_kv_heads, head_dim]: the normed, rotated keys
    int pos_bias;         // added to dst_pos[s]: -1 when the caller hands the attended lengths instead of positions
};

// ---- quantise-on-write into a cache view ----------------------------------------------------------------
// E = elements per thread: 16 for long writes (prefill: bound by instruction issue, so the per-chunk costs are paid
// half as often), 8 for short ones (a decode step's single token per sequence: latency matters, not throughput).
template <int KIND, int E>
__global__ void __launch_bounds__(kQThreads) kv_write_kernel(ViewDev view, const uint16_t *__restrict__ k_new,
                                                             const uint16_t *__restrict__ v_new, int n_seqs, int n_tokens,
                                                             const int32_t *__restrict__ dst_pos,
                                                             const uint16_t *__restrict__ sin, const uint16_t *__restrict__ cos,
                                                             int rotary_dim, int n_positions, int *__restrict__ err, KNormArgs kn) {
    // a decode launch that follows as a programmatic dependent may start now (it waits for this grid's completion before
    // it reads the cache); a no-op for every other successor
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    __shared__ float smid[256];
    fill_midpoints(KIND, smid);
    __syncthreads();
    // grid: x = groups of kUnroll * 256 E-element chunks of one sequence's new rows, y = 2 * sequence + (0: K, 1: V).
    // A thread owns E consecutive elements of a (token, head) row (16-byte loads; at E = 16 one 16-byte store of int8
    // codes): the index split, the page division, the pointer loads, the IEEE division of the scale and the shuffles
    // are paid once per chunk.  head_dim and the block are powers of two (64, 128, 256), the number of kv heads usually
    // is: shifts instead of divisions.
    const bool is_v = (blockIdx.y & 1) != 0;
    const int s = static_cast<int>(blockIdx.y >> 1);
    const int D = view.head_dim, H = view.n_kv_heads;
    constexpr int kUnroll = kWriteElems / E;
    const uint32_t cpr = static_cast<uint32_t>(D) / static_cast<uint32_t>(E);
    const uint32_t total = static_cast<uint32_t>(n_tokens) * static_cast<uint32_t>(H) * cpr;
    const int base_pos = dst_pos ? dst_pos[s] + kn.pos_bias : 0;
    void *const *data_pages = is_v ? view.v_pages : view.k_pages;
    void *const *scale_pages = is_v ? view.v_scale_pages : view.k_scale_pages;
    const int tpb = view.block / E;
    const int bpr = D / view.block;  // blocks per (token, head) row
    const int cpr_shift = __ffs(static_cast<int>(cpr)) - 1, block_shift = __ffs(view.block) - 1;
    const bool h_pow2 = (H & (H - 1)) == 0;
    const int h_shift = __ffs(H) - 1;
#pragma unroll 2
    for (int u = 0; u < kUnroll; ++u) {
        const uint32_t chunk = (blockIdx.x * static_cast<uint32_t>(kUnroll) + u) * static_cast<uint32_t>(kQThreads) + threadIdx.x;
        if (chunk - threadIdx.x >= total) break;  // (uniform over the block)
        const bool live = chunk < total;
        const uint32_t cc = live ? chunk : 0u;  // dead lanes still take part in the shuffles
        const uint32_t row_in_seq = cc >> cpr_shift;   // (token, head)
        const int d0 = static_cast<int>(cc & (cpr - 1u)) * E;
        const int t = static_cast<int>(h_pow2 ? row_in_seq >> h_shift : row_in_seq / static_cast<uint32_t>(H));
        const int h = static_cast<int>(row_in_seq - static_cast<uint32_t>(t) * static_cast<uint32_t>(H));
        const int64_t row = static_cast<int64_t>(s) * n_tokens * H + row_in_seq;  // (seq, token, head)
        const int pos = base_pos + t;
        const int page = pos / view.page_tokens;
        bool ok = live && pos >= 0 && page < view.pages_per_seq;
        if (!is_v && sin != nullptr && (pos < 0 || pos >= n_positions)) ok = false;
        if (live && !ok) atomicOr(err, HS_DEVERR_KV_WRITE_RANGE);  // recorded, access skipped
        const uint16_t *src = (is_v ? v_new : k_new) + row * D;
        float x[E];
        if (kn.weight != nullptr && !is_v) {
            // ---- K with its per-head RMS norm fused in (qwen3_5.rs:1077-1091; llama.rs:929-992): the row's sum of squares is
            // formed exactly as hs_qk_norm_rope forms it (an 8-element chain per 16-byte chunk, then pairwise over the chunks
            // of the row), so the normed, rotated values - and with them the stored codes - equal the two-kernel route bit
            // for bit.  Dead and refused lanes carry zeros and still take part in the shuffles.
            float ssq[E / 8];
#pragma unroll
            for (int part = 0; part < E / 8; ++part) {
                float p8[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                if (ok) unpack8_bf16(*reinterpret_cast<const uint4 *>(src + d0 + 8 * part), p8);
                float ss = 0.0f;
#pragma unroll
                for (int i = 0; i < 8; ++i) { x[8 * part + i] = p8[i]; ss = fmaf(p8[i], p8[i], ss); }
                ssq[part] = ss;
            }
            float ss = ssq[0];
            if constexpr (E == 16) ss += ssq[1];
            for (uint32_t off = 1; off < cpr; off <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
            const float rrms = rsqrtf(ss * (1.0f / static_cast<float>(D)) + kn.eps);
            const float add = kn.plus_one ? 1.0f : 0.0f;
            const bool rope = sin != nullptr && ok;
            const int half = rotary_dim >> 1;
#pragma unroll
            for (int part = 0; part < E / 8; ++part) {
                const int dd = d0 + 8 * part;
                // the normed chunk as bf16 pairs (one packed conversion per pair = the one rounding to the model dtype), rotated in
                // packed bf16 arithmetic like load_row8_rope: the same values as the scalar form, bit for bit
                uint32_t ow[4];
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    ow[i] = pack_bf16(x[8 * part + 2 * i] * rrms * (kn.weight[dd + 2 * i] + add), x[8 * part + 2 * i + 1] * rrms * (kn.weight[dd + 2 * i + 1] + add));
                if (rope && dd < rotary_dim) {
                    const bool first = dd < half;
                    const int pd = first ? dd + half : dd - half;  // the rotation partner's chunk, normed the same way
                    float p8[8];
                    unpack8_bf16(*reinterpret_cast<const uint4 *>(src + pd), p8);
                    const int j0 = first ? dd : dd - half;
                    const uint16_t *srow = sin + static_cast<int64_t>(pos) * half + j0;
                    const uint16_t *crow = cos + static_cast<int64_t>(pos) * half + j0;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint32_t pw = pack_bf16(p8[2 * i] * rrms * (kn.weight[pd + 2 * i] + add), p8[2 * i + 1] * rrms * (kn.weight[pd + 2 * i + 1] + add));
                        const uint32_t sw = static_cast<uint32_t>(srow[2 * i]) | (static_cast<uint32_t>(srow[2 * i + 1]) << 16);
                        const uint32_t cw = static_cast<uint32_t>(crow[2 * i]) | (static_cast<uint32_t>(crow[2 * i + 1]) << 16);
                        const __nv_bfloat162 own = *reinterpret_cast<const __nv_bfloat162 *>(&ow[i]), par = *reinterpret_cast<const __nv_bfloat162 *>(&pw);
                        const __nv_bfloat162 s2 = *reinterpret_cast<const __nv_bfloat162 *>(&sw), c2 = *reinterpret_cast<const __nv_bfloat162 *>(&cw);
                        const __nv_bfloat162 oc = __hmul2(own, c2), ps = __hmul2(par, s2);
                        const __nv_bfloat162 r = first ? __hsub2(oc, ps) : __hadd2(ps, oc);  // x1*cos - x2*sin | x1*sin + x2*cos
                        ow[i] = *reinterpret_cast<const uint32_t *>(&r);
                    }
                }
                if (kn.k_out != nullptr && ok)  // the normed, rotated keys in bf16, for a prompt's own attention
                    *reinterpret_cast<uint4 *>(kn.k_out + row * D + dd) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
#pragma unroll
                for (int i = 0; i < 4; ++i) { x[8 * part + 2 * i] = bf16lo(ow[i]); x[8 * part + 2 * i + 1] = bf16hi(ow[i]); }
            }
        } else {
#pragma unroll
            for (int part = 0; part < E / 8; ++part) {
                float p8[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                if (ok) load_row8_rope(src, d0 + 8 * part, is_v ? nullptr : sin, cos, pos, rotary_dim, p8);
#pragma unroll
                for (int i = 0; i < 8; ++i) x[8 * part + i] = p8[i];
            }
        }
        const int64_t in_page = static_cast<int64_t>(pos - page * view.page_tokens) * H + h;  // (token, head) row inside the page
        const int64_t pidx = static_cast<int64_t>(s) * view.pages_per_seq + page;
        if (KIND == HS_KV_BF16) {
            if (ok) {
                uint16_t *dst = reinterpret_cast<uint16_t *>(data_pages[pidx]) + in_page * D + d0;
#pragma unroll
                for (int part = 0; part < E / 8; ++part) {
                    uint4 w;
                    w.x = pack_bf16(x[8 * part], x[8 * part + 1]); w.y = pack_bf16(x[8 * part + 2], x[8 * part + 3]);
                    w.z = pack_bf16(x[8 * part + 4], x[8 * part + 5]); w.w = pack_bf16(x[8 * part + 6], x[8 * part + 7]);
                    reinterpret_cast<uint4 *>(dst)[part] = w;
                }
            }
            continue;
        }
        constexpr int QK = KIND == HS_KV_BF16 ? HS_KV_INT8 : KIND;
        int c[E];
        float a = quantize_n<QK, E>(x, tpb, view.scale_dtype, smid, c);
        if (!ok) continue;
        uint8_t *codes = reinterpret_cast<uint8_t *>(data_pages[pidx]);
        void *scales = scale_pages[pidx];
        if ((d0 & (view.block - 1)) == 0) store_scale(scales, in_page * bpr + (d0 >> block_shift), view.scale_dtype, a);
        const int64_t e0 = in_page * D + d0;
        if constexpr (E == 8) {
            store_codes8<QK>(codes, e0, e0 + 8, c, true);
        } else {
#pragma unroll
            for (int part = 0; part < E / 16; ++part) {
                const int *cp = c + 16 * part;
                if (QK == HS_KV_INT8) {
                    uint4 w;
                    w.x = cp[0] | (cp[1] << 8) | (cp[2] << 16) | (cp[3] << 24);
                    w.y = cp[4] | (cp[5] << 8) | (cp[6] << 16) | (cp[7] << 24);
                    w.z = cp[8] | (cp[9] << 8) | (cp[10] << 16) | (cp[11] << 24);
                    w.w = cp[12] | (cp[13] << 8) | (cp[14] << 16) | (cp[15] << 24);
                    reinterpret_cast<uint4 *>(codes + e0)[part] = w;
                } else {  // the even element in the high nibble
                    uint2 w;
                    w.x = ((cp[0] << 4) | cp[1]) | (((cp[2] << 4) | cp[3]) << 8) | (((cp[4] << 4) | cp[5]) << 16) | (((cp[6] << 4) | cp[7]) << 24);
                    w.y = ((cp[8] << 4) | cp[9]) | (((cp[10] << 4) | cp[11]) << 8) | (((cp[12] << 4) | cp[13]) << 16) | (((cp[14] << 4) | cp[15]) << 24);
                    reinterpret_cast<uint2 *>(codes + (e0 >> 1))[part] = w;
                }
            }
        }
    }
}

// ---- gather-dequantise (LayerKVCache::get compatibility read) ------------------------------------------------
__global__ void __launch_bounds__(kQThreads) kv_gather_kernel(ViewDev view, const int32_t *__restrict__ seq_lens, int n_seqs,
                                                              int out_tokens, uint16_t *__restrict__ k_out,
                                                              uint16_t *__restrict__ v_out) {
    __shared__ float stab[16];
    if (view.kind >= HS_KV_NF4 && threadIdx.x < 16) stab[threadIdx.x] = view.kind == HS_KV_NF4 ? c_nf4[threadIdx.x] : c_fp4[threadIdx.x];
    __syncthreads();
    const bool is_v = blockIdx.y == 1;
    const int D = view.head_dim, H = view.n_kv_heads;
    const int cpr = D / 8;
    const int64_t chunk = static_cast<int64_t>(blockIdx.x) * kQThreads + threadIdx.x;
    const int64_t total = static_cast<int64_t>(n_seqs) * out_tokens * H * cpr;
    if (chunk >= total) return;
    const int d0 = static_cast<int>(chunk % cpr) * 8;
    const int64_t row = chunk / cpr;
    const int h = static_cast<int>(row % H);
    const int64_t st = row / H;
    const int t = static_cast<int>(st % out_tokens);
    const int s = static_cast<int>(st / out_tokens);
    uint4 w = make_uint4(0, 0, 0, 0);
    const int page = t / view.page_tokens;
    if (t < seq_lens[s] && page < view.pages_per_seq) {
        const int64_t pidx = static_cast<int64_t>(s) * view.pages_per_seq + page;
        const int64_t in_page = static_cast<int64_t>(t - page * view.page_tokens) * H + h;
        const void *data = (is_v ? view.v_pages : view.k_pages)[pidx];
        if (view.kind == HS_KV_BF16) {
            w = *reinterpret_cast<const uint4 *>(reinterpret_cast<const uint16_t *>(data) + in_page * D + d0);
        } else {
            const void *scales = (is_v ? view.v_scale_pages : view.k_scale_pages)[pidx];
            const float a = load_scale(scales, in_page * (D / view.block) + d0 / view.block, view.scale_dtype);
            float v[8];
            const uint8_t *codes = reinterpret_cast<const uint8_t *>(data);
            if (view.kind == HS_KV_INT8) {
                uint2 cw = *reinterpret_cast<const uint2 *>(codes + in_page * D + d0);
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(code8(((i < 4 ? cw.x : cw.y) >> (8 * (i & 3))) & 0xff), a);
            } else {
                uint32_t cw = *reinterpret_cast<const uint32_t *>(codes + ((in_page * D + d0) >> 1));
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    int byte = (cw >> (8 * (i >> 1))) & 0xff;
                    v[i] = __fmul_rn(stab[(i & 1) ? (byte & 0xf) : (byte >> 4)], a);
                }
            }
            w.x = pack_bf16(v[0], v[1]); w.y = pack_bf16(v[2], v[3]); w.z = pack_bf16(v[4], v[5]); w.w = pack_bf16(v[6], v[7]);
        }
    }
    *reinterpret_cast<uint4 *>((is_v ? v_out : k_out) + row * D + d0) = w;
}

}  // namespace hs

using namespace hs;

extern "C" {

int32_t hs_quantize_blockwise(int32_t kind, const void *src, int32_t dtype, int64_t n, int32_t block, int32_t scale_dtype,
                              uint8_t *codes, void *absmax, hs_stream_t stream) {
    if (int32_t st = check_device()) return st;
    if (kind < HS_KV_INT8 || kind > HS_KV_FP4) return fail(HS_ERR_ARG, "hs_quantize_blockwise: unknown kind %d", kind);
    if (dtype < HS_DTYPE_BF16 || dtype > HS_DTYPE_F32) return fail(HS_ERR_ARG, "hs_quantize_blockwise: unknown dtype %d", dtype);
    if (block != 64 && block != 128 && block != 256) return fail(HS_ERR_UNSUPPORTED, "hs_quantize_blockwise: block %d (supported: 64, 128, 256)", block);
    if (scale_dtype != HS_SCALE_F32 && scale_dtype != HS_SCALE_F16) return fail(HS_ERR_ARG, "hs_quantize_blockwise: unknown scale dtype %d", scale_dtype);
    if (n < 0) return fail(HS_ERR_ARG, "hs_quantize_blockwise: negative n");
    if (n == 0) return HS_OK;
    if (!src || !codes || !absmax) return fail(HS_ERR_ARG, "hs_quantize_blockwise: NULL pointer");
    const size_t esz = dtype == HS_DTYPE_F32 ? 4 : 2;
    if (!aligned(src, esz) || !aligned(absmax, scale_dtype == HS_SCALE_F16 ? 2 : 4))
        return fail(HS_ERR_ARG, "hs_quantize_blockwise: misaligned pointer");
    if (!aligned(codes, kind == HS_KV_INT8 ? 8 : 4)) return fail(HS_ERR_ARG, "hs_quantize_blockwise: codes must be 8-byte aligned");
    const int vec_ok = aligned(src, 16) ? 1 : 0;
    const int64_t chunks = (n + 7) / 8;
    // whole quantisation blocks per CTA: kQThreads*8 elements is a multiple of every supported block
    const unsigned grid = static_cast<unsigned>((chunks + kQThreads - 1) / kQThreads);
    cudaStream_t s = as_stream(stream);
    if (kind == HS_KV_INT8) quantize_flat_kernel<HS_KV_INT8><<<grid, kQThreads, 0, s>>>(src, dtype, n, block, scale_dtype, codes, absmax, vec_ok);
    else if (kind == HS_KV_NF4) quantize_flat_kernel<HS_KV_NF4><<<grid, kQThreads, 0, s>>>(src, dtype, n, block, scale_dtype, codes, absmax, vec_ok);
    else quantize_flat_kernel<HS_KV_FP4><<<grid, kQThreads, 0, s>>>(src, dtype, n, block, scale_dtype, codes, absmax, vec_ok);
    return check_launch("hs_quantize_blockwise");
}

int32_t hs_dequantize_blockwise(int32_t kind, const uint8_t *codes, const void *absmax, int64_t n, int32_t block,
                                int32_t scale_dtype, void *out, int32_t dtype, hs_stream_t stream) {
    if (int32_t st = check_device()) return st;
    if (kind < HS_KV_INT8 || kind > HS_KV_FP4) return fail(HS_ERR_ARG, "hs_dequantize_blockwise: unknown kind %d", kind);
    if (dtype < HS_DTYPE_BF16 || dtype > HS_DTYPE_F32) return fail(HS_ERR_ARG, "hs_dequantize_blockwise: unknown dtype %d", dtype);
    if (block <= 0) return fail(HS_ERR_ARG, "hs_dequantize_blockwise: block must be positive");
    if (scale_dtype != HS_SCALE_F32 && scale_dtype != HS_SCALE_F16) return fail(HS_ERR_ARG, "hs_dequantize_blockwise: unknown scale dtype %d", scale_dtype);
    if (n < 0) return fail(HS_ERR_ARG, "hs_dequantize_blockwise: negative n");
    if (n == 0) return HS_OK;
    if (!codes || !absmax || !out) return fail(HS_ERR_ARG, "hs_dequantize_blockwise: NULL pointer");
    if (block % 8 != 0) return fail(HS_ERR_UNSUPPORTED, "hs_dequantize_blockwise: block must be a multiple of 8");
    if (!aligned(out, dtype == HS_DTYPE_F32 ? 4 : 2) || !aligned(absmax, scale_dtype == HS_SCALE_F16 ? 2 : 4))
        return fail(HS_ERR_ARG, "hs_dequantize_blockwise: misaligned pointer");
    const int64_t chunks = (n + 7) / 8;
    const unsigned grid = static_cast<unsigned>((chunks + kQThreads - 1) / kQThreads);
    dequantize_flat_kernel<<<grid, kQThreads, 0, as_stream(stream)>>>(kind, codes, absmax, n, block, scale_dtype, out, dtype);
    return check_launch("hs_dequantize_blockwise");
}

int32_t hs_rope_apply(const void *x, void *out, const void *sin, const void *cos, const int32_t *positions, int64_t n_rows,
                      int32_t n_heads, int32_t head_dim, int32_t rotary_dim, int32_t n_positions, hs_stream_t stream) {
    if (int32_t st = check_device()) return st;
    if (n_rows < 0 || n_heads <= 0 || head_dim <= 0 || n_positions <= 0) return fail(HS_ERR_ARG, "hs_rope_apply: bad sizes");
    if (head_dim % 8 != 0 || rotary_dim % 16 != 0 || rotary_dim < 0 || rotary_dim > head_dim)
        return fail(HS_ERR_UNSUPPORTED, "hs_rope_apply: head_dim %% 8 and rotary_dim %% 16 must be 0, rotary_dim <= head_dim");
    if (n_rows == 0) return HS_OK;
    if (!x || !out || !sin || !cos || !positions) return fail(HS_ERR_ARG, "hs_rope_apply: NULL pointer");
    if (!aligned(x, 16) || !aligned(out, 16) || !aligned(sin, 2) || !aligned(cos, 2) || !aligned(positions, 4))
        return fail(HS_ERR_ARG, "hs_rope_apply: x and out must be 16-byte aligned");
    if (x == out && rotary_dim > 0) return fail(HS_ERR_ARG, "hs_rope_apply: in-place rotation is not supported (a lane reads its partner half)");
    int *err = device_error_word();
    if (!err) return fail(HS_ERR_DEVICE, "hs_rope_apply: device error word unavailable");
    const int64_t chunks = n_rows * n_heads * (head_dim / 8);
    const unsigned grid = static_cast<unsigned>((chunks + kQThreads - 1) / kQThreads);
    rope_kernel<<<grid, kQThreads, 0, as_stream(stream)>>>(
        reinterpret_cast<const uint16_t *>(x), reinterpret_cast<uint16_t *>(out), reinterpret_cast<const uint16_t *>(sin),
        reinterpret_cast<const uint16_t *>(cos), positions, n_rows, n_heads, head_dim, rotary_dim, n_positions, err);
    return check_launch("hs_rope_apply");
}

static int32_t kv_write_impl(const char *who, const hs_kv_view *view, const void *k_new, const void *v_new, int32_t n_seqs, int32_t n_tokens,
                             const int32_t *dst_pos, const void *sin, const void *cos, int32_t rotary_dim, int32_t n_positions, hs::KNormArgs kn,
                             hs_stream_t stream) {
    if (int32_t st = check_device()) return st;
    if (int32_t st = validate_view(view)) return st;
    if (n_seqs < 0 || n_tokens < 0) return fail(HS_ERR_ARG, "%s: negative sizes", who);
    if (n_seqs == 0 || n_tokens == 0) return HS_OK;
    if (!k_new || !v_new) return fail(HS_ERR_ARG, "%s: NULL input", who);
    if (!aligned(k_new, 16) || !aligned(v_new, 16)) return fail(HS_ERR_ARG, "%s: inputs must be 16-byte aligned", who);
    if (sin != nullptr) {
        if (!cos) return fail(HS_ERR_ARG, "%s: sin given without cos", who);
        if (rotary_dim <= 0 || rotary_dim % 16 != 0 || rotary_dim > view->head_dim || n_positions <= 0)
            return fail(HS_ERR_UNSUPPORTED, "%s: rotary_dim must be a positive multiple of 16 <= head_dim", who);
    }
    if (kn.weight != nullptr && (!aligned(kn.weight, 16) || (kn.k_out && !aligned(kn.k_out, 16))))
        return fail(HS_ERR_ARG, "%s: the norm weight and the key output must be 16-byte aligned", who);
    ViewDev d = to_dev(view);
    const int64_t elems = static_cast<int64_t>(n_tokens) * d.n_kv_heads * d.head_dim;  // per sequence and per K / V
    if (elems / 8 > 0x7fffffffLL || n_seqs > 32767) return fail(HS_ERR_UNSUPPORTED, "%s: more than 2^31 chunks per sequence or 32767 sequences in one call", who);
    const bool wide = elems >= (1 << 16);  // long writes: 16 elements per thread
    dim3 grid(static_cast<unsigned>((elems + static_cast<int64_t>(kQThreads) * kWriteElems - 1) / (static_cast<int64_t>(kQThreads) * kWriteElems)), 2u * static_cast<unsigned>(n_seqs));
    cudaStream_t s = as_stream(stream);
    int *err = device_error_word();
    if (!err) return fail(HS_ERR_DEVICE, "%s: device error word unavailable", who);
    const uint16_t *k = reinterpret_cast<const uint16_t *>(k_new), *v = reinterpret_cast<const uint16_t *>(v_new);
    const uint16_t *sn = reinterpret_cast<const uint16_t *>(sin), *cs = reinterpret_cast<const uint16_t *>(cos);
#define HS_KV_WRITE(K) do { if (wide) kv_write_kernel<K, HS_KV_WRITE_WIDE><<<grid, kQThreads, 0, s>>>(d, k, v, n_seqs, n_tokens, dst_pos, sn, cs, rotary_dim, n_positions, err, kn); \
                            else kv_write_kernel<K, 8><<<grid, kQThreads, 0, s>>>(d, k, v, n_seqs, n_tokens, dst_pos, sn, cs, rotary_dim, n_positions, err, kn); } while (0)
    switch (view->kind) {
        case HS_KV_BF16: HS_KV_WRITE(HS_KV_BF16); break;
        case HS_KV_INT8: HS_KV_WRITE(HS_KV_INT8); break;
        case HS_KV_NF4: HS_KV_WRITE(HS_KV_NF4); break;
        default: HS_KV_WRITE(HS_KV_FP4); break;
    }
#undef HS_KV_WRITE
    return check_launch(who);
}

int32_t hs_kv_quantize_write(const hs_kv_view *view, const void *k_new, const void *v_new, int32_t n_seqs, int32_t n_tokens,
                             const int32_t *dst_pos, const void *sin, const void *cos, int32_t rotary_dim,
                             int32_t n_positions, hs_stream_t stream) {
    return kv_write_impl("hs_kv_quantize_write", view, k_new, v_new, n_seqs, n_tokens, dst_pos, sin, cos, rotary_dim, n_positions,
                         hs::KNormArgs{nullptr, 0.0f, 0, nullptr, 0}, stream);
}

}  // extern "C"

// hs_kv_quantize_write of one new token per sequence at position seq_lens[s] - 1 (used by hs_attn_decode_append when the
// caller gives no positions and the attention kernel does not take the write itself)
int32_t hs::kv_write_at_end(const hs_kv_view *view, const void *k_new, const void *v_new, int32_t n_seqs, const int32_t *seq_lens, const void *sin,
                            const void *cos, int32_t rotary_dim, int32_t n_positions, hs_stream_t stream) {
    return kv_write_impl("hs_attn_decode_append", view, k_new, v_new, n_seqs, 1, seq_lens, sin, cos, rotary_dim, n_positions,
                         hs::KNormArgs{nullptr, 0.0f, 0, nullptr, -1}, stream);
}

extern "C" {

int32_t hs_kv_norm_rope_quantize_write(const hs_kv_view *view, const void *k_proj, const void *v_new, int32_t n_seqs, int32_t n_tokens,
                                       const int32_t *dst_pos, const float *k_norm_weight, float eps, int32_t weight_plus_one, const void *sin,
                                       const void *cos, int32_t rotary_dim, int32_t n_positions, void *k_out, hs_stream_t stream) {
    if (!k_norm_weight) return fail(HS_ERR_ARG, "hs_kv_norm_rope_quantize_write: NULL norm weight (use hs_kv_quantize_write)");
    return kv_write_impl("hs_kv_norm_rope_quantize_write", view, k_proj, v_new, n_seqs, n_tokens, dst_pos, sin, cos, rotary_dim, n_positions,
                         hs::KNormArgs{k_norm_weight, eps, weight_plus_one, reinterpret_cast<uint16_t *>(k_out), 0}, stream);
}

int32_t hs_kv_gather_dequantize(const hs_kv_view *view, const int32_t *seq_lens, int32_t n_seqs, int32_t out_tokens,
                                void *k_out, void *v_out, hs_stream_t stream) {
    if (int32_t st = check_device()) return st;
    if (int32_t st = validate_view(view)) return st;
    if (n_seqs < 0 || out_tokens < 0) return fail(HS_ERR_ARG, "hs_kv_gather_dequantize: negative sizes");
    if (n_seqs == 0 || out_tokens == 0) return HS_OK;
    if (!seq_lens || !k_out || !v_out) return fail(HS_ERR_ARG, "hs_kv_gather_dequantize: NULL pointer");
    if (!aligned(k_out, 16) || !aligned(v_out, 16)) return fail(HS_ERR_ARG, "hs_kv_gather_dequantize: outputs must be 16-byte aligned");
    ViewDev d = to_dev(view);
    const int64_t chunks = static_cast<int64_t>(n_seqs) * out_tokens * d.n_kv_heads * (d.head_dim / 8);
    dim3 grid(static_cast<unsigned>((chunks + kQThreads - 1) / kQThreads), 2);
    kv_gather_kernel<<<grid, kQThreads, 0, as_stream(stream)>>>(d, seq_lens, n_seqs, out_tokens,
                                                               reinterpret_cast<uint16_t *>(k_out), reinterpret_cast<uint16_t *>(v_out));
    return check_launch("hs_kv_gather_dequantize");
}

}  // extern "C"
