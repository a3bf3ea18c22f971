// Decode attention (one query token per sequence) over a bf16 / int8 / 4-bit KV cache view, with a
// flat split-KV partition over all sequences and a log-sum-exp merge.
//
// Fused replacement of cache.get() -> GQA expansion -> transposes -> fp32 upcast -> q@K^T*scale ->
// softmax -> @V (architectures/llama.rs:605-640,847-872,1023-1119; the batched ragged form
// llama.rs:710-844 with its padding mask 2540-2572; qwen3_5.rs:992-1059 for the gated variant).
// The cache is read exactly once, in its stored precision, and dequantised in registers.
//
// This file holds the shape-generic CUDA-core kernel (any supported kind, head_dim 64/128/256,
// group 1/2/4/8) and the merge kernel.  It is HBM-bound: per cached token and kv head it moves
// 2*head_dim code bytes plus the scales, and does 2*group*head_dim FMAs.
#include <mutex>

#include "hs_common.cuh"

namespace hs {

constexpr int kDecTile = 64;  // tokens per tile of the flat partition
constexpr int kDecWarps = 4;
constexpr int kDecThreads = kDecWarps * 32;
constexpr int kKind4Bit = HS_KV_NF4;  // NF4 and FP4 share one instantiation (table chosen at run time)

__device__ __forceinline__ int ceil_div_i(int a, int b) { return (a + b - 1) / b; }

// Raw (unscaled) values of EPL consecutive elements starting at element `e` of a page.
template <int KIND, int EPL>
struct Chunk {
    static constexpr int kWords = KIND == HS_KV_BF16 ? EPL / 2 : (KIND == HS_KV_INT8 ? EPL / 4 : EPL / 8);
    uint32_t w[kWords];

    __device__ __forceinline__ void load(const void *page, int64_t e) {
        if constexpr (kWords == 8) {
            const uint4 *p = reinterpret_cast<const uint4 *>(reinterpret_cast<const uint16_t *>(page) + e);
            uint4 a = p[0], b = p[1];
            w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w; w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
        } else {
            const char *base = reinterpret_cast<const char *>(page) +
                               (KIND == HS_KV_BF16 ? e * 2 : (KIND == HS_KV_INT8 ? e : e / 2));
            if constexpr (kWords == 4) {
                uint4 a = *reinterpret_cast<const uint4 *>(base);
                w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w;
            } else if constexpr (kWords == 2) {
                uint2 a = *reinterpret_cast<const uint2 *>(base);
                w[0] = a.x; w[1] = a.y;
            } else {
                w[0] = *reinterpret_cast<const uint32_t *>(base);
            }
        }
    }
    __device__ __forceinline__ void zero() {
#pragma unroll
        for (int i = 0; i < kWords; ++i) w[i] = 0;
    }
    // element i as a float before the block scale is applied (int8: code - 127; 4-bit: table value)
    __device__ __forceinline__ float get(int i, const float *stab) const {
        if constexpr (KIND == HS_KV_BF16) {
            return (i & 1) ? bf16hi(w[i >> 1]) : bf16lo(w[i >> 1]);
        } else if constexpr (KIND == HS_KV_INT8) {
            // 2^23 + byte, built with one byte permute, minus (2^23 + 127): exact
            return __uint_as_float(__byte_perm(w[i >> 2], 0x4B000000u, 0x7650 + (i & 3))) - 8388735.0f;
        } else {
            uint32_t byte = (w[i >> 3] >> (8 * ((i >> 1) & 3))) & 0xffu;
            return stab[(i & 1) ? (byte & 0xfu) : (byte >> 4)];
        }
    }
};

template <int KIND, int D, int G, int EPL>
__global__ void __launch_bounds__(kDecThreads)
decode_generic_kernel(ViewDev view, const uint16_t *__restrict__ q, const int32_t *__restrict__ seq_lens, int n_seqs,
                      int n_q_heads, float scale_log2, float *__restrict__ o_part, float *__restrict__ lse_part,
                      int *__restrict__ err) {
    constexpr int LPT = D / EPL;         // lanes per token
    constexpr int TPW = 32 / LPT;        // tokens per warp step
    constexpr int NG = kDecWarps * TPW;  // lane groups per CTA
    constexpr int U = 2;                 // tokens in flight per lane group
    extern __shared__ float smem[];      // [NG][G][D + 2] merge buffer
    __shared__ float stab[16];
    if (KIND == kKind4Bit && threadIdx.x < 16) stab[threadIdx.x] = view.kind == HS_KV_NF4 ? c_nf4[threadIdx.x] : c_fp4[threadIdx.x];
    __syncthreads();

    const int kvh = blockIdx.y, H = view.n_kv_heads;
    const int64_t cta = blockIdx.x;
    const int cap = view.page_tokens * view.pages_per_seq;  // lengths beyond the view's pages are cut (and recorded)
    int64_t total = 0;
    bool over = false;
    for (int r = 0; r < n_seqs; ++r) {
        over |= seq_lens[r] > cap;
        total += ceil_div_i(min(max(seq_lens[r], 0), cap), kDecTile);
    }
    if (over && threadIdx.x == 0 && cta == 0 && kvh == 0) atomicOr(err, HS_DEVERR_DECODE_RANGE);
    // never more working CTAs than tiles (the merge uses the same rule)
    const int64_t n_ctas = total < static_cast<int64_t>(gridDim.x) ? (total > 0 ? total : 1) : static_cast<int64_t>(gridDim.x);
    if (cta >= n_ctas) return;
    const int64_t t_begin = part_begin(cta, total, n_ctas), t_end = part_begin(cta + 1, total, n_ctas);
    if (t_begin >= t_end) return;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane / LPT, li = lane % LPT, d0 = li * EPL;
    const int grp = warp * TPW + sub;
    const int bpr = D / view.block;  // scale blocks per (token, head) row
    const int sblk = d0 / view.block;
    const float kscale_mul = KIND == HS_KV_INT8 ? (1.0f / 127.0f) : 1.0f;

    int64_t acc_tiles = 0;
    for (int r = 0; r < n_seqs && acc_tiles < t_end; ++r) {
        const int L = min(max(seq_lens[r], 0), cap);
        const int nt = ceil_div_i(L, kDecTile);
        const int64_t lo = max(t_begin, acc_tiles), hi = min(t_end, acc_tiles + nt);
        const int64_t seq_tile0 = acc_tiles;
        acc_tiles += nt;
        if (lo >= hi) continue;
        const int tok_begin = static_cast<int>(lo - seq_tile0) * kDecTile;
        const int tok_end = min(L, static_cast<int>(hi - seq_tile0) * kDecTile);
        // query of this group's heads, packed bf16 pairs
        uint32_t qw[G][EPL / 2];
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const uint16_t *qp = q + (static_cast<int64_t>(r) * n_q_heads + kvh * G + g) * D + d0;
#pragma unroll
            for (int i = 0; i < EPL / 8; ++i) {
                uint4 a = reinterpret_cast<const uint4 *>(qp)[i];
                qw[g][4 * i] = a.x; qw[g][4 * i + 1] = a.y; qw[g][4 * i + 2] = a.z; qw[g][4 * i + 3] = a.w;
            }
        }
        float m[G], l[G], o[G][EPL];
#pragma unroll
        for (int g = 0; g < G; ++g) {
            m[g] = -INFINITY; l[g] = 0.0f;
#pragma unroll
            for (int i = 0; i < EPL; ++i) o[g][i] = 0.0f;
        }
        void *const *kp = view.k_pages + static_cast<int64_t>(r) * view.pages_per_seq;
        void *const *vp = view.v_pages + static_cast<int64_t>(r) * view.pages_per_seq;
        void *const *ksp = KIND == HS_KV_BF16 ? nullptr : view.k_scale_pages + static_cast<int64_t>(r) * view.pages_per_seq;
        void *const *vsp = KIND == HS_KV_BF16 ? nullptr : view.v_scale_pages + static_cast<int64_t>(r) * view.pages_per_seq;

        for (int tb = tok_begin; tb < tok_end; tb += NG * U) {  // warp-uniform trip count
            Chunk<KIND, EPL> kc[U], vc[U];
            float ks[U], vs[U];
            bool valid[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int t = tb + u * NG + grp;
                valid[u] = t < tok_end;
                ks[u] = 1.0f; vs[u] = 1.0f;
                if (valid[u]) {
                    const int page = view.pages_per_seq == 1 ? 0 : t / view.page_tokens;
                    const int64_t row = static_cast<int64_t>(t - page * view.page_tokens) * H + kvh;
                    kc[u].load(kp[page], row * D + d0);
                    vc[u].load(vp[page], row * D + d0);
                    if constexpr (KIND != HS_KV_BF16) {
                        ks[u] = load_scale(ksp[page], row * bpr + sblk, view.scale_dtype) * kscale_mul;
                        vs[u] = load_scale(vsp[page], row * bpr + sblk, view.scale_dtype) * kscale_mul;
                    }
                } else {
                    kc[u].zero(); vc[u].zero();
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                float s[G];
#pragma unroll
                for (int g = 0; g < G; ++g) s[g] = 0.0f;
#pragma unroll
                for (int i = 0; i < EPL; ++i) {
                    const float kf = kc[u].get(i, stab);
#pragma unroll
                    for (int g = 0; g < G; ++g) {
                        const float qf = (i & 1) ? bf16hi(qw[g][i >> 1]) : bf16lo(qw[g][i >> 1]);
                        s[g] = fmaf(qf, kf, s[g]);
                    }
                }
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    float v = s[g] * ks[u];
#pragma unroll
                    for (int off = 1; off < LPT; off <<= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
                    s[g] = valid[u] ? v * scale_log2 : -INFINITY;
                }
                float p[G];
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    const float mn = fmaxf(m[g], s[g]);
                    const float corr = (mn == -INFINITY) ? 1.0f : exp2f(m[g] - mn);
                    p[g] = (mn == -INFINITY) ? 0.0f : exp2f(s[g] - mn);
                    l[g] = l[g] * corr + p[g];
                    m[g] = mn;
                    if (corr != 1.0f) {
#pragma unroll
                        for (int i = 0; i < EPL; ++i) o[g][i] *= corr;
                    }
                    p[g] *= vs[u];
                }
#pragma unroll
                for (int i = 0; i < EPL; ++i) {
                    const float vf = vc[u].get(i, stab);
#pragma unroll
                    for (int g = 0; g < G; ++g) o[g][i] = fmaf(p[g], vf, o[g][i]);
                }
            }
        }
        // ---- merge the NG lane groups through shared memory ----
        __syncthreads();  // previous segment's readers are done
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float *dst = smem + (static_cast<int64_t>(grp) * G + g) * (D + 2);
#pragma unroll
            for (int i = 0; i < EPL; ++i) dst[d0 + i] = o[g][i];
            if (li == 0) { dst[D] = m[g]; dst[D + 1] = l[g]; }
        }
        __syncthreads();
        const int slot = static_cast<int>(cta) + r;
        for (int idx = threadIdx.x; idx < G * D; idx += kDecThreads) {
            const int g = idx / D, d = idx % D;
            float M = -INFINITY;
            for (int j = 0; j < NG; ++j) M = fmaxf(M, smem[(static_cast<int64_t>(j) * G + g) * (D + 2) + D]);
            float num = 0.0f, den = 0.0f;
            for (int j = 0; j < NG; ++j) {
                const float *src = smem + (static_cast<int64_t>(j) * G + g) * (D + 2);
                const float wgt = src[D] == -INFINITY ? 0.0f : exp2f(src[D] - M);
                num = fmaf(wgt, src[d], num);
                den = fmaf(wgt, src[D + 1], den);
            }
            const int64_t hrow = static_cast<int64_t>(slot) * n_q_heads + kvh * G + g;
            o_part[hrow * D + d] = den > 0.0f ? num / den : 0.0f;
            if (d == 0) lse_part[hrow] = den > 0.0f ? (M + log2f(den)) * 0.6931471805599453f : -INFINITY;
        }
    }
}

// Merge the split-KV partials of one sequence, kMergeHeads query heads per CTA.  The slot range of the
// sequence is recomputed from seq_lens with the same partition arithmetic the decode kernel used: CTA c
// and sequence r share slots (c + r) * ppp + k, k < ppp (ppp = partials each pair writes).
constexpr int kMergeThreads = 256;
constexpr int kMergeHeads = 4;
constexpr int kMergeMaxParts = 1280;  // >= decode_max_ctas() * kMaxPartsPerPair on a 148-SM part (checked on the host)
__global__ void __launch_bounds__(kMergeThreads)
decode_merge_kernel(const int32_t *__restrict__ seq_lens, int n_seqs, int n_q_heads, int D, int n_ctas, int tile, int cap,
                    int ppp, const float *__restrict__ o_part, const float *__restrict__ lse_part, uint16_t *__restrict__ out,
                    const uint16_t *__restrict__ gate, float *__restrict__ o_shard, float *__restrict__ lse_shard) {
    __shared__ int s_slot[kMergeMaxParts];
    __shared__ float s_w[kMergeMaxParts * kMergeHeads];
    __shared__ float s_den[kMergeHeads], s_max[kMergeHeads];
    __shared__ int s_nparts;
    const int r = blockIdx.x, h0 = blockIdx.y * kMergeHeads, lane = threadIdx.x & 31;
    const int nh = min(kMergeHeads, n_q_heads - h0);
    // every warp computes the tile prefix redundantly, one coalesced load per 32 sequences
    long long total = 0, before = 0;
    for (int base = 0; base < n_seqs; base += 32) {
        const int i = base + lane;
        const int t = i < n_seqs ? ceil_div_i(min(max(seq_lens[i], 0), cap), tile) : 0;
        total += t;
        before += i < r ? t : 0;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        total += __shfl_xor_sync(0xffffffffu, total, off);
        before += __shfl_xor_sync(0xffffffffu, before, off);
    }
    const long long nt = ceil_div_i(min(max(seq_lens[r], 0), cap), tile);
    if (total < n_ctas) n_ctas = total > 0 ? static_cast<int>(total) : 1;  // the decode kernels never use more CTAs than tiles
    if (threadIdx.x == 0) {
        // CTAs whose tile range overlaps [before, before + nt); a CTA with an empty range wrote nothing
        int n = 0;
        if (nt > 0) {
            long long c = before * n_ctas / total;
            while (c > 0 && part_begin(c, total, n_ctas) > before) --c;
            while (part_begin(c + 1, total, n_ctas) <= before) ++c;
            for (; c < n_ctas && part_begin(c, total, n_ctas) < before + nt; ++c) {
                if (part_begin(c, total, n_ctas) >= part_begin(c + 1, total, n_ctas)) continue;
                for (int k = 0; k < ppp && n < kMergeMaxParts; ++k) s_slot[n++] = static_cast<int>((c + r) * ppp + k);
            }
        }
        s_nparts = n;
    }
    __syncthreads();
    const int np = s_nparts;
    for (int i = threadIdx.x; i < np * nh; i += kMergeThreads) {
        const int pi = i / nh, hh = i - pi * nh;
        s_w[pi * kMergeHeads + hh] = lse_part[static_cast<int64_t>(s_slot[pi]) * n_q_heads + h0 + hh];
    }
    __syncthreads();
    if (threadIdx.x < nh) {
        float M = -INFINITY;
        for (int pi = 0; pi < np; ++pi) M = fmaxf(M, s_w[pi * kMergeHeads + threadIdx.x]);
        s_max[threadIdx.x] = M;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < np * nh; i += kMergeThreads) {
        const int pi = i / nh, hh = i - pi * nh;
        const float ls = s_w[pi * kMergeHeads + hh];
        s_w[pi * kMergeHeads + hh] = ls == -INFINITY ? 0.0f : __expf(ls - s_max[hh]);
    }
    __syncthreads();
    if (threadIdx.x < nh) {
        float den = 0.0f;
        for (int pi = 0; pi < np; ++pi) den += s_w[pi * kMergeHeads + threadIdx.x];
        s_den[threadIdx.x] = den;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < nh * D; idx += kMergeThreads) {
        const int hh = idx / D, d = idx - hh * D;
        const int64_t row = static_cast<int64_t>(r) * n_q_heads + h0 + hh;
        float num = 0.0f;
        for (int pi = 0; pi < np; ++pi)
            num = fmaf(s_w[pi * kMergeHeads + hh], o_part[(static_cast<int64_t>(s_slot[pi]) * n_q_heads + h0 + hh) * D + d], num);
        const float den = s_den[hh];
        const float o = den > 0.0f ? num / den : 0.0f;
        if (o_shard != nullptr) {
            o_shard[row * D + d] = o;
            if (d == 0) lse_shard[row] = den > 0.0f ? s_max[hh] + __logf(den) : -INFINITY;
            continue;
        }
        float res = o;
        if (gate != nullptr) {
            const float gv = bf16_bits_to_f32(gate[row * D + d]);
            res = bf16_round(o) * bf16_round(1.0f / (1.0f + __expf(-gv)));  // ctx * sigmoid(gate) in bf16 (qwen3_5.rs:1056-1059)
        }
        out[row * D + d] = f32_to_bf16_bits(res);
    }
}

// Merge of externally produced partials (KV-length shards from several GPUs, or a caller's own split).
// Part p's outputs start at o_parts + p * stride_o floats ([n_rows, D] dense), its log-sum-exps at lse_parts + p * stride_l.
__global__ void merge_parts_kernel(const float *__restrict__ o_parts, const float *__restrict__ lse_parts, int n_parts,
                                   int64_t stride_o, int64_t stride_l, int D, uint16_t *__restrict__ out,
                                   const uint16_t *__restrict__ gate) {
    const int64_t row = blockIdx.x;
    const int d = threadIdx.x;
    float M = -INFINITY;
    for (int p = 0; p < n_parts; ++p) M = fmaxf(M, lse_parts[p * stride_l + row]);
    float num = 0.0f, den = 0.0f;
    for (int p = 0; p < n_parts; ++p) {
        const float ls = lse_parts[p * stride_l + row];
        const float wgt = ls == -INFINITY ? 0.0f : __expf(ls - M);
        num = fmaf(wgt, o_parts[p * stride_o + row * D + d], num);
        den += wgt;
    }
    float res = den > 0.0f ? num / den : 0.0f;
    if (gate != nullptr) {
        const float gv = bf16_bits_to_f32(gate[row * D + d]);
        res = bf16_round(res) * bf16_round(1.0f / (1.0f + __expf(-gv)));
    }
    out[row * D + d] = f32_to_bf16_bits(res);
}

static int decode_max_ctas() { return 4 * sm_count(); }
constexpr int kMaxPartsPerPair = 2;

// decode_tc.cu: tensor-core kernel for the int8 / head_dim 128 / 8 kv heads / group 4 shape
int32_t decode_int8_tc_try(const ViewDev &v, const uint16_t *q, const int32_t *seq_lens, int n_seqs, int n_q_heads,
                           float softmax_scale, float *o_part, float *lse_part, int *err, cudaStream_t s, int *n_ctas_out,
                           uint16_t *out, const uint16_t *gate, float *o_shard, float *lse_shard, int *merged_out,
                           const ShardArgs *shard, int after_write, const AppendArgs *append);

template <int KIND, int D, int G>
static int32_t launch_generic(const ViewDev &v, const uint16_t *q, const int32_t *seq_lens, int n_seqs, int n_q_heads,
                              float scale_log2, float *o_part, float *lse_part, int *err, int n_ctas, cudaStream_t s) {
    constexpr int EPL = (G == 8) ? 8 : 16;
    constexpr int NG = kDecWarps * (32 / (D / EPL));
    const size_t smem = static_cast<size_t>(NG) * G * (D + 2) * sizeof(float);
    auto kern = decode_generic_kernel<KIND, D, G, EPL>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) return fail(static_cast<int32_t>(e), "hs_attn_decode: %s", cudaGetErrorString(e));
    }
    dim3 grid(n_ctas, v.n_kv_heads);
    kern<<<grid, kDecThreads, smem, s>>>(v, q, seq_lens, n_seqs, n_q_heads, scale_log2, o_part, lse_part, err);
    return HS_OK;
}

template <int KIND, int D>
static int32_t dispatch_g(int G, const ViewDev &v, const uint16_t *q, const int32_t *seq_lens, int n_seqs, int n_q_heads,
                          float scale_log2, float *o_part, float *lse_part, int *err, int n_ctas, cudaStream_t s) {
    switch (G) {
        case 1: return launch_generic<KIND, D, 1>(v, q, seq_lens, n_seqs, n_q_heads, scale_log2, o_part, lse_part, err, n_ctas, s);
        case 2: return launch_generic<KIND, D, 2>(v, q, seq_lens, n_seqs, n_q_heads, scale_log2, o_part, lse_part, err, n_ctas, s);
        case 4: return launch_generic<KIND, D, 4>(v, q, seq_lens, n_seqs, n_q_heads, scale_log2, o_part, lse_part, err, n_ctas, s);
        case 8: return launch_generic<KIND, D, 8>(v, q, seq_lens, n_seqs, n_q_heads, scale_log2, o_part, lse_part, err, n_ctas, s);
        default: return fail(HS_ERR_UNSUPPORTED, "hs_attn_decode: n_q_heads / n_kv_heads = %d (supported: 1, 2, 4, 8)", G);
    }
}

template <int KIND>
static int32_t dispatch_d(int D, int G, const ViewDev &v, const uint16_t *q, const int32_t *seq_lens, int n_seqs,
                          int n_q_heads, float scale_log2, float *o_part, float *lse_part, int *err, int n_ctas,
                          cudaStream_t s) {
    switch (D) {
        case 64: return dispatch_g<KIND, 64>(G, v, q, seq_lens, n_seqs, n_q_heads, scale_log2, o_part, lse_part, err, n_ctas, s);
        case 128: return dispatch_g<KIND, 128>(G, v, q, seq_lens, n_seqs, n_q_heads, scale_log2, o_part, lse_part, err, n_ctas, s);
        case 256: return dispatch_g<KIND, 256>(G, v, q, seq_lens, n_seqs, n_q_heads, scale_log2, o_part, lse_part, err, n_ctas, s);
        default: return fail(HS_ERR_UNSUPPORTED, "hs_attn_decode: head_dim %d", D);
    }
}

// ---- decode scratch that lives inside the library ------------------------------------------------
// Backing store of hs_attn_decode_static(): the split-KV partials go here instead of into a workspace the
// caller would have had to allocate.  Every GPU that loads the library holds these bytes until exit.
constexpr int64_t kStaticScratchBytes = 24ll << 20;  // 24 MiB
constexpr int kStaticMaxDevices = 64;
static __device__ __align__(256) unsigned char g_decode_static_scratch[kStaticScratchBytes];
// Device address of the array on each device.  The array's name is only a host-side handle: the address a
// kernel can use has to be asked for, per device, with that device current.
static void *g_static_scratch_ptr[kStaticMaxDevices] = {nullptr};
static std::mutex g_static_scratch_mutex;

static int32_t static_scratch_for_current_device(void **out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(HS_ERR_DEVICE, "hs_attn_decode_static: no usable CUDA device: %s", cudaGetErrorString(e));
    }
    if (dev < 0 || dev >= kStaticMaxDevices) return fail(HS_ERR_DEVICE, "hs_attn_decode_static: device ordinal %d is beyond the table of %d", dev, kStaticMaxDevices);
    std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
    if (g_static_scratch_ptr[dev] == nullptr) {
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, g_decode_static_scratch);
        if (e != cudaSuccess || p == nullptr) {
            cudaGetLastError();
            return fail(e != cudaSuccess ? static_cast<int32_t>(e) : HS_ERR_DEVICE, "hs_attn_decode_static: cudaGetSymbolAddress failed: %s",
                        cudaGetErrorString(e));
        }
        g_static_scratch_ptr[dev] = p;
    }
    *out = g_static_scratch_ptr[dev];
    return HS_OK;
}

int32_t decode_impl(const void *q, const hs_kv_view *view, const int32_t *seq_lens, int32_t n_seqs, int32_t n_q_heads, float softmax_scale,
                    void *out, const void *gate, void *workspace, int64_t workspace_bytes, float *o_shard, float *lse_shard,
                    const ShardArgs *shard, hs_stream_t stream, int after_write = 0, const AppendArgs *append = nullptr, int *appended = nullptr);

}  // namespace hs

using namespace hs;

extern "C" {

int64_t hs_attn_decode_workspace_bytes(int32_t n_seqs, int32_t n_q_heads, int32_t head_dim) {
    if (n_seqs < 0 || n_q_heads <= 0 || head_dim <= 0) return HS_ERR_ARG;
    const int64_t slots = (static_cast<int64_t>(decode_max_ctas()) + n_seqs) * kMaxPartsPerPair;
    return slots * n_q_heads * (static_cast<int64_t>(head_dim) + 1) * 4;
}

int32_t hs_attn_decode(const void *q, const hs_kv_view *view, const int32_t *seq_lens, int32_t n_seqs, int32_t n_q_heads,
                       float softmax_scale, void *out, const void *gate, void *workspace, int64_t workspace_bytes,
                       float *o_shard, float *lse_shard, hs_stream_t stream) {
    return hs::decode_impl(q, view, seq_lens, n_seqs, n_q_heads, softmax_scale, out, gate, workspace, workspace_bytes, o_shard, lse_shard,
                           nullptr, stream);
}

}  // extern "C"

// The body of hs_attn_decode; `shard` (optional) makes the tensor-core kernel exchange its result with the other GPUs of
// a shard group and merge again (hs_attn_decode_sharded); only that kernel can, so other shapes are refused then.
int32_t hs::decode_impl(const void *q, const hs_kv_view *view, const int32_t *seq_lens, int32_t n_seqs, int32_t n_q_heads,
                        float softmax_scale, void *out, const void *gate, void *workspace, int64_t workspace_bytes,
                        float *o_shard, float *lse_shard, const ShardArgs *shard, hs_stream_t stream, int after_write, const AppendArgs *append,
                        int *appended) {
    if (appended) *appended = 0;
    if (int32_t st = check_device()) return st;
    if (int32_t st = validate_view(view)) return st;
    if (n_seqs < 0 || n_q_heads <= 0) return fail(HS_ERR_ARG, "hs_attn_decode: bad sizes");
    if (n_seqs == 0) return HS_OK;
    if (n_q_heads % view->n_kv_heads != 0) return fail(HS_ERR_ARG, "hs_attn_decode: n_q_heads %d not a multiple of n_kv_heads %d", n_q_heads, view->n_kv_heads);
    if (!q || !seq_lens || !workspace) return fail(HS_ERR_ARG, "hs_attn_decode: NULL pointer");
    if ((o_shard == nullptr) != (lse_shard == nullptr)) return fail(HS_ERR_ARG, "hs_attn_decode: o_shard and lse_shard go together");
    if (!o_shard && !out && !(shard && shard->push_only)) return fail(HS_ERR_ARG, "hs_attn_decode: no output");
    if (!aligned(q, 16) || !aligned(workspace, 16) || (out && !aligned(out, 2)) || (gate && !aligned(gate, 2)) || !aligned(seq_lens, 4))
        return fail(HS_ERR_ARG, "hs_attn_decode: q and workspace must be 16-byte aligned");
    const int D = view->head_dim, G = n_q_heads / view->n_kv_heads;
    const int64_t need = hs_attn_decode_workspace_bytes(n_seqs, n_q_heads, D);
    if (workspace_bytes < need) return fail(HS_ERR_WORKSPACE, "hs_attn_decode: workspace %lld < %lld bytes", (long long)workspace_bytes, (long long)need);
    int *err = device_error_word();
    if (!err) return fail(HS_ERR_DEVICE, "hs_attn_decode: device error word unavailable");

    ViewDev v = to_dev(view);
    int n_ctas = (3 * sm_count() + v.n_kv_heads - 1) / v.n_kv_heads;
    n_ctas = max(1, min(n_ctas, decode_max_ctas()));
    const int64_t slots = (static_cast<int64_t>(decode_max_ctas()) + n_seqs) * kMaxPartsPerPair;
    float *o_part = reinterpret_cast<float *>(workspace);
    float *lse_part = o_part + slots * n_q_heads * D;
    const float scale_log2 = softmax_scale * 1.4426950408889634f;
    cudaStream_t s = as_stream(stream);
    const uint16_t *qp = reinterpret_cast<const uint16_t *>(q);
    int32_t st;
    int tile = kDecTile, tc_ctas = 0, ppp = 1, merged = 0;
    prof_begin(s);
    st = decode_int8_tc_try(v, qp, seq_lens, n_seqs, n_q_heads, softmax_scale, o_part, lse_part, err, s, &tc_ctas,
                            reinterpret_cast<uint16_t *>(out), reinterpret_cast<const uint16_t *>(gate), o_shard, lse_shard, &merged, shard, after_write, append);
    if (st == HS_OK && append && tc_ctas == 0) {  // the tensor-core kernel did not take the launch: nothing was written, the caller writes
        prof_end(s);
        return HS_OK;
    }
    if (appended && append && tc_ctas > 0) *appended = 1;
    if (st == HS_OK && shard && tc_ctas == 0) {
        prof_end(s);
        return fail(HS_ERR_UNSUPPORTED, "hs_attn_decode_sharded: only the tensor-core decode kernel exchanges shard results (quantised cache, 8 kv heads x 128 "
                                        "with 32 query heads or 2 x 256 with 16, cooperative launch available); use hs_attn_decode with o_shard / lse_shard, an "
                                        "all-gather and hs_attn_merge_partials_strided for this shape");
    }
    if (st == HS_OK && tc_ctas > 0) {
        n_ctas = tc_ctas;
        tile = 16;
    } else if (st == HS_OK) {
        switch (view->kind) {
            case HS_KV_BF16: st = dispatch_d<HS_KV_BF16>(D, G, v, qp, seq_lens, n_seqs, n_q_heads, scale_log2, o_part, lse_part, err, n_ctas, s); break;
            case HS_KV_INT8: st = dispatch_d<HS_KV_INT8>(D, G, v, qp, seq_lens, n_seqs, n_q_heads, scale_log2, o_part, lse_part, err, n_ctas, s); break;
            default: st = dispatch_d<kKind4Bit>(D, G, v, qp, seq_lens, n_seqs, n_q_heads, scale_log2, o_part, lse_part, err, n_ctas, s); break;
        }
    }
    prof_end(s);
    if (st != HS_OK) return st;
    if (int32_t e = check_launch("hs_attn_decode")) return e;
    if (merged) return HS_OK;  // the decode kernel merged its own partials behind a grid barrier
    if (static_cast<int64_t>(n_ctas) * ppp > kMergeMaxParts) return fail(HS_ERR_UNSUPPORTED, "hs_attn_decode: %d partial slots exceed the merge kernel's table", n_ctas * ppp);
    dim3 mgrid(n_seqs, (n_q_heads + kMergeHeads - 1) / kMergeHeads);
    decode_merge_kernel<<<mgrid, kMergeThreads, 0, s>>>(seq_lens, n_seqs, n_q_heads, D, n_ctas, tile, v.page_tokens * v.pages_per_seq, ppp, o_part,
                                            lse_part, reinterpret_cast<uint16_t *>(out), reinterpret_cast<const uint16_t *>(gate),
                                            o_shard, lse_shard);
    return check_launch("hs_attn_decode (merge)");
}

extern "C" {

int32_t hs_attn_merge_partials_strided(const float *o_parts, const float *lse_parts, int32_t n_parts, int64_t part_stride_o,
                                       int64_t part_stride_lse, int64_t n_rows, int32_t head_dim, void *out, const void *gate,
                                       hs_stream_t stream) {
    if (int32_t st = check_device()) return st;
    if (n_parts <= 0 || n_rows < 0 || head_dim <= 0 || head_dim > 1024) return fail(HS_ERR_ARG, "hs_attn_merge_partials: bad sizes");
    if (part_stride_o < n_rows * head_dim || part_stride_lse < n_rows) return fail(HS_ERR_ARG, "hs_attn_merge_partials: part strides overlap");
    if (n_rows == 0) return HS_OK;
    if (!o_parts || !lse_parts || !out) return fail(HS_ERR_ARG, "hs_attn_merge_partials: NULL pointer");
    if (n_rows > 0x7fffffffLL) return fail(HS_ERR_ARG, "hs_attn_merge_partials: too many rows");
    merge_parts_kernel<<<static_cast<unsigned>(n_rows), head_dim, 0, as_stream(stream)>>>(
        o_parts, lse_parts, n_parts, part_stride_o, part_stride_lse, head_dim, reinterpret_cast<uint16_t *>(out),
        reinterpret_cast<const uint16_t *>(gate));
    return check_launch("hs_attn_merge_partials");
}

int32_t hs_attn_merge_partials(const float *o_parts, const float *lse_parts, int32_t n_parts, int64_t n_rows, int32_t head_dim,
                               void *out, const void *gate, hs_stream_t stream) {
    return hs_attn_merge_partials_strided(o_parts, lse_parts, n_parts, n_rows * head_dim, n_rows, n_rows, head_dim, out, gate, stream);
}


int64_t hs_attn_decode_static_max_bytes(void) { return kStaticScratchBytes; }

int32_t hs_attn_decode_static(const void *q, const hs_kv_view *view, const int32_t *seq_lens, int32_t n_seqs, int32_t n_q_heads,
                              float softmax_scale, void *out, const void *gate, hs_stream_t stream) {
    if (int32_t st = check_device()) return st;
    if (int32_t st = validate_view(view)) return st;
    if (n_seqs < 0 || n_q_heads <= 0) return fail(HS_ERR_ARG, "hs_attn_decode_static: bad sizes");
    const int64_t need = hs_attn_decode_workspace_bytes(n_seqs, n_q_heads, view->head_dim);
    if (need < 0 || need > kStaticScratchBytes)
        return fail(HS_ERR_WORKSPACE,
                    "hs_attn_decode_static: n_seqs %d x n_q_heads %d x head_dim %d needs %lld bytes of scratch, the built-in array holds "
                    "%lld; use hs_attn_decode with a caller-provided workspace",
                    n_seqs, n_q_heads, view->head_dim, (long long)need, (long long)kStaticScratchBytes);
    void *scratch = nullptr;
    if (int32_t st = static_scratch_for_current_device(&scratch)) return st;
    // Nothing in the scratch has to start at zero: each launch writes every partial slot it later reads.
    return hs_attn_decode(q, view, seq_lens, n_seqs, n_q_heads, softmax_scale, out, gate, scratch, kStaticScratchBytes, nullptr,
                          nullptr, stream);
}


int32_t hs_attn_decode_append(const void *q, const void *k_new, const void *v_new, const hs_kv_view *view, const int32_t *dst_pos,
                              const int32_t *seq_lens, int32_t n_seqs, int32_t n_q_heads, float softmax_scale, const void *sin, const void *cos,
                              int32_t rotary_dim, int32_t n_positions, void *out, const void *gate, void *workspace, int64_t workspace_bytes,
                              hs_stream_t stream) {
    if (!k_new || !v_new) return fail(HS_ERR_ARG, "hs_attn_decode_append: NULL new token");
    if (dst_pos == nullptr) {
        // the new token goes to position seq_lens[s] - 1: the attention kernel can write it itself (u8 caches on the tensor-core
        // kernel: one launch per step); otherwise the write kernel runs first, at those positions
        if (!aligned(k_new, 16) || !aligned(v_new, 16)) return fail(HS_ERR_ARG, "hs_attn_decode_append: inputs must be 16-byte aligned");
        if (sin != nullptr && (!cos || rotary_dim <= 0 || rotary_dim % 16 != 0 || (view && rotary_dim > view->head_dim) || n_positions <= 0))
            return fail(HS_ERR_UNSUPPORTED, "hs_attn_decode_append: rotary_dim must be a positive multiple of 16 <= head_dim");
        AppendArgs ap{reinterpret_cast<const uint16_t *>(k_new), reinterpret_cast<const uint16_t *>(v_new), reinterpret_cast<const uint16_t *>(sin),
                      reinterpret_cast<const uint16_t *>(cos), rotary_dim, n_positions};
        int appended = 0;
        if (view && view->kind == HS_KV_INT8) {
            if (int32_t st = decode_impl(q, view, seq_lens, n_seqs, n_q_heads, softmax_scale, out, gate, workspace, workspace_bytes, nullptr, nullptr,
                                         nullptr, stream, 0, &ap, &appended))
                return st;
            if (appended || n_seqs == 0) return HS_OK;
        }
        if (int32_t st = kv_write_at_end(view, k_new, v_new, n_seqs, seq_lens, sin, cos, rotary_dim, n_positions, stream)) return st;
        return decode_impl(q, view, seq_lens, n_seqs, n_q_heads, softmax_scale, out, gate, workspace, workspace_bytes, nullptr, nullptr, nullptr, stream, 1);
    }
    if (int32_t st = hs_kv_quantize_write(view, k_new, v_new, n_seqs, 1, dst_pos, sin, cos, rotary_dim, n_positions, stream)) return st;
    return decode_impl(q, view, seq_lens, n_seqs, n_q_heads, softmax_scale, out, gate, workspace, workspace_bytes, nullptr, nullptr, nullptr, stream, 1);
}

int32_t hs_attn_decode_step(const hs_kv_view *view, const void *host_in, void *dev_in, const int32_t *dst_pos, const int32_t *seq_lens,
                            int32_t n_seqs, int32_t n_q_heads, float softmax_scale, const void *sin, const void *cos, int32_t rotary_dim,
                            int32_t n_positions, void *dev_out, void *host_out, void *workspace, int64_t workspace_bytes, int32_t flags,
                            hs_stream_t stream) {
    if (int32_t st = check_device()) return st;
    if (int32_t st = validate_view(view)) return st;
    if (n_seqs < 0 || n_q_heads <= 0) return fail(HS_ERR_ARG, "hs_attn_decode_step: bad sizes");
    if (n_seqs == 0) return HS_OK;
    if (!host_in || !dev_in || !dev_out || !host_out || !seq_lens)
        return fail(HS_ERR_ARG, "hs_attn_decode_step: NULL pointer");
    if (!aligned(dev_in, 16)) return fail(HS_ERR_ARG, "hs_attn_decode_step: dev_in must be 16-byte aligned");
    const int64_t D = view->head_dim;
    const int64_t q_elems = static_cast<int64_t>(n_seqs) * n_q_heads * D, kv_elems = static_cast<int64_t>(n_seqs) * view->n_kv_heads * D;
    if ((q_elems * 2) % 16 != 0 || (kv_elems * 2) % 16 != 0) return fail(HS_ERR_ARG, "hs_attn_decode_step: q and k/v parts must be multiples of 16 bytes");
    cudaStream_t s = as_stream(stream);
    cudaError_t e = cudaMemcpyAsync(dev_in, host_in, static_cast<size_t>(q_elems + 2 * kv_elems) * 2, cudaMemcpyHostToDevice, s);
    if (e != cudaSuccess) return fail(static_cast<int32_t>(e), "hs_attn_decode_step: %s", cudaGetErrorString(e));
    uint16_t *qd = reinterpret_cast<uint16_t *>(dev_in), *kd = qd + q_elems, *vd = kd + kv_elems;
    // cache update + attention: one launch when the new tokens go to seq_lens - 1 (dst_pos == NULL) on a u8 cache, else the write
    // kernel and the attention kernel as its programmatic dependent; q came with the copy before both
    if (int32_t st = hs_attn_decode_append(qd, kd, vd, view, dst_pos, seq_lens, n_seqs, n_q_heads, softmax_scale, sin, cos, rotary_dim, n_positions, dev_out,
                                           nullptr, workspace, workspace_bytes, stream))
        return st;
    // (letting the kernel store into mapped host memory instead of this copy was measured: 9 us slower per step; copy kernels over
    // mapped pinned memory in place of the two cudaMemcpyAsync calls: 3 us faster of 102, not worth a second mechanism; the host
    // polling a word that the stream writes behind the copy, instead of cudaStreamSynchronize: 106 against 104 us)
    e = cudaMemcpyAsync(host_out, dev_out, static_cast<size_t>(q_elems) * 2, cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess && (flags & HS_STEP_SYNC)) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return fail(static_cast<int32_t>(e), "hs_attn_decode_step: %s", cudaGetErrorString(e));
    return HS_OK;
}

}  // extern "C"
