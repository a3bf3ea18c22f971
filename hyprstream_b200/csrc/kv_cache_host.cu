// Host-side cache objects: a C++ mirror of the reference's LayerKVCache and BlockPool
// (crates/hyprstream/src/runtime/kv_cache.rs:477-680, 1029-1900) over device-resident, token-granular storage.
//
// What is kept: names and meaning of new / new_paged / update / get / clear / truncate_to / seq_pos /
// memory_usage; growth in 1024-token chunks capped at max_seq_len (kv_cache.rs:700,1146-1200); 256-token pages
// from a shared pool with a LIFO free list, owner tags, typed exhaustion and roll-back of a half-finished
// allocation (kv_cache.rs:477,515-680,1460-1473); overflow and empty-cache errors raised before any launch
// (kv_cache.rs:1288-1294,1500-1503); pages returned to the pool on drop (kv_cache.rs:1889-1898).
// What differs on purpose: quantised codes and scales stay in HBM (the reference keeps them in host Vec<u8>,
// kv_cache.rs:721-732,845-856,919-921); every token is quantised when written (no bf16 staging buffer, no
// whole-history re-quantisation, kv_cache.rs:1204-1272); truncate_to is a length change for every kind (the
// reference clears a quantised cache, kv_cache.rs:1717-1720); paged storage may be quantised (kv_cache.rs:1111).
//
// This file is host code only; it launches kernels solely through the C ABI in include/hs_attn.h.
#include <algorithm>
#include <atomic>
#include <mutex>
#include <numeric>
#include <vector>

#include "hs_common.cuh"

namespace hs {

constexpr int kDefaultChunk = 1024;  // kv_cache.rs:700 DEFAULT_CHUNK_SIZE

// ---- device allocator (replaceable) ---------------------------------------------------------------
static void *default_alloc(size_t bytes) {
    void *p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return p;
}
static void default_free(void *p) { cudaFree(p); }
static hs_alloc_fn g_alloc = default_alloc;
static hs_free_fn g_free = default_free;

struct Geometry {
    int kind, block, scale_dtype, n_kv_heads, head_dim;
    size_t row_bytes() const {  // code / value bytes of one token (all kv heads)
        const size_t per = kind == HS_KV_BF16 ? 2 * head_dim : (kind == HS_KV_INT8 ? head_dim : head_dim / 2);
        return per * n_kv_heads;
    }
    size_t scale_row_bytes() const {
        if (kind == HS_KV_BF16) return 0;
        return static_cast<size_t>(n_kv_heads) * (head_dim / block) * (scale_dtype == HS_SCALE_F16 ? 2 : 4);
    }
    bool same(const Geometry &o) const {
        return kind == o.kind && block == o.block && scale_dtype == o.scale_dtype && n_kv_heads == o.n_kv_heads && head_dim == o.head_dim;
    }
};

static int32_t check_geometry(const Geometry &g, const char *who) {
    if (g.kind < HS_KV_BF16 || g.kind > HS_KV_FP4) return fail(HS_ERR_ARG, "%s: unknown kind %d", who, g.kind);
    if (g.n_kv_heads <= 0) return fail(HS_ERR_ARG, "%s: n_kv_heads must be positive", who);
    if (g.head_dim != 64 && g.head_dim != 128 && g.head_dim != 256) return fail(HS_ERR_UNSUPPORTED, "%s: head_dim %d", who, g.head_dim);
    if (g.kind != HS_KV_BF16) {
        if (g.block != 64 && g.block != 128 && g.block != 256) return fail(HS_ERR_UNSUPPORTED, "%s: block %d", who, g.block);
        if (g.head_dim % g.block != 0) return fail(HS_ERR_UNSUPPORTED, "%s: block %d must divide head_dim %d", who, g.block, g.head_dim);
        if (g.scale_dtype != HS_SCALE_F32 && g.scale_dtype != HS_SCALE_F16) return fail(HS_ERR_ARG, "%s: unknown scale dtype", who);
    }
    return HS_OK;
}

// Four device buffers for `tokens` tokens: K data, V data, K scales, V scales.
struct Slab {
    unsigned char *p[4] = {nullptr, nullptr, nullptr, nullptr};
    size_t bytes[4] = {0, 0, 0, 0};
    int tokens = 0;

    int32_t allocate(const Geometry &g, int n_tokens) {
        tokens = n_tokens;
        bytes[0] = bytes[1] = g.row_bytes() * n_tokens;
        bytes[2] = bytes[3] = g.scale_row_bytes() * n_tokens;
        for (int i = 0; i < 4; ++i) {
            if (bytes[i] == 0) continue;
            p[i] = static_cast<unsigned char *>(g_alloc(bytes[i]));
            if (!p[i]) {
                release();
                return fail(static_cast<int32_t>(cudaErrorMemoryAllocation), "cache storage: device allocation of %zu bytes failed", bytes[i]);
            }
        }
        return HS_OK;
    }
    void release() {
        for (int i = 0; i < 4; ++i) {
            if (p[i]) g_free(p[i]);
            p[i] = nullptr;
            bytes[i] = 0;
        }
        tokens = 0;
    }
    size_t total() const { return bytes[0] + bytes[1] + bytes[2] + bytes[3]; }
};

}  // namespace hs

// ---- BlockPool (kv_cache.rs:515-680) ------------------------------------------------------------------
struct hs_pool {
    std::atomic<int> refs{1};       // the handle + every cache created from the pool (Arc<BlockPool>, kv_cache.rs:1111-1130)
    hs::Geometry geo;
    int page_tokens = 0, n_blocks = 0;
    hs::Slab slab;                  // one slab cut into n_blocks pages; a unit is a (K, V) page pair
    std::vector<int> free_list;     // LIFO
    std::vector<int64_t> owner;     // -1 = free
    std::mutex mu;

    int allocate(int64_t who) {     // -1 when exhausted
        std::lock_guard<std::mutex> lock(mu);
        if (free_list.empty()) return -1;
        const int id = free_list.back();
        free_list.pop_back();
        owner[id] = who;
        return id;
    }
    bool release(int64_t who, int id) {
        std::lock_guard<std::mutex> lock(mu);
        if (id < 0 || id >= n_blocks || owner[id] != who) return false;
        owner[id] = -1;
        free_list.push_back(id);
        return true;
    }
    void page_ptrs(int id, void *out[4]) const {
        const size_t d = geo.row_bytes() * page_tokens, s = geo.scale_row_bytes() * page_tokens;
        out[0] = slab.p[0] + d * id;
        out[1] = slab.p[1] + d * id;
        out[2] = slab.p[2] ? slab.p[2] + s * id : nullptr;
        out[3] = slab.p[3] ? slab.p[3] + s * id : nullptr;
    }
};

// ---- LayerKVCache (kv_cache.rs:1029-1900) ------------------------------------------------------------------
struct hs_cache {
    hs::Geometry geo;
    int max_seq_len = 0, seq_pos = 0, capacity = 0;
    // bumped whenever storage that a view's pointer tables may reference is released or replaced (growth of a contiguous
    // cache, pages returned by clear / truncate_to / offload, restore); a view records it per cache and compares
    unsigned long long generation = 1;
    hs::Slab slab;              // contiguous storage
    hs_pool *pool = nullptr;    // paged storage
    int64_t owner = 0;
    std::vector<int> blocks;

    int page_tokens() const { return pool ? pool->page_tokens : std::max(capacity, 1); }

    int32_t reserve(int end_pos) {
        using namespace hs;
        if (pool) {
            const int need = (end_pos + pool->page_tokens - 1) / pool->page_tokens;
            std::vector<int> got;
            while (static_cast<int>(blocks.size() + got.size()) < need) {
                const int id = pool->allocate(owner);
                if (id < 0) {
                    for (int b : got) pool->release(owner, b);  // nothing leaks (kv_cache.rs:1462-1470)
                    return fail(HS_ERR_POOL_EXHAUSTED, "block pool exhausted (%d blocks in use)", pool->n_blocks);
                }
                got.push_back(id);
            }
            blocks.insert(blocks.end(), got.begin(), got.end());
            capacity = static_cast<int>(blocks.size()) * pool->page_tokens;
            return HS_OK;
        }
        if (end_pos <= capacity) return HS_OK;
        // whole growth chunks, capped at max_seq_len rounded up to 32 tokens: the storage may hold a few tokens more than
        // the cache may use (update() still refuses positions past max_seq_len), so that every view cuts into pages of a
        // multiple of 32 tokens, which the tensor-core decode kernel's tiles need
        const int new_cap = std::min((max_seq_len + 31) / 32 * 32, (end_pos + kDefaultChunk - 1) / kDefaultChunk * kDefaultChunk);
        Slab grown;
        if (int32_t st = grown.allocate(geo, new_cap)) return st;
        // writes to the old slab may be in flight on any stream: wait for the device before copying it (growth is rare)
        if (slab.p[0]) {
            cudaError_t es = cudaDeviceSynchronize();
            if (es != cudaSuccess) {
                grown.release();
                return fail(static_cast<int32_t>(es), "cache growth: %s", cudaGetErrorString(es));
            }
        }
        for (int i = 0; i < 4; ++i) {
            if (!grown.p[i]) continue;
            cudaError_t e = cudaSuccess;
            if (slab.p[i]) e = cudaMemcpy(grown.p[i], slab.p[i], slab.bytes[i], cudaMemcpyDeviceToDevice);
            if (e == cudaSuccess) e = cudaMemset(grown.p[i] + slab.bytes[i], 0, grown.bytes[i] - slab.bytes[i]);
            if (e != cudaSuccess) {
                grown.release();
                return fail(static_cast<int32_t>(e), "cache growth: %s", cudaGetErrorString(e));
            }
        }
        if (slab.p[0]) ++generation;  // views built on the old slab are stale
        slab.release();
        slab = grown;
        capacity = new_cap;
        return HS_OK;
    }
    void release_pages(size_t keep) {
        if (!pool) return;
        if (keep < blocks.size()) ++generation;
        for (size_t i = keep; i < blocks.size(); ++i) pool->release(owner, blocks[i]);
        blocks.resize(std::min(keep, blocks.size()));
        capacity = static_cast<int>(blocks.size()) * pool->page_tokens;
    }
    // page rows of this cache cut into pages of `pt` tokens (pt divides the capacity for contiguous storage)
    void page_rows(int pt, std::vector<void *> rows[4]) const {
        if (pool) {
            for (int b : blocks) {
                void *ptrs[4];
                pool->page_ptrs(b, ptrs);
                for (int a = 0; a < 4; ++a) rows[a].push_back(ptrs[a]);
            }
            return;
        }
        if (capacity == 0) return;
        const size_t d = geo.row_bytes() * pt, s = geo.scale_row_bytes() * pt;
        for (int j = 0; j < capacity / pt; ++j) {
            rows[0].push_back(slab.p[0] + d * j);
            rows[1].push_back(slab.p[1] + d * j);
            rows[2].push_back(slab.p[2] ? slab.p[2] + s * j : nullptr);
            rows[3].push_back(slab.p[3] ? slab.p[3] + s * j : nullptr);
        }
    }
};

struct hs_view {
    hs_kv_view view{};
    void **table = nullptr;  // device: [4][n][pages_per_seq]
    std::vector<const hs_cache *> caches;           // the caches the tables were built from ...
    std::vector<unsigned long long> generations;    // ... and their generation at that time
    std::vector<int> capacities;                    // a paged cache that grew has pages the tables do not list
};

using namespace hs;

static int32_t build_view(hs_cache *const *caches, int n, hs_view *out) {
    if (!caches || n <= 0) return fail(HS_ERR_ARG, "hs_view_create: no caches");
    const hs_cache *c0 = caches[0];
    if (!c0) return fail(HS_ERR_ARG, "hs_view_create: NULL cache");
    int pt = 0;
    for (int i = 0; i < n; ++i) {
        if (!caches[i]) return fail(HS_ERR_ARG, "hs_view_create: NULL cache");
        if (!caches[i]->geo.same(c0->geo) || (caches[i]->pool != nullptr) != (c0->pool != nullptr))
            return fail(HS_ERR_ARG, "hs_view_create: caches of one batch must share geometry and storage kind");
        if (c0->pool) {
            if (caches[i]->pool->page_tokens != c0->pool->page_tokens) return fail(HS_ERR_ARG, "hs_view_create: page sizes differ");
            pt = c0->pool->page_tokens;
        } else {
            pt = std::gcd(pt, std::max(caches[i]->capacity, 1));  // contiguous caches of different capacities: common page size
        }
    }
    std::vector<std::vector<void *>> rows(4 * static_cast<size_t>(n));
    size_t pps = 1;
    for (int i = 0; i < n; ++i) {
        std::vector<void *> r[4];
        caches[i]->page_rows(pt, r);
        pps = std::max(pps, r[0].size());
        for (int a = 0; a < 4; ++a) rows[static_cast<size_t>(a) * n + i] = std::move(r[a]);
    }
    std::vector<void *> host(4 * static_cast<size_t>(n) * pps, nullptr);
    for (int a = 0; a < 4; ++a)
        for (int i = 0; i < n; ++i) {
            const auto &r = rows[static_cast<size_t>(a) * n + i];
            std::copy(r.begin(), r.end(), host.begin() + (static_cast<size_t>(a) * n + i) * pps);
        }
    out->table = static_cast<void **>(g_alloc(host.size() * sizeof(void *)));
    if (!out->table) return fail(static_cast<int32_t>(cudaErrorMemoryAllocation), "hs_view_create: device allocation failed");
    cudaError_t e = cudaMemcpy(out->table, host.data(), host.size() * sizeof(void *), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
        g_free(out->table);
        out->table = nullptr;
        return fail(static_cast<int32_t>(e), "hs_view_create: %s", cudaGetErrorString(e));
    }
    hs_kv_view &v = out->view;
    v.kind = c0->geo.kind; v.scale_dtype = c0->geo.scale_dtype; v.block = c0->geo.block;
    v.n_kv_heads = c0->geo.n_kv_heads; v.head_dim = c0->geo.head_dim;
    v.page_tokens = pt; v.pages_per_seq = static_cast<int32_t>(pps); v.reserved = 0;
    const size_t stride = static_cast<size_t>(n) * pps;
    v.k_pages = out->table; v.v_pages = out->table + stride;
    v.k_scale_pages = v.kind == HS_KV_BF16 ? nullptr : out->table + 2 * stride;
    v.v_scale_pages = v.kind == HS_KV_BF16 ? nullptr : out->table + 3 * stride;
    out->caches.assign(caches, caches + n);
    out->generations.resize(n);
    out->capacities.resize(n);
    for (int i = 0; i < n; ++i) {
        out->generations[i] = caches[i]->generation;
        out->capacities[i] = caches[i]->capacity;
    }
    return HS_OK;
}

extern "C" {

int32_t hs_host_set_allocator(hs_alloc_fn alloc_fn, hs_free_fn free_fn) {
    if ((alloc_fn == nullptr) != (free_fn == nullptr)) return fail(HS_ERR_ARG, "hs_host_set_allocator: give both functions or neither");
    g_alloc = alloc_fn ? alloc_fn : default_alloc;
    g_free = free_fn ? free_fn : default_free;
    return HS_OK;
}

int32_t hs_pool_create(int32_t n_blocks, int32_t page_tokens, int32_t kind, int32_t block, int32_t scale_dtype, int32_t n_kv_heads,
                       int32_t head_dim, hs_pool **out) {
    if (!out) return fail(HS_ERR_ARG, "hs_pool_create: NULL output");
    *out = nullptr;
    if (n_blocks <= 0 || page_tokens <= 0) return fail(HS_ERR_ARG, "hs_pool_create: n_blocks and page_tokens must be positive");
    Geometry g{kind, block, scale_dtype, n_kv_heads, head_dim};
    if (int32_t st = check_geometry(g, "hs_pool_create")) return st;
    hs_pool *p = new hs_pool();
    p->geo = g; p->page_tokens = page_tokens; p->n_blocks = n_blocks;
    if (int32_t st = p->slab.allocate(g, n_blocks * page_tokens)) { delete p; return st; }
    for (int i = 0; i < 4; ++i)
        if (p->slab.p[i]) cudaMemset(p->slab.p[i], 0, p->slab.bytes[i]);
    for (int i = n_blocks - 1; i >= 0; --i) p->free_list.push_back(i);
    p->owner.assign(n_blocks, -1);
    *out = p;
    return HS_OK;
}
// The pool's storage goes when the handle and every cache created from it are gone, whichever is dropped last.
static void pool_unref(hs_pool *pool) {
    if (!pool || pool->refs.fetch_sub(1, std::memory_order_acq_rel) != 1) return;
    pool->slab.release();
    delete pool;
}
void hs_pool_destroy(hs_pool *pool) { pool_unref(pool); }
int32_t hs_pool_num_free(const hs_pool *pool) { return pool ? static_cast<int32_t>(pool->free_list.size()) : 0; }

int32_t hs_cache_create(int32_t max_seq_len, int32_t kind, int32_t block, int32_t scale_dtype, int32_t n_kv_heads, int32_t head_dim,
                        hs_cache **out) {
    if (!out) return fail(HS_ERR_ARG, "hs_cache_create: NULL output");
    *out = nullptr;
    if (max_seq_len <= 0) return fail(HS_ERR_ARG, "hs_cache_create: max_seq_len must be positive");
    Geometry g{kind, block, scale_dtype, n_kv_heads, head_dim};
    if (int32_t st = check_geometry(g, "hs_cache_create")) return st;
    hs_cache *c = new hs_cache();
    c->geo = g; c->max_seq_len = max_seq_len;
    *out = c;
    return HS_OK;
}
int32_t hs_cache_create_paged(int32_t max_seq_len, hs_pool *pool, int64_t owner, hs_cache **out) {
    if (!out) return fail(HS_ERR_ARG, "hs_cache_create_paged: NULL output");
    *out = nullptr;
    if (!pool || max_seq_len <= 0 || owner < 0) return fail(HS_ERR_ARG, "hs_cache_create_paged: bad arguments");
    hs_cache *c = new hs_cache();
    c->geo = pool->geo; c->max_seq_len = max_seq_len; c->pool = pool; c->owner = owner;
    pool->refs.fetch_add(1, std::memory_order_relaxed);
    *out = c;
    return HS_OK;
}
void hs_cache_destroy(hs_cache *cache) {
    if (!cache) return;
    cache->release_pages(0);
    cache->slab.release();
    pool_unref(cache->pool);
    delete cache;
}
int32_t hs_cache_reserve(hs_cache *cache, int32_t n_tokens) {
    if (!cache || n_tokens < 0) return fail(HS_ERR_ARG, "hs_cache_reserve: bad arguments");
    if (n_tokens > cache->max_seq_len) return fail(HS_ERR_CACHE_OVERFLOW, "hs_cache_reserve: %d tokens exceed max_seq_len %d", n_tokens, cache->max_seq_len);
    return cache->reserve(n_tokens);
}

int32_t hs_cache_update(hs_cache *cache, const void *k_new, const void *v_new, int32_t n_tokens, int32_t start_pos, const void *sin,
                        const void *cos, int32_t rotary_dim, int32_t n_positions, hs_stream_t stream) {
    if (!cache || n_tokens < 0 || start_pos < 0) return fail(HS_ERR_ARG, "hs_cache_update: bad arguments");
    const int end_pos = start_pos + n_tokens;
    if (end_pos > cache->max_seq_len)
        return fail(HS_ERR_CACHE_OVERFLOW, "Cache overflow: trying to cache %d tokens starting at position %d, but max_seq_len is %d", n_tokens,
                    start_pos, cache->max_seq_len);
    if (n_tokens == 0) return HS_OK;
    if (int32_t st = cache->reserve(end_pos)) return st;
    hs_view v;
    hs_cache *one[1] = {cache};
    if (int32_t st = build_view(one, 1, &v)) return st;
    int32_t *pos_dev = static_cast<int32_t *>(g_alloc(sizeof(int32_t)));
    int32_t st = pos_dev ? HS_OK : fail(static_cast<int32_t>(cudaErrorMemoryAllocation), "hs_cache_update: device allocation failed");
    if (st == HS_OK) {
        cudaError_t e = cudaMemcpyAsync(pos_dev, &start_pos, sizeof(int32_t), cudaMemcpyHostToDevice, as_stream(stream));
        if (e != cudaSuccess) st = fail(static_cast<int32_t>(e), "hs_cache_update: %s", cudaGetErrorString(e));
    }
    if (st == HS_OK) st = hs_kv_quantize_write(&v.view, k_new, v_new, 1, n_tokens, pos_dev, sin, cos, rotary_dim, n_positions, stream);
    // the pointer table and the position word must outlive the launch: wait for it before releasing them
    cudaError_t e = cudaStreamSynchronize(as_stream(stream));
    if (st == HS_OK && e != cudaSuccess) st = fail(static_cast<int32_t>(e), "hs_cache_update: %s", cudaGetErrorString(e));
    if (pos_dev) g_free(pos_dev);
    if (v.table) g_free(v.table);
    if (st == HS_OK) cache->seq_pos = end_pos;
    return st;
}

int32_t hs_cache_get(hs_cache *cache, void *k_out, void *v_out, hs_stream_t stream) {
    if (!cache || !k_out || !v_out) return fail(HS_ERR_ARG, "hs_cache_get: bad arguments");
    if (cache->seq_pos == 0) return fail(HS_ERR_CACHE_EMPTY, "Cache is empty");
    hs_view v;
    hs_cache *one[1] = {cache};
    if (int32_t st = build_view(one, 1, &v)) return st;
    int32_t *len_dev = static_cast<int32_t *>(g_alloc(sizeof(int32_t)));
    int32_t st = len_dev ? HS_OK : fail(static_cast<int32_t>(cudaErrorMemoryAllocation), "hs_cache_get: device allocation failed");
    if (st == HS_OK) {
        cudaError_t e = cudaMemcpyAsync(len_dev, &cache->seq_pos, sizeof(int32_t), cudaMemcpyHostToDevice, as_stream(stream));
        if (e != cudaSuccess) st = fail(static_cast<int32_t>(e), "hs_cache_get: %s", cudaGetErrorString(e));
    }
    if (st == HS_OK) st = hs_kv_gather_dequantize(&v.view, len_dev, 1, cache->seq_pos, k_out, v_out, stream);
    cudaError_t e = cudaStreamSynchronize(as_stream(stream));
    if (st == HS_OK && e != cudaSuccess) st = fail(static_cast<int32_t>(e), "hs_cache_get: %s", cudaGetErrorString(e));
    if (len_dev) g_free(len_dev);
    if (v.table) g_free(v.table);
    return st;
}

int32_t hs_cache_clear(hs_cache *cache) {
    if (!cache) return fail(HS_ERR_ARG, "hs_cache_clear: NULL cache");
    cache->seq_pos = 0;
    cache->release_pages(0);
    return HS_OK;
}
int32_t hs_cache_truncate_to(hs_cache *cache, int32_t n_tokens) {
    if (!cache || n_tokens < 0) return fail(HS_ERR_ARG, "hs_cache_truncate_to: bad arguments");
    if (n_tokens >= cache->seq_pos) return HS_OK;
    cache->seq_pos = n_tokens;
    if (cache->pool) cache->release_pages((n_tokens + cache->pool->page_tokens - 1) / cache->pool->page_tokens);
    return HS_OK;
}
int32_t hs_cache_seq_pos(const hs_cache *cache) { return cache ? cache->seq_pos : 0; }
int32_t hs_cache_set_seq_pos(hs_cache *cache, int32_t n_tokens) {
    if (!cache || n_tokens < 0 || n_tokens > cache->capacity) return fail(HS_ERR_ARG, "hs_cache_set_seq_pos: position outside the reserved capacity");
    cache->seq_pos = n_tokens;
    return HS_OK;
}
int32_t hs_cache_capacity(const hs_cache *cache) { return cache ? cache->capacity : 0; }
int32_t hs_cache_num_pages(const hs_cache *cache) { return cache ? static_cast<int32_t>(cache->blocks.size()) : 0; }
int64_t hs_cache_memory_usage(const hs_cache *cache) {
    if (!cache) return 0;
    if (cache->pool) {
        const size_t per = 2 * (cache->geo.row_bytes() + cache->geo.scale_row_bytes()) * cache->pool->page_tokens;
        return static_cast<int64_t>(per * cache->blocks.size());
    }
    return static_cast<int64_t>(cache->slab.total());
}

// ---- CPU offload / restore (LayerKVCache::to_device, kv_cache.rs:1838-1858) ----
// The reference moves full-precision K/V to the other device and does nothing for quantised (already on the host
// there) and paged storage ("use block pool eviction instead").  Here every kind lives in HBM, so every kind can be
// parked in host memory: the used rows go out as [K data][V data][K scales][V scales], the device storage (or the
// pages) is released, and restore brings the same bytes back - codes and scales are never re-quantised.
int64_t hs_cache_offload_bytes(const hs_cache *cache) {
    if (!cache) return 0;
    return static_cast<int64_t>(2 * (cache->geo.row_bytes() + cache->geo.scale_row_bytes())) * cache->seq_pos;
}

// copies `n` token rows of all four arrays between the cache's storage and a packed host image
static int32_t copy_rows(hs_cache *cache, unsigned char *host, int n, bool to_host, cudaStream_t s, const char *who) {
    const size_t row[4] = {cache->geo.row_bytes(), cache->geo.row_bytes(), cache->geo.scale_row_bytes(), cache->geo.scale_row_bytes()};
    const int pt = cache->pool ? cache->pool->page_tokens : std::max(cache->capacity, 1);
    std::vector<void *> rows[4];
    cache->page_rows(pt, rows);
    size_t off = 0;
    for (int a = 0; a < 4; ++a) {
        if (row[a] == 0) continue;
        for (int t0 = 0, page = 0; t0 < n; t0 += pt, ++page) {
            const size_t bytes = row[a] * static_cast<size_t>(std::min(pt, n - t0));
            unsigned char *dev = static_cast<unsigned char *>(rows[a][page]);
            cudaError_t e = to_host ? cudaMemcpyAsync(host + off, dev, bytes, cudaMemcpyDeviceToHost, s)
                                    : cudaMemcpyAsync(dev, host + off, bytes, cudaMemcpyHostToDevice, s);
            if (e != cudaSuccess) return fail(static_cast<int32_t>(e), "%s: %s", who, cudaGetErrorString(e));
            off += bytes;
        }
    }
    cudaError_t e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return fail(static_cast<int32_t>(e), "%s: %s", who, cudaGetErrorString(e));
    return HS_OK;
}

int32_t hs_cache_offload(hs_cache *cache, void *host_buf, int64_t host_bytes, hs_stream_t stream) {
    if (!cache || (!host_buf && cache->seq_pos > 0)) return fail(HS_ERR_ARG, "hs_cache_offload: bad arguments");
    if (host_bytes < hs_cache_offload_bytes(cache))
        return fail(HS_ERR_ARG, "hs_cache_offload: host buffer of %lld bytes, %lld needed", static_cast<long long>(host_bytes),
                    static_cast<long long>(hs_cache_offload_bytes(cache)));
    if (cache->seq_pos > 0)
        if (int32_t st = copy_rows(cache, static_cast<unsigned char *>(host_buf), cache->seq_pos, true, as_stream(stream), "hs_cache_offload")) return st;
    cache->seq_pos = 0;
    cache->release_pages(0);
    if (cache->slab.p[0]) ++cache->generation;
    cache->slab.release();
    if (!cache->pool) cache->capacity = 0;
    return HS_OK;
}

int32_t hs_cache_snapshot(const hs_cache *cache, void *host_buf, int64_t host_bytes, hs_stream_t stream) {
    if (!cache || (!host_buf && cache->seq_pos > 0)) return fail(HS_ERR_ARG, "hs_cache_snapshot: bad arguments");
    if (host_bytes < hs_cache_offload_bytes(cache))
        return fail(HS_ERR_ARG, "hs_cache_snapshot: host buffer of %lld bytes, %lld needed", static_cast<long long>(host_bytes),
                    static_cast<long long>(hs_cache_offload_bytes(cache)));
    if (cache->seq_pos == 0) return HS_OK;
    return copy_rows(const_cast<hs_cache *>(cache), static_cast<unsigned char *>(host_buf), cache->seq_pos, true, as_stream(stream), "hs_cache_snapshot");
}

int32_t hs_cache_restore(hs_cache *cache, const void *host_buf, int64_t host_bytes, int32_t n_tokens, hs_stream_t stream) {
    if (!cache || n_tokens < 0 || (!host_buf && n_tokens > 0)) return fail(HS_ERR_ARG, "hs_cache_restore: bad arguments");
    if (cache->seq_pos != 0) return fail(HS_ERR_ARG, "hs_cache_restore: the cache holds %d tokens; clear it first", cache->seq_pos);
    if (n_tokens > cache->max_seq_len)
        return fail(HS_ERR_CACHE_OVERFLOW, "hs_cache_restore: %d tokens exceed max_seq_len %d", n_tokens, cache->max_seq_len);
    const int64_t need = static_cast<int64_t>(2 * (cache->geo.row_bytes() + cache->geo.scale_row_bytes())) * n_tokens;
    if (host_bytes < need)
        return fail(HS_ERR_ARG, "hs_cache_restore: host image of %lld bytes, %lld needed", static_cast<long long>(host_bytes), static_cast<long long>(need));
    if (n_tokens == 0) return HS_OK;
    if (int32_t st = cache->reserve(n_tokens)) return st;
    if (int32_t st = copy_rows(cache, const_cast<unsigned char *>(static_cast<const unsigned char *>(host_buf)), n_tokens, false, as_stream(stream),
                               "hs_cache_restore"))
        return st;
    cache->seq_pos = n_tokens;
    return HS_OK;
}

int32_t hs_view_create(hs_cache *const *caches, int32_t n_caches, hs_view **out) {
    if (!out) return fail(HS_ERR_ARG, "hs_view_create: NULL output");
    *out = nullptr;
    hs_view *v = new hs_view();
    if (int32_t st = build_view(caches, n_caches, v)) { delete v; return st; }
    *out = v;
    return HS_OK;
}
const hs_kv_view *hs_view_get(const hs_view *view) { return view ? &view->view : nullptr; }
int32_t hs_view_is_current(const hs_view *view) {
    if (!view) return fail(HS_ERR_ARG, "hs_view_is_current: NULL view");
    for (size_t i = 0; i < view->caches.size(); ++i) {
        const hs_cache *c = view->caches[i];
        if (c->generation != view->generations[i])
            return fail(HS_ERR_ARG, "hs_view_is_current: cache %zu released or replaced storage after the view was built (growth, clear, "
                                    "truncate_to, offload); build a new view", i);
        if (c->capacity != view->capacities[i])
            return fail(HS_ERR_ARG, "hs_view_is_current: cache %zu changed capacity (%d -> %d tokens) after the view was built; its new pages "
                                    "are not in the view's tables", i, view->capacities[i], c->capacity);
    }
    return HS_OK;
}
void hs_view_destroy(hs_view *view) {
    if (!view) return;
    if (view->table) g_free(view->table);
    delete view;
}

}  // extern "C"
