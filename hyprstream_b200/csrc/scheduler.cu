// Continuous-batching scheduler for the batched decode step: admits sequences while the block pool has pages for them,
// defers them when it has not, plans one step at a time (prompts to prefill, the decode batch with its cache view and
// position arrays), and retires finished sequences so that their pages serve the ones that were deferred.
//
// The reference has the pieces but no loop: a batched step (torch_engine.rs:1475-1501 forward_batched_step, Llama only)
// that no production caller drives, two configuration values (config/mod.rs:2146-2152: continuous_batching, off by
// default, and continuous_batch_max, default 16), and a typed, fail-soft pool-exhaustion error whose documentation says
// what a scheduler should do with it (kv_cache.rs:482-505: "turn it into admission-defer ... retry the sequence on a
// later step once other sequences release blocks").  This file is that loop, over the host cache objects of
// kv_cache_host.cu.  It is host code; the only device work is the upload of two small integer arrays per step and the
// cache view, both skipped when a plan is asked for without device objects (the form the CPU tests drive, with a host
// allocator installed through hs_host_set_allocator and a fake step function).
#include <algorithm>
#include <deque>
#include <vector>

#include "hs_common.cuh"

struct hs_sched_seq {
    int64_t id = 0;
    int32_t prompt_len = 0, max_new_tokens = 0, generated = 0;
    bool prefilled = false;
    hs_cache *cache = nullptr;
};

struct hs_sched {
    hs_pool *pool = nullptr;
    int32_t batch_max = 16, max_seq_len = 0;
    std::deque<hs_sched_seq> waiting;     // FIFO: the head is admitted first; a deferred head blocks the ones behind it
    std::vector<hs_sched_seq> running;    // admission order
    // the current plan
    std::vector<int64_t> plan_prefill_ids, plan_decode_ids;
    std::vector<int32_t> plan_prefill_len;
    std::vector<hs_cache *> plan_prefill_caches, plan_decode_caches;
    std::vector<int32_t> host_pos, host_len;
    hs_view *view = nullptr;
    std::vector<hs_cache *> view_members;
    int32_t *dev_pos = nullptr, *dev_len = nullptr;
    int32_t dev_cap = 0;
    bool planned = false;
    // counters
    int64_t n_deferred = 0, n_stalled = 0, n_admitted = 0, n_retired = 0, n_steps = 0;
};

using namespace hs;

static void sched_drop_view(hs_sched *s) {
    if (s->view) hs_view_destroy(s->view);
    s->view = nullptr;
    s->view_members.clear();
}

extern "C" {

int32_t hs_sched_create(hs_pool *pool, int32_t continuous_batch_max, int32_t max_seq_len, hs_sched **out) {
    if (!out) return fail(HS_ERR_ARG, "hs_sched_create: NULL output");
    *out = nullptr;
    if (!pool || continuous_batch_max <= 0 || max_seq_len <= 0) return fail(HS_ERR_ARG, "hs_sched_create: a pool and positive limits are required");
    hs_sched *s = new hs_sched();
    s->pool = pool;
    s->batch_max = continuous_batch_max;
    s->max_seq_len = max_seq_len;
    *out = s;
    return HS_OK;
}

void hs_sched_destroy(hs_sched *sched) {
    if (!sched) return;
    sched_drop_view(sched);
    for (auto &q : sched->running)
        if (q.cache) hs_cache_destroy(q.cache);
    if (sched->dev_pos) cudaFree(sched->dev_pos);
    if (sched->dev_len) cudaFree(sched->dev_len);
    cudaGetLastError();
    delete sched;
}

int32_t hs_sched_submit(hs_sched *sched, int64_t seq_id, int32_t prompt_len, int32_t max_new_tokens) {
    if (!sched || prompt_len <= 0 || max_new_tokens <= 0) return fail(HS_ERR_ARG, "hs_sched_submit: a prompt and a token budget are required");
    if (seq_id < 0) return fail(HS_ERR_ARG, "hs_sched_submit: sequence ids are >= 0 (they tag the pool's pages)");
    if (prompt_len + max_new_tokens > sched->max_seq_len)
        return fail(HS_ERR_CACHE_OVERFLOW, "hs_sched_submit: %d prompt + %d new tokens exceed max_seq_len %d", prompt_len, max_new_tokens, sched->max_seq_len);
    for (const auto &q : sched->running)
        if (q.id == seq_id) return fail(HS_ERR_ARG, "hs_sched_submit: sequence %lld is running already", static_cast<long long>(seq_id));
    for (const auto &q : sched->waiting)
        if (q.id == seq_id) return fail(HS_ERR_ARG, "hs_sched_submit: sequence %lld is queued already", static_cast<long long>(seq_id));
    hs_sched_seq q;
    q.id = seq_id; q.prompt_len = prompt_len; q.max_new_tokens = max_new_tokens;
    sched->waiting.push_back(q);
    return HS_OK;
}

int32_t hs_sched_plan_step(hs_sched *sched, int32_t flags, hs_sched_plan *plan, hs_stream_t stream) {
    if (!sched || !plan) return fail(HS_ERR_ARG, "hs_sched_plan_step: NULL argument");
    if (sched->planned) return fail(HS_ERR_ARG, "hs_sched_plan_step: the previous plan was not committed");
    hs_sched &s = *sched;
    s.plan_prefill_ids.clear(); s.plan_prefill_len.clear(); s.plan_prefill_caches.clear();
    s.plan_decode_ids.clear(); s.plan_decode_caches.clear(); s.host_pos.clear(); s.host_len.clear();
    int deferred_now = 0, stalled_now = 0;
    // ---- decode batch: every running sequence that has been prefilled and gets room for its next token ----
    for (auto &q : s.running) {
        if (!q.prefilled) continue;
        const int32_t pos = hs_cache_seq_pos(q.cache);
        const int32_t st = hs_cache_reserve(q.cache, pos + 1);
        if (st == HS_ERR_POOL_EXHAUSTED) {  // no page for its next token: it sits this step out and keeps what it has
            ++stalled_now;
            continue;
        }
        if (st != HS_OK) return st;
        s.plan_decode_ids.push_back(q.id);
        s.plan_decode_caches.push_back(q.cache);
        s.host_pos.push_back(pos);
        s.host_len.push_back(pos + 1);
    }
    // ---- admission: FIFO, while the batch has room and the pool has pages for the whole prompt plus one token ----
    while (!s.waiting.empty() && static_cast<int32_t>(s.running.size()) < s.batch_max) {
        hs_sched_seq q = s.waiting.front();
        if (int32_t st = hs_cache_create_paged(s.max_seq_len, s.pool, q.id, &q.cache)) return st;
        const int32_t st = hs_cache_reserve(q.cache, q.prompt_len + 1);
        if (st == HS_ERR_POOL_EXHAUSTED) {  // fail-soft (kv_cache.rs:482-505): the sequence stays queued and is retried on a later step
            hs_cache_destroy(q.cache);      // (reserve rolled its partial allocation back)
            ++deferred_now;
            break;
        }
        if (st != HS_OK) { hs_cache_destroy(q.cache); return st; }
        s.waiting.pop_front();
        s.running.push_back(q);
        ++s.n_admitted;
        s.plan_prefill_ids.push_back(q.id);
        s.plan_prefill_len.push_back(q.prompt_len);
        s.plan_prefill_caches.push_back(q.cache);
    }
    s.n_deferred += deferred_now;
    s.n_stalled += stalled_now;
    // nothing can move and nothing will free pages: the pool is too small for what is running
    if (s.plan_decode_ids.empty() && s.plan_prefill_ids.empty() && (stalled_now > 0 || (deferred_now > 0 && s.running.empty())))
        return fail(HS_ERR_POOL_EXHAUSTED, "hs_sched_plan_step: no sequence can make progress (%d stalled, %d deferred, %d pages free)", stalled_now,
                    deferred_now, hs_pool_num_free(s.pool));
    // ---- device objects of the decode batch ----
    plan->view = nullptr; plan->dst_pos = nullptr; plan->seq_lens = nullptr;
    const int32_t nd = static_cast<int32_t>(s.plan_decode_ids.size());
    if ((flags & HS_SCHED_DEVICE_OBJECTS) && nd > 0) {
        // the view is rebuilt when the batch's membership changed or a member's pages did (a page added for this step)
        if (!s.view || s.view_members != s.plan_decode_caches || hs_view_is_current(s.view) != HS_OK) {
            sched_drop_view(&s);
            if (int32_t st = hs_view_create(s.plan_decode_caches.data(), nd, &s.view)) return st;
            s.view_members = s.plan_decode_caches;
        }
        if (nd > s.dev_cap) {
            if (s.dev_pos) cudaFree(s.dev_pos);
            if (s.dev_len) cudaFree(s.dev_len);
            s.dev_pos = s.dev_len = nullptr;
            const int32_t cap = std::max(nd, s.batch_max);
            cudaError_t e = cudaMalloc(&s.dev_pos, sizeof(int32_t) * cap);
            if (e == cudaSuccess) e = cudaMalloc(&s.dev_len, sizeof(int32_t) * cap);
            if (e != cudaSuccess) return fail(static_cast<int32_t>(e), "hs_sched_plan_step: %s", cudaGetErrorString(e));
            s.dev_cap = cap;
        }
        cudaError_t e = cudaMemcpyAsync(s.dev_pos, s.host_pos.data(), sizeof(int32_t) * nd, cudaMemcpyHostToDevice, as_stream(stream));
        if (e == cudaSuccess) e = cudaMemcpyAsync(s.dev_len, s.host_len.data(), sizeof(int32_t) * nd, cudaMemcpyHostToDevice, as_stream(stream));
        if (e == cudaSuccess) e = cudaStreamSynchronize(as_stream(stream));  // the host vectors are reused by the next plan
        if (e != cudaSuccess) return fail(static_cast<int32_t>(e), "hs_sched_plan_step: %s", cudaGetErrorString(e));
        plan->view = hs_view_get(s.view);
        plan->dst_pos = s.dev_pos;
        plan->seq_lens = s.dev_len;
    }
    plan->n_prefill = static_cast<int32_t>(s.plan_prefill_ids.size());
    plan->prefill_ids = s.plan_prefill_ids.data();
    plan->prefill_lens = s.plan_prefill_len.data();
    plan->prefill_caches = s.plan_prefill_caches.data();
    plan->n_decode = nd;
    plan->decode_ids = s.plan_decode_ids.data();
    plan->decode_caches = s.plan_decode_caches.data();
    plan->host_dst_pos = s.host_pos.data();
    plan->n_deferred = deferred_now;
    plan->n_stalled = stalled_now;
    plan->n_waiting = static_cast<int32_t>(s.waiting.size());
    plan->n_running = static_cast<int32_t>(s.running.size());
    s.planned = true;
    return HS_OK;
}

int32_t hs_sched_commit_step(hs_sched *sched, const int64_t *finished_ids, int32_t n_finished) {
    if (!sched || n_finished < 0 || (n_finished > 0 && !finished_ids)) return fail(HS_ERR_ARG, "hs_sched_commit_step: bad arguments");
    if (!sched->planned) return fail(HS_ERR_ARG, "hs_sched_commit_step: no plan to commit");
    hs_sched &s = *sched;
    // the step ran: prompts are in their caches (the host prefilled them through hs_cache_update), decoded sequences grew by one
    for (auto &q : s.running) {
        if (std::find(s.plan_prefill_ids.begin(), s.plan_prefill_ids.end(), q.id) != s.plan_prefill_ids.end()) {
            q.prefilled = true;
            if (hs_cache_seq_pos(q.cache) < q.prompt_len)  // a host that wrote through a view rather than hs_cache_update
                if (int32_t st = hs_cache_set_seq_pos(q.cache, q.prompt_len)) return st;
        }
        const auto it = std::find(s.plan_decode_ids.begin(), s.plan_decode_ids.end(), q.id);
        if (it != s.plan_decode_ids.end()) {
            const int32_t pos = s.host_pos[it - s.plan_decode_ids.begin()];
            if (int32_t st = hs_cache_set_seq_pos(q.cache, pos + 1)) return st;
            ++q.generated;
        }
    }
    // retire: the token budget is used up, or the host says the sequence ended (end-of-sequence token, client gone)
    bool any = false;
    for (auto it = s.running.begin(); it != s.running.end();) {
        const bool done = it->generated >= it->max_new_tokens ||
                          (n_finished > 0 && std::find(finished_ids, finished_ids + n_finished, it->id) != finished_ids + n_finished);
        if (!done) { ++it; continue; }
        if (!any) sched_drop_view(&s);  // the view's tables point into pages that go back to the pool now
        any = true;
        hs_cache_destroy(it->cache);    // pages return to the pool (Drop, kv_cache.rs:1889-1898)
        it = s.running.erase(it);
        ++s.n_retired;
    }
    s.planned = false;
    ++s.n_steps;
    return HS_OK;
}

int32_t hs_sched_cancel(hs_sched *sched, int64_t seq_id) {
    if (!sched) return fail(HS_ERR_ARG, "hs_sched_cancel: NULL scheduler");
    if (sched->planned) return fail(HS_ERR_ARG, "hs_sched_cancel: commit the current plan first");
    hs_sched &s = *sched;
    for (auto it = s.waiting.begin(); it != s.waiting.end(); ++it)
        if (it->id == seq_id) {
            s.waiting.erase(it);
            return HS_OK;
        }
    for (auto it = s.running.begin(); it != s.running.end(); ++it)
        if (it->id == seq_id) {
            sched_drop_view(&s);
            hs_cache_destroy(it->cache);
            s.running.erase(it);
            ++s.n_retired;
            return HS_OK;
        }
    return fail(HS_ERR_ARG, "hs_sched_cancel: sequence %lld is neither queued nor running", static_cast<long long>(seq_id));
}

int32_t hs_sched_stats(const hs_sched *sched, hs_sched_stats_t *out) {
    if (!sched || !out) return fail(HS_ERR_ARG, "hs_sched_stats: NULL argument");
    out->n_waiting = static_cast<int32_t>(sched->waiting.size());
    out->n_running = static_cast<int32_t>(sched->running.size());
    out->n_admitted = sched->n_admitted; out->n_retired = sched->n_retired;
    out->n_deferred = sched->n_deferred; out->n_stalled = sched->n_stalled; out->n_steps = sched->n_steps;
    out->pages_free = hs_pool_num_free(sched->pool);
    out->reserved = 0;
    return HS_OK;
}

}  // extern "C"
