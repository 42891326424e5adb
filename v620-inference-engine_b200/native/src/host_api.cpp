// C ABI of the native host runtime (libqw_host.so): n-gram ids, PLE table, safetensors, block store
// with disk tier, host sampler, chunker, thread pool.  Used from Python through ctypes and from the
// C API shim.  Functions return 0 / a count on success and -1 on error (message via qwh_last_error).
#include <sys/stat.h>

#include <algorithm>

#include "block_store.hpp"
#include "chunker.hpp"
#include "ngram_ple.hpp"
#include "sampler.hpp"
#include "slot_logic.hpp"
#include "spec_planner.hpp"

using namespace qwh;

static thread_local std::string g_err;
#include "pinned_pool.hpp"
#define API extern "C" __attribute__((visibility("default")))
#define GUARD(body, bad)                              \
    try { body } catch (const std::exception &e) {    \
        g_err = e.what();                             \
        return bad;                                   \
    }

API const char *qwh_last_error() { return g_err.c_str(); }

// ---- n-gram ids
API void *qwh_ngram_new(int vocab, int eos, int ngram, int heads, long long vocab_base, unsigned long long seed, int image_pad,
                        int video_pad) {
    GUARD(NgramSpec s; s.vocab = vocab; s.eos = eos; s.ngram = ngram; s.heads = heads; s.vocab_base = vocab_base; s.seed = seed;
          s.image_pad = image_pad; s.video_pad = video_pad; return new NgramHasher(s);, nullptr)
}
API void qwh_ngram_free(void *h) { delete static_cast<NgramHasher *>(h); }
API long long qwh_ngram_total_rows(void *h) { return static_cast<NgramHasher *>(h)->total_rows(); }
API int qwh_ngram_sizes(void *h, long long *sizes, long long *offsets, unsigned long long *mult) {
    auto *n = static_cast<NgramHasher *>(h);
    for (size_t i = 0; i < n->sizes().size(); ++i) { sizes[i] = n->sizes()[i]; offsets[i] = n->offsets()[i]; }
    for (size_t i = 0; i < n->mult().size(); ++i) mult[i] = n->mult()[i];
    return int(n->sizes().size());
}
API int qwh_ngram_ids(void *h, const int32_t *hist, int n_hist, const int32_t *tokens, int n, long long *ids) {
    GUARD(static_cast<NgramHasher *>(h)->ids_for(hist, n_hist, tokens, n, reinterpret_cast<int64_t *>(ids)); return 0;, -1)
}

// ---- thread pool
API void *qwh_pool_new(int threads) { return new ThreadPool(threads); }
API void qwh_pool_free(void *p) { delete static_cast<ThreadPool *>(p); }
API int qwh_pool_size(void *p) { return static_cast<ThreadPool *>(p)->size(); }
// Self check: `rounds` loops over [0, n) in pieces of at least `grain`; every index must be visited exactly once per loop
// and no piece may be shorter than it has to be.  Returns the number of violations seen.
API long long qwh_pool_check(void *p, long long n, long long grain, int rounds) {
    ThreadPool &pool = *static_cast<ThreadPool *>(p);
    std::vector<unsigned char> hits(size_t(n > 0 ? n : 0));
    long long bad = 0;
    for (int r = 0; r < rounds; ++r) {
        std::fill(hits.begin(), hits.end(), 0);
        std::atomic<long long> pieces{0}, wrong{0};
        pool.parallel_for(n, grain, [&](int64_t lo, int64_t hi) {
            if (lo < 0 || hi > n || lo >= hi) wrong.fetch_add(1);
            for (int64_t i = lo; i < hi && i < n; ++i) ++hits[size_t(i)];
            pieces.fetch_add(1);
        });
        bad += wrong.load();
        for (unsigned char h : hits) bad += h != 1;
        if (n > 0 && (pieces.load() < 1 || pieces.load() > (long long)pool.size() * 4)) ++bad;
    }
    return bad;
}

// ---- PLE table
API void *qwh_ple_open(const char *dir, int width) { GUARD(return new PleTable(dir, width);, nullptr) }
API void qwh_ple_free(void *t) { delete static_cast<PleTable *>(t); }
API long long qwh_ple_rows(void *t) { return static_cast<PleTable *>(t)->rows(); }
API int qwh_ple_layout(void *t) { return int(static_cast<PleTable *>(t)->layout()); }
API int qwh_ple_gather(void *t, const long long *ids, int T, int heads, float *out, void *pool) {
    GUARD(static_cast<PleTable *>(t)->gather(reinterpret_cast<const int64_t *>(ids), T, heads, out, static_cast<ThreadPool *>(pool)); return 0;, -1)
}
API int qwh_ple_pin(void *t, int lock, int wait) {
    GUARD(auto *p = static_cast<PleTable *>(t); p->pin_in_background(lock != 0); if (wait) p->wait_pinned(); return 0;, -1)
}

// ---- safetensors
API void *qwh_st_open(const char *path) { GUARD(auto *s = new SafeTensors(); s->add_file(path); return s;, nullptr) }
API int qwh_st_add(void *s, const char *path) { GUARD(static_cast<SafeTensors *>(s)->add_file(path); return 0;, -1) }
API void qwh_st_free(void *s) { delete static_cast<SafeTensors *>(s); }
API int qwh_st_count(void *s) { return int(static_cast<SafeTensors *>(s)->count()); }
API int qwh_st_info(void *s, const char *name, int *dtype, long long *shape, int *ndim, const void **data, unsigned long long *nbytes) {
    GUARD(const TensorView &t = static_cast<SafeTensors *>(s)->get(name); *dtype = int(t.dtype); *ndim = int(t.shape.size());
          for (size_t i = 0; i < t.shape.size() && i < 8; ++i) shape[i] = t.shape[i]; *data = t.data; *nbytes = t.nbytes; return 0;, -1)
}

// ---- block store
API void *qwh_store_new(unsigned long long layout, unsigned ranks, unsigned long long ram_budget, const char *disk_dir,
                        unsigned long long disk_budget) {
    GUARD(return new BlockStore(layout, ranks, size_t(ram_budget), disk_dir ? disk_dir : "", size_t(disk_budget));, nullptr)
}
API void qwh_store_free(void *s) { delete static_cast<BlockStore *>(s); }
API unsigned long long qwh_store_root() { return STORE_ROOT; }
API unsigned long long qwh_block_key(unsigned long long parent, const int32_t *t, int n) { return block_key(parent, t, size_t(n)); }
API unsigned long long qwh_store_save_block(void *s, unsigned long long parent, long long start, const int32_t *tokens, int n,
                                            const void *kv, unsigned long long bytes) {
    GUARD(return static_cast<BlockStore *>(s)->save_block(parent, start, tokens, n, kv, size_t(bytes));, 0)
}
API int qwh_store_save_snapshot(void *s, unsigned long long key, const void *snap, unsigned long long bytes, const float *logits,
                                int nlogits, int anchor) {
    GUARD(return static_cast<BlockStore *>(s)->save_snapshot(key, snap, size_t(bytes), logits, nlogits, anchor != 0) ? 0 : -1;, -1)
}
API int qwh_store_lookup(void *s, const int32_t *tokens, long long n, unsigned long long *keys, int max_keys, int *snap_depth) {
    GUARD(auto path = static_cast<BlockStore *>(s)->lookup(tokens, n, snap_depth);
          const int m = std::min<int>(int(path.size()), max_keys); for (int i = 0; i < m; ++i) keys[i] = path[size_t(i)]; return m;, -1)
}
// size query (out == null) or copy; returns the payload size, -1 when the payload is gone
API long long qwh_store_get(void *s, unsigned long long key, int snap, void *out, unsigned long long cap, float *logits, int max_logits,
                            int *nlogits) {
    GUARD(std::vector<uint8_t> buf; std::vector<float> lg;
          bool ok = snap ? static_cast<BlockStore *>(s)->get_snapshot(key, buf, &lg) : static_cast<BlockStore *>(s)->get_kv(key, buf);
          if (!ok) return -1;
          if (out && cap >= buf.size()) std::memcpy(out, buf.data(), buf.size());
          if (nlogits) *nlogits = int(lg.size());
          if (logits) std::memcpy(logits, lg.data(), sizeof(float) * std::min<size_t>(lg.size(), size_t(max_logits)));
          return (long long)buf.size();, -1)
}
API int qwh_store_block_info(void *s, unsigned long long key, long long *start, int *ntok, int *has_snap, int *in_ram, int *on_disk) {
    const BlockStore::Node *n = static_cast<BlockStore *>(s)->find(key);
    if (!n) return -1;
    *start = n->start; *ntok = int(n->tokens.size()); *has_snap = n->has_snap; *in_ram = !n->kv.empty(); *on_disk = n->kv_disk;
    return 0;
}
API void qwh_store_note_restore(void *s, unsigned long long key, long long tokens) { static_cast<BlockStore *>(s)->note_restore(key, tokens); }
API int qwh_store_prefetch(void *s, const unsigned long long *keys, int n, int last_snapshot) {
    return static_cast<BlockStore *>(s)->prefetch(reinterpret_cast<const uint64_t *>(keys), n, last_snapshot != 0);
}
API int qwh_store_loads_pending(void *s) { return static_cast<BlockStore *>(s)->loads_pending(); }
API void qwh_store_flush(void *s) { static_cast<BlockStore *>(s)->flush(); }
API int qwh_store_thin(void *s, long long gap) { return static_cast<BlockStore *>(s)->thin(gap); }
API void qwh_store_stats(void *s, unsigned long long *out7) {
    const StoreStats st = static_cast<BlockStore *>(s)->stats();
    out7[0] = st.hits; out7[1] = st.tokens_restored; out7[2] = st.snapshots_saved; out7[3] = st.ram_bytes;
    out7[4] = st.disk_bytes; out7[5] = st.blocks; out7[6] = st.snapshots;
}

// ---- sampler
struct qwh_sampling {
    float temperature, top_p;
    int32_t top_k;
    float min_p, presence_penalty, frequency_penalty, repetition_penalty;
    uint64_t seed;
};
API void *qwh_rng_new(unsigned long long seed) { return new std::mt19937_64(seed); }
API void qwh_rng_free(void *r) { delete static_cast<std::mt19937_64 *>(r); }
API int qwh_sample(const float *logits, int V, const qwh_sampling *p, const int32_t *hist, long long n_hist, long long prompt_end,
                   void *rng, float *logprob) {
    GUARD(SamplingParams sp; sp.temperature = p->temperature; sp.top_p = p->top_p; sp.top_k = p->top_k; sp.min_p = p->min_p;
          sp.presence_penalty = p->presence_penalty; sp.frequency_penalty = p->frequency_penalty;
          sp.repetition_penalty = p->repetition_penalty; sp.seed = p->seed;
          return sample_token(logits, V, sp, hist, size_t(n_hist), size_t(prompt_end), *static_cast<std::mt19937_64 *>(rng), logprob);, -1)
}
API void qwh_sampler_full_sort(int on) { sampler_full_sort_flag() = on; }
API int qwh_top_logprobs(const float *logits, int V, int k, int32_t *ids, float *lps) { return top_logprobs(logits, V, k, ids, lps); }
API float qwh_lse(const float *logits, int V) { return log_sum_exp(logits, V); }

// ---- slot and prompt decisions
API int qwh_choose_slot(int n, const unsigned char *busy, const long long *capacity, const long long *kept, const long long *used, long long need) {
    return choose_slot(n, busy, reinterpret_cast<const int64_t *>(capacity), reinterpret_cast<const int64_t *>(kept),
                       reinterpret_cast<const int64_t *>(used), need);
}
API int qwh_start_way(long long keep, long long snapshot, long long stored) { return start_way(keep, snapshot, stored); }
API long long qwh_capture_point(const int32_t *prompt, long long n, long long done, long long end, long long last_capture, int boundary, long long min_gap) {
    return capture_point(prompt, n, done, end, last_capture, boundary, min_gap);
}
API int qwh_best_snapshot(int m, const long long *snap_n, const unsigned char *has_logits, long long common, long long prompt_len) {
    return best_snapshot(m, reinterpret_cast<const int64_t *>(snap_n), has_logits, common, prompt_len);
}

// ---- speculative-step planner
API void *qwh_spec_new(int slots, double base, double beta, double probe_accept, int plain_first, int plain_grow, int plain_max) {
    return new SpecPlanner(slots, SpecTuning{base, beta, probe_accept, plain_first, plain_grow, plain_max});
}
API void qwh_spec_free(void *h) { delete static_cast<SpecPlanner *>(h); }
API void *qwh_spec_slots(void *h) { return static_cast<SpecPlanner *>(h)->slots(); }
API int qwh_spec_draft_count(void *h, int slot, int k_max) { return static_cast<SpecPlanner *>(h)->draft_count(slot, k_max); }
API double qwh_spec_best_rate(void *h, double a, int k_max, int *k) {
    double r;
    static_cast<SpecPlanner *>(h)->best_rate(a, k_max, &r, k);
    return r;
}
API int qwh_spec_plan(void *h, int n, const int32_t *slot, const long long *budget, const long long *room, const unsigned char *can_draft, int k,
                      int max_drafts, int max_run, int max_rows, int forced, int32_t *want, int *bad) {
    return static_cast<SpecPlanner *>(h)->plan(n, slot, reinterpret_cast<const int64_t *>(budget), reinterpret_cast<const int64_t *>(room), can_draft, k,
                                              max_drafts, max_run, max_rows, forced, want, bad);
}
API int qwh_spec_note_plain_step(void *h, int slot) { return static_cast<SpecPlanner *>(h)->note_plain_step(slot); }
API int qwh_spec_accept(void *h, int slot, const int32_t *sampled, const int32_t *drafts, int n_drafts, const int32_t *stop, int n_stop, int forced) {
    return static_cast<SpecPlanner *>(h)->accept(slot, sampled, drafts, n_drafts, stop, n_stop, forced);
}

// ---- chunker
API int qwh_chunk(const int32_t *tok, long long n, int boundary, long long *starts, long long *lens, unsigned long long *hashes, int cap) {
    auto c = chunk_prompt(tok, n, boundary);
    const int m = std::min<int>(int(c.size()), cap);
    for (int i = 0; i < m; ++i) { starts[i] = c[size_t(i)].start; lens[i] = c[size_t(i)].len; hashes[i] = c[size_t(i)].hash; }
    return int(c.size());
}

// ---- pinned pool (+ NUMA placement)
API void *qwh_pinned_new(unsigned long long unit_bytes, unsigned long long arena_bytes, int standing_units, int use_cuda, int policy,
                         int node) {
    GUARD(return new PinnedPool(size_t(unit_bytes), size_t(arena_bytes), standing_units, use_cuda != 0, NumaPolicy(policy), node);, nullptr)
}
API void qwh_pinned_free(void *p) { delete static_cast<PinnedPool *>(p); }
API void qwh_pinned_reserve(void *p, int n) { static_cast<PinnedPool *>(p)->reserve(n); }
API void *qwh_pinned_get(void *p) { GUARD(return static_cast<PinnedPool *>(p)->get();, nullptr) }
API int qwh_pinned_put(void *p, void *unit) { GUARD(static_cast<PinnedPool *>(p)->put(unit); return 0;, -1) }
API unsigned long long qwh_pinned_unit_bytes(void *p) { return static_cast<PinnedPool *>(p)->unit_bytes(); }
API void qwh_pinned_stats(void *p, long long *i5, double *d2, int *x2) {
    const PoolStats s = static_cast<PinnedPool *>(p)->stats();
    i5[0] = s.arenas; i5[1] = s.units_total; i5[2] = s.units_free; i5[3] = s.gets; i5[4] = s.waits;
    d2[0] = s.wait_seconds; d2[1] = s.pin_seconds;
    x2[0] = s.cuda_registered; x2[1] = s.numa_node;
}
API int qwh_numa_nodes() { return numa_nodes(); }
