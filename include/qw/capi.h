/* qw engine - C ABI of the library `libqw_engine.so`.
 *
 * The ABI (function names, argument order, struct layouts) is the one clients of the qw engine already
 * link against, so a host written for it (the qwserve server through ctypes, C tools) works unchanged.
 * One handle owns one engine on this node's GPUs with a fixed set of sequence slots.
 *
 * Rules common to all calls:
 *   - one thread drives a handle; calls never overlap (qw_engine_failure is the exception);
 *   - functions returning int or int64_t: a value >= 0 is success, -1 is failure and qw_error(h) then
 *     holds the reason; qw_acquire* returning -1 with an EMPTY error string means "no free slot";
 *   - token ids are int32; ids below zero stand for vision tokens inside the engine.
 */
#ifndef QW_CAPI_H
#define QW_CAPI_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct qw_handle qw_handle;

/* ---------------------------------------------------------------- plain-data structs */

/* Sampling controls of one request. */
typedef struct qw_sampling {
    float temperature;        /* 0 selects the most likely token */
    float top_p;              /* 1 disables nucleus truncation */
    int32_t top_k;            /* 0 disables the top-k cut */
    float min_p;              /* 0 disables the relative-probability floor */
    float presence_penalty;
    float frequency_penalty;
    float repetition_penalty; /* 1 disables it */
    uint64_t seed;            /* 0 draws from the engine's own generator */
} qw_sampling;

/* Counters of the prefix cache since start. */
typedef struct qw_cache_stats {
    uint64_t hits, tokens_restored, snapshots_saved;
    uint64_t ram_bytes, disk_bytes, blocks, snapshots;
    uint64_t prompt_tokens;          /* all prompt tokens seen */
    uint64_t reused_tokens;          /* of those, taken from a slot or the cache */
    uint64_t blend_candidate_tokens; /* tokens behind the reuse point that sit in chunks seen before */
} qw_cache_stats;

/* Seconds a slot's current request spent per phase since its qw_begin_prompt. */
typedef struct qw_slot_timing {
    double restore_s;  /* restoring from the caches */
    double prefill_s;  /* prefill calls it took part in (saves included) */
    double save_s;     /* of that: saving to the prefix cache */
    double pin_wait_s; /* of that: waiting for pinned buffers */
} qw_slot_timing;

/* One image or video of a prompt.  The prompt carries the pad token at each of the media's positions. */
typedef struct qw_media {
    uint64_t hash;         /* content hash = identity of its tokens in the prefix cache */
    int32_t video;         /* 0: image, 1: video */
    int32_t t, h, w;       /* patch grid: t temporal slices of h x w patches */
    const float *patches;  /* fp32 [t*h*w][1536] in merge-window order */
    const int64_t *starts; /* first token position of each slice (h*w/4 tokens per slice), t entries */
} qw_media;

/* One request of a qw_generate step. */
typedef struct qw_step_req {
    int32_t slot;
    int32_t pending; /* the sampled token that has not been decoded yet */
    int32_t budget;  /* tokens the request may still emit, >= 1 */
    int32_t flags;   /* QW_STEP_* */
    qw_sampling sampling;
} qw_step_req;

#define QW_STEP_LOGITS 1 /* keep the full logits of the request's rows for qw_top_logprobs */

/* ---------------------------------------------------------------- lifetime */

/* options_json: an object such as {"model_dir": "...", "ple_dir": "...", "slots": [131072, 65536],
 * "prefill_chunk": 4096, "devices": [0, 1, 2, 3, 4, 5, 6, 7]}.  On failure returns NULL and writes the
 * reason into err (errlen bytes). */
qw_handle *qw_open(const char *options_json, char *err, int errlen);
void qw_close(qw_handle *h);
/* Writes the slots' conversations to the disk tier of the prefix cache (when one is configured) and
 * waits for the files; call with no request in flight, typically before exiting. */
int qw_persist(qw_handle *h);
const char *qw_error(qw_handle *h);
/* Health of the engine: 0 while it works.  After a rank's job failed or a collective gave up, the
 * reason is copied into buf and its length (without the terminating 0) is returned; the engine stays
 * unusable until the process restarts.  May be called from any thread. */
int qw_engine_failure(qw_handle *h, char *buf, int buflen);

/* ---------------------------------------------------------------- prefix cache */

/* The token that opens a chat message: states just before such tokens are kept, so prompts that share
 * everything up to a message boundary share the work. */
int qw_set_boundary_token(qw_handle *h, int32_t id);
int qw_get_cache_stats(qw_handle *h, qw_cache_stats *out);
int qw_get_slot_timing(qw_handle *h, int slot, qw_slot_timing *out);

/* ---------------------------------------------------------------- slots and prompts */

int qw_num_slots(qw_handle *h);
int64_t qw_slot_capacity(qw_handle *h, int slot);

/* Reserves a free slot able to hold n + max_new tokens, preferring the one that can reuse most of
 * `tokens`.  -1 with an empty qw_error: every suitable slot is busy. */
int qw_acquire(qw_handle *h, const int32_t *tokens, int64_t n, int64_t max_new);
int qw_acquire_media(qw_handle *h, const int32_t *tokens, int64_t n, int64_t max_new, const qw_media *media, int n_media);
int qw_release(qw_handle *h, int slot);

/* Makes the slot hold exactly tokens[0..n) in one call; returns how many tokens were reused. */
int64_t qw_set_prompt(qw_handle *h, int slot, const int32_t *tokens, int64_t n);
int64_t qw_set_prompt_media(qw_handle *h, int slot, const int32_t *tokens, int64_t n, const qw_media *media, int n_media);
/* 1 when the vision tower is loaded. */
int qw_has_vision(qw_handle *h);

/* The same in steps, so that other slots can decode in between.  qw_begin_prompt restores what the
 * caches hold and returns the reused tokens (media must stay valid until the prompt is in);
 * qw_prefill_some prefills at most max_tokens more and returns 1 once the prompt is complete, else 0. */
int64_t qw_begin_prompt(qw_handle *h, int slot, const int32_t *tokens, int64_t n, const qw_media *media, int n_media);
int qw_prefill_some(qw_handle *h, int slot, int64_t max_tokens);
/* Before qw_begin_prompt: 1 while cache entries of this prompt that exist only on disk are being read
 * into RAM in the background (poll), 0 when nothing is left to load, -1 on error. */
int qw_prefetch(qw_handle *h, int slot, const int32_t *tokens, int64_t n, const qw_media *media, int n_media);
/* qw_prefill_some for several slots at once (one pass when their pieces fit a prefill chunk);
 * done[i] becomes 1 once slots[i] holds its whole prompt. */
int qw_prefill_batch(qw_handle *h, int n, const int32_t *slots, const int64_t *max_tokens, int32_t *done);
/* Samples the token that follows the slot's prompt; *lp receives its log-probability. */
int32_t qw_sample_prompt(qw_handle *h, int slot, const qw_sampling *p, float *lp);

/* ---------------------------------------------------------------- decoding */

/* One batched step: row i appends tokens[i] to slots[i]; rows of one slot are consecutive. */
int qw_decode(qw_handle *h, int n, const int32_t *slots, const int32_t *tokens);
/* Samples from row `row` of the last qw_decode. */
int32_t qw_sample_row(qw_handle *h, int row, const qw_sampling *p, float *lp);

/* 1 when the MTP head is loaded and qw_generate drafts tokens. */
int qw_has_mtp(qw_handle *h);
/* Tokens that end the request in `slot` (EOS and the request's stop_token_ids). */
int qw_set_stop_tokens(qw_handle *h, int slot, const int32_t *ids, int n);
/* One generation step for n requests on distinct slots: each pending token plus up to k drafts are
 * decoded and 1..k+1 tokens per request are emitted (never more than its budget).  For request i:
 * counts[i] tokens in tokens[i*(k+1) ...] with their logprobs at the same indices, first_rows[i] = row
 * of its first token for qw_top_logprobs (token j is row first_rows[i] + j), stopped[i] = 1 when its last
 * token is a stop token.  k = 0 decodes without drafts. */
int qw_generate(qw_handle *h, int n, const qw_step_req *reqs, int k, int32_t *tokens, float *logprobs, int32_t *counts,
                int32_t *first_rows, int32_t *stopped);

/* The k most likely (id, logprob) of the raw distribution of a decode / generate row, or after the
 * last sampled prompt when row < 0.  Returns the number written. */
int qw_top_logprobs(qw_handle *h, int row, int k, int32_t *ids, float *lps);
int qw_top_logprobs_prompt(qw_handle *h, int slot, int k, int32_t *ids, float *lps);

#ifdef __cplusplus
}
#endif
#endif /* QW_CAPI_H */
