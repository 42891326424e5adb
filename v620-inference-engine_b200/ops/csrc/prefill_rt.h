// C structs of the token-major prefill runtime (prefill_rt.cu): the work buffers of a chunk and the
// description of one chunk job.  Python (torch) allocates every buffer and fills these structs through
// ctypes mirrors with the same field order (ops/structs.py); the runtime only enqueues kernels.
// (Role of the reference's PrefillBuf / run_prefill_rank, src/engine/rank.hpp:37-215 and
// src/engine/prefill.hip:46-496.)
#pragma once

#include "runtime.h"

extern "C" {

// Row-indexed buffers hold `cap` rows (the chunk size); micro-batch lane l of a chunk of T rows works on
// rows [r0_l, r0_l + n_l) of each.  Pair-indexed buffers (expert-sorted rows) hold cap * top_k rows and a
// lane uses the rows from r0_l * top_k on.
typedef struct QwPrefillBufs {
    float *X;            // [cap][hc][SH] residual streams
    void *xn;            // bf16 [cap][hc*SH]
    float *d;            // [hc_ksplit][cap][hc_ld] partial down projections (one rank)
    void *u;             // bf16 [cap][hc_rank]
    float *inj_a, *inj_b;// [cap][hc]
    float *g;            // [cap][hc*SH]
    void *bin;           // bf16 [cap][H] block input (one rank; with a channel it lives in the channel's region)
    float *proj;         // [cap][proj_ld]
    void *o;             // bf16 [cap][o_ld]
    float *out_a, *out_b;// [cap][H] block outputs (one rank); [cap][SH] scratch for a reduced pending output (several ranks)
    float *qkv, *decay, *beta;       // GDN: [cap][qkv_l], [cap][VL], [cap][VL]
    float *q, *iq, *scores;          // QSA: [cap][QL][256], [cap][IH][128], [cap][score_cap]
    int *sel, *sel_n;                // [cap][idx_topk], [cap]
    float *rs;           // [cap][nrs_ld] router logits | shared gate | shared gate/up rows
    int *pe;             // [cap][top_k]
    float *pw;           // [cap][top_k]
    void *sh_h;          // bf16 [cap][SF]
    float *sd;           // [cap][H]
    void *xperm;         // bf16 [cap*top_k + 128][H]
    void *h13;           // bf16 [cap*top_k][2F]
    void *h;             // bf16 [cap*top_k + 128][F]
    float *y;            // [cap*top_k][H]
    int *inv, *src_token;// [cap*top_k]
    void *t13, *t2;      // int4 [2][max_tiles] tile tables, one per lane
    float *gdn_scratch;  // [2][gdn_scratch_lane]
    void *ple_e;         // bf16 [cap][H]
    float *ple_kv;       // [cap][ple_ld]
    float *ple_send, *ple_red;       // [cap][16]
    float *ple_gv, *ple_nc;          // [cap][hc*SH]
    // MTP pass
    float *Xm;           // [cap][hc][SH] hidden states shifted by the pending row
    void *hn, *en;       // bf16 [cap*hc][H] (one rank), [cap][H]
    float *fh, *fe;      // [cap*hc][SH], [cap][SH]
    float *mtp_ssq;      // [2][cap] (several ranks: local sums, reduced sums)
    int *mtp_tok;        // [cap] the token after each MTP row's position
    float *hid_out;      // [hc][SH] out: hidden state of the chunk's last position (the next call's pending MTP row)
    void *amax16;        // [4] floats of scratch for the argmax merge
    // row tables of the chunk (device): lane-relative run tables (run_start = 0, run_len[r0_l] = n_l)
    const int *tokens, *slot, *pos, *run_start, *run_len, *ctx3;
    // row tables of the MTP pass
    const int *m_slot, *m_pos, *m_run_start, *m_run_len;
    // vision rows: X[over_rows[j]] = over_emb[j] (fp32 [n_over][H])
    const int *over_rows;
    const float *over_emb;
    // KV spill: device copies of one slot's host pages of one layer (K and V), filled before a QSA layer's attention
    // so that the attention kernel gathers its rows from device memory (null: the kernels read the host pages directly)
    void *stage_k, *stage_v;
    int cap, hc_ld, hc_ksplit, nrs_ld, proj_ld, o_ld, ple_ld, max_tiles;
    long long gdn_scratch_lane;
} QwPrefillBufs;

typedef void (*QwPrefillHook)(void *user, int layer, int which, const void *bin, int ld_bin, int r0, int n);

typedef struct QwPrefillJob {
    const QwModel *md;
    const QwPrefillBufs *b;
    void *tp[2];               // QwTp channel of each lane (null with one rank)
    cudaStream_t stream[2];    // lane 0 runs on stream[0] (the caller's stream); lane 1 on stream[1]
    int T;                     // rows of the chunk
    int lanes;                 // 1 or 2 micro-batches
    int base;                  // position of the chunk's first row in its slot
    int want_logits;           // lm_head + argmax of the last row into the model's logits / amax buffers (row 0)
    int layer_limit;           // < 0: all layers
    int mtp_rows;              // rows of the MTP pass (0: none)
    int mtp_base;              // position of the first MTP row
    int has_pending;           // Xm row 0 comes from md->b.hidden_out row 0 (the previous call's last hidden state)
    int n_over;                // rows whose embedding is replaced
    int n0;                    // two lanes: rows of lane 0 (lane 1 takes the rest)
    QwPrefillHook hook;        // optional: called (after the stream work is enqueued) with each block input
    void *hook_user;
    int slot;                  // the chunk's slot (host copy of the row table's value)
    int pad_;
} QwPrefillJob;

// Enqueues the chunk of every job (one job per rank; more than one only when several ranks are emulated in one
// process on one stream, where each kernel is issued for all ranks before the next).  Returns 0 or the first
// launcher's error code * 1000 - line.
int qwrt_prefill(const QwPrefillJob *const *jobs, int njobs);
long long qwrt_prefill_sizes(int which);     // 0: sizeof(QwPrefillBufs), 1: sizeof(QwPrefillJob), 2: sizeof(QwTp)
long long qwrt_prefill_last_launches(void);

}  // extern "C"
