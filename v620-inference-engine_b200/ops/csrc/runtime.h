// C structs of the device runtime: per-rank weights in engine layout, per-rank work buffers, the
// slot-state tables and the row tables of one batched step.  Python (torch) allocates all memory
// and fills these structs through ctypes mirrors with the same field order; the runtime only
// enqueues kernels on the stream it is given, so a step can be captured into a CUDA graph.
//
// This plays the role of the reference's per-rank state (src/engine/rank.hpp:37-215) and graph body
// (src/engine/decode.hip:40-163) with a runtime rank count and bf16 dense weights.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

extern "C" {

typedef struct QwDims {
    int ranks, rank;
    int H, hc, hc_rank, SH;            // hidden, streams, mixer rank, residual columns per rank
    int n_layers, vocab, vocab_l;
    int QL, KVL, IH, proj_qsa;         // local q heads, local kv heads, indexer heads, qsa projection rows
    int KL, VL, proj_gdn;              // local gdn k heads, v heads, projection rows
    int E, E_l, e_first, top_k, F, SF; // experts, local experts, first local expert, top-k, ffn, shared-ffn columns
    int ple_layer, ple_kv, ngram_heads, ngram_dim, ple_taps, ple_dil;
    int idx_ratio, idx_topk, nsplit;   // tokens per group, groups selected, attention splits
    int max_rows;                      // rows the buffers are sized for
    int slots, max_pages, n_dev_pages, ck_cap, score_cap;
    float eps;
} QwDims;

typedef struct QwHc {
    const float *w1;       // (1+w) [hc][SH]
    const void *Wd;        // bf16 [R+n_inj][hc][SH]
    const void *Wu;        // bf16 [SH][hc][R]
    int n_inj;             // hc, or 0 for a final mixer
    int pad_;
} QwHc;

typedef struct QwLayer {
    int is_qsa;
    int state_index;       // index among the layers of the same kind (KV / GDN state tables)
    QwHc attn_hc, mlp_hc;
    // attention block
    const void *Wproj;     // bf16 [proj rows][H]
    const void *Wout;      // bf16 [H][VL*128] or [H][QL*256]
    const float *cw, *A_log, *dt_bias, *gdn_norm;   // GDN
    const float *qn1, *kn1, *iqn1, *ikn1;           // QSA (1+w)
    // MoE
    const void *Wrs;       // bf16 [E + 1 + 2*SF][H]
    const void *w13, *s13; // q4 [E_l][2F][H/8], bf16 [E_l][2F][H/128]
    const void *w2, *s2;   // q4 [E_l][H][F/8],  bf16 [E_l][H][F/128]
    const void *Wsd;       // bf16 [H][SF]
} QwLayer;

typedef struct QwPle {
    const void *Wkv;               // bf16 [hc*SH + SH][H]
    const float *nk1, *nq1, *nc1;  // (1+w) [hc][SH]
    const float *cw;               // [hc*SH][taps]
    const void *const *shards;     // device array of table shard pointers (host-mapped memory)
    const void *const *scales;
    long long rows_per_shard, rows;
    int layout, enabled;
} QwPle;

typedef struct QwMtp {
    int enabled, pad_;
    QwLayer layer;             // a QSA decoder layer (its KV lives at state index n_qsa)
    QwHc final_hc;
    const void *fc_h, *fc_e;   // bf16 [SH][H]: this rank's output rows
    const float *nh1;          // (1+w) [hc*H]: pre_fc_norm_hidden
    const float *ne1;          // (1+w) [H]: pre_fc_norm_embedding
    void *hn, *en;             // bf16 [rows*hc][H], [rows][H]
    float *fh, *fe;            // fp32 [rows*hc][SH], [rows][SH]
} QwMtp;

typedef struct QwState {
    // per QSA layer (index = state_index): host arrays of n_qsa device pointers
    void *const *k_dev;
    void *const *v_dev;
    void *const *k_host;
    void *const *v_host;
    void *const *ck;           // bf16 [slots][ck_cap][128]
    float *const *raw_ring;    // [slots][RAW_RING][128]
    // per GDN layer
    float *const *gdn_S;       // [slots][VL][128][128]
    float *const *gdn_ring;    // [slots][GDN_RING][qkv_l]
    float *ple_ring;           // [slots][PLE_RING][hc*SH]
    const int *page_table;     // [slots][max_pages]
} QwState;

typedef struct QwBuffers {
    float *X;            // [rows][hc][SH]
    void *y;             // bf16 [rows][hc][SH]
    float *send, *red;   // [rows][hc_send]
    void *bin;           // bf16 [rows][H]
    float *proj;         // [rows][max proj]
    float *inj_a, *inj_b;// [rows][hc]
    float *partial;      // [rows][H] block output before the reduce-scatter
    float *out_a, *out_b;// [rows][SH] block outputs after it
    void *o;             // bf16 [rows][max(VL*128, QL*256)]
    float *qkv, *decay, *beta;        // GDN
    float *q, *iq, *scores;           // QSA
    int *sel, *sel_n;
    float *pm, *pl, *pacc;
    float *rs;           // [rows][E+1+2SF]
    int *pair_expert;
    float *pair_w;
    void *sh_h, *moe_h;  // bf16 [rows][SF], [rows*top_k][F]
    void *ple_e;         // bf16 [rows][H]
    float *ple_kv, *ple_send, *ple_red, *ple_gv, *ple_nc;
    float *logits;       // [rows][vocab_l]
    float *amax_val;     // [rows]
    int *amax_idx;
    float *lse_max, *lse_sum;
    float *gdn_save;     // optional [n_gdn][rows][VL][128][128]
    float *hidden_out;   // optional [rows][hc][SH]: X after the last combine (MTP input)
    float *X2;           // second residual buffer: a mixer with a deferred combine writes X here and the two swap
    unsigned int *ticket;// one zeroed word for the router kernel's last-block election
} QwBuffers;

typedef struct QwRows {
    int M;
    int max_groups;      // upper bound of visible groups over the rows (sizes the score grid)
    const int *tokens;   // [M]
    const int *slot, *pos, *run_start, *run_len;
    const int *ctx3;     // [M][3] n-gram context (token, previous, one before; -1 = none)
} QwRows;

// Collective hook.  kind: 0 all-reduce fp32 (src -> dst, rows x n), 1 all-gather of bf16 slices into
// dst[rows][ranks*n] (this rank's slice is already in place), 2 reduce-scatter fp32 src[rows][ranks*n]
// -> dst[rows][n].  With ranks == 1 it is never called.
typedef void (*QwCommFn)(void *user, int kind, int site, const void *src, void *dst, int rows, int n,
                         cudaStream_t stream);

typedef struct QwModel {
    QwDims d;
    const QwLayer *layers;     // host array [n_layers]
    QwHc final_hc;
    QwPle ple;
    const void *embed;         // bf16 [vocab][H]
    const void *lm_head;       // bf16 [vocab_l][H]
    QwState st;
    QwBuffers b;
    QwCommFn comm;
    void *comm_user;
    const void *p2p;           // QwP2P (p2p.cu): when set, collectives run as this library's peer-memory kernels
    float *amax_pairs;         // [rows][ranks*2] inside the symmetric region (gather target of the argmax merge)
    long long off_amax;        // its offset inside the region
    long long off_bin;         // offset of b.bin inside the region
    QwMtp mtp;
    float *mtp_hid;            // several ranks: [rows*hc][H] fp32 inside the symmetric region, the gathered hidden states of an MTP pass
    long long off_mtp_hid;     // its offset inside the region
    long long off_logits;      // several ranks: offset of the [rows][vocab] fp32 logits matrix inside the region (b.logits = this rank's column slice)
    int logits_ld;             // row stride of b.logits in floats (0: vocab_l, dense)
    int pad2_;
} QwModel;

// flags of qwrt_decode
#define QWRT_SAVE_GDN 1        // keep the GDN state after every row (speculative rollback)
#define QWRT_NO_HEAD 2         // skip lm_head (prefill rows whose logits are not needed)
#define QWRT_KEEP_HIDDEN 4     // copy X after the final combine to hidden_out
#define QWRT_CHAIN 8           // feed each row's argmax back as its next token and advance its position (one row per slot)

int qwrt_decode(const QwModel *md, const QwRows *rows, int flags, int n_layers_run, cudaStream_t stream);

// One MTP pass over the rows: input b.hidden_out (the pre-final-mixer state of each row's position) and
// rows->tokens (the token AFTER that position); output logits / argmax of the position after that, and the MTP's
// own pre-final-mixer state back in b.hidden_out (the input of a chained next draft).  Several ranks: peer-memory collectives only.
int qwrt_mtp(const QwModel *md, const QwRows *rows, int flags, cudaStream_t stream);

}  // extern "C"
