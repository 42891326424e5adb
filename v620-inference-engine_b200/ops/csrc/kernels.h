// Prototypes of the kernel launchers (extern "C", one per kernel family).  Every launcher
// enqueues on the given stream, allocates nothing and returns 0 on success, -1 for unsupported
// shapes and -2 for a launch error.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

extern "C" {

// gemv.cu
int qwk_gemv_bf16(const void *W, const void *x, float *y, void *y_bf16, int N, int K, int M, int ldw, int ldx, int ldy, int accumulate, int nsplit, long long w_split, long long x_split, long long y_split, cudaStream_t s);

// moe.cu
int qwk_moe_router(const void *Wrs, const void *x, float *rs, int nrs, int K, int M, int ldx, int E, int top_k, int F, int e_first, int e_local, int *pair_expert, float *pair_w, void *sh_h, unsigned int *ticket, cudaStream_t s);
int qwk_moe_route(const float *rs, int ld_rs, int M, int E, int top_k, int F, int e_first, int e_local, int *pair_expert, float *pair_w, void *sh_h, cudaStream_t s);
int qwk_moe_gate_up_pair(const void *w13, const void *s13, const void *x, int ldx, const int *pair_expert, int M, int top_k, int F, int K, void *h, cudaStream_t s);
int qwk_moe_down_combine(const void *w2, const void *s2, const void *h, const int *pair_expert, const float *pair_w, int M, int top_k, int F, int H, const void *shared_down, int ld_sd, const void *sh_h, int SF, float *out, int ldo, cudaStream_t s);

// hc.cu
int qwk_embed_rows(const int *tokens, const void *table, int ld_table, int col0, int SH, int hc, int vocab, float *X, int M, cudaStream_t s);
int qwk_hc_pre(float *X, const float *pend, int ld_pend, const float *inj, int ld_inj, const float *w1, int SH, int hc, void *y, float *ssq, int ld_ssq, int M, cudaStream_t s);
int qwk_hc_up_mix(const float *red, int ld_red, const void *Wu, const float *X, const float *w1, int SH, int hc, int R, int n_inj, int H, float eps, int M, float *inj, int ld_inj, void *bin, int ld_bin, int bin_col0, cudaStream_t s);
int qwk_hc_down(const float *Xin, float *Xout, const float *pend, int ld_pend, const float *inj_prev, const float *w1, const void *Wd, float *send, int ld_send, int SH, int hc, int down, int M, cudaStream_t s);

// gdn.cu
int qwk_gdn_conv(const float *proj, int ld_proj, float *ring, const float *cw, const float *A_log, const float *dt_bias, int KL, int VL, int M, const int *slot, const int *pos, const int *run_start, const int *run_len, float *qkv, float *decay, float *beta, float eps, cudaStream_t s);
int qwk_gdn_scan(const float *qkv, const float *decay, const float *beta, const float *proj, int ld_proj, float *S, float *save, const float *norm_w, int KL, int VL, int M, const int *slot, const int *pos, const int *run_start, const int *run_len, void *o, float eps, cudaStream_t s);
int qwk_gdn_step(const float *proj, int ld_proj, float *ring, const float *cw, const float *A_log, const float *dt_bias, const float *norm_w, int KL, int VL, int M, const int *slot, const int *pos, const int *run_start, const int *run_len, float *S, float *save, float *qkv, float *decay, float *beta, void *o, float eps, cudaStream_t s);

// qsa.cu
int qwk_rope_init(double theta, int rope_dim);
int qwk_qsa_prep(const float *proj, int ld_proj, int QL, int KVL, int IH, const float *qn1, const float *kn1, const float *iqn1, const float *ikn1, int M, const int *slot, const int *pos, const int *run_start, const int *run_len, void *k_dev, void *v_dev, void *k_host, void *v_host, int n_dev_pages, const int *page_table, int max_pages, float *q, float *iq, float *raw_ring, void *ck, int ck_cap, int ratio, float eps, cudaStream_t s);
int qwk_qsa_scores(const float *iq, int IH, const void *ck, int ck_cap, int M, const int *slot, const int *pos, int ratio, int topk_blocks, float *scores, int ld_scores, int max_groups, cudaStream_t s);
int qwk_qsa_select(const float *scores, int ld_scores, int M, const int *pos, int ratio, int topk, int *sel, int *sel_n, cudaStream_t s);
int qwk_qsa_attend(const float *q, int QL, int KVL, int M, const int *slot, const int *pos, void *k_dev, void *v_dev, void *k_host, void *v_host, int n_dev_pages, const int *page_table, int max_pages, const int *sel, const int *sel_n, int topk, int ratio, int nsplit, float *pm, float *pl, float *pacc, const float *proj, int ld_proj, void *o, cudaStream_t s);

// ple.cu
int qwk_ple_init(const unsigned long long *mult, int ngram, const unsigned long long *sizes, const long long *offsets, int heads, int eos, const float *f8_lut);
int qwk_ple_gather(const int *ctx, const void *const *shards, const void *const *scales, long long rows_per_shard, long long rows, int layout, int width, int heads, void *e, long long *ids_out, int M, cudaStream_t s);
int qwk_ple_stats(const float *kv, int ld_kv, const float *X, const float *nk1, const float *nq1, int SH, int hc, float *send, int ld_send, int M, cudaStream_t s);
int qwk_ple_apply(const float *kv, int ld_kv, const float *red, int ld_red, const float *nc1, const float *cw, int SH, int hc, int H, float eps, int taps, int dil, float *gv, float *nc, float *ring, float *X, int M, const int *slot, const int *pos, const int *run_start, const int *run_len, cudaStream_t s);

// logits.cu
int qwk_advance_rows(int *tokens, int *pos, int *ctx3, const int *next, int M, cudaStream_t s);
int qwk_row_reduce(const float *logits, int ld, int V, int idx0, int M, float *out_val, int *out_idx, float *out_max, float *out_sum, cudaStream_t s);
int qwk_merge_argmax(const float *vals, const int *idx, int ranks, int M, int stride, int *out_idx, float *out_val, cudaStream_t s);

}  // extern "C"
