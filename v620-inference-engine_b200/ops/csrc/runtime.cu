// The device runtime: enqueues one batched step (M rows, each appending a token to a slot) of the
// whole model on a stream.  Used for decode (M = rows of the step), for speculative verification
// (several rows per slot) and for row-batched prefill.  It allocates nothing and never
// synchronises, so the caller may capture it into a CUDA graph per row count.
//
// Per sublayer the schedule is: hc_pre -> down GEMV -> [all-reduce] -> hc_up_mix -> [all-gather] ->
// block -> [reduce-scatter]; collectives go through the QwCommFn hook (not called with one rank).
// (Role of the reference's record_batch, src/engine/decode.hip:40-163.)
#include "runtime.h"

#include "kernels.h"
#include "fuse.cuh"

#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

namespace qw {
ErrorWord *g_err_ptr = nullptr;
PfArgs g_pf = {};
int *g_moe_stats = nullptr;
SharedAct g_shared_act = {nullptr, 0, 0, 0, nullptr};
FuseOut g_fo = {};
FuseIn g_fi = {};
}

// 1: collectives ride in the producer / consumer kernels; 0: stand-alone collective kernels.
// Builds with -DQW_DIAG add timing instruments that make a step compute garbage on purpose: mode 2 (nothing is sent or
// waited for, so a step costs what its kernels alone cost), a mask of collective kinds to leave out, and QW_SKIP=name,...
// which leaves out every launch whose launcher call contains one of the names.  None of it is in the shipped library.
static int g_fuse = 1;
// MoE balance statistics (QW_MOE_STATS): a device array of one counter per layer (+ one for the MTP layer); every
// routing launch adds the number of expert pairs that fall on this rank.  Null = off.
static int *g_moe_stats_base = nullptr;
extern "C" __attribute__((visibility("default"))) int qwrt_set_moe_stats(int *base) {
    g_moe_stats_base = base;
    return 0;
}
#ifdef QW_DIAG
static int g_fuse_kinds = 7;    // bit k clear = collectives of kind k (0 all-reduce, 1 all-gather, 2 reduce-scatter) are skipped
extern "C" __attribute__((visibility("default"))) int qwrt_set_fuse_kinds(int mask) {
    g_fuse_kinds = mask & 7;
    return 0;
}
constexpr int FUSE_MODE_MAX = 2;
#else
constexpr int g_fuse_kinds = 7;
constexpr int FUSE_MODE_MAX = 1;
#endif
static qw::FuseOut fuse_out_of(const void *p2p, int kind, unsigned k, int mode, int n) {
    return (g_fuse_kinds >> kind) & 1 ? qw::make_fuse_out(p2p, kind, k, mode, n) : qw::FuseOut{};
}
static qw::FuseIn fuse_in_of(const void *p2p, int kind, unsigned k, int n) {
    return (g_fuse_kinds >> kind) & 1 ? qw::make_fuse_in(p2p, kind, k, n) : qw::FuseIn{};
}
extern "C" __attribute__((visibility("default"))) int qwrt_set_fuse(int mode) {
    g_fuse = mode < 0 || mode > FUSE_MODE_MAX ? 1 : mode;
    return 0;
}

// Registers the device error word (8 bytes, zeroed by the caller) that kernels with bounded waits report to.
#ifdef QW_DEVICE_CHECKS
extern "C" int qw_dcheck_set_hc(void *p);
extern "C" int qw_dcheck_set_qsa(void *p);
#endif
extern "C" __attribute__((visibility("default"))) int qwk_set_error_word(void *p) {
    qw::g_err_ptr = (qw::ErrorWord *)p;
#ifdef QW_DEVICE_CHECKS
    if (qw_dcheck_set_hc(p) || qw_dcheck_set_qsa(p)) return -2;      // the checked kernels report to the same word
#endif
    return 0;
}
// 1 in the checked build of the library (-DQW_DEVICE_CHECKS), 0 otherwise.
extern "C" __attribute__((visibility("default"))) int qwk_device_checks(void) {
#ifdef QW_DEVICE_CHECKS
    return 1;
#else
    return 0;
#endif
}

namespace {

struct Ctx {
    const QwModel *md;
    const QwRows *rows;
    cudaStream_t s;
    int site;
    int err;
    long long launches;
    float *X, *Xalt;     // current residual buffer and its ping-pong partner
    // fused collectives: the block input's all-gather and the pending block output's reduce-scatter are
    // waited for by the kernels that read them
    bool fuse, mute;
    bool bin_pending, pend_fused;
    int bin_site, pend_site;
};

#ifdef QW_DIAG
// Timing diagnostic: QW_SKIP=name[,name...] leaves out every launch whose launcher call contains one of the names
// (e.g. QW_SKIP=qwk_hc_down).  The step's results are then wrong; the step time shows what the kernels cost in place.
bool skipped(const char *expr) {
    static std::vector<std::string> names;
    static bool parsed = false;
    if (!parsed) {
        parsed = true;
        if (const char *e = getenv("QW_SKIP")) {
            std::string cur;
            for (const char *p = e;; ++p) {
                if (*p == ',' || *p == 0) {
                    if (!cur.empty()) names.push_back(cur);
                    cur.clear();
                    if (*p == 0) break;
                } else {
                    cur.push_back(*p);
                }
            }
        }
    }
    for (const auto &n : names)
        if (strstr(expr, n.c_str())) return true;
    return false;
}
#else
inline bool skipped(const char *) { return false; }
#endif

long long g_last_launches = 0;      // kernels enqueued by the most recent qwrt_decode / qwrt_mtp call

// Runs a launcher that enqueues `n` kernels; remembers the first failure and counts the launches.
#define QW_TRYN(n, expr)                   \
    do {                                   \
        if (!skipped(#expr)) {             \
            int rc__ = (expr);             \
            c.launches += (n);             \
            if (rc__ != 0 && c.err == 0) c.err = rc__ * 1000 - __LINE__; \
        }                                  \
    } while (0)

// A launch that takes the one-shot options armed just before it (fused collective ends, the shared expert's activation);
// they are cleared afterwards whether or not the launcher took them.  `wptr` / `wbytes` name the weights it streams.
#define QW_OP(n, wptr, wbytes, expr)                                              \
    do {                                                                          \
        (void)(wptr);                                                             \
        (void)(wbytes);                                                           \
        if (c.mute) {                                                             \
            qw::g_fo = qw::FuseOut{};                                             \
            qw::g_fi = qw::FuseIn{};                                              \
        }                                                                         \
        QW_TRYN(n, expr);                                                         \
        qw::g_fo = qw::FuseOut{};                                                 \
        qw::g_fi = qw::FuseIn{};                                                  \
        qw::g_shared_act = qw::SharedAct{nullptr, 0, 0, 0, nullptr};              \
    } while (0)

inline int hc_send(const QwDims &d) { return d.hc + d.hc * (d.hc_rank + d.hc); }

void comm(Ctx &c, int kind, const void *src, void *dst, int rows, int n) {
    const QwModel &md = *c.md;
    ++c.site;
    if (md.d.ranks > 1 && md.p2p) {
        int rc = 0;
        if (kind == 0) rc = qwk_p2p_allreduce(md.p2p, (unsigned)c.site, (const float *)src, (float *)dst, rows, n, c.s);
        else if (kind == 1) rc = qwk_p2p_allgather(md.p2p, (unsigned)c.site, 1, md.off_bin, rows, n, 2, c.s);
        else rc = qwk_p2p_reduce_scatter(md.p2p, (unsigned)c.site, (const float *)src, (float *)dst, rows, n, c.s);
        c.launches += 1;
        if (rc != 0 && c.err == 0) c.err = rc * 1000 - __LINE__;
        return;
    }
    if (md.d.ranks > 1 && md.comm) md.comm(md.comm_user, kind, c.site, src, dst, rows, n, c.s);
}

// One mixer: X (+= pending) -> block input (bf16 [M][H], all ranks' columns) and injection logits.
void mix(Ctx &c, const QwHc &w, const float *pend, const float *inj_prev, float *inj_out) {
    const QwModel &md = *c.md;
    const QwDims &d = md.d;
    const QwBuffers &b = md.b;
    const int M = c.rows->M, ld = hc_send(d);
    const int down = d.hc_rank + w.n_inj;
    if (c.fuse) {
        // the down projection consumes the pending block output's reduce-scatter and sends the all-reduce
        if (pend && c.pend_fused) qw::g_fi = fuse_in_of(md.p2p, 2, (unsigned)c.pend_site, d.SH);
        qw::g_fo = fuse_out_of(md.p2p, 0, (unsigned)(c.site + 1), 1, ld);
    }
    // fused: deferred combine (into the partner buffer) + sums of squares + down projection
    QW_OP(1, w.Wd, (size_t)down * d.hc * d.SH * 2,
          qwk_hc_down(c.X, pend ? c.Xalt : nullptr, pend, d.SH, inj_prev, w.w1, w.Wd, b.send, ld, d.SH, d.hc, down, M, c.s));
    if (pend) {
        float *t = c.X;
        c.X = c.Xalt;
        c.Xalt = t;
    }
    const float *red = b.send;
    if (c.fuse) {
        ++c.site;
        // the up projection consumes that all-reduce and sends its columns of the block input (all-gather)
        qw::g_fi = fuse_in_of(md.p2p, 0, (unsigned)c.site, ld);
        qw::g_fo = fuse_out_of(md.p2p, 1, (unsigned)(c.site + 1), 1, d.SH);
    } else if (d.ranks > 1) {
        comm(c, 0, b.send, b.red, M, ld);
        red = b.red;
    } else {
        ++c.site;
    }
    QW_OP(1, w.Wu, (size_t)d.SH * d.hc * d.hc_rank * 2,
          qwk_hc_up_mix(red, ld, w.Wu, c.X, w.w1, d.SH, d.hc, d.hc_rank, w.n_inj, d.H, d.eps, M, inj_out, d.hc, b.bin, d.H,
                        d.rank * d.SH, c.s));
    if (c.fuse) {
        ++c.site;
        c.bin_site = c.site;
        c.bin_pending = true;          // the next kernel that reads the block input waits for it
    } else {
        comm(c, 1, b.bin, b.bin, M, d.SH);
    }
}

// Before the first kernel that reads the gathered block input.
inline void await_bin(Ctx &c) {
    if (c.bin_pending) qw::g_fi = fuse_in_of(c.md->p2p, 1, (unsigned)c.bin_site, c.md->d.SH);
    c.bin_pending = false;
}

// Before the kernel that writes the block output `partial`: it also sends the reduce-scatter.
inline void send_partial(Ctx &c, bool fused) {
    const QwDims &d = c.md->d;
    if (fused && c.fuse)
        qw::g_fo = fuse_out_of(c.md->p2p, 2, (unsigned)(c.site + 1), 2, d.SH);
}

void gdn_block(Ctx &c, const QwLayer &L, int flags) {
    const QwModel &md = *c.md;
    const QwDims &d = md.d;
    const QwBuffers &b = md.b;
    const QwRows &r = *c.rows;
    const int M = r.M, gi = L.state_index;
    const int qkv_l = (2 * d.KL + d.VL) * 128;
    await_bin(c);
    QW_OP(1, L.Wproj, (size_t)d.proj_gdn * d.H * 2,
          qwk_gemv_bf16(L.Wproj, b.bin, b.proj, nullptr, d.proj_gdn, d.H, M, d.H, d.H, d.proj_gdn, 0, 1, 0, 0, 0, c.s));
    float *save = nullptr;
    if ((flags & QWRT_SAVE_GDN) && b.gdn_save)
        save = b.gdn_save + (size_t)gi * d.max_rows * d.VL * 128 * 128;
    if (M <= 12) {
        QW_OP(1, nullptr, 0, qwk_gdn_step(b.proj, d.proj_gdn, md.st.gdn_ring[gi], L.cw, L.A_log, L.dt_bias, L.gdn_norm,
                                            d.KL, d.VL, M, r.slot, r.pos, r.run_start, r.run_len, md.st.gdn_S[gi], save,
                                            b.qkv, b.decay, b.beta, b.o, d.eps, c.s));
    } else {
        QW_TRYN(3, qwk_gdn_step(b.proj, d.proj_gdn, md.st.gdn_ring[gi], L.cw, L.A_log, L.dt_bias, L.gdn_norm,
                                            d.KL, d.VL, M, r.slot, r.pos, r.run_start, r.run_len, md.st.gdn_S[gi], save,
                                            b.qkv, b.decay, b.beta, b.o, d.eps, c.s));
    }
    (void)qkv_l;
    const int K = d.VL * 128;
    send_partial(c, true);
    QW_OP(1, L.Wout, (size_t)d.H * K * 2, qwk_gemv_bf16(L.Wout, b.o, b.partial, nullptr, d.H, K, M, K, K, d.H, 0, 1, 0, 0, 0, c.s));
}

void qsa_block(Ctx &c, const QwLayer &L) {
    const QwModel &md = *c.md;
    const QwDims &d = md.d;
    const QwBuffers &b = md.b;
    const QwRows &r = *c.rows;
    const QwState &st = md.st;
    const int M = r.M, qi = L.state_index;
    await_bin(c);
    QW_OP(1, L.Wproj, (size_t)d.proj_qsa * d.H * 2,
          qwk_gemv_bf16(L.Wproj, b.bin, b.proj, nullptr, d.proj_qsa, d.H, M, d.H, d.H, d.proj_qsa, 0, 1, 0, 0, 0, c.s));
    QW_TRYN((M <= 16 - d.idx_ratio ? 1 : 2), qwk_qsa_prep(b.proj, d.proj_qsa, d.QL, d.KVL, d.IH, L.qn1, L.kn1, L.iqn1, L.ikn1, M, r.slot, r.pos,
                        r.run_start, r.run_len, st.k_dev[qi], st.v_dev[qi], st.k_host ? st.k_host[qi] : nullptr,
                        st.v_host ? st.v_host[qi] : nullptr, d.n_dev_pages, st.page_table, d.max_pages, b.q, b.iq,
                        st.raw_ring[qi], st.ck[qi], d.ck_cap, d.idx_ratio, d.eps, c.s));
    QW_TRYN((r.max_groups > d.idx_topk ? 1 : 0), qwk_qsa_scores(b.iq, d.IH, st.ck[qi], d.ck_cap, M, r.slot, r.pos, d.idx_ratio, d.idx_topk, b.scores,
                          d.score_cap, r.max_groups, c.s));
    QW_TRYN(1, qwk_qsa_select(b.scores, d.score_cap, M, r.pos, d.idx_ratio, d.idx_topk, b.sel, b.sel_n, c.s));
    QW_TRYN(2 + (st.k_host ? qwk_spill_cache_active(0) : 0), qwk_qsa_attend(b.q, d.QL, d.KVL, M, r.slot, r.pos, st.k_dev[qi], st.v_dev[qi],
                          st.k_host ? st.k_host[qi] : nullptr, st.v_host ? st.v_host[qi] : nullptr, d.n_dev_pages,
                          st.page_table, d.max_pages, b.sel, b.sel_n, d.idx_topk, d.idx_ratio, d.nsplit, b.pm, b.pl,
                          b.pacc, b.proj, d.proj_qsa, b.o, c.s));
    const int K = d.QL * 256;
    send_partial(c, true);
    QW_OP(1, L.Wout, (size_t)d.H * K * 2, qwk_gemv_bf16(L.Wout, b.o, b.partial, nullptr, d.H, K, M, K, K, d.H, 0, 1, 0, 0, 0, c.s));
}

void moe_block(Ctx &c, const QwLayer &L, bool fuse_out = true, int stats_index = -1) {
    const QwModel &md = *c.md;
    const QwDims &d = md.d;
    const QwBuffers &b = md.b;
    const int M = c.rows->M;
    const int nrs = d.E + 1 + 2 * d.SF;
    await_bin(c);
    if (g_moe_stats_base && stats_index >= 0) qw::g_moe_stats = g_moe_stats_base + stats_index;
    // the shared expert's activation is formed by extra blocks of the gate/up launch, not by the router's last block
    QW_OP(1, L.Wrs, (size_t)nrs * d.H * 2, qwk_moe_router(L.Wrs, b.bin, b.rs, nrs, d.H, M, d.H, d.E, d.top_k, d.SF, d.e_first, d.E_l, b.pair_expert,
                              b.pair_w, nullptr, b.ticket, L.w13, L.w2, (long long)2 * d.F * d.H / 2, (long long)d.H * d.F / 2, c.s));
    qw::g_shared_act = qw::SharedAct{b.rs, nrs, d.E, d.SF, b.sh_h};
    QW_OP(1, nullptr, 0, qwk_moe_gate_up_pair(L.w13, L.s13, b.bin, d.H, b.pair_expert, M, d.top_k, d.F, d.H, b.moe_h, c.s));
    send_partial(c, fuse_out);
    QW_OP(1, L.Wsd, (size_t)d.H * d.SF * 2, qwk_moe_down_combine(L.w2, L.s2, b.moe_h, b.pair_expert, b.pair_w, M, d.top_k, d.F, d.H, L.Wsd, d.SF, b.sh_h,
                                d.SF, b.partial, d.H, c.s));
}

// partial [M][H] -> out [M][SH] (this rank's columns, summed over ranks)
const float *scatter(Ctx &c, float *out, bool fused = true) {
    const QwModel &md = *c.md;
    const QwDims &d = md.d;
    if (d.ranks == 1) {
        ++c.site;
        return md.b.partial;        // SH == H: the partial is the result
    }
    if (c.fuse && fused) {
        // the kernel that wrote `partial` has sent it; the next down projection adds up the slots
        ++c.site;
        c.pend_site = c.site;
        c.pend_fused = true;
        return out;
    }
    c.pend_fused = false;
    comm(c, 2, md.b.partial, out, c.rows->M, d.SH);
    return out;
}

void ple_block(Ctx &c) {
    const QwModel &md = *c.md;
    const QwDims &d = md.d;
    const QwBuffers &b = md.b;
    const QwRows &r = *c.rows;
    const QwPle &p = md.ple;
    const int M = r.M;
    QW_TRYN(1, qwk_ple_gather(r.ctx3, p.shards, p.scales, p.rows_per_shard, p.rows, p.layout, d.ngram_dim, d.ngram_heads,
                          b.ple_e, nullptr, M, c.s));
    QW_OP(1, p.Wkv, (size_t)d.ple_kv * d.H * 2,
          qwk_gemv_bf16(p.Wkv, b.ple_e, b.ple_kv, nullptr, d.ple_kv, d.H, M, d.H, d.H, d.ple_kv, 0, 1, 0, 0, 0, c.s));
    QW_TRYN(1, qwk_ple_stats(b.ple_kv, d.ple_kv, c.X, p.nk1, p.nq1, d.SH, d.hc, b.ple_send, 16, M, c.s));
    const float *red = b.ple_send;
    if (d.ranks > 1) {
        comm(c, 0, b.ple_send, b.ple_red, M, 16);
        red = b.ple_red;
    } else {
        ++c.site;
    }
    QW_TRYN(3, qwk_ple_apply(b.ple_kv, d.ple_kv, red, 16, p.nc1, p.cw, d.SH, d.hc, d.H, d.eps, d.ple_taps, d.ple_dil,
                         b.ple_gv, b.ple_nc, md.st.ple_ring, c.X, M, r.slot, r.pos, r.run_start, r.run_len, c.s));
}

}  // namespace

// lm_head over the gathered block input, per-row reductions, the vocabulary-parallel argmax merge, and (chained
// steps) the rows' advance to their sampled tokens.
static void head(Ctx &c, int flags) {
    const QwModel *md = c.md;
    const QwDims &d = md->d;
    const QwBuffers &b = md->b;
    const int M = c.rows->M;
    await_bin(c);
    const int ldl = md->logits_ld > 0 ? md->logits_ld : d.vocab_l;      // rows of the logits buffer (a slice of the all-rank matrix, or dense)
    QW_OP(1, c.md->lm_head, (size_t)d.vocab_l * d.H * 2, qwk_gemv_bf16(c.md->lm_head, b.bin, b.logits, nullptr, d.vocab_l, d.H, M, d.H, d.H, ldl, 0, 1, 0, 0, 0,
                         c.s));
    QW_TRYN(1, qwk_row_reduce(b.logits, ldl, d.vocab_l, d.rank * d.vocab_l, M, b.amax_val, b.amax_idx, b.lse_max,
                          b.lse_sum, c.s));
    if (d.ranks > 1 && md->p2p && md->amax_pairs) {
        // vocabulary-parallel argmax: gather every rank's (value, index) and merge on the device
        QW_TRYN(1, qwk_amax_pack(b.amax_val, b.amax_idx, md->amax_pairs, M, d.rank, d.ranks, c.s));
        ++c.site;
        QW_TRYN(1, qwk_p2p_allgather(md->p2p, (unsigned)c.site, 3, md->off_amax, M, 2, 4, c.s));
        QW_TRYN(1, qwk_amax_merge(md->amax_pairs, M, d.ranks, b.amax_idx, b.amax_val, c.s));
    }
    if ((flags & QWRT_CHAIN) && (d.ranks == 1 || md->p2p))
        QW_TRYN(1, qwk_advance_rows(const_cast<int *>(c.rows->tokens), const_cast<int *>(c.rows->pos),
                                const_cast<int *>(c.rows->ctx3), b.amax_idx, M, c.s));
}

// The launch sequence of one step.
static void walk(Ctx &c, int flags, int n_layers_run) {
    const QwModel *md = c.md;
    const QwDims &d = md->d;
    const QwBuffers &b = md->b;
    const int M = c.rows->M;
    c.X = b.X;
    c.Xalt = b.X2;
    c.site = 0;
    c.fuse = d.ranks > 1 && md->p2p && g_fuse;
    c.mute = FUSE_MODE_MAX > 1 && g_fuse == 2;
    c.bin_pending = c.pend_fused = false;
    if (d.ranks > 1 && md->p2p) QW_TRYN(1, qwk_p2p_bump_base(md->p2p, 4096u, c.s));
    QW_TRYN(1, qwk_embed_rows(c.rows->tokens, c.md->embed, d.H, d.rank * d.SH, d.SH, d.hc, d.vocab, b.X, M, c.s));
    const float *pend = nullptr;
    float *inj_attn = b.inj_a, *inj_mlp = b.inj_b;
    for (int l = 0; l < n_layers_run; ++l) {
        const QwLayer &L = c.md->layers[l];
        if (l == d.ple_layer && c.md->ple.enabled) {
            if (pend) QW_TRYN(1, qwk_hc_pre(c.X, pend, d.SH, inj_mlp, d.hc, nullptr, d.SH, d.hc, nullptr, nullptr, 0, M, c.s));
            pend = nullptr;
            ple_block(c);
        }
        mix(c, L.attn_hc, pend, inj_mlp, inj_attn);
        if (L.is_qsa) qsa_block(c, L);
        else gdn_block(c, L, flags);
        const float *out_attn = scatter(c, b.out_a);
        mix(c, L.mlp_hc, out_attn, inj_attn, inj_mlp);
        // the layer before the n-gram embedding layer hands its output to hc_pre, which reads a plain buffer
        const bool fuse_out = !(l + 1 == d.ple_layer && c.md->ple.enabled);
        moe_block(c, L, fuse_out, l);
        // The MoE output stays pending: the next mixer's hc_pre (or the final one) folds it into X
        // before anything overwrites `partial`, so with one rank it can be used in place.
        pend = scatter(c, b.out_b, fuse_out);
    }
    mix(c, c.md->final_hc, pend, inj_mlp, nullptr);
    if ((flags & QWRT_KEEP_HIDDEN) && b.hidden_out)
        cudaMemcpyAsync(b.hidden_out, c.X, sizeof(float) * (size_t)M * d.hc * d.SH, cudaMemcpyDeviceToDevice, c.s);
    if (!(flags & QWRT_NO_HEAD)) head(c, flags);
}

// The MTP pass (see runtime.h).
static void walk_mtp(Ctx &c, int flags) {
    const QwModel *md = c.md;
    const QwDims &d = md->d;
    const QwBuffers &b = md->b;
    const QwMtp &t = md->mtp;
    const int M = c.rows->M;
    c.X = b.X;
    c.Xalt = b.X2;
    c.site = 0;
    c.fuse = d.ranks > 1 && md->p2p && g_fuse;
    c.mute = FUSE_MODE_MAX > 1 && g_fuse == 2;
    c.bin_pending = c.pend_fused = false;
    const float *hidden = b.hidden_out;
    if (d.ranks > 1) {
        // The input norm is one RMS over all hc * H values of a row and the fc products take whole rows: gather the ranks'
        // column slices of the hidden states into a [M*hc][H] matrix inside the symmetric region.  The fc matrices are
        // sliced by output rows, so their products are this rank's columns of the new residual: no collective after them.
        QW_TRYN(1, qwk_p2p_bump_base(md->p2p, 4096u, c.s));
        {
            cudaMemcpy2DAsync(md->mtp_hid + (size_t)d.rank * d.SH, sizeof(float) * (size_t)d.H, b.hidden_out, sizeof(float) * (size_t)d.SH,
                              sizeof(float) * (size_t)d.SH, (size_t)M * d.hc, cudaMemcpyDeviceToDevice, c.s);
        }
        ++c.site;
        QW_TRYN(1, qwk_p2p_allgather(md->p2p, (unsigned)c.site, 3, md->off_mtp_hid, M * d.hc, d.SH, 4, c.s));
        hidden = md->mtp_hid;
    }
    QW_TRYN(1, qwk_mtp_norm(hidden, c.rows->tokens, md->embed, d.vocab, t.nh1, t.ne1, d.H, d.hc, d.eps, t.hn, t.en, M, c.s));
    QW_OP(1, t.fc_h, (size_t)d.SH * d.H * 2,
          qwk_gemv_bf16(t.fc_h, t.hn, t.fh, nullptr, d.SH, d.H, M * d.hc, d.H, d.H, d.SH, 0, 1, 0, 0, 0, c.s));
    QW_OP(1, t.fc_e, (size_t)d.SH * d.H * 2, qwk_gemv_bf16(t.fc_e, t.en, t.fe, nullptr, d.SH, d.H, M, d.H, d.H, d.SH, 0, 1, 0, 0, 0, c.s));
    QW_TRYN(1, qwk_mtp_add(t.fh, t.fe, d.SH, d.hc, c.X, M, c.s));
    float *inj_attn = b.inj_a, *inj_mlp = b.inj_b;
    mix(c, t.layer.attn_hc, nullptr, inj_mlp, inj_attn);
    qsa_block(c, t.layer);
    const float *out_attn = scatter(c, b.out_a);
    mix(c, t.layer.mlp_hc, out_attn, inj_attn, inj_mlp);
    moe_block(c, t.layer, true, d.n_layers);
    const float *pend = scatter(c, b.out_b);
    mix(c, t.final_hc, pend, inj_mlp, nullptr);
    cudaMemcpyAsync(b.hidden_out, c.X, sizeof(float) * (size_t)M * d.hc * d.SH, cudaMemcpyDeviceToDevice, c.s);
    head(c, flags);
}

extern "C" __attribute__((visibility("default"))) int qwrt_decode(const QwModel *md, const QwRows *rows, int flags,
                                                                   int n_layers_run, cudaStream_t stream) {
    Ctx c{};
    c.md = md; c.rows = rows; c.s = stream; c.X = md->b.X; c.Xalt = md->b.X2;
    const QwDims &d = md->d;
    const QwBuffers &b = md->b;
    const int M = rows->M;
    if (M < 1 || M > d.max_rows) return -1;
    if (n_layers_run < 0 || n_layers_run > d.n_layers) n_layers_run = d.n_layers;
    c.launches = 0;
    walk(c, flags, n_layers_run);
    g_last_launches = c.launches;
    return c.err;
}

// Kernels enqueued by the most recent qwrt_decode / qwrt_mtp call (what one replay of its graph launches).
extern "C" __attribute__((visibility("default"))) long long qwrt_last_launches() { return g_last_launches; }

extern "C" __attribute__((visibility("default"))) int qwrt_mtp(const QwModel *md, const QwRows *rows, int flags,
                                                                cudaStream_t stream) {
    if (!md->mtp.enabled || (md->d.ranks != 1 && (!md->p2p || !md->mtp_hid))) return -1;
    const int M = rows->M;
    if (M < 1 || M * md->d.hc > md->d.max_rows * md->d.hc) return -1;
    Ctx c{};
    c.md = md; c.rows = rows; c.s = stream; c.X = md->b.X; c.Xalt = md->b.X2;
    c.launches = 0;
    walk_mtp(c, flags);
    g_last_launches = c.launches;
    return c.err;
}

// All ranks' logits of the last step side by side: with several ranks the logits buffer is this rank's column slice of a
// [rows][vocab] matrix inside the symmetric region (logits_ld = vocab); this gathers the other ranks' slices of rows
// 0..M-1 into it.  Outside the step's graph; `k` must differ from the step's own collective indices (use >= 4000).
extern "C" __attribute__((visibility("default"))) int qwrt_gather_logits(const QwModel *md, int M, unsigned int k, cudaStream_t s) {
    if (md->d.ranks == 1) return 0;
    if (!md->p2p || md->logits_ld <= 0) return -1;
    return qwk_p2p_allgather(md->p2p, k, 3, md->off_logits, M, md->d.vocab_l, 4, s);
}
