// The token-major prefill runtime: enqueues one chunk of T prompt rows of one slot through the whole
// model - every dense product on the tcgen05 GEMM, the routed experts as grouped tcgen05 GEMMs over
// expert-sorted rows with q4 weights converted in the kernel, the chunked GDN scan, tensor-core QSA
// attention over the paged KV - on one rank or on several (tensor + expert parallel, the collectives
// carried by the kernels, tp.cuh), as one or two micro-batches.
//
// Two micro-batches: the chunk's rows are split in two lanes that run the same schedule on two
// streams with two channels, so one lane's exchange and waits hide under the other lane's products.
// The state a layer keeps between rows (GDN state and conv ring, KV pages, compressed keys, raw-key
// ring, PLE ring) is touched in row order: lane 1 waits for an event that lane 0 records after the
// stateful kernels of the same layer.
//
// The schedule is built as a list of single-kernel steps and then executed step by step for every
// job.  A process that drives one GPU passes one job.  A process that emulates several ranks on one
// GPU passes one job per rank with all jobs on one stream: each kernel is then issued for all ranks
// before the next one, so a kernel that waits for other ranks' data finds it complete and never
// spins - which is how the multi-rank path is tested on a single device.
// (Role of the reference's run_prefill_rank, src/engine/prefill.hip:46-496: micro-batches :34-45 and
// :72-110, collective sites :208-224, :318, :340, MTP pass shifted by one row :400-430.)
#include "prefill_rt.h"

#include <functional>
#include <vector>

#include "kernels.h"
#include "tp.cuh"

namespace {

struct Lane {
    int r0, n;
    cudaStream_t s;
    QwTp *tp;
};

struct PCtx {
    const QwPrefillJob *job;
    const QwModel *md;
    const QwPrefillBufs *b;
    Lane lane[3];          // two micro-batch lanes, and [2] the MTP pass (all of its rows on lane 0's stream and channel)
    cudaEvent_t ev[4];     // fork, join, and two alternating state events
    int err;
    long long launches;
};

typedef std::function<void(PCtx &)> Op;

long long g_prefill_launches = 0;
int g_profile = 0;
std::vector<cudaEvent_t> g_prof_ev;
double g_prof_ms[16] = {};

#define PF_TRY(n_, expr)                                                   \
    do {                                                                   \
        int rc__ = (expr);                                                 \
        c.launches += (n_);                                                \
        if (rc__ != 0 && c.err == 0) c.err = rc__ * 1000 - __LINE__;       \
    } while (0)

enum Pend { PEND_NONE = 0, PEND_A = 1, PEND_B = 2 };
enum Inj { INJ_NONE = 0, INJ_A = 1, INJ_B = 2 };

inline float *f_at(float *p, long long row, long long stride) { return p + row * stride; }
inline const float *f_at(const float *p, long long row, long long stride) { return p + row * stride; }
inline void *h_at(void *p, long long row, long long stride) { return (char *)p + row * stride * 2; }      // 16-bit elements
inline int *i_at(int *p, long long row, long long stride) { return p + row * stride; }
inline const int *i_at(const int *p, long long row, long long stride) { return p + row * stride; }

inline float *inj_of(const QwPrefillBufs &b, int which, int r0, int hc) {
    return which == INJ_A ? b.inj_a + (long long)r0 * hc : which == INJ_B ? b.inj_b + (long long)r0 * hc : nullptr;
}

// The block input of lane l: inside the channel's region (lane-relative rows) or the local matrix.
inline const void *bin_of(const PCtx &c, int l) {
    const Lane &L = c.lane[l];
    if (L.tp) return (const char *)L.tp->peer[L.tp->rank] + L.tp->off_buf[2];
    return h_at(c.b->bin, L.r0, c.md->d.H);
}

// Profile categories of a step (qwrt_prefill_profile).
enum Cat { CAT_MIX_GLUE = 0, CAT_MIX_GEMM, CAT_PROJ, CAT_GDN, CAT_QSA, CAT_OUT, CAT_ROUTE, CAT_EXPERTS, CAT_COMBINE, CAT_PLE, CAT_OTHER,
           CAT_MTP, CAT_GUARD, CAT_GLUE_NORM, CAT_GLUE_MID, CAT_GLUE_MIX, CAT_COUNT };

struct Step {
    Op fn;
    int cat, lane;
};

struct Builder {
    std::vector<Step> ops;
    int cur_cat = CAT_OTHER, cur_lane = 0;
    const QwDims d;
    const bool tp;          // several ranks
    const int lanes;
    explicit Builder(const QwPrefillJob &j) : d(j.md->d), tp(j.tp[0] != nullptr), lanes(j.lanes) {}

    void add(Op op) { ops.push_back(Step{std::move(op), cur_cat, cur_lane}); }

    // Two lanes on several ranks: a kernel that spins inside can fill the GPU and keep the other lane's kernels - which
    // another rank may be waiting for - from being scheduled, and two ranks doing that to each other never finish.  So
    // with two lanes every collective is first awaited by a one-block kernel on the consumer's stream; the consumer
    // then finds its flags set.  (With one lane a spinning kernel only ever waits for kernels that peers can run.)
    void guard(int l, int kind) {
        if (!tp || lanes < 2) return;
        const int keep = cur_cat;
        cur_cat = CAT_GUARD;
        cur_lane = l;
        add([=](PCtx &c) {
            const Lane &L = c.lane[l];
            PF_TRY(1, qwk_tp_wait(L.tp, kind, L.s));
        });
        cur_cat = keep;
    }

    // One mixer of lane l: X (+= pending block output) -> block input + injection logits.
    //   hc_sel: 0 attention mixer of layer li, 1 MoE mixer of layer li, 2 the model's final mixer, 3 / 4 / 5 the same of the MTP layer
    void mix(int l, int li, int hc_sel, int pend, int inj_prev, int inj_out) {
        cur_lane = l;
        auto hc_of = [li, hc_sel](const PCtx &c) -> const QwHc & {
            const QwModel &m = *c.md;
            switch (hc_sel) {
                case 0: return m.layers[li].attn_hc;
                case 1: return m.layers[li].mlp_hc;
                case 2: return m.final_hc;
                case 3: return m.mtp.layer.attn_hc;
                case 4: return m.mtp.layer.mlp_hc;
                default: return m.mtp.final_hc;
            }
        };
        const int hc = d.hc, SH = d.SH, R = d.hc_rank, H = d.H;
        if (!tp) {
            cur_cat = CAT_MIX_GLUE;
            add([=](PCtx &c) {
                const Lane &L = c.lane[l];
                const QwPrefillBufs &b = *c.b;
                const float *pe = pend == PEND_A ? b.out_a + (long long)L.r0 * H : pend == PEND_B ? b.out_b + (long long)L.r0 * H : nullptr;
                PF_TRY(1, qwk_hc_prenorm_T(f_at(b.X, L.r0, hc * SH), pe, H, inj_of(b, inj_prev, L.r0, hc), hc_of(c).w1, SH, hc, d.eps,
                                           h_at(b.xn, L.r0, hc * SH), L.n, L.s));
            });
            cur_cat = CAT_MIX_GEMM;
            add([=](PCtx &c) {
                const Lane &L = c.lane[l];
                const QwPrefillBufs &b = *c.b;
                const QwHc &w = hc_of(c);
                PF_TRY(1, qwk_gemm_bf16_tc_splitk(h_at(b.xn, L.r0, hc * SH), w.Wd, f_at(b.d, L.r0, b.hc_ld), L.n, R + w.n_inj, hc * SH,
                                                  hc * SH, hc * SH, b.hc_ld, b.hc_ksplit, (long long)b.cap * b.hc_ld, L.s));
            });
            cur_cat = CAT_GLUE_MID;
            add([=](PCtx &c) {
                const Lane &L = c.lane[l];
                const QwPrefillBufs &b = *c.b;
                const QwHc &w = hc_of(c);
                PF_TRY(1, qwk_hc_mid_T(f_at(b.d, L.r0, b.hc_ld), b.hc_ld, R, w.n_inj, hc, h_at(b.u, L.r0, R), inj_of(b, inj_out, L.r0, hc),
                                       L.n, b.hc_ksplit, (long long)b.cap * b.hc_ld, L.s));
            });
            cur_cat = CAT_MIX_GEMM;
            add([=](PCtx &c) {
                const Lane &L = c.lane[l];
                const QwPrefillBufs &b = *c.b;
                PF_TRY(1, qwk_gemm_bf16_tc(h_at(b.u, L.r0, R), hc_of(c).Wu, f_at(b.g, L.r0, hc * SH), L.n, hc * SH, R, R, R, hc * SH, 0, L.s));
            });
            cur_cat = CAT_GLUE_MIX;
            add([=](PCtx &c) {
                const Lane &L = c.lane[l];
                const QwPrefillBufs &b = *c.b;
                PF_TRY(1, qwk_hc_mix_T(f_at(b.g, L.r0, hc * SH), h_at(b.xn, L.r0, hc * SH), SH, h_at(b.bin, L.r0, H), H, L.n, L.s));
            });
            return;
        }
        // several ranks: the pending block output is the reduce-scatter (kind 3) that the previous block sent
        if (pend != PEND_NONE) guard(l, 3);
        cur_cat = CAT_MIX_GLUE;
        add([=](PCtx &c) {
            const Lane &L = c.lane[l];
            const QwPrefillBufs &b = *c.b;
            PF_TRY(1, qwk_hc_prenorm_tp(L.tp, f_at(b.X, L.r0, hc * SH), nullptr, SH, pend == PEND_NONE ? -1 : 3,
                                        inj_of(b, inj_prev, L.r0, hc), SH, hc, L.n, L.s));
        });
        guard(l, 0);
        cur_cat = CAT_GLUE_NORM;
        add([=](PCtx &c) {
            const Lane &L = c.lane[l];
            const QwPrefillBufs &b = *c.b;
            PF_TRY(1, qwk_hc_norm_tp(L.tp, f_at(b.X, L.r0, hc * SH), hc_of(c).w1, SH, hc, H, d.eps, h_at(b.xn, L.r0, hc * SH), L.n, L.s));
        });
        cur_cat = CAT_MIX_GEMM;
        add([=](PCtx &c) {
            const Lane &L = c.lane[l];
            const QwPrefillBufs &b = *c.b;
            const QwHc &w = hc_of(c);
            PF_TRY(1, qwk_gemm_bf16_tc_tp(L.tp, h_at(b.xn, L.r0, hc * SH), w.Wd, nullptr, L.n, R + w.n_inj, hc * SH, hc * SH, hc * SH,
                                          b.hc_ld, 0, -1, 1, 1, b.hc_ld, L.s));
        });
        guard(l, 1);
        cur_cat = CAT_GLUE_MID;
        add([=](PCtx &c) {
            const Lane &L = c.lane[l];
            const QwPrefillBufs &b = *c.b;
            const QwHc &w = hc_of(c);
            PF_TRY(1, qwk_hc_mid_tp(L.tp, b.hc_ld, R, w.n_inj, hc, h_at(b.u, L.r0, R), inj_of(b, inj_out, L.r0, hc), L.n, L.s));
        });
        cur_cat = CAT_MIX_GEMM;
        add([=](PCtx &c) {
            const Lane &L = c.lane[l];
            const QwPrefillBufs &b = *c.b;
            PF_TRY(1, qwk_gemm_bf16_tc(h_at(b.u, L.r0, R), hc_of(c).Wu, f_at(b.g, L.r0, hc * SH), L.n, hc * SH, R, R, R, hc * SH, 0, L.s));
        });
        cur_cat = CAT_GLUE_MIX;
        add([=](PCtx &c) {
            const Lane &L = c.lane[l];
            const QwPrefillBufs &b = *c.b;
            PF_TRY(1, qwk_hc_mix_tp(L.tp, f_at(b.g, L.r0, hc * SH), h_at(b.xn, L.r0, hc * SH), SH, H, L.n, L.s));
        });
    }

    void hook(int l, int li, int which) {
        cur_lane = l;
        add([=](PCtx &c) {
            if (!c.job->hook) return;
            const Lane &L = c.lane[l];
            c.job->hook(c.job->hook_user, li, which, bin_of(c, l), c.md->d.H, L.r0, L.n);
        });
    }

    // Lane 1 touches a layer's sequential state after lane 0; lane 0 of the next chunk after lane 1 (the join at the chunk's end).
    void state_begin(int l, int slot_ev) {
        if (lanes < 2 || l != 1) return;
        cur_cat = CAT_PROJ;
        cur_cat = CAT_OTHER;
        add([=](PCtx &c) { cudaStreamWaitEvent(c.lane[1].s, c.ev[2 + slot_ev], 0); });
    }
    void state_end(int l, int slot_ev) {
        if (lanes < 2 || l != 0) return;
        cur_cat = CAT_PROJ;
        cur_cat = CAT_OTHER;
        add([=](PCtx &c) { cudaEventRecord(c.ev[2 + slot_ev], c.lane[0].s); });
    }

    // The attention block of a layer for lane l.  mtp: the MTP head's layer with the MTP row tables.
    void attn_block(int l, int li, bool mtp, int ev_slot) {
        cur_lane = l;
        auto layer_of = [li, mtp](const PCtx &c) -> const QwLayer & { return mtp ? c.md->mtp.layer : c.md->layers[li]; };
        const int H = d.H;
        struct RowsAt {
            const int *slot, *pos, *rs, *rl;
        };
        auto rows_of = [mtp](const PCtx &c, const Lane &L) {
            const QwPrefillBufs &b = *c.b;
            if (mtp) return RowsAt{b.m_slot + L.r0, b.m_pos + L.r0, b.m_run_start + L.r0, b.m_run_len + L.r0};
            return RowsAt{b.slot + L.r0, b.pos + L.r0, b.run_start + L.r0, b.run_len + L.r0};
        };
        // projection: reads the gathered block input first
        guard(l, 2);
        cur_cat = CAT_PROJ;
        add([=](PCtx &c) {
            const Lane &L = c.lane[l];
            const QwPrefillBufs &b = *c.b;
            const QwLayer &w = layer_of(c);
            const int N = w.is_qsa ? d.proj_qsa : d.proj_gdn;
            if (L.tp)
                PF_TRY(1, qwk_gemm_bf16_tc_tp(L.tp, bin_of(c, l), w.Wproj, f_at(b.proj, L.r0, b.proj_ld), L.n, N, H, H, H, b.proj_ld, 0, 2, 0, 0,
                                              0, L.s));
            else
                PF_TRY(1, qwk_gemm_bf16_tc(bin_of(c, l), w.Wproj, f_at(b.proj, L.r0, b.proj_ld), L.n, N, H, H, H, b.proj_ld, 0, L.s));
        });
        state_begin(l, ev_slot);
        // stateful part 1 (writes the layer's state)
        cur_cat = CAT_GDN;
        add([=](PCtx &c) {
            const Lane &L = c.lane[l];
            const QwPrefillBufs &b = *c.b;
            const QwLayer &w = layer_of(c);
            const QwState &st = c.md->st;
            const RowsAt r = rows_of(c, L);
            float *proj = f_at(b.proj, L.r0, b.proj_ld);
            if (w.is_qsa) {
                const int qi = w.state_index;
                PF_TRY(1, qwk_qsa_prep(proj, b.proj_ld, d.QL, d.KVL, d.IH, w.qn1, w.kn1, w.iqn1, w.ikn1, L.n, r.slot, r.pos, r.rs, r.rl,
                                       st.k_dev[qi], st.v_dev[qi], st.k_host ? st.k_host[qi] : nullptr, st.v_host ? st.v_host[qi] : nullptr,
                                       d.n_dev_pages, st.page_table, d.max_pages, f_at(b.q, L.r0, d.QL * 256), f_at(b.iq, L.r0, d.IH * 128),
                                       st.raw_ring[qi], st.ck[qi], d.ck_cap, d.idx_ratio, d.eps, L.s));
            } else {
                const int gi = w.state_index;
                const int qkv_l = (2 * d.KL + d.VL) * 128;
                PF_TRY(1, qwk_gdn_conv(proj, b.proj_ld, st.gdn_ring[gi], w.cw, w.A_log, w.dt_bias, d.KL, d.VL, L.n, r.slot, r.pos, r.rs, r.rl,
                                       f_at(b.qkv, L.r0, qkv_l), f_at(b.decay, L.r0, d.VL), f_at(b.beta, L.r0, d.VL), d.eps, L.s));
            }
        });
        // stateful part 2 (GDN: the scan; QSA: nothing else writes state)
        cur_cat = CAT_GDN;
        add([=](PCtx &c) {
            const Lane &L = c.lane[l];
            const QwPrefillBufs &b = *c.b;
            const QwLayer &w = layer_of(c);
            if (w.is_qsa) return;
            const QwState &st = c.md->st;
            const RowsAt r = rows_of(c, L);
            const int gi = w.state_index;
            const int qkv_l = (2 * d.KL + d.VL) * 128;
            PF_TRY(3, qwk_gdn_scan_chunked(f_at(b.qkv, L.r0, qkv_l), f_at(b.decay, L.r0, d.VL), f_at(b.beta, L.r0, d.VL),
                                           f_at(b.proj, L.r0, b.proj_ld), b.proj_ld, st.gdn_S[gi], w.gdn_norm, d.KL, d.VL, L.n, r.slot,
                                           b.gdn_scratch + (long long)(l == 1) * b.gdn_scratch_lane, h_at(b.o, L.r0, b.o_ld), d.eps, L.s));
        });
        state_end(l, ev_slot);
        // QSA: indexer scores, selection, attention (read-only on the state)
        cur_cat = CAT_QSA;
        add([=](PCtx &c) {
            const Lane &L = c.lane[l];
            const QwPrefillBufs &b = *c.b;
            const QwLayer &w = layer_of(c);
            if (!w.is_qsa) return;
            const QwState &st = c.md->st;
            const RowsAt r = rows_of(c, L);
            const int qi = w.state_index;
            const int first_pos = (mtp ? c.job->mtp_base : c.job->base) + L.r0;
            const int max_groups = (first_pos + L.n) / d.idx_ratio;
            PF_TRY(1, qwk_qsa_scores(f_at(b.iq, L.r0, d.IH * 128), d.IH, st.ck[qi], d.ck_cap, L.n, r.slot, r.pos, d.idx_ratio, d.idx_topk,
                                     f_at(b.scores, L.r0, d.score_cap), d.score_cap, max_groups, L.s));
        });
        cur_cat = CAT_QSA;
        add([=](PCtx &c) {
            const Lane &L = c.lane[l];
            const QwPrefillBufs &b = *c.b;
            const QwLayer &w = layer_of(c);
            if (!w.is_qsa) return;
            const RowsAt r = rows_of(c, L);
            PF_TRY(1, qwk_qsa_select(f_at(b.scores, L.r0, d.score_cap), d.score_cap, L.n, r.pos, d.idx_ratio, d.idx_topk,
                                     i_at(b.sel, L.r0, d.idx_topk), b.sel_n + L.r0, L.s));
        });
        cur_cat = CAT_QSA;
        add([=](PCtx &c) {
            const Lane &L = c.lane[l];
            const QwPrefillBufs &b = *c.b;
            const QwLayer &w = layer_of(c);
            if (!w.is_qsa) return;
            const QwState &st = c.md->st;
            const RowsAt r = rows_of(c, L);
            const int qi = w.state_index;
            void *kh = st.k_host ? st.k_host[qi] : nullptr, *vh = st.v_host ? st.v_host[qi] : nullptr;
            // KV spill: the slot's host pages of this layer (the rows this chunk just wrote among them) are copied into
            // the staging buffers and the attention reads them there: a gather of ~2,000 rows per query over the host
            // link costs more than one sequential copy of the pages (host pages of slot s are [s * spill, (s + 1) * spill))
            if (kh && b.stage_k && b.stage_v && c.job->lanes == 1 && d.slots > 0) {
                const int quota = d.n_dev_pages / d.slots, spill = d.max_pages - quota;
                const int last_pos = (mtp ? c.job->mtp_base : c.job->base) + L.r0 + L.n;          // one past the last position
                const int used = (last_pos + 255) / 256 - quota;                                   // host pages in use
                if (spill > 0 && used > 0) {
                    const long long page_bytes = 256ll * d.KVL * 256 * 2;
                    const long long off = (long long)c.job->slot * spill * page_bytes, n = (long long)(used < spill ? used : spill) * page_bytes;
                    if (cudaMemcpyAsync(b.stage_k, (const char *)kh + off, (size_t)n, cudaMemcpyHostToDevice, L.s) != cudaSuccess ||
                        cudaMemcpyAsync(b.stage_v, (const char *)vh + off, (size_t)n, cudaMemcpyHostToDevice, L.s) != cudaSuccess) {
                        if (c.err == 0) c.err = -2000 - __LINE__;
                        return;
                    }
                    c.launches += 2;
                    kh = (char *)b.stage_k - off;
                    vh = (char *)b.stage_v - off;
                }
            }
            PF_TRY(1, qwk_qsa_attend_mma(f_at(b.q, L.r0, d.QL * 256), d.QL, d.KVL, L.n, r.slot, r.pos, st.k_dev[qi], st.v_dev[qi],
                                         kh, vh, d.n_dev_pages,
                                         st.page_table, d.max_pages, i_at(b.sel, L.r0, d.idx_topk), b.sel_n + L.r0, d.idx_topk, d.idx_ratio,
                                         f_at(b.proj, L.r0, b.proj_ld), b.proj_ld, h_at(b.o, L.r0, b.o_ld), L.s));
        });
        // out projection (K depends on the layer kind, which every rank knows alike: resolve when run)
        cur_cat = CAT_OUT;
        add([=](PCtx &c) {
            const Lane &L = c.lane[l];
            const QwPrefillBufs &b = *c.b;
            const QwLayer &w = layer_of(c);
            const int K = w.is_qsa ? d.QL * 256 : d.VL * 128;
            const void *o = h_at(b.o, L.r0, b.o_ld);
            if (L.tp)
                PF_TRY(1, qwk_gemm_bf16_tc_tp(L.tp, o, w.Wout, nullptr, L.n, H, K, b.o_ld, K, H, 0, -1, 2, 3, 0, L.s));
            else
                PF_TRY(1, qwk_gemm_bf16_tc(o, w.Wout, f_at(b.out_a, L.r0, H), L.n, H, K, b.o_ld, K, H, 0, L.s));
        });
    }

    void moe(int l, int li, bool mtp) {
        cur_lane = l;
        auto layer_of = [li, mtp](const PCtx &c) -> const QwLayer & { return mtp ? c.md->mtp.layer : c.md->layers[li]; };
        const int H = d.H, F = d.F, k = d.top_k, E = d.E_l;
        const int nrs = d.E + 1 + 2 * d.SF;
        guard(l, 2);
        cur_cat = CAT_ROUTE;
        add([=](PCtx &c) {
            const Lane &L = c.lane[l];
            const QwPrefillBufs &b = *c.b;
            const QwLayer &w = layer_of(c);
            if (L.tp)
                PF_TRY(1, qwk_gemm_bf16_tc_tp(L.tp, bin_of(c, l), w.Wrs, f_at(b.rs, L.r0, b.nrs_ld), L.n, nrs, H, H, H, b.nrs_ld, 0, 2, 0, 0, 0, L.s));
            else
                PF_TRY(1, qwk_gemm_bf16_tc(bin_of(c, l), w.Wrs, f_at(b.rs, L.r0, b.nrs_ld), L.n, nrs, H, H, H, b.nrs_ld, 0, L.s));
        });
        cur_cat = CAT_ROUTE;
        add([=](PCtx &c) {
            const Lane &L = c.lane[l];
            const QwPrefillBufs &b = *c.b;
            PF_TRY(1, qwk_moe_route(f_at(b.rs, L.r0, b.nrs_ld), b.nrs_ld, L.n, d.E, k, d.SF, c.md->d.e_first, E, i_at(b.pe, L.r0, k),
                                    f_at(b.pw, L.r0, k), h_at(b.sh_h, L.r0, d.SF), L.s));
        });
        cur_cat = CAT_ROUTE;
        add([=](PCtx &c) {
            const Lane &L = c.lane[l];
            const QwPrefillBufs &b = *c.b;
            const long long p0 = (long long)L.r0 * k;
            PF_TRY(3, qwk_moe_sort_T(i_at(b.pe, L.r0, k), L.n, k, E, 2 * F, H, b.max_tiles, b.inv + p0, b.src_token + p0,
                                     (char *)b.t13 + (long long)(l == 1) * b.max_tiles * 16, (char *)b.t2 + (long long)(l == 1) * b.max_tiles * 16, bin_of(c, l), H,
                                     H, h_at(b.xperm, p0, H), L.s));
        });
        cur_cat = CAT_EXPERTS;
        add([=](PCtx &c) {
            const Lane &L = c.lane[l];
            const QwPrefillBufs &b = *c.b;
            const QwLayer &w = layer_of(c);
            const long long p0 = (long long)L.r0 * k;
            PF_TRY(1, qwk_gemm_q4_tc_grouped(h_at(b.xperm, p0, H), w.w13, w.s13, h_at(b.h13, p0, 2 * F),
                                             (char *)b.t13 + (long long)(l == 1) * b.max_tiles * 16, b.max_tiles, L.n * k, (long long)E * 2 * F, 2 * F, H, H,
                                             2 * F, 1, L.s));
        });
        cur_cat = CAT_EXPERTS;
        add([=](PCtx &c) {
            const Lane &L = c.lane[l];
            const QwPrefillBufs &b = *c.b;
            const long long p0 = (long long)L.r0 * k;
            PF_TRY(1, qwk_swiglu_T(h_at(b.h13, p0, 2 * F), F, h_at(b.h, p0, F), (long long)L.n * k, L.s));
        });
        cur_cat = CAT_EXPERTS;
        add([=](PCtx &c) {
            const Lane &L = c.lane[l];
            const QwPrefillBufs &b = *c.b;
            const QwLayer &w = layer_of(c);
            const long long p0 = (long long)L.r0 * k;
            PF_TRY(1, qwk_gemm_q4_tc_grouped(h_at(b.h, p0, F), w.w2, w.s2, f_at(b.y, p0, H),
                                             (char *)b.t2 + (long long)(l == 1) * b.max_tiles * 16, b.max_tiles, L.n * k, (long long)E * H, H, F, F, H, 0,
                                             L.s));
        });
        cur_cat = CAT_COMBINE;
        add([=](PCtx &c) {
            const Lane &L = c.lane[l];
            const QwPrefillBufs &b = *c.b;
            PF_TRY(1, qwk_gemm_bf16_tc(h_at(b.sh_h, L.r0, d.SF), layer_of(c).Wsd, f_at(b.sd, L.r0, H), L.n, H, d.SF, d.SF, d.SF, H, 0, L.s));
        });
        cur_cat = CAT_COMBINE;
        add([=](PCtx &c) {
            const Lane &L = c.lane[l];
            const QwPrefillBufs &b = *c.b;
            const long long p0 = (long long)L.r0 * k;
            if (L.tp)
                PF_TRY(1, qwk_moe_combine_tp(L.tp, f_at(b.y, p0, H), H, b.inv + p0, f_at(b.pw, L.r0, k), k, f_at(b.sd, L.r0, H), H, L.n, L.s));
            else
                PF_TRY(1, qwk_moe_combine_T(f_at(b.y, p0, H), H, b.inv + p0, f_at(b.pw, L.r0, k), k, f_at(b.sd, L.r0, H), H,
                                            f_at(b.out_b, L.r0, H), L.n, L.s));
        });
    }

    // The n-gram embedding layer's extra input, applied to X before the layer's first mixer.
    void ple(int l, int pend, int inj_prev) {
        cur_lane = l;
        const int H = d.H, hc = d.hc, SH = d.SH;
        if (pend != PEND_NONE) {
            if (tp) {
                // fold the pending reduce-scatter into X: reduce its parts to a local matrix first
                guard(l, 3);
                cur_cat = CAT_PLE;
                add([=](PCtx &c) {
                    const Lane &L = c.lane[l];
                    PF_TRY(1, qwk_tp_reduce(L.tp, 3, f_at(c.b->out_b, L.r0, SH), (long long)L.n * SH, L.s));
                });
            }
            cur_cat = CAT_PLE;
            add([=](PCtx &c) {
                const Lane &L = c.lane[l];
                const QwPrefillBufs &b = *c.b;
                const int ld = tp ? SH : H;
                const float *pe = tp ? f_at(b.out_b, L.r0, SH) : (pend == PEND_A ? f_at(b.out_a, L.r0, H) : f_at(b.out_b, L.r0, H));
                PF_TRY(1, qwk_hc_pre(f_at(b.X, L.r0, hc * SH), pe, ld, inj_of(b, inj_prev, L.r0, hc), hc, nullptr, SH, hc, nullptr, nullptr, 0,
                                     L.n, L.s));
            });
        }
        cur_cat = CAT_PLE;
        add([=](PCtx &c) {
            const Lane &L = c.lane[l];
            const QwPrefillBufs &b = *c.b;
            const QwPle &p = c.md->ple;
            PF_TRY(1, qwk_ple_gather(b.ctx3 + 3 * L.r0, p.shards, p.scales, p.rows_per_shard, p.rows, p.layout, d.ngram_dim, d.ngram_heads,
                                     h_at(b.ple_e, L.r0, H), nullptr, L.n, L.s));
        });
        cur_cat = CAT_PLE;
        add([=](PCtx &c) {
            const Lane &L = c.lane[l];
            const QwPrefillBufs &b = *c.b;
            PF_TRY(1, qwk_gemm_bf16_tc(h_at(b.ple_e, L.r0, H), c.md->ple.Wkv, f_at(b.ple_kv, L.r0, b.ple_ld), L.n, d.ple_kv, H, H, H, b.ple_ld, 0,
                                       L.s));
        });
        cur_cat = CAT_PLE;
        add([=](PCtx &c) {
            const Lane &L = c.lane[l];
            const QwPrefillBufs &b = *c.b;
            const QwPle &p = c.md->ple;
            PF_TRY(1, qwk_ple_stats(f_at(b.ple_kv, L.r0, b.ple_ld), b.ple_ld, f_at(b.X, L.r0, hc * SH), p.nk1, p.nq1, SH, hc,
                                    f_at(b.ple_send, L.r0, 16), 16, L.n, L.s));
        });
        if (tp) {
            // all-reduce of the 16 statistics per row, as two steps: every rank sends before any rank adds
            cur_cat = CAT_PLE;
            add([=](PCtx &c) {
                const Lane &L = c.lane[l];
                PF_TRY(1, qwk_tp_push(L.tp, 4, f_at(c.b->ple_send, L.r0, 16), 64, L.n, 64, 0, L.s));
            });
            guard(l, 4);
            cur_cat = CAT_PLE;
            add([=](PCtx &c) {
                const Lane &L = c.lane[l];
                PF_TRY(1, qwk_tp_reduce(L.tp, 4, f_at(c.b->ple_red, L.r0, 16), (long long)L.n * 16, L.s));
            });
        }
        state_begin(l, 0);
        cur_cat = CAT_PLE;
        add([=](PCtx &c) {
            const Lane &L = c.lane[l];
            const QwPrefillBufs &b = *c.b;
            const QwPle &p = c.md->ple;
            const float *red = tp ? f_at(b.ple_red, L.r0, 16) : f_at(b.ple_send, L.r0, 16);
            PF_TRY(3, qwk_ple_apply(f_at(b.ple_kv, L.r0, b.ple_ld), b.ple_ld, red, 16, p.nc1, p.cw, SH, hc, H, d.eps, d.ple_taps, d.ple_dil,
                                    f_at(b.ple_gv, L.r0, hc * SH), f_at(b.ple_nc, L.r0, hc * SH), c.md->st.ple_ring, f_at(b.X, L.r0, hc * SH), L.n,
                                    b.slot + L.r0, b.pos + L.r0, b.run_start + L.r0, b.run_len + L.r0, L.s));
        });
        state_end(l, 0);
    }
};

void build(Builder &B, const QwPrefillJob &j) {
    const QwModel &md = *j.md;
    const QwDims &d = md.d;
    const int lanes = j.lanes;
    const int hc = d.hc, SH = d.SH, H = d.H;
    // embedding rows (and the rows whose embedding the vision tower supplies) for the whole chunk, then the fork: lane 1's
    // stream starts after what the caller's stream holds so far
    B.add([=](PCtx &c) {
        const QwPrefillBufs &b = *c.b;
        cudaStream_t s = c.lane[0].s;
        PF_TRY(1, qwk_embed_rows(b.tokens, c.md->embed, H, c.md->d.rank * SH, SH, hc, d.vocab, b.X, c.job->T, s));
        if (c.job->n_over > 0) PF_TRY(1, qwk_embed_override(b.X, b.over_rows, b.over_emb, H, c.md->d.rank * SH, SH, hc, c.job->n_over, s));
    });
    if (lanes == 2) {
        B.add([](PCtx &c) {
            cudaEventRecord(c.ev[0], c.lane[0].s);
            cudaStreamWaitEvent(c.lane[1].s, c.ev[0], 0);
        });
    }
    int pend = PEND_NONE, inj_prev = INJ_NONE;
    const int n_layers = j.layer_limit < 0 || j.layer_limit > d.n_layers ? d.n_layers : j.layer_limit;
    for (int li = 0; li < n_layers; ++li) {
        const int ev_slot = li & 1;
        for (int l = 0; l < lanes; ++l) {
            if (li == d.ple_layer && md.ple.enabled) B.ple(l, pend, inj_prev);
            const int pend_here = (li == d.ple_layer && md.ple.enabled) ? PEND_NONE : pend;
            B.mix(l, li, 0, pend_here, inj_prev, INJ_A);
            B.hook(l, li, 0);
            B.attn_block(l, li, false, ev_slot);
            B.mix(l, li, 1, PEND_A, INJ_A, INJ_B);
            B.hook(l, li, 1);
            B.moe(l, li, false);
        }
        pend = PEND_B;
        inj_prev = INJ_B;
    }
    for (int l = 0; l < lanes; ++l) B.mix(l, 0, 2, pend, inj_prev, INJ_NONE);
    // join: everything after this runs on the caller's stream
    B.cur_cat = CAT_OTHER;
    B.cur_lane = 0;
    if (lanes == 2) {
        B.add([](PCtx &c) {
            cudaEventRecord(c.ev[1], c.lane[1].s);
            cudaStreamWaitEvent(c.lane[0].s, c.ev[1], 0);
        });
    }
    B.cur_cat = CAT_OTHER;
    B.cur_lane = 0;
    if (j.want_logits) {
        const int ll = lanes - 1;          // the lane that holds the chunk's last row
        if (B.tp) B.add([=](PCtx &c) { PF_TRY(1, qwk_tp_wait(c.lane[ll].tp, 2, c.lane[0].s)); });
        B.add([=](PCtx &c) {
            const Lane &L = c.lane[ll];
            const QwBuffers &mb = c.md->b;
            const void *last = (const char *)bin_of(c, ll) + (long long)(L.n - 1) * H * 2;
            cudaStream_t s = c.lane[0].s;
            PF_TRY(1, qwk_gemv_bf16(c.md->lm_head, last, mb.logits, nullptr, d.vocab_l, H, 1, H, H, d.vocab_l, 0, 1, 0, 0, 0, s));
            PF_TRY(1, qwk_row_reduce(mb.logits, d.vocab_l, d.vocab_l, c.md->d.rank * d.vocab_l, 1, mb.amax_val, mb.amax_idx, mb.lse_max, mb.lse_sum, s));
        });
        if (B.tp) {
            B.add([=](PCtx &c) {
                const QwBuffers &mb = c.md->b;
                PF_TRY(2, qwk_tp_argmax_send(c.lane[0].tp, mb.amax_val, mb.amax_idx, c.b->amax16, 1, c.lane[0].s));
            });
            B.add([=](PCtx &c) {
                const QwBuffers &mb = c.md->b;
                PF_TRY(1, qwk_tp_argmax_merge(c.lane[0].tp, 1, mb.amax_idx, mb.amax_val, c.lane[0].s));
            });
        }
    }
    // ---- MTP pass over the rows whose next token is known, shifted by the pending row of the previous call
    if (j.mtp_rows > 0 && md.mtp.enabled) {
        const int n = j.mtp_rows, hp = j.has_pending ? 1 : 0;
        // the hidden state of the chunk's last position is the next call's pending row
        B.cur_cat = CAT_MTP;
        B.add([=](PCtx &c) {
            const QwPrefillBufs &b = *c.b;
            cudaStream_t s = c.lane[0].s;
            const size_t row = sizeof(float) * (size_t)hc * SH;
            cudaMemcpyAsync(b.hid_out, b.X + (size_t)(c.job->T - 1) * hc * SH, row, cudaMemcpyDeviceToDevice, s);
            if (hp) cudaMemcpyAsync(b.Xm, c.md->b.hidden_out, row, cudaMemcpyDeviceToDevice, s);
            if (n - hp > 0) cudaMemcpyAsync(b.Xm + (size_t)hp * hc * SH, b.X, row * (size_t)(n - hp), cudaMemcpyDeviceToDevice, s);
        });
        if (!B.tp) {
            B.cur_cat = CAT_MTP;
            B.add([=](PCtx &c) {
                const QwPrefillBufs &b = *c.b;
                const QwMtp &t = c.md->mtp;
                PF_TRY(1, qwk_mtp_norm(b.Xm, b.mtp_tok, c.md->embed, d.vocab, t.nh1, t.ne1, H, hc, d.eps, b.hn, b.en, n, c.lane[0].s));
            });
            B.cur_cat = CAT_MTP;
            B.add([=](PCtx &c) {
                const QwPrefillBufs &b = *c.b;
                PF_TRY(1, qwk_gemm_bf16_tc(b.hn, c.md->mtp.fc_h, b.fh, n * hc, H, H, H, H, H, 0, c.lane[0].s));
            });
        } else {
            B.cur_cat = CAT_MTP;
            B.add([=](PCtx &c) {
                const QwPrefillBufs &b = *c.b;
                PF_TRY(1, qwk_mtp_ssq(b.Xm, hc * SH, b.mtp_ssq, n, c.lane[0].s));
            });
            B.cur_cat = CAT_MTP;
            B.add([=](PCtx &c) {
                const int n4 = (n + 3) & ~3;
                PF_TRY(1, qwk_tp_push(c.lane[0].tp, 4, c.b->mtp_ssq, (long long)n4 * 4, 1, n4 * 4, 0, c.lane[0].s));
            });
            B.cur_cat = CAT_MTP;
            B.add([=](PCtx &c) {
                const QwPrefillBufs &b = *c.b;
                PF_TRY(1, qwk_tp_reduce(c.lane[0].tp, 4, b.mtp_ssq + b.cap, (long long)((n + 3) & ~3), c.lane[0].s));
            });
            B.cur_cat = CAT_MTP;
            B.add([=](PCtx &c) {
                const QwPrefillBufs &b = *c.b;
                const QwMtp &t = c.md->mtp;
                PF_TRY(1, qwk_mtp_norm_tp(c.lane[0].tp, b.Xm, b.mtp_ssq + b.cap, b.mtp_tok, c.md->embed, d.vocab, t.nh1, t.ne1, H, hc, d.eps, b.en,
                                          n, c.lane[0].s));
            });
            B.cur_cat = CAT_MTP;
            B.add([=](PCtx &c) {
                const QwPrefillBufs &b = *c.b;
                QwTp *tp = c.lane[0].tp;
                const void *hn = (const char *)tp->peer[tp->rank] + tp->off_buf[5];
                PF_TRY(1, qwk_gemm_bf16_tc_tp(tp, hn, c.md->mtp.fc_h, b.fh, n * hc, SH, H, H, H, SH, 0, 5, 0, 0, 0, c.lane[0].s));
            });
        }
        B.cur_cat = CAT_MTP;
        B.add([=](PCtx &c) {
            const QwPrefillBufs &b = *c.b;
            PF_TRY(1, qwk_gemm_bf16_tc(b.en, c.md->mtp.fc_e, b.fe, n, SH, H, H, H, SH, 0, c.lane[0].s));
        });
        B.cur_cat = CAT_MTP;
        B.add([=](PCtx &c) {
            const QwPrefillBufs &b = *c.b;
            PF_TRY(1, qwk_mtp_add(b.fh, b.fe, SH, hc, b.X, n, c.lane[0].s));
        });
        B.mix(2, 0, 3, PEND_NONE, INJ_NONE, INJ_A);
        B.attn_block(2, 0, true, 0);
        B.mix(2, 0, 4, PEND_A, INJ_A, INJ_B);
        B.moe(2, 0, true);
        // the MTP layer's output is not needed for prompt rows: only its KV / indexer state matters.  On several ranks the
        // reduce-scatter of its MoE output stays unconsumed, which the next collective of that kind simply overwrites.
    }
}

cudaEvent_t *events_for_device() {
    static cudaEvent_t ev[64][4];
    static bool made[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (!made[dev]) {
        for (int i = 0; i < 4; ++i) cudaEventCreateWithFlags(&ev[dev][i], cudaEventDisableTiming);
        made[dev] = true;
    }
    return ev[dev];
}

}  // namespace

extern "C" __attribute__((visibility("default"))) int qwrt_prefill(const QwPrefillJob *const *jobs, int njobs) {
    if (njobs < 1 || njobs > 8) return -1;
    const QwPrefillJob &j0 = *jobs[0];
    if (j0.T < 1 || j0.T > j0.b->cap || j0.lanes < 1 || j0.lanes > 2) return -1;
    if (j0.lanes == 2 && (njobs > 1 || j0.T < 2)) return -1;          // emulated ranks share one stream: one lane
    std::vector<PCtx> ctx(njobs);
    cudaEvent_t *ev = events_for_device();
    for (int i = 0; i < njobs; ++i) {
        const QwPrefillJob &j = *jobs[i];
        if (j.T != j0.T || j.lanes != j0.lanes || j.mtp_rows != j0.mtp_rows || (j.tp[0] == nullptr) != (j0.tp[0] == nullptr)) return -1;
        PCtx &c = ctx[i];
        c.job = &j; c.md = j.md; c.b = j.b; c.err = 0; c.launches = 0;
        for (int e = 0; e < 4; ++e) c.ev[e] = ev[e];
        int n0 = j.T;
        if (j.lanes == 2) {
            n0 = j.n0;
            if (n0 < 1 || n0 >= j.T || n0 != j0.n0) return -1;
        }
        c.lane[0] = Lane{0, n0, j.stream[0], (QwTp *)j.tp[0]};
        c.lane[1] = Lane{n0, j.T - n0, j.stream[1], (QwTp *)j.tp[1]};
        c.lane[2] = Lane{0, j.mtp_rows, j.stream[0], (QwTp *)j.tp[0]};
    }
    Builder B(j0);
    build(B, j0);
    if (g_profile && njobs == 1) {
        // every step between two events on its stream; read back after the chunk (the streams are synchronised: a diagnostic)
        const size_t n = B.ops.size();
        if (g_prof_ev.size() < 2 * n) {
            const size_t old = g_prof_ev.size();
            g_prof_ev.resize(2 * n);
            for (size_t k = old; k < 2 * n; ++k) cudaEventCreate(&g_prof_ev[k]);
        }
        for (size_t k = 0; k < n; ++k) {
            cudaStream_t s = ctx[0].lane[B.ops[k].lane].s;
            cudaEventRecord(g_prof_ev[2 * k], s);
            B.ops[k].fn(ctx[0]);
            cudaEventRecord(g_prof_ev[2 * k + 1], s);
        }
        cudaStreamSynchronize(ctx[0].lane[0].s);
        cudaStreamSynchronize(ctx[0].lane[1].s);
        for (size_t k = 0; k < n; ++k) {
            float ms = 0.f;
            if (cudaEventElapsedTime(&ms, g_prof_ev[2 * k], g_prof_ev[2 * k + 1]) == cudaSuccess) g_prof_ms[B.ops[k].cat] += ms;
        }
    } else {
        for (size_t k = 0; k < B.ops.size(); ++k)
            for (int i = 0; i < njobs; ++i) B.ops[k].fn(ctx[i]);
    }
    long long launches = 0;
    int err = 0;
    for (auto &c : ctx) {
        launches += c.launches;
        if (c.err && !err) err = c.err;
    }
    g_prefill_launches = launches;
    return err;
}

extern "C" __attribute__((visibility("default"))) long long qwrt_prefill_sizes(int which) {
    return which == 0 ? (long long)sizeof(QwPrefillBufs) : which == 1 ? (long long)sizeof(QwPrefillJob) : (long long)sizeof(QwTp);
}

extern "C" __attribute__((visibility("default"))) long long qwrt_prefill_last_launches(void) { return g_prefill_launches; }

// Profiling of the chunks that follow (one job per call): device time of every step, added up per category
// (mixer glue, mixer GEMMs, projection, GDN, QSA, out projection, routing, expert GEMMs, shared down + combine, PLE, other,
// MTP pass, guard waits).  qwrt_prefill_profile_read copies the sums (milliseconds) out and clears them.
extern "C" __attribute__((visibility("default"))) int qwrt_prefill_profile(int on) {
    g_profile = on;
    return 0;
}
extern "C" __attribute__((visibility("default"))) int qwrt_prefill_profile_read(double *out, int n) {
    for (int i = 0; i < n && i < 16; ++i) {
        out[i] = g_prof_ms[i];
        g_prof_ms[i] = 0.0;
    }
    return CAT_COUNT;
}
