// CPU fp32 reference of the forward pass, read straight from the memory-mapped checkpoint: one sequence, one
// token per call, every intermediate fp32 (norm statistics in double), weights at their stored precision
// (bf16 dense rows, int4 g128 experts dequantised on the fly).  It is the oracle the engine's logits are
// compared with (the role of the reference's src/ref/ref_model.cpp:86-531; the math follows its docs/MODEL.md).
#pragma once
#include <algorithm>
#include <cmath>
#include <memory>
#include <numeric>

#include "json.hpp"
#include "ngram_ple.hpp"
#include "safetensors.hpp"
#include "threadpool.hpp"

namespace qwh {

struct RefConfig {
    int hidden = 2560, hc = 4, hc_rank = 320, n_layers = 48, vocab = 248320, eos = 248044;
    int image_pad = 248056, video_pad = 248057, qsa_every = 4;
    int q_heads = 24, kv_heads = 2, head_dim = 256, rope_dim = 64, idx_heads = 4, idx_dim = 128, idx_budget = 2048, idx_ratio = 4;
    int gdn_qk_heads = 16, gdn_v_heads = 48, gdn_dim = 128, gdn_conv = 4;
    int n_experts = 512, top_k = 10, ffn = 640, qgroup = 128;
    int ple_layer = 1, ngram = 3, ngram_heads = 16, ple_conv = 4, ple_dilation = 3;
    int64_t ngram_vocab_base = 20000000;
    uint64_t ple_seed = 1234;
    double rope_theta = 1e7, eps = 1e-6;
    std::vector<int> layer_is_qsa;      // empty: layer i is QSA when i % qsa_every == qsa_every - 1

    int hch() const { return hc * hidden; }
    bool is_qsa(int l) const { return layer_is_qsa.empty() ? l % qsa_every == qsa_every - 1 : layer_is_qsa[size_t(l)] != 0; }
    int index_of(int l, bool qsa) const { int n = 0; for (int i = 0; i < l; ++i) n += is_qsa(i) == qsa; return n; }
    int topk_blocks() const { return idx_budget / idx_ratio; }
    int gdn_key() const { return gdn_qk_heads * gdn_dim; }
    int gdn_val() const { return gdn_v_heads * gdn_dim; }
    int gdn_qkv() const { return 2 * gdn_key() + gdn_val(); }

    // config.json of the checkpoint (HF keys, optionally under text_config); an object "qw" may override any field by name.
    static RefConfig from_json(const Json &root) {
        RefConfig c;
        const Json &t = root.has("text_config") ? root["text_config"] : root;
        auto geti = [&](const Json &j, const char *k, int &v) { if (j.has(k)) v = int(j[k].as_int()); };
        geti(t, "hidden_size", c.hidden); geti(t, "num_hidden_layers", c.n_layers); geti(t, "vocab_size", c.vocab);
        geti(t, "num_attention_heads", c.q_heads); geti(t, "num_key_value_heads", c.kv_heads); geti(t, "head_dim", c.head_dim);
        geti(t, "num_experts", c.n_experts); geti(t, "num_experts_per_tok", c.top_k); geti(t, "moe_intermediate_size", c.ffn);
        geti(t, "hc_count", c.hc); geti(t, "hc_lowrank", c.hc_rank); geti(t, "linear_num_key_heads", c.gdn_qk_heads);
        geti(t, "linear_num_value_heads", c.gdn_v_heads); geti(t, "linear_key_head_dim", c.gdn_dim);
        geti(t, "linear_conv_kernel_dim", c.gdn_conv);
        if (root.has("qw")) {
            const Json &q = root["qw"];
            geti(q, "hidden", c.hidden); geti(q, "hc", c.hc); geti(q, "hc_rank", c.hc_rank); geti(q, "n_layers", c.n_layers);
            geti(q, "vocab", c.vocab); geti(q, "eos", c.eos); geti(q, "image_pad", c.image_pad); geti(q, "video_pad", c.video_pad);
            geti(q, "qsa_every", c.qsa_every); geti(q, "q_heads", c.q_heads); geti(q, "kv_heads", c.kv_heads);
            geti(q, "head_dim", c.head_dim); geti(q, "rope_dim", c.rope_dim); geti(q, "idx_heads", c.idx_heads);
            geti(q, "idx_dim", c.idx_dim); geti(q, "idx_budget", c.idx_budget); geti(q, "idx_ratio", c.idx_ratio);
            geti(q, "gdn_qk_heads", c.gdn_qk_heads); geti(q, "gdn_v_heads", c.gdn_v_heads); geti(q, "gdn_dim", c.gdn_dim);
            geti(q, "gdn_conv", c.gdn_conv); geti(q, "n_experts", c.n_experts); geti(q, "top_k", c.top_k); geti(q, "ffn", c.ffn);
            geti(q, "qgroup", c.qgroup); geti(q, "ple_layer", c.ple_layer); geti(q, "ngram", c.ngram);
            geti(q, "ngram_heads", c.ngram_heads); geti(q, "ple_conv", c.ple_conv); geti(q, "ple_dilation", c.ple_dilation);
            if (q.has("ngram_vocab_base")) c.ngram_vocab_base = q["ngram_vocab_base"].as_int();
            if (q.has("ple_seed")) c.ple_seed = uint64_t(q["ple_seed"].as_int());
            if (q.has("rope_theta")) c.rope_theta = q["rope_theta"].as_double();
            if (q.has("eps")) c.eps = q["eps"].as_double();
            if (q.has("layer_types"))
                for (auto &e : q["layer_types"].arr) c.layer_is_qsa.push_back(e.as_str() == "qsa");
        }
        return c;
    }
};

class RefModel {
public:
    RefModel(const std::string &model_dir, const std::string &ple_dir, int threads = 0)
        : pool_(threads > 0 ? threads : int(std::max(1u, std::thread::hardware_concurrency()))) {
        cfg = RefConfig::from_json(Json::parse(PleTable::read_file(model_dir + "/config.json")));
        st_.add_dir(model_dir);
        NgramSpec ns;
        ns.vocab = cfg.vocab; ns.eos = cfg.eos; ns.ngram = cfg.ngram; ns.heads = cfg.ngram_heads; ns.image_pad = cfg.image_pad;
        ns.video_pad = cfg.video_pad; ns.vocab_base = cfg.ngram_vocab_base; ns.seed = cfg.ple_seed;
        hasher_ = std::make_unique<NgramHasher>(ns);
        if (!ple_dir.empty()) table_ = std::make_unique<PleTable>(ple_dir, cfg.hidden / cfg.ngram_heads);      // one row per n-gram head
        reset();
    }

    RefConfig cfg;

    void reset() {
        const RefConfig &c = cfg;
        int n_gdn = 0, n_qsa = 0;
        for (int l = 0; l < c.n_layers; ++l) (c.is_qsa(l) ? n_qsa : n_gdn)++;
        gdn_conv_.assign(static_cast<size_t>(n_gdn), std::vector<float>(static_cast<size_t>(c.gdn_conv - 1) * c.gdn_qkv(), 0.f));
        gdn_S_.assign(static_cast<size_t>(n_gdn), std::vector<float>(static_cast<size_t>(c.gdn_v_heads) * c.gdn_dim * c.gdn_dim, 0.f));
        qsa_.assign(size_t(n_qsa), Cache());
        ple_hist_.assign(size_t(c.ple_conv - 1) * c.ple_dilation * c.hch(), 0.f);
        tokens_.clear();
    }
    int n_tokens() const { return int(tokens_.size()); }

    // Appends one token; returns its logits [vocab].
    std::vector<float> forward(int token) {
        const RefConfig &c = cfg;
        const int H = c.hidden, HCH = c.hch();
        const int real = token >= 0 ? token : (((-token) & 1) ? c.image_pad : c.video_pad);
        std::vector<float> X(static_cast<size_t>(HCH));
        {
            const TensorView &e = dense("embed_tokens.weight");
            const uint16_t *row = reinterpret_cast<const uint16_t *>(e.data) + size_t(real) * H;
            for (int s = 0; s < c.hc; ++s)
                for (int i = 0; i < H; ++i) X[size_t(s) * H + i] = bf16_to_f32(row[i]);
        }
        std::vector<float> pend_out, pend_inj;
        const int pos = n_tokens();
        for (int l = 0; l < c.n_layers; ++l) {
            const std::string p = "layers." + std::to_string(l) + ".";
            if (!pend_out.empty()) combine(X, pend_out, pend_inj);
            if (l == c.ple_layer && table_) ple(X, token);
            std::vector<float> a_in, a_inj;
            hc_mix(p + "attn_hyper_connection.", X, true, a_in, a_inj);
            std::vector<float> a_out = c.is_qsa(l) ? qsa(qsa_[size_t(c.index_of(l, true))], p + "self_attn.", a_in, pos)
                                                   : gdn(c.index_of(l, false), p + "linear_attn.", a_in);
            combine(X, a_out, a_inj);
            std::vector<float> m_in;
            hc_mix(p + "mlp_hyper_connection.", X, true, m_in, pend_inj);
            pend_out = moe(p + "mlp.", m_in);
        }
        combine(X, pend_out, pend_inj);
        std::vector<float> y, none;
        hc_mix("hyper_connection_mixer.", X, false, y, none);
        tokens_.push_back(token);
        return linear("lm_head.weight", y);
    }

private:
    struct Cache { std::vector<std::vector<float>> k, v, raw, ck; };

    static std::string full(const std::string &n) { return "model.language_model." + n; }
    const TensorView &dense(const std::string &n) const { return st_.get(full(n)); }

    // y = W x for a bf16 matrix [out][in], rows in parallel
    std::vector<float> linear(const std::string &name, const std::vector<float> &x) {
        const TensorView &t = dense(name);
        QWH_CHECK(t.dtype == DType::BF16 && t.shape.size() == 2 && size_t(t.shape[1]) == x.size(), name + ": shape");
        const int64_t out = t.shape[0], in = t.shape[1];
        std::vector<float> y(static_cast<size_t>(out), 0.f);
        const uint16_t *w = reinterpret_cast<const uint16_t *>(t.data);
        pool_.parallel_for(out, 64, [&](int64_t a, int64_t b) {
            for (int64_t r = a; r < b; ++r) {
                const uint16_t *row = w + r * in;
                float acc = 0.f;
                for (int64_t i = 0; i < in; ++i) acc += bf16_to_f32(row[i]) * x[size_t(i)];
                y[size_t(r)] = acc;
            }
        });
        return y;
    }
    std::vector<float> vec(const std::string &name) const {
        const TensorView &t = dense(name);
        std::vector<float> v(static_cast<size_t>(t.numel()));
        const uint16_t *p = reinterpret_cast<const uint16_t *>(t.data);
        if (t.dtype == DType::BF16) for (size_t i = 0; i < v.size(); ++i) v[i] = bf16_to_f32(p[i]);
        else if (t.dtype == DType::F32) std::memcpy(v.data(), t.data, v.size() * 4);
        else fail(name + ": dtype");
        return v;
    }
    // y = W x for one routed expert's int4 g128 matrix (checkpoint nibble order: element i of a word at bits 4 i, value + 8)
    std::vector<float> expert_linear(const std::string &prefix, const std::vector<float> &x) const {
        const TensorView &pk = st_.get(full(prefix + ".weight_packed")), &sc = st_.get(full(prefix + ".weight_scale"));
        const int64_t out = pk.shape[0], words = pk.shape[1], groups = sc.shape[1];
        QWH_CHECK(size_t(words) * 8 == x.size(), prefix + ": shape");
        const uint32_t *w = reinterpret_cast<const uint32_t *>(pk.data);
        const uint16_t *s = reinterpret_cast<const uint16_t *>(sc.data);
        const int64_t gw = words / groups;
        std::vector<float> y(static_cast<size_t>(out));
        for (int64_t r = 0; r < out; ++r) {
            float acc = 0.f;
            for (int64_t g = 0; g < groups; ++g) {
                float part = 0.f;
                for (int64_t j = g * gw; j < (g + 1) * gw; ++j) {
                    const uint32_t word = w[r * words + j];
                    for (int i = 0; i < 8; ++i) part += float(int((word >> (4 * i)) & 15u) - 8) * x[size_t(j * 8 + i)];
                }
                acc += part * bf16_to_f32(s[r * groups + g]);
            }
            y[size_t(r)] = acc;
        }
        return y;
    }

    static float sigmoid(float v) { return 1.f / (1.f + std::exp(-v)); }
    static float silu(float v) { return v * sigmoid(v); }
    // x * rsqrt(mean(x^2) + eps) over n values (statistics in double)
    float rms_scale(const float *x, int n) const {
        double s = 0;
        for (int i = 0; i < n; ++i) s += double(x[i]) * x[i];
        return float(1.0 / std::sqrt(s / n + cfg.eps));
    }
    void gemma_norm(float *x, const float *w, int n) const {
        const float r = rms_scale(x, n);
        for (int i = 0; i < n; ++i) x[i] = x[i] * r * (1.f + w[i]);
    }
    // NeoX rotation of the first rope_dim dims
    void rope(float *x, int pos) const {
        const int half = cfg.rope_dim / 2;
        for (int i = 0; i < half; ++i) {
            const double inv = std::pow(cfg.rope_theta, -2.0 * i / cfg.rope_dim);
            const float cs = float(std::cos(pos * inv)), sn = float(std::sin(pos * inv));
            const float a = x[i], b = x[i + half];
            x[i] = a * cs - b * sn;
            x[i + half] = b * cs + a * sn;
        }
    }

    void hc_mix(const std::string &p, const std::vector<float> &X, bool inject, std::vector<float> &block_in, std::vector<float> &inj) {
        const RefConfig &c = cfg;
        const int H = c.hidden;
        std::vector<float> xn = X, w = vec(p + "hc_norm.weight");
        for (int s = 0; s < c.hc; ++s) gemma_norm(xn.data() + size_t(s) * H, w.data() + size_t(s) * H, H);
        std::vector<float> d = linear(p + "input_mix_weight_down.weight", xn);
        if (inject) inj = linear(p + "block_inject_weight.weight", xn);
        for (auto &v : d) v = silu(v / float(c.hc));
        std::vector<float> g = linear(p + "input_mix_weight_up.weight", d);
        block_in.assign(size_t(H), 0.f);
        for (int s = 0; s < c.hc; ++s)
            for (int i = 0; i < H; ++i) block_in[size_t(i)] += sigmoid(g[size_t(s) * H + i]) * xn[size_t(s) * H + i];
        for (auto &v : block_in) v /= float(c.hc);
    }
    void combine(std::vector<float> &X, const std::vector<float> &out, const std::vector<float> &inj) const {
        const int H = cfg.hidden;
        for (int s = 0; s < cfg.hc; ++s) {
            const float w = 2.f * sigmoid(inj[size_t(s)] / float(cfg.hc));
            for (int i = 0; i < H; ++i) X[size_t(s) * H + i] += w * out[size_t(i)];
        }
    }

    void ple(std::vector<float> &X, int token) {
        const RefConfig &c = cfg;
        const int H = c.hidden, HCH = c.hch();
        const std::string p = "layers." + std::to_string(c.ple_layer) + ".ple.";
        int32_t hist[2];
        const int nh = std::min<int>(2, n_tokens());
        for (int i = 0; i < nh; ++i) hist[i] = tokens_[tokens_.size() - size_t(nh) + size_t(i)];
        std::vector<int64_t> ids(static_cast<size_t>(c.ngram_heads));
        const int32_t tk = token;
        hasher_->ids_for(hist, nh, &tk, 1, ids.data());
        std::vector<float> e(static_cast<size_t>(H));
        table_->gather(ids.data(), 1, c.ngram_heads, e.data(), &pool_);
        std::vector<float> key = linear(p + "key_proj.weight", e), val = linear(p + "value_proj.weight", e);
        std::vector<float> nk = vec(p + "norm_key.weight"), nq = vec(p + "norm_query.weight"), ncw = vec(p + "norm_conv.weight");
        std::vector<float> q = X, gv(static_cast<size_t>(HCH), 0.f), nc(static_cast<size_t>(HCH), 0.f);
        for (int s = 0; s < c.hc; ++s) {
            gemma_norm(key.data() + size_t(s) * H, nk.data() + size_t(s) * H, H);
            gemma_norm(q.data() + size_t(s) * H, nq.data() + size_t(s) * H, H);
            float gs = 0.f;
            for (int i = 0; i < H; ++i) gs += key[size_t(s) * H + i] * q[size_t(s) * H + i];
            gs /= std::sqrt(float(H));
            const float mag = std::sqrt(std::max(std::fabs(gs), 1e-6f));
            const float gate = sigmoid((gs > 0.f ? 1.f : gs < 0.f ? -1.f : 0.f) * mag);
            for (int i = 0; i < H; ++i) gv[size_t(s) * H + i] = nc[size_t(s) * H + i] = gate * val[size_t(i)];
            gemma_norm(nc.data() + size_t(s) * H, ncw.data() + size_t(s) * H, H);
        }
        // dilated causal conv over the history ring [hist rows][hch] + this row
        const int histn = (c.ple_conv - 1) * c.ple_dilation;
        std::vector<float> cw = vec(p + "conv1d.weight");      // [hch][conv]
        for (int ch = 0; ch < HCH; ++ch) {
            float acc = 0.f;
            for (int k = 0; k < c.ple_conv; ++k) {
                const int row = k * c.ple_dilation;            // index into [hist..., new]
                const float v = row < histn ? ple_hist_[size_t(row) * HCH + ch] : nc[size_t(ch)];
                acc += cw[size_t(ch) * c.ple_conv + k] * v;
            }
            X[size_t(ch)] += gv[size_t(ch)] + silu(acc);
        }
        // shift the history by one row
        std::move(ple_hist_.begin() + HCH, ple_hist_.end(), ple_hist_.begin());
        std::copy(nc.begin(), nc.end(), ple_hist_.end() - HCH);
    }

    std::vector<float> gdn(int gi, const std::string &p, const std::vector<float> &x) {
        const RefConfig &c = cfg;
        const int D = c.gdn_dim, QKV = c.gdn_qkv(), KEY = c.gdn_key();
        std::vector<float> qkv = linear(p + "in_proj_qkv.weight", x), z = linear(p + "in_proj_z.weight", x);
        std::vector<float> b = linear(p + "in_proj_b.weight", x), a = linear(p + "in_proj_a.weight", x);
        std::vector<float> cw = vec(p + "conv1d.weight");       // [qkv][conv]
        std::vector<float> &ring = gdn_conv_[size_t(gi)];       // [conv-1][qkv], oldest first
        std::vector<float> act(static_cast<size_t>(QKV));
        for (int ch = 0; ch < QKV; ++ch) {
            float acc = 0.f;
            for (int k = 0; k < c.gdn_conv; ++k)
                acc += cw[size_t(ch) * c.gdn_conv + k] * (k < c.gdn_conv - 1 ? ring[size_t(k) * QKV + ch] : qkv[size_t(ch)]);
            act[size_t(ch)] = silu(acc);
        }
        std::move(ring.begin() + QKV, ring.end(), ring.begin());
        std::copy(qkv.begin(), qkv.end(), ring.end() - QKV);
        std::vector<float> A = vec(p + "A_log"), dt = vec(p + "dt_bias"), nw = vec(p + "norm.weight");
        const int rep = c.gdn_v_heads / c.gdn_qk_heads;
        std::vector<float> o(static_cast<size_t>(c.gdn_val()));
        std::vector<float> &S = gdn_S_[size_t(gi)];             // [vh][k][v]
        for (int h = 0; h < c.gdn_v_heads; ++h) {
            const int kh = h / rep;
            const float *qh = act.data() + size_t(kh) * D, *kh_ = act.data() + KEY + size_t(kh) * D;
            const float *vh = act.data() + 2 * KEY + size_t(h) * D;
            float qs = 0.f, ksq = 0.f;
            for (int i = 0; i < D; ++i) { qs += qh[i] * qh[i]; ksq += kh_[i] * kh_[i]; }
            const float qn = 1.f / std::sqrt(qs + float(c.eps)) / std::sqrt(float(D)), kn = 1.f / std::sqrt(ksq + float(c.eps));
            const float sp_in = a[size_t(h)] + dt[size_t(h)];
            const float sp = sp_in > 20.f ? sp_in : std::log1p(std::exp(sp_in));
            const float decay = std::exp(-std::exp(A[size_t(h)]) * sp), beta = sigmoid(b[size_t(h)]);
            float *Sh = S.data() + size_t(h) * D * D;
            std::vector<float> u(static_cast<size_t>(D));
            for (int v = 0; v < D; ++v) {
                float dot = 0.f;
                for (int k = 0; k < D; ++k) dot += Sh[size_t(k) * D + v] * decay * (kh_[k] * kn);
                u[size_t(v)] = (vh[v] - dot) * beta;
            }
            float ssq = 0.f;
            float *oh = o.data() + size_t(h) * D;
            for (int v = 0; v < D; ++v) {
                float acc = 0.f;
                for (int k = 0; k < D; ++k) {
                    float &s = Sh[size_t(k) * D + v];
                    s = s * decay + (kh_[k] * kn) * u[size_t(v)];
                    acc += s * (qh[k] * qn);
                }
                oh[v] = acc;
                ssq += acc * acc;
            }
            const float r = float(1.0 / std::sqrt(double(ssq) / D + c.eps));
            for (int v = 0; v < D; ++v) oh[v] = oh[v] * r * nw[size_t(v)] * sigmoid(z[size_t(h) * D + v]);
        }
        return linear(p + "out_proj.weight", o);
    }

    std::vector<float> qsa(Cache &cache, const std::string &p, const std::vector<float> &x, int pos) {
        const RefConfig &c = cfg;
        const int D = c.head_dim, ID = c.idx_dim;
        std::vector<float> qg = linear(p + "q_proj.weight", x);       // [q_heads][2][D]: query, gate
        std::vector<float> k = linear(p + "k_proj.weight", x), v = linear(p + "v_proj.weight", x);
        std::vector<float> iq = linear(p + "indexer.index_qk_proj.weight", x);
        std::vector<float> qn = vec(p + "q_norm.weight"), kn = vec(p + "k_norm.weight");
        std::vector<float> iqn = vec(p + "indexer.q_layernorm.weight"), ikn = vec(p + "indexer.k_layernorm.weight");
        for (int h = 0; h < c.q_heads; ++h) { float *q = qg.data() + size_t(h) * 2 * D; gemma_norm(q, qn.data(), D); rope(q, pos); }
        for (int h = 0; h < c.kv_heads; ++h) { float *kk = k.data() + size_t(h) * D; gemma_norm(kk, kn.data(), D); rope(kk, pos); }
        for (int h = 0; h < c.idx_heads; ++h) { float *q = iq.data() + size_t(h) * ID; gemma_norm(q, iqn.data(), ID); rope(q, pos); }
        cache.k.push_back(k);
        cache.v.push_back(v);
        cache.raw.emplace_back(iq.begin() + size_t(c.idx_heads) * ID, iq.end());
        if ((pos + 1) % c.idx_ratio == 0) {
            std::vector<float> mean(static_cast<size_t>(ID), 0.f);
            for (int t = pos + 1 - c.idx_ratio; t <= pos; ++t)
                for (int i = 0; i < ID; ++i) mean[size_t(i)] += cache.raw[size_t(t)][size_t(i)];
            for (auto &m : mean) m /= float(c.idx_ratio);
            gemma_norm(mean.data(), ikn.data(), ID);
            rope(mean.data(), pos + 1 - c.idx_ratio);
            cache.ck.push_back(mean);
        }
        // positions attended by this query
        std::vector<int> sel;
        const int nb = (pos + 1) / c.idx_ratio, topk = c.topk_blocks();
        if (nb <= topk) {
            sel.resize(size_t(pos + 1));
            std::iota(sel.begin(), sel.end(), 0);
        } else {
            std::vector<float> score(static_cast<size_t>(nb), 0.f);
            for (int g = 0; g < nb; ++g) {
                float s = 0.f;
                for (int h = 0; h < c.idx_heads; ++h) {
                    float d = 0.f;
                    for (int i = 0; i < ID; ++i) d += cache.ck[size_t(g)][size_t(i)] * iq[size_t(h) * ID + i];
                    s += std::max(d, 0.f);
                }
                score[size_t(g)] = s / std::sqrt(float(ID));
            }
            std::vector<int> order(static_cast<size_t>(nb), 0);
            std::iota(order.begin(), order.end(), 0);
            std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return score[size_t(a)] > score[size_t(b)]; });
            for (int j = 0; j < topk; ++j)
                for (int t = 0; t < c.idx_ratio; ++t) sel.push_back(order[size_t(j)] * c.idx_ratio + t);
            for (int t = nb * c.idx_ratio; t <= pos; ++t) sel.push_back(t);
        }
        const int rep = c.q_heads / c.kv_heads;
        std::vector<float> o(static_cast<size_t>(c.q_heads) * D);
        for (int h = 0; h < c.q_heads; ++h) {
            const float *q = qg.data() + size_t(h) * 2 * D, *gate = q + D;
            const int kvh = h / rep;
            std::vector<double> logit(sel.size());
            double mx = -1e300;
            for (size_t j = 0; j < sel.size(); ++j) {
                const float *kk = cache.k[size_t(sel[j])].data() + size_t(kvh) * D;
                float d = 0.f;
                for (int i = 0; i < D; ++i) d += q[i] * kk[i];
                logit[j] = double(d / std::sqrt(float(D)));
                mx = std::max(mx, logit[j]);
            }
            double sum = 0;
            for (auto &l : logit) { l = std::exp(l - mx); sum += l; }
            float *oh = o.data() + size_t(h) * D;
            std::fill(oh, oh + D, 0.f);
            for (size_t j = 0; j < sel.size(); ++j) {
                const float w = float(logit[j] / sum);
                const float *vv = cache.v[size_t(sel[j])].data() + size_t(kvh) * D;
                for (int i = 0; i < D; ++i) oh[i] += w * vv[i];
            }
            for (int i = 0; i < D; ++i) oh[i] *= sigmoid(gate[i]);
        }
        return linear(p + "o_proj.weight", o);
    }

    std::vector<float> moe(const std::string &p, const std::vector<float> &x) {
        const RefConfig &c = cfg;
        std::vector<float> logits = linear(p + "gate.weight", x);
        const float mx = *std::max_element(logits.begin(), logits.end());
        double sum = 0;
        std::vector<float> pr(logits.size());
        for (size_t i = 0; i < pr.size(); ++i) { pr[i] = std::exp(logits[i] - mx); sum += pr[i]; }
        for (auto &v : pr) v = float(v / sum);
        std::vector<int> order(pr.size());
        std::iota(order.begin(), order.end(), 0);
        std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return pr[size_t(a)] > pr[size_t(b)]; });
        float top = 0.f;
        for (int j = 0; j < c.top_k; ++j) top += pr[size_t(order[size_t(j)])];
        std::vector<float> out(static_cast<size_t>(c.hidden), 0.f);
        std::vector<std::vector<float>> ys(static_cast<size_t>(c.top_k));
        pool_.parallel_for(c.top_k, 1, [&](int64_t a, int64_t b) {
            for (int64_t j = a; j < b; ++j) {
                const std::string e = p + "experts." + std::to_string(order[size_t(j)]) + ".";
                std::vector<float> g = expert_linear(e + "gate_proj", x), u = expert_linear(e + "up_proj", x);
                for (size_t i = 0; i < g.size(); ++i) g[i] = silu(g[i]) * u[i];
                ys[size_t(j)] = expert_linear(e + "down_proj", g);
            }
        });
        for (int j = 0; j < c.top_k; ++j) {
            const float w = pr[size_t(order[size_t(j)])] / top;
            for (size_t i = 0; i < out.size(); ++i) out[i] += w * ys[size_t(j)][i];
        }
        std::vector<float> g = linear(p + "shared_expert.gate_proj.weight", x), u = linear(p + "shared_expert.up_proj.weight", x);
        for (size_t i = 0; i < g.size(); ++i) g[i] = silu(g[i]) * u[i];
        std::vector<float> y = linear(p + "shared_expert.down_proj.weight", g);
        const float sg = sigmoid(linear(p + "shared_expert_gate.weight", x)[0]);
        for (size_t i = 0; i < out.size(); ++i) out[i] += sg * y[i];
        return out;
    }

    SafeTensors st_;
    std::unique_ptr<NgramHasher> hasher_;
    std::unique_ptr<PleTable> table_;
    ThreadPool pool_;
    std::vector<std::vector<float>> gdn_conv_, gdn_S_;
    std::vector<Cache> qsa_;
    std::vector<float> ple_hist_;
    std::vector<int32_t> tokens_;
};

}  // namespace qwh
