// N-gram row ids and the host-resident PLE table (roles of the reference's src/core/ple.cpp).
// ids: EOS-segmented 2-/3-gram hashes, one per hash head, into per-head prime-sized sub-tables.
// table: META.json + shard_<i>.safetensors in one of four layouts; gather = 16 rows -> one embedding.
#pragma once
#include <array>
#include <atomic>

#include "safetensors.hpp"
#include "threadpool.hpp"

namespace qwh {

struct NgramSpec {
    int vocab = 248320, eos = 248044, ngram = 3, heads = 16, image_pad = 248056, video_pad = 248057;
    int64_t vocab_base = 20000000;
    uint64_t seed = 1234;
};

class NgramHasher {
public:
    explicit NgramHasher(const NgramSpec &s = NgramSpec()) : spec_(s) {
        const uint64_t max_mult = ((uint64_t(1) << 63) - 1) / uint64_t(s.vocab);
        const uint64_t half = std::max<uint64_t>(1, max_mult / 2);
        for (int i = 0; i < s.ngram; ++i) mult_.push_back(2 * (splitmix(s.seed + GAMMA * uint64_t(i + 1)) % half) + 1);
        uint64_t p = uint64_t(s.vocab_base - 1);
        int64_t off = 0;
        for (int h = 0; h < s.heads; ++h) {
            uint64_t c = p + 1;
            if (c <= 2) c = 2;
            else {
                if (c % 2 == 0) ++c;
                while (!prime(c)) c += 2;
            }
            p = c;
            sizes_.push_back(int64_t(p));
            offsets_.push_back(off);
            off += int64_t(p);
        }
        total_ = off;
    }
    int heads() const { return spec_.heads; }
    int64_t total_rows() const { return total_; }
    const std::vector<int64_t> &sizes() const { return sizes_; }
    const std::vector<int64_t> &offsets() const { return offsets_; }
    const std::vector<uint64_t> &mult() const { return mult_; }
    int real_token(int t) const { return t >= 0 ? t : (((-t) & 1) ? spec_.image_pad : spec_.video_pad); }

    // ids[t*heads + h] for the tokens appended after `hist` (only its last ngram-1 entries matter).
    void ids_for(const int32_t *hist, int n_hist, const int32_t *tokens, int n, int64_t *ids) const {
        const int keep = std::min(n_hist, spec_.ngram - 1);
        std::vector<int32_t> ctx;
        for (int i = n_hist - keep; i < n_hist; ++i) ctx.push_back(real_token(hist[i]));
        for (int i = 0; i < n; ++i) ctx.push_back(real_token(tokens[i]));
        int prev_eos = -1;
        for (int i = 0; i < keep; ++i) if (ctx[size_t(i)] == spec_.eos) prev_eos = i;
        const int per = spec_.heads / (spec_.ngram - 1);
        for (int t = 0; t < n; ++t) {
            const int pos = keep + t;
            uint64_t tok[8];
            for (int s = 0; s < spec_.ngram; ++s) {
                const int idx = pos - s;
                const bool valid = s == 0 || (idx >= 0 && idx > prev_eos);
                tok[s] = uint64_t(valid ? ctx[size_t(idx)] : spec_.eos);
            }
            for (int order = 2; order <= spec_.ngram; ++order) {
                uint64_t mixed = tok[0] * mult_[0];
                for (int i = 1; i < order; ++i) mixed ^= tok[i] * mult_[size_t(i)];
                for (int j = 0; j < per; ++j) {
                    const int h = (order - 2) * per + j;
                    ids[size_t(t) * spec_.heads + h] = int64_t(mixed % uint64_t(sizes_[size_t(h)])) + offsets_[size_t(h)];
                }
            }
            if (ctx[size_t(pos)] == spec_.eos) prev_eos = pos;
        }
    }

private:
    static constexpr uint64_t GAMMA = 0x9E3779B97F4A7C15ull;
    static uint64_t splitmix(uint64_t v) {
        v += GAMMA;
        v = (v ^ (v >> 30)) * 0xBF58476D1CE4E5B9ull;
        v = (v ^ (v >> 27)) * 0x94D049BB133111EBull;
        return v ^ (v >> 31);
    }
    static uint64_t mulmod(uint64_t a, uint64_t b, uint64_t m) { return uint64_t((unsigned __int128)a * b % m); }
    static uint64_t powmod(uint64_t b, uint64_t e, uint64_t m) {
        uint64_t r = 1;
        for (b %= m; e; e >>= 1, b = mulmod(b, b, m)) if (e & 1) r = mulmod(r, b, m);
        return r;
    }
    static bool prime(uint64_t n) {              // deterministic Miller-Rabin for 64-bit inputs
        if (n < 2) return false;
        for (uint64_t p : {2ull, 3ull, 5ull, 7ull, 11ull, 13ull, 17ull, 19ull, 23ull, 29ull, 31ull, 37ull})
            if (n % p == 0) return n == p;
        uint64_t d = n - 1;
        int s = 0;
        while (d % 2 == 0) { d /= 2; ++s; }
        for (uint64_t a : {2ull, 325ull, 9375ull, 28178ull, 450775ull, 9780504ull, 1795265022ull}) {
            if (a % n == 0) continue;
            uint64_t x = powmod(a, d, n);
            if (x == 1 || x == n - 1) continue;
            bool comp = true;
            for (int r = 1; r < s && comp; ++r) {
                x = mulmod(x, x, n);
                if (x == n - 1) comp = false;
            }
            if (comp) return false;
        }
        return true;
    }
    NgramSpec spec_;
    std::vector<uint64_t> mult_;
    std::vector<int64_t> sizes_, offsets_;
    int64_t total_ = 0;
};

class PleTable {
public:
    enum class Layout { Int4, Int8, Bf16, F8 };
    PleTable(const std::string &dir, int width) : width_(width) {
        Json meta = Json::parse(read_file(dir + "/META.json"));
        const std::string l = meta["layout"].as_str();
        if (l == "group16_int4_fp16scale_lownibblefirst") layout_ = Layout::Int4;
        else if (l == "group16_int8_fp16scale") layout_ = Layout::Int8;
        else if (l == "bf16") layout_ = Layout::Bf16;
        else if (l == "f8e4m3_tensorscale") layout_ = Layout::F8;
        else fail("PLE sidecar: unsupported layout " + l);
        QWH_CHECK(meta["width"].as_int() == width, "PLE sidecar: width");
        rows_ = meta["rows"].as_int();
        const int64_t n = meta["shards"].as_int();
        rows_per_shard_ = (rows_ + n - 1) / n;
        const float scale = meta.has("scale") ? float(meta["scale"].as_double()) : 1.f;
        for (int b = 0; b < 256; ++b) lut_[size_t(b)] = f8e4m3_to_f32(uint8_t(b)) * scale;
        const char *name = layout_ == Layout::Int4 ? "weight_i4" : layout_ == Layout::Int8 ? "weight_i8"
                           : layout_ == Layout::F8 ? "weight_f8" : "weight";
        for (int64_t s = 0; s < n; ++s) {
            auto st = std::make_unique<SafeTensors>();
            st->add_file(dir + "/shard_" + std::to_string(s) + ".safetensors");
            const TensorView &q = st->get(name);
            const int64_t w = layout_ == Layout::Int4 ? width / 2 : width;
            QWH_CHECK(q.shape.size() == 2 && q.dim(1) == w, "PLE shard layout");
            q_.push_back(q.data);
            if (layout_ == Layout::Int4 || layout_ == Layout::Int8) scale_.push_back(reinterpret_cast<const uint16_t *>(st->get("weight_scale").data));
            shards_.push_back(std::move(st));
        }
    }
    ~PleTable() { stop_ = true; if (pin_.joinable()) pin_.join(); }
    Layout layout() const { return layout_; }
    int64_t rows() const { return rows_; }
    int64_t rows_per_shard() const { return rows_per_shard_; }
    const uint8_t *shard_data(size_t s) const { return q_[s]; }
    size_t n_shards() const { return q_.size(); }

    void row(int64_t id, float *out) const {
        id %= rows_;
        const int64_t s = id / rows_per_shard_, r = id % rows_per_shard_;
        const int W = width_;
        if (layout_ == Layout::F8) {
            const uint8_t *v = q_[size_t(s)] + r * W;
            for (int j = 0; j < W; ++j) out[j] = lut_[v[j]];
        } else if (layout_ == Layout::Bf16) {
            const uint16_t *v = reinterpret_cast<const uint16_t *>(q_[size_t(s)]) + r * W;
            for (int j = 0; j < W; ++j) out[j] = bf16_to_f32(v[j]);
        } else if (layout_ == Layout::Int8) {
            const int8_t *v = reinterpret_cast<const int8_t *>(q_[size_t(s)]) + r * W;
            const uint16_t *sc = scale_[size_t(s)] + r * (W / 16);
            for (int j = 0; j < W; ++j) out[j] = float(v[j]) * f16_to_f32(sc[j / 16]);
        } else {
            const uint8_t *v = q_[size_t(s)] + r * (W / 2);
            const uint16_t *sc = scale_[size_t(s)] + r * (W / 16);
            for (int j = 0; j < W; ++j) {
                const uint8_t b = v[j >> 1];
                out[j] = float(int((j & 1) ? (b >> 4) : (b & 0xf)) - 8) * f16_to_f32(sc[j / 16]);
            }
        }
    }
    // out[t][h*width ..] = row(ids[t][h]) for T tokens, split over the pool.
    void gather(const int64_t *ids, int T, int heads, float *out, ThreadPool *pool) const {
        auto body = [&](int64_t b, int64_t e) {
            for (int64_t t = b; t < e; ++t)
                for (int h = 0; h < heads; ++h) row(ids[t * heads + h], out + (t * heads + h) * width_);
        };
        if (pool) pool->parallel_for(T, 8, body);
        else body(0, T);
    }
    // Reads (and optionally mlocks) the table in a background thread so the first requests do not page-fault.
    void pin_in_background(bool lock) {
        pin_ = std::thread([this, lock] {
            size_t bytes = 0;
            bool pinned = lock;
            for (auto &st : shards_)
                for (auto &f : st->files()) {
                    if (stop_) return;
                    if (!pinned || !f->lock()) { pinned = false; f->touch(); }
                    bytes += f->size;
                }
            pinned_bytes_ = bytes;
            logf("PLE table: %.2f GB %s", double(bytes) / 1e9, pinned ? "pinned" : "read into the page cache");
        });
    }
    void wait_pinned() { if (pin_.joinable()) pin_.join(); }

    static std::string read_file(const std::string &p) {
        std::FILE *f = std::fopen(p.c_str(), "rb");
        if (!f) fail("cannot open " + p);
        std::string s;
        char buf[4096];
        size_t n;
        while ((n = std::fread(buf, 1, sizeof buf, f)) > 0) s.append(buf, n);
        std::fclose(f);
        return s;
    }

private:
    int width_;
    Layout layout_ = Layout::F8;
    int64_t rows_ = 0, rows_per_shard_ = 0;
    std::array<float, 256> lut_{};
    std::vector<std::unique_ptr<SafeTensors>> shards_;
    std::vector<const uint8_t *> q_;
    std::vector<const uint16_t *> scale_;
    std::thread pin_;
    std::atomic<bool> stop_{false};
    std::atomic<size_t> pinned_bytes_{0};
};

}  // namespace qwh
