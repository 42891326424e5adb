// Prefix cache: hash-chained blocks of up to 256 tokens in host RAM with an optional disk tier.
//
// A block's key is an FNV-1a hash over its parent's key and its tokens (tokens are compared on a hit),
// so a prompt's path through the store is found 256 tokens at a time; leaf blocks may be partial.
// A block carries an opaque KV payload (what the engine exported for those tokens) and optionally a
// snapshot payload (the recurrent state at the block's end, plus the logits there), which is what
// lets a restore stop at that block.  RAM and disk budgets are enforced LRU-first on leaves.
// File format of the disk tier (one file per block `<hash>.qwb` / snapshot `<hash>.qws`): header
// {magic[8], layout, hash, parent, ntok, ranks, nlogits, rank_bytes} | tokens (blocks) | logits | payload,
// written to a temporary name and renamed; files with another layout id are dropped at scan.
// (Formats and key chain of the reference's src/session/block_store.cpp:30-40 and
// src/session/disk_tier.cpp:20-31; the store itself is organised differently: payloads are byte
// buffers handed in by the engine layer, and the disk writer is a simple background queue.)
#pragma once
#include <dirent.h>
#include <sys/stat.h>

#include <algorithm>

#include <condition_variable>
#include <deque>
#include <mutex>
#include <thread>
#include <unordered_map>
#include <vector>

#include "common.hpp"

namespace qwh {

constexpr int BLOCK_TOKENS = 256;
constexpr uint64_t STORE_ROOT = 0x9e3779b97f4a7c15ull;

inline uint64_t block_key(uint64_t parent, const int32_t *t, size_t n) {
    uint64_t h = parent ^ (0xcbf29ce484222325ull + n);
    for (size_t i = 0; i < n; ++i) {
        const uint32_t v = uint32_t(t[i]);
        for (int b = 0; b < 4; ++b) {
            h ^= (v >> (8 * b)) & 0xff;
            h *= 1099511628211ull;
        }
    }
    return h == STORE_ROOT ? h + 1 : h;
}

#pragma pack(push, 1)
struct DiskHeader {
    char magic[8];
    uint64_t layout, hash, parent;
    int64_t ntok;
    uint32_t ranks, nlogits;
    uint64_t rank_bytes;
};
#pragma pack(pop)
static_assert(sizeof(DiskHeader) == 56, "disk header layout");
constexpr char MAGIC_BLOCK2[9] = "QWBLOCK2";
constexpr char MAGIC_BLOCK1[9] = "QWBLOCK1";
constexpr char MAGIC_SNAP[9] = "QWSNAPS1";

struct StoreStats {
    uint64_t hits = 0, tokens_restored = 0, snapshots_saved = 0, ram_bytes = 0, disk_bytes = 0, blocks = 0, snapshots = 0;
};

class BlockStore {
public:
    struct Node {
        uint64_t key = 0, parent = STORE_ROOT;
        int64_t start = 0;
        std::vector<int32_t> tokens;
        std::vector<uint8_t> kv;            // in RAM (empty when only on disk)
        std::vector<uint8_t> snap;
        std::vector<float> logits;
        bool has_snap = false, kv_disk = false, snap_disk = false, anchor = false;
        size_t kv_bytes = 0, snap_bytes = 0;    // payload sizes (also when only on disk)
        uint64_t used = 0;
        uint32_t hits = 0;
        int children = 0;
        int64_t end() const { return start + int64_t(tokens.size()); }
    };

    BlockStore(uint64_t layout, uint32_t ranks, size_t ram_budget, std::string disk_dir, size_t disk_budget)
        : layout_(layout), ranks_(ranks), ram_budget_(ram_budget), disk_budget_(disk_budget), dir_(std::move(disk_dir)) {
        if (!dir_.empty()) {
            ::mkdir(dir_.c_str(), 0755);
            scan();
            writer_ = std::thread([this] { write_loop(); });
        }
    }
    ~BlockStore() {
        flush();
        {
            std::lock_guard<std::mutex> lk(qmu_);
            stop_ = true;
        }
        qcv_.notify_all();
        if (writer_.joinable()) writer_.join();
        {
            std::lock_guard<std::mutex> lk(lmu_);          // stop_ is read under either queue's mutex
            loads_.clear();
        }
        lcv_.notify_all();
        if (loader_.joinable()) loader_.join();
    }

    // Stores tokens [start, start+n) after `parent` with their KV payload; returns the block's key.
    uint64_t save_block(uint64_t parent, int64_t start, const int32_t *tokens, int n, const void *kv, size_t kv_bytes) {
        QWH_CHECK(n > 0 && n <= BLOCK_TOKENS, "block size");
        std::lock_guard<std::mutex> lk(mu_);
        const uint64_t k = block_key(parent, tokens, size_t(n));
        auto it = nodes_.find(k);
        if (it != nodes_.end()) {
            if (it->second.tokens.size() == size_t(n) && std::equal(tokens, tokens + n, it->second.tokens.begin())) {
                it->second.used = ++clock_;
                if (it->second.kv.empty() && kv) {          // back into RAM
                    it->second.kv.assign((const uint8_t *)kv, (const uint8_t *)kv + kv_bytes);
                    ram_ += kv_bytes;
                }
                return k;
            }
            return 0;       // hash collision with other tokens: not stored
        }
        Node nd;
        nd.key = k; nd.parent = parent; nd.start = start;
        nd.tokens.assign(tokens, tokens + n);
        nd.kv.assign((const uint8_t *)kv, (const uint8_t *)kv + kv_bytes);
        nd.kv_bytes = kv_bytes;
        nd.used = ++clock_;
        ram_ += kv_bytes;
        nodes_[k] = std::move(nd);
        children_[parent].push_back(k);
        if (auto p = nodes_.find(parent); p != nodes_.end()) ++p->second.children;
        enqueue(k, false);
        enforce();
        return k;
    }
    bool save_snapshot(uint64_t key, const void *snap, size_t bytes, const float *logits, int nlogits, bool anchor) {
        std::lock_guard<std::mutex> lk(mu_);
        auto it = nodes_.find(key);
        if (it == nodes_.end()) return false;
        Node &nd = it->second;
        if (nd.has_snap) ram_ -= nd.snap.size();
        nd.snap.assign((const uint8_t *)snap, (const uint8_t *)snap + bytes);
        nd.snap_bytes = bytes;
        nd.logits.assign(logits, logits + (logits ? nlogits : 0));
        nd.has_snap = true;
        nd.anchor = nd.anchor || anchor;
        ram_ += bytes;
        ++stats_.snapshots_saved;
        enqueue(key, true);
        enforce();
        return true;
    }

    // Walks the chain for `tokens`; returns the keys of the matching blocks in order.  `snap_depth` = number of
    // leading blocks up to (and including) the deepest one that has a snapshot (0 when none): a restore uses those.
    std::vector<uint64_t> lookup(const int32_t *tokens, int64_t n, int *snap_depth) {
        std::lock_guard<std::mutex> lk(mu_);
        std::vector<uint64_t> path;
        uint64_t parent = STORE_ROOT;
        int64_t pos = 0;
        *snap_depth = 0;
        while (pos < n) {
            uint64_t found = 0;
            auto ch = children_.find(parent);
            if (ch == children_.end()) break;
            // prefer the longest child that matches (a full block over a partial leaf)
            size_t best = 0;
            for (uint64_t ck : ch->second) {
                const Node &c = nodes_.at(ck);
                const size_t len = c.tokens.size();
                if (int64_t(len) <= n - pos && len > best && std::equal(c.tokens.begin(), c.tokens.end(), tokens + pos)) {
                    best = len;
                    found = ck;
                }
            }
            if (!found) break;
            Node &nd = nodes_.at(found);
            nd.used = ++clock_;
            path.push_back(found);
            if (nd.has_snap) *snap_depth = int(path.size());
            pos += int64_t(best);
            parent = found;
            if (best < size_t(BLOCK_TOKENS)) break;      // a partial leaf ends the chain
        }
        return path;
    }
    // Payload access (loads from disk when the block is not in RAM).  Returns false when it is gone.
    bool get_kv(uint64_t key, std::vector<uint8_t> &out) { return get(key, false, out, nullptr); }
    bool get_snapshot(uint64_t key, std::vector<uint8_t> &out, std::vector<float> *logits) { return get(key, true, out, logits); }
    void note_restore(uint64_t key, int64_t tokens) {
        std::lock_guard<std::mutex> lk(mu_);
        ++stats_.hits;
        stats_.tokens_restored += uint64_t(tokens);
        if (auto it = nodes_.find(key); it != nodes_.end()) ++it->second.hits;
    }
    const Node *find(uint64_t key) {
        std::lock_guard<std::mutex> lk(mu_);
        auto it = nodes_.find(key);
        return it == nodes_.end() ? nullptr : &it->second;
    }
    StoreStats stats() {
        std::lock_guard<std::mutex> lk(mu_);
        StoreStats s = stats_;
        s.ram_bytes = ram_;
        s.disk_bytes = disk_;
        s.blocks = nodes_.size();
        for (auto &kv : nodes_) s.snapshots += kv.second.has_snap ? 1 : 0;
        return s;
    }
    // Background loads: the payloads (KV, and the snapshot when asked) of blocks that are only on disk are read into RAM
    // by a loader thread, so that a later restore finds them there.  Returns how many reads were queued.
    int prefetch(const uint64_t *keys, int n, bool last_snapshot) {
        int queued = 0;
        std::lock_guard<std::mutex> lk(lmu_);
        for (int i = 0; i < n; ++i) {
            bool kv_need = false, snap_need = false;
            {
                std::lock_guard<std::mutex> lk2(mu_);
                auto it = nodes_.find(keys[i]);
                if (it == nodes_.end()) continue;
                const Node &nd = it->second;
                kv_need = nd.kv.empty() && nd.kv_disk;
                snap_need = last_snapshot && i == n - 1 && nd.snap.empty() && nd.snap_disk;
            }
            if (kv_need) { loads_.push_back({keys[i], false}); ++queued; }
            if (snap_need) { loads_.push_back({keys[i], true}); ++queued; }
        }
        if (queued && !loader_.joinable()) loader_ = std::thread([this] { load_loop(); });
        lcv_.notify_all();
        return queued;
    }
    int loads_pending() {
        std::lock_guard<std::mutex> lk(lmu_);
        return int(loads_.size()) + (loading_ ? 1 : 0);
    }
    // Waits until every queued disk write has been done.
    void flush() {
        std::unique_lock<std::mutex> lk(qmu_);
        qdone_.wait(lk, [&] { return queue_.empty() && !writing_; });
    }
    // Drops snapshots that are closer than `gap` tokens to the next kept one further down the same conversation.  Never an
    // anchor, a snapshot that was restored from (hits), a leaf or a branch point.  Deepest first, so that "the next kept
    // one" is already decided when a snapshot is looked at; the result does not depend on the map's order.
    // (Role of the reference's QW_SNAP_KEEP_GAP thinning: src/session/block_store.cpp:499-541.)
    int thin(int64_t gap) {
        std::lock_guard<std::mutex> lk(mu_);
        std::vector<Node *> cand;
        for (auto &kv : nodes_) {
            Node &nd = kv.second;
            if (nd.has_snap && !nd.anchor && nd.hits == 0 && nd.children == 1) cand.push_back(&nd);
        }
        std::sort(cand.begin(), cand.end(), [](const Node *a, const Node *b) { return a->end() != b->end() ? a->end() > b->end() : a->key < b->key; });
        int dropped = 0;
        for (Node *nd : cand) {
            // the nearest snapshot below, following only children
            const Node *next = nd;
            for (;;) {
                auto ch = children_.find(next->key);
                if (ch == children_.end() || ch->second.size() != 1) { next = nullptr; break; }
                next = &nodes_.at(ch->second[0]);
                if (next->has_snap) break;
            }
            if (!next || next->end() - nd->end() >= gap) continue;
            ram_ -= nd->snap.size();
            if (nd->snap_disk) {
                disk_ -= std::min(disk_, sizeof(DiskHeader) + nd->logits.size() * 4 + nd->snap_bytes);
                std::remove(path(nd->key, true).c_str());
                nd->snap_disk = false;
            }
            nd->snap.clear(); nd->snap.shrink_to_fit(); nd->logits.clear();
            nd->has_snap = false;
            nd->snap_bytes = 0;
            ++dropped;
        }
        return dropped;
    }

private:
    std::string path(uint64_t hash, bool snap) const {
        char name[40];
        std::snprintf(name, sizeof name, "/%016llx.%s", (unsigned long long)hash, snap ? "qws" : "qwb");
        return dir_ + name;
    }
    void enqueue(uint64_t key, bool snap) {
        if (dir_.empty()) return;
        std::lock_guard<std::mutex> lk(qmu_);
        queue_.push_back({key, snap});
        qcv_.notify_all();
    }
    void load_loop() {
        for (;;) {
            std::pair<uint64_t, bool> job;
            {
                std::unique_lock<std::mutex> lk(lmu_);
                lcv_.wait(lk, [&] { return stop_ || !loads_.empty(); });
                if (stop_) return;
                job = loads_.front();
                loads_.pop_front();
                loading_ = true;
            }
            std::vector<uint8_t> tmp;
            std::vector<float> lg;
            get(job.first, job.second, tmp, &lg);          // leaves the payload in RAM (subject to the budget)
            {
                std::lock_guard<std::mutex> lk(lmu_);
                loading_ = false;
            }
        }
    }
    void write_loop() {
        for (;;) {
            std::pair<uint64_t, bool> job;
            {
                std::unique_lock<std::mutex> lk(qmu_);
                qcv_.wait(lk, [&] { return stop_ || !queue_.empty(); });
                if (queue_.empty()) return;
                job = queue_.front();
                queue_.pop_front();
                writing_ = true;
            }
            write_one(job.first, job.second);
            {
                std::lock_guard<std::mutex> lk(qmu_);
                writing_ = false;
            }
            qdone_.notify_all();
        }
    }
    void write_one(uint64_t key, bool snap) {
        DiskHeader h{};
        std::vector<int32_t> toks;
        std::vector<float> logits;
        std::vector<uint8_t> payload;
        {
            std::lock_guard<std::mutex> lk(mu_);
            auto it = nodes_.find(key);
            if (it == nodes_.end()) return;
            const Node &nd = it->second;
            if (snap ? (!nd.has_snap || nd.snap.empty()) : nd.kv.empty()) return;
            std::memcpy(h.magic, snap ? MAGIC_SNAP : MAGIC_BLOCK2, 8);
            h.layout = layout_; h.hash = key; h.parent = nd.parent;
            h.ntok = int64_t(nd.tokens.size()); h.ranks = ranks_;
            payload = snap ? nd.snap : nd.kv;
            if (snap) logits = nd.logits; else toks = nd.tokens;
            h.nlogits = uint32_t(logits.size());
            h.rank_bytes = payload.size() / (ranks_ ? ranks_ : 1);
        }
        const std::string fin = path(key, snap), tmp = fin + ".tmp";
        std::FILE *f = std::fopen(tmp.c_str(), "wb");
        if (!f) return;
        bool ok = std::fwrite(&h, 1, sizeof h, f) == sizeof h;
        if (!snap) ok = ok && std::fwrite(toks.data(), 4, toks.size(), f) == toks.size();
        ok = ok && std::fwrite(logits.data(), 4, logits.size(), f) == logits.size();
        ok = ok && std::fwrite(payload.data(), 1, payload.size(), f) == payload.size();
        ok = (std::fclose(f) == 0) && ok;
        if (!ok || std::rename(tmp.c_str(), fin.c_str()) != 0) { std::remove(tmp.c_str()); return; }
        std::lock_guard<std::mutex> lk(mu_);
        auto it = nodes_.find(key);
        if (it == nodes_.end()) return;
        const size_t bytes = sizeof h + toks.size() * 4 + logits.size() * 4 + payload.size();
        if (snap && !it->second.has_snap) {          // the snapshot was dropped while its file was being written
            std::remove(fin.c_str());
            return;
        }
        (snap ? it->second.snap_disk : it->second.kv_disk) = true;
        disk_ += bytes;
        enforce();
    }
    bool read_file(uint64_t key, bool snap, std::vector<uint8_t> &payload, std::vector<float> *logits, std::vector<int32_t> *toks,
                   DiskHeader *hout) const {
        std::FILE *f = std::fopen(path(key, snap).c_str(), "rb");
        if (!f) return false;
        DiskHeader h{};
        bool ok = std::fread(&h, 1, sizeof h, f) == sizeof h && h.layout == layout_ && h.ranks == ranks_ && h.hash == key &&
                  (snap ? std::memcmp(h.magic, MAGIC_SNAP, 8) == 0
                        : (std::memcmp(h.magic, MAGIC_BLOCK2, 8) == 0 || std::memcmp(h.magic, MAGIC_BLOCK1, 8) == 0));
        std::vector<int32_t> t;
        if (ok && !snap) {
            ok = h.ntok > 0 && h.ntok <= BLOCK_TOKENS;
            if (ok) { t.resize(size_t(h.ntok)); ok = std::fread(t.data(), 4, t.size(), f) == t.size(); }
        }
        std::vector<float> lg(ok ? h.nlogits : 0);
        ok = ok && std::fread(lg.data(), 4, lg.size(), f) == lg.size();
        if (ok) {
            payload.resize(size_t(h.rank_bytes) * h.ranks);
            ok = std::fread(payload.data(), 1, payload.size(), f) == payload.size();
        }
        std::fclose(f);
        if (ok) {
            if (logits) *logits = std::move(lg);
            if (toks) *toks = std::move(t);
            if (hout) *hout = h;
        }
        return ok;
    }
    bool get(uint64_t key, bool snap, std::vector<uint8_t> &out, std::vector<float> *logits) {
        {
            std::lock_guard<std::mutex> lk(mu_);
            auto it = nodes_.find(key);
            if (it == nodes_.end()) return false;
            Node &nd = it->second;
            nd.used = ++clock_;
            if (snap ? (nd.has_snap && !nd.snap.empty()) : !nd.kv.empty()) {
                out = snap ? nd.snap : nd.kv;
                if (logits) *logits = nd.logits;
                return true;
            }
            if (!(snap ? nd.snap_disk : nd.kv_disk)) return false;
        }
        std::vector<float> lg;
        if (!read_file(key, snap, out, &lg, nullptr, nullptr)) return false;
        std::lock_guard<std::mutex> lk(mu_);
        auto it = nodes_.find(key);
        if (it != nodes_.end()) {           // keep it in RAM again
            Node &nd = it->second;
            if (snap) { nd.snap = out; nd.logits = lg; nd.has_snap = true; }
            else nd.kv = out;
            ram_ += out.size();
            enforce();
        }
        if (logits) *logits = std::move(lg);
        return true;
    }
    // Index rebuild: every readable file becomes a node that is "only on disk"; orphans are dropped.
    void scan() {
        DIR *d = opendir(dir_.c_str());
        if (!d) return;
        std::vector<std::pair<uint64_t, bool>> files;
        while (dirent *e = readdir(d)) {
            const std::string n = e->d_name;
            if (n.size() == 20 && (n.substr(16) == ".qwb" || n.substr(16) == ".qws")) files.push_back({std::stoull(n.substr(0, 16), nullptr, 16), n[19] == 's'});
            else if (n.size() > 4 && n.substr(n.size() - 4) == ".tmp") std::remove((dir_ + "/" + n).c_str());
        }
        closedir(d);
        for (int pass = 0; pass < 2; ++pass)             // blocks first, then snapshots
            for (auto &f : files) {
                if (f.second != (pass == 1)) continue;
                std::vector<uint8_t> payload;
                std::vector<float> lg;
                std::vector<int32_t> toks;
                DiskHeader h{};
                if (!read_file(f.first, f.second, payload, &lg, &toks, &h)) { std::remove(path(f.first, f.second).c_str()); continue; }
                const size_t bytes = sizeof h + toks.size() * 4 + lg.size() * 4 + payload.size();
                if (!f.second) {
                    Node nd;
                    nd.key = h.hash; nd.parent = h.parent; nd.tokens = toks; nd.kv_disk = true; nd.kv_bytes = payload.size();
                    nodes_[nd.key] = std::move(nd);
                    disk_ += bytes;
                } else if (auto it = nodes_.find(h.hash); it != nodes_.end()) {
                    it->second.has_snap = true; it->second.snap_disk = true; it->second.snap_bytes = payload.size();
                    disk_ += bytes;
                } else std::remove(path(f.first, true).c_str());
            }
        // link children, compute starts, drop blocks whose parent is missing
        bool changed = true;
        while (changed) {
            changed = false;
            for (auto it = nodes_.begin(); it != nodes_.end();) {
                if (it->second.parent != STORE_ROOT && !nodes_.count(it->second.parent)) {
                    std::remove(path(it->first, false).c_str());
                    std::remove(path(it->first, true).c_str());
                    it = nodes_.erase(it);
                    changed = true;
                } else ++it;
            }
        }
        for (auto &kv : nodes_) {
            children_[kv.second.parent].push_back(kv.first);
            if (auto p = nodes_.find(kv.second.parent); p != nodes_.end()) ++p->second.children;
        }
        for (auto &kv : nodes_) {
            int64_t start = 0;
            for (uint64_t p = kv.second.parent; p != STORE_ROOT; p = nodes_.at(p).parent) start += int64_t(nodes_.at(p).tokens.size());
            kv.second.start = start;
        }
    }
    // LRU: RAM payloads of the least recently used nodes go first (they stay on disk when written); over the disk
    // budget, least recently used leaves are deleted.
    void enforce() {
        while (ram_ > ram_budget_) {
            Node *victim = nullptr;
            for (auto &kv : nodes_) {
                Node &nd = kv.second;
                if (nd.kv.empty() && nd.snap.empty()) continue;
                if (!victim || nd.used < victim->used) victim = &nd;
            }
            if (!victim) break;
            const bool keep_on_disk = !dir_.empty();
            ram_ -= victim->kv.size() + victim->snap.size();
            if (keep_on_disk && (victim->kv_disk || victim->kv.empty()) && (victim->snap_disk || victim->snap.empty())) {
                victim->kv.clear(); victim->kv.shrink_to_fit();
                victim->snap.clear(); victim->snap.shrink_to_fit();
            } else if (!keep_on_disk && victim->children == 0) {
                erase(victim->key);
            } else if (!keep_on_disk) {
                victim->kv.clear(); victim->snap.clear(); victim->has_snap = false;     // inner node without payload: a hole
                erase_subtree(victim->key);
            } else {
                ram_ += victim->kv.size() + victim->snap.size();      // not written yet: try again later
                victim->used = ++clock_;
                break;
            }
        }
        while (!dir_.empty() && disk_ > disk_budget_) {
            Node *victim = nullptr;
            for (auto &kv : nodes_)
                if (kv.second.children == 0 && (kv.second.kv_disk || kv.second.snap_disk) && (!victim || kv.second.used < victim->used)) victim = &kv.second;
            if (!victim) break;
            erase(victim->key);
        }
    }
    void erase(uint64_t key) {
        auto it = nodes_.find(key);
        if (it == nodes_.end()) return;
        Node &nd = it->second;
        ram_ -= nd.kv.size() + nd.snap.size();
        if (nd.kv_disk) { disk_ -= std::min(disk_, sizeof(DiskHeader) + nd.tokens.size() * 4 + nd.kv_bytes); std::remove(path(key, false).c_str()); }
        if (nd.snap_disk) { disk_ -= std::min(disk_, sizeof(DiskHeader) + nd.logits.size() * 4 + nd.snap_bytes); std::remove(path(key, true).c_str()); }
        auto &sib = children_[nd.parent];
        sib.erase(std::remove(sib.begin(), sib.end(), key), sib.end());
        if (auto p = nodes_.find(nd.parent); p != nodes_.end()) --p->second.children;
        children_.erase(key);
        nodes_.erase(it);
    }
    void erase_subtree(uint64_t key) {
        auto ch = children_.find(key);
        if (ch != children_.end()) {
            const std::vector<uint64_t> kids = ch->second;
            for (uint64_t k : kids) erase_subtree(k);
        }
        erase(key);
    }

    uint64_t layout_;
    uint32_t ranks_;
    size_t ram_budget_, disk_budget_, ram_ = 0, disk_ = 0;
    std::string dir_;
    std::mutex mu_;
    std::unordered_map<uint64_t, Node> nodes_;
    std::unordered_map<uint64_t, std::vector<uint64_t>> children_;
    uint64_t clock_ = 0;
    StoreStats stats_;
    // disk writer
    std::mutex qmu_;
    std::condition_variable qcv_, qdone_;
    std::deque<std::pair<uint64_t, bool>> queue_;
    bool stop_ = false, writing_ = false;
    std::thread writer_;
    // background loader
    std::mutex lmu_;
    std::condition_variable lcv_;
    std::deque<std::pair<uint64_t, bool>> loads_;
    bool loading_ = false;
    std::thread loader_;
};

}  // namespace qwh
