// Decisions of the speculative generation loop, per slot and per step (no device work happens here).
//
//   how many drafts   the K in 1..k_max that maximises expected tokens per unit of step cost,
//                     (1 + a + ... + a^K) / (base + beta (K - 1)), with a the slot's running acceptance; none when
//                     even the best K is expected to emit less than a plain step;
//   plain stretches   when drafting stops paying it is switched off for a stretch of steps (first, + grow per repeat,
//                     up to max), then probed again from a fixed acceptance; a good spell resets the stretch length;
//   what fits         a run never exceeds the request's budget, the slot's room, the per-request run limit or - over
//                     all requests of the step - the row limit (the longest runs are trimmed first);
//   what is kept      of a verified run: the drafts that equal the tokens sampled behind them, up to a stop token;
//                     the acceptance average moves by a tenth of the step's acceptance.
//
// The per-slot state is an array of plain structs that the Python session maps directly (ctypes), so both sides read
// and write the same memory.  (Reference: best_rate / draft_count / plain_step and the accept loop of
// src/session/generate.cpp:30-43,49-86,119-313.)
#pragma once
#include <algorithm>
#include <cstdint>
#include <vector>

namespace qwh {

struct SpecSlot {
    double accept;            // running acceptance of this slot's drafts
    int32_t plain_left;       // steps left of the current stretch without drafts
    int32_t plain_stretch;    // length of the next stretch
};

struct SpecTuning {
    double base, beta, probe_accept;
    int32_t plain_first, plain_grow, plain_max;
};

enum SpecError { SPEC_OK = 0, SPEC_NO_BUDGET = -1, SPEC_SLOT_FULL = -2, SPEC_TOO_MANY = -3 };

class SpecPlanner {
public:
    SpecPlanner(int slots, const SpecTuning &t) : tune_(t), slot_(size_t(slots > 0 ? slots : 0)) {
        for (SpecSlot &s : slot_) s = SpecSlot{0.5, 0, t.plain_first};
    }
    SpecSlot *slots() { return slot_.data(); }
    int count() const { return int(slot_.size()); }

    // Expected tokens per unit cost for the best K <= k_max at acceptance a.
    void best_rate(double a, int k_max, double *rate, int *k) const {
        double best = 0.0, expect = 1.0, p = 1.0;
        int bk = 1;
        for (int K = 1; K <= k_max; ++K) {
            p *= a;
            expect += p;
            const double r = expect / (tune_.base + tune_.beta * double(K - 1));
            if (r > best) { best = r; bk = K; }
        }
        *rate = best;
        *k = bk;
    }
    int draft_count(int slot, int k_max) const {
        if (k_max <= 1) return k_max;
        double rate;
        int k;
        best_rate(slot_[size_t(slot)].accept, k_max, &rate, &k);
        return rate >= 1.0 ? k : 0;
    }

    // want[i] = drafts of request i this step.  room[i]: tokens the slot can still take after the pending one (negative:
    // the slot is full); can_draft[i]: the slot has an MTP input; forced: drafts are not subject to the acceptance rule.
    // On an error *bad names the request; slots of earlier requests may already have entered a stretch.
    int plan(int n, const int32_t *slot, const int64_t *budget, const int64_t *room, const uint8_t *can_draft, int k, int max_drafts,
             int max_run, int max_rows, int forced, int32_t *want, int *bad) {
        for (int i = 0; i < n; ++i) {
            *bad = i;
            if (budget[i] < 1) return SPEC_NO_BUDGET;
            int64_t kk = can_draft[i] ? std::min<int64_t>({int64_t(k), budget[i] - 1, int64_t(max_drafts)}) : 0;
            if (max_run > 0) kk = std::min<int64_t>(kk, max_run - 1);
            if (kk < 0) kk = 0;
            if (kk > 0 && !forced) {
                SpecSlot &s = slot_[size_t(slot[i])];
                if (s.plain_left > 0) {
                    kk = 0;
                } else {
                    kk = draft_count(slot[i], int(kk));
                    if (kk == 0 && k > 1) {                 // drafting stopped paying: a stretch of plain steps starts
                        s.plain_left = s.plain_stretch;
                        s.plain_stretch = std::min(tune_.plain_max, s.plain_stretch + tune_.plain_grow);
                    }
                }
            }
            if (kk > room[i]) {
                kk = room[i];
                if (kk < 0) return SPEC_SLOT_FULL;
            }
            want[i] = int32_t(kk);
        }
        *bad = -1;
        if (n > max_rows) return SPEC_TOO_MANY;
        int64_t rows = n;
        for (int i = 0; i < n; ++i) rows += want[i];
        while (rows > max_rows) {                           // trim the longest runs first (the first of equals)
            int longest = 0;
            for (int i = 1; i < n; ++i)
                if (want[i] > want[longest]) longest = i;
            --want[longest];
            --rows;
        }
        return SPEC_OK;
    }

    // A step without drafts inside a stretch.  Returns the steps left; at the stretch's end the next step probes.
    int note_plain_step(int slot) {
        SpecSlot &s = slot_[size_t(slot)];
        if (s.plain_left > 0 && --s.plain_left == 0) s.accept = std::max(s.accept, tune_.probe_accept);
        return s.plain_left;
    }

    // Rows kept of a verified run: sampled[j] is the token drawn behind run token j (run = pending + drafts).  forced >= 0:
    // exactly min(forced, n_drafts) drafts are kept whatever was drawn.  Updates the slot's acceptance average.
    int accept(int slot, const int32_t *sampled, const int32_t *drafts, int n_drafts, const int32_t *stop, int n_stop, int forced) {
        int n_acc = 1;
        if (forced >= 0) {
            n_acc = std::min(forced, n_drafts) + 1;
        } else {
            while (n_acc <= n_drafts && sampled[n_acc - 1] == drafts[n_acc - 1] &&
                   std::find(stop, stop + n_stop, sampled[n_acc - 1]) == stop + n_stop)
                ++n_acc;
        }
        if (n_drafts > 0) {
            SpecSlot &s = slot_[size_t(slot)];
            s.accept = 0.9 * s.accept + 0.1 * (double(n_acc - 1) / double(n_drafts));
            if (s.accept >= 0.5) s.plain_stretch = tune_.plain_first;      // a good spell: the next stretch starts short again
        }
        return n_acc;
    }

private:
    SpecTuning tune_;
    std::vector<SpecSlot> slot_;
};

}  // namespace qwh
