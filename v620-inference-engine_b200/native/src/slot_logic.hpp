// Decisions about slots and prompts that need no device: which free slot a request goes to, which of the four ways a
// prompt starts, where a prefill piece ends so that a device snapshot can be taken at a message boundary, and which
// device snapshot a prompt can go back to.  The session gathers the inputs (what each slot shares with the prompt, what
// the block store holds) and carries out the decision.
// (Reference: Session::acquire and begin_keys, src/session/session.cpp:69-158,214-312; plan_captures,
// src/session/prefix_cache.cpp:41-78.)
#pragma once
#include <cstdint>

namespace qwh {

// The free slot that holds the request (capacity >= need) and keeps the most of its prompt; among equals the one used
// longest ago.  kept[i]: prompt tokens that need no prefill if slot i is chosen.  -1: no slot.
inline int choose_slot(int n, const uint8_t *busy, const int64_t *capacity, const int64_t *kept, const int64_t *used, int64_t need) {
    int best = -1;
    for (int i = 0; i < n; ++i) {
        if (busy[i] || capacity[i] < need) continue;
        if (best < 0 || kept[i] > kept[best] || (kept[i] == kept[best] && used[i] < used[best])) best = i;
    }
    return best;
}

enum StartWay { START_RESET = 0, START_IN_PLACE = 1, START_DEVICE_SNAPSHOT = 2, START_STORE = 3 };

// keep: tokens the slot would continue from in place; snapshot: depth of the best device snapshot of this slot (0: none);
// stored: tokens the block store can restore.  Whichever keeps most; a device snapshot must beat both others (it costs
// copies), continuing in place wins a tie with the store (it costs nothing).
inline int start_way(int64_t keep, int64_t snapshot, int64_t stored) {
    if (snapshot > 0 && snapshot > (keep > stored ? keep : stored)) return START_DEVICE_SNAPSHOT;
    if (keep >= stored && keep > 0) return START_IN_PLACE;
    return stored > 0 ? START_STORE : START_RESET;
}

// Where the piece [done, end) of `prompt` (n tokens) should end: at the last boundary token inside it that lies at least
// min_gap tokens after the previous capture; `end` when there is none (or no boundary token is set).
inline int64_t capture_point(const int32_t *prompt, int64_t n, int64_t done, int64_t end, int64_t last_capture, int32_t boundary, int64_t min_gap) {
    if (boundary < 0) return end;
    const int64_t lo = (done + 1 > last_capture + min_gap) ? done + 1 : last_capture + min_gap;
    for (int64_t p = (end < n - 1 ? end : n - 1); p >= lo; --p)
        if (prompt[p] == boundary) return p;
    return end;
}

// The deepest of a slot's device snapshots (depths snap_n[0..m), snap_has_logits) that lies inside what the slot and the
// prompt share (`common`); a snapshot as deep as the whole prompt only counts when it carries the logits of its position,
// since otherwise nothing would be left to produce them.  Returns its index or -1.
inline int best_snapshot(int m, const int64_t *snap_n, const uint8_t *snap_has_logits, int64_t common, int64_t prompt_len) {
    int best = -1;
    for (int i = 0; i < m; ++i) {
        const int64_t d = snap_n[i];
        if (d < 1 || d > common) continue;
        if (d >= prompt_len && !(d == prompt_len && snap_has_logits[i])) continue;
        if (best < 0 || d > snap_n[best]) best = i;
    }
    return best;
}

}  // namespace qwh
