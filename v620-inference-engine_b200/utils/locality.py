"""How local is the sparse attention's choice of groups from one decode step to the next?

The device cache in front of spilled KV pages only pays if a group that a step selects was selected shortly before.
This counter takes every step's selected groups and answers: of the distinct groups selected, how many lie in
spilled pages, and how many of those were last selected at most K positions earlier, for K = 1, 2, 4, ..., 32.
For a speculative run of several rows it counts the rows' spilled selections and how many of them are distinct
(rows of one run share most of their groups, so one fetch serves several rows).
(The reference counts the same on the device per QSA layer: src/kernels/qsa.hip:293-339, switched on with
QW_SPILL_LOCALITY; here the selection lists are read back and counted on the host, which an experiment can afford.)
"""
from __future__ import annotations

from typing import Dict, Iterable, Sequence

import numpy as np

WINDOWS = (1, 2, 4, 8, 16, 32)
NEVER = -(1 << 40)


class LocalityCounter:
    def __init__(self, groups: int):
        self.last = np.full(int(groups), NEVER, dtype=np.int64)     # position at which each group was last selected
        self.selected = 0            # distinct groups selected, all steps
        self.spilled = 0             # of those, in spilled pages
        self.within = np.zeros(len(WINDOWS), dtype=np.int64)       # spilled and last selected <= K positions ago
        self.run_rows = 0            # spilled selections summed over the rows of runs
        self.run_distinct = 0        # distinct spilled groups per run, summed
        self.steps = 0

    @staticmethod
    def _distinct(groups: Iterable[int]) -> np.ndarray:
        return np.unique(np.asarray(list(groups) if not isinstance(groups, np.ndarray) else groups, dtype=np.int64))

    def step(self, pos: int, groups: Iterable[int], spilled: np.ndarray) -> None:
        """One single-row decode step at position ``pos`` that selected ``groups``; ``spilled[g]`` says whether
        group g's tokens live in host memory."""
        g = self._distinct(groups)
        g = g[(g >= 0) & (g < len(self.last))]
        self.steps += 1
        self.selected += len(g)
        gs = g[np.asarray(spilled, dtype=bool)[g]]
        self.spilled += len(gs)
        age = int(pos) - self.last[gs]
        for i, k in enumerate(WINDOWS):
            self.within[i] += int((age <= k).sum())
        self.last[gs] = int(pos)

    def run(self, rows: Sequence[Iterable[int]], spilled: np.ndarray) -> None:
        """One verification run: ``rows[i]`` are the groups row i selected."""
        sp = np.asarray(spilled, dtype=bool)
        seen = []
        for groups in rows:
            g = self._distinct(groups)
            g = g[(g >= 0) & (g < len(self.last))]
            gs = g[sp[g]]
            self.run_rows += len(gs)
            seen.append(gs)
        if seen:
            self.run_distinct += len(np.unique(np.concatenate(seen)))

    def report(self) -> Dict[str, object]:
        sp = max(1, self.spilled)
        return {"steps": self.steps, "groups_selected": self.selected, "groups_spilled": self.spilled,
                "spilled_share": round(self.spilled / max(1, self.selected), 4),
                "reselected_within": {str(k): round(int(self.within[i]) / sp, 4) for i, k in enumerate(WINDOWS)},
                "run_spilled_selections": self.run_rows, "run_spilled_distinct": self.run_distinct,
                "run_sharing": round(self.run_rows / max(1, self.run_distinct), 3)}


def spilled_groups(page_table_row: np.ndarray, n_dev_pages: int, page: int, ratio: int) -> np.ndarray:
    """``spilled[g]`` for one slot from its page-table row: group g (``ratio`` tokens) is spilled when its page's
    entry is a host page (an index at or beyond the device pool)."""
    per_page = page // ratio
    return np.repeat(np.asarray(page_table_row) >= int(n_dev_pages), per_page)
