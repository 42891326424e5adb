"""Selection-locality counter (host side): spilled share, re-selection within K positions, sharing inside a run."""
import numpy as np

from qwb200.utils.locality import WINDOWS, LocalityCounter, spilled_groups


def test_spilled_groups_follow_the_page_table():
    # 4 pages of 256 tokens, groups of 4 tokens: pages 0 and 1 on the device (ids < 2), pages 2 and 3 in host memory
    sp = spilled_groups(np.array([0, 1, 2, 3]), n_dev_pages=2, page=256, ratio=4)
    assert sp.shape == (256,) and not sp[:128].any() and sp[128:].all()


def test_reselection_windows():
    sp = np.zeros(100, dtype=bool)
    sp[50:] = True
    c = LocalityCounter(100)
    c.step(1000, [1, 2, 60, 61, 61], sp)              # duplicates count once; 60 and 61 are spilled, never seen before
    assert (c.selected, c.spilled, int(c.within.sum())) == (4, 2, 0)
    c.step(1001, [60, 70], sp)                         # 60 again after 1 position
    c.step(1004, [61, 70, 3], sp)                      # 61 after 4 positions, 70 after 3
    c.step(1040, [60], sp)                             # 60 after 39: outside every window
    r = c.report()
    assert r["steps"] == 4 and r["groups_spilled"] == 2 + 2 + 2 + 1
    within = dict(zip(WINDOWS, c.within.tolist()))
    assert within == {1: 1, 2: 1, 4: 3, 8: 3, 16: 3, 32: 3}
    assert r["reselected_within"]["4"] == round(3 / 7, 4)
    assert r["spilled_share"] == round(7 / 10, 4)


def test_out_of_range_groups_are_ignored_and_runs_share():
    sp = np.ones(10, dtype=bool)
    c = LocalityCounter(10)
    c.step(5, [-1, 3, 10, 99], sp)
    assert c.selected == 1 and c.spilled == 1
    c.run([[1, 2, 3], [2, 3, 4], [3, 4, 5]], sp)
    r = c.report()
    assert r["run_spilled_selections"] == 9 and r["run_spilled_distinct"] == 5 and r["run_sharing"] == 1.8
