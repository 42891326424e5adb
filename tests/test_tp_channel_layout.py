"""Layout of the prefill channel's region (pure arithmetic, no GPU): every collective kind's buffer holds what the kernels
put there for a 4,096-row chunk of the full model on 2, 4 and 8 ranks, buffers do not overlap, everything is aligned for
16-byte stores and TMA, and the flags have a 64-byte line per (kind, rank)."""
import pytest

from qwb200.models.config import ModelConfig, ShardConfig
from qwb200.ops import structs as S
from qwb200.parallel import tp_channel


@pytest.mark.parametrize("ranks", [2, 4, 8])
@pytest.mark.parametrize("mtp", [False, True])
def test_region_layout_full_model(ranks, mtp):
    cfg = ModelConfig.full()
    sc = ShardConfig(cfg, ranks, 0)
    rows = 4096
    lay = tp_channel.layout(cfg, sc, rows, mtp)
    part, offs = lay["part_bytes"], lay["off_buf"]
    assert len(part) == len(offs) == S.TP_KINDS
    # what a chunk puts into each kind's part
    need = {S.TP_SSQ: rows * cfg.hc * 4,                              # one sum of squares per (row, stream)
            S.TP_DOWN: rows * lay["hc_ld"] * 4,                      # the mixer's partial down projection, padded rows
            S.TP_RS: rows * sc.sh * 4,                               # this rank's columns of a block output, fp32
            S.TP_BIN: rows * cfg.hidden * 2,                         # the gathered block input, bf16
            S.TP_SMALL: 4096}
    if mtp:
        need[S.TP_WIDE] = rows * cfg.hc * cfg.hidden * 2            # the MTP pass's normalised hidden streams, bf16
    for k, n in need.items():
        assert part[k] >= n, (k, part[k], n)
    assert lay["hc_ld"] >= cfg.hc_down and lay["hc_ld"] % 8 == 0
    # flags first: one 64-byte line per (kind, source rank), then the buffers in kind order without overlap
    assert lay["off_flags"] == 0 and offs[0] >= S.TP_KINDS * 8 * 64
    whole = {k: (part[k] if k in (S.TP_BIN, S.TP_WIDE) else ranks * part[k]) for k in range(S.TP_KINDS)}
    for k in range(S.TP_KINDS):
        assert offs[k] % 256 == 0 and part[k] % 256 == 0
        if k + 1 < S.TP_KINDS:
            assert offs[k] + whole[k] <= offs[k + 1]
    assert lay["nbytes"] == offs[-1] + whole[S.TP_KINDS - 1]
    # the reduce-scatter buffer is what bounds the region: ranks x rows x (hidden / ranks) fp32 = rows x hidden x 4
    assert whole[S.TP_RS] >= rows * cfg.hidden * 4
    assert lay["nbytes"] < (2 << 30)


def test_kinds_are_the_ones_the_kernels_name():
    assert (S.TP_SSQ, S.TP_DOWN, S.TP_BIN, S.TP_RS, S.TP_SMALL, S.TP_WIDE) == (0, 1, 2, 3, 4, 5) and S.TP_KINDS == 6
