"""What an engine configuration will take, estimated from shapes before anything is loaded, and the checks made with it.

Loading a 72 GB checkpoint and pinning tens of gigabytes of host memory takes minutes; a configuration that cannot
fit should be refused in the first second, with the numbers.  ``estimate`` gives one rank's device bytes (weights, KV
pages and recurrent state, buffers) and pinned host bytes (spilled KV); ``check`` compares them with what the device
and the host have; ``wait_for_device`` waits for another process to leave the GPUs.
(The reference does the same in its engine constructor: the wait for busy cards, src/engine/engine.hip:87-111, the
VRAM estimate that ``QW_VRAM_CHECK=0`` skips, :125-146, and the host-memory check for the spill pool, :147-163.)

The weight figure follows the checkpoint's shapes: int4 experts with one bf16 scale per group, bf16 everything else;
experts, projections, mixers and the lm_head are split over the ranks, the embedding table is held by every rank.
Against the sizes this engine reports after loading the full model (72.2 / 36.8 / 19.1 / 10.3 GB on 1 / 2 / 4 / 8 ranks)
it is within 3 %.
"""
from __future__ import annotations

import time
from typing import Callable, Dict, Optional, Tuple

from ..models.config import ModelConfig, ShardConfig

KV_PAGE, RAW_RING, GDN_RING, PLE_RING = 256, 16, 16, 32          # engine.device_model's constants
GB = float(1 << 30)


def weight_bytes(cfg: ModelConfig, ranks: int) -> int:
    h, hc = cfg.hidden, cfg.hc
    n_layers = cfg.n_layers + (1 if cfg.mtp else 0)                  # the MTP head is one more QSA + MoE layer
    n_qsa = cfg.n_qsa + (1 if cfg.mtp else 0)
    expert = 3 * cfg.ffn * h                                          # gate, up, down
    experts = n_layers * cfg.n_experts * (expert // 2 + expert // cfg.qgroup * 2)
    mixer = hc * h + cfg.hc_down * hc * h + hc * h * cfg.hc_rank      # norm weights, down (+ inject rows), up
    moe_dense = cfg.n_experts * h * 2 + 3 * cfg.ffn * h + h           # router (fp32 counted as two bf16), shared expert, its gate
    gdn = cfg.gdn_qkv * h + cfg.gdn_val * h + 2 * cfg.gdn_v_heads * h + h * cfg.gdn_val + cfg.gdn_qkv * cfg.gdn_conv
    qsa = (2 * cfg.q_heads * cfg.head_dim + 2 * cfg.kv_heads * cfg.head_dim + cfg.idx_heads * cfg.idx_dim + cfg.idx_dim) * h \
        + h * cfg.q_heads * cfg.head_dim
    dense = n_layers * (2 * mixer + moe_dense) + cfg.n_gdn * gdn + n_qsa * qsa
    dense += mixer                                                    # the final mixer
    dense += (hc * h + h) * h                                         # PLE key / value projections
    if cfg.mtp:
        dense += 2 * h * h + mixer                                    # fc_hidden, fc_embedding, the head's own final mixer
    lm_head = cfg.vocab * h
    embed = cfg.vocab * h
    return (experts + 2 * (dense + lm_head)) // ranks + 2 * embed


def state_bytes(cfg: ModelConfig, ranks: int, slots: int, slot_tokens: int, dev_pages: Optional[int], max_rows: int,
                save_gdn: bool) -> int:
    sc = ShardConfig(cfg, ranks, 0)
    nkv = cfg.n_qsa + (1 if cfg.mtp else 0)
    cap = (slot_tokens + KV_PAGE - 1) // KV_PAGE * KV_PAGE
    pages = slots * (cap // KV_PAGE) if dev_pages is None else int(dev_pages)
    row = sc.kvh_l * cfg.head_dim
    kv = nkv * 2 * pages * KV_PAGE * row * 2
    ck = nkv * slots * (cap // cfg.idx_ratio) * cfg.idx_dim * 2
    rings = nkv * slots * RAW_RING * cfg.idx_dim * 4 + cfg.n_gdn * slots * GDN_RING * sc.gdn_qkv_l * 4 + slots * PLE_RING * sc.xw * 4
    gdn = cfg.n_gdn * slots * sc.gdn_state * 4
    if save_gdn:
        gdn += cfg.n_gdn * max_rows * sc.gdn_state * 4              # the state after every row of a verification step
    return kv + ck + rings + gdn


def host_kv_bytes(cfg: ModelConfig, ranks: int, host_pages: int) -> int:
    sc = ShardConfig(cfg, ranks, 0)
    nkv = cfg.n_qsa + (1 if cfg.mtp else 0)
    return nkv * 2 * int(host_pages) * KV_PAGE * sc.kvh_l * cfg.head_dim * 2


def buffer_bytes(cfg: ModelConfig, ranks: int, max_rows: int, prefill_chunk: int) -> int:
    """Step buffers and the prefill chunk's scratch: a generous allowance rather than a sum of shapes (the token-major
    path keeps about 1.4 MB per token of the chunk on one rank: activations of the widest projection in fp32 and bf16,
    the expert pairs' inputs and outputs, the scoring tile), plus the CUDA context, graphs and allocator slack."""
    per_token = int(1.4e6 * cfg.hidden / 2560 / max(1, ranks) ** 0.5)
    return prefill_chunk * per_token + max_rows * 4 * (cfg.vocab // ranks + 64 * cfg.hidden) + (3 << 30)


def estimate(cfg: ModelConfig, ranks: int = 1, slots: int = 1, slot_tokens: int = 8192, dev_pages: Optional[int] = None,
             host_pages: int = 0, max_rows: int = 32, prefill_chunk: int = 4096, save_gdn: bool = True) -> Dict[str, float]:
    """One rank's plan in GB: ``weights_gb``, ``state_gb``, ``buffers_gb``, ``device_gb`` (their sum), ``host_kv_gb``."""
    w = weight_bytes(cfg, ranks)
    s = state_bytes(cfg, ranks, slots, slot_tokens, dev_pages, max_rows, save_gdn)
    b = buffer_bytes(cfg, ranks, max_rows, prefill_chunk)
    return {"weights_gb": w / GB, "state_gb": s / GB, "buffers_gb": b / GB, "device_gb": (w + s + b) / GB,
            "host_kv_gb": host_kv_bytes(cfg, ranks, host_pages) / GB}


def host_available_bytes(meminfo: str = "/proc/meminfo") -> Optional[int]:
    try:
        with open(meminfo) as f:
            for ln in f:
                if ln.startswith("MemAvailable:"):
                    return int(ln.split()[1]) * 1024
    except (OSError, ValueError, IndexError):
        pass
    return None


def check(plan: Dict[str, float], device_total_bytes: int, host_available: Optional[int] = None, local_ranks: int = 1,
          spare_gb: float = 2.0) -> None:
    """Raise ``ValueError`` with the numbers when the plan cannot fit: the device estimate against the device's total
    memory (not its free memory: who else is on the GPU is ``wait_for_device``'s business), the spilled KV of all
    ranks on this host against the host's available memory."""
    total = device_total_bytes / GB
    if plan["device_gb"] + spare_gb > total:
        raise ValueError(f"the configuration does not fit the GPU: weights {plan['weights_gb']:.1f} GB + slots {plan['state_gb']:.1f} GB + "
                         f"buffers {plan['buffers_gb']:.1f} GB = {plan['device_gb']:.1f} GB of {total:.1f} GB ({spare_gb:.0f} GB must stay free): fewer or "
                         "smaller resident slots, KV spill with a smaller resident part, or more GPUs (QW_VRAM_CHECK=0 skips this check)")
    need_host = plan["host_kv_gb"] * local_ranks
    if host_available is not None and need_host > 0 and need_host > host_available / GB * 0.9:
        raise ValueError(f"the spilled KV needs {need_host:.1f} GB of pinned host memory and the host has {host_available / GB:.1f} GB "
                         "available: a smaller slot_max_tokens or fewer slots (QW_VRAM_CHECK=0 skips this check)")


def wait_for_device(mem_info: Callable[[], Tuple[int, int]], limit_s: float, log: Callable[[str], None] = lambda m: None,
                    poll_s: float = 5.0, sleep: Callable[[float], None] = time.sleep, clock: Callable[[], float] = time.time) -> bool:
    """Wait (at most ``limit_s`` seconds) until nine tenths of the device's memory are free: another process - a test on
    the same box, a model still unloading - holds the GPU.  ``mem_info() -> (free, total)`` is the smallest free and the
    total over the engine's GPUs.  Returns whether the device was free in the end."""
    t0 = clock()
    told = False
    while True:
        free, total = mem_info()
        ok = free >= total // 10 * 9
        waited = clock() - t0
        if ok or waited >= limit_s:
            if told:
                log(f"the GPUs are {'free' if ok else 'still busy'} after {waited:.0f} s")
            return ok
        if not told:
            log(f"the GPUs are in use ({free / GB:.1f} of {total / GB:.1f} GB free on the fullest): waiting up to {limit_s:.0f} s")
            told = True
        sleep(poll_s)
