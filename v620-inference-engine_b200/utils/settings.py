"""One validated settings object for everything the reference reads ad hoc from ``QW_*`` environment variables
(about eighty ``getenv`` calls spread over its sources, listed in its docs/ENGINE_GUIDE.md:162-213).  The variable
names are kept as aliases so that a deployment's environment file keeps working; every value is parsed and range
checked once, unknown ``QW_*`` names are reported, and the effective settings are logged once at start.

Precedence: explicit keyword / JSON option > environment > default."""
from __future__ import annotations

import dataclasses
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Mapping, Optional


def _bool(v: str) -> bool:
    s = str(v).strip().lower()
    if s in ("1", "true", "on", "yes"):
        return True
    if s in ("0", "false", "off", "no", ""):
        return False
    raise ValueError(f"not a boolean: {v!r}")


def _ints(v) -> List[int]:
    if isinstance(v, (list, tuple)):
        return [int(x) for x in v]
    return [int(x) for x in str(v).split(",") if x.strip()]


@dataclass
class Settings:
    # ---- tracing / diagnostics
    trace: bool = False                 # QW_TRACE: per-step and per-generate host timers
    profile: bool = False               # QW_PROFILE: per-chunk prefill timing (CUDA events)
    moe_stats: bool = False             # QW_MOE_STATS: per-layer busiest-rank / mean expert pairs
    guard: bool = False                 # QW_GUARD: guard zones behind device buffers, checked after every step
    device_checks: bool = False         # QW_DEVICE_CHECKS: bounds checks on data-derived indices in the kernels
    spec_log: bool = False              # QW_SPEC_LOG: acceptance log of speculative steps
    log_interval: float = 30.0          # QW_LOG_INTERVAL: seconds between the scheduler's stats lines
    # ---- engine
    nograph: bool = False               # QW_NOGRAPH: run steps without CUDA graphs
    no_mtp: bool = False                # QW_NO_MTP
    no_vision: bool = False             # QW_NO_VISION
    gpu_sampling: bool = True           # QW_GPU_SAMPLING: 0 draws every token with the host sampler
    slots: List[int] = field(default_factory=lambda: [131072, 32768, 32768, 32768])      # QW_SLOTS
    slot_max_tokens: int = 0            # QW_SLOT_MAX_TOKENS (with spill)
    kv_spill: bool = False              # QW_KV_SPILL (on | off)
    slot_spill: List[int] = field(default_factory=list)     # QW_SLOT_SPILL: tokens beyond each slot's device part, per slot ("0,131072,...")
    spill: bool = True                  # QW_SPILL=0 forces KV spill off whatever else asks for it
    spill_cache_mb: int = 256           # QW_SPILL_CACHE_MB: device cache in front of the host KV pages (0 = none)
    spill_cache_stats: bool = False     # QW_SPILL_CACHE_STATS: count hits and misses
    spill_stage: bool = True            # QW_SPILL_STAGE: prefill attention reads spilled pages from a device copy made per layer
    spill_policy: str = "auto"          # QW_SPILL_POLICY: auto | bind | preferred | interleave | process
    prefill_chunk: int = 4096           # QW_PREFILL_CHUNK
    prefill_piece: int = 2048           # QW_PREFILL_PIECE
    qsa_attend_rows: bool = False       # QW_QSA_ATTEND_ROWS: token-major prefill attends with the decode kernels (CUDA cores)
    moe_dequant_scratch: bool = False   # QW_MOE_DEQUANT_SCRATCH: token-major prefill converts a layer's q4 experts to bf16 before its GEMMs
    gdn_sequential: bool = False        # QW_GDN_SEQUENTIAL: token-major prefill scans GDN layers row by row (not chunked)
    prefill_py: bool = False            # QW_PREFILL_PY: token-major prefill scheduled from Python, kernel by kernel (one GPU; the native runtime is the default)
    prefill_lanes: int = 0              # QW_PREFILL_LANES: micro-batches per chunk, 1 or 2 (0 = two on eight GPUs, one below)
    spec_max_rows: int = 0              # QW_SPEC_MAX_ROWS: longest verification run of one request, pending token included (0 = the engine's limit, 13)
    weight_cache_dir: str = ""          # QW_WEIGHT_CACHE_DIR
    ple_dir: str = ""                   # QW_PLE_DIR
    ple_pin: bool = True                # QW_PLE_PIN
    vram_check: bool = True             # QW_VRAM_CHECK: refuse a configuration whose estimate does not fit the GPU or the host, before loading
    # ---- session / caches
    host_cache_gb: float = 128.0        # QW_HOST_CACHE_GB
    disk_cache_dir: str = ""            # QW_DISK_CACHE_DIR
    disk_cache_gb: float = 200.0        # QW_DISK_CACHE_GB
    snap_min_gap: int = 1024            # QW_SNAP_MIN_GAP
    snap_keep_gap: int = 0              # QW_SNAP_KEEP_GAP: stored snapshots closer than this many tokens to the next kept one are dropped (0 = keep all)
    pool_reserve_gb: float = 0.0        # QW_POOL_RESERVE_GB: pinned block units kept ready for a burst of prefix-cache saves (0 = two units)
    vision_cache_gb: float = 2.0        # QW_VISION_CACHE_GB
    # ---- server
    decode_share: float = 0.25          # QW_DECODE_SHARE
    stuck_seconds: float = 300.0        # QW_STUCK_SECONDS
    exit_grace: float = 30.0            # QW_EXIT_GRACE
    watchdog_exit: bool = True          # QW_WATCHDOG_EXIT
    start_wait_s: float = 0.0           # QW_START_WAIT_S: at start, wait up to this long for another process to leave the GPUs (0 = do not wait)
    thinking_budget: int = 0            # QW_THINKING_BUDGET
    reasoning_effort: str = ""          # QW_REASONING_EFFORT
    media_fetch: bool = True            # QW_MEDIA_FETCH
    media_allow_private: bool = False   # QW_MEDIA_ALLOW_PRIVATE
    vision_max_pixels: int = 1920 * 1088    # QW_VISION_MAX_PIXELS
    video_max_pixels: int = 0           # QW_VIDEO_MAX_PIXELS (0 = the model's own limit)
    unknown: List[str] = field(default_factory=list)

    ALIASES = {}                        # old variable name -> field (none at present)
    # variables of the reference that have no meaning in this engine (PCIe transport, int8 copies, rank threads, ...):
    # accepted and ignored, so an old environment file does not produce warnings
    IGNORED = {"QW_COMM_CONCURRENT_MAX", "QW_COMM_PUSH2D", "QW_COMM_RECV_BYTES", "QW_COMM_ROWWISE", "QW_COMM_SPLIT", "QW_INT8_DENSE",
               "QW_INT8_DIR", "QW_INT8_DUMP", "QW_INT8_EXPERTS", "QW_INT8_SKIP", "QW_KV_PAIRS", "QW_KV_PAIR_CHECK", "QW_LOAD_SERIAL", "QW_LOAD_THREADS",
               "QW_MOE_PAIR_MAX", "QW_NO_SPLIT", "QW_POOL_ARENA", "QW_POOL_PREPIN", "QW_POOL_SERIAL", "QW_PREFILL_BATCH",
               "QW_PREFILL_PIPELINE", "QW_RESERVE_AHEAD", "QW_SHARE_MIN", "QW_SHARE_WAIT", "QW_SLOT_MOVE", "QW_SLOT_MOVE_IDLE_S", "QW_SNAP_SYSTEM_MIN",
               "QW_SPEC_BASE", "QW_SPEC_COST", "QW_SPEC_MIXED", "QW_SPILL_LOCALITY", "QW_SPILL_MARGIN_GB",
               "QW_SPILL_NC", "QW_SPILL_NUMA", "QW_VIT_GEMM_ATTN", "QW_MOE_MMA", "QW_SKIP"}

    def validate(self) -> "Settings":
        def need(cond, msg):
            if not cond:
                raise ValueError("settings: " + msg)
        need(self.prefill_chunk >= 0 and self.prefill_chunk % 256 == 0, "prefill_chunk must be a multiple of 256")
        need(self.prefill_piece > 0 and self.prefill_piece % 256 == 0, "prefill_piece must be a positive multiple of 256")
        need(0.0 < self.decode_share <= 1.0, "decode_share must be in (0, 1]")
        need(self.prefill_lanes in (0, 1, 2), "prefill_lanes must be 0, 1 or 2")
        need(0 <= self.spec_max_rows <= 32, "spec_max_rows must be in 0..32")
        need(len(self.slots) >= 1 and all(s >= 256 for s in self.slots), "slots: at least one slot of >= 256 tokens")
        need(all(s >= 0 and s % 256 == 0 for s in self.slot_spill), "slot_spill: multiples of 256 tokens")
        need(self.slot_max_tokens >= 0 and self.slot_max_tokens % 256 == 0, "slot_max_tokens must be a multiple of 256")
        need(self.spill_policy in ("auto", "bind", "preferred", "interleave", "process"), "spill_policy")
        need(self.reasoning_effort in ("", "low", "medium", "high", "xhigh"), "reasoning_effort")
        need(self.host_cache_gb >= 0 and self.disk_cache_gb >= 0 and self.vision_cache_gb >= 0, "cache sizes must not be negative")
        need(self.stuck_seconds > 0 and self.exit_grace >= 0, "stuck_seconds / exit_grace")
        return self

    @classmethod
    def from_env(cls, env: Optional[Mapping[str, str]] = None, **overrides: Any) -> "Settings":
        env = os.environ if env is None else env
        s = cls()
        fields = {f.name: f for f in dataclasses.fields(cls) if f.name != "unknown"}
        for k, v in env.items():
            if not k.startswith("QW_"):
                continue
            name = cls.ALIASES.get(k, k[3:].lower())
            if name not in fields:
                if k not in cls.IGNORED:
                    s.unknown.append(k)
                continue
            s._set(name, v)
        for k, v in overrides.items():
            if v is None:
                continue
            if k not in fields:
                raise ValueError(f"settings: unknown option {k!r}")
            s._set(k, v)
        return s.validate()

    def _set(self, name: str, v: Any) -> None:
        cur = getattr(self, name)
        try:
            if isinstance(cur, bool):
                v = v if isinstance(v, bool) else _bool(v)
            elif isinstance(cur, int):
                v = int(v)
            elif isinstance(cur, float):
                v = float(v)
            elif isinstance(cur, list):
                v = _ints(v)
            else:
                v = str(v)
        except (TypeError, ValueError) as ex:
            raise ValueError(f"settings: QW_{name.upper()}={v!r}: {ex}") from ex
        setattr(self, name, v)

    def describe(self) -> str:
        """One line per group with the values that differ from the defaults first."""
        d, cur = Settings(), dataclasses.asdict(self)
        changed = {k: v for k, v in cur.items() if k != "unknown" and v != getattr(d, k)}
        out = ["settings: " + (", ".join(f"{k}={v}" for k, v in sorted(changed.items())) or "all defaults")]
        if self.unknown:
            out.append("settings: unknown variables ignored: " + ", ".join(sorted(self.unknown)))
        return "\n".join(out)

    def export_env(self, env: Dict[str, str]) -> None:
        """Write the values that other layers read from the environment (the server's media policy) back into ``env``."""
        env["QW_MEDIA_FETCH"] = "1" if self.media_fetch else "0"
        env["QW_MEDIA_ALLOW_PRIVATE"] = "1" if self.media_allow_private else "0"
        env["QW_VISION_MAX_PIXELS"] = str(self.vision_max_pixels)
        if self.video_max_pixels:
            env["QW_VIDEO_MAX_PIXELS"] = str(self.video_max_pixels)


_current: Optional[Settings] = None


def get() -> Settings:
    """The process-wide settings (parsed from the environment on first use)."""
    global _current
    if _current is None:
        _current = Settings.from_env()
    return _current


def set_current(s: Settings) -> None:
    global _current
    _current = s
