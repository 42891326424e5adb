"""``python -m qwserve``: load the engine through its C API and serve the OpenAI-style HTTP API
(reference behaviour: server/qwserve/__main__.py:15-69)."""
import argparse
import logging
import sys

from aiohttp import web


def parse_args(argv=None):
    p = argparse.ArgumentParser(prog="qwserve")
    p.add_argument("--host", default="127.0.0.1")
    p.add_argument("--port", type=int, default=8000)
    p.add_argument("--model-dir", required=True, help="checkpoint directory (config.json, safetensors, tokenizer.json)")
    p.add_argument("--ple-dir", default=None, help="directory of the n-gram embedding table")
    p.add_argument("--lib", default=None, help="path of libqw_engine.so")
    p.add_argument("--served-model-name", default="qw")
    p.add_argument("--slots", default="131072,32768,32768,32768", help="context capacity of each slot, comma separated")
    p.add_argument("--kv-spill", choices=["on", "off"], default="off", help="keep KV pages beyond the resident window in host memory")
    p.add_argument("--slot-max-tokens", type=int, default=0, help="with --kv-spill on: total capacity of a slot")
    p.add_argument("--weight-cache-dir", default=None, help="directory for the converted-weights cache (faster restarts)")
    p.add_argument("--prefill-chunk", type=int, default=4096)
    p.add_argument("--reasoning-effort", default=None, choices=[None, "low", "medium", "high", "xhigh"])
    p.add_argument("--thinking-budget", type=int, default=0, help="default reasoning budget in tokens (0 = unlimited)")
    p.add_argument("--mtp", type=int, default=3, help="draft tokens per step (0 = plain decoding)")
    p.add_argument("--host-cache-gb", type=float, default=32.0)
    p.add_argument("--disk-cache-dir", default=None)
    p.add_argument("--disk-cache-gb", type=float, default=0.0)
    p.add_argument("--no-vision", action="store_true")
    p.add_argument("--no-dashboard", action="store_true")
    p.add_argument("--devices", default="0", help="GPUs of the engine, comma separated: 1, 2, 4 or 8 of them (tensor + expert parallel)")
    p.add_argument("--synthetic", default=None, help="serve a random-weight model of this size (tiny|slice2|full): for tests")
    return p.parse_args(argv)


def main(argv=None):
    a = parse_args(argv)
    logging.basicConfig(level=logging.INFO, format="%(asctime)s %(message)s")
    from .api import Server, make_app
    from .engine import Engine
    from .prompt import Prompter
    from .scheduler import Scheduler
    opts = {"model_dir": a.model_dir, "ple_dir": a.ple_dir, "prefill_chunk": a.prefill_chunk,
            "slots": [int(x) for x in a.slots.split(",")], "host_cache_gb": a.host_cache_gb, "mtp": a.mtp > 0,
            "vision": not a.no_vision, "devices": [int(x) for x in a.devices.split(",") if x.strip() != ""]}
    if a.mtp > 12:
        raise SystemExit("--mtp: at most 12 drafts per step (a verification run must not wrap the 16-row state rings)")
    if a.synthetic:
        opts["synthetic"] = a.synthetic
    if a.kv_spill == "on":
        opts["kv_spill"], opts["slot_max_tokens"] = True, a.slot_max_tokens
    if a.weight_cache_dir:
        opts["weight_cache_dir"] = a.weight_cache_dir
    if a.disk_cache_dir:
        opts["disk_cache_dir"], opts["disk_cache_gb"] = a.disk_cache_dir, a.disk_cache_gb
    eng = Engine(opts, a.lib)
    prompter = Prompter(a.model_dir)
    pre = None
    if not a.no_vision and eng.has_vision:
        from .vision import Preprocessor
        pre = Preprocessor(a.model_dir)
    # server-side switches that deployments set through the environment (QW_STUCK_SECONDS, QW_EXIT_GRACE, QW_DECODE_SHARE, ...)
    import os

    def envf(name, default):
        try:
            return float(os.environ.get(name, default))
        except ValueError:
            raise SystemExit(f"{name} must be a number")
    sched = Scheduler(eng, drafts=a.mtp, prefill_piece=min(int(envf("QW_PREFILL_PIECE", 2048)), a.prefill_chunk),
                      decode_share=envf("QW_DECODE_SHARE", 0.25), stuck_seconds=envf("QW_STUCK_SECONDS", 300),
                      exit_grace=envf("QW_EXIT_GRACE", 30), log_interval=envf("QW_LOG_INTERVAL", 30), log=logging.info)
    from .api import model_sampling_defaults
    srv = Server(eng, prompter, sched, a.served_model_name, preprocessor=pre, default_effort=a.reasoning_effort,
                 default_budget=a.thinking_budget, sampling_defaults=model_sampling_defaults(a.model_dir))
    im_end = prompter.token_id("<|im_end|>")
    if im_end is not None:
        eng.set_boundary_token(im_end)
    sched.start(watchdog=os.environ.get("QW_WATCHDOG_EXIT", "1") != "0")
    web.run_app(make_app(srv, dashboard=not a.no_dashboard), host=a.host, port=a.port, access_log=None)
    eng.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
