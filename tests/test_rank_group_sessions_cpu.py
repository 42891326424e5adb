"""Two ranks on CPU, each a real Session over the rule-based engine, behind one ``CApi``: rank 0 in this process, rank 1
a worker process that replays every call.  Nothing is exchanged but the calls, so the ranks stay in step only if
everything above the kernels is deterministic - slot choice, reuse decisions, draft counts, acceptance."""
import json
import os
import sys

from rule_engine import RuleOps, patch_session_module

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TESTS = os.path.dirname(os.path.abspath(__file__))


def test_two_ranks_replay_a_serving_session_identically(tmp_path, monkeypatch):
    patch_session_module(monkeypatch)
    from qwb200.capi_impl import CApi
    from qwb200.engine.sampling import SamplingParams
    from qwb200.parallel.rank_group import RankGroup
    from qwb200.session.session import StepReq
    opts = {"slots": 3, "unreliable_drafts": True}
    env = dict(os.environ, PYTHONPATH=TESTS + os.pathsep + ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    group = RankGroup.spawn(2, ["--builder", "rule_engine:build_rank"], {"options": opts, "master_port": 0},
                            lambda: RuleOps(dict(opts, rank=0)), ready_timeout=120, ack_timeout=60, env=env)
    api = CApi(group.local, group)
    try:
        ops = api.ops                                      # the group: every call runs on both ranks
        system = [(i * 37) % 250 for i in range(700)]
        pending = {}
        for turn, tail in enumerate(([1, 2, 3], [9, 8, 7, 6], [1, 2, 3])):
            prompt = system + tail
            slot = ops.acquire(prompt, 64)
            assert slot >= 0
            ops.begin_prompt(slot, prompt)
            while not ops.prefill_some(slot, 256):
                pass
            tok, _ = ops.sample_prompt(slot, SamplingParams())
            pending[slot] = tok
            for _ in range(6):                             # speculative steps for every request in flight
                outs = ops.generate([StepReq(s, t, 32, 0, SamplingParams()) for s, t in sorted(pending.items())], 3)
                for (s, _), o in zip(sorted(pending.items()), outs):
                    pending[s] = o.tokens[-1]
            if turn == 1:                                  # one request ends: its slot is free for the repeat of the first prompt
                ops.release(slot)
                del pending[slot]
        assert api.failure() == ""
        ops.dump(str(tmp_path / "state"))
        a = json.load(open(tmp_path / "state.rank0"))
        b = json.load(open(tmp_path / "state.rank1"))
        assert a == b and a["fed"] > 700 and any(len(t) > 700 for t in a["tokens"])
        assert a["stats"]["reused_tokens"] >= 512          # the shared system prompt came from the store or a snapshot on both ranks
    finally:
        api.close()


def test_media_prompts_reach_every_rank(tmp_path, monkeypatch):
    patch_session_module(monkeypatch)
    """A prompt with an image on two ranks: the media descriptors are read on rank 0, travel to the worker by value, both
    ranks map the pad tokens to the same vision ids and feed the same tokens."""
    import ctypes as C
    import numpy as np
    from qwb200.capi_impl import CApi, QwMedia
    from qwb200.models.config import ModelConfig
    from qwb200.parallel.rank_group import RankGroup
    from rule_engine import StubTower, build_rank_with_vision
    opts = {"slots": 2}
    env = dict(os.environ, PYTHONPATH=TESTS + os.pathsep + ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    group = RankGroup.spawn(2, ["--builder", "rule_engine:build_rank_with_vision"], {"options": opts, "master_port": 0},
                            lambda: build_rank_with_vision({"options": opts, "rank": 0}, 2, patch_module=False), ready_timeout=120, ack_timeout=60, env=env)
    api = CApi(group.local, group)
    try:
        vc, cfg = StubTower().cfg, ModelConfig.tiny()
        h, w = 4, 6
        n_img = h * w // (vc.merge * vc.merge)
        patches = np.random.default_rng(3).standard_normal((2 * h * w, vc.patch_in)).astype(np.float32)
        starts = np.asarray([4], dtype=np.int64)
        toks = np.asarray([5, 6, 7, 8] + [cfg.image_pad] * n_img + [9, 10, 11], dtype=np.int32)
        m = (QwMedia * 1)(QwMedia(hash=77, video=0, t=1, h=h, w=w, patches=patches.ctypes.data_as(C.POINTER(C.c_float)),
                                  starts=starts.ctypes.data_as(C.POINTER(C.c_int64))))
        slot = api.acquire(toks.ctypes.data, len(toks), 16, C.addressof(m), 1)
        assert slot >= 0
        api.begin_prompt(slot, toks.ctypes.data, len(toks), C.addressof(m), 1)
        while not api.prefill_some(slot, 256):
            pass
        assert api.failure() == ""
        api.ops.dump(str(tmp_path / "media"))
        a = json.load(open(tmp_path / "media.rank0"))
        b = json.load(open(tmp_path / "media.rank1"))
        fed = a["tokens"][slot]
        assert a == b and len(fed) == len(toks) and all(t < 0 for t in fed[4:4 + n_img]) and fed[:4] == [5, 6, 7, 8]
    finally:
        api.close()
