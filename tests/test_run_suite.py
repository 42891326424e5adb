"""The measurement suite's harness on a fake runner: order, JSON collection, failures recorded without stopping."""
import subprocess
import types

from qwb200.tools import run_suite as RS


def test_suite_collects_last_json_line_and_goes_on_after_a_failure():
    calls = []

    def fake(cmd, **kw):
        calls.append(cmd)
        name = [c for c in cmd if c.startswith("qwb200.tools.") or c.endswith("bench.py")][0]
        if name.endswith("gemv_bench"):
            return types.SimpleNamespace(returncode=3, stdout="boom\n", stderr="trace")
        if name.endswith("launch_bench"):
            raise subprocess.TimeoutExpired(cmd, 1)
        return types.SimpleNamespace(returncode=0, stdout='noise\n{"a": 1}\n{"value": 2}\n', stderr="")
    rep = RS.run_suite(1, ["kernels", "decode", "comm"], True, 5, runner=fake)
    r = rep["results"]
    assert list(r) == ["gemm_bench", "gemv_bench", "launch_bench", "bench", "rows_bench"]          # comm needs more than one GPU
    assert r["gemm_bench"]["json"] == {"value": 2} and r["gemm_bench"]["rc"] == 0
    assert r["gemv_bench"]["rc"] == 3 and "boom" in r["gemv_bench"]["tail"]
    assert r["launch_bench"]["rc"] == -9
    assert r["bench"]["json"] == {"value": 2}


def test_multi_gpu_plan_uses_torchrun_on_loopback():
    plan = RS.stages(4, False)
    cmd = dict(plan["comm"])["comm_bench"]
    assert "torch.distributed.run" in cmd and "127.0.0.1" in cmd and cmd[cmd.index("--nproc-per-node") + 1] == "4"
    assert "--gpus" in dict(plan["decode"])["bench"]
