"""Host-side contract checks that need no GPU: the reference arm of bench.py prints one JSON line with the keys the
bench contract names, and the drop-in's small host decisions (dispatch rule for non-16-bit weights, shared-memory fit
of the packed 8-bit gate/up kernel) behave as documented."""
import json
import os
import subprocess
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_contract_line():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                        "--warmup", "1"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
                "scaling", "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in d, key
    assert d["impl"] == "reference" and d["unit"] == "tokens/s" and d["higher_is_better"] is True
    assert d["value"] > 0 and d["e2e"]["value"] == d["value"]
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1 and d["cpu_baseline"]["sample"]
    assert "workload" in d["config"] and "Llama-3.1-8B" in d["config"]["workload"]


def test_other_ranks_of_the_reference_arm_print_nothing():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2"],
                       capture_output=True, text=True, timeout=120, cwd=ROOT, env=env)
    assert r.returncode == 0 and r.stdout.strip() == ""


def test_dropin_host_decisions():
    from muillm_b200 import muillm_ext as ext

    # fp16 / bf16 weights on a GPU dispatch to the kernels; anything else on a GPU takes torch's ops; CPU tensors are
    # left to the operators, which refuse them
    class FakeW:
        def __init__(self, is_cuda, dtype):
            self.is_cuda, self.dtype = is_cuda, dtype
    assert not ext._not_dispatchable_on_gpu(FakeW(True, torch.float16))
    assert not ext._not_dispatchable_on_gpu(FakeW(True, torch.bfloat16))
    assert ext._not_dispatchable_on_gpu(FakeW(True, torch.float32))
    assert not ext._not_dispatchable_on_gpu(FakeW(False, torch.float32))
    # packed 8-bit gate/up: one row of H = 4096 fits beside two weight stages, a row of 80k activations does not
    assert ext._packed_gateup_fits(1, 4096, 7)
    assert ext._packed_gateup_fits(1, 14336, 7)
    assert not ext._packed_gateup_fits(1, 81920, 7)
