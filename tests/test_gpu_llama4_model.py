"""A whole Llama-4 text model (BASELINE config 5's architecture at toy size: MoE with a shared expert and top-1 sigmoid
routing in every layer, chunked attention of 8 tokens with interleaved rope + QK L2 norm in three layers, full
attention with temperature tuning and no rope in the fourth) decoded through the library's kernels, against Hugging
Face `Llama4ForCausalLM.generate(do_sample=False)` itself: fixture tests/golden/hf_llama4_model.npz (weights, prompt,
HF's 24 tokens and last-prompt-token logits in fp32; made by tests/golden/make_golden.py llama4_model). The 36 positions
cross four chunk boundaries."""
import os

import numpy as np
import pytest
import torch

from muillm_b200 import capi
from muillm_b200.llama4 import Llama4DecodeRunner, llama4_weights_from_state_dict

pytestmark = pytest.mark.gpu

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
CFG = dict(layers=4, hidden=128, expert_intermediate=64, heads=2, kv_heads=1, head_dim=64, vocab=256, experts=4, top_k=1,
           eps=1e-5, rope_theta=500000.0, chunk=8, use_rope=[True, True, True, False], use_qk_norm=True,
           temperature_tuning=True, attn_scale=0.1, floor_scale=4.0)


def _runner(flags):
    d = np.load(os.path.join(GOLD, "hf_llama4_model.npz"))
    assert [bool(v) for v in d["no_rope_layers"]] == CFG["use_rope"]
    sd = {k[3:]: torch.from_numpy(d[k]) for k in d.files if k.startswith("sd/")}
    w = llama4_weights_from_state_dict(sd, CFG, dtype=torch.float16)
    return d, Llama4DecodeRunner(w, CFG, max_seq=64, flags=flags)


@pytest.mark.parametrize("flags", [0, capi.MUI_FLAG_PDL])
def test_first_24_greedy_tokens_equal_hf_generate(flags):
    d, run = _runner(flags)
    got = run.greedy(torch.from_numpy(d["prompt"])[0], 24).cpu()
    want = torch.from_numpy(d["tokens"])[0]
    assert torch.equal(got, want), f"{got.tolist()} != {want.tolist()}"
    assert capi.device_status() == 0


def test_prompt_logits_close_to_hf_fp32():
    d, run = _runner(0)
    logits = None
    for t in d["prompt"][0].tolist():
        logits = run.step(t)
    torch.testing.assert_close(logits.float().cpu(), torch.from_numpy(d["prompt_logits"]), rtol=2e-2, atol=2e-2)


def test_captured_device_loop_equals_host_loop():
    """Token, position and attended length kept on the device and the step replayed as a CUDA graph produce the
    tokens of the host-driven loop (same model with one chunk spanning the cache, which the device loop requires)."""
    d = np.load(os.path.join(GOLD, "hf_llama4_model.npz"))
    sd = {k[3:]: torch.from_numpy(d[k]) for k in d.files if k.startswith("sd/")}
    cfg = dict(CFG, chunk=64)
    w = llama4_weights_from_state_dict(sd, cfg, dtype=torch.float16)
    prompt = torch.from_numpy(d["prompt"])[0]
    want = Llama4DecodeRunner(w, cfg, max_seq=64, flags=capi.MUI_FLAG_PDL).greedy(prompt, 16).cpu().tolist()
    run = Llama4DecodeRunner(w, cfg, max_seq=64, flags=capi.MUI_FLAG_PDL)
    logits = None
    for t in prompt.tolist():
        logits = run.step(t)
    got = [int(torch.argmax(logits.float()).item())]
    run.start_device_loop(got[0], pos=prompt.numel())
    run.step_device()
    got.append(int(run.d_token.item()))
    run.capture(warmup=2)           # two more eager steps on the capture stream
    torch.cuda.synchronize()
    for i in range(12):
        run.replay(1)
        torch.cuda.synchronize()
        got.append(int(run.d_token.item()))
    # tokens 2 and 3 were produced (and consumed) by the warm-up steps inside capture()
    assert got[:2] == want[:2] and got[2:] == want[4:16], f"{got} vs {want}"
    assert capi.device_status() == 0
