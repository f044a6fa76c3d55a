"""Greedy tokens of the GPU decode stack against Hugging Face `LlamaForCausalLM.generate(do_sample=False)` itself
(fixture tests/golden/hf_llama_d64.npz: weights, prompt, the 32 tokens HF generated, made by make_golden.py)."""
import os

import numpy as np
import pytest
import torch

from muillm_b200 import capi
from muillm_b200.decoder_stack import LlamaDecodeStack
from muillm_b200.hf import llama_weights_from_state_dict

pytestmark = pytest.mark.gpu

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
CFG = dict(layers=2, hidden=128, intermediate=256, heads=2, kv_heads=1, head_dim=64, vocab=256, eps=1e-5,
           rope_theta=500000.0)


@pytest.mark.parametrize("flags,graph", [(0, False), (capi.MUI_FLAG_PDL, True)])
def test_first_32_greedy_tokens_equal_hf_generate(flags, graph):
    d = np.load(os.path.join(GOLD, "hf_llama_d64.npz"))
    sd = {k[3:]: torch.from_numpy(d[k]) for k in d.files if k.startswith("sd/")}
    w = llama_weights_from_state_dict(sd, CFG["layers"], dtype=torch.float16)
    stack = LlamaDecodeStack(w, CFG, max_seq=64, batch=1, max_new_tokens=64, flags=flags)
    prompt = torch.from_numpy(d["prompt"])
    got = stack.greedy(prompt, 32, use_graph=graph).cpu()
    want = torch.from_numpy(d["tokens"])
    assert torch.equal(got, want), f"{got.tolist()} != {want.tolist()}"
    assert capi.device_status() == 0


def test_prompt_logits_close_to_hf_fp32():
    d = np.load(os.path.join(GOLD, "hf_llama_d64.npz"))
    sd = {k[3:]: torch.from_numpy(d[k]) for k in d.files if k.startswith("sd/")}
    w = llama_weights_from_state_dict(sd, CFG["layers"], dtype=torch.float16)
    stack = LlamaDecodeStack(w, CFG, max_seq=64, batch=1, max_new_tokens=64)
    stack.reset(0)
    stack.prefill(torch.from_numpy(d["prompt"]))
    got = stack.logits().float().cpu()
    torch.testing.assert_close(got, torch.from_numpy(d["prompt_logits"]), rtol=2e-2, atol=2e-2)
