"""The Llama-4 decode step as ONE call into the C decode stack (mui_llama4_stack_*), and the two launches it adds:
the fused Llama-4 attention (prologue + ring / plain cache write + attention) and the router + top-k kernel.

Whole model: Hugging Face `Llama4ForCausalLM.generate(do_sample=False)` itself — fixtures hf_llama4_model.npz (head
dim 64: the stack runs the prologue, the cache write and flash decoding as separate launches) and
hf_llama4_model_d128.npz (head dim 128: the fused attention launch, both its cluster and its one-CTA-per-KV-head
variant), made by tests/golden/make_golden.py. 12-token prompt + 24 tokens cross four boundaries of the 8-token
attention chunk, so the ring caches of the chunked layers wrap several times.
Kernels: against the CPU oracle's composition of the same steps."""
import math
import os

import numpy as np
import pytest
import torch

from muillm_b200 import capi
from muillm_b200.llama4 import Llama4DecodeRunner, Llama4DecodeStack, llama4_freqs, llama4_weights_from_state_dict
from oracle import decode_oracle as oracle

pytestmark = pytest.mark.gpu

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
CFG = dict(layers=4, hidden=128, expert_intermediate=64, heads=2, kv_heads=1, head_dim=64, vocab=256, experts=4, top_k=1,
           eps=1e-5, rope_theta=500000.0, chunk=8, use_rope=[True, True, True, False], use_qk_norm=True,
           temperature_tuning=True, attn_scale=0.1, floor_scale=4.0)
FIXTURES = {64: "hf_llama4_model.npz", 128: "hf_llama4_model_d128.npz"}


def _load(head_dim, dtype=torch.float16):
    d = np.load(os.path.join(GOLD, FIXTURES[head_dim]))
    cfg = dict(CFG, head_dim=head_dim)
    assert [bool(v) for v in d["no_rope_layers"]] == cfg["use_rope"]
    sd = {k[3:]: torch.from_numpy(d[k]) for k in d.files if k.startswith("sd/")}
    return d, cfg, llama4_weights_from_state_dict(sd, cfg, dtype=dtype)


@pytest.mark.parametrize("head_dim", [64, 128])
@pytest.mark.parametrize("flags,graph", [(0, False), (capi.MUI_FLAG_PDL, False), (capi.MUI_FLAG_PDL, True), (0, True)])
def test_first_24_greedy_tokens_equal_hf_generate(head_dim, flags, graph):
    d, cfg, w = _load(head_dim)
    stack = Llama4DecodeStack(w, cfg, max_seq=64, max_new_tokens=64, flags=flags)
    got = stack.greedy(torch.from_numpy(d["prompt"]), 24, use_graph=graph).cpu()
    want = torch.from_numpy(d["tokens"])
    assert torch.equal(got, want), f"{got.tolist()} != {want.tolist()}"
    assert capi.device_status() == 0


@pytest.mark.parametrize("head_dim", [64, 128])
def test_prompt_logits_close_to_hf_fp32(head_dim):
    d, cfg, w = _load(head_dim)
    stack = Llama4DecodeStack(w, cfg, max_seq=64, max_new_tokens=64)
    stack.reset(0)
    stack.prefill(torch.from_numpy(d["prompt"]))
    torch.testing.assert_close(stack.logits().float().cpu(), torch.from_numpy(d["prompt_logits"]), rtol=2e-2,
                               atol=2e-2)


def test_stack_equals_kernel_by_kernel_runner_past_the_short_context_limit():
    """400 positions (beyond the 384 rows of the one-CTA-per-KV-head attention kernel, with a chunk of 96 that the
    ring wraps four times): the stack, stepped eagerly over the prompt and then by graph replay, against the runner
    that chains the stand-alone kernels from Python over plain caches. Both are fed the runner's greedy tokens, so
    every position is compared: logits within tolerance, and the same arg-max unless the runner's own logits hold the
    two candidates within the same tolerance. A handful of steps may miss the tolerance: where two router logits of a
    layer are one rounding step apart, the attention kernels' different summation orders can route that token to
    another expert (seen at one step in 24 in bf16); such a step stands alone, an error in the caches would not."""
    d, cfg, w = _load(128, dtype=torch.float16)
    cfg = dict(cfg, chunk=96)
    prompt = torch.randint(3, 256, (1, 40), generator=torch.Generator().manual_seed(5))
    steps = 400
    for flags in (0, capi.MUI_FLAG_PDL):
        run = Llama4DecodeRunner(w, cfg, max_seq=512)
        stack = Llama4DecodeStack(w, cfg, max_seq=512, max_new_tokens=512, flags=flags)
        stack.reset(0)
        side = torch.cuda.Stream()
        tok = int(prompt[0, 0])
        flips, outliers = 0, []
        for t in range(steps):
            ref = run.step(tok).float()
            tt = torch.tensor([tok], dtype=torch.int64)
            if t < prompt.shape[1]:
                stack.set_tokens(tt)
                stack.step()
            else:
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    if t == prompt.shape[1]:
                        stack.capture()
                    stack.set_tokens(tt)
                    stack.replay(1)
                torch.cuda.current_stream().wait_stream(side)
            got = stack.logits().float()
            err = float((got - ref).abs().max())
            a, b = int(torch.argmax(ref)), int(stack.next_tokens()[0].item())
            if err > 3e-2:
                outliers.append((t, round(err, 3)))
            elif a != b:
                assert float(ref[0, a] - ref[0, b]) < 3e-2, f"flags {flags} step {t}: runner {a}, stack {b}"
                flips += 1
            tok = int(prompt[0, t + 1]) if t + 1 < prompt.shape[1] else a
        assert len(outliers) <= 6, f"flags {flags}: logits off at steps {outliers}"
        assert all(t2 - t1 > 1 for (t1, _), (t2, _) in zip(outliers, outliers[1:])), \
            f"flags {flags}: consecutive steps off: {outliers}"
        assert flips <= 8, f"flags {flags}: {flips} arg-max flips in {steps} steps"
    assert capi.device_status() == 0


def _fused_attention(q, k, v, kc, vc, freqs, pos, rope, norm, tune, chunk, flags, eps=1e-5, attn_scale=0.1,
                     floor_scale=4.0, ws=None):
    B, Hq, _, D = q.shape
    Hkv = k.shape[1]
    qkv = torch.cat([q.reshape(B, Hq * D), k.reshape(B, Hkv * D), v.reshape(B, Hkv * D)], dim=1).contiguous()
    out = torch.empty(B, Hq * D, dtype=q.dtype, device=q.device)
    pid = torch.full((B,), pos, dtype=torch.int64, device=q.device)
    cp = torch.tensor([pos], dtype=torch.int64, device=q.device)
    capi.check(capi.lib().mui_llama4_rope_flash_decode(
        torch.cuda.current_stream().cuda_stream, capi.MUI_F16 if q.dtype == torch.float16 else capi.MUI_BF16, B, Hq,
        Hkv, D, kc.shape[2], freqs.shape[0], qkv.data_ptr(), freqs.data_ptr(), pid.data_ptr(), cp.data_ptr(),
        int(rope), int(norm), eps, int(tune), attn_scale, floor_scale, chunk, 1.0 / math.sqrt(D), kc.data_ptr(),
        vc.data_ptr(), out.data_ptr(), None if ws is None else ws.data_ptr(), 0 if ws is None else ws.numel(),
        kc.shape[2], flags))
    return out


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("case", [
    # (B, Hq, Hkv, position, chunk, cache rows, rope, norm, tune)
    (1, 10, 2, 37, 0, 64, True, True, False),       # Scout TP4 head counts, plain cache
    (1, 5, 1, 150, 64, 64, True, True, False),      # ring: row 22 of a 64-row chunk
    (1, 5, 1, 191, 64, 64, True, False, False),     # last row of a chunk
    (1, 5, 1, 192, 64, 64, True, True, False),      # first row of a chunk: attends itself only
    (2, 8, 2, 300, 0, 512, False, False, True),     # no-rope layer with temperature tuning, two sequences
    (1, 8, 8, 600, 0, 1024, True, True, True),      # beyond the one-CTA limit: cluster kernel and 4-way token split
    (1, 32, 8, 4000, 0, 4096, True, True, False),   # 16-way token split, 4 query heads per KV head
    (2, 5, 1, 2047, 2048, 2048, True, True, False),  # last row of a 2048-row ring, 8-way split, two sequences
], ids=["tp4", "ring22", "ring-last", "ring-first", "nope-b2", "long", "split16", "ring2048"])
def test_fused_llama4_attention_matches_oracle(dtype, case):
    B, Hq, Hkv, pos, chunk, rows, rope, norm, tune = case
    D = 128
    g = torch.Generator().manual_seed(pos + Hq)
    q = torch.randn(B, Hq, 1, D, generator=g).to(dtype)
    k = torch.randn(B, Hkv, 1, D, generator=g).to(dtype)
    v = torch.randn(B, Hkv, 1, D, generator=g).to(dtype)
    kc = torch.randn(B, Hkv, rows, D, generator=g).to(dtype)
    vc = torch.randn(B, Hkv, rows, D, generator=g).to(dtype)
    freqs = llama4_freqs(4096, D, 500000.0, "cpu")
    # oracle: the three prologue stages, the cache write at the ring / plain row, attention over the rows in view
    pe = freqs[pos: pos + 1].unsqueeze(0).expand(B, 1, D // 2, 2)
    cpos = torch.tensor([pos], dtype=torch.int64)
    qo, ko = q, k
    if rope:
        qo, ko = oracle.complex_rope(qo, pe), oracle.complex_rope(ko, pe)
    if norm:
        qo, ko = oracle.l2norm(qo, 1e-5), oracle.l2norm(ko, 1e-5)
    if tune:
        qo = oracle.temperature_tuning(qo, cpos, 0.1, 4.0)
    row = pos % chunk if chunk else pos
    kc_ref, vc_ref = kc.clone(), vc.clone()
    kc_ref[:, :, row] = ko[:, :, 0]
    vc_ref[:, :, row] = v[:, :, 0]
    want = oracle.decode_attention(qo, kc_ref[:, :, : row + 1], vc_ref[:, :, : row + 1]).reshape(B, Hq * D)
    # cluster kernel; token-split tensor-core kernel (twice: the second call finds the counters back at zero);
    # one CTA per KV head where the rows fit
    variants = [0, capi.MUI_FLAG_SPLIT_CONTEXT, capi.MUI_FLAG_SPLIT_CONTEXT]
    if row + 1 <= 384:
        variants.append(capi.MUI_FLAG_SHORT_CONTEXT)
    ws = torch.zeros(capi.lib().mui_flash_decode_workspace_bytes(B, Hq, Hkv, D, rows), dtype=torch.uint8, device="cuda")
    for flags in variants:
        kd, vd = kc.cuda(), vc.cuda()
        got = _fused_attention(q.cuda(), k.cuda(), v.cuda(), kd, vd, freqs.cuda(), pos, rope, norm, tune, chunk, flags,
                               ws=ws)
        torch.cuda.synchronize()
        torch.testing.assert_close(got.float().cpu(), want.float(), rtol=1e-2, atol=2e-3)
        # the new row was written where the ring says, bit for bit what the stand-alone prologue kernel gives; every
        # other row is untouched
        assert torch.equal(vd.cpu(), vc_ref)
        kd = kd.cpu()
        untouched = torch.ones(rows, dtype=torch.bool)
        untouched[row] = False
        assert torch.equal(kd[:, :, untouched], kc[:, :, untouched])
        torch.testing.assert_close(kd[:, :, row].float(), ko[:, :, 0].float(), rtol=1e-2, atol=1e-3)
    assert capi.device_status() == 0


def test_fused_llama4_attention_refuses_rows_past_the_cache():
    """A position whose row lies outside the cache records MUI_DEV_BAD_LENGTH and writes nothing."""
    D, rows = 128, 16
    z = torch.zeros(1, 1, 1, D, dtype=torch.float16, device="cuda")
    kc = torch.ones(1, 1, rows, D, dtype=torch.float16, device="cuda")
    vc = torch.ones(1, 1, rows, D, dtype=torch.float16, device="cuda")
    freqs = llama4_freqs(64, D, 500000.0, "cuda")
    _fused_attention(z, z, z, kc, vc, freqs, 20, True, False, False, 0, 0)
    status = capi.device_status(clear=True)
    assert status >> 24 == 5, f"expected MUI_DEV_BAD_LENGTH, got {status:#x}"
    assert torch.all(kc == 1) and torch.all(vc == 1)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("E,H,k", [(16, 5120, 1), (4, 128, 1), (128, 2048, 4), (7, 100, 2)])
def test_router_topk_kernel_matches_gemv_then_topk(dtype, E, H, k):
    g = torch.Generator().manual_seed(E + H)
    x = torch.randn(1, H, generator=g).to(dtype)
    nw = (1 + 0.01 * torch.randn(H, generator=g)).to(dtype)
    W = (torch.randn(E, H, generator=g) * 0.05).to(dtype)
    logits = oracle.linear(x, W, norm_weights=nw, eps=1e-5)
    want_s, want_i = oracle.topk_sigmoid(logits.reshape(1, 1, E), k)
    scratch = torch.zeros(E, dtype=torch.float32, device="cuda")
    counter = torch.zeros(16, dtype=torch.int32, device="cuda")
    vals = torch.empty(k, dtype=dtype, device="cuda")
    idx = torch.empty(k, dtype=torch.int64, device="cuda")
    xc, nc, Wc = x.cuda(), nw.cuda(), W.cuda()
    for _ in range(2):  # the second call finds the counter back at zero
        capi.check(capi.lib().mui_router_topk_sigmoid_forward(
            torch.cuda.current_stream().cuda_stream, capi.MUI_F16 if dtype == torch.float16 else capi.MUI_BF16, E, H,
            k, nc.data_ptr(), 1e-5, Wc.data_ptr(), xc.data_ptr(), scratch.data_ptr(), counter.data_ptr(),
            vals.data_ptr(), idx.data_ptr(), 0))
    torch.cuda.synchronize()
    assert int(counter[0]) == 0
    got_logits = scratch.cpu()
    torch.testing.assert_close(got_logits, logits.float().reshape(-1), rtol=1e-2, atol=2e-3)
    # indices: the oracle's, unless its logits at the two candidates are a rounding step apart
    wi, gi = want_i.reshape(-1).tolist(), idx.cpu().tolist()
    for a, b in zip(wi, gi):
        if a != b:
            assert abs(float(logits.reshape(-1)[a]) - float(logits.reshape(-1)[b])) < 2e-2, (wi, gi)
    torch.testing.assert_close(vals.float().cpu(), torch.sigmoid(got_logits[idx.cpu()]).to(dtype).float(), rtol=1e-2,
                               atol=1e-3)
