"""Pins the CPU oracle against the golden fixtures of tests/golden/ (made by tests/golden/make_golden.py from the
reference's importable Python and from the HF modules its tests compare to). Runs without a GPU."""
import os

import numpy as np
import pytest
import torch

from oracle import decode_oracle as oracle

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(scope="module")
def ref():
    return np.load(os.path.join(GOLD, "reference_python.npz"))


@pytest.fixture(scope="module")
def hf():
    return np.load(os.path.join(GOLD, "hf_modules.npz"))


def T(a, dtype=None):
    t = torch.from_numpy(np.asarray(a))
    return t.to(dtype) if dtype is not None else t


@pytest.mark.parametrize("gs", [128, 32])
def test_rtn_group_quantizer_bit_exact(ref, gs):
    w = T(ref[f"rtn_g{gs}_w"], torch.float16)
    shift = gs.bit_length() - 1
    q, sm = oracle.rtn_group_quantize(w, group_shift=shift)
    assert torch.equal(q, T(ref[f"rtn_g{gs}_q"]))
    assert torch.equal(sm, T(ref[f"rtn_g{gs}_scales_min"], torch.float16))
    deq = oracle.rtn_group_dequantize(q, sm, group_shift=shift)
    # the reference de-quantises in fp16 arithmetic (uint8 * fp16 scale + fp16 min); fp32 math rounded once
    # differs from it by at most two fp16 ulps at the weight magnitude (|w| < 0.125)
    torch.testing.assert_close(deq, T(ref[f"rtn_g{gs}_dequant_f16"]), rtol=0, atol=6.2e-5)


@pytest.mark.parametrize("k", [1, 2])
def test_topk_sigmoid(ref, k):
    logits = T(ref[f"topk{k}_logits"], torch.bfloat16)
    v, i = oracle.topk_sigmoid(logits, k)
    assert torch.equal(i, T(ref[f"topk{k}_indices"]))
    assert torch.equal(v.float(), T(ref[f"topk{k}_values"]))


def test_rmsnorm_matches_reference_cpu_branch(ref):
    x = T(ref["ref_rmsnorm_x"], torch.float16)
    w = T(ref["ref_rmsnorm_w"], torch.float16)
    y = oracle.rmsnorm(x, w, 1e-5)
    assert torch.equal(y.float(), T(ref["ref_rmsnorm_y"]))


def test_fused_norm_linear_matches_hf(hf):
    x, nw, w, b = (T(hf[k]) for k in ("hf_normlinear_x", "hf_normlinear_nw", "hf_normlinear_w", "hf_normlinear_b"))
    y32 = oracle.linear(x, w, norm_weights=nw, eps=1e-5, add_bias=b)
    torch.testing.assert_close(y32, T(hf["hf_normlinear_f32_y"]), rtol=1e-5, atol=1e-5)
    h = torch.float16
    y16 = oracle.linear(x.to(h), w.to(h), norm_weights=nw.to(h), eps=1e-5, add_bias=b.to(h))
    torch.testing.assert_close(y16.float(), T(hf["hf_normlinear_f16_y"]), rtol=1e-2, atol=1e-3)


def test_mlp_matches_hf(hf):
    y = oracle.mlp(T(hf["hf_mlp_x"]), T(hf["hf_mlp_gate"]), T(hf["hf_mlp_up"]), T(hf["hf_mlp_down"]))
    torch.testing.assert_close(y, T(hf["hf_mlp_y"]), rtol=1e-5, atol=1e-5)


def test_rope_and_attention_match_hf(hf):
    cos, sin = oracle.rope_tables(37, 32, 500000.0, torch.float32)
    torch.testing.assert_close(cos, T(hf["hf_rope_cos"]), rtol=1e-6, atol=1e-6)
    torch.testing.assert_close(sin, T(hf["hf_rope_sin"]), rtol=1e-6, atol=1e-6)
    q, k = T(hf["hf_rope_q"]), T(hf["hf_rope_k"])
    pos = torch.arange(37)[None, :].expand(2, 37)
    qr = oracle.rope_apply(q, cos, sin, pos)
    kr = oracle.rope_apply(k, cos, sin, pos)
    torch.testing.assert_close(qr, T(hf["hf_rope_q_rot"]), rtol=1e-6, atol=1e-6)
    torch.testing.assert_close(kr, T(hf["hf_rope_k_rot"]), rtol=1e-6, atol=1e-6)
    out = oracle.decode_attention(qr[:, :, -1:, :], kr, T(hf["hf_attn_v"]))
    torch.testing.assert_close(out, T(hf["hf_attn_out"]), rtol=1e-5, atol=1e-5)


def _weights_from_hf_state_dict(hf, layers):
    sd = {k[len("hf_model_sd/"):]: T(hf[k]).float() for k in hf.files if k.startswith("hf_model_sd/")}
    w = {"embed": sd["model.embed_tokens.weight"], "lm_head": sd["lm_head.weight"], "norm": sd["model.norm.weight"],
         "qkv": [], "o": [], "gate": [], "up": [], "down": [], "ln1": [], "ln2": []}
    for l in range(layers):
        p = f"model.layers.{l}."
        w["qkv"].append(torch.cat([sd[p + "self_attn.q_proj.weight"], sd[p + "self_attn.k_proj.weight"],
                                   sd[p + "self_attn.v_proj.weight"]], dim=0))
        w["o"].append(sd[p + "self_attn.o_proj.weight"])
        w["gate"].append(sd[p + "mlp.gate_proj.weight"])
        w["up"].append(sd[p + "mlp.up_proj.weight"])
        w["down"].append(sd[p + "mlp.down_proj.weight"])
        w["ln1"].append(sd[p + "input_layernorm.weight"])
        w["ln2"].append(sd[p + "post_attention_layernorm.weight"])
    return w


def test_whole_model_greedy_tokens_match_hf_generate(hf):
    """The oracle decoder (QKV concatenated like MuiMultiLinear, token-by-token prefill, static cache) reproduces
    HF LlamaForCausalLM.generate(do_sample=False): same 32 tokens, same prompt logits."""
    cfg = dict(layers=2, hidden=128, intermediate=256, heads=4, kv_heads=2, head_dim=32, vocab=256, eps=1e-5,
               rope_theta=500000.0)
    w = _weights_from_hf_state_dict(hf, 2)
    prompt = T(hf["hf_model_prompt"])
    model = oracle.LlamaOracle(w, cfg, max_T=64)
    logits = model.forward(prompt)
    torch.testing.assert_close(logits, T(hf["hf_model_prompt_logits"]), rtol=1e-4, atol=1e-4)
    toks = oracle.LlamaOracle(w, cfg, max_T=64).greedy(prompt, 32)
    assert torch.equal(toks, T(hf["hf_model_tokens"]))


def test_symmetric_row_quantizer_round_trip():
    g = torch.Generator().manual_seed(0)
    w = (torch.randn(16, 64, generator=g) * 0.02).to(torch.float16)
    q, s = oracle.rtn_symrow_quantize(w)
    assert q.dtype == torch.int8 and q.abs().max() <= 127 and (q.abs().amax(dim=1) == 127).all()
    err = (oracle.rtn_symrow_dequantize(q, s) - w.float()).abs()
    assert (err <= 0.51 * s.float()[:, None] + 1e-6).all()


def test_all_reduce_fixed_order_is_deterministic():
    g = torch.Generator().manual_seed(0)
    parts = [torch.randn(1, 64, generator=g) for _ in range(8)]
    a = oracle.all_reduce_fixed_order(parts, torch.float16)
    b = oracle.all_reduce_fixed_order(parts, torch.float16)
    assert torch.equal(a, b)
    torch.testing.assert_close(a.float(), torch.stack(parts).sum(0), rtol=2e-3, atol=2e-3)


# ---- Llama-4 attention prologue and sliding window (HF Llama-4 building blocks) ----------------------------------


@pytest.fixture(scope="module")
def l4():
    return np.load(os.path.join(GOLD, "hf_llama4_ops.npz"))


@pytest.mark.parametrize("tag,dtype", [("f16", torch.float16), ("bf16", torch.bfloat16)])
def test_llama4_complex_rope_and_l2norm_bit_exact(l4, tag, dtype):
    pe = T(l4["l4_pos_embeds"])
    for name in ("q", "k"):
        x = T(l4[f"l4_{name}"], dtype)
        rot = oracle.complex_rope(x, pe)
        assert torch.equal(rot.float(), T(l4[f"l4_rope_{tag}_{name}"]))
        assert torch.equal(oracle.l2norm(rot, 1e-5).float(), T(l4[f"l4_norm_{tag}_{name}"]))


def test_llama4_temperature_tuning_bit_exact(l4):
    q = T(l4["l4_q"], torch.bfloat16)
    got = oracle.temperature_tuning(q, T(l4["l4_temp_pos"]), 0.1, 8192.0)
    assert torch.equal(got.float(), T(l4["l4_temp_bf16_q"]))


def test_sliding_window_states_match_hf_layer(l4):
    ks, vs = T(l4["l4_slide_k"], torch.float16), T(l4["l4_slide_v"], torch.float16)
    W = 6
    kc = torch.zeros(1, ks.shape[1], W, ks.shape[3], dtype=torch.float16)
    vc = torch.zeros_like(kc)
    _, _, kc, vc = oracle.sliding_cache_update(ks[:, :, :4], vs[:, :, :4], kc, vc, torch.arange(4), 4)
    for step in range(4, 12):
        k_st, v_st, kc, vc = oracle.sliding_cache_update(ks[:, :, step:step + 1], vs[:, :, step:step + 1], kc, vc,
                                                         torch.tensor([step]), step + 1)
        assert torch.equal(k_st.float(), T(l4[f"l4_slide_states_k_{step}"])), step
        assert torch.equal(v_st.float(), T(l4[f"l4_slide_states_v_{step}"])), step


def test_add_tokens_check_finished_matches_generation_loop_semantics():
    ids = torch.tensor([[5, 6, 7], [8, 9, 10], [1, 2, 3]])
    nxt = torch.tensor([11, 2, 99], dtype=torch.int32)
    unf = torch.tensor([1, 1, 0])
    out, u = oracle.add_tokens_check_finished(ids, nxt, unf, True, 0, torch.tensor([2, 77]), True, 5)
    assert out.tolist() == [[5, 6, 7, 11], [8, 9, 10, 2], [1, 2, 3, 0]]
    assert u.tolist() == [1, 0, 0]
    out, u = oracle.add_tokens_check_finished(ids, nxt, unf, True, 0, torch.tensor([2]), True, 4)
    assert u.tolist() == [0, 0, 0]
    out, u = oracle.add_tokens_check_finished(ids, nxt, unf, False, 0, torch.tensor([2]), False, -1)
    assert out[:, -1].tolist() == [11, 2, 99] and u.tolist() == [1, 1, 0]


@pytest.fixture(scope="module")
def moe_mask():
    return np.load(os.path.join(GOLD, "hf_moe_mask.npz"))


def test_moe_mlp_matches_hf_llama4_moe_block(moe_mask):
    """Router (plain linear), top-k + sigmoid, routed experts on score-scaled inputs, shared expert: HF
    `Llama4TextMoe` (the module tests/test_gateupdownmlpmoe.py of the reference compares with), fp32."""
    m = moe_mask
    x, k = T(m["moe_x"]), int(m["moe_top_k"])
    logits = oracle.linear(x.reshape(1, -1), T(m["moe_router_w"]))
    np.testing.assert_allclose(logits.numpy(), m["moe_router_logits"], rtol=1e-5, atol=1e-6)
    scores, idx = oracle.topk_sigmoid(logits, k)
    E = m["moe_router_w"].shape[0]
    y = oracle.moe_mlp(x, T(m["moe_gate"]), T(m["moe_up"]), T(m["moe_down"]), 1, 1 + E, scores, idx)
    np.testing.assert_allclose(y.numpy(), m["moe_y"], rtol=1e-5, atol=1e-6)


def test_masked_decode_attention_matches_hf_eager_attention(moe_mask):
    """One query token over a cache with masked-out rows: HF `eager_attention_forward` with an additive mask."""
    m = moe_mask
    o = oracle.decode_attention(T(m["mattn_q"]), T(m["mattn_k"]), T(m["mattn_v"]), mask=T(m["mattn_mask"]))
    np.testing.assert_allclose(o.numpy(), m["mattn_out"], rtol=1e-5, atol=1e-6)


def test_packed_gateup_layout_matches_the_references_packing_code():
    """`parity_utils.reference_gateup_pack` (what the GPU tests and benchmarks feed to the packed 8-bit gate/up kernel)
    reproduces the tensors the reference's own packing code built from RTNQuantizer outputs (fixture
    reference_pack.npz: muillm/modules/quantized/int8gateupdownmlp.py:211-230)."""
    from parity_utils import reference_gateup_pack

    m = np.load(os.path.join(GOLD, "reference_pack.npz"))
    pack, sm = reference_gateup_pack(T(m["gate_q"]), T(m["gate_scales_min"]), T(m["up_q"]), T(m["up_scales_min"]))
    assert np.array_equal(pack.numpy(), m["pack"]) and np.array_equal(sm.numpy(), m["pack_scales_min"])
    assert tuple(pack.shape) == (12, 256, 2) and tuple(sm.shape) == (24, 2, 2)
    # and the oracle's quantiser made the same bytes the reference's RTNQuantizer did, so packing oracle outputs
    # gives the reference's pack
    g = torch.Generator().manual_seed(5)
    gw = (torch.randn(12, 256, generator=g) * 0.02).to(torch.float16)
    gq, gsm = oracle.rtn_group_quantize(gw, group_shift=7)
    assert np.array_equal(gq.numpy(), m["gate_q"]) and np.array_equal(gsm.float().numpy(), m["gate_scales_min"])
