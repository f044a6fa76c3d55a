"""The `muillm_ext` drop-in driven the way the reference's Python modules drive the torch extension: module handles
built once, then one call per layer / per stack per token — compared with the CPU oracle."""
import math

import pytest
import torch

from muillm_b200 import muillm_ext as ext
from oracle import decode_oracle as oracle

pytestmark = pytest.mark.gpu

CFG = dict(layers=2, hidden=256, intermediate=512, heads=4, kv_heads=2, head_dim=64, vocab=320, eps=1e-5,
           rope_theta=500000.0)


def _build_llama_stack(w, cfg, comm, engine, max_T):
    Hq, Hkv, D = cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
    cos, sin = oracle.rope_tables(max_T, D, cfg["rope_theta"], w["embed"].dtype)
    cos, sin = cos.cuda(), sin.cuda()
    embed = ext.muillm_embedding_module_init(engine, w["embed"].cuda())
    keep, decoders = [], []
    stack_rotary = ext.muillm_rotary_embedding_module_init(engine, 0, cos, sin)
    for l in range(cfg["layers"]):
        qkv_lin = ext.muillm_parallel_linear_module_init(engine, comm, w["qkv"][l].cuda(),
                                                         norm_weights=w["ln1"][l].cuda(), epsilon=cfg["eps"],
                                                         sharding_dim=0)
        slices = [(0, Hq * D), (Hq * D, (Hq + Hkv) * D), ((Hq + Hkv) * D, (Hq + 2 * Hkv) * D)]
        multilinear = ext.muillm_parallel_multilinear_module_init(engine, comm, qkv_lin, slices, 0)
        rotary = ext.muillm_rotary_embedding_module_init(engine, l, cos, sin)
        o_proj = ext.muillm_parallel_linear_module_init(engine, comm, w["o"][l].cuda(), sharding_dim=1)
        attention = ext.muillm_parallel_attention_module_init(engine, comm, rotary, o_proj, Hq, Hkv, D)
        mlp = ext.muillm_parallel_gateupdownmlp_module_init(engine, comm, ext.GATEUPSILU_FUSED, w["ln2"][l].cuda(),
                                                            w["gate"][l].cuda(), w["up"][l].cuda(),
                                                            w["down"][l].cuda(), cfg["eps"])
        decoders.append(ext.muillm_parallel_decoder_module_init(engine, comm, multilinear, attention, mlp))
        keep += [qkv_lin, multilinear, rotary, o_proj, attention, mlp]
    stack = ext.muillm_parallel_decoder_stack_init(engine, comm, embed, stack_rotary, decoders)
    return stack, keep + decoders + [embed, stack_rotary]


CFG128 = dict(layers=2, hidden=512, intermediate=768, heads=8, kv_heads=2, head_dim=128, vocab=320, eps=1e-5,
              rope_theta=500000.0)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("cache_kind,fused,cfg", [("static", "1", CFG), ("static", "0", CFG), ("dynamic", "1", CFG),
                                                  ("static", "1", CFG128), ("static", "0", CFG128)])
def test_decoder_stack_through_module_handles(dtype, cache_kind, fused, cfg, monkeypatch):
    """fused = 1: a decode step on a static cache is one call into the C decode stack; 0: one call per module."""
    monkeypatch.setattr(ext, "FUSED_DECODER_STACK", fused == "1")
    max_T, B = 48, 2
    w = oracle.make_llama_weights(cfg, dtype, seed=3, std=0.06)
    engine = ext.muillm_engine_init()
    comm = ext.muillm_comm_init(engine, 1, 1, 0, 0)
    stack, keep = _build_llama_stack(w, cfg, comm, engine, max_T)
    L, Hkv, D = cfg["layers"], cfg["kv_heads"], cfg["head_dim"]
    if cache_kind == "static":
        kc = [torch.zeros(B, Hkv, max_T, D, dtype=dtype, device="cuda") for _ in range(L)]
        vc = [torch.zeros(B, Hkv, max_T, D, dtype=dtype, device="cuda") for _ in range(L)]
        cache = ext.muillm_static_kvcache_module_init(engine, kc, vc, 0)
    else:
        kc = [torch.zeros(B, Hkv, 0, D, dtype=dtype, device="cuda") for _ in range(L)]
        vc = [torch.zeros(B, Hkv, 0, D, dtype=dtype, device="cuda") for _ in range(L)]
        cache = ext.muillm_dynamic_kvcache_module_init(engine, kc, vc, 0)
    orc = oracle.LlamaOracle(w, cfg, max_T=max_T, batch=B)
    g = torch.Generator().manual_seed(11)
    tokens = torch.randint(0, cfg["vocab"], (B, 20), generator=g)
    lm_head, norm = w["lm_head"].cuda(), w["norm"].cuda()
    for t in range(tokens.shape[1]):
        ids = tokens[:, t:t + 1].contiguous()
        want = orc.forward(ids)
        pos = torch.full((B, 1), t, dtype=torch.int64, device="cuda")
        cpos = torch.tensor([t], dtype=torch.int64, device="cuda")
        h = ext.muillm_parallel_decoder_stack_forward(stack, cache, ids.cuda(), None, None, pos, cpos)
        assert h.shape == (B, 1, cfg["hidden"])
        logits = ext.muillm_linear_forward(engine, h, lm_head, norm_weights=norm, epsilon=cfg["eps"])
        tol = dict(rtol=2e-2, atol=2e-2) if dtype == torch.float16 else dict(rtol=5e-2, atol=1e-1)
        torch.testing.assert_close(logits.float().cpu().reshape(B, -1), want, **tol)
    assert ext.muillm_kvcache_module_get_set_seen_tokens(cache, 0) == tokens.shape[1]
    assert (stack._fused is not None) == (fused == "1" and cache_kind == "static")
    if cache_kind == "static":
        k_back, v_back = ext.muillm_static_kvcache_module_sync_back(cache)
        torch.testing.assert_close(k_back[0][:, :, :20].float().cpu(), orc.k_cache[0][:, :, :20].float(), rtol=1e-2,
                                   atol=1e-2)
    else:
        k_back, v_back = ext.muillm_dynamic_kvcache_module_sync_back(cache)
        assert k_back[1].shape[2] == 20 and v_back[1].shape[2] == 20
        torch.testing.assert_close(v_back[1].float().cpu(), orc.v_cache[1][:, :, :20].float(), rtol=1e-2, atol=1e-2)
    ext.muillm_parallel_decoder_stack_deinit(stack)
    for m in keep:
        m.release()


def test_prefill_rows_take_the_gemm_path_and_agree_with_decode_rows():
    """More than 8 rows go through the RMSNorm kernel + torch GEMM (as the reference does); same result as row by row."""
    dtype = torch.float16
    g = torch.Generator().manual_seed(5)
    x = torch.randn(1, 12, 256, generator=g).to(dtype).cuda()
    W = (torch.randn(384, 256, generator=g) * 0.05).to(dtype).cuda()
    nw = (1 + 0.01 * torch.randn(256, generator=g)).to(dtype).cuda()
    lin = ext.muillm_linear_module_init(None, W, norm_weights=nw, epsilon=1e-5)
    full = ext.muillm_linear_module_forward(lin, x)
    rows = torch.cat([ext.muillm_linear_module_forward(lin, x[:, i:i + 1].contiguous()) for i in range(12)], dim=1)
    torch.testing.assert_close(full.float(), rows.float(), rtol=1e-2, atol=2e-3)
    ext.muillm_linear_module_deinit(lin)
    assert lin.weights is None


@pytest.mark.parametrize("use_rope,use_qk_norm,use_temp", [(True, True, False), (False, False, True),
                                                          (True, False, False)])
def test_llama4_attention_module_with_hybrid_chunked_cache(use_rope, use_qk_norm, use_temp):
    dtype = torch.bfloat16
    B, Hq, Hk, D, H, W = 1, 8, 2, 128, 512, 6
    g = torch.Generator().manual_seed(17)
    Wo = (torch.randn(H, Hq * D, generator=g) * 0.03).to(dtype)
    o_proj = ext.muillm_parallel_linear_module_init(None, ext.muillm_comm_init(None, 1, 1, 0, 0), Wo.cuda(),
                                                    sharding_dim=1)
    layer = 1  # layer 1 of 2 is the sliding one; layer 0 advances the token count
    att = ext.muillm_parallel_llama4_attention_module_init(None, None, o_proj, Hq, Hk, D, use_rope, use_qk_norm, 1e-5,
                                                           use_temp, 0.1, 4.0, layer)
    kc = [torch.zeros(B, Hk, 16, D, dtype=dtype, device="cuda"), torch.zeros(B, Hk, W, D, dtype=dtype, device="cuda")]
    vc = [torch.zeros_like(kc[0]), torch.zeros_like(kc[1])]
    cache = ext.muillm_hybrid_chunked_kvcache_module_init(None, kc, vc, [False, True], W, 0)
    ok, ov = torch.zeros(B, Hk, W, D, dtype=dtype), torch.zeros(B, Hk, W, D, dtype=dtype)
    seen = 0
    for step in range(10):
        qkv = torch.randn(B, 1, (Hq + 2 * Hk) * D, generator=g).to(dtype)
        res = torch.randn(B, 1, H, generator=g).to(dtype)
        ang = torch.rand(B, 1, D // 2, generator=g) * 6.28
        pe = torch.stack((ang.cos(), ang.sin()), dim=-1).contiguous()
        cpos = torch.tensor([step], dtype=torch.int64)
        # layer 0 (static) sees the token first and moves the count
        dummy = torch.zeros(B, Hk, 1, D, dtype=dtype, device="cuda")
        ext.muillm_hybrid_chunked_kvcache_module_update(cache, dummy, dummy, cpos.cuda(), 0)
        seen += 1
        q = qkv[..., :Hq * D]
        k = qkv[..., Hq * D:(Hq + Hk) * D]
        v = qkv[..., (Hq + Hk) * D:]
        # oracle
        q4, k4, v4 = (q.reshape(B, Hq, 1, D), k.reshape(B, Hk, 1, D), v.reshape(B, Hk, 1, D))
        if use_rope:
            q4, k4 = oracle.complex_rope(q4, pe), oracle.complex_rope(k4, pe)
        if use_qk_norm:
            q4, k4 = oracle.l2norm(q4, 1e-5), oracle.l2norm(k4, 1e-5)
        if use_temp:
            q4 = oracle.temperature_tuning(q4, cpos, 0.1, 4.0)
        k_st, v_st, ok, ov = oracle.sliding_cache_update(k4, v4, ok, ov, cpos, seen)
        attn = oracle.decode_attention(q4, k_st, v_st).reshape(B, 1, Hq * D)
        want = oracle.linear(attn, Wo, residual=res)
        qkv_d = qkv.cuda()
        got = ext.muillm_parallel_llama4_attention_module_rope_forward(
            att, cache, qkv_d[..., :Hq * D], qkv_d[..., Hq * D:(Hq + Hk) * D], qkv_d[..., (Hq + Hk) * D:], None,
            res.cuda(), pe.cuda(), cpos.cuda())
        torch.testing.assert_close(got.float().cpu(), want.float(), rtol=2e-2, atol=2e-2)
    k_back, _ = ext.muillm_hybrid_chunked_kvcache_module_sync_back(cache)
    assert torch.equal(k_back[1].cpu(), ok)


def test_moe_module_routes_like_the_oracle():
    dtype = torch.bfloat16
    H, I, shared, routed, top_k = 512, 256, 1, 8, 1
    E = shared + routed
    g = torch.Generator().manual_seed(23)
    x = torch.randn(1, 1, H, generator=g).to(dtype)
    nw = (1 + 0.01 * torch.randn(H, generator=g)).to(dtype)
    Wr = (torch.randn(routed, H, generator=g) * 0.2).to(dtype)
    G = (torch.randn(E * I, H, generator=g) * 0.03).to(dtype)
    U = (torch.randn(E * I, H, generator=g) * 0.03).to(dtype)
    Dw = (torch.randn(E * H, I, generator=g) * 0.03).to(dtype)
    router = ext.muillm_linear_module_init(None, Wr.cuda(), norm_weights=nw.cuda(), epsilon=1e-5)
    moe = ext.muillm_parallel_gateupdownmlpmoe_module_init(None, ext.muillm_comm_init(None, 1, 1, 0, 0), router,
                                                           shared, routed, top_k, nw.cuda(), G.cuda(), U.cuda(),
                                                           Dw.cuda(), 1e-5)
    logits = oracle.linear(x, Wr, norm_weights=nw, eps=1e-5)
    scores, idx = oracle.topk_sigmoid(logits, top_k)
    want = oracle.moe_mlp(x, G, U, Dw, shared, E, scores, idx, norm_weights=nw, eps=1e-5, residual=x)
    xc = x.cuda()
    got = ext.muillm_parallel_gateupdownmlpmoe_module_forward(moe, xc, residual=xc)
    torch.testing.assert_close(got.float().cpu(), want.float(), rtol=2e-2, atol=8e-3)


def test_packed_int8_gateup_of_the_reference_format():
    dtype = torch.float16
    I, H, shift = 256, 512, 7
    g = torch.Generator().manual_seed(29)
    G = (torch.randn(I, H, generator=g) * 0.05).to(dtype)
    U = (torch.randn(I, H, generator=g) * 0.05).to(dtype)
    x = torch.randn(1, H, generator=g).to(dtype)
    nw = (1 + 0.01 * torch.randn(H, generator=g)).to(dtype)
    gq, gs = oracle.rtn_group_quantize(G, group_shift=shift)
    uq, us = oracle.rtn_group_quantize(U, group_shift=shift)
    pack = torch.cat([gq[:, :, None], uq[:, :, None]], dim=2).contiguous()
    scales = torch.cat([gs[:, None, :], us[:, None, :]], dim=1).contiguous()
    want = oracle.gateup_silu(x, oracle.rtn_group_dequantize(gq, gs, shift), oracle.rtn_group_dequantize(uq, us, shift),
                              norm_weights=nw, eps=1e-5)
    got = ext.muillm_int8_gateupsilu_forward(nw.cuda(), 1e-5, pack.cuda(), scales.cuda(), shift, x.cuda())
    torch.testing.assert_close(got.float().cpu(), want.float(), rtol=1e-2, atol=2e-3)
    dg, du = ext.muillm_int8_gateupsilu_dequantize_forward(pack.cuda(), scales.cuda(), shift)
    torch.testing.assert_close(dg.float().cpu(), oracle.rtn_group_dequantize(gq, gs, shift).float(), rtol=0, atol=1e-3)
    torch.testing.assert_close(du.float().cpu(), oracle.rtn_group_dequantize(uq, us, shift).float(), rtol=0, atol=1e-3)


def test_synchronizer_and_embedding():
    emb = ext.muillm_embedding_module_init(None, torch.arange(40, dtype=torch.float16).reshape(10, 4).cuda())
    out = ext.muillm_embedding_module_forward(emb, torch.tensor([[3, 9]], device="cuda"))
    assert out.shape == (1, 2, 4) and out[0, 1].tolist() == [36.0, 37.0, 38.0, 39.0]
    sync = ext.muillm_sync_init()
    assert ext.muillm_item_bool(sync, torch.tensor(True, device="cuda")) is True
    assert math.isclose(ext.muillm_item_f32(sync, torch.tensor(1.5, device="cuda")), 1.5)
    assert ext.muillm_to_cpu(sync, torch.ones(2, device="cuda")).device.type == "cpu"
