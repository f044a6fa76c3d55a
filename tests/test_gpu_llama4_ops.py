"""GPU parity of the Llama-4 attention prologue (interleaved rope, QK L2 norm, temperature scale), the sliding-window
cache, the dimension sum and the token bookkeeping against the CPU oracle and the HF fixtures, through the C ABI."""
import os

import numpy as np
import pytest
import torch

from muillm_b200 import capi, ops
from oracle import decode_oracle as oracle

pytestmark = pytest.mark.gpu

DTYPES = [torch.float16, torch.bfloat16]
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _gen(seed):
    return torch.Generator().manual_seed(seed)


def _packed_qk(B, T, Hq, Hk, D, dtype, g):
    """q and k as strided views of one packed [B, T, (Hq + 2 Hk) D] projection output, like the reference's QKV."""
    qkv = torch.randn(B, T, (Hq + 2 * Hk) * D, generator=g).to(dtype)
    q = qkv[..., :Hq * D].view(B, T, Hq, D).transpose(1, 2)
    k = qkv[..., Hq * D:(Hq + Hk) * D].view(B, T, Hk, D).transpose(1, 2)
    return qkv, q, k


def _views(qkv_dev, B, T, Hq, Hk, D):
    q = qkv_dev[..., :Hq * D].view(B, T, Hq, D).transpose(1, 2)
    k = qkv_dev[..., Hq * D:(Hq + Hk) * D].view(B, T, Hk, D).transpose(1, 2)
    return q, k


def _pos_embeds(B, T, D, g):
    ang = torch.rand(B, T, D // 2, generator=g) * 6.28
    return torch.stack((ang.cos(), ang.sin()), dim=-1).contiguous()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("B,T,Hq,Hk,D", [(1, 1, 40, 8, 128), (2, 3, 5, 2, 128), (1, 7, 3, 1, 64), (2, 1, 4, 4, 256),
                                        (1, 2, 2, 1, 6)])
def test_complex_rope_bit_exact_vs_oracle(dtype, B, T, Hq, Hk, D):
    g = _gen(B * 100 + T * 10 + D)
    qkv, q, k = _packed_qk(B, T, Hq, Hk, D, dtype, g)
    pe = _pos_embeds(B, T, D, g)
    qd, kd = _views(qkv.cuda(), B, T, Hq, Hk, D)
    got_q, got_k = ops.muillm_complex_rope_forward_no_cache(qd, kd, pe.cuda())
    # fp32 complex product of 16-bit inputs rounded once: the device uses the same two products and one add,
    # fused multiply-add contraction can move the last fp32 bit, which survives rounding only at ties
    for got, x in ((got_q, q), (got_k, k)):
        want = oracle.complex_rope(x, pe)
        assert got.is_contiguous() and got.shape == want.shape
        torch.testing.assert_close(got.float().cpu(), want.float(), rtol=1e-2, atol=1e-3)
        ulp_off = (got.cpu().view(torch.int16).int() - want.view(torch.int16).int()).abs().max().item()
        assert ulp_off <= 1


@pytest.mark.parametrize("tag,dtype", [("f16", torch.float16), ("bf16", torch.bfloat16)])
def test_prologue_against_hf_fixture(tag, dtype):
    l4 = np.load(os.path.join(GOLD, "hf_llama4_ops.npz"))
    q = torch.from_numpy(l4["l4_q"]).to(dtype).cuda()
    k = torch.from_numpy(l4["l4_k"]).to(dtype).cuda()
    pe = torch.from_numpy(l4["l4_pos_embeds"]).cuda()
    rq, rk = ops.muillm_complex_rope_forward_no_cache(q, k, pe)
    torch.testing.assert_close(rq.float().cpu(), torch.from_numpy(l4[f"l4_rope_{tag}_q"]), rtol=1e-2, atol=1e-3)
    torch.testing.assert_close(rk.float().cpu(), torch.from_numpy(l4[f"l4_rope_{tag}_k"]), rtol=1e-2, atol=1e-3)
    nq, nk = ops.muillm_qkl2norm_forward(rq, rk, 1e-5)
    torch.testing.assert_close(nq.float().cpu(), torch.from_numpy(l4[f"l4_norm_{tag}_q"]), rtol=1e-2, atol=1e-3)
    torch.testing.assert_close(nk.float().cpu(), torch.from_numpy(l4[f"l4_norm_{tag}_k"]), rtol=1e-2, atol=1e-3)
    # fused launch == the separate launches, bit for bit
    fq, fk = ops.llama4_qk_prologue(q, k, position_embeds=pe, qk_norm_eps=1e-5)
    assert torch.equal(fq, nq) and torch.equal(fk, nk)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows_q,rows_k,D", [(40, 8, 128), (1, 1, 64), (33, 0, 256), (7, 3, 2)])
def test_qkl2norm(dtype, rows_q, rows_k, D):
    g = _gen(rows_q + D)
    q = (torch.randn(rows_q, D, generator=g) * 3).to(dtype)
    k = (torch.randn(max(rows_k, 1), D, generator=g) * 0.1).to(dtype)[:rows_k]
    got_q, got_k = ops.muillm_qkl2norm_forward(q.cuda(), k.cuda(), 1e-6)
    torch.testing.assert_close(got_q.float().cpu(), oracle.l2norm(q, 1e-6).float(), rtol=1e-2, atol=1e-3)
    torch.testing.assert_close(got_k.float().cpu(), oracle.l2norm(k, 1e-6).float(), rtol=1e-2, atol=1e-3)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("K", [128, 5120, 1000, 7])
def test_l2norm_rows_of_any_width(dtype, K):
    x = torch.randn(3, 2, K, generator=_gen(K)).to(dtype)
    got = ops.muillm_l2norm_forward(x.cuda(), 1e-5)
    torch.testing.assert_close(got.float().cpu(), oracle.l2norm(x, 1e-5).float(), rtol=1e-2, atol=1e-3)


@pytest.mark.parametrize("dtype", DTYPES)
def test_temperature_tuning_and_full_prologue(dtype):
    g = _gen(9)
    B, T, Hq, Hk, D = 1, 3, 10, 2, 128
    qkv, q, k = _packed_qk(B, T, Hq, Hk, D, dtype, g)
    pos = torch.tensor([8190, 8191, 40000])
    qd, kd = _views(qkv.cuda(), B, T, Hq, Hk, D)
    got = ops.muillm_apply_temperature_tuning(qd, pos.cuda(), 0.1, 8192.0)
    want = oracle.temperature_tuning(q, pos, 0.1, 8192.0)
    torch.testing.assert_close(got.float().cpu(), want.float(), rtol=1e-2, atol=1e-3)
    assert (got[:, :, 0].float().cpu() == q[:, :, 0].float()).all(), "scale is exactly 1 below the first floor step"
    # no-rope layer: norm + temperature in one launch equals the two calls
    nq, nk = ops.muillm_qkl2norm_forward(qd.contiguous(), kd.contiguous(), 1e-5)
    tq = ops.muillm_apply_temperature_tuning(nq, pos.cuda(), 0.1, 8192.0)
    fq, fk = ops.llama4_qk_prologue(qd, kd, qk_norm_eps=1e-5, cache_position=pos.cuda(), attn_scale=0.1,
                                    floor_scale=8192.0)
    assert torch.equal(fq, tq) and torch.equal(fk, nk)


def test_temperature_fixture_bf16():
    l4 = np.load(os.path.join(GOLD, "hf_llama4_ops.npz"))
    q = torch.from_numpy(l4["l4_q"]).to(torch.bfloat16).cuda()
    got = ops.muillm_apply_temperature_tuning(q, torch.from_numpy(l4["l4_temp_pos"]).cuda(), 0.1, 8192.0)
    torch.testing.assert_close(got.float().cpu(), torch.from_numpy(l4["l4_temp_bf16_q"]), rtol=1e-2, atol=1e-3)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("W,prefill,steps,chunk", [(6, 4, 8, 1), (8, 8, 5, 1), (8, 13, 4, 1), (16, 3, 6, 4),
                                                   (5, 2, 3, 7)])
def test_sliding_cache_sequence_bit_exact(dtype, W, prefill, steps, chunk):
    """First fill, in-place scatter until the window is full, then shifts; also chunks longer than the window."""
    g = _gen(W * 31 + prefill)
    B, Hk, D = 2, 3, 16
    total = prefill + steps * chunk
    ks = torch.randn(B, Hk, total, D, generator=g).to(dtype)
    vs = torch.randn(B, Hk, total, D, generator=g).to(dtype)
    kc, vc = torch.zeros(B, Hk, W, D, dtype=dtype), torch.zeros(B, Hk, W, D, dtype=dtype)
    kcd, vcd = kc.cuda(), vc.cuda()
    ksd, vsd = ks.cuda(), vs.cuda()
    seen, start = 0, 0
    for n in [prefill] + [chunk] * steps:
        pos = torch.arange(start, start + n)
        seen += n
        sl = slice(start, start + n)
        fits = seen <= W or seen == n
        want_k, want_v, kc, vc = oracle.sliding_cache_update(ks[:, :, sl], vs[:, :, sl], kc, vc,
                                                             pos if fits else None, seen)
        got_k, got_v = ops.muillm_sliding_kvcache_update(ksd[:, :, sl], vsd[:, :, sl], kcd, vcd,
                                                         pos.clamp(max=W - 1).cuda(), seen)
        assert torch.equal(got_k.cpu(), want_k) and torch.equal(got_v.cpu(), want_v), (seen, n)
        if seen > W and seen != n:
            kcd, vcd = got_k, got_v  # the caller keeps the fresh buffers, as the reference's hybrid cache does
        assert torch.equal(kcd.cpu(), kc) and torch.equal(vcd.cpu(), vc)
        start += n


def test_sliding_cache_matches_hf_layer_fixture():
    l4 = np.load(os.path.join(GOLD, "hf_llama4_ops.npz"))
    ks = torch.from_numpy(l4["l4_slide_k"]).half().cuda()
    vs = torch.from_numpy(l4["l4_slide_v"]).half().cuda()
    W = 6
    kc = torch.zeros(1, ks.shape[1], W, ks.shape[3], dtype=torch.float16, device="cuda")
    vc = torch.zeros_like(kc)
    ops.muillm_sliding_kvcache_update(ks[:, :, :4], vs[:, :, :4], kc, vc, torch.arange(4).cuda(), 4)
    for step in range(4, 12):
        k_st, v_st = ops.muillm_sliding_kvcache_update(ks[:, :, step:step + 1], vs[:, :, step:step + 1], kc, vc,
                                                       torch.tensor([min(step, W - 1)]).cuda(), step + 1)
        if step + 1 > W:
            kc, vc = k_st, v_st
        assert torch.equal(k_st.float().cpu(), torch.from_numpy(l4[f"l4_slide_states_k_{step}"]))
        assert torch.equal(v_st.float().cpu(), torch.from_numpy(l4[f"l4_slide_states_v_{step}"]))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape,dim,keep", [((1, 1, 2, 5120), 2, False), ((3, 4, 7), 1, True), ((2, 9), -1, False),
                                            ((5, 1, 33), 0, False), ((2, 3, 4, 5), -2, True)])
def test_reduce_sum(dtype, shape, dim, keep):
    x = torch.randn(*shape, generator=_gen(sum(shape))).to(dtype)
    got = ops.muillm_reduce_sum_forward(x.cuda(), dim, keep)
    want = oracle.reduce_sum(x, dim, keep)
    assert got.shape == want.shape
    torch.testing.assert_close(got.float().cpu(), want.float(), rtol=1e-2, atol=1e-3)


@pytest.mark.parametrize("B,T", [(1, 16), (3, 300), (5, 0), (2, 1)])
@pytest.mark.parametrize("has_eos,has_max", [(True, True), (True, False), (False, True), (False, False)])
def test_add_tokens_check_finished_bit_exact(B, T, has_eos, has_max):
    g = _gen(B * 7 + T)
    ids = torch.randint(0, 1000, (B, T), generator=g)
    nxt = torch.randint(0, 6, (B,), generator=g).to(torch.int32)
    unf = torch.randint(0, 2, (B,), generator=g)
    eos = torch.tensor([2, 4, 1000])
    for max_len in (T + 1, T + 2, 10_000):
        want_ids, want_unf = oracle.add_tokens_check_finished(ids, nxt, unf, has_eos, 7, eos, has_max, max_len)
        got_ids, got_unf = ops.muillm_add_tokens_check_finished(ids.cuda(), nxt.cuda(), unf.cuda(), has_eos, 7,
                                                                eos.cuda(), has_max, max_len)
        assert torch.equal(got_ids.cpu(), want_ids)
        assert torch.equal(got_unf.cpu(), want_unf)


def test_argument_errors_are_reported():
    q = torch.zeros(1, 2, 1, 300, dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError, match="head dim"):
        ops.muillm_qkl2norm_forward(q, q, 1e-5)
    k = torch.zeros(1, 1, 1, 8, dtype=torch.float16, device="cuda")
    cache = torch.zeros(1, 1, 4, 8, dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError, match="seen_tokens"):
        ops.muillm_sliding_kvcache_update(k, k, cache, cache.clone(), torch.zeros(1, dtype=torch.int64).cuda(), 0)
    assert capi.device_status() == 0
