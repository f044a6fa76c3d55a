"""GPU parity of RMSNorm, RoPE + static-cache write-out and flash decoding against the CPU oracle."""

import pytest
import torch

from muillm_b200 import capi, ops
from oracle import decode_oracle as oracle

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-2, 1e-3
DTYPES = [torch.float16, torch.bfloat16]


def _gen(seed):
    return torch.Generator().manual_seed(seed)


def _close(got, want, rtol=RTOL, atol=ATOL):
    got, want = got.float().cpu(), want.float()
    assert got.shape == want.shape
    assert torch.isfinite(got).all()
    torch.testing.assert_close(got, want, rtol=rtol, atol=atol)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,K", [(1, 4096), (4, 4096), (3, 100), (2, 8192), (0, 64)])
@pytest.mark.parametrize("weighted", [True, False])
def test_rmsnorm(dtype, rows, K, weighted):
    g = _gen(K + rows)
    x = torch.randn(rows, K, generator=g).to(dtype)
    w = (1 + 0.01 * torch.randn(K, generator=g)).to(dtype) if weighted else None
    want = oracle.rmsnorm(x, w, 1e-5)
    got = ops.muillm_rmsnorm_forward(w.cuda() if weighted else None, x.cuda(), 1e-5)
    _close(got, want)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("B,T,Hq,Hkv,D", [(1, 1, 32, 8, 128), (4, 1, 8, 2, 64), (2, 5, 4, 4, 128), (1, 16, 32, 8, 128)])
def test_rope_static_cache(dtype, B, T, Hq, Hkv, D):
    """q,k,v are strided views of a packed QKV output, like the reference's caller produces."""
    max_T, prev = 64, 7
    g = _gen(T + B)
    qkv = torch.randn(B, T, (Hq + 2 * Hkv) * D, generator=g).to(dtype)
    q = qkv[..., : Hq * D].view(B, T, Hq, D).transpose(1, 2)
    k = qkv[..., Hq * D: (Hq + Hkv) * D].view(B, T, Hkv, D).transpose(1, 2)
    v = qkv[..., (Hq + Hkv) * D:].view(B, T, Hkv, D).transpose(1, 2)
    cos, sin = oracle.rope_tables(max_T, D, 500000.0, dtype)
    position_ids = (torch.arange(prev, prev + T)[None, :] + torch.arange(B)[:, None]).to(torch.int64)
    position_ids = position_ids.clamp(max=max_T - 1)
    cache_position = torch.arange(prev, prev + T, dtype=torch.int64)
    kc = torch.randn(B, Hkv, max_T, D, generator=g).to(dtype)
    vc = torch.randn(B, Hkv, max_T, D, generator=g).to(dtype)
    kc_ref, vc_ref = kc.clone(), vc.clone()
    q_ref, ks_ref, vs_ref = oracle.rope_write_static_cache(q, k, v, cos, sin, position_ids, kc_ref, vc_ref,
                                                           cache_position, prev + T)
    qkv_c = qkv.cuda()
    qc = qkv_c[..., : Hq * D].view(B, T, Hq, D).transpose(1, 2)
    kcu = qkv_c[..., Hq * D: (Hq + Hkv) * D].view(B, T, Hkv, D).transpose(1, 2)
    vcu = qkv_c[..., (Hq + Hkv) * D:].view(B, T, Hkv, D).transpose(1, 2)
    kc_g, vc_g = kc.cuda(), vc.cuda()
    q_out, ks, vs = ops.muillm_rope_forward_static_cache(position_ids.cuda(), cos.cuda(), sin.cuda(), qc, kcu, vcu,
                                                         kc_g, vc_g, cache_position.cuda(), prev + T)
    _close(q_out, q_ref)
    _close(ks, ks_ref)
    assert ks.shape == (B, Hkv, prev + T, D)
    # v rows are copied bit-exactly; untouched cache rows stay bit-identical
    assert torch.equal(vs.cpu(), vs_ref)
    assert torch.equal(vc_g.cpu(), vc_ref)
    assert torch.equal(kc_g.cpu()[:, :, :prev], kc[:, :, :prev])
    assert torch.equal(kc_g.cpu()[:, :, prev + T:], kc[:, :, prev + T:])

    # no-cache variant
    q2, k2 = ops.muillm_rope_forward_no_cache(position_ids.cuda(), cos.cuda(), sin.cuda(), qc, kcu)
    _close(q2, q_ref)
    _close(k2, oracle.rope_apply(k, cos, sin, position_ids))

    # plain scatter (no rotation)
    kc2, vc2 = kc.cuda(), vc.cuda()
    ops.muillm_static_kvcache_update(kcu, vcu, kc2, vc2, cache_position.cuda(), prev + T)
    want_k = kc.clone()
    want_k[:, :, cache_position] = k
    assert torch.equal(kc2.cpu(), want_k)
    assert torch.equal(vc2.cpu(), vc_ref)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("B,Hq,Hkv,D,S,max_T", [
    (1, 32, 8, 128, 17, 4096),     # short sequence inside a long static cache (strided K/V)
    (1, 32, 8, 128, 272, 4096),
    (1, 32, 8, 128, 4096, 4096),   # full cache
    (4, 8, 8, 64, 33, 33),         # MHA, head dim 64, contiguous
    (2, 8, 1, 128, 1000, 1024),    # one KV head, 8 query heads per group
    (3, 10, 2, 128, 1, 16),        # a single token, group of 5
    (1, 4, 2, 128, 0, 16),         # empty sequence -> zeros
])
def test_flash_decode(dtype, B, Hq, Hkv, D, S, max_T):
    g = _gen(S + B)
    q = torch.randn(B, Hq, 1, D, generator=g).to(dtype)
    kc = torch.randn(B, Hkv, max_T, D, generator=g).to(dtype)
    vc = torch.randn(B, Hkv, max_T, D, generator=g).to(dtype)
    want = oracle.decode_attention(q, kc[:, :, :S], vc[:, :, :S])
    kg, vg = kc.cuda(), vc.cuda()
    got = ops.muillm_causal_transformer_decoding_no_mask(q.cuda(), kg.narrow(2, 0, S), vg.narrow(2, 0, S))
    assert got.shape == (B, 1, Hq * D)
    _close(got, want)
    # twice in a row: the arrival counters in the workspace must have been left at zero
    got2 = ops.muillm_causal_transformer_decoding_no_mask(q.cuda(), kg.narrow(2, 0, S), vg.narrow(2, 0, S))
    _close(got2, want)
    if S > 0:
        # device-resident sequence length (graph replay form): attend S tokens of a max_T launch
        seq = torch.tensor([S], dtype=torch.int32, device="cuda")
        got3 = ops._flash_decode(q.cuda(), kg, vg, None, seq_len_dev=seq)
        _close(got3, want)


@pytest.mark.parametrize("dtype", DTYPES)
def test_flash_decode_masked_ragged_batch(dtype):
    """Left-padded ragged batch: additive mask, 0 = keep, finfo.min = drop."""
    B, Hq, Hkv, D, S = 4, 32, 8, 128, 96
    g = _gen(21)
    q = torch.randn(B, Hq, 1, D, generator=g).to(dtype)
    k = torch.randn(B, Hkv, S, D, generator=g).to(dtype)
    v = torch.randn(B, Hkv, S, D, generator=g).to(dtype)
    lengths = [96, 5, 40, 1]
    mask = torch.zeros(B, 1, 1, S, dtype=dtype)
    for b, n in enumerate(lengths):
        mask[b, ..., : S - n] = torch.finfo(dtype).min
    want = oracle.decode_attention(q, k, v, mask=mask)
    got = ops.muillm_causal_transformer_decoding_masked(q.cuda(), k.cuda(), v.cuda(), mask.cuda())
    _close(got, want)
    # the masked result equals the unmasked result on the unpadded suffix
    for b, n in enumerate(lengths):
        alone = ops.muillm_causal_transformer_decoding_no_mask(
            q[b:b + 1].cuda(), k[b:b + 1, :, S - n:].cuda(), v[b:b + 1, :, S - n:].cuda())
        _close(alone, got[b:b + 1].cpu(), rtol=1e-3, atol=1e-3)


def test_flash_decode_softmax_shift_invariance():
    """Size-independent property at full cache length: duplicating the KV sequence leaves the output unchanged."""
    dtype = torch.float16
    B, Hq, Hkv, D, S = 1, 32, 8, 128, 2048
    g = _gen(9)
    q = torch.randn(B, Hq, 1, D, generator=g).to(dtype).cuda()
    k = torch.randn(B, Hkv, S, D, generator=g).to(dtype).cuda()
    v = torch.randn(B, Hkv, S, D, generator=g).to(dtype).cuda()
    a = ops.muillm_causal_transformer_decoding_no_mask(q, k, v)
    b = ops.muillm_causal_transformer_decoding_no_mask(q, torch.cat([k, k], 2), torch.cat([v, v], 2))
    _close(a, b.cpu(), rtol=2e-3, atol=2e-3)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("B,Hq,Hkv,S", [(1, 32, 8, 1), (1, 32, 8, 2), (1, 32, 8, 17), (1, 32, 8, 280), (1, 32, 8, 385), (1, 32, 8, 386),
                                        (1, 32, 8, 513),
                                        (2, 8, 1, 2000), (3, 4, 4, 65), (1, 8, 8, 4096), (2, 8, 1, 300), (2, 4, 2, 384),
                                        (1, 16, 2, 97)])
@pytest.mark.parametrize("variant", [0, capi.MUI_FLAG_SHORT_CONTEXT, capi.MUI_FLAG_SHORT_CONTEXT | capi.MUI_FLAG_PDL,
                                     capi.MUI_FLAG_SPLIT_CONTEXT, capi.MUI_FLAG_SPLIT_CONTEXT | capi.MUI_FLAG_PDL])
def test_fused_rope_cache_write_attention(dtype, B, Hq, Hkv, S, variant):
    """One launch = RoPE(q, k_new) + cache write + attention over S tokens (the new one last): the cluster kernel, the
    one-CTA-per-head tensor-core kernel that stages the history in shared memory (at most 384 tokens; a longer
    sequence must be refused through the device status word, not computed wrongly), and the same kernel with the
    tokens split over several CTAs per KV head (sized for the whole 4096-row cache: 16 CTAs, of which a short sequence
    uses few) whose last arriver merges the parts."""
    D, max_T = 128, 4096
    g = _gen(S + B + Hq)
    qkv = torch.randn(B, (Hq + 2 * Hkv) * D, generator=g).to(dtype)
    kc = torch.randn(B, Hkv, max_T, D, generator=g).to(dtype)
    vc = torch.randn(B, Hkv, max_T, D, generator=g).to(dtype)
    cos, sin = oracle.rope_tables(max_T, D, 500000.0, dtype)
    pos = S - 1
    position_ids = torch.full((B, 1), pos, dtype=torch.int64)
    if B > 1:
        position_ids[1, 0] = max(0, pos - 3)  # per-sequence RoPE positions may differ from the cache row
    cache_position = torch.tensor([pos], dtype=torch.int64)
    q = qkv[:, : Hq * D].view(B, Hq, 1, D)
    k = qkv[:, Hq * D: (Hq + Hkv) * D].view(B, Hkv, 1, D)
    v = qkv[:, (Hq + Hkv) * D:].view(B, Hkv, 1, D)
    kc_ref, vc_ref = kc.clone(), vc.clone()
    q_rot, ks, vs = oracle.rope_write_static_cache(q, k, v, cos, sin, position_ids, kc_ref, vc_ref, cache_position, S)
    want = oracle.decode_attention(q_rot, ks, vs)
    kc_g, vc_g = kc.cuda(), vc.cuda()
    ws = None
    if variant & capi.MUI_FLAG_SPLIT_CONTEXT:
        ws = torch.zeros(capi.lib().mui_flash_decode_workspace_bytes(B, Hq, Hkv, D, max_T), dtype=torch.uint8,
                         device="cuda")
    got = ops.rope_flash_decode(qkv.cuda(), cos.cuda(), sin.cuda(), position_ids.view(-1).cuda(), cache_position.cuda(),
                                torch.tensor([S], dtype=torch.int32, device="cuda"), kc_g, vc_g, Hq, flags=variant,
                                workspace=ws)
    if (variant & capi.MUI_FLAG_SHORT_CONTEXT) and S > 384:
        torch.cuda.synchronize()
        status = capi.device_status(clear=True)
        assert status >> 24 == 5, f"expected the bad-length status, got {status:#x}"
        assert torch.equal(kc_g.cpu(), kc), "a refused launch must not touch the cache"
        return
    _close(got, want)
    # the cache got exactly the rows the stand-alone RoPE kernel writes, and nothing else moved
    _close(kc_g[:, :, pos], kc_ref[:, :, pos])
    assert torch.equal(vc_g.cpu(), vc_ref)
    keep = torch.ones(max_T, dtype=torch.bool)
    keep[pos] = False
    assert torch.equal(kc_g.cpu()[:, :, keep], kc[:, :, keep])
    if ws is not None:
        assert int(ws[:4096].view(torch.int32).abs().sum()) == 0, "the arrival counters must be back at zero"
