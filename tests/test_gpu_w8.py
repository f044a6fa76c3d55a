"""GPU parity of the weight-only 8-bit kernels (BASELINE config 2 and the reference's group/min format) against the
CPU oracle: quantised weights and scales are produced by the oracle quantisers (bit-exact to the reference's
RTNQuantizer, see test_oracle_golden.py) on the host and fed unchanged to the kernels."""
import pytest
import torch

from muillm_b200 import capi, ops
from oracle import decode_oracle as oracle

pytestmark = pytest.mark.gpu

DTYPES = [torch.float16, torch.bfloat16]
PATHS = {"auto": 0, "generic": capi.MUI_FLAG_FORCE_GENERIC}


def _gen(seed):
    return torch.Generator().manual_seed(seed)


def _close(got, want, rtol=1e-2, atol=1e-3):
    got, want = got.float().cpu(), want.float()
    assert got.shape == want.shape and torch.isfinite(got).all()
    torch.testing.assert_close(got, want, rtol=rtol, atol=atol)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("path", list(PATHS))
@pytest.mark.parametrize("N,K,B", [(4096, 4096, 1), (515, 1024, 3), (64, 96, 2), (33, 40, 1), (1024, 14336, 8)])
def test_linear_symmetric_per_row(dtype, path, N, K, B):
    g = _gen(N + K + B)
    W = (torch.randn(N, K, generator=g) * 0.02).to(dtype)
    q, s = oracle.rtn_symrow_quantize(W)
    x = torch.randn(B, K, generator=g).to(dtype)
    nw = (1 + 0.01 * torch.randn(K, generator=g)).to(dtype)
    res = torch.randn(B, N, generator=g).to(dtype)
    want = oracle.linear(x, oracle.rtn_symrow_dequantize(q, s), norm_weights=nw, eps=1e-5, residual=res, out_dtype=dtype)
    got = ops.muillm_int8_linear_forward(x.cuda(), q.cuda(), s.cuda(), 0, norm_weights=nw.cuda(), epsilon=1e-5,
                                         residual=res.cuda(), flags=PATHS[path])
    _close(got, want)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("N,K,B,shift", [(512, 1024, 1, 7), (96, 256, 4, 5), (40, 64, 2, 3), (256, 4096, 1, 7)])
def test_linear_group_min_reference_format(dtype, N, K, B, shift):
    g = _gen(N + K + shift)
    W = (torch.randn(N, K, generator=g) * 0.02).to(dtype)
    q, sm = oracle.rtn_group_quantize(W, group_shift=shift)
    x = torch.randn(B, K, generator=g).to(dtype)
    ab = (torch.randn(N, generator=g) * 0.1).to(dtype)
    want = oracle.linear(x, oracle.rtn_group_dequantize(q, sm, group_shift=shift), add_bias=ab, out_dtype=dtype)
    got = ops.muillm_int8_linear_forward(x.cuda(), q.cuda(), sm.cuda(), shift, add_bias=ab.cuda())
    _close(got, want)
    # whole-matrix de-quantisation
    deq = ops.muillm_int8_dequantize_forward(q.cuda(), sm.cuda(), shift)
    _close(deq, oracle.rtn_group_dequantize(q, sm, group_shift=shift).to(dtype), rtol=0, atol=0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("path", list(PATHS))
@pytest.mark.parametrize("B", [1, 2, 4, 8])
def test_int8_mlp_llama3_8b_shape(dtype, path, B):
    """BASELINE config 2: hidden 4096, intermediate 14336, symmetric per-row int8 with 16-bit scales."""
    H, I = 4096, 14336
    g = _gen(B)
    mk = lambda *s: (torch.randn(*s, generator=g) * 0.02).to(dtype)
    (gq, gs), (uq, us), (dq, ds) = (oracle.rtn_symrow_quantize(mk(I, H)), oracle.rtn_symrow_quantize(mk(I, H)),
                                    oracle.rtn_symrow_quantize(mk(H, I)))
    x = torch.randn(B, H, generator=g).to(dtype)
    nw = (1 + 0.01 * torch.randn(H, generator=g)).to(dtype)
    want_t = oracle.gateup_silu(x, oracle.rtn_symrow_dequantize(gq, gs), oracle.rtn_symrow_dequantize(uq, us),
                                norm_weights=nw, eps=1e-5, out_dtype=dtype)
    xc = x.cuda()
    t = ops.int8_gateup_silu(xc, gq.cuda(), gs.cuda(), uq.cuda(), us.cuda(), norm_weights=nw.cuda(), epsilon=1e-5,
                             flags=PATHS[path])
    _close(t, want_t)
    want_y = oracle.linear(t.cpu(), oracle.rtn_symrow_dequantize(dq, ds), residual=x, out_dtype=dtype)
    y = ops.muillm_int8_linear_forward(t, dq.cuda(), ds.cuda(), 0, residual=xc, flags=PATHS[path])
    _close(y, want_y)


def test_quantised_weights_reach_the_kernel_bit_exact():
    """De-quantising on the GPU what the host quantiser produced returns exactly q * s (no re-quantisation)."""
    g = _gen(0)
    W = (torch.randn(64, 128, generator=g) * 0.02).to(torch.float16)
    q, s = oracle.rtn_symrow_quantize(W)
    deq = ops.muillm_int8_dequantize_forward(q.cuda(), s.cuda(), 0).cpu()
    assert torch.equal(deq, oracle.rtn_symrow_dequantize(q, s).to(torch.float16))


# ---------------------------------------------------------------------------------------------------------------
# the reference's per-group {scale, min} format on the bulk-copy pipeline (groups of >= 32, K % 32 == 0) and on the
# plain-load kernel, and its element-interleaved gate/up pack
# ---------------------------------------------------------------------------------------------------------------
from parity_utils import reference_gateup_pack as _group_pack  # noqa: E402  (the reference's own pack layout)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("path", list(PATHS))
@pytest.mark.parametrize("N,K,B,shift", [(4096, 4096, 1, 7), (515, 6144, 3, 7), (1024, 14336, 1, 7), (130, 1024, 8, 5),
                                         (256, 8192, 2, 9), (64, 4096, 4, 11),
                                         # batches whose whole-row staging leaves the pipeline no room: half batches
                                         (256, 14336, 4, 7), (144, 14336, 8, 7)])
def test_linear_group_min_both_kernels(dtype, path, N, K, B, shift):
    g = _gen(N + K + shift + B)
    W = (torch.randn(N, K, generator=g) * 0.02 + 0.003).to(dtype)
    q, sm = oracle.rtn_group_quantize(W, group_shift=shift)
    x = (torch.randn(B, K, generator=g) + 0.25).to(dtype)  # a non-zero mean exercises the min * sum(x) term
    nw = (1 + 0.01 * torch.randn(K, generator=g)).to(dtype)
    res = torch.randn(B, N, generator=g).to(dtype)
    want = oracle.linear(x, oracle.rtn_group_dequantize(q, sm, group_shift=shift), norm_weights=nw, eps=1e-5,
                         residual=res, out_dtype=dtype)
    got = ops.muillm_int8_linear_forward(x.cuda(), q.cuda(), sm.cuda(), shift, norm_weights=nw.cuda(), epsilon=1e-5,
                                         residual=res.cuda(), flags=PATHS[path])
    _close(got, want)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("I,H,B,shift", [(14336, 4096, 1, 7), (1000, 4096, 4, 7), (72, 3072, 2, 5), (520, 2048, 8, 6),
                                         (264, 8192, 8, 7)])
def test_gateup_group_min_split_and_packed(dtype, I, H, B, shift):
    g = _gen(I + H + B)
    mk = lambda *s: (torch.randn(*s, generator=g) * 0.02 + 0.002).to(dtype)
    gq, gsm = oracle.rtn_group_quantize(mk(I, H), group_shift=shift)
    uq, usm = oracle.rtn_group_quantize(mk(I, H), group_shift=shift)
    x = (torch.randn(B, H, generator=g) + 0.1).to(dtype)
    nw = (1 + 0.01 * torch.randn(H, generator=g)).to(dtype)
    want = oracle.gateup_silu(x, oracle.rtn_group_dequantize(gq, gsm, group_shift=shift),
                              oracle.rtn_group_dequantize(uq, usm, group_shift=shift), norm_weights=nw, eps=1e-5,
                              out_dtype=dtype)
    xc, nwc = x.cuda(), nw.cuda()
    split = ops.int8_gateup_silu(xc, gq.cuda(), gsm.cuda(), uq.cuda(), usm.cuda(), group_size_shift=shift,
                                 norm_weights=nwc, epsilon=1e-5)
    _close(split, want)
    generic = ops.int8_gateup_silu(xc, gq.cuda(), gsm.cuda(), uq.cuda(), usm.cuda(), group_size_shift=shift,
                                   norm_weights=nwc, epsilon=1e-5, flags=capi.MUI_FLAG_FORCE_GENERIC)
    _close(generic, want)
    pack, sm = _group_pack(gq, gsm, uq, usm)
    packed = ops.int8_gateup_silu_packed(xc, pack.cuda(), sm.cuda(), shift, norm_weights=nwc, epsilon=1e-5)
    _close(packed, want)


def test_packed_gateup_refuses_what_the_pipeline_cannot_serve():
    I, H, shift = 64, 64, 3  # groups of 8 weights
    pack = torch.zeros(I, H, 2, dtype=torch.uint8).cuda()
    sm = torch.zeros(I * (H >> shift), 2, 2, dtype=torch.float16).cuda()
    x = torch.zeros(1, H, dtype=torch.float16).cuda()
    with pytest.raises(RuntimeError, match="packed 8-bit gate/up"):
        ops.int8_gateup_silu_packed(x, pack, sm, shift)
