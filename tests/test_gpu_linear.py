"""GPU parity of the GEMV-shaped kernels (linear, gate/up+SiLU, MLP) against the CPU oracle, through the C ABI.

Tolerance is the one the north star states for 16-bit outputs: 1e-2 relative / 1e-3 absolute.
"""
import pytest
import torch

from muillm_b200 import capi, ops
from oracle import decode_oracle as oracle

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-2, 1e-3
DTYPES = [torch.float16, torch.bfloat16]
PATHS = {"auto": 0, "generic": capi.MUI_FLAG_FORCE_GENERIC, "pdl": capi.MUI_FLAG_PDL}


def _gen(seed):
    return torch.Generator().manual_seed(seed)


def _close(got, want):
    got, want = got.float().cpu(), want.float()
    assert got.shape == want.shape
    assert torch.isfinite(got).all()
    torch.testing.assert_close(got, want, rtol=RTOL, atol=ATOL)


def _mk(shape, g, std, dtype):
    return (torch.randn(*shape, generator=g) * std).to(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("path", list(PATHS))
@pytest.mark.parametrize("N,K", [(6144, 4096), (4096, 14336), (37, 1000), (33, 77), (16, 4096), (1, 8), (300, 520)])
def test_linear_fused_norm(dtype, path, N, K):
    """Config-1 style: y = W · rmsnorm(x), seeded N(0,1) activations, N(0,0.02) weights, norm 1+N(0,0.01)."""
    g = _gen(0)
    x = torch.randn(1, K, generator=g).to(dtype)
    nw = (1 + 0.01 * torch.randn(K, generator=g)).to(dtype)
    W = _mk((N, K), g, 0.02, dtype)
    want = oracle.linear(x, W, norm_weights=nw, eps=1e-5)
    got = ops.muillm_linear_forward(None, x.cuda(), W.cuda(), norm_weights=nw.cuda(), epsilon=1e-5, flags=PATHS[path])
    _close(got, want)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("path", ["auto", "generic"])
@pytest.mark.parametrize("B", [1, 2, 3, 4, 5, 8])
def test_linear_batch_epilogue(dtype, path, B):
    """Small batches with every epilogue term: SiLU, mul_bias, add_bias, residual."""
    N, K = 515, 1024
    g = _gen(B)
    x = torch.randn(B, K, generator=g).to(dtype)
    W = _mk((N, K), g, 0.03, dtype)
    mb = (1 + 0.1 * torch.randn(N, generator=g)).to(dtype)
    ab = _mk((N,), g, 0.5, dtype)
    res = _mk((B, N), g, 1.0, dtype)
    for act, name in ((capi.MUI_ACT_IDENTITY, "identity"), (capi.MUI_ACT_SILU, "silu")):
        want = oracle.linear(x, W, activation=name, mul_bias=mb, add_bias=ab, residual=res)
        got = ops.muillm_linear_forward(None, x.cuda(), W.cuda(), mul_bias=mb.cuda(), add_bias=ab.cuda(),
                                        residual=res.cuda(), activation=act, flags=PATHS[path])
        _close(got, want)


@pytest.mark.parametrize("dtype", DTYPES)
def test_linear_misaligned_weights_take_generic_path(dtype):
    """A weight view that is not 16-byte aligned must still give the right answer (scalar loads)."""
    N, K = 64, 256
    g = _gen(3)
    x = torch.randn(1, K, generator=g).to(dtype)
    Wbuf = _mk((N * K + 8,), g, 0.05, dtype).cuda()
    W = Wbuf[1:1 + N * K].view(N, K)
    assert W.data_ptr() % 16 != 0
    want = oracle.linear(x, W.cpu())
    got = ops.muillm_linear_forward(None, x.cuda(), W)
    _close(got, want)
    with pytest.raises(RuntimeError):
        ops.muillm_linear_forward(None, x.cuda(), W, flags=capi.MUI_FLAG_FORCE_PIPELINE)


def test_linear_rejects_bad_arguments():
    x = torch.zeros(9, 64, dtype=torch.float16, device="cuda")
    W = torch.zeros(8, 64, dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError):  # more than 8 rows is not a GEMV
        ops.muillm_linear_forward(None, x, W)
    with pytest.raises(RuntimeError):  # fp32 is not a supported dtype
        ops.muillm_linear_forward(None, x[:1].float(), W.float())
    with pytest.raises(RuntimeError):  # non-contiguous input
        ops.muillm_linear_forward(None, x[:1, ::2], W[:, :32].contiguous())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("path", list(PATHS))
@pytest.mark.parametrize("I,H,B", [(14336, 4096, 1), (1000, 512, 1), (77, 40, 2), (2048, 1024, 4), (520, 4096, 8)])
def test_gateup_silu(dtype, path, I, H, B):
    g = _gen(I + B)
    x = torch.randn(B, H, generator=g).to(dtype)
    nw = (1 + 0.01 * torch.randn(H, generator=g)).to(dtype)
    G = _mk((I, H), g, 0.02, dtype)
    U = _mk((I, H), g, 0.02, dtype)
    want = oracle.gateup_silu(x, G, U, norm_weights=nw, eps=1e-5)
    got = ops.gateup_silu(x.cuda(), G.cuda(), U.cuda(), norm_weights=nw.cuda(), epsilon=1e-5, flags=PATHS[path])
    _close(got, want)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("B", [1, 2, 4, 8])
def test_mlp_llama3_8b_shape(dtype, B):
    """Gate/up+SiLU then down with residual at the Llama-3-8B MLP shape (hidden 4096, intermediate 14336)."""
    H, I = 4096, 14336
    g = _gen(7)
    x = torch.randn(B, H, generator=g).to(dtype)
    nw = (1 + 0.01 * torch.randn(H, generator=g)).to(dtype)
    G = _mk((I, H), g, 0.02, dtype)
    U = _mk((I, H), g, 0.02, dtype)
    Dw = _mk((H, I), g, 0.02, dtype)
    xc = x.cuda()
    got = ops.muillm_gateupsilu_forward(None, nw.cuda(), 1e-5, G.cuda(), U.cuda(), Dw.cuda(), xc, xc)
    # Stage 1: the intermediate t against the oracle.
    t_gpu = ops.gateup_silu(xc, G.cuda(), U.cuda(), norm_weights=nw.cuda(), epsilon=1e-5)
    _close(t_gpu, oracle.gateup_silu(x, G, U, norm_weights=nw, eps=1e-5))
    # Stage 2: the down projection + residual against the oracle applied to that same 16-bit t (a t value
    # that rounds the other way by one 16-bit ulp moves y by more than the tolerance when y nearly cancels).
    want = oracle.linear(t_gpu.cpu(), Dw, residual=x)
    _close(got, want)
    # End to end the two compositions still agree to a few 16-bit ulps of the operands' magnitude.
    full = oracle.mlp(x, G, U, Dw, norm_weights=nw, eps=1e-5, residual=x)
    torch.testing.assert_close(got.float().cpu(), full.float(), rtol=2e-2, atol=8e-3)


@pytest.mark.parametrize("dtype", DTYPES)
def test_linear_is_deterministic(dtype):
    """Same inputs, same bits: no atomics or arrival-order dependent sums on the path."""
    g = _gen(11)
    x = torch.randn(1, 4096, generator=g).to(dtype).cuda()
    W = _mk((6144, 4096), g, 0.02, dtype).cuda()
    a = ops.muillm_linear_forward(None, x, W)
    b = ops.muillm_linear_forward(None, x, W)
    assert torch.equal(a, b)
    c = ops.muillm_linear_forward(None, x, W, flags=capi.MUI_FLAG_FORCE_GENERIC)
    _close(c, a.cpu())


def test_linear_full_size_linearity():
    """Size-independent property at the lm_head shape (128256 x 4096): W(x1 + x2) == W x1 + W x2 within rounding."""
    dtype = torch.float16
    g = _gen(5)
    N, K = 128256, 4096
    W = (torch.randn(N, K, generator=g, dtype=torch.float32) * 0.02).to(dtype).cuda()
    x1 = torch.randn(1, K, generator=g).to(dtype).cuda()
    x2 = torch.randn(1, K, generator=g).to(dtype).cuda()
    y1 = ops.muillm_linear_forward(None, x1, W).float()
    y2 = ops.muillm_linear_forward(None, x2, W).float()
    y12 = ops.muillm_linear_forward(None, (x1.float() + x2.float()).to(dtype), W).float()
    torch.testing.assert_close(y12, y1 + y2, rtol=2e-2, atol=2e-2)
    # spot-check 64 seeded rows against the oracle
    rows = torch.randint(0, N, (64,), generator=g)
    want = oracle.linear(x1.cpu(), W[rows.cuda()].cpu())
    _close(y1[:, rows.cuda()].to(dtype), want)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("B,N,K,norm", [
    (8, 8192, 14336, False),   # down projection of the 70B architecture cut in two: did not fit whole-row staging
    (8, 2560, 8192, True),     # QKV of the 70B architecture cut in four, fused norm
    (3, 4096, 2064, False),    # ragged last chunk (2064 = 2048 + 16)
    (2, 40000, 2048, True),    # 271 rows per CTA: 17 row blocks, two groups of accumulators
    (5, 515, 4096, True),      # rows not a multiple of the tile, batch padded to 8
])
def test_linear_batches_staged_chunk_by_chunk(dtype, B, N, K, norm):
    """Batches whose activations the pipeline stages one 2048-element chunk at a time (whole rows would leave the
    weight ring less than three stages): every epilogue term, with and without the fused norm, with dependent launch."""
    g = _gen(B + N)
    x = torch.randn(B, K, generator=g).to(dtype)
    W = _mk((N, K), g, 0.02, dtype)
    nw = (1 + 0.01 * torch.randn(K, generator=g)).to(dtype) if norm else None
    res = _mk((B, N), g, 1.0, dtype)
    ab = _mk((N,), g, 0.5, dtype)
    want = oracle.linear(x, W, norm_weights=nw, eps=1e-5, add_bias=ab, residual=res)
    for flags in (capi.MUI_FLAG_FORCE_PIPELINE, capi.MUI_FLAG_FORCE_PIPELINE | capi.MUI_FLAG_PDL):
        got = ops.muillm_linear_forward(None, x.cuda(), W.cuda(), norm_weights=None if nw is None else nw.cuda(),
                                        epsilon=1e-5, add_bias=ab.cuda(), residual=res.cuda(), flags=flags)
        _close(got, want)
    assert capi.device_status() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("B,I,H", [(8, 14336, 8192), (4, 20000, 4096), (2, 1000, 8192)])
def test_gateup_batches_staged_chunk_by_chunk(dtype, B, I, H):
    """Gate/up + SiLU for batches at the 70B shard shape (97 gate rows per CTA: 13 row blocks) and with more row blocks
    per CTA than one group of accumulators holds (136 rows: 17 blocks)."""
    g = _gen(I + B)
    x = torch.randn(B, H, generator=g).to(dtype)
    nw = (1 + 0.01 * torch.randn(H, generator=g)).to(dtype)
    G = _mk((I, H), g, 0.02, dtype)
    U = _mk((I, H), g, 0.02, dtype)
    want = oracle.gateup_silu(x, G, U, norm_weights=nw, eps=1e-5)
    Gc, Uc = G.cuda(), U.cuda()
    for flags in (capi.MUI_FLAG_FORCE_PIPELINE, capi.MUI_FLAG_FORCE_PIPELINE | capi.MUI_FLAG_PDL):
        got = ops.gateup_silu(x.cuda(), Gc, Uc, norm_weights=nw.cuda(), epsilon=1e-5, flags=flags)
        _close(got, want)
    assert capi.device_status() == 0
