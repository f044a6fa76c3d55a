"""The prefill GEMM on the tcgen05 tensor cores (mui_prefill_linear_forward, mui_prefill_gateup_silu_forward) against
the CPU oracle: more than 8 rows, tile edges in every dimension (rows of W not a multiple of 128, tokens not a multiple
of 16, several token tiles, K not a multiple of the 64-element stage), every epilogue term."""
import pytest
import torch

from muillm_b200 import capi, ops
from oracle import decode_oracle as oracle

pytestmark = pytest.mark.gpu

DTYPES = [torch.float16, torch.bfloat16]


def _close(got, want, dtype):
    tol = dict(rtol=1e-2, atol=1e-3) if dtype == torch.float16 else dict(rtol=2e-2, atol=4e-3)
    assert torch.isfinite(got).all()
    torch.testing.assert_close(got.float().cpu(), want.float(), **tol)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K", [(16, 128, 64), (16, 128, 256), (48, 384, 4096), (100, 515, 1000), (256, 256, 512),
                                   (300, 130, 328), (9, 6144, 4096), (1024, 1024, 1024)])
def test_prefill_linear_matches_oracle(dtype, M, N, K):
    g = torch.Generator().manual_seed(M + N + K)
    x = torch.randn(M, K, generator=g).to(dtype)
    W = (torch.randn(N, K, generator=g) * 0.02).to(dtype)
    want = oracle.linear(x, W)
    got = ops.prefill_linear(x.cuda(), W.cuda())
    _close(got, want, dtype)
    assert capi.device_status() == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_prefill_linear_epilogue_terms(dtype):
    M, N, K = 40, 200, 512
    g = torch.Generator().manual_seed(4)
    x = torch.randn(M, K, generator=g).to(dtype)
    W = (torch.randn(N, K, generator=g) * 0.03).to(dtype)
    mb = (1 + 0.1 * torch.randn(N, generator=g)).to(dtype)
    ab = (torch.randn(N, generator=g) * 0.5).to(dtype)
    res = torch.randn(M, N, generator=g).to(dtype)
    for act, name in ((capi.MUI_ACT_IDENTITY, "identity"), (capi.MUI_ACT_SILU, "silu")):
        want = oracle.linear(x, W, activation=name, mul_bias=mb, add_bias=ab, residual=res)
        got = ops.prefill_linear(x.cuda(), W.cuda(), mul_bias=mb.cuda(), add_bias=ab.cuda(), residual=res.cuda(),
                                 activation=act, flags=capi.MUI_FLAG_PDL)
        _close(got, want, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,I,H", [(32, 256, 128), (77, 1000, 512), (256, 14336, 4096), (300, 520, 320)])
def test_prefill_gateup_matches_oracle(dtype, M, I, H):
    g = torch.Generator().manual_seed(M + I)
    x = torch.randn(M, H, generator=g).to(dtype)
    G = (torch.randn(I, H, generator=g) * 0.02).to(dtype)
    U = (torch.randn(I, H, generator=g) * 0.02).to(dtype)
    want = oracle.gateup_silu(x, G, U)
    got = ops.prefill_gateup_silu(x.cuda(), G.cuda(), U.cuda())
    _close(got, want, dtype)
    assert capi.device_status() == 0


def test_prefill_rejects_bad_arguments():
    x = torch.zeros(16, 20, dtype=torch.float16, device="cuda")
    W = torch.zeros(32, 20, dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError, match="multiple of 16 bytes"):
        ops.prefill_linear(x, W)
