"""GPU parity of the router top-k sigmoid and the MoE MLP against the CPU oracle, through the C ABI."""
import pytest
import torch

from muillm_b200 import capi, ops
from oracle import decode_oracle as oracle

pytestmark = pytest.mark.gpu

DTYPES = [torch.float16, torch.bfloat16]


def _gen(seed):
    return torch.Generator().manual_seed(seed)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,M,k", [(1, 16, 1), (1, 128, 1), (3, 128, 8), (2, 4096, 4), (1, 5, 5), (4, 33, 2)])
def test_topk_sigmoid(dtype, rows, M, k):
    g = _gen(M + k)
    logits = torch.randn(rows, 1, M, generator=g).to(dtype)
    logits[0, 0, M // 2] = logits[0, 0, 0]  # a tie: the lower index must win
    want_v, want_i = oracle.topk_sigmoid(logits, k)
    got_v, got_i = ops.muillm_topk_sigmoid_forward(logits.cuda(), k)
    assert torch.equal(got_i.cpu(), want_i)
    torch.testing.assert_close(got_v.float().cpu(), want_v.float(), rtol=1e-2, atol=1e-3)


def test_topk_sigmoid_wide_single_expert_warp_boundary():
    """k == 1 over more experts than a warp holds (the reference's k == 1 kernel only reduces inside warp 0)."""
    logits = torch.zeros(1, 1, 200, dtype=torch.float16)
    logits[0, 0, 150] = 3.0
    v, i = ops.muillm_topk_sigmoid_forward(logits.cuda(), 1)
    assert i.item() == 150
    assert abs(v.item() - torch.sigmoid(torch.tensor(3.0)).item()) < 1e-3


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("path", [0, capi.MUI_FLAG_FORCE_GENERIC, capi.MUI_FLAG_PDL])
@pytest.mark.parametrize("H,I,shared,routed,top_k", [
    (512, 256, 1, 4, 1),      # shared + top-1, the reference's test shape class
    (5120, 2048, 1, 16, 1),   # Llama-4-Scout per-rank shape at TP4
    (256, 136, 0, 8, 2),      # no shared expert, top-2, odd intermediate size
    (320, 64, 2, 3, 3),
])
def test_moe_mlp(dtype, path, H, I, shared, routed, top_k):
    g = _gen(H + I + top_k)
    E = shared + routed
    x = torch.randn(1, 1, H, generator=g).to(dtype)
    nw = (1 + 0.01 * torch.randn(H, generator=g)).to(dtype)
    G = (torch.randn(E * I, H, generator=g) * 0.03).to(dtype)
    U = (torch.randn(E * I, H, generator=g) * 0.03).to(dtype)
    Dw = (torch.randn(E * H, I, generator=g) * 0.03).to(dtype)
    router_logits = torch.randn(1, 1, routed, generator=g).to(dtype)
    scores, idx = oracle.topk_sigmoid(router_logits, top_k)
    want = oracle.moe_mlp(x, G, U, Dw, shared, E, scores, idx, norm_weights=nw, eps=1e-5, residual=x)
    xc = x.cuda()
    got = ops.muillm_gateupsilumoe_forward(None, shared, routed, nw.cuda(), 1e-5, G.cuda(), U.cuda(), Dw.cuda(), xc, xc,
                                           scores.reshape(-1).cuda(), idx.reshape(-1).cuda(), flags=path)
    tol = dict(rtol=1e-2, atol=2e-3) if dtype == torch.float16 else dict(rtol=2e-2, atol=8e-3)
    torch.testing.assert_close(got.float().cpu(), want.float(), **tol)
