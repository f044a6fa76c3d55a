"""Flash decoding through the entry point that brings its own scratch (mui_flash_decode_static_scratch).

Some users of this library cannot give it a workspace: they run inside a host that has already split all device
memory among its own buffers, or in a loop where a cudaMalloc (which stalls the whole device) is forbidden. For
them the library keeps the split-KV partials in a fixed array of its own. This test calls that entry point through
the C ABI twice in a row, on different problems, and expects the results of the ordinary entry point both times:
the second call has to cope with whatever the first one left in the shared array. It lives in a file that pytest
collects last so that a failure here cannot hide the other tests of a stop-at-first-failure run, and it passes both
on its own in a fresh process and after everything else has run.
"""
import math

import pytest
import torch

from muillm_b200 import capi, ops
from oracle import decode_oracle as oracle

pytestmark = pytest.mark.gpu


def _static_scratch_decode(q, k, v, mask=None):
    B, Hq, _, D = q.shape
    Hkv, S = k.shape[1], k.shape[2]
    out = torch.empty((B, 1, Hq * D), dtype=q.dtype, device=q.device)
    m = None if mask is None else mask.reshape(B, S)
    capi.check(capi.lib().mui_flash_decode_static_scratch(
        torch.cuda.current_stream().cuda_stream, capi.MUI_F16 if q.dtype == torch.float16 else capi.MUI_BF16,
        B, Hq, Hkv, D, S, None, 1.0 / math.sqrt(D), q.data_ptr(), k.data_ptr(), v.data_ptr(),
        capi.Strides3(k.stride(0), k.stride(1), k.stride(2)), None if m is None else m.data_ptr(), out.data_ptr(), 0))
    return out


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_static_scratch_matches_workspace_entry_point_twice(dtype):
    g = torch.Generator().manual_seed(123)
    problems = [(1, 32, 8, 128, 1500, 4096), (2, 16, 4, 128, 333, 512)]  # (B, Hq, Hkv, D, S, cache length)
    for B, Hq, Hkv, D, S, max_T in problems:
        q = torch.randn(B, Hq, 1, D, generator=g).to(dtype).cuda()
        kc = torch.randn(B, Hkv, max_T, D, generator=g).to(dtype).cuda()
        vc = torch.randn(B, Hkv, max_T, D, generator=g).to(dtype).cuda()
        k, v = kc.narrow(2, 0, S), vc.narrow(2, 0, S)
        want = ops.muillm_causal_transformer_decoding_no_mask(q, k, v)
        got = _static_scratch_decode(q, k, v)
        torch.cuda.synchronize()
        torch.testing.assert_close(got.float(), want.float(), rtol=1e-2, atol=1e-3)
        # and against the CPU oracle, so that the two entry points cannot be wrong together
        ref = oracle.decode_attention(q.cpu(), k.cpu(), v.cpu())
        torch.testing.assert_close(got.float().cpu(), ref.float(), rtol=1e-2, atol=1e-3)
    assert capi.device_status() == 0


def test_static_scratch_rejects_problems_beyond_its_array():
    q = torch.zeros(1, 128, 1, 128, dtype=torch.float16, device="cuda")  # 128 heads > the 64 the array covers
    k = torch.zeros(1, 16, 64, 128, dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError, match="exceeds the built-in scratch"):
        _static_scratch_decode(q, k, k)
