"""Small fixed workloads for profiling one kernel at a time (e.g. under `ncu -k regex:<kernel> -c 2`).

  python -m benchmarks.profile_cases gateup     # fused gate/up+SiLU GEMV, Llama-3-8B MLP shape, 4 distinct layers
  python -m benchmarks.profile_cases linear     # QKV-shaped fused-norm GEMV (6144 x 4096), 8 distinct matrices
  python -m benchmarks.profile_cases attention  # fused RoPE + cache write + attention, 32 q / 8 kv heads, S = 2048
  python -m benchmarks.profile_cases w8         # int8 (per-row scale) gate/up GEMV, same MLP shape
  python -m benchmarks.profile_cases attention_short  # one-CTA-per-KV-head tensor-core attention, S = 256
  python -m benchmarks.profile_cases attention_split  # the same kernel with the tokens split over CTAs, S = 4096
  python -m benchmarks.profile_cases down       # down projection 4096 x 14336 + residual, 4 distinct matrices
  python -m benchmarks.profile_cases lm_head    # fused-norm lm_head 128256 x 4096, 2 distinct matrices (2.1 GB)
  python -m benchmarks.profile_cases w8_down    # int8 (per-row scale) down projection
  python -m benchmarks.profile_cases w8_packed  # uint8 per-group gate/up on the reference's interleaved pack
  python -m benchmarks.profile_cases moe        # MoE MLP, shared + top-1 of 16 experts, H = 5120, I = 2048 (bf16)
  python -m benchmarks.profile_cases prefill    # tcgen05 prefill GEMM, 256 rows, 14336 x 4096

Each case keeps well under 2 GB on the device, uses inputs larger than L2 in total so that weights come from
HBM, launches the kernel a handful of times and synchronises.
"""
import sys

import torch

from muillm_b200 import capi, ops


def _gateup(dtype=torch.float16, w8=False):
    H, I, L = 4096, 14336, 4
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(0)
    x = torch.randn(1, H, device=dev, generator=g).to(dtype)
    nw = torch.ones(H, device=dev, dtype=dtype)
    ws = []
    for _ in range(L):
        G = (torch.randn(I, H, device=dev, generator=g) * 0.02).to(dtype)
        U = (torch.randn(I, H, device=dev, generator=g) * 0.02).to(dtype)
        if w8:
            def q(w):
                s = (w.float().abs().amax(dim=1) / 127.0).clamp(min=1e-8).to(dtype)
                return torch.round(w.float() / s.float()[:, None]).clamp(-127, 127).to(torch.int8), s
            ws.append(q(G) + q(U))
        else:
            ws.append((G, U))
    for rep in range(2):
        for w in ws:
            if w8:
                ops.int8_gateup_silu(x, w[0], w[1], w[2], w[3], norm_weights=nw, epsilon=1e-5)
            else:
                ops.gateup_silu(x, w[0], w[1], norm_weights=nw, epsilon=1e-5)
    torch.cuda.synchronize()


def _linear(dtype=torch.float16):
    N, K, L = 6144, 4096, 8
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(0)
    x = torch.randn(1, K, device=dev, generator=g).to(dtype)
    nw = torch.ones(K, device=dev, dtype=dtype)
    ws = [(torch.randn(N, K, device=dev, generator=g) * 0.02).to(dtype) for _ in range(L)]
    for rep in range(2):
        for w in ws:
            ops.muillm_linear_forward(None, x, w, norm_weights=nw, epsilon=1e-5)
    torch.cuda.synchronize()


def _attention(dtype=torch.float16, S=2048, flags=0):
    B, Hq, Hkv, D, max_T = 1, 32, 8, 128, 4096
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(0)
    qkv = torch.randn(B, (Hq + 2 * Hkv) * D, device=dev, generator=g).to(dtype)
    caches = [(torch.randn(B, Hkv, max_T, D, device=dev, generator=g).to(dtype),
               torch.randn(B, Hkv, max_T, D, device=dev, generator=g).to(dtype)) for _ in range(16)]
    cos = torch.ones(max_T, D, device=dev, dtype=dtype)
    sin = torch.zeros(max_T, D, device=dev, dtype=dtype)
    pos = torch.full((B,), S - 1, dtype=torch.int64, device=dev)
    cpos = torch.tensor([S - 1], dtype=torch.int64, device=dev)
    sl = torch.tensor([S], dtype=torch.int32, device=dev)
    for kc, vc in caches:
        ops.rope_flash_decode(qkv, cos, sin, pos, cpos, sl, kc, vc, Hq, flags=flags)
    torch.cuda.synchronize()


def _attention_split(dtype=torch.float16, S=4096):
    B, Hq, Hkv, D, max_T = 1, 32, 8, 128, 4096
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(0)
    qkv = torch.randn(B, (Hq + 2 * Hkv) * D, device=dev, generator=g).to(dtype)
    caches = [(torch.randn(B, Hkv, max_T, D, device=dev, generator=g).to(dtype),
               torch.randn(B, Hkv, max_T, D, device=dev, generator=g).to(dtype)) for _ in range(16)]
    cos = torch.ones(max_T, D, device=dev, dtype=dtype)
    sin = torch.zeros(max_T, D, device=dev, dtype=dtype)
    pos = torch.full((B,), S - 1, dtype=torch.int64, device=dev)
    cpos = torch.tensor([S - 1], dtype=torch.int64, device=dev)
    sl = torch.tensor([S], dtype=torch.int32, device=dev)
    ws = torch.zeros(capi.lib().mui_flash_decode_workspace_bytes(B, Hq, Hkv, D, max_T), dtype=torch.uint8, device=dev)
    for kc, vc in caches:
        ops.rope_flash_decode(qkv, cos, sin, pos, cpos, sl, kc, vc, Hq, flags=capi.MUI_FLAG_SPLIT_CONTEXT,
                              workspace=ws, max_attended=S)
    torch.cuda.synchronize()


def _rand(n, k, dtype, g, dev):
    return (torch.randn(n, k, device=dev, generator=g) * 0.02).to(dtype)


def _down(dtype=torch.float16, w8=False):
    H, I, L = 4096, 14336, 4
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(0)
    t = torch.randn(1, I, device=dev, generator=g).to(dtype)
    res = torch.randn(1, H, device=dev, generator=g).to(dtype)
    ws = [_rand(H, I, dtype, g, dev) for _ in range(L)]
    if w8:
        def q(w):
            s = (w.float().abs().amax(dim=1) / 127.0).clamp(min=1e-8).to(dtype)
            return torch.round(w.float() / s.float()[:, None]).clamp(-127, 127).to(torch.int8), s
        ws = [q(w) for w in ws]
    for rep in range(2):
        for w in ws:
            if w8:
                ops.muillm_int8_linear_forward(t, w[0], w[1], 0, residual=res)
            else:
                ops.muillm_linear_forward(None, t, w, residual=res)
    torch.cuda.synchronize()


def _lm_head(dtype=torch.float16):
    V, H = 128256, 4096
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(0)
    x = torch.randn(1, H, device=dev, generator=g).to(dtype)
    nw = torch.ones(H, device=dev, dtype=dtype)
    ws = [torch.empty(V, H, dtype=dtype, device=dev).normal_(0.0, 0.02, generator=g) for _ in range(2)]
    for rep in range(2):
        for w in ws:
            ops.muillm_linear_forward(None, x, w, norm_weights=nw, epsilon=1e-5)
    torch.cuda.synchronize()


def _w8_packed(dtype=torch.float16, shift=7):
    from benchmarks.kernel_bench import _q8_group

    H, I, L = 4096, 14336, 4
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(0)
    x = torch.randn(1, H, device=dev, generator=g).to(dtype)
    nw = torch.ones(H, device=dev, dtype=dtype)
    ws = []
    for _ in range(L):
        (gq, gsm), (uq, usm) = _q8_group(_rand(I, H, dtype, g, dev), shift), _q8_group(_rand(I, H, dtype, g, dev), shift)
        ws.append((torch.stack([gq, uq], dim=-1).contiguous(), torch.stack([gsm, usm], dim=1).contiguous()))
    for rep in range(2):
        for pack, sm in ws:
            ops.int8_gateup_silu_packed(x, pack, sm, shift, norm_weights=nw, epsilon=1e-5)
    torch.cuda.synchronize()


def _moe(dtype=torch.bfloat16):
    H, I, shared, routed, L = 5120, 2048, 1, 16, 3
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(0)
    E = shared + routed
    x = torch.randn(1, 1, H, device=dev, generator=g).to(dtype)
    nw = torch.ones(H, device=dev, dtype=dtype)
    sets = [(_rand(E * I, H, dtype, g, dev), _rand(E * I, H, dtype, g, dev), _rand(E * H, I, dtype, g, dev))
            for _ in range(L)]
    scores = torch.full((1,), 0.7, device=dev, dtype=dtype)
    for j, (G, U, Dw) in enumerate(sets):
        for e in range(3):
            idx = torch.tensor([(5 * j + 3 * e) % routed], dtype=torch.int64, device=dev)
            ops.muillm_gateupsilumoe_forward(None, shared, routed, nw, 1e-5, G, U, Dw, x, x, scores, idx)
    torch.cuda.synchronize()


def _prefill(dtype=torch.float16):
    M, N, K, L = 256, 14336, 4096, 4
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(0)
    x = torch.randn(M, K, device=dev, generator=g).to(dtype)
    ws = [_rand(N, K, dtype, g, dev) for _ in range(L)]
    for rep in range(2):
        for w in ws:
            ops.prefill_linear(x, w)
    torch.cuda.synchronize()


def main():
    case = sys.argv[1] if len(sys.argv) > 1 else "gateup"
    torch.cuda.set_device(0)
    {"gateup": _gateup, "linear": _linear, "attention": _attention, "w8": lambda: _gateup(w8=True),
     "attention_short": lambda: _attention(S=256, flags=capi.MUI_FLAG_SHORT_CONTEXT),
     "attention_split": _attention_split, "down": _down, "lm_head": _lm_head, "w8_down": lambda: _down(w8=True),
     "w8_packed": _w8_packed, "moe": _moe, "prefill": _prefill}[case]()
    assert capi.device_status() == 0
    print("ok", case)


if __name__ == "__main__":
    main()
