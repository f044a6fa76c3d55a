"""Per-kernel HBM throughput of the decode path: `python -m benchmarks.kernel_bench [--json out.json]`.

Every case runs one kernel over several distinct weight sets (in total larger than the 126 MB L2, so each launch
streams from HBM), as a CUDA graph of back-to-back launches with programmatic dependent launch, timed with CUDA
events after warm-up. Reported per launch: microseconds, algorithmic GB/s (weights + scales + activations in and out,
each counted once) and that figure as a fraction of 8 TB/s.

Cases: the fused RMSNorm -> QKV GEMV at the Mistral-7B shape, the int8 (per-row scale) gate/up+SiLU and down GEMVs
of the Llama-3-8B MLP at batch 1/2/4/8, the five GEMV shapes of a Llama-3.1-8B decode step, fused attention at several
sequence lengths, and the MoE MLP at the Llama-4-Scout per-rank shape.
"""
import argparse
import json

import torch

from muillm_b200 import capi, ops

NOMINAL_GBS = 8000.0


def _time_graph(fns, iters_per_graph, replays=5):
    """fns: list of callables (one per weight set); returns seconds per launch."""
    n = len(fns)
    for i in range(n):
        fns[i]()
    torch.cuda.synchronize()
    st = torch.cuda.Stream()
    gr = torch.cuda.CUDAGraph()
    with torch.cuda.stream(st):
        with torch.cuda.graph(gr, stream=st):
            for i in range(iters_per_graph):
                fns[i % n]()
    for _ in range(3):
        gr.replay()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(replays):
        gr.replay()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) * 1e-3 / (replays * iters_per_graph)


def _randw(n, k, dtype, g, dev):
    return (torch.randn(n, k, device=dev, generator=g) * 0.02).to(dtype)


def _q8(w):
    s = (w.float().abs().amax(dim=1) / 127.0).clamp(min=1e-8).to(w.dtype)
    return torch.round(w.float() / s.float()[:, None]).clamp(-127, 127).to(torch.int8), s


def _sets_for(bytes_per_set):
    return max(3, min(12, int(3.0e8 // max(bytes_per_set, 1)) + 1))


def case_linear(name, N, K, B, dtype, norm, residual, dev, g, flags):
    L = _sets_for(N * K * 2)
    ws = [_randw(N, K, dtype, g, dev) for _ in range(L)]
    x = torch.randn(B, K, device=dev, generator=g).to(dtype)
    nw = torch.ones(K, device=dev, dtype=dtype) if norm else None
    res = torch.randn(B, N, device=dev, generator=g).to(dtype) if residual else None
    fns = [(lambda w=w: ops.muillm_linear_forward(None, x, w, norm_weights=nw, epsilon=1e-5, residual=res, flags=flags))
           for w in ws]
    nbytes = N * K * 2 + B * K * 2 + B * N * 2 + (K * 2 if norm else 0) + (B * N * 2 if residual else 0)
    return name, _time_graph(fns, 4 * L), nbytes


def case_gateup(name, I, H, B, dtype, dev, g, flags, w8=False):
    L = _sets_for(2 * I * H * (1 if w8 else 2))
    x = torch.randn(B, H, device=dev, generator=g).to(dtype)
    nw = torch.ones(H, device=dev, dtype=dtype)
    fns = []
    for _ in range(L):
        G, U = _randw(I, H, dtype, g, dev), _randw(I, H, dtype, g, dev)
        if w8:
            (gq, gs), (uq, us) = _q8(G), _q8(U)
            fns.append(lambda gq=gq, gs=gs, uq=uq, us=us: ops.int8_gateup_silu(x, gq, gs, uq, us, norm_weights=nw,
                                                                               epsilon=1e-5, flags=flags))
        else:
            fns.append(lambda G=G, U=U: ops.gateup_silu(x, G, U, norm_weights=nw, epsilon=1e-5, flags=flags))
        del G, U
    nbytes = 2 * I * H * (1 if w8 else 2) + (4 * I if w8 else 0) + B * H * 2 + H * 2 + B * I * 2
    return name, _time_graph(fns, 4 * L), nbytes


def case_down_w8(name, H, I, B, dtype, dev, g, flags):
    L = _sets_for(H * I)
    qs = [_q8(_randw(H, I, dtype, g, dev)) for _ in range(L)]
    t = torch.randn(B, I, device=dev, generator=g).to(dtype)
    res = torch.randn(B, H, device=dev, generator=g).to(dtype)
    fns = [(lambda q=q, s=s: ops.muillm_int8_linear_forward(t, q, s, 0, residual=res, flags=flags)) for q, s in qs]
    nbytes = H * I + 2 * H + B * I * 2 + 2 * B * H * 2
    return name, _time_graph(fns, 4 * L), nbytes


def _q8_group(w, shift=7):
    """The reference's per-group format: uint8 q and {scale, min} pairs (muillm/quantization/rtnquantizer.py:48-88)."""
    gs = 1 << shift
    t = w.float().reshape(-1, gs)
    mx, mn = t.amax(dim=1, keepdim=True), t.amin(dim=1, keepdim=True)
    rng = (mx - mn).clamp(min=1e-6)
    mn = (mn + mx) * 0.5 - rng * 0.5
    sc = rng / 255
    q = t.sub(mn).div(sc).clamp(0, 255).round().to(torch.uint8).reshape_as(w)
    return q, torch.cat([sc, mn], dim=-1).to(w.dtype)


def case_group_gateup_packed(name, I, H, B, dtype, dev, g, flags, shift=7):
    """gate/up on the reference's interleaved [I, H, 2] pack with [I * G, 2, 2] {scale, min} pairs."""
    L = _sets_for(2 * I * H)
    x = torch.randn(B, H, device=dev, generator=g).to(dtype)
    nw = torch.ones(H, device=dev, dtype=dtype)
    fns = []
    for _ in range(L):
        (gq, gsm), (uq, usm) = _q8_group(_randw(I, H, dtype, g, dev), shift), _q8_group(_randw(I, H, dtype, g, dev), shift)
        pack = torch.stack([gq, uq], dim=-1).contiguous()
        sm = torch.stack([gsm, usm], dim=1).contiguous()
        del gq, uq
        fns.append(lambda pack=pack, sm=sm: ops.int8_gateup_silu_packed(x, pack, sm, shift, norm_weights=nw,
                                                                        epsilon=1e-5, flags=flags))
    nbytes = 2 * I * H + 2 * I * (H >> shift) * 4 + B * H * 2 + H * 2 + B * I * 2
    return name, _time_graph(fns, 4 * L), nbytes


def case_group_down(name, H, I, B, dtype, dev, g, flags, shift=7):
    L = _sets_for(H * I)
    qs = [_q8_group(_randw(H, I, dtype, g, dev), shift) for _ in range(L)]
    t = torch.randn(B, I, device=dev, generator=g).to(dtype)
    res = torch.randn(B, H, device=dev, generator=g).to(dtype)
    fns = [(lambda q=q, s=s: ops.muillm_int8_linear_forward(t, q, s, shift, residual=res, flags=flags)) for q, s in qs]
    nbytes = H * I + H * (I >> shift) * 4 + B * I * 2 + 2 * B * H * 2
    return name, _time_graph(fns, 4 * L), nbytes


def case_attention(name, S, dtype, dev, g, flags, short=False, split=False):
    B, Hq, Hkv, D, max_T = 1, 32, 8, 128, 4096
    L = 12
    qkv = torch.randn(B, (Hq + 2 * Hkv) * D, device=dev, generator=g).to(dtype)
    caches = [(torch.randn(B, Hkv, max_T, D, device=dev, generator=g).to(dtype),
               torch.randn(B, Hkv, max_T, D, device=dev, generator=g).to(dtype)) for _ in range(L)]
    cos = torch.ones(max_T, D, device=dev, dtype=dtype)
    sin = torch.zeros(max_T, D, device=dev, dtype=dtype)
    pos = torch.full((B,), S - 1, dtype=torch.int64, device=dev)
    cpos = torch.tensor([S - 1], dtype=torch.int64, device=dev)
    sl = torch.tensor([S], dtype=torch.int32, device=dev)
    ws = None
    if short:
        flags = flags | capi.MUI_FLAG_SHORT_CONTEXT
    if split:
        flags = flags | capi.MUI_FLAG_SPLIT_CONTEXT
        ws = torch.zeros(capi.lib().mui_flash_decode_workspace_bytes(B, Hq, Hkv, D, max_T), dtype=torch.uint8, device=dev)
    fns = [(lambda kc=kc, vc=vc: ops.rope_flash_decode(qkv, cos, sin, pos, cpos, sl, kc, vc, Hq, flags=flags,
                                                       workspace=ws, max_attended=S))
           for kc, vc in caches]
    nbytes = 2 * B * Hkv * S * D * 2 + (Hq + 2 * Hkv) * D * 2 + Hq * D * 2
    return name, _time_graph(fns, 4 * L), nbytes


def case_moe(name, H, I, shared, routed, dtype, dev, g, flags):
    E = shared + routed
    L = 3
    x = torch.randn(1, 1, H, device=dev, generator=g).to(dtype)
    nw = torch.ones(H, device=dev, dtype=dtype)
    sets = [(_randw(E * I, H, dtype, g, dev), _randw(E * I, H, dtype, g, dev), _randw(E * H, I, dtype, g, dev))
            for _ in range(L)]
    scores = torch.full((1,), 0.7, device=dev, dtype=dtype)
    fns = []
    for j, (G, U, Dw) in enumerate(sets):
        for e in range(4):
            idx = torch.tensor([(5 * j + 3 * e) % routed], dtype=torch.int64, device=dev)
            fns.append(lambda G=G, U=U, Dw=Dw, idx=idx: ops.muillm_gateupsilumoe_forward(
                None, shared, routed, nw, 1e-5, G, U, Dw, x, x, scores, idx, flags=flags))
    nbytes = (shared + 1) * 3 * I * H * 2 + 4 * H * 2
    return name + " (2 launches)", _time_graph(fns, 2 * len(fns)), nbytes


def case_prefill(M, N, K, dtype, dev, g):
    """The tcgen05 prefill GEMM beside torch's (cuBLAS) at the same shape: microseconds and dense TFLOP/s."""
    import torch.nn.functional as F

    L = _sets_for(N * K * 2)
    ws = [_randw(N, K, dtype, g, dev) for _ in range(L)]
    x = torch.randn(M, K, device=dev, generator=g).to(dtype)
    ours = _time_graph([(lambda w=w: ops.prefill_linear(x, w)) for w in ws], 4 * L)
    blas = _time_graph([(lambda w=w: F.linear(x, w)) for w in ws], 4 * L)
    flops = 2.0 * M * N * K
    return {"case": f"prefill GEMM M={M} N={N} K={K}", "us": ours * 1e6, "tflops": flops / ours / 1e12,
            "cublas_us": blas * 1e6, "cublas_tflops": flops / blas / 1e12, "weight_gbs": N * K * 2 / ours / 1e9}


def run(dtype=torch.float16):
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator(device=dev).manual_seed(0)
    flags = capi.MUI_FLAG_PDL
    rows = []

    def add(r):
        name, sec, nbytes = r
        gbs = nbytes / sec / 1e9
        rows.append({"case": name, "us": sec * 1e6, "bytes": nbytes, "gbs": gbs, "of_8tbs": gbs / NOMINAL_GBS})
        print(f"{name:58s} {sec * 1e6:8.2f} us {gbs:8.1f} GB/s {gbs / NOMINAL_GBS:6.3f} of 8 TB/s", flush=True)
        torch.cuda.empty_cache()

    add(case_linear("norm+QKV GEMV 6144x4096 (Mistral-7B), fp16", 6144, 4096, 1, dtype, True, False, dev, g, flags))
    for B in (1, 2, 4, 8):
        add(case_gateup(f"int8 gate/up+SiLU 2x14336x4096, B={B}", 14336, 4096, B, dtype, dev, g, flags, w8=True))
        add(case_down_w8(f"int8 down 4096x14336 + residual, B={B}", 4096, 14336, B, dtype, dev, g, flags))
    for B in (1, 4):
        add(case_group_gateup_packed(f"uint8 group-128 packed gate/up+SiLU 14336x4096x2, B={B}", 14336, 4096, B, dtype,
                                     dev, g, flags))
        add(case_group_down(f"uint8 group-128 down 4096x14336 + residual, B={B}", 4096, 14336, B, dtype, dev, g, flags))
    add(case_linear("o_proj 4096x4096 + residual, fp16", 4096, 4096, 1, dtype, False, True, dev, g, flags))
    add(case_gateup("gate/up+SiLU 2x14336x4096, fp16", 14336, 4096, 1, dtype, dev, g, flags))
    for B in (2, 8):
        add(case_gateup(f"gate/up+SiLU 2x14336x4096, fp16, B={B}", 14336, 4096, B, dtype, dev, g, flags))
    add(case_linear("down 4096x14336 + residual, fp16", 4096, 14336, 1, dtype, False, True, dev, g, flags))
    add(case_linear("norm+lm_head 128256x4096, fp16", 128256, 4096, 1, dtype, True, False, dev, g, flags))
    add(case_linear("QKV 6144x4096, bf16", 6144, 4096, 1, torch.bfloat16, True, False, dev, g, flags))
    for S in (256, 2048, 4096):
        add(case_attention(f"rope+cache+attention 32q/8kv d128, S={S}", S, dtype, dev, g, flags))
    for S in (64, 256, 384):
        add(case_attention(f"rope+cache+attention, one CTA per KV head, S={S}", S, dtype, dev, g, flags, short=True))
    for S in (1024, 2048, 4096):
        add(case_attention(f"rope+cache+attention, tokens split over CTAs, S={S}", S, dtype, dev, g, flags, split=True))
    add(case_moe("MoE MLP shared+top-1 of 16, H=5120 I=2048, bf16", 5120, 2048, 1, 16, torch.bfloat16, dev, g, flags))
    for (M, N, K) in ((16, 6144, 4096), (64, 6144, 4096), (256, 6144, 4096), (256, 14336, 4096), (1024, 6144, 4096),
                      (2048, 4096, 14336)):
        r = case_prefill(M, N, K, dtype, dev, g)
        rows.append(r)
        print(f"{r['case']:58s} {r['us']:8.2f} us {r['tflops']:7.1f} TFLOP/s (torch/cuBLAS {r['cublas_us']:8.2f} us "
              f"{r['cublas_tflops']:7.1f} TFLOP/s); weights at {r['weight_gbs']:.0f} GB/s", flush=True)
        torch.cuda.empty_cache()
    assert capi.device_status() == 0
    return rows


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--json", default=None)
    ap.add_argument("--md", default=None, help="also write the table as markdown rows")
    args = ap.parse_args()
    rows = run()
    if args.json:
        with open(args.json, "w") as f:
            json.dump(rows, f, indent=1)
    if args.md:
        with open(args.md, "w") as f:
            f.write("| case | us per launch | GB/s | of 8 TB/s |\n|---|---|---|---|\n")
            for r in rows:
                if "gbs" in r:
                    f.write(f"| {r['case']} | {r['us']:.2f} | {r['gbs']:.1f} | {r['of_8tbs']:.3f} |\n")
            f.write("\n| prefill case | us | TFLOP/s | torch (cuBLAS) us | torch TFLOP/s |\n|---|---|---|---|---|\n")
            for r in rows:
                if "tflops" in r:
                    f.write(f"| {r['case']} | {r['us']:.2f} | {r['tflops']:.1f} | {r['cublas_us']:.2f} | "
                            f"{r['cublas_tflops']:.1f} |\n")


if __name__ == "__main__":
    main()
