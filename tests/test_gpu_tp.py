"""Multi-GPU parity of the communicator and the fused sharded layers: one process per GPU (spawned here), results
against the CPU oracle on the un-sharded weights. Needs at least 2 GPUs; skipped otherwise."""
import os
import traceback

import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import decode_oracle as oracle  # noqa: E402
from parity_utils import check_greedy_tokens  # noqa: E402


def _world():
    return min(torch.cuda.device_count(), 8) if torch.cuda.is_available() else 0


def _worker(rank, world, key, fn_name, ret):
    try:
        os.environ["NCCL_NVLS_ENABLE"] = "0"
        torch.cuda.set_device(rank)
        from muillm_b200 import capi
        from muillm_b200.comm import MuiCommunicator

        comm = MuiCommunicator(rank=rank, world_size=world, key=key, capacity_elems=1 << 18, timeout_s=60.0)
        globals()[fn_name](rank, world, comm)
        torch.cuda.synchronize()
        assert capi.device_status() == 0, "a kernel recorded a device-side status"
        # all ranks leave together: nobody unmaps a segment a peer may still push into
        comm.all_reduce_sum(torch.zeros(8, device="cuda"))
        torch.cuda.synchronize()
        comm.close()
        ret[rank] = "ok"
    except Exception:  # pragma: no cover
        ret[rank] = traceback.format_exc()


def _run(fn_name):
    world = _world()
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    key = f"tp{os.getpid()}_{fn_name}"
    procs = [ctx.Process(target=_worker, args=(r, world, key, fn_name, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
    for p in procs:
        if p.is_alive():  # pragma: no cover
            p.terminate()
    for r in range(world):
        assert ret.get(r) == "ok", f"rank {r}: {ret.get(r)}"


def _case_all_reduce_and_broadcast(rank, world, comm):
    for dtype, n in ((torch.float16, 8192), (torch.bfloat16, 5120), (torch.float32, 1000), (torch.float16, 128256)):
        parts = [torch.randn(1, n, generator=torch.Generator().manual_seed(50 + r)).to(dtype) for r in range(world)]
        want = oracle.all_reduce_fixed_order(parts, dtype)
        for _ in range(3):  # repeated calls walk through both buffer generations
            got = comm.all_reduce_sum(parts[rank].cuda())
        assert torch.equal(got.cpu(), want), "all-reduce differs from the fixed-order fp32 sum"
    tok = torch.tensor([1234 + rank, 7], dtype=torch.int64, device="cuda")
    for src in range(world):
        out = comm.broadcast(tok, src)
        assert out.tolist() == [1234 + src, 7]


def _case_parallel_linear(rank, world, comm):
    for dtype in (torch.float16, torch.bfloat16):
        for (B, N, K) in ((1, 4096, 4096), (1, 8192, 1024 * world), (4, 515, 256 * world), (1, 128, 8 * world),
                          (8, 2048, 4096 * world)):  # the last one: activations staged chunk by chunk
            g = torch.Generator().manual_seed(N + K + B)
            W = (torch.randn(N, K, generator=g) * 0.02).to(dtype)
            x = torch.randn(B, K, generator=g).to(dtype)
            res = torch.randn(B, N, generator=g).to(dtype)
            ab = (torch.randn(N, generator=g) * 0.1).to(dtype)
            ks = K // world
            want = oracle.linear(x, W, add_bias=ab, residual=res)
            for _ in range(2):
                got = comm.parallel_linear(x[:, rank * ks:(rank + 1) * ks].contiguous().cuda(),
                                           W[:, rank * ks:(rank + 1) * ks].contiguous().cuda(), add_bias=ab.cuda(),
                                           residual=res.cuda())
            torch.testing.assert_close(got.float().cpu(), want.float(), rtol=1e-2, atol=2e-3)
            # every rank holds the same bits: compare against rank 0's result
            ref0 = comm.broadcast(got.view(torch.int16).to(torch.int32), 0)
            assert torch.equal(ref0, got.view(torch.int16).to(torch.int32)), "ranks disagree bitwise"


def _case_parallel_mlp(rank, world, comm):
    dtype = torch.float16
    H, I, B = 1024, 512 * world, 1
    g = torch.Generator().manual_seed(3)
    x = torch.randn(B, H, generator=g).to(dtype)
    nw = (1 + 0.01 * torch.randn(H, generator=g)).to(dtype)
    G = (torch.randn(I, H, generator=g) * 0.03).to(dtype)
    U = (torch.randn(I, H, generator=g) * 0.03).to(dtype)
    Dw = (torch.randn(H, I, generator=g) * 0.03).to(dtype)
    want = oracle.mlp(x, G, U, Dw, norm_weights=nw, eps=1e-5, residual=x)
    s = I // world
    sl = slice(rank * s, (rank + 1) * s)
    xc = x.cuda()
    got = comm.parallel_mlp(xc, nw.cuda(), 1e-5, G[sl].contiguous().cuda(), U[sl].contiguous().cuda(),
                            Dw[:, sl].contiguous().cuda(), residual=xc)
    torch.testing.assert_close(got.float().cpu(), want.float(), rtol=1e-2, atol=2e-3)


def _case_parallel_moe(rank, world, comm):
    from muillm_b200 import capi

    for dtype in (torch.float16, torch.bfloat16):
        for (H, I, shared, routed, top_k) in ((512, 64 * world, 1, 4, 1), (5120, 256 * world, 1, 16, 1),
                                              (256, 24 * world, 0, 8, 2)):
            g = torch.Generator().manual_seed(H + I + top_k)
            E = shared + routed
            x = torch.randn(1, 1, H, generator=g).to(dtype)
            nw = (1 + 0.01 * torch.randn(H, generator=g)).to(dtype)
            G = (torch.randn(E, I, H, generator=g) * 0.03).to(dtype)
            U = (torch.randn(E, I, H, generator=g) * 0.03).to(dtype)
            Dw = (torch.randn(E, H, I, generator=g) * 0.03).to(dtype)
            scores, idx = oracle.topk_sigmoid(torch.randn(1, 1, routed, generator=g).to(dtype), top_k)
            want = oracle.moe_mlp(x, G.reshape(E * I, H), U.reshape(E * I, H), Dw.reshape(E * H, I), shared, E, scores,
                                  idx, norm_weights=nw, eps=1e-5, residual=x)
            # every expert's intermediate dimension is split across the ranks
            s = I // world
            sl = slice(rank * s, (rank + 1) * s)
            Gl = G[:, sl].reshape(E * s, H).contiguous().cuda()
            Ul = U[:, sl].reshape(E * s, H).contiguous().cuda()
            Dl = Dw[:, :, sl].reshape(E * H, s).contiguous().cuda()
            xc = x.cuda()
            for flags in (0, capi.MUI_FLAG_PDL):
                got = comm.parallel_moe_mlp(shared, routed, nw.cuda(), 1e-5, Gl, Ul, Dl, xc, xc,
                                            scores.reshape(-1).cuda(), idx.reshape(-1).cuda(), flags=flags)
                tol = dict(rtol=1e-2, atol=2e-3) if dtype == torch.float16 else dict(rtol=2e-2, atol=8e-3)
                torch.testing.assert_close(got.float().cpu(), want.float(), **tol)


def _case_tp_llama4_runner(rank, world, comm):
    """Llama-4 architecture (MoE + shared expert, chunked and full attention layers) sharded over the ranks against
    the same model on one GPU (which tests/test_gpu_llama4_model.py holds to Hugging Face), token by token on the
    single-GPU run's own greedy tokens."""
    from muillm_b200 import capi
    from muillm_b200.llama4 import Llama4DecodeRunner, shard_llama4_weights

    cfg = dict(layers=3, hidden=256, expert_intermediate=64, heads=8, kv_heads=8, head_dim=64, vocab=512, experts=4,
               top_k=1, eps=1e-5, rope_theta=500000.0, chunk=8, use_rope=[True, True, False], use_qk_norm=True,
               temperature_tuning=True, attn_scale=0.1, floor_scale=4.0)
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(3)
    H, I, D, E = cfg["hidden"], cfg["expert_intermediate"], cfg["head_dim"], cfg["experts"] + 1

    def rn(*shape):
        return (torch.randn(*shape, generator=g) * 0.08).to(dtype).cuda()

    def nw():
        return (1 + 0.01 * torch.randn(H, generator=g)).to(dtype).cuda()

    L = cfg["layers"]
    w = {"embed": rn(cfg["vocab"], H), "lm_head": rn(cfg["vocab"], H), "norm": nw(),
         "qkv": [rn((cfg["heads"] + 2 * cfg["kv_heads"]) * D, H) for _ in range(L)],
         "o": [rn(H, cfg["heads"] * D) for _ in range(L)], "router": [rn(cfg["experts"], H) for _ in range(L)],
         "gate": [rn(E * I, H) for _ in range(L)], "up": [rn(E * I, H) for _ in range(L)],
         "down": [rn(E * H, I) for _ in range(L)], "ln1": [nw() for _ in range(L)], "ln2": [nw() for _ in range(L)]}
    prompt = torch.randint(0, cfg["vocab"], (10,), generator=g)
    single = Llama4DecodeRunner(w, cfg, max_seq=64)
    wl, cl = shard_llama4_weights(w, cfg, rank, world)
    for flags in (0, capi.MUI_FLAG_PDL):
        single.reset()
        tp = Llama4DecodeRunner(wl, cl, max_seq=64, flags=flags, comm=comm)
        tok = int(prompt[0])
        for step in range(28):
            a = single.step(tok)
            b = tp.step(tok)
            torch.testing.assert_close(b.float(), a.float(), rtol=3e-2, atol=3e-2)
            tok = int(prompt[step + 1]) if step + 1 < prompt.numel() else int(torch.argmax(a.float()).item())


def _case_tp_llama4_stack(rank, world, comm):
    """The Llama-4 C decode stack sharded over the ranks (heads, expert intermediate, lm_head rows; fused all-reduces
    in o_proj and the expert down projection, distributed arg-max) against the same stack on one GPU, teacher-forced on
    the single-GPU run's tokens: logits of this rank's vocabulary rows and the chosen token at every step."""
    from muillm_b200 import capi
    from muillm_b200.llama4 import Llama4DecodeStack, shard_llama4_weights

    cfg = dict(layers=4, hidden=256, expert_intermediate=128, heads=8, kv_heads=8, head_dim=128, vocab=512, experts=4,
               top_k=1, eps=1e-5, rope_theta=500000.0, chunk=8, use_rope=[True, True, True, False], use_qk_norm=True,
               temperature_tuning=True, attn_scale=0.1, floor_scale=4.0)
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(3)
    H, I, D, E = cfg["hidden"], cfg["expert_intermediate"], cfg["head_dim"], cfg["experts"] + 1

    def rn(*shape):
        return (torch.randn(*shape, generator=g) * 0.08).to(dtype).cuda()

    def nw():
        return (1 + 0.01 * torch.randn(H, generator=g)).to(dtype).cuda()

    L = cfg["layers"]
    w = {"embed": rn(cfg["vocab"], H), "lm_head": rn(cfg["vocab"], H), "norm": nw(),
         "qkv": [rn((cfg["heads"] + 2 * cfg["kv_heads"]) * D, H) for _ in range(L)],
         "o": [rn(H, cfg["heads"] * D) for _ in range(L)], "router": [rn(cfg["experts"], H) for _ in range(L)],
         "gate": [rn(E * I, H) for _ in range(L)], "up": [rn(E * I, H) for _ in range(L)],
         "down": [rn(E * H, I) for _ in range(L)], "ln1": [nw() for _ in range(L)], "ln2": [nw() for _ in range(L)]}
    prompt = torch.randint(0, cfg["vocab"], (1, 10), generator=g)
    wl, cl = shard_llama4_weights(w, cfg, rank, world, shard_lm_head=True)
    vl, off = cfg["vocab"] // world, cl["vocab_offset"]
    for flags in (0, capi.MUI_FLAG_PDL):
        single = Llama4DecodeStack(w, cfg, max_seq=64, max_new_tokens=64, flags=flags)
        tp = Llama4DecodeStack(wl, cl, max_seq=64, max_new_tokens=64, flags=flags, comm=comm)
        single.reset(0)
        tp.reset(0)
        tok = prompt[:, 0].contiguous()
        for step in range(30):
            single.set_tokens(tok)
            single.step()
            tp.set_tokens(tok)
            tp.step()
            a, b = single.logits().float(), tp.logits().float()
            torch.testing.assert_close(b, a[:, off: off + vl], rtol=3e-2, atol=3e-2)
            ta, tb = int(single.next_tokens()[0].item()), int(tp.next_tokens()[0].item())
            if ta != tb:
                # the winner comes from another rank's rows: compare on the single-GPU logits
                assert abs(float(a[0, ta]) - float(a[0, tb])) < 3e-2, f"step {step}: {ta} vs {tb}"
            tok = prompt[:, step + 1].contiguous() if step + 1 < prompt.shape[1] else torch.tensor([ta])
        # graph replay of the sharded stack reproduces its own eager tokens
        want = tp.greedy(prompt, 16, use_graph=False).cpu()
        got = tp.greedy(prompt, 16, use_graph=True).cpu()
        assert torch.equal(got, want), f"flags {flags}: graph {got.tolist()} vs eager {want.tolist()}"
        del single, tp


def _case_tp_decode_stack(rank, world, comm):
    from muillm_b200 import capi
    from muillm_b200.decoder_stack import LlamaDecodeStack, shard_llama_weights

    cfg = dict(layers=3, hidden=512, intermediate=1024, heads=8, kv_heads=8, head_dim=64, vocab=1024, eps=1e-5,
               rope_theta=500000.0)
    dtype = torch.float16
    w = oracle.make_llama_weights(cfg, dtype, seed=0, std=0.08)
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, cfg["vocab"], (1, 16), generator=g)
    want = oracle.LlamaOracle(w, cfg, max_T=64).greedy(prompt, 32)
    wl, cl = shard_llama_weights(w, cfg, rank, world)
    wl = {k: ([t.cuda() for t in v] if isinstance(v, list) else v.cuda()) for k, v in wl.items()}
    for flags, graph in ((0, False), (capi.MUI_FLAG_PDL, True)):
        stack = LlamaDecodeStack(wl, cl, max_seq=64, batch=1, flags=flags, comm=comm)
        # all 32 positions are checked: identical tokens, or (teacher-forced on the oracle's sequence) a flip only
        # where the oracle's two best logits are a near-tie — the sharded fp32 sums round in another order
        check_greedy_tokens(stack, w, cfg, prompt, want, 64, graph, label=f"tp{world} flags={flags} graph={graph}")
        del stack


def test_all_reduce_and_broadcast():
    _run("_case_all_reduce_and_broadcast")


def test_parallel_linear_fused_all_reduce():
    _run("_case_parallel_linear")


def test_parallel_mlp_fused_all_reduce():
    _run("_case_parallel_mlp")


def test_tp_decode_stack_greedy_tokens():
    _run("_case_tp_decode_stack")


def test_parallel_moe_mlp_fused_all_reduce():
    _run("_case_parallel_moe")


def test_tp_llama4_runner_matches_single_gpu():
    _run("_case_tp_llama4_runner")


def test_tp_llama4_stack_matches_single_gpu():
    _run("_case_tp_llama4_stack")
