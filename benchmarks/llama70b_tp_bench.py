"""Tensor-parallel decode of a Llama-3.3-70B-architecture model (BASELINE config 4), random-init bf16:

  python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
      -m benchmarks.llama70b_tp_bench [--steps 64] [--warmup 8] [--layers 80] [--json out.json]

80 layers, hidden 8192, 64 query / 8 KV heads of 128, intermediate 28672, vocabulary 128256; QKV and gate/up cut by
output rows (whole heads per rank), o_proj and down by input columns with the [B, 8192] all-reduce fused into the
GEMV epilogue (two per layer), lm_head by rows with a distributed arg-max. Every tensor is generated from its own
seed, on the GPU, one tensor at a time, and only this rank's slice is kept: the full model never exists on a device,
yet every N shards the same model.

Rank 0 prints JSON lines:
  * "parity":   a `--parity-layers`-deep model of the same width, the sharded stack's first 32 greedy tokens
                against the un-sharded stack on rank 0 (benchmarks/parity.py);
  * "decode b1": batch 1, 16-token prompt, K graph replays: tokens/s, bytes a rank streams per step and that as a
                fraction of 8 TB/s;
  * "decode b8 ragged": batch 8, prompt lengths uniform in [8, 512] (seed 2), left-padded with attention mask
                and per-sequence RoPE positions (LlamaDecodeStack.greedy_ragged): aggregate tokens/s;
  * "all-reduce": microseconds per stand-alone all-reduce of [B, 8192] bf16 (B = 1, 8) in a graph of back-to-back
                launches, and the fused GEMV + all-reduce minus the same GEMV for the o_proj and down shards.
Times are CUDA-event times, maximum over ranks.
"""
import argparse
import json
import os

import torch
import torch.distributed as dist

from benchmarks.parity import tp_parity
from benchmarks.timing import time_graph
from muillm_b200 import capi, ops
from muillm_b200.comm import MuiCommunicator
from muillm_b200.decoder_stack import LlamaDecodeStack

LLAMA70B = dict(layers=80, hidden=8192, intermediate=28672, heads=64, kv_heads=8, head_dim=128, vocab=128256,
                eps=1e-5, rope_theta=500000.0)
TENSOR_IDS = {"embed": 1, "lm_head": 2, "norm": 3, "qkv": 4, "o": 5, "gate": 6, "up": 7, "down": 8, "ln1": 9, "ln2": 10}


def _full_tensor(name, layer, shape, dtype, dev, norm=False):
    """The whole tensor `name` of `layer`, from its own seed (the same on every rank)."""
    g = torch.Generator(device=dev).manual_seed(1_000_003 * TENSOR_IDS[name] + layer)
    if norm:
        return (1.0 + 0.01 * torch.randn(*shape, device=dev, generator=g)).to(dtype)
    return torch.empty(*shape, dtype=dtype, device=dev).normal_(0.0, 0.02, generator=g)


def build_weights(cfg, rank, world, dtype, dev, keep_full=False):
    """This rank's shard (and, with keep_full, the un-sharded tensors as well), one tensor at a time."""
    H, I, V, D = cfg["hidden"], cfg["intermediate"], cfg["vocab"], cfg["head_dim"]
    Hq, Hkv = cfg["heads"], cfg["kv_heads"]
    hq, hkv, il, vl = Hq // world, Hkv // world, I // world, V // world
    full = {k: [] for k in ("qkv", "o", "gate", "up", "down", "ln1", "ln2")} if keep_full else None
    loc = {k: [] for k in ("qkv", "o", "gate", "up", "down", "ln1", "ln2")}

    def rows(t, a, b):
        return t[a:b].clone()

    def cols(t, a, b):
        return t[:, a:b].contiguous()

    embed = _full_tensor("embed", 0, (V, H), dtype, dev)
    lm = _full_tensor("lm_head", 0, (V, H), dtype, dev)
    norm = _full_tensor("norm", 0, (H,), dtype, dev, norm=True)
    loc.update(embed=embed, norm=norm, lm_head=rows(lm, rank * vl, (rank + 1) * vl))
    if keep_full:
        full.update(embed=embed, norm=norm, lm_head=lm)
    del lm
    for l in range(cfg["layers"]):
        t = _full_tensor("qkv", l, ((Hq + 2 * Hkv) * D, H), dtype, dev)
        q = t[rank * hq * D:(rank + 1) * hq * D]
        k = t[Hq * D + rank * hkv * D: Hq * D + (rank + 1) * hkv * D]
        v = t[(Hq + Hkv) * D + rank * hkv * D: (Hq + Hkv) * D + (rank + 1) * hkv * D]
        loc["qkv"].append(torch.cat([q, k, v], dim=0))
        if keep_full:
            full["qkv"].append(t)
        t = _full_tensor("o", l, (H, Hq * D), dtype, dev)
        loc["o"].append(cols(t, rank * hq * D, (rank + 1) * hq * D))
        if keep_full:
            full["o"].append(t)
        for name in ("gate", "up"):
            t = _full_tensor(name, l, (I, H), dtype, dev)
            loc[name].append(rows(t, rank * il, (rank + 1) * il))
            if keep_full:
                full[name].append(t)
        t = _full_tensor("down", l, (H, I), dtype, dev)
        loc["down"].append(cols(t, rank * il, (rank + 1) * il))
        if keep_full:
            full["down"].append(t)
        for name in ("ln1", "ln2"):
            t = _full_tensor(name, l, (H,), dtype, dev, norm=True)
            loc[name].append(t)
            if keep_full:
                full[name].append(t)
        del t
    local_cfg = dict(cfg)
    local_cfg.update(heads=hq, kv_heads=hkv, intermediate=il, vocab=vl, embed_vocab=V, vocab_offset=rank * vl)
    return loc, local_cfg, full


def bytes_per_rank_step(cfg, world):
    H, I, V, D = cfg["hidden"], cfg["intermediate"], cfg["vocab"], cfg["head_dim"]
    per_layer = ((cfg["heads"] + 2 * cfg["kv_heads"]) * D * H + cfg["heads"] * D * H + 3 * I * H) // world + 2 * H
    return 2 * (cfg["layers"] * per_layer + V * H // world + H)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--layers", type=int, default=80)
    ap.add_argument("--parity-layers", type=int, default=2)
    ap.add_argument("--skip-b8", action="store_true")
    ap.add_argument("--json", default=None)
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", device_id=dev)
    comm = MuiCommunicator(rank=rank, world_size=world, key="l70" + os.environ.get("MASTER_PORT", "0"),
                           capacity_elems=1 << 17)
    dtype = torch.bfloat16
    flags = capi.MUI_FLAG_PDL
    K, W = args.steps, max(3, args.warmup)
    lines = []

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(sec):
        t = torch.tensor([sec], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    def emit(line):
        lines.append(line)
        if rank == 0:
            print(json.dumps(line), flush=True)

    # ---- parity on a shallow model of the same width ----
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, LLAMA70B["vocab"], (1, 16), generator=g)
    pcfg = dict(LLAMA70B, layers=args.parity_layers)
    wl, lcfg, full = build_weights(pcfg, rank, world, dtype, dev, keep_full=(rank == 0))
    stack = LlamaDecodeStack(wl, lcfg, max_seq=256, batch=1, max_new_tokens=64, flags=flags, comm=comm)
    par = tp_parity(stack, lambda: LlamaDecodeStack(full, pcfg, max_seq=256, batch=1, max_new_tokens=64, flags=flags),
                    prompt, rank, dev)
    par.update(case="parity", gpus=world, layers=args.parity_layers, width="hidden 8192, 64q/8kv, intermediate 28672")
    emit(par)
    del stack, wl, full
    torch.cuda.empty_cache()

    # ---- the full-depth model, this rank's shard only ----
    cfg = dict(LLAMA70B, layers=args.layers)
    wl, lcfg, _ = build_weights(cfg, rank, world, dtype, dev)
    torch.cuda.empty_cache()
    nbytes = bytes_per_rank_step(cfg, world)

    # batch 1
    stack = LlamaDecodeStack(wl, lcfg, max_seq=1024, batch=1, max_new_tokens=16 + W + K + 8, flags=flags, comm=comm)
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        stack.reset(0)
        stack.prefill(prompt)
        stack.capture()
        stack.replay(W)
    barrier()
    s_ev, e_ev = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(st):
        s_ev.record(st)
        stack.replay(K)
        e_ev.record(st)
    barrier()
    sec = max_over_ranks(s_ev.elapsed_time(e_ev) * 1e-3)
    emit({"case": "decode b1", "gpus": world, "layers": args.layers, "steps": K, "warmup": W, "tokens_per_s": K / sec,
          "ms_per_step": sec / K * 1e3, "bytes_per_rank_step": nbytes, "per_rank_tbs": nbytes * K / sec / 1e12,
          "of_8tbs": nbytes * K / sec / 8e12, "launches_per_step": stack.launches_per_step,
          "all_reduces_per_step": 2 * args.layers + 1, "device_status": capi.device_status()})
    del stack

    # batch 8, ragged prompts
    if not args.skip_b8:
        B = 8
        lens = torch.randint(8, 513, (B,), generator=torch.Generator().manual_seed(2)).tolist()
        gp = torch.Generator().manual_seed(3)
        prompts = [torch.randint(0, cfg["vocab"], (n,), generator=gp) for n in lens]
        stack = LlamaDecodeStack(wl, lcfg, max_seq=1024, batch=B, max_new_tokens=max(lens) + W + K + 8, flags=flags,
                                 comm=comm)
        timing = {"warm_steps": W, "barrier": barrier}
        stack.greedy_ragged(prompts, 1 + W + K, use_graph=True, timing=timing)
        sec = max_over_ranks(timing["replay_seconds"])
        steps = timing["replay_steps"]
        emit({"case": "decode b8 ragged", "gpus": world, "layers": args.layers, "prompt_lengths": lens, "steps": steps,
              "tokens_per_s": B * steps / sec, "tokens_per_s_per_user": steps / sec, "ms_per_step": sec / steps * 1e3,
              "bytes_per_rank_step": nbytes, "of_8tbs": nbytes * steps / sec / 8e12,
              "device_status": capi.device_status()})
        del stack

    # all-reduce of [B, 8192] alone and fused
    H = cfg["hidden"]
    for B in (1, 8):
        src = torch.randn(B, H, device=dev).to(dtype)
        dst = torch.empty_like(src)
        ours = max_over_ranks(time_graph([lambda: comm.all_reduce_sum(src, flags=flags, out=dst)], 200, sync=barrier))
        buf = src.clone()
        nccl = max_over_ranks(time_graph([lambda: dist.all_reduce(buf)], 200, sync=barrier))
        row = {"case": "all-reduce", "shape": [B, H], "gpus": world, "alone_us": ours * 1e6, "nccl_us": nccl * 1e6}
        for name, ws in (("o_proj", wl["o"]), ("down", wl["down"])):
            sets = ws[:6]
            x = torch.randn(B, sets[0].shape[1], device=dev).to(dtype)
            res = torch.randn(B, H, device=dev).to(dtype)
            y = torch.empty(B, H, device=dev, dtype=dtype)
            fused = max_over_ranks(time_graph(
                [(lambda w=w: comm.parallel_linear(x, w, residual=res, flags=flags, out=y)) for w in sets], 48,
                replays=10, sync=barrier))
            plain = max_over_ranks(time_graph(
                [(lambda w=w: ops.muillm_linear_forward(None, x, w, residual=res, flags=flags, out=y)) for w in sets],
                48, replays=10, sync=barrier))
            row[name] = {"K_local": sets[0].shape[1], "fused_us": fused * 1e6, "gemv_us": plain * 1e6,
                         "added_us": (fused - plain) * 1e6}
        emit(row)

    status = capi.device_status()
    barrier()
    if rank == 0 and args.json:
        with open(args.json, "w") as f:
            json.dump({"gpus": world, "device_status": status, "lines": lines}, f, indent=1)
    comm.all_reduce_sum(torch.zeros(8, device=dev))
    torch.cuda.synchronize()
    barrier()
    comm.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
