"""Tensor-parallel batch-1 decode of a Llama-4-Scout-17B-16E-architecture model (BASELINE config 5), random-init bf16:

  python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
      -m benchmarks.llama4_bench --steps 128 --warmup 8 [--layers 48]

48 layers, hidden 5120, 40 query / 8 KV heads, head dim 128, 16 routed experts (top-1 sigmoid) + a shared expert with
intermediate 8192, chunked attention window 8192, vocabulary 202048; 32-token random prompt, then greedy tokens from a
captured CUDA graph of the C decode stack's step (mui_llama4_stack_*, token fed back on the device). For the timed
model every rank builds only its own shard, so the full model never exists on one device; before that, a
`--parity-layers`-deep model of the same width, built identically on every rank and sharded, is checked against the
un-sharded stack on rank 0 (benchmarks/parity.py). Rank 0 prints one JSON line; the time is the maximum over ranks of
CUDA-event time around the replays.

Bytes a rank streams per token: its rows of QKV and o_proj, the router, the gate/up/down shards of the shared and of
the one selected expert in every layer, and its rows of the lm_head.
"""
import argparse
import json
import os

import torch

SCOUT = dict(layers=48, hidden=5120, expert_intermediate=8192, heads=40, kv_heads=8, head_dim=128, vocab=202048,
             experts=16, top_k=1, eps=1e-5, rope_theta=500000.0, chunk=8192, use_qk_norm=True, temperature_tuning=True,
             attn_scale=0.1, floor_scale=8192.0)
PROMPT_LEN = 32
MAX_SEQ = 16384


def local_weights(cfg, rank, world, dtype, dev):
    """This rank's shard, generated in place (normal(0, 0.02) weights, norm weights 1 + normal(0, 0.01))."""
    H, D = cfg["hidden"], cfg["head_dim"]
    hq, hkv, il = cfg["heads"] // world, cfg["kv_heads"] // world, cfg["expert_intermediate"] // world
    E = cfg["experts"] + 1
    g = torch.Generator(device=dev).manual_seed(1000 + rank)
    gr = torch.Generator(device=dev).manual_seed(7)   # replicated tensors: same seed on every rank

    def rn(gen, *shape):
        return torch.empty(*shape, dtype=dtype, device=dev).normal_(0.0, 0.02, generator=gen)

    def nw():
        return (1.0 + 0.01 * torch.randn(H, device=dev, generator=gr)).to(dtype)

    L = cfg["layers"]
    w = {"embed": rn(gr, cfg["vocab"], H), "norm": nw(), "lm_head": rn(g, cfg["vocab"] // world, H),
         "ln1": [nw() for _ in range(L)], "ln2": [nw() for _ in range(L)],
         "router": [rn(gr, cfg["experts"], H) for _ in range(L)],
         "qkv": [rn(g, (hq + 2 * hkv) * D, H) for _ in range(L)], "o": [rn(g, H, hq * D) for _ in range(L)],
         "gate": [rn(g, E * il, H) for _ in range(L)], "up": [rn(g, E * il, H) for _ in range(L)],
         "down": [rn(g, E * H, il) for _ in range(L)]}
    local = dict(cfg)
    local.update(heads=hq, kv_heads=hkv, expert_intermediate=il, world=world, rank=rank,
                 lm_head_sharded=world > 1, vocab_offset=rank * (cfg["vocab"] // world))
    return w, local


def bytes_per_token_per_rank(cfg, world):
    H, D = cfg["hidden"], cfg["head_dim"]
    hq, hkv, il = cfg["heads"] // world, cfg["kv_heads"] // world, cfg["expert_intermediate"] // world
    per_layer = (hq + 2 * hkv) * D * H + H * hq * D + cfg["experts"] * H + (1 + cfg["top_k"]) * 3 * il * H + 2 * H
    return 2 * (cfg["layers"] * per_layer + (cfg["vocab"] // world) * H + H)


def common_model(cfg, dtype, dev):
    """A whole (un-sharded) model of `cfg` from per-tensor seeds: every rank builds the same one and shards it."""
    H, D, I = cfg["hidden"], cfg["head_dim"], cfg["expert_intermediate"]
    E = cfg["experts"] + 1
    names = ["embed", "lm_head", "norm", "qkv", "o", "router", "gate", "up", "down", "ln1", "ln2"]

    def t(name, layer, shape, norm=False):
        g = torch.Generator(device=dev).manual_seed(7919 * (names.index(name) + 1) + layer)
        if norm:
            return (1.0 + 0.01 * torch.randn(*shape, device=dev, generator=g)).to(dtype)
        return torch.empty(*shape, dtype=dtype, device=dev).normal_(0.0, 0.02, generator=g)

    L = cfg["layers"]
    return {"embed": t("embed", 0, (cfg["vocab"], H)), "lm_head": t("lm_head", 0, (cfg["vocab"], H)),
            "norm": t("norm", 0, (H,), True),
            "qkv": [t("qkv", l, ((cfg["heads"] + 2 * cfg["kv_heads"]) * D, H)) for l in range(L)],
            "o": [t("o", l, (H, cfg["heads"] * D)) for l in range(L)],
            "router": [t("router", l, (cfg["experts"], H)) for l in range(L)],
            "gate": [t("gate", l, (E * I, H)) for l in range(L)], "up": [t("up", l, (E * I, H)) for l in range(L)],
            "down": [t("down", l, (E * H, I)) for l in range(L)],
            "ln1": [t("ln1", l, (H,), True) for l in range(L)], "ln2": [t("ln2", l, (H,), True) for l in range(L)]}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--layers", type=int, default=SCOUT["layers"])
    ap.add_argument("--parity-layers", type=int, default=4)
    args = ap.parse_args()

    import torch.distributed as dist

    from benchmarks.parity import tp_parity
    from muillm_b200 import capi
    from muillm_b200.comm import MuiCommunicator
    from muillm_b200.llama4 import Llama4DecodeStack, shard_llama4_weights

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    dtype, flags = torch.bfloat16, capi.MUI_FLAG_PDL
    comm = None
    if world > 1:
        comm = MuiCommunicator(rank=rank, world_size=world, key="l4bench" + os.environ.get("MASTER_PORT", "0"),
                               capacity_elems=1 << 16)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, SCOUT["vocab"], (1, PROMPT_LEN), generator=g)
    K, W = args.steps, max(3, args.warmup)

    # ---- parity: a shallow model of the same width, sharded stack against the un-sharded one on rank 0 ----
    parity = None
    if world > 1 and args.parity_layers > 0:
        pcfg = dict(SCOUT, layers=args.parity_layers)
        pcfg["use_rope"] = [(l + 1) % 4 != 0 for l in range(pcfg["layers"])]
        full = common_model(pcfg, dtype, dev)
        wl, lcfg = shard_llama4_weights(full, pcfg, rank, world, shard_lm_head=True)
        if rank != 0:
            full = None
        torch.cuda.empty_cache()
        pstack = Llama4DecodeStack(wl, lcfg, max_seq=256, max_new_tokens=96, flags=flags, comm=comm)
        parity = tp_parity(pstack, lambda: Llama4DecodeStack(full, pcfg, max_seq=256, max_new_tokens=96, flags=flags),
                           prompt, rank, dev)
        parity["layers"] = args.parity_layers
        del pstack, wl, full
        torch.cuda.empty_cache()

    # ---- the full-depth model: this rank's shard only ----
    cfg = dict(SCOUT, layers=args.layers)
    cfg["use_rope"] = [(l + 1) % 4 != 0 for l in range(cfg["layers"])]
    w, local = local_weights(cfg, rank, world, dtype, dev)
    stack = Llama4DecodeStack(w, local, max_seq=MAX_SEQ, max_new_tokens=PROMPT_LEN + W + K + 8, flags=flags, comm=comm)
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
    seconds = s_ev.elapsed_time(e_ev) * 1e-3
    status = capi.device_status()
    t = torch.tensor([seconds], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    seconds = float(t.item())
    if rank == 0:
        nbytes = bytes_per_token_per_rank(cfg, world)
        line = {"metric": "bs=1 decode tokens/s/user (Llama-4-Scout-17B-16E arch)", "value": K / seconds,
                "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": seconds / K * 1e3,
                "higher_is_better": True, "scaling": "strong", "dtype": "bf16", "data": "synthetic",
                "config": {"workload": f"Llama-4-Scout-arch decode (BASELINE config 5), {cfg['layers']} layers, bs=1, "
                                       f"{PROMPT_LEN}-token prompt, attention chunk {cfg['chunk']} (ring caches of "
                                       f"{min(MAX_SEQ, cfg['chunk'])} rows in the rope layers, plain caches of "
                                       f"{MAX_SEQ} rows in the others)",
                           "parallelism": f"tp{world}",
                           "launch": "CUDA graph of one C-stack decode step, programmatic dependent launch"},
                "launches_per_step": stack.launches_per_step,
                "hbm_fraction": {"bytes_per_step_per_rank": nbytes, "achieved_gbs": nbytes * K / seconds / 1e9,
                                 "of_nominal_8tbs": nbytes * K / seconds / 1e9 / 8000.0},
                "reference_published_tok_s": {"4x MI300X": 190.0}, "device_status": status}
        if parity is not None:
            line["parity"] = parity
        print(json.dumps(line), flush=True)
    barrier()
    if comm is not None:
        comm.all_reduce_sum(torch.zeros(8, device=dev))
        torch.cuda.synchronize()
        barrier()
        comm.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
