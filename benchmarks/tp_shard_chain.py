"""One rank's share of a tensor-parallel decode step WITHOUT the collectives, on a single GPU:

  python -m benchmarks.tp_shard_chain [--arch 8b|70b] [--worlds 1,2,4,8] [--steps 64] [--timeline]

Builds the decode stack at the per-rank shapes of a world-N tensor-parallel run (heads, KV heads, intermediate and
vocabulary divided by N; random weights) and times CUDA-graph replays of its decode step. The result is the floor a
rank's step time would have if the all-reduces were free: weight streaming plus the chain of dependent launches. The
gap between the measured N-GPU step and this figure is what the collectives (and the skew between ranks) cost.

--timeline adds the device-side timeline of one middle layer of the replayed graph, from the records the kernels
write themselves (%globaltimer; mui_trace_enable): per launch the first CTA's start relative to the previous launch's
last CTA end, how long until the first CTA got past its wait for the previous kernel, until the last CTA had its
activations staged, and the whole launch.
"""
import argparse
import json

import torch

from benchmarks.timing import read_trace
from muillm_b200 import capi
from muillm_b200.decoder_stack import LlamaDecodeStack

ARCH = {
    "8b": dict(layers=32, hidden=4096, intermediate=14336, heads=32, kv_heads=8, head_dim=128, vocab=128256, eps=1e-5,
               rope_theta=500000.0),
    "70b": dict(layers=80, hidden=8192, intermediate=28672, heads=64, kv_heads=8, head_dim=128, vocab=128256, eps=1e-5,
                rope_theta=500000.0),
}


def local_weights(cfg, dtype, dev, seed=0):
    g = torch.Generator(device=dev).manual_seed(seed)
    H, I, V, D = cfg["hidden"], cfg["intermediate"], cfg["vocab"], cfg["head_dim"]

    def rn(*shape):
        return torch.empty(*shape, dtype=dtype, device=dev).normal_(0.0, 0.02, generator=g)

    def nw():
        return (1.0 + 0.01 * torch.randn(H, device=dev, generator=g)).to(dtype)

    L = cfg["layers"]
    return {"embed": rn(V, H), "lm_head": rn(V, H), "norm": nw(),
            "qkv": [rn((cfg["heads"] + 2 * cfg["kv_heads"]) * D, H) for _ in range(L)],
            "o": [rn(H, cfg["heads"] * D) for _ in range(L)], "gate": [rn(I, H) for _ in range(L)],
            "up": [rn(I, H) for _ in range(L)], "down": [rn(H, I) for _ in range(L)],
            "ln1": [nw() for _ in range(L)], "ln2": [nw() for _ in range(L)]}


def bytes_per_step(cfg):
    H, I, V, D = cfg["hidden"], cfg["intermediate"], cfg["vocab"], cfg["head_dim"]
    per_layer = (cfg["heads"] + 2 * cfg["kv_heads"]) * D * H + cfg["heads"] * D * H + 3 * I * H + 2 * H
    return 2 * (cfg["layers"] * per_layer + V * H + H)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--arch", default="8b", choices=sorted(ARCH))
    ap.add_argument("--worlds", default="1,2,4,8")
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--prompt", type=int, default=16)
    ap.add_argument("--timeline", action="store_true")
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    dtype = torch.float16 if args.arch == "8b" else torch.bfloat16
    full = ARCH[args.arch]
    for world in [int(v) for v in args.worlds.split(",")]:
        cfg = dict(full)
        cfg.update(heads=full["heads"] // world, kv_heads=full["kv_heads"] // world,
                   intermediate=full["intermediate"] // world, vocab=full["vocab"] // world)
        w = local_weights(cfg, dtype, dev)
        stack = LlamaDecodeStack(w, cfg, max_seq=4096, batch=args.batch, max_new_tokens=args.prompt + 3 * args.steps + 8,
                                 flags=capi.MUI_FLAG_PDL)
        prompt = torch.randint(0, cfg["vocab"], (args.batch, args.prompt), generator=torch.Generator().manual_seed(1))
        st = torch.cuda.Stream()
        nrec = stack.launches_per_step + 8
        tbuf = torch.empty(nrec * 64, dtype=torch.uint8, device=dev).fill_(255)
        with torch.cuda.stream(st):
            stack.reset(0)
            stack.prefill(prompt)
            if args.timeline:  # records are bound to launches at capture time and rewritten on every replay
                capi.check(capi.lib().mui_trace_enable(st.cuda_stream, tbuf.data_ptr(), nrec))
            stack.capture()
            if args.timeline:
                capi.check(capi.lib().mui_trace_enable(None, None, 0))
            stack.replay(args.steps)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record(st)
            stack.replay(args.steps)
            e.record(st)
        torch.cuda.synchronize()
        ms = s.elapsed_time(e) / args.steps
        nbytes = bytes_per_step(cfg)
        print(json.dumps({"arch": args.arch, "emulated_world": world, "batch": args.batch, "ms_per_step": ms,
                          "tokens_per_s": 1e3 / ms, "bytes_per_step": nbytes, "tbs": nbytes / ms / 1e9,
                          "launches": stack.launches_per_step, "us_per_launch": ms * 1e3 / stack.launches_per_step,
                          "device_status": capi.device_status()}), flush=True)
        if args.timeline:
            with torch.cuda.stream(st):
                tbuf.fill_(255)
                stack.replay(1)
            torch.cuda.synchronize()
            import ctypes
            tags = (ctypes.c_int * nrec)()
            n = min(capi.lib().mui_trace_count(tags, nrec), nrec)
            recs = read_trace(tbuf, n)
            names = {1: "linear", 2: "gate/up", 3: "attention", 4: "rope", 5: "all-reduce"}
            per_layer = max(1, (stack.launches_per_step - 2) // cfg["layers"])
            first = 1 + per_layer * (cfg["layers"] // 2)
            rows = []
            for i in range(first, min(first + per_layer + 1, n)):
                r, prev = recs[i], recs[i - 1]
                if None in (r["start"], r["end"], prev["end"]):
                    continue
                rows.append({"kernel": names.get(tags[i], str(tags[i])),
                             "gap_after_prev_end_us": (r["start"] - prev["end"]) / 1e3,
                             "start_to_past_wait_us": None if r["past_wait"] is None else (r["past_wait"] - r["start"]) / 1e3,
                             "start_to_staged_us": None if r["staged"] is None else (r["staged"] - r["start"]) / 1e3,
                             "launch_us": (r["end"] - r["start"]) / 1e3})
            print(json.dumps({"emulated_world": world, "timeline_of_layer": cfg["layers"] // 2, "launches": rows}), flush=True)
        del stack, w
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
