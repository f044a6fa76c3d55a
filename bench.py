"""Headline benchmark: bs=1 decode tokens/s/user of a Llama-3.1-8B-architecture model (random-init fp16,
16-token prompt, static KV cache 4096), one decode step per "step".

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Prints ONE JSON line. `value` is tokens/s with the token fed back on the device (CUDA-graph replay of the
decode step); `e2e` is the same loop driven from the host through the public decode-stack API with the token
id copied host->device and the arg-max copied device->host every step. `roofline` is measured live for the
dominant kernel (the fused gate/up+SiLU GEMV); `cpu_baseline` times the CPU oracle (PyTorch fp32 on the host
cores) on a bounded sample. `--impl reference` times that CPU path alone.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

LLAMA31_8B = dict(layers=32, hidden=4096, intermediate=14336, heads=32, kv_heads=8, head_dim=128, vocab=128256,
                  eps=1e-5, rope_theta=500000.0)
PROMPT_LEN = 16
MAX_SEQ = 4096
# Llama 3 8B fp16 bs=1 on MI300X: 1 GPU and tensor-parallel 4 (the reference's published figures, its README.md:56-57)
BASELINE_TOK_S = {1: 210.0, 4: 420.0}
NOMINAL_HBM_GBS = 8000.0


def weight_bytes_per_token(cfg):
    H, I, V = cfg["hidden"], cfg["intermediate"], cfg["vocab"]
    qkv = (cfg["heads"] + 2 * cfg["kv_heads"]) * cfg["head_dim"] * H
    per_layer = qkv + cfg["heads"] * cfg["head_dim"] * H + 3 * I * H + 2 * H
    return 2 * (cfg["layers"] * per_layer + V * H + H)


def kv_bytes_per_token(cfg, seq):
    return 2 * cfg["layers"] * cfg["kv_heads"] * cfg["head_dim"] * 2 * seq


def measured_peak_gbs():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.samples = []
        self._stop = threading.Event()
        self._thread = None

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5).stdout
                parts = [p.strip() for p in out.strip().split(",")]
                if len(parts) >= 8:
                    self.samples.append(parts)
            except Exception:
                pass
            self._stop.wait(0.1)

    def __enter__(self):
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._thread.join(timeout=6)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        sm = sorted(float(s[0]) for s in self.samples if s[0].replace(".", "").isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[4 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": float(self.samples[0][1]),
                "power_w_max": max(float(s[2]) for s in self.samples), "samples": len(self.samples), "reasons": reasons}


def make_gpu_weights(cfg, dtype, device, seed):
    import torch

    g = torch.Generator(device=device).manual_seed(seed)
    H, I, V = cfg["hidden"], cfg["intermediate"], cfg["vocab"]
    qkv_n = (cfg["heads"] + 2 * cfg["kv_heads"]) * cfg["head_dim"]

    def rn(*shape):
        return (torch.randn(*shape, device=device, dtype=torch.float32, generator=g) * 0.02).to(dtype)

    def nw():
        return (1.0 + 0.01 * torch.randn(H, device=device, dtype=torch.float32, generator=g)).to(dtype)

    w = {"embed": rn(V, H), "lm_head": rn(V, H), "norm": nw(), "qkv": [], "o": [], "gate": [], "up": [], "down": [],
         "ln1": [], "ln2": []}
    for _ in range(cfg["layers"]):
        w["qkv"].append(rn(qkv_n, H))
        w["o"].append(rn(H, cfg["heads"] * cfg["head_dim"]))
        w["gate"].append(rn(I, H))
        w["up"].append(rn(I, H))
        w["down"].append(rn(H, I))
        w["ln1"].append(nw())
        w["ln2"].append(nw())
    return w


def time_dominant_kernel(w, cfg, flags):
    """Average duration of the fused gate/up+SiLU GEMV at the model's (per-rank) shape: a CUDA graph of 4 passes over
    the 32 layers' distinct weights (7.5 GB per pass on one GPU, so every launch streams from HBM), launched
    back to back with dependent launch as in the decode step, CUDA events around 3 replays."""
    import torch

    from benchmarks.timing import time_graph
    from muillm_b200 import ops

    H, I, L = cfg["hidden"], cfg["intermediate"], cfg["layers"]
    x = torch.randn(1, H, device=w["embed"].device, dtype=w["embed"].dtype)
    t = torch.empty(1, I, device=x.device, dtype=x.dtype)
    fns = [(lambda l=l: ops.gateup_silu(x, w["gate"][l], w["up"][l], norm_weights=w["ln2"][l], epsilon=cfg["eps"],
                                        flags=flags, out=t)) for l in range(L)]
    seconds = time_graph(fns, 4 * L, replays=3, warm_replays=1)
    algo_bytes = 2 * I * H * 2 + H * 2 * 2 + I * 2  # gate+up weights, x + norm weight, t out
    return seconds, algo_bytes


def time_plugin_e2e(w, cfg, prompt, K, W, max_seq):
    """The same decode loop through the reference-facing plugin surface (`muillm_ext` module handles, the calls the
    reference's Python makes: csrc/module.cpp:280-431): per token one `muillm_parallel_decoder_stack_forward`, the
    final-norm lm_head through `muillm_linear_forward`, arg-max in torch as the reference samples; the token id is
    copied host->device from pinned memory and the arg-max device->host every step. Returns tokens/s."""
    import torch

    from muillm_b200 import muillm_ext as ext
    from muillm_b200.decoder_stack import rope_tables

    Hq, Hkv, D, L = cfg["heads"], cfg["kv_heads"], cfg["head_dim"], cfg["layers"]
    dev, dt = w["embed"].device, w["embed"].dtype
    engine = ext.muillm_engine_init()
    comm = ext.muillm_comm_init(engine, 1, 1, 0, 0)
    cos, sin = rope_tables(max_seq, D, cfg["rope_theta"], dt, dev)
    embed = ext.muillm_embedding_module_init(engine, w["embed"])
    stack_rotary = ext.muillm_rotary_embedding_module_init(engine, 0, cos, sin)
    keep, decoders = [], []
    for l in range(L):
        qkv_lin = ext.muillm_parallel_linear_module_init(engine, comm, w["qkv"][l], norm_weights=w["ln1"][l],
                                                         epsilon=cfg["eps"], sharding_dim=0)
        slices = [(0, Hq * D), (Hq * D, (Hq + Hkv) * D), ((Hq + Hkv) * D, (Hq + 2 * Hkv) * D)]
        multilinear = ext.muillm_parallel_multilinear_module_init(engine, comm, qkv_lin, slices, 0)
        rotary = ext.muillm_rotary_embedding_module_init(engine, l, cos, sin)
        o_proj = ext.muillm_parallel_linear_module_init(engine, comm, w["o"][l], sharding_dim=1)
        attention = ext.muillm_parallel_attention_module_init(engine, comm, rotary, o_proj, Hq, Hkv, D)
        mlp = ext.muillm_parallel_gateupdownmlp_module_init(engine, comm, ext.GATEUPSILU_FUSED, w["ln2"][l],
                                                            w["gate"][l], w["up"][l], w["down"][l], cfg["eps"])
        decoders.append(ext.muillm_parallel_decoder_module_init(engine, comm, multilinear, attention, mlp))
        keep += [qkv_lin, multilinear, rotary, o_proj, attention, mlp]
    stack = ext.muillm_parallel_decoder_stack_init(engine, comm, embed, stack_rotary, decoders)
    kc = [torch.zeros(1, Hkv, max_seq, D, dtype=dt, device=dev) for _ in range(L)]
    vc = [torch.zeros(1, Hkv, max_seq, D, dtype=dt, device=dev) for _ in range(L)]
    cache = ext.muillm_static_kvcache_module_init(engine, kc, vc, 0)
    tok_in = torch.zeros(1, 1, dtype=torch.int64).pin_memory()
    tok_out = torch.zeros(1, dtype=torch.int64).pin_memory()
    pos_h = torch.zeros(1, 1, dtype=torch.int64).pin_memory()

    def step(t):
        pos_h[0, 0] = t
        ids = tok_in.to(dev, non_blocking=True)
        pos = pos_h.to(dev, non_blocking=True)
        h = ext.muillm_parallel_decoder_stack_forward(stack, cache, ids, None, None, pos, pos.view(1))
        logits = ext.muillm_linear_forward(engine, h, w["lm_head"], norm_weights=w["norm"], epsilon=cfg["eps"])
        tok_out.copy_(torch.argmax(logits.view(1, -1), dim=-1), non_blocking=True)
        torch.cuda.current_stream().synchronize()
        tok_in[0, 0] = tok_out[0]

    t = 0
    for i in range(prompt.shape[1]):
        tok_in[0, 0] = prompt[0, i]
        step(t)
        t += 1
    for _ in range(W):
        step(t)
        t += 1
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(K):
        step(t)
        t += 1
    torch.cuda.synchronize()
    seconds = time.perf_counter() - t0
    ext.muillm_parallel_decoder_stack_deinit(stack)
    for m in keep + decoders + [embed, stack_rotary]:
        m.release()
    return K / seconds


def cpu_decode_sample(cfg, seconds_budget=20.0, sample_layers=2, tokens=3):
    """Times the CPU oracle (PyTorch fp32, all host threads) on `sample_layers` decoder layers + the lm_head for
    `tokens` decode steps at sequence length ~PROMPT_LEN and scales the layer time to the full depth."""
    import torch

    from oracle import decode_oracle as oracle

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    sub = dict(cfg)
    sub["layers"] = sample_layers
    w = oracle.make_llama_weights(sub, torch.float32, seed=0)
    model = oracle.LlamaOracle(w, sub, max_T=64)
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, cfg["vocab"], (1, 2), generator=g)
    model.forward(prompt)  # warm-up (2 tokens)
    H = cfg["hidden"]
    t_layers, t_head, done = 0.0, 0.0, 0
    t_start = time.time()
    for _ in range(tokens):
        tok = torch.randint(0, cfg["vocab"], (1, 1), generator=g)
        t0 = time.time()
        model.forward(tok)
        t1 = time.time()
        h = torch.randn(1, H)
        t2 = time.time()
        oracle.linear(h, w["lm_head"], norm_weights=w["norm"], eps=cfg["eps"], out_dtype=torch.float32)
        t3 = time.time()
        t_head += t3 - t2
        t_layers += (t1 - t0) - (t3 - t2)  # forward() includes one lm_head
        done += 1
        if time.time() - t_start > seconds_budget:
            break
    per_layer = max(t_layers / done, 1e-9) / sample_layers
    per_token = per_layer * cfg["layers"] + t_head / done
    return {"value": 1.0 / per_token, "unit": "tokens/s", "cores": threads, "kind": "port",
            "sample": f"{sample_layers} of {cfg['layers']} decoder layers + lm_head, {done} decode tokens, fp32 PyTorch "
                      f"CPU oracle; layer time scaled to {cfg['layers']} layers"}


WORKLOAD = ("Llama-3.1-8B-arch decode (BASELINE config 3): 32 layers, hidden 4096, 32q/8kv heads, head_dim 128, "
            "intermediate 14336, vocab 128256, bs=1, 16-token prompt, static KV cache 4096")


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = LLAMA31_8B
    t0 = time.time()
    res = cpu_decode_sample(cfg, seconds_budget=60.0, sample_layers=2, tokens=max(1, args.steps))
    v = res["value"]
    line = {
        "impl": "reference", "metric": "bs=1 decode tokens/s/user (Llama-3-8B arch)", "value": v, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 / v,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "global_batch": 1, "seq_len": f"{PROMPT_LEN}..{PROMPT_LEN + max(1, args.steps)}",
                   "parallelism": "host cores (PyTorch fp32 restatement of the path; the reference's own kernels are "
                                  "HIP-only and cannot be built here)"},
        "cpu_baseline": res,
        "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "wall_s": time.time() - t0,
    }
    print(json.dumps(line), flush=True)


def run_gpu(args):
    import torch
    import torch.distributed as dist

    from benchmarks.parity import tp_parity
    from muillm_b200 import capi
    from muillm_b200.comm import MuiCommunicator
    from muillm_b200.decoder_stack import LlamaDecodeStack, shard_llama_weights

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    cfg = LLAMA31_8B
    dtype = torch.float16
    flags = capi.MUI_FLAG_PDL
    K, W = args.steps, max(3, args.warmup)
    w = make_gpu_weights(cfg, dtype, dev, seed=0)
    comm = None
    local_cfg = cfg
    full_w = None
    if world > 1:
        # tensor parallelism: every rank builds the same seeded weights and keeps its shard
        comm = MuiCommunicator(rank=rank, world_size=world, key="bench" + os.environ.get("MASTER_PORT", "0"),
                               capacity_elems=1 << 16)
        full_w = w if rank == 0 else None  # rank 0 keeps the un-sharded weights until the parity check is done
        w, local_cfg = shard_llama_weights(w, cfg, rank, world)
        torch.cuda.empty_cache()
    stack = LlamaDecodeStack(w, local_cfg, max_seq=MAX_SEQ, batch=1, max_new_tokens=max(PROMPT_LEN + W + K, 48) + 8,
                             flags=flags, comm=comm)
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, cfg["vocab"], (1, PROMPT_LEN), generator=g)
    parity = None
    if world > 1:
        parity = tp_parity(stack, lambda: LlamaDecodeStack(full_w, cfg, max_seq=256, batch=1, max_new_tokens=64,
                                                           flags=flags), prompt, rank, dev)
        full_w = None
        torch.cuda.empty_cache()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    stream = torch.cuda.Stream()
    # ---- device-resident loop: prompt token by token, W warm-up steps, then K timed graph replays ----
    with torch.cuda.stream(stream):
        stack.reset(0)
        stack.prefill(prompt)
        stack.capture()
        stack.replay(W)
    barrier()
    with ClockSampler(local_rank) as clocks:
        s_ev, e_ev = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            s_ev.record(stream)
            stack.replay(K)
            e_ev.record(stream)
        barrier()
        dev_seconds = s_ev.elapsed_time(e_ev) * 1e-3
        # ---- end-to-end loop: host feeds the token (pinned H2D), reads the arg-max back (D2H) every step ----
        tok_in = torch.zeros(1, dtype=torch.int64).pin_memory()
        tok_out = torch.zeros(1, dtype=torch.int64).pin_memory()
        with torch.cuda.stream(stream):
            stack.reset(0)
            stack.prefill(prompt)
            stack.capture()
            nxt = stack.next_tokens()
            tok_out.copy_(nxt, non_blocking=True)
            stream.synchronize()
            for _ in range(W):
                tok_in.copy_(tok_out)
                stack.set_tokens(tok_in)
                stack.replay(1)
                tok_out.copy_(nxt, non_blocking=True)
                stream.synchronize()
        barrier()
        t0 = time.perf_counter()
        with torch.cuda.stream(stream):
            for _ in range(K):
                tok_in.copy_(tok_out)
                stack.set_tokens(tok_in)
                stack.replay(1)
                tok_out.copy_(nxt, non_blocking=True)
                stream.synchronize()
        barrier()
        e2e_seconds = time.perf_counter() - t0
    plugin_tok_s, plugin_error = None, None
    if world == 1:
        try:
            with torch.cuda.stream(stream):
                plugin_tok_s = time_plugin_e2e(w, cfg, prompt, K, W, MAX_SEQ)
        except Exception as e:  # the headline numbers above do not depend on this leg: report it instead of dying
            plugin_error = f"{type(e).__name__}: {e}"
    long_ctx = None
    if world == 1:
        # the same decode step with ~4000 tokens already in the KV cache (rows of zeros: timing only): the stack
        # then runs the token-split attention kernel instead of the short-context one
        try:
            S0, steps_long = MAX_SEQ - 96, 32
            with torch.cuda.stream(stream):
                long_stack = LlamaDecodeStack(w, cfg, max_seq=MAX_SEQ, batch=1, max_new_tokens=64, flags=flags)
                long_stack.reset(S0)
                long_stack.set_tokens(prompt[:, 0].contiguous())
                long_stack.capture()
                long_stack.replay(8)
                ls, le = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                ls.record(stream)
                long_stack.replay(steps_long)
                le.record(stream)
            torch.cuda.synchronize()
            sec = ls.elapsed_time(le) * 1e-3 / steps_long
            long_ctx = {"S": f"{S0 + 8}..{S0 + 8 + steps_long}", "tokens_per_s": 1.0 / sec, "ms_per_step": sec * 1e3,
                        "kv_bytes_per_step": kv_bytes_per_token(cfg, S0 + 8 + steps_long // 2)}
            del long_stack
        except Exception as e:
            long_ctx = {"error": f"{type(e).__name__}: {e}"}
    with torch.cuda.stream(stream):
        k_seconds, k_bytes = time_dominant_kernel(w, local_cfg, flags)
    status = capi.device_status()
    if comm is not None:
        barrier()

    t = torch.tensor([dev_seconds, e2e_seconds], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_seconds, e2e_seconds = t.tolist()
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # one user; with N > 1 the model is sharded N ways (tensor parallelism, two fused all-reduces per layer)
    users = 1
    value = users * K / dev_seconds
    e2e_value = users * K / e2e_seconds
    peak, peak_kind = measured_peak_gbs()
    achieved = k_bytes / k_seconds / 1e9
    seq_mid = PROMPT_LEN + W + K // 2
    # bytes one GPU streams per step: its 1/world shard of the weights and of the KV cache
    step_bytes = (weight_bytes_per_token(cfg) + kv_bytes_per_token(cfg, seq_mid)) // world
    cpu = cpu_decode_sample(cfg) if not args.no_cpu_baseline else None
    line = {
        "metric": "bs=1 decode tokens/s/user (Llama-3-8B arch)",
        "value": value, "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": dev_seconds / K * 1e3, "higher_is_better": True,
        "scaling": "strong",
        "vs_baseline": (value / BASELINE_TOK_S[world]) if world in BASELINE_TOK_S else None,
        "dtype": "f16", "data": "synthetic",
        "config": {"workload": WORKLOAD,
                   "global_batch": users, "seq_len": f"{PROMPT_LEN + W}..{PROMPT_LEN + W + K}",
                   "parallelism": "single GPU" if world == 1 else f"tp{world} (sharded QKV/o_proj/MLP/lm_head, "
                                                                    f"GEMV + all-reduce fused over NVLink peer stores)",
                   "l2": "every step streams 15.0 GB of weights, far above the 126 MB L2 (no flush needed)",
                   "launch": "CUDA graph of one decode step replayed K times, programmatic dependent launch"},
        "hbm_fraction": {"bytes_per_step": step_bytes, "achieved_gbs": step_bytes * K / dev_seconds / 1e9,
                         "of_measured_peak": step_bytes * K / dev_seconds / 1e9 / peak,
                         "of_nominal_8tbs": step_bytes * K / dev_seconds / 1e9 / NOMINAL_HBM_GBS},
        "roofline": {"bound": "hbm", "kernel": f"gemv_pipe_kernel<half, NB=1, gate/up+SiLU> "
                                               f"(I={local_cfg['intermediate']}, H=4096)",
                     "achieved": achieved, "peak": peak, "peak_source": peak_kind, "unit": "GB/s",
                     "frac": achieved / peak, "traffic": GATEUP_DRAM_TRAFFIC_BYTES if world == 1 else None,
                     "algorithmic_bytes": k_bytes, "avg_launch_us": k_seconds * 1e6,
                     "timing": "CUDA graph of back-to-back launches over the layers' distinct weights"},
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": 8, "d2h_bytes_per_step": 8},
        "gpu_launches": K * stack.launches_per_step,
        "clocks": clocks.summary(),
        "device_status": status,
    }
    if cpu is not None:
        line["cpu_baseline"] = cpu
    if plugin_tok_s is not None:
        # the same metric through the muillm_ext module handles the reference's Python would call (one decoder-stack
        # call per token, lm_head and arg-max issued from Python): what a drop-in user of the reference gets
        line["e2e_plugin"] = {"value": plugin_tok_s, "unit": "tokens/s", "api": "muillm_ext module handles",
                              "h2d_bytes_per_step": 16, "d2h_bytes_per_step": 8}
    elif plugin_error is not None:
        line["e2e_plugin"] = {"error": plugin_error}
    if long_ctx is not None:
        line["long_context"] = long_ctx
    if parity is not None:
        line["parity"] = parity
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# dram__bytes_read.sum + dram__bytes_write.sum of one gate/up launch at the single-GPU shape (14336 x 4096 x 2, fp16),
# mean of the two launches of an `ncu --set full` capture of this kernel
GATEUP_DRAM_TRAFFIC_BYTES = 238540416


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
