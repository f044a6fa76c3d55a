"""Latency of the one-shot all-reduce over NVLink peer stores, alone and fused into the GEMV epilogue, beside NCCL:

  python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
      -m benchmarks.comm_bench [--json out.json] [--trace]

Every figure is a CUDA graph of back-to-back launches with programmatic dependent launch, timed with CUDA events
after warm-up and a barrier, maximum over ranks, microseconds per launch:
  * `alone`  mui_comm_all_reduce_sum of n 16-bit elements (n = 4096, 5120, 8192 = the hidden sizes of the 8B, Scout
             and 70B architectures, and 65536);
  * `nccl`   torch.distributed.all_reduce (NCCL) of the same tensor, captured the same way;
  * `fused`  the K-sharded GEMV with the all-reduce in its epilogue (mui_parallel_linear_forward) and the same GEMV
             without the collective; `added` is their difference. Shapes: o_proj and down of the 8B and 70B
             architectures cut N ways along K.
--trace adds, per rank, the device-side timeline of the fused launches (median over launches): kernel start -> last
partial pushed -> first / last CTA that has every peer's partials -> kernel end.
"""
import argparse
import json
import os
import statistics

import torch
import torch.distributed as dist

from benchmarks.timing import read_trace, time_graph
from muillm_b200 import capi, ops
from muillm_b200.comm import MuiCommunicator


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--json", default=None)
    ap.add_argument("--trace", action="store_true")
    ap.add_argument("--iters", type=int, default=200)
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", device_id=dev)
    comm = MuiCommunicator(rank=rank, world_size=world, key="cb" + os.environ.get("MASTER_PORT", "0"),
                           capacity_elems=1 << 17)
    flags = capi.MUI_FLAG_PDL
    dtype = torch.bfloat16
    g = torch.Generator(device=dev).manual_seed(10 + rank)
    rows = []

    def sync():
        dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(sec):
        t = torch.tensor([sec], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    def report(row):
        rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)

    for n in (4096, 5120, 8192, 65536):
        src = torch.randn(1, n, device=dev, generator=g).to(dtype)
        dst = torch.empty_like(src)
        ours = max_over_ranks(time_graph([lambda: comm.all_reduce_sum(src, flags=flags, out=dst)], args.iters, sync=sync))
        buf = src.clone()
        nccl = max_over_ranks(time_graph([lambda: dist.all_reduce(buf)], args.iters, sync=sync))
        report({"case": "all-reduce alone", "elements": n, "dtype": "bf16", "gpus": world, "ours_us": ours * 1e6,
                "nccl_us": nccl * 1e6})

    shapes = [("8B o_proj", 4096, 4096), ("8B down", 4096, 14336), ("70B o_proj", 8192, 8192),
              ("70B down", 8192, 28672)]
    for name, N, Kt in shapes:
        K = Kt // world
        L = max(3, min(12, int(2.6e8 // (N * K * 2)) + 1))
        ws = [(torch.randn(N, K, device=dev, generator=g) * 0.02).to(dtype) for _ in range(L)]
        x = torch.randn(1, K, device=dev, generator=g).to(dtype)
        res = torch.randn(1, N, device=dev, generator=g).to(dtype)
        y = torch.empty(1, N, device=dev, dtype=dtype)
        fused = max_over_ranks(time_graph(
            [(lambda w=w: comm.parallel_linear(x, w, residual=res, flags=flags, out=y)) for w in ws], 4 * L, replays=10,
            sync=sync))
        plain = max_over_ranks(time_graph(
            [(lambda w=w: ops.muillm_linear_forward(None, x, w, residual=res, flags=flags, out=y)) for w in ws], 4 * L,
            replays=10, sync=sync))
        row = {"case": "GEMV + all-reduce, " + name, "N": N, "K_local": K, "gpus": world, "fused_us": fused * 1e6,
               "gemv_us": plain * 1e6, "added_us": (fused - plain) * 1e6}
        if args.trace:
            nrec = 4 * L
            tbuf = torch.empty(nrec * 64, dtype=torch.uint8, device=dev)
            st = torch.cuda.Stream()
            with torch.cuda.stream(st):
                capi.check(capi.lib().mui_trace_enable(st.cuda_stream, tbuf.data_ptr(), nrec))
                gr = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gr, stream=st):
                    for i in range(nrec):
                        comm.parallel_linear(x, ws[i % L], residual=res, flags=flags, out=y)
                capi.check(capi.lib().mui_trace_enable(None, None, 0))
                for _ in range(3):
                    tbuf.fill_(255)
                    gr.replay()
            torch.cuda.synchronize()
            recs = read_trace(tbuf, nrec)[2:]

            def med(f):
                vals = [f(r) for r in recs if None not in (r["start"], r["end"], r["pushed"], r["all_seen"], r["first_seen"])]
                return statistics.median(vals) / 1e3 if vals else None
            tl = {"kernel_us": med(lambda r: r["end"] - r["start"]),
                  "start_to_last_push_us": med(lambda r: r["pushed"] - r["start"]),
                  "last_push_to_first_cta_complete_us": med(lambda r: r["first_seen"] - r["pushed"]),
                  "last_push_to_last_cta_complete_us": med(lambda r: r["all_seen"] - r["pushed"]),
                  "last_cta_complete_to_end_us": med(lambda r: r["end"] - r["all_seen"])}
            gathered = [None] * world
            dist.all_gather_object(gathered, tl)
            row["timeline_per_rank"] = gathered
        report(row)
        del ws

    status = capi.device_status()
    sync()
    if rank == 0:
        if args.json:
            with open(args.json, "w") as f:
                json.dump({"gpus": world, "device_status": status, "rows": rows}, f, indent=1)
    comm.all_reduce_sum(torch.zeros(8, device=dev))
    torch.cuda.synchronize()
    sync()
    comm.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
