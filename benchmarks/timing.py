"""Timing helpers shared by the benchmarks: CUDA graphs of back-to-back launches timed with CUDA events."""
import torch


def time_graph(fns, iters_per_graph, replays=5, warm_replays=3, sync=None):
    """fns: callables (e.g. one per weight set); the graph holds `iters_per_graph` launches cycling through them.
    Returns seconds per launch of `replays` timed replays after `warm_replays` untimed ones. `sync` (optional) is
    called right before the timed region (e.g. a barrier between ranks)."""
    n = len(fns)
    for i in range(n):
        fns[i]()
    torch.cuda.synchronize()
    st = torch.cuda.Stream()
    gr = torch.cuda.CUDAGraph()
    with torch.cuda.stream(st):
        with torch.cuda.graph(gr, stream=st, capture_error_mode="thread_local"):
            for i in range(iters_per_graph):
                fns[i % n]()
    for _ in range(warm_replays):
        gr.replay()
    torch.cuda.synchronize()
    if sync is not None:
        sync()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(replays):
        gr.replay()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) * 1e-3 / (replays * iters_per_graph)


def read_trace(buf, n):
    """Decodes `n` launch-trace records (mui_trace_enable) from the uint8/int64 device buffer `buf` into a list of
    dicts of ns values: start, end, past_wait, staged, pushed, all_seen, first_seen (None where not written)."""
    words = buf.view(torch.int64).cpu().view(-1, 8)[:n]
    out = []
    for r in words.tolist():
        def plain(v):
            return None if v == -1 else v

        def comp(v):
            return None if v == -1 else (~v) & 0xFFFFFFFFFFFFFFFF
        out.append({"start": plain(r[0]), "end": comp(r[1]), "past_wait": plain(r[2]), "staged": comp(r[3]),
                    "pushed": comp(r[4]), "all_seen": comp(r[5]), "first_seen": plain(r[6])})
    return out
