"""Host cost of one call through the Python layers above the C ABI (`python -m benchmarks.call_overhead`):

  * a ctypes call that does nothing on the device (mui_version);
  * ops.muillm_linear_forward on a tiny GEMV (argument checks, output allocation by torch, ctypes marshalling, one
    kernel launch), issued back to back without synchronising — the per-call host time a per-layer Python loop pays;
  * one decode step of the C decode stack (mui_llama_stack_step: 13 launches for a 2-layer model) and one CUDA-graph
    replay of it, for the cost per launch once the loop is in C.
A compiled pybind11 module would save the ctypes marshalling of the first two lines; the decode loop itself makes one
call per token, so that saving is a fraction of a microsecond per token."""
import json
import time

import torch

from muillm_b200 import capi, ops
from muillm_b200.decoder_stack import LlamaDecodeStack


def _per_call(fn, n):
    fn()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(n):
        fn()
    dt = time.perf_counter() - t0
    torch.cuda.synchronize()
    return dt / n * 1e6


def main():
    dev = torch.device("cuda", 0)
    lib = capi.lib()
    x = torch.randn(1, 256, device=dev, dtype=torch.float16)
    w = torch.randn(64, 256, device=dev, dtype=torch.float16)
    out = torch.empty(1, 64, device=dev, dtype=torch.float16)
    cfg = dict(layers=2, hidden=256, intermediate=512, heads=2, kv_heads=1, head_dim=128, vocab=512, eps=1e-5,
               rope_theta=500000.0)
    g = torch.Generator(device=dev).manual_seed(0)
    ws = {"embed": torch.randn(512, 256, device=dev, generator=g).half(), "lm_head": torch.randn(512, 256, device=dev, generator=g).half(),
          "norm": torch.ones(256, device=dev).half(),
          "qkv": [torch.randn(512, 256, device=dev, generator=g).half() * 0.05 for _ in range(2)],
          "o": [torch.randn(256, 256, device=dev, generator=g).half() * 0.05 for _ in range(2)],
          "gate": [torch.randn(512, 256, device=dev, generator=g).half() * 0.05 for _ in range(2)],
          "up": [torch.randn(512, 256, device=dev, generator=g).half() * 0.05 for _ in range(2)],
          "down": [torch.randn(256, 512, device=dev, generator=g).half() * 0.05 for _ in range(2)],
          "ln1": [torch.ones(256, device=dev).half() for _ in range(2)], "ln2": [torch.ones(256, device=dev).half() for _ in range(2)]}
    stack = LlamaDecodeStack(ws, cfg, max_seq=4096, batch=1, max_new_tokens=4000, flags=capi.MUI_FLAG_PDL)
    res = {"ctypes_noop_us": _per_call(lib.mui_version, 20000),
           "ops_linear_forward_us": _per_call(lambda: ops.muillm_linear_forward(None, x, w), 3000),
           "ops_linear_forward_preallocated_us": _per_call(lambda: ops.muillm_linear_forward(None, x, w, out=out), 3000)}
    stack.reset(0)
    res["c_stack_step_13_launches_us"] = _per_call(stack.step, 1000)
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        stack.reset(0)
        stack.capture()
        res["c_stack_graph_replay_us"] = _per_call(lambda: stack.replay(1), 1000)
    torch.cuda.synchronize()
    print(json.dumps(res))


if __name__ == "__main__":
    main()
