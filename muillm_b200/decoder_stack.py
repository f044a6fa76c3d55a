"""Host-side wrapper of the C decode stack (mui_llama_stack_*): owns the device tensors (weights, KV caches,
scratch, output tokens) through torch and drives prefill/greedy decoding.

It plays the role the reference gives to `_MuiParallelDecoderStack` + the model forward for q_len == 1
(muillm/modules/models/llama/model.py:332-357, muillm/modules/decoder/paralleldecoderstack.py): one call per
token instead of one Python dispatch per layer, here also for a single GPU and replayable from a CUDA graph.
"""
import ctypes
import math
from ctypes import c_int64, c_void_p

import torch

from . import capi


def rope_tables(max_pos, dim, theta, dtype, device):
    """cos/sin tables [max_pos, dim] of the default Llama RoPE, as HF's LlamaRotaryEmbedding computes them
    (fp32 math, cast to the model dtype; muillm/modules/attention/rotaryembedding.py:313-337)."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.int64).float() / dim))
    t = torch.arange(max_pos, dtype=torch.float32)
    freqs = torch.outer(t, inv_freq)
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(dtype).to(device), emb.sin().to(dtype).to(device)


def shard_llama_weights(weights, cfg, rank, world):
    """This rank's tensor-parallel shard of un-sharded Llama weights, and the per-rank config.

    QKV and gate/up are cut by output rows so that whole heads stay on a rank (q heads, then k heads, then v heads
    of the rank, concatenated — muillm/modules/parallelmultilinear.py:340-387), o_proj and down by input columns
    (muillm/modules/parallellinear.py:422-467), lm_head by rows; embedding and norms are replicated."""
    Hq, Hkv, D, I, V = cfg["heads"], cfg["kv_heads"], cfg["head_dim"], cfg["intermediate"], cfg["vocab"]
    if Hq % world or Hkv % world or I % world or V % world:
        raise RuntimeError("heads, kv_heads, intermediate and vocab must be divisible by the tensor-parallel degree")
    hq, hkv, il, vl = Hq // world, Hkv // world, I // world, V // world
    out = {"embed": weights["embed"], "norm": weights["norm"],
           "lm_head": weights["lm_head"][rank * vl:(rank + 1) * vl].contiguous(),
           "qkv": [], "o": [], "gate": [], "up": [], "down": [], "ln1": weights["ln1"], "ln2": weights["ln2"]}
    for l in range(cfg["layers"]):
        w = weights["qkv"][l]
        q = w[rank * hq * D:(rank + 1) * hq * D]
        k = w[Hq * D + rank * hkv * D: Hq * D + (rank + 1) * hkv * D]
        v = w[(Hq + Hkv) * D + rank * hkv * D: (Hq + Hkv) * D + (rank + 1) * hkv * D]
        out["qkv"].append(torch.cat([q, k, v], dim=0).contiguous())
        out["o"].append(weights["o"][l][:, rank * hq * D:(rank + 1) * hq * D].contiguous())
        out["gate"].append(weights["gate"][l][rank * il:(rank + 1) * il].contiguous())
        out["up"].append(weights["up"][l][rank * il:(rank + 1) * il].contiguous())
        out["down"].append(weights["down"][l][:, rank * il:(rank + 1) * il].contiguous())
    local = dict(cfg)
    local.update(heads=hq, kv_heads=hkv, intermediate=il, vocab=vl, embed_vocab=V, vocab_offset=rank * vl)
    return out, local


class LlamaDecodeStack:
    """weights: dict with 'embed', 'lm_head', 'norm' tensors and per-layer lists 'qkv', 'o', 'gate', 'up',
    'down', 'ln1', 'ln2' (CUDA, contiguous, fp16 or bf16). cfg: dict with layers, hidden, intermediate, heads,
    kv_heads, head_dim, vocab, eps, rope_theta."""

    def __init__(self, weights, cfg, max_seq, batch=1, max_new_tokens=4096, flags=0, comm=None):
        self.lib = capi.lib()
        self.cfg = dict(cfg)
        self.w = weights
        dev = weights["embed"].device
        dt = weights["embed"].dtype
        self.device, self.dtype = dev, dt
        self.batch, self.max_seq = batch, max_seq
        self.flags = flags
        L, Hkv, D = cfg["layers"], cfg["kv_heads"], cfg["head_dim"]
        for name in ("embed", "lm_head", "norm"):
            assert weights[name].is_cuda and weights[name].is_contiguous() and weights[name].dtype == dt
        self.k_cache = [torch.zeros(batch, Hkv, max_seq, D, dtype=dt, device=dev) for _ in range(L)]
        self.v_cache = [torch.zeros(batch, Hkv, max_seq, D, dtype=dt, device=dev) for _ in range(L)]
        self.cos, self.sin = rope_tables(max_seq, D, cfg["rope_theta"], dt, dev)
        c = capi.LlamaConfig(
            capi.MUI_F16 if dt == torch.float16 else capi.MUI_BF16, L, cfg["hidden"], cfg["intermediate"],
            cfg["heads"], Hkv, D, cfg["vocab"], max_seq, batch, float(cfg["eps"]), 1.0 / math.sqrt(D),
            int(cfg.get("embed_vocab", 0)), int(cfg.get("vocab_offset", 0)))
        self._c = c
        nbytes = self.lib.mui_llama_stack_scratch_bytes(ctypes.byref(c))
        if nbytes == 0:
            raise RuntimeError("muillm_b200: " + self.lib.mui_last_error().decode())
        self.scratch = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
        self.out_tokens = torch.zeros(max_new_tokens, batch, dtype=torch.int64, device=dev)

        def arr(tensors):
            for t in tensors:
                assert t.is_cuda and t.is_contiguous() and t.dtype == dt
            return (c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])

        self._arrays = {k: arr(weights[k]) for k in ("qkv", "o", "gate", "up", "down", "ln1", "ln2")}
        self._arrays["k_cache"] = arr(self.k_cache)
        self._arrays["v_cache"] = arr(self.v_cache)
        w = capi.LlamaWeights(
            weights["embed"].data_ptr(), weights["norm"].data_ptr(), weights["lm_head"].data_ptr(),
            self.cos.data_ptr(), self.sin.data_ptr(),
            self._arrays["qkv"], self._arrays["o"], self._arrays["gate"], self._arrays["up"], self._arrays["down"],
            self._arrays["ln1"], self._arrays["ln2"], self._arrays["k_cache"], self._arrays["v_cache"])
        h = c_void_p()
        capi.check(self.lib.mui_llama_stack_create(ctypes.byref(c), ctypes.byref(w), self.scratch.data_ptr(),
                                                   self.scratch.numel(), ctypes.byref(h)))
        self._h = h
        self._captured = False
        self.comm = comm  # keeps the communicator alive as long as the stack uses it
        if comm is not None:
            capi.check(self.lib.mui_llama_stack_set_comm(h, comm.handle))
        self.reset(0)

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            self.lib.mui_llama_stack_destroy(h)
            self._h = None

    def _stream(self):
        return torch.cuda.current_stream().cuda_stream

    def reset(self, position=0, position_ids=None):
        pid = None
        if position_ids is not None:
            pid = (c_int64 * self.batch)(*[int(p) for p in position_ids])
        capi.check(self.lib.mui_llama_stack_reset(self._h, self._stream(), int(position), pid,
                                                  self.out_tokens.data_ptr(), self.out_tokens.shape[0]))
        self._captured = False

    def set_tokens(self, tokens):
        """tokens: int64 tensor [batch] on the host (pinned or not) or on the device."""
        assert tokens.dtype == torch.int64 and tokens.numel() == self.batch
        capi.check(self.lib.mui_llama_stack_set_tokens(self._h, self._stream(), tokens.data_ptr(),
                                                       1 if tokens.is_cuda else 0))

    def set_position_ids(self, position_ids):
        """Per-sequence RoPE positions of the next step: int64 tensor [batch], host or device."""
        assert position_ids.dtype == torch.int64 and position_ids.numel() == self.batch
        capi.check(self.lib.mui_llama_stack_set_position_ids(self._h, self._stream(), position_ids.data_ptr(),
                                                             1 if position_ids.is_cuda else 0))

    def set_attention_mask(self, mask):
        """Additive mask [batch, max_seq] of the model dtype on the device (0 keeps a cache row, anything else drops
        it), applied by every layer's attention; None clears it. The stack keeps a reference to the tensor."""
        if mask is not None:
            assert mask.is_cuda and mask.is_contiguous() and mask.dtype == self.dtype
            assert tuple(mask.shape) == (self.batch, self.max_seq)
        self._mask = mask
        capi.check(self.lib.mui_llama_stack_set_attention_mask(self._h, mask.data_ptr() if mask is not None else None))
        self._captured = False

    def step(self):
        capi.check(self.lib.mui_llama_stack_step(self._h, self._stream(), self.flags))

    def capture(self):
        capi.check(self.lib.mui_llama_stack_capture(self._h, self._stream(), self.flags))
        self._captured = True

    def replay(self, steps=1):
        capi.check(self.lib.mui_llama_stack_replay(self._h, self._stream(), steps))

    def logits(self):
        """View of the last step's logits [batch, vocab] (model dtype)."""
        lp, sp = c_void_p(), c_void_p()
        capi.check(self.lib.mui_llama_stack_logits(self._h, ctypes.byref(lp), ctypes.byref(sp)))
        off = lp.value - self.scratch.data_ptr()
        n = self.batch * self.cfg["vocab"]
        return self.scratch[off: off + 2 * n].view(self.dtype).view(self.batch, self.cfg["vocab"])

    def state(self):
        """View of the int64 device state: [step, tokens in cache, cache position, position_ids[batch],
        next tokens[batch]]."""
        lp, sp = c_void_p(), c_void_p()
        capi.check(self.lib.mui_llama_stack_logits(self._h, ctypes.byref(lp), ctypes.byref(sp)))
        off = sp.value - self.scratch.data_ptr()
        n = 3 + 2 * self.batch
        return self.scratch[off: off + 8 * n].view(torch.int64)

    def next_tokens(self):
        """View of the tokens the next step will consume (the last step's arg-max), int64 [batch]."""
        return self.state()[3 + self.batch:]

    @property
    def launches_per_step(self):
        """Kernels one decode step launches: embedding, per layer {QKV, attention (one fused launch at head dim 128,
        else RoPE + flash decoding), o_proj, gate/up, down}, lm_head, arg-max."""
        fused = self.cfg["head_dim"] == 128 and not (self.flags & capi.MUI_FLAG_FORCE_GENERIC)
        return 3 + (5 if fused else 6) * self.cfg["layers"]

    def prefill(self, prompt):
        """Feeds prompt [batch, T] token by token through the decode step; the arg-max after the last prompt
        token is the first generated token (row 0 of out_tokens after reset counts steps, so callers read
        out_tokens[T-1])."""
        T = prompt.shape[1]
        for t in range(T):
            self.set_tokens(prompt[:, t].contiguous())
            self.step()

    def greedy(self, prompt, new_tokens, use_graph=True):
        """Greedy decoding: returns int64 [batch, new_tokens] (device)."""
        self.reset(0)
        T = prompt.shape[1]
        self.prefill(prompt)
        remaining = new_tokens - 1
        if remaining > 0:
            if use_graph:
                s = torch.cuda.Stream()
                s.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(s):
                    if not self._captured:
                        self.capture()
                    self.replay(remaining)
                torch.cuda.current_stream().wait_stream(s)
            else:
                for _ in range(remaining):
                    self.step()
        return self.out_tokens[T - 1: T - 1 + new_tokens].transpose(0, 1).contiguous()

    def greedy_ragged(self, prompts, new_tokens, use_graph=True, pad_token=0, timing=None):
        """Greedy decoding of `batch` prompts of different lengths (list of 1-D int64 tensors), left-padded to the
        longest one as the HF tokenizer hands them to the reference's generation loop: the padding rows of a sequence
        are masked out of its attention for good and its RoPE positions start at its first real token
        (position_ids = cumsum(attention_mask) - 1). Returns int64 [batch, new_tokens] (device). With a dict as
        `timing` (graph path), the CUDA-event time of the graph replays is left in timing["replay_seconds"] together
        with timing["replay_steps"]; `timing["warm_steps"]` of the new tokens run as untimed replays first."""
        assert len(prompts) == self.batch
        lens = [int(p.numel()) for p in prompts]
        T = max(lens)
        pads = torch.tensor([T - n for n in lens], dtype=torch.int64)
        padded = torch.full((self.batch, T), int(pad_token), dtype=torch.int64)
        for b, p in enumerate(prompts):
            padded[b, T - lens[b]:] = p.cpu()
        # a sequence's padding rows are dropped from the step of its first real token on; while it is still being
        # padded it attends its own padding (results unused), so no step ever has an empty attention set
        mask = torch.zeros(self.batch, self.max_seq, dtype=self.dtype, device=self.device)
        self.reset(0)
        self.set_attention_mask(mask)
        try:
            for t in range(T):
                for b in range(self.batch):
                    if t > 0 and int(pads[b]) == t:
                        mask[b, :t] = torch.finfo(self.dtype).min
                self.set_position_ids(torch.clamp(t - pads, min=0))
                self.set_tokens(padded[:, t].contiguous())
                self.step()
            remaining = new_tokens - 1
            if remaining > 0:
                if use_graph:
                    s = torch.cuda.Stream()
                    s.wait_stream(torch.cuda.current_stream())
                    with torch.cuda.stream(s):
                        self.capture()
                        warm = min(int(timing.get("warm_steps", 0)), remaining) if timing is not None else 0
                        if warm:
                            self.replay(warm)
                        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        if timing is not None and callable(timing.get("barrier")):
                            s.synchronize()
                            timing["barrier"]()
                        ev0.record(s)
                        self.replay(remaining - warm)
                        ev1.record(s)
                    torch.cuda.current_stream().wait_stream(s)
                    if timing is not None:
                        torch.cuda.synchronize()
                        timing["replay_seconds"] = ev0.elapsed_time(ev1) * 1e-3
                        timing["replay_steps"] = remaining - warm
                else:
                    for _ in range(remaining):
                        self.step()
            out = self.out_tokens[T - 1: T - 1 + new_tokens].transpose(0, 1).contiguous()
            torch.cuda.synchronize()
        finally:
            self.set_attention_mask(None)
        return out
