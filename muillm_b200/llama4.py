"""Batch-1 decode of a Llama-4 text model (MoE with a shared expert and top-k sigmoid routing, chunked attention in
the rope layers, full attention with temperature tuning in the no-rope layers) as a chain of the library's kernels:
the per-token path the reference runs through MuiLLMParallelLlama4DecoderStack
(csrc/modules/parallel_llama4_decoder_stack.cpp, parallel_llama4_decoder_module.cpp:25-66,
parallel_llama4_attention_module.cpp:45-134, parallel_gateupmoe_module.cpp).

Per layer and token, six launches:
  fused RMSNorm -> QKV GEMV; rope / QK L2 norm / temperature scale (one launch); K/V row written into a static cache;
  flash decoding over the rows the layer may see; o_proj GEMV + residual; fused RMSNorm -> router GEMV; top-k sigmoid;
  MoE gate/up+SiLU over the shared and the selected experts; expert down projections summed + residual.
Chunked attention needs neither a ring buffer nor a mask here: every layer keeps a plain [1, Hkv, max_seq, D] cache and
a chunked layer hands flash decoding the strided view of the rows of the current chunk.

`Llama4DecodeRunner` makes one Python call per launch (kept as the kernel-by-kernel cross-check); `Llama4DecodeStack`
runs the whole step as one call into the C decode stack (mui_llama4_stack_*): six launches per layer, ring caches for
the chunked layers, token and position on the device, replayable as a CUDA graph.
"""
import ctypes
import math
from ctypes import c_int, c_void_p

import torch

from . import capi, ops
from .decoder_stack import LlamaDecodeStack


def llama4_config_from_hf(c):
    """dict for Llama4DecodeRunner from a transformers Llama4TextConfig (or an object with the same attributes)."""
    theta = getattr(c, "rope_theta", None)
    if theta is None:
        theta = (getattr(c, "rope_parameters", None) or {}).get("rope_theta", 500000.0)
    return dict(layers=c.num_hidden_layers, hidden=c.hidden_size, expert_intermediate=c.intermediate_size,
                heads=c.num_attention_heads, kv_heads=c.num_key_value_heads, head_dim=c.head_dim, vocab=c.vocab_size,
                experts=c.num_local_experts, top_k=c.num_experts_per_tok, eps=c.rms_norm_eps, rope_theta=float(theta),
                chunk=c.attention_chunk_size, use_rope=[bool(v) for v in c.no_rope_layers],
                use_qk_norm=bool(c.use_qk_norm), temperature_tuning=bool(c.attn_temperature_tuning),
                attn_scale=float(c.attn_scale), floor_scale=float(c.floor_scale))


def llama4_weights_from_state_dict(sd, cfg, dtype=torch.bfloat16, device="cuda"):
    """HF parameter names -> the packed layout the kernels stream: q, k, v rows concatenated; gate and up rows of the
    shared expert followed by those of every routed expert ([(1+E)*I, H]); down matrices stacked the same way
    ([(1+E)*H, I]). HF stores the routed experts transposed and gate|up fused ([E, H, 2I] and [E, I, H]); they are
    split and transposed once here (muillm/modules/moe/gateupdownmlpmoe.py does the same at replacement time)."""

    def t(name):
        return torch.as_tensor(sd[name]).to(device=device, dtype=dtype).contiguous()

    I = cfg["expert_intermediate"]
    lm_head = "lm_head.weight" if "lm_head.weight" in sd else "model.embed_tokens.weight"
    w = {"embed": t("model.embed_tokens.weight"), "lm_head": t(lm_head), "norm": t("model.norm.weight"),
         "qkv": [], "o": [], "router": [], "gate": [], "up": [], "down": [], "ln1": [], "ln2": []}
    for l in range(cfg["layers"]):
        p = f"model.layers.{l}."
        w["qkv"].append(torch.cat([t(p + "self_attn.q_proj.weight"), t(p + "self_attn.k_proj.weight"),
                                   t(p + "self_attn.v_proj.weight")], dim=0).contiguous())
        w["o"].append(t(p + "self_attn.o_proj.weight"))
        w["ln1"].append(t(p + "input_layernorm.weight"))
        w["ln2"].append(t(p + "post_attention_layernorm.weight"))
        w["router"].append(t(p + "feed_forward.router.weight"))
        gu = t(p + "feed_forward.experts.gate_up_proj")          # [E, H, 2I]
        dn = t(p + "feed_forward.experts.down_proj")             # [E, I, H]
        gates = [t(p + "feed_forward.shared_expert.gate_proj.weight")]
        ups = [t(p + "feed_forward.shared_expert.up_proj.weight")]
        downs = [t(p + "feed_forward.shared_expert.down_proj.weight")]
        for e in range(cfg["experts"]):
            gates.append(gu[e, :, :I].t())
            ups.append(gu[e, :, I:].t())
            downs.append(dn[e].t())
        w["gate"].append(torch.cat(gates, dim=0).contiguous())
        w["up"].append(torch.cat(ups, dim=0).contiguous())
        w["down"].append(torch.cat(downs, dim=0).contiguous())
    return w


def shard_llama4_weights(w, cfg, rank, world, shard_lm_head=False):
    """Tensor-parallel shard of packed Llama-4 weights, partitioned as the reference does
    (muillm/modules/parallelmultilinear.py:340-387, muillm/modules/moe/parallelgateupdownmlpmoe.py): whole query / KV
    heads per rank, o_proj by input columns, every expert's intermediate dimension split across the ranks; embedding,
    router and norms replicated, the lm_head replicated or split by rows. Returns (weights, per-rank cfg)."""
    Hq, Hkv, D, H = cfg["heads"], cfg["kv_heads"], cfg["head_dim"], cfg["hidden"]
    I, E = cfg["expert_intermediate"], cfg["experts"] + 1
    if Hq % world or Hkv % world or I % world:
        raise RuntimeError("heads, KV heads and the expert intermediate size must be divisible by the world size")
    hq, hkv, il = Hq // world, Hkv // world, I // world
    out = {k: w[k] for k in ("embed", "lm_head", "norm", "router", "ln1", "ln2")}
    out.update(qkv=[], o=[], gate=[], up=[], down=[])
    for l in range(cfg["layers"]):
        qkv = w["qkv"][l]
        q, k, v = qkv[: Hq * D], qkv[Hq * D: (Hq + Hkv) * D], qkv[(Hq + Hkv) * D:]
        out["qkv"].append(torch.cat([q[rank * hq * D: (rank + 1) * hq * D], k[rank * hkv * D: (rank + 1) * hkv * D],
                                     v[rank * hkv * D: (rank + 1) * hkv * D]], dim=0).contiguous())
        out["o"].append(w["o"][l][:, rank * hq * D: (rank + 1) * hq * D].contiguous())
        sl = slice(rank * il, (rank + 1) * il)
        out["gate"].append(w["gate"][l].view(E, I, H)[:, sl].reshape(E * il, H).contiguous())
        out["up"].append(w["up"][l].view(E, I, H)[:, sl].reshape(E * il, H).contiguous())
        out["down"].append(w["down"][l].view(E, H, I)[:, :, sl].reshape(E * H, il).contiguous())
    local = dict(cfg)
    local.update(heads=hq, kv_heads=hkv, expert_intermediate=il, world=world, rank=rank)
    if shard_lm_head:
        # rows of the head per rank and a distributed arg-max (Llama4DecodeRunner._argmax) instead of full logits
        V = cfg["vocab"]
        if V % world:
            raise RuntimeError("the vocabulary must be divisible by the world size to shard the lm_head")
        out["lm_head"] = w["lm_head"][rank * (V // world): (rank + 1) * (V // world)].contiguous()
        local.update(lm_head_sharded=True, vocab_offset=rank * (V // world))
    return out, local


class Llama4DecodeRunner:
    """Greedy batch-1 decoding of a Llama-4 text model over the packed weights of llama4_weights_from_state_dict."""

    def __init__(self, weights, cfg, max_seq, flags=0, comm=None):
        """With `comm` (a MuiCommunicator of more than one rank) weights and cfg are this rank's shard
        (shard_llama4_weights): o_proj and the expert down projections end in the fused all-reduce."""
        self.w, self.cfg, self.max_seq, self.flags = weights, dict(cfg), max_seq, flags
        self.comm = comm
        dev, dt = weights["embed"].device, weights["embed"].dtype
        self.device, self.dtype = dev, dt
        Hkv, D = cfg["kv_heads"], cfg["head_dim"]
        self.k_cache = [torch.zeros(1, Hkv, max_seq, D, dtype=dt, device=dev) for _ in range(cfg["layers"])]
        self.v_cache = [torch.zeros(1, Hkv, max_seq, D, dtype=dt, device=dev) for _ in range(cfg["layers"])]
        # interleaved-pair rotation angles per position, as (cos, sin) pairs: what HF's Llama4TextRotaryEmbedding
        # returns as complex numbers (freqs_cis)
        inv = 1.0 / (cfg["rope_theta"] ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
        ang = torch.outer(torch.arange(max_seq, dtype=torch.float32), inv)
        self.freqs = torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).to(dev).contiguous()  # [max_seq, D/2, 2]
        self.pos = 0

    def reset(self):
        self.pos = 0

    def _layers(self, h, cache_position, pe, pos=None, seq_len_dev=None):
        """The decoder layers for one token. Host mode: `pos` is the python position (chunked layers attend a view of
        their chunk). Device mode (`pos` None): the attended length comes from the device int32 `seq_len_dev`, which is
        what lets a captured step replay; the caches must then not be longer than the attention chunk."""
        c, w, f = self.cfg, self.w, self.flags
        Hq, Hkv, D = c["heads"], c["kv_heads"], c["head_dim"]
        for l in range(c["layers"]):
            rope = c["use_rope"][l]
            qkv = ops.muillm_linear_forward(None, h, w["qkv"][l], norm_weights=w["ln1"][l], epsilon=c["eps"], flags=f)
            q = qkv[..., : Hq * D].view(1, Hq, 1, D)
            k = qkv[..., Hq * D: (Hq + Hkv) * D].view(1, Hkv, 1, D)
            v = qkv[..., (Hq + Hkv) * D:].view(1, Hkv, 1, D)
            tune = c["temperature_tuning"] and not rope
            norm = c["use_qk_norm"] and rope
            if rope or norm or tune:
                q, k = ops.llama4_qk_prologue(q, k, position_embeds=pe if rope else None,
                                              qk_norm_eps=c["eps"] if norm else None,
                                              cache_position=cache_position if tune else None,
                                              attn_scale=c["attn_scale"], floor_scale=c["floor_scale"], flags=f)
            seen = self.max_seq if pos is None else pos + 1
            k_all, v_all = ops.muillm_static_kvcache_update(k, v, self.k_cache[l], self.v_cache[l], cache_position,
                                                            seen, flags=f)
            if pos is not None and rope and c["chunk"]:
                # chunked attention: only the rows of the chunk the new token belongs to
                start = (pos // c["chunk"]) * c["chunk"]
                k_all, v_all = k_all.narrow(2, start, pos + 1 - start), v_all.narrow(2, start, pos + 1 - start)
            q = q if q.is_contiguous() else q.contiguous()
            attn = ops._flash_decode(q, k_all, v_all, None, flags=f, seq_len_dev=seq_len_dev)
            if self.comm is not None:
                h = self.comm.parallel_linear(attn, w["o"][l], residual=h, flags=f)
            else:
                h = ops.muillm_linear_forward(None, attn, w["o"][l], residual=h, flags=f)
            logits = ops.muillm_linear_forward(None, h, w["router"][l], norm_weights=w["ln2"][l], epsilon=c["eps"],
                                               flags=f)
            scores, idx = ops.muillm_topk_sigmoid_forward(logits, c["top_k"], flags=f)
            if self.comm is not None:
                h = self.comm.parallel_moe_mlp(1, c["experts"], w["ln2"][l], c["eps"], w["gate"][l], w["up"][l],
                                               w["down"][l], h, h, scores.reshape(-1), idx.reshape(-1), flags=f)
            else:
                h = ops.muillm_gateupsilumoe_forward(None, 1, c["experts"], w["ln2"][l], c["eps"], w["gate"][l],
                                                     w["up"][l], w["down"][l], h, h, scores.reshape(-1),
                                                     idx.reshape(-1), flags=f)
        # logits of this rank's rows of the lm_head (all of them unless the head was sharded)
        return ops.muillm_linear_forward(None, h, w["lm_head"], norm_weights=w["norm"], epsilon=c["eps"],
                                         flags=f).view(1, -1)

    def step(self, token):
        """One token (python int or 0-dim tensor) in, logits [1, vocab] (model dtype) out; advances the position."""
        c, w = self.cfg, self.w
        pos = self.pos
        if pos >= self.max_seq:
            raise RuntimeError("the static cache is full")
        tok = torch.as_tensor([int(token)], dtype=torch.int64, device=self.device)
        h = w["embed"].index_select(0, tok).view(1, 1, c["hidden"])
        cache_position = torch.tensor([pos], dtype=torch.int64, device=self.device)
        pe = self.freqs[pos: pos + 1].unsqueeze(0)   # [1, 1, D/2, 2]
        logits = self._layers(h, cache_position, pe, pos=pos)
        self.pos = pos + 1
        return logits

    # ---- device-resident loop: token, position and attended length live on the GPU, so a step can be captured ----
    def _argmax(self, logits):
        """Next token from this rank's logits; with a row-sharded lm_head the ranks exchange their (max, index) pairs
        through one small fp32 all-reduce (each rank fills only its own slot) and pick the same winner."""
        lf = logits.float().view(-1)
        val, idx = torch.max(lf, dim=0)
        off = int(self.cfg.get("vocab_offset", 0))
        if self.comm is None or not self.cfg.get("lm_head_sharded", False):
            return (idx + off).view(1)
        world, rank = self.cfg["world"], self.cfg["rank"]
        mine = torch.zeros(world, 2, dtype=torch.float32, device=self.device)
        mine[rank, 0] = val
        mine[rank, 1] = (idx + off).float()          # vocabulary indices are exact in fp32 (< 2**24)
        allp = self.comm.all_reduce_sum(mine)
        win = torch.argmax(allp[:, 0])                # ties go to the lower rank, i.e. the lower index
        return allp[:, 1].index_select(0, win.view(1)).long()   # no host round trip: the step stays capturable

    def start_device_loop(self, token, pos):
        """Puts the decode state on the device: the next step consumes `token` at position `pos`."""
        if self.cfg["chunk"] and self.max_seq > self.cfg["chunk"]:
            raise RuntimeError("the device loop needs caches no longer than the attention chunk")
        self.d_token = torch.tensor([int(token)], dtype=torch.int64, device=self.device)
        self.d_pos = torch.tensor([int(pos)], dtype=torch.int64, device=self.device)
        self.d_len = torch.tensor([int(pos) + 1], dtype=torch.int32, device=self.device)
        self.pos = None
        self._graph = None

    def step_device(self):
        """One decode step entirely from device state; leaves the arg-max token as the next input."""
        c, w = self.cfg, self.w
        h = w["embed"].index_select(0, self.d_token).view(1, 1, c["hidden"])
        pe = self.freqs.index_select(0, self.d_pos).unsqueeze(0)
        logits = self._layers(h, self.d_pos, pe, pos=None, seq_len_dev=self.d_len)
        self.d_token.copy_(self._argmax(logits))
        self.d_pos.add_(1)
        self.d_len.add_(1)

    def capture(self, warmup=2):
        """Captures step_device as a CUDA graph on a side stream (after `warmup` eager steps there, which also
        create the per-stream workspaces); replay(n) then runs n steps without host work per launch."""
        self._stream = torch.cuda.Stream()
        self._stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self._stream):
            for _ in range(warmup):
                self.step_device()
        self._stream.synchronize()
        self._graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self._graph, stream=self._stream):
            self.step_device()
        return self

    def replay(self, steps=1):
        for _ in range(steps):
            self._graph.replay()

    def greedy(self, prompt, new_tokens):
        """prompt: 1-D int64 tensor; returns the new_tokens greedy continuation (int64, device)."""
        self.reset()
        logits = None
        for t in prompt.reshape(-1).tolist():
            logits = self.step(t)
        out = []
        for _ in range(new_tokens):
            nxt = int(torch.argmax(logits.float(), dim=-1).item())
            out.append(nxt)
            if len(out) < new_tokens:
                logits = self.step(nxt)
        return torch.tensor(out, dtype=torch.int64, device=self.device)


def llama4_freqs(max_pos, head_dim, theta, device):
    """[max_pos, head_dim/2, 2] fp32 (cos, sin) of the interleaved-pair rotation angles: what HF's
    Llama4TextRotaryEmbedding returns as complex numbers (freqs_cis)."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    ang = torch.outer(torch.arange(max_pos, dtype=torch.float32), inv)
    return torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).to(device).contiguous()


class Llama4DecodeStack(LlamaDecodeStack):
    """Greedy batch-1 decoding of a Llama-4 text model through the C decode stack: same weights dict and cfg as
    Llama4DecodeRunner (packed experts, shared expert first; with `comm` this rank's shard from
    shard_llama4_weights(..., shard_lm_head=True) or llama4_bench.local_weights). The methods of LlamaDecodeStack
    (reset, set_tokens, step, capture, replay, prefill, greedy, logits, next_tokens) apply unchanged.

    The per-token path the reference runs through MuiLLMParallelLlama4DecoderStack
    (csrc/modules/parallel_llama4_decoder_stack.cpp:18-60)."""

    def __init__(self, weights, cfg, max_seq, max_new_tokens=4096, flags=0, comm=None):
        self.lib = capi.lib()
        self.cfg = dict(cfg)
        self.w = weights
        dev, dt = weights["embed"].device, weights["embed"].dtype
        self.device, self.dtype = dev, dt
        self.batch, self.max_seq, self.flags = 1, max_seq, flags
        L, Hkv, D = cfg["layers"], cfg["kv_heads"], cfg["head_dim"]
        c = capi.Llama4Config(
            capi.MUI_F16 if dt == torch.float16 else capi.MUI_BF16, L, cfg["hidden"], cfg["expert_intermediate"],
            cfg["heads"], Hkv, D, weights["lm_head"].shape[0], max_seq, int(cfg.get("chunk") or 0), cfg["experts"],
            cfg["top_k"], 1, float(cfg["eps"]), 1.0 / math.sqrt(D), int(bool(cfg["use_qk_norm"])),
            int(bool(cfg["temperature_tuning"])), float(cfg["attn_scale"]), float(cfg["floor_scale"]),
            int(weights["embed"].shape[0]) if comm is not None else 0, int(cfg.get("vocab_offset", 0)))
        self._c = c
        self.cfg["vocab"] = int(weights["lm_head"].shape[0])  # rows of this rank's lm_head (logits view)
        use_rope = [int(bool(v)) for v in cfg["use_rope"]]
        rows = [self.lib.mui_llama4_stack_cache_rows(ctypes.byref(c), r) for r in use_rope]
        self.k_cache = [torch.zeros(1, Hkv, n, D, dtype=dt, device=dev) for n in rows]
        self.v_cache = [torch.zeros(1, Hkv, n, D, dtype=dt, device=dev) for n in rows]
        self.freqs = llama4_freqs(max_seq, D, cfg["rope_theta"], dev)
        nbytes = self.lib.mui_llama4_stack_scratch_bytes(ctypes.byref(c))
        if nbytes == 0:
            raise RuntimeError("muillm_b200: " + self.lib.mui_last_error().decode())
        self.scratch = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
        self.out_tokens = torch.zeros(max_new_tokens, 1, dtype=torch.int64, device=dev)

        def arr(tensors):
            for t in tensors:
                assert t.is_cuda and t.is_contiguous() and t.dtype == dt
            return (c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])

        self._arrays = {k: arr(weights[k]) for k in ("qkv", "o", "router", "gate", "up", "down", "ln1", "ln2")}
        self._arrays["k_cache"] = arr(self.k_cache)
        self._arrays["v_cache"] = arr(self.v_cache)
        self._use_rope = (c_int * L)(*use_rope)
        w = capi.Llama4Weights(
            weights["embed"].data_ptr(), weights["norm"].data_ptr(), weights["lm_head"].data_ptr(),
            self.freqs.data_ptr(), self._use_rope,
            self._arrays["qkv"], self._arrays["o"], self._arrays["router"], self._arrays["gate"], self._arrays["up"],
            self._arrays["down"], self._arrays["ln1"], self._arrays["ln2"], self._arrays["k_cache"],
            self._arrays["v_cache"])
        h = c_void_p()
        capi.check(self.lib.mui_llama4_stack_create(ctypes.byref(c), ctypes.byref(w), self.scratch.data_ptr(),
                                                    self.scratch.numel(), ctypes.byref(h)))
        self._h = h
        self._captured = False
        self.comm = comm
        if comm is not None:
            capi.check(self.lib.mui_llama_stack_set_comm(h, comm.handle))
        self.reset(0)

    def router_state(self):
        """Views of the last step's router outputs: logits [layers, experts] (fp32) and chosen experts
        [layers, top_k] (int64)."""
        lp, ip = c_void_p(), c_void_p()
        capi.check(self.lib.mui_llama4_stack_router_state(self._h, ctypes.byref(lp), ctypes.byref(ip)))
        L, E = self.cfg["layers"], self.cfg["experts"]
        lo = lp.value - self.scratch.data_ptr()
        io = ip.value - self.scratch.data_ptr()
        logits = self.scratch[lo: lo + 4 * L * E].view(torch.float32).view(L, E)
        idx = self.scratch[io: io + 8 * L * 8].view(torch.int64).view(L, 8)[:, : self.cfg["top_k"]]
        return logits, idx

    @property
    def launches_per_step(self):
        """embedding, per layer {QKV, attention, o_proj, router + top-k, expert gate/up, expert down}, lm_head,
        arg-max; head dims other than 128 run the attention as prologue + cache write + flash decoding."""
        fused = self.cfg["head_dim"] == 128 and not (self.flags & capi.MUI_FLAG_FORCE_GENERIC)
        return 3 + (6 if fused else 8) * self.cfg["layers"]
