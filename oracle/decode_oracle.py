"""CPU oracle of the decode hot path — TEST INFRASTRUCTURE, not product code.

Plain PyTorch fp32 restatements of the algorithms the reference (Epliz/muiLLM) implements in its HIP
kernels, written against the HF/torch layer semantics the reference's own tests compare to. Only
tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import this module; nothing under
muillm_b200/ does.

Pinning: tests/golden/make_golden.py runs the importable parts of the reference itself
(muillm.quantization.rtnquantizer, the CPU branches of MuiRMSNorm / MuiGateUpDownMLP / the MoE fallback,
topk_sigmoid) and the HF modules the reference's tests use as expectations (LlamaRMSNorm, nn.Linear,
LlamaMLP, apply_rotary_pos_emb, eager attention, LlamaForCausalLM greedy generate) and stores their
outputs in tests/golden/*.npz; tests/test_oracle_golden.py checks every function here against them.
The reference stores no golden vectors of its own for this path, and its fused kernels (fused-norm
GEMV, flash decoding, RoPE write-out, all-reduce) have no test in the reference, so for those the HF
modules are the only pin.

All functions take/return CPU tensors. Inputs in fp16/bf16 are up-converted exactly; math is fp32 unless
noted; `out_dtype` rounds the result once at the end like the kernels do.
"""
import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F


# ---------------------------------------------------------------------------------------------------
# RMSNorm — HF semantics (transformers LlamaRMSNorm): fp32 variance, x*rsqrt(var+eps) rounded to the input
# dtype, then multiplied by the weight in the input dtype. The reference's kernels use eps/K instead of
# eps (csrc/linear/linear_fp16_kernels.cu:388-390,597; csrc/norm/rmsnorm_fp16_kernels.cu:49-51,101), a
# ~1e-5 relative deviation from HF that is not reproduced here.
# ---------------------------------------------------------------------------------------------------
def rmsnorm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    dt = x.dtype
    xf = x.float()
    var = xf.pow(2).mean(-1, keepdim=True)
    xn = (xf * torch.rsqrt(var + eps)).to(dt)
    if weight is None:
        return xn
    return (weight.float() * xn.float()).to(dt)


# ---------------------------------------------------------------------------------------------------
# Linear with fused norm / activation / biases / residual.
# Epilogue order follows csrc/linear/linear_fp16_kernels.cu:337-353: act -> *mul_bias -> +add_bias -> +residual.
# ---------------------------------------------------------------------------------------------------
def linear(x, weight, norm_weights=None, eps=0.0, activation="identity", mul_bias=None, add_bias=None,
           residual=None, out_dtype=None, accumulate=torch.float32):
    xn = rmsnorm(x, norm_weights, eps) if norm_weights is not None else x
    y = F.linear(xn.to(accumulate), weight.to(accumulate))
    if activation == "silu":
        y = F.silu(y)
    if mul_bias is not None:
        y = y * mul_bias.to(accumulate)
    if add_bias is not None:
        y = y + add_bias.to(accumulate)
    if residual is not None:
        y = y + residual.to(accumulate)
    return y.to(out_dtype if out_dtype is not None else x.dtype)


# ---------------------------------------------------------------------------------------------------
# Gate/up + SiLU and the whole MLP (csrc/ffn/gateup_fp16_kernels.cu:334-339, csrc/ffn/gateup.cu:161-219).
# The intermediate t is rounded to the activation dtype, as it round-trips memory in 16 bits.
# ---------------------------------------------------------------------------------------------------
def gateup_silu(x, gate_w, up_w, norm_weights=None, eps=0.0, out_dtype=None):
    xn = rmsnorm(x, norm_weights, eps) if norm_weights is not None else x
    g = F.linear(xn.float(), gate_w.float())
    u = F.linear(xn.float(), up_w.float())
    return (F.silu(g) * u).to(out_dtype if out_dtype is not None else x.dtype)


def mlp(x, gate_w, up_w, down_w, norm_weights=None, eps=0.0, residual=None, out_dtype=None):
    t = gateup_silu(x, gate_w, up_w, norm_weights, eps)
    return linear(t, down_w, residual=residual, out_dtype=out_dtype if out_dtype is not None else x.dtype)


# ---------------------------------------------------------------------------------------------------
# Weight-only 8-bit round-to-nearest quantisers.
#  * group/min format: restatement of muillm/quantization/rtnquantizer.py:49-88 (uint8, per group of
#    2**group_shift input columns a (scale, min) pair, fp32 op order amax/amin -> range clamp 1e-6 ->
#    sub, div, clamp, round-half-even).
#  * symmetric per-row: s = absmax_row / 127 stored in the weight dtype, q = round(W / s) clamped to
#    [-127, 127] — the format BASELINE config 2 names.
# ---------------------------------------------------------------------------------------------------
def rtn_group_quantize(w: torch.Tensor, group_shift: int = 7, f: float = 1.0) -> Tuple[torch.Tensor, torch.Tensor]:
    gs = 1 << group_shift
    tq = w.reshape(-1, gs).to(torch.float32)
    max_val = tq.amax(dim=1, keepdim=True)
    min_val = tq.amin(dim=1, keepdim=True)
    val_range = (f * (max_val - min_val)).clamp(min=1e-6)
    center = (min_val + max_val) * 0.5
    min_val = center - val_range * 0.5
    scales = val_range / 255
    q = tq.sub(min_val).div(scales).clamp(0, 255).round().to(torch.uint8).reshape_as(w)
    return q, torch.concat([scales, min_val], dim=-1).to(w.dtype)


def rtn_group_dequantize(q: torch.Tensor, scales_min: torch.Tensor, group_shift: int = 7) -> torch.Tensor:
    """fp32 de-quantised weights q*scale+min with the stored (16-bit) scale/min values."""
    gs = 1 << group_shift
    qg = q.reshape(-1, gs).float()
    s = scales_min[:, None, 0].float()
    m = scales_min[:, None, 1].float()
    return (qg * s + m).reshape(q.shape)


def rtn_symrow_quantize(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    wf = w.float()
    s = (wf.abs().amax(dim=1) / 127.0).clamp(min=1e-8).to(w.dtype)
    q = torch.round(wf / s.float()[:, None]).clamp(-127, 127).to(torch.int8)
    return q, s


def rtn_symrow_dequantize(q: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    return q.float() * s.float()[:, None]


# ---------------------------------------------------------------------------------------------------
# Rotary embedding: cos/sin tables as HF LlamaRotaryEmbedding builds them (default rope type; the
# reference's MuiRotaryEmbedding caches the same, muillm/modules/attention/rotaryembedding.py:313-337),
# rotate-half application (rotaryembedding.py:23-64; csrc/rope/rotary_fp16_kernels.cu:712-752) and the
# static-cache write + narrow (csrc/rope/rotary.cu:751-755).
# ---------------------------------------------------------------------------------------------------
def rope_tables(max_pos: int, dim: int, theta: float, dtype: torch.dtype) -> Tuple[torch.Tensor, torch.Tensor]:
    inv_freq = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.int64).float() / dim))
    t = torch.arange(max_pos, dtype=torch.float32)
    freqs = torch.outer(t, inv_freq)
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def rotate_half(x):
    x1 = x[..., : x.shape[-1] // 2]
    x2 = x[..., x.shape[-1] // 2:]
    return torch.cat((-x2, x1), dim=-1)


def rope_apply(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, position_ids: torch.Tensor) -> torch.Tensor:
    """x [B,H,T,D]; cos/sin [S,D]; position_ids [B,T] -> fp32 math, rounded once to x.dtype."""
    c = cos[position_ids].unsqueeze(1).float()  # [B,1,T,D]
    s = sin[position_ids].unsqueeze(1).float()
    xf = x.float()
    return (xf * c + rotate_half(xf) * s).to(x.dtype)


def rope_write_static_cache(q, k, v, cos, sin, position_ids, k_cache, v_cache, cache_position, seen_tokens):
    """Returns (q_rot, K[:, :, :seen], V[:, :, :seen]) and updates the caches in place."""
    q_rot = rope_apply(q, cos, sin, position_ids)
    k_rot = rope_apply(k, cos, sin, position_ids)
    k_cache[:, :, cache_position] = k_rot
    v_cache[:, :, cache_position] = v
    return q_rot, k_cache[:, :, :seen_tokens], v_cache[:, :, :seen_tokens]


# ---------------------------------------------------------------------------------------------------
# Decode attention for one query token with grouped-query heads. Mask semantics of the reference kernel:
# a position is kept iff its additive mask value equals 0 (csrc/attention/flash_decoding_fp16_kernels.cu:
# 386-393); GQA mapping kv_head = q_head // (Hq/Hkv) (:226). Fallback math of the reference:
# muillm/modules/attention/baseattention.py:219-253. Returns [B, 1, Hq*D].
# ---------------------------------------------------------------------------------------------------
def decode_attention(q, k, v, mask=None, scale=None, out_dtype=None):
    B, Hq, T, D = q.shape
    assert T == 1
    Hkv = k.shape[1]
    G = Hq // Hkv
    kf = k.float().repeat_interleave(G, dim=1)
    vf = v.float().repeat_interleave(G, dim=1)
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    scores = torch.matmul(q.float(), kf.transpose(2, 3)) * scale  # [B,Hq,1,S]
    if mask is not None:
        keep = (mask.reshape(B, 1, 1, -1).float() == 0)
        scores = scores.masked_fill(~keep, float("-inf"))
    probs = torch.softmax(scores, dim=-1)
    probs = torch.nan_to_num(probs, nan=0.0)  # fully masked row -> zeros
    out = torch.matmul(probs, vf)  # [B,Hq,1,D]
    return out.transpose(1, 2).reshape(B, 1, Hq * D).to(out_dtype if out_dtype is not None else q.dtype)


# ---------------------------------------------------------------------------------------------------
# Router top-k + sigmoid (muillm/modules/topk.py:39-44): top-k of the logits, sigmoid in fp32 of the
# selected values, cast back. Ties resolve to the lowest index.
# ---------------------------------------------------------------------------------------------------
def topk_sigmoid(logits: torch.Tensor, k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    lf = logits.float()
    # stable descending sort => ties keep the lowest index first
    order = torch.sort(lf, dim=-1, descending=True, stable=True).indices[..., :k]
    vals = torch.gather(lf, -1, order)
    return torch.sigmoid(vals).to(logits.dtype), order


# ---------------------------------------------------------------------------------------------------
# MoE MLP for one token: shared experts first (score 1), then the routed ones; the router score scales
# the gate and up pre-activations, i.e. the expert input (csrc/moeffn/gateupmoe_fp16_kernels.cu:355-363);
# per-expert down projections are summed, residual added once (csrc/moeffn/moelinear_fp16_kernels.cu:
# 363-375). Weights are packed [(n_shared + n_experts) * I, H] and [(n_shared + n_experts) * H, I].
# ---------------------------------------------------------------------------------------------------
def moe_mlp(x, gate_w, up_w, down_w, num_shared, num_experts_total, router_scores, router_indices,
            norm_weights=None, eps=0.0, residual=None, out_dtype=None):
    H = x.shape[-1]
    I = gate_w.shape[0] // num_experts_total
    xn = rmsnorm(x, norm_weights, eps) if norm_weights is not None else x
    xf = xn.reshape(1, H).float()
    y = torch.zeros(1, H, dtype=torch.float32)
    slots = [(e, 1.0) for e in range(num_shared)]
    for j in range(router_indices.numel()):
        slots.append((num_shared + int(router_indices.reshape(-1)[j]), float(router_scores.reshape(-1)[j].float())))
    for e, s in slots:
        g = F.linear(xf, gate_w[e * I:(e + 1) * I].float()) * s
        u = F.linear(xf, up_w[e * I:(e + 1) * I].float()) * s
        t = (F.silu(g) * u).to(x.dtype)
        y = y + F.linear(t.float(), down_w[e * H:(e + 1) * H].float())
    if residual is not None:
        y = y + residual.reshape(1, H).float()
    return y.reshape(x.shape).to(out_dtype if out_dtype is not None else x.dtype)


# ---------------------------------------------------------------------------------------------------
# All-reduce of per-rank fp32 partial sums in fixed rank order 0..P-1, one rounding. (The reference sums
# 16-bit partials pairwise in half precision, csrc/comms/comm_p2p.cu:889-895 — a documented deviation.)
# ---------------------------------------------------------------------------------------------------
# ---- Llama-4 attention prologue, windowed cache, bookkeeping -------------------------------------------------


def complex_rope(x: torch.Tensor, position_embeds: torch.Tensor) -> torch.Tensor:
    """x [B, H, T, D] times (cos + j sin) on interleaved (even, odd) pairs; position_embeds fp32 [B, T, D/2, 2].
    Follows the reference's CPU branch and HF `apply_rotary_emb` (muillm/modules/attention/llama4attention.py:58-73,
    kernel csrc/rope/rotary_fp16_kernels.cu:842-942): complex product in fp32, one rounding."""
    xc = torch.view_as_complex(x.float().reshape(*x.shape[:-1], -1, 2).contiguous())
    fc = torch.view_as_complex(position_embeds.float().contiguous())
    return torch.view_as_real(xc * fc[:, None, :, :]).flatten(3).to(x.dtype)


def l2norm(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x * rsqrt(mean(x^2) + eps) in fp32, one rounding (HF Llama4TextL2Norm; kernel csrc/norm/qkl2norm_fp16_kernels.cu:35-140
    places eps inside the sum instead)."""
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype)


def temperature_tuning(q: torch.Tensor, cache_position: torch.Tensor, attn_scale: float, floor_scale: float):
    """q [B, H, T, D] scaled per token (muillm/modules/attention/llama4attention.py:76-108,
    csrc/temperaturetuning/temperature_tuning_fp16_kernels.cu:10-46)."""
    s = torch.log1p(torch.floor((cache_position.float() + 1.0) / floor_scale)) * attn_scale + 1.0
    return (q.float() * s.view(1, 1, -1, 1)).to(q.dtype)


def sliding_cache_update(k_in, v_in, k_cache, v_cache, cache_position, seen_tokens):
    """The three modes of csrc/kvcaches/sliding_kvcache.cpp:87-246 (seen_tokens counts the new tokens); returns
    (k_states, v_states, k_cache, v_cache) with the caches the caller keeps afterwards."""
    T, W = k_in.shape[2], k_cache.shape[2]
    if seen_tokens == T:
        n = min(T, W)
        k_cache[:, :, :n] = k_in[:, :, T - n:]
        v_cache[:, :, :n] = v_in[:, :, T - n:]
        return k_in, v_in, k_cache, v_cache
    if seen_tokens > W:
        n = min(T, W)
        k_new = torch.cat((k_cache[:, :, n:], k_in[:, :, T - n:]), dim=2)
        v_new = torch.cat((v_cache[:, :, n:], v_in[:, :, T - n:]), dim=2)
        return k_new, v_new, k_new, v_new
    k_cache[:, :, cache_position] = k_in
    v_cache[:, :, cache_position] = v_in
    return k_cache[:, :, :seen_tokens], v_cache[:, :, :seen_tokens], k_cache, v_cache


def reduce_sum(x: torch.Tensor, dim: int, keep_dim: bool) -> torch.Tensor:
    """fp32 sum over one dimension, one rounding (csrc/reduce/reduce.cu:33-153)."""
    return x.float().sum(dim=dim, keepdim=keep_dim).to(x.dtype)


def add_tokens_check_finished(input_ids, next_tokens, unfinished, has_eos, pad_token_id, eos_ids, has_max_length,
                              max_length):
    """The bookkeeping of HF `GenerationMixin._sample` that csrc/generation/generation.cu:30-213 fuses: finished
    sequences receive the pad token, the token is appended, then the eos / max-length criteria update the mask."""
    tok = next_tokens.to(torch.int64)
    if has_eos:
        tok = tok * unfinished + pad_token_id * (1 - unfinished)
    out = torch.cat((input_ids, tok[:, None]), dim=1)
    done = torch.zeros_like(unfinished, dtype=torch.bool)
    if has_max_length:
        done |= out.shape[1] >= max_length
    if has_eos:
        done |= torch.isin(tok, eos_ids)
    return out, unfinished & (~done).to(torch.int64)


def all_reduce_fixed_order(partials, out_dtype):
    acc = torch.zeros_like(partials[0], dtype=torch.float32)
    for p in partials:
        acc = acc + p.float()
    return acc.to(out_dtype)


# ---------------------------------------------------------------------------------------------------
# A whole Llama-architecture decoder in terms of the functions above (used for greedy-token parity and
# as the CPU baseline model). Weights: dict with per-layer lists; KV cache static [B,Hkv,max_T,D].
# Structure follows muillm/modules/decoder/decoder.py:95-165 and muillm/modules/models/llama/model.py:213-435.
# ---------------------------------------------------------------------------------------------------
class LlamaOracle:
    def __init__(self, weights: dict, cfg: dict, max_T: int, batch: int = 1, all_reduce=None):
        """all_reduce: None for un-sharded weights; for a tensor-parallel shard (muillm_b200.decoder_stack
        .shard_llama_weights) a callable that sums an fp32 tensor of partial results over the ranks in rank order —
        it is applied to the o_proj and down partials before the residual is added and the sum is rounded, the
        order of operations of the fused GEMV + all-reduce."""
        self.w = weights
        self.cfg = cfg
        self.all_reduce = all_reduce
        dt = weights["embed"].dtype
        self.dtype = dt
        L, Hkv, D = cfg["layers"], cfg["kv_heads"], cfg["head_dim"]
        self.k_cache = [torch.zeros(batch, Hkv, max_T, D, dtype=dt) for _ in range(L)]
        self.v_cache = [torch.zeros(batch, Hkv, max_T, D, dtype=dt) for _ in range(L)]
        self.cos, self.sin = rope_tables(max_T, D, cfg["rope_theta"], dt)
        self.seen = 0

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        """token_ids [B, T] -> logits of the last position [B, vocab] (fp32). Processes T tokens one by one."""
        cfg, w = self.cfg, self.w
        Hq, Hkv, D = cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
        B, T = token_ids.shape
        logits = None
        for t in range(T):
            h = w["embed"][token_ids[:, t]]  # [B, H]
            pos = self.seen
            position_ids = torch.full((B, 1), pos, dtype=torch.int64)
            cache_position = torch.tensor([pos], dtype=torch.int64)
            for l in range(cfg["layers"]):
                qkv = linear(h, w["qkv"][l], norm_weights=w["ln1"][l], eps=cfg["eps"])
                q = qkv[:, : Hq * D].reshape(B, Hq, 1, D)
                k = qkv[:, Hq * D: (Hq + Hkv) * D].reshape(B, Hkv, 1, D)
                v = qkv[:, (Hq + Hkv) * D:].reshape(B, Hkv, 1, D)
                q, ks, vs = rope_write_static_cache(q, k, v, self.cos, self.sin, position_ids, self.k_cache[l],
                                                    self.v_cache[l], cache_position, pos + 1)
                attn = decode_attention(q, ks, vs).reshape(B, Hq * D)
                if self.all_reduce is None:
                    h = linear(attn, w["o"][l], residual=h)
                    h = mlp(h, w["gate"][l], w["up"][l], w["down"][l], norm_weights=w["ln2"][l], eps=cfg["eps"],
                            residual=h)
                else:
                    part = linear(attn, w["o"][l], out_dtype=torch.float32)
                    h = (self.all_reduce(part) + h.float()).to(self.dtype)
                    t = gateup_silu(h, w["gate"][l], w["up"][l], norm_weights=w["ln2"][l], eps=cfg["eps"])
                    part = linear(t, w["down"][l], out_dtype=torch.float32)
                    h = (self.all_reduce(part) + h.float()).to(self.dtype)
            self.seen += 1
            logits = linear(h, w["lm_head"], norm_weights=w["norm"], eps=cfg["eps"], out_dtype=torch.float32)
        return logits

    def greedy(self, prompt: torch.Tensor, new_tokens: int) -> torch.Tensor:
        logits = self.forward(prompt)
        out = []
        for _ in range(new_tokens):
            nxt = logits.argmax(dim=-1)
            out.append(nxt)
            logits = self.forward(nxt[:, None])
        return torch.stack(out, dim=1)


def make_llama_weights(cfg: dict, dtype: torch.dtype, seed: int = 0, std: float = 0.02) -> dict:
    """Seeded random-init weights of a Llama-architecture model (normal std 0.02 like HF's default init,
    RMSNorm weights 1 + N(0, 0.01))."""
    g = torch.Generator().manual_seed(seed)
    H, I, V = cfg["hidden"], cfg["intermediate"], cfg["vocab"]
    Hq, Hkv, D = cfg["heads"], cfg["kv_heads"], cfg["head_dim"]

    def rn(*shape):
        return (torch.randn(*shape, generator=g) * std).to(dtype)

    def nw():
        return (1.0 + 0.01 * torch.randn(H, generator=g)).to(dtype)

    w = {"embed": rn(V, H), "lm_head": rn(V, H), "norm": nw(), "qkv": [], "o": [], "gate": [], "up": [],
         "down": [], "ln1": [], "ln2": []}
    for _ in range(cfg["layers"]):
        w["qkv"].append(rn((Hq + 2 * Hkv) * D, H))
        w["o"].append(rn(H, Hq * D))
        w["gate"].append(rn(I, H))
        w["up"].append(rn(I, H))
        w["down"].append(rn(H, I))
        w["ln1"].append(nw())
        w["ln2"].append(nw())
    return w
