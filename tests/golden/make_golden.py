"""Generates the golden fixtures under tests/golden/ (run once in the authoring container; needs the reference
checkout, whose location is $MUILLM_REFERENCE, and transformers). Committed beside the fixtures it made.

Sources of truth, in order of authority:
 * the reference's own Python, imported unmodified with a stub `muillm_ext` (the CPU branches never call it):
   `muillm.quantization.rtnquantizer.RTNQuantizer` (quantise / de-quantise), `MuiRMSNorm.forward` CPU branch
   (muillm/modules/norm/rmsnorm.py:138-146), `topk_sigmoid` non-fp16 branch (muillm/modules/topk.py:39-44);
 * the HF modules the reference's tests compare against (tests/test_linear.py, test_gateupdownmlp.py,
   test_rmsnorm.py, test_rotaryembedding.py): LlamaRMSNorm, nn.Linear, LlamaMLP, LlamaRotaryEmbedding +
   apply_rotary_pos_emb, eager attention with repeat_kv, LlamaForCausalLM greedy generation.
Inputs are seeded; outputs are stored in fp32 (and int for quantised weights / tokens).
"""
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.environ.get("MUILLM_REFERENCE")  # checkout of the reference; required for the fixtures made from it


class _Stub(types.ModuleType):
    def __getattr__(self, name):
        if name.startswith("__"):
            raise AttributeError(name)

        def _f(*a, **k):
            raise RuntimeError("muillm_ext stub called: " + name)

        return _f


def reference_fixtures(out):
    sys.modules["muillm_ext"] = _Stub("muillm_ext")
    sys.path.insert(0, REF)
    from muillm.quantization.rtnquantizer import RTNQuantizer
    from muillm.modules.topk import topk_sigmoid
    from muillm.modules.norm.rmsnorm import MuiRMSNorm
    from muillm.engineconfig import MuiEngineConfig  # noqa: F401  (import check only)

    g = torch.Generator().manual_seed(0)
    # RTN group quantiser: fp16 weights [24, 256], group 128 and group 32
    w = (torch.randn(24, 256, generator=g) * 0.02).to(torch.float16)
    w[3, :128] = 0.0125  # a constant group exercises the range clamp
    for gs in (128, 32):
        q = RTNQuantizer(n_bit=8, groupsize=gs)
        wq, sm = q.group_quantize_tensor(w)
        wd = q.group_dequantize_tensor(wq, sm, dtype=torch.float16)
        out[f"rtn_g{gs}_w"] = w.float().numpy()
        out[f"rtn_g{gs}_q"] = wq.numpy()
        out[f"rtn_g{gs}_scales_min"] = sm.float().numpy()
        out[f"rtn_g{gs}_dequant_f16"] = wd.float().numpy()

    # top-k sigmoid, bf16 branch (torch.topk + fp32 sigmoid)
    logits = torch.randn(3, 1, 16, generator=g).to(torch.bfloat16)
    for k in (1, 2):
        v, i = topk_sigmoid(logits, k)
        out[f"topk{k}_logits"] = logits.float().numpy()
        out[f"topk{k}_values"] = v.float().numpy()
        out[f"topk{k}_indices"] = i.numpy()

    # MuiRMSNorm CPU branch (built without the engine: only weight/eps/dispatchable are touched by forward)
    norm = MuiRMSNorm.__new__(MuiRMSNorm)
    torch.nn.Module.__init__(norm)
    norm.weight = torch.nn.Parameter((1 + 0.01 * torch.randn(320, generator=g)).to(torch.float16))
    norm.variance_epsilon = 1e-5
    norm.dispatchable = False
    x = torch.randn(5, 320, generator=g).to(torch.float16)
    out["ref_rmsnorm_x"] = x.float().numpy()
    out["ref_rmsnorm_w"] = norm.weight.detach().float().numpy()
    out["ref_rmsnorm_y"] = norm(x).detach().float().numpy()


def hf_fixtures(out):
    from transformers import LlamaConfig, LlamaForCausalLM
    from transformers.models.llama.modeling_llama import (LlamaMLP, LlamaRMSNorm, LlamaRotaryEmbedding,
                                                          apply_rotary_pos_emb, repeat_kv)

    torch.manual_seed(0)
    g = torch.Generator().manual_seed(1)
    cfg = LlamaConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=8,
                      num_key_value_heads=2, head_dim=32, vocab_size=512, rms_norm_eps=1e-5, rope_theta=500000.0,
                      max_position_embeddings=128, attention_bias=False, mlp_bias=False, tie_word_embeddings=False)
    small = LlamaConfig(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                        num_key_value_heads=2, head_dim=32, vocab_size=256, rms_norm_eps=1e-5, rope_theta=500000.0,
                        max_position_embeddings=128, attention_bias=False, mlp_bias=False,
                        tie_word_embeddings=False)

    # fused RMSNorm -> linear (config-1 style), fp16 modules evaluated by HF in fp16 on CPU
    norm = LlamaRMSNorm(256, eps=1e-5)
    norm.weight.data = 1 + 0.01 * torch.randn(256, generator=g)
    lin = torch.nn.Linear(256, 384, bias=True)
    lin.weight.data = torch.randn(384, 256, generator=g) * 0.05
    lin.bias.data = torch.randn(384, generator=g) * 0.1
    x = torch.randn(2, 256, generator=g)
    out["hf_normlinear_x"] = x.numpy()
    out["hf_normlinear_nw"] = norm.weight.detach().clone().numpy()
    out["hf_normlinear_w"] = lin.weight.detach().clone().numpy()
    out["hf_normlinear_b"] = lin.bias.detach().clone().numpy()
    import copy
    for dt, tag in ((torch.float32, "f32"), (torch.float16, "f16")):
        n, l, xx = copy.deepcopy(norm).to(dt), copy.deepcopy(lin).to(dt), x.to(dt)
        y = l(n(xx))
        out[f"hf_normlinear_{tag}_y"] = y.detach().float().numpy()

    # MLP
    mlp = LlamaMLP(cfg)
    for p in mlp.parameters():
        p.data = torch.randn(p.shape, generator=g) * 0.05
    xm = torch.randn(3, 256, generator=g)
    out["hf_mlp_x"] = xm.numpy()
    out["hf_mlp_gate"] = mlp.gate_proj.weight.detach().numpy()
    out["hf_mlp_up"] = mlp.up_proj.weight.detach().numpy()
    out["hf_mlp_down"] = mlp.down_proj.weight.detach().numpy()
    out["hf_mlp_y"] = mlp(xm).detach().numpy()

    # rotary embedding tables + application, and eager GQA attention for one query token
    rot = LlamaRotaryEmbedding(cfg)
    B, Hq, Hkv, D, S = 2, 8, 2, 32, 37
    pos = torch.arange(S)[None, :].expand(B, S)
    cos, sin = rot(torch.zeros(1, dtype=torch.float32), pos)
    out["hf_rope_cos"] = cos[0].numpy()
    out["hf_rope_sin"] = sin[0].numpy()
    q = torch.randn(B, Hq, S, D, generator=g)
    k = torch.randn(B, Hkv, S, D, generator=g)
    v = torch.randn(B, Hkv, S, D, generator=g)
    qr, kr = apply_rotary_pos_emb(q, k, cos, sin)
    out["hf_rope_q"], out["hf_rope_k"] = q.numpy(), k.numpy()
    out["hf_rope_q_rot"], out["hf_rope_k_rot"] = qr.numpy(), kr.numpy()
    q1 = qr[:, :, -1:, :]
    kk, vv = repeat_kv(kr, Hq // Hkv), repeat_kv(v, Hq // Hkv)
    att = torch.softmax(torch.matmul(q1, kk.transpose(2, 3)) / (D ** 0.5), dim=-1, dtype=torch.float32)
    o = torch.matmul(att, vv).transpose(1, 2).reshape(B, 1, Hq * D)
    out["hf_attn_v"] = v.numpy()
    out["hf_attn_out"] = o.numpy()

    # whole model: greedy tokens and last-position logits of the prompt
    # (weights are rounded to fp16 values so that the fixture can store them exactly in 16 bits)
    model = LlamaForCausalLM(small).eval()
    with torch.no_grad():
        for p in model.parameters():
            if p.dim() > 1:
                p.copy_((torch.randn(p.shape, generator=g) * 0.08).half().float())
            else:
                p.copy_((1 + 0.01 * torch.randn(p.shape, generator=g)).half().float())
    prompt = torch.randint(0, 256, (1, 16), generator=g)
    with torch.no_grad():
        gen = model.generate(prompt, max_new_tokens=32, do_sample=False, pad_token_id=0)
        logits = model(prompt).logits[:, -1]
    out["hf_model_prompt"] = prompt.numpy()
    out["hf_model_tokens"] = gen[:, 16:].numpy()
    out["hf_model_prompt_logits"] = logits.numpy()
    sd = model.state_dict()
    for name, t in sd.items():
        out["hf_model_sd/" + name] = t.half().numpy()


def llama4_fixtures(out):
    """HF Llama-4 building blocks: interleaved rotary embedding, QK L2 norm, temperature scale, sliding window."""
    from transformers.cache_utils import StaticSlidingWindowLayer
    from transformers.models.llama4.modeling_llama4 import Llama4TextL2Norm, apply_rotary_emb

    g = torch.Generator().manual_seed(4)
    B, Hq, Hk, T, D = 2, 5, 2, 3, 128
    # HF layout is [B, T, H, D] here (rope runs before the transpose); fixtures are stored as [B, H, T, D]
    q = torch.randn(B, T, Hq, D, generator=g)
    k = torch.randn(B, T, Hk, D, generator=g)
    ang = torch.rand(B, T, D // 2, generator=g) * 6.28
    freqs_cis = torch.polar(torch.ones_like(ang), ang)
    for dt, tag in ((torch.float16, "f16"), (torch.bfloat16, "bf16")):
        qr, kr = apply_rotary_emb(q.to(dt), k.to(dt), freqs_cis)
        out[f"l4_rope_{tag}_q"] = qr.float().transpose(1, 2).contiguous().numpy()
        out[f"l4_rope_{tag}_k"] = kr.float().transpose(1, 2).contiguous().numpy()
        nrm = Llama4TextL2Norm(1e-5)
        out[f"l4_norm_{tag}_q"] = nrm(qr).float().transpose(1, 2).contiguous().numpy()
        out[f"l4_norm_{tag}_k"] = nrm(kr).float().transpose(1, 2).contiguous().numpy()
    out["l4_q"] = q.transpose(1, 2).contiguous().numpy()
    out["l4_k"] = k.transpose(1, 2).contiguous().numpy()
    out["l4_pos_embeds"] = torch.view_as_real(freqs_cis).contiguous().numpy()
    # temperature tuning as in Llama4TextAttention.forward (floor_scale 8192, attn_scale 0.1)
    cache_position = torch.tensor([8190, 8191, 40000])
    scales = torch.log1p(torch.floor((cache_position.float() + 1.0) / 8192.0)) * 0.1 + 1.0
    qt = (q.to(torch.bfloat16) * scales.view(1, T, 1, 1)).to(torch.bfloat16)
    out["l4_temp_pos"] = cache_position.numpy()
    out["l4_temp_bf16_q"] = qt.float().transpose(1, 2).contiguous().numpy()
    # sliding window of 6 rows: 4-token prefill, then single-token steps past the window
    W, Hs, Ds = 6, 2, 8
    layer = StaticSlidingWindowLayer(max_cache_len=W, sliding_window=W)
    ks = torch.randn(1, Hs, 12, Ds, generator=g).half()
    vs = torch.randn(1, Hs, 12, Ds, generator=g).half()
    out["l4_slide_k"], out["l4_slide_v"] = ks.float().numpy(), vs.float().numpy()
    kk, vv = layer.update(ks[:, :, :4], vs[:, :, :4], {"cache_position": torch.arange(4)})
    for step in range(4, 12):
        kk, vv = layer.update(ks[:, :, step:step + 1], vs[:, :, step:step + 1],
                              {"cache_position": torch.tensor([step])})
        n = min(step + 1, W)
        out[f"l4_slide_states_k_{step}"] = kk[:, :, :n].float().numpy().copy()
        out[f"l4_slide_states_v_{step}"] = vv[:, :, :n].float().numpy().copy()


def hf_llama_d64_fixture(out):
    """A whole HF Llama with head dim 64 (the smallest the GPU attention kernels take): weights, prompt, greedy tokens."""
    from transformers import LlamaConfig, LlamaForCausalLM

    g = torch.Generator().manual_seed(21)
    cfg = LlamaConfig(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=2,
                      num_key_value_heads=1, head_dim=64, vocab_size=256, rms_norm_eps=1e-5, rope_theta=500000.0,
                      max_position_embeddings=128, attention_bias=False, mlp_bias=False, tie_word_embeddings=False)
    model = LlamaForCausalLM(cfg).eval()
    with torch.no_grad():
        for p in model.parameters():
            if p.dim() > 1:
                p.copy_((torch.randn(p.shape, generator=g) * 0.08).half().float())
            else:
                p.copy_((1 + 0.01 * torch.randn(p.shape, generator=g)).half().float())
    prompt = torch.randint(0, 256, (1, 16), generator=g)
    with torch.no_grad():
        gen = model.generate(prompt, max_new_tokens=32, do_sample=False, pad_token_id=0)
        logits = model(prompt).logits[:, -1]
    out["prompt"] = prompt.numpy()
    out["tokens"] = gen[:, 16:].numpy()
    out["prompt_logits"] = logits.numpy()
    top2 = torch.topk(logits[0], 2).values
    out["prompt_top2_margin"] = (top2[0] - top2[1]).numpy()
    for name, t in model.state_dict().items():
        out["sd/" + name] = t.half().numpy()


LLAMA4_TINY = dict(vocab_size=256, hidden_size=128, intermediate_size=64, intermediate_size_mlp=128,
                   num_hidden_layers=4, num_attention_heads=2, num_key_value_heads=1, head_dim=64, num_local_experts=4,
                   num_experts_per_tok=1, interleave_moe_layer_step=1, attention_chunk_size=8, rope_theta=500000.0,
                   rms_norm_eps=1e-5, use_qk_norm=True, attn_temperature_tuning=True, floor_scale=4, attn_scale=0.1,
                   max_position_embeddings=128, no_rope_layer_interval=4, tie_word_embeddings=False, pad_token_id=0,
                   bos_token_id=1, eos_token_id=2)


def hf_llama4_model_fixture(out, head_dim=None):
    """A whole HF Llama-4 text model (MoE with a shared expert and top-1 sigmoid routing in every layer, chunked
    attention of 8 tokens with rope + QK L2 norm in layers 0-2, full attention with temperature tuning and no rope
    in layer 3): fp16-representable weights, a 12-token prompt and the 24 tokens generate(do_sample=False) produced in
    fp32, so the run crosses four chunk boundaries. The seed is the first whose smallest top-2 logit margin over the
    24 steps exceeds 0.05, which keeps a 16-bit implementation on the same tokens."""
    from transformers import Llama4ForCausalLM, Llama4TextConfig

    kw = dict(LLAMA4_TINY)
    if head_dim is not None:  # the same model at another head size (128: the size the fused attention kernels serve)
        kw["head_dim"] = head_dim
    cfg = Llama4TextConfig(attn_implementation="eager", **kw)
    for seed in range(40, 80 if head_dim is None else 400):
        g = torch.Generator().manual_seed(seed)
        model = Llama4ForCausalLM(cfg).eval()
        with torch.no_grad():
            for p in model.parameters():
                if p.dim() > 1:
                    p.copy_((torch.randn(p.shape, generator=g) * 0.08).half().float())
                else:
                    p.copy_((1 + 0.01 * torch.randn(p.shape, generator=g)).half().float())
        prompt = torch.randint(3, 256, (1, 12), generator=g)
        with torch.no_grad():
            gen = model.generate(prompt, max_new_tokens=24, do_sample=False, pad_token_id=0, eos_token_id=None,
                                 output_scores=True, return_dict_in_generate=True)
        margins = []
        for sc in gen.scores:
            top2 = torch.topk(sc[0].float(), 2).values
            margins.append(float(top2[0] - top2[1]))
        if min(margins) > 0.05:
            break
    else:
        raise RuntimeError("no seed with clear margins")
    out["seed"] = np.array(seed)
    out["prompt"] = prompt.numpy()
    out["tokens"] = gen.sequences[:, 12:].numpy()
    out["margins"] = np.array(margins, dtype=np.float32)
    out["no_rope_layers"] = np.array(cfg.no_rope_layers)
    with torch.no_grad():
        out["prompt_logits"] = model(prompt).logits[:, -1].numpy()
    for name, t in model.state_dict().items():
        out["sd/" + name] = t.half().numpy()


def hf_moe_and_masked_attention_fixture(out):
    """Two pins the other fixtures do not hold directly: the Llama-4 MoE block (router, top-k sigmoid, routed experts
    on score-scaled inputs, shared expert; the module the reference's tests/test_gateupdownmlpmoe.py compares with)
    and eager GQA attention of one query token under an additive mask (the call of tests on masked decoding)."""
    from types import SimpleNamespace

    from transformers import Llama4TextConfig
    from transformers.models.llama.modeling_llama import eager_attention_forward
    from transformers.models.llama4.modeling_llama4 import Llama4TextMoe

    torch.manual_seed(3)
    g = torch.Generator().manual_seed(4)
    cfg = Llama4TextConfig(hidden_size=64, intermediate_size=48, intermediate_size_mlp=48, num_local_experts=6,
                           num_experts_per_tok=2, num_hidden_layers=1, num_attention_heads=4, num_key_value_heads=2,
                           head_dim=16, vocab_size=64)
    moe = Llama4TextMoe(cfg).float().eval()
    with torch.no_grad():
        for p_ in moe.parameters():
            p_.copy_(torch.randn(p_.shape, generator=g) * 0.1)
        x = torch.randn(1, 1, 64, generator=g)
        y, router_logits = moe(x)
    E, H, I = 6, 64, 48
    gu = moe.experts.gate_up_proj.detach()  # [E, H, 2I]: x @ gate_up -> (gate | up)
    out["moe_x"] = x.numpy()
    out["moe_router_w"] = moe.router.weight.detach().numpy()
    out["moe_router_logits"] = router_logits.detach().numpy()
    # row-major [rows, H] matrices, shared expert first, as the kernels take them
    out["moe_gate"] = torch.cat([moe.shared_expert.gate_proj.weight.detach()] +
                                [gu[e, :, :I].t().contiguous() for e in range(E)], 0).numpy()
    out["moe_up"] = torch.cat([moe.shared_expert.up_proj.weight.detach()] +
                              [gu[e, :, I:].t().contiguous() for e in range(E)], 0).numpy()
    out["moe_down"] = torch.cat([moe.shared_expert.down_proj.weight.detach()] +
                                [moe.experts.down_proj[e].detach().t().contiguous() for e in range(E)], 0).numpy()
    out["moe_y"] = y.detach().reshape(1, 1, 64).numpy()
    out["moe_top_k"] = np.array(2)

    B, Hq, Hkv, D, S = 2, 8, 2, 32, 29
    q = torch.randn(B, Hq, 1, D, generator=g)
    k = torch.randn(B, Hkv, S, D, generator=g)
    v = torch.randn(B, Hkv, S, D, generator=g)
    keep = torch.rand(B, S, generator=g) > 0.3
    keep[:, -1] = True  # the new token always attends itself
    mask = torch.where(keep, 0.0, torch.finfo(torch.float32).min)[:, None, None, :]
    module = SimpleNamespace(num_key_value_groups=Hq // Hkv, training=False)
    o, _ = eager_attention_forward(module, q, k, v, mask, scaling=D ** -0.5, dropout=0.0)
    out["mattn_q"], out["mattn_k"], out["mattn_v"] = q.numpy(), k.numpy(), v.numpy()
    out["mattn_mask"] = mask[:, 0, 0, :].numpy()
    out["mattn_out"] = o.reshape(B, 1, Hq * D).numpy()


def reference_pack_fixture(out):
    """The reference's own packing of per-group 8-bit gate / up weights (muillm/modules/quantized/
    int8gateupdownmlp.py:211-230), run on quantised tensors made by its RTNQuantizer."""
    from types import SimpleNamespace

    sys.modules["muillm_ext"] = _Stub("muillm_ext")
    sys.path.insert(0, REF)
    from muillm.modules.quantized.int8gateupdownmlp import MuiInt8GateUpDownMLP
    from muillm.quantization.rtnquantizer import RTNQuantizer

    g = torch.Generator().manual_seed(5)
    q = RTNQuantizer(n_bit=8, groupsize=128)
    gw = (torch.randn(12, 256, generator=g) * 0.02).to(torch.float16)
    uw = (torch.randn(12, 256, generator=g) * 0.02).to(torch.float16)
    gq, gsm = q.group_quantize_tensor(gw)
    uq, usm = q.group_quantize_tensor(uw)
    me = SimpleNamespace()
    me._pack_gateup_weights = lambda a, b: MuiInt8GateUpDownMLP._pack_gateup_weights(me, a, b)
    pack, sm = MuiInt8GateUpDownMLP._pack_gateup_linears(
        me, SimpleNamespace(weights_uint8=gq, scales_min_vals=gsm), SimpleNamespace(weights_uint8=uq, scales_min_vals=usm))
    out["gate_q"], out["up_q"] = gq.numpy(), uq.numpy()
    out["gate_scales_min"], out["up_scales_min"] = gsm.float().numpy(), usm.float().numpy()
    out["pack"], out["pack_scales_min"] = pack.numpy(), sm.float().numpy()


def main():
    if sys.argv[1:] == ["pack"]:
        d = {}
        reference_pack_fixture(d)
        np.savez_compressed(os.path.join(HERE, "reference_pack.npz"), **d)
        print("reference_pack.npz", os.path.getsize(os.path.join(HERE, "reference_pack.npz")) // 1024, "KiB", d["pack"].shape,
              d["pack_scales_min"].shape)
        return
    if sys.argv[1:] == ["moe_mask"]:
        d = {}
        hf_moe_and_masked_attention_fixture(d)
        np.savez_compressed(os.path.join(HERE, "hf_moe_mask.npz"), **d)
        print("hf_moe_mask.npz", os.path.getsize(os.path.join(HERE, "hf_moe_mask.npz")) // 1024, "KiB")
        return
    if sys.argv[1:] == ["llama4_model"]:
        d = {}
        hf_llama4_model_fixture(d)
        np.savez_compressed(os.path.join(HERE, "hf_llama4_model.npz"), **d)
        print("hf_llama4_model.npz", os.path.getsize(os.path.join(HERE, "hf_llama4_model.npz")) // 1024, "KiB",
              "seed", int(d["seed"]), "min margin", float(d["margins"].min()), "no_rope_layers", d["no_rope_layers"])
        return
    if sys.argv[1:] == ["llama4_model_d128"]:
        d = {}
        hf_llama4_model_fixture(d, head_dim=128)
        np.savez_compressed(os.path.join(HERE, "hf_llama4_model_d128.npz"), **d)
        print("hf_llama4_model_d128.npz", os.path.getsize(os.path.join(HERE, "hf_llama4_model_d128.npz")) // 1024,
              "KiB", "seed", int(d["seed"]), "min margin", float(d["margins"].min()))
        return
    if sys.argv[1:] == ["llama4"]:
        l4 = {}
        llama4_fixtures(l4)
        np.savez_compressed(os.path.join(HERE, "hf_llama4_ops.npz"), **l4)
        print("hf_llama4_ops.npz", os.path.getsize(os.path.join(HERE, "hf_llama4_ops.npz")) // 1024, "KiB")
        return
    if sys.argv[1:] == ["llama_d64"]:
        d = {}
        hf_llama_d64_fixture(d)
        np.savez_compressed(os.path.join(HERE, "hf_llama_d64.npz"), **d)
        print("hf_llama_d64.npz", os.path.getsize(os.path.join(HERE, "hf_llama_d64.npz")) // 1024, "KiB")
        return
    ref, hf = {}, {}
    # HF first: in this container, running the reference's bf16/fp16 CPU branches first left the later fp32
    # batched matmul inside LlamaRotaryEmbedding at reduced precision (cos/sin off by 2e-4); in a fresh
    # interpreter state the tables are exact, which the check below enforces.
    hf_fixtures(hf)
    inv = 1.0 / (500000.0 ** (torch.arange(0, 32, 2, dtype=torch.int64).float() / 32))
    fr = torch.outer(torch.arange(37).float(), inv)
    assert np.array_equal(hf["hf_rope_cos"], torch.cat((fr, fr), -1).cos().numpy()), "rope tables not exact"
    reference_fixtures(ref)
    np.savez_compressed(os.path.join(HERE, "reference_python.npz"), **ref)
    np.savez_compressed(os.path.join(HERE, "hf_modules.npz"), **hf)
    for f in ("reference_python.npz", "hf_modules.npz"):
        print(f, os.path.getsize(os.path.join(HERE, f)) // 1024, "KiB")


if __name__ == "__main__":
    main()
