"""Weights of a Hugging Face Llama-architecture checkpoint in the layout the decode stack takes: q, k and v
projections concatenated along the output rows (as MuiMultiLinear does, muillm/modules/multilinear.py:229-237),
everything else as stored."""
import torch

from .decoder_stack import LlamaDecodeStack


def llama_config_from_hf(hf_config):
    """dict for LlamaDecodeStack from a transformers LlamaConfig (or an object with the same attributes)."""
    head_dim = getattr(hf_config, "head_dim", None) or hf_config.hidden_size // hf_config.num_attention_heads
    theta = getattr(hf_config, "rope_theta", None)
    if theta is None:
        theta = (getattr(hf_config, "rope_parameters", None) or {}).get("rope_theta", 10000.0)
    return dict(layers=hf_config.num_hidden_layers, hidden=hf_config.hidden_size,
                intermediate=hf_config.intermediate_size, heads=hf_config.num_attention_heads,
                kv_heads=hf_config.num_key_value_heads, head_dim=head_dim, vocab=hf_config.vocab_size,
                eps=hf_config.rms_norm_eps, rope_theta=float(theta))


def llama_weights_from_state_dict(sd, num_layers, dtype=torch.float16, device="cuda"):
    """sd: mapping of HF parameter names ('model.layers.0.self_attn.q_proj.weight', ...) to tensors."""

    def t(name):
        return torch.as_tensor(sd[name]).to(device=device, dtype=dtype).contiguous()

    lm_head = "lm_head.weight" if "lm_head.weight" in sd else "model.embed_tokens.weight"  # tied embeddings
    w = {"embed": t("model.embed_tokens.weight"), "lm_head": t(lm_head), "norm": t("model.norm.weight"),
         "qkv": [], "o": [], "gate": [], "up": [], "down": [], "ln1": [], "ln2": []}
    for l in range(num_layers):
        p = f"model.layers.{l}."
        w["qkv"].append(torch.cat([t(p + "self_attn.q_proj.weight"), t(p + "self_attn.k_proj.weight"),
                                   t(p + "self_attn.v_proj.weight")], dim=0).contiguous())
        w["o"].append(t(p + "self_attn.o_proj.weight"))
        w["gate"].append(t(p + "mlp.gate_proj.weight"))
        w["up"].append(t(p + "mlp.up_proj.weight"))
        w["down"].append(t(p + "mlp.down_proj.weight"))
        w["ln1"].append(t(p + "input_layernorm.weight"))
        w["ln2"].append(t(p + "post_attention_layernorm.weight"))
    return w


def decode_stack_from_hf(model, max_seq, batch=1, max_new_tokens=4096, flags=0, dtype=None):
    """A LlamaDecodeStack over the weights of a transformers LlamaForCausalLM (copied to the GPU in `dtype`, default
    the model's own 16-bit dtype or fp16)."""
    cfg = llama_config_from_hf(model.config)
    if dtype is None:
        dtype = model.dtype if model.dtype in (torch.float16, torch.bfloat16) else torch.float16
    w = llama_weights_from_state_dict(model.state_dict(), cfg["layers"], dtype=dtype)
    return LlamaDecodeStack(w, cfg, max_seq=max_seq, batch=batch, max_new_tokens=max_new_tokens, flags=flags)
