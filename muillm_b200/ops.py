"""Tensor-level entry points over the C ABI, named and shaped like the stateless functions of the
reference's `muillm_ext` module (csrc/module.cpp:177-277): they take torch CUDA tensors, allocate the
output with torch (device memory and streams are torch's job here) and launch on torch's current stream.

Every function fails loudly when the CUDA library is missing or a tensor is not a contiguous CUDA
tensor of a supported dtype — there is no eager/PyTorch fallback inside.
"""
import ctypes
import math

import torch

from . import capi
from .capi import Strides3


def _dtype_code(t):
    if t.dtype == torch.float16:
        return capi.MUI_F16
    if t.dtype == torch.bfloat16:
        return capi.MUI_BF16
    raise RuntimeError(f"Unsupported dtype {t.dtype} (float16 or bfloat16 expected)")


def _check_input(t, name):
    if t is None:
        return
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")


def _ptr(t):
    return None if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _rows(x):
    """Number of activation rows: everything but the last dimension."""
    return x.numel() // x.shape[-1] if x.numel() else 0


def muillm_linear_forward(engine, x, weights, norm_weights=None, epsilon=0.0, mul_bias=None, add_bias=None,
                          residual=None, activation=capi.MUI_ACT_IDENTITY, flags=0, out=None):
    """y = act(W · rmsnorm(x)) * mul_bias + add_bias + residual (csrc/module.cpp:178, csrc/linear/linear.cu:160-207).

    x [..., K] with at most 8 rows, weights [N, K]; returns [..., N]."""
    for t, n in ((x, "x"), (weights, "weights"), (norm_weights, "norm_weights"), (mul_bias, "mul_bias"),
                 (add_bias, "add_bias"), (residual, "residual")):
        _check_input(t, n)
    N, K = weights.shape
    if x.shape[-1] != K:
        raise RuntimeError(f"x last dim {x.shape[-1]} != K {K}")
    if norm_weights is not None and norm_weights.numel() != K:
        raise RuntimeError("fused normalization is not supported when sharding on dim 1 (K != NORM_K)")
    B = _rows(x)
    y = out if out is not None else torch.empty(x.shape[:-1] + (N,), dtype=x.dtype, device=x.device)
    capi.check(capi.lib().mui_linear_forward(
        _stream(), _dtype_code(x), B, N, K, _ptr(norm_weights), float(epsilon), _ptr(weights), int(activation),
        _ptr(mul_bias), _ptr(add_bias), _ptr(residual), _ptr(x), _ptr(y), flags))
    return y


def muillm_gateupsilu_forward(engine, norm_weights, epsilon, gate_weights, up_weights, down_weights, residual, x,
                              flags=0):
    """down(silu(gate(xn)) * up(xn)) + residual (csrc/module.cpp:182, csrc/ffn/gateup.cu:176-219)."""
    for t, n in ((x, "x"), (gate_weights, "gate_weights"), (up_weights, "up_weights"),
                 (down_weights, "down_weights"), (norm_weights, "norm_weights"), (residual, "residual")):
        _check_input(t, n)
    I, H = gate_weights.shape
    B = _rows(x)
    t = torch.empty((B, I), dtype=x.dtype, device=x.device)
    y = torch.empty(x.shape[:-1] + (down_weights.shape[0],), dtype=x.dtype, device=x.device)
    capi.check(capi.lib().mui_gateupdown_forward(
        _stream(), _dtype_code(x), B, I, H, _ptr(norm_weights), float(epsilon), _ptr(gate_weights),
        _ptr(up_weights), _ptr(down_weights), _ptr(residual), _ptr(x), _ptr(t), _ptr(y), flags))
    return y


def gateup_silu(x, gate_weights, up_weights, norm_weights=None, epsilon=0.0, flags=0, out=None):
    """t = silu(G xn) * (U xn) only (the first kernel of the MLP)."""
    for t, n in ((x, "x"), (gate_weights, "gate_weights"), (up_weights, "up_weights"),
                 (norm_weights, "norm_weights")):
        _check_input(t, n)
    I, H = gate_weights.shape
    B = _rows(x)
    if out is None:
        out = torch.empty(x.shape[:-1] + (I,), dtype=x.dtype, device=x.device)
    capi.check(capi.lib().mui_gateup_silu_forward(
        _stream(), _dtype_code(x), B, I, H, _ptr(norm_weights), float(epsilon), _ptr(gate_weights),
        _ptr(up_weights), _ptr(x), _ptr(out), flags))
    return out


def prefill_linear(x, weights, mul_bias=None, add_bias=None, residual=None, activation=capi.MUI_ACT_IDENTITY, flags=0):
    """y = act(x W^T) * mul_bias + add_bias + residual for any number of rows (x [..., K], weights [N, K]) on the
    tcgen05 tensor cores: the prefill / batched counterpart of muillm_linear_forward."""
    for t, n in ((x, "x"), (weights, "weights"), (mul_bias, "mul_bias"), (add_bias, "add_bias"),
                 (residual, "residual")):
        _check_input(t, n)
    N, K = weights.shape
    if x.shape[-1] != K:
        raise RuntimeError(f"x last dim {x.shape[-1]} != K {K}")
    M = x.numel() // K
    y = torch.empty(x.shape[:-1] + (N,), dtype=x.dtype, device=x.device)
    capi.check(capi.lib().mui_prefill_linear_forward(
        _stream(), _dtype_code(x), M, N, K, _ptr(weights), int(activation), _ptr(mul_bias), _ptr(add_bias),
        _ptr(residual), _ptr(x), _ptr(y), flags))
    return y


def prefill_gateup_silu(x, gate_weights, up_weights, flags=0):
    """t = silu(x G^T) * (x U^T) for any number of rows on the tcgen05 tensor cores (no fused norm)."""
    for t, n in ((x, "x"), (gate_weights, "gate_weights"), (up_weights, "up_weights")):
        _check_input(t, n)
    I, H = gate_weights.shape
    M = x.numel() // H
    out = torch.empty(x.shape[:-1] + (I,), dtype=x.dtype, device=x.device)
    capi.check(capi.lib().mui_prefill_gateup_silu_forward(
        _stream(), _dtype_code(x), M, I, H, _ptr(gate_weights), _ptr(up_weights), _ptr(x), _ptr(out), flags))
    return out


def muillm_rmsnorm_forward(weights, x, epsilon, flags=0):
    """RMSNorm over the last dim (csrc/module.cpp:251, csrc/norm/rmsnorm.cu:31-84). weights may be None (L2 norm)."""
    _check_input(x, "x")
    _check_input(weights, "weights")
    K = x.shape[-1]
    y = torch.empty_like(x)
    capi.check(capi.lib().mui_rmsnorm_forward(_stream(), _dtype_code(x), _rows(x), K, _ptr(weights), float(epsilon),
                                              _ptr(x), _ptr(y), flags))
    return y


def _strides3(t):
    """(batch, head, token) element strides of a [B, H, T, D] view whose innermost stride is 1."""
    if t.dim() != 4 or t.stride(3) != 1:
        raise RuntimeError("expected a [B, H, T, D] tensor with innermost stride 1")
    return Strides3(t.stride(0), t.stride(1), t.stride(2))


def muillm_rope_forward_static_cache(position_ids, cos_cached, sin_cached, q_in, k_in, v_in, k_cache, v_cache,
                                     cache_position, seen_tokens, flags=0):
    """RoPE on q,k + write of k,v at cache_position; returns (q_out, K[:, :, :seen], V[:, :, :seen])
    (csrc/rope/rotary.cu:603-756)."""
    for t, n in ((position_ids, "position_ids"), (cos_cached, "cos_cached"), (sin_cached, "sin_cached"),
                 (k_cache, "k_cache"), (v_cache, "v_cache"), (cache_position, "cache_position")):
        _check_input(t, n)
    B, Hq, T, D = q_in.shape
    Hkv = k_in.shape[1]
    max_T = k_cache.shape[2]
    if cos_cached.dim() == 2:
        layout = 0
    elif cos_cached.dim() == 3:
        layout = 1
    else:
        raise RuntimeError("Unknown rotary cache layout")
    q_out = torch.empty((B, Hq, T, D), dtype=q_in.dtype, device=q_in.device)
    capi.check(capi.lib().mui_rope_forward(
        _stream(), _dtype_code(q_in), B, T, max_T, Hq, Hkv, D, layout, _ptr(position_ids), _ptr(cos_cached),
        _ptr(sin_cached), _ptr(q_in), _strides3(q_in), _ptr(k_in), _strides3(k_in), _ptr(v_in), _strides3(v_in),
        _ptr(q_out), None, _ptr(k_cache), _ptr(v_cache), _ptr(cache_position), flags))
    return q_out, k_cache.narrow(2, 0, seen_tokens), v_cache.narrow(2, 0, seen_tokens)


def muillm_rope_forward_no_cache(position_ids, cos_cached, sin_cached, q_in, k_in, flags=0):
    """RoPE on q,k without cache (csrc/rope/rotary.cu:188)."""
    B, Hq, T, D = q_in.shape
    Hkv = k_in.shape[1]
    layout = 0 if cos_cached.dim() == 2 else 1
    q_out = torch.empty((B, Hq, T, D), dtype=q_in.dtype, device=q_in.device)
    k_out = torch.empty((B, Hkv, T, D), dtype=k_in.dtype, device=k_in.device)
    z = Strides3(0, 0, 0)
    capi.check(capi.lib().mui_rope_forward(
        _stream(), _dtype_code(q_in), B, T, 0, Hq, Hkv, D, layout, _ptr(position_ids), _ptr(cos_cached),
        _ptr(sin_cached), _ptr(q_in), _strides3(q_in), _ptr(k_in), _strides3(k_in), None, z, _ptr(q_out),
        _ptr(k_out), None, None, None, flags))
    return q_out, k_out


def muillm_static_kvcache_update(k_in, v_in, k_cache, v_cache, cache_position, seen_tokens, flags=0):
    """Scatter of the new k,v rows at cache_position (csrc/kvcaches/static_kvcache.cpp:35-120)."""
    B, Hkv, T, D = k_in.shape
    max_T = k_cache.shape[2]
    capi.check(capi.lib().mui_static_kvcache_update(
        _stream(), _dtype_code(k_in), B, T, max_T, Hkv, D, _ptr(k_in), _strides3(k_in), _ptr(v_in),
        _strides3(v_in), _ptr(k_cache), _ptr(v_cache), _ptr(cache_position), flags))
    return k_cache.narrow(2, 0, seen_tokens), v_cache.narrow(2, 0, seen_tokens)


_fd_workspaces = {}


def _fd_workspace(device, nbytes):
    key = (device.index, torch.cuda.current_stream().cuda_stream)
    ws = _fd_workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        _fd_workspaces[key] = ws
    return ws


def _flash_decode(q, k, v, mask, flags=0, seq_len_dev=None, scale=None):
    _check_input(q, "q")
    _check_input(mask, "m")
    B, Hq, T, D = q.shape
    if T != 1:
        raise RuntimeError("flash decoding expects exactly one query token (T == 1)")
    Hkv, S = k.shape[1], k.shape[2]
    if k.stride() != v.stride():
        raise RuntimeError("k and v must have the same strides")
    if mask is not None:
        mask = mask.reshape(B, S)
    out = torch.empty((B, 1, Hq * D), dtype=q.dtype, device=q.device)
    lib = capi.lib()
    nbytes = lib.mui_flash_decode_workspace_bytes(B, Hq, Hkv, D, S)
    ws = _fd_workspace(q.device, nbytes)
    capi.check(lib.mui_flash_decode(
        _stream(), _dtype_code(q), B, Hq, Hkv, D, S, _ptr(seq_len_dev),
        float(scale if scale is not None else 1.0 / math.sqrt(D)), _ptr(q), _ptr(k), _ptr(v), _strides3(k),
        _ptr(mask), _ptr(out), _ptr(ws), ws.numel(), flags))
    return out


def muillm_causal_transformer_decoding_no_mask(q, k, v, flags=0):
    """softmax(q Kᵀ / sqrt(d)) V for one query token (csrc/module.cpp:276, csrc/attention/flash_decoding.cu:288-305)."""
    return _flash_decode(q, k, v, None, flags)


def muillm_causal_transformer_decoding_masked(q, k, v, m, flags=0):
    """Same with an additive [B,1,1,S] mask; positions whose mask value is 0 are kept
    (csrc/module.cpp:277, csrc/attention/flash_decoding.cu:307-325)."""
    return _flash_decode(q, k, v, m, flags)


def muillm_topk_sigmoid_forward(router_logits, top_k, flags=0):
    """(sigmoid(top-k values), int64 indices) over the last dim (csrc/module.cpp:253, csrc/topk/topk.cu:34-93)."""
    _check_input(router_logits, "router_logits")
    M = router_logits.shape[-1]
    rows = _rows(router_logits)
    values = torch.empty(router_logits.shape[:-1] + (top_k,), dtype=router_logits.dtype, device=router_logits.device)
    indices = torch.empty(router_logits.shape[:-1] + (top_k,), dtype=torch.int64, device=router_logits.device)
    capi.check(capi.lib().mui_topk_sigmoid_forward(_stream(), _dtype_code(router_logits), rows, M, int(top_k),
                                                   _ptr(router_logits), _ptr(values), _ptr(indices), flags))
    return values, indices


def muillm_gateupsilumoe_forward(engine, num_shared_experts, num_dynamic_experts, norm_weights, epsilon, gate_weights,
                                 up_weights, down_weights, residual, x, router_scores, router_indices, flags=0):
    """MoE MLP for one token (csrc/module.cpp:183, csrc/moeffn/gateupmoe.cu:221-272)."""
    for t, n in ((x, "x"), (gate_weights, "gate_weights"), (up_weights, "up_weights"), (down_weights, "down_weights"),
                 (norm_weights, "norm_weights"), (residual, "residual"), (router_scores, "router_scores"),
                 (router_indices, "router_indices")):
        _check_input(t, n)
    if _rows(x) != 1:
        raise RuntimeError("the MoE kernels serve one token (B*T == 1); batches go to the batched fallback")
    E = num_shared_experts + num_dynamic_experts
    H = x.shape[-1]
    I = gate_weights.shape[0] // E
    top_k = router_indices.numel()
    if router_indices.dtype != torch.int64:
        raise RuntimeError("router_indices must be int64")
    t = torch.empty((num_shared_experts + top_k, I), dtype=x.dtype, device=x.device)
    y = torch.empty_like(x)
    capi.check(capi.lib().mui_moe_mlp_forward(
        _stream(), _dtype_code(x), num_shared_experts, num_dynamic_experts, top_k, I, H, _ptr(norm_weights),
        float(epsilon), _ptr(gate_weights), _ptr(up_weights), _ptr(down_weights), _ptr(residual), _ptr(x),
        _ptr(router_scores), _ptr(router_indices), _ptr(t), _ptr(y), flags))
    return y


def muillm_embedding_forward(weights, inputs, flags=0):
    """Row gather out[..., :] = weights[inputs[...], :] for int64 token ids (csrc/embedding/embedding_xx16_kernels.cu:26)."""
    _check_input(weights, "weights")
    _check_input(inputs, "inputs")
    if inputs.dtype != torch.int64:
        raise RuntimeError("token ids must be int64")
    vocab, H = weights.shape
    out = torch.empty(tuple(inputs.shape) + (H,), dtype=weights.dtype, device=weights.device)
    capi.check(capi.lib().mui_embedding_forward(_stream(), _dtype_code(weights), inputs.numel(), H, vocab,
                                                _ptr(weights), _ptr(inputs), _ptr(out), flags))
    return out


def _w8_fmt(qweights):
    if qweights.dtype == torch.int8:
        return capi.MUI_W8_SYM_ROW
    if qweights.dtype == torch.uint8:
        return capi.MUI_W8_GROUP_MIN
    raise RuntimeError("quantised weights must be int8 (symmetric per-row) or uint8 (per-group scale/min)")


def muillm_int8_linear_forward(x, weights, scales_min_vals, group_size_shift, norm_weights=None, epsilon=0.0,
                               mul_bias=None, add_bias=None, residual=None, flags=0):
    """Linear on weight-only 8-bit weights (csrc/module.cpp:181, csrc/int8_linear_kernels.cu:703-784). uint8 weights
    take the reference's [N*G, 2] scale/min pairs; int8 weights take one scale per output row."""
    for t, n in ((x, "x"), (weights, "weights"), (scales_min_vals, "scales_min_vals"),
                 (norm_weights, "norm_weights"), (mul_bias, "mul_bias"), (add_bias, "add_bias"),
                 (residual, "residual")):
        _check_input(t, n)
    N, K = weights.shape
    B = _rows(x)
    y = torch.empty(x.shape[:-1] + (N,), dtype=x.dtype, device=x.device)
    capi.check(capi.lib().mui_linear_w8_forward(
        _stream(), _dtype_code(x), _w8_fmt(weights), int(group_size_shift), B, N, K, _ptr(norm_weights),
        float(epsilon), _ptr(weights), _ptr(scales_min_vals), capi.MUI_ACT_IDENTITY, _ptr(mul_bias), _ptr(add_bias),
        _ptr(residual), _ptr(x), _ptr(y), flags))
    return y


def int8_gateup_silu(x, gate_q, gate_scales, up_q, up_scales, group_size_shift=0, norm_weights=None, epsilon=0.0,
                     flags=0):
    """t = silu(G xn) * (U xn) on 8-bit gate/up weights (first kernel of muillm_int8_gateupsilu_forward,
    csrc/int8_gateup_kernels.cu:871-940)."""
    for t, n in ((x, "x"), (gate_q, "gate_q"), (up_q, "up_q"), (gate_scales, "gate_scales"),
                 (up_scales, "up_scales"), (norm_weights, "norm_weights")):
        _check_input(t, n)
    I, H = gate_q.shape
    B = _rows(x)
    out = torch.empty(x.shape[:-1] + (I,), dtype=x.dtype, device=x.device)
    capi.check(capi.lib().mui_gateup_silu_w8_forward(
        _stream(), _dtype_code(x), _w8_fmt(gate_q), int(group_size_shift), B, I, H, _ptr(norm_weights),
        float(epsilon), _ptr(gate_q), _ptr(gate_scales), _ptr(up_q), _ptr(up_scales), _ptr(x), _ptr(out), flags))
    return out


def int8_gateup_silu_packed(x, gate_up_q, gate_up_scales_min, group_size_shift, norm_weights=None, epsilon=0.0,
                            flags=0):
    """t = silu(G xn) * (U xn) on the reference's own packed layout: gate_up_q [I, H, 2] uint8 (gate, up interleaved
    element by element), gate_up_scales_min [I * G, 2, 2] (gate {scale, min}, up {scale, min}) as built by
    muillm/modules/quantized/int8gateupdownmlp.py:211-230. Raises capi.MuiError (MUI_ERR_UNSUPPORTED) for shapes the
    pipeline kernel does not serve."""
    for t, n in ((x, "x"), (gate_up_q, "gate_up_q"), (gate_up_scales_min, "gate_up_scales_min"),
                 (norm_weights, "norm_weights")):
        _check_input(t, n)
    I, H, two = gate_up_q.shape
    if two != 2 or gate_up_q.dtype != torch.uint8:
        raise ValueError("gate_up_q must be a uint8 [I, H, 2] tensor")
    B = _rows(x)
    out = torch.empty(x.shape[:-1] + (I,), dtype=x.dtype, device=x.device)
    capi.check(capi.lib().mui_gateup_silu_w8_packed_forward(
        _stream(), _dtype_code(x), int(group_size_shift), B, I, H, _ptr(norm_weights), float(epsilon),
        _ptr(gate_up_q), _ptr(gate_up_scales_min), _ptr(x), _ptr(out), flags))
    return out


def muillm_int8_dequantize_forward(weights, scales_min_vals, group_size_shift, dtype=None):
    """Whole-matrix de-quantisation (csrc/module.cpp:180, csrc/int8_dequantization_kernel.cu:74)."""
    _check_input(weights, "weights")
    _check_input(scales_min_vals, "scales_min_vals")
    N, K = weights.shape
    out = torch.empty((N, K), dtype=scales_min_vals.dtype, device=weights.device)
    capi.check(capi.lib().mui_w8_dequantize(_stream(), _dtype_code(scales_min_vals), _w8_fmt(weights),
                                            int(group_size_shift), N, K, _ptr(weights), _ptr(scales_min_vals),
                                            _ptr(out)))
    return out


def rope_flash_decode(qkv, cos_table, sin_table, position_ids, cache_position, seq_len, k_cache, v_cache, num_q_heads,
                      flags=0, workspace=None, max_attended=None):
    """Fused decode attention for one new token per sequence: RoPE on q and the new k, K/V cache write at
    cache_position, attention over the first `seq_len` cache rows (the new one included). qkv is the packed QKV
    projection output [B, (Hq + 2*Hkv) * D]; position_ids [B] int64, cache_position [1] int64 and seq_len [1] int32
    are device tensors. Returns [B, 1, Hq * D]. One launch in place of muillm_rope_forward_static_cache +
    muillm_causal_transformer_decoding_no_mask. With `workspace` (uint8 tensor of flash_decode_workspace_bytes, first
    4 KiB zero) and MUI_FLAG_SPLIT_CONTEXT the tokens are split over several CTAs per KV head, sized for
    `max_attended` tokens (default: the cache length)."""
    for t, n in ((qkv, "qkv"), (cos_table, "cos_table"), (sin_table, "sin_table"), (position_ids, "position_ids"),
                 (cache_position, "cache_position"), (seq_len, "seq_len"), (k_cache, "k_cache"), (v_cache, "v_cache")):
        _check_input(t, n)
    B, Hkv, max_seq, D = k_cache.shape
    out = torch.empty((B, 1, num_q_heads * D), dtype=qkv.dtype, device=qkv.device)
    capi.check(capi.lib().mui_rope_flash_decode_ws(
        _stream(), _dtype_code(qkv), B, num_q_heads, Hkv, D, max_seq, _ptr(qkv), _ptr(cos_table), _ptr(sin_table),
        _ptr(position_ids), _ptr(cache_position), _ptr(seq_len), 1.0 / math.sqrt(D), _ptr(k_cache), _ptr(v_cache),
        _ptr(out), _ptr(workspace), 0 if workspace is None else workspace.numel(),
        max_seq if max_attended is None else int(max_attended), flags))
    return out


# ---- Llama-4 attention prologue, windowed cache, bookkeeping ------------------------------------------------


def muillm_complex_rope_forward_no_cache(q_in, k_in, position_embeds, flags=0):
    """Interleaved-pair rotary embedding with fp32 (cos, sin) pairs [B, T, D/2, 2] (a complex tensor viewed as
    real works too); returns contiguous (q_out, k_out) (csrc/rope/rotary.cu:798-915)."""
    if position_embeds.is_complex():
        position_embeds = torch.view_as_real(position_embeds)
    _check_input(position_embeds, "position_embeds")
    if position_embeds.dim() != 4 or position_embeds.dtype != torch.float32:
        raise RuntimeError("Complex ROPE only supported with BTE layout")
    B, Hq, T, D = q_in.shape
    Hk = k_in.shape[1]
    q_out = torch.empty((B, Hq, T, D), dtype=q_in.dtype, device=q_in.device)
    k_out = torch.empty((B, Hk, T, D), dtype=k_in.dtype, device=k_in.device)
    capi.check(capi.lib().mui_complex_rope_forward(
        _stream(), _dtype_code(q_in), B, T, Hq, Hk, D, _ptr(position_embeds), _ptr(q_in), _strides3(q_in),
        _ptr(k_in), _strides3(k_in), _ptr(q_out), _ptr(k_out), flags))
    return q_out, k_out


def muillm_qkl2norm_forward(q, k, epsilon, flags=0):
    """L2 norm over the last dimension of q and of k in one launch (csrc/norm/qkl2norm.cu:38-100)."""
    _check_input(q, "q")
    _check_input(k, "k")
    D = q.shape[-1]
    if k.shape[-1] != D:
        raise RuntimeError("The last dimension of q and k must be the same")
    q_out, k_out = torch.empty_like(q), torch.empty_like(k)
    capi.check(capi.lib().mui_qkl2norm_forward(_stream(), _dtype_code(q), q.numel() // D, k.numel() // D, D, _ptr(q),
                                               _ptr(k), _ptr(q_out), _ptr(k_out), float(epsilon), flags))
    return q_out, k_out


def muillm_l2norm_forward(x, epsilon, flags=0):
    """x * rsqrt(mean(x^2) + eps) over the last dimension (csrc/norm/l2norm.cu:28-76): the RMSNorm kernel
    without weights."""
    _check_input(x, "x")
    K = x.shape[-1]
    y = torch.empty_like(x)
    capi.check(capi.lib().mui_rmsnorm_forward(_stream(), _dtype_code(x), _rows(x), K, None, float(epsilon), _ptr(x),
                                              _ptr(y), flags))
    return y


def muillm_apply_temperature_tuning(query_states, cache_position, attn_scale, floor_scale, flags=0):
    """q * (log1p(floor((cache_position + 1) / floor_scale)) * attn_scale + 1) for q [B, H, T, D]
    (csrc/temperaturetuning/temperature_tuning.cu)."""
    _check_input(cache_position, "cache_position")
    B, H, T, D = query_states.shape
    out = torch.empty((B, H, T, D), dtype=query_states.dtype, device=query_states.device)
    capi.check(capi.lib().mui_temperature_tuning_forward(
        _stream(), _dtype_code(query_states), B, T, H, D, _ptr(query_states), _strides3(query_states),
        _ptr(cache_position), _ptr(out), float(attn_scale), float(floor_scale), flags))
    return out


def llama4_qk_prologue(q_in, k_in, position_embeds=None, qk_norm_eps=None, cache_position=None, attn_scale=0.0,
                       floor_scale=1.0, flags=0):
    """Complex rope -> QK L2 norm -> temperature scale (q only) in one launch; any stage may be absent."""
    if position_embeds is not None and position_embeds.is_complex():
        position_embeds = torch.view_as_real(position_embeds)
    B, Hq, T, D = q_in.shape
    Hk = k_in.shape[1]
    q_out = torch.empty((B, Hq, T, D), dtype=q_in.dtype, device=q_in.device)
    k_out = torch.empty((B, Hk, T, D), dtype=k_in.dtype, device=k_in.device)
    capi.check(capi.lib().mui_llama4_qk_prologue(
        _stream(), _dtype_code(q_in), B, T, Hq, Hk, D, _ptr(position_embeds), 0 if qk_norm_eps is None else 1,
        float(qk_norm_eps or 0.0), _ptr(cache_position), float(attn_scale), float(floor_scale), _ptr(q_in),
        _strides3(q_in), _ptr(k_in), _strides3(k_in), _ptr(q_out), _ptr(k_out), flags))
    return q_out, k_out


def muillm_sliding_kvcache_update(k_in, v_in, k_cache, v_cache, cache_position, seen_tokens, flags=0):
    """Sliding-window cache update with rows in chronological order (csrc/kvcaches/sliding_kvcache.cpp:87-246).
    Returns the (key, value) states to attend: the inputs on the first fill, the first seen_tokens cache rows
    while the window is not full, else a fresh pair of full-window buffers the caller keeps as the cache."""
    _check_input(k_cache, "k_cache")
    _check_input(v_cache, "v_cache")
    _check_input(cache_position, "cache_position")
    B, Hk, T, D = k_in.shape
    Hv = v_in.shape[1]
    max_T = k_cache.shape[2]
    full = seen_tokens > max_T and seen_tokens != T
    k_new = torch.empty_like(k_cache) if full else None
    v_new = torch.empty_like(v_cache) if full else None
    mode = ctypes.c_int(-1)
    capi.check(capi.lib().mui_sliding_kvcache_update(
        _stream(), _dtype_code(k_in), B, T, max_T, Hk, Hv, D, _ptr(k_in), _strides3(k_in), _ptr(v_in),
        _strides3(v_in), _ptr(k_cache), _ptr(v_cache), _ptr(k_new), _ptr(v_new), _ptr(cache_position),
        int(seen_tokens), ctypes.byref(mode), flags))
    if mode.value == 0:
        return k_in, v_in
    if mode.value == 1:
        return k_new, v_new
    return k_cache.narrow(2, 0, seen_tokens), v_cache.narrow(2, 0, seen_tokens)


def muillm_reduce_sum_forward(x, dim, keep_dim, flags=0):
    """Sum over one dimension with fp32 accumulation (csrc/reduce/reduce.cu:33-153)."""
    _check_input(x, "x")
    if x.dim() < 1:
        raise RuntimeError("Input tensor must have at least one dimension")
    if dim < 0:
        dim += x.dim()
    if not 0 <= dim < x.dim():
        raise RuntimeError("Invalid dimension for reduction")
    sizes = list(x.shape)
    Bo = 1
    for s in sizes[:dim]:
        Bo *= s
    N = 1
    for s in sizes[dim + 1:]:
        N *= s
    M = sizes[dim]
    out_sizes = sizes[:dim] + ([1] if keep_dim else []) + sizes[dim + 1:]
    y = torch.empty(out_sizes, dtype=x.dtype, device=x.device)
    capi.check(capi.lib().mui_reduce_sum_forward(_stream(), _dtype_code(x), Bo, M, N, _ptr(x), _ptr(y), flags))
    return y


def muillm_add_tokens_check_finished(input_ids, next_tokens, unfinished_sequences, has_eos_stopping_criteria,
                                     pad_token_id, eos_token_ids, has_max_length_stopping_criteria, max_length,
                                     flags=0):
    """Append the next token to input_ids [B, T] and update the unfinished mask
    (csrc/generation/generation.cu:119-213). next_tokens int32, the other tensors int64."""
    for t, n in ((input_ids, "input_ids"), (next_tokens, "next_tokens"), (unfinished_sequences,
                                                                         "unfinished_sequences")):
        _check_input(t, n)
    if input_ids.dtype != torch.int64:
        raise RuntimeError("input_ids must be of type int64")
    if unfinished_sequences.dtype != torch.int64:
        raise RuntimeError("unfinished_sequences must be of type int64")
    if next_tokens.dtype != torch.int32:
        raise RuntimeError("next_tokens must be of type int")
    B, T = input_ids.shape
    if unfinished_sequences.shape[0] != B:
        raise RuntimeError("unfinished_sequences doesn't have the shape [B]")
    n_eos = 0 if eos_token_ids is None else int(eos_token_ids.numel())
    out = torch.empty((B, T + 1), dtype=torch.int64, device=input_ids.device)
    unf = torch.empty_like(unfinished_sequences)
    capi.check(capi.lib().mui_add_tokens_check_finished(
        _stream(), B, T, _ptr(input_ids), _ptr(next_tokens), _ptr(unfinished_sequences),
        1 if has_eos_stopping_criteria else 0, int(pad_token_id or 0), _ptr(eos_token_ids), n_eos,
        1 if has_max_length_stopping_criteria else 0, int(max_length if max_length is not None else -1), _ptr(out),
        _ptr(unf), flags))
    return out, unf
