"""ctypes binding of the C ABI declared in include/muillm_b200.h.

`lib()` loads muillm_b200/lib/libmuillm_b200.so (built by `python -m muillm_b200.build`) and raises if
it is missing: there is no fallback path. `check()` turns a non-zero mui_status_t into a RuntimeError
carrying mui_last_error(), which is how the reference surfaces failures (TORCH_CHECK -> RuntimeError,
csrc/linear/linear.cu:72-74).
"""
import ctypes
import os
from ctypes import (POINTER, Structure, c_char_p, c_float, c_int, c_int64, c_longlong, c_size_t, c_uint,
                    c_void_p)

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libmuillm_b200.so")

MUI_OK = 0
MUI_ERR_INVALID_ARG = 1
MUI_ERR_UNSUPPORTED = 2
MUI_ERR_CUDA = 3
MUI_ERR_DEVICE = 4
MUI_ERR_COMM = 5

MUI_F16 = 0
MUI_BF16 = 1
MUI_COMM_F32 = 2

MUI_ACT_IDENTITY = 0
MUI_ACT_SILU = 1

MUI_W8_SYM_ROW = 0
MUI_W8_GROUP_MIN = 1

MUI_FLAG_PDL = 1
MUI_FLAG_FORCE_GENERIC = 2
MUI_FLAG_FORCE_PIPELINE = 4
MUI_FLAG_SHORT_CONTEXT = 16
MUI_FLAG_SPLIT_CONTEXT = 32


class Strides3(Structure):
    _fields_ = [("batch", c_int64), ("head", c_int64), ("tok", c_int64)]


class DeviceProps(Structure):
    _fields_ = [
        ("device", c_int),
        ("sm_count", c_int),
        ("cc_major", c_int),
        ("cc_minor", c_int),
        ("smem_per_block_optin", c_int),
        ("l2_bytes", c_int),
        ("total_mem", c_size_t),
    ]


class LlamaConfig(Structure):
    _fields_ = [
        ("dtype", c_int),
        ("layers", c_int), ("hidden", c_int), ("intermediate", c_int), ("heads", c_int), ("kv_heads", c_int),
        ("head_dim", c_int), ("vocab", c_int),
        ("max_seq", c_int),
        ("batch", c_int),
        ("rms_eps", c_float),
        ("attn_scale", c_float),
        ("embed_vocab", c_int),
        ("vocab_offset", c_int),
    ]


class LlamaWeights(Structure):
    _fields_ = [
        ("embed", c_void_p), ("final_norm", c_void_p), ("lm_head", c_void_p),
        ("cos_table", c_void_p), ("sin_table", c_void_p),
        ("qkv", POINTER(c_void_p)), ("o", POINTER(c_void_p)), ("gate", POINTER(c_void_p)),
        ("up", POINTER(c_void_p)), ("down", POINTER(c_void_p)), ("ln1", POINTER(c_void_p)),
        ("ln2", POINTER(c_void_p)), ("k_cache", POINTER(c_void_p)), ("v_cache", POINTER(c_void_p)),
    ]


class Llama4Config(Structure):
    _fields_ = [
        ("dtype", c_int),
        ("layers", c_int), ("hidden", c_int), ("expert_intermediate", c_int), ("heads", c_int), ("kv_heads", c_int),
        ("head_dim", c_int), ("vocab", c_int),
        ("max_seq", c_int), ("chunk", c_int),
        ("num_experts", c_int), ("top_k", c_int), ("num_shared", c_int),
        ("rms_eps", c_float), ("softmax_scale", c_float),
        ("use_qk_norm", c_int), ("temperature_tuning", c_int),
        ("attn_scale", c_float), ("floor_scale", c_float),
        ("embed_vocab", c_int), ("vocab_offset", c_int),
    ]


class Llama4Weights(Structure):
    _fields_ = [
        ("embed", c_void_p), ("final_norm", c_void_p), ("lm_head", c_void_p),
        ("freqs", c_void_p), ("use_rope", POINTER(c_int)),
        ("qkv", POINTER(c_void_p)), ("o", POINTER(c_void_p)), ("router", POINTER(c_void_p)),
        ("gate", POINTER(c_void_p)), ("up", POINTER(c_void_p)), ("down", POINTER(c_void_p)),
        ("ln1", POINTER(c_void_p)), ("ln2", POINTER(c_void_p)), ("k_cache", POINTER(c_void_p)),
        ("v_cache", POINTER(c_void_p)),
    ]


# name -> (restype, argtypes); every symbol include/muillm_b200.h declares appears here
PROTOTYPES = {
    "mui_status_string": (c_char_p, [c_int]),
    "mui_last_error": (c_char_p, []),
    "mui_version": (c_int, []),
    "mui_device_props": (c_int, [c_int, POINTER(DeviceProps)]),
    "mui_device_status": (c_int, [POINTER(c_uint), c_int]),
    "mui_trace_enable": (c_int, [c_void_p, c_void_p, c_int]),
    "mui_trace_count": (c_int, [POINTER(c_int), c_int]),
    "mui_linear_forward": (
        c_int,
        [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_float, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
         c_void_p, c_void_p, c_uint],
    ),
    "mui_gateup_silu_forward": (
        c_int,
        [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_uint],
    ),
    "mui_gateupdown_forward": (
        c_int,
        [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
         c_void_p, c_void_p, c_uint],
    ),
    "mui_linear_w8_forward": (
        c_int,
        [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_float, c_void_p, c_void_p, c_int, c_void_p,
         c_void_p, c_void_p, c_void_p, c_void_p, c_uint],
    ),
    "mui_gateup_silu_w8_forward": (
        c_int,
        [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_float, c_void_p, c_void_p, c_void_p,
         c_void_p, c_void_p, c_void_p, c_uint],
    ),
    "mui_gateup_silu_w8_packed_forward": (
        c_int,
        [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_void_p,
         c_uint],
    ),
    "mui_w8_dequantize": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "mui_rmsnorm_forward": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_float, c_void_p, c_void_p, c_uint]),
    "mui_rope_forward": (
        c_int,
        [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
         Strides3, c_void_p, Strides3, c_void_p, Strides3, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_uint],
    ),
    "mui_static_kvcache_update": (
        c_int,
        [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, Strides3, c_void_p, Strides3, c_void_p,
         c_void_p, c_void_p, c_uint],
    ),
    "mui_flash_decode_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int, c_int]),
    "mui_flash_decode": (
        c_int,
        [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_float, c_void_p, c_void_p, c_void_p,
         Strides3, c_void_p, c_void_p, c_void_p, c_size_t, c_uint],
    ),
    "mui_rope_flash_decode": (
        c_int,
        [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
         c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_uint],
    ),
    "mui_rope_flash_decode_ws": (
        c_int,
        [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
         c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_int, c_uint],
    ),
    "mui_flash_decode_static_scratch": (
        c_int,
        [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_float, c_void_p, c_void_p, c_void_p,
         Strides3, c_void_p, c_void_p, c_uint],
    ),
    "mui_complex_rope_forward": (
        c_int,
        [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, Strides3, c_void_p, Strides3,
         c_void_p, c_void_p, c_uint],
    ),
    "mui_qkl2norm_forward": (
        c_int,
        [c_void_p, c_int, c_longlong, c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_uint],
    ),
    "mui_temperature_tuning_forward": (
        c_int,
        [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, Strides3, c_void_p, c_void_p, c_float, c_float,
         c_uint],
    ),
    "mui_llama4_qk_prologue": (
        c_int,
        [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_float, c_void_p, c_float, c_float,
         c_void_p, Strides3, c_void_p, Strides3, c_void_p, c_void_p, c_uint],
    ),
    "mui_sliding_kvcache_update": (
        c_int,
        [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, Strides3, c_void_p, Strides3,
         c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, POINTER(c_int), c_uint],
    ),
    "mui_reduce_sum_forward": (c_int, [c_void_p, c_int, c_longlong, c_int, c_longlong, c_void_p, c_void_p, c_uint]),
    "mui_add_tokens_check_finished": (
        c_int,
        [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_int, c_int,
         c_longlong, c_void_p, c_void_p, c_uint],
    ),
    "mui_topk_sigmoid_forward": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_uint]),
    "mui_moe_gateup_silu_forward": (
        c_int,
        [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_float, c_void_p, c_void_p, c_void_p,
         c_void_p, c_void_p, c_void_p, c_uint],
    ),
    "mui_moe_down_forward": (
        c_int,
        [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
         c_void_p, c_uint],
    ),
    "mui_moe_mlp_forward": (
        c_int,
        [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_float, c_void_p, c_void_p, c_void_p,
         c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_uint],
    ),
    "mui_bootstrap_allgather": (c_int, [c_int, c_int, c_char_p, c_void_p, c_size_t, c_void_p, ctypes.c_double]),
    "mui_comm_ipc_handle_bytes": (c_size_t, []),
    "mui_comm_create": (c_int, [c_int, c_int, c_size_t, POINTER(c_void_p)]),
    "mui_comm_ipc_handle": (c_int, [c_void_p, c_void_p]),
    "mui_comm_open_peers": (c_int, [c_void_p, c_void_p]),
    "mui_comm_init_local": (c_int, [c_int, c_int, c_char_p, c_size_t, ctypes.c_double, POINTER(c_void_p)]),
    "mui_comm_destroy": (c_int, [c_void_p]),
    "mui_comm_info": (c_int, [c_void_p, POINTER(c_int), POINTER(c_int), POINTER(c_size_t)]),
    "mui_comm_all_reduce_sum": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_size_t, c_uint]),
    "mui_comm_broadcast": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_size_t, c_uint]),
    "mui_parallel_linear_forward": (
        c_int,
        [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_void_p,
         c_void_p, c_void_p, c_uint],
    ),
    "mui_parallel_gateupdown_forward": (
        c_int,
        [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_void_p,
         c_void_p, c_void_p, c_void_p, c_uint],
    ),
    "mui_parallel_moe_mlp_forward": (
        c_int,
        [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_float, c_void_p, c_void_p,
         c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_uint],
    ),
    "mui_embedding_forward": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_uint]),
    "mui_llama_stack_scratch_bytes": (c_size_t, [POINTER(LlamaConfig)]),
    "mui_llama_stack_create": (
        c_int, [POINTER(LlamaConfig), POINTER(LlamaWeights), c_void_p, c_size_t, POINTER(c_void_p)]),
    "mui_llama_stack_destroy": (c_int, [c_void_p]),
    "mui_llama4_stack_cache_rows": (c_int, [POINTER(Llama4Config), c_int]),
    "mui_llama4_stack_scratch_bytes": (c_size_t, [POINTER(Llama4Config)]),
    "mui_llama4_stack_create": (
        c_int, [POINTER(Llama4Config), POINTER(Llama4Weights), c_void_p, c_size_t, POINTER(c_void_p)]),
    "mui_prefill_linear_forward": (
        c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                c_uint]),
    "mui_prefill_gateup_silu_forward": (
        c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_uint]),
    "mui_llama4_stack_router_state": (c_int, [c_void_p, POINTER(c_void_p), POINTER(c_void_p)]),
    "mui_llama4_rope_flash_decode": (
        c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                c_int, c_int, c_float, c_int, c_float, c_float, c_int, c_float, c_void_p, c_void_p, c_void_p, c_void_p,
                c_size_t, c_int, c_uint]),
    "mui_router_topk_sigmoid_forward": (
        c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_void_p,
                c_void_p, c_void_p, c_uint]),
    "mui_llama_stack_set_comm": (c_int, [c_void_p, c_void_p]),
    "mui_llama_stack_reset": (c_int, [c_void_p, c_void_p, c_int, POINTER(c_int64), c_void_p, c_int]),
    "mui_llama_stack_set_attention_mask": (c_int, [c_void_p, c_void_p]),
    "mui_llama_stack_set_position_ids": (c_int, [c_void_p, c_void_p, c_void_p, c_int]),
    "mui_llama_stack_set_tokens": (c_int, [c_void_p, c_void_p, c_void_p, c_int]),
    "mui_llama_stack_step": (c_int, [c_void_p, c_void_p, c_uint]),
    "mui_llama_stack_capture": (c_int, [c_void_p, c_void_p, c_uint]),
    "mui_llama_stack_replay": (c_int, [c_void_p, c_void_p, c_int]),
    "mui_llama_stack_forward_hidden": (
        c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_uint]),
    "mui_llama_stack_logits": (c_int, [c_void_p, POINTER(c_void_p), POINTER(c_void_p)]),
}

_lib = None


def lib():
    """Returns the loaded library with prototypes applied; raises if the .so is missing."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} not found: build it with `python -m muillm_b200.build` (there is no fallback path)"
            )
        l = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(l, name)  # AttributeError if the symbol is not exported
            fn.restype = res
            fn.argtypes = args
        _lib = l
    return _lib


def check(status):
    if status != MUI_OK:
        l = lib()
        raise RuntimeError(
            f"muillm_b200: {l.mui_status_string(status).decode()} — {l.mui_last_error().decode()}"
        )


def device_status(clear=True):
    """Synchronises and returns the device status word (0 = no kernel reported a timed-out wait)."""
    code = c_uint(0)
    check(lib().mui_device_status(ctypes.byref(code), 1 if clear else 0))
    return code.value
