"""Drop-in for the reference's `muillm_ext` torch extension (csrc/module.cpp:177-432): the same 89 function names,
argument orders, keyword names and defaults, handle objects instead of raw C++ pointers, all device work done by
libmuillm_b200.so through the C ABI.

    sys.modules["muillm_ext"] = muillm_b200.muillm_ext      # before importing the reference's Python package

Dispatch rule, as in the reference's C++ modules (e.g. csrc/modules/parallel_linear_module.cpp:41-92): inputs with
at most 8 rows in total (decode) run the library's GEMV kernels; larger inputs (prefill) take torch's GEMM
(`F.linear`), which is what the reference does there too (`at::linear`). Nothing here computes on the CPU: a CPU
tensor or a missing library raises.

Handles keep references to the tensors they were given (ownership stays with Python, csrc/modules/linear_module.cpp:21-25);
`*_deinit` drops them. Child modules are borrowed, as in the reference.
"""
import os

import torch
import torch.nn.functional as F

from . import ops
from .comm import MuiCommunicator

_MAX_GEMV_ROWS = 8

GATEUPSILU_FUSED = 0
GATEUPSILU_UNFUSED = 1
GATEUPSILU_SPLIT = 2

# ---- stateless operators: same names and argument orders as csrc/module.cpp:178-277 --------------------------------

muillm_int8_dequantize_forward = ops.muillm_int8_dequantize_forward
muillm_int8_linear_forward = ops.muillm_int8_linear_forward
muillm_l2norm_forward = ops.muillm_l2norm_forward
muillm_qkl2norm_forward = ops.muillm_qkl2norm_forward
muillm_rmsnorm_forward = ops.muillm_rmsnorm_forward
muillm_reduce_sum_forward = ops.muillm_reduce_sum_forward
muillm_topk_sigmoid_forward = ops.muillm_topk_sigmoid_forward
muillm_rope_forward_no_cache = ops.muillm_rope_forward_no_cache
muillm_rope_forward_static_cache = ops.muillm_rope_forward_static_cache
muillm_complex_rope_forward_no_cache = ops.muillm_complex_rope_forward_no_cache
muillm_static_kvcache_update = ops.muillm_static_kvcache_update
muillm_sliding_kvcache_update = ops.muillm_sliding_kvcache_update
muillm_causal_transformer_decoding_no_mask = ops.muillm_causal_transformer_decoding_no_mask
muillm_causal_transformer_decoding_masked = ops.muillm_causal_transformer_decoding_masked


def _rows(x):
    return x.numel() // x.shape[-1] if x.numel() else 0


# rows > 8 (prefill): this library's tcgen05 GEMM with the epilogue fused; False hands them to torch's GEMM, as the
# reference does (torch's is the faster of the two at present, see the per-kernel benchmark)
PREFILL_TENSOR_CORE_KERNEL = True


def _tensor_core_prefill_ok(x, *weights):
    """The tcgen05 prefill GEMM takes 16-bit contiguous operands with rows that are multiples of 16 bytes."""
    if not PREFILL_TENSOR_CORE_KERNEL:
        return False
    if x.dtype not in (torch.float16, torch.bfloat16) or x.shape[-1] % 8 or not x.is_contiguous():
        return False
    return all(w.is_contiguous() and w.dtype == x.dtype and w.data_ptr() % 16 == 0 for w in weights) and \
        x.data_ptr() % 16 == 0


def _not_dispatchable_on_gpu(weights):
    """The reference's modules dispatch to their kernels only for fp16 / bf16 weights on a GPU and use torch's ops
    otherwise (csrc/modules/linear_module.cpp:29-32, 60-80). The drop-in does the same for other dtypes ON THE GPU;
    CPU tensors are refused by the operators themselves (this library has no CPU path)."""
    return weights.is_cuda and weights.dtype not in (torch.float16, torch.bfloat16)


def _torch_rmsnorm(x, norm_weights, epsilon):
    if norm_weights is None:
        return x
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + epsilon)).to(x.dtype) * norm_weights


def _linear_any_rows(x, weights, norm_weights=None, epsilon=0.0, mul_bias=None, add_bias=None, residual=None):
    """Decode rows -> GEMV kernel; prefill -> RMSNorm kernel + the tcgen05 GEMM with the epilogue fused (the reference
    calls at::linear there, csrc/modules/linear_module.cpp:40-80); other dtypes / layouts -> torch GEMM."""
    if _not_dispatchable_on_gpu(weights) and x.is_cuda:
        y = F.linear(_torch_rmsnorm(x, norm_weights, epsilon), weights)
        y = y * mul_bias if mul_bias is not None else y
        y = y + add_bias if add_bias is not None else y
        return y + residual if residual is not None else y
    if _rows(x) <= _MAX_GEMV_ROWS:
        return ops.muillm_linear_forward(None, x, weights, norm_weights=norm_weights, epsilon=epsilon,
                                         mul_bias=mul_bias, add_bias=add_bias, residual=residual)
    xn = ops.muillm_rmsnorm_forward(norm_weights, x.contiguous(), epsilon) if norm_weights is not None else x
    if _tensor_core_prefill_ok(xn, weights) and (residual is None or residual.is_contiguous()):
        return ops.prefill_linear(xn, weights, mul_bias=mul_bias, add_bias=add_bias, residual=residual)
    y = F.linear(xn, weights)
    if mul_bias is not None:
        y = y * mul_bias
    if add_bias is not None:
        y = y + add_bias
    if residual is not None:
        y = y + residual
    return y


def muillm_linear_forward(engine, x, weights, norm_weights=None, epsilon=0.0, mul_bias=None, add_bias=None,
                          residual=None):
    return _linear_any_rows(x, weights, norm_weights, epsilon, mul_bias, add_bias, residual)


def _mlp_any_rows(norm_weights, epsilon, gate_weights, up_weights, down_weights, residual, x):
    if _not_dispatchable_on_gpu(gate_weights) and x.is_cuda:
        xn = _torch_rmsnorm(x, norm_weights, epsilon)
        y = F.linear(F.silu(F.linear(xn, gate_weights)) * F.linear(xn, up_weights), down_weights)
        return y + residual if residual is not None else y
    if _rows(x) <= _MAX_GEMV_ROWS:
        return ops.muillm_gateupsilu_forward(None, norm_weights, epsilon, gate_weights, up_weights, down_weights,
                                             residual, x)
    xn = ops.muillm_rmsnorm_forward(norm_weights, x.contiguous(), epsilon) if norm_weights is not None else x
    if _tensor_core_prefill_ok(xn, gate_weights, up_weights, down_weights) and \
            (residual is None or residual.is_contiguous()):
        t = ops.prefill_gateup_silu(xn, gate_weights, up_weights)
        return ops.prefill_linear(t, down_weights, residual=residual)
    y = F.linear(F.silu(F.linear(xn, gate_weights)) * F.linear(xn, up_weights), down_weights)
    return y + residual if residual is not None else y


def muillm_gateupsilu_forward(engine, norm_weights, epsilon, gate_weights, up_weights, down_weights, residual, x):
    return _mlp_any_rows(norm_weights, epsilon, gate_weights, up_weights, down_weights, residual, x)


# the reference's split-K variant differs only in how its kernels divide the work
muillm_gateupsilu_split_forward = muillm_gateupsilu_forward


def muillm_gateupsilumoe_forward(engine, num_shared_experts, num_dynamic_experts, norm_weights, epsilon, gate_weights,
                                 up_weights, down_weights, residual, x, router_scores, router_indices):
    return ops.muillm_gateupsilumoe_forward(engine, num_shared_experts, num_dynamic_experts, norm_weights, epsilon,
                                            gate_weights, up_weights, down_weights, residual, x, router_scores,
                                            router_indices)


def _split_gateup_pack(gate_up_weights, gate_up_scales_min_vals, group_size_shift):
    """The reference packs gate and up element-interleaved, [I, H, 2] uint8 with [I*G, 2, 2] (gate/up, scale/min) pairs
    (muillm/modules/quantized/int8gateupdownmlp.py:211-230); the kernels stream two plain matrices, so the pack is
    split once per tensor. The halves live on the packed tensor object itself (they go when it goes) and are redone
    when either tensor was written in place since (torch's version counters)."""
    key = (gate_up_weights._version, gate_up_scales_min_vals._version, gate_up_scales_min_vals.data_ptr(),
           group_size_shift)
    hit = getattr(gate_up_weights, "_mui_split_halves", None)
    if hit is None or hit[0] != key:
        I, H, _ = gate_up_weights.shape
        G = H >> group_size_shift
        sm = gate_up_scales_min_vals.reshape(I * G, 2, 2)
        hit = (key, (gate_up_weights[:, :, 0].contiguous(), sm[:, 0, :].contiguous(),
                     gate_up_weights[:, :, 1].contiguous(), sm[:, 1, :].contiguous()))
        gate_up_weights._mui_split_halves = hit
    return hit[1]


def muillm_int8_gateupsilu_dequantize_forward(gate_up_weights, gate_up_scales_min_vals, group_size_shift):
    """Packed 8-bit gate/up -> (gate, up) 16-bit matrices (csrc/int8_gateup_kernels.cu, dequantize entry)."""
    gq, gs, uq, us = _split_gateup_pack(gate_up_weights, gate_up_scales_min_vals, group_size_shift)
    return (ops.muillm_int8_dequantize_forward(gq, gs, group_size_shift),
            ops.muillm_int8_dequantize_forward(uq, us, group_size_shift))


def _packed_gateup_fits(rows, H, group_size_shift):
    """Shared memory of the packed gate/up kernel: staged activations (rows rounded up to 1/2/4/8), group sums,
    partial tiles and at least two 64.25 KiB weight stages inside 226 KiB (gemv_w8g.cuh, gm_layout)."""
    nb = 1 if rows <= 1 else 2 if rows <= 2 else 4 if rows <= 4 else 8
    fixed = nb * (H + 8) * 2 + (H >> group_size_shift) * 32 + 2 * 16 * 32 * nb * 4 + 256
    return fixed + 2 * 16 * (4096 + 16) <= 226 * 1024


def muillm_int8_gateupsilu_forward(norm_weights, epsilon, gate_up_weights, gate_up_scales_min_vals, group_size_shift,
                                   x):
    """silu(G xn) * (U xn) on the reference's packed 8-bit weights (csrc/int8_gateup_kernels.cu:871-940). Decode rows
    stream the pack as it is (the kernel splits the interleaved bytes in registers); shapes that kernel does not
    serve (groups under 32 weights, unaligned rows, more than 8 rows) go through the split halves."""
    rows = x.numel() // x.shape[-1]
    if (rows <= 8 and 5 <= group_size_shift <= 11 and gate_up_weights.shape[1] % 16 == 0
            and gate_up_weights.is_contiguous() and gate_up_scales_min_vals.is_contiguous()
            and gate_up_weights.data_ptr() % 16 == 0 and gate_up_scales_min_vals.data_ptr() % 8 == 0
            and _packed_gateup_fits(1, gate_up_weights.shape[1], group_size_shift)):  # batches split themselves
        return ops.int8_gateup_silu_packed(x, gate_up_weights, gate_up_scales_min_vals, group_size_shift,
                                           norm_weights=norm_weights, epsilon=epsilon)
    gq, gs, uq, us = _split_gateup_pack(gate_up_weights, gate_up_scales_min_vals, group_size_shift)
    return ops.int8_gateup_silu(x, gq, gs, uq, us, group_size_shift=group_size_shift, norm_weights=norm_weights,
                                epsilon=epsilon)


def muillm_apply_temperature_tuning(query_states, cache_position, attn_scale, floor_scale):
    return ops.muillm_apply_temperature_tuning(query_states, cache_position, attn_scale, floor_scale)


def muillm_add_tokens_check_finished(input_ids, next_tokens, unfinished_sequences, has_eos_stopping_criteria,
                                     pad_token_id, eos_token_id, has_max_length_stopping_criteria, max_length):
    return ops.muillm_add_tokens_check_finished(input_ids, next_tokens, unfinished_sequences,
                                                has_eos_stopping_criteria, pad_token_id, eos_token_id,
                                                has_max_length_stopping_criteria, max_length)


def muillm_rope_forward_dynamic_cache(position_ids, cos_cached, sin_cached, q_in, k_in, v_in, prev_k_cache,
                                      prev_v_cache):
    """RoPE + append to a growing cache; returns (q_out, k_cache_out, v_cache_out) with T_prev + T rows
    (csrc/rope/rotary.cu:376-600). The reference copies the whole cache into a fresh tensor every call; here the
    returned tensors are views of a buffer that grows by doubling, and a returned key tensor passed back as
    `prev_k_cache` (the same Python object) is extended in place."""
    B, Hk, T, D = k_in.shape
    prev = prev_k_cache.shape[2]
    k_buf, v_buf = _dyn_buffers(prev_k_cache, prev_v_cache, prev + T)
    pos = torch.arange(prev, prev + T, dtype=torch.int64, device=k_in.device)
    q_out, k_out, v_out = ops.muillm_rope_forward_static_cache(position_ids, cos_cached, sin_cached, q_in, k_in, v_in,
                                                               k_buf, v_buf, pos, prev + T)
    k_out._mui_dyn_buffers = (k_buf, v_buf)  # lets the next call extend in place
    return q_out, k_out, v_out


def _dyn_buffers(prev_k, prev_v, need_rows):
    owner = getattr(prev_k, "_mui_dyn_buffers", None)
    if owner is not None:
        k_buf, v_buf = owner
        if k_buf.shape[2] >= need_rows and k_buf.data_ptr() == prev_k.data_ptr():
            return k_buf, v_buf
    B, H, prev, D = prev_k.shape
    cap = 64
    while cap < need_rows:
        cap *= 2
    k_buf = torch.empty((B, H, cap, D), dtype=prev_k.dtype, device=prev_k.device)
    v_buf = torch.empty((B, H, cap, D), dtype=prev_v.dtype, device=prev_v.device)
    k_buf[:, :, :prev].copy_(prev_k)
    v_buf[:, :, :prev].copy_(prev_v)
    return k_buf, v_buf


# ---- engine, synchronizer, communicator ------------------------------------------------------------------------


class muillm_engine_ptr:
    """Stands for the reference's engine handle (csrc/engine.h:14-16); the library keeps its per-device state itself."""


def muillm_engine_init():
    from . import capi

    capi.lib()  # fail here, loudly, if the CUDA library is missing
    return muillm_engine_ptr()


class muillm_synchronizer_ptr:
    pass


def muillm_sync_init():
    return muillm_synchronizer_ptr()


def muillm_item_bool(sync, tensor):
    return bool(tensor.item())


def muillm_item_f16(sync, tensor):
    return float(tensor.item())


def muillm_item_f32(sync, tensor):
    return float(tensor.item())


def muillm_to_cpu(sync, tensor):
    return tensor.cpu()


class muillm_comm_ptr:
    def __init__(self, comm=None, world_size=1, rank=0):
        self.comm = comm
        self.world_size = world_size
        self.rank = rank


def muillm_comm_init(engine, world_size, local_size, rank, local_rank):
    """One process per GPU; ranks of one node find each other through a rendezvous key taken from MUILLM_COMM_KEY or
    MASTER_PORT (csrc/comms/comm.h:12-56 uses local sockets the same way)."""
    if world_size <= 1:
        return muillm_comm_ptr()
    key = os.environ.get("MUILLM_COMM_KEY") or ("muillm" + os.environ.get("MASTER_PORT", "0"))
    return muillm_comm_ptr(MuiCommunicator(rank=rank, world_size=world_size, key=key), world_size, rank)


def _world(comm):
    return 1 if comm is None or comm.comm is None else comm.world_size


def muillm_all_reduce_sum(comm, tensor):
    if _world(comm) > 1:
        tensor.copy_(comm.comm.all_reduce_sum(tensor))
    return tensor


def muillm_broadcast(comm, tensor, src):
    if _world(comm) > 1:
        tensor.copy_(comm.comm.broadcast(tensor, src))
    return tensor


def _parallel_linear(comm, x, weights, norm_weights, epsilon, mul_bias, add_bias, residual, sharding_dim, reduce):
    """csrc/parallel_linear_kernels.cu:50-173: sharding_dim 0 = rows of the weight (outputs stay sharded), 1 = columns
    (partial sums, all-reduced when `reduce`); bias and residual enter on rank 0 only when summing."""
    world = _world(comm)
    if world == 1 or sharding_dim == 0:
        return _linear_any_rows(x, weights, norm_weights, epsilon, mul_bias, add_bias, residual)
    if norm_weights is not None:
        raise RuntimeError("normalizing sharded inputs is unsupported for sharding_dim 1")
    if sharding_dim != 1:
        raise RuntimeError("unsupported sharding dim")
    if reduce and _rows(x) <= _MAX_GEMV_ROWS:
        return comm.comm.parallel_linear(x, weights, mul_bias=mul_bias, add_bias=add_bias, residual=residual)
    first = comm.rank == 0
    y = _linear_any_rows(x, weights, None, 0.0, mul_bias, add_bias if first else None, residual if first else None)
    if reduce:
        y = comm.comm.all_reduce_sum(y)
    return y


def muillm_parallel_linear_forward(engine, comm, x, weights, norm_weights=None, epsilon=0.0, mul_bias=None,
                                   add_bias=None, residual=None, sharding_dim=1, reduce=False):
    return _parallel_linear(comm, x, weights, norm_weights, epsilon, mul_bias, add_bias, residual, sharding_dim, reduce)


def muillm_parallel_gateupsilu_forward(engine, comm, norm_weights, epsilon, gate_weights, up_weights, down_weights,
                                       residual, x, reduce=True):
    """Row-sharded gate/up, column-sharded down (csrc/parallel_gateup_kernels.cu:6-112)."""
    world = _world(comm)
    if world == 1:
        return _mlp_any_rows(norm_weights, epsilon, gate_weights, up_weights, down_weights, residual, x)
    if reduce and _rows(x) <= _MAX_GEMV_ROWS:
        return comm.comm.parallel_mlp(x, norm_weights, epsilon, gate_weights, up_weights, down_weights,
                                      residual=residual)
    y = _mlp_any_rows(norm_weights, epsilon, gate_weights, up_weights, down_weights,
                      residual if comm.rank == 0 else None, x)
    return comm.comm.all_reduce_sum(y) if reduce else y


muillm_parallel_gateupsilu_split_forward = muillm_parallel_gateupsilu_forward


def muillm_parallel_gateupsilumoe_forward(engine, comm, num_shared_experts, num_dynamic_experts, norm_weights, epsilon,
                                          gate_weights, up_weights, down_weights, residual, x, router_scores,
                                          router_indices, reduce=True):
    """csrc/parallel_gateupmoe_kernels.cu:6-125."""
    world = _world(comm)
    if world == 1:
        return ops.muillm_gateupsilumoe_forward(engine, num_shared_experts, num_dynamic_experts, norm_weights,
                                                epsilon, gate_weights, up_weights, down_weights, residual, x,
                                                router_scores, router_indices)
    if reduce:
        return comm.comm.parallel_moe_mlp(num_shared_experts, num_dynamic_experts, norm_weights, epsilon,
                                          gate_weights, up_weights, down_weights, residual, x, router_scores,
                                          router_indices)
    return ops.muillm_gateupsilumoe_forward(engine, num_shared_experts, num_dynamic_experts, norm_weights, epsilon,
                                            gate_weights, up_weights, down_weights,
                                            residual if comm.rank == 0 else None, x, router_scores, router_indices)


muillm_parallel_gateupsilumoe_split_forward = muillm_parallel_gateupsilumoe_forward

# ---- module handles (csrc/modules/*.cpp) -------------------------------------------------------------------------


class _Handle:
    def release(self):
        for k in list(self.__dict__):
            setattr(self, k, None)


class muillm_linear_module_ptr(_Handle):
    def __init__(self, weights, norm_weights, epsilon, mul_bias, add_bias):
        self.weights, self.norm_weights, self.epsilon = weights, norm_weights, epsilon
        self.mul_bias, self.add_bias = mul_bias, add_bias

    def forward(self, inputs, residual=None):
        return _linear_any_rows(inputs, self.weights, self.norm_weights, self.epsilon, self.mul_bias, self.add_bias,
                                residual)


def muillm_linear_module_init(engine, weights, norm_weights=None, epsilon=0.0, mul_bias=None, add_bias=None):
    return muillm_linear_module_ptr(weights, norm_weights, epsilon, mul_bias, add_bias)


def muillm_linear_module_deinit(module):
    module.release()


def muillm_linear_module_forward(module, inputs, residual=None):
    return module.forward(inputs, residual)


class muillm_embedding_module_ptr(_Handle):
    def __init__(self, weights):
        self.weights = weights

    def forward(self, inputs):
        if _not_dispatchable_on_gpu(self.weights) and inputs.is_cuda:
            return F.embedding(inputs, self.weights)
        return ops.muillm_embedding_forward(self.weights, inputs)


def muillm_embedding_module_init(engine, weights):
    return muillm_embedding_module_ptr(weights)


def muillm_embedding_module_deinit(module):
    module.release()


def muillm_embedding_module_forward(module, inputs):
    return module.forward(inputs)


class muillm_parallel_linear_module_ptr(_Handle):
    def __init__(self, comm, weights, norm_weights, epsilon, mul_bias, add_bias, sharding_dim):
        self.comm, self.weights, self.norm_weights, self.epsilon = comm, weights, norm_weights, epsilon
        self.mul_bias, self.add_bias, self.sharding_dim = mul_bias, add_bias, sharding_dim

    def forward(self, inputs, residual=None, collect_outputs=False):
        if collect_outputs and self.sharding_dim == 0 and _world(self.comm) > 1:
            raise RuntimeError("all_gather is not implemented")
        return _parallel_linear(self.comm, inputs, self.weights, self.norm_weights, self.epsilon, self.mul_bias,
                                self.add_bias, residual, self.sharding_dim, collect_outputs)


def muillm_parallel_linear_module_init(engine, comm, weights, norm_weights=None, epsilon=0.0, mul_bias=None,
                                       add_bias=None, sharding_dim=1):
    return muillm_parallel_linear_module_ptr(comm, weights, norm_weights, epsilon, mul_bias, add_bias, sharding_dim)


def muillm_parallel_linear_module_deinit(module):
    module.release()


def muillm_parallel_linear_module_forward(module, inputs, residual=None, reduce=False):
    return module.forward(inputs, residual, reduce)


class muillm_parallel_multilinear_module_ptr(_Handle):
    """One packed projection + views of its output (csrc/modules/parallel_multilinear_module.cpp:24-69)."""

    def __init__(self, comm, linear, slices, sharding_dim):
        self.comm, self.linear, self.slices, self.sharding_dim = comm, linear, list(slices), sharding_dim

    def forward(self, inputs, collect_outputs):
        if self.sharding_dim == 1:
            out = self.linear.forward(inputs, None, collect_outputs)
            return [out[..., a:b] for a, b in self.slices]
        out = self.linear.forward(inputs, None, False)
        parts = [out[..., a:b] for a, b in self.slices]
        if collect_outputs and _world(self.comm) > 1:
            raise RuntimeError("all_gather is not implemented")
        return parts


def muillm_parallel_multilinear_module_init(engine, comm, linear, slices, sharding_dim):
    return muillm_parallel_multilinear_module_ptr(comm, linear, slices, sharding_dim)


def muillm_parallel_multilinear_module_deinit(module):
    module.release()


def muillm_parallel_multilinear_module_forward(module, input, collect_outputs):
    return module.forward(input, collect_outputs)


class muillm_parallel_igateupdownmlp_module_ptr(_Handle):
    def __init__(self, comm, method, norm_weights, gate_weights, up_weights, down_weights, variance_epsilon):
        if method not in (GATEUPSILU_FUSED, GATEUPSILU_SPLIT):
            raise RuntimeError("Unsupported method")
        self.comm, self.norm_weights, self.epsilon = comm, norm_weights, variance_epsilon
        self.gate_weights, self.up_weights, self.down_weights = gate_weights, up_weights, down_weights

    def forward(self, inputs, residual=None, reduce=True):
        return muillm_parallel_gateupsilu_forward(None, self.comm, self.norm_weights, self.epsilon, self.gate_weights,
                                                  self.up_weights, self.down_weights, residual, inputs, reduce)


def muillm_parallel_gateupdownmlp_module_init(engine, comm, method, norm_weights, gate_weights, up_weights,
                                              down_weights, variance_epsilon):
    return muillm_parallel_igateupdownmlp_module_ptr(comm, method, norm_weights, gate_weights, up_weights,
                                                     down_weights, variance_epsilon)


def muillm_parallel_gateupdownmlp_module_deinit(module):
    module.release()


def muillm_parallel_gateupdownmlp_module_forward(module, inputs, residual=None, reduce=True):
    return module.forward(inputs, residual, reduce)


class muillm_parallel_gateupdownmlpmoe_module_ptr(_Handle):
    """Router (a linear with the layer norm fused in) -> top-k sigmoid -> expert MLPs
    (csrc/modules/parallel_gateupmoe_module.cpp:39-72). The router sees the inputs only; the reference's C++ module
    also hands it the residual, which its Python path (muillm/modules/moe/gateupdownmlpmoe.py:273-275) does not."""

    def __init__(self, comm, router, num_shared_experts, num_dynamic_experts, num_routed_experts, norm_weights,
                 gate_weights, up_weights, down_weights, variance_epsilon):
        self.comm, self.router = comm, router
        self.num_shared_experts, self.num_dynamic_experts = num_shared_experts, num_dynamic_experts
        self.num_routed_experts = num_routed_experts
        self.norm_weights, self.epsilon = norm_weights, variance_epsilon
        self.gate_weights, self.up_weights, self.down_weights = gate_weights, up_weights, down_weights

    def forward(self, inputs, residual=None, reduce=True):
        if _rows(inputs) != 1:
            raise RuntimeError("the MoE kernels take one token at a time")
        logits = self.router.forward(inputs)
        scores, indices = ops.muillm_topk_sigmoid_forward(logits, self.num_routed_experts)
        return muillm_parallel_gateupsilumoe_forward(None, self.comm, self.num_shared_experts,
                                                     self.num_dynamic_experts, self.norm_weights, self.epsilon,
                                                     self.gate_weights, self.up_weights, self.down_weights, residual,
                                                     inputs, scores.reshape(-1), indices.reshape(-1), reduce)


def muillm_parallel_gateupdownmlpmoe_module_init(engine, comm, router, num_shared_experts, num_dynamic_experts,
                                                 num_routed_experts, norm_weights, gate_weights, up_weights,
                                                 down_weights, variance_epsilon):
    return muillm_parallel_gateupdownmlpmoe_module_ptr(comm, router, num_shared_experts, num_dynamic_experts,
                                                       num_routed_experts, norm_weights, gate_weights, up_weights,
                                                       down_weights, variance_epsilon)


def muillm_parallel_gateupdownmlpmoe_module_deinit(module):
    module.release()


def muillm_parallel_gateupdownmlpmoe_module_forward(module, inputs, residual=None, reduce=True):
    return module.forward(inputs, residual, reduce)


# ---- KV caches (csrc/modules/kvcache.h, static_kvcache.cpp, dynamic_kvcache.cpp, hybrid_chunked_kvcache.cpp) ---------


class muillm_kvcache_module_ptr(_Handle):
    STATIC, DYNAMIC, HYBRID_CHUNKED = 0, 1, 2

    def __init__(self, kind, key_cache, value_cache, seen_tokens):
        self.kind = kind
        self.key_cache, self.value_cache = list(key_cache), list(value_cache)
        self._seen_tokens = int(seen_tokens)

    def get_set_seen_tokens(self, seen_tokens):
        if seen_tokens > self._seen_tokens:
            self._seen_tokens = int(seen_tokens)
        return self._seen_tokens


class _HybridChunkedCache(muillm_kvcache_module_ptr):
    def __init__(self, key_cache, value_cache, is_sliding, window_size, seen_tokens):
        super().__init__(self.HYBRID_CHUNKED, key_cache, value_cache, seen_tokens)
        self.is_sliding, self.window_size = list(is_sliding), int(window_size)

    def update(self, key_states, value_states, cache_positions, layer_index):
        """csrc/modules/hybrid_chunked_kvcache.cpp:23-77: the token count moves with layer 0; sliding layers keep a
        chronological window, the others a static cache."""
        T = key_states.shape[-2]
        if layer_index == 0:
            self._seen_tokens += T
        seen = self._seen_tokens
        if self.is_sliding[layer_index]:
            k_out, v_out = ops.muillm_sliding_kvcache_update(key_states, value_states, self.key_cache[layer_index],
                                                             self.value_cache[layer_index], cache_positions, seen)
            if seen != T and seen > self.window_size:
                self.key_cache[layer_index], self.value_cache[layer_index] = k_out, v_out
            return k_out, v_out
        return ops.muillm_static_kvcache_update(key_states, value_states, self.key_cache[layer_index],
                                                self.value_cache[layer_index], cache_positions, seen)


def muillm_kvcache_module_get_set_seen_tokens(module, seen_tokens):
    return module.get_set_seen_tokens(seen_tokens)


def muillm_static_kvcache_module_init(engine, key_cache, value_cache, seen_tokens):
    return muillm_kvcache_module_ptr(muillm_kvcache_module_ptr.STATIC, key_cache, value_cache, seen_tokens)


def _sync_back(module, kind, what):
    if module.kind != kind:
        raise RuntimeError(f"expected a {what} cache")
    return module.key_cache, module.value_cache


def muillm_static_kvcache_module_deinit(module):
    module.release()


def muillm_static_kvcache_module_sync_back(module):
    return _sync_back(module, muillm_kvcache_module_ptr.STATIC, "static")


def muillm_dynamic_kvcache_module_init(engine, key_cache, value_cache, seen_tokens):
    return muillm_kvcache_module_ptr(muillm_kvcache_module_ptr.DYNAMIC, key_cache, value_cache, seen_tokens)


def muillm_dynamic_kvcache_module_deinit(module):
    module.release()


def muillm_dynamic_kvcache_module_sync_back(module):
    return _sync_back(module, muillm_kvcache_module_ptr.DYNAMIC, "dynamic")


def muillm_hybrid_chunked_kvcache_module_init(engine, key_cache, value_cache, is_sliding, window_size, seen_tokens):
    return _HybridChunkedCache(key_cache, value_cache, is_sliding, window_size, seen_tokens)


def muillm_hybrid_chunked_kvcache_module_update(module, key_states, value_states, cache_position, layer_index):
    if module.kind != muillm_kvcache_module_ptr.HYBRID_CHUNKED:
        raise RuntimeError("expected a hybrid chunked cache")
    return module.update(key_states, value_states, cache_position, layer_index)


def muillm_hybrid_chunked_kvcache_module_deinit(module):
    module.release()


def muillm_hybrid_chunked_kvcache_module_sync_back(module):
    return _sync_back(module, muillm_kvcache_module_ptr.HYBRID_CHUNKED, "hybrid chunked")


# ---- rotary embedding, attention, decoder, decoder stack ----------------------------------------------------------


class muillm_rotary_embedding_module_ptr(_Handle):
    """csrc/modules/rotary_module.cpp:25-125. cos/sin tables are [S, D]; the kernels index them with position_ids
    directly, so no per-step gather (`muillm_compute_rotary_embed_positions`) is launched."""

    def __init__(self, layer_idx, cos_cached, sin_cached):
        self.layer_idx, self.cos_cached, self.sin_cached = layer_idx, cos_cached, sin_cached

    def compute_rotary_pos_emb(self, x, position_ids):
        return self.cos_cached, self.sin_cached

    def forward(self, cache, q_in, k_in, v_in, position_ids, cos_sin, cache_positions):
        cos, sin = cos_sin if cos_sin is not None else self.compute_rotary_pos_emb(k_in, position_ids)
        position_ids = position_ids.contiguous()
        if cache is None:
            q, k = ops.muillm_rope_forward_no_cache(position_ids, cos, sin, q_in, k_in)
            return q, k, v_in
        layer = self.layer_idx
        if layer == 0:
            cache._seen_tokens += k_in.shape[-2]
        if cache.kind == muillm_kvcache_module_ptr.STATIC:
            return ops.muillm_rope_forward_static_cache(position_ids, cos, sin, q_in, k_in, v_in,
                                                        cache.key_cache[layer], cache.value_cache[layer],
                                                        cache_positions, cache._seen_tokens)
        if cache.kind == muillm_kvcache_module_ptr.DYNAMIC:
            q, k_all, v_all = muillm_rope_forward_dynamic_cache(position_ids, cos, sin, q_in, k_in, v_in,
                                                                cache.key_cache[layer], cache.value_cache[layer])
            cache.key_cache[layer], cache.value_cache[layer] = k_all, v_all
            return q, k_all, v_all
        raise RuntimeError("unsupported cache type")


def muillm_rotary_embedding_module_init(engine, layer_idx, cos_cached, sin_cached):
    return muillm_rotary_embedding_module_ptr(layer_idx, cos_cached, sin_cached)


def muillm_rotary_embedding_module_deinit(module):
    module.release()


def muillm_rotary_embedding_module_forward(module, cache, q_in, k_in, v_in, position_ids, cos_sin, cache_positions):
    return module.forward(cache, q_in, k_in, v_in, position_ids, cos_sin, cache_positions)


def _decode_attention(q, k, v, m):
    if m is not None:
        return ops.muillm_causal_transformer_decoding_masked(q, k, v, m)
    return ops.muillm_causal_transformer_decoding_no_mask(q, k, v)


def _split_heads(x, heads, head_dim):
    """[B, T, heads*D] (possibly a strided slice of the packed QKV output) -> [B, heads, T, D] view
    (csrc/modules/parallel_attention_module.cpp:63-77)."""
    bsz, q_len = x.shape[0], x.shape[1]
    if q_len == 1:
        return x.view(bsz, heads, q_len, head_dim)
    return x.view(bsz, q_len, heads, head_dim).transpose(1, 2)


class muillm_parallel_attention_module_ptr(_Handle):
    def __init__(self, comm, rotary, o_proj, num_tp_heads, num_tp_key_value_heads, head_dim):
        self.comm, self.rotary, self.o_proj = comm, rotary, o_proj
        self.num_tp_heads, self.num_tp_key_value_heads, self.head_dim = num_tp_heads, num_tp_key_value_heads, head_dim

    def forward(self, q, k, v, m=None, residual=None):
        attn = _decode_attention(q, k, v, m)
        return self.o_proj.forward(attn, residual, True)

    def rope_forward(self, cache, q, k, v, m, residual, position_ids, cos_sin, cache_positions):
        q_r = _split_heads(q, self.num_tp_heads, self.head_dim)
        k_r = _split_heads(k, self.num_tp_key_value_heads, self.head_dim)
        v_r = _split_heads(v, self.num_tp_key_value_heads, self.head_dim)
        q_rot, k_all, v_all = self.rotary.forward(cache, q_r, k_r, v_r, position_ids, cos_sin, cache_positions)
        return self.forward(q_rot, k_all, v_all, m, residual)


def muillm_parallel_attention_module_init(engine, comm, rotary, o_proj, num_tp_heads, num_tp_key_value_heads,
                                          head_dim):
    return muillm_parallel_attention_module_ptr(comm, rotary, o_proj, num_tp_heads, num_tp_key_value_heads, head_dim)


def muillm_parallel_attention_module_deinit(module):
    module.release()


def muillm_parallel_attention_module_forward(module, q, k, v, m=None, residual=None):
    return module.forward(q, k, v, m, residual)


def muillm_parallel_attention_module_rope_forward(module, cache, q, k, v, m, residual, position_ids, cos_sin,
                                                  cache_positions):
    return module.rope_forward(cache, q, k, v, m, residual, position_ids, cos_sin, cache_positions)


class muillm_parallel_llama4_attention_module_ptr(_Handle):
    """csrc/modules/parallel_llama4_attention_module.cpp:45-134; rope, QK norm and temperature scale are one launch."""

    def __init__(self, comm, o_proj, num_tp_heads, num_tp_key_value_heads, head_dim, use_rope, use_qk_norm,
                 norm_epsilon, use_temperature_tuning, attention_scale, floor_scale, layer_index):
        self.comm, self.o_proj = comm, o_proj
        self.num_tp_heads, self.num_tp_key_value_heads, self.head_dim = num_tp_heads, num_tp_key_value_heads, head_dim
        self.use_rope, self.use_qk_norm, self.norm_epsilon = use_rope, use_qk_norm, norm_epsilon
        self.use_temperature_tuning, self.attention_scale, self.floor_scale = (use_temperature_tuning, attention_scale,
                                                                               floor_scale)
        self.layer_index = layer_index

    def forward(self, q, k, v, m=None, residual=None):
        attn = _decode_attention(q, k, v, m)
        return self.o_proj.forward(attn, residual, True)

    def rope_forward(self, cache, q, k, v, m, residual, position_embeds, cache_positions):
        q_r = _split_heads(q, self.num_tp_heads, self.head_dim)
        k_r = _split_heads(k, self.num_tp_key_value_heads, self.head_dim)
        v_r = _split_heads(v, self.num_tp_key_value_heads, self.head_dim)
        if self.use_rope or self.use_qk_norm or self.use_temperature_tuning:
            q_r, k_r = ops.llama4_qk_prologue(
                q_r, k_r, position_embeds=position_embeds if self.use_rope else None,
                qk_norm_eps=self.norm_epsilon if self.use_qk_norm else None,
                cache_position=cache_positions if self.use_temperature_tuning else None,
                attn_scale=self.attention_scale, floor_scale=self.floor_scale)
        if cache is None or cache.kind != muillm_kvcache_module_ptr.HYBRID_CHUNKED:
            raise RuntimeError("expected a hybrid chunked cache")
        k_all, v_all = cache.update(k_r, v_r, cache_positions, self.layer_index)
        return self.forward(q_r, k_all, v_all, m, residual)


def muillm_parallel_llama4_attention_module_init(engine, comm, o_proj, num_tp_heads, num_tp_key_value_heads, head_dim,
                                                 use_rope, use_qk_norm, norm_epsilon, use_temperature_tuning,
                                                 attention_scale, floor_scale, layer_index):
    return muillm_parallel_llama4_attention_module_ptr(comm, o_proj, num_tp_heads, num_tp_key_value_heads, head_dim,
                                                       use_rope, use_qk_norm, norm_epsilon, use_temperature_tuning,
                                                       attention_scale, floor_scale, layer_index)


def muillm_parallel_llama4_attention_module_deinit(module):
    module.release()


def muillm_parallel_llama4_attention_module_forward(module, q, k, v, m=None, residual=None):
    return module.forward(q, k, v, m, residual)


def muillm_parallel_llama4_attention_module_rope_forward(module, cache, q, k, v, m, residual, position_embeds,
                                                         cache_positions):
    return module.rope_forward(cache, q, k, v, m, residual, position_embeds, cache_positions)


class muillm_parallel_decoder_module_ptr(_Handle):
    """csrc/modules/parallel_decoder_module.cpp:22-62."""

    def __init__(self, comm, multilinear, attention, mlp):
        self.comm, self.multilinear, self.attention, self.mlp = comm, multilinear, attention, mlp

    def forward(self, cache, h, m, position_ids, cos_sin, cache_positions):
        q, k, v = self.multilinear.forward(h, False)
        attn_out = self.attention.rope_forward(cache, q, k, v, m, h, position_ids, cos_sin, cache_positions)
        return self.mlp.forward(attn_out, attn_out, True)


def muillm_parallel_decoder_module_init(engine, comm, multilinear, attention, mlp):
    return muillm_parallel_decoder_module_ptr(comm, multilinear, attention, mlp)


def muillm_parallel_decoder_module_deinit(module):
    module.release()


def muillm_parallel_decoder_module_forward(module, cache, h, m, position_ids, cos_sin, cache_positions):
    return module.forward(cache, h, m, position_ids, cos_sin, cache_positions)


class muillm_parallel_llama4_decoder_module_ptr(_Handle):
    """csrc/modules/parallel_llama4_decoder_module.cpp:25-66."""

    def __init__(self, comm, multilinear, attention, mlp, use_chunked_attention):
        self.comm, self.multilinear, self.attention, self.mlp = comm, multilinear, attention, mlp
        self.use_chunked_attention = use_chunked_attention

    def forward(self, cache, h, mask, chunked_mask, position_embeds, cache_positions):
        q, k, v = self.multilinear.forward(h, False)
        m = chunked_mask if self.use_chunked_attention else mask
        attn_out = self.attention.rope_forward(cache, q, k, v, m, h, position_embeds, cache_positions)
        return self.mlp.forward(attn_out, attn_out, True)


def muillm_parallel_llama4_decoder_module_init(engine, comm, multilinear, attention, mlp, use_chunked_attention):
    return muillm_parallel_llama4_decoder_module_ptr(comm, multilinear, attention, mlp, use_chunked_attention)


def muillm_parallel_llama4_decoder_module_deinit(module):
    module.release()


def muillm_parallel_llama4_decoder_module_forward(module, cache, h, mask, chunked_mask, position_embeds,
                                                  cache_positions):
    return module.forward(cache, h, mask, chunked_mask, position_embeds, cache_positions)


class _FusedLayers:
    """The decoder layers of a stack as ONE call into the C decode stack (mui_llama_stack_forward_hidden) instead of
    ~10 Python-dispatched launches per layer. Built from the module handles' own tensors (nothing is copied) for a
    given static cache; valid for one new token per sequence without an attention mask."""

    def __init__(self, stack, cache, batch):
        import ctypes
        import math
        from ctypes import c_void_p

        from . import capi

        lib = capi.lib()
        decs = stack.decoders
        first = decs[0]
        att, lin = first.attention, first.multilinear.linear
        w_qkv = lin.weights
        dt, dev = w_qkv.dtype, w_qkv.device
        Hq, Hkv, D = att.num_tp_heads, att.num_tp_key_value_heads, att.head_dim
        hidden = w_qkv.shape[1]
        inter = first.mlp.gate_weights.shape[0]
        max_seq = cache.key_cache[0].shape[2]
        embed = stack.embed_tokens.weights
        cos, sin = stack.rotary_embedding.cos_cached, stack.rotary_embedding.sin_cached
        self.keep = [cos, sin, embed]
        cfg = capi.LlamaConfig(capi.MUI_F16 if dt == torch.float16 else capi.MUI_BF16, len(decs), hidden, inter, Hq,
                               Hkv, D, embed.shape[0], max_seq, batch, float(lin.epsilon), 1.0 / math.sqrt(D), 0, 0)
        nbytes = lib.mui_llama_stack_scratch_bytes(ctypes.byref(cfg))
        if nbytes == 0:
            raise RuntimeError("muillm_b200: " + lib.mui_last_error().decode())
        self.scratch = torch.zeros(nbytes, dtype=torch.uint8, device=dev)

        def arr(tensors):
            self.keep.extend(tensors)
            return (c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])

        self.arrays = [arr([d.multilinear.linear.weights for d in decs]), arr([d.attention.o_proj.weights for d in decs]),
                       arr([d.mlp.gate_weights for d in decs]), arr([d.mlp.up_weights for d in decs]),
                       arr([d.mlp.down_weights for d in decs]), arr([d.multilinear.linear.norm_weights for d in decs]),
                       arr([d.mlp.norm_weights for d in decs]), arr(list(cache.key_cache)),
                       arr(list(cache.value_cache))]
        # final norm and lm_head stay with the caller: the two slots only have to be non-null
        w = capi.LlamaWeights(embed.data_ptr(), decs[0].mlp.norm_weights.data_ptr(), embed.data_ptr(), cos.data_ptr(),
                              sin.data_ptr(), *self.arrays)
        h = c_void_p()
        capi.check(lib.mui_llama_stack_create(ctypes.byref(cfg), ctypes.byref(w), self.scratch.data_ptr(),
                                              self.scratch.numel(), ctypes.byref(h)))
        self.lib, self.h, self.hidden, self.batch, self.dtype = lib, h, hidden, batch, dt
        self.comm = stack.comm.comm if stack.comm is not None else None
        if self.comm is not None:
            capi.check(lib.mui_llama_stack_set_comm(h, self.comm.handle))
        self.cache_ptrs = [t.data_ptr() for t in cache.key_cache]
        from .capi import MUI_FLAG_PDL
        self.flags = MUI_FLAG_PDL

    def __del__(self):
        h = getattr(self, "h", None)
        if h:
            self.lib.mui_llama_stack_destroy(h)

    def forward(self, input_ids, input_embeds, position_ids, cache_positions, seen_tokens):
        from . import capi

        out = torch.empty((self.batch, 1, self.hidden), dtype=self.dtype, device=self.scratch.device)
        tok = None if input_embeds is not None else input_ids.reshape(-1).contiguous()
        emb = input_embeds.contiguous() if input_embeds is not None else None
        pos = position_ids.reshape(-1).contiguous()
        capi.check(self.lib.mui_llama_stack_forward_hidden(
            self.h, torch.cuda.current_stream().cuda_stream, None if tok is None else tok.data_ptr(),
            None if emb is None else emb.data_ptr(), pos.data_ptr(), cache_positions.data_ptr(), int(seen_tokens),
            out.data_ptr(), self.flags))
        return out


# the decoder-stack handle runs a decode step as one call into the C decode stack where the modules allow it
FUSED_DECODER_STACK = True


class muillm_parallel_decoder_stack_ptr(_Handle):
    """csrc/modules/parallel_decoder_stack.cpp:22-45: embedding (unless embeddings are given), the rotary tables
    once, then the decoders in order. One new token per sequence on a static cache without a mask — the decode step —
    runs as a single call into the C decode stack (module attribute FUSED_DECODER_STACK = False keeps the per-module
    path, which the tests use as a cross-check)."""

    def __init__(self, comm, embed_tokens, rotary_embedding, decoders):
        self.comm, self.embed_tokens, self.rotary_embedding, self.decoders = (comm, embed_tokens, rotary_embedding,
                                                                              list(decoders))
        self._fused = None

    def _fused_for(self, cache, batch, q_len, m):
        if not FUSED_DECODER_STACK:
            return None
        if q_len != 1 or m is not None or batch > 8 or cache is None or self.embed_tokens is None or \
                self.rotary_embedding is None or cache.kind != muillm_kvcache_module_ptr.STATIC:
            return None
        f = self._fused
        if f is not None and f.batch == batch and f.cache_ptrs == [t.data_ptr() for t in cache.key_cache]:
            return f
        for d in self.decoders:
            lin = getattr(getattr(d, "multilinear", None), "linear", None)
            ok = (isinstance(d, muillm_parallel_decoder_module_ptr) and lin is not None and
                  lin.norm_weights is not None and lin.mul_bias is None and lin.add_bias is None and
                  d.multilinear.sharding_dim == 0 and len(d.multilinear.slices) == 3 and
                  d.attention.o_proj.sharding_dim == 1 and d.attention.o_proj.add_bias is None and
                  d.attention.o_proj.mul_bias is None and d.mlp.norm_weights is not None and
                  isinstance(d.mlp, muillm_parallel_igateupdownmlp_module_ptr) and
                  lin.weights.dtype in (torch.float16, torch.bfloat16) and lin.weights.is_cuda and
                  d.attention.rotary is not None)
            if not ok:
                return None
        if self.rotary_embedding.cos_cached.dim() != 2 or self.rotary_embedding.cos_cached.dtype != \
                self.decoders[0].multilinear.linear.weights.dtype:
            return None
        self._fused = _FusedLayers(self, cache, batch)
        return self._fused

    def forward(self, cache, input_ids, input_embeds, m, position_ids, cache_positions):
        batch = (input_embeds if input_embeds is not None else input_ids).shape[0]
        q_len = (input_embeds if input_embeds is not None else input_ids).shape[1]
        fused = self._fused_for(cache, batch, q_len, m)
        if fused is not None:
            cache._seen_tokens += 1  # the per-module path moves the count in layer 0's rotary module
            return fused.forward(input_ids, input_embeds, position_ids, cache_positions, cache._seen_tokens)
        h = input_embeds if input_embeds is not None else self.embed_tokens.forward(input_ids)
        cos_sin = None
        if self.rotary_embedding is not None:
            cos_sin = self.rotary_embedding.compute_rotary_pos_emb(h, position_ids)
        for decoder in self.decoders:
            h = decoder.forward(cache, h, m, position_ids, cos_sin, cache_positions)
        return h


def muillm_parallel_decoder_stack_init(engine, comm, embed_tokens_module, rotary_emb_module, decoders):
    return muillm_parallel_decoder_stack_ptr(comm, embed_tokens_module, rotary_emb_module, decoders)


def muillm_parallel_decoder_stack_deinit(module):
    module.release()


def muillm_parallel_decoder_stack_forward(module, cache, input_ids, input_embeds, m, position_ids, cache_positions):
    return module.forward(cache, input_ids, input_embeds, m, position_ids, cache_positions)


class muillm_parallel_llama4_decoder_stack_ptr(_Handle):
    """csrc/modules/parallel_llama4_decoder_stack.cpp."""

    def __init__(self, comm, decoders):
        self.comm, self.decoders = comm, list(decoders)

    def forward(self, cache, h, mask, chunked_mask, position_embeds, cache_positions):
        for decoder in self.decoders:
            h = decoder.forward(cache, h, mask, chunked_mask, position_embeds, cache_positions)
        return h


def muillm_parallel_llama4_decoder_stack_init(engine, comm, decoders):
    return muillm_parallel_llama4_decoder_stack_ptr(comm, decoders)


def muillm_parallel_llama4_decoder_stack_deinit(module):
    module.release()


def muillm_parallel_llama4_decoder_stack_forward(module, cache, h, mask, chunked_mask, position_embeds,
                                                 cache_positions):
    return module.forward(cache, h, mask, chunked_mask, position_embeds, cache_positions)


# the pybind handle classes the reference exports by name (csrc/module.cpp:281-300 and the module headers)
muillm_linear_module_ptr_t = muillm_linear_module_ptr
muillm_embedding_module_ptr_t = muillm_embedding_module_ptr
muillm_parallel_linear_module_ptr_t = muillm_parallel_linear_module_ptr
muillm_parallel_multilinear_module_ptr_t = muillm_parallel_multilinear_module_ptr
muillm_parallel_igateupdownmlp_module_ptr_t = muillm_parallel_igateupdownmlp_module_ptr
muillm_kvcache_module_ptr_t = muillm_kvcache_module_ptr
muillm_rotary_embedding_module_ptr_t = muillm_rotary_embedding_module_ptr
muillm_parallel_attention_module_ptr_t = muillm_parallel_attention_module_ptr
muillm_parallel_llama4_attention_module_ptr_t = muillm_parallel_llama4_attention_module_ptr
muillm_parallel_decoder_module_ptr_t = muillm_parallel_decoder_module_ptr
muillm_parallel_llama4_decoder_module_ptr_t = muillm_parallel_llama4_decoder_module_ptr
muillm_parallel_decoder_stack_ptr_t = muillm_parallel_decoder_stack_ptr
muillm_parallel_llama4_decoder_stack_ptr_t = muillm_parallel_llama4_decoder_stack_ptr
