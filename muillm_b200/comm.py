"""Tensor-parallel communicator wrapper (one process per GPU, one node).

Mirrors the reference's `MuiCommunicator` (muillm/comms/communicator.py:104-134: ranks from WORLD_SIZE / RANK /
LOCAL_RANK, `all_reduce_sum`, `broadcast`) on top of mui_comm_*: one-shot push all-reduce over peer memory, bootstrap
over a UNIX socket, and the fused sharded layers (`parallel_linear`, `parallel_mlp`).
"""
import ctypes
import os
from ctypes import c_size_t, c_void_p

import torch

from . import capi
from .ops import _check_input, _dtype_code, _ptr, _rows, _stream


class MuiCommunicator:
    def __init__(self, rank=None, world_size=None, key=None, capacity_elems=1 << 20, timeout_s=60.0):
        self.lib = capi.lib()
        self.rank = int(os.environ.get("RANK", "0")) if rank is None else rank
        self.world_size = int(os.environ.get("WORLD_SIZE", "1")) if world_size is None else world_size
        key = key if key is not None else os.environ.get("MASTER_PORT", "0")
        h = c_void_p()
        capi.check(self.lib.mui_comm_init_local(self.rank, self.world_size, str(key).encode(), capacity_elems,
                                                float(timeout_s), ctypes.byref(h)))
        self._h = h

    def close(self):
        if getattr(self, "_h", None):
            self.lib.mui_comm_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()

    @property
    def handle(self):
        return self._h

    def capacity(self):
        cap = c_size_t(0)
        capi.check(self.lib.mui_comm_info(self._h, None, None, ctypes.byref(cap)))
        return cap.value

    def all_reduce_sum(self, tensor, flags=0, out=None):
        """Returns the sum over ranks of `tensor` (fp16, bf16 or fp32), same shape (csrc/module.cpp
        muillm_all_reduce_sum); written into `out` when given."""
        _check_input(tensor, "tensor")
        if tensor.dtype == torch.float32:
            code = capi.MUI_COMM_F32
        else:
            code = _dtype_code(tensor)
        if out is None:
            out = torch.empty_like(tensor)
        capi.check(self.lib.mui_comm_all_reduce_sum(self._h, _stream(), code, _ptr(tensor), _ptr(out), tensor.numel(),
                                                    flags))
        return out

    def broadcast(self, tensor, src, flags=0):
        """Every rank returns rank `src`'s tensor (any dtype whose byte size is a multiple of 4)."""
        _check_input(tensor, "tensor")
        out = torch.empty_like(tensor)
        capi.check(self.lib.mui_comm_broadcast(self._h, _stream(), int(src), _ptr(tensor), _ptr(out),
                                               tensor.numel() * tensor.element_size(), flags))
        return out

    def parallel_linear(self, x, weights, mul_bias=None, add_bias=None, residual=None, flags=0, out=None):
        """K-sharded linear + fused all-reduce: x [..., K_local], weights [N, K_local] -> [..., N] on every rank;
        add_bias / residual are applied once (rank 0), as muillm/modules/parallellinear.py:464-467 does."""
        for t, n in ((x, "x"), (weights, "weights"), (mul_bias, "mul_bias"), (add_bias, "add_bias"),
                     (residual, "residual")):
            _check_input(t, n)
        N, K = weights.shape
        y = out if out is not None else torch.empty(x.shape[:-1] + (N,), dtype=x.dtype, device=x.device)
        capi.check(self.lib.mui_parallel_linear_forward(
            self._h, _stream(), _dtype_code(x), _rows(x), N, K, None, 0.0, _ptr(weights), _ptr(mul_bias),
            _ptr(add_bias), _ptr(residual), _ptr(x), _ptr(y), flags))
        return y

    def parallel_mlp(self, x, norm_weights, epsilon, gate_weights, up_weights, down_weights, residual=None, flags=0):
        """Sharded MLP: gate/up [I_local, H] local, down [H, I_local] + fused all-reduce
        (muillm_parallel_gateupsilu_forward, csrc/parallel_gateup_kernels.cu:6-112)."""
        for t, n in ((x, "x"), (gate_weights, "gate_weights"), (up_weights, "up_weights"),
                     (down_weights, "down_weights"), (norm_weights, "norm_weights"), (residual, "residual")):
            _check_input(t, n)
        I, H = gate_weights.shape
        B = _rows(x)
        t = torch.empty((B, I), dtype=x.dtype, device=x.device)
        y = torch.empty(x.shape[:-1] + (H,), dtype=x.dtype, device=x.device)
        capi.check(self.lib.mui_parallel_gateupdown_forward(
            self._h, _stream(), _dtype_code(x), B, I, H, _ptr(norm_weights), float(epsilon), _ptr(gate_weights),
            _ptr(up_weights), _ptr(down_weights), _ptr(residual), _ptr(x), _ptr(t), _ptr(y), flags))
        return y

    def parallel_moe_mlp(self, num_shared_experts, num_dynamic_experts, norm_weights, epsilon, gate_weights,
                         up_weights, down_weights, residual, x, router_scores, router_indices, flags=0):
        """Sharded MoE MLP for one token: packed expert shards [(shared + routed) * I_local, H] /
        [(shared + routed) * H, I_local], replicated router outputs, all-reduce fused into the down kernel
        (muillm_parallel_gateupsilumoe_forward, csrc/parallel_gateupmoe_kernels.cu:6-125)."""
        for t, n in ((x, "x"), (gate_weights, "gate_weights"), (up_weights, "up_weights"),
                     (down_weights, "down_weights"), (norm_weights, "norm_weights"), (residual, "residual"),
                     (router_scores, "router_scores"), (router_indices, "router_indices")):
            _check_input(t, n)
        total = num_shared_experts + num_dynamic_experts
        H = x.shape[-1]
        I = gate_weights.shape[0] // total
        top_k = 0 if router_indices is None else router_indices.shape[-1]
        t = torch.empty((num_shared_experts + top_k, I), dtype=x.dtype, device=x.device)
        y = torch.empty_like(x)
        capi.check(self.lib.mui_parallel_moe_mlp_forward(
            self._h, _stream(), _dtype_code(x), num_shared_experts, num_dynamic_experts, top_k, I, H,
            _ptr(norm_weights), float(epsilon), _ptr(gate_weights), _ptr(up_weights), _ptr(down_weights),
            _ptr(residual), _ptr(x), _ptr(router_scores), _ptr(router_indices), _ptr(t), _ptr(y), flags))
        return y
