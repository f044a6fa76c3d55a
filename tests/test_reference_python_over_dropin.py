"""Where a checkout of the reference is given in $MUILLM_REFERENCE, its own Python modules are imported with the
drop-in registered as `muillm_ext` and built the way `init_engine` builds them, which goes through the drop-in's
engine / module-handle life cycle (no GPU here, so nothing is computed). Skipped elsewhere."""
import importlib
import os
import sys

import pytest
import torch

REF = os.environ.get("MUILLM_REFERENCE", "")
pytestmark = pytest.mark.skipif(not (REF and os.path.isdir(os.path.join(REF, "muillm"))),
                                reason="no reference checkout at $MUILLM_REFERENCE")


@pytest.fixture(scope="module")
def ref_modules():
    from muillm_b200 import muillm_ext as shim

    saved_ext, saved_path = sys.modules.get("muillm_ext"), list(sys.path)
    sys.modules["muillm_ext"] = shim
    sys.path.insert(0, REF)
    try:
        yield shim
    finally:
        sys.path[:] = saved_path
        if saved_ext is None:
            sys.modules.pop("muillm_ext", None)
        else:
            sys.modules["muillm_ext"] = saved_ext
        for name in [n for n in sys.modules if n == "muillm" or n.startswith("muillm.")]:
            del sys.modules[name]


IMPORTABLE = ["muillm.engineconfig", "muillm.modules.linear", "muillm.modules.multilinear",
              "muillm.modules.gateupdownmlp", "muillm.modules.norm.rmsnorm", "muillm.modules.norm.qkl2norm",
              "muillm.modules.topk", "muillm.modules.moe.gateupdownmlpmoe",
              "muillm.modules.attention.causaltransformerdecoding", "muillm.modules.attention.temperaturetuning",
              "muillm.modules.decoder.paralleldecoderstack", "muillm.comms.communicator",
              "muillm.synchronization.synchronizer", "muillm.sampling.generation", "muillm.modules.quantized.int8linear",
              "muillm.modules.quantized.int8gateupdownmlp", "muillm.modules.parallellinear", "muillm.modules.reduce"]


def test_reference_modules_import_over_the_dropin(ref_modules):
    for name in IMPORTABLE:
        importlib.import_module(name)


def test_reference_linear_module_life_cycle_on_cpu(ref_modules, monkeypatch):
    from muillm.engineconfig import MuiEngineConfig
    from muillm.modules.linear import MuiLinear

    monkeypatch.setattr(torch.cuda, "device_count", lambda: 1)  # the constructor only compares against the count
    cfg = MuiEngineConfig(tensor_parallelism=1)
    assert isinstance(cfg.cpp_engine, ref_modules.muillm_engine_ptr)
    lin = MuiLinear(cfg, in_features=32, out_features=16, bias=True, variance_epsilon=1e-5, normalize=True,
                    dtype=torch.float32)
    lin.finalize_init()
    handle = lin.cpp_module
    assert isinstance(handle, ref_modules.muillm_linear_module_ptr) and handle.weights is lin.weight
    # the reference's C++ module would fall back to at::linear for CPU tensors; the drop-in has no CPU path and says so
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        lin(torch.randn(2, 3, 32))
    lin.finalize_deinit()
    assert handle.weights is None


def test_packed_gateup_layout_is_the_references(ref_modules):
    """The pack layout the GPU tests and benchmarks feed to `mui_gateup_silu_w8_packed_forward` is the one the
    reference's own packing code produces (muillm/modules/quantized/int8gateupdownmlp.py:211-230)."""
    from muillm.modules.quantized.int8gateupdownmlp import MuiInt8GateUpDownMLP
    from types import SimpleNamespace

    from parity_utils import reference_gateup_pack

    g = torch.Generator().manual_seed(0)
    I, H, G = 6, 256, 2
    gq = torch.randint(0, 256, (I, H), generator=g, dtype=torch.uint8)
    uq = torch.randint(0, 256, (I, H), generator=g, dtype=torch.uint8)
    gsm = torch.randn(I * G, 2, generator=g).to(torch.float16)
    usm = torch.randn(I * G, 2, generator=g).to(torch.float16)
    gate = SimpleNamespace(weights_uint8=gq, scales_min_vals=gsm)
    up = SimpleNamespace(weights_uint8=uq, scales_min_vals=usm)
    # the two packing methods use no module state: run them on a stand-in instead of building a whole MLP module
    me = SimpleNamespace()
    me._pack_gateup_weights = lambda g_, u_: MuiInt8GateUpDownMLP._pack_gateup_weights(me, g_, u_)
    ref_pack, ref_sm = MuiInt8GateUpDownMLP._pack_gateup_linears(me, gate, up)
    pack, sm = reference_gateup_pack(gq, gsm, uq, usm)
    assert torch.equal(pack, ref_pack) and torch.equal(sm, ref_sm)
    assert ref_pack.is_contiguous() and ref_sm.is_contiguous()

