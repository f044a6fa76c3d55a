"""CPU checks of the Llama-4 host logic: the packed weight layout built from a Hugging Face state dict (fixture
tests/golden/hf_llama4_model.npz) and the tensor-parallel shards, which must tile the un-sharded matrices exactly."""
import os

import numpy as np
import pytest
import torch

from muillm_b200.llama4 import llama4_weights_from_state_dict, shard_llama4_weights

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
CFG = dict(layers=4, hidden=128, expert_intermediate=64, heads=2, kv_heads=1, head_dim=64, vocab=256, experts=4, top_k=1,
           eps=1e-5, rope_theta=500000.0, chunk=8, use_rope=[True, True, True, False], use_qk_norm=True,
           temperature_tuning=True, attn_scale=0.1, floor_scale=4.0)


def _packed():
    d = np.load(os.path.join(GOLD, "hf_llama4_model.npz"))
    sd = {k[3:]: torch.from_numpy(d[k]) for k in d.files if k.startswith("sd/")}
    return sd, llama4_weights_from_state_dict(sd, CFG, dtype=torch.float16, device="cpu")


def test_packed_layout_matches_hf_expert_math():
    """silu(x G^T) * (x U^T) then D over the packed rows of expert e equals HF's bmm over gate_up_proj / down_proj."""
    sd, w = _packed()
    H, I, E = CFG["hidden"], CFG["expert_intermediate"], CFG["experts"]
    g = torch.Generator().manual_seed(0)
    x = torch.randn(1, H, generator=g)
    for l in (0, 3):
        p = f"model.layers.{l}.feed_forward."
        gu, dn = sd[p + "experts.gate_up_proj"].float(), sd[p + "experts.down_proj"].float()
        for e in range(E):
            gate, up = (x @ gu[e]).chunk(2, dim=-1)
            want = (up * torch.nn.functional.silu(gate)) @ dn[e]
            G = w["gate"][l][(1 + e) * I: (2 + e) * I].float()
            U = w["up"][l][(1 + e) * I: (2 + e) * I].float()
            D = w["down"][l][(1 + e) * H: (2 + e) * H].float()
            got = (torch.nn.functional.silu(x @ G.t()) * (x @ U.t())) @ D.t()
            torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-6)
        assert torch.equal(w["gate"][l][:I], sd[p + "shared_expert.gate_proj.weight"])
        assert torch.equal(w["down"][l][:H], sd[p + "shared_expert.down_proj.weight"])
        assert torch.equal(w["router"][l], sd[p + "router.weight"])


@pytest.mark.parametrize("world", [2, 4])
def test_shards_tile_the_unsharded_weights(world):
    H, I, D, E = 64, 16, 8, 3
    cfg = dict(CFG, layers=2, hidden=H, expert_intermediate=I, heads=8, kv_heads=4, head_dim=D, vocab=32, experts=E - 1)
    g = torch.Generator().manual_seed(1)
    rn = lambda *s: torch.randn(*s, generator=g)  # noqa: E731
    L = cfg["layers"]
    w = {"embed": rn(32, H), "lm_head": rn(32, H), "norm": rn(H), "ln1": [rn(H)] * L, "ln2": [rn(H)] * L,
         "router": [rn(E - 1, H) for _ in range(L)], "qkv": [rn((8 + 2 * 4) * D, H) for _ in range(L)],
         "o": [rn(H, 8 * D) for _ in range(L)], "gate": [rn(E * I, H) for _ in range(L)],
         "up": [rn(E * I, H) for _ in range(L)], "down": [rn(E * H, I) for _ in range(L)]}
    shards = [shard_llama4_weights(w, cfg, r, world, shard_lm_head=True) for r in range(world)]
    hq, hkv, il = 8 // world, 4 // world, I // world
    for l in range(L):
        q = torch.cat([s["qkv"][l][: hq * D] for s, _ in shards])
        k = torch.cat([s["qkv"][l][hq * D: (hq + hkv) * D] for s, _ in shards])
        v = torch.cat([s["qkv"][l][(hq + hkv) * D:] for s, _ in shards])
        assert torch.equal(torch.cat([q, k, v]), w["qkv"][l])
        assert torch.equal(torch.cat([s["o"][l] for s, _ in shards], dim=1), w["o"][l])
        gate = torch.cat([s["gate"][l].view(E, il, H) for s, _ in shards], dim=1).reshape(E * I, H)
        down = torch.cat([s["down"][l].view(E, H, il) for s, _ in shards], dim=2).reshape(E * H, I)
        assert torch.equal(gate, w["gate"][l]) and torch.equal(down, w["down"][l])
    assert torch.equal(torch.cat([s["lm_head"] for s, _ in shards]), w["lm_head"])
    assert [c["vocab_offset"] for _, c in shards] == [r * (32 // world) for r in range(world)]
    assert all(c["heads"] == hq and c["kv_heads"] == hkv and c["expert_intermediate"] == il for _, c in shards)
    with pytest.raises(RuntimeError):
        shard_llama4_weights(w, cfg, 0, 3)
