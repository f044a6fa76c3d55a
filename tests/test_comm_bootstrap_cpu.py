"""CPU tests of the communicator's host side: the UNIX-socket all-gather used for the IPC-handle exchange (2 and 3
processes, no GPU), its bounded waits when a peer never shows up, and the fixed-order reduction the device code
implements, cross-checked through a gloo process group of world size 2."""
import ctypes
import multiprocessing as mp
import os
import time

import pytest
import torch

from muillm_b200 import capi


def _allgather_worker(rank, world, key, q, delay=0.0, timeout=20.0):
    lib = capi.lib()
    time.sleep(delay)
    blob = bytes([rank + 1]) * 64
    out = ctypes.create_string_buffer(world * 64)
    s = lib.mui_bootstrap_allgather(rank, world, key.encode(), blob, 64, out, timeout)
    q.put((rank, s, out.raw, lib.mui_last_error().decode()))


@pytest.mark.parametrize("world", [2, 3])
def test_bootstrap_allgather_between_processes(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    key = f"t{os.getpid()}_{world}"
    procs = [ctx.Process(target=_allgather_worker, args=(r, world, key, q, 0.2 * (world - r))) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=60) for _ in range(world)]
    for p in procs:
        p.join(timeout=30)
    want = b"".join(bytes([r + 1]) * 64 for r in range(world))
    for rank, status, table, err in results:
        assert status == capi.MUI_OK, err
        assert table == want


def test_bootstrap_times_out_when_a_peer_never_arrives():
    lib = capi.lib()
    out = ctypes.create_string_buffer(2 * 64)
    t0 = time.time()
    s = lib.mui_bootstrap_allgather(0, 2, f"lonely{os.getpid()}".encode(), b"x" * 64, 64, out, 1.0)
    assert s == capi.MUI_ERR_COMM and time.time() - t0 < 10
    assert b"peers connected" in lib.mui_last_error()
    t0 = time.time()
    s = lib.mui_bootstrap_allgather(1, 2, f"noserver{os.getpid()}".encode(), b"x" * 64, 64, out, 1.0)
    assert s == capi.MUI_ERR_COMM and time.time() - t0 < 10
    assert b"could not reach rank 0" in lib.mui_last_error()


def test_comm_argument_validation_without_gpu():
    lib = capi.lib()
    h = ctypes.c_void_p()
    assert lib.mui_comm_create(3, 2, 1024, ctypes.byref(h)) == capi.MUI_ERR_INVALID_ARG
    assert lib.mui_comm_create(0, 9, 1024, ctypes.byref(h)) == capi.MUI_ERR_INVALID_ARG
    assert lib.mui_comm_all_reduce_sum(None, None, 0, None, None, 4, 0) == capi.MUI_ERR_INVALID_ARG
    assert lib.mui_comm_ipc_handle_bytes() == 64


def _gloo_worker(rank, world, port, q):
    import torch.distributed as dist

    from oracle import decode_oracle as oracle

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = torch.Generator().manual_seed(100 + rank)
    # K-sharded linear: every rank holds a column slice of W and of x; rank 0 adds the residual
    N, K = 48, 64
    gw = torch.Generator().manual_seed(7)
    W = (torch.randn(N, K, generator=gw) * 0.05).half()
    x = torch.randn(1, K, generator=gw).half()
    res = torch.randn(1, N, generator=gw).half()
    ks = K // world
    part = torch.nn.functional.linear(x[:, rank * ks:(rank + 1) * ks].float(), W[:, rank * ks:(rank + 1) * ks].float())
    if rank == 0:
        part = part + res.float()
    gathered = [torch.zeros_like(part) for _ in range(world)]
    dist.all_gather(gathered, part)
    y = oracle.all_reduce_fixed_order(gathered, torch.float16)
    full = oracle.linear(x, W, residual=res)
    q.put((rank, y, full))
    dist.destroy_process_group()


def test_sharded_linear_fixed_order_reduce_gloo_world2():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_gloo_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(2)]
    for p in procs:
        p.join(timeout=30)
    ys = {r: y for r, y, _ in res}
    assert torch.equal(ys[0], ys[1])  # bit-identical on all ranks
    torch.testing.assert_close(ys[0].float(), res[0][2].float(), rtol=1e-2, atol=1e-3)


def _gloo_decoder_worker(rank, world, port, q):
    import torch.distributed as dist

    from muillm_b200.decoder_stack import shard_llama_weights
    from oracle import decode_oracle as oracle

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = dict(layers=2, hidden=64, intermediate=96, heads=4, kv_heads=2, head_dim=16, vocab=40, eps=1e-5,
               rope_theta=10000.0)
    w = oracle.make_llama_weights(cfg, torch.float16, seed=2, std=0.1)
    wl, cl = shard_llama_weights(w, cfg, rank, world)

    def all_reduce(part):
        parts = [torch.zeros_like(part) for _ in range(world)]
        dist.all_gather(parts, part.contiguous())
        total = parts[0].clone()
        for p in parts[1:]:
            total += p  # rank order, fp32
        return total

    sharded = oracle.LlamaOracle(wl, cl, max_T=16, all_reduce=all_reduce)
    toks = torch.randint(0, cfg["vocab"], (1, 6), generator=torch.Generator().manual_seed(3))
    local_logits = sharded.forward(toks)  # this rank's vocabulary shard
    shards = [torch.zeros_like(local_logits) for _ in range(world)]
    dist.all_gather(shards, local_logits)
    q.put((rank, torch.cat(shards, dim=-1), cl))
    dist.destroy_process_group()


def test_sharded_decoder_matches_unsharded_oracle_gloo_world2():
    """shard_llama_weights + the rank-ordered fp32 sum reproduce the un-sharded decoder: the host-side sharding of
    the tensor-parallel decode stack, checked on CPU with two gloo ranks."""
    from oracle import decode_oracle as oracle

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 31500 + os.getpid() % 2000
    procs = [ctx.Process(target=_gloo_decoder_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in range(2)]
    for p in procs:
        p.join(timeout=30)
    cfg = dict(layers=2, hidden=64, intermediate=96, heads=4, kv_heads=2, head_dim=16, vocab=40, eps=1e-5,
               rope_theta=10000.0)
    w = oracle.make_llama_weights(cfg, torch.float16, seed=2, std=0.1)
    toks = torch.randint(0, cfg["vocab"], (1, 6), generator=torch.Generator().manual_seed(3))
    want = oracle.LlamaOracle(w, cfg, max_T=16).forward(toks)
    by_rank = {r: (lg, cl) for r, lg, cl in res}
    assert torch.equal(by_rank[0][0], by_rank[1][0])
    assert by_rank[1][1]["vocab_offset"] == 20 and by_rank[1][1]["heads"] == 2 and by_rank[1][1]["kv_heads"] == 1
    torch.testing.assert_close(by_rank[0][0], want, rtol=2e-2, atol=2e-2)
