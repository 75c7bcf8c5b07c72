"""The N > 1 path on CPU: two gloo ranks, each computing its own KV heads with the oracle, and
the one collective of the path (the gather of per-head outputs) through the package's module."""
from __future__ import annotations

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import semblo_oracle as O


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank: int, world: int, port: int, results) -> None:
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from semblo_b200.head_parallel import HeadGather, kv_head_shard, q_head_shard
        hq, hkv, dim, length = 8, 4, 64, 96
        data = O.mixture_inputs(length=length, num_q_heads=hq, num_kv_heads=hkv, head_dim=dim, centres=4, seed=5)
        kv, qh = kv_head_shard(hkv, rank, world), q_head_shard(hq, hkv, rank, world)
        qpos = torch.arange(length)
        local, _ = O.dense_causal_attention(data["q_post"][:, qh.start:qh.stop], data["k_post"][:, kv.start:kv.stop],
                                            data["v"][:, kv.start:kv.stop], qpos, dim ** -0.5)
        gather = HeadGather()
        full = gather(local.float())
        again = torch.empty_like(full)
        gather(local.float(), again)                      # second call reuses the staging buffer
        want, _ = O.dense_causal_attention(data["q_post"], data["k_post"], data["v"], qpos, dim ** -0.5)
        results[rank] = (float((full - want.float()).abs().max()), bool(torch.equal(full, again)), tuple(full.shape))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_two_ranks_gather_head_outputs():
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(100)
        assert p.exitcode == 0
    for r in range(world):
        err, same, shape = results[r]
        assert shape == (96, 8, 64)
        assert same
        assert err < 1e-5


def test_shards_are_consecutive_and_checked():
    from semblo_b200.head_parallel import kv_head_shard, q_head_shard
    assert list(kv_head_shard(8, 3, 4)) == [6, 7]
    assert list(q_head_shard(32, 8, 1, 8)) == [4, 5, 6, 7]
    with pytest.raises(ValueError):
        kv_head_shard(6, 0, 4)
    with pytest.raises(ValueError):
        kv_head_shard(8, 4, 4)
