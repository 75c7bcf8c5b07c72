"""Head-parallel sharding of the sparse-attention path over the GPUs of one node.

The path partitions by KV head: every KV head (with its group of query heads) owns its own
index, selection and attention, so the ranks exchange nothing while they compute.  The only
collective is the gather of the per-head outputs, as in tensor-parallel vLLM
(the reference runs under vLLM's tensor parallelism: semblo/vllm_plugin/model.py:1169-1269
is executed per rank on that rank's heads).  Everything here works on CPU tensors with the
gloo backend as well, which is how the multi-rank logic is tested without GPUs."""
from __future__ import annotations

import torch
import torch.distributed as dist


def kv_head_shard(num_kv_heads: int, rank: int, world: int) -> range:
    """The KV heads rank ``rank`` of ``world`` owns: consecutive, equal shares."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside a world of {world}")
    if num_kv_heads % world != 0:
        raise ValueError(f"{num_kv_heads} KV heads do not split evenly over {world} ranks")
    per = num_kv_heads // world
    return range(rank * per, (rank + 1) * per)


def q_head_shard(num_q_heads: int, num_kv_heads: int, rank: int, world: int) -> range:
    """The query heads that go with kv_head_shard (query heads of a KV head are adjacent)."""
    kv = kv_head_shard(num_kv_heads, rank, world)
    group = num_q_heads // num_kv_heads
    if group * num_kv_heads != num_q_heads:
        raise ValueError("query heads must be a multiple of the KV heads")
    return range(kv.start * group, kv.stop * group)


class HeadGather:
    """Gathers per-rank outputs [T, Hq / world, D] into [T, Hq, D] with one all-gather.

    The receive buffer is kept between calls (fixed address: the call can sit inside a captured
    graph when the backend supports it)."""

    def __init__(self, group=None) -> None:
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self._stage = None

    def __call__(self, local: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        if self.world == 1:
            if out is None:
                return local
            out.copy_(local)
            return out
        t, hl, d = local.shape
        if self._stage is None or self._stage.shape != (self.world * t, hl, d) or self._stage.dtype != local.dtype \
                or self._stage.device != local.device:
            self._stage = torch.empty(self.world * t, hl, d, dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(self._stage, local.contiguous(), group=self.group)   # rank-major rows
        full = self._stage.view(self.world, t, hl, d).permute(1, 0, 2, 3).reshape(t, self.world * hl, d)
        if out is None:
            return full.contiguous()
        out.copy_(full)
        return out
