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
    """The all-gather of per-rank outputs [T, Hq / world, D].

    The gathered tensor is kept rank-major, ``[world, T, Hq / world, D]`` (what one NCCL
    all-gather writes): head ``r * Hq / world + j`` of token ``t`` is ``full[r, t, j]``, and
    :meth:`as_heads` gives the ``[T, Hq, D]`` view of it without moving a byte.  A consumer that
    wants the heads of a token contiguous (an output projection reading ``[T, Hq * D]``) copies
    once, or better reads the view.

    ``issue`` runs the collective on a communication stream behind an event recorded on the
    caller's stream, so the next chunk computes while this one travels; ``wait`` makes the
    caller's stream wait for everything issued.  On CPU tensors (gloo) both are synchronous."""

    def __init__(self, group=None) -> None:
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self._stage = None
        self._comm = None
        self._pending = False

    @staticmethod
    def as_heads(full: torch.Tensor) -> torch.Tensor:
        """[world, T, Hl, D] -> the [T, world * Hl, D] view (strided, no copy)."""
        w, t, hl, d = full.shape
        return full.permute(1, 0, 2, 3).reshape(t, w * hl, d) if w == 1 else full.permute(1, 0, 2, 3).flatten(1, 2)

    def issue(self, local: torch.Tensor, full: torch.Tensor) -> None:
        """Gather ``local`` [T, Hl, D] (contiguous) from every rank into ``full`` [world, T, Hl, D].
        ``local`` and ``full`` must stay untouched until :meth:`wait`."""
        if tuple(full.shape) != (self.world,) + tuple(local.shape) or not full.is_contiguous() \
                or not local.is_contiguous():
            raise ValueError("full must be a contiguous [world, T, Hl, D] and local a contiguous [T, Hl, D]")
        if self.world == 1:
            full[0].copy_(local)
            return
        if not local.is_cuda:
            dist.all_gather_into_tensor(full.flatten(0, 1), local, group=self.group)
            return
        if self._comm is None:
            self._comm = torch.cuda.Stream(device=local.device)
        ready = torch.cuda.Event()
        ready.record()
        self._comm.wait_event(ready)
        with torch.cuda.stream(self._comm):
            dist.all_gather_into_tensor(full.flatten(0, 1), local, group=self.group)
        self._pending = True

    def wait(self) -> None:
        if self._pending:
            torch.cuda.current_stream().wait_stream(self._comm)
            self._pending = False

    def __call__(self, local: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """Synchronous form: returns (or fills) the [T, Hq, D] tensor."""
        if self.world == 1:
            if out is None:
                return local
            out.copy_(local)
            return out
        t, hl, d = local.shape
        if self._stage is None or self._stage.shape != (self.world, t, hl, d) or self._stage.dtype != local.dtype \
                or self._stage.device != local.device:
            self._stage = torch.empty(self.world, t, hl, d, dtype=local.dtype, device=local.device)
        self.issue(local.contiguous(), self._stage)
        self.wait()
        full = self.as_heads(self._stage)
        if out is None:
            return full.contiguous()
        out.copy_(full)
        return out
