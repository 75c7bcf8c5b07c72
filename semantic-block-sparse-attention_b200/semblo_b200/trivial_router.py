"""The query routing vector (mirror of semblo/vllm_plugin/trivial_router.py:48-75)."""
from __future__ import annotations

import torch

from ._lib import check, lib, ptr, require_cuda, stream_ptr
from .flat_index import routing_mode


def trivial_router_vectors(x: torch.Tensor, factors: int = 1, out: torch.Tensor | None = None) -> torch.Tensor:
    """[Q, Hq, D] bf16 -> [Q, Hq, D] bf16: normalise in fp32, round, normalise, round.

    Only ``factors == 1`` (whole-vector routing, the default) is implemented."""
    require_cuda(x)
    routing_mode()
    if factors != 1:
        raise RuntimeError("only whole-vector routing (factors == 1) is implemented")
    if x.dtype != torch.bfloat16:
        raise ValueError("routing queries must be bf16")
    q, h, d = x.shape
    flat = x.reshape(q * h, d)
    if flat.stride(1) != 1:
        flat = flat.contiguous()
    if out is None:
        out = torch.empty(q, h, d, dtype=x.dtype, device=x.device)
    elif out.shape != x.shape or out.dtype != x.dtype or not out.is_contiguous():
        raise ValueError("out must be a contiguous bf16 tensor of the input's shape")
    check(lib().semblo_routing_normalize(ptr(flat), 0, q * h, d, flat.stride(0), None, None, ptr(out), 1,
                                         stream_ptr()))
    return out
