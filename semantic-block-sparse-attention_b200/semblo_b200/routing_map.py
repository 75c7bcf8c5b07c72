"""The routing map: pre-RoPE keys and queries into the space the blocks are built in.

Mirror of semblo/vllm_plugin/routing_map.py (``SembloQueryState`` 21-30, ``routing_normalize``
35-64, ``SembloKeyRouter`` 67-94).  The method routes on the pre-RoPE keys themselves, so the map
is the identity by default; a linear map W [Hkv, I, D] per layer and KV head can be loaded instead
(the reference's routing-key comparisons: non-rotary dimensions, PCA, random projections).  Keys and
queries go through the same map and the result is normalised over the whole vector.  The projection
is a plain batched GEMM (torch).  The kernels behind it route in a space of the head dimension, so a
map into fewer dimensions (I < D) is followed by zero padding up to D: zeros change neither a norm
nor a dot product nor a mean, so the clusters, the scores and the selection are those of the
I-dimensional space.  A map into more dimensions than the head has is refused."""
from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import nn
from torch.nn import functional as F

from .flat_index import routing_normalize


@dataclass
class SembloQueryState:
    """What the selection kernels read for a chunk of queries."""
    vectors: torch.Tensor                         # [B, Q, Hq, R, I]
    mixture_weights: torch.Tensor | None = None   # [B, Q, Hq, R], uniform


class SembloKeyRouter(nn.Module):
    """The routing map of one layer: ``weight`` [Hkv, I, D], the identity by default."""

    def __init__(self, num_kv_heads: int, head_dim: int, index_dim: int, num_factors: int = 1) -> None:
        super().__init__()
        if index_dim <= 0 or index_dim % max(int(num_factors), 1) != 0:
            raise ValueError("index_dim must be positive and divisible by num_factors")
        if index_dim > head_dim:
            raise ValueError("the kernels route in a space of the head dimension: index_dim must not exceed head_dim")
        self.num_kv_heads, self.head_dim, self.index_dim = int(num_kv_heads), int(head_dim), int(index_dim)
        self.num_factors = int(num_factors)
        self.weight = nn.Parameter(torch.zeros(num_kv_heads, index_dim, head_dim), requires_grad=False)
        if index_dim == head_dim:
            with torch.no_grad():
                self.weight.copy_(torch.eye(head_dim).expand(num_kv_heads, head_dim, head_dim))
        self._identity_key = None

    def is_identity(self) -> bool:
        """Decided once per loaded weight (one comparison on the device, one host read): never per call,
        a recorded decode step must not synchronise."""
        key = (self.weight.data_ptr(), self.weight._version)
        if self._identity_key is None or self._identity_key[0] != key:
            w = self.weight
            same = bool(w.shape[1] == w.shape[2] and torch.equal(
                w, torch.eye(w.shape[1], dtype=w.dtype, device=w.device).expand_as(w)))
            self._identity_key = (key, same)
        return self._identity_key[1]

    def load_weight(self, weight: torch.Tensor) -> None:
        """Replace the map ([Hkv, I, D]); the identity decision is taken again at the next use.  (A weight
        written behind the parameter's back, through ``.data``, is not noticed: load it here or through
        ``load_state_dict``.)"""
        with torch.no_grad():
            self.weight.copy_(weight)
        self._identity_key = None

    def project(self, keys: torch.Tensor) -> torch.Tensor:
        """[..., Hkv, D] -> [..., Hkv, I], without normalisation."""
        return torch.einsum("...hd,hid->...hi", keys, self.weight.to(dtype=keys.dtype))

    def project_queries(self, q_pre: torch.Tensor) -> torch.Tensor:
        """[Q, Hq, D] -> [Q, Hq, I]: a query goes through the map of its KV head."""
        hq = int(q_pre.shape[1])
        q_to_kv = torch.div(torch.arange(hq, device=self.weight.device) * self.num_kv_heads, hq, rounding_mode="floor")
        per_q = self.weight.to(dtype=q_pre.dtype).index_select(0, q_to_kv)
        return torch.einsum("qhd,hid->qhi", q_pre, per_q)

    def widen(self, projected: torch.Tensor) -> torch.Tensor:
        """[..., I] -> [..., D]: the projection in the width the kernels route in (zeros after dimension I)."""
        if self.index_dim == self.head_dim:
            return projected
        return F.pad(projected, (0, self.head_dim - self.index_dim))

    def forward(self, keys: torch.Tensor) -> torch.Tensor:
        if keys.ndim != 4:
            raise ValueError("keys must have shape [B,L,Hkv,D]")
        if keys.shape[2:] != (self.num_kv_heads, self.head_dim):
            raise ValueError("key tensor does not match router dimensions")
        if self.is_identity():
            return routing_normalize(keys[0])[None] if keys.shape[0] == 1 else torch.stack(
                [routing_normalize(k) for k in keys])
        projected = self.widen(self.project(keys))
        return torch.stack([routing_normalize(p.contiguous()) for p in projected])


# ---------------------------------------------------------------------------------- map makers
# The maps of the reference's routing-key comparisons (scripts/make_routing_map.py:44-120 there), as
# [Hkv, I, D] fp32 tensors ready for ``SembloKeyRouter.load_weight`` or ``runtime_weights.write_runtime_weights``.

def non_rotary_map(num_kv_heads: int, head_dim: int, rotary_dims: int) -> torch.Tensor:
    """The identity with the first ``rotary_dims`` (rotated) dimensions zeroed: routing on the
    dimensions that RoPE leaves alone.  Square."""
    if not 0 <= rotary_dims <= head_dim:
        raise ValueError("rotary_dims must lie in [0, head_dim]")
    eye = torch.eye(head_dim, dtype=torch.float32)
    eye[:rotary_dims] = 0
    return eye.expand(num_kv_heads, head_dim, head_dim).contiguous()


def random_map(num_kv_heads: int, head_dim: int, index_dim: int, generator: torch.Generator) -> torch.Tensor:
    """Per KV head a random map with orthonormal rows (index_dim <= head_dim): the Q factor of a
    float64 Gaussian matrix, transposed."""
    if not 0 < index_dim <= head_dim:
        raise ValueError("index_dim must lie in (0, head_dim]")
    maps = []
    for _ in range(num_kv_heads):
        q, _r = torch.linalg.qr(torch.randn(head_dim, index_dim, generator=generator, dtype=torch.float64))
        maps.append(q.T.contiguous().to(torch.float32))
    return torch.stack(maps)


def pca_map(keys: torch.Tensor, index_dim: int, rank: int | None = None) -> torch.Tensor:
    """Per KV head the top ``rank`` eigenvectors of the uncentred Gram matrix of pre-RoPE keys
    [L, Hkv, D] (float64 eigendecomposition, largest eigenvalue first) as rows of [Hkv, index_dim, D];
    rows past ``rank`` are zero."""
    length, heads, dim = keys.shape
    rank = index_dim if rank is None else int(rank)
    if not 0 < rank <= index_dim <= dim:
        raise ValueError("need 0 < rank <= index_dim <= head_dim")
    x = keys.detach().to(torch.float32).permute(1, 0, 2).contiguous()          # [Hkv, L, D]
    gram = torch.matmul(x.transpose(1, 2), x).to(torch.float64).cpu()          # [Hkv, D, D]
    out = torch.zeros(heads, index_dim, dim, dtype=torch.float64)
    for h in range(heads):
        _vals, vecs = torch.linalg.eigh(gram[h])                               # ascending eigenvalues
        out[h, :rank] = vecs[:, -rank:].flip(1).T
    return out.to(torch.float32)
