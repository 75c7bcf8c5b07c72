"""The sparse attention core as the ``semblo::attention`` operator.

Same schema, same in-place contract and the same layer table as
semblo/vllm_plugin/attention_op.py:45-112: the traced side of a layer projects Q/K/V and
calls the operator with a caller-allocated ``output``; the operator looks the layer up by
vLLM's per-layer name and runs its ``attention_forward``.  This module takes the place of the
reference's module of the same name (one of the two registers the schema in a process)."""
from __future__ import annotations

from typing import Any

import torch

_OP_NAMESPACE = "semblo"
_OP_NAME = "attention"
SPLITTING_OP_NAME = f"{_OP_NAMESPACE}::{_OP_NAME}"

_LAYERS: dict[str, Any] = {}


def register_layer(layer_name: str, layer: Any) -> None:
    """Make ``layer`` reachable from the operator under ``layer_name``."""
    _LAYERS[str(layer_name)] = layer


def registered_layer(layer_name: str) -> Any:
    layer = _LAYERS.get(str(layer_name))
    if layer is None:
        raise RuntimeError(f"no semblo layer is registered as {layer_name!r}; the operator is reachable "
                           "only through a layer that registered itself")
    return layer


def _attention(positions, hidden_states, q_post, k_post, v_states, q_pre, k_pre, output, layer_name: str) -> None:
    registered_layer(layer_name).attention_forward(positions, hidden_states, q_post, k_post, v_states, q_pre,
                                                   k_pre, output)


def _attention_fake(positions, hidden_states, q_post, k_post, v_states, q_pre, k_pre, output, layer_name: str) -> None:
    return None


_LIBRARY: torch.library.Library | None = None


def _register() -> None:
    global _LIBRARY
    library = torch.library.Library(_OP_NAMESPACE, "FRAGMENT")
    library.define(f"{_OP_NAME}(Tensor positions, Tensor hidden_states, Tensor q_post, Tensor? k_post, "
                   "Tensor? v_states, Tensor q_pre, Tensor? k_pre, Tensor(a!) output, str layer_name) -> ()")
    # the operator exists on the device only: there is no CPU path behind it
    library.impl(_OP_NAME, _attention, "CUDA")
    library._register_fake(_OP_NAME, _attention_fake)
    _LIBRARY = library


_register()
sparse_attention_op = getattr(torch.ops, _OP_NAMESPACE).attention
