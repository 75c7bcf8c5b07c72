"""The routing maps of a prepared model directory: the side-car file and its manifest.

Mirror of semblo/vllm_plugin/runtime_weights.py of the reference (names, file format and error
behaviour; 26-357 there).  The base model's weights are loaded from the directory as usual; the
routing map of every sparse layer (``semblo_key_router.weight`` [Hkv, I, D], routing_map.py) comes
from ``semblo_runtime.safetensors``, and ``semblo_runtime.json`` records the file's hash and every
tensor's shape, dtype and content hash.  A file is verified before a single tensor is copied; a
tensor whose leading (head) dimension is ``tp_size`` times the parameter's is cut to the rank's
contiguous block of heads, which is how the KV-head shards of a multi-GPU run get their maps.
``write_runtime_weights`` produces such a directory (the reference writes it from its checkpoint
preparation scripts: scripts/prepare_nemotron_checkpoint.py:81-100).
"""
from __future__ import annotations

import hashlib
import json
import logging
import re
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Iterable, Iterator, Mapping, Sequence

import torch
from torch import nn

LOGGER = logging.getLogger(__name__)

RUNTIME_WEIGHTS_FILE = "semblo_runtime.safetensors"
RUNTIME_MANIFEST_FILE = "semblo_runtime.json"
RUNTIME_SCHEMA_VERSION = 1

# the attention block is ``self_attn`` in Qwen3.5 and ``mixer`` in Nemotron-H; file names say ``self_attn``
_BLOCKS = ("self_attn", "mixer")
_LAYER_AT_END = re.compile(r"(?:^|\.)layers\.(\d+)$")
_LAYER_ROUTER = re.compile(r"^layers\.\d+\.self_attn\.semblo_")
_QUERY_ROUTER = ".self_attn.semblo_query_router."


def _safetensors():
    try:
        from safetensors import torch as st
    except ImportError as exc:                       # pragma: no cover - the image ships it
        raise RuntimeError("the routing-map side-car needs the safetensors package") from exc
    return st


def sha256_file(path: str | Path) -> str:
    h = hashlib.sha256()
    with Path(path).open("rb") as f:
        while True:
            block = f.read(1 << 20)
            if not block:
                return h.hexdigest()
            h.update(block)


def _tensor_sha256(tensor: torch.Tensor) -> str:
    raw = tensor.detach().contiguous().cpu().view(torch.uint8).numpy().tobytes()
    return hashlib.sha256(raw).hexdigest()


def canonical_runtime_name(name: str) -> str | None:
    """``<prefix>.layers.<i>.<self_attn|mixer>.semblo_<rest>`` -> ``layers.<i>.self_attn.semblo_<rest>``;
    None for any other parameter.  The prefix differs between model implementations
    (``model.``, ``model.language_model.``), the file does not."""
    for block in _BLOCKS:
        at = name.find(f".{block}.semblo_")
        if at < 0:
            continue
        layer = _LAYER_AT_END.search(name[:at])
        if layer is None:
            return None
        return f"layers.{int(layer.group(1))}.self_attn.{name[at + len(block) + 2:]}"
    return None


def is_runtime_parameter(name: str) -> bool:
    return canonical_runtime_name(name) is not None


def semblo_config_fields(config: Mapping[str, object]) -> dict[str, object]:
    """The ``semblo_*`` keys of a checkpoint config (of its ``text_config`` when it has one)."""
    text = config.get("text_config", config)
    if not isinstance(text, Mapping):
        raise ValueError("checkpoint text_config must be a JSON object")
    return {str(k): v for k, v in text.items() if str(k).startswith("semblo_")}


@dataclass(frozen=True)
class RuntimeWeightsManifest:
    schema_version: int
    source_checkpoint: str
    source_config_sha256: str
    weights_file: str
    weights_sha256: str
    tensor_names: tuple[str, ...]
    tensor_shapes: dict[str, list[int]]
    tensor_dtypes: dict[str, str]
    tensor_sha256: dict[str, str]
    semblo_config: dict[str, object]

    def to_dict(self) -> dict[str, object]:
        d = asdict(self)
        d["tensor_names"] = list(self.tensor_names)
        return d

    @classmethod
    def from_dict(cls, raw: Mapping[str, object]) -> "RuntimeWeightsManifest":
        version = raw.get("schema_version", -1)
        if int(version) != RUNTIME_SCHEMA_VERSION:
            raise ValueError(f"semblo runtime weights schema {version!r} is not supported "
                             f"(this loader reads version {RUNTIME_SCHEMA_VERSION})")
        per_tensor = {key: {str(n): ([int(x) for x in v] if key == "tensor_shapes" else str(v))
                            for n, v in dict(raw[key]).items()}
                      for key in ("tensor_shapes", "tensor_dtypes", "tensor_sha256")}
        plain = {key: str(raw[key]) for key in ("source_checkpoint", "source_config_sha256", "weights_file",
                                                "weights_sha256")}
        return cls(schema_version=RUNTIME_SCHEMA_VERSION, tensor_names=tuple(map(str, raw["tensor_names"])),
                   semblo_config=dict(raw["semblo_config"]), **plain, **per_tensor)


def read_runtime_manifest(directory: str | Path) -> RuntimeWeightsManifest:
    path = Path(directory).expanduser().resolve() / RUNTIME_MANIFEST_FILE
    if not path.is_file():
        raise FileNotFoundError(f"no routing-map manifest at {path}")
    return RuntimeWeightsManifest.from_dict(json.loads(path.read_text(encoding="utf-8")))


def verify_runtime_weights(directory: str | Path) -> RuntimeWeightsManifest:
    """File hash, tensor names, shapes, dtypes and content hashes against the manifest; raises on the
    first difference."""
    root = Path(directory).expanduser().resolve()
    manifest = read_runtime_manifest(root)
    path = root / manifest.weights_file
    if not path.is_file():
        raise FileNotFoundError(f"the manifest names {path}, which does not exist")
    digest = sha256_file(path)
    if digest != manifest.weights_sha256:
        raise ValueError(f"{path.name}: sha256 {digest} differs from the manifest's {manifest.weights_sha256}")
    tensors = _safetensors().load_file(str(path), device="cpu")
    if sorted(tensors) != sorted(manifest.tensor_names):
        raise ValueError(f"{path.name}: the tensor names differ from the manifest's")
    for name in manifest.tensor_names:
        t = tensors[name]
        found = {"shape": list(t.shape), "dtype": str(t.dtype), "content hash": _tensor_sha256(t)}
        want = {"shape": manifest.tensor_shapes[name], "dtype": manifest.tensor_dtypes[name],
                "content hash": manifest.tensor_sha256[name]}
        for what in found:
            if found[what] != want[what]:
                raise ValueError(f"{name}: {what} {found[what]} differs from the manifest's {want[what]}")
    return manifest


def write_runtime_weights(directory: str | Path, tensors: Mapping[str, torch.Tensor], config: Mapping[str, object],
                          source: str) -> RuntimeWeightsManifest:
    """Write ``tensors`` (canonical names) and their manifest into ``directory``; ``config`` is the
    checkpoint's config.json content (its hash and its ``semblo_*`` keys go into the manifest)."""
    root = Path(directory).expanduser().resolve()
    root.mkdir(parents=True, exist_ok=True)
    names = tuple(sorted(tensors))
    for n in names:
        if not _LAYER_ROUTER.match(n):
            raise ValueError(f"{n!r} is not a canonical routing-map name (layers.<i>.self_attn.semblo_...)")
    ordered = {n: tensors[n].detach().contiguous().cpu() for n in names}
    path = root / RUNTIME_WEIGHTS_FILE
    _safetensors().save_file(ordered, str(path))
    manifest = RuntimeWeightsManifest(
        schema_version=RUNTIME_SCHEMA_VERSION,
        source_checkpoint=str(source),
        source_config_sha256=hashlib.sha256(json.dumps(dict(config), sort_keys=True).encode()).hexdigest(),
        weights_file=RUNTIME_WEIGHTS_FILE,
        weights_sha256=sha256_file(path),
        tensor_names=names,
        tensor_shapes={n: list(ordered[n].shape) for n in names},
        tensor_dtypes={n: str(ordered[n].dtype) for n in names},
        tensor_sha256={n: _tensor_sha256(ordered[n]) for n in names},
        semblo_config=semblo_config_fields(config),
    )
    (root / RUNTIME_MANIFEST_FILE).write_text(
        json.dumps(manifest.to_dict(), ensure_ascii=False, indent=2, sort_keys=True) + "\n", encoding="utf-8")
    return manifest


def _targets(module: nn.Module) -> dict[str, tuple[str, nn.Parameter]]:
    found: dict[str, tuple[str, nn.Parameter]] = {}
    for actual, parameter in module.named_parameters():
        canonical = canonical_runtime_name(actual)
        if canonical is None:
            continue
        if canonical in found:
            raise ValueError(f"{actual} and {found[canonical][0]} both stand for {canonical!r}")
        found[canonical] = (actual, parameter)
    return found


def _without_query_router(tensors: Mapping[str, torch.Tensor], names: Sequence[str]):
    """Files of an earlier format also hold a query router.  Queries go through the key-side map, to which
    a query router with zero residual and zero mixture adds nothing: such tensors are dropped, any other
    query router raises."""
    kept = {}
    for name, t in tensors.items():
        if _QUERY_ROUTER not in name:
            kept[name] = t
        elif name.rsplit(".", 1)[-1] in ("down", "up", "mixture_weight", "mixture_bias") and bool(t.any()):
            raise ValueError(f"{name} holds non-zero values: a trained query router is not supported "
                             "(queries go through the key-side map)")
    return kept, [n for n in names if n in kept]


def load_runtime_tensors_into_module(module: nn.Module, tensors: Mapping[str, torch.Tensor],
                                     tensor_names: Sequence[str], *, require_exact_match: bool = True,
                                     allow_unused_layer_parameters: bool = False, tp_rank: int = 0,
                                     tp_size: int = 1) -> set[str]:
    """Copy full-size tensors, keyed by canonical name and taken in ``tensor_names`` order, into the
    ``semblo_*`` parameters of ``module``; returns the model's names of the parameters written.

    ``allow_unused_layer_parameters`` skips whole router groups of layers the model has no router for
    (layers outside the sparse set are dense); any other name without a parameter raises, and so does a
    parameter without a tensor unless ``require_exact_match`` is off.  Every routing parameter carries
    its heads in dimension 0 and a rank owns one contiguous block of heads, so a tensor whose leading
    dimension is ``tp_size`` times the parameter's is cut to rows
    ``[tp_rank * local, (tp_rank + 1) * local)``; equal shapes are copied whole."""
    if sorted(tensor_names) != sorted(tensors):
        raise ValueError("tensor_names must name exactly the tensors given")
    tensors, tensor_names = _without_query_router(tensors, tensor_names)
    targets = _targets(module)
    in_file, in_model = set(tensors), set(targets)
    no_parameter = in_file - in_model
    skipped: set[str] = set()
    if no_parameter and allow_unused_layer_parameters:
        skipped = {n for n in no_parameter if _LAYER_ROUTER.match(n)}
        no_parameter -= skipped
        if skipped:
            LOGGER.warning("%d routing tensors belong to layers without a router here (dense layers) and are "
                           "left out: %s", len(skipped), ", ".join(sorted(skipped)[:8]))
    if no_parameter:
        raise ValueError("the file holds tensors the model has no parameter for: "
                         + ", ".join(sorted(no_parameter)[:8]))
    no_tensor = in_model - in_file
    if require_exact_match and no_tensor:
        raise ValueError("the model has routing parameters the file does not hold: "
                         + ", ".join(sorted(no_tensor)[:8]))
    written: set[str] = set()
    with torch.no_grad():
        for canonical in tensor_names:
            if canonical in skipped:
                continue
            actual, parameter = targets[canonical]
            t = tensors[canonical]
            if tuple(t.shape) != tuple(parameter.shape):
                local = int(parameter.shape[0]) if parameter.ndim > 0 else 0
                sharded = (tp_size > 1 and t.ndim == parameter.ndim and local > 0
                           and int(t.shape[0]) == local * tp_size
                           and tuple(t.shape[1:]) == tuple(parameter.shape[1:]))
                if not sharded:
                    raise ValueError(f"{canonical}: the file has {tuple(t.shape)}, the parameter "
                                     f"{tuple(parameter.shape)} (tp_size={tp_size})")
                t = t[tp_rank * local:(tp_rank + 1) * local]
            parameter.copy_(t.to(device=parameter.device, dtype=parameter.dtype))
            written.add(actual)
    return written


def load_runtime_weights_into_module(module: nn.Module, directory: str | Path, *, require_exact_match: bool = True,
                                     allow_unused_layer_parameters: bool = False, tp_rank: int = 0,
                                     tp_size: int = 1) -> set[str]:
    """Verify the side-car of ``directory`` (a missing or altered file raises), then load it in the
    manifest's order; keyword arguments as in ``load_runtime_tensors_into_module``."""
    root = Path(directory).expanduser().resolve()
    manifest = verify_runtime_weights(root)
    tensors = _safetensors().load_file(str(root / manifest.weights_file), device="cpu")
    return load_runtime_tensors_into_module(
        module, tensors, manifest.tensor_names, require_exact_match=require_exact_match,
        allow_unused_layer_parameters=allow_unused_layer_parameters, tp_rank=tp_rank, tp_size=tp_size)


def filter_base_weight_iterator(weights: Iterable[tuple[str, torch.Tensor]]) -> Iterator[tuple[str, torch.Tensor]]:
    """The base checkpoint's (name, tensor) stream without routing parameters: those are loaded from the
    side-car only, whether or not the checkpoint also holds them."""
    for name, tensor in weights:
        if not is_runtime_parameter(name):
            yield name, tensor
