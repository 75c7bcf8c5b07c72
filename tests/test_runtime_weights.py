"""The routing-map side-car (semblo_b200/runtime_weights.py) against a directory written and verified by
the reference's own code (tests/golden/runtime_weights/, made by tests/golden/make_runtime_weights_golden.py),
and the cases the reference tests: canonical names (test_nemotron_h_port.py:14-20), verification of a
prepared directory (test_prepare_qwen3_5_checkpoint.py:67-68)."""
import json
import pathlib
import shutil

import pytest
import torch
from torch import nn

from semblo_b200 import runtime_weights as RW
from semblo_b200.routing_map import SembloKeyRouter

GOLDEN = pathlib.Path(__file__).resolve().parent / "golden" / "runtime_weights"


def _golden_tensors():
    g = torch.Generator().manual_seed(20240607)
    return {
        "layers.3.self_attn.semblo_key_router.weight": torch.randn(4, 8, 8, generator=g).to(torch.bfloat16),
        "layers.7.self_attn.semblo_key_router.weight": torch.randn(4, 6, 8, generator=g),
    }


_CONFIG = {"architectures": ["SembloNemotronHForCausalLM"], "head_dim": 8, "num_key_value_heads": 4,
           "semblo_index_dim": 8, "semblo_layer_indices": [3, 7], "semblo_target_tokens": 4096}


class _Block(nn.Module):
    def __init__(self, hkv, dim, index_dim):
        super().__init__()
        self.semblo_key_router = SembloKeyRouter(hkv, dim, index_dim)
        self.qkv_proj = nn.Linear(4, 4)


class _Model(nn.Module):
    """Layers 3 and 7 carry a router (under ``mixer`` like Nemotron-H or ``self_attn`` like Qwen3.5)."""

    def __init__(self, hkv=4, block="self_attn", prefix_depth=1):
        super().__init__()
        layers = nn.ModuleList()
        for i in range(8):
            holder = nn.Module()
            if i in (3, 7):
                setattr(holder, block, _Block(hkv, 8, 8 if i == 3 else 6))
            layers.append(holder)
        inner = nn.Module()
        inner.layers = layers
        if prefix_depth == 2:
            outer = nn.Module()
            outer.language_model = inner
            inner = outer
        self.model = inner


def test_canonical_names():
    assert RW.canonical_runtime_name("model.layers.5.mixer.semblo_key_router.weight") \
        == "layers.5.self_attn.semblo_key_router.weight"
    assert RW.canonical_runtime_name("model.language_model.layers.4.self_attn.semblo_key_router.weight") \
        == "layers.4.self_attn.semblo_key_router.weight"
    assert RW.canonical_runtime_name("model.layers.5.mixer.qkv_proj.weight") is None
    assert RW.canonical_runtime_name("model.layers.5.mixer.in_proj.weight") is None
    assert RW.canonical_runtime_name("model.norm.self_attn.semblo_key_router.weight") is None
    assert RW.is_runtime_parameter("layers.0.self_attn.semblo_key_router.weight")
    kept = list(RW.filter_base_weight_iterator([("model.layers.3.self_attn.semblo_key_router.weight", torch.zeros(1)),
                                                ("model.layers.3.self_attn.qkv_proj.weight", torch.zeros(1))]))
    assert [n for n, _ in kept] == ["model.layers.3.self_attn.qkv_proj.weight"]


def test_reads_a_directory_the_reference_wrote():
    manifest = RW.verify_runtime_weights(GOLDEN)
    want = _golden_tensors()
    assert manifest.tensor_names == tuple(sorted(want))
    assert manifest.semblo_config == {k: v for k, v in _CONFIG.items() if k.startswith("semblo_")}
    for block, depth in (("self_attn", 1), ("mixer", 1), ("self_attn", 2)):
        model = _Model(block=block, prefix_depth=depth)
        written = RW.load_runtime_weights_into_module(model, GOLDEN)
        assert len(written) == 2 and all(n.endswith("semblo_key_router.weight") for n in written)
        for name, parameter in model.named_parameters():
            canonical = RW.canonical_runtime_name(name)
            if canonical is not None:
                assert torch.equal(parameter.data, want[canonical].to(parameter.dtype))
        router = dict(model.named_modules())[[n for n, _ in model.named_modules() if n.endswith(f"3.{block}")][0]]
        assert not router.semblo_key_router.is_identity()      # the loaded weight is noticed


def test_writer_gives_the_reference_manifest(tmp_path):
    ours = RW.write_runtime_weights(tmp_path, _golden_tensors(), _CONFIG, "x")
    theirs = RW.read_runtime_manifest(GOLDEN)
    for field in ("schema_version", "source_config_sha256", "weights_file", "tensor_names", "tensor_shapes",
                  "tensor_dtypes", "tensor_sha256", "semblo_config"):
        assert getattr(ours, field) == getattr(theirs, field), field
    assert RW.verify_runtime_weights(tmp_path) == ours
    on_disk = json.loads((tmp_path / RW.RUNTIME_MANIFEST_FILE).read_text())
    assert sorted(on_disk) == sorted(json.loads((GOLDEN / RW.RUNTIME_MANIFEST_FILE).read_text()))
    with pytest.raises(ValueError):
        RW.write_runtime_weights(tmp_path / "bad", {"model.layers.3.self_attn.semblo_key_router.weight": torch.zeros(1)},
                                 _CONFIG, "x")


def test_heads_are_cut_for_a_rank():
    """A file with 4 KV heads into ranks that hold 2 each (tensor parallelism over KV heads)."""
    want = _golden_tensors()
    for rank in range(2):
        model = _Model(hkv=2)
        RW.load_runtime_weights_into_module(model, GOLDEN, tp_rank=rank, tp_size=2)
        for name, parameter in model.named_parameters():
            canonical = RW.canonical_runtime_name(name)
            if canonical is not None:
                assert torch.equal(parameter.data, want[canonical][2 * rank:2 * rank + 2].to(parameter.dtype))
    with pytest.raises(ValueError):
        RW.load_runtime_weights_into_module(_Model(hkv=2), GOLDEN)                 # no tp_size: shapes differ
    with pytest.raises(ValueError):
        RW.load_runtime_weights_into_module(_Model(hkv=3), GOLDEN, tp_rank=0, tp_size=2)


def test_mismatches_raise(tmp_path):
    for f in GOLDEN.iterdir():
        shutil.copy(f, tmp_path / f.name)
    RW.verify_runtime_weights(tmp_path)
    # a model without layer 7's router: refused, unless whole unused layers may be skipped
    model = _Model()
    del model.model.layers[7].self_attn
    with pytest.raises(ValueError):
        RW.load_runtime_weights_into_module(model, tmp_path)
    assert len(RW.load_runtime_weights_into_module(model, tmp_path, allow_unused_layer_parameters=True)) == 1
    # a model with a router the file does not hold
    model = _Model()
    model.model.layers[5].self_attn = _Block(4, 8, 8)
    with pytest.raises(ValueError):
        RW.load_runtime_weights_into_module(model, tmp_path)
    assert len(RW.load_runtime_weights_into_module(model, tmp_path, require_exact_match=False)) == 2
    # a query router of the earlier file format: zero tensors are dropped, trained ones refused
    t = _golden_tensors()
    names = sorted(t) + ["layers.3.self_attn.semblo_query_router.down"]
    t["layers.3.self_attn.semblo_query_router.down"] = torch.zeros(2, 2)
    assert len(RW.load_runtime_tensors_into_module(_Model(), t, names)) == 2
    t["layers.3.self_attn.semblo_query_router.down"] = torch.ones(2, 2)
    with pytest.raises(ValueError):
        RW.load_runtime_tensors_into_module(_Model(), t, names)
    with pytest.raises(ValueError):
        RW.load_runtime_tensors_into_module(_Model(), _golden_tensors(), ["layers.3.self_attn.semblo_key_router.weight"])
    # an altered manifest, an altered file, a missing file, an unknown schema
    manifest = json.loads((tmp_path / RW.RUNTIME_MANIFEST_FILE).read_text())
    broken = dict(manifest, tensor_shapes=dict(manifest["tensor_shapes"],
                                               **{"layers.7.self_attn.semblo_key_router.weight": [4, 8, 6]}))
    (tmp_path / RW.RUNTIME_MANIFEST_FILE).write_text(json.dumps(broken))
    with pytest.raises(ValueError):
        RW.verify_runtime_weights(tmp_path)
    (tmp_path / RW.RUNTIME_MANIFEST_FILE).write_text(json.dumps(dict(manifest, schema_version=2)))
    with pytest.raises(ValueError):
        RW.verify_runtime_weights(tmp_path)
    (tmp_path / RW.RUNTIME_MANIFEST_FILE).write_text(json.dumps(manifest))
    blob = bytearray((tmp_path / RW.RUNTIME_WEIGHTS_FILE).read_bytes())
    blob[-1] ^= 1
    (tmp_path / RW.RUNTIME_WEIGHTS_FILE).write_bytes(bytes(blob))
    with pytest.raises(ValueError):
        RW.verify_runtime_weights(tmp_path)
    (tmp_path / RW.RUNTIME_WEIGHTS_FILE).unlink()
    with pytest.raises(FileNotFoundError):
        RW.verify_runtime_weights(tmp_path)
    with pytest.raises(FileNotFoundError):
        RW.read_runtime_manifest(tmp_path / "nowhere")
    with pytest.raises(ValueError):
        RW.semblo_config_fields({"text_config": 3})
