"""SembloVllmConfig.from_hf_config: the checkpoint keys and the environment overrides of the hot path, after
the reference's tests/test_budget_from_environment.py:33-58 and tests/test_decode_only_budget.py:59-110."""
import types

import pytest

from semblo_b200.config import SembloVllmConfig
from semblo_b200.model import SembloAttention

# what the paper's settings turn on; without these the package refuses the config (it builds that path only)
PATH = {"semblo_enabled": True, "semblo_vllm_pack_prompt_kv": True, "semblo_fused_select_block_queries": 32,
        "semblo_vllm_own_prompt_cache": "True", "semblo_flat_unit_tokens": 64}
BASE = dict(PATH, semblo_target_tokens=4096, semblo_vllm_token_capacity=262144)
ENV = ("SEMBLO_TARGET_TOKENS", "SEMBLO_DECODE_TARGET_TOKENS", "SEMBLO_DENSE_TAIL_TOKENS", "SEMBLO_PREFILL_CHUNK",
       "SEMBLO_RUNTIME_CHECKS", "SEMBLO_ENGAGE_ABOVE_TOKENS", "SEMBLO_FULL_GRAPH_DECODE", "SEMBLO_ATTN_CHUNK")


@pytest.fixture(autouse=True)
def clean_env(monkeypatch):
    for name in ENV:
        monkeypatch.delenv(name, raising=False)


def _build(text):
    return SembloVllmConfig.from_hf_config(types.SimpleNamespace(text_config=text))


def test_budget_from_config_and_environment(monkeypatch):
    assert _build(BASE).target_tokens == 4096
    monkeypatch.setenv("SEMBLO_TARGET_TOKENS", "16384")
    assert _build(BASE).target_tokens == 16384
    assert _build(dict(PATH, semblo_vllm_token_capacity=262144)).target_tokens == 16384
    with pytest.raises(ValueError, match="token_capacity"):       # checked after the override is applied
        _build(dict(PATH, semblo_vllm_token_capacity=4096))


class _Layer:
    """The lines of ``_init_semblo_runtime`` that decide a layer's budgets."""

    def __init__(self, rc, layer_idx):
        self.layer_idx = layer_idx
        self.layer_target_tokens = rc.layer_target_tokens.get(layer_idx, rc.target_tokens)
        self.layer_decode_target_tokens = (
            self.layer_target_tokens if layer_idx in rc.layer_target_tokens or not rc.decode_target_tokens
            else rc.decode_target_tokens)


def test_decode_only_budget(monkeypatch):
    text = dict(PATH, semblo_target_tokens=8192, semblo_vllm_token_capacity=524288)
    monkeypatch.setenv("SEMBLO_TARGET_TOKENS", "16384")
    rc = _build(text)
    assert rc.decode_target_tokens == 0
    assert (_Layer(rc, 3).layer_target_tokens, _Layer(rc, 3).layer_decode_target_tokens) == (16384, 16384)
    monkeypatch.setenv("SEMBLO_TARGET_TOKENS", "32768")
    monkeypatch.setenv("SEMBLO_DECODE_TARGET_TOKENS", "524288")
    layer = _Layer(_build(text), 3)
    assert (layer.layer_target_tokens, layer.layer_decode_target_tokens) == (32768, 524288)
    # the budget is chosen per step: a prefill after a decode is back on its own
    rule = SembloAttention._target_for_step
    assert [rule(layer, False), rule(layer, True), rule(layer, False)] == [32768, 524288, 32768]
    # a per-layer budget wins over the decode-only one
    rc = _build(dict(text, semblo_target_tokens_per_layer={"3": 4096}))
    assert _Layer(rc, 3).layer_decode_target_tokens == 4096 and _Layer(rc, 4).layer_decode_target_tokens == 524288
    monkeypatch.delenv("SEMBLO_DECODE_TARGET_TOKENS")
    assert _build(dict(text, semblo_decode_target_tokens=262144)).decode_target_tokens == 262144
    with pytest.raises(ValueError):
        _build(dict(text, semblo_target_tokens_per_layer=[4096]))
    with pytest.raises(ValueError):
        _build(dict(text, semblo_target_tokens_per_layer={"3": 0}))


def test_other_keys_and_overrides(monkeypatch):
    text = dict(BASE, layer_types=["linear_attention", "full_attention", "linear_attention", "full_attention"],
                semblo_selection_temperature=0.1, semblo_bucket_size_penalty=0.25, semblo_vllm_query_chunk_size=8192,
                semblo_vllm_codebook_seed=7, semblo_runtime_weights_file="semblo_runtime.safetensors",
                semblo_runtime_manifest_file="semblo_runtime.json", semblo_index_dim=256)
    rc = _build(text)
    assert rc.layer_indices == (1, 3) and rc.mode == "sparse" and rc.own_prompt_cache is True
    assert (rc.selection_temperature, rc.bucket_size_penalty, rc.query_chunk_size, rc.codebook_seed) == (0.1, 0.25, 8192, 7)
    assert rc.runtime_weights_file == "semblo_runtime.safetensors" and rc.index_dim == 256
    assert rc.engage_above_tokens == 131072 and rc.runtime_checks is True and rc.prefill_chunk == 0
    assert _build(dict(text, semblo_layer_indices=[3])).layer_indices == (3,)
    assert SembloVllmConfig.from_hf_config(text).layer_indices == (1, 3)            # a plain dict, no text_config
    monkeypatch.setenv("SEMBLO_ENGAGE_ABOVE_TOKENS", "0")
    monkeypatch.setenv("SEMBLO_RUNTIME_CHECKS", "off")
    monkeypatch.setenv("SEMBLO_PREFILL_CHUNK", "8192")
    rc = _build(text)
    assert (rc.engage_above_tokens, rc.runtime_checks, rc.prefill_chunk) == (0, False, 8192)
    monkeypatch.setenv("SEMBLO_ENGAGE_ABOVE_TOKENS", "65536")
    assert _build(text).engage_above_tokens == 65536
    monkeypatch.setenv("SEMBLO_FULL_GRAPH_DECODE", "1")                               # every request engages the index
    assert _build(text).engage_above_tokens == 0
    with pytest.raises(ValueError):
        SembloVllmConfig.from_hf_config(types.SimpleNamespace(text_config=text), identity_router=True)
    # what this package does not build is refused, not ignored
    for bad in ({"semblo_vllm_own_prompt_cache": "False"}, {"semblo_vllm_own_prompt_cache": "perhaps"},
                {"semblo_flat_unit_tokens": 0}, {"semblo_vllm_mode": "all_tokens"}, {"semblo_enabled": False},
                {"semblo_kmeans_init": "kmeans++"}, {"semblo_dense_tail_tokens": 128}):
        with pytest.raises(ValueError):
            _build(dict(text, **bad))
    monkeypatch.setenv("SEMBLO_DENSE_TAIL_TOKENS", "64")
    with pytest.raises(ValueError):
        _build(text)
    monkeypatch.delenv("SEMBLO_DENSE_TAIL_TOKENS")
    monkeypatch.setenv("SEMBLO_ATTN_CHUNK", "4096")                                   # a slice variable of an earlier scheme
    with pytest.raises(ValueError, match="SEMBLO_PREFILL_CHUNK"):
        _build(text)
