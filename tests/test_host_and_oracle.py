"""CPU-side checks: the oracle's device-only restatements against an independent float64
loop, the C-ABI library's exported symbols, and host logic that needs no GPU."""
from __future__ import annotations

import ctypes
import os
import re
from pathlib import Path

import pytest
import torch

from oracle import semblo_oracle as O

ROOT = Path(__file__).resolve().parent.parent


def _problem(sink):
    data = O.mixture_inputs(length=1536, num_q_heads=4, num_kv_heads=2, head_dim=32, centres=12, seed=4)
    product = O.routing_normalize(data["k_pre"])
    index = O.build_flat(product, unit_tokens=16, min_clusters_log2=5, kmeans_sample_size=512, fit_iters=3,
                         seed=1, sink=sink, page_align=16)
    O.pack_prompt_kv(index, data["k_post"], data["v"])
    return data, index


@pytest.mark.parametrize("sink", [0, 32])
def test_prefill_body_against_a_per_query_float64_loop(sink):
    data, index = _problem(sink)
    target, local, cs, ce = 128, 64, 1024, 1024 + 63
    ws = cs - local
    sizes = O.causal_sizes_at(index, ws - 1)
    qpos = torch.arange(cs, ce + 1)
    vectors = O.trivial_router_vectors(data["q_pre"][cs:ce + 1])
    sel = O.select_clusters(vectors, index.codebooks, sizes, temperature=0.1, beta=0.25, target_tokens=target, sink=sink)
    if sink:
        assert bool(sel[..., 0].all())
    out, natt = O.sparse_chunk_attention(data["q_post"][cs:ce + 1], index, sel, sizes, qpos,
                                         data["k_post"][ws:ce + 1], data["v"][ws:ce + 1], ws, 32 ** -0.5)
    k, v = data["k_post"].double(), data["v"].double()
    for qi in (0, 17, 63):
        p = cs + qi
        for h in range(2):
            # the attended POSITIONS: members of selected clusters below the window, plus the window
            keys = [pos for pos in range(ws) if bool(sel[qi, h, index.assign[h, pos]])] + list(range(ws, p + 1))
            assert len(keys) == int(natt[qi, h])
            for t in range(2):
                q = data["q_post"][p, h * 2 + t].double()
                logits = (k[keys, h] @ q) * 32 ** -0.5
                w = torch.softmax(logits, dim=0)
                want = w @ v[keys, h]
                torch.testing.assert_close(out[qi, h * 2 + t], want, atol=1e-9, rtol=1e-9)


def test_decode_step_against_a_float64_loop():
    data, index = _problem(32)
    a = O.make_arena(capacity=2048, num_clusters=128, num_kv_heads=2, head_dim=32, page_align=16, reserve=256,
                     kv_dtype=torch.bfloat16, desc_dtype=torch.bfloat16, keep_kpre=True)
    short = O.build_flat(O.routing_normalize(data["k_pre"][:1500]), unit_tokens=16, min_clusters_log2=5,
                         kmeans_sample_size=512, fit_iters=3, seed=1, sink=32, page_align=16)
    O.pack_prompt_kv(short, data["k_post"][:1500], data["v"][:1500])
    O.arena_adopt(a, short)
    assert int(a.prompt_length_t) == 1500
    for pos in range(1500, 1504):
        out, sel, natt = O.decode_step(a, q_post=data["q_post"][pos], q_pre=data["q_pre"][pos], pos=pos,
                                       k_post=data["k_post"][pos], v=data["v"][pos], k_pre=data["k_pre"][pos],
                                       temperature=0.1, beta=0.25, target_tokens=128, sink=32, sm_scale=32 ** -0.5)
        assert bool(sel[:, 0].all())
        for h in range(2):
            keys = [p for p in range(1500) if bool(sel[h, short.assign[h, p]])] + list(range(1500, pos + 1))
            assert len(keys) == int(natt[h])
            q = data["q_post"][pos, h * 2].double()
            w = torch.softmax((data["k_post"][keys, h].double() @ q) * 32 ** -0.5, dim=0)
            torch.testing.assert_close(out[h * 2], w @ data["v"][keys, h].double(), atol=1e-9, rtol=1e-9)


def test_flush_moves_the_oldest_suffix_tokens_into_their_clusters():
    data, index = _problem(0)
    a = O.make_arena(capacity=2048, num_clusters=128, num_kv_heads=2, head_dim=32, page_align=16, reserve=256,
                     kv_dtype=torch.bfloat16, desc_dtype=torch.bfloat16, keep_kpre=True, packed_capacity=2048 + 256)
    short = O.build_flat(O.routing_normalize(data["k_pre"][:1400]), unit_tokens=16, min_clusters_log2=5,
                         kmeans_sample_size=512, fit_iters=3, seed=1, page_align=16)
    O.pack_prompt_kv(short, data["k_post"][:1400], data["v"][:1400])
    O.arena_adopt(a, short)
    for pos in range(1400, 1440):
        O.suffix_write(a, pos, data["k_post"][pos], data["v"][pos], data["k_pre"][pos])
    before = int(a.sizes.sum())
    O.flush_arena(a, 1400, 1424, 16)
    assert int(a.prompt_length_t) == 1424 and int(a.sizes.sum()) == before + 2 * 24
    for h in range(2):
        for c in range(128):
            lo, n = int(a.indptr[h, c]), int(a.sizes[h, c])
            pos = a.posting[h, lo:lo + n]
            assert bool((pos[1:] > pos[:-1]).all())
            assert torch.equal(a.packed_kv[0, lo:lo + n, h].float(), data["k_post"][pos.long(), h].float())


def test_library_exports_every_declared_symbol():
    from semblo_b200 import _lib
    header = (ROOT / "include" / "semblo_b200.h").read_text()
    declared = set(re.findall(r"\b(semblo_[a-z_0-9]+)\s*\(", header))
    assert declared, "no declarations found"
    assert declared == set(_lib.exported_symbols())
    handle = ctypes.CDLL(str(_lib.library_path()))
    for name in declared:
        assert hasattr(handle, name), name
    assert _lib.lib().semblo_version() >= 100


def test_product_path_refuses_cpu_tensors_and_ablation_flags(monkeypatch):
    from semblo_b200 import flat_index
    from semblo_b200.state import ProductPostingIndex, flat_num_clusters
    with pytest.raises(RuntimeError, match="CUDA"):
        flat_index.routing_normalize(torch.randn(4, 2, 64).to(torch.bfloat16))
    monkeypatch.setenv("SEMBLO_ROUTING_NORMALIZE", "half")
    with pytest.raises(RuntimeError, match="whole-vector"):
        flat_index.routing_mode()
    monkeypatch.delenv("SEMBLO_ROUTING_NORMALIZE")
    assert [flat_num_clusters(n, 64, 7) for n in (8192, 131072, 524288, 1048576)] == [128, 2048, 8192, 16384]
    monkeypatch.setenv("SEMBLO_FLAT_CLUSTERS", "4096")
    assert flat_num_clusters(65536, 64, 7) == 4096


def test_arena_cluster_count_matches_the_reference_table(golden):
    from semblo_b200.arena import arena_cluster_count
    for length, unit, ml, want in golden["cluster_count_table"].tolist():
        assert arena_cluster_count(length, unit, ml) == want


def test_gather_form_of_the_prefill_body_agrees_with_the_masked_form():
    data, index = _problem(32)
    cs, ce, ws = 1024, 1024 + 15, 960
    sizes = O.causal_sizes_at(index, ws - 1)
    qpos = torch.arange(cs, ce + 1)
    sel = O.select_clusters(O.trivial_router_vectors(data["q_pre"][cs:ce + 1]), index.codebooks, sizes,
                            temperature=0.1, beta=0.25, target_tokens=128, sink=32)
    want, _ = O.sparse_chunk_attention(data["q_post"][cs:ce + 1], index, sel, sizes, qpos, data["k_post"][ws:ce + 1],
                                       data["v"][ws:ce + 1], ws, 32 ** -0.5)
    got = O.sparse_chunk_attention_gather(data["q_post"][cs:ce + 1], index, sel, sizes, qpos,
                                          data["k_post"][ws:ce + 1], data["v"][ws:ce + 1], ws, 32 ** -0.5,
                                          dtype=torch.float64)
    torch.testing.assert_close(got, want, atol=1e-9, rtol=1e-9)


def test_routing_map_projection_and_identity_detection():
    """routing_map.SembloKeyRouter (routing_map.py:67-94 of the reference): identity by default, a query
    goes through the map of its KV head, and a loaded weight is noticed."""
    from semblo_b200.routing_map import SembloKeyRouter
    hkv, hq, dim = 2, 8, 16
    router = SembloKeyRouter(hkv, dim, dim)
    assert router.is_identity()
    g = torch.Generator().manual_seed(0)
    keys = torch.randn(5, hkv, dim, generator=g)
    queries = torch.randn(7, hq, dim, generator=g)
    assert torch.equal(router.project(keys), keys) and torch.equal(router.project_queries(queries), queries)
    w = torch.randn(hkv, dim, dim, generator=g)
    router.load_weight(w)
    assert not router.is_identity()
    torch.testing.assert_close(router.project(keys), torch.einsum("lhd,hid->lhi", keys, w))
    want_q = torch.stack([queries[:, t] @ w[t // (hq // hkv)].T for t in range(hq)], dim=1)
    torch.testing.assert_close(router.project_queries(queries), want_q)
    with pytest.raises(ValueError):
        SembloKeyRouter(hkv, dim, 0)
    with pytest.raises(ValueError):
        router(keys)                       # [B, L, Hkv, D] is required
    # a map into fewer dimensions: the kernels get the projection followed by zeros, which leaves the
    # partition of the oracle's build where it is (norms, dot products and means ignore the zeros)
    narrow = SembloKeyRouter(hkv, dim, 10)
    assert not narrow.is_identity()
    narrow.load_weight(w[:, :10])
    proj = narrow.project(keys)
    assert tuple(proj.shape) == (5, hkv, 10)
    wide = narrow.widen(proj)
    assert tuple(wide.shape) == (5, hkv, dim) and torch.equal(wide[..., :10], proj) and not wide[..., 10:].any()
    with pytest.raises(ValueError):
        SembloKeyRouter(hkv, dim, dim + 2)


def test_routing_map_makers():
    """The maps of the reference's routing-key comparisons (scripts/make_routing_map.py:44-120)."""
    from semblo_b200.routing_map import SembloKeyRouter, non_rotary_map, pca_map, random_map
    hkv, dim = 2, 16
    w = non_rotary_map(hkv, dim, 4)
    assert tuple(w.shape) == (hkv, dim, dim) and not w[:, :4].any() and torch.equal(w[0, 4:, 4:], torch.eye(12))
    g = torch.Generator().manual_seed(4)
    r = random_map(hkv, dim, 6, g)
    assert tuple(r.shape) == (hkv, 6, dim)
    torch.testing.assert_close(r @ r.transpose(1, 2), torch.eye(6).expand(hkv, 6, 6), atol=1e-5, rtol=0)
    assert not torch.allclose(r[0], r[1])
    # keys that live in a 3-dimensional subspace per head: the top 3 rows span it, the 4th explains nothing
    basis = torch.linalg.qr(torch.randn(hkv, dim, 3, generator=g))[0]                      # [Hkv, D, 3]
    coef = torch.randn(200, hkv, 3, generator=g) * torch.tensor([5.0, 2.0, 1.0])
    keys = torch.einsum("lhr,hdr->lhd", coef, basis)
    p = pca_map(keys, 8, rank=4)
    assert tuple(p.shape) == (hkv, 8, dim) and not p[:, 4:].any()
    torch.testing.assert_close(p[:, :4] @ p[:, :4].transpose(1, 2), torch.eye(4).expand(hkv, 4, 4), atol=1e-5, rtol=0)
    inside = torch.einsum("hid,hdr->hir", p[:, :3], basis)                                # rows 0-2 lie in the span
    torch.testing.assert_close((inside ** 2).sum(-1), torch.ones(hkv, 3), atol=1e-4, rtol=0)
    explained = torch.einsum("lhd,hid->lhi", keys, p).pow(2).sum(0)                       # [Hkv, 8]
    assert (explained[:, 0] > explained[:, 1]).all() and (explained[:, 1] > explained[:, 2]).all()
    assert (explained[:, 3] < 1e-3 * explained[:, 2]).all()
    for made in (w, r, p):
        router = SembloKeyRouter(hkv, dim, made.shape[1])
        router.load_weight(made)
        assert not router.is_identity()
    with pytest.raises(ValueError):
        random_map(hkv, dim, dim + 1, g)
    with pytest.raises(ValueError):
        pca_map(keys, 4, rank=5)


def test_zero_padded_routing_space_gives_the_same_index():
    """What a narrowing routing map relies on: the oracle's index build on I-dimensional routing keys and on
    the same keys followed by zeros is the same partition."""
    length, hkv, idim, dim = 1024, 2, 24, 32
    data = O.mixture_inputs(length=length, num_q_heads=4, num_kv_heads=hkv, head_dim=dim, centres=12, seed=5)
    g = torch.Generator().manual_seed(1)
    w = torch.randn(hkv, idim, dim, generator=g)
    proj = torch.einsum("lhd,hid->lhi", data["k_pre"].float(), w)
    proj = torch.nn.functional.normalize(proj, dim=-1).to(torch.bfloat16)
    padded = torch.nn.functional.pad(proj, (0, dim - idim))
    a = O.build_flat(proj, unit_tokens=32, min_clusters_log2=3, kmeans_sample_size=512, fit_iters=4, seed=7)
    b = O.build_flat(padded, unit_tokens=32, min_clusters_log2=3, kmeans_sample_size=512, fit_iters=4, seed=7)
    same = (a.assign == b.assign).float().mean().item()
    assert same > 0.995, same


def test_suffix_flusher_bookkeeping(monkeypatch):
    """suffix_flush.SuffixFlusher (suffix_flush.py:211-283 of the reference) with the flush itself replaced
    by a recorder: counting starts at the first single-token step after anything else, a flush is due when
    the exact suffix reaches keep + every, it moves all but the newest `keep` positions of every arena, and a
    new prompt starts a new count."""
    from types import SimpleNamespace
    from semblo_b200 import suffix_flush as F
    monkeypatch.setenv("SEMBLO_SUFFIX_FLUSH_EVERY", "4")
    monkeypatch.setenv("SEMBLO_SUFFIX_KEEP_EXACT", "3")
    calls = []

    def fake_flush(arena, module, frm, to, tmp=None):
        calls.append((module, frm, to))
        arena.index.prompt_length = to
        return 0

    monkeypatch.setattr(F, "flush_layer", fake_flush)
    arenas = {l: SimpleNamespace(index=SimpleNamespace(prompt_length=100), suffix_kpre=object()) for l in (2, 5)}
    state = SimpleNamespace(index_buffers={("arena", 2): arenas[2], ("arena", 5): arenas[5], "other": 1,
                                           (("arena", 2), "sig"): 0},
                            prompt_epoch=1, source_modules={2: "m2", 5: "m5"})
    holder = SimpleNamespace(modules=lambda: [SimpleNamespace(), SimpleNamespace(runtime_state=state)])
    runner = SimpleNamespace(model=SimpleNamespace(model=holder))          # wrapped once
    one = SimpleNamespace(total_num_scheduled_tokens=1, num_scheduled_tokens={"r": 1})
    chunk = SimpleNamespace(total_num_scheduled_tokens=100, num_scheduled_tokens={"r": 100})
    fl = F.SuffixFlusher()
    assert (fl.keep, fl.every) == (3, 4)
    fl.before_step(runner, chunk)
    assert fl.pending_reset and fl.state is None and not calls
    for step in range(7):                       # 7 tokens written before the 8th step: suffix 7 = keep + every
        fl.before_step(runner, one)
        assert not calls, step
    fl.before_step(runner, one)
    assert calls == [("m2", 100, 104), ("m5", 100, 104)] and fl.flushes == 1 and fl.written == 8
    for step in range(3):
        fl.before_step(runner, one)
    assert len(calls) == 2
    fl.before_step(runner, one)                 # 11 written, suffix 111 - 104 = 7 again
    assert calls[2:] == [("m2", 104, 108), ("m5", 104, 108)]
    # two requests in a step, then a new prompt of 50 tokens
    fl.before_step(runner, SimpleNamespace(total_num_scheduled_tokens=2, num_scheduled_tokens={"a": 1, "b": 1}))
    assert fl.pending_reset
    state.prompt_epoch = 2
    for a in arenas.values():
        a.index.prompt_length = 50
    fl.before_step(runner, one)
    assert (fl.prompt_len, fl.written) == (50, 1) and len(calls) == 4
    # an arena without stored pre-RoPE keys cannot be flushed: nothing happens
    arenas[5].suffix_kpre = None
    before = fl.written
    fl.before_step(runner, one)
    assert fl.written == before
    arenas[5].suffix_kpre = object()
    state.source_modules.pop(5)
    fl.written = 6
    fl.before_step(runner, one)
    with pytest.raises(RuntimeError):
        fl.before_step(runner, one)

