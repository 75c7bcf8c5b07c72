"""The operator boundary: a layer subclass with fixed projections is driven through
``torch.ops.semblo.attention`` for a whole prompt (index build, packing, the query-chunk loop),
the adoption into the decode arena and a few generated tokens, as the reference's model hooks
drive it (semblo/vllm_plugin/model.py:1130-1269)."""
from __future__ import annotations

import os
from types import SimpleNamespace

import pytest
import torch

from oracle import semblo_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from semblo_b200 import _lib
    _lib.lib()
    return torch.device("cuda:0")


def _make_layer(data, dev, *, hq, hkv, dim, cfg, state, name):
    from semblo_b200.model import SembloAttention

    class Layer(SembloAttention):
        """The model-specific half: projections are lookups into the synthetic tensors."""

        def __init__(self):
            super().__init__()
            self.num_heads, self.num_kv_heads, self.head_dim = hq, hkv, dim
            self.scaling = dim ** -0.5
            self.is_kv_shared_layer = False
            self.attn = SimpleNamespace(layer_name=name)
            self._init_semblo_runtime(runtime_config=cfg, runtime_state=state, layer_idx=0, source_layer_idx=0,
                                      uses_sparse_attention=True, builds_product_index=True,
                                      attention_logits_soft_cap=None)

        def _project_qkv(self, positions, hidden_states):
            idx = positions.long()
            d = {k: v[idx] for k, v in data.items()}
            n = idx.numel()
            if n == 1:
                # a serving engine hands the decode step the same buffers every time
                if getattr(self, "_step_buffers", None) is None:
                    self._step_buffers = {k: torch.empty_like(v) for k, v in d.items()}
                for k, v in d.items():
                    self._step_buffers[k].copy_(v)
                d = self._step_buffers
            return (d["q_post"].reshape(n, hq * dim), d["k_post"].reshape(n, hkv * dim), d["v"], d["q_pre"],
                    d["k_pre"], None)

        def _finish_output(self, attn_output, gate):
            return attn_output

    return Layer()


def test_prompt_and_decode_through_the_operator(dev):
    from semblo_b200 import _lib
    from semblo_b200.config import SembloVllmConfig
    from semblo_b200.fused_prefill import CausalSnapshot, fused_chunk_attention
    from semblo_b200.state import SembloRuntimeState
    from semblo_b200.trivial_router import trivial_router_vectors
    import semblo_b200
    dim, hq, hkv, sink, length, target, local, chunk, steps = 128, 8, 2, 64, 5120, 256, 128, 1024, 5
    cpu = O.mixture_inputs(length=length + steps, num_q_heads=hq, num_kv_heads=hkv, head_dim=dim, centres=24, seed=5)
    data = {k: v.to(dev) for k, v in cpu.items()}
    cfg = SembloVllmConfig(token_capacity=8192, target_tokens=target, flat_unit_tokens=32, index_dim=dim,
                           flat_min_clusters_log2=7, kmeans_sample_size=1024, query_chunk_size=chunk,
                           packed_decode_num_splits=4)
    state = SembloRuntimeState(max_model_len=8192 + 512)
    env = dict(SEMBLO_SINK_TOKENS=str(sink), SEMBLO_FA3_LOCAL=str(local), SEMBLO_FULL_GRAPH_DECODE="1",
               SEMBLO_FLAT_UNIT_TOKENS="32", SEMBLO_FA3_ALIGN="16")
    os.environ.update(env)
    try:
        layer = _make_layer(data, dev, hq=hq, hkv=hkv, dim=dim, cfg=cfg, state=state, name="model.layers.0.self_attn.attn")
        calls = semblo_b200.SPARSE_ATTENTION_CALLS
        positions = torch.arange(length, device=dev)
        hidden = torch.zeros(length, 8, dtype=torch.bfloat16, device=dev)
        out = layer._sparse_layer_forward(positions, hidden).view(length, hq, dim)
        torch.cuda.synchronize()
        _lib.status_for(dev).raise_if_set()
        assert semblo_b200.SPARSE_ATTENTION_CALLS > calls          # the sparse path ran
        index = state.get(0)
        assert index.original_kv is None                            # the prompt-order views were dropped
        arena = layer._arena(data["q_post"])
        assert arena.adopted_epoch == state.prompt_epoch
        assert int(arena.prompt_length_t.item()) == length
        # the same chunk loop by hand over the same index: identical bytes
        index.original_kv = (data["k_post"][:length], data["v"][:length])
        snap = CausalSnapshot(index)
        want = torch.empty(length, hq, dim, dtype=torch.bfloat16, device=dev)
        selections = {}
        for cs in range(0, length, chunk):
            ce = cs + chunk - 1
            qv = trivial_router_vectors(data["q_pre"][cs:ce + 1])
            fused_chunk_attention(data["q_post"][cs:ce + 1], SimpleNamespace(vectors=qv.view(1, chunk, hq, 1, dim)),
                                  index, torch.arange(cs, ce + 1, dtype=torch.int32, device=dev), snap, cs, ce,
                                  temperature=0.1, beta=0.25, target_tokens=target, sm_scale=dim ** -0.5,
                                  out=want[cs:ce + 1])
            if O.chunk_plan(cs, target, local) > 0:
                selections[cs] = O.unpack_bits(snap.qmask[:chunk].cpu())
        assert torch.equal(out, want)
        # and the oracle on the kernel's own selections
        oidx = O.FlatIndex(codebooks=index.codebooks.cpu(), posting_positions=index.posting_positions.cpu(),
                           bucket_indptr=index.bucket_indptr.cpu(), bucket_sizes=index.bucket_sizes.cpu(),
                           inverse_positions=index.inverse_positions().cpu(), assign=index.orig_bucket.cpu().long(),
                           prompt_length=length, page_align=16, packed_kv=index.packed_kv.cpu())
        ref = O.prefill_attention(cpu["q_post"][:length], cpu["q_pre"][:length], cpu["k_post"][:length],
                                  cpu["v"][:length], oidx, temperature=0.1, beta=0.25, target_tokens=target, sink=sink,
                                  local=local, sm_scale=dim ** -0.5, chunk=chunk, selections=dict(selections))
        diff = (out.cpu().double() - ref).abs()
        assert float(diff.max()) <= 2e-2 and float(diff.mean()) <= 1e-3
        # generated tokens: one position per call through the same operator
        aref = O.make_arena(capacity=8192, num_clusters=arena.num_clusters, num_kv_heads=hkv, head_dim=dim,
                            page_align=16, reserve=arena.reserve, kv_dtype=torch.bfloat16, desc_dtype=torch.bfloat16)
        O.arena_adopt(aref, oidx)
        for s in range(steps):
            pos = length + s
            o = layer._sparse_layer_forward(torch.tensor([pos], device=dev), hidden[:1]).view(hq, dim)
            _lib.status_for(dev).raise_if_set()
            ws = arena.fused_decode_ws
            sel = torch.zeros(hkv, arena.num_clusters, dtype=torch.bool)
            for h in range(hkv):
                n = int(ws.rcount[h])
                ids = torch.searchsorted(aref.indptr[h].contiguous(), ws.rstart[h, :n].cpu(), right=True) - 1
                sel[h, ids] = True
            wd, _, _ = O.decode_step(aref, q_post=cpu["q_post"][pos], q_pre=cpu["q_pre"][pos], pos=pos,
                                     k_post=cpu["k_post"][pos], v=cpu["v"][pos], temperature=0.1, beta=0.25,
                                     target_tokens=target, sink=sink, sm_scale=dim ** -0.5, sel=sel)
            d = (o.cpu().double() - wd).abs()
            assert float(d.max()) <= 2e-2 and float(d.mean()) <= 1e-3, (s, float(d.max()))
        # a second prompt reuses the arena's buffers (same addresses) under a new epoch
        ptr_before = arena.packed_kv.data_ptr()
        out2 = layer._sparse_layer_forward(positions, hidden).view(length, hq, dim)
        torch.cuda.synchronize()
        assert layer._arena(data["q_post"]).packed_kv.data_ptr() == ptr_before
        assert torch.equal(out2, out)
    finally:
        for k in env:
            os.environ.pop(k, None)


def test_decode_without_an_arena_is_recorded_and_replayed(dev):
    """Without SEMBLO_FULL_GRAPH_DECODE the generated tokens go through the decode kernels over the
    request's own index plus the layer's store of generated K/V, merged by log-sum-exp
    (model.py:579-616, 788-854 of the reference), and the step is recorded after two eager steps
    and replayed (decode_graph.py:125-249)."""
    from semblo_b200 import _lib
    from semblo_b200.config import SembloVllmConfig
    from semblo_b200.state import SembloRuntimeState
    dim, hq, hkv, sink, length, target, local, chunk, steps = 128, 8, 2, 64, 5120, 256, 128, 1024, 7
    # eight rows beyond the generated tokens: the out-of-sequence position below is still a valid row
    cpu = O.mixture_inputs(length=length + steps + 8, num_q_heads=hq, num_kv_heads=hkv, head_dim=dim, centres=24, seed=9)
    data = {k: v.to(dev) for k, v in cpu.items()}
    cfg = SembloVllmConfig(token_capacity=8192, target_tokens=target, flat_unit_tokens=32, index_dim=dim,
                           flat_min_clusters_log2=7, kmeans_sample_size=1024, query_chunk_size=chunk,
                           packed_decode_num_splits=4, decode_num_splits=2)
    state = SembloRuntimeState(max_model_len=8192)
    env = dict(SEMBLO_SINK_TOKENS=str(sink), SEMBLO_FA3_LOCAL=str(local), SEMBLO_FLAT_UNIT_TOKENS="32",
               SEMBLO_FA3_ALIGN="16")
    os.environ.update(env)
    os.environ.pop("SEMBLO_FULL_GRAPH_DECODE", None)
    try:
        layer = _make_layer(data, dev, hq=hq, hkv=hkv, dim=dim, cfg=cfg, state=state, name="model.layers.1.self_attn.attn")
        hidden = torch.zeros(length, 8, dtype=torch.bfloat16, device=dev)
        layer._sparse_layer_forward(torch.arange(length, device=dev), hidden)
        index = state.get(0)
        store = state.suffix_kv[0]
        assert store.shape[1] == (8192 + 255) // 256 - length // 256
        oidx = O.FlatIndex(codebooks=index.codebooks.cpu(), posting_positions=index.posting_positions.cpu(),
                           bucket_indptr=index.bucket_indptr.cpu(), bucket_sizes=index.bucket_sizes.cpu(),
                           inverse_positions=index.inverse_positions().cpu(), assign=index.orig_bucket.cpu().long(),
                           prompt_length=length, page_align=16, packed_kv=index.packed_kv.cpu())
        clusters = int(index.num_buckets)
        aref = O.make_arena(capacity=8192, num_clusters=clusters, num_kv_heads=hkv, head_dim=dim, page_align=16,
                            reserve=1024, kv_dtype=torch.bfloat16, desc_dtype=torch.bfloat16)
        O.arena_adopt(aref, oidx)
        step_pos = torch.zeros(1, dtype=torch.int64, device=dev)          # the engine's own position buffer
        for s in range(steps):
            pos = length + s
            step_pos.fill_(pos)
            o = layer._sparse_layer_forward(step_pos, hidden[:1]).view(hq, dim).clone()
            torch.cuda.synchronize()
            _lib.status_for(dev).raise_if_set()
            assert layer._decode_graph.captured == (s >= 2)
            ws = index._decode_ws
            sel = torch.zeros(hkv, clusters, dtype=torch.bool)
            for h in range(hkv):
                n = int(ws.rcount[h])
                ids = torch.searchsorted(oidx.bucket_indptr[h].contiguous(), ws.rstart[h, :n].cpu(), right=True) - 1
                sel[h, ids] = True
            wd, _, _ = O.decode_step(aref, q_post=cpu["q_post"][pos], q_pre=cpu["q_pre"][pos], pos=pos,
                                     k_post=cpu["k_post"][pos], v=cpu["v"][pos], temperature=0.1, beta=0.25,
                                     target_tokens=target, sink=sink, sm_scale=dim ** -0.5, sel=sel)
            d = (o.cpu().double() - wd).abs()
            assert float(d.max()) <= 2e-2 and float(d.mean()) <= 1e-3, (s, float(d.max()))
        assert layer._decode_graph.replays == steps - 3                   # steps 3.. reuse the recording of step 2
        assert int(index.max_position) == length + steps - 1
        # the store holds the generated K/V at their absolute positions
        rel = length - (length // 256) * 256
        assert torch.equal(store[0, 0, rel:rel + steps].cpu(), cpu["k_post"][length:length + steps])
        # a position out of sequence is refused on the host
        step_pos.fill_(length + steps + 5)
        state.expected_next_position = 0                                  # force the host to read the position
        with pytest.raises(ValueError):
            layer._sparse_layer_forward(step_pos, hidden[:1])
        # a new prompt drops the recording (its store and index are new memory)
        layer._sparse_layer_forward(torch.arange(length, device=dev), hidden)
        assert not layer._decode_graph.captured or state.suffix_kv[0] is store
    finally:
        for k in env:
            os.environ.pop(k, None)


def test_streamed_sessions_through_the_layer(dev):
    """The two prefill routes that bypass the operator (model.py:1271-1287, 1431-1529 and
    token_outer_prefill.py:127-212 of the reference): the layer-major session gives the bytes of
    the one-call prefill; the token-order session gives the bytes of the streamed store driven
    directly, leaves its index with the runtime state, and generated tokens follow."""
    from semblo_b200 import _lib
    from semblo_b200.config import SembloVllmConfig
    from semblo_b200.state import SembloRuntimeState
    from semblo_b200.token_outer import TokenOuterPrefillSession
    dim, hq, hkv, sink, length, target, chunk, steps = 128, 8, 2, 64, 6144, 256, 1024, 3
    cpu = O.mixture_inputs(length=length + steps, num_q_heads=hq, num_kv_heads=hkv, head_dim=dim, centres=24, seed=21)
    data = {k: v.to(dev) for k, v in cpu.items()}
    cfg = SembloVllmConfig(token_capacity=8192, target_tokens=target, flat_unit_tokens=32, index_dim=dim,
                           flat_min_clusters_log2=7, kmeans_sample_size=1024, query_chunk_size=chunk,
                           packed_decode_num_splits=4, decode_num_splits=2)
    env = dict(SEMBLO_SINK_TOKENS=str(sink), SEMBLO_FA3_LOCAL="0", SEMBLO_FLAT_UNIT_TOKENS="32", SEMBLO_FA3_ALIGN="16")
    os.environ.update(env)
    os.environ.pop("SEMBLO_FULL_GRAPH_DECODE", None)
    try:
        positions = torch.arange(length, device=dev)
        hidden = torch.zeros(length, 8, dtype=torch.bfloat16, device=dev)
        one = _make_layer(data, dev, hq=hq, hkv=hkv, dim=dim, cfg=cfg, state=SembloRuntimeState(max_model_len=8192),
                          name="model.layers.2.self_attn.attn")
        want = one._sparse_layer_forward(positions, hidden).clone()
        # ---- layer-major: keys for every slice, ingest, queries for every slice
        state = SembloRuntimeState(max_model_len=8192)
        layer = _make_layer(data, dev, hq=hq, hkv=hkv, dim=dim, cfg=cfg, state=state, name="model.layers.3.self_attn.attn")
        sess = layer.begin_streamed_prefill(positions)
        with pytest.raises(RuntimeError):
            sess.ingest()                                               # nothing staged yet
        for s0 in range(0, length, chunk):
            sess.keys(positions[s0:s0 + chunk], hidden[s0:s0 + chunk], s0, s0 + chunk)
        sess.ingest()
        got = torch.cat([sess.queries(positions[s0:s0 + chunk], positions[s0:s0 + chunk], hidden[s0:s0 + chunk], s0)
                         for s0 in range(0, length, chunk)])
        sess.finish()
        torch.cuda.synchronize()
        _lib.status_for(dev).raise_if_set()
        assert torch.equal(got, want)
        assert state.get(0).original_kv is None and 0 in state.suffix_kv
        # ---- token order: one pass, the index fitted on the prompt's head
        state2 = SembloRuntimeState(max_model_len=8192)
        layer2 = _make_layer(data, dev, hq=hq, hkv=hkv, dim=dim, cfg=cfg, state=state2, name="model.layers.4.self_attn.attn")
        sess2 = layer2.begin_token_outer_prefill(positions, chunk)
        direct = TokenOuterPrefillSession(total_tokens=length, chunk=chunk, num_q_heads=hq, num_kv_heads=hkv, head_dim=dim,
                                          target_tokens=target, temperature=0.1, beta=0.25, sm_scale=dim ** -0.5,
                                          flat_unit_tokens=32, flat_min_clusters_log2=7, page_align=16, device=dev,
                                          kmeans_sample_size=1024, codebook_seed=0, query_chunk_size=chunk)
        for s0 in range(0, length, chunk):
            sl = slice(s0, s0 + chunk)
            a = sess2.slice(hidden[sl], s0, s0 + chunk).view(chunk, hq, dim)
            b = direct.slice(data["q_post"][sl], data["q_pre"][sl], data["k_post"][sl], data["v"][sl], data["k_pre"][sl],
                             s0, s0 + chunk)
            assert torch.equal(a, b), s0
        sess2.finish()
        direct.finish()
        index = state2.get(0)
        assert index is sess2.inner.index and torch.equal(index.bucket_sizes, direct.index.bucket_sizes)
        assert int(index.bucket_sizes.sum()) == length * hkv
        # generated tokens over the streamed index
        oidx = O.FlatIndex(codebooks=index.codebooks.cpu(), posting_positions=index.posting_positions.cpu(),
                           bucket_indptr=index.bucket_indptr.cpu(), bucket_sizes=index.bucket_sizes.cpu(),
                           inverse_positions=index.inverse_positions().cpu(), assign=index.orig_bucket.cpu().long(),
                           prompt_length=length, page_align=16, packed_kv=index.packed_kv.cpu())
        clusters = int(index.num_buckets)
        aref = O.make_arena(capacity=16384, num_clusters=clusters, num_kv_heads=hkv, head_dim=dim, page_align=16,
                            reserve=1024, kv_dtype=torch.bfloat16, desc_dtype=torch.bfloat16)
        O.arena_adopt(aref, oidx)
        step_pos = torch.zeros(1, dtype=torch.int64, device=dev)
        for s in range(steps):
            pos = length + s
            step_pos.fill_(pos)
            o = layer2._sparse_layer_forward(step_pos, hidden[:1]).view(hq, dim).clone()
            torch.cuda.synchronize()
            _lib.status_for(dev).raise_if_set()
            ws = index._decode_ws
            sel = torch.zeros(hkv, clusters, dtype=torch.bool)
            for h in range(hkv):
                n = int(ws.rcount[h])
                ids = torch.searchsorted(oidx.bucket_indptr[h].contiguous(), ws.rstart[h, :n].cpu(), right=True) - 1
                sel[h, ids] = True
            wd, _, _ = O.decode_step(aref, q_post=cpu["q_post"][pos], q_pre=cpu["q_pre"][pos], pos=pos,
                                     k_post=cpu["k_post"][pos], v=cpu["v"][pos], temperature=0.1, beta=0.25,
                                     target_tokens=target, sink=sink, sm_scale=dim ** -0.5, sel=sel)
            d = (o.cpu().double() - wd).abs()
            assert float(d.max()) <= 2e-2 and float(d.mean()) <= 1e-3, (s, float(d.max()))
    finally:
        for k in env:
            os.environ.pop(k, None)


@pytest.mark.parametrize("arena_mode,index_dim", [(True, 128), (False, 128), (True, 96), (False, 64)])
def test_loaded_routing_map(dev, arena_mode, index_dim):
    """A linear routing map (routing_map.py:67-94, model.py:432-489 of the reference), square or into
    fewer dimensions: keys and queries go through it before they are normalised.  The layer with the
    map loaded gives the bytes of a layer with the identity map that is handed the projected pre-RoPE
    tensors (followed by zeros up to the head dimension, which change no norm and no dot product),
    prompt and decode."""
    from semblo_b200 import _lib
    from semblo_b200.config import SembloVllmConfig
    from semblo_b200.state import SembloRuntimeState
    dim, hq, hkv, sink, length, target, local, chunk, steps = 128, 8, 2, 64, 4096, 256, 128, 1024, 4
    cpu = O.mixture_inputs(length=length + steps, num_q_heads=hq, num_kv_heads=hkv, head_dim=dim, centres=24, seed=31)
    data = {k: v.to(dev) for k, v in cpu.items()}
    import dataclasses
    cfg = SembloVllmConfig(token_capacity=8192, target_tokens=target, flat_unit_tokens=32, index_dim=dim,
                           flat_min_clusters_log2=7, kmeans_sample_size=1024, query_chunk_size=chunk,
                           packed_decode_num_splits=4, decode_num_splits=2)
    cfg_map = dataclasses.replace(cfg, index_dim=index_dim)
    env = dict(SEMBLO_SINK_TOKENS=str(sink), SEMBLO_FA3_LOCAL=str(local), SEMBLO_FLAT_UNIT_TOKENS="32", SEMBLO_FA3_ALIGN="16")
    if arena_mode:
        env["SEMBLO_FULL_GRAPH_DECODE"] = "1"
    os.environ.update(env)
    if not arena_mode:
        os.environ.pop("SEMBLO_FULL_GRAPH_DECODE", None)
    try:
        mapped = _make_layer(data, dev, hq=hq, hkv=hkv, dim=dim, cfg=cfg_map, state=SembloRuntimeState(max_model_len=8192 + 512),
                             name=f"model.layers.{5 + arena_mode}.self_attn.attn")
        g = torch.Generator().manual_seed(3)
        w = torch.linalg.qr(torch.randn(hkv, dim, dim, generator=g))[0] + 0.05 * torch.randn(hkv, dim, dim, generator=g)
        mapped.semblo_key_router.load_weight(w[:, :index_dim])
        router = mapped._router(dev)
        assert not router.is_identity()
        assert tuple(router.project(data["k_pre"]).shape[-2:]) == (hkv, index_dim)
        projected = dict(data)
        projected["k_pre"] = router.widen(router.project(data["k_pre"])).contiguous()
        projected["q_pre"] = router.widen(router.project_queries(data["q_pre"])).contiguous()
        plain = _make_layer(projected, dev, hq=hq, hkv=hkv, dim=dim, cfg=cfg,
                            state=SembloRuntimeState(max_model_len=8192 + 512), name=f"model.layers.{7 + arena_mode}.self_attn.attn")
        assert plain._router(dev).is_identity()
        positions = torch.arange(length, device=dev)
        hidden = torch.zeros(length, 8, dtype=torch.bfloat16, device=dev)
        a = mapped._sparse_layer_forward(positions, hidden)
        b = plain._sparse_layer_forward(positions, hidden)
        torch.cuda.synchronize()
        _lib.status_for(dev).raise_if_set()
        assert torch.equal(a, b)
        assert torch.equal(mapped.runtime_state.get(0).bucket_sizes, plain.runtime_state.get(0).bucket_sizes)
        # and not the partition of the unprojected keys
        third = _make_layer(data, dev, hq=hq, hkv=hkv, dim=dim, cfg=cfg, state=SembloRuntimeState(max_model_len=8192 + 512),
                            name=f"model.layers.{9 + arena_mode}.self_attn.attn")
        third._sparse_layer_forward(positions, hidden)
        assert not torch.equal(third.runtime_state.get(0).bucket_sizes, plain.runtime_state.get(0).bucket_sizes)
        pa, pb = torch.zeros(1, dtype=torch.int64, device=dev), torch.zeros(1, dtype=torch.int64, device=dev)
        for s_ in range(steps):
            pa.fill_(length + s_)
            pb.fill_(length + s_)
            oa = mapped._sparse_layer_forward(pa, hidden[:1]).clone()
            ob = plain._sparse_layer_forward(pb, hidden[:1]).clone()
            torch.cuda.synchronize()
            _lib.status_for(dev).raise_if_set()
            assert torch.equal(oa, ob), s_
    finally:
        for k in env:
            os.environ.pop(k, None)


def test_loaded_routing_map_in_the_token_order_session_and_the_flush(dev):
    """The two other users of the key router (token_outer_prefill.py:258 and suffix_flush.py:193 of the
    reference): with a map loaded (here into fewer dimensions) the token-order session and the suffix flush
    give the bytes of a layer with the identity map that is handed the projected pre-RoPE tensors."""
    import dataclasses
    from semblo_b200 import _lib
    from semblo_b200 import suffix_flush as F
    from semblo_b200.config import SembloVllmConfig
    from semblo_b200.state import SembloRuntimeState
    dim, index_dim, hq, hkv, sink, length, target, chunk, steps, keep = 128, 80, 8, 2, 64, 6144, 256, 1024, 24, 8
    cpu = O.mixture_inputs(length=length + steps + 4, num_q_heads=hq, num_kv_heads=hkv, head_dim=dim, centres=24, seed=33)
    data = {k: v.to(dev) for k, v in cpu.items()}
    cfg = SembloVllmConfig(token_capacity=8192, target_tokens=target, flat_unit_tokens=32, index_dim=dim,
                           flat_min_clusters_log2=7, kmeans_sample_size=1024, query_chunk_size=chunk,
                           packed_decode_num_splits=4, decode_num_splits=2)
    cfg_map = dataclasses.replace(cfg, index_dim=index_dim)
    env = dict(SEMBLO_SINK_TOKENS=str(sink), SEMBLO_FA3_LOCAL="0", SEMBLO_FLAT_UNIT_TOKENS="32", SEMBLO_FA3_ALIGN="16",
               SEMBLO_FULL_GRAPH_DECODE="1", SEMBLO_SUFFIX_FLUSH_EVERY="16", SEMBLO_SUFFIX_KEEP_EXACT=str(keep))
    os.environ.update(env)
    try:
        g = torch.Generator().manual_seed(5)
        w = torch.linalg.qr(torch.randn(hkv, dim, dim, generator=g))[0][:, :index_dim]
        mapped = _make_layer(data, dev, hq=hq, hkv=hkv, dim=dim, cfg=cfg_map, state=SembloRuntimeState(max_model_len=8192 + 512),
                             name="model.layers.11.self_attn.attn")
        mapped.semblo_key_router.load_weight(w)
        router = mapped._router(dev)
        projected = dict(data)
        projected["k_pre"] = router.widen(router.project(data["k_pre"])).contiguous()
        projected["q_pre"] = router.widen(router.project_queries(data["q_pre"])).contiguous()
        plain = _make_layer(projected, dev, hq=hq, hkv=hkv, dim=dim, cfg=cfg, state=SembloRuntimeState(max_model_len=8192 + 512),
                            name="model.layers.12.self_attn.attn")
        positions = torch.arange(length, device=dev)
        hidden = torch.zeros(length, 8, dtype=torch.bfloat16, device=dev)
        sa, sb = mapped.begin_token_outer_prefill(positions, chunk), plain.begin_token_outer_prefill(positions, chunk)
        for s0 in range(0, length, chunk):
            a = sa.slice(hidden[s0:s0 + chunk], s0, s0 + chunk)
            b = sb.slice(hidden[s0:s0 + chunk], s0, s0 + chunk)
            assert torch.equal(a, b), s0
        sa.finish()
        sb.finish()
        torch.cuda.synchronize()
        _lib.status_for(dev).raise_if_set()
        assert torch.equal(mapped.runtime_state.get(0).bucket_sizes, plain.runtime_state.get(0).bucket_sizes)
        pa, pb = torch.zeros(1, dtype=torch.int64, device=dev), torch.zeros(1, dtype=torch.int64, device=dev)

        def step(s_):
            pa.fill_(length + s_)
            pb.fill_(length + s_)
            oa = mapped._sparse_layer_forward(pa, hidden[:1]).clone()
            ob = plain._sparse_layer_forward(pb, hidden[:1]).clone()
            torch.cuda.synchronize()
            _lib.status_for(dev).raise_if_set()
            assert torch.equal(oa, ob), s_

        for s_ in range(steps):
            step(s_)
        frm, to = F.flush_range(length, steps, length, keep, 16)
        arena_a, arena_b = mapped._arena(data["q_post"]), plain._arena(data["q_post"])
        # the stored pre-RoPE keys are the layer's inputs: raw under the map, projected in the plain layer
        wa = F.flush_layer(arena_a, mapped, frm, to)
        wb = F.flush_arena(arena_b, frm, to)
        torch.cuda.synchronize()
        assert wa == wb and int(arena_a.prompt_length_t.item()) == to
        assert torch.equal(arena_a.sizes, arena_b.sizes) and torch.equal(arena_a.indptr, arena_b.indptr)
        assert torch.equal(arena_a.posting[:, :wa], arena_b.posting[:, :wa])
        assert torch.equal(arena_a.packed_kv[:, :wa], arena_b.packed_kv[:, :wa])
        assert int(arena_a.sizes.sum()) == hkv * to
        # and not the assignment of the unprojected keys
        moved = F.nearest_cluster(F.routing_normalize(data["k_pre"][frm:to].contiguous()), arena_a.codebooks)
        routed = F.nearest_cluster(router(data["k_pre"][frm:to][None])[0], arena_a.codebooks)
        assert not torch.equal(moved, routed)
        for s_ in range(steps, steps + 4):
            step(s_)
    finally:
        for k in env:
            os.environ.pop(k, None)


def test_side_car_maps_load_into_the_layers(dev, tmp_path):
    """runtime_weights: a PCA map of the prompt's own keys is written as a side-car, verified and loaded into
    a model whose layer sits at ``model.layers.4.self_attn``; the layer then routes exactly as with the map
    loaded by hand.  With two ranks' worth of heads in the file, a rank's layer gets its block of heads."""
    from semblo_b200 import _lib
    from semblo_b200 import runtime_weights as RW
    from semblo_b200.config import SembloVllmConfig
    from semblo_b200.routing_map import pca_map
    from semblo_b200.state import SembloRuntimeState
    dim, index_dim, hq, hkv, sink, length, target, chunk = 128, 48, 8, 2, 64, 4096, 256, 1024
    cpu = O.mixture_inputs(length=length, num_q_heads=hq, num_kv_heads=hkv, head_dim=dim, centres=24, seed=37)
    data = {k: v.to(dev) for k, v in cpu.items()}
    cfg = SembloVllmConfig(token_capacity=8192, target_tokens=target, flat_unit_tokens=32, index_dim=index_dim,
                           flat_min_clusters_log2=7, kmeans_sample_size=1024, query_chunk_size=chunk,
                           packed_decode_num_splits=4, decode_num_splits=2)
    env = dict(SEMBLO_SINK_TOKENS=str(sink), SEMBLO_FA3_LOCAL="128", SEMBLO_FLAT_UNIT_TOKENS="32", SEMBLO_FA3_ALIGN="16")
    os.environ.update(env)
    os.environ.pop("SEMBLO_FULL_GRAPH_DECODE", None)
    try:
        w = pca_map(cpu["k_pre"], index_dim, rank=40)                     # [Hkv, 48, 128], rows 40.. zero
        other = torch.randn(hkv, index_dim, dim)                          # the heads of a second rank
        name = "layers.4.self_attn.semblo_key_router.weight"
        RW.write_runtime_weights(tmp_path / "one", {name: w}, {"semblo_index_dim": index_dim}, "test")
        RW.write_runtime_weights(tmp_path / "two", {name: torch.cat([other, w])}, {"semblo_index_dim": index_dim}, "test")

        def model_with_layer(tag):
            layer = _make_layer(data, dev, hq=hq, hkv=hkv, dim=dim, cfg=cfg, state=SembloRuntimeState(max_model_len=8192),
                                name=f"model.layers.{tag}.self_attn.attn")
            holders = torch.nn.ModuleList([torch.nn.Module() for _ in range(5)])
            holders[4].self_attn = layer
            model = torch.nn.Module()
            model.model = torch.nn.Module()
            model.model.layers = holders
            return model, layer

        by_hand = _make_layer(data, dev, hq=hq, hkv=hkv, dim=dim, cfg=cfg, state=SembloRuntimeState(max_model_len=8192),
                              name="model.layers.20.self_attn.attn")
        by_hand.semblo_key_router.load_weight(w)
        positions = torch.arange(length, device=dev)
        hidden = torch.zeros(length, 8, dtype=torch.bfloat16, device=dev)
        want = by_hand._sparse_layer_forward(positions, hidden).clone()
        for tag, directory, kw in ((21, "one", {}), (22, "two", dict(tp_rank=1, tp_size=2))):
            model, layer = model_with_layer(tag)
            assert layer._router(dev).is_identity() is False            # zeros [Hkv, 48, 128] until loaded
            written = RW.load_runtime_weights_into_module(model, tmp_path / directory, **kw)
            assert written == {"model.layers.4.self_attn.semblo_key_router.weight"}
            got = layer._sparse_layer_forward(positions, hidden)
            torch.cuda.synchronize()
            _lib.status_for(dev).raise_if_set()
            assert torch.equal(got, want), directory
            assert torch.equal(layer.runtime_state.get(0).bucket_sizes, by_hand.runtime_state.get(0).bucket_sizes)
    finally:
        for k in env:
            os.environ.pop(k, None)


def test_suffix_flusher_drives_the_layer_arena(dev):
    """suffix_flush.SuffixFlusher called before every engine step, as the reference's execute_model hook does
    (suffix_flush.py:211-283): the prompt step resets the count, the decode steps are counted, and when the
    exact suffix reaches keep + every its older part moves into the arena's clusters; decode goes on."""
    from semblo_b200 import _lib
    from semblo_b200 import suffix_flush as F
    from semblo_b200.config import SembloVllmConfig
    from semblo_b200.state import SembloRuntimeState
    dim, hq, hkv, sink, length, target, chunk, steps, keep, every = 128, 8, 2, 64, 4096, 256, 1024, 44, 8, 16
    cpu = O.mixture_inputs(length=length + steps, num_q_heads=hq, num_kv_heads=hkv, head_dim=dim, centres=24, seed=35)
    data = {k: v.to(dev) for k, v in cpu.items()}
    cfg = SembloVllmConfig(token_capacity=8192, target_tokens=target, flat_unit_tokens=32, index_dim=dim,
                           flat_min_clusters_log2=7, kmeans_sample_size=1024, query_chunk_size=chunk,
                           packed_decode_num_splits=4, decode_num_splits=2)
    env = dict(SEMBLO_SINK_TOKENS=str(sink), SEMBLO_FA3_LOCAL="128", SEMBLO_FLAT_UNIT_TOKENS="32", SEMBLO_FA3_ALIGN="16",
               SEMBLO_FULL_GRAPH_DECODE="1", SEMBLO_SUFFIX_FLUSH_EVERY=str(every), SEMBLO_SUFFIX_KEEP_EXACT=str(keep))
    os.environ.update(env)
    try:
        state = SembloRuntimeState(max_model_len=8192 + 512)
        layer = _make_layer(data, dev, hq=hq, hkv=hkv, dim=dim, cfg=cfg, state=state, name="model.layers.13.self_attn.attn")
        model = torch.nn.Module()
        model.layer = layer
        runner = SimpleNamespace(model=model)
        flusher = F.SuffixFlusher()
        hidden = torch.zeros(length, 8, dtype=torch.bfloat16, device=dev)
        flusher.before_step(runner, SimpleNamespace(total_num_scheduled_tokens=length, num_scheduled_tokens={"r": length}))
        layer._sparse_layer_forward(torch.arange(length, device=dev), hidden)
        arena = layer._arena(data["q_post"])
        one = SimpleNamespace(total_num_scheduled_tokens=1, num_scheduled_tokens={"r": 1})
        pos = torch.zeros(1, dtype=torch.int64, device=dev)
        want_len, flushes = length, 0
        for s_ in range(steps):
            due = F.flush_range(length, s_, want_len, keep, every)
            flusher.before_step(runner, one)
            if due is not None:
                want_len, flushes = due[1], flushes + 1
            assert flusher.state is state and flusher.flushes == flushes
            assert int(arena.prompt_length_t.item()) == want_len == int(arena.index.prompt_length)
            assert int(arena.sizes.sum()) == hkv * want_len
            pos.fill_(length + s_)
            out = layer._sparse_layer_forward(pos, hidden[:1])
            torch.cuda.synchronize()
            _lib.status_for(dev).raise_if_set()
            assert bool(torch.isfinite(out.float()).all())
        assert flushes == 2 and want_len == length + 32
    finally:
        for k in env:
            os.environ.pop(k, None)


def test_operator_refuses_what_it_does_not_serve(dev):
    from semblo_b200.attention_op import registered_layer
    from semblo_b200.config import SembloVllmConfig
    with pytest.raises(RuntimeError):
        registered_layer("no.such.layer")
    with pytest.raises(ValueError):
        SembloVllmConfig(token_capacity=1024, target_tokens=64, flat_unit_tokens=32, index_dim=128,
                         own_prompt_cache=False).validate()
    with pytest.raises(ValueError):
        SembloVllmConfig(token_capacity=1024, target_tokens=64, flat_unit_tokens=0, index_dim=128).validate()
