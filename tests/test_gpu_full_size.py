"""The benchmark configurations' full sizes through properties that do not depend on the size: sampled
queries of the 131072-token prefill against the oracle's per-query gather on the kernel's own
selection, determinism of a whole step, and the store invariants of the 262144-token
token-order streamed prefill (every key sits where the inverse map says, in position order
inside its cluster)."""
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


def _env(cfg):
    import bench
    bench.set_env(cfg)


def _clear_env():
    for k in ("SEMBLO_FLAT_UNIT_TOKENS", "SEMBLO_FA3_ALIGN", "SEMBLO_SINK_TOKENS", "SEMBLO_FA3_LOCAL"):
        os.environ.pop(k, None)


def test_prefill_131072_sampled_queries_and_determinism(dev):
    import bench
    from semblo_b200 import _lib
    from semblo_b200.fused_prefill import CausalSnapshot, fused_chunk_attention
    from semblo_b200.flat_index import routing_normalize
    from semblo_b200.state import ProductPostingIndex
    from semblo_b200.trivial_router import trivial_router_vectors
    cfg = dict(bench.PREFILL)
    _env(cfg)
    try:
        L, hq, hkv, dim, chunk = cfg["length"], cfg["hq"], cfg["hkv"], cfg["dim"], cfg["chunk"]
        x = bench.mixture_inputs_device(cfg, 4242, dev)
        step = bench.PrefillStep(cfg, dev)
        step.prepare()
        out_a = torch.empty(L, hq, dim, dtype=torch.bfloat16, device=dev)
        out_b = torch.empty_like(out_a)
        step.run(x, out_a)
        index = step.run(x, out_b)
        torch.cuda.synchronize()
        _lib.status_for(dev).raise_if_set()
        assert bool(torch.isfinite(out_a.float()).all())
        assert torch.equal(out_a, out_b), "two runs of the same step differ"
        # one sparse chunk again, keeping its selection; then sampled queries against the oracle
        cs = 12 * chunk
        ce = cs + chunk - 1
        snap = CausalSnapshot(index)
        qv = trivial_router_vectors(x["q_pre"][cs:ce + 1])
        state = SimpleNamespace(vectors=qv.view(1, chunk, hq, 1, dim))
        out_c = torch.empty(chunk, hq, dim, dtype=torch.bfloat16, device=dev)
        fused_chunk_attention(x["q_post"][cs:ce + 1], state, index, step.positions32[cs:ce + 1], snap, cs, ce,
                              temperature=cfg["temperature"], beta=cfg["beta"], target_tokens=cfg["target"],
                              sm_scale=dim ** -0.5, out=out_c)
        torch.cuda.synchronize()
        assert torch.equal(out_c, out_a[cs:ce + 1])
        ws = cs - cfg["local"]
        sizes = snap.advance(ws - 1).cpu()
        g = torch.Generator().manual_seed(3)
        pick = torch.randperm(chunk, generator=g)[:24].sort().values
        sel = O.unpack_bits(snap.qmask[:chunk].cpu()[pick])
        # the page table maps logical packed rows to pool rows: undo it for the oracle's view
        pt = step.page_table.long().cpu()
        width = int(index.posting_positions.shape[1])
        rows = torch.arange(width)
        phys = pt[rows // 16] * 16 + rows % 16
        packed = index.packed_kv.cpu()[:, phys]
        oidx = O.FlatIndex(codebooks=index.codebooks.cpu(), posting_positions=index.posting_positions.cpu(),
                           bucket_indptr=index.bucket_indptr.cpu(), bucket_sizes=index.bucket_sizes.cpu(),
                           inverse_positions=index.inverse_positions().cpu(), assign=index.orig_bucket.cpu().long(),
                           prompt_length=L, page_align=16, packed_kv=packed)
        qpos = (cs + pick)
        want = O.sparse_chunk_attention_gather(x["q_post"][cs:ce + 1].cpu()[pick], oidx, sel, sizes, qpos,
                                               x["k_post"][ws:ce + 1].cpu(), x["v"][ws:ce + 1].cpu(), ws,
                                               dim ** -0.5, dtype=torch.float32)
        diff = (out_c.cpu()[pick].float() - want).abs()
        assert float(diff.max()) <= 2e-2, f"sampled queries: max-abs {float(diff.max()):.4g}"
        assert float(diff.mean()) <= 1e-3
        # budget property of the selection: every sampled query reaches the budget without the sink
        held = sel.clone()
        held[..., 0] = False
        tokens = (held * sizes[None]).sum(-1)
        assert bool((tokens >= cfg["target"] - cfg["sink"]).all())
    finally:
        _clear_env()


def test_token_order_prefill_262144_store_invariants(dev):
    import bench
    from semblo_b200 import _lib
    from semblo_b200.token_outer import TokenOuterPrefillSession
    cfg = dict(bench.PREFILL)
    cfg.update(length=262144, local=0)
    _env(cfg)
    try:
        L, hq, hkv, dim, chunk = cfg["length"], cfg["hq"], cfg["hkv"], cfg["dim"], cfg["chunk"]
        x = bench.mixture_inputs_device(cfg, 99, dev)
        sess = TokenOuterPrefillSession(total_tokens=L, chunk=chunk, num_q_heads=hq, num_kv_heads=hkv, head_dim=dim,
                                        target_tokens=cfg["target"], temperature=cfg["temperature"], beta=cfg["beta"],
                                        sm_scale=dim ** -0.5, flat_unit_tokens=cfg["unit"],
                                        flat_min_clusters_log2=cfg["min_log2"], page_align=16, device=dev)
        assert sess.fit_at == 24576                       # min(65536, 4 * 4096) -> the first slice boundary past it
        out = torch.empty(chunk, hq, dim, dtype=torch.bfloat16, device=dev)
        for start in range(0, L, chunk):
            sl = slice(start, start + chunk)
            sess.slice(x["q_post"][sl], x["q_pre"][sl], x["k_post"][sl], x["v"][sl], x["k_pre"][sl], start,
                       start + chunk, out=out)
        torch.cuda.synchronize()
        _lib.status_for(dev).raise_if_set()
        assert bool(torch.isfinite(out.float()).all())
        ix = sess.index
        assert int(ix.num_buckets) == 4096                # the count of the whole prompt
        sizes, indptr = ix.bucket_sizes.long(), ix.bucket_indptr.long()
        assert bool((sizes.sum(1) == L).all())
        assert bool((indptr[:, :-1] + sizes <= indptr[:, 1:]).all()), "a cluster outgrew its run"
        inv, assign = ix._inverse_positions.long(), ix.orig_bucket.long()
        lo = indptr.gather(1, assign)
        assert bool(((inv >= lo) & (inv < lo + sizes.gather(1, assign))).all())
        pos = torch.arange(L, device=dev)
        for h in range(hkv):
            assert torch.equal(ix.posting_positions[h][inv[h]].long(), pos)
            assert torch.equal(ix.packed_kv[0, :, h][inv[h]], x["k_post"][:, h])
            assert torch.equal(ix.packed_kv[1, :, h][inv[h]], x["v"][:, h])
            # rows of a cluster ascend with positions: sort by (cluster, position) and by (cluster, row) agree
            a = torch.argsort(assign[h] * (2 * L) + pos)
            b = torch.argsort(assign[h] * (4 * L) + inv[h])
            assert torch.equal(a, b)
    finally:
        _clear_env()
