"""Parity of the CUDA path against the CPU oracle on the same seeded inputs.

Every call goes through the C ABI (libsemblo_b200.so via ctypes).  Integer stages are
compared bit for bit; float-dependent integer results (assignment, selection) must be
identical wherever the oracle's own margin is not tiny; attention outputs are held to
2e-2 max-abs / 1e-3 mean-abs in bf16 (the reference's tolerance for this path)."""
from __future__ import annotations

import os

import pytest
import torch

from oracle import semblo_oracle as O

pytestmark = pytest.mark.gpu

MAX_ABS = 2e-2
MEAN_ABS = 1e-3


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from semblo_b200 import _lib
    _lib.lib()          # raises if the extension is missing: no silent fallback
    return torch.device("cuda:0")


def _status_ok(dev):
    from semblo_b200 import _lib
    _lib.status_for(dev).raise_if_set()


def _close_attention(got: torch.Tensor, want: torch.Tensor, what: str):
    diff = (got.double().cpu() - want.double().cpu()).abs()
    assert float(diff.max()) <= MAX_ABS, f"{what}: max-abs {float(diff.max()):.4g}"
    assert float(diff.mean()) <= MEAN_ABS, f"{what}: mean-abs {float(diff.mean()):.4g}"


def _unit(n, d, seed, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return torch.nn.functional.normalize(torch.randn(n, d, generator=g), dim=-1).to(dtype)


# ---------------------------------------------------------------------- routing space
@pytest.mark.parametrize("dim", [64, 128, 256])
def test_routing_normalize_and_query_vectors(dev, dim):
    from semblo_b200 import flat_index, trivial_router
    g = torch.Generator().manual_seed(dim)
    x = (torch.randn(777, 4, dim, generator=g) * 3).to(torch.bfloat16)
    got = flat_index.routing_normalize(x.to(dev)).cpu()
    want = O.routing_normalize(x)
    bad = (got.float() - want.float()).abs() > 0
    assert float(bad.float().mean()) < 2e-3           # differences are single bf16 roundings
    assert float((got.float() - want.float()).abs().max()) <= 2 ** -7 * 0.26
    qv = trivial_router.trivial_router_vectors(x.to(dev)).cpu()
    want_q = O.trivial_router_vectors(x)
    assert float(((qv.float() - want_q.float()).abs() > 0).float().mean()) < 4e-3
    assert float((qv.float() - want_q.float()).abs().max()) <= 2 ** -7 * 0.26
    _, f32, b16 = flat_index._normalize_space(want.to(dev)[:, 0].contiguous())
    torch.testing.assert_close(f32.cpu(), O.routing_space(want[:, 0]), atol=2e-7, rtol=0)
    assert torch.equal(b16.cpu().float(), O.routing_space(want[:, 0]).to(torch.bfloat16).float()) or \
        float(((b16.cpu().float() - O.routing_space(want[:, 0]).to(torch.bfloat16).float()).abs() > 0).float().mean()) < 1e-3


# ---------------------------------------------------------------------- assignment
@pytest.mark.parametrize("dim,n,clusters", [(256, 3000, 2048), (128, 1111, 127), (64, 500, 40), (256, 129, 128)])
def test_assign_argmax_matches_oracle_outside_rounding_boundaries(dev, dim, n, clusters):
    from semblo_b200 import flat_index
    x = _unit(n, dim, 1)
    # clustered data: many bf16 ties, as in a real prompt
    c = torch.nn.functional.normalize(x[torch.randperm(n, generator=torch.Generator().manual_seed(2))[:clusters]]
                                      + 0.05 * torch.randn(clusters, dim, generator=torch.Generator().manual_seed(3)), dim=-1)
    want, sim32 = O.argmax_sim(x, c, return_sim=True)
    got = flat_index.assign_flat_buckets(x.to(torch.bfloat16).to(dev), c.to(dev)).cpu().long()
    _status_ok(dev)
    differ = got != want
    margin = O.assign_margin(sim32)
    # a differing row must sit on a bf16 rounding boundary of one of its top columns
    assert bool((margin[differ] < 3e-6).all()), f"{int(differ.sum())} rows differ, worst margin {float(margin[differ].max()) if differ.any() else 0}"
    assert float(differ.float().mean()) < 2e-3
    # and the chosen centroid must still tie with the oracle's after rounding
    simb = sim32.to(torch.bfloat16).float()
    rows = torch.nonzero(differ).flatten()
    if rows.numel():
        step = simb[rows, want[rows]].abs() * 2 ** -7
        assert bool(((simb[rows, want[rows]] - simb[rows, got[rows]]).abs() <= step + 1e-12).all())


def test_kmeans_update_with_empty_cluster_restart(dev):
    from semblo_b200._lib import lib, ptr, check, stream_ptr
    n, dim, clusters = 5000, 128, 96
    sample = _unit(n, dim, 5)
    g = torch.Generator().manual_seed(6)
    assign = torch.randint(0, clusters - 3, (n,), generator=g)      # clusters 93..95 stay empty
    repl = torch.randperm(n, generator=g)
    want, _ = O.kmeans_update(sample, assign, clusters, repl)
    s_d, a_d = sample.to(dev), assign.to(torch.int32).to(dev)
    repl_d = repl.to(dev)
    counts = torch.empty(clusters, dtype=torch.int32, device=dev)
    ip = torch.empty(clusters + 1, dtype=torch.int32, device=dev)
    er = torch.empty(clusters, dtype=torch.int32, device=dev)
    ne = torch.empty(1, dtype=torch.int32, device=dev)
    check(lib().semblo_cluster_counts(ptr(a_d), n, n, 1, clusters, 1, ptr(counts), ptr(ip), None, ptr(er), ptr(ne), stream_ptr()))
    assert int(ne.item()) == 3
    assert torch.equal(counts.cpu().long(), torch.bincount(assign, minlength=clusters))
    ws_bytes = int(lib().semblo_layout_workspace_bytes(n, 1))
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    cf = torch.empty(clusters, dim, dtype=torch.float32, device=dev)
    cb = torch.empty(clusters, dim, dtype=torch.bfloat16, device=dev)
    check(lib().semblo_kmeans_update(ptr(s_d), ptr(a_d), n, clusters, dim, ptr(ip), ptr(er), ptr(repl_d),
                                     ptr(cf), ptr(cb), ptr(ws), ws_bytes, stream_ptr()))
    torch.testing.assert_close(cf.cpu(), want, atol=2e-6, rtol=0)
    assert torch.equal(cb.cpu().float(), cf.cpu().to(torch.bfloat16).float())
    # deterministic: a second run gives the same bytes
    cf2 = torch.empty_like(cf)
    check(lib().semblo_kmeans_update(ptr(s_d), ptr(a_d), n, clusters, dim, ptr(ip), ptr(er), ptr(repl_d),
                                     ptr(cf2), ptr(cb), ptr(ws), ws_bytes, stream_ptr()))
    assert torch.equal(cf, cf2)


# ---------------------------------------------------------------------- layout / pack / snapshot
@pytest.mark.parametrize("length,heads,clusters,align", [(5000, 3, 64, 16), (70000, 2, 2048, 16), (4097, 1, 512, 1),
                                                         (300, 2, 256, 16)])
def test_layout_is_bit_identical(dev, length, heads, clusters, align):
    from semblo_b200._lib import lib, ptr, check, stream_ptr
    g = torch.Generator().manual_seed(length)
    # skewed sizes with empty clusters
    w = torch.rand(clusters, generator=g) ** 3
    w[::7] = 0
    assign = torch.multinomial(w, heads * length, replacement=True, generator=g).view(heads, length)
    cap = length + clusters * (align - 1 if align > 1 else 0)
    cap += (-cap) % 256
    a_d = assign.to(torch.int32).to(dev)
    posting = torch.empty(heads, cap, dtype=torch.int32, device=dev)
    indptr = torch.empty(heads, clusters + 1, dtype=torch.int32, device=dev)
    sizes = torch.empty(heads, clusters, dtype=torch.int32, device=dev)
    inverse = torch.empty(heads, length, dtype=torch.int32, device=dev)
    ws_bytes = int(lib().semblo_layout_workspace_bytes(length, heads)) + heads * (clusters + 1) * 4
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    check(lib().semblo_build_layout(ptr(a_d), length, heads, clusters, align, ptr(posting), cap, ptr(indptr),
                                    ptr(sizes), ptr(inverse), ptr(ws), ws_bytes, stream_ptr()))
    for h in range(heads):
        order, ip, counts, inv = O.layout_from_assign(assign[h], clusters, align)
        assert torch.equal(sizes[h].cpu(), counts)
        assert torch.equal(indptr[h].cpu(), ip)
        assert torch.equal(posting[h, :order.numel()].cpu(), order)
        assert bool((posting[h, order.numel():].cpu() == order[0]).all())
        assert torch.equal(inverse[h].cpu(), inv)


def test_pack_and_snapshot_are_bit_identical(dev):
    from semblo_b200.state import ProductPostingIndex
    from semblo_b200.fused_prefill import CausalSnapshot
    length, heads, dim, clusters = 2000, 2, 128, 64
    keys = O.mixture_inputs(length=length, num_q_heads=heads, num_kv_heads=heads, head_dim=dim, centres=20,
                            seed=11)["k_pre"]
    product = O.routing_normalize(keys)
    g = torch.Generator().manual_seed(3)
    cents = [_unit(clusters, dim, 40 + h) for h in range(heads)]
    os.environ["SEMBLO_FLAT_UNIT_TOKENS"] = "32"
    try:
        index = ProductPostingIndex.build(product.to(dev), torch.arange(length, device=dev), flat_unit_tokens=32,
                                          flat_min_clusters_log2=6, page_align=16,
                                          centroids=[c.to(dev) for c in cents])
    finally:
        os.environ.pop("SEMBLO_FLAT_UNIT_TOKENS", None)
    assert index.num_buckets == clusters
    # oracle layout from the kernel's own assignment: the integer stages must agree exactly
    assign = index.orig_bucket.cpu().long()
    ref = O.build_flat(product, unit_tokens=32, min_clusters_log2=6, page_align=16, centroids=cents)
    assert float((assign != ref.assign).float().mean()) < 2e-3
    for h in range(heads):
        order, ip, counts, inv = O.layout_from_assign(assign[h], clusters, 16)
        assert torch.equal(index.bucket_sizes[h].cpu(), counts)
        assert torch.equal(index.bucket_indptr[h].cpu(), ip)
        assert torch.equal(index.posting_positions[h, :order.numel()].cpu(), order)
        assert torch.equal(index.inverse_positions()[h].cpu(), inv)
    assert float((index.codebooks.cpu().float() - ref.codebooks.float()).abs().max()) <= 2 ** -8
    k = torch.randn(length, heads, dim, generator=g).to(torch.bfloat16)
    v = torch.randn(length, heads, dim, generator=g).to(torch.bfloat16)
    packed = index.pack_prompt_kv(k.to(dev), v.to(dev)).cpu()
    fake = O.FlatIndex(codebooks=None, posting_positions=index.posting_positions.cpu(), bucket_indptr=None,
                       bucket_sizes=None, inverse_positions=None, assign=None, prompt_length=length, page_align=16)
    assert torch.equal(packed.float(), O.pack_prompt_kv(fake, k, v).float())
    # paged pool: the same rows behind a random page permutation
    n_pages = packed.shape[1] // 16
    table = torch.randperm(n_pages, generator=g).to(torch.int32)
    paged = index.pack_prompt_kv(k.to(dev), v.to(dev), page_table=table.to(dev)).cpu()
    view = paged.view(2, n_pages, 16, heads, dim)[:, table.long()].reshape(packed.shape)
    assert torch.equal(view.float(), packed.float())
    snap = CausalSnapshot(index)
    for p in (0, 17, 999, 1000, 1999):
        got = snap.advance(p).cpu()
        want = torch.stack([torch.bincount(assign[h, :p + 1], minlength=clusters) for h in range(heads)]).int()
        assert torch.equal(got, want)


def test_centred_build(dev):
    """SEMBLO_ROUTING_CENTER=1: the prompt's mean key is taken out per head before the space is
    normalised (state.py:649-670 of the reference); given centroids are refused with it."""
    from semblo_b200.state import ProductPostingIndex
    length, heads, dim = 4096, 2, 128
    g = torch.Generator().manual_seed(5)
    keys = O.mixture_inputs(length=length, num_q_heads=heads, num_kv_heads=heads, head_dim=dim, centres=20,
                            seed=13)["k_pre"]
    keys = (keys.float() + 6.0 * torch.randn(1, heads, dim, generator=g)).to(torch.bfloat16)   # one dominant direction
    product = O.routing_normalize(keys)
    env = dict(SEMBLO_FLAT_UNIT_TOKENS="32", SEMBLO_ROUTING_CENTER="1")
    os.environ.update(env)
    try:
        kw = dict(flat_unit_tokens=32, flat_min_clusters_log2=6, page_align=16, kmeans_sample_size=1024, codebook_seed=3)
        index = ProductPostingIndex.build(product.to(dev), torch.arange(length, device=dev), **kw)
        with pytest.raises(RuntimeError):
            ProductPostingIndex.build(product.to(dev), torch.arange(length, device=dev),
                                      centroids=[_unit(128, dim, 1).to(dev)] * heads, **kw)
        os.environ.pop("SEMBLO_ROUTING_CENTER")
        plain = ProductPostingIndex.build(product.to(dev), torch.arange(length, device=dev), **kw)
    finally:
        for k in env:
            os.environ.pop(k, None)
    _status_ok(dev)
    clusters = int(index.num_buckets)
    assert int((plain.bucket_sizes > 0).sum()) < int((index.bucket_sizes > 0).sum())
    # the oracle's assignment of the centred keys to the kernel's own centroids
    cents = [torch.cat([index.codebooks[h, 0], index.codebooks[h, 1]], dim=-1).cpu().float() for h in range(heads)]
    ref = O.build_flat(product, unit_tokens=32, min_clusters_log2=6, page_align=16, centroids=cents, center=True)
    assign = index.orig_bucket.cpu().long()
    assert float((assign != ref.assign).float().mean()) < 1e-2
    for h in range(heads):
        order, ip, counts, inv = O.layout_from_assign(assign[h], clusters, 16)
        assert torch.equal(index.bucket_sizes[h].cpu(), counts)
        assert torch.equal(index.posting_positions[h, :order.numel()].cpu(), order)


# ---------------------------------------------------------------------- scoring + selection
def _small_problem(length, hq, hkv, dim, centres, seed, unit, min_log2, sink):
    data = O.mixture_inputs(length=length, num_q_heads=hq, num_kv_heads=hkv, head_dim=dim, centres=centres, seed=seed)
    product = O.routing_normalize(data["k_pre"])
    index = O.build_flat(product, unit_tokens=unit, min_clusters_log2=min_log2, kmeans_sample_size=1024,
                         fit_iters=4, seed=0, sink=sink, page_align=16)
    O.pack_prompt_kv(index, data["k_post"], data["v"])
    return data, index


def _gpu_index(index, dev):
    from semblo_b200.state import ProductPostingIndex
    gi = ProductPostingIndex(codebooks=index.codebooks.to(dev), posting_positions=index.posting_positions.to(dev),
                             bucket_indptr=index.bucket_indptr.to(dev), bucket_sizes=index.bucket_sizes.to(dev),
                             prompt_length=index.prompt_length, max_position=index.prompt_length - 1,
                             page_align=16, flat_clusters=int(index.bucket_sizes.shape[1]),
                             _inverse_positions=index.inverse_positions.to(dev),
                             orig_bucket=index.assign.to(torch.int32).to(dev))
    gi.packed_kv = index.packed_kv.to(dev)
    return gi


@pytest.mark.parametrize("dim,hq,hkv,sink", [(256, 8, 2, 64), (128, 8, 2, 0), (128, 16, 2, 0)])
def test_scores_and_selection(dev, dim, hq, hkv, sink):
    from semblo_b200.fused_prefill import theta_select_bitmask_flat
    length, target = 6144, 512
    data, index = _small_problem(length, hq, hkv, dim, 24, 21 + dim, 32, 7, sink)
    clusters = index.bucket_sizes.shape[1]
    sizes = O.causal_sizes_at(index, 4000)
    qs = slice(4100, 4100 + 333)
    vectors = O.trivial_router_vectors(data["q_pre"][qs])
    sel_sizes, sel_target = (O.hold_out_sink(sizes, target, sink) if sink else (sizes, target))
    score_ref = O.penalized_scores(O.mixture_prob(vectors, index.codebooks, 0.1, torch.float64), sel_sizes[None], 0.25)
    sel_ref, margin = O.select_clusters(vectors, index.codebooks, sizes, temperature=0.1, beta=0.25,
                                        target_tokens=target, sink=sink, return_margin=True)
    counts = torch.empty(333, hkv, dtype=torch.int32, device=dev)
    tokens = torch.empty(333, hkv, dtype=torch.int32, device=dev)
    qmask, score = theta_select_bitmask_flat(vectors.to(dev), index.codebooks.to(dev), sel_sizes.to(dev),
                                             temperature=0.1, beta=0.25, target_tokens=sel_target,
                                             force_sink=bool(sink), counts=counts, tokens=tokens,
                                             top1=(top1 := torch.empty(hkv, 333, dtype=torch.int32, device=dev)))
    _status_ok(dev)
    assert torch.equal(top1.cpu().long().t(), score.cpu().argmax(dim=-1))
    live = (sel_sizes > 0)[None].expand(333, -1, -1)
    err = (score.cpu().double() - score_ref)[live].abs()
    assert float(err.max()) < 5e-5, float(err.max())
    assert bool((score.cpu()[~live] == O.NEG_BIG).all())
    sel = O.unpack_bits(qmask.cpu())
    assert sel.shape[-1] == clusters
    differ = (sel != sel_ref).any(dim=-1)
    assert bool((margin[differ] < 1e-4).all()), (int(differ.sum()), float(margin[differ].max()) if differ.any() else 0)
    assert float(differ.float().mean()) < 0.02
    # the selection the kernel reports is exactly the rule applied to its own scores
    sel_own = O.theta_select(score.cpu(), sel_sizes[None], sel_target, 16)
    if sink:
        sel_own = sel_own.clone()
        sel_own[..., 0] = True
    assert torch.equal(sel, sel_own)
    held = sel_own.clone()
    if sink:
        held[..., 0] = False
    assert torch.equal(counts.cpu(), held.sum(-1).int())
    assert torch.equal(tokens.cpu(), (held * sel_sizes[None]).sum(-1).int())


# ---------------------------------------------------------------------- prefill attention
@pytest.mark.parametrize("dim,hq,hkv", [(256, 8, 2), (128, 4, 1), (128, 16, 2), (256, 16, 1)])
def test_dense_causal_attention(dev, dim, hq, hkv):
    from semblo_b200.fused_prefill import window_attention
    length = 700
    data = O.mixture_inputs(length=length, num_q_heads=hq, num_kv_heads=hkv, head_dim=dim, centres=8, seed=3)
    sm_scale = dim ** -0.5
    qpos = torch.arange(length)
    want, lse_want = O.dense_causal_attention(data["q_post"], data["k_post"], data["v"], qpos, sm_scale)
    lse = torch.empty(length, hq, dtype=torch.float32, device=dev)
    att = torch.zeros(1, dtype=torch.int64, device=dev)
    got = window_attention(data["q_post"].to(dev), qpos.int().to(dev), ordered_k=data["k_post"].to(dev),
                                   ordered_v=data["v"].to(dev), sm_scale=sm_scale, lse=lse, attended=att)
    _status_ok(dev)
    _close_attention(got, want, "dense prefix")
    torch.testing.assert_close(lse.cpu().double(), lse_want, atol=2e-3, rtol=0)
    assert int(att.item()) == hkv * length * (length + 1) // 2
    # a later chunk over a window: positions [ws, p]
    qs = slice(400, 700)
    want_w, _ = O.dense_causal_attention(data["q_post"][qs], data["k_post"][200:], data["v"][200:], qpos[qs],
                                         sm_scale, k_start=200)
    got_w = window_attention(data["q_post"][qs].contiguous().to(dev), qpos[qs].int().to(dev),
                                     ordered_k=data["k_post"][200:].contiguous().to(dev),
                                     ordered_v=data["v"][200:].contiguous().to(dev), ordered_pos0=200,
                                     local_start=200, sm_scale=sm_scale)
    _close_attention(got_w, want_w, "window")


@pytest.mark.parametrize("dim,hq,hkv,sink,paged", [(256, 8, 2, 64, True), (128, 8, 2, 0, False),
                                                   (128, 16, 2, 0, True), (256, 16, 1, 64, False)])
def test_sparse_chunk_attention_matches_oracle_on_the_same_selection(dev, dim, hq, hkv, sink, paged):
    from semblo_b200.fused_prefill import window_attention
    length, target, local = 6144, 512, 128
    data, index = _small_problem(length, hq, hkv, dim, 24, 77 + dim, 32, 7, sink)
    cs, ce = 4096, 4096 + 499
    ws = cs - local
    sizes = O.causal_sizes_at(index, ws - 1)
    qpos = torch.arange(cs, ce + 1)
    vectors = O.trivial_router_vectors(data["q_pre"][cs:ce + 1])
    sel = O.select_clusters(vectors, index.codebooks, sizes, temperature=0.1, beta=0.25, target_tokens=target, sink=sink)
    # a few queries with nothing selected on head 0 (the sparse part alone must then give zeros),
    # and one that selects a single cluster
    sel[3, 0] = False
    sel[250, 0] = False
    sel[499, 0] = False
    sel[100, 0] = False
    sel[100, 0, int(sizes[0].argmax())] = True
    sm_scale = dim ** -0.5
    want, natt = O.sparse_chunk_attention(data["q_post"][cs:ce + 1], index, sel, sizes, qpos,
                                          data["k_post"][ws:ce + 1], data["v"][ws:ce + 1], ws, sm_scale)
    packed = index.packed_kv.to(dev)
    table = None
    if paged:
        n_pages = packed.shape[1] // 16
        perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(5))
        pool = torch.empty_like(packed).view(2, n_pages, 16, hkv, dim)
        pool[:, perm] = packed.view(2, n_pages, 16, hkv, dim)
        packed = pool.view(2, n_pages * 16, hkv, dim).contiguous()
        table = perm.to(torch.int32).to(dev)
    order = torch.stack([torch.randperm(500, generator=torch.Generator().manual_seed(h)) for h in range(hkv)]).int()
    # the two-launch form: exact window first, then the row-gather sparse kernel merged into it
    from semblo_b200.fused_prefill import sparse_gather_attention
    for q_order in (None, order.to(dev)):
        lse = torch.empty(500, hq, dtype=torch.float32, device=dev)
        out2 = torch.empty(500, hq, dim, dtype=torch.bfloat16, device=dev)
        att2 = torch.zeros(2, dtype=torch.int64, device=dev)
        window_attention(data["q_post"][cs:ce + 1].contiguous().to(dev), qpos.int().to(dev),
                         ordered_k=data["k_post"][ws:ce + 1].contiguous().to(dev),
                         ordered_v=data["v"][ws:ce + 1].contiguous().to(dev), ordered_pos0=ws, local_start=ws,
                         sm_scale=sm_scale, out=out2, lse=lse, attended=att2)
        sparse_gather_attention(data["q_post"][cs:ce + 1].contiguous().to(dev), packed_kv=packed,
                                qmask=O.pack_bits(sel).to(dev), causal_sizes=sizes.to(dev),
                                indptr=index.bucket_indptr.to(dev), sm_scale=sm_scale, out=out2, lse=lse, merge=True,
                                page_table=table, q_order=q_order, attended=att2)
        _status_ok(dev)
        _close_attention(out2, want, "window + gathered clusters")
        assert int(att2[0].item()) == int(natt.sum())
        assert int(att2[1].item()) >= int(natt.max()) - 500 - local
    # the sparse part alone
    empty_k = data["k_post"][ws:ws].contiguous()
    want_s, _ = O.sparse_chunk_attention(data["q_post"][cs:ce + 1], index, sel, sizes, qpos, empty_k,
                                         data["v"][ws:ws].contiguous(), ws, sm_scale)
    out3 = torch.empty(500, hq, dim, dtype=torch.bfloat16, device=dev)
    sparse_gather_attention(data["q_post"][cs:ce + 1].contiguous().to(dev), packed_kv=packed,
                            qmask=O.pack_bits(sel).to(dev), causal_sizes=sizes.to(dev),
                            indptr=index.bucket_indptr.to(dev), sm_scale=sm_scale, out=out3, lse=None, merge=False,
                            page_table=table)
    _status_ok(dev)
    _close_attention(out3, want_s, "gathered clusters alone")
    group = hq // hkv
    for qi in (3, 250, 499):
        assert float(out3[qi, :group].float().abs().max()) == 0.0, "a query with an empty selection must give zeros"


def test_gather_launch_order_counts_union_rows(dev):
    """work[tile, head] = rows in the union of the tile's selections; the order is a permutation of
    the (tile, head) pairs, one KV head after the other, each head's by descending work class
    (64 classes of equal width)."""
    from semblo_b200.fused_prefill import gather_launch_order
    q_count, hkv, clusters, hq = 1000, 2, 256, 8             # G = 4: tiles of 32 queries, the last one ragged
    g = torch.Generator().manual_seed(11)
    sel = torch.rand(q_count, hkv, clusters, generator=g) < 0.1
    sizes = torch.randint(0, 90, (hkv, clusters), generator=g, dtype=torch.int32)
    order = torch.stack([torch.randperm(q_count, generator=g) for _ in range(hkv)]).int()
    tiles = (q_count + 31) // 32
    got = gather_launch_order(order.to(dev), O.pack_bits(sel).to(dev), sizes.to(dev), hq)
    # a second call that also returns the work counts
    work = torch.empty(tiles * hkv, dtype=torch.int32, device=dev)
    got2 = gather_launch_order(order.to(dev), O.pack_bits(sel).to(dev), sizes.to(dev), hq, work=work)
    want = torch.zeros(tiles, hkv, dtype=torch.int64)
    for h in range(hkv):
        rows = sel[order[h].long(), h]
        for t in range(tiles):
            want[t, h] = int((rows[32 * t:32 * t + 32].any(0).long() * sizes[h].long()).sum())
    assert torch.equal(work.cpu().long().view(tiles, hkv), want)
    for o in (got.cpu().long(), got2.cpu().long()):
        assert sorted(o.tolist()) == list(range(tiles * hkv))
        classes = min(64, 1024 // hkv)
        cls = want.view(-1)[o] * classes // (int(want.max()) + 1)
        key = (o % hkv) * classes + (classes - 1 - cls)             # head-major, then descending work
        assert bool((key[:-1] <= key[1:]).all())
    # without a tile order the tiles are consecutive queries
    got3 = gather_launch_order(None, O.pack_bits(sel).to(dev), sizes.to(dev), hq, work=work)
    want3 = torch.stack([torch.stack([(sel[32 * t:32 * t + 32, h].any(0).long() * sizes[h].long()).sum()
                                      for h in range(hkv)]) for t in range(tiles)])
    assert torch.equal(work.cpu().long().view(tiles, hkv), want3)
    assert sorted(got3.cpu().tolist()) == list(range(tiles * hkv))


def test_argsort_and_top1_keys(dev):
    from semblo_b200.fused_prefill import argsort_keys
    g = torch.Generator().manual_seed(1)
    for n, heads, mx in ((5000, 3, 2048), (333, 1, 200), (8192, 4, 16384), (8192, 8, 2048), (8193, 2, 2048),
                         (1, 2, 1), (31, 1, 2), (1025, 3, 33), (4096, 2, 1000)):
        keys = torch.randint(0, mx, (heads, n), generator=g).int()
        got = argsort_keys(keys.to(dev), mx).cpu().long()
        want = torch.argsort(keys.long(), dim=1, stable=True)
        assert torch.equal(got, want)


def test_launches_issued_ahead_give_the_same_bytes(dev):
    """fused_prefill.WindowAhead: the dense-prefix chunks, the windows and the routing vectors made
    ahead on a second stream, with fewer buffers than chunks so that every buffer is used again."""
    from types import SimpleNamespace
    from semblo_b200.fused_prefill import CausalSnapshot, WindowAhead, fused_chunk_attention
    from semblo_b200.trivial_router import trivial_router_vectors
    dim, hq, hkv, sink, length, target, local, chunk = 128, 8, 2, 64, 6144, 128, 128, 512
    data, index = _small_problem(length, hq, hkv, dim, 24, 9, 32, 7, sink)
    gi = _gpu_index(index, dev)
    q, qp = data["q_post"].to(dev), data["q_pre"].to(dev)
    k, v = data["k_post"].to(dev), data["v"].to(dev)
    pos = torch.arange(length, dtype=torch.int32, device=dev)
    os.environ["SEMBLO_SINK_TOKENS"] = str(sink)
    os.environ["SEMBLO_FA3_LOCAL"] = str(local)
    sm_scale = dim ** -0.5
    try:
        outs = []
        for ahead in (0, 2, 16):
            gi.original_kv = (k, v)
            snap = CausalSnapshot(gi)
            out = torch.zeros(length, hq, dim, dtype=torch.bfloat16, device=dev)
            window = None
            if ahead:
                window = WindowAhead(q, pos, k, v, chunk=chunk, target_tokens=target, sm_scale=sm_scale, out=out,
                                     ahead=ahead, router_input=qp)
                assert window.partial.shape[0] == min(ahead, 10)        # 12 chunks, the first two are dense
            for cs in range(0, length, chunk):
                ce = cs + chunk - 1
                if window is not None:
                    vec = window.vectors_for(cs)
                    assert (vec is None) == (cs <= 4 * target)
                else:
                    vec = trivial_router_vectors(qp[cs:ce + 1]).view(1, chunk, hq, 1, dim)
                fused_chunk_attention(q[cs:ce + 1], SimpleNamespace(vectors=vec), gi, pos[cs:ce + 1], snap, cs, ce,
                                      temperature=0.1, beta=0.25, target_tokens=target, sm_scale=sm_scale,
                                      out=out[cs:ce + 1], window=window)
            if window is not None:
                window.finish()
            torch.cuda.synchronize()
            _status_ok(dev)
            outs.append(out)
        assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
        # a window planned with another budget is refused
        window = WindowAhead(q, pos, k, v, chunk=chunk, target_tokens=4 * target, sm_scale=sm_scale,
                             out=torch.empty_like(outs[0]), ahead=2)
        with pytest.raises(RuntimeError):
            fused_chunk_attention(q[1024:1536], SimpleNamespace(vectors=None), gi, pos[1024:1536], CausalSnapshot(gi),
                                  1024, 1535, temperature=0.1, beta=0.25, target_tokens=target, sm_scale=sm_scale,
                                  out=window.out[1024:1536], window=window)
        window.finish()
        torch.cuda.synchronize()
    finally:
        os.environ.pop("SEMBLO_SINK_TOKENS", None)
        os.environ.pop("SEMBLO_FA3_LOCAL", None)


def test_prefill_chunk_loop_end_to_end(dev):
    """The reference's chunk loop (dense prefix chunks, then selection + sparse body) through the
    mirrored Python entry points, against the oracle evaluated on the kernel's own selections."""
    from types import SimpleNamespace
    from semblo_b200.fused_prefill import CausalSnapshot, fused_chunk_attention
    from semblo_b200.trivial_router import trivial_router_vectors
    dim, hq, hkv, sink, length, target, local, chunk = 128, 8, 2, 64, 5120, 256, 128, 1024
    data, index = _small_problem(length, hq, hkv, dim, 24, 5, 32, 7, sink)
    gi = _gpu_index(index, dev)
    gi.original_kv = (data["k_post"].to(dev), data["v"].to(dev))
    os.environ["SEMBLO_SINK_TOKENS"] = str(sink)
    os.environ["SEMBLO_FA3_LOCAL"] = str(local)
    try:
        snap = CausalSnapshot(gi)
        out = torch.empty(length, hq, dim, dtype=torch.bfloat16, device=dev)
        sm_scale = dim ** -0.5
        selections = {}
        for cs in range(0, length, chunk):
            ce = cs + chunk - 1
            qv = trivial_router_vectors(data["q_pre"][cs:ce + 1].to(dev))
            state = SimpleNamespace(vectors=qv.view(1, chunk, hq, 1, dim))
            fused_chunk_attention(data["q_post"][cs:ce + 1].to(dev), state, gi,
                                  torch.arange(cs, ce + 1, dtype=torch.int32, device=dev), snap, cs, ce,
                                  temperature=0.1, beta=0.25, target_tokens=target, sm_scale=sm_scale,
                                  out=out[cs:ce + 1])
            if O.chunk_plan(cs, target, local) > 0:
                selections[cs] = O.unpack_bits(snap.qmask[:chunk].cpu())
        _status_ok(dev)
    finally:
        os.environ.pop("SEMBLO_SINK_TOKENS", None)
        os.environ.pop("SEMBLO_FA3_LOCAL", None)
    assert len(selections) == 3                     # chunks starting at 2048, 3072, 4096 are sparse
    want = O.prefill_attention(data["q_post"], data["q_pre"], data["k_post"], data["v"], index, temperature=0.1,
                               beta=0.25, target_tokens=target, sink=sink, local=local, sm_scale=sm_scale,
                               chunk=chunk, selections=dict(selections))
    _close_attention(out, want, "prefill end to end")
    # selection parity with the oracle's own selections
    own = {}
    O.prefill_attention(data["q_post"], data["q_pre"], data["k_post"], data["v"], index, temperature=0.1, beta=0.25,
                        target_tokens=target, sink=sink, local=local, sm_scale=sm_scale, chunk=chunk, selections=own)
    rows = sum(int((selections[c] != own[c]).any(-1).sum()) for c in selections)
    assert rows <= 0.02 * 3 * chunk * hkv


# ---------------------------------------------------------------------- decode
@pytest.mark.parametrize("dim,hq,hkv,sink,splits,mask", [(256, 8, 2, 64, 8, 7), (128, 8, 2, 0, 8, 7),
                                                         (256, 8, 2, 64, 2, 7), (128, 16, 2, 64, 3, 15)])
def test_decode_steps_through_the_arena(dev, dim, hq, hkv, sink, splits, mask):
    """splits = 2 or 3 gives a CTA several resident-row chunks; mask 15 launches the three stages
    strictly one after the other."""
    from types import SimpleNamespace
    from semblo_b200.arena import DecodeArena
    from semblo_b200.fused_decode import fused_decode_step
    length, target, steps = 6000, 512, 6
    data, index = _small_problem(length + steps, hq, hkv, dim, 24, 9 + dim, 32, 7, sink)
    # the index covers the prompt only
    prompt = {k: v[:length] for k, v in data.items()}
    product = O.routing_normalize(prompt["k_pre"])
    index = O.build_flat(product, unit_tokens=32, min_clusters_log2=7, kmeans_sample_size=1024, fit_iters=4,
                         seed=0, sink=sink, page_align=16)
    O.pack_prompt_kv(index, prompt["k_post"], prompt["v"])
    clusters = index.bucket_sizes.shape[1]
    ref = O.make_arena(capacity=8192, num_clusters=256, num_kv_heads=hkv, head_dim=dim, page_align=16, reserve=512,
                       kv_dtype=torch.bfloat16, desc_dtype=torch.bfloat16, keep_kpre=True)
    O.arena_adopt(ref, index)
    arena = DecodeArena(capacity=8192, num_kv_heads=hkv, head_dim=dim, num_clusters=256, page_align=16, device=dev,
                        reserve=512, keep_kpre=True)
    assert arena.width == ref.posting.shape[1] and clusters <= 256
    arena.adopt(_gpu_index(index, dev))
    assert torch.equal(arena.suffix_table.cpu(), ref.suffix_table)
    layer = SimpleNamespace(num_heads=hq, num_kv_heads=hkv, head_dim=dim)
    sm_scale = dim ** -0.5
    out = torch.empty(1, hq * dim, dtype=torch.bfloat16, device=dev)
    os.environ["SEMBLO_SINK_TOKENS"] = str(sink)
    try:
        for s in range(steps):
            pos = length + s
            args = dict(q_post=data["q_post"][pos], q_pre=data["q_pre"][pos], k_post=data["k_post"][pos],
                        v=data["v"][pos], k_pre=data["k_pre"][pos])
            vectors = O.trivial_router_vectors(args["q_pre"])
            sel_ref, csr_ref, margin = O.decode_select(vectors, ref, temperature=0.1, beta=0.25, target_tokens=target,
                                                       sink=sink, return_margin=True)
            fused_decode_step(layer, arena, q_post=args["q_post"][None].contiguous().to(dev),
                              q_pre=args["q_pre"][None].contiguous().to(dev),
                              positions=torch.tensor([pos], device=dev), k_post=args["k_post"][None].contiguous().to(dev),
                              v_states=args["v"][None].contiguous().to(dev), k_pre=args["k_pre"][None].contiguous().to(dev),
                              output=out, temperature=0.1, beta=0.25, target_tokens=target, sm_scale=sm_scale,
                              num_splits=splits, stage_mask=mask)
            _status_ok(dev)
            ws = arena.fused_decode_ws
            assert torch.equal(ws.vectors.cpu().float(), vectors.float()) or \
                float(((ws.vectors.cpu().float() - vectors.float()).abs() > 0).float().mean()) < 4e-3
            # the kernel's selection, recovered from its CSR
            sel = torch.zeros(hkv, 256, dtype=torch.bool)
            for h in range(hkv):
                n = int(ws.rcount[h])
                starts = ws.rstart[h, :n].cpu()
                ids = torch.searchsorted(ref.indptr[h].contiguous(), starts, right=True) - 1
                # clusters with equal starts are empty: take the last one with that start
                sel[h, ids] = True
                lens = ws.rlen[h, :n].cpu()
                assert torch.equal(lens, ref.sizes[h][ids])
                assert torch.equal(ws.rcum[h, :n].cpu(), (lens.cumsum(0) - lens).int())
                assert int(ws.rtokens[h]) == int(lens.sum())
            differ = (sel != sel_ref).any(-1)
            assert bool((margin[differ] < 1e-4).all())
            want, _, _ = O.decode_step(ref, q_post=args["q_post"], q_pre=args["q_pre"], pos=pos, k_post=args["k_post"],
                                       v=args["v"], k_pre=args["k_pre"], temperature=0.1, beta=0.25,
                                       target_tokens=target, sink=sink, sm_scale=sm_scale, sel=sel)
            _close_attention(out.view(hq, dim), want, f"decode step {s}")
        assert torch.equal(arena.suffix_kv.cpu().float(), ref.suffix_kv.float())
        assert torch.equal(arena.suffix_kpre.cpu().float(), ref.suffix_kpre.float())
    finally:
        os.environ.pop("SEMBLO_SINK_TOKENS", None)


@pytest.mark.parametrize("clusters", [128, 2048, 4096])
def test_threshold_selection_on_given_scores_is_exact(dev, clusters):
    """Register-resident (C <= 2048) and shared-memory (larger C) selectors against the oracle's
    float32 rule on identical scores: the result is a pure function of (scores, sizes)."""
    from semblo_b200._lib import lib, ptr, check, stream_ptr
    g = torch.Generator().manual_seed(clusters)
    nq, hkv, target = 77, 3, 900
    sizes = torch.randint(0, 40, (hkv, clusters), generator=g).int()
    sizes[:, ::5] = 0
    sizes[2] = (sizes[2] > 30).int()                      # everything fits for head 2
    score = torch.randn(nq, hkv, clusters, generator=g) * 2
    score = torch.where(sizes[None] > 0, score, torch.full_like(score, O.NEG_BIG))
    want = O.theta_select(score, sizes[None], target, 16)
    qmask = torch.empty(nq, hkv, clusters // 32, dtype=torch.int32, device=dev)
    counts = torch.empty(nq, hkv, dtype=torch.int32, device=dev)
    tokens = torch.empty(nq, hkv, dtype=torch.int32, device=dev)
    top1 = torch.empty(hkv, nq, dtype=torch.int32, device=dev)
    score_d, sizes_d = score.to(dev), sizes.to(dev)          # keep the device copies alive across the call
    check(lib().semblo_select_clusters(ptr(score_d), ptr(sizes_d), nq, hkv, clusters, target, 16, 0,
                                       ptr(qmask), ptr(counts), ptr(tokens), ptr(top1), 0.0, stream_ptr()))
    assert torch.equal(O.unpack_bits(qmask.cpu()), want)
    assert torch.equal(counts.cpu(), want.sum(-1).int())
    assert torch.equal(tokens.cpu(), (want * sizes[None]).sum(-1).int())
    assert torch.equal(top1.cpu().long().t(), score.argmax(-1))


# ---------------------------------------------------------------------- decode without an arena
def test_decode_over_the_index_paged_suffix_and_merge(dev):
    """The decode path of a request that has no arena (fused_prefill.py:625-718, paged_attention.py:50-78,
    961-1128): sparse attention over the packed prompt with its log-sum-exp, attention over the generated
    suffix read from a paged cache through a block table, and their exact merge - each against the oracle,
    and the merged result against the oracle's whole decode step."""
    from types import SimpleNamespace
    from semblo_b200.fused_prefill import fused_decode_attention
    from semblo_b200.paged_attention import (PagedSparseAttentionResult, PostingTiles, merge_paged_attention_results,
                                             paged_posting_attention)
    from semblo_b200.trivial_router import trivial_router_vectors
    dim, hq, hkv, sink, length, target, gen = 128, 8, 2, 64, 6000, 512, 37
    data, index = _small_problem(length + gen + 1, hq, hkv, dim, 24, 3, 32, 7, sink)
    prompt = {k: v[:length] for k, v in data.items()}
    index = O.build_flat(O.routing_normalize(prompt["k_pre"]), unit_tokens=32, min_clusters_log2=7,
                         kmeans_sample_size=1024, fit_iters=4, seed=0, sink=sink, page_align=16)
    O.pack_prompt_kv(index, prompt["k_post"], prompt["v"])
    gi = _gpu_index(index, dev)
    clusters = index.bucket_sizes.shape[1]
    pos = length + gen                                   # the query's position: `gen` generated tokens before it
    q_post, q_pre = data["q_post"][pos], data["q_pre"][pos]
    sm_scale = dim ** -0.5
    os.environ["SEMBLO_SINK_TOKENS"] = str(sink)
    try:
        qv = trivial_router_vectors(q_pre[None].to(dev))
        state = SimpleNamespace(vectors=qv.view(1, 1, hq, 1, dim))
        res = fused_decode_attention(q_post[None].to(dev), state, gi, torch.tensor([pos], dtype=torch.int32, device=dev),
                                     temperature=0.1, beta=0.25, target_tokens=target, sm_scale=sm_scale, num_splits=6)
        _status_ok(dev)
    finally:
        os.environ.pop("SEMBLO_SINK_TOKENS", None)
    # the oracle on the kernel's own selection: an arena without suffix is the index itself
    ref = O.make_arena(capacity=8192, num_clusters=clusters, num_kv_heads=hkv, head_dim=dim, page_align=16, reserve=256,
                       kv_dtype=torch.bfloat16, desc_dtype=torch.bfloat16)
    O.arena_adopt(ref, index)
    ws = gi._decode_ws
    sel = torch.zeros(hkv, clusters, dtype=torch.bool)
    for h in range(hkv):
        n = int(ws.rcount[h])
        ids = torch.searchsorted(ref.indptr[h].contiguous(), ws.rstart[h, :n].cpu(), right=True) - 1
        sel[h, ids] = True
    sel_ref, _, margin = O.decode_select(O.trivial_router_vectors(q_pre), ref, temperature=0.1, beta=0.25,
                                         target_tokens=target, sink=sink, return_margin=True)
    assert bool((margin[(sel != sel_ref).any(-1)] < 1e-4).all())
    group = hq // hkv
    want_p = torch.empty(hq, dim, dtype=torch.float64)
    lse_p = torch.empty(hq, dtype=torch.float64)
    for h in range(hkv):
        rows = torch.cat([torch.arange(int(ref.indptr[h, c]), int(ref.indptr[h, c]) + int(ref.sizes[h, c]))
                          for c in torch.nonzero(sel[h]).flatten().tolist()])
        o, l = O._masked_attention(q_post[None, h * group:(h + 1) * group], ref.packed_kv[0, rows, h],
                                   ref.packed_kv[1, rows, h], torch.ones(1, rows.numel(), dtype=torch.bool), sm_scale)
        want_p[h * group:(h + 1) * group], lse_p[h * group:(h + 1) * group] = o[0], l[0]
    _close_attention(res.output[0], want_p, "decode over the index")
    torch.testing.assert_close(res.logsumexp[0].cpu().double(), lse_p, atol=2e-3, rtol=0)
    # the generated suffix in a paged cache with 16-token blocks behind a permuted block table
    block, n_blocks = 16, (length + gen + 1 + 15) // 16 + 3
    perm = torch.randperm(n_blocks, generator=torch.Generator().manual_seed(8))
    cache = torch.zeros(2, n_blocks, block, hkv, dim, dtype=torch.bfloat16)
    for p in range(length, pos + 1):
        cache[0, perm[p // block], p % block] = data["k_post"][p]
        cache[1, perm[p // block], p % block] = data["v"][p]
    reserve = 64                                          # the tiles cover reserved ground past the query too
    spos = torch.arange(length, length + reserve, dtype=torch.int32)
    tile = 16
    slots = reserve // tile
    tiles = PostingTiles(starts=(torch.arange(slots, dtype=torch.int32) * tile).view(1, 1, -1).expand(1, hkv, -1).contiguous().to(dev),
                         lengths=torch.full((1, hkv, slots), tile, dtype=torch.int32, device=dev),
                         counts=torch.full((1, hkv), slots, dtype=torch.int32, device=dev),
                         selected_tokens=torch.full((1, hkv), reserve, dtype=torch.int32, device=dev))
    sres = paged_posting_attention(q_post[None].to(dev), cache.to(dev), spos[None].expand(hkv, -1).contiguous().to(dev),
                                   tiles, torch.tensor([pos], dtype=torch.int32, device=dev),
                                   torch.zeros(1, dtype=torch.int32, device=dev), perm.int()[None].to(dev),
                                   block_size=block, sm_scale=sm_scale, softcap=None, token_tile=tile, num_splits=2,
                                   return_logsumexp=True)
    _status_ok(dev)
    ks, vs = data["k_post"][length:pos + 1], data["v"][length:pos + 1]
    want_s = torch.empty(hq, dim, dtype=torch.float64)
    lse_s = torch.empty(hq, dtype=torch.float64)
    for h in range(hkv):
        o, l = O._masked_attention(q_post[None, h * group:(h + 1) * group], ks[:, h], vs[:, h],
                                   torch.ones(1, ks.shape[0], dtype=torch.bool), sm_scale)
        want_s[h * group:(h + 1) * group], lse_s[h * group:(h + 1) * group] = o[0], l[0]
    _close_attention(sres.output[0], want_s, "suffix through the block table")
    torch.testing.assert_close(sres.logsumexp[0].cpu().double(), lse_s, atol=2e-3, rtol=0)
    merged = merge_paged_attention_results(res, sres)
    want_m, lse_m = O.merge_states(want_p, lse_p, want_s, lse_s)
    _close_attention(merged.output[0], want_m, "merged decode")
    torch.testing.assert_close(merged.logsumexp[0].cpu().double(), lse_m, atol=2e-3, rtol=0)
    # a state with nothing attended merges as the other one
    empty = PagedSparseAttentionResult(output=torch.zeros_like(res.output),
                                       logsumexp=torch.full_like(res.logsumexp, float("-inf")))
    again = merge_paged_attention_results(empty, sres)
    assert torch.equal(again.output, sres.output)
