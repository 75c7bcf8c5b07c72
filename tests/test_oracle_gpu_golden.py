"""The CPU oracle against outputs of the reference's own GPU kernels (Triton), recorded by
tests/golden/make_golden_gpu.py into tests/golden/reference_gpu_golden.npz: the query router,
the centroid scores, the bisected-threshold selection in both of its branches, the fused decode
step and the Triton sparse prefill body.  A section the generator could not run on its device is
recorded as an error there and skipped here with that message."""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import semblo_oracle as O

PATH = Path(__file__).resolve().parent / "golden" / "reference_gpu_golden.npz"


@pytest.fixture(scope="module")
def gold():
    if not PATH.exists():
        pytest.skip("tests/golden/reference_gpu_golden.npz has not been generated")
    return np.load(PATH)


def _section(gold, name, key):
    err = f"error_{name}"
    if err in gold.files:
        pytest.skip("the reference kernel did not run on the generating device: " + bytes(gold[err]).decode())
    return gold[key]


def _bf16(a):
    return torch.from_numpy(np.ascontiguousarray(a)).view(torch.bfloat16)


def _params(gold):
    return json.loads(bytes(gold["meta"]).decode())["params"]


@pytest.mark.parametrize("name", ["theta512", "theta4096"])
def test_router_scores_and_threshold_selection(gold, name):
    p = _params(gold)
    q_pre = _bf16(_section(gold, name, f"{name}_q_pre"))
    codebooks = _bf16(gold[f"{name}_codebooks"])
    sizes = torch.from_numpy(gold[f"{name}_sizes"])               # [1, Hkv, C]
    target = int(gold[f"{name}_target"])
    vectors_ref = _bf16(gold[f"{name}_vectors"]).reshape(q_pre.shape)
    prob_ref = torch.from_numpy(gold[f"{name}_prob"])
    qmask_ref = torch.from_numpy(gold[f"{name}_qmask"])
    # a7: the query router (trivial_router.py:23-45) against its Triton kernel
    vectors = O.trivial_router_vectors(q_pre)
    differ = (vectors.float() != vectors_ref.float())
    assert float(differ.float().mean()) < 5e-3
    assert float((vectors.float() - vectors_ref.float()).abs().max()) <= 2 ** -8
    # a8 scores: the tensor-core kernel accumulates bf16 products in fp32
    prob = O.mixture_prob(vectors_ref, codebooks, p["temperature"])
    live = (sizes[0] > 0)[None].expand_as(prob_ref)
    rel = ((prob - prob_ref).abs() / prob_ref.clamp_min(1e-30))[live]
    assert float(rel.max()) < 2e-3, float(rel.max())
    # the threshold rule is a pure function of (prob, sizes): exact on the reference's own prob
    score = O.penalized_scores(prob_ref, sizes, p["beta"]).float()
    sel, margin = O.theta_select(score, sizes, target, 16, return_margin=True)
    sel_ref = O.unpack_bits(qmask_ref)
    differ = (sel != sel_ref).any(-1)
    # log() of the two libraries may differ in the last bit: only rows with a score on a midpoint may move
    assert bool((margin[differ] < 1e-6).all()), (int(differ.sum()), margin[differ])
    assert int(differ.sum()) <= 1
    same = ~differ
    assert torch.equal(torch.from_numpy(gold[f"{name}_counts"])[same], sel.sum(-1).int()[same])
    assert torch.equal(torch.from_numpy(gold[f"{name}_tokens"])[same], (sel * sizes).sum(-1).int()[same])
    assert torch.equal(O.unpack_bits(torch.from_numpy(gold[f"{name}_bitmask"]))[0], sel_ref.any(0))
    # end to end from the oracle's own scores: identical outside the oracle's margin band
    sel_own, margin_own = O.select_clusters(vectors_ref, codebooks, sizes[0], temperature=p["temperature"],
                                            beta=p["beta"], target_tokens=target, return_margin=True)
    differ = (sel_own != sel_ref).any(-1)
    assert bool((margin_own[differ] < 1e-4).all())
    assert float(differ.float().mean()) < 0.05


def _problem(gold):
    p = _params(gold)
    n = p["length"] - p["decode_steps"]
    data = O.mixture_inputs(length=p["length"], num_q_heads=p["hq"], num_kv_heads=p["hkv"], head_dim=p["dim"],
                            centres=p["centres"], seed=p["seed"])
    index = O.FlatIndex(codebooks=_bf16(gold["index_codebooks"]), posting_positions=torch.from_numpy(gold["index_posting"]),
                        bucket_indptr=torch.from_numpy(gold["index_indptr"]), bucket_sizes=torch.from_numpy(gold["index_sizes"]),
                        inverse_positions=torch.from_numpy(gold["index_inverse"]),
                        assign=torch.from_numpy(gold["index_assign"]).long(), prompt_length=n, page_align=16)
    O.pack_prompt_kv(index, data["k_post"][:n], data["v"][:n])
    return p, data, index, n


def test_fused_decode_step(gold):
    out_ref = _bf16(_section(gold, "decode", "decode_out"))
    p, data, index, n = _problem(gold)
    hq, hkv, dim = p["hq"], p["hkv"], p["dim"]
    clusters = int(index.bucket_sizes.shape[1])
    arena = O.make_arena(capacity=8192, num_clusters=clusters, num_kv_heads=hkv, head_dim=dim, page_align=16,
                         reserve=p["reserve"], kv_dtype=torch.bfloat16, desc_dtype=torch.bfloat16, keep_kpre=True)
    O.arena_adopt(arena, index)
    assert torch.equal(arena.suffix_table, torch.from_numpy(gold["decode_suffix_table"]))
    for s in range(p["decode_steps"]):
        pos = n + s
        sel_ref = torch.from_numpy(gold["decode_sel"][s])
        vectors = O.trivial_router_vectors(data["q_pre"][pos])
        vec_ref = _bf16(gold["decode_vectors"][s]).reshape(hq, dim)
        assert float((vectors.float() != vec_ref.float()).float().mean()) < 5e-3
        sel, csr, margin = O.decode_select(vec_ref, arena, temperature=p["temperature"], beta=p["beta"],
                                           target_tokens=p["target"], sink=p["sink"], return_margin=True)
        differ = (sel != sel_ref).any(-1)
        assert bool((margin[differ] < 1e-4).all()), (s, margin[differ])
        for h in range(hkv):
            if not bool(differ[h]):
                assert int(gold["decode_rcount"][s][h]) == int(sel[h].sum())
                assert int(gold["decode_rtokens"][s][h]) == int((sel[h] * arena.sizes[h]).sum())
        want, _, _ = O.decode_step(arena, q_post=data["q_post"][pos], q_pre=data["q_pre"][pos], pos=pos,
                                   k_post=data["k_post"][pos], v=data["v"][pos], k_pre=data["k_pre"][pos],
                                   temperature=p["temperature"], beta=p["beta"], target_tokens=p["target"],
                                   sink=p["sink"], sm_scale=dim ** -0.5, sel=sel_ref)
        diff = (out_ref[s].reshape(hq, dim).double() - want).abs()
        assert float(diff.max()) <= 2e-2, (s, float(diff.max()))
        assert float(diff.mean()) <= 1e-3
    stored = _bf16(gold["decode_suffix_kv"])
    assert torch.equal(arena.suffix_kv[:, :1, :8].float(), stored.float())


def test_triton_sparse_prefill_body(gold):
    out_ref = _bf16(_section(gold, "union", "union_out"))
    p, data, index, n = _problem(gold)
    hq, hkv, dim = p["hq"], p["hkv"], p["dim"]
    clusters = int(index.bucket_sizes.shape[1])
    cs = int(gold["union_chunk_start"])
    qn = out_ref.shape[0]
    sel = torch.from_numpy(np.unpackbits(gold["union_sel"], axis=-1)[..., :clusters].astype(np.bool_))
    sizes = O.causal_sizes_at(index, cs - 1)
    # the generator selected with the oracle on its own host: the same rule here
    vectors = O.trivial_router_vectors(data["q_pre"][cs:cs + qn])
    sel_here, margin = O.select_clusters(vectors, index.codebooks, sizes, temperature=p["temperature"],
                                         beta=p["beta"], target_tokens=p["target"], sink=p["sink"], return_margin=True)
    differ = (sel_here != sel).any(-1)
    assert bool((margin[differ] < 1e-4).all())
    qpos = torch.arange(cs, cs + qn)
    empty = data["k_post"][cs:cs]
    want, natt, lse = O.sparse_chunk_attention(data["q_post"][cs:cs + qn], index, sel, sizes, qpos, empty,
                                               data["v"][cs:cs], cs, dim ** -0.5, return_lse=True)
    diff = (out_ref.reshape(qn, hq, dim).double() - want).abs()
    assert float(diff.max()) <= 2e-2, float(diff.max())
    assert float(diff.mean()) <= 1e-3
    lse_ref = torch.from_numpy(gold["union_lse"]).double()
    assert float((lse_ref - lse).abs().max()) <= 2e-3
    # union size of every block of 16 queries: the rows the body walked
    gq = 16
    union = (sel.view(qn // gq, gq, hkv, clusters).any(1) * sizes[None]).sum(-1)
    assert torch.equal(torch.from_numpy(gold["union_tokens"]).long(), union.long())
