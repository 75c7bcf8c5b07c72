"""Golden outputs of the reference's own GPU kernels, for pinning the CPU oracle.

    python tests/golden/make_golden_gpu.py [--ref baseline/_ref] [--out tests/golden/reference_gpu_golden.npz]

Needs a CUDA device, Triton, and the reference importable from ``--ref`` (a pip --target install of
the reference checkout; the reference is never imported by the product code).  It runs, on small
seeded inputs,

  * ``trivial_router_vectors`` (Triton), ``flat_mixture_scores_qtiled`` and ``theta_select_bitmask_flat``
    of semblo/vllm_plugin/fused_select.py at 512 clusters (register-resident bisection) and at 4096
    clusters (streamed bisection);
  * ``fused_decode_step`` of semblo/vllm_plugin/fused_decode.py for a few steps over a small arena;
  * ``build_union_slots`` + ``union_block_attention`` (per-query strict selection) of
    semblo/vllm_plugin/fused_union.py / fused_body.py: the Triton sparse prefill body;

and stores the inputs that cannot be regenerated from seeds (the integer index, which depends on
the host's matmul kernels) together with the kernels' outputs.  A section whose kernel does not
run on the device at hand is recorded under ``error_<section>`` instead.  tests/test_oracle_gpu_golden.py
checks the oracle against the file on the CPU."""
from __future__ import annotations

import argparse
import json
import os
import sys
import traceback
import types
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from oracle import semblo_oracle as O  # noqa: E402

PARAMS = dict(temperature=0.1, beta=0.25, seed=11, length=4096 + 4, dim=128, hq=8, hkv=2, centres=16,
              unit=32, min_log2=7, sink=64, target=512, decode_steps=4, reserve=512)


def small_problem(p):
    """Seeded mixture inputs and a CPU-built index (the oracle's build is pinned to the reference's CPU
    build by tests/golden/make_golden.py)."""
    n = p["length"] - p["decode_steps"]
    data = O.mixture_inputs(length=p["length"], num_q_heads=p["hq"], num_kv_heads=p["hkv"], head_dim=p["dim"],
                            centres=p["centres"], seed=p["seed"])
    index = O.build_flat(O.routing_normalize(data["k_pre"][:n]), unit_tokens=p["unit"],
                         min_clusters_log2=p["min_log2"], kmeans_sample_size=1024, fit_iters=4, seed=0,
                         sink=p["sink"], page_align=16)
    O.pack_prompt_kv(index, data["k_post"][:n], data["v"][:n])
    return data, index, n


def bits_to_np(t):
    return t.detach().cpu().numpy()


def section_theta(out, name, *, clusters, queries, hq, hkv, dim, target, seed, dev):
    from semblo.vllm_plugin.fused_select import flat_mixture_scores_qtiled, theta_select_bitmask_flat
    from semblo.vllm_plugin.trivial_router import trivial_router_vectors
    g = torch.Generator().manual_seed(seed)
    cb = torch.nn.functional.normalize(torch.randn(hkv, clusters, dim, generator=g), dim=-1)
    # queries near some centroids, so the scores have a clear head and a long tail
    pick = torch.randint(0, clusters, (queries, hkv), generator=g)
    q = cb[torch.arange(hkv)[None, :], pick][:, :, None, :] + 0.08 * torch.randn(queries, hkv, hq // hkv, dim, generator=g)
    q_pre = q.reshape(queries, hq, dim).to(torch.bfloat16)
    codebooks = torch.stack((cb[..., :dim // 2], cb[..., dim // 2:]), dim=1).to(torch.bfloat16).contiguous()
    sizes = torch.randint(0, 70, (1, hkv, clusters), generator=g).int()
    sizes[:, :, ::9] = 0
    vectors = trivial_router_vectors(q_pre.to(dev), 1).view(queries, hq, 1, dim)
    logmix = torch.zeros(queries, hq, 1, dtype=torch.float32, device=dev)
    prob = flat_mixture_scores_qtiled(vectors, logmix, codebooks.to(dev), temperature=PARAMS["temperature"])
    bitmask = torch.zeros(1, hkv, clusters // 32, dtype=torch.int32, device=dev)
    qmask = torch.empty(queries, hkv, clusters // 32, dtype=torch.int32, device=dev)
    counts, tokens = theta_select_bitmask_flat(vectors, logmix, codebooks.to(dev), sizes.to(dev), bitmask,
                                               temperature=PARAMS["temperature"], beta=PARAMS["beta"],
                                               target_tokens=target, g_union=queries, qmask=qmask)
    torch.cuda.synchronize()
    out[f"{name}_q_pre"] = q_pre.view(torch.int16).numpy()
    out[f"{name}_codebooks"] = codebooks.view(torch.int16).numpy()
    out[f"{name}_sizes"] = sizes.numpy()
    out[f"{name}_target"] = np.int64(target)
    out[f"{name}_vectors"] = vectors.cpu().view(torch.int16).numpy()
    out[f"{name}_prob"] = bits_to_np(prob)
    out[f"{name}_qmask"] = bits_to_np(qmask)
    out[f"{name}_bitmask"] = bits_to_np(bitmask)
    out[f"{name}_counts"] = bits_to_np(counts)
    out[f"{name}_tokens"] = bits_to_np(tokens)


def store_index(out, index):
    out["index_codebooks"] = index.codebooks.view(torch.int16).numpy()
    out["index_posting"] = index.posting_positions.numpy()
    out["index_indptr"] = index.bucket_indptr.numpy()
    out["index_sizes"] = index.bucket_sizes.numpy()
    out["index_inverse"] = index.inverse_positions.numpy()
    out["index_assign"] = index.assign.to(torch.int32).numpy()


def section_decode(out, data, index, n, dev):
    from semblo.vllm_plugin.fused_decode import fused_decode_step
    p = PARAMS
    hq, hkv, dim = p["hq"], p["hkv"], p["dim"]
    clusters = int(index.bucket_sizes.shape[1])
    ref = O.make_arena(capacity=8192, num_clusters=clusters, num_kv_heads=hkv, head_dim=dim, page_align=16,
                       reserve=p["reserve"], kv_dtype=torch.bfloat16, desc_dtype=torch.bfloat16, keep_kpre=True)
    O.arena_adopt(ref, index)
    arena = types.SimpleNamespace(
        num_clusters=clusters, reserve=p["reserve"], suffix_block=256, sizes=ref.sizes.to(dev),
        indptr=ref.indptr.to(dev), posting=ref.posting.to(dev), packed_kv=ref.packed_kv.to(dev),
        codebooks=ref.codebooks.to(dev), prompt_length_t=ref.prompt_length_t.to(dev),
        suffix_kv=ref.suffix_kv.to(dev), suffix_kpre=ref.suffix_kpre.to(dev), suffix_table=ref.suffix_table.to(dev),
        index=types.SimpleNamespace(prompt_length=n))
    layer = types.SimpleNamespace(num_heads=hq, num_kv_heads=hkv, head_dim=dim,
                                  runtime_config=types.SimpleNamespace(triton_token_tile=16))
    os.environ["SEMBLO_SINK_TOKENS"] = str(p["sink"])
    outs, csr = [], []
    try:
        for s in range(p["decode_steps"]):
            pos = n + s
            o = torch.zeros(1, hq * dim, dtype=torch.bfloat16, device=dev)
            fused_decode_step(layer, arena, q_post=data["q_post"][pos:pos + 1].contiguous().to(dev),
                              q_pre=data["q_pre"][pos:pos + 1].contiguous().to(dev),
                              positions=torch.tensor([pos], device=dev),
                              k_post=data["k_post"][pos:pos + 1].contiguous().to(dev),
                              v_states=data["v"][pos:pos + 1].contiguous().to(dev),
                              k_pre=data["k_pre"][pos:pos + 1].contiguous().to(dev), output=o,
                              temperature=p["temperature"], beta=p["beta"], target_tokens=p["target"],
                              sm_scale=dim ** -0.5, num_splits=8)
            torch.cuda.synchronize()
            ws = arena.fused_decode_ws
            outs.append(o.cpu().view(torch.int16).numpy())
            sel = np.zeros((hkv, clusters), dtype=np.bool_)
            for h in range(hkv):
                cnt = int(ws.rcount[h])
                starts = ws.rstart[h, :cnt].cpu()
                ids = torch.searchsorted(ref.indptr[h].contiguous(), starts, right=True) - 1
                sel[h, ids.numpy()] = True
            csr.append(dict(sel=sel, rcount=ws.rcount.cpu().numpy().copy(), rtokens=ws.rtokens.cpu().numpy().copy(),
                            vectors=ws.vectors.cpu().view(torch.int16).numpy().copy(),
                            prob=ws.prob_ws.cpu().numpy().copy()))
    finally:
        os.environ.pop("SEMBLO_SINK_TOKENS", None)
    out["decode_out"] = np.stack(outs)
    out["decode_sel"] = np.stack([c["sel"] for c in csr])
    out["decode_rcount"] = np.stack([c["rcount"] for c in csr])
    out["decode_rtokens"] = np.stack([c["rtokens"] for c in csr])
    out["decode_vectors"] = np.stack([c["vectors"] for c in csr])
    out["decode_prob"] = np.stack([c["prob"] for c in csr])
    out["decode_suffix_kv"] = arena.suffix_kv.cpu().view(torch.int16).numpy()[:, :1, :8]
    out["decode_suffix_table"] = arena.suffix_table.cpu().numpy()


def section_union_body(out, data, index, n, dev):
    """The Triton sparse body with per-query strict selection over one chunk of queries."""
    from semblo.vllm_plugin.fused_body import union_block_attention
    from semblo.vllm_plugin.fused_union import build_union_slots
    p = PARAMS
    hq, hkv, dim = p["hq"], p["hkv"], p["dim"]
    clusters = int(index.bucket_sizes.shape[1])
    cs, qn, gq = 3072, 64, 16
    sizes = O.causal_sizes_at(index, cs - 1)                                       # [Hkv, C]
    vectors = O.trivial_router_vectors(data["q_pre"][cs:cs + qn])
    sel = O.select_clusters(vectors, index.codebooks, sizes, temperature=p["temperature"], beta=p["beta"],
                            target_tokens=p["target"], sink=p["sink"])              # [Q, Hkv, C] bool
    qmask = O.pack_bits(sel)
    nb = qn // gq
    bitmask = O.pack_bits(sel.view(nb, gq, hkv, clusters).any(1))
    sizes3 = sizes[None].expand(nb, -1, -1).contiguous()
    umax = int(index.posting_positions.shape[1])
    union_idx, union_tokens, _, slot_rowmask = build_union_slots(
        bitmask.to(dev), sizes3.to(dev), index.bucket_indptr.to(dev), rmax=clusters, umax=umax,
        qmask=qmask.to(dev), queries_per_block=gq)
    qpos = torch.arange(cs, cs + qn, dtype=torch.int32)
    o, lse = union_block_attention(data["q_post"][cs:cs + qn].contiguous().to(dev), index.packed_kv.to(dev),
                                   index.posting_positions.to(dev), union_idx, union_tokens, qpos.to(dev),
                                   queries_per_block=gq, sm_scale=dim ** -0.5, return_logsumexp=True,
                                   slot_rowmask=slot_rowmask)
    torch.cuda.synchronize()
    out["union_chunk_start"] = np.int64(cs)
    out["union_sel"] = np.packbits(sel.numpy(), axis=-1)
    out["union_tokens"] = union_tokens.cpu().numpy()
    out["union_out"] = o.cpu().view(torch.int16).numpy()
    out["union_lse"] = lse.cpu().numpy()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=str(ROOT / "baseline" / "_ref"))
    ap.add_argument("--out", default=str(ROOT / "tests" / "golden" / "reference_gpu_golden.npz"))
    args = ap.parse_args()
    sys.path.insert(0, args.ref)
    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device")
    dev = torch.device("cuda:0")
    import triton
    out = {"meta": np.frombuffer(json.dumps(dict(params=PARAMS, torch=torch.__version__, triton=triton.__version__,
                                                   device=torch.cuda.get_device_name(0))).encode(), dtype=np.uint8)}
    errors = {}

    def run(name, fn):
        try:
            fn()
            print(f"[{name}] ok")
        except Exception as e:  # record and go on: each section stands alone
            errors[name] = f"{type(e).__name__}: {e}"
            print(f"[{name}] FAILED: {errors[name]}")
            traceback.print_exc()

    run("theta512", lambda: section_theta(out, "theta512", clusters=512, queries=96, hq=8, hkv=2, dim=128,
                                          target=700, seed=5, dev=dev))
    run("theta4096", lambda: section_theta(out, "theta4096", clusters=4096, queries=12, hq=8, hkv=2, dim=128,
                                           target=3000, seed=6, dev=dev))
    data, index, n = small_problem(PARAMS)
    store_index(out, index)
    run("decode", lambda: section_decode(out, data, index, n, dev))
    run("union", lambda: section_union_body(out, data, index, n, dev))
    for k, v in errors.items():
        out[f"error_{k}"] = np.frombuffer(v.encode()[:2000], dtype=np.uint8)
    np.savez_compressed(args.out, **out)
    print("wrote", args.out, {k: v for k, v in errors.items()})


if __name__ == "__main__":
    main()
