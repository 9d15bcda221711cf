"""GPU parity of the prefill path (routing, forward, backward) against the FP64 oracle and the
golden vectors produced by the reference.  Everything goes through the C ABI via moba_opt.

Tolerances (bf16 inputs, FP64 oracle under the kernel's own routes): max-abs <= 2e-2 and
rel-RMS <= 5e-3 for outputs and gradients; block selection bit-exact.  The max-abs bound is taken
relative to max(1, max|reference|): gradients reach magnitudes where one bf16 ulp of the stored
result already exceeds 2e-2 (ulp(8) = 0.03), while attention outputs are O(1) so for them the bound
is the plain 2e-2.
"""
import numpy as np
import pytest
import torch

from helpers import (PREFILL_GOLDENS, ROUTE_GOLDENS, bits_to_torch, config1_inputs, cu_from_lens, load, rel_rms,
                     torch_to_f64, unpack_selected)
from oracle import moba_oracle as mo

pytestmark = pytest.mark.gpu

MAX_ABS, REL_RMS = 2e-2, 5e-3


def _run(q, k, v, cu, chunk, topk, d_out=None, **flags):
    import moba_opt
    import moba_opt.grouped_attention as ga
    dev = "cuda"
    q, k, v = (t.to(dev).requires_grad_(d_out is not None) for t in (q, k, v))
    cu_t = torch.tensor(cu, dtype=torch.int32, device=dev)
    max_len = int(np.diff(cu).max())
    cfg = {"chunk_size": chunk, "topk": topk, "route_precision": "fp32", "stable_routes": True, **flags}
    captured = {}
    ga.ROUTE_HOOK = lambda **kw: captured.update(kw)
    try:
        out, lse = ga.moba_prefill(q, k, v, cu_t, max_len, cfg, return_lse=True)
    finally:
        ga.ROUTE_HOOK = None
    grads = None
    if d_out is not None:
        grads = torch.autograd.grad(out, (q, k, v), grad_outputs=d_out.to(dev))
    ga.check_status()
    return out, lse, captured, grads


def _check_close(name, got, ref):
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    assert np.isfinite(got).all(), name
    plain = np.abs(got - ref).max()
    err = plain / max(1.0, np.abs(ref).max())
    rr = rel_rms(got, ref)
    print(f"{name}: max-abs {plain:.3e}, |ref|max {np.abs(ref).max():.3e}, scaled max-abs {err:.3e}, rel-rms {rr:.3e}")
    assert err <= MAX_ABS and rr <= REL_RMS, f"{name}: max-abs {plain:.3e} scaled {err:.3e} rel-rms {rr:.3e}"


@pytest.mark.parametrize("name", PREFILL_GOLDENS)
def test_routes_bit_exact_and_forward_matches_reference(name):
    g = load(name)
    q, k, v = (bits_to_torch(g[x]) for x in ("q", "k", "v"))
    cu = cu_from_lens(g["lens"])
    out, lse, captured, _ = _run(q, k, v, cu, int(g["chunk"]), int(g["topk"]))
    if g["selected_stable"].shape[0]:
        assert torch.equal(captured["selected"], torch.from_numpy(g["selected_stable"]))
        assert np.array_equal(captured["filtered_chunk_indices"].numpy(), g["filtered"])
        assert np.array_equal(captured["cu_chunk"].numpy(), g["cu_chunk"])
        assert np.array_equal(captured["chunk_to_batch"].numpy(), g["chunk_to_batch"])
    else:
        assert not captured  # dense fallback: no sparse route
    _check_close("out", torch_to_f64(out), g["out"])
    if "lse" in g:
        np.testing.assert_allclose(torch_to_f64(lse), g["lse"], atol=5e-4, rtol=2e-5)


@pytest.mark.parametrize("name", PREFILL_GOLDENS + ROUTE_GOLDENS)
@pytest.mark.parametrize("precision", ["upstream", "fp32"])
def test_routes_bit_exact_under_both_route_precisions(name, precision):
    """Selection equal to the reference's own ROUTE_HOOK tensor for route_precision='upstream' (its default: chunk
    means rounded to bf16, src/moba_opt/grouped_attention.py:35,52) and 'fp32'.  The route-only fixtures have chunk
    sizes 40 and 24 (mean = FP32 sum / C, not a shift) and rows on which the two precisions choose differently."""
    g = load(name)
    q, k = (bits_to_torch(g[x]) for x in ("q", "k"))
    cu = cu_from_lens(g["lens"])
    _, _, captured, _ = _run(q, k, k, cu, int(g["chunk"]), int(g["topk"]), route_precision=precision)
    tag = "upstream" if precision == "upstream" else "stable"
    want = unpack_selected(g, tag) if name in ROUTE_GOLDENS else g[f"selected_{tag}"]
    if want.shape[0]:
        assert torch.equal(captured["selected"], torch.from_numpy(want))
    else:
        assert not captured


def test_default_config_routes_like_the_reference_default():
    """A caller that passes only chunk_size and topk gets route_precision='upstream', as in the reference."""
    import moba_opt
    import moba_opt.grouped_attention as ga
    g = load("r_upstream_mqa")
    q, k = (bits_to_torch(g[x]).cuda() for x in ("q", "k"))
    cu = torch.tensor(cu_from_lens(g["lens"]), dtype=torch.int32, device="cuda")
    captured = {}
    ga.ROUTE_HOOK = lambda **kw: captured.update(kw)
    try:
        moba_opt.run_impl("opt_gqa_cuda", q, k, k, cu, int(g["lens"].max()), {"chunk_size": int(g["chunk"]), "topk": int(g["topk"])})
    finally:
        ga.ROUTE_HOOK = None
    ga.check_status()
    assert torch.equal(captured["selected"], torch.from_numpy(unpack_selected(g, "upstream")))


def test_config1_routes_and_forward():
    g = load("config1")
    q, k, v, _ = config1_inputs()
    cu = np.array([0, 2048])
    out, lse, captured, _ = _run(q, k, v, cu, 256, 3)
    selected = np.unpackbits(g["selected_packed"])[:np.prod(g["selected_shape"])].reshape(g["selected_shape"]).astype(bool)
    assert np.array_equal(captured["selected"].numpy(), selected)
    rows = g["rows"]
    _check_close("out", torch_to_f64(out)[rows], g["out_rows"])
    np.testing.assert_allclose(torch_to_f64(lse)[rows], g["lse_rows"], atol=5e-4, rtol=2e-5)


@pytest.mark.parametrize("lens,hq,hkv,dim,chunk,topk", [
    ((700, 1300), 4, 2, 64, 256, 3),     # several 128-row tiles per chunk, partial tail chunks
    ((1024,), 8, 2, 128, 128, 5),        # chunk == tile, D = 128
    ((333,), 2, 1, 96, 48, 4),           # head_dim padded to 128, chunk not a multiple of 8
    ((2000,), 6, 1, 64, 500, 2),         # chunk not a multiple of the tile
    ((64, 64, 64), 4, 4, 32, 16, 17),    # widest supported topk
])
def test_forward_against_oracle_on_seeded_inputs(lens, hq, hkv, dim, chunk, topk):
    rng = torch.Generator().manual_seed(1234)
    total = sum(lens)
    q, k, v = [torch.randn(total, h, dim, generator=rng).bfloat16() for h in (hq, hkv, hkv)]
    cu = cu_from_lens(lens)
    out, lse, captured, _ = _run(q, k, v, cu, chunk, topk)
    qf, kf, vf = (torch_to_f64(t) for t in (q, k, v))
    r = mo.route_prefill(qf, kf, cu, chunk, topk)
    got = captured["selected"].numpy()
    diff_rows = (got != r["selected"]).any(axis=0).T          # [T,Hq]
    # an FP32 gate may only differ from the FP64 one where the decision margin is inside rounding
    bound = 64 * np.finfo(np.float32).eps * r["scale"]
    assert (r["margin"][diff_rows] <= bound[diff_rows]).all()
    assert diff_rows.mean() < 1e-3
    sel = mo.sel_from_selected(got, r["filtered"], r["sel"].shape[-1])
    ref = mo.attention_fixed_route(qf, kf, vf, cu, sel, chunk)
    _check_close("out", torch_to_f64(out), ref["out"])
    np.testing.assert_allclose(torch_to_f64(lse), ref["lse"], atol=2e-3, rtol=2e-5)


def test_dense_fallback_topk1_is_full_causal():
    rng = torch.Generator().manual_seed(7)
    lens = (300, 150)
    q, k, v = [torch.randn(450, h, 64, generator=rng).bfloat16() for h in (4, 2, 2)]
    cu = cu_from_lens(lens)
    out, lse, captured, _ = _run(q, k, v, cu, 64, 1)
    assert not captured
    qf, kf, vf = (torch_to_f64(t) for t in (q, k, v))
    ref = mo.attention_fixed_route(qf, kf, vf, cu, mo.dense_sel(cu, 64, 4), 64)
    _check_close("out", torch_to_f64(out), ref["out"])


def test_forward_is_bit_repeatable():
    rng = torch.Generator().manual_seed(99)
    q, k, v = [torch.randn(1024, h, 64, generator=rng).bfloat16() for h in (4, 2, 2)]
    cu = np.array([0, 1024])
    first, lse0, _, _ = _run(q, k, v, cu, 128, 4)
    for _ in range(5):
        again, lse1, _, _ = _run(q, k, v, cu, 128, 4)
        assert torch.equal(first, again) and torch.equal(lse0, lse1)


# --------------------------------------------------------------------------- gradients
@pytest.mark.parametrize("name", PREFILL_GOLDENS)
def test_gradients_match_reference(name):
    g = load(name)
    q, k, v, do = (bits_to_torch(g[x]) for x in ("q", "k", "v", "g"))
    cu = cu_from_lens(g["lens"])
    _, _, _, grads = _run(q, k, v, cu, int(g["chunk"]), int(g["topk"]), d_out=do)
    for key, got in zip(("dq", "dk", "dv"), grads):
        _check_close(key, torch_to_f64(got), g[key])


def test_config1_gradients():
    g = load("config1")
    q, k, v, do = config1_inputs()
    _, _, _, grads = _run(q, k, v, np.array([0, 2048]), 256, 3, d_out=do)
    rows = g["rows"]
    for key, got in zip(("dq", "dk", "dv"), grads):
        _check_close(key, torch_to_f64(got)[rows], g[f"{key}_rows"])
        np.testing.assert_allclose(torch_to_f64(got).sum(), g["sums"][2 + ("dq", "dk", "dv").index(key)],
                                   atol=2e-3 * g["abs_sums"][2 + ("dq", "dk", "dv").index(key)] ** 0.5 + 1.0)


@pytest.mark.parametrize("lens,hq,hkv,dim,chunk,topk", [
    ((700, 1300), 4, 2, 64, 256, 3),
    ((1024,), 8, 2, 128, 128, 5),
    ((333,), 2, 1, 96, 48, 4),
    ((2000,), 6, 1, 64, 500, 2),
    ((300, 150), 4, 2, 64, 64, 1),       # dense fallback
])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "fp16"])
def test_gradients_against_oracle_on_seeded_inputs(lens, hq, hkv, dim, chunk, topk, dtype):
    rng = torch.Generator().manual_seed(4321)
    total = sum(lens)
    q, k, v = [torch.randn(total, h, dim, generator=rng).to(dtype) for h in (hq, hkv, hkv)]
    do = torch.randn(total, hq, dim, generator=rng).to(dtype)
    cu = cu_from_lens(lens)
    out, lse, captured, grads = _run(q, k, v, cu, chunk, topk, d_out=do)
    qf, kf, vf, dof = (torch_to_f64(t) for t in (q, k, v, do))
    if topk == 1:
        sel = mo.dense_sel(cu, chunk, hq)
    else:
        r = mo.route_prefill(qf, kf, cu, chunk, topk)
        sel = mo.sel_from_selected(captured["selected"].numpy(), r["filtered"], r["sel"].shape[-1])
    ref = mo.attention_fixed_route(qf, kf, vf, cu, sel, chunk, d_out=dof)
    _check_close("out", torch_to_f64(out), ref["out"])
    for key, got in zip(("dq", "dk", "dv"), grads):
        _check_close(key, torch_to_f64(got), ref[key])


@pytest.mark.parametrize("lens,hq,hkv,dim,chunk,topk", [((1500, 800), 4, 2, 64, 256, 3), ((1024,), 8, 2, 128, 128, 5)])
def test_deterministic_backward_is_bit_repeatable(lens, hq, hkv, dim, chunk, topk):
    """deterministic_backward=True (the counterpart of deterministic=True in the reference's two backward calls,
    src/moba_opt/mixed_attention.py:185,220): dQ of a row is the sum of the contributions of many key blocks; summed in
    fixed point it has the same bits run after run, and it still meets the tolerance against the oracle."""
    rng = torch.Generator().manual_seed(77)
    total = sum(lens)
    q, k, v = [torch.randn(total, h, dim, generator=rng).bfloat16() for h in (hq, hkv, hkv)]
    do = torch.randn(total, hq, dim, generator=rng).bfloat16()
    cu = cu_from_lens(lens)
    _, _, captured, first = _run(q, k, v, cu, chunk, topk, d_out=do, deterministic_backward=True)
    for _ in range(20):
        _, _, _, again = _run(q, k, v, cu, chunk, topk, d_out=do, deterministic_backward=True)
        for a, b in zip(first, again):
            assert torch.equal(a, b)
    qf, kf, vf, dof = (torch_to_f64(t) for t in (q, k, v, do))
    r = mo.route_prefill(qf, kf, cu, chunk, topk)
    sel = mo.sel_from_selected(captured["selected"].numpy(), r["filtered"], r["sel"].shape[-1])
    ref = mo.attention_fixed_route(qf, kf, vf, cu, sel, chunk, d_out=dof)
    for key, got in zip(("dq", "dk", "dv"), first):
        _check_close(key, torch_to_f64(got), ref[key])
    _, _, _, plain = _run(q, k, v, cu, chunk, topk, d_out=do)
    assert torch.equal(plain[1], first[1]) and torch.equal(plain[2], first[2])      # dK, dV do not depend on the mode
    with pytest.raises(ValueError):
        _run(q, k, v, cu, chunk, topk, d_out=do, deterministic_backward=1)


def test_non_contiguous_inputs_and_sequence_isolation():
    """Strided q/k/v views give the same result, and rows of one sequence do not depend on another
    sequence's tokens (tests/test_attention_opt.py causal & sequence isolation in the reference)."""
    rng = torch.Generator().manual_seed(5)
    lens = (200, 184)
    total = sum(lens)
    qkv = torch.randn(total, 8, 64, generator=rng).bfloat16()       # fused [T, Hq+2*Hkv, D] projection
    q, k, v = qkv[:, :4], qkv[:, 4:6], qkv[:, 6:8]
    cu = cu_from_lens(lens)
    out_view, _, _, _ = _run(q, k, v, cu, 64, 3)
    out_cont, _, _, _ = _run(q.contiguous(), k.contiguous(), v.contiguous(), cu, 64, 3)
    assert torch.equal(out_view, out_cont)
    k2, v2 = k.clone(), v.clone()
    k2[200:] = torch.randn(184, 2, 64, generator=rng).bfloat16()
    v2[200:] = torch.randn(184, 2, 64, generator=rng).bfloat16()
    out_other, _, _, _ = _run(q.contiguous(), k2, v2, cu, 64, 3)
    assert torch.equal(out_other[:200], out_cont[:200])


def test_full_size_config2_properties():
    """BASELINE configs[1] at full size (4 x 32768 tokens, 14/2 heads, D=64, chunk 2048, topk 3), checked
    through properties that do not need the whole oracle: (a) sampled query rows of sequence 0 / KV group 0
    against the FP64 oracle under the kernel's own routes (output and dQ rows), and dK / dV of one whole 128-key
    block (the last block of chunk 14 of sequence 0: every query that attends it lies behind it in chunks 14 and
    15, so an oracle run over those rows gives the block's complete gradient); (b) the forward is
    bit-repeatable; (c) <Q, dQ> = <K, dK> per sequence (the loss depends on Q and K only through Q K^T,
    so the two inner products are the same sum of S * dS); (d) gradients are linear in dO; (e) another
    sequence's tokens do not change a sequence's rows."""
    lens, hq, hkv, dim, chunk, topk = (32768,) * 4, 14, 2, 64, 2048, 3
    total, G = sum(lens), hq // hkv
    rng = torch.Generator().manual_seed(2024)
    q, k, v = [(torch.randn(total, h, dim, generator=rng) * dim ** -0.5).bfloat16() for h in (hq, hkv, hkv)]
    do = torch.randn(total, hq, dim, generator=rng).bfloat16()
    cu = cu_from_lens(lens)
    out, lse, captured, grads = _run(q, k, v, cu, chunk, topk, d_out=do)
    out2, _, _, _ = _run(q, k, v, cu, chunk, topk)
    assert torch.equal(out, out2)                                                     # (b)
    dq, dk, dv = (g.float().cpu() for g in grads)
    qf32, kf32 = q.float(), k.float()
    for b in range(len(lens)):                                                        # (c)
        s, e = cu[b], cu[b + 1]
        lhs = float((qf32[s:e].double() * dq[s:e].double()).sum())
        rhs = float((kf32[s:e].double() * dk[s:e].double()).sum())
        scale_ref = float((qf32[s:e].double().abs() * dq[s:e].double().abs()).sum())
        assert abs(lhs - rhs) <= 2e-3 * scale_ref, (b, lhs, rhs, scale_ref)
    # (a) sampled rows of sequence 0, KV group 0
    L = lens[0]
    rows = np.concatenate([np.arange(c * chunk + 1000, c * chunk + 1064) for c in (0, 3, 15)])
    qs, ks, vs = (torch_to_f64(t[:L, :n]) for t, n in ((q, G), (k, 1), (v, 1)))
    sel = mo.sel_from_selected(captured["selected"].numpy()[:, :G, :L], captured["filtered_chunk_indices"].numpy(), topk - 1)
    ref = mo.attention_fixed_route(qs, ks, vs, np.array([0, L]), sel, chunk, d_out=torch_to_f64(do[rows, :G]), rows=rows,
                                   row_block=64)
    _check_close("out rows", torch_to_f64(out.cpu()[rows, :G]), ref["out"])
    _check_close("dq rows", dq[rows, :G].numpy(), ref["dq"][rows])
    lo, hi = 15 * chunk - 128, 15 * chunk
    rows = np.arange(lo, L)
    ref = mo.attention_fixed_route(qs, ks, vs, np.array([0, L]), sel, chunk, d_out=torch_to_f64(do[rows, :G]), rows=rows,
                                   row_block=256, key_range=(lo, hi))
    _check_close("dk block", dk[lo:hi, :1].numpy(), ref["dk"])
    _check_close("dv block", dv[lo:hi, :1].numpy(), ref["dv"])
    # (d) linearity in dO and (e) isolation, on the forward/backward of the same batch
    do2 = torch.randn(total, hq, dim, generator=rng).bfloat16()
    _, _, _, g2 = _run(q, k, v, cu, chunk, topk, d_out=do2)
    _, _, _, g12 = _run(q, k, v, cu, chunk, topk, d_out=(do.float() + do2.float()).bfloat16())
    for name, a1, a2, a12 in zip(("dq", "dk", "dv"), grads, g2, g12):
        lin = a1.float() + a2.float()
        err = (a12.float() - lin).abs().max().item() / max(1.0, lin.abs().max().item())
        assert err <= 3e-2 and rel_rms(a12.float().cpu().numpy(), lin.cpu().numpy()) <= 1e-2, (name, err)
    k3, v3 = k.clone(), v.clone()
    k3[cu[1]:] = (torch.randn(total - cu[1], hkv, dim, generator=rng) * dim ** -0.5).bfloat16()
    v3[cu[1]:] = (torch.randn(total - cu[1], hkv, dim, generator=rng) * dim ** -0.5).bfloat16()
    out3, _, _, _ = _run(q, k3, v3, cu, chunk, topk)
    assert torch.equal(out3[:cu[1]], out[:cu[1]])


def test_remembered_offsets_follow_in_place_changes_of_cu_seqlens():
    """The offsets of a cu_seqlens tensor are read from the device once and reused while the tensor's version counter
    stands; an in-place change must be seen by the next call (here: it makes the offsets invalid, then valid again
    with a different split, whose result must equal a fresh tensor's)."""
    import moba_opt
    g = torch.Generator().manual_seed(5)
    q, k, v = (torch.randn(96, h, 16, generator=g).bfloat16().cuda() for h in (4, 2, 2))
    cfg = {"chunk_size": 16, "topk": 2}
    cu = torch.tensor([0, 48, 96], dtype=torch.int32, device="cuda")
    first = moba_opt.run_impl("opt_gqa_cuda", q, k, v, cu, 48, cfg)
    assert torch.equal(first, moba_opt.run_impl("opt_gqa_cuda", q, k, v, cu, 48, cfg))
    cu[1] = 200
    with pytest.raises(ValueError):
        moba_opt.run_impl("opt_gqa_cuda", q, k, v, cu, 48, cfg)
    cu[1] = 32
    fresh = torch.tensor([0, 32, 96], dtype=torch.int32, device="cuda")
    assert torch.equal(moba_opt.run_impl("opt_gqa_cuda", q, k, v, cu, 64, cfg),
                       moba_opt.run_impl("opt_gqa_cuda", q, k, v, fresh, 64, cfg))
    assert not torch.equal(first, moba_opt.run_impl("opt_gqa_cuda", q, k, v, fresh, 64, cfg))
