"""GPU parity of the prefill path (routing, forward, backward) against the FP64 oracle and the
golden vectors produced by the reference.  Everything goes through the C ABI via moba_opt.

Tolerances (bf16 inputs, FP64 oracle under the kernel's own routes): max-abs <= 2e-2 and
rel-RMS <= 5e-3 for outputs and gradients; block selection bit-exact.
"""
import numpy as np
import pytest
import torch

from helpers import PREFILL_GOLDENS, bf16_bits_to_torch, config1_inputs, cu_from_lens, load, rel_rms, torch_to_f64
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
    err = np.abs(got - ref).max()
    rr = rel_rms(got, ref)
    assert err <= MAX_ABS and rr <= REL_RMS, f"{name}: max-abs {err:.3e} rel-rms {rr:.3e}"


@pytest.mark.parametrize("name", PREFILL_GOLDENS)
def test_routes_bit_exact_and_forward_matches_reference(name):
    g = load(name)
    q, k, v = (bf16_bits_to_torch(g[x]) for x in ("q", "k", "v"))
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
