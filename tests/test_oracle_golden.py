"""Pins the numpy oracle to outputs of the reference's own Python code (tests/golden/*.npz)."""
import numpy as np
import pytest

from oracle import moba_oracle as mo
from helpers import (DECODE_GOLDENS, PREFILL_GOLDENS, ROUTE_GOLDENS, bits_to_f64, config1_inputs, cu_from_lens, load,
                     torch_to_f64, unpack_selected)


@pytest.mark.parametrize("name", PREFILL_GOLDENS)
def test_chunk_metadata_matches_reference(name):
    g = load(name)
    cu_chunk, chunk_to_batch, filtered = mo.calc_chunks(cu_from_lens(g["lens"]), int(g["chunk"]))
    assert np.array_equal(cu_chunk, g["cu_chunk"])
    assert np.array_equal(chunk_to_batch, g["chunk_to_batch"])
    assert np.array_equal(filtered, g["filtered"])


@pytest.mark.parametrize("name", PREFILL_GOLDENS)
def test_route_matches_reference_bit_exact(name):
    g = load(name)
    q, k = bits_to_f64(g["q"]), bits_to_f64(g["k"])
    r = mo.route_prefill(q, k, cu_from_lens(g["lens"]), int(g["chunk"]), int(g["topk"]))
    assert r["selected"].shape == g["selected_stable"].shape
    # The reference evaluates the gate in FP32; rows whose decision margin is inside an FP32
    # rounding bound may legitimately differ.  There must be none in these fixtures.
    assert np.array_equal(r["selected"], g["selected_stable"])
    assert np.array_equal(r["selected"], g["selected_topk"])  # no exact ties: torch.topk picks the same set
    R = r["sel"].shape[-1]
    assert np.array_equal(mo.sel_from_selected(g["selected_stable"], g["filtered"], R), r["sel"])
    back = mo.selected_from_sel(r["sel"], g["filtered"], q.shape[0], q.shape[1]) if R else r["selected"]
    assert np.array_equal(back, g["selected_stable"])


@pytest.mark.parametrize("name", PREFILL_GOLDENS + ROUTE_GOLDENS)
def test_upstream_route_matches_reference_bit_exact(name):
    """route_precision='upstream' (the reference's default, src/moba_opt/grouped_attention.py:35,52): chunk means
    rounded to the input format before the gate.  The route-only fixtures are shaped so that this changes some rows."""
    g = load(name)
    q, k = bits_to_f64(g["q"]), bits_to_f64(g["k"])
    cu = cu_from_lens(g["lens"])
    rounding = mo.fp16_round if str(g.get("dtype", "")) == "float16" else mo.bf16_round     # to the format of the inputs
    r = mo.route_prefill(q, k, cu, int(g["chunk"]), int(g["topk"]), mean_rounding=rounding)
    if name in ROUTE_GOLDENS:
        want, fp32 = unpack_selected(g, "upstream"), unpack_selected(g, "stable")
        assert (want != fp32).any()                                  # the fixture does discriminate the two precisions
        assert np.array_equal(mo.route_prefill(q, k, cu, int(g["chunk"]), int(g["topk"]))["selected"], fp32)
    else:
        want = g["selected_upstream"]
        assert np.array_equal(g["selected_upstream_topk"], want)     # no exact ties: torch.topk picks the same set
    assert np.array_equal(r["selected"], want)


@pytest.mark.parametrize("name", PREFILL_GOLDENS)
def test_attention_and_gradients_match_reference(name):
    g = load(name)
    q, k, v, do = (bits_to_f64(g[x]) for x in ("q", "k", "v", "g"))
    cu = cu_from_lens(g["lens"])
    R = min(int(g["topk"]) - 1, g["filtered"].size)
    sel = mo.sel_from_selected(g["selected_stable"], g["filtered"], R)
    res = mo.attention_fixed_route(q, k, v, cu, sel, int(g["chunk"]), d_out=do, row_block=50)
    for key in ("out", "dq", "dk", "dv"):
        np.testing.assert_allclose(res[key], g[key], rtol=2e-6, atol=2e-6, err_msg=key)
    if "lse" in g:
        np.testing.assert_allclose(res["lse"], g["lse"], rtol=1e-6, atol=1e-6)
        np.testing.assert_allclose(res["out"], g["out_fixed"], rtol=2e-6, atol=2e-6)
    # forward-only evaluation of a row subset agrees with the full evaluation
    rows = np.arange(0, q.shape[0], 7)
    sub = mo.attention_fixed_route(q, k, v, cu, sel, int(g["chunk"]), rows=rows)
    np.testing.assert_allclose(sub["out"], res["out"][rows], rtol=1e-12, atol=1e-12)


def test_config1_matches_reference():
    g = load("config1")
    qt, kt, vt, gt = config1_inputs()
    q, k, v, do = (torch_to_f64(t) for t in (qt, kt, vt, gt))
    cu = np.array([0, 2048])
    r = mo.route_prefill(q, k, cu, 256, 3)
    selected = np.unpackbits(g["selected_packed"])[:np.prod(g["selected_shape"])].reshape(g["selected_shape"]).astype(bool)
    assert np.array_equal(r["selected"], selected)
    assert int(selected.sum()) == 26624
    res = mo.attention_fixed_route(q, k, v, cu, r["sel"], 256, d_out=do)
    rows = g["rows"]
    for key in ("out", "dq", "dk", "dv"):
        np.testing.assert_allclose(res[key][rows], g[f"{key}_rows"], rtol=1e-9, atol=1e-9, err_msg=key)
    np.testing.assert_allclose(res["lse"][rows], g["lse_rows"], rtol=1e-10, atol=1e-10)
    sums = np.array([res[x].sum() for x in ("out", "lse", "dq", "dk", "dv")])
    np.testing.assert_allclose(sums, g["sums"], rtol=1e-7, atol=1e-6)
    assert float(g["fixed_vs_grouped"]) < 1e-12
    assert mo.attended_pairs(cu, 256, 3) * 8 == 8_921_088  # attended (q,k) pairs x heads at config 1


@pytest.mark.parametrize("name", DECODE_GOLDENS)
def test_decode_attention_matches_reference(name):
    g = load(name)
    n = len(g["lengths"])
    keys = [bits_to_f64(g[f"k{i}"]) for i in range(n)]
    values = [bits_to_f64(g[f"v{i}"]) for i in range(n)]
    q = bits_to_f64(g["q"])
    ids, pos = list(range(n)), [int(x) - 1 for x in g["lengths"]]
    out, lse = mo.decode_attend(q, keys, values, ids, pos, int(g["chunk"]), g["selected"])
    np.testing.assert_allclose(out, g["out_sparse"], rtol=1e-10, atol=1e-12)
    np.testing.assert_allclose(lse, g["lse_sparse"], rtol=1e-10, atol=1e-12)
    out, lse = mo.decode_attend(q, keys, values, ids, pos, int(g["chunk"]), None)
    np.testing.assert_allclose(out, g["out_dense"], rtol=1e-10, atol=1e-12)
    np.testing.assert_allclose(lse, g["lse_dense"], rtol=1e-10, atol=1e-12)


def test_merge_matches_reference():
    g = load("merge")
    P = g["self_out"].shape[0]
    out = np.empty_like(g["out"])
    lse = np.empty_like(g["lse"])
    for p in range(P):
        rows = np.nonzero(g["mapping"] == p)[0]
        o, l = mo.merge_branches([g["self_out"][p:p + 1]] + [g["remote_out"][m:m + 1] for m in rows],
                                 [g["self_lse"][p:p + 1]] + [g["remote_lse"][m:m + 1] for m in rows])
        out[p], lse[p] = o[0], l[0]
    np.testing.assert_allclose(out, g["out"], rtol=1e-12, atol=1e-12)
    np.testing.assert_allclose(lse, g["lse"], rtol=1e-12, atol=1e-12)


# ---- closed-form known answers the reference's tests use (tests/test_cache_layout.py:83-98,
# tests/test_paged_decode.py:146-159, tests/test_stable_routes.py:39-49)
def test_decode_uniform_attention_known_answer():
    n, d = 11, 8
    keys = [np.zeros((n, 1, d))]
    values = [np.arange(n * d, dtype=np.float64).reshape(n, 1, d)]
    out, lse = mo.decode_attend(np.ones((1, 2, d)), keys, values, [0], [n - 1], 4, None)
    np.testing.assert_allclose(out[0, 0], values[0][:, 0].mean(0))
    np.testing.assert_allclose(lse, np.log(n))


def test_decode_route_known_answer_and_tie_rule():
    # three complete chunks of 4 tokens + one partial; means are unit vectors scaled per chunk
    means = np.zeros((3, 1, 4))
    means[0, 0, 0], means[1, 0, 0], means[2, 0, 0] = 1.0, 3.0, 2.0
    q = np.zeros((1, 2, 4))
    q[0, 0, 0], q[0, 1, 0] = 1.0, -1.0   # head 1 reverses the ranking
    r = mo.decode_route(q, [means], [0], [13], 4, 3)
    assert r["selected"][0, 0].tolist() == [3, 1, 2]
    assert r["selected"][0, 1].tolist() == [3, 0, 2]
    tie = np.zeros((3, 1, 4))
    r = mo.decode_route(q, [tie], [0], [13], 4, 3)
    assert r["selected"][0, 0].tolist() == [3, 0, 1]          # exact ties -> lowest chunk first
    r = mo.decode_route(q, [means], [0], [7], 4, 4)           # only chunk 0 is complete before pos 7
    assert r["selected"][0, 0].tolist() == [1, 0, -1, -1]


def test_dense_sel_is_dense_causal():
    rng = np.random.default_rng(0)
    lens = (23, 40)
    cu = cu_from_lens(lens)
    q, k, v = rng.standard_normal((63, 4, 8)), rng.standard_normal((63, 2, 8)), rng.standard_normal((63, 2, 8))
    sel = mo.dense_sel(cu, 16, 4)
    got = mo.attention_fixed_route(q, k, v, cu, sel, 16)["out"]
    for b in range(2):
        s0, s1 = cu[b], cu[b + 1]
        for h in range(4):
            logits = q[s0:s1, h] @ k[s0:s1, h // 2].T * 8 ** -0.5
            logits = np.where(np.tril(np.ones_like(logits, dtype=bool)), logits, -np.inf)
            p = np.exp(logits - logits.max(1, keepdims=True))
            ref = (p / p.sum(1, keepdims=True)) @ v[s0:s1, h // 2]
            np.testing.assert_allclose(got[s0:s1, h], ref, rtol=1e-12, atol=1e-12)


def test_bf16_round_matches_torch():
    import torch
    x = torch.randn(4096, generator=torch.Generator().manual_seed(5)) * 37
    np.testing.assert_array_equal(mo.bf16_round(x.numpy()), x.bfloat16().float().numpy().astype(np.float64))
