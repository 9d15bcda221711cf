"""Standalone merge operator against the reference's golden vectors and the FP64 oracle.  The cases follow
the reference's merge tests (tests/test_merge_cuda.py:27-150, tests/test_merge_coverage.py:12-43): fp32 atol
1e-5 / rtol 1e-4, bf16 2e-2, identity without remote rows (bit exact), extreme LSE values without NaN, odd
row counts, contribution counts that are not powers of two, capacity overflow and bad mappings rejected,
every head dimension 8..256 step 8, bit-repeatable results."""
import numpy as np
import pytest
import torch

from helpers import load
from oracle import moba_oracle as mo

pytestmark = pytest.mark.gpu


def _oracle(self_out, self_lse, remote_out, remote_lse, mapping):
    P, D = self_out.shape[0] * self_out.shape[1], self_out.shape[2]
    so = self_out.double().cpu().numpy().reshape(P, D)
    sl = self_lse.double().cpu().numpy().reshape(P)
    ro = remote_out.double().cpu().numpy().reshape(-1, D)
    rl = remote_lse.double().cpu().numpy().reshape(-1)
    mp = mapping.cpu().numpy()
    out, lse = np.empty((P, D)), np.empty(P)
    for p in range(P):
        rows = np.nonzero(mp == p)[0]
        o, l = mo.merge_branches([so[p:p + 1]] + [ro[m:m + 1] for m in rows], [sl[p:p + 1]] + [rl[m:m + 1] for m in rows])
        out[p], lse[p] = o[0], l[0]
    return out.reshape(self_out.shape), lse.reshape(self_lse.shape)


def _case(T, H, D, M, seed, dtype=torch.float32, kcap=None):
    g = torch.Generator().manual_seed(seed)
    so = torch.randn(T, H, D, generator=g).to("cuda", dtype)
    sl = torch.randn(T, H, generator=g).cuda() * 3
    ro = torch.randn(M, 1, D, generator=g).to("cuda", dtype)
    rl = torch.randn(M, generator=g).cuda() * 3
    P = T * H
    if kcap is None:
        mp = torch.randint(0, P, (M,), generator=g)
    else:  # at most kcap contributions per row
        mp = torch.cat([torch.randperm(P, generator=g) for _ in range(kcap)])[:M]
    return so, sl, ro, rl, mp.cuda()


def test_matches_reference_golden():
    from moba_opt.ops.merge_cuda import merge_forward_cuda
    g = load("merge")
    P, D = g["self_out"].shape
    so = torch.from_numpy(g["self_out"]).cuda().view(P, 1, D)
    out, lse = merge_forward_cuda(so, torch.from_numpy(g["self_lse"]).cuda().view(P, 1), torch.from_numpy(g["remote_out"]).cuda(),
                                  torch.from_numpy(g["remote_lse"]).cuda(), torch.from_numpy(g["mapping"]).cuda())
    np.testing.assert_allclose(out.double().cpu().numpy().reshape(P, D), g["out"], atol=1e-5, rtol=1e-4)
    np.testing.assert_allclose(lse.double().cpu().numpy().reshape(P), g["lse"], atol=1e-5, rtol=1e-4)


@pytest.mark.parametrize("T,H,D,M,dtype", [(37, 3, 64, 200, torch.float32), (128, 4, 128, 900, torch.bfloat16),
                                           (5, 1, 8, 0, torch.float32), (61, 2, 40, 333, torch.bfloat16),
                                           (128, 4, 128, 900, torch.float16), (61, 2, 40, 333, torch.float16),
                                           (33, 2, 12, 100, torch.float16)])
def test_against_oracle(T, H, D, M, dtype):
    from moba_opt.ops.merge_cuda import merge_forward_cuda
    so, sl, ro, rl, mp = _case(T, H, D, M, 7 + M, dtype, kcap=5)
    out, lse = merge_forward_cuda(so, sl, ro, rl, mp, deterministic=True)
    want, want_lse = _oracle(so, sl, ro, rl, mp)
    tol = dict(atol=1e-5, rtol=1e-4) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    np.testing.assert_allclose(out.double().cpu().numpy(), want, **tol)
    np.testing.assert_allclose(lse.double().cpu().numpy(), want_lse, atol=1e-5, rtol=1e-5)
    if M == 0:  # no remote rows: the self branch comes back bit for bit
        assert torch.equal(out, so) and torch.equal(lse, sl)


@pytest.mark.parametrize("D", list(range(8, 257, 8)))
def test_every_head_dimension(D):
    from moba_opt.ops.merge_cuda import merge_forward_cuda
    so, sl, ro, rl, mp = _case(9, 2, D, 40, D, torch.bfloat16, kcap=3)
    out, lse = merge_forward_cuda(so, sl, ro, rl, mp)
    want, want_lse = _oracle(so, sl, ro, rl, mp)
    np.testing.assert_allclose(out.double().cpu().numpy(), want, atol=2e-2, rtol=2e-2)
    np.testing.assert_allclose(lse.double().cpu().numpy(), want_lse, atol=1e-5, rtol=1e-5)


def test_extreme_lse_values_give_no_nan():
    from moba_opt.ops.merge_cuda import merge_forward_cuda
    so, sl, ro, rl, mp = _case(16, 2, 32, 64, 3, kcap=2)
    sl[0, 0], sl[1, 0], sl[2, 0] = 1e30, -1e30, float("-inf")
    rl[:8] = torch.tensor([1e30, -1e30, float("-inf"), 0.0, 1e30, -1e30, 5.0, -5.0]).cuda()
    out, lse = merge_forward_cuda(so, sl, ro, rl, mp)
    assert not torch.isnan(out).any() and not torch.isnan(lse).any()
    want, want_lse = _oracle(so, sl, ro, rl, mp)
    ok = np.isfinite(want).all(axis=-1) & np.isfinite(want_lse)
    np.testing.assert_allclose(out.double().cpu().numpy()[ok], want[ok], atol=1e-5, rtol=1e-4)


def test_capacity_overflow_and_bad_mapping_are_rejected():
    from moba_opt.ops.merge_cuda import merge_forward_cuda
    so, sl, ro, rl, mp = _case(4, 1, 16, 12, 11)
    mp[:] = 2  # twelve contributions for one row
    with pytest.raises(RuntimeError):
        merge_forward_cuda(so, sl, ro, rl, mp, kmax=8)
    out, _ = merge_forward_cuda(so, sl, ro, rl, mp)  # kmax derived from the mapping: fits
    assert torch.isfinite(out).all()
    bad = mp.clone(); bad[3] = 4
    with pytest.raises(ValueError):
        merge_forward_cuda(so, sl, ro, rl, bad)
    with pytest.raises(ValueError):
        merge_forward_cuda(so, sl, ro, rl, bad, kmax=12)
    with pytest.raises(ValueError):
        merge_forward_cuda(so, sl, ro, rl, mp.float())
    with pytest.raises(ValueError):
        merge_forward_cuda(so, sl, ro, rl, mp, deterministic=1)


def test_bit_repeatable():
    from moba_opt.ops.merge_cuda import merge_forward_cuda
    so, sl, ro, rl, mp = _case(257, 3, 64, 3000, 5, torch.bfloat16, kcap=7)
    first = merge_forward_cuda(so, sl, ro, rl, mp, deterministic=True)
    for _ in range(20):
        again = merge_forward_cuda(so, sl, ro, rl, mp, deterministic=True)
        assert torch.equal(first[0], again[0]) and torch.equal(first[1], again[1])


def test_legacy_names_run_the_same_engine():
    import moba_opt
    g = torch.Generator().manual_seed(1)
    q, k, v = [torch.randn(600, 4, 64, generator=g).bfloat16().cuda() for _ in range(3)]
    cu = torch.tensor([0, 600], dtype=torch.int32, device="cuda")
    cfg = {"chunk_size": 64, "topk": 3}
    ref = moba_opt.run_impl("opt_gqa_cuda", q, k, v, cu, 600, cfg)
    for name in ("opt_merge_cuda", "opt_merge_atomic"):
        assert torch.equal(moba_opt.run_impl(name, q, k, v, cu, 600, cfg), ref)
    with pytest.raises(ValueError):
        moba_opt.run_impl("opt_merge_cuda", q, k[:, :2], v[:, :2], cu, 600, cfg)


@pytest.mark.parametrize("heads,kv_heads,dim,chunk,topk,lens", [(8, 2, 64, 64, 3, (300, 212)), (4, 4, 128, 128, 4, (700,)), (6, 1, 32, 16, 9, (200,))])
def test_merge_stage_fixture_of_the_prefill_forward(heads, kv_heads, dim, chunk, topk, lens):
    """The merge-stage payload of moba_opt.diagnostic (the counterpart of the reference's MERGE_HOOK dump,
    scripts/dump_merge_fixtures.py:29-60): the self branch and the per-slot remote rows it lists, merged by the
    standalone operator and by the FP64 oracle, give the output and LSE the fused forward returned - which pins the
    epilogue merge of the forward kernel as an operator of its own."""
    from moba_opt import diagnostic
    from moba_opt.ops.merge_cuda import merge_forward_cuda
    payload = diagnostic.dump_merge_fixture(sum(lens), heads, kv_heads, dim, chunk, topk, seq_lens=lens, seed=5)
    inp, exp = payload["inputs"], payload["expected"]
    total = sum(lens)
    assert inp["self_out"].shape == (total, heads, dim) and inp["remote_out"].shape[1:] == (1, dim)
    counts = torch.bincount(inp["mapping"], minlength=total * heads)
    per_row = np.concatenate([np.minimum(topk - 1, np.arange(n) // chunk) for n in lens])      # selected chunks per token
    assert torch.equal(counts.reshape(total, heads), torch.from_numpy(per_row)[:, None].expand(total, heads))
    want, want_lse = _oracle(inp["self_out"], inp["self_lse"], inp["remote_out"], inp["remote_lse"], inp["mapping"])
    np.testing.assert_allclose(exp["output"].double().numpy(), want, atol=2e-2, rtol=2e-2)
    np.testing.assert_allclose(exp["mixed_lse"].double().numpy(), want_lse, atol=2e-3, rtol=2e-5)
    dev = {k_: v_.cuda() for k_, v_ in inp.items()}
    out, lse = merge_forward_cuda(dev["self_out"], dev["self_lse"], dev["remote_out"], dev["remote_lse"], dev["mapping"])
    np.testing.assert_allclose(out.double().cpu().numpy(), exp["output"].double().numpy(), atol=2e-2, rtol=2e-2)
    np.testing.assert_allclose(lse.double().cpu().numpy(), exp["mixed_lse"].double().numpy(), atol=2e-3, rtol=2e-5)
    # the hook form: same phases, same tensor names as the reference's diagnostic forward
    seen = {}
    diagnostic.MERGE_HOOK = lambda phase, tensors: seen.__setitem__(phase, sorted(tensors))
    try:
        q = torch.randn(64, 4, 32, generator=torch.Generator().manual_seed(1)).bfloat16().cuda()
        diagnostic.moba_attn_varlen(q, q, q, torch.tensor([0, 64], dtype=torch.int32, device="cuda"), 64, 16, 3)
    finally:
        diagnostic.MERGE_HOOK = None
    assert seen == {"inputs": ["mapping", "remote_lse", "remote_out", "self_lse", "self_out"], "outputs": ["mixed_lse", "output"]}
