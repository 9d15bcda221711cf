"""The decode path against the reference's own GPU decode, on the same inputs, on the same machine.

The reference's cache and prepared decode (src/moba_opt/kv_cache.py, prepared_decode.py over the Triton kernels of
ops/paged_decode.py and ops/prepared_decode.py) need only torch and triton, so oracle/make_ref.py can put an unmodified
copy of those five files under the git-ignored oracle/_ref/ and they run on the GPU box.  This is what pins the decode
routing and the chunk means to the reference itself rather than to closed-form answers: same appends, same queries,
then chunk means (at most one bf16 ulp apart), block selection (equal as sets per head; a differing head must have a
decision margin inside FP32 rounding), outputs and LSE (bf16: atol = rtol = 0.02, LSE atol 5e-4 - the reference's own
test tolerances, tests/test_paged_decode.py:56-60) for eager attends and for prepared steps replayed from CUDA graphs.
Skipped where oracle/_ref is absent (make_ref runs wherever a checkout of the reference is present at build time).
"""
import numpy as np
import pytest
import torch

from helpers import torch_to_f64
from oracle import moba_oracle as mo
from oracle.make_ref import load_ref_decode

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref():
    mods = load_ref_decode()
    if mods is None:
        pytest.skip("the reference's decode modules are not under oracle/_ref (or triton is missing)")
    return mods


def rand(shape, seed, dtype=torch.bfloat16):
    return torch.randn(shape, generator=torch.Generator().manual_seed(seed)).to("cuda", dtype)


def _same_routes(ours, theirs, q, means, positions, chunk, hk):
    """Per (row, head): True where both picked the same chunks; a differing head must be a near tie in FP64."""
    a, b = ours.cpu().numpy(), theirs.cpu().numpy()
    assert a.shape == b.shape and (a[:, :, 0] == b[:, :, 0]).all()
    same = (np.sort(a[:, :, 1:], axis=-1) == np.sort(b[:, :, 1:], axis=-1)).all(axis=-1)
    qf = torch_to_f64(q)
    G = q.shape[1] // hk
    for row, head in zip(*np.nonzero(~same)):
        history = positions[row] // chunk
        m = torch_to_f64(means[row][:history, head // G])
        scores = np.sort(m @ qf[row, head])[::-1]
        k = (a[row, head, 1:] >= 0).sum()
        bound = 64 * np.finfo(np.float32).eps * float((np.abs(m) @ np.abs(qf[row, head])).max())
        assert scores[k - 1] - scores[k] <= bound, (row, head)
    return same


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "fp16"])
@pytest.mark.parametrize("hq,hk,dim,page,chunk,topk,lens", [
    (12, 2, 128, 48, 256, 4, (1000, 3000, 517)),
    (8, 8, 64, 16, 128, 3, (700,)),
    (14, 2, 64, 7, 64, 9, (333, 90, 1200)),
    (32, 8, 128, 16, 1024, 4, (5000, 2047)),
])
def test_eager_attend_matches_the_reference_cache(ref, hq, hk, dim, page, chunk, topk, lens, dtype):
    from moba_opt import PagedKVCache
    import moba_opt.grouped_attention as ga
    from functools import partial
    rand = partial(globals()["rand"], dtype=dtype)
    ulp = 2.0 ** -10 if dtype == torch.float16 else 2.0 ** -7
    theirs_mod, _ = ref
    n, cap = len(lens), max(lens) + 8
    mine = PagedKVCache(n, cap, hk, dim, page_size=page, chunk_size=chunk, dtype=dtype)
    theirs = theirs_mod.PagedKVCache(n, cap, hk, dim, page_size=page, chunk_size=chunk, dtype=dtype)
    k, v = rand((sum(lens), hk, dim), 11), rand((sum(lens), hk, dim), 12)
    cu = [0] + [int(x) for x in np.cumsum(lens)]
    for cache in (mine, theirs):
        cache.append(k, v, sequence_ids=list(range(n)), cu_seqlens=cu)
    assert mine.lengths == theirs.lengths and mine.page_table == theirs.page_table
    for sid, length in enumerate(lens):
        closed = length // chunk
        if closed:
            a, b = mine._means[sid, :closed].float(), theirs._means[sid, :closed].float()
            assert ((a - b).abs() <= ulp * b.abs() + 1e-7).all()          # one ulp of the format at most
    ids = list(range(n)) + [0]
    positions = [length - 1 for length in lens] + [min(lens[0] - 1, 3 * chunk + 1)]
    q = rand((len(ids), hq, dim), 13)
    got = mine.attend(q, sequence_ids=ids, positions=positions, topk=topk)
    want = theirs.attend(q, sequence_ids=ids, positions=positions, topk=topk)
    ga.check_status()
    same = _same_routes(got.selected_blocks, want.selected_blocks, q, [mine._means[s] for s in ids], positions, chunk, hk)
    assert same.mean() > 0.95
    torch.testing.assert_close(got.output[torch.from_numpy(same)], want.output[torch.from_numpy(same)], atol=0.02, rtol=0.02)
    torch.testing.assert_close(got.lse[torch.from_numpy(same)], want.lse[torch.from_numpy(same)], atol=5e-4, rtol=2e-5)
    got, want = (c.attend(q, sequence_ids=ids, positions=positions, mode="dense") for c in (mine, theirs))
    torch.testing.assert_close(got.output, want.output, atol=0.02, rtol=0.02)
    torch.testing.assert_close(got.lse, want.lse, atol=5e-4, rtol=2e-5)


@pytest.mark.parametrize("graph", [False, True])
def test_prepared_steps_match_the_reference_plan(ref, graph):
    from moba_opt import PagedKVCache
    import moba_opt.grouped_attention as ga
    theirs_mod, _ = ref
    hq, hk, dim, page, chunk, topk, lens = 12, 2, 128, 48, 64, 4, (500, 130, 64)
    n = len(lens)
    caches = [cls(n, 640, hk, dim, page_size=page, chunk_size=chunk) for cls in (PagedKVCache, theirs_mod.PagedKVCache)]
    k, v = rand((sum(lens), hk, dim), 21), rand((sum(lens), hk, dim), 22)
    for cache in caches:
        cache.append(k, v, sequence_ids=list(range(n)), cu_seqlens=[0] + [int(x) for x in np.cumsum(lens)])
    plans = [c.prepare_decode(list(range(n)), hq, topk=topk, stable_routes=True) for c in caches]
    try:
        if graph:
            for p in plans:
                p.capture("step")
        for step in range(chunk + 3):                       # crosses a chunk boundary for every sequence at some step
            q, kn, vn = rand((n, hq, dim), 100 + step), rand((n, hk, dim), 200 + step), rand((n, hk, dim), 300 + step)
            got, want = (p.step(q, kn, vn, use_graph=graph) for p in plans)
            ga.check_status()
            assert got.positions == want.positions
            same = _same_routes(got.selected_blocks, want.selected_blocks, q, [caches[0]._means[s] for s in range(n)],
                                list(got.positions), chunk, hk)
            mask = torch.from_numpy(same)
            torch.testing.assert_close(got.output[mask], want.output[mask], atol=0.02, rtol=0.02)
            torch.testing.assert_close(got.lse[mask], want.lse[mask], atol=5e-4, rtol=2e-5)
    finally:
        for p in plans:
            p.close()
    assert caches[0].lengths == caches[1].lengths and caches[0].page_table == caches[1].page_table
    for sid in range(n):
        closed = caches[0].lengths[sid] // chunk
        a, b = caches[0]._means[sid, :closed].float(), caches[1]._means[sid, :closed].float()
        assert ((a - b).abs() <= 2.0 ** -7 * b.abs() + 1e-30).all()
