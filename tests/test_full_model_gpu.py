"""Full-model session (examples/full_qwen2.py of this package) on a small random Qwen2-architecture model: the dense
session against the Hugging Face forward of the same weights, graph backends against eager (bit for bit), the
in-graph greedy loop against a host-driven one, decode against a fresh prefill of the extended prompt, life-cycle
errors.  Logit tolerances (bf16 model): relative L2 <= 2e-2 against an independent implementation."""
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

sys.path.insert(0, str(Path(__file__).resolve().parents[1] / "moba-merge-cuda_b200" / "examples"))


@pytest.fixture(scope="module")
def model():
    from full_qwen2 import random_qwen2
    return random_qwen2(hidden=128, layers=3, heads=4, kv_heads=2, ffn=256, vocab=300, max_positions=512, seed=3)


def _rel_l2(a, b):
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-12))


def _ids(n, seed=0, vocab=300):
    return torch.randint(0, vocab, (1, n), generator=torch.Generator().manual_seed(seed)).cuda()


def test_dense_session_matches_hf_forward(model):
    from full_qwen2 import FullQwen2Session
    ids = _ids(70)
    with torch.no_grad():
        want = model(ids).logits[0].float()
    with FullQwen2Session(model, 128, mode="dense", chunk=16, page=8) as s:
        got = s.prefill(ids[:, :50])
        assert _rel_l2(got[0].float(), want[49]) <= 2e-2
        s.prepare()
        for i in range(50, 70):
            got = s.step(int(ids[0, i]))
            assert _rel_l2(got[0].float(), want[i]) <= 2e-2, i


@pytest.mark.parametrize("backend", ["attention_graph", "model_graph"])
def test_graph_backends_equal_eager_bit_for_bit(model, backend):
    from full_qwen2 import FullQwen2Session
    ids = _ids(100, seed=1)
    kw = dict(mode="moba", chunk=16, topk=3, page=8, dense_layers=(1,), stable_routes=True)
    logits = {}
    for name in ("eager", backend):
        with FullQwen2Session(model, 160, backend=name, **kw) as s:
            s.prefill(ids[:, :90])
            s.prepare()
            logits[name] = [s.step(int(ids[0, i])).clone() for i in range(90, 100)]
    for a, b in zip(logits["eager"], logits[backend]):
        assert torch.equal(a, b)


def test_in_graph_greedy_loop_matches_host_driven_greedy(model):
    from full_qwen2 import FullQwen2Session
    ids = _ids(64, seed=2)
    kw = dict(mode="moba", chunk=16, topk=3, page=8, stable_routes=True)
    with FullQwen2Session(model, 128, backend="model_graph", **kw) as s:
        s.prefill(ids)
        s.prepare()
        fast = s.generate(24)
    with FullQwen2Session(model, 128, backend="eager", **kw) as s:
        token = int(s.prefill(ids).argmax(-1))
        s.prepare()
        slow = []
        for _ in range(24):
            slow.append(token)
            token = int(s.step(token).argmax(-1))
    assert fast.tolist() == slow


def test_decode_step_agrees_with_prefill_of_the_extended_prompt(model):
    from full_qwen2 import FullQwen2Session
    ids = _ids(97, seed=4)
    kw = dict(mode="moba", chunk=16, topk=3, page=8, stable_routes=True)
    with FullQwen2Session(model, 160, **kw) as s:
        s.prefill(ids[:, :96])
        s.prepare()
        stepped = s.step(int(ids[0, 96]))[0].float()
    with FullQwen2Session(model, 160, **kw) as s:
        fresh = s.prefill(ids)[0].float()
    assert _rel_l2(stepped, fresh) <= 3e-2


def test_every_chunk_selected_is_the_dense_model(model):
    from full_qwen2 import FullQwen2Session
    ids = _ids(60, seed=5)
    out = []
    for kw in (dict(mode="dense"), dict(mode="moba", topk=8)):      # 128 / 16 = 8 chunks <= topk
        with FullQwen2Session(model, 128, chunk=16, page=8, **kw) as s:
            out.append(s.prefill(ids).clone())
    assert torch.equal(out[0], out[1])


def test_life_cycle_errors(model):
    from full_qwen2 import FullQwen2Session
    ids = _ids(20, seed=6)
    with pytest.raises(ValueError):
        FullQwen2Session(model, 64, mode="sparse")
    with pytest.raises(ValueError):
        FullQwen2Session(model, 64, backend="graph")
    with pytest.raises(ValueError):
        FullQwen2Session(model, 64, dense_layers=(7,))
    s = FullQwen2Session(model, 24, mode="moba", chunk=8, topk=2, page=4)
    with pytest.raises(ValueError):
        s.prepare()                       # nothing prefilled yet
    with pytest.raises(ValueError):
        s.prefill(_ids(24))               # prompt must stay below the capacity
    s.prefill(ids)
    with pytest.raises(ValueError):
        s.step(1)                         # prepare first
    s.prepare()
    with pytest.raises(ValueError):
        s.step(300)                       # not a token of the vocabulary
    for i in range(4):
        s.step(i)
    with pytest.raises(ValueError):
        s.step(5)                         # capacity 24 reached: rejected before anything is modified
    s.close()
    with pytest.raises(ValueError):
        s.step(1)


def test_fused_glue_step_agrees_with_the_module_by_module_step(model):
    from full_qwen2 import FullQwen2Session
    ids = _ids(80, seed=7)
    kw = dict(mode="moba", chunk=16, topk=3, page=8, stable_routes=True)
    logits = {}
    for fused in (False, True):
        with FullQwen2Session(model, 128, fused_glue=fused, **kw) as s:
            assert s.fused_glue == fused
            s.prefill(ids[:, :70])
            s.prepare()
            logits[fused] = [s.step(int(ids[0, i])).float().clone() for i in range(70, 80)]
    for a, b in zip(logits[False], logits[True]):
        assert _rel_l2(b, a) <= 5e-3


@pytest.mark.parametrize("k,n", [(896, 1152), (896, 896), (4864, 896), (128, 40), (8, 1), (1032, 77), (16384, 9),
                                 (64, 40000), (4864, 6000)])   # the last two: more outputs than fit in four resident waves
@pytest.mark.parametrize("bias", [False, True])
@pytest.mark.parametrize("norm", [False, True])
def test_decode_linear_matches_torch(k, n, bias, norm):
    """moba_decode_linear against the module arithmetic it replaces: residual add in bf16, RMSNorm as the Hugging Face
    module computes it, projection with FP32 accumulation and one rounding."""
    import ctypes
    from moba_opt import _ext
    lib = _ext.lib()
    g = torch.Generator().manual_seed(k * 31 + n)
    rnd = lambda *shape: torch.randn(*shape, generator=g).cuda().bfloat16()
    w, b = rnd(n, k) * k ** -0.5, (rnd(n) if bias else None)
    h, d, nw = rnd(k), rnd(k), (1 + 0.1 * torch.randn(k, generator=g)).cuda().bfloat16()
    y, h_out = torch.empty(n, device="cuda", dtype=torch.bfloat16), torch.empty(k, device="cuda", dtype=torch.bfloat16)
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    if norm:
        rc = lib.moba_decode_linear(None, h.data_ptr(), d.data_ptr(), nw.data_ptr(), 1e-6, h_out.data_ptr(), w.data_ptr(),
                                    None if b is None else b.data_ptr(), k, n, 0, y.data_ptr(), st)
        res = h + d
        assert rc == 0 and torch.equal(h_out, res)
        f = res.float()
        x = nw * (f * torch.rsqrt(f.pow(2).mean() + 1e-6)).bfloat16()
    else:
        x = h
        rc = lib.moba_decode_linear(x.data_ptr(), None, None, None, 0.0, None, w.data_ptr(), None if b is None else b.data_ptr(),
                                    k, n, 0, y.data_ptr(), st)
        assert rc == 0
    want = w.double() @ x.double() + (0 if b is None else b.double())
    assert _rel_l2(y, want) <= 4e-3
    np.testing.assert_allclose(y.double().cpu().numpy(), want.cpu().numpy(), atol=0.03, rtol=0.02)


@pytest.mark.parametrize("k,ffn", [(896, 4864), (128, 256), (8192, 5), (40, 33)])
def test_decode_linear_gate_up_epilogue(k, ffn):
    import ctypes
    from moba_opt import _ext
    lib = _ext.lib()
    g = torch.Generator().manual_seed(k + ffn)
    w = (torch.randn(2 * ffn, k, generator=g) * k ** -0.5).cuda().bfloat16()
    x = torch.randn(k, generator=g).cuda().bfloat16()
    y = torch.empty(ffn, device="cuda", dtype=torch.bfloat16)
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.moba_decode_linear(x.data_ptr(), None, None, None, 0.0, None, w.data_ptr(), None, k, ffn, 1, y.data_ptr(), st) == 0
    gu = (w.double() @ x.double())
    want = torch.nn.functional.silu(gu[:ffn]) * gu[ffn:]
    assert _rel_l2(y, want) <= 8e-3


def test_decode_linear_contract():
    import ctypes
    from moba_opt import _ext
    lib = _ext.lib()
    t = torch.zeros(64, 64, device="cuda", dtype=torch.bfloat16)
    p, st = t.data_ptr(), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    call = lambda *a: lib.moba_decode_linear(*a, st)
    assert call(p, None, None, None, 0.0, None, p, None, 12, 4, 0, p) != 0          # k not a multiple of 8
    assert call(p, p, None, p, 0.0, None, p, None, 64, 4, 0, p) != 0                # two input sources
    assert call(None, None, None, None, 0.0, None, p, None, 64, 4, 0, p) != 0       # none
    assert call(p, None, None, None, 0.0, None, p, p, 64, 4, 1, p) != 0             # bias with the gate/up epilogue
    assert call(p, None, None, None, 0.0, None, p, None, 16392, 1, 0, p) != 0       # row longer than a group can hold
    assert call(p + 2, None, None, None, 0.0, None, p, None, 64, 4, 0, p) != 0      # unaligned input
    h, d2, o = t.data_ptr(), t[8:].data_ptr(), t[16:].data_ptr()
    assert call(None, h, d2, p, 1e-6, h, p, None, 64, 4, 0, o) == 1                 # new residual written in place of h_in
    assert call(None, h, d2, p, 1e-6, d2, p, None, 64, 4, 0, o) == 1                # ... or of delta
    assert call(None, h, d2, p, 1e-6, t[24:].data_ptr(), p, None, 64, 4, 0, o) == 0
    torch.cuda.synchronize()


@pytest.mark.parametrize("position", [0, 1, 777, 16384, 131071])
def test_step_inputs_match_the_rotary_module_and_embedding(model, position):
    """moba_decode_step_inputs against the modules it replaces in a step: embedding row and rotary cos / sin, bit for bit."""
    import ctypes
    from moba_opt import _ext
    lib = _ext.lib()
    body, cfg = model.model, model.config
    dim = cfg.hidden_size // cfg.num_attention_heads
    tok = torch.tensor([[123]], device="cuda")
    pos = torch.tensor([position], device="cuda", dtype=torch.int32)
    want_h = body.embed_tokens(tok)[0]
    cos, sin = body.rotary_emb(want_h[None], pos.long()[None])
    inv = body.rotary_emb.inv_freq.float().contiguous()
    h = torch.empty(1, cfg.hidden_size, device="cuda", dtype=torch.bfloat16)
    c, s_ = torch.empty(1, dim, device="cuda", dtype=torch.bfloat16), torch.empty(1, dim, device="cuda", dtype=torch.bfloat16)
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.moba_decode_step_inputs(tok.data_ptr(), body.embed_tokens.weight.data_ptr(), cfg.hidden_size, pos.data_ptr(),
                                       inv.data_ptr(), float(body.rotary_emb.attention_scaling), dim, 1, h.data_ptr(), c.data_ptr(),
                                       s_.data_ptr(), st) == 0
    assert torch.equal(h, want_h)
    assert torch.equal(c, cos[0].to(torch.bfloat16)) and torch.equal(s_, sin[0].to(torch.bfloat16))


def test_row_wise_glue_kernels_agree_with_the_single_row_forms():
    """moba_add_rmsnorm, moba_rope_split and moba_silu_mul switch to 16-byte accesses from 64 rows on; the results must
    be those of the small-batch kernels (rotary embedding and SiLU*up bit for bit, the norm within one bf16 step, its
    sum of squares being taken in another order)."""
    import ctypes
    from moba_opt import _ext
    lib = _ext.lib()
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    g = torch.Generator().manual_seed(11)
    rnd = lambda *shape: torch.randn(*shape, generator=g).cuda().bfloat16()
    rows, hidden, hq, hk, dim, ffn = 100, 896, 14, 2, 64, 4864
    ptr = lambda t: t.data_ptr()

    def halves(call, *outs):
        """Runs `call(first_row, count)` over all rows at once and as two halves of 50 (the small-batch path)."""
        call(0, rows)
        big = [o.clone() for o in outs]
        for o in outs:
            o.zero_()
        call(0, 50)
        call(50, 50)
        return big, outs

    h, d, w = rnd(rows, hidden), rnd(rows, hidden), rnd(hidden)
    h_out, y = torch.empty_like(h), torch.empty_like(h)
    big, small = halves(lambda r0, n: lib.moba_add_rmsnorm(ptr(h[r0:]), ptr(d[r0:]), ptr(w), 1e-6, n, hidden, ptr(h_out[r0:]),
                                                          ptr(y[r0:]), st), h_out, y)
    assert torch.equal(big[0], small[0])
    diff = (big[1].float() - small[1].float()).abs()
    assert float((diff / small[1].float().abs().clamp_min(1e-3)).max()) <= 2 ** -7

    qkv, cos, sin = rnd(rows, (hq + 2 * hk) * dim), rnd(rows, dim), rnd(rows, dim)
    q, k, v = torch.empty(rows, hq, dim, device="cuda", dtype=torch.bfloat16), torch.empty(rows, hk, dim, device="cuda", dtype=torch.bfloat16), torch.empty(rows, hk, dim, device="cuda", dtype=torch.bfloat16)
    big, small = halves(lambda r0, n: lib.moba_rope_split(ptr(qkv[r0:]), ptr(cos[r0:]), ptr(sin[r0:]), n, hq, hk, dim, ptr(q[r0:]),
                                                         ptr(k[r0:]), ptr(v[r0:]), st), q, k, v)
    assert all(torch.equal(a, b) for a, b in zip(big, small))

    gu, act = rnd(rows, 2 * ffn), torch.empty(rows, ffn, device="cuda", dtype=torch.bfloat16)
    big, small = halves(lambda r0, n: lib.moba_silu_mul(ptr(gu[r0:]), n, ffn, ptr(act[r0:]), st), act)
    assert torch.equal(big[0], small[0])


@pytest.mark.parametrize("n", [1, 7, 8, 300, 4099, 151936, 1 << 20])
def test_argmax_matches_torch_and_takes_the_lowest_index_among_ties(n):
    import ctypes
    from moba_opt import _ext
    lib = _ext.lib()
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    ws = torch.zeros(lib.moba_argmax_workspace_bytes(), dtype=torch.uint8, device="cuda")
    out = torch.full((1,), -1, dtype=torch.long, device="cuda")
    g = torch.Generator().manual_seed(n)
    for trial in range(3):      # the workspace is left ready for the next call
        x = torch.randn(n, generator=g).cuda().bfloat16()
        if trial == 1 and n > 8:
            top = float(x.float().max()) + 1.0
            x[n - 1], x[n // 2], x[n // 3] = top, top, top          # ties: the lowest index wins
        if trial == 2 and n > 8:
            x[0] = float("nan")                                     # NaN never wins
        assert lib.moba_argmax_bf16(x.data_ptr(), n, ws.data_ptr(), ws.numel(), out.data_ptr(), st) == 0
        ref = x.float().clone()
        ref[ref.isnan()] = -float("inf")
        want = int((ref == ref.max()).nonzero()[0, 0])
        assert int(out[0]) == want
