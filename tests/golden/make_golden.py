"""Generates tests/golden/*.npz by running the reference's own Python code on CPU.

Run where a checkout of the reference project is available:
    python tests/golden/make_golden.py --reference /path/to/reference

What is executed from the reference (never copied):
  * routing: src/moba_opt/grouped_attention.py::opt_gqa_cuda on CPU tensors with its CUDA-only
    input check disabled and the attention launch intercepted, so the ROUTE_HOOK tensor is the
    reference's own block selection (route_precision='fp32' with stable_routes=True and with the
    torch.topk variant, and route_precision='upstream', the reference's default, whose chunk means
    are rounded to bf16 before the gate);
  * reference/fixed_route_attention.py, reference/grouped_reference.py (+ torch autograd for the
    gradients), reference/decode_reference.py, reference/merge_reference.py.
The un-vendored upstream `moba` package the reference imports is satisfied in memory from the
reference's own verbatim copy (src/moba_opt/diagnostic.py); nothing is written to the checkout.
"""
import argparse
import importlib.util
import itertools
import sys
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def load_reference(root):
    sys.path.insert(0, str(root / "src"))
    sys.path.insert(0, str(root))
    shim, eff = types.ModuleType("moba"), types.ModuleType("moba.moba_efficient")
    sys.modules["moba"], sys.modules["moba.moba_efficient"] = shim, eff
    spec = importlib.util.spec_from_file_location("_ref_diag", root / "src/moba_opt/diagnostic.py")
    diag = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(diag)
    eff.calc_chunks, eff.moba_attn_varlen = diag.calc_chunks, diag.moba_attn_varlen
    import moba_opt.grouped_attention as grouped
    from reference.decode_reference import decode_reference
    from reference.fixed_route_attention import fixed_route_attention
    from reference.grouped_reference import grouped_reference
    from reference.merge_reference import merge_grouped_reference
    return grouped, fixed_route_attention, grouped_reference, decode_reference, merge_grouped_reference


class _Stop(Exception):
    pass


def reference_route(grouped, q, k, v, cu, max_len, cfg):
    """Runs the reference's routing code and returns its ROUTE_HOOK payload (CPU tensors)."""
    captured = {}

    def hook(**kw):
        captured.update({name: t.detach().clone() for name, t in kw.items()})
        raise _Stop()

    saved = grouped._validate
    grouped._validate = lambda *a, **kw: None
    grouped.ROUTE_HOOK = hook
    try:
        grouped.opt_gqa_cuda(q, k, v, cu, max_len, cfg)
    except _Stop:
        pass
    except Exception:
        # No candidate chunk: the reference falls through to its dense FlashAttention call, which
        # cannot run on CPU.  The route is then empty by definition.
        if captured:
            raise
        cu_chunk, filtered, _, chunk_batch = sys.modules["moba.moba_efficient"].calc_chunks(cu, cfg["chunk_size"])
        captured.update(cu_chunk=cu_chunk, filtered_chunk_indices=filtered, chunk_to_batch=chunk_batch,
                        selected=torch.zeros((0, q.shape[1], q.shape[0]), dtype=torch.bool))
    finally:
        grouped.ROUTE_HOOK = None
        grouped._validate = saved
    return captured


def f32(t):
    """FP64 reference results are stored as float32 (relative error 6e-8) to keep fixtures small."""
    return t.numpy().astype(np.float32)


def bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def make_inputs(lens, hq, hkv, dim, seed, dtype, scale=1.0):
    rng = torch.Generator().manual_seed(seed)
    total = sum(lens)
    q, k, v = [(torch.randn(total, h, dim, generator=rng) * scale).to(dtype) for h in (hq, hkv, hkv)]
    g = torch.randn(total, hq, dim, generator=rng).to(dtype)
    cu = torch.tensor([0] + list(itertools.accumulate(lens)), dtype=torch.int32)
    return q, k, v, g, cu


PREFILL_CASES = [
    # name, lens, hq, hkv, dim, chunk, topk, seed
    ("p_gqa_small", (35, 62), 8, 2, 64, 16, 4, 61),
    ("p_mha_tail", (97,), 4, 4, 32, 24, 3, 62),
    ("p_mqa_multi", (40, 17, 130), 6, 1, 128, 32, 3, 63),
    ("p_k9", (200,), 4, 2, 64, 16, 9, 64),
    ("p_one_chunk", (9, 12), 4, 2, 16, 16, 4, 65),
    ("p_gqa_256", (180, 140), 14, 2, 64, 64, 3, 66),
    # IEEE half inputs (the reference takes both 16-bit formats, baseline_adapter.py:13); the record says so in `dtype`
    ("p_fp16_gqa", (150, 90), 8, 2, 64, 32, 3, 70, torch.float16),
    ("p_fp16_d128", (260,), 6, 1, 128, 24, 4, 71, torch.float16),
]


def prefill_cases(ref, out_dir):
    grouped, fixed_route_attention, grouped_reference, _, _ = ref
    for name, lens, hq, hkv, dim, chunk, topk, seed, *rest in PREFILL_CASES:
        dtype = rest[0] if rest else torch.bfloat16
        q, k, v, g, cu = make_inputs(lens, hq, hkv, dim, seed, dtype)
        rec = dict(lens=np.asarray(lens), hq=hq, hkv=hkv, dim=dim, chunk=chunk, topk=topk, seed=seed,
                   q=bits(q), k=bits(k), v=bits(v), g=bits(g))
        if dtype != torch.bfloat16:
            rec["dtype"] = np.asarray(str(dtype).replace("torch.", ""))
        for tag, precision, stable in (("stable", "fp32", True), ("topk", "fp32", False), ("upstream", "upstream", True),
                                       ("upstream_topk", "upstream", False)):
            cfg = {"chunk_size": chunk, "topk": topk, "route_precision": precision, "stable_routes": stable}
            route = reference_route(grouped, q, k, v, cu, max(lens), cfg)
            rec[f"selected_{tag}"] = route["selected"].numpy()
            if tag == "stable":
                rec["cu_chunk"] = route["cu_chunk"].numpy()
                rec["filtered"] = route["filtered_chunk_indices"].numpy()
                rec["chunk_to_batch"] = route["chunk_to_batch"].numpy()
                full = dict(route, cu_seqlens=cu, chunk_size=chunk, topk=topk, max_seqlen=max(lens))
                qd, kd, vd = (t.double().requires_grad_(True) for t in (q, k, v))
                out = grouped_reference(qd, kd, vd, cu, full)
                dq, dk, dv = torch.autograd.grad(out, (qd, kd, vd), grad_outputs=g.double())
                rec.update(out=f32(out.detach()), dq=f32(dq), dk=f32(dk), dv=f32(dv))
                if hq == hkv:
                    o2, lse = fixed_route_attention(q, k, v, cu, full)
                    rec.update(out_fixed=f32(o2), lse=f32(lse))
        np.savez_compressed(out_dir / f"{name}.npz", **rec)
        print(name, "selected pairs", int(rec["selected_stable"].sum()))


ROUTE_CASES = [
    # name, lens, hq, hkv, dim, chunk, topk, seed: many candidates and chunk sizes that are not powers of two, so that
    # rounding the chunk means to bf16 (route_precision='upstream') changes some rows' selection
    ("r_upstream_gqa", (700, 500), 6, 2, 128, 40, 5, 68),
    ("r_upstream_mqa", (1500,), 4, 1, 64, 24, 4, 69),
]


def route_cases(ref, out_dir):
    """Route-only fixtures: inputs and the reference's selection under both route precisions (bit-packed)."""
    grouped = ref[0]
    for name, lens, hq, hkv, dim, chunk, topk, seed in ROUTE_CASES:
        q, k, v, _, cu = make_inputs(lens, hq, hkv, dim, seed, torch.bfloat16)
        rec = dict(lens=np.asarray(lens), hq=hq, hkv=hkv, dim=dim, chunk=chunk, topk=topk, seed=seed, q=bits(q), k=bits(k))
        for tag, precision in (("stable", "fp32"), ("upstream", "upstream")):
            cfg = {"chunk_size": chunk, "topk": topk, "route_precision": precision, "stable_routes": True}
            route = reference_route(grouped, q, k, v, cu, max(lens), cfg)
            rec[f"selected_{tag}_packed"] = np.packbits(route["selected"].numpy())
            rec["selected_shape"] = np.asarray(route["selected"].shape)
            rec["filtered"] = route["filtered_chunk_indices"].numpy()
        differ = int((np.unpackbits(rec["selected_stable_packed"]) != np.unpackbits(rec["selected_upstream_packed"])).sum())
        np.savez_compressed(out_dir / f"{name}.npz", **rec)
        print(name, "selection bits that differ between the two precisions:", differ)


def config1_case(ref, out_dir):
    """BASELINE config 1: T=2048, 8 MHA heads, D=64, chunk 256, topk 3, seed 0 (q, k, v, then dO).
    Inputs are regenerated from the seed by the tests; only the route (bit-packed), sampled rows of
    the outputs and whole-tensor sums are stored."""
    grouped, fixed_route_attention, grouped_reference, _, _ = ref
    rng = torch.Generator().manual_seed(0)
    q, k, v = [torch.randn(2048, 8, 64, generator=rng).bfloat16() for _ in range(3)]
    g = torch.randn(2048, 8, 64, generator=rng).bfloat16()
    cu = torch.tensor([0, 2048], dtype=torch.int32)
    cfg = {"chunk_size": 256, "topk": 3, "route_precision": "fp32", "stable_routes": True}
    route = reference_route(grouped, q, k, v, cu, 2048, cfg)
    full = dict(route, cu_seqlens=cu, chunk_size=256, topk=3, max_seqlen=2048)
    qd, kd, vd = (t.double().requires_grad_(True) for t in (q, k, v))
    out = grouped_reference(qd, kd, vd, cu, full)
    dq, dk, dv = torch.autograd.grad(out, (qd, kd, vd), grad_outputs=g.double())
    o2, lse = fixed_route_attention(q, k, v, cu, full)
    rows = np.arange(0, 2048, 37)
    rec = dict(selected_packed=np.packbits(route["selected"].numpy()), selected_shape=np.asarray(route["selected"].shape),
               rows=rows, q_head=bits(q)[:4], out_rows=out.detach().numpy()[rows], lse_rows=lse.numpy()[rows],
               dq_rows=dq.numpy()[rows], dk_rows=dk.numpy()[rows], dv_rows=dv.numpy()[rows],
               sums=np.asarray([out.sum().item(), lse.sum().item(), dq.sum().item(), dk.sum().item(), dv.sum().item()]),
               abs_sums=np.asarray([out.abs().sum().item(), lse.abs().sum().item(), dq.abs().sum().item(),
                                    dk.abs().sum().item(), dv.abs().sum().item()]),
               fixed_vs_grouped=np.asarray((o2 - out.detach()).abs().max().item()))
    np.savez_compressed(out_dir / "config1.npz", **rec)
    print("config1 selected pairs", int(route["selected"].sum()))


DECODE_CASES = [
    # name, lengths, hq, hkv, dim, chunk, topk, seed
    ("d_small", (37, 90, 5), 8, 2, 64, 16, 4, 201),
    ("d_d128", (200, 131), 12, 2, 128, 32, 4, 202),
    ("d_mha", (64, 65), 4, 4, 32, 8, 3, 203),
    ("d_fp16", (150, 47), 12, 2, 64, 16, 4, 204, torch.float16),
]


def decode_cases(ref, out_dir):
    _, _, _, decode_reference, _ = ref
    for name, lengths, hq, hkv, dim, chunk, topk, seed, *rest in DECODE_CASES:
        dtype = rest[0] if rest else torch.bfloat16
        rng = torch.Generator().manual_seed(seed)
        keys = [torch.randn(n, hkv, dim, generator=rng).to(dtype) for n in lengths]
        values = [torch.randn(n, hkv, dim, generator=rng).to(dtype) for n in lengths]
        ids = list(range(len(lengths)))
        pos = [n - 1 for n in lengths]
        q = torch.randn(len(ids), hq, dim, generator=rng).to(dtype)
        # a legal hand-made route: current chunk first, then the most recent complete chunks per head parity
        R = topk - 1
        selected = torch.full((len(ids), hq, 1 + R), -1, dtype=torch.int32)
        for row, p in enumerate(pos):
            cur = p // chunk
            selected[row, :, 0] = cur
            for h in range(hq):
                cand = list(range(cur))[h % 2::2][:R] if cur else []
                for s, c in enumerate(cand):
                    selected[row, h, 1 + s] = c
        out_s, lse_s = decode_reference(q, keys, values, ids, pos, chunk_size=chunk, selected_blocks=selected)
        out_d, lse_d = decode_reference(q, keys, values, ids, pos, chunk_size=chunk)
        rec = dict(lengths=np.asarray(lengths), hq=hq, hkv=hkv, dim=dim, chunk=chunk, topk=topk, q=bits(q),
                   selected=selected.numpy(), out_sparse=out_s.numpy(), lse_sparse=lse_s.numpy(),
                   out_dense=out_d.numpy(), lse_dense=lse_d.numpy())
        if dtype != torch.bfloat16:
            rec["dtype"] = np.asarray(str(dtype).replace("torch.", ""))
        for i, (kk, vv) in enumerate(zip(keys, values)):
            rec[f"k{i}"], rec[f"v{i}"] = bits(kk), bits(vv)
        np.savez_compressed(out_dir / f"{name}.npz", **rec)
        print(name)


def merge_case(ref, out_dir):
    *_, merge_grouped_reference = ref
    rng = torch.Generator().manual_seed(301)
    P, M, D = 40, 70, 16
    so, ro = torch.randn(P, D, generator=rng), torch.randn(M, D, generator=rng)
    sl, rl = torch.randn(P, generator=rng) * 3, torch.randn(M, generator=rng) * 3
    mapping = torch.randint(0, P, (M,), generator=rng)
    o, l = merge_grouped_reference(so, sl, ro, rl, mapping)
    np.savez_compressed(out_dir / "merge.npz", self_out=so.numpy(), self_lse=sl.numpy(), remote_out=ro.numpy(),
                        remote_lse=rl.numpy(), mapping=mapping.numpy(), out=o.numpy(), lse=l.numpy())
    print("merge")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the reference checkout")
    args = ap.parse_args()
    torch.set_num_threads(8)
    ref = load_reference(Path(args.reference))
    prefill_cases(ref, HERE)
    route_cases(ref, HERE)
    config1_case(ref, HERE)
    decode_cases(ref, HERE)
    merge_case(ref, HERE)


if __name__ == "__main__":
    main()
