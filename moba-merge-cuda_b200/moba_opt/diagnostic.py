"""Merge-stage fixtures for cross-machine comparison.

The reference exposes the inputs and outputs of its merge stage through a module hook on its diagnostic forward
(src/moba_opt/diagnostic.py:24-27,141-147,200-205: `MERGE_HOOK("inputs", {...})`, `MERGE_HOOK("outputs", {...})`) and
dumps them as fixtures with scripts/dump_merge_fixtures.py:29-60.  Here the merge is the epilogue of the forward kernel,
so the self branch never exists in memory on the normal path.  This module materialises the same payload on request:

  inputs   self_out [T,H,D], self_lse [T,H] fp32 (natural log)   the own-chunk causal attention alone
           remote_out [M,1,D], remote_lse [M] fp32, mapping [M]   one row per selected (query row, chunk) pair, row p = t*H + h
  outputs  output [T,H,D], mixed_lse [T,H] fp32                   what the forward returns

`moba_attn_varlen` has the reference entry point's signature and fires `MERGE_HOOK` the same way; `dump_merge_fixture`
returns the payload of the reference's dump script (CPU tensors), and the module runs as a script:

    python -m moba_opt.diagnostic --tokens 4096 --heads 8 --kv-heads 2 --head-dim 64 --chunk 256 --topk 3 --out fixture.pt

The self branch comes from a second launch of the same forward kernel with routing switched off (remote_k = 0 on the
same chunking); the remote rows are the kernel's own per-slot partial results, read from its scratch buffer.
"""
import argparse
import ctypes
import itertools
import math

import torch

from . import _ext
from . import grouped_attention as ga
from .baseline_adapter import _validate

MERGE_HOOK = None


def _forward(lib, plan, q, k, v, remote_k, flags, state=None):
    """One forward through the C ABI; returns (out, lse, scratch, state)."""
    dev = q.device
    d = plan.desc(q, k, v, remote_k, flags)
    if state is None:
        state = ga.route(q, k, plan, remote_k, flags)
    nbytes = lib.moba_prefill_fwd_scratch_bytes(ctypes.byref(d))
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    out = torch.empty_like(q)
    lse = torch.empty(q.shape[:2], dtype=torch.float32, device=dev)
    _ext.check(lib.moba_prefill_fwd(ctypes.byref(d), q.data_ptr(), k.data_ptr(), v.data_ptr(), state.data_ptr(), scratch.data_ptr(),
                                    nbytes, out.data_ptr(), lse.data_ptr(), ga._status_word(dev).data_ptr(), ga._stream(dev)),
               "moba_prefill_fwd")
    return out, lse, scratch, state


@torch.no_grad()
def merge_stage(q, k, v, cu_seqlens, max_seqlen, config):
    """(inputs, outputs) dictionaries of the merge stage, tensors on q's device."""
    cu = _validate(q, k, v, cu_seqlens, allow_gqa=True, max_seqlen=max_seqlen, config=config)
    lib = _ext.lib()
    chunk = int(config["chunk_size"])
    flags = 1 if config.get("route_precision", "upstream") == "upstream" else 0
    plan = ga.get_plan(cu, chunk, q.device)
    remote_k = min(int(config["topk"]) - 1, plan.num_routable)
    q, k, v = (ga._aligned(t) for t in (q, k, v))
    total, hq, dim = q.shape
    with torch.cuda.device(q.device):
        self_out, self_lse, _, _ = _forward(lib, plan, q, k, v, 0, 0)                 # own chunks only: the self branch
        if remote_k == 0:
            output, mixed_lse = self_out, self_lse
            remote_out = q.new_empty((0, 1, dim))
            remote_lse = torch.empty(0, dtype=torch.float32, device=q.device)
            mapping = torch.empty(0, dtype=torch.int64, device=q.device)
        else:
            output, mixed_lse, scratch, state = _forward(lib, plan, q, k, v, remote_k, flags)
            slots = total * hq * remote_k
            part_o = scratch[: slots * dim * 2].view(torch.bfloat16).view(slots, dim)
            lse_at = (slots * dim * 2 + 255) // 256 * 256
            part_lse = scratch[lse_at: lse_at + slots * 4].view(torch.float32)        # log2 domain
            chosen = ga.selected_table(state, total, hq, remote_k).reshape(-1) >= 0
            index = torch.nonzero(chosen).reshape(-1)
            remote_out = part_o[index].reshape(-1, 1, dim)
            remote_lse = part_lse[index] * math.log(2.0)
            mapping = index // remote_k
    ga.check_status()
    inputs = dict(self_out=self_out, self_lse=self_lse, remote_out=remote_out, remote_lse=remote_lse, mapping=mapping)
    return inputs, dict(output=output, mixed_lse=mixed_lse)


def moba_attn_varlen(q, k, v, cu_seqlens, max_seqlen, moba_chunk_size, moba_topk):
    """The reference diagnostic entry point's signature (src/moba_opt/diagnostic.py:83-206): forward only, fires
    MERGE_HOOK("inputs", ...) and MERGE_HOOK("outputs", ...) when the hook is set, returns the output."""
    config = {"chunk_size": moba_chunk_size, "topk": moba_topk}
    if MERGE_HOOK is None:
        return ga.moba_prefill(q, k, v, cu_seqlens, max_seqlen, config)
    inputs, outputs = merge_stage(q, k, v, cu_seqlens, max_seqlen, config)
    MERGE_HOOK("inputs", inputs)
    MERGE_HOOK("outputs", outputs)
    return outputs["output"]


def dump_merge_fixture(total_tokens, heads, kv_heads, head_dim, chunk_size, topk, seq_lens=None, seed=0, device="cuda"):
    """Payload of the reference's dump script (scripts/dump_merge_fixtures.py:29-60) for seeded N(0,1) bf16 inputs drawn
    the way that script draws them (q, then k, then v, FP32 on the CPU generator, cast to bf16)."""
    global MERGE_HOOK
    gen = torch.Generator().manual_seed(seed)
    mk = lambda h: torch.randn((total_tokens, h, head_dim), generator=gen, dtype=torch.float32).to(device=device, dtype=torch.bfloat16)
    q, k, v = mk(heads), mk(kv_heads), mk(kv_heads)
    lens = list(seq_lens) if seq_lens else [total_tokens]
    cu = torch.tensor([0] + list(itertools.accumulate(lens)), device=device, dtype=torch.int32)
    got = {}
    saved, MERGE_HOOK = MERGE_HOOK, lambda phase, tensors: got.__setitem__(phase, {n: t.detach().cpu() for n, t in tensors.items()})
    try:
        moba_attn_varlen(q, k, v, cu, max(lens), chunk_size, topk)
    finally:
        MERGE_HOOK = saved
    return dict(inputs=got["inputs"], expected=dict(output=got["outputs"]["output"], mixed_lse=got["outputs"]["mixed_lse"]),
                config=dict(total_tokens=total_tokens, heads=heads, kv_heads=kv_heads, head_dim=head_dim, chunk_size=chunk_size,
                            topk=topk, dtype="bfloat16", seq_lens=lens), seed=seed)


def main():
    ap = argparse.ArgumentParser(description="dump the merge-stage inputs and outputs of one seeded forward")
    ap.add_argument("--tokens", type=int, required=True)
    ap.add_argument("--heads", type=int, required=True)
    ap.add_argument("--kv-heads", type=int)
    ap.add_argument("--head-dim", type=int, default=64)
    ap.add_argument("--chunk", type=int, required=True)
    ap.add_argument("--topk", type=int, required=True)
    ap.add_argument("--seq-lens", type=int, nargs="*")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--out", required=True)
    args = ap.parse_args()
    payload = dump_merge_fixture(args.tokens, args.heads, args.kv_heads or args.heads, args.head_dim, args.chunk, args.topk,
                                 args.seq_lens, args.seed, args.device)
    torch.save(payload, args.out)
    print(args.out, "remote rows:", payload["inputs"]["mapping"].numel())


if __name__ == "__main__":
    main()
