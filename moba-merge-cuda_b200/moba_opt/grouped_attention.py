"""Native GQA/MQA MoBA prefill with autograd: the drop-in for the reference's
`opt_gqa_cuda(q, k, v, cu_seqlens, max_seqlen, config)` (src/moba_opt/grouped_attention.py:29-99).

The host does only what needs Python: the input contract, chunk/tile metadata derived from
cu_seqlens (cached per batch shape), buffer allocation through torch, and three C-ABI calls
(route, forward, backward) on the current stream.  Routing, expert packing, attention, the LSE merge
and the gradients all run in the sm_100a kernels of libmoba_b200.so; there is no other code path.
"""
import ctypes
from collections import OrderedDict

import numpy as np
import torch

from . import _ext
from .api import register
from .baseline_adapter import _validate

# Test hook with the reference's signature (grouped_attention.py:16,72-74): called with
# cu_chunk, filtered_chunk_indices, chunk_to_batch and selected [F,Hq,T] bool after routing.
ROUTE_HOOK = None

_TILE = 128
_PLAN_CACHE = OrderedDict()
_STATUS = {}


class PrefillPlan:
    """Chunk and query-tile metadata of one packed batch (chunking rule of
    src/moba_opt/diagnostic.py:30-80), resident on the device as int32 arrays."""

    def __init__(self, cu, chunk_size, device):
        cu = np.asarray(cu, dtype=np.int64)
        lens = np.diff(cu)
        nchunk = (lens + chunk_size - 1) // chunk_size
        tpc = (chunk_size + _TILE - 1) // _TILE
        chunk_start, chunk_seq, chunk_local = [0], [], []
        qt_chunk, qt_tok0, qt_local, qt_cost = [], [], [], []
        filtered = []
        for b, (length, n) in enumerate(zip(lens.tolist(), nchunk.tolist())):
            for j in range(n):
                size = chunk_size if j < n - 1 else length - (n - 1) * chunk_size
                c = len(chunk_seq)
                if j < n - 1:
                    filtered.append(c)
                chunk_seq.append(b)
                chunk_local.append(j)
                start = chunk_start[-1]
                for i in range((size + _TILE - 1) // _TILE):
                    qt_chunk.append(c)
                    qt_tok0.append(start + i * _TILE)
                    qt_local.append(j * tpc + i)
                    qt_cost.append(i)
                chunk_start.append(start + size)
        self.cu = tuple(int(x) for x in cu)
        self.chunk_size = int(chunk_size)
        self.total_tokens = int(cu[-1])
        self.num_seqs = len(lens)
        self.num_chunks = len(chunk_seq)
        self.num_qtiles = len(qt_chunk)
        self.max_chunks_per_seq = int(nchunk.max())
        self.max_tiles_per_seq = int(max(qt_local) + 1)
        self.num_routable = len(filtered)
        cost = np.asarray(qt_cost)
        leaders = np.flatnonzero(cost % 2 == 0)  # tiles 2i, 2i+1 of a chunk form a pair; 2i+1 may be missing
        has_partner = np.zeros(len(leaders), dtype=bool)
        nxt = leaders + 1
        ok = nxt < len(cost)
        has_partner[ok] = (np.asarray(qt_chunk)[nxt[ok]] == np.asarray(qt_chunk)[leaders[ok]])
        order = leaders[np.argsort(-(cost[leaders] + has_partner), kind="stable")]
        self.num_self_pairs = len(order)
        kv_order = np.lexsort((cost, np.asarray(chunk_local)[np.asarray(qt_chunk)]))
        arrays = [cu, chunk_start, chunk_seq, chunk_local, qt_chunk, qt_tok0, qt_local, order, kv_order]
        sizes = [len(a) for a in arrays]
        flat = np.concatenate([np.asarray(a, dtype=np.int32) for a in arrays])
        self._flat = torch.from_numpy(flat).to(device)
        views = self._flat.split(sizes)
        (self.cu_seqlens, self.chunk_start, self.chunk_seq, self.chunk_local,
         self.qtile_chunk, self.qtile_tok0, self.qtile_local, self.self_pairs, self.kv_order) = views
        self.filtered = np.asarray(filtered, dtype=np.int64)
        self.chunk_to_batch = np.asarray(chunk_seq, dtype=np.int64)
        self.cu_chunk = np.asarray(chunk_start, dtype=np.int64)

    def desc(self, q, k, v, remote_k, flags=0):
        d = _ext.PrefillDesc()
        d.flags = flags | (4 if q.dtype == torch.float16 else 0)    # MOBA_INPUT_FP16
        d.total_tokens, d.num_seqs = self.total_tokens, self.num_seqs
        d.hq, d.hkv, d.dim = q.shape[1], k.shape[1], q.shape[2]
        d.chunk_size, d.remote_k = self.chunk_size, remote_k
        d.num_chunks, d.num_qtiles = self.num_chunks, self.num_qtiles
        d.num_self_pairs = self.num_self_pairs
        d.max_tiles_per_seq, d.max_chunks_per_seq = self.max_tiles_per_seq, self.max_chunks_per_seq
        d.q_stride_t, d.q_stride_h = q.stride(0), q.stride(1)
        d.k_stride_t, d.k_stride_h = k.stride(0), k.stride(1)
        d.v_stride_t, d.v_stride_h = v.stride(0), v.stride(1)
        for name in ("cu_seqlens", "chunk_start", "chunk_seq", "chunk_local", "qtile_chunk", "qtile_tok0",
                     "qtile_local", "self_pairs", "kv_order"):
            setattr(d, name, getattr(self, name).data_ptr())
        return d


def get_plan(cu, chunk_size, device):
    key = (tuple(cu), int(chunk_size), str(device))
    plan = _PLAN_CACHE.get(key)
    if plan is None:
        plan = PrefillPlan(cu, chunk_size, device)
        _PLAN_CACHE[key] = plan
        if len(_PLAN_CACHE) > 16:
            _PLAN_CACHE.popitem(last=False)
    else:
        _PLAN_CACHE.move_to_end(key)
    return plan


def _status_word(device):
    t = _STATUS.get(device)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _STATUS[device] = t
    return t


def check_status(device=None):
    """Synchronises and raises RuntimeError if any kernel since the last check recorded an error
    bit (bounded barrier wait expired, out-of-range table entry)."""
    devices = list(_STATUS) if device is None else [torch.device(device)]
    for dev in devices:
        t = _STATUS.get(dev)
        if t is None:
            continue
        bits = int(t.item())
        if bits:
            t.zero_()
            raise RuntimeError(f"CUDA execution failed (status bits {bits:#x}); discard the outputs")


def _aligned(t):
    """Kernels use 16-byte vector loads: strides multiple of 8 elements and a 16-byte aligned base."""
    if t.stride(0) % 8 or t.stride(1) % 8 or t.data_ptr() % 16:
        return t.contiguous()
    return t


def _stream(device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def route(q, k, plan, remote_k, flags=0):
    """Runs the routing kernels; returns the opaque route-state tensor (uint8)."""
    lib = _ext.lib()
    d = plan.desc(q, k, k, remote_k, flags)
    state = torch.empty(lib.moba_prefill_route_state_bytes(ctypes.byref(d)), dtype=torch.uint8, device=q.device)
    nbytes = lib.moba_prefill_route_scratch_bytes(ctypes.byref(d))
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
    with _ext.nvtx("moba.route"):
        _ext.check(lib.moba_prefill_route(ctypes.byref(d), q.data_ptr(), k.data_ptr(), state.data_ptr(),
                                          scratch.data_ptr(), nbytes, _stream(q.device)), "moba_prefill_route")
    return state


def selected_table(state, total, hq, remote_k):
    """sel [T,Hq,R] int32 view of a route state: chosen global chunk ids, ascending, -1 padded."""
    return state[: total * hq * remote_k * 4].view(torch.int32).view(total, hq, remote_k)


class _MobaPrefill(torch.autograd.Function):
    """Forward + backward through the C ABI; the counterpart of OptMixedAttention
    (src/moba_opt/mixed_attention.py:40-225) with routing included."""

    @staticmethod
    def forward(ctx, q, k, v, plan, remote_k, flags, bwd_flags):
        lib = _ext.lib()
        q, k, v = _aligned(q), _aligned(k), _aligned(v)
        with torch.cuda.device(q.device):
            state = route(q, k, plan, remote_k, flags)
            if ROUTE_HOOK is not None and remote_k > 0:
                _fire_hook(plan, state, q.shape[0], q.shape[1], remote_k)
            d = plan.desc(q, k, v, remote_k)
            nbytes = lib.moba_prefill_fwd_scratch_bytes(ctypes.byref(d))
            scratch = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
            out = torch.empty((q.shape[0], q.shape[1], q.shape[2]), dtype=q.dtype, device=q.device)
            lse = torch.empty((q.shape[0], q.shape[1]), dtype=torch.float32, device=q.device)
            with _ext.nvtx("moba.forward"):
                _ext.check(lib.moba_prefill_fwd(ctypes.byref(d), q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                                state.data_ptr(), scratch.data_ptr(), nbytes,
                                                out.data_ptr(), lse.data_ptr(), _status_word(q.device).data_ptr(),
                                                _stream(q.device)), "moba_prefill_fwd")
        ctx.save_for_backward(q, k, v, out, lse, state)
        ctx.plan, ctx.remote_k, ctx.bwd_flags = plan, remote_k, bwd_flags
        ctx.mark_non_differentiable(lse)
        return out, lse

    @staticmethod
    def backward(ctx, d_out, _d_lse):
        lib = _ext.lib()
        q, k, v, out, lse, state = ctx.saved_tensors
        plan, remote_k = ctx.plan, ctx.remote_k
        d_out = d_out.contiguous()
        with torch.cuda.device(q.device):
            d = plan.desc(q, k, v, remote_k, ctx.bwd_flags)
            nbytes = lib.moba_prefill_bwd_scratch_bytes(ctypes.byref(d))
            scratch = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
            dq = torch.empty(q.shape, dtype=q.dtype, device=q.device)
            dk = torch.empty(k.shape, dtype=k.dtype, device=q.device)
            dv = torch.empty(v.shape, dtype=v.dtype, device=q.device)
            with _ext.nvtx("moba.backward"):
                _ext.check(lib.moba_prefill_bwd(ctypes.byref(d), q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                                lse.data_ptr(), d_out.data_ptr(), state.data_ptr(),
                                                scratch.data_ptr(), nbytes, dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                                                _status_word(q.device).data_ptr(), _stream(q.device)), "moba_prefill_bwd")
        return dq, dk, dv, None, None, None, None


def _fire_hook(plan, state, total, hq, remote_k):
    sel = selected_table(state, total, hq, remote_k).cpu().numpy()
    lookup = np.full(plan.num_chunks, -1, dtype=np.int64)
    lookup[plan.filtered] = np.arange(plan.filtered.size)
    selected = np.zeros((plan.filtered.size, hq, total), dtype=bool)
    t_idx, h_idx, s_idx = np.nonzero(sel >= 0)
    selected[lookup[sel[t_idx, h_idx, s_idx]], h_idx, t_idx] = True
    ROUTE_HOOK(cu_chunk=torch.from_numpy(plan.cu_chunk).to(torch.int32),
               filtered_chunk_indices=torch.from_numpy(plan.filtered),
               chunk_to_batch=torch.from_numpy(plan.chunk_to_batch).to(torch.int32),
               selected=torch.from_numpy(selected))


def moba_prefill(q, k, v, cu_seqlens, max_seqlen, config, *, return_lse=False):
    """opt_gqa_cuda plus optional access to the global LSE [T,Hq] (fp32, natural log)."""
    cu = _validate(q, k, v, cu_seqlens, allow_gqa=True, max_seqlen=max_seqlen, config=config)
    chunk_size = int(config["chunk_size"])
    precision = config.get("route_precision", "upstream")   # the reference's default (grouped_attention.py:35)
    deterministic = config.get("deterministic_merge", True)
    stable = config.get("stable_routes", True)
    repeatable_grads = config.get("deterministic_backward", False)
    if precision not in ("upstream", "fp32"):
        raise ValueError("route_precision")
    if not isinstance(deterministic, bool) or not isinstance(stable, bool) or not isinstance(repeatable_grads, bool):
        raise ValueError("routing flags must be bool")
    flags = 1 if precision == "upstream" else 0  # MOBA_ROUTE_BF16_MEANS
    plan = get_plan(cu, chunk_size, q.device)
    remote_k = min(int(config["topk"]) - 1, plan.num_routable)
    if remote_k == 0:
        # K=1 or no routable chunk: dense causal attention over every whole sequence
        # (grouped_attention.py:41-46), expressed as one chunk per sequence.
        plan = get_plan(cu, max(b - a for a, b in zip(cu, cu[1:])), q.device)
    out, lse = _MobaPrefill.apply(q, k, v, plan, remote_k, flags, 2 if repeatable_grads else 0)   # MOBA_BWD_DETERMINISTIC
    return (out, lse) if return_lse else out


def opt_gqa_cuda(q, k, v, cu_seqlens, max_seqlen, config):
    """Drop-in for the reference entry point; differentiable w.r.t. q, k, v.
    The gate is always FP32 with the lowest-chunk tie rule and the merge is always order-deterministic
    (the reference's stable_routes=True, deterministic_merge=True behaviour; both flags are accepted
    and type-checked; where the reference's default stable_routes=False leaves the order among exactly
    tied scores to torch.topk, the lowest chunk wins here).  route_precision defaults to 'upstream' as in
    the reference (grouped_attention.py:35): the chunk means are rounded to bf16 before the gate
    (grouped_attention.py:52); 'fp32' keeps them in FP32.  One key of this package's own:
    deterministic_backward (bool, default False) sums dQ in fixed point, so that the gradients are
    bit-repeatable too (the reference gets that from FlashAttention's deterministic=True,
    mixed_attention.py:185,220); dK, dV and the forward always are."""
    return moba_prefill(q, k, v, cu_seqlens, max_seqlen, config)


def _opt_mha(q, k, v, cu_seqlens, max_seqlen, config):
    """The reference's earlier entry points for equal head counts (src/moba_opt/mixed_attention.py:411-420:
    `opt_merge_atomic`, `opt_merge_cuda`, which differ only in the merge backend).  Same engine; grouped
    heads are rejected as they are there."""
    if q.dim() == 3 and k.dim() == 3 and q.shape[1] != k.shape[1]:
        raise ValueError("q and k/v must have the same number of heads for this implementation")
    return moba_prefill(q, k, v, cu_seqlens, max_seqlen, config)


def opt_merge_atomic(q, k, v, cu_seqlens, max_seqlen, config):
    return _opt_mha(q, k, v, cu_seqlens, max_seqlen, config)


def opt_merge_cuda(q, k, v, cu_seqlens, max_seqlen, config):
    return _opt_mha(q, k, v, cu_seqlens, max_seqlen, config)


register("opt_gqa_cuda", opt_gqa_cuda)
register("opt_merge_atomic", opt_merge_atomic)
register("opt_merge_cuda", opt_merge_cuda)
