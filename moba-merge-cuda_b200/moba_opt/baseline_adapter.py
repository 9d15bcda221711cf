"""Input contract of the prefill entry points.

Behaviourally the checks of the reference (src/moba_opt/baseline_adapter.py:23-76): every violation
is a ValueError raised before any device work, and `validate_shapes` / `validate_config` stay usable
without a CUDA runtime.  Two limits differ on purpose: topk may go up to 17 (reference: 9) because
the long-context configuration needs 12, and the prefill kernels take head_dim up to 128 (the
reference: 256; the decode cache here goes to 256 as well).  Each is refused here, as a ValueError,
before anything is launched.  bf16 and fp16 inputs are both taken, as by the reference.
"""
import numbers

import torch

SUPPORTED_DTYPES = (torch.bfloat16, torch.float16)
MAINLINE_HEAD_DIMS = tuple(range(8, 257, 8))      # the reference's envelope; the decode cache accepts all of it
PREFILL_HEAD_DIMS = tuple(range(8, 129, 8))       # what the prefill kernels are compiled for
MAX_TOPK = 17


def _fail(message):
    raise ValueError(message)


def _as_count(value, what):
    """A strictly positive integer that is not a bool."""
    ok = isinstance(value, numbers.Integral) and not isinstance(value, bool) and value >= 1
    return int(value) if ok else _fail(f"{what}: expected a positive integer, got {value!r}")


def validate_shapes(q_shape, k_shape, v_shape, allow_gqa=False, head_dims=PREFILL_HEAD_DIMS):
    """Checks [T,H,D] shapes and returns the group size Hq // Hkv (baseline_adapter.py:23-34)."""
    shapes = {"q": tuple(q_shape), "k": tuple(k_shape), "v": tuple(v_shape)}
    for name, shape in shapes.items():
        if len(shape) != 3 or min(shape) < 1:
            _fail(f"{name} must be a non-empty [T,H,D] tensor, got {shape}")
    (tq, hq, dq), (tk, hk, dk) = shapes["q"], shapes["k"]
    if shapes["v"] != shapes["k"]:
        _fail(f"k and v must have the same shape, got {shapes['k']} and {shapes['v']}")
    if tq != tk or dq != dk:
        _fail(f"q and k must agree on tokens and head_dim, got {shapes['q']} and {shapes['k']}")
    if dq not in head_dims:
        _fail(f"head_dim {dq} unsupported: need a multiple of 8 between {head_dims[0]} and {head_dims[-1]}")
    if hq % hk:
        _fail(f"{hq} query heads cannot be grouped over {hk} KV heads")
    if hq != hk and not allow_gqa:
        _fail("this entry point is MHA only (Hq must equal Hkv)")
    return hq // hk


def validate_config(config):
    """chunk_size / topk / causal / dropout rules (baseline_adapter.py:37-43)."""
    _as_count(config.get("chunk_size"), "chunk_size")
    if _as_count(config.get("topk"), "topk") > MAX_TOPK:
        _fail(f"topk above {MAX_TOPK} is not supported ({MAX_TOPK - 1} routed blocks at most)")
    if config.get("causal", True) is not True:
        _fail("MoBA prefill is causal; causal=False is not supported")
    if config.get("dropout", 0.0) != 0:
        _fail("attention dropout is not supported")


def _check_qkv(q, k, v):
    for name, t in (("q", q), ("k", k), ("v", v)):
        if not isinstance(t, torch.Tensor):
            _fail(f"{name} must be a torch.Tensor")
        if t.dim() != 3:
            _fail(f"{name} must be [T,H,D], got shape {tuple(t.shape)}")
        if t.dtype not in SUPPORTED_DTYPES:
            _fail(f"{name} has dtype {t.dtype}; the CUDA path takes {SUPPORTED_DTYPES}")
        if not t.is_cuda:
            _fail(f"{name} must live on a CUDA device")
        if t.stride(-1) != 1:
            _fail(f"{name}: the head_dim axis must be contiguous")
    if not (q.device == k.device == v.device) or not (q.dtype == k.dtype == v.dtype):
        _fail("q, k and v must share one device and one dtype")


_CU_MEMO = {}   # id(tensor) -> (weak reference, version counter, offsets)


def _known_offsets(cu_seqlens):
    """cu_seqlens as a Python list.  Reading it is the call's only device-to-host copy, and it waits for everything
    already enqueued on the stream; a caller that passes the same, unmodified tensor again (every layer of a model,
    every step of a loop) gets the list remembered from the first call instead, so the host keeps running ahead of the
    device.  The tensor's version counter, which every in-place write through torch increments, guards the memo."""
    import weakref
    entry = _CU_MEMO.get(id(cu_seqlens))
    if entry is not None and entry[0]() is cu_seqlens and entry[1] == cu_seqlens._version:
        return entry[2]
    offsets = cu_seqlens.tolist()
    for key in [k for k, e in _CU_MEMO.items() if e[0]() is None]:
        del _CU_MEMO[key]
    if len(_CU_MEMO) >= 32:
        _CU_MEMO.pop(next(iter(_CU_MEMO)))
    _CU_MEMO[id(cu_seqlens)] = (weakref.ref(cu_seqlens), cu_seqlens._version, offsets)
    return offsets


def _check_cu_seqlens(cu_seqlens, q):
    if not isinstance(cu_seqlens, torch.Tensor):
        _fail("cu_seqlens must be a torch.Tensor")
    if cu_seqlens.dtype != torch.int32 or not cu_seqlens.is_cuda or cu_seqlens.device != q.device:
        _fail("cu_seqlens must be an int32 tensor on q's CUDA device")
    if cu_seqlens.dim() != 1 or cu_seqlens.numel() < 2 or not cu_seqlens.is_contiguous():
        _fail("cu_seqlens must be a contiguous 1-D tensor of B+1 >= 2 offsets")
    offsets = _known_offsets(cu_seqlens)
    increasing = all(b > a for a, b in zip(offsets, offsets[1:]))
    if offsets[0] != 0 or offsets[-1] != q.shape[0] or not increasing:
        _fail(f"cu_seqlens must run from 0 to T in strictly increasing steps, got {offsets}")
    return offsets


def _validate(q, k, v, cu_seqlens, *, allow_gqa=False, max_seqlen=None, config=None):
    """Whole-call contract (baseline_adapter.py:46-76).  Returns cu_seqlens as a Python list."""
    _check_qkv(q, k, v)
    validate_shapes(q.shape, k.shape, v.shape, allow_gqa)
    offsets = _check_cu_seqlens(cu_seqlens, q)
    if max_seqlen is not None:
        longest = max(b - a for a, b in zip(offsets, offsets[1:]))
        if _as_count(max_seqlen, "max_seqlen") != longest:
            _fail(f"max_seqlen is {max_seqlen} but the longest sequence has {longest} tokens")
    if config is not None:
        validate_config(config)
    return offsets
