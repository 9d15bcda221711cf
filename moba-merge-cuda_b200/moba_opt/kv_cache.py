"""Inference KV caches with incremental MoBA attention: `PagedKVCache` and `ContiguousKVCache`.

The public surface, the meaning of every argument and the error behaviour are the reference's
(src/moba_opt/kv_cache.py:36-300); the way the host gets there is built around the C ABI of
libmoba_b200.so instead:

  * every append - one token or a whole prompt - is one `moba_prefill_to_cache` launch (pages and the
    means of the chunks it completes in a single pass over K); the host builds no per-token index
    arrays for it;
  * the device copies of the page table and the lengths are edited, never re-uploaded: a call
    stages the entries that changed (newly mapped pages, new lengths) together with whatever
    small vectors its launches need in one pinned block, sends that block with one asynchronous
    copy and applies it with `moba_cache_update`;
  * the union lists and the split-K workspace of `attend` are kept between calls of the same shape.

Operations are serialised by a lock and bound to the CUDA stream that was current when the cache was
built; other streams and external graph capture are refused.  Validation failures never modify the
cache, and the CPU layout is committed only after every launch of a call was accepted.

Differences to the reference, all by design of the CUDA kernels: head_dim must be a multiple of 8 (8..256), chunk_size may be up to 8192 (reference: 1024), topk up
to 17 (reference: 9), and routing always breaks exact score ties towards the lowest chunk.
"""
import ctypes
import enum
import threading
from dataclasses import dataclass

import numpy as np
import torch

from . import _ext
from .cache_layout import PageAllocator, positive_int
from .grouped_attention import _status_word

MAX_CHUNK = 8192
MAX_TOPK = 17


# ----------------------------------------------------------------------------------------- native side
class CacheDesc(ctypes.Structure):
    """Mirror of moba_cache_desc in include/moba_b200.h."""
    _fields_ = ([(n, ctypes.c_int32) for n in ("batch_slots", "max_seq_len", "page_size", "num_pages", "table_width",
                                               "chunk_size", "max_chunks", "hkv", "dim", "flags")]
                + [(n, ctypes.c_void_p) for n in ("k_cache", "v_cache", "table", "lengths", "means")])


_P, _VP, _I, _SZ = ctypes.POINTER(CacheDesc), ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
# entry point -> (result type, argument types); every decode entry point of include/moba_b200.h is bound from this table
_DECODE_ABI = {
    "moba_cache_update": (_I, [_P, _VP, _I, _VP, _VP, _I, _I, _VP]),
    "moba_decode_metadata": (_I, [_P, _VP, _VP, _VP, _I, _I, _VP]),
    "moba_decode_append": (_I, [_P, _VP, _VP, _VP, _VP, _I, _VP, _VP]),
    "moba_decode_means": (_I, [_P, _VP, _VP, _I, _I, _VP, _VP]),
    "moba_decode_step_begin": (_I, [_P, _VP, _VP, _VP, _I, _I, _VP, _VP, _VP, _VP, _VP, _VP, _VP, _VP]),
    "moba_decode_stage_inputs": (_I, [_VP, _VP, _SZ, _VP, _VP, _SZ, _VP, _VP, _SZ, _VP]),
    "moba_prefill_to_cache": (_I, [_P, _VP, _VP, _VP, _VP, _VP, _I, _I, _VP, _VP]),
    "moba_decode_union_capacity": (_I, [_I, _I, _I, _I]),
    "moba_decode_route": (_I, [_P, _VP, _VP, _VP, _I, _I, _I, _I, _VP, _VP, _VP, _VP, _VP, _VP]),
    "moba_decode_attend_workspace_bytes": (_SZ, [_P, _I, _I, _I]),
    "moba_decode_attend": (_I, [_P, _VP, _VP, _VP, _I, _I, _VP, _I, _VP, _VP, _VP, _I, _VP, _SZ, _VP, _VP, _VP, _VP]),
}


def decode_library():
    """libmoba_b200.so with the decode entry points typed (once per process)."""
    lib = _ext.lib()
    if not getattr(lib, "_decode_abi_bound", False):
        if lib.moba_abi_sizeof(1) != ctypes.sizeof(CacheDesc):
            raise ImportError("libmoba_b200.so was built from another revision of include/moba_b200.h (moba_cache_desc)")
        for name, (restype, argtypes) in _DECODE_ABI.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = restype, argtypes
        lib._decode_abi_bound = True
    return lib


# ----------------------------------------------------------------------------------------- small contracts
def _ints(values, name):
    """A Python sequence of ints or a CPU int32/int64 vector, as a tuple of ints (kv_cache.py:16-25 of the reference)."""
    if isinstance(values, torch.Tensor):
        ok = values.device.type == "cpu" and values.dim() == 1 and values.dtype in (torch.int32, torch.int64)
        if not ok:
            raise ValueError(f"{name} must be a Python sequence or CPU int32/int64 vector")
        values = values.tolist()
    if not isinstance(values, (list, tuple)):
        raise ValueError(f"{name} must be a Python sequence or CPU integer vector")
    if any(isinstance(x, bool) or not isinstance(x, int) for x in values):
        raise ValueError(f"{name} must contain integers")
    return tuple(values)


def wants_dense(mode, topk):
    """Whether a request means dense attention: mode 'dense', or 'moba' with topk == 1 (kv_cache.py:28-33)."""
    if mode not in ("moba", "dense"):
        raise ValueError("mode must be moba or dense")
    if positive_int(topk, "topk") > MAX_TOPK:
        raise ValueError(f"topk must be in [1,{MAX_TOPK}]")
    return mode == "dense" or topk == 1


class AppendResult:
    """Where an append put its tokens: `sequence_ids` and `positions`, one entry per appended token in input order
    (the reference's frozen dataclass, kv_cache.py:36-40).  The two tuples are built on first use: a whole-prompt
    append has no use for 10^5 Python integers unless somebody asks."""
    __slots__ = ("_ids", "_starts", "_counts", "_cache")

    def __init__(self, ids, starts, counts):
        self._ids, self._starts, self._counts, self._cache = tuple(ids), tuple(starts), tuple(counts), None

    def _expand(self):
        if self._cache is None:
            seqs = tuple(s for s, n in zip(self._ids, self._counts) for _ in range(n))
            pos = tuple(p for first, n in zip(self._starts, self._counts) for p in range(first, first + n))
            self._cache = (seqs, pos)
        return self._cache

    @property
    def sequence_ids(self):
        return self._expand()[0]

    @property
    def positions(self):
        return self._expand()[1]

    def __eq__(self, other):
        return isinstance(other, AppendResult) and self._expand() == other._expand()

    def __repr__(self):
        return f"AppendResult(sequence_ids={self.sequence_ids}, positions={self.positions})"


@dataclass(frozen=True)
class DecodeResult:
    output: torch.Tensor
    lse: torch.Tensor
    selected_blocks: object   # [Nq,Hq,slots] int32, own chunk first, -1 padded; None for dense
    sequence_ids: tuple
    positions: tuple


class CacheLife(enum.Enum):
    READY = "ready"        # ordinary operations allowed
    LEASED = "leased"      # a PreparedDecode owns the cache
    BROKEN = "broken"      # a launch failed: contents undefined


@dataclass(frozen=True)
class TensorRule:
    """What a q / k / v argument has to satisfy; `check` raises ValueError with the reference's wording."""
    name: str
    heads: object = None        # exact head count, or None
    tokens: object = None       # exact token count, or None
    finite: bool = True

    def check(self, cache, t):
        n = self.name
        if not isinstance(t, torch.Tensor) or t.dim() != 3:
            raise ValueError(f"{n} must be [N,H,D]")
        if t.device != cache.device or t.dtype != cache.dtype:
            raise ValueError(f"{n} must match cache device and dtype")
        if t.requires_grad:
            raise ValueError("KV cache/decode is inference-only; detach Q/K/V")
        if t.shape[0] < 1 or t.shape[1] < 1 or t.shape[2] != cache.head_dim:
            raise ValueError(f"{n} has an invalid shape")
        if t.stride(-1) != 1:
            raise ValueError(f"{n} last dimension must be contiguous")
        if self.heads is not None and t.shape[1] != self.heads:
            raise ValueError(f"{n} KV head count differs from cache")
        if self.tokens is not None and t.shape[0] != self.tokens:
            raise ValueError(f"{n} token count differs")
        if self.finite and not bool(torch.isfinite(t).all()):      # reads a flag back: the host waits for the stream
            raise ValueError(f"{n} contains NaN/Inf")


class HostStaging:
    """Small int32 vectors of a call, sent to the device as one block: the vectors are laid out back to back in a
    pinned buffer, copied with one asynchronous transfer and returned as views of one device tensor.  A few pinned
    buffers are used in turn, so the host waits only if the copy that last used a buffer is still in flight."""

    def __init__(self, device, slots=4, words=4096):
        self.device = device
        self._pinned = [torch.empty(words, dtype=torch.int32, pin_memory=True) for _ in range(slots)]
        self._busy = [None] * slots
        self._next = 0

    def send(self, *vectors):
        arrays = [np.ascontiguousarray(v, dtype=np.int32).reshape(-1) for v in vectors]
        sizes = [a.size for a in arrays]
        total = sum(sizes)
        if total == 0:
            empty = torch.empty(0, dtype=torch.int32, device=self.device)
            return tuple(empty for _ in arrays)
        slot = self._next
        self._next = (slot + 1) % len(self._pinned)
        if self._busy[slot] is not None:
            self._busy[slot].synchronize()
        if self._pinned[slot].numel() < total:
            self._pinned[slot] = torch.empty(max(total, 2 * self._pinned[slot].numel()), dtype=torch.int32, pin_memory=True)
        host = self._pinned[slot].numpy()
        at = 0
        for a in arrays:
            host[at:at + a.size] = a
            at += a.size
        dev = torch.empty(total, dtype=torch.int32, device=self.device)
        dev.copy_(self._pinned[slot][:total], non_blocking=True)
        done = torch.cuda.Event()
        done.record()
        self._busy[slot] = done
        return dev.split(sizes)


# ----------------------------------------------------------------------------------------- the cache
class PagedKVCache:
    def __init__(self, batch_size, max_seq_len, num_kv_heads, head_dim, *, page_size=16, num_pages=None, chunk_size=128,
                 dtype=torch.bfloat16, device="cuda"):
        batch_size = positive_int(batch_size, "batch_size")
        max_seq_len = positive_int(max_seq_len, "max_seq_len")
        page_size = positive_int(page_size, "page_size")
        self.num_kv_heads = positive_int(num_kv_heads, "num_kv_heads")
        self.head_dim = positive_int(head_dim, "head_dim")
        if self.head_dim > 256 or self.head_dim % 8:
            raise ValueError("decode head_dim must be a multiple of 8 in [8,256]")
        self.chunk_size = positive_int(chunk_size, "chunk_size")
        if self.chunk_size > MAX_CHUNK:
            raise ValueError(f"cache chunk_size must be <={MAX_CHUNK}")
        if dtype not in (torch.bfloat16, torch.float16):
            raise ValueError("cache dtype must be BF16 or FP16")
        wanted = torch.device(device)
        if wanted.type != "cuda":
            raise ValueError("cache device must be CUDA")
        if num_pages is None:
            num_pages = batch_size * (-(-max_seq_len // page_size))
        self._layout = PageAllocator(batch_size, max_seq_len, page_size, num_pages, self.chunk_size)
        self.dtype = dtype
        self._lock = threading.RLock()
        self._life = CacheLife.READY
        self._owner = None                    # the PreparedDecode that holds the lease, if any
        # The NaN/Inf check of q, k, v (the reference's contract) reads a flag back, so every eager call waits for the
        # device.  A caller that vouches for its tensors may set this to False, as prepare_decode(check_finite=False)
        # does for prepared steps; it is an attribute rather than an argument to leave the reference's signatures alone.
        self.check_finite = True
        self._lib = decode_library()
        with torch.cuda.device(wanted):
            self.device = torch.device("cuda", torch.cuda.current_device())
            self._stream = torch.cuda.current_stream(self.device).cuda_stream
            lay = self._layout
            self.k_cache = torch.empty((lay.num_pages, page_size, self.num_kv_heads, self.head_dim), dtype=dtype, device=self.device)
            self.v_cache = torch.empty_like(self.k_cache)
            self._table = torch.full((batch_size, lay.table_width), -1, dtype=torch.int32, device=self.device)
            self._lengths = torch.zeros(batch_size, dtype=torch.int32, device=self.device)
            self._max_chunks = -(-max_seq_len // self.chunk_size)
            self._means = torch.empty((batch_size, self._max_chunks, self.num_kv_heads, self.head_dim), dtype=dtype,
                                      device=self.device)
            self._candidate_count = 0
            self._status = _status_word(self.device)
            self._staging = HostStaging(self.device)
            self._attend_buffers = {}         # (rows, Hq, slots, umax) -> union lists + split-K workspace, kept between calls

    # ------------------------------------------------------------------ views of the CPU layout
    @property
    def lengths(self):
        return self._owner.lengths if self._owner is not None else self._layout.lengths

    @property
    def page_table(self):
        """Immutable CPU snapshot of the logical->physical page map."""
        return self._owner.page_table if self._owner is not None else self._layout.tables

    # ------------------------------------------------------------------ plumbing shared with PreparedDecode
    def _desc(self):
        lay = self._layout
        d = CacheDesc(lay.batch_size, lay.max_seq_len, lay.page_size, lay.num_pages, lay.table_width, self.chunk_size,
                      self._max_chunks, self.num_kv_heads, self.head_dim, 1 if self.dtype == torch.float16 else 0)   # MOBA_CACHE_FP16
        d.k_cache, d.v_cache = self.k_cache.data_ptr(), self.v_cache.data_ptr()
        d.table, d.lengths, d.means = self._table.data_ptr(), self._lengths.data_ptr(), self._means.data_ptr()
        return d

    def _launch(self, name, *args):
        """One C-ABI call on the cache's stream; a refused launch leaves the cache contents undefined."""
        with _ext.nvtx(name):
            status = getattr(self._lib, name)(*args, ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream))
        if status != 0:
            self._life = CacheLife.BROKEN
        _ext.check(status, name)

    def _guard(self, *, lease_ok=False):
        """Raises unless an operation may run now: cache intact, not leased (unless the lease holder asks), no foreign
        graph capture, on the cache's own stream."""
        if self._life is CacheLife.BROKEN:
            raise RuntimeError("CUDA execution failed; discard this cache")
        if self._life is CacheLife.LEASED and not lease_ok:
            raise ValueError("prepared decode owns cache; close it before ordinary cache operations")
        if torch.cuda.is_current_stream_capturing():
            raise ValueError("CUDA Graph capture is unsupported for this cache API")
        if torch.cuda.current_stream(self.device).cuda_stream != self._stream:
            raise ValueError("cross-stream cache access is unsupported")

    def _refuse_pool_aliases(self, *tensors):
        pools = {self.k_cache.untyped_storage().data_ptr(), self.v_cache.untyped_storage().data_ptr()}
        if any(t.untyped_storage().data_ptr() in pools for t in tensors):
            raise ValueError("append inputs must not alias KV cache storage; clone first")

    def _routable(self, lengths):
        """Chunks some query could be routed to: every complete chunk that is not the last chunk of its sequence."""
        c = self.chunk_size
        return sum(max(0, -(-n // c) - 1) for n in lengths)

    def _segments(self, token_count, sequence_ids, cu_seqlens):
        """(sequence ids, tokens per sequence) of an append of `token_count` tokens."""
        ids = self._layout.validate_ids(_ints(sequence_ids, "sequence_ids"), unique=True)
        cu = tuple(range(len(ids) + 1)) if cu_seqlens is None else _ints(cu_seqlens, "cu_seqlens")
        if len(cu) != len(ids) + 1 or cu[0] != 0 or cu[-1] != token_count:
            raise ValueError("append cu_seqlens must start at 0 and end at N")
        counts = tuple(b - a for a, b in zip(cu, cu[1:]))
        if min(counts) <= 0:
            raise ValueError("append sequences must be nonempty")
        return ids, counts

    # ------------------------------------------------------------------ append
    def prepare_decode(self, sequence_ids, num_q_heads, *, topk=4, mode="moba", check_finite=True, stable_routes=False):
        from .prepared_decode import PreparedDecode
        return PreparedDecode(self, sequence_ids, num_q_heads, topk=topk, mode=mode, check_finite=check_finite,
                              stable_routes=stable_routes)

    def _checked_kv(self, k, v, check_finite=True):
        check_finite = check_finite and self.check_finite
        TensorRule("k", heads=self.num_kv_heads, finite=check_finite).check(self, k)
        TensorRule("v", heads=self.num_kv_heads, tokens=k.shape[0], finite=check_finite).check(self, v)

    def _store(self, k, v, ids, counts, extra=()):
        """Plans the append on the CPU, sends the changed table entries, the new lengths, the segment description and
        the caller's `extra` vectors in one block, applies the edits and stores the tokens with their chunk means.
        Returns (plan, first position of every segment, device views of `extra`); the CPU layout is committed once
        both launches were accepted."""
        lay = self._layout
        starts = [lay.lengths[s] for s in ids]
        plan = lay.plan_append(ids, counts, tokens=False)
        cu = np.zeros(len(ids) + 1, dtype=np.int32)
        np.cumsum(counts, out=cu[1:])
        edits = np.asarray(plan.page_edits, dtype=np.int32).reshape(-1, 3)
        sent = self._staging.send(edits, ids, [plan.lengths[s] for s in ids], starts, cu, *extra)
        d_edits, d_ids, d_lengths, d_starts, d_cu = sent[:5]
        desc = self._desc()
        self._launch("moba_cache_update", ctypes.byref(desc), d_edits.data_ptr() if len(edits) else None, len(edits),
                     d_ids.data_ptr(), d_lengths.data_ptr(), len(ids), 0)
        c = self.chunk_size
        touched = max((first + n - 1) // c - first // c + 1 for first, n in zip(starts, counts))
        k, v = k.contiguous(), v.contiguous()
        self._launch("moba_prefill_to_cache", ctypes.byref(desc), k.data_ptr(), v.data_ptr(), d_ids.data_ptr(), d_starts.data_ptr(),
                     d_cu.data_ptr(), len(ids), touched, self._status.data_ptr())
        lay.commit(plan)
        self._candidate_count = self._routable(plan.lengths)
        return plan, starts, sent[5:]

    @torch.no_grad()
    def append(self, k, v, *, sequence_ids, cu_seqlens=None):
        with self._lock, torch.cuda.device(self.device):
            self._guard()
            self._checked_kv(k, v)
            self._refuse_pool_aliases(k, v)
            ids, counts = self._segments(k.shape[0], sequence_ids, cu_seqlens)
            _, starts, _ = self._store(k, v, ids, counts)
            return AppendResult(ids, starts, counts)

    @torch.no_grad()
    def append_prefill(self, k, v, *, sequence_ids, cu_seqlens=None, check_finite=True):
        """`append` for the hand-off from a prefill pass: same contract and resulting cache state; returns the new
        lengths of the given sequences instead of per-token positions.  `check_finite=False` leaves out the NaN/Inf
        check of k and v, which reads a flag back from the device and so makes the host wait for everything enqueued
        before (as `prepare_decode` offers for decode steps)."""
        with self._lock, torch.cuda.device(self.device):
            self._guard()
            self._checked_kv(k, v, check_finite)
            self._refuse_pool_aliases(k, v)
            ids, counts = self._segments(k.shape[0], sequence_ids, cu_seqlens)
            plan, _, _ = self._store(k, v, ids, counts)
            return tuple(plan.lengths[s] for s in ids)

    # ------------------------------------------------------------------ attend
    def _query_rows(self, q, sequence_ids, positions):
        TensorRule("q", finite=self.check_finite).check(self, q)
        if q.shape[1] % self.num_kv_heads:
            raise ValueError("Hq must be a multiple of Hkv")
        ids = self._layout.validate_ids(_ints(sequence_ids, "sequence_ids"))
        if len(ids) != q.shape[0]:
            raise ValueError("one sequence ID per query row required")
        lengths = self.lengths
        pos = tuple(lengths[s] - 1 for s in ids) if positions is None else _ints(positions, "positions")
        if len(pos) != len(ids) or any(p < 0 or p >= lengths[s] for s, p in zip(ids, pos)):
            raise ValueError("query positions must refer to cached tokens")
        if q.shape[0] * q.shape[1] >= 2 ** 31:
            raise ValueError("query grid exceeds int32 capacity")
        return ids, pos

    def _attend_scratch(self, rows, hq, slots, umax, desc):
        """Union lists and split-K workspace for this launch shape.  Their contents do not outlive a call (the kernel
        leaves the workspace's arrival counters at zero), so one set per shape serves every call."""
        key = (rows, hq, slots, umax)
        found = self._attend_buffers.get(key)
        if found is None:
            if len(self._attend_buffers) >= 8:
                self._attend_buffers.pop(next(iter(self._attend_buffers)))
            hk, dev = self.num_kv_heads, self.device
            nbytes = self._lib.moba_decode_attend_workspace_bytes(ctypes.byref(desc), rows, hq, slots)
            found = dict(u_chunk=torch.empty((rows, hk, umax), dtype=torch.int32, device=dev),
                         u_mask=torch.empty((rows, hk, umax), dtype=torch.int32, device=dev),
                         u_count=torch.empty((rows, hk), dtype=torch.int32, device=dev),
                         workspace=torch.zeros(nbytes, dtype=torch.uint8, device=dev), nbytes=nbytes)
            self._attend_buffers[key] = found
        return found

    def _attend_rows(self, q, ids, pos, topk, dense, d_ids, d_pos):
        """Routing (unless dense) and attention for validated query rows whose sequence ids and positions are already on
        the device."""
        q = q.contiguous()
        rows, hq, _ = q.shape
        desc, lib = self._desc(), self._lib
        out = torch.empty_like(q)
        lse = torch.empty((rows, hq), dtype=torch.float32, device=self.device)
        selected, remote = None, 0
        if dense:
            slots, umax = self._max_chunks, 1
        else:
            # result width as in the reference: min(topk-1, routable chunks in the whole cache)
            remote = min(int(topk) - 1, self._candidate_count)
            width = max(1, remote, max(pos) // self.chunk_size)
            if width * hq * rows >= 2 ** 31:
                raise ValueError("route score grid exceeds int32 capacity")
            slots, umax = remote + 1, lib.moba_decode_union_capacity(hq, self.num_kv_heads, remote, width)
            selected = torch.empty((rows, hq, slots), dtype=torch.int32, device=self.device)
        buf = self._attend_scratch(rows, hq, slots, umax, desc)
        union = (buf["u_chunk"].data_ptr(), buf["u_mask"].data_ptr(), buf["u_count"].data_ptr())
        if not dense:
            self._launch("moba_decode_route", ctypes.byref(desc), q.data_ptr(), d_ids.data_ptr(), d_pos.data_ptr(), rows, hq, remote,
                         width, None, selected.data_ptr(), *union)
        self._launch("moba_decode_attend", ctypes.byref(desc), q.data_ptr(), d_ids.data_ptr(), d_pos.data_ptr(), rows, hq,
                     None if dense else selected.data_ptr(), slots, *(union if not dense else (None, None, None)), umax,
                     buf["workspace"].data_ptr(), buf["nbytes"], out.data_ptr(), lse.data_ptr(), self._status.data_ptr())
        return DecodeResult(out, lse, selected, ids, pos)

    @torch.no_grad()
    def attend(self, q, *, sequence_ids, positions=None, topk=4, mode="moba"):
        with self._lock, torch.cuda.device(self.device):
            self._guard()
            dense = wants_dense(mode, topk)
            ids, pos = self._query_rows(q, sequence_ids, positions)
            d_ids, d_pos = self._staging.send(ids, pos)
            return self._attend_rows(q, ids, pos, topk, dense, d_ids, d_pos)

    @torch.no_grad()
    def append_and_attend(self, q, k, v, *, sequence_ids, cu_seqlens=None, topk=4, mode="moba"):
        """Appends k, v and attends with one query per appended token (token i of a segment sees the cache up to and
        including itself)."""
        with self._lock, torch.cuda.device(self.device):
            self._guard()
            dense = wants_dense(mode, topk)
            self._checked_kv(k, v)
            TensorRule("q", tokens=k.shape[0], finite=self.check_finite).check(self, q)
            self._refuse_pool_aliases(q, k, v)
            if q.shape[1] % self.num_kv_heads:
                raise ValueError("Hq must be a multiple of Hkv")
            if q.shape[0] * q.shape[1] >= 2 ** 31:
                raise ValueError("query grid exceeds int32 capacity")
            ids, counts = self._segments(k.shape[0], sequence_ids, cu_seqlens)
            starts = [self._layout.lengths[s] for s in ids]
            row_ids = np.repeat(np.asarray(ids, dtype=np.int32), counts)
            row_pos = np.concatenate([np.arange(first, first + n, dtype=np.int32) for first, n in zip(starts, counts)])
            _, _, (d_ids, d_pos) = self._store(k, v, ids, counts, extra=(row_ids, row_pos))
            return self._attend_rows(q, tuple(row_ids.tolist()), tuple(row_pos.tolist()), topk, dense, d_ids, d_pos)

    # ------------------------------------------------------------------ reset / read-back
    @torch.no_grad()
    def reset(self, sequence_ids=None):
        with self._lock, torch.cuda.device(self.device):
            self._guard()
            ids = tuple(range(self._layout.batch_size)) if sequence_ids is None else _ints(sequence_ids, "sequence_ids")
            staged = self._layout.clone()      # a copy first: a failure while staging publishes nothing
            staged.reset(ids)
            d_ids, d_zero = self._staging.send(ids, [0] * len(ids))
            desc = self._desc()
            self._launch("moba_cache_update", ctypes.byref(desc), None, 0, d_ids.data_ptr(), d_zero.data_ptr(), len(ids), 1)
            self._layout = staged
            self._candidate_count = self._routable(staged.lengths)

    @torch.no_grad()
    def materialize(self, sequence_id):
        """Reads one sequence's K/V back in logical order (diagnostics and tests only)."""
        with self._lock, torch.cuda.device(self.device):
            self._guard(lease_ok=True)
            sid = self._layout.validate_ids([sequence_id])[0]
            page = self._layout.page_size
            pos = torch.arange(self.lengths[sid], device=self.device)
            pages = self._table[sid, pos // page].long()
            return self.k_cache[pages, pos % page], self.v_cache[pages, pos % page]


class ContiguousKVCache(PagedKVCache):
    """One physical slab per sequence: a paged cache whose page is a whole sequence
    (kv_cache.py:294-300 of the reference)."""

    def __init__(self, batch_size, max_seq_len, num_kv_heads, head_dim, **kwargs):
        if "page_size" in kwargs or "num_pages" in kwargs:
            raise ValueError("ContiguousKVCache owns page_size/num_pages")
        super().__init__(batch_size, max_seq_len, num_kv_heads, head_dim, page_size=max_seq_len, num_pages=batch_size,
                         **kwargs)
