"""Inference KV caches with incremental MoBA attention: `PagedKVCache` and `ContiguousKVCache`.

Public surface, argument meaning and error behaviour follow the reference
(src/moba_opt/kv_cache.py:36-300).  The cache owns the page pools and the CPU page allocator; all
device work (append through the page table, chunk means, routing, split-K paged attention) is done
by the decode kernels of libmoba_b200.so.  Operations are serialised by a lock and bound to the CUDA
stream that was current when the cache was built; other streams and external graph capture are
rejected.  Validation failures never modify the cache.

Differences to the reference, all by design of the CUDA kernels: the cache dtype is bf16 only,
head_dim must be a multiple of 8 (8..256), chunk_size may be up to 8192 (reference: 1024), topk up
to 17 (reference: 9), and routing always breaks exact score ties towards the lowest chunk.
"""
import ctypes
import threading
from dataclasses import dataclass

import torch

from . import _ext
from .cache_layout import PageAllocator, positive_int
from .grouped_attention import _status_word

MAX_CHUNK = 8192
MAX_TOPK = 17


def _ints(values, name):
    """Python sequence or CPU int32/int64 vector -> tuple of ints (kv_cache.py:16-25)."""
    if isinstance(values, torch.Tensor):
        if values.device.type != "cpu" or values.dim() != 1 or values.dtype not in (torch.int32, torch.int64):
            raise ValueError(f"{name} must be a Python sequence or CPU int32/int64 vector")
        values = values.tolist()
    if not isinstance(values, (list, tuple)):
        raise ValueError(f"{name} must be a Python sequence or CPU integer vector")
    for x in values:
        if isinstance(x, bool) or not isinstance(x, int):
            raise ValueError(f"{name} must contain integers")
    return tuple(values)


def _mode(mode, topk):
    """True when the request means dense attention: mode 'dense' or topk == 1 (kv_cache.py:28-33)."""
    if mode not in ("moba", "dense"):
        raise ValueError("mode must be moba or dense")
    if positive_int(topk, "topk") > MAX_TOPK:
        raise ValueError(f"topk must be in [1,{MAX_TOPK}]")
    return mode == "dense" or topk == 1


@dataclass(frozen=True)
class AppendResult:
    sequence_ids: tuple
    positions: tuple


@dataclass(frozen=True)
class DecodeResult:
    output: torch.Tensor
    lse: torch.Tensor
    selected_blocks: object   # [Nq,Hq,slots] int32, own chunk first, -1 padded; None for dense
    sequence_ids: tuple
    positions: tuple


class _CacheDesc(ctypes.Structure):
    """Mirror of moba_cache_desc in include/moba_b200.h."""
    _fields_ = ([(n, ctypes.c_int32) for n in ("batch_slots", "max_seq_len", "page_size", "num_pages", "table_width",
                                               "chunk_size", "max_chunks", "hkv", "dim")]
                + [(n, ctypes.c_void_p) for n in ("k_cache", "v_cache", "table", "lengths", "means")])


def _bind(lib):
    if getattr(lib, "_decode_bound", False):
        return
    P, vp, i, sz = ctypes.POINTER(_CacheDesc), ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
    lib.moba_decode_metadata.argtypes = [P, vp, vp, vp, i, i, vp]
    lib.moba_decode_append.argtypes = [P, vp, vp, vp, vp, i, vp, vp]
    lib.moba_decode_means.argtypes = [P, vp, vp, i, i, vp, vp]
    lib.moba_decode_step_begin.argtypes = [P, vp, vp, vp, i, i, vp, vp, vp, vp, vp, vp, vp, vp]
    lib.moba_decode_stage_inputs.argtypes = [vp, vp, ctypes.c_size_t, vp, vp, ctypes.c_size_t, vp, vp, ctypes.c_size_t, vp]
    lib.moba_prefill_to_cache.argtypes = [P, vp, vp, vp, vp, vp, i, i, vp, vp]
    lib.moba_decode_union_capacity.argtypes = [i, i, i, i]
    lib.moba_decode_route.argtypes = [P, vp, vp, vp, i, i, i, i, vp, vp, vp, vp, vp, vp]
    lib.moba_decode_attend_workspace_bytes.restype = sz
    lib.moba_decode_attend_workspace_bytes.argtypes = [P, i, i, i]
    lib.moba_decode_attend.argtypes = [P, vp, vp, vp, i, i, vp, i, vp, vp, vp, i, vp, sz, vp, vp, vp, vp]
    lib._decode_bound = True


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
        if dtype != torch.bfloat16:
            raise ValueError("cache dtype must be BF16")
        wanted = torch.device(device)
        if wanted.type != "cuda":
            raise ValueError("cache device must be CUDA")
        if num_pages is None:
            num_pages = batch_size * (-(-max_seq_len // page_size))
        self._layout = PageAllocator(batch_size, max_seq_len, page_size, num_pages, self.chunk_size)
        self.dtype = dtype
        self._lock = threading.RLock()
        self._prepared_owner = None
        self._invalid = False
        self._lib = _ext.lib()
        _bind(self._lib)
        with torch.cuda.device(wanted):
            self.device = torch.device("cuda", torch.cuda.current_device())
            self._stream = torch.cuda.current_stream(self.device).cuda_stream
            lay = self._layout
            pool = (lay.num_pages, page_size, self.num_kv_heads, self.head_dim)
            self.k_cache = torch.empty(pool, dtype=dtype, device=self.device)
            self.v_cache = torch.empty_like(self.k_cache)
            self._table = torch.full((batch_size, lay.table_width), -1, dtype=torch.int32, device=self.device)
            self._lengths = torch.zeros(batch_size, dtype=torch.int32, device=self.device)
            self._max_chunks = -(-max_seq_len // self.chunk_size)
            self._means = torch.empty((batch_size, self._max_chunks, self.num_kv_heads, self.head_dim), dtype=dtype,
                                      device=self.device)
            self._candidate_count = 0
            self._status = _status_word(self.device)

    # ------------------------------------------------------------------ views of the CPU layout
    @property
    def lengths(self):
        owner = self._prepared_owner
        return owner.lengths if owner is not None else self._layout.lengths

    @property
    def page_table(self):
        """Immutable CPU snapshot of the logical->physical page map."""
        owner = self._prepared_owner
        return owner.page_table if owner is not None else self._layout.tables

    # ------------------------------------------------------------------ helpers
    def _desc(self):
        lay = self._layout
        d = _CacheDesc(lay.batch_size, lay.max_seq_len, lay.page_size, lay.num_pages, lay.table_width, self.chunk_size,
                       self._max_chunks, self.num_kv_heads, self.head_dim)
        d.k_cache, d.v_cache = self.k_cache.data_ptr(), self.v_cache.data_ptr()
        d.table, d.lengths, d.means = self._table.data_ptr(), self._lengths.data_ptr(), self._means.data_ptr()
        return d

    def _cuda_stream(self):
        return ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def _check_stream(self, *, allow_prepared=False):
        if self._invalid:
            raise RuntimeError("CUDA execution failed; discard this cache")
        if self._prepared_owner is not None and not allow_prepared:
            raise ValueError("prepared decode owns cache; close it before ordinary cache operations")
        if torch.cuda.is_current_stream_capturing():
            raise ValueError("CUDA Graph capture is unsupported for this cache API")
        if torch.cuda.current_stream(self.device).cuda_stream != self._stream:
            raise ValueError("cross-stream cache access is unsupported")

    def _tensor(self, tensor, name, *, expected_heads=None, expected_tokens=None, check_finite=True):
        if not isinstance(tensor, torch.Tensor) or tensor.dim() != 3:
            raise ValueError(f"{name} must be [N,H,D]")
        if tensor.device != self.device or tensor.dtype != self.dtype:
            raise ValueError(f"{name} must match cache device and dtype")
        if tensor.requires_grad:
            raise ValueError("KV cache/decode is inference-only; detach Q/K/V")
        n, h, d = tensor.shape
        if n < 1 or h < 1 or d != self.head_dim:
            raise ValueError(f"{name} has an invalid shape")
        if tensor.stride(-1) != 1:
            raise ValueError(f"{name} last dimension must be contiguous")
        if expected_heads is not None and h != expected_heads:
            raise ValueError(f"{name} KV head count differs from cache")
        if expected_tokens is not None and n != expected_tokens:
            raise ValueError(f"{name} token count differs")
        if check_finite and not bool(torch.isfinite(tensor).all()):   # reads a flag back: waits for the stream
            raise ValueError(f"{name} contains NaN/Inf")

    def _reject_storage_alias(self, *tensors):
        pools = {self.k_cache.untyped_storage().data_ptr(), self.v_cache.untyped_storage().data_ptr()}
        for t in tensors:
            if t.untyped_storage().data_ptr() in pools:
                raise ValueError("append inputs must not alias KV cache storage; clone first")

    def _gpu(self, data):
        return torch.tensor(data, dtype=torch.int32, device=self.device)

    def _upload(self, *vectors):
        """One host->device copy for several small int vectors; returns views into it."""
        sizes = [len(v) for v in vectors]
        flat = [x for v in vectors for x in v]
        return self._gpu(flat).split(sizes) if flat else tuple(self._gpu([]) for _ in vectors)

    def _count_candidates(self, lengths):
        c = self.chunk_size
        return sum(max(0, -(-n // c) - 1) for n in lengths)

    def _append_counts(self, token_count, sequence_ids, cu_seqlens):
        ids = self._layout.validate_ids(_ints(sequence_ids, "sequence_ids"), unique=True)
        cu = tuple(range(len(ids) + 1)) if cu_seqlens is None else _ints(cu_seqlens, "cu_seqlens")
        if len(cu) != len(ids) + 1 or cu[0] != 0 or cu[-1] != token_count:
            raise ValueError("append cu_seqlens must start at 0 and end at N")
        counts = tuple(b - a for a, b in zip(cu, cu[1:]))
        if min(counts) <= 0:
            raise ValueError("append sequences must be nonempty")
        return ids, counts

    def _run(self, status, what):
        if status != 0:
            self._invalid = True
        _ext.check(status, what)

    # ------------------------------------------------------------------ public operations
    def prepare_decode(self, sequence_ids, num_q_heads, *, topk=4, mode="moba", check_finite=True, stable_routes=False):
        from .prepared_decode import PreparedDecode
        return PreparedDecode(self, sequence_ids, num_q_heads, topk=topk, mode=mode, check_finite=check_finite,
                              stable_routes=stable_routes)

    @torch.no_grad()
    def append(self, k, v, *, sequence_ids, cu_seqlens=None):
        with self._lock, torch.cuda.device(self.device):
            self._check_stream()
            self._tensor(k, "k", expected_heads=self.num_kv_heads)
            self._tensor(v, "v", expected_heads=self.num_kv_heads, expected_tokens=k.shape[0])
            self._reject_storage_alias(k, v)
            ids, counts = self._append_counts(k.shape[0], sequence_ids, cu_seqlens)
            return self._append_validated(k, v, ids, counts)[0]

    @torch.no_grad()
    def append_prefill(self, k, v, *, sequence_ids, cu_seqlens=None, check_finite=True):
        """`append` for whole prompts (the hand-off from a prefill pass): same contract and resulting cache state, but
        one launch writes the pages and the means of the completed chunks in a single pass over K, and the host builds
        no per-token index arrays.  `check_finite=False` leaves out the NaN/Inf check of k and v, which reads a flag
        back from the device and so makes the host wait for everything enqueued before (as `prepare_decode` offers
        for decode steps).  Returns the new lengths of the given sequences."""
        with self._lock, torch.cuda.device(self.device):
            self._check_stream()
            self._tensor(k, "k", expected_heads=self.num_kv_heads, check_finite=check_finite)
            self._tensor(v, "v", expected_heads=self.num_kv_heads, expected_tokens=k.shape[0], check_finite=check_finite)
            self._reject_storage_alias(k, v)
            ids, counts = self._append_counts(k.shape[0], sequence_ids, cu_seqlens)
            starts = [self._layout.lengths[s] for s in ids]
            plan = self._layout.plan_append(ids, counts, tokens=False)
            cu = [0]
            for n in counts:
                cu.append(cu[-1] + n)
            table = self._gpu(plan.tables)
            lengths, seqs, start, cu_dev = self._upload(plan.lengths, ids, starts, cu)
            self._table.copy_(table)
            self._lengths.copy_(lengths)
            c = self.chunk_size
            touched = max((first + n - 1) // c - first // c + 1 for first, n in zip(starts, counts))
            d, st = self._desc(), self._cuda_stream()
            k, v = k.contiguous(), v.contiguous()
            self._run(self._lib.moba_prefill_to_cache(ctypes.byref(d), k.data_ptr(), v.data_ptr(), seqs.data_ptr(), start.data_ptr(),
                                                      cu_dev.data_ptr(), len(ids), touched, self._status.data_ptr(), st),
                      "moba_prefill_to_cache")
            self._layout.commit(plan)
            self._candidate_count = self._count_candidates(plan.lengths)
            return tuple(plan.lengths[s] for s in ids)

    def _append_validated(self, k, v, ids, counts):
        """Caller holds the lock and has validated the inputs.  Metadata is staged first, the CPU layout
        is committed only after every launch was accepted."""
        plan = self._layout.plan_append(ids, counts)
        table = self._gpu(plan.tables)
        lengths, tok_seq, tok_pos, closed_seq, closed_chunk = self._upload(
            plan.lengths, plan.token_sequences, plan.token_positions,
            [s for s, _ in plan.completed_chunks], [c for _, c in plan.completed_chunks])
        self._table.copy_(table)
        self._lengths.copy_(lengths)
        d, st = self._desc(), self._cuda_stream()
        k, v = k.contiguous(), v.contiguous()
        self._run(self._lib.moba_decode_append(ctypes.byref(d), k.data_ptr(), v.data_ptr(), tok_seq.data_ptr(),
                                               tok_pos.data_ptr(), k.shape[0], self._status.data_ptr(), st), "moba_decode_append")
        if plan.completed_chunks:
            self._run(self._lib.moba_decode_means(ctypes.byref(d), closed_seq.data_ptr(), closed_chunk.data_ptr(),
                                                  len(plan.completed_chunks), 0, self._status.data_ptr(), st), "moba_decode_means")
        self._layout.commit(plan)
        self._candidate_count = self._count_candidates(plan.lengths)
        return AppendResult(plan.token_sequences, plan.token_positions), tok_seq, tok_pos

    def _query_metadata(self, q, sequence_ids, positions):
        self._tensor(q, "q")
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

    @torch.no_grad()
    def attend(self, q, *, sequence_ids, positions=None, topk=4, mode="moba"):
        with self._lock, torch.cuda.device(self.device):
            self._check_stream()
            dense = _mode(mode, topk)
            ids, pos = self._query_metadata(q, sequence_ids, positions)
            return self._attend_validated(q, ids, pos, topk, dense)

    def _attend_validated(self, q, ids, pos, topk, dense, gpu_metadata=None):
        q = q.contiguous()
        nq, hq, _ = q.shape
        gpu_ids, gpu_pos = self._upload(ids, pos) if gpu_metadata is None else gpu_metadata
        d, st, lib = self._desc(), self._cuda_stream(), self._lib
        out = torch.empty_like(q)
        lse = torch.empty((nq, hq), dtype=torch.float32, device=self.device)
        selected = None
        sel_ptr = uc_ptr = um_ptr = un_ptr = None
        umax, slots = 1, self._max_chunks
        if not dense:
            # result width as in the reference: min(topk-1, routable chunks in the whole cache)
            remote = min(int(topk) - 1, self._candidate_count)
            width = max(1, remote, max(pos) // self.chunk_size)
            if width * hq * nq >= 2 ** 31:
                raise ValueError("route score grid exceeds int32 capacity")
            umax = lib.moba_decode_union_capacity(hq, self.num_kv_heads, remote, width)
            selected = torch.empty((nq, hq, remote + 1), dtype=torch.int32, device=self.device)
            u_chunk = torch.empty((nq, self.num_kv_heads, umax), dtype=torch.int32, device=self.device)
            u_mask = torch.empty_like(u_chunk)
            u_count = torch.empty((nq, self.num_kv_heads), dtype=torch.int32, device=self.device)
            self._run(lib.moba_decode_route(ctypes.byref(d), q.data_ptr(), gpu_ids.data_ptr(), gpu_pos.data_ptr(), nq, hq,
                                            remote, width, None, selected.data_ptr(), u_chunk.data_ptr(), u_mask.data_ptr(),
                                            u_count.data_ptr(), st), "moba_decode_route")
            sel_ptr, uc_ptr, um_ptr, un_ptr = selected.data_ptr(), u_chunk.data_ptr(), u_mask.data_ptr(), u_count.data_ptr()
            slots = remote + 1
        nbytes = lib.moba_decode_attend_workspace_bytes(ctypes.byref(d), nq, hq, slots)
        workspace = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        workspace[: nq * self.num_kv_heads * 4].zero_()
        self._run(lib.moba_decode_attend(ctypes.byref(d), q.data_ptr(), gpu_ids.data_ptr(), gpu_pos.data_ptr(), nq, hq,
                                         sel_ptr, slots, uc_ptr, um_ptr, un_ptr, umax, workspace.data_ptr(), nbytes,
                                         out.data_ptr(), lse.data_ptr(), self._status.data_ptr(), st), "moba_decode_attend")
        return DecodeResult(out, lse, selected, ids, pos)

    @torch.no_grad()
    def append_and_attend(self, q, k, v, *, sequence_ids, cu_seqlens=None, topk=4, mode="moba"):
        with self._lock, torch.cuda.device(self.device):
            self._check_stream()
            dense = _mode(mode, topk)
            self._tensor(k, "k", expected_heads=self.num_kv_heads)
            self._tensor(v, "v", expected_heads=self.num_kv_heads, expected_tokens=k.shape[0])
            self._tensor(q, "q", expected_tokens=k.shape[0])
            self._reject_storage_alias(q, k, v)
            if q.shape[1] % self.num_kv_heads:
                raise ValueError("Hq must be a multiple of Hkv")
            if q.shape[0] * q.shape[1] >= 2 ** 31:
                raise ValueError("query grid exceeds int32 capacity")
            ids, counts = self._append_counts(k.shape[0], sequence_ids, cu_seqlens)
            info, gpu_ids, gpu_pos = self._append_validated(k, v, ids, counts)
            return self._attend_validated(q, info.sequence_ids, info.positions, topk, dense, gpu_metadata=(gpu_ids, gpu_pos))

    @torch.no_grad()
    def reset(self, sequence_ids=None):
        with self._lock, torch.cuda.device(self.device):
            self._check_stream()
            ids = tuple(range(self._layout.batch_size)) if sequence_ids is None else _ints(sequence_ids, "sequence_ids")
            # reset a copy first so that a failure while staging metadata publishes nothing
            staged = self._layout.clone()
            staged.reset(ids)
            table, lengths = self._gpu(staged.tables), self._gpu(staged.lengths)
            self._table.copy_(table)
            self._lengths.copy_(lengths)
            self._layout = staged
            self._candidate_count = self._count_candidates(staged.lengths)

    @torch.no_grad()
    def materialize(self, sequence_id):
        """Reads one sequence's K/V back in logical order (diagnostics and tests only)."""
        with self._lock, torch.cuda.device(self.device):
            self._check_stream(allow_prepared=True)
            sid = self._layout.validate_ids([sequence_id])[0]
            page = self._layout.page_size
            pos = torch.arange(self.lengths[sid], device=self.device)
            pages = self._table[sid, pos // page].long()
            return self.k_cache[pages, pos % page], self.v_cache[pages, pos % page]


class ContiguousKVCache(PagedKVCache):
    """One physical slab per sequence: a paged cache whose page is a whole sequence
    (kv_cache.py:294-300)."""

    def __init__(self, batch_size, max_seq_len, num_kv_heads, head_dim, **kwargs):
        if "page_size" in kwargs or "num_pages" in kwargs:
            raise ValueError("ContiguousKVCache owns page_size/num_pages")
        super().__init__(batch_size, max_seq_len, num_kv_heads, head_dim, page_size=max_seq_len, num_pages=batch_size,
                         **kwargs)
