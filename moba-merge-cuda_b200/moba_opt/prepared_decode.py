"""`PreparedDecode`: a fixed set of sequences decoded one token per step from persistent buffers,
optionally replayed as a CUDA graph.

The surface and the error behaviour are the reference's (src/moba_opt/prepared_decode.py:15-204): an
exclusive lease on the cache, `.q/.k/.v/.output/.lse/.selected/.scores` at fixed addresses, `step`,
`attend`, `capture("step"|"attend")`, `close`, `.delta_uploads`.  Outputs are views of the
persistent buffers and are overwritten by the next call.

How a step runs here: the host plans the pages (a few integer operations) and, only when some
sequence opens a new page, sends a 2 x b int32 delta from a ring of pinned buffers; the device work is
three launches whose shapes were fixed at preparation - `moba_decode_step_begin` (metadata, append and
predicated chunk mean in one kernel), `moba_decode_route`, `moba_decode_attend` - two for dense plans.
Fixed shapes, fixed addresses and positions read from device memory are what make the step capturable.

Besides the reference's methods there is a small driver interface for callers that run several plans
inside one graph of their own (a model session with one plan per layer): `plan_step`, `send_delta`,
`launch`, `replay`, `commit_step`, `mark_failed`, and `VisibleState` to put the cache back after a
capture.
"""
import ctypes
import enum

import torch

from . import _ext
from .cache_layout import IncrementalLayout, positive_int
from .kv_cache import CacheLife, DecodeResult, _ints, wants_dense


def current_stream_handle(device_index):
    """The current CUDA stream of the device as an integer handle (the cheapest route torch offers; a step asks twice)."""
    raw = getattr(torch._C, "_cuda_getCurrentRawStream", None)
    return raw(device_index) if raw is not None else torch.cuda.current_stream(device_index).cuda_stream


def _storage_address(t):
    return t.untyped_storage().data_ptr()


class PlanLife(enum.Enum):
    OPEN = "open"
    FAILED = "failed"      # a launch or replay raised: buffers and cache contents are undefined
    CLOSED = "closed"


class VisibleState:
    """The cache state a capture must not change: page table, lengths, chunk means, the plan's pending delta and its
    upload counter.  Taken on entry, put back on exit (also when the body raises)."""

    def __init__(self, plan):
        self.plan = plan

    def __enter__(self):
        p, c = self.plan, self.plan.cache
        self._targets = (c._table, c._lengths, c._means, p.delta)
        self._saved = [t.clone() for t in self._targets]
        self._uploads = p.delta_uploads
        return self

    @property
    def lengths(self):
        return self._saved[1]

    def __exit__(self, *exc):
        for target, snapshot in zip(self._targets, self._saved):
            target.copy_(snapshot)
        self.plan.delta_uploads = self._uploads
        return False


class PreparedDecode:
    def __init__(self, cache, sequence_ids, num_q_heads, *, topk=4, mode="moba", check_finite=True, stable_routes=False):
        with cache._lock, torch.cuda.device(cache.device):
            cache._guard()
            self.num_q_heads = positive_int(num_q_heads, "num_q_heads")
            if self.num_q_heads % cache.num_kv_heads:
                raise ValueError("Hq must be a multiple of Hkv")
            for flag, name in ((check_finite, "check_finite"), (stable_routes, "stable_routes")):
                if not isinstance(flag, bool):
                    raise ValueError(f"{name} must be bool")
            self.stable_routes = stable_routes     # exact ties always go to the lowest chunk; the flag is accepted
            self.check_finite = check_finite
            self.dense = wants_dense(mode, topk)
            self.cache = cache
            self._state = IncrementalLayout(cache._layout, _ints(sequence_ids, "sequence_ids"))
            self.ids = self._state.ids
            lib = self._lib = cache._lib
            b, h, d, hk = len(self.ids), self.num_q_heads, cache.head_dim, cache.num_kv_heads
            history = (cache._layout.max_seq_len - 1) // cache.chunk_size
            self.width = max(1, history)
            if b * h * self.width >= 2 ** 31:
                raise ValueError("route score grid exceeds int32 capacity")
            self.remote = 0 if self.dense else min(topk - 1, history)
            self._life = PlanLife.OPEN
            self._graphs = {}
            self.delta_uploads = 0
            dev, dt = cache.device, cache.dtype
            new = lambda shape, dtype=dt, fill=None: (torch.empty(shape, dtype=dtype, device=dev) if fill is None
                                                      else torch.full(shape, fill, dtype=dtype, device=dev))
            self.q, self.k, self.v = new((b, h, d), fill=0), new((b, hk, d), fill=0), new((b, hk, d), fill=0)
            self.output = new((b, h, d))
            self.lse = new((b, h), torch.float32)
            self.scores = new((b, h, self.width), torch.float32)
            self.selected = new((b, h, self.remote + 1), torch.int32)
            self.gpu_ids = torch.tensor(self.ids, dtype=torch.int32, device=dev)
            self.positions = new((b,), torch.int32, fill=-1)     # read as a hint by the step's first launch: start defined
            self.delta = new((2, b), torch.int32, fill=-1)
            # pinned staging buffers for the page-table delta, used in turn so that an upload need not wait for the copy
            self._delta_ring = [torch.empty((2, b), dtype=torch.int32, pin_memory=True) for _ in range(4)]
            self._delta_done = [None] * len(self._delta_ring)
            self._delta_next = 0
            self._row_of = {sid: i for i, sid in enumerate(self.ids)}
            # what a caller's q / k / v must not share storage with; the pools and the buffers live as long as the plan
            self._device_index = dev.index
            self._pool_storage = frozenset(_storage_address(t) for t in (cache.k_cache, cache.v_cache))
            self._input_storage = frozenset(_storage_address(t) for t in (self.q, self.k, self.v))
            self._step_pairs = ((self.q, "q"), (self.k, "k"), (self.v, "v"))
            self._umax = lib.moba_decode_union_capacity(h, hk, self.remote, self.width)
            self._u_chunk = new((b, hk, self._umax), torch.int32)
            self._u_mask = new((b, hk, self._umax), torch.int32)
            self._u_count = new((b, hk), torch.int32)
            self._slots = cache._max_chunks if self.dense else self.remote + 1
            desc = cache._desc()
            self._ws_bytes = lib.moba_decode_attend_workspace_bytes(ctypes.byref(desc), b, h, self._slots)
            self._workspace = torch.zeros(self._ws_bytes, dtype=torch.uint8, device=dev)
            # the lease is published only after every allocation above succeeded
            cache._owner, cache._life = self, CacheLife.LEASED

    # ------------------------------------------------------------------ state seen from outside
    @property
    def closed(self):
        return self._life is PlanLife.CLOSED

    @property
    def failed(self):
        return self._life is PlanLife.FAILED

    @property
    def lengths(self):
        with self.cache._lock:
            return tuple(self._state.lengths)

    @property
    def page_table(self):
        with self.cache._lock:
            return tuple(tuple(row) for row in self._state.tables)

    def _usable(self):
        if self._life is PlanLife.CLOSED or self.cache._owner is not self:
            raise ValueError("prepared decode is closed or no longer owns cache")
        if self._life is PlanLife.FAILED:
            raise RuntimeError("CUDA execution failed; discard prepared decode and cache")
        if torch.cuda.is_current_stream_capturing():
            raise ValueError("use capture(), not external capture")
        if current_stream_handle(self._device_index) != self.cache._stream:
            raise ValueError("cross-stream cache access is unsupported")

    def _accept(self, tensor, target, name):
        """The caller's tensor for the fixed buffer `target`: same shape, device, dtype, contiguous, no gradient, no
        overlap with the cache pools or with another of the plan's input buffers, finite unless the plan skips that.
        The buffer itself passes all but the last by construction."""
        if tensor is not target:
            if not isinstance(tensor, torch.Tensor) or tensor.shape != target.shape:
                raise ValueError(f"{name} must have fixed shape {tuple(target.shape)}")
            if tensor.device != target.device or tensor.dtype != target.dtype or not tensor.is_contiguous():
                raise ValueError(f"{name} must match device/dtype and be contiguous")
            if tensor.requires_grad:
                raise ValueError("prepared decode is inference-only")
            where = _storage_address(tensor)
            if where in self._pool_storage:
                raise ValueError("append inputs must not alias KV cache storage; clone first")
            if where in self._input_storage:
                raise ValueError("input aliases another prepared workspace; clone first")
        if self.check_finite and not bool(torch.isfinite(tensor).all()):
            raise ValueError(f"{name} contains NaN/Inf")

    # ------------------------------------------------------------------ driver interface
    def _stream(self):
        return ctypes.c_void_p(current_stream_handle(self._device_index))

    def plan_step(self):
        """Positions and page openings of the next one-token step; raises (cache full, pool empty) without side effects."""
        return self._state.plan()

    def commit_step(self, plan):
        self._state.commit(plan)

    def mark_failed(self):
        self._life = PlanLife.FAILED

    def stage_inputs(self, pairs):
        """Caller's tensors into the fixed buffers: one launch for all of them when they are contiguous and 16-byte
        aligned, tensor copies otherwise."""
        todo = [(t, target) for t, target in pairs if t is not target]
        if not todo:
            return
        args = []
        for t, target in todo:
            src, dst, size = t.data_ptr(), target.data_ptr(), t.numel() * t.element_size()
            if (src | dst | size) & 15 or t.dtype != target.dtype or not t.is_contiguous():
                break
            args += (dst, src, size)
        else:
            args += (None, None, 0) * (3 - len(todo))
            if self._lib.moba_decode_stage_inputs(*args, self._stream()) == 0:
                return
        for t, target in todo:
            target.copy_(t)

    def send_delta(self, plan):
        """Only when some sequence opens a page: an asynchronous 2 x b int32 copy from one of a few pinned staging
        buffers; the host waits only if the copy that last used the buffer (four uploads ago) is still pending, so a
        step that opens a page does not drain the stream."""
        if not plan.updates:
            return
        slot = self._delta_next
        self._delta_next = (slot + 1) % len(self._delta_ring)
        if self._delta_done[slot] is not None:
            self._delta_done[slot].synchronize()
        host = self._delta_ring[slot]
        view = host.numpy()
        view.fill(-1)
        for sid, logical, physical in plan.updates:
            row = self._row_of[sid]
            view[0, row], view[1, row] = logical, physical
        self.delta.copy_(host, non_blocking=True)
        done = torch.cuda.Event()
        done.record()
        self._delta_done[slot] = done
        self.delta_uploads += 1

    def launch(self, kind, projected=None):
        """The device work of one step ("step": append + route + attend) or one attend ("attend": route + attend of
        the newest cached token), on the current stream.  `projected` = (qkv [b, (Hq + 2 Hkv) * D], cos, sin [b, D]):
        the fused q/k/v projection of the new tokens; rotary embedding and split into `q`, `k`, `v` then run inside
        the step's first launch."""
        c, lib, st = self.cache, self._lib, self._stream()
        d = c._desc()
        b, h = len(self.ids), self.num_q_heads
        status = c._status.data_ptr()
        ids, pos = self.gpu_ids.data_ptr(), self.positions.data_ptr()
        union = (self._u_chunk.data_ptr(), self._u_mask.data_ptr(), self._u_count.data_ptr())
        if kind == "step":
            qkv, cos, sin = (None, None, None) if projected is None else (t.data_ptr() for t in projected)
            buffers = (self.q.data_ptr(), self.k.data_ptr(), self.v.data_ptr())
            _ext.check(lib.moba_decode_step_begin(ctypes.byref(d), ids, pos, self.delta.data_ptr(), b, h, qkv, cos, sin,
                                                  *buffers, status, st), "moba_decode_step_begin")
        else:
            _ext.check(lib.moba_decode_metadata(ctypes.byref(d), ids, pos, self.delta.data_ptr(), b, 0, st), "moba_decode_metadata")
        if not self.dense:
            _ext.check(lib.moba_decode_route(ctypes.byref(d), self.q.data_ptr(), ids, pos, b, h, self.remote, self.width,
                                             self.scores.data_ptr(), self.selected.data_ptr(), *union, st), "moba_decode_route")
        _ext.check(lib.moba_decode_attend(ctypes.byref(d), self.q.data_ptr(), ids, pos, b, h,
                                          None if self.dense else self.selected.data_ptr(), self._slots, *union, self._umax,
                                          self._workspace.data_ptr(), self._ws_bytes, self.output.data_ptr(),
                                          self.lse.data_ptr(), status, st), "moba_decode_attend")

    def replay(self, kind):
        self._graphs[kind].replay()

    def _execute(self, kind, use_graph):
        try:
            with _ext.nvtx("moba.decode." + kind):
                self.replay(kind) if use_graph else self.launch(kind)
        except Exception:
            self.mark_failed()
            raise

    def _result(self, positions):
        return DecodeResult(self.output, self.lse, None if self.dense else self.selected, self.ids, positions)

    # ------------------------------------------------------------------ the reference's operations
    @torch.no_grad()
    def attend(self, q, *, use_graph=False):
        with self.cache._lock, torch.cuda.device(self._device_index):
            self._usable()
            self._accept(q, self.q, "q")
            pos = tuple(self._state.lengths[s] - 1 for s in self.ids)
            if min(pos) < 0:
                raise ValueError("query positions must refer to cached tokens")
            if use_graph and "attend" not in self._graphs:
                raise ValueError("capture('attend') first")
            self.stage_inputs(((q, self.q),))
            self._execute("attend", use_graph)
            return self._result(pos)

    @torch.no_grad()
    def step(self, q, k, v, *, use_graph=False):
        """Appends one token per leased sequence and attends with it.  Validation and capacity errors
        are raised before anything is modified."""
        with self.cache._lock, torch.cuda.device(self._device_index):
            self._usable()
            pairs = ((q, self.q), (k, self.k), (v, self.v))
            for (tensor, target), (_, name) in zip(pairs, self._step_pairs):
                self._accept(tensor, target, name)
            if use_graph and "step" not in self._graphs:
                raise ValueError("capture('step') first")
            plan = self._state.plan()
            self.stage_inputs(pairs)
            if plan.updates:
                self.send_delta(plan)
            self._execute("step", use_graph)
            self._state.commit(plan)
            return self._result(plan.positions)

    @torch.no_grad()
    def capture(self, kind="step"):
        """Records the device work of one step (or one attend) as a CUDA graph.  The work runs for real while it is
        recorded - twice before, as a warm-up, and once under capture - so the visible cache state (page table, lengths,
        means, pending delta) is saved first and put back afterwards."""
        if kind not in ("step", "attend"):
            raise ValueError("kind must be step or attend")
        c = self.cache
        with c._lock, torch.cuda.device(c.device):
            self._usable()
            if kind in self._graphs:
                raise ValueError("graph already captured")
            plan = self.plan_step() if kind == "step" else None
            if kind == "attend" and any(self._state.lengths[s] == 0 for s in self.ids):
                raise ValueError("attend capture requires nonempty cached sequences")
            main = torch.cuda.current_stream(c.device)
            side = torch.cuda.Stream(device=c.device)
            with VisibleState(self) as visible:
                try:
                    if plan is not None:
                        self.send_delta(plan)
                    side.wait_stream(main)
                    with torch.cuda.stream(side):
                        for _ in range(2):
                            self.launch(kind)
                            c._lengths.copy_(visible.lengths)
                    main.wait_stream(side)
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph, stream=side):
                        self.launch(kind)
                    self._graphs[kind] = graph
                finally:
                    main.wait_stream(side)
            return self

    def close(self):
        if self._life is PlanLife.CLOSED:
            return
        c = self.cache
        with c._lock, torch.cuda.device(c.device):
            if c._owner is not self:
                raise ValueError("prepared ownership lost")
            if torch.cuda.current_stream(c.device).cuda_stream != c._stream:
                raise ValueError("cross-stream cache access is unsupported")
            if self._life is PlanLife.FAILED:
                c._life = CacheLife.BROKEN
            else:
                self._state.publish(c._layout)
                c._candidate_count = c._routable(self._state.lengths)
                c._life = CacheLife.READY
            c._owner = None
            self._graphs.clear()
            self._life = PlanLife.CLOSED

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
