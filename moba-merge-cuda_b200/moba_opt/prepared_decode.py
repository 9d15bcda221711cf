"""`PreparedDecode`: a fixed set of sequences decoded one token per step with persistent buffers,
optionally replayed as a CUDA graph.

Surface and error behaviour follow the reference (src/moba_opt/prepared_decode.py:15-204): an
exclusive lease on the cache, `.q/.k/.v/.output/.lse/.selected/.scores` buffers at fixed addresses,
`step`, `attend`, `capture("step"|"attend")`, `close`, `.delta_uploads`.  The host does the page
planning and, only when a sequence opens a new page, uploads a 2 x b int32 delta; everything else
of a step is five kernel launches (metadata, append, means, route, attention) whose launch shapes
were fixed at preparation, which is what makes the step capturable.

Outputs are views of the persistent buffers and are overwritten by the next call.
"""
import ctypes

import torch

from . import _ext
from .cache_layout import IncrementalLayout, positive_int
from .kv_cache import DecodeResult, _ints, _mode


class PreparedDecode:
    def __init__(self, cache, sequence_ids, num_q_heads, *, topk=4, mode="moba", check_finite=True, stable_routes=False):
        with cache._lock, torch.cuda.device(cache.device):
            cache._check_stream()
            self.num_q_heads = positive_int(num_q_heads, "num_q_heads")
            if self.num_q_heads % cache.num_kv_heads:
                raise ValueError("Hq must be a multiple of Hkv")
            if not isinstance(check_finite, bool):
                raise ValueError("check_finite must be bool")
            if not isinstance(stable_routes, bool):
                raise ValueError("stable_routes must be bool")
            self.stable_routes = stable_routes     # ties always go to the lowest chunk; the flag is accepted
            self.dense = _mode(mode, topk)
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
            self.check_finite = check_finite
            self.closed = False
            self.failed = False
            self._graphs = {}
            self.delta_uploads = 0
            dev, dt = cache.device, cache.dtype
            self.q = torch.zeros((b, h, d), dtype=dt, device=dev)
            self.k = torch.zeros((b, hk, d), dtype=dt, device=dev)
            self.v = torch.zeros_like(self.k)
            self.output = torch.empty_like(self.q)
            self.lse = torch.empty((b, h), dtype=torch.float32, device=dev)
            self.scores = torch.empty((b, h, self.width), dtype=torch.float32, device=dev)
            self.selected = torch.empty((b, h, self.remote + 1), dtype=torch.int32, device=dev)
            self.gpu_ids = torch.tensor(self.ids, dtype=torch.int32, device=dev)
            self.positions = torch.empty(b, dtype=torch.int32, device=dev)
            self.delta = torch.full((2, b), -1, dtype=torch.int32, device=dev)
            # pinned staging buffers for the page-table delta, used in turn so that an upload need not wait for the copy
            self._delta_ring = [torch.empty((2, b), dtype=torch.int32, pin_memory=True) for _ in range(4)]
            self._delta_done = [None] * len(self._delta_ring)
            self._delta_next = 0
            self._row_of = {sid: i for i, sid in enumerate(self.ids)}
            self._umax = lib.moba_decode_union_capacity(h, hk, self.remote, self.width)
            self._u_chunk = torch.empty((b, hk, self._umax), dtype=torch.int32, device=dev)
            self._u_mask = torch.empty_like(self._u_chunk)
            self._u_count = torch.empty((b, hk), dtype=torch.int32, device=dev)
            self._slots = cache._max_chunks if self.dense else self.remote + 1
            desc = cache._desc()
            self._ws_bytes = lib.moba_decode_attend_workspace_bytes(ctypes.byref(desc), b, h, self._slots)
            self._workspace = torch.zeros(self._ws_bytes, dtype=torch.uint8, device=dev)
            # the lease is published only after every allocation above succeeded
            cache._prepared_owner = self

    # ------------------------------------------------------------------ CPU views
    @property
    def lengths(self):
        with self.cache._lock:
            return tuple(self._state.lengths)

    @property
    def page_table(self):
        with self.cache._lock:
            return tuple(tuple(row) for row in self._state.tables)

    # ------------------------------------------------------------------ checks
    def _check(self):
        if self.closed or self.cache._prepared_owner is not self:
            raise ValueError("prepared decode is closed or no longer owns cache")
        if self.failed:
            raise RuntimeError("CUDA execution failed; discard prepared decode and cache")
        if torch.cuda.is_current_stream_capturing():
            raise ValueError("use capture(), not external capture")
        if torch.cuda.current_stream(self.cache.device).cuda_stream != self.cache._stream:
            raise ValueError("cross-stream cache access is unsupported")

    def _input(self, tensor, target, name):
        if not isinstance(tensor, torch.Tensor) or tensor.shape != target.shape:
            raise ValueError(f"{name} must have fixed shape {tuple(target.shape)}")
        if tensor.device != target.device or tensor.dtype != target.dtype or not tensor.is_contiguous():
            raise ValueError(f"{name} must match device/dtype and be contiguous")
        if tensor.requires_grad:
            raise ValueError("prepared decode is inference-only")
        self.cache._reject_storage_alias(tensor)
        own = {x.untyped_storage().data_ptr() for x in (self.q, self.k, self.v)}
        if tensor is not target and tensor.untyped_storage().data_ptr() in own:
            raise ValueError("input aliases another prepared workspace; clone first")
        if self.check_finite and not bool(torch.isfinite(tensor).all()):
            raise ValueError(f"{name} contains NaN/Inf")

    # ------------------------------------------------------------------ device work
    def _stage(self, pairs):
        """Caller's tensors into the fixed buffers: one launch for all of them when they are contiguous and 16-byte
        aligned, tensor copies otherwise."""
        todo = [(t, target) for t, target in pairs if t is not target]
        if not todo:
            return
        if all(t.is_contiguous() and t.dtype == target.dtype and t.data_ptr() % 16 == 0 and target.data_ptr() % 16 == 0
               and (t.numel() * t.element_size()) % 16 == 0 for t, target in todo):
            args = []
            for t, target in todo + [(None, None)] * (3 - len(todo)):
                args += [None, None, 0] if t is None else [target.data_ptr(), t.data_ptr(), t.numel() * t.element_size()]
            st = ctypes.c_void_p(torch.cuda.current_stream(self.cache.device).cuda_stream)
            if self._lib.moba_decode_stage_inputs(*args, st) == 0:
                return
        for t, target in todo:
            target.copy_(t)

    def _upload(self, plan):
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
            view[0, row] = logical
            view[1, row] = physical
        self.delta.copy_(host, non_blocking=True)
        done = torch.cuda.Event()
        done.record()
        self._delta_done[slot] = done
        self.delta_uploads += 1

    def _compute(self, append, projected=None):
        """Launches of one step.  `projected` = (qkv [b, (Hq + 2 Hkv) * D], cos, sin [b, D]): the fused q/k/v
        projection of the new tokens; rotary embedding and split into `q`, `k`, `v` then run inside the first launch."""
        c, lib = self.cache, self._lib
        d = c._desc()
        st = ctypes.c_void_p(torch.cuda.current_stream(c.device).cuda_stream)
        b, h = len(self.ids), self.num_q_heads
        status = c._status.data_ptr()
        ids, pos = self.gpu_ids.data_ptr(), self.positions.data_ptr()
        if append:
            qkv, cos, sin = (None, None, None) if projected is None else (t.data_ptr() for t in projected)
            _ext.check(lib.moba_decode_step_begin(ctypes.byref(d), ids, pos, self.delta.data_ptr(), b, h, qkv, cos, sin,
                                                  self.q.data_ptr(), self.k.data_ptr(), self.v.data_ptr(), status, st),
                       "moba_decode_step_begin")
        else:
            _ext.check(lib.moba_decode_metadata(ctypes.byref(d), ids, pos, self.delta.data_ptr(), b, 0, st),
                       "moba_decode_metadata")
        sel = None
        if not self.dense:
            _ext.check(lib.moba_decode_route(ctypes.byref(d), self.q.data_ptr(), ids, pos, b, h, self.remote, self.width,
                                             self.scores.data_ptr(), self.selected.data_ptr(), self._u_chunk.data_ptr(),
                                             self._u_mask.data_ptr(), self._u_count.data_ptr(), st), "moba_decode_route")
            sel = self.selected.data_ptr()
        _ext.check(lib.moba_decode_attend(ctypes.byref(d), self.q.data_ptr(), ids, pos, b, h, sel, self._slots,
                                          self._u_chunk.data_ptr(), self._u_mask.data_ptr(), self._u_count.data_ptr(),
                                          self._umax, self._workspace.data_ptr(), self._ws_bytes, self.output.data_ptr(),
                                          self.lse.data_ptr(), status, st), "moba_decode_attend")

    def _run(self, kind, use_graph):
        try:
            if use_graph:
                self._graphs[kind].replay()
            else:
                self._compute(kind == "step")
        except Exception:
            self.failed = True
            raise

    def _result(self, positions):
        return DecodeResult(self.output, self.lse, None if self.dense else self.selected, self.ids, positions)

    # ------------------------------------------------------------------ public operations
    @torch.no_grad()
    def attend(self, q, *, use_graph=False):
        with self.cache._lock, torch.cuda.device(self.cache.device):
            self._check()
            self._input(q, self.q, "q")
            pos = tuple(self._state.lengths[s] - 1 for s in self.ids)
            if min(pos) < 0:
                raise ValueError("query positions must refer to cached tokens")
            if use_graph and "attend" not in self._graphs:
                raise ValueError("capture('attend') first")
            if q is not self.q:
                self.q.copy_(q)
            self._run("attend", use_graph)
            return self._result(pos)

    @torch.no_grad()
    def step(self, q, k, v, *, use_graph=False):
        """Appends one token per leased sequence and attends with it.  Validation and capacity errors
        are raised before anything is modified."""
        with self.cache._lock, torch.cuda.device(self.cache.device):
            self._check()
            for tensor, target, name in ((q, self.q, "q"), (k, self.k, "k"), (v, self.v, "v")):
                self._input(tensor, target, name)
            if use_graph and "step" not in self._graphs:
                raise ValueError("capture('step') first")
            plan = self._state.plan()
            self._stage(((q, self.q), (k, self.k), (v, self.v)))
            self._upload(plan)
            self._run("step", use_graph)
            self._state.commit(plan)
            return self._result(plan.positions)

    @torch.no_grad()
    def capture(self, kind="step"):
        """Captures the device work of one step (or one attend) into a CUDA graph.  The visible cache
        state (page table, lengths, means, delta) is restored afterwards."""
        if kind not in ("step", "attend"):
            raise ValueError("kind must be step or attend")
        c = self.cache
        with c._lock, torch.cuda.device(c.device):
            self._check()
            if kind in self._graphs:
                raise ValueError("graph already captured")
            plan = self._state.plan() if kind == "step" else None
            if kind == "attend" and any(self._state.lengths[s] == 0 for s in self.ids):
                raise ValueError("attend capture requires nonempty cached sequences")
            targets = (c._table, c._lengths, c._means, self.delta)
            saved = [t.clone() for t in targets]
            uploads = self.delta_uploads
            main = torch.cuda.current_stream(c.device)
            side = torch.cuda.Stream(device=c.device)
            side.wait_stream(main)
            try:
                if plan is not None:
                    self._upload(plan)
                side.wait_stream(main)
                with torch.cuda.stream(side):
                    for _ in range(2):          # warm-up outside the capture
                        self._compute(kind == "step")
                        c._lengths.copy_(saved[1])
                main.wait_stream(side)
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    self._compute(kind == "step")
                self._graphs[kind] = graph
            finally:
                main.wait_stream(side)
                for target, snapshot in zip(targets, saved):
                    target.copy_(snapshot)
                self.delta_uploads = uploads
            return self

    def close(self):
        if self.closed:
            return
        c = self.cache
        with c._lock, torch.cuda.device(c.device):
            if c._prepared_owner is not self:
                raise ValueError("prepared ownership lost")
            if torch.cuda.current_stream(c.device).cuda_stream != c._stream:
                raise ValueError("cross-stream cache access is unsupported")
            if self.failed:
                c._invalid = True
            else:
                self._state.publish(c._layout)
                c._candidate_count = c._count_candidates(self._state.lengths)
            c._prepared_owner = None
            self._graphs.clear()
            self.closed = True

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
