"""Batch-1 full-model inference session for a Qwen2-architecture model on top of moba_opt: prefill through
`opt_gqa_cuda`, one paged KV cache per layer, decode through `PreparedDecode`, and optionally the whole decode step
(embedding to logits and the greedy argmax) as one CUDA graph.

Counterpart of the reference's experimental session (examples/full_qwen2.py:19-214, qwen2_attention.py): same
constructor vocabulary (mode, chunk, topk, backend, page, dense_layers, prefill_mode, routing flags), same life cycle
(`prefill_hidden` -> `prepare` -> `step` ... -> `close`).  Differences: every attention, dense layers included, runs
on this package's kernels (dense prefill is the K=1 fallback of `opt_gqa_cuda`, dense decode is
`prepare_decode(mode="dense")`), so no FlashAttention is needed; and `greedy_step()` keeps the chosen token on the
device, so a greedy loop replays the graph without a host round trip.  The weights and the rotary tables stay in the
unchanged Hugging Face module and the projections are plain library GEMMs; in the decode step the elementwise glue of
a layer (residual add + RMSNorm, rotary embedding + q/k/v split, SiLU * up) runs as three single-launch kernels of this
package unless `fused_glue=False` asks for the Hugging Face modules.
"""
import torch
import torch.nn.functional as F

from moba_opt import PagedKVCache
from moba_opt.cache_layout import positive_int
from moba_opt.grouped_attention import opt_gqa_cuda


def _rotate_half(x):
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def _apply_rope(x, cos, sin):
    """x [tokens, heads, dim]; cos/sin [tokens, dim] (the Hugging Face 'rotate half' convention)."""
    return x * cos[:, None, :] + _rotate_half(x) * sin[:, None, :]


class FullQwen2Session:
    BACKENDS = ("eager", "attention_graph", "model_graph")

    def __init__(self, model, capacity, *, mode="dense", chunk=128, topk=4, backend="eager", page=16,
                 deterministic_merge=False, stable_routes=False, route_precision="upstream", dense_layers=(),
                 prefill_mode="match", fused_glue=True):
        if mode not in ("dense", "moba"):
            raise ValueError("mode")
        if backend not in self.BACKENDS:
            raise ValueError("backend")
        cfg = model.config
        if cfg.model_type != "qwen2":
            raise ValueError("Qwen2 architecture required")
        if getattr(cfg, "use_sliding_window", False):
            raise ValueError("sliding window unsupported")
        if model.training or any(p.requires_grad for p in model.parameters()):
            raise ValueError("eval model with gradients disabled required")
        self.capacity = positive_int(capacity, "capacity")
        self.chunk, self.topk = positive_int(chunk, "chunk"), positive_int(topk, "topk")
        if prefill_mode not in ("match", "dense"):
            raise ValueError("prefill_mode")
        if route_precision not in ("upstream", "fp32"):
            raise ValueError("route_precision")
        if not isinstance(deterministic_merge, bool) or not isinstance(stable_routes, bool):
            raise ValueError("stability flags must be bool")
        layers = model.model.layers
        dense_layers = tuple(dense_layers)
        if len(set(dense_layers)) != len(dense_layers) or any(
                isinstance(i, bool) or not isinstance(i, int) or not 0 <= i < len(layers) for i in dense_layers):
            raise ValueError("dense_layers must be unique valid layer indices")
        self.model, self.mode, self.backend, self.prefill_mode = model, mode, backend, prefill_mode
        every_chunk = mode == "moba" and (self.capacity + self.chunk - 1) // self.chunk <= self.topk
        self.effective_dense = mode == "dense" or self.topk == 1 or every_chunk
        self.layer_dense = tuple(self.effective_dense or i in dense_layers for i in range(len(layers)))
        self.route_config = dict(chunk_size=self.chunk, topk=self.topk, deterministic_merge=deterministic_merge,
                                 stable_routes=stable_routes, route_precision=route_precision)
        self.dense_config = dict(self.route_config, topk=1)
        self.device = next(model.parameters()).device
        if self.device.type != "cuda":
            raise ValueError("CUDA model required")
        self.dtype = next(model.parameters()).dtype
        self.stream = torch.cuda.current_stream(self.device).cuda_stream
        self.hq, self.hk = cfg.num_attention_heads, cfg.num_key_value_heads
        self.dim = getattr(cfg, "head_dim", None) or cfg.hidden_size // self.hq
        self.caches = [PagedKVCache(1, self.capacity, self.hk, self.dim, page_size=page, chunk_size=self.chunk,
                                    dtype=self.dtype, device=self.device) for _ in layers]
        self.plans, self.graph, self.closed, self.failed = [], None, False, False
        self.input = torch.zeros((1, 1), device=self.device, dtype=torch.long)   # token of the next step
        self.logits = None
        self.next_token = torch.zeros((1, 1), device=self.device, dtype=torch.long)
        # fused q/k/v projection per layer: one GEMM instead of three
        self.packed = []
        for layer in layers:
            a = layer.self_attn
            bias = None if a.q_proj.bias is None else torch.cat([a.q_proj.bias, a.k_proj.bias, a.v_proj.bias], 0)
            self.packed.append((torch.cat([a.q_proj.weight, a.k_proj.weight, a.v_proj.weight], 0), bias))
        # Decode step on this package's kernels (moba_decode_linear with the norms and SiLU * up inside, moba_rope_split)
        # instead of the Hugging Face modules' many small launches; needs bf16 and bias-free gate/up projections.
        if not isinstance(fused_glue, bool):
            raise ValueError("fused_glue must be bool")
        self.fused_glue = fused_glue and self.dtype == torch.bfloat16 and all(
            l.mlp.gate_proj.bias is None and l.mlp.up_proj.bias is None for l in layers) and (
            cfg.hidden_size % 8 == 0 and cfg.hidden_size <= 8192 and cfg.intermediate_size % 8 == 0
            and cfg.intermediate_size <= 16384 and (cfg.num_attention_heads * (
                getattr(cfg, "head_dim", None) or cfg.hidden_size // cfg.num_attention_heads)) % 8 == 0)
        if self.fused_glue:
            from moba_opt import _ext
            self._lib = _ext.lib()
            self.gate_up = [torch.cat([l.mlp.gate_proj.weight, l.mlp.up_proj.weight], 0) for l in layers]
            hidden, ffn = cfg.hidden_size, cfg.intermediate_size
            new = lambda n: torch.empty((1, n), dtype=self.dtype, device=self.device)
            self._h, self._y, self._act = [new(hidden), new(hidden)], new(hidden), new(ffn)
            self._qkv, self._att, self._down = new((self.hq + 2 * self.hk) * self.dim), new(hidden), new(hidden)
            self._argmax_ws = torch.zeros(self._lib.moba_argmax_workspace_bytes(), dtype=torch.uint8, device=self.device)
            # rotary table inside the step's first launch when the model uses the default rotary type
            rotary = model.model.rotary_emb
            self._inv_freq = None
            if getattr(rotary, "rope_type", "default") == "default" and rotary.inv_freq.numel() * 2 == self.dim:
                self._inv_freq = rotary.inv_freq.detach().float().contiguous()
                self._rope_scale = float(getattr(rotary, "attention_scaling", 1.0))
                self._h0, self._cos, self._sin = new(hidden), new(self.dim), new(self.dim)

    # ------------------------------------------------------------------ helpers
    def _check(self):
        if self.closed or self.failed:
            raise ValueError("closed/failed session")
        if torch.cuda.current_stream(self.device).cuda_stream != self.stream:
            raise ValueError("cross-stream session")

    def _project(self, index, hidden, cos, sin):
        """hidden [tokens, hidden] -> q [tokens, Hq, D], k, v [tokens, Hkv, D] with rotary position applied."""
        tokens = hidden.shape[0]
        qkv = F.linear(hidden, *self.packed[index])
        q, k, v = qkv.split((self.hq * self.dim, self.hk * self.dim, self.hk * self.dim), dim=-1)
        q = _apply_rope(q.view(tokens, self.hq, self.dim), cos, sin)
        k = _apply_rope(k.view(tokens, self.hk, self.dim), cos, sin)
        return q.contiguous(), k.contiguous(), v.reshape(tokens, self.hk, self.dim).contiguous()

    def _rope(self, hidden, positions):
        cos, sin = self.model.model.rotary_emb(hidden[None], positions[None])
        return cos[0].to(self.dtype), sin[0].to(self.dtype)

    # ------------------------------------------------------------------ prefill
    @torch.no_grad()
    def prefill_hidden(self, ids):
        """Runs the prompt through every layer, filling the caches; returns the final normed hidden states
        [1, tokens, hidden]."""
        self._check()
        if self.plans or any(c.lengths[0] for c in self.caches):
            raise ValueError("fresh session required")
        if ids.dim() != 2 or ids.shape[0] != 1 or not 0 < ids.shape[1] < self.capacity:
            raise ValueError("batch=1, nonempty prefix below capacity required")
        if ids.device != self.device or ids.dtype != torch.long:
            raise ValueError("CUDA int64 token IDs required")
        t = ids.shape[1]
        body = self.model.model
        h = body.embed_tokens(ids)[0]
        cos, sin = self._rope(h, torch.arange(t, device=self.device))
        cu = torch.tensor([0, t], device=self.device, dtype=torch.int32)
        if self.fused_glue:
            return self._prefill_hidden_fused(h, cos, sin, cu, t)
        for i, layer in enumerate(body.layers):
            q, k, v = self._project(i, layer.input_layernorm(h), cos, sin)
            self.caches[i].append_prefill(k, v, sequence_ids=[0], cu_seqlens=[0, t], check_finite=False)
            dense = self.layer_dense[i] or self.prefill_mode == "dense"
            out = opt_gqa_cuda(q, k, v, cu, t, self.dense_config if dense else self.route_config)
            h = h + layer.self_attn.o_proj(out.reshape(t, -1))
            h = h + layer.mlp(layer.post_attention_layernorm(h))
        return body.norm(h)[None]

    def _prefill_hidden_fused(self, h, cos, sin, cu, t):
        """The same layers with the elementwise work between the GEMMs as single launches over all rows (residual add +
        RMSNorm, rotary embedding + q/k/v split, SiLU * up) instead of the modules' chains of small kernels."""
        import ctypes
        lib, body, cfg = self._lib, self.model.model, self.model.config
        st = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        hidden, ffn = cfg.hidden_size, cfg.intermediate_size

        def check(rc):
            if rc:
                raise RuntimeError("glue kernel launch failed (status %d)" % rc)

        def add_norm(h_in, delta, norm, h_out, y):
            check(lib.moba_add_rmsnorm(h_in.data_ptr(), None if delta is None else delta.data_ptr(), norm.weight.data_ptr(),
                                       float(norm.variance_epsilon), t, hidden, None if h_out is None else h_out.data_ptr(),
                                       y.data_ptr(), st))

        new = lambda *shape: torch.empty(shape, dtype=self.dtype, device=self.device)
        h = h.contiguous()
        cos, sin = cos.contiguous(), sin.contiguous()
        y, res, act = new(t, hidden), [new(t, hidden), new(t, hidden)], new(t, ffn)
        q, k, v = new(t, self.hq, self.dim), new(t, self.hk, self.dim), new(t, self.hk, self.dim)
        delta, flip = None, 0
        for i, layer in enumerate(body.layers):
            if delta is None:
                add_norm(h, None, layer.input_layernorm, None, y)
            else:
                add_norm(h, delta, layer.input_layernorm, res[flip], y)
                h, flip = res[flip], flip ^ 1
            qkv = F.linear(y, *self.packed[i])
            check(lib.moba_rope_split(qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(), t, self.hq, self.hk, self.dim,
                                      q.data_ptr(), k.data_ptr(), v.data_ptr(), st))
            self.caches[i].append_prefill(k, v, sequence_ids=[0], cu_seqlens=[0, t], check_finite=False)
            dense = self.layer_dense[i] or self.prefill_mode == "dense"
            out = opt_gqa_cuda(q, k, v, cu, t, self.dense_config if dense else self.route_config)
            att = layer.self_attn.o_proj(out.reshape(t, -1))
            add_norm(h, att, layer.post_attention_layernorm, res[flip], y)
            h, flip = res[flip], flip ^ 1
            gu = F.linear(y, self.gate_up[i])
            check(lib.moba_silu_mul(gu.data_ptr(), t, ffn, act.data_ptr(), st))
            delta = layer.mlp.down_proj(act)
        add_norm(h, delta, body.norm, None, y)
        return y[None]

    @torch.no_grad()
    def prefill(self, ids):
        """Prefill and return the logits of the last prompt position [1, vocab]; the greedy token is kept on the
        device as the input of the next step."""
        hidden = self.prefill_hidden(ids)
        self.logits = self.model.lm_head(hidden[:, -1])
        self.next_token.copy_(self.logits.argmax(-1, keepdim=True))
        self.input.copy_(self.next_token)
        return self.logits

    # ------------------------------------------------------------------ decode
    @torch.no_grad()
    def prepare(self):
        self._check()
        if self.plans:
            raise ValueError("already prepared")
        if not self.caches[0].lengths[0]:
            raise ValueError("prefill first")
        self.plans = [c.prepare_decode([0], self.hq, mode="dense" if dense else self.mode, topk=self.topk,
                                       check_finite=False, stable_routes=self.route_config["stable_routes"])
                      for c, dense in zip(self.caches, self.layer_dense)]
        if self.backend == "attention_graph":
            for p in self.plans:
                p.capture("step")
        elif self.backend == "model_graph":
            self._capture_model()

    def _compute_step(self):
        """Device work of one decode step, embedding to logits and greedy token; no host synchronisation."""
        if self.fused_glue:
            return self._compute_step_fused()
        body = self.model.model
        h = body.embed_tokens(self.input)[0]                                   # [1, hidden]
        position = self.caches[0]._lengths[:1].to(torch.long)                  # the new token's position
        cos, sin = self._rope(h, position)
        for i, (layer, p) in enumerate(zip(body.layers, self.plans)):
            q, k, v = self._project(i, layer.input_layernorm(h), cos, sin)
            p.q.copy_(q)
            p.k.copy_(k)
            p.v.copy_(v)
            self._attend(p)
            h = h + layer.self_attn.o_proj(p.output.reshape(1, -1))
            h = h + layer.mlp(layer.post_attention_layernorm(h))
        self.logits = self.model.lm_head(body.norm(h))
        self.next_token.copy_(self.logits.argmax(-1, keepdim=True))
        return self.logits

    def _attend(self, p):
        if self.backend == "attention_graph":
            p.replay("step")
        else:
            p.launch("step")

    def _compute_step_fused(self):
        """The same step in six launches per dense layer and seven per MoBA layer: every projection is one
        `moba_decode_linear` (the weight read once, all loads in flight), with the residual add + RMSNorm in front of
        the q/k/v and the gate/up projections and SiLU * up behind the latter inside the same launch; rotary embedding
        and split of q/k/v run inside the first launch of the attention step (metadata + append + chunk mean), then
        routing (MoBA layers) and the attention kernel."""
        import ctypes
        lib, body, cfg = self._lib, self.model.model, self.model.config
        st = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        hidden, ffn = cfg.hidden_size, cfg.intermediate_size

        def check(rc):
            if rc:
                raise RuntimeError("decode step kernel launch failed (status %d)" % rc)

        def ptr(t):
            return None if t is None else t.data_ptr()

        def linear(x, weight, bias, out, *, norm=None, h_in=None, delta=None, h_out=None, epilogue=0):
            n = out.shape[-1]
            check(lib.moba_decode_linear(ptr(x), ptr(h_in), ptr(delta), None if norm is None else norm.weight.data_ptr(),
                                         0.0 if norm is None else float(norm.variance_epsilon), ptr(h_out), weight.data_ptr(),
                                         ptr(bias), weight.shape[1], n, epilogue, out.data_ptr(), st))

        if self._inv_freq is not None:              # embedding row + rotary table of the new position: one launch
            h, cos, sin = self._h0, self._cos, self._sin
            check(lib.moba_decode_step_inputs(self.input.data_ptr(), body.embed_tokens.weight.data_ptr(), hidden,
                                              self.caches[0]._lengths.data_ptr(), self._inv_freq.data_ptr(), self._rope_scale,
                                              self.dim, 1, h.data_ptr(), cos.data_ptr(), sin.data_ptr(), st))
        else:
            h = body.embed_tokens(self.input)[0]
            position = self.caches[0]._lengths[:1].to(torch.long)
            cos, sin = self._rope(h, position)
            cos, sin = cos.contiguous(), sin.contiguous()
        delta, flip = None, 0
        for i, (layer, p) in enumerate(zip(body.layers, self.plans)):
            weight, bias = self.packed[i]
            if delta is None:                       # first layer: the embedding is the residual
                linear(None, weight, bias, self._qkv, norm=layer.input_layernorm, h_in=h)
            else:                                   # h <- h + (MLP output of the previous layer), normalise, project
                linear(None, weight, bias, self._qkv, norm=layer.input_layernorm, h_in=h, delta=delta, h_out=self._h[flip])
                h, flip = self._h[flip], flip ^ 1
            if self.backend == "attention_graph":   # the plan's own graph starts from its q, k, v buffers
                check(lib.moba_rope_split(self._qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(), 1, self.hq, self.hk, self.dim,
                                          p.q.data_ptr(), p.k.data_ptr(), p.v.data_ptr(), st))
                p.replay("step")
            else:                                   # rotary embedding + split inside the step's first launch
                p.launch("step", projected=(self._qkv, cos, sin))
            o = layer.self_attn.o_proj
            linear(p.output, o.weight, o.bias, self._att)
            linear(None, self.gate_up[i], None, self._act, norm=layer.post_attention_layernorm, h_in=h, delta=self._att,
                   h_out=self._h[flip], epilogue=1)
            h, flip = self._h[flip], flip ^ 1
            down = layer.mlp.down_proj
            linear(self._act, down.weight, down.bias, self._down)
            delta = self._down
        check(lib.moba_add_rmsnorm(h.data_ptr(), delta.data_ptr(), body.norm.weight.data_ptr(), float(body.norm.variance_epsilon),
                                   1, hidden, None, self._y.data_ptr(), st))
        self.logits = self.model.lm_head(self._y)
        if self.logits.dtype == torch.bfloat16 and self.logits.is_contiguous():
            check(lib.moba_argmax_bf16(self.logits.data_ptr(), self.logits.shape[-1], self._argmax_ws.data_ptr(),
                                       self._argmax_ws.numel(), self.next_token.data_ptr(), st))
        else:
            self.next_token.copy_(self.logits.argmax(-1, keepdim=True))
        return self.logits

    @torch.no_grad()
    def _capture_model(self):
        """Captures `_compute_step` as one CUDA graph.  The visible state of every cache (page table, lengths,
        means, pending page-table delta) is restored afterwards."""
        from contextlib import ExitStack
        from moba_opt.prepared_decode import VisibleState
        main = torch.cuda.current_stream(self.device)
        side = torch.cuda.Stream(device=self.device)
        with ExitStack() as stack:
            saved = [stack.enter_context(VisibleState(p)) for p in self.plans]
            try:
                for p in self.plans:
                    p.send_delta(p.plan_step())
                side.wait_stream(main)
                with torch.cuda.stream(side):
                    for _ in range(2):                      # warm-up outside the capture
                        self._compute_step()
                        for c, state in zip(self.caches, saved):
                            c._lengths.copy_(state.lengths)
                main.wait_stream(side)
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    self._compute_step()
                self.graph = graph
            finally:
                main.wait_stream(side)

    def _advance(self):
        if not self.plans:
            raise ValueError("prepare first")
        plans = [p.plan_step() for p in self.plans]     # raises before anything is modified when a cache is full
        for p, plan in zip(self.plans, plans):
            p.send_delta(plan)
        try:
            if self.graph is not None:
                self.graph.replay()
            else:
                self._compute_step()
        except Exception:
            self.failed = True
            for p in self.plans:
                p.mark_failed()
            raise
        for p, plan in zip(self.plans, plans):
            p.commit_step(plan)
        return self.logits

    @torch.no_grad()
    def step(self, token):
        """Teacher-forced step: feeds `token` (a CPU int), returns the logits [1, vocab] of the next position."""
        self._check()
        if isinstance(token, bool) or not isinstance(token, int) or not 0 <= token < self.model.config.vocab_size:
            raise ValueError("one valid CPU token ID required")
        self.input.fill_(token)
        return self._advance()

    @torch.no_grad()
    def greedy_step(self):
        """Feeds the previous step's (or the prefill's) greedy token, which never leaves the device."""
        self._check()
        self.input.copy_(self.next_token)
        return self._advance()

    @torch.no_grad()
    def generate(self, steps):
        """`steps` greedy steps; returns the chosen token ids [steps] (one device-to-host copy at the end)."""
        out = torch.empty(steps, dtype=torch.long, device=self.device)
        for i in range(steps):
            out[i] = self.next_token[0, 0]
            self.greedy_step()
        return out.cpu()

    def close(self):
        if self.closed:
            return
        for p in self.plans:
            p.close()
        self.graph = None
        self.closed = True

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def random_qwen2(*, hidden=896, layers=24, heads=14, kv_heads=2, ffn=4864, vocab=151936, rope_theta=1e6, max_positions=32768,
                 seed=0, device="cuda", dtype=torch.bfloat16):
    """A randomly initialised (N(0, 0.02)) Qwen2-architecture model; the defaults are the 0.5B shape."""
    from transformers import Qwen2Config, Qwen2ForCausalLM
    cfg = Qwen2Config(hidden_size=hidden, num_hidden_layers=layers, num_attention_heads=heads, num_key_value_heads=kv_heads,
                      intermediate_size=ffn, vocab_size=vocab, rope_theta=rope_theta, max_position_embeddings=max_positions,
                      tie_word_embeddings=True, use_sliding_window=False, initializer_range=0.02)
    torch.manual_seed(seed)
    with torch.device(device):
        model = Qwen2ForCausalLM(cfg).to(dtype)
    model.eval()
    for p in model.parameters():
        p.requires_grad_(False)
    return model
