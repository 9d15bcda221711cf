"""CPU FP64 restatement of the reference's MoBA algorithm (numpy). TEST INFRASTRUCTURE ONLY.

This module is the checker for the CUDA path: only tests, the smoke check and the CPU-baseline
leg of the benchmark may import it.  The shipped library never routes through it.

Parity is pinned: every function here is checked against outputs of the reference's own Python
code (its routing code in src/moba_opt/grouped_attention.py run on CPU tensors, and its FP64
oracles under reference/), stored as fixtures under tests/golden/ by tests/golden/make_golden.py.

Each function cites the reference lines it follows (paths relative to the reference project).
"""
import numpy as np

NEG_INF = -np.inf


# ----------------------------------------------------------------------------- chunk metadata
def calc_chunks(cu_seqlens, chunk_size):
    """Chunk metadata of a packed batch.  Follows src/moba_opt/diagnostic.py:30-80.

    Returns (cu_chunk [n+1], chunk_to_batch [n], filtered [F]) where `filtered` lists every chunk
    except the last chunk of each sequence (the only chunks that can be routed to).
    """
    cu = np.asarray(cu_seqlens, dtype=np.int64)
    lens = cu[1:] - cu[:-1]
    nchunk = (lens + chunk_size - 1) // chunk_size
    cu_chunk = [0]
    chunk_to_batch = []
    filtered = []
    for b, (length, n) in enumerate(zip(lens.tolist(), nchunk.tolist())):
        for c in range(n):
            size = chunk_size if c < n - 1 else length - (n - 1) * chunk_size
            if c < n - 1:
                filtered.append(len(chunk_to_batch))
            chunk_to_batch.append(b)
            cu_chunk.append(cu_chunk[-1] + size)
    return (np.asarray(cu_chunk, dtype=np.int64), np.asarray(chunk_to_batch, dtype=np.int64),
            np.asarray(filtered, dtype=np.int64))


# ----------------------------------------------------------------------------- prefill routing
def route_prefill(q, k, cu_seqlens, chunk_size, topk, *, mean_rounding=None):
    """Per (token, query head) block selection.  Follows src/moba_opt/grouped_attention.py:48-71
    (route_precision='fp32', stable_routes=True), evaluated in FP64.

    q [T,Hq,D], k [T,Hkv,D]: arrays holding the (bf16-representable) input values.
    mean_rounding: optional callable applied to the chunk means (e.g. rounding to bf16 for
    route_precision='upstream', grouped_attention.py:52).

    Returns dict:
      selected [F,Hq,T] bool   - the reference's ROUTE_HOOK tensor
      sel      [T,Hq,R] int32  - global chunk ids chosen per row, ascending, -1 padded (R = min(topk-1, F))
      margin   [T,Hq]   float64 - gap between the last chosen and the best rejected score (inf when
                                  nothing legal was rejected); rows with a small margin are the only
                                  ones on which an FP32 evaluation may legitimately differ
      scale    [T,Hq]   float64 - sum_d |q_d| * max_c |mean_c,d|, the magnitude an FP32 rounding bound scales with
    """
    q = np.asarray(q, dtype=np.float64)
    k = np.asarray(k, dtype=np.float64)
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    G = Hq // Hkv
    cu = np.asarray(cu_seqlens, dtype=np.int64)
    cu_chunk, chunk_to_batch, filtered = calc_chunks(cu, chunk_size)
    F = filtered.size
    R = min(int(topk) - 1, F)
    selected = np.zeros((F, Hq, T), dtype=bool)
    sel = np.full((T, Hq, max(R, 0)), -1, dtype=np.int32)
    margin = np.full((T, Hq), np.inf)
    scale = np.zeros((T, Hq))
    if R <= 0:
        return dict(selected=selected, sel=sel, margin=margin, scale=scale, cu_chunk=cu_chunk,
                    chunk_to_batch=chunk_to_batch, filtered=filtered)
    means = np.stack([k[cu_chunk[c]:cu_chunk[c + 1]].mean(axis=0) for c in filtered])  # [F,Hkv,D]
    if mean_rounding is not None:
        means = mean_rounding(means)
    means_q = np.repeat(means, G, axis=1)  # [F,Hq,D]
    gate = np.einsum("fhd,thd->fht", means_q, q)  # [F,Hq,T]
    pos = np.arange(T)
    ends = cu_chunk[filtered + 1]
    seq_ends = cu[chunk_to_batch[filtered] + 1]
    invalid = (pos[None, :] < ends[:, None]) | (pos[None, :] >= seq_ends[:, None])  # [F,T]
    gate = np.where(invalid[:, None, :], NEG_INF, gate)
    absbound = np.einsum("fhd,thd->fht", np.abs(means_q), np.abs(q))
    absbound = np.where(invalid[:, None, :], 0.0, absbound)
    scale[:] = absbound.max(axis=0).T
    remaining = gate.copy()
    chosen_val = np.full((Hq, T), np.inf)
    for _ in range(R):
        idx = remaining.argmax(axis=0)  # first (lowest chunk) on exact ties, like torch.argmax
        val = np.take_along_axis(remaining, idx[None], axis=0)[0]
        hit = np.isfinite(val)
        f_idx, h_idx, t_idx = idx[hit], *np.nonzero(hit)
        selected[f_idx, h_idx, t_idx] = True
        chosen_val = np.where(hit, val, chosen_val)
        np.put_along_axis(remaining, idx[None], NEG_INF, axis=0)
    best_rejected = remaining.max(axis=0)  # [Hq,T]
    has_sel = selected.any(axis=0)
    m = np.where(has_sel & np.isfinite(best_rejected), chosen_val - best_rejected, np.inf)
    margin[:] = m.T
    # compact ascending list of global chunk ids
    for f in range(F):
        h_idx, t_idx = np.nonzero(selected[f])
        if h_idx.size == 0:
            continue
        slot = (sel[t_idx, h_idx] >= 0).sum(axis=-1)
        sel[t_idx, h_idx, slot] = filtered[f]
    return dict(selected=selected, sel=sel, margin=margin, scale=scale, cu_chunk=cu_chunk,
                chunk_to_batch=chunk_to_batch, filtered=filtered)


def sel_from_selected(selected, filtered, R):
    """Compact [T,Hq,R] chunk-id table (ascending, -1 padded) from the [F,Hq,T] bool tensor."""
    F, Hq, T = selected.shape
    sel = np.full((T, Hq, R), -1, dtype=np.int32)
    for f in range(F):
        h_idx, t_idx = np.nonzero(selected[f])
        if h_idx.size == 0:
            continue
        slot = (sel[t_idx, h_idx] >= 0).sum(axis=-1)
        sel[t_idx, h_idx, slot] = filtered[f]
    return sel


def selected_from_sel(sel, filtered, T, Hq):
    """Inverse of sel_from_selected."""
    lookup = {int(c): f for f, c in enumerate(np.asarray(filtered).tolist())}
    selected = np.zeros((len(lookup), Hq, T), dtype=bool)
    t_idx, h_idx, s_idx = np.nonzero(sel >= 0)
    for t, h, s in zip(t_idx.tolist(), h_idx.tolist(), s_idx.tolist()):
        selected[lookup[int(sel[t, h, s])], h, t] = True
    return selected


# ----------------------------------------------------------------------------- prefill attention
def attention_fixed_route(q, k, v, cu_seqlens, sel, chunk_size, *, d_out=None, rows=None, row_block=512, key_range=None):
    """FP64 MoBA attention under a fixed route, optionally with gradients, in query blocks (the
    reference oracle builds whole [L,L] masks; this is the same math tiled over queries).

    Forward follows reference/fixed_route_attention.py:74-119 and reference/grouped_reference.py:6-36
    (softmax scale D**-0.5, natural-log LSE).  Gradients are the closed-form derivative of that
    forward with the route held fixed (what autograd gives for grouped_reference).

    sel [T,Hq,R]: global chunk ids per row (-1 padded); R may be 0.
    rows: optional 1-D array of packed token indices to evaluate; default all.  With `rows`, d_out is
    [len(rows),Hq,D] and dq/dk/dv hold only the contributions of those rows.
    key_range: optional (lo, hi) of packed key tokens.  With it, only dk[lo:hi] and dv[lo:hi] are formed (returned as
    arrays of hi-lo rows) and dq is left out: the gradient of one key block costs the forward of the rows that attend
    it plus two small products, which is what makes a block of a 128K-token sequence checkable on a CPU.
    Returns dict(out [n,Hq,D], lse [n,Hq]) and, when d_out is given, dq, dk, dv (full size).
    """
    q = np.asarray(q, dtype=np.float64)
    k = np.asarray(k, dtype=np.float64)
    v = np.asarray(v, dtype=np.float64)
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    G = Hq // Hkv
    cu = np.asarray(cu_seqlens, dtype=np.int64)
    cu_chunk, chunk_to_batch, _ = calc_chunks(cu, chunk_size)
    chunk_of_token = np.repeat(np.arange(cu_chunk.size - 1), np.diff(cu_chunk))
    scale = D ** -0.5
    want_grad = d_out is not None
    all_rows = np.arange(T) if rows is None else np.asarray(rows, dtype=np.int64)
    out = np.zeros((all_rows.size, Hq, D))
    lse = np.zeros((all_rows.size, Hq))
    if want_grad:
        d_out = np.asarray(d_out, dtype=np.float64)
        if key_range is None:
            dq = np.zeros_like(q)
            dk = np.zeros_like(k)
            dv = np.zeros_like(v)
        else:
            k_lo, k_hi = int(key_range[0]), int(key_range[1])
            dk = np.zeros((k_hi - k_lo,) + k.shape[1:])
            dv = np.zeros((k_hi - k_lo,) + v.shape[1:])
    seq_of_row = np.searchsorted(cu, all_rows, side="right") - 1
    for b in np.unique(seq_of_row):
        s0, s1 = int(cu[b]), int(cu[b + 1])
        local = np.nonzero(seq_of_row == b)[0]
        for lo in range(0, local.size, row_block):
            idx = local[lo:lo + row_block]
            r = all_rows[idx]
            own_chunk = chunk_of_token[r]
            for h in range(Hq):
                g = h // G
                # Key set of a row (reference/fixed_route_attention.py:93-113, reference/grouped_reference.py:19-31):
                # its own chunk up to and including the row, plus every selected chunk in full.  The reference builds
                # a dense [L, L] mask; here the same set is walked chunk by chunk, so the cost follows the attended
                # pairs and a 128K-token sequence stays checkable.
                attended = np.concatenate([own_chunk[:, None], sel[r, h]], axis=1)
                pieces = []
                m = np.full(r.size, NEG_INF)
                for c in np.unique(attended[attended >= 0]).tolist():
                    ridx = np.nonzero((attended == c).any(axis=1))[0]
                    k0, k1 = int(cu_chunk[c]), int(cu_chunk[c + 1])
                    logits = (q[r[ridx], h] @ k[k0:k1, g].T) * scale
                    causal = own_chunk[ridx] == c
                    if causal.any():
                        future = np.arange(k0, k1)[None, :] > r[ridx][:, None]
                        logits = np.where(causal[:, None] & future, NEG_INF, logits)
                    m[ridx] = np.maximum(m[ridx], logits.max(axis=1))
                    pieces.append((k0, k1, ridx, logits))
                z = np.zeros(r.size)
                o = np.zeros((r.size, D))
                for i, (k0, k1, ridx, logits) in enumerate(pieces):
                    p = np.exp(logits - m[ridx, None])
                    z[ridx] += p.sum(axis=1)
                    o[ridx] += p @ v[k0:k1, g]
                    pieces[i] = (k0, k1, ridx, p)
                o /= z[:, None]
                out[idx, h] = o
                lse[idx, h] = m + np.log(z)
                if want_grad:
                    do = d_out[idx, h]
                    delta = (do * o).sum(axis=1)
                    for k0, k1, ridx, p in pieces:
                        lo_k, hi_k = (k0, k1) if key_range is None else (max(k0, k_lo), min(k1, k_hi))
                        if lo_k >= hi_k:
                            continue
                        pn = p[:, lo_k - k0:hi_k - k0] / z[ridx, None]
                        ds = pn * (do[ridx] @ v[lo_k:hi_k, g].T - delta[ridx, None]) * scale
                        base = 0 if key_range is None else k_lo
                        dk[lo_k - base:hi_k - base, g] += ds.T @ q[r[ridx], h]
                        dv[lo_k - base:hi_k - base, g] += pn.T @ do[ridx]
                        if key_range is None:
                            dq[r[ridx], h] += ds @ k[lo_k:hi_k, g]
    res = dict(out=out, lse=lse)
    if want_grad and key_range is not None:
        res.update(dk=dk, dv=dv)
    elif want_grad:
        res.update(dq=dq, dk=dk, dv=dv)
    return res


def dense_sel(cu_seqlens, chunk_size, Hq):
    """Route table under which attention_fixed_route is dense causal attention: every row selects
    every earlier chunk of its sequence (the K=1 / no-candidate fallback of
    src/moba_opt/grouped_attention.py:41-46 attends the whole causal prefix)."""
    cu = np.asarray(cu_seqlens, dtype=np.int64)
    cu_chunk, chunk_to_batch, _ = calc_chunks(cu, chunk_size)
    T = int(cu[-1])
    n = cu_chunk.size - 1
    per_seq = np.bincount(chunk_to_batch, minlength=cu.size - 1)
    R = max(int(per_seq.max()) - 1, 0)
    sel = np.full((T, Hq, R), -1, dtype=np.int32)
    first_chunk = np.concatenate(([0], np.cumsum(per_seq)))[:-1]
    for c in range(n):
        b = chunk_to_batch[c]
        prev = np.arange(first_chunk[b], c)
        sel[cu_chunk[c]:cu_chunk[c + 1], :, :prev.size] = prev
    return sel


# ----------------------------------------------------------------------------- merge
def merge_branches(outs, lses):
    """Global-softmax merge of per-branch attention results.  reference/merge_reference.py:11-30,
    src/moba_opt/ops/merge.cu:113-151.  outs: list of [N,D]; lses: list of [N] (may be -inf)."""
    ls = np.stack([np.asarray(l, dtype=np.float64) for l in lses])
    os_ = [np.asarray(o, dtype=np.float64) for o in outs]
    m = ls.max(axis=0)
    w = np.exp(ls - m)
    z = w.sum(axis=0)
    o = sum(w[j][:, None] * os_[j] for j in range(len(os_))) / z[:, None]
    return o, m + np.log(z)


# ----------------------------------------------------------------------------- decode
def chunk_means(keys, chunk_size, rounding=None):
    """Means of every *complete* chunk of one cached sequence, keys [L,Hkv,D].  FP64 mean then the
    cache-dtype rounding the reference stores (src/moba_opt/ops/paged_decode.py:41-44)."""
    keys = np.asarray(keys, dtype=np.float64)
    n = keys.shape[0] // chunk_size
    means = keys[:n * chunk_size].reshape(n, chunk_size, *keys.shape[1:]).mean(axis=1)
    return means if rounding is None else rounding(means)


def decode_route(q, means_per_seq, sequence_ids, positions, chunk_size, topk, width=None):
    """Decode block selection.  Follows src/moba_opt/ops/paged_decode.py:48-64 (score, legality
    (c+1)*C <= pos), src/moba_opt/ops/prepared_decode.py:45-55,78-94 (stable top-k: descending
    score, lowest chunk on exact ties; slot 0 = pos//C; -1 padding).

    q [Nq,Hq,D]; means_per_seq: list indexed by sequence id of [n_chunks,Hkv,D] arrays (already
    rounded to the cache dtype).  Returns dict(selected [Nq,Hq,1+R] int32 with remote slots in
    selection order, margin [Nq,Hq], scale [Nq,Hq]).
    """
    q = np.asarray(q, dtype=np.float64)
    nq, Hq, D = q.shape
    R = int(topk) - 1 if width is None else min(int(topk) - 1, width)
    selected = np.full((nq, Hq, 1 + R), -1, dtype=np.int32)
    margin = np.full((nq, Hq), np.inf)
    scale = np.zeros((nq, Hq))
    for row, (sid, pos) in enumerate(zip(sequence_ids, positions)):
        means = np.asarray(means_per_seq[sid], dtype=np.float64)
        Hkv = means.shape[1]
        G = Hq // Hkv
        legal = [c for c in range(means.shape[0]) if (c + 1) * chunk_size <= pos]
        selected[row, :, 0] = pos // chunk_size
        for h in range(Hq):
            if not legal:
                continue
            sc = means[legal, h // G] @ q[row, h]
            scale[row, h] = (np.abs(means[legal, h // G]) @ np.abs(q[row, h])).max()
            order = sorted(range(len(legal)), key=lambda i: (-sc[i], legal[i]))
            take = order[:R]
            for s, i in enumerate(take):
                selected[row, h, 1 + s] = legal[i]
            if len(order) > len(take) and take:
                margin[row, h] = sc[take[-1]] - sc[order[len(take)]]
    return dict(selected=selected, margin=margin, scale=scale)


def decode_attend(q, keys, values, sequence_ids, positions, chunk_size, selected=None):
    """FP64 attention of single query rows over cached sequences.  Follows
    reference/decode_reference.py:10-38: dense prefix [0,pos] when `selected` is None, else the
    union of the listed chunks clipped to tokens <= pos.  keys/values: lists indexed by sequence id
    of [L,Hkv,D].  Returns (out [Nq,Hq,D], lse [Nq,Hq])."""
    q = np.asarray(q, dtype=np.float64)
    nq, Hq, D = q.shape
    out = np.zeros((nq, Hq, D))
    lse = np.zeros((nq, Hq))
    for row, (sid, pos) in enumerate(zip(sequence_ids, positions)):
        kk = np.asarray(keys[sid], dtype=np.float64)
        vv = np.asarray(values[sid], dtype=np.float64)
        G = Hq // kk.shape[1]
        for h in range(Hq):
            if selected is None:
                tok = np.arange(pos + 1)
            else:
                chunks = [int(c) for c in selected[row, h] if c >= 0]
                cur = pos // chunk_size
                if not chunks or chunks[0] != cur or len(set(chunks)) != len(chunks):
                    raise ValueError("route must include current chunk exactly once")
                if any(c >= cur for c in chunks[1:]):
                    raise ValueError("route sees a future/nonhistorical chunk")
                tok = np.concatenate([np.arange(c * chunk_size, min((c + 1) * chunk_size, pos + 1)) for c in chunks])
            logits = (kk[tok, h // G] @ q[row, h]) * D ** -0.5
            m = logits.max()
            p = np.exp(logits - m)
            z = p.sum()
            out[row, h] = (p / z) @ vv[tok, h // G]
            lse[row, h] = m + np.log(z)
    return out, lse


# ----------------------------------------------------------------------------- helpers
def bf16_round(x):
    """Round-to-nearest-even to bfloat16 precision, returned as float64."""
    a = np.asarray(x, dtype=np.float32)
    u = a.view(np.uint32).astype(np.uint64)
    rounded = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return rounded.astype(np.uint32).view(np.float32).astype(np.float64).reshape(a.shape)


def fp16_round(x):
    return np.asarray(x, dtype=np.float32).astype(np.float16).astype(np.float64)


def attended_pairs(cu_seqlens, chunk_size, topk):
    """Number of attended (query, key) pairs per query head:
    sum over chunks c of s_c(s_c+1)/2 + s_c * min(topk-1, index of c in its sequence) * chunk_size."""
    cu = np.asarray(cu_seqlens, dtype=np.int64)
    total = 0
    for a, b in zip(cu[:-1].tolist(), cu[1:].tolist()):
        length = b - a
        n = (length + chunk_size - 1) // chunk_size
        for c in range(n):
            s = chunk_size if c < n - 1 else length - (n - 1) * chunk_size
            total += s * (s + 1) // 2 + s * min(topk - 1, c) * chunk_size
    return total
