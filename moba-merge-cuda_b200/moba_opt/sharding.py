"""Multi-GPU partitioning of the MoBA path (one process per GPU, torch.distributed).

The path shards into independent units and has no exchange step: a KV head together with its group
of query heads never interacts with another group (routing, attention, merge and every gradient are
per group), and decode requests never interact at all.  So each rank works on its own units with the
single-GPU kernels and the only collective is the optional gather of outputs at the end.

  prefill  KV-head groups: rank r owns kv heads [r*Hkv/N, (r+1)*Hkv/N) and their query heads; where there are fewer
           KV heads than ranks the sequences of the batch are the second independent axis (`unit_slices`: rank =
           sequence part * head parts + head part)
  decode   requests:       request i lives on rank i mod N, or - when the contexts differ a lot in length - on the
                           rank `balance_requests` gives it (its own cache, its own prepared plan either way)
"""
import torch
import torch.distributed as dist


def kv_group_slices(hq, hkv, world, rank):
    """(query-head slice, kv-head slice) owned by `rank` when Hkv kv heads are split over `world` ranks."""
    if hq % hkv:
        raise ValueError("Hq must be divisible by Hkv")
    if hkv % world:
        raise ValueError(f"{hkv} KV heads cannot be split evenly over {world} ranks")
    if not 0 <= rank < world:
        raise ValueError("rank outside the group")
    per, group = hkv // world, hq // hkv
    return slice(rank * per * group, (rank + 1) * per * group), slice(rank * per, (rank + 1) * per)


def unit_grid(hkv, num_seqs, world):
    """(head parts, sequence parts) of a batch of `num_seqs` sequences with `hkv` KV heads over `world` ranks: heads are
    split as far as they go (the largest common divisor of world and Hkv), whole sequences take the rest."""
    head_parts = max(d for d in range(1, world + 1) if world % d == 0 and hkv % d == 0)
    seq_parts = world // head_parts
    if num_seqs % seq_parts:
        raise ValueError(f"{hkv} KV heads x {num_seqs} sequences cannot be split evenly over {world} ranks")
    return head_parts, seq_parts


def unit_slices(hq, hkv, num_seqs, world, rank):
    """(query-head slice, kv-head slice, range of sequences) owned by `rank`; rank = sequence part * head parts + head part."""
    if not 0 <= rank < world:
        raise ValueError("rank outside the group")
    head_parts, seq_parts = unit_grid(hkv, num_seqs, world)
    qs, ks = kv_group_slices(hq, hkv, head_parts, rank % head_parts)
    per = num_seqs // seq_parts
    return qs, ks, range((rank // head_parts) * per, (rank // head_parts + 1) * per)


def requests_of_rank(num_requests, world, rank):
    """Decode requests served by `rank`: i mod world == rank."""
    if not 0 <= rank < world:
        raise ValueError("rank outside the group")
    return list(range(rank, num_requests, world))


def expected_decode_tokens(context, chunk_size, topk, group_heads):
    """Tokens a routed decode step reads for one (request, KV head): the current, partial chunk plus the expected union
    of the topk-1 earlier chunks that each of the `group_heads` query heads of the group picks (independent picks among
    the n complete chunks: n * (1 - (1 - r/n) ** heads) with r = min(topk-1, n))."""
    n = (context - 1) // chunk_size if context > 0 else 0
    r = min(topk - 1, n)
    union = n * (1.0 - (1.0 - r / n) ** group_heads) if n else 0.0
    return union * chunk_size + (context - n * chunk_size)


def balance_requests(costs, world):
    """Spreads requests of unequal cost over `world` ranks: in order of decreasing cost (ties: lower index first), each
    request goes to the rank with the smallest total so far (ties: lower rank).  Deterministic, so every rank
    computes the same assignment without talking.  Returns one ascending list of request indices per rank."""
    if world < 1:
        raise ValueError("world must be positive")
    totals = [0.0] * world
    owned = [[] for _ in range(world)]
    for i in sorted(range(len(costs)), key=lambda i: (-float(costs[i]), i)):
        r = min(range(world), key=lambda r: (totals[r], r))
        totals[r] += float(costs[i])
        owned[r].append(i)
    return [sorted(rows) for rows in owned]


class RowGather:
    """Per-step gather of decode outputs to every rank, in request order, for a fixed assignment (one list of request
    indices per rank, as `balance_requests` returns; rank r's local rows are in the order of assignment[r]).  Buffers
    and the reordering index are built once; a call is one copy into the send slot, one all-gather and one
    index-select."""

    def __init__(self, assignment, like, group=None):
        self.group, self.world = group, dist.get_world_size(group)
        if len(assignment) != self.world:
            raise ValueError("one list of requests per rank required")
        self.assignment = [list(rows) for rows in assignment]
        self.width = max(len(rows) for rows in self.assignment)
        tail = tuple(like.shape[1:])
        self.parts = like.new_zeros((self.world, self.width) + tail)
        self.mine = self.parts[dist.get_rank(group)]
        total = sum(len(rows) for rows in self.assignment)
        where = [0] * total
        for r, rows in enumerate(self.assignment):
            for j, request in enumerate(rows):
                where[request] = r * self.width + j
        self.where = torch.tensor(where, dtype=torch.long, device=like.device)
        self.nccl = dist.get_backend(group) == "nccl"

    def __call__(self, local):
        if self.world == 1:
            return local
        send = self.mine if self.nccl else torch.zeros_like(self.mine)
        send[: local.shape[0]].copy_(local)
        if self.nccl:      # in place: the send slot is this rank's slice of the receive buffer
            dist.all_gather_into_tensor(self.parts, send, group=self.group)
        else:
            dist.all_gather(list(self.parts.unbind(0)), send, group=self.group)
        return self.parts.reshape((self.world * self.width,) + tuple(self.parts.shape[2:])).index_select(0, self.where)


def gather_assigned(local, assignment, group=None):
    """One-off form of `RowGather`."""
    return RowGather(assignment, local, group)(local)


def gather_heads(local, group=None):
    """All-gathers per-rank head slices [T, H/N, D] into [T, H, D] in rank order (no autograd)."""
    world = dist.get_world_size(group)
    if world == 1:
        return local
    parts = [torch.empty_like(local) for _ in range(world)]
    dist.all_gather(parts, local.contiguous(), group=group)
    return torch.cat(parts, dim=1)


def gather_units(local, head_parts, seq_parts, group=None):
    """All-gathers the outputs [T/seq_parts, H/head_parts, D] of the ranks of a `unit_slices` split (equal shapes: the
    sequence parts hold the same number of tokens) into [T, H, D]: tokens in sequence order, heads in head order."""
    world = dist.get_world_size(group)
    if world != head_parts * seq_parts:
        raise ValueError("the split does not match the group")
    if world == 1:
        return local
    parts = [torch.empty_like(local) for _ in range(world)]
    dist.all_gather(parts, local.contiguous(), group=group)
    return torch.cat([torch.cat(parts[s * head_parts:(s + 1) * head_parts], dim=1) for s in range(seq_parts)], dim=0)


def gather_rows(local, num_rows, group=None):
    """All-gathers per-rank request rows (rank r holds rows r, r+N, ...) back into request order."""
    world = dist.get_world_size(group)
    if world == 1:
        return local
    rank_rows = [len(requests_of_rank(num_rows, world, r)) for r in range(world)]
    width = max(rank_rows)
    padded = local.new_zeros((width,) + tuple(local.shape[1:]))
    padded[: local.shape[0]] = local
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded, group=group)
    out = local.new_empty((num_rows,) + tuple(local.shape[1:]))
    for r in range(world):
        out[r::world] = parts[r][: rank_rows[r]]
    return out


def prefill_sharded(q, k, v, cu_seqlens, max_seqlen, config, *, group=None, attend=None, gather=True):
    """Runs the prefill on this rank's KV-head groups of full [T,H,D] inputs and (optionally) gathers
    the outputs.  `attend` defaults to the registered `opt_gqa_cuda`; gradients, when wanted, are taken
    on the local output - they stay sharded exactly like the heads."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    qs, ks = kv_group_slices(q.shape[1], k.shape[1], world, rank)
    if attend is None:
        from .grouped_attention import opt_gqa_cuda as attend
    local = attend(q[:, qs], k[:, ks], v[:, ks], cu_seqlens, max_seqlen, config)
    return gather_heads(local.detach(), group) if gather else local
