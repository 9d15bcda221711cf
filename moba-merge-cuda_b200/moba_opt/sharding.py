"""Multi-GPU partitioning of the MoBA path (one process per GPU, torch.distributed).

The path shards into independent units and has no exchange step: a KV head together with its group
of query heads never interacts with another group (routing, attention, merge and every gradient are
per group), and decode requests never interact at all.  So each rank works on its own units with the
single-GPU kernels and the only collective is the optional gather of outputs at the end.

  prefill  KV-head groups: rank r owns kv heads [r*Hkv/N, (r+1)*Hkv/N) and their query heads
  decode   requests:       request i lives on rank i mod N (its own cache, its own prepared plan)
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


def requests_of_rank(num_requests, world, rank):
    """Decode requests served by `rank`: i mod world == rank."""
    if not 0 <= rank < world:
        raise ValueError("rank outside the group")
    return list(range(rank, num_requests, world))


def gather_heads(local, group=None):
    """All-gathers per-rank head slices [T, H/N, D] into [T, H, D] in rank order (no autograd)."""
    world = dist.get_world_size(group)
    if world == 1:
        return local
    parts = [torch.empty_like(local) for _ in range(world)]
    dist.all_gather(parts, local.contiguous(), group=group)
    return torch.cat(parts, dim=1)


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
