"""Multi-rank host logic on CPU (gloo, world size 2): head-group sharding of the prefill with the
output gather, and request sharding of decode.  The attention itself is the FP64 oracle here - the
point is that slicing, ownership and gather order reproduce the single-process result."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_attend(q, k, v, cu, max_len, cfg):
    from oracle import moba_oracle as mo
    qf, kf, vf = (t.double().numpy() for t in (q, k, v))
    r = mo.route_prefill(qf, kf, cu.numpy(), cfg["chunk_size"], cfg["topk"])
    return torch.from_numpy(mo.attention_fixed_route(qf, kf, vf, cu.numpy(), r["sel"], cfg["chunk_size"])["out"])


def _worker(rank, world, port, results):
    for p in (ROOT, ROOT / "moba-merge-cuda_b200"):
        sys.path.insert(0, str(p))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from moba_opt import sharding
        g = torch.Generator().manual_seed(3)
        q, k, v = torch.randn(96, 8, 16, generator=g), torch.randn(96, 4, 16, generator=g), torch.randn(96, 4, 16, generator=g)
        cu = torch.tensor([0, 40, 96], dtype=torch.int32)
        cfg = {"chunk_size": 16, "topk": 3}
        full = sharding.prefill_sharded(q, k, v, cu, 56, cfg, attend=_oracle_attend)
        whole = _oracle_attend(q, k, v, cu, 56, cfg)
        ok_prefill = torch.equal(full, whole)
        qs, ks = sharding.kv_group_slices(8, 4, world, rank)
        # decode rows: rank r serves requests r, r+2, ...
        mine = sharding.requests_of_rank(7, world, rank)
        local = torch.tensor([[float(i), float(i * i)] for i in mine])
        rows = sharding.gather_rows(local, 7)
        ok_rows = torch.equal(rows, torch.tensor([[float(i), float(i * i)] for i in range(7)]))
        # decode rows under a cost-balanced assignment (unequal numbers of requests per rank)
        assignment = sharding.balance_requests([9, 1, 1, 1, 8, 1, 1], world)
        local = torch.tensor([[float(i), float(i * i)] for i in assignment[rank]])
        ok_assigned = torch.equal(sharding.gather_assigned(local, assignment),
                                  torch.tensor([[float(i), float(i * i)] for i in range(7)]))
        results[rank] = (ok_prefill, ok_rows and ok_assigned, (qs.start, qs.stop, ks.start, ks.stop), mine)
    finally:
        dist.destroy_process_group()


def _unit_worker(rank, world, port, results):
    """Head x sequence split: 2 KV heads and 2 equal sequences over 4 ranks, one (KV head, sequence) unit each."""
    for p in (ROOT, ROOT / "moba-merge-cuda_b200"):
        sys.path.insert(0, str(p))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from moba_opt import sharding
        g = torch.Generator().manual_seed(5)
        q, k, v = torch.randn(96, 4, 16, generator=g), torch.randn(96, 2, 16, generator=g), torch.randn(96, 2, 16, generator=g)
        cu = torch.tensor([0, 48, 96], dtype=torch.int32)
        cfg = {"chunk_size": 16, "topk": 3}
        head_parts, seq_parts = sharding.unit_grid(2, 2, world)
        qs, ks, seqs = sharding.unit_slices(4, 2, 2, world, rank)
        lo, hi = int(cu[seqs.start]), int(cu[seqs.stop])
        local = _oracle_attend(q[lo:hi, qs], k[lo:hi, ks], v[lo:hi, ks], cu[seqs.start:seqs.stop + 1] - lo, 48, cfg)
        full = sharding.gather_units(local, head_parts, seq_parts)
        results[rank] = (torch.equal(full, _oracle_attend(q, k, v, cu, 48, cfg)), (head_parts, seq_parts),
                         (qs.start, qs.stop, ks.start, ks.stop, seqs.start, seqs.stop))
    finally:
        dist.destroy_process_group()


def test_four_rank_head_and_sequence_split():
    world, port = 4, _free_port()
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_unit_worker, args=(world, port, results), nprocs=world, join=True)
        out = dict(results)
    assert all(out[r][0] for r in range(world)), "gathered head x sequence split differs from the single-process result"
    assert out[0][1] == (2, 2)
    assert [out[r][2] for r in range(world)] == [(0, 2, 0, 1, 0, 1), (2, 4, 1, 2, 0, 1), (0, 2, 0, 1, 1, 2), (2, 4, 1, 2, 1, 2)]


def test_two_rank_sharding_and_gather():
    world, port = 2, _free_port()
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
        out = dict(results)
    assert out[0][0] and out[1][0], "gathered sharded prefill differs from the single-process result"
    assert out[0][1] and out[1][1], "gathered decode rows are out of order"
    assert out[0][2] == (0, 4, 0, 2) and out[1][2] == (4, 8, 2, 4)
    assert out[0][3] == [0, 2, 4, 6] and out[1][3] == [1, 3, 5]


def test_partition_contract():
    from moba_opt import sharding
    assert sharding.kv_group_slices(32, 8, 8, 3) == (slice(12, 16), slice(3, 4))
    assert sharding.kv_group_slices(14, 2, 1, 0) == (slice(0, 14), slice(0, 2))
    with pytest.raises(ValueError):
        sharding.kv_group_slices(14, 2, 4, 0)       # 2 kv heads cannot feed 4 ranks
    with pytest.raises(ValueError):
        sharding.kv_group_slices(14, 4, 2, 0)
    with pytest.raises(ValueError):
        sharding.requests_of_rank(8, 2, 2)
    # 2 KV heads x 4 sequences (the headline configuration): heads first, then whole sequences
    assert [sharding.unit_grid(2, 4, n) for n in (1, 2, 4, 8)] == [(1, 1), (2, 1), (2, 2), (2, 4)]
    assert sharding.unit_grid(8, 1, 8) == (8, 1)
    assert sharding.unit_slices(14, 2, 4, 8, 5) == (slice(7, 14), slice(1, 2), range(2, 3))
    with pytest.raises(ValueError):
        sharding.unit_grid(2, 4, 16)                # 8 units cannot feed 16 ranks
    covered = sorted(i for r in range(4) for i in sharding.requests_of_rank(64, 4, r))
    assert covered == list(range(64))


def test_balanced_request_assignment():
    from moba_opt import sharding
    costs = [int(x) for x in np.random.default_rng(0).integers(4096, 65537, size=64)]
    for world in (1, 2, 4, 8):
        owned = sharding.balance_requests(costs, world)
        assert sorted(i for rows in owned for i in rows) == list(range(64))
        totals = [sum(costs[i] for i in rows) for rows in owned]
        assert max(totals) - min(totals) <= max(costs)              # greedy bound: no rank is a whole request ahead
        naive = [sum(costs[i] for i in range(r, 64, world)) for r in range(world)]
        assert max(totals) <= max(naive)
    assert sharding.balance_requests([5, 5, 5], 2) == [[0, 2], [1]]    # ties: lower index first, lower rank first
    # cost model of a routed decode step: bounded by the context, saturating once the heads' picks cover the chunks
    assert sharding.expected_decode_tokens(100, 2048, 4, 6) == 100
    assert sharding.expected_decode_tokens(3 * 2048 + 7, 2048, 4, 6) == 3 * 2048 + 7        # 3 chunks, all picked
    assert 8 * 2048 < sharding.expected_decode_tokens(65536, 2048, 4, 6) < 18 * 2048 + 2048
