"""Host-side sharding logic, including a 2-rank gloo run on CPU."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flashdeberta_b200.dist import (ShardPlan, gather_packed, gather_sequences, partition_by_tokens,
                                    quadratic_weight_from_times, shard_batch)


def _config3_lengths():
    g = torch.Generator(device="cpu").manual_seed(2)
    u = torch.rand(256, dtype=torch.float64, generator=g)
    import math
    return torch.floor(torch.exp(math.log(64) + u * (math.log(8192) - math.log(64)))).long().tolist()


def test_partition_covers_everything_once_and_balances_tokens():
    lens = _config3_lengths()
    assert len(lens) == 256 and min(lens) >= 64 and max(lens) < 8192
    for n in (1, 2, 4, 8):
        bins = partition_by_tokens(lens, n)
        flat = sorted(i for b in bins for i in b)
        assert flat == list(range(256))
        tok = [sum(lens[i] for i in b) for b in bins]
        assert max(tok) / (sum(tok) / n) < 1.01, (n, tok)
    # cost-balanced variant keeps the quadratic term even too
    bins = partition_by_tokens(lens, 8, quadratic_weight=1 / 4096)
    cost = [sum(lens[i] + lens[i] ** 2 / 4096 for i in b) for b in bins]
    assert max(cost) / (sum(cost) / 8) < 1.03


def test_partition_edge_cases():
    assert partition_by_tokens([], 4) == [[], [], [], []]
    assert partition_by_tokens([5], 3) == [[0], [], []]
    assert partition_by_tokens([3, 3, 3, 3], 2) == [[0, 2], [1, 3]]
    with pytest.raises(ValueError):
        partition_by_tokens([1], 0)


def test_shard_batch_cuts_to_longest_owned():
    ids = torch.arange(4 * 10).view(4, 10)
    mask = torch.zeros(4, 10, dtype=torch.long)
    for b, n in enumerate([10, 2, 7, 1]):
        mask[b, :n] = 1
    got = [shard_batch(ids, mask, r, 2) for r in range(2)]
    assert got[0][2] == [0] and got[0][0].shape == (1, 10)
    assert got[1][2] == [1, 2, 3] and got[1][0].shape == (3, 7)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, lens, fail_rank):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, L, hid = len(lens), max(lens), 6
        full = torch.arange(B * L * hid, dtype=torch.float32).view(B, L, hid)
        mask = torch.zeros(B, L, dtype=torch.long)
        for b, n in enumerate(lens):
            mask[b, :n] = 1
        full = full * mask.unsqueeze(-1)
        owned = partition_by_tokens(lens, world)[rank]
        Lr = max([lens[i] for i in owned], default=1)
        local = full[owned, :Lr] if owned else torch.zeros(0, 1, hid)
        # a rank that failed on the host reports through the same object exchange the gather uses
        status = [None] * world
        dist.all_gather_object(status, "error: injected" if rank == fail_rank else "ok")
        if any(s != "ok" for s in status):
            assert status[fail_rank].startswith("error")
            return
        out = gather_sequences(local, lens, L, rank, world)
        assert torch.equal(out, full)
        # the packed form of the same exchange: only valid rows travel, padded to the largest shard
        plan = ShardPlan(lens, world)
        packed_full = torch.cat([full[b, :n] for b, n in enumerate(lens)])
        mine = packed_full[plan.local_rows(rank)]
        assert mine.shape[0] == plan.tokens[rank] == sum(lens[i] for i in owned)
        assert torch.equal(gather_packed(mine, plan), packed_full)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("lens,fail_rank", [([9, 3, 5, 1, 7], -1), ([4], -1), ([6, 6, 2], 1)])
def test_two_rank_gather_on_gloo(lens, fail_rank):
    mp.spawn(_worker, args=(2, _free_port(), lens, fail_rank), nprocs=2, join=True)


def test_shard_plan_and_cost_weight():
    lens = _config3_lengths()
    plan = ShardPlan(lens, 8)
    assert sum(plan.tokens) == plan.total == 350907 and plan.max_tokens / (plan.total / 8) < 1.001
    rows = torch.cat([plan.local_rows(r) for r in range(8)])
    assert torch.equal(torch.sort(rows).values, torch.arange(plan.total))  # every row owned exactly once
    perm = plan.gather_permutation("cpu")
    assert perm.numel() == plan.total and len(set(perm.tolist())) == plan.total
    for r in range(8):
        cu = plan.cu_seqlens(r)
        assert cu[-1] == plan.tokens[r] and len(cu) == len(plan.bins[r]) + 1
        assert plan.max_seqlen(r) == max(lens[i] for i in plan.bins[r])
    # a step whose attention (all of it quadratic here: no position terms counted) takes half of the time
    w = quadratic_weight_from_times(10.0, 5.0, [1000] * 4, att_span=0)
    assert abs(w - 1 / 1000) < 1e-9
    # with that weight the quadratic part of the cost is balanced too
    w = quadratic_weight_from_times(100.0, 60.0, lens)
    bins = partition_by_tokens(lens, 8, quadratic_weight=w)
    quad = [sum(lens[i] ** 2 for i in b) for b in bins]
    cost = [sum(lens[i] + w * lens[i] ** 2 for i in b) for b in bins]
    assert max(cost) / (sum(cost) / 8) < 1.01 and max(quad) / (sum(quad) / 8) < 1.06
