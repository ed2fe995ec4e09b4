"""The sharded packed forward on two GPUs (NCCL): skipped where fewer than two devices are visible."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, lens):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from transformers.models.deberta_v2.configuration_deberta_v2 import DebertaV2Config
        from flashdeberta_b200 import FlashDebertaV2Model, ops
        from flashdeberta_b200.dist import ShardPlan, sharded_forward_packed
        torch.manual_seed(1)  # same weights on every rank
        cfg = DebertaV2Config(vocab_size=500, hidden_size=128, num_hidden_layers=2, num_attention_heads=2,
                              intermediate_size=256, relative_attention=True, position_buckets=256,
                              max_relative_positions=512, pos_att_type="c2p|p2c", share_att_key=True,
                              norm_rel_ebd="layer_norm", position_biased_input=False, type_vocab_size=0)
        model = FlashDebertaV2Model(cfg).eval().to(dev).bfloat16()
        g = torch.Generator().manual_seed(3)
        ids = torch.randint(1, 500, (sum(lens),), generator=g)
        plan = ShardPlan(lens, world, quadratic_weight=1 / 2000)
        got = sharded_forward_packed(model, ids[plan.local_rows(rank)].to(dev), plan)
        assert got.shape == (sum(lens), 128)
        # every rank holds the same gathered rows
        other = [torch.empty_like(got) for _ in range(world)]
        dist.all_gather(other, got)
        assert all(torch.equal(o, got) for o in other)
        # and they are what one GPU computes on the whole batch (attention bits are identical per sequence; the dense
        # layers see another row count)
        one = ShardPlan(lens, 1)
        with torch.no_grad():
            whole = model(input_ids=ids.to(dev).view(1, -1), max_seqlen=one.max_seqlen(0),
                          cu_seqlens=torch.tensor(one.cu_seqlens(0), dtype=torch.int32, device=dev)).last_hidden_state[0]
        d = (got.float() - whole.float()).abs()
        assert d.max().item() < 0.1 and d.mean().item() < 5e-3, (d.max().item(), d.mean().item())
        # the attention itself: a rank's shard of q, k, v gives the very bits of the whole batch
        H, D = 2, 64
        q, k, v = (torch.randn(sum(lens), H, D, generator=g).bfloat16().to(dev) for _ in range(3))
        pk, pq = (torch.randn(H, 512, D, generator=g).bfloat16().to(dev) for _ in range(2))
        kw = dict(position_buckets=256, max_relative_positions=512)
        cu_all = torch.tensor(ShardPlan(lens, 1).cu_seqlens(0), dtype=torch.int32, device=dev)
        full = ops.disentangled_attention(q, k, v, pk, pq, cu_seqlens=cu_all, max_seqlen=max(lens), **kw)
        rows = plan.local_rows(rank).to(dev)
        cu = torch.tensor(plan.cu_seqlens(rank), dtype=torch.int32, device=dev)
        mine = ops.disentangled_attention(q[rows], k[rows], v[rows], pk, pq, cu_seqlens=cu, max_seqlen=plan.max_seqlen(rank), **kw)
        assert torch.equal(mine, full[rows])
        ops.check_status(dev)
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_sharded_packed_forward():
    mp.spawn(_worker, args=(2, _free_port(), [900, 64, 4000, 333, 1200, 65, 700, 128]), nprocs=2, join=True)
