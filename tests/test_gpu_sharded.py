"""Row-sharded table: G ranks emulated in one process on one GPU (all peer pointers local, phases
run rank after rank) against the unsharded optimizer fed with the union of the ranks' batches;
plus a real two-process NCCL run when two GPUs are visible (needs a B200)."""
import os
import socket

import numpy as np
import pytest
import torch

from tests.util import RTOL_ATOMIC, close

pytestmark = pytest.mark.gpu


def _rank_batch(rank, step, n_total, B, K, D):
    g = torch.Generator().manual_seed(1000 * step + rank)
    neg = torch.randint(0, n_total, (B, K), generator=g)
    pos = torch.randint(0, n_total, (B,), generator=g)
    anchors = torch.randint(0, n_total, (2, B), generator=g)
    anchors[1, : B // 2] = anchors[0, : B // 2]          # rows shared between lookups of one rank
    if rank > 0:
        neg[0, :K // 2] = _rank_batch(0, step, n_total, B, K, D)[0][0, :K // 2]   # and between ranks
    center = (torch.rand(B, 1, D, generator=g) - 0.5) * 0.2
    offset = torch.rand(B, 1, D, generator=g) * 0.05
    return neg, pos, anchors, center, offset


def _rank_forward_backward(emb_forward, batch, world):
    """One rank's part of a step: lazy candidate lookups, dense anchor lookups, box scores, loss."""
    from smore_b200 import ext_ops
    neg, pos, anchors, center, offset = batch
    B, K = neg.shape
    c = center.cuda().requires_grad_()
    o = offset.cuda().requires_grad_()
    pos_rows = emb_forward(pos.cuda(), "positive_entity")
    neg_rows = emb_forward(neg.view(-1).cuda(), "negative_entity")
    a0 = emb_forward(anchors[0].cuda(), None)
    a1 = emb_forward(anchors[1].cuda(), None)
    q_c = c + (a0 + 0.5 * a1).unsqueeze(1)
    d_out, d_in = ext_ops.box_dist_both(neg_rows.view(B, K, -1), q_c, o)
    p_out, p_in = ext_ops.box_dist_both(pos_rows.unsqueeze(1), q_c, o)
    neg_logit = 2.0 - d_out - 0.02 * d_in
    pos_logit = 2.0 - p_out - 0.02 * p_in
    loss = (-torch.nn.functional.logsigmoid(pos_logit).mean()
            - torch.nn.functional.logsigmoid(-neg_logit).mean()) / 2 / world
    loss.backward()
    return loss.item(), c.grad.clone(), o.grad.clone()


@pytest.mark.parametrize("world,squeeze", [(2, True), (3, False), (4, True)])
def test_emulated_ranks_match_unsharded_optimizer(world, squeeze):
    from smore_b200 import embedding, sharded
    n_total, D, B, K = 1003, 64, 6, 50                 # 1003 rows: the last shard is shorter
    caps = (B * K + 2 * B, B, B)
    torch.manual_seed(0)
    full = (torch.rand(n_total, D) - 0.5) * 0.2

    shards = sharded.ShardGroup.emulated(world, n_total, D, caps, squeeze=squeeze)
    for s in shards:
        s.table.zero_()
        s.table[:s.local_rows] = full[s.base:s.base + s.local_rows].cuda()
    opts = [sharded.ShardedAdamOptimizer(s, barrier=lambda: None) for s in shards]

    ref_emb = embedding.SparseEmbedding(n_total, D)
    ref_emb.embedding.data.copy_(full)
    ref_emb = ref_emb.cuda()
    ref_emb.train()

    class Args(object):
        optim_mode = ("aggr", "adam", "gpu", squeeze, 0)
        share_optim_stats = False

    ref_opt = embedding.AdamEmbedOptimizer(Args(), ref_emb, 0, lazy_names=("negative_entity", "positive_entity"))

    lr = 1e-2
    for step in range(3):
        batches = [_rank_batch(r, step, n_total, B, K, D) for r in range(world)]
        # sharded: every rank's forward/backward, then (past the barrier) every owner's update
        for o_ in opts:
            o_.zero_grad()
        got = [_rank_forward_backward(opts[r].forward, batches[r], world) for r in range(world)]
        for o_ in opts:
            o_.apply_grad(lr)
        # unsharded: the same batches through one optimizer, one update
        ref_opt.zero_grad()
        want = [_rank_forward_backward(ref_emb, batches[r], world) for r in range(world)]
        ref_opt.apply_grad(lr)
        torch.cuda.synchronize()
        for (l1, c1, o1), (l2, c2, o2) in zip(got, want):
            close(l1, l2, 1e-5, what="loss")
            close(c1.cpu().numpy(), c2.cpu().numpy(), RTOL_ATOMIC, what="query gradient")
            close(o1.cpu().numpy(), o2.cpu().numpy(), RTOL_ATOMIC, what="offset gradient")
        table = torch.cat([s.table[:s.local_rows] for s in shards]).cpu().numpy()
        m = torch.cat([s.m[:s.local_rows] for s in shards]).cpu().numpy()
        v = torch.cat([s.v[:s.local_rows] for s in shards]).cpu().numpy()
        close(table, ref_emb.embedding.data.cpu().numpy(), RTOL_ATOMIC, what="table step %d" % step)
        close(m, ref_opt.state("state_sum_fo").cpu().numpy(), RTOL_ATOMIC, what="m step %d" % step)
        close(v, ref_opt.state("state_sum_sq").cpu().numpy(), RTOL_ATOMIC, what="v step %d" % step)
        # rows nobody looked up are bit-identical to the initial table
        touched = np.zeros(n_total, bool)
        for b in batches:
            for t in (b[0], b[1], b[2]):
                touched[t.numpy().reshape(-1)] = True
        if step == 0:
            assert np.array_equal(table[~touched], full.numpy()[~touched])


def test_owner_side_index_sets_are_exact():
    """What an owner de-duplicates equals the sorted distinct ids of its range over all ranks."""
    from smore_b200 import sharded
    world, n_total, D, B, K = 3, 500, 8, 4, 30
    caps = (B * K + 2 * B, B, B)
    shards = sharded.ShardGroup.emulated(world, n_total, D, caps, squeeze=True)
    for s in shards:
        s.table.uniform_(-0.1, 0.1)
    opts = [sharded.ShardedAdamOptimizer(s, barrier=lambda: None) for s in shards]
    batches = [_rank_batch(r, 7, n_total, B, K, D) for r in range(world)]
    for o_ in opts:
        o_.zero_grad()
    for r in range(world):
        _rank_forward_backward(opts[r].forward, batches[r], world)
    all_ids = torch.cat([torch.cat([b[1], b[0].view(-1), b[2].view(-1)]) for b in batches])
    for o_ in opts:
        o_.apply_grad(1e-3)
        torch.cuda.synchronize()
        sh = o_.shard
        mine = all_ids[(all_ids >= sh.base) & (all_ids < sh.base + sh.S)] - sh.base
        want = torch.unique(mine)
        nu = int(o_._o_nuniq[0])
        assert nu == want.numel()
        assert torch.equal(o_._o_uniq[:nu].cpu(), want)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _two_process_worker(rank, world, port, n_total, D, B, K, out_dir, prefetch=False, steps=2, exchange="p2p"):
    import torch.distributed as dist
    from smore_b200 import sharded
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    caps = (B * K + 2 * B, B, B)
    shard = sharded.ShardGroup.from_process_group(n_total, D, caps, squeeze=True, exchange=exchange)
    torch.manual_seed(0)
    full = (torch.rand(n_total, D) - 0.5) * 0.2
    shard.table.zero_()
    shard.table[:shard.local_rows] = full[shard.base:shard.base + shard.local_rows].cuda()
    opt = sharded.ShardedAdamOptimizer(shard, exchange=exchange)
    batches = [tuple(t.cuda() for t in _rank_batch(rank, step, n_total, B, K, D)) for step in range(steps)]
    for step in range(steps):
        opt.zero_grad()
        if prefetch and step + 1 < steps:
            # the next step's rows are pulled from the peers' memory on a side stream (bulk copies)
            # while this step runs, and repaired from the owners' updated-rows bitmaps afterwards
            nxt = batches[step + 1]
            opt.prefetch([nxt[1], nxt[0].view(-1), nxt[2][0]])
        if prefetch and step > 0:
            assert opt._ready is not None
        _rank_forward_backward(opt.forward, batches[step], world)
        opt.apply_grad(1e-2)
    torch.cuda.synchronize()
    from smore_b200 import _lib
    assert _lib.async_status() == 0
    torch.save(shard.table[:shard.local_rows].cpu(), os.path.join(out_dir, "shard%d.pt" % rank))
    dist.barrier()
    shard.close()
    dist.destroy_process_group()


def _emulated_table(world, n_total, D, B, K, steps):
    from smore_b200 import sharded
    caps = (B * K + 2 * B, B, B)
    shards = sharded.ShardGroup.emulated(world, n_total, D, caps, squeeze=True)
    torch.manual_seed(0)
    full = (torch.rand(n_total, D) - 0.5) * 0.2
    for s in shards:
        s.table.zero_()
        s.table[:s.local_rows] = full[s.base:s.base + s.local_rows].cuda()
    opts = [sharded.ShardedAdamOptimizer(s, barrier=lambda: None) for s in shards]
    for step in range(steps):
        for o_ in opts:
            o_.zero_grad()
        for r in range(world):
            _rank_forward_backward(opts[r].forward, _rank_batch(r, step, n_total, B, K, D), world)
        for o_ in opts:
            o_.apply_grad(1e-2)
    return torch.cat([s.table[:s.local_rows] for s in shards]).cpu()


@pytest.mark.parametrize("world", [1, 2])
def test_all_to_all_exchange_matches_peer_memory_exchange(tmp_path, world):
    """ShardedAdamOptimizer(exchange="nccl"): rows and row gradients travel through
    torch.distributed.all_to_all_single instead of peer-mapped memory, the owner-side kernels read the
    received blocks.  Real processes over NCCL (a one-rank group exercises the same code on a single
    GPU) against the one-process emulation of the peer-memory path."""
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    n_total, D, B, K, steps = 1003, 64, 6, 50, 3
    for attempt in range(3):
        try:
            mp.spawn(_two_process_worker,
                     args=(world, _free_port(), n_total, D, B, K, str(tmp_path), False, steps, "nccl"),
                     nprocs=world, join=True)
            break
        except Exception as exc:
            if "EADDRINUSE" not in str(exc) or attempt == 2:
                raise
    real = torch.cat([torch.load(os.path.join(str(tmp_path), "shard%d.pt" % r)) for r in range(world)])
    close(real.numpy(), _emulated_table(world, n_total, D, B, K, steps).numpy(), RTOL_ATOMIC, what="all-to-all table")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("prefetch", [False, True])
def test_two_processes_over_nvlink_match_emulation(tmp_path, prefetch):
    """The same steps run by two real processes (NCCL barriers, peer memory mapped by the
    symmetric-memory allocator; with `prefetch` the background row pull and the refresh from the
    owners' bitmaps run on real peer memory) and by the one-process emulation give the same table."""
    import torch.multiprocessing as mp
    from smore_b200 import sharded
    world, n_total, D, B, K = 2, 1003, 64, 6, 50
    steps = 4 if prefetch else 2
    for attempt in range(3):
        try:
            mp.spawn(_two_process_worker, args=(world, _free_port(), n_total, D, B, K, str(tmp_path), prefetch, steps),
                     nprocs=world, join=True)
            break
        except Exception as exc:       # the port found free a moment ago may have been taken since
            if "EADDRINUSE" not in str(exc) or attempt == 2:
                raise
    real = torch.cat([torch.load(os.path.join(str(tmp_path), "shard%d.pt" % r)) for r in range(world)])
    caps = (B * K + 2 * B, B, B)
    shards = sharded.ShardGroup.emulated(world, n_total, D, caps, squeeze=True)
    torch.manual_seed(0)
    full = (torch.rand(n_total, D) - 0.5) * 0.2
    for s in shards:
        s.table.zero_()
        s.table[:s.local_rows] = full[s.base:s.base + s.local_rows].cuda()
    opts = [sharded.ShardedAdamOptimizer(s, barrier=lambda: None) for s in shards]
    for step in range(steps):
        for o_ in opts:
            o_.zero_grad()
        for r in range(world):
            _rank_forward_backward(opts[r].forward, _rank_batch(r, step, n_total, B, K, D), world)
        for o_ in opts:
            o_.apply_grad(1e-2)
    emu = torch.cat([s.table[:s.local_rows] for s in shards]).cpu()
    close(real.numpy(), emu.numpy(), RTOL_ATOMIC, what="two-process table")


@pytest.mark.parametrize("world", [2, 4])
def test_prefetch_with_refresh_equals_fetch_after_the_update(world):
    """Rows pulled for step s+1 while step s still runs, then repaired from the owners' updated-rows
    bitmaps, give bit-identical tables, state and losses to pulling everything after the update."""
    from smore_b200 import sharded
    n_total, D, B, K = 1003, 64, 6, 50
    caps = (B * K + 2 * B, B, B)
    torch.manual_seed(0)
    full = (torch.rand(n_total, D) - 0.5) * 0.2
    steps = 5
    batches = [[tuple(t.cuda() for t in _rank_batch(r, s, n_total, B, K, D)) for r in range(world)]
               for s in range(steps)]

    def first_group(batch):
        neg, pos, anchors = batch[0], batch[1], batch[2]
        return [pos, neg.view(-1), anchors[0]]

    results = []
    for use_prefetch in (False, True):
        shards = sharded.ShardGroup.emulated(world, n_total, D, caps, squeeze=True)
        for s in shards:
            s.table.zero_()
            s.table[:s.local_rows] = full[s.base:s.base + s.local_rows].cuda()
        opts = [sharded.ShardedAdamOptimizer(s, barrier=lambda: None) for s in shards]
        losses = []
        for step in range(steps):
            for r, o_ in enumerate(opts):
                o_.zero_grad()
                # step 3 deliberately looks up something else than what was prepared for it
                if use_prefetch and step + 1 < steps:
                    nxt = batches[step + 1][r] if step != 2 else batches[0][r]
                    o_.prefetch(first_group(nxt))
            if use_prefetch and step > 0 and step != 3:
                assert all(o_._ready is not None for o_ in opts)
            losses.append([_rank_forward_backward(opts[r].forward, batches[step][r], world)[0]
                           for r in range(world)])
            if use_prefetch:
                assert all(o_._ready is None for o_ in opts)       # consumed or dropped
            for o_ in opts:
                o_.apply_grad(1e-2)
        torch.cuda.synchronize()
        results.append((losses, torch.cat([s.table[:s.local_rows] for s in shards]).cpu(),
                        torch.cat([s.m[:s.local_rows] for s in shards]).cpu(),
                        torch.cat([s.v[:s.local_rows] for s in shards]).cpu()))
    (l0, t0, m0, v0), (l1, t1, m1, v1) = results
    # the only non-deterministic part of a step is the order of atomic adds into shared rows
    close(np.array(l1), np.array(l0), 1e-6, what="loss")
    close(t1.numpy(), t0.numpy(), RTOL_ATOMIC, what="table")
    close(m1.numpy(), m0.numpy(), RTOL_ATOMIC, what="m")
    close(v1.numpy(), v0.numpy(), RTOL_ATOMIC, what="v")


def test_shard_states_round_trip_through_reference_checkpoint_keys():
    """load_full (reference checkpoint entries) -> steps -> shard_state -> merge == concatenated shards;
    a second group of shards loaded from the merged entries continues bit-identically."""
    from smore_b200 import sharded
    world, n_total, D, B, K = 3, 1003, 64, 6, 50
    caps = (B * K + 2 * B, B, B)
    torch.manual_seed(1)
    full = (torch.rand(n_total, D) - 0.5) * 0.2

    def make(entries):
        shards = sharded.ShardGroup.emulated(world, n_total, D, caps, squeeze=True)
        for s in shards:
            s.load_full(entries["entity_embedding.embedding"], entries.get("entity_embedding.state_sum_fo"),
                        entries.get("entity_embedding.state_sum_sq"))
        return shards, [sharded.ShardedAdamOptimizer(s, barrier=lambda: None) for s in shards]

    def run(shards, opts, steps):
        for step in steps:
            for o_ in opts:
                o_.zero_grad()
            for r in range(world):
                _rank_forward_backward(opts[r].forward, _rank_batch(r, step, n_total, B, K, D), world)
            for o_ in opts:
                o_.apply_grad(1e-2)
        torch.cuda.synchronize()
        return sharded.merge_shard_states([s.shard_state() for s in shards])

    shards, opts = make({"entity_embedding.embedding": full})
    first = run(shards, opts, [0, 1])
    assert torch.equal(first["entity_embedding.embedding"], torch.cat([s.table[:s.local_rows] for s in shards]).cpu())
    assert first["entity_embedding.state_sum_sq"].shape == (n_total, 1)
    want = run(shards, opts, [2])
    shards2, opts2 = make(first)
    for o_ in opts2:
        o_.step = 2                              # the optimizer's step count is part of a checkpoint
    got = run(shards2, opts2, [2])
    for k in want:
        close(got[k].numpy(), want[k].numpy(), RTOL_ATOMIC, what=k)
