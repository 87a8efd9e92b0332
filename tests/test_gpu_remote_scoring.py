"""Owner-side scoring on a row-sharded table (needs a B200): the candidate rows stay with their
owners, queries / scores / upstream gradients / query gradients travel instead.

G ranks are emulated in one process on one GPU (all peer pointers local): the phases that the
autograd function separates by barriers are run for all ranks one after the other.  Checked against
the unsharded optimizer on the union of the ranks' batches: scores, query gradients, and table /
Adam state after the step, with rows that only one pair touches (updated inside the owners' backward
kernel), rows that several pairs touch, and rows that pairs share with the ranks' ordinary lookups
(positives), whose gradients come back through the id lists.  A real two-process run over NCCL goes
through the autograd function itself."""
import os

import numpy as np
import pytest
import torch

from tests.util import RTOL, RTOL_ATOMIC, close

pytestmark = pytest.mark.gpu

D = 320        # rows of 1280 bytes: the narrowest the ragged row-stream kernels take


def _batch(rank, step, n_total, B, K, U=1):
    """U = 2: union queries, two branches per query ([B, U, 1, D] operands, [B, U, K] results)."""
    g = torch.Generator().manual_seed(77 * step + rank)
    neg = torch.randint(0, n_total, (B, K), generator=g)
    pos = torch.randint(0, n_total, (B,), generator=g)
    neg[1, :K // 2] = neg[0, :K // 2]                   # rows shared between queries of one rank
    if rank > 0:
        neg[0, :K // 4] = _batch(0, step, n_total, B, K, U)[0][0, :K // 4]  # and between ranks
    pos[0] = neg[2, 3]                                  # a row both scored remotely and looked up
    qshape, gshape = ((B, 1, D), (B, K)) if U == 1 else ((B, U, 1, D), (B, U, K))
    center = (torch.rand(*qshape, generator=g) - 0.5) * 0.2
    offset = torch.rand(*qshape, generator=g) * 0.05
    g_out = torch.randn(*gshape, generator=g) * 0.1
    g_in = torch.randn(*gshape, generator=g) * 0.1
    return neg, pos, center, offset, g_out, g_in


def _reference_step(ref_emb, ref_opt, batches, lr, fused):
    from smore_b200 import ext_ops
    ref_opt.zero_grad()
    if fused:
        ref_opt.announce_lr(lr)
    outs, losses = [], []
    for neg, pos, center, offset, g_out, g_in in batches:       # every forward read of the step first
        B, K = neg.shape
        c, o = center.cuda().requires_grad_(), offset.cuda().requires_grad_()
        neg_rows = ref_emb(neg.view(-1).cuda(), "negative_entity")
        pos_rows = ref_emb(pos.cuda(), "positive_entity")
        d_out, d_in = ext_ops.box_dist_both(neg_rows.view(B, K, -1), c, o)
        c1, o1 = (c, o) if c.dim() == 3 else (c[:, 0], o[:, 0])     # the positives meet the first branch
        p_out, p_in = ext_ops.box_dist_both(pos_rows.unsqueeze(1), c1, o1)
        losses.append((d_out * g_out.cuda()).sum() + (d_in * g_in.cuda()).sum() + (p_out + 0.5 * p_in).sum())
        outs.append([d_out.detach(), d_in.detach(), c, o])
    for loss, out in zip(losses, outs):
        loss.backward()
        out[2], out[3] = out[2].grad.clone(), out[3].grad.clone()
    ref_opt.apply_grad(lr)
    return outs


@pytest.mark.parametrize("world,U,early", [(1, 1, False), (2, 1, False), (3, 1, False), (3, 2, False), (8, 1, False),
                                           (8, 2, False), (2, 1, True), (8, 2, True)])
def test_emulated_owner_side_scoring_matches_unsharded_optimizer(world, U, early):
    """early: the owners de-duplicate the step's rows on a side stream during the forward pass (every
    lookup of the step is then made before the scoring op's forward, as the reference's model does)."""
    from smore_b200 import _lib, embedding, ext_ops, sharded
    n_total, B, K = 1501, 6, 40
    caps = (2 * B, B, B)
    torch.manual_seed(0)
    full = (torch.rand(n_total, D) - 0.5) * 0.2
    spec = sharded.RemoteSpec(pairs=B * U * K, queries=B * U, dim=D)
    shards = sharded.ShardGroup.emulated(world, n_total, D, caps, squeeze=True, remote=spec)
    for s in shards:
        s.table.zero_()
        s.table[:s.local_rows] = full[s.base:s.base + s.local_rows].cuda()
    opts = [sharded.ShardedAdamOptimizer(s, barrier=lambda: None, early_owner_plan=early) for s in shards]

    ref_emb = embedding.SparseEmbedding(n_total, D)
    ref_emb.embedding.data.copy_(full)
    ref_emb = ref_emb.cuda()
    ref_emb.train()

    class Args(object):
        optim_mode = ("aggr", "adam", "gpu", True, 0)
        share_optim_stats = False

    ref_opt = embedding.AdamEmbedOptimizer(Args(), ref_emb, 0, lazy_names=("negative_entity", "positive_entity"))
    lr = 1e-2
    _lib.async_status_clear()

    def positives_loss(r, leaves, handles):
        c, o = leaves[r]
        c1, o1 = (c, o) if U == 1 else (c[:, 0], o[:, 0])
        p_out, p_in = ext_ops.box_dist_both(handles[r][0].unsqueeze(1), c1, o1)
        return (p_out + 0.5 * p_in).sum()

    for step in range(3):
        batches = [_batch(r, step, n_total, B, K, U) for r in range(world)]
        want = _reference_step(ref_emb, ref_opt, batches, lr, fused=step == 1)
        out_shape = (B, K) if U == 1 else (B, U, K)

        for o_ in opts:
            o_.zero_grad()
            o_.announce_lr(lr)
        leaves, handles = [], []
        for r, (neg, pos, center, offset, g_out, g_in) in enumerate(batches):
            c, o = center.cuda().requires_grad_(), offset.cuda().requires_grad_()
            leaves.append((c, o))
            pos_rows = opts[r].forward(pos.cuda(), "positive_entity")
            neg_rows = opts[r].forward(neg.view(-1).cuda(), "negative_entity")
            assert isinstance(neg_rows, sharded.RemoteRows)
            handles.append((pos_rows, neg_rows))
        # (early plan: the ranks' ordinary lookups are used, so their id lists exist, before the scoring op)
        pos_losses = [positives_loss(r, leaves, handles) for r in range(world)] if early else None
        # forward: publish | every owner's share | collect
        for r in range(world):
            c, o = leaves[r]
            opts[r].remote_publish("box_both", c.detach().view(B * U, D), o.detach().view(B * U, D), B, K)
        for o_ in opts:
            o_.remote_owner_forward()
        for r in range(world):
            d_out, d_in = opts[r].remote_collect_forward(out_shape)
            close(d_out.cpu().numpy(), want[r][0].cpu().numpy(), RTOL, what="dist_out rank %d" % r)
            close(d_in.cpu().numpy(), want[r][1].cpu().numpy(), RTOL, what="dist_in rank %d" % r)
        # the ranks' ordinary lookups (positives) take the usual route: rows fetched, gradients in the lists
        for r in range(world):
            (pos_losses[r] if early else positives_loss(r, leaves, handles)).backward()
        # backward: publish upstream gradients | every owner's share | collect
        for r in range(world):
            opts[r].remote_publish_upstream([batches[r][4].cuda(), batches[r][5].cuda()])
        for o_ in opts:
            o_.remote_owner_backward()
        for r in range(world):
            g_c, g_o = opts[r].remote_collect_backward()
            c, o = leaves[r]
            close((c.grad.view(B * U, D) + g_c).cpu().numpy(), want[r][2].view(B * U, D).cpu().numpy(), RTOL_ATOMIC,
                  what="center gradient rank %d" % r)
            close((o.grad.view(B * U, D) + g_o).cpu().numpy(), want[r][3].view(B * U, D).cpu().numpy(), RTOL_ATOMIC,
                  what="offset gradient rank %d" % r)
        for o_ in opts:
            o_.apply_grad(lr)
        torch.cuda.synchronize()
        assert _lib.async_status() == 0
        table = torch.cat([s.table[:s.local_rows] for s in shards]).cpu().numpy()
        m = torch.cat([s.m[:s.local_rows] for s in shards]).cpu().numpy()
        v = torch.cat([s.v[:s.local_rows] for s in shards]).cpu().numpy()
        close(table, ref_emb.embedding.data.cpu().numpy(), RTOL_ATOMIC, what="table step %d" % step)
        close(m, ref_opt.state("state_sum_fo").cpu().numpy(), RTOL_ATOMIC, what="m step %d" % step)
        close(v, ref_opt.state("state_sum_sq").cpu().numpy(), RTOL_ATOMIC, what="v step %d" % step)
        touched = np.zeros(n_total, bool)
        for b in batches:
            touched[b[0].numpy().reshape(-1)] = True
            touched[b[1].numpy()] = True
        if step == 0:
            assert np.array_equal(table[~touched], full.numpy()[~touched])
        # the owners' distinct rows are exactly the ids of their range
        all_ids = torch.cat([torch.cat([b[0].view(-1), b[1]]) for b in batches])
        for o_ in opts:
            sh = o_.shard
            mine = torch.unique(all_ids[(all_ids >= sh.base) & (all_ids < sh.base + sh.S)] - sh.base)
            nu = int(o_._r_nuniq[0])
            assert nu == mine.numel()
            got = o_._r_uniq[:nu].cpu()
            assert torch.equal(torch.where(got < 0, ~got, got), mine)     # (~row: updated inside the backward kernel)
            assert int((got < 0).sum()) > 0


def test_union_queries_and_capacity_overflow_report():
    """[B, U, 1, dim] operands: every branch is scored as a query of its own.  And: more pairs than an
    owner's buffers hold are dropped and reported through the status word, nothing is overrun."""
    from smore_b200 import _lib, ext_ops, sharded
    n_total, B, K, U = 900, 4, 32, 2
    torch.manual_seed(3)
    full = (torch.rand(n_total, D) - 0.5) * 0.2
    spec = sharded.RemoteSpec(pairs=B * U * K, queries=B * U, dim=D)
    (shard,) = sharded.ShardGroup.emulated(1, n_total, D, (2 * B, B, B), squeeze=True, remote=spec)
    shard.table.copy_(full.cuda())
    opt = sharded.ShardedAdamOptimizer(shard, barrier=lambda: None)
    _lib.async_status_clear()
    opt.zero_grad()
    opt.announce_lr(1e-3)
    neg = torch.randint(0, n_total, (B, K))
    c = ((torch.rand(B, U, 1, D) - 0.5) * 0.2).cuda().requires_grad_()
    o = (torch.rand(B, U, 1, D) * 0.05).cuda().requires_grad_()
    rows = opt.forward(neg.view(-1).cuda(), "negative_entity").view(B, K, -1)
    d_out, d_in = ext_ops.box_dist_both(rows, c, o)          # one rank: the autograd function runs all phases itself
    assert d_out.shape == (B, U, K)
    ent = full[neg].cuda()                                    # [B, K, D]
    for u in range(U):
        w_out, w_in = ext_ops.box_dist_both(ent, c[:, u].detach(), o[:, u].detach())
        close(d_out[:, u].detach().cpu().numpy(), w_out.cpu().numpy(), RTOL, what="union branch %d out" % u)
        close(d_in[:, u].detach().cpu().numpy(), w_in.cpu().numpy(), RTOL, what="union branch %d in" % u)
    (d_out.sum() + d_in.sum()).backward()
    opt.apply_grad(1e-3)
    torch.cuda.synchronize()
    assert _lib.async_status() == 0
    assert c.grad is not None and torch.isfinite(c.grad).all()

    # an owner whose buffers are too small for what arrives
    small = sharded.RemoteSpec(pairs=B * K, queries=B, dim=D, owner_pairs=K)
    (shard2,) = sharded.ShardGroup.emulated(1, n_total, D, (2 * B, B, B), squeeze=True, remote=small)
    shard2.table.copy_(full.cuda())
    opt2 = sharded.ShardedAdamOptimizer(shard2, barrier=lambda: None)
    opt2.zero_grad()
    opt2.announce_lr(1e-3)
    rows2 = opt2.forward(neg.view(-1).cuda(), "negative_entity").view(B, K, -1)
    d2 = ext_ops.l1_dist(rows2, c[:, 0].detach())
    torch.cuda.synchronize()
    assert _lib.async_status() & _lib.STATUS_CAPACITY
    assert torch.isnan(d2).any()                               # the dropped pairs read NaN
    _lib.async_status_clear()


def _worker(rank, world, port, n_total, B, K, out_dir, steps):
    import torch.distributed as dist
    from smore_b200 import _lib, ext_ops, sharded
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    spec = sharded.RemoteSpec(pairs=B * K, queries=B, dim=D)
    shard = sharded.ShardGroup.from_process_group(n_total, D, (2 * B, B, B), squeeze=True, remote=spec)
    torch.manual_seed(0)
    full = (torch.rand(n_total, D) - 0.5) * 0.2
    shard.table.zero_()
    shard.table[:shard.local_rows] = full[shard.base:shard.base + shard.local_rows].cuda()
    opt = sharded.ShardedAdamOptimizer(shard)
    for step in range(steps):
        neg, pos, center, offset, g_out, g_in = _batch(rank, step, n_total, B, K)
        opt.zero_grad()
        opt.announce_lr(1e-2)
        c, o = center.cuda().requires_grad_(), offset.cuda().requires_grad_()
        pos_rows = opt.forward(pos.cuda(), "positive_entity")
        neg_rows = opt.forward(neg.view(-1).cuda(), "negative_entity")
        d_out, d_in = ext_ops.box_dist_both(neg_rows.view(B, K, -1), c, o)
        p_out, p_in = ext_ops.box_dist_both(pos_rows.unsqueeze(1), c, o)
        loss = (d_out * g_out.cuda()).sum() + (d_in * g_in.cuda()).sum() + (p_out + 0.5 * p_in).sum()
        loss.backward()
        opt.apply_grad(1e-2)
    torch.cuda.synchronize()
    assert _lib.async_status() == 0
    torch.save({"table": shard.table[:shard.local_rows].cpu(), "g_c": c.grad.cpu(), "g_o": o.grad.cpu()},
               os.path.join(out_dir, "rank%d.pt" % rank))
    dist.barrier()
    shard.close()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_processes_score_each_others_rows(tmp_path):
    import torch.multiprocessing as mp
    from smore_b200 import embedding
    from tests.test_gpu_sharded import _free_port
    world, n_total, B, K, steps = 2, 1501, 6, 40, 3
    for attempt in range(3):
        try:
            mp.spawn(_worker, args=(world, _free_port(), n_total, B, K, str(tmp_path), steps), nprocs=world, join=True)
            break
        except Exception as exc:
            if "EADDRINUSE" not in str(exc) or attempt == 2:
                raise
    torch.manual_seed(0)
    full = (torch.rand(n_total, D) - 0.5) * 0.2
    ref_emb = embedding.SparseEmbedding(n_total, D)
    ref_emb.embedding.data.copy_(full)
    ref_emb = ref_emb.cuda()
    ref_emb.train()

    class Args(object):
        optim_mode = ("aggr", "adam", "gpu", True, 0)
        share_optim_stats = False

    ref_opt = embedding.AdamEmbedOptimizer(Args(), ref_emb, 0, lazy_names=("negative_entity", "positive_entity"))
    for step in range(steps):
        want = _reference_step(ref_emb, ref_opt, [_batch(r, step, n_total, B, K) for r in range(world)], 1e-2, False)
    got = [torch.load(os.path.join(str(tmp_path), "rank%d.pt" % r)) for r in range(world)]
    table = torch.cat([g["table"] for g in got]).numpy()
    close(table, ref_emb.embedding.data.cpu().numpy(), RTOL_ATOMIC, what="table after %d steps" % steps)
    for r in range(world):
        close(got[r]["g_c"].numpy(), want[r][2].cpu().numpy(), RTOL_ATOMIC, what="center gradient rank %d" % r)
        close(got[r]["g_o"].numpy(), want[r][3].cpu().numpy(), RTOL_ATOMIC, what="offset gradient rank %d" % r)


def test_long_candidate_lists_and_queries_without_rows_on_an_owner():
    """K beyond what the selection keeps in registers (1024 ids per query and pass), and a query whose
    candidates all belong to one owner (the other owner's segment is empty)."""
    from smore_b200 import _lib, ext_ops, sharded
    world, n_total, B, K = 2, 2000, 3, 2309
    torch.manual_seed(5)
    full = (torch.rand(n_total, D) - 0.5) * 0.2
    spec = sharded.RemoteSpec(pairs=B * K, queries=B, dim=D)
    shards = sharded.ShardGroup.emulated(world, n_total, D, (2 * B, B, B), squeeze=True, remote=spec)
    for s in shards:
        s.table.zero_()
        s.table[:s.local_rows] = full[s.base:s.base + s.local_rows].cuda()
    opts = [sharded.ShardedAdamOptimizer(s, barrier=lambda: None) for s in shards]
    _lib.async_status_clear()
    negs, cs = [], []
    for r in range(world):
        neg = torch.randint(0, n_total, (B, K), generator=torch.Generator().manual_seed(r))
        neg[1] = torch.randint(0, shards[0].S, (K,), generator=torch.Generator().manual_seed(9 + r))   # owner 0 only
        c = ((torch.rand(B, 1, D, generator=torch.Generator().manual_seed(20 + r)) - 0.5) * 0.2).cuda()
        opts[r].zero_grad()
        opts[r].announce_lr(1e-3)
        opts[r].forward(neg.view(-1).cuda(), "negative_entity")
        negs.append(neg)
        cs.append(c)
    for r in range(world):
        opts[r].remote_publish("l1", cs[r].view(B, D), None, B, K)
    for o_ in opts:
        o_.remote_owner_forward()
    for r in range(world):
        (d,) = opts[r].remote_collect_forward((B, K))
        want = ext_ops.l1_dist(full[negs[r]].cuda(), cs[r])
        close(d.cpu().numpy(), want.cpu().numpy(), RTOL, what="l1 rank %d" % r)
    gs = [torch.randn(B, K, generator=torch.Generator().manual_seed(40 + r)).cuda() for r in range(world)]
    for r in range(world):
        opts[r].remote_publish_upstream([gs[r]])
    for o_ in opts:
        o_.remote_owner_backward()
    for r in range(world):
        g_c, _ = opts[r].remote_collect_backward()
        c = cs[r].clone().requires_grad_()
        (ext_ops.l1_dist(full[negs[r]].cuda(), c) * gs[r]).sum().backward()
        close(g_c.cpu().numpy(), c.grad.view(B, D).cpu().numpy(), RTOL_ATOMIC, what="query gradient rank %d" % r)
    for o_ in opts:
        o_.apply_grad(1e-3)
    torch.cuda.synchronize()
    assert _lib.async_status() == 0
