"""Host-side logic of the row-sharded table, on CPU: arena layout, ownership, pointer tables, and
the handle exchange / barrier pattern over a two-process gloo group."""
import os

import pytest
import socket

import torch

from smore_b200 import sharded


def test_arena_layout_is_aligned_and_disjoint():
    lay = sharded.ArenaLayout((1000, 64, 64), 400)
    assert lay.span == 1128 and lay.prefix == [0, 1000, 1064, 1128]
    regions = []
    for p in range(3):
        regions.append((lay.nuniq_offset(p), 8))
        regions.append((lay.ids_offset(p), lay.plan_caps[p] * 8))
        regions.append((lay.grads_offset(p), lay.plan_caps[p] * 400 * 4))
    regions.sort()
    for (a, n), (b, _) in zip(regions, regions[1:]):
        assert a + n <= b
    assert regions[-1][0] + regions[-1][1] <= lay.nbytes
    assert lay.off_ids % 256 == 0 and lay.off_grads % 256 == 0
    for p in range(3):
        assert lay.grads_offset(p) % 16 == 0 and lay.ids_offset(p) % 8 == 0


def test_remote_block_layout_is_aligned_and_disjoint():
    """The peer-visible block of owner-side scoring: descriptor, candidate ids, queries, results,
    upstream gradients, partial query gradients."""
    spec = sharded.RemoteSpec(pairs=1024 * 1024 * 2, queries=2048, dim=400)
    lay = sharded.RemoteLayout(spec, world=8)
    P, QD = spec.pairs, spec.queries * spec.dim
    regions = [(lay.off_desc, 32), (lay.off_ids, P * 8)]
    regions += [(lay.off_queries + i * lay.stride_queries, QD * 4) for i in range(2)]
    regions += [(lay.off_results + i * lay.stride_pairs, P * 4) for i in range(2)]
    regions += [(lay.off_upstream + i * lay.stride_pairs, P * 4) for i in range(2)]
    regions += [(lay.off_partial + i * lay.stride_partial, 8 * QD * 4) for i in range(2)]
    regions.sort()
    for (a, n), (b, _) in zip(regions, regions[1:]):
        assert a + n <= b
    assert regions[-1][0] + regions[-1][1] <= lay.nbytes
    assert all(a % 16 == 0 for a, _ in regions)
    with pytest.raises(ValueError):
        sharded.RemoteSpec(pairs=10, queries=2, dim=30)          # rows are read 16 bytes at a time


def test_ownership_partitions_the_id_space():
    for n, g in [(1003, 3), (86054151, 8), (5, 8), (64, 1)]:
        S = sharded.shard_rows(n, g)
        ids = torch.tensor([0, S - 1, S, n - 1]).clamp_(0, n - 1)
        own = sharded.owner_of(ids, n, g)
        assert int(own.max()) < g and int(own.min()) >= 0
        assert (ids - own * S >= 0).all() and (ids - own * S < S).all()
        assert S * g >= n and S * (g - 1) < n or g == 1 or n < g


def test_pointer_tables_follow_list_order():
    lay = sharded.ArenaLayout((10, 4), 8)
    tabs = sharded.pointer_tables(lay, [1 << 20, 2 << 20, 3 << 20])
    assert len(tabs["ids"]) == 6
    assert tabs["ids"][0] == (1 << 20) + lay.ids_offset(0) and tabs["ids"][3] == (2 << 20) + lay.ids_offset(1)
    assert tabs["grads"][5] == (3 << 20) + lay.grads_offset(1)
    assert tabs["nuniq"][2] == (2 << 20) + lay.nuniq_offset(0)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _gloo_worker(rank, world, port, out_dir):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    handles = sharded.exchange_handles([b"table-%d" % rank, b"arena-%d" % rank])
    lay = sharded.ArenaLayout((16, 4), 8)
    tabs = sharded.pointer_tables(lay, [(g + 1) << 24 for g in range(world)])
    # the barrier pattern of a step: a one-element all-reduce; every rank's phase-1 write is visible
    # to every rank after it
    store = torch.zeros(world)
    store[rank] = rank + 1.0
    dist.all_reduce(store)
    torch.save({"handles": handles, "tabs": tabs, "store": store}, os.path.join(out_dir, "r%d.pt" % rank))
    dist.barrier()
    dist.destroy_process_group()


def test_handle_exchange_and_barrier_over_gloo(tmp_path):
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_gloo_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    views = [torch.load(os.path.join(str(tmp_path), "r%d.pt" % r), weights_only=False) for r in range(world)]
    assert views[0]["handles"] == views[1]["handles"] == [[b"table-0", b"arena-0"], [b"table-1", b"arena-1"]]
    assert views[0]["tabs"] == views[1]["tabs"]          # every rank indexes the lists identically
    assert views[0]["store"].tolist() == views[1]["store"].tolist() == [1.0, 2.0]


def test_shard_states_merge_to_reference_checkpoint_keys():
    """Per-rank shard states -> the keys a reference checkpoint holds for the entity table, and back."""
    import torch
    from smore_b200 import sharded
    n, w, world = 1003, 8, 4
    full = {"embedding": torch.randn(n, w), "state_sum_fo": torch.randn(n, w), "state_sum_sq": torch.rand(n, 1)}
    states = []
    for r in reversed(range(world)):          # any order
        st = {"rank": r, "world": world, "n_rows_total": n, "width": w, "squeeze": True}
        st.update({k: sharded.rows_of_rank(v, r, world).clone() for k, v in full.items()})
        states.append(st)
    assert sum(st["embedding"].shape[0] for st in states) == n
    merged = sharded.merge_shard_states(states)
    assert sorted(merged) == ["entity_embedding.embedding", "entity_embedding.state_sum_fo",
                              "entity_embedding.state_sum_sq"]
    for k, v in full.items():
        assert torch.equal(merged["entity_embedding." + k], v)
    with pytest.raises(ValueError):
        sharded.merge_shard_states(states[:-1])
    states[0]["width"] = 9
    with pytest.raises(ValueError):
        sharded.merge_shard_states(states)
