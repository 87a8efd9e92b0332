"""The knowledge-graph binary (`train_bidir.bin`) written by smore_b200.kg_format.

Byte-exact against the reference's own container: the same triplets built and dumped by
KG::load_from_numpy + KG::dump (smore/cpp_sampler/src/lib/knowledge_graph.cpp, compiled where it lies
by oracle/build.py into oracle/_ref/libsmore_ref_kg.so); and a file written here is loaded by the
reference's KG::load and queried.  Skipped where that library was not built.  The format properties
are checked without it as well.
"""
import ctypes
import os

import numpy as np
import pytest

from smore_b200 import kg_format

HERE = os.path.dirname(os.path.abspath(__file__))
REF_KG = os.path.join(os.path.dirname(HERE), "oracle", "_ref", "libsmore_ref_kg.so")


def _ref():
    if not os.path.exists(REF_KG):
        pytest.skip("reference knowledge-graph library not built")
    lib = ctypes.CDLL(REF_KG)
    vp, sz, u64 = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_uint64
    lib.ref_kg_build_and_dump.argtypes = [vp, sz, u64, u64, ctypes.c_int, ctypes.c_int, ctypes.c_char_p]
    lib.ref_kg_load_and_query.argtypes = [ctypes.c_char_p, ctypes.c_int, vp, sz, vp, vp]
    return lib


def _triplets(rng, num_ent, num_rel, n, duplicates=True):
    h = rng.integers(0, num_ent, n)
    r = rng.integers(0, num_rel, n)
    t = rng.integers(0, num_ent, n)
    if duplicates and n > 10:
        h[:5], r[:5], t[:5] = h[5:10], r[5:10], t[5:10]          # repeated edges are stored once
    return h, r, t


@pytest.mark.parametrize("num_ent,num_rel,n,reverse,use64", [
    (50, 6, 400, True, False), (1000, 14, 5000, False, False), (7, 2, 3, True, True), (300, 8, 2000, False, True),
    (20, 4, 0, True, False), (64, 2, 4000, True, False)])
def test_written_file_is_byte_identical_to_the_reference_dump(tmp_path, num_ent, num_rel, n, reverse, use64):
    lib = _ref()
    rng = np.random.default_rng(num_ent + n)
    raw_rel = num_rel if reverse else num_rel // 2
    h, r, t = _triplets(rng, num_ent, raw_rel, n)
    dtype = np.uint64 if use64 else np.uint32
    mine, theirs = str(tmp_path / "mine.bin"), str(tmp_path / "theirs.bin")
    n_edges = kg_format.write_kg(mine, h, r, t, num_ent, num_rel, dtype=dtype, has_reverse_edges=reverse)
    trip = np.ascontiguousarray(np.stack([h, r, t], axis=1).astype(np.int64))
    if n == 0:
        pytest.skip("the reference builder does nothing for an empty edge list (setup_edges returns early)")
    assert lib.ref_kg_build_and_dump(trip.ctypes.data, n, num_ent, num_rel, int(reverse), int(use64), theirs.encode()) == 0
    a, b = open(mine, "rb").read(), open(theirs, "rb").read()
    assert len(a) == len(b) and a == b
    assert kg_format.read_kg(mine, dtype)["num_edges"] == n_edges


def test_reference_loader_reads_a_written_file(tmp_path):
    lib = _ref()
    rng = np.random.default_rng(3)
    num_ent, num_rel = 500, 10
    h, r, t = kg_format.synthetic_triplets(num_ent, num_rel // 2, 6000, seed=1)
    path = str(tmp_path / "train_bidir.bin")
    n_edges = kg_format.write_kg(path, h, r, t, num_ent, num_rel, has_reverse_edges=False)
    # queries: existing forward edges, their reverses, and random non-edges
    q = np.concatenate([np.stack([h[:200], 2 * r[:200], t[:200]], 1), np.stack([t[:200], 2 * r[:200] + 1, h[:200]], 1),
                        np.stack([rng.integers(0, num_ent, 200), rng.integers(0, num_rel, 200),
                                  rng.integers(0, num_ent, 200)], 1)]).astype(np.int64)
    q = np.ascontiguousarray(q)
    ans = np.zeros((q.shape[0], 4), np.int64)
    stats = np.zeros(4, np.uint64)
    assert lib.ref_kg_load_and_query(path.encode(), 0, q.ctypes.data, q.shape[0], ans.ctypes.data, stats.ctypes.data) == 0
    assert stats[:3].tolist() == [num_ent, num_rel, n_edges]
    fh, fr, ft = np.concatenate([h, t]), np.concatenate([2 * r, 2 * r + 1]), np.concatenate([t, h])
    edges = set(zip(fh.tolist(), fr.tolist(), ft.tolist()))
    assert len(edges) == n_edges
    out_deg = np.zeros(num_ent, np.int64)
    in_deg = np.zeros(num_ent, np.int64)
    for s, _, d in edges:
        out_deg[s] += 1
        in_deg[d] += 1
    for (s, rel, d), (fwd, bwd, od, idg) in zip(q.tolist(), ans.tolist()):
        assert bool(fwd) == ((s, rel, d) in edges)
        assert bool(bwd) == ((d, rel, s) in edges)          # ent_in is indexed by the tail
        assert od == out_deg[s] and idg == in_deg[s]


def test_format_properties_without_the_reference(tmp_path):
    rng = np.random.default_rng(9)
    num_ent, num_rel = 40, 5
    h, r, t = _triplets(rng, num_ent, num_rel, 300)
    path = str(tmp_path / "kg.bin")
    n_edges = kg_format.write_kg(path, h, r, t, num_ent, num_rel)
    kg = kg_format.read_kg(path)
    edges = sorted(set(zip(h.tolist(), r.tolist(), t.tolist())))
    assert kg["num_edges"] == n_edges == len(edges)
    # size: 3 header words + per list 1 + 2 E + 3 P + M words
    pairs_out = len(set((a, b) for a, b, _ in edges))
    pairs_in = len(set((c, b) for _, b, c in edges))
    assert os.path.getsize(path) == 4 * (3 + 2 * (1 + 2 * num_ent + n_edges) + 3 * (pairs_out + pairs_in))
    for s in range(num_ent):
        for rel in range(num_rel):
            want = [c for a, b, c in edges if a == s and b == rel]
            assert kg_format.neighbours(kg["out"], s, rel).tolist() == want
            want_in = sorted(a for a, b, c in edges if c == s and b == rel)
            assert kg_format.neighbours(kg["in"], s, rel).tolist() == want_in
    # entities without edges keep the empty range (0, 0)
    lonely = sorted(set(range(num_ent)) - set(h.tolist()))
    for s in lonely:
        assert kg["out"]["src_rel_map"][s].tolist() == [0, 0]
    with pytest.raises(ValueError):
        kg_format.write_kg(path, [num_ent], [0], [0], num_ent, num_rel)


def test_synthetic_triplets_have_the_requested_marginals():
    h, r, t = kg_format.synthetic_triplets(100000, 200, 400000, seed=2, zipf_out=1.2, zipf_rel=1.0)
    assert h.min() >= 0 and h.max() < 100000 and r.max() < 200 and t.max() < 100000
    deg = np.sort(np.bincount(h, minlength=100000))[::-1]
    assert deg[0] > 50 * deg[1000] > 0            # heavy head, long tail
    rel = np.sort(np.bincount(r, minlength=200))[::-1]
    assert 3 < rel[0] / max(rel[9], 1) < 30       # ~ 1/rank
    h2, r2, t2 = kg_format.synthetic_triplets(100000, 200, 400000, seed=2)
    assert np.array_equal(h, h2) and np.array_equal(r, r2) and np.array_equal(t, t2)
