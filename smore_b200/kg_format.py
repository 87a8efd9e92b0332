"""The knowledge-graph binary the reference's online sampler loads (`train_bidir.bin`).

The sampler (smore/cpp_sampler) reads a graph with KG<Dtype>::load
(src/lib/knowledge_graph.cpp:348-362): three Dtype words `num_ent, num_rel, num_edges`, then two
"sorted lists" - the outgoing and the incoming adjacency - each laid out by SortedList<Dtype>::dump
(:55-62) as

    num_frag_rels                      one word: number of distinct (entity, relation) pairs
    src_rel_map [2 * num_ent]          per entity: [first, last+1) of its rows in rel_dst_map
    rel_dst_map [3 * num_frag_rels]    per (entity, relation): relation id, [first, last+1) in dst_list
    dst_list    [num_edges]            neighbour ids, grouped by (entity, relation), ascending

Edges are de-duplicated and ordered by (entity, relation, neighbour) (setup_edges, :96-180); an entity
without edges keeps the range (0, 0).  Dtype is uint32 (`KG32`) or uint64 (`KG64`).  Triplets given
without reverse edges get them the way the loader adds them (relation r -> 2r forward, 2r+1 backward,
:391-409).

This module writes and reads that file with numpy, and draws synthetic graphs with the marginals of
the Freebase-scale configuration (power-law out-degree and relation frequencies), so that the real
sampler can be fed at any scale without a dataset.
"""
import numpy as np

__all__ = ["sorted_list", "write_kg", "read_kg", "synthetic_triplets", "neighbours"]


def _with_reverse(heads, rels, tails):
    h = np.concatenate([heads, tails])
    r = np.concatenate([rels * 2, rels * 2 + 1])
    t = np.concatenate([tails, heads])
    return h, r, t


def sorted_list(src, rel, dst, num_ent, dtype=np.uint32):
    """The four arrays of one SortedList for edges src --rel--> dst (any order, duplicates allowed)."""
    src, rel, dst = (np.asarray(a, dtype=np.int64) for a in (src, rel, dst))
    if src.size:
        order = np.lexsort((dst, rel, src))
        src, rel, dst = src[order], rel[order], dst[order]
        keep = np.ones(src.size, bool)
        keep[1:] = (src[1:] != src[:-1]) | (rel[1:] != rel[:-1]) | (dst[1:] != dst[:-1])
        src, rel, dst = src[keep], rel[keep], dst[keep]
    n_edges = src.size
    new_pair = np.ones(n_edges, bool)
    new_pair[1:] = (src[1:] != src[:-1]) | (rel[1:] != rel[:-1])
    pair_start = np.flatnonzero(new_pair)
    n_pairs = pair_start.size
    rel_dst_map = np.empty((n_pairs, 3), dtype=np.int64)
    rel_dst_map[:, 0] = rel[pair_start]
    rel_dst_map[:, 1] = pair_start
    rel_dst_map[:, 2] = np.append(pair_start[1:], n_edges)
    src_rel_map = np.zeros((num_ent, 2), dtype=np.int64)
    pair_src = src[pair_start]
    new_src = np.ones(n_pairs, bool)
    new_src[1:] = pair_src[1:] != pair_src[:-1]
    first = np.flatnonzero(new_src)
    src_rel_map[pair_src[first], 0] = first
    src_rel_map[pair_src[first], 1] = np.append(first[1:], n_pairs)
    return (np.array([n_pairs], dtype=dtype), src_rel_map.astype(dtype).reshape(-1),
            rel_dst_map.astype(dtype).reshape(-1), dst.astype(dtype))


def write_kg(path, heads, rels, tails, num_ent, num_rel, dtype=np.uint32, has_reverse_edges=True):
    """Write the binary for the triplets (heads[i], rels[i], tails[i]).  With has_reverse_edges=False the
    relation ids are those of the raw graph (< num_rel / 2) and the reverse edges are added.  Returns
    the number of distinct edges stored."""
    heads, rels, tails = (np.asarray(a, dtype=np.int64) for a in (heads, rels, tails))
    if not has_reverse_edges:
        heads, rels, tails = _with_reverse(heads, rels, tails)
    if heads.size and (heads.min() < 0 or tails.min() < 0 or max(heads.max(), tails.max()) >= num_ent):
        raise ValueError("entity id outside [0, %d)" % num_ent)
    if rels.size and (rels.min() < 0 or rels.max() >= num_rel):
        raise ValueError("relation id outside [0, %d)" % num_rel)
    if max(num_ent * 2, heads.size) > np.iinfo(dtype).max:
        raise ValueError("graph too large for %s words" % np.dtype(dtype).name)
    out = sorted_list(heads, rels, tails, num_ent, dtype)
    inc = sorted_list(tails, rels, heads, num_ent, dtype)
    n_edges = out[3].size
    with open(path, "wb") as f:
        np.array([num_ent, num_rel, n_edges], dtype=dtype).tofile(f)
        for arrays in (out, inc):
            for a in arrays:
                a.tofile(f)
    return n_edges


def read_kg(path, dtype=np.uint32):
    """The file back as a dict: num_ent, num_rel, num_edges, and `out` / `in` sorted lists
    (num_frag_rels, src_rel_map [num_ent, 2], rel_dst_map [num_frag_rels, 3], dst_list)."""
    words = np.fromfile(path, dtype=dtype)
    num_ent, num_rel, num_edges = (int(x) for x in words[:3])
    pos = 3
    kg = {"num_ent": num_ent, "num_rel": num_rel, "num_edges": num_edges}
    for name in ("out", "in"):
        n_pairs = int(words[pos])
        pos += 1
        srm = words[pos:pos + 2 * num_ent].reshape(num_ent, 2)
        pos += 2 * num_ent
        rdm = words[pos:pos + 3 * n_pairs].reshape(n_pairs, 3)
        pos += 3 * n_pairs
        dst = words[pos:pos + num_edges]
        pos += num_edges
        kg[name] = {"num_frag_rels": n_pairs, "src_rel_map": srm, "rel_dst_map": rdm, "dst_list": dst}
    if pos != words.size:
        raise ValueError("%s: %d words expected, file has %d" % (path, pos, words.size))
    return kg


def neighbours(sorted_list_dict, entity, relation):
    """dst ids of (entity, relation) in a sorted list read by read_kg (ascending; empty if none)."""
    lo, hi = (int(x) for x in sorted_list_dict["src_rel_map"][entity])
    rows = sorted_list_dict["rel_dst_map"][lo:hi]
    hit = np.flatnonzero(rows[:, 0] == relation)
    if hit.size == 0:
        return sorted_list_dict["dst_list"][:0]
    a, b = (int(x) for x in rows[hit[0], 1:3])
    return sorted_list_dict["dst_list"][a:b]


def _power_law(rng, n, size, s):
    """Ranks in [0, n) with probability ~ (rank + 1)^-s, by inverse CDF of the continuous law."""
    u = rng.random(size)
    if abs(s - 1.0) < 1e-9:
        x = np.exp(u * np.log(n))
    else:
        x = (1.0 + u * (float(n) ** (1.0 - s) - 1.0)) ** (1.0 / (1.0 - s))
    return np.clip(np.floor(x).astype(np.int64), 1, n) - 1


def synthetic_triplets(num_ent, num_raw_rel, num_edges, seed=0, zipf_out=1.2, zipf_rel=1.0):
    """Triplets (without reverse edges) with power-law head popularity (exponent zipf_out) and relation
    frequency (zipf_rel), uniform tails; ranks are mapped to ids through fixed permutation-like
    multipliers so that popular entities are spread over the id range (and over table shards)."""
    rng = np.random.default_rng(seed)

    def spread(ranks, n):
        m = 2654435761 % n
        while m < 2 or np.gcd(m, n) != 1:
            m += 1
        return (ranks * m + 12345) % n

    heads = spread(_power_law(rng, num_ent, num_edges, zipf_out), num_ent)
    rels = spread(_power_law(rng, num_raw_rel, num_edges, zipf_rel), num_raw_rel)
    tails = rng.integers(0, num_ent, num_edges)
    return heads, rels, tails
