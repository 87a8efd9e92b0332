"""Generate the golden vectors under tests/golden/ from the reference's own Python code.

Run once, in a container where the reference tree is mounted:

    python tests/golden/make_golden.py [--reference /path/to/smore-checkout]

What is executed is the reference's code, imported from its tree, on CPU:
  * the pure-torch twins that sit beside each custom op
    (smore/common/torchext/dist_func/*.py: naive_l1, naive_l2, naive_box_dist_out,
    naive_box_dist_in, naive_rotate_dist, naive_complex_sim, naive_innerprod), with the
    self-check loss `sum(out ** 2) * 3.14` those files use, differentiated by autograd;
  * the models' native logits (smore/models/{vec,box,rotate}.py: native_cal_logit) on a
    training-shaped batch (per-query negatives and a two-branch union);
  * the evaluation step test_step_mp (smore/training/train_process.py:94-169) with a stand-in model
    that returns seeded logits: its logged MRR / HITS per query (reference_ranking.npz);
  * merge_grad_indices / merge_grad_list and AdamEmbedOptimizer / AdaGradEmbedOptimizer /
    SGDEmbedOptimizer.update_step (smore/common/embedding/embed_optimizer.py) for three
    consecutive steps, with full and row-wise second moments.
The reference imports three modules that are not installed here and that this path does
not need for its arithmetic: `extlib_cuda` (the CUDA extension being replaced), and
`torch_scatter` (only `scatter(src, index, dim=0, reduce="sum")` is reached, stood in for
by zeros().index_add_()).  The optimizer classes are driven through a small in-memory
stand-in for EmbeddingRW (read = table[idx], additive write = index_add_, as
smore/common/embedding/embed_rw.py:74-77,102-111 do for a GPU-resident table).
Inputs are seeded; outputs are stored as float32/int64 arrays in .npz files.
"""
import argparse
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _install_stubs():
    ext = types.ModuleType("extlib_cuda")
    sys.modules["extlib_cuda"] = ext
    ts = types.ModuleType("torch_scatter")

    def scatter(src, index, dim=0, reduce="sum"):
        assert dim == 0 and reduce == "sum"
        n = int(index.max().item()) + 1 if index.numel() else 0
        out = torch.zeros((n,) + tuple(src.shape[1:]), dtype=src.dtype)
        out.index_add_(0, index, src)
        return out

    ts.scatter = scatter
    sys.modules["torch_scatter"] = ts
    for name in ("tensorboardX", "pickle5", "libsampler"):
        if name not in sys.modules:
            m = types.ModuleType(name)
            m.SummaryWriter = m.GlobalSummaryWriter = object
            sys.modules[name] = m
    if "smore.cpp_sampler.online_sampler" not in sys.modules:
        m = types.ModuleType("smore.cpp_sampler.online_sampler")
        m.OnlineSampler = object
        sys.modules["smore.cpp_sampler.online_sampler"] = m


def _np(t):
    return t.detach().cpu().numpy().copy()


def op_cases(out):
    from smore.common.torchext.dist_func import (box_dist, complex_dist, distmult_dist, l1_dist, l2_dist,
                                                 rotate_dist)
    twins = {
        "l1": (l1_dist.naive_l1, 1, 1),
        "l2": (l2_dist.naive_l2, 1, 1),
        "box_out": (box_dist.naive_box_dist_out, 1, 2),
        "box_in": (box_dist.naive_box_dist_in, 1, 2),
        "rotate": (rotate_dist.naive_rotate_dist, 2, 2),
        "complex": (complex_dist.naive_complex_sim, 2, 2),
        "distmult": (distmult_dist.naive_innerprod, 1, 1),
    }
    # (be, ne, bc, nc, dim): the reference self-check shape, then training-like broadcasts
    shapes = {
        "selfcheck": (30, 1, 1, 20, 200),
        "per_query_neg": (6, 9, 6, 1, 52),
        "shared_neg": (1, 11, 5, 1, 36),
        "positives": (7, 1, 7, 1, 33),
    }
    for sname, (be, ne, bc, nc, dim) in shapes.items():
        for op, (fn, mul, nq) in twins.items():
            g = torch.Generator().manual_seed((sum(map(ord, sname + op)) * 7919) % (2 ** 31))
            entity = torch.randn(be, ne, dim * mul, generator=g).requires_grad_()
            qs = [torch.randn(bc, nc, dim, generator=g) for _ in range(nq)]
            if op.startswith("box"):
                qs[1] = qs[1].abs() * 0.7   # box offsets are non-negative in the models
            qs = [q.requires_grad_() for q in qs]
            res = fn(entity, *qs)
            loss = torch.sum(res ** 2) * 3.14
            loss.backward()
            key = "%s/%s/" % (sname, op)
            out[key + "entity"] = _np(entity)
            for i, q in enumerate(qs):
                out[key + "q%d" % i] = _np(q)
                out[key + "g_q%d" % i] = _np(q.grad)
            out[key + "out"] = _np(res)
            out[key + "g_entity"] = _np(entity.grad)


def logit_cases(out):
    from smore.models.box import BoxReasoning
    from smore.models.rotate import RotateReasoning
    from smore.models.vec import VecReasoning
    B, K, U, D = 5, 8, 2, 44
    g = torch.Generator().manual_seed(1234)
    me = types.SimpleNamespace(gamma=12.0, cen=0.02)
    ent = (torch.rand(B, K, D, generator=g) - 0.5) * 0.6
    center = (torch.rand(B, U, 1, D, generator=g) - 0.5) * 0.6
    offset = torch.rand(B, U, 1, D, generator=g) * 0.3
    out["logit/box/entity"], out["logit/box/center"], out["logit/box/offset"] = _np(ent), _np(center), _np(offset)
    out["logit/box/out"] = _np(BoxReasoning.native_cal_logit(me, ent, None, (center, offset)))
    out["logit/vec/out"] = _np(VecReasoning.native_cal_logit(me, ent, None, (center,)))
    ent2 = (torch.rand(B, K, 2 * D, generator=g) - 0.5) * 0.6
    re = (torch.rand(B, U, 1, D, generator=g) - 0.5) * 0.6
    im = (torch.rand(B, U, 1, D, generator=g) - 0.5) * 0.6
    out["logit/rotate/entity"], out["logit/rotate/re"], out["logit/rotate/im"] = _np(ent2), _np(re), _np(im)
    out["logit/rotate/out"] = _np(RotateReasoning.native_cal_logit(me, ent2, None, (re, im)))


class _MemRW:
    """What EmbeddingRW does for a table that lives on the compute device."""

    def __init__(self, t):
        self.embed = t

    def read(self, indices, name=None):
        return self.embed[indices.view(-1)]

    def write(self, indices, values, name=None, additive=False):
        if additive:
            self.embed.index_add_(0, indices, values)
        else:
            self.embed.index_copy_(0, indices, values)


def optimizer_cases(out):
    from smore.common.embedding import embed_optimizer as eo
    N, D = 97, 24
    g = torch.Generator().manual_seed(77)
    idx_lists, grad_lists = [], []
    for step in range(3):
        idx = [torch.randint(0, N, (n,), generator=g) for n in (5, 40, 5)]
        grads = [torch.randn(i.numel(), D, generator=g) * 0.1 for i in idx]
        idx_lists.append(idx)
        grad_lists.append(grads)
        out["opt/step%d/idx" % step] = _np(torch.cat(idx))
        out["opt/step%d/grad" % step] = _np(torch.cat(grads))
    table0 = (torch.rand(N, D, generator=g) - 0.5)
    out["opt/table0"] = _np(table0)
    lr = 1e-2
    out["opt/lr"] = np.float64(lr)
    for opt_name, cls in (("adam", eo.AdamEmbedOptimizer), ("adagrad", eo.AdaGradEmbedOptimizer),
                          ("sgd", eo.SGDEmbedOptimizer)):
        for squeeze in (False, True):
            if opt_name == "sgd" and squeeze:
                continue
            table = table0.clone()
            me = types.SimpleNamespace(optimizer_device="gpu", squeeze=squeeze, step=0, embed_rw=_MemRW(table))
            if opt_name == "adam":
                me.state_sum_fo_rw = _MemRW(torch.zeros(N, D))
                me.state_sum_sq_rw = _MemRW(torch.zeros(N, 1) if squeeze else torch.zeros(N, D))
            elif opt_name == "adagrad":
                me.state_sum_rw = _MemRW(torch.zeros(N, 1) if squeeze else torch.zeros(N, D))
            tag = "opt/%s_%s/" % (opt_name, "rowwise" if squeeze else "full")
            for step in range(3):
                me.step += 1
                merged_idx, inverse = eo.merge_grad_indices(idx_lists[step])
                merged_grad = eo.merge_grad_list(grad_lists[step], inverse)
                if opt_name == "adam" and not squeeze:
                    out["opt/step%d/uniq" % step] = _np(merged_idx)
                    out["opt/step%d/inverse" % step] = _np(inverse)
                    out["opt/step%d/merged_grad" % step] = _np(merged_grad)
                cls.update_step(me, merged_idx, inverse, merged_grad, lr)
                out[tag + "table_after%d" % step] = _np(table)
                if opt_name == "adam":
                    out[tag + "m_after%d" % step] = _np(me.state_sum_fo_rw.embed)
                    out[tag + "v_after%d" % step] = _np(me.state_sum_sq_rw.embed)
                elif opt_name == "adagrad":
                    out[tag + "v_after%d" % step] = _np(me.state_sum_rw.embed)


class _StubLoader(list):
    """What test_step_mp needs of a DataLoader: iteration, len(), .dataset.all_entity_idx."""

    def __init__(self, items, n_entities):
        super().__init__(items)
        self.dataset = types.SimpleNamespace(all_entity_idx=torch.arange(n_entities).unsqueeze(0))


class _StubModel:
    """Returns prepared logits for whatever query it is asked to score against all entities."""

    def __init__(self, logits):
        self.logits = logits
        self.entity_embedding = lambda idx: torch.zeros(1, 1)

    def eval(self):
        return self

    def __call__(self, positive, negative_sample, query_structure, query_mat, device=None, all_neg=None):
        return None, self.logits[int(query_mat[0, 0])].reshape(1, -1).clone(), None


def ranking_cases(out):
    """The reference's evaluation step itself - smore/training/train_process.py:94-169, test_step_mp -
    run on the CPU for one query at a time with a model that returns seeded logits over N candidates:
    what it logs per query structure (MRR, HITS1/3/10, HITS1max) is what the library's filtered ranks
    have to reproduce.  Cases: continuous logits; logits quantised so that many candidates tie with
    each other (but no answer ties with anything); one answer that ties with other candidates."""
    import torch.distributed as dist
    if not dist.is_initialized():
        import tempfile
        dist.init_process_group("gloo", init_method="file://" + os.path.join(tempfile.mkdtemp(), "store"),
                                rank=0, world_size=1)
    from smore.training.train_process import test_step_mp
    g = torch.Generator().manual_seed(4242)
    N = 3000
    cases = []      # (logits [N], easy ids, hard ids, tag)
    for tag, n_easy, n_hard, levels in (("plain", 0, 1, 0), ("plain", 5, 3, 0), ("plain", 40, 60, 0),
                                        ("ties_elsewhere", 7, 9, 6), ("ties_elsewhere", 0, 25, 3),
                                        ("tie_on_answer", 2, 2, 4)):
        logits = torch.randn(N, generator=g)
        ids = torch.randperm(N, generator=g)[:n_easy + n_hard].tolist()
        easy, hard = ids[:n_easy], ids[n_easy:]
        if levels:
            logits = torch.round(logits * levels) / levels
            if tag == "ties_elsewhere":
                # give every answer a value no other candidate has
                for j, a in enumerate(easy + hard):
                    logits[a] = logits[a] + 0.01 + 0.0001 * j
        if n_hard:
            logits[hard[0]] = logits.max() + (1.0 if tag != "tie_on_answer" else 0.0)
        cases.append((logits, easy, hard, tag))
    args = types.SimpleNamespace(eval_link_pred=False, eval_batch_size=1, print_on_screen=False, nentity=N,
                                 test_log_steps=1000000)
    model = _StubModel([c[0] for c in cases])
    out["rank/n_cases"] = np.int64(len(cases))
    for i, (logits, easy, hard, tag) in enumerate(cases):
        structure = ("e", ("r",))
        item = (None, [[i, 0]], [(i, (0,))], [structure], [set(easy)], [set(hard)])
        collected = []
        buf = types.SimpleNamespace(put=collected.append)
        test_step_mp(model, args, None, _StubLoader([item], N), buf, 0, "cpu", "test")
        logs = collected[0][0][structure]
        out["rank/%d/logits" % i] = _np(logits)
        out["rank/%d/easy" % i] = np.array(sorted(set(easy)), np.int64)
        out["rank/%d/hard" % i] = np.array(sorted(set(hard)), np.int64)
        out["rank/%d/tag" % i] = np.array(tag)
        out["rank/%d/metrics" % i] = np.array([logs[k] for k in ("MRR", "HITS1", "HITS3", "HITS10", "HITS1max")],
                                              np.float64)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("SMORE_REFERENCE_DIR", ""),
                    help="checkout of the reference (default: $SMORE_REFERENCE_DIR)")
    a = ap.parse_args()
    if not os.path.isdir(os.path.join(a.reference, "smore")):
        raise SystemExit("give the reference checkout with --reference or $SMORE_REFERENCE_DIR")
    sys.path.insert(0, a.reference)
    _install_stubs()
    torch.manual_seed(1)
    torch.set_num_threads(1)
    for name, fn in (("ops", op_cases), ("logits", logit_cases), ("optimizer", optimizer_cases),
                     ("ranking", ranking_cases)):
        out = {}
        fn(out)
        path = os.path.join(HERE, "reference_%s.npz" % name)
        np.savez_compressed(path, **out)
        print(path, len(out), "arrays", os.path.getsize(path) // 1024, "KiB")


if __name__ == "__main__":
    main()
