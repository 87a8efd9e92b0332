"""The reference's OWN callers on top of this library.

Nothing here restates the reference: its op front-ends (smore/common/torchext/dist_func/*.py), its
models' custom_cal_logit, and its training step train_step_mp (train_process.py:172-249) are imported
from the reference package (oracle/ref_harness.py) and run with

    sys.modules["extlib_cuda"]                            = smore_b200.extlib_cuda
    sys.modules["smore.common.torchext.ext_ops"]          = smore_b200.ext_ops        (table-resident rows)
    embedding optimizers                                  = smore_b200.embedding.*

and compared with the same reference code on its torch-native path (naive_* twins, native_cal_logit,
its own AdamEmbedOptimizer) on the same GPU.  Skipped where the reference package is not available.
"""
import contextlib
import importlib
import io
import re

import numpy as np
import pytest
import torch

from oracle import ref_harness as rh
from tests.util import RTOL, RTOL_ATOMIC, close

needs_reference = pytest.mark.skipif(rh.locate() is None, reason="reference package not available")
FLOAT = re.compile(r"[-+]?(?:\d+\.\d*|\.\d+|\d+)(?:[eE][-+]?\d+)?")


@pytest.fixture()
def shim():
    from smore_b200 import extlib_cuda
    rh.forget()
    rh.install(extlib=extlib_cuda)
    yield extlib_cuda
    rh.forget()


@needs_reference
def test_reference_modules_import_against_the_shim(shim):
    """CPU: every module of the reference that sits on the path resolves its imports with the shim in
    place, and binds the shim's functions."""
    for name in ("box_dist", "l1_dist", "l2_dist", "rotate_dist", "complex_dist", "distmult_dist"):
        mod = importlib.import_module("smore.common.torchext.dist_func." + name)
        assert mod.extlib is shim
    ops = importlib.import_module("smore.common.torchext.ext_ops")
    for fn in ("l1_dist", "l2_dist", "box_dist_in", "box_dist_out", "rotate_dist", "complex_sim", "distmult_sim"):
        assert callable(getattr(ops, fn))
    importlib.import_module("smore.models.box")
    importlib.import_module("smore.common.embedding.embed_rw")
    tp = importlib.import_module("smore.training.train_process")
    assert callable(tp.train_step_mp) and callable(tp.test_step_mp)


# module, fast function, torch twin, self-check, entity row parts, query operands
FRONT_ENDS = [
    ("box_dist", "box_dist_out", "naive_box_dist_out", "test_box", 1, 2),
    ("box_dist", "box_dist_in", "naive_box_dist_in", None, 1, 2),
    ("l1_dist", "l1_dist", "naive_l1", "test_l1", 1, 1),
    ("l2_dist", "l2_dist", "naive_l2", "test_l2", 1, 1),
    ("rotate_dist", "rotate_dist", "naive_rotate_dist", "test_rotate", 2, 2),
    ("complex_dist", "complex_sim", "naive_complex_sim", "test_complex", 2, 2),
    ("distmult_dist", "distmult_sim", "naive_innerprod", "test_innerprod", 1, 1),
]


@pytest.mark.gpu
@needs_reference
@pytest.mark.parametrize("module,fast,twin,selfcheck,mul,nq", FRONT_ENDS)
def test_reference_front_ends_run_on_the_shim(shim, module, fast, twin, selfcheck, mul, nq):
    mod = importlib.import_module("smore.common.torchext.dist_func." + module)
    # (1) the file's own self-check ([30,1,400] x [1,20,400], loss = sum(out^2) * 3.14): it prints the
    # loss of the extension path, the loss of the torch twin and the mean |difference| of each gradient
    if selfcheck is not None:
        torch.manual_seed(1)
        buf = io.StringIO()
        with contextlib.redirect_stdout(buf):
            getattr(mod, selfcheck)()
        lines = [ln for ln in buf.getvalue().splitlines() if FLOAT.search(ln)]
        numbers = [float(FLOAT.search(ln).group(0)) for ln in lines]
        loss_fast, loss_twin, grad_diffs = numbers[0], numbers[1], numbers[2:]
        assert abs(loss_fast - loss_twin) <= 1e-5 * abs(loss_twin), buf.getvalue()
        assert len(grad_diffs) >= 2
        # gradients of this loss are of the order of 2 * 3.14 * |out| ~ 1e3..1e4; their mean absolute
        # difference between the two paths is rounding noise
        assert max(grad_diffs) <= 1e-5 * max(1.0, abs(loss_twin)) ** 0.5 * 10, buf.getvalue()

    # (2) 3-D per-query candidates and a 4-D two-branch union, forward and every gradient
    g = torch.Generator(device="cuda").manual_seed(5)
    B, K, dim = 6, 40, 52
    for union in (False, True):
        ent = ((torch.rand(B, K, dim * mul, device="cuda", generator=g) - 0.5) * 0.6).requires_grad_()
        qshape = (B, 2, 1, dim) if union else (B, 1, dim)
        qs = [((torch.rand(*qshape, device="cuda", generator=g) - 0.5) * 0.6) for _ in range(nq)]
        if module == "box_dist":
            qs[1] = qs[1].abs() * 0.5
        qs = [q.requires_grad_() for q in qs]
        got = getattr(mod, fast)(ent, *qs)
        want = getattr(mod, twin)(ent.unsqueeze(1) if union else ent, *qs)
        assert got.shape == want.shape
        scale = float(want.detach().abs().max()) if fast not in ("complex_sim", "distmult_sim") else \
            float(getattr(mod, twin)((ent.unsqueeze(1) if union else ent).detach().abs(), *[q.detach().abs() for q in qs]).max())
        close(got.detach().cpu().numpy(), want.detach().cpu().numpy(), RTOL, scale, what=fast)
        w = torch.randn(got.shape, device="cuda", generator=g)
        grads_fast = torch.autograd.grad((got * w).sum(), [ent] + qs)
        grads_twin = torch.autograd.grad((want * w).sum(), [ent] + qs)
        for a, b, nm in zip(grads_fast, grads_twin, ["entity", "q0", "q1"]):
            close(a.cpu().numpy(), b.cpu().numpy(), RTOL_ATOMIC, what="%s grad %s union=%s" % (fast, nm, union))


@pytest.mark.gpu
@needs_reference
@pytest.mark.parametrize("geo", ["box", "rotate", "vec"])
def test_reference_custom_cal_logit_equals_native(shim, geo):
    """<Model>.custom_cal_logit (box.py:157-164, rotate.py:137-142, vec.py:85-90) through the shim
    against the same model's native_cal_logit, per-query candidates with a two-branch union."""
    model = rh.build_model(geo, 500, 20, 44, 12.0, 8, "custom", device="cuda:0")
    g = torch.Generator(device="cuda").manual_seed(9)
    B, K, D = 8, 33, 44
    width = D * (2 if geo == "rotate" else 1)
    ent = (torch.rand(B, K, width, device="cuda", generator=g) - 0.5) * 0.6
    n_parts = 1 if geo == "vec" else 2
    query = [(torch.rand(B, 2, 1, D, device="cuda", generator=g) - 0.5) * 0.6 for _ in range(n_parts)]
    if geo == "box":
        query[1] = query[1].abs()
    got = model.custom_cal_logit(ent, None, query)
    want = model.native_cal_logit(ent, None, query)
    assert got.shape == want.shape == (B, K)
    close(got.cpu().numpy(), want.cpu().numpy(), RTOL, scale=float(want.abs().max()) + model.gamma, what=geo)


def _batches(n_ent, n_rel, B, K, structures, seed):
    g = torch.Generator().manual_seed(seed)
    cols = {"1p": "er", "2p": "err", "3p": "errr", "2i": "erer", "3i": "ererer", "ip": "ererr", "pi": "errer",
            "2u": "ereru", "up": "ererur"}
    out = []
    for s in structures:
        q = torch.empty(B, len(cols[s]), dtype=torch.int64)
        for c, kind in enumerate(cols[s]):
            q[:, c] = (torch.randint(0, n_ent, (B,), generator=g) if kind == "e" else
                       torch.randint(0, n_rel, (B,), generator=g) if kind == "r" else -1)
        pos = torch.randint(0, n_ent, (B,), generator=g)
        neg = torch.randint(0, n_ent, (B, K), generator=g)
        neg[1, :5] = neg[0, :5]          # rows shared between queries
        neg[2, :3] = pos[:3]             # and between lookups
        out.append((s, pos, neg, q))
    return out


def _run_reference_train_steps(mode, geo, batches, lr, adv, n_ent, n_rel, dim, gamma, B):
    """`batches` through the reference's train_step_mp on cuda:0.
    mode 'native'  the reference alone: native_cal_logit, its own AdamEmbedOptimizer (torch index ops)
    mode 'shim'    custom_cal_logit -> reference dist_func -> smore_b200.extlib_cuda; rows gathered;
                   smore_b200.embedding.AdamEmbedOptimizer
    mode 'rows'    smore_b200.ext_ops as the op module, negative / positive lookups table-resident"""
    from smore_b200 import embedding, ext_ops, extlib_cuda
    rh.forget()
    rh.install(extlib=extlib_cuda, ext_ops=ext_ops if mode == "rows" else None)
    rh.ensure_group()
    from smore.training.train_process import train_step_mp
    args = rh.train_args(adv=adv, optim_mode="(aggr,adam,gpu,True,0)")
    model = rh.build_model(geo, n_ent, n_rel, dim, gamma, B, "native" if mode == "native" else "custom",
                           device="cuda:0", seed=21)
    if mode == "native":
        opts = rh.reference_embedding_optimizers(model, args, 0)
    else:
        lazy = ("negative_entity", "positive_entity") if mode == "rows" else ()
        opts = {"entity_embedding": embedding.AdamEmbedOptimizer(args, model.entity_embedding, 0, lazy_names=lazy)}
    # the dense parameters get a vanishing learning rate: torch's Adam divides every element by its own
    # |gradient|, which turns rounding-noise-sized gradient elements into full-size steps of either sign;
    # what the library feeds the dense parameters is compared through their gradients instead
    dense = rh.dense_optimizer(model, 1e-9)
    dev_batches = [(s, p.cuda(), n.cuda(), q.cuda()) for s, p, n, q in batches]
    it = rh.batch_iterator(dev_batches)
    losses = []
    state = {}
    for step in range(len(batches)):
        log = train_step_mp(model, [dense], opts, it, args, step, lr, "cuda:0", 1)
        losses.append(log["loss"])
        for name, p in model.named_dense_parameters():
            if p.grad is not None:
                state["grad%d/%s" % (step, name)] = p.grad.detach().cpu().numpy().copy()
    torch.cuda.synchronize()
    state["losses"] = np.array(losses)
    state["table"] = model.entity_embedding.embedding.detach().cpu().numpy().copy()
    rh.forget()
    return state


@pytest.mark.gpu
@needs_reference
@pytest.mark.parametrize("geo,mode", [("box", "shim"), ("box", "rows"), ("rotate", "shim"), ("rotate", "rows"),
                                      ("vec", "rows")])
def test_reference_train_step_on_this_library(geo, mode):
    """Five steps (1p, 2i, 2u, up, pi) of the reference's train_step_mp with this library behind its
    three seams equal the same five steps of the reference on its own torch-native path: losses,
    the entity table (Adam with row-wise second moment) and the gradient of every dense parameter."""
    n_ent, n_rel, dim, B, K = 3000, 30, 48, 16, 64
    gamma, lr = 12.0, 1e-3
    batches = _batches(n_ent, n_rel, B, K, ["1p", "2i", "2u", "up", "pi"], seed=3)
    want = _run_reference_train_steps("native", geo, batches, lr, 0.5, n_ent, n_rel, dim, gamma, B)
    got = _run_reference_train_steps(mode, geo, batches, lr, 0.5, n_ent, n_rel, dim, gamma, B)
    np.testing.assert_allclose(got["losses"], want["losses"], rtol=1e-5)
    # a touched row moves by a few lr per step (Adam); the two tables may differ by RTOL_ATOMIC of that
    steps = len(batches)
    diff = np.abs(want["table"] - got["table"]).max()
    assert diff <= RTOL_ATOMIC * 10 * lr * steps, "entity table differs by %g" % diff
    # gradients of every dense parameter (relation tables, intersection nets) after each step: what the
    # ops' query gradients turn into
    grads = [k for k in want if k.startswith("grad")]
    assert len(grads) >= steps and set(grads) == set(k for k in got if k.startswith("grad"))
    for k in grads:
        close(got[k], want[k], RTOL_ATOMIC, what=k)
