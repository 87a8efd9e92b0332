"""Drive the reference's OWN Python (models, op front-ends, training and test steps) from tests
and from the benchmark's reference arm.

TEST INFRASTRUCTURE: nothing under smore_b200/ imports this module.

The reference package is imported from a checkout ($SMORE_REFERENCE_DIR) or from the copy that
oracle/build.py places under oracle/_ref/pyref.  Four of its imports do not resolve on a machine
without its build products and extra wheels; they are stood in for as follows:

  extlib_cuda       the module under test (smore_b200.extlib_cuda) when `extlib` is given, else an
                    empty module (enough for the torch-native code paths, which never call it)
  torch_scatter     only scatter(src, index, dim=0, reduce="sum") is reached
                    (embed_optimizer.py:47); stood in for by zeros().index_add_()
  tensorboardX, pickle5, libsampler, smore.cpp_sampler.online_sampler
                    imported at module level by train_process.py / main_train.py, never used by
                    train_step_mp / test_step_mp themselves

Everything that computes is the reference's code: `KGReasoning.forward`, `custom_cal_logit` /
`native_cal_logit`, `train_step_mp` (train_process.py:172-249), `test_step_mp` (:94-169), and its
embedding optimizers (`reference_embedding_optimizers`).
"""
import os
import sys
import types

import torch

HERE = os.path.dirname(os.path.abspath(__file__))

STRUCTURES = {          # smore/common/config.py:21-43
    "1p": ("e", ("r",)),
    "2p": ("e", ("r", "r")),
    "3p": ("e", ("r", "r", "r")),
    "2i": (("e", ("r",)), ("e", ("r",))),
    "3i": (("e", ("r",)), ("e", ("r",)), ("e", ("r",))),
    "ip": ((("e", ("r",)), ("e", ("r",))), ("r",)),
    "pi": (("e", ("r", "r")), ("e", ("r",))),
    "2u": (("e", ("r",)), ("e", ("r",)), ("u",)),
    "up": ((("e", ("r",)), ("e", ("r",)), ("u",)), ("r",)),
}


def locate():
    """Directory that holds the reference's `smore` package, or None."""
    for cand in (os.environ.get("SMORE_REFERENCE_DIR", ""), os.path.join(HERE, "_ref", "pyref")):
        if cand and os.path.isfile(os.path.join(cand, "smore", "common", "torchext", "ext_ops.py")):
            return cand
    return None


def _scatter_sum(src, index, dim=0, reduce="sum"):
    assert dim == 0 and reduce == "sum"
    n = int(index.max().item()) + 1 if index.numel() else 0
    out = torch.zeros((n,) + tuple(src.shape[1:]), dtype=src.dtype, device=src.device)
    out.index_add_(0, index, src)
    return out


def install(extlib=None, ext_ops=None):
    """Make `import smore...` resolve to the reference package with the stand-ins above.  Call it
    before the first import of the reference (after forget(), to change the stand-ins: the
    reference's modules bind them at import).  `ext_ops`, when given, is installed as
    smore.common.torchext.ext_ops - the module the reference's models take their ops from."""
    root = locate()
    if root is None:
        raise RuntimeError("reference package not found: set SMORE_REFERENCE_DIR or run oracle/build.py "
                           "where the reference checkout is available")
    if root not in sys.path:
        sys.path.insert(0, root)
    sys.modules["extlib_cuda"] = extlib if extlib is not None else types.ModuleType("extlib_cuda")
    if "torch_scatter" not in sys.modules:
        ts = types.ModuleType("torch_scatter")
        ts.scatter = _scatter_sum
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
    if ext_ops is not None:
        sys.modules["smore.common.torchext.ext_ops"] = ext_ops
    return root


def forget():
    """Drop the imported reference modules (to import them again against another extlib_cuda)."""
    for name in [n for n in sys.modules if n == "smore" or n.startswith("smore.")]:
        del sys.modules[name]
    sys.modules.pop("extlib_cuda", None)


def ensure_group():
    """train_step_mp / test_step_mp call torch.distributed; give them a one-rank group if none exists."""
    import torch.distributed as dist
    if not dist.is_initialized():
        import tempfile
        store = os.path.join(tempfile.mkdtemp(prefix="smore_ref_"), "store")
        dist.init_process_group("gloo", init_method="file://" + store, rank=0, world_size=1)


def train_args(adv=None, optim_mode="(aggr,adam,gpu,True,0)", share_optim_stats=False):
    """The fields train_step_mp and the embedding optimizers read from the parsed command line."""
    return types.SimpleNamespace(
        reg_coeff=0.0, negative_adversarial_sampling=adv is not None,
        adversarial_temperature=adv if adv is not None else 1.0,
        online_sample_mode="(0,0,u,u,0)", optim_mode=optim_mode, share_optim_stats=share_optim_stats)


def build_model(geo, nentity, nrelation, dim, gamma, batch_size, logit_impl, cen=0.02, device="cpu", seed=0):
    """A reference model with the entity table sparse (row-wise optimizer) and relations dense, as the
    training recipes configure it (--sparse_embeddings e ... --sparse_device gpu)."""
    from smore.common.util import query_name_dict
    torch.manual_seed(seed)
    common = dict(nentity=nentity, nrelation=nrelation, hidden_dim=dim, gamma=gamma, optim_mode=None,
                  batch_size=batch_size, test_batch_size=1, sparse_embeddings="e", sparse_device="gpu",
                  use_cuda=False, query_name_dict=query_name_dict, logit_impl=logit_impl)
    if geo == "box":
        from smore.models.box import BoxReasoning
        model = BoxReasoning(box_mode=("none", cen), **common)
    elif geo == "rotate":
        from smore.models.rotate import RotateReasoning
        model = RotateReasoning(rotate_mode=("Mean", True), **common)
    elif geo == "vec":
        from smore.models.vec import VecReasoning
        model = VecReasoning(model_config=("l1",), **common)
    else:
        raise ValueError("geo %r" % (geo,))
    if str(device) != "cpu":
        model.to_device(str(device))
    elif geo == "box":
        model.zero_offset_tensor = torch.zeros([batch_size, 1, dim])
        model.empty_logit_tensor = torch.tensor([])
    return model


class MemoryRW(object):
    """EmbeddingRW (embed_rw.py:95-134) for a table that already lives on the compute device, CPU
    included: read = table[idx], write = index_add_ / index_copy_, as embed_rw.py:74-77,102-111 do
    for a GPU-resident table.  The reference class itself asserts a GPU and opens a CUDA stream
    (embed_rw.py:46-48), so the CPU reference arm drives the reference optimizers through this."""

    def __init__(self, embed, gpu_id=-1):
        self.embed = embed.data
        self.gpu_id = gpu_id
        self.dummy_job = types.SimpleNamespace(sync=lambda: None)

    def read(self, indices, name=None):
        out = self.embed if indices is None else self.embed[indices.view(-1)]
        out.job_handle = self.dummy_job
        return out

    def write(self, indices, values, name=None, additive=False):
        if additive:
            self.embed.index_add_(0, indices, values)
        else:
            self.embed.index_copy_(0, indices, values)
        return self.dummy_job


def reference_embedding_optimizers(model, args, gpu_id):
    """The reference's own row-wise optimizers for the model's sparse embeddings
    (train_process.py:290-293).
    gpu_id == -1: tables and state in host memory through MemoryRW.
    gpu_id >= 0:  the reference keeps optimizer state on the GPU only when it is shared through the
                  embedding module (--share_optim_stats: main_train.py:165-166 registers the state as
                  buffers, which then move to the device with the module); that route is taken here."""
    from smore.common.embedding import embed_optimizer as eo
    cls = eo.get_optim_class(args)
    embeds = list(model.named_sparse_embeddings())
    if gpu_id == -1:
        eo.EmbeddingRW = MemoryRW
    else:
        args.share_optim_stats = True
        cls.prepare_optimizers(args, [e for _, e in embeds])
        for _, e in embeds:
            e.cuda(gpu_id)
    return {name: cls(args, embed, gpu_id) for name, embed in embeds}


def dense_optimizer(model, lr):
    params = [p for _, p in model.named_dense_parameters()]
    return torch.optim.Adam(params, lr=lr)


def one_batch_iterator(pos, neg, queries, structure):
    """What next(train_iterator) yields (online_sampler.py:149-184) for one prepared batch, forever."""
    weight = torch.ones(pos.shape[0])
    while True:
        yield pos, neg, None, weight, queries, [STRUCTURES[structure]]


def batch_iterator(batches):
    """batches: iterable of (structure name, pos, neg, queries)."""
    for s, pos, neg, q in batches:
        yield pos, neg, None, torch.ones(pos.shape[0]), q, [STRUCTURES[s]]
