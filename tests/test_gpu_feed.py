"""BatchFeeder: pinned, double-buffered, asynchronous host -> device hand-off of sampled batches."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_feeder_delivers_batches_in_order_and_reuses_staging():
    from smore_b200.feed import BatchFeeder
    feeder = BatchFeeder("cuda:0", depth=2)
    g = torch.Generator().manual_seed(0)
    batches = [(torch.randint(0, 1000, (64,), generator=g), torch.randint(0, 1000, (64, 128), generator=g),
                torch.rand(64, 128, generator=g), torch.rand(64, generator=g),
                torch.randint(0, 50, (64, 3), generator=g)) for _ in range(7)]
    feeder.submit(0, *batches[0])
    for i in range(len(batches)):
        if i + 1 < len(batches):
            feeder.submit(i + 1, *batches[i + 1])        # one batch ahead of the consumer
        assert feeder.peek().tag == i
        got = feeder.get()
        assert got.tag == i
        # consume on the current stream without any host synchronisation in between
        sums = [t.double().sum() for t in got.tensors]
        for s, src, t in zip(sums, batches[i], got.tensors):
            assert t.is_cuda and t.dtype == src.dtype and t.shape == src.shape
            assert abs(s.item() - src.double().sum().item()) < 1e-6 * max(1.0, abs(src.double().sum().item()))
            assert torch.equal(t.cpu(), src)
    assert len(feeder) == 0
    assert all(len(slot) == 5 for slot in feeder._staging)   # five pinned buffers per slot, reused
    with pytest.raises(RuntimeError):
        feeder.get()
    feeder.submit("a", torch.zeros(3))
    feeder.submit("b", torch.zeros(3))
    with pytest.raises(RuntimeError):
        feeder.submit("c", torch.zeros(3))
    with pytest.raises(TypeError):
        BatchFeeder("cuda:0").submit("x", torch.zeros(3, device="cuda"))
