"""Hand-off of sampled batches from the host sampler to the GPU step.

The reference's sampler thread produces, per step, CPU tensors (online_sampler.py:149-184):
`positive_sample int64 [B]`, `negative_sample int64 [B, K]` (or `[1, K]` shared), `is_negative
float [B, K]`, `subsampling_weight float [B]`, `query args int64 [B, n_args]`, and train_step_mp
moves them to the device one by one, synchronously, at the start of the step
(train_process.py:179-190).  `BatchFeeder` does that move ahead of time: batches are copied into
pinned staging buffers (two sets, reused) and from there to the device on a copy stream while the
previous step computes; `get()` makes the consuming stream wait for the copy, not the host.
"""
import collections

import torch

Batch = collections.namedtuple("Batch", "tensors event tag")


class BatchFeeder(object):
    """feeder.submit(tag, *cpu_tensors) queues a batch; feeder.get() returns the oldest queued batch
    as device tensors, ready on the current stream.  At most `depth` batches are in flight; their
    pinned staging buffers are reused in rotation, so submit() blocks the host only when it runs
    `depth` batches ahead of the consumer."""

    def __init__(self, device, depth=2):
        self.device = torch.device(device)
        self.depth = int(depth)
        self.stream = torch.cuda.Stream(self.device)
        self._staging = [dict() for _ in range(self.depth)]   # slot -> {(position, shape, dtype): pinned tensor}
        self._copied = [None] * self.depth                     # event: the slot's last H2D copies are done
        self._queue = collections.deque()
        self._n = 0

    def _pinned(self, slot, pos, t):
        key = (pos, tuple(t.shape), t.dtype)
        buf = self._staging[slot].get(key)
        if buf is None:
            buf = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
            self._staging[slot][key] = buf
        return buf

    def submit(self, tag, *cpu_tensors):
        if len(self._queue) >= self.depth:
            raise RuntimeError("BatchFeeder: %d batches already in flight; call get() first" % self.depth)
        slot = self._n % self.depth
        self._n += 1
        if self._copied[slot] is not None:
            self._copied[slot].synchronize()      # the staging buffers of this slot are free again
        staged = []
        for pos, t in enumerate(cpu_tensors):
            if t.is_cuda:
                raise TypeError("BatchFeeder.submit takes host tensors")
            buf = self._pinned(slot, pos, t)
            buf.copy_(t)
            staged.append(buf)
        with torch.cuda.stream(self.stream):
            dev = [b.to(self.device, non_blocking=True) for b in staged]
            event = torch.cuda.Event()
            event.record(self.stream)
        self._copied[slot] = event
        self._queue.append(Batch(dev, event, tag))

    def get(self):
        if not self._queue:
            raise RuntimeError("BatchFeeder: nothing queued")
        batch = self._queue.popleft()
        consumer = torch.cuda.current_stream(self.device)
        consumer.wait_event(batch.event)
        for t in batch.tensors:
            t.record_stream(consumer)
        return batch

    def peek(self):
        """The oldest queued batch without consuming it (e.g. to hand its id tensors to
        ShardedAdamOptimizer.prefetch together with `batch.event`)."""
        return self._queue[0] if self._queue else None

    def __len__(self):
        return len(self._queue)
