"""Batch data parallelism for the spectral path: one process per GPU, each rank owns a slice of
the batch.  Forward needs no communication; a training step reduces the parameter gradients once.

The reference has no distributed code at all (no NCCL/MPI/DataParallel anywhere in its sources);
this is the minimal layer the path needs on an 8-GPU NVSwitch box:

* ``shard_range``           - which batch elements a rank owns;
* ``allreduce_gradients``   - one blocking all-reduce of all gradients after ``backward()``;
* ``GradientReducer``       - the same sum, but launched bucket by bucket (one bucket per layer)
                              from autograd hooks while the rest of the backward pass still runs;
* ``max_over_ranks``        - reduction used for device-time reporting.

The real-space ``kernel.grad`` ([f_in, f_out, n_grid]) is what gets reduced, not the ~14x larger
spectral gradient: the kernel transform is linear, so the two orders commute.
"""
import datetime

import torch
import torch.distributed as dist


def shard_range(n, rank, world):
    """Contiguous [start, stop) of `n` batch elements owned by `rank`; sizes differ by at most 1,
    every element is owned exactly once, empty ranges are allowed when world > n."""
    if not (0 <= rank < world):
        raise ValueError("rank %d outside world of %d" % (rank, world))
    base, rem = divmod(n, world)
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


def _active():
    return dist.is_available() and dist.is_initialized()


def _trainable(params):
    ps = [p for p in params if p.requires_grad]
    if ps:
        dt, dev = ps[0].dtype, ps[0].device
        for p in ps:
            if p.dtype != dt or p.device != dev:
                raise TypeError("gradient bucket needs one dtype and one device, got %s/%s and %s/%s"
                                % (dt, dev, p.dtype, p.device))
    return ps


def allreduce_gradients(params, average=False, group=None):
    """Sum (or average) ``.grad`` of the given parameters over all ranks with ONE all-reduce of a
    flat bucket (the gradients of this path are a few MB, so latency, not bandwidth, decides).

    The bucket layout is the same on every rank whatever happened locally: every parameter with
    ``requires_grad`` takes part, and one whose ``.grad`` is still None on this rank (an empty batch
    shard, an unused or skipped branch) contributes zeros and receives the reduced value - so ranks
    can never disagree on the element count of the collective.  Returns the number of elements
    reduced; a no-op returning 0 when torch.distributed is not initialised."""
    if not _active():
        return 0
    ps = _trainable(params)
    if not ps:
        return 0
    flat = torch.cat([(p.grad if p.grad is not None else torch.zeros_like(p)).reshape(-1)
                      for p in ps])
    dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
    if average:
        flat /= dist.get_world_size(group)
    off = 0
    for p in ps:
        n = p.numel()
        piece = flat[off:off + n].view_as(p)
        if p.grad is None:
            p.grad = piece.clone()
        else:
            p.grad.copy_(piece)
        off += n
    return flat.numel()


class GradientReducer:
    """Gradient all-reduce overlapped with the backward pass.

    The parameters are grouped into buckets - by default one per module that owns parameters, in
    registration order, i.e. one per layer.  Each bucket owns a flat buffer and the parameters'
    ``.grad`` are views into it, so nothing is copied before or after the collective.  A
    post-accumulate hook on every parameter marks it ready; as soon as a whole bucket is ready its
    all-reduce is launched asynchronously (NCCL runs it on its own stream, ordered after the
    kernels that produced the gradients) while autograd continues with the earlier layers.
    ``finish()`` launches whatever has not been launched (parameters that received no gradient on
    this rank contribute the zeros their views hold), waits, and averages if asked to.

    Collectives must be issued in the same order on every rank, whatever order the hooks fire in
    and even on a rank that ran no backward at all: buckets are therefore launched strictly from
    the last one to the first, a bucket waiting for its successors.

    Usage per step:  ``reducer.zero_grad(); loss.backward(); reducer.finish()``.
    Without an initialised process group the hooks do nothing and ``finish()`` returns 0."""

    def __init__(self, module, average=False, group=None, buckets=None):
        self.average = average
        self.group = group
        if buckets is None:
            buckets = []
            for m in module.modules():
                own = [p for p in m.parameters(recurse=False) if p.requires_grad]
                if own:
                    buckets.append(own)
        self.buckets = [_trainable(b) for b in buckets if b]
        all_params = [p for b in self.buckets for p in b]
        _trainable(all_params)
        self.flat = [torch.zeros(sum(p.numel() for p in b), dtype=b[0].dtype, device=b[0].device)
                     for b in self.buckets]
        self._where = {}
        self._handles = []
        for bi, b in enumerate(self.buckets):
            for p in b:
                self._where[p] = bi
                self._handles.append(p.register_post_accumulate_grad_hook(self._on_grad))
        self._pending = [0] * len(self.buckets)
        self._next = len(self.buckets) - 1
        self._works = []
        self.suspended = False   # True: hooks launch nothing (a purely local backward pass)
        self.zero_grad()

    def _views(self, bi):
        off = 0
        for p in self.buckets[bi]:
            n = p.numel()
            yield p, self.flat[bi][off:off + n].view_as(p)
            off += n

    def zero_grad(self):
        """Clears the buckets and points every ``.grad`` at its slice (call instead of
        ``module.zero_grad()``, which would detach the gradients from the buckets)."""
        for bi in range(len(self.buckets)):
            self.flat[bi].zero_()
            for p, view in self._views(bi):
                p.grad = view
            self._pending[bi] = len(self.buckets[bi])
        self._next = len(self.buckets) - 1
        self._works = []

    def _launch_ready(self, force=False):
        while self._next >= 0 and (force or self._pending[self._next] == 0):
            bi = self._next
            for p, view in self._views(bi):   # a hook-less step may have replaced .grad
                if p.grad is None:
                    p.grad = view
                elif p.grad.data_ptr() != view.data_ptr():
                    view.copy_(p.grad)
                    p.grad = view
            self._works.append(dist.all_reduce(self.flat[bi], op=dist.ReduceOp.SUM,
                                               group=self.group, async_op=True))
            self._next -= 1

    def _on_grad(self, p):
        if self.suspended or not _active():
            return
        bi = self._where[p]
        self._pending[bi] -= 1
        self._launch_ready()

    def finish(self, timeout_s=None):
        """Launches the remaining buckets, waits for all of them and returns the number of
        elements reduced.  With ``timeout_s`` the host waits at most that long for each bucket and
        raises ``TimeoutError`` if a peer never joined its all-reduce (failure detection on the
        host: nothing on the GPU is made to fault; the process group is unusable afterwards and the
        caller is expected to tear the job down)."""
        if not _active():
            return 0
        self._launch_ready(force=True)
        for i, w in enumerate(self._works):
            if timeout_s is None:
                w.wait()
                continue
            try:
                done = w.wait(datetime.timedelta(seconds=float(timeout_s)))
            except RuntimeError as e:     # gloo and NCCL both raise on an expired wait
                raise TimeoutError("gradient all-reduce %d of %d did not complete within %.1f s: %s"
                                   % (i + 1, len(self._works), timeout_s, e)) from e
            if done is False:
                raise TimeoutError("gradient all-reduce %d of %d did not complete within %.1f s"
                                   % (i + 1, len(self._works), timeout_s))
        self._works = []
        if self.average:
            world = dist.get_world_size(self.group)
            for f in self.flat:
                f /= world
        return sum(f.numel() for f in self.flat)

    def remove(self):
        for h in self._handles:
            h.remove()
        self._handles = []


def max_over_ranks(value, device="cpu", group=None):
    """Max of a python float over ranks (used for device-time reporting)."""
    if not _active():
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
