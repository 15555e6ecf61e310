"""CUDA-graph replay of an inference forward pass.

The layers of this path are short kernels (tens of microseconds each at the bandwidths the
reference's models use), so a forward pass launched op by op from Python is partly launch-bound.
``GraphedForward`` captures one forward pass of any module built from this package's ops (plus
ordinary torch ops) into a CUDA graph and replays it on new inputs of the same shape.

All constant tables are built during the warm-up passes that precede the capture, so nothing inside
the captured region allocates through the library.
"""
import torch


class GraphedForward:
    def __init__(self, module, example_input, warmup=3):
        assert example_input.is_cuda, "GraphedForward needs a CUDA example input"
        self.module = module
        self.static_in = example_input.clone()
        side = torch.cuda.Stream(device=example_input.device)
        side.wait_stream(torch.cuda.current_stream(example_input.device))
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(warmup):  # builds tables, sizes the allocator pools
                module(self.static_in)
        torch.cuda.current_stream(example_input.device).wait_stream(side)
        torch.cuda.synchronize(example_input.device)
        self.graph = torch.cuda.CUDAGraph()
        with torch.no_grad(), torch.cuda.graph(self.graph):
            self.static_out = module(self.static_in)

    def __call__(self, x):
        """Copies ``x`` (device or pinned host tensor of the captured shape) into the graph's input
        buffer, replays the forward pass and returns the graph's output buffer (overwritten by the
        next call)."""
        self.static_in.copy_(x, non_blocking=True)
        self.graph.replay()
        return self.static_out


class InterleavedForward:
    """Throughput mode for resident inputs: ``lanes`` captured copies of the forward pass replay on
    their own streams, successive batches going to successive lanes.  The kernels of one pass depend
    on each other and each ends with a partly filled last wave of blocks; with two passes in flight
    the blocks of one fill the SMs the other leaves idle.

        fwd = InterleavedForward(net, example_device_batch)
        fwd.fork()                          # lanes start after the work already on this stream
        for x in batches:
            lane = fwd.submit(x)            # fwd.output(lane) is valid after fwd.join() (or after
        fwd.join()                          # the lane's next-but-one submit has not yet happened)
    """

    def __init__(self, module, example_input, lanes=2):
        assert lanes >= 1
        dev = example_input.device
        self.device = dev
        self.slots = [GraphedForward(module, example_input) for _ in range(lanes)]
        self.streams = [torch.cuda.Stream(device=dev) for _ in range(lanes)]
        self.done = [torch.cuda.Event() for _ in range(lanes)]
        self.n = 0

    def fork(self):
        cur = torch.cuda.current_stream(self.device)
        for st in self.streams:
            st.wait_stream(cur)

    def submit(self, x):
        lane = self.n % len(self.slots)
        with torch.cuda.stream(self.streams[lane]):
            self.slots[lane](x)
            self.done[lane].record(self.streams[lane])
        self.n += 1
        return lane

    def output(self, lane):
        return self.slots[lane].static_out

    def join(self):
        cur = torch.cuda.current_stream(self.device)
        for ev in self.done:
            cur.wait_event(ev)


class PipelinedForward:
    """Inference on batches that arrive in pinned host memory, with the host-to-device copy of the
    next batch overlapped with the forward pass of the current one.

    Two captured copies of the forward pass (``GraphedForward``) alternate, each on its own compute
    stream (so the tail of one pass overlaps the head of the next); a copy stream uploads batch
    i + 1 into the idle copy's input buffer while batch i runs; another stream returns each result
    to pinned host memory, so that the small device-to-host copy does not sit between two replays.  ``submit`` never
    blocks the host; ``wait`` blocks until everything submitted so far has reached the host.

        pipe = PipelinedForward(net, example_device_batch)
        for x_host, y_host in zip(batches, results):      # pinned tensors
            pipe.submit(x_host, y_host)
        pipe.wait()
    """

    def __init__(self, module, example_input, depth=2):
        assert depth >= 2
        dev = example_input.device
        self.device = dev
        self.slots = [GraphedForward(module, example_input) for _ in range(depth)]
        self.copy_stream = torch.cuda.Stream(device=dev)
        self.read_stream = torch.cuda.Stream(device=dev)
        self.compute = [torch.cuda.Stream(device=dev) for _ in range(depth)]   # one per slot
        self.uploaded = [torch.cuda.Event() for _ in range(depth)]
        self.consumed = [torch.cuda.Event() for _ in range(depth)]   # slot's input buffer is free again
        self.returned = [torch.cuda.Event() for _ in range(depth)]   # slot's result has reached the host
        self.n_uploaded = 0
        self.n_run = 0

    def prefetch(self, x_host):
        """Start the upload of the next batch (pinned host tensor) on the copy stream."""
        slot = self.n_uploaded % len(self.slots)
        if self.n_uploaded >= len(self.slots):
            self.copy_stream.wait_event(self.consumed[slot])
        with torch.cuda.stream(self.copy_stream):
            self.slots[slot].static_in.copy_(x_host, non_blocking=True)
            self.uploaded[slot].record(self.copy_stream)
        self.n_uploaded += 1

    def join_uploads(self):
        """Make the current stream wait for the most recent upload (so that an event recorded next
        on the current stream also covers that upload)."""
        if self.n_uploaded:
            slot = (self.n_uploaded - 1) % len(self.slots)
            torch.cuda.current_stream(self.device).wait_event(self.uploaded[slot])

    def join_results(self):
        """Make the current stream wait for the most recent read-back (so that an event recorded
        next on the current stream also covers every result copied so far)."""
        if self.n_run:
            slot = (self.n_run - 1) % len(self.slots)
            torch.cuda.current_stream(self.device).wait_event(self.returned[slot])

    def run(self, y_host):
        """Forward pass on the oldest uploaded batch; the result is copied into ``y_host`` (pinned)
        asynchronously on the read-back stream."""
        assert self.n_run < self.n_uploaded, "run() without a prefetched batch"
        slot = self.n_run % len(self.slots)
        st = self.compute[slot]      # the slots replay on their own streams: two passes in flight
        st.wait_stream(torch.cuda.current_stream(self.device))
        st.wait_event(self.uploaded[slot])
        if self.n_run >= len(self.slots):
            st.wait_event(self.returned[slot])     # the slot's previous result has left its buffer
        g = self.slots[slot]
        with torch.cuda.stream(st):
            g.graph.replay()
            self.consumed[slot].record(st)
        self.read_stream.wait_event(self.consumed[slot])
        with torch.cuda.stream(self.read_stream):
            y_host.copy_(g.static_out, non_blocking=True)
            self.returned[slot].record(self.read_stream)
        self.n_run += 1

    def submit(self, x_host, y_host):
        """Upload ``x_host`` and run every batch that is ready but one, so that one upload is always
        in flight behind the forward pass; call ``flush`` for the results of the last batch."""
        self.prefetch(x_host)
        self._pending = getattr(self, "_pending", [])
        self._pending.append(y_host)
        while len(self._pending) > 1:
            self.run(self._pending.pop(0))

    def flush(self):
        for y in getattr(self, "_pending", []):
            self.run(y)
        self._pending = []

    def wait(self):
        self.flush()
        torch.cuda.synchronize(self.device)
