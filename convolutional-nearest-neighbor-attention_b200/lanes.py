"""Several batches in flight on one GPU.

The forward of the ConvNN ViT is a chain of ~64 kernels, most of them persistent (one CTA per SM) and
each ending with a tail in which the SMs that have finished their share wait for the last ones: the
MLP kernel's 197 row tiles on 74 CTA pairs leave a third of the pairs idle for the last third of the
kernel, the output projection's 394 tiles on 148 CTAs likewise.  A second batch that runs the same
chain on another stream fills those tails with its own kernels' CTAs.  Measured on a B200, ViT-Tiny
ConvNN-Attention, 256 images per batch: 1.61 ms per batch with one batch in flight, 1.52 ms with two
(three or four: 1.53 ms).  The reference runs one batch at a time (main.py's evaluation loop); the
results per batch are the same bits either way.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch


class ForwardLanes:
    """CUDA graphs of ``model``'s forward over fixed input buffers, replayed on ``lanes`` streams.

    Input buffer k belongs to lane ``k % lanes``.  The graphs of one lane share a memory pool (their
    intermediates occupy the same addresses and stay in L2 from one replay to the next); lanes have
    pools of their own, because their replays overlap in time.  Usage::

        fl = ForwardLanes(model, [buf0, buf1, buf2, buf3], lanes=2)
        fl.fork()                              # the lanes start after what the current stream holds
        for i in range(n):
            k = i % 4
            with fl.lane(k):                   # current stream := the lane of buffer k
                fl.replay(k)                   # logits of buffer k -> fl.outputs[k]
                consume(fl.outputs[k])         # stream-ordered after the replay
        fl.join()                              # the current stream waits for every lane
    """

    def __init__(self, model, inputs: Sequence[torch.Tensor], lanes: int = 2, warmup: int = 2):
        if not inputs or not all(x.is_cuda for x in inputs):
            raise ValueError("ForwardLanes needs CUDA input buffers")
        self.lanes = max(1, min(int(lanes), len(inputs)))
        dev = inputs[0].device
        self.streams = [torch.cuda.Stream(dev) for _ in range(self.lanes)]
        self.graphs: List[Optional[torch.cuda.CUDAGraph]] = [None] * len(inputs)
        self.outputs: List[Optional[torch.Tensor]] = [None] * len(inputs)
        self.done = [torch.cuda.Event() for _ in inputs]
        with torch.no_grad():
            for x in inputs[: self.lanes]:
                for _ in range(warmup):
                    model(x)
            torch.cuda.synchronize(dev)
            for lane in range(self.lanes):
                pool = None
                for k in range(lane, len(inputs), self.lanes):
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, pool=pool):
                        y = model(inputs[k])
                    pool = pool or g.pool()
                    self.graphs[k], self.outputs[k] = g, y
        torch.cuda.synchronize(dev)

    def stream_of(self, k: int) -> torch.cuda.Stream:
        return self.streams[k % self.lanes]

    def lane(self, k: int):
        """Context manager: the lane stream of input buffer ``k`` becomes the current stream."""
        return torch.cuda.stream(self.stream_of(k))

    def replay(self, k: int, after: Optional[torch.cuda.Event] = None) -> torch.Tensor:
        """Enqueue the forward of input buffer ``k`` on its lane (behind ``after``, e.g. the copy that
        fills the buffer); ``self.done[k]`` is recorded behind it.  Returns the static output."""
        st = self.stream_of(k)
        if after is not None:
            st.wait_event(after)
        with torch.cuda.stream(st):
            self.graphs[k].replay()
            self.done[k].record(st)
        return self.outputs[k]

    def fork(self):
        cur = torch.cuda.current_stream()
        for st in self.streams:
            st.wait_stream(cur)

    def join(self):
        cur = torch.cuda.current_stream()
        for st in self.streams:
            cur.wait_stream(st)
