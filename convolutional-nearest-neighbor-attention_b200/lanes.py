"""Several batches in flight on one GPU.

The forward of the ConvNN ViT is a chain of ~64 kernels, most of them persistent (one CTA per SM) and
each ending with a tail in which the SMs that have finished their share wait for the last ones: the
MLP kernel's 197 row tiles on 74 CTA pairs leave a third of the pairs idle for the last third of the
kernel, the output projection's 394 tiles on 148 CTAs likewise, and between two kernels of a chain the
GPU is empty for a launch latency.  A second batch that runs the same chain beside the first fills
those gaps with its own kernels' CTAs.  Measured on a B200, ViT-Tiny ConvNN-Attention, 256 images per
batch: 1.61 ms per batch one after another, 1.41-1.43 ms with two forwards as the two branches of ONE
CUDA graph.  (Two graphs replayed on two streams gave 1.52 ms in some runs and 1.62 ms in others: how
the two chains interleave then depends on the phase they happen to fall into; branches of one graph
start together at every replay.)  The reference runs one batch at a time (main.py's evaluation loop);
the results per batch are the same bits either way.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch


class ForwardLanes:
    """CUDA graphs of ``model``'s forward over fixed input buffers, ``lanes`` forwards per graph.

    Consecutive input buffers form a group (buffers g * lanes ... g * lanes + lanes - 1); one graph
    holds the forwards of a group as parallel branches, so a replay runs them side by side.  All graphs
    share one memory pool (they are replayed one after another on one stream).  Usage::

        fl = ForwardLanes(model, [buf0, buf1, buf2, buf3], lanes=2)     # groups (0, 1) and (2, 3)
        for i in range(n):
            g = i % fl.n_groups
            outs = fl.replay(g)                # logits of the group's buffers, on the current stream
            for y in outs: consume(y)          # stream-ordered after the replay
    """

    def __init__(self, model, inputs: Sequence[torch.Tensor], lanes: int = 2, warmup: int = 2):
        if not inputs or not all(x.is_cuda for x in inputs):
            raise ValueError("ForwardLanes needs CUDA input buffers")
        self.lanes = max(1, min(int(lanes), len(inputs)))
        dev = inputs[0].device
        self.groups: List[List[int]] = [list(range(g, min(g + self.lanes, len(inputs))))
                                        for g in range(0, len(inputs), self.lanes)]
        self.n_groups = len(self.groups)
        self.outputs: List[Optional[torch.Tensor]] = [None] * len(inputs)
        self.graphs: List[torch.cuda.CUDAGraph] = []
        self.done = [torch.cuda.Event() for _ in self.groups]
        side = [torch.cuda.Stream(dev) for _ in range(self.lanes - 1)]
        with torch.no_grad():
            for x in inputs[: self.lanes]:
                for _ in range(warmup):
                    model(x)
            torch.cuda.synchronize(dev)
            pool = None
            for group in self.groups:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, pool=pool):
                    cur = torch.cuda.current_stream()
                    for st in side[: len(group) - 1]:
                        st.wait_stream(cur)                # the branches start together
                    self.outputs[group[0]] = model(inputs[group[0]])
                    for st, k in zip(side, group[1:]):
                        with torch.cuda.stream(st):
                            self.outputs[k] = model(inputs[k])
                    for st in side[: len(group) - 1]:
                        cur.wait_stream(st)
                pool = pool or g.pool()
                self.graphs.append(g)
        torch.cuda.synchronize(dev)

    def replay(self, g: int, after: Sequence[torch.cuda.Event] = ()) -> List[torch.Tensor]:
        """Enqueue the forwards of group ``g`` on the current stream (behind the events ``after``, e.g.
        the copies that fill its buffers); ``self.done[g]`` is recorded behind them.  Returns the
        static outputs of the group's buffers."""
        cur = torch.cuda.current_stream()
        for e in after:
            cur.wait_event(e)
        self.graphs[g].replay()
        self.done[g].record(cur)
        return [self.outputs[k] for k in self.groups[g]]
