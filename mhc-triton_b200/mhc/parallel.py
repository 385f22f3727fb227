"""Data parallelism over the batch axis for stacks of HyperConnection layers.

The mixing weights of a batch element depend only on that element's own sequence, so whole
sequences are sharded across ranks with no communication in the forward pass and none for any
activation gradient.  The only exchange is one SUM all-reduce of the replicated-parameter
gradients (phi, the 24 base/bias entries, the three scales) per step.  `GradSync` makes the
backward kernels write those gradients straight into one flat fp32 buffer, which is the
all-reduce operand (no pack or copy kernels), and starts the collective of each layer on a
side stream as soon as that layer's weight gradients are launched, so it overlaps the pass
that writes dH and the rest of the backward.

The reference project has no distributed code; SUM (not mean) keeps the result equal to the
single-device gradient, which is a sum over batch elements (src/mhc/ops.py:187-194,213 there).
"""

from typing import Iterable, List, Optional

import torch
import torch.distributed as dist


def shard_batch(t: torch.Tensor, rank: int, world_size: int) -> torch.Tensor:
    """Contiguous slice of whole batch elements owned by `rank` (sizes differ by at most one)."""
    B = t.shape[0]
    base, rem = divmod(B, world_size)
    lo = rank * base + min(rank, rem)
    hi = lo + base + (1 if rank < rem else 0)
    return t[lo:hi]


def sink_numel(dim: int) -> int:
    """Elements of one layer's flat gradient record: phi [4*dim, 24], bias [24], alpha [3]."""
    return 4 * dim * 24 + 27


class GradSync:
    """Owns the flat gradient buffer of a list of fused-dynamic HyperConnection layers.

    After construction every parameter's .grad is a view into `self.flat`; a backward pass
    overwrites the record of each layer (or adds to it when `accumulate` is set), and
    `finish()` makes the current stream wait for the all-reduces.  Typical step:

        sync = GradSync(layers)            # once
        loss.backward()                    # all-reduces start inside the backward
        sync.finish()                      # before the optimizer reads .grad
    """

    def __init__(self, layers: Iterable[torch.nn.Module], process_group=None, overlap: bool = True):
        self.layers: List[torch.nn.Module] = list(layers)
        if not self.layers:
            raise ValueError("GradSync needs at least one layer")
        self.group = process_group
        sizes = []
        for l in self.layers:
            if not getattr(l, "use_fused_weights", False):
                raise ValueError("GradSync supports fused dynamic HyperConnection layers only")
        dev = self.layers[0].phi.device
        for l in self.layers:
            for p in l.parameters():
                if p.dtype != torch.float32 or p.device != dev:
                    raise ValueError("GradSync needs fp32 parameters on one device")
            sizes.append(sink_numel(l.dim))
        self.flat = torch.zeros(sum(sizes), device=dev, dtype=torch.float32)
        self.records = []
        off = 0
        for l, n in zip(self.layers, sizes):
            rec = self.flat[off:off + n]
            off += n
            K24 = 4 * l.dim * 24
            l.grad_sink = rec
            l.grads_ready_hook = self._on_layer_ready
            l.phi.grad = rec[:K24].view(4 * l.dim, 24)
            l.H_pre_base.grad = rec[K24:K24 + 4]
            l.H_post_base.grad = rec[K24 + 4:K24 + 8]
            l.H_res_base.grad = rec[K24 + 8:K24 + 24].view(4, 4)
            l.alpha_pre.grad = rec[K24 + 24:K24 + 25]
            l.alpha_post.grad = rec[K24 + 25:K24 + 26]
            l.alpha_res.grad = rec[K24 + 26:K24 + 27]
            self.records.append(rec)
        self.overlap = overlap and dev.type == "cuda"
        self.side = torch.cuda.Stream(device=dev) if self.overlap else None
        self._pending = []

    # -- called from the backward of a layer, right after its weight-gradient kernels were launched
    def _on_layer_ready(self, rec: torch.Tensor) -> None:
        if not self._distributed():
            return
        if self.overlap:
            ev = torch.cuda.Event()
            ev.record()
            self.side.wait_event(ev)
            with torch.cuda.stream(self.side):
                dist.all_reduce(rec, op=dist.ReduceOp.SUM, group=self.group)
                done = torch.cuda.Event()
                done.record()
            self._pending.append(done)
        else:
            dist.all_reduce(rec, op=dist.ReduceOp.SUM, group=self.group)

    def _distributed(self) -> bool:
        return dist.is_available() and dist.is_initialized() and dist.get_world_size(self.group) > 1

    def finish(self) -> None:
        """Order everything after the collectives started during the backward."""
        for ev in self._pending:
            torch.cuda.current_stream().wait_event(ev)
        self._pending.clear()

    def all_reduce_now(self) -> None:
        """One collective over the whole flat buffer (for callers that do not use the hooks)."""
        if self._distributed():
            dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, group=self.group)

    def zero(self) -> None:
        self.flat.zero_()
