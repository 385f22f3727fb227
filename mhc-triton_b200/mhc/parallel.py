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
        opt.zero_grad()                    # any form: see below
        loss.backward()                    # all-reduces start inside the backward
        sync.finish()                      # before the optimizer reads .grad
        opt.step()

    `zero_grad(set_to_none=True)` (torch's default) drops the views; the backward of each layer
    and `finish()` bind them again (`attach()`), so the optimizer always finds the freshly written
    record in `.grad`.  `zero_grad(set_to_none=False)` merely zeroes a record the next backward
    overwrites.
    """

    def __init__(self, layers: Iterable[torch.nn.Module], process_group=None, overlap: bool = True,
                 check_ranks: bool = True):
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
        self._views = {}     # record address -> [(parameter, its view of the record)]
        off = 0
        for l, n in zip(self.layers, sizes):
            rec = self.flat[off:off + n]
            off += n
            K24 = 4 * l.dim * 24
            l.grad_sink = rec
            l.grads_ready_hook = self._on_layer_ready
            self._views[rec.data_ptr()] = [
                (l.phi, rec[:K24].view(4 * l.dim, 24)),
                (l.H_pre_base, rec[K24:K24 + 4]),
                (l.H_post_base, rec[K24 + 4:K24 + 8]),
                (l.H_res_base, rec[K24 + 8:K24 + 24].view(4, 4)),
                (l.alpha_pre, rec[K24 + 24:K24 + 25]),
                (l.alpha_post, rec[K24 + 25:K24 + 26]),
                (l.alpha_res, rec[K24 + 26:K24 + 27]),
            ]
            self.records.append(rec)
        self.attach()
        if check_ranks and self._distributed():
            self._check_same_layout(sizes)
        self.overlap = overlap and dev.type == "cuda"
        self.side = torch.cuda.Stream(device=dev) if self.overlap else None
        self._pending = []
        # One event per layer, recorded by the layer's backward between the kernels that complete the
        # record and the pass that writes dH: the collective on the side stream waits for it and so
        # runs beside that pass.  (Recorded once here so that it owns a CUDA event.)
        self._events = {}
        if self.overlap and self._distributed():
            with torch.cuda.device(dev):
                for l, rec in zip(self.layers, self.records):
                    ev = torch.cuda.Event()
                    ev.record()
                    self._events[rec.data_ptr()] = ev
                    l.grads_ready_event = ev

    def attach(self, rec: Optional[torch.Tensor] = None) -> None:
        """Make .grad of every parameter (of the layer owning `rec`, or of all layers) the view of the
        flat record again.  Needed after anything that replaced or dropped .grad, e.g.
        `optimizer.zero_grad()` with set_to_none=True; the backward and `finish()` call it."""
        groups = self._views.values() if rec is None else (self._views[rec.data_ptr()],)
        for views in groups:
            for p, v in views:
                if p.grad is not v:
                    p.grad = v

    # -- called from the backward of a layer, right after its weight-gradient kernels were launched
    def _on_layer_ready(self, rec: torch.Tensor) -> None:
        self.attach(rec)
        if not self._distributed():
            return
        if self.overlap:
            ev = self._events.get(rec.data_ptr())
            if ev is None:       # no event of the layer's own: order after everything launched so far
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

    def _check_same_layout(self, sizes) -> None:
        """Every rank must reduce records of the same sizes in the same order; a mismatch (different
        layer count or width on some rank) would otherwise corrupt gradients or hang the collective.
        All ranks learn of it here, on the host, and all raise."""
        world = dist.get_world_size(self.group)
        seen = [None] * world
        dist.all_gather_object(seen, list(sizes), group=self.group)
        if any(s != seen[0] for s in seen):
            raise ValueError(f"GradSync: ranks disagree on the gradient record layout: {seen}")

    def _distributed(self) -> bool:
        return dist.is_available() and dist.is_initialized() and dist.get_world_size(self.group) > 1

    def finish(self) -> None:
        """Order everything after the collectives started during the backward, and make sure the
        parameters' .grad are the views of the record."""
        self.attach()
        for ev in self._pending:
            torch.cuda.current_stream().wait_event(ev)
        self._pending.clear()

    def all_reduce_now(self) -> None:
        """One collective over the whole flat buffer (for callers that do not use the hooks)."""
        if self._distributed():
            dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, group=self.group)

    def all_reduce_async(self) -> None:
        """One collective over the whole flat buffer on the side stream, after everything launched so
        far on the current stream; `finish()` (or `wait_reduced()`) orders later work after it.  For
        steps replayed from CUDA graphs, which keep collectives out of the graph: replay, call this,
        and wait only where the reduced gradients are used or the record is written again."""
        if not self._distributed():
            return
        if not self.overlap:
            return self.all_reduce_now()
        ev = torch.cuda.Event()
        ev.record()
        self.side.wait_event(ev)
        with torch.cuda.stream(self.side):
            dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, group=self.group)
            done = torch.cuda.Event()
            done.record()
        self._pending.append(done)

    def wait_reduced(self) -> None:
        """Make the current stream wait for the collectives started so far (no re-binding of .grad)."""
        for ev in self._pending:
            torch.cuda.current_stream().wait_event(ev)
        self._pending.clear()

    def set_hooks(self, enabled: bool) -> None:
        """Enable or disable the in-backward start of the collectives (disable while capturing the
        step into a CUDA graph: collectives stay outside the graph, see all_reduce_async)."""
        for l, rec in zip(self.layers, self.records):
            l.grads_ready_hook = self._on_layer_ready if enabled else None
            l.grads_ready_event = self._events.get(rec.data_ptr()) if enabled else None

    def zero(self) -> None:
        self.flat.zero_()


# ---------------------------------------------------------------------------------------------
# Sequence sharding: every rank holds a slice [B, S_local, 4, D] of every sequence.  The mixing
# weights depend on the mean over the WHOLE sequence, so the forward needs one small all-reduce
# (the pooled state, [B, 4*D] fp32) and the backward one more (the 24 weight gradients per batch
# element, [B, 24] fp32).  Activations never move.  Parameter gradients come out complete and
# identical on every rank of the sequence group: do not sum them over that group again.
# ---------------------------------------------------------------------------------------------
class _SequenceShardedMix(torch.autograd.Function):
    @staticmethod
    def forward(ctx, H, H_pre_base, H_post_base, H_res_base, phi, alpha_pre, alpha_post, alpha_res, sinkhorn_iters,
                eps, group, total_len):
        from ._kernels import fused_dynamic_weights_forward, meanpool_forward, stream_mix_forward
        S_local = H.shape[1]
        x = meanpool_forward(H) * (S_local / total_len)
        if _group_size(group) > 1:
            dist.all_reduce(x, op=dist.ReduceOp.SUM, group=group)
        bias = torch.cat([H_pre_base.reshape(-1), H_post_base.reshape(-1), H_res_base.reshape(-1)]).float()
        H_pre, H_post, H_res, saved = fused_dynamic_weights_forward(
            x, phi, bias, alpha_pre, alpha_post, alpha_res, sinkhorn_iters, eps, return_saved=True)
        # the residual mix is not written: the closure recomputes it from H (see ops.add_residual_from_state)
        branch_input, _ = stream_mix_forward(H, H_pre, H_res, want_residual=False)
        H_residual = branch_input.new_empty(1).expand(H.shape)   # storage-less carrier of the residual's gradient
        ctx.save_for_backward(H, x, phi, bias, alpha_pre, alpha_post, alpha_res, saved, H_pre, H_res)
        ctx.meta = (sinkhorn_iters, eps, group, total_len, H_pre_base.shape, H_post_base.shape, H_res_base.shape)
        ctx.mark_non_differentiable(H_pre, H_res)
        ctx.set_materialize_grads(False)
        return branch_input, H_residual, H_post, H_pre, H_res

    @staticmethod
    def backward(ctx, d_bi, dHr, dH_post, _a, _b):
        from ._backward import (fused_dynamic_weights_backward, stream_mix_backward_apply,
                                stream_mix_backward_reduce)
        H, x, phi, bias, alpha_pre, alpha_post, alpha_res, saved, H_pre, H_res = ctx.saved_tensors
        iters, eps, group, total_len, s_pre, s_post, s_res = ctx.meta
        B, S, _, D = H.shape
        if d_bi is None:
            d_bi = torch.zeros(B, S, D, device=H.device, dtype=H.dtype)
        if dHr is None:
            dHr = torch.zeros_like(H)
        if dH_post is None:
            dH_post = torch.zeros(B, 4, device=H.device)
        dH_pre, dH_res = stream_mix_backward_reduce(d_bi, dHr, H)
        packed = torch.cat([dH_pre, dH_post.float(), dH_res.reshape(B, 16)], dim=1).contiguous()
        if _group_size(group) > 1:
            dist.all_reduce(packed, op=dist.ReduceOp.SUM, group=group)
        gx, gphi, gbias, galpha = fused_dynamic_weights_backward(
            x, phi, bias, alpha_pre, alpha_post, alpha_res, saved, packed[:, 0:4], packed[:, 4:8],
            packed[:, 8:24].reshape(B, 4, 4), iters, eps)
        dH = stream_mix_backward_apply(d_bi, dHr, H_pre, H_res, gx, H, inv_S=1.0 / total_len)
        return (dH, gbias[0:4].reshape(s_pre), gbias[4:8].reshape(s_post), gbias[8:24].reshape(s_res),
                gphi.to(phi.dtype), galpha[0:1].reshape_as(alpha_pre), galpha[1:2].reshape_as(alpha_post),
                galpha[2:3].reshape_as(alpha_res), None, None, None, None)


def _group_size(group) -> int:
    if not (dist.is_available() and dist.is_initialized()):
        return 1
    return dist.get_world_size(group)


class SequenceShardedHyperConnection(torch.nn.Module):
    """Wraps a fused dynamic HyperConnection for inputs sharded along the sequence axis.

    forward(H_local) takes this rank's [B, S_local, 4, D] slice and returns
    (branch_input_local, add_residual) exactly like the wrapped layer; `total_len` is the global
    sequence length (default: S_local times the group size).  Use it when the batch is smaller
    than the number of GPUs or one sequence does not fit one GPU.
    """

    def __init__(self, layer: torch.nn.Module, process_group=None, total_len: Optional[int] = None):
        super().__init__()
        if not getattr(layer, "use_fused_weights", False):
            raise ValueError("sequence sharding supports fused dynamic HyperConnection layers only")
        self.layer, self.group, self.total_len = layer, process_group, total_len

    def forward(self, H: torch.Tensor):
        from .ops import add_residual_from_state
        l = self.layer
        total = self.total_len if self.total_len is not None else H.shape[1] * _group_size(self.group)
        branch_input, stand_in, H_post, _, H_res = _SequenceShardedMix.apply(
            H, l.H_pre_base, l.H_post_base, l.H_res_base, l.phi, l.alpha_pre, l.alpha_post, l.alpha_res,
            l.sinkhorn_iters, l.eps, self.group, total)

        def add_residual(branch_output: torch.Tensor) -> torch.Tensor:
            return add_residual_from_state(stand_in, H, H_res, branch_output, H_post)

        return branch_input, add_residual
