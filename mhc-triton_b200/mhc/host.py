"""One layer step for activations that live in (pinned) host memory.

`HostStreamedStep` runs HyperConnection forward + backward for a batch whose hyper-hidden state
and upstream gradient sit in host buffers and whose results (H_new, dH, parameter gradients) go
back to host buffers.  Batch elements are independent in this layer, so the batch is cut into
groups of whole sequences and three CUDA streams overlap the host-to-device copy of group i+1, the
kernels of group i and the device-to-host copy of group i-1 (PCIe is full duplex).  Parameter
gradients accumulate across groups in the layer's flat gradient record.
"""

from typing import Callable, Optional

import torch

from .parallel import GradSync


class HostStreamedStep:
    def __init__(self, layer, sync: Optional[GradSync] = None, group: int = 1, slots: int = 3,
                 branch: Optional[Callable[[torch.Tensor], torch.Tensor]] = None):
        """layer: a fused dynamic HyperConnection on a CUDA device; sync: its GradSync (created if
        missing); group: batch elements per pipeline stage; slots: staging buffers in flight."""
        self.layer = layer
        self.sync = sync if sync is not None else GradSync([layer])
        self.group, self.nslots, self.branch = group, max(2, slots), branch
        self.dev = layer.phi.device
        self.s_in = torch.cuda.Stream(device=self.dev)
        self.s_out = torch.cuda.Stream(device=self.dev)
        self._stage = None
        self._free_ev = [None] * self.nslots   # per staging slot: the backward that last read it (kept across calls)
        self._next = 0                         # running group count: consecutive calls rotate through the slots

    def _staging(self, shape, dtype):
        key = (tuple(shape), dtype)
        if self._stage is None or self._stage[0] != key:
            bufs = [(torch.empty(shape, device=self.dev, dtype=dtype), torch.empty(shape, device=self.dev, dtype=dtype))
                    for _ in range(self.nslots)]
            self._stage = (key, bufs)
            self._free_ev = [None] * self.nslots
        return self._stage[1]

    def __call__(self, H_host: torch.Tensor, g_host: torch.Tensor, out_H_new: torch.Tensor, out_dH: torch.Tensor,
                 out_param_grads: Optional[torch.Tensor] = None) -> None:
        """All four activation buffers are host tensors [B, S, 4, D] (pinned for real overlap).
        out_param_grads, if given, receives the flat gradient record (phi | bias | alpha).
        Returns after queueing everything; synchronise the device (or the current stream)
        before reading the outputs."""
        layer, sync = self.layer, self.sync
        B = H_host.shape[0]
        G = self.group
        bufs = self._staging((G,) + tuple(H_host.shape[1:]), H_host.dtype)
        comp = torch.cuda.current_stream(self.dev)
        free_ev = self._free_ev
        first = self._next
        hook = layer.grads_ready_hook
        n_groups = (B + G - 1) // G
        keep = []
        for i in range(n_groups):
            lo, hi = i * G, min(B, (i + 1) * G)
            n = hi - lo
            slot = (first + i) % self.nslots
            Hd, gd = bufs[slot]
            with torch.cuda.stream(self.s_in):
                if free_ev[slot] is not None:   # also holds across calls: the previous call's kernels may still read it
                    self.s_in.wait_event(free_ev[slot])
                Hd[:n].copy_(H_host[lo:hi], non_blocking=True)
                ev_in = torch.cuda.Event()
                ev_in.record(self.s_in)          # the forward needs only H ...
                gd[:n].copy_(g_host[lo:hi], non_blocking=True)
                ev_in_g = torch.cuda.Event()
                ev_in_g.record(self.s_in)        # ... the upstream gradient arrives while it runs
            comp.wait_event(ev_in)
            Hin = Hd[:n].detach().requires_grad_(True)
            layer.grad_accumulate = i > 0
            layer.grads_ready_hook = hook if i == n_groups - 1 else None
            bi, add = layer(Hin)
            H_new = add(bi if self.branch is None else self.branch(bi))
            ev_fwd = torch.cuda.Event()
            ev_fwd.record(comp)
            comp.wait_event(ev_in_g)
            H_new.backward(gd[:n])
            ev_bwd = torch.cuda.Event()
            ev_bwd.record(comp)
            free_ev[slot] = ev_bwd
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(ev_fwd)
                out_H_new[lo:hi].copy_(H_new.detach(), non_blocking=True)
                self.s_out.wait_event(ev_bwd)
                out_dH[lo:hi].copy_(Hin.grad, non_blocking=True)
            H_new.record_stream(self.s_out)
            Hin.grad.record_stream(self.s_out)
            keep.append((H_new, Hin))
        self._next = (first + n_groups) % self.nslots
        layer.grad_accumulate = False
        layer.grads_ready_hook = hook
        sync.finish()
        if out_param_grads is not None:
            out_param_grads.copy_(sync.flat, non_blocking=True)
        done = torch.cuda.Event()
        done.record(self.s_out)
        comp.wait_event(done)
