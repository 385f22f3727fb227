"""HyperConnection: multi-stream residual connection with constrained mixing weights.

Constructor arguments, parameter names / shapes / registration order, the three weight
modes and the forward contract follow the reference module (src/mhc/module.py:10-224
there), so state dicts interchange with it.
"""

from typing import Callable, Tuple

import torch
import torch.nn as nn

from .ops import (add_residual_from_state, fused_add_residual, fused_dynamic_weights, fused_stream_mix,
                  hyper_connection_mix, pooled_sums_of, sequence_mean_pool, sinkhorn_knopp, version_of)


class HyperConnection(nn.Module):
    """Manifold-constrained hyper-connection over 4 residual streams.

    forward(H) with H of shape (batch, seq, 4, dim) returns ``(branch_input, add_residual)``;
    run the wrapped layer on ``branch_input`` (batch, seq, dim) and call
    ``add_residual(branch_output)`` to get the updated (batch, seq, 4, dim) state.

    Args:
        dim: width of each stream
        num_streams: must be 4
        layer_idx: selects which stream the pre-mix weights favour at initialisation
        dynamic: compute the weights from the (sequence mean-pooled) input
        sinkhorn_iters: Sinkhorn-Knopp iterations for the residual mixing matrix
        init_scale: initial value of the learnable scales of the dynamic part
        eps: numerical-stability constant of the fused dynamic path
        use_fused_weights: single projection ``phi`` [4*dim, 24] (True) or three linear maps
    """

    def __init__(self, dim: int, num_streams: int = 4, layer_idx: int = 0, dynamic: bool = True,
                 sinkhorn_iters: int = 20, init_scale: float = 0.1, eps: float = 1e-6,
                 use_fused_weights: bool = True):
        super().__init__()
        if num_streams != 4:
            raise ValueError("Triton kernels require num_streams=4")
        self.dim = dim
        self.num_streams = num_streams
        self.dynamic = dynamic
        self.sinkhorn_iters = sinkhorn_iters
        self.init_scale = init_scale
        self.layer_idx = layer_idx
        self.eps = eps
        self.use_fused_weights = use_fused_weights and dynamic
        # Optional flat fp32 buffer [4*dim*24 + 27]; when set, the fused backward writes the
        # gradients of phi, the three base tensors (as the 24-entry bias) and the three scales
        # into it back to back (see mhc.parallel).
        self.grad_sink = None
        self.grads_ready_hook = None
        self.grads_ready_event = None  # torch.cuda.Event recorded by the backward once grad_sink is complete
        self.grad_accumulate = False   # add to grad_sink instead of overwriting it
        # Fused dynamic path: do not write H_residual in forward(); add_residual() recomputes the residual
        # mix from H in the same kernel that adds the branch output (8 of 46 bytes per element less).
        self.materialize_residual = False

        n = num_streams
        in_dim = n * dim
        self.H_post_base = nn.Parameter(torch.ones(n))
        pre = torch.zeros(n)
        pre[layer_idx % n] = 1.0
        self.H_pre_base = nn.Parameter(pre)
        self.H_res_base = nn.Parameter(torch.eye(n))
        if dynamic:
            if use_fused_weights:
                self.phi = nn.Parameter(torch.zeros(in_dim, n * n + 2 * n))
                # one-element 1-D tensors (sharding wrappers dislike 0-d parameters)
                self.alpha_pre = nn.Parameter(torch.tensor([init_scale]))
                self.alpha_post = nn.Parameter(torch.tensor([init_scale]))
                self.alpha_res = nn.Parameter(torch.tensor([init_scale]))
            else:
                self.W_post = nn.Linear(in_dim, n, bias=False)
                self.W_pre = nn.Linear(in_dim, n, bias=False)
                self.W_res = nn.Linear(in_dim, n * n, bias=False)
                for lin in (self.W_post, self.W_pre, self.W_res):
                    nn.init.zeros_(lin.weight)
                self.scale_post = nn.Parameter(torch.tensor([init_scale]))
                self.scale_pre = nn.Parameter(torch.tensor([init_scale]))
                self.scale_res = nn.Parameter(torch.tensor([init_scale]))

    # -- weights ------------------------------------------------------------------------
    def _compute_weights(self, H: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """(H_post, H_pre, H_res) -- note the order -- through the individual ops."""
        n, B = self.num_streams, H.shape[0]
        if not self.dynamic:
            H_post = torch.sigmoid(self.H_post_base).unsqueeze(0).expand(B, -1)
            sp = torch.sigmoid(self.H_pre_base)
            H_pre = (sp / (sp.sum() + 1e-8)).unsqueeze(0).expand(B, -1)
            H_res = sinkhorn_knopp(self.H_res_base.unsqueeze(0).expand(B, -1, -1).contiguous(), self.sinkhorn_iters)
            return H_post.contiguous(), H_pre.contiguous(), H_res.contiguous()
        x = sequence_mean_pool(H)  # fp32 [B, 4*dim]
        if self.use_fused_weights:
            bias = torch.cat([self.H_pre_base, self.H_post_base, self.H_res_base.flatten()])
            H_pre, H_post, H_res = fused_dynamic_weights(x, self.phi, bias, self.alpha_pre, self.alpha_post,
                                                         self.alpha_res, self.sinkhorn_iters, self.eps)
            return H_post.contiguous(), H_pre.contiguous(), H_res.contiguous()
        x = x.to(self.W_post.weight.dtype)
        x = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + self.eps)
        d_post = self.W_post(x) * self.scale_post
        d_pre = self.W_pre(x) * self.scale_pre
        d_res = self.W_res(x).reshape(B, n, n) * self.scale_res
        H_post = torch.sigmoid(self.H_post_base + d_post)
        sp = torch.sigmoid(self.H_pre_base + d_pre)
        H_pre = sp / (sp.sum(dim=-1, keepdim=True) + 1e-8)
        H_res = sinkhorn_knopp((self.H_res_base + d_res).contiguous(), self.sinkhorn_iters)
        return H_post.contiguous(), H_pre.contiguous(), H_res.contiguous()

    # -- forward ------------------------------------------------------------------------
    # The kernels are reached through ctypes, which a tracing compiler cannot see into: under
    # torch.compile the layer runs as an opaque eager call and the model around it is compiled.
    @torch.compiler.disable
    def forward(self, H: torch.Tensor) -> Tuple[torch.Tensor, Callable[[torch.Tensor], torch.Tensor]]:
        if self.use_fused_weights:
            lazy = not self.materialize_residual
            branch_input, H_residual, H_post, _, H_res = hyper_connection_mix(
                H, self.H_pre_base, self.H_post_base, self.H_res_base, self.phi, self.alpha_pre, self.alpha_post,
                self.alpha_res, self.sinkhorn_iters, self.eps, self.grad_sink, self.grads_ready_hook,
                self.grad_accumulate, pooled_sums_of(H), lazy, self.grads_ready_event)
            if lazy:
                version = version_of(H)

                def add_residual(branch_output: torch.Tensor, pool_for_next: bool = False) -> torch.Tensor:
                    """pool_for_next=True: also accumulate the token sums the NEXT HyperConnection needs
                    for its mean-pool (pass the returned tensor to it as is)."""
                    if version_of(H) != version:
                        raise RuntimeError("H was modified in place between HyperConnection.forward and add_residual "
                                           "(set layer.materialize_residual = True if that is intended)")
                    return add_residual_from_state(H_residual, H, H_res, branch_output, H_post, pool_for_next)

                return branch_input, add_residual
        else:
            H_post, H_pre, H_res = self._compute_weights(H)
            branch_input, H_residual = fused_stream_mix(H, H_pre, H_res)

        def add_residual(branch_output: torch.Tensor, pool_for_next: bool = False) -> torch.Tensor:
            """pool_for_next=True: also accumulate the token sums the NEXT HyperConnection needs for its
            mean-pool, so that layer reads H once instead of twice (pass the returned tensor to it as is)."""
            return fused_add_residual(H_residual, branch_output, H_post, pool_for_next)

        return branch_input, add_residual

    def extra_repr(self) -> str:
        return (f"dim={self.dim}, num_streams={self.num_streams}, dynamic={self.dynamic}, "
                f"sinkhorn_iters={self.sinkhorn_iters}, use_fused_weights={self.use_fused_weights}")

    def init_weights(self, layer_idx=None):
        """Re-initialise all parameters; optionally change the layer index first."""
        if layer_idx is not None:
            self.layer_idx = layer_idx
        with torch.no_grad():
            self.H_post_base.fill_(1.0)
            self.H_pre_base.zero_()
            self.H_pre_base[self.layer_idx % self.num_streams] = 1.0
            self.H_res_base.copy_(torch.eye(self.num_streams))
            if self.dynamic:
                if self.use_fused_weights:
                    self.phi.zero_()
                    for a in (self.alpha_pre, self.alpha_post, self.alpha_res):
                        a.fill_(self.init_scale)
                else:
                    for lin in (self.W_post, self.W_pre, self.W_res):
                        lin.weight.zero_()
