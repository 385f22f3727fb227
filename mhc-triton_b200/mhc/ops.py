"""Autograd ops of the hyper-connection path, backed by the sm_100a CUDA library.

Public functions and their semantics follow the reference's src/mhc/ops.py:231-323:
sinkhorn_knopp, fused_stream_mix, fused_add_residual, fused_dynamic_weights.
`hyper_connection_mix` is the fused node the module uses: mean-pool + dynamic weights +
stream mix in one autograd Function, so that the gradient of the pooled state is folded into
the single write of dH instead of a separate read-modify-write pass.
"""

from typing import Tuple

import torch

from ._backward import (add_residual_backward, fused_dynamic_weights_backward, hc_mix_backward, sinkhorn_backward,
                        stream_mix_backward)
from ._kernels import (add_residual_forward, add_residual_mix_forward, fused_dynamic_weights_forward, hc_mix_forward,
                       meanpool_forward, sinkhorn_forward, stream_mix_forward)


# The public functions below are opaque to torch.compile (the kernels are reached through ctypes):
# a compiled model calls them eagerly and compiles what surrounds them.


class _SinkhornKnopp(torch.autograd.Function):
    """Saves only M; the backward recomputes the iterations (reference: src/mhc/ops.py:15-29)."""

    @staticmethod
    def forward(ctx, M, num_iters, eps):
        ctx.save_for_backward(M)
        ctx.num_iters, ctx.eps = num_iters, eps
        return sinkhorn_forward(M, num_iters, eps)

    @staticmethod
    def backward(ctx, grad_output):
        (M,) = ctx.saved_tensors
        return sinkhorn_backward(M, grad_output, ctx.num_iters, ctx.eps), None, None


class _FusedStreamMix(torch.autograd.Function):
    """Reference: src/mhc/ops.py:32-49."""

    @staticmethod
    def forward(ctx, H, H_pre, H_res):
        branch_input, H_residual = stream_mix_forward(H, H_pre, H_res)
        ctx.save_for_backward(H, H_pre, H_res)
        ctx.set_materialize_grads(False)
        return branch_input, H_residual

    @staticmethod
    def backward(ctx, grad_branch_input, grad_H_residual):
        H, H_pre, H_res = ctx.saved_tensors
        if grad_branch_input is None and grad_H_residual is None:
            return None, None, None
        if grad_branch_input is None:
            grad_branch_input = torch.zeros(H.shape[0], H.shape[1], H.shape[3], device=H.device, dtype=H.dtype)
        if grad_H_residual is None:
            grad_H_residual = torch.zeros_like(H)
        dH, dH_pre, dH_res = stream_mix_backward(grad_branch_input, grad_H_residual, H, H_pre, H_res)
        return dH, dH_pre.to(H_pre.dtype), dH_res.to(H_res.dtype)


class _FusedAddResidual(torch.autograd.Function):
    """Reference: src/mhc/ops.py:52-69.  The gradient of H_residual is the upstream gradient
    itself and is returned without a copy."""

    @staticmethod
    def forward(ctx, H_residual, branch_output, H_post, pool):
        ctx.save_for_backward(branch_output, H_post)
        ctx.set_materialize_grads(False)
        if pool:
            H_new, partials = add_residual_forward(H_residual, branch_output, H_post, pool=True)
            ctx.mark_non_differentiable(partials)
            return H_new, partials
        return add_residual_forward(H_residual, branch_output, H_post)

    @staticmethod
    def backward(ctx, grad_H_new, _unused=None):
        if grad_H_new is None:
            return None, None, None, None
        branch_output, H_post = ctx.saved_tensors
        dH_residual, d_bo, dH_post = add_residual_backward(grad_H_new, branch_output, H_post)
        return dH_residual, d_bo.to(branch_output.dtype), dH_post.to(H_post.dtype), None


class _AddResidualFromState(torch.autograd.Function):
    """H_new = H_res @ H + H_post * branch_output with the residual mix recomputed from H.

    `stand_in` is the storage-less second output of the fused node run with lazy_residual=True;
    the gradient with respect to the residual mix (which equals the upstream gradient) is returned
    for it, and the fused node turns it into the gradients of H and H_res, exactly as it does for
    a materialised H_residual.  That is why H and H_res receive no gradient from this node."""

    @staticmethod
    def forward(ctx, stand_in, H, H_res, branch_output, H_post, pool):
        ctx.save_for_backward(branch_output, H_post)
        ctx.set_materialize_grads(False)
        if pool:
            H_new, partials = add_residual_mix_forward(H, H_res, branch_output, H_post, pool=True)
            ctx.mark_non_differentiable(partials)
            return H_new, partials
        return add_residual_mix_forward(H, H_res, branch_output, H_post)

    @staticmethod
    def backward(ctx, grad_H_new, _unused=None):
        if grad_H_new is None:
            return None, None, None, None, None, None
        branch_output, H_post = ctx.saved_tensors
        dH_residual, d_bo, dH_post = add_residual_backward(grad_H_new, branch_output, H_post)
        return dH_residual, None, None, d_bo.to(branch_output.dtype), dH_post.to(H_post.dtype), None


class _FusedDynamicWeights(torch.autograd.Function):
    """Reference: src/mhc/ops.py:72-228.  The scales are read on the device (no .item())."""

    @staticmethod
    def forward(ctx, x, phi, bias, alpha_pre, alpha_post, alpha_res, sinkhorn_iters, eps):
        H_pre, H_post, H_res, saved = fused_dynamic_weights_forward(
            x, phi, bias, alpha_pre, alpha_post, alpha_res, sinkhorn_iters, eps, return_saved=True)
        ctx.save_for_backward(x, phi, bias, alpha_pre, alpha_post, alpha_res, saved)
        ctx.sinkhorn_iters, ctx.eps = sinkhorn_iters, eps
        ctx.set_materialize_grads(False)
        return H_pre, H_post, H_res

    @staticmethod
    def backward(ctx, grad_H_pre, grad_H_post, grad_H_res):
        x, phi, bias, alpha_pre, alpha_post, alpha_res, saved = ctx.saved_tensors
        B = x.shape[0]
        if grad_H_pre is None:
            grad_H_pre = torch.zeros(B, 4, device=x.device)
        if grad_H_post is None:
            grad_H_post = torch.zeros(B, 4, device=x.device)
        if grad_H_res is None:
            grad_H_res = torch.zeros(B, 4, 4, device=x.device)
        gx, gphi, gbias, galpha = fused_dynamic_weights_backward(
            x, phi, bias, alpha_pre, alpha_post, alpha_res, saved, grad_H_pre, grad_H_post, grad_H_res,
            ctx.sinkhorn_iters, ctx.eps)
        return (gx.to(x.dtype), gphi.to(phi.dtype), gbias.to(bias.dtype),
                galpha[0:1].reshape_as(alpha_pre).to(alpha_pre.dtype),
                galpha[1:2].reshape_as(alpha_post).to(alpha_post.dtype),
                galpha[2:3].reshape_as(alpha_res).to(alpha_res.dtype), None, None)


class _SequenceMeanPool(torch.autograd.Function):
    """x = H.mean(dim=1).reshape(B, 4*D) in fp32 (reference: src/mhc/module.py:123)."""

    @staticmethod
    def forward(ctx, H):
        ctx.shape, ctx.dtype = H.shape, H.dtype
        return meanpool_forward(H)

    @staticmethod
    def backward(ctx, gx):
        B, S, n, D = ctx.shape
        return (gx.reshape(B, 1, n, D) / S).to(ctx.dtype).expand(B, S, n, D)


class _HyperConnectionMix(torch.autograd.Function):
    """Mean-pool + dynamic weights + stream mix as one autograd node.

    Inputs : H, H_pre_base, H_post_base, H_res_base, phi, alpha_pre, alpha_post, alpha_res
    Outputs: branch_input, H_residual, H_post
    Forward and backward are one library call each.  Backward: one reduction pass (dH_pre,
    dH_res), the small weights backward, then one apply pass that writes dH once, including
    grad_x / S.  When `grad_sink` (a flat fp32
    buffer of 4*D*24 + 27 elements) is given, grad_phi / grad_bias / grad_alpha are written
    straight into it, ready for one all-reduce, and `ready_hook` is told so; `ready_event`, if
    given, is recorded on the stream between the kernels that fill the buffer and the pass that
    writes dH, so a collective that waits for it overlaps that pass.
    """

    @staticmethod
    def forward(ctx, H, H_pre_base, H_post_base, H_res_base, phi, alpha_pre, alpha_post, alpha_res,
                sinkhorn_iters, eps, grad_sink, ready_hook, accumulate, pooled, lazy_residual, ready_event=None):
        branch_input, H_residual, H_post, H_pre, H_res, x, saved = hc_mix_forward(
            H, H_pre_base, H_post_base, H_res_base, phi, alpha_pre, alpha_post, alpha_res, sinkhorn_iters, eps,
            pooled=pooled, want_residual=not lazy_residual)
        if lazy_residual:
            # A stand-in with H's shape and no storage of its own: it only carries the gradient of the
            # (never materialised) residual mix back to this node.  Its values are meaningless.
            H_residual = branch_input.new_empty(1).expand(H.shape)
        ctx.save_for_backward(H, x, phi, H_pre_base, H_post_base, H_res_base, alpha_pre, alpha_post, alpha_res,
                              saved, H_pre, H_res)
        ctx.sinkhorn_iters, ctx.eps, ctx.grad_sink, ctx.ready_hook = sinkhorn_iters, eps, grad_sink, ready_hook
        ctx.accumulate = bool(accumulate) and grad_sink is not None
        ctx.ready_event = ready_event
        ctx.mark_non_differentiable(H_pre, H_res)
        ctx.set_materialize_grads(False)   # no zero-filled gradients for outputs nobody used
        return branch_input, H_residual, H_post, H_pre, H_res

    @staticmethod
    def backward(ctx, d_branch_input, dH_residual, dH_post, _unused_pre, _unused_res):
        (H, x, phi, pre_b, post_b, res_b, alpha_pre, alpha_post, alpha_res, saved, H_pre, H_res) = ctx.saved_tensors
        B, S, _, D = H.shape
        if d_branch_input is None:
            d_branch_input = torch.zeros(B, S, D, device=H.device, dtype=H.dtype)
        if dH_residual is None:
            dH_residual = torch.zeros_like(H)
        if dH_post is None:
            dH_post = torch.zeros(B, 4, device=H.device, dtype=torch.float32)
        dH, gphi, gbias, galpha = hc_mix_backward(
            d_branch_input, dH_residual, dH_post, H, x, phi, pre_b, post_b, res_b, alpha_pre, alpha_post, alpha_res,
            saved, H_pre, H_res, ctx.sinkhorn_iters, ctx.eps, param_grads=ctx.grad_sink, accumulate=ctx.accumulate,
            ready_event=ctx.ready_event)
        if ctx.ready_hook is not None:
            ctx.ready_hook(ctx.grad_sink)
        if ctx.grad_sink is not None:  # the parameters' .grad tensors are views of the sink already
            return (dH,) + (None,) * 15
        return (dH, gbias[0:4].reshape(pre_b.shape).to(pre_b.dtype), gbias[4:8].reshape(post_b.shape).to(post_b.dtype),
                gbias[8:24].reshape(res_b.shape).to(res_b.dtype), gphi.to(phi.dtype),
                galpha[0:1].reshape_as(alpha_pre).to(alpha_pre.dtype),
                galpha[1:2].reshape_as(alpha_post).to(alpha_post.dtype),
                galpha[2:3].reshape_as(alpha_res).to(alpha_res.dtype), None, None, None, None, None, None, None, None)


@torch.compiler.disable
def sinkhorn_knopp(M: torch.Tensor, num_iters: int = 20, eps: float = 1e-8) -> torch.Tensor:
    """Project (batch, 4, 4) matrices to (approximately) doubly stochastic ones by `num_iters`
    alternating row / column normalisations of |M| + eps."""
    return _SinkhornKnopp.apply(M, num_iters, eps)


@torch.compiler.disable
def fused_stream_mix(H: torch.Tensor, H_pre: torch.Tensor, H_res: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """H (batch, seq, 4, dim), H_pre (batch, 4), H_res (batch, 4, 4) ->
    branch_input (batch, seq, dim), H_residual (batch, seq, 4, dim)."""
    return _FusedStreamMix.apply(H, H_pre, H_res)


@torch.compiler.disable
def fused_add_residual(H_residual: torch.Tensor, branch_output: torch.Tensor, H_post: torch.Tensor,
                       pool_for_next: bool = False) -> torch.Tensor:
    """H_new[n] = H_residual[n] + H_post[n] * branch_output, per batch element.

    With pool_for_next=True the same kernel also accumulates the per-chunk token sums of H_new and
    the returned tensor carries them (attribute `_mhc_pooled`); a HyperConnection that receives
    this very tensor as its input uses them instead of reading H once more for its mean-pool."""
    if not pool_for_next:
        return _FusedAddResidual.apply(H_residual, branch_output, H_post, False)
    H_new, partials = _FusedAddResidual.apply(H_residual, branch_output, H_post, True)
    H_new._mhc_pooled = (partials, version_of(H_new))
    return H_new


@torch.compiler.disable
def add_residual_from_state(stand_in, H, H_res, branch_output, H_post, pool_for_next: bool = False) -> torch.Tensor:
    """Second half of a layer whose fused node ran with lazy_residual=True (see hyper_connection_mix):
    H_new = H_res @ H + H_post * branch_output, the residual mix recomputed from H."""
    if not pool_for_next:
        return _AddResidualFromState.apply(stand_in, H, H_res, branch_output, H_post, False)
    H_new, partials = _AddResidualFromState.apply(stand_in, H, H_res, branch_output, H_post, True)
    H_new._mhc_pooled = (partials, version_of(H_new))
    return H_new


def version_of(t: torch.Tensor):
    """In-place modification counter of t, or None for inference tensors (which keep none)."""
    return None if t.is_inference() else t._version


def pooled_sums_of(H: torch.Tensor):
    """Token sums attached to H by fused_add_residual(pool_for_next=True), or None if absent, of the
    wrong shape, or if H was modified in place since."""
    tag = getattr(H, "_mhc_pooled", None)
    if tag is None:
        return None
    partials, version = tag
    if version_of(H) != version or H.dim() != 4 or partials.shape[0] != H.shape[0] or \
            partials.shape[2] != 4 * H.shape[3] or partials.device != H.device:
        return None
    return partials


@torch.compiler.disable
def fused_dynamic_weights(x, phi, bias, alpha_pre, alpha_post, alpha_res, sinkhorn_iters: int = 20,
                          eps: float = 1e-6) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """x [batch, in_dim], phi [in_dim, 24], bias [24], three one-element scale tensors ->
    H_pre [batch, 4] (rows sum to 1), H_post [batch, 4] in (0, 2), H_res [batch, 4, 4]
    (Sinkhorn-projected).  Outputs are fp32."""
    return _FusedDynamicWeights.apply(x, phi, bias, alpha_pre, alpha_post, alpha_res, sinkhorn_iters, eps)


@torch.compiler.disable
def sequence_mean_pool(H: torch.Tensor) -> torch.Tensor:
    """H (batch, seq, 4, dim) -> fp32 (batch, 4*dim) mean over the sequence axis."""
    return _SequenceMeanPool.apply(H)


@torch.compiler.disable
def hyper_connection_mix(H, H_pre_base, H_post_base, H_res_base, phi, alpha_pre, alpha_post, alpha_res,
                         sinkhorn_iters: int = 20, eps: float = 1e-6, grad_sink=None, ready_hook=None,
                         accumulate: bool = False, pooled=None, lazy_residual: bool = False, ready_event=None):
    """Fused pooled-weights + stream-mix node; returns
    (branch_input, H_residual, H_post, H_pre, H_res); the last two carry no gradient.
    With `grad_sink` the parameter gradients are written into that flat buffer and no
    gradient is returned for the parameters; `ready_hook(grad_sink)` is called as soon as
    the kernels that fill it have been launched; `accumulate` adds to the buffer instead of
    overwriting it; `pooled` are token sums of H from the previous layer (see fused_add_residual).
    With lazy_residual=True the second output is a storage-less stand-in to be passed to
    add_residual_from_state, which recomputes the residual mix from H.  `ready_event`: a
    torch.cuda.Event the backward records once the parameter gradients are complete in stream
    order (before dH is)."""
    return _HyperConnectionMix.apply(H, H_pre_base, H_post_base, H_res_base, phi, alpha_pre, alpha_post, alpha_res,
                                     sinkhorn_iters, eps, grad_sink, ready_hook, accumulate, pooled, lazy_residual,
                                     ready_event)
