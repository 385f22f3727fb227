"""The four public ops registered with torch.library (namespace ``mhc``), for code that is
compiled with ``torch.compile(fullgraph=True)`` or exported.

The plain functions in ``mhc.ops`` reach the kernels through ctypes from inside
``torch.autograd.Function``s, which a tracing compiler cannot look into (they are marked opaque and
cause a graph break).  Here every kernel call is a ``torch.library.custom_op`` with a fake
(shape-only) implementation and an autograd formula made of other custom ops, so the tracer sees
ordinary operators:

    from mhc.library import sinkhorn_knopp, fused_stream_mix, fused_add_residual, fused_dynamic_weights

Same signatures and results as the functions of the same names in ``mhc.ops`` (which follow the
reference's src/mhc/ops.py:231-323).
"""

from typing import Tuple

import torch
from torch import Tensor

from . import _backward as B
from . import _kernels as K


# ------------------------------------------------------------------------------ Sinkhorn
@torch.library.custom_op("mhc::sinkhorn_fwd", mutates_args=())
def _sinkhorn_fwd(M: Tensor, iters: int, eps: float) -> Tensor:
    return K.sinkhorn_forward(M, iters, eps)


@_sinkhorn_fwd.register_fake
def _(M, iters, eps):
    return torch.empty_like(M, memory_format=torch.contiguous_format)


@torch.library.custom_op("mhc::sinkhorn_bwd", mutates_args=())
def _sinkhorn_bwd(M: Tensor, dP: Tensor, iters: int, eps: float) -> Tensor:
    return B.sinkhorn_backward(M, dP, iters, eps)


@_sinkhorn_bwd.register_fake
def _(M, dP, iters, eps):
    return torch.empty_like(M, memory_format=torch.contiguous_format)


def _sinkhorn_setup(ctx, inputs, output):
    M, ctx.iters, ctx.eps = inputs
    ctx.save_for_backward(M)


def _sinkhorn_grad(ctx, g):
    (M,) = ctx.saved_tensors
    return _sinkhorn_bwd(M, g.contiguous(), ctx.iters, ctx.eps), None, None


_sinkhorn_fwd.register_autograd(_sinkhorn_grad, setup_context=_sinkhorn_setup)


# ---------------------------------------------------------------------------- stream mix
@torch.library.custom_op("mhc::stream_mix_fwd", mutates_args=())
def _stream_mix_fwd(H: Tensor, H_pre: Tensor, H_res: Tensor) -> Tuple[Tensor, Tensor]:
    return K.stream_mix_forward(H, H_pre, H_res)


@_stream_mix_fwd.register_fake
def _(H, H_pre, H_res):
    Bn, S, _, D = H.shape
    return H.new_empty(Bn, S, D), torch.empty_like(H, memory_format=torch.contiguous_format)


@torch.library.custom_op("mhc::stream_mix_bwd", mutates_args=())
def _stream_mix_bwd(d_bi: Tensor, dHr: Tensor, H: Tensor, H_pre: Tensor, H_res: Tensor) -> Tuple[Tensor, Tensor, Tensor]:
    return B.stream_mix_backward(d_bi, dHr, H, H_pre, H_res)


@_stream_mix_bwd.register_fake
def _(d_bi, dHr, H, H_pre, H_res):
    Bn = H.shape[0]
    return (torch.empty_like(H, memory_format=torch.contiguous_format),
            H.new_empty(Bn, 4, dtype=torch.float32), H.new_empty(Bn, 4, 4, dtype=torch.float32))


def _mix_setup(ctx, inputs, output):
    ctx.save_for_backward(*inputs)


def _mix_grad(ctx, g_bi, g_hr):
    H, H_pre, H_res = ctx.saved_tensors
    dH, dH_pre, dH_res = _stream_mix_bwd(g_bi.contiguous(), g_hr.contiguous(), H, H_pre, H_res)
    return dH, dH_pre.to(H_pre.dtype), dH_res.to(H_res.dtype)


_stream_mix_fwd.register_autograd(_mix_grad, setup_context=_mix_setup)


# -------------------------------------------------------------------------- add residual
@torch.library.custom_op("mhc::add_residual_fwd", mutates_args=())
def _add_residual_fwd(H_residual: Tensor, branch_output: Tensor, H_post: Tensor) -> Tensor:
    return K.add_residual_forward(H_residual, branch_output, H_post)


@_add_residual_fwd.register_fake
def _(H_residual, branch_output, H_post):
    return torch.empty_like(H_residual, memory_format=torch.contiguous_format)


@torch.library.custom_op("mhc::add_residual_bwd", mutates_args=())
def _add_residual_bwd(dH_new: Tensor, branch_output: Tensor, H_post: Tensor) -> Tuple[Tensor, Tensor]:
    _, d_bo, dH_post = B.add_residual_backward(dH_new, branch_output, H_post)
    return d_bo, dH_post


@_add_residual_bwd.register_fake
def _(dH_new, branch_output, H_post):
    return (torch.empty_like(branch_output, dtype=dH_new.dtype, memory_format=torch.contiguous_format),
            dH_new.new_empty(dH_new.shape[0], 4, dtype=torch.float32))


def _add_setup(ctx, inputs, output):
    _, branch_output, H_post = inputs
    ctx.save_for_backward(branch_output, H_post)


def _add_grad(ctx, g):
    branch_output, H_post = ctx.saved_tensors
    g = g.contiguous()
    d_bo, dH_post = _add_residual_bwd(g, branch_output, H_post)
    return g, d_bo.to(branch_output.dtype), dH_post.to(H_post.dtype)   # the residual's gradient is g itself


_add_residual_fwd.register_autograd(_add_grad, setup_context=_add_setup)


# ------------------------------------------------------------------------ dynamic weights
@torch.library.custom_op("mhc::dynamic_weights_fwd", mutates_args=())
def _dynamic_weights_fwd(x: Tensor, phi: Tensor, bias: Tensor, alpha_pre: Tensor, alpha_post: Tensor,
                         alpha_res: Tensor, iters: int, eps: float) -> Tuple[Tensor, Tensor, Tensor, Tensor]:
    return K.fused_dynamic_weights_forward(x, phi, bias, alpha_pre, alpha_post, alpha_res, iters, eps,
                                           return_saved=True)


@_dynamic_weights_fwd.register_fake
def _(x, phi, bias, alpha_pre, alpha_post, alpha_res, iters, eps):
    Bn = x.shape[0]
    f = dict(dtype=torch.float32)
    return x.new_empty(Bn, 4, **f), x.new_empty(Bn, 4, **f), x.new_empty(Bn, 4, 4, **f), x.new_empty(Bn, 32, **f)


@torch.library.custom_op("mhc::dynamic_weights_bwd", mutates_args=())
def _dynamic_weights_bwd(x: Tensor, phi: Tensor, bias: Tensor, alpha_pre: Tensor, alpha_post: Tensor,
                         alpha_res: Tensor, saved: Tensor, g_pre: Tensor, g_post: Tensor, g_res: Tensor,
                         iters: int, eps: float) -> Tuple[Tensor, Tensor, Tensor, Tensor]:
    gx, gphi, gbias, galpha = B.fused_dynamic_weights_backward(x, phi, bias, alpha_pre, alpha_post, alpha_res, saved,
                                                               g_pre, g_post, g_res, iters, eps)
    return gx, gphi.clone(), gbias.clone(), galpha.clone()   # the wrapper returns views of one buffer


@_dynamic_weights_bwd.register_fake
def _(x, phi, bias, alpha_pre, alpha_post, alpha_res, saved, g_pre, g_post, g_res, iters, eps):
    f = dict(dtype=torch.float32)
    return (x.new_empty(x.shape, **f), x.new_empty(phi.shape, **f), x.new_empty(24, **f), x.new_empty(3, **f))


def _dw_setup(ctx, inputs, output):
    x, phi, bias, a_pre, a_post, a_res, ctx.iters, ctx.eps = inputs
    ctx.save_for_backward(x, phi, bias, a_pre, a_post, a_res, output[3])


def _dw_grad(ctx, g_pre, g_post, g_res, _g_saved):
    x, phi, bias, a_pre, a_post, a_res, saved = ctx.saved_tensors
    gx, gphi, gbias, galpha = _dynamic_weights_bwd(x, phi, bias, a_pre, a_post, a_res, saved, g_pre.contiguous(),
                                                   g_post.contiguous(), g_res.contiguous(), ctx.iters, ctx.eps)
    return (gx.to(x.dtype), gphi.to(phi.dtype), gbias.to(bias.dtype), galpha[0:1].reshape(a_pre.shape).to(a_pre.dtype),
            galpha[1:2].reshape(a_post.shape).to(a_post.dtype), galpha[2:3].reshape(a_res.shape).to(a_res.dtype),
            None, None)


_dynamic_weights_fwd.register_autograd(_dw_grad, setup_context=_dw_setup)


# --------------------------------------------------------------------------- public names
def sinkhorn_knopp(M: Tensor, num_iters: int = 20, eps: float = 1e-8) -> Tensor:
    return _sinkhorn_fwd(M, num_iters, eps)


def fused_stream_mix(H: Tensor, H_pre: Tensor, H_res: Tensor) -> Tuple[Tensor, Tensor]:
    return _stream_mix_fwd(H, H_pre, H_res)


def fused_add_residual(H_residual: Tensor, branch_output: Tensor, H_post: Tensor) -> Tensor:
    return _add_residual_fwd(H_residual, branch_output, H_post)


def fused_dynamic_weights(x: Tensor, phi: Tensor, bias: Tensor, alpha_pre, alpha_post, alpha_res,
                          sinkhorn_iters: int = 20, eps: float = 1e-6) -> Tuple[Tensor, Tensor, Tensor]:
    """alpha_* are one-element tensors (they then receive gradients) or Python floats."""
    alpha_pre, alpha_post, alpha_res = [a if isinstance(a, Tensor) else torch.full((1,), float(a), device=x.device)
                                        for a in (alpha_pre, alpha_post, alpha_res)]
    H_pre, H_post, H_res, _ = _dynamic_weights_fwd(x, phi, bias, alpha_pre, alpha_post, alpha_res, sinkhorn_iters, eps)
    return H_pre, H_post, H_res
