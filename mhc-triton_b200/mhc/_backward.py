"""Backward launch wrappers (reference counterparts: src/mhc/_backward.py:503-626 there).

Weight gradients (dH_pre, dH_post, dH_res) are reduced inside the CUDA library, in a fixed
order, and returned as fp32.
"""

from typing import Optional, Tuple

import torch

from . import _lib as L
from ._kernels import _check, _alpha_dev

_ABS0 = {"zero": L.ABS0_ZERO, "plus_one": L.ABS0_PLUS_ONE}
_abs_grad_at_zero = "zero"


def set_abs_grad_at_zero(mode: str) -> None:
    """Convention for d|m|/dm at m == 0 in the Sinkhorn backward.

    "zero" (default) matches autograd of the reference's PyTorch path; "plus_one" matches
    the reference's device kernel (src/mhc/_backward.py:106-121 there).
    """
    global _abs_grad_at_zero
    if mode not in _ABS0:
        raise ValueError("mode must be 'zero' or 'plus_one'")
    _abs_grad_at_zero = mode


def get_abs_grad_at_zero() -> str:
    return _abs_grad_at_zero


def sinkhorn_backward(M_orig: torch.Tensor, dP: torch.Tensor, num_iters: int = 20, eps: float = 1e-8) -> torch.Tensor:
    """dM for P = Sinkhorn(|M| + eps), recomputing the forward from M (no saved state)."""
    _check(M_orig.shape[-2:] == (4, 4) and dP.shape == M_orig.shape, "Expected matching (..., 4, 4) tensors")
    L.require_cuda(M_orig, dP)
    M_orig = M_orig.contiguous()
    dP = dP.to(M_orig.dtype).contiguous()
    dM = torch.empty_like(M_orig)
    with torch.cuda.device(M_orig.device):
        L.call("mhc_sinkhorn_bwd", L.stream_of(M_orig), L.ptr(M_orig), L.ptr(dP), L.ptr(dM), M_orig.numel() // 16,
                                          L.dtype_code(M_orig), int(num_iters), float(eps), _ABS0[_abs_grad_at_zero])
    return dM


def add_residual_backward(dH_new: torch.Tensor, branch_output: torch.Tensor, H_post: torch.Tensor,
                          block_dim: int = 128) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """(dH_residual, d_branch_output, dH_post [B,4] fp32).  dH_residual IS dH_new (made
    contiguous if it was not): the identity gradient is aliased, not copied."""
    B, S, n, D = dH_new.shape
    _check(n == 4 and tuple(branch_output.shape) == (B, S, D) and tuple(H_post.shape) == (B, 4), "shape mismatch")
    L.require_cuda(dH_new, branch_output, H_post)
    dH_new = dH_new.contiguous()
    branch_output = branch_output.to(dH_new.dtype).contiguous()
    H_post = L.f32c(H_post)
    d_bo = torch.empty_like(branch_output)
    dH_post = torch.empty(B, 4, device=dH_new.device, dtype=torch.float32)
    buf, nbytes = L.scratch(L.OP_ADD_RESIDUAL_BWD, B, S, D, dH_new)
    with torch.cuda.device(dH_new.device):
        L.call("mhc_add_residual_bwd", L.stream_of(dH_new), L.ptr(dH_new), L.ptr(branch_output), L.ptr(H_post), L.ptr(d_bo),
               L.ptr(dH_post), L.ptr(buf), nbytes, L.tickets(dH_new, B), B, S, D, L.dtype_code(dH_new))
    return dH_new, d_bo, dH_post


def _mix_bwd_inputs(d_branch_input, dH_residual, H):
    B, S, n, D = H.shape
    _check(n == 4 and tuple(d_branch_input.shape) == (B, S, D) and dH_residual.shape == H.shape, "shape mismatch")
    L.require_cuda(d_branch_input, dH_residual, H)
    H = H.contiguous()
    return d_branch_input.to(H.dtype).contiguous(), dH_residual.to(H.dtype).contiguous(), H


def stream_mix_backward(d_branch_input: torch.Tensor, dH_residual: torch.Tensor, H: torch.Tensor,
                        H_pre: torch.Tensor, H_res: torch.Tensor,
                        block_dim: int = 128) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """(dH, dH_pre [B,4] fp32, dH_res [B,4,4] fp32) in one pass over the data."""
    d_bi, dHr, H = _mix_bwd_inputs(d_branch_input, dH_residual, H)
    B, S, _, D = H.shape
    H_pre, H_res = L.f32c(H_pre), L.f32c(H_res)
    dH = torch.empty_like(H)
    dH_pre = torch.empty(B, 4, device=H.device, dtype=torch.float32)
    dH_res = torch.empty(B, 4, 4, device=H.device, dtype=torch.float32)
    buf, nbytes = L.scratch(L.OP_STREAM_MIX_BWD, B, S, D, H)
    with torch.cuda.device(H.device):
        L.call("mhc_stream_mix_bwd", L.stream_of(H), L.ptr(d_bi), L.ptr(dHr), L.ptr(H), L.ptr(H_pre), L.ptr(H_res), L.ptr(dH),
                                            L.ptr(dH_pre), L.ptr(dH_res), L.ptr(buf), nbytes, B, S, D,
                                            L.dtype_code(H))
    return dH, dH_pre, dH_res


def stream_mix_backward_reduce(d_branch_input, dH_residual, H) -> Tuple[torch.Tensor, torch.Tensor]:
    """Only (dH_pre, dH_res): first pass of the two-pass backward."""
    d_bi, dHr, H = _mix_bwd_inputs(d_branch_input, dH_residual, H)
    B, S, _, D = H.shape
    dH_pre = torch.empty(B, 4, device=H.device, dtype=torch.float32)
    dH_res = torch.empty(B, 4, 4, device=H.device, dtype=torch.float32)
    buf, nbytes = L.scratch(L.OP_STREAM_MIX_BWD, B, S, D, H)
    with torch.cuda.device(H.device):
        L.call("mhc_stream_mix_bwd_reduce", L.stream_of(H), L.ptr(d_bi), L.ptr(dHr), L.ptr(H), L.ptr(dH_pre), L.ptr(dH_res),
                                                   L.ptr(buf), nbytes, B, S, D, L.dtype_code(H))
    return dH_pre, dH_res


def stream_mix_backward_apply(d_branch_input, dH_residual, H_pre, H_res, grad_x: Optional[torch.Tensor],
                              like: torch.Tensor, inv_S: Optional[float] = None) -> torch.Tensor:
    """dH = mix-transpose of the upstream gradients + grad_x * inv_S broadcast over the sequence
    (second pass; grad_x is the fp32 [B, 4*D] gradient of the pooled state, or None; inv_S
    defaults to 1 / S of `like` and is 1 / (global sequence length) under sequence sharding)."""
    B, S, _, D = like.shape
    d_bi = d_branch_input.to(like.dtype).contiguous()
    dHr = dH_residual.to(like.dtype).contiguous()
    H_pre, H_res = L.f32c(H_pre), L.f32c(H_res)
    if grad_x is not None:
        _check(tuple(grad_x.shape) == (B, 4 * D), "grad_x shape mismatch")
        grad_x = L.f32c(grad_x)
    dH = torch.empty_like(like, memory_format=torch.contiguous_format)
    with torch.cuda.device(like.device):
        L.call("mhc_stream_mix_bwd_apply", L.stream_of(like), L.ptr(d_bi), L.ptr(dHr), L.ptr(H_pre), L.ptr(H_res), L.ptr(grad_x),
                                                  (1.0 / S) if inv_S is None else float(inv_S), L.ptr(dH), B, S, D, L.dtype_code(like))
    return dH


def fused_dynamic_weights_backward(x, phi, bias, alpha_pre, alpha_post, alpha_res, saved, dH_pre, dH_post, dH_res,
                                   sinkhorn_iters: int = 20, eps: float = 1e-6, param_grads=None):
    """Gradients of fused_dynamic_weights_forward, all fp32:
    (grad_x [B,K], grad_phi [K,24], grad_bias [24], grad_alpha [3] = pre, post, res).

    `param_grads`, if given, is a flat fp32 buffer of K*24 + 27 elements that receives
    grad_phi, grad_bias and grad_alpha back to back (the returned tensors are views of it),
    so that one collective can reduce all replicated-parameter gradients without a pack step.
    """
    B, K = x.shape
    L.require_cuda(x, phi, bias, saved, dH_pre, dH_post, dH_res)
    x, phi, bias = L.f32c(x), L.f32c(phi), L.f32c(bias)
    a = [_alpha_dev(v, x) for v in (alpha_pre, alpha_post, alpha_res)]
    dH_pre, dH_post, dH_res = L.f32c(dH_pre), L.f32c(dH_post), L.f32c(dH_res)
    if param_grads is None:
        param_grads = torch.empty(K * 24 + 27, device=x.device, dtype=torch.float32)
    _check(param_grads.numel() == K * 24 + 27 and param_grads.dtype == torch.float32 and param_grads.is_contiguous(),
           "param_grads must be a contiguous fp32 buffer of K*24 + 27 elements")
    g_phi = param_grads[:K * 24].view(K, 24)
    g_bias = param_grads[K * 24:K * 24 + 24]
    g_alpha = param_grads[K * 24 + 24:]
    grad_x = torch.empty(B, K, device=x.device, dtype=torch.float32)
    buf, nbytes = L.scratch(L.OP_DYNAMIC_WEIGHTS_BWD, B, 0, (K + 3) // 4, x)
    with torch.cuda.device(x.device):
        L.call("mhc_dynamic_weights_bwd", L.stream_of(x), L.ptr(x), L.ptr(phi), L.ptr(bias), L.ptr(a[0]), L.ptr(a[1]), L.ptr(a[2]), L.ptr(saved), L.ptr(dH_pre),
            L.ptr(dH_post), L.ptr(dH_res), L.ptr(grad_x), L.ptr(g_phi), L.ptr(g_bias), L.ptr(g_alpha), L.ptr(buf),
            nbytes, B, K, int(sinkhorn_iters), float(eps), _ABS0[_abs_grad_at_zero], 0)
    return grad_x, g_phi, g_bias, g_alpha


def hc_mix_backward(d_branch_input, dH_residual, dH_post, H, x, phi, H_pre_base, H_post_base, H_res_base,
                    alpha_pre, alpha_post, alpha_res, saved, H_pre, H_res, sinkhorn_iters: int = 20,
                    eps: float = 1e-6, param_grads=None, accumulate: bool = False, ready_event=None):
    """Fused backward of hc_mix_forward in ONE library call.  Returns
    (dH, grad_phi [4D,24], grad_bias [24], grad_alpha [3]) with the last three being views of the
    flat fp32 record `param_grads` (allocated here when not given; layout phi | bias | alpha).
    `ready_event` (a torch.cuda.Event that has been recorded at least once, so that it owns a CUDA
    event) is recorded by the library on the current stream between the kernels that write the
    parameter gradients and the pass that writes dH."""
    B, S, _, D = H.shape
    K = 4 * D
    d_bi, dHr, H = _mix_bwd_inputs(d_branch_input, dH_residual, H)
    L.require_cuda(dH_post, x, phi, saved, H_pre, H_res)
    phi, pre_b, post_b, res_b = L.f32c(phi), L.f32c(H_pre_base), L.f32c(H_post_base), L.f32c(H_res_base)
    a = [_alpha_dev(v, H) for v in (alpha_pre, alpha_post, alpha_res)]
    dH_post = L.f32c(dH_post)
    if param_grads is None:
        param_grads = torch.empty(K * 24 + 27, device=H.device, dtype=torch.float32)
        accumulate = False
    _check(param_grads.numel() == K * 24 + 27 and param_grads.dtype == torch.float32 and param_grads.is_contiguous(),
           "param_grads must be a contiguous fp32 buffer of 4*D*24 + 27 elements")
    g_phi = param_grads[:K * 24].view(K, 24)
    g_bias = param_grads[K * 24:K * 24 + 24]
    g_alpha = param_grads[K * 24 + 24:]
    dH = torch.empty_like(H)
    small = torch.empty(B * (K + 20), device=H.device, dtype=torch.float32)
    grad_x, dH_pre, dH_res = small[:B * K], small[B * K:B * K + 4 * B], small[B * K + 4 * B:]
    buf, nbytes = L.scratch(L.OP_HC_MIX_BWD, B, S, D, H)
    with torch.cuda.device(H.device):
        L.call("mhc_hc_mix_bwd", L.stream_of(H), L.ptr(d_bi), L.ptr(dHr), L.ptr(dH_post), L.ptr(H), L.ptr(x), L.ptr(phi),
               L.ptr(pre_b), L.ptr(post_b), L.ptr(res_b), L.ptr(a[0]), L.ptr(a[1]), L.ptr(a[2]), L.ptr(saved),
               L.ptr(H_pre), L.ptr(H_res), L.ptr(dH), L.ptr(g_phi), L.ptr(g_bias), L.ptr(g_alpha), L.ptr(grad_x),
               L.ptr(dH_pre), L.ptr(dH_res), L.ptr(buf), nbytes, L.tickets(H, B),
               (ready_event.cuda_event or None) if ready_event is not None else None, B, S, D, L.dtype_code(H),
               int(sinkhorn_iters), float(eps), _ABS0[_abs_grad_at_zero], 1 if accumulate else 0)
    return dH, g_phi, g_bias, g_alpha
