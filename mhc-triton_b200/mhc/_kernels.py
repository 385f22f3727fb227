"""Forward launch wrappers: validate, allocate outputs with torch, call the C ABI.

Names and signatures follow the launch wrappers of the reference
(src/mhc/_kernels.py:597-752 there); `block_dim` is accepted and ignored because the
tiling is fixed inside the CUDA kernels.
"""

from typing import Tuple

import torch

from . import _lib as L


def _check(cond, msg):
    if not cond:
        raise AssertionError(msg)


def sinkhorn_forward(M: torch.Tensor, num_iters: int = 20, eps: float = 1e-8) -> torch.Tensor:
    """P = Sinkhorn(|M| + eps) for M of shape (..., 4, 4); same dtype as M."""
    _check(M.shape[-2:] == (4, 4), "Expected (..., 4, 4)")
    L.require_cuda(M)
    M = M.contiguous()
    P = torch.empty_like(M)
    with torch.cuda.device(M.device):
        L.call("mhc_sinkhorn_fwd", L.stream_of(M), L.ptr(M), L.ptr(P), M.numel() // 16, L.dtype_code(M), int(num_iters),
                                          float(eps))
    return P


def stream_mix_forward(H: torch.Tensor, H_pre: torch.Tensor, H_res: torch.Tensor,
                       block_dim: int = 128, want_residual: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """(branch_input [B,S,D], H_residual [B,S,4,D]) in H's dtype; with want_residual=False the
    residual mix is not written and None is returned in its place."""
    _check(H.dim() == 4, "H must be [batch, seq, 4, dim]")
    B, S, n, D = H.shape
    _check(n == 4, "num_streams must be 4")
    _check(tuple(H_pre.shape) == (B, 4), f"H_pre shape mismatch: {tuple(H_pre.shape)} vs ({B}, 4)")
    _check(tuple(H_res.shape) == (B, 4, 4), f"H_res shape mismatch: {tuple(H_res.shape)} vs ({B}, 4, 4)")
    L.require_cuda(H, H_pre, H_res)
    H = H.contiguous()
    H_pre, H_res = L.f32c(H_pre), L.f32c(H_res)
    bi = torch.empty(B, S, D, device=H.device, dtype=H.dtype)
    Hr = torch.empty_like(H) if want_residual else None
    with torch.cuda.device(H.device):
        L.call("mhc_stream_mix_fwd", L.stream_of(H), L.ptr(H), L.ptr(H_pre), L.ptr(H_res), L.ptr(bi), L.ptr(Hr), B, S, D,
                                            L.dtype_code(H))
    return bi, Hr


def add_residual_forward(H_residual: torch.Tensor, branch_output: torch.Tensor, H_post: torch.Tensor,
                         block_dim: int = 128, pool: bool = False):
    """H_new = H_residual + H_post[:, None, :, None] * branch_output[:, :, None, :].
    With pool=True returns (H_new, partials): partials [B, chunks, 4*D] fp32 are the token sums of
    H_new per chunk, which the next layer's fused forward accepts in place of its own pooling pass."""
    _check(H_residual.dim() == 4, "H_residual must be [batch, seq, 4, dim]")
    B, S, n, D = H_residual.shape
    _check(n == 4, "num_streams must be 4")
    _check(tuple(branch_output.shape) == (B, S, D), "branch_output shape mismatch")
    _check(tuple(H_post.shape) == (B, 4), "H_post shape mismatch")
    L.require_cuda(H_residual, branch_output, H_post)
    H_residual = H_residual.contiguous()
    branch_output = branch_output.to(H_residual.dtype).contiguous()
    H_post = L.f32c(H_post)
    H_new = torch.empty_like(H_residual)
    if pool:
        chunks = L.load().mhc_add_residual_pool_chunks(S, D)
        partials = torch.empty(B, chunks, 4 * D, device=H_residual.device, dtype=torch.float32)
        with torch.cuda.device(H_residual.device):
            L.call("mhc_add_residual_pool_fwd", L.stream_of(H_residual), L.ptr(H_residual), L.ptr(branch_output),
                   L.ptr(H_post), L.ptr(H_new), L.ptr(partials), B, S, D, L.dtype_code(H_residual))
        return H_new, partials
    with torch.cuda.device(H_residual.device):
        L.call("mhc_add_residual_fwd", L.stream_of(H_residual), L.ptr(H_residual), L.ptr(branch_output), L.ptr(H_post), L.ptr(H_new),
                                              B, S, D, L.dtype_code(H_residual))
    return H_new


def meanpool_forward(H: torch.Tensor) -> torch.Tensor:
    """x[b, n*D+d] = mean_s H[b,s,n,d] as fp32 [B, 4*D] (fp32 accumulation, fixed order)."""
    _check(H.dim() == 4 and H.shape[2] == 4, "H must be [batch, seq, 4, dim]")
    B, S, _, D = H.shape
    _check(S > 0, "empty sequence")
    L.require_cuda(H)
    H = H.contiguous()
    x = torch.empty(B, 4 * D, device=H.device, dtype=torch.float32)
    buf, nbytes = L.scratch(L.OP_MEANPOOL_FWD, B, S, D, H)
    with torch.cuda.device(H.device):
        L.call("mhc_meanpool_fwd", L.stream_of(H), L.ptr(H), L.ptr(x), L.ptr(buf), nbytes, B, S, D, L.dtype_code(H))
    return x


last_dynamic_weights_scratch = None


def _alpha_dev(a, like: torch.Tensor) -> torch.Tensor:
    """A scale as a one-element fp32 device tensor (Python floats are uploaded without a sync)."""
    if torch.is_tensor(a):
        _check(a.numel() == 1, "alpha must have one element")
        L.require_cuda(a)
        return L.f32c(a.reshape(1))
    return torch.full((1,), float(a), device=like.device, dtype=torch.float32)


def fused_dynamic_weights_forward(x: torch.Tensor, phi: torch.Tensor, bias: torch.Tensor, alpha_pre, alpha_post,
                                  alpha_res, sinkhorn_iters: int = 20, eps: float = 1e-6, return_saved: bool = False):
    """(H_pre [B,4], H_post [B,4], H_res [B,4,4]), always fp32.

    alpha_* may be Python floats (as in the reference signature) or one-element device
    tensors; tensors are read on the device, so no host synchronisation happens.
    With return_saved=True a fourth tensor [B,32] with the raw projections, sum(x^2) and
    inv_rms is returned for the backward.
    """
    _check(x.dim() == 2, "x must be [batch, in_dim]")
    B, K = x.shape
    _check(tuple(phi.shape) == (K, 24), f"phi shape mismatch: {tuple(phi.shape)} vs ({K}, 24)")
    _check(tuple(bias.shape) == (24,), f"bias shape mismatch: {tuple(bias.shape)} vs (24,)")
    L.require_cuda(x, phi, bias)
    x, phi, bias = L.f32c(x), L.f32c(phi), L.f32c(bias)
    a = [_alpha_dev(v, x) for v in (alpha_pre, alpha_post, alpha_res)]
    H_pre = torch.empty(B, 4, device=x.device, dtype=torch.float32)
    H_post = torch.empty(B, 4, device=x.device, dtype=torch.float32)
    H_res = torch.empty(B, 4, 4, device=x.device, dtype=torch.float32)
    saved = torch.empty(B, 32, device=x.device, dtype=torch.float32)
    buf, nbytes = L.scratch(L.OP_DYNAMIC_WEIGHTS_FWD, B, 0, (K + 3) // 4, x)
    global last_dynamic_weights_scratch
    last_dynamic_weights_scratch = buf     # its first int is the status word of the many-rows kernels (0 = fine)
    with torch.cuda.device(x.device):
        L.call("mhc_dynamic_weights_fwd", L.stream_of(x), L.ptr(x), L.ptr(phi), L.ptr(bias), L.ptr(a[0]), L.ptr(a[1]),
                                                 L.ptr(a[2]), L.ptr(H_pre), L.ptr(H_post), L.ptr(H_res), L.ptr(saved),
                                                 L.ptr(buf), nbytes, B, K, int(sinkhorn_iters), float(eps))
    if return_saved:
        return H_pre, H_post, H_res, saved
    return H_pre, H_post, H_res


def hc_mix_forward(H, H_pre_base, H_post_base, H_res_base, phi, alpha_pre, alpha_post, alpha_res,
                   sinkhorn_iters: int = 20, eps: float = 1e-6, pooled=None, want_residual: bool = True):
    """Fused forward of the module's dynamic path in ONE library call: sequence mean-pool,
    dynamic weights, stream mix.  Returns
    (branch_input, H_residual, H_post, H_pre, H_res, x, saved); x [B,4D] and saved [B,32]
    are what the fused backward needs.  `pooled` ([B, chunks, 4D] fp32 token sums of H from the
    previous layer's add_residual_forward(pool=True)) replaces the pooling pass over H.  With
    want_residual=False H_residual is not written (returned as None): the caller adds the residual
    with add_residual_mix_forward, which recomputes the mix from H."""
    _check(H.dim() == 4 and H.shape[2] == 4, "H must be [batch, seq, 4, dim]")
    B, S, _, D = H.shape
    _check(S > 0 and D > 0, "empty sequence or width")
    _check(tuple(phi.shape) == (4 * D, 24), f"phi shape mismatch: {tuple(phi.shape)} vs ({4 * D}, 24)")
    _check(H_pre_base.numel() == 4 and H_post_base.numel() == 4 and H_res_base.numel() == 16, "base parameter shapes")
    L.require_cuda(H, phi, H_pre_base, H_post_base, H_res_base)
    H = H.contiguous()
    phi, pre_b, post_b, res_b = L.f32c(phi), L.f32c(H_pre_base), L.f32c(H_post_base), L.f32c(H_res_base)
    a = [_alpha_dev(v, H) for v in (alpha_pre, alpha_post, alpha_res)]
    dev = H.device
    small = torch.empty(B * 56, device=dev, dtype=torch.float32)   # one allocation for the small outputs
    H_pre, H_post = small[:4 * B].view(B, 4), small[4 * B:8 * B].view(B, 4)
    H_res, saved = small[8 * B:24 * B].view(B, 4, 4), small[24 * B:].view(B, 32)
    x = torch.empty(B, 4 * D, device=dev, dtype=torch.float32)
    bi = torch.empty(B, S, D, device=dev, dtype=H.dtype)
    Hr = torch.empty_like(H) if want_residual else None
    buf, nbytes = L.scratch(L.OP_HC_MIX_FWD, B, S, D, H)
    chunks = 0
    if pooled is not None:
        _check(pooled.dim() == 3 and pooled.shape[0] == B and pooled.shape[2] == 4 * D and pooled.dtype == torch.float32
               and pooled.is_contiguous() and pooled.device == dev, "pooled must be contiguous fp32 [B, chunks, 4*D]")
        chunks = pooled.shape[1]
    with torch.cuda.device(dev):
        L.call("mhc_hc_mix_fwd", L.stream_of(H), L.ptr(H), L.ptr(phi), L.ptr(pre_b), L.ptr(post_b), L.ptr(res_b),
               L.ptr(a[0]), L.ptr(a[1]), L.ptr(a[2]), L.ptr(x), L.ptr(H_pre), L.ptr(H_post), L.ptr(H_res), L.ptr(saved),
               L.ptr(bi), L.ptr(Hr), L.ptr(pooled), chunks, L.ptr(buf), nbytes, L.tickets(H, B), B, S, D,
               L.dtype_code(H), int(sinkhorn_iters), float(eps))
    return bi, Hr, H_post, H_pre, H_res, x, saved


def add_residual_mix_forward(H: torch.Tensor, H_res: torch.Tensor, branch_output: torch.Tensor, H_post: torch.Tensor,
                             pool: bool = False):
    """H_new = H_res @ H (over the stream axis) + H_post * branch_output in one kernel: the residual
    mix is recomputed from H instead of being read from a materialised H_residual.  With pool=True
    returns (H_new, partials) as add_residual_forward does."""
    _check(H.dim() == 4 and H.shape[2] == 4, "H must be [batch, seq, 4, dim]")
    B, S, _, D = H.shape
    _check(tuple(branch_output.shape) == (B, S, D), "branch_output shape mismatch")
    _check(tuple(H_post.shape) == (B, 4) and tuple(H_res.shape) == (B, 4, 4), "weight shape mismatch")
    L.require_cuda(H, H_res, branch_output, H_post)
    H = H.contiguous()
    branch_output = branch_output.to(H.dtype).contiguous()
    H_post, H_res = L.f32c(H_post), L.f32c(H_res)
    H_new = torch.empty_like(H)
    partials = None
    if pool:
        chunks = L.load().mhc_add_residual_pool_chunks(S, D)
        partials = torch.empty(B, chunks, 4 * D, device=H.device, dtype=torch.float32)
    with torch.cuda.device(H.device):
        L.call("mhc_add_residual_mix_fwd", L.stream_of(H), L.ptr(H), L.ptr(H_res), L.ptr(branch_output), L.ptr(H_post),
               L.ptr(H_new), L.ptr(partials), B, S, D, L.dtype_code(H))
    return (H_new, partials) if pool else H_new
