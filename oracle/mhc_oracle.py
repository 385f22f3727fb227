"""CPU oracle for the mHC hyper-connection hot path.

TEST INFRASTRUCTURE ONLY.  This file is a CPU restatement (plain PyTorch tensor
algebra, any float dtype, fp64 capable) of the reference algorithm.  It is the
checker that the parity tests, the smoke test and the benchmark's CPU-baseline
leg compare against or time.  Nothing in the shipped package imports it, and
the shipped package has no CPU path of its own.

Parity status: PINNED.  Every function below is checked against fixtures that
were produced by importing the reference's own pure-PyTorch implementation
(src/mhc/_torch_baseline.py) -- see tests/golden/make_golden.py and
tests/test_oracle_golden.py -- and against the tolerances the reference's own
tests state (tests/test_mhc.py:25-160).

Each function cites the reference lines it restates (paths are relative to the
reference project root).

Index convention of the 24 projected values (src/mhc/_kernels.py:496-522):
  0..3  -> pre-mix weights, 4..7 -> post-distribution weights,
  8..23 -> residual mixing matrix, row-major 4x4.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Optional

import torch

N_STREAMS = 4
N_OUT = N_STREAMS * N_STREAMS + 2 * N_STREAMS  # 24


# ---------------------------------------------------------------------------
# Sinkhorn-Knopp
# ---------------------------------------------------------------------------
def sinkhorn(M: torch.Tensor, iters: int = 20, eps: float = 1e-8) -> torch.Tensor:
    """Alternate row / column normalisation of |M| + eps.

    Restates src/mhc/_torch_baseline.py:26-35 (same arithmetic as the device
    kernel src/mhc/_kernels.py:75-125): the magnitude is taken first, eps is
    added to the start matrix AND to every row / column sum, and one iteration
    is "divide rows by their sums, then divide columns by their sums".
    """
    P = torch.abs(M) + eps
    for _ in range(iters):
        P = P / (P.sum(-1, keepdim=True) + eps)
        P = P / (P.sum(-2, keepdim=True) + eps)
    return P


def sinkhorn_grad(
    M: torch.Tensor,
    dP: torch.Tensor,
    iters: int = 20,
    eps: float = 1e-8,
    sign_of_zero: float = 0.0,
) -> torch.Tensor:
    """Closed-form gradient of `sinkhorn` with respect to M.

    Restates the backward recurrence of src/mhc/_backward.py:142-244.  For a
    normalisation y = x / (sum(x) + eps) along an axis, the pull-back is
    dx = (dy - <dy, y>) / (sum(x) + eps) along that axis.  The recurrence walks
    the iterations in reverse, column step first, then row step.

    `sign_of_zero` selects d|m|/dm at m == 0: 0.0 is what autograd of
    src/mhc/_torch_baseline.py:27 yields; +1.0 is what the device kernel of the
    reference uses (src/mhc/_backward.py:106-121).
    """
    P = torch.abs(M) + eps
    saved = []
    for _ in range(iters):
        r = P.sum(-1, keepdim=True) + eps
        Pr = P / r
        c = Pr.sum(-2, keepdim=True) + eps
        P = Pr / c
        saved.append((r, Pr, c, P))
    d = dP
    for r, Pr, c, Pc in reversed(saved):
        d = (d - (d * Pc).sum(-2, keepdim=True)) / c
        d = (d - (d * Pr).sum(-1, keepdim=True)) / r
    sgn = torch.sign(M)
    if sign_of_zero != 0.0:
        sgn = torch.where(M == 0, torch.full_like(M, sign_of_zero), sgn)
    return d * sgn


# ---------------------------------------------------------------------------
# Dynamic weights (projection + RMS norm + activations + Sinkhorn)
# ---------------------------------------------------------------------------
def dynamic_weights(
    x: torch.Tensor,
    phi: torch.Tensor,
    bias: torch.Tensor,
    alpha_pre: torch.Tensor,
    alpha_post: torch.Tensor,
    alpha_res: torch.Tensor,
    iters: int = 20,
    eps: float = 1e-6,
):
    """Pooled state -> (H_pre [B,4], H_post [B,4], H_res [B,4,4]).

    Restates src/mhc/_torch_baseline.py:72-111 (device form:
    src/mhc/_kernels.py:413-579).  One eps value is used in the RMS, in the
    pre-mix normaliser and throughout the Sinkhorn projection.
    """
    B, K = x.shape
    proj = x @ phi                                               # [B,24]
    inv_rms = 1.0 / torch.sqrt((x * x).sum(-1, keepdim=True) / K + eps)
    gain = torch.cat([
        alpha_pre.reshape(1).expand(N_STREAMS),
        alpha_post.reshape(1).expand(N_STREAMS),
        alpha_res.reshape(1).expand(N_STREAMS * N_STREAMS),
    ])
    s = inv_rms * gain * proj + bias                             # [B,24]
    sig_pre = torch.sigmoid(s[:, 0:4])
    H_pre = sig_pre / (sig_pre.sum(-1, keepdim=True) + eps)
    H_post = 2.0 * torch.sigmoid(s[:, 4:8])
    H_res = sinkhorn(s[:, 8:24].reshape(B, 4, 4), iters, eps)
    return H_pre, H_post, H_res


# ---------------------------------------------------------------------------
# Streaming ops
# ---------------------------------------------------------------------------
def stream_mix(H: torch.Tensor, H_pre: torch.Tensor, H_res: torch.Tensor):
    """(branch_input [B,S,D], H_residual [B,S,4,D]).

    Restates src/mhc/_torch_baseline.py:135-143 / src/mhc/_kernels.py:203-230:
      branch_input[b,s,d]  = sum_n H_pre[b,n]   * H[b,s,n,d]
      H_residual[b,s,n,d]  = sum_m H_res[b,n,m] * H[b,s,m,d]
    """
    bi = (H * H_pre[:, None, :, None]).sum(2)
    Hr = (H_res[:, None, :, :, None] * H[:, :, None, :, :]).sum(3)
    return bi, Hr


def add_residual(H_residual: torch.Tensor, branch_output: torch.Tensor, H_post: torch.Tensor):
    """H_new[b,s,n,d] = H_residual[b,s,n,d] + H_post[b,n] * branch_output[b,s,d].

    Restates src/mhc/_torch_baseline.py:160-166 / src/mhc/_kernels.py:307-310.
    """
    return H_residual + H_post[:, None, :, None] * branch_output[:, :, None, :]


# ---------------------------------------------------------------------------
# Whole layer
# ---------------------------------------------------------------------------
@dataclass
class LayerParams:
    """Parameters of one hyper-connection layer, reference names and shapes
    (src/mhc/module.py:67-101)."""

    H_post_base: torch.Tensor            # [4]
    H_pre_base: torch.Tensor             # [4]
    H_res_base: torch.Tensor             # [4,4]
    phi: Optional[torch.Tensor] = None   # [4D,24]   (fused dynamic)
    alpha_pre: Optional[torch.Tensor] = None   # [1]
    alpha_post: Optional[torch.Tensor] = None  # [1]
    alpha_res: Optional[torch.Tensor] = None   # [1]
    W_post: Optional[torch.Tensor] = None      # [4,4D]   (unfused dynamic; Linear.weight)
    W_pre: Optional[torch.Tensor] = None       # [4,4D]
    W_res: Optional[torch.Tensor] = None       # [16,4D]
    scale_post: Optional[torch.Tensor] = None  # [1]
    scale_pre: Optional[torch.Tensor] = None
    scale_res: Optional[torch.Tensor] = None

    def tensors(self) -> Dict[str, torch.Tensor]:
        return {k: v for k, v in self.__dict__.items() if v is not None}

    def to(self, dtype) -> "LayerParams":
        return LayerParams(**{k: v.detach().clone().to(dtype) for k, v in self.tensors().items()})


def default_params(dim: int, layer_idx: int = 0, init_scale: float = 0.1,
                   mode: str = "fused", dtype=torch.float32) -> LayerParams:
    """Initial values as in src/mhc/module.py:67-101."""
    n = N_STREAMS
    pre = torch.zeros(n, dtype=dtype)
    pre[layer_idx % n] = 1.0
    p = LayerParams(torch.ones(n, dtype=dtype), pre, torch.eye(n, dtype=dtype))
    if mode == "fused":
        p.phi = torch.zeros(n * dim, N_OUT, dtype=dtype)
        p.alpha_pre = torch.tensor([init_scale], dtype=dtype)
        p.alpha_post = torch.tensor([init_scale], dtype=dtype)
        p.alpha_res = torch.tensor([init_scale], dtype=dtype)
    elif mode == "unfused":
        p.W_post = torch.zeros(n, n * dim, dtype=dtype)
        p.W_pre = torch.zeros(n, n * dim, dtype=dtype)
        p.W_res = torch.zeros(n * n, n * dim, dtype=dtype)
        p.scale_post = torch.tensor([init_scale], dtype=dtype)
        p.scale_pre = torch.tensor([init_scale], dtype=dtype)
        p.scale_res = torch.tensor([init_scale], dtype=dtype)
    elif mode != "static":
        raise ValueError(mode)
    return p


def layer_weights(p: LayerParams, H: torch.Tensor, mode: str = "fused",
                  iters: int = 20, eps: float = 1e-6):
    """(H_pre, H_post, H_res) for the three modes of the reference module.

    fused    : src/mhc/module.py:119-139 (mean over the sequence axis first)
    static   : src/mhc/module.py:106-117 (plain sigmoid for H_post, literal 1e-8)
    unfused  : src/mhc/module.py:141-163 (manual RMS norm, three linear maps)
    """
    B, S, n, D = H.shape
    if mode == "static":
        H_post = torch.sigmoid(p.H_post_base)[None].expand(B, -1)
        sp = torch.sigmoid(p.H_pre_base)
        H_pre = (sp / (sp.sum() + 1e-8))[None].expand(B, -1)
        H_res = sinkhorn(p.H_res_base[None].expand(B, -1, -1), iters, 1e-8)
        return H_pre, H_post, H_res
    x = H.mean(1).reshape(B, n * D)
    if mode == "fused":
        bias = torch.cat([p.H_pre_base, p.H_post_base, p.H_res_base.reshape(-1)])
        return dynamic_weights(x, p.phi, bias, p.alpha_pre, p.alpha_post, p.alpha_res, iters, eps)
    xn = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    d_post = (xn @ p.W_post.T) * p.scale_post
    d_pre = (xn @ p.W_pre.T) * p.scale_pre
    d_res = (xn @ p.W_res.T).reshape(B, n, n) * p.scale_res
    H_post = torch.sigmoid(p.H_post_base + d_post)
    sp = torch.sigmoid(p.H_pre_base + d_pre)
    H_pre = sp / (sp.sum(-1, keepdim=True) + 1e-8)
    H_res = sinkhorn(p.H_res_base + d_res, iters, 1e-8)
    return H_pre, H_post, H_res


def layer_forward(p: LayerParams, H: torch.Tensor, branch: Optional[Callable] = None,
                  mode: str = "fused", iters: int = 20, eps: float = 1e-6):
    """One layer: weights -> mix -> branch -> add (src/mhc/module.py:165-182).
    Returns (branch_input, H_new)."""
    H_pre, H_post, H_res = layer_weights(p, H, mode, iters, eps)
    bi, Hr = stream_mix(H, H_pre, H_res)
    bo = bi if branch is None else branch(bi)
    return bi, add_residual(Hr, bo, H_post)


def layer_fwd_bwd(p: LayerParams, H: torch.Tensor, g: torch.Tensor,
                  branch: Optional[Callable] = None, mode: str = "fused",
                  iters: int = 20, eps: float = 1e-6, dtype=None) -> Dict[str, torch.Tensor]:
    """Forward + backward of one layer with upstream gradient g on H_new.

    Gradients come from autograd through the restated forward, exactly how the
    reference obtains them for its CPU path.  `dtype` (e.g. torch.float64)
    re-runs the same algebra at another precision: the fp64 run is the arbiter
    when fp32 summation-order noise exceeds a stated tolerance.
    Returns branch_input, H_new, dH and one "d<name>" entry per parameter.
    """
    if dtype is not None:
        p, H, g = p.to(dtype), H.to(dtype), g.to(dtype)
    leaves = {k: v.detach().clone().requires_grad_(True) for k, v in p.tensors().items()}
    Hl = H.detach().clone().requires_grad_(True)
    bi, H_new = layer_forward(LayerParams(**leaves), Hl, branch, mode, iters, eps)
    H_new.backward(g)
    out = {"branch_input": bi.detach(), "H_new": H_new.detach(), "dH": Hl.grad}
    for k, v in leaves.items():
        out["d" + k] = v.grad if v.grad is not None else torch.zeros_like(v)
    return out
