"""Full-size configurations: properties that do not need an oracle over the whole tensor, plus an
oracle check on one batch element (batch elements are independent in this layer).

config 2: 2**20 fp32 4x4 matrices, 20 iterations, forward + backward.
config 4: bf16 H(8, 4096, 4, 4096), phi [16384, 24] ~ N(0, 0.02^2), identity branch.
"""

import pytest
import torch

from oracle import mhc_oracle as O
from tests.util import assert_close, assert_close_norm, to_module

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_config2_sinkhorn_one_million_matrices():
    from mhc import sinkhorn_knopp
    torch.manual_seed(0)
    N = 2 ** 20
    M = torch.randn(N, 4, 4)
    dP = torch.randn(N, 4, 4)
    for name, Min in (("logits", M), ("exp(logits)", torch.exp(M))):
        Md = Min.to(DEV).requires_grad_(True)
        P = sinkhorn_knopp(Md, 20, 1e-8)
        P.backward(dP.to(DEV))
        # the last step is a column normalisation: column sums are 1 for every matrix
        assert (P.sum(-2) - 1).abs().max() < 1e-5, name
        assert (P >= 0).all() and torch.isfinite(Md.grad).all()
        idx = torch.arange(0, N, 257)
        Pref = O.sinkhorn(Min[idx].double(), 20, 1e-8)
        assert_close(P[idx], Pref, 1e-5, 1e-6, name + " P")
        # row sums equal the oracle's (20 iterations do not always converge to 1)
        assert (P[idx].sum(-1).cpu().double() - Pref.sum(-1)).abs().max() < 1e-5
        dref = O.sinkhorn_grad(Min[idx].double(), dP[idx].double(), 20, 1e-8)
        got = Md.grad[idx].cpu().double()
        err = (got - dref).abs().reshape(len(idx), -1).max(-1).values
        scale = dref.abs().reshape(len(idx), -1).max(-1).values
        assert (err <= 1e-5 + 1e-4 * scale).all(), (name, float((err / (1e-5 + 1e-4 * scale)).max()))
        # gradients are orthogonal to rescaling M: sum(M * dM) = 0 for a scale-invariant map (eps aside)
        inv = (Md.grad * Md.detach()).sum((-1, -2)).abs().cpu()
        assert (inv[idx] <= 1e-3 * (Md.grad.abs() * Md.detach().abs()).sum((-1, -2)).cpu()[idx] + 1e-4).all(), name


def _c4_inputs(B=8, S=4096, D=4096):
    gen = torch.Generator(device=DEV).manual_seed(0)
    H = torch.cat([torch.randn(1, S, 4, D, device=DEV, generator=gen).bfloat16() for _ in range(B)])
    g = torch.cat([torch.randn(1, S, 4, D, device=DEV, generator=gen).bfloat16() for _ in range(B)])
    return H, g


def test_config4_identity_weights_are_exact_copies():
    from mhc import fused_add_residual, fused_stream_mix
    H, _ = _c4_inputs()
    B = H.shape[0]
    H_pre = torch.zeros(B, 4, device=DEV); H_pre[:, 2] = 1.0
    H_res = torch.eye(4, device=DEV).expand(B, 4, 4).contiguous()
    bi, Hr = fused_stream_mix(H, H_pre, H_res)
    assert torch.equal(bi, H[:, :, 2]) and torch.equal(Hr, H)
    H_new = fused_add_residual(Hr, bi, torch.zeros(B, 4, device=DEV))
    assert torch.equal(H_new, H)
    # a permutation matrix permutes the streams
    perm = torch.tensor([3, 0, 1, 2], device=DEV)
    Pm = torch.zeros(4, 4, device=DEV); Pm[torch.arange(4, device=DEV), perm] = 1.0
    _, Hr = fused_stream_mix(H, H_pre, Pm.expand(B, 4, 4).contiguous())
    assert torch.equal(Hr, H[:, :, perm])


def _layer_against_oracle_on_one_batch_element(B, S, D, b):
    from mhc import HyperConnection
    from tests.test_gpu_parity import _oracle_with_storage_rounding
    H, g = _c4_inputs(B, S, D)
    p = O.default_params(D, 0, 0.1)
    gen = torch.Generator().manual_seed(0)
    p.phi.copy_((torch.randn(24, 4 * D, generator=gen) * 0.02).T)
    hc = to_module(HyperConnection(dim=D), p).to(DEV)
    Hd = H.requires_grad_(True)
    bi, add = hc(Hd)
    H_new = add(bi)
    H_new.backward(g)
    torch.cuda.synchronize()
    # the same element alone gives bit-identical activations (reduction layout independent of the batch)
    H1 = H[b:b + 1].detach().clone().requires_grad_(True)
    for q in hc.parameters():
        q.grad = None
    bi1, add1 = hc(H1)
    H_new1 = add1(bi1)
    H_new1.backward(g[b:b + 1])
    assert torch.equal(bi1, bi[b:b + 1]) and torch.equal(H_new1, H_new[b:b + 1]) and torch.equal(H1.grad, Hd.grad[b:b + 1])
    # oracle (fp32 math on the up-cast bf16 values) on that element: rtol 2e-2
    torch.set_num_threads(max(1, torch.get_num_threads()))
    Hc, gc = H[b:b + 1].detach().cpu(), g[b:b + 1].cpu()
    ref = O.layer_fwd_bwd(p, Hc.float(), gc.float(), None, "fused")
    assert_close_norm(bi1, ref["branch_input"], 2e-2, 0, "branch_input")
    assert_close_norm(H_new1, ref["H_new"], 2e-2, 0, "H_new")
    assert_close_norm(H1.grad, ref["dH"], 2e-2, 0, "dH")
    for n, q in hc.named_parameters():
        if not n.startswith("alpha"):
            assert_close_norm(q.grad, ref["d" + n], 2e-2, 1e-6, n)
    del ref
    # The three scale gradients are sums of 4 / 4 / 16 signed terms that largely cancel, so they are
    # checked against the fp64 oracle that rounds the activations where the device stores them (the
    # only roundings the device path has), at the same 2e-2.
    ref_r = _oracle_with_storage_rounding(p, Hc, gc, lambda t: t, torch.bfloat16)
    for n, q in hc.named_parameters():
        if n.startswith("alpha"):
            assert_close_norm(q.grad, ref_r["d" + n], 2e-2, 1e-6, n + " (storage-rounded oracle)")


def test_config4_layer_against_oracle_on_one_batch_element():
    _layer_against_oracle_on_one_batch_element(8, 4096, 4096, 5)


def test_config5_width_layer_against_oracle_on_one_batch_element():
    """The per-GPU shape of config 5 (two sequences of 4096 tokens, D = 7168, one layer)."""
    _layer_against_oracle_on_one_batch_element(2, 4096, 7168, 1)


def test_config3_layer_with_linear_branch_on_one_batch_element():
    """config 3: bf16 H(8, 4096, 4, 2048), branch = bf16 Linear(2048 -> 2048), fwd + bwd; one batch
    element against the fp64 oracle on the up-cast values (rtol 2e-2, norm-wise)."""
    from mhc import HyperConnection
    B, S, D = 8, 4096, 2048
    H, g = _c4_inputs(B, S, D)
    p = O.default_params(D, 0, 0.1)
    gen = torch.Generator().manual_seed(0)
    p.phi.copy_((torch.randn(24, 4 * D, generator=gen) * 0.02).T)
    hc = to_module(HyperConnection(dim=D), p).to(DEV)
    torch.manual_seed(0)
    lin = torch.nn.Linear(D, D).bfloat16()
    lin_d = torch.nn.Linear(D, D).bfloat16()
    lin_d.load_state_dict(lin.state_dict())
    lin_d = lin_d.to(DEV)
    Hd = H.requires_grad_(True)
    bi, add = hc(Hd)
    H_new = add(lin_d(bi))
    H_new.backward(g)
    torch.cuda.synchronize()
    b = 2
    W, bias = lin.weight.detach().double(), lin.bias.detach().double()
    ref = O.layer_fwd_bwd(p, H[b:b + 1].detach().float().cpu(), g[b:b + 1].float().cpu(),
                          lambda t: t @ W.T + bias, "fused", dtype=torch.float64)
    assert_close_norm(bi[b:b + 1], ref["branch_input"], 2e-2, 0, "branch_input")
    assert_close_norm(H_new[b:b + 1], ref["H_new"], 2e-2, 0, "H_new")
    assert_close_norm(Hd.grad[b:b + 1], ref["dH"], 2e-2, 0, "dH")
