"""The CPU oracle against fixtures produced by the reference's own PyTorch code.

Tolerances: forward values follow the reference's tests (tests/test_mhc.py:35,88-89,136
in the reference: 1e-5 / 1e-4 absolute); everything else uses rtol 1e-5 / atol 1e-6 in
fp32, and 1e-10 when both sides ran in fp64.
"""

import torch

from oracle import mhc_oracle as O
from tests import cases


def close(a, b, rtol=1e-5, atol=1e-6):
    assert a.shape == b.shape, (a.shape, b.shape)
    assert torch.allclose(a, b, rtol=rtol, atol=atol), float((a - b).abs().max())


def test_sinkhorn_forward_and_grads(golden):
    g = golden("sinkhorn.npz")
    close(O.sinkhorn(g["M"], 20, 1e-8), g["P"])
    close(O.sinkhorn(g["M8"], 20, 1e-8), g["P8"])
    close(O.sinkhorn(g["M"].double(), 20, 1e-8), g["P_f64"], 1e-12, 1e-14)
    close(O.sinkhorn_grad(g["M"], g["dP"], 20, 1e-8), g["dM"], 1e-4, 1e-5)
    close(O.sinkhorn_grad(g["M"].double(), g["dP"].double(), 20, 1e-8), g["dM_f64"], 1e-9, 1e-12)
    ones = torch.ones_like(g["M"])
    assert (O.sinkhorn_grad(g["M"], ones, 20, 1e-8) - g["dM_sumloss"]).abs().max() < 1e-4


def test_sinkhorn_zero_and_sign_cases(golden):
    g = golden("sinkhorn.npz")
    for T in (1, 5, 20):
        close(O.sinkhorn(g["Mz"], T, 1e-6), g[f"Pz_T{T}"])
        dM = O.sinkhorn_grad(g["Mz"].double(), g["dPz"].double(), T, 1e-6).float()
        ref = g[f"dMz_T{T}"]
        assert (dM - ref).abs().max() <= 1e-6 + 1e-4 * ref.abs().max()
        # autograd convention: exact zeros in M receive zero gradient
        assert (dM[g["Mz"] == 0] == 0).all()


def test_sinkhorn_autograd_matches_closed_form():
    torch.manual_seed(0)
    M = torch.randn(32, 4, 4, dtype=torch.float64, requires_grad=True)
    dP = torch.randn(32, 4, 4, dtype=torch.float64)
    O.sinkhorn(M, 20, 1e-6).backward(dP)
    close(O.sinkhorn_grad(M.detach(), dP, 20, 1e-6), M.grad, 1e-10, 1e-12)


def test_dynamic_weights(golden):
    g = golden("dynamic_weights.npz")
    names = ("x", "phi", "bias", "alpha_pre", "alpha_post", "alpha_res")
    for tag, dt, rtol, atol in (("", torch.float32, 1e-5, 1e-6), ("_f64", torch.float64, 1e-10, 1e-12)):
        leaves = [g[n].to(dt).clone().requires_grad_(True) for n in names]
        H_pre, H_post, H_res = O.dynamic_weights(*leaves, 20, 1e-6)
        close(H_pre, g["H_pre" + tag], rtol, atol)
        close(H_post, g["H_post" + tag], rtol, atol)
        close(H_res, g["H_res" + tag], rtol, atol)
        ((H_pre * g["g_pre"].to(dt)).sum() + (H_post * g["g_post"].to(dt)).sum()
         + (H_res * g["g_res"].to(dt)).sum()).backward()
        for n, l in zip(names, leaves):
            ref = g["d" + n + tag]
            assert (l.grad - ref).abs().max() <= atol + rtol * ref.abs().max() * 10, n


def test_stream_mix_and_add_residual(golden):
    g = golden("stream_mix.npz")
    leaves = [g[n].clone().requires_grad_(True) for n in ("H", "H_pre", "H_res")]
    bi, Hr = O.stream_mix(*leaves)
    assert (bi - g["bi"]).abs().max() < 1e-5 and (Hr - g["Hr"]).abs().max() < 1e-5
    ((bi * g["g_bi"]).sum() + (Hr * g["g_hr"]).sum()).backward()
    close(leaves[0].grad, g["dH"], 1e-5, 1e-5)
    close(leaves[1].grad, g["dH_pre"], 1e-5, 1e-4)
    close(leaves[2].grad, g["dH_res"], 1e-5, 1e-4)
    a = golden("add_residual.npz")
    leaves = [a[n].clone().requires_grad_(True) for n in ("Hr", "bo", "H_post")]
    H_new = O.add_residual(*leaves)
    assert (H_new - a["H_new"]).abs().max() < 1e-6
    H_new.backward(a["g"])
    close(leaves[0].grad, a["dHr"])
    close(leaves[1].grad, a["dbo"], 1e-5, 1e-5)
    close(leaves[2].grad, a["dH_post"], 1e-5, 1e-4)


def _params_from(g, prefix):
    kw = {k[len(prefix):]: v for k, v in g.items() if k.startswith(prefix)}
    return O.LayerParams(**kw)


def test_layer_small_all_modes(golden):
    g = golden("layer_small.npz")
    Wb = g["Wb"]
    for mode in ("fused", "unfused", "static"):
        p = _params_from(g, f"{mode}.param.")
        # fp64 against fp64: the restatement is the same function
        r = O.layer_fwd_bwd(p, g["H"], g["g"], lambda t: torch.tanh(t @ Wb.double()), mode, dtype=torch.float64)
        for k, v in r.items():
            ref = g[f"{mode}.{k}_f64"]
            assert (v - ref).abs().max() <= 1e-12 + 1e-9 * ref.abs().max(), (mode, k)
        # fp32 against fp32 at the contract tolerance, norm-wise
        r = O.layer_fwd_bwd(p, g["H"], g["g"], lambda t: torch.tanh(t @ Wb), mode)
        for k, v in r.items():
            ref = g[f"{mode}.{k}"]
            assert (v - ref).abs().max() <= 1e-6 + 1e-5 * ref.abs().max() * 4, (mode, k)


def test_layer_c1(golden):
    g = golden("layer_c1.npz")
    H, up = cases.c1_inputs()
    assert torch.equal(H.flatten()[::97], g["H_sample"]), "seeded inputs differ from the fixture's"
    assert torch.equal(up.flatten()[::97], g["g_sample"])
    for tag in ("default", "perturbed"):
        p = cases.c1_params(tag)
        r64 = O.layer_fwd_bwd(p, H, up, None, "fused", dtype=torch.float64)
        r32 = O.layer_fwd_bwd(p, H, up, None, "fused")
        for k in r32:
            if k in ("branch_input", "H_new", "dH"):
                ref64 = g[f"{tag}.{k}_sample_f64"]
                assert (r64[k].flatten()[::97] - ref64).abs().max() <= 1e-12 + 1e-9 * ref64.abs().max(), (tag, k)
                ref = g[f"{tag}.{k}_sample"]
                assert (r32[k].flatten()[::97] - ref).abs().max() <= 1e-6 + 1e-5 * ref.abs().max(), (tag, k)
            else:
                ref64 = g[f"{tag}.{k}_f64"]
                assert (r64[k] - ref64).abs().max() <= 1e-12 + 1e-8 * ref64.abs().max(), (tag, k)
                # fp32: both sides carry summation-order noise; bound it by the noise of the
                # reference's own fp32 run against its fp64 run (x4) plus the contract tolerance
                ref = g[f"{tag}.{k}"]
                noise = (ref.double() - ref64).abs().max()
                assert (r32[k].double() - ref64).abs().max() <= 1e-6 + 1e-5 * ref64.abs().max() + 4 * noise, (tag, k)
