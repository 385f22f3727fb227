"""The torch.library registration of the four ops (mhc.library).

CPU part: the operators exist with the expected schemas, and their shape-only implementations and
autograd formulas agree with each other on `meta` tensors (no kernel runs).
GPU part: the registered ops give bit-identical results and gradients to the plain ops of mhc.ops,
pass torch.library.opcheck, and trace under torch.compile(fullgraph=True) without a graph break.
"""

import pytest
import torch

B, S, D = 2, 24, 64


def _inputs(device, dtype=torch.float32, seed=0):
    g = torch.Generator().manual_seed(seed)

    def r(*shape, scale=1.0, dt=torch.float32):
        t = (torch.randn(*shape, generator=g) * scale).to(dt)
        return (torch.empty(t.shape, dtype=dt, device="meta") if device == "meta" else t.to(device)).requires_grad_(True)

    return dict(H=r(B, S, 4, D, dt=dtype), bo=r(B, S, D, dt=dtype), x=r(B, 4 * D), phi=r(4 * D, 24, scale=0.05),
                bias=r(24, scale=0.5), a_pre=r(1, scale=0.1), a_post=r(1, scale=0.1), a_res=r(1, scale=0.1),
                M=r(B, 4, 4))


def _layer(ops, t):
    """One hyper-connection step written with the four ops; returns the tensors a caller sees."""
    H_pre, H_post, H_res = ops.fused_dynamic_weights(t["x"], t["phi"], t["bias"], t["a_pre"], t["a_post"], t["a_res"], 20, 1e-6)
    bi, Hr = ops.fused_stream_mix(t["H"], H_pre, H_res)
    H_new = ops.fused_add_residual(Hr, t["bo"] + bi, H_post)
    P = ops.sinkhorn_knopp(t["M"], 20, 1e-8)
    return H_new, P


def test_schemas_registered():
    import mhc.library  # noqa: F401
    for name, nret in [("sinkhorn_fwd", 1), ("sinkhorn_bwd", 1), ("stream_mix_fwd", 2), ("stream_mix_bwd", 3),
                       ("add_residual_fwd", 1), ("add_residual_bwd", 2), ("dynamic_weights_fwd", 4),
                       ("dynamic_weights_bwd", 4)]:
        op = getattr(torch.ops.mhc, name).default
        assert len(op._schema.returns) == nret, name
        assert not op._schema.is_mutable, name


def test_meta_forward_backward_shapes():
    from mhc import library
    t = _inputs("meta", torch.bfloat16)
    H_new, P = _layer(library, t)
    assert H_new.shape == (B, S, 4, D) and H_new.dtype == torch.bfloat16 and P.shape == (B, 4, 4)
    grads = torch.autograd.grad([H_new, P], list(t.values()), [torch.empty_like(H_new), torch.empty_like(P)])
    for (k, v), g in zip(t.items(), grads):
        assert g.shape == v.shape and g.dtype == v.dtype, k


def test_python_float_scales_accepted_on_meta():
    from mhc import library
    t = _inputs("meta")
    H_pre, H_post, H_res = library.fused_dynamic_weights(t["x"], t["phi"], t["bias"], 0.01, 0.02, 0.03)
    assert H_pre.shape == (B, 4) and H_post.shape == (B, 4) and H_res.shape == (B, 4, 4)


def _step(H, bo, x, phi, bias, a_pre, a_post, a_res, M):
    from mhc import library
    return _layer(library, dict(H=H, bo=bo, x=x, phi=phi, bias=bias, a_pre=a_pre, a_post=a_post, a_res=a_res, M=M))


def test_fullgraph_trace_on_meta():
    """Forward and backward trace as one graph each: no graph break at any of the ops."""
    compiled = torch.compile(_step, fullgraph=True, backend="aot_eager")
    t = _inputs("meta", torch.bfloat16)
    H_new, P = compiled(**t)
    (H_new.float().square().mean() + P.square().sum()).backward()
    assert all(v.grad is not None and v.grad.shape == v.shape for v in t.values())


# ------------------------------------------------------------------------------------ GPU
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_registered_ops_equal_plain_ops(dtype):
    import mhc
    from mhc import library
    outs = []
    for ops in (mhc, library):
        t = _inputs("cuda", dtype, seed=3)
        H_new, P = _layer(ops, t)
        g = torch.Generator().manual_seed(9)
        gH = torch.randn(H_new.shape, generator=g).to("cuda", dtype)
        gP = torch.randn(P.shape, generator=g).to("cuda")
        grads = torch.autograd.grad([H_new, P], list(t.values()), [gH, gP])
        outs.append((H_new, P, grads, list(t)))
    (Ha, Pa, ga, names), (Hb, Pb, gb, _) = outs
    assert torch.equal(Ha, Hb) and torch.equal(Pa, Pb)
    for n, a, b in zip(names, ga, gb):
        assert torch.equal(a, b), n


@pytest.mark.gpu
def test_opcheck():
    from mhc import library  # noqa: F401
    t = _inputs("cuda", seed=5)
    oc = torch.library.opcheck
    H_pre, H_post, H_res, saved = torch.ops.mhc.dynamic_weights_fwd(t["x"], t["phi"], t["bias"], t["a_pre"], t["a_post"],
                                                                    t["a_res"], 20, 1e-6)
    H_pre, H_post, H_res = (v.detach().requires_grad_(True) for v in (H_pre, H_post, H_res))
    oc(torch.ops.mhc.sinkhorn_fwd.default, (t["M"], 20, 1e-8))
    oc(torch.ops.mhc.stream_mix_fwd.default, (t["H"], H_pre, H_res))
    oc(torch.ops.mhc.add_residual_fwd.default, (t["H"], t["bo"], H_post))
    oc(torch.ops.mhc.dynamic_weights_fwd.default, (t["x"], t["phi"], t["bias"], t["a_pre"], t["a_post"], t["a_res"], 20, 1e-6))
    with torch.no_grad():
        gH = torch.randn_like(t["H"])
        oc(torch.ops.mhc.sinkhorn_bwd.default, (t["M"].detach(), torch.randn_like(t["M"]), 20, 1e-8))
        oc(torch.ops.mhc.stream_mix_bwd.default, (t["bo"].detach(), gH, t["H"].detach(), H_pre.detach(), H_res.detach()))
        oc(torch.ops.mhc.add_residual_bwd.default, (gH, t["bo"].detach(), H_post.detach()))
        oc(torch.ops.mhc.dynamic_weights_bwd.default,
           (t["x"].detach(), t["phi"].detach(), t["bias"].detach(), t["a_pre"].detach(), t["a_post"].detach(),
            t["a_res"].detach(), saved, torch.randn(B, 4, device="cuda"), torch.randn(B, 4, device="cuda"),
            torch.randn(B, 4, 4, device="cuda"), 20, 1e-6))


@pytest.mark.gpu
def test_fullgraph_compile_matches_eager():
    compiled = torch.compile(_step, fullgraph=True, backend="aot_eager")
    res = []
    for fn in (_step, compiled):
        t = _inputs("cuda", torch.bfloat16, seed=11)
        H_new, P = fn(**t)
        (H_new.float().square().mean() + P.square().sum()).backward()
        res.append((H_new.detach(), P.detach(), {k: v.grad for k, v in t.items()}))
    assert torch.equal(res[0][0], res[1][0]) and torch.equal(res[0][1], res[1][1])
    for k in res[0][2]:
        assert torch.equal(res[0][2][k], res[1][2][k]), k
