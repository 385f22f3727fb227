"""CUDA path vs the CPU oracle and the golden fixtures, on identical seeded inputs.

Tolerances (stated by the task contract): fp32 rtol 1e-5 / atol 1e-6; bf16/fp16 inputs
rtol 2e-2 against the fp32 oracle run on up-cast inputs; Sinkhorn row/column sums within
1e-5 of the oracle's.  Reductions whose fp32 oracle is itself noisier than that band are
compared with the fp64 oracle, allowing the fp32 oracle's own distance to fp64 as slack.
"""

import pytest
import torch

from oracle import mhc_oracle as O
from tests import cases
from tests.util import assert_close, assert_close_norm, maxdiff, to_module

pytestmark = pytest.mark.gpu
DEV = "cuda"
RT, AT = 1e-5, 1e-6


def dev(t):
    return t.detach().clone().to(DEV)


# ------------------------------------------------------------------ Sinkhorn
def test_sinkhorn_golden(golden):
    from mhc import sinkhorn_knopp
    g = golden("sinkhorn.npz")
    M = dev(g["M"]).requires_grad_(True)
    P = sinkhorn_knopp(M, 20, 1e-8)
    assert_close(P, g["P"], RT, AT, "P")
    P.backward(dev(g["dP"]))
    assert_close_norm(M.grad, g["dM_f64"], RT, AT, "dM", extra=2 * maxdiff(g["dM"], g["dM_f64"]))
    P8 = sinkhorn_knopp(dev(g["M8"]))
    assert_close(P8, g["P8"], RT, AT, "P8")
    # row / column sums equal the oracle's within 1e-5
    assert maxdiff(P8.sum(-1), g["P8"].sum(-1)) < 1e-5 and maxdiff(P8.sum(-2), g["P8"].sum(-2)) < 1e-5


@pytest.mark.parametrize("T", [1, 5, 20])
def test_sinkhorn_zero_sign_cases(golden, T):
    import mhc
    g = golden("sinkhorn.npz")
    M = dev(g["Mz"]).requires_grad_(True)
    P = mhc.sinkhorn_knopp(M, T, 1e-6)
    assert_close(P, g[f"Pz_T{T}"], RT, AT)
    P.backward(dev(g["dPz"]))
    ref = O.sinkhorn_grad(g["Mz"].double(), g["dPz"].double(), T, 1e-6)
    assert_close_norm(M.grad, ref, 1e-4, 1e-6, "dM")
    assert (M.grad[M == 0] == 0).all()
    mhc.set_abs_grad_at_zero("plus_one")
    try:
        M2 = dev(g["Mz"]).requires_grad_(True)
        mhc.sinkhorn_knopp(M2, T, 1e-6).backward(dev(g["dPz"]))
        ref1 = O.sinkhorn_grad(g["Mz"].double(), g["dPz"].double(), T, 1e-6, sign_of_zero=1.0)
        assert_close_norm(M2.grad, ref1, 1e-4, 1e-6, "dM(+1)")
    finally:
        mhc.set_abs_grad_at_zero("zero")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("batch", [1, 127, 4099])
def test_sinkhorn_batches_and_dtypes(dtype, batch):
    from mhc import sinkhorn_knopp
    torch.manual_seed(batch)
    M = torch.randn(batch, 4, 4).to(dtype)
    dP = torch.randn(batch, 4, 4).to(dtype)
    Md = dev(M).requires_grad_(True)
    P = sinkhorn_knopp(Md, 20, 1e-6)
    assert P.dtype == dtype
    P.backward(dev(dP))
    Pref = O.sinkhorn(M.double(), 20, 1e-6)
    dref = O.sinkhorn_grad(M.double(), dP.double(), 20, 1e-6)
    if dtype == torch.float32:
        assert_close(P, Pref, RT, AT)
        assert maxdiff(P.sum(-1), Pref.sum(-1)) < 1e-5 and maxdiff(P.sum(-2), Pref.sum(-2)) < 1e-5
        assert_close_norm(Md.grad.reshape(batch, -1), dref.reshape(batch, -1), 1e-4, 1e-5)
    else:
        assert_close(P, Pref, 2e-2, 1e-3)
        assert_close_norm(Md.grad, dref, 2e-2, 1e-3)


def test_sinkhorn_misaligned_view():
    from mhc import sinkhorn_knopp
    torch.manual_seed(3)
    flat = torch.randn(1 + 5 * 16)
    M = flat[1:].view(5, 4, 4)               # 4-byte aligned only
    Md = dev(flat)[1:].view(5, 4, 4)
    assert Md.data_ptr() % 16 != 0
    assert_close(sinkhorn_knopp(Md, 20, 1e-6), O.sinkhorn(M, 20, 1e-6), RT, AT)


# ------------------------------------------------------------ dynamic weights
def test_dynamic_weights_golden(golden):
    from mhc import fused_dynamic_weights
    g = golden("dynamic_weights.npz")
    names = ("x", "phi", "bias", "alpha_pre", "alpha_post", "alpha_res")
    leaves = [dev(g[n]).requires_grad_(True) for n in names]
    H_pre, H_post, H_res = fused_dynamic_weights(*leaves, 20, 1e-6)
    assert H_pre.dtype == H_post.dtype == H_res.dtype == torch.float32
    for got, key in ((H_pre, "H_pre"), (H_post, "H_post"), (H_res, "H_res")):
        assert_close(got, g[key], RT, AT, key)
    ((H_pre * dev(g["g_pre"])).sum() + (H_post * dev(g["g_post"])).sum() + (H_res * dev(g["g_res"])).sum()).backward()
    for n, l in zip(names, leaves):
        ref64, ref32 = g["d" + n + "_f64"], g["d" + n]
        assert l.grad.shape == ref32.shape and l.grad.dtype == torch.float32
        assert_close_norm(l.grad, ref64, RT, AT, "d" + n, extra=2 * maxdiff(ref32, ref64))


def _dw_oracle(x, phi, bias, al, gp, gq, gr):
    """fp64 oracle leaves (with .grad), fp32 oracle leaves (with .grad) and the fp64 outputs of the
    dynamic-weights op for upstream gradients gp, gq, gr.  The fp32 run measures how far plain fp32
    arithmetic of the same formulas strays from fp64 on these inputs; tests allow twice that on top
    of rtol 1e-5 / atol 1e-6."""
    outs = None
    runs = []
    for dt in (torch.float64, torch.float32):
        leaves = [t.to(dt).requires_grad_(True) for t in (x, phi, bias, *al)]
        a, b, c = O.dynamic_weights(*leaves, 20, 1e-6)
        ((a * gp.to(dt)).sum() + (b * gq.to(dt)).sum() + (c * gr.to(dt)).sum()).backward()
        runs.append(leaves)
        if outs is None:
            outs = (a.detach(), b.detach(), c.detach())
    return runs[0], runs[1], outs


@pytest.mark.parametrize("B,K", [(1, 4), (2, 100), (16, 4 * 512), (5, 4 * 1000 + 4)])
def test_dynamic_weights_shapes(B, K):
    from mhc import fused_dynamic_weights
    torch.manual_seed(B * 1000 + K)
    x = torch.randn(B, K)
    phi = torch.randn(K, 24) * 0.05
    bias = torch.randn(24)
    al = [torch.tensor([0.3]), torch.tensor([-0.2]), torch.tensor([0.5])]
    gp, gq, gr = torch.randn(B, 4), torch.randn(B, 4), torch.randn(B, 4, 4)
    ref, ref32, (a, b, c) = _dw_oracle(x, phi, bias, al, gp, gq, gr)
    lv = [dev(t).requires_grad_(True) for t in (x, phi, bias, *al)]
    a2, b2, c2 = fused_dynamic_weights(*lv, 20, 1e-6)
    assert_close(a2, a, RT, AT, "H_pre"); assert_close(b2, b, RT, AT, "H_post"); assert_close(c2, c, 2e-5, AT, "H_res")
    ((a2 * dev(gp)).sum() + (b2 * dev(gq)).sum() + (c2 * dev(gr)).sum()).backward()
    for r, r32, l, n in zip(ref, ref32, lv, "x phi bias a_pre a_post a_res".split()):
        # rtol 1e-5 against fp64, plus twice the distance of the fp32 oracle's own gradient from fp64
        assert_close_norm(l.grad, r.grad, RT, AT, "d" + n, extra=2 * maxdiff(r32.grad, r.grad))


# ------------------------------------------------------------- streaming ops
def test_stream_ops_golden(golden):
    from mhc import fused_add_residual, fused_stream_mix
    g = golden("stream_mix.npz")
    lv = [dev(g[n]).requires_grad_(True) for n in ("H", "H_pre", "H_res")]
    bi, Hr = fused_stream_mix(*lv)
    assert_close(bi, g["bi"], RT, AT, "bi"); assert_close(Hr, g["Hr"], RT, AT, "Hr")
    ((bi * dev(g["g_bi"])).sum() + (Hr * dev(g["g_hr"])).sum()).backward()
    assert_close(lv[0].grad, g["dH"], RT, 2 * AT, "dH")
    assert_close_norm(lv[1].grad, g["dH_pre"], RT, AT, "dH_pre"); assert_close_norm(lv[2].grad, g["dH_res"], RT, AT, "dH_res")
    a = golden("add_residual.npz")
    lv = [dev(a[n]).requires_grad_(True) for n in ("Hr", "bo", "H_post")]
    H_new = fused_add_residual(*lv)
    assert_close(H_new, a["H_new"], RT, AT, "H_new")
    H_new.backward(dev(a["g"]))
    assert_close(lv[0].grad, a["dHr"], 0, 0, "dHr")
    assert_close(lv[1].grad, a["dbo"], RT, 2 * AT, "dbo"); assert_close_norm(lv[2].grad, a["dH_post"], RT, AT, "dH_post")


# the last two: rows of 320 / 640 / 896 packs, which take column groups narrower than 256 (several tokens abreast)
SHAPES = [(1, 1, 8), (2, 5, 24), (1, 33, 7), (3, 130, 100), (2, 64, 1024), (1, 257, 2056), (2, 40, 8 * 300),
          (2, 37, 8 * 320), (1, 21, 7168)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,S,D", SHAPES)
def test_stream_ops_shapes(dtype, B, S, D):
    """Ragged sizes: odd D (scalar path), S not a multiple of the chunk, single token."""
    from mhc import fused_add_residual, fused_stream_mix
    torch.manual_seed(B * 7919 + S * 31 + D)
    H = torch.randn(B, S, 4, D).to(dtype)
    H_pre = torch.softmax(torch.randn(B, 4), -1)
    H_res = O.sinkhorn(torch.randn(B, 4, 4))
    H_post = 2 * torch.sigmoid(torch.randn(B, 4))
    bo = torch.randn(B, S, D).to(dtype)
    g_bi, g_hr, g_new = torch.randn(B, S, D).to(dtype), torch.randn(B, S, 4, D).to(dtype), torch.randn(B, S, 4, D).to(dtype)
    f = lambda t: t.double().requires_grad_(True)
    rH, rpre, rres, rpost, rbo = f(H), f(H_pre), f(H_res), f(H_post), f(bo)
    bi, Hr = O.stream_mix(rH, rpre, rres)
    ((bi * g_bi.double()).sum() + (Hr * g_hr.double()).sum()).backward()
    Hr_in = Hr.detach().to(dtype)
    rHr = f(Hr_in)
    Hn = O.add_residual(rHr, rbo, rpost)
    Hn.backward(g_new.double())

    dH_, dpre, dres, dpost = (dev(t).requires_grad_(True) for t in (H, H_pre, H_res, H_post))
    dbo = dev(bo).requires_grad_(True)
    bi2, Hr2 = fused_stream_mix(dH_, dpre, dres)
    assert bi2.dtype == dtype and Hr2.dtype == dtype
    ((bi2.float() * dev(g_bi).float()).sum() + (Hr2.float() * dev(g_hr).float()).sum()).backward()
    dHr_in = dev(Hr_in).requires_grad_(True)
    Hn2 = fused_add_residual(dHr_in, dbo, dpost)
    Hn2.backward(dev(g_new))
    rt, at = (RT, 4 * AT) if dtype == torch.float32 else (2e-2, 2e-2)
    assert_close(bi2, bi, rt, at, "bi"); assert_close(Hr2, Hr, rt, at, "Hr"); assert_close(Hn2, Hn, rt, at, "H_new")
    assert_close(dH_.grad, rH.grad, rt, at, "dH"); assert_close(dbo.grad, rbo.grad, rt, at, "dbo")
    assert torch.equal(dHr_in.grad, dev(g_new)), "dH_residual must be the upstream gradient itself"
    wt = 1e-5 if dtype == torch.float32 else 1e-5   # weight grads are fp32 sums of exact products either way
    assert_close_norm(dpre.grad, rpre.grad, wt, AT, "dH_pre"); assert_close_norm(dres.grad, rres.grad, wt, AT, "dH_res")
    assert_close_norm(dpost.grad, rpost.grad, wt, AT, "dH_post")


def test_noncontiguous_and_misaligned_inputs():
    from mhc import fused_stream_mix
    torch.manual_seed(9)
    B, S, D = 2, 9, 16
    big = torch.randn(B, S, 4, D + 3)
    H = big[..., 3:]                          # non-contiguous view, made contiguous by the wrapper
    flat = torch.randn(B * S * 4 * D + 1)
    H2 = flat[1:].view(B, S, 4, D)            # contiguous but only 4-byte aligned: scalar path
    H_pre = torch.softmax(torch.randn(B, 4), -1)
    H_res = O.sinkhorn(torch.randn(B, 4, 4))
    for Hc, Hd in ((H, dev(big)[..., 3:]), (H2, dev(flat)[1:].view(B, S, 4, D))):
        bi, Hr = fused_stream_mix(Hd, dev(H_pre), dev(H_res))
        rbi, rHr = O.stream_mix(Hc, H_pre, H_res)
        assert_close(bi, rbi, RT, 2 * AT); assert_close(Hr, rHr, RT, 2 * AT)


def test_empty_batch():
    from mhc import fused_add_residual, fused_stream_mix, sinkhorn_knopp
    assert sinkhorn_knopp(torch.empty(0, 4, 4, device=DEV)).shape == (0, 4, 4)
    bi, Hr = fused_stream_mix(torch.empty(0, 5, 4, 8, device=DEV), torch.empty(0, 4, device=DEV), torch.empty(0, 4, 4, device=DEV))
    assert bi.shape == (0, 5, 8) and Hr.shape == (0, 5, 4, 8)
    assert fused_add_residual(Hr, bi, torch.empty(0, 4, device=DEV)).shape == (0, 5, 4, 8)


# ------------------------------------------------------------------ whole layer
def _run_module(hc, H, g, branch):
    import mhc  # noqa: F401
    for p in hc.parameters():
        p.grad = None
    Hd = dev(H).requires_grad_(True)
    bi, add = hc(Hd)
    H_new = add(branch(bi))
    H_new.backward(dev(g))
    out = {"branch_input": bi, "H_new": H_new, "dH": Hd.grad}
    for n, p in hc.named_parameters():
        out["d" + n.replace(".weight", "")] = p.grad
    return out


@pytest.mark.parametrize("mode", ["fused", "unfused", "static"])
def test_layer_small_golden(golden, mode):
    from mhc import HyperConnection
    g = golden("layer_small.npz")
    kw = dict(fused=dict(dynamic=True), unfused=dict(dynamic=True, use_fused_weights=False), static=dict(dynamic=False))[mode]
    hc = HyperConnection(dim=64, layer_idx=1, **kw)
    p = O.LayerParams(**{k[len(mode) + 7:]: v for k, v in g.items() if k.startswith(mode + ".param.")})
    to_module(hc, p).to(DEV)
    Wb = dev(g["Wb"])
    out = _run_module(hc, g["H"], g["g"], lambda t: torch.tanh(t @ Wb))
    for k, v in out.items():
        ref32, ref64 = g[f"{mode}.{k}"], g[f"{mode}.{k}_f64"]
        assert_close_norm(v, ref64, RT, AT, f"{mode}.{k}", extra=2 * maxdiff(ref32, ref64))
        if k in ("branch_input", "H_new"):
            assert_close(v, ref32, RT, 2 * AT, k)


@pytest.mark.parametrize("tag", ["default", "perturbed"])
def test_layer_c1(golden, tag):
    """Config 1: HyperConnection(512) on fp32 H(2,128,4,512), identity branch, fwd+bwd."""
    from mhc import HyperConnection
    g = golden("layer_c1.npz")
    H, up = cases.c1_inputs()
    p = cases.c1_params(tag)
    hc = to_module(HyperConnection(dim=512, num_streams=4, layer_idx=0, dynamic=True, sinkhorn_iters=20,
                                   init_scale=0.1), p).to(DEV)
    out = _run_module(hc, H, up, lambda t: t)
    ref32 = O.layer_fwd_bwd(p, H, up, None, "fused")
    ref64 = O.layer_fwd_bwd(p, H, up, None, "fused", dtype=torch.float64)
    for k, v in out.items():
        if k in ("branch_input", "H_new", "dH"):
            assert_close(v, ref64[k], RT, 2 * AT, k)                 # full tensors vs the fp64 oracle
            assert_close(v.flatten()[::97], g[f"{tag}.{k}_sample"], RT, 4 * AT, k + " (fixture)")
        else:
            gold32, gold64 = g[f"{tag}.{k}"], g[f"{tag}.{k}_f64"]
            noise = max(maxdiff(gold32, gold64), maxdiff(ref32[k], ref64[k]))
            assert_close_norm(v, gold64, RT, AT, k, extra=2 * noise)
    if tag == "default":
        # |.| kink: off-diagonal residual-base gradients are exactly zero under the default convention
        off = ~torch.eye(4, dtype=torch.bool)
        assert (out["dH_res_base"].cpu()[off] == 0).all()


class _StoreAs(torch.autograd.Function):
    """Round a tensor (and, on the way back, its gradient) to a storage dtype: emulates the points
    where the device path keeps activations in half precision."""

    @staticmethod
    def forward(ctx, t, dtype):
        ctx.dtype = dtype
        return t.to(dtype).to(t.dtype)

    @staticmethod
    def backward(ctx, g):
        return g.to(ctx.dtype).to(g.dtype), None


def _oracle_with_storage_rounding(p, H, up, branch, dtype):
    """fp64 oracle whose activations are rounded to `dtype` wherever the device path stores them
    (branch_input, H_residual, branch_output, H_new and their gradients); weights and weight
    gradients stay unrounded, as on the device."""
    p64 = p.to(torch.float64)
    leaves = {k: v.requires_grad_(True) for k, v in p64.tensors().items()}
    Hl = H.double().requires_grad_(True)
    H_pre, H_post, H_res = O.layer_weights(O.LayerParams(**leaves), Hl, "fused", 20, 1e-6)
    bi, Hr = O.stream_mix(Hl, H_pre, H_res)
    bi, Hr = _StoreAs.apply(bi, dtype), _StoreAs.apply(Hr, dtype)
    bo = _StoreAs.apply(branch(bi), dtype)
    H_new = _StoreAs.apply(O.add_residual(Hr, bo, H_post), dtype)
    H_new.backward(up.double())
    out = {"branch_input": bi.detach(), "H_new": H_new.detach(), "dH": Hl.grad}
    out.update({"d" + k: v.grad for k, v in leaves.items()})
    return out


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_layer_half_precision(dtype):
    """Half-precision H with fp32 parameters (the mixed configuration of configs 3-5, reduced
    size).  Outputs and weight gradients are within rtol 2e-2 of the fp32-exact oracle on the
    up-cast input; the three scalar scale gradients are sums with heavy cancellation, so they are
    held to rtol 2e-2 against the oracle that rounds activations where the device stores them."""
    from mhc import HyperConnection
    torch.manual_seed(0)
    B, S, D = 2, 512, 512
    H = torch.randn(B, S, 4, D).to(dtype)
    up = torch.randn(B, S, 4, D).to(dtype)
    p = cases.perturb_params_(O.default_params(D, 0, 0.1), 21)
    hc = to_module(HyperConnection(dim=D), p).to(DEV)
    lin = torch.nn.Linear(D, D).to(dtype)           # the branch's own weights are half precision too
    W, bvec = lin.weight.detach().double(), lin.bias.detach().double()
    branch_ref = lambda t: t @ W.T + bvec
    lin_d = torch.nn.Linear(D, D).to(dtype)
    lin_d.load_state_dict(lin.state_dict()); lin_d = lin_d.to(DEV)
    out = _run_module(hc, H, up, lin_d)
    ref = O.layer_fwd_bwd(p, H.float(), up.float(), branch_ref, "fused", dtype=torch.float64)
    ref_r = _oracle_with_storage_rounding(p, H, up, branch_ref, dtype)
    for k, v in out.items():
        if k in ("branch_input", "H_new", "dH"):
            assert v.dtype == dtype
            assert_close_norm(v, ref[k], 2e-2, 0, k)
            assert_close_norm(v, ref_r[k], 1e-2, 0, k + " (storage-rounded oracle)")
        else:
            assert v.dtype == torch.float32
            assert_close_norm(v, ref_r[k], 2e-2, 1e-6, k + " (storage-rounded oracle)")
            if not k.startswith("dalpha"):
                assert_close_norm(v, ref[k], 2e-2, 1e-6, k)


def test_determinism_and_shard_invariance():
    """Two runs are bit-identical, and a batch shard reproduces the full batch's per-element
    results bit for bit (the reduction layout does not depend on the batch size)."""
    from mhc import HyperConnection
    torch.manual_seed(1)
    B, S, D = 4, 300, 256
    H = torch.randn(B, S, 4, D).bfloat16()
    up = torch.randn(B, S, 4, D).bfloat16()
    p = cases.perturb_params_(O.default_params(D, 0, 0.1), 2)
    hc = to_module(HyperConnection(dim=D), p).to(DEV)
    a = _run_module(hc, H, up, lambda t: t)
    a = {k: v.clone() for k, v in a.items()}
    b = _run_module(hc, H, up, lambda t: t)
    for k in a:
        assert torch.equal(a[k], b[k]), k
    c = _run_module(hc, H[1:3], up[1:3], lambda t: t)
    for k in ("branch_input", "H_new", "dH"):
        assert torch.equal(a[k][1:3], c[k]), k


def test_unfused_ops_match_fused_node():
    """The public ops chained by hand (as the reference module does) give the same result as the
    fused node the module uses."""
    import mhc
    torch.manual_seed(4)
    B, S, D = 2, 70, 96
    H = torch.randn(B, S, 4, D)
    up = torch.randn(B, S, 4, D)
    p = cases.perturb_params_(O.default_params(D, 0, 0.1), 8)
    hc = to_module(mhc.HyperConnection(dim=D), p).to(DEV)
    fused = _run_module(hc, H, up, lambda t: t)
    fused = {k: v.clone() for k, v in fused.items()}
    for q in hc.parameters():
        q.grad = None
    Hd = dev(H).requires_grad_(True)
    H_post, H_pre, H_res = hc._compute_weights(Hd)
    bi, Hr = mhc.fused_stream_mix(Hd, H_pre, H_res)
    H_new = mhc.fused_add_residual(Hr, bi, H_post)
    H_new.backward(dev(up))
    assert_close(bi, fused["branch_input"], 0, 0); assert_close(H_new, fused["H_new"], 0, 0)
    assert_close(Hd.grad, fused["dH"], RT, 2 * AT, "dH")
    for n, q in hc.named_parameters():
        assert_close_norm(q.grad, fused["d" + n], RT, AT, n)


def test_host_streamed_step_matches_direct_run():
    """The host-buffer pipeline (groups of batch elements on three streams, parameter gradients
    accumulated across groups) reproduces the direct on-device step."""
    import mhc
    torch.manual_seed(5)
    B, S, D = 5, 130, 64
    H = torch.randn(B, S, 4, D).bfloat16()
    up = torch.randn(B, S, 4, D).bfloat16()
    p = cases.perturb_params_(O.default_params(D, 0, 0.1), 12)
    hc = to_module(mhc.HyperConnection(dim=D), p).to(DEV)
    direct = _run_module(hc, H, up, lambda t: t)
    direct = {k: v.clone() for k, v in direct.items()}
    for q in hc.parameters():
        q.grad = None
    step = mhc.HostStreamedStep(hc, group=2)
    Hh, gh = H.pin_memory(), up.pin_memory()
    out_new, out_dH = torch.empty_like(Hh).pin_memory(), torch.empty_like(Hh).pin_memory()
    flat = torch.empty(step.sync.flat.numel()).pin_memory()
    for _ in range(2):      # the second call must not accumulate on top of the first
        step(Hh, gh, out_new, out_dH, flat)
    torch.cuda.synchronize()
    assert torch.equal(out_new, direct["H_new"].cpu()) and torch.equal(out_dH, direct["dH"].cpu())
    for n, q in hc.named_parameters():
        assert_close_norm(q.grad, direct["d" + n], RT, AT, n)
    assert torch.equal(flat[:4 * D * 24].view(4 * D, 24), hc.phi.grad.cpu())


def test_host_streamed_step_back_to_back_calls_with_different_data():
    """Two calls queued without a synchronisation in between, each with its own inputs and outputs: the
    second call's uploads must not overwrite staging buffers that the first call's kernels still read."""
    import mhc
    torch.manual_seed(6)
    B, S, D = 1, 2048, 1024                     # one group per call, kernels long enough to still run
    p = cases.perturb_params_(O.default_params(D, 0, 0.1), 13)
    hc = to_module(mhc.HyperConnection(dim=D), p).to(DEV)
    data = [(torch.randn(B, S, 4, D).bfloat16(), torch.randn(B, S, 4, D).bfloat16()) for _ in range(4)]
    direct = []
    for H, up in data:
        r = _run_module(hc, H, up, lambda t: t)
        direct.append((r["H_new"].cpu(), r["dH"].cpu()))
    step = mhc.HostStreamedStep(hc, group=1, slots=2)
    pinned = [(H.pin_memory(), up.pin_memory(), torch.empty_like(H).pin_memory(), torch.empty_like(H).pin_memory())
              for H, up in data]
    for Hh, gh, out_new, out_dH in pinned:      # four calls on two slots, no synchronisation in between
        step(Hh, gh, out_new, out_dH)
    torch.cuda.synchronize()
    for (Hh, gh, out_new, out_dH), (want_new, want_dH) in zip(pinned, direct):
        assert torch.equal(out_new, want_new) and torch.equal(out_dH, want_dH)


def test_layer_stack_with_mlp_branches():
    """Reduced form of the 16-layer configuration: a stack of dynamic layers, each wrapping a
    2-layer SiLU MLP branch, fp32, against the oracle chained the same way."""
    import mhc
    torch.manual_seed(11)
    B, S, D, Lyr = 2, 48, 64, 3
    H = torch.randn(B, S, 4, D)
    up = torch.randn(B, S, 4, D)
    params = [cases.perturb_params_(O.default_params(D, i, 0.1), 30 + i) for i in range(Lyr)]
    W1 = [torch.randn(D, 4 * D) / D ** 0.5 for _ in range(Lyr)]
    W2 = [torch.randn(4 * D, D) / (4 * D) ** 0.5 for _ in range(Lyr)]

    def run(make_layer, mm, Hin, g):
        Hin = Hin.requires_grad_(True)
        layers = [make_layer(i) for i in range(Lyr)]
        h = Hin
        for i, lay in enumerate(layers):
            bi, add = lay(h)
            h = add(torch.nn.functional.silu(bi @ mm(W1[i])) @ mm(W2[i]))
        h.backward(g)
        return h, Hin.grad, layers

    # oracle chain in fp64
    leaves = [{k: v.double().requires_grad_(True) for k, v in p.tensors().items()} for p in params]

    def oracle_layer(i):
        lp = O.LayerParams(**leaves[i])

        def fwd(h):
            H_pre, H_post, H_res = O.layer_weights(lp, h, "fused", 20, 1e-6)
            bi, Hr = O.stream_mix(h, H_pre, H_res)
            return bi, lambda bo: O.add_residual(Hr, bo, H_post)
        return fwd

    out_ref, dH_ref, _ = run(oracle_layer, lambda w: w.double(), H.double(), up.double())
    out, dH, layers = run(lambda i: to_module(mhc.HyperConnection(dim=D, layer_idx=i), params[i]).to(DEV),
                          lambda w: w.to(DEV), dev(H), dev(up))
    assert_close_norm(out, out_ref, RT, AT, "H_out"); assert_close_norm(dH, dH_ref, 1e-4, AT, "dH")
    for i, lay in enumerate(layers):
        for n, q in lay.named_parameters():
            assert_close_norm(q.grad, leaves[i][n].grad, 1e-4, AT, f"layer{i}.{n}")


def test_unused_outputs_get_no_gradient_buffers():
    """Only one of an op's outputs feeds the loss: the missing upstream gradients count as zero."""
    import mhc
    torch.manual_seed(2)
    B, S, D = 2, 20, 32
    H = torch.randn(B, S, 4, D)
    H_pre = torch.softmax(torch.randn(B, 4), -1)
    H_res = O.sinkhorn(torch.randn(B, 4, 4))
    g = torch.randn(B, S, D)
    ref = [t.clone().double().requires_grad_(True) for t in (H, H_pre, H_res)]
    (O.stream_mix(*ref)[0] * g.double()).sum().backward()
    lv = [dev(t).requires_grad_(True) for t in (H, H_pre, H_res)]
    (mhc.fused_stream_mix(*lv)[0] * dev(g)).sum().backward()
    assert_close(lv[0].grad, ref[0].grad, RT, 2 * AT); assert_close_norm(lv[1].grad, ref[1].grad, RT, AT)
    assert float(lv[2].grad.abs().max()) == 0.0
    # module: loss on branch_input only (add_residual never called)
    p = cases.perturb_params_(O.default_params(D, 0, 0.1), 9)
    hc = to_module(mhc.HyperConnection(dim=D), p).to(DEV)
    Hd = dev(H).requires_grad_(True)
    bi, _ = hc(Hd)
    (bi * dev(g)).sum().backward()
    leaves = {k: v.double().requires_grad_(True) for k, v in p.tensors().items()}
    Hl = H.double().requires_grad_(True)
    a, b_, c = O.layer_weights(O.LayerParams(**leaves), Hl, "fused", 20, 1e-6)
    (O.stream_mix(Hl, a, c)[0] * g.double()).sum().backward()
    assert_close(Hd.grad, Hl.grad, RT, 2 * AT, "dH")
    assert_close_norm(hc.phi.grad, leaves["phi"].grad, 1e-4, AT, "dphi")


def test_sinkhorn_backward_checkpointed_equals_plain_sweep(tmp_path):
    """The default backward (register checkpoints) is bit-identical to the plain O(T^2) sweep,
    which a child process selects through the environment."""
    import os
    import subprocess
    import sys
    from mhc import sinkhorn_knopp
    from tests.conftest import PKG_DIR, ROOT
    out = tmp_path / "plain.pt"
    code = (
        "import sys, torch\n"
        f"sys.path.insert(0, {PKG_DIR!r})\n"
        "from mhc._backward import sinkhorn_backward\n"
        "torch.manual_seed(3)\n"
        "res = {}\n"
        "for T in (1, 3, 4, 5, 20, 23):\n"
        "    M = torch.randn(1000, 4, 4); dP = torch.randn(1000, 4, 4)\n"
        "    res[T] = sinkhorn_backward(M.cuda(), dP.cuda(), T, 1e-6).cpu()\n"
        f"torch.save(res, {str(out)!r})\n")
    env = dict(os.environ, MHC_SINKHORN_PLAIN="1")
    subprocess.run([sys.executable, "-c", code], check=True, env=env, cwd=ROOT)
    plain = torch.load(out)
    from mhc._backward import sinkhorn_backward
    torch.manual_seed(3)
    for T in (1, 3, 4, 5, 20, 23):
        M = torch.randn(1000, 4, 4); dP = torch.randn(1000, 4, 4)
        got = sinkhorn_backward(M.cuda(), dP.cuda(), T, 1e-6).cpu()
        assert torch.equal(got, plain[T]), T


def test_sequence_sharded_wrapper_single_rank_equals_layer():
    """With one rank the sequence-sharded wrapper is the layer itself (same kernels, unfused chain)."""
    import mhc
    from mhc.parallel import SequenceShardedHyperConnection
    torch.manual_seed(6)
    B, S, D = 2, 90, 64
    H = torch.randn(B, S, 4, D)
    up = torch.randn(B, S, 4, D)
    p = cases.perturb_params_(O.default_params(D, 0, 0.1), 14)
    hc = to_module(mhc.HyperConnection(dim=D), p).to(DEV)
    a = {k: v.clone() for k, v in _run_module(hc, H, up, lambda t: t).items()}
    b = _run_module(SequenceShardedHyperConnection(hc), H, up, lambda t: t)
    for k in ("branch_input", "H_new"):
        assert torch.equal(a[k], b[k]), k
    assert_close(b["dH"], a["dH"], RT, 2 * AT, "dH")
    for n, _ in hc.named_parameters():
        assert_close_norm(b["dlayer." + n], a["d" + n], RT, AT, n)


@pytest.mark.parametrize("dtype,B,S,D", [(torch.float32, 2, 150, 96), (torch.bfloat16, 2, 300, 512), (torch.float32, 1, 70, 20),
                                           (torch.bfloat16, 2, 70, 2560), (torch.bfloat16, 1, 3, 512), (torch.float32, 2, 1, 256)])
def test_cross_layer_pooling_matches_separate_pooling(dtype, B, S, D):
    """add_residual(pool_for_next=True) hands the next layer the token sums of H_new: that layer
    launches no mean-pool kernel and gives the same results (the pooled state only differs in
    summation order)."""
    import mhc
    from mhc import _lib
    torch.manual_seed(8)
    H = torch.randn(B, S, 4, D).to(dtype)
    up = torch.randn(B, S, 4, D).to(dtype)
    ps = [cases.perturb_params_(O.default_params(D, i, 0.1), 40 + i) for i in range(2)]
    layers = [to_module(mhc.HyperConnection(dim=D, layer_idx=i), ps[i]).to(DEV) for i in range(2)]

    def run(pool):
        for l in layers:
            for q in l.parameters():
                q.grad = None
        Hd = dev(H).requires_grad_(True)
        bi, add = layers[0](Hd)
        H1 = add(torch.tanh(bi), pool_for_next=pool)
        assert (mhc.ops.pooled_sums_of(H1) is not None) == pool
        _lib.profile_start()
        bi2, add2 = layers[1](H1)
        names = set(_lib.profile_stop())
        H2 = add2(bi2 * 0.5)
        H2.backward(dev(up))
        return H1, H2, Hd.grad, [q.grad.clone() for l in layers for q in l.parameters()], names

    H1a, H2a, dHa, ga, na = run(False)
    H1b, H2b, dHb, gb, nb = run(True)
    assert "k_meanpool_partial" in na and "k_meanpool_partial" not in nb
    assert torch.equal(H1a, H1b)
    rt, at = (RT, 4 * AT) if dtype == torch.float32 else (2e-2, 2e-2)
    assert_close_norm(H2b, H2a, rt, at, "H2"); assert_close_norm(dHb, dHa, rt, at, "dH")
    for x, y in zip(gb, ga):
        assert_close_norm(x, y, 1e-4 if dtype == torch.float32 else 2e-2, AT)
    # a tensor modified in place no longer carries valid sums
    H1b.detach().add_(1.0)
    assert mhc.ops.pooled_sums_of(H1b) is None


@pytest.mark.parametrize("n_layers,D", [(1, 128), (2, 512)])
def test_step_replayed_from_cuda_graph_equals_eager(n_layers, D):
    """Forward + backward captured in a CUDA graph (kernels chained by programmatic dependent
    launch, no host synchronisation anywhere in the step) replays to the eager results, also
    after the static input buffers are refilled.  Two layers: the first add-residual also pools
    for the second (the kernel with the shared-memory ring of loads and a raised shared-memory limit)."""
    import mhc
    torch.manual_seed(13)
    B, S = 2, 160
    hcs = [to_module(mhc.HyperConnection(dim=D, layer_idx=i), cases.perturb_params_(O.default_params(D, i, 0.1), 17 + i)).to(DEV)
           for i in range(n_layers)]
    sync = mhc.GradSync(hcs)
    H = torch.randn(B, S, 4, D, device=DEV).bfloat16().requires_grad_(True)
    g = torch.randn(B, S, 4, D, device=DEV).bfloat16()
    out = {}

    def step():
        H.grad = None
        h = H
        for i, hc in enumerate(hcs):
            bi, add = hc(h)
            h = add(torch.tanh(bi), pool_for_next=i + 1 < n_layers)
        h.backward(g)
        out["H_new"], out["dH"] = h, H.grad

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            step()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    static_new, static_dH = out["H_new"], out["dH"]
    for seed in (1, 2):
        torch.manual_seed(seed)
        with torch.no_grad():
            H.copy_(torch.randn(B, S, 4, D, device=DEV).bfloat16())
            g.copy_(torch.randn(B, S, 4, D, device=DEV).bfloat16())
        graph.replay()
        torch.cuda.synchronize()
        got = (static_new.clone(), static_dH.clone(), sync.flat.clone())
        step()
        torch.cuda.synchronize()
        assert torch.equal(got[0], out["H_new"]) and torch.equal(got[1], out["dH"]) and torch.equal(got[2], sync.flat)


def test_whole_module_in_half_precision():
    """The reference's benchmark casts the whole module to fp16 (parameters too): parameters are
    up-cast per call, gradients come back in the parameters' dtype."""
    import mhc
    torch.manual_seed(3)
    B, S, D = 2, 256, 256
    H = torch.randn(B, S, 4, D).half()
    up = torch.randn(B, S, 4, D).half()
    p = cases.perturb_params_(O.default_params(D, 0, 0.1), 23)
    hc = to_module(mhc.HyperConnection(dim=D), p).to(DEV).half()
    p16 = O.LayerParams(**{k: v.half().float() for k, v in p.tensors().items()})   # what the module holds after .half()
    out = _run_module(hc, H, up, lambda t: t * 0.5)
    ref = O.layer_fwd_bwd(p16, H.float(), up.float(), lambda t: t * 0.5, "fused", dtype=torch.float64)
    for k, v in out.items():
        assert v.dtype == torch.float16, k
        assert_close_norm(v, ref[k], 2e-2, 2e-3 if k.startswith("dalpha") else 1e-4, k)


def test_layer_inside_a_compiled_model():
    """torch.compile of a model that contains the layer: the layer itself runs eagerly (opaque
    call), results equal the uncompiled model."""
    import mhc

    class Block(torch.nn.Module):
        def __init__(self, D):
            super().__init__()
            self.hc = mhc.HyperConnection(dim=D)
            self.lin = torch.nn.Linear(D, D)

        def forward(self, H):
            bi, add = self.hc(H)
            return add(torch.nn.functional.gelu(self.lin(bi))) * 1.5

    torch.manual_seed(21)
    D = 64
    blk = Block(D).to(DEV)
    with torch.no_grad():
        blk.hc.phi.copy_(torch.randn(4 * D, 24, device=DEV) * 0.02)
    H = torch.randn(2, 40, 4, D, device=DEV)
    want = blk(H.clone().requires_grad_(True))
    got = torch.compile(blk, backend="eager")(H.clone().requires_grad_(True))
    assert torch.equal(got, want)
    got.sum().backward()
    assert blk.hc.phi.grad is not None and torch.isfinite(blk.hc.phi.grad).all()


def test_per_token_weights_through_reshape():
    """The paper's per-token formulation (weights from every token's own 4*D state, not from the
    sequence mean) is the same layer applied to H viewed as [B*S, 1, 4, D]: every entry point
    takes any number of rows, and from 64 rows on the dynamic-weights kernels tile over rows."""
    import mhc
    torch.manual_seed(31)
    B, S, D = 2, 37, 48
    H = torch.randn(B * S, 1, 4, D)
    up = torch.randn(B * S, 1, 4, D)
    p = cases.perturb_params_(O.default_params(D, 0, 0.1), 19)
    hc = to_module(mhc.HyperConnection(dim=D), p).to(DEV)
    out = _run_module(hc, H, up, lambda t: torch.tanh(t))
    ref = O.layer_fwd_bwd(p, H, up, torch.tanh, "fused", dtype=torch.float64)
    for k, v in out.items():
        assert_close_norm(v, ref[k], 1e-4 if k.startswith("d") else RT, 4 * AT, k)


@pytest.mark.parametrize("B,K", [(64, 4 * 64), (200, 4 * 100 + 4), (1000, 4 * 256), (130, 4 * 33 + 2), (300, 4 * 1100),
                                 (2500, 4 * 128), (4096 + 17, 2048), (129, 128)])
def test_dynamic_weights_many_rows(B, K):
    """From 64 rows on the op switches to kernels tiled over rows (per-token use); same results.
    Covers the register-tiled projection (K % 4 == 0) with one and with several K slices, the scalar
    projection (K % 4 != 0), ragged last row blocks, and several row tiles in the backward."""
    from mhc import fused_dynamic_weights
    torch.manual_seed(B + K)
    x = torch.randn(B, K)
    phi = torch.randn(K, 24) * 0.05
    bias = torch.randn(24)
    al = [torch.tensor([0.3]), torch.tensor([-0.2]), torch.tensor([0.5])]
    gp, gq, gr = torch.randn(B, 4), torch.randn(B, 4), torch.randn(B, 4, 4)
    ref, ref32, (a, b, c) = _dw_oracle(x, phi, bias, al, gp, gq, gr)
    lv = [dev(t).requires_grad_(True) for t in (x, phi, bias, *al)]
    a2, b2, c2 = fused_dynamic_weights(*lv, 20, 1e-6)
    assert_close(a2, a, RT, AT, "H_pre"); assert_close(b2, b, RT, AT, "H_post"); assert_close(c2, c, 2e-5, 4 * AT, "H_res")   # row-tiled path: longer sequential fp32 sums over K
    ((a2 * dev(gp)).sum() + (b2 * dev(gq)).sum() + (c2 * dev(gr)).sum()).backward()
    for r, r32, l, n in zip(ref, ref32, lv, "x phi bias a_pre a_post a_res".split()):
        assert_close_norm(l.grad, r.grad, RT, AT, "d" + n, extra=2 * maxdiff(r32.grad, r.grad))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_lazy_residual_equals_materialised_residual(dtype):
    """Default module path (H_residual never written, residual mix recomputed inside add residual)
    against the two-kernel forward: bit-identical in fp32, one rounding apart in bf16; and the
    closure refuses to run after an in-place change of H."""
    import mhc
    torch.manual_seed(41)
    B, S, D = 2, 130, 72
    H = torch.randn(B, S, 4, D).to(dtype)
    up = torch.randn(B, S, 4, D).to(dtype)
    p = cases.perturb_params_(O.default_params(D, 0, 0.1), 27)
    hc = to_module(mhc.HyperConnection(dim=D), p).to(DEV)
    lazy = {k: v.clone() for k, v in _run_module(hc, H, up, torch.tanh).items()}
    hc.materialize_residual = True
    full = _run_module(hc, H, up, torch.tanh)
    hc.materialize_residual = False
    for k in lazy:
        if dtype == torch.float32:
            assert torch.equal(lazy[k], full[k]), k
        elif k in ("branch_input",):
            assert torch.equal(lazy[k], full[k]), k
        else:
            assert_close_norm(lazy[k], full[k], 2e-2, 1e-6, k)
    Hd = dev(H).requires_grad_(False)
    bi, add = hc(Hd)
    Hd.add_(1.0)
    with pytest.raises(RuntimeError, match="modified in place"):
        add(bi)


def test_inference_mode_and_no_grad():
    """Forward under torch.inference_mode() / no_grad (tensors without version counters or graphs)."""
    import mhc
    torch.manual_seed(2)
    B, S, D = 2, 50, 64
    H = torch.randn(B, S, 4, D)
    p = cases.perturb_params_(O.default_params(D, 0, 0.1), 6)
    hc = to_module(mhc.HyperConnection(dim=D), p).to(DEV)
    ref_bi, ref_new = O.layer_forward(p.to(torch.float64), H.double(), torch.tanh)
    with torch.inference_mode():
        bi, add = hc(dev(H))
        H1 = add(torch.tanh(bi), pool_for_next=True)
        bi2, add2 = hc(H1)                      # consumes the attached sums
        assert_close(bi, ref_bi, RT, 2 * AT); assert_close(H1, ref_new, RT, 4 * AT)
    with torch.no_grad():
        bi, add = hc(dev(H))
        assert_close(add(torch.tanh(bi)), ref_new, RT, 4 * AT)
