"""Generate the golden fixtures in this directory from the reference itself.

Run where the reference checkout is available (it is not needed to run the
tests):

    MHC_REFERENCE_SRC=/path/to/mHC-triton/src python tests/golden/make_golden.py

The script imports the reference's pure-PyTorch implementation
(src/mhc/_torch_baseline.py, loaded by file path so that its Triton-backed
siblings are never touched), feeds it seeded CPU inputs and stores inputs,
outputs and autograd gradients as .npz files.  All tensors are float32 unless
a key ends in "_f64" (the same reference code run on float64 copies of the
inputs; the arbiter for summation-order noise).

Fixtures written:
  sinkhorn.npz         sinkhorn_knopp_torch fwd + grads; shapes/seeds of the
                       reference tests (tests/test_mhc.py:25-65) plus sign/zero cases
  dynamic_weights.npz  fused_dynamic_weights_torch fwd + all grads
  stream_mix.npz       fused_stream_mix_torch fwd + all grads
  add_residual.npz     fused_add_residual_torch fwd + all grads
  layer_small.npz      HyperConnectionTorch fwd+bwd, fused / unfused / static modes
  layer_c1.npz         HyperConnectionTorch on H(2,128,4,512): full parameter grads,
                       strided samples of the activations; default init and a
                       perturbed-parameter variant
"""

import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
SAMPLE_STRIDE = 97


def load_reference():
    src = os.environ.get("MHC_REFERENCE_SRC")
    if not src:
        raise SystemExit("set MHC_REFERENCE_SRC to the src/ directory of a checkout of the reference project")
    path = os.path.join(src, "mhc", "_torch_baseline.py")
    sys.dont_write_bytecode = True
    spec = importlib.util.spec_from_file_location("mhc_reference_torch_baseline", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def npy(t):
    return t.detach().cpu().numpy()


def save(name, d):
    np.savez_compressed(os.path.join(HERE, name), **{k: npy(v) if torch.is_tensor(v) else np.asarray(v)
                                                   for k, v in d.items()})
    print(name, {k: tuple(v.shape) for k, v in d.items() if hasattr(v, "shape")})


def gen_sinkhorn(ref):
    out = {}
    torch.manual_seed(42)
    M = torch.randn(4, 4, 4)
    out["M"] = M
    Ml = M.clone().requires_grad_(True)
    P = ref.sinkhorn_knopp_torch(Ml, 20, 1e-8)
    P.sum().backward()
    out["P"], out["dM_sumloss"] = P, Ml.grad
    dP = torch.randn(4, 4, 4)
    Ml = M.clone().requires_grad_(True)
    ref.sinkhorn_knopp_torch(Ml, 20, 1e-8).backward(dP)
    out["dP"], out["dM"] = dP, Ml.grad
    Md = M.double().requires_grad_(True)
    Pd = ref.sinkhorn_knopp_torch(Md, 20, 1e-8)
    Pd.backward(dP.double())
    out["P_f64"], out["dM_f64"] = Pd, Md.grad
    torch.manual_seed(42)
    M8 = torch.randn(8, 4, 4)
    out["M8"], out["P8"] = M8, ref.sinkhorn_knopp_torch(M8, 20, 1e-8)
    # other iteration counts / eps, exact zeros and a negative-only matrix
    torch.manual_seed(7)
    Mz = torch.randn(6, 4, 4)
    Mz[0] = torch.eye(4)
    Mz[1] = -Mz[1].abs()
    Mz[2, 1, :] = 0.0
    dPz = torch.randn(6, 4, 4)
    for it, eps in ((1, 1e-6), (5, 1e-6), (20, 1e-6)):
        Ml = Mz.clone().requires_grad_(True)
        Pz = ref.sinkhorn_knopp_torch(Ml, it, eps)
        Pz.backward(dPz)
        out[f"Pz_T{it}"], out[f"dMz_T{it}"] = Pz, Ml.grad
    out["Mz"], out["dPz"] = Mz, dPz
    save("sinkhorn.npz", out)


def gen_dynamic_weights(ref):
    torch.manual_seed(1)
    B, K = 3, 4 * 40
    x = torch.randn(B, K)
    phi = torch.randn(K, 24) * 0.05
    bias = torch.cat([torch.tensor([1.0, 0, 0, 0]), torch.ones(4), torch.eye(4).flatten()]) + 0.1 * torch.randn(24)
    al = [torch.tensor([0.1]), torch.tensor([0.2]), torch.tensor([0.3])]
    g_pre, g_post, g_res = torch.randn(B, 4), torch.randn(B, 4), torch.randn(B, 4, 4)
    out = dict(x=x, phi=phi, bias=bias, alpha_pre=al[0], alpha_post=al[1], alpha_res=al[2],
               g_pre=g_pre, g_post=g_post, g_res=g_res)
    for tag, dt in (("", torch.float32), ("_f64", torch.float64)):
        leaves = [t.clone().to(dt).requires_grad_(True) for t in (x, phi, bias, *al)]
        H_pre, H_post, H_res = ref.fused_dynamic_weights_torch(*leaves, 20, 1e-6)
        loss = (H_pre * g_pre.to(dt)).sum() + (H_post * g_post.to(dt)).sum() + (H_res * g_res.to(dt)).sum()
        loss.backward()
        out.update({"H_pre" + tag: H_pre, "H_post" + tag: H_post, "H_res" + tag: H_res})
        for nme, l in zip(("x", "phi", "bias", "alpha_pre", "alpha_post", "alpha_res"), leaves):
            out["d" + nme + tag] = l.grad
    save("dynamic_weights.npz", out)


def gen_stream_ops(ref):
    torch.manual_seed(42)
    B, S, D = 2, 8, 24
    H = torch.randn(B, S, 4, D)
    H_pre = torch.softmax(torch.randn(B, 4), -1)
    H_res = ref.sinkhorn_knopp_torch(torch.randn(B, 4, 4))
    g_bi, g_hr = torch.randn(B, S, D), torch.randn(B, S, 4, D)
    leaves = [t.clone().requires_grad_(True) for t in (H, H_pre, H_res)]
    bi, Hr = ref.fused_stream_mix_torch(*leaves)
    ((bi * g_bi).sum() + (Hr * g_hr).sum()).backward()
    save("stream_mix.npz", dict(H=H, H_pre=H_pre, H_res=H_res, g_bi=g_bi, g_hr=g_hr, bi=bi, Hr=Hr,
                                dH=leaves[0].grad, dH_pre=leaves[1].grad, dH_res=leaves[2].grad))
    bo = torch.randn(B, S, D)
    H_post = torch.sigmoid(torch.randn(B, 4)) * 2
    g = torch.randn(B, S, 4, D)
    leaves = [t.clone().requires_grad_(True) for t in (Hr.detach(), bo, H_post)]
    H_new = ref.fused_add_residual_torch(*leaves)
    H_new.backward(g)
    save("add_residual.npz", dict(Hr=Hr, bo=bo, H_post=H_post, g=g, H_new=H_new,
                                  dHr=leaves[0].grad, dbo=leaves[1].grad, dH_post=leaves[2].grad))


def perturb_(hc, seed):
    """Randomise every parameter in place so that no projected value sits on |.|'s kink."""
    gen = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for name, p in hc.named_parameters():
            if name == "phi" or name.startswith("W_"):
                p.copy_(torch.randn(p.shape, generator=gen) * 0.02)
            elif name.startswith("alpha") or name.startswith("scale"):
                p.add_(torch.randn(p.shape, generator=gen) * 0.02)
            else:
                p.add_(torch.randn(p.shape, generator=gen) * 0.1)


def run_layer(hc, H, g, branch):
    for p in hc.parameters():
        p.grad = None
    Hl = H.clone().requires_grad_(True)
    bi, add = hc(Hl)
    H_new = add(branch(bi))
    H_new.backward(g)
    res = {"branch_input": bi, "H_new": H_new, "dH": Hl.grad}
    for n, p in hc.named_parameters():
        res["d" + n.replace(".weight", "")] = p.grad if p.grad is not None else torch.zeros_like(p)
    return res


def gen_layer_small(ref):
    out = {}
    B, S, D = 2, 16, 64
    torch.manual_seed(3)
    H = torch.randn(B, S, 4, D)
    g = torch.randn(B, S, 4, D)
    Wb = torch.randn(D, D) / D ** 0.5
    out.update(H=H, g=g, Wb=Wb)
    for mode, kw in (("fused", dict(dynamic=True)), ("unfused", dict(dynamic=True, use_fused_weights=False)),
                     ("static", dict(dynamic=False))):
        hc = ref.HyperConnectionTorch(dim=D, layer_idx=1, **kw)
        perturb_(hc, 11)
        for n, p in hc.named_parameters():
            out[f"{mode}.param.{n.replace('.weight', '')}"] = p.detach().clone()
        res = run_layer(hc, H, g, lambda t: torch.tanh(t @ Wb))
        for k, v in res.items():
            out[f"{mode}.{k}"] = v
        hc64 = ref.HyperConnectionTorch(dim=D, layer_idx=1, **kw).double()
        hc64.load_state_dict({k: v.double() for k, v in hc.state_dict().items()})
        res = run_layer(hc64, H.double(), g.double(), lambda t: torch.tanh(t @ Wb.double()))
        for k, v in res.items():
            out[f"{mode}.{k}_f64"] = v
    save("layer_small.npz", out)


def c1_inputs():
    """Config 1 inputs (fp32 H of shape (2, 128, 4, 512)): seed 0, H then the upstream gradient."""
    torch.manual_seed(0)
    H = torch.randn(2, 128, 4, 512)
    g = torch.randn(2, 128, 4, 512)
    return H, g


def gen_layer_c1(ref):
    out = {}
    H, g = c1_inputs()
    out["H_sample"] = H.flatten()[::SAMPLE_STRIDE]
    out["g_sample"] = g.flatten()[::SAMPLE_STRIDE]
    for tag, seed in (("default", None), ("perturbed", 5)):
        hc = ref.HyperConnectionTorch(dim=512, num_streams=4, layer_idx=0, dynamic=True,
                                      sinkhorn_iters=20, init_scale=0.1)
        if seed is not None:
            perturb_(hc, seed)
        for dt_tag, dt in (("", torch.float32), ("_f64", torch.float64)):
            m = hc if dt == torch.float32 else None
            if m is None:
                m = ref.HyperConnectionTorch(dim=512, layer_idx=0).double()
                m.load_state_dict({k: v.double() for k, v in hc.state_dict().items()})
            res = run_layer(m, H.to(dt), g.to(dt), lambda t: t)
            for k, v in res.items():
                if k in ("branch_input", "H_new", "dH"):
                    out[f"{tag}.{k}_sample{dt_tag}"] = v.flatten()[::SAMPLE_STRIDE]
                    out[f"{tag}.{k}_sum{dt_tag}"] = v.double().sum()
                else:
                    out[f"{tag}.{k}{dt_tag}"] = v
    save("layer_c1.npz", out)


if __name__ == "__main__":
    torch.set_num_threads(1)   # fixed summation order inside the reference's reductions
    ref = load_reference()
    gen_sinkhorn(ref)
    gen_dynamic_weights(ref)
    gen_stream_ops(ref)
    gen_layer_small(ref)
    gen_layer_c1(ref)
