"""The in-kernel finish of the deterministic sums (ticket counters) against the separate finish
kernels: bit-identical outputs and gradients, counters left at zero, and programmatic dependent
launch on or off makes no difference to any result."""

import os
import subprocess
import sys

import pytest
import torch

from oracle import mhc_oracle as O
from tests import cases
from tests.conftest import ROOT
from tests.util import to_module

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _layer_step(dtype, B, S, D, seed):
    import mhc
    torch.manual_seed(seed)
    H = torch.randn(B, S, 4, D, device=DEV).to(dtype).requires_grad_(True)
    g = torch.randn(B, S, 4, D, device=DEV).to(dtype)
    hc = to_module(mhc.HyperConnection(dim=D), cases.perturb_params_(O.default_params(D, 0, 0.1), seed)).to(DEV)
    bi, add = hc(H)
    H_new = add(torch.tanh(bi))
    H_new.backward(g)
    out = {"branch_input": bi.detach(), "H_new": H_new.detach(), "dH": H.grad.detach()}
    out.update({"d" + k: v.grad.detach() for k, v in hc.named_parameters()})
    return out


@pytest.mark.parametrize("dtype,B,S,D", [(torch.float32, 3, 130, 96), (torch.bfloat16, 2, 513, 1024),
                                          (torch.bfloat16, 16, 64, 256), (torch.float32, 17, 40, 33)])
def test_ticket_finish_is_bit_identical(dtype, B, S, D):
    from mhc import _lib as L
    try:
        L.set_ticket_finish(True)
        a = _layer_step(dtype, B, S, D, 3)
        a2 = _layer_step(dtype, B, S, D, 3)              # a second run on the same (self-resetting) counters
        L.set_ticket_finish(False)
        b = _layer_step(dtype, B, S, D, 3)
    finally:
        L.set_ticket_finish(True)
    torch.cuda.synchronize()
    for k in a:
        assert torch.equal(a[k], b[k]), k
        assert torch.equal(a[k], a2[k]), k
    for buf in L._tickets.values():                      # every kernel left its counters at zero
        assert int(buf.abs().max()) == 0


def test_add_residual_bwd_tickets_through_c_abi():
    from mhc import _lib as L
    lib = L.load()
    torch.manual_seed(0)
    B, S, D = 5, 77, 200
    g = torch.randn(B, S, 4, D, device=DEV).bfloat16()
    bo = torch.randn(B, S, D, device=DEV).bfloat16()
    H_post = torch.rand(B, 4, device=DEV)
    st = torch.cuda.current_stream().cuda_stream
    nbytes = lib.mhc_scratch_bytes(L.OP_ADD_RESIDUAL_BWD, B, S, D, L.MHC_BF16)
    outs = []
    tick = torch.zeros(B, device=DEV, dtype=torch.int32)
    for t in (None, tick.data_ptr(), tick.data_ptr()):
        scratch = torch.empty(nbytes // 4 + 1, device=DEV)
        dbo, post = torch.empty_like(bo), torch.full((B, 4), float("nan"), device=DEV)
        L.check(lib.mhc_add_residual_bwd(g.data_ptr(), bo.data_ptr(), H_post.data_ptr(), dbo.data_ptr(), post.data_ptr(),
                                         scratch.data_ptr(), nbytes, t, B, S, D, L.MHC_BF16, st))
        outs.append((dbo, post))
    torch.cuda.synchronize()
    assert int(tick.abs().max()) == 0
    for dbo, post in outs[1:]:
        assert torch.equal(dbo, outs[0][0]) and torch.equal(post, outs[0][1])
    want = (g.double() * bo.double()[:, :, None, :]).sum((1, 3))
    assert (outs[1][1].double() - want).abs().max() <= 1e-6 + 1e-5 * want.abs().max()


_PDL_SCRIPT = r"""
import sys, torch
sys.path[:0] = [{root!r}, {pkg!r}]
import mhc
torch.manual_seed(5)
dev = "cuda"
layers = [mhc.HyperConnection(dim=256, layer_idx=i).to(dev) for i in range(3)]
gen = torch.Generator(device=dev).manual_seed(7)
for l in layers:
    with torch.no_grad():
        l.phi.copy_(torch.randn(l.phi.shape, device=dev, generator=gen) * 0.02)
H = torch.randn(2, 300, 4, 256, device=dev, generator=gen).bfloat16().requires_grad_(True)
h = H
for i, l in enumerate(layers):                 # every kernel reads what the kernel before it wrote
    bi, add = l(h)
    h = add(bi * 0.5, pool_for_next=(i + 1 < len(layers)))
h.backward(torch.randn(h.shape, device=dev, generator=gen).bfloat16())
torch.cuda.synchronize()
out = [h.detach().float().cpu(), H.grad.float().cpu()] + [p.grad.float().cpu() for l in layers for p in l.parameters()]
torch.save(out, sys.argv[1])
"""


def test_results_do_not_depend_on_programmatic_dependent_launch(tmp_path):
    """A three-layer chain with MHC_PDL=1 and MHC_PDL=0 (each in a process of its own: the switch is
    read once per process).  With dependent launch every kernel is scheduled while its producer still
    runs, so a load that slipped above the kernel's dependency wait would show up as a difference."""
    script = _PDL_SCRIPT.format(root=ROOT, pkg=os.path.join(ROOT, "mhc-triton_b200"))
    outs = []
    for flag in ("1", "0"):
        path = str(tmp_path / f"pdl{flag}.pt")
        env = dict(os.environ, MHC_PDL=flag)
        subprocess.run([sys.executable, "-c", script, path], check=True, env=env, timeout=600)
        outs.append(torch.load(path))
    for a, b in zip(*outs):
        assert torch.equal(a, b)


@pytest.mark.parametrize("rows,K", [(64, 64), (128, 32), (300, 4 * 100 + 4), (1000, 4 * 256), (4096 + 17, 2048)])
def test_many_rows_tensor_core_forward_status_and_parity(rows, K):
    """The tcgen05 forward of the many-rows dynamic weights: every bounded wait completed (status
    word 0), outputs within the fp32 band of the fp64 oracle, and the saved record (raw projections,
    sum of squares, inverse RMS) matches what the backward expects."""
    from mhc import _kernels as KK
    torch.manual_seed(rows + K)
    x = torch.randn(rows, K)
    phi = torch.randn(K, 24) * 0.05
    bias = torch.randn(24)
    al = [torch.tensor([0.3]), torch.tensor([-0.2]), torch.tensor([0.5])]
    a, b, c = O.dynamic_weights(x.double(), phi.double(), bias.double(), *[t.double() for t in al], 20, 1e-6)
    d = lambda t: t.to(DEV)
    a2, b2, c2, saved = KK.fused_dynamic_weights_forward(d(x), d(phi), d(bias), *[d(t) for t in al], 20, 1e-6, return_saved=True)
    torch.cuda.synchronize()
    assert int(KK.last_dynamic_weights_scratch.view(torch.int32)[0]) == 0
    from tests.util import assert_close
    assert_close(a2, a, 1e-5, 1e-6, "H_pre"); assert_close(b2, b, 1e-5, 1e-6, "H_post"); assert_close(c2, c, 2e-5, 4e-6, "H_res")
    raw = x.double() @ phi.double()
    assert (saved[:, :24].double().cpu() - raw).abs().max() <= 1e-5 * raw.abs().max() + 1e-6
    q = (x.double() ** 2).sum(-1)
    assert ((saved[:, 24].double().cpu() - q).abs() <= 1e-5 * q).all()
