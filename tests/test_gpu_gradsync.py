"""GradSync on one GPU inside a stock training loop: `optimizer.zero_grad()` (which sets every
.grad to None) followed by backward, `finish()` and `optimizer.step()`.  The layer that writes its
parameter gradients into the flat record must train exactly like the same layer without GradSync
(parameter update pattern of the reference's training test, tests/test_mhc.py:181-206 there)."""

import copy

import pytest
import torch

from oracle import mhc_oracle as O
from tests import cases
from tests.util import to_module

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("set_to_none", [True, False])
def test_adam_steps_under_gradsync_equal_plain_autograd(set_to_none):
    import mhc
    from mhc.parallel import GradSync
    dev = torch.device("cuda", 0)
    torch.manual_seed(11)
    B, S, D = 3, 130, 96
    H = torch.randn(B, S, 4, D, device=dev)
    g = torch.randn(B, S, 4, D, device=dev)
    layer = to_module(mhc.HyperConnection(dim=D), cases.perturb_params_(O.default_params(D, 0, 0.1), 13)).to(dev)
    plain = copy.deepcopy(layer)
    sync = GradSync([layer])
    opt = torch.optim.Adam(layer.parameters(), lr=1e-2)
    plain_opt = torch.optim.Adam(plain.parameters(), lr=1e-2)
    start = {k: v.detach().clone() for k, v in layer.named_parameters()}
    for _ in range(3):
        opt.zero_grad(set_to_none=set_to_none)
        if set_to_none:
            assert layer.phi.grad is None
        bi, add = layer(H)
        add(torch.tanh(bi)).backward(g)
        sync.finish()
        assert layer.phi.grad is not None and layer.phi.grad.data_ptr() == sync.flat.data_ptr()
        opt.step()
        plain_opt.zero_grad()
        bi, add = plain(H)
        add(torch.tanh(bi)).backward(g)
        plain_opt.step()
    for (name, a), (_, b) in zip(layer.named_parameters(), plain.named_parameters()):
        assert (a - start[name]).abs().max() > 0, f"{name} never changed"
        assert torch.equal(a, b), f"{name}: {float((a - b).abs().max()):.3e}"
