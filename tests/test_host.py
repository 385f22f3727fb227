"""CPU-only checks: the C-ABI library loads and exports what the header declares, argument
validation returns status codes without touching a GPU, and the host-side module mirrors the
reference's interface."""

import ctypes
import os
import re

import pytest
import torch

from tests.conftest import ROOT


def header_functions():
    text = open(os.path.join(ROOT, "include", "mhc_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mhc_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from mhc import _lib
    lib = _lib.load()
    names = header_functions()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), n
    assert sorted(_lib.EXPORTS) == names
    assert lib.mhc_version() == 200


def test_status_codes_without_gpu():
    from mhc import _lib
    lib = _lib.load()
    # null pointers / bad arguments are rejected before any CUDA call
    assert lib.mhc_sinkhorn_fwd(None, None, 4, _lib.MHC_F32, 20, 1e-8, None) == 1
    assert b"null" in lib.mhc_last_error_string()
    assert lib.mhc_status_name(1) == b"MHC_ERR_NULL_POINTER"
    assert lib.mhc_sinkhorn_fwd(None, None, 0, _lib.MHC_F32, 20, 1e-8, None) == 0      # empty batch is a no-op
    assert lib.mhc_stream_mix_fwd(None, None, None, None, None, 2, 8, 16, 7, None) == 3  # unknown dtype
    assert lib.mhc_stream_mix_fwd(None, None, None, None, None, -1, 8, 16, 0, None) == 2
    # Scalar arguments are checked before pointers, so these cases pass null pointers throughout: even
    # if the check aimed at regressed, the null-pointer check behind it would still stop any launch.
    assert lib.mhc_add_residual_bwd(None, None, None, None, None, None, 8, None, 2, 64, 64, 0, None) == 5  # scratch too small
    assert lib.mhc_sinkhorn_bwd(None, None, None, 1, 0, 20, 1e-8, 9, None) == 4
    assert lib.mhc_add_residual_bwd(None, None, None, None, None, None, 1 << 30, None, 2, 64, 64, 0, None) == 1
    # a ticket pointer that is not 4-byte aligned is refused (host addresses; nothing is launched)
    buf = ctypes.create_string_buffer(64)
    p = (ctypes.addressof(buf) + 15) & ~15
    assert lib.mhc_add_residual_bwd(p, p, p, p, p, p, 1 << 30, p + 2, 2, 64, 64, 0, None) == 6
    assert lib.mhc_status_name(6) == b"MHC_ERR_MISALIGNED"
    with pytest.raises(_lib.MhcError):
        _lib.check(5)


def test_scratch_sizes():
    from mhc import _lib
    lib = _lib.load()
    B, S, D = 8, 4096, 4096
    n = lib.mhc_scratch_bytes(_lib.OP_STREAM_MIX_BWD, B, S, D, _lib.MHC_BF16)
    assert 0 < n < 64 << 20
    assert 0 < lib.mhc_scratch_bytes(_lib.OP_ADD_RESIDUAL_BWD, B, S, D, _lib.MHC_BF16) <= 4 << 20
    # per-batch-element layout: scratch is linear in B
    assert lib.mhc_scratch_bytes(_lib.OP_MEANPOOL_FWD, 2 * B, S, D, 1) == 2 * lib.mhc_scratch_bytes(_lib.OP_MEANPOOL_FWD, B, S, D, 1)
    assert lib.mhc_scratch_bytes(99, B, S, D, 1) < 0 and lib.mhc_scratch_bytes(0, -1, S, D, 1) < 0
    # dynamic weights: per-row records only below 64 rows; from 64 rows on (per-token use) also the
    # grad_phi partial sums of up to 32 row tiles and the column sums of up to 64 summing CTAs
    K = 4 * D
    few = lib.mhc_scratch_bytes(_lib.OP_DYNAMIC_WEIGHTS_BWD, 16, 0, D, 0)
    assert few == 16 * 56 * 4
    many = lib.mhc_scratch_bytes(_lib.OP_DYNAMIC_WEIGHTS_BWD, 32768, 0, D, 0)
    tc = 64 + 64 + 2 * 32 * K     # the tensor-core pass: alignment slack, status header, phi split in two [K, 32]
    assert many == 4 * (32768 * 56 + 32 * K * 24 + 64 * 27 * 2 + 2 + tc)
    one_tile = lib.mhc_scratch_bytes(_lib.OP_DYNAMIC_WEIGHTS_BWD, 100, 0, D, 0)
    assert one_tile == 4 * (100 * 56 + 1 * K * 24 + 64 * 27 * 2 + 2 + tc)
    # forward: [row, K slice, 25] partial sums with at most 128 slices of at least 256 k (few rows); from 64 rows on
    # at least the tensor-core projection's split copy of phi (256-byte header + two [32, K] arrays)
    assert lib.mhc_scratch_bytes(_lib.OP_DYNAMIC_WEIGHTS_FWD, 64, 0, D, 0) == 256 + 2 * 32 * K * 4
    assert lib.mhc_scratch_bytes(_lib.OP_DYNAMIC_WEIGHTS_FWD, 8, 0, D, 0) == 8 * 64 * 25 * 4


def test_no_cpu_fallback():
    import mhc
    with pytest.raises(RuntimeError, match="CUDA"):
        mhc.sinkhorn_knopp(torch.randn(2, 4, 4))
    with pytest.raises(RuntimeError, match="CUDA"):
        mhc.fused_stream_mix(torch.randn(1, 2, 4, 8), torch.rand(1, 4), torch.rand(1, 4, 4))
    hc = mhc.HyperConnection(dim=8)
    with pytest.raises(RuntimeError, match="CUDA"):
        hc(torch.randn(1, 2, 4, 8))


def test_shape_errors_are_assertion_errors():
    import mhc
    with pytest.raises(AssertionError):
        mhc.sinkhorn_knopp(torch.randn(2, 3, 4))
    with pytest.raises(AssertionError):
        mhc.fused_stream_mix(torch.randn(1, 2, 3, 8), torch.rand(1, 4), torch.rand(1, 4, 4))
    with pytest.raises(AssertionError):
        mhc.fused_dynamic_weights(torch.randn(2, 16), torch.randn(16, 23), torch.randn(24), torch.ones(1),
                                  torch.ones(1), torch.ones(1))


def test_module_interface_matches_reference():
    import mhc
    with pytest.raises(ValueError, match="num_streams=4"):
        mhc.HyperConnection(dim=8, num_streams=2)
    hc = mhc.HyperConnection(dim=16, layer_idx=6, init_scale=0.25)
    assert list(hc.state_dict().keys()) == ["H_post_base", "H_pre_base", "H_res_base", "phi", "alpha_pre",
                                            "alpha_post", "alpha_res"]
    assert hc.phi.shape == (64, 24) and hc.alpha_pre.shape == (1,)
    assert torch.equal(hc.H_pre_base.data, torch.tensor([0., 0., 1., 0.]))
    assert torch.equal(hc.H_res_base.data, torch.eye(4)) and float(hc.alpha_res.detach()) == 0.25
    assert "use_fused_weights=True" in repr(hc) and "dim=16" in repr(hc)
    with torch.no_grad():
        hc.phi.add_(1.0); hc.alpha_pre.fill_(3.0)
    hc.init_weights(layer_idx=1)
    assert float(hc.phi.detach().abs().sum()) == 0 and float(hc.alpha_pre.detach()) == 0.25
    assert torch.equal(hc.H_pre_base.data, torch.tensor([0., 1., 0., 0.]))
    un = mhc.HyperConnection(dim=16, use_fused_weights=False)
    assert list(un.state_dict().keys()) == ["H_post_base", "H_pre_base", "H_res_base", "scale_post", "scale_pre",
                                            "scale_res", "W_post.weight", "W_pre.weight", "W_res.weight"]
    st = mhc.HyperConnection(dim=16, dynamic=False, use_fused_weights=True)
    assert st.use_fused_weights is False and list(st.state_dict().keys()) == ["H_post_base", "H_pre_base", "H_res_base"]


def test_package_surface():
    import mhc
    for name in ("HyperConnection", "sinkhorn_knopp", "fused_stream_mix", "fused_add_residual",
                 "fused_dynamic_weights"):
        assert name in mhc.__all__ and hasattr(mhc, name)
    assert mhc.__version__ == "0.1.0"
    with pytest.raises(ValueError):
        mhc.set_abs_grad_at_zero("minus")
