"""The allocation-free add-residual backward, called through the C ABI.

mhc_add_residual_bwd_noalloc exists for hosts that cannot hand the library scratch memory (no
device allocator of their own, or a loop that must never call cudaMalloc); its partial sums live
in a fixed array inside the library.  It must give what mhc_add_residual_bwd gives with
caller-provided scratch -- on a first call and again on a second call that reuses the same
array with different data -- and must refuse shapes that do not fit the array.

The file name sorts after every other test file on purpose: if this test fails, a run that stops
at the first failure has already run the rest of the suite.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _both(lib, L, g, bo, H_post):
    B, S, _, D = g.shape
    st = torch.cuda.current_stream().cuda_stream
    code = L.dtype_code(g)
    ref_dbo, ref_post = torch.empty_like(bo), torch.empty(B, 4, device=g.device)
    nbytes = lib.mhc_scratch_bytes(L.OP_ADD_RESIDUAL_BWD, B, S, D, code)
    scratch = torch.empty(nbytes // 4 + 1, device=g.device)
    L.check(lib.mhc_add_residual_bwd(g.data_ptr(), bo.data_ptr(), H_post.data_ptr(), ref_dbo.data_ptr(),
                                     ref_post.data_ptr(), scratch.data_ptr(), nbytes, None, B, S, D, code, st))
    new_dbo, new_post = torch.full_like(bo, float("nan")), torch.full((B, 4), float("nan"), device=g.device)
    L.check(lib.mhc_add_residual_bwd_noalloc(g.data_ptr(), bo.data_ptr(), H_post.data_ptr(), new_dbo.data_ptr(),
                                             new_post.data_ptr(), B, S, D, code, st))
    torch.cuda.synchronize()
    return (ref_dbo, ref_post), (new_dbo, new_post)


def test_noalloc_matches_scratch_version_twice():
    from mhc import _lib as L
    lib = L.load()
    dev = "cuda"
    # two calls in a row, different shapes and data, the second reusing the array the first left dirty
    for seed, (B, S, D, dtype) in enumerate([(3, 200, 512, torch.bfloat16), (2, 130, 100, torch.float32)]):
        torch.manual_seed(seed)
        g = torch.randn(B, S, 4, D, device=dev).to(dtype)
        bo = torch.randn(B, S, D, device=dev).to(dtype)
        H_post = 2 * torch.sigmoid(torch.randn(B, 4, device=dev))
        (ref_dbo, ref_post), (new_dbo, new_post) = _both(lib, L, g, bo, H_post)
        # same kernels, same fixed reduction order: identical, and in any case within the suite's fp32 tolerance
        assert torch.equal(new_dbo, ref_dbo)
        assert torch.allclose(new_post, ref_post, rtol=1e-5, atol=1e-6)
        assert torch.equal(new_post, ref_post)
        # and both agree with a direct fp64 evaluation
        want = (g.double() * bo.double()[:, :, None, :]).sum((1, 3))
        assert (new_post.double() - want).abs().max() <= 1e-6 + 1e-5 * want.abs().max()


def test_noalloc_rejects_oversized_shapes():
    from mhc import _lib as L
    lib = L.load()
    cap = lib.mhc_add_residual_bwd_noalloc_max_bytes()
    assert cap == 1 << 20
    # Partial sums far beyond the built-in area.  The size check comes before the pointer checks, so the
    # call is made with null pointers: nothing could be launched even if the size check were lost.
    B, S, D = 64, 65536, 8192
    rc = lib.mhc_add_residual_bwd_noalloc(None, None, None, None, None, B, S, D, L.MHC_BF16, None)
    assert rc == 5 and b"built-in area" in lib.mhc_last_error_string()
