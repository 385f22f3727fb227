"""Seeded inputs shared by the parity tests (drawn on the CPU so that every
implementation sees bit-identical values)."""

import torch

from oracle import mhc_oracle as O

PARAM_ORDER = ("H_post_base", "H_pre_base", "H_res_base", "phi", "alpha_pre", "alpha_post", "alpha_res")


def perturb_params_(p: "O.LayerParams", seed: int) -> "O.LayerParams":
    """Same recipe as tests/golden/make_golden.py:perturb_ for the fused parameter set:
    draws follow the registration order of the reference module's parameters."""
    gen = torch.Generator().manual_seed(seed)
    for name in PARAM_ORDER:
        t = getattr(p, name)
        if name == "phi":
            t.copy_(torch.randn(t.shape, generator=gen) * 0.02)
        elif name.startswith("alpha"):
            t.add_(torch.randn(t.shape, generator=gen) * 0.02)
        else:
            t.add_(torch.randn(t.shape, generator=gen) * 0.1)
    return p


def c1_inputs():
    """Config 1: fp32 H(2,128,4,512) and upstream gradient from seed 0."""
    torch.manual_seed(0)
    H = torch.randn(2, 128, 4, 512)
    g = torch.randn(2, 128, 4, 512)
    return H, g


def c1_params(tag: str) -> "O.LayerParams":
    p = O.default_params(512, 0, 0.1)
    return p if tag == "default" else perturb_params_(p, 5)
