"""Batch sharding + gradient all-reduce with two CPU ranks over gloo.

The device kernels are not involved: each rank obtains its shard's parameter gradients from
the CPU oracle, places them in the flat record that GradSync owns (the layout the CUDA backward
writes), and the SUM all-reduce must reproduce the unsharded gradients; activations and their
gradients must equal the corresponding slices of the unsharded run.
"""

import os

import pytest
import torch
import torch.distributed as dist

from oracle import mhc_oracle as O
from tests import cases
from tests.util import run_ranks


def _fill_record(layer, grads):
    K24 = 4 * layer.dim * 24
    rec = layer.grad_sink
    rec[:K24] = grads["dphi"].reshape(-1)
    rec[K24:K24 + 4] = grads["dH_pre_base"]
    rec[K24 + 4:K24 + 8] = grads["dH_post_base"]
    rec[K24 + 8:K24 + 24] = grads["dH_res_base"].reshape(-1)
    rec[K24 + 24] = grads["dalpha_pre"][0]
    rec[K24 + 25] = grads["dalpha_post"][0]
    rec[K24 + 26] = grads["dalpha_res"][0]


def _worker(rank, world, port, B, use_hook, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import mhc
        from mhc.parallel import GradSync, shard_batch
        torch.manual_seed(0)
        S, D = 24, 32
        H = torch.randn(B, S, 4, D)
        g = torch.randn(B, S, 4, D)
        p = cases.perturb_params_(O.default_params(D, 0, 0.1), 3)
        full = O.layer_fwd_bwd(p, H, g, None, "fused", dtype=torch.float64)
        Hs, gs = shard_batch(H, rank, world), shard_batch(g, rank, world)
        mine = O.layer_fwd_bwd(p, Hs, gs, None, "fused", dtype=torch.float64)
        lo = sum(shard_batch(H, r, world).shape[0] for r in range(rank))
        for k in ("branch_input", "H_new", "dH"):       # no communication needed for these
            ref = full[k][lo:lo + Hs.shape[0]]            # fp64; BLAS blocking may differ with the batch size
            assert (mine[k] - ref).abs().max() <= 1e-12 * (1 + ref.abs().max()), k
        layer = mhc.HyperConnection(dim=D)
        sync = GradSync([layer], overlap=True)            # CPU tensors: falls back to the in-line collective
        assert layer.phi.grad.data_ptr() == sync.flat.data_ptr()
        _fill_record(layer, {k: v.float() for k, v in mine.items()})
        if use_hook:
            layer.grads_ready_hook(layer.grad_sink)
            sync.finish()
        else:
            sync.all_reduce_now()
        for name, q_ in layer.named_parameters():
            ref = full["d" + name].float()
            assert q_.grad.shape == ref.shape
            assert (q_.grad - ref).abs().max() <= 1e-6 + 1e-5 * ref.abs().max(), name
        q.put((rank, "ok"))
    except Exception as e:  # report instead of hanging the peer
        q.put((rank, f"{type(e).__name__}: {e}"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("B,use_hook", [(4, False), (5, True)])
def test_two_rank_gradient_allreduce(B, use_hook):
    results = run_ranks(_worker, 2, B, use_hook, timeout=120)
    assert results == [(0, "ok"), (1, "ok")], results


def _params_of(layer):
    """The layer's current parameters as oracle LayerParams (detached copies)."""
    return O.LayerParams(**{k: v.detach().clone() for k, v in layer.named_parameters()})


def _optimizer_worker(rank, world, port, q):
    """Three Adam steps with the stock `opt.zero_grad()` (which sets every .grad to None) under GradSync
    must move the parameters exactly as three Adam steps on the unsharded gradients do."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import copy
        import mhc
        from mhc.parallel import GradSync, shard_batch
        from tests.util import to_module
        torch.manual_seed(0)
        B, S, D = 4, 16, 16
        H = torch.randn(B, S, 4, D)
        g = torch.randn(B, S, 4, D)
        layer = to_module(mhc.HyperConnection(dim=D), cases.perturb_params_(O.default_params(D, 0, 0.1), 7))
        ref = copy.deepcopy(layer)
        sync = GradSync([layer])
        opt = torch.optim.Adam(layer.parameters(), lr=1e-2)
        ref_opt = torch.optim.Adam(ref.parameters(), lr=1e-2)
        Hs, gs = shard_batch(H, rank, world), shard_batch(g, rank, world)
        start = layer.phi.detach().clone()
        for _ in range(3):
            opt.zero_grad()
            assert layer.phi.grad is None                       # this is what the stock call does
            mine = O.layer_fwd_bwd(_params_of(layer), Hs, gs, None, "fused")
            _fill_record(layer, mine)                           # what the CUDA backward does on a GPU
            layer.grads_ready_hook(layer.grad_sink)
            sync.finish()
            assert layer.phi.grad is not None and layer.phi.grad.data_ptr() == sync.flat.data_ptr()
            opt.step()
            full = O.layer_fwd_bwd(_params_of(ref), H, g, None, "fused")
            for name, q_ in ref.named_parameters():
                q_.grad = full["d" + name].clone()
            ref_opt.step()
        assert (layer.phi - start).abs().max() > 1e-3           # the optimizer did move the parameters
        for (name, a), (_, b) in zip(layer.named_parameters(), ref.named_parameters()):
            assert (a - b).abs().max() <= 1e-4 * (1 + b.abs().max()), name
        q.put((rank, "ok"))
    except Exception as e:
        q.put((rank, f"{type(e).__name__}: {e}"))
    finally:
        dist.destroy_process_group()


def test_three_adam_steps_with_stock_zero_grad():
    assert run_ranks(_optimizer_worker, 2, timeout=120) == [(0, "ok"), (1, "ok")]


def test_shard_batch_covers_batch_once():
    from mhc.parallel import shard_batch, sink_numel
    t = torch.arange(11)
    for world in (1, 2, 3, 4, 8):
        parts = [shard_batch(t, r, world) for r in range(world)]
        assert torch.equal(torch.cat(parts), t)
        assert max(len(p) for p in parts) - min(len(p) for p in parts) <= 1
    assert sink_numel(4096) == 16384 * 24 + 27


def test_gradsync_rejects_unsupported_layers():
    import mhc
    from mhc.parallel import GradSync
    with pytest.raises(ValueError):
        GradSync([])
    with pytest.raises(ValueError):
        GradSync([mhc.HyperConnection(dim=8, dynamic=False)])
    with pytest.raises(ValueError):
        GradSync([mhc.HyperConnection(dim=8).half()])


def _mismatch_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import datetime
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    try:
        import mhc
        from mhc.parallel import GradSync
        layers = [mhc.HyperConnection(dim=16 if rank == 0 else 32)]     # rank 1 was built with another width
        try:
            GradSync(layers)
            q.put((rank, "no error"))
        except ValueError as e:
            q.put((rank, "ValueError" if "disagree" in str(e) else str(e)))
    except Exception as e:
        q.put((rank, f"{type(e).__name__}: {e}"))
    finally:
        dist.destroy_process_group()


def test_mismatched_layers_are_reported_on_every_rank():
    """A configuration fault injected on the host: ranks built with different layer widths.  The
    check runs before any collective on gradients, so nothing hangs and every rank raises."""
    results = run_ranks(_mismatch_worker, 2, timeout=120)
    assert results == [(0, "ValueError"), (1, "ValueError")], results
