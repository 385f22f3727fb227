"""Two GPU ranks over NCCL: batch-sharded HyperConnection with the in-backward gradient all-reduce
against the unsharded CPU oracle, the sequence-sharded wrapper, and the layer under FSDP2
(`fully_shard`) against the same block run unsharded.  Skipped on boxes with fewer than two GPUs."""

import copy
import datetime
import os

import pytest
import torch
import torch.distributed as dist

from oracle import mhc_oracle as O
from tests import cases
from tests.util import run_ranks, to_module

pytestmark = pytest.mark.gpu

# A rank whose peer failed before a collective gives up after this long instead of sitting in an
# NCCL kernel until the default watchdog limit.
_PG_TIMEOUT = datetime.timedelta(seconds=90)


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=_PG_TIMEOUT)
    try:
        import mhc
        from mhc.parallel import GradSync, shard_batch
        torch.manual_seed(0)
        B, S, D = 6, 200, 128
        H = torch.randn(B, S, 4, D)
        g = torch.randn(B, S, 4, D)
        p = cases.perturb_params_(O.default_params(D, 0, 0.1), 3)
        full = O.layer_fwd_bwd(p, H, g, None, "fused", dtype=torch.float64)
        hc = to_module(mhc.HyperConnection(dim=D), p).to(dev)
        sync = GradSync([hc])
        Hs = shard_batch(H, rank, world).to(dev).requires_grad_(True)
        gs = shard_batch(g, rank, world).to(dev)
        lo = sum(shard_batch(H, r, world).shape[0] for r in range(rank))
        for _ in range(2):                      # the second pass overwrites the record, it must not accumulate
            Hs.grad = None
            bi, add = hc(Hs)
            H_new = add(bi)
            H_new.backward(gs)
            sync.finish()
        torch.cuda.synchronize()
        n = Hs.shape[0]
        for k, v in (("branch_input", bi), ("H_new", H_new), ("dH", Hs.grad)):
            ref = full[k][lo:lo + n]
            assert (v.double().cpu() - ref).abs().max() <= 2e-6 + 1e-5 * ref.abs().max(), k
        for name, q_ in hc.named_parameters():
            ref = full["d" + name]
            assert (q_.grad.double().cpu() - ref).abs().max() <= 1e-6 + 1e-5 * ref.abs().max(), name
        q.put((rank, "ok"))
    except Exception as e:
        q.put((rank, f"{type(e).__name__}: {e}"))
    finally:
        dist.destroy_process_group()


def _seq_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=_PG_TIMEOUT)
    try:
        import mhc
        from mhc.parallel import SequenceShardedHyperConnection
        torch.manual_seed(1)
        B, S, D = 3, 192, 64                     # fewer sequences than would keep 8 GPUs busy: shard the sequence
        H = torch.randn(B, S, 4, D)
        g = torch.randn(B, S, 4, D)
        p = cases.perturb_params_(O.default_params(D, 0, 0.1), 4)
        full = O.layer_fwd_bwd(p, H, g, None, "fused", dtype=torch.float64)
        hc = to_module(mhc.HyperConnection(dim=D), p).to(dev)
        sp = SequenceShardedHyperConnection(hc)
        Sl = S // world
        sl = slice(rank * Sl, (rank + 1) * Sl)
        Hs = H[:, sl].contiguous().to(dev).requires_grad_(True)
        bi, add = sp(Hs)
        H_new = add(bi)
        H_new.backward(g[:, sl].contiguous().to(dev))
        torch.cuda.synchronize()
        for k, v in (("branch_input", bi), ("H_new", H_new), ("dH", Hs.grad)):
            ref = full[k][:, sl]
            assert (v.double().cpu() - ref).abs().max() <= 2e-6 + 1e-5 * ref.abs().max(), k
        for name, q_ in hc.named_parameters():     # complete on every rank, no further reduction
            ref = full["d" + name]
            assert (q_.grad.double().cpu() - ref).abs().max() <= 1e-6 + 1e-5 * ref.abs().max(), name
        q.put((rank, "ok"))
    except Exception as e:
        q.put((rank, f"{type(e).__name__}: {e}"))
    finally:
        dist.destroy_process_group()


def _adam_worker(rank, world, port, q):
    """Three Adam steps with the stock `opt.zero_grad()` (set_to_none=True) under GradSync on a batch
    shard per rank equal three Adam steps of the same layer on the whole batch without GradSync."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=_PG_TIMEOUT)
    try:
        import mhc
        from mhc.parallel import GradSync, shard_batch
        torch.manual_seed(3)
        B, S, D = 4, 96, 64
        H = torch.randn(B, S, 4, D)
        g = torch.randn(B, S, 4, D)
        p = cases.perturb_params_(O.default_params(D, 0, 0.1), 9)
        layer = to_module(mhc.HyperConnection(dim=D), p).to(dev)
        ref = copy.deepcopy(layer)
        sync = GradSync([layer])
        opt = torch.optim.Adam(layer.parameters(), lr=1e-2)
        ref_opt = torch.optim.Adam(ref.parameters(), lr=1e-2)
        Hs, gs = shard_batch(H, rank, world).to(dev), shard_batch(g, rank, world).to(dev)
        Hf, gf = H.to(dev), g.to(dev)
        start = layer.phi.detach().clone()
        for _ in range(3):
            opt.zero_grad()
            assert layer.phi.grad is None
            bi, add = layer(Hs)
            add(bi).backward(gs)
            sync.finish()
            assert layer.phi.grad is not None
            opt.step()
            ref_opt.zero_grad()
            bi, add = ref(Hf)
            add(bi).backward(gf)
            ref_opt.step()
        torch.cuda.synchronize()
        assert (layer.phi - start).abs().max() > 1e-3
        for (name, a), (_, b) in zip(layer.named_parameters(), ref.named_parameters()):
            assert (a - b).abs().max() <= 1e-4 * (1 + b.abs().max()), name
        q.put((rank, "ok"))
    except Exception as e:
        q.put((rank, f"{type(e).__name__}: {e}"))
    finally:
        dist.destroy_process_group()


class _Block(torch.nn.Module):
    """A residual block around the layer: H_new = add_residual(tanh(Linear(branch_input)))."""

    def __init__(self, hc, D):
        super().__init__()
        self.hc = hc
        self.branch = torch.nn.Linear(D, D)

    def forward(self, H):
        branch_input, add_residual = self.hc(H)
        return add_residual(torch.tanh(self.branch(branch_input)))


def _fsdp_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=_PG_TIMEOUT)
    try:
        import mhc
        from mhc.parallel import shard_batch
        from torch.distributed.fsdp import fully_shard
        torch.manual_seed(2)
        B, S, D = 4, 160, 128
        H = torch.randn(B, S, 4, D)
        g = torch.randn(B, S, 4, D)
        p = cases.perturb_params_(O.default_params(D, 0, 0.1), 5)
        ref = _Block(to_module(mhc.HyperConnection(dim=D), p), D).to(dev)   # same seed: same Linear on every rank
        blk = copy.deepcopy(ref)
        fully_shard(blk.hc)            # the layer's parameters are sharded, gathered for forward and backward,
        fully_shard(blk)               # and freed in between (the layer is not the root)
        Hf = H.to(dev).requires_grad_(True)
        out_f = ref(Hf)
        out_f.backward(g.to(dev))
        Hs = shard_batch(H, rank, world).to(dev).requires_grad_(True)
        lo = sum(shard_batch(H, r, world).shape[0] for r in range(rank))
        n = Hs.shape[0]
        for _ in range(2):
            Hs.grad = None
            blk.zero_grad(set_to_none=True)
            out = blk(Hs)
            out.backward(shard_batch(g, rank, world).to(dev))
        torch.cuda.synchronize()
        for k, a, b in (("H_new", out, out_f[lo:lo + n]), ("dH", Hs.grad, Hf.grad[lo:lo + n])):
            assert (a - b).abs().max() <= 1e-5 * (1 + b.abs().max()), k
        for (name, prm), (_, rp) in zip(blk.named_parameters(), ref.named_parameters()):
            got = prm.grad.full_tensor() * world          # FSDP averages over ranks; the unsharded run sums
            assert got.shape == rp.grad.shape, name
            assert (got - rp.grad).abs().max() <= 1e-5 * (1 + rp.grad.abs().max()), name
        q.put((rank, "ok"))
    except Exception as e:
        q.put((rank, f"{type(e).__name__}: {e}"))
    finally:
        dist.destroy_process_group()


def _spawn2(worker):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    results = run_ranks(worker, 2, timeout=300)
    assert results == [(0, "ok"), (1, "ok")], results


def test_two_gpu_fsdp2_block_matches_unsharded():
    _spawn2(_fsdp_worker)


def test_two_gpu_sequence_sharded_layer_matches_oracle():
    _spawn2(_seq_worker)


def test_two_gpu_sharded_layer_matches_oracle():
    _spawn2(_worker)


def test_two_gpu_adam_steps_with_stock_zero_grad():
    _spawn2(_adam_worker)
