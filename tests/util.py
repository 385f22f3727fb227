"""Comparison helpers for the parity tests."""


def maxdiff(a, b):
    return float((a.detach().double().cpu() - b.detach().double().cpu()).abs().max()) if a.numel() else 0.0


def assert_close(a, b, rtol, atol, what=""):
    """Element-wise |a-b| <= atol + rtol*|b|."""
    a, b = a.detach().double().cpu(), b.detach().double().cpu()
    assert a.shape == b.shape, (what, a.shape, b.shape)
    bad = (a - b).abs() > atol + rtol * b.abs()
    assert not bad.any(), f"{what}: {int(bad.sum())}/{a.numel()} outside tol, max abs diff {float((a - b).abs().max()):.3e}"


def assert_close_norm(a, b, rtol, atol, what="", extra=0.0):
    """Norm-wise max|a-b| <= atol + rtol*max|b| (+ extra)."""
    a, b = a.detach().double().cpu(), b.detach().double().cpu()
    assert a.shape == b.shape, (what, a.shape, b.shape)
    if a.numel() == 0:
        return
    d = float((a - b).abs().max())
    lim = atol + rtol * float(b.abs().max()) + extra
    assert d <= lim, f"{what}: max abs diff {d:.3e} > {lim:.3e}"


def to_module(hc, params):
    """Copy oracle LayerParams into a HyperConnection (names match the state dict)."""
    sd = {}
    for k, v in params.tensors().items():
        sd[k + ".weight" if k.startswith("W_") else k] = v.detach().clone()
    hc.load_state_dict(sd)
    return hc


def free_port():
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def run_ranks(worker, world, *args, timeout=300):
    """Run `worker(rank, world, port, *args, queue)` on `world` spawned child processes and return
    the sorted list of what they put on the queue.  Whatever happens (a rank raised before a
    collective, a timeout while waiting), children that are still alive afterwards are terminated,
    so no rank is left waiting inside a collective after the test has ended."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=worker, args=(r, world, port) + tuple(args) + (q,), daemon=True)
             for r in range(world)]
    for pr in procs:
        pr.start()
    try:
        results = [q.get(timeout=timeout) for _ in procs]
        for pr in procs:
            pr.join(timeout=60)
    finally:
        for pr in procs:
            if pr.is_alive():
                pr.terminate()
        for pr in procs:
            pr.join(timeout=10)
            if pr.is_alive():
                pr.kill()
    return sorted(results)
