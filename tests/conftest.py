import os
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def lib():
    from token2tile_b200 import _lib
    return _lib.load()


@pytest.fixture(scope="session")
def small_case():
    """H=2, N=4096 locality-mixture inputs and an oracle state (CPU tensors)."""
    from oracle import t2t_oracle as O
    from token2tile_b200.synth import GRIDS, locality_mixture
    H, N, CQ = 2, 4096, 32
    q, k, v = locality_mixture(H, GRIDS["cpu"])
    op = O.OracleOperator(H, N, CQ, s_frac=0.05)
    state = op.init_state(q, k)
    return dict(H=H, N=N, CQ=CQ, q=q, k=k, v=v, state=state)


def run_gloo_ranks(worker, world, args=(), attempts=3, timeout=180):
    """Spawn `world` CPU processes running worker(rank, world, port, queue, *args) and
    collect one queue item per rank.  A rendezvous can fail when another process
    grabs the port between probing and binding: the launch is retried on a fresh
    port before the test gives up."""
    import queue as _queue
    import socket
    import torch.multiprocessing as mp
    last = None
    for _ in range(attempts):
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            port = s.getsockname()[1]
        ctx = mp.get_context("spawn")
        q = ctx.Queue()
        procs = [ctx.Process(target=worker, args=(r, world, port, q, *args)) for r in range(world)]
        for p in procs:
            p.start()
        items = []
        try:
            for _ in procs:
                items.append(q.get(timeout=timeout))
        except _queue.Empty as exc:
            last = exc
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.terminate()
        if len(items) == world:
            return items
    raise AssertionError(f"gloo ranks did not finish after {attempts} attempts: {last!r}")
