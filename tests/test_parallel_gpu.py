"""Two replicas on two GPUs: the gradient sum through peer memory inside the step's graph against
the NCCL all-reduce between two graphs (tests/dp_worker.py).  Skipped with fewer than two GPUs."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_peer_reduce_equals_nccl_on_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    worker = Path(__file__).parent / "dp_worker.py"
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29533", str(worker)]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert "DP_WORKER_OK" in res.stdout, res.stdout[-2000:] + res.stderr[-2000:]


def test_peer_buffer_create_exports_a_handle():
    """One process can only create and free its side of the rendezvous (opening one's own handle is not
    allowed by the driver); the two-process form is what dp_worker.py runs."""
    import ctypes as C

    from tiny_cnn_b200 import ops
    from tiny_cnn_b200._lib import check
    ctx = ops.Context(0)
    dev, handle = C.c_void_p(), (C.c_ubyte * 64)()
    check(ctx.lib.b200_peer_buffer_create(ctx.handle, 1 << 20, C.byref(dev), handle))
    assert dev.value and any(bytes(handle))
    ctx.sync()
    import cuda.bindings.runtime as rt  # read the fresh buffer back: it must be zero-filled
    host = (C.c_ubyte * 4096)()
    (err,) = rt.cudaMemcpy(C.addressof(host), dev.value, 4096, rt.cudaMemcpyKind.cudaMemcpyDeviceToHost)
    assert int(err) == 0 and not any(bytes(host))
    check(ctx.lib.b200_peer_buffer_destroy(ctx.handle, dev))
    assert ctx.lib.b200_peer_buffer_create(ctx.handle, 0, C.byref(dev), handle) != 0  # an empty buffer is refused
