"""Row-sharded decode on 2+ GPUs of one node (skipped on a single GPU): one process per GPU,
output slices all-gathered inside the per-token graph — by peer stores fused into the producing
kernels (default), by a peer-store gather kernel, or by NCCL; every rank's logits slice is checked
against the CPU oracle, and the public peer exchange against the oracle matvec."""
import ctypes as C
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def gpu_count(cuda) -> int:
    n = C.c_int(0)
    return n.value if cuda.mg_get_device_count(C.byref(n)) == 0 else 0


@pytest.mark.parametrize("world,mode", [(2, "stamped"), (2, "fused"), (2, "peer"), (2, "nccl"), (4, "stamped"), (4, "fused"),
                                        (8, "stamped"), (8, "nccl")])
def test_sharded_decoder_matches_oracle(cuda, world, mode):
    if gpu_count(cuda) < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MODGRAD_DECODER_GATHER=mode)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                        "--master-addr", "127.0.0.1", "--master-port", str(29600 + world),
                        str(ROOT / "tests" / "sharded_worker.py")],
                       env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, (r.stdout[-1500:], r.stderr[-3000:])
    assert "SHARDED_OK" in r.stdout and "PEER_MATVEC_OK" in r.stdout, r.stdout[-1500:]


@pytest.mark.parametrize("world,mode", [(2, "stamped"), (2, "peer"), (2, "nccl"), (4, "peer")])
def test_sharded_typed_engine_from_a_mixed_gguf_matches_oracle(cuda, world, mode):
    """Q4_K / Q5_K / Q6_K projections with a Q6_K embedding and LM head, row-sharded: exchanges fused into the
    Q4_K / attention / SwiGLU kernels with a gather kernel behind the other types (the default), gather kernels
    only, or NCCL."""
    if gpu_count(cuda) < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MODGRAD_DECODER_GATHER=mode)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                        "--master-addr", "127.0.0.1", "--master-port", str(29700 + world),
                        str(ROOT / "tests" / "typed_sharded_worker.py")],
                       env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, (r.stdout[-1500:], r.stderr[-3000:])
    assert "TYPED_SHARDED_OK" in r.stdout, r.stdout[-1500:]


@pytest.mark.parametrize("mode", ["stamped", "fused"])
def test_bounded_wait_runs_out_when_a_peer_does_not_launch(cuda, mode):
    """A peer that skips a step between launches: the waiting rank's bounded wait expires, the token
    fails with a time-out that names the exchange, later tokens fail at once, the context stays
    usable.  No GPU is faulted or hung (NVLS off, plain peer stores)."""
    if gpu_count(cuda) < 2:
        pytest.skip("needs 2 GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MODGRAD_DECODER_GATHER=mode)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29650", str(ROOT / "tests" / "timeout_worker.py")],
                       env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, (r.stdout[-1500:], r.stderr[-3000:])
    line = [l for l in r.stdout.splitlines() if l.startswith("TIMEOUT_RESULT")]
    assert line, r.stdout[-1500:]
    assert "timeout:" in line[0] and "did not arrive" in line[0] and "second failed" in line[0], line[0]
