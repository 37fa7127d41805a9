"""Worker of the bounded-wait test in tests/test_gpu_sharded.py (world 2, one process per GPU).

Both ranks decode two tokens together.  Then — between steps, with nothing in flight — rank 1 simply
does not launch its next token.  Rank 0 launches alone: its wait for rank 1's output (the consumer's
poll of the stamped words, or the flag handshake in the "fused" mode) runs out under a lowered spin
limit, the kernels return, the token fails with a time-out status that names the exchange, the next
token fails at once, and the CUDA context stays usable (a plain matvec afterwards is correct).
Nothing faults or hangs; both ranks leave together after a host barrier."""
import os
import sys
import time
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

import oracle  # noqa: E402
from modgrad_b200 import decoder as dec, shard, synth  # noqa: E402
from modgrad_b200.backend import DeviceBuffer, Runtime, kern  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("gloo")
    cfg = dec.DecoderConfig(n_layers=2, d_model=512, n_heads=8, n_kv_heads=2, head_dim=128, d_ff=1024, vocab=640,
                            max_seq=40)
    d = dec.Q4KDecoder(cfg, rank, world, shard.nccl_id_from_torch(rank))
    d.load_random(3)
    d.set_exchange_spin_limit(1 << 16)          # a fraction of a second instead of seconds
    for tok in (5, 9):                          # two healthy steps
        d.forward_token(tok)
    dist.barrier()
    result = "idle"
    if rank == 0:                               # rank 1 skips this step: nothing of it is in flight
        t0 = time.perf_counter()
        try:
            d.forward_token(11)
            result = "no error"
        except Runtime as e:
            result = f"timeout: {e}"
        first = time.perf_counter() - t0
        t0 = time.perf_counter()
        try:
            d.forward_token(12)
            result += " | second: no error"
        except Runtime:
            result += " | second failed"
        second = time.perf_counter() - t0
        # the context is still usable: an ordinary matvec gives the right answer
        orc = oracle.lib()
        rng = np.random.Generator(np.random.PCG64(1))
        w, x = synth.q4k_matrix(256, 1024, rng), synth.activations(1024, rng)
        wd, xd, yd = DeviceBuffer(w.nbytes), DeviceBuffer(x.nbytes), DeviceBuffer(1024)
        wd.copy_from_host_bytes(w)
        xd.copy_from_host(x)
        kern.matvec_q4k(wd.ptr, xd.ptr, yd.ptr, 256, 4)
        kern.sync()
        y64 = orc.matvec_f64(w, x, 256, 4)
        err = float(np.max(np.abs(yd.copy_to_host(256) - y64)) / np.sqrt(np.mean(y64 ** 2)))
        result += f" | matvec_err={err:.1e} first={first:.3f}s second={second:.3f}s"
        assert err <= 1e-5
    dist.barrier()                              # both ranks leave together
    outs = [None] * world
    dist.all_gather_object(outs, result)
    if rank == 0:
        print("TIMEOUT_RESULT", outs[0], flush=True)
    d.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
