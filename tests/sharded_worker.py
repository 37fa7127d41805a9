"""Worker of tests/test_gpu_sharded.py: one rank of a row-sharded decode (launched by
torch.distributed.run, one process per GPU).  Every rank checks ITS slice of the logits against
the CPU oracle's full logits for a teacher-forced token sequence, and that greedy generation
picks the same tokens on every rank."""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

import oracle  # noqa: E402
from modgrad_b200 import decoder as dec, shard  # noqa: E402
from oracle.loader import MODE_F64  # noqa: E402
from test_gpu_decoder import oracle_model  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("gloo")  # host-side plumbing only: the data path gathers with NCCL inside the engine
    cfg = dec.DecoderConfig(n_layers=2, d_model=512, n_heads=8, n_kv_heads=2, head_dim=128, d_ff=1024, vocab=640,
                            max_seq=40)
    seed, prefill = 21, 10
    nccl_id = shard.nccl_id_from_torch(rank)
    d = dec.Q4KDecoder(cfg, rank, world, nccl_id)
    d.load_random(seed, prefill=prefill)
    orc = oracle.lib()
    ccfg, layers, g, keep = oracle_model(orc, cfg, seed, prefill)
    sh = d.shard
    worst = 0.0
    for step, tok in enumerate([5, 77, 601, 9]):
        want = orc.forward_token(ccfg, layers, g["embed"], g["lm_head"], g["out_norm"], prefill + step, tok, MODE_F64)
        got, nxt = d.forward_token(tok)
        mine = want[rank * sh.v_loc:(rank + 1) * sh.v_loc]
        err = float(np.max(np.abs(got - mine)) / np.sqrt(np.mean(want.astype(np.float64) ** 2)))
        worst = max(worst, err)
        # every rank learns of a failure on the host and all leave together, between steps: a rank
        # that left alone would keep the others waiting inside their next exchange
        verdicts = [None] * world
        dist.all_gather_object(verdicts, (rank, step, err, nxt, int(orc.argmax(want))))
        bad = [v for v in verdicts if not (v[2] < 1e-3 and v[3] == v[4])]
        assert not bad, bad
    modes = [None] * world
    dist.all_gather_object(modes, d.gather_mode())
    assert all(m == os.environ.get("MODGRAD_DECODER_GATHER", "stamped") for m in modes), modes
    d.set_position(0)
    toks, ms = d.generate(3, 8)
    gathered = [None] * world
    dist.all_gather_object(gathered, toks.tolist())
    assert all(t == gathered[0] for t in gathered), gathered
    if rank == 0:
        print(f"SHARDED_OK world={world} worst_logit_err={worst:.2e} tokens={gathered[0]}", flush=True)
    d.close()
    peer_matvec_check(rank, world, orc)
    dist.destroy_process_group()


def peer_matvec_check(rank, world, orc):
    """The public exchange: every rank computes ITS rows of two matvecs straight into the shared
    arena with the all-gather fused into the kernel; all ranks must end up with the full vectors."""
    import ctypes as C
    from modgrad_b200 import _lib, synth
    lib = _lib.load()
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    out_dim, in_dim = 1024, 1536
    rng = np.random.Generator(np.random.PCG64(77))
    ws = [synth.q4k_matrix(out_dim, in_dim, rng) for _ in range(2)]
    x = synth.activations(in_dim, rng)
    lo, hi = rank * out_dim // world, (rank + 1) * out_dim // world
    row_bytes = in_dim // 256 * 144
    handle, xh = (C.c_ubyte * 64)(), C.c_void_p()
    off0 = lib.mg_peer_arena_offset()
    assert lib.mg_peer_exchange_create(off0 + 2 * 4 * out_dim, rank, world, handle, C.byref(xh)) == 0
    gathered = [None] * world
    dist.all_gather_object(gathered, bytes(handle))
    blob = (C.c_ubyte * (64 * world)).from_buffer_copy(b"".join(gathered))
    assert lib.mg_peer_exchange_open(xh, blob) == 0
    dist.barrier()
    arena = lib.mg_peer_arena(xh)
    xd = torch.from_numpy(x).to(dev)
    for rep in range(3):  # alternating buffers, as the contract asks
        for site, w in enumerate(ws):
            wd = torch.from_numpy(np.ascontiguousarray(w[lo * row_bytes:hi * row_bytes])).to(dev)
            assert lib.mg_peer_fuse_next(xh, site) == 0
            assert lib.launch_matvec_q4k_on_stream(wd.data_ptr(), xd.data_ptr(), arena + off0 + 4 * (site * out_dim + lo),
                                                   hi - lo, in_dim // 256, None) == 0
    torch.cuda.synchronize()
    assert lib.mg_peer_exchange_status(xh) == 0
    for site, w in enumerate(ws):
        got = np.empty(out_dim, np.float32)
        assert lib.mg_memcpy_d2h(got.ctypes.data_as(C.c_void_p), arena + off0 + 4 * site * out_dim, 4 * out_dim) == 0
        want = orc.matvec_f64(w, x, out_dim, in_dim // 256)
        err = float(np.max(np.abs(got - want)) / np.sqrt(np.mean(want.astype(np.float64) ** 2)))
        assert err <= 1e-5, (rank, site, err)
    dist.barrier()
    lib.mg_peer_exchange_destroy(xh)
    if rank == 0:
        print(f"PEER_MATVEC_OK world={world}", flush=True)


if __name__ == "__main__":
    main()
