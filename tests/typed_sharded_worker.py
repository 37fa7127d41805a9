"""Worker of tests/test_gpu_sharded.py: one rank of a row-sharded TYPED engine (Q4_K / Q5_K / Q6_K
projections, Q6_K embedding and LM head), loaded from a GGUF file this rank writes, launched by
torch.distributed.run with one process per GPU.  Every rank checks its slice of the logits against a
forward pass composed from the CPU oracle's pieces, and that greedy generation picks the same tokens
on every rank."""
import os
import sys
import tempfile
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

import gguf_writer as gw  # noqa: E402
import oracle  # noqa: E402
from modgrad_b200 import decoder as dec, shard  # noqa: E402
from test_gpu_decoder_typed import MIX, Q6, mixed_model, oracle_forward  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("gloo")  # host-side plumbing only
    cfg = dec.DecoderConfig(n_layers=2, d_model=512, n_heads=8, n_kv_heads=2, head_dim=128, d_ff=1024, vocab=640,
                            max_seq=40, rms_eps=1e-6, rope_base=1e6)
    layers, g = mixed_model(cfg, 51, MIX, Q6, Q6)
    nccl_id = shard.nccl_id_from_torch(rank)
    with tempfile.TemporaryDirectory() as tmp:
        path = Path(tmp) / f"mixed_rank{rank}.gguf"
        path.write_bytes(gw.decoder_gguf(cfg, layers, g))
        d = dec.Q4KDecoder.from_gguf(path, cfg.max_seq, rank, world, nccl_id)
    assert d.weight_type(0, dec.W_V) == 14 and d.weight_type(0, dec.W_K) == 13 and d.weight_type(0, dec.W_LM_HEAD) == 14
    orc = oracle.lib()
    sh = d.shard
    caches = [(np.zeros(cfg.max_seq * cfg.kv_dim, dtype=np.float16), np.zeros(cfg.max_seq * cfg.kv_dim, dtype=np.float16))
              for _ in range(cfg.n_layers)]
    worst = 0.0
    for pos, tok in enumerate([5, 77, 601, 9]):
        want = oracle_forward(orc, cfg, layers, g, caches, pos, tok)
        got, nxt = d.forward_token(tok)
        mine = want[rank * sh.v_loc:(rank + 1) * sh.v_loc]
        err = float(np.max(np.abs(got - mine)) / np.sqrt(np.mean(want.astype(np.float64) ** 2)))
        worst = max(worst, err)
        # every rank learns of a failure on the host and all leave together, between steps
        verdicts = [None] * world
        dist.all_gather_object(verdicts, (rank, pos, err, nxt, int(orc.argmax(want))))
        bad = [v for v in verdicts if not (v[2] < 1e-3 and v[3] == v[4])]
        assert not bad, bad
    modes = [None] * world
    dist.all_gather_object(modes, d.gather_mode())
    # the typed engine has no stamped exchanges: it fuses with the flag handshake unless asked for less
    want_mode = {"nccl": "nccl", "peer": "peer"}.get(os.environ.get("MODGRAD_DECODER_GATHER", ""), "fused")
    assert all(m == want_mode for m in modes), modes
    d.set_position(0)
    toks, ms = d.generate(3, 8)
    gathered = [None] * world
    dist.all_gather_object(gathered, toks.tolist())
    assert all(t == gathered[0] for t in gathered), gathered
    if rank == 0:
        print(f"TYPED_SHARDED_OK world={world} mode={want_mode} worst_logit_err={worst:.2e} tokens={gathered[0]}", flush=True)
    d.close()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
