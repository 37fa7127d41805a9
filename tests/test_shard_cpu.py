"""CPU tests of the multi-GPU host logic: the row partition, and a world-size-2 gloo run in
which each rank computes its row shard (with the CPU oracle standing in for the device) and
the gathered slices equal the unsharded result."""
import ctypes as C
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from modgrad_b200 import _lib, decoder as dec, shard, synth

ROOT = Path(__file__).resolve().parent.parent


def test_row_range_partitions_exactly():
    for n in (1, 7, 512, 3584, 18944, 152064):
        for world in (1, 2, 3, 4, 8):
            if n < world:
                continue
            spans = [shard.row_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1


@pytest.mark.parametrize("cfg", [dec.QWEN25_7B, dec.DecoderConfig(2, 8192, 64, 8, 128, 28672, 1024, 64)])
def test_decoder_shard_matches_c_abi(cfg, cuda):
    for world in (1, 2, 4, 8):
        seen = []
        for rank in range(world):
            sh = shard.decoder_shard(cfg, rank, world)
            out = (C.c_int * 8)()
            cs = cfg.c_struct()
            assert cuda.mg_decoder_shard_ranges(C.byref(cs), rank, world, out) == 0
            assert list(out)[:7] == [sh.h0, sh.h1, sh.kv0, sh.kv1, sh.d_loc, sh.f_loc, sh.v_loc]
            seen.append((sh.h0, sh.h1))
            hl, kvl = sh.h1 - sh.h0, sh.kv1 - sh.kv0
            assert hl % kvl == 0 and hl // kvl in (1, 2, 3, 4, 7, 8)   # group sizes the attention kernel has
        assert seen[0][0] == 0 and seen[-1][1] == cfg.n_heads
        assert all(a[1] == b[0] for a, b in zip(seen, seen[1:]))
    cs = dec.QWEN25_7B.c_struct()
    assert cuda.mg_decoder_shard_ranges(C.byref(cs), 0, 3, (C.c_int * 8)()) != 0   # 3 ranks do not divide
    with pytest.raises(ValueError):
        shard.decoder_shard(dec.QWEN25_7B, 0, 3)


def test_slices_reassemble():
    cfg = dec.DecoderConfig(1, 512, 4, 2, 128, 1024, 64, 8)
    lw = dec.layer_weights(cfg, 0, 3)
    for name, (o, i) in cfg.shapes().items():
        parts = []
        for rank in range(2):
            parts.append(shard.slice_layer(cfg, shard.decoder_shard(cfg, rank, 2), lw)[name])
        assert np.array_equal(np.concatenate(parts), lw[name]), name


def test_slices_of_other_k_quants_reassemble():
    """Row slices are whole rows of blocks whatever the block size (Q5_K 176 bytes, Q6_K 210): the typed engine
    shards such tensors over the same row ranges."""
    cfg = dec.DecoderConfig(1, 512, 4, 2, 128, 1024, 64, 8)
    lw = dec.layer_weights(cfg, 0, 3)
    rng = np.random.Generator(np.random.PCG64(5))
    for name, kind in (("wk", 5), ("wv", 6), ("wdown", 6), ("wo", 5)):
        o, i = cfg.shapes()[name]
        lw[name] = synth.kquant_matrix(kind, o, i, rng)
    for name, (o, i) in cfg.shapes().items():
        parts = [shard.slice_layer(cfg, shard.decoder_shard(cfg, rank, 2), lw)[name] for rank in range(2)]
        assert np.array_equal(np.concatenate(parts), lw[name]), name
        assert all(p.size * 2 == lw[name].size for p in parts), name


WORKER = r"""
import os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, os.environ["MG_ROOT"])
import oracle
from modgrad_b200 import shard, synth
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
orc = oracle.lib()
out_dim, in_dim = 300, 1024
rng = np.random.Generator(np.random.PCG64(5))
w = synth.q4k_matrix(out_dim, in_dim, rng)
x = synth.activations(in_dim, rng)
lo, hi = shard.row_range(out_dim, rank, world)
y_loc = orc.matvec(shard.q4k_rows(w, out_dim, in_dim, lo, hi), x, hi - lo, in_dim // 256, 2)
sizes = [shard.row_range(out_dim, r, world) for r in range(world)]
parts = [torch.empty(b - a, dtype=torch.float32) for a, b in sizes]
dist.all_gather(parts, torch.from_numpy(y_loc))
y = torch.cat(parts).numpy()
full = orc.matvec(w, x, out_dim, in_dim // 256, 2)
assert np.array_equal(y, full), "gathered row shards differ from the unsharded matvec"
if rank == 0:
    print("SHARD_OK")
dist.destroy_process_group()
"""


def test_world2_gloo_row_shards_gather_to_full(tmp_path, orc):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, MG_ROOT=str(ROOT), MASTER_ADDR="127.0.0.1", MASTER_PORT="29541")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29541", str(script)],
                       env=env, capture_output=True, text=True, timeout=240)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "SHARD_OK" in r.stdout
