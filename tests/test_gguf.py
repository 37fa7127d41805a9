"""GGUF header parser (mg_gguf_*), no GPU needed: a writer in tests/ emits v2 / v3 files; the parser
must return what was written, with the reference's conversions and error messages
(crates/modgrad-device/src/kfd/gguf.rs:153-234, :236-252, :665-694)."""
import struct

import numpy as np
import pytest

import gguf_writer as gw
from modgrad_b200 import gguf
from modgrad_b200.backend import Runtime


def small_file(version=3):
    meta = [("general.architecture", gw.T_STR, "llama"), ("llama.block_count", gw.T_U32, 2),
            ("llama.context_length", gw.T_I32, 4096), ("llama.big", gw.T_U64, 2 ** 32 + 7),
            ("llama.rope.freq_base", gw.T_F32, 1e6), ("llama.eps64", gw.T_F64, 1e-6), ("flag", gw.T_BOOL, 1),
            ("u8", gw.T_U8, 200), ("i8", gw.T_I8, -3), ("u16", gw.T_U16, 60000), ("i16", gw.T_I16, -1234), ("i64", gw.T_I64, -5),
            ("tok", gw.T_ARR, (gw.T_STR, ["a", "bc", ""])),
            ("nested", gw.T_ARR, (gw.T_ARR, [(gw.T_U8, [1, 2]), (gw.T_U8, [])])),
            ("swa", gw.T_ARR, (gw.T_BOOL, [1, 0, 1]))]
    w = np.arange(2 * 144, dtype=np.uint8)
    n = np.arange(5, dtype=np.float32)
    tensors = [("blk.0.attn_q.weight", (256, 2), gw.GGML_Q4_K, w), ("norm", (5,), gw.GGML_F32, n),
               ("h", (3, 2), gw.GGML_F16, np.arange(6, dtype=np.float16))]
    return gw.write_gguf(meta, tensors, version=version), w, n


@pytest.mark.parametrize("version", [2, 3])
def test_parse_round_trip(version):
    data, w, n = small_file(version)
    with gguf.GgufFile.parse(data) as g:
        assert g.version == version and g.data_offset % 32 == 0
        assert g.meta_str("general.architecture") == "llama"
        assert g.meta_u32("llama.block_count") == 2
        assert g.meta_u32("llama.context_length") == 4096          # I32 -> u32 (gguf.rs:120)
        assert g.meta_u32("llama.big") == 7                         # U64 truncated (gguf.rs:121)
        assert g.meta_u32("llama.rope.freq_base") is None           # F32 is not a u32
        assert g.meta_f32("llama.rope.freq_base") == np.float32(1e6)
        assert g.meta_f32("llama.eps64") == np.float32(1e-6)        # F64 -> f32 (gguf.rs:128)
        assert g.meta_f32("llama.block_count") is None
        assert g.meta_str("missing") is None and g.meta_u32("missing") is None
        assert g.meta_array_len("tok") == 3 and g.meta_array_len("nested") == 2 and g.meta_array_len("flag") == -1
        ts = g.tensors()
        assert [t.name for t in ts] == ["blk.0.attn_q.weight", "norm", "h"]       # file order
        assert ts[0].dims == (256, 2) and ts[0].dtype == gguf.Q4_K and ts[0].data_bytes == 2 * 144
        assert ts[1].dims == (5,) and ts[1].data_bytes == 20 and ts[2].data_bytes == 12
        # tensor_file_offset = data_offset + offset; tensor data 32-byte aligned
        assert ts[0].file_offset == g.data_offset and all(t.file_offset % 32 == 0 for t in ts)
        assert data[ts[0].file_offset:ts[0].file_offset + 288] == w.tobytes()
        assert data[ts[1].file_offset:ts[1].file_offset + 20] == n.tobytes()


def test_block_sizes_match_the_reference_table(cuda):
    import ctypes as C
    want = {0: (4, 1), 1: (2, 1), 30: (2, 1), 2: (18, 32), 3: (20, 32), 6: (22, 32), 7: (24, 32), 8: (34, 32), 9: (36, 32),
            10: (84, 256), 11: (110, 256), 12: (144, 256), 13: (176, 256), 14: (210, 256), 15: (292, 256), 16: (0, 1), 99: (0, 1)}
    for dt, (bb, be) in want.items():
        b, e = C.c_size_t(), C.c_size_t()
        cuda.mg_gguf_block_size(dt, C.byref(b), C.byref(e))
        assert (b.value, e.value) == (bb, be), dt


def test_malformed_files_are_refused_with_the_reference_messages():
    data, _, _ = small_file()
    cases = [
        (b"GGML" + data[4:], "not a GGUF file"),
        (data[:4] + struct.pack("<I", 1) + data[8:], "unsupported GGUF version 1"),
        (data[:4] + struct.pack("<I", 4) + data[8:], "unsupported GGUF version 4"),
        (data[:3], "failed to fill whole buffer"),
        (data[:40], "failed to fill whole buffer"),                     # cut inside the metadata
        (data[:24] + struct.pack("<Q", 2_000_000) + data[32:], "string too long"),   # first key's length
    ]
    # an unknown metadata value type
    bad = bytearray(gw.write_gguf([("k", gw.T_U32, 1)], []))
    at = 24 + 8 + 1
    bad[at:at + 4] = struct.pack("<I", 13)
    cases.append((bytes(bad), "unknown GGUF value type 13"))
    # a tensor count far beyond the file
    cases.append((data[:8] + struct.pack("<Q", 10 ** 12) + data[16:], "failed to fill whole buffer|string too long"))
    for blob, msg in cases:
        with pytest.raises(Runtime, match=msg):
            gguf.GgufFile.parse(blob)
    with pytest.raises(Runtime, match="cannot open"):
        gguf.GgufFile.open("/nonexistent/file.gguf")


def test_open_maps_a_file(tmp_path):
    data, w, _ = small_file()
    p = tmp_path / "m.gguf"
    p.write_bytes(data)
    with gguf.GgufFile.open(p) as g:
        assert g.meta_u32("llama.block_count") == 2 and len(g.tensors()) == 3
