"""Builds tests/golden/q4k_kats.json: hand-constructed Q4_K known-answer blocks.

The reference tree has no golden vector for Q4_K, and it cannot be executed where this
repository is built, so these vectors are derived from the FORMAT DEFINITION
(crates/modgrad-device/src/kfd/gguf.rs:255-265 layout, :334-342 six-bit unpack, :376-402
element order) with exact integer / rational arithmetic written out below — not by calling
any implementation under test (neither the oracle nor the CUDA library is imported here).

Every expected value is exactly representable in f32, so comparison is bit-exact.

Run:  python tests/golden/make_q4k_kats.py
"""
from __future__ import annotations

import json
import struct
from fractions import Fraction
from pathlib import Path

OUT = Path(__file__).resolve().parent / "q4k_kats.json"


def half_value(h: int):
    """Exact value of a half bit pattern as a Fraction; None for inf/NaN (exponent 31).
    The sign of a zero is carried separately (see `half_sign`)."""
    sign = -1 if (h >> 15) & 1 else 1
    exp = (h >> 10) & 0x1F
    mant = h & 0x3FF
    if exp == 31:
        return None
    if exp == 0:
        return sign * Fraction(mant, 1024) * Fraction(1, 2 ** 14)
    return sign * (1 + Fraction(mant, 1024)) * (Fraction(2) ** (exp - 15))


def half_sign(h: int) -> bool:
    return bool((h >> 15) & 1)


def f32_bits(v: Fraction, negative_zero: bool = False) -> int:
    if v == 0 and negative_zero:
        return 0x80000000
    f = float(v)
    assert Fraction(f) == v, f"{v} is not exact in binary floating point"
    b = struct.pack("<f", f)
    assert Fraction(struct.unpack("<f", b)[0]) == v, f"{v} is not exact in f32"
    return struct.unpack("<I", b)[0]


def block(d_bits: int, dmin_bits: int, scales12: list[int], qs128: list[int]) -> list[int]:
    assert len(scales12) == 12 and len(qs128) == 128
    return [d_bits & 0xFF, d_bits >> 8, dmin_bits & 0xFF, dmin_bits >> 8] + scales12 + qs128


def element_source(e: int):
    """Element e of a block -> (sub-block, byte index in qs, uses high nibble)."""
    sub = e // 32
    group = e // 64
    return sub, 32 * group + (e % 32), (sub % 2) == 1


def expected_block(d_bits, dmin_bits, sc, m, qs):
    """Exact dequantised values; requires every intermediate to be exact in f32."""
    d = half_value(d_bits)
    dmin = half_value(dmin_bits)
    # IEEE signed zeros: a product carries the XOR of its operands' signs (sc, m, q >= +0),
    # and x - y is -0 only for (-0) - (+0).  Non-finite scales become +0.0 (gguf.rs:371-372).
    d_neg = half_sign(d_bits) if d is not None else False
    dmin_neg = half_sign(dmin_bits) if dmin is not None else False
    d = Fraction(0) if d is None else d
    dmin = Fraction(0) if dmin is None else dmin
    out = []
    for e in range(256):
        sub, bi, high = element_source(e)
        q = (qs[bi] >> 4) if high else (qs[bi] & 0xF)
        d1 = d * sc[sub]
        m1 = dmin * m[sub]
        f32_bits(d1); f32_bits(m1); f32_bits(d1 * q)   # each rounding step must be exact
        v = d1 * q - m1
        neg_zero = (v == 0 and d1 * q == 0 and m1 == 0 and d_neg and not dmin_neg)
        out.append((v, neg_zero))
    return out


UNIT_SCALES = [1, 1, 1, 1, 0, 0, 0, 0, 1, 1, 1, 1]            # sc = 1, m = 0 for all 8 sub-blocks
UNIT_SC, UNIT_M = [1] * 8, [0] * 8
# scales header worked by hand in the docstring of `kat_scale_unpack`
MIXED_SCALES = [0x40, 0x81, 0xC2, 0x03, 0x44, 0x85, 0xC6, 0x07, 0x21, 0x43, 0x65, 0x87]
MIXED_SC = [0, 1, 2, 3, 17, 35, 53, 7]
MIXED_M = [4, 5, 6, 7, 18, 36, 54, 8]


def kat_one_hot():
    """d = 1.0, dmin = 0, every scale 1: one non-zero nibble per sub-block at a known place."""
    qs = [0] * 128
    where = {}
    for s in range(8):
        e = 32 * s + (5 * s + 3) % 32
        v = s + 1
        sub, bi, high = element_source(e)
        assert sub == s
        qs[bi] |= (v << 4) if high else v
        where[e] = v
    exp = [(Fraction(where.get(e, 0)), False) for e in range(256)]
    assert exp == expected_block(0x3C00, 0x0000, UNIT_SC, UNIT_M, qs)
    return dict(name="one_hot_unit_scales", block=block(0x3C00, 0, UNIT_SCALES, qs), expected=exp,
                derived_from="element order: kfd/gguf.rs:376-402; the same order in kernels/matvec_q4k.hip:13-18, :87-89 and "
                             "kfd/kernels/matvec_q4k.s:45-57")


def kat_scale_unpack():
    """Six-bit unpack, j >= 4 taking its top two bits from bytes 0..7:
    bytes 40 81 C2 03 | 44 85 C6 07 | 21 43 65 87 ->
      sc = [0,1,2,3, 1|(1<<4)=17, 3|(2<<4)=35, 5|(3<<4)=53, 7|(0<<4)=7]
      m  = [4,5,6,7, 2|(1<<4)=18, 4|(2<<4)=36, 6|(3<<4)=54, 8|(0<<4)=8]"""
    qs = [(i * 7 + 1) & 0xFF for i in range(128)]
    exp = expected_block(0x4000, 0x3800, MIXED_SC, MIXED_M, qs)  # d = 2.0, dmin = 0.5
    return dict(name="mixed_scales_affine", block=block(0x4000, 0x3800, MIXED_SCALES, qs), expected=exp,
                sc=MIXED_SC, m=MIXED_M,
                derived_from="six-bit unpack: kfd/gguf.rs:334-342 (device copy kernels/matvec_q4k.hip:41-53); affine "
                             "dequantisation: kfd/gguf.rs:386-398")


def kat_all_ones_header():
    """scales bytes all 0xFF -> every six-bit field is 63."""
    qs = [0xF0 if i % 2 else 0x0F for i in range(128)]
    exp = expected_block(0x3400, 0x3000, [63] * 8, [63] * 8, qs)  # d = 0.25, dmin = 0.125
    return dict(name="all_ones_header", block=block(0x3400, 0x3000, [0xFF] * 12, qs), expected=exp,
                sc=[63] * 8, m=[63] * 8, derived_from="kfd/gguf.rs:334-342 (every field 63), :386-398")


def kat_specials():
    """Non-finite and sub-normal super-block scales."""
    qs = [(i * 13 + 5) & 0xFF for i in range(128)]
    cases = []
    for name, d_bits, dmin_bits in [
        ("d_inf", 0x7C00, 0x3800), ("d_nan", 0x7E01, 0x3800), ("d_neg_inf", 0xFC00, 0x0000),
        ("dmin_inf", 0x3C00, 0x7C00), ("dmin_nan", 0x3C00, 0xFFFF), ("both_nonfinite", 0x7C00, 0xFC00),
        ("d_min_subnormal", 0x0001, 0x0000), ("d_neg_subnormal", 0x83FF, 0x0000),
        ("dmin_subnormal", 0x3C00, 0x0200), ("d_neg_zero", 0x8000, 0x3C00), ("d_max_half", 0x7BFF, 0x0000),
    ]:
        exp = expected_block(d_bits, dmin_bits, MIXED_SC, MIXED_M, qs)
        cases.append(dict(name="special_" + name, block=block(d_bits, dmin_bits, MIXED_SCALES, qs), expected=exp,
                          derived_from="half decode kfd/gguf.rs:281-292; non-finite scales become 0: kfd/gguf.rs:371-372"))
    return cases


def main():
    kats = [kat_one_hot(), kat_scale_unpack(), kat_all_ones_header()] + kat_specials()
    out = []
    for k in kats:
        exp = k["expected"]
        rec = dict(name=k["name"], block_hex=bytes(k["block"]).hex(),
                   expected_f32_bits=[f32_bits(v, nz) for v, nz in exp])
        rec["derived_from"] = k["derived_from"]   # the reference lines this expectation follows
        if "sc" in k:
            rec["sc"], rec["m"] = k["sc"], k["m"]
        # matvec known answers with integer activations: x[e] = (e % 7) - 3 and a one-hot
        x = [Fraction((e % 7) - 3) for e in range(256)]
        rec["x_ramp"] = [int(v) for v in x]
        y = sum(w * xv for (w, _), xv in zip(exp, x))
        rec["y_ramp"] = [y.numerator, y.denominator]
        out.append(rec)
    OUT.write_text(json.dumps(dict(
        about="hand-built Q4_K known-answer blocks; see make_q4k_kats.py", kats=out), indent=0))
    print(f"wrote {OUT} ({len(out)} vectors)")


if __name__ == "__main__":
    main()
