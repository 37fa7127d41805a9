"""Builds tests/golden/kquant_kats.json: hand-constructed Q5_K and Q6_K known-answer blocks.

Derived from the FORMAT DEFINITIONS with exact rational arithmetic — no implementation under test is
imported (neither the oracle nor the CUDA library):
  Q5_K  crates/modgrad-device/src/kfd/gguf.rs:421-455   (176 bytes: d, dmin, scales[12], qh[32], ql[128];
        element 64g + 32*hi + l takes nibble hi of ql[32g + l], its fifth bit is bit 2g + hi of qh[l],
        scale / min of sub-block 2g + hi unpacked as for Q4_K, gguf.rs:406-419)
  Q6_K  crates/modgrad-device/src/kfd/gguf.rs:458-484   (210 bytes: ql[128], qh[64], 16 signed scales, d;
        element 128G + 32k + l = (nibble (k >= 2) of ql[64G + 32(k & 1) + l] | bits 2k, 2k+1 of
        qh[32G + l] << 4) - 32, scale sc[8G + 2k + l / 16])
Every expected value is exactly representable in f32, so the comparison is bit-exact.  Each record
carries `derived_from`: the reference lines its expectation follows.

Run:  python tests/golden/make_kquant_kats.py
"""
from __future__ import annotations

import json
import struct
from fractions import Fraction
from pathlib import Path

OUT = Path(__file__).resolve().parent / "kquant_kats.json"


def half_value(h: int):
    sign = -1 if (h >> 15) & 1 else 1
    exp, mant = (h >> 10) & 0x1F, h & 0x3FF
    if exp == 31:
        return None  # inf / NaN -> the dequantiser uses 0 (gguf.rs:426-427, :467)
    if exp == 0:
        return sign * Fraction(mant, 1024) * Fraction(1, 2 ** 14)
    return sign * (1 + Fraction(mant, 1024)) * (Fraction(2) ** (exp - 15))


def f32_bits(v, negative_zero: bool = False) -> int:
    if isinstance(v, tuple):
        v, negative_zero = v
    if v == 0 and negative_zero:
        return 0x80000000
    f = float(v)
    b = struct.pack("<f", f)
    assert Fraction(struct.unpack("<f", b)[0]) == v, f"{v} is not exact in f32"
    return struct.unpack("<I", b)[0]


def unpack_k4(scales12, j):
    if j < 4:
        return scales12[j] & 63, scales12[j + 4] & 63
    return (scales12[j + 4] & 0xF) | ((scales12[j - 4] >> 6) << 4), (scales12[j + 4] >> 4) | ((scales12[j] >> 6) << 4)


def q5k_expected(d_bits, dmin_bits, scales12, qh, ql):
    d, dmin = half_value(d_bits) or Fraction(0), half_value(dmin_bits) or Fraction(0)
    out = []
    for e in range(256):
        g, hi, l = e // 64, (e // 32) & 1, e % 32
        sc, m = unpack_k4(scales12, 2 * g + hi)
        nib = (ql[32 * g + l] >> 4) if hi else (ql[32 * g + l] & 0xF)
        q = nib + 16 * ((qh[l] >> (2 * g + hi)) & 1)
        d1, m1 = d * sc, dmin * m
        f32_bits(d1); f32_bits(m1); f32_bits(d1 * q)      # every rounding step must be exact
        out.append(d1 * q - m1)
    return out


def q6k_expected(d_bits, sc16, qh, ql):
    d = half_value(d_bits) or Fraction(0)
    out = []
    for e in range(256):
        G, k, l = e // 128, (e // 32) & 3, e % 32
        src = ql[64 * G + 32 * (k & 1) + l]
        nib = (src >> 4) if k >= 2 else (src & 0xF)
        q = (nib | (((qh[32 * G + l] >> (2 * k)) & 3) << 4)) - 32
        s = sc16[8 * G + 2 * k + l // 16]
        s = s - 256 if s >= 128 else s                     # signed byte
        ds = d * s
        f32_bits(ds)
        # IEEE signed zeros: a product carries the XOR of its operands' signs; a non-finite d was
        # replaced by +0.0, (float)0 is +0.0
        d_neg = half_value(d_bits) is not None and bool((d_bits >> 15) & 1)
        out.append((ds * q, d_neg ^ (s < 0) ^ (q < 0)))
    return out


MIXED_SCALES = [0x40, 0x81, 0xC2, 0x03, 0x44, 0x85, 0xC6, 0x07, 0x21, 0x43, 0x65, 0x87]   # sc 0,1,2,3,17,35,53,7


def q5k_block(d_bits, dmin_bits, scales12, qh, ql):
    return [d_bits & 0xFF, d_bits >> 8, dmin_bits & 0xFF, dmin_bits >> 8] + scales12 + qh + ql


def q6k_block(d_bits, sc16, qh, ql):
    return ql + qh + sc16 + [d_bits & 0xFF, d_bits >> 8]


def main():
    kats = []
    # ---- Q5_K ----
    unit = [1, 1, 1, 1, 0, 0, 0, 0, 1, 1, 1, 1]
    ql, qh = [0] * 128, [0] * 32
    for s in range(8):          # one non-zero weight per sub-block, alternately with / without the fifth bit
        g, hi, l = s // 2, s & 1, (7 * s + 2) % 32
        ql[32 * g + l] |= ((s + 1) << 4) if hi else (s + 1)
        if s % 2 == 0:
            qh[l] |= 1 << s
    kats.append(dict(name="q5k_one_hot_unit_scales", kind=5, block=q5k_block(0x3C00, 0, unit, qh, ql),
                     expected=q5k_expected(0x3C00, 0, unit, qh, ql), derived_from="gguf.rs:421-455 (fifth bit 2g+hi of qh[l])"))
    ql = [(i * 7 + 1) & 0xFF for i in range(128)]
    qh = [(i * 37 + 11) & 0xFF for i in range(32)]
    kats.append(dict(name="q5k_mixed_scales_affine", kind=5, block=q5k_block(0x4000, 0x3800, MIXED_SCALES, qh, ql),
                     expected=q5k_expected(0x4000, 0x3800, MIXED_SCALES, qh, ql), derived_from="gguf.rs:406-419, :421-455"))
    kats.append(dict(name="q5k_all_ones", kind=5, block=q5k_block(0x3400, 0x3000, [0xFF] * 12, [0xFF] * 32, [0xFF] * 128),
                     expected=q5k_expected(0x3400, 0x3000, [0xFF] * 12, [0xFF] * 32, [0xFF] * 128),
                     derived_from="gguf.rs:421-455 (q = 31, sc = m = 63)"))
    for name, db, mb in [("d_inf", 0x7C00, 0x3800), ("dmin_nan", 0x3C00, 0x7E01), ("d_subnormal", 0x0003, 0x0000)]:
        kats.append(dict(name="q5k_special_" + name, kind=5, block=q5k_block(db, mb, MIXED_SCALES, qh, ql),
                         expected=q5k_expected(db, mb, MIXED_SCALES, qh, ql), derived_from="gguf.rs:424-427 (non-finite -> 0)"))
    # ---- Q6_K ----
    ql, qh = [0] * 128, [0] * 64
    sc = [1] * 16
    placed = {}
    for i in range(16):         # one weight per 16-element scale group set to a known 6-bit value (others stay 0 -> -32)
        e = 16 * i + (5 * i + 3) % 16
        G, k, l = e // 128, (e // 32) & 3, e % 32
        v = (4 * i + 1) & 63
        idx = 64 * G + 32 * (k & 1) + l
        ql[idx] |= ((v & 0xF) << 4) if k >= 2 else (v & 0xF)
        qh[32 * G + l] |= (v >> 4) << (2 * k)
        placed[e] = v - 32
    exp = q6k_expected(0x3C00, sc, qh, ql)
    assert all(exp[e][0] == placed.get(e, -32) for e in range(256))
    kats.append(dict(name="q6k_placed_values_unit_scales", kind=6, block=q6k_block(0x3C00, sc, qh, ql), expected=exp,
                     derived_from="gguf.rs:470-481 (element order and the two high bits)"))
    ql = [(i * 11 + 3) & 0xFF for i in range(128)]
    qh = [(i * 29 + 7) & 0xFF for i in range(64)]
    sc = [1, 0xFF, 2, 0xFE, 64, 0xC0, 127, 0x80, 3, 0xFD, 5, 0xFB, 7, 0xF9, 9, 0xF7]   # signed: 1,-1,2,-2,64,-64,127,-128,...
    kats.append(dict(name="q6k_signed_scales", kind=6, block=q6k_block(0x3800, sc, qh, ql),
                     expected=q6k_expected(0x3800, sc, qh, ql), derived_from="gguf.rs:476 (scales are signed bytes)"))
    for name, db in [("d_inf", 0x7C00), ("d_nan", 0xFE00), ("d_subnormal", 0x0001), ("d_negative", 0xBC00)]:
        kats.append(dict(name="q6k_special_" + name, kind=6, block=q6k_block(db, sc, qh, ql),
                         expected=q6k_expected(db, sc, qh, ql), derived_from="gguf.rs:466-467 (non-finite -> 0)"))
    out = []
    for k in kats:
        x = [Fraction((i * 37) % 64 - 32, 64) for i in range(256)]
        y = sum((w[0] if isinstance(w, tuple) else w) * xi for w, xi in zip(k["expected"], x))
        out.append(dict(name=k["name"], kind=k["kind"], derived_from=k["derived_from"], block_hex=bytes(k["block"]).hex(),
                        expected_f32_bits=[f32_bits(v) for v in k["expected"]],
                        x_ramp=[float(v) for v in x], y_ramp=[y.numerator, y.denominator]))
    OUT.write_text(json.dumps(dict(about="Q5_K / Q6_K known-answer blocks from the format definition (exact rational arithmetic); "
                                         "made by tests/golden/make_kquant_kats.py", kats=out), indent=0))
    print(f"wrote {len(out)} KATs to {OUT}")


if __name__ == "__main__":
    main()
