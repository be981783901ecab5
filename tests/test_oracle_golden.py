"""Pin the CPU oracle: the reference's own known-answer vectors and the committed
outputs of its unmodified ``quantize_and_pack`` (tests/golden/make_golden.py)."""
from pathlib import Path

import numpy as np
import pytest

from oracle import jf_oracle as O

GOLD = np.load(Path(__file__).parent / "golden" / "pack_golden.npz")


def _vals(bits16, dt):
    if dt == "bf16":
        return O.bf16_bits_to_f32(bits16)
    return bits16.view(np.float16).astype(np.float32)


# --- reference tests/test_int_pack.py:10-27 (wire bytes, scale == 1, round trip) ------
@pytest.mark.parametrize("group_size", (64, 128))
@pytest.mark.parametrize("bits,values,planes", (
    (2, (-1, 0, 1, 0), (0x6E,)),
    (3, (-3, -2, -1, 0, 1, 2, 3, 0), (0x29, 0xCB, 0xBC)),
    (4, (-7, 7), (0x1F,)),
))
def test_known_wire_bytes_round_trip(bits, values, planes, group_size):
    x = np.tile(np.array(values, np.float32), 128 // len(values)).reshape(1, 128)
    data, scales = O.quantize_and_pack(x, group_size, bits)
    assert np.array_equal(O.bf16_bits_to_f32(scales), np.ones_like(scales, np.float32))
    repeats = 128 // (8 if bits == 3 else 8 // bits)
    expected = np.array([b for b in planes for _ in range(repeats)], np.uint8)
    assert np.array_equal(data[0], expected)
    assert np.array_equal(O.unpack(data, scales, bits, group_size), x)


# --- reference tests/test_int_pack.py:30-35 (zero groups stay finite) ----------------
@pytest.mark.parametrize("bits", (2, 3, 4))
def test_zero_groups_remain_finite(bits):
    x = np.zeros((2, 128), np.float32)
    data, scales = O.quantize_and_pack(x, 64, bits)
    s = O.bf16_bits_to_f32(scales)
    assert np.isfinite(s).all() and (s > 0).all()
    assert np.array_equal(O.unpack(data, scales, bits, 64), x)


# --- byte-for-byte against the reference run in the build container ------------------
@pytest.mark.parametrize("dt", ("bf16", "fp16"))
@pytest.mark.parametrize("bits", (2, 3, 4))
@pytest.mark.parametrize("gs", (64, 128))
def test_pack_matches_reference_bytes(dt, bits, gs):
    x = _vals(GOLD[f"x_{dt}"], dt)
    data, scales = O.quantize_and_pack(x, gs, bits)
    key = f"{dt}_b{bits}_g{gs}"
    assert np.array_equal(scales, GOLD[key + "_scales"])
    assert np.array_equal(data, GOLD[key + "_data"])
    back = O.f32_to_bf16_bits(O.unpack(data, scales, bits, gs))
    assert np.array_equal(back, GOLD[key + "_unpack"])
    # decode_codes inverts pack_codes
    q, _ = O.quantize_codes(x, gs, bits)
    assert np.array_equal(O.decode_codes(data, bits) - O.offset_of(bits), q.astype(np.int32))


# --- reference tests/test_runtime_edge_cases.py:13-26 (top-k width routing) ----------
@pytest.mark.parametrize("length,expected", [(1, 32), (17, 32), (31, 32), (32, 32), (63, 32),
                                            (64, 64), (255, 128), (256, 256), (4096, 256)])
def test_select_top_k_table(length, expected):
    assert O.select_top_k(256, length, (32, 64, 128, 256)) == expected


@pytest.mark.parametrize("requested,length,supported", [(0, 128, (32, 64)), (16, 128, (32, 64)),
                                                       (32, 0, (32, 64)), (32, -1, (32, 64)),
                                                       (256, 128, ())])
def test_select_top_k_rejects(requested, length, supported):
    assert O.select_top_k(requested, length, supported) is None


# --- reference tests/test_runtime_edge_cases.py:29-35 (TP-local head map) ------------
def test_head_map_tp2_local():
    m = O.head_map(2, 32, 8, 256)
    assert m.shape == (2, 32, 256) and m.flags["C_CONTIGUOUS"]
    for h in range(32):
        assert (m[:, h] == h // 8).all()


def test_bf16_rne():
    x = np.array([1.0, 1.00390625, 1.01171875, -3.0e38, 1e-40, 0.0], np.float32)
    import torch
    want = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(O.f32_to_bf16_bits(x), want)
    r = np.random.default_rng(0).standard_normal(10000).astype(np.float32)
    want = torch.from_numpy(r).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(O.f32_to_bf16_bits(r), want)


def test_fma_f32_single_rounding():
    rng = np.random.default_rng(1)
    a = rng.integers(-30000, 30000, 20000).astype(np.float32)
    b = rng.random(20000).astype(np.float32) * 0.03
    c = rng.standard_normal(20000).astype(np.float32) * 50
    got = O._fma_f32(a, b, c)
    from fractions import Fraction
    for i in range(0, 20000, 97):
        exact = Fraction(float(a[i])) * Fraction(float(b[i])) + Fraction(float(c[i]))
        lo = np.float32(float(exact))  # python float() of a Fraction is correctly rounded to f64
        # correctly rounded fp32 of the exact rational:
        cand = [np.nextafter(lo, np.float32(-np.inf)), lo, np.nextafter(lo, np.float32(np.inf))]
        best = min(cand, key=lambda v: (abs(Fraction(float(v)) - exact), int(v.view(np.uint32)) & 1))
        assert got[i] == best


def test_topk_tie_rule_and_padding():
    s = np.array([1.0, 3.0, 3.0, -1.0, 3.0, 0.5], np.float32)
    assert O.topk_select(s, 2).tolist() == [1, 2]
    assert O.topk_select(s, 4).tolist() == [1, 2, 4, 0]
    assert O.topk_select(s, 8).tolist() == [1, 2, 4, 0, 5, 3, -1, -1]
    assert O.topk_select(np.zeros(0, np.float32), 4).tolist() == [-1] * 4
