"""Pins the CPU oracle against the reference's own known-answer tests.

Each test restates one test of the reference (file:line in the docstring) with
the same inputs and the same expected values / tolerances, evaluated by the
oracle instead of the Rust code.  Nothing here touches a GPU.
"""
import math

import numpy as np
import pytest

from allpaka_b200 import synth

Q8_0, Q4_K, Q5_K, Q6_K, Q5_0, Q3_K, Q2_K = 8, 12, 13, 14, 6, 11, 10


def half_bits(orc, x):
    return orc.f32_to_f16(x)


def put_f16(orc, buf, at, x):
    h = orc.f32_to_f16(x)
    buf[at] = h & 0xFF
    buf[at + 1] = h >> 8


# ---- crates/allpaka-gguf/src/dequant.rs tests ---------------------------------

def test_f16_round_trips_and_specials(orc):
    """dequant.rs:302-315"""
    for x in [1.0, -1.0, 0.5, 2.0, 65504.0, 0.099975586]:
        back = orc.f16_to_f32(orc.f32_to_f16(x))
        assert abs(back - x) <= abs(x) * 1e-3
    assert orc.f16_to_f32(0x0000) == 0.0
    assert math.copysign(1.0, orc.f16_to_f32(0x8000)) == -1.0
    assert math.isinf(orc.f16_to_f32(0x7C00))
    assert math.isnan(orc.f16_to_f32(0x7C01))
    assert abs(orc.f16_to_f32(0x0001) - 2.0 ** -24) < 1e-12


def test_f16_matches_numpy_for_every_bit_pattern(orc):
    """dtype lib.rs:129-147 vs IEEE half (numpy) on all 65536 patterns."""
    bits = np.arange(65536, dtype=np.uint16)
    want = bits.view(np.float16).astype(np.float32)
    got = np.array([orc.f16_to_f32(int(b)) for b in bits], dtype=np.float32)
    nan = np.isnan(want)
    assert np.array_equal(np.isnan(got), nan)
    assert np.array_equal(got[~nan].view(np.uint32), want[~nan].view(np.uint32))


def test_f32_to_f16_is_round_to_nearest_even(orc):
    """dtype lib.rs:151-184 vs numpy's RNE conversion."""
    rng = np.random.default_rng(7)
    xs = np.concatenate([
        rng.standard_normal(4000).astype(np.float32) * 10.0 ** rng.integers(-9, 6, 4000),
        np.array([0.0, -0.0, 65504.0, 65520.0, 1e-8, 6e-8, 6.1e-5, np.inf, -np.inf], np.float32),
    ]).astype(np.float32)
    with np.errstate(over="ignore"):
        want = xs.astype(np.float16).view(np.uint16)
    got = np.array([orc.f32_to_f16(float(x)) for x in xs], dtype=np.uint16)
    assert np.array_equal(got, want)


def test_bf16_conversions(orc):
    """dtype lib.rs:188-201 and the SIMD==scalar test at lib.rs:428-458."""
    vals = [(i - 38.0) * 0.125 for i in range(77)]
    for v in vals:
        b = orc.f32_to_bf16(v)
        assert b == int(synth.to_bf16_bits(np.array([v], np.float32))[0])
        assert orc.bf16_to_f32(b) == float(synth.bf16_bits_to_f32(np.array([b], np.uint16))[0])


def test_q8_0_is_scale_times_value(orc):
    """dequant.rs:317-331"""
    block = np.zeros(34, dtype=np.uint8)
    put_f16(orc, block, 0, 0.5)
    block[2] = np.int8(10).view(np.uint8)
    block[3] = np.int8(-20).view(np.uint8)
    block[33] = 127
    out = orc.dequant(Q8_0, block, 32)
    assert out.size == 32
    assert out[0] == 5.0 and out[1] == -10.0 and out[31] == 63.5 and out[2] == 0.0


def test_k4_scale_packing_reassembles_split_fields(orc):
    """dequant.rs:429-444"""
    packed = np.zeros(12, dtype=np.uint8)
    packed[0] = 33
    packed[4] = 21
    packed[9] = (0b1001 << 4) | 0b0110
    packed[1] |= 0b10 << 6
    packed[5] |= 0b01 << 6
    assert orc.scale_min_k4(0, packed) == (33.0, 21.0)
    assert orc.scale_min_k4(5, packed) == (38.0, 25.0)


def test_pack_scales_k4_is_the_inverse_of_scale_min_k4(orc):
    rng = np.random.default_rng(3)
    sc = rng.integers(0, 64, size=(50, 8), dtype=np.uint8)
    mn = rng.integers(0, 64, size=(50, 8), dtype=np.uint8)
    p = synth.pack_scales_k4(sc, mn)
    for r in range(50):
        for j in range(8):
            assert orc.scale_min_k4(j, p[r]) == (float(sc[r, j]), float(mn[r, j]))


def test_q4_k_low_and_high_nibbles_go_to_adjacent_sub_blocks(orc):
    """dequant.rs:448-468"""
    block = np.zeros(144, dtype=np.uint8)
    put_f16(orc, block, 0, 1.0)
    put_f16(orc, block, 2, 1.0)
    block[4], block[5], block[8], block[9] = 2, 3, 1, 2
    block[16] = 0x75
    out = orc.dequant(Q4_K, block, 256)
    assert out[0] == 9.0 and out[1] == -1.0
    assert out[32] == 19.0 and out[33] == -2.0
    assert np.all(out[64:] == 0.0)


def test_a_wrong_byte_count_is_an_error(orc):
    """dequant.rs:549-554 and dtype lib.rs:475-492"""
    with pytest.raises(ValueError):
        orc.dequant(Q8_0, np.zeros(33, np.uint8), 32)
    with pytest.raises(ValueError):
        orc.dequant(99, np.zeros(4, np.uint8), 1)
    assert orc.expected_bytes(Q4_K, 512) == 288
    assert orc.expected_bytes(99, 64) == 0
    assert orc.expected_bytes(Q4_K, 300) == 0


# ---- crates/allpaka-backend/src/quantmat/mod.rs tests --------------------------

def q8_0_block(orc, values):
    """mod.rs:745-761: quantise 32 floats to a Q8_0 block in the test itself."""
    values = np.asarray(values, dtype=np.float32)
    amax = np.float32(np.max(np.abs(values)))
    d = np.float32(amax / np.float32(127.0))
    idv = np.float32(1.0) / d if d > 0 else np.float32(0.0)
    out = np.zeros(34, dtype=np.uint8)
    bits = orc.f32_to_f16(float(d))
    out[0], out[1] = bits & 0xFF, bits >> 8
    d_back = np.float32(orc.f16_to_f32(bits))
    exact = np.zeros(32, dtype=np.float32)
    for i, v in enumerate(values):
        t = np.float32(v * idv)
        q = int(np.clip(math.copysign(math.floor(abs(float(t)) + 0.5), float(t)), -127, 127))
        out[2 + i] = np.int8(q).view(np.uint8)
        exact[i] = d_back * np.float32(q)
    return out, exact


def seq_dot(a, b):
    s = np.float32(0.0)
    for x, y in zip(a, b):
        s = np.float32(s + np.float32(np.float32(x) * np.float32(y)))
    return s


def test_a_quantised_matmul_matches_the_hand_computed_product(orc):
    """mod.rs:774-798 (m = 2: the f32 row_dot path)"""
    w0 = [float(i) - 16.0 for i in range(32)]
    w1 = [1.0] * 32
    b0, e0 = q8_0_block(orc, w0)
    b1, e1 = q8_0_block(orc, w1)
    data = np.concatenate([b0, b1])
    x = np.array([(i % 7) * 0.25 for i in range(64)], dtype=np.float32)
    y = orc.matmul(Q8_0, data, 2, 32, x, m=2)
    for i in range(2):
        xi = x[i * 32:(i + 1) * 32]
        assert abs(y[i, 0] - seq_dot(e0, xi)) < 1e-4
        assert abs(y[i, 1] - seq_dot(e1, xi)) < 1e-4


def q8_act_error_bound(w, x):
    """mod.rs:864-872"""
    bound = 0.0
    for wb, xb in zip(np.split(w, len(w) // 32), np.split(x, len(x) // 32)):
        bound += float(np.max(np.abs(xb))) / 127.0 / 2.0 * float(np.sum(np.abs(wb)))
    return bound


def test_q5_k_high_bit_adds_sixteen_for_the_owning_sub_block(orc):
    """dequant.rs:470-495"""
    block = np.zeros(176, dtype=np.uint8)
    put_f16(orc, block, 0, 1.0)
    put_f16(orc, block, 2, 0.0)
    block[4:8] = 1          # scales of sub-blocks 0..3
    block[12:16] = 0x01     # low nibble: scale of sub-blocks 4..7
    block[16] = 0b0000_1001  # qh[0]: bit 0 -> sub-block 0, bit 3 -> sub-block 3
    out = orc.dequant(Q5_K, block, 256)
    assert out[0] == 16.0 and out[1] == 0.0
    assert out[32] == 0.0                      # bit 1 not set: sub-block 1 unaffected
    assert out[96] == 16.0 and out[97] == 0.0  # sub-block 3 = pair 1 high nibbles
    assert orc.expected_bytes(Q5_K, 512) == 352 and orc.expected_bytes(Q5_K, 100) == 0


def test_q5_k_block_dots_recombine_to_the_row_dot(orc):
    """The int32 block dots are what dot_q5_k_i8 scales, the min term rides on the exact block sums
    (q8_acts.rs:253-258)."""
    x = synth.normal_f32(512, 25)
    d, sm, q = orc.q8acts(x)
    w = synth.q5_k_matrix(3, 512, 26)
    dots = orc.block_dots(Q5_K, w, 3, 512, q)
    wv = w.reshape(3, 2, 176)
    for j in range(3):
        total = np.float32(0.0)
        for sb in range(2):
            dd = np.float32(wv[j, sb, 0:2].view(np.float16)[0])
            dmin = np.float32(wv[j, sb, 2:4].view(np.float16)[0])
            for k in range(8):
                sc, mn = orc.scale_min_k4(k, wv[j, sb, 4:16])
                b = sb * 8 + k
                dot = np.float32(np.float32(dots[0, j, b]) * d[b])
                a = np.float32(np.float32(dd * np.float32(sc)) * dot)
                m = np.float32(np.float32(dmin * np.float32(mn)) * sm[b])
                total = np.float32(total + np.float32(a - m))
        assert total == np.float32(orc.dot_row(Q5_K, wv[j].reshape(-1), x, q8=True))


def test_q6_k_reassembles_six_bit_values_from_the_right_bits(orc):
    """dequant.rs:374-409: one chosen element per quarter, everything else zero."""
    block = np.zeros(210, dtype=np.uint8)
    put_f16(orc, block, 208, 1.0)
    block[192:208] = 1
    block[0] = 0x05
    block[128] = 0b0000_0001           # quarter 0, l=0: 5 | 1<<4 = 21 -> -11
    block[35] = 0x02
    block[131] = 0b0000_1000           # quarter 1, l=3: 2 | 2<<4 = 34 -> 2
    block[7] |= 0x90
    block[135] |= 0b0001_0000          # quarter 2, l=7: 9 | 16 = 25 -> -7
    block[41] |= 0xF0
    block[137] |= 0b1100_0000          # quarter 3, l=9: 15 | 48 = 63 -> 31
    out = orc.dequant(Q6_K, block, 256)
    assert out[0] == -11.0 and out[32 + 3] == 2.0 and out[64 + 7] == -7.0 and out[96 + 9] == 31.0
    assert out[1] == -32.0
    assert np.all(out[128:] == -32.0)


def test_q6_k_negative_scales_flip_the_sign(orc):
    """dequant.rs:412-425"""
    block = np.zeros(210, dtype=np.uint8)
    put_f16(orc, block, 208, 0.5)
    block[192] = np.uint8(np.int8(-2).view(np.uint8))
    out = orc.dequant(Q6_K, block, 256)
    assert out[0] == 32.0 and out[16] == 0.0


def test_q6_k_block_dots_recombine_to_the_row_dot(orc):
    """The per-block integers sc0*dot0 + sc1*dot1 are exactly what dot_q6_k_i8 scales
    (q8_acts.rs:336-343)."""
    x = synth.normal_f32(512, 15)
    d, s, q = orc.q8acts(x)
    w = synth.q6_k_matrix(3, 512, 16)
    dots = orc.block_dots(Q6_K, w, 3, 512, q)
    wv = w.reshape(3, 2, 210)
    for j in range(3):
        total = np.float32(0.0)
        for b in range(16):
            dw = np.float32(wv[j, b // 8, 208:210].view(np.float16)[0])
            total = np.float32(total + np.float32(np.float32(dw * d[b]) * np.float32(dots[0, j, b])))
        assert total == np.float32(orc.dot_row(Q6_K, wv[j].reshape(-1), x, q8=True))
    assert orc.expected_bytes(Q6_K, 512) == 420 and orc.expected_bytes(Q6_K, 300) == 0


def test_q5_0_is_scale_times_five_bit_value_minus_16(orc):
    """dequant.rs:128-141: element j = low nibble of qs[j] with bit j of qh on top, element j + 16 = high
    nibble with bit j + 16; x = d * (q - 16)."""
    block = np.zeros(22, dtype=np.uint8)
    put_f16(orc, block, 0, 0.5)
    block[6] = 0xA3                      # element 0: 3, element 16: 10
    block[6 + 15] = 0x0F                 # element 15: 15, element 31: 0
    block[2] = 0b0000_0001               # bit 0: element 0 -> 3 | 16 = 19
    block[5] = 0b1000_0000               # bit 31: element 31 -> 0 | 16 = 16
    out = orc.dequant(Q5_0, block, 32)
    assert out[0] == 0.5 * 3 and out[16] == 0.5 * (10 - 16) and out[15] == 0.5 * (15 - 16) and out[31] == 0.0
    assert out[1] == -8.0
    assert orc.expected_bytes(Q5_0, 64) == 44 and orc.expected_bytes(Q5_0, 48) == 0


def test_q5_0_block_dots_recombine_to_the_row_dot(orc):
    """total += d * d_x[b] * dot (q8_acts.rs:122)."""
    x = synth.normal_f32(128, 25)
    d, s, q = orc.q8acts(x)
    w = synth.q5_0_matrix(3, 128, 26)
    dots = orc.block_dots(Q5_0, w, 3, 128, q)
    wv = w.reshape(3, 4, 22)
    vals = orc.dequant(Q5_0, w, 3 * 128).reshape(3, 4, 32)
    for j in range(3):
        total = np.float32(0.0)
        for b in range(4):
            dw = np.float32(wv[j, b, 0:2].view(np.float16)[0])
            if dw > 0:
                codes = np.rint(vals[j, b] / dw).astype(np.int64)
                assert dots[0, j, b] == int(np.sum(codes * q[b * 32:(b + 1) * 32].astype(np.int64)))
            total = np.float32(total + np.float32(np.float32(dw * d[b]) * np.float32(dots[0, j, b])))
        assert total == np.float32(orc.dot_row(Q5_0, wv[j].reshape(-1), x, q8=True))


def test_q2_k_values_scales_mins_and_order(orc):
    """dequant.rs:143-174: x = d * (sc & 15) * q - dmin * (sc >> 4); block blk = 4 * half + shift index,
    sub-block byte 2 * blk + group."""
    block = np.zeros(84, dtype=np.uint8)
    put_f16(orc, block, 80, 0.5)
    put_f16(orc, block, 82, 0.25)
    block[0] = 0x35                      # sub-block 0: scale 5, min 3
    block[3] = 0x12                      # sub-block 3 (block 1, group 1): scale 2, min 1
    block[8] = 0xF0                      # sub-block 8 (block 4 = half 1, shift 0): scale 0, min 15
    block[16] = 0b11_10_01_10            # l = 0 of half 0: blocks 0..3 take 2, 1, 2, 3
    block[16 + 16] = 0b00_00_11_00       # l = 16 of half 0: block 1 takes 3
    out = orc.dequant(Q2_K, block, 256)
    assert out[0] == 0.5 * 5 * 2 - 0.25 * 3 and out[1] == -0.25 * 3
    assert out[32] == 0.0                # block 1, group 0: scale and min 0
    assert out[32 + 16] == 0.5 * 2 * 3 - 0.25 * 1 and out[32 + 17] == -0.25
    assert out[128] == -0.25 * 15
    assert orc.expected_bytes(Q2_K, 512) == 168 and orc.expected_bytes(Q2_K, 300) == 0


def test_q2_k_block_dots_and_mins_recombine_to_the_row_dot(orc):
    """total += dl * dotq - ml * sum_x per sub-block, dotq and sum_x over the activation codes
    (q8_acts.rs:156-170)."""
    x = synth.normal_f32(512, 45)
    d, s, q = orc.q8acts(x)
    w = synth.q2_k_matrix(2, 512, 46)
    dots = orc.block_dots(Q2_K, w, 2, 512, q)
    wv = w.reshape(2, 2, 84)
    for j in range(2):
        total = np.float32(0.0)
        for b in range(16):
            blk = wv[j, b // 8]
            dw = np.float32(blk[80:82].view(np.float16)[0])
            dm = np.float32(blk[82:84].view(np.float16)[0])
            vals = (blk[16 + ((b % 8) // 4) * 32: 16 + ((b % 8) // 4) * 32 + 32] >> (2 * (b % 4))) & 3
            xq = q[b * 32:(b + 1) * 32].astype(np.int64)
            want_int = 0
            for g in range(2):
                sc = int(blk[2 * (b % 8) + g])
                dot = int(np.sum(vals[g * 16:(g + 1) * 16].astype(np.int64) * xq[g * 16:(g + 1) * 16]))
                want_int += (sc & 15) * dot
                dl = np.float32(dw * np.float32(sc & 15))
                ml = np.float32(dm * np.float32(sc >> 4))
                dotq = np.float32(np.float32(dot) * d[b])
                sum_x = np.float32(np.float32(int(np.sum(xq[g * 16:(g + 1) * 16]))) * d[b])
                total = np.float32(total + np.float32(np.float32(dl * dotq) - np.float32(ml * sum_x)))
            assert dots[0, j, b] == want_int
        assert total == np.float32(orc.dot_row(Q2_K, wv[j].reshape(-1), x, q8=True))


def test_q3_k_values_scales_and_order(orc):
    """dequant.rs:176-204: x = d * (scale - 32) * q, q = two bits of qs minus 4 where the hmask bit of
    the block is clear; block blk = 4 * half + shift index, sub-block scale index 2 * blk + group."""
    block = np.zeros(110, dtype=np.uint8)
    put_f16(orc, block, 108, 0.25)
    block[96:108] = 0
    block[96] = 0x0B | (0x03 << 4)       # raw[0] low nibble 11, raw[8] low nibble 3
    block[104] = 0b0001_0010             # raw[0] += 2 << 4 = 43, raw[4] += 0, raw[8] += 1 << 4 = 19
    block[32] = 0b10_01_11_10            # l = 0 of half 0: blocks 0..3 take 2, 3, 1, 2
    block[0] = 0b0000_0101               # hmask[0]: blocks 0 and 2 keep their value, the others lose 4
    out = orc.dequant(Q3_K, block, 256)
    assert out[0] == 0.25 * (43 - 32) * 2             # block 0, group 0: scale raw[0]
    assert out[32] == 0.25 * (0 - 32) * (3 - 4)       # block 1: raw[2] = 0
    assert out[64] == 0.25 * (0 - 32) * 1             # block 2: raw[4] = 0
    assert out[96] == 0.25 * (0 - 32) * (2 - 4)
    assert out[1] == 0.25 * (43 - 32) * -4 and out[16] == 0.25 * (0 - 32) * -4
    assert out[128] == 0.25 * (19 - 32) * -4          # block 4, group 0: raw[8]
    assert orc.expected_bytes(Q3_K, 512) == 220 and orc.expected_bytes(Q3_K, 300) == 0


def test_q3_k_block_dots_recombine_to_the_row_dot(orc):
    """total += d * dx * (sc0 * dot0 + sc1 * dot1) (q8_acts.rs:206-210)."""
    x = synth.normal_f32(512, 35)
    d, s, q = orc.q8acts(x)
    w = synth.q3_k_matrix(3, 512, 36)
    dots = orc.block_dots(Q3_K, w, 3, 512, q)
    wv = w.reshape(3, 2, 110)
    for j in range(3):
        total = np.float32(0.0)
        for b in range(16):
            dw = np.float32(wv[j, b // 8, 108:110].view(np.float16)[0])
            total = np.float32(total + np.float32(np.float32(dw * d[b]) * np.float32(dots[0, j, b])))
        assert total == np.float32(orc.dot_row(Q3_K, wv[j].reshape(-1), x, q8=True))


def test_fused_q4_k_dot_matches_dequant_then_dot(orc):
    """mod.rs:812-838"""
    block = np.zeros(144, dtype=np.uint8)
    put_f16(orc, block, 0, 0.25)
    put_f16(orc, block, 2, 0.5)
    for j in range(12):
        block[4 + j] = (7 + j * 13) & 0x3F
    for i in range(128):
        block[16 + i] = (i * 37 + 11) & 0xFF
    x = np.array([((i % 13) - 6.0) * 0.3 for i in range(256)], dtype=np.float32)
    fused = orc.matmul(Q4_K, block, 1, 256, x, m=1)[0, 0]
    row = orc.dequant(Q4_K, block, 256)
    reference = float(seq_dot(row, x))
    assert abs(fused - reference) < q8_act_error_bound(row, x) + 1e-3 * (1.0 + abs(reference))


def test_integer_q8_0_matvec_matches_reference_within_bound(orc):
    """mod.rs:900-921"""
    w0 = [(i - 16.0) * 0.11 for i in range(32)]
    w1 = [((i * 7 % 13) - 6.0) * 0.3 for i in range(32)]
    b0, e0 = q8_0_block(orc, w0)
    b1, e1 = q8_0_block(orc, w1)
    x = np.array([((i % 9) - 4.0) * 0.17 for i in range(32)], dtype=np.float32)
    y = orc.matmul(Q8_0, np.concatenate([b0, b1]), 2, 32, x, m=1)[0]
    for yi, exact in zip(y, (e0, e1)):
        want = float(seq_dot(exact, x))
        assert abs(yi - want) < q8_act_error_bound(exact, x) + 1e-4


def test_size_mismatches_are_errors(orc):
    """mod.rs:923-937"""
    b = np.zeros(34, dtype=np.uint8)
    with pytest.raises(ValueError):
        orc.matmul(Q8_0, b, 2, 32, np.zeros(32, np.float32))
    with pytest.raises(ValueError):
        orc.matmul(Q8_0, b, 1, 33, np.zeros(33, np.float32))
    with pytest.raises(ValueError):
        orc.matmul(Q8_0, b, 1, 32, np.zeros(16, np.float32))


# ---- crates/allpaka-backend/src/quantmat/kernel_tests.rs ------------------------

N_IN = 512


def kt_row(ty):
    be, bb = synth.BLOCK[ty]
    row = synth.lcg_bytes(N_IN // be * bb, 0x5EED ^ bb)
    return synth.tame_scales(row, ty)


def kt_acts():
    return np.array([((i * 7 % 23) - 11.0) * 0.03 for i in range(N_IN)], dtype=np.float32)


@pytest.mark.parametrize("ty", [Q8_0, Q5_0, Q2_K, Q3_K, Q4_K, Q5_K, Q6_K])
def test_float_dot_kernels_match_the_dequantizer(orc, ty):
    """kernel_tests.rs:58-88"""
    x = kt_acts()
    r = kt_row(ty)
    w = orc.dequant(ty, r, N_IN)
    got = orc.dot_row(ty, r, x, q8=False)
    want = float(seq_dot(w, x))
    mag = float(np.sum(np.abs(w * x)))
    assert abs(got - want) <= 1e-4 * mag + 1e-5


@pytest.mark.parametrize("ty", [Q8_0, Q5_0, Q2_K, Q3_K, Q4_K, Q5_K, Q6_K])
def test_q8_activation_kernels_match_the_dequantizer(orc, ty):
    """kernel_tests.rs:90-121"""
    x = kt_acts()
    d, s, q = orc.q8acts(x)
    seen = np.repeat(d, 32) * q.astype(np.float32)
    r = kt_row(ty)
    w = orc.dequant(ty, r, N_IN)
    got = orc.dot_row(ty, r, x, q8=True)
    want_q8 = float(seq_dot(w, seen))
    want_f32 = float(seq_dot(w, x))
    mag = float(np.sum(np.abs(w * x)))
    tol = 2e-3 * mag + 1e-4
    assert abs(got - want_q8) <= tol or abs(got - want_f32) <= tol


def test_integer_dot_is_exact(orc):
    """kernel_tests.rs:123-129"""
    a = np.array([(i * 37 % 255) & 0xFF for i in range(64)], dtype=np.uint8).view(np.int8)
    b = np.array([(i * 11 % 255) & 0xFF for i in range(64)], dtype=np.uint8).view(np.int8)
    want = int(np.sum(a.astype(np.int64) * b.astype(np.int64)))
    assert orc.dot_i8(a, b) == want


def test_q8acts_rounds_half_away_from_zero_and_keeps_exact_sums(orc):
    """q8_acts.rs:26-63: d = amax/127, q = round(v/d) half away, sum sequential f32."""
    x = np.zeros(64, dtype=np.float32)
    x[0], x[1], x[2], x[3] = 127.0, 0.5, -0.5, 1.5
    x[32:] = 0.0
    d, s, q = orc.q8acts(x)
    assert d[0] == 1.0 and list(q[:4]) == [127, 1, -1, 2]
    assert d[1] == 0.0 and np.all(q[32:] == 0)
    assert s[0] == np.float32(127.0 + 0.5 - 0.5 + 1.5)
    rng = np.random.default_rng(11)
    x = rng.standard_normal(320).astype(np.float32)
    d, s, q = orc.q8acts(x)
    for b in range(10):
        xs = x[b * 32:(b + 1) * 32]
        db = np.float32(np.max(np.abs(xs)) / np.float32(127.0))
        assert d[b] == db
        idv = np.float32(1.0) / db
        want = [int(math.copysign(math.floor(abs(float(np.float32(v * idv))) + 0.5), float(v))) for v in xs]
        assert list(q[b * 32:(b + 1) * 32]) == want
        acc = np.float32(0.0)
        for v in xs:
            acc = np.float32(acc + v)
        assert s[b] == acc


def test_block_dots_recombine_to_the_row_dot(orc):
    """The int32 block dots are exactly what dot_q8_0_i8 / dot_q4_k_i8 scale
    (q8_acts.rs:86-96, 267-301)."""
    x = synth.normal_f32(512, 5)
    d, s, q = orc.q8acts(x)
    w = synth.q8_0_matrix(4, 512, 6)
    dots = orc.block_dots(Q8_0, w, 4, 512, q)
    wv = w.reshape(4, 16, 34)
    for j in range(4):
        total = np.float32(0.0)
        for b in range(16):
            dw = np.float32(wv[j, b, 0:2].view(np.float16)[0])
            total = np.float32(total + np.float32(np.float32(dw * d[b]) * np.float32(dots[0, j, b])))
        assert total == np.float32(orc.dot_row(Q8_0, wv[j].reshape(-1), x, q8=True))


# ---- crates/allpaka-backend/src/ops/mod.rs tests -------------------------------

def close(a, b):
    return abs(a - b) < 1e-5


def test_rmsnorm_invariants(orc):
    """ops/mod.rs:119-148"""
    x = orc.rmsnorm([3.0, -4.0, 12.0, 0.0], [1.0] * 4, 0.0)
    rms = math.sqrt(float(np.sum(x * x)) / 4.0)
    assert close(rms, 1.0)
    assert x[0] > 0 and x[1] < 0 and x[3] == 0.0
    y = orc.rmsnorm([1.0, 1.0], [2.0, 3.0], 0.0)
    assert close(y[0], 2.0) and close(y[1], 3.0)
    z = orc.rmsnorm(np.zeros(8), np.ones(8), 1e-5)
    assert np.all(np.isfinite(z))


def test_rmsnorm_is_f64_accumulated_and_into_matches_in_place(orc):
    """ops/norm.rs:115-118, 193-198: f64 mean, f64 scale, cast, then * w."""
    x = synth.normal_f32(5120, 21)
    g = synth.gamma(5120, 22)
    got = orc.rmsnorm_into(x, g, 1e-6)
    assert np.array_equal(got, orc.rmsnorm(x, g, 1e-6))
    ss = orc.sum_sq_f64(x)
    exact = math.fsum(float(v) * float(v) for v in x)
    assert abs(ss - exact) <= 1e-12 * exact
    scale = 1.0 / math.sqrt(ss / 5120 + float(np.float32(1e-6)))
    want = (x.astype(np.float64) * scale).astype(np.float32) * g
    assert np.array_equal(got, want)


def test_silu_and_swiglu(orc):
    """ops/mod.rs:167-190"""
    assert orc.silu(0.0) == 0.0
    assert close(orc.silu(1.0), 1.0 / (1.0 + math.exp(-1.0)))
    assert abs(orc.silu(-20.0)) < 1e-7
    assert close(orc.silu(20.0), 20.0)
    gate = np.array([i * 0.7 for i in range(-25, 26)], dtype=np.float32)
    up = np.array([i * 0.5 - 3.0 for i in range(len(gate))], dtype=np.float32)
    got = orc.swiglu(gate, up)
    for gv, g, u in zip(got, gate, up):
        assert close(gv, orc.silu(float(g)) * float(u))


def test_rope_identity_norm_and_pairing(orc):
    """ops/mod.rs:193-225, 255-263"""
    orig = np.array([i - 3.5 for i in range(8)], dtype=np.float32)
    assert np.array_equal(orc.rope_neox(orig, 0, 10000.0), orig)
    x = orc.rope_neox(orig, 17, 10000.0)
    assert close(float(np.sum(orig * orig)), float(np.sum(x * x)))
    assert not np.array_equal(x, orig)
    e = np.zeros(8, dtype=np.float32)
    e[0] = 1.0
    r = orc.rope_neox(e, 1, 10000.0)
    assert close(r[4], math.sin(1.0)) and r[1] == 0.0
    ones = orc.rope_neox(np.ones(8, np.float32), 1, 10000.0)
    assert abs(ones[0] - 1.0) > 0.3 and abs(ones[3] - 1.0) < 0.01


def test_cached_rope_is_bit_identical_to_the_naive_form(orc):
    """ops/mod.rs:229-251"""
    inv = orc.rope_inv_freq(8, 10000.0)
    for pos in (0, 1, 17, 5000):
        table = orc.rope_sin_cos(pos, inv)
        orig = np.array([i - 3.5 for i in range(8)], dtype=np.float32)
        assert np.array_equal(orc.rope_neox(orig, pos, 10000.0), orc.rope_neox_table(orig, table))


def test_partial_rotary_leaves_the_tail(orc):
    """ops/rope.rs:66-81: a table shorter than half the head rotates only the lead."""
    inv = orc.rope_inv_freq(4, 10000.0)
    table = orc.rope_sin_cos(3, inv)
    x = np.arange(8, dtype=np.float32) + 1.0
    y = orc.rope_neox_table(x, table)
    assert np.array_equal(y[4:], x[4:])
    assert not np.array_equal(y[:4], x[:4])


def test_rope_dot_products_depend_only_on_relative_position(orc):
    """ops/mod.rs:269-290"""
    q = np.array([((i * 7 + 3) % 5) - 2.0 for i in range(8)], dtype=np.float32)
    k = np.array([((i * 3 + 1) % 7) - 3.0 for i in range(8)], dtype=np.float32)

    def dot_at(pq, pk):
        return float(np.sum(orc.rope_neox(q, pq, 10000.0) * orc.rope_neox(k, pk, 10000.0)))

    assert close(dot_at(5, 3), dot_at(102, 100))
    assert close(dot_at(9, 0), dot_at(59, 50))
    assert not close(dot_at(5, 3), dot_at(5, 0))


# ---- crates/allpaka-backend/tests/gpu_cuda_parity.rs fixture --------------------

def cuda_parity_fixture():
    """gpu_cuda_parity.rs:75-105: 8x64 Q8_0 from the LCG region, scales tamed."""
    region = synth.lcg_bytes(8 * 2 * 34, 0xC0FFEE00D15CAFE1)
    w = synth.tame_scales(region.copy(), Q8_0)
    x = np.array([((i % 13) - 6.0) * 0.1 for i in range(64)], dtype=np.float32)
    return w, x


def test_cuda_parity_fixture_on_the_oracle(orc):
    """gpu_cuda_parity.rs:108-127 with the oracle in the GPU's place.  The
    reference's CUDA Q8_0 kernel multiplies f32 activations, so its tolerance
    applies to the f32-activation path; the Q8-activation path (what the CPU
    runs at m = 1) is held to the activation-quantisation bound instead."""
    w, x = cuda_parity_fixture()
    got_f32 = orc.matmul(Q8_0, w, 8, 64, x, m=1, act_mode=orc.ACT_F32)[0]
    got_q8 = orc.matmul(Q8_0, w, 8, 64, x, m=1)[0]
    for j in range(8):
        row = orc.dequant(Q8_0, w[j * 68:(j + 1) * 68], 64)
        want = float(seq_dot(row, x))
        assert abs(got_f32[j] - want) < 1e-3 + 1e-3 * abs(want)
        assert abs(got_q8[j] - want) < q8_act_error_bound(row, x) + 1e-4


def test_attend_group_matches_the_naive_reference(orc):
    """crates/allpaka-model/src/model/attention.rs:569-629: 8 q heads, 2 kv heads, head_dim 16, 33
    positions from the test's own LCG; the one-pass online softmax against the buffered one."""
    n_heads, n_kv, hd, positions = 8, 2, 16, 33
    kv_dim, q_dim, group = n_kv * hd, n_heads * hd, n_heads // n_kv
    state = 0x123456789ABCDEF0

    def rnd():
        nonlocal state
        state = (state * 6364136223846793005 + 1) & 0xFFFFFFFFFFFFFFFF
        return np.float32(np.float32(state >> 40) / np.float32(1 << 24) * np.float32(2.0) - np.float32(1.0))

    kc = np.zeros((positions, kv_dim), np.uint16)
    vc = np.zeros((positions, kv_dim), np.uint16)
    for t in range(positions):
        k = np.array([rnd() for _ in range(kv_dim)], np.float32)
        v = np.array([rnd() for _ in range(kv_dim)], np.float32)
        kc[t], vc[t] = orc.kv_store(k), orc.kv_store(v)
    q = np.array([rnd() for _ in range(q_dim)], np.float32)
    scale = np.float32(1.0) / np.sqrt(np.float32(hd))
    pos = positions - 1
    got = orc.attend_one(q, kc, vc, kv_dim, n_kv, hd, group, 0, pos, scale)
    want = np.concatenate([orc.attend_head(q[i * hd:(i + 1) * hd], kc, vc, kv_dim, i // group, hd, pos, scale)
                           for i in range(n_heads)])
    assert np.all(np.abs(got - want) < 1e-5 * (1.0 + np.abs(want)))
    # the cache keeps IEEE halves: the store is the dtype conversion the other known answers pin
    assert orc.kv_store(np.array([1.0, -2.5, 65504.0, 1e-8, 70000.0], np.float32)).tolist() == \
        [0x3C00, 0xC100, 0x7BFF, 0x0000, 0x7C00]
