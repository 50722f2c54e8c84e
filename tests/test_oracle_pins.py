"""Pins the CPU oracle against every known answer the reference's own tests hold for the MoE
path that needs no checkpoint, and against the CUDA toolkit's host conversions."""
import math

import numpy as np
import pytest


def all_bf16_floats():
    bits = np.arange(65536, dtype=np.uint32) << 16
    v = bits.view(np.float32)
    return v[np.isfinite(v)]


def test_e2m1_table(orc):
    # amd-gfx906/prefill/tests/p92_pf_moe_test.hip:15-20
    mags = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    for code in range(16):
        want = mags[code & 7] * (-1.0 if code & 8 else 1.0)
        assert orc.cpu().orc_decode_e2m1(code) == want
        assert orc.pin().pin_decode_e2m1(code) == want


def test_ue4m3_decode(orc):
    # amd-gfx906/prefill/tests/p92_pf_moe_test.hip:21-28 and decode/tests/p92_nvfp4_ref_test.cpp:18-23
    for b in range(128):
        e, m = b >> 3, b & 7
        if e == 0:
            want = m * 2.0 ** -9
        elif b == 127:
            want = math.nan
        else:
            want = np.uint32(((e + 120) << 23) | (m << 20)).view(np.float32)
        got = orc.cpu().orc_decode_e4m3(b)
        pin = orc.pin().pin_decode_e4m3(b)
        if b == 127:
            assert math.isnan(got) and math.isnan(pin)
        else:
            assert got == want == pin
            assert orc.cpu().orc_decode_e4m3(b | 0x80) == -want


def test_encoders_match_cuda_headers(orc):
    base = all_bf16_floats()
    rng = np.random.default_rng(5)
    mids = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, 7.0, 448.0, 464.0, 2.0 ** -10, 2.0 ** -9 * 1.5],
                    dtype=np.float32)
    near = np.concatenate([np.nextafter(mids, np.float32(0)), mids, np.nextafter(mids, np.float32(1e9))])
    values = np.concatenate([base, base * np.float32(1 / 6), near, -near,
                             rng.standard_normal(200000).astype(np.float32) * 3,
                             rng.standard_normal(200000).astype(np.float32) * 200]).astype(np.float32)
    values = np.ascontiguousarray(values[: values.size // 2 * 2])
    got8 = np.empty(values.size, np.uint8)
    pin8 = np.empty(values.size, np.uint8)
    orc.cpu().orc_encode_e4m3_array(values, got8, values.size)
    orc.pin().pin_encode_e4m3_array(values, pin8, values.size)
    assert np.array_equal(got8, pin8)
    got4 = np.empty(values.size, np.uint8)
    orc.cpu().orc_encode_e2m1_array(values, got4, values.size)
    pin4 = np.empty(values.size // 2, np.uint8)
    orc.pin().pin_encode_e2m1x2_array(values, pin4, values.size // 2)
    # nibble order: first value of the pair in the LOW nibble (p92_nvfp4_wave64.h:12-20)
    assert np.array_equal(got4[0::2] | (got4[1::2] << 4), pin4)


def test_router_forced_tie(orc):
    # amd-gfx906/decode/tests/p92_router_test.hip:100-110
    logits = np.full((1, 256), -20.0, np.float32)
    logits[0, [200, 7, 64]] = 3.0
    ids, weights, _ = orc.router_top8(logits, np.zeros(256, np.float32))
    assert list(ids[0, :3]) == [7, 64, 200]


def test_router_invariants_and_scalar_reference(orc):
    # invariants: tests/moe_forward_test.cpp:143-157; scalar reference: p92_router_test.hip:60-72
    rng = np.random.default_rng(20260908)
    w = orc.f32_to_bf16(rng.standard_normal((256, 2560)).astype(np.float32) * 0.02)
    bias = (rng.standard_normal(256) * 0.05).astype(np.float32)
    for rows in (1, 4):
        x = orc.f32_to_bf16(rng.standard_normal((rows, 2560)).astype(np.float32))
        logits = orc.router_logits(x, w)
        ids, weights, margin = orc.router_top8(logits, bias)
        lg = orc.bf16_to_f32(x).astype(np.float64) @ orc.bf16_to_f32(w).astype(np.float64).T
        assert np.sqrt(((logits - lg) ** 2).sum() / (lg ** 2).sum()) < 1e-5
        for r in range(rows):
            assert len(set(ids[r])) == 8 and ids[r].min() >= 0 and ids[r].max() < 256
            assert (weights[r] > 0).all() and abs(weights[r].sum() - 2.5) <= 1e-5
            sc = (1.0 / (1.0 + np.exp(-lg[r].astype(np.float32)))).astype(np.float32)
            sel = sc + bias
            t = sel.copy()
            want = []
            for _ in range(8):
                bi = 0
                for e in range(1, 256):
                    if t[e] > t[bi] or (t[e] == t[bi] and e < bi):
                        bi = e
                want.append(bi)
                t[bi] = -3e38
            if margin[r] > 1e-5:
                assert list(ids[r]) == want


def test_logits_orders_differ_only_in_rounding(orc):
    rng = np.random.default_rng(3)
    w = orc.f32_to_bf16(rng.standard_normal((256, 2560)).astype(np.float32) * 0.02)
    x = orc.f32_to_bf16(rng.standard_normal((1, 2560)).astype(np.float32))
    a = orc.router_logits(x, w, gemv_order=True)
    b = orc.router_logits(x, w, gemv_order=False)
    assert np.abs(a - b).max() < 1e-5 and not np.array_equal(a, b)


@pytest.mark.parametrize("rows", [1, 2, 3, 4, 5, 63, 64, 65])
def test_permute_is_the_reference_ranking(orc, rows):
    rng = np.random.default_rng(rows)
    ids = np.stack([rng.choice(256, 8, replace=False) for _ in range(rows)]).astype(np.int32)
    order, position, counts, offsets = orc.permute(ids)
    rank = np.empty(rows * 8, np.int32)
    orc.cpu().orc_permute_ranking(ids.reshape(-1), rows * 8, rank)       # cuda/nvfp4_grouped.cu:117-132
    assert np.array_equal(position, rank)
    assert np.array_equal(np.sort(order), np.arange(rows * 8))           # a permutation (p92_pf_moe_test.hip:124-142)
    assert np.array_equal(order[position], np.arange(rows * 8))
    assert np.array_equal(counts, np.bincount(ids.reshape(-1), minlength=256))
    # host scan of src/model.cpp:1528-1540: expert-major, then row-major / slot-minor
    walk = [r * 8 + s for e in range(256) for r in range(rows) for s in range(8) if ids[r, s] == e]
    assert list(order) == walk


def test_permute_all_rows_one_expert(orc):
    ids = np.tile(np.arange(8, dtype=np.int32), (16, 1))
    order, position, counts, offsets = orc.permute(ids)
    assert counts[:8].tolist() == [16] * 8 and counts[8:].sum() == 0
    assert order[:16].tolist() == [r * 8 for r in range(16)]


def test_swizzle_layout_formula(orc):
    # cuda/nvfp4_ops.cu:869-890
    rows, cols = 200, 10
    lin = np.arange(rows * cols, dtype=np.uint32).astype(np.uint8).reshape(rows, cols)
    sw = orc.swizzle_scales(lin)
    assert sw.size == 256 * 12
    for r, c in [(0, 0), (1, 0), (31, 3), (32, 0), (127, 9), (128, 5), (199, 9)]:
        rb, rib = divmod(r, 128)
        at = (rb * 3 + c // 4) * 512 + (rib % 32) * 16 + (rib // 32) * 4 + c % 4
        assert sw[at] == lin[r, c]
    assert sw.sum() == lin.astype(np.uint64).sum()   # padding is zero


def test_quantize_block_known_answers(orc):
    # one block whose amax is 6 -> scale 1.0 (0x38), values map to themselves
    vals = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0.5, -1, -1.5, -2, -3, -4, -6, 0.25], np.float32)
    packed, scales = orc.nvfp4_quantize(orc.f32_to_bf16(vals).reshape(1, 16))
    assert scales[0, 0] == 0x38
    codes = [0, 1, 2, 3, 4, 5, 6, 7, 9, 10, 11, 12, 13, 14, 15, 0]     # 0.25 ties to even -> 0
    want = [codes[2 * i] | (codes[2 * i + 1] << 4) for i in range(8)]
    assert packed[0].tolist() == want
    # all-zero block: scale 0, every nibble 0 (multiplier forced to 0, cuda/nvfp4_ops.cu:831)
    packed, scales = orc.nvfp4_quantize(np.zeros((1, 16), np.uint16))
    assert scales[0, 0] == 0 and not packed.any()


def test_weight_pack_scale(orc):
    # cuda/nvfp4_pack.cu:255-256; N(0,0.02) weights give weight_scale_2 ~ 3.5e-5
    # (amd-gfx906/decode/receipts/03_EXPERT_PATH.md:16-17)
    rng = np.random.default_rng(11)
    w = orc.f32_to_bf16(rng.standard_normal((256, 512)).astype(np.float32) * 0.02)
    packed, scales, alpha = orc.nvfp4_pack_weight(w)
    amax = np.abs(orc.bf16_to_f32(w)).max()
    assert alpha == np.float32(amax / np.float32(6.0 * 448.0))
    assert 2e-5 < alpha < 6e-5
    assert scales.max() == 0x7e      # the block holding amax saturates the E4M3 scale at 448


def test_nvfp4_dot_against_independent_decode(orc):
    # same gate as amd-gfx906/decode/tests/p92_nvfp4_ref_test.cpp: natural-order double reference
    rng = np.random.default_rng(12345)
    for K, rows in ((2560, 8), (1024, 8)):
        w = rng.integers(0, 256, (rows, K // 2), dtype=np.uint8)
        ws = rng.integers(0, 127, (rows, K // 16), dtype=np.uint8)
        x = rng.integers(0, 256, (1, K // 2), dtype=np.uint8)
        xs = rng.integers(0, 120, (1, K // 16), dtype=np.uint8)
        out = np.empty((1, rows), np.uint16)
        orc.cpu().orc_nvfp4_gemv(x.reshape(-1), w.reshape(-1), xs.reshape(-1), ws.reshape(-1), out.reshape(-1),
                                 1, rows, K, 1.0)
        mags = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0.0, -.5, -1, -1.5, -2, -3, -4, -6])

        def dec(p, s):
            v = np.empty(p.size * 2)
            v[0::2] = mags[p & 15]
            v[1::2] = mags[p >> 4]
            sc = np.array([orc.cpu().orc_decode_e4m3(int(b)) for b in s], dtype=np.float64)
            return v * np.repeat(sc, 16)

        xv = dec(x[0], xs[0])
        for r in range(rows):
            want = float(dec(w[r], ws[r]) @ xv)
            got = float(orc.bf16_to_f32(out[0, r:r + 1])[0])
            assert abs(got - want) <= 2 ** -7 * abs(want) + 1e-3


def test_fnv1a(orc):
    # tests/moe_forward_test.cpp:61-70: low byte first
    assert orc.cpu().orc_fnv1a_bf16(np.zeros(0, np.uint16), 0) == 1469598103934665603
    h = 1469598103934665603
    for byte in (0x34, 0x12):
        h = ((h ^ byte) * 1099511628211) % 2 ** 64
    assert orc.cpu().orc_fnv1a_bf16(np.array([0x1234], np.uint16), 1) == h
