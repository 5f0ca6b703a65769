"""CPU tests of the checker itself: known answers, hand-computed streams, internal consistency."""
import numpy as np
import pytest

from oracle import oracle as o


def test_round_half_away_matches_reference_rule():
    # bsiFunctions.cpp:759-771 / quant.cuh:24-29: std::round semantics on double(float(x)) * 10^dp
    assert o.round_half_away(2.5) == 3
    assert o.round_half_away(-2.5) == -3
    assert o.round_half_away(0.49999999) == 0
    assert o.round_half_away(-0.5) == -1
    assert o.round_half_away(float(np.float32(0.005)) * 100.0) == 0      # float32(0.005) < 0.005 -> 0.49999998 -> 0
    assert o.round_half_away(float(np.float32(0.025)) * 100.0) == 3      # float32(0.025) > 0.025 -> 2.50000004 -> 3
    assert o.round_half_away(float(np.float32(0.125)) * 100.0) == 13     # exact tie 12.5 -> away from zero
    assert o.round_half_away(float(np.float32(-0.125)) * 100.0) == -13
    assert o.round_half_away(float("nan")) == 0
    assert o.round_half_away(1e30) == 2 ** 63 - 1


def test_compute_shift():
    # quant.cuh:82-108: bits = bit width of max, shift = max(0, bits - (fixed_bits - 1)), capped at 62
    assert o.compute_shift(0, 7) == 0
    assert o.compute_shift(63, 7) == 0
    assert o.compute_shift(64, 7) == 1
    assert o.compute_shift(127, 7) == 1
    assert o.compute_shift(128, 7) == 2
    assert o.compute_shift(31, 6) == 0
    assert o.compute_shift(32, 6) == 1
    assert o.compute_shift(2 ** 63, 7) == 58
    assert o.compute_shift(2 ** 63, 2) == 62


def test_known_answer_vectors_of_reference_cpu_tests():
    # bsi_ops/benchmarks/test_bsi_simple.py:21-35 and test_fix_verification.py:41-55:
    # [1,2,3,4].[4,3,2,1] = 20, negated key = -20; results are sum(round(q*10^dp)*round(k*10^dp))/10^(2dp)
    q = np.array([[1.0, 2.0, 3.0, 4.0]], np.float32)
    k = np.array([[4.0, 3.0, 2.0, 1.0], [-4.0, -3.0, -2.0, -1.0], [0.5, 0.5, 0.5, 0.5]], np.float32)
    out = o.cpu_dot(q, k, decimal_places=2)
    np.testing.assert_allclose(out, [[20.0, -20.0, 5.0]], atol=0.0)
    # K @ q style 3x4 case (test_bsi_simple.py:43-69)
    K = np.array([[1, 0, 0, 0], [0.5, 0.5, 0.5, 0.5], [1, 2, 3, 4]], np.float32)
    qv = np.array([[1.0, 2.0, 3.0, 4.0]], np.float32)
    np.testing.assert_allclose(o.cpu_dot(qv, K, 2), [[1.0, 5.0, 30.0]], atol=0.0)
    # matrix_multiplication_test.py:5-18 pattern: every entry a plain integer dot
    rng = np.random.default_rng(5)
    a = rng.integers(-9, 10, (5, 16)).astype(np.float32)
    b = rng.integers(-9, 10, (7, 16)).astype(np.float32)
    np.testing.assert_allclose(o.cpu_dot(a, b, 1), a @ b.T, atol=0.0)


def test_cpu_dot_equals_integer_dot_of_rounded_values():
    rng = np.random.default_rng(1)
    q = rng.standard_normal((9, 300)).astype(np.float32)
    k = (rng.standard_normal((11, 300)) * 0.3).astype(np.float32)
    qi = np.array([[o.round_half_away(float(v) * 100.0) for v in row] for row in q], np.int64)
    ki = np.array([[o.round_half_away(float(v) * 100.0) for v in row] for row in k], np.int64)
    np.testing.assert_array_equal(o.cpu_dot(q, k, 2), (qi @ ki.T) / 10000.0)
    one = o.cpu_dot(q, k, 2, threads=1)
    np.testing.assert_array_equal(one, o.cpu_dot(q, k, 2, threads=0))


def test_quantize_pack_layout_and_values():
    x = np.zeros((1, 130), np.float32)
    x[0, 0] = 0.63      # 63 -> fits 7 bits, shift 0
    x[0, 1] = -0.63     # -63 = 0b1000001 in 7-bit two's complement
    x[0, 65] = 0.01
    x[0, 129] = -0.01
    r = o.quantize_pack(x, 2, 7, chunk_mode=True)
    assert r["shifts"].tolist() == [[0]] and r["scales"].tolist() == [[1.0]]
    assert r["qvals"][0, :2].tolist() == [63, -63] and r["qvals"][0, 65] == 1 and r["qvals"][0, 129] == -1
    w = r["words"][0]
    assert w.shape == (7, 3)
    # element 0 = 63 = 0b0111111: slices 0..5, bit 0 of word 0; element 1 = -63: slices 0 and 6, bit 1
    assert int(w[0, 0]) == 3
    for s in range(1, 6):
        assert int(w[s, 0]) == 1
    assert int(w[6, 0]) == 2
    # |v| = 64 needs 7 magnitude bits, so it forces shift 1 even though -64 itself would fit
    x2 = x.copy(); x2[0, 1] = -0.64
    r2 = o.quantize_pack(x2, 2, 7, chunk_mode=True)
    assert r2["shifts"].tolist() == [[1]] and r2["qvals"][0, :2].tolist() == [32, -32]
    assert int(w[0, 1]) == 2                  # element 65 -> word 1 bit 1, slice 0
    assert all(int(w[s, 2]) == 2 for s in range(7))   # element 129 = -1: every slice, word 2 bit 1


def test_chunk_shift_is_per_256_elements_and_row_shift_is_global():
    x = np.full((1, 512), 0.10, np.float32)
    x[0, 300] = 5.0       # 500 -> 9 bits -> shift 3 in chunk 1 only
    c = o.quantize_pack(x, 2, 7, chunk_mode=True)
    assert c["shifts"].tolist() == [[0, 3]]
    assert c["qvals"][0, 0] == 10 and c["qvals"][0, 300] == 63 and c["qvals"][0, 301] == 1  # (10+4)>>3
    r = o.quantize_pack(x, 2, 7, chunk_mode=False)
    assert r["shifts"].tolist() == [3] and r["qvals"][0, 0] == 1 and r["qvals"][0, 300] == 63


def test_weighted_popcount_equals_integer_product():
    rng = np.random.default_rng(0)
    xq = (rng.standard_normal((40, 1024)) * np.where(rng.random((40, 1024)) < 0.01, 20, 1)).astype(np.float32)
    xk = (rng.standard_normal((48, 1024)) * 0.02).astype(np.float32)
    a, ia = o.fixed_dot(xq, xk, want_iacc=True, via="i8")
    b, ib = o.fixed_dot(xq, xk, want_iacc=True, via="popc")
    np.testing.assert_array_equal(ia, ib)
    np.testing.assert_array_equal(a.view(np.uint32), b.view(np.uint32))
    assert np.abs(ia).max() <= 256 * 64 * 32
    # close to the float product: error is the quantisation step, not a bug
    assert np.abs(a - xq @ xk.T).max() < 2.0


def _ewah_python(words, compress):
    """Independent, literal transcription of the sequential loop (ewah.cuh:178-232) in Python."""
    W = len(words)
    out, idx = [], 0
    ones = (1 << 64) - 1
    while idx < W:
        run_len = run_bit = 0
        if compress and words[idx] in (0, ones):
            fill = words[idx]
            run_bit = 1 if fill == ones else 0
            k = idx
            while k < W and words[k] == fill:
                k += 1
            run_len, idx = k - idx, k
        start = idx
        while idx < W and not (compress and words[idx] in (0, ones)):
            idx += 1
        lit = idx - start
        out.append(run_bit | ((run_len & 0xFFFFFFFF) << 1) | (lit << 33))
        out.extend(words[start:idx])
    return out


@pytest.mark.parametrize("W", [1, 4, 33, 100])
def test_ewah_encode_decode_against_python_walk(W):
    rng = np.random.default_rng(W)
    ones = np.uint64(0xFFFFFFFFFFFFFFFF)
    slices = []
    for kind in range(12):
        w = rng.integers(1, 2 ** 63, W, dtype=np.uint64)
        if kind % 4 == 1:
            w[:] = 0
        elif kind % 4 == 2:
            w[rng.random(W) < 0.6] = 0
            w[rng.random(W) < 0.3] = ones
        elif kind % 4 == 3:
            w[:] = ones
            if W > 2:
                w[W // 2] = 5
        slices.append(w)
    words = np.stack(slices)
    for flags in (np.ones(12, np.int32), np.zeros(12, np.int32)):
        stream, off, length = o.ewah_encode(words, flags)
        for s in range(12):
            want = _ewah_python([int(v) for v in words[s]], int(flags[s]))
            got = [int(v) for v in stream[off[s]: off[s] + length[s]]]
            assert got == want
            np.testing.assert_array_equal(o.ewah_decode(stream[off[s]: off[s] + length[s]], W), words[s])


def test_compress_flag_threshold_half():
    # M = 1 - (1-p)^128 - p^128 <= 0.5  <=>  p <= ~0.0054 or p >= ~0.9946 (ewah.cuh:84-102)
    W = 128
    bits = W * 64
    counts = np.array([0, int(0.005 * bits), int(0.006 * bits), bits // 2, int(0.994 * bits), int(0.9955 * bits), bits],
                      np.uint64)
    assert o.compress_flags(counts, W, 0.5).tolist() == [1, 1, 0, 0, 0, 1, 1]


def test_relu_activations_compress_sign_slice_to_one_word():
    # FC2-like activations are non-negative: the sign slice is all zero -> one RLW(run of W zero words)
    rng = np.random.default_rng(3)
    x = np.maximum(rng.standard_normal((4, 8192)), 0).astype(np.float32)
    r = o.quantize_pack(x, 2, 7, chunk_mode=True)
    words = r["words"].reshape(4 * 7, 128)
    flags = o.compress_flags(o.slice_popcount(words), 128, 0.5)
    assert flags.reshape(4, 7)[:, 6].tolist() == [1, 1, 1, 1]
    stream, off, length = o.ewah_encode(words, flags)
    for q in range(4):
        s = q * 7 + 6
        assert length[s] == 1 and int(stream[off[s]]) == (128 << 1)


def test_variable_slice_mode_restatement():
    """Variable-slice mode: slice-count rule (bsi_vector_cuda.cpp:746-754), two's-complement slices with the
    reference's per-row weights reproduce the exact integer dot, and the print-style known answers of the
    reference's CPU scripts hold (test_bsi_simple.py: [1,2,3,4].[4,3,2,1] = 20, negated = -20)."""
    assert [o.variable_slices(m) for m in (0, 1, 2, 3, 4, 255, 256, 2 ** 40)] == [2, 3, 4, 4, 5, 10, 11, 43]
    q = np.array([[1, 2, 3, 4], [-1, -2, -3, -4], [0.5, 0.25, 0, -0.125]], np.float32)
    k = np.array([[4, 3, 2, 1], [1, 0, 0, 0]], np.float32)
    out = o.variable_dot(q, k, 2)
    np.testing.assert_allclose(out[:2], [[20, 1], [-20, -1]], rtol=0, atol=1e-6)
    qa, kb = o.variable_pack(q, 2), o.variable_pack(k, 2, per_row=True)
    assert qa["S"] == 9 + 2 and list(kb["row_slices"]) == [9 + 2, 7 + 2]          # 400 -> 9 bits, 100 -> 7 bits
    assert list(qa["negative"]) == [False, True, True] and qa["weights"][0, -1] > 0 > qa["weights"][1, -1]
    np.testing.assert_array_equal(o.variable_dot_popc(qa, kb, 2).view(np.uint32), out.view(np.uint32))
    rng = np.random.default_rng(3)
    xq = rng.standard_normal((6, 200)).astype(np.float32) * 3
    xk = (rng.standard_normal((5, 200)) * 0.05).astype(np.float32)
    a = o.variable_dot(xq, xk, 2)
    b = o.variable_dot_popc(o.variable_pack(xq, 2), o.variable_pack(xk, 2, per_row=True), 2)
    np.testing.assert_array_equal(a.view(np.uint32), b.view(np.uint32))
