"""EWAH / verbatim slice encoder and decoder, through the C ABI, against the CPU checker."""
import numpy as np
import pytest
import torch

import _capi_helpers as H
import _inputs
from oracle import oracle as o

pytestmark = pytest.mark.gpu
DEV = "cuda"
ONES = np.uint64(0xFFFFFFFFFFFFFFFF)


def _structured(S, W, seed):
    rng = np.random.default_rng(seed)
    w = rng.integers(1, 2 ** 63, (S, W), dtype=np.uint64)
    for s in range(S):
        k = s % 8
        if k == 0:
            w[s] = 0
        elif k == 1:
            w[s] = ONES
        elif k == 2:
            w[s][rng.random(W) < 0.7] = 0
        elif k == 3:
            w[s][rng.random(W) < 0.5] = 0
            w[s][rng.random(W) < 0.4] = ONES
        elif k == 4:
            w[s] = 0
            w[s][rng.integers(0, W)] = 1       # very sparse: compressible
        elif k == 5:
            w[s] = ONES
            w[s][rng.integers(0, W)] = ~np.uint64(1 << 5)
        elif k == 6:
            w[s][: W // 2] = 0
            w[s][W // 2:] = ONES
        # k == 7: dense random literals
    return w


def _compare(words_np, threshold):
    S, W = words_np.shape
    wt = torch.from_numpy(words_np.view(np.int64)).to(DEV)
    counts = o.slice_popcount(words_np)
    flags = o.compress_flags(counts, W, threshold)
    stream, off, length = o.ewah_encode(words_np, flags)

    g_stream, g_off, g_len, g_flags = H.ewah_encode(wt, threshold)
    np.testing.assert_array_equal(g_flags.cpu().numpy(), flags)
    np.testing.assert_array_equal(g_off.cpu().numpy(), off)
    np.testing.assert_array_equal(g_len.cpu().numpy(), length)
    np.testing.assert_array_equal(H.as_u64(g_stream), stream)

    s_stream, s_off, s_len, s_flags, s_counts, s_sizes = H.ewah_steps(wt, threshold)
    np.testing.assert_array_equal(H.as_u64(s_counts), counts)
    np.testing.assert_array_equal(s_flags.cpu().numpy(), flags)
    np.testing.assert_array_equal(H.as_u64(s_sizes), length.astype(np.uint64))
    np.testing.assert_array_equal(H.as_u64(s_stream), stream)
    np.testing.assert_array_equal(s_len.cpu().numpy(), length)

    back = H.ewah_decode(g_stream, g_off, g_len, W)
    np.testing.assert_array_equal(H.as_u64(back), words_np)
    return flags, length


@pytest.mark.parametrize("W", [1, 3, 4, 31, 32, 33, 64, 128, 257])
def test_ewah_structured_words(W):
    for thr in (0.5, 0.2, 1.0, 0.0):
        _compare(_structured(40, W, W), thr)


def test_ewah_many_slices_offsets_scan():
    # more slices than one scan tile (8192) so that the carry across tiles is exercised
    _compare(_structured(3000, 8, 7), 0.5)
    _compare(_structured(20011, 4, 5), 0.5)


def test_ewah_offsets_is_an_exclusive_prefix_sum():
    import ctypes as C
    from bsipytorch_b200 import capi
    for S in (1, 5, 1024, 8191, 8192, 8193, 70001):
        sizes = torch.randint(0, 300, (S,), generator=torch.Generator().manual_seed(S), dtype=torch.int64).to(DEV)
        off = torch.full((S,), -1, dtype=torch.int64, device=DEV)
        total = torch.full((1,), -1, dtype=torch.int64, device=DEV)
        capi.check(capi.lib().bsi_b200_ewah_offsets(capi.ptr(sizes), S, capi.ptr(off), capi.ptr(total), capi.stream_ptr()))
        want = torch.cumsum(sizes, 0) - sizes
        assert torch.equal(off, want) and int(total.item()) == int(sizes.sum().item())


def test_ewah_on_packed_activations():
    q, _ = _inputs.fc2(Q=24, R=8)
    got = H.quantize_pack(q.to(DEV), 2, 7, True)
    words = H.as_u64(got["words"]).reshape(24 * 7, 128)
    flags, length = _compare(words, 0.5)
    assert flags.reshape(24, 7)[:, 6].all() and (length.reshape(24, 7)[:, 6] == 1).all()
    assert (length.reshape(24, 7)[:, 0] == 129).all()      # dense low slices stay verbatim: RLW + 128 literals
    q, _ = _inputs.fc1(Q=24, R=8)
    got = H.quantize_pack(q.to(DEV), 2, 7, True)
    _compare(H.as_u64(got["words"]).reshape(24 * 7, 32), 0.5)


def test_ewah_decode_truncated_and_overlong_streams():
    # decode pads with zeros when the stream ends early and stops at W when it is too long (ewah.cuh:16-32)
    W = 16
    stream = np.array([(3 << 1) | (2 << 33), 7, 9, 1 | (40 << 1)], np.uint64)   # 3 zero words, 2 literals, 40 one-words
    want = o.ewah_decode(stream, W)
    t = torch.from_numpy(stream.view(np.int64)).to(DEV)
    off = torch.zeros(2, dtype=torch.int64, device=DEV)
    length = torch.tensor([4, 2], dtype=torch.int32, device=DEV)    # second "slice": the same stream cut after 2 words
    back = H.as_u64(H.ewah_decode(t, off, length, W))
    np.testing.assert_array_equal(back[0], want)
    np.testing.assert_array_equal(back[1], o.ewah_decode(stream[:2], W))


def test_ewah_matches_reference_kernels():
    from oracle import ref_gpu
    if not ref_gpu.available():
        pytest.skip("reference kernels not built on this machine")
    for W, thr in [(32, 0.5), (128, 0.5), (33, 0.2), (4, 1.0)]:
        words_np = _structured(64, W, 100 + W)
        wt = torch.from_numpy(words_np.view(np.int64)).to(DEV)
        r_stream, r_off, r_len, r_flags, r_counts = ref_gpu.ewah_encode(wt, thr)
        g_stream, g_off, g_len, g_flags = H.ewah_encode(wt, thr)
        assert torch.equal(g_flags, r_flags) and torch.equal(g_off, r_off) and torch.equal(g_len, r_len)
        assert torch.equal(g_stream, r_stream)
        assert torch.equal(H.ewah_decode(g_stream, g_off, g_len, W), ref_gpu.ewah_decode(r_stream, r_off, r_len, W))
