"""Fused quantise + bit-slice pack, through the C ABI, against the CPU checker (bit-exact)."""
import numpy as np
import pytest
import torch

import _capi_helpers as H
import _inputs
from bsipytorch_b200 import capi
from oracle import oracle as o

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _check(x_cpu, bits, chunk_mode, dp=2, clip_k=0.0):
    got = H.quantize_pack(x_cpu.to(DEV), dp, bits, chunk_mode, clip_k=clip_k)
    want = o.quantize_pack(x_cpu.float().numpy(), dp, bits, chunk_mode, clip_k)
    D = x_cpu.shape[1]
    np.testing.assert_array_equal(got["shifts"].cpu().numpy(), want["shifts"])
    np.testing.assert_array_equal(got["scales"].cpu().numpy(), want["scales"])
    np.testing.assert_array_equal(H.as_u64(got["words"]), want["words"])
    q8 = got["q8"].cpu().numpy()
    np.testing.assert_array_equal(q8[:, :D], want["qvals"])
    assert not q8[:, D:].any(), "padding columns of the int8 image must be zero"
    return got


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(64, 2048), (33, 768), (5, 256), (7, 250), (3, 777), (1, 64), (2, 8192)])
@pytest.mark.parametrize("chunk_mode", [True, False])
def test_pack_matches_oracle(dtype, shape, chunk_mode):
    g = torch.Generator().manual_seed(shape[0] * 131 + shape[1])
    x = torch.randn(*shape, generator=g) * torch.where(torch.rand(*shape, generator=g) < 0.01, 20.0, 1.0)
    _check(x.to(dtype), 7 if chunk_mode else 6, chunk_mode)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("chunk_mode", [True, False])
def test_pack_edge_rows(dtype, chunk_mode):
    _check(_inputs.edge_rows(512, dtype), 7, chunk_mode)
    _check(_inputs.edge_rows(512, dtype), 6, chunk_mode)


@pytest.mark.parametrize("bits", [2, 3, 4, 5, 8])
def test_pack_other_bit_widths(bits):
    g = torch.Generator().manual_seed(bits)
    _check(torch.randn(9, 512, generator=g), bits, True)
    _check(torch.randn(9, 512, generator=g) * 0.02, bits, False)


@pytest.mark.parametrize("dp", [0, 1, 3])
def test_pack_other_decimal_places(dp):
    g = torch.Generator().manual_seed(dp)
    _check(torch.randn(6, 512, generator=g), 7, True, dp=dp)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_pack_mixes_fast_and_generic_chunks(dtype):
    """Chunks holding huge, infinite or NaN values leave the fast quantiser for the 64-bit one; their
    neighbours stay on the fast one. Both give the checker's integers."""
    g = torch.Generator().manual_seed(11)
    x = torch.randn(40, 1024, generator=g)
    big = 6.0e4 if dtype == torch.float16 else 3.0e7      # x100 reaches 2^23 either way
    x[1, 5] = big
    x[2, 300] = -big
    x[3, 600] = float("inf")
    x[4, 1000] = float("-inf")
    x[5, 0] = float("nan")
    x[6, 256:512] = big
    x[7] = big
    _check(x.to(dtype), 7, True)
    _check(x.to(dtype), 6, False)


def test_pack_generic_queue_overflow():
    """More generic-path chunks than one warp can queue: the warp redoes all of its chunks."""
    g = torch.Generator().manual_seed(12)
    x = torch.randn(5000, 2048, generator=g)
    x[:, ::256] = 1.0e6                                   # every chunk of every row is out of fast range
    x[::7] = torch.randn(2048, generator=g)               # ... except the rows left plain
    _check(x, 7, True)
    _check(x.to(torch.bfloat16), 7, True)


def test_pack_config_distributions():
    q, k = _inputs.fc1(Q=64, R=96)
    _check(q, 7, True)
    _check(k, 6, False)
    q, k = _inputs.fc2(Q=16, R=32)
    got = _check(q, 7, True)
    assert not got["words"][:, 6, :].any(), "relu activations: the sign slice is empty"


def test_pack_unaligned_rows_take_the_scalar_path():
    # A view whose rows start at odd element offsets cannot use 16-byte loads.
    g = torch.Generator().manual_seed(9)
    base = torch.randn(10, 515, generator=g).to(torch.float16).to(DEV)
    x = base[:, 3:]                     # D = 512, ldx = 515, misaligned start
    rows, D = x.shape
    words = torch.zeros(rows, 7, 8, dtype=torch.int64, device=DEV)
    scales = torch.zeros(rows, 2, dtype=torch.float32, device=DEV)
    rc = capi.lib().bsi_b200_quantize_pack(capi.ptr(x), capi.DTYPE_F16, rows, D, 515, 2, 7, 1, capi.ptr(words),
                                           capi.ptr(scales), None, None, 0, capi.stream_ptr())
    capi.check(rc)
    want = o.quantize_pack(x.float().cpu().numpy(), 2, 7, True)
    np.testing.assert_array_equal(H.as_u64(words), want["words"])
    np.testing.assert_array_equal(scales.cpu().numpy(), want["scales"])


def test_pack_empty_and_bad_arguments():
    L = capi.lib()
    x = torch.zeros(4, 64, device=DEV)
    assert L.bsi_b200_quantize_pack(capi.ptr(x), 0, 0, 64, 64, 2, 7, 1, None, None, None, None, 0, None) == capi.OK
    assert L.bsi_b200_quantize_pack(capi.ptr(x), 0, 4, 64, 32, 2, 7, 1, None, None, None, None, 0, None) == capi.ERR_INVALID
    q8 = torch.zeros(4, 256, dtype=torch.int8, device=DEV)
    # ld8 smaller than 256 * chunks
    assert L.bsi_b200_quantize_pack(capi.ptr(x), 0, 4, 64, 64, 2, 7, 1, None, None, None, capi.ptr(q8), 128, None) == capi.ERR_INVALID


def test_recombine_inverts_the_slices():
    g = torch.Generator().manual_seed(4)
    for bits, chunk_mode, D in [(7, True, 1024), (6, False, 768), (8, True, 256), (3, True, 512), (7, False, 320)]:
        x = torch.randn(12, D, generator=g).to(DEV)
        got = H.quantize_pack(x, 2, bits, chunk_mode)
        q8 = H.recombine_i8(got["words"])
        W = (D + 63) // 64
        torch.testing.assert_close(q8[:, : 64 * W], got["q8"][:, : 64 * W], rtol=0, atol=0)
        assert not q8[:, 64 * W:].any()


def test_pack_matches_reference_kernels():
    """Same inputs through the reference's own kernels (compiled unmodified for sm_100a)."""
    from oracle import ref_gpu
    if not ref_gpu.available():
        pytest.skip("reference kernels not built on this machine")
    for dtype in (torch.float32, torch.float16, torch.bfloat16):
        q, k = _inputs.fc1(Q=96, R=160, D=2048, dtype=dtype)
        mine = H.quantize_pack(q.to(DEV), 2, 7, True)
        words, shifts, scales = ref_gpu.pack_queries_chunk(q.to(DEV), 2, 7)
        assert torch.equal(mine["words"], words) and torch.equal(mine["shifts"], shifts) and torch.equal(mine["scales"], scales)
    q, k = _inputs.fc1(Q=8, R=160, D=2048)
    mine = H.quantize_pack(k.to(DEV), 2, 6, False)
    words, shifts, scales, ints = ref_gpu.pack_rows(k.to(DEV), 2, 6)
    assert torch.equal(mine["words"], words) and torch.equal(mine["shifts"], shifts) and torch.equal(mine["scales"], scales)
    assert torch.equal(mine["q8"][:, :2048].long(), ints)
    edge = _inputs.edge_rows(512).to(DEV)
    mine = H.quantize_pack(edge, 2, 7, True)
    words, shifts, scales = ref_gpu.pack_queries_chunk(edge, 2, 7)
    assert torch.equal(mine["words"], words) and torch.equal(mine["shifts"], shifts)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("clip_k", [1.5, 3.0, 50.0])
def test_pack_with_outlier_clipping(dtype, clip_k):
    """BSI_FIXED_CLIP_K of the reference: the shift of a chunk / row follows min(max |v|, clip_k * mean |v|); outliers
    saturate. Against the checker, and against the reference's own kernels where they were built."""
    g = torch.Generator().manual_seed(int(clip_k * 10))
    x = torch.randn(37, 1000, generator=g) * torch.where(torch.rand(37, 1000, generator=g) < 0.02, 30.0, 1.0)
    x[3] = 0.0
    x[4, 10] = 1.0e4
    x = x.to(dtype)
    got_c = _check(x, 7, True, clip_k=clip_k)
    got_r = _check(x * 0.02, 6, False, clip_k=clip_k)
    plain = H.quantize_pack(x.to(DEV), 2, 7, True)
    if clip_k < 10:
        assert not torch.equal(plain["shifts"], got_c["shifts"]), "clipping must change some shifts on this input"
        assert int(got_c["q8"].max()) == 63 and int(got_c["q8"].min()) == -64     # saturated outliers
    from oracle import ref_gpu
    if ref_gpu.available():
        words, shifts, scales = ref_gpu.pack_queries_chunk(x.to(DEV), 2, 7, clip_k=clip_k)
        assert torch.equal(got_c["words"], words) and torch.equal(got_c["shifts"], shifts) and torch.equal(got_c["scales"], scales)
        words, shifts, scales, ints = ref_gpu.pack_rows((x * 0.02).to(DEV), 2, 6, clip_k=clip_k)
        assert torch.equal(got_r["words"], words) and torch.equal(got_r["shifts"], shifts)
        assert torch.equal(got_r["q8"][:, :1000].long(), ints)
