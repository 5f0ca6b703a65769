"""Dot core, through the C ABI: every engine against the CPU checker, bit-exact.

Integer per-chunk accumulators must equal the weighted popcount sum exactly; float32 outputs are
compared bit for bit as well (tolerance the task allows: rtol 1e-5 / atol 1e-6 -- we ask for zero).
"""
import numpy as np
import pytest
import torch

import _capi_helpers as H
import _inputs
from bsipytorch_b200 import capi
from oracle import oracle as o

pytestmark = pytest.mark.gpu
DEV = "cuda"
# 1000 + n pins single-CTA tiles of width n; 3000 + n pins paired-CTA (cta_group::2) tiles of width n
ENGINES = {"simt": capi.ENGINE_SIMT, "tcgen05": capi.ENGINE_TCGEN05, "tcgen05_bn64": 1064,
           "tcgen05_bn128": 1128, "tcgen05_bn256": 1256, "pair_bn64": 3064, "pair_bn96": 3096, "pair_bn128": 3128,
           "pair_bn160": 3160, "pair_bn192": 3192, "pair_bn224": 3224, "pair_bn256": 3256}


def _prepare(q, k, bits_q=7, bits_k=6, chunk_mode=True, dp=2):
    qa = H.quantize_pack(q.to(DEV), dp, bits_q, chunk_mode)
    kb = H.quantize_pack(k.to(DEV), dp, bits_k, False)
    Bw = torch.from_numpy(o.slice_weights(bits_k, kb["scales"].cpu().numpy())).to(DEV)
    return qa, kb, Bw


def _oracle(q, k, bits_q=7, bits_k=6, chunk_mode=True, dp=2):
    qa = o.quantize_pack(q.float().numpy(), dp, bits_q, chunk_mode)
    kb = o.quantize_pack(k.float().numpy(), dp, bits_k, False)
    chunks = (q.shape[1] + 255) // 256
    return o.dot_i8(o.pad_i8(qa["qvals"], chunks), qa["scales"], o.pad_i8(kb["qvals"], chunks),
                    kb["scales"], o.scale_inv(dp), want_iacc=True)


def _assert_bits(got, want):
    np.testing.assert_array_equal(got.cpu().numpy().view(np.uint32), want.view(np.uint32))


SHAPES = [(64, 256, 2048), (70, 100, 512), (200, 300, 1024), (128, 256, 256), (1, 1, 256), (130, 513, 768),
          (33, 65, 250), (512, 1100, 512), (300, 2000, 256)]


@pytest.mark.parametrize("engine", list(ENGINES))
@pytest.mark.parametrize("shape", SHAPES)
def test_dot_i8_engines_match_oracle(engine, shape):
    Q, R, D = shape
    q, k = _inputs.fc1(Q=Q, R=R, D=D, seed=Q + R + D, dtype=torch.float32)
    qa, kb, _ = _prepare(q, k)
    out, iacc = H.dot_i8(qa["q8"], qa["scales"], kb["q8"], kb["scales"], o.scale_inv(2), ENGINES[engine], True)
    want, want_i = _oracle(q, k)
    np.testing.assert_array_equal(iacc.cpu().numpy(), want_i)
    _assert_bits(out, want)
    # the same call without the debug output
    out2 = H.dot_i8(qa["q8"], qa["scales"], kb["q8"], kb["scales"], o.scale_inv(2), ENGINES[engine], False)
    assert torch.equal(out, out2)
    assert capi.device_status() == 0


@pytest.mark.parametrize("shape", [(64, 256, 2048), (70, 100, 512), (96, 160, 1024)])
def test_dot_words_bmma_matches_oracle(shape):
    Q, R, D = shape
    q, k = _inputs.fc1(Q=Q, R=R, D=D, seed=11 + Q, dtype=torch.float16)
    qa, kb, Bw = _prepare(q, k)
    out, iacc = H.dot_words(qa["words"], qa["scales"], kb["words"], Bw, o.scale_inv(2), True)
    want, want_i = _oracle(q, k)
    np.testing.assert_array_equal(iacc.cpu().numpy(), want_i)
    _assert_bits(out, want)
    # and the weighted-popcount form of the checker on the same words
    pop = o.dot_popc(H.as_u64(qa["words"]), qa["scales"].cpu().numpy(), H.as_u64(kb["words"]), Bw.cpu().numpy(),
                     o.scale_inv(2))
    _assert_bits(out, pop)


@pytest.mark.parametrize("engine", ["simt", "tcgen05"])
def test_dot_row_scale_mode(engine):
    # one scale per query row (qs_stride = 0): the mode used when the word count is not a multiple of 4
    q, k = _inputs.c1(Q=40, R=72, D=320)
    qa, kb, _ = _prepare(q, k, chunk_mode=False)
    out, iacc = H.dot_i8(qa["q8"], qa["scales"], kb["q8"], kb["scales"], o.scale_inv(2), ENGINES[engine], True)
    want, want_i = _oracle(q, k, chunk_mode=False)
    np.testing.assert_array_equal(iacc.cpu().numpy(), want_i)
    _assert_bits(out, want)


@pytest.mark.parametrize("bits", [(8, 8), (4, 4), (7, 7), (2, 3)])
def test_dot_other_slice_counts(bits):
    bq, bk = bits
    q, k = _inputs.c1(Q=48, R=80, D=512, seed=bq * 10 + bk)
    qa, kb, Bw = _prepare(q, k, bq, bk)
    want, want_i = _oracle(q, k, bq, bk)
    out, iacc = H.dot_i8(qa["q8"], qa["scales"], kb["q8"], kb["scales"], o.scale_inv(2), capi.ENGINE_TCGEN05, True)
    np.testing.assert_array_equal(iacc.cpu().numpy(), want_i)
    _assert_bits(out, want)
    if bits in [(8, 8), (4, 4), (7, 7)]:
        out_b = H.dot_words(qa["words"], qa["scales"], kb["words"], Bw, o.scale_inv(2))
        _assert_bits(out_b, want)


def test_dot_extreme_accumulators():
    # every query element +63 / -64 and every key element -32 / +31: |I| reaches 256*64*32 = 2^19
    Q, R, D = 32, 32, 512
    q = torch.full((Q, D), 0.63)
    q[1::2] = -0.64 * 1.0
    q[1::2, 0] = -0.63      # keep max |v| at 64 -> shift 1 for odd rows; even rows shift 0
    k = torch.full((R, D), 0.31)
    k[1::2] = -0.31
    qa, kb, _ = _prepare(q, k)
    want, want_i = _oracle(q, k)
    for engine in ("simt", "tcgen05"):
        out, iacc = H.dot_i8(qa["q8"], qa["scales"], kb["q8"], kb["scales"], o.scale_inv(2), ENGINES[engine], True)
        np.testing.assert_array_equal(iacc.cpu().numpy(), want_i)
        _assert_bits(out, want)
    assert np.abs(want_i).max() >= 256 * 63 * 31


def test_dot_matches_reference_kernels():
    """The reference's fixed76 chunk-scale kernels (rsweep4 + tail) on the same packed operands."""
    from oracle import ref_gpu
    if not ref_gpu.available():
        pytest.skip("reference kernels not built on this machine")
    for (Q, R, D) in [(64, 256, 2048), (96, 160, 1024), (128, 512, 4096)]:
        q, k = _inputs.fc1(Q=Q, R=R, D=D, seed=Q)
        qa, kb, Bw = _prepare(q, k)
        ref = ref_gpu.dot_fixed76(qa["words"], qa["scales"], kb["words"], Bw, o.scale_inv(2))
        for engine in ("simt", "tcgen05"):
            out = H.dot_i8(qa["q8"], qa["scales"], kb["q8"], kb["scales"], o.scale_inv(2), ENGINES[engine])
            assert torch.equal(out, ref), engine
        assert torch.equal(H.dot_words(qa["words"], qa["scales"], kb["words"], Bw, o.scale_inv(2)), ref)


def test_pair_kernel_fc1_matches_reference_kernels():
    """The kernel the benchmark times (paired CTAs, automatic tile width at Q = 512) against the reference's own
    fixed76 kernels on the full FC1 operands, and every other tile width on a 512 x 1024 column block."""
    from oracle import ref_gpu
    if not ref_gpu.available():
        pytest.skip("reference kernels not built on this machine")
    q, k = _inputs.fc1()
    qa, kb, Bw = _prepare(q, k)
    si = o.scale_inv(2)
    ref = ref_gpu.dot_fixed76(qa["words"], qa["scales"], kb["words"], Bw, si)
    out = H.dot_i8(qa["q8"], qa["scales"], kb["q8"], kb["scales"], si, capi.ENGINE_TCGEN05)
    assert torch.equal(out, ref)
    for width in (64, 96, 128, 160, 192, 224, 256):
        out = H.dot_i8(qa["q8"], qa["scales"], kb["q8"][:1024].contiguous(), kb["scales"][:1024].contiguous(), si, 3000 + width)
        assert torch.equal(out, ref[:, :1024]), width
    assert capi.device_status() == 0


@pytest.mark.parametrize("cfg", ["fc1", "fc2"])
def test_dot_full_size_configs(cfg):
    """BASELINE sizes: engines agree bit for bit with each other, and with the checker on a row sample."""
    q, k = (_inputs.fc1() if cfg == "fc1" else _inputs.fc2())
    qa, kb, Bw = _prepare(q, k)
    si = o.scale_inv(2)
    out_tc = H.dot_i8(qa["q8"], qa["scales"], kb["q8"], kb["scales"], si, capi.ENGINE_TCGEN05)
    out_simt = H.dot_i8(qa["q8"], qa["scales"], kb["q8"], kb["scales"], si, capi.ENGINE_SIMT)
    assert torch.equal(out_tc, out_simt)
    out_bmma = H.dot_words(qa["words"], qa["scales"], kb["words"], Bw, si)
    assert torch.equal(out_tc, out_bmma)
    rows = torch.arange(0, q.shape[0], 37)
    want, _ = _oracle(q[rows], k)
    _assert_bits(out_tc[rows.to(DEV)], want)
    # linearity in the integer domain: doubling a key row's scale doubles that output column exactly
    bw2 = kb["scales"].clone()
    bw2[5] *= 2
    out2 = H.dot_i8(qa["q8"], qa["scales"], kb["q8"], bw2, si, capi.ENGINE_TCGEN05)
    assert torch.equal(out2[:, 5], out_tc[:, 5] * 2) and torch.equal(out2[:, 6:], out_tc[:, 6:])
    assert capi.device_status() == 0


def test_dot_bad_arguments():
    L = capi.lib()
    a = torch.zeros(4, 256, dtype=torch.int8, device=DEV)
    f = torch.ones(4, 1, device=DEV)
    out = torch.zeros(4, 4, device=DEV)
    import ctypes as C
    args = lambda lda, ldo, eng: (capi.ptr(a), lda, capi.ptr(f), 1, capi.ptr(a), 256, capi.ptr(f), 4, 4, 1,
                                   C.c_float(1.0), capi.ptr(out), ldo, None, eng, None)
    assert L.bsi_b200_dot_i8(*args(128, 4, 0)) == capi.ERR_INVALID      # lda < 256 * chunks
    assert L.bsi_b200_dot_i8(*args(256, 2, 0)) == capi.ERR_INVALID      # ldo < R
    assert L.bsi_b200_dot_i8(*args(256, 4, 3)) == capi.ERR_INVALID      # BMMA engine needs slice words
    assert L.bsi_b200_dot_i8(*args(256, 4, 1032)) == capi.ERR_INVALID   # tile width not 64/128/256


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape", [(512, 1024, 512), (300, 520, 256), (130, 67, 512), (64, 256, 1024)])
def test_linear_i8_fuses_cast_and_bias(dtype, shape):
    """y = cast(dot) + cast(bias) from the fused entry point equals dot (float32) followed by the
    separate cast + bias kernel, which is the reference layer's arithmetic."""
    import ctypes as C
    Q, R, D = shape
    q, k = _inputs.fc1(Q=Q, R=R, D=D, seed=Q * 3 + R, dtype=torch.float32)
    qa, kb, _ = _prepare(q, k)
    g = torch.Generator().manual_seed(R)
    bias = (torch.randn(R, generator=g) * 0.5).to(DEV)
    out = H.dot_i8(qa["q8"], qa["scales"], kb["q8"], kb["scales"], o.scale_inv(2), capi.ENGINE_TCGEN05)
    code = {torch.float32: capi.DTYPE_F32, torch.float16: capi.DTYPE_F16, torch.bfloat16: capi.DTYPE_BF16}[dtype]
    chunks = D // 256
    L = capi.lib()
    for b in (bias, None):
        want = out.to(dtype) + b.to(dtype) if b is not None else out.to(dtype)
        if dtype == torch.float32 and b is not None:
            want = out + b
        y = torch.full((Q, R), float("nan"), dtype=dtype, device=DEV)
        rc = L.bsi_b200_linear_i8(capi.ptr(qa["q8"]), qa["q8"].shape[1], capi.ptr(qa["scales"]), chunks,
                                  capi.ptr(kb["q8"]), kb["q8"].shape[1], capi.ptr(kb["scales"]), capi.ptr(b), Q, R,
                                  chunks, C.c_float(float(o.scale_inv(2))), capi.ptr(y), R, code, capi.stream_ptr())
        capi.check(rc, "bsi_b200_linear_i8")
        assert torch.equal(y, want)
        y2 = torch.empty_like(y)
        capi.check(L.bsi_b200_cast_bias(capi.ptr(out), R, capi.ptr(b), Q, R, capi.ptr(y2), R, code, capi.stream_ptr()))
        assert torch.equal(y2, want)
    assert capi.device_status() == 0


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("Q,R,D,relu", [(300, 512, 1024, True), (64, 256, 256, False), (513, 768, 512, True)])
def test_linear_requant_equals_linear_then_pack(dtype, Q, R, D, relu):
    """The re-quantising epilogue stores the integers and chunk scales that the pack kernel derives from the
    layer-type output of the plain fused linear (cast + bias, optional ReLU)."""
    from bsipytorch_b200 import bsi_ops

    g = torch.Generator().manual_seed(Q + R + D)
    x = (torch.randn(Q, D, generator=g) * torch.where(torch.rand(Q, D, generator=g) < 0.01, 20.0, 1.0)).to(dtype).to(DEV)
    w = (torch.randn(R, D, generator=g) * 0.05).to(DEV)
    bias = torch.randn(R, generator=g).to(DEV)
    cap = bsi_ops.build_bsi_keys_cuda(w, 2, 0.5)[0]
    q8 = torch.empty(Q, D, dtype=torch.int8, device=DEV)
    sc = torch.empty(Q, D // 256, dtype=torch.float32, device=DEV)
    bsi_ops.pack_queries_into(x, q8, sc, 2)
    y = bsi_ops.linear_from_packed(q8, sc, cap, bias, 2, dtype, relu)
    want_q8 = torch.empty(Q, R, dtype=torch.int8, device=DEV)
    want_sc = torch.empty(Q, R // 256, dtype=torch.float32, device=DEV)
    bsi_ops.pack_queries_into(y, want_q8, want_sc, 2)
    # two destinations at once
    got_q8 = torch.full((2, Q, R), 99, dtype=torch.int8, device=DEV)
    got_sc = torch.full((2, Q, R // 256), -1.0, dtype=torch.float32, device=DEV)
    bsi_ops.linear_from_packed_requant(q8, sc, cap, bias, 2, dtype, relu, [got_q8[0].data_ptr(), got_q8[1].data_ptr()], R,
                                       [got_sc[0].data_ptr(), got_sc[1].data_ptr()], R // 256)
    # a column block of a wider matrix
    wide_q8 = torch.full((Q, 2 * R), 99, dtype=torch.int8, device=DEV)
    wide_sc = torch.full((Q, 2 * (R // 256)), -1.0, dtype=torch.float32, device=DEV)
    bsi_ops.linear_from_packed_requant(q8, sc, cap, bias, 2, dtype, relu, [wide_q8.data_ptr() + R], 2 * R,
                                       [wide_sc.data_ptr() + 4 * (R // 256)], 2 * (R // 256))
    assert bsi_ops.device_status() == 0
    for i in range(2):
        assert torch.equal(got_sc[i], want_sc)
        assert torch.equal(got_q8[i], want_q8)
    assert torch.equal(wide_q8[:, R:], want_q8) and torch.equal(wide_sc[:, R // 256:], want_sc)
    assert (wide_q8[:, :R] == 99).all() and (wide_sc[:, : R // 256] == -1.0).all()
    assert (want_q8 != 0).any()


def test_linear_requant_reports_values_it_cannot_express():
    from bsipytorch_b200 import bsi_ops

    x = torch.full((32, 256), 60000.0, dtype=torch.float16, device=DEV)        # the dot overflows float16: inf
    w = torch.full((256, 256), 0.3, device=DEV)
    cap = bsi_ops.build_bsi_keys_cuda(w, 2, 0.5)[0]
    q8 = torch.empty(32, 256, dtype=torch.int8, device=DEV)
    sc = torch.empty(32, 1, dtype=torch.float32, device=DEV)
    bsi_ops.pack_queries_into(x, q8, sc, 2)
    out_q8 = torch.full((32, 256), 99, dtype=torch.int8, device=DEV)
    out_sc = torch.full((32, 1), -1.0, dtype=torch.float32, device=DEV)
    bsi_ops.linear_from_packed_requant(q8, sc, cap, None, 2, torch.float16, False, [out_q8.data_ptr()], 256,
                                       [out_sc.data_ptr()], 1)
    assert bsi_ops.device_status() == 48
    assert bsi_ops.device_status() == 0          # reading clears it
    assert not out_q8.any()


def _key_bounds(k8):
    """[3, R] float32: sum of |k| over each key row, the largest such sum over one 256-element chunk, sum of k^2."""
    k32 = k8.to(torch.int32)
    per_chunk = k32.abs().view(k8.shape[0], -1, 256).sum(2)
    return torch.stack([per_chunk.sum(1), per_chunk.amax(1), (k32 * k32).sum(1)]).to(torch.float32).contiguous()


@pytest.mark.parametrize("engine", [3256, 3224, 3128, 3064])
def test_exact_integer_route_gives_the_float_chain_bits(engine):
    """With the row sums of |k| registered for a key image, tiles whose prefix sums provably stay below 2^24
    accumulate in int32; tiles that fail the bound keep the float32 chain. Same bits either way, and the same as
    without the registration and as the checker."""
    L = capi.lib()
    Q, R, D = 600, 1100, 1024
    g = torch.Generator().manual_seed(engine)
    q = torch.randn(Q, D, generator=g)
    q[256:512] *= 3.0e4                      # tile rows 256..511: chunk shifts around 15, the bound fails
    q[5, 300] = 900.0                        # a lone outlier in a tile that passes
    k = torch.randn(R, D, generator=g) * 0.02
    k[700] = 0.0                             # an all-zero key row
    qa, kb, _ = _prepare(q, k)
    want, _ = _oracle(q, k)
    capi.exact_int_tiles()
    plain = H.dot_i8(qa["q8"], qa["scales"], kb["q8"], kb["scales"], o.scale_inv(2), engine)
    assert capi.exact_int_tiles() == 0
    abs_sum = _key_bounds(kb["q8"])
    capi.check(L.bsi_b200_register_key_bounds(capi.ptr(kb["q8"]), capi.ptr(abs_sum), R, 64))
    try:
        got = H.dot_i8(qa["q8"], qa["scales"], kb["q8"], kb["scales"], o.scale_inv(2), engine)
        n_int = capi.exact_int_tiles()
        bn = engine - 3000
        tiles_n = -(-R // bn)
        # 8 epilogue warps per tile pair... every (warp, tile) with rows outside 256..511 passes, the others fail
        assert 0 < n_int < 3 * tiles_n * 16
        # the debug dump of the per-chunk integers is unaffected
        got_dbg, iacc = H.dot_i8(qa["q8"], qa["scales"], kb["q8"], kb["scales"], o.scale_inv(2), engine, want_iacc=True)
        assert torch.equal(got_dbg, got)
        capi.exact_int_tiles()
    finally:
        capi.check(L.bsi_b200_unregister_key_bounds(capi.ptr(kb["q8"])))
    _assert_bits(plain, want)
    _assert_bits(got, want)
    H.dot_i8(qa["q8"], qa["scales"], kb["q8"], kb["scales"], o.scale_inv(2), engine)
    assert capi.exact_int_tiles() == 0       # unregistered again
    assert capi.device_status() == 0


def test_exact_integer_route_row_scale_and_16bit_outputs():
    """The same route under a single scale per query row and in the layer epilogues (cast + bias, re-quantisation)."""
    import ctypes as C
    L = capi.lib()
    Q, R, D = 512, 768, 512
    q, k = _inputs.c1(Q=Q, R=R, D=D, seed=5)
    qa, kb, _ = _prepare(q, k, chunk_mode=False)
    want, _ = _oracle(q, k, chunk_mode=False)
    abs_sum = _key_bounds(kb["q8"])
    plain = H.dot_i8(qa["q8"], qa["scales"], kb["q8"], kb["scales"], o.scale_inv(2), 3256)
    qc, _, _ = _prepare(q, k)
    chunks = D // 256
    bias = torch.linspace(-1, 1, R, device=DEV)

    def linear(code_dtype):
        y = torch.empty(Q, R, dtype=code_dtype, device=DEV)
        code = capi.DTYPE_F16 if code_dtype == torch.float16 else capi.DTYPE_BF16
        capi.check(L.bsi_b200_linear_i8_act(capi.ptr(qc["q8"]), qc["q8"].shape[1], capi.ptr(qc["scales"]), chunks,
                                            capi.ptr(kb["q8"]), kb["q8"].shape[1], capi.ptr(kb["scales"]), capi.ptr(bias),
                                            Q, R, chunks, C.c_float(float(o.scale_inv(2))), capi.ptr(y), R, code, 1,
                                            capi.stream_ptr()))
        return y

    y_plain = [linear(torch.float16), linear(torch.bfloat16)]
    capi.exact_int_tiles()
    capi.check(L.bsi_b200_register_key_bounds(capi.ptr(kb["q8"]), capi.ptr(abs_sum), R, 64))
    try:
        got = H.dot_i8(qa["q8"], qa["scales"], kb["q8"], kb["scales"], o.scale_inv(2), 3256)
        assert capi.exact_int_tiles() > 0
        y_int = [linear(torch.float16), linear(torch.bfloat16)]
        assert capi.exact_int_tiles() > 0
    finally:
        capi.check(L.bsi_b200_unregister_key_bounds(capi.ptr(kb["q8"])))
    _assert_bits(plain, want)
    _assert_bits(got, want)
    for a, b in zip(y_plain, y_int):
        assert torch.equal(a, b)


def test_exact_integer_route_by_the_norm_bound():
    """FC1-like activations (1 % outliers of 20 sigma) sit at chunk shifts around 7, where the two cheap bounds fail;
    with the packer's chunk sums of squares registered for the query image the Cauchy-Schwarz bound holds and the
    integer route runs -- same bits. The sums themselves are checked against the packed integers."""
    L = capi.lib()
    Q, R, D = 512, 1024, 2048
    q, k = _inputs.fc1(Q=Q, R=R, D=D)
    kb = H.quantize_pack(k.to(DEV), 2, 6, False)
    chunks = D // 256
    x = q.to(DEV)
    words = torch.zeros(Q, 7, D // 64, dtype=torch.int64, device=DEV)
    scales = torch.ones(Q, chunks, dtype=torch.float32, device=DEV)
    q8 = torch.zeros(Q, D, dtype=torch.int8, device=DEV)
    norms = torch.full((Q, chunks), -1.0, dtype=torch.float32, device=DEV)
    import ctypes as C
    capi.check(L.bsi_b200_quantize_pack_norms(capi.ptr(x), capi.DTYPE_F16, Q, D, D, 2, 7, 1, C.c_float(0.0), capi.ptr(words),
                                              capi.ptr(scales), None, capi.ptr(q8), D, capi.ptr(norms), capi.stream_ptr()))
    want_n = (q8.view(Q, chunks, 256).to(torch.float64) ** 2).sum(2) * scales.to(torch.float64) ** 2
    assert torch.equal(norms.to(torch.float64), want_n)
    want, _ = _oracle(q, k)
    bounds = _key_bounds(kb["q8"])
    capi.exact_int_tiles()
    capi.check(L.bsi_b200_register_key_bounds(capi.ptr(kb["q8"]), capi.ptr(bounds), R, 64))
    try:
        got_cheap = H.dot_i8(q8, scales, kb["q8"], kb["scales"], o.scale_inv(2), 3256)
        n_cheap = capi.exact_int_tiles()
        capi.check(L.bsi_b200_register_query_bounds(capi.ptr(q8), capi.ptr(norms), chunks))
        got = H.dot_i8(q8, scales, kb["q8"], kb["scales"], o.scale_inv(2), 3256)
        n_norm = capi.exact_int_tiles()
    finally:
        capi.check(L.bsi_b200_unregister_key_bounds(capi.ptr(kb["q8"])))
        capi.check(L.bsi_b200_unregister_query_bounds(capi.ptr(q8)))
    _assert_bits(got_cheap, want)
    _assert_bits(got, want)
    tiles = 2 * 4 * 16                           # 2 x 4 tiles of 256 x 256, 16 epilogue warps per tile pair
    assert n_cheap < tiles and n_norm == tiles   # the norm bound covers every warp of every tile
    # a chunk that took the 64-bit fallback reports infinity, which fails the test safely
    x2 = x.clone()
    x2[3, 5] = float("inf")
    capi.check(L.bsi_b200_quantize_pack_norms(capi.ptr(x2), capi.DTYPE_F16, Q, D, D, 2, 7, 1, C.c_float(0.0), capi.ptr(words),
                                              capi.ptr(scales), None, capi.ptr(q8), D, capi.ptr(norms), capi.stream_ptr()))
    assert torch.isinf(norms[3, 0]) and torch.isfinite(norms[3, 1:]).all() and torch.isfinite(norms[4]).all()
