"""The `bsi_ops` entry points the reference's microbenchmark and OPT layer call.

Written the way the reference's own scripts use the module (benchmark_dot_kernel_micro.py,
verify_tc_dot_correctness.py, verify_accuracy_bsi.py), then checked against the CPU checker.
"""
import os

import numpy as np
import pytest
import torch

import _capi_helpers as H
import _inputs
import bsipytorch_b200
from bsipytorch_b200 import capi
from bsipytorch_b200.linear import BSIQuantizedLinear, quantize_model_bsi
from oracle import oracle as o

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def bsi_ops():
    return bsipytorch_b200.install_as_bsi_ops()


def _bits(t):
    return t.detach().cpu().numpy().view(np.uint32)


def test_packed_entry_matches_oracle_config1(bsi_ops):
    q, k = _inputs.c1()
    keys_cap, mem, num_keys, d, W = bsi_ops.build_bsi_keys_cuda(k, 2, 0.5)          # CPU tensor, as the layer passes it
    assert (num_keys, d, W) == (256, 2048, 32) and mem == 256 * 6 * 32 * 8
    qcap = bsi_ops.build_bsi_queries_cuda_batch_packed(q.to(DEV), 2, 0.5)
    out, ns_total, ns_q, ns_s = bsi_ops.batch_dot_product_multiquery_cuda_batch_caps(qcap, keys_cap)
    assert out.shape == (64, 256) and out.dtype == torch.float32 and out.is_cuda
    assert (ns_total, ns_q, ns_s) == (0, 0.0, 0.0)          # timings are zero unless BSI_PROFILE=1
    want, want_i = o.fixed_dot(q.numpy(), k.numpy(), want_iacc=True)
    np.testing.assert_array_equal(_bits(out), want.view(np.uint32))
    out2, iacc = bsi_ops.debug_dot_iacc(qcap, keys_cap)
    np.testing.assert_array_equal(iacc.cpu().numpy(), want_i)
    # and within the documented tolerance of the float product it approximates
    assert float((out.cpu() - q @ k.T).abs().max()) < 2.0


def test_capsule_contents_match_oracle(bsi_ops):
    q, k = _inputs.fc1(Q=32, R=64, D=1024)
    keys_cap, *_ = bsi_ops.build_bsi_keys_cuda(k.to(DEV), 2, 0.5)
    kt = bsi_ops.debug_keys_tensors(keys_cap)
    kb = o.quantize_pack(k.numpy(), 2, 6, False)
    np.testing.assert_array_equal(H.as_u64(kt["words"]), kb["words"])
    np.testing.assert_array_equal(kt["slice_weights"].cpu().numpy(), o.slice_weights(6, kb["scales"]))
    qcap = bsi_ops.build_bsi_queries_cuda_batch_packed(q.to(DEV), 2)
    qt = bsi_ops.debug_query_batch_tensors(qcap)
    qa = o.quantize_pack(q.float().numpy(), 2, 7, True)
    np.testing.assert_array_equal(H.as_u64(qt["words"]), qa["words"])
    np.testing.assert_array_equal(qt["scales"].cpu().numpy(), qa["scales"])
    np.testing.assert_array_equal(qt["slice_weights"].cpu().numpy(), np.tile(o.slice_weights(7), (32, 1)))


def test_list_entry_microbenchmark_flow(bsi_ops):
    # benchmark_dot_kernel_micro.py:31-57
    torch.manual_seed(123)
    K = torch.randn(256, 2048, dtype=torch.float32, device="cpu")
    keys_cap, _, _, _, _ = bsi_ops.build_bsi_keys_cuda(K, 2, 0.5)
    Q = torch.randn(128, 2048, dtype=torch.float32, device=DEV)
    query_caps = bsi_ops.build_bsi_queries_cuda_batch(Q, 2, 0.5)
    assert isinstance(query_caps, list) and len(query_caps) == 128
    assert dict(bsi_ops.bsi_keys_cuda_stats(keys_cap)) == {
        "W": 32, "d": 2048, "num_keys": 256, "decimals": 2, "threshold": 0.5, "Sb_counts": {6: 256}}
    assert dict(bsi_ops.bsi_query_caps_stats(query_caps)) == {"Q": 128, "W": 32, "S_counts": {7: 128}}
    out, *_ = bsi_ops.batch_dot_product_multiquery_cuda_caps(query_caps, keys_cap)
    want = o.fixed_dot(Q.cpu().numpy(), K.numpy())
    np.testing.assert_array_equal(_bits(out), want.view(np.uint32))
    # a permuted sub-list is gathered row by row
    idx = [5, 3, 100, 7]
    out_sub, *_ = bsi_ops.batch_dot_product_multiquery_cuda_caps([query_caps[i] for i in idx], keys_cap)
    assert torch.equal(out_sub, out[idx])
    # packed entry gives the same bits (verify_tc_dot_correctness.py compares two paths of one op)
    out_p, *_ = bsi_ops.batch_dot_product_multiquery_cuda_batch_caps(
        bsi_ops.build_bsi_queries_cuda_batch_packed(Q, 2, 0.5), keys_cap)
    assert torch.allclose(out, out_p, rtol=1e-2, atol=5e-3) and torch.equal(out, out_p)


def test_engines_agree_through_the_module(bsi_ops, monkeypatch):
    q, k = _inputs.fc1(Q=96, R=160, D=1024)
    keys_cap, *_ = bsi_ops.build_bsi_keys_cuda(k, 2, 0.5)
    qcap = bsi_ops.build_bsi_queries_cuda_batch_packed(q.to(DEV), 2, 0.5)
    outs = {}
    for eng in ["tcgen05", "simt", "bmma", "tcgen05:64", "tcgen05:128"]:
        monkeypatch.setenv("BSI_B200_ENGINE", eng)
        outs[eng] = bsi_ops.batch_dot_product_multiquery_cuda_batch_caps(qcap, keys_cap)[0]
    for eng, t in outs.items():
        assert torch.equal(t, outs["tcgen05"]), eng


def test_profile_env_returns_kernel_times(bsi_ops, monkeypatch):
    monkeypatch.setenv("BSI_PROFILE", "1")
    q, k = _inputs.c1()
    keys_cap, *_ = bsi_ops.build_bsi_keys_cuda(k, 2, 0.5)
    bsi_ops.reset_last_query_build_profile_cuda()
    assert bsi_ops.get_last_query_build_profile_cuda() == (0, 0, 0)
    qcap = bsi_ops.build_bsi_queries_cuda_batch_packed(q.to(DEV), 2, 0.5)
    quant_ns, pack_ns, total_ns = bsi_ops.get_last_query_build_profile_cuda()
    assert total_ns > 0 and total_ns == quant_ns + pack_ns
    out, ns_total, ns_q, ns_s = bsi_ops.batch_dot_product_multiquery_cuda_batch_caps(qcap, keys_cap)
    assert ns_total > 0 and ns_q == pytest.approx(ns_total / 64) and ns_s == pytest.approx(ns_total / (64 * 256))


def test_error_behaviour(bsi_ops):
    q, k = _inputs.c1(Q=32, R=64, D=512)
    keys_cap, *_ = bsi_ops.build_bsi_keys_cuda(k, 2, 0.5)
    with pytest.raises(RuntimeError, match="Decimal mismatch between queries and keys"):
        bsi_ops.batch_dot_product_multiquery_cuda_batch_caps(
            bsi_ops.build_bsi_queries_cuda_batch_packed(q.to(DEV), 3, 0.5), keys_cap)
    with pytest.raises(RuntimeError, match="Word count mismatch"):
        bsi_ops.batch_dot_product_multiquery_cuda_batch_caps(
            bsi_ops.build_bsi_queries_cuda_batch_packed(q[:, :256].contiguous().to(DEV), 2, 0.5), keys_cap)
    with pytest.raises(RuntimeError, match="2D"):
        bsi_ops.build_bsi_keys_cuda(k[0], 2, 0.5)
    with pytest.raises(RuntimeError, match="2D"):
        bsi_ops.build_bsi_queries_cuda_batch_packed(q[0].to(DEV), 2, 0.5)
    with pytest.raises(RuntimeError, match="capsule"):
        bsi_ops.batch_dot_product_multiquery_cuda_batch_caps(keys_cap, keys_cap)


def test_row_scale_mode_when_words_not_multiple_of_four(bsi_ops):
    # D = 320 -> W = 5: the reference switches the queries to one scale per row (bsi_vector_cuda.cpp:985)
    q, k = _inputs.c1(Q=40, R=72, D=320)
    keys_cap, *_ = bsi_ops.build_bsi_keys_cuda(k, 2, 0.5)
    qcap = bsi_ops.build_bsi_queries_cuda_batch_packed(q.to(DEV), 2, 0.5)
    qt = bsi_ops.debug_query_batch_tensors(qcap)
    assert qt["chunk_mode"] is False and qt["scales"].shape == (40,)
    out, *_ = bsi_ops.batch_dot_product_multiquery_cuda_batch_caps(qcap, keys_cap)
    want = o.fixed_dot(q.numpy(), k.numpy())
    np.testing.assert_array_equal(_bits(out), want.view(np.uint32))


def test_single_query_and_hybrid_builders(bsi_ops):
    g = torch.Generator().manual_seed(7)
    v = torch.relu(torch.randn(4096, generator=g)).to(DEV)
    cap, mem, S, W = bsi_ops.build_bsi_query_cuda(v, 2, 0.5)
    assert (S, W) == (7, 64) and mem == 7 * 64 * 8
    hcap, hmem, hS, hW = bsi_ops.build_bsi_query_cuda_hybrid(v, 2, 0.5)
    a, b = bsi_ops.debug_query_tensors(cap), bsi_ops.debug_query_tensors(hcap)
    assert torch.equal(a["words"], b["words"])              # EWAH encode -> decode is lossless
    assert a["twos_complement"] is False
    want = o.quantize_pack(v.cpu().numpy()[None], 2, 7, False)
    np.testing.assert_array_equal(H.as_u64(a["words"]), want["words"][0])
    np.testing.assert_array_equal(a["slice_weights"].cpu().numpy(), o.slice_weights(7, want["scales"])[0])
    flags = o.compress_flags(o.slice_popcount(want["words"][0]), 64, 0.5)
    stream, off, length = o.ewah_encode(want["words"][0], flags)
    assert hmem == 8 * len(stream) + 7 * 64 * 8 and length[6] == 1
    k = torch.randn(8, 4096, generator=g) * 0.02
    keys_cap, *_ = bsi_ops.build_bsi_keys_cuda(k, 2, 0.5)
    out, *_ = bsi_ops.batch_dot_product_multiquery_cuda_caps([cap], keys_cap)
    out_h, *_ = bsi_ops.batch_dot_product_multiquery_cuda_caps([hcap], keys_cap)
    assert torch.equal(out, out_h)
    neg, *_ = bsi_ops.build_bsi_query_cuda(-v, 2, 0.5)
    assert bsi_ops.debug_query_tensors(neg)["twos_complement"] is True


def test_ewah_module_helpers(bsi_ops):
    q, _ = _inputs.fc2(Q=8, R=8)
    qcap = bsi_ops.build_bsi_queries_cuda_batch_packed(q.to(DEV), 2, 0.5)
    words = bsi_ops.debug_query_batch_tensors(qcap)["words"].view(8 * 7, 128)
    stream, off, length, flags = bsi_ops.ewah_encode_words(words, 0.5)
    wn = H.as_u64(words)
    f = o.compress_flags(o.slice_popcount(wn), 128, 0.5)
    s, of, ln = o.ewah_encode(wn, f)
    np.testing.assert_array_equal(H.as_u64(stream), s)
    np.testing.assert_array_equal(length.cpu().numpy(), ln)
    assert torch.equal(bsi_ops.ewah_decode_words(stream, off, length, 128), words)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_bsi_quantized_linear_matches_reference_arithmetic(bsi_ops, dtype):
    # verify_accuracy_bsi.py:118-215: y = dot(x, W).to(dtype) + bias.to(dtype)
    torch.manual_seed(0)
    lin = torch.nn.Linear(768, 3072, bias=True)
    lin.weight.data.normal_(0, 0.02)
    lin.bias.data.normal_(0, 0.02)
    x = torch.randn(2, 24, 768).to(dtype)
    layer = BSIQuantizedLinear(lin.to(DEV), decimalPlaces=2, compress_threshold=0.5)
    y = layer(x.to(DEV))
    assert y.shape == (2, 24, 3072) and y.dtype == dtype
    want = torch.from_numpy(o.fixed_dot(x.view(-1, 768).float().numpy(), lin.weight.detach().cpu().numpy()))
    want = want.to(dtype) + lin.bias.detach().cpu().to(dtype)
    assert torch.equal(y.view(-1, 3072).cpu(), want)
    layer.fused = False
    y2 = layer(x.to(DEV))
    assert torch.equal(y, y2)
    assert layer.dot_calls == 2 and layer.dot_output_elements_total == 2 * 48 * 3072
    assert layer.weight_bsi_memory_bytes == 3072 * 6 * 12 * 8


def test_quantize_model_bsi_walk(bsi_ops):
    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.q_proj = torch.nn.Linear(256, 256)
            self.fc1 = torch.nn.Linear(256, 512)
            self.fc2 = torch.nn.Linear(512, 256)
            self.lm_head = torch.nn.Linear(256, 100, bias=False)

        def forward(self, x):
            return self.lm_head(self.fc2(torch.relu(self.fc1(self.q_proj(x)))))

    torch.manual_seed(1)
    m = Block().to(DEV)
    x = torch.randn(4, 256, device=DEV)
    dense = m(x)
    quantize_model_bsi(m, decimalPlaces=2, scope="mlp", compress_threshold=0.5, verbose=False)
    assert isinstance(m.fc1, BSIQuantizedLinear) and isinstance(m.q_proj, torch.nn.Linear)
    quantize_model_bsi(m, decimalPlaces=2, scope="all", compress_threshold=0.5, verbose=False)
    assert isinstance(m.q_proj, BSIQuantizedLinear) and isinstance(m.lm_head, torch.nn.Linear)
    y = m(x)
    assert y.shape == dense.shape and torch.isfinite(y).all()
    assert float((y - dense).abs().max()) < 0.5
    assert capi.device_status() == 0


def test_keyset_save_load_round_trip(bsi_ops, tmp_path):
    """save_keyset / load_keyset: the stored form (row scales + EWAH / verbatim slice streams) gives back the same
    slices, int8 image and scales, and the same dot, without the dense weights."""
    g = torch.Generator().manual_seed(77)
    k = torch.randn(300, 1000, generator=g) * 0.02
    k[5] = 0.0                                  # an all-zero row: every slice is one run
    k[6, :512] = 0.0                            # half-empty row
    k[7] = 0.31                                 # constant row: slices are all-ones / all-zeros runs
    q = torch.randn(64, 1000, generator=g).to(DEV)
    for thr in (0.5, 0.2):
        cap, mem, R, d, W = bsi_ops.build_bsi_keys_cuda(k, 2, thr)
        out_dir = str(tmp_path / f"keys_{thr}")
        assert bsi_ops.save_keyset(cap, out_dir) is None
        path = os.path.join(out_dir, "keyset.bsik")
        mem2, disk = bsi_ops.keyset_size_on_disk(cap)
        assert mem2 == mem and disk == os.path.getsize(path)
        # a verbatim slice costs one marker word more than in memory; the file adds one length per slice, one scale
        # per row and the header
        assert disk <= mem + R * 6 * 12 + R * 4 + 64
        cap2, mem3, R2, d2, W2 = bsi_ops.load_keyset(out_dir)
        assert (mem3, R2, d2, W2) == (mem, R, d, W)
        a, b = bsi_ops.debug_keys_tensors(cap), bsi_ops.debug_keys_tensors(cap2)
        for name in ("words", "q8", "scales", "slice_weights"):
            assert torch.equal(a[name], b[name]), name
        assert bsi_ops.bsi_keys_cuda_stats(cap2)["decimals"] == 2
        qcap = bsi_ops.build_bsi_queries_cuda_batch_packed(q, 2, thr)
        want, *_ = bsi_ops.batch_dot_product_multiquery_cuda_batch_caps(qcap, cap)
        got, *_ = bsi_ops.batch_dot_product_multiquery_cuda_batch_caps(qcap, cap2)
        assert torch.equal(got, want)
        assert bsi_ops.load_keyset(path)[2] == R     # the file itself is accepted too
    # a damaged file is refused
    raw = bytearray(open(path, "rb").read())
    raw[-3] ^= 0x40
    bad = str(tmp_path / "bad.bsik")
    open(bad, "wb").write(bytes(raw))
    with pytest.raises(RuntimeError, match="checksum"):
        bsi_ops.load_keyset(bad)
    open(bad, "wb").write(bytes(raw[:100]))
    with pytest.raises(RuntimeError):
        bsi_ops.load_keyset(bad)


def test_outlier_clipping_env(bsi_ops, monkeypatch):
    """BSI_FIXED_CLIP_K > 0 (bsi_vector_cuda.cpp:295-307): builders and dots follow the checker's clipped shifts; the
    fused additions, which have no clipping variant, refuse to run."""
    monkeypatch.setenv("BSI_FIXED_CLIP_K", "3.0")
    q, k = _inputs.fc1(Q=40, R=96, D=1024)
    keys_cap, *_ = bsi_ops.build_bsi_keys_cuda(k, 2, 0.5)
    qcap = bsi_ops.build_bsi_queries_cuda_batch_packed(q.to(DEV), 2, 0.5)
    qt = bsi_ops.debug_query_batch_tensors(qcap)
    qa = o.quantize_pack(q.float().numpy(), 2, 7, True, 3.0)
    np.testing.assert_array_equal(H.as_u64(qt["words"]), qa["words"])
    np.testing.assert_array_equal(qt["scales"].cpu().numpy(), qa["scales"])
    assert not np.array_equal(qa["scales"], o.quantize_pack(q.float().numpy(), 2, 7, True)["scales"])
    out, *_ = bsi_ops.batch_dot_product_multiquery_cuda_batch_caps(qcap, keys_cap)
    want = o.fixed_dot(q.float().numpy(), k.numpy(), clip_k=3.0)
    np.testing.assert_array_equal(_bits(out), want.view(np.uint32))
    out_l, *_ = bsi_ops.batch_dot_product_multiquery_cuda_caps(bsi_ops.build_bsi_queries_cuda_batch(q.to(DEV), 2, 0.5), keys_cap)
    assert torch.equal(out_l, out)
    y = bsi_ops.bsi_linear_forward(q.to(DEV), keys_cap, None, 2)          # packs through the same builder
    assert torch.equal(y, out.to(y.dtype))
    q8 = torch.empty(40, 1024, dtype=torch.int8, device=DEV)
    sc = torch.empty(40, 4, dtype=torch.float32, device=DEV)
    with pytest.raises(RuntimeError, match="BSI_FIXED_CLIP_K"):
        bsi_ops.pack_queries_into(q.to(DEV), q8, sc, 2)
