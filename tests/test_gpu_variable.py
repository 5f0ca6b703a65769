"""Variable-slice mode (the reference's mode when no BSI_FIXED_BITS* variable is set): the decimal integers are
sliced without a shift, the slice count follows from the data, the dot is the exact integer dot.

Checked against the CPU restatement (oracle.variable_*) and, where they were built, against the reference's own
kernels: its int64 rounding + ballot packer for the slices and its generic float-weight dot kernels (tensor-core
and plain) for the outputs."""
import ctypes as C

import numpy as np
import pytest
import torch

import _capi_helpers as H
import _inputs
import bsipytorch_b200
from bsipytorch_b200 import capi
from oracle import oracle as o

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture()
def ops(monkeypatch):
    monkeypatch.setenv("BSI_FIXED_BITS_QUERIES", "0")
    monkeypatch.setenv("BSI_FIXED_BITS_KEYS", "0")
    return bsipytorch_b200.install_as_bsi_ops()


def _bits(t):
    return t.detach().cpu().numpy().view(np.uint32)


def test_pack_plain_and_absmax_match_oracle():
    L = capi.lib()
    g = torch.Generator().manual_seed(4)
    for dtype, rows, D, scale in [(torch.float32, 37, 1000, 1.0), (torch.float16, 64, 2048, 30.0), (torch.bfloat16, 5, 70, 0.02)]:
        x = (torch.randn(rows, D, generator=g) * scale).to(dtype)
        x[1] = x[1].abs()                                          # a row without negatives
        want = o.variable_pack(x.float().numpy(), 2)
        xd = x.to(DEV)
        amax = torch.zeros(rows, dtype=torch.int64, device=DEV)
        neg = torch.zeros(rows, dtype=torch.int32, device=DEV)
        code = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}[dtype]
        capi.check(L.bsi_b200_decimal_absmax(capi.ptr(xd), code, rows, D, D, 2, capi.ptr(amax), capi.ptr(neg), capi.stream_ptr()))
        np.testing.assert_array_equal(amax.cpu().numpy(), np.abs(want["ints"]).max(axis=1))
        np.testing.assert_array_equal(neg.cpu().numpy() != 0, want["negative"])
        S, W, chunks = want["S"], (D + 63) // 64, (D + 255) // 256
        words = torch.zeros(rows, S, W, dtype=torch.int64, device=DEV)
        lo = torch.full((rows, chunks * 256), 99, dtype=torch.int8, device=DEV)
        hi = torch.full((rows, chunks * 256), 99, dtype=torch.int8, device=DEV)
        capi.check(L.bsi_b200_pack_plain(capi.ptr(xd), code, rows, D, D, 2, S, capi.ptr(words), capi.ptr(lo), capi.ptr(hi),
                                         chunks * 256, capi.stream_ptr()))
        np.testing.assert_array_equal(H.as_u64(words), want["words"])
        v = hi.cpu().numpy().astype(np.int64) * 128 + lo.cpu().numpy().astype(np.int64)
        np.testing.assert_array_equal(v[:, :D], want["ints"])
        assert not v[:, D:].any() and int(lo.min()) >= 0


def test_list_entry_on_config1_matches_oracle_and_reference_kernels(ops):
    """C1 (Q=64, R=256, D=2048, float32) through the entry points the reference's microbenchmark calls."""
    q, k = _inputs.c1()
    keys_cap, mem, num_keys, d, W = ops.build_bsi_keys_cuda(k, 2, 0.5)
    qa, kb = o.variable_pack(q.numpy(), 2), o.variable_pack(k.numpy(), 2, per_row=True)
    assert mem == int(kb["row_slices"].sum()) * W * 8
    caps = ops.build_bsi_queries_cuda_batch(q.to(DEV), 2, 0.5)
    out, *_ = ops.batch_dot_product_multiquery_cuda_caps(caps, keys_cap)
    want = o.variable_dot(q.numpy(), k.numpy(), 2)
    np.testing.assert_array_equal(_bits(out), want.view(np.uint32))
    kt, qt = ops.debug_keys_tensors(keys_cap), ops.debug_query_tensors(caps[3])
    np.testing.assert_array_equal(H.as_u64(kt["words"]), kb["words"])
    np.testing.assert_array_equal(kt["slice_weights"].cpu().numpy(), kb["weights"])
    np.testing.assert_array_equal(H.as_u64(qt["words"]), qa["words"][3])
    np.testing.assert_array_equal(qt["slice_weights"].cpu().numpy(), qa["weights"][3])
    stats = ops.bsi_keys_cuda_stats(keys_cap)
    hist = {int(s): int((kb["row_slices"] == s).sum()) for s in np.unique(kb["row_slices"])}
    assert {int(a): int(b) for a, b in stats["Sb_counts"].items()} == hist
    assert dict(ops.bsi_query_caps_stats(caps)["S_counts"]) == {qa["S"]: 64}
    # the packed entry and the dp4a engine give the same bits
    qcap = ops.build_bsi_queries_cuda_batch_packed(q.to(DEV), 2, 0.5)
    out2, *_ = ops.batch_dot_product_multiquery_cuda_batch_caps(qcap, keys_cap)
    assert torch.equal(out, out2)
    from oracle import ref_gpu
    if ref_gpu.available():
        rq, _ = ref_gpu.pack_plain(q.to(DEV), 2, qa["S"])
        rk, _ = ref_gpu.pack_plain(k.to(DEV), 2, kb["S"])
        np.testing.assert_array_equal(H.as_u64(rq), qa["words"])
        np.testing.assert_array_equal(H.as_u64(rk), kb["words"])
        Aw, Bw = torch.from_numpy(qa["weights"]).to(DEV), torch.from_numpy(kb["weights"]).to(DEV)
        for tc in (True, False):
            ref = ref_gpu.dot_generic(rq, Aw, rk, Bw, o.scale_inv(2), tensor_core=tc)
            assert torch.equal(out, ref), tc
    assert capi.device_status() == 0


def test_two_digit_queries_and_mixed_modes(ops, monkeypatch):
    g = torch.Generator().manual_seed(9)
    q = torch.randn(96, 1024, generator=g) * 8.0                    # |v| up to a few thousand: two 8-bit digits
    q[0, 0], q[1, 1] = 163.83, -163.83                              # the largest values the two digits hold
    k = torch.randn(200, 1024, generator=g) * 0.02
    keys_cap, *_ = ops.build_bsi_keys_cuda(k, 2, 0.5)
    qcap = ops.build_bsi_queries_cuda_batch_packed(q.to(DEV), 2, 0.5)
    assert ops.debug_query_batch_tensors(qcap)["S"] == 16
    out, *_ = ops.batch_dot_product_multiquery_cuda_batch_caps(qcap, keys_cap)
    np.testing.assert_array_equal(_bits(out), o.variable_dot(q.numpy(), k.numpy(), 2).view(np.uint32))
    # variable queries against fixed 6-bit keys: (integer dot * 2^shift_r) * scale_inv
    monkeypatch.setenv("BSI_FIXED_BITS_KEYS", "6")
    fixed_keys, *_ = ops.build_bsi_keys_cuda(k, 2, 0.5)
    out_f, *_ = ops.batch_dot_product_multiquery_cuda_batch_caps(qcap, fixed_keys)
    kb = o.quantize_pack(k.numpy(), 2, 6, False)
    exact = o.decimal_ints(q.numpy(), 2) @ kb["qvals"].astype(np.int64).T
    want = (exact.astype(np.float32) * kb["scales"][None, :]) * o.scale_inv(2)
    np.testing.assert_array_equal(_bits(out_f), want.view(np.uint32))
    # fixed 7-bit chunk-scale queries against variable keys: the fixed-bit recurrence with unit key scales
    monkeypatch.setenv("BSI_FIXED_BITS_QUERIES", "7")
    q7 = ops.build_bsi_queries_cuda_batch_packed(q.to(DEV), 2, 0.5)
    out_v, *_ = ops.batch_dot_product_multiquery_cuda_batch_caps(q7, keys_cap)
    qa = o.quantize_pack(q.numpy(), 2, 7, True)
    kv = o.decimal_ints(k.numpy(), 2).astype(np.int8)
    want = o.dot_i8(o.pad_i8(qa["qvals"], 4), qa["scales"], o.pad_i8(kv, 4), np.ones(200, np.float32), o.scale_inv(2))
    np.testing.assert_array_equal(_bits(out_v), want.view(np.uint32))
    assert capi.device_status() == 0


def test_variable_limits_layer_and_keyset_file(ops, tmp_path):
    g = torch.Generator().manual_seed(2)
    with pytest.raises(RuntimeError, match="queries beyond 16383"):
        ops.build_bsi_queries_cuda_batch_packed(torch.full((2, 256), 200.0, device=DEV), 2, 0.5)
    with pytest.raises(RuntimeError, match="keys beyond 127"):
        ops.build_bsi_keys_cuda(torch.full((2, 256), 1.5), 2, 0.5)
    # an all-zero batch has two slices (bsi_vector_cuda.cpp:753)
    z = ops.build_bsi_queries_cuda_batch_packed(torch.zeros(3, 256, device=DEV), 2, 0.5)
    assert ops.debug_query_batch_tensors(z)["S"] == 2
    # the layer: y = dot.to(dtype) + bias.to(dtype)
    from bsipytorch_b200.linear import BSIQuantizedLinear
    lin = torch.nn.Linear(512, 384).to(DEV)
    lin.weight.data.normal_(0, 0.02, generator=None)
    x = torch.randn(4, 9, 512, generator=g).to(DEV)
    layer = BSIQuantizedLinear(lin, decimalPlaces=2, compress_threshold=0.5)
    y = layer(x)
    want = torch.from_numpy(o.variable_dot(x.view(-1, 512).cpu().numpy(), lin.weight.detach().cpu().numpy(), 2)).to(DEV)
    assert torch.equal(y.view(-1, 384), want + lin.bias.detach())
    # a variable key set keeps its mode and its per-row slice counts through a file
    cap = layer._bsi_keys_cuda
    ops.save_keyset(cap, str(tmp_path))
    cap2, *_ = ops.load_keyset(str(tmp_path))
    a, b = ops.debug_keys_tensors(cap), ops.debug_keys_tensors(cap2)
    assert torch.equal(a["words"], b["words"]) and torch.equal(a["q8"], b["q8"])
    assert dict(ops.bsi_keys_cuda_stats(cap)["Sb_counts"]) == dict(ops.bsi_keys_cuda_stats(cap2)["Sb_counts"])
    layer2 = BSIQuantizedLinear(keyset=str(tmp_path), bias=lin.bias.detach())
    assert torch.equal(layer2(x), y)
