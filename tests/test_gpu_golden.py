"""The CUDA library against the fixtures produced by the reference's own kernels (bit-exact)."""
import numpy as np
import pytest
import torch

import _capi_helpers as H
import _golden
from bsipytorch_b200 import capi
from oracle import oracle as o

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def g():
    return _golden.load()


@pytest.mark.parametrize("name", _golden.DOT_CASES)
def test_pack_and_dot_against_reference_outputs(g, name):
    q, k = _golden.case_inputs(g, name)
    qa = H.quantize_pack(q.to(DEV), 2, 7, True)
    kb = H.quantize_pack(k.to(DEV), 2, 6, False)
    np.testing.assert_array_equal(H.as_u64(qa["words"]), g[f"{name}_q_words"])
    np.testing.assert_array_equal(qa["scales"].cpu().numpy(), g[f"{name}_q_scales"])
    np.testing.assert_array_equal(H.as_u64(kb["words"]), g[f"{name}_k_words"])
    np.testing.assert_array_equal(kb["scales"].cpu().numpy(), g[f"{name}_k_scales"])
    want = g[f"{name}_out"].view(np.uint32)
    # 1xxx: single-CTA tiles of that width; 3xxx: the paired-CTA kernel (the one the benchmark times), every width
    for engine in (capi.ENGINE_TCGEN05, capi.ENGINE_SIMT, 1064, 1128, 3064, 3096, 3128, 3160, 3192, 3224, 3256):
        out = H.dot_i8(qa["q8"], qa["scales"], kb["q8"], kb["scales"], o.scale_inv(2), engine)
        np.testing.assert_array_equal(out.cpu().numpy().view(np.uint32), want)
    Bw = torch.from_numpy(g[f"{name}_Bw"]).to(DEV)
    out = H.dot_words(qa["words"], qa["scales"], kb["words"], Bw, o.scale_inv(2))
    np.testing.assert_array_equal(out.cpu().numpy().view(np.uint32), want)


@pytest.mark.parametrize("name", _golden.DOT_CASES)
def test_ewah_against_reference_streams(g, name):
    words = g[f"{name}_q_words"]
    w2 = torch.from_numpy(words.reshape(-1, words.shape[2]).view(np.int64)).to(DEV)
    stream, off, length, flags = H.ewah_encode(w2, 0.5)
    np.testing.assert_array_equal(H.as_u64(stream), g[f"{name}_ewah_stream"])
    np.testing.assert_array_equal(off.cpu().numpy(), g[f"{name}_ewah_off"])
    np.testing.assert_array_equal(length.cpu().numpy(), g[f"{name}_ewah_len"])
    np.testing.assert_array_equal(flags.cpu().numpy(), g[f"{name}_ewah_flags"])


@pytest.mark.parametrize("W", [5, 33, 128])
def test_ewah_structured_against_reference(g, W):
    words = g[f"ewah{W}_words"]
    wt = torch.from_numpy(words.view(np.int64)).to(DEV)
    for thr in (0.5, 0.2, 1.0):
        tag = f"ewah{W}_t{int(thr * 10)}"
        stream, off, length, flags = H.ewah_encode(wt, thr)
        np.testing.assert_array_equal(H.as_u64(stream), g[f"{tag}_stream"])
        np.testing.assert_array_equal(length.cpu().numpy(), g[f"{tag}_len"])
        np.testing.assert_array_equal(flags.cpu().numpy(), g[f"{tag}_flags"])


@pytest.fixture(scope="module")
def m():
    return _golden.load_modes()


@pytest.mark.parametrize("tag", ["row", "rowr"])
def test_row_scale_dot_against_reference_outputs(m, tag):
    """One scale per query row (no chunk scales): the reference's generic kernels, tensor-core and plain."""
    q = torch.from_numpy(m[f"{tag}_q"].copy())
    k = _golden.f16(m, f"{tag}_k_f16bits").float()
    qa = H.quantize_pack(q.to(DEV), 2, 7, False)
    kb = H.quantize_pack(k.to(DEV), 2, 6, False)
    np.testing.assert_array_equal(H.as_u64(qa["words"]), m[f"{tag}_q_words"])
    np.testing.assert_array_equal(qa["scales"].cpu().numpy(), m[f"{tag}_q_scales"])
    np.testing.assert_array_equal(H.as_u64(kb["words"]), m[f"{tag}_k_words"])
    want = m[f"{tag}_out_tc"].view(np.uint32)
    np.testing.assert_array_equal(want, m[f"{tag}_out_plain"].view(np.uint32))
    for engine in (capi.ENGINE_TCGEN05, capi.ENGINE_SIMT, 1064, 3064, 3256):
        out = H.dot_i8(qa["q8"], qa["scales"], kb["q8"], kb["scales"], o.scale_inv(2), engine)
        np.testing.assert_array_equal(out.cpu().numpy().view(np.uint32), want)


def test_outlier_clipping_against_reference_outputs(m):
    x = _golden.f16(m, "clip_x_f16bits")
    qa = H.quantize_pack(x.to(DEV), 2, 7, True, clip_k=3.0)
    np.testing.assert_array_equal(H.as_u64(qa["words"]), m["clip_words"])
    np.testing.assert_array_equal(qa["shifts"].cpu().numpy(), m["clip_shifts"])
    k = _golden.f16(m, "clip_k_f16bits").float()
    kb = H.quantize_pack(k.to(DEV), 2, 6, False, clip_k=3.0)
    np.testing.assert_array_equal(H.as_u64(kb["words"]), m["clip_row_words"])
    np.testing.assert_array_equal(kb["shifts"].cpu().numpy(), m["clip_row_shifts"])
    np.testing.assert_array_equal(kb["q8"][:, :k.shape[1]].cpu().numpy(), m["clip_row_ints"])


def test_variable_slice_mode_against_reference_outputs(m, monkeypatch):
    import bsipytorch_b200
    monkeypatch.setenv("BSI_FIXED_BITS_QUERIES", "0")
    monkeypatch.setenv("BSI_FIXED_BITS_KEYS", "0")
    ops = bsipytorch_b200.install_as_bsi_ops()
    q = torch.from_numpy(m["var_q"].copy())
    k = _golden.f16(m, "var_k_f16bits").float()
    keys_cap, *_ = ops.build_bsi_keys_cuda(k, 2, 0.5)
    qcap = ops.build_bsi_queries_cuda_batch_packed(q.to(DEV), 2, 0.5)
    np.testing.assert_array_equal(H.as_u64(ops.debug_query_batch_tensors(qcap)["words"]), m["var_q_words"])
    np.testing.assert_array_equal(H.as_u64(ops.debug_keys_tensors(keys_cap)["words"]), m["var_k_words"])
    out, *_ = ops.batch_dot_product_multiquery_cuda_batch_caps(qcap, keys_cap)
    np.testing.assert_array_equal(out.cpu().numpy().view(np.uint32), m["var_out_tc"].view(np.uint32))
    np.testing.assert_array_equal(out.cpu().numpy().view(np.uint32), m["var_out_plain"].view(np.uint32))
