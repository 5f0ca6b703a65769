"""Pins the CPU checker against outputs of the reference's own CUDA kernels.

The fixture file was written on a B200 by tests/golden/make_golden_from_ref.py, which drives the
reference's bsi_cuda_kernels.cu (compiled unmodified) through its extern "C" launchers.
"""
import numpy as np
import pytest

import _golden
from oracle import oracle as o


@pytest.fixture(scope="module")
def g():
    return _golden.load()


@pytest.mark.parametrize("name", _golden.DOT_CASES)
def test_query_and_key_packing(g, name):
    q, k = _golden.case_inputs(g, name)
    qa = o.quantize_pack(q.float().numpy(), 2, 7, True)
    np.testing.assert_array_equal(qa["words"], g[f"{name}_q_words"])
    np.testing.assert_array_equal(qa["shifts"], g[f"{name}_q_shifts"])
    np.testing.assert_array_equal(qa["scales"], g[f"{name}_q_scales"])
    kb = o.quantize_pack(k.numpy(), 2, 6, False)
    np.testing.assert_array_equal(kb["words"], g[f"{name}_k_words"])
    np.testing.assert_array_equal(kb["shifts"], g[f"{name}_k_shifts"])
    np.testing.assert_array_equal(kb["scales"], g[f"{name}_k_scales"])
    np.testing.assert_array_equal(kb["qvals"], g[f"{name}_k_ints"])
    np.testing.assert_array_equal(o.slice_weights(6, kb["scales"]), g[f"{name}_Bw"])


@pytest.mark.parametrize("name", _golden.DOT_CASES)
def test_fixed76_dot_outputs_bit_exact(g, name):
    q, k = _golden.case_inputs(g, name)
    want = g[f"{name}_out"]
    got = o.fixed_dot(q.float().numpy(), k.numpy(), 2, via="i8")
    np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))
    got_p = o.dot_popc(g[f"{name}_q_words"], g[f"{name}_q_scales"], g[f"{name}_k_words"], g[f"{name}_Bw"],
                       o.scale_inv(2))
    np.testing.assert_array_equal(got_p.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("name", _golden.DOT_CASES)
def test_ewah_of_query_slices(g, name):
    words = g[f"{name}_q_words"]
    w2 = words.reshape(-1, words.shape[2])
    counts = o.slice_popcount(w2)
    np.testing.assert_array_equal(counts, g[f"{name}_ewah_counts"])
    flags = o.compress_flags(counts, w2.shape[1], 0.5)
    np.testing.assert_array_equal(flags, g[f"{name}_ewah_flags"])
    stream, off, length = o.ewah_encode(w2, flags)
    np.testing.assert_array_equal(stream, g[f"{name}_ewah_stream"])
    np.testing.assert_array_equal(off, g[f"{name}_ewah_off"])
    np.testing.assert_array_equal(length, g[f"{name}_ewah_len"])


@pytest.mark.parametrize("tag", ["f32", "f16", "bf16"])
def test_edge_rows(g, tag):
    x = g[f"edge_{tag}_x"]
    c = o.quantize_pack(x, 2, 7, True)
    np.testing.assert_array_equal(c["words"], g[f"edge_{tag}_words"])
    np.testing.assert_array_equal(c["shifts"], g[f"edge_{tag}_shifts"])
    r = o.quantize_pack(x, 2, 6, False)
    np.testing.assert_array_equal(r["words"], g[f"edge_{tag}_row_words"])
    np.testing.assert_array_equal(r["shifts"], g[f"edge_{tag}_row_shifts"])


def test_bf16_activations(g):
    c = o.quantize_pack(g["bf16_x"], 2, 7, True)
    np.testing.assert_array_equal(c["words"], g["bf16_words"])
    np.testing.assert_array_equal(c["shifts"], g["bf16_shifts"])


@pytest.mark.parametrize("W", [5, 33, 128])
@pytest.mark.parametrize("thr", [0.5, 0.2, 1.0])
def test_ewah_structured(g, W, thr):
    words = g[f"ewah{W}_words"]
    tag = f"ewah{W}_t{int(thr * 10)}"
    flags = o.compress_flags(o.slice_popcount(words), W, thr)
    np.testing.assert_array_equal(flags, g[f"{tag}_flags"])
    stream, off, length = o.ewah_encode(words, flags)
    np.testing.assert_array_equal(stream, g[f"{tag}_stream"])
    np.testing.assert_array_equal(off, g[f"{tag}_off"])
    np.testing.assert_array_equal(length, g[f"{tag}_len"])
    for s in range(words.shape[0]):
        np.testing.assert_array_equal(o.ewah_decode(stream[off[s]: off[s] + length[s]], W), words[s])


@pytest.fixture(scope="module")
def m():
    return _golden.load_modes()


def test_variable_slice_mode_against_reference_kernels(m):
    q, k = m["var_q"], _golden.f16(m, "var_k_f16bits").float().numpy()
    qa, kb = o.variable_pack(q, 2), o.variable_pack(k, 2, per_row=True)
    np.testing.assert_array_equal(qa["ints"], m["var_q_ints"])
    np.testing.assert_array_equal(kb["ints"], m["var_k_ints"])
    np.testing.assert_array_equal(qa["words"], m["var_q_words"])
    np.testing.assert_array_equal(kb["words"], m["var_k_words"])
    want = o.variable_dot(q, k, 2).view(np.uint32)
    np.testing.assert_array_equal(want, m["var_out_tc"].view(np.uint32))
    np.testing.assert_array_equal(want, m["var_out_plain"].view(np.uint32))


@pytest.mark.parametrize("tag", ["row", "rowr"])
def test_row_scale_dot_against_reference_kernels(m, tag):
    q, k = m[f"{tag}_q"], _golden.f16(m, f"{tag}_k_f16bits").float().numpy()
    qa = o.quantize_pack(q, 2, 7, False)
    kb = o.quantize_pack(k, 2, 6, False)
    np.testing.assert_array_equal(qa["words"], m[f"{tag}_q_words"])
    np.testing.assert_array_equal(qa["scales"], m[f"{tag}_q_scales"])
    np.testing.assert_array_equal(kb["words"], m[f"{tag}_k_words"])
    np.testing.assert_array_equal(kb["scales"], m[f"{tag}_k_scales"])
    got = o.fixed_dot(q, k, 2, chunk_scale=False).view(np.uint32)
    np.testing.assert_array_equal(got, m[f"{tag}_out_tc"].view(np.uint32))
    np.testing.assert_array_equal(got, m[f"{tag}_out_plain"].view(np.uint32))


def test_outlier_clipping_against_reference_kernels(m):
    x = _golden.f16(m, "clip_x_f16bits").float().numpy()
    qa = o.quantize_pack(x, 2, 7, True, 3.0)
    np.testing.assert_array_equal(qa["words"], m["clip_words"])
    np.testing.assert_array_equal(qa["shifts"], m["clip_shifts"])
    k = _golden.f16(m, "clip_k_f16bits").float().numpy()
    kb = o.quantize_pack(k, 2, 6, False, 3.0)
    np.testing.assert_array_equal(kb["words"], m["clip_row_words"])
    np.testing.assert_array_equal(kb["shifts"], m["clip_row_shifts"])
    np.testing.assert_array_equal(kb["qvals"], m["clip_row_ints"])
    assert not np.array_equal(qa["shifts"], o.quantize_pack(x, 2, 7, True)["shifts"])
