"""The C-ABI library loads and exports every symbol the header declares (no compute calls)."""
import os
import re

from bsipytorch_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "bsi_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(bsi_b200_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    names = _declared()
    assert len(names) >= 15
    L = capi.lib()
    for n in names:
        assert hasattr(L, n), f"{n} declared in include/bsi_b200.h but not exported"
        assert n in capi.SIGNATURES, f"{n} has no ctypes signature"
    assert sorted(capi.SIGNATURES) == names


def test_version_and_status_strings():
    L = capi.lib()
    assert L.bsi_b200_version() == 100
    assert L.bsi_b200_status_string(0) == b"ok"
    assert b"timed out" in L.bsi_b200_status_string(capi.ERR_TIMEOUT)


def test_argument_validation_needs_no_gpu():
    # Rejected before any CUDA call, so this runs on a CPU-only machine.
    L = capi.lib()
    assert L.bsi_b200_quantize_pack(None, 0, 4, 64, 64, 2, 9, 1, None, None, None, None, 0, None) == capi.ERR_UNSUPPORTED
    assert L.bsi_b200_quantize_pack(None, 7, 4, 64, 64, 2, 7, 1, None, None, None, None, 0, None) == capi.ERR_INVALID
    assert L.bsi_b200_quantize_pack(None, 0, 0, 64, 64, 2, 7, 1, None, None, None, None, 0, None) == capi.OK
    assert L.bsi_b200_dot_i8(None, 256, None, 1, None, 256, None, 4, 4, 1, 1.0, None, 4, None, 0, None) == capi.ERR_INVALID
    assert b"null" in L.bsi_b200_last_error()
    assert L.bsi_b200_ewah_scratch_bytes(10) >= 2 * 10 * 8      # per-slice sizes, block sums, a few words of bounds


def test_extension_module_exposes_reference_entry_points():
    import bsipytorch_b200
    ops = bsipytorch_b200.bsi_ops
    for n in ["build_bsi_keys_cuda", "build_bsi_queries_cuda_batch_packed", "build_bsi_queries_cuda_batch",
              "batch_dot_product_multiquery_cuda_batch_caps", "batch_dot_product_multiquery_cuda_caps",
              "get_last_query_build_profile_cuda", "reset_last_query_build_profile_cuda", "bsi_keys_cuda_stats",
              "bsi_query_caps_stats", "build_bsi_query_cuda", "build_bsi_query_cuda_hybrid", "cuda_builder_version",
              "CUDA_BUILDER_VERSION"]:
        assert hasattr(ops, n), n
    assert bsipytorch_b200.install_as_bsi_ops() is ops
    import bsi_ops
    assert bsi_ops is ops
