"""CPU-only checks of the C-ABI library: it builds, loads and exports what the header declares."""

import ctypes
import os
import re

import pytest

from conftest import ROOT


@pytest.fixture(scope="module")
def lib_path():
    from flashquant_b200 import build
    return build.build_native()


def header_symbols():
    text = open(os.path.join(ROOT, "include", "flashquant_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fq_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_entry_points():
    syms = header_symbols()
    for must in ["fq_tq4_compress", "fq_tq4_decompress", "fq_tq4_compress_append",
                 "fq_tq4_compress_append_qjl", "fq_split_k_paged_decode",
                 "fq_paged_decode_partials", "fq_split_k_merge", "fq_last_error_string"]:
        assert must in syms


def test_library_exports_every_declared_symbol(lib_path):
    lib = ctypes.CDLL(lib_path)
    for name in header_symbols():
        assert hasattr(lib, name), f"{name} declared in the header but not exported"


def test_ctypes_table_matches_header(lib_path):
    from flashquant_b200 import _native
    assert sorted(_native.SIGNATURES) == header_symbols()
    lib = _native.load()
    assert lib.fq_version() >= 100


def test_argument_errors_need_no_gpu(lib_path):
    # argument validation happens before any CUDA call
    from flashquant_b200 import _native
    lib = _native.load()
    rc = lib.fq_tq4_compress(None, 0, None, None, None, 15, None, None, 4, 128, None)
    assert rc == -1 and b"null" in lib.fq_last_error_string()
    rc = lib.fq_tq4_compress(None, 0, None, None, None, 15, None, None, -1, 128, None)
    assert rc == -1
    assert lib.fq_tq4_compress(None, 0, None, None, None, 15, None, None, 0, 128, None) == 0
    assert lib.fq_paged_decode_workspace_bytes(32, 32, 8, 128, 8) >= 32 * 32 * 8 * 132 * 4


def test_host_step_layout_and_new_entry_points_need_no_gpu(lib_path):
    """Host-only parts of the newer entry points: the packed step's offsets, workspace sizes and
    argument checks that run before any CUDA call."""
    from flashquant_b200 import _native
    lib = _native.load()
    off = (ctypes.c_uint64 * 8)()
    assert lib.fq_decode_step_offsets(32, 32, 8, 128, 256, 1, off) == 0
    key, value, slots, lens, table, q, out, total = list(off)
    assert all(o % 256 == 0 for o in off)
    assert key == 0 and key < value < slots < lens < table < q < out < total
    assert value - key >= 32 * 8 * 128 * 2 and slots - value >= 32 * 8 * 128 * 2
    assert lens - slots >= 32 * 8 and table - lens >= 32 * 4 and q - table >= 32 * 256 * 4
    assert out - q >= 32 * 32 * 128 * 2 and total - out >= 32 * 32 * 128 * 2
    assert total == lib.fq_decode_step_host_staging_bytes(32, 32, 8, 128, 256, 1)
    assert lib.fq_decode_step_offsets(32, 32, 8, 128, 256, 1, None) == -1
    assert lib.fq_decode_step_offsets(-1, 32, 8, 128, 256, 1, off) == -1
    # paged prefill: sizes, and refusals that precede every launch
    need = lib.fq_paged_tq4_prefill_workspace_bytes(1000, 32, 128)
    assert need >= 256 + 1000 * 32 * 128 * (2 + 4)
    assert lib.fq_paged_tq4_prefill_workspace_bytes(-1, 32, 128) == 0
    args = [None, 2, None, None, 4, None, None, None, 8, None, 16, None, 2, 100, 50, 32, 8, 128, 16,
            64, 0.1, None, None, 0, None]
    assert lib.fq_paged_tq4_prefill(*args) == -1 and b"null" in lib.fq_last_error_string()
    empty = list(args)
    empty[13] = 0                                   # no query tokens: nothing to do
    assert lib.fq_paged_tq4_prefill(*empty) == 0
    bad = list(args)
    bad[12] = -1
    assert lib.fq_paged_tq4_prefill(*bad) == -1


def test_package_refuses_cpu_tensors(lib_path):
    import torch
    import flashquant_b200 as fq
    from flashquant_b200._native import FlashQuantNativeError
    with pytest.raises(FlashQuantNativeError):
        fq.tq4_compress(torch.randn(2, 1, 128), torch.eye(128), torch.zeros(15))


def test_pybind_module_exports_the_probed_names():
    """The reference's Python layer looks for these attributes on ``flashquant._C``."""
    from flashquant_b200 import build
    build.build_pybind()
    import torch  # noqa: F401  (the module links against libtorch)
    from flashquant_b200 import _C
    for name in ["tq4_compress", "tq4_decompress", "fused_tq_attention", "split_k_paged_decode",
                 "fused_paged_tq4_decode", "tq4_compress_append", "tq4_compress_append_qjl",
                 "paged_tq4_prefill"]:
        assert hasattr(_C, name)
    assert not hasattr(_C, "codebook")  # would hijack the reference's Lloyd-Max solver
    import pytest
    with pytest.raises(RuntimeError):
        _C.tq4_compress(torch.randn(2, 1, 128), torch.zeros(128, 64), torch.zeros(128, 64),
                        torch.zeros(15), None)
