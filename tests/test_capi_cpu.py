"""CPU tests of the C-ABI library: it builds, loads, exports every declared symbol, and refuses to
compute without an initialised sm_100 device (no CPU fallback)."""
import os
import re

import pytest

from orin_llm_b200 import build, capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    build.build()
    return capi.lib()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "orin_attn_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(oattn_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree():
    assert declared_symbols() == sorted(capi.EXPORTS)


def test_library_exports_every_declared_symbol(lib):
    for name in declared_symbols():
        assert hasattr(lib, name), name


def test_error_strings(lib):
    assert lib.oattn_strerror(capi.OK) == b"ok"
    for code in range(1, 6):
        assert len(lib.oattn_strerror(code)) > 0


def test_no_compute_without_device(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("GPU present; covered by the gpu tests")
    assert lib.oattn_init(0) == capi.ERR_CUDA
    assert b"cudaSetDevice" in lib.oattn_last_cuda_error()
    assert lib.oattn_sm_count() == 0
    assert lib.oattn_decode_workspace_bytes(28, 4, 128) == 0
    # every compute entry point reports "device not initialised" instead of doing anything
    assert lib.oattn_combine(16, 2, 16, 4, 128, None) == capi.ERR_DEVICE
    assert lib.oattn_kv_shift(16, 16, 1, 1, 128, 8, 0, 1, None) == capi.ERR_DEVICE
    assert lib.oattn_decode(16, None, None, 16, 16, 16, 4, 2, 128, 8, 16, 0.1, 0, None, 256, 1 << 20, None) == capi.ERR_DEVICE
    assert lib.oattn_prefill(16, None, None, 16, 16, 16, 4, 2, 128, 8, 0, 4, 0.1, 0, None, 256, 1 << 20, None) == capi.ERR_DEVICE


def test_prefill_workspace_size(lib):
    assert lib.oattn_prefill_workspace_bytes(32, 8, 128, 512) == 512 * 32 * 128 * 2 + 256
    assert lib.oattn_prefill_workspace_bytes(32, 8, 96, 512) == 0      # head_dim not covered
    assert lib.oattn_prefill_workspace_bytes(34, 8, 128, 512) == 0     # n_head not a multiple of n_kv


def test_ops_refuses_cpu():
    import torch
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    from orin_llm_b200 import ops
    with pytest.raises(RuntimeError):
        ops.init(0)
