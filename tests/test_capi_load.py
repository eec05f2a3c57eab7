"""CPU tests of the drop-in boundary: the C-ABI library loads without a GPU and exports every entry point that
include/vknn_cuda.h declares; without a device it reports VKC_ERR_NO_DEVICE instead of falling back."""
import ctypes as C

import pytest

import vknn_b200


def test_library_exports_every_declared_symbol():
    declared = vknn_b200.declared_symbols()
    assert len(declared) >= 25 and "vkc_attn_prefill" in declared and "vkc_gemm" in declared
    assert vknn_b200.exported_symbols() == declared


def test_null_context_is_refused_without_compute():
    lib = vknn_b200.load_library()
    assert lib.vkc_gemm(None, None, None, None, None, None, 1, 1, 1, 1, 0, 0, 0, 1, 1, 1, 0, 0, 0, None) == -1
    assert lib.vkc_layernorm(None, None, None, None, None, 1, 1, 1e-5, 0, None) == -1
    assert lib.vkc_attn_decode_workspace_bytes(32, 32, 8, 8192, 128) == 32 * 32 * 16 * 130 * 4
    assert lib.vkc_attn_decode_workspace_bytes(0, 32, 8, 8192, 128) == 0


def test_no_device_means_error_not_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    lib = vknn_b200.load_library()
    h = C.c_void_p()
    assert lib.vkc_ctx_create(0, C.byref(h)) == -6 and not h.value
    with pytest.raises(vknn_b200.VkcError):
        vknn_b200.Context(0)
