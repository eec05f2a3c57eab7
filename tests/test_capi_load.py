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
    assert lib.vkc_attn_decode_workspace_bytes(32, 32, 8, 8192, 128) == 32 * 32 * 18 * 130 * 4 + 32 * 8 * 4
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


def test_header_is_plain_c(tmp_path):
    """The boundary is a C ABI: the header must compile as C99 (what a cgo / JNI / ctypes-generator binding would see), and the
    Python mirror of struct vkc_fanout must have the layout the C compiler gives it."""
    import os
    import shutil
    import subprocess
    if not shutil.which("gcc"):
        pytest.skip("no C compiler")
    inc = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include")
    src = tmp_path / "t.c"
    src.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "vknn_cuda.h"\n'
                   'int main(void) { printf("%zu %zu %zu %zu %zu\\n", sizeof(vkc_fanout), offsetof(vkc_fanout, dest), '
                   'offsetof(vkc_fanout, flag), offsetof(vkc_fanout, state), offsetof(vkc_fanout, mcast)); return 0; }\n')
    exe = tmp_path / "t"
    subprocess.check_call(["gcc", "-std=c99", "-Wall", "-Werror", "-pedantic", "-I", inc, str(src), "-o", str(exe)])
    size, o_dest, o_flag, o_state, o_mcast = (int(v) for v in subprocess.check_output([str(exe)]).split())
    from vknn_b200.capi import Fanout
    assert (C.sizeof(Fanout), Fanout.dest.offset, Fanout.flag.offset, Fanout.state.offset, Fanout.mcast.offset) == (size, o_dest, o_flag, o_state, o_mcast)


def test_peer_and_fanout_entry_points_refuse_a_null_context():
    lib = vknn_b200.load_library()
    assert lib.vkc_peer_wait(None, None, 1, None, None) == -1
    assert lib.vkc_peer_export(None, None, None) == -1
    assert lib.vkc_peer_close(None, None) == -1
    assert lib.vkc_layernorm_fanout(None, None, None, None, 1, 1, 1e-5, 1, None, None) == -1
    assert lib.vkc_copy_rows(None, None, None, None, None, 1, 1, 1, None) == -1
    assert lib.vkc_gather_rows(None, None, None, None, 1, 1, 1, 1, 1, 0, None) == -1
    assert lib.vkc_gemm_gated(None, None, None, None, None, None, 1, 1, 1, 1, 0, 0, 0, 1, 1, 1, 0, 0, 1, -1, None, None) == -1
    assert lib.vkc_device_info(None, None, 0, None, None) == -1


def test_gate_struct_layout(tmp_path):
    """The Python mirror of struct vkc_gate has the layout the C compiler gives it."""
    import os
    import shutil
    import subprocess
    if not shutil.which("gcc"):
        pytest.skip("no C compiler")
    inc = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include")
    src = tmp_path / "g.c"
    src.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "vknn_cuda.h"\n'
                   'int main(void) { printf("%zu %zu %zu\\n", sizeof(vkc_gate), offsetof(vkc_gate, n), offsetof(vkc_gate, state)); return 0; }\n')
    exe = tmp_path / "g"
    subprocess.check_call(["gcc", "-std=c99", "-Wall", "-Werror", "-pedantic", "-I", inc, str(src), "-o", str(exe)])
    size, o_n, o_state = (int(v) for v in subprocess.check_output([str(exe)]).split())
    from vknn_b200.capi import Gate
    assert (C.sizeof(Gate), Gate.n.offset, Gate.state.offset) == (size, o_n, o_state)
