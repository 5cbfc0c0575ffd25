"""CPU-only checks of the drop-in boundary: the shared library loads, exports every function that
include/decoding_attn_b200.h declares (and the C++ decoding_attn of include/decoding_attn.h), the
ctypes mirror of da_decode_args_t has the C layout, and argument errors are reported as status
codes without touching a GPU."""
import ctypes
import os
import re
import subprocess
import tempfile

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "decoding_attn_b200.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(da_[a-z_0-9]+)\s*\(", text)))


def test_header_declares_the_expected_surface():
    names = declared_functions()
    for must in ("da_decode_fwd", "da_decode_fwd_host", "da_decode_fwd_static", "da_merge_partials",
                 "da_decode_workspace_bytes", "da_device_status", "da_last_error"):
        assert must in names


def test_library_exports_every_declared_symbol(native_lib):
    lib = native_lib.lib()
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert set(native_lib.EXPORTS) <= set(declared_functions())
    # the C++ entry point with the reference's signature (mangled)
    out = subprocess.run(["nm", "-D", "--defined-only", native_lib.LIB_PATH], capture_output=True, text=True).stdout
    assert "_Z13decoding_attnPvS_S_S_PimmmmmmbbP11CUstream_st" in out


def test_ctypes_struct_matches_c_layout(native_lib):
    src = ('#include <stdio.h>\n#include <stddef.h>\n#include "decoding_attn_b200.h"\n'
           'int main(){printf("%zu %zu %zu %zu %zu\\n", sizeof(da_decode_args_t), offsetof(da_decode_args_t,q),'
           'offsetof(da_decode_args_t,max_seq_k), offsetof(da_decode_args_t,softmax_scale),'
           'offsetof(da_decode_args_t,stream));return 0;}')
    with tempfile.TemporaryDirectory() as d:
        c = os.path.join(d, "t.c")
        open(c, "w").write(src)
        exe = os.path.join(d, "t")
        subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), c, "-o", exe], check=True)
        size, off_q, off_max, off_scale, off_stream = map(int, subprocess.check_output([exe]).split())
    A = native_lib.DecodeArgs
    assert ctypes.sizeof(A) == size
    assert (A.q.offset, A.max_seq_k.offset, A.softmax_scale.offset, A.stream.offset) == (
        off_q, off_max, off_scale, off_stream)


def test_argument_errors_without_a_gpu(native_lib):
    lib = native_lib.lib()
    a = native_lib.DecodeArgs()
    assert lib.da_decode_fwd(ctypes.byref(a)) == native_lib.DA_ERR_INVALID_ARG  # struct_size 0
    assert b"struct_size" in lib.da_last_error()
    a.struct_size = ctypes.sizeof(native_lib.DecodeArgs)
    assert lib.da_decode_fwd(ctypes.byref(a)) == native_lib.DA_ERR_INVALID_ARG  # null pointers
    assert lib.da_decode_fwd(None) == native_lib.DA_ERR_INVALID_ARG
    assert lib.da_status_string(native_lib.DA_ERR_UNSUPPORTED) == b"unsupported shape"
    assert lib.da_merge_partials(None, None, 1, 1, 128, 128, 128, 1, 1, None, None, None, 0, None) == \
        native_lib.DA_ERR_INVALID_ARG


def test_python_package_fails_loudly_without_library(tmp_path):
    code = ("import os, sys; os.environ['DA_LIB_PATH'] = %r; sys.path.insert(0, %r)\n"
            "from decoding_attention_b200 import cabi\n"
            "try:\n    cabi.lib()\nexcept ImportError as e:\n    print('IMPORTERROR')\n") % (
        str(tmp_path / "missing.so"), ROOT)
    out = subprocess.run(["python", "-c", code], capture_output=True, text=True).stdout
    assert "IMPORTERROR" in out
