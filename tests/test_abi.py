"""The C-ABI library builds, loads without a GPU and exports every declared symbol."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from kvax_b200 import _lib, build
    if not os.path.exists(_lib.LIB_PATH):
        build.build()
    return _lib.load()


def test_every_declared_symbol_is_exported(lib):
    header = open(os.path.join(ROOT, "include", "kvax_b200.h")).read()
    declared = set(re.findall(r"\b(kvax_b200_[a-z_]+)\s*\(", header))
    assert {"kvax_b200_mask_build", "kvax_b200_attn_fwd", "kvax_b200_attn_bwd", "kvax_b200_permute_tokens"} <= declared
    from kvax_b200 import _lib
    assert declared == set(_lib.EXPORTS)
    for name in declared:
        assert hasattr(lib, name), name


def test_header_is_plain_c():
    """The boundary is a C ABI: the header has to compile as C99 on its own."""
    import subprocess
    res = subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-fsyntax-only", "-x", "c",
                          os.path.join(ROOT, "include", "kvax_b200.h")], capture_output=True, text=True)
    assert res.returncode == 0, res.stderr


def test_version_and_error_strings(lib):
    assert b"sm_100a" in lib.kvax_b200_version()
    assert lib.kvax_b200_error_string(0) == b"ok"
    assert b"workspace" in lib.kvax_b200_error_string(-3)


def test_argument_checks_without_a_device(lib):
    """Rejected calls return an error code before anything touches a device."""
    from kvax_b200 import _lib
    assert lib.kvax_b200_mask_build(None, None, 0, None) == -1
    p = _lib.MaskParams()
    assert lib.kvax_b200_mask_workspace_bytes(p) == 0
    assert lib.kvax_b200_attn_fwd(None, None, 0, None) == -1
    assert lib.kvax_b200_attn_bwd(None, None, 0, None) == -1
    assert lib.kvax_b200_permute_tokens(None, None, 1, 8, 4, 1, 0, None) == -1
    f = _lib.AttnFwdParams()
    assert lib.kvax_b200_attn_fwd_workspace_bytes(f) == 0


def test_struct_sizes_match_the_header():
    """ctypes mirrors of the header structs (sizes follow from the C layout rules)."""
    from kvax_b200 import _lib
    assert ctypes.sizeof(_lib.MaskDesc) == 48
    assert ctypes.sizeof(_lib.BlockMask) == 40
    assert ctypes.sizeof(_lib.AttnShape) == 4 * 10 + 8 * 12 + 8 * 4 + 8
    # checked against the C compiler: sizeof of every struct of the header
    import subprocess
    import tempfile
    src = '#include <stdio.h>\n#include "kvax_b200.h"\nint main(void){printf("%zu %zu %zu %zu %zu %zu\\n",' \
          "sizeof(kvax_b200_mask_desc),sizeof(kvax_b200_mask_params),sizeof(kvax_b200_block_mask),sizeof(kvax_b200_attn_shape)," \
          "sizeof(kvax_b200_attn_fwd_params),sizeof(kvax_b200_attn_bwd_params));return 0;}\n"
    with tempfile.TemporaryDirectory() as d:
        with open(os.path.join(d, "s.c"), "w") as f:
            f.write(src)
        subprocess.run(["gcc", "-std=c99", "-I", os.path.join(ROOT, "include"), os.path.join(d, "s.c"), "-o", os.path.join(d, "s")],
                       check=True)
        sizes = [int(x) for x in subprocess.run([os.path.join(d, "s")], capture_output=True, text=True, check=True).stdout.split()]
    mirrors = (_lib.MaskDesc, _lib.MaskParams, _lib.BlockMask, _lib.AttnShape, _lib.AttnFwdParams, _lib.AttnBwdParams)
    assert sizes == [ctypes.sizeof(m) for m in mirrors]
