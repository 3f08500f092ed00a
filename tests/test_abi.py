"""The C ABI without a GPU: the library loads, exports every function include/bivmoe.h
declares, the header is valid C whose structs have the sizes the ctypes mirror assumes,
and the product path has no fallback when the library is missing.  No compute calls."""
import ctypes as C
import os
import re
import subprocess
import sys

import pytest

from biv_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "bivmoe.h")


def declared_functions():
    text = open(HEADER).read()
    return sorted(set(re.findall(r"BIVMOE_API\s+[^;(]*?\b(bivmoe_\w+)\s*\(", text)))


def test_library_exports_every_declared_function():
    names = declared_functions()
    assert len(names) >= 30
    lib = capi.lib()
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing
    # and the ctypes mirror binds exactly the header's functions
    assert sorted(capi.SYMBOLS) == names


def test_header_is_plain_c_and_struct_sizes_match_the_ctypes_mirror(tmp_path):
    src = tmp_path / "sizes.c"
    src.write_text('#include <stdio.h>\n#include "bivmoe.h"\n'
                   "int main(void) {\n"
                   '    printf("%zu %zu %zu\\n", sizeof(bivmoe_experts), sizeof(bivmoe_desc), '
                   "sizeof(bivmoe_peer_info));\n    return 0;\n}\n")
    exe = tmp_path / "sizes"
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-I", os.path.dirname(HEADER), str(src), "-o",
                    str(exe)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()
    assert [int(v) for v in out] == [C.sizeof(capi.Experts), C.sizeof(capi.Desc), C.sizeof(capi.PeerInfo)]


def test_no_fallback_when_the_library_is_missing():
    code = ("import biv_b200.capi as c\n"
            "c.LIB_PATH = c.LIB_PATH + '.absent'\n"
            "try:\n    c.lib()\nexcept ImportError as e:\n    print('ImportError', 'no CPU fallback' in str(e))\n")
    out = subprocess.run([sys.executable, "-c", code], check=True, capture_output=True, text=True, cwd=ROOT)
    assert out.stdout.split() == ["ImportError", "True"]


def test_nothing_in_the_package_imports_the_oracle():
    pkg = os.path.join(ROOT, "biv_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert not re.search(r"^\s*(import|from)\s+oracle\b", text, re.M), f
                assert "libbivmoe_oracle" not in text, f
