"""CPU checks of the drop-in boundary: the shared library loads without a GPU, exports
every symbol that include/b200mat.h declares (and nothing undeclared), the Python
structs match the C layout, and an operation without a device fails loudly."""
import ctypes as ct
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "b200mat.h")
LIB = os.path.join(ROOT, "deepnet_b200", "libb200mat.so")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"^\s*(?:const\s+)?(?:unsigned\s+)?(?:int|void|float|char)\s*\*?\s*(\w+)\s*\(", text, flags=re.M)
    return sorted(set(names))


def test_header_compiles_as_c():
    subprocess.check_call(["gcc", "-std=c99", "-fsyntax-only", "-x", "c", HEADER])


def test_library_exports_every_declared_symbol():
    assert os.path.exists(LIB), "build the library first (python -m deepnet_b200.build)"
    lib = ct.CDLL(LIB)
    names = declared_functions()
    assert len(names) > 100
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_no_undeclared_exports():
    out = subprocess.check_output(["nm", "-D", "--defined-only", LIB], text=True)
    exported = {l.split()[-1] for l in out.splitlines() if " T " in l and not l.split()[-1].startswith("_")}
    extra = sorted(exported - set(declared_functions()))
    assert not extra, extra


def test_struct_layouts_match_header():
    from deepnet_b200 import b200mat
    assert ct.sizeof(b200mat.cudamat) == 40          # cudamat/cudamat.cuh:21-29 on LP64
    assert ct.sizeof(b200mat.rnd_struct) == 16       # same size as the reference's two pointers
    assert b200mat.cudamat.size.offset == 24 and b200mat.cudamat.is_trans.offset == 32
    code = r'''
#include <stdio.h>
#include "b200mat.h"
int main(void) { printf("%zu %zu %zu %zu\n", sizeof(cudamat), sizeof(rnd_struct), sizeof(b200_pass), sizeof(b200_fused_gemm)); return 0; }
'''
    exe = "/tmp/b200mat_abi_probe"
    subprocess.run(["gcc", "-x", "c", "-", "-I", os.path.join(ROOT, "include"), "-o", exe], input=code, text=True, check=True)
    sizes = [int(x) for x in subprocess.check_output([exe], text=True).split()]
    assert sizes == [ct.sizeof(b200mat.cudamat), ct.sizeof(b200mat.rnd_struct), ct.sizeof(b200mat._Pass),
                     ct.sizeof(b200mat._FusedGemm)]


def test_no_device_is_a_loud_failure_not_a_fallback():
    from deepnet_b200 import b200mat
    lib = ct.CDLL(LIB)
    if lib.b200_device_count() > 0:
        pytest.skip("a device is present")
    with pytest.raises(b200mat.CUDAMatException):
        b200mat.empty((2, 2))


def test_product_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "deepnet_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "eigenmat_oracle" not in text and "liboracle" not in text, f
