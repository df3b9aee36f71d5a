"""The binding INTEGRATION.md describes, executed: the REFERENCE project's own Python package
(src/thor_fp4 of a thor-fp4 checkout) with its loader pointed at this repository's shared library.

Needs a checkout of the reference: the directory named by THOR_FP4_REFERENCE, else a directory `reference`
beside this repository; skipped when there is none (nothing of the reference is copied here).  Without a GPU
the test declares every ctypes signature the reference binds (its _decl_core / _decl_cutlass / _decl_fused)
on this library - a missing or renamed export fails there - and calls the size helpers through the
reference's ops module.  With a GPU it goes on to run the reference's own quantizer and Linear test files
(tests/test_quant.py, tests/test_linear.py of the checkout) over this library.
"""
import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
LIB = ROOT / "thor-fp4_b200" / "build" / "libthorfp4_b200.so"


def _reference_checkout():
    cands = [os.environ.get("THOR_FP4_REFERENCE"), str(ROOT.parent / "reference")]
    for c in cands:
        if c and (Path(c) / "src" / "thor_fp4" / "_ext.py").exists():
            return Path(c)
    return None


# what the maintainer's edit of src/thor_fp4/_ext.py amounts to, applied from outside: every role of the reference's
# loader (core / cutlass / fused) is served by the one library
_PATCH = textwrap.dedent('''
    import ctypes, sys
    sys.path.insert(0, r"{ref}/src")
    sys.path.insert(0, r"{ref}/tests")
    import thor_fp4._ext as E
    assert E.__file__.startswith(r"{ref}"), E.__file__          # the reference's module, not this repository's
    lib = ctypes.CDLL(r"{lib}")
    E._decl_core(lib)
    E._decl_cutlass(lib)
    lib.tfc4_variant_index.argtypes = [ctypes.c_char_p]; lib.tfc4_variant_index.restype = ctypes.c_int
    E._decl_fused(lib)
    E._core = E._cutlass = E._fused = lib
    import thor_fp4
    from thor_fp4 import ops
    assert ops.pad_rows(300) == 384 and ops.packed_bytes(300, 1024) == 384 * 512 and ops.scale_bytes(300, 1024) == 384 * 64
    assert ops.mx_packed_bytes(300, 1024, "mxfp8") == 384 * 1024 and ops.mx_scale_bytes(300, 1024) == 384 * 32
    assert E.cutlass().tfc4_n_variants() > 0 and E.fused().tfc4f_n_variants() == 8
    assert E.fused().tfc4f_sfd_bytes(300, 1024) == 384 * 32
    print("BINDING_OK")
''')


def test_reference_loader_binds_every_symbol_on_this_library():
    ref = _reference_checkout()
    if ref is None:
        pytest.skip("no checkout of the reference project at THOR_FP4_REFERENCE or beside this repository")
    r = subprocess.run([sys.executable, "-c", _PATCH.format(ref=ref, lib=LIB)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "BINDING_OK" in r.stdout, r.stdout + r.stderr


@pytest.mark.gpu
def test_reference_package_passes_its_own_quantizer_and_linear_tests_on_this_library():
    ref = _reference_checkout()
    if ref is None:
        pytest.skip("no checkout of the reference project at THOR_FP4_REFERENCE or beside this repository")
    code = _PATCH.format(ref=ref, lib=LIB) + textwrap.dedent('''
        rc = lib.tfp4_init(0)
        assert rc == 0, rc
        import pytest
        sys.exit(pytest.main(["-q", "-x", "-p", "no:cacheprovider", r"{ref}/tests/test_quant.py", r"{ref}/tests/test_linear.py"]))
    ''').format(ref=ref)
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=900, cwd=str(ref / "tests"))
    assert r.returncode == 0, (r.stdout[-3000:] + r.stderr[-2000:])
