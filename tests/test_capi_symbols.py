"""The C-ABI library builds, loads and exports every entry point the header declares; compute
wrappers refuse CPU tensors (there is no fallback path)."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from xdit_b200 import _capi, build

    build.build()
    return _capi.load()


def _declared():
    text = open(os.path.join(ROOT, "include", "xdit_b200.h")).read()
    return sorted(set(re.findall(r"XDIT_API\s+[\w\s\*]+?\b(xdit_\w+)\s*\(", text)))


def test_header_declares_expected_entry_points():
    from xdit_b200 import _capi

    assert _declared() == sorted(_capi.EXPORTS)


def test_every_declared_symbol_is_exported(lib):
    for name in _declared():
        assert hasattr(lib, name), name
        assert ctypes.cast(getattr(lib, name), ctypes.c_void_p).value


def test_struct_sizes_match_header():
    """ctypes mirrors must have the C layout: compile a tiny probe with the header and compare."""
    import subprocess
    import tempfile

    from xdit_b200 import _capi

    src = r'''
#include <stdio.h>
#include "xdit_b200.h"
int main(void) {
  printf("%zu %zu %zu %zu %zu %zu\n", sizeof(struct xdit_caps), sizeof(struct xdit_seq),
         sizeof(struct xdit_attn_params), sizeof(struct xdit_pack_job), sizeof(struct xdit_kv_patch_params),
         sizeof(struct xdit_prologue_params));
  return 0;
}'''
    with tempfile.TemporaryDirectory() as d:
        c = os.path.join(d, "probe.c")
        open(c, "w").write(src)
        exe = os.path.join(d, "probe")
        subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), c, "-o", exe], check=True)
        sizes = [int(x) for x in subprocess.run([exe], capture_output=True, text=True, check=True).stdout.split()]
    mirrors = [_capi.Caps, _capi.Seq, _capi.AttnParams, _capi.PackJob, _capi.KvPatchParams, _capi.PrologueParams]
    assert sizes == [ctypes.sizeof(m) for m in mirrors]


def test_argument_errors_need_no_gpu(lib):
    from xdit_b200 import _capi

    assert lib.xdit_attn_fwd(None, None) == -1  # XDIT_E_NULL
    assert b"NULL" in lib.xdit_last_error_string()
    p = _capi.AttnParams()
    p.dtype = 7
    assert lib.xdit_attn_which(ctypes.byref(p)) == -4  # XDIT_E_DTYPE
    assert lib.xdit_ulysses_pack(None, 1, 0, 1, 2, 8, 2, None) == -1
    assert lib.xdit_merge_out_lse(None, None, None, None, None, 0, 1, 8, 1, None) == -1


def test_no_cpu_fallback():
    from xdit_b200 import ops

    x = torch.zeros(1, 2, 4, 8)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        ops.attn_fwd(x, x, x)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        ops.kv_patch_update(x, x, x, x, 0)


def test_missing_library_fails_loudly(monkeypatch):
    from xdit_b200 import _capi

    monkeypatch.setattr(_capi, "_lib", None)
    monkeypatch.setattr(_capi, "LIB_PATH", "/nonexistent/libxdit_b200.so")
    with pytest.raises(RuntimeError, match="no fallback"):
        _capi.load()


def test_product_does_not_import_oracle():
    """Nothing under xdit_b200/ may reference the oracle."""
    pkg = os.path.join(ROOT, "xdit_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.lower(), os.path.join(dirpath, f)
