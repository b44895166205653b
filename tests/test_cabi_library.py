"""The C-ABI shared library: loads, exports every declared symbol, validates
arguments on the host (no kernel is launched in this file)."""

import ctypes
import re
from pathlib import Path

import pytest

from slinoss_b200 import _C

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib():
    from slinoss_b200.build import build
    build()
    return _C.lib()


def test_header_symbols_are_exported(lib):
    header = (ROOT / "include" / "slinoss_b200.h").read_text()
    declared = re.findall(r"SL_API\s+[\w\s\*]+?\b(sl_\w+)\s*\(", header)
    assert len(declared) == len(set(declared)) == 22 and set(declared) == set(_C.EXPORTED_SYMBOLS)
    for name in declared:
        assert getattr(lib, name) is not None
    # ... and nothing else: every dynamic `sl_*` symbol of the library is declared in the header
    import shutil
    import subprocess
    if shutil.which("nm"):
        out = subprocess.run(["nm", "-D", "--defined-only", str(_C.lib_path())], capture_output=True,
                             text=True, check=True).stdout
        exported = {ln.split()[-1] for ln in out.splitlines() if ln.split() and ln.split()[-1].startswith("sl_")}
        assert exported == set(declared), exported ^ set(declared)


def test_version_and_status_strings(lib):
    assert lib.sl_version() >= 100
    assert lib.sl_status_string(0) == b"ok"
    texts = {lib.sl_status_string(i) for i in range(9)}
    assert len(texts) == 9 and lib.sl_status_string(99) == b"unknown status"


def test_workspace_sizes(lib):
    small = lib.sl_workspace_bytes(_C.WS_SCAN_BWD, 1, 2, 2, 64, 64, 64, 64, _C.SL_BF16, _C.PATH_SIMT)
    big = lib.sl_workspace_bytes(_C.WS_SCAN_BWD, 2, 2, 2, 64, 64, 64, 64, _C.SL_BF16, _C.PATH_SIMT)
    assert 0 < small < big and small % 256 == 0
    assert lib.sl_workspace_bytes(_C.WS_SCAN_FWD, 1, 2, 2, 64, 64, 64, 64, _C.SL_F32, _C.PATH_SIMT) == 0
    assert lib.sl_workspace_bytes(_C.WS_SCAN_BWD, 0, 2, 2, 64, 64, 64, 64, _C.SL_F32, _C.PATH_SIMT) == 0


def test_arguments_are_validated_before_any_launch(lib):
    buf = ctypes.create_string_buffer(4096)
    p = ctypes.addressof(buf) // 256 * 256 + 256
    null = None
    call = lambda *a: lib.sl_v2x2ssd_fwd(*a)
    dims = (1, 2, 2, 4, 4, 2, 4)
    # missing U
    assert call(null, p, p, p, p, null, null, null, p, null, null, *dims, 0, 0, 0, null, 0, null) == 1
    # only one of B_prev / U_prev
    assert call(p, p, p, p, p, null, p, null, p, null, null, *dims, 0, 0, 0, null, 0, null) == 1
    # groups do not divide heads
    assert call(p, p, p, p, p, null, null, null, p, null, null, 1, 3, 2, 4, 4, 2, 4, 0, 0, 0, null, 0,
                null) == 2
    # unknown dtype code
    assert call(p, p, p, p, p, null, null, null, p, null, null, *dims, 7, 0, 0, null, 0, null) == 4
    # misaligned K
    assert call(p, p, p + 4, p, p, null, null, null, p, null, null, *dims, 0, 0, 0, null, 0, null) == 3
    # backward without a workspace
    assert lib.sl_v2x2ssd_bwd(p, p, p, p, p, null, null, null, null, null, p, null, p, p, p, p, p, null,
                              null, null, *dims, 0, 0, 1, null, 0, null) == 5
    # decode / tail / scanprep null checks
    assert lib.sl_v2x2ssd_decode(null, p, p, p, p, p, null, null, p, p, 1, 2, 2, 4, 2, 0, 0, null) == 1
    assert lib.sl_mixer_tail_fwd(null, p, 8, null, null, p, 1e-5, p, 1, 2, 4, 4, 0, null) == 1
    assert lib.sl_mixer_tail_fwd(p, p, 8, null, null, p, 1e-5, p, 1, 2, 4, 4096, 0, null) == 4


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_C, "_lib", None)
    monkeypatch.setattr(_C, "_LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(RuntimeError, match="there is no fallback path"):
        _C.lib()


def test_alias_makes_reference_style_imports_resolve_to_this_package():
    import subprocess
    import sys
    code = ("import slinoss_b200.alias as a; a.install(); import slinoss; "
            "from slinoss.ops.v2x2ssd import v2x2ssd; from slinoss.layers import SLinOSSMixer; "
            "from slinoss.blocks import SLinOSSStack; import slinoss_b200 as sb; "
            "import importlib; assert SLinOSSMixer is sb.SLinOSSMixer and v2x2ssd is importlib.import_module('slinoss_b200.ops.v2x2ssd').v2x2ssd; "
            "a.uninstall(); import sys; assert 'slinoss' not in sys.modules; print('ok')")
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=str(ROOT))
    assert out.returncode == 0 and out.stdout.strip() == "ok", out.stderr
