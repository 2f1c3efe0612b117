"""The C-ABI library builds, loads without a GPU, and exports exactly what include/tachyon_b200.h declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared():
    text = open(os.path.join(ROOT, "include", "tachyon_b200.h")).read()
    return sorted(set(re.findall(r"^TB_API [^;]*?\b(tb_\w+)\(", text, flags=re.M)))


@pytest.fixture(scope="module")
def lib_path():
    from tachyon_b200 import build

    return build.build()


def test_header_declares_the_entry_points():
    names = declared()
    assert "tb_gemv_q8" in names and "tb_attend_decode" in names and "tb_decoder_step" in names
    assert len(names) >= 45


def test_library_exports_every_declared_symbol(lib_path):
    lib = ctypes.CDLL(lib_path)
    missing = [n for n in declared() if not hasattr(lib, n)]
    assert not missing, missing


def test_binding_covers_the_header(lib_path):
    from tachyon_b200 import _lib

    assert sorted(_lib.SIGNATURES) == declared()


def test_binding_passes_as_many_arguments_as_the_header_takes():
    """A missing entry in a ctypes signature shifts every later argument: a pointer then travels as 32 bits."""
    from tachyon_b200 import _lib

    text = open(os.path.join(ROOT, "include", "tachyon_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    for name, args in re.findall(r"^TB_API [^;(]*?\b(tb_\w+)\(([^;]*?)\);", text, flags=re.M | re.S):
        args = args.strip()
        count = 0 if args in ("", "void") else args.count(",") + 1
        assert len(_lib.SIGNATURES[name][1]) == count, f"{name}: the header takes {count} arguments"
        # pointers must be declared as pointers
        for i, a in enumerate(args.split(",") if count else []):
            if "*" in a:
                assert _lib.SIGNATURES[name][1][i] in (ctypes.c_void_p, ctypes.c_char_p) or hasattr(_lib.SIGNATURES[name][1][i], "contents"), f"{name}: argument {i} is a pointer"


def test_library_needs_no_cuda_runtime_library(lib_path):
    import subprocess

    needed = subprocess.run(["readelf", "-d", lib_path], capture_output=True, text=True).stdout
    assert "libcudart" not in needed, "the CUDA runtime must be linked statically"


def test_no_gpu_is_reported_not_papered_over(lib_path):
    import tachyon_b200 as tb

    if os.path.exists("/dev/nvidiactl"):
        pytest.skip("a GPU is present")
    with pytest.raises(tb.Error) as e:
        tb.Context(0)
    assert e.value.status in (1, 3, 4)  # no driver / no such GPU / CUDA error: never a silent CPU path


def test_bad_descriptors_are_rejected_before_launch(lib_path):
    """Host-side validation needs no GPU for null contexts."""
    lib = ctypes.CDLL(lib_path)
    lib.tb_last_error.restype = ctypes.c_char_p
    assert lib.tb_sync(None) == 3
    assert b"null" in lib.tb_last_error()
    assert lib.tb_attend_decode(None, None) == 3


def test_a_missing_driver_is_reported():
    """crates/tachyon/tests/no_driver.rs:5-12: with $TACHYON_LIBCUDA naming a file that is not there, listing the devices and
    opening a context both fail cleanly with NoDriver, and the message names the variable.  Its own process: the driver is
    looked for once per process."""
    import subprocess
    import sys

    code = (
        "import ctypes as C, sys; sys.path.insert(0, %r)\n"
        "from tachyon_b200 import _lib\n"
        "lib = _lib.load(); n = C.c_int(-1); h = C.c_void_p()\n"
        "a = lib.tb_devices(C.byref(n)); m1 = lib.tb_last_error().decode()\n"
        "b = lib.tb_context_new(0, C.byref(h)); m2 = lib.tb_last_error().decode()\n"
        "print(a, b, n.value, h.value, 'TACHYON_LIBCUDA' in m1 and 'TACHYON_LIBCUDA' in m2)\n"
    ) % os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, TACHYON_LIBCUDA="/nonexistent/libcuda.so.1")
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, timeout=120)
    assert out.returncode == 0, out.stderr[-1500:]
    assert out.stdout.split() == ["1", "1", "0", "None", "True"], out.stdout
