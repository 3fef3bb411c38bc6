"""CPU-side checks of the C ABI: the library loads, exports every symbol the header declares,
and rejects bad arguments on the host before touching the device.  No compute calls here."""

import ctypes
import os
import re

import pytest

from gpu_ragged_dot_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "ragged_dot_b200.h")


@pytest.fixture(scope="module")
def lib():
    build.build_library()
    return _lib.load()


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(rd_[a-z_0-9]+)\s*\(", text)))


def test_header_symbols_all_exported(lib):
    names = declared_symbols()
    assert {"rd_gmm", "rd_tgmm", "rd_metadata", "rd_workspace_bytes", "rd_status_string",
            "rd_version", "rd_device_status"} <= set(names)
    for name in names:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"


def test_version_and_status_strings(lib):
    assert lib.rd_version() == 2
    assert _lib.status_string(0) == "ok"
    for code in range(1, 10):
        assert _lib.status_string(code) not in ("ok", "unknown status")
    assert _lib.status_string(999) == "unknown status"


def test_workspace_bytes(lib):
    n = ctypes.c_size_t(0)
    assert lib.rd_workspace_bytes(8192, 8, ctypes.byref(n)) == 0
    u = (8192 + 127) // 128 + 8
    assert n.value >= 4 * (8 + 2 * 8 + 1 + 2 * u) and n.value % 256 == 0
    assert lib.rd_workspace_bytes(-1, 8, ctypes.byref(n)) == 1
    assert lib.rd_workspace_bytes(0, 0, ctypes.byref(n)) == 0 and n.value > 0


def test_argument_validation_happens_on_the_host(lib):
    """Every call below must be refused before any CUDA work (there is no GPU here)."""
    cfg = None
    a16 = 0x1000  # fake, 16-byte aligned "pointers": never dereferenced on these paths
    gmm = lambda **kw: lib.rd_gmm(
        kw.get("x", a16), kw.get("A", a16), kw.get("gs", a16), kw.get("y", a16), kw.get("ws", a16),
        kw.get("ws_bytes", 1 << 20), kw.get("m", 128), kw.get("k", 64), kw.get("n", 64), kw.get("g", 2),
        kw.get("trans", 0), kw.get("dtype", 1), cfg, None)
    assert gmm(k=58) == 1  # k not a multiple of 8
    assert gmm(n=77) == 1
    assert gmm(m=-1) == 1
    assert gmm(dtype=7) == 2
    assert gmm(x=a16 + 2) == 3  # misaligned
    assert gmm(A=None) == 3
    assert gmm(ws_bytes=16) == 4
    assert gmm(m=0) == 0  # nothing to do
    tg = lambda **kw: lib.rd_tgmm(
        kw.get("x", a16), kw.get("d", a16), kw.get("gs", a16), kw.get("out", a16), kw.get("ws", a16),
        kw.get("ws_bytes", 1 << 20), kw.get("m", 128), kw.get("k", 64), kw.get("n", 64), kw.get("g", 2),
        kw.get("dtype", 1), cfg, None)
    assert tg(k=60) == 1
    assert tg(dtype=-1) == 2
    assert tg(out=a16 + 8) == 3
    assert tg(ws_bytes=0) == 4
    assert tg(g=0) == 0
    ts = lambda **kw: lib.rd_tgmm_strided(
        a16, a16, a16, a16, a16, 1 << 20, 128, kw.get("k", 64), 64, kw.get("g", 2), kw.get("seg", 2),
        kw.get("dtype", 1), cfg, None)
    assert ts(seg=0) == 1
    assert ts(k=60) == 1
    assert ts(dtype=2, seg=2) == 5  # the float32 kernels have no strided form
    assert ts(g=0) == 0
    pull = lambda **kw: lib.rd_ep_combine_pull(
        kw.get("routing", a16), a16, kw.get("tokens", 8), kw.get("top_k", 2), kw.get("row_bytes", 256),
        kw.get("experts", 8), kw.get("world", 2), a16, 64, kw.get("dtype", 1), kw.get("out", a16), 0, None)
    assert pull(top_k=9) == 1
    assert pull(row_bytes=250) == 1
    assert pull(experts=7) == 1
    assert pull(dtype=2) == 2
    assert pull(routing=None) == 3
    assert pull(out=a16 + 4) == 3
    assert pull(tokens=0) == 0
    f8 = lambda **kw: lib.rd_gmm_fp8(
        kw.get("x", a16), a16, kw.get("nw", 2), a16, kw.get("g2w", None), None, kw.get("y", a16), a16,
        kw.get("ws_bytes", 1 << 20), kw.get("m", 128), kw.get("k", 64), kw.get("n", 64), kw.get("g", 2), cfg, None)
    assert f8(k=24) == 1      # rows of k bytes must be multiples of 16 bytes
    assert f8(n=20) == 1
    assert f8(nw=3) == 1      # without an index there is one weight matrix per group
    assert f8(x=a16 + 4) == 3
    assert f8(ws_bytes=8) == 4
    assert f8(m=0) == 0
    assert lib.rd_metadata(a16, -1, 16, 8, None, None, None, None, None) == 1
    assert lib.rd_metadata(a16, 4, 16, 0, None, None, None, None, None) == 1
    assert lib.rd_device_status(None, None) == 3


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.load()


def test_xla_ffi_shim_compiles_on_its_own():
    """csrc/xla_ffi_shim.cc must stay a valid translation unit.  Where jaxlib's FFI headers are
    installed the handlers are compiled against them; elsewhere (as in the image this library was
    developed in) the file compiles to nothing, which still catches a broken include guard."""
    import shutil
    import subprocess

    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("no g++")
    src = os.path.join(ROOT, "gpu_ragged_dot_b200", "csrc", "xla_ffi_shim.cc")
    cmd = [gxx, "-std=c++17", "-fsyntax-only", "-I/usr/local/cuda/include", src]
    try:
        import jax  # noqa: F401

        cmd[3:3] = ["-I" + jax.ffi.include_dir()]
    except Exception:
        pass
    proc = subprocess.run(cmd, capture_output=True, text=True)
    assert proc.returncode == 0, proc.stderr
    text = open(src).read()
    assert "ffi::DataType::F32" in text and "RD_DTYPE_F32" in text  # float32 reaches the TF32 kernels


def test_probe_program_builds():
    """The stand-alone hardware probes compile for sm_100a without a GPU."""
    import os

    from gpu_ragged_dot_b200 import probe

    assert os.path.exists(probe.build_probe())
