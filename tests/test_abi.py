"""CPU-side checks of the C ABI: the library loads, exports every symbol the header declares,
and rejects bad arguments with status codes before touching the GPU."""
import ctypes
import os
import re

import pytest

from falkon_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "falkon_b200.h")


@pytest.fixture(scope="module")
def lib():
    _lib.build()
    return _lib.load()


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(flk_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(lib):
    names = declared_symbols()
    assert len(names) >= 14
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/falkon_b200.h but not exported"
    assert set(names) == set(_lib.EXPORTED_SYMBOLS)


def test_version_and_status_names(lib):
    assert lib.flk_version() >= 100
    assert lib.flk_status_name(0) == b"FLK_OK"
    assert lib.flk_status_name(-3) == b"FLK_ERR_WORKSPACE"
    assert lib.flk_status_name(-7) == b"FLK_ERR_TIMEOUT"


def test_workspace_queries_are_pure_host_arithmetic(lib):
    small = lib.flk_fdmmv_workspace_bytes(0, 0, 20000, 1000, 10, 1, 0)
    big = lib.flk_fdmmv_workspace_bytes(0, 0, 10_000_000, 50_000, 28, 1, 0)
    assert 0 < small < big < 16 * 2**30
    assert lib.flk_fmmv_workspace_bytes(0, 0, 20000, 1000, 10, 1, 0) <= small
    assert lib.flk_fdmmv_host_workspace_bytes(0, 0, 20000, 1000, 10, 1, 0) > small
    # fp64 goes to the SIMT / DMMA kernels, fp32 to the tensor-core kernels (resident operands up to d = 30,
    # K-loop variant up to d = 1024)
    assert lib.flk_uses_tensor_cores(0, 0, 28, 1, 0) == 1
    assert lib.flk_uses_tensor_cores(0, 3, 30, 4, 0) == 1
    assert lib.flk_uses_tensor_cores(0, 0, 31, 1, 0) == 1
    assert lib.flk_uses_tensor_cores(0, 0, 1024, 1, 0) == 1
    assert lib.flk_uses_tensor_cores(0, 0, 1025, 1, 0) == 0
    assert lib.flk_uses_tensor_cores(1, 0, 9, 1, 0) == 0
    assert lib.flk_uses_tensor_cores(0, 0, 28, 1, _lib.FLAG_FORCE_SIMT) == 0
    assert lib.flk_fmmv_workspace_bytes(7, 0, 10, 10, 2, 1, 0) == _lib.FLK_ERR_BAD_ARG
    assert lib.flk_fmmv_workspace_bytes(0, 9, 10, 10, 2, 1, 0) == _lib.FLK_ERR_BAD_ARG
    assert lib.flk_fmmv_workspace_bytes(0, 0, -1, 10, 2, 1, 0) == _lib.FLK_ERR_BAD_ARG


def test_host_workspace_covers_the_shorter_last_chunk(lib):
    """The host-buffer entry points stage the operands and run the product in row chunks inside one workspace.  A
    product's workspace is not monotonic in its row count, so the part left after the staged operands must hold the
    need of BOTH chunk lengths (1,250,000 rows in eight chunks used to size it for the full chunk only, and the
    shorter last chunk asked for 11 MB more)."""
    pad = lambda b: -(-max(b, 1) // 256) * 256
    m, d, t = 50_000, 28, 1
    for n in (1_250_000, 2_500_000, 5_000_000, 10_000_000, 3_333_333, 400_001, 131_072 * 3 + 17):
        chunks = max(1, min(8, n // 131_072))
        chunk_rows = -(-(-(-n // chunks)) // 512) * 512
        n_chunks = -(-n // chunk_rows)
        last = n - (n_chunks - 1) * chunk_rows
        total = lib.flk_fdmmv_host_workspace_bytes(0, 0, n, m, d, t, 0)
        staged = pad(n * d * 4) + pad(m * d * 4) + pad(m * t * 4) + pad(n * t * 4) + pad(m * t * 4)
        inner = total - staged
        for rows in {min(n, chunk_rows), last}:
            assert inner >= lib.flk_fdmmv_workspace_bytes(0, 0, rows, m, d, t, 0), (n, rows)


def test_argument_errors_return_status_codes(lib):
    sig = (ctypes.c_double * 1)(1.0)
    dummy = ctypes.c_void_p(4096)
    # null X1
    st = lib.flk_fmmv(0, 0, None, 10, 4, 1, dummy, 5, 4, 1, 4, dummy, 1, 1, 1, dummy, 1, 1, sig, 1, dummy, 1 << 30, 0, None)
    assert st == _lib.FLK_ERR_BAD_ARG and b"X1" in lib.flk_last_error()
    # neither stride is 1
    st = lib.flk_fmmv(0, 0, dummy, 10, 8, 2, dummy, 5, 4, 1, 4, dummy, 1, 1, 1, dummy, 1, 1, sig, 1, dummy, 1 << 30, 0, None)
    assert st == _lib.FLK_ERR_LAYOUT
    # sigma of the wrong length
    st = lib.flk_fmmv(0, 0, dummy, 10, 4, 1, dummy, 5, 4, 1, 4, dummy, 1, 1, 1, dummy, 1, 1, sig, 3, dummy, 1 << 30, 0, None)
    assert st == _lib.FLK_ERR_BAD_ARG
    # missing / undersized / misaligned workspace
    st = lib.flk_fmmv(0, 0, dummy, 10, 4, 1, dummy, 5, 4, 1, 4, dummy, 1, 1, 1, dummy, 1, 1, sig, 1, None, 0, 0, None)
    assert st == _lib.FLK_ERR_WORKSPACE
    st = lib.flk_fmmv(0, 0, dummy, 10, 4, 1, dummy, 5, 4, 1, 4, dummy, 1, 1, 1, dummy, 1, 1, sig, 1, dummy, 16, 0, None)
    assert st == _lib.FLK_ERR_WORKSPACE
    st = lib.flk_fmmv(0, 0, dummy, 10, 4, 1, dummy, 5, 4, 1, 4, dummy, 1, 1, 1, dummy, 1, 1, sig, 1, ctypes.c_void_p(4100), 1 << 30, 0, None)
    assert st == _lib.FLK_ERR_WORKSPACE
    # fdmmv without v and w
    st = lib.flk_fdmmv(0, 0, dummy, 10, 4, 1, dummy, 5, 4, 1, 4, None, 0, 0, None, 0, 0, 1, dummy, 1, 1, sig, 1, dummy, 1 << 30, 0, None)
    assert st == _lib.FLK_ERR_BAD_ARG
    # forcing the tensor-core kernel where it does not apply
    st = lib.flk_fmmv(1, 0, dummy, 10, 4, 1, dummy, 5, 4, 1, 4, dummy, 1, 1, 1, dummy, 1, 1, sig, 1, dummy, 1 << 30, _lib.FLAG_FORCE_TC, None)
    assert st == _lib.FLK_ERR_UNSUPPORTED


def test_kernel_matrix_entry_point_checks_arguments(lib):
    sig = (ctypes.c_double * 1)(1.0)
    dummy = ctypes.c_void_p(4096)
    need = lib.flk_fmm_workspace_bytes(0, 1000, 500, 10, 0)
    need64 = lib.flk_fmm_workspace_bytes(0, 1000, 500, 10, _lib.FLAG_FP64_MATH)
    assert 0 < need < need64  # fp64 arithmetic on fp32 data needs fp64 operand copies
    assert lib.flk_fmm_workspace_bytes(1, 1000, 500, 10, 0) == need64
    st = lib.flk_fmm(0, 0, None, 10, 4, 1, dummy, 5, 4, 1, 4, dummy, 5, 1, sig, 1, dummy, 1 << 30, 0, None)
    assert st == _lib.FLK_ERR_BAD_ARG and b"X1" in lib.flk_last_error()
    st = lib.flk_fmm(0, 0, dummy, 10, 4, 1, dummy, 5, 4, 1, 4, dummy, 7, 3, sig, 1, dummy, 1 << 30, 0, None)
    assert st == _lib.FLK_ERR_LAYOUT  # out: neither stride is 1
    st = lib.flk_fmm(0, 0, dummy, 10, 4, 1, dummy, 5, 4, 1, 4, dummy, 5, 1, sig, 1, dummy, 16, 0, None)
    assert st == _lib.FLK_ERR_WORKSPACE
    st = lib.flk_fmm(0, 5, dummy, 10, 4, 1, dummy, 5, 4, 1, 4, dummy, 5, 1, sig, 1, dummy, 1 << 30, 0, None)
    assert st == _lib.FLK_ERR_BAD_ARG  # unknown kernel id


def test_kgrad_argument_checks(lib):
    """flk_kgrad validates before touching the device: the checks run without a GPU."""
    dummy = ctypes.c_void_p(4096)
    sig = (ctypes.c_double * 1)(1.0)
    big = 1 << 30

    def call(X1=dummy, n=10, G=dummy, g_rs=2, g_cs=1, v=dummy, t=2, out_rs=5, out_cs=1, ws=dummy, ws_bytes=big,
             kernel=0):
        return lib.flk_kgrad(0, kernel, X1, n, 4, 1, dummy, 5, 4, 1, 4, G, g_rs, g_cs, v, t, 2, 1, dummy, out_rs,
                             out_cs, sig, 1, ws, ws_bytes, 0, None)

    assert call(X1=None) == _lib.FLK_ERR_BAD_ARG
    assert call(G=None) == _lib.FLK_ERR_BAD_ARG
    assert call(v=None) == _lib.FLK_ERR_BAD_ARG           # t > 0 needs the second factor
    assert call(t=0) == _lib.FLK_ERR_BAD_ARG              # t == 0 means "G is n x m": v must be NULL
    assert call(t=-1) == _lib.FLK_ERR_BAD_ARG
    assert call(g_rs=3, g_cs=2) == _lib.FLK_ERR_LAYOUT
    assert call(out_rs=7, out_cs=3) == _lib.FLK_ERR_LAYOUT
    assert call(ws_bytes=16) == _lib.FLK_ERR_WORKSPACE
    assert call(kernel=4) == _lib.FLK_ERR_BAD_ARG
    assert call(n=64 * 65535 + 1) == _lib.FLK_ERR_UNSUPPORTED
    assert b"split the rows" in lib.flk_last_error()


def test_plain_c_client(lib, tmp_path):
    """The boundary is usable from C with nothing but the header and the shared library."""
    import shutil
    import subprocess

    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    libdir = os.path.dirname(_lib.LIB_PATH)
    exe = str(tmp_path / "abi_client")
    cmd = [gcc, "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"),
           os.path.join(ROOT, "tests", "abi_client.c"), "-o", exe, "-L", libdir, "-lfalkon_b200",
           "-Wl,-rpath," + libdir]
    subprocess.run(cmd, check=True, capture_output=True, text=True)
    res = subprocess.run([exe], capture_output=True, text=True)
    assert res.returncode == 0 and res.stdout.startswith("ok"), res.stdout + res.stderr


def test_status_maps_to_reference_exception_types(lib):
    lib.flk_fmmv_workspace_bytes(0, 0, -1, 10, 2, 1, 0)
    with pytest.raises(ValueError):
        _lib.raise_for_status(_lib.FLK_ERR_BAD_ARG)
    with pytest.raises(ValueError):
        _lib.raise_for_status(_lib.FLK_ERR_LAYOUT)
    with pytest.raises(MemoryError):
        _lib.raise_for_status(_lib.FLK_ERR_WORKSPACE)
    with pytest.raises(NotImplementedError):
        _lib.raise_for_status(_lib.FLK_ERR_UNSUPPORTED)
    with pytest.raises(RuntimeError):
        _lib.raise_for_status(_lib.FLK_ERR_CUDA)


def test_register_report_parser_and_guard():
    """The build reads `ptxas -v` and refuses a tensor-core sweep that spills or whose launch register count is not
    the one its register re-partitioning assumes (falkon_b200/_lib.py: parse_ptxas, check_ptxas)."""
    from falkon_b200 import _lib

    def entry(mangled, stack, st, ld, regs):
        return (f"ptxas info    : Compiling entry function '{mangled}' for 'sm_100a'\n"
                f"ptxas info    : Function properties for {mangled}\n"
                f"    {stack} bytes stack frame, {st} bytes spill stores, {ld} bytes spill loads\n"
                f"ptxas info    : Used {regs} registers, used 1 barriers, 16 bytes smem\n")

    tc = "_ZN3flk2tc13kmv_tc_kernelILi0ELi3ELi1ELb1EEEvNS0_9SweepArgsE"
    tck = "_ZN3flk3tck14kmv_tck_kernelILi0ELi1ELi2EEEvNS0_10SweepArgsLE"
    tck_wide = "_ZN3flk3tck14kmv_tck_kernelILi0ELi32ELi0EEEvNS0_10SweepArgsLE"
    good = _lib.parse_ptxas(entry(tc, 0, 0, 0, 80) + entry(tck, 0, 0, 0, 96) + entry(tck_wide, 8, 8, 16, 96))
    assert len(good) == 3 and _lib.check_ptxas(good) == []
    assert any("spill" in p for p in _lib.check_ptxas(_lib.parse_ptxas(entry(tc, 8, 4, 4, 80))))
    assert any("registers per thread" in p for p in _lib.check_ptxas(_lib.parse_ptxas(entry(tc, 0, 0, 0, 72))))
    assert any("allowance" in p for p in _lib.check_ptxas(_lib.parse_ptxas(entry(tc, 0, 0, 0, 80) + entry(tck_wide, 64, 80, 200, 96))))
    assert any("no tc::kmv_tc_kernel" in p for p in _lib.check_ptxas(_lib.parse_ptxas(entry(tck, 0, 0, 0, 96))))
    # the library on disk was built under the same guard: its report has no offending row
    import os

    if os.path.exists(_lib.PTXAS_REPORT):
        rows = [l.split(" | ") for l in open(_lib.PTXAS_REPORT).read().splitlines()[2:]]
        tc_rows = [r for r in rows if "tc::kmv_tc_kernel" in r[0]]
        assert tc_rows and all(r[1] == "80" and r[3] == "0" and r[4] == "0" for r in tc_rows)
