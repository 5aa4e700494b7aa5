"""Acceptance tests on the GPU with the reference's own material:
 - its unmodified host drivers (gemm/conv/capsule `*-run-fpga.cpp -DTINY`, `aot/gemm-run.cpp`),
   built here against the per-design stubs and libt2sp_b200.so by oracle/build_ref_drivers.sh
   (the binaries travel with the repository; the reference tree itself is not needed to run them);
   each validates the result with its own golden loop and prints `Success`;
 - the reference's deterministic fixtures from tests/golden/kat.npz through the C ABI;
 - device-resident buffers and the exec_time.txt report."""
import ctypes
import os
import subprocess

import numpy as np
import pytest

import t2sp_b200
from t2sp_b200 import Buffer
from tests.util import call_gemm, library_env

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
KAT = np.load(os.path.join(ROOT, "tests", "golden", "kat.npz"))


@pytest.mark.parametrize("name", ["gemm_tiny", "conv_tiny", "capsule_tiny", "aot_gemm", "oneapi_gemm_tiny", "oneapi_conv_tiny",
                                  "oneapi_capsule_tiny", "blas_sgemm_a10", "blas_ssyrk_s10", "syrk_tiny", "ger_tiny"])
def test_unmodified_reference_driver(lib, name, tmp_path):
    exe = os.path.join(ROOT, "tests", "_bin", name)
    if not os.path.exists(exe):
        pytest.skip("driver binary not built (needs the reference tree at build time)")
    res = subprocess.run([exe], capture_output=True, text=True, timeout=300, cwd=str(tmp_path))
    assert res.returncode == 0, (res.stdout[-300:], res.stderr[-500:])
    assert res.stdout.strip().splitlines()[-1].startswith("Success")
    assert "ERROR" not in res.stdout


@pytest.mark.parametrize("name", ["gemm_gpu_flow", "conv_gpu_flow", "capsule_gpu_flow", "gemm_cm_flow", "conv_cm_flow",
                                  "capsule_cm_flow"])
def test_unmodified_gpu_flow_driver(lib, name, tmp_path):
    """The reference's GPU-flow drivers (t2s/tests/performance/{gemm,conv,capsule}/*-run-gpu.cpp, -DITER=1),
    written against util/l0_rt_helpers.h: built with include/l0/l0_rt_helpers.h in its place; and their CM-runtime
    twins (*-run-gpu-cm.cpp), built with include/cm/ in place of the CM runtime headers. Each checks the
    plain 2-D result of the GPU design's size with its own golden loop and prints `Pass!`."""
    exe = os.path.join(ROOT, "tests", "_bin", name)
    if not os.path.exists(exe):
        pytest.skip("driver binary not built (needs the reference tree at build time)")
    res = subprocess.run([exe], capture_output=True, text=True, timeout=600, cwd=str(tmp_path))
    assert res.returncode == 0, (res.stdout[-300:], res.stderr[-500:])
    assert res.stdout.strip().splitlines()[-1].startswith("Pass")


def test_runtime_buffer_class_through_the_device_interface(lib, tmp_path):
    """tests/drivers/runtime_buffer_flow.cpp: a caller that holds Halide::Runtime::Buffer objects, as the
    reference's hosts do. The class calls through buffer.device_interface (copy_to_host, crops, slices,
    device_free in the destructor: HalideBuffer.h:229-252,388,418,1615), so the interface must be the
    real 15-entry function table of HalideRuntime.h:713-738."""
    exe = os.path.join(ROOT, "tests", "_bin", "runtime_buffer_flow")
    if not os.path.exists(exe):
        pytest.skip("driver binary not built (needs the reference tree's HalideBuffer.h at build time)")
    res = subprocess.run([exe], capture_output=True, text=True, timeout=300, cwd=str(tmp_path))
    assert res.returncode == 0, (res.stdout[-600:], res.stderr[-500:])
    assert res.stdout.strip().splitlines()[-1].startswith("Success")


@pytest.mark.parametrize("name", ["gemm_large_a10", "conv_large_a10", "capsule_large_a10"])
def test_large_mode_driver_reports_throughput_and_roofline(lib, name, tmp_path):
    """The reference's drivers in performance mode (no -DTINY: A10 design constants, e.g. a
    10240 x 8192 x 16384 GEMM): after the run they read exec_time.txt back through ExecTime(), print a
    GFlops line and call roofline(), which writes roofline.png (gemm-run-fpga.cpp:88-108); here those
    helpers are csrc/roofline_shim.cpp."""
    exe = os.path.join(ROOT, "tests", "_bin", name)
    if not os.path.exists(exe):
        pytest.skip("driver binary not built (needs the reference tree at build time)")
    env = dict(os.environ, BITSTREAM=str(tmp_path / "a.aocx"))
    res = subprocess.run([exe], capture_output=True, text=True, timeout=900, cwd=str(tmp_path), env=env)
    assert res.returncode == 0, (res.stdout[-600:], res.stderr[-500:])
    assert "GFlops" in res.stdout, res.stdout[-600:]
    png = tmp_path / "roofline.png"
    assert png.exists() and png.stat().st_size > 100 and png.read_bytes()[:8] == b"\x89PNG\r\n\x1a\n"
    assert (tmp_path / "exec_time.txt").exists()


def test_golden_aot_gemm_fixture(lib):
    a, b, exact = KAT["aot_gemm_a"], KAT["aot_gemm_b"], KAT["aot_gemm_c_exact"].astype(np.float64)
    rc, C6 = call_gemm(a, b, "f32", tiled=(4, 2, 4, 4))
    assert rc == 0
    # undo the tiling: element (jjj,iii,jj,ii,j,i) holds C[iii + 2*ii + 8*i, jjj + 4*jj + 16*j]
    C = C6.transpose(0, 2, 4, 1, 3, 5).reshape(16, 32)
    nz = np.abs(exact) > 0
    assert np.all(np.abs(C.astype(np.float64) - exact)[nz] < 0.005 * np.abs(exact)[nz])   # aot/gemm-run.cpp:78
    assert np.max(np.abs(C - exact)) / np.max(np.abs(exact)) < 1e-5


def test_golden_sequential_fixtures_exact(lib):
    rc, C = call_gemm(KAT["seq_gemm_a"], KAT["seq_gemm_b"], "f32")
    assert rc == 0 and np.array_equal(C, KAT["seq_gemm_c_exact"].astype(np.float32))
    c = np.zeros((8, 8, 8), np.float32)
    cb = Buffer.from_numpy(c)
    assert t2sp_b200.ttm(Buffer.from_numpy(KAT["seq_ttm_a"]), Buffer.from_numpy(KAT["seq_ttm_b"]), cb) == 0
    assert np.array_equal(cb.keepalive, KAT["seq_ttm_c_exact"].astype(np.float32))
    d = np.zeros((8, 8), np.float32)
    db = Buffer.from_numpy(d)
    assert t2sp_b200.mttkrp(Buffer.from_numpy(KAT["seq_mttkrp_a"]), Buffer.from_numpy(KAT["seq_mttkrp_b"]),
                            Buffer.from_numpy(KAT["seq_mttkrp_c"]), db) == 0
    assert np.array_equal(db.keepalive, KAT["seq_mttkrp_d_exact"].astype(np.float32))


def test_device_resident_buffers_and_exec_time(lib, tmp_path):
    """halide_device_malloc / copy_to_device / copy_to_host protocol: inputs copied once, the
    result stays on the device until asked for; exec_time.txt is written like the reference's."""
    M = N = K = 256
    A = (np.arange(M * K) % 7 - 3).astype(np.float32).reshape(M, K)
    B = (np.arange(K * N) % 5 - 2).astype(np.float32).reshape(K, N)
    C = np.zeros((M, N), np.float32)
    a, b, c = Buffer.from_numpy(A), Buffer.from_numpy(B), Buffer.from_numpy(C)
    for x in (a, b):
        assert lib.t2sp_b200_copy_to_device(x.ptr) == 0
    assert lib.t2sp_b200_device_malloc(c.ptr) == 0
    with library_env(T2SP_B200_EXEC_TIME_FILE=str(tmp_path / "exec_time.txt")):
        assert t2sp_b200.gemm(a, b, c) == 0
    assert c.raw.flags & 2 and not np.any(C)              # device_dirty set, host copy untouched
    assert lib.t2sp_b200_copy_to_host(c.ptr) == 0
    assert np.array_equal(c.keepalive, (A.astype(np.float64) @ B.astype(np.float64)).astype(np.float32))
    lines = (tmp_path / "exec_time.txt").read_text().split()
    assert float(lines[0]) > 0 and "kernel_unloader" in lines
    assert lib.t2sp_b200_last_kernel_ns() > 0
    for x in (a, b, c):
        assert lib.t2sp_b200_device_free(x.ptr) == 0 and x.raw.device == 0


def test_injected_allocation_failure_is_an_error_code(lib):
    A = np.ones((512, 512), np.float32)
    C = np.zeros((512, 512), np.float32)
    with library_env(T2SP_B200_FAIL_ALLOC_ABOVE="1"):
        rc = t2sp_b200.gemm(Buffer.from_numpy(A), Buffer.from_numpy(A), Buffer.from_numpy(C))
    assert rc == -16                                       # halide_error_code_device_malloc_failed
    rc = t2sp_b200.gemm(Buffer.from_numpy(A), Buffer.from_numpy(A), Buffer.from_numpy(C))
    assert rc == 0                                         # the library stays usable


def test_unaligned_rows_are_repacked(lib):
    # TMA needs 16-byte aligned row pitches: K = 30 fp32 elements is 120 bytes, N = 66 is 264 bytes.
    # Such operands are copied once on the device into a padded scratch block and read from there.
    A = (np.arange(64 * 30) % 9 - 4).astype(np.float32).reshape(64, 30)
    B = (np.arange(30 * 66) % 7 - 3).astype(np.float32).reshape(30, 66)
    rc, C = call_gemm(A, B, "f32")
    assert rc == 0
    assert np.array_equal(C, (A.astype(np.float64) @ B.astype(np.float64)).astype(np.float32))


def test_aot_runtime_entry_points_round_trip(lib):
    """halide_device_and_host_malloc / halide_copy_to_device / halide_copy_to_host / halide_device_and_host_free
    under the reference runtime's names (t2s/src/AOT-OpenCL-Runtime.cpp:119-441)."""
    P = ctypes.c_void_p
    b = Buffer((64, 16), "f32")          # no host, no device yet
    lib.halide_device_and_host_malloc.argtypes = [P, P, P]
    lib.halide_copy_to_device.argtypes = [P, P, P]
    lib.halide_copy_to_host.argtypes = [P, P]
    lib.halide_device_and_host_free.argtypes = [P, P]
    assert lib.halide_device_and_host_malloc(None, b.ptr, None) == 0
    assert b.raw.host and b.raw.device
    host = np.ctypeslib.as_array(ctypes.cast(b.raw.host, ctypes.POINTER(ctypes.c_float)), shape=(16, 64))
    host[:] = np.arange(16 * 64, dtype=np.float32).reshape(16, 64)
    b.raw.flags |= 1                      # host_dirty
    assert lib.halide_copy_to_device(None, b.ptr, None) == 0
    host[:] = -1.0
    b.raw.flags |= 2                      # device_dirty: the device copy is the current one
    assert lib.halide_copy_to_host(None, b.ptr) == 0
    assert np.array_equal(host, np.arange(16 * 64, dtype=np.float32).reshape(16, 64))
    assert lib.halide_opencl_wait_for_kernels_finish(None) == 0
    assert lib.halide_device_and_host_free(None, b.ptr) == 0
    assert not b.raw.host and not b.raw.device
