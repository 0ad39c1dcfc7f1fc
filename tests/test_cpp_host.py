"""The C++ host mirror (include/smeg.hpp) above the C ABI: compiled against the in-tree library and run for everything that
needs no GPU -- IEEE conversions against numpy, parameter checks with the reference's messages, the epilogue builder (call
order, trailing activation, scalars rounded to T, resolve, validate), the gate/up interleave against the Python mirror, and
the error path of a failing library call.  The program's `gpu` mode (closed-form products through the same classes) is for a
machine with a B200."""
import os
import subprocess

import numpy as np
import pytest

import sme_gemm_b200 as sg

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def program(tmp_path_factory):
    sg.lib()                                               # the library is built
    out = tmp_path_factory.mktemp("cpp") / "host_mirror_check"
    libdir = os.path.dirname(sg.LIB_PATH)
    cmd = ["g++", "-std=c++17", "-O1", "-Wall", "-Wextra", "-Werror", "-I", os.path.join(ROOT, "include"),
           os.path.join(ROOT, "tests", "cpp", "host_mirror_check.cc"), "-L", libdir, "-lsmeg_b200", f"-Wl,-rpath,{libdir}",
           "-o", str(out)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-4000:]
    return str(out)


def test_cpp_mirror_host_side(program, tmp_path):
    rng = np.random.default_rng(3)
    edge = np.array([0.0, -0.0, 1.0, -1.0, 65504.0, 65519.9, 65520.0, 65536.0, 1e9, -1e9, np.inf, -np.inf, np.nan,
                     2.0 ** -24, 2.0 ** -25, 2.0 ** -25 * 1.0001, 2.0 ** -26, 2.0 ** -14, 2.0 ** -14 * 0.9999, 6.1e-5, 5.96e-8,
                     0.1, 0.2, 1.0 / 3.0, 1e-40, 3.3895314e38], np.float32)
    bits = rng.integers(0, 1 << 32, 200000, dtype=np.uint64).astype(np.uint32).view(np.float32)
    near = (rng.standard_normal(100000) * np.exp(rng.uniform(-20, 12, 100000))).astype(np.float32)
    xs = np.concatenate([edge, bits, near]).astype(np.float32)
    xs.tofile(tmp_path / "in.f32")
    r = subprocess.run([program, "cpu", str(tmp_path / "in.f32"), str(tmp_path)], capture_output=True, text=True)
    assert r.returncode == 0 and "CPU CHECKS OK" in r.stdout, r.stdout[-3000:] + r.stderr[-1000:]
    # conversions: crate `half` semantics = numpy's
    widened = np.fromfile(tmp_path / "f16_to_f32.bin", np.float32)
    want = np.arange(65536, dtype=np.uint16).view(np.float16).astype(np.float32)
    assert np.array_equal(widened.view(np.uint32)[~np.isnan(want)], want.view(np.uint32)[~np.isnan(want)])
    assert np.isnan(widened[np.isnan(want)]).all()
    with np.errstate(over="ignore", invalid="ignore"):
        want16 = xs.astype(np.float16)
    got16 = np.fromfile(tmp_path / "f32_to_f16.bin", np.uint16).view(np.float16)
    ok = ~np.isnan(want16)
    assert np.array_equal(got16.view(np.uint16)[ok], want16.view(np.uint16)[ok]) and np.isnan(got16[~ok]).all()
    u = xs.view(np.uint32).astype(np.uint64)
    wantb = (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16)
    gotb = np.fromfile(tmp_path / "f32_to_bf16.bin", np.uint16)
    finite = ~np.isnan(xs)
    assert np.array_equal(gotb[finite], wantb[finite])
    assert (((gotb[~finite] & 0x7F80) == 0x7F80) & ((gotb[~finite] & 0x007F) != 0)).all()          # NaN stays NaN
    # interleave == the Python mirror's
    n, k = 70, 5
    g = np.arange(n * k, dtype=np.float32)
    up = -g - 1.0
    for name, layout in (("outin", sg.WeightLayout.OutIn), ("inout", sg.WeightLayout.InOut)):
        got = np.fromfile(tmp_path / f"interleave_{name}.bin", np.float32).reshape(k, 2 * n)
        assert np.array_equal(got, sg.interleave_gate_up(g, up, layout, n, k))


def test_cpp_mirror_reports_a_failing_library_call(program):
    """Without a usable device the library returns a non-zero code and the mirror throws: no CPU fallback behind it.
    (On a machine with a B200 the same mode runs the closed-form products instead.)"""
    import torch
    if torch.cuda.is_available():
        pytest.skip("needs a machine without a GPU")
    r = subprocess.run([program, "gpu"], capture_output=True, text=True)
    assert r.returncode == 3
    assert "smeg_q4_create failed with rc -" in r.stdout
