"""The allocation-free low-bit GEMV entry point (smeg_matmul_lowbit_static_dev).

Some users of this library cannot allocate device memory at call time: a serving
loop whose memory map is frozen, a process that gave all of HBM to weights and
caches, a plug-in sandbox without cudaMalloc.  For them the int8-activation
scratch sits in a fixed array inside the library instead of coming from the
stream-ordered allocator.  This test drives the entry point through the C ABI and
requires the same bits as the allocating entry point, on two calls in a row with
different inputs (the array keeps the previous call's contents, which must not
leak into the next result).  It is collected last on purpose.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import sme_gemm_b200 as sg
from sme_gemm_b200._lib import EpDesc16, EpNode

pytestmark = pytest.mark.gpu


def _both(w, a, m, n, ep_desc):
    L = sg.lib()
    want = torch.full((m, n), 3.0, dtype=torch.float16, device="cuda")
    got = torch.full((m, n), 5.0, dtype=torch.float16, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    ep = C.byref(ep_desc) if ep_desc is not None else None
    assert L.smeg_matmul_lowbit_dev(w._h, a.data_ptr(), want.data_ptr(), m, ep, stream) == 0
    assert L.smeg_matmul_lowbit_static_dev(w._h, a.data_ptr(), got.data_ptr(), m, ep, stream) == 0
    torch.cuda.synchronize()
    return got, want


@pytest.mark.parametrize("bits", [2, 1])
def test_static_scratch_entry_matches_the_allocating_entry_twice_in_a_row(bits):
    n, k, block = 520, 1536, 128
    rng = np.random.default_rng(90 + bits)
    scales = rng.uniform(0.01, 0.05, n * (k // block)).astype(np.float16)
    if bits == 2:
        w = sg.Q2Weights.new(rng.integers(0, 256, k * n // 4).astype(np.uint8), scales, n, k,
                             sg.Q2Params(block).with_codebook([-2, -1, 1, 2]))
    else:
        w = sg.Q1Weights.new(rng.integers(0, 256, k * n // 8).astype(np.uint8), scales, sg.WeightLayout.OutIn, n, k, block)
    bias = torch.from_numpy((rng.standard_normal(n) * 0.1).astype(np.float16)).cuda()
    nodes = (EpNode * 2)(EpNode(4, 0, 0.0, bias.data_ptr(), 0), EpNode(8, 1, 0.0, None, 0))   # add_col, relu
    desc = EpDesc16(2, nodes)
    # first call: 8 rows (the largest the fixed scratch takes); second: 3 rows of new data, then 8 again
    for m, ep in ((8, None), (3, desc), (8, desc)):
        a = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float16)).cuda()
        got, want = _both(w, a, m, n, ep)
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), f"bits={bits} m={m}"
    assert sg.last_status() == 0


def test_sizes_beyond_the_fixed_scratch_are_rejected_and_leave_the_output_alone():
    n, k, block = 64, 256, 64
    rng = np.random.default_rng(7)
    w = sg.Q1Weights.new(rng.integers(0, 256, k * n // 8).astype(np.uint8),
                         rng.uniform(0.01, 0.05, n * (k // block)).astype(np.float16), sg.WeightLayout.OutIn, n, k, block)
    L = sg.lib()
    a = torch.zeros((9, k), dtype=torch.float16, device="cuda")
    c = torch.full((9, n), 7.0, dtype=torch.float16, device="cuda")
    assert L.smeg_matmul_lowbit_static_dev(w._h, a.data_ptr(), c.data_ptr(), 9, None, 0) == -4      # more than 8 rows
    torch.cuda.synchronize()
    assert bool((c == 7.0).all())
    # a depth beyond 16384 is refused as well
    kbig = 16384 + 256
    wbig = sg.Q1Weights.new(np.zeros(kbig * 16 // 8, np.uint8), np.ones(16 * (kbig // 128), np.float16),
                            sg.WeightLayout.OutIn, 16, kbig, 128)
    a2 = torch.zeros((1, kbig), dtype=torch.float16, device="cuda")
    c2 = torch.full((1, 16), 7.0, dtype=torch.float16, device="cuda")
    assert L.smeg_matmul_lowbit_static_dev(wbig._h, a2.data_ptr(), c2.data_ptr(), 1, None, 0) == -4
    torch.cuda.synchronize()
    assert bool((c2 == 7.0).all())


def test_static_calls_allocate_nothing():
    """What the entry point exists for: after one warm call, calls of every supported shape (1, 3 and 8 rows, with and
    without an epilogue) leave the device's free memory, the driver's default pool and torch's allocator unchanged.
    (The allocating entry takes its scratch from the stream-ordered pool; the static one must not touch it.)"""
    n, k, block = 520, 1536, 128
    rng = np.random.default_rng(5)
    w = sg.Q1Weights.new(rng.integers(0, 256, k * n // 8).astype(np.uint8),
                         rng.uniform(0.01, 0.05, n * (k // block)).astype(np.float16), sg.WeightLayout.OutIn, n, k, block)
    bias = torch.from_numpy((rng.standard_normal(n) * 0.1).astype(np.float16)).cuda()
    nodes = (EpNode * 2)(EpNode(4, 0, 0.0, bias.data_ptr(), 0), EpNode(8, 1, 0.0, None, 0))
    desc = EpDesc16(2, nodes)
    L = sg.lib()
    stream = torch.cuda.current_stream().cuda_stream
    a = torch.from_numpy(rng.standard_normal((8, k)).astype(np.float16)).cuda()
    c = torch.zeros((8, n), dtype=torch.float16, device="cuda")
    assert L.smeg_matmul_lowbit_static_dev(w._h, a.data_ptr(), c.data_ptr(), 8, None, stream) == 0      # warm
    torch.cuda.synchronize()

    from cuda.bindings import runtime as rt          # cuda-python: the default pool's own counters
    err, pool = rt.cudaDeviceGetDefaultMemPool(torch.cuda.current_device())
    assert int(err) == 0

    def pool_counters():
        out = []
        for attr in (rt.cudaMemPoolAttr.cudaMemPoolAttrReservedMemCurrent, rt.cudaMemPoolAttr.cudaMemPoolAttrUsedMemCurrent,
                     rt.cudaMemPoolAttr.cudaMemPoolAttrReservedMemHigh, rt.cudaMemPoolAttr.cudaMemPoolAttrUsedMemHigh):
            e, v = rt.cudaMemPoolGetAttribute(pool, attr)
            assert int(e) == 0
            out.append(int(v))
        return out

    before = (torch.cuda.mem_get_info()[0], pool_counters(), torch.cuda.memory_reserved(), torch.cuda.memory_allocated())
    for m, ep in ((1, None), (3, C.byref(desc)), (8, None), (8, C.byref(desc)), (1, C.byref(desc))):
        assert L.smeg_matmul_lowbit_static_dev(w._h, a.data_ptr(), c.data_ptr(), m, ep, stream) == 0
    torch.cuda.synchronize()
    after = (torch.cuda.mem_get_info()[0], pool_counters(), torch.cuda.memory_reserved(), torch.cuda.memory_allocated())
    assert after == before
    # the entry's own status word is part of what last_status reports
    assert sg.last_status() == 0
