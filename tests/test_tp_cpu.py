"""The tensor-parallel partition of the MLP block, checked on the CPU with two
gloo ranks: the host-side sharding (sme_gemm_b200.tp) feeds the ORACLE as the
compute stand-in, the ranks exchange f32 partials with one all-reduce, and the
result is compared with the unsharded oracle block."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _rank_main(rank, world, port, d, f, m, out_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle as orc
    from sme_gemm_b200.host import WeightLayout, interleave_gate_up
    from sme_gemm_b200.tp import shard_bounds, shard_weights
    rng = np.random.default_rng(77)
    wg = (rng.standard_normal((f, d)) * 0.05).astype(np.float32)
    wu = (rng.standard_normal((f, d)) * 0.05).astype(np.float32)
    wd = (rng.standard_normal((d, f)) * 0.05).astype(np.float32)
    x = rng.standard_normal((m, d)).astype(np.float16)
    y0 = rng.standard_normal((m, d)).astype(np.float32)
    lo, hi = shard_bounds(f, rank, world)
    sg_, su_, sd_ = shard_weights(wg, wu, wd, rank, world)
    fl = hi - lo
    both = interleave_gate_up(sg_, su_, WeightLayout.OutIn, fl, d)
    guq, gus, _ = orc.q4_quantize(both, 1, 2 * fl, d)
    dq, ds, _ = orc.q4_quantize(sd_, 0, d, fl)
    raw = orc.matmul_q4(x, guq, gus, None, 2 * fl, d, 32, m)
    hid = orc.glu(raw, m, fl)
    part = orc.gemm16_f32(hid, orc.q4_dequant(dq, ds, None, d, fl), m, d, fl)
    t = torch.from_numpy(part)
    dist.all_reduce(t)
    y = y0.copy()
    orc.add_f16(orc.f32_to_f16_bits(t.numpy()), y)
    np.save(os.path.join(out_dir, f"y{rank}.npy"), y)
    np.save(os.path.join(out_dir, f"hid{rank}.npy"), hid)
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2])
def test_two_gloo_ranks_match_the_unsharded_block(tmp_path, world):
    sys.path.insert(0, ROOT)
    import oracle as orc
    from sme_gemm_b200.host import WeightLayout, interleave_gate_up
    from sme_gemm_b200.tp import shard_bounds
    d, f, m = 96, 320, 3
    port = 29500 + os.getpid() % 2000
    mp.spawn(_rank_main, args=(world, port, d, f, m, str(tmp_path)), nprocs=world, join=True)
    rng = np.random.default_rng(77)
    wg = (rng.standard_normal((f, d)) * 0.05).astype(np.float32)
    wu = (rng.standard_normal((f, d)) * 0.05).astype(np.float32)
    wd = (rng.standard_normal((d, f)) * 0.05).astype(np.float32)
    x = rng.standard_normal((m, d)).astype(np.float16)
    y0 = rng.standard_normal((m, d)).astype(np.float32)
    both = interleave_gate_up(wg, wu, WeightLayout.OutIn, f, d)
    guq, gus, _ = orc.q4_quantize(both, 1, 2 * f, d)
    dq, ds, _ = orc.q4_quantize(wd, 0, d, f)
    want = y0.copy()
    orc.mlp_accumulate(x, want, m, d, f, guq, gus, dq, ds)
    hid_full = orc.glu(orc.matmul_q4(x, guq, gus, None, 2 * f, d, 32, m), m, f)
    ys = [np.load(tmp_path / f"y{r}.npy") for r in range(world)]
    assert np.array_equal(ys[0], ys[1]), "ranks disagree after the all-reduce"
    # gate/up: each rank's hidden units are bit-identical to the unsharded ones
    for r in range(world):
        lo, hi = shard_bounds(f, r, world)
        assert np.array_equal(np.load(tmp_path / f"hid{r}.npy"), hid_full[:, lo:hi])
    # down: f32 partials summed across ranks differ from one f32 K-sum only by summation order
    assert np.max(np.abs(ys[0] - want) / (1 + np.abs(want))) <= 2e-3


def test_shard_bounds_cover_every_chunk_once():
    from sme_gemm_b200.tp import shard_bounds
    for f in (14336, 320, 1024):
        for world in (1, 2, 4, 8):
            if world > f // 32:
                continue
            spans = [shard_bounds(f, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == f
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            assert all(lo % 32 == 0 and hi % 32 == 0 and hi > lo for lo, hi in spans)
    assert shard_bounds(14336, 3, 8) == (5376, 7168)
