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


def _attn_oracle(orc, x16, wq, wo, heads, kv_heads, hd, m, d):
    """One prefill block of m rows through the oracle: Q4 [q | k | v] projection, causal attention, f16 rounding, and the
    out projection's un-rounded f32 sums."""
    n = (heads + 2 * kv_heads) * hd
    qq, qs, _ = orc.q4_quantize(wq, 0, n, d)
    oq, os_, _ = orc.q4_quantize(wo, 0, wo.shape[0], heads * hd)
    qkv = orc.matmul_q4(x16, qq, qs, None, n, d, 32, m).reshape(m, n)                     # f16 bits
    q_len, kv_len = heads * hd, kv_heads * hd
    q = orc.f16_bits_to_f32(np.ascontiguousarray(qkv[:, :q_len]))
    k, v = np.ascontiguousarray(qkv[:, q_len:q_len + kv_len]), np.ascontiguousarray(qkv[:, q_len + kv_len:])
    att = orc.attention_kv_causal(q, k, v, 0, m, heads, kv_heads, hd, float(np.float32(1.0) / np.sqrt(np.float32(hd))))
    att16 = orc.f32_to_f16_bits(att)
    return qkv, orc.gemm16_f32(att16, orc.q4_dequant(oq, os_, None, wo.shape[0], heads * hd), m, wo.shape[0], heads * hd)


def _attn_rank_main(rank, world, port, shape, out_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle as orc
    from sme_gemm_b200.tp import shard_attention_weights, shard_heads
    d, heads, kv_heads, hd, m = shape
    rng = np.random.default_rng(78)
    wq = (rng.standard_normal(((heads + 2 * kv_heads) * hd, d)) * 0.08).astype(np.float32)
    wo = (rng.standard_normal((d, heads * hd)) * 0.08).astype(np.float32)
    x16 = rng.standard_normal((m, d)).astype(np.float16)
    _, hl, _, kvl = shard_heads(heads, kv_heads, rank, world)
    sq, so = shard_attention_weights(wq, wo, heads, kv_heads, hd, rank, world)
    qkv, part = _attn_oracle(orc, x16, sq, so, hl, kvl, hd, m, d)
    t = torch.from_numpy(part)
    dist.all_reduce(t)
    np.save(os.path.join(out_dir, f"sum{rank}.npy"), t.numpy())
    np.save(os.path.join(out_dir, f"qkv{rank}.npy"), qkv)
    dist.destroy_process_group()


def test_two_gloo_ranks_of_head_sharded_attention_match_the_unsharded_block(tmp_path):
    """Attention split by heads: a rank's projected q / k / v columns are the unsharded block's bit for bit (whole rows of
    the fused projection), its heads attend independently, and the out projection's f32 partials summed over the ranks
    differ from the one-rank sum by summation order only."""
    sys.path.insert(0, ROOT)
    import oracle as orc
    from sme_gemm_b200.tp import shard_heads
    world = 2
    d, heads, kv_heads, hd, m = 64, 8, 4, 16, 5
    port = 31500 + os.getpid() % 2000
    mp.spawn(_attn_rank_main, args=(world, port, (d, heads, kv_heads, hd, m), str(tmp_path)), nprocs=world, join=True)
    rng = np.random.default_rng(78)
    wq = (rng.standard_normal(((heads + 2 * kv_heads) * hd, d)) * 0.08).astype(np.float32)
    wo = (rng.standard_normal((d, heads * hd)) * 0.08).astype(np.float32)
    x16 = rng.standard_normal((m, d)).astype(np.float16)
    qkv, want = _attn_oracle(orc, x16, wq, wo, heads, kv_heads, hd, m, d)
    sums = [np.load(tmp_path / f"sum{r}.npy") for r in range(world)]
    assert np.array_equal(sums[0], sums[1])
    q_len, kv_len = heads * hd, kv_heads * hd
    for r in range(world):
        h0, hl, kv0, kvl = shard_heads(heads, kv_heads, r, world)
        got = np.load(tmp_path / f"qkv{r}.npy")
        assert np.array_equal(got[:, :hl * hd], qkv[:, h0 * hd:(h0 + hl) * hd])
        assert np.array_equal(got[:, hl * hd:(hl + kvl) * hd], qkv[:, q_len + kv0 * hd:q_len + (kv0 + kvl) * hd])
        assert np.array_equal(got[:, (hl + kvl) * hd:], qkv[:, q_len + kv_len + kv0 * hd:q_len + kv_len + (kv0 + kvl) * hd])
    assert np.max(np.abs(sums[0] - want) / (1 + np.abs(want))) <= 1e-5


def test_shard_heads_keeps_query_groups_with_their_kv_head():
    from sme_gemm_b200.tp import shard_heads
    assert shard_heads(32, 8, 3, 4) == (24, 8, 6, 2)
    assert shard_heads(8, 8, 1, 2) == (4, 4, 4, 4)
    for heads, kv in ((32, 8), (16, 16), (8, 2)):
        for world in (1, 2):
            spans = [shard_heads(heads, kv, r, world) for r in range(world)]
            assert sum(s[1] for s in spans) == heads and sum(s[3] for s in spans) == kv
            for h0, hl, kv0, kvl in spans:
                group = heads // kv
                # query head h uses KV head h / group: a rank's query heads use exactly its KV heads
                assert h0 // group == kv0 and (h0 + hl - 1) // group == kv0 + kvl - 1
    with pytest.raises(AssertionError):
        shard_heads(8, 2, 0, 4)
