"""The tensor-parallel finish over peer memory (smeg_mlp_reduce_finish_dev) on two or more GPUs of one box:
one kernel per rank sums the ranks' f32 partials in rank order, rounds to f16 and adds to the residual
stream.  Checked bit for bit against the same arithmetic done with an all-gather and torch adds.
Needs at least two GPUs; skipped otherwise."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

WORKER = r'''
import os, sys
import torch, torch.distributed as dist
sys.path.insert(0, os.getcwd())
import sme_gemm_b200 as sg
from sme_gemm_b200.tp import PeerReduce
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
ok = True
for (m, d) in ((1, 4096), (256, 4096), (7, 100)):
    peer = PeerReduce(m, d)
    g = torch.Generator(device="cuda").manual_seed(1234)          # same residual stream on every rank
    y = torch.randn(m, d, device="cuda", generator=g)
    for step in range(4):
        gp = torch.Generator(device="cuda").manual_seed(100 * step + rank)
        part = torch.randn(m, d, device="cuda", generator=gp) * 3.0
        peer.partial.copy_(part)
        parts = [torch.empty_like(part) for _ in range(world)]
        dist.all_gather(parts, part)
        total = parts[0].clone()
        for s in range(1, world):
            total = total + parts[s]
        want = y + total.half().float()
        peer.finish(y)
        torch.cuda.synchronize()
        if sg.last_status() != 0 or not torch.equal(y, want):
            ok = False
            print(f"rank {rank}: mismatch at m={m} d={d} step {step}: status {sg.last_status()}, "
                  f"max diff {(y - want).abs().max().item()}", flush=True)
        y = want.clone()
    dist.barrier()
flag = torch.tensor([1 if ok else 0], device="cuda")
dist.all_reduce(flag, op=dist.ReduceOp.MIN)
if rank == 0:
    print("PEER_REDUCE_OK" if int(flag.item()) == 1 else "PEER_REDUCE_FAILED", flush=True)
dist.destroy_process_group()
'''


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs on one box")
def test_peer_reduce_finish_equals_gathered_sum_bit_for_bit(tmp_path):
    world = min(torch.cuda.device_count(), 8)
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                          "--master-addr", "127.0.0.1", "--master-port", "29731", str(script)],
                         capture_output=True, text=True, timeout=280, env=env, cwd=os.getcwd())
    assert "PEER_REDUCE_OK" in out.stdout, out.stdout[-2000:] + out.stderr[-2000:]


WORKER_MLP = r'''
import os, sys
import numpy as np
import torch, torch.distributed as dist
sys.path.insert(0, os.getcwd())
import sme_gemm_b200 as sg
from sme_gemm_b200.tp import PeerReduce, TpMlp
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
d, f = 512, 2048
rng = np.random.default_rng(9)
wg = (rng.standard_normal((f, d)) * 0.05).astype(np.float32)
wu = (rng.standard_normal((f, d)) * 0.05).astype(np.float32)
wd = (rng.standard_normal((d, f)) * 0.05).astype(np.float32)
whole = sg.Mlp.gated(sg.GatedLinear.quantize(wg, wu, sg.WeightLayout.OutIn, f, d, sg.Gate.Silu),
                     sg.Linear.quantize(wd, sg.WeightLayout.OutIn, d, f))
ok = True
for m in (1, 3, 200):
    tp = TpMlp.quantize(wg, wu, wd, rank, world)
    tp.peer = PeerReduce(m, d)
    x = torch.from_numpy(rng.standard_normal((m, d)).astype(np.float16)).cuda()
    y0 = torch.from_numpy(rng.standard_normal((m, d)).astype(np.float32)).cuda()
    for step in range(3):
        y = y0.clone()
        tp.accumulate(x, y, m)
        want = y0.clone()
        whole.accumulate(x, want, m)          # the unsharded block on this GPU
        torch.cuda.synchronize()
        rel = float(((y - want).abs() / (1 + want.abs())).max().item())
        # every rank holds the same bits
        bits = y.view(torch.int32).to(torch.int64).sum().reshape(1)
        lo, hi = bits.clone(), bits.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN); dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        if sg.last_status() != 0 or rel > 1e-2 or int(lo.item()) != int(hi.item()):
            ok = False
            print(f"rank {rank}: m={m} step {step}: max_rel {rel}, identical {int(lo.item()) == int(hi.item())}", flush=True)
    dist.barrier()
flag = torch.tensor([1 if ok else 0], device="cuda")
dist.all_reduce(flag, op=dist.ReduceOp.MIN)
if rank == 0:
    print("TP_MLP_OK" if int(flag.item()) == 1 else "TP_MLP_FAILED", flush=True)
dist.destroy_process_group()
'''


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs on one box")
def test_sharded_mlp_with_peer_reduce_matches_the_unsharded_block(tmp_path):
    """The whole tensor-parallel block -- sharded GEMMs, sum over peer memory, rounding, residual add -- against the
    one-GPU block (tolerance of an f32 sum taken in another order) and bit for bit across ranks."""
    world = min(torch.cuda.device_count(), 8)
    script = tmp_path / "worker_mlp.py"
    script.write_text(WORKER_MLP)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                          "--master-addr", "127.0.0.1", "--master-port", "29741", str(script)],
                         capture_output=True, text=True, timeout=280, env=env, cwd=os.getcwd())
    assert "TP_MLP_OK" in out.stdout, out.stdout[-2000:] + out.stderr[-2000:]


def _call(y, bufs, flags, rank, world, seq, oneshot):
    import ctypes as C
    from sme_gemm_b200._lib import check, lib
    b = (C.c_uint64 * world)(*[t.data_ptr() for t in bufs])
    f = (C.c_uint64 * world)(*[t.data_ptr() for t in flags])
    check("smeg_mlp_reduce_finish_dev",
          lib().smeg_mlp_reduce_finish_dev(y.data_ptr(), b, f, rank, world, y.numel(), seq, oneshot,
                                           torch.cuda.current_stream().cuda_stream))


FLAG_WORDS = 1288      # SMEG_TP_FLAG_WORDS


def _buffer(part):
    """A rank's buffer as the kernel wants it: the f32 partial followed by room for as many f16 results."""
    n = part.numel()
    buf = torch.zeros(n + n // 2 + 2, dtype=torch.float32, device="cuda")
    buf[:n].copy_(part.reshape(-1))
    return buf


@pytest.mark.parametrize("oneshot", [0, 1])
@pytest.mark.parametrize("m,d", [(1, 4096), (64, 4096), (3, 20), (300, 4096)])
def test_single_rank_reduce_finish_is_the_rounding_and_the_residual_add(m, d, oneshot):
    """world = 1: the kernel's own flags, slice and add; y += f32(f16(partial)) exactly."""
    import sme_gemm_b200 as sg
    g = torch.Generator(device="cuda").manual_seed(5)
    y = torch.randn(m, d, device="cuda", generator=g)
    flags = torch.zeros(FLAG_WORDS, dtype=torch.int32, device="cuda")
    for seq in (1, 2, 3):
        part = torch.randn(m, d, device="cuda", generator=g) * 5.0
        want = y + part.half().float()
        _call(y, [_buffer(part)], [flags], 0, 1, seq, oneshot)
        torch.cuda.synchronize()
        assert sg.last_status() == 0
        assert torch.equal(y, want)


def test_a_peer_that_never_arrives_ends_the_wait_with_the_status_raised_and_y_untouched():
    """Two ranks' buffers and flags stand on this one GPU and the second rank never runs: nothing sets its
    "ready" flag, the bounded wait (one second) runs out, the kernel returns, the status word says so.
    The kernel keeps no state of its own between calls, so a call after the timed-out one works."""
    import sme_gemm_b200 as sg
    y = torch.ones(2, 64, device="cuda")
    part = torch.full((2, 64), 3.0, device="cuda")
    bufs = [_buffer(part) for _ in range(2)]
    flags = [torch.zeros(FLAG_WORDS, dtype=torch.int32, device="cuda") for _ in range(2)]
    _call(y, bufs, flags, 0, 2, 1, 0)
    torch.cuda.synchronize()
    assert sg.last_status() & 4          # STATUS_PEER_TIMEOUT; reading clears the word
    assert sg.last_status() == 0
    assert torch.equal(y, torch.ones_like(y))
    assert int(flags[1][0].item()) == 1  # rank 0 did announce its partial to the absent rank
    # the next call, alone in its group, is unaffected
    fresh = torch.zeros(FLAG_WORDS, dtype=torch.int32, device="cuda")
    _call(y, [bufs[0]], [fresh], 0, 1, 1, 0)
    torch.cuda.synchronize()
    assert sg.last_status() == 0
    assert torch.equal(y, torch.full_like(y, 4.0))


WORKER_LAYER = r'''
import os, sys
import numpy as np
import torch, torch.distributed as dist
sys.path.insert(0, os.getcwd())
import sme_gemm_b200 as sg
from sme_gemm_b200.tp import PeerReduce, TpMlp, TpSelfAttention
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
d, f, heads, kv_heads, hd = 512, 1024, 16, 8, 32
rng = np.random.default_rng(21)
wq = (rng.standard_normal(((heads + 2 * kv_heads) * hd, d)) * 0.05).astype(np.float32)
wo = (rng.standard_normal((d, heads * hd)) * 0.05).astype(np.float32)
wg = (rng.standard_normal((f, d)) * 0.05).astype(np.float32)
wu = (rng.standard_normal((f, d)) * 0.05).astype(np.float32)
wd = (rng.standard_normal((d, f)) * 0.05).astype(np.float32)
g1 = (1 + 0.1 * rng.standard_normal(d)).astype(np.float32)
g2 = (1 + 0.1 * rng.standard_normal(d)).astype(np.float32)
OutIn = sg.WeightLayout.OutIn
def norms():
    return sg.Norm.rms(g1, 1e-5), sg.Norm.rms(g2, 1e-5)
n1, n2 = norms()
whole = sg.Block(n1, sg.SelfAttention(sg.Linear.quantize(wq, OutIn, wq.shape[0], d), sg.Linear.quantize(wo, OutIn, d, heads * hd),
                                      heads, kv_heads, hd),
                 n2, sg.Mlp.gated(sg.GatedLinear.quantize(wg, wu, OutIn, f, d, sg.Gate.Silu), sg.Linear.quantize(wd, OutIn, d, f)))
ok = True
for use_peer in (True, False):
    n1, n2 = norms()
    attn = TpSelfAttention.quantize(wq, wo, heads, kv_heads, hd, rank, world)
    mlp = TpMlp.quantize(wg, wu, wd, rank, world)
    layer = sg.Block(n1, attn, n2, mlp)
    cache, cache_w = layer.cache(64), whole.cache(64)
    assert cache.kv_heads() == kv_heads // world and cache.heads() == heads // world
    x = torch.from_numpy(rng.standard_normal((9, d)).astype(np.float32)).cuda()
    xs = [x[:5].contiguous(), x[5:6].contiguous(), x[6:9].contiguous()]         # a prompt, one decode step, three more rows
    for part in xs:
        m = part.shape[0]
        if use_peer:
            attn.peer = mlp.peer = PeerReduce(m, d)
        y, want = part.clone(), part.clone()
        layer.accumulate(y, cache, m)
        whole.accumulate(want, cache_w, m)
        torch.cuda.synchronize()
        rel = float(((y - want).abs() / (1 + want.abs())).max().item())
        bits = y.view(torch.int32).to(torch.int64).sum().reshape(1)
        lo, hi = bits.clone(), bits.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN); dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        if sg.last_status() != 0 or rel > 1e-2 or int(lo.item()) != int(hi.item()) or cache.len() != cache_w.len():
            ok = False
            print(f"rank {rank}: peer={use_peer} m={m}: max_rel {rel}, identical {int(lo.item()) == int(hi.item())}", flush=True)
    dist.barrier()
flag = torch.tensor([1 if ok else 0], device="cuda")
dist.all_reduce(flag, op=dist.ReduceOp.MIN)
if rank == 0:
    print("TP_LAYER_OK" if int(flag.item()) == 1 else "TP_LAYER_FAILED", flush=True)
dist.destroy_process_group()
'''


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs on one box")
def test_a_whole_layer_sharded_by_heads_and_hidden_units_matches_the_one_gpu_layer(tmp_path):
    """Block(norm1, TpSelfAttention, norm2, TpMlp) on two GPUs -- attention split by heads with per-rank KV caches, the MLP by
    hidden units, both sums over peer memory (then over the collective library) -- against the one-GPU Block through a
    prompt and decode steps, and bit for bit across ranks."""
    world = 2
    script = tmp_path / "worker_layer.py"
    script.write_text(WORKER_LAYER)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                          "--master-addr", "127.0.0.1", "--master-port", "29751", str(script)],
                         capture_output=True, text=True, timeout=280, env=env, cwd=os.getcwd())
    assert "TP_LAYER_OK" in out.stdout, out.stdout[-2000:] + out.stderr[-2000:]
