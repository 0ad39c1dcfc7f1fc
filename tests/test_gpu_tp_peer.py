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
