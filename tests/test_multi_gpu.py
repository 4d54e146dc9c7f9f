"""Sequence split over real GPUs with NCCL (needs >= 2 devices; skipped otherwise).

Each rank holds the same sequence, attends its own range of cold blocks (the last rank also
the hot window), the (m, l, o) states are all-gathered over NVLink and merged by the LSE
combine kernel; the result must equal the single-device decode.  The same states then go
through the peer-memory exchange kernel, which must give the same bits.
"""

from __future__ import annotations

import os
import socket
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r"""
import os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, os.environ["TQ_ROOT"])
from turboquant_pro_b200 import KVContext
from turboquant_pro_b200.parallel import SequenceSplitDecoder
from turboquant_pro_b200.synth import make_kv, make_q

rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
h, grp, n = 2, 4, 6000
k, v = make_kv(5, h, n, dtype=np.float16)
q = torch.from_numpy(make_q(5, h * grp))[None].cuda().to(torch.bfloat16)
ctx = KVContext(n_layers=1, n_seqs=1, n_kv_heads=h, n_q_heads=h * grp, value_bits=3,
                hot_window=512, max_tokens_per_seq=n, kv_dtype="float16", seed=5,
                device=int(os.environ["LOCAL_RANK"]))
ctx.append(0, torch.from_numpy(k)[None].cuda(), torch.from_numpy(v)[None].cuda())
full = ctx.decode(0, q)
split = SequenceSplitDecoder(ctx).decode(0, q)
torch.cuda.synchronize()
err = (split - full).abs().max().item()
ok = torch.allclose(split, full, rtol=1e-3, atol=1e-4) and ctx.status() == 0
# the same states exchanged and merged by one kernel over peer memory: the same bits
from turboquant_pro_b200.parallel import PeerExchange, split_blocks, gather_states
nb = ctx.lengths(0, 0)[1] // ctx.block_tokens
lo, hi, with_hot = split_blocks(nb, rank, world)
ex = PeerExchange(h * grp, 128, ctx.device)
for it in range(4):
    mlo = ctx.decode_partial(0, q, lo, hi, with_hot).reshape(h * grp, 130).contiguous()
    via_nccl = ctx.lse_combine(gather_states(mlo))
    via_peer = ex.gather_merge(mlo)
    fused = ctx.decode_exchange(0, q, lo, hi, with_hot, ex).reshape(h * grp, 128)
    torch.cuda.synchronize()
    ok = ok and torch.equal(via_peer, via_nccl) and torch.equal(fused, via_nccl) \
        and ex.status() == 0
ex.close()
flag = torch.tensor([1 if ok else 0], device="cuda")
dist.all_reduce(flag, op=dist.ReduceOp.MIN)
if rank == 0:
    print("SEQSPLIT", "OK" if flag.item() == 1 else "FAIL", err)
dist.destroy_process_group()
sys.exit(0 if flag.item() == 1 else 1)
"""


def test_sequence_split_nccl(tmp_path):
    import torch

    if not torch.cuda.is_available():
        pytest.fail("CUDA device required for -m gpu tests")
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    world = 2 if n < 4 else 4
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, TQ_ROOT=ROOT, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
           f"--nproc-per-node={world}", "--master-addr", "127.0.0.1", "--master-port", str(port),
           str(script)]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    assert "SEQSPLIT OK" in out.stdout
