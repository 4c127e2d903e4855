"""Multi-GPU data parallelism: the fused peer-memory path must produce the same training
trajectory as the NCCL baseline path. Runs as child processes (one per GPU) when at least two
GPUs are visible; NVLS is disabled in NCCL for these runs."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

WORKER = r'''
import json, os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["REPO_ROOT"])
from mythos_b200.models import DenseModel, TransformerConfig
from mythos_b200.parallel.zero import ZeroEngine
from mythos_b200.train.data import ZipfStream
from mythos_b200.train.trainer import TrainConfig, Trainer
from mythos_b200.ops import native
mode = sys.argv[1]
rank = int(os.environ["RANK"]); local = int(os.environ["LOCAL_RANK"])
torch.cuda.set_device(local)
dev = torch.device("cuda", local)
dist.init_process_group("nccl", device_id=dev)
torch.manual_seed(7)
cfg = TransformerConfig(vocab_size=512, hidden_size=256, num_layers=2, num_heads=2, head_dim=128, ffn_hidden_size=512,
                        max_seq_len=256, oil_block_size=256, codebook_group=4)
with torch.device(dev):
    model = DenseModel(cfg)
dp = ZeroEngine(dist.group.WORLD, dev, mode=mode)
tr = Trainer(model, TrainConfig(batch_size=4, micro_batch_size=2, seq_length=256, lr=1e-3, warmup_steps=2,
                                codebook_ema_interval=0), device=dev, dp=dp)
data = ZipfStream(cfg.vocab_size, 4, 256, seed=11 + rank)
losses = [tr.train_step(*data.next_batch()).item() for _ in range(6)]
torch.cuda.synchronize(); native.check_status(dev)
dp.gather_master()
digest = float(tr.store.master.double().abs().sum())
if rank == 0:
    print("RESULT " + json.dumps({"mode": dp.mode, "losses": losses, "digest": digest}))
dist.destroy_process_group()
'''


def _run(mode: str, n: int):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, REPO_ROOT=root, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr",
           "127.0.0.1", "--master-port", "29611", "--no-python", sys.executable, "-c", WORKER, mode]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    line = [l for l in res.stdout.splitlines() if l.startswith("RESULT ")][-1]
    return json.loads(line[len("RESULT "):])


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_fused_zero_matches_nccl_baseline():
    n = 2
    fused = _run("fused", n)
    base = _run("nccl", n)
    assert fused["mode"] == "fused" and base["mode"] == "nccl"
    for a, b in zip(fused["losses"], base["losses"]):
        assert abs(a - b) < 5e-2, (fused["losses"], base["losses"])
    assert fused["losses"][-1] < fused["losses"][0]
    assert abs(fused["digest"] - base["digest"]) < 1e-3 * base["digest"]
