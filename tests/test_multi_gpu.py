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


TP_WORKER = r'''
import json, os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["REPO_ROOT"])
from mythos_b200.infer.engine import InferenceEngine, TPContext
from mythos_b200.models import DenseModel, TransformerConfig
from mythos_b200.ops import native
rank = int(os.environ["RANK"]); local = int(os.environ["LOCAL_RANK"]); world = int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(local)
dev = torch.device("cuda", local)
dist.init_process_group("nccl", device_id=dev)
torch.manual_seed(3)
cfg = TransformerConfig(vocab_size=1024, hidden_size=512, num_layers=2, num_heads=4, head_dim=128, num_kv_heads=2,
                        ffn_hidden_size=1024, max_seq_len=256, oil_block_size=256, codebook_group=2,
                        weight_format="oil8", attn_format="oil4")
with torch.device(dev):
    model = DenseModel(cfg)
for p in model.parameters():
    dist.broadcast(p.data, src=0)
B, S, new = 3, 128, 8
prompts = torch.randint(0, cfg.vocab_size, (B, S), generator=torch.Generator().manual_seed(5), dtype=torch.int32)
single = InferenceEngine.from_model(model, device=dev, max_batch=4, max_seq_len=256)
ref = single.generate(prompts, max_new_tokens=new, use_graph=False)
tp = TPContext(dist.group.WORLD, dev, max_tokens=B * S, hidden=cfg.hidden_size, vocab_shard=cfg.vocab_size // world,
               max_batch=4)
eng = InferenceEngine.from_model(model, device=dev, max_batch=4, max_seq_len=256, tp=tp)
out = eng.generate(prompts, max_new_tokens=new, use_graph=False)
out_g = eng.generate(prompts, max_new_tokens=new, use_graph=True)
torch.cuda.synchronize(); native.check_status(dev)
if rank == 0:
    print("RESULT " + json.dumps({"ref": ref.tokens, "tp": out.tokens, "tp_graph": out_g.tokens}))
dist.destroy_process_group()
'''


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
@pytest.mark.parametrize("row_flags", ["0", "1"])
def test_tensor_parallel_engine_matches_single_gpu(row_flags):
    """row_flags = 1: decode-sized sums run as the single-launch kernel with per-row flags."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, REPO_ROOT=root, NCCL_NVLS_ENABLE="0", MYTHOS_TP_ROW_FLAGS=row_flags)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29621", "--no-python", sys.executable, "-c", TP_WORKER]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    r = json.loads([l for l in res.stdout.splitlines() if l.startswith("RESULT ")][-1][len("RESULT "):])
    assert r["tp"] == r["tp_graph"]
    same = sum(int(a == b) for x, y in zip(r["ref"], r["tp"]) for a, b in zip(x, y))
    total = sum(len(x) for x in r["ref"])
    # sharded accumulation order differs from the single-GPU order; greedy paths may split at a near-tie
    assert same >= 0.7 * total, r
    assert [x[0] for x in r["ref"]] == [x[0] for x in r["tp"]]


EP_WORKER = r'''
import json, os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["REPO_ROOT"])
from mythos_b200.models import TransformerConfig
from mythos_b200.models.moe import ExpertParallel, MoEFFN
from mythos_b200.ops import native
from mythos_b200.parallel.vocab_ce import vocab_parallel_cross_entropy
from mythos_b200.train.param_store import ParamStore
rank = int(os.environ["RANK"]); local = int(os.environ["LOCAL_RANK"]); world = int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(local)
dev = torch.device("cuda", local)
dist.init_process_group("nccl", device_id=dev)
cfg = TransformerConfig(vocab_size=256, hidden_size=256, num_layers=1, num_heads=2, head_dim=128, ffn_hidden_size=256,
                        max_seq_len=128, oil_block_size=64, weight_format="fp32", num_experts=4, moe_top_k=2,
                        moe_ffn_hidden_size=256)
T = 96
torch.manual_seed(0)                      # the same expert weights on every rank
ref = MoEFFN(cfg)
nat = MoEFFN(cfg, exchange=ExpertParallel(dist.group.WORLD, dev, cap_rows=T * cfg.moe_top_k, dim=cfg.hidden_size))
nat.load_state_dict(ref.state_dict())
store = ParamStore(nat, dev)
store.refresh_compute()
xs = [torch.randn(T, 256, generator=torch.Generator().manual_seed(100 + r)) for r in range(world)]
dys = [torch.randn(T, 256, generator=torch.Generator().manual_seed(200 + r)) for r in range(world)]
# reference: every rank's tokens through all experts on the CPU in fp32
xr = torch.cat(xs).requires_grad_()
yr = ref(xr)
(yr * torch.cat(dys)).sum().backward()
xg = xs[rank].to(dev).to(torch.bfloat16).requires_grad_()
yg = nat(xg)
(yg.float() * dys[rank].to(dev)).sum().backward()
torch.cuda.synchronize(); native.check_status(dev)
sl = slice(rank * T, (rank + 1) * T)
res = {"y": float((yg.float().cpu() - yr[sl]).abs().max() / (yr.abs().max() + 1e-6)),
       "dx": float((xg.grad.float().cpu() - xr.grad[sl]).norm() / xr.grad[sl].norm())}
epr = cfg.num_experts // world
worst = 0.0
for e in range(rank * epr, (rank + 1) * epr):   # local experts saw the tokens of every rank
    for mods_n, mods_r in ((nat.experts_up, ref.experts_up), (nat.experts_down, ref.experts_down)):
        g_ref = mods_r[e].weight.grad
        g_nat = mods_n[e].weight.main_grad.cpu()
        worst = max(worst, float((g_nat - g_ref).norm() / (g_ref.norm() + 1e-9)))
res["dw_local"] = worst

# vocabulary-parallel cross-entropy over NCCL against the full rows
rows, V = 64, 4096
full = (torch.randn(rows, V, generator=torch.Generator().manual_seed(9)) * 3).to(torch.bfloat16)
tg = torch.randint(0, V, (rows,), generator=torch.Generator().manual_seed(10), dtype=torch.int32)
v = V // world
shard = full[:, rank * v:(rank + 1) * v].contiguous().to(dev).requires_grad_()
loss = vocab_parallel_cross_entropy(shard, tg.to(dev), dist.group.WORLD)
loss.backward()
fr = full.float().requires_grad_()
want = torch.nn.functional.cross_entropy(fr, tg.long())
want.backward()
res["ce_loss"] = abs(loss.item() - want.item())
res["ce_grad"] = float((shard.grad.float().cpu() - fr.grad[:, rank * v:(rank + 1) * v]).abs().max()) * rows
out = [None] * world
dist.all_gather_object(out, res)
if rank == 0:
    print("RESULT " + json.dumps(out))
dist.destroy_process_group()
'''


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_expert_parallel_moe_and_vocab_parallel_loss_on_two_gpus():
    """Expert parallelism: every rank routes its own tokens, expert FFNs run on the owner rank over
    peer-memory dispatch / combine; outputs, input gradients and the local experts' weight
    gradients must match all experts applied to all tokens in fp32. Then the sharded loss."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, REPO_ROOT=root, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29631", "--no-python", sys.executable, "-c", EP_WORKER]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    ranks = json.loads([l for l in res.stdout.splitlines() if l.startswith("RESULT ")][-1][len("RESULT "):])
    for r in ranks:
        assert r["y"] < 5e-2 and r["dx"] < 8e-2 and r["dw_local"] < 8e-2, ranks
        assert r["ce_loss"] < 5e-3 and r["ce_grad"] < 5e-2, ranks
