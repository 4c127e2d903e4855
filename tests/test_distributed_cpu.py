"""Multi-process paths on CPU ranks (gloo): pipeline-parallel 1F1B gradients equal single-process
gradients; a rank that never joins makes the others fail with a timeout instead of hanging;
checkpoints written at one world size load at another."""
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

PP_WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["REPO_ROOT"])
from mythos_b200.models import DenseModel, TransformerConfig
from mythos_b200.parallel.pp import PipelineStage, split_layers
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
torch.manual_seed(0)
cfg = TransformerConfig(vocab_size=64, hidden_size=32, num_layers=4, num_heads=2, head_dim=16, ffn_hidden_size=64,
                        max_seq_len=16, oil_block_size=32, weight_format="fp32")
model = DenseModel(cfg)          # same seed on every rank: identical weights
M, mb, S = 4, 2, 8
g = torch.Generator().manual_seed(1)
ids = torch.randint(0, 64, (M, mb, S), generator=g, dtype=torch.int32)
tg = torch.randint(0, 64, (M, mb, S), generator=g, dtype=torch.int32)
stage = PipelineStage(model, None, micro_batches=M)
loss = stage.train_step(ids, tg, hidden_shape=(mb, S, 32))
# single-process reference on every rank
ref = DenseModel(cfg); ref.load_state_dict(model.state_dict())
total = 0.0
for i in range(M):
    l = ref(ids[i], tg[i]) / M
    l.backward(); total += float(l)
lo, hi = split_layers(4, world)[rank]
ok = True
for k in range(lo, hi):
    for (n, p), (_, q) in zip(model.layers[k].named_parameters(), ref.layers[k].named_parameters()):
        if p.grad is None or not torch.allclose(p.grad, q.grad, atol=1e-5):
            ok = False
if rank == world - 1:
    ok = ok and abs(float(loss) - total) < 1e-5 and torch.allclose(model.lm_head.weight.grad, ref.lm_head.weight.grad, atol=1e-5)
if rank == 0:
    ok = ok and torch.allclose(model.tok_embeddings.weight.grad, ref.tok_embeddings.weight.grad, atol=1e-5)
flag = torch.tensor([1 if ok else 0]); dist.all_reduce(flag, op=dist.ReduceOp.MIN)
if rank == 0: print("PP_OK" if int(flag) == 1 else "PP_MISMATCH")
dist.destroy_process_group()
'''

TIMEOUT_WORKER = r'''
import datetime, os, sys, torch, torch.distributed as dist
rank = int(os.environ["RANK"])
if rank == 1:
    sys.exit(0)          # this rank leaves before the first collective
dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=3))
try:
    t = torch.ones(1); dist.all_reduce(t)
    print("UNEXPECTED_SUCCESS")
except Exception as e:
    print("DETECTED", type(e).__name__)
'''


VOCAB_CE_WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["REPO_ROOT"])
from mythos_b200.parallel.vocab_ce import vocab_parallel_cross_entropy
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
torch.manual_seed(0)
rows, V = 24, 40 * world
full = torch.randn(rows, V) * 3
targets = torch.randint(-2, V + 3, (rows,), dtype=torch.int32)       # out-of-range ids are clamped
ref_in = full.clone().requires_grad_(True)
ref = torch.nn.functional.cross_entropy(ref_in, targets.long().clamp(0, V - 1))
ref.backward()
v = V // world
shard = full[:, rank * v:(rank + 1) * v].clone().requires_grad_(True)
loss = vocab_parallel_cross_entropy(shard, targets, dist.group.WORLD)
loss.backward()
ok = abs(loss.item() - ref.item()) < 1e-5 and torch.allclose(shard.grad, ref_in.grad[:, rank * v:(rank + 1) * v], atol=1e-6)
flag = torch.tensor([1.0 if ok else 0.0]); dist.all_reduce(flag, op=dist.ReduceOp.MIN)
if rank == 0 and flag.item() == 1.0:
    print("VOCAB_CE_OK")
dist.destroy_process_group()
'''


def _torchrun(n, code, port, timeout=240, extra_env=None):
    env = dict(os.environ, REPO_ROOT=ROOT, **(extra_env or {}))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr",
           "127.0.0.1", "--master-port", str(port), "--no-python", sys.executable, "-c", code]
    return subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)


@pytest.mark.parametrize("stages", [2, 4])
def test_pipeline_1f1b_matches_single_process(stages):
    res = _torchrun(stages, PP_WORKER, 29700 + stages)
    assert "PP_OK" in res.stdout, res.stdout[-1500:] + res.stderr[-3000:]


@pytest.mark.parametrize("world", [2, 3])
def test_vocab_parallel_cross_entropy_matches_full_rows(world):
    res = _torchrun(world, VOCAB_CE_WORKER, 29720 + world)
    assert "VOCAB_CE_OK" in res.stdout, res.stdout[-1500:] + res.stderr[-3000:]


def test_missing_rank_is_detected_by_timeout_not_hang():
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29711", WORLD_SIZE="2")
    procs = [subprocess.Popen([sys.executable, "-c", TIMEOUT_WORKER], env=dict(env, RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True) for r in range(2)]
    out0, err0 = procs[0].communicate(timeout=120)
    procs[1].communicate(timeout=30)
    assert "UNEXPECTED_SUCCESS" not in out0
    assert "DETECTED" in out0 or procs[0].returncode != 0, out0 + err0[-1500:]


def test_checkpoint_written_for_one_layout_loads_into_another(tmp_path):
    """Optimizer state is stored per parameter: emulate resharding by loading a checkpoint into a
    trainer whose flat layout is padded for a different world size."""
    from mythos_b200.models import DenseModel, TransformerConfig
    from mythos_b200.train.data import ZipfStream
    from mythos_b200.train.param_store import ParamStore
    from mythos_b200.train.trainer import TrainConfig, Trainer

    torch.manual_seed(0)
    cfg = TransformerConfig(vocab_size=64, hidden_size=32, num_layers=2, num_heads=2, head_dim=16, ffn_hidden_size=64,
                            max_seq_len=16, oil_block_size=32)
    tr = Trainer(DenseModel(cfg), TrainConfig(batch_size=4, seq_length=16, lr=1e-2, warmup_steps=0), device="cpu")
    data = ZipfStream(64, 4, 16, seed=0)
    for _ in range(3):
        tr.train_step(*data.next_batch())
    path = str(tmp_path / "ck.oil")
    tr.save_checkpoint(path)
    assert os.path.exists(path + ".opt") and os.path.exists(path + "idx")
    tr2 = Trainer(DenseModel(cfg), TrainConfig(batch_size=4, seq_length=16, lr=1e-2, warmup_steps=0), device="cpu")
    tr2.store = ParamStore(tr2.model, "cpu", world_size=8)       # a layout padded for 8 ranks
    tr2.m = torch.zeros(tr2.store.total)
    tr2.v = torch.zeros(tr2.store.total)
    tr2.store.shard = tr2.store.total                              # this process plays every shard
    tr2.load_checkpoint(path)
    assert tr2.step == 3
    for s1, s2 in zip(tr.store.slots, tr2.store.slots):
        a = tr.m[s1.offset:s1.offset + s1.numel]
        b = tr2.m[s2.offset:s2.offset + s2.numel]
        assert torch.allclose(a, b)
    batch = data.next_batch()
    l1, l2 = tr.train_step(*batch), tr2.train_step(*batch)
    assert abs(float(l1) - float(l2)) < 2e-3


@pytest.mark.parametrize("fmt", ["oil8", "i2s"])
def test_resume_restores_fp32_masters_of_quantised_layers(tmp_path, fmt):
    """The .oil file stores centroids / trits; the fp32 master weights travel in the .master file, so
    a resumed run has the same masters and follows the same trajectory as an uninterrupted one."""
    from mythos_b200.models import DenseModel, TransformerConfig
    from mythos_b200.train.data import ZipfStream
    from mythos_b200.train.trainer import TrainConfig, Trainer

    cfg = TransformerConfig(vocab_size=64, hidden_size=32, num_layers=2, num_heads=2, head_dim=16, ffn_hidden_size=64,
                            max_seq_len=16, oil_block_size=32, weight_format=fmt)
    tc = TrainConfig(batch_size=4, seq_length=16, lr=1e-2, warmup_steps=0)
    torch.manual_seed(0)
    tr = Trainer(DenseModel(cfg), tc, device="cpu")
    data = ZipfStream(64, 4, 16, seed=0)
    for _ in range(3):
        tr.train_step(*data.next_batch())
    path = str(tmp_path / "ck.oil")
    tr.save_checkpoint(path)
    assert os.path.exists(path + ".master")
    torch.manual_seed(1)                                            # different initial weights
    tr2 = Trainer(DenseModel(cfg), tc, device="cpu")
    tr2.load_checkpoint(path)
    quantised = [s for s in tr.store.slots if s.module is not None]
    assert quantised
    for s1, s2 in zip(tr.store.slots, tr2.store.slots):
        a = tr.store.master[s1.offset:s1.offset + s1.numel]
        b = tr2.store.master[s2.offset:s2.offset + s2.numel]
        if s1.module is not None:
            assert torch.equal(a, b), s1.name                       # not collapsed onto centroids
            assert not torch.equal(a, s1.module.quantize_now(a.view(s1.param.shape)).reshape(-1).float())
    for _ in range(4):                                              # the trajectories stay together
        batch = data.next_batch()
        l1, l2 = tr.train_step(*batch), tr2.train_step(*batch)
        assert abs(float(l1) - float(l2)) < 1e-5
    for s1, s2 in zip(tr.store.slots, tr2.store.slots):
        if s1.module is not None:
            assert torch.allclose(tr.store.master[s1.offset:s1.offset + s1.numel],
                                  tr2.store.master[s2.offset:s2.offset + s2.numel], atol=1e-6)
