"""End-to-end checks on the GPU: the native training path of a small dense model agrees with the
CPU reference path step by step, and a short run reduces the loss."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _small_cfg():
    from mythos_b200.models import TransformerConfig

    return TransformerConfig(vocab_size=512, hidden_size=256, num_layers=2, num_heads=2, head_dim=128,
                             ffn_hidden_size=512, max_seq_len=256, oil_block_size=64, weight_format="oil8")


def test_native_loss_and_grads_match_cpu_reference():
    from mythos_b200.models import DenseModel
    from mythos_b200.train.param_store import ParamStore

    torch.manual_seed(0)
    cfg = _small_cfg()
    cpu = DenseModel(cfg)
    gpu = DenseModel(cfg)
    gpu.load_state_dict(cpu.state_dict())
    store = ParamStore(gpu, "cuda")
    store.refresh_compute()
    ids = torch.randint(0, cfg.vocab_size, (2, 256), dtype=torch.int32)
    tg = torch.randint(0, cfg.vocab_size, (2, 256), dtype=torch.int32)
    loss_c = cpu(ids, tg)
    loss_c.backward()
    loss_g = gpu(ids.cuda(), tg.cuda())
    loss_g.backward()
    torch.cuda.synchronize()
    assert abs(loss_g.item() - loss_c.item()) < 3e-2, (loss_g.item(), loss_c.item())
    checked = 0
    for (n, pc), (_, pg) in zip(cpu.named_parameters(), gpu.named_parameters()):
        g_ref = pc.grad.float()
        g_nat = pg.main_grad.float().cpu()
        denom = g_ref.norm().item() + 1e-8
        rel = (g_nat - g_ref).norm().item() / denom
        assert rel < 8e-2, f"{n}: relative gradient error {rel}"
        checked += 1
    assert checked > 5


def test_short_training_run_reduces_loss():
    from mythos_b200.models import DenseModel
    from mythos_b200.ops import native
    from mythos_b200.train.data import ZipfStream
    from mythos_b200.train.trainer import TrainConfig, Trainer

    torch.manual_seed(1)
    cfg = _small_cfg()
    with torch.device("cuda"):
        model = DenseModel(cfg)
    tr = Trainer(model, TrainConfig(batch_size=8, micro_batch_size=4, seq_length=256, lr=2e-3, warmup_steps=3,
                                    max_steps=40, codebook_ema_interval=10), device="cuda")
    data = ZipfStream(cfg.vocab_size, 8, 256, seed=3)
    before = native.launch_count()
    losses = []
    for _ in range(25):
        ids, tg = data.next_batch()
        losses.append(tr.train_step(ids, tg).item())
    assert native.launch_count() > before
    assert losses[-1] < losses[0] - 0.3, losses
    assert all(l == l for l in losses)


def test_activation_checkpointing_same_update_less_memory():
    """Recomputing block activations in the backward pass gives the same loss and gradients on the
    native path and a lower peak of allocated memory."""
    from mythos_b200.models import DenseModel, TransformerConfig
    from mythos_b200.train.param_store import ParamStore

    cfg = TransformerConfig(vocab_size=512, hidden_size=256, num_layers=6, num_heads=2, head_dim=128,
                            ffn_hidden_size=512, max_seq_len=512, oil_block_size=64, weight_format="oil8")
    torch.manual_seed(0)
    with torch.device("cuda"):
        model = DenseModel(cfg).train()
    store = ParamStore(model, "cuda")
    store.refresh_compute()
    ids = torch.randint(0, cfg.vocab_size, (8, 512), dtype=torch.int32, device="cuda")
    tg = torch.randint(0, cfg.vocab_size, (8, 512), dtype=torch.int32, device="cuda")
    res = []
    for ckpt in (False, True):
        model.activation_checkpointing = ckpt
        store.zero_grad()
        torch.cuda.synchronize()
        torch.cuda.reset_peak_memory_stats()
        base = torch.cuda.memory_allocated()
        loss = model(ids, tg)
        loss.backward()
        torch.cuda.synchronize()
        res.append((loss.item(), store.grad.clone(), torch.cuda.max_memory_allocated() - base))
        del loss
    assert res[0][0] == res[1][0]
    assert torch.allclose(res[0][1], res[1][1], rtol=1e-3, atol=1e-5)
    assert res[1][2] < 0.7 * res[0][2], (res[0][2], res[1][2])


def test_mixed_format_model_trains_and_decodes_on_the_gpu():
    """weight_format="mixed" (per-block OIL8 / OIL4 / ternary / binary): the native training path
    re-quantises block by block, the loss goes down, and the inference engine decodes the model."""
    from mythos_b200.infer.engine import InferenceEngine
    from mythos_b200.models import DenseModel, TransformerConfig
    from mythos_b200.train.data import ZipfStream
    from mythos_b200.train.trainer import TrainConfig, Trainer

    torch.manual_seed(2)
    cfg = TransformerConfig(vocab_size=512, hidden_size=256, num_layers=2, num_heads=2, head_dim=128,
                            ffn_hidden_size=512, max_seq_len=256, oil_block_size=256, weight_format="mixed")
    with torch.device("cuda"):
        model = DenseModel(cfg)
    up = model.layers[0].ffn.up_proj
    assert up.fmt == "mixed" and len(set(up.block_formats.tolist())) >= 2
    tr = Trainer(model, TrainConfig(batch_size=8, micro_batch_size=4, seq_length=256, lr=2e-3, warmup_steps=3,
                                    max_steps=40, codebook_ema_interval=0), device="cuda")
    data = ZipfStream(cfg.vocab_size, 8, 256, seed=3)
    losses = [tr.train_step(*data.next_batch()).item() for _ in range(20)]
    assert losses[-1] < losses[0] - 0.2, losses
    # the compute image of a mixed layer equals its per-block quantiser applied to the master weights
    tr.store.refresh_compute()
    want = up.quantize_now(up.weight.detach())
    assert torch.equal(up.weight.compute.detach().float(), want.float().view_as(up.weight))
    eng = InferenceEngine.from_model(model, device="cuda", max_batch=2, max_seq_len=128)
    ids = torch.randint(0, cfg.vocab_size, (2, 32), dtype=torch.int32)
    out = eng.generate(ids, max_new_tokens=4, use_graph=False)
    with torch.no_grad():
        ref_first = model(ids.cuda())[:, -1].float().argmax(-1).tolist()
    assert [t[0] for t in out.tokens] == ref_first
