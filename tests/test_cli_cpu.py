"""The command-line tools end to end on the CPU with a tiny model: train -> info -> infer ->
finetune (adapters, full with a frozen base, periodic saves) -> convert -> bench."""
import hashlib
import json
import os

import numpy as np
import pytest
import torch

CORPUS = ("the quick brown fox jumps over the lazy dog. " * 60 + "pack my box with five dozen liquor jugs. " * 60)


@pytest.fixture(scope="module")
def trained(tmp_path_factory):
    from mythos_b200.tools import train

    d = tmp_path_factory.mktemp("cli")
    data = d / "corpus.txt"
    data.write_text(CORPUS)
    model = d / "tiny.oil"
    rc = train.main(["--model", str(model), "--data", str(data), "--batch-size", "2", "--seq-length", "32", "--epochs", "1",
                     "--max-steps", "6", "--vocab-size", "300", "--dim", "64", "--n-layers", "2", "--num-heads", "2",
                     "--weight-format", "oil8", "--block-size", "64", "--lr", "1e-3", "--gpu", "cpu", "--seed", "1",
                     "--log-interval", "3"])
    assert rc == 0 and model.exists() and (d / "tiny.vocab").exists() and (d / "tiny.oilidx").exists()
    return d, model, data


def test_train_writes_a_verifiable_container(trained, capsys):
    from mythos_b200.oil.container import file_sha256, verify
    from mythos_b200.oil.model_io import load_model, save_model
    from mythos_b200.tools import info

    d, model, _ = trained
    assert len(verify(str(model))) > 10          # every tensor matches its sidecar digest
    digest = file_sha256(str(model))
    assert digest == hashlib.sha256(model.read_bytes()).hexdigest()
    # save -> load -> save reproduces the file bit for bit
    m, _ = load_model(str(model), device="cpu")
    again = d / "again.oil"
    save_model(m, str(again))
    assert file_sha256(str(again)) == digest
    assert info.main([str(model), "--json", "--verify"]) == 0
    out = json.loads(capsys.readouterr().out)
    assert out["architecture"]["hidden_size"] == 64 and out["num_tensors"] > 0
    assert 7.5 < out["avg_bpw"] < 33 and out["format_share"]["oil8"] > 0.5 and out["verified_tensors"] > 10


def test_infer_positional_and_flags(trained, capsys):
    from mythos_b200.tools import infer

    d, model, _ = trained
    assert infer.main([str(model), "the quick", "--max-tokens", "5", "--temperature", "0", "--gpu", "cpu"]) == 0
    first = capsys.readouterr().out
    assert infer.main(["-m", str(model), "-p", "the quick", "-t", "5", "--temperature", "0", "--gpu", "cpu", "-o",
                       str(d / "gen.txt")]) == 0
    capsys.readouterr()
    assert (d / "gen.txt").read_text().strip() and first.strip()
    assert infer.main([str(model), "the quick", "-t", "3", "--temperature", "0", "--gpu", "cpu", "--precision", "int8"]) == 0


@pytest.mark.parametrize("method", ["lora", "qlora", "dora", "full"])
def test_finetune_methods(trained, method):
    from mythos_b200.oil.container import OILReader
    from mythos_b200.tools import finetune

    d, model, data = trained
    out = d / f"ft_{method}.oil"
    argv = ["--model", str(model), "--data", str(data), "--output", str(out), "--max-steps", "4", "--batch-size", "2",
            "--seq-length", "32", "--method", method, "--lora-rank", "4", "--gpu", "cpu", "--log-interval", "2"]
    if method == "full":
        argv += ["--freeze-base", "--save-interval", "2"]
    assert finetune.main(argv) == 0 and out.exists()
    names = OILReader(str(out)).tensor_names()
    if method == "full":
        base = OILReader(str(model))
        tuned = OILReader(str(out))
        frozen = [n for n in names if n.endswith("q_proj.weight") or n.endswith("qkv_proj.weight")]
        assert frozen and all(np.array_equal(base.read_tensor(n), tuned.read_tensor(n)) for n in frozen)
        norms = [n for n in names if "norm" in n]
        assert any(not np.array_equal(base.read_tensor(n), tuned.read_tensor(n)) for n in norms)
    else:
        assert any(".lora." in n for n in names)


def test_convert_and_bench(trained, capsys):
    from mythos_b200.oil.container import OILReader
    from mythos_b200.tools import bench, convert

    d, model, _ = trained
    raw = d / "w.bin"
    vals = np.arange(8, dtype="<f4")
    raw.write_bytes(vals.tobytes())
    assert convert.main(["--input", str(raw), "--output", str(d / "w.oil"), "--format", "rawfp32"]) == 0
    assert np.array_equal(OILReader(str(d / "w.oil")).read_tensor("weights"), vals)
    sd = {"layer.weight": torch.randn(64, 128), "layer.bias": torch.randn(64)}
    torch.save(sd, d / "sd.pt")
    assert convert.main(["-i", str(d / "sd.pt"), "-o", str(d / "sd.oil"), "--weight-format", "oil4", "--block-size", "64"]) == 0
    got = OILReader(str(d / "sd.oil")).read_tensor("layer.weight").reshape(64, 128)
    assert np.abs(got - sd["layer.weight"].numpy()).mean() < 0.2
    capsys.readouterr()
    prompts = d / "prompts.txt"
    prompts.write_text("the quick\npack my box\n")
    assert bench.main(["--inference", "--model", str(model), "--prompts", str(prompts), "--max-tokens", "4", "--gpu", "cpu",
                       "--output", str(d / "bench.json")]) == 0
    row = json.loads((d / "bench.json").read_text())
    assert row["prompts"] == 2 and row["tokens_per_s"] > 0 and row["ms_per_token"] > 0


def test_train_streaming_with_augmentation_and_curriculum(tmp_path):
    from mythos_b200.tools import train

    data = tmp_path / "corpus.txt"
    data.write_text(CORPUS * 3)
    model = tmp_path / "s.oil"
    rc = train.main(["--model", str(model), "--data", str(data), "--streaming", "--batch-size", "2", "--seq-length", "32",
                     "--epochs", "2", "--max-steps", "8", "--vocab-size", "300", "--dim", "64", "--n-layers", "1",
                     "--num-heads", "2", "--weight-format", "fp32", "--gpu", "cpu", "--mask-prob", "0.1",
                     "--replace-prob", "0.05", "--curriculum-epochs", "2", "--log-interval", "4"])
    assert rc == 0 and model.exists() and (tmp_path / "s.vocab").exists()
