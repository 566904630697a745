"""The training driver end to end on one GPU: a tiny model trains on a repeating token pattern, writes the reference's
safetensors layout plus optimizer state, and a second run resumes from it (step count and moments included)."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_train_save_resume(tmp_path, capsys):
    from cgpt_b200 import train_cli
    from safetensors import safe_open
    tokens = np.tile(np.arange(97, dtype=np.int32) % 50, 400)          # learnable: next token is a function of the current
    path = str(tmp_path / "tokens.npy")
    np.save(path, tokens)
    out1, out2 = str(tmp_path / "run1"), str(tmp_path / "run2")
    common = ["--input", path, "--model", "tiny", "--vocab-size", "64", "--batch-size", "4", "--sequence-length", "64",
              "--validation-interval", "20", "--validation-batches", "2", "--learning-rate", "1e-3",
              "--min-learning-rate", "1e-4", "--save-avg-loss"]
    assert train_cli.main(common + ["--max-steps", "40", "--output-dir", out1]) == 0
    text = capsys.readouterr().out
    pick = lambda t: [float(l.split(" loss ")[1].split()[0]) for l in t.splitlines()
                      if l.startswith("step ") and "/" in l.split()[1]]
    losses = pick(text)
    assert len(losses) == 4 and losses[-1] < 0.5 * losses[0], text
    assert "validation loss" in text
    assert os.path.exists(os.path.join(out1, "model.safetensors")) and os.path.exists(os.path.join(out1, "optimizer.safetensors"))
    assert open(os.path.join(out1, "loss.csv")).readline().strip() == "step,loss"
    with safe_open(os.path.join(out1, "model.safetensors"), framework="pt") as f:
        assert "lm_head.weight" in f.keys() and f.get_tensor("model.layers.1.self_attn.q_norm.weight").dtype == torch.float16
    # resume: continues at step 40 with the saved moments, so the loss keeps falling from where it was
    assert train_cli.main(common + ["--max-steps", "60", "--load-dir", out1, "--output-dir", out2]) == 0
    text2 = capsys.readouterr().out
    assert "resuming at step 40" in text2
    losses2 = pick(text2)
    assert len(losses2) == 2 and max(losses2) < 0.5 * losses[0], text2   # a cold restart would be back near ln(64)
    with safe_open(os.path.join(out2, "optimizer.safetensors"), framework="pt") as f:
        assert '"step": 60' in f.metadata()["extra"]


def test_loss_on_random_tokens_stays_at_entropy(tmp_path, capsys):
    """Uniform random ids cannot be predicted: the training loss (always measured on a batch the model has not seen)
    must stay near ln(vocab). A driver that lets the GPU re-read a staging buffer would train on one batch repeatedly
    and report a loss well below it."""
    import math
    from cgpt_b200 import train_cli
    args = ["--synthetic", "600000", "--model", "tiny", "--vocab-size", "4096", "--batch-size", "8", "--sequence-length", "128",
            "--max-steps", "40", "--validation-interval", "40", "--validation-batches", "2", "--learning-rate", "1e-3",
            "--min-learning-rate", "1e-3", "--output-dir", str(tmp_path / "o")]
    assert train_cli.main(args) == 0
    text = capsys.readouterr().out
    losses = [float(l.split(" loss ")[1].split()[0]) for l in text.splitlines() if l.startswith("step ") and "/" in l.split()[1]]
    assert len(losses) == 4 and all(abs(x - math.log(4096)) < 0.35 for x in losses), text


def test_asynchronous_loss_read_equals_synchronous_read():
    """TrainStep.read_loss_async: the pinned copies, consumed one step late as a logging loop does, hold exactly the
    values a synchronous read after each step returns."""
    import torch
    from cgpt_b200 import model as M
    from cgpt_b200.train import TrainStep
    opts = M.TransformerModelOptions(512, 2, M.TransformerBlockOptions(256, 512, 2, 1, 128, 128))
    ids = torch.randint(0, 512, (6, 2 * 64), dtype=torch.int32, generator=torch.Generator().manual_seed(3)).pin_memory()
    targets = torch.roll(ids, -1, dims=1).contiguous().pin_memory()

    def run(asynchronous):
        ts = TrainStep(opts, 2, 64, seed=5)
        out, pending = [], None
        for i in range(6):
            ts.upload_batch(ids[i], targets[i])      # on the step's stream: ordered after the previous step
            ts.step()
            if asynchronous:
                handle = ts.read_loss_async()
                if pending is not None:
                    out.append(pending.value())
                pending = handle
            else:
                out.append(ts.read_loss())
        if asynchronous:
            out.append(pending.value())
        return out

    assert run(True) == run(False)


def test_mid_run_checkpoint_resumes_to_the_same_weights(tmp_path, capsys):
    """--checkpoint-interval writes <output>/step-N while later steps are already enqueued on the step's stream. A run that
    resumes from a checkpoint taken at a step that is no logging point (13) must end with exactly the weights and
    optimizer state of the uninterrupted run: the checkpoint holds a consistent state (step drained before the copies,
    step counter refreshed) and the resumed run continues the epoch where the saved one stopped."""
    from cgpt_b200 import train_cli
    from safetensors import safe_open
    tokens = np.random.default_rng(5).integers(0, 200, 40000).astype(np.int32)
    path = str(tmp_path / "tokens.npy")
    np.save(path, tokens)
    out_a, out_b = str(tmp_path / "a"), str(tmp_path / "b")
    common = ["--input", path, "--model", "tiny", "--vocab-size", "256", "--batch-size", "4", "--sequence-length", "64",
              "--validation-interval", "100", "--validation-batches", "1", "--learning-rate", "1e-3", "--min-learning-rate", "1e-4",
              "--max-steps", "30", "--epochs", "3"]
    assert train_cli.main(common + ["--checkpoint-interval", "13", "--output-dir", out_a]) == 0
    capsys.readouterr()
    mid = os.path.join(out_a, "step-13")
    assert os.path.exists(os.path.join(mid, "optimizer.safetensors"))
    with safe_open(os.path.join(mid, "optimizer.safetensors"), framework="pt") as f:
        assert '"step": 13' in f.metadata()["extra"]
    assert train_cli.main(common + ["--load-dir", mid, "--output-dir", out_b]) == 0
    assert "resuming at step 13" in capsys.readouterr().out
    for name in ("model.safetensors", "optimizer.safetensors"):
        with safe_open(os.path.join(out_a, name), framework="pt") as fa, safe_open(os.path.join(out_b, name), framework="pt") as fb:
            assert sorted(fa.keys()) == sorted(fb.keys())
            for k in fa.keys():
                assert torch.equal(fa.get_tensor(k), fb.get_tensor(k)), f"{name}:{k} differs between the resumed and the uninterrupted run"
