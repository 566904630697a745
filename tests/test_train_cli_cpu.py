"""Host-side logic of the training driver and the checkpoint format (no GPU): flag defaults against the reference
trainer's (train/train.cpp:40-64), sample split, schedule lengths, rank slicing, safetensors round trip."""
import numpy as np
import pytest
import torch

from cgpt_b200 import checkpoint, train_cli
from cgpt_b200 import model as M
from cgpt_b200 import optim as O


def _args(*argv):
    return train_cli.resolve_arguments(train_cli.build_parser().parse_args(list(argv)))


def test_defaults_match_reference_trainer():
    a = _args("--synthetic", "100000")
    assert (a.vocab_size, a.batch_size, a.sequence_length, a.epochs, a.max_steps) == (32000, 8, 1024, 10, 0)
    assert (a.validation_interval, a.validation_batches) == (500, 64)
    assert (a.learning_rate, a.min_learning_rate, a.warmup_steps, a.loss_scale) == (3.0e-4, 3.0e-5, 0, 1024.0)
    assert (a.model, a.validation_fraction, a.save_avg_loss) == ("small", 0.1, False)
    assert _args("--synthetic", "9", "--model", "104m").batch_size == 1          # train.cpp:339
    assert _args("--synthetic", "9", "--model", "104m", "--batch-size", "32").batch_size == 32


@pytest.mark.parametrize("bad", [["--validation-fraction", "1.0"], ["--learning-rate", "0"], ["--min-learning-rate", "1"],
                                 ["--loss-scale", "0"], ["--batch-size", "0"]])
def test_invalid_arguments_raise(bad):
    with pytest.raises(ValueError):
        _args("--synthetic", "1000", *bad)
    with pytest.raises(ValueError):
        _args()                                   # neither --input nor --synthetic
    with pytest.raises(ValueError):
        _args("--input", "x.npy", "--synthetic", "5")


def test_split_is_disjoint_and_shaped():
    tokens = np.arange(10_000, dtype=np.int32)
    sp = train_cli.split_samples(tokens, batch=4, seq=16, validation_fraction=0.1)
    n = (tokens.size - 1) // 16
    assert sp.train.shape[1] == sp.validation.shape[1] == 17
    assert sp.train.shape[0] + sp.validation.shape[0] == n
    assert sp.validation.shape[0] == int(n * 0.1)
    starts = np.concatenate([sp.train[:, 0], sp.validation[:, 0]])
    assert len(set(starts.tolist())) == n and np.all(starts % 16 == 0)
    assert np.all(sp.train[:, 1:] == sp.train[:, :-1] + 1)             # targets are the next token
    with pytest.raises(RuntimeError):
        train_cli.split_samples(tokens[:100], batch=4, seq=16, validation_fraction=0.1)
    # the validation set never drops below one batch nor leaves less than one training batch
    assert train_cli.split_samples(tokens, 8, 16, 0.001).validation.shape[0] == 8
    assert train_cli.split_samples(tokens, 8, 16, 0.999).train.shape[0] == 8


def test_schedule_lengths_and_rank_slices():
    a = _args("--synthetic", "1000", "--epochs", "3")
    assert train_cli.schedule_lengths(a, 100) == (300, 6)                 # 2 % warm-up
    a = _args("--synthetic", "1000", "--max-steps", "40", "--warmup-steps", "5")
    assert train_cli.schedule_lengths(a, 100) == (40, 5)
    a = _args("--synthetic", "1000", "--epochs", "1")
    assert train_cli.schedule_lengths(a, 1) == (1, 0)
    g = np.arange(8 * 5).reshape(8, 5)
    assert np.array_equal(np.concatenate([train_cli.rank_slice(g, r, 2) for r in range(4)]), g)


def test_checkpoint_round_trip(tmp_path):
    opts = M.preset("tiny", vocabulary_size=64)
    a = M.ModelStorage(opts, torch.float16, seed=1, device="cpu")
    b = M.ModelStorage(opts, torch.float16, seed=2, device="cpu")
    names = [n for n, _ in checkpoint.named_parameters(a)]
    assert names[0] == "model.embed_tokens.weight" and "model.layers.1.mlp.down_proj.weight" in names
    assert len(names) == 2 + 11 * opts.num_layers
    checkpoint.save_model(str(tmp_path), a)
    checkpoint.load_model(str(tmp_path), b)
    for (_, x), (_, y) in zip(checkpoint.named_parameters(a), checkpoint.named_parameters(b)):
        assert torch.equal(x, y)
    mk = lambda st, k: [O.AdamWState(p.float() + k, torch.full_like(p, 0.5 * k, dtype=torch.float32),
                                     torch.full_like(p, 0.25 * k, dtype=torch.float32), 7 * k)
                        for p, _ in st.parameters_and_gradients()]
    sa, sb = mk(a, 1), mk(b, 3)
    checkpoint.save_optimizer(str(tmp_path), a, sa, {"step": 123})
    assert checkpoint.has_optimizer(str(tmp_path))
    assert checkpoint.load_optimizer(str(tmp_path), b, sb) == {"step": 123}
    for x, y in zip(sa, sb):
        assert torch.equal(x.master_parameter, y.master_parameter) and torch.equal(x.first_moment, y.first_moment)
        assert torch.equal(x.second_moment, y.second_moment) and y.step == 7
    # a model of another shape is refused
    c = M.ModelStorage(M.preset("tiny", vocabulary_size=32), torch.float16, seed=1, device="cpu")
    with pytest.raises(ValueError):
        checkpoint.load_model(str(tmp_path), c)


def test_presets_have_the_documented_sizes():
    """Parameter counts of the presets (tied embedding, 11 tensors per block, final norm): 104m = 104,090,624 and the
    1.3B configuration = 1,147,772,928; model FLOPs per token of the 104m step as quoted for the benchmark."""
    import math
    from cgpt_b200 import model as M, profiling

    def count(o):
        per_block = sum(math.prod(s) for s in M.block_param_shapes(o.block_options).values())
        return o.vocabulary_size * o.block_options.hidden_size + o.num_layers * per_block + o.block_options.hidden_size

    assert count(M.preset("104m")) == 104_090_624
    assert count(M.preset("1.3b")) == 1_147_772_928
    o = M.preset("104m")
    assert profiling.model_flops_per_token(o) + profiling.attention_flops_per_token(o, 1024) == 683_147_264
    with pytest.raises(ValueError):
        M.preset("no-such-model")


def test_learning_rate_schedule_matches_reference_header():
    """LearningRateScheduler.learning_rate() against values produced by the reference's own header-only scheduler
    (include/optim/lr_scheduler.h:37-51; fixture generated by tests/golden/make_lr_golden.py): warm-up, cosine part, the
    last step (exactly the minimum) and steps past the end."""
    import json
    from pathlib import Path
    from cgpt_b200.optim import LearningRateScheduler, LearningRateSchedulerOptions
    cases = json.loads((Path(__file__).parent / "golden" / "lr_schedule.json").read_text())
    assert len(cases) >= 5
    for c in cases:
        s = LearningRateScheduler(LearningRateSchedulerOptions(c["initial"], c["minimum"], c["warmup"], c["total"]))
        for step, want in zip(c["steps"], c["values"]):
            got = s.learning_rate(step)
            assert abs(got - want) <= 2e-7 * max(abs(want), c["initial"]), (c, step, got, want)
        # the last step returns the minimum itself, not a value of the cosine (the fixture holds it as fp32)
        assert s.learning_rate(c["total"] - 1) == c["minimum"]
        assert np.float32(c["minimum"]) == np.float32(c["values"][c["steps"].index(c["total"] - 1)])
