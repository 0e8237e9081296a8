"""engine.save / engine.load: resuming reproduces the uninterrupted trajectory."""
import tempfile

import torch


def _engine(split):
    from flextrain_b200.models.llama import preset
    from flextrain_b200.testing import build_llama_engine, reset_runtime
    reset_runtime()
    cfg = preset("tiny", num_layers=3, hidden=64, num_heads=2, ffn=128, vocab=128, seq_len=32)
    g = torch.Generator().manual_seed(3)
    data = [torch.randint(0, 128, (2, 33), generator=g) for _ in range(12)]
    cursor = {"i": 0}

    def batch_fn():
        t = data[cursor["i"] % len(data)]
        cursor["i"] += 1
        return t[:, :-1].contiguous(), t[:, 1:].contiguous()

    ft_cfg = {"batch_size": 4, "micro_batch_size": 2, "mixed_precision": {"device_dtype": "fp32"},
              "split_ratio": split}
    model, opt, eng = build_llama_engine(cfg, ft_cfg, batch_fn, lr=1e-2, backend="gloo")
    return eng, cursor


def _loss(eng):
    r = eng.train_iteration()
    return sum(float(x.detach()) for x in r) / len(r)


def test_resume_matches_uninterrupted_run():
    from flextrain_b200.testing import reset_runtime
    split = {"parameter": [0.5, 0.5], "optimizer": [0.25, 0.75], "checkpoint": [1.0, 0.0],
             "gradient": [1.0, 0.0]}
    eng, _ = _engine(split)
    straight = [_loss(eng) for _ in range(6)]
    eng.shutdown()
    with tempfile.TemporaryDirectory() as d:
        eng, _ = _engine(split)
        first = [_loss(eng) for _ in range(3)]
        eng.save(d)
        eng.shutdown()
        # a fresh process would build the model again; different tier split on purpose
        eng, cursor = _engine({"parameter": [0.0, 1.0], "optimizer": [0.0, 1.0],
                               "checkpoint": [0.0, 1.0], "gradient": [0.0, 1.0]})
        for _ in range(2):
            _loss(eng)                          # disturb the state before loading
        eng.load(d)
        cursor["i"] = 6                         # data position after 3 steps of 2 micro-batches
        rest = [_loss(eng) for _ in range(3)]
        assert eng.global_steps == 6
        eng.shutdown()
    reset_runtime()
    assert first == straight[:3]
    assert max(abs(a - b) for a, b in zip(rest, straight[3:])) < 1e-5
