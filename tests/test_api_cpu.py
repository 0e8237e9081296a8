import argparse

import pytest
import torch

import flextrain_b200 as ft
from flextrain_b200.llm_func import LLMFunc, retrieve_llm_loss, set_llm_func


def test_config_arguments():
    p = ft.add_config_arguments(argparse.ArgumentParser())
    a = p.parse_args(["--flextrain", "--flextrain-config", "c.json"])
    assert a.flextrain and a.flextrain_config == "c.json"
    assert not p.parse_args([]).flextrain


def test_llm_func_registry_and_loss_retrieval():
    from flextrain_b200.llm_func import reset_llm_func
    reset_llm_func()
    with pytest.raises(NotImplementedError):
        LLMFunc.get_batch()
    set_llm_func(lambda i: i, lambda: ((1,), (), ()), lambda x: (x, ()), lambda s, e: (lambda *a: a),
                 lambda p, q: p, lambda o, l: o)
    assert LLMFunc.get_layer(3) == 3 and LLMFunc.get_batch() == ((1,), (), ())
    t = torch.tensor(2.0)
    assert retrieve_llm_loss(t) is t
    assert retrieve_llm_loss(["x", torch.ones(3), torch.tensor([4.0])]).item() == 4.0
    with pytest.raises(ValueError):
        retrieve_llm_loss([torch.ones(3)])


def test_public_names():
    for name in ("Init", "LLMFunc", "set_llm_func", "initialize", "init_distributed", "distributed",
                 "add_config_arguments", "shutdown_init_context", "restore_init_context",
                 "FlexTrainEngine", "FlexTrainOptimizer", "op_builder", "init_flextrain_config"):
        assert hasattr(ft, name)
    with pytest.raises(AttributeError):
        ft.no_such_name
    from flextrain_b200.checkpointing import (checkpointed_backward, checkpointed_forward,  # noqa
                                              detach_variable, get_cuda_rng_tracker,
                                              model_parallel_cuda_manual_seed)
    from flextrain_b200.ops.adam import FlexTrainAdam  # noqa
    from flextrain_b200.ops.adam.cpu_adam import FlexTrainCPUAdam  # noqa
    from flextrain_b200.optimizer import FlexTrainCPUOptimizer, FlexTrainOptimizer  # noqa


def test_engine_shims_and_health(fresh_runtime):
    from flextrain_b200.models.llama import preset
    from flextrain_b200.testing import build_llama_engine
    cfg = preset("tiny", num_layers=2, hidden=64, num_heads=2, ffn=128, vocab=128, seq_len=16)
    tok = torch.randint(0, 128, (2, 17))
    ft_cfg = {"batch_size": 2, "micro_batch_size": 2, "mixed_precision": {"device_dtype": "fp32"}}
    model, opt, eng = build_llama_engine(cfg, ft_cfg, lambda: (tok[:, :-1], tok[:, 1:]), backend="gloo")
    calls = []
    eng.register_post_step_function(lambda: calls.append(1))
    assert eng.step() is None and eng.loss_scale == 1.0 and not eng.dynamic_loss_scaling
    eng.override_loss_scale(8.0)
    l0 = float(eng.train_iteration()[0].detach())
    l1 = float(eng.train_iteration()[0].detach())
    assert calls == [1, 1] and eng.loss_scale == 8.0 and l1 < l0    # scale-invariant update
    h = eng.health()
    assert h["global_steps"] == 2 and h["skipped_steps"] == 0 and h["last_step_seconds"] > 0
    assert eng.train() is eng and eng.eval() is eng
    eng.shutdown()


def test_engine_stats_counts_tier_traffic():
    """``engine.stats()`` books the bytes that cross tiers: with parameters and
    optimizer state split over DRAM and NVMe every step must move both."""
    import tempfile
    import torch
    from flextrain_b200.models.llama import preset
    from flextrain_b200.testing import build_llama_engine, reset_runtime
    reset_runtime()
    cfg = preset("tiny", num_layers=3, hidden=64, num_heads=4, ffn=128, vocab=128, seq_len=16)
    data = torch.randint(0, cfg.vocab, (2, cfg.seq_len + 1))
    with tempfile.TemporaryDirectory() as tmp:
        ft_cfg = {"batch_size": 2, "micro_batch_size": 2,
                  "mixed_precision": {"device_dtype": "fp32", "dynamic_loss_scaling": False},
                  "split_ratio": {"parameter": [0.0, 0.5], "optimizer": [0.0, 0.5],
                                  "checkpoint": [0.0, 1.0], "gradient": [0.0, 1.0]},
                  "nvme_swap": {"swap_dir": tmp}}
        model, opt, eng = build_llama_engine(cfg, ft_cfg, lambda: (data[:, :-1], data[:, 1:]),
                                             init_device="cpu", backend="gloo")
        eng.stats(reset=True)
        eng.train_iteration()
        eng.synchronize()
        st = eng.stats()
        tr = st["traffic_bytes"]
        assert tr["nvme_read"] > 0 and tr["nvme_write"] > 0
        assert tr["h2h"] > 0                       # CPU run: tier copies are host to host
        assert st["global_steps"] == 1 and st["last_step_seconds"] > 0
        assert eng.stats(reset=True)["traffic_bytes"]["nvme_read"] == tr["nvme_read"]
        assert eng.stats()["traffic_bytes"]["nvme_read"] == 0
        eng.shutdown()
    reset_runtime()


def test_strict_overflow_skips_the_whole_step():
    """engine.strict_overflow: a non-finite gradient anywhere skips every update
    of that step (layer units and replicated parameters alike) and the next
    clean step proceeds from untouched state."""
    import torch
    from flextrain_b200.llm_func import LLMFunc
    from flextrain_b200.models.llama import preset
    from flextrain_b200.testing import build_llama_engine, reset_runtime
    reset_runtime()
    cfg = preset("tiny", num_layers=3, hidden=64, num_heads=4, ffn=128, vocab=128, seq_len=16)
    data = torch.randint(0, cfg.vocab, (2, cfg.seq_len + 1))
    ft_cfg = {"batch_size": 2, "micro_batch_size": 2,
              "mixed_precision": {"device_dtype": "fp32", "dynamic_loss_scaling": False},
              "split_ratio": {"parameter": [0.0, 1.0], "optimizer": [0.0, 1.0],
                              "checkpoint": [0.0, 1.0], "gradient": [0.0, 1.0]},
              "engine": {"strict_overflow": True}}
    model, opt, eng = build_llama_engine(cfg, ft_cfg, lambda: (data[:, :-1], data[:, 1:]),
                                         init_device="cpu", backend="gloo")
    poison = {"on": False}
    clean_loss = LLMFunc.loss

    def loss(outputs, inputs):
        out = clean_loss(outputs, inputs)
        return out * float("inf") if poison["on"] else out

    LLMFunc.loss = staticmethod(loss)
    try:
        eng.train_iteration()
        eng.synchronize()
        before = [eng.opts.read_states(u)[0].clone() for u in range(eng.num_units)]
        nl_before = eng.optimizer.non_layerwise_state()["master"].clone()
        poison["on"] = True
        eng.train_iteration()
        eng.synchronize()
        assert eng.skipped_steps == 1
        for u in range(eng.num_units):
            assert torch.equal(eng.opts.read_states(u)[0], before[u])
        assert torch.equal(eng.optimizer.non_layerwise_state()["master"], nl_before)
        poison["on"] = False
        first = float(eng.train_iteration()[0].detach())
        eng.synchronize()
        assert first == first and eng.skipped_steps == 1
        assert not torch.equal(eng.opts.read_states(0)[0], before[0])
    finally:
        LLMFunc.loss = staticmethod(clean_loss)
        eng.shutdown()
        reset_runtime()


def test_eval_iteration_is_forward_only_and_matches_the_plain_model(fresh_runtime):
    """Validation pass: the losses equal a plain forward of the same weights, the
    model is in eval mode meanwhile (dropout off) and training resumes unchanged."""
    from flextrain_b200.models.gpt import GPTModel, preset
    from flextrain_b200.testing import build_gpt_engine
    cfg = preset("tiny", num_layers=3, hidden=64, num_heads=2, vocab=128, seq_len=16, dropout=0.2)
    gen = torch.Generator().manual_seed(5)
    batches = [torch.randint(0, 128, (2, 17), generator=gen) for _ in range(32)]
    served = []

    def batch_fn():
        t = batches[len(served)]
        served.append(t)
        return t[:, :-1], t[:, 1:]

    ft_cfg = {"batch_size": 4, "micro_batch_size": 2, "checkpoint_interval": 2,
              "mixed_precision": {"device_dtype": "fp32"},
              "split_ratio": {"parameter": [0.5, 0.5], "optimizer": [0.0, 1.0],
                              "checkpoint": [0.0, 1.0], "gradient": [0.0, 1.0], "alpha": 0.5}}
    model, opt, eng = build_gpt_engine(cfg, ft_cfg, batch_fn, backend="gloo")
    # a plain copy with the same initial weights (same seed, same construction order)
    torch.manual_seed(0)
    plain = GPTModel(cfg).eval()
    got = [float(l) for l in eng.eval_iteration()]
    assert len(got) == 2 and len(served) == 2
    with torch.no_grad():
        want = [float(plain(t[:, :-1], t[:, 1:])) for t in served]
    assert max(abs(a - b) for a, b in zip(got, want)) < 1e-5
    assert model.training                               # mode restored
    three = eng.eval_iteration(micro_batches=3)
    assert len(three) == 3 and len(served) == 5
    # training after a validation pass behaves like training without it
    l_after_eval = [float(l.detach()) for l in eng.train_iteration()]
    assert eng.global_steps == 1 and len(l_after_eval) == 2
    # a pass after the update sees the new weights: the same batch scores differently
    eng.synchronize()
    batches[len(served)] = served[0]
    e2 = float(eng.eval_iteration(micro_batches=1)[0])
    assert e2 == e2 and e2 != got[0] and abs(e2 - got[0]) < 1.0
    eng.shutdown()


def test_optimizer_accepts_bare_tensors_and_single_tensor_groups():
    """The reference iterates its argument as a list of dicts only
    (flextrain/optimizer.py:113-129); here a bare iterable of tensors and a group whose
    ``params`` is one tensor are normalised the way torch.optim does."""
    from flextrain_b200.optimizer import _normalise_param_groups
    a, b = torch.nn.Parameter(torch.zeros(3)), torch.nn.Parameter(torch.zeros(2))
    defaults = {"lr": 1e-3, "weight_decay": 0.01}
    bare = _normalise_param_groups(iter([a, b]), defaults)
    assert len(bare) == 1 and bare[0]["params"] == [a, b] and bare[0]["lr"] == 1e-3
    single = _normalise_param_groups([{"params": a, "lr": 0.5}, {"params": [b]}], defaults)
    assert single[0]["params"] == [a] and single[0]["lr"] == 0.5 and single[1]["weight_decay"] == 0.01
    with pytest.raises(ValueError):
        _normalise_param_groups([], defaults)
