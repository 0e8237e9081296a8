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


# ------------------------------------------------- resume on another world size
def _elastic_worker(rank, world, port, directory, action, steps_before, steps_after, queue):
    import os
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.set_num_threads(2)
    import flextrain_b200 as ft
    from flextrain_b200.models.llama import preset
    from flextrain_b200.testing import build_llama_engine, reset_runtime
    ft.init_distributed(dist_backend="gloo")
    cfg = preset("tiny", num_layers=3, hidden=64, num_heads=2, ffn=136, vocab=128, seq_len=32)
    g = torch.Generator().manual_seed(11)
    data = [torch.randint(0, 128, (4, 33), generator=g) for _ in range(steps_before + steps_after)]
    per_rank = 4 // world
    mbs = min(2, per_rank)
    cursor = {"step": steps_before if action == "load" else 0, "mb": 0}

    def batch_fn():
        t = data[cursor["step"]]
        lo = rank * per_rank + cursor["mb"] * mbs
        cursor["mb"] += 1
        if cursor["mb"] * mbs >= per_rank:
            cursor["mb"], cursor["step"] = 0, cursor["step"] + 1
        return t[lo:lo + mbs, :-1].contiguous(), t[lo:lo + mbs, 1:].contiguous()

    ft_cfg = {"batch_size": 4, "micro_batch_size": mbs, "mixed_precision": {"device_dtype": "fp32"},
              "split_ratio": {"parameter": [0.5, 0.5], "optimizer": [0.25, 0.75],
                              "checkpoint": [1.0, 0.0], "gradient": [1.0, 0.0]}}
    model, opt, eng = build_llama_engine(cfg, ft_cfg, batch_fn, lr=1e-2, weight_decay=0.01)

    def loss():
        r = eng.train_iteration()
        local = sum(float(x.detach()) for x in r) / len(r)
        return ft.distributed.all_reduce_scalar(local) / world

    out = []
    if action == "save":
        for _ in range(steps_before):
            loss()
        eng.save(directory)
    else:
        eng.load(directory)
        assert eng.global_steps == steps_before
    out = [loss() for _ in range(steps_after)]
    eng.synchronize()
    eng.shutdown()
    if rank == 0:
        queue.put(out)
    reset_runtime()


def _elastic(world, directory, action, steps_before=3, steps_after=3):
    import os
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = 27000 + (os.getpid() * 3 + world * 17 + len(action)) % 2000
    procs = [ctx.Process(target=_elastic_worker,
                         args=(r, world, port, directory, action, steps_before, steps_after, queue))
             for r in range(world)]
    for p in procs:
        p.start()
    out = queue.get(timeout=600)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    return out


def test_checkpoint_of_two_ranks_resumes_on_one_and_on_four():
    """Shards are re-cut when the world size changed: the continuation on 1 or 4
    ranks follows the continuation of the 2 ranks that wrote the checkpoint."""
    with tempfile.TemporaryDirectory() as d:
        straight = _elastic(2, d, "save")            # 3 steps, save, 3 more steps
        on_one = _elastic(1, d, "load")
        on_four = _elastic(4, d, "load")
    assert max(abs(a - b) for a, b in zip(on_one, straight)) < 1e-5, (on_one, straight)
    assert max(abs(a - b) for a, b in zip(on_four, straight)) < 1e-5, (on_four, straight)


# --------------------------------------------------- named weights in and out
def _export_worker(rank, world, port, path):
    import os
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.set_num_threads(2)
    import flextrain_b200 as ft
    from flextrain_b200.models.gpt import preset
    from flextrain_b200.testing import build_gpt_engine, reset_runtime
    ft.init_distributed(dist_backend="gloo")
    cfg = preset("tiny", num_layers=3, hidden=64, num_heads=2, vocab=128, seq_len=32)
    g = torch.Generator().manual_seed(21)
    data = [torch.randint(0, 128, (2, 33), generator=g) for _ in range(2)]
    cursor = {"i": 0}

    def batch_fn():
        t = data[cursor["i"]][rank:rank + 1]
        cursor["i"] += 1
        return t[:, :-1].contiguous(), t[:, 1:].contiguous()

    ft_cfg = {"batch_size": 2, "micro_batch_size": 1, "checkpoint_interval": 2,
              "mixed_precision": {"device_dtype": "fp32"},
              "split_ratio": {"parameter": [0.5, 0.5], "optimizer": [0.25, 0.75],
                              "checkpoint": [1.0, 0.0], "gradient": [1.0, 0.0]}}
    model, opt, eng = build_gpt_engine(cfg, ft_cfg, batch_fn, lr=1e-2, weight_decay=0.0, adamw_mode=True)
    for _ in range(2):
        eng.train_iteration()
    sd = eng.export_state_dict()
    assert (sd is not None) == (rank == 0)
    if rank == 0:
        torch.save(sd, path)
    eng.shutdown()
    reset_runtime()


def test_export_gives_the_trained_weights_and_import_restores_them(fresh_runtime):
    import os
    import torch.multiprocessing as mp
    from flextrain_b200.models.gpt import GPTModel, preset
    from flextrain_b200.testing import build_gpt_engine
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "weights.pt")
        ctx = mp.get_context("spawn")
        port = 25000 + os.getpid() % 2000
        procs = [ctx.Process(target=_export_worker, args=(r, 2, port, path)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout=300)
            assert p.exitcode == 0
        exported = torch.load(path)
    # the same two steps with plain AdamW
    cfg = preset("tiny", num_layers=3, hidden=64, num_heads=2, vocab=128, seq_len=32)
    torch.manual_seed(0)
    plain = GPTModel(cfg)
    optim = torch.optim.AdamW(plain.parameters(), lr=1e-2, weight_decay=0.0)
    g = torch.Generator().manual_seed(21)
    data = [torch.randint(0, 128, (2, 33), generator=g) for _ in range(2)]
    for t in data:
        optim.zero_grad()
        plain(t[:, :-1], t[:, 1:]).backward()
        optim.step()
    want = dict(plain.named_parameters())
    assert set(exported) == set(want)
    for name, w in want.items():
        assert exported[name].shape == w.shape
        # Adam turns gradients that are zero up to rounding (key biases) into noise of a
        # fraction of lr: a few elements may sit further out than the rest
        diff = (exported[name] - w.detach()).abs()
        assert float(diff.max()) < 2e-4 and float((diff > 2e-5).float().mean()) < 0.01, name

    # import into a fresh engine with another layout: a validation pass sees those weights
    probe = torch.randint(0, 128, (2, 33), generator=g)
    ft_cfg = {"batch_size": 2, "micro_batch_size": 2, "mixed_precision": {"device_dtype": "fp32"},
              "split_ratio": {"parameter": [0.0, 1.0], "optimizer": [0.0, 1.0],
                              "checkpoint": [0.0, 1.0], "gradient": [0.0, 1.0]}}
    torch.manual_seed(123)                     # different initial weights on purpose
    model, opt, eng = build_gpt_engine(cfg, ft_cfg, lambda: (probe[:, :-1], probe[:, 1:]), seed=123,
                                       backend="gloo")
    before = float(eng.eval_iteration()[0])
    eng.import_state_dict(exported)
    after = float(eng.eval_iteration()[0])
    with torch.no_grad():
        expect = float(plain.eval()(probe[:, :-1], probe[:, 1:]))
    assert abs(after - expect) < 1e-5 and abs(before - expect) > 1e-3
    bad = dict(exported)
    bad.pop("wte")
    try:
        eng.import_state_dict(bad)
        raise AssertionError("a missing parameter must be reported")
    except KeyError:
        pass
    eng.import_state_dict(bad, strict=False)           # keeps the current embedding
    assert abs(float(eng.eval_iteration()[0]) - expect) < 1e-5
    eng.shutdown()
