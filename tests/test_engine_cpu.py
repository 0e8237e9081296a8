"""End-to-end engine runs on CPU (gloo): a tiny Llama must reproduce plain
``torch.optim.Adam`` step for step under every partition / tier layout."""
import os
import tempfile

import pytest
import torch
import torch.multiprocessing as mp

from flextrain_b200.models.llama import LlamaModel, preset

STEPS = 10
TOL = 1e-5


def _data(steps=STEPS, batch=2, seq=128, vocab=1024):
    g = torch.Generator().manual_seed(1)
    return [torch.randint(0, vocab, (batch, seq + 1), generator=g) for _ in range(steps)]


def _reference_losses(cfg, data, lr=1e-3, weight_decay=0.0, adamw=False):
    torch.manual_seed(0)
    model = LlamaModel(cfg)
    cls = torch.optim.AdamW if adamw else torch.optim.Adam
    decay = [p for p in model.parameters() if p.dim() > 1]
    no_decay = [p for p in model.parameters() if p.dim() <= 1]
    opt = cls([{"params": decay, "weight_decay": weight_decay},
               {"params": no_decay, "weight_decay": 0.0}], lr=lr, betas=(0.9, 0.999), eps=1e-8)
    out = []
    for t in data:
        loss = model(t[:, :-1], t[:, 1:])
        opt.zero_grad()
        loss.backward()
        opt.step()
        out.append(loss.item())
    return out


def _worker(rank, world, port, ft_config, model_kwargs, steps, queue, adamw, weight_decay):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.set_num_threads(2)
    from flextrain_b200.testing import build_llama_engine, reset_runtime
    import flextrain_b200 as ft
    ft.init_distributed(dist_backend="gloo")
    cfg = preset("tiny", **model_kwargs)
    data = _data(steps)
    mbs = ft_config["micro_batch_size"]
    per_rank = ft_config["batch_size"] // world
    cursor = {"step": 0, "mb": 0}

    def batch_fn():
        t = data[cursor["step"]]
        lo = rank * per_rank + cursor["mb"] * mbs
        cursor["mb"] += 1
        if cursor["mb"] * mbs >= per_rank:
            cursor["mb"] = 0
            cursor["step"] += 1
        piece = t[lo:lo + mbs]
        return piece[:, :-1].contiguous(), piece[:, 1:].contiguous()

    model, opt, eng = build_llama_engine(cfg, ft_config, batch_fn, lr=1e-3,
                                         weight_decay=weight_decay, adamw_mode=adamw)
    losses = []
    for _ in range(steps):
        rst = eng.train_iteration()
        local = sum(float(r.detach()) for r in rst) / len(rst)
        losses.append(ft.distributed.all_reduce_scalar(local) / world)
    eng.synchronize()
    eng.shutdown()
    if rank == 0:
        queue.put(losses)
    reset_runtime()


def _run(world, ft_config, model_kwargs=None, steps=STEPS, adamw=False, weight_decay=0.0):
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = 29500 + (os.getpid() * 7 + world * 13 + len(str(ft_config))) % 2000
    procs = [ctx.Process(target=_worker, args=(r, world, port, ft_config, model_kwargs or {}, steps,
                                               queue, adamw, weight_decay)) for r in range(world)]
    for p in procs:
        p.start()
    losses = queue.get(timeout=600)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    return losses


def _config(**over):
    cfg = {"batch_size": 2, "micro_batch_size": 1,
           "mixed_precision": {"device_dtype": "fp32"},
           "split_ratio": {"optimizer": [0.0, 1.0], "parameter": [0.0, 1.0],
                           "checkpoint": [0.0, 1.0], "gradient": [0.0, 1.0], "alpha": 0.25}}
    for k, v in over.items():
        if isinstance(v, dict) and k in cfg:
            cfg[k] = {**cfg[k], **v}
        else:
            cfg[k] = v
    return cfg


def _check(losses, ref, tol=TOL):
    assert len(losses) == len(ref)
    worst = max(abs(a - b) for a, b in zip(losses, ref))
    assert worst <= tol, f"loss differs from torch.optim.Adam by {worst}"


@pytest.fixture(scope="module")
def ref_losses():
    return _reference_losses(preset("tiny"), _data())


def test_baseline_config_world2_all_cpu(ref_losses):
    """Tiny Llama, gloo world 2, fp32, optimizer states 100% on CPU, 10 steps."""
    _check(_run(2, _config()), ref_losses)


def test_world1_two_micro_batches(ref_losses):
    _check(_run(1, _config()), ref_losses)


def test_world2_device_tier_and_interval2(ref_losses):
    cfg = _config(checkpoint_interval=2,
                  split_ratio={"optimizer": [0.5, 0.5], "parameter": [0.3, 0.7],
                               "checkpoint": [1.0, 0.0], "gradient": [1.0, 0.0], "alpha": 0.0})
    _check(_run(2, cfg), ref_losses)


def test_world2_optimizer_ahead_of_parameters(ref_losses):
    """Device Adam share larger than the device parameter share (cross-tier staging)."""
    cfg = _config(split_ratio={"optimizer": [0.6, 0.4], "parameter": [0.25, 0.75],
                               "checkpoint": [0.5, 0.5], "gradient": [0.5, 0.5], "alpha": 0.5})
    _check(_run(2, cfg), ref_losses)


def test_world1_nvme_tiers(ref_losses):
    with tempfile.TemporaryDirectory() as d:
        cfg = _config(nvme_swap={"swap_dir": d, "aio_thread_count": 2},
                      split_ratio={"optimizer": [0.2, 0.3], "parameter": [0.2, 0.3],
                                   "checkpoint": [0.2, 0.3], "gradient": [0.5, 0.5], "alpha": 0.1})
        cfg["batch_size"], cfg["micro_batch_size"] = 2, 1
        _check(_run(1, cfg), ref_losses)
        names = os.listdir(d)
        assert any(n.startswith("rank0_PARA_layer") for n in names)
        assert any(n.startswith("rank0_OPTS_layer") and n.endswith(".swp.0") for n in names)


def test_world1_nvme_optimizer_state_of_a_single_unit(ref_losses):
    """All layers in one unit with its optimizer state half on NVMe: every step reads the file the
    step before wrote, whose write-back is left in flight by the host update - the read must wait
    for it (and the two sets of staging buffers must alternate without mixing steps)."""
    from flextrain_b200.models.llama import preset as _preset
    with tempfile.TemporaryDirectory() as d:
        cfg = _config(nvme_swap={"swap_dir": d, "aio_thread_count": 2},
                      checkpoint_interval=_preset("tiny").num_layers,
                      split_ratio={"optimizer": [0.0, 0.5], "parameter": [0.0, 1.0],
                                   "checkpoint": [0.0, 1.0], "gradient": [0.0, 1.0], "alpha": 0.0})
        _check(_run(1, cfg), ref_losses)
        assert sum(n.startswith("rank0_OPTS_layer") for n in os.listdir(d)) == 3      # master, m, v of one unit


def test_world2_adamw_weight_decay():
    ref = _reference_losses(preset("tiny"), _data(6), weight_decay=0.1, adamw=True)
    cfg = _config(split_ratio={"optimizer": [0.5, 0.5], "parameter": [0.5, 0.5]})
    # decoupled decay differs from torch's foreach kernels by an ulp per step, which
    # the loss amplifies to a few 1e-6 relative; plain Adam above is bit-exact
    _check(_run(2, cfg, steps=6, adamw=True, weight_decay=0.1), ref, tol=1e-4)


def test_world2_four_micro_batches_three_buffers():
    """batch 4 over 2 ranks = 2 micro-batches per rank, with a 3-deep gather ring."""
    data = _data(6, batch=4)
    torch.manual_seed(0)
    ref = _reference_losses(preset("tiny"), data)
    cfg = _config(batch_size=4, engine={"num_unit_buffers": 3})

    # same data generator inside workers: patch through env
    os.environ["FT_TEST_BATCH"] = "4"
    try:
        losses = _run_batch4(cfg, 6)
    finally:
        os.environ.pop("FT_TEST_BATCH", None)
    _check(losses, ref)


def _worker_b4(rank, world, port, ft_config, steps, queue):
    global _data
    orig = _data
    _data = lambda steps=STEPS, batch=4, seq=128, vocab=1024: orig(steps, batch, seq, vocab)  # noqa
    _worker(rank, world, port, ft_config, {}, steps, queue, False, 0.0)


def _run_batch4(ft_config, steps):
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = 29500 + (os.getpid() * 11 + 977) % 2000
    procs = [ctx.Process(target=_worker_b4, args=(r, 2, port, ft_config, steps, queue))
             for r in range(2)]
    for p in procs:
        p.start()
    losses = queue.get(timeout=600)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    return losses


def _worker_b8(rank, world, port, ft_config, steps, queue):
    global _data
    orig = _data
    _data = lambda steps=STEPS, batch=8, seq=128, vocab=1024: orig(steps, batch, seq, vocab)  # noqa
    _worker(rank, world, port, ft_config, {}, steps, queue, False, 0.0)


def test_world8_host_optimizer_and_deferred_updates():
    """Eight ranks (the size of the target box) with every tier on the host and
    alpha-deferred updates: the host-side scheduling (gather order, pinned pool,
    worker thread, heartbeats) must neither stall nor drift from plain Adam."""
    steps = 4
    data = _data(steps, batch=8)
    ref = _reference_losses(preset("tiny"), data)
    cfg = _config(batch_size=8)
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = 29500 + (os.getpid() * 13 + 1531) % 2000
    procs = [ctx.Process(target=_worker_b8, args=(r, 8, port, cfg, steps, queue)) for r in range(8)]
    for p in procs:
        p.start()
    losses = queue.get(timeout=600)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    _check(losses, ref)


def _reference_losses_clipped(cfg, data, clip, lr=1e-3):
    torch.manual_seed(0)
    model = LlamaModel(cfg)
    decay = [p for p in model.parameters() if p.dim() > 1]
    no_decay = [p for p in model.parameters() if p.dim() <= 1]
    opt = torch.optim.Adam([{"params": decay, "weight_decay": 0.0},
                            {"params": no_decay, "weight_decay": 0.0}], lr=lr, betas=(0.9, 0.999), eps=1e-8)
    out, norms = [], []
    for t in data:
        loss = model(t[:, :-1], t[:, 1:])
        opt.zero_grad()
        loss.backward()
        norms.append(float(torch.nn.utils.clip_grad_norm_(model.parameters(), clip)))
        opt.step()
        out.append(loss.item())
    return out, norms


def test_world2_gradient_clipping_by_global_norm():
    """engine.gradient_clipping: one global norm over layer shards of both ranks
    and the replicated parameters, updates held until it is known; must equal
    torch's clip_grad_norm_ + Adam.  The clip value is far below the gradient
    norm of this model (about 1.5), so every step is clipped."""
    clip = 0.25
    ref, norms = _reference_losses_clipped(preset("tiny"), _data(), clip)
    assert min(norms) > clip
    cfg = _config(engine={"gradient_clipping": clip},
                  split_ratio={"optimizer": [0.0, 0.5], "parameter": [0.0, 1.0],
                               "checkpoint": [0.0, 1.0], "gradient": [0.0, 1.0], "alpha": 0.25})
    with tempfile.TemporaryDirectory() as tmp:
        cfg["nvme_swap"] = {"swap_dir": tmp}
        _check(_run(2, cfg), ref, tol=2e-5)


def test_world1_strict_overflow_matches_streaming_updates(ref_losses):
    """engine.strict_overflow without any overflow: same numbers as the
    streaming updates, just applied after backward."""
    _check(_run(1, _config(engine={"strict_overflow": True})), ref_losses)


def test_world2_clipping_with_device_and_nvme_tiers():
    """Deferred updates through every tier at once: device share of the optimizer
    ahead of the device share of the parameters (staged output), host share and
    NVMe share, two ranks, clipping active."""
    clip = 0.25
    ref, _ = _reference_losses_clipped(preset("tiny"), _data(), clip)
    with tempfile.TemporaryDirectory() as tmp:
        cfg = _config(engine={"gradient_clipping": clip},
                      split_ratio={"optimizer": [0.5, 0.3], "parameter": [0.3, 0.5],
                                   "checkpoint": [0.5, 0.5], "gradient": [1.0, 0.0], "alpha": 0.25},
                      nvme_swap={"swap_dir": tmp})
        _check(_run(2, cfg), ref, tol=2e-5)


def test_world1_parameters_in_place_with_host_optimizer(ref_losses):
    """All parameters on the compute device at world size 1 (the engine then computes
    straight from the base copy, no gather) while the optimizer state lives on the host:
    the next step's forward of a unit must wait for that unit's host update to have
    landed in the base copy.  Three buffers and host checkpoints make the forward reach
    the unit early enough to lose the race if it does not."""
    cfg = _config(engine={"num_unit_buffers": 3}, checkpoint_interval=2,
                  split_ratio={"optimizer": [0.0, 1.0], "parameter": [1.0, 0.0],
                               "checkpoint": [0.5, 0.5], "gradient": [1.0, 0.0], "alpha": 0.0})
    for _ in range(2):
        _check(_run(1, cfg), ref_losses)
