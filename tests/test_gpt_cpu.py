"""GPT family on CPU: op statements against ATen, and a tiny GPT through the
engine (gloo) against plain ``torch.optim.Adam`` step for step."""
import os

import pytest
import torch
import torch.multiprocessing as mp
import torch.nn.functional as TF

from flextrain_b200.models.gpt import GPTConfig, GPTModel, preset
from flextrain_b200.ops import reference as ref

STEPS = 8
TOL = 2e-5


def test_reference_ops_match_aten():
    torch.manual_seed(0)
    x = torch.randn(3, 7, 64)
    w, b = torch.randn(64), torch.randn(64)
    assert torch.allclose(ref.layernorm(x, w, b, 1e-5), TF.layer_norm(x, (64,), w, b, 1e-5), atol=1e-5)
    assert torch.allclose(ref.bias_gelu(x, b), TF.gelu(x + b, approximate="tanh"), atol=1e-6)
    assert torch.equal(ref.bias_add(x, b), x + b)


def test_presets_and_parameter_count():
    cfg = preset("gpt2-small")
    assert cfg.head_dim == 64 and cfg.ffn == 3072
    # 124M-class model: 12 layers x 7.09M + embeddings (padded vocabulary)
    assert 120e6 < cfg.total_numel < 130e6
    tiny = preset("tiny")
    model = GPTModel(tiny)
    assert sum(p.numel() for p in model.parameters()) == tiny.total_numel
    untied = GPTModel(preset("tiny", tie_embeddings=False))
    assert sum(p.numel() for p in untied.parameters()) == preset("tiny", tie_embeddings=False).total_numel
    with pytest.raises(ValueError):
        GPTConfig(hidden=100, num_heads=3)
    with pytest.raises(ValueError):
        model.pre_process(torch.zeros(1, tiny.seq_len + 1, dtype=torch.long))


def test_block_matches_a_plain_torch_block():
    """The fused-QKV block equals the textbook statement of a GPT-2 block."""
    torch.manual_seed(1)
    cfg = preset("tiny")
    model = GPTModel(cfg)
    blk = model.blocks[0]
    for p in (blk.bqkv, blk.bo, blk.b_fc, blk.b_proj, blk.ln1_b, blk.ln2_b):
        torch.nn.init.normal_(p, std=0.1)
    x = torch.randn(2, 16, cfg.hidden)
    H, nh, d = cfg.hidden, cfg.num_heads, cfg.head_dim
    h = TF.layer_norm(x, (H,), blk.ln1_w, blk.ln1_b, cfg.eps)
    q, k, v = (h @ blk.wqkv.T + blk.bqkv).split(H, dim=-1)
    q, k, v = (t.view(2, 16, nh, d).transpose(1, 2) for t in (q, k, v))
    a = TF.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(2, 16, H)
    y = x + a @ blk.wo.T + blk.bo
    h = TF.layer_norm(y, (H,), blk.ln2_w, blk.ln2_b, cfg.eps)
    y = y + TF.gelu(h @ blk.w_fc.T + blk.b_fc, approximate="tanh") @ blk.w_proj.T + blk.b_proj
    assert torch.allclose(blk(x), y, atol=2e-5)


def _data(steps=STEPS, batch=2, seq=128, vocab=1024):
    g = torch.Generator().manual_seed(3)
    return [torch.randint(0, vocab, (batch, seq + 1), generator=g) for _ in range(steps)]


def _reference_losses(cfg, data, lr=1e-3):
    torch.manual_seed(0)
    model = GPTModel(cfg)
    model.train()
    decay = [p for p in model.parameters() if p.dim() > 1]
    no_decay = [p for p in model.parameters() if p.dim() <= 1]
    opt = torch.optim.AdamW([{"params": decay, "weight_decay": 0.01},
                             {"params": no_decay, "weight_decay": 0.0}], lr=lr)
    out = []
    for t in data:
        loss = model(t[:, :-1], t[:, 1:])
        opt.zero_grad()
        loss.backward()
        opt.step()
        out.append(loss.item())
    return out


def _worker(rank, world, port, ft_config, model_kwargs, steps, queue):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.set_num_threads(2)
    from flextrain_b200.testing import build_gpt_engine, reset_runtime
    import flextrain_b200 as ft
    ft.init_distributed(dist_backend="gloo")
    cfg = preset("tiny", **model_kwargs)
    data = _data(steps, batch=ft_config["batch_size"])
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

    model, opt, eng = build_gpt_engine(cfg, ft_config, batch_fn, lr=1e-3, weight_decay=0.01,
                                       adamw_mode=True)
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


def _run(world, ft_config, model_kwargs=None, steps=STEPS):
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = 31500 + (os.getpid() * 7 + world * 13 + len(str(ft_config)) + len(str(model_kwargs))) % 2000
    procs = [ctx.Process(target=_worker, args=(r, world, port, ft_config, model_kwargs or {}, steps, queue))
             for r in range(world)]
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
    cfg.update(over)
    return cfg


def _check(losses, ref_losses):
    worst = max(abs(a - b) for a, b in zip(losses, ref_losses))
    assert len(losses) == len(ref_losses) and worst <= TOL, f"loss differs from AdamW by {worst}"


def test_tied_gpt_world2_matches_adamw():
    """Embedding shared between the first and the last stage: its gradient is the
    sum of both uses and one Adam update is applied."""
    _check(_run(2, _config()), _reference_losses(preset("tiny"), _data()))


def test_untied_gpt_world1_device_tier_interval2():
    cfg = _config(checkpoint_interval=2,
                  split_ratio={"optimizer": [0.5, 0.5], "parameter": [0.3, 0.7],
                               "checkpoint": [1.0, 0.0], "gradient": [1.0, 0.0], "alpha": 0.0})
    _check(_run(1, cfg, {"tie_embeddings": False}),
           _reference_losses(preset("tiny", tie_embeddings=False), _data()))


def test_dropout_masks_are_replayed_in_the_recomputation():
    """One micro-batch per step on one rank draws its dropout masks in the order of a
    plain forward pass; the engine recomputes every unit in backward, so it only
    reproduces plain AdamW if each recomputation sees the masks of its first pass."""
    cfg = _config(batch_size=1)
    data = _data(batch=1)
    _check(_run(1, cfg, {"dropout": 0.1}), _reference_losses(preset("tiny", dropout=0.1), data))
