"""Metrics sink: one JSON line per step with throughput and traffic, Prometheus gauges."""
import json

import torch

from flextrain_b200.utils.metrics import MetricsLog, _loss_value, read_metrics


def test_loss_forms():
    assert _loss_value(None) is None
    assert _loss_value([torch.tensor(1.0), torch.tensor(3.0)]) == 2.0
    assert _loss_value([(torch.tensor(2.0), torch.zeros(3))]) == 2.0          # loss callbacks may return tuples
    assert _loss_value(4.0) == 4.0


def _engine(tmp_path):
    from flextrain_b200.models.llama import preset
    from flextrain_b200.testing import build_llama_engine
    cfg = preset("tiny", num_layers=2, hidden=64, num_heads=2, ffn=136, vocab=128, seq_len=16)
    data = torch.randint(0, 128, (2, 17), generator=torch.Generator().manual_seed(0))
    ft_cfg = {"batch_size": 2, "micro_batch_size": 2, "mixed_precision": {"device_dtype": "fp32"},
              "split_ratio": {"parameter": [0.0, 1.0], "optimizer": [0.0, 1.0], "checkpoint": [0.0, 1.0],
                              "gradient": [0.0, 1.0]},
              "nvme_swap": {"swap_dir": str(tmp_path / "swap")}, "engine": {"gradient_clipping": 1.0}}
    return build_llama_engine(cfg, ft_cfg, lambda: (data[:, :-1].contiguous(), data[:, 1:].contiguous()),
                              lr=1e-3, backend="gloo")


def test_one_record_per_step(fresh_runtime, tmp_path):
    model, opt, eng = _engine(tmp_path)
    path = str(tmp_path / "m.jsonl")
    log = MetricsLog(path, eng, tokens_per_step=32, flops_per_token=1e6, n_gpus=1, extra={"run": "t"})
    for _ in range(3):
        rec = log.step(eng.train_iteration(), note=1)
    log.close()
    eng.shutdown()
    rows = read_metrics(path)
    assert [r["step"] for r in rows] == [1, 2, 3]
    for r in rows:
        assert r["tokens_per_s"] > 0 and r["tflops_per_gpu"] > 0 and r["loss"] > 0
        assert r["run"] == "t" and r["note"] == 1 and r["lr"] == 1e-3 and r["grad_norm"] > 0
        assert isinstance(r["traffic_bytes"], dict)
        json.dumps(r)
    assert rows[-1] == json.loads(json.dumps(rec))
    assert rows[2]["loss"] < rows[0]["loss"]


def test_prometheus_gauges(fresh_runtime, tmp_path):
    model, opt, eng = _engine(tmp_path)
    log = MetricsLog(None, eng, tokens_per_step=32, prometheus_port=0)         # 0: registry only, no server
    log.step(eng.train_iteration())
    eng.shutdown()
    from prometheus_client import generate_latest
    text = generate_latest(log.registry).decode()
    assert "flextrain_step 1.0" in text and "flextrain_tokens_per_s" in text
