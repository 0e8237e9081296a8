"""Logging helpers and the environment report (CPU only)."""
import json
import logging
import types

from flextrain_b200 import env_report
from flextrain_b200.utils import logging as ft_logging


class _Capture(logging.Handler):
    def __init__(self):
        super().__init__()
        self.records = []

    def emit(self, record):
        self.records.append(record)


def _with_capture(fn):
    cap = _Capture()
    ft_logging.logger.addHandler(cap)
    try:
        fn()
    finally:
        ft_logging.logger.removeHandler(cap)
    return cap.records


def test_rank0_logger_is_silent_on_other_ranks(monkeypatch):
    monkeypatch.setenv("RANK", "1")
    assert _with_capture(lambda: ft_logging.rank0_logger.info("hidden")) == []
    monkeypatch.setenv("RANK", "0")
    recs = _with_capture(lambda: ft_logging.rank0_logger.info("shown"))
    assert [r.getMessage() for r in recs] == ["shown"]
    # the record points at the caller, not at the forwarding wrapper
    assert recs[0].filename == "test_logging_and_report.py"


def test_warning_once_emits_once():
    recs = _with_capture(lambda: [ft_logging.warning_once("only once, please") for _ in range(3)])
    assert len(recs) == 1 and recs[0].levelno == logging.WARNING


def test_print_rank0(monkeypatch, capsys):
    monkeypatch.setenv("RANK", "3")
    ft_logging.print_rank0("nope")
    monkeypatch.setenv("RANK", "0")
    ft_logging.print_rank0("yes", 1)
    assert capsys.readouterr().out == "yes 1\n"


def test_log_configuration_lists_public_attributes(monkeypatch):
    monkeypatch.setenv("RANK", "0")
    cfg = types.SimpleNamespace(batch_size=8, _hidden=1, alpha=0.25)
    recs = _with_capture(lambda: ft_logging.log_configuration(cfg, "Demo"))
    text = recs[0].getMessage()
    assert text.splitlines()[0] == "Demo:"
    assert "batch_size" in text and "alpha" in text and "_hidden" not in text


def test_env_report_collects_versions_and_native_state():
    rep = env_report.collect(probe_nvme=True)
    json.dumps(rep)                                   # serialisable
    import torch
    assert rep["torch"] == torch.__version__
    assert rep["target_arch"] == "sm_100a"
    assert set(rep["native"]) == {"ft_host", "ft_cuda"}
    assert rep["native"]["ft_host"]["built"]
    assert rep["nvme_backend"] in ("io_uring", "aio", "psync") or rep["nvme_backend"].startswith("unavailable")
    text = env_report.format_report(rep)
    assert "libft_host.so" in text and "libft_cuda.so" in text


def test_env_report_cli(capsys):
    assert env_report.main(["--json", "--no-nvme"]) == 0
    out = json.loads(capsys.readouterr().out)
    assert "nvme_backend" not in out and out["flextrain_b200"]
