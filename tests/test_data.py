"""Token file and micro-batch feeder (CPU)."""
import numpy as np
import pytest
import torch

from flextrain_b200.data import MicroBatchFeeder, SyntheticTokens, TokenFile


def _file(tmp_path, n=5000, suffix=".u16"):
    return TokenFile.write(str(tmp_path / f"tokens{suffix}"), np.arange(n) % 60000)


def test_token_file_round_trip_and_bounds(tmp_path):
    tf = _file(tmp_path)
    assert len(tf) == 5000
    assert np.array_equal(tf.window(10, 5), np.arange(10, 15))
    with pytest.raises(IndexError):
        tf.window(4999, 2)
    with pytest.raises(ValueError):
        TokenFile.write(str(tmp_path / "bad.u16"), [70000])
    wide = TokenFile.write(str(tmp_path / "wide.u32"), [70000, 1, 2])
    assert wide.window(0, 3).tolist() == [70000, 1, 2]
    with pytest.raises(ValueError):
        TokenFile(str(tmp_path / "tokens.u16").replace(".u16", ".dat"))


def test_feeder_windows_are_shifted_labels_and_deterministic(tmp_path):
    tf = _file(tmp_path)
    a = MicroBatchFeeder(tf, micro_batch_size=3, seq_len=16, rank=0, world=2, seed=7)
    b = MicroBatchFeeder(tf, micro_batch_size=3, seq_len=16, rank=0, world=2, seed=7)
    other = MicroBatchFeeder(tf, micro_batch_size=3, seq_len=16, rank=1, world=2, seed=7)
    for n in range(5):
        tok, lab = a()
        tok2, lab2 = b()
        assert tok.shape == (3, 16) and tok.dtype == torch.int64
        assert torch.equal(tok[:, 1:], lab[:, :-1])                 # labels = tokens shifted by one
        assert torch.equal(tok, tok2) and torch.equal(lab, lab2)
        # the file holds consecutive integers: a window is start .. start + 16
        starts = a.window_starts(n)
        assert torch.equal(tok[:, 0], torch.from_numpy(starts))
        assert torch.equal(lab[:, -1], tok[:, 0] + 16)
        assert not torch.equal(tok, other()[0])
    for f in (a, b, other):
        f.close()


def test_feeder_resume_continues_the_stream(tmp_path):
    tf = _file(tmp_path)
    full = MicroBatchFeeder(tf, 2, 8, seed=1, depth=3)
    want = [full()[0].clone() for _ in range(7)]
    first = MicroBatchFeeder(tf, 2, 8, seed=1, depth=3)
    for _ in range(4):
        first()
    state = first.state_dict()
    assert state["consumed"] == 4
    second = MicroBatchFeeder(tf, 2, 8, seed=1, depth=2)
    second.load_state_dict(state)
    got = [second()[0] for _ in range(3)]
    assert all(torch.equal(g, w) for g, w in zip(got, want[4:]))
    with pytest.raises(ValueError):
        MicroBatchFeeder(tf, 2, 8, seed=2).load_state_dict(state)
    for f in (full, first, second):
        f.close()


def test_returned_batches_survive_buffer_reuse(tmp_path):
    """A batch handed out stays intact while later ones are prepared into the same buffers."""
    tf = _file(tmp_path)
    f = MicroBatchFeeder(tf, 2, 8, depth=1)
    kept = [f() for _ in range(4)]
    again = MicroBatchFeeder(tf, 2, 8, depth=1)
    for tok, lab in kept:
        t2, l2 = again()
        assert torch.equal(tok, t2) and torch.equal(lab, l2)
    f.close()
    again.close()


def test_synthetic_tokens_and_argument_checks(tmp_path):
    f = MicroBatchFeeder(SyntheticTokens(100), 4, 32, seed=3)
    tok, lab = f()
    assert tok.max() < 100 and tok.min() >= 0 and torch.equal(tok[:, 1:], lab[:, :-1])
    f.close()
    with pytest.raises(ValueError):
        MicroBatchFeeder(SyntheticTokens(100), 0, 32)
    with pytest.raises(ValueError):
        MicroBatchFeeder(SyntheticTokens(100), 1, 32, rank=2, world=2)
    with pytest.raises(ValueError):
        MicroBatchFeeder(_file(tmp_path, n=10), 1, 32)
    with pytest.raises(ValueError):
        SyntheticTokens(1)
