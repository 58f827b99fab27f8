"""The plain implementation against the reference engine's own CPU path (stored logits),
and against properties that follow from the formulas."""

import pathlib

import pytest
import torch
from safetensors.torch import load_file

import plain_qwen3 as plain
from tiny_configs import TINY

GOLDEN = pathlib.Path(__file__).parent / "golden"


@pytest.mark.parametrize("name", ["a", "b"])
def test_plain_matches_reference_engine(name):
    cfg, _ = TINY[name]
    gold = load_file(str(GOLDEN / f"qwen3_tiny_{name}.safetensors"))
    w = {k[2:]: v for k, v in gold.items() if k.startswith("w.")}  # the weights the reference ran on
    assert set(w) == set(plain.random_checkpoint(cfg, seed=11))
    ids, other = gold["ids"].tolist(), gold["other"].tolist()
    mine = plain.forward(w, cfg, ids)
    assert (mine - gold["whole"]).abs().max() < 2e-5
    assert (mine - gold["mixed_a"]).abs().max() < 2e-5
    mine_b = plain.forward(w, cfg, other)[: gold["mixed_b"].shape[0]]
    assert (mine_b - gold["mixed_b"]).abs().max() < 2e-5
    assert torch.equal(mine.argmax(-1), gold["whole"].argmax(-1))


def test_float64_oracle_agrees_with_float32():
    cfg, _ = TINY["b"]
    w = plain.random_checkpoint(cfg, seed=3)
    ids = list(range(7, 60))
    a = plain.forward(w, cfg, ids)
    b = plain.forward(w, cfg, ids, dtype=torch.float64)
    assert (a.double() - b).abs().max() < 1e-5


def test_rms_norm_unit_rms_and_gain():
    x = torch.randn(5, 48)
    y = plain.rms_norm(x, torch.ones(48), 0.0)
    assert torch.allclose((y * y).mean(-1), torch.ones(5), atol=1e-5)
    gain = torch.arange(48.0)
    assert torch.allclose(plain.rms_norm(x, gain, 0.0), y * gain, atol=1e-5)


def test_rope_identity_norm_and_relative_distance():
    q, k = torch.randn(1, 1, 32), torch.randn(1, 1, 32)
    zero = plain.rope_angles(torch.tensor([0]), 32, 1e4)
    assert torch.allclose(plain.apply_rope(q, zero), q)

    def dot(m, n):
        a = plain.apply_rope(q, plain.rope_angles(torch.tensor([m]), 32, 1e4))
        b = plain.apply_rope(k, plain.rope_angles(torch.tensor([n]), 32, 1e4))
        return (a * b).sum()

    assert torch.allclose(dot(5, 2), dot(103, 100), atol=1e-4)
    r = plain.apply_rope(q, plain.rope_angles(torch.tensor([77]), 32, 1e4))
    assert torch.allclose(r.norm(), q.norm(), atol=1e-5)


def test_attention_first_token_and_window():
    q, k, v = torch.randn(9, 4, 16), torch.randn(9, 2, 16), torch.randn(9, 2, 16)
    out = plain.attention(q, k, v)
    assert torch.allclose(out[0, 0], v[0, 0], atol=1e-6)
    assert torch.allclose(out[0, 3], v[0, 1], atol=1e-6)
    # a window of 1 sees only itself; a window >= T equals no window
    w1 = plain.attention(q, k, v, window=1)
    assert torch.allclose(w1[:, 0], v[:, 0], atol=1e-6)
    assert torch.allclose(plain.attention(q, k, v, window=9), out, atol=1e-6)
    # a prefix's outputs do not depend on what follows
    assert torch.allclose(plain.attention(q[:5], k[:5], v[:5]), out[:5], atol=1e-6)


def test_attention_rows_is_attention_row_by_row():
    g = torch.Generator().manual_seed(0)
    q, k, v = torch.randn(40, 6, 16, generator=g), torch.randn(40, 2, 16, generator=g), torch.randn(40, 2, 16, generator=g)
    rows = torch.tensor([0, 7, 23, 39])
    for window in (None, 9):
        whole = plain.attention(q, k, v, window)
        assert torch.allclose(plain.attention_rows(q[rows], k, v, rows, window), whole[rows], atol=1e-6)


def test_sampling_distribution_rules():
    logits = torch.tensor([0.4, 0.3, 0.2, 0.1]).log()
    d = plain.sampling_distribution(logits, 1.0, 0, 1.0)
    assert torch.allclose(d, torch.tensor([0.4, 0.3, 0.2, 0.1]), atol=1e-6)
    assert plain.sampling_distribution(logits, 1.0, 2, 1.0).nonzero().flatten().tolist() == [0, 1]
    assert plain.sampling_distribution(logits, 1.0, 0, 0.6).nonzero().flatten().tolist() == [0, 1]
    assert plain.sampling_distribution(logits, 1.0, 0, 0.01).nonzero().flatten().tolist() == [0]
    assert plain.sampling_distribution(logits, 0.0, 20, 0.5).tolist() == [1, 0, 0, 0]
    pen = plain.sampling_distribution(logits, 0.0, 0, 1.0, presence_penalty=2.0, generated=[0, 0])
    assert pen.argmax() == 1
