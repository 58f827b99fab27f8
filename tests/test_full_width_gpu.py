"""Layers of the served width against the plain implementation, in every way of cutting.

Two layers with the sizes of Qwen3-8B (hidden 4,096; 32 query and 8 kv heads of 128; intermediate
12,288; rope theta 1e6; untied head) and a vocabulary of 8,000, random weights, replayed through
the trace replayer (the loader, cache manager, step function and kernels that generation uses)
and held to `plain_qwen3.forward` on the CPU, in float32 and in bfloat16: each request whole; its
last 32 tokens one by one; portions of changing size down to two tokens; and up to four live
requests mixed, portions of some beside single tokens of others, in a pool so small that pages
are used again (the reference's analogue on its own engine: tests/test_runner.py:103-141).

Only these widths pick the GEMM's other plans, so the steps are sized to meet each of them as
part of a model: 1 to 8 tokens (weights as the MMA's rows, K cut, partial sums added up by the
consumer), 33 to 64 and 65 to 256 (swapped with wider token tiles), 257 to 512 (the unswapped
form on few tiles) and more than 512 tokens in a step.
"""

import numpy as np
import pytest

from helpers import Oracle, check, checkpoint, mixed_trace, prompts, write_folder

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]

WIDE = dict(
    architectures=["Qwen3ForCausalLM"], vocab_size=8000, hidden_size=4096, intermediate_size=12288,
    num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
    rms_norm_eps=1e-6, rope_theta=1000000.0, tie_word_embeddings=False,
    max_position_embeddings=4096, hidden_act="silu",
)  # fmt: skip
BLOCK_SIZE = 16
LENGTHS = [700, 300, 90, 45]  # whole: a step of more than 512, of 257-512, of 65-256 and of 33-64 tokens


@pytest.fixture(scope="module")
def wide(tmp_path_factory):
    w = checkpoint(WIDE, seed=31)
    folder = write_folder(WIDE, w, tmp_path_factory.mktemp("wide"))
    ps = prompts(WIDE, LENGTHS, seed=12)
    return folder, ps, [Oracle(w, WIDE, p) for p in ps]


def replayer(folder, dtype, max_tokens):
    from atomserve_b200.engine.replay import TraceReplayer

    return TraceReplayer(folder, dtype, max_tokens, BLOCK_SIZE)


def pool_for(ps, live):
    return sum(sorted((-(-len(p) // 64) * 64 for p in ps), reverse=True)[:live])


@pytest.mark.parametrize("dtype", DTYPES)
def test_whole_then_last_32_one_by_one(wide, dtype):
    folder, ps, oracle = wide
    rp = replayer(folder, dtype, pool_for(ps, 1))
    for i, (p, ref) in enumerate(zip(ps, oracle)):
        logits = rp.step([dict(id=f"w{i}", tokens=p, want=list(range(len(p))))], end=[f"w{i}"])
        check(logits, ref, dtype, f"wide request {i} whole")
    for i, (p, ref) in enumerate(zip(ps, oracle)):
        head = len(p) - 32
        logits = rp.step([dict(id=i, tokens=p[:head], want=[head - 1])], end=[])
        check(logits, ref[head - 1 : head], dtype, f"wide request {i} head")
        for j in range(head, len(p)):
            logits = rp.step([dict(id=i, tokens=[p[j]], want=[0])], end=[i] if j == len(p) - 1 else [])
            check(logits, ref[j : j + 1], dtype, f"wide request {i} position {j}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_portions_of_changing_size(wide, dtype):
    folder, ps, oracle = wide
    rp = replayer(folder, dtype, pool_for(ps, 1))
    sizes = [520, 2, 40, 130, 7, 300, 3, 64, 33, 257]
    for i, (p, ref) in enumerate(zip(ps, oracle)):
        at, k = 0, 2 * i
        while at < len(p):
            n = min(sizes[k % len(sizes)], len(p) - at)
            k += 1
            last = at + n == len(p)
            logits = rp.step([dict(id=i, tokens=p[at : at + n], want=list(range(n)))], end=[i] if last else [])
            check(logits, ref[at : at + n], dtype, f"wide request {i} portion {at}:{at + n}")
            at += n


@pytest.mark.parametrize("dtype", DTYPES)
def test_mixed_requests_reusing_pages(wide, dtype):
    """Every request three times over, four live at a time; the portions run to 300 tokens, so a
    mixed step holds anything from a handful of tokens to several hundred."""
    folder, ps, oracle = wide
    ps3, oracle3 = ps * 3, oracle * 3
    rp = replayer(folder, dtype, pool_for(ps3, 4))  # any four of them fit: 2,432 of the 3,405 tokens
    rng = np.random.default_rng(17)
    step_sizes = []
    for entries, end in mixed_trace(ps3, rng, largest=300):
        logits = rp.step([dict(id=e["id"], tokens=e["tokens"], want=e["want"]) for e in entries], end=end)
        row = 0
        for e in entries:
            n = len(e["tokens"])
            check(logits[row : row + n], oracle3[e["id"]][e["at"] : e["at"] + n], dtype,
                  f"wide request {e['id']} at {e['at']}")  # fmt: skip
            row += n
        step_sizes.append(row)
    assert sum(len(p) for p in ps3) > rp.cache.num_blocks * BLOCK_SIZE, "the pool never had to reuse a page"
    met = {(s > 8) + (s > 32) + (s > 64) + (s > 256) + (s > 512) for s in step_sizes}
    assert {0, 3, 4} <= met, f"mixed steps of {sorted(set(step_sizes))} tokens miss a GEMM plan"
