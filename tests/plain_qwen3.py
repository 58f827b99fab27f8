"""Plain, slow Qwen3 (dense) in PyTorch: the oracle that every engine test compares with.

Whole sequences, no cache, no batching, one function per part, nothing imported from the
package under test. Each function is written from the formulas of the reference engine
(aneesh-sathe/atomserve) and cites the place, as `file:line` inside that project.

Weights are a dict from checkpoint tensor name to tensor (the names a Qwen3 checkpoint
uses, atomserve/loader.py:108-128); the configuration is the parsed config.json dict.
All arithmetic runs in `dtype` (float32 by default; float64 gives a tighter oracle).

The sliding window is the one thing without a counterpart in the reference, which
rejects windowed checkpoints (atomserve/config.py:43-44). Its rule here: a query at
position p sees keys at positions j with p - window < j <= p.
"""

from __future__ import annotations

import math

import torch


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """weight * x / sqrt(mean(x^2) + eps) over the last dim; no mean subtraction, no bias,
    plain weight (not 1 + weight). atomserve/model.py:125-139."""
    variance = (x * x).mean(dim=-1, keepdim=True)
    return weight * (x * torch.rsqrt(variance + eps))


def rope_inv_freq(head_dim: int, theta: float) -> torch.Tensor:
    """Frequency of pair i of head_dim/2 pairs: theta^(-2i/head_dim), computed in float32.
    atomserve/model.py:142-148."""
    exponents = torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim
    return 1.0 / (theta**exponents)


def rope_angles(positions: torch.Tensor, head_dim: int, theta: float) -> torch.Tensor:
    """angle[t, i] = position_t * inv_freq_i in float32, duplicated to head_dim columns.
    atomserve/model.py:165-168."""
    inv_freq = rope_inv_freq(head_dim, theta)
    angles = positions.to(torch.float32)[:, None] * inv_freq[None, :]
    return torch.cat([angles, angles], dim=-1)


def apply_rope(x: torch.Tensor, angles: torch.Tensor) -> torch.Tensor:
    """Rotate-half pairing (i, i + head_dim/2): (a cos - b sin, b cos + a sin).
    x: [T, heads, head_dim], angles: [T, head_dim]. atomserve/model.py:172-185; the kernel
    form keeps cos/sin in float32 and rounds once (atomserve/kernels.py:115-124)."""
    half = x.shape[-1] // 2
    cos = angles.cos().to(x.dtype)[:, None, :]
    sin = angles.sin().to(x.dtype)[:, None, :]
    rotated = torch.cat([-x[..., half:], x[..., :half]], dim=-1)
    return x * cos + rotated * sin


def attention(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int | None = None
) -> torch.Tensor:
    """Causal grouped-query attention of one whole sequence, longhand.

    q: [T, H, hd]; k, v: [T, KV, hd]. Query head j uses kv head j // (H / KV)
    (atomserve/model.py:230 `enable_gqa`; longhand tests/test_model_unit.py:58-60). A query at
    position p sees keys 0..p (atomserve/model.py:222-224); scale head_dim^-0.5
    (atomserve/kernels.py:680); softmax over keys; no softcap, no sinks.
    """
    T, H, hd = q.shape
    group = H // k.shape[1]
    k = k.repeat_interleave(group, dim=1)
    v = v.repeat_interleave(group, dim=1)
    scores = torch.einsum("thd,shd->hts", q, k) * hd**-0.5
    pos = torch.arange(T)
    visible = pos[None, :] <= pos[:, None]
    if window is not None:
        visible &= pos[None, :] > pos[:, None] - window
    scores = scores.masked_fill(~visible[None], float("-inf"))
    probs = torch.softmax(scores, dim=-1)
    return torch.einsum("hts,shd->thd", probs, v)


def attention_rows(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, positions: torch.Tensor,
                   window: int | None = None) -> torch.Tensor:  # fmt: skip
    """`attention` for a few queries of a long sequence: q [n, H, hd] are the queries at
    `positions` [n]; k, v [S, KV, hd] hold every key of the sequence. The same formula row by
    row (query at p sees keys j <= p, and j > p - window with a window; head j uses kv head
    j // group; scale head_dim^-0.5; atomserve/model.py:222-231), without the S x S scores that
    whole long sequences would need."""
    n, H, hd = q.shape
    group = H // k.shape[1]
    k = k.repeat_interleave(group, dim=1).transpose(0, 1)  # [H, S, hd]
    v = v.repeat_interleave(group, dim=1).transpose(0, 1)
    out = torch.empty_like(q)
    for i in range(n):
        p = int(positions[i])
        first = 0 if window is None else max(0, p - window + 1)
        scores = torch.einsum("hd,hsd->hs", q[i], k[:, first : p + 1]) * hd**-0.5
        out[i] = torch.einsum("hs,hsd->hd", torch.softmax(scores, dim=-1), v[:, first : p + 1])
    return out


def _same(x: torch.Tensor) -> torch.Tensor:
    return x


def attention_block(
    x: torch.Tensor, w: dict, prefix: str, cfg: dict, positions: torch.Tensor, window: int | None,
    rnd=_same,
) -> torch.Tensor:  # fmt: skip
    """q/k/v projections, per-head RMSNorm of q and k before RoPE (one [hd] gain for all
    heads, v untouched), attention, output projection. atomserve/model.py:292-336.
    `rnd` rounds every intermediate result (see `forward`)."""
    T = x.shape[0]
    H, KV, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], head_dim_of(cfg)
    q = rnd(x @ w[prefix + "self_attn.q_proj.weight"].T).view(T, H, hd)
    k = rnd(x @ w[prefix + "self_attn.k_proj.weight"].T).view(T, KV, hd)
    v = rnd(x @ w[prefix + "self_attn.v_proj.weight"].T).view(T, KV, hd)
    q = rnd(rms_norm(q, w[prefix + "self_attn.q_norm.weight"], cfg["rms_norm_eps"]))
    k = rnd(rms_norm(k, w[prefix + "self_attn.k_norm.weight"], cfg["rms_norm_eps"]))
    angles = rope_angles(positions, hd, cfg["rope_theta"])
    q, k = rnd(apply_rope(q, angles)), rnd(apply_rope(k, angles))
    out = rnd(attention(q, k, v, window))
    return out.reshape(T, H * hd) @ w[prefix + "self_attn.o_proj.weight"].T


def swiglu_mlp(x: torch.Tensor, w: dict, prefix: str, rnd=_same) -> torch.Tensor:
    """down( silu(gate(x)) * up(x) ), silu(g) = g / (1 + exp(-g)). atomserve/model.py:339-360,
    atomserve/kernels.py:447-448."""
    gate = rnd(x @ w[prefix + "mlp.gate_proj.weight"].T)
    up = rnd(x @ w[prefix + "mlp.up_proj.weight"].T)
    return rnd((gate / (1.0 + torch.exp(-gate))) * up) @ w[prefix + "mlp.down_proj.weight"].T


def head_dim_of(cfg: dict) -> int:
    """head_dim, by default hidden_size // num_attention_heads. atomserve/config.py:55."""
    return cfg.get("head_dim", cfg["hidden_size"] // cfg["num_attention_heads"])


def layer_window(cfg: dict, layer: int) -> int | None:
    """Window of a layer: `sliding_window` for layers >= max_window_layers when
    use_sliding_window is set, else none (no counterpart in the reference)."""
    if cfg.get("use_sliding_window") and layer >= cfg.get("max_window_layers", 0):
        return cfg["sliding_window"]
    return None


def forward(
    w: dict, cfg: dict, ids: list[int], dtype: torch.dtype = torch.float32,
    activations: torch.dtype | None = None,
) -> torch.Tensor:  # fmt: skip
    """Logits at every position of one whole sequence: [len(ids), vocab].

    Embedding gather without scaling; per layer x = x + attn(norm(x)), x = x + mlp(norm(x));
    final norm; lm_head, which is the embedding when tie_word_embeddings.
    atomserve/model.py:363-385, atomserve/loader.py:131-138.

    `activations=torch.bfloat16` rounds the result of every operation to bfloat16, as the
    reference's PyTorch path does when it serves in bf16 (atomserve/cli.py:56-60): the
    yardstick for how far a bfloat16 engine may lie from the float32 logits."""
    w = {name: t.to(dtype) for name, t in w.items()}
    rnd = _same if activations is None else (lambda t: t.to(activations).to(dtype))
    eps = cfg["rms_norm_eps"]
    positions = torch.arange(len(ids))
    x = w["model.embed_tokens.weight"][torch.tensor(ids, dtype=torch.long)]
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        h = rnd(rms_norm(x, w[p + "input_layernorm.weight"], eps))
        x = rnd(x + attention_block(h, w, p, cfg, positions, layer_window(cfg, i), rnd))
        h = rnd(rms_norm(x, w[p + "post_attention_layernorm.weight"], eps))
        x = rnd(x + swiglu_mlp(h, w, p, rnd))
    x = rnd(rms_norm(x, w["model.norm.weight"], eps))
    head = "model.embed_tokens.weight" if cfg.get("tie_word_embeddings", False) else "lm_head.weight"
    return x @ w[head].T


def greedy_generate(w: dict, cfg: dict, prompt: list[int], max_tokens: int) -> list[int]:
    """Greedy decoding by recomputing the whole sequence for every token."""
    ids = list(prompt)
    for _ in range(max_tokens):
        ids.append(int(forward(w, cfg, ids)[-1].argmax()))
    return ids[len(prompt) :]


def sampling_distribution(
    logits: torch.Tensor,
    temperature: float,
    top_k: int,
    top_p: float,
    presence_penalty: float = 0.0,
    generated: list[int] | None = None,
) -> torch.Tensor:
    """The distribution one row is sampled from, dense over the vocabulary [vocab].

    Order of the steps (atomserve/sampler.py:82-118, 144-168): the presence penalty is subtracted
    once from every distinct generated token; top-k on raw logits (0 or >= vocab: all;
    temperature 0: the single best); divide by the temperature; softmax over the kept; top-p
    drops a token once the mass ranked above it reaches top_p (the best always stays). The
    draw picks token i with probability p_i / sum(p) (exponential race, :120-129).
    """
    logits = logits.to(torch.float32).clone()
    vocab = logits.shape[0]
    if presence_penalty != 0 and generated:
        for token in set(generated):
            logits[token] -= presence_penalty
    k = 1 if temperature == 0 else top_k if 0 < top_k < vocab else vocab
    values, indices = torch.sort(logits, descending=True, stable=True)
    values, indices = values[:k], indices[:k]
    probs = torch.softmax(values / (temperature if temperature > 0 else 1.0), dim=-1)
    mass_before = probs.cumsum(dim=-1) - probs
    probs = probs.masked_fill(mass_before >= top_p, 0.0) if temperature > 0 else probs
    dense = torch.zeros(vocab)
    dense[indices] = probs
    return dense / dense.sum()


def random_checkpoint(cfg: dict, seed: int) -> dict:
    """Seeded float32 tensors under checkpoint names: matrices N(0, 0.02), norm gains
    1 + N(0, 0.1). Test-side generator, independent of the package's own."""
    g = torch.Generator().manual_seed(seed)
    d, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    H, KV, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], head_dim_of(cfg)

    def mat(*shape):
        return torch.randn(*shape, generator=g) * 0.02

    def gain(n):
        return 1.0 + torch.randn(n, generator=g) * 0.1

    w = {"model.embed_tokens.weight": mat(V, d)}
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        w[p + "input_layernorm.weight"] = gain(d)
        w[p + "self_attn.q_proj.weight"] = mat(H * hd, d)
        w[p + "self_attn.k_proj.weight"] = mat(KV * hd, d)
        w[p + "self_attn.v_proj.weight"] = mat(KV * hd, d)
        w[p + "self_attn.q_norm.weight"] = gain(hd)
        w[p + "self_attn.k_norm.weight"] = gain(hd)
        w[p + "self_attn.o_proj.weight"] = mat(d, H * hd)
        w[p + "post_attention_layernorm.weight"] = gain(d)
        w[p + "mlp.gate_proj.weight"] = mat(I, d)
        w[p + "mlp.up_proj.weight"] = mat(I, d)
        w[p + "mlp.down_proj.weight"] = mat(d, I)
    w["model.norm.weight"] = gain(d)
    if not cfg.get("tie_word_embeddings", False):
        w["lm_head.weight"] = mat(V, d)
    return w


def _self_check() -> None:
    cfg = dict(
        vocab_size=50, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
        num_attention_heads=4, num_key_value_heads=2, head_dim=8, rms_norm_eps=1e-6,
        rope_theta=1e4, tie_word_embeddings=True,
    )  # fmt: skip
    w = random_checkpoint(cfg, 0)
    out = forward(w, cfg, [1, 2, 3, 4, 5])
    assert out.shape == (5, 50) and math.isfinite(float(out.abs().max()))


if __name__ == "__main__":
    _self_check()
    print("ok")
