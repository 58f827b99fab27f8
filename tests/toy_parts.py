"""Parts defined by the tests, registered through the package's public registries.

Two uses. (1) Every hot part again in plain torch (`torch_*` kinds and the architecture
"ToyTorchLM"), reading and writing the paged cache through the same CacheView: with these
the scheduler, cache manager, runner and engine run whole on the CPU. (2) `ema_mixer`, a mixer
with state of its own (one vector per request, kept in the state slots), to show that such a
part is registered, built and stepped without touching the package; `latent_mixer`, a mixer
whose cache pages hold one tensor (a narrow latent per token) instead of keys and values;
`toy_top1_experts`, a feed-forward that routes each token to one of a few small experts;
`toy_interpolated_rotary`, another rotary position encoding (positions compressed by a factor,
only a part of the head rotated) that the package's attention runs through its fused kernel; and
`toy_sqrt_rotation`, an encoding that is no rotation by position x frequency and so applies
itself (`encode`) between the attention part's norm and its cache write.

They follow the package's interfaces and nothing else of it; the oracle stays plain_qwen3.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

import plain_qwen3 as plain
from atomserve_b200.config.registry import register_architecture
from atomserve_b200.parts import (
    CacheView, FeedForward, KVCacheSpec, LayerCall, LayerSpec, Mixer, ModelSpec, Norm, PageSpec, PageTensor, Part,
    PartSpec, PositionEncoding, StateSpec, StepContext, TensorSpec, register_part,
)  # fmt: skip


class TorchRMSNorm(Norm):
    def __init__(self, hidden_size, prefix, eps):
        self.width, self.eps, self.name = hidden_size, eps, prefix + "weight"

    def tensor_specs(self):
        return [TensorSpec(self.name, (self.width,), kind="gain", init="gain")]

    def load(self, tensors):
        self.gain = tensors[self.name]

    def forward(self, x, rows=None):
        if rows is not None:
            x = x[rows.long()]
        return plain.rms_norm(x.float(), self.gain, self.eps).to(x.dtype)


class TorchEmbedding(Part):
    def __init__(self, hidden_size, prefix, vocab_size):
        self.shape, self.name = (vocab_size, hidden_size), prefix + "weight"

    def tensor_specs(self):
        return [TensorSpec(self.name, self.shape)]

    def load(self, tensors):
        self.table = tensors[self.name]

    def forward(self, token_ids):
        return self.table[token_ids.long()]


class TorchHead(Part):
    def __init__(self, hidden_size, prefix, vocab_size, tied):
        self.shape, self.name, self.tied = (vocab_size, hidden_size), prefix + "weight", tied

    def tensor_specs(self):
        return [] if self.tied else [TensorSpec(self.name, self.shape)]

    def load(self, tensors):
        if not self.tied:
            self.weight = tensors[self.name]

    def tie(self, embedding):
        self.weight = embedding.table

    def forward(self, hidden):
        return hidden.float() @ self.weight.float().T


class TorchSwiGLU(FeedForward):
    def __init__(self, hidden_size, prefix, intermediate_size):
        self.d, self.i, self.p = hidden_size, intermediate_size, prefix

    def tensor_specs(self):
        return [TensorSpec(self.p + "gate_proj.weight", (self.i, self.d)),
                TensorSpec(self.p + "up_proj.weight", (self.i, self.d)),
                TensorSpec(self.p + "down_proj.weight", (self.d, self.i))]  # fmt: skip

    def load(self, tensors):
        self.w = {n: tensors[self.p + n + "_proj.weight"] for n in ("gate", "up", "down")}

    def forward(self, h, residual, ctx):
        gate, up = h @ self.w["gate"].T, h @ self.w["up"].T
        return residual + (torch.nn.functional.silu(gate) * up) @ self.w["down"].T


class TorchAttention(Mixer):
    """Paged GQA attention with q/k norm and rotary encoding, one request at a time."""

    def __init__(self, hidden_size, prefix, num_heads, num_kv_heads, head_dim, eps, theta, window=None):
        self.d, self.p, self.H, self.KV, self.hd = hidden_size, prefix, num_heads, num_kv_heads, head_dim
        self.eps, self.theta, self.window = eps, theta, window

    def cache_spec(self):
        return KVCacheSpec(self.KV, self.hd, self.window)

    def tensor_specs(self):
        p, d, hd = self.p, self.d, self.hd
        return [TensorSpec(p + "q_proj.weight", (self.H * hd, d)), TensorSpec(p + "k_proj.weight", (self.KV * hd, d)),
                TensorSpec(p + "v_proj.weight", (self.KV * hd, d)), TensorSpec(p + "o_proj.weight", (d, self.H * hd)),
                TensorSpec(p + "q_norm.weight", (hd,), "gain", "gain"), TensorSpec(p + "k_norm.weight", (hd,), "gain", "gain")]  # fmt: skip

    def load(self, tensors):
        self.w = {n: tensors[self.p + n + ".weight"] for n in ("q_proj", "k_proj", "v_proj", "o_proj", "q_norm", "k_norm")}

    def forward(self, h, residual, ctx, cache, write_cache=True):
        T, H, KV, hd = h.shape[0], self.H, self.KV, self.hd
        angles = plain.rope_angles(ctx.positions.long().cpu(), hd, self.theta).to(h.device)
        q = plain.apply_rope(plain.rms_norm((h @ self.w["q_proj"].T).view(T, H, hd), self.w["q_norm"], self.eps), angles)
        bs = cache.block_size
        if write_cache:
            k = plain.apply_rope(plain.rms_norm((h @ self.w["k_proj"].T).view(T, KV, hd), self.w["k_norm"], self.eps), angles)
            v = (h @ self.w["v_proj"].T).view(T, KV, hd)
            slots = cache.slots.long()
            cache.k[slots // bs, :, slots % bs] = k.to(cache.k.dtype)
            cache.v[slots // bs, :, slots % bs] = v.to(cache.v.dtype)
        out = torch.empty(T, H, hd, dtype=h.dtype, device=h.device)
        row = 0
        for r, (n, start) in enumerate(zip(ctx.host_q_lens, ctx.host_pos_start)):
            end = start + n
            lo = 0 if self.window is None else max(0, start - self.window + 1)
            pos = torch.arange(lo, end, device=h.device)
            blocks = cache.block_tables[r].long()[pos // bs]
            keys, values = cache.k[blocks, :, pos % bs].float(), cache.v[blocks, :, pos % bs].float()
            group = H // KV
            kk, vv = keys.repeat_interleave(group, 1), values.repeat_interleave(group, 1)
            scores = torch.einsum("thd,shd->hts", q[row : row + n].float(), kk) * hd**-0.5
            qpos = torch.arange(start, end, device=h.device)
            visible = pos[None, :] <= qpos[:, None]
            if self.window is not None:
                visible &= pos[None, :] > qpos[:, None] - self.window
            scores = scores.masked_fill(~visible[None], float("-inf"))
            out[row : row + n] = torch.einsum("hts,shd->thd", scores.softmax(-1), vv).to(h.dtype)
            row += n
        return residual + out.view(T, H * hd) @ self.w["o_proj"].T


class EmaMixer(Mixer):
    """A mixer with constant-size state: s_t = decay * s_{t-1} + (1 - decay) * W x_t, y_t = s_t,
    one state vector per request, carried across steps in the request's state slot."""

    def __init__(self, hidden_size, prefix, decay):
        self.d, self.p, self.decay = hidden_size, prefix, decay

    def state_specs(self):
        return [StateSpec("ema", (self.d,), torch.float32)]

    def tensor_specs(self):
        return [TensorSpec(self.p + "in_proj.weight", (self.d, self.d))]

    def load(self, tensors):
        self.w = tensors[self.p + "in_proj.weight"]

    def forward(self, h, residual, ctx, cache, write_cache=True):
        u = (h @ self.w.T).float()
        out = torch.empty_like(u)
        state = cache.state["ema"]
        row = 0
        for n, slot in zip(ctx.host_q_lens, ctx.host_state_slots):
            s = state[slot].clone()
            for t in range(row, row + n):
                s = self.decay * s + (1 - self.decay) * u[t]
                out[t] = s
            state[slot] = s
            row += n
        return residual + out.to(h.dtype)


class LatentMixer(Mixer):
    """A mixer whose pages hold a single tensor: per token one latent vector c_t = W_down x_t of
    width `rank` (one "head"), which serves as key and as value. Output y_t = W_up sum_s
    softmax_s(q_t . c_s / sqrt(rank)) c_s over s <= t, with q_t = W_q x_t."""

    def __init__(self, hidden_size, prefix, rank):
        self.d, self.p, self.rank = hidden_size, prefix, rank

    def cache_spec(self):
        return PageSpec((PageTensor("latent", 1, self.rank),))

    def tensor_specs(self):
        return [TensorSpec(self.p + "down.weight", (self.rank, self.d)), TensorSpec(self.p + "query.weight", (self.rank, self.d)),
                TensorSpec(self.p + "up.weight", (self.d, self.rank))]  # fmt: skip

    def load(self, tensors):
        self.w = {n: tensors[self.p + n + ".weight"] for n in ("down", "query", "up")}

    def forward(self, h, residual, ctx, cache, write_cache=True):
        bs, pages = cache.block_size, cache.pages["latent"]  # [blocks, 1, block_size, rank]
        c, q = h @ self.w["down"].T, (h @ self.w["query"].T).float()
        if write_cache:
            slots = cache.slots.long()
            pages[slots // bs, 0, slots % bs] = c.to(pages.dtype)
        out = torch.empty(h.shape[0], self.rank, dtype=torch.float32, device=h.device)
        row = 0
        for r, (n, start) in enumerate(zip(ctx.host_q_lens, ctx.host_pos_start)):
            pos = torch.arange(start + n, device=h.device)
            latents = pages[cache.block_tables[r].long()[pos // bs], 0, pos % bs].float()  # [start + n, rank]
            scores = q[row : row + n] @ latents.T * self.rank**-0.5
            visible = pos[None, :] <= torch.arange(start, start + n, device=h.device)[:, None]
            out[row : row + n] = scores.masked_fill(~visible, float("-inf")).softmax(-1) @ latents
            row += n
        return residual + out.to(h.dtype) @ self.w["up"].T


def latent_mixer_reference(h: torch.Tensor, down, query, up) -> torch.Tensor:
    """LatentMixer on one whole sequence, in float64, without a cache."""
    h, down, query, up = (t.double() for t in (h, down, query, up))
    c, q = h @ down.T, h @ query.T
    T = h.shape[0]
    scores = (q @ c.T) * down.shape[0] ** -0.5
    scores = scores.masked_fill(torch.arange(T)[None, :] > torch.arange(T)[:, None], float("-inf"))
    return (scores.softmax(-1) @ c) @ up.T


def ema_reference(u: torch.Tensor, decay: float) -> torch.Tensor:
    s, out = torch.zeros_like(u[0]), []
    for t in range(u.shape[0]):
        s = decay * s + (1 - decay) * u[t]
        out.append(s)
    return torch.stack(out)


class Top1Experts(FeedForward):
    """A feed-forward with routing: router logits in float32, each token goes to the expert with
    the largest logit (ties to the lower index) and is scaled by that logit's softmax weight.
    Every expert is a small SwiGLU. All experts run on all tokens and a mask picks, so the step
    has no data-dependent shapes and can be captured in a graph."""

    def __init__(self, hidden_size, prefix, num_experts, expert_size):
        self.d, self.p, self.e, self.i = hidden_size, prefix, num_experts, expert_size

    def tensor_specs(self):
        specs = [TensorSpec(self.p + "router.weight", (self.e, self.d))]
        for x in range(self.e):
            specs += [TensorSpec(self.p + f"experts.{x}.gate_proj.weight", (self.i, self.d)),
                      TensorSpec(self.p + f"experts.{x}.up_proj.weight", (self.i, self.d)),
                      TensorSpec(self.p + f"experts.{x}.down_proj.weight", (self.d, self.i))]  # fmt: skip
        return specs

    def load(self, tensors):
        self.router = tensors[self.p + "router.weight"]
        self.experts = [tuple(tensors[self.p + f"experts.{x}.{n}_proj.weight"] for n in ("gate", "up", "down"))
                        for x in range(self.e)]  # fmt: skip

    def forward(self, h, residual, ctx):
        return residual + top1_experts_reference(h, self.router, self.experts)


def top1_experts_reference(h, router, experts):
    logits = h.float() @ router.float().T
    weight, choice = torch.softmax(logits, dim=-1).max(dim=-1)
    out = torch.zeros_like(h, dtype=torch.float32)
    for x, (gate, up, down) in enumerate(experts):
        y = (torch.nn.functional.silu(h @ gate.T) * (h @ up.T)) @ down.T
        out += y.float() * (weight * (choice == x)).unsqueeze(-1)
    return out.to(h.dtype)


class InterpolatedRotary(PositionEncoding):
    """Rotary encoding with positions divided by `factor` and only the first `rotary_dim`
    elements of a head rotated. It gives the attention part what it asks of a position encoding:
    `prepare(device)`, `inv_freq` (float32, one entry per rotated pair) and `rotary_dim`."""

    def __init__(self, hidden_size, prefix, head_dim, theta, factor, rotary_dim):
        self.head_dim, self.theta, self.factor, self.rotary_dim = head_dim, float(theta), float(factor), rotary_dim
        self.inv_freq = None

    def prepare(self, device):
        exponents = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32) / self.rotary_dim
        self.inv_freq = (1.0 / (self.theta**exponents) / self.factor).to(device)


class SqrtRotation(PositionEncoding):
    """An encoding that is not "angle = position x frequency": pair i of the whole head turns by
    sqrt(position) * theta^(-2i/head_dim). It has no fused form, so the attention part hands it
    the normalised queries and keys (`encode`) and stores what comes back."""

    def __init__(self, hidden_size, prefix, head_dim, theta):
        self.head_dim, self.theta = head_dim, float(theta)

    def encode(self, q, k, ctx):
        turn = lambda x: sqrt_rotation_reference(x, ctx.positions.cpu(), self.theta).to(x.device, x.dtype)  # noqa: E731
        return turn(q), (turn(k) if k is not None else None)


def sqrt_rotation_reference(x, positions, theta):
    """x [T, heads, head_dim] turned as SqrtRotation says, in float64."""
    hd = x.shape[-1]
    x = x.double().cpu()
    inv = 1.0 / (theta ** (torch.arange(0, hd, 2, dtype=torch.float64) / hd))
    angle = positions.double().sqrt()[:, None] * inv[None, :]
    cos, sin = angle.cos()[:, None, :], angle.sin()[:, None, :]
    a, b = x[..., : hd // 2], x[..., hd // 2 :]
    return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)


def interpolated_rotary_reference(x, positions, theta, factor, rotary_dim):
    """x [T, heads, head_dim] rotated as InterpolatedRotary says, in float64."""
    x = x.double()
    inv = 1.0 / (theta ** (torch.arange(0, rotary_dim, 2, dtype=torch.float64) / rotary_dim)) / factor
    angle = positions.double()[:, None] * inv[None, :]
    cos, sin = angle.cos()[:, None, :], angle.sin()[:, None, :]
    half = rotary_dim // 2
    a, b = x[..., :half], x[..., half:rotary_dim]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, x[..., rotary_dim:]], dim=-1)


register_part("norm", "torch_rms_norm", TorchRMSNorm)
register_part("feed_forward", "toy_top1_experts", Top1Experts)
register_part("position", "toy_interpolated_rotary", InterpolatedRotary)
register_part("embedding", "torch_embedding", TorchEmbedding)
register_part("head", "torch_head", TorchHead)
register_part("feed_forward", "torch_swiglu", TorchSwiGLU)
register_part("mixer", "torch_attention", TorchAttention)
register_part("mixer", "ema_mixer", EmaMixer)
register_part("mixer", "latent_mixer", LatentMixer)
register_part("position", "toy_sqrt_rotation", SqrtRotation)


@dataclass(frozen=True)
class ToyConfig:
    """A Qwen3-shaped model whose parts are the torch ones above (same tensor names, so the
    plain implementation is its oracle too)."""

    raw: tuple  # the Qwen3 config dict as sorted items

    architecture = "ToyTorchLM"

    @classmethod
    def from_dict(cls, raw):
        return cls(tuple(sorted((k, tuple(v) if isinstance(v, list) else v) for k, v in raw.items())))

    def to_dict(self):
        return {k: list(v) if isinstance(v, tuple) else v for k, v in self.raw}


def toy_spec(config: ToyConfig) -> ModelSpec:
    c = config.to_dict()
    hd, eps = plain.head_dim_of(c), c["rms_norm_eps"]
    layers = []
    for i in range(c["num_hidden_layers"]):
        p = f"model.layers.{i}."
        layers.append(LayerSpec(
            "pre_norm",
            PartSpec("torch_attention", dict(num_heads=c["num_attention_heads"], num_kv_heads=c["num_key_value_heads"],
                                             head_dim=hd, eps=eps, theta=c["rope_theta"],
                                             window=plain.layer_window(c, i)), p + "self_attn."),
            PartSpec("torch_swiglu", dict(intermediate_size=c["intermediate_size"]), p + "mlp."),
            PartSpec("torch_rms_norm", dict(eps=eps), p + "input_layernorm."),
            PartSpec("torch_rms_norm", dict(eps=eps), p + "post_attention_layernorm."),
        ))  # fmt: skip
    tied = c.get("tie_word_embeddings", False)
    return ModelSpec(
        hidden_size=c["hidden_size"], vocab_size=c["vocab_size"], max_positions=c["max_position_embeddings"],
        embedding=PartSpec("torch_embedding", dict(vocab_size=c["vocab_size"]), "model.embed_tokens."),
        layers=tuple(layers), schedule=tuple(LayerCall(i) for i in range(len(layers))),
        final_norm=PartSpec("torch_rms_norm", dict(eps=eps), "model.norm."),
        head=PartSpec("torch_head", dict(vocab_size=c["vocab_size"], tied=tied), "lm_head."),
        ignored_tensors=("lm_head.weight",) if tied else (),
    )  # fmt: skip


register_architecture("ToyTorchLM", ToyConfig, toy_spec)


def toy_model(cfg: dict, w: dict, device="cpu"):
    """A ToyTorchLM of a Qwen3 config dict with the given float32 checkpoint."""
    from atomserve_b200.parts import build_model

    model = build_model(toy_spec(ToyConfig.from_dict({**cfg, "architectures": ["ToyTorchLM"]})))
    model.load({k: v.to(device) for k, v in w.items()})
    return model


class ArgmaxSampler:
    """Greedy sampling in torch, for engines that run on the CPU in tests."""

    def sample(self, logits, seqs):
        return logits.argmax(-1).tolist() if seqs else []

    def release(self, seq_id):
        pass


class LaunchedArgmax:
    def __init__(self, ids):
        self.device_ids = ids


class TwoPhaseArgmaxSampler(ArgmaxSampler):
    """The same in the two phases of the package's sampler (start a step's sampling, read it
    later), which is what lets the engine launch a step ahead of the one it is reading."""

    def launch(self, logits, seqs, ahead=0):
        return LaunchedArgmax(logits.argmax(-1).to(torch.int32))

    def collect(self, picked):
        return picked.device_ids.tolist()
