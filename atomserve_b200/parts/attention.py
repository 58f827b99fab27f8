"""Grouped-query attention over cache pages, with optional per-head RMSNorm of q and k before
the position encoding (Qwen3's form, atomserve/model.py:292-336), an optional sliding window,
and no biases. Sizes, eps, the position encoding and the window are parameters."""

from __future__ import annotations

import torch

from atomserve_b200 import ops
from atomserve_b200.parts.base import CacheView, KVCacheSpec, Mixer, Norm, StepContext, build_part, register_part
from atomserve_b200.parts.spec import PartSpec, TensorSpec


class GQAttention(Mixer):
    def __init__(
        self,
        hidden_size: int,
        prefix: str,
        num_heads: int,
        num_kv_heads: int,
        head_dim: int,
        qk_norm_eps: float | None = None,
        position: PartSpec | None = None,
        window: int | None = None,
        scale: float | None = None,
    ):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads are not a multiple of {num_kv_heads} kv heads")
        self.hidden_size, self.prefix = hidden_size, prefix
        self.num_heads, self.num_kv_heads, self.head_dim = num_heads, num_kv_heads, head_dim
        self.qk_norm_eps = qk_norm_eps
        self.window = window
        self.scale = float(scale) if scale is not None else head_dim**-0.5
        self.position = build_part("position", position, hidden_size) if position else None
        self.qkv_proj = self.o_proj = self.q_gain = self.k_gain = None

    def cache_spec(self) -> KVCacheSpec:
        return KVCacheSpec(self.num_kv_heads, self.head_dim, self.window)

    def tensor_specs(self) -> list[TensorSpec]:
        p, d, hd = self.prefix, self.hidden_size, self.head_dim
        specs = [
            TensorSpec(p + "q_proj.weight", (self.num_heads * hd, d)),
            TensorSpec(p + "k_proj.weight", (self.num_kv_heads * hd, d)),
            TensorSpec(p + "v_proj.weight", (self.num_kv_heads * hd, d)),
            TensorSpec(p + "o_proj.weight", (d, self.num_heads * hd)),
        ]
        if self.qk_norm_eps is not None:
            specs += [
                TensorSpec(p + "q_norm.weight", (hd,), kind="gain", init="gain"),
                TensorSpec(p + "k_norm.weight", (hd,), kind="gain", init="gain"),
            ]
        return specs

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        p = self.prefix
        # q, k and v stacked along the output rows: one product instead of three
        # (atomserve/loader.py:112-116)
        self.qkv_proj = torch.cat([tensors[p + f"{n}_proj.weight"] for n in "qkv"]).contiguous()
        self.o_proj = tensors[p + "o_proj.weight"]
        if self.qk_norm_eps is not None:
            self.q_gain, self.k_gain = tensors[p + "q_norm.weight"], tensors[p + "k_norm.weight"]
        if self.position is not None:
            self.position.prepare(self.o_proj.device)

    def forward(self, h: torch.Tensor, residual: torch.Tensor, ctx: StepContext,
                cache: CacheView | None, write_cache: bool = True) -> torch.Tensor:  # fmt: skip
        return ops.linear(self.attend(h, ctx, cache, write_cache), self.o_proj, residual)

    def forward_then(self, h: torch.Tensor, residual: torch.Tensor, ctx: StepContext, cache: CacheView | None,
                     write_cache: bool, then: Norm) -> tuple[torch.Tensor, torch.Tensor]:  # fmt: skip
        after_linear = getattr(then, "after_linear", None)
        if after_linear is None:
            return super().forward_then(h, residual, ctx, cache, write_cache, then)
        return after_linear(self.attend(h, ctx, cache, write_cache), self.o_proj, residual)

    def attend(self, h: torch.Tensor, ctx: StepContext, cache: CacheView | None, write_cache: bool) -> torch.Tensor:
        """The heads' outputs side by side, [T, H * hd], before the output projection."""
        H, KV, hd = self.num_heads, self.num_kv_heads, self.head_dim
        pos = self.position
        # reading another entry's keys and values, only queries are projected
        weight, kv_heads = (self.qkv_proj, KV) if write_cache else (self.qkv_proj[: H * hd], 0)
        qkv = None
        if ops.qk_norm_rope_store_takes_partial(hd, pos.rotary_dim if pos else None):
            # with few tokens the product stays as the GEMM's partial sums and the next kernel adds them up
            qkv = ops.linear_partial(h, weight)
        if qkv is None:
            qkv = ops.linear(h, weight)
        q = ops.qk_norm_rope_store(
            qkv, H, kv_heads, hd, ctx.positions,
            q_gain=self.q_gain, k_gain=self.k_gain, eps=self.qk_norm_eps or 0.0,
            inv_freq=pos.inv_freq if pos else None, rotary_dim=pos.rotary_dim if pos else 0,
            slots=cache.slots if write_cache else None,
            k_cache=cache.k if write_cache else None, v_cache=cache.v if write_cache else None,
        )  # fmt: skip
        out = ops.paged_attention(
            q, cache.k, cache.v, cache.block_tables, ctx.req_q_start, ctx.req_pos_start,
            num_requests=ctx.num_requests, max_context=ctx.max_context, window=self.window,
            scale=self.scale, host_q_lens=ctx.host_q_lens or None,
        )  # fmt: skip
        return out.view(-1, H * hd)


register_part("mixer", "gqa_attention", GQAttention)
