"""Grouped-query attention over cache pages, with optional per-head RMSNorm of q and k before
the position encoding (Qwen3's form, atomserve/model.py:292-336), an optional sliding window,
and no biases. Sizes, eps, the position encoding and the window are parameters."""

from __future__ import annotations

import torch

from atomserve_b200 import ops
from atomserve_b200.parts.base import CacheView, KVCacheSpec, Mixer, Norm, PageSpec, StepContext, build_part, register_part
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

    def cache_spec(self) -> PageSpec:
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
        # the position encoding says how it is applied: by the fused kernel below (a rotation by
        # position x frequency), or by its own `encode` on the normalised queries and keys
        rotary = self.position.fused_rotary() if self.position is not None else None
        if self.position is not None and rotary is None:
            q = self._project_encode_store(h, ctx, cache, write_cache)
        else:
            # reading another entry's keys and values, only queries are projected
            weight, kv_heads = (self.qkv_proj, KV) if write_cache else (self.qkv_proj[: H * hd], 0)
            qkv = None
            if ops.qk_norm_rope_store_takes_partial(hd, rotary.rotary_dim if rotary else None):
                # with few tokens the product stays as the GEMM's partial sums and the next kernel adds them up
                qkv = ops.linear_partial(h, weight)
            if qkv is None:
                qkv = ops.linear(h, weight)
            q = ops.qk_norm_rope_store(
                qkv, H, kv_heads, hd, ctx.positions,
                q_gain=self.q_gain, k_gain=self.k_gain, eps=self.qk_norm_eps or 0.0,
                inv_freq=rotary.inv_freq if rotary else None, rotary_dim=rotary.rotary_dim if rotary else 0,
                slots=cache.slots if write_cache else None,
                k_cache=cache.k if write_cache else None, v_cache=cache.v if write_cache else None,
            )  # fmt: skip
        out = ops.paged_attention(
            q, cache.k, cache.v, cache.block_tables, ctx.req_q_start, ctx.req_pos_start,
            num_requests=ctx.num_requests, max_context=ctx.max_context, window=self.window,
            scale=self.scale, host_q_lens=ctx.host_q_lens or None,
        )  # fmt: skip
        return out.view(-1, H * hd)


    def _project_encode_store(self, h: torch.Tensor, ctx: StepContext, cache: CacheView | None, write_cache: bool) -> torch.Tensor:
        """The path for an encoding that is no fused rotation: the same kernel normalises q and k
        without turning or storing them, the encoding's `encode` works the positions in, and a
        second pass of the kernel (no norm, no rotation) writes keys and values to their pages."""
        H, KV, hd = self.num_heads, self.num_kv_heads, self.head_dim
        T = h.shape[0]
        kv_heads = KV if write_cache else 0
        qkv = ops.linear(h, self.qkv_proj if write_cache else self.qkv_proj[: H * hd])
        normed = qkv
        if self.qk_norm_eps is not None:
            heads = qkv.view(T, H + 2 * kv_heads, hd)
            q = ops.rms_norm(heads[:, :H].reshape(T * H, hd), self.q_gain, self.qk_norm_eps).view(T, H, hd)
            k = ops.rms_norm(heads[:, H : H + kv_heads].reshape(T * kv_heads, hd), self.k_gain, self.qk_norm_eps).view(T, kv_heads, hd) if kv_heads else None
        else:
            heads = qkv.view(T, H + 2 * kv_heads, hd)
            q, k = heads[:, :H].contiguous(), (heads[:, H : H + kv_heads].contiguous() if kv_heads else None)
        q, k = self.position.encode(q, k, ctx)
        if not write_cache:
            return q.contiguous()
        normed = torch.cat([q.reshape(T, H * hd), k.reshape(T, KV * hd), qkv[:, (H + KV) * hd :]], dim=1)
        return ops.qk_norm_rope_store(normed, H, KV, hd, ctx.positions, q_gain=None, k_gain=None, eps=0.0, inv_freq=None,
                                      rotary_dim=0, slots=cache.slots, k_cache=cache.k, v_cache=cache.v)  # fmt: skip


register_part("mixer", "gqa_attention", GQAttention)
