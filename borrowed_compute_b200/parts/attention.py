"""Grouped-query causal attention over the paged cache.

Per row: q, k, v = x Wq^T, x Wk^T, x Wv^T (one fused product); q and k rotated by the
row's position; k and v appended to the sequence's cache; every head attends to the cached
positions of its kv head; the output product adds into the residual stream
(crates/bc-infer/src/model.rs:324-338; launch order crates/bc-infer/src/gpu/mod.rs:456-484).
"""

from __future__ import annotations

from typing import Any, Dict, Mapping, Optional

import torch

from .. import ops
from . import products
from .base import MIXERS, POSITION_ENCODINGS, CacheNeed, Mixer, RunMemory, Runtime, StepContext, TensorSpec


@MIXERS.register("gqa_attention")
class GroupedQueryAttention(Mixer):
    def __init__(self, hidden_size: int, heads: int, kv_heads: int, head_dim: int, position: Mapping[str, Any],
                 window: int = 0, scale: Optional[float] = None):
        super().__init__(hidden_size=hidden_size, heads=heads, kv_heads=kv_heads, head_dim=head_dim, position=position,
                         window=window, scale=scale)
        if heads % kv_heads:
            raise ValueError(f"{heads} heads are not a multiple of {kv_heads} kv heads")
        if head_dim % 16 or head_dim > 256:
            raise ValueError(f"head size {head_dim} is not a multiple of 16 up to 256: the attention kernels refuse it")
        self.hidden_size, self.heads, self.kv_heads, self.head_dim = int(hidden_size), int(heads), int(kv_heads), int(head_dim)
        self.window = int(window)
        self.scale = float(scale) if scale is not None else 1.0 / float(head_dim) ** 0.5
        pos = dict(position)
        self.position = POSITION_ENCODINGS.get(pos.pop("kind"))(**pos)

    def tensors(self) -> Dict[str, TensorSpec]:
        q, kv, e = self.heads * self.head_dim, self.kv_heads * self.head_dim, self.hidden_size
        return {
            "q_proj.weight": TensorSpec((q, e)),
            "k_proj.weight": TensorSpec((kv, e)),
            "v_proj.weight": TensorSpec((kv, e)),
            "o_proj.weight": TensorSpec((e, q)),
        }

    def cache_need(self) -> Optional[CacheNeed]:
        return CacheNeed.keys_values(self.kv_heads, self.head_dim, self.window)

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        super().load(tensors, rt)
        # One product for q, k and v: rows of Wq, then Wk, then Wv.
        self.w_qkv = torch.cat([tensors["q_proj.weight"], tensors["k_proj.weight"], tensors["v_proj.weight"]], dim=0).contiguous()
        self.w_o = tensors["o_proj.weight"].contiguous()
        self.position.load({}, rt)

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx: StepContext, mem: RunMemory) -> None:
        rows = x.shape[0]
        H, G, D = self.heads, self.kv_heads, self.head_dim
        qkv = torch.empty((rows, (H + 2 * G) * D), dtype=x.dtype, device=x.device)
        products.linear(x, self.w_qkv, qkv, products.EPI_STORE, "qkv product")
        table = self.position.rotary()
        att = torch.empty((rows, H * D), dtype=x.dtype, device=x.device)
        if ctx.decode and ops.attention_decode_accepts(H, G, D, qkv.dtype):
            # One token a sequence: rotation and the cache append ride inside the attention kernel.
            ops.attention_decode(qkv, (H + 2 * G) * D, mem.k_pages, mem.v_pages, mem.page_table, ctx.row_pos, ctx.row_slot, att,
                                 H, G, D, window=self.window, scale=self.scale, fuse=2 if mem.writes else 1,
                                 cos_sin=None if table is None else table.cos_sin, pairing=0 if table is None else table.pairing,
                                 reach=ctx.max_total)
        else:
            ops.rope_append(qkv, None if table is None else table.cos_sin, ctx.row_pos, ctx.row_slot, mem.page_table,
                            mem.k_pages, mem.v_pages, H, G, D, 0 if table is None else table.pairing, write_cache=mem.writes)
            self.attend(qkv, att, ctx, mem)
        products.linear(att, self.w_o, residual, products.EPI_ADD_F32, "output product")

    def attend(self, qkv: torch.Tensor, out: torch.Tensor, ctx: StepContext, mem: RunMemory) -> None:
        H, G, D = self.heads, self.kv_heads, self.head_dim
        if not ctx.decode and ops.attention_prefill_accepts(H, G, D, qkv.dtype):
            ops.attention_prefill(qkv, (H + 2 * G) * D, mem.k_pages, mem.v_pages, mem.page_table, ctx.seq_rows, ctx.seq_slot,
                                  ctx.seq_start, out, ctx.seqs, ctx.max_new, H, G, D, window=self.window, scale=self.scale)
            return
        ops.attention_rows(qkv, (H + 2 * G) * D, mem.k_pages, mem.v_pages, mem.page_table, ctx.row_pos, ctx.row_slot, out,
                           H, G, D, window=self.window, scale=self.scale)
