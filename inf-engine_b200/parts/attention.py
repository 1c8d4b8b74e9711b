"""Grouped-query causal attention over the paged cache
(engine/llama_attention.py:83-141).

q, k and v come from one matrix product over the row-concatenated weights;
a fused kernel rotates q and k and writes k and v into the pages of the step's
tokens; the attention kernel then reads every key and value through the block
table, so a prompt portion, a decode token and a whole prompt take the same
path.  kv head c serves query heads c*g .. c*g+g-1 (:27-44) inside the kernel;
nothing is expanded in memory.  Scores are scaled by head_dim**-0.5 (the
library default the reference relies on, :123-137).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import kernels
from ..cache.manager import CacheRequirement
from ..weights.loader import ExpectedTensor
from .linear import Linear, stream_into_residual, stream_normed
from .registry import build_position, position_class, register_mixer


@dataclass
class CacheView:
    """The cache of one run of a layer, as its mixer sees it."""

    kind: str                               # "kv" | "state" | "none"
    group: int = -1                         # index of the kv group (for block tables and slots in ctx)
    k: torch.Tensor | None = None           # [n_pages, n_kv_heads, page_size, head_dim]
    v: torch.Tensor | None = None
    state: torch.Tensor | None = None       # [max_requests, *state_shape]
    write: bool = True                      # False: this run reads another run's cache


@register_mixer("attention")
class PagedAttention:
    graph_safe = True

    @staticmethod
    def expected_tensors(spec):
        out = {
            spec.q_proj: ExpectedTensor((spec.n_heads * spec.head_dim, spec.hidden)),
            spec.k_proj: ExpectedTensor((spec.n_kv_heads * spec.head_dim, spec.hidden)),
            spec.v_proj: ExpectedTensor((spec.n_kv_heads * spec.head_dim, spec.hidden)),
            spec.o_proj: ExpectedTensor((spec.hidden, spec.n_heads * spec.head_dim)),
        }
        out.update(position_class(spec.position).expected_tensors(spec.position))
        return out

    def __init__(self, spec, tensors, rt):
        if spec.n_heads % spec.n_kv_heads:
            raise ValueError(f"{spec.n_heads} query heads are not a multiple of {spec.n_kv_heads} kv heads")
        if spec.head_dim % 16 or spec.head_dim > 256:
            raise ValueError(f"attention kernels take head sizes in steps of 16 up to 256, not {spec.head_dim}")
        if spec.window is not None and spec.window <= 0:
            raise ValueError("an attention window must be positive")
        self.spec = spec
        self.rt = rt
        ws = [tensors[spec.q_proj], tensors[spec.k_proj], tensors[spec.v_proj]]
        dtype = torch.float32 if any(w.dtype is torch.float32 for w in ws) else ws[0].dtype
        self.qkv = Linear(torch.cat([w.to(dtype) for w in ws], dim=0).contiguous(), rt, "qkv")
        self.o = Linear(tensors[spec.o_proj], rt, "o")
        self.position = build_position(spec.position, tensors, rt)
        self.scale = float(spec.head_dim) ** -0.5
        self.q_width = spec.n_heads * spec.head_dim
        self.kv_width = spec.n_kv_heads * spec.head_dim

    def cache_requirement(self) -> CacheRequirement:
        s = self.spec
        return CacheRequirement(kind="kv", n_kv_heads=s.n_kv_heads, head_dim=s.head_dim, window=s.window,
                                dtype=self.rt.act_dtype)

    def can_fuse(self, n_tokens: int, norm) -> bool:
        return hasattr(norm, "fusable_rms") and self.qkv.streams(n_tokens, normed=True) and self.o.streams(n_tokens)

    def forward_fused(self, residual: torch.Tensor, norm, ctx, cache: CacheView) -> None:
        """residual += o(attention(qkv(norm(residual)))): the norm rides in the qkv product's prologue and the
        residual sum in the output product's epilogue."""
        rt = self.rt
        n = residual.shape[0]
        qkv = rt.ws.take("attn_qkv", (n, self.q_width + 2 * self.kv_width), rt.act_dtype)
        stream_normed(self.qkv, residual, qkv, n, "bf16", norm, ctx)
        out = self._rotate_write_attend(qkv, ctx, cache)
        stream_into_residual(self.o, out, residual, n, ctx, rt)

    def forward(self, x: torch.Tensor, ctx, cache: CacheView) -> torch.Tensor:
        s, rt = self.spec, self.rt
        n = x.shape[0]
        qkv = self.qkv(x, rt.ws.take("attn_qkv", (n, self.q_width + 2 * self.kv_width), rt.act_dtype))
        out = self._rotate_write_attend(qkv, ctx, cache)
        return self.o(out, rt.ws.take("mixer_out", (n, s.hidden), rt.act_dtype))

    def _rotate_write_attend(self, qkv: torch.Tensor, ctx, cache: CacheView) -> torch.Tensor:
        s, rt = self.spec, self.rt
        n = qkv.shape[0]
        q = qkv[:, :self.q_width]
        k = qkv[:, self.q_width:self.q_width + self.kv_width]
        v = qkv[:, self.q_width + self.kv_width:]
        kvctx = ctx.kv[cache.group]
        tables = self.position.rotary_tables()
        # a position encoding may bias the scores by distance (float32 [n_heads, D]); only the general kernel takes it
        bias_of = getattr(self.position, "score_bias", None)
        bias = bias_of() if bias_of is not None else None
        out = rt.ws.take("attn_out", (n, self.q_width), rt.act_dtype)
        if (tables is not None and bias is None and ctx.max_q_len == 1 and ctx.n_tokens == ctx.n_requests
                and rt.act_dtype is torch.bfloat16 and s.head_dim in kernels.MMA_HEAD_DIMS
                and s.n_heads // s.n_kv_heads <= 16):
            # a decode step: rotation and cache write ride in the attention kernel
            n_splits, split_keys = decode_splits(ctx.keys_cap, ctx.n_requests * s.n_kv_heads,
                                                 *kernels.attention_decode_geometry(s.head_dim),
                                                 block_slots=2 * kernels.sm_count())
            scratch = self._decode_scratch(ctx, n_splits)
            kernels.attention_decode_fused(q, k, v, out, cache.k, cache.v, kvctx.block_table, ctx.q_start,
                                           ctx.ctx_before, scratch, tables[0], tables[1], ctx.positions,
                                           kvctx.slot_mapping, ctx.n_requests, s.n_heads, s.n_kv_heads, s.head_dim,
                                           ctx.page_size, s.window, self.scale, cache.write, n_splits, split_keys)
            return out
        if tables is None:
            self.position.rotate(q, k, ctx)
        cos, sin = tables if tables is not None else (None, None)
        # a step of prompt portions only, on the tcgen05 kernel: q is rotated where that kernel reads it
        q_in_kernel = tables is not None and bias is None and self._portions_only_on_tcgen05(ctx)
        kernels.rope_kv_write(q, k, v, cos, sin, ctx.positions, kvctx.slot_mapping,
                              cache.k if cache.write else None, cache.v if cache.write else None,
                              s.n_heads, s.n_kv_heads, s.head_dim, ctx.page_size, rotate_q=not q_in_kernel)
        self._attend(q, out, cache, ctx, kvctx, (cos, sin, ctx.positions) if q_in_kernel else (None, None, None), bias)
        return out

    def _portions_only_on_tcgen05(self, ctx) -> bool:
        s = self.spec
        group = s.n_heads // s.n_kv_heads
        if not (self.rt.act_dtype is torch.bfloat16 and s.head_dim in kernels.MMA_HEAD_DIMS):
            return False
        if ctx.max_q_len * group < TCGEN05_MIN_ROWS or ctx.max_q_len * group <= 16:
            return False
        if not kernels.attention_tcgen05_supports(s.head_dim, ctx.page_size, s.window):
            return False
        return ctx.keys_of_small_requests(group, 16)[0] == 0

    def _decode_scratch(self, ctx, n_splits: int) -> torch.Tensor:
        s = self.spec
        n = kernels.attention_decode_scratch_floats(ctx.n_tokens, s.n_heads, n_splits, s.head_dim)
        return self.rt.ws.take("attn_scratch", (n,), torch.float32)   # zero when made; tickets stay zero

    def _attend(self, q, out, cache, ctx, kvctx, rotate=(None, None, None), bias=None) -> None:
        s = self.spec
        group = s.n_heads // s.n_kv_heads
        if bias is None and self.rt.act_dtype is torch.bfloat16 and s.head_dim in kernels.MMA_HEAD_DIMS:
            # tensor-core kernels, built for this head size when first used
            n_small, small_keys = (ctx.n_requests, ctx.keys_cap) if ctx.max_q_len * group <= 16 \
                else ctx.keys_of_small_requests(group, 16)
            if ctx.n_requests * s.n_kv_heads > kernels.attention_decode_ticket_words(s.head_dim):
                n_small = 0        # more (request, kv head) pairs than the split-key kernel has tickets for
            if n_small:
                # requests with at most 16 rows (decode tokens, as a rule): the split-key kernel; in a mixed step
                # it leaves the others alone, and the prefill kernel below is given those only
                n_splits, split_keys = decode_splits(small_keys, n_small * s.n_kv_heads,
                                                      *kernels.attention_decode_geometry(s.head_dim),
                                                      block_slots=2 * kernels.sm_count())
                scratch = self._decode_scratch(ctx, n_splits)
                kernels.attention_decode_mma(q, out, cache.k, cache.v, kvctx.block_table, ctx.q_start,
                                             ctx.ctx_before, scratch, ctx.n_requests, ctx.n_tokens, s.n_heads,
                                             s.n_kv_heads, s.head_dim, ctx.page_size, s.window, self.scale,
                                             n_splits, split_keys)
            if n_small == ctx.n_requests:
                return
            more_than = 16 if n_small else 0
            if (ctx.max_q_len * group >= TCGEN05_MIN_ROWS
                    and kernels.attention_tcgen05_supports(s.head_dim, ctx.page_size, s.window)):
                # prompt portions: tcgen05 tensor cores, tiles of 128 rows by 128 keys
                work_req, work_pair0, n_work = ctx.attention_work(group, 128, more_than)
                kernels.attention_tcgen05(q, out, cache.k, cache.v, kvctx.block_table, ctx.q_start, ctx.ctx_before,
                                          work_req, work_pair0, n_work, s.n_heads, s.n_kv_heads, s.head_dim,
                                          ctx.page_size, self.scale, *rotate)
            else:
                rows = 64      # tiles of 128 rows (8 warps) leave one block per SM at this register count: slower
                work_req, work_pair0, n_work = ctx.attention_work(group, rows, more_than)
                kernels.attention_prefill_mma(q, out, cache.k, cache.v, kvctx.block_table, ctx.q_start,
                                              ctx.ctx_before, work_req, work_pair0, n_work, s.n_heads,
                                              s.n_kv_heads, s.head_dim, ctx.page_size, s.window, self.scale, rows)
            return
        work_req, work_pair0, n_work = ctx.attention_work(group, 32)
        kernels.attention_general(q, out, cache.k, cache.v, kvctx.block_table, ctx.q_start, ctx.ctx_before,
                                  work_req, work_pair0, n_work, s.n_heads, s.n_kv_heads, s.head_dim,
                                  ctx.page_size, s.window, self.scale, bias)


# fewer (token, head-in-group) rows than this in every request: the 64-row mma.sync tiles waste less
TCGEN05_MIN_ROWS = 128


def decode_splits(keys: int, n_streams: int, warps_per_block: int = 6, max_blocks: int = 64,
                  block_slots: int = 296) -> tuple[int, int]:
    """How the decode kernel cuts the keys: (number of splits, keys per split).

    One warp works on one split of one (request, kv head); a block's ``warps_per_block`` warps take
    consecutive splits and add up in shared memory, the blocks of a stream add up as a cluster (up to 8) or
    through memory.  Measured on B200: a step is fastest when its blocks fill the places the SMs have for
    them (``block_slots``: two a SM) once and no more (batch 8 at 2,048 keys: 3, 4, 5, 6 blocks a stream
    take 0.970, 0.946, 0.946, 1.043 ms a step; batch 64: 1, 2, 3 blocks 1.90, 2.16, 2.35 ms), and every warp
    of every block has keys: the blocks per stream follow from the number of streams, the split is the
    stream's keys over that many warps, in steps of 32 keys between 64 and 512.  Few streams get short
    splits and several blocks each (latency), many streams one block each (nothing leaves the block).
    ``keys`` is an upper bound of the keys any request of the step holds, the tighter the better.
    """
    keys = max(int(keys), 1)
    w = max(int(warps_per_block), 1)
    blocks = max(1, int(block_slots) // max(n_streams, 1))
    blocks = min(blocks, max(1, keys // (64 * w)), max_blocks)           # no split shorter than 64 keys
    blocks = max(blocks, -(-keys // (512 * w)))                           # nor longer than 512, if the launch allows
    blocks = min(blocks, max_blocks)
    split_keys = max(64, -(-keys // (blocks * w * 32)) * 32)
    return -(-keys // split_keys), split_keys
