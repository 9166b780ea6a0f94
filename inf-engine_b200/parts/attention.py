"""Grouped-query causal attention over the paged cache
(engine/llama_attention.py:83-141).

q, k and v come from one matrix product over the row-concatenated weights;
a fused kernel rotates q and k and writes k and v into the pages of the step's
tokens; the attention kernel then reads every key and value through the block
table, so a prompt portion, a decode token and a whole prompt take the same
path.  kv head c serves query heads c*g .. c*g+g-1 (:27-44) inside the kernel;
nothing is expanded in memory.  Scores are scaled by head_dim**-0.5 (the
library default the reference relies on, :123-137) unless the spec names a scale.

Options of the spec beyond that: an RMS norm of every query and key head before
the scores (``qk_norm``, fused with the cache write), a learned multiplier of
each head's scores (``head_scale``), a bias by distance from the position
encoding, and values of another head size than queries and keys
(``v_head_dim``).  A layer that uses one of them runs the general kernel, which
computes scores and weights in float32; the tensor-core kernels take none.

Further options: biases of the three projections, an RMS norm over the WHOLE q
row and k row (all heads at once) with gains of the row's size, a rotation of
neighbouring pairs of each head's first dimensions with angles worked out from
the position (``rotary_pairs``), keys at the start of the sequence that stay
visible beside a window (``keep_first``), and a multiplier of the output
(``out_scale``, for a mixer that is one of several summed side by side).  One
kernel adds the biases, norms, rotates and writes the cache
(``rownorm_rotate_write``); the general attention kernel takes the rest.
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
    parts: list | None = None               # kind "several": one view per part of the run's requirement


@register_mixer("attention")
class PagedAttention:
    graph_safe = True

    @staticmethod
    def expected_tensors(spec):
        out = {
            spec.q_proj: ExpectedTensor((spec.n_heads * spec.head_dim, spec.hidden)),
            spec.k_proj: ExpectedTensor((spec.n_kv_heads * spec.head_dim, spec.hidden)),
            spec.v_proj: ExpectedTensor((spec.n_kv_heads * spec.value_dim, spec.hidden)),
        }
        for name, width in ((spec.q_bias, spec.n_heads * spec.head_dim), (spec.k_bias, spec.n_kv_heads * spec.head_dim),
                            (spec.v_bias, spec.n_kv_heads * spec.value_dim)):
            if name is not None:
                out[name] = ExpectedTensor((width,))
        if spec.qk_norm is not None:
            for name in (spec.qk_norm.q_weight, spec.qk_norm.k_weight):
                if name is not None:
                    out[name] = ExpectedTensor((spec.head_dim,), init="gain")
        if spec.q_row_norm is not None:
            out[spec.q_row_norm] = ExpectedTensor((spec.n_heads * spec.head_dim,), init="gain")
        if spec.k_row_norm is not None:
            out[spec.k_row_norm] = ExpectedTensor((spec.n_kv_heads * spec.head_dim,), init="gain")
        out.update(position_class(spec.position).expected_tensors(spec.position))
        if spec.head_scale is not None:
            out[spec.head_scale] = ExpectedTensor((spec.n_heads,), init="gain")
        out[spec.o_proj] = ExpectedTensor((spec.hidden, spec.n_heads * spec.value_dim))
        return out

    def __init__(self, spec, tensors, rt):
        if spec.n_heads % spec.n_kv_heads:
            raise ValueError(f"{spec.n_heads} query heads are not a multiple of {spec.n_kv_heads} kv heads")
        if not (0 < spec.head_dim <= 256 and 0 < spec.value_dim <= 256):
            raise ValueError(f"attention kernels take head sizes up to 256, not {spec.head_dim} and {spec.value_dim}")
        if spec.window is not None and spec.window <= 0:
            raise ValueError("an attention window must be positive")
        self.spec = spec
        self.rt = rt
        ws = [tensors[spec.q_proj], tensors[spec.k_proj], tensors[spec.v_proj]]
        dtype = torch.float32 if any(w.dtype is torch.float32 for w in ws) else ws[0].dtype
        self.qkv = Linear(torch.cat([w.to(dtype) for w in ws], dim=0).contiguous(), rt, "qkv")
        self.o_weight = tensors[spec.o_proj]
        self.o = Linear(self.o_weight, rt, "o")
        self.position = build_position(spec.position, tensors, rt)
        self.scale = float(spec.scale) if spec.scale is not None else float(spec.head_dim) ** -0.5
        self.v_dim = spec.value_dim
        self.q_width = spec.n_heads * spec.head_dim
        self.k_width = spec.n_kv_heads * spec.head_dim
        self.v_width = spec.n_kv_heads * self.v_dim
        self.out_width = spec.n_heads * self.v_dim
        self.kv_width = self.k_width            # where keys and values have one size
        qn = spec.qk_norm
        self.q_gain = tensors[qn.q_weight] if qn is not None and qn.q_weight is not None else None
        self.k_gain = tensors[qn.k_weight] if qn is not None and qn.k_weight is not None else None
        if self.q_gain is not None and self.k_gain is not None and self.q_gain.dtype != self.k_gain.dtype:
            self.q_gain, self.k_gain = self.q_gain.float(), self.k_gain.float()
        self.head_scale = tensors[spec.head_scale].float().contiguous() if spec.head_scale is not None else None
        # biases, whole-row norms and the pair rotation ride in one kernel before the attention
        self.pair_rotation = getattr(self.position, "pair_rotation", None)        # (inv_freq, rot_dims) or None
        rowwise = [tensors[n] for n in (spec.q_bias, spec.k_bias, spec.v_bias, spec.q_row_norm, spec.k_row_norm) if n is not None]
        self.row_mode = bool(rowwise) or self.pair_rotation is not None
        if self.row_mode:
            if qn is not None:
                raise NotImplementedError("norms per head together with whole-row norms or biases are not built")
            rdtype = torch.float32 if any(t.dtype is torch.float32 for t in rowwise) else (rowwise[0].dtype if rowwise else torch.float32)
            pick = lambda n: tensors[n].to(rdtype).contiguous() if n is not None else None
            self.q_bias, self.k_bias, self.v_bias = pick(spec.q_bias), pick(spec.k_bias), pick(spec.v_bias)
            self.q_row_gain, self.k_row_gain = pick(spec.q_row_norm), pick(spec.k_row_norm)
        self.keep_first = int(spec.keep_first) if spec.window is not None else 0
        self.out_scale = float(spec.out_scale)
        self.core_width = self.out_width
        # the tensor-core kernels and the fused decode kernel know none of these; such a layer runs the general kernel
        self.plain = (qn is None and self.head_scale is None and self.v_dim == spec.head_dim and not self.row_mode
                      and not self.keep_first and self.out_scale == 1.0)

    def cache_requirement(self) -> CacheRequirement:
        s = self.spec
        return CacheRequirement(kind="kv", n_kv_heads=s.n_kv_heads, head_dim=s.head_dim, window=s.window,
                                dtype=self.rt.act_dtype, v_head_dim=None if self.v_dim == s.head_dim else self.v_dim,
                                keep_first=self.keep_first)

    def can_fuse(self, n_tokens: int, norm) -> bool:
        return hasattr(norm, "fusable_rms") and self.qkv.streams(n_tokens, normed=True) and self.o.streams(n_tokens)

    def forward_fused(self, residual: torch.Tensor, norm, ctx, cache: CacheView) -> None:
        """residual += o(attention(qkv(norm(residual)))): the norm rides in the qkv product's prologue and the
        residual sum in the output product's epilogue."""
        rt = self.rt
        n = residual.shape[0]
        qkv = rt.ws.take("attn_qkv", (n, self.q_width + self.k_width + self.v_width), rt.act_dtype)
        stream_normed(self.qkv, residual, qkv, n, "bf16", norm, ctx)
        out = self._rotate_write_attend(qkv, ctx, cache)
        stream_into_residual(self.o, out, residual, n, ctx, rt)

    def forward(self, x: torch.Tensor, ctx, cache: CacheView) -> torch.Tensor:
        s, rt = self.spec, self.rt
        n = x.shape[0]
        qkv = self.qkv(x, rt.ws.take("attn_qkv", (n, self.q_width + self.k_width + self.v_width), rt.act_dtype))
        out = self._rotate_write_attend(qkv, ctx, cache)
        return self.o(out, rt.ws.take("mixer_out", (n, s.hidden), rt.act_dtype))

    def forward_core(self, x: torch.Tensor, ctx, cache: CacheView, out: torch.Tensor) -> None:
        """``out`` ([n, heads * value size], may be a column slice) = the heads' outputs times ``out_scale``: what goes
        into the output projection (a mixer that runs several side by side multiplies them all at once)."""
        rt = self.rt
        n = x.shape[0]
        qkv = self.qkv(x, rt.ws.take("attn_qkv", (n, self.q_width + self.k_width + self.v_width), rt.act_dtype))
        self._rotate_write_attend(qkv, ctx, cache, out)

    def _rotate_write_attend(self, qkv: torch.Tensor, ctx, cache: CacheView, out: torch.Tensor | None = None) -> torch.Tensor:
        s, rt = self.spec, self.rt
        n = qkv.shape[0]
        q = qkv[:, :self.q_width]
        k = qkv[:, self.q_width:self.q_width + self.k_width]
        v = qkv[:, self.q_width + self.k_width:]
        kvctx = ctx.kv[cache.group]
        tables = self.position.rotary_tables()
        # a position encoding may bias the scores by distance (float32 [n_heads, D]); only the general kernel takes it
        bias_of = getattr(self.position, "score_bias", None)
        bias = bias_of() if bias_of is not None else None
        if out is None:
            out = rt.ws.take("attn_out", (n, self.out_width), rt.act_dtype)
        if self.row_mode:
            if tables is not None:
                raise NotImplementedError("a table rotation together with whole-row norms or biases is not built")
            inv_freq, rot_dims = self.pair_rotation if self.pair_rotation is not None else (None, 0)
            kpool, vpool = (cache.k, cache.v) if cache.write else (None, None)
            kernels.rownorm_rotate_write(q, k, v, self.q_bias, self.k_bias, self.v_bias, self.q_row_gain, self.k_row_gain,
                                         s.row_norm_eps, inv_freq, rot_dims, ctx.positions, kvctx.slot_mapping, kpool,
                                         vpool, s.n_heads, s.n_kv_heads, s.head_dim, self.v_dim, ctx.page_size)
            self._attend(q, out, cache, ctx, kvctx, bias=bias, head_scale=self.head_scale)
            return out
        if not self.plain:
            return self._attend_general(q, k, v, out, ctx, cache, kvctx, tables, bias)
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

    def _attend_general(self, q, k, v, out, ctx, cache, kvctx, tables, bias) -> torch.Tensor:
        """A layer with head norms, a multiplier per head or values of their own size: one kernel norms q and k and
        writes keys and values into their pages (fused as the rotation and the write are for a plain layer), then
        the general attention kernel, whose scores and weights are float32, reads everything through the block
        table.  With a rotation as well, the norm comes first and the rotating kernel writes the cache."""
        s = self.spec
        eps = s.qk_norm.eps if s.qk_norm is not None else 0.0
        kpool, vpool = (cache.k, cache.v) if cache.write else (None, None)
        if tables is None:
            self.position.rotate(q, k, ctx)
            kernels.headnorm_kv_write(q, k, v, self.q_gain, self.k_gain, eps, kvctx.slot_mapping, kpool, vpool,
                                      s.n_heads, s.n_kv_heads, s.head_dim, self.v_dim, ctx.page_size)
        else:
            if self.v_dim != s.head_dim:
                raise NotImplementedError("a rotation with values of another head size than the keys is not built")
            kernels.headnorm_kv_write(q, k, v, self.q_gain, self.k_gain, eps, None, None, None, s.n_heads,
                                      s.n_kv_heads, s.head_dim, self.v_dim, ctx.page_size)
            kernels.rope_kv_write(q, k, v, tables[0], tables[1], ctx.positions, kvctx.slot_mapping, kpool, vpool,
                                  s.n_heads, s.n_kv_heads, s.head_dim, ctx.page_size)
        self._attend(q, out, cache, ctx, kvctx, bias=bias, head_scale=self.head_scale)
        return out

    def _bias_log2e(self, bias):
        """The bias table in the exponent's units (times log2 e), as the tensor-core kernels' bias build takes it."""
        if bias is None:
            return None
        got = getattr(self, "_bias_scaled", None)
        if got is None or got[0] is not bias:
            got = (bias, (bias * kernels.LOG2E).contiguous())
            self._bias_scaled = got
        return got[1]

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
        n = kernels.attention_decode_scratch_floats(ctx.n_tokens, s.n_heads, n_splits, s.head_dim, not self.plain)
        return self.rt.ws.take("attn_scratch", (n,), torch.float32)   # zero when made; tickets stay zero

    def _attend(self, q, out, cache, ctx, kvctx, rotate=(None, None, None), bias=None, head_scale=None) -> None:
        s = self.spec
        group = s.n_heads // s.n_kv_heads
        extras = bias is not None or head_scale is not None
        # a bias by distance or a multiplier per head: the bias build of the mma.sync kernels (scores, maxima and
        # sums in float32, weights to two bfloat16 terms); the tcgen05 kernel has no such input
        if (self.rt.act_dtype is torch.bfloat16 and s.head_dim in kernels.MMA_HEAD_DIMS and self.v_dim == s.head_dim
                and (not extras or group <= 16) and not self.keep_first and self.out_scale == 1.0 and not self.row_mode):
            extra = dict(score_bias_log2e=self._bias_log2e(bias), head_scale=head_scale) if extras else {}
            # tensor-core kernels, built for this head size when first used
            n_small, small_keys = (ctx.n_requests, ctx.keys_cap) if ctx.max_q_len * group <= 16 \
                else ctx.keys_of_small_requests(group, 16)
            if ctx.n_requests * s.n_kv_heads > kernels.attention_decode_ticket_words(s.head_dim, extras):
                n_small = 0        # more (request, kv head) pairs than the split-key kernel has tickets for
            if n_small:
                # requests with at most 16 rows (decode tokens, as a rule): the split-key kernel; in a mixed step
                # it leaves the others alone, and the prefill kernel below is given those only
                n_splits, split_keys = decode_splits(small_keys, n_small * s.n_kv_heads,
                                                      *kernels.attention_decode_geometry(s.head_dim, extras),
                                                      block_slots=2 * kernels.sm_count())
                scratch = self._decode_scratch(ctx, n_splits)
                kernels.attention_decode_mma(q, out, cache.k, cache.v, kvctx.block_table, ctx.q_start,
                                             ctx.ctx_before, scratch, ctx.n_requests, ctx.n_tokens, s.n_heads,
                                             s.n_kv_heads, s.head_dim, ctx.page_size, s.window, self.scale,
                                             n_splits, split_keys, **extra)
            if n_small == ctx.n_requests:
                return
            more_than = 16 if n_small else 0
            if (not extras and ctx.max_q_len * group >= TCGEN05_MIN_ROWS
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
                                              s.n_kv_heads, s.head_dim, ctx.page_size, s.window, self.scale, rows,
                                              **extra)
            return
        # float32 arithmetic on CUDA cores: requests that bring at most 16 rows (decode tokens) get a block per (token,
        # head) whose warps split the keys; the others the tile kernel, with a work list of those requests only
        # (layers without the newer options keep the tile kernel for every request: all their cuts then walk the same
        # key tiles and agree with each other to the last bits)
        newer = self.row_mode or self.keep_first or self.out_scale != 1.0
        n_small = 0 if not newer else (ctx.n_requests if ctx.max_q_len * group <= 16 else ctx.keys_of_small_requests(group, 16)[0])
        if n_small:
            kernels.attention_rows(q, out, cache.k, cache.v, kvctx.block_table, ctx.q_start, ctx.ctx_before,
                                   ctx.n_requests, 16, s.n_heads, s.n_kv_heads, s.head_dim, ctx.page_size, s.window,
                                   self.scale, bias, head_scale, self.v_dim, self.keep_first, self.out_scale)
            if n_small == ctx.n_requests:
                return
        if (newer and self.rt.act_dtype is torch.bfloat16 and s.head_dim in kernels.MMA_HEAD_DIMS and self.v_dim == s.head_dim
                and group <= 16):
            # prompt portions of a layer with kept first keys, a multiplier of its output or scores that must be
            # float32: the tensor-core kernels' bias build (float32 scores, maxima and sums; weights to two bfloat16 terms)
            work_req, work_pair0, n_work = ctx.attention_work(group, 64, 16 if n_small else 0)
            kernels.attention_prefill_mma(q, out, cache.k, cache.v, kvctx.block_table, ctx.q_start, ctx.ctx_before,
                                          work_req, work_pair0, n_work, s.n_heads, s.n_kv_heads, s.head_dim,
                                          ctx.page_size, s.window, self.scale, 64,
                                          score_bias_log2e=self._bias_log2e(bias), head_scale=head_scale,
                                          keep_first=self.keep_first, out_scale=self.out_scale, float32_scores=True)
            return
        work_req, work_pair0, n_work = ctx.attention_work(group, 32, 16 if n_small else 0)
        kernels.attention_general(q, out, cache.k, cache.v, kvctx.block_table, ctx.q_start, ctx.ctx_before,
                                  work_req, work_pair0, n_work, s.n_heads, s.n_kv_heads, s.head_dim,
                                  ctx.page_size, s.window, self.scale, bias, head_scale, self.v_dim, self.keep_first,
                                  self.out_scale)


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
