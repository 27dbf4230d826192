"""Grouped-query attention over the paged cache: projections (with optional
biases, added before the per-head norms), optional per-head q/k norm, optional
position encoding, append of k and v to the entry's pages, causal attention
over all earlier keys or a window of them, output projection added to the
residual stream (crates/nncpu/src/model/forward.rs:197-439).

q, k and v projections are stored as one matrix so the input is read once.
An entry that reads another entry's cache has no k/v projection at all
(crates/nncpu/src/model/forward.rs:210,240-255).
"""
from __future__ import annotations

import torch

from .. import perf
from ..cache import KVRequest
from ..errors import UnsupportedModel
from ..kernels import ops
from ..weights.params import ParamSpec
from . import base
from .base import Mixer, register_mixer


@register_mixer("attention")
class Attention(Mixer):
    accepts_deferred_norm = True    # x goes to Runtime.linear, which finishes a norm's unfinished output

    def __init__(self, spec, reads_other_cache: bool = False):
        s = self.spec = spec
        self.shared_kv = reads_other_cache
        if s.n_heads % s.n_kv_heads:
            raise UnsupportedModel(f"{s.name}: {s.n_heads} heads over {s.n_kv_heads} key/value heads")
        if s.qk_norm is not None and s.qk_norm.kind != "rmsnorm":
            raise UnsupportedModel(f"{s.name}: per-head norm of kind {s.qk_norm.kind!r} is not supported")
        self.q_size = s.n_heads * s.head_dim
        self.kv_size = 0 if reads_other_cache else s.n_kv_heads * s.head_dim
        self.position = None if s.position is None else base.build("position", s.position)

    def kv_request(self):
        s = self.spec
        return None if self.shared_kv else KVRequest(s.n_kv_heads, s.head_dim, s.window)

    def _proj_names(self):
        return ["q_proj"] if self.shared_kv else ["q_proj", "k_proj", "v_proj"]

    def params(self):
        s, p = self.spec, []
        sizes = {"q_proj": self.q_size, "k_proj": self.kv_size, "v_proj": self.kv_size}
        for n in self._proj_names():
            p.append(ParamSpec(f"{s.name}.{n}.weight", (sizes[n], s.hidden_size)))
            if s.qkv_bias:
                p.append(ParamSpec(f"{s.name}.{n}.bias", (sizes[n],)))
        p.append(ParamSpec(f"{s.name}.o_proj.weight", (s.hidden_size, self.q_size)))
        if s.out_bias_optional:
            p.append(ParamSpec(f"{s.name}.o_proj.bias", (s.hidden_size,), required=False))
        if s.qk_norm is not None:
            p.append(ParamSpec(f"{s.qk_norm.name}.q_norm.weight", (s.head_dim,), init=("one_plus_normal", 0.1)))
            if not self.shared_kv:
                p.append(ParamSpec(f"{s.qk_norm.name}.k_norm.weight", (s.head_dim,), init=("one_plus_normal", 0.1)))
        return p

    def bind(self, tensors, rt):
        s, self.rt = self.spec, rt
        names = self._proj_names()
        ws = [tensors.pop(f"{s.name}.{n}.weight") for n in names]
        self.w_qkv = ws[0] if len(ws) == 1 else torch.cat(ws, dim=0).contiguous()
        del ws
        self.b_qkv = None
        if s.qkv_bias:
            bs = [tensors.pop(f"{s.name}.{n}.bias") for n in names]
            self.b_qkv = bs[0] if len(bs) == 1 else torch.cat(bs, dim=0).contiguous()
        self.w_o = tensors[f"{s.name}.o_proj.weight"]
        self.b_o = tensors.get(f"{s.name}.o_proj.bias")
        self.q_gamma = self.k_gamma = None
        if s.qk_norm is not None:
            self.q_gamma = tensors[f"{s.qk_norm.name}.q_norm.weight"]
            self.k_gamma = tensors.get(f"{s.qk_norm.name}.k_norm.weight")
        if self.position is not None:
            self.position.bind(tensors, rt)

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_qkv, self.w_o))

    def forward(self, ctx, x, residual, cache):
        s, rt = self.spec, self.rt
        n = x.shape[0]
        eps = s.qk_norm.eps if s.qk_norm else 0.0
        attn = rt.empty(n, self.q_size)
        if self._fused_qkv(x, cache):
            # a prompt: norm, rotation and the cache append happen in the projection's epilogue, on its
            # float32 accumulators; its threads are tokens, so the rotation table is laid out by pair
            q = rt.empty(n, self.q_size)
            with rt.phase("attn_rope"):
                cos_sin = None if self.position is None else self.position.tables(ctx, by_pair=True)
            norm_in = None
            if isinstance(x, base.DeferredNorm):      # the norm before rides on this product
                x, norm_in = x.x_gamma, (x.bins, x.request.eps)
            with rt.phase("attn_qkv", self.w_qkv, n):
                ops.linear_tc_qkv(x, self.w_qkv, self.q_gamma, self.k_gamma, eps, cos_sin, ctx.tok_seq, ctx.tok_pos,
                                  cache.block_table, cache.k_pages, cache.v_pages, q, rt.workspace, s.n_heads,
                                  s.n_kv_heads, s.head_dim, norm_in=norm_in)
            with self._core_phase(ctx, cache):
                self._attend(ctx, q, cache, attn)
        else:
            # the projections stay in float32 until the per-head norm and the rotation have been applied
            qkv = rt.empty(n, self.q_size + 2 * self.kv_size, dtype=torch.float32)
            with rt.phase("attn_qkv", self.w_qkv, n):
                rt.linear(x, self.w_qkv, self.b_qkv, qkv)
            with rt.phase("attn_rope"):
                cos_sin = None if self.position is None else self.position.tables(ctx)
            if self._decode_from_projections(ctx, cache):
                # a decode step: norm, rotation and append are the attention kernel's own first steps
                with self._core_phase(ctx, cache):
                    n_splits, scratch = self._decode_splits(ctx)
                    ops.attention_decode_mma_from_qkv(qkv, self.q_gamma, self.k_gamma, eps, cos_sin, cache.k_pages,
                                                      cache.v_pages, not self.shared_kv, cache.block_table, ctx.tok_seq,
                                                      ctx.tok_pos, attn, scratch, s.n_heads, s.n_kv_heads, s.head_dim,
                                                      s.scale, s.window, n_splits)
            else:
                q = rt.empty(n, self.q_size)
                with rt.phase("attn_rope"):
                    ops.qk_norm_rope_append(qkv, self.q_gamma, self.k_gamma, eps, cos_sin, ctx.tok_seq, ctx.tok_pos,
                                            cache.block_table, cache.k_pages, cache.v_pages, q, s.n_heads,
                                            0 if self.shared_kv else s.n_kv_heads, s.head_dim)
                with self._core_phase(ctx, cache):
                    self._attend(ctx, q, cache, attn)
        with rt.phase("attn_out", self.w_o, n):
            # the last write into the residual stream: it may leave the next norm its input
            rt.linear(attn, self.w_o, self.b_o, residual, accumulate=True, then_norm=getattr(ctx, "next_norm", None))

    def _core_phase(self, ctx, cache):
        """The profiler's scope of the attention itself: every token streams the keys and values of its span
        (crates/nncpu/src/model/forward.rs:382-386)."""
        if not perf.enabled():
            return perf._NULL
        s = self.spec
        keys = ctx.span_sum(s.window)
        return self.rt.phase("attn_core", nbytes=2.0 * keys * s.n_kv_heads * s.head_dim * cache.k_pages.element_size(),
                             flops=4.0 * keys * self.q_size)

    def _decode_from_projections(self, ctx, cache) -> bool:
        """Whether this step's attention can start from the float32 projections: a decode step on the tensor-core
        kernel, every lane of a head rotated (or none), norm weights of one type."""
        s = self.spec
        return (ctx.is_decode and self.rt.dtype == torch.bfloat16 and cache.k_pages.dtype == torch.bfloat16
                and ops.attention_mma_supported(s.n_heads, s.n_kv_heads, s.head_dim)
                and (self.position is None or self.position.half * 2 == s.head_dim)
                and (self.q_gamma is None or self.k_gamma is None or self.q_gamma.dtype == self.k_gamma.dtype))

    def _decode_splits(self, ctx):
        """Splits of every token's keys in a decode step, and the scratch their merge needs (None: they merge
        inside a thread-block cluster)."""
        s = self.spec
        longest = min(ctx.max_kv_len, s.window) if s.window > 0 else ctx.max_kv_len
        n_splits = ops.attention_decode_splits(ctx.n_tokens, s.n_kv_heads, longest, self.rt.sm_count)
        floats = 0 if n_splits <= ops.DECODE_CLUSTER_MAX_SPLITS else ops.attention_decode_scratch_floats(
            ctx.n_tokens, s.n_heads, s.n_kv_heads, s.head_dim, n_splits)
        return n_splits, (self.rt.empty(floats, dtype=torch.float32) if floats else None)

    def _fused_qkv(self, x, cache) -> bool:
        s = self.spec
        if isinstance(x, base.DeferredNorm):
            x = x.x_gamma
        return (not self.shared_kv and self.b_qkv is None and x.dtype == torch.bfloat16
                and self.w_qkv.dtype == torch.bfloat16 and cache.k_pages.dtype == torch.bfloat16
                and (self.position is None or (self.position.tables_by_pair and self.position.half * 2 == s.head_dim))
                and ops.linear_tc_qkv_supported(x, s.n_heads, s.n_kv_heads, s.head_dim))

    def _attend(self, ctx, q, cache, attn):
        """bfloat16 with a head size the tensor-core kernels take: split-key
        decode, tcgen05 prefill for prompts, mma.sync prefill for a few tokens
        per sequence; everything else: the 32-bit kernel."""
        s = self.spec
        if not ops.attention_mma_supported(s.n_heads, s.n_kv_heads, s.head_dim, q, cache.k_pages, attn):
            ops.attention(q, cache.k_pages, cache.v_pages, cache.block_table, ctx.tok_seq, ctx.tok_pos, attn,
                          s.n_heads, s.n_kv_heads, s.head_dim, s.scale, s.window)
        elif ctx.is_decode:
            n_splits, scratch = self._decode_splits(ctx)
            ops.attention_decode_mma(q, cache.k_pages, cache.v_pages, cache.block_table, ctx.tok_seq, ctx.tok_pos,
                                     attn, scratch, s.n_heads, s.n_kv_heads, s.head_dim, s.scale, s.window, n_splits)
        elif ctx.n_tokens >= 32 * ctx.n_seqs and ops.attention_prefill_tc_supported(
                s.n_heads, s.n_kv_heads, s.head_dim, q, cache.k_pages, attn):
            # prompts: 128-row tiles on the tcgen05 tensor cores
            ops.attention_prefill_tc(q, cache.k_pages, cache.v_pages, cache.block_table, ctx.cu_seqlens, ctx.tok_pos,
                                     attn, self.rt.workspace.status, ctx.n_seqs, s.n_heads, s.n_kv_heads, s.head_dim,
                                     s.scale, s.window)
        else:
            # a few new tokens per sequence: 64-row tiles
            ops.attention_prefill_mma(q, cache.k_pages, cache.v_pages, cache.block_table, ctx.cu_seqlens, ctx.tok_pos,
                                      attn, ctx.n_seqs, s.n_heads, s.n_kv_heads, s.head_dim, s.scale, s.window)
