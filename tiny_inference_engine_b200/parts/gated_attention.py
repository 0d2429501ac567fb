"""Sliding-window grouped-query attention with the options that `GQAttention` does not have:

    q, k, v, gate = h Wq^T + bq, h Wk^T + bk, h Wv^T + bv, h Wg^T      one product, the four weights stacked
    q, k   = (x / sqrt(mean over ALL heads of x^2 + eps)) * w            one norm over the whole projection
    q, k   = rotation of the first `rotary_dim` dimensions of each head (the position part's table)
    v      = (1 - lambda) v + lambda v_first                              `value_mix` "blend"; "source" keeps v as v_first
    k, v  -> cache pages (keys of `head_dim`, values of `value_dim`)
    out    = (softmax(scale q k^T over the last `window` keys) v * sigmoid(gate)) Wo^T + bo

Every size and constant is a parameter, and each option can be left out (`bias`, `span_norm`, `output_gate`,
`value_mix`, `window` 0 = all keys). The values that a "source" layer computes for the tokens of a step stay in a
workspace buffer that "blend" layers of the same step read: they belong to the same tokens, so nothing of it is
cached. The output product's bias is left to the block (`output_bias`), which adds it in float32.
"""
from __future__ import annotations

import math

import torch

from .. import ops
from ..errors import InvalidArgument
from ..weights.loader import TensorNeed
from .attention import MAX_SPLITS, NUM_SMS, SPLIT_KEYS, decode_splits
from .base import CacheNeed, Mixer, build_part, register_part, to_compute

_MIX_MODES = {None: 0, "none": 0, "source": 1, "blend": 2}


class GatedWindowAttention(Mixer):
    launches_only = False

    def __init__(self, spec, dtype, prefix: str = ""):
        p = spec.params
        self.prefix = prefix + p.get("prefix", "")
        self.hidden = int(p["hidden_size"])
        self.heads, self.kv_heads = int(p["num_heads"]), int(p["num_kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.value_dim = int(p.get("value_dim") or self.head_dim)
        self.window = int(p.get("window") or 0)
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.head_dim)
        self.eps = float(p.get("eps", 1e-6))
        self.bias = bool(p.get("bias", False))
        self.span_norm = bool(p.get("span_norm", False))
        self.output_gate = bool(p.get("output_gate", False))
        if p.get("value_mix") not in _MIX_MODES:
            raise InvalidArgument(f"value_mix must be one of none, source, blend; got {p.get('value_mix')!r}")
        self.mix_mode = _MIX_MODES[p.get("value_mix")]
        if self.heads <= 0 or self.kv_heads <= 0 or self.heads % self.kv_heads:
            raise InvalidArgument(f"{self.heads} heads are not a multiple of {self.kv_heads} kv heads")
        self.dtype = dtype
        self.position = build_part("position", p["position"], dtype, prefix=self.prefix)
        self.scale *= float(self.position.score_scale())
        # bfloat16 value heads smaller than the key heads are kept padded with zeros to the key heads' size (in the
        # cache, in the heads' outputs, in the gate's rows and in the output product's columns) where that size is
        # one the tensor-core attention kernels take: `out_dim` is the width a head's output has downstream.
        self.out_dim = self.value_dim
        if dtype == torch.bfloat16 and self.value_dim < self.head_dim and self.head_dim in (64, 128, 256) and \
                self.heads // self.kv_heads <= 16:
            self.out_dim = self.head_dim
        self.q_dim, self.k_dim = self.heads * self.head_dim, self.kv_heads * self.head_dim
        self.v_dim, self.o_dim = self.kv_heads * self.value_dim, self.heads * self.out_dim
        # columns of the stacked product, each section starting at a multiple of 8 (16 bytes of bfloat16)
        self.q_off = 0
        self.k_off = _up8(self.q_dim)
        self.v_off = self.k_off + _up8(self.k_dim)
        self.g_off = self.v_off + _up8(self.v_dim)
        self.width = self.g_off + (_up8(self.o_dim) if self.output_gate else 0)
        self.output_bias = None

    # -- weights
    def _name(self, leaf):
        return self.prefix + leaf

    def needs(self):
        D = self.hidden
        n = {self._name("q"): TensorNeed((self.q_dim, D)), self._name("k"): TensorNeed((self.k_dim, D)),
             self._name("v"): TensorNeed((self.v_dim, D)), self._name("o"): TensorNeed((D, self.heads * self.value_dim))}
        if self.bias:
            n.update({self._name("q.b"): TensorNeed((self.q_dim,), "norm"), self._name("k.b"): TensorNeed((self.k_dim,), "norm"),
                      self._name("v.b"): TensorNeed((self.v_dim,), "norm"), self._name("o.b"): TensorNeed((D,), "norm")})
        if self.span_norm:
            n.update({self._name("q.norm"): TensorNeed((self.q_dim,), "norm"),
                      self._name("k.norm"): TensorNeed((self.k_dim,), "norm")})
        if self.output_gate:
            n[self._name("g")] = TensorNeed((self.heads * self.value_dim, D))
        # only a blending layer reads the weight; a checkpoint may carry it for the others too (the source layer's
        # is never used), so there it is accepted and ignored
        n[self._name("vmix")] = TensorNeed((), "norm", optional=self.mix_mode != 2)
        n.update(self.position.needs())
        return n

    def bind(self, get):
        stacked = torch.zeros((self.width, self.hidden), dtype=self.dtype, device=get(self._name("q")).device)
        for leaf, off, n in (("q", self.q_off, self.q_dim), ("k", self.k_off, self.k_dim), ("v", self.v_off, self.v_dim)):
            stacked[off:off + n] = to_compute(get(self._name(leaf)), self.dtype)
        H, Dv, Do = self.heads, self.value_dim, self.out_dim
        if self.output_gate:      # head h's gate rows at h * out_dim (rows of the padding stay zero: they gate zeros)
            stacked[self.g_off:self.g_off + self.o_dim].view(H, Do, self.hidden)[:, :Dv] = \
                to_compute(get(self._name("g")), self.dtype).view(H, Dv, self.hidden)
        self.gemm_in = ops.bound_gemm(stacked, split_many=False)
        self.w_in = self.gemm_in.w
        w_o = to_compute(get(self._name("o")), self.dtype)
        if Do != Dv:              # columns of the padding are zero
            padded = torch.zeros((self.hidden, H, Do), dtype=self.dtype, device=w_o.device)
            padded[:, :, :Dv] = w_o.view(self.hidden, H, Dv)
            w_o = padded.view(self.hidden, H * Do)
        self.gemm_o = ops.bound_gemm(w_o.contiguous(), split_many=True)
        self.w_o = self.gemm_o.w
        f32 = lambda leaf: get(self._name(leaf)).to(torch.float32).contiguous()
        self.bq, self.bk, self.bv = (f32("q.b"), f32("k.b"), f32("v.b")) if self.bias else (None, None, None)
        self.output_bias = f32("o.b") if self.bias else None
        self.wq, self.wk = (f32("q.norm"), f32("k.norm")) if self.span_norm else (None, None)
        self.lam = f32("vmix").reshape(1) if self.mix_mode == 2 else None
        self.position.bind(get)
        self._capacity = None

    def cache_need(self):
        return CacheNeed("window" if self.window > 0 else "full", self.kv_heads, self.head_dim, self.window,
                         value_dim=0 if self.out_dim == self.head_dim else self.value_dim)

    # -- one step
    def forward(self, h, ctx, cache, state):
        T = h.shape[0]
        H, G, Dk, Dv = self.heads, self.kv_heads, self.head_dim, self.value_dim
        Do = self.out_dim               # a head's width in the value plane and downstream (Dv, or Dk with zeros behind Dv)
        g = ctx.groups[cache.group]
        if not cache.writes:
            raise InvalidArgument("this attention computes its own keys and values: it cannot read another entry's cache")
        proj = ctx.ws.rows("gattn.proj", T, self.width, self.dtype)
        self.gemm_in(h, proj)
        table = None if self.position.is_identity else self.position.fused_table()
        if table is None and not self.position.is_identity:
            raise InvalidArgument("this attention takes a rotation by a frequency table (or none) as its position encoding")
        v_first = ctx.ws.rows("gattn.v_first", T, self.v_dim, torch.float32) if self.mix_mode else None
        ops.qkv_span_prep(proj, self.q_off, self.k_off, self.v_off, self.bq, self.bk, self.bv, self.wq, self.wk, self.eps,
                          table, ctx.positions, g.slots, cache.k, cache.v, H, G, Dk, Dv, self.mix_mode, v_first, self.lam)
        attn = ctx.ws.rows("gattn.out", T, self.o_dim, self.dtype)
        q = proj[:, :self.q_dim]
        if Dk == Do and ops.attention_decode_tma_takes(q, H, G, Dk, cache.k.shape[2]):
            self._attend_tensor_cores(q, attn, ctx, g, cache)
        else:
            self._attend_cuda_cores(q, attn, ctx, g, cache)
        if self.output_gate:
            ops.sigmoid_gate_mul(attn, proj[:, self.g_off:self.g_off + self.o_dim])
        out = ctx.ws.rows("mixer.out", T, self.hidden, self.dtype)
        if self._capacity is None:
            self._capacity = ops.partial_capacity(ctx.ws.max_rows, self.gemm_o.N, self.gemm_o.K)
        return self.gemm_o(attn, out, lambda m: ctx.ws.flat("mixer.out.partial", m, torch.float32, self._capacity))


    def _attend_tensor_cores(self, q, attn, ctx, g, cache):
        """bfloat16 with keys and values of one size that the TMA-fed kernels take (64, 128, 256): the score and value
        products run on the tensor cores with float accumulation; the float softmax weights enter the value product
        as two bfloat16 terms (`exact_weights`), so that they keep 16 bits of mantissa."""
        H, G, Dh = self.heads, self.kv_heads, self.head_dim
        if ctx.multi_rows > 0:
            ops.attention_prompt_tma(q, cache.k, cache.v, attn, ctx.query_start, ctx.context_lens, g.block_tables, ctx.multi_seqs,
                                     ctx.multi_max_queries, H, G, Dh, self.scale, self.window, exact_weights=True)
        if ctx.single_count > 0:
            longest = ctx.single_max_context if self.window <= 0 else min(ctx.single_max_context, self.window)
            page = cache.k.shape[2]
            lens = ctx.single_contexts if self.window <= 0 else None
            key = ("decode_splits", longest, ctx.single_count, G, page, lens is None)
            splits = ctx.memo.get(key)
            if splits is None:
                splits = ctx.memo[key] = decode_splits(longest, ctx.single_count, G, page, lens)
            split_keys, max_splits = splits
            scratch = ctx.ws.flat("attn.split", ops.attention_split_scratch_floats(ctx.max_seqs, H, Dh, MAX_SPLITS), torch.float32)
            counters = ctx.ws.zeros("attn.counters", ctx.max_seqs * G, torch.int32)
            cluster = max_splits in ops.CLUSTER_SPLITS and ctx.single_count * G * max_splits <= 2 * NUM_SMS
            ops.attention_decode_tma(q, cache.k, cache.v, attn, ctx.query_start, ctx.context_lens, g.block_tables, H, G, Dh,
                                     self.scale, ctx.multi_seqs, ctx.single_count, split_keys, max_splits, scratch, counters,
                                     self.window, cluster=cluster, exact_weights=True)

    def _attend_cuda_cores(self, q, attn, ctx, g, cache):
        """float32, or heads of other sizes (keys and values may differ): one warp per (row, head), everything float."""
        H, G, Dk, Dv = self.heads, self.kv_heads, self.head_dim, self.out_dim
        n = ctx.multi_rows
        if n > 0:
            ops.attention_rows_dv(q[:n], cache.k, cache.v, attn[:n], ctx.seq_of_row[:n], ctx.query_start, ctx.context_lens,
                                  g.block_tables, H, G, Dk, Dv, self.scale, self.window)
        if ctx.single_count > 0:
            longest = ctx.single_max_context if self.window <= 0 else min(ctx.single_max_context, self.window)
            split_keys = SPLIT_KEYS
            while math.ceil(longest / split_keys) > MAX_SPLITS:
                split_keys *= 2
            max_splits = max(1, math.ceil(longest / split_keys))
            scratch = ctx.ws.flat("gattn.split", ops.attention_split_scratch_floats(ctx.max_seqs, H, Dv, MAX_SPLITS), torch.float32)
            ops.attention_split_dv(q, cache.k, cache.v, attn, ctx.query_start, ctx.context_lens, g.block_tables, H, G, Dk, Dv,
                                   self.scale, ctx.single_seqs, ctx.single_count, split_keys, max_splits, scratch, self.window)


def _up8(n: int) -> int:
    return (n + 7) // 8 * 8


register_part("mixer", "gated_window_attention", GatedWindowAttention, replace=True)
