"""Attention whose keys and values come from one latent vector per token.

    c_q   = rmsnorm(h Wdq^T) * w_dq                              the query latent
    q     = c_q Wuq^T                                            per head [head_dim unrotated | rot_dim rotated]
    c, r  = rmsnorm((h Wdkv^T)[:rank]) * w_dkv, rotation((h Wdkv^T)[rank:])     the latent, and one rotated key part for all heads
    k_h   = [Wuk_h c | r],   v_h = Wuv_h c                       per head
    out   = ((softmax(scale q k^T over the last `window` keys) v)_h * sigmoid(h Wg^T)_h) Wo^T      one gate per head

The cache keeps [c | r] per token and nothing per head: with q'_h = [Wuk_h^T q_h,plain | rotation(q_h,rot)] the score is
q'_h . [c | r], and the weighted sum of values is Wuv_h applied to the weighted sum of latents. So every head attends
over the same rows (one kv head of `rank + rot_dim`, whose value is its first `rank` elements: `CacheNeed.value_dim`
-1), and the two per-head maps are products batched over heads on either side. Every size and constant is a
parameter; `window` 0 keeps all keys; `output_gate` False leaves the gate out.
"""
from __future__ import annotations

import math

import torch

from .. import ops
from ..errors import InvalidArgument
from ..weights.loader import TensorNeed
from .attention import MAX_SPLITS, SPLIT_KEYS
from .base import CacheNeed, Mixer, build_part, register_part, to_compute


LATENT_SPLIT_KEYS = 128     # keys per split of a sequence that brings one token (two key tiles of the tensor-core kernel; shorter
                            # splits cost the merge more than they save the split kernel)


def _up8(n: int) -> int:
    return (n + 7) // 8 * 8


class LatentAttention(Mixer):
    launches_only = False

    def __init__(self, spec, dtype, prefix: str = ""):
        p = spec.params
        self.prefix = prefix + p.get("prefix", "")
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["num_heads"])
        self.dim, self.rot, self.vdim = int(p["head_dim"]), int(p["rot_dim"]), int(p["value_dim"])
        self.rank, self.q_rank = int(p["kv_rank"]), int(p["q_rank"])
        self.window = int(p.get("window") or 0)
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.dim + self.rot)
        self.eps = float(p.get("eps", 1e-6))
        self.output_gate = bool(p.get("output_gate", True))
        if min(self.heads, self.dim, self.vdim, self.rank, self.q_rank) <= 0 or self.rot < 0 or self.rot % 2:
            raise InvalidArgument(f"latent attention: bad sizes heads={self.heads} dim={self.dim} rot={self.rot} vdim={self.vdim} "
                                  f"ranks={self.rank}, {self.q_rank}")
        if self.rank > 512 or self.rank + self.rot > 1024:
            raise InvalidArgument(f"latent attention: a latent of {self.rank} (at most 512) with a rotated part of {self.rot} (together at "
                                  f"most 1024) is more than the kernels take")
        self.dtype = dtype
        self.position = build_part("position", p["position"], dtype, prefix=self.prefix) if self.rot else None
        if self.position is not None:
            self.scale *= float(self.position.score_scale())
        self.key_dim = self.rank + self.rot
        # columns of the stacked product over h: the query latent, the key/value latent with the rotated part, the gates
        self.q_off = 0
        self.kv_off = _up8(self.q_rank)
        self.g_off = self.kv_off + _up8(self.key_dim)
        self.width = self.g_off + (_up8(self.heads) if self.output_gate else 0)
        self.output_bias = None

    def _name(self, leaf):
        return self.prefix + leaf

    def needs(self):
        D, H, n = self.hidden, self.heads, self._name
        out = {n("dq"): TensorNeed((self.q_rank, D)), n("dq.norm"): TensorNeed((self.q_rank,), "norm"),
               n("uq"): TensorNeed((H * (self.dim + self.rot), self.q_rank)),
               n("dkv"): TensorNeed((self.key_dim, D)), n("dkv.norm"): TensorNeed((self.rank,), "norm"),
               n("uk"): TensorNeed((H * self.dim, self.rank)), n("uv"): TensorNeed((H * self.vdim, self.rank)),
               n("o"): TensorNeed((D, H * self.vdim))}
        if self.output_gate:
            out[n("g")] = TensorNeed((H, D))
        if self.position is not None:
            out.update(self.position.needs())
        return out

    def bind(self, get):
        n, H = self._name, self.heads
        stacked = torch.zeros((self.width, self.hidden), dtype=self.dtype, device=get(n("dq")).device)
        stacked[self.q_off:self.q_off + self.q_rank] = to_compute(get(n("dq")), self.dtype)
        stacked[self.kv_off:self.kv_off + self.key_dim] = to_compute(get(n("dkv")), self.dtype)
        if self.output_gate:
            stacked[self.g_off:self.g_off + H] = to_compute(get(n("g")), self.dtype)
        self.gemm_in = ops.bound_gemm(stacked, split_many=False)
        self.w_in = self.gemm_in.w
        self.gemm_uq = ops.bound_gemm(to_compute(get(n("uq")), self.dtype).contiguous(), split_many=False)
        self.w_uq = self.gemm_uq.w
        # per head: q' = Wuk_h^T q_plain (weights [heads, rank, dim]) and out_h = Wuv_h ctx_h (weights [heads, vdim, rank])
        self.w_fold = to_compute(get(n("uk")), self.dtype).view(H, self.dim, self.rank).transpose(1, 2).contiguous()
        self.w_uv = to_compute(get(n("uv")), self.dtype).view(H, self.vdim, self.rank).contiguous()
        self.gemm_o = ops.bound_gemm(to_compute(get(n("o")), self.dtype).contiguous(), split_many=True)
        self.w_o = self.gemm_o.w
        self.wq_norm = get(n("dq.norm")).to(torch.float32).contiguous()
        self.wkv_norm = get(n("dkv.norm")).to(torch.float32).contiguous()
        if self.position is not None:
            self.position.bind(get)
        self._capacity = None

    def cache_need(self):
        return CacheNeed("window" if self.window > 0 else "full", 1, self.key_dim, self.window, value_dim=-1)

    def forward(self, h, ctx, cache, state):
        T, H = h.shape[0], self.heads
        g = ctx.groups[cache.group]
        if not cache.writes:
            raise InvalidArgument("this attention computes its own keys and values: it cannot read another entry's cache")
        table = None
        if self.position is not None:
            table = self.position.fused_table()
            if table is None or 2 * table.numel() != self.rot:
                raise InvalidArgument("latent attention takes a rotation by a frequency table over the whole rotated part")
        proj = ctx.ws.rows("lattn.proj", T, self.width, self.dtype)
        self.gemm_in(h, proj)
        cq = ctx.ws.rows("lattn.cq", T, self.q_rank, self.dtype)
        ops.latent_prep(proj, self.q_off, self.q_rank, self.kv_off, self.rank, self.rot, self.wq_norm, self.wkv_norm, self.eps,
                        table, ctx.positions, g.slots, cq, cache.k)
        q = ctx.ws.rows("lattn.q", T, H * (self.dim + self.rot), self.dtype)
        self.gemm_uq(cq, q)
        folded = ctx.ws.rows("lattn.folded", T, H * self.key_dim, self.dtype)
        ops.gemm_heads(q, self.w_fold, folded, H)
        ops.latent_query_rot(q, self.dim, self.rot, table, ctx.positions, folded, self.rank, H)
        mixed = ctx.ws.rows("lattn.mixed", T, H * self.rank, self.dtype)       # per head: the weighted sum of latents
        self._attend(folded, mixed, ctx, g, cache)
        attn = ctx.ws.rows("lattn.out", T, H * self.vdim, self.dtype)
        ops.gemm_heads(mixed, self.w_uv, attn, H)
        if self.output_gate:
            ops.head_gate_mul(attn, proj[:, self.g_off:self.g_off + H], H, self.vdim)
        out = ctx.ws.rows("mixer.out", T, self.hidden, self.dtype)
        if self._capacity is None:
            self._capacity = ops.partial_capacity(ctx.ws.max_rows, self.gemm_o.N, self.gemm_o.K)
        return self.gemm_o(attn, out, lambda m: ctx.ws.flat("mixer.out.partial", m, torch.float32, self._capacity))

    def _attend(self, folded, mixed, ctx, g, cache):
        """One kv head of `key_dim` for all query heads; a value is the first `rank` elements of its key. bfloat16 with
        sizes in whole MMA steps runs on the tensor cores, everything else (float32 above all) on the CUDA cores."""
        H = self.heads
        n = ctx.multi_rows
        if ops.attention_latent_mma_takes(folded, cache.k, self.key_dim, self.rank):
            if n > 0:
                ops.attention_latent_prompt(folded, cache.k, mixed, ctx.query_start, ctx.context_lens, g.block_tables, ctx.multi_seqs,
                                            ctx.multi_max_queries, H, self.key_dim, self.rank, self.scale, self.window)
            if ctx.single_count > 0:
                longest = ctx.single_max_context if self.window <= 0 else min(ctx.single_max_context, self.window)
                split_keys = LATENT_SPLIT_KEYS
                while math.ceil(longest / split_keys) > MAX_SPLITS:
                    split_keys *= 2
                max_splits = max(1, math.ceil(longest / split_keys))
                scratch = ctx.ws.flat("lattn.split", ops.attention_split_scratch_floats(ctx.max_seqs, H, self.rank, MAX_SPLITS), torch.float32)
                ops.attention_latent_split(folded, cache.k, mixed, ctx.query_start, ctx.context_lens, g.block_tables, H, self.key_dim,
                                           self.rank, self.scale, ctx.single_seqs, ctx.single_count, split_keys, max_splits, scratch,
                                           self.window)
            return
        if n > 0:
            ops.attention_rows_dv(folded[:n], cache.k, cache.k, mixed[:n], ctx.seq_of_row[:n], ctx.query_start, ctx.context_lens,
                                  g.block_tables, H, 1, self.key_dim, self.rank, self.scale, self.window, values_in_keys=True)
        if ctx.single_count > 0:
            longest = ctx.single_max_context if self.window <= 0 else min(ctx.single_max_context, self.window)
            split_keys = SPLIT_KEYS
            while math.ceil(longest / split_keys) > MAX_SPLITS:
                split_keys *= 2
            max_splits = max(1, math.ceil(longest / split_keys))
            scratch = ctx.ws.flat("lattn.split", ops.attention_split_scratch_floats(ctx.max_seqs, H, self.rank, MAX_SPLITS), torch.float32)
            ops.attention_split_dv(folded, cache.k, cache.k, mixed, ctx.query_start, ctx.context_lens, g.block_tables, H, 1,
                                   self.key_dim, self.rank, self.scale, ctx.single_seqs, ctx.single_count, split_keys, max_splits,
                                   scratch, self.window, values_in_keys=True)


register_part("mixer", "latent_attention", LatentAttention, replace=True)
