"""Gated linear attention: a recurrent mixer whose matrix state decays with one factor per key channel.

Per head a float32 matrix S (key channels x value channels), zero at the start of a sequence, is carried from token
to token:

    q, k, v = (h Wq^T) * q_scale, h Wk^T, h Wv^T                     q_scale defaults to head_dim^(-1/2)
    decay   = sigmoid((h Wa1^T) Wa2^T + b_a2)^(1 / tau)               per head and key channel, in (0, 1)
    S <- diag(decay) S + k v^T;   o = S^T q                            the read-out sees the token's own write
    out     = ((o / rms(o)) * w_norm * silu(h Wg^T)) Wo^T              the norm per head of value_dim, w_norm shared by heads

The state of a request is one float32 row in a state slot. All projections that read h are one stacked product; the
second step of the decay projection writes float32, and everything that enters the recurrence after the projections
(the decays, S itself, the read-out's norm) is float32 in either compute dtype. The recurrence is the kernel of the
delta rule in its plain mode (no correction along the key). The decay projection's inner size comes from its tensors'
shapes (`decay_rank`).
"""
from __future__ import annotations

import torch

from .. import ops
from ..errors import InvalidArgument
from ..weights.loader import TensorNeed
from .base import Mixer, StateNeed, register_part, to_compute


def _up8(n: int) -> int:
    return (n + 7) // 8 * 8


class GatedLinearAttention(Mixer):
    launches_only = False
    graph_safe = True       # the kernels read the step from device tensors only and skip sequences without a slot

    def __init__(self, spec, dtype, prefix: str = ""):
        p = spec.params
        self.prefix = prefix + p.get("prefix", "")
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["num_heads"])
        self.dim, self.vdim = int(p["head_dim"]), int(p["value_dim"])
        self.tau = float(p["tau"])
        self.decay_rank = int(p["decay_rank"])
        self.eps = float(p.get("eps", 1e-6))
        self.q_scale = float(p["q_scale"]) if p.get("q_scale") is not None else float(self.dim) ** -0.5
        if min(self.heads, self.vdim, self.decay_rank) <= 0 or not 0 < self.dim <= 256 or self.tau <= 0:
            raise InvalidArgument(f"gated linear attention: bad sizes heads={self.heads} dim={self.dim} (1 to 256) vdim={self.vdim} "
                                  f"tau={self.tau}")
        self.dtype = dtype
        self.nqk, self.nv = self.heads * self.dim, self.heads * self.vdim
        self.q_off = 0
        self.k_off = _up8(self.nqk)
        self.v_off = self.k_off + _up8(self.nqk)
        self.g_off = self.v_off + _up8(self.nv)
        self.a_off = self.g_off + _up8(self.nv)
        self.width = self.a_off + _up8(self.decay_rank)
        self.state_floats = self.heads * self.dim * self.vdim
        self.output_bias = None

    def _name(self, leaf):
        return self.prefix + leaf

    def needs(self):
        D, n = self.hidden, self._name
        return {n("q"): TensorNeed((self.nqk, D)), n("k"): TensorNeed((self.nqk, D)), n("v"): TensorNeed((self.nv, D)),
                n("g"): TensorNeed((self.nv, D)), n("o"): TensorNeed((D, self.nv)), n("norm"): TensorNeed((self.vdim,), "norm"),
                n("a1"): TensorNeed((self.decay_rank, D)), n("a2"): TensorNeed((self.nqk, self.decay_rank)),
                n("a2.b"): TensorNeed((self.nqk,), "norm")}

    def bind(self, get):
        n = self._name
        stacked = torch.zeros((self.width, self.hidden), dtype=self.dtype, device=get(n("q")).device)
        for leaf, off, rows in (("q", self.q_off, self.nqk), ("k", self.k_off, self.nqk), ("v", self.v_off, self.nv),
                                ("g", self.g_off, self.nv), ("a1", self.a_off, self.decay_rank)):
            stacked[off:off + rows] = to_compute(get(n(leaf)), self.dtype)
        self.gemm_in = ops.bound_gemm(stacked, split_many=False)
        self.w_in = self.gemm_in.w
        a2 = to_compute(get(n("a2")), self.dtype)
        padded = torch.zeros((a2.shape[0], _up8(self.decay_rank)), dtype=self.dtype, device=a2.device)      # k padded to the section's width
        padded[:, :self.decay_rank] = a2
        self.gemm_a2 = ops.bound_gemm(padded, split_many=False)
        self.w_a2 = self.gemm_a2.w
        self.gemm_o = ops.bound_gemm(to_compute(get(n("o")), self.dtype).contiguous(), split_many=True)
        self.w_o = self.gemm_o.w
        self.a2_bias = get(n("a2.b")).to(torch.float32).contiguous()
        self.norm_w = get(n("norm")).to(torch.float32).contiguous()
        self._capacity = None

    def state_need(self):
        return StateNeed((self.state_floats,), torch.float32)

    def forward(self, h, ctx, cache, state):
        T, H, dim, vdim = h.shape[0], self.heads, self.dim, self.vdim
        if state is None:
            raise InvalidArgument("gated linear attention needs state slots (make the cache with `make_cache`)")
        proj = ctx.ws.rows("gla.proj", T, self.width, self.dtype)
        self.gemm_in(h, proj)
        decay = ctx.ws.rows("gla.decay", T, self.nqk, torch.float32)
        self.gemm_a2(proj[:, self.a_off:self.a_off + _up8(self.decay_rank)], decay)
        qn = ctx.ws.rows("gla.q", T, self.nqk, torch.float32)
        kn = ctx.ws.rows("gla.k", T, self.nqk, torch.float32)
        vn = ctx.ws.rows("gla.v", T, self.nv, torch.float32)
        ops.gla_prep(proj, self.q_off, self.k_off, self.v_off, H, dim, vdim, self.q_scale, self.tau, self.a2_bias, qn, kn, vn, decay)
        o = ctx.ws.rows("gla.o", T, self.nv, torch.float32)
        ops.delta_rule(qn, kn, vn, None, decay, state, self.state_floats, proj, self.q_off, self.k_off, self.v_off,
                       ctx.query_start, ctx.state_slots, ctx.S, H, H, dim, vdim, 1, o, plain=True)
        gated = ctx.ws.rows("gla.gated", T, self.nv, self.dtype)
        ops.head_norm_gate(o, proj[:, self.g_off:self.g_off + self.nv], self.norm_w, self.eps, gated, H, vdim, ops.GATE_SILU)
        out = ctx.ws.rows("mixer.out", T, self.hidden, self.dtype)
        if self._capacity is None:
            self._capacity = ops.partial_capacity(ctx.ws.max_rows, self.gemm_o.N, self.gemm_o.K)
        return self.gemm_o(gated, out, lambda m: ctx.ws.flat("mixer.out.partial", m, torch.float32, self._capacity))


register_part("mixer", "gated_linear_attention", GatedLinearAttention, replace=True)
