"""A gated delta rule with one decay per key channel: a recurrent mixer whose state has a fixed size.

Per value head a float32 matrix S (key channels x value channels) is carried from token to token:

    q, k, v  = silu(conv(h Wq^T)), silu(conv(h Wk^T)), silu(conv(h Wv^T))    short causal convolutions over time
    q, k     = unit vectors per head (x / sqrt(sum x^2 + unit_eps)), q times head_dim^(-1/2)
    beta     = sigmoid(h Wb^T)                                               one per value head
    decay    = exp(-exp(A_log[head]) * softplus((h Wa1^T) Wa2^T + dt_bias))   one per head and key channel
    S <- diag(decay) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q     the read-out sees the token's write
    out      = ((o / rms(o)) * w_norm * sigmoid((h Wg1^T) Wg2^T)) Wo^T          per head of value_dim

Value head i reads q/k head i // (heads / kv_heads). The state of a request is one float32 row in a state slot:
S of every head, then the convolutions' last `taps - 1` inputs. All projections that read h are one stacked
product; what enters the recurrence after them (decays, beta, unit norms, S itself) is float32 in either
compute dtype. Sizes and constants are parameters (`num_heads`, `num_kv_heads`, `head_dim`, `value_dim`,
`conv_taps`, `unit_eps`, `eps`); the two low-rank projections take their inner size from the tensors' shapes
(`decay_rank`, `gate_rank`).
"""
from __future__ import annotations

import torch

from .. import ops
from ..errors import InvalidArgument
from ..weights.loader import TensorNeed
from .base import Mixer, StateNeed, register_part, to_compute


def _up8(n: int) -> int:
    return (n + 7) // 8 * 8


class ChannelGatedDelta(Mixer):
    launches_only = False
    graph_safe = True       # the kernels read the step from device tensors only and skip sequences without a slot

    def __init__(self, spec, dtype, prefix: str = ""):
        p = spec.params
        self.prefix = prefix + p.get("prefix", "")
        self.hidden = int(p["hidden_size"])
        self.heads, self.kv_heads = int(p["num_heads"]), int(p["num_kv_heads"])
        self.dim, self.vdim = int(p["head_dim"]), int(p["value_dim"])
        self.taps = int(p.get("conv_taps", 1))
        self.decay_rank, self.gate_rank = int(p["decay_rank"]), int(p["gate_rank"])
        self.unit_eps = float(p.get("unit_eps", 1e-6))
        self.eps = float(p.get("eps", 1e-6))
        self.q_scale = float(p["q_scale"]) if p.get("q_scale") is not None else float(self.dim) ** -0.5
        if self.heads <= 0 or self.kv_heads <= 0 or self.heads % self.kv_heads:
            raise InvalidArgument(f"{self.heads} heads are not a multiple of {self.kv_heads} kv heads")
        if not 1 <= self.taps <= 16 or not 0 < self.dim <= 256:
            raise InvalidArgument(f"the delta rule takes 1 to 16 convolution taps and key heads of up to 256, got {self.taps} and {self.dim}")
        self.dtype = dtype
        self.qk, self.nv = self.kv_heads * self.dim, self.heads * self.vdim
        self.channels = 2 * self.qk + self.nv
        # columns of the stacked product; sections that feed another product start at multiples of 8
        self.q_off = 0
        self.k_off = self.qk
        self.v_off = 2 * self.qk
        self.a_off = _up8(self.channels)
        self.g_off = self.a_off + _up8(self.decay_rank)
        self.b_off = self.g_off + _up8(self.gate_rank)
        self.width = _up8(self.b_off + self.heads)
        self.state_floats = self.heads * self.dim * self.vdim
        self.output_bias = None

    def _name(self, leaf):
        return self.prefix + leaf

    def needs(self):
        D, n = self.hidden, self._name
        return {n("q"): TensorNeed((self.qk, D)), n("k"): TensorNeed((self.qk, D)), n("v"): TensorNeed((self.nv, D)),
                n("q.conv"): TensorNeed((self.qk, self.taps)), n("k.conv"): TensorNeed((self.qk, self.taps)),
                n("v.conv"): TensorNeed((self.nv, self.taps)), n("b"): TensorNeed((self.heads, D)),
                n("A_log"): TensorNeed((self.heads,), "norm"), n("norm"): TensorNeed((self.vdim,), "norm"),
                n("a1"): TensorNeed((self.decay_rank, D)), n("a2"): TensorNeed((self.heads * self.dim, self.decay_rank)),
                n("dt_bias"): TensorNeed((self.heads * self.dim,), "norm"),
                n("g1"): TensorNeed((self.gate_rank, D)), n("g2"): TensorNeed((self.nv, self.gate_rank)),
                n("o"): TensorNeed((D, self.nv))}

    def bind(self, get):
        n = self._name
        stacked = torch.zeros((self.width, self.hidden), dtype=self.dtype, device=get(n("q")).device)
        for leaf, off, rows in (("q", self.q_off, self.qk), ("k", self.k_off, self.qk), ("v", self.v_off, self.nv),
                                ("a1", self.a_off, self.decay_rank), ("g1", self.g_off, self.gate_rank),
                                ("b", self.b_off, self.heads)):
            stacked[off:off + rows] = to_compute(get(n(leaf)), self.dtype)
        self.gemm_in = ops.bound_gemm(stacked, split_many=False)
        self.w_in = self.gemm_in.w

        def second(leaf, rank):       # the second step of a low-rank projection; its k is padded to the section's width
            w = to_compute(get(n(leaf)), self.dtype)
            padded = torch.zeros((w.shape[0], _up8(rank)), dtype=self.dtype, device=w.device)
            padded[:, :rank] = w
            return ops.bound_gemm(padded, split_many=False)

        self.gemm_a2, self.gemm_g2 = second("a2", self.decay_rank), second("g2", self.gate_rank)
        self.w_a2, self.w_g2 = self.gemm_a2.w, self.gemm_g2.w
        self.gemm_o = ops.bound_gemm(to_compute(get(n("o")), self.dtype).contiguous(), split_many=True)
        self.w_o = self.gemm_o.w
        f32 = lambda leaf: get(n(leaf)).to(torch.float32).contiguous()
        self.conv_w = torch.cat([f32("q.conv"), f32("k.conv"), f32("v.conv")], dim=0).contiguous()
        self.a_log, self.dt_bias, self.norm_w = f32("A_log"), f32("dt_bias"), f32("norm")
        self._capacity = None

    def state_need(self):
        return StateNeed((self.state_floats + (self.taps - 1) * self.channels,), torch.float32)

    def forward(self, h, ctx, cache, state):
        T = h.shape[0]
        H, G, dim, vdim = self.heads, self.kv_heads, self.dim, self.vdim
        if state is None:
            raise InvalidArgument("the delta rule needs state slots (make the cache with `make_cache`)")
        proj = ctx.ws.rows("delta.proj", T, self.width, self.dtype)
        self.gemm_in(h, proj)
        a_raw = ctx.ws.rows("delta.a", T, H * dim, torch.float32)
        gate = ctx.ws.rows("delta.gate", T, self.nv, torch.float32)
        self.gemm_a2(proj[:, self.a_off:self.a_off + _up8(self.decay_rank)], a_raw)
        self.gemm_g2(proj[:, self.g_off:self.g_off + _up8(self.gate_rank)], gate)
        qn = ctx.ws.rows("delta.q", T, self.qk, torch.float32)
        kn = ctx.ws.rows("delta.k", T, self.qk, torch.float32)
        vn = ctx.ws.rows("delta.v", T, self.nv, torch.float32)
        beta = ctx.ws.rows("delta.beta", T, H, torch.float32)
        ops.delta_prep(proj, self.q_off, self.k_off, self.v_off, self.b_off, self.conv_w, state, self.state_floats,
                       ctx.seq_of_row, ctx.query_start, ctx.state_slots, H, G, dim, vdim, self.taps, self.unit_eps,
                       self.q_scale, qn, kn, vn, beta, a_raw, self.dt_bias, self.a_log)       # a_raw leaves as the decays
        o = ctx.ws.rows("delta.o", T, self.nv, torch.float32)
        ops.delta_rule(qn, kn, vn, beta, a_raw, state, self.state_floats, proj, self.q_off,
                       self.k_off, self.v_off, ctx.query_start, ctx.state_slots, ctx.S, H, G, dim, vdim, self.taps, o)
        gated = ctx.ws.rows("delta.gated", T, self.nv, self.dtype)
        ops.delta_out(o, gate, self.norm_w, self.eps, gated, H, vdim)
        out = ctx.ws.rows("mixer.out", T, self.hidden, self.dtype)
        if self._capacity is None:
            self._capacity = ops.partial_capacity(ctx.ws.max_rows, self.gemm_o.N, self.gemm_o.K)
        return self.gemm_o(gated, out, lambda m: ctx.ws.flat("mixer.out.partial", m, torch.float32, self._capacity))


register_part("mixer", "channel_gated_delta", ChannelGatedDelta, replace=True)
