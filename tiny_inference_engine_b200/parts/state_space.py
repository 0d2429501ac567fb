"""A state-space mixer in its dual, attention-like form: a recurrence with one scalar decay per head.

    [z | x | B | C | dt] = h Win^T             z, x: heads * value_dim; B, C: groups * state_size; dt: heads
    x, B, C = silu(conv(x, B, C) + b_conv)     a short causal convolution per channel over time (the sequence padded with zeros on its left)
    dt      = softplus(dt + dt_bias)           unbounded above
    S <- exp(-exp(A_log_h) dt) S + dt B x^T;   y = S^T C + D_h x      per head; head h reads group h // (heads / groups)
    out     = (norm_parts(y * silu(z)) * w_norm) Wo^T                  the gate first; each of `norm_groups` equal parts of the
                                                                       row is divided by its own root mean square

S (state_size x value_dim per head) is float32 and starts at zero. A request's state is one float32 row in a state
slot: S of every head, then the convolution's last `taps - 1` inputs. What enters the recurrence after the
projection and the convolution (step sizes, decays, S, the norm) is float32 in either compute dtype. The recurrence
is the kernel of the delta rule in its plain mode with the step size as the factor on the written value and one decay
for all key channels of a head: B plays the key, C the query, x the value.
"""
from __future__ import annotations

import torch

from .. import ops
from ..errors import InvalidArgument
from ..weights.loader import TensorNeed
from .base import Mixer, StateNeed, register_part, to_compute


def _up8(n: int) -> int:
    return (n + 7) // 8 * 8


class StateSpaceDual(Mixer):
    launches_only = False
    graph_safe = True       # the kernels read the step from device tensors only and skip sequences without a slot

    def __init__(self, spec, dtype, prefix: str = ""):
        p = spec.params
        self.prefix = prefix + p.get("prefix", "")
        self.hidden = int(p["hidden_size"])
        self.heads, self.groups = int(p["num_heads"]), int(p["num_groups"])
        self.vdim, self.state_size = int(p["value_dim"]), int(p["state_size"])
        self.taps = int(p.get("conv_taps", 1))
        self.norm_parts = int(p.get("norm_groups", 1))
        self.eps = float(p.get("eps", 1e-6))
        if min(self.heads, self.groups, self.vdim) <= 0 or self.heads % self.groups:
            raise InvalidArgument(f"state-space mixer: {self.heads} heads are not a multiple of {self.groups} groups")
        if not 1 <= self.taps <= 16 or not 0 < self.state_size <= 256:
            raise InvalidArgument(f"state-space mixer: 1 to 16 convolution taps and a state of up to 256, got {self.taps} and {self.state_size}")
        self.inner = self.heads * self.vdim
        if self.norm_parts <= 0 or self.inner % self.norm_parts:
            raise InvalidArgument(f"state-space mixer: a row of {self.inner} does not split into {self.norm_parts} equal parts")
        self.dtype = dtype
        self.ngn = self.groups * self.state_size
        self.channels = self.inner + 2 * self.ngn
        # columns of the input product, as the checkpoint orders them
        self.z_off, self.x_off = 0, self.inner
        self.b_off = 2 * self.inner
        self.c_off = self.b_off + self.ngn
        self.dt_off = self.c_off + self.ngn
        self.in_rows = self.dt_off + self.heads
        self.width = _up8(self.in_rows)
        self.state_floats = self.heads * self.state_size * self.vdim
        self.output_bias = None

    def _name(self, leaf):
        return self.prefix + leaf

    def needs(self):
        D, n = self.hidden, self._name
        return {n("in"): TensorNeed((self.in_rows, D)), n("conv"): TensorNeed((self.channels, self.taps)),
                n("conv.b"): TensorNeed((self.channels,), "norm"), n("dt_bias"): TensorNeed((self.heads,), "norm"),
                n("A_log"): TensorNeed((self.heads,), "norm"), n("D"): TensorNeed((self.heads,), "norm"),
                n("norm"): TensorNeed((self.inner,), "norm"), n("o"): TensorNeed((D, self.inner))}

    def bind(self, get):
        n = self._name
        w_in = to_compute(get(n("in")), self.dtype)
        stacked = torch.zeros((self.width, self.hidden), dtype=self.dtype, device=w_in.device)
        stacked[:self.in_rows] = w_in
        self.gemm_in = ops.bound_gemm(stacked, split_many=False)
        self.w_in = self.gemm_in.w
        self.gemm_o = ops.bound_gemm(to_compute(get(n("o")), self.dtype).contiguous(), split_many=True)
        self.w_o = self.gemm_o.w
        f32 = lambda leaf: get(n(leaf)).to(torch.float32).contiguous()
        # the recurrence's kernels list channels as query, key, value: C, B, x (the checkpoint: x, B, C)
        conv, bias = f32("conv"), f32("conv.b")
        x_end, b_end = self.inner, self.inner + self.ngn
        self.conv_w = torch.cat([conv[b_end:], conv[x_end:b_end], conv[:x_end]], dim=0).contiguous()
        self.conv_b = torch.cat([bias[b_end:], bias[x_end:b_end], bias[:x_end]], dim=0).contiguous()
        self.dt_bias, self.a_log, self.skip, self.norm_w = f32("dt_bias"), f32("A_log"), f32("D"), f32("norm")
        self._capacity = None

    def state_need(self):
        return StateNeed((self.state_floats + (self.taps - 1) * self.channels,), torch.float32)

    def forward(self, h, ctx, cache, state):
        T, H, G, N, vdim = h.shape[0], self.heads, self.groups, self.state_size, self.vdim
        if state is None:
            raise InvalidArgument("the state-space mixer needs state slots (make the cache with `make_cache`)")
        proj = ctx.ws.rows("ssd.proj", T, self.width, self.dtype)
        self.gemm_in(h, proj)
        cn = ctx.ws.rows("ssd.c", T, self.ngn, torch.float32)
        bn = ctx.ws.rows("ssd.b", T, self.ngn, torch.float32)
        xn = ctx.ws.rows("ssd.x", T, self.inner, torch.float32)
        dt = ctx.ws.rows("ssd.dt", T, H, torch.float32)
        decay = ctx.ws.rows("ssd.decay", T, H, torch.float32)
        ops.ssd_prep(proj, self.c_off, self.b_off, self.x_off, self.dt_off, self.conv_w, self.conv_b, state, self.state_floats,
                     ctx.seq_of_row, ctx.query_start, ctx.state_slots, H, G, N, vdim, self.taps, self.dt_bias, self.a_log,
                     cn, bn, xn, dt, decay)
        o = ctx.ws.rows("ssd.o", T, self.inner, torch.float32)
        ops.delta_rule(cn, bn, xn, dt, decay, state, self.state_floats, proj, self.c_off, self.b_off, self.x_off,
                       ctx.query_start, ctx.state_slots, ctx.S, H, G, N, vdim, self.taps, o, plain=True, decay_per_head=True)
        gated = ctx.ws.rows("ssd.gated", T, self.inner, self.dtype)
        ops.ssd_out(o, xn, proj[:, self.z_off:self.z_off + self.inner], self.skip, self.norm_w, self.eps, gated, H, vdim,
                    self.norm_parts)
        out = ctx.ws.rows("mixer.out", T, self.hidden, self.dtype)
        if self._capacity is None:
            self._capacity = ops.partial_capacity(ctx.ws.max_rows, self.gemm_o.N, self.gemm_o.K)
        return self.gemm_o(gated, out, lambda m: ctx.ws.flat("mixer.out.partial", m, torch.float32, self._capacity))


register_part("mixer", "state_space_dual", StateSpaceDual, replace=True)
