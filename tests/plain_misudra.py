"""A plain, slow Misudra in numpy: whole sequences, no cache, no state carried between calls, one function
per mechanism. Arithmetic is float64 on the stored values. Nothing here imports the engine package: the
tests compare the two.

A Misudra model lists its layers in any order. A layer is a mixer behind a norm and, optionally, a
feed-forward behind a norm (both added to the residual stream). Mixers:

  latent_attention  queries through a normed latent; keys and values from one normed latent per token plus
                    one rotated key part shared by all heads; a sliding window; a sigmoid gate per head;
  gla               gated linear attention: a matrix state per head, decayed by one factor per key channel;
  mamba2            a state-space recurrence with a scalar decay per head behind a short causal convolution.

Feed-forwards: `dense` (a gated unit with the tanh form of gelu and biases) and `moe` (softmax router, experts
in blocks of consecutive experts of which only the best blocks may be chosen, clamped gated experts).

The token embedding passes a norm; a span of layers may run several times in a row (`loop`), and ahead of each
pass (and of the first) the stream is mixed with the embedding output by one product over their concatenation.
"""
from __future__ import annotations

import json
import struct
from pathlib import Path

import numpy as np


# --------------------------------------------------------------------------- small functions

def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
    return np.logaddexp(0.0, z)


def silu(z):
    return z * sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (z + 0.044715 * z ** 3)))


def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    x = np.asarray(x, dtype=np.float64)
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)


def f64(a):
    return np.asarray(a, dtype=np.float64)


_act = None       # with `bfloat16_activations()`: rounds what a 16-bit pipeline would keep in 16 bits


class bfloat16_activations:
    """Within this context the outputs of `linear` and of the layers' norms are rounded to bfloat16 (the weights of the
    tests are bfloat16 values already): the difference to the exact result is the noise that a pipeline with 16-bit
    activations cannot avoid, which is what a tolerance for such a pipeline is measured against."""

    def __enter__(self):
        global _act
        _act = lambda y: round_bf16(y).astype(np.float64)

    def __exit__(self, *exc):
        global _act
        _act = None


def linear(x, w, b=None):
    y = f64(x) @ f64(w).T
    y = y if b is None else y + f64(b)
    return y if _act is None else _act(y)


def kept(y):
    """A value that a 16-bit pipeline hands from one kernel to the next (or keeps in its cache)."""
    return y if _act is None else _act(y)


def layer_norm(x, w, eps):
    """The norm ahead of a sublayer: rms times a plain weight."""
    y = rms(x, eps) * f64(w)
    return y if _act is None else _act(y)


# --------------------------------------------------------------------------- latent attention

def rotate_half(x, positions, dims, base):
    """x [T, ..., dims]: dimension i turns with dimension i + dims/2 by the angle pos * base^(-2i/dims)."""
    half = dims // 2
    freq = np.float64(base) ** (-2.0 * np.arange(half) / dims)
    ang = f64(positions)[:, None] * freq[None, :]
    shape = (len(positions),) + (1,) * (x.ndim - 2) + (half,)
    c, s = np.cos(ang).reshape(shape), np.sin(ang).reshape(shape)
    a, b = x[..., :half], x[..., half:dims]
    return np.concatenate([a * c - b * s, b * c + a * s], axis=-1)


def window_softmax(scores, window):
    """scores [T, T] -> weights: row i sees columns j with 0 <= i - j < window."""
    T = scores.shape[0]
    i = np.arange(T)
    d = i[:, None] - i[None, :]
    s = np.where((d >= 0) & (d < window), scores, -np.inf)
    s = s - s.max(axis=-1, keepdims=True)
    p = np.exp(s)
    return p / p.sum(axis=-1, keepdims=True)


def latent_attention_mixer(h, w, p, mx, eps, positions):
    H, dim, rot, vdim, R = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
    T = h.shape[0]
    base = mx["rot"]["base"] if rot else 1.0
    cq = kept(rms(linear(h, w[p + "dq"]), eps) * f64(w[p + "dq.norm"]))
    q = linear(cq, w[p + "uq"]).reshape(T, H, dim + rot)
    q_plain, q_rot = q[..., :dim], rotate_half(q[..., dim:], positions, rot, base)
    kv = linear(h, w[p + "dkv"])
    c = kept(rms(kv[:, :R], eps) * f64(w[p + "dkv.norm"]))
    k_rot = kept(rotate_half(kv[:, R:], positions, rot, base))                # [T, rot], one for all heads
    k_plain = linear(c, w[p + "uk"]).reshape(T, H, dim)
    v = linear(c, w[p + "uv"]).reshape(T, H, vdim)
    gate = sigmoid(linear(h, w[p + "g"]))                                      # [T, H]
    out = np.zeros((T, H, vdim))
    for a in range(H):
        s = (q_plain[:, a] @ k_plain[:, a].T + q_rot[:, a] @ k_rot.T) * mx["scale"]
        out[:, a] = (window_softmax(s, mx["mask"]["size"]) @ v[:, a]) * gate[:, a:a + 1]
    return linear(kept(out.reshape(T, H * vdim)), w[p + "o"])


# --------------------------------------------------------------------------- recurrences

def decayed_outer_recurrence(q, k, v, decay):
    """Per head a matrix S (key channels x value channels) from zero: S <- diag(decay_t) S + k_t v_t^T, o_t = S^T q_t.
    q, k, decay [T, heads, dim] (decay may be [T, heads, 1]); v [T, heads, vdim] -> [T, heads, vdim]."""
    T, H, dim = q.shape
    S = np.zeros((H, dim, v.shape[-1]))
    out = np.zeros(v.shape)
    for t in range(T):
        S = decay[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = np.einsum("hdv,hd->hv", S, q[t])
    return out


def gla_mixer(h, w, p, mx, eps):
    H, dim, vdim = mx["heads"], mx["dim"], mx["vdim"]
    T = h.shape[0]
    q = (linear(h, w[p + "q"]) * dim ** -0.5).reshape(T, H, dim)
    k = linear(h, w[p + "k"]).reshape(T, H, dim)
    v = linear(h, w[p + "v"]).reshape(T, H, vdim)
    z = linear(linear(h, w[p + "a1"]), w[p + "a2"], w[p + "a2.b"])
    alpha = (sigmoid(z) ** (1.0 / mx["tau"])).reshape(T, H, dim)
    o = decayed_outer_recurrence(q, k, v, alpha)
    o = rms(o, eps) * f64(w[p + "norm"])                                        # per head, over vdim
    return linear(kept(o.reshape(T, H * vdim) * silu(linear(h, w[p + "g"]))), w[p + "o"])


def causal_conv(x, taps_w, bias):
    """x [T, C], taps_w [C, taps] (column taps - 1 weighs the current token); the sequence is padded with zeros on its left."""
    T, C = x.shape
    taps = taps_w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, C)), f64(x)], axis=0)
    y = np.zeros((T, C))
    for i in range(taps):
        y += padded[i:i + T] * f64(taps_w)[:, i][None, :]
    return y + f64(bias)


def mamba2_mixer(h, w, p, mx, eps):
    H, vdim, N, G = mx["heads"], mx["vdim"], mx["state"], mx["groups"]
    T = h.shape[0]
    inner = H * vdim
    u = linear(h, w[p + "in"])
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].reshape(T, H, vdim)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + f64(w[p + "dt_bias"]))                                   # [T, H]
    decay = np.exp(-np.exp(f64(w[p + "A_log"]))[None, :] * dt)                  # [T, H]
    group_of = np.arange(H) // (H // G)
    y = decayed_outer_recurrence(C[:, group_of], B[:, group_of], dt[:, :, None] * x, decay[:, :, None])
    y = y + f64(w[p + "D"])[None, :, None] * x
    y = y.reshape(T, inner) * silu(z)
    parts = mx["norm_groups"]
    y = rms(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * f64(w[p + "norm"])
    return linear(kept(y), w[p + "o"])


# --------------------------------------------------------------------------- feed-forwards

def dense_mlp(h, w, p):
    g = gelu_tanh(linear(h, w[p + "gate"], w[p + "gate.b"]))
    return linear(kept(g * linear(h, w[p + "up"], w[p + "up.b"])), w[p + "down"], w[p + "down.b"])


def route(scores, top, group_count, group_keep):
    """scores [E] -> (chosen experts, their weights). Experts lie in `group_count` equal blocks of consecutive experts; a
    group counts as much as its best expert, and only experts of the `group_keep` best groups can be chosen."""
    E = len(scores)
    per = E // group_count
    best = scores.reshape(group_count, per).max(axis=1)
    kept = np.argsort(-best, kind="stable")[:group_keep]
    allowed = np.zeros(E, dtype=bool)
    for g in kept:
        allowed[g * per:(g + 1) * per] = True
    order = np.argsort(-np.where(allowed, scores, -np.inf), kind="stable")[:top]
    return order, scores[order] / (scores[order].sum() + 1e-20)


def clamped_expert(h, gate, up, down, limit):
    g = np.minimum(linear(h, gate), limit)
    u = np.clip(linear(h, up), -limit, limit)
    return linear(kept(g * sigmoid(1.702 * g) * (u + 1.0)), down)


def moe_mlp(h, w, p, mlp, chosen_out=None):
    r = mlp["router"]
    z = linear(h, w[p + "router"])
    z = z - z.max(axis=-1, keepdims=True)
    s = np.exp(z)
    s /= s.sum(axis=-1, keepdims=True)
    out = np.zeros((h.shape[0], w[p + "e0.down"].shape[0]))
    for t in range(h.shape[0]):
        ids, weights = route(s[t], r["top"], r["groups"]["count"], r["groups"]["keep"])
        if chosen_out is not None:
            chosen_out.append((ids, weights, np.sort(s[t])[::-1]))
        for e, a in zip(ids, weights):
            q = f"{p}e{int(e)}."
            out[t] += a * clamped_expert(h[t:t + 1], w[q + "gate"], w[q + "up"], w[q + "down"], mlp["expert"]["limit"])[0]
    return out


# --------------------------------------------------------------------------- the model

def run_order(cfg):
    """Layer indices in the order they run, and the places (indices into that list) where a pass of the loop starts."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n)), []
    a, b, times = loop["start"], loop["stop"], loop["times"]
    order, starts = list(range(a)), []
    for _ in range(times):
        starts.append(len(order))
        order += list(range(a, b))
    return order + list(range(b, n)), starts


def forward(w, cfg, tokens, layers_out=None, routes_out=None):
    """float64 logits [T, vocab] of one sequence from position 0. With `layers_out` (a list) the residual stream
    after every layer run is appended to it."""
    eps = cfg["norm"]["eps"]
    tokens = np.asarray(tokens, dtype=np.int64)
    pos = np.arange(len(tokens))
    x = rms(f64(w["embed"])[tokens], eps) * f64(w["embed.norm"])
    x0 = x.copy()
    order, starts = run_order(cfg)
    for place, i in enumerate(order):
        if place in starts:
            x = linear(np.concatenate([x, x0], axis=-1), w["loop.in"])
        layer, p = cfg["layers"][i], f"l{i}."
        h = layer_norm(x, w[p + "norm1"], eps)
        kind = layer["type"]
        if kind == "latent_attention":
            y = latent_attention_mixer(h, w, p + "mix.", layer["mixer"], eps, pos)
        elif kind == "gla":
            y = gla_mixer(h, w, p + "mix.", layer["mixer"], eps)
        elif kind == "mamba2":
            y = mamba2_mixer(h, w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(f"unknown layer type {kind}")
        x = x + y
        mlp = layer.get("mlp")
        if mlp is not None:
            h = layer_norm(x, w[p + "norm2"], eps)
            x = x + (dense_mlp(h, w, p + "mlp.") if mlp["kind"] == "dense" else moe_mlp(h, w, p + "mlp.", mlp, routes_out))
        if layers_out is not None:
            layers_out.append(x.copy())
    return linear(layer_norm(x, w["final.norm"], eps), w["head"])


def generate(w, cfg, prompt, n):
    """Greedy: n tokens after the prompt, each the argmax of the logits at the last position."""
    tokens = list(prompt)
    for _ in range(n):
        tokens.append(int(np.argmax(forward(w, cfg, tokens)[-1])))
    return tokens[len(prompt):]


# --------------------------------------------------------------------------- configurations and weights for tests

def dense(ff=80):
    return {"ff": ff, "kind": "dense"}


def moe(ff=24, experts=8, top=2, groups=4, keep=2, limit=1.5):
    return {"expert": {"ff": ff, "limit": limit}, "kind": "moe",
            "router": {"experts": experts, "groups": {"count": groups, "keep": keep}, "top": top}}


def latent_layer(heads=4, dim=16, rot_dim=8, vdim=24, kv_rank=40, q_rank=48, window=24, base=10000.0, scale=None, mlp="dense"):
    mixer = {"dim": dim, "heads": heads, "kv_rank": kv_rank, "mask": {"size": window}, "q_rank": q_rank,
             "rot": {"base": base, "dims": rot_dim}, "rot_dim": rot_dim,
             "scale": scale if scale is not None else (dim + rot_dim) ** -0.5, "vdim": vdim}
    if rot_dim == 0:
        del mixer["rot"]                # nothing is rotated: the configuration need not say how
    return {"type": "latent_attention", "mixer": mixer, "mlp": dense() if mlp == "dense" else mlp}


def gla_layer(heads=2, dim=24, vdim=16, tau=8.0, mlp="dense"):
    return {"type": "gla", "mixer": {"dim": dim, "heads": heads, "tau": tau, "vdim": vdim},
            "mlp": dense() if mlp == "dense" else mlp}


def mamba2_layer(heads=4, vdim=16, state=16, groups=2, conv=3, norm_groups=2, mlp="dense"):
    return {"type": "mamba2", "mixer": {"conv": conv, "groups": groups, "heads": heads, "norm_groups": norm_groups,
                                        "state": state, "vdim": vdim},
            "mlp": dense() if mlp == "dense" else mlp}


def make_config(layers, vocab=160, width=64, eps=1e-6, loop=None):
    cfg = {"architecture": "Misudra", "layers": list(layers), "norm": {"eps": eps}, "vocab": vocab, "width": width}
    if loop is not None:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def tensor_shapes(cfg, decay_rank=8):
    """name -> shape. `decay_rank` is where the two steps of a gla layer's decay projection meet."""
    D = cfg["width"]
    s = {"embed": (cfg["vocab"], D), "embed.norm": (D,), "final.norm": (D,), "head": (cfg["vocab"], D)}
    if cfg.get("loop"):
        s["loop.in"] = (D, 2 * D)
    for i, layer in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", layer["mixer"]
        s[p + "norm1"] = (D,)
        m = p + "mix."
        if layer["type"] == "latent_attention":
            H, dim, rot, vdim, R, Q = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"], mx["q_rank"]
            s.update({m + "dq": (Q, D), m + "dq.norm": (Q,), m + "uq": (H * (dim + rot), Q), m + "dkv": (R + rot, D),
                      m + "dkv.norm": (R,), m + "uk": (H * dim, R), m + "uv": (H * vdim, R), m + "g": (H, D),
                      m + "o": (D, H * vdim)})
        elif layer["type"] == "gla":
            H, dim, vdim = mx["heads"], mx["dim"], mx["vdim"]
            s.update({m + "q": (H * dim, D), m + "k": (H * dim, D), m + "v": (H * vdim, D), m + "g": (H * vdim, D),
                      m + "o": (D, H * vdim), m + "norm": (vdim,), m + "a1": (decay_rank, D),
                      m + "a2": (H * dim, decay_rank), m + "a2.b": (H * dim,)})
        else:
            H, vdim, N, G = mx["heads"], mx["vdim"], mx["state"], mx["groups"]
            inner, ch = H * vdim, H * vdim + 2 * G * N
            s.update({m + "in": (2 * inner + 2 * G * N + H, D), m + "conv": (ch, mx["conv"]), m + "conv.b": (ch,),
                      m + "dt_bias": (H,), m + "A_log": (H,), m + "D": (H,), m + "norm": (inner,), m + "o": (D, inner)})
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        s[p + "norm2"] = (D,)
        f = p + "mlp."
        if mlp["kind"] == "dense":
            ff = mlp["ff"]
            s.update({f + "gate": (ff, D), f + "gate.b": (ff,), f + "up": (ff, D), f + "up.b": (ff,),
                      f + "down": (D, ff), f + "down.b": (D,)})
        else:
            ff = mlp["expert"]["ff"]
            for e in range(mlp["router"]["experts"]):
                s.update({f"{f}e{e}.gate": (ff, D), f"{f}e{e}.up": (ff, D), f"{f}e{e}.down": (D, ff)})
            s[f + "router"] = (mlp["router"]["experts"], D)
    return s


def round_bf16(x):
    a = np.ascontiguousarray(x, dtype=np.float32)
    bits = a.view(np.uint32).astype(np.uint64)
    rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16) << 16
    return rounded.astype(np.uint32).view(np.float32).reshape(np.shape(x))


def random_weights(cfg, seed, decay_rank=8, sharp=3.0, expert_gain=1.0):
    """float32 weights that bfloat16 holds exactly (so that both dtypes load the same model). Matrices are
    N(0, 1/in); the query and key paths of attention layers are `sharp` times larger so that attention is not flat
    and a key that is lost or misplaced moves the logits. `expert_gain` scales what the experts add to the stream:
    with random routers some token's choice between two experts is always a close call that 16-bit rounding decides
    the other way, and a small gain keeps such a flip within a 16-bit tolerance (32-bit runs see the experts to the
    last digit either way)."""
    rng = np.random.default_rng(seed)
    w = {}
    for name, shape in tensor_shapes(cfg, decay_rank).items():
        leaf = name.split(".")[-1]
        if name == "embed":
            t = rng.standard_normal(shape)
        elif leaf in ("norm1", "norm2") or name in ("final.norm", "embed.norm") or name.endswith(".norm"):
            t = 1.0 + rng.standard_normal(shape) * 0.1
        elif leaf == "b" and len(shape) == 1:
            t = rng.standard_normal(shape) * (1.0 if name.endswith("a2.b") else 0.2)
        elif leaf == "A_log":
            t = rng.uniform(-2.0, 0.5, shape)
        elif leaf == "dt_bias":
            t = rng.uniform(-3.0, 0.0, shape)
        elif leaf == "D":
            t = rng.standard_normal(shape)
        elif leaf == "conv":
            t = rng.standard_normal(shape) * 0.5
        else:
            t = rng.standard_normal(shape) / np.sqrt(shape[-1])
            if leaf in ("uq", "dkv"):
                t = t * sharp
            if leaf == "router":
                t = t * 4.0
            if leaf == "a2":
                t = t * 3.0
            if leaf == "down" and ".mlp.e" in name:
                t = t * expert_gain
        w[name] = round_bf16(np.asarray(t, dtype=np.float32))
    return w


def write_safetensors(path, tensors, bf16=True):
    """One file: 8-byte little-endian header length, JSON header, data. bf16 stores the upper 16 bits."""
    header, blobs, off = {}, [], 0
    for name, t in tensors.items():
        shape = list(np.shape(t))
        a = np.ascontiguousarray(t, dtype=np.float32).reshape(-1)
        if bf16:
            data = (a.view(np.uint32) >> 16).astype("<u2").tobytes()
            dt = "BF16"
        else:
            data = a.astype("<f4").tobytes()
            dt = "F32"
        header[name] = {"dtype": dt, "shape": shape, "data_offsets": [off, off + len(data)]}
        blobs.append(data)
        off += len(data)
    hj = json.dumps(header).encode()
    hj += b" " * (-len(hj) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


def write_model_dir(path, cfg, weights, bf16=True):
    path = Path(path)
    path.mkdir(parents=True, exist_ok=True)
    (path / "config.json").write_text(json.dumps(cfg))
    write_safetensors(path / "model.safetensors", weights, bf16=bf16)
