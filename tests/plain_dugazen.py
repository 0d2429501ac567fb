"""A plain, slow Dugazen in numpy: whole sequences, no cache, no state carried between calls, one
function per mechanism. Arithmetic is float64 on the stored values. Nothing here imports the engine
package: the tests compare the two.

A Dugazen model alternates, in any order its configuration lists, two kinds of layer:

  attention      sliding-window grouped-query attention with biases, an RMS norm over the whole q (and k)
                 projection, a rotation of the first `rot.dims` dimensions of each head, keys and values of
                 different sizes, values blended with those of the first blending layer, a sigmoid gate
                 on the heads' outputs;
  channel_delta  a gated delta rule with one decay per key channel: a matrix state per head that is
                 decayed row by row, corrected towards the token's value along its key, and read by its
                 query; short causal convolutions ahead of q, k and v.

Every sublayer sits between two norms: x += m * norm_after(sublayer(norm_before(x))).
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


def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    x = np.asarray(x, dtype=np.float64)
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)


_act = None       # with `bfloat16_activations()`: rounds what a 16-bit pipeline would keep in 16 bits


class bfloat16_activations:
    """Within this context the outputs of `linear` and of the layers' norms are rounded to bfloat16 (the weights
    of the tests are bfloat16 values already): the difference to the exact result is the noise that a pipeline
    with 16-bit activations cannot avoid, which is what a tolerance for such a pipeline is measured against."""

    def __enter__(self):
        global _act
        _act = lambda y: round_bf16(y).astype(np.float64)

    def __exit__(self, *exc):
        global _act
        _act = None


def norm_one_plus(x, w, eps):
    """The layers' norm: the weight is stored as its distance from one."""
    y = rms(x, eps) * (1.0 + np.asarray(w, dtype=np.float64))
    return y if _act is None else _act(y)


def linear(x, w, b=None):
    y = np.asarray(x, dtype=np.float64) @ np.asarray(w, dtype=np.float64).T
    y = y if b is None else y + np.asarray(b, dtype=np.float64)
    return y if _act is None else _act(y)


# --------------------------------------------------------------------------- attention layer

def rotate_partial(x, positions, heads, dim, rot_dims, base):
    """Dimension i < rot_dims/2 of each head turns with dimension i + rot_dims/2 by the angle
    pos * base^(-2i/rot_dims); dimensions from rot_dims on stay."""
    T = x.shape[0]
    half = rot_dims // 2
    freq = np.float64(base) ** (-2.0 * np.arange(half) / rot_dims)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * freq[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    v = np.array(x, dtype=np.float64).reshape(T, heads, dim)
    a, b = v[..., :half].copy(), v[..., half:rot_dims].copy()
    v[..., :half] = a * c - b * s
    v[..., half:rot_dims] = b * c + a * s
    return v.reshape(T, heads * dim)


def windowed_attention(q, k, v, heads, kv_heads, dim, vdim, scale, window):
    """Query i sees keys j with 0 <= i - j < window; softmax over those; [T, heads * vdim]."""
    T = q.shape[0]
    q = q.reshape(T, heads, dim)
    k = k.reshape(T, kv_heads, dim)
    v = v.reshape(T, kv_heads, vdim)
    out = np.zeros((T, heads, vdim))
    per = heads // kv_heads
    i = np.arange(T)
    seen = (i[:, None] - i[None, :] >= 0) & (i[:, None] - i[None, :] < window)
    for h in range(heads):
        g = h // per
        s = (q[:, h] @ k[:, g].T) * scale
        s = np.where(seen, s, -np.inf)
        s = s - s.max(axis=-1, keepdims=True)
        p = np.exp(s)
        p /= p.sum(axis=-1, keepdims=True)
        out[:, h] = p @ v[:, g]
    return out.reshape(T, heads * vdim)


def attention_mixer(h, w, p, mx, eps, positions, v_first):
    """Returns (output [T, width], this layer's values before blending when it is the first blending layer,
    else v_first unchanged)."""
    H, G, dim, vdim = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    q = linear(h, w[p + "q"], w[p + "q.b"])
    k = linear(h, w[p + "k"], w[p + "k.b"])
    v = linear(h, w[p + "v"], w[p + "v.b"])
    q = rms(q, eps) * w[p + "q.norm"].astype(np.float64)        # over all heads at once
    k = rms(k, eps) * w[p + "k.norm"].astype(np.float64)
    q = rotate_partial(q, positions, H, dim, mx["rot"]["dims"], mx["rot"]["base"])
    k = rotate_partial(k, positions, G, dim, mx["rot"]["dims"], mx["rot"]["base"])
    if mx.get("v_mix"):
        if v_first is None:
            v_first = v
        else:
            lam = float(np.asarray(w[p + "vmix"], dtype=np.float64).reshape(()))
            v = (1.0 - lam) * v + lam * v_first
    o = windowed_attention(q, k, v, H, G, dim, vdim, mx["scale"], mx["mask"]["size"])
    o = o * sigmoid(linear(h, w[p + "g"]))
    return linear(o, w[p + "o"], w[p + "o.b"]), v_first


# --------------------------------------------------------------------------- channel_delta layer

def short_conv(x, taps_w):
    """y[t, c] = sum_i taps_w[c, i] * x[t - (taps - 1) + i, c], zeros before the start; then silu."""
    T, C = x.shape
    taps = taps_w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, C)), np.asarray(x, dtype=np.float64)], axis=0)
    y = np.zeros((T, C))
    for i in range(taps):
        y += padded[i:i + T] * taps_w[:, i].astype(np.float64)[None, :]
    return silu(y)


def unit(x):
    return x / np.sqrt((x * x).sum(axis=-1, keepdims=True) + 1e-6)


def delta_rule(q, k, v, beta, decay):
    """One head. q, k [T, dim] (unit vectors, q scaled), v [T, vdim], beta [T], decay [T, dim] in (0, 1).
    S (dim x vdim) starts at zero; per token: rows of S shrink by decay, S takes k (beta (v - S^T k))^T,
    and the output is S^T q (it sees the token's own write)."""
    T, dim = q.shape
    S = np.zeros((dim, v.shape[1]))
    out = np.zeros((T, v.shape[1]))
    for t in range(T):
        S = decay[t][:, None] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + np.outer(k[t], u)
        out[t] = S.T @ q[t]
    return out


def channel_delta_mixer(h, w, p, mx, eps):
    H, G, dim, vdim = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    T = h.shape[0]
    q = short_conv(linear(h, w[p + "q"]), w[p + "q.conv"]).reshape(T, G, dim)
    k = short_conv(linear(h, w[p + "k"]), w[p + "k.conv"]).reshape(T, G, dim)
    v = short_conv(linear(h, w[p + "v"]), w[p + "v.conv"]).reshape(T, H, vdim)
    q = unit(q) * dim ** -0.5
    k = unit(k)
    beta = sigmoid(linear(h, w[p + "b"]))                                            # [T, H]
    step = softplus(linear(linear(h, w[p + "a1"]), w[p + "a2"]) + w[p + "dt_bias"].astype(np.float64))
    rate = np.exp(w[p + "A_log"].astype(np.float64))                                  # [H]
    decay = np.exp(-rate[None, :, None] * step.reshape(T, H, dim))                    # [T, H, dim]
    gate = sigmoid(linear(linear(h, w[p + "g1"]), w[p + "g2"])).reshape(T, H, vdim)
    per = H // G
    out = np.zeros((T, H, vdim))
    for hd in range(H):
        o = delta_rule(q[:, hd // per], k[:, hd // per], v[:, hd], beta[:, hd], decay[:, hd])
        out[:, hd] = rms(o, eps) * w[p + "norm"].astype(np.float64) * gate[:, hd]
    return linear(out.reshape(T, H * vdim), w[p + "o"])


# --------------------------------------------------------------------------- feed-forward, model

def clamped_glu(h, w, p, limit):
    g = np.minimum(linear(h, w[p + "gate"]), limit)
    u = np.clip(linear(h, w[p + "up"]), -limit, limit)
    return linear(g * sigmoid(1.702 * g) * (u + 1.0), w[p + "down"])


def forward(w, cfg, tokens, layers_out=None):
    """float64 logits [T, vocab] of one sequence from position 0. With `layers_out` (a list) the residual
    stream after every layer is appended to it."""
    eps, m = cfg["norm"]["eps"], cfg["residual_mult"]
    tokens = np.asarray(tokens, dtype=np.int64)
    pos = np.arange(len(tokens))
    x = w["embed"][tokens].astype(np.float64)
    v_first = None
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = norm_one_plus(x, w[p + "norm1"], eps)
        if layer["type"] == "attention":
            y, v_first = attention_mixer(h, w, p + "mix.", layer["mixer"], eps, pos, v_first)
        elif layer["type"] == "channel_delta":
            y = channel_delta_mixer(h, w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(f"unknown layer type {layer['type']}")
        x = x + m * norm_one_plus(y, w[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            h = norm_one_plus(x, w[p + "norm2"], eps)
            y = clamped_glu(h, w, p + "mlp.", layer["mlp"]["limit"])
            x = x + m * norm_one_plus(y, w[p + "norm2b"], eps)
        if layers_out is not None:
            layers_out.append(x.copy())
    return linear(norm_one_plus(x, w["final.norm"], eps), w["head"]) * cfg["logit_scale"]


def generate(w, cfg, prompt, n):
    """Greedy: n tokens after the prompt, each the argmax of the logits at the last position."""
    tokens = list(prompt)
    for _ in range(n):
        tokens.append(int(np.argmax(forward(w, cfg, tokens)[-1])))
    return tokens[len(prompt):]


# --------------------------------------------------------------------------- configurations and weights for tests

def attention_layer(heads=4, kv_heads=2, dim=32, vdim=16, window=24, rot_dims=16, base=10000.0, scale=None,
                    v_mix=True, ff=96, limit=3.0):
    return {"type": "attention",
            "mixer": {"dim": dim, "heads": heads, "kv_heads": kv_heads, "mask": {"size": window},
                      "rot": {"base": base, "dims": rot_dims}, "scale": scale if scale is not None else dim ** -0.5,
                      "v_mix": v_mix, "vdim": vdim},
            "mlp": None if ff is None else {"ff": ff, "kind": "dense", "limit": limit}}


def delta_layer(heads=4, kv_heads=2, dim=16, vdim=24, conv=3, ff=None, limit=3.0):
    return {"type": "channel_delta",
            "mixer": {"conv": conv, "dim": dim, "heads": heads, "kv_heads": kv_heads, "vdim": vdim},
            "mlp": None if ff is None else {"ff": ff, "kind": "dense", "limit": limit}}


def make_config(layers, vocab=160, width=64, eps=1e-6, residual_mult=0.5, logit_scale=1.5):
    return {"architecture": "Dugazen", "layers": list(layers), "logit_scale": logit_scale, "norm": {"eps": eps},
            "residual_mult": residual_mult, "vocab": vocab, "width": width}


def tensor_shapes(cfg, low_rank=8, gate_rank=None):
    """name -> shape. The two-step projections of a channel_delta layer meet at `low_rank` (a1/a2) and
    `gate_rank` (g1/g2; None: the same)."""
    gate_rank = low_rank if gate_rank is None else gate_rank
    D = cfg["width"]
    s = {"embed": (cfg["vocab"], D), "final.norm": (D,), "head": (cfg["vocab"], D)}
    for i, layer in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", layer["mixer"]
        H, G, dim, vdim = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
        s[p + "norm1"] = s[p + "norm1b"] = (D,)
        if layer["type"] == "attention":
            s.update({p + "mix.q": (H * dim, D), p + "mix.q.b": (H * dim,), p + "mix.k": (G * dim, D),
                      p + "mix.k.b": (G * dim,), p + "mix.v": (G * vdim, D), p + "mix.v.b": (G * vdim,),
                      p + "mix.q.norm": (H * dim,), p + "mix.k.norm": (G * dim,), p + "mix.g": (H * vdim, D),
                      p + "mix.o": (D, H * vdim), p + "mix.o.b": (D,)})
            if mx.get("v_mix"):
                s[p + "mix.vmix"] = ()
        else:
            s.update({p + "mix.q": (G * dim, D), p + "mix.q.conv": (G * dim, mx["conv"]), p + "mix.k": (G * dim, D),
                      p + "mix.k.conv": (G * dim, mx["conv"]), p + "mix.v": (H * vdim, D),
                      p + "mix.v.conv": (H * vdim, mx["conv"]), p + "mix.b": (H, D), p + "mix.A_log": (H,),
                      p + "mix.norm": (vdim,), p + "mix.a1": (low_rank, D), p + "mix.a2": (H * dim, low_rank),
                      p + "mix.dt_bias": (H * dim,), p + "mix.g1": (gate_rank, D), p + "mix.g2": (H * vdim, gate_rank),
                      p + "mix.o": (D, H * vdim)})
        if layer.get("mlp") is not None:
            ff = layer["mlp"]["ff"]
            s.update({p + "norm2": (D,), p + "norm2b": (D,), p + "mlp.gate": (ff, D), p + "mlp.up": (ff, D),
                      p + "mlp.down": (D, ff)})
    return s


def round_bf16(x):
    a = np.ascontiguousarray(x, dtype=np.float32)
    bits = a.view(np.uint32).astype(np.uint64)
    rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16) << 16
    return rounded.astype(np.uint32).view(np.float32).reshape(np.shape(x))      # (a scalar stays a scalar)


def random_weights(cfg, seed, low_rank=8, sharp=4.0, gate_rank=None):
    """float32 weights that bfloat16 holds exactly (so that both dtypes load the same model). Matrices are
    N(0, 1/in); norm weights and biases are small; q and k projections of attention layers are `sharp`
    times larger so that attention is not flat and a key that is lost or misplaced moves the logits."""
    rng = np.random.default_rng(seed)
    w = {}
    for name, shape in tensor_shapes(cfg, low_rank, gate_rank).items():
        leaf = name.split(".")[-1]
        if name in ("embed",):
            t = rng.standard_normal(shape)
        elif leaf in ("norm1", "norm2", "norm1b", "norm2b") or name == "final.norm":
            t = rng.standard_normal(shape) * 0.1
        elif name.endswith("q.norm") or name.endswith("k.norm") or name.endswith("mix.norm"):
            t = 1.0 + rng.standard_normal(shape) * 0.1
        elif leaf == "b" and len(shape) == 1:
            t = rng.standard_normal(shape) * 0.2
        elif leaf == "vmix":
            t = np.asarray(rng.uniform(0.2, 0.6))
        elif leaf == "A_log":
            t = rng.uniform(-1.0, 0.5, shape)
        elif leaf == "dt_bias":
            t = rng.uniform(-3.0, 0.0, shape)
        elif leaf == "conv":
            t = rng.standard_normal(shape) * 0.5
        else:
            t = rng.standard_normal(shape) / np.sqrt(shape[-1])
            if name.endswith("mix.q") or name.endswith("mix.k"):
                kind = cfg["layers"][int(name[1:name.index(".")])]["type"]
                if kind == "attention":
                    t = t * sharp
        w[name] = round_bf16(np.asarray(t, dtype=np.float32))
    return w


def write_safetensors(path, tensors, bf16=True):
    """One file: 8-byte little-endian header length, JSON header, data. bf16 stores the upper 16 bits."""
    header, blobs, off = {}, [], 0
    for name, t in tensors.items():
        shape = list(np.shape(t))                      # (a scalar keeps the shape [])
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
