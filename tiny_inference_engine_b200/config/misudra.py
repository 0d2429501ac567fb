"""Misudra: a decoder whose configuration lists its layers in any order. A layer is a mixer behind a norm and,
unless its `mlp` is null, a feed-forward behind a norm, both added to the residual stream. Mixers:

  latent_attention  queries through a normed latent; keys and values from one normed latent per token plus one rotated
                    key part that all heads share (the cache keeps those, nothing per head); a sliding window; a
                    sigmoid gate per head;
  gla               gated linear attention: a matrix state per head that decays with one factor per key channel;
  mamba2            a state-space recurrence with one decay per head behind a short causal convolution.

Feed-forwards: `dense` (a gated unit with the tanh form of GELU, biases on its three products) and `moe` (softmax
router over experts in blocks of consecutive experts, clamped gated experts without biases). The token embedding passes a norm.
`loop` runs layers start .. stop-1 `times` times in a row with the same weights (each pass with a cache and a state of
its own); ahead of every pass, the first too, the stream becomes W_in [stream; embedding output]. config.json:

    {"architecture": "Misudra", "vocab": V, "width": D, "norm": {"eps": e},
     "loop": {"start": a, "stop": b, "times": n},                                   (optional)
     "layers": [{"type": "latent_attention", "mixer": {"heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank", "scale",
                                                        "mask": {"size"}, "rot": {"base", "dims"}}, "mlp": ...},
                {"type": "gla", "mixer": {"heads", "dim", "vdim", "tau"}, "mlp": ...},
                {"type": "mamba2", "mixer": {"heads", "vdim", "state", "groups", "conv", "norm_groups"}, "mlp": ...}],
     with "mlp": {"kind": "dense", "ff"} | {"kind": "moe", "expert": {"ff", "limit"},
                                            "router": {"experts", "top", "groups": {"count", "keep"}}} | null}

Tensors: `embed`, `embed.norm`, `head`, `final.norm`, `loop.in` (with a loop), and per layer i `l<i>.norm1|norm2`,
`l<i>.mix.*`, `l<i>.mlp.*`. The inner size of a gla layer's two-step decay projection (a1/a2) is not in config.json:
it is read from the checkpoint's tensor shapes, or given to `parse_misudra_config`.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from ..errors import LoadError, UnsupportedError
from .registry import Architecture, register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, RunEntry

# Constants that the design fixes.
EXPERT_SLOPE = 1.702       # an expert's unit: y = g * sigmoid(EXPERT_SLOPE * g) * (u + EXPERT_UP_SHIFT)
EXPERT_UP_SHIFT = 1.0
DENSE_ACTIVATION = "gelu_tanh"
DEFAULT_DECAY_RANK = 16    # inner size of a gla layer's a1/a2 when no checkpoint says (random weights)
DEFAULT_MAX_POSITIONS = 1 << 17
MIXERS = ("latent_attention", "gla", "mamba2")


@dataclass
class MisudraConfig:
    vocab: int
    width: int
    eps: float
    layers: list = field(default_factory=list)        # the configuration's own dictionaries, validated
    loop: dict | None = None                          # {"start", "stop", "times"} or None
    decay_ranks: dict = field(default_factory=dict)   # layer index -> inner size of a gla layer's decay projection
    max_positions: int = DEFAULT_MAX_POSITIONS

    def to_dict(self) -> dict:
        d = {"architecture": "Misudra", "layers": self.layers, "norm": {"eps": self.eps}, "vocab": self.vocab, "width": self.width}
        if self.loop is not None:
            d["loop"] = dict(self.loop)
        return d

    def run_layers(self) -> tuple[list[int], list[int]]:
        """(layer index of every run entry in order, the entries at which a pass of the loop starts)."""
        n = len(self.layers)
        if self.loop is None:
            return list(range(n)), []
        a, b, times = self.loop["start"], self.loop["stop"], self.loop["times"]
        order, starts = list(range(a)), []
        for _ in range(times):
            starts.append(len(order))
            order += list(range(a, b))
        return order + list(range(b, n)), starts


def _req(d, key: str, where: str):
    if not isinstance(d, dict) or key not in d:
        raise LoadError(f"config.json: {where} has no '{key}'")
    return d[key]


def _positive_int(v, what: str) -> int:
    if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
        raise LoadError(f"config.json: {what} must be a positive integer, got {v!r}")
    return v


def _check_mixer(kind: str, mx: dict, where: str) -> None:
    w = where + "'s mixer"
    pos = lambda key: _positive_int(_req(mx, key, w), f"{where} mixer.{key}")
    if kind == "latent_attention":
        for key in ("heads", "dim", "vdim", "kv_rank", "q_rank"):
            pos(key)
        rot = _req(mx, "rot_dim", w)
        if not isinstance(rot, int) or isinstance(rot, bool) or rot < 0 or rot % 2:
            raise LoadError(f"config.json: {where} mixer.rot_dim must be an even integer, got {rot!r}")
        _positive_int(_req(_req(mx, "mask", w), "size", where + "'s mask"), f"{where} mask.size")
        _req(mx, "scale", w)
        if rot:
            r = _req(mx, "rot", w)
            _req(r, "base", where + "'s rot")
            if _req(r, "dims", where + "'s rot") != rot:
                raise LoadError(f"config.json: {where}: rot.dims {r['dims']} differs from rot_dim {rot}: the rotated part is rotated whole")
    elif kind == "gla":
        for key in ("heads", "dim", "vdim"):
            pos(key)
        if not float(_req(mx, "tau", w)) > 0:
            raise LoadError(f"config.json: {where} mixer.tau must be positive, got {mx['tau']!r}")
    else:
        for key in ("heads", "vdim", "state", "groups", "conv", "norm_groups"):
            pos(key)
        if mx["heads"] % mx["groups"]:
            raise LoadError(f"config.json: {where}: {mx['heads']} heads are not a multiple of {mx['groups']} groups")
        if (mx["heads"] * mx["vdim"]) % mx["norm_groups"]:
            raise LoadError(f"config.json: {where}: {mx['heads']} heads of {mx['vdim']} do not split into {mx['norm_groups']} equal parts")


def _check_mlp(mlp, where: str) -> None:
    if mlp is None:
        return
    w = where + "'s mlp"
    kind = _req(mlp, "kind", w)
    if kind == "dense":
        _positive_int(_req(mlp, "ff", w), f"{where} mlp.ff")
    elif kind == "moe":
        ex, r = _req(mlp, "expert", w), _req(mlp, "router", w)
        _positive_int(_req(ex, "ff", w + " expert"), f"{where} mlp.expert.ff")
        _req(ex, "limit", w + " expert")
        E = _positive_int(_req(r, "experts", w + " router"), f"{where} mlp.router.experts")
        top = _positive_int(_req(r, "top", w + " router"), f"{where} mlp.router.top")
        g = r.get("groups") or {"count": 1, "keep": 1}
        count = _positive_int(_req(g, "count", w + " router groups"), f"{where} mlp.router.groups.count")
        keep = _positive_int(_req(g, "keep", w + " router groups"), f"{where} mlp.router.groups.keep")
        if E % count or keep > count or top > keep * (E // count):
            raise LoadError(f"config.json: {where}: cannot choose {top} of {E} experts in {count} groups of which {keep} are kept")
    else:
        raise UnsupportedError(f"config.json: {where} has a feed-forward of kind '{kind}' (supported: dense, moe)")


def parse_misudra_config(j: dict, decay_ranks: dict | None = None) -> MisudraConfig:
    layers = _req(j, "layers", "the configuration")
    if not isinstance(layers, list) or not layers:
        raise LoadError("config.json: 'layers' must be a non-empty list")
    for i, layer in enumerate(layers):
        where = f"layer {i}"
        kind = _req(layer, "type", where)
        if kind not in MIXERS:
            raise UnsupportedError(f"config.json: {where} has type '{kind}' (supported: {', '.join(MIXERS)})")
        _check_mixer(kind, _req(layer, "mixer", where), where)
        _check_mlp(layer.get("mlp"), where)
    loop = j.get("loop")
    if loop is not None:
        a, b, times = (_req(loop, k, "'loop'") for k in ("start", "stop", "times"))
        if not all(isinstance(v, int) and not isinstance(v, bool) for v in (a, b, times)) or not 0 <= a < b <= len(layers) or times < 1:
            raise LoadError(f"config.json: loop start={a!r} stop={b!r} times={times!r} does not name layers of this model")
        loop = {"start": a, "stop": b, "times": times}
    return MisudraConfig(vocab=_positive_int(_req(j, "vocab", "the configuration"), "vocab"),
                         width=_positive_int(_req(j, "width", "the configuration"), "width"),
                         eps=float(_req(_req(j, "norm", "the configuration"), "eps", "'norm'")), layers=layers, loop=loop,
                         decay_ranks=dict(decay_ranks or {}), max_positions=int(j.get("max_positions", DEFAULT_MAX_POSITIONS)))


def decay_ranks_from_shapes(shapes: dict) -> dict:
    """layer index -> rows of `l<i>.mix.a1` from a checkpoint's tensor shapes."""
    out = {}
    for name, shape in shapes.items():
        parts = name.split(".")
        if len(parts) == 3 and parts[1] == "mix" and parts[2] == "a1" and parts[0][:1] == "l" and parts[0][1:].isdigit():
            out[int(parts[0][1:])] = int(shape[0])
    return out


def misudra_spec(c: MisudraConfig) -> ModelSpec:
    D = c.width

    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"name": name, "size": D, "eps": c.eps})

    layers = []
    for i, layer in enumerate(c.layers):
        p, mx, kind = f"l{i}.", layer["mixer"], layer["type"]
        if kind == "latent_attention":
            rot = mx["rot_dim"]
            mixer = PartSpec("latent_attention", {
                "prefix": p + "mix.", "hidden_size": D, "num_heads": mx["heads"], "head_dim": mx["dim"], "rot_dim": rot,
                "value_dim": mx["vdim"], "kv_rank": mx["kv_rank"], "q_rank": mx["q_rank"], "window": mx["mask"]["size"],
                "scale": float(mx["scale"]), "eps": c.eps, "output_gate": True,
                "position": PartSpec("rope", {"theta": float(mx["rot"]["base"]), "head_dim": rot, "rotary_dim": rot}) if rot else None})
        elif kind == "gla":
            rank = c.decay_ranks.get(i, c.decay_ranks.get(str(i), DEFAULT_DECAY_RANK))
            mixer = PartSpec("gated_linear_attention", {
                "prefix": p + "mix.", "hidden_size": D, "num_heads": mx["heads"], "head_dim": mx["dim"], "value_dim": mx["vdim"],
                "tau": float(mx["tau"]), "decay_rank": int(rank), "eps": c.eps})
        else:
            mixer = PartSpec("state_space_dual", {
                "prefix": p + "mix.", "hidden_size": D, "num_heads": mx["heads"], "num_groups": mx["groups"],
                "value_dim": mx["vdim"], "state_size": mx["state"], "conv_taps": mx["conv"], "norm_groups": mx["norm_groups"],
                "eps": c.eps})
        mlp = layer.get("mlp")
        if mlp is None:
            ffn = None
        elif mlp["kind"] == "dense":
            ffn = PartSpec("biased_glu", {"prefix": p + "mlp.", "hidden_size": D, "intermediate_size": mlp["ff"],
                                          "activation": DENSE_ACTIVATION})
        else:
            r = mlp["router"]
            g = r.get("groups") or {"count": 1, "keep": 1}
            ffn = PartSpec("routed_experts", {
                "prefix": p + "mlp.", "hidden_size": D, "intermediate_size": mlp["expert"]["ff"], "num_experts": r["experts"],
                "top": r["top"], "group_count": g["count"], "group_keep": g["keep"], "limit": float(mlp["expert"]["limit"]),
                "slope": EXPERT_SLOPE, "up_shift": EXPERT_UP_SHIFT})
        layers.append(LayerSpec(prefix=p, block=PartSpec("prenorm", {}), mixer=mixer, mixer_norm=norm(p + "norm1"), ffn=ffn,
                                ffn_norm=None if ffn is None else norm(p + "norm2")))
    order, starts = c.run_layers()
    mix_in = PartSpec("concat_projection", {"name": "loop.in", "hidden_size": D}) if starts else None
    run_order = tuple(RunEntry(l, before=mix_in if i in starts else None) for i, l in enumerate(order))
    return ModelSpec(architecture="Misudra", hidden_size=D, vocab_size=c.vocab, max_positions=c.max_positions,
                     embedding=PartSpec("normed_token_embedding", {"name": "embed", "vocab_size": c.vocab, "hidden_size": D,
                                                                   "norm": norm("embed.norm")}),
                     layers=tuple(layers), run_order=run_order, final_norm=norm("final.norm"),
                     head=PartSpec("lm_head", {"name": "head", "tied": False, "vocab_size": c.vocab, "hidden_size": D}))


register_architecture(Architecture(name="Misudra", parse_config=parse_misudra_config, build_spec=misudra_spec,
                                   model_types=("misudra",), shapes_to_config=decay_ranks_from_shapes), replace=True)
