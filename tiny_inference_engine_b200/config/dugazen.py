"""Dugazen: a decoder that mixes, in any order its configuration lists, two kinds of layer:

  attention      sliding-window grouped-query attention with biases, one RMS norm over the whole q (and k)
                 projection, a rotation of the first `rot.dims` dimensions of each head, keys of `dim` and values
                 of `vdim`, values blended with those of the first blending layer, a sigmoid gate on the heads;
  channel_delta  a gated delta rule with one decay per head and key channel, behind short causal convolutions.

Every sublayer sits between two norms whose weights are stored around zero, and what it adds to the residual
stream is multiplied by `residual_mult`; a layer may have no feed-forward (`mlp` null). The logits are multiplied
by `logit_scale`. config.json:

    {"architecture": "Dugazen", "vocab": V, "width": D, "norm": {"eps": e}, "residual_mult": m, "logit_scale": c,
     "layers": [{"type": "attention", "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "mask": {"size"},
                                                "rot": {"base", "dims"}, "v_mix"},
                 "mlp": {"kind": "dense", "ff", "limit"} | null},
                {"type": "channel_delta", "mixer": {"heads", "kv_heads", "dim", "vdim", "conv"}, "mlp": ...}, ...]}

Tensors: `embed`, `head`, `final.norm`, and per layer i `l<i>.norm1|norm1b|norm2|norm2b`, `l<i>.mix.*`,
`l<i>.mlp.gate|up|down`. The inner sizes of a channel_delta layer's two-step projections (a1/a2, g1/g2) are not in
config.json: they are read from the checkpoint's tensor shapes (`ranks`), or given to `parse_dugazen_config`.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from ..errors import LoadError, UnsupportedError
from .registry import Architecture, register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, RunEntry

# Constants that the design fixes.
GLU_SLOPE = 1.702          # y = g * sigmoid(GLU_SLOPE * g) * (u + GLU_UP_SHIFT)
GLU_UP_SHIFT = 1.0
UNIT_EPS = 1e-6            # inside the root of the delta rule's unit norms
DEFAULT_RANK = 16          # inner size of a1/a2 and g1/g2 when no checkpoint says (random weights)
DEFAULT_MAX_POSITIONS = 1 << 17


@dataclass
class DugazenConfig:
    vocab: int
    width: int
    eps: float
    residual_mult: float
    logit_scale: float
    layers: list = field(default_factory=list)        # the configuration's own dictionaries, validated
    ranks: dict = field(default_factory=dict)          # layer index -> (decay rank, gate rank)
    max_positions: int = DEFAULT_MAX_POSITIONS

    def to_dict(self) -> dict:
        return {"architecture": "Dugazen", "layers": self.layers, "logit_scale": self.logit_scale,
                "norm": {"eps": self.eps}, "residual_mult": self.residual_mult, "vocab": self.vocab, "width": self.width}


def _req(d: dict, key: str, where: str):
    if not isinstance(d, dict) or key not in d:
        raise LoadError(f"config.json: {where} has no '{key}'")
    return d[key]


def _positive_int(v, what: str) -> int:
    if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
        raise LoadError(f"config.json: {what} must be a positive integer, got {v!r}")
    return v


def parse_dugazen_config(j: dict, ranks: dict | None = None) -> DugazenConfig:
    layers = _req(j, "layers", "the configuration")
    if not isinstance(layers, list) or not layers:
        raise LoadError("config.json: 'layers' must be a non-empty list")
    for i, layer in enumerate(layers):
        where = f"layer {i}"
        kind = _req(layer, "type", where)
        mx = _req(layer, "mixer", where)
        for key in ("heads", "kv_heads", "dim", "vdim"):
            _positive_int(_req(mx, key, where + "'s mixer"), f"{where} mixer.{key}")
        if mx["heads"] % mx["kv_heads"]:
            raise LoadError(f"config.json: {where}: {mx['heads']} heads are not a multiple of {mx['kv_heads']} kv heads")
        if kind == "attention":
            _positive_int(_req(_req(mx, "mask", where), "size", where + "'s mask"), f"{where} mask.size")
            rot = _req(mx, "rot", where)
            dims = _positive_int(_req(rot, "dims", where + "'s rot"), f"{where} rot.dims")
            if dims % 2 or dims > mx["dim"]:
                raise LoadError(f"config.json: {where}: rot.dims {dims} must be even and at most dim {mx['dim']}")
            _req(rot, "base", where + "'s rot")
            _req(mx, "scale", where + "'s mixer")
        elif kind == "channel_delta":
            _positive_int(_req(mx, "conv", where + "'s mixer"), f"{where} mixer.conv")
        else:
            raise UnsupportedError(f"config.json: {where} has type '{kind}' (supported: attention, channel_delta)")
        mlp = layer.get("mlp")
        if mlp is not None:
            if _req(mlp, "kind", where + "'s mlp") != "dense":
                raise UnsupportedError(f"config.json: {where} has a feed-forward of kind '{mlp['kind']}' (supported: dense)")
            _positive_int(_req(mlp, "ff", where + "'s mlp"), f"{where} mlp.ff")
            _req(mlp, "limit", where + "'s mlp")
    mixing = [l["mixer"] for l in layers if l["type"] == "attention" and l["mixer"].get("v_mix")]
    if len({(m["kv_heads"], m["vdim"]) for m in mixing}) > 1:
        raise LoadError("config.json: layers that blend values (v_mix) must have value heads of one size")
    return DugazenConfig(vocab=_positive_int(_req(j, "vocab", "the configuration"), "vocab"),
                         width=_positive_int(_req(j, "width", "the configuration"), "width"),
                         eps=float(_req(_req(j, "norm", "the configuration"), "eps", "'norm'")),
                         residual_mult=float(_req(j, "residual_mult", "the configuration")),
                         logit_scale=float(_req(j, "logit_scale", "the configuration")), layers=layers,
                         ranks=dict(ranks or {}),
                         max_positions=int(j.get("max_positions", DEFAULT_MAX_POSITIONS)))


def ranks_from_shapes(shapes: dict) -> dict:
    """layer index -> (rows of `l<i>.mix.a1`, rows of `l<i>.mix.g1`) from a checkpoint's tensor shapes."""
    out = {}
    for name, shape in shapes.items():
        parts = name.split(".")
        if len(parts) == 3 and parts[1] == "mix" and parts[2] == "a1" and parts[0][:1] == "l" and parts[0][1:].isdigit():
            g1 = shapes.get(f"{parts[0]}.mix.g1")
            if g1 is not None:
                out[int(parts[0][1:])] = (int(shape[0]), int(g1[0]))
    return out


def dugazen_spec(c: DugazenConfig) -> ModelSpec:
    D = c.width

    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm_one_plus", {"name": name, "size": D, "eps": c.eps})

    layers, mixing_seen = [], False
    for i, layer in enumerate(c.layers):
        p, mx = f"l{i}.", layer["mixer"]
        if layer["type"] == "attention":
            mix = "none"
            if mx.get("v_mix"):
                mix, mixing_seen = ("blend" if mixing_seen else "source"), True
            mixer = PartSpec("gated_window_attention", {
                "prefix": p + "mix.", "hidden_size": D, "num_heads": mx["heads"], "num_kv_heads": mx["kv_heads"],
                "head_dim": mx["dim"], "value_dim": mx["vdim"], "window": mx["mask"]["size"], "scale": float(mx["scale"]),
                "eps": c.eps, "bias": True, "span_norm": True, "output_gate": True, "value_mix": mix,
                "position": PartSpec("rope", {"theta": float(mx["rot"]["base"]), "head_dim": mx["dim"],
                                              "rotary_dim": mx["rot"]["dims"]})})
        else:
            decay_rank, gate_rank = c.ranks.get(i, c.ranks.get(str(i), (DEFAULT_RANK, DEFAULT_RANK)))
            mixer = PartSpec("channel_gated_delta", {
                "prefix": p + "mix.", "hidden_size": D, "num_heads": mx["heads"], "num_kv_heads": mx["kv_heads"],
                "head_dim": mx["dim"], "value_dim": mx["vdim"], "conv_taps": mx["conv"], "unit_eps": UNIT_EPS,
                "eps": c.eps, "decay_rank": decay_rank, "gate_rank": gate_rank})
        mlp = layer.get("mlp")
        ffn = None if mlp is None else PartSpec("clamped_glu", {
            "prefix": p + "mlp.", "hidden_size": D, "intermediate_size": mlp["ff"], "limit": float(mlp["limit"]),
            "slope": GLU_SLOPE, "up_shift": GLU_UP_SHIFT})
        layers.append(LayerSpec(prefix=p, block=PartSpec("sandwich_norm", {"residual_mult": c.residual_mult}), mixer=mixer,
                                mixer_norm=norm(p + "norm1"), mixer_post_norm=norm(p + "norm1b"), ffn=ffn,
                                ffn_norm=None if ffn is None else norm(p + "norm2"),
                                ffn_post_norm=None if ffn is None else norm(p + "norm2b")))
    return ModelSpec(architecture="Dugazen", hidden_size=D, vocab_size=c.vocab, max_positions=c.max_positions,
                     embedding=PartSpec("token_embedding", {"name": "embed", "vocab_size": c.vocab, "hidden_size": D}),
                     layers=tuple(layers), run_order=tuple(RunEntry(l) for l in range(len(layers))),
                     final_norm=norm("final.norm"),
                     head=PartSpec("lm_head", {"name": "head", "tied": False, "vocab_size": c.vocab, "hidden_size": D,
                                               "logit_scale": c.logit_scale}))


register_architecture(Architecture(name="Dugazen", parse_config=parse_dugazen_config, build_spec=dugazen_spec,
                                   model_types=("dugazen",), shapes_to_config=ranks_from_shapes), replace=True)
