"""Dugazen without a GPU: configuration, model description, tensor names and shapes, and the plain
implementation's own properties (what a window and a recurrence must and must not see)."""
import numpy as np
import pytest
import torch

import plain_dugazen as plain
from tiny_inference_engine_b200.config import load_config, parse_dugazen_config, dugazen_spec
from tiny_inference_engine_b200.errors import LoadError, UnsupportedError
from tiny_inference_engine_b200.parts.model import Model, expected_tensors
from tiny_inference_engine_b200.weights.loader import SafetensorsSource, bind_check

A, D = plain.attention_layer, plain.delta_layer
CFG = plain.make_config([D(heads=3, kv_heads=1, dim=40, vdim=20, conv=2), A(), A(v_mix=False, ff=None), D(ff=80), A(window=5)],
                        vocab=97, width=72, eps=1e-5, residual_mult=1.3, logit_scale=0.5)


def test_config_json_picks_the_architecture_and_every_size_comes_from_it(tmp_path):
    w = plain.random_weights(CFG, 1, low_rank=3, gate_rank=7)
    plain.write_model_dir(tmp_path, CFG, w)
    arch, cfg, spec = load_config(tmp_path)
    assert arch.name == "Dugazen" and spec.architecture == "Dugazen"
    assert (spec.hidden_size, spec.vocab_size, len(spec.layers)) == (72, 97, 5)
    assert cfg.ranks == {0: (3, 7), 3: (3, 7)}            # read from the checkpoint's shapes: config.json has no key for them
    model = Model(spec, torch.float32)
    needs = model.needs()
    required = {n: tuple(t.shape) for n, t in needs.items() if not t.optional}
    assert required == {n: tuple(s) for n, s in plain.tensor_shapes(CFG, 3, 7).items() if n != "l1.mix.vmix"}
    assert needs["l1.mix.vmix"].optional and needs["l2.mix.vmix"].optional and not needs["l4.mix.vmix"].optional
    bind_check(needs, SafetensorsSource(tmp_path), what="Dugazen")
    kinds = [l.mixer.kind for l in spec.layers]
    assert kinds == ["channel_gated_delta", "gated_window_attention", "gated_window_attention", "channel_gated_delta",
                     "gated_window_attention"]
    # the first blending layer is the source, later ones blend, a layer without v_mix does neither
    assert [l.mixer.params.get("value_mix") for l in spec.layers if l.mixer.kind == "gated_window_attention"] == ["source", "none", "blend"]
    assert [l.ffn is None for l in spec.layers] == [True, False, True, False, False]
    assert spec.layers[1].block.params["residual_mult"] == 1.3 and spec.head.params["logit_scale"] == 0.5
    cache = model.cache_needs()
    assert cache[0] is None and cache[3] is None
    assert (cache[1].kind, cache[1].kv_heads, cache[1].head_dim, cache[1].window, cache[1].value_dim) == ("window", 2, 32, 24, 16)
    assert cache[4].window == 5
    state = model.state_needs()
    assert state[1] is None and state[0].shape == (3 * 40 * 20 + (2 - 1) * (2 * 40 + 60),) and state[0].dtype == torch.float32
    assert state[3].shape == (4 * 16 * 24 + (3 - 1) * (2 * 32 + 96),)


def test_cache_groups_take_value_heads_of_their_own_size():
    from tiny_inference_engine_b200.cache.manager import CacheManager
    model = Model(dugazen_spec(parse_dugazen_config(CFG)), torch.float32)
    cm = CacheManager(model.cache_needs(), 8, num_pages=10)
    assert [(g.kind, g.kv_heads, g.head_dim, g.window, g.value_dim, g.entries) for g in cm.groups] == \
        [("window", 2, 32, 24, 16, (1, 2)), ("window", 2, 32, 5, 16, (4,))]


def test_what_the_configuration_rejects():
    def broken(change):
        import copy
        c = copy.deepcopy(CFG)
        change(c)
        return c
    with pytest.raises(UnsupportedError, match="type 'conv'"):
        parse_dugazen_config(broken(lambda c: c["layers"][0].update(type="conv")))
    with pytest.raises(UnsupportedError, match="kind 'routed'"):
        parse_dugazen_config(broken(lambda c: c["layers"][1]["mlp"].update(kind="routed")))
    with pytest.raises(LoadError, match="no 'residual_mult'"):
        parse_dugazen_config(broken(lambda c: c.pop("residual_mult")))
    with pytest.raises(LoadError, match="not a multiple"):
        parse_dugazen_config(broken(lambda c: c["layers"][1]["mixer"].update(heads=3)))
    with pytest.raises(LoadError, match="rot.dims"):
        parse_dugazen_config(broken(lambda c: c["layers"][1]["mixer"]["rot"].update(dims=34)))
    with pytest.raises(LoadError, match="value heads of one size"):
        parse_dugazen_config(broken(lambda c: c["layers"][4]["mixer"].update(vdim=8)))
    with pytest.raises(LoadError, match="mask"):
        parse_dugazen_config(broken(lambda c: c["layers"][1]["mixer"].pop("mask")))


def test_random_weights_need_no_checkpoint():
    spec = dugazen_spec(parse_dugazen_config(CFG))
    names = expected_tensors(spec)
    assert names["l0.mix.a1"].shape[0] == names["l0.mix.g2"].shape[1] == 16      # the default inner size


def test_plain_window_and_recurrence_see_what_they_should():
    cfg = plain.make_config([A(window=6, ff=None, v_mix=False)], vocab=50, width=32)
    w = plain.random_weights(cfg, 2)
    toks = np.random.default_rng(0).integers(0, 50, 30).tolist()
    base = plain.forward(w, cfg, toks)
    moved = list(toks)
    moved[10] = (toks[10] + 1) % 50
    other = plain.forward(w, cfg, moved)
    assert np.allclose(other[:10], base[:10]) and np.allclose(other[16:], base[16:])     # rows 10..15 see token 10
    assert all(np.abs(other[i] - base[i]).max() > 1e-6 for i in range(10, 16))
    cfg = plain.make_config([D(conv=3)], vocab=50, width=32)
    w = plain.random_weights(cfg, 2)
    base, other = plain.forward(w, cfg, toks), plain.forward(w, cfg, moved)
    assert np.allclose(other[:10], base[:10]) and all(np.abs(other[i] - base[i]).max() > 1e-9 for i in range(10, 30))
    # a prefix's logits do not depend on what follows
    assert np.allclose(plain.forward(w, cfg, toks[:12]), base[:12])
