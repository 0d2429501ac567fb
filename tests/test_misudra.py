"""Misudra without a GPU: configuration, model description, run order, tensor names and shapes, cache and state needs,
and the plain implementation's own properties (what a window, a recurrence and the routing must and must not do)."""
import copy

import numpy as np
import pytest
import torch

import plain_misudra as plain
from tiny_inference_engine_b200.config import load_config, misudra_spec, parse_misudra_config
from tiny_inference_engine_b200.errors import LoadError, UnsupportedError
from tiny_inference_engine_b200.parts.model import Model, expected_tensors
from tiny_inference_engine_b200.weights.loader import SafetensorsSource, bind_check

L, G, M, moe = plain.latent_layer, plain.gla_layer, plain.mamba2_layer, plain.moe
CFG = plain.make_config([M(heads=6, vdim=10, state=12, groups=3, conv=2, norm_groups=3),
                         L(heads=3, dim=12, rot_dim=6, vdim=10, kv_rank=20, q_rank=14, window=7, mlp=moe(ff=20, experts=6, top=3, groups=3, keep=2)),
                         G(heads=3, dim=20, vdim=12, tau=3.0, mlp=None), L(window=5, mlp=plain.dense(50))],
                        vocab=97, width=72, eps=1e-5, loop=(1, 3, 2))


def test_config_json_picks_the_architecture_and_every_size_comes_from_it(tmp_path):
    w = plain.random_weights(CFG, 1, decay_rank=3)
    plain.write_model_dir(tmp_path, CFG, w)
    arch, cfg, spec = load_config(tmp_path)
    assert arch.name == "Misudra" and spec.architecture == "Misudra"
    assert (spec.hidden_size, spec.vocab_size, len(spec.layers)) == (72, 97, 4)
    assert cfg.decay_ranks == {2: 3}                      # read from the checkpoint's shapes: config.json has no key for it
    model = Model(spec, torch.float32)
    needs = model.needs()
    assert {n: tuple(t.shape) for n, t in needs.items()} == {n: tuple(s) for n, s in plain.tensor_shapes(CFG, 3).items()}
    bind_check(needs, SafetensorsSource(tmp_path), what="Misudra")
    assert [l.mixer.kind for l in spec.layers] == ["state_space_dual", "latent_attention", "gated_linear_attention", "latent_attention"]
    assert [None if l.ffn is None else l.ffn.kind for l in spec.layers] == ["biased_glu", "routed_experts", None, "biased_glu"]
    # layers 1 and 2 run twice; each pass starts with the stream input, and every entry has a cache or state of its own
    assert [(e.layer, e.before is not None) for e in spec.run_order] == [(0, False), (1, True), (2, False), (1, True), (2, False), (3, False)]
    assert spec.run_order[1].before is spec.run_order[3].before and len(model.stream_inputs) == 2
    cache = model.cache_needs()
    assert [c is None for c in cache] == [True, False, True, False, True, False]
    assert (cache[1].kind, cache[1].kv_heads, cache[1].head_dim, cache[1].window, cache[1].value_dim) == ("window", 1, 26, 7, -1)
    assert cache[5].window == 5 and cache[5].head_dim == 40 + 8
    state = model.state_needs()
    assert state[1] is None and state[0].shape == (6 * 12 * 10 + (2 - 1) * (60 + 2 * 36),) and state[0].dtype == torch.float32
    assert state[2].shape == state[4].shape == (3 * 20 * 12,)


def test_a_keys_only_cache_group_per_shape_and_planes_per_run_entry():
    from tiny_inference_engine_b200.cache.manager import CacheManager
    model = Model(misudra_spec(parse_misudra_config(CFG)), torch.float32)
    cm = CacheManager(model.cache_needs(), 8, num_pages=10, dtype=torch.float32)
    assert [(g.kind, g.kv_heads, g.head_dim, g.window, g.value_dim, g.entries) for g in cm.groups] == \
        [("window", 1, 26, 7, -1, (1, 3)), ("window", 1, 48, 5, -1, (5,))]
    assert cm.bytes_per_page == (2 * 26 + 48) * 8 * 4      # keys only: a value lives inside its key


def test_without_a_loop_layers_run_once_and_nothing_is_mixed_in():
    cfg = plain.make_config([G(), M(mlp=None)])
    spec = misudra_spec(parse_misudra_config(cfg))
    assert [(e.layer, e.before) for e in spec.run_order] == [(0, None), (1, None)]
    assert "loop.in" not in expected_tensors(spec)
    looped = misudra_spec(parse_misudra_config(plain.make_config([G(), M(mlp=None)], loop=(0, 2, 3))))
    assert [e.layer for e in looped.run_order] == [0, 1, 0, 1, 0, 1] and [e.before is not None for e in looped.run_order] == [True, False] * 3
    assert tuple(expected_tensors(looped)["loop.in"].shape) == (64, 128)


def test_what_the_configuration_rejects():
    def broken(change):
        c = copy.deepcopy(CFG)
        change(c)
        return c
    with pytest.raises(UnsupportedError, match="type 'conv'"):
        parse_misudra_config(broken(lambda c: c["layers"][0].update(type="conv")))
    with pytest.raises(UnsupportedError, match="kind 'routed'"):
        parse_misudra_config(broken(lambda c: c["layers"][1]["mlp"].update(kind="routed")))
    with pytest.raises(LoadError, match="no 'norm'"):
        parse_misudra_config(broken(lambda c: c.pop("norm")))
    with pytest.raises(LoadError, match="not a multiple"):
        parse_misudra_config(broken(lambda c: c["layers"][0]["mixer"].update(groups=4)))
    with pytest.raises(LoadError, match="rot.dims"):
        parse_misudra_config(broken(lambda c: c["layers"][1]["mixer"]["rot"].update(dims=4)))
    with pytest.raises(LoadError, match="cannot choose"):
        parse_misudra_config(broken(lambda c: c["layers"][1]["mlp"]["router"].update(top=5)))
    with pytest.raises(LoadError, match="mask"):
        parse_misudra_config(broken(lambda c: c["layers"][1]["mixer"].pop("mask")))
    with pytest.raises(LoadError, match="loop"):
        parse_misudra_config(broken(lambda c: c["loop"].update(stop=9)))
    with pytest.raises(LoadError, match="equal parts"):
        parse_misudra_config(broken(lambda c: c["layers"][0]["mixer"].update(norm_groups=7)))


def test_random_weights_need_no_checkpoint():
    names = expected_tensors(misudra_spec(parse_misudra_config(CFG)))
    assert names["l2.mix.a1"].shape[0] == names["l2.mix.a2"].shape[1] == 16      # the default inner size


def test_plain_window_and_recurrences_see_what_they_should():
    toks = np.random.default_rng(0).integers(0, 50, 30).tolist()
    moved = list(toks)
    moved[10] = (toks[10] + 1) % 50
    cfg = plain.make_config([L(window=6, mlp=None)], vocab=50, width=32)
    w = plain.random_weights(cfg, 2)
    base, other = plain.forward(w, cfg, toks), plain.forward(w, cfg, moved)
    assert np.allclose(other[:10], base[:10]) and np.allclose(other[16:], base[16:])     # rows 10..15 see token 10
    assert all(np.abs(other[i] - base[i]).max() > 1e-6 for i in range(10, 16))
    for layer in (G(mlp=None), M(conv=3, mlp=None)):
        cfg = plain.make_config([layer], vocab=50, width=32)
        w = plain.random_weights(cfg, 2)
        base, other = plain.forward(w, cfg, toks), plain.forward(w, cfg, moved)
        assert np.allclose(other[:10], base[:10]) and all(np.abs(other[i] - base[i]).max() > 1e-9 for i in range(10, 30))
        assert np.allclose(plain.forward(w, cfg, toks[:12]), base[:12])                  # a prefix does not depend on what follows


def test_plain_routing_keeps_to_the_best_groups():
    r = np.random.default_rng(3)
    for _ in range(50):
        s = r.dirichlet(np.ones(12))
        ids, weights = plain.route(s, top=3, group_count=4, group_keep=2)
        best = np.argsort(-s.reshape(4, 3).max(axis=1))[:2]
        assert all(i // 3 in best for i in ids) and abs(weights.sum() - 1) < 1e-9 and len(set(ids.tolist())) == 3
        allowed = sorted((s[i] for i in range(12) if i // 3 in best), reverse=True)
        assert np.allclose(sorted(s[ids], reverse=True), allowed[:3])
    ids, _ = plain.route(np.array([0.4, 0.1, 0.3, 0.2]), top=2, group_count=1, group_keep=1)
    assert ids.tolist() == [0, 2]                           # one group: the plain top-k


def test_a_random_model_folder_from_a_configuration(tmp_path):
    """`tie make-random` writes config.json and weights of every tensor the description names; the folder loads back."""
    import json
    from tiny_inference_engine_b200.cli.main import main
    (tmp_path / "config.json").write_text(json.dumps(CFG))
    assert main(["make-random", "-o", str(tmp_path / "m"), "--config", str(tmp_path / "config.json"), "--seed", "3"]) == 0
    arch, cfg, spec = load_config(tmp_path / "m")
    assert arch.name == "Misudra" and cfg.decay_ranks == {2: 16}
    bind_check(Model(spec, torch.float32).needs(), SafetensorsSource(tmp_path / "m"), what="Misudra")
