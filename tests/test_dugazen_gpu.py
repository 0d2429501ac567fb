"""Dugazen through the engine against the plain implementation (tests/plain_dugazen.py): each mechanism alone,
prompts whole and token by token, portions down to two tokens, mixed batches, pages and state slots that are
used again, keys at a window's edge and far back in the recurrence, the first tokens of a sequence, long
decoding, sizes of several kinds, greedy generation through the engine's own entry point and scheduler."""
import numpy as np
import pytest
import torch

import plain_dugazen as plain
from conftest import assert_logits_close, rel_err

pytestmark = pytest.mark.gpu

A, D = plain.attention_layer, plain.delta_layer

# Configurations. None is a model anyone serves: sizes are chosen to differ from one another in every place where
# two sizes could be mistaken for each other (heads and kv heads, key and value sizes, the two inner ranks).
MIXED = plain.make_config([A(), D(), A(ff=None), D(ff=80), A(heads=4, kv_heads=2, dim=32, vdim=16, window=24)])
ODD = plain.make_config([D(heads=3, kv_heads=1, dim=40, vdim=20, conv=2), D(heads=2, kv_heads=2, dim=24, vdim=36, conv=1, ff=56),
                         A(heads=6, kv_heads=3, dim=24, vdim=40, window=7, rot_dims=24, v_mix=False, ff=None),
                         A(heads=2, kv_heads=2, dim=20, vdim=66, window=50, rot_dims=8, scale=0.31, limit=1.5),
                         A(heads=4, kv_heads=2, dim=16, vdim=66, window=3, rot_dims=2, v_mix=True, ff=40)],
                        vocab=97, width=72, eps=1e-5, residual_mult=1.3, logit_scale=0.5)
ONES = plain.make_config([A(heads=1, kv_heads=1, dim=8, vdim=8, window=1, rot_dims=8), D(heads=1, kv_heads=1, dim=8, vdim=8, conv=5),
                          A(heads=1, kv_heads=1, dim=8, vdim=8, window=1000, rot_dims=4)], vocab=33, width=16,
                         residual_mult=1.0, logit_scale=1.0)
# keys and values of one size that the tensor-core attention kernels take (bfloat16 runs there)
SQUARE = plain.make_config([A(heads=4, kv_heads=2, dim=64, vdim=64, window=40, rot_dims=32), D(),
                            A(heads=4, kv_heads=2, dim=64, vdim=64, window=300, rot_dims=64, ff=None)], width=64)
# value heads smaller than key heads of a size the tensor-core kernels take (bfloat16 keeps them padded with zeros)
PADDED = plain.make_config([A(heads=4, kv_heads=2, dim=64, vdim=24, window=40, rot_dims=32), D(),
                            A(heads=8, kv_heads=1, dim=128, vdim=64, window=70, rot_dims=64, v_mix=False, ff=None),
                            A(heads=4, kv_heads=2, dim=64, vdim=24, window=300, rot_dims=64, ff=None)], width=64)
CONFIGS = {"padded": (PADDED, dict(low_rank=8, gate_rank=8), 16), "mixed": (MIXED, dict(low_rank=8, gate_rank=5), 16), "odd": (ODD, dict(low_rank=3, gate_rank=16), 8),
           "ones": (ONES, dict(low_rank=1, gate_rank=2), 4), "square": (SQUARE, dict(low_rank=8, gate_rank=8), 16)}
class Want:
    """The plain implementation's logits, and how far the same implementation moves when its activations are
    rounded to bfloat16 (largest difference of a row relative to its largest logit, worst row)."""

    def __init__(self, rows, noise):
        self.rows, self.noise = np.asarray(rows), noise

    def __getitem__(self, idx):
        return Want(self.rows[idx], self.noise)


def reference(w, cfg, toks):
    exact = plain.forward(w, cfg, toks)
    with plain.bfloat16_activations():
        rounded = plain.forward(w, cfg, toks)
    return Want(exact, rel_err(rounded, exact))


def close(got, want, dtype, what):
    """float32: 1e-4 of the row's largest logit and the same argmax. bfloat16: four times the noise of 16-bit
    activations on this very model and prompt, and at least 2e-2 (the engine rounds at other places than the
    plain implementation does, so the two differ by about that noise, not by less)."""
    if dtype == "float32":
        assert_logits_close(got, want.rows, dtype, what)
    else:
        err, tol = rel_err(got, want.rows), max(2e-2, 4.0 * want.noise)
        assert err <= tol, f"{what}: relative error {err:.3e} above {tol:.1e} (bfloat16; noise of rounding {want.noise:.1e})"


class Harness:
    """A model folder, the engine's model, cache, state slots and step function; `step` takes
    [(request id, tokens, wanted places)] like the trace runner and returns {(id, position): logits}."""

    def __init__(self, tmp, cfg, weights, dtype, page=16, pages=64, slots=4, max_tokens=512):
        from tiny_inference_engine_b200 import StepRunner, load_model, make_cache
        plain.write_model_dir(tmp, cfg, weights)
        self.model = load_model(tmp, dtype)
        self.cache, self.states = make_cache(self.model, page_size=page, num_pages=pages, max_requests=slots)
        self.runner = StepRunner(self.model, self.cache, max_tokens=max_tokens, max_seqs=8, max_logit_rows=max_tokens,
                                 states=self.states)
        self.live = {}

    def step(self, entries, end=()):
        from tiny_inference_engine_b200 import StepEntry
        batch, keys = [], []
        for rid, tokens, want in entries:
            if rid not in self.live:
                self.live[rid] = [self.cache.new_request(), 0]
            req, have = self.live[rid]
            assert self.cache.reserve(req, have + len(tokens)), "pool too small for the test"
            batch.append(StepEntry(req, list(tokens), have, list(want)))
            keys += [(rid, have + w) for w in want]
        logits = self.runner.run(batch)
        for (rid, tokens, _), e in zip(entries, batch):
            self.live[rid][1] += len(tokens)
            self.cache.advance_window(e.cache, self.live[rid][1])
        out = {}
        if logits is not None:
            host = logits.float().cpu().numpy()
            out = {k: host[i] for i, k in enumerate(keys)}
        torch.cuda.synchronize()
        self.runner.check()
        for rid in end:
            self.cache.release(self.live.pop(rid)[0])
        return out

    def whole(self, rid, tokens):
        got = self.step([(rid, tokens, range(len(tokens)))], end=[rid])
        return np.stack([got[(rid, i)] for i in range(len(tokens))])

    def in_portions(self, rid, tokens, sizes):
        rows, at, i = {}, 0, 0
        while at < len(tokens):
            n = min(sizes[i % len(sizes)], len(tokens) - at)
            rows.update(self.step([(rid, tokens[at:at + n], range(n))]))
            at, i = at + n, i + 1
        self.cache.release(self.live.pop(rid)[0])
        return np.stack([rows[(rid, j)] for j in range(len(tokens))])


def tokens_of(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


@pytest.fixture(scope="module")
def truth():
    """Plain logits, computed once per (configuration, seed, length)."""
    memo = {}

    def get(name, toks):
        cfg, ranks, _ = CONFIGS[name]
        key = (name, tuple(toks))
        if key not in memo:
            memo[key] = reference(plain.random_weights(cfg, 5, **ranks), cfg, toks)
        return memo[key]
    return get


# ---------------------------------------------------------------------------------------------- each mechanism alone

SINGLE = {
    "attention": plain.make_config([A(ff=None, v_mix=False)]),
    "attention_full_rotation_no_window_in_reach": plain.make_config([A(ff=None, rot_dims=32, window=500, v_mix=False)]),
    "attention_heads_of_one_size": plain.make_config([A(heads=4, kv_heads=1, dim=128, vdim=128, window=30, rot_dims=64, ff=None, v_mix=False)]),
    "value_blend": plain.make_config([A(ff=None), A(ff=None, v_mix=False), A(ff=None)]),
    "delta": plain.make_config([D()]),
    "delta_one_tap_heads_alike": plain.make_config([D(heads=2, kv_heads=2, conv=1)]),
    "feed_forward_clamps": plain.make_config([D(ff=48, limit=0.4)], residual_mult=2.0),
    "widths_that_are_no_multiples_of_eight": plain.make_config(
        [A(heads=2, kv_heads=1, dim=12, vdim=10, window=9, rot_dims=6, ff=50), D(heads=2, kv_heads=1, dim=12, vdim=10, conv=3)],
        vocab=51, width=36),
    "two_norms_and_scales": plain.make_config([A(v_mix=False, limit=9.0)], eps=1e-2, residual_mult=0.25, logit_scale=3.0),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(SINGLE))
def test_each_mechanism_alone(tmp_path, name, dtype):
    cfg = SINGLE[name]
    w = plain.random_weights(cfg, 3, low_rank=4, gate_rank=6)
    if name == "feed_forward_clamps":      # both branches reach their limits
        for k in w:
            if k.endswith("mlp.gate") or k.endswith("mlp.up"):
                w[k] = plain.round_bf16(w[k] * 3.0)
    toks = tokens_of(cfg, 61, 1)
    got = Harness(tmp_path, cfg, w, dtype).whole("a", toks)
    close(got, reference(w, cfg, toks), dtype, name)


def test_the_clamp_test_reaches_the_limits():
    cfg = SINGLE["feed_forward_clamps"]
    w = plain.random_weights(cfg, 3, low_rank=4, gate_rank=6)
    x = np.random.default_rng(0).standard_normal((200, cfg["width"]))
    g = plain.linear(x, w["l0.mlp.gate"] * 3.0)
    assert (g > 0.4).mean() > 0.1 and (np.abs(plain.linear(x, w["l0.mlp.up"] * 3.0)) > 0.4).mean() > 0.2


# ---------------------------------------------------------------------------------------------- whole models

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompts_decoding_and_portions(tmp_path, truth, name, dtype):
    """The same logits at every position whether the prompt comes whole, token by token from the first token on
    (the convolutions' zero padding, a state that starts empty), or in portions of several sizes down to two."""
    cfg, ranks, page = CONFIGS[name]
    w = plain.random_weights(cfg, 5, **ranks)
    toks = tokens_of(cfg, 150, 2)
    want = truth(name, toks)
    hs = Harness(tmp_path, cfg, w, dtype, page=page, pages=256 // page * 2)
    close(hs.whole("w", toks), want, dtype, f"{name} whole")
    close(hs.in_portions("d", toks, [1]), want, dtype, f"{name} token by token")
    close(hs.in_portions("p", toks, [2, 3, 17, 2, 1, 40, 5]), want, dtype, f"{name} portions")
    close(hs.in_portions("q", toks, [1, 1, 2, 64, 7]), want, dtype, f"{name} first tokens one by one, then portions")
    # most of it in one step, then the rest one by one
    rows = hs.step([("m", toks[:101], [100])])
    for i in range(101, 150):
        rows.update(hs.step([("m", toks[i:i + 1], [0])]))
    hs.cache.release(hs.live.pop("m")[0])
    close(np.stack([rows[("m", i)] for i in range(100, 150)]), want[100:], dtype, f"{name} prompt then decoding")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "odd", "square", "padded"])
def test_mixed_batches_on_a_small_pool_with_two_state_slots(tmp_path, truth, name, dtype):
    """Requests of unequal lengths, portions of some beside single tokens of others, never more than two alive:
    pages and state slots are given back and used again, and every row equals the request run alone."""
    cfg, ranks, page = CONFIGS[name]
    w = plain.random_weights(cfg, 5, **ranks)
    lengths = [70, 33, 2, 90, 47, 64]
    reqs = [tokens_of(cfg, n, 10 + i) for i, n in enumerate(lengths)]
    want = [truth(name, r) for r in reqs]
    hs = Harness(tmp_path, cfg, w, dtype, page=page, pages=(2 * 128) // page, slots=2)
    rows, at = {}, [0] * len(reqs)
    pending, alive, turn = list(range(len(reqs))), [], 0
    sizes = [5, 1, 2, 31, 1, 1, 16, 3]
    while pending or alive:
        while pending and len(alive) < 2:
            alive.append(pending.pop(0))
        entries, ended = [], []
        for k, i in enumerate(alive):
            n = min(1 if (turn + k) % 3 == 0 else sizes[(turn + i) % len(sizes)], lengths[i] - at[i])
            entries.append((f"r{i}", reqs[i][at[i]:at[i] + n], range(n)))
            at[i] += n
            if at[i] == lengths[i]:
                ended.append(i)
        rows.update(hs.step(entries, end=[f"r{i}" for i in ended]))
        alive = [i for i in alive if i not in ended]
        turn += 1
    assert hs.states.num_free == 2 and all(p.num_free == p.num_blocks for p in hs.cache.pools)
    for i, r in enumerate(reqs):
        close(np.stack([rows[(f"r{i}", j)] for j in range(len(r))]), want[i], dtype, f"{name} request {i} in mixed batches")


# ---------------------------------------------------------------------------------------------- edges that random weights would hide

def _mark_a_token(w, cfg, marked, seed):
    """Gives token `marked` an embedding that no other token's embedding has a part of (they are made orthogonal to
    it, and the first layer's input norm gets the weight one), so that a projection row set to that direction
    answers to this token alone. Returns the direction (entries +-1)."""
    width = cfg["width"]
    d = np.sign(np.random.default_rng(seed).standard_normal(width)).astype(np.float32)
    e = w["embed"].astype(np.float64)
    e -= np.outer(e @ d, d) / width
    e[marked] = 2.0 * d
    w["embed"] = plain.round_bf16(e)
    w["l0.norm1"][:] = 0.0
    return d


def _peaked_attention(window, at, dim=16, vdim=24):
    """One attention layer in which the key of the token at place `at` gets a score far above all others from every
    query while it is in the window: the last key dimension (outside the rotated ones) answers to that token alone, and
    every query has a large entry there."""
    cfg = plain.make_config([A(heads=2, kv_heads=1, dim=dim, vdim=vdim, window=window, rot_dims=4, v_mix=False, ff=None, scale=1.0)],
                            vocab=40, width=32, logit_scale=1.0)
    w = plain.random_weights(cfg, 8, sharp=1.0)
    marked = 7
    d = _mark_a_token(w, cfg, marked, 1)
    w["l0.mix.k"][dim - 1] = 0.5 * d
    w["l0.mix.k.b"][:] = 0.0
    w["l0.mix.q.b"][dim - 1] = w["l0.mix.q.b"][2 * dim - 1] = 6.0 * (dim / 16) ** 0.5
    w["l0.mix.q.norm"][:] = 1.0
    w["l0.mix.k.norm"][:] = 4.0
    w["l0.mix.v"] = plain.round_bf16(w["l0.mix.v"] * 4.0)
    toks = [t if t != marked else marked + 1 for t in tokens_of(cfg, 90, 4)]
    toks[at] = marked
    return cfg, w, toks


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes", [(16, 24), (64, 64), (64, 40)])       # the last two run on the tensor cores in bfloat16
def test_a_key_just_inside_and_just_outside_the_window(tmp_path, dtype, sizes):
    """A key that dominates every score while it is seen: the rows where it is the window's oldest key and the
    rows right after it left differ visibly, in a prompt, in portions cut at the edge, and token by token, with
    the key on a page's border."""
    window, at = 21, 31                                   # page 8: the key is a page's last slot; page 16: its 16th
    cfg, w, toks = _peaked_attention(window, at, *sizes)
    ref = reference(w, cfg, toks)
    want = ref.rows
    last_in, first_out = at + window - 1, at + window
    # the test shows what it is meant to: one key more or less in the window moves those rows far beyond tolerance
    wider = plain.forward(w, plain.make_config([dict(cfg["layers"][0], mixer=dict(cfg["layers"][0]["mixer"], mask={"size": window + 1}))],
                                               vocab=40, width=32, logit_scale=1.0), toks)
    assert rel_err(wider[first_out:first_out + 1], want[first_out:first_out + 1]) > 0.2
    assert rel_err(wider[last_in:last_in + 1], want[last_in:last_in + 1]) < 1e-9
    for page in (8, 16):
        hs = Harness(tmp_path / f"p{page}", cfg, w, dtype, page=page, pages=256 // page)
        close(hs.whole("w", toks), ref, dtype, f"whole, page {page}")
        close(hs.in_portions("a", toks, [last_in + 1, 1, 2, 50]), ref, dtype, f"cut after the last row that sees it, page {page}")
        close(hs.in_portions("b", toks, [last_in, 2, 1, 50]), ref, dtype, f"cut before it, page {page}")
        close(hs.in_portions("c", toks, [at, 1] + [1] * 60), ref, dtype, f"token by token over the edge, page {page}")


def _far_memory():
    """One delta layer whose key channel 5 answers to one token alone, with decays close to one: what that token
    wrote at place 3 stays in the state's row 5, and every later query reads it."""
    cfg = plain.make_config([D(heads=2, kv_heads=1, dim=16, vdim=12, conv=4)], vocab=50, width=32, logit_scale=1.0)
    w = plain.random_weights(cfg, 9, low_rank=4)
    marked = 11
    d = _mark_a_token(w, cfg, marked, 2)
    w["l0.mix.k"][5] = 0.25 * d
    w["l0.mix.k.conv"][5] = [0.0, 0.0, 0.0, 1.0]
    w["l0.mix.A_log"][:] = -6.0                            # rate exp(-6): a decay per token of 1 - 1e-3 or closer to one
    w["l0.mix.dt_bias"][:] = -1.0
    toks = [t if t != marked else marked + 1 for t in tokens_of(cfg, 400, 6)]
    other = list(toks)
    toks[3] = marked
    return cfg, w, toks, other


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_recurrence_remembers_a_token_hundreds_back(tmp_path, dtype):
    """Decays close to one: what the first tokens wrote into the state still decides the last rows. The state is
    carried through a prompt portion, through another, and through decoding, and a second request in another
    slot in between does not touch it."""
    cfg, w, toks, other = _far_memory()
    want, moved = reference(w, cfg, toks), plain.forward(w, cfg, other)
    assert rel_err(moved[-5:], want.rows[-5:]) > 5e-2      # a token 396 back is still felt
    hs = Harness(tmp_path, cfg, w, dtype, pages=64, max_tokens=512)
    close(hs.whole("w", toks), want, dtype, "whole")
    rows = hs.step([("a", toks[:130], range(130))])
    rows.update(hs.step([("x", other[:77], [])]))                       # another request takes another slot
    rows.update(hs.step([("a", toks[130:300], range(170)), ("x", other[77:78], [])]))
    for i in range(300, 400):
        rows.update(hs.step([("a", toks[i:i + 1], [0])] + ([("x", other[78 + i - 300:79 + i - 300], [])] if i % 2 else [])))
    close(np.stack([rows[("a", i)] for i in range(400)]), want, dtype, "portions, then decoding beside another request")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_through_captured_steps_and_slots_used_again(tmp_path, truth, dtype):
    """Three requests decode together for 200 steps (steps of one token each are captured as graphs and replayed),
    end at different times, and a fourth takes over a slot and pages that were just given back."""
    cfg, ranks, page = CONFIGS["mixed"]
    w = plain.random_weights(cfg, 5, **ranks)
    reqs = [tokens_of(cfg, n, 20 + i) for i, n in enumerate([230, 215, 260, 120])]
    want = [truth("mixed", r) for r in reqs]
    hs = Harness(tmp_path, cfg, w, dtype, page=page, pages=3 * 272 // page, slots=3)
    rows = hs.step([(f"r{i}", reqs[i][:12 + i], range(12 + i)) for i in range(3)])
    at = [12, 13, 14, 0]
    alive = [0, 1, 2]
    while alive:
        ended = [i for i in alive if at[i] + 1 == len(reqs[i])]
        rows.update(hs.step([(f"r{i}", reqs[i][at[i]:at[i] + 1], [0]) for i in alive], end=[f"r{i}" for i in ended]))
        for i in alive:
            at[i] += 1
        alive = [i for i in alive if i not in ended]
        if ended and at[3] == 0:                          # the newcomer's prompt rides beside the others' single tokens
            rows.update(hs.step([("r3", reqs[3][:40], range(40))] + [(f"r{i}", reqs[i][at[i]:at[i] + 1], [0]) for i in alive]))
            for i in alive:
                at[i] += 1
            at[3] = 40
            alive.append(3)
    assert hs.runner.graph_replays > 100, "decode steps of this model are meant to be captured"
    for i, r in enumerate(reqs):
        close(np.stack([rows[(f"r{i}", j)] for j in range(len(r))]), want[i], dtype, f"request {i}")


# ---------------------------------------------------------------------------------------------- the engine's own entry points

def test_greedy_generation_through_the_engine_and_its_scheduler(tmp_path):
    """`load_engine` + `generate` / `generate_batch`: the scheduler admits, cuts prompts into portions under a small
    token budget, runs on a small pool; the tokens are the plain implementation's greedy ones."""
    from tiny_inference_engine_b200 import SamplingParams, ServingConfig, load_engine
    cfg, ranks, page = CONFIGS["mixed"]
    w = plain.random_weights(cfg, 5, **ranks)
    plain.write_model_dir(tmp_path, cfg, w)
    prompts = [tokens_of(cfg, n, 30 + i) for i, n in enumerate([19, 3, 41, 1, 27])]
    want = [plain.generate(w, cfg, p, 24) for p in prompts]
    engine = load_engine(tmp_path, dtype="float32", num_pages=40, page_size=page,
                         serving=ServingConfig(max_seqs=3, max_tokens_per_step=16))
    assert engine.generate(prompts[0], SamplingParams(max_tokens=24)) == want[0]
    assert engine.generate_batch(prompts, SamplingParams(max_tokens=24)) == want
    tight = load_engine(tmp_path, dtype="float32", num_pages=9, page_size=page,
                        serving=ServingConfig(max_seqs=3, max_tokens_per_step=16))
    assert tight.generate_batch(prompts, SamplingParams(max_tokens=24)) == want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_of_a_dugazen_model(tmp_path, truth, dtype):
    from test_replay_gpu import Replay
    cfg, ranks, page = CONFIGS["odd"]
    w = plain.random_weights(cfg, 5, **ranks)
    plain.write_model_dir(tmp_path / "m", cfg, w)
    reqs = [tokens_of(cfg, n, 40 + i) for i, n in enumerate([100, 37, 64, 2, 81])]
    want = [truth("odd", r) for r in reqs]
    V = cfg["vocab"]
    rp = Replay(tmp_path / "m", dtype, tmp_path / "out", max_tokens=4 * 128, page_size=page)
    try:
        got = rp.step([("a", reqs[0][:50], range(50)), ("b", reqs[1], range(37))], end=["b"]).reshape(87, V)
        close(got[:50], want[0][:50], dtype, "a, first portion")
        close(got[50:], want[1], dtype, "b whole beside it")
        got = rp.step([("c", reqs[2][:2], [1]), ("a", reqs[0][50:51], [0]), ("d", reqs[3], [0, 1])], end=["d"]).reshape(4, V)
        noise = max(x.noise for x in want)
        close(got, Want(np.stack([want[2].rows[1], want[0].rows[50], want[3].rows[0], want[3].rows[1]]), noise), dtype,
              "three requests, one step")
        assert rp.step([("e", reqs[4][:80], [])]) is None
        got = rp.step([("e", reqs[4][80:], [0]), ("a", reqs[0][51:], range(49)), ("c", reqs[2][2:], [61])],
                      end=["a", "c", "e"]).reshape(51, V)
        close(got, Want(np.concatenate([want[4].rows[80:81], want[0].rows[51:], want[2].rows[63:64]]), noise), dtype, "the rest")
    finally:
        rp.close()


# ---------------------------------------------------------------------------------------------- sizes drawn at random

def _random_config(seed):
    """A configuration with every size, count, constant and the order of layers drawn from what the design allows."""
    r = np.random.default_rng(seed)
    pick = lambda *xs: xs[int(r.integers(len(xs)))]
    kv_v, vdim_mix = pick(1, 2, 3), pick(8, 20, 24, 32, 64)          # blending layers agree on their value heads
    tensor_core = seed % 3 == 0                                       # every third draw: key heads the tensor cores take
    layers = []
    for _ in range(int(r.integers(2, 6))):
        ff = pick(None, 24, 50, 64)
        if r.random() < 0.55:
            mix = bool(r.random() < 0.6)
            kv = kv_v if mix else pick(1, 2, 4)
            dim = pick(64, 128) if tensor_core else pick(8, 12, 20, 32, 48)
            vdim = vdim_mix if mix else pick(4, 16, 40, dim)
            rot = pick(2, 4, dim // 2 // 2 * 2, dim // 2 * 2)
            layers.append(A(heads=kv * pick(1, 2, 4), kv_heads=kv, dim=dim, vdim=vdim, window=pick(1, 2, 5, 16, 33, 64, 400),
                            rot_dims=max(2, rot), base=pick(100.0, 10000.0, 1e6), scale=pick(None, 0.2, 0.05), v_mix=mix, ff=ff,
                            limit=pick(0.5, 2.0, 7.0)))
        else:
            kv = pick(1, 2, 3)
            layers.append(D(heads=kv * pick(1, 2), kv_heads=kv, dim=pick(8, 12, 32, 40, 64, 128), vdim=pick(4, 16, 20, 36, 64),
                            conv=pick(1, 2, 3, 4, 5), ff=ff, limit=pick(0.5, 2.0, 7.0)))
    cfg = plain.make_config(layers, vocab=pick(33, 97, 160, 301), width=pick(24, 36, 64, 72, 128), eps=pick(1e-6, 1e-5, 1e-3),
                            residual_mult=pick(0.3, 0.7, 1.0, 1.6), logit_scale=pick(0.5, 1.0, 2.5))
    return cfg, dict(low_rank=pick(1, 3, 8, 24), gate_rank=pick(2, 8, 17)), pick(4, 8, 16, 32)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(9))
def test_configurations_drawn_at_random(tmp_path, seed, dtype):
    cfg, ranks, page = _random_config(seed)
    w = plain.random_weights(cfg, 100 + seed, **ranks)
    a, b = tokens_of(cfg, 83, seed), tokens_of(cfg, 31, 50 + seed)
    want_a, want_b = reference(w, cfg, a), reference(w, cfg, b)
    hs = Harness(tmp_path, cfg, w, dtype, page=page, pages=-(-256 // page), slots=2)
    close(hs.whole("w", a), want_a, dtype, f"seed {seed} whole")
    rows = hs.step([("a", a[:40], range(40))])
    rows.update(hs.step([("a", a[40:42], [0, 1]), ("b", b[:17], range(17))]))            # a portion of two beside a prompt
    rows.update(hs.step([("b", b[17:], range(14)), ("a", a[42:43], [0])], end=["b"]))    # a prompt's end beside one token
    rows.update(hs.step([("a", a[43:70], range(27))]))
    for i in range(70, 83):
        rows.update(hs.step([("a", a[i:i + 1], [0])]))
    close(np.stack([rows[("a", i)] for i in range(83)]), want_a, dtype, f"seed {seed} in portions and decoded")
    close(np.stack([rows[("b", i)] for i in range(31)]), want_b, dtype, f"seed {seed} the request beside it")
