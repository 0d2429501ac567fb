"""Misudra through the engine against the plain implementation (tests/plain_misudra.py): each mechanism alone,
prompts whole and token by token, portions down to two tokens, mixed batches, pages and state slots that are used
again, keys at a window's edge and far back in a recurrence, the first tokens of a sequence, long decoding, sizes
of several kinds, greedy generation through the engine's own entry point and scheduler."""
import numpy as np
import pytest
import torch

import plain_misudra as plain
from conftest import assert_logits_close, rel_err

pytestmark = pytest.mark.gpu

L, G, M, moe = plain.latent_layer, plain.gla_layer, plain.mamba2_layer, plain.moe

# Configurations. None is a model anyone serves: sizes differ from one another wherever two could be mistaken for each other.
MIXED = plain.make_config([M(), L(mlp=moe()), G(mlp=moe(ff=40, experts=6, top=3, groups=3, keep=2)), M(mlp=moe()), L(), G(mlp=None)],
                          loop=(1, 4, 2))
ODD = plain.make_config([L(heads=3, dim=12, rot_dim=6, vdim=10, kv_rank=20, q_rank=14, window=7, mlp=moe(ff=20, experts=6, top=3, groups=3, keep=2)),
                         G(heads=3, dim=20, vdim=12, tau=3.0, mlp=None),
                         M(heads=6, vdim=10, state=12, groups=3, conv=2, norm_groups=3, mlp=plain.dense(50)),
                         L(heads=2, dim=20, rot_dim=2, vdim=66, kv_rank=34, q_rank=9, window=50, scale=0.31, mlp=None)],
                        vocab=97, width=36, eps=1e-5, loop=(0, 3, 3))
ONES = plain.make_config([L(heads=1, dim=8, rot_dim=2, vdim=8, kv_rank=8, q_rank=8, window=1, mlp=moe(ff=8, experts=2, top=1, groups=1, keep=1)),
                          G(heads=1, dim=8, vdim=8, tau=1.0), M(heads=1, vdim=8, state=8, groups=1, conv=1, norm_groups=1),
                          L(heads=1, dim=8, rot_dim=4, vdim=8, kv_rank=8, q_rank=8, window=1000, mlp=None)], vocab=33, width=16,
                         loop=(3, 4, 1))
# sizes in whole 16-byte pieces and larger heads: what tensor-core kernels take where the engine has them for a mechanism
SQUARE = plain.make_config([L(heads=8, dim=32, rot_dim=32, vdim=32, kv_rank=96, q_rank=64, window=40, mlp=moe(ff=64, experts=8, top=2, groups=2, keep=1)),
                            M(heads=4, vdim=32, state=64, groups=1, conv=4, norm_groups=1, mlp=moe(ff=32, experts=12, top=3, groups=4, keep=3)),
                            G(heads=2, dim=64, vdim=64, tau=12.0),
                            L(heads=16, dim=64, rot_dim=64, vdim=64, kv_rank=64, q_rank=128, window=300)], width=128, loop=(0, 2, 2))
# What the experts of the whole-model tests add to the stream is scaled down: among hundreds of random routing
# decisions some are close calls that bfloat16 rounding decides the other way, in the plain implementation with rounded
# activations as in the engine; at this gain such a flip stays within the bfloat16 tolerance. The experts at full gain
# are held to float32 accuracy by `test_each_mechanism_alone` and by the kernels' own tests below.
GAIN = 0.1
CONFIGS = {"mixed": (MIXED, 8, 16), "odd": (ODD, 3, 8), "ones": (ONES, 1, 4), "square": (SQUARE, 16, 16)}


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
    [(request id, tokens, wanted places)] and returns {(id, position): logits}."""

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
    """Plain logits, computed once per (configuration, tokens)."""
    memo = {}

    def get(name, toks):
        cfg, rank, _ = CONFIGS[name]
        key = (name, tuple(toks))
        if key not in memo:
            memo[key] = reference(plain.random_weights(cfg, 5, decay_rank=rank, expert_gain=GAIN), cfg, toks)
        return memo[key]
    return get


# ---------------------------------------------------------------------------------------------- each mechanism alone

SINGLE = {
    "latent_attention": plain.make_config([L(mlp=None)]),
    "latent_attention_window_out_of_reach_no_gate_effect": plain.make_config([L(heads=2, dim=8, rot_dim=16, vdim=8, kv_rank=24, q_rank=16, window=500, mlp=None)]),
    "latent_attention_sizes_in_whole_pieces": plain.make_config([L(heads=8, dim=64, rot_dim=32, vdim=64, kv_rank=96, q_rank=64, window=30, mlp=None)], width=128),
    "latent_attention_more_heads_than_a_tile_has_rows": plain.make_config([L(heads=40, dim=16, rot_dim=16, vdim=8, kv_rank=32, q_rank=32, window=20, mlp=None)]),
    "latent_attention_no_rotated_part": plain.make_config([L(heads=2, dim=16, rot_dim=0, vdim=8, kv_rank=32, q_rank=24, window=12, mlp=None)]),
    "gla": plain.make_config([G(mlp=None)]),
    "gla_fast_decay": plain.make_config([G(heads=3, dim=8, vdim=40, tau=0.5, mlp=None)]),
    "mamba2": plain.make_config([M(mlp=None)]),
    "mamba2_one_group_one_tap_whole_row_norm": plain.make_config([M(heads=3, vdim=24, state=40, groups=1, conv=1, norm_groups=1, mlp=None)]),
    "mamba2_a_group_per_head": plain.make_config([M(heads=4, vdim=8, state=8, groups=4, conv=5, norm_groups=4, mlp=None)]),
    "dense_feed_forward": plain.make_config([G(mlp=plain.dense(72))]),
    "experts": plain.make_config([G(mlp=moe(ff=24, experts=12, top=3, groups=4, keep=2))]),
    "experts_all_groups_kept_clamps_reached": plain.make_config([M(mlp=moe(ff=16, experts=5, top=5, groups=1, keep=1, limit=0.3))]),
    "experts_half_of_them_chosen": plain.make_config([G(mlp=moe(ff=8, experts=18, top=9, groups=2, keep=2))]),
    "loop_over_everything": plain.make_config([G(mlp=None), M(mlp=None)], loop=(0, 2, 3)),
    "loop_of_one_pass": plain.make_config([G(mlp=None), L(mlp=None)], loop=(1, 2, 1)),
    "widths_that_are_no_multiples_of_eight": plain.make_config(
        [L(heads=2, dim=6, rot_dim=4, vdim=10, kv_rank=13, q_rank=11, window=9, mlp=plain.dense(50)),
         G(heads=2, dim=12, vdim=10, tau=2.0, mlp=moe(ff=9, experts=3, top=2, groups=1, keep=1)),
         M(heads=2, vdim=9, state=7, groups=1, conv=3, norm_groups=2, mlp=None)], vocab=51, width=36, eps=1e-3, loop=(1, 3, 2)),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(SINGLE))
def test_each_mechanism_alone(tmp_path, name, dtype):
    cfg = SINGLE[name]
    w = plain.random_weights(cfg, 3, decay_rank=4)
    if name.startswith("experts_all"):      # both branches reach their limits
        for k in w:
            if k.endswith(".gate") or k.endswith(".up"):
                w[k] = plain.round_bf16(w[k] * 3.0)
    toks = tokens_of(cfg, 61, 1)
    got = Harness(tmp_path, cfg, w, dtype).whole("a", toks)
    close(got, reference(w, cfg, toks), dtype, name)


def test_routing_by_groups_differs_from_plain_top_k():
    """The group rule matters in the test models: some token's choice differs from the plain top-k of its scores."""
    scores = np.array([0.30, 0.02, 0.25, 0.01, 0.20, 0.19, 0.02, 0.01])
    ids, weights = plain.route(scores, top=3, group_count=4, group_keep=2)
    assert sorted(ids.tolist()) == [0, 1, 2] and abs(weights.sum() - 1.0) < 1e-12      # groups 0 and 1 are kept: 0.20 is out of reach


# ---------------------------------------------------------------------------------------------- whole models

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompts_decoding_and_portions(tmp_path, truth, name, dtype):
    """The same logits at every position whether the prompt comes whole, token by token from the first token on
    (the convolutions' zero padding, states that start empty), or in portions of several sizes down to two."""
    cfg, rank, page = CONFIGS[name]
    w = plain.random_weights(cfg, 5, decay_rank=rank, expert_gain=GAIN)
    toks = tokens_of(cfg, 150, 2)
    want = truth(name, toks)
    hs = Harness(tmp_path, cfg, w, dtype, page=page, pages=256 // page * 2)
    close(hs.whole("w", toks), want, dtype, f"{name} whole")
    close(hs.in_portions("d", toks, [1]), want, dtype, f"{name} token by token")
    close(hs.in_portions("p", toks, [2, 3, 17, 2, 1, 40, 5]), want, dtype, f"{name} portions")
    close(hs.in_portions("q", toks, [1, 1, 2, 64, 7]), want, dtype, f"{name} first tokens one by one, then portions")
    rows = hs.step([("m", toks[:101], [100])])
    for i in range(101, 150):
        rows.update(hs.step([("m", toks[i:i + 1], [0])]))
    hs.cache.release(hs.live.pop("m")[0])
    close(np.stack([rows[("m", i)] for i in range(100, 150)]), want[100:], dtype, f"{name} prompt then decoding")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "odd", "square"])
def test_mixed_batches_on_a_small_pool_with_two_state_slots(tmp_path, truth, name, dtype):
    """Requests of unequal lengths, portions of some beside single tokens of others, never more than two alive:
    pages and state slots are given back and used again, and every row equals the request run alone."""
    cfg, rank, page = CONFIGS[name]
    w = plain.random_weights(cfg, 5, decay_rank=rank, expert_gain=GAIN)
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

def _mark_a_token(w, cfg, marked, first_norm="l0.norm1"):
    """Gives token `marked` an embedding along a direction d that lives in the first half of the width, and every other
    token an embedding with no part along d but a fixed part along a second direction e in the other half. The norms
    ahead of the first mixer get the weight one. Returns (d, e), entries +-1 or 0."""
    width = cfg["width"]
    half = width // 2
    r = np.random.default_rng(1)
    d, e = np.zeros(width, dtype=np.float32), np.zeros(width, dtype=np.float32)
    d[:half] = np.sign(r.standard_normal(half))
    e[half:] = np.sign(r.standard_normal(width - half))
    emb = w["embed"].astype(np.float64)
    emb -= np.outer(emb @ d, d) / half + np.outer(emb @ e, e) / (width - half)
    emb += 1.0 * e[None, :]
    emb[marked] = 2.0 * d
    w["embed"] = plain.round_bf16(emb)
    w["embed.norm"][:] = 1.0
    w[first_norm][:] = 1.0
    return d, e


def _peaked_attention(window, at, dim=16, rot=8, vdim=24, rank=32):
    """One latent attention layer in which the key of the token at place `at` gets a score far above all others from
    every other token's query while it is in the window: one latent channel answers to that token alone, one
    unrotated key dimension of every head reads that channel, and every query has a large entry there."""
    cfg = plain.make_config([L(heads=2, dim=dim, rot_dim=rot, vdim=vdim, kv_rank=rank, q_rank=16, window=window, mlp=None, scale=1.0)],
                            vocab=40, width=32)
    w = plain.random_weights(cfg, 8, sharp=1.0)
    marked = 7
    d, e = _mark_a_token(w, cfg, marked)
    p = "l0.mix."
    w[p + "dkv"][3] = 0.5 * d                       # latent channel 3: the marked token only
    w[p + "dkv.norm"][:] = 1.0
    w[p + "uk"][:, 3] = 0.0
    w[p + "uk"][dim - 1] = 0.0
    w[p + "uk"][2 * dim - 1] = 0.0
    w[p + "uk"][dim - 1, 3] = w[p + "uk"][2 * dim - 1, 3] = 1.0        # the last unrotated key dimension of both heads reads it
    w[p + "dq"][5] = 0.5 * e                        # query latent channel 5: the same for every other token
    w[p + "dq.norm"][:] = 1.0
    for head in range(2):
        row = head * (dim + rot) + dim - 1
        w[p + "uq"][row] = 0.0
        w[p + "uq"][row, 5] = 3.0
    w[p + "uv"] = plain.round_bf16(w[p + "uv"] * 4.0)
    toks = [t if t != marked else marked + 1 for t in tokens_of(cfg, 90, 4)]
    toks[at] = marked
    return cfg, w, toks


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes", [(16, 8, 24, 32), (64, 64, 64, 64), (32, 32, 40, 96)])
def test_a_key_just_inside_and_just_outside_the_window(tmp_path, dtype, sizes):
    """A key that dominates every score while it is seen: the rows where it is the window's oldest key and the rows
    right after it left differ visibly, in a prompt, in portions cut at the edge, and token by token, with the key on
    a page's border."""
    window, at = 21, 31                                   # page 8: the key is a page's last slot; page 16: its 16th
    cfg, w, toks = _peaked_attention(window, at, *sizes)
    ref = reference(w, cfg, toks)
    want = ref.rows
    last_in, first_out = at + window - 1, at + window
    wider = dict(cfg, layers=[dict(cfg["layers"][0], mixer=dict(cfg["layers"][0]["mixer"], mask={"size": window + 1}))])
    moved = plain.forward(w, wider, toks)
    assert rel_err(moved[first_out:first_out + 1], want[first_out:first_out + 1]) > 0.2      # one key more in the window shows
    assert rel_err(moved[last_in:last_in + 1], want[last_in:last_in + 1]) < 1e-9
    for page in (8, 16):
        hs = Harness(tmp_path / f"p{page}", cfg, w, dtype, page=page, pages=256 // page)
        close(hs.whole("w", toks), ref, dtype, f"whole, page {page}")
        close(hs.in_portions("a", toks, [last_in + 1, 1, 2, 50]), ref, dtype, f"cut after the last row that sees it, page {page}")
        close(hs.in_portions("b", toks, [last_in, 2, 1, 50]), ref, dtype, f"cut before it, page {page}")
        close(hs.in_portions("c", toks, [at, 1] + [1] * 60), ref, dtype, f"token by token over the edge, page {page}")


def _far_memory(kind):
    """One recurrent layer with decays close to one in which one key channel answers to one token alone: what that
    token wrote at place 3 stays in the state, and every later query reads it."""
    if kind == "gla":
        cfg = plain.make_config([G(heads=2, dim=16, vdim=12, tau=4.0, mlp=None)], vocab=50, width=32)
    else:
        cfg = plain.make_config([M(heads=2, vdim=12, state=16, groups=1, conv=4, norm_groups=1, mlp=None)], vocab=50, width=32)
    w = plain.random_weights(cfg, 9, decay_rank=4)
    marked = 11
    d, _ = _mark_a_token(w, cfg, marked)
    p = "l0.mix."
    if kind == "gla":
        w[p + "k"][5] = 0.5 * d
        w[p + "a2"][:] = 0.0
        w[p + "a2.b"][:] = 0.0                              # sigmoid(0)^(1/4): other channels forget within a few tokens
        w[p + "a2.b"][5] = w[p + "a2.b"][16 + 5] = 9.0      # sigmoid(9)^(1/4): channel 5 decays by 1 - 3e-5 a token
    else:
        inner, N = 24, 16
        w[p + "in"][2 * inner + 5] = 0.5 * d               # channel 5 of B
        w[p + "conv"][inner + 5] = [0.0, 0.0, 0.0, 1.0]
        w[p + "conv.b"][inner + 5] = 0.0
        w[p + "A_log"][:] = -7.0                            # rate exp(-7): decays of 1 - 1e-3 or closer to one
        w[p + "dt_bias"][:] = 0.0
    toks = [t if t != marked else marked + 1 for t in tokens_of(cfg, 400, 6)]
    other = list(toks)
    toks[3] = marked
    return cfg, w, toks, other


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", ["gla", "mamba2"])
def test_the_recurrence_remembers_a_token_hundreds_back(tmp_path, kind, dtype):
    """Decays close to one: what the first tokens wrote into the state still decides the last rows. The state is
    carried through a prompt portion, through another, and through decoding, and a second request in another slot in
    between does not touch it."""
    cfg, w, toks, other = _far_memory(kind)
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
    cfg, rank, page = CONFIGS["mixed"]
    w = plain.random_weights(cfg, 5, decay_rank=rank, expert_gain=GAIN)
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
    cfg, rank, page = CONFIGS["mixed"]
    w = plain.random_weights(cfg, 5, decay_rank=rank, expert_gain=GAIN)
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


def test_the_command_line_generates_the_plain_greedy_tokens(tmp_path, capsys):
    from tiny_inference_engine_b200.cli.main import main
    cfg, rank, page = CONFIGS["mixed"]
    w = plain.random_weights(cfg, 5, decay_rank=rank, expert_gain=GAIN)
    plain.write_model_dir(tmp_path, cfg, w)
    prompt = tokens_of(cfg, 21, 77)
    assert main(["generate", "-m", str(tmp_path), "-p", " ".join(map(str, prompt)), "--temp", "0", "--max-tokens", "12",
                 "--dtype", "float32", "--kv-mem", "64M", "--max-tokens-per-step", "8", "--max-seqs", "2"]) == 0
    assert [int(t) for t in capsys.readouterr().out.split()] == plain.generate(w, cfg, prompt, 12)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_of_a_misudra_model(tmp_path, truth, dtype):
    from test_replay_gpu import Replay
    cfg, rank, page = CONFIGS["odd"]
    w = plain.random_weights(cfg, 5, decay_rank=rank, expert_gain=GAIN)
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
    """A configuration with every size, count, constant, the order of layers and the loop drawn from what the design allows."""
    r = np.random.default_rng(seed)
    pick = lambda *xs: xs[int(r.integers(len(xs)))]

    def mlp():
        kind = pick("none", "dense", "moe", "moe")
        if kind == "none":
            return None
        if kind == "dense":
            return plain.dense(pick(24, 50, 64))
        groups = pick(1, 2, 3, 4)
        per = pick(1, 2, 4)
        keep = int(r.integers(1, groups + 1))
        return moe(ff=pick(8, 20, 32), experts=groups * per, top=int(r.integers(1, min(keep * per, 6) + 1)), groups=groups, keep=keep,
                   limit=pick(0.5, 2.0, 7.0))
    aligned = seed % 3 == 0                                # every third draw: sizes in whole 16-byte pieces
    layers = []
    for _ in range(int(r.integers(2, 6))):
        kind = pick("latent", "gla", "mamba2")
        if kind == "latent":
            dim, rot = (pick(32, 64), pick(32, 64)) if aligned else (pick(4, 12, 20, 32), pick(2, 4, 6, 16))
            layers.append(L(heads=pick(1, 2, 3, 8), dim=dim, rot_dim=rot, vdim=pick(16, 64) if aligned else pick(4, 10, 40),
                            kv_rank=pick(32, 96) if aligned else pick(5, 16, 28, 50), q_rank=pick(16, 64) if aligned else pick(3, 12, 24),
                            window=pick(1, 2, 5, 16, 33, 64, 400), base=pick(100.0, 10000.0, 1e6), scale=pick(None, 0.2, 0.05), mlp=mlp()))
        elif kind == "gla":
            layers.append(G(heads=pick(1, 2, 3), dim=pick(8, 12, 32, 40, 64, 128), vdim=pick(4, 16, 20, 36, 64), tau=pick(1.0, 4.0, 20.0),
                            mlp=mlp()))
        else:
            groups = pick(1, 2, 3)
            heads = groups * pick(1, 2)
            vdim = pick(4, 8, 12, 32)
            parts = pick(*[n for n in (1, 2, 3, 4, heads) if (heads * vdim) % n == 0])
            layers.append(M(heads=heads, vdim=vdim, state=pick(4, 16, 24, 64, 128), groups=groups, conv=pick(1, 2, 3, 4, 5), norm_groups=parts,
                            mlp=mlp()))
    loop = None
    if r.random() < 0.7:
        a = int(r.integers(0, len(layers)))
        b = int(r.integers(a + 1, len(layers) + 1))
        loop = (a, b, int(r.integers(1, 4)))
    cfg = plain.make_config(layers, vocab=pick(33, 97, 160, 301), width=pick(24, 36, 64, 72, 128), eps=pick(1e-6, 1e-5, 1e-3), loop=loop)
    return cfg, pick(1, 3, 8, 24), pick(4, 8, 16, 32)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(12))
def test_configurations_drawn_at_random(tmp_path, seed, dtype):
    cfg, rank, page = _random_config(seed)
    w = plain.random_weights(cfg, 100 + seed, decay_rank=rank, expert_gain=GAIN)
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


# ---------------------------------------------------------------------------------------------- the experts' kernels alone

@pytest.mark.parametrize("shape", [(20, 4, 5, 3), (6, 3, 3, 2), (5, 5, 1, 1), (64, 8, 8, 4), (12, 1, 12, 1), (2, 1, 1, 1), (257, 6, 1, 1)])
def test_routing_kernel_against_the_plain_rule(shape):
    from tiny_inference_engine_b200 import ops
    E, top, groups, keep = shape
    r = np.random.default_rng(E)
    logits = (r.standard_normal((97, E)) * 3.0).astype(np.float32)
    ids = torch.empty((97, top), dtype=torch.int32, device="cuda")
    weights = torch.empty((97, top), dtype=torch.float32, device="cuda")
    ops.moe_route(torch.from_numpy(logits).cuda(), top, groups, keep, ids, weights)
    ids, weights = ids.cpu().numpy(), weights.cpu().numpy()
    for t in range(97):
        z = logits[t].astype(np.float64)
        s = np.exp(z - z.max())
        want_ids, want_w = plain.route(s / s.sum(), top, groups, keep)
        assert ids[t].tolist() == want_ids.tolist(), f"token {t}"
        assert np.allclose(weights[t], want_w, rtol=1e-5, atol=1e-7)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens", [1, 7, 300])
def test_grouped_products_against_plain_sums(tokens, dtype):
    """Tokens listed by expert on the device, both grouped products, the weighted partial sums: against a loop over pairs."""
    from tiny_inference_engine_b200 import ops
    E, top, D, I = 5, 3, 40, 24
    g = torch.Generator().manual_seed(tokens)
    h = torch.randn((tokens, D), generator=g).to(dtype).cuda()
    w1 = (torch.randn((E, 2 * I, D), generator=g) / D ** 0.5).to(dtype).cuda()
    w2 = (torch.randn((E, D, I), generator=g) / I ** 0.5).to(dtype).cuda()
    ids = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(tokens)]).to(torch.int32).cuda()
    weights = torch.rand((tokens, top), generator=g).cuda()
    for block_m in (4, 16, 64):
        tiles = ops.moe_max_tiles(tokens * top, E, block_m)
        sorted_pairs = torch.empty(tiles * block_m, dtype=torch.int32, device="cuda")
        tile_expert = torch.empty(tiles, dtype=torch.int32, device="cuda")
        meta = torch.zeros(4, dtype=torch.int32, device="cuda")
        ops.moe_align(ids, E, block_m, sorted_pairs, tile_expert, meta)
        listed = sorted_pairs[:int(meta[0]) * block_m].cpu().numpy()
        assert sorted(listed[listed >= 0].tolist()) == list(range(tokens * top))          # every pair once
        for i, pair in enumerate(listed):
            assert pair < 0 or int(ids.view(-1)[pair]) == int(tile_expert[i // block_m])   # in its expert's tiles
        first = torch.empty((tokens * top, 2 * I), dtype=dtype, device="cuda")
        ops.moe_gemm(h, w1, first, top, block_m, sorted_pairs, tile_expert, meta, tiles)
        want = torch.stack([w1[int(ids[t, s])].float() @ h[t].float() for t in range(tokens) for s in range(top)])
        assert torch.allclose(first.float(), want, rtol=2e-2 if dtype == torch.bfloat16 else 1e-5, atol=2e-2 if dtype == torch.bfloat16 else 1e-5)
        act = first[:, :I].contiguous()
        partial = torch.zeros(top * tokens * D, dtype=torch.float32, device="cuda")
        ops.moe_gemm(act, w2, None, top, block_m, sorted_pairs, tile_expert, meta, tiles, second=True, partial=partial,
                     weights=weights.view(-1))
        want = torch.stack([torch.stack([weights[t, s] * (w2[int(ids[t, s])].float() @ act[t * top + s].float()) for t in range(tokens)])
                            for s in range(top)])
        assert torch.allclose(partial.view(top, tokens, D), want, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("tokens", [40, 700])
def test_grouped_products_on_the_tensor_cores(tokens):
    """bfloat16 prompts: rows copied into the listed order, the grouped products over weights in k-blocks, the weighted
    results back to their tokens; and the few-rows kernel over the same weights."""
    from tiny_inference_engine_b200 import ops
    E, top, D, I = 6, 2, 72, 40
    g = torch.Generator().manual_seed(tokens)
    h = torch.randn((tokens, D), generator=g).to(torch.bfloat16).cuda()
    w1 = (torch.randn((E, 2 * I, D), generator=g) / D ** 0.5).to(torch.bfloat16).cuda()
    w2 = (torch.randn((E, D, I), generator=g) / I ** 0.5).to(torch.bfloat16).cuda()
    b1, b2 = ops.pack_k_blocks(w1.view(E * 2 * I, D)), ops.pack_k_blocks(w2.view(E * D, I))
    ids = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(tokens)]).to(torch.int32).cuda()
    ids[:, 0] = torch.where(ids[:, 0] == 4, ids[:, 1], ids[:, 0])          # expert 4 mostly idle, some experts busier
    weights = torch.rand((tokens, top), generator=g).cuda()
    want1 = torch.stack([w1[int(ids[t, s])].float() @ h[t].float() for t in range(tokens) for s in range(top)])
    for block_m in (4, ops.GROUPED_TILE):
        tiles = ops.moe_max_tiles(tokens * top, E, block_m)
        sorted_pairs = torch.empty(tiles * block_m, dtype=torch.int32, device="cuda")
        tile_expert = torch.empty(tiles, dtype=torch.int32, device="cuda")
        meta = torch.zeros(4, dtype=torch.int32, device="cuda")
        ops.moe_align(ids, E, block_m, sorted_pairs, tile_expert, meta)
        partial = torch.zeros(top * tokens * D, dtype=torch.float32, device="cuda")
        if block_m == 4:
            first = torch.empty((tokens * top, 2 * I), dtype=torch.bfloat16, device="cuda")
            ops.moe_gemm(h, b1, first, top, 4, sorted_pairs, tile_expert, meta, tiles, blocks_of=(2 * I, D))
            assert torch.allclose(first.float(), want1, rtol=2e-2, atol=2e-2)
            act = first[:, :I].contiguous()
            ops.moe_gemm(act, b2, None, top, 4, sorted_pairs, tile_expert, meta, tiles, second=True, partial=partial,
                         weights=weights.view(-1), blocks_of=(D, I))
        else:
            rows = tiles * block_m
            xs = torch.full((rows, D), float("nan"), dtype=torch.bfloat16, device="cuda")
            ops.moe_gather(h, sorted_pairs, meta, top, xs)
            first = torch.empty((rows, 2 * I), dtype=torch.bfloat16, device="cuda")
            ops.gemm_grouped(xs, b1, first, 2 * I, D, meta, tile_expert)
            listed = sorted_pairs[:int(meta[0]) * block_m].cpu().numpy()
            at = {int(p): r for r, p in enumerate(listed) if p >= 0}
            order = torch.tensor([at[p] for p in range(tokens * top)], device="cuda")
            assert torch.allclose(first[order].float(), want1, rtol=2e-2, atol=2e-2)
            act = first[:, :I].contiguous()
            y = torch.empty((rows, D), dtype=torch.bfloat16, device="cuda")
            ops.gemm_grouped(act, b2, y, D, I, meta, tile_expert)
            ops.moe_combine(y, sorted_pairs, meta, top, weights.view(-1), partial, tokens)
            act = act[order]
        torch.cuda.synchronize()
        want = torch.stack([torch.stack([weights[t, s] * (w2[int(ids[t, s])].float() @ act[t * top + s].float()) for t in range(tokens)])
                            for s in range(top)])
        assert torch.allclose(partial.view(top, tokens, D), want, rtol=2e-2, atol=2e-2), f"tiles of {block_m}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(5, 3, 24, 40, 8), (300, 4, 64, 96, 32), (130, 2, 10, 6, 0), (1000, 16, 128, 64, 64)])
def test_products_batched_over_heads(shape, dtype):
    """out[t, h, :N] = w[h] a[t, h, :K] with the heads side by side in a row and room behind each head's result."""
    from tiny_inference_engine_b200 import ops
    T, H, N, K, room = shape
    g = torch.Generator().manual_seed(T)
    a = torch.randn((T, H * (K + 8)), generator=g).to(dtype).cuda()
    w = (torch.randn((H, N, K), generator=g) / K ** 0.5).to(dtype).cuda()
    out = torch.zeros((T, H * (N + room)), dtype=dtype, device="cuda")
    ops.gemm_heads(a, w, out, H)
    want = torch.einsum("thk,hnk->thn", a.view(T, H, K + 8)[:, :, :K].float(), w.float())
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
    assert torch.allclose(out.view(T, H, N + room)[:, :, :N].float(), want, rtol=tol, atol=tol)
    assert (out.view(T, H, N + room)[:, :, N:] == 0).all()                  # what lies behind a head's result is left alone
