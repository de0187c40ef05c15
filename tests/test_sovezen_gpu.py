"""Sovezen through the engine against the plain implementation (tests/plain_sovezen.py, float64).

Three small models that differ in every size and option (tests/sovezen_models.py) are run whole, as a prompt
followed by single tokens, in portions down to two tokens, and as mixed batches in a pool whose pages and slots
are used again; single mechanisms are isolated by one-layer configurations; weights are bent where random ones
would hide a fault (a far key among hundreds, a sink, a position's angle, one expert among many).

Bounds.  The measure is the RMS over the vocabulary of the logits' difference (mean taken off) over the RMS of
the wanted logits, the largest over the rows.  float32: the engine computes what the plain implementation
computes in another order of float additions: 2e-4.  bfloat16: what rounding alone does depends on the model, so it
is measured: the plain implementation is run once more with the operands and results of its products rounded to
bfloat16 values, and the engine may be three times as far from the exact logits as that run is (at least 2e-2).
The bfloat16 runs use routers whose choices no rounding can turn (sovezen_models.make_weights says why); routers
that choose token by token run in float32.  A lost key, sink, expert or factor moves the logits by their own size.
"""
import numpy as np
import pytest
import torch

import plain_sovezen as plain
from sovezen_models import CONFIGS, _config, dense, layer, make_weights, moe, plain_queries, rel_error, rotated, write_model

pytestmark = pytest.mark.gpu

BOUND_F32 = 2e-4
_cache = {}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """(name, dtype) -> (config, weights, model folder); the bfloat16 models have decisive routers."""
    base = tmp_path_factory.mktemp("sovezen")
    out = {}
    for i, (name, cfg) in enumerate(sorted(CONFIGS.items())):
        for dtype in ("float32", "bfloat16"):
            w = make_weights(cfg, seed=200 + i, decisive_router=dtype == "bfloat16")
            out[name, dtype] = (cfg, w, write_model(cfg, w, str(base / f"{name}_{dtype}")))
    return out


def _engine(model_dir, dtype, max_tokens=512, page_size=16, max_requests=4):
    from sandyrt_b200.engine.step import Engine
    from sandyrt_b200.models.model import load_model

    model = load_model(model_dir, device="cuda:0", dtype=getattr(torch, dtype))
    eng = Engine(model, max_tokens=max_tokens, page_size=page_size, max_requests=max_requests)
    eng.cache.device_caches.poison()
    return eng


def _tokens(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], size=n).tolist()


def _want(cfg, w, ids):
    key = (id(w), tuple(ids))
    if key not in _cache:
        _cache[key] = [plain.forward(cfg, w, ids).numpy(), None]
    return _cache[key][0]


def _bound(cfg, w, ids, dtype):
    if dtype == "float32":
        return BOUND_F32
    want = _want(cfg, w, ids)
    entry = _cache[(id(w), tuple(ids))]
    if entry[1] is None:
        entry[1] = rel_error(plain.forward_rounded(cfg, w, ids).numpy(), want)
    return max(2e-2, 3 * entry[1])


def _run_cuts(eng, rid, ids, cuts, release=True):
    from sandyrt_b200.engine.step import StepEntry

    rows, pos = [], 0
    for n in cuts:
        rows.append(eng.step([StepEntry(rid, ids[pos:pos + n], list(range(n)))]).cpu().numpy().copy())
        pos += n
    assert pos == len(ids)
    eng.check_status()
    if release:
        eng.release(rid)
    return np.concatenate(rows, axis=0)


def _check(got, model, ids, dtype, what):
    cfg, w = model
    e, bound = rel_error(got, _want(cfg, w, ids)), _bound(cfg, w, ids, dtype)
    assert e < bound, f"{what}: relative error {e:.3e} (bound {bound:.1e})"


# ---- whole models under every way of cutting the work -------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole_prompts_and_first_tokens(models, name, dtype):
    cfg, w, path = models[name, dtype]
    eng = _engine(path, dtype)
    for i, n in enumerate([1, 2, 5, 33, 150]):
        ids = _tokens(cfg, n, seed=i)
        _check(_run_cuts(eng, f"r{i}", ids, [n]), (cfg, w), ids, dtype, f"{name}: whole prompt of {n}")
    eng.cache.alloc.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_prompt_then_single_tokens(models, name, dtype):
    """Most of the request in one step, the last 40 tokens one by one (the later ones replay a recorded graph)."""
    cfg, w, path = models[name, dtype]
    eng = _engine(path, dtype)
    ids = _tokens(cfg, 131, seed=7)
    got = _run_cuts(eng, "r", ids, [91] + [1] * 40)
    _check(got, (cfg, w), ids, dtype, f"{name}: prompt + 40 single tokens")
    assert eng.graph_replays > 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_portions_of_changing_size(models, name, dtype):
    cfg, w, path = models[name, dtype]
    eng = _engine(path, dtype)
    ids = _tokens(cfg, 101, seed=11)
    for cuts in ([24, 24, 24, 24, 5], [2, 3, 17, 16, 15, 31, 2, 13, 2], [1, 2, 1, 3, 94], [64, 37], [16, 16, 32, 1, 1, 35]):
        assert sum(cuts) == len(ids)
        _check(_run_cuts(eng, "r", ids, cuts), (cfg, w), ids, dtype, f"{name}: portions {cuts}")
    eng.cache.alloc.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_in_every_division(models, dtype):
    """The first few tokens of a request (position 0 turns nothing, a lone token's softmax holds its sink and itself)."""
    cfg, w, path = models["A", dtype]
    eng = _engine(path, dtype)
    ids = _tokens(cfg, 6, seed=13)
    for cuts in ([1] * 6, [2, 2, 2], [1, 5], [5, 1], [3, 1, 2], [6]):
        _check(_run_cuts(eng, "r", ids, cuts), (cfg, w), ids, dtype, f"first tokens as {cuts}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_mixed_batches_with_pages_and_slots_used_again(models, name, dtype):
    """Up to four live requests, portions of some beside single tokens of others; the pool holds 12 pages of 16
    tokens for requests that need 24 in all, pages poisoned.  Each request's rows must equal what it gives alone."""
    from sandyrt_b200.engine.step import StepEntry

    cfg, w, path = models[name, dtype]
    eng = _engine(path, dtype, max_tokens=192, page_size=16, max_requests=4)
    lengths = [37, 50, 21, 64, 45, 30, 58, 17]
    prompts = [_tokens(cfg, n, seed=20 + i) for i, n in enumerate(lengths)]
    rng = np.random.default_rng(1)
    fed = [0] * len(prompts)
    got = [[] for _ in prompts]
    live, nxt, slots_seen = [], 0, []
    while nxt < len(prompts) or live:
        while nxt < len(prompts) and len(live) < 4:
            if sum(-(-lengths[r] // 16) for r in live) + -(-lengths[nxt] // 16) > 12:
                break
            live.append(nxt)
            nxt += 1
        entries = []
        for r in live:
            left = lengths[r] - fed[r]
            n = int(rng.integers(2, min(left, 19) + 1)) if left > 8 and rng.random() < 0.6 else 1
            entries.append(StepEntry(r, prompts[r][fed[r]:fed[r] + n], list(range(n))))
        if rng.random() < 0.3 and len(entries) > 1:
            entries.pop(int(rng.integers(0, len(entries))))
        out = eng.step(entries).cpu().numpy()
        row = 0
        for e in entries:
            n = len(e.tokens)
            got[e.rid].append(out[row:row + n].copy())
            row += n
            fed[e.rid] += n
            slots_seen.append((e.rid, eng.cache.alloc.slot(e.rid)))
        for r in list(live):
            if fed[r] == lengths[r]:
                eng.release(r)
                live.remove(r)
        eng.cache.alloc.check()
    eng.check_status()
    assert len({s for _, s in slots_seen}) <= 4 and len({r for r, _ in slots_seen}) == 8      # slots were used again
    for r, ids in enumerate(prompts):
        _check(np.concatenate(got[r], axis=0), (cfg, w), ids, dtype, f"{name}: mixed request {r}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_batch_gives_each_request_what_it_gives_alone(models, dtype):
    """Unequal requests in one step against each alone: same rows, beyond rounding.  The experts see other
    neighbours in their groups, the attention other tiles."""
    from sandyrt_b200.engine.step import StepEntry

    cfg, w, path = models["C", dtype]
    eng = _engine(path, dtype)
    prompts = [_tokens(cfg, n, seed=40 + n) for n in (70, 3, 29, 1)]
    alone = [_run_cuts(eng, f"a{i}", p, [len(p)]) for i, p in enumerate(prompts)]
    out = eng.step([StepEntry(f"b{i}", p, list(range(len(p)))) for i, p in enumerate(prompts)]).cpu().numpy()
    row = 0
    for i, p in enumerate(prompts):
        e = rel_error(out[row:row + len(p)], alone[i])
        assert e < (1e-5 if dtype == "float32" else 2e-2), f"request {i} in a batch differs from itself alone by {e:.2e}"
        row += len(p)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_across_page_borders(models, dtype):
    """300 single tokens behind a short prompt, pages of 8: every page border is crossed by a decoded token."""
    cfg, w, path = models["A", dtype]
    eng = _engine(path, dtype, max_tokens=512, page_size=8)
    ids = _tokens(cfg, 310, seed=3)
    got = _run_cuts(eng, "r", ids, [10] + [1] * 300)
    _check(got, (cfg, w), ids, dtype, "A: 300 decoded tokens")


# ---- single mechanisms --------------------------------------------------------------------------------
def _one_model(tmp_path, cfg, seed, bend=None, decisive=False):
    w = make_weights(cfg, seed, decisive_router=decisive)
    if bend:
        bend(w)
        w = {k: v.to(torch.bfloat16).to(torch.float32) for k, v in w.items()}
    return w, write_model(cfg, w, str(tmp_path / f"m{seed}"))


ONE_LAYER = {
    "rotated, no feed-forward": lambda: [layer(rotated(3, 24, 8, 20, 40, base=30.0), None)],
    "query latent, no feed-forward": lambda: [layer(plain_queries(3, 24, 20, 40, 28), None)],
    "dense feed-forward": lambda: [layer(plain_queries(1, 8, 8, 16, 8), dense(72))],
    "a latent wider than the tensor-core kernels take": lambda: [layer(rotated(2, 16, 48, 16, 296, base=1000.0), None)],
    "routed feed-forward": lambda: [layer(plain_queries(1, 8, 8, 16, 8), moe(6, 3, 24))],
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", sorted(ONE_LAYER))
def test_each_mechanism_alone(tmp_path, which, dtype):
    cfg = _config(61, 48, ONE_LAYER[which](), eps=1e-5, logit_scale=1.3)
    w, path = _one_model(tmp_path, cfg, seed=5, decisive=dtype == "bfloat16")
    eng = _engine(path, dtype)
    ids = _tokens(cfg, 90, seed=1)
    _check(_run_cuts(eng, "r", ids, [90]), (cfg, w), ids, dtype, f"{which}, whole")
    _check(_run_cuts(eng, "r", ids, [40, 2, 30] + [1] * 18), (cfg, w), ids, dtype, f"{which}, in portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("form", ["rotated", "query latent"])
def test_a_far_key_among_hundreds_and_the_sink(tmp_path, form, dtype):
    """Attention alone, 400 tokens.  The query projection is scaled up so that scores are sharp: every query then
    looks at one or two keys, mostly far back, and a key that is lost or shifted by one changes the logits by far
    more than the bound.  Then (rotated form) the sinks are raised until they take most of the weight: leaving them
    out would multiply the attention's output several times."""
    mixer = rotated(4, 16, 16, 16, 24, base=10000.0, scale=1.0) if form == "rotated" else plain_queries(4, 16, 16, 24, 16, scale=1.0)
    cfg = _config(53, 64, [layer(mixer, None)], eps=1e-5, logit_scale=1.0)
    q_name = "l0.mix.q" if form == "rotated" else "l0.mix.uq"

    def sharp(w):
        w[q_name] *= 6.0

    def sunk(w):
        w["l0.mix.sink"] = torch.full((4,), 6.0)

    for bend, what in ((sharp, "sharp scores"), (sunk, "heavy sinks")):
        if bend is sunk and form != "rotated":
            continue
        w, path = _one_model(tmp_path, cfg, seed=9 if bend is sharp else 10, bend=bend)
        ids = _tokens(cfg, 400, seed=2)
        want = _want(cfg, w, ids)
        if bend is sunk:       # the sink matters: without it the logits are somewhere else entirely
            w2 = dict(w)
            w2["l0.mix.sink"] = torch.full((4,), -30.0)
            assert rel_error(_want(cfg, w2, ids), want) > 0.2
        eng = _engine(path, dtype, max_tokens=512, page_size=16)
        _check(_run_cuts(eng, "r", ids, [400]), (cfg, w), ids, dtype, f"{what}, whole")
        _check(_run_cuts(eng, "r", ids, [250, 100, 18] + [1] * 32), (cfg, w), ids, dtype, f"{what}, portions and single tokens")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_positions_decide_which_key_wins(tmp_path, dtype):
    """The unrotated parts are switched off, so a score is the rotated parts' alone and depends on the distance
    between query and key.  With a small base every pair of entries turns fast: a position that is off by one, or
    pairs taken as (i, i + n/2) instead of neighbours, gives other logits altogether."""
    cfg = _config(53, 64, [layer(rotated(2, 8, 16, 16, 24, base=8.0, scale=1.0), None)], eps=1e-5, logit_scale=1.0)

    def bend(w):
        w["l0.mix.uk"] *= 0.0
        w["l0.mix.q"] *= 3.0

    w, path = _one_model(tmp_path, cfg, seed=21, bend=bend)
    ids = _tokens(cfg, 200, seed=4)
    eng = _engine(path, dtype)
    _check(_run_cuts(eng, "r", ids, [200]), (cfg, w), ids, dtype, "rotated parts alone, whole")
    _check(_run_cuts(eng, "r", ids, [3, 61, 100, 2] + [1] * 34), (cfg, w), ids, dtype, "rotated parts alone, portions and single tokens")


def test_routers_that_choose_token_by_token(tmp_path):
    """float32, ordinary routers: the choices change from token to token (checked), every expert is used, and a step
    of many tokens groups them by expert while single tokens go one by one."""
    cfg = _config(89, 56, [layer(plain_queries(2, 8, 8, 16, 8), moe(7, 2, 16)), layer(rotated(2, 8, 8, 8, 8), moe(4, 3, 24))],
                  eps=1e-5, logit_scale=0.8)
    w, path = _one_model(tmp_path, cfg, seed=31)
    ids = _tokens(cfg, 260, seed=8)
    assert plain.router_margin(cfg, w, ids) > 1e-4
    w64 = {k: v.to(torch.float64) for k, v in w.items()}
    h = plain.rms_norm(w64["embed"][torch.tensor(ids)], w64["l0.norm1"], 1e-5)
    chosen = (h @ w64["l0.mlp.router"].t() + w64["l0.mlp.router.b"]).topk(2, -1).indices
    assert len(set(chosen.flatten().tolist())) == 7 and len({tuple(sorted(c)) for c in chosen.tolist()}) > 8
    eng = _engine(path, "float32")
    _check(_run_cuts(eng, "r", ids, [260]), (cfg, w), ids, "float32", "token-by-token routing, whole")
    _check(_run_cuts(eng, "r", ids, [33, 2, 190, 5] + [1] * 30), (cfg, w), ids, "float32", "token-by-token routing, portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_batch_decoding_with_many_heads_on_one_latent(tmp_path, dtype):
    """Four requests of about 700 tokens decode side by side in a layer of 16 heads: 4 x 16 x 768 (token, head, key)
    triples a step, which in bfloat16 is where the decode attention takes the heads of a group as the rows of one
    tensor-core product (rows of 64; a second layer with rows of 128).  Scores are sharpened so that far keys win."""
    from sandyrt_b200.engine.step import StepEntry

    cfg = _config(59, 64, [layer(rotated(16, 16, 16, 8, 48, base=10000.0, scale=1.0), None),
                           layer(plain_queries(16, 16, 8, 128, 24, scale=1.0), dense(48))], eps=1e-5, logit_scale=1.0)

    def sharp(w):
        w["l0.mix.q"] *= 3.0
        w["l1.mix.uq"] *= 3.0

    w, path = _one_model(tmp_path, cfg, seed=51, bend=sharp)
    lengths = [700, 689, 703, 650]
    seqs = [_tokens(cfg, n, seed=70 + i) for i, n in enumerate(lengths)]
    eng = _engine(path, dtype, max_tokens=3072, page_size=16)
    n_decoded = 9
    for i, ids in enumerate(seqs):
        eng.step([StepEntry(i, ids[:-n_decoded], [])])
    got = [[] for _ in seqs]
    for k in range(n_decoded):
        out = eng.step([StepEntry(i, [ids[len(ids) - n_decoded + k]], [0]) for i, ids in enumerate(seqs)]).cpu().numpy()
        for i in range(len(seqs)):
            got[i].append(out[i:i + 1].copy())
    eng.check_status()
    for i, ids in enumerate(seqs):
        want = _want(cfg, w, ids)[-n_decoded:]
        bound = BOUND_F32 if dtype == "float32" else max(2e-2, 3 * rel_error(plain.forward_rounded(cfg, w, ids).numpy()[-n_decoded:], want))
        e = rel_error(np.concatenate(got[i]), want)
        assert e < bound, f"request {i}: relative error {e:.3e} (bound {bound:.1e})"


def test_options_at_their_edges(tmp_path):
    """A rotated layer without a rotated part (rot_dim 0), a router that takes 40 of 48 experts, a layer without a
    feed-forward whose file still holds its second factor (it is read past), a logit scale of one; float32."""
    mixer = rotated(3, 16, 0, 8, 24)
    mixer["mixer"]["rot"] = {"dims": 0, "base": 10000.0}
    cfg = _config(67, 40, [layer(mixer, moe(48, 40, 8)), layer(plain_queries(2, 8, 8, 16, 8), None)], eps=1e-5, logit_scale=1.0)
    w = make_weights(cfg, seed=41)
    on_disk = dict(w)
    on_disk["l1.ls2"] = torch.ones(40)
    path = write_model(cfg, on_disk, str(tmp_path / "edges"))
    ids = _tokens(cfg, 70, seed=9)
    assert plain.router_margin(cfg, w, ids) > 1e-4
    eng = _engine(path, "float32")
    _check(_run_cuts(eng, "r", ids, [70]), (cfg, w), ids, "float32", "edges, whole")
    _check(_run_cuts(eng, "r", ids, [31, 2, 30] + [1] * 7), (cfg, w), ids, "float32", "edges, in portions")


# ---- the entry point --------------------------------------------------------------------------------------
def test_greedy_generation_through_the_entry_point(models):
    """LLM.generate (scheduler, prompt portions, decode bursts) on three requests at once, float32: the same tokens
    as greedy decoding with the plain implementation, wherever its top two logits are clearly apart."""
    from sandyrt_b200.engine.llm import LLM

    cfg, w, path = models["A", "float32"]
    llm = LLM(path, dtype="float32", cache_tokens=1024, max_live=4, prefill_chunk_tokens=24, max_step_tokens=64)
    prompts = [_tokens(cfg, n, seed=60 + n) for n in (5, 40, 71)]
    outs = llm.generate(prompts, max_tokens=20)
    for p, r in zip(prompts, outs):
        assert r.finish_reason == "length" and len(r.output_ids) == 20
        ids = list(p)
        for tok in r.output_ids:
            l = _want(cfg, w, ids)[-1]
            top2 = np.sort(l)[-2:]
            if top2[1] - top2[0] > 1e-3:
                assert tok == int(np.argmax(l)), f"token {len(ids) - len(p)} of the request with {len(p)} prompt tokens"
            ids.append(tok)
