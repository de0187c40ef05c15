"""Panupel through the engine against the plain implementation (tests/plain_panupel.py, float64).

Four small models that differ in every size and option (tests/panupel_models.py) are run whole, as a prompt
followed by single tokens, in portions down to two tokens, and as mixed batches in a pool whose pages and
state slots are used again; single mechanisms are isolated by configurations that switch the others off;
weights are bent where random ones would hide a fault (a far key, a sink, the recurrences' long memory).

Bounds.  The measure is the RMS over the vocabulary of the logits' difference (mean taken off) over the RMS of
the wanted logits, the largest over the rows.  float32: the engine computes what the plain implementation
computes in another order of float additions: 2e-4.  bfloat16: what rounding alone does depends on the model (these
small ones, with unit-norm keys, exponential gates and multipliers near one, are touchy: 1 to 13 % on the worst row),
so it is measured: the plain implementation is run once more with the operands and results of its products rounded
to bfloat16 values, and the engine may be three times as far from the exact logits as that run is (at least 2e-2).
A lost key, state or sink moves the logits by their own size.
"""
import numpy as np
import pytest
import torch

import plain_panupel as plain
from panupel_models import CONFIGS, delta, make_weights, parallel, rel_error, write_model, _config, _left

pytestmark = pytest.mark.gpu

BOUND_F32 = 2e-4
_cache = {}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """name -> (config, weights, model folder)."""
    base = tmp_path_factory.mktemp("panupel")
    out = {}
    for i, (name, cfg) in enumerate(sorted(CONFIGS.items())):
        w = make_weights(cfg, seed=100 + i)
        out[name] = (cfg, w, write_model(cfg, w, str(base / name)))
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
        _cache[key] = [plain.forward(cfg, w, ids)[0].numpy(), None]
    return _cache[key][0]


def _bound(cfg, w, ids, dtype):
    if dtype == "float32":
        return BOUND_F32
    want = _want(cfg, w, ids)
    entry = _cache[(id(w), tuple(ids))]
    if entry[1] is None:
        entry[1] = rel_error(plain.forward_rounded(cfg, w, ids)[0].numpy(), want)
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
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_whole_prompts_and_first_tokens(models, name, dtype):
    cfg, w, path = models[name]
    eng = _engine(path, dtype)
    for i, n in enumerate([1, 2, 5, 33, 150]):
        ids = _tokens(cfg, n, seed=i)
        _check(_run_cuts(eng, f"r{i}", ids, [n]), (cfg, w), ids, dtype, f"{name}: whole prompt of {n}")
    eng.cache.alloc.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_prompt_then_single_tokens(models, name, dtype):
    """Most of the request in one step, the last 40 tokens one by one (the later ones replay a recorded graph)."""
    cfg, w, path = models[name]
    eng = _engine(path, dtype)
    ids = _tokens(cfg, 131, seed=7)
    got = _run_cuts(eng, "r", ids, [91] + [1] * 40)
    _check(got, (cfg, w), ids, dtype, f"{name}: prompt + 40 single tokens")
    assert eng.graph_replays > 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_portions_of_changing_size(models, name, dtype):
    cfg, w, path = models[name]
    eng = _engine(path, dtype)
    ids = _tokens(cfg, 101, seed=11)
    for cuts in ([24, 24, 24, 24, 5], [2, 3, 17, 16, 15, 31, 2, 13, 2], [1, 2, 1, 3, 94], [64, 37], [16, 16, 32, 1, 1, 35]):
        assert sum(cuts) == len(ids)
        _check(_run_cuts(eng, "r", ids, cuts), (cfg, w), ids, dtype, f"{name}: portions {cuts}")
    eng.cache.alloc.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
def test_first_tokens_in_every_division(models, name, dtype):
    """The first few tokens of a request, where a convolution still reads zeros and the matrix memory's
    stabiliser still sits at its start value, cut in every way."""
    cfg, w, path = models[name]
    eng = _engine(path, dtype)
    ids = _tokens(cfg, 6, seed=13)
    for cuts in ([1] * 6, [2, 2, 2], [1, 5], [5, 1], [3, 1, 2], [6]):
        _check(_run_cuts(eng, "r", ids, cuts), (cfg, w), ids, dtype, f"{name}: first tokens as {cuts}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_mixed_batches_with_pages_and_slots_used_again(models, name, dtype):
    """Up to four live requests (the engine has four state slots), portions of some beside single tokens of others;
    the pool holds 12 pages of 16 tokens for requests that need 24 in all, pages poisoned.  Each request's rows must
    equal what it gives alone."""
    from sandyrt_b200.engine.step import StepEntry

    cfg, w, path = models[name]
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
    """Unequal requests in one step against each alone: same rows, beyond rounding (float32: the same bits are
    not promised, the same numbers to 1e-5 are)."""
    from sandyrt_b200.engine.step import StepEntry

    cfg, w, path = models["B"]
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
    """300 single tokens behind a short prompt, pages of 8: every page border is crossed by a decoded token, and the
    recurrent states are carried through hundreds of steps."""
    cfg, w, path = models["A"]
    eng = _engine(path, dtype, max_tokens=512, page_size=8)
    ids = _tokens(cfg, 310, seed=3)
    got = _run_cuts(eng, "r", ids, [10] + [1] * 300)
    _check(got, (cfg, w), ids, dtype, "A: 300 decoded tokens")


# ---- single mechanisms --------------------------------------------------------------------------------
def _one_model(tmp_path, cfg, seed, bend=None):
    w = make_weights(cfg, seed)
    if bend:
        bend(w)
        w = {k: v.to(torch.bfloat16).to(torch.float32) for k, v in w.items()}
    return w, write_model(cfg, w, str(tmp_path / f"m{seed}"))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["attention", "matrix_memory", "delta"])
def test_each_mixer_alone(tmp_path, which, dtype):
    """One layer, no feed-forward; for the parallel layer one side's scale is zero, so the other stands alone."""
    if which == "delta":
        cfg = _config(61, 48, [delta(3, 1, 24, 20, 3)], eps=1e-5, mult=1.0)
    else:
        cfg = _config(61, 48, [parallel(_left(3, 1, 16, 32, rot={"dims": 12, "base": 30.0}), {"heads": 2, "dim": 24, "vdim": 40, "gate_cap": 6.0},
                                        left_scale=1.3 if which == "attention" else 0.0,
                                        right_scale=0.0 if which == "attention" else 0.9)], eps=1e-5, mult=1.0)
    w, path = _one_model(tmp_path, cfg, seed=5)
    eng = _engine(path, dtype)
    ids = _tokens(cfg, 90, seed=1)
    _check(_run_cuts(eng, "r", ids, [90]), (cfg, w), ids, dtype, f"{which} alone, whole")
    _check(_run_cuts(eng, "r", ids, [40, 2, 30] + [1] * 18), (cfg, w), ids, dtype, f"{which} alone, in portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_key_among_hundreds_and_the_sink(tmp_path, dtype):
    """Attention alone, 400 tokens.  The query projection is scaled up so that scores are sharp: every query then
    looks at one or two keys, mostly far back, and a key that is lost or shifted by one changes the logits by far
    more than the bound.  Then the sinks are raised until they take most of the weight: leaving them out would
    multiply the attention's output several times."""
    cfg = _config(53, 64, [parallel(_left(4, 2, 16, 16, rot={"dims": 16, "base": 10000.0}, scale=1.0), {"heads": 1, "dim": 8, "vdim": 8, "gate_cap": 5.0},
                                    left_scale=1.0, right_scale=0.0)], eps=1e-5, mult=1.0)

    def sharp(w):
        w["l0.mix.left.q"] *= 6.0

    def sunk(w):
        w["l0.mix.left.sink"] = torch.full((4,), 6.0)

    for bend, what in ((sharp, "sharp scores"), (sunk, "heavy sinks")):
        w, path = _one_model(tmp_path, cfg, seed=9 if bend is sharp else 10, bend=bend)
        ids = _tokens(cfg, 400, seed=2)
        want = _want(cfg, w, ids)
        if bend is sunk:       # the sink matters: without it the logits are somewhere else entirely
            w2 = dict(w)
            w2["l0.mix.left.sink"] = torch.full((4,), -30.0)
            assert rel_error(_want(cfg, w2, ids), want) > 0.2
        eng = _engine(path, dtype, max_tokens=512, page_size=16)
        _check(_run_cuts(eng, "r", ids, [400]), (cfg, w), ids, dtype, f"{what}, whole")
        _check(_run_cuts(eng, "r", ids, [250, 100, 18] + [1] * 32), (cfg, w), ids, dtype, f"{what}, portions and single tokens")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_recurrences_that_remember_the_first_token(tmp_path, dtype):
    """Forget gates and decays pushed to one: what the first tokens wrote still dominates the state 200 tokens
    later, so a state that is lost, zeroed or mixed up between requests shows at the end."""
    cfg = _config(47, 40, [delta(2, 2, 16, 12, 2), parallel(_left(1, 1, 16, 16), {"heads": 2, "dim": 16, "vdim": 12, "gate_cap": 9.0},
                                                            left_scale=0.0, right_scale=1.0)], eps=1e-5, mult=1.0)

    def remember(w):
        w["l0.mix.A_log"] = torch.full((2,), -6.0)
        w["l1.mix.right.f.b"] = torch.full((2,), 8.0)
        w["l1.mix.right.i.b"] = torch.full((2,), -2.0)

    w, path = _one_model(tmp_path, cfg, seed=12, bend=remember)
    a, b = _tokens(cfg, 200, seed=5), _tokens(cfg, 200, seed=6)
    c = [b[0]] + a[1:]                                    # differs from a only in its first token
    wa, wc = _want(cfg, w, a), _want(cfg, w, c)
    assert rel_error(wc[-1:], wa[-1:]) > 0.05               # the first token still matters at the end
    from sandyrt_b200.engine.step import StepEntry
    eng = _engine(path, dtype, max_requests=2)
    # two requests side by side, cut differently; then a third in the slot of the first
    got = {0: [], 1: []}
    pa = pb = 0
    for na, nb in [(30, 1), (1, 60), (69, 39), (1, 1)] + [(1, 1)] * 99:
        out = eng.step([StepEntry("a", a[pa:pa + na], list(range(na))), StepEntry("b", b[pb:pb + nb], list(range(nb)))]).cpu().numpy()
        got[0].append(out[:na].copy())
        got[1].append(out[na:].copy())
        pa, pb = pa + na, pb + nb
    assert pa == 200 and pb == 200
    _check(np.concatenate(got[0]), (cfg, w), a, dtype, "request a beside b")
    _check(np.concatenate(got[1]), (cfg, w), b, dtype, "request b beside a")
    eng.release("a")
    _check(_run_cuts(eng, "c", c, [200]), (cfg, w), c, dtype, "request c in a's slot")


# ---- the entry point --------------------------------------------------------------------------------------
def test_greedy_generation_through_the_entry_point(models):
    """LLM.generate (scheduler, prompt portions, decode bursts) on three requests at once, float32: the same tokens
    as greedy decoding with the plain implementation, wherever its top two logits are clearly apart."""
    from sandyrt_b200.engine.llm import LLM

    cfg, w, path = models["A"]
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
