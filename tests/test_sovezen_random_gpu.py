"""Sovezen configurations drawn at random against the plain implementation: sizes that divide by nothing (odd head
sizes, latents and widths, 33 experts), one to four layers of either form with any feed-forward, layers on other
layers' tensors.  Every configuration runs whole, as a prompt with 32 single tokens behind it, and in portions, in
float32 (2e-4) and in bfloat16 (three times what rounding alone does; routers whose choices no rounding can turn)."""
import random

import numpy as np
import pytest
import torch

import plain_sovezen as plain
from sovezen_models import _config, dense, layer, make_weights, moe, plain_queries, rel_error, rotated, write_model

pytestmark = pytest.mark.gpu


def rand_cfg(rng):
    width = rng.choice([40, 48, 72, 90, 100, 128, 66])
    n_layers = rng.randint(1, 4)
    layers = []
    for i in range(n_layers):
        if layers and rng.random() < 0.25:
            j = rng.randrange(len(layers))
            while 'weights_of' in layers[j]: j = layers[j]['weights_of']
            l = {k: v for k, v in layers[j].items()}
            l = layer({'type': l['type'], 'mixer': l['mixer']}, l['mlp'], weights_of=j)
            layers.append(l); continue
        H = rng.choice([1, 2, 3, 4, 5, 8, 16])
        d = rng.choice([8, 15, 16, 24, 32, 40])
        e = rng.choice([7, 8, 16, 24, 48])
        c = rng.choice([12, 16, 21, 32, 48, 64, 100])
        if rng.random() < 0.5:
            r = rng.choice([2, 6, 8, 16, 32, 5])
            dims = r - (r % 2) if rng.random() < 0.7 else max(2, (r // 2) - ((r // 2) % 2))
            m = rotated(H, d, r, e, c, base=rng.choice([10.0, 1000.0, 1e6]), dims=dims)
        else:
            m = plain_queries(H, d, e, c, rng.choice([8, 9, 24, 40]))
        k = rng.random()
        if k < 0.4: f = dense(rng.choice([16, 30, 64, 11]))
        elif k < 0.85:
            E = rng.choice([2, 3, 8, 16, 33]); f = moe(E, rng.randint(1, min(E, 6)), rng.choice([8, 12, 16, 9]))
        else: f = None
        layers.append(layer(m, f))
    return _config(rng.choice([50, 97, 200]), width, layers, eps=rng.choice([1e-5, 1e-6]), logit_scale=rng.choice([0.25, 1.0, 1.7]))


@pytest.mark.parametrize("seed", range(20))
def test_random_configuration(tmp_path, seed):
    from sandyrt_b200.engine.step import Engine, StepEntry
    from sandyrt_b200.models.model import load_model

    cfg = rand_cfg(random.Random(seed))
    ids = np.random.default_rng(seed).integers(0, cfg["vocab"], size=97).tolist()
    for dtype in ("float32", "bfloat16"):
        w = make_weights(cfg, seed=seed, decisive_router=dtype == "bfloat16")
        path = write_model(cfg, w, str(tmp_path / dtype))
        eng = Engine(load_model(path, device="cuda:0", dtype=getattr(torch, dtype)), max_tokens=512, page_size=16, max_requests=4)
        eng.cache.device_caches.poison()
        want = plain.forward(cfg, w, ids).numpy()
        bound = 2e-4 if dtype == "float32" else max(2e-2, 3 * rel_error(plain.forward_rounded(cfg, w, ids).numpy(), want))
        for cuts in ([97], [40, 2, 23] + [1] * 32, [3, 17, 64, 13]):
            rows, pos = [], 0
            for n in cuts:
                rows.append(eng.step([StepEntry("r", ids[pos:pos + n], list(range(n)))]).cpu().numpy().copy())
                pos += n
            eng.check_status()
            eng.release("r")
            e = rel_error(np.concatenate(rows), want)
            assert e < bound, f"{dtype}, portions {cuts[:4]}: relative error {e:.3e} (bound {bound:.1e}); layers {cfg['layers']}"
