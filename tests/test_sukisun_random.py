"""Seeded random configurations of the Sukisun decoder: widths, heads, head sizes, ranks, partly rotated key parts,
layers that borrow a cache, recurrences with several groups, norm parts and one to six taps, layers with and without
a feed-forward, in every order.  Each runs five requests whole and mixed (four live at a time on a small pool) in both
number formats against the plain implementation; in float32 the two ways agree bit for bit."""
import random

import pytest
import torch

import replay_lib as rl
from sukisun_helpers import config, latent, layer, make_model, mamba, plain_logits, poison, rel_err, seeded_ids

pytestmark = pytest.mark.gpu


def random_config(case):
    """A pure function of the case number."""
    r = random.Random(case)
    width = r.choice([48, 64, 72, 96, 100, 128, 136, 160, 192, 256])
    n = r.randint(2, 8)
    families = []                                   # latent sizes that layers of one cache share
    for _ in range(2):
        rot = r.choice([8, 16, 32, 64])
        rank = r.choice([16, 24, 32, 48, 56, 64, 96, 128, 30])
        if r.random() < 0.5 and (rank + rot) % 32:          # often a cached row of a multiple of 32 features
            rank = max(32, (rank + rot + 31) // 32 * 32 - rot)
        dims = rot if r.random() < 0.6 else r.choice(list(range(0, rot + 1, 2)))
        families.append(dict(rot=rot, rank=rank, dims=dims, base=r.choice([100.0, 10000.0, 500000.0]), owner=None))
    layers = []
    for i in range(n):
        if r.random() < 0.3:
            heads = r.choice([1, 2, 3, 4, 6, 8])
            groups = r.choice([g for g in (1, 2, 3, 4) if heads % g == 0])
            vdim = r.choice([8, 12, 16, 32, 64, 80, 96])
            parts = r.choice([g for g in (1, 2, 3, 4, 8) if (heads * vdim) % g == 0])
            m = mamba(heads, vdim, r.choice([4, 8, 9, 16, 32, 64, 100, 128]), groups=groups, conv=r.randint(1, 6), norm_groups=parts)
            layers.append(layer("mamba2", m, ff=r.choice([None, 64, 100, 256])))
        else:
            f = r.choice(families)
            heads, dim = r.choice([1, 2, 3, 4, 5, 6, 8, 12]), r.choice([8, 16, 24, 32, 40, 64])
            vdim = dim + f["rot"] if r.random() < 0.4 else r.choice([8, 16, 20, 32, 48, 64, 80, 128])
            kv_from = f["owner"] if f["owner"] is not None and r.random() < 0.5 else None
            m = latent(heads, dim, f["rot"], vdim, r.choice([16, 24, 40, 64, 80, 96]), f["rank"], r.uniform(0.05, 0.3), base=f["base"],
                       dims=f["dims"], kv_from=kv_from)
            if kv_from is None and f["owner"] is None:
                f["owner"] = i
            layers.append(layer("latent_attention", m, ff=r.choice([None, 64, 100, 256, 384])))
    return config(r.randint(50, 700), width, r.uniform(1.0, 16.0), r.choice([1e-5, 1e-6]), layers)


@pytest.mark.parametrize("case", [0, 1, 2, 3, 5, 8, 13, 21])
def test_random_configuration(model_root, case):
    from beglin_b200 import Engine
    cfg = random_config(case)
    reqs = {f"r{i}": seeded_ids(n, cfg["vocab"], 100 * case + i) for i, n in enumerate([150, 40, 9, 200, 66])}
    mixed, peak = rl.mixed(reqs, seed=case)
    for dtype, tol in (("float32", 1e-4), ("bfloat16", 8e-2)):
        stored = torch.float32 if dtype == "float32" else torch.bfloat16
        folder = make_model(model_root, f"random{case}", seed=case, dtype=stored, config_json=cfg)
        res = {}
        for way, steps, tokens in (("whole", rl.whole(reqs), 256), ("mixed", mixed, peak)):
            eng = Engine.from_folder(folder, dtype=dtype, max_tokens=tokens, page_size=16, max_requests=4, kv_split=64)
            poison(eng)
            res[way] = rl.run_in_process(eng, steps)
            eng.cache.check()
            for rid, ids in reqs.items():
                rows = torch.stack([res[way][(rid, p)] for p in range(len(ids))])
                assert torch.isfinite(rows).all(), (dtype, way, rid)
                assert rel_err(rows, plain_logits(folder, ids)) < tol, (dtype, way, rid)
        if dtype == "float32":
            for key, row in res["whole"].items():
                assert torch.equal(row, res["mixed"][key]), key
