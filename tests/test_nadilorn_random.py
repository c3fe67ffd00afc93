"""Random configurations of the Nadilorn decoder: `random_config(case)` is a pure function of the case number and draws
every size, the order of the layers' feed-forwards, the windows and the constants; each case runs whole and mixed with
other requests on a small pool, in float32 (against the oracle and bit for bit between the two ways) and in bfloat16.
The bfloat16 cases draw sizes in multiples of 8 (what the tensor-core products take) and experts of at least 8 inner
features: an expert of five features, of which the square of relu keeps one or two, hands the norm behind it a result
whose rounding error is a large part of it, which is the weights' conditioning and not a kernel's fault."""
import random

import pytest
import torch

import replay_lib as rl
from nadilorn_helpers import TOL_BF16, TOL_F32, attn, check_against_plain, config, dense, layer, make_model, moe, poison, seeded_ids

pytestmark = pytest.mark.gpu


def random_config(case: int, even: bool = False):
    rng = random.Random(1000 + case)
    unit = 8 if even else 1
    width = rng.choice([64, 128, 192]) if even else rng.randrange(24, 100)
    layers = []
    for _ in range(rng.randrange(1, 5)):
        kv = rng.choice([1, 1, 2, 3])
        heads = kv * rng.choice([1, 1, 2, 3, 4])
        dim = rng.choice([32, 64, 128]) if even else 2 * rng.randrange(2, 20)
        vdim = rng.choice([dim, dim, 16, 32, 64]) if even else rng.choice([dim, rng.randrange(1, 40)])
        window = rng.choice([None, 1, 2, rng.randrange(3, 20), rng.randrange(20, 200)])
        rot = rng.choice([0, dim, 2 * rng.randrange(1, dim // 2 + 1)])
        factor = rng.choice([None, 1.0, 2.0, 3.7, 8.0])
        mixer = attn(heads, kv, dim, vdim, rng.uniform(0.3, 2.0) / dim ** 0.5, window=window, rot=rot,
                     base=rng.choice([10.0, 1000.0, 1e6]), factor=factor)
        kind = rng.choice(["dense", "moe", "moe", None])
        if kind == "dense":
            mlp = dense(unit * rng.randrange(2, 30))
        elif kind == "moe":
            experts = rng.randrange(1, 10)
            mlp = moe(experts, rng.randrange(1, experts + 1), unit * rng.randrange(1, 12))
        else:
            mlp = None
        layers.append(layer(mixer, mlp))
    return config(rng.randrange(30, 300), width, rng.choice([1e-6, 1e-5, 1e-3]), layers), rng.choice([4, 8, 16, 32, 64])


@pytest.mark.parametrize("case", range(12))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_random_configuration(model_root, case, dtype):
    cfg, page = random_config(case, even=(dtype == "bfloat16"))
    stored = torch.float32 if dtype == "float32" else torch.bfloat16
    folder = make_model(model_root, f"random{case}", seed=case, dtype=stored, config_json=cfg)
    reqs = {f"r{i}": seeded_ids(n, cfg["vocab"], 7 * case + i) for i, n in enumerate([61, 18, 130, 40, 77])}
    mixed_steps, peak = rl.mixed(reqs, seed=case)
    from beglin_b200 import Engine
    results = {}
    for way, (steps, tokens) in {"whole": (rl.whole(reqs), 192), "mixed": (mixed_steps, peak)}.items():
        eng = Engine.from_folder(folder, dtype=dtype, max_tokens=max(tokens, page), page_size=page, max_requests=4, kv_split=64)
        poison(eng)
        results[way] = rl.run_in_process(eng, steps)
        eng.cache.check()
        check_against_plain(results[way], folder, reqs, TOL_F32 if dtype == "float32" else TOL_BF16)
    if dtype == "float32":
        for key, row in results["whole"].items():
            assert torch.equal(row, results["mixed"][key]), key
