"""Configurations, lively random weights and comparison helpers for the tests of the Sukisun decoder.

The configurations differ from one another in every size: heads that differ between the mixers of one
model, head sizes that are no powers of two, a rotated part of which only some features turn, ranks and
widths that are no multiples of 8, several groups of B and C, norms in two and three parts, convolutions of
two, three and five taps, a model that begins with a recurrence, layers that read another layer's cache.
"""
import json
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "plain"))
import sukisun_plain as plain  # noqa: E402

TOL_F32 = 3e-5
TOL_BF16 = 4e-2


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base=10000.0, dims=None, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale,
         "rot": {"base": base, "dims": rot_dim if dims is None else dims}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def mamba(heads, vdim, state, groups=1, conv=4, norm_groups=1):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def layer(kind, mixer, ff=None):
    return {"type": kind, "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def config(vocab, width, scale, eps, layers):
    return {"architecture": "Sukisun", "vocab": vocab, "width": width, "embedding": {"scale": scale}, "norm": {"eps": eps},
            "layers": layers}


# odd sizes everywhere; begins with a recurrence; layers 2 and 5 read layer 1's cache with heads of their own
ODD = config(211, 72, 3.0, 1e-6, [
    layer("mamba2", mamba(4, 12, 20, groups=2, conv=3, norm_groups=2), ff=100),
    layer("latent_attention", latent(3, 8, 12, 20, 24, 40, 0.3, base=100.0, dims=8)),
    layer("latent_attention", latent(5, 16, 12, 8, 32, 40, 0.2, base=100.0, dims=8, kv_from=1), ff=64),
    layer("mamba2", mamba(2, 24, 9, groups=1, conv=2, norm_groups=3)),
    layer("latent_attention", latent(2, 24, 6, 16, 16, 26, 0.25, base=5000.0), ff=48),
    layer("latent_attention", latent(3, 8, 12, 20, 24, 40, 0.3, base=100.0, dims=8, kv_from=1)),
])
# sharp attention: a large score scale makes every softmax pick out single keys, most of them far back
SHARP = config(150, 64, 2.0, 1e-5, [
    layer("latent_attention", latent(4, 16, 16, 16, 32, 32, 3.0), ff=96),
    layer("latent_attention", latent(4, 16, 16, 16, 32, 32, 3.0, kv_from=0)),
    layer("latent_attention", latent(2, 8, 24, 32, 16, 48, 2.0, base=300.0), ff=96),
])
# sizes in multiples of 64: in bfloat16 the products of few-token steps run this package's tensor-core kernels,
# whose partial sums the kernels behind them add up
EVEN = config(320, 128, 8.0, 1e-5, [
    layer("latent_attention", latent(4, 32, 32, 64, 64, 64, 0.125), ff=256),
    layer("mamba2", mamba(8, 16, 64, groups=2, conv=5, norm_groups=4), ff=256),
    layer("latent_attention", latent(4, 32, 32, 64, 64, 64, 0.125, kv_from=0)),
    layer("mamba2", mamba(4, 64, 16, groups=4, conv=4, norm_groups=1)),
])
CONFIGS = {"odd": (ODD, 8), "sharp": (SHARP, 16), "even": (EVEN, 16)}        # name -> (config, page size)


def lively_tensors(cfg_json, seed, dtype):
    """Random weights under which every mechanism matters: matrices of unit gain, decays and step sizes spread
    over their ranges, skip weights, activation numbers and depth weights away from their neutral values.  The
    names and shapes come from the framework's loader; the values are drawn here."""
    from beglin_b200.config import load_config
    from beglin_b200.weights import expected_tensors
    arch, cfg = load_config(dict(cfg_json))
    spec = arch.build_spec(cfg)
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, role in expected_tensors(spec).items():
        shape = tuple(role.shape)
        r = lambda *s: torch.randn(*s, generator=g)
        u = lambda lo, hi: lo + (hi - lo) * torch.rand(shape, generator=g)
        if name == "embed":
            t = r(*shape) * 0.5
        elif name.endswith(".A_log"):
            t = u(-1.5, 1.0)
        elif name.endswith(".dt_bias"):
            t = u(-3.0, 1.0)
        elif name.endswith(".mix.D"):
            t = 1.0 + 0.5 * r(*shape)
        elif name.endswith(".mlp.act"):
            t = torch.tensor([0.3, -0.4]) + 0.5 * r(*shape)
        elif name.endswith(".dwa"):
            t = 0.25 * r(*shape)
            t[-1] += 1.0
        elif name.endswith(".conv"):
            t = 0.5 * r(*shape)
        elif name.endswith(".conv.b"):
            t = 0.2 * r(*shape)
        elif len(shape) == 1:                       # norm weights
            t = 1.0 + 0.2 * r(*shape)
        else:
            t = r(*shape) * (1.2 / shape[1] ** 0.5)
        out[name] = t.to(dtype)
    return out


def make_model(root, name, seed=0, dtype=torch.float32, config_json=None):
    """Write a model folder with lively random weights under `root` and return its path."""
    from beglin_b200.weights import write_safetensors
    cfg = CONFIGS[name][0] if config_json is None else config_json
    folder = os.path.join(str(root), f"sukisun_{name}_{seed}_{str(dtype).split('.')[-1]}")
    if not os.path.exists(os.path.join(folder, "model.safetensors")):
        os.makedirs(folder, exist_ok=True)
        with open(os.path.join(folder, "config.json"), "w") as f:
            json.dump(cfg, f, indent=1)
        write_safetensors(os.path.join(folder, "model.safetensors"), lively_tensors(cfg, seed, dtype))
    return folder


_CACHE = {}


def plain_logits(folder, ids):
    """float64 logits [T, vocab] of the whole sequence from the plain implementation."""
    if folder not in _CACHE:
        _CACHE[folder] = plain.read_folder(folder, torch.float64)
    key = (folder, tuple(ids))
    if key not in _CACHE:
        cfg, w = _CACHE[folder]
        _CACHE[key] = plain.forward(cfg, w, list(ids))
    return _CACHE[key]


def rel_err(got, want):
    want = want.to(torch.float64).cpu()
    got = got.to(torch.float64).cpu()
    return float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))


def seeded_ids(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def check_against_plain(got, folder, reqs, tol):
    """got: {(request, position): logits row}; every position of every request against the plain logits."""
    worst = 0.0
    for rid, ids in reqs.items():
        want = plain_logits(folder, ids)
        rows = torch.stack([got[(rid, p)] for p in range(len(ids))])
        assert torch.isfinite(rows).all(), rid
        err = rel_err(rows, want)
        if err > tol:
            per_pos = (rows.double() - want).abs().max(dim=1).values / want.abs().max()
            first = int((per_pos > tol).nonzero()[0])
            raise AssertionError(f"{rid}: relative error {err:.3g} > {tol:g}; first wrong position {first} of {len(ids)}")
        worst = max(worst, err)
    return worst


def poison(engine):
    """NaN in every page and every state slot: a read of something that was never written, or of what an
    earlier request left, shows.  (A slot is zeroed when a request starts.)"""
    for g in engine.cache.kv_groups:
        g.device_pool.fill_(float("nan"))
    for g in engine.cache.state_groups:
        g.slab.fill_(float("nan"))
