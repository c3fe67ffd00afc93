"""Configurations, lively random weights and comparison helpers for the tests of the Nadilorn decoder.

The configurations differ from one another and from layer to layer in every size: one to four query heads per kv head,
values narrower than, as wide as and wider than keys, head sizes that are no powers of two, windows shorter than a page,
of several pages and none at all, rotation of a part of a head, of all of it and none, frequency divisors, one to all
experts chosen, inner sizes that are no multiples of 8, layers without a feed-forward.
"""
import json
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "plain"))
import nadilorn_plain as plain  # noqa: E402

TOL_F32 = 3e-5
TOL_BF16 = 4e-2
ROUTE_DIMS = 4          # features of the stream that a "decisive" model keeps for its routers alone


def attn(heads, kv_heads, dim, vdim, scale, window=None, rot=None, base=10000.0, factor=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    if rot:
        m["rot"] = {"base": base, "dims": rot}
        if factor is not None:
            m["rot"]["scaling"] = {"factor": factor}
    return m


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def layer(mixer, mlp=None):
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def config(vocab, width, eps, layers):
    return {"architecture": "Nadilorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


# odd sizes everywhere; every layer differs from the others
ODD = config(211, 72, 1e-6, [
    layer(attn(3, 1, 10, 6, 0.4, window=13, rot=6, base=100.0, factor=2.5), dense(100)),
    layer(attn(4, 2, 12, 12, 0.3, window=40, rot=12, base=5000.0), moe(5, 2, 20)),
    layer(attn(2, 2, 16, 24, 0.25)),                                                       # no window, no rotation, no feed-forward
    layer(attn(4, 1, 8, 14, 0.35, window=7, rot=4, base=50.0, factor=3.0), moe(3, 3, 9)),
    layer(attn(3, 3, 6, 2, 0.5, window=100, rot=2, base=10.0, factor=1.5), moe(6, 1, 12)),
])
# sharp attention: a large score scale makes every softmax pick out single keys
SHARP = config(150, 64, 1e-5, [
    layer(attn(4, 2, 16, 8, 2.5, window=150, rot=8, base=1000.0, factor=4.0), dense(96)),
    layer(attn(2, 1, 24, 16, 2.0, window=33, rot=24, base=300.0), moe(4, 2, 24)),
    layer(attn(4, 4, 8, 8, 3.0, rot=4, base=20.0, factor=2.0), dense(48)),
])
# sizes in multiples of 64: in bfloat16 the products run this package's tensor-core kernels, also the experts'
EVEN = config(320, 128, 1e-5, [
    layer(attn(4, 2, 64, 64, 0.125, window=80, rot=32, base=10000.0, factor=4.0), dense(256)),
    layer(attn(4, 1, 64, 32, 0.125, window=70, rot=64, base=10000.0), moe(8, 2, 64)),
    layer(attn(2, 2, 128, 128, 0.09, window=200, rot=64, base=200000.0, factor=16.0), moe(4, 1, 128)),
    layer(attn(8, 2, 32, 64, 0.18, rot=16, base=1000.0, factor=2.0)),
])
CONFIGS = {"odd": (ODD, 8), "sharp": (SHARP, 16), "even": (EVEN, 16)}        # name -> (config, page size)


def lively_tensors(cfg_json, seed, dtype, decisive=False):
    """Random weights under which every mechanism matters: matrices of unit gain, norm weights spread around one,
    routers whose scores differ.  The names and shapes come from the framework's loader; the values are drawn here.

    `decisive`: for runs in a rounded number format, where a router that reads rounded rows could choose another expert
    than the oracle on a close call.  The last ROUTE_DIMS features of the stream then belong to the routers alone: the
    embedding puts small dyadic numbers there, every layer norm's weight is zero there (so no sublayer ever adds to
    them), and a router reads nothing else; its logits are then exact in every format and its choices the oracle's."""
    from beglin_b200.config import load_config
    from beglin_b200.weights import expected_tensors
    arch, cfg = load_config(dict(cfg_json))
    spec = arch.build_spec(cfg)
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, role in expected_tensors(spec).items():
        shape = tuple(role.shape)
        r = lambda *s: torch.randn(*s, generator=g)
        pick = lambda values, *s: torch.tensor(values)[torch.randint(0, len(values), s, generator=g)]
        if name == "embed":
            t = r(*shape) * 0.5
            if decisive:
                t[:, -ROUTE_DIMS:] = pick([-2.0, -1.0, -0.5, 0.5, 1.0, 2.0], shape[0], ROUTE_DIMS)
        elif name.endswith(".router"):
            t = r(*shape) * (3.0 / shape[1] ** 0.5)
            if decisive:
                t = torch.zeros(shape)
                t[:, -ROUTE_DIMS:] = pick([-1.5, -1.0, -0.5, 0.5, 1.0, 1.5], shape[0], ROUTE_DIMS)
        elif len(shape) == 1:                       # norm weights
            t = 1.0 + 0.2 * r(*shape)
            if decisive and (name.endswith(".norm1") or name.endswith(".norm2")):
                t[-ROUTE_DIMS:] = 0.0
        else:
            t = r(*shape) * (1.2 / shape[1] ** 0.5)
        out[name] = t.to(dtype)
    return out


def make_model(root, name, seed=0, dtype=torch.float32, config_json=None, decisive=None):
    """Write a model folder with lively random weights under `root` and return its path.  A folder stored in bfloat16
    gets decisive routers unless told otherwise."""
    from beglin_b200.weights import write_safetensors
    cfg = CONFIGS[name][0] if config_json is None else config_json
    decisive = (dtype != torch.float32) if decisive is None else decisive
    folder = os.path.join(str(root), f"nadilorn_{name}_{seed}_{str(dtype).split('.')[-1]}_{int(decisive)}")
    if not os.path.exists(os.path.join(folder, "model.safetensors")):
        os.makedirs(folder, exist_ok=True)
        with open(os.path.join(folder, "config.json"), "w") as f:
            json.dump(cfg, f, indent=1)
        write_safetensors(os.path.join(folder, "model.safetensors"), lively_tensors(cfg, seed, dtype, decisive))
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
    """NaN in every page: a read of something that was never written, or of what an earlier request left, shows."""
    for g in engine.cache.kv_groups:
        g.device_pool.fill_(float("nan"))
    for g in engine.cache.state_groups:
        g.slab.fill_(float("nan"))
