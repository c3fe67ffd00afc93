"""The Nadilorn decoder's configuration reader, its description as parts, the tensors it asks for and the cache needs of
its layers; and the plain implementation's small functions against closed forms.  No GPU."""
import copy
import math

import pytest
import torch

from nadilorn_helpers import CONFIGS, ODD, attn, config, dense, layer, lively_tensors, moe, plain

from beglin_b200.config import ConfigError, load_config
from beglin_b200.parts.cache_need import PagedKVNeed
from beglin_b200.weights import expected_tensors


def test_reads_every_size_and_constant():
    arch, cfg = load_config(dict(ODD))
    assert arch.name == "Nadilorn" and cfg.vocab == 211 and cfg.width == 72 and cfg.norm_eps == 1e-6
    m0, m2 = cfg.layers[0].mixer, cfg.layers[2].mixer
    assert (m0.heads, m0.kv_heads, m0.dim, m0.vdim, m0.window, m0.rot_dims, m0.rot_base, m0.rot_factor, m0.scale) == \
        (3, 1, 10, 6, 13, 6, 100.0, 2.5, 0.4)
    assert m2.window is None and m2.rot_dims == 0 and cfg.layers[2].mlp is None
    assert cfg.layers[1].mixer.rot_factor == 1.0                      # no scaling key: the frequencies as they are
    f1, f3 = cfg.layers[1].mlp, cfg.layers[3].mlp
    assert (f1.kind, f1.experts, f1.top, f1.ff) == ("moe", 5, 2, 20) and (f3.experts, f3.top, f3.ff) == (3, 3, 9)
    assert cfg.layers[0].mlp.kind == "dense" and cfg.layers[0].mlp.ff == 100
    assert cfg.to_json_dict() == ODD                                   # and back


def test_spec_carries_the_options():
    arch, cfg = load_config(dict(ODD))
    spec = arch.build_spec(cfg)
    assert [l.block for l in spec.layers] == ["postnorm", "postnorm", "postnorm_mixer", "postnorm", "postnorm"]
    a = spec.layers[0].mixer
    assert a.sink and a.gate == "elementwise" and a.qk_norm == "projection" and a.qk_norm_eps == 1e-6
    assert (a.head_dim, a.value_dim, a.window, a.scale) == (10, 6, 13, 0.4)
    assert a.position.pairing == "split_half" and a.position.rotary_dim == 6 and a.position.freq_divisor == 2.5
    assert spec.layers[2].mixer.position.kind == "none" and spec.layers[2].mixer.window is None
    assert spec.layers[0].feed_forward.activation == "gelu_tanh"
    r = spec.layers[3].feed_forward
    assert (r.experts, r.top, r.intermediate, r.activation, r.renormalize, r.scale_input) == (3, 3, 9, "relu2", False, True)
    assert spec.head_name == "head" and spec.final_norm.kind == "rmsnorm"


def test_tensor_names_and_shapes():
    arch, cfg = load_config(dict(ODD))
    t = expected_tensors(arch.build_spec(cfg))
    assert tuple(t["l0.mix.q"].shape) == (30, 72) and tuple(t["l0.mix.k"].shape) == (10, 72)
    assert tuple(t["l0.mix.v"].shape) == (6, 72) and tuple(t["l0.mix.g"].shape) == (18, 72) and tuple(t["l0.mix.o"].shape) == (72, 18)
    assert tuple(t["l0.mix.q.norm"].shape) == (30,) and tuple(t["l0.mix.k.norm"].shape) == (10,)
    assert tuple(t["l1.mlp.router"].shape) == (5, 72) and tuple(t["l1.mlp.e4.up"].shape) == (20, 72)
    assert tuple(t["l1.mlp.e0.down"].shape) == (72, 20) and "l1.mlp.e5.up" not in t
    assert tuple(t["l0.mlp.gate"].shape) == (100, 72) and tuple(t["l0.mlp.down"].shape) == (72, 100)
    assert "l2.norm2" not in t and "l2.norm1" in t and not any(n.startswith("l2.mlp") for n in t)
    assert tuple(t["head"].shape) == (211, 72) and tuple(t["final.norm"].shape) == (72,) and tuple(t["embed"].shape) == (211, 72)


def test_cache_needs_follow_the_layers():
    from beglin_b200.parts import registry
    arch, cfg = load_config(dict(ODD))
    spec = arch.build_spec(cfg)
    needs = [registry.mixer_class(l.mixer.kind).cache_need(l.mixer) for l in spec.layers]
    assert needs[0] == PagedKVNeed(1, 10, 13, 6) and needs[1] == PagedKVNeed(2, 12, 40, None)
    assert needs[2] == PagedKVNeed(2, 16, None, 24)
    assert needs[1].page_shape(8) == (2, 2, 8, 12)                    # values as wide as keys: the common layout
    assert needs[0].page_shape(8) == (1 * 8 * (10 + 6),)              # else flat: keys, then values


@pytest.mark.parametrize("change,what", [
    (lambda c: c["layers"][0].__setitem__("type", "conv"), "type"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("kv_heads", 2), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 5), "even"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 12), "at most"),
    (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 6), "exceeds"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "glu"), "kind"),
    (lambda c: c["layers"][0]["mixer"].pop("vdim"), "vdim"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.__setitem__("layers", []), "empty"),
    (lambda c: c["layers"][0]["mixer"]["mask"].__setitem__("size", 0), "positive"),
])
def test_bad_configurations_are_refused(change, what):
    c = copy.deepcopy(ODD)
    change(c)
    with pytest.raises(ConfigError) as e:
        load_config(c)
    assert what in str(e.value)


def test_decisive_weights_keep_the_routing_features():
    t = lively_tensors(CONFIGS["odd"][0], 1, torch.bfloat16, decisive=True)
    assert float(t["l1.norm1"][-4:].abs().max()) == 0.0 and float(t["l1.mlp.router"][:, :-4].abs().max()) == 0.0


# ----------------------------------------------------------------------------- the oracle's small functions
def test_plain_sink_softmax():
    s = torch.tensor([0.3, -1.2, 2.0], dtype=torch.float64)
    p = plain.sink_softmax(s)
    assert torch.allclose(p, torch.exp(s) / (1.0 + torch.exp(s).sum()))
    assert float(p.sum()) < 1.0
    big = plain.sink_softmax(torch.tensor([800.0, 799.0], dtype=torch.float64))        # no overflow
    assert torch.isfinite(big).all() and abs(float(big.sum()) - 1.0) < 1e-12
    small = plain.sink_softmax(torch.tensor([-800.0], dtype=torch.float64))            # all the weight stays with the sink
    assert float(small[0]) == 0.0


def test_plain_rotation_is_a_rotation_in_halves():
    v = torch.randn(3, 2, 10, dtype=torch.float64)
    out = plain.turn_halves(v, [0, 5, 9], 100.0, 6, 2.0)
    assert torch.equal(out[0], v[0]) and torch.equal(out[:, :, 6:], v[:, :, 6:])       # position 0 and the features beyond
    a = 5 * 100.0 ** (-2.0 * 1 / 6) / 2.0                                              # pair (1, 4) at position 5
    assert torch.allclose(out[1, :, 1], v[1, :, 1] * math.cos(a) - v[1, :, 4] * math.sin(a))
    assert torch.allclose(out[1, :, 4], v[1, :, 4] * math.cos(a) + v[1, :, 1] * math.sin(a))
    assert torch.allclose((out[..., :6] ** 2).sum(-1), (v[..., :6] ** 2).sum(-1))


def test_plain_experts_scale_the_input():
    torch.manual_seed(0)
    d, ff, E = 6, 5, 4
    w = {"router": torch.randn(E, d, dtype=torch.float64)}
    for e in range(E):
        w[f"e{e}.up"], w[f"e{e}.down"] = torch.randn(ff, d, dtype=torch.float64), torch.randn(d, ff, dtype=torch.float64)
    h = torch.randn(3, d, dtype=torch.float64)
    out = plain.routed_experts(w, "", h, E, 2)
    s = torch.sigmoid(h @ w["router"].T)
    for t in range(3):
        top = torch.topk(s[t], 2).indices.tolist()
        # the square of relu is homogeneous of degree two: scaling the input by s scales the result by s^2
        want = sum(s[t, e] ** 2 * (torch.clamp(h[t] @ w[f"e{e}.up"].T, min=0) ** 2) @ w[f"e{e}.down"].T for e in top)
        assert torch.allclose(out[t], want)


def test_plain_gelu():
    z = torch.linspace(-4, 4, 9, dtype=torch.float64)
    assert torch.allclose(plain.gelu_tanh(z), torch.nn.functional.gelu(z, approximate="tanh"))
