"""The Sukisun configuration and description without a GPU: config.json keys and their checks, the run order with
shared caches, what the cache manager is asked for, the loader's names, and the plain implementation against
itself where two of its functions must agree."""
import copy
import json
import os

import pytest
import torch

from sukisun_helpers import CONFIGS, EVEN, ODD, lively_tensors, make_model, plain, seeded_ids


def load(cfg):
    from beglin_b200.config import load_config
    arch, c = load_config(copy.deepcopy(cfg))
    return arch, c, arch.build_spec(c)


def test_registry_reads_the_architecture_string():
    arch, c, spec = load(ODD)
    assert arch.name == "Sukisun" and c.vocab == 211 and c.width == 72 and len(c.layers) == 6
    assert c.to_json_dict() == ODD
    assert spec.embed_scale == 3.0 and spec.head_name is None and spec.final_norm.kind == "layernorm"


def test_run_order_shares_caches_and_layers_differ():
    from beglin_b200.parts import FixedStateNeed, PagedLatentNeed, registry
    from beglin_b200.cache import CacheManager
    _, _, spec = load(ODD)
    assert [(s.layer, s.cache) for s in spec.order] == [(0, None), (1, None), (2, 1), (3, None), (4, None), (5, 1)]
    assert [l.block for l in spec.layers] == ["prenorm_combined", "prenorm_mixer_combined", "prenorm_combined",
                                              "prenorm_mixer_combined", "prenorm_combined", "prenorm_mixer_combined"]
    assert [l.combiner.terms for l in spec.layers] == [2, 3, 4, 5, 6, 7] and spec.layers[0].combiner.total == 7
    assert spec.layers[2].mixer.own_kv is False and spec.layers[2].mixer.n_heads == 5
    assert spec.layers[1].mixer.position.rotary_dim == 8 and spec.layers[1].mixer.position.pairing == "interleaved"
    needs = []
    for st in spec.order:
        need = None
        if st.cache is None:
            for _, family, cls, pspec in registry.layer_slots(spec.layers[st.layer]):
                if family == "mixer":
                    need = cls.cache_need(pspec)
        needs.append(need)
    assert needs[1] == PagedLatentNeed(52) and needs[4] == PagedLatentNeed(32) and needs[2] is None and needs[5] is None
    assert isinstance(needs[0], FixedStateNeed) and needs[0].shape == (4 * 20 * 12 + 2 * 128,)
    cache = CacheManager(needs, page_size=8, num_pages=6, max_requests=2)
    assert len(cache.kv_groups) == 2 and len(cache.state_groups) == 2
    cache.allocate("cpu", torch.bfloat16)
    assert tuple(cache.kv_groups[0].device_pool.shape) == (1, 7, 8, 52)
    assert cache.state_groups[0].slab.dtype == torch.float32 and cache.state_groups[0].slab.shape[:2] == (1, 3)
    cache.add_request("a")
    cache.reserve([("a", 20)])
    cache.commit([("a", 20)])
    assert cache.pages_held("a") == 3
    cache.release("a")
    cache.check()


@pytest.mark.parametrize("change,match", [
    (lambda c: c["layers"][2]["mixer"].update(kv_from=3), "kv_from"),               # names a recurrence
    (lambda c: c["layers"][2]["mixer"].update(kv_from=2), "kv_from"),               # names itself
    (lambda c: c["layers"][5]["mixer"].update(kv_from=2), "kv_from"),               # names a layer that borrows too
    (lambda c: c["layers"][2]["mixer"].update(kv_rank=48), "differ"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=14), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"].update(groups=3), "groups"),
    (lambda c: c["layers"][0]["mixer"].update(norm_groups=5), "norm_groups"),
    (lambda c: c["layers"][0].update(type="rwkv"), "not known"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "not known"),
    (lambda c: c["layers"][1]["mixer"].pop("vdim"), "vdim"),
    (lambda c: c.update(layers=[]), "empty"),
    (lambda c: c.pop("embedding"), "embedding"),
    (lambda c: c.update(width="72"), "not a number"),
])
def test_configurations_that_are_refused(change, match):
    from beglin_b200.config import ConfigError
    cfg = copy.deepcopy(ODD)
    change(cfg)
    with pytest.raises(ConfigError, match=match):
        load(cfg)


def test_weights_bind_by_name_and_misfits_are_listed(tmp_path):
    from beglin_b200.weights import Checkpoint, WeightError, bind, write_safetensors
    folder = make_model(tmp_path, "odd", seed=1, dtype=torch.bfloat16)
    _, _, spec = load(ODD)
    ck = Checkpoint(folder)
    bound = bind(spec, ck, folder)
    assert "l2.mix.dkv" not in bound and "l1.mix.dkv" in bound and "l3.mlp.up" not in bound and "l5.dwa" in bound
    assert tuple(bound["l2.mix.uk"].shape) == (5 * 16, 40) and bound["l0.mix.A_log"].dtype == torch.bfloat16
    ck.close()
    t = lively_tensors(ODD, 1, torch.bfloat16)
    del t["l4.mix.g"]
    t["l2.mix.dkv"] = torch.zeros(52, 72, dtype=torch.bfloat16)
    t["l0.dwa"] = torch.zeros(3, dtype=torch.bfloat16)
    bad = tmp_path / "bad"
    os.makedirs(bad)
    write_safetensors(str(bad / "model.safetensors"), t)
    with open(bad / "config.json", "w") as f:
        json.dump(ODD, f)
    ck = Checkpoint(str(bad))
    with pytest.raises(WeightError) as e:
        bind(spec, ck, str(bad))
    assert e.value.missing == ["l4.mix.g"] and e.value.unexpected == ["l2.mix.dkv"] and e.value.wrong_shape[0][0] == "l0.dwa"
    ck.close()


def test_random_weights_mode_writes_a_loadable_folder(tmp_path):
    from beglin_b200.weights import Checkpoint, bind, write_random_model
    folder = write_random_model(str(tmp_path / "m"), EVEN, seed=3)
    _, _, spec = load(EVEN)
    ck = Checkpoint(folder)
    bound = bind(spec, ck, folder)
    dwa = bound["l3.dwa"].float()
    assert dwa.shape == (5,) and abs(float(dwa[-1]) - 1.0) < 0.2 and float(dwa[:-1].abs().max()) < 0.2
    ck.close()


def test_plain_recurrence_continues_from_any_cut():
    """The plain Mamba-2 function on a whole sequence equals its own token-by-token recurrence written out with an
    explicit state, which is what a cache has to carry: the state S and the last taps-1 inputs of the convolution."""
    cfg = copy.deepcopy(ODD)
    m = cfg["layers"][0]["mixer"]
    t = {k: v.double() for k, v in lively_tensors(cfg, 4, torch.float32).items()}
    h = torch.randn(13, cfg["width"], dtype=torch.float64, generator=torch.Generator().manual_seed(0))
    whole = plain.mamba2(h, t, "l0.", m, 1e-6)
    H, P, N, G, taps = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
    inner = H * P
    S = torch.zeros(H, N, P, dtype=torch.float64)
    tail = torch.zeros(taps - 1, inner + 2 * G * N, dtype=torch.float64)
    rows = []
    for tok in range(13):
        proj = t["l0.mix.in"] @ h[tok]
        z, xbc, dt = proj[:inner], proj[inner:2 * inner + 2 * G * N], proj[2 * inner + 2 * G * N:]
        window = torch.cat([tail, xbc[None]], 0)
        tail = window[1:]
        conv = plain.silu((window * t["l0.mix.conv"].t()).sum(0) + t["l0.mix.conv.b"])
        x, B, C = conv[:inner].reshape(H, P), conv[inner:inner + G * N].reshape(G, N), conv[inner + G * N:].reshape(G, N)
        dt = plain.softplus(dt + t["l0.mix.dt_bias"])
        y = torch.zeros(H, P, dtype=torch.float64)
        for hh in range(H):
            g = hh // (H // G)
            S[hh] = torch.exp(-torch.exp(t["l0.mix.A_log"][hh]) * dt[hh]) * S[hh] + dt[hh] * torch.outer(B[g], x[hh])
            y[hh] = S[hh].t() @ C[g] + t["l0.mix.D"][hh] * x[hh]
        y = y.reshape(inner) * plain.silu(z)
        y = plain.rms_unit(y.reshape(m["norm_groups"], -1), 1e-6).reshape(inner) * t["l0.mix.norm"]
        rows.append(t["l0.mix.o"] @ y)
    assert (torch.stack(rows) - whole).abs().max() < 1e-10


def test_plain_attention_in_the_latent_space_is_the_same_attention():
    """Scores taken against the cached latent with the query carried through W_uk, and values made from the weighted
    sum of latents, equal the plain per-head keys and values: the identity the engine's kernels rest on."""
    cfg = copy.deepcopy(ODD)
    m = cfg["layers"][1]["mixer"]
    t = {k: v.double() for k, v in lively_tensors(cfg, 4, torch.float32).items()}
    T = 9
    h = torch.randn(T, cfg["width"], dtype=torch.float64, generator=torch.Generator().manual_seed(1))
    c, kr = plain.latent_of(h, t, "l1.", m, 1e-6)
    want = plain.latent_attention(h, t, "l1.", m, 1e-6, c, kr)
    H, dim, rot, vd, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = plain.rms_unit(h @ t["l1.mix.dq"].t(), 1e-6) * t["l1.mix.dq.norm"]
    q = (cq @ t["l1.mix.uq"].t()).reshape(T, H, dim + rot)
    qr = plain.rotate_pairs(q[..., dim:], torch.arange(T), m["rot"]["base"], m["rot"]["dims"])
    uk, uv = t["l1.mix.uk"].reshape(H, dim, rank), t["l1.mix.uv"].reshape(H, vd, rank)
    gate = torch.sigmoid(h @ t["l1.mix.g"].t())
    out = torch.zeros(T, H, vd, dtype=torch.float64)
    for i in range(T):
        for hh in range(H):
            a = uk[hh].t() @ q[i, hh, :dim]
            s = (c[:i + 1] @ a + kr[:i + 1] @ qr[i, hh]) * m["scale"]
            o = torch.softmax(s, 0) @ c[:i + 1]
            out[i, hh] = (uv[hh] @ o) * gate[i, hh]
    got = out.reshape(T, H * vd) @ t["l1.mix.o"].t()
    assert (got - want).abs().max() < 1e-10
