"""Every mechanism of the Sukisun decoder alone, as the framework's part or kernel, against the plain function of
the same mechanism: the centred norm, the xIELU feed-forward, the depth-weighted average, attention through a
latent (own cache and another layer's, prompt portions and single tokens, part of the rotated features
turning), and the Mamba-2 recurrence (several groups, norm in parts, portions down to one token, two requests in
one step)."""
import pytest
import torch

from sukisun_helpers import plain, rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOLS = [(torch.float32, 2e-5), (torch.bfloat16, 3e-2)]


def ctx_for(dtype, page=8, kv_split=64):
    from beglin_b200.csrc import ops
    from beglin_b200.parts import BuildContext
    c = BuildContext(device=DEV, compute_dtype=dtype, page_size=page, kv_split=kv_split)
    c.status = ops.new_status(DEV)
    return c


def rnd(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g) * scale


class Requests:
    """A cache manager for the stages of one or two mixers, and step batches for named requests."""

    def __init__(self, needs, page, dtype, pages=40, slots=3):
        from beglin_b200.cache import CacheManager
        self.cache = CacheManager(needs, page_size=page, num_pages=pages, max_requests=slots)
        self.cache.allocate(DEV, dtype)
        for g in self.cache.kv_groups:
            g.device_pool.fill_(float("nan"))
        for g in self.cache.state_groups:
            g.slab.fill_(float("nan"))

    def batch(self, portions):
        """portions: [(request, number of new tokens)]; requests are added when first seen."""
        from beglin_b200.engine.batch import Entry, StepBatch
        for rid, _ in portions:
            if not self.cache.has(rid):
                self.cache.add_request(rid)
        starts = [self.cache.length(r) for r, _ in portions]
        plan = [(r, s + n) for (r, n), s in zip(portions, starts)]
        self.cache.reserve(plan)
        b = StepBatch([Entry(r, [0] * n, []) for r, n in portions], starts, DEV, self.cache)
        self.cache.commit(plan)
        return b


@pytest.mark.parametrize("dtype,tol", TOLS)
def test_centred_norm_with_the_add_in_front(dtype, tol):
    from beglin_b200.parts import NormSpec
    from beglin_b200.parts.norm import LayerNorm
    ctx = ctx_for(dtype)
    d, T = 72, 9
    w = 1 + rnd(d, seed=1, scale=0.3)
    norm = LayerNorm(NormSpec(size=d, eps=1e-5, kind="layernorm"), {"weight": w}, ctx)
    x = (rnd(T, d, seed=2) + 3.0).to(DEV)                        # a mean far from zero: an RMS norm would differ visibly
    delta = rnd(3, T, d, seed=3).to(DEV)                         # partial sums, added in order
    x0 = x.clone()
    h = norm.add_norm(x, delta)
    want_x = x0.double().cpu() + delta.double().cpu().sum(0)
    assert (x.double().cpu() - want_x).abs().max() < 1e-5
    wq = w.double()                                              # stored in 32-bit, a norm weight stays so
    assert rel_err(h, plain.layer_norm(want_x, wq, 1e-5)) < tol
    rows = torch.tensor([7, 2], dtype=torch.int32, device=DEV)
    before = x.clone()
    some = norm.add_norm(x, None, rows=rows, update=False)
    assert torch.equal(x, before)
    assert rel_err(some, plain.layer_norm(want_x[[7, 2]], wq, 1e-5)) < tol


@pytest.mark.parametrize("dtype,tol", TOLS)
def test_dense_feed_forward_with_xielu(dtype, tol):
    from beglin_b200.csrc import ops
    from beglin_b200.parts import DenseActSpec
    from beglin_b200.parts.mlp import DenseAct
    ctx = ctx_for(dtype)
    d, ff, T = 40, 100, 11
    z = torch.linspace(-6, 6, 4 * ff).reshape(4, ff).to(DEV)
    act = torch.tensor([0.75, -1.25])
    out = torch.empty((4, ff), dtype=dtype, device=DEV)
    ops.xielu(z, act.to(DEV), out)
    assert rel_err(out, plain.xielu(z.double().cpu(), act[0].double(), act[1].double())) < tol
    parts = torch.stack([z * 0.25, z * 0.5, z * 0.25])            # partial sums of a product
    ops.xielu(parts, act.to(DEV), out)
    assert rel_err(out, plain.xielu(z.double().cpu(), act[0].double(), act[1].double())) < tol
    t = {"up.weight": rnd(ff, d, seed=7, scale=0.3), "down.weight": rnd(d, ff, seed=9, scale=0.2), "act": act}
    part = DenseAct(DenseActSpec(hidden=d, intermediate=ff), t, ctx)
    h = rnd(T, d, seed=6).to(dtype)
    w = {"l.mlp.up": t["up.weight"].to(dtype).double(), "l.mlp.down": t["down.weight"].to(dtype).double(),
         "l.mlp.act": act.to(dtype).double()}
    got = part.forward(h.to(DEV), None)
    if got.dim() == 3:
        got = got.sum(0)
    assert rel_err(got, plain.dense_feed_forward(h.double(), w, "l.")) < tol * 2


def test_depth_average_keeps_every_result():
    from beglin_b200.parts import DepthAverageSpec
    from beglin_b200.parts.depth import DepthAverage
    from beglin_b200.parts.stream import ResidualStream
    ctx = ctx_for(torch.float32)
    T, d, n = 5, 24, 3
    ws = [rnd(i + 2, seed=20 + i) for i in range(n)]
    parts = [DepthAverage(DepthAverageSpec(terms=i + 2, total=n + 1), {"weight": ws[i]}, ctx) for i in range(n)]
    x0 = rnd(T, d, seed=1)
    stream = ResidualStream(x0.clone().to(DEV))
    results = [x0.double()]
    x = x0.double()
    for i in range(n):
        parts[i].begin(stream)
        stream.x += 0.5                                            # a sublayer that adds in place,
        owed = rnd(2, T, d, seed=30 + i)                          # and one whose partial sums are still owed
        stream.owe(owed.to(DEV))
        parts[i].forward(stream, None)
        results.append(x + 0.5 + owed.double().sum(0))
        x = sum(ws[i][j].double() * results[j] for j in range(i + 2))
        assert stream.pending is None
        assert rel_err(stream.x, x) < 1e-6, i
    assert rel_err(stream.history, torch.stack(results)) < 1e-6


def latent_weights(spec, seed, dtype):
    from beglin_b200.parts.latent_attention import LatentAttention
    t = {}
    for k, role in enumerate(LatentAttention.expected_tensors(spec)):
        if len(role.shape) == 1:
            t[role.name] = (1 + rnd(*role.shape, seed=seed + k, scale=0.2)).to(dtype)
        else:
            t[role.name] = rnd(*role.shape, seed=seed + k, scale=1.3 / role.shape[1] ** 0.5).to(dtype)
    return t


def plain_names(t, p):
    """A part's tensors under the names the plain implementation reads."""
    m = {"q_down.weight": "mix.dq", "q_down.norm": "mix.dq.norm", "q_up.weight": "mix.uq", "kv_down.weight": "mix.dkv",
         "kv_down.norm": "mix.dkv.norm", "k_up.weight": "mix.uk", "v_up.weight": "mix.uv", "gate.weight": "mix.g",
         "o_proj.weight": "mix.o", "in_proj.weight": "mix.in", "conv.weight": "mix.conv", "conv.bias": "mix.conv.b",
         "dt_bias": "mix.dt_bias", "A_log": "mix.A_log", "D": "mix.D", "norm.weight": "mix.norm"}
    return {p + m[k]: v.double() for k, v in t.items()}


@pytest.mark.parametrize("dtype,tol", TOLS)
@pytest.mark.parametrize("dims", [12, 8, 0])
def test_latent_attention_own_and_borrowed_cache(dtype, tol, dims):
    """Two mixers: the first appends to its cache, the second (other heads and sizes) reads that cache.  A prompt of
    150 tokens in portions of 70, 2, 77 and 1 over pages of 8 and splits of 64 keys, against the plain function
    on the whole sequence.  `dims` of the 12 rotated features turn (all, some, none)."""
    from beglin_b200.parts import LatentAttentionSpec, PositionSpec
    from beglin_b200.parts.latent_attention import LatentAttention
    ctx = ctx_for(dtype, page=8, kv_split=64)
    d, eps, T = 56, 1e-5, 150
    pos = PositionSpec(kind="rope" if dims else "none", rotary_dim=dims, theta=50.0, pairing="interleaved")
    s1 = LatentAttentionSpec(hidden=d, n_heads=3, dim=10, rot_dim=12, vdim=20, q_rank=24, kv_rank=36, scale=0.4, eps=eps,
                             position=pos)
    s2 = LatentAttentionSpec(hidden=d, n_heads=5, dim=16, rot_dim=12, vdim=6, q_rank=16, kv_rank=36, scale=0.3, eps=eps,
                             position=pos, own_kv=False)
    assert "kv_down.weight" not in [r.name for r in LatentAttention.expected_tensors(s2)]
    assert LatentAttention.cache_need(s2) is None and LatentAttention.cache_need(s1).width == 48
    t1, t2 = latent_weights(s1, 100, dtype), latent_weights(s2, 200, dtype)
    m1, m2 = LatentAttention(s1, t1, ctx), LatentAttention(s2, t2, ctx)
    h1, h2 = rnd(T, d, seed=5).to(dtype), rnd(T, d, seed=6).to(dtype)
    reqs = Requests([LatentAttention.cache_need(s1)], 8, dtype)
    outs1, outs2, at = [], [], 0
    for n in (70, 2, 77, 1):
        b = reqs.batch([("r", n)])
        view = reqs.cache.view(0, b)
        for m, h, outs in ((m1, h1, outs1), (m2, h2, outs2)):
            o = m.forward(h[at:at + n].to(DEV), b, view)
            outs.append(o.float().sum(0) if o.dim() == 3 else o.float())
        at += n
    cfg = lambda s: {"heads": s.n_heads, "dim": s.dim, "rot_dim": s.rot_dim, "vdim": s.vdim, "kv_rank": s.kv_rank,
                     "scale": s.scale, "rot": {"base": 50.0, "dims": dims}}
    w1, w2 = plain_names(t1, "a."), plain_names(t2, "b.")
    c, kr = plain.latent_of(h1.double(), w1, "a.", cfg(s1), eps)
    want1 = plain.latent_attention(h1.double(), w1, "a.", cfg(s1), eps, c, kr)
    want2 = plain.latent_attention(h2.double(), w2, "b.", cfg(s2), eps, c, kr)
    assert rel_err(torch.cat(outs1), want1) < tol
    assert rel_err(torch.cat(outs2), want2) < tol


@pytest.mark.parametrize("dtype,tol", TOLS)
@pytest.mark.parametrize("heads,vdim,state,groups,conv,norm_groups", [(4, 12, 20, 2, 3, 2), (2, 24, 9, 1, 2, 3),
                                                                       (6, 8, 70, 3, 5, 1), (1, 40, 4, 1, 1, 5),
                                                                       (2, 80, 16, 2, 4, 1)])
def test_mamba2_portions_and_two_requests(dtype, tol, heads, vdim, state, groups, conv, norm_groups):
    """Two sequences through one mixer in steps that hold portions of both (17 and 1, 1 and 30, 3 and 2, ...), against
    the plain recurrence over each whole sequence; then a third request in the slot that the first gave back."""
    from beglin_b200.parts import Mamba2Spec
    from beglin_b200.parts.mamba2 import Mamba2
    ctx = ctx_for(dtype)
    d, eps = 48, 1e-5
    spec = Mamba2Spec(hidden=d, n_heads=heads, vdim=vdim, state=state, groups=groups, conv=conv, norm_groups=norm_groups, eps=eps)
    t = {}
    for k, role in enumerate(Mamba2.expected_tensors(spec)):
        if role.name in ("A_log", "dt_bias"):
            t[role.name] = (rnd(*role.shape, seed=300 + k) - 0.5).to(dtype)
        elif role.name in ("D", "norm.weight"):
            t[role.name] = (1 + rnd(*role.shape, seed=300 + k, scale=0.3)).to(dtype)
        elif role.name.startswith("conv"):
            t[role.name] = rnd(*role.shape, seed=300 + k, scale=0.5).to(dtype)
        else:
            t[role.name] = rnd(*role.shape, seed=300 + k, scale=1.2 / role.shape[1] ** 0.5).to(dtype)
    part = Mamba2(spec, t, ctx)
    reqs = Requests([Mamba2.cache_need(spec)], 8, dtype, slots=2)
    hs = {"a": rnd(40, d, seed=1).to(dtype), "b": rnd(40, d, seed=2).to(dtype), "c": rnd(25, d, seed=3).to(dtype)}
    cuts = [[("a", 17), ("b", 1)], [("a", 1), ("b", 30)], [("b", 3), ("a", 2)], [("a", 20)], [("b", 6)]]
    outs = {"a": [], "b": [], "c": []}
    at = {"a": 0, "b": 0, "c": 0}

    def run(portions):
        b = reqs.batch(portions)
        h = torch.cat([hs[r][at[r]:at[r] + n] for r, n in portions]).to(DEV)
        o = part.forward(h, b, reqs.cache.view(0, b))
        o = o.float().sum(0) if o.dim() == 3 else o.float()
        row = 0
        for r, n in portions:
            outs[r].append(o[row:row + n].cpu())
            row += n
            at[r] += n

    for portions in cuts:
        run(portions)
    reqs.cache.release("a")
    run([("c", 24)])                                              # c takes a's slot
    run([("c", 1)])
    m = {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}
    w = plain_names(t, "l.")
    for r in ("a", "b", "c"):
        want = plain.mamba2(hs[r].double(), w, "l.", m, eps)
        assert rel_err(torch.cat(outs[r]), want) < tol, r


def test_mamba2_state_is_kept_in_32_bit():
    """In bfloat16 the slot that carries the recurrence is float32 all the same."""
    from beglin_b200.parts import Mamba2Spec
    from beglin_b200.parts.mamba2 import Mamba2
    need = Mamba2.cache_need(Mamba2Spec(hidden=8, n_heads=2, vdim=4, state=3, groups=1, conv=4, norm_groups=1, eps=1e-5))
    assert need.dtype == "float32" and need.shape == (2 * 3 * 4 + 3 * (8 + 6),)
    reqs = Requests([need], 8, torch.bfloat16)
    assert reqs.cache.state_groups[0].slab.dtype == torch.float32


@pytest.mark.parametrize("dim,rot,dims", [(32, 32, 32), (48, 16, 8), (64, 64, 64)])
def test_latent_attention_long_portions_through_per_head_keys(dim, rot, dims):
    """bfloat16 with dim + rot_dim = vdim = 64 or 128: a portion of one request of 128 rows and more makes every head's
    keys and values from the cached rows and runs the grouped-query kernel on the tensor cores; shorter portions and
    single tokens score against the cached rows themselves.  Both against the plain function, the second portion
    seeing what the first left in the cache."""
    from beglin_b200.parts import LatentAttentionSpec, PositionSpec
    from beglin_b200.parts.latent_attention import LatentAttention
    dtype = torch.bfloat16
    ctx = ctx_for(dtype, page=16, kv_split=64)
    d, eps, T = 96, 1e-5, 391
    pos = PositionSpec(kind="rope", rotary_dim=dims, theta=1000.0, pairing="interleaved")
    spec = LatentAttentionSpec(hidden=d, n_heads=3, dim=dim, rot_dim=rot, vdim=dim + rot, q_rank=40, kv_rank=56, scale=0.2,
                               eps=eps, position=pos)
    t = latent_weights(spec, 500, dtype)
    part = LatentAttention(spec, t, ctx)
    assert part.expand is not None
    h = rnd(T, d, seed=8).to(dtype)
    reqs = Requests([LatentAttention.cache_need(spec)], 16, dtype)
    outs, at = [], 0
    for n in (150, 40, 200, 1):                        # per-head keys, cached rows, per-head keys over 190 earlier positions, one token
        b = reqs.batch([("r", n)])
        o = part.forward(h[at:at + n].to(DEV), b, reqs.cache.view(0, b))
        outs.append(o.float().sum(0) if o.dim() == 3 else o.float())
        at += n
    m = {"heads": 3, "dim": dim, "rot_dim": rot, "vdim": dim + rot, "kv_rank": 56, "scale": 0.2, "rot": {"base": 1000.0, "dims": dims}}
    w = plain_names(t, "a.")
    c, kr = plain.latent_of(h.double(), w, "a.", m, eps)
    want = plain.latent_attention(h.double(), w, "a.", m, eps, c, kr)
    assert rel_err(torch.cat(outs), want) < 3e-2


@pytest.mark.parametrize("H,rank,rot,dims", [(6, 96, 32, 32), (3, 64, 64, 16), (20, 256, 64, 64), (40, 512, 64, 64), (1, 24, 8, 8)])
def test_latent_attention_kernels_agree(H, rank, rot, dims):
    """The tensor-core kernel (bfloat16 products, float sums) against the CUDA-core kernel (float throughout) on the same
    bfloat16 cache: three requests of 5, 333 and 70 positions whose steps bring 5, 40 and 1 rows, over pages of 16 and
    splits of 64 keys; then the three with one row each, the way a decoding step runs.  And the CUDA-core kernel against
    a plain softmax over the cached rows."""
    from beglin_b200.csrc import ops
    from beglin_b200.parts import PagedLatentNeed
    plan = ops.latent_attention_mma_plan(rank, rot)
    assert plan is not None
    rows_mma, stages = plan
    width, dim = rank + rot, 8
    reqs = Requests([PagedLatentNeed(width)], 16, torch.bfloat16, pages=40)
    lens = {"a": 5, "b": 333, "c": 70}
    new = {"a": 5, "b": 40, "c": 1}
    for r, n in lens.items():                              # what the requests hold before the step
        if n > new[r]:
            reqs.batch([(r, n - new[r])])
    pool = reqs.cache.kv_groups[0].device_pool[0]
    pool.copy_(rnd(*pool.shape, seed=1, scale=0.5).to(torch.bfloat16))
    for decode in (False, True):
        portions = [(r, 1 if decode else new[r]) for r in lens]
        b = reqs.batch(portions)
        T = b.n_rows
        view = reqs.cache.view(0, b)
        q_lat = rnd(H, T, rank, seed=2, scale=0.3).to(DEV)
        q_raw = rnd(T, H * (dim + rot), seed=3).to(torch.bfloat16).to(DEV)
        cos_sin = None
        if dims:
            ang = rnd(T, dims // 2, seed=4)
            cos_sin = torch.stack([torch.cos(ang), torch.sin(ang)], -1).contiguous().to(DEV)
        outs = {}
        for name in ("generic", "mma"):
            if name == "generic":
                rows, tile = ops.latent_attention_plan(rank, rot)
                hc, st = min(H, rows), 0
            else:
                rows, tile, st = rows_mma, 64, stages
                hc = min(H, rows)
            bq = 1 if decode else max(1, rows // hc)
            qblk, n_qblk = b.query_blocks(bq)
            out = torch.empty((H, T, rank), dtype=torch.float32, device=DEV)
            ops.latent_attention(q_lat, q_raw, dim, rot, dims, cos_sin, view.pool, view.block_table, b.positions, qblk, n_qblk,
                                 b.max_position, bq, hc, tile, 64, 0.2, out, None, mma_stages=st)
            outs[name] = out.cpu().double()
        assert torch.isfinite(outs["mma"]).all()
        assert rel_err(outs["mma"], outs["generic"]) < 2e-2, decode
        # the plain softmax over the cached rows, for every row of the step
        qr = q_raw.float().cpu().double().reshape(T, H, dim + rot)[:, :, dim:]
        if dims:
            cs = cos_sin.cpu().double()
            u, v = qr[..., 0:dims:2].clone(), qr[..., 1:dims:2].clone()
            qr = qr.clone()
            qr[..., 0:dims:2] = u * cs[:, None, :, 0] - v * cs[:, None, :, 1]
            qr[..., 1:dims:2] = v * cs[:, None, :, 0] + u * cs[:, None, :, 1]
        row = 0
        for i, (r, n) in enumerate(portions):
            table = view.block_table[i].cpu()
            for k in range(n):
                pos = int(b.positions[row])
                keys = torch.stack([pool[int(table[s // 16]), s % 16] for s in range(pos + 1)]).float().cpu().double()
                for hh in range(H):
                    qfull = torch.cat([q_lat[hh, row].cpu().double(), qr[row, hh]])
                    pr = torch.softmax(keys @ qfull * 0.2, 0)
                    want = pr @ keys[:, :rank]
                    assert (outs["generic"][hh, row] - want).abs().max() < 1e-4 * max(1.0, float(want.abs().max())), (r, k, hh)
                row += 1
