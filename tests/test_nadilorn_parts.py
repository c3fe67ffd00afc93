"""Each mechanism of the Nadilorn decoder alone, kernel against the plain implementation's function of the same name (or
a closed form written here): the norm on a sublayer's result, the query/key norm with rotation and cache append, the
attention with values of another size, a window and the enlarged denominator, the output gate, the gated GELU, and
the routed experts piece by piece and as a part."""
import math

import pytest
import torch

from nadilorn_helpers import plain

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def ops():
    from beglin_b200.csrc import ops as o
    return o


def close(got, want, tol):
    got, want = got.double().cpu(), want.double().cpu()
    err = float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))
    assert err < tol, err


# ----------------------------------------------------------------------------- norm on the result
@pytest.mark.parametrize("T,d,parts,ydt", [(5, 72, 1, torch.float32), (3, 256, 4, torch.float32), (70, 100, 1, torch.bfloat16),
                                           (2, 1000, 3, torch.float32), (9, 37, 1, torch.float32)])
@pytest.mark.parametrize("lowp", [False, True])
def test_rmsnorm_add(T, d, parts, ydt, lowp):
    g = torch.Generator().manual_seed(T * d)
    x = torch.randn(T, d, generator=g)
    y = (torch.randn(parts, T, d, generator=g) * 3 if parts > 1 else torch.randn(T, d, generator=g) * 3).to(ydt)
    w = 1 + 0.3 * torch.randn(d, generator=g)
    ysum = y.double().sum(0) if parts > 1 else y.double()
    want = x.double() + plain.rms_norm(ysum, w.double(), 1e-5)
    xd = x.to(DEV)
    lp = torch.empty(T, d, dtype=torch.bfloat16, device=DEV) if lowp else None
    ops().rmsnorm_add(xd, y.to(DEV), w.to(DEV), 1e-5, lp)
    close(xd, want, 2e-6)
    if lowp:
        assert torch.equal(lp, xd.to(torch.bfloat16))


@pytest.mark.parametrize("T,d,top,scale,lowp", [(13, 24, 3, False, False), (70, 128, 2, True, True), (5, 37, 1, False, True)])
def test_rmsnorm_add_of_routed_rows(T, d, top, scale, lowp):
    """The norm on the result when the result is still the experts' rows: they are added up per token in rank order,
    normed and added to the stream in one kernel."""
    g = torch.Generator().manual_seed(T + d)
    x = torch.randn(T, d, generator=g)
    yp = torch.randn(T * top, d, generator=g) * 2
    wts = torch.rand(T * top, generator=g)
    row_of = torch.randperm(T * top, generator=g).int()
    w = 1 + 0.3 * torch.randn(d, generator=g)
    terms = yp.double()[row_of.long()] * (wts.double()[:, None] if scale else 1.0)
    want = x.double() + plain.rms_norm(terms.reshape(T, top, d).sum(1), w.double(), 1e-5)
    xd = x.to(DEV)
    lp = torch.empty(T, d, dtype=torch.bfloat16, device=DEV) if lowp else None
    ops().rmsnorm_add_routed(xd, yp.to(DEV), row_of.to(DEV), wts.to(DEV), top, scale, w.to(DEV), 1e-5, lp)
    close(xd, want, 2e-6)
    if lowp:
        assert torch.equal(lp, xd.to(torch.bfloat16))


# ----------------------------------------------------------------------------- query/key norm, rotation, append
def scattered_tables(lengths, page, n_pages, seed):
    """A block table per request over pages handed out in a shuffled order."""
    g = torch.Generator().manual_seed(seed)
    order = torch.randperm(n_pages, generator=g).tolist()
    width = max(-(-n // page) for n in lengths)
    table = torch.full((len(lengths), width), -1, dtype=torch.int32)
    for r, n in enumerate(lengths):
        for i in range(-(-n // page)):
            table[r, i] = order.pop()
    return table


@pytest.mark.parametrize("nh,nkv,hd,vd,rot,dtype", [(3, 1, 10, 6, 6, torch.float32), (4, 2, 12, 12, 12, torch.float32),
                                                      (2, 2, 16, 24, 0, torch.float32), (4, 2, 64, 32, 32, torch.bfloat16),
                                                      (8, 8, 8, 2, 4, torch.float32)])
@pytest.mark.parametrize("parts", [1, 3])
def test_qk_norm_rope_append(nh, nkv, hd, vd, rot, dtype, parts):
    o = ops()
    g = torch.Generator().manual_seed(nh * hd + vd)
    lengths, page = [13, 5], 8
    T = sum(lengths)
    positions = torch.cat([torch.arange(40, 40 + lengths[0]), torch.arange(3, 3 + lengths[1])]).int()
    row_req = torch.cat([torch.zeros(lengths[0]), torch.ones(lengths[1])]).int()
    table = scattered_tables([40 + lengths[0], 3 + lengths[1]], page, 12, 1)
    qd, kd, vdd, extra = nh * hd, nkv * hd, nkv * vd, 5
    src = torch.randn(parts, T, qd + kd + vdd + extra, generator=g) if parts > 1 else torch.randn(T, qd + kd + vdd + extra, generator=g)
    if parts == 1:
        src = src.to(dtype)
    elif dtype == torch.bfloat16:
        pass                                     # partial sums are float whatever the compute type
    wq, wk = 1 + 0.3 * torch.randn(qd, generator=g), 1 + 0.3 * torch.randn(kd, generator=g)
    eps, base, divisor = 1e-5, 50.0, 2.5
    rows = (src.double().sum(0) if parts > 1 else src.double())
    q = plain.rms_norm(rows[:, :qd], wq.double(), eps).reshape(T, nh, hd)
    k = plain.rms_norm(rows[:, qd:qd + kd], wk.double(), eps).reshape(T, nkv, hd)
    v = rows[:, qd + kd:qd + kd + vdd].reshape(T, nkv, vd)
    cos_sin = None
    if rot:
        q = plain.turn_halves(q, positions.tolist(), base, rot, divisor)
        k = plain.turn_halves(k, positions.tolist(), base, rot, divisor)
        inv = (base ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot) / divisor).float().to(DEV)
        cos_sin = torch.empty(T, rot // 2, 2, dtype=torch.float32, device=DEV)
        o.rope_table(positions.to(DEV), inv, cos_sin)
    n_pages = 12
    pool = torch.full((n_pages, nkv * page * (hd + vd)), float("nan"), dtype=dtype, device=DEV)
    q_out = torch.empty(T, qd, dtype=dtype, device=DEV)
    o.qk_norm_rope_append(src.to(DEV), q_out, T, nh, nkv, hd, vd, rot, False, wq.to(DEV), wk.to(DEV), eps, cos_sin,
                          positions.to(DEV), row_req.to(DEV), table.to(DEV), pool, page, None)
    tol = 3e-6 if dtype == torch.float32 else 1e-2
    close(q_out, q.reshape(T, qd), tol)
    pool = pool.cpu().double()
    for t in range(T):
        p = int(positions[t])
        pg = pool[int(table[int(row_req[t]), p // page])]
        keys = pg[:nkv * page * hd].reshape(nkv, page, hd)[:, p % page]
        vals = pg[nkv * page * hd:].reshape(nkv, page, vd)[:, p % page]
        close(keys, k[t], tol)
        close(vals, v[t], tol)
    assert int(torch.isnan(pool).sum()) == pool.numel() - T * (kd + vdd)          # nothing else was written


def test_qk_norm_rope_append_interleaved_pairs():
    """The other pairing of the rotation, (2i, 2i + 1), and no norm at all."""
    o = ops()
    T, nh, nkv, hd, vd, rot = 4, 2, 1, 8, 8, 6
    g = torch.Generator().manual_seed(2)
    src = torch.randn(T, (nh + 2 * nkv) * hd, generator=g)
    positions = torch.tensor([0, 1, 7, 30]).int()
    inv = (10.0 ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot)).float()
    cos_sin = torch.empty(T, rot // 2, 2, dtype=torch.float32, device=DEV)
    o.rope_table(positions.to(DEV), inv.to(DEV), cos_sin)
    pool = torch.zeros(4, 2, nkv, 8, hd, dtype=torch.float32, device=DEV)
    q_out = torch.empty(T, nh * hd, dtype=torch.float32, device=DEV)
    o.qk_norm_rope_append(src.to(DEV), q_out, T, nh, nkv, hd, vd, rot, True, None, None, 0.0, cos_sin, positions.to(DEV),
                          torch.zeros(T, dtype=torch.int32, device=DEV), torch.tensor([[2, 0, 3, 1]], dtype=torch.int32, device=DEV),
                          pool, 8, None)
    q = src[:, :nh * hd].double().reshape(T, nh, hd).clone()
    want = q.clone()
    for t in range(T):
        for i in range(rot // 2):
            a = float(positions[t]) * float(inv[i].double())
            want[t, :, 2 * i] = q[t, :, 2 * i] * math.cos(a) - q[t, :, 2 * i + 1] * math.sin(a)
            want[t, :, 2 * i + 1] = q[t, :, 2 * i + 1] * math.cos(a) + q[t, :, 2 * i] * math.sin(a)
    close(q_out, want.reshape(T, -1), 3e-6)
    assert torch.equal(pool[1, 1, 0, 6].cpu(), src[3, (nh + nkv) * hd:])                      # position 30: page index 3 -> page 1


# ----------------------------------------------------------------------------- attention
def plain_attention_rows(q, keys, vals, positions, scale, window, sink=True):
    """q [T, H, hd] at `positions` of ONE sequence whose keys [L, G, hd] and values [L, G, vd] are given whole."""
    T, H, _ = q.shape
    G = keys.shape[1]
    out = torch.zeros(T, H, vals.shape[2], dtype=torch.float64)
    for t in range(T):
        p = int(positions[t])
        first = 0 if not window else max(0, p - window + 1)
        seen = list(range(first, p + 1))
        for h in range(H):
            s = (keys[seen, h // (H // G)] @ q[t, h]) * scale
            w = plain.sink_softmax(s) if sink else torch.softmax(s, 0)
            out[t, h] = (w[:, None] * vals[seen, h // (H // G)]).sum(0)
    return out


def run_attention(q, keys, vals, lengths, new, scale, window, sink, dtype, page=16, split=64, prefer="generic", decode=False):
    """Requests with `lengths[r]` cached positions of which the last `new[r]` are the step's rows."""
    o = ops()
    H, hd = q[0].shape[1:]
    G, vd = keys[0].shape[1], vals[0].shape[2]
    n_pages = sum(-(-n // page) for n in lengths) + 3
    table = scattered_tables(lengths, page, n_pages, 7)
    flat = hd != vd
    pool = torch.full((n_pages, G * page * (hd + vd)), float("nan"), dtype=dtype)
    for r, n in enumerate(lengths):
        for p in range(n):
            pg = pool[int(table[r, p // page])]
            pg[:G * page * hd].view(G, page, hd)[:, p % page] = keys[r][p].to(dtype)
            pg[G * page * hd:].view(G, page, vd)[:, p % page] = vals[r][p].to(dtype)
    if not flat:
        pool = pool.view(n_pages, 2, G, page, hd)
    rows = torch.cat([q[r] for r in range(len(lengths))]).to(dtype)
    T = rows.shape[0]
    positions = torch.cat([torch.arange(n - m, n) for n, m in zip(lengths, new)]).int()
    kernel, bq, tile = o.attention_plan(H // G, hd, dtype, decode, prefer, page, vd=vd)
    blocks = []
    r0 = 0
    for r, m in enumerate(new):
        for f in range(0, m, bq):
            blocks.append([r, r0 + f, min(bq, m - f)])
        r0 += m
    qblk = torch.tensor(blocks, dtype=torch.int32, device=DEV)
    out = torch.empty(T, H * vd, dtype=dtype, device=DEV)
    o.attention(rows.reshape(T, H * hd).to(DEV), H * hd, pool.to(DEV), table.to(DEV), positions.to(DEV), qblk, len(blocks),
                int(positions.max()), T, H, G, hd, window or 0, split, tile, bq, scale, out, o.new_status(DEV), kernel, vd=vd, sink=sink)
    return out.reshape(T, H, vd)


@pytest.mark.parametrize("H,G,hd,window", [(6, 2, 64, 100), (4, 1, 128, None), (2, 2, 128, 70), (8, 2, 64, 300)])
@pytest.mark.parametrize("how", ["tcgen05", "mma", "mma_decode"])
@pytest.mark.parametrize("sink", [True, False])
def test_tensor_core_attention_with_sink(H, G, hd, window, how, sink):
    """The tensor-core kernels (tcgen05 for portions, mma.sync for portions and for single tokens) with the enlarged
    denominator and a window, pages of 16 and of 64, against the plain softmax."""
    g = torch.Generator().manual_seed(H * hd)
    decode = how == "mma_decode"
    lengths, new = ([150, 333, 9, 600], [1, 1, 1, 1]) if decode else ([150, 333, 9], [37, 130, 9])
    rnd = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64).to(torch.bfloat16).double()
    keys, vals = [rnd(n, G, hd) for n in lengths], [rnd(n, G, hd) for n in lengths]
    q = [rnd(m, H, hd) for m in new]
    scale = 1.3 / math.sqrt(hd)
    for page in (16, 64):
        got = run_attention(q, keys, vals, lengths, new, scale, window, sink, torch.bfloat16, page=page, split=256,
                            prefer="mma" if decode else how, decode=decode)
        want = torch.cat([plain_attention_rows(q[r], keys[r], vals[r], range(n - m, n), scale, window, sink=sink)
                          for r, (n, m) in enumerate(zip(lengths, new))])
        close(got, want, 1e-2)


@pytest.mark.parametrize("H,G,hd,vd,window", [(3, 1, 10, 6, 13), (4, 2, 12, 12, 40), (2, 2, 16, 24, None), (6, 3, 64, 32, 100),
                                                (2, 1, 128, 128, 70), (4, 4, 8, 2, 1)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_with_sink_window_and_value_size(H, G, hd, vd, window, dtype):
    """Three requests of unequal lengths in one step: a prompt's portion, a single decoded token far into its sequence,
    and a short first portion; against the plain softmax with the enlarged denominator."""
    g = torch.Generator().manual_seed(H * hd + vd)
    lengths, new = [150, 333, 9], [37, 1, 9]
    keys = [torch.randn(n, G, hd, generator=g, dtype=torch.float64) for n in lengths]
    vals = [torch.randn(n, G, vd, generator=g, dtype=torch.float64) for n in lengths]
    q = [torch.randn(m, H, hd, generator=g, dtype=torch.float64) for m in new]
    if dtype == torch.bfloat16:
        keys, vals, q = [[t.to(dtype).double() for t in ts] for ts in (keys, vals, q)]
    scale = 1.3 / math.sqrt(hd)
    got = run_attention(q, keys, vals, lengths, new, scale, window, True, dtype)
    want = torch.cat([plain_attention_rows(q[r], keys[r], vals[r], range(n - m, n), scale, window)
                      for r, (n, m) in enumerate(zip(lengths, new))])
    close(got, want, 5e-6 if dtype == torch.float32 else 1e-2)
    if window == 1:                                # a row that sees itself alone: the sink takes its share
        s = (keys[0][149, 0] @ q[0][36, 0]) * scale
        close(got[36, 0], vals[0][149, 0] * torch.exp(s) / (1 + torch.exp(s)), 1e-5 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("place", ["far", "window_last", "window_out", "page_border"])
def test_attention_one_key_stands_out(place):
    """Among 600 keys one is made to stand out for the last query (its score far above the rest): far back, the
    oldest key of the window, just outside it, or the last key of a page.  Its value, scaled up, is what the row returns
    when it is seen, and is absent when it is not."""
    g = torch.Generator().manual_seed(5)
    L, G, H, hd, vd, window = 600, 1, 2, 16, 8, {"far": None, "window_last": 100, "window_out": 100, "page_border": None}[place]
    at = {"far": 11, "window_last": L - 100, "window_out": L - 101, "page_border": 16 * 20 - 1}[place]
    keys = torch.randn(L, G, hd, generator=g, dtype=torch.float64) * 0.3
    vals = torch.randn(L, G, vd, generator=g, dtype=torch.float64)
    q = torch.randn(1, H, hd, generator=g, dtype=torch.float64) * 0.3
    keys[at, 0] = q[0, 0] / q[0, 0].norm() * 8.0
    q[0, 0] *= 8.0 / (0.3 * math.sqrt(hd))
    vals[at] *= 30.0
    got = run_attention([q], [keys], [vals], [L], [1], 1.0, window, True, torch.float32)
    want = plain_attention_rows(q, keys, vals, [L - 1], 1.0, window)
    close(got, want, 1e-5)
    seen = place != "window_out"
    assert (float(got[0, 0].abs().max()) > 5.0) == seen


# ----------------------------------------------------------------------------- gate, gated GELU
@pytest.mark.parametrize("parts", [1, 2])
def test_sigmoid_gate(parts):
    g = torch.Generator().manual_seed(1)
    T, n, col0, W = 7, 18, 11, 40
    out = torch.randn(T, n, generator=g)
    src = torch.randn(parts, T, W, generator=g) if parts > 1 else torch.randn(T, W, generator=g)
    gate = (src.sum(0) if parts > 1 else src)[:, col0:col0 + n]
    want = out.double() * torch.sigmoid(gate.double())
    od = out.to(DEV)
    ops().sigmoid_gate(od, src.to(DEV), col0, n)
    close(od, want, 2e-6)


@pytest.mark.parametrize("im,block,parts,dtype", [(100, 0, 1, torch.float32), (128, 64, 1, torch.bfloat16), (64, 64, 3, torch.float32),
                                                   (20, 0, 2, torch.float32), (256, 64, 1, torch.float32)])
def test_gated_gelu(im, block, parts, dtype):
    g = torch.Generator().manual_seed(im)
    T = 6
    gu = (torch.randn(parts, T, 2 * im, generator=g) * 2 if parts > 1 else (torch.randn(T, 2 * im, generator=g) * 2).to(dtype))
    rows = gu.double().sum(0) if parts > 1 else gu.double()
    if block:
        rows = rows.reshape(T, im // block, 2, block)
        gate, up = rows[:, :, 0].reshape(T, im), rows[:, :, 1].reshape(T, im)
    else:
        gate, up = rows[:, :im], rows[:, im:]
    out = torch.empty(T, im, dtype=dtype, device=DEV)
    ops().swiglu(gu.to(DEV), out, block, "gelu_tanh")
    close(out, plain.gelu_tanh(gate) * up, 2e-6 if dtype == torch.float32 else 1e-2)


# ----------------------------------------------------------------------------- routed experts
def test_router_logits_and_choice():
    o = ops()
    g = torch.Generator().manual_seed(3)
    T, d, E, top = 70, 50, 11, 3
    h = torch.randn(T, d, generator=g)
    router = torch.randn(E, d, generator=g)
    logits = torch.empty(T, E, dtype=torch.float32, device=DEV)
    o.route_logits(h.to(DEV), router.to(DEV), logits)
    close(logits, h.double() @ router.double().T, 2e-6)
    hb = h.to(torch.bfloat16)
    o.route_logits(hb.to(DEV), router.to(DEV), logits)                    # rows in bfloat16, float arithmetic
    close(logits, hb.double() @ router.double().T, 2e-6)
    z = torch.randn(T, E, generator=g) * 6
    z[5, 2] = z[5, 7] = 30.0                                              # equal, and both round to a score of one
    z[6] = 25.0 + torch.arange(E) * 0.5                                   # all scores round to one: the logits decide
    ids = torch.empty(T, top, dtype=torch.int32, device=DEV)
    w = torch.empty(T, top, dtype=torch.float32, device=DEV)
    o.route_topk(z.to(DEV), top, ids, w)
    want = torch.sort(z.double(), dim=1, descending=True, stable=True)
    assert torch.equal(ids.cpu().long(), want.indices[:, :top])
    assert ids[5, 0] == 2 and ids[5, 1] == 7 and ids[6].tolist() == [10, 9, 8]
    close(w, torch.sigmoid(want.values[:, :top]), 2e-6)
    o.route_topk(z.to(DEV), top, ids, w, sigmoid=True, renorm=True)
    s = torch.sigmoid(want.values[:, :top])
    close(w, s / s.sum(1, keepdim=True), 2e-6)
    # logits and choice as one kernel, rows in either type, a number of tokens that is no multiple of a block's
    for rows in (h, hb):
        o.route(rows.to(DEV), router.to(DEV), top, ids, w, logits=logits)
        zz = rows.double() @ router.double().T
        close(logits, zz, 2e-6)
        srt = torch.sort(logits.cpu().double(), dim=1, descending=True, stable=True)
        assert torch.equal(ids.cpu().long(), srt.indices[:, :top])
        close(w, torch.sigmoid(srt.values[:, :top]), 2e-6)


@pytest.mark.parametrize("A,E", [(1, 1), (7, 3), (300, 5), (5000, 64), (64, 200)])
def test_route_sort(A, E):
    g = torch.Generator().manual_seed(A)
    ids = torch.randint(0, E, (A,), generator=g).int()
    if E > 2:
        ids[ids == 1] = 0                                                 # an expert without rows
    off = torch.empty(E + 1, dtype=torch.int32, device=DEV)
    row_of, src_of = torch.empty(A, dtype=torch.int32, device=DEV), torch.empty(A, dtype=torch.int32, device=DEV)
    ops().route_sort(ids.to(DEV), E, off, row_of, src_of)
    off, row_of, src_of = off.cpu(), row_of.cpu().long(), src_of.cpu().long()
    counts = torch.bincount(ids.long(), minlength=E)
    assert torch.equal(off[1:].long() - off[:-1].long(), counts) and off[0] == 0
    assert sorted(row_of.tolist()) == list(range(A)) and torch.equal(src_of[row_of], torch.arange(A))
    for a in range(0, A, max(1, A // 50)):
        assert off[ids[a]] <= row_of[a] < off[ids[a] + 1]


@pytest.mark.parametrize("E,N,K,loads,dtype,tc", [
    (5, 20, 72, [3, 0, 40, 1, 17], torch.float32, False), (3, 9, 33, [2, 2, 2], torch.float32, False),
    (8, 64, 128, [0, 100, 3, 0, 16, 17, 300, 1], torch.bfloat16, True), (4, 256, 64, [1, 0, 0, 2], torch.bfloat16, True),
    (2, 130, 200, [700, 5], torch.bfloat16, True), (2, 1024, 64, [4000, 1100], torch.bfloat16, True), (3, 40, 36, [9, 1, 50], torch.bfloat16, False), (1, 128, 64, [33], torch.bfloat16, True)])
@pytest.mark.parametrize("act", ["none", "relu2"])
def test_grouped_product(E, N, K, loads, dtype, tc, act):
    """Experts with unequal numbers of rows, some with none, on the CUDA-core kernel and on the tcgen05 kernel (row tiles of
    16 to 256; the last case has more CTAs than SMs, which run two to an SM with two stages each)."""
    o = ops()
    g = torch.Generator().manual_seed(E * N + K)
    A = sum(loads)
    x = (torch.randn(A, K, generator=g)).to(dtype)
    w = (torch.randn(E, N, K, generator=g) / math.sqrt(K)).to(dtype)
    off = torch.tensor([sum(loads[:e]) for e in range(E + 1)], dtype=torch.int32)
    for out_dtype in ([torch.float32] if dtype == torch.float32 else [torch.float32, torch.bfloat16]):
        out = torch.full((A, N), float("nan"), dtype=out_dtype, device=DEV)
        status = o.new_status(DEV)
        o.gemm_grouped(x.to(DEV), w.to(DEV), off.to(DEV), out, act, status, tensor_cores=tc)
        o.raise_on_status(status)
        want = torch.cat([x[off[e]:off[e + 1]].double() @ w[e].double().T for e in range(E)])
        if act == "relu2":
            want = plain.relu_squared(want)
        close(out, want, 3e-6 if dtype == torch.float32 else (2e-5 if out_dtype == torch.float32 else 1e-2))


@pytest.mark.parametrize("scale_input", [True, False])
def test_gather_and_combine(scale_input):
    o = ops()
    g = torch.Generator().manual_seed(9)
    T, d, top = 13, 24, 3
    x = torch.randn(T, d, generator=g)
    wts = torch.rand(T * top, generator=g)
    perm = torch.randperm(T * top, generator=g)
    row_of = perm.int()
    src_of = torch.empty_like(row_of)
    src_of[perm] = torch.arange(T * top, dtype=torch.int32)
    xp = torch.empty(T * top, d, dtype=torch.float32, device=DEV)
    o.route_gather(x.to(DEV), wts.to(DEV), src_of.to(DEV), xp, top, scale=scale_input)
    want = x.double()[src_of.long() // top] * (wts.double()[src_of.long()][:, None] if scale_input else 1.0)
    close(xp, want, 1e-6)
    yp = torch.randn(T * top, d, generator=g)
    out = torch.empty(T, d, dtype=torch.float32, device=DEV)
    o.route_combine(yp.to(DEV), wts.to(DEV), row_of.to(DEV), out, top, scale=not scale_input)
    terms = yp.double()[row_of.long()] * (1.0 if scale_input else wts.double()[:, None])
    close(out, terms.reshape(T, top, d).sum(1), 2e-6)


@pytest.mark.parametrize("d,ff,E,top,dtype,T", [(72, 20, 5, 2, torch.float32, 41), (48, 9, 3, 3, torch.float32, 7), (128, 64, 8, 2, torch.bfloat16, 150),
                                                  (64, 128, 4, 1, torch.bfloat16, 3), (40, 12, 6, 1, torch.bfloat16, 20)])
def test_routed_experts_part(d, ff, E, top, dtype, T):
    """The part as a layer runs it against the oracle's function, with router logits that cannot be a close call in
    bfloat16 (small dyadic numbers in the last four features, which the router alone reads)."""
    from beglin_b200.parts import BuildContext, RoutedExpertsSpec
    from beglin_b200.parts.moe import RoutedExperts
    g = torch.Generator().manual_seed(d + ff)
    w = {"router": torch.randn(E, d, generator=g) * 0.5}
    h = torch.randn(T, d, generator=g)
    if dtype == torch.bfloat16:
        w["router"][:, :-4] = 0.0
        w["router"][:, -4:] = torch.tensor([-1.5, -1.0, -0.5, 0.5, 1.0, 1.5])[torch.randint(0, 6, (E, 4), generator=g)]
        h[:, -4:] = torch.tensor([-2.0, -1.0, 1.0, 2.0])[torch.randint(0, 4, (T, 4), generator=g)]
    for e in range(E):
        w[f"e{e}.up"] = torch.randn(ff, d, generator=g) / math.sqrt(d)
        w[f"e{e}.down"] = torch.randn(d, ff, generator=g) / math.sqrt(ff)
    w = {n: t.to(dtype) for n, t in w.items()}
    h = h.to(dtype)
    ctx = BuildContext(device=DEV, compute_dtype=dtype, status=ops().new_status(DEV))
    spec = RoutedExpertsSpec(hidden=d, intermediate=ff, experts=E, top=top)
    tensors = {"router.weight": w["router"]}
    for e in range(E):
        tensors[f"experts.{e}.up.weight"], tensors[f"experts.{e}.down.weight"] = w[f"e{e}.up"], w[f"e{e}.down"]
    part = RoutedExperts(spec, tensors, ctx)
    got = part.forward(h.to(DEV), None)
    ops().raise_on_status(ctx.status)
    want = plain.routed_experts({n: t.double() for n, t in w.items()}, "", h.double(), E, top)
    close(got, want, 5e-6 if dtype == torch.float32 else 2e-2)
