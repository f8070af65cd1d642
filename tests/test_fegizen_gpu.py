"""Fegizen on the GPU against the plain implementation (tests/plain_fegizen.py): each mechanism alone through its
kernels, then whole models under schedules (whole, token by token, portions down to two tokens, mixed batches on a
pool so small that pages and slots are used again), windows' edges in prompts and in decoding, a far token that only
the recurrent state carries, long decoding, random configurations, and greedy generation through generate()."""
import math
from types import SimpleNamespace

import pytest
import torch

import fegizen_tiny as ft
import plain_fegizen as pf
import tiny

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
F64 = torch.float64


def rel_err(got, want):
    return float((got.double().cpu() - want).abs().max() / want.abs().max())


def i32(values):
    return torch.tensor(values, dtype=torch.int32, device=DEV)


def fake_batch(lens, slots):
    """What the kernels read of a step's descriptor: sequences of `lens` new tokens in state slots `slots`."""
    starts = [sum(lens[:i]) for i in range(len(lens))]
    return SimpleNamespace(n_seqs=len(lens), row_seq=i32([s for s, n in enumerate(lens) for _ in range(n)]),
                           seq_q_start_d=i32(starts), seq_q_len_d=i32(lens), seq_slot_d=i32(slots))


# ---------------------------------------------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("width", [8, 50, 256, 1000, 4100])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_centring_norm_with_the_add_in_front(width, dtype):
    """Rows far from zero (a mean a hundred times the spread, where a variance formed as mean of squares minus squared
    mean would lose everything), the part's output arriving as three shares; the sum is written back to the stream."""
    from flambeau_b200.kernels import ops
    g = torch.Generator().manual_seed(width)
    n, eps = 9, 1e-5
    x = torch.randn(n, width, generator=g) + 100.0
    shares = torch.randn(3, n, width, generator=g)
    w = (torch.randn(width, generator=g) + 1).to(DT[dtype])
    total = x.double() + shares.double().sum(0)
    want = pf.centred_norm(total, w.double(), eps)
    xd, sd = x.to(DEV), shares.to(DEV).contiguous()
    out = torch.empty((n, width), dtype=DT[dtype], device=DEV)
    ops.add_layer_norm(xd, sd[0], w.to(DEV), eps, out, n_partials=3, partial_stride=sd.stride(0))
    assert rel_err(out, want) < (2e-4 if dtype == "float32" else 1e-2)      # (the float32 sum of ~100 keeps 1e-5 of a unit)
    assert rel_err(xd, total) < 1e-6
    out32 = torch.empty((n, width), dtype=torch.float32, device=DEV)
    ops.add_layer_norm(xd, None, w.to(DEV), eps, out32)
    assert rel_err(out32, want) < 2e-4


@pytest.mark.parametrize("taps", [1, 2, 3, 4, 5])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("layout", [(40, 7, 3), (72, 8, 4)], ids=["ragged", "by16bytes"])
def test_convolution_over_time_across_steps(taps, dtype, layout):
    """Three requests in three slots, fed in steps of unequal portions (one token, two, many; portions shorter than
    the taps follow each other), their kept inputs at an offset inside the slot; then a slot zeroed and used again.
    Once with a width and an offset that leave nothing aligned, once with rows that move as 16-byte vectors."""
    from flambeau_b200.kernels import ops
    D, off, pad = layout
    g = torch.Generator().manual_seed(taps)
    lengths = [23, 9, 40]
    w = (torch.randn(D, taps, generator=g) * 0.5).to(DT[dtype])
    hs = [torch.randn(L, D, generator=g) for L in lengths]
    want = [pf.add_time_conv(h.double(), w.double()) for h in hs]
    state = torch.zeros((4, off + (taps - 1) * D + pad), dtype=torch.float32, device=DEV)
    state[3].fill_(float("nan"))
    wt = w.t().float().contiguous().to(DEV)            # tap by tap, as the part hands the weights to the kernel
    slots, at, got = [2, 0, 1], [0, 0, 0], [[], [], []]
    for portion in [[1, 2, 5], [1, 1, 17], [2, 0, 1], [3, 6, 16], [16, 0, 1]]:
        live = [(s, k) for s, k in enumerate(portion) if k]
        h = torch.cat([hs[s][at[s]:at[s] + k] for s, k in live]).to(DEV)
        out = torch.empty((h.shape[0], D), dtype=DT[dtype], device=DEV)
        ops.time_conv(h, wt, state, off, fake_batch([k for _, k in live], [slots[s] for s, _ in live]), out,
                      h.shape[0])
        r = 0
        for s, k in live:
            got[s].append(out[r:r + k].cpu())
            r += k
            at[s] += k
    assert at == lengths
    tol = 1e-6 if dtype == "float32" else 1e-2
    for s in range(3):
        assert rel_err(torch.cat(got[s]), want[s]) < tol
    assert bool((state[:3, :off] == 0).all()) and bool((state[:3, off + (taps - 1) * D:] == 0).all()), \
        "numbers beside the kept inputs were written"
    assert bool(torch.isnan(state[3]).all()), "a slot that no sequence of the step uses was written"
    state[slots[1]].zero_()
    out = torch.empty((lengths[1], D), dtype=DT[dtype], device=DEV)
    ops.time_conv(hs[1].to(DEV), wt, state, off, fake_batch([lengths[1]], [slots[1]]), out, lengths[1])
    assert rel_err(out, want[1]) < tol


def test_mix_over_depth():
    """The newest result is the stream plus the part's shares; the stream becomes the weighted sum of all so far."""
    from flambeau_b200.kernels import ops
    g = torch.Generator().manual_seed(4)
    n, D, slots = 11, 72, 5
    history = torch.randn(slots, n + 2, D, generator=g)
    weights = torch.randn(slots, generator=g)
    for count, parts in ((2, 0), (3, 1), (5, 3)):
        x = torch.randn(n + 2, D, generator=g)
        shares = torch.randn(max(parts, 1), n + 2, D, generator=g)
        newest = x.double() + (shares.double().sum(0) if parts else 0)
        want = sum(weights[j].double() * history[j].double() for j in range(count - 1)) + weights[count - 1].double() * newest
        xd, hd_, sd = x.to(DEV), history.to(DEV), shares.to(DEV).contiguous()
        ops.depth_average(xd, sd[0] if parts else None, parts, sd.stride(0), hd_, count, weights.to(DEV), n)
        assert rel_err(xd[:n], want[:n]) < 1e-6 and rel_err(hd_[count - 1, :n], newest[:n]) < 1e-6
        assert torch.equal(xd[n:].cpu(), x[n:]), "rows beyond the step's tokens were written"


@pytest.mark.parametrize("stretch", [None, {"factor": 4.0, "original": 16, "fast": 8.0, "slow": 1.0},
                                     {"factor": 40.0, "original": 4096, "fast": 32.0, "slow": 1.0}], ids=["plain", "s4", "s40"])
def test_rotation_tables_of_neighbouring_pairs(stretch):
    from flambeau_b200.engine.runtime import Runtime
    from flambeau_b200.kernels import ops
    from flambeau_b200.parts.positions import RotaryNeighbours
    dims, base = 12, 5e5
    part = RotaryNeighbours(Runtime(DEV, "float32"), head_dim=16, theta=base, rotary_dim=dims, stretch=stretch)
    rot = {"base": base, "dims": dims}
    if stretch:
        rot["scaling"] = stretch
    freqs, mag = pf.rotary_frequencies(rot)
    assert torch.allclose(torch.tensor(part.frequencies, dtype=F64), freqs, rtol=1e-12) and part.magnitude == pytest.approx(mag)
    positions = [0, 1, 2, 63, 64, 1000, 100000]
    n = len(positions)
    cos = torch.empty((n, dims // 2), dtype=torch.float32, device=DEV)
    sin = torch.empty_like(cos)
    ops.rope_table(i32(positions), part.inv_freq(), cos, sin, part.magnitude)
    g = torch.Generator().manual_seed(0)
    x = torch.randn(n, 3 * 16, generator=g)
    want = pf.rotate_neighbours(x.double().reshape(n, 3, 16), positions, freqs, mag).reshape(n, 48)
    xd = x.to(DEV)
    ops.rope_neighbours(xd, cos, sin, dims // 2, 3, 16)
    assert rel_err(xd, want) < 2e-6


def paged_rows(seqs, rows, *, window, page_size, dtype, seed=0, writable=False):
    """Cache rows [tokens, width] of some sequences scattered over pages handed out in random order (one key/value
    head whose rows are keys and values at once); slots never written hold NaN; a table row starts at the first page
    the window still needs.  `seqs`: (tokens before the step, tokens of the step)."""
    from flambeau_b200.cache.manager import LayerCacheView
    g = torch.Generator().manual_seed(seed)
    width = rows[0].shape[1]
    first = [max(0, ctx - window + 1) // page_size if window else 0 for ctx, _ in seqs]
    count = [-(-(ctx + n) // page_size) - fp for (ctx, n), fp in zip(seqs, first)]
    total = sum(count) + 3
    order = torch.randperm(total, generator=g).tolist()
    table = torch.full((len(seqs), max(count) + 1), -1, dtype=torch.int32)
    pool = torch.full((total, 1, page_size, width), float("nan"), dtype=dtype)
    for s, ((ctx, n), fp) in enumerate(zip(seqs, first)):
        for j in range(count[s]):
            page = order.pop()
            table[s, j] = page
            lo = (fp + j) * page_size
            hi = min(lo + page_size, ctx + n)
            pool[page, 0, :hi - lo] = rows[s][lo:hi].to(dtype)
    pool = pool.to(DEV)
    return LayerCacheView(pool, pool, table.to(DEV), i32(first), page_size, writable, 0, None), table, first


@pytest.mark.parametrize("sizes", [(24, 40, 8, 8), (80, 96, 16, 16), (8, 20, 6, 6), (56, 48, 16, 10), (16, 64, 0, 0)], ids=str)
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_latents_are_normed_turned_and_written_to_their_pages(sizes, dtype):
    """Shares of the stacked projection in; the query's latent out; the token's cache row [latent | rotated key part]
    in its page, at positions across page borders; a reader of another layer's cache writes nothing."""
    from flambeau_b200.kernels import ops
    Rq, Rc, r, dims = sizes
    dt = DT[dtype]
    g = torch.Generator().manual_seed(Rq)
    page, eps, base = 8, 1e-4, 300.0
    positions = [0, 1, 7, 8, 9, 33, 34, 1000, 1001]
    n = len(positions)
    kv_off = Rq + 3                                            # (other columns may lie between the two latents)
    cols = kv_off + Rc + r + 5
    shares = torch.randn(3, n, cols, generator=g) * 3
    proj = shares.sum(0).double()
    wq, wc = (torch.randn(Rq, generator=g) + 1).to(dt), (torch.randn(Rc, generator=g) - 1).to(dt)
    freqs, mag = pf.rotary_frequencies({"base": base, "dims": dims, "scaling": {"factor": 3.0, "original": 8, "fast": 4.0, "slow": 1.0}}) \
        if dims else (torch.zeros(0, dtype=F64), 1.0)
    want_cq = pf.unit_rms(proj[:, :Rq], eps) * wq.double()
    want_c = pf.unit_rms(proj[:, kv_off:kv_off + Rc], eps) * wc.double()
    want_kr = pf.rotate_neighbours(proj[:, kv_off + Rc:kv_off + Rc + r], positions, freqs, mag) if dims else \
        proj[:, kv_off + Rc:kv_off + Rc + r]
    cache, table, _ = paged_rows([(0, max(positions) + 1)], [torch.zeros(max(positions) + 1, Rc + r)], window=0,
                                 page_size=page, dtype=dt, writable=True)
    half = dims // 2
    ang = torch.tensor(positions, dtype=F64)[:, None] * freqs[None]
    cos, sin = (torch.cos(ang) * mag).float().to(DEV), (torch.sin(ang) * mag).float().to(DEV)
    cq = torch.empty((n, Rq), dtype=dt, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    sh = shares.to(DEV).contiguous()
    ops.mla_latents(sh[0], Rq, wq.to(DEV), cq, kv_off, Rc, r, wc.to(DEV), eps, cos if half else None,
                    sin if half else None, half, cache, i32(positions), i32([0] * n), status, n_partials=3,
                    partial_stride=sh.stride(0))
    assert int(status.item()) == 0
    tol = 1e-5 if dtype == "float32" else 1e-2
    assert rel_err(cq, want_cq) < tol
    for row, p in enumerate(positions):
        got = cache.k_pool[int(table[0, p // page]), 0, p % page]
        assert rel_err(got[:Rc], want_c[row]) < tol
        if r:
            assert rel_err(got[Rc:], want_kr[row]) < tol
    before = cache.k_pool.clone()
    cache.writable = False
    cq.zero_()
    ops.mla_latents(sh[0], Rq, wq.to(DEV), cq, kv_off, Rc, r, None, eps, cos if half else None, sin if half else None,
                    half, cache, i32(positions), i32([0] * n), status, n_partials=3, partial_stride=sh.stride(0))
    assert rel_err(cq, want_cq) < tol and torch.equal(before.nan_to_num(7.0), cache.k_pool.nan_to_num(7.0))


@pytest.mark.parametrize("shape", [(3, 24, 40, 0), (4, 32, 96, 16), (20, 4, 20, 6), (1, 130, 70, 8), (2, 96, 33, 0)], ids=str)
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rows", [(13, 2), (150, 1), (70, 3)], ids=str)
def test_a_map_per_head(shape, dtype, rows):
    """out_h = W_h a_h for every head, the input as shares or as one array; behind the map either a turned tail of
    the head that is copied along, or a sigmoid gate.  Few rows in two shares, several row tiles in one share, and a
    ragged second tile in three."""
    from flambeau_b200.kernels import ops
    H, K, N, rot = shape
    dt = DT[dtype]
    g = torch.Generator().manual_seed(H * K)
    n, parts = rows
    w = (torch.randn(H, N, K, generator=g) * 0.3).to(dt)
    positions = list(range(100, 100 + n))
    freqs, mag = pf.rotary_frequencies({"base": 50.0, "dims": rot}) if rot else (None, 1.0)
    shares = torch.randn(parts, n, H * (K + rot) + 8, generator=g)
    a = shares.sum(0).double()[:, :H * (K + rot)].reshape(n, H, K + rot)
    want = torch.einsum("hnk,thk->thn", w.double(), a[..., :K])
    if rot:
        want = torch.cat([want, pf.rotate_neighbours(a[..., K:], positions, freqs, mag)], dim=-1)
    out = torch.empty((n, H * (N + rot)), dtype=dt, device=DEV)
    cos = sin = None
    if rot:
        ang = torch.tensor(positions, dtype=F64)[:, None] * freqs[None]
        cos, sin = torch.cos(ang).float().to(DEV), torch.sin(ang).float().to(DEV)
    sh = shares.to(DEV).contiguous()
    ops.head_linear(sh[0], K + rot, w.to(DEV), out, N + rot, n, n_partials=parts, partial_stride=sh.stride(0), cos=cos,
                    sin=sin, half=rot // 2, rot=rot)
    tol = 1e-5 if dtype == "float32" else 1.5e-2
    assert rel_err(out, want.reshape(n, -1)) < tol
    # the second use: an input in the engine's dtype, a gate that arrives as shares at an offset
    a2 = torch.randn(n, H * (K + 8), generator=g).to(dt)
    gate = torch.randn(2, n, 5 + H * N + 3, generator=g)
    want = torch.einsum("hnk,thk->thn", w.double(), a2.double().reshape(n, H, K + 8)[..., :K]).reshape(n, H * N) \
        * torch.sigmoid(gate.sum(0).double()[:, 5:5 + H * N])
    out = torch.empty((n, H * N), dtype=dt, device=DEV)
    gd = gate.to(DEV).contiguous()
    ops.head_linear(a2.to(DEV), K + 8, w.to(DEV), out, N, n, gate=gd[0], gate_off=5, gate_partials=2,
                    gate_partial_stride=gd.stride(0))
    assert rel_err(out, want) < tol


LATENT_GEOMETRIES = [(4, 112, 136, 16), (20, 26, 1, 16), (1, 64, 500, 32), (3, 48, 20, 8), (2, 64, 40, 64), (8, 160, 33, 16),
                     (32, 64, 40, 16), (24, 128, 100, 32), (17, 64, 30, 16)]   # (more than 16 heads on the one key/value head)


@pytest.mark.parametrize("geometry", LATENT_GEOMETRIES, ids=lambda g: "h%d-row%d-w%d-p%d" % g)
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_whose_cache_rows_are_keys_and_values(geometry, dtype):
    """All heads over one key/value head whose cache rows serve as keys and as values.  Sequences that are first
    tokens, decoded tokens far into a request and at page borders, portions starting in mid-page beyond the window and
    portions of two tokens.  For the first and the last query of each, the key at the window's far edge is made to
    dominate and the key one further (just outside) even more: if that one were seen it would take the softmax over."""
    from flambeau_b200.kernels import ops
    nh, hd, window, page = geometry
    dt = DT[dtype]
    seqs = [(0, 1), (0, 37), (199, 1), (page * 3 - 1, 1), (page * 3, 1), (page * 2 + 5, 29), (150, 2), (63, 70), (10, 300)]
    g = torch.Generator().manual_seed(5)
    scale = 0.9 / math.sqrt(hd)
    qs, ks = [], []
    for ctx, n in seqs:
        T = ctx + n
        q = torch.randn(n, nh, hd, generator=g).to(dt).double()
        k = torch.randn(T, hd, generator=g).to(dt).double()
        for row in {0, n - 1}:
            p = ctx + row
            unit = q[row, 0] / (q[row, 0] ** 2).sum()
            edge = p - window + 1
            if edge >= 0:
                k[edge] = (unit * 12.0 / scale).to(dt).double()
            if edge - 1 >= 0:
                k[edge - 1] = (unit * 30.0 / scale).to(dt).double()
        qs.append(q)
        ks.append(k)
    cache, _, _ = paged_rows(seqs, ks, window=window, page_size=page, dtype=dt)
    want = []
    for (ctx, n), q, k in zip(seqs, qs, ks):
        i = torch.arange(ctx, ctx + n)[:, None]
        j = torch.arange(ctx + n)[None, :]
        seen = (i - j >= 0) & (i - j < window)
        s = (torch.einsum("ihd,jd->hij", q, k) * scale).masked_fill(~seen[None], -math.inf)
        want.append(torch.einsum("hij,jd->ihd", torch.softmax(s, -1), k).reshape(n, nh * hd))
    want = torch.cat(want)
    lens = [n for _, n in seqs]
    starts = [sum(lens[:i]) for i in range(len(lens))]
    q_d = torch.cat([q.reshape(q.shape[0], -1) for q in qs]).to(dt).to(DEV).contiguous()
    out = torch.empty((sum(lens), nh * hd), dtype=dt, device=DEV)
    rt = SimpleNamespace(status=torch.zeros(1, dtype=torch.int32, device=DEV))
    batch = SimpleNamespace(n_seqs=len(seqs), seq_q_len=lens, seq_q_start_d=i32(starts), seq_q_len_d=i32(lens),
                            seq_pos_start_d=i32([c for c, _ in seqs]), max_q_len=max(lens),
                            max_kv_len=max(c + n for c, n in seqs), multi_seqs_d=None, n_multi=0,
                            positions=i32([p for c, n in seqs for p in range(c, c + n)]),
                            row_seq=i32([s for s, n in enumerate(lens) for _ in range(n)]))
    ops.paged_attention(SimpleNamespace(batch=batch, runtime=rt), q_d, out, cache, nh, 1, hd, window, scale, vd=hd,
                        weights_float32=True)
    assert int(rt.status.item()) == 0
    assert rel_err(out, want) < (2e-5 if dtype == "float32" else 1.5e-2)


# ---------------------------------------------------------------------------------------------------------------
# parts alone, through the step context, cache and state slots the engine uses
# ---------------------------------------------------------------------------------------------------------------
def run_mixer_in_steps(bench, parts, H, steps, width):
    """parts: [(part, call index)] run one after the other on the same rows (an owner of cache rows, then readers);
    returns per part {request: [T, width] float64}."""
    got = [{k: torch.zeros(len(v), width, dtype=F64) for k, v in H.items()} for _ in parts]
    for step in steps:
        ctx, _ = bench.begin([(rid, [1] * k, []) for rid, _, k in step], width)
        h = torch.cat([H[rid][s:s + k] for rid, s, k in step]).cuda()
        for i, (part, call) in enumerate(parts):
            ctx.pending_slabs = 1
            part.forward(ctx, h, ctx.delta, call)
            out = ctx.delta_slabs[:ctx.pending_slabs].sum(0).double().cpu()
            row = 0
            for rid, s, k in step:
                got[i][rid][s:s + k] = out[row:row + k]
                row += k
        bench.end()
    return got


STEPS = [[("a", 0, 17)], [("a", 17, 11), ("b", 0, 20)], [("a", 28, 1), ("b", 20, 1)], [("a", 29, 2), ("b", 21, 2)],
         [("a", 31, 1)], [("a", 32, 40), ("b", 23, 1)], [("a", 72, 1)]]


@pytest.mark.parametrize("sizes", [(2, 16, 8, 24, 40, 24, 9, 20), (4, 32, 16, 32, 96, 80, 30, 30), (20, 4, 6, 8, 20, 40, 1, 1),
                                   (1, 32, 16, 32, 48, 56, 500, 40), (3, 8, 0, 16, 24, 16, 5, 64)], ids=str)
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_latent_attention_part_and_a_reader_of_its_cache(sizes, dtype):
    """A mixer that owns its cache rows and one that reads them (its own heads, query latent, window, no map to the
    latents), over steps of portions, single tokens and two tokens of two requests, against whole sequences."""
    from test_parts_gpu import Bench, bind_random
    from flambeau_b200.cache.manager import CallPlan
    from flambeau_b200.parts.latent_attention import LatentAttention
    from flambeau_b200.parts.spec import PartSpec
    H, d, r, e, Rc, Rq, W, W2 = sizes
    width, eps, scale = 40, 1e-5, 0.3
    stretch = {"factor": 4.0, "original": 16, "fast": 8.0, "slow": 1.0}
    pos = PartSpec("position", "rotary_neighbours", dict(head_dim=r, theta=1e4, rotary_dim=r, stretch=stretch)) if r else None
    std = 0.3 if dtype == "float32" else 0.15
    own_kw = dict(width=width, num_heads=H, head_dim=d, rot_dim=r, value_dim=e, kv_rank=Rc, q_rank=Rq, window=W,
                  scale=scale, eps=eps, position=pos, keep_window=max(W, W2), init_std=std)
    read_kw = dict(width=width, num_heads=H + 1, head_dim=d + 8, rot_dim=r, value_dim=e + 8, kv_rank=Rc, q_rank=Rq + 8,
                   window=W2, scale=scale * 0.7, eps=eps, position=pos, shares_latent=True, init_std=std)
    owner = LatentAttention(None, "o.", **own_kw)
    b = Bench(dtype, plans=[CallPlan(kv=owner.cache_requirement()), CallPlan(cache_from=0)])
    owner, reader = LatentAttention(b.rt, "o.", **own_kw), LatentAttention(b.rt, "r.", **read_kw)
    Wt = dict(bind_random(owner, DT[dtype]), **bind_random(reader, DT[dtype], seed=1))
    assert "r.dkv" not in Wt and "o.dkv" in Wt
    g = torch.Generator().manual_seed(2)
    Hs = {"a": torch.randn(73, width, generator=g).to(DT[dtype]), "b": torch.randn(24, width, generator=g).to(DT[dtype])}
    got_o, got_r = run_mixer_in_steps(b, [(owner, 0), (reader, 1)], Hs, STEPS, width)
    rot = {"base": 1e4, "dims": r, "scaling": stretch}
    m_own = {"heads": H, "dim": d, "rot_dim": r, "vdim": e, "kv_rank": Rc, "mask": {"size": W}, "rot": rot, "scale": scale}
    m_read = {"heads": H + 1, "dim": d + 8, "rot_dim": r, "vdim": e + 8, "kv_rank": Rc, "mask": {"size": W2}, "rot": rot,
              "scale": scale * 0.7}
    tol = 2e-5 if dtype == "float32" else 2e-2
    for rid, h in Hs.items():
        positions = list(range(len(h)))
        want, latent = pf.latent_attention(h.double(), Wt, "o.", m_own, eps, positions)
        assert rel_err(got_o[rid], want) < tol, rid
        want, _ = pf.latent_attention(h.double(), Wt, "r.", m_read, eps, positions, latent=latent)
        assert rel_err(got_r[rid], want) < tol, rid


@pytest.mark.parametrize("sizes", [(2, 24, 16, 8.0), (4, 48, 32, 16.0), (1, 40, 8, 2.0), (3, 12, 20, 1.0), (2, 136, 72, 30.0),
                                   (1, 300, 24, 4.0), (2, 50, 24, 4.0)], ids=str)
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gated_linear_attention_part_across_steps(sizes, dtype):
    """The mixer alone with its float32 state slots, two requests in portions, single tokens and pairs; then the
    request's slot is given back, taken by a new request and must start from zero."""
    from test_parts_gpu import Bench, bind_random
    from flambeau_b200.cache.manager import CallPlan
    from flambeau_b200.parts.linear_attention import GatedLinearAttention
    H, dk, dv, tau = sizes
    width, eps = 40, 1e-5
    kw = dict(width=width, num_heads=H, key_dim=dk, value_dim=dv, tau=tau, eps=eps, decay_rank=6,
              init_std=0.3 if dtype == "float32" else 0.15)
    part = GatedLinearAttention(None, "m.", **kw)
    b = Bench(dtype, plans=[CallPlan(state=part.state_requirement())])
    part = GatedLinearAttention(b.rt, "m.", **kw)
    Wt = bind_random(part, DT[dtype])
    g = torch.Generator().manual_seed(3)
    Hs = {"a": torch.randn(73, width, generator=g).to(DT[dtype]), "b": torch.randn(24, width, generator=g).to(DT[dtype])}
    (got,) = run_mixer_in_steps(b, [(part, 0)], Hs, STEPS, width)
    m = {"heads": H, "dim": dk, "vdim": dv, "tau": tau}
    tol = 2e-5 if dtype == "float32" else 2e-2
    for rid, h in Hs.items():
        assert rel_err(got[rid], pf.gated_linear_attention(h.double(), Wt, "m.", m, eps)) < tol, rid
    decays = pf.channel_decays(Hs["a"].double(), Wt, "m.", m)
    assert float(decays.median()) < 0.9995 and float(decays.std()) > 0.003, \
        "decays that all vanish or all stay at one would hide a lost state"
    for rid in ("a", "b"):
        b.engine.cache.release(rid)
    (again,) = run_mixer_in_steps(b, [(part, 0)], {"c": Hs["b"]}, [[("c", 0, 3)], [("c", 3, 21)]], width)
    assert rel_err(again["c"], pf.gated_linear_attention(Hs["b"].double(), Wt, "m.", m, eps)) < tol


@pytest.mark.parametrize("shape", [(5, 64, 6, 2, 3, 24, 40, 1.5), (300, 96, 40, 1, 5, 16, 0, 1.0), (33, 32, 3, 3, 2, 32, 16, 0.5),
                                   (2, 48, 4, 0, 1, 20, 0, 2.0), (700, 64, 8, 4, 4, 40, 24, 2.0), (1, 64, 1, 1, 2, 8, 8, 1.0)], ids=str)
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_routed_experts_scored_over_all_with_identity_experts(shape, dtype):
    """The part alone: scores over all router outputs, the correction that only moves the choice, shares over their
    sum times the router's scale, experts without weights that hand the input on, and a shared expert.  The router's
    map is wide so that choices are rarely close; one correction is large so that it always wins a place."""
    from test_parts_gpu import Bench
    from flambeau_b200.parts.moe import RoutedExperts
    from flambeau_b200.parts.spec import PartSpec
    n, D, E, I, K, ff, shared, scale = shape
    dt = DT[dtype]
    b = Bench(dtype, max_step_tokens=1024, cache_tokens=1024)
    shared_spec = PartSpec("feed_forward", "gated_mlp", dict(width=D, inner=shared, activation="silu",
                                                             names=("gate", "up", "down")), "m.shared.") if shared else None
    part = RoutedExperts(b.rt, "m.", width=D, inner=ff, experts=E, top=K, activation="silu", gated=True,
                         rule="softmax_of_all", weight_scale=scale, identity=I, bias_name="correction", shared=shared_spec)
    g = torch.Generator().manual_seed(n)
    w = {}
    for name, ts in part.tensor_specs().items():
        std = 1.0 if name.endswith("router") else 0.05 if name.endswith("correction") else 0.2
        w[name] = (torch.randn(ts.shape, generator=g) * std).to(dt)
    w["m.correction"][-1] += 2.0                    # the last output (an identity expert where there is one) always wins
    part.bind({k: v.to(DEV) for k, v in w.items()})
    h = torch.randn(n, D, generator=g).to(dt)
    mlp = {"router": {"experts": E, "identity": I, "top": K, "scale": scale}, "shared": {"ff": shared} if shared else None}
    w64 = {k: v.double() for k, v in w.items()}
    want = pf.routed_ff(h.double(), w64, "m.", mlp)
    chosen, _ = pf.route(h.double(), w64, "m.", mlp["router"])
    assert bool((chosen == E + I - 1).any(dim=1).all())
    ctx, _ = b.begin([("a", [1] * n, [])], D)
    ctx.pending_slabs = 1
    part.forward(ctx, h.to(DEV), ctx.delta)
    b.end()
    out = ctx.delta_slabs[:ctx.pending_slabs].sum(0)
    # a token whose choice was close may go to another expert in bfloat16: all but a few rows must agree
    err = (out.double().cpu() - want).abs().max(dim=1).values / want.abs().max()
    tol = 2e-5 if dtype == "float32" else 2e-2
    assert int((err > tol).sum()) <= (0 if dtype == "float32" else n // 50), float(err.max())


# ---------------------------------------------------------------------------------------------------------------
# whole models under schedules
# ---------------------------------------------------------------------------------------------------------------
SHARP = {"float32": 0.25, "bfloat16": 0.12}
LENGTHS = {"FA": [1, 9, 40, 75, 33, 21, 64, 110], "FB": [2, 70, 17, 48, 130, 5], "FC": [30, 3]}


def tolerance(dtype, pcfg, W, requests):
    """(bound on the worst position, bound on the median position), as fractions of the logit scale.  float32: 1e-4
    for both.  bfloat16: three times what rounding alone causes, which the plain implementation measures on the same
    requests by rounding the values a 16-bit engine keeps in 16 bits; never below the 2e-2 and a quarter of it that fit
    the framework's other models."""
    if dtype == "float32":
        return 1e-4, 1e-4
    noise = [pf.rounding_noise(pcfg, W, toks) for toks in requests.values()]
    worst, median = max(w for w, _ in noise), max(m for _, m in noise)
    return max(tiny.TOL["bfloat16"], 3.0 * worst), max(tiny.TOL["bfloat16"] / 4, 3.0 * median)


def compare(got, want, tol, what):
    import numpy as np
    errs = []
    for rid, ref in want.items():
        ref = ref.numpy()
        scale = float(np.abs(ref).max())
        for p in range(ref.shape[0]):
            assert (rid, p) in got, f"{what}: no logits for request {rid} position {p}"
            errs.append((float(np.abs(got[(rid, p)].astype(np.float64) - ref[p]).max()) / scale, rid, p))
    assert all(math.isfinite(e) for e, _, _ in errs), f"{what}: logits that are not finite"
    worst = max(errs)
    median = sorted(e for e, _, _ in errs)[len(errs) // 2]
    print(f"[compare] {what}: worst {worst[0]:.3e} at {worst[1:]}, median {median:.3e} (bounds {tol[0]:.1e}, {tol[1]:.1e})")
    assert worst[0] <= tol[0], f"{what}: error {worst[0]:.3e} of the logit scale at {worst[1:]} exceeds {tol[0]:.1e}"
    assert median <= tol[1], f"{what}: median error {median:.3e} of the logit scale exceeds {tol[1]:.1e}"
    return worst[0]


def make_case(name, cfg, folder, dtype, lengths, seed, request_seed=4):
    ft.make_folder(folder, cfg, seed=seed, dtype=dtype, sharp=SHARP[dtype], steady_router=dtype == "bfloat16")
    requests = tiny.random_requests({"vocab_size": cfg["vocab"]}, lengths, seed=request_seed)
    pcfg, W = pf.read_folder(folder)
    want = {rid: pf.forward(pcfg, W, toks) for rid, toks in requests.items()}
    return dict(name=name, dtype=dtype, cfg=cfg, folder=folder, requests=requests, want=want,
                tol=tolerance(dtype, pcfg, W, requests))


@pytest.fixture(scope="module", params=[(c, d) for c in ("FA", "FB") for d in ("float32", "bfloat16")],
                ids=lambda p: f"{p[0]}-{p[1]}")
def case(request, tmp_path_factory):
    name, dtype = request.param
    return make_case(name, ft.CONFIGS[name], tmp_path_factory.mktemp(f"f{name}{dtype}"), dtype, LENGTHS[name],
                     seed=17 if name == "FA" else 29)


def run(case, schedule, tmp_path, cuda_graphs=True):
    from flambeau_b200.engine.step import Engine, EngineOptions
    from flambeau_b200.engine.trace import replay
    tokens = schedule.max_live_tokens(case["requests"])
    engine = Engine.from_folder(case["folder"], EngineOptions(
        dtype=case["dtype"], cache_tokens=tokens, max_requests=4, max_step_tokens=max(tokens, 128),
        max_seq_len=max(tokens, 192), cuda_graphs=cuda_graphs))
    replay(engine, schedule.lines(), tmp_path)
    run.last_engine = engine
    engine.cache.check_invariants()
    assert not engine.cache.requests, "requests left live after the trace"
    assert all(g.pool.n_free == g.pool.n_pages for g in engine.cache.groups), "pages lost"
    got = tiny.read_rows(tmp_path, schedule, case["cfg"]["vocab"])
    return compare(got, case["want"], case["tol"], f"{case['name']} {case['dtype']}")


def test_whole(case, tmp_path):
    run(case, tiny.schedule_whole(case["requests"]), tmp_path)


def test_last_tokens_one_by_one_past_the_windows(case, tmp_path):
    """The tail is longer than FA's windows (9 and 20) and than two of FB's (1 and 40), so windows pass over decoded
    tokens and the cache gives pages back while decoding."""
    run(case, tiny.schedule_tail(case["requests"], 45), tmp_path)


def test_portions_down_to_two_tokens(case, tmp_path):
    """Portions shorter than the taps of the convolutions follow each other; portions end inside windows and pages."""
    run(case, tiny.schedule_portions(case["requests"]), tmp_path)
    run(case, tiny.schedule_portions(case["requests"], sizes=(2, 31, 2, 2, 17, 64, 3)), tmp_path / "b")


@pytest.mark.parametrize("seed", [1, 2])
def test_mixed_batches_with_pages_and_slots_used_again(case, tmp_path, seed):
    sched = tiny.schedule_mixed(case["requests"], seed=seed)
    total_pages = sum(-(-len(t) // 16) for t in case["requests"].values())
    assert sched.max_live_tokens(case["requests"]) // 16 < total_pages, "the pool must be smaller than all requests"
    assert len(case["requests"]) > 4, "more requests than slots, so that slots are used again"
    run(case, sched, tmp_path)


def test_every_token_decoded_from_the_first(case, tmp_path):
    """One token a step from position 0 (replayed from CUDA graphs where the engine captures them): the first tokens
    of a sequence, where the convolutions read zeros and the state is empty, and a long decoding."""
    rid = max(case["requests"], key=lambda r: len(case["requests"][r]))
    toks = case["requests"][rid]
    s = tiny.Schedule()
    for p, t in enumerate(toks):
        s.add([(rid, [t], [0], p)], end=[rid] if p == len(toks) - 1 else [])
    one = dict(case, requests={rid: toks}, want={rid: case["want"][rid]})
    run(one, s, tmp_path)
    assert run.last_engine.graph_replays > len(toks) // 2, "single-token steps are replayed from a captured graph"


def test_a_reader_right_behind_its_owner(tmp_path):
    c = make_case("FC", ft.CONFIGS["FC"], tmp_path / "m", "float32", LENGTHS["FC"], seed=3, request_seed=2)
    run(c, tiny.schedule_portions(c["requests"], sizes=(5, 2, 9)), tmp_path / "o")
    run(c, tiny.schedule_tail(c["requests"], 12), tmp_path / "t")


def random_config(seed: int) -> dict:
    """A configuration drawn from a seed: widths that are and are not multiples of 8, odd head sizes, windows from one
    key to beyond the requests, rotated parts from none to larger than the unrotated, one to five taps, experts with
    and without identity and shared ones, layers without feed-forward, readers of earlier layers' latents."""
    import random
    rng = random.Random(seed)
    width = rng.choice([40, 72, 100, 128, 36])
    owners = {}
    layers = []
    for i in range(rng.randint(1, 5)):
        mlp = None
        roll = rng.random()
        if roll < 0.4:
            mlp = ft.dense(rng.choice([24, 40, 100]))
        elif roll < 0.85:
            experts, identity = rng.randint(1, 10), rng.choice([0, 0, 1, 3])
            mlp = ft.moe(experts, identity, rng.randint(1, min(experts + identity, 4)), rng.choice([8, 16, 24, 40]),
                         rng.choice([1.0, 2.5, 0.5]), rng.choice([None, 8, 32]))
        if rng.random() < 0.5:
            layers.append(ft.layer(rng.choice(["gla", "gla_2"]),
                                   ft.linear(rng.choice([1, 2, 3, 5]), rng.choice([4, 12, 16, 36, 72]),
                                             rng.choice([8, 12, 16, 40]), rng.choice([1.0, 4.0, 16.0])), mlp))
            continue
        heads, d, e = rng.choice([1, 2, 3, 6]), rng.choice([4, 8, 12, 16, 32]), rng.choice([8, 12, 16, 24])
        window = rng.choice([1, 2, 5, 16, 17, 31, 64, 500])
        if owners and rng.random() < 0.5:
            src = rng.choice(sorted(owners))
            r, Rc, base, scaling = owners[src]
            mixer = ft.latent(heads, d, r, e, Rc, rng.choice([8, 20, 32]), window, base, rng.uniform(0.1, 0.4), scaling, kv_from=src)
        else:
            r, Rc, base = rng.choice([0, 2, 4, 8, 16]), rng.choice([8, 20, 24, 48, 64]), rng.choice([100.0, 1e4, 5e5])
            scaling = rng.choice([None, (2.0, 32, 4.0, 1.0), (16.0, 16, 32.0, 0.5)])
            owners[i] = (r, Rc, base, scaling)
            mixer = ft.latent(heads, d, r, e, Rc, rng.choice([8, 20, 32]), window, base, rng.uniform(0.1, 0.4), scaling)
        layers.append(ft.layer("latent_attention", mixer, mlp))
    cfg = {"architecture": "Fegizen", "canon": {"taps": rng.randint(1, 5)}, "embedding": {"scale": rng.uniform(0.3, 3.0)},
           "norm": {"eps": rng.choice([1e-5, 1e-6])}, "vocab": rng.randint(50, 400), "width": width, "layers": layers}
    if rng.random() < 0.7:
        cfg["logit_scale"] = rng.choice([0.25, 2.0])
    return cfg


@pytest.mark.parametrize("seed", [201, 202, 203, 204, 205, 206, 207, 208])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_random_configurations_under_a_mixed_schedule(tmp_path, seed, dtype):
    cfg = random_config(seed)
    c = make_case(f"random {seed}", cfg, tmp_path / "m", dtype, [1, 37, 80, 2, 55, 21], seed=seed, request_seed=seed)
    run(c, tiny.schedule_mixed(c["requests"], seed=seed), tmp_path / "o")


def logits_at_the_end(folder, tokens, cut, dtype="float32"):
    """The last position's logits, the request fed as tokens[:cut] and then the rest (a single token when cut is
    len - 1: the position is then a decoded one)."""
    from flambeau_b200.engine.step import Engine, EngineOptions
    engine = Engine.from_folder(folder, EngineOptions(dtype=dtype, cache_tokens=1024, max_requests=2, max_step_tokens=512))
    engine.step([("a", tokens[:cut], [])])
    return engine.step([("a", tokens[cut:], [len(tokens) - cut - 1])], end=["a"])[0].double().cpu()


@pytest.mark.parametrize("window", [1, 11, 16, 17, 70])
def test_the_window_ends_where_it_should_in_prompts_and_in_decoding(tmp_path, window):
    """One latent-attention layer, one tap, no feed-forward, float32: a token then reaches later positions through its
    cache row alone.  Changing the token just outside the last query's window leaves its logits as they were; changing
    the one just inside moves them.  The last position is once part of a portion, once a decoded token; windows that
    end at, before and behind a page border."""
    cfg = {"architecture": "Fegizen", "canon": {"taps": 1}, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-5},
           "vocab": 150, "width": 48,
           "layers": [ft.layer("latent_attention", ft.latent(3, 8, 8, 16, 24, 16, window, 1e4, 0.3, (4.0, 16, 8.0, 1.0)), None)]}
    folder = ft.make_folder(tmp_path / "m", cfg, seed=8, dtype="float32")
    base = tiny.random_requests({"vocab_size": cfg["vocab"]}, [100], seed=1)["r0"]
    p = len(base) - 1

    def changed(at):
        t = list(base)
        t[at] = (t[at] + 1) % cfg["vocab"]
        return t
    for cut in (60, p - 1, p):                      # (p: the last token is decoded alone)
        ref = logits_at_the_end(folder, base, cut)
        scale = float(ref.abs().max())
        assert float((logits_at_the_end(folder, changed(p - window), cut) - ref).abs().max()) / scale < 1e-5, cut
        if window > 1:
            assert float((logits_at_the_end(folder, changed(p - window + 1), cut) - ref).abs().max()) / scale > 1e-4, cut
    pcfg, W = pf.read_folder(folder)
    assert rel_err(logits_at_the_end(folder, base, 37), pf.forward(pcfg, W, base)[-1]) < 1e-4


def test_the_state_carries_a_far_token_and_a_freed_slot_forgets_it(tmp_path):
    """One linear-attention layer, float32: a token hundreds of positions back still moves the last logits (the
    state has carried it, through portions and single tokens); a second request in the slot the first one gave back
    gets the logits of a request that runs alone."""
    from flambeau_b200.engine.step import Engine, EngineOptions
    cfg = {"architecture": "Fegizen", "canon": {"taps": 2}, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-5},
           "vocab": 150, "width": 48, "layers": [ft.layer("gla", ft.linear(2, 16, 24, 64.0), ft.dense(40))]}
    folder = ft.make_folder(tmp_path / "m", cfg, seed=9, dtype="float32")
    base = tiny.random_requests({"vocab_size": cfg["vocab"]}, [300], seed=2)["r0"]
    other = list(base)
    other[3] = (other[3] + 1) % cfg["vocab"]
    ref = logits_at_the_end(folder, base, 280)
    assert float((logits_at_the_end(folder, other, 299) - ref).abs().max()) / float(ref.abs().max()) > 1e-4
    pcfg, W = pf.read_folder(folder)
    assert rel_err(ref, pf.forward(pcfg, W, base)[-1]) < 1e-4
    engine = Engine.from_folder(folder, EngineOptions(dtype="float32", cache_tokens=512, max_requests=1, max_step_tokens=512))
    engine.step([("a", other, [])], end=["a"])
    again = engine.step([("b", base, [len(base) - 1])], end=["b"])[0].double().cpu()
    assert float((again - ref).abs().max()) / float(ref.abs().max()) < 1e-5


def test_a_far_key_among_hundreds_is_found(tmp_path):
    """A window longer than the request, float32.  One head's maps are rebuilt so that its query for one token points
    along another token's latent (its rotated part switched off): where the first stands last and the second hundreds
    of positions back and nowhere else, that far key takes most of the head's softmax, so that losing the key, or its
    page, would move the logits by far more than any rounding."""
    cfg = {"architecture": "Fegizen", "canon": {"taps": 1}, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-5},
           "vocab": 90, "width": 32,
           "layers": [ft.layer("latent_attention", ft.latent(2, 8, 4, 8, 16, 8, 1000, 1e4, 1.0), None)]}
    folder = ft.make_folder(tmp_path / "m", cfg, seed=10, dtype="float32", sharp=0.3)
    pcfg, W = pf.read_folder(folder)
    m, eps, asks, answers = cfg["layers"][0]["mixer"], 1e-5, 85, 84
    h = pf.add_time_conv(pf.centred_norm(pf.embed([asks, answers], W["embed"], 1.0), W["l0.norm1"], eps), W["l0.canon1"])
    c, _ = pf.latent_keys(h[1:], W, "l0.mix.", m, eps, [0])
    cq = pf.unit_rms(h[:1] @ W["l0.mix.dq"].T, eps) * W["l0.mix.dq.norm"]
    tensors = ft.read_tensors(folder)
    uk, uq = tensors["l0.mix.uk"], tensors["l0.mix.uq"]
    uk[:8] = 0.0
    uk[0] = (c[0] / c[0].norm()).float()
    uq[:12] = 0.0
    uq[0] = (3.0 * cq[0] / cq[0].norm()).float()
    ft.write_tensors(folder, tensors)
    pcfg, W = pf.read_folder(folder)
    base = tiny.random_requests({"vocab_size": 80}, [400], seed=3)["r0"]      # tokens from 80 on are kept for the far key
    far = list(base)
    far[7], far[-1] = answers, asks
    want = pf.forward(pcfg, W, far)[-1]
    for cut in (150, len(far) - 1):
        assert rel_err(logits_at_the_end(folder, far, cut), want) < 1e-4
    moved = list(far)
    moved[7] = 86
    assert float((pf.forward(pcfg, W, moved)[-1] - want).abs().max()) / float(want.abs().max()) > 2e-2, \
        "the far key does not matter in this model: the test would show nothing"


# ---------------------------------------------------------------------------------------------------------------
# generation through the entry point and the scheduler
# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name,dtype", [("FA", "float32"), ("FB", "bfloat16")])
def test_greedy_generation(tmp_path, name, dtype):
    from flambeau_b200 import generate
    cfg = ft.CONFIGS[name]
    folder = ft.make_folder(tmp_path / "m", cfg, seed=41, dtype=dtype, sharp=SHARP[dtype], steady_router=dtype == "bfloat16")
    pcfg, W = pf.read_folder(folder)
    prompts = list(tiny.random_requests({"vocab_size": cfg["vocab"]}, [3, 26, 50, 1, 12], seed=6).values())
    n_new = 10
    outs = generate(folder, prompts, max_tokens=n_new, temperature=0.0, dtype=dtype, prefill_chunk_tokens=16,
                    prefill_ubatch=40, inflight_slots=3)
    tol = tolerance("bfloat16", pcfg, W, {i: p for i, p in enumerate(prompts)})[0]
    for prompt, out in zip(prompts, outs):
        assert len(out) == n_new
        toks = list(prompt)
        for t in out:
            logits = pf.forward(pcfg, W, toks)[-1]
            best = float(logits.max())
            if dtype == "float32":
                assert t == int((logits == best).nonzero()[0]), "greedy token differs from the plain implementation"
            else:
                gap = float(best - logits[t]) / float(logits.abs().max())
                assert gap <= 2 * tol, f"token {t} is {gap:.3f} of the scale below the best logit"
            toks.append(t)


def test_command_line_infer_and_replay(tmp_path):
    """The programs a user runs: `flambeau infer` (greedy, float32: the tokens are the plain implementation's) and
    `bin/trace_run` fed two requests step by step (their last logits are the plain implementation's)."""
    import json
    import subprocess
    import sys
    from pathlib import Path
    import numpy as np
    root = Path(__file__).resolve().parent.parent
    cfg = ft.CONFIGS["FC"]
    folder = ft.make_folder(tmp_path / "m", cfg, seed=12, dtype="float32")
    pcfg, W = pf.read_folder(folder)
    prompt = tiny.random_requests({"vocab_size": cfg["vocab"]}, [14], seed=3)["r0"]
    proc = subprocess.run([sys.executable, str(root / "bin" / "flambeau"), "infer", "--model", str(folder), "--max-tokens",
                           "4", "--dtype", "float32", "--prompt", ",".join(map(str, prompt))],
                          capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    out = [int(t) for t in proc.stdout.strip().splitlines()[-1].split(",")]
    toks = list(prompt)
    for t in out:
        logits = pf.forward(pcfg, W, toks)[-1]
        assert t == int((logits == logits.max()).nonzero()[0])
        toks.append(t)
    other = tiny.random_requests({"vocab_size": cfg["vocab"]}, [9], seed=5)["r0"]
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": prompt[:6], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": prompt[6:13], "want": []},
                                     {"id": "b", "tokens": other[:8], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "b", "tokens": other[8:], "want": [0]},
                                     {"id": "a", "tokens": prompt[13:], "want": [0]}], "end": ["a", "b"]}]
    proc = subprocess.run([str(root / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32", "--out",
                           str(tmp_path / "o"), "--max-tokens", "128"], input="\n".join(json.dumps(x) for x in steps) + "\n",
                          capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [ln for ln in proc.stdout.splitlines() if ln.startswith("done")] == ["done 0", "done 1", "done 2"]
    got = np.fromfile(tmp_path / "o" / "2.f32", dtype="<f4").reshape(2, cfg["vocab"])
    for row, seq in zip(got, (other, prompt)):
        assert rel_err(torch.from_numpy(row.copy()), pf.forward(pcfg, W, seq)[-1]) < 1e-4
