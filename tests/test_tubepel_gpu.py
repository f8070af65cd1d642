"""Tubepel on the GPU against the plain implementation (tests/plain_tubepel.py): each mechanism alone through its
kernels and parts, then whole models under schedules (whole, token by token, portions down to two tokens, mixed
batches on a pool so small that pages and slots are used again), the edges of windows and of the kept first keys in
prompts and in decoding, a far key among hundreds, long decoding, random configurations, and greedy generation through
generate()."""
import math
from types import SimpleNamespace

import pytest
import torch

import plain_tubepel as pt
import tiny
import tubepel_tiny as tt

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
F64 = torch.float64


def rel_err(got, want):
    return float((got.double().cpu() - want).abs().max() / want.abs().max())


def i32(values):
    return torch.tensor(values, dtype=torch.int32, device=DEV)


# ---------------------------------------------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("shape", [(1, 8, 1), (2, 192, 2), (3, 50, 3), (4, 1000, 1), (8, 260, 8), (2, 4100, 4)], ids=str)
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_streams_write_read_and_norm_in_one_pass(shape, dtype):
    """The kernel between two sublayers: the output of the one before (as split-K shares) is written into every copy
    of the stream, the next one's read is formed and normalised.  Also the first sublayer of a step (nothing to
    write), the read alone (float32 rows), and chosen rows that are read and not written back."""
    from flambeau_b200.kernels import ops
    S, D, parts = shape
    n, eps = 37, 1e-5
    g = torch.Generator().manual_seed(S * 1000 + D)
    xs = torch.randn(S, n, D, generator=g) * 3.0
    y = torch.randn(parts, n, D, generator=g)
    w = {"in": torch.randn(S, generator=g), "out": torch.randn(S, generator=g), "mix": torch.randn(S, S, generator=g)}
    nw = (1.0 + 0.1 * torch.randn(D, generator=g)).to(DT[dtype])
    w64 = {k: v.double() for k, v in w.items()}
    new = pt.streams_write(xs.double(), y.double().sum(0), w64, "")
    want_h = pt.rms_norm(pt.streams_read(new, w64, ""), nw.double(), eps)
    wd = {k: v.to(DEV).contiguous() for k, v in w.items()}
    tol = 1e-5 if dtype == "float32" else 6e-3
    xs_d, y_d, out = xs.to(DEV).contiguous(), y.to(DEV).contiguous(), torch.empty(n, D, dtype=DT[dtype], device=DEV)
    ops.hc_step(xs_d, y_d[0], parts, y_d.stride(0), wd["mix"], wd["out"], wd["in"], nw.to(DEV), eps, 0.0, out, n)
    assert rel_err(xs_d, new) < 1e-6 and rel_err(out, want_h) < tol
    # nothing to write: the copies stay as they are
    xs_d = xs.to(DEV).contiguous()
    ops.hc_step(xs_d, None, 0, 0, None, None, wd["in"], nw.to(DEV), eps, 0.0, out, n)
    assert torch.equal(xs_d.cpu(), xs)
    assert rel_err(out, pt.rms_norm(pt.streams_read(xs.double(), w64, ""), nw.double(), eps)) < tol
    # the read alone, and the sum of the copies at the end of a step, for chosen rows, without writing back
    u = torch.empty(n, D, dtype=torch.float32, device=DEV)
    ops.hc_step(xs_d, None, 0, 0, None, None, wd["in"], None, 0.0, 0.0, u, n)
    assert rel_err(u, pt.streams_read(xs.double(), w64, "")) < 1e-6
    rows = [5, 0, 36, 5]
    ops.hc_step(xs_d, y_d[0], parts, y_d.stride(0), wd["mix"], wd["out"], None, None, 0.0, 0.0, u, n, rows=i32(rows))
    assert torch.equal(xs_d.cpu(), xs), "chosen rows are read, the copies are not touched"
    assert rel_err(u[:4], new.sum(0)[rows]) < 1e-6


@pytest.mark.parametrize("shape", [(5, 96, 3, 64), (70, 50, 1, 7), (300, 256, 8, 0)], ids=str)
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_output_gate(shape, dtype):
    from flambeau_b200.kernels import ops
    n, I, parts, off = shape
    g = torch.Generator().manual_seed(n)
    a = torch.randn(n, I, generator=g).to(DT[dtype])
    z = torch.randn(parts, n, off + I + 3, generator=g)
    a_d, z_d = a.to(DEV), z.to(DEV)
    ops.sigmoid_gate(a_d, z_d[0][:, off:off + I], n, parts, z_d.stride(0))
    want = a.double() * torch.sigmoid(z.double().sum(0)[:, off:off + I])
    assert rel_err(a_d, want) < (1e-6 if dtype == "float32" else 5e-3)


def paged_keys_and_values(seqs, ks, vs, *, page_size, dtype, seed=0, window=0, keep=0, given_back=False):
    """Keys [tokens, kv heads, d] and values [tokens, kv heads, e] of some sequences scattered over pages handed out
    in random order; slots never written hold NaN.  `seqs`: (tokens before the step, tokens of the step).
    `given_back`: the cache has given back what the window had passed before the step, but for the pages of the kept
    first keys: those pages do not exist (whatever reads them reads NaN), and a table row is the kept pages' columns,
    then the pages from the first live one on."""
    from flambeau_b200.cache.manager import LayerCacheView
    g = torch.Generator().manual_seed(seed)
    G, d, e = ks[0].shape[1], ks[0].shape[2], vs[0].shape[2]
    kept = -(-keep // page_size) if given_back and window and keep else 0
    first = [max(kept, max(0, ctx - window + 1) // page_size) if given_back and window else kept for ctx, _ in seqs]
    count = [-(-(ctx + n) // page_size) for ctx, n in seqs]
    total = sum(count) + 3
    order = torch.randperm(total, generator=g).tolist()
    table = torch.full((len(seqs), max(count) + 1), -1, dtype=torch.int32)
    k_pool = torch.full((total, G, page_size, d), float("nan"), dtype=dtype)
    v_pool = torch.full((total, G, page_size, e), float("nan"), dtype=dtype)
    for s, (ctx, n) in enumerate(seqs):
        for j in range(count[s]):
            if kept <= j < first[s]:
                continue                                    # given back
            page = order.pop()
            table[s, j if j < kept else j - first[s] + kept] = page
            lo, hi = j * page_size, min((j + 1) * page_size, ctx + n)
            k_pool[page, :, :hi - lo] = ks[s][lo:hi].transpose(0, 1).to(dtype)
            v_pool[page, :, :hi - lo] = vs[s][lo:hi].transpose(0, 1).to(dtype)
    return LayerCacheView(k_pool.to(DEV), v_pool.to(DEV), table.to(DEV), i32(first), page_size, False, 0, None, kept)


KEPT_GEOMETRIES = [(8, 2, 64, 64, 120, 3, 16), (4, 2, 16, 24, 9, 2, 16), (6, 1, 64, 64, 70, 66, 16), (2, 2, 128, 128, 40, 130, 32),
                   (8, 4, 32, 32, 33, 17, 8), (3, 3, 24, 8, 20, 1, 16), (2, 1, 8, 8, 1, 1, 16), (4, 4, 64, 64, 100, 64, 64),
                   (2, 1, 40, 40, 30, 0, 16), (20, 1, 64, 64, 50, 5, 16)]


@pytest.mark.parametrize("geometry", KEPT_GEOMETRIES, ids=lambda g: "h%d-g%d-d%d-e%d-w%d-f%d-p%d" % g)
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("given_back", [False, True], ids=["all-pages", "dead-pages-given-back"])
def test_attention_under_a_window_that_keeps_the_first_keys(geometry, dtype, given_back):
    """Grouped heads over the paged cache with a sink in every head.  Sequences that are first tokens, positions just
    behind the window's length (where the kept keys first part from the window), decoded tokens far into a request and
    at page borders, portions starting in mid-page and portions of two tokens.  For the first and the last query of
    each, four keys are made to stand out along the query of head 0: the key at the window's far edge (seen), the one
    just outside it (stronger, not seen), the last kept key (seen) and the first key that is not kept (strongest, not
    seen unless the window reaches it): a mask that is one key off anywhere takes the softmax over.  Once with every
    page in the table, once with the pages between the kept keys and the window given back (reading one is reading
    NaN)."""
    from flambeau_b200.kernels import ops
    nh, nkv, d, e, window, keep, page = geometry
    dt = DT[dtype]
    seqs = [(0, 1), (0, 37), (window, 1), (window + 1, 1), (window + keep, 2), (199, 1), (page * 3 - 1, 1), (page * 3, 1),
            (page * 2 + 5, 29), (150, 2), (63, 70), (10, 300), (window + 40, 1)]
    g = torch.Generator().manual_seed(5)
    scale = 0.9 / math.sqrt(d)
    group = torch.arange(nh) // (nh // nkv)
    qs, ks, vs = [], [], []
    for ctx, n in seqs:
        T = ctx + n
        q = torch.randn(n, nh, d, generator=g).to(dt).double()
        k = torch.randn(T, nkv, d, generator=g).to(dt).double()
        v = torch.randn(T, nkv, e, generator=g).to(dt).double()
        for row in {0, n - 1}:
            p = ctx + row
            unit = q[row, 0] / (q[row, 0] ** 2).sum()
            for at, strength in ((p - window + 1, 12.0), (p - window, 30.0), (keep - 1, 14.0), (keep, 40.0)):
                if 0 <= at <= p and not (at == keep and p - at < window) and not (at == p - window and at < keep):
                    k[at, 0] = (unit * strength / scale).to(dt).double()
        qs.append(q)
        ks.append(k)
        vs.append(v)
    sinks = torch.randn(nh, generator=g)
    cache = paged_keys_and_values(seqs, ks, vs, page_size=page, dtype=dt, window=window, keep=keep, given_back=given_back)
    want = []
    for (ctx, n), q, k, v in zip(seqs, qs, ks, vs):
        seen = pt.visible(ctx + n, window, keep)[ctx:]
        s = torch.einsum("ihd,jhd->hij", q, k[:, group]) * scale
        a = pt.softmax_with_sink(s, seen, sinks.double())
        want.append(torch.einsum("hij,jhe->ihe", a, v[:, group]).reshape(n, nh * e))
    want = torch.cat(want)
    lens = [n for _, n in seqs]
    starts = [sum(lens[:i]) for i in range(len(lens))]
    q_d = torch.cat([q.reshape(q.shape[0], -1) for q in qs]).to(dt).to(DEV).contiguous()
    out = torch.empty((sum(lens), nh * e), dtype=dt, device=DEV)
    rt = SimpleNamespace(status=torch.zeros(1, dtype=torch.int32, device=DEV))
    multi = [s for s, n in enumerate(lens) if n > 1]
    batch = SimpleNamespace(n_seqs=len(seqs), seq_q_len=lens, seq_q_start_d=i32(starts), seq_q_len_d=i32(lens),
                            seq_pos_start_d=i32([c for c, _ in seqs]), max_q_len=max(lens),
                            max_kv_len=max(c + n for c, n in seqs), multi_seqs_d=i32(multi), n_multi=len(multi),
                            positions=i32([p for c, n in seqs for p in range(c, c + n)]),
                            row_seq=i32([s for s, n in enumerate(lens) for _ in range(n)]))
    ops.paged_attention(SimpleNamespace(batch=batch, runtime=rt), q_d, out, cache, nh, nkv, d, window, scale, vd=e,
                        sinks=sinks.to(DEV), weights_float32=True, keep_first=keep)
    assert int(rt.status.item()) == 0
    assert rel_err(out, want) < (2e-5 if dtype == "float32" else 1.5e-2)


# ---------------------------------------------------------------------------------------------------------------
# parts alone, through the step context and cache the engine uses
# ---------------------------------------------------------------------------------------------------------------
def run_mixer_in_steps(bench, part, H, steps, width):
    """Returns {request: [T, width] float64}: the part's output for every token, the requests fed as `steps` say."""
    got = {k: torch.zeros(len(v), width, dtype=F64) for k, v in H.items()}
    for step in steps:
        ctx, _ = bench.begin([(rid, [1] * k, []) for rid, _, k in step], width)
        h = torch.cat([H[rid][s:s + k] for rid, s, k in step]).cuda()
        ctx.pending_slabs = 1
        part.forward(ctx, h, ctx.delta, 0)
        out = ctx.delta_slabs[:ctx.pending_slabs].sum(0).double().cpu()
        row = 0
        for rid, s, k in step:
            got[rid][s:s + k] = out[row:row + k]
            row += k
        bench.end()
    return got


STEPS = [[("a", 0, 17)], [("a", 17, 11), ("b", 0, 20)], [("a", 28, 1), ("b", 20, 1)], [("a", 29, 2), ("b", 21, 2)],
         [("a", 31, 1)], [("a", 32, 40), ("b", 23, 1)], [("a", 72, 1)], [("a", 73, 100)], [("a", 173, 1)]]


@pytest.mark.parametrize("sizes", [(2, 16, 8, 24, 40, 24), (4, 32, 16, 32, 96, 80), (5, 4, 6, 8, 20, 40), (1, 32, 16, 32, 48, 56),
                                   (3, 8, 0, 16, 24, 16)], ids=str)
@pytest.mark.parametrize("pairing", ["neighbours", "halves"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_latent_attention_part_with_either_pairing(sizes, pairing, dtype):
    """Causal attention over latents without a window and without a gate, the rotated parts turned with neighbours or
    with the two halves as pairs, over steps of portions, single tokens and two tokens against whole sequences."""
    from test_parts_gpu import Bench, bind_random
    from flambeau_b200.cache.manager import CallPlan
    from flambeau_b200.parts.latent_attention import LatentAttention
    from flambeau_b200.parts.spec import PartSpec
    H, d, r, e, Rc, Rq = sizes
    width, eps, scale = 40, 1e-5, 0.3
    kind = {"neighbours": "rotary_neighbours", "halves": "rotary_half"}[pairing]
    pos = PartSpec("position", kind, dict(head_dim=r, theta=1e3, rotary_dim=r)) if r else None
    kw = dict(width=width, num_heads=H, head_dim=d, rot_dim=r, value_dim=e, kv_rank=Rc, q_rank=Rq, window=0, scale=scale,
              eps=eps, position=pos, gate=False, init_std=0.3 if dtype == "float32" else 0.15)
    b = Bench(dtype, plans=[CallPlan(kv=LatentAttention(None, "o.", **kw).cache_requirement())])
    part = LatentAttention(b.rt, "o.", **kw)
    Wt = bind_random(part, DT[dtype])
    assert "o.g" not in Wt
    g = torch.Generator().manual_seed(2)
    Hs = {"a": torch.randn(174, width, generator=g).to(DT[dtype]), "b": torch.randn(24, width, generator=g).to(DT[dtype])}
    got = run_mixer_in_steps(b, part, Hs, STEPS, width)
    m = {"heads": H, "dim": d, "rot_dim": r, "vdim": e, "kv_rank": Rc, "rot": {"base": 1e3, "dims": r}, "scale": scale}
    for rid, h in Hs.items():
        want = pt.latent_attention(h.double(), Wt, "o.", m, eps, list(range(len(h))), pairing)
        assert rel_err(got[rid], want) < (2e-5 if dtype == "float32" else 2e-2), rid


@pytest.mark.parametrize("sizes", [(4, 2, 16, 24, 9, 2, 8), (6, 1, 64, 64, 70, 66, 16), (3, 3, 24, 8, 0, 0, 0), (2, 1, 8, 8, 1, 1, 4),
                                   (4, 2, 64, 64, 30, 4, 64), (2, 2, 32, 32, 20, 0, 32)], ids=str)
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_part_with_kept_keys_sink_and_gate(sizes, dtype):
    """The paged attention part as this design uses it: grouped heads, part of a head rotated, a window that keeps the
    first keys, a sink, values of their own width and the sigmoid gate on the heads' outputs, across steps."""
    from test_parts_gpu import Bench, bind_random
    from flambeau_b200.cache.manager import CallPlan
    from flambeau_b200.parts.attention import PagedAttention
    from flambeau_b200.parts.spec import PartSpec
    H, G, d, e, W, F, R = sizes
    width, scale = 48, 0.25
    names = {"q": "q", "k": "k", "v": "v", "o": "o", "sink": "sink", "g": "g"}
    pos = PartSpec("position", "rotary_half", dict(head_dim=d, theta=1e4, rotary_dim=R)) if R else None
    kw = dict(width=width, num_heads=H, num_kv_heads=G, head_dim=d, value_dim=e, window=W, keep_first=F, scale=scale,
              sink=True, gate=True, names=names, weights_float32=True, position=pos,
              init_std=0.3 if dtype == "float32" else 0.15)
    b = Bench(dtype, plans=[CallPlan(kv=PagedAttention(None, "m.", **kw).cache_requirement())])
    part = PagedAttention(b.rt, "m.", **kw)
    Wt = bind_random(part, DT[dtype])
    g = torch.Generator().manual_seed(3)
    Hs = {"a": torch.randn(174, width, generator=g).to(DT[dtype]), "b": torch.randn(24, width, generator=g).to(DT[dtype])}
    got = run_mixer_in_steps(b, part, Hs, STEPS, width)
    m = {"heads": H, "kv_heads": G, "dim": d, "vdim": e, "scale": scale}
    if W:
        m["mask"] = {"size": W, "keep_first": F}
    if R:
        m["rot"] = {"base": 1e4, "dims": R}
    for rid, h in Hs.items():
        want = pt.windowed_attention(h.double(), Wt, "m.", m, list(range(len(h))))
        assert rel_err(got[rid], want) < (2e-5 if dtype == "float32" else 2e-2), rid


@pytest.mark.parametrize("shape", [(5, 64, 48), (64, 96, 80), (65, 96, 80), (300, 40, 24), (700, 128, 384)], ids=str)
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_plain_feed_forward(shape, dtype):
    """Few rows (shares of K and the activation kernel) and many (the activation in the product's epilogue)."""
    from test_parts_gpu import Bench, bind_random
    from flambeau_b200.parts.feedforward import PlainMLP
    n, D, ff = shape
    b = Bench(dtype, max_step_tokens=1024, cache_tokens=1024)
    part = PlainMLP(b.rt, "m.", width=D, inner=ff, activation="relu_squared", init_std=0.2)
    Wt = bind_random(part, DT[dtype])
    h = torch.randn(n, D, generator=torch.Generator().manual_seed(n)).to(DT[dtype])
    ctx, _ = b.begin([("a", [1] * n, [])], D)
    ctx.pending_slabs = 1
    part.forward(ctx, h.to(DEV), ctx.delta)
    b.end()
    out = ctx.delta_slabs[:ctx.pending_slabs].sum(0)
    assert rel_err(out, pt.dense_ff(h.double(), Wt, "m.")) < (2e-5 if dtype == "float32" else 2e-2)


@pytest.mark.parametrize("shape", [(5, 64, 6, 3, 24, 40), (300, 96, 40, 5, 16, 0), (33, 32, 3, 2, 32, 16), (2, 48, 4, 1, 20, 0),
                                   (700, 64, 8, 4, 40, 24), (1, 64, 1, 1, 8, 8), (90, 36, 5, 5, 12, 0)], ids=str)
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_routed_experts_whose_scores_scale_their_inputs(shape, dtype):
    """The part alone: sigmoid scores, the largest chosen, not renormalised, multiplied into what the expert reads,
    and a shared expert; few rows and many, a width that is no multiple of 8, all experts chosen."""
    from test_parts_gpu import Bench
    from flambeau_b200.parts.moe import RoutedExperts
    from flambeau_b200.parts.spec import PartSpec
    n, D, E, K, ff, shared = shape
    dt = DT[dtype]
    b = Bench(dtype, max_step_tokens=1024, cache_tokens=1024)
    shared_spec = PartSpec("feed_forward", "gated_mlp", dict(width=D, inner=shared, activation="silu",
                                                             names=("gate", "up", "down")), "m.shared.") if shared else None
    part = RoutedExperts(b.rt, "m.", width=D, inner=ff, experts=E, top=K, activation="silu", gated=True, rule="sigmoid",
                         share_on_input=True, router_bias=False, shared=shared_spec)
    g = torch.Generator().manual_seed(n)
    w = {name: (torch.randn(ts.shape, generator=g) * (0.3 if name.endswith("router") else 0.2)).to(dt)
         for name, ts in part.tensor_specs().items()}
    assert not any(name.endswith(".b") for name in w)
    part.bind({k: v.to(DEV) for k, v in w.items()})
    h = torch.randn(n, D, generator=g).to(dt)
    mlp = {"router": {"experts": E, "top": K}, "shared": {"ff": shared} if shared else None}
    w64 = {k: v.double() for k, v in w.items()}
    want = pt.routed_ff(h.double(), w64, "m.", mlp)
    ctx, _ = b.begin([("a", [1] * n, [])], D)
    ctx.pending_slabs = 1
    part.forward(ctx, h.to(DEV), ctx.delta)
    b.end()
    out = ctx.delta_slabs[:ctx.pending_slabs].sum(0)
    # a token whose choice was close may go to another expert in bfloat16: all but a few rows must agree
    err = (out.double().cpu() - want).abs().max(dim=1).values / want.abs().max()
    tol = 2e-5 if dtype == "float32" else 2e-2
    assert int((err > tol).sum()) <= (0 if dtype == "float32" or K == E else n // 50), float(err.max())


# ---------------------------------------------------------------------------------------------------------------
# whole models under schedules
# ---------------------------------------------------------------------------------------------------------------
SHARP = {"float32": 0.25, "bfloat16": 0.12}
LENGTHS = {"TA": [1, 9, 40, 75, 33, 21, 64, 110], "TB": [2, 70, 17, 48, 150, 5], "TC": [30, 3]}


def tolerance(dtype, pcfg, W, requests):
    """(bound on the worst position, bound on the median position), as fractions of the logit scale.  float32: 1e-4
    for both.  bfloat16: three times what rounding alone causes, which the plain implementation measures on the same
    requests by rounding the values a 16-bit engine keeps in 16 bits; never below the 2e-2 and a quarter of it that fit
    the framework's other models."""
    if dtype == "float32":
        return 1e-4, 1e-4
    noise = [pt.rounding_noise(pcfg, W, toks) for toks in requests.values()]
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
    tt.make_folder(folder, cfg, seed=seed, dtype=dtype, sharp=SHARP[dtype], steady_router=dtype == "bfloat16")
    requests = tiny.random_requests({"vocab_size": cfg["vocab"]}, lengths, seed=request_seed)
    pcfg, W = pt.read_folder(folder)
    want = {rid: pt.forward(pcfg, W, toks) for rid, toks in requests.items()}
    return dict(name=name, dtype=dtype, cfg=cfg, folder=folder, requests=requests, want=want,
                tol=tolerance(dtype, pcfg, W, requests))


@pytest.fixture(scope="module", params=[(c, d) for c in ("TA", "TB") for d in ("float32", "bfloat16")],
                ids=lambda p: f"{p[0]}-{p[1]}")
def case(request, tmp_path_factory):
    name, dtype = request.param
    return make_case(name, tt.CONFIGS[name], tmp_path_factory.mktemp(f"t{name}{dtype}"), dtype, LENGTHS[name],
                     seed=17 if name == "TA" else 29)


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
    """The tail is longer than TA's windows (9 and 20), so windows pass over decoded tokens, the kept first keys part
    from the window while decoding, and the group without kept keys gives pages back."""
    run(case, tiny.schedule_tail(case["requests"], 45), tmp_path)


def test_portions_down_to_two_tokens(case, tmp_path):
    run(case, tiny.schedule_portions(case["requests"]), tmp_path)
    run(case, tiny.schedule_portions(case["requests"], sizes=(2, 31, 2, 2, 17, 64, 3)), tmp_path / "b")


@pytest.mark.parametrize("seed", [1, 2])
def test_mixed_batches_with_pages_used_again(case, tmp_path, seed):
    sched = tiny.schedule_mixed(case["requests"], seed=seed)
    total_pages = sum(-(-len(t) // 16) for t in case["requests"].values())
    assert sched.max_live_tokens(case["requests"]) // 16 < total_pages, "the pool must be smaller than all requests"
    assert len(case["requests"]) > 4, "more requests than slots, so that slots are used again"
    run(case, sched, tmp_path)


def test_every_token_decoded_from_the_first(case, tmp_path):
    """One token a step from position 0 (replayed from CUDA graphs where the engine captures them): the first tokens
    of a sequence, and a long decoding."""
    rid = max(case["requests"], key=lambda r: len(case["requests"][r]))
    toks = case["requests"][rid]
    s = tiny.Schedule()
    for p, t in enumerate(toks):
        s.add([(rid, [t], [0], p)], end=[rid] if p == len(toks) - 1 else [])
    one = dict(case, requests={rid: toks}, want={rid: case["want"][rid]})
    run(one, s, tmp_path)
    assert run.last_engine.graph_replays > len(toks) // 2, "single-token steps are replayed from a captured graph"


def test_a_plain_residual_and_a_window_of_one_key(tmp_path):
    for dtype in ("float32", "bfloat16"):
        c = make_case("TC", tt.CONFIGS["TC"], tmp_path / dtype, dtype, LENGTHS["TC"], seed=3, request_seed=2)
        run(c, tiny.schedule_portions(c["requests"], sizes=(5, 2, 9)), tmp_path / dtype / "o")
        run(c, tiny.schedule_tail(c["requests"], 12), tmp_path / dtype / "t")


def random_config(seed: int) -> dict:
    """A configuration drawn from a seed: widths that are and are not multiples of 8, odd head sizes, windows from one
    key to beyond the requests, kept keys from none to more than a tile, one to four streams or none, loops, experts
    with and without a shared one, layers without feed-forward."""
    import random
    rng = random.Random(seed)
    width = rng.choice([40, 72, 100, 128, 36])
    layers = []
    for _ in range(rng.randint(1, 4)):
        mlp = None
        roll = rng.random()
        if roll < 0.4:
            mlp = tt.dense(rng.choice([24, 40, 100]))
        elif roll < 0.85:
            experts = rng.randint(1, 10)
            mlp = tt.moe(experts, rng.randint(1, min(experts, 4)), rng.choice([8, 16, 24, 40]), rng.choice([None, 8, 32]))
        if rng.random() < 0.5:
            heads, kv = rng.choice([(1, 1), (2, 1), (4, 2), (6, 3), (3, 3)])
            d = rng.choice([8, 16, 24, 32, 64])
            window = rng.choice([0, 1, 2, 5, 16, 17, 31, 64, 500])
            layers.append(tt.layer("attention", tt.attention(
                heads, kv, d, rng.choice([d, d, 8, 24]), window, rng.choice([0, 1, 3, 16, 70]),
                rng.choice([0, 2, d // 2, d]), rng.choice([100.0, 1e4, 5e5]), rng.uniform(0.1, 0.4)), mlp))
        else:
            layers.append(tt.layer(rng.choice(["latent_attention", "latent_attention_2"]), tt.latent(
                rng.choice([1, 2, 3, 6]), rng.choice([4, 8, 12, 16, 32]), rng.choice([0, 2, 4, 8, 16]),
                rng.choice([8, 12, 16, 24]), rng.choice([8, 20, 24, 48, 64]), rng.choice([8, 20, 32]),
                rng.choice([100.0, 1e4, 5e5]), rng.uniform(0.1, 0.4)), mlp))
    cfg = {"architecture": "Tubepel", "norm": {"eps": rng.choice([1e-5, 1e-6])}, "vocab": rng.randint(50, 400),
           "width": width, "layers": layers}
    streams = rng.choice([None, 1, 2, 3, 4])
    if streams:
        cfg["streams"] = streams
    if rng.random() < 0.6:
        start = rng.randint(0, len(layers) - 1)
        cfg["loop"] = {"start": start, "stop": rng.randint(start, len(layers)), "times": rng.randint(1, 3)}
    return cfg


@pytest.mark.parametrize("seed", [301, 302, 303, 304, 305, 306, 307, 308])
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


@pytest.mark.parametrize("edges", [(1, 1), (11, 3), (16, 16), (17, 5), (70, 66), (40, 0)], ids=str)
def test_windows_and_kept_keys_end_where_they_should_in_prompts_and_in_decoding(tmp_path, edges):
    """One attention layer on one stream without feed-forward, float32: a token then reaches later positions through
    its key and value alone.  Changing the token just outside the last query's window, or the first token that is not
    kept, leaves its logits as they were; changing the one just inside the window, or the last kept token, moves them.
    The last position is once part of a portion, once a decoded token."""
    window, keep = edges
    cfg = {"architecture": "Tubepel", "norm": {"eps": 1e-5}, "vocab": 150, "width": 48, "streams": 1,
           "layers": [tt.layer("attention", tt.attention(3, 1, 16, 24, window, keep, 8, 1e4, 0.3), None)]}
    folder = tt.make_folder(tmp_path / "m", cfg, seed=8, dtype="float32")
    base = tiny.random_requests({"vocab_size": cfg["vocab"]}, [160], seed=1)["r0"]
    p = len(base) - 1

    def changed(at):
        t = list(base)
        t[at] = (t[at] + 1) % cfg["vocab"]
        return t

    def moves(at, cut, ref):
        return float((logits_at_the_end(folder, changed(at), cut) - ref).abs().max()) / float(ref.abs().max())
    for cut in (60, p - 1, p):                      # (p: the last token is decoded alone)
        ref = logits_at_the_end(folder, base, cut)
        assert moves(p - window, cut, ref) < 1e-5, cut
        assert moves(keep, cut, ref) < 1e-5, cut
        if window > 1:
            assert moves(p - window + 1, cut, ref) > 1e-4, cut
        if keep:
            assert moves(keep - 1, cut, ref) > 1e-5, cut
    pcfg, W = pt.read_folder(folder)
    assert rel_err(logits_at_the_end(folder, base, 37), pt.forward(pcfg, W, base)[-1]) < 1e-4


def test_a_far_key_among_hundreds_is_found(tmp_path):
    """Causal attention over latents, float32.  One head's maps are rebuilt so that its query for one token points
    along another token's latent (its rotated part switched off): where the first stands last and the second hundreds
    of positions back and nowhere else, that far key takes most of the head's softmax, so that losing the key, or its
    page, would move the logits by far more than any rounding."""
    cfg = {"architecture": "Tubepel", "norm": {"eps": 1e-5}, "vocab": 90, "width": 32,
           "layers": [tt.layer("latent_attention_2", tt.latent(2, 8, 4, 8, 16, 8, 1e4, 1.0), None)]}
    folder = tt.make_folder(tmp_path / "m", cfg, seed=10, dtype="float32", sharp=0.3)
    pcfg, W = pt.read_folder(folder)
    eps, asks, answers = 1e-5, 85, 84
    h = pt.rms_norm(W["embed"][[asks, answers]], W["l0.norm1"], eps)
    c = pt.rms_norm((h[1:] @ W["l0.mix.dkv"].T)[:, :16], W["l0.mix.dkv.norm"], eps)
    cq = pt.rms_norm(h[:1] @ W["l0.mix.dq"].T, W["l0.mix.dq.norm"], eps)
    tensors = tt.read_tensors(folder)
    uk, uq = tensors["l0.mix.uk"], tensors["l0.mix.uq"]
    uk[:8] = 0.0
    uk[0] = (c[0] / c[0].norm()).float()
    uq[:12] = 0.0
    uq[0] = (3.0 * cq[0] / cq[0].norm()).float()
    tt.write_tensors(folder, tensors)
    pcfg, W = pt.read_folder(folder)
    base = tiny.random_requests({"vocab_size": 80}, [400], seed=3)["r0"]      # tokens from 80 on are kept for the far key
    far = list(base)
    far[7], far[-1] = answers, asks
    want = pt.forward(pcfg, W, far)[-1]
    for cut in (150, len(far) - 1):
        assert rel_err(logits_at_the_end(folder, far, cut), want) < 1e-4
    moved = list(far)
    moved[7] = 86
    assert float((pt.forward(pcfg, W, moved)[-1] - want).abs().max()) / float(want.abs().max()) > 2e-2, \
        "the far key does not matter in this model: the test would show nothing"


# ---------------------------------------------------------------------------------------------------------------
# generation through the entry point and the scheduler
# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name,dtype", [("TA", "float32"), ("TB", "bfloat16")])
def test_greedy_generation(tmp_path, name, dtype):
    from flambeau_b200 import generate
    cfg = tt.CONFIGS[name]
    folder = tt.make_folder(tmp_path / "m", cfg, seed=41, dtype=dtype, sharp=SHARP[dtype], steady_router=dtype == "bfloat16")
    pcfg, W = pt.read_folder(folder)
    prompts = list(tiny.random_requests({"vocab_size": cfg["vocab"]}, [3, 26, 50, 1, 12], seed=6).values())
    n_new = 10
    outs = generate(folder, prompts, max_tokens=n_new, temperature=0.0, dtype=dtype, prefill_chunk_tokens=16,
                    prefill_ubatch=40, inflight_slots=3)
    tol = tolerance("bfloat16", pcfg, W, {i: p for i, p in enumerate(prompts)})[0]
    for prompt, out in zip(prompts, outs):
        assert len(out) == n_new
        toks = list(prompt)
        for t in out:
            logits = pt.forward(pcfg, W, toks)[-1]
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
    cfg = tt.CONFIGS["TC"]
    folder = tt.make_folder(tmp_path / "m", cfg, seed=12, dtype="float32")
    pcfg, W = pt.read_folder(folder)
    prompt = tiny.random_requests({"vocab_size": cfg["vocab"]}, [14], seed=3)["r0"]
    proc = subprocess.run([sys.executable, str(root / "bin" / "flambeau"), "infer", "--model", str(folder), "--max-tokens",
                           "4", "--dtype", "float32", "--prompt", ",".join(map(str, prompt))],
                          capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    out = [int(t) for t in proc.stdout.strip().splitlines()[-1].split(",")]
    toks = list(prompt)
    for t in out:
        logits = pt.forward(pcfg, W, toks)[-1]
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
        assert rel_err(torch.from_numpy(row.copy()), pt.forward(pcfg, W, seq)[-1]) < 1e-4
