"""Nodepel on the GPU against the plain implementation (tests/plain_nodepel.py): each mechanism alone through its
kernels, then whole models under schedules (whole, token by token, portions down to two tokens, mixed batches on a
pool so small that pages and slots are used again), long decoding, and greedy generation through generate()."""
import math
from types import SimpleNamespace

import pytest
import torch

import nodepel_tiny as nt
import plain_nodepel as pn
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
class PagedKV:
    """Keys and values of some sequences scattered over pages that were handed out in random order; slots that were
    never written hold NaN; a table row starts at the first page the window still needs."""

    def __init__(self, seqs, k, v, *, window, page_size, dtype, seed=0):
        from flambeau_b200.cache.manager import LayerCacheView
        g = torch.Generator().manual_seed(seed)
        nkv, hd, vd = k[0].shape[1], k[0].shape[2], v[0].shape[2]
        first = [max(0, ctx - window + 1) // page_size if window else 0 for ctx, _ in seqs]
        count = [-(-(ctx + n) // page_size) - fp for (ctx, n), fp in zip(seqs, first)]
        total = sum(count) + 3
        order = torch.randperm(total, generator=g).tolist()
        table = torch.full((len(seqs), max(count) + 1), -1, dtype=torch.int32)
        k_pool = torch.full((total, nkv, page_size, hd), float("nan"), dtype=dtype)
        v_pool = torch.full((total, nkv, page_size, vd), float("nan"), dtype=dtype)
        for s, ((ctx, n), fp) in enumerate(zip(seqs, first)):
            for j in range(count[s]):
                page = order.pop()
                table[s, j] = page
                lo = (fp + j) * page_size
                hi = min(lo + page_size, ctx + n)
                k_pool[page, :, :hi - lo] = k[s][lo:hi].transpose(0, 1).to(dtype)
                v_pool[page, :, :hi - lo] = v[s][lo:hi].transpose(0, 1).to(dtype)
        self.view = LayerCacheView(k_pool.to(DEV), v_pool.to(DEV), table.to(DEV), i32(first), page_size, False, 0, None)


ATTN_GEOMETRIES = [  # heads, kv heads, key size, value size, window, page size
    (4, 2, 16, 32, 20, 16), (6, 1, 24, 8, 33, 8), (3, 3, 20, 40, 1, 16), (2, 1, 64, 128, 100, 32),
    (8, 2, 48, 48, 0, 16), (1, 1, 136, 72, 7, 64), (4, 1, 64, 64, 50, 16), (8, 2, 128, 128, 100, 16),
    (6, 2, 40, 40, 33, 8), (16, 1, 128, 128, 90, 32)]


@pytest.mark.parametrize("geometry", ATTN_GEOMETRIES, ids=lambda g: "h%d.%d-k%d-v%d-w%d-p%d" % g)
@pytest.mark.parametrize("dtype", ["float32", "bfloat16", "bfloat16-tensor-cores"])
def test_windowed_attention_with_a_sink(geometry, dtype):
    """Sequences that are first tokens, decoded tokens far into a request and at page borders, portions that start
    in mid-page beyond the window and portions of two tokens.  For the first and the last query of each, the key at
    the window's far edge is made to dominate, and the key one further (just outside) even more: if that one were
    seen, it would take the softmax over.  The sink of every other head is made large, so that leaving it out shows."""
    from flambeau_b200.kernels import ops
    nh, nkv, hd, vd, window, page = geometry
    tensor_cores = dtype.endswith("tensor-cores")          # the kernels the engine serves bfloat16 with
    dtype = dtype.split("-")[0]
    if tensor_cores and vd != hd:
        pytest.skip("value rows of another width than key rows run on the float32-math kernel")
    dt = DT[dtype]
    seqs = [(0, 1), (0, 37), (199, 1), (page * 3 - 1, 1), (page * 3, 1), (page * 2 + 5, 29), (150, 2), (63, 70),
            (10, 300)]
    g = torch.Generator().manual_seed(5)

    def rnd(*shape, s=1.0):
        return (torch.randn(*shape, generator=g) * s).to(dt).double()
    scale = 0.9 / math.sqrt(hd)
    sink = (torch.randn(nh, generator=g) * 1.5)
    sink[::2] += 6.0
    qs, ks, vs = [], [], []
    for ctx, n in seqs:
        T = ctx + n
        q, k, v = rnd(n, nh, hd), rnd(T, nkv, hd), rnd(T, nkv, vd, s=2.0)
        for row in {0, n - 1}:
            p = ctx + row
            for hh in range(0, nh, max(1, nh // 2)):
                unit = q[row, hh] / (q[row, hh] ** 2).sum()
                edge = p - window + 1 if window else 0
                if edge >= 0:
                    k[edge, hh // (nh // nkv)] = (unit * 12.0 / scale).to(dt).double()
                if window and edge - 1 >= 0:
                    k[edge - 1, hh // (nh // nkv)] = (unit * 30.0 / scale).to(dt).double()
        qs.append(q); ks.append(k); vs.append(v)
    kv = PagedKV(seqs, ks, vs, window=window, page_size=page, dtype=dt)
    want = []
    for (ctx, n), q, k, v in zip(seqs, qs, ks, vs):
        T = ctx + n
        i = torch.arange(ctx, T)[:, None]
        j = torch.arange(T)[None, :]
        mask = (i - j >= 0) & ((i - j < window) if window else True)
        heads = [pn.sink_softmax((q[:, hh] @ k[:, hh // (nh // nkv)].T) * scale, mask, sink[hh].double())
                 @ v[:, hh // (nh // nkv)] for hh in range(nh)]
        want.append(torch.cat(heads, dim=-1))
    want = torch.cat(want)
    lens = [n for _, n in seqs]
    q_d = torch.cat([q.reshape(q.shape[0], -1) for q in qs]).to(dt).to(DEV).contiguous()
    out = torch.empty((sum(lens), nh * vd), dtype=dt, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    pos = i32([p for ctx, n in seqs for p in range(ctx, ctx + n)])
    c = kv.view
    if tensor_cores:
        assert ops.mma_attention_supported(q_d, nh, nkv, hd)
        G = nh // nkv
        starts = [sum(lens[:i]) for i in range(len(lens))]
        args = (c.k_pool, c.v_pool, c.block_table, i32(starts), i32(lens), i32([ctx for ctx, _ in seqs]), len(seqs),
                max(lens), max(ctx + n for ctx, n in seqs), any(ops.attention_is_short(n, nh, nkv) for n in lens),
                any(not ops.attention_is_short(n, nh, nkv) for n in lens), nh, nkv, hd, window, scale, status)
        # the weights as two bfloat16 numbers each through P V: what is left is the rounding of the output
        exact = torch.empty_like(out)
        ops.paged_attention_mma(q_d, exact, *args, table_base=c.table_base, sinks=sink.float().to(DEV),
                                weights_float32=True)
        assert rel_err(exact, want) < 5e-3
        ops.paged_attention_mma(q_d, out, *args, table_base=c.table_base, sinks=sink.float().to(DEV))
    else:
        ops.paged_attention_simt(q_d, out, c.k_pool, c.v_pool, c.block_table, pos,
                                 i32([s for s, n in enumerate(lens) for _ in range(n)]), nh, nkv, hd, window, scale,
                                 status, table_base=c.table_base, sinks=sink.float().to(DEV), vd=vd)
    assert int(status.item()) == 0
    assert rel_err(out, want) < (2e-5 if dtype == "float32" else 1.5e-2)


@pytest.mark.parametrize("reach", ["projection", "head", None])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_norm_rotation_and_cache_write_behind_the_projection(reach, dtype):
    """Split-K shares in, q out, k and v in their pages: the norm over the whole projection, over every head, or
    none; a rotation of part of the head; value rows of their own width; positions across page borders."""
    from flambeau_b200.cache.manager import LayerCacheView
    from flambeau_b200.kernels import ops
    nh, nkv, hd, vd, page, rot = 6, 2, 24, 40, 8, 10
    dt = DT[dtype]
    g = torch.Generator().manual_seed(2)
    positions = [0, 1, 7, 8, 9, 33, 34, 1000, 1001]            # one sequence of 9 rows at scattered positions
    n = len(positions)
    cols = nh * hd + nkv * hd + nkv * vd
    shares = torch.randn(3, n, cols + 5, generator=g)
    proj = shares.sum(0).double()[:, :cols]
    qw, kw = torch.randn(nh * hd if reach == "projection" else hd, generator=g) + 2, \
        torch.randn(nkv * hd if reach == "projection" else hd, generator=g) - 2
    eps, base = 1e-3, 77.0
    q = proj[:, :nh * hd]
    k = proj[:, nh * hd:nh * hd + nkv * hd]
    if reach == "projection":
        q, k = pn.plain_norm(q, qw.double(), eps), pn.plain_norm(k, kw.double(), eps)
    q, k = q.reshape(n, nh, hd), k.reshape(n, nkv, hd)
    if reach == "head":
        q, k = pn.plain_norm(q, qw.double(), eps), pn.plain_norm(k, kw.double(), eps)
    q, k = pn.rotate_half(q, positions, base, rot), pn.rotate_half(k, positions, base, rot)
    v = proj[:, nh * hd + nkv * hd:].reshape(n, nkv, vd)
    pages = max(positions) // page + 1
    table = torch.randperm(pages, generator=g).to(torch.int32)
    cache = LayerCacheView(torch.zeros((pages, nkv, page, hd), dtype=dt, device=DEV),
                           torch.zeros((pages, nkv, page, vd), dtype=dt, device=DEV), table[None].to(DEV).contiguous(),
                           i32([0]), page, True, 0, None)
    half = rot // 2
    freq = torch.pow(torch.tensor(base, dtype=F64), -2.0 * torch.arange(half, dtype=F64) / rot)
    ang = torch.tensor(positions, dtype=F64)[:, None] * freq[None]
    q_out = torch.empty((n, nh * hd), dtype=dt, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    sh = shares.to(DEV).contiguous()
    ops.qk_norm_rope_kv_write(sh[0], qw.to(dt).to(DEV) if reach else None, kw.to(dt).to(DEV) if reach else None, reach,
                              eps, 0.0, torch.cos(ang).float().to(DEV), torch.sin(ang).float().to(DEV), half, q_out,
                              cache, i32(positions), i32([0] * n), nh, nkv, hd, vd, status, n_partials=3,
                              partial_stride=sh.stride(0))
    assert int(status.item()) == 0
    tol = 1e-5 if dtype == "float32" else 1e-2
    assert rel_err(q_out.view(n, nh, hd), q) < tol * (3 if reach else 1)
    for r, p in enumerate(positions):
        pg = int(table[p // page])
        assert rel_err(cache.k_pool[pg, :, p % page], k[r]) < tol * (3 if reach else 1)
        assert rel_err(cache.v_pool[pg, :, p % page], v[r]) < tol


@pytest.mark.parametrize("sizes", [(4, 2, 8, 16, 4), (2, 1, 16, 24, 3), (3, 3, 24, 8, 2), (2, 2, 40, 12, 1),
                                   (1, 1, 136, 72, 4), (4, 1, 300, 20, 2)], ids=str)
def test_gated_delta_rule_across_steps(sizes):
    """Three requests in three state slots, fed in steps of unequal portions (one token, two tokens, many), then a slot
    zeroed and used again; the outputs of every step and the state at the end against the plain recurrence over the
    whole sequences."""
    from flambeau_b200.kernels import ops
    H, G, dk, dv, taps = sizes
    g = torch.Generator().manual_seed(11)
    C = 2 * G * dk + H * dv
    cols = C + 2 * H + H * dv
    lengths = [23, 9, 40]
    conv_w = torch.randn(C, taps, generator=g) * 0.5
    a_log, dt_bias, norm_w = torch.randn(H, generator=g) * 0.5 - 1, torch.randn(H, generator=g) * 0.5, \
        torch.randn(dv, generator=g) + 1
    eps = 1e-5
    proj = [torch.randn(L, cols, generator=g) for L in lengths]

    def plain(x):
        x = x.double()
        n = x.shape[0]
        act = pn.silu(pn.short_convolution(x[:, :C], conv_w.double()))
        q = pn.unit_vector(act[:, :G * dk].reshape(n, G, dk)) * dk ** -0.5
        k = pn.unit_vector(act[:, G * dk:2 * G * dk].reshape(n, G, dk))
        v = act[:, 2 * G * dk:].reshape(n, H, dv)
        beta = torch.sigmoid(x[:, C:C + H])
        decay = torch.exp(-torch.exp(a_log.double())[None] * pn.softplus(x[:, C + H:C + 2 * H] + dt_bias.double()[None]))
        gate = pn.silu(x[:, C + 2 * H:]).reshape(n, H, dv)
        heads = [pn.plain_norm(pn.delta_rule(q[:, hh // (H // G)], k[:, hh // (H // G)], v[:, hh], beta[:, hh],
                                             decay[:, hh]), norm_w.double(), eps) * gate[:, hh] for hh in range(H)]
        return torch.cat(heads, dim=-1)
    want = [plain(x) for x in proj]
    S, tail = H * dk * dv, (taps - 1) * C
    state = torch.zeros((4, S + tail), dtype=torch.float32, device=DEV)
    state[3].fill_(float("nan"))                     # a slot nobody uses
    slots = [2, 0, 1]
    at = [0, 0, 0]
    got = [[], [], []]
    steps = [[1, 2, 5], [2, 1, 17], [3, 0, 1], [16, 6, 16], [1, 0, 1]]
    for portion in steps:
        live = [(s, k) for s, k in enumerate(portion) if k]
        x = torch.cat([proj[s][at[s]:at[s] + k] for s, k in live])
        shares = torch.stack([x * 0.25, x * 0.75]).to(DEV).contiguous()
        n = x.shape[0]
        b = fake_batch([k for _, k in live], [slots[s] for s, _ in live])
        qkv = torch.empty((n, C), dtype=torch.float32, device=DEV)
        beta, decay = torch.empty((n, H), dtype=torch.float32, device=DEV), torch.empty((n, H), dtype=torch.float32, device=DEV)
        ops.gdr_prepare(shares[0], conv_w.to(DEV), taps, a_log.to(DEV), dt_bias.to(DEV), state, S, b, qkv, beta, decay,
                        G, H, dk, dv, dk ** -0.5, 1e-6, n_partials=2, partial_stride=shares.stride(0))
        o = torch.empty((n, H * dv), dtype=torch.float32, device=DEV)
        ops.gdr_recurrent(qkv, beta, decay, state, b, o, G, H, dk, dv)
        out = torch.empty((n, H * dv), dtype=torch.float32, device=DEV)
        ops.gdr_out_norm(o, shares[0], C + 2 * H, norm_w.to(DEV), eps, out, H, dv, n_partials=2,
                         partial_stride=shares.stride(0))
        r = 0
        for s, k in live:
            got[s].append(out[r:r + k].cpu())
            r += k
            at[s] += k
    assert at == lengths
    for s in range(3):
        assert rel_err(torch.cat(got[s]), want[s]) < 2e-5
    # a slot given back and used again starts from zero once more
    state[slots[1]].zero_()
    b = fake_batch([lengths[1]], [slots[1]])
    x = torch.stack([proj[1], torch.zeros_like(proj[1])]).to(DEV).contiguous()
    n = lengths[1]
    qkv = torch.empty((n, C), dtype=torch.float32, device=DEV)
    beta, decay = torch.empty((n, H), dtype=torch.float32, device=DEV), torch.empty((n, H), dtype=torch.float32, device=DEV)
    ops.gdr_prepare(x[0], conv_w.to(DEV), taps, a_log.to(DEV), dt_bias.to(DEV), state, S, b, qkv, beta, decay, G, H, dk,
                    dv, dk ** -0.5, 1e-6, n_partials=2, partial_stride=x.stride(0))
    o = torch.empty((n, H * dv), dtype=torch.float32, device=DEV)
    ops.gdr_recurrent(qkv, beta, decay, state, b, o, G, H, dk, dv)
    out = torch.empty((n, H * dv), dtype=torch.float32, device=DEV)
    ops.gdr_out_norm(o, x[0], C + 2 * H, norm_w.to(DEV), eps, out, H, dv, n_partials=2, partial_stride=x.stride(0))
    assert rel_err(out, want[1]) < 2e-5
    assert bool(torch.isnan(state[3]).all()), "a slot that no sequence of the step uses was written"


@pytest.mark.parametrize("shape", [(5, 64, 6, 2, 24, 40), (300, 96, 40, 5, 16, 24), (33, 32, 4, 1, 32, 0),
                                   (2, 48, 3, 3, 20, 8), (700, 64, 8, 2, 40, 0), (900, 64, 4, 2, 40, 16),
                                   (1300, 128, 5, 3, 136, 0)], ids=str)
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_routed_experts(shape, dtype, tmp_path):
    """The part alone: router, choice, shares, the grouped products and the shared expert against the plain
    implementation; the router's weights are wide, so that choices are rarely close.  The shapes reach every row tile
    of the grouped products (16 rows while experts hold few tokens, 64, and 128 on the tensor cores once they hold
    hundreds)."""
    from flambeau_b200.engine.runtime import Runtime
    from flambeau_b200.parts.moe import RoutedExperts
    n, D, E, K, ff, shared = shape
    dt = DT[dtype]
    rt = Runtime(DEV, dtype)
    part = RoutedExperts(rt, "m.", width=D, inner=ff, experts=E, top=K, shared_inner=shared or None)
    g = torch.Generator().manual_seed(3)
    w = {}
    for name, ts in part.tensor_specs().items():
        std = 1.0 if name.endswith("router") else 0.5 if name.endswith("router.b") else 0.2
        w[name] = (torch.randn(ts.shape, generator=g) * std).to(dt)
    part.bind({k: v.to(DEV) for k, v in w.items()})
    h = (torch.randn(n, D, generator=g)).to(dt)
    mlp = {"router": {"experts": E, "top": K}, "shared": {"ff": shared} if shared else None}
    want = pn.routed_experts(h.double(), {k: v.double() for k, v in w.items()}, "m.", mlp)
    out = torch.empty((n, D), dtype=torch.float32, device=DEV)
    ctx = SimpleNamespace(n_tokens=n, ws=rt.ws, max_slabs=4, runtime=rt, pending_slabs=1)
    part.forward(ctx, h.to(DEV), out)
    assert rel_err(out, want) < (2e-5 if dtype == "float32" else 1.5e-2)


def test_side_by_side_outputs_are_normed_and_mixed():
    from flambeau_b200.kernels import ops
    n, H = 7, 100
    g = torch.Generator().manual_seed(1)
    a, b = torch.randn(3, n, H, generator=g), torch.randn(1, n, H, generator=g) * 5
    wa, wb = torch.randn(H, generator=g), torch.randn(H, generator=g)
    want = 0.5 * pn.plain_norm(a.sum(0).double(), wa.double(), 1e-4) + 0.25 * pn.plain_norm(b[0].double(), wb.double(), 1e-4)
    out = torch.empty((n, H), dtype=torch.float32, device=DEV)
    ad, bd = a.to(DEV).contiguous(), b.to(DEV).contiguous()
    ops.branch_norm_mix([(ad[0], 3, ad.stride(0), wa.to(DEV), 0.5), (bd[0], 1, 0, wb.to(DEV), 0.25)], 1e-4, out, n)
    assert rel_err(out, want) < 1e-5


# ---------------------------------------------------------------------------------------------------------------
# whole models under schedules
# ---------------------------------------------------------------------------------------------------------------
SHARP = {"float32": 0.2, "bfloat16": 0.1}
LENGTHS = {"NA": [1, 9, 40, 75, 33, 21, 64, 110], "NB": [2, 70, 17, 48, 130, 5], "NC": [30, 3]}


def tolerance(dtype, pcfg, W, requests):
    """(bound on the worst position, bound on the median position), as fractions of the logit scale.  float32: 1e-4
    for both.  bfloat16: three times what rounding alone causes, which the plain implementation measures on the
    same requests by rounding the values a 16-bit engine keeps in 16 bits (the recurrent side's gates and head norms
    and the squared activations pass that rounding on several times larger than attention does, at single positions
    by several per cent, so a bound taken from attention-only models would not fit); never below the 2e-2 and a
    quarter of it that fit the framework's other models."""
    if dtype == "float32":
        return 1e-4, 1e-4
    noise = [pn.rounding_noise(pcfg, W, toks) for toks in requests.values()]       # spikes sit at single positions
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


@pytest.fixture(scope="module", params=[(c, d) for c in ("NA", "NB") for d in ("float32", "bfloat16")],
                ids=lambda p: f"{p[0]}-{p[1]}")
def case(request, tmp_path_factory):
    name, dtype = request.param
    cfg = nt.CONFIGS[name]
    folder = nt.make_folder(tmp_path_factory.mktemp(f"n{name}{dtype}"), cfg, seed=17 if name == "NA" else 29,
                            dtype=dtype, sharp=SHARP[dtype], steady_router=dtype == "bfloat16")
    requests = tiny.random_requests({"vocab_size": cfg["vocab"]}, LENGTHS[name], seed=4)
    pcfg, W = pn.load_folder(folder)
    want = {rid: pn.forward(pcfg, W, toks) for rid, toks in requests.items()}
    return dict(name=name, dtype=dtype, cfg=cfg, folder=folder, requests=requests, want=want,
                tol=tolerance(dtype, pcfg, W, requests))


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


def test_last_tokens_one_by_one_past_every_window(case, tmp_path):
    """The tail is longer than every window of NA and than three of NB's, so windows pass over decoded tokens."""
    run(case, tiny.schedule_tail(case["requests"], 45), tmp_path)


def test_portions_down_to_two_tokens(case, tmp_path):
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
    """One token a step from position 0 (replayed from CUDA graphs where the engine captures them)."""
    rid = max(case["requests"], key=lambda r: len(case["requests"][r]))
    toks = case["requests"][rid]
    s = tiny.Schedule()
    for p, t in enumerate(toks):
        s.add([(rid, [t], [0], p)], end=[rid] if p == len(toks) - 1 else [])
    one = dict(case, requests={rid: toks}, want={rid: case["want"][rid]})
    run(one, s, tmp_path)
    assert run.last_engine.graph_replays > len(toks) // 2, "single-token steps are replayed from a captured graph"


def test_no_loop_at_all(tmp_path):
    cfg = nt.CONFIGS["NC"]
    folder = nt.make_folder(tmp_path / "m", cfg, seed=3, dtype="float32")
    requests = tiny.random_requests({"vocab_size": cfg["vocab"]}, LENGTHS["NC"], seed=2)
    pcfg, W = pn.load_folder(folder)
    c = dict(name="NC", dtype="float32", cfg=cfg, folder=folder, requests=requests, tol=(1e-4, 1e-4),
             want={rid: pn.forward(pcfg, W, toks) for rid, toks in requests.items()})
    run(c, tiny.schedule_portions(requests, sizes=(5, 2, 9)), tmp_path / "o")


def random_config(seed: int) -> dict:
    """A configuration drawn from a seed: widths that are and are not multiples of 8, odd head sizes, windows from one
    key to beyond the requests, rotations of none, part or all of a head, one to five taps, one to a dozen experts
    with and without a shared one, layers without feed-forward, a loop anywhere or none."""
    import random
    rng = random.Random(seed)
    width = rng.choice([40, 72, 100, 128, 36])
    n_layers = rng.randint(1, 4)
    layers = []
    for _ in range(n_layers):
        g = rng.choice([1, 2, 3])
        h = g * rng.choice([1, 2, 4])
        d = rng.choice([8, 12, 16, 20, 24, 32, 40, 64])
        e = rng.choice([d, d, 8, 24, 48])
        dims = rng.choice([0, 2, d // 2 // 2 * 2, d // 2 * 2])
        Gr = rng.choice([1, 2, 3])
        Hr = Gr * rng.choice([1, 2])
        mlp = None
        if rng.random() < 0.8:
            experts = rng.randint(1, 12)
            mlp = (experts, rng.randint(1, min(experts, 4)), rng.choice([8, 16, 24, 40]), rng.choice([None, 8, 32]))
        layers.append(nt.layer((h, g, d, e, rng.choice([1, 2, 5, 16, 17, 31, 64, 500]), rng.choice([100.0, 1e4, 1e6]), dims,
                                rng.uniform(0.1, 0.4)),
                               (Hr, Gr, rng.choice([4, 8, 12, 16, 36, 72]), rng.choice([8, 12, 16, 40]), rng.randint(1, 5)),
                               mlp))
    cfg = {"architecture": "Nodepel", "embedding": {"scale": rng.uniform(0.3, 3.0)}, "norm": {"eps": rng.choice([1e-5, 1e-6])},
           "vocab": rng.randint(50, 400), "width": width, "layers": layers}
    if rng.random() < 0.7:
        start = rng.randint(0, n_layers - 1)
        cfg["loop"] = {"start": start, "stop": rng.randint(start + 1, n_layers), "times": rng.randint(1, 3)}
    return cfg


@pytest.mark.parametrize("seed", [101, 102, 103, 104, 105, 106, 107, 108])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_random_configurations_under_a_mixed_schedule(tmp_path, seed, dtype):
    cfg = random_config(seed)
    folder = nt.make_folder(tmp_path / "m", cfg, seed=seed, dtype=dtype, sharp=SHARP[dtype],
                            steady_router=dtype == "bfloat16")
    requests = tiny.random_requests({"vocab_size": cfg["vocab"]}, [1, 37, 80, 2, 55, 21], seed=seed)
    pcfg, W = pn.load_folder(folder)
    c = dict(name=f"random {seed}", dtype=dtype, cfg=cfg, folder=folder, requests=requests,
             want={rid: pn.forward(pcfg, W, toks) for rid, toks in requests.items()},
             tol=tolerance(dtype, pcfg, W, requests))
    run(c, tiny.schedule_mixed(requests, seed=seed), tmp_path / "o")


def test_heads_of_64_and_128_in_bfloat16(tmp_path):
    """Head sizes that the tensor-core attention for portions takes (64 and 128, values as wide as keys), prompts of a
    few hundred tokens fed whole, in portions and token by token, so that the sink passes every one of its kernels
    inside a whole model."""
    cfg = {"architecture": "Nodepel", "embedding": {"scale": 1.5}, "norm": {"eps": 1e-6}, "vocab": 300, "width": 128,
           "layers": [nt.layer((4, 2, 64, 64, 70, 1e4, 32, 0.125), (2, 1, 32, 64, 4), (6, 2, 32, 64)),
                      nt.layer((2, 1, 128, 128, 150, 1e6, 128, 0.09), (4, 2, 64, 32, 2), None)]}
    folder = nt.make_folder(tmp_path / "m", cfg, seed=23, dtype="bfloat16", sharp=SHARP["bfloat16"], steady_router=True)
    requests = tiny.random_requests({"vocab_size": cfg["vocab"]}, [330, 40, 170], seed=9)
    pcfg, W = pn.load_folder(folder)
    c = dict(name="wide heads", dtype="bfloat16", cfg=cfg, folder=folder, requests=requests,
             want={rid: pn.forward(pcfg, W, toks) for rid, toks in requests.items()},
             tol=tolerance("bfloat16", pcfg, W, requests))
    run(c, tiny.schedule_whole(requests), tmp_path / "w")
    run(c, tiny.schedule_portions(requests, sizes=(150, 2, 64, 33, 17)), tmp_path / "p")
    run(c, tiny.schedule_tail(requests, 20), tmp_path / "t")


def test_the_state_carries_a_far_token_and_the_window_does_not(tmp_path):
    """One layer, float32.  With the recurrent side's output weight zeroed only the window is left: changing the token
    just outside the last query's window leaves its logits as they were, changing the one just inside moves them.
    With the recurrent side back, a token far outside the window moves them too: the state has carried it."""
    from flambeau_b200.engine.step import Engine, EngineOptions
    from flambeau_b200.weights.safetensors_io import SafetensorsFile, write_safetensors
    W_ = 11
    cfg = dict(nt.CONFIG_NC, layers=[nt.layer((2, 1, 16, 32, W_, 1e4, 8, 0.25), (2, 1, 16, 16, 3), (4, 2, 16, 16))])
    base = tiny.random_requests({"vocab_size": cfg["vocab"]}, [40], seed=1)["r0"]
    p = len(base) - 1

    def changed(at):
        t = list(base)
        t[at] = (t[at] + 1) % cfg["vocab"]
        return t

    def logits_of(folder, tokens, cut):
        engine = Engine.from_folder(folder, EngineOptions(dtype="float32", cache_tokens=256, max_requests=2,
                                                          max_step_tokens=128))
        engine.step([("a", tokens[:cut], [])])
        return engine.step([("a", tokens[cut:], [len(tokens) - cut - 1])], end=["a"])[0].double().cpu()
    full = nt.make_folder(tmp_path / "full", cfg, seed=8, dtype="float32")
    f = SafetensorsFile(full / "model.safetensors")
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    f.close()
    tensors["l0.mix.right.A_log"] = torch.full_like(tensors["l0.mix.right.A_log"], -4.0)     # a state that fades slowly
    write_safetensors(full / "model.safetensors", tensors)
    tensors["l0.mix.right.out"] = torch.zeros_like(tensors["l0.mix.right.out"])
    (tmp_path / "left").mkdir()
    (tmp_path / "left" / "config.json").write_text((full / "config.json").read_text())
    write_safetensors(tmp_path / "left" / "model.safetensors", tensors)
    ref = logits_of(tmp_path / "left", base, 25)
    scale = float(ref.abs().max())
    assert float((logits_of(tmp_path / "left", changed(p - W_), 33) - ref).abs().max()) / scale < 1e-5
    assert float((logits_of(tmp_path / "left", changed(p - W_ + 1), 38) - ref).abs().max()) / scale > 1e-3
    ref = logits_of(full, base, 25)
    assert float((logits_of(full, changed(3), 31) - ref).abs().max()) / float(ref.abs().max()) > 1e-4


# ---------------------------------------------------------------------------------------------------------------
# generation through the entry point and the scheduler
# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name,dtype", [("NA", "float32"), ("NB", "bfloat16")])
def test_greedy_generation(tmp_path, name, dtype):
    from flambeau_b200 import generate
    cfg = nt.CONFIGS[name]
    folder = nt.make_folder(tmp_path / "m", cfg, seed=41, dtype=dtype, sharp=SHARP[dtype],
                            steady_router=dtype == "bfloat16")
    pcfg, W = pn.load_folder(folder)
    prompts = list(tiny.random_requests({"vocab_size": cfg["vocab"]}, [3, 26, 50, 1, 12], seed=6).values())
    n_new = 10
    outs = generate(folder, prompts, max_tokens=n_new, temperature=0.0, dtype=dtype, prefill_chunk_tokens=16,
                    prefill_ubatch=40, inflight_slots=3)
    tol = tolerance("bfloat16", pcfg, W, {i: p for i, p in enumerate(prompts)})[0]
    for prompt, out in zip(prompts, outs):
        assert len(out) == n_new
        toks = list(prompt)
        for t in out:
            logits = pn.forward(pcfg, W, toks)[-1]
            best = float(logits.max())
            if dtype == "float32":
                lowest = int((logits == best).nonzero()[0])
                assert t == lowest, "greedy token differs from the plain implementation"
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
    cfg = nt.CONFIGS["NC"]
    folder = nt.make_folder(tmp_path / "m", cfg, seed=12, dtype="float32")
    pcfg, W = pn.load_folder(folder)
    prompt = tiny.random_requests({"vocab_size": cfg["vocab"]}, [14], seed=3)["r0"]
    proc = subprocess.run([sys.executable, str(root / "bin" / "flambeau"), "infer", "--model", str(folder), "--max-tokens",
                           "4", "--dtype", "float32", "--prompt", ",".join(map(str, prompt))],
                          capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    out = [int(t) for t in proc.stdout.strip().splitlines()[-1].split(",")]
    toks = list(prompt)
    for t in out:
        logits = pn.forward(pcfg, W, toks)[-1]
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
        want = pn.forward(pcfg, W, seq)[-1]
        assert rel_err(torch.from_numpy(row.copy()), want) < 1e-4
