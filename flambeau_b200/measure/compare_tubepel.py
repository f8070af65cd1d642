"""Tubepel beside Fegizen at equal size: prefill and decode throughput and, kernel by kernel, how far each is from
its roofline.

`bench.py --only tubepel` runs, for each size of SIZES, a Tubepel model (layers that alternate grouped-query attention
under a window that keeps the first keys, with a sink and an output gate, in front of a dense squared-ReLU
feed-forward, and causal attention over cached latents in front of routed experts whose scores scale their inputs,
all on several copies of the residual stream) and a Fegizen model (the framework's closest design: attention over
cached latents under a window and gated linear attention, routed experts with a shared expert) with the same width,
head counts, latents, window, vocabulary, experts and number of layers, both with random weights in bfloat16, through
the same engine calls: one decode step of `batch` sequences that each hold `context` tokens, and one step of `prefill`
prompt tokens.  Per design it reports tokens a second and, per launcher (CUDA events around every launcher call of an
eager step, so serialised kernels), launches and microseconds a launch, the work of one launch and the fraction of the
measured peak that bounds it.  `like` pairs every kernel of the new design with the kernel of Fegizen that does the
like job and gives the ratio of their fractions (below 0.5: more than twice as far from the roofline).

Work of one launch over `rows` rows (D = width, S = copies of the stream):
  attention_window   4 * seen * heads * key size flops over the window's and the kept keys; bytes: live keys and values
                     of the key/value heads + queries and outputs
  attention_latent   4 * seen * heads * row flops, row = latent + rotated part (the cache row is key and value at
                     once), every earlier key seen; bytes: all keys * row * 2 + queries and outputs
  cache_write        the projection's float32 rows in, the rounded queries and the cache rows out
  stream_step        S copies in and out (float32), the sublayer's output in, normalised rows out
  output_gate        the heads' outputs in and out, the gate's float32 columns in
  head_map           as measure/compare_fegizen.py counts it
  routed_product     6 * pairs * D * expert inner size flops for both products; bytes: the weights of the experts that
                     were chosen, once
  expert_gather      the tokens' rows in (once per chosen expert) and out, scaled on the way
"""
from __future__ import annotations

import gc

import torch

from ..config.tubepel import TubepelConfig
from ..engine.batch import Entry
from ..engine.step import Engine, EngineOptions
from ..kernels import ops
from . import work, workloads
from .compare import PAGE
from .compare_fegizen import SIZES as FEGIZEN_SIZES, CLASS_OF as FEGIZEN_CLASSES, fegizen_config, kernel_work as fegizen_work
from .compare_nodepel import fp32_fma_tflops
from .timers import SectionTimer

# what Tubepel adds to the sizes of measure/compare_fegizen.py: copies of the stream, kept first keys, the dense
# feed-forward's inner size (what a token passes through in the routed layers: its experts and the shared one)
SIZES = {k: dict(v, streams=4, keep_first=4, dense_ff=v["top"] * v["expert_ff"] + v["shared_ff"])
         for k, v in FEGIZEN_SIZES.items()}

CLASS_OF = dict(FEGIZEN_CLASSES, rope_kv_write="cache_write", hc_step="stream_step", sigmoid_gate="output_gate")

# (kernel of Tubepel, the like kernel of Fegizen); kernels that only Tubepel has are set beside the kernel of Fegizen
# that is bound by the same thing (rows through memory: its norm)
LIKE = [("attention_latent", "attention"), ("attention_window", "attention"), ("cache_write", "cache_write"),
        ("stream_step", "norm"), ("output_gate", "norm"), ("head_map", "head_map"), ("routed_product", "routed_product"),
        ("expert_gather", "expert_gather"), ("expert_combine", "expert_combine"), ("router", "router"),
        ("activation", "gate_mul")]


def tubepel_config(size: dict, layers: int) -> TubepelConfig:
    moe = {"kind": "moe", "router": {"experts": size["experts"], "top": size["top"]}, "expert": {"ff": size["expert_ff"]},
           "shared": {"ff": size["shared_ff"]}}
    window = {"type": "attention",
              "mixer": {"heads": size["heads"], "kv_heads": size["kv_heads"], "dim": size["qk_row"], "vdim": size["v_row"],
                        "mask": {"size": size["window"], "keep_first": size["keep_first"]},
                        "rot": {"base": 1e6, "dims": size["qk_row"] // 2}, "scale": size["qk_row"] ** -0.5},
              "mlp": {"kind": "dense", "ff": size["dense_ff"]}}
    latent = {"type": "latent_attention",
              "mixer": {"heads": size["heads"], "dim": size["dim"], "rot_dim": size["rot_dim"], "vdim": size["vdim"],
                        "kv_rank": size["kv_rank"], "q_rank": size["q_rank"], "rot": {"base": 1e6, "dims": size["rot_dim"]},
                        "scale": (size["dim"] + size["rot_dim"]) ** -0.5}, "mlp": moe}
    return TubepelConfig.from_dict({
        "architecture": "Tubepel", "norm": {"eps": 1e-6}, "streams": size["streams"], "vocab": size["vocab"],
        "width": size["width"], "layers": [window if i % 2 == 0 else latent for i in range(layers)]})


def configs(size: dict, layers: int) -> dict:
    return {"tubepel": tubepel_config(size, layers), "fegizen": fegizen_config(size, layers)}


def sections_by_class(engine, entries, end=(), reps: int = 3) -> dict:
    """class -> (launches, milliseconds) per step of one eager step; the attention launches are told apart by their
    key/value heads (one: over latents), products are keyed by their matrix."""
    was = engine.use_graphs
    engine.use_graphs = False
    try:
        engine.step(entries, end=end)
        totals: dict = {}
        for _ in range(reps):
            torch.cuda._sleep(int(40.0 * 2.0e6))
            with SectionTimer() as t:
                logits = engine.step(entries, end=end)
                if logits is not None:
                    ops.sample(logits, torch.zeros(logits.shape[0], dtype=torch.int32, device=logits.device))
            for what, note, ms in t.sections():
                key = CLASS_OF.get(what) or (f"product {note[1]}x{note[2]}" if what.startswith("gemm") and note else what)
                if key == "attention" and note:
                    key = "attention_latent" if note[1] == 1 else "attention_window"
                n, total = totals.get(key, (0, 0.0))
                totals[key] = (n + 1, total + ms)
        return {k: (n / reps, total / reps) for k, (n, total) in totals.items()}
    finally:
        engine.use_graphs = was


def kernel_work(size: dict, rows: int, contexts) -> dict:
    """class -> flops / bytes of one launch of a Tubepel kernel."""
    D, S, W, F = size["width"], size["streams"], size["window"], size["keep_first"]
    H, G, dq, dv = size["heads"], size["kv_heads"], size["qk_row"], size["v_row"]
    row = size["kv_rank"] + size["rot_dim"]
    pairs = rows * size["top"]
    experts_read = min(size["experts"], pairs)
    if len(contexts) == rows:
        seen_w = sum(work.live_keys(c, W) + min(F, max(0, c - W)) for c in contexts)
        keys_w, seen_l = seen_w, sum(contexts)
        keys_l = seen_l
    else:
        ctx = contexts[0]
        seen_w = work.keys_seen(range(ctx - rows, ctx), W)
        keys_w = ctx - (max(0, ctx - rows - W + 1) if W else 0)
        seen_l, keys_l = sum(range(ctx - rows + 1, ctx + 1)), ctx
    cols_w = H * dq + G * (dq + dv) + H * dv
    cols_l = size["q_rank"] + row
    return {
        "attention_window": dict(flops=4.0 * seen_w * H * dq, bytes=keys_w * G * (dq + dv) * 2 + rows * H * 2 * dq * 2),
        "attention_latent": dict(flops=4.0 * seen_l * H * row, bytes=keys_l * row * 2 + 2 * rows * H * row * 2),
        # (the mean of its two uses: the windowed side's rotary + cache write, the latents' norms + cache row)
        "cache_write": dict(bytes=rows * ((cols_w - H * dv) * (4 + 2) + cols_l * (4 + 2)) / 2.0),
        "stream_step": dict(bytes=rows * D * (4 * (2 * S + 1) + 2)),
        "output_gate": dict(bytes=rows * H * dv * (2 + 2 + 4)),
        "head_map": dict(flops=2.0 * rows * H * size["kv_rank"] * (size["dim"] + size["vdim"]) / 2.0,
                         bytes=rows * H * ((size["dim"] + size["rot_dim"]) * 4 + 2 * row * 2 + size["vdim"] * 2) / 2.0),
        "routed_product": dict(flops=6.0 * pairs * D * size["expert_ff"], bytes=experts_read * 3 * D * size["expert_ff"] * 2),
        "expert_gather": dict(bytes=pairs * D * 2 * 2),
        "expert_combine": dict(bytes=rows * D * 4 * (size["top"] + 2)),
        "router": dict(bytes=rows * size["experts"] * 4),
        "activation": dict(bytes=rows * size["dense_ff"] * (4 + 2)),
    }


def kernel_table(engine, design: str, size: dict, layers: int, entries, end, rows: int, contexts, peaks: dict) -> dict:
    secs = sections_by_class(engine, entries, end=end)
    if design == "fegizen":
        works = fegizen_work("fegizen", size, layers, rows, contexts)
        works["expert_gather"] = dict(bytes=rows * size["top"] * size["width"] * 2 * 2)
        works["gate_mul"] = dict(bytes=rows * size["shared_ff"] * (8 + 2))
        secs = {("attention" if k.startswith("attention") else k): v for k, v in secs.items()}
    else:
        works = kernel_work(size, rows, contexts)
    fma_peak = fp32_fma_tflops(engine.runtime.device)
    table = {}
    for key, (n, total) in sorted(secs.items()):
        r = {"launches": round(n, 2), "us": round(total * 1e3 / max(n, 1e-9), 2)}
        w = works.get(key)
        if w and r["us"] > 0:
            sec = r["us"] * 1e-6
            by_mem = w.get("bytes", 0.0) / sec / 1e9 / peaks["hbm_gbs"]
            by_math = w.get("flops", 0.0) / sec / 1e12 / peaks["bf16_tflops"]
            by_fma = w.get("fma_flops", 0.0) / sec / 1e12 / fma_peak
            best = max(by_mem, by_math, by_fma)
            r.update(bound="hbm" if best == by_mem else "tensor" if best == by_math else "fp32 fma", frac=round(best, 4))
        table[key] = r
    return table


def measure(name: str, size: dict, layers: int, batch: int, context: int, prefill: int, steps: int, warmup: int,
            peaks: dict, gen, say) -> dict:
    out = {"size": dict(size), "layers": layers, "batch": batch, "context": context, "prefill_tokens": prefill}
    for design, cfg in configs(size, layers).items():
        say(f"{name}: building {design}, {layers} layers")
        # Tubepel's latents have no window: every page of a request stays until it ends
        live = context if design == "tubepel" else min(context, size["window"] + PAGE)
        per_seq = -(-(live + 2 * PAGE + steps + warmup + 64) // PAGE) * PAGE
        engine = Engine.from_config(cfg, seed=0, options=EngineOptions(
            dtype="bfloat16", page_size=PAGE, cache_tokens=max(batch * per_seq + 512, prefill + PAGE),
            max_requests=batch, max_step_tokens=max(prefill, batch), max_seq_len=context + 4096))
        workloads.randomise_cache(engine)
        ms, launches = workloads.decode_device(engine, batch, context, steps, warmup, gen)
        pre_ms = workloads.prefill_step(engine, prefill, gen)
        rec = {"decode_ms": round(ms, 4), "decode_tok_s": round(batch / (ms / 1e3), 1), "launches_per_step": launches,
               "prefill_ms": round(pre_ms, 3), "prefill_tok_s": round(prefill / (pre_ms / 1e3), 1),
               "weight_bytes": engine.model.step_weight_bytes(), "kv_bytes_per_token": engine.cache.kv_bytes_per_token(),
               "state_bytes_per_request": engine.cache.state_bytes_per_request()}
        # what a decode step must read: every weight that takes part (of the routed experts those that the batch's
        # tokens are expected to choose between them, each once), the live keys and values, and the state twice
        if design == "tubepel":
            W, F = size["window"], size["keep_first"]
            per_tok = {0: 0, 1: 0}                 # bytes a cached token costs in a windowed and in a latent layer
            per_tok[0] = size["kv_heads"] * (size["qk_row"] + size["v_row"]) * 2
            per_tok[1] = (size["kv_rank"] + size["rot_dim"]) * 2
            n_w, n_l = (layers + 1) // 2, layers // 2
            seen_w = work.live_keys(context, W) + min(F, max(0, context - W))
            nbytes = rec["weight_bytes"] + batch * (n_w * seen_w * per_tok[0] + n_l * context * per_tok[1])
            moe_layers = n_l
        else:
            nbytes = work.decode_step_bytes(rec["weight_bytes"], rec["kv_bytes_per_token"], [context] * batch, size["window"])
            moe_layers = layers
        E, K = size["experts"], size["top"]
        distinct = E * (1.0 - (1.0 - K / E) ** batch)
        nbytes += moe_layers * (distinct - K) * 3 * size["width"] * size["expert_ff"] * 2 + 2 * batch * rec["state_bytes_per_request"]
        rec["decode_bytes"] = int(nbytes)
        rec["decode_hbm_frac"] = round(nbytes / (ms / 1e3) / 1e9 / peaks["hbm_gbs"], 4)
        vocab = engine.model.vocab_size
        ids = workloads.seat(engine, [context] * batch)
        entries = [Entry(r, [int(torch.randint(0, vocab, (1,), generator=gen))], [0]) for r in ids]
        toks = torch.randint(0, vocab, (prefill,), generator=gen).tolist()
        rec[f"decode_b{batch}"] = kernel_table(engine, design, size, layers, entries, (), batch, [context] * batch, peaks)
        engine.cache.release_all()
        rec[f"prefill_{prefill}"] = kernel_table(engine, design, size, layers, [Entry("prompt", toks, [prefill - 1])],
                                                 ("prompt",), prefill, [prefill], peaks)
        engine.cache.release_all()
        out[design] = rec
        engine = None
        gc.collect()
        torch.cuda.empty_cache()
    t, f = out["tubepel"], out["fegizen"]
    out["tubepel_over_fegizen"] = {"decode_tok_s": round(t["decode_tok_s"] / f["decode_tok_s"], 3),
                                   "prefill_tok_s": round(t["prefill_tok_s"] / f["prefill_tok_s"], 3)}
    like = {}
    for label in (f"decode_b{batch}", f"prefill_{prefill}"):
        rows = {}
        for ours, theirs in LIKE:
            a, b = t[label].get(ours), f[label].get(theirs)
            if a and b and "frac" in a and "frac" in b and b["frac"] > 0:
                rows[ours] = {"like": theirs, "frac": a["frac"], "like_frac": b["frac"], "ratio": round(a["frac"] / b["frac"], 3)}
        like[label] = rows
    out["like"] = like
    return out


def run(sizes, layers: int, batch: int, prefill: int, steps: int, warmup: int, peaks: dict, gen, say) -> dict:
    result = {}
    for name in sizes:
        size = SIZES[name]
        result[name] = measure(name, size, layers, batch, 2 * size["window"], prefill, steps, warmup, peaks, gen, say)
    return result
