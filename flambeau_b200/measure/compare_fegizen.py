"""Fegizen beside Nodepel at equal size: prefill and decode throughput and, kernel by kernel, how far each is from
its roofline.

`bench.py --only fegizen` runs, for each size of SIZES, a Fegizen model (layers that alternate gated linear attention
and attention over cached latents under a window, a convolution over time in front of every sublayer, routed experts
with identity experts and a shared expert, a mix over depth behind every layer) and a Nodepel model (the framework's
closest design: windowed attention beside a gated delta rule in every layer, routed experts with a shared expert)
with the same width, head counts, window, vocabulary, experts and number of layers, both with random weights in
bfloat16, through the same engine calls: one decode step of `batch` sequences that each hold `context` tokens, and
one step of `prefill` prompt tokens.  Per design it reports tokens a second and, per launcher (CUDA events around
every launcher call of an eager step, so serialised kernels), launches and microseconds per layer that runs it, the
work of one launch and the fraction of the measured peak that bounds it.  `like` pairs every kernel of the new design
with the kernel of Nodepel that does the like job and gives the ratio of their fractions (below 0.5: more than twice
as far from the roofline).

Work of one launch over `rows` rows (D = width):
  attention          4 * seen * heads * row flops, row = latent + rotated part (the cache row is key and value at
                     once); bytes: live keys * row * 2 + queries and outputs.  Nodepel: as measure/compare.py counts it
  recurrence         per token and head 5 * dk * dv flops (k v^T, the decay and the add as one fused multiply-add, S^T q)
                     against the delta rule's 8; float32 on the CUDA cores; per request the state once in and out
  recurrence_prepare the projection's float32 rows in, q, k, v and the decays out (Nodepel: rows in, q, k, v out)
  cache_write        the projection's float32 rows in, the query's latent and the cache row out
  norm               the stream in and out, the part's output in, normalised rows out (float32 here, as the convolution
                     that follows rounds once; bfloat16 in Nodepel)
  time_conv          normalised float32 rows in, bfloat16 rows out
  depth_mix          every kept result so far in, the newest and the stream out (averaged over the layers)
  head_map           2 * rows * heads * in * out flops for the map per head in front of and behind the attention (on
                     the tensor cores when serving) and the rows it reads and writes
  routed_product     4 * pairs * D * expert inner size flops for both products (6 with a gate); bytes: the weights of the
                     experts that were chosen, once
"""
from __future__ import annotations

import gc

import torch

from ..config.fegizen import FegizenConfig
from ..engine.batch import Entry
from ..engine.step import Engine, EngineOptions
from . import work, workloads
from .compare import PAGE, sections_by_class
from .compare_nodepel import SIZES as NODEPEL_SIZES, configs as nodepel_configs, fp32_fma_tflops

# what Fegizen adds to the sizes of measure/compare_nodepel.py: the latent attention's unrotated and rotated key size,
# value size, the two latents, taps, identity experts
SIZES = {
    "1b": dict(NODEPEL_SIZES["1b"], dim=128, rot_dim=64, vdim=128, kv_rank=192, q_rank=768, taps=4, identity=2, tau=16.0),
    "7b": dict(NODEPEL_SIZES["7b"], dim=128, rot_dim=64, vdim=128, kv_rank=192, q_rank=1536, taps=4, identity=2, tau=16.0),
}

CLASS_OF = {"paged_attention_mma": "attention", "paged_attention_simt": "attention",
            "qk_norm_rope_kv_write": "cache_write", "mla_latents": "cache_write",
            "add_rms_norm": "norm", "add_layer_norm": "norm", "gate_mul": "gate_mul",
            "gdr_prepare": "recurrence_prepare", "gla_prepare": "recurrence_prepare",
            "gdr_recurrent": "recurrence", "gla_recurrent": "recurrence", "gdr_out_norm": "recurrence_out",
            "branch_norm_mix": "branch_mix", "moe_choose": "router", "moe_sort": "expert_order",
            "moe_gather_rows": "expert_gather", "moe_combine": "expert_combine", "activation": "activation",
            "gemm_tc_grouped": "routed_product", "gemm_tc_grouped_gated": "routed_product",
            "gemm_simt_grouped": "routed_product", "time_conv": "time_conv", "depth_average": "depth_mix",
            "head_linear": "head_map"}

# (kernel of Fegizen, the like kernel of Nodepel); kernels that only Fegizen has are set beside the kernel of Nodepel
# that is bound by the same thing (rows through memory: its norm)
LIKE = [("attention", "attention"), ("cache_write", "cache_write"), ("recurrence", "recurrence"),
        ("recurrence_prepare", "recurrence_prepare"), ("recurrence_out", "recurrence_out"), ("norm", "norm"),
        ("time_conv", "norm"), ("depth_mix", "norm"), ("routed_product", "routed_product"),
        ("expert_combine", "expert_combine"), ("router", "router")]


def fegizen_config(size: dict, layers: int) -> FegizenConfig:
    moe = {"kind": "moe", "router": {"experts": size["experts"], "identity": size["identity"], "top": size["top"],
                                     "scale": 1.0}, "expert": {"ff": size["expert_ff"]}, "shared": {"ff": size["shared_ff"]}}
    linear = {"type": "gla", "mixer": {"heads": size["r_heads"], "dim": size["r_dk"], "vdim": size["r_dv"],
                                       "tau": size["tau"], "decay_rank": 16}, "mlp": moe}
    latent = {"type": "latent_attention",
              "mixer": {"heads": size["heads"], "dim": size["dim"], "rot_dim": size["rot_dim"], "vdim": size["vdim"],
                        "kv_rank": size["kv_rank"], "q_rank": size["q_rank"], "mask": {"size": size["window"]},
                        "rot": {"base": 1e6, "dims": size["rot_dim"],
                                "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}},
                        "scale": (size["dim"] + size["rot_dim"]) ** -0.5}, "mlp": moe}
    return FegizenConfig.from_dict({
        "architecture": "Fegizen", "canon": {"taps": size["taps"]}, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
        "logit_scale": 1.0, "vocab": size["vocab"], "width": size["width"],
        "layers": [linear if i % 2 == 0 else latent for i in range(layers)]})


def configs(size: dict, layers: int) -> dict:
    return {"fegizen": fegizen_config(size, layers), "nodepel": nodepel_configs(size, layers)["nodepel"]}


def seen_and_keys(size: dict, rows: int, contexts):
    W = size["window"]
    if len(contexts) == rows:
        seen = sum(work.live_keys(c, W) for c in contexts)
        return seen, seen
    ctx = contexts[0]
    return work.keys_seen(range(ctx - rows, ctx), W), ctx - (max(0, ctx - rows - W + 1) if W else 0)


def kernel_work(design: str, size: dict, layers: int, rows: int, contexts) -> dict:
    """class -> flops / fma_flops / bytes of one launch."""
    D, n_seqs = size["width"], (len(contexts) if len(contexts) == rows else 1)
    seen, keys = seen_and_keys(size, rows, contexts)
    H, dk, dv = size["r_heads"], size["r_dk"], size["r_dv"]
    pairs = rows * size["top"]
    experts_read = min(size["experts"], pairs)
    if design == "fegizen":
        row = size["kv_rank"] + size["rot_dim"]
        Ha = size["heads"]
        proj = size["q_rank"] + row + Ha * size["vdim"]
        r_cols = 2 * H * dk + 2 * H * dv + 16
        return {
            "attention": dict(flops=4.0 * seen * Ha * row, bytes=keys * row * 2 + 2 * rows * Ha * row * 2),
            "cache_write": dict(bytes=rows * (proj * 4 + (size["q_rank"] + row) * 2)),
            "recurrence": dict(fma_flops=5.0 * rows * H * dk * dv, bytes=n_seqs * 2 * H * dk * dv * 4 + rows * H * dv * 4),
            "recurrence_prepare": dict(bytes=rows * 4 * (r_cols + 3 * H * dk + H * dv)),
            "recurrence_out": dict(bytes=rows * H * dv * (4 + 4 + 2)),
            "norm": dict(bytes=rows * D * (4 + 4 + 4 + 4)),
            "time_conv": dict(bytes=rows * D * (4 + 2)),
            "depth_mix": dict(bytes=rows * D * 4 * ((layers + 3) / 2.0 + 3)),
            # (the mean of its two uses: float32 query rows in and latent-sized rows out; those in, value rows out
            # and the gate's float32 rows in)
            "head_map": dict(flops=2.0 * rows * Ha * size["kv_rank"] * (size["dim"] + size["vdim"]) / 2.0,
                             bytes=rows * Ha * ((size["dim"] + size["rot_dim"]) * 4 + 2 * row * 2
                                                + size["vdim"] * (2 + 4)) / 2.0),
            "routed_product": dict(flops=6.0 * pairs * D * size["expert_ff"],
                                   bytes=experts_read * 3 * D * size["expert_ff"] * 2),
            "expert_combine": dict(bytes=rows * D * 4 * (size["top"] + 2)),
            "router": dict(bytes=rows * (size["experts"] + size["identity"]) * 4),
        }
    Ha, G = size["heads"], size["kv_heads"]
    cols = Ha * size["qk_row"] + G * (size["qk_row"] + size["v_row"])
    Gr = size["r_qk_heads"]
    r_cols = 2 * Gr * dk + H * dv
    return {
        "attention": dict(flops=4.0 * seen * Ha * size["qk_row"],
                          bytes=keys * G * (size["qk_row"] + size["v_row"]) * 2 + rows * Ha * 2 * size["qk_row"] * 2),
        "cache_write": dict(bytes=rows * cols * (4 + 2)),
        "recurrence": dict(fma_flops=8.0 * rows * H * dk * dv, bytes=n_seqs * 2 * H * dk * dv * 4 + rows * H * dv * 4),
        "recurrence_prepare": dict(bytes=rows * 4 * (r_cols + 2 * H + H * dv + r_cols + 2 * H)),
        "recurrence_out": dict(bytes=rows * H * dv * (4 + 4 + 2)),
        "norm": dict(bytes=rows * D * (4 + 4 + 4 + 2)),
        "routed_product": dict(flops=4.0 * pairs * D * size["expert_ff"],
                               bytes=experts_read * 2 * D * size["expert_ff"] * 2),
        "expert_combine": dict(bytes=rows * D * 4 * (size["top"] + 2)),
        "router": dict(bytes=rows * size["experts"] * 4),
    }


def kernel_table(engine, design: str, size: dict, layers: int, entries, end, rows: int, contexts, peaks: dict) -> dict:
    """class -> launches a step, microseconds a launch, and for the classes with counted work the bound and the
    fraction of its measured peak."""
    secs = sections_by_class(engine, entries, end=end)
    merged: dict = {}
    for key, (n, total) in secs.items():
        key = CLASS_OF.get(key, key)
        a, b = merged.get(key, (0, 0.0))
        merged[key] = (a + n, b + total)
    works = kernel_work(design, size, layers, rows, contexts)
    fma_peak = fp32_fma_tflops(engine.runtime.device)
    table = {}
    for key, (n, total) in sorted(merged.items()):
        row = {"launches": round(n, 2), "us": round(total * 1e3 / max(n, 1e-9), 2)}
        w = works.get(key)
        if w and row["us"] > 0:
            sec = row["us"] * 1e-6
            by_mem = w.get("bytes", 0.0) / sec / 1e9 / peaks["hbm_gbs"]
            by_math = w.get("flops", 0.0) / sec / 1e12 / peaks["bf16_tflops"]
            by_fma = w.get("fma_flops", 0.0) / sec / 1e12 / fma_peak
            best = max(by_mem, by_math, by_fma)
            row.update(bound="hbm" if best == by_mem else "tensor" if best == by_math else "fp32 fma", frac=round(best, 4))
        table[key] = row
    return table


def measure(name: str, size: dict, layers: int, batch: int, context: int, prefill: int, steps: int, warmup: int,
            peaks: dict, gen, say) -> dict:
    out = {"size": dict(size), "layers": layers, "batch": batch, "context": context, "prefill_tokens": prefill}
    for design, cfg in configs(size, layers).items():
        say(f"{name}: building {design}, {layers} layers")
        live = min(context, size["window"] + PAGE)
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
        nbytes = work.decode_step_bytes(rec["weight_bytes"], rec["kv_bytes_per_token"], [context] * batch, size["window"])
        E, K = size["experts"], size["top"]
        distinct = E * (1.0 - (1.0 - K / E) ** batch)
        per_expert = (3 if design == "fegizen" else 2) * size["width"] * size["expert_ff"] * 2
        nbytes += layers * (distinct - K) * per_expert + 2 * batch * rec["state_bytes_per_request"]
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
    f, m = out["fegizen"], out["nodepel"]
    out["fegizen_over_nodepel"] = {"decode_tok_s": round(f["decode_tok_s"] / m["decode_tok_s"], 3),
                                   "prefill_tok_s": round(f["prefill_tok_s"] / m["prefill_tok_s"], 3)}
    like = {}
    for label in (f"decode_b{batch}", f"prefill_{prefill}"):
        rows = {}
        for ours, theirs in LIKE:
            a, b = f[label].get(ours), m[label].get(theirs)
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
