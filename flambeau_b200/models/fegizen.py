"""Fegizen: configuration -> ModelSpec.

A decoder of pre-norm blocks whose norms take the mean off (a weight, no bias).  What every sublayer reads is first
joined by a short causal convolution of itself over time (`canon1` in front of the mixer, `canon2` in front of the
feed-forward).  The mixer is, layer by layer, either attention over cached latents under a sliding window (queries
through a latent of their own, one rotated key part shared by the heads, rotary frequencies stretched, a sigmoid
gate on the heads' outputs; a layer may read an earlier layer's latents instead of forming its own) or gated linear
attention (a decay per key channel, a float32 matrix of state per head).  The feed-forward is dense (GELU-gated) or a
mixture of SiLU-gated experts chosen by softmax scores plus a correction, some of them experts without weights that
hand their input on, beside a shared expert.  After every layer the stream is replaced by a learned mix of the
embedding output and all layers' results so far (`dwa`).  The embedding and the logits are scaled.  Tensor names are
the checkpoint's: embed, l<i>.norm1 / norm2 / canon1 / canon2 / dwa, l<i>.mix.*, l<i>.mlp.*, final.norm, head.
"""
from __future__ import annotations

from ..config.fegizen import ARCHITECTURE, FegizenConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerCall, ModelSpec, PartSpec

NORM_INIT = ("one_plus_normal", 0.1)
DENSE_NAMES = ("gate", "up", "down")


def build_spec(cfg: FegizenConfig) -> ModelSpec:
    D = cfg.width
    n = len(cfg.layers)

    def norm(prefix, name):
        return PartSpec("norm", "layernorm", dict(width=D, eps=cfg.norm_eps, init=NORM_INIT, weight_name=name), prefix)

    def conv(prefix, name):
        if not cfg.canon_taps:
            return None
        return PartSpec("input_map", "time_conv", dict(width=D, taps=cfg.canon_taps, weight_name=name), prefix)

    # a layer whose latents are read by later layers keeps them as far back as the furthest-looking reader wants
    keep = {}
    for i, layer in enumerate(cfg.layers):
        if layer.type == "latent_attention":
            owner = layer.mixer.kv_from if layer.mixer.kv_from is not None else i
            w = layer.mixer.window
            keep[owner] = 0 if (owner in keep and keep[owner] == 0) or w == 0 else max(keep.get(owner, 1), w)

    layers, order = [], []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer.mixer
        if layer.type == "latent_attention":
            mixer = PartSpec("mixer", "latent_attention", dict(
                width=D, num_heads=m.heads, head_dim=m.dim, rot_dim=m.rot_dim, value_dim=m.vdim, kv_rank=m.kv_rank,
                q_rank=m.q_rank, window=m.window, scale=m.scale, eps=cfg.norm_eps,
                shares_latent=m.kv_from is not None, keep_window=keep[i] if m.kv_from is None else m.window,
                position=PartSpec("position", "rotary_neighbours", dict(
                    head_dim=m.rot_dim, theta=m.rot_base, rotary_dim=m.rot_dims,
                    stretch=m.stretch.to_dict() if m.stretch is not None else None)) if m.rot_dims else None),
                p + "mix.")
            order.append(LayerCall(i, cache_from=m.kv_from))
        else:
            mixer = PartSpec("mixer", "gated_linear_attention", dict(
                width=D, num_heads=m.heads, key_dim=m.dim, value_dim=m.vdim, tau=m.tau, eps=cfg.norm_eps,
                decay_rank=m.decay_rank), p + "mix.")
            order.append(LayerCall(i))
        params = dict(mixer=mixer, mixer_norm=norm(p, "norm1"), mixer_input=conv(p, "canon1"))
        f = layer.mlp
        if f is not None:
            if f.kind == "dense":
                ff = PartSpec("feed_forward", "gated_mlp", dict(width=D, inner=f.ff, activation="gelu_tanh",
                                                                names=DENSE_NAMES), p + "mlp.")
            else:
                shared = None
                if f.shared_ff is not None:
                    shared = PartSpec("feed_forward", "gated_mlp", dict(width=D, inner=f.shared_ff, activation="silu",
                                                                        names=DENSE_NAMES), p + "mlp.shared.")
                ff = PartSpec("feed_forward", "routed_experts", dict(
                    width=D, inner=f.ff, experts=f.experts, top=f.top, activation="silu", gated=True,
                    rule="softmax_of_all", weight_scale=f.scale, identity=f.identity, bias_name="correction",
                    shared=shared), p + "mlp.")
            params.update(feed_forward=ff, feed_forward_norm=norm(p, "norm2"), feed_forward_input=conv(p, "canon2"))
        block = PartSpec("block", "pre_norm", params, p)
        layers.append(PartSpec("block", "depth_averaged", dict(block=block, depth=i + 2, slots=n + 1, width=D,
                                                               weight_name="dwa"), p))
    return ModelSpec(
        hidden_size=D, vocab_size=cfg.vocab,
        embedding=PartSpec("embedding", "token_embedding", dict(vocab=cfg.vocab, width=D, scale=cfg.embedding_scale,
                                                                weight_name="embed"), ""),
        layers=layers, order=order, final_norm=norm("final.", "norm"),
        head=PartSpec("head", "lm_head", dict(vocab=cfg.vocab, width=D, weight_name="head", scale=cfg.logit_scale), ""))


register_architecture(ARCHITECTURE, FegizenConfig, build_spec, replace=True)
