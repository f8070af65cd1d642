"""Tubepel: configuration -> ModelSpec.

A decoder of pre-norm blocks (plain-weight RMS norms) on several copies of the residual stream: every sublayer reads
a learned mix of the copies and writes its output back into all of them through learned weights (`hc1.*` for the
mixer, `hc2.*` for the feed-forward); at the end the stream is the sum of the copies.  Without `streams` the blocks
are plain pre-norm blocks on one stream.  The mixer is, layer by layer, causal attention over cached latents
(queries through a latent of their own, one rotated key part shared by the heads; two type names that differ in which
dimensions a rotation pairs: neighbours, or the two halves of the rotated part) or grouped-query attention under a
sliding window that keeps the first tokens of a request visible, with a rotation on part of a head, a learned sink in
every head's softmax and a sigmoid gate on the heads' outputs.  The feed-forward is dense (W_down relu(W_up h)^2) or
a mixture of SiLU-gated experts chosen by the sigmoids of the router's logits, whose scores scale what the experts
read, beside a shared expert.  A stretch of layers [loop.start, loop.stop) runs loop.times times in a row on the same
weights, every pass with a cache of its own.  Tensor names are the checkpoint's: embed, l<i>.norm1 / norm2,
l<i>.hc1.* / hc2.*, l<i>.mix.*, l<i>.mlp.*, final.norm, head.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.tubepel import ARCHITECTURE, LATENT_PAIRING, TubepelConfig
from ..parts.spec import LayerCall, ModelSpec, PartSpec

NORM_INIT = ("one_plus_normal", 0.1)
ATTENTION_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "sink": "sink", "g": "g"}
ROTARY_PARTS = {"neighbours": "rotary_neighbours", "halves": "rotary_half"}


def build_spec(cfg: TubepelConfig) -> ModelSpec:
    D = cfg.width

    def norm(prefix, name):
        return PartSpec("norm", "rmsnorm", dict(width=D, eps=cfg.norm_eps, init=NORM_INIT, weight_name=name), prefix)

    layers = []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer.mixer
        if layer.type in LATENT_PAIRING:
            position = None
            if m.rot_dims:
                position = PartSpec("position", ROTARY_PARTS[LATENT_PAIRING[layer.type]],
                                    dict(head_dim=m.rot_dim, theta=m.rot_base, rotary_dim=m.rot_dims))
            mixer = PartSpec("mixer", "latent_attention", dict(
                width=D, num_heads=m.heads, head_dim=m.dim, rot_dim=m.rot_dim, value_dim=m.vdim, kv_rank=m.kv_rank,
                q_rank=m.q_rank, window=0, scale=m.scale, eps=cfg.norm_eps, gate=False, position=position), p + "mix.")
        else:
            mixer = PartSpec("mixer", "attention", dict(
                width=D, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim, value_dim=m.vdim, window=m.window,
                keep_first=m.keep_first, scale=m.scale, sink=True, gate=True, names=ATTENTION_NAMES,
                weights_float32=True,
                position=PartSpec("position", "rotary_half", dict(head_dim=m.dim, theta=m.rot_base, rotary_dim=m.rot_dims))
                if m.rot_dims else None), p + "mix.")
        params = dict(mixer=mixer, mixer_norm=norm(p, "norm1"))
        f = layer.mlp
        if f is not None:
            if f.kind == "dense":
                ff = PartSpec("feed_forward", "mlp", dict(width=D, inner=f.ff, activation="relu_squared",
                                                          names=("up", "down")), p + "mlp.")
            else:
                shared = None
                if f.shared_ff is not None:
                    shared = PartSpec("feed_forward", "gated_mlp", dict(width=D, inner=f.shared_ff, activation="silu",
                                                                        names=("gate", "up", "down")), p + "mlp.shared.")
                ff = PartSpec("feed_forward", "routed_experts", dict(
                    width=D, inner=f.ff, experts=f.experts, top=f.top, activation="silu", gated=True, rule="sigmoid",
                    share_on_input=True, router_bias=False, shared=shared), p + "mlp.")
            params.update(feed_forward=ff, feed_forward_norm=norm(p, "norm2"))
        if cfg.streams:
            params.update(streams=cfg.streams, width=D, names=("hc1.", "hc2."))
            layers.append(PartSpec("block", "hyper_connections", params, p))
        else:
            layers.append(PartSpec("block", "pre_norm", params, p))

    n = len(cfg.layers)
    if cfg.loop is None:
        order = [LayerCall(i) for i in range(n)]
    else:
        lp = cfg.loop
        order = [LayerCall(i) for i in range(lp.start)]
        for t in range(lp.times):
            order += [LayerCall(i, pass_index=t) for i in range(lp.start, lp.stop)]
        order += [LayerCall(i) for i in range(lp.stop, n)]
    return ModelSpec(
        hidden_size=D, vocab_size=cfg.vocab,
        embedding=PartSpec("embedding", "token_embedding", dict(vocab=cfg.vocab, width=D, weight_name="embed"), ""),
        layers=layers, order=order, final_norm=norm("final.", "norm"),
        head=PartSpec("head", "lm_head", dict(vocab=cfg.vocab, width=D, weight_name="head"), ""))


register_architecture(ARCHITECTURE, TubepelConfig, build_spec, replace=True)
