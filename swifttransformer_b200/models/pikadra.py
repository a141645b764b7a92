"""Pikadra put together from the parts.

A decoder-only model whose layers are listed in the configuration:

  embedding     x0 = embed[token] * embedding.scale
  layer i       h = N(x);  x <- x + (mixer(h) + ff(h))                      (block ``parallel``)
                N: RMS norm whose weight is kept as its difference from one ('l<i>.norm1', ``rmsnorm_offset``)
  mixer         'latent_attention': queries and keys/values through normed latents, a rotated key part shared by the
                heads (halves layout), a sink in the softmax, a sigmoid gate per head (``latent_attention``)
  feed-forward  dense: down(silu(gate h) * (up h)) (``gated``); moe: routed experts of that form plus a shared one
                with a sigmoid gate per token (``routed_experts``); or none
  loop          the layers start..stop-1 run ``times`` times with the same weights, every pass with cache entries of
                its own and opened by x <- W_in [x ; x0] + step[pass]            (block ``reentry``)
  output        N(x) with 'final.norm', product with the embedding table, times logit_scale, tanh cap

Tensor names are those of the design's checkpoints: 'embed', 'loop.in', 'loop.step', 'l<i>.norm1', 'l<i>.mix.*',
'l<i>.mlp.*' (experts 'l<i>.mlp.e<j>.*', 'l<i>.mlp.router', 'l<i>.mlp.shared.*'), 'final.norm'.  The model has no
position table and no context limit of its own.
"""
from __future__ import annotations

from ..config.pikadra import PikadraConfig
from ..parts.base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS
from ..parts.embedding import Embedding, OutputHead
from .base import LayerStep, ModelDef
from .registry import register_model


def _gated(W, inner, p):
    return FEED_FORWARDS.build("gated", hidden=W, inner=inner, activation="silu", gate_name=p + "gate",
                               up_name=p + "up", down_name=p + "down", float_out=True)


@register_model(PikadraConfig.ARCHITECTURE)
def build_pikadra(cfg: PikadraConfig) -> ModelDef:
    W, eps = cfg.width, cfg.norm_eps
    embedding = Embedding(cfg.vocab, W, W, "embed", scale=cfg.embedding_scale)
    blocks = []
    for i, layer in enumerate(cfg.layers):
        p, mx = f"l{i}.", layer["mixer"]
        m = p + "mix."
        rot = mx.get("rot") if mx["rot_dim"] else None
        mixer = MIXERS.build(
            "latent_attention", hidden=W, num_heads=mx["heads"], dim=mx["dim"], rot=mx["rot_dim"], vdim=mx["vdim"],
            kv_rank=mx["kv_rank"], q_rank=mx["q_rank"], scale=mx["scale"], eps=eps,
            qk_position=POSITION_ENCODINGS.build("rotary_halves", dims=rot["dims"], base=rot["base"]) if rot else None,
            names={"dq": m + "dq", "uq": m + "uq", "dkv": m + "dkv", "uk": m + "uk", "uv": m + "uv", "o": m + "o",
                   "q_norm": m + "dq.norm", "kv_norm": m + "dkv.norm", "sink": m + "sink", "gate": m + "g"})
        mlp = layer.get("mlp")
        if mlp is None:
            ffn = None
        elif mlp["kind"] == "dense":
            ffn = _gated(W, mlp["ff"], p + "mlp.")
        else:
            n, sh = mlp["router"]["experts"], mlp.get("shared")
            shared = FEED_FORWARDS.build("gated", hidden=W, inner=sh["ff"], activation="silu",
                                         gate_name=p + "mlp.shared.gate", up_name=p + "mlp.shared.up",
                                         down_name=p + "mlp.shared.down") if sh else None
            ffn = FEED_FORWARDS.build(
                "routed_experts", hidden=W, inner=mlp["expert"]["ff"], num_experts=n, top=mlp["router"]["top"],
                activation="silu", router_name=p + "mlp.router", shared=shared,
                shared_gate_name=p + "mlp.shared.sg" if sh else None,
                expert_names=[{k: f"{p}mlp.e{j}.{k}" for k in ("gate", "up", "down")} for j in range(n)])
        blocks.append(BLOCKS.build("parallel", mixer=mixer, feed_forward=ffn,
                                   norm1=NORMS.build("rmsnorm_offset", width=W, eps=eps, name=p + "norm1")))
    order, entry = [], 0
    reentry = None
    if cfg.loop:
        reentry = len(blocks)
        blocks.append(BLOCKS.build("reentry", width=W, passes=cfg.loop[2], in_name="loop.in", step_name="loop.step"))
    for i, t, opens in cfg.layer_runs():
        if opens:
            order.append(LayerStep(block=reentry, cache=-1, turn=t))
        order.append(LayerStep(block=i, cache=entry))       # every run of a layer has a cache entry of its own
        entry += 1
    final_norm = NORMS.build("rmsnorm_offset", width=W, eps=eps, name="final.norm")
    head = OutputHead(cfg.vocab, W, W, "head", tied_to="embed", scale=cfg.logit_scale, softcap=cfg.logit_softcap)
    return ModelDef(cfg, embedding, POSITION_ENCODINGS.build("none"), blocks, order, final_norm, head)
