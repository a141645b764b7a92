"""Fanidra put together from the parts.

A decoder-only model whose layers are listed in the configuration, each with a mixer of its own kind:

  embedding     x = embed[token] * embedding.scale
  layer i       x <- x + m * N(mixer(x + conv(x)));  x <- x + m * N(ff(x))        (block ``norm_after``)
                N: RMS norm with a single gain ('l<i>.norm1', 'l<i>.norm2'); m = residual_mult;
                conv: the convolution over time in front of the mixer ('l<i>.canon1', ``input_conv``)
  mixers        'attention': differential attention with short convolutions, query/key norm, rotated pairs,
                capped scores and a block-diagonal mask (``differential_attention``);
                'hgrn2': the gated linear recurrence (``hgrn2``)
  feed-forward  down(gelu_tanh(gate h) * (up h))  (``gated``)
  output        N(x) with 'final.norm', then the product with 'head'

Tensor names are those of the design's checkpoints: 'embed', 'l<i>.mix.*', 'l<i>.mlp.*', 'final.norm', 'head'.
The model has no position table and no context limit of its own.
"""
from __future__ import annotations

from ..config.fanidra import FanidraConfig
from ..parts.base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS
from ..parts.embedding import Embedding, OutputHead
from .base import LayerStep, ModelDef
from .registry import register_model


@register_model(FanidraConfig.ARCHITECTURE)
def build_fanidra(cfg: FanidraConfig) -> ModelDef:
    W, eps = cfg.width, cfg.norm_eps
    embedding = Embedding(cfg.vocab, W, W, "embed", scale=cfg.embedding_scale)
    blocks = []
    for i, layer in enumerate(cfg.layers):
        p, mx = f"l{i}.", layer["mixer"]
        m = p + "mix."
        if layer["type"] == "attention":
            rot = mx.get("rot")
            mixer = MIXERS.build(
                "differential_attention", hidden=W, num_heads=mx["heads"], num_kv_heads=mx.get("kv_heads", mx["heads"]),
                dim=mx["dim"], vdim=mx["vdim"], conv_taps=mx["conv"], scale=mx["scale"], softcap=mx.get("softcap", 0.0),
                block=mx["mask"]["size"] if mx.get("mask") else None, diff=mx["diff"], eps=eps,
                qk_position=POSITION_ENCODINGS.build("rotary_pairs", dims=rot["dims"], base=rot["base"]) if rot else None,
                names={"q": m + "q", "k": m + "k", "v": m + "v", "o": m + "o", "q_norm": m + "q.norm",
                       "k_norm": m + "k.norm", "lq1": m + "lq1", "lk1": m + "lk1", "lq2": m + "lq2", "lk2": m + "lk2"})
        else:
            mixer = MIXERS.build("hgrn2", hidden=W, num_heads=mx["heads"], dim=mx["dim"], vdim=mx["vdim"], eps=eps,
                                 names={"q": m + "q", "f": m + "f", "v": m + "v", "o": m + "o", "f_bias": m + "f.b",
                                        "lower": m + "lower", "norm": m + "norm"})
        if cfg.canon_taps:
            mixer = MIXERS.build("input_conv", inner=mixer, width=W, taps=cfg.canon_taps, name=p + "canon1")
        mlp = layer.get("mlp")
        ffn = FEED_FORWARDS.build("gated", hidden=W, inner=mlp["ff"], activation="gelu_tanh", gate_name=p + "mlp.gate",
                                  up_name=p + "mlp.up", down_name=p + "mlp.down") if mlp is not None else None
        norm = lambda name: NORMS.build("rmsnorm_scalar", width=W, eps=eps, name=name)
        blocks.append(BLOCKS.build("norm_after", mixer=mixer, feed_forward=ffn, norm1=norm(p + "norm1"),
                                   norm2=norm(p + "norm2") if ffn is not None else None, mult=cfg.residual_mult))
    final_norm = NORMS.build("rmsnorm_scalar", width=W, eps=eps, name="final.norm")
    head = OutputHead(cfg.vocab, W, W, "head")
    order = [LayerStep(block=i, cache=i) for i in range(len(blocks))]
    return ModelDef(cfg, embedding, POSITION_ENCODINGS.build("none"), blocks, order, final_norm, head)
