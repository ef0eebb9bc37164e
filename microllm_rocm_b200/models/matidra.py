"""The Matidra decoder as data: which parts, with which sizes, in which order.

token embedding -> layers of [mixer -> layer norm of (alpha x + mixer(x)) -> gated feed-forward with the tanh form of
gelu -> layer norm of (alpha x + ff(x))] -> layer norm -> head.  The sublayers read the stream itself (no norm in
front of them).  A layer's mixer is either softmax attention whose values are the projected keys (rms norm of q and k
per head, rotation of a part of each head in interleaved pairs with stretched frequencies), or two mixers side by side
on the same input whose results are added with fixed weights: softmax attention behind short convolutions (no rotation,
a query temperature, an output gate) and a gated delta rule with a decay per key channel.

Tensor names: `embed`, `final.norm`(+`.b`), `head`; layer i: `l<i>.norm1`, `l<i>.norm2` (+`.b`),
`l<i>.mix.{q,k,o,q.norm,k.norm}` or `l<i>.mix.left.{q,k,v,g,o,q.norm,k.norm,q.conv,k.conv,v.conv}` and
`l<i>.mix.right.{q,k,v,q.conv,k.conv,v.conv,b,a1,a2,A_log,dt_bias,g1,g2,norm,o}`, `l<i>.mlp.{gate,up,down}`.

This file only describes; the parts it names live in `parts/` and know nothing of it.
"""
from __future__ import annotations

from ..config.matidra import ARCHITECTURE, PRESETS, MatidraConfig, sizes_from_tensors
from ..config.registry import Architecture, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, RunSpec

SOFTMAX_NAMES = dict(q="q", k="k", v="v", o="o", q_norm="q.norm", k_norm="k.norm", gate="g", q_conv="q.conv",
                     k_conv="k.conv", v_conv="v.conv")
DELTA_NAMES = dict(q="q", k="k", v="v", o="o", q_conv="q.conv", k_conv="k.conv", v_conv="v.conv", beta="b", a1="a1", a2="a2",
                   a_log="A_log", dt_bias="dt_bias", g1="g1", g2="g2", norm="norm")


def _softmax(cfg: MatidraConfig, m: dict, prefix: str, *, values: str, conv: int, gate: bool) -> PartSpec:
    params = dict(prefix=prefix, hidden_size=cfg.width, num_heads=m["heads"], num_kv_heads=m["kv_heads"], dim=m["dim"],
                  vdim=m["vdim"], scale=float(m["scale"]), eps=float(cfg.norm_eps), values=values, conv=conv, gate=gate,
                  qk_norm=True, names=SOFTMAX_NAMES)
    if m.get("q_temp"):
        params["q_temp"] = (float(m["q_temp"]["coef"]), int(m["q_temp"]["every"]))
    rot = m.get("rot")
    if rot:
        sc = rot.get("scaling")
        position = dict(head_dim=m["dim"], rotary_dim=int(rot["dims"]), theta=float(rot["base"]), layout="interleaved")
        if sc:
            position["stretch"] = dict(factor=float(sc["factor"]), original=float(sc["original"]), fast=float(sc["fast"]),
                                       slow=float(sc["slow"]))
        params["position"] = PartSpec("rotary", position)
    return PartSpec("normed_attention", params)


def _mixer(cfg: MatidraConfig, layer: dict) -> PartSpec:
    m = layer["mixer"]
    if layer["type"] == "attention":
        return _softmax(cfg, m, "mix.", values="keys", conv=1, gate=False)
    left, right = m["left"], m["right"]
    return PartSpec("parallel", dict(
        prefix="mix.", hidden_size=cfg.width,
        branches=(("left", float(m["left_scale"]), _softmax(cfg, left, "left.", values="projected", conv=int(left.get("conv", 1)), gate=True)),
                  ("right", float(m["right_scale"]), PartSpec("gated_delta_rule", dict(
                      prefix="right.", hidden_size=cfg.width, num_heads=right["heads"], num_kv_heads=right["kv_heads"],
                      dim=right["dim"], vdim=right["vdim"], conv=int(right.get("conv", 1)), a_rank=right["a_rank"],
                      g_rank=right["g_rank"], eps=float(cfg.norm_eps), names=DELTA_NAMES))))))


def build_spec(cfg: MatidraConfig) -> ModelSpec:
    cfg.validate()
    w, eps = cfg.width, float(cfg.norm_eps)
    norm = lambda name, **more: PartSpec("layernorm", dict(prefix="", name=name, bias_name=name + ".b", size=w, eps=eps, **more))
    layers, tolerated = [], []
    for i, layer in enumerate(cfg.layers):
        mlp = layer.get("mlp")
        feed_forward = PartSpec("none") if mlp is None else PartSpec("swiglu", dict(
            prefix="mlp.", hidden_size=w, intermediate_size=mlp["ff"], names=("gate", "up", "down"), activation="gelu_tanh"))
        layers.append(LayerSpec(prefix=f"l{i}.", block=PartSpec("post_norm_residual", dict(alpha=float(cfg.postln_alpha))),
                                mixer_norm=norm("norm1"), mixer=_mixer(cfg, layer),
                                ffn_norm=norm("norm2", absent=mlp is None), feed_forward=feed_forward))
        if mlp is None:
            tolerated += [f"l{i}.norm2", f"l{i}.norm2.b"]
    spec = ModelSpec(
        architecture=ARCHITECTURE, hidden_size=w, vocab_size=cfg.vocab, max_position=cfg.max_positions,
        embedding=PartSpec("token_embedding", dict(name="embed", vocab_size=cfg.vocab, hidden_size=w)),
        position=PartSpec("none"), layers=layers, order=[RunSpec(layer=i) for i in range(len(layers))],
        final_norm=norm("final.norm"),
        head=PartSpec("lm_head", dict(name="head", vocab_size=cfg.vocab, hidden_size=w, tied_to=None)),
        tolerated_tensors=tuple(tolerated))
    spec.validate()
    return spec


register_architecture(Architecture(name=ARCHITECTURE, config_class=MatidraConfig, build_spec=build_spec,
                                   presets=PRESETS, sizes_from_tensors=sizes_from_tensors), replace=True)
