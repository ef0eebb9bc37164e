"""The Gedalix decoder as data: which parts, with which sizes, in which order.

scaled token embedding + learned positions -> runs of [RMSNorm -> latent attention -> scaled residual ->
RMSNorm -> routed experts (+ shared expert) -> scaled residual] -> RMSNorm -> head.  A stretch of layers may run
several times in a row with the same weights (each pass with caches of its own); every pass starts by adding a row of
a small table to the residual stream, and every pass but the first the embedding output as well.

Tensor names: `embed`, `pos`, `loop.step`, `final.norm`, `head`; layer i: `l<i>.norm1`, `l<i>.norm2`, `l<i>.ls1`,
`l<i>.ls2`, `l<i>.mix.{q,dkv,dkv.norm,uk,uv,sink,g,o}`, `l<i>.mlp.{router,router.b,e<k>.{gate,up,down},
shared.{gate,up,down,sg}}`.

This file only describes; the parts it names live in `parts/` and know nothing of it.
"""
from __future__ import annotations

from ..config.gedalix import ARCHITECTURE, PRESETS, GedalixConfig
from ..config.registry import Architecture, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, RunSpec

MIXER_NAMES = dict(q="q", dkv="dkv", dkv_norm="dkv.norm", uk="uk", uv="uv", o="o", sink="sink", gate="g")


def _mixer(cfg: GedalixConfig, m: dict) -> PartSpec:
    params = dict(prefix="mix.", hidden_size=cfg.width, num_heads=m["heads"], dim=m["dim"], rot_dim=m["rot_dim"],
                  vdim=m["vdim"], kv_rank=m["kv_rank"], scale=float(m["scale"]), eps=float(cfg.norm_eps), sink=True,
                  gate=True, names=MIXER_NAMES)
    if m["rot_dim"]:
        rot = m.get("rot") or {}
        params["position"] = PartSpec("rotary", dict(head_dim=m["rot_dim"], rotary_dim=int(rot.get("dims", m["rot_dim"])),
                                                     theta=float(rot["base"]), layout="split_half"))
    return PartSpec("latent_attention", params)


def _feed_forward(cfg: GedalixConfig, mlp) -> PartSpec:
    if mlp is None:
        return PartSpec("none")
    params = dict(prefix="mlp.", hidden_size=cfg.width, experts=mlp["router"]["experts"], top=mlp["router"]["top"],
                  expert_size=mlp["expert"]["ff"], expert_names=("e{}.gate", "e{}.up", "e{}.down"), router_name="router",
                  router_bias_name="router.b")
    if mlp.get("shared") is not None:
        params["shared"] = PartSpec("swiglu", dict(prefix="shared.", hidden_size=cfg.width,
                                                   intermediate_size=mlp["shared"]["ff"], names=("gate", "up", "down")))
        params["shared_gate_name"] = "shared.sg"
    return PartSpec("routed_experts", params)


def build_spec(cfg: GedalixConfig) -> ModelSpec:
    cfg.validate()
    w, eps = cfg.width, float(cfg.norm_eps)
    norm = lambda name: PartSpec("rmsnorm", dict(prefix="", name=name, size=w, eps=eps))
    layers, tolerated = [], []
    for i, layer in enumerate(cfg.layers):
        layers.append(LayerSpec(
            prefix=f"l{i}.",
            block=PartSpec("pre_norm_residual", dict(residual_scale=float(cfg.residual_mult), layer_scale=("ls1", "ls2"), size=w)),
            mixer_norm=norm("norm1"), mixer=_mixer(cfg, layer["mixer"]),
            ffn_norm=norm("norm2") if layer.get("mlp") is not None else PartSpec("rmsnorm", dict(prefix="", name="norm2", size=w, eps=eps, absent=True)),
            feed_forward=_feed_forward(cfg, layer.get("mlp"))))
        if layer.get("mlp") is None:             # a layer without a feed-forward: its second norm and scale may still be stored
            tolerated += [f"l{i}.norm2", f"l{i}.ls2"]
    order = []
    for index, opens in cfg.run_order():
        entry = None
        if opens is not None:
            entry = PartSpec("pass_entry", dict(prefix="", name="loop.step", rows=cfg.loop[2], row=opens, hidden_size=w,
                                                add_embedding=opens > 0))
        order.append(RunSpec(layer=index, entry=entry))
    spec = ModelSpec(
        architecture=ARCHITECTURE, hidden_size=w, vocab_size=cfg.vocab, max_position=cfg.max_positions,
        embedding=PartSpec("token_embedding", dict(name="embed", vocab_size=cfg.vocab, hidden_size=w,
                                                   scale=float(cfg.embedding_scale))),
        position=PartSpec("learned", dict(prefix="", name="pos", max_position=cfg.max_positions, hidden_size=w)),
        layers=layers, order=order, final_norm=norm("final.norm"),
        head=PartSpec("lm_head", dict(name="head", vocab_size=cfg.vocab, hidden_size=w, tied_to=None)),
        tolerated_tensors=tuple(tolerated))
    spec.validate()
    return spec


register_architecture(Architecture(name=ARCHITECTURE, config_class=GedalixConfig, build_spec=build_spec,
                                   presets=PRESETS), replace=True)
