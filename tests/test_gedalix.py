"""Host-side tests of the Gedalix architecture: configuration, run order, the model as data, tensor names, the
cache manager's paged rows, and the plain implementation's own consistency."""
import copy
import math

import pytest
import torch

from microllm_rocm_b200.cache.manager import CacheManager
from microllm_rocm_b200.config import ConfigError, GedalixConfig, architecture_of, find_preset, get_architecture
from microllm_rocm_b200.parts.base import PagedKVNeed, PagedRowsNeed, Runtime
from microllm_rocm_b200.parts.build import build_model
from tests.gedalix_cases import CASES, random_weights, raw_config
from tests.plain import gedalix_plain as plain


def test_the_architecture_is_chosen_by_the_singular_key():
    raw = raw_config("a")
    assert "architectures" not in raw and raw["architecture"] == "Gedalix"
    arch = architecture_of(raw)
    assert arch.name == "Gedalix" and arch.config_class is GedalixConfig
    cfg = arch.config_class.from_dict(raw)
    assert GedalixConfig.from_dict(cfg.to_dict()) == cfg
    assert cfg.max_position_embeddings == raw["max_positions"] and cfg.vocab_size == raw["vocab"]


@pytest.mark.parametrize("loop, want", [
    (None, [(0, None), (1, None), (2, None), (3, None)]),
    ({"start": 1, "stop": 3, "times": 2}, [(0, None), (1, 0), (2, None), (1, 1), (2, None), (3, None)]),
    ({"start": 0, "stop": 4, "times": 1}, [(0, 0), (1, None), (2, None), (3, None)]),
    ({"start": 3, "stop": 4, "times": 3}, [(0, None), (1, None), (2, None), (3, 0), (3, 1), (3, 2)]),
])
def test_run_order(loop, want):
    raw = raw_config("a")
    raw["layers"] = [copy.deepcopy(raw["layers"][0]) for _ in range(4)]
    raw["loop"] = loop
    cfg = GedalixConfig.from_dict(raw)
    assert cfg.run_order() == want
    assert plain.layer_order(raw) == want
    spec = get_architecture("Gedalix").build_spec(cfg)
    assert [(r.layer, None if r.entry is None else r.entry.params["row"]) for r in spec.order] == want
    for r in spec.order:
        if r.entry is not None:
            assert r.entry.params["add_embedding"] == (r.entry.params["row"] > 0)


def test_bad_configurations_are_refused():
    for change in (lambda r: r["layers"][0].update(type="other"), lambda r: r.update(loop={"start": 2, "stop": 1, "times": 2}),
                   lambda r: r["layers"][0]["mixer"].update(heads=0), lambda r: r["layers"][0]["mlp"]["router"].update(top=99),
                   lambda r: r["layers"][0]["mixer"]["rot"].update(dims=3), lambda r: r.pop("width")):
        raw = raw_config("a")
        change(raw)
        with pytest.raises(ConfigError):
            GedalixConfig.from_dict(raw)


@pytest.mark.parametrize("key", sorted(CASES))
def test_the_model_declares_the_checkpoints_names(key):
    raw = raw_config(key)
    cfg = GedalixConfig.from_dict(raw)
    model = build_model(get_architecture("Gedalix").build_spec(cfg), Runtime(torch.device("cpu"), torch.float32))
    declared = {n: tuple(s.shape) for n, s in model.expected_tensors().items()}
    weights = random_weights(raw, 0)
    assert declared == {n: tuple(t.shape) for n, t in weights.items()}
    # one cache of rows per run, a looped layer one per pass
    runs = cfg.run_order()
    assert len(model.cache_entries) == len(runs)
    for (index, _), entry in zip(runs, model.cache_entries.values()):
        m = raw["layers"][index]["mixer"]
        assert entry.need == PagedRowsNeed(m["kv_rank"] + m["rot_dim"], None)
    # stacked experts and the fused input projection are filled piece by piece
    destinations, pieces = model.placements()
    for i, layer in enumerate(raw["layers"]):
        m = layer["mixer"]
        q = m["heads"] * (m["dim"] + m["rot_dim"])
        assert pieces[f"l{i}.mix.dkv"] == (f"l{i}.mix.in_proj.weight", q)
        assert pieces[f"l{i}.mix.g"] == (f"l{i}.mix.in_proj.weight", q + m["kv_rank"] + m["rot_dim"])
        if layer["mlp"]:
            ff = layer["mlp"]["expert"]["ff"]
            last = layer["mlp"]["router"]["experts"] - 1
            assert pieces[f"l{i}.mlp.e{last}.up"] == (f"l{i}.mlp.experts.gate_up", last * 2 * ff + ff)
            assert pieces[f"l{i}.mlp.e{last}.down"] == (f"l{i}.mlp.experts.down", last * raw["width"])
            assert pieces[f"l{i}.mlp.router"] == (f"l{i}.mlp.router.rows", 0)
            if layer["mlp"].get("shared"):
                assert pieces[f"l{i}.mlp.shared.sg"] == (f"l{i}.mlp.router.rows", last + 1)
    model.bind({n: t.float() for n, t in weights.items()})          # the pieces themselves bind too
    assert model.bound


def test_presets_build():
    arch, cfg = find_preset("gedalix-tiny")
    assert arch.name == "Gedalix" and len(cfg.run_order()) == 5


def test_paged_rows_share_pools_and_tables_with_keys_and_values():
    entries = {"rows": PagedRowsNeed(24), "kv": PagedKVNeed(2, 8), "rows2": PagedRowsNeed(40)}
    cache = CacheManager(entries, page_size=4, num_pages=6, max_requests=2, device=torch.device("cpu"))
    assert list(cache.groups) == ["full"]
    assert tuple(cache.kv_storage["rows"].shape) == (7, 4, 24) and tuple(cache.kv_storage["kv"].shape) == (7, 2, 2, 4, 8)
    assert cache.add("a") and cache.reserve("a", 9)
    cache.commit("a", 9)
    assert cache.block_table("full", ["a"]) == [[0, 1, 2]]
    cache.release("a")
    assert cache.add("b") and cache.reserve("b", 3)
    assert cache.block_table("full", ["b"]) == [[2]]           # the page freed last is used again first
    cache.check()


def test_plain_attention_without_expansion_equals_expansion():
    """The identity the engine rests on: scores and outputs through the latent equal those through expanded keys and values."""
    torch.manual_seed(0)
    H, T, dim, rot, rank, vdim = 3, 9, 8, 4, 12, 10
    F = torch.float64
    q, qr = torch.randn(H, T, dim, dtype=F), torch.randn(H, T, rot, dtype=F)
    c, kr = torch.randn(T, rank, dtype=F), torch.randn(T, rot, dtype=F)
    uk, uv = torch.randn(H, dim, rank, dtype=F), torch.randn(H, vdim, rank, dtype=F)
    sink = torch.randn(H, dtype=F)
    k = torch.einsum("hdr,tr->htd", uk, c)
    v = torch.einsum("hvr,tr->htv", uv, c)
    direct = plain.sink_softmax_attention(torch.cat([q, qr], -1), torch.cat([k, kr[None].expand(H, T, rot)], -1), v, 0.3, sink)
    a = torch.einsum("hdr,htd->htr", uk, q)
    latent = plain.sink_softmax_attention(torch.cat([a, qr], -1), torch.cat([c, kr], -1)[None].expand(H, T, rank + rot),
                                          c[None].expand(H, T, rank), 0.3, sink)
    through = torch.einsum("hvr,thr->thv", uv, latent)
    assert torch.allclose(direct, through, atol=1e-12)
    # the sink only enlarges the denominator: without it the weights sum to one
    no_sink = plain.sink_softmax_attention(torch.cat([q, qr], -1), torch.cat([k, kr[None].expand(H, T, rot)], -1),
                                           torch.ones(H, T, 1, dtype=F), 0.3, None)
    assert torch.allclose(no_sink, torch.ones_like(no_sink))
    with_sink = plain.sink_softmax_attention(torch.cat([q, qr], -1), torch.cat([k, kr[None].expand(H, T, rot)], -1),
                                             torch.ones(H, T, 1, dtype=F), 0.3, sink)
    assert (with_sink < 1).all()
    first = 1.0 / (1.0 + torch.exp(sink - 0.3 * ((q[:, 0] * k[:, 0]).sum(-1) + (qr[:, 0] * kr[0]).sum(-1))))
    assert torch.allclose(with_sink[0, :, 0], first)
    assert math.isclose(float(plain.rms(torch.tensor([[3.0, 4.0]], dtype=F), 0.0)[0, 0]), 3.0 / math.sqrt(12.5))
