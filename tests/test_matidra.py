"""Host-side tests of the Matidra design: configuration, the model description, the cache manager's books for mixers
with several caches, and identities of the plain implementation that the GPU tests lean on."""
import copy
import math

import pytest
import torch

from tests.matidra_cases import CASES, case, raw_config, write_folder
from tests.plain import matidra_plain as plain


def _model(raw, dtype=torch.float32):
    from microllm_rocm_b200.config import get_architecture
    from microllm_rocm_b200.config.matidra import MatidraConfig
    from microllm_rocm_b200.parts.base import Runtime
    from microllm_rocm_b200.parts.build import build_model
    arch = get_architecture("Matidra")
    return build_model(arch.build_spec(MatidraConfig.from_dict(raw)), Runtime(torch.device("cpu"), dtype))


def _with_ranks(key):
    from microllm_rocm_b200.config.matidra import sizes_from_tensors
    raw, weights = case(key)
    return sizes_from_tensors(raw, {n: tuple(t.shape) for n, t in weights.items()}), weights


@pytest.mark.parametrize("key", sorted(CASES))
def test_declared_tensors_are_the_checkpoints(key):
    raw, weights = _with_ranks(key)
    expected = _model(raw).expected_tensors()
    assert set(expected) == set(weights)
    for name, spec in expected.items():
        assert tuple(spec.shape) == tuple(weights[name].shape), name


def test_inner_widths_come_from_the_tensors_shapes(tmp_path):
    from microllm_rocm_b200.config.qwen2 import ConfigError
    from microllm_rocm_b200.config.matidra import MatidraConfig
    from microllm_rocm_b200.config.registry import load_config
    raw, weights = case("a")
    with pytest.raises(ConfigError):
        MatidraConfig.from_dict(raw)                     # config.json alone does not say them
    folder = write_folder(str(tmp_path / "m"), raw, weights)
    arch, cfg = load_config(folder)
    assert arch.name == "Matidra"
    right = cfg.layers[0]["mixer"]["right"]
    assert (right["a_rank"], right["g_rank"]) == CASES["a"]["ranks"]
    again = MatidraConfig.from_dict(cfg.to_dict())
    assert again == cfg and hash(again) == hash(cfg)


def test_refusals():
    from microllm_rocm_b200.config.qwen2 import ConfigError
    from microllm_rocm_b200.config.matidra import MatidraConfig
    good, _ = _with_ranks("a")
    def broken(change):
        raw = copy.deepcopy(good)
        change(raw)
        with pytest.raises(ConfigError):
            MatidraConfig.from_dict(raw)
    broken(lambda r: r.pop("postln_alpha"))
    broken(lambda r: r["layers"][0].__setitem__("type", "mamba"))
    broken(lambda r: r["layers"][1]["mixer"].__setitem__("vdim", 48))             # values are the keys
    broken(lambda r: r["layers"][1]["mixer"]["rot"].__setitem__("dims", 13))
    broken(lambda r: r["layers"][0]["mixer"]["left"].__setitem__("kv_heads", 2))  # 3 heads do not divide
    broken(lambda r: r["layers"][0]["mlp"].__setitem__("kind", "moe"))
    broken(lambda r: r["layers"][0]["mixer"]["right"].__setitem__("conv", 0))


def test_every_mixer_gets_its_caches_and_the_pages_hold_both_widths():
    from microllm_rocm_b200.cache.manager import CacheManager, page_shape
    from microllm_rocm_b200.parts.base import FixedStateNeed, PagedKVNeed
    raw, _ = _with_ranks("a")
    model = _model(raw)
    names = set(model.cache_entries)
    assert names == {"run0.left.kv", "run0.left.conv", "run0.right.state", "run0.right.conv", "run1",
                     "run2.left.kv", "run2.left.conv", "run2.right.state", "run2.right.conv"}
    kv = model.cache_entries["run0.left.kv"].need
    assert isinstance(kv, PagedKVNeed) and (kv.head_dim, kv.value_dim) == (16, 24)
    assert page_shape(kv, 8) == (3 * 8 * (16 + 24),)
    assert page_shape(model.cache_entries["run1"].need, 8) == (2, 2, 8, 32)        # equal widths: the other kernels' layout
    assert model.cache_entries["run0.right.state"].need == FixedStateNeed((4, 16, 8), torch.float32)
    assert model.cache_entries["run0.left.conv"].need.shape == (2, 3 * 16 + 3 * 16 + 3 * 24)
    manager = CacheManager(model.cache_entries, page_size=8, num_pages=6, max_requests=2)
    assert manager.add("x") and manager.add("y") and not manager.add("z")
    assert manager.reserve("x", 30) and not manager.reserve("y", 30)
    manager.commit("x", 30); manager.release("x"); manager.check()
    assert manager.add("z") and manager.slot("z") == 0                              # the freed slot is used again


def test_no_convolution_means_no_convolution_state():
    raw, _ = _with_ranks("b")
    names = set(_model(raw).cache_entries)
    assert "run1.left" in names and "run1.left.conv" not in names and "run1.right.conv" in names


def test_stretched_frequencies_equal_the_plain_ones():
    from microllm_rocm_b200.parts.rotary import stretched_frequencies
    for dims, base, sc in ((12, 5000.0, {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 2.0}),
                           (32, 5e5, {"factor": 3.0, "original": 128, "fast": 16.0, "slow": 1.0}),
                           (4, 777.0, {"factor": 1.5, "original": 16, "fast": 4.0, "slow": 1.0})):
        freq, magnitude = stretched_frequencies(base, dims, sc)
        want, want_magnitude = plain.stretched_frequencies(dims, base, sc)
        assert torch.allclose(torch.from_numpy(freq).double(), want, rtol=1e-6)
        assert magnitude == pytest.approx(want_magnitude)
        plain_f, _ = plain.stretched_frequencies(dims, base, None)
        assert (want <= plain_f + 1e-12).all() and (want < plain_f).any()           # some pairs really are slowed down


def test_plain_delta_rule_carries_its_state():
    torch.manual_seed(0)
    T, H, dk, dv = 23, 2, 5, 7
    q, k = torch.randn(T, H, dk, dtype=plain.F), torch.randn(T, H, dk, dtype=plain.F)
    v, g, beta = torch.randn(T, H, dv, dtype=plain.F), torch.rand(T, H, dk, dtype=plain.F), torch.rand(T, H, dtype=plain.F)
    whole, S = plain.delta_rule(q, k, v, g, beta)
    a, Sa = plain.delta_rule(q[:9], k[:9], v[:9], g[:9], beta[:9])
    b, Sb = plain.delta_rule(q[9:], k[9:], v[9:], g[9:], beta[9:], Sa)
    assert torch.allclose(torch.cat([a, b]), whole) and torch.allclose(Sb, S)
    # the read-out sees the current token's write: with g = 1, beta = 1 and an empty state, o_0 = v_0 (k_0 . q_0)
    o, _ = plain.delta_rule(q[:1], k[:1], v[:1], torch.ones(1, H, dk, dtype=plain.F), torch.ones(1, H, dtype=plain.F))
    assert torch.allclose(o[0], v[0] * (k[0] * q[0]).sum(-1, keepdim=True))


def test_plain_convolution_and_temperature_edges():
    u = torch.arange(12, dtype=plain.F).view(6, 2)
    w = torch.tensor([[1.0, 10.0, 100.0], [0.0, 0.0, 1.0]], dtype=plain.F)
    y = plain.short_convolution(u, w)
    assert y[0].tolist() == [0.0, 1.0] and y[2, 0].item() == 0 * 1 + 2 * 10 + 4 * 100     # the last column is the current token's
    raw, weights = _with_ranks("d")
    # the query temperature steps where floor((p + 1) / every) does: positions 1|2 and 4|5 for every = 3
    m = raw["layers"][0]["mixer"]["left"]
    steps = [1.0 + m["q_temp"]["coef"] * math.log((p + 1) // m["q_temp"]["every"] + 1) for p in range(6)]
    assert steps[0] == steps[1] == 1.0 and steps[2] > steps[1] and steps[4] == steps[2] and steps[5] > steps[4]
