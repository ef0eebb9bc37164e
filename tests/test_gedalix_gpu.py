"""The Gedalix decoder on the GPU against its plain float64 restatement: each mechanism alone, then whole models cut
in every way (whole prompts, a tail decoded token by token, portions down to two tokens, mixed batches over a pool
so small that pages and slots are used again), in true fp32 and in bf16, and greedy generation through the
scheduler."""
import math

import pytest
import torch

from tests.gedalix_cases import CASES, random_weights, raw_config, write_folder
from tests.helpers import collect, random_tokens, steps_mixed, steps_portions, steps_prefill_then_decode, steps_whole
from tests.plain import gedalix_plain as plain

pytestmark = pytest.mark.gpu

FP32_TOL = 2e-5          # of the largest |logit| (measured worst: 2e-6)
BF16_TOL = 0.03          # of the largest |logit| (measured worst: 0.012)
DEV = "cuda:0"


def tol(dtype):
    return FP32_TOL if dtype == "float32" else BF16_TOL


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for key in CASES:
        raw = raw_config(key)
        weights = random_weights(raw, seed=len(key) + ord(key[0]))
        out[key] = (write_folder(str(tmp_path_factory.mktemp("gedalix_" + key)), raw, weights), raw, weights)
    return out


def engine_for(folder, dtype, max_tokens=1024, page_size=16, max_requests=4):
    from microllm_rocm_b200.engine.loading import load_engine
    return load_engine(folder, dtype=dtype, page_size=page_size, max_tokens=max_tokens, max_requests=max_requests)


_plain = {}


def plain_logits(key, raw, weights, tokens):
    k = (key, id(weights), tuple(tokens))
    if k not in _plain:
        _plain[k] = plain.forward(raw, weights, list(tokens)).float()
    return _plain[k]


def compare(got, key, raw, weights, requests, dtype):
    worst = 0.0
    for rid, toks in requests.items():
        ref = plain_logits(key, raw, weights, toks)
        rows = torch.stack([got[(rid, p)] for p in range(len(toks))])
        err = (rows - ref).abs().amax(dim=1) / ref.abs().max()
        assert torch.isfinite(rows).all(), f"case {key} request {rid}: logits that are not finite"
        over = err > tol(dtype)
        # bf16 rounds the router's input: where two experts' logits are a rounding error apart the choice may flip, and
        # that position (it alone) lands far off.  Such positions are rare; fp32 allows none.
        allowed = 0 if dtype == "float32" else max(1, len(toks) // 25)
        if int(over.sum()) > allowed:
            pos = int(over.nonzero()[0])
            raise AssertionError(f"case {key} request {rid}: {int(over.sum())} positions over the tolerance {tol(dtype)} ({allowed} allowed), "
                                 f"the first is {pos} of {len(toks)} (error {float(err[pos]):.3e} of the largest |logit|)")
        err = err[~over] if (~over).any() else err
        worst = max(worst, float(err.max()))
    print(f"[gedalix parity] case {key} {dtype}: worst error {worst:.3e} of the largest |logit|")
    return worst


def requests_for(raw, lengths, seed=0):
    return {f"r{i}": random_tokens(n, raw["vocab"], seed + 100 * i + n) for i, n in enumerate(lengths)}


# ------------------------------------------------------------------------------------------- mechanisms alone
@pytest.mark.parametrize("table_dtype", [torch.float32, torch.bfloat16])
def test_scaled_embedding_and_learned_positions(table_dtype):
    from microllm_rocm_b200.kernels import ops
    torch.manual_seed(1)
    table = torch.randn(50, 24, device=DEV).to(table_dtype)
    pos_table = torch.randn(40, 24, device=DEV).to(table_dtype)
    ids = torch.tensor([3, 49, 0, 7, 7], dtype=torch.int32, device=DEV)
    positions = torch.tensor([0, 39, 5, 6, 1], dtype=torch.int32, device=DEV)
    out = torch.empty(5, 24, device=DEV)
    ops.embed_gather_scaled(table, ids, out, 2.5)
    ops.add_table_rows(out, pos_table, positions)
    want = table.float()[ids.long()] * 2.5 + pos_table.float()[positions.long()]
    assert torch.allclose(out, want, atol=1e-6)


def test_scaled_add_norm_and_pass_entry():
    from microllm_rocm_b200.kernels import ops
    torch.manual_seed(2)
    x = torch.randn(7, 40, device=DEV)
    delta = torch.randn(3, 7, 40, device=DEV)                 # three partial sums
    scale, w, v = torch.randn(40, device=DEV), torch.randn(40, device=DEV), torch.randn(40, device=DEV)
    x0 = torch.randn(7, 40, device=DEV)
    want_x = x.double() + scale.double() * delta.double().sum(0)
    want = plain.rms(want_x, 1e-4) * w.double()
    res, out = x.clone(), torch.empty(7, 40, device=DEV)
    ops.add_scaled_rmsnorm(res, delta, scale, w, 1e-4, out)
    assert torch.allclose(res.double(), want_x, atol=1e-5) and torch.allclose(out.double(), want, atol=1e-5)
    res2 = x.clone()
    ops.add_scaled_inplace(res2, delta[0], scale)
    assert torch.allclose(res2, x + scale * delta[0], atol=1e-6)
    a, b = x.clone(), x.clone()
    ops.stream_entry(a, None, v)
    ops.stream_entry(b, x0, v)
    assert torch.allclose(a, x + v, atol=1e-6) and torch.allclose(b, x + x0 + v, atol=1e-6)


@pytest.mark.parametrize("experts, top", [(5, 2), (7, 1), (4, 4), (40, 6)])
def test_router_choice_weights_and_sorted_pairs(experts, top):
    from microllm_rocm_b200.kernels import moe
    torch.manual_seed(experts)
    T, W = 37, 48
    x, wr, b, sg = torch.randn(T, W, device=DEV), torch.randn(experts, W, device=DEV), torch.randn(experts, device=DEV), torch.randn(1, W, device=DEV)
    ids = torch.empty(T, top, dtype=torch.int32, device=DEV)
    weights, gate = torch.empty(T, top, device=DEV), torch.empty(T, device=DEV)
    both = torch.cat([wr, sg, torch.zeros(2, W, device=DEV)])            # router rows, the gate's row, padding
    logits = torch.stack([x[:, :20] @ both[:, :20].T, x[:, 20:] @ both[:, 20:].T])     # two partial sums of a split product
    moe.select(logits, experts, b, top, ids, weights, experts, gate)
    z = x.double() @ wr.double().T + b.double()
    chosen = torch.topk(z, top, dim=-1)
    assert torch.equal(ids.long().cpu(), chosen.indices.cpu())
    assert torch.allclose(weights.double(), torch.softmax(chosen.values, -1), atol=1e-5)
    assert torch.allclose(weights.sum(-1), torch.ones(T, device=DEV), atol=1e-6)
    assert torch.allclose(gate.double(), torch.sigmoid(x.double() @ sg.double().T)[:, 0], atol=1e-5)
    offsets = torch.empty(experts + 1, dtype=torch.int32, device=DEV)
    order = torch.empty(T * top, dtype=torch.int32, device=DEV)
    moe.align(ids, experts, offsets, order)
    offsets, order, flat = offsets.cpu().tolist(), order.cpu().tolist(), ids.cpu().reshape(-1).tolist()
    assert offsets[0] == 0 and offsets[-1] == T * top and sorted(order) == list(range(T * top))
    for e in range(experts):
        assert all(flat[pair] == e for pair in order[offsets[e]:offsets[e + 1]])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows, row_tile", [(5, 16), (100, 64), (100, 16)])
def test_grouped_product_over_sorted_rows_and_per_head(dtype, rows, row_tile):
    from microllm_rocm_b200.kernels import grouped
    torch.manual_seed(rows)
    G, N, K, top = 3, 21, 36, 2
    atol = 1e-4 if dtype == torch.float32 else 0.06
    w = torch.randn(G, N, K, device=DEV).to(dtype)
    # (a) rows sorted by group, read through a list of (token, choice) pairs, written back to the pairs' own rows
    a = torch.randn(rows, K, device=DEV).to(dtype)
    group_of_pair = torch.randint(0, G, (rows * top,))
    order = torch.argsort(group_of_pair, stable=True).to(torch.int32)
    counts = torch.bincount(group_of_pair, minlength=G)
    offsets = torch.cat([torch.zeros(1, dtype=torch.long), counts.cumsum(0)]).to(torch.int32)
    out = torch.zeros(rows * top, N, device=DEV)
    grouped.grouped_linear(a, w, out, rows=rows * top, group_offsets=offsets.to(DEV), a_rows=order.to(DEV), c_rows=order.to(DEV),
                           a_row_div=top, row_tile=row_tile)
    want = torch.stack([a.double()[pair // top] @ w.double()[group_of_pair[pair]].T for pair in range(rows * top)])
    assert torch.allclose(out.double(), want, atol=atol)
    # (b) one product per head over all rows, column blocks of the input and the output, a factor on the result
    a2 = torch.randn(rows, G * K + 5, device=DEV).to(dtype)
    out2 = torch.zeros(rows, G * (N + 2), device=DEV).to(dtype)
    factor = torch.rand(rows, G * (N + 2), device=DEV)
    grouped.grouped_linear(a2, w, out2, rows=rows, a_group_cols=K, c_group_cols=N + 2, factor=factor, row_tile=row_tile)
    for g in range(G):
        want2 = (a2.double()[:, g * K:(g + 1) * K] @ w.double()[g].T) * factor.double()[:, g * (N + 2):g * (N + 2) + N]
        assert torch.allclose(out2.double()[:, g * (N + 2):g * (N + 2) + N], want2, atol=atol)
        assert (out2[:, g * (N + 2) + N:(g + 1) * (N + 2)] == 0).all()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["a", "b"])
def test_every_run_of_the_layers_against_the_plain_residual_stream(folders, key, dtype):
    """The residual stream after every run (a looped layer counts each time): mixer, feed-forward, scales, pass entries."""
    from microllm_rocm_b200.engine.step import StepEntry
    folder, raw, weights = folders[key]
    tokens = random_tokens(45, raw["vocab"], 5)
    want = []
    plain.forward(raw, weights, tokens, collect=want)
    engine = engine_for(folder, dtype)
    got = {}
    engine.cache.add("x")
    engine.step([StepEntry("x", tokens, [0])], tensor_sink=lambda name, t: got.__setitem__(name, None if t is None else t.detach().clone()))
    engine.check_device_errors()
    runs = [n for n in got if n.endswith(".residual")]
    assert len(runs) == len(want)
    for name, ref in zip(runs, want):
        x = got[name].double()
        delta = got[name.replace(".residual", ".delta")]
        if delta is not None:
            x = x + (delta.double() if delta.dim() == 2 else delta.double().sum(0))
        err = float((x.cpu() - ref).abs().max() / ref.abs().max())
        assert err < (1e-5 if dtype == "float32" else 0.02), f"{name}: {err}"


@pytest.mark.parametrize("rows, row_tile", [(3, 16), (70, 16), (200, 64), (700, 128)])
def test_tensor_core_grouped_product_equals_the_plain_one(rows, row_tile):
    """bf16 operands on mma.sync against float64, sorted rows and per-head column blocks, K with a ragged last tile,
    the gate-times-up epilogue."""
    from microllm_rocm_b200.kernels import grouped
    torch.manual_seed(rows)
    G, N, K, top = 5, 72, 104, 2
    w = (torch.randn(G, N, K, device=DEV) * K ** -0.5).bfloat16()
    a = torch.randn(rows, K, device=DEV).bfloat16()
    assert grouped.mma_supported(a, w)
    group_of_pair = torch.randint(0, G, (rows * top,))
    group_of_pair[group_of_pair == 3] = 4                       # a group without rows
    order = torch.argsort(group_of_pair, stable=True).to(torch.int32).to(DEV)
    offsets = torch.cat([torch.zeros(1, dtype=torch.long), torch.bincount(group_of_pair, minlength=G).cumsum(0)]).to(torch.int32).to(DEV)
    out = torch.zeros(rows * top, N, device=DEV)
    grouped.grouped_linear(a, w, out, rows=rows * top, group_offsets=offsets, a_rows=order, c_rows=order, a_row_div=top, row_tile=row_tile)
    want = torch.stack([a.double()[pair // top] @ w.double()[group_of_pair[pair]].T for pair in range(rows * top)])
    assert torch.allclose(out.double(), want, atol=2e-3)
    # gate rows over up rows, silu(gate) * up as the epilogue; the output is in sorted order
    w2 = (torch.randn(G, 2 * 40, K, device=DEV) * K ** -0.5).bfloat16()
    act = torch.zeros(rows * top, 40, device=DEV, dtype=torch.bfloat16)
    grouped.grouped_silu_mul(a, w2, act, rows=rows * top, group_offsets=offsets, a_rows=order, a_row_div=top, row_tile=row_tile)
    for place, pair in enumerate(order.cpu().tolist()):
        gu = a.double()[pair // top] @ w2.double()[group_of_pair[pair]].T
        assert torch.allclose(act[place].double(), gu[:40] * torch.sigmoid(gu[:40]) * gu[40:], atol=0.02)
    # per head over all rows, with a factor
    a2 = torch.randn(rows, G * K, device=DEV).bfloat16()
    out2 = torch.zeros(rows, G * N, device=DEV, dtype=torch.bfloat16)
    factor = torch.rand(rows, G * N, device=DEV)
    grouped.grouped_linear(a2, w, out2, rows=rows, a_group_cols=K, c_group_cols=N, factor=factor, row_tile=row_tile)
    want2 = torch.cat([a2.double()[:, g * K:(g + 1) * K] @ w.double()[g].T for g in range(G)], 1) * factor.double()
    assert torch.allclose(out2.double(), want2, atol=0.03)


# ------------------------------------------------------------------------------------------- whole models, every cut
LENGTHS = {"a": [1, 2, 17, 70, 133], "b": [3, 9, 40, 65, 150], "c": [31, 129], "d": [5, 64, 97], "e": [2, 33, 140]}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", sorted(CASES))
@pytest.mark.parametrize("cut", ["whole", "tail", "portions"])
def test_one_request_at_a_time(folders, key, dtype, cut):
    folder, raw, weights = folders[key]
    reqs = requests_for(raw, LENGTHS[key])
    steps = {"whole": steps_whole, "tail": steps_prefill_then_decode, "portions": steps_portions}[cut](reqs)
    got = collect(engine_for(folder, dtype), steps)
    compare(got, key, raw, weights, reqs, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["a", "b"])
def test_mixed_batches_over_a_tight_pool(folders, key, dtype):
    """Up to four live requests, portions beside single tokens, some left out of a step; the pool holds just the peak,
    so pages go from one request to the next; every position must equal what the request gives alone."""
    folder, raw, weights = folders[key]
    reqs = requests_for(raw, [60, 33, 150, 90, 47, 128, 75, 20, 101, 64], seed=9)
    steps, peak = steps_mixed(reqs, max_live=4, seed=3)
    engine = engine_for(folder, dtype, max_tokens=peak, max_requests=4)
    got = collect(engine, steps)
    compare(got, key, raw, weights, reqs, dtype)
    pool = engine.cache.groups["full"].pool
    assert pool.total_allocations > pool.num_pages, "the pool was never tight enough to use a page again"


@pytest.mark.parametrize("key", ["c", "d"])
def test_tensor_core_attention_and_products_track_the_plain_kernels(folders, key):
    """bf16, the same schedule twice: on the tensor-core kernels (attention with key splits in the decoded tail, grouped
    products) and on the plain ones.  Tiles of 16 (token, head) rows span several tokens here (two and four heads)."""
    from microllm_rocm_b200.kernels import grouped, latent
    folder, raw, weights = folders[key]
    assert latent.mma_supported(raw["layers"][0]["mixer"]["kv_rank"], raw["layers"][0]["mixer"]["rot_dim"])
    reqs = requests_for(raw, [3, 50, 290], seed=2)
    steps, peak = steps_mixed(reqs, max_live=3, seed=5, decode_tail=20)
    fast = collect(engine_for(folder, "bfloat16", max_tokens=peak), steps)
    latent.USE_TENSOR_CORES = grouped.USE_TENSOR_CORES = False
    try:
        slow = collect(engine_for(folder, "bfloat16", max_tokens=peak), steps)
    finally:
        latent.USE_TENSOR_CORES = grouped.USE_TENSOR_CORES = True
    compare(fast, key, raw, weights, reqs, "bfloat16")
    compare(slow, key, raw, weights, reqs, "bfloat16")
    far = [k for k in fast if float((fast[k] - slow[k]).abs().max()) > 0.03 * float(slow[k].abs().max())]
    assert len(far) <= len(fast) // 25, f"{len(far)} of {len(fast)} positions differ between the kernels"


def test_fp32_does_not_depend_on_cuts_batches_or_pages(folders):
    folder, raw, weights = folders["a"]
    reqs = requests_for(raw, [70, 133, 20, 45], seed=4)
    whole = collect(engine_for(folder, "float32"), steps_whole(reqs))
    portions = collect(engine_for(folder, "float32", page_size=8), steps_portions(reqs, sizes=(2, 9, 2, 30, 1, 5)))
    steps, peak = steps_mixed(reqs, max_live=3, seed=1)
    mixed = collect(engine_for(folder, "float32", max_tokens=peak), steps)
    for k in whole:
        assert torch.equal(whole[k], portions[k]) and torch.equal(whole[k], mixed[k]), f"{k} differs between schedules"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_far_keys_page_borders_and_the_sink_decide_the_output(tmp_path_factory, dtype):
    """Peaky attention (queries scaled up): single keys, far back and at page borders, carry a position's output, in a
    prompt of several hundred tokens and in the tokens decoded after it; large sinks take most of the weight elsewhere.
    A key lost at a page's edge, a sink left out or scaled, or a position off by one would show at once."""
    raw = raw_config("c")
    for name, sharp, sink in (("sharp", 5.0, 1.0), ("sinks", 2.0, 4.0)):
        weights = random_weights(raw, seed=11, sharp=sharp, sink=sink)
        folder = write_folder(str(tmp_path_factory.mktemp("gedalix_" + name)), raw, weights)
        reqs = {"long": random_tokens(700, raw["vocab"], 21), "edge": random_tokens(16 * 9 + 1, raw["vocab"], 22)}
        for page_size, steps in ((16, steps_prefill_then_decode(reqs, tail=40)), (32, steps_portions(reqs, sizes=(127, 2, 33, 1, 64, 300)))):
            got = collect(engine_for(folder, dtype, max_tokens=1100, page_size=page_size), steps)
            compare(got, "c-" + name, raw, weights, reqs, dtype)
    # the attention really is peaky: dropping the sinks changes the sharp model's logits by far more than the tolerance
    no_sink = {k: (torch.full_like(v, -30.0) if k.endswith("mix.sink") else v) for k, v in weights.items()}
    a = plain.forward(raw, weights, reqs["edge"][:40])
    b = plain.forward(raw, no_sink, reqs["edge"][:40])
    assert float((a - b).abs().max() / a.abs().max()) > 10 * BF16_TOL


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_mixer_with_a_window_of_keys(dtype):
    """Latent attention takes a window as a parameter (no Gedalix configuration sets one): a model description with
    windows of 40 and 33 keys on its two layers, built from the same parts.  The cache manager gives pages behind a
    window back while the request lives; keys just inside and just outside the window, in prompt portions and in decoded
    tokens, at page borders (pages of 8 and 16), against the plain implementation with the same window."""
    import dataclasses

    from microllm_rocm_b200.config import GedalixConfig, get_architecture
    from microllm_rocm_b200.config.spec import PartSpec
    from microllm_rocm_b200.engine.loading import make_engine, prepare_kernels
    from microllm_rocm_b200.parts.base import Runtime
    from microllm_rocm_b200.parts.build import build_model
    from microllm_rocm_b200.weights.loader import target_dtype
    raw = raw_config("d")
    weights = random_weights(raw, seed=31, sharp=4.0)
    windows = [40, 33]
    spec = get_architecture("Gedalix").build_spec(GedalixConfig.from_dict(raw))
    layers = [dataclasses.replace(layer, mixer=PartSpec(layer.mixer.kind, {**layer.mixer.params, "window": w}))
              for layer, w in zip(spec.layers, windows)]
    spec = dataclasses.replace(spec, layers=layers)
    plain_raw = raw_config("d")
    for layer, w in zip(plain_raw["layers"], windows):
        layer["mixer"]["window"] = w
    reqs = {"w0": random_tokens(150, raw["vocab"], 41), "w1": random_tokens(77, raw["vocab"], 42)}
    rt = Runtime(torch.device(DEV), torch.float32 if dtype == "float32" else torch.bfloat16)
    for page_size, steps in ((8, steps_prefill_then_decode(reqs, tail=60)), (16, steps_portions(reqs, sizes=(39, 2, 41, 1, 33, 7)))):
        model = build_model(spec, rt)
        prepare_kernels(model)
        model.bind({n: weights[n].to(device=DEV, dtype=target_dtype(ws.role, rt)).contiguous() for n, ws in model.expected_tensors().items()})
        engine = make_engine(model, page_size, 64, 4, max_step_tokens=160)
        assert set(engine.cache.groups) == {"window40", "window33"}
        got = collect(engine, steps)
        compare(got, "d-window", plain_raw, weights, reqs, dtype)
        assert engine.cache.pages_released_by_window > 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_from_the_first_token(folders, dtype):
    """One token per step from position 0 on, over many pages."""
    folder, raw, weights = folders["d"]
    reqs = {"d": random_tokens(150, raw["vocab"], 8)}
    got = collect(engine_for(folder, dtype, page_size=8), steps_prefill_then_decode(reqs, tail=149))
    compare(got, "d", raw, weights, reqs, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_scheduler(folders, dtype):
    from microllm_rocm_b200.engine.llm import LLM
    from microllm_rocm_b200.sampling import GenerationConfig
    folder, raw, weights = folders["a"]
    prompts = [random_tokens(n, raw["vocab"], 50 + n) for n in (9, 40, 3)]
    llm = LLM(folder, dtype=dtype, page_size=16, max_tokens=512)
    outs = llm.generate(prompts, GenerationConfig(max_new_tokens=12, temperature=0.0))
    for prompt, got in zip(prompts, outs):
        assert len(got) == 12
        seq = list(prompt)
        for i, token in enumerate(got):
            ref = plain.forward(raw, weights, seq)[-1]
            if dtype == "float32":
                assert token == int(ref.argmax()), f"token {i} differs from the plain greedy choice"
            else:       # bf16 may leave the fp32 choice at a near tie: every pick must be a near maximum of the plain logits
                assert float(ref.max() - ref[token]) <= 0.05 * float(ref.abs().max())
            seq.append(token)
