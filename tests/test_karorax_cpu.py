"""The Karorax model in the engine (step function, cache and state manager, scheduler) on the CPU stand-in kernels
against the plain implementation; its parts alone against the plain functions; its configuration."""
import copy

import pytest
import torch

import plain_karorax as plain
import replay_modes
from helpers import assert_close, make_runner, random_tokens
from karorax_configs import CONFIGS, PAGE_SIZE, config_dict, make_karorax_folder
from torch_kernels import TorchKernels

REL = 1e-4


def _runner(tmp_path, name, num_pages=64, sharpen=1.0, **kw):
    folder = make_karorax_folder(tmp_path, name, sharpen=sharpen)
    runner = make_runner(folder, TorchKernels(), dtype="float32", device="cpu", page_size=PAGE_SIZE[name], num_pages=num_pages, **kw)
    config, weights = plain.read_folder(folder)
    return runner, config, weights


# ---- configuration --------------------------------------------------------------------------------------------------
def test_config_round_trip():
    from kvcache_b200.config import config_from_dict
    for name in CONFIGS:
        c = config_from_dict(config_dict(name))
        assert config_from_dict(c.to_dict()) == c
    c = config_from_dict(config_dict("A"))
    assert [l.type for l in c.layers] == ["latent_attention", "parallel", "latent_attention", "parallel"] and c.layers[3].mlp is None
    m = c.layers[0].mixer
    assert (m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank, m.window, m.kv_from) == (3, 8, 4, 12, 20, 11, None) and m.rot.dims == 4
    assert c.layers[2].mixer.kv_from == 0 and c.layers[2].mixer.window == 19
    left, right = c.layers[1].mixer.left, c.layers[1].mixer.right
    assert (left.heads, left.kv_heads, left.dim, left.vdim, left.softcap) == (4, 2, 16, 8, 20.0) and left.q_temp.every == 7
    assert right.decay == (0.5, 0.97, 0.8) and c.layers[0].mlp.ff == 48 and c.layers[1].mlp.shared_ff == 40
    assert c.logit_softcap == 9.0 and c.bigram.buckets == 97
    b = config_from_dict(config_dict("B"))
    assert b.layers[0].mlp.shared_ff is None and b.layers[0].mixer.left.q_temp is None and b.layers[0].mixer.left.softcap is None
    assert b.layers[1].mixer.window is None and b.bigram is None and b.logit_softcap is None


def test_config_faults_are_all_reported():
    from kvcache_b200.config import ConfigError, config_from_dict
    bad = config_dict("A")
    bad["layers"][0]["mixer"].pop("kv_rank")
    bad["layers"][1]["mixer"]["left"]["kv_heads"] = 3
    bad["layers"][1]["mlp"]["router"]["top"] = 9
    bad["layers"][1]["mixer"]["right"]["decay"] = [0.5, 0.9]
    bad["layers"][3]["type"] = "convolution"
    bad["layers"][2]["mixer"]["kv_from"] = 1
    del bad["norm"]
    with pytest.raises(ConfigError) as info:
        config_from_dict(bad)
    text = str(info.value)
    for piece in ("kv_rank", "not a multiple of kv_heads", "top 9", "2 numbers for 3 heads", "convolution", "kv_from 1", "norm"):
        assert piece in text, piece
    other = config_dict("A")
    other["layers"][2]["mixer"]["rot"]["base"] = 5.0          # the reader must agree with its source in what is cached
    with pytest.raises(ConfigError, match="must equal those of layer 0"):
        config_from_dict(other)


def test_model_as_data(tmp_path):
    """Cache entries: one row of kv_rank + rot_dim numbers per token for a latent layer that projects its own latent, none
    for a layer that reads another's (its call names the other's entry, which keeps the wider of the windows); pages and a
    float32 matrix per head for a parallel layer; one int32 per request for the pair embedding, after the layers' entries."""
    from kvcache_b200.cache import CacheManager
    from kvcache_b200.engine.loading import load_model
    model = load_model(make_karorax_folder(tmp_path, "A"), "float32", "cpu", max_positions=64)
    entries = model.cache_entries()
    assert len(entries) == 4
    assert (entries[0].kv.num_kv_heads, entries[0].kv.head_dim, entries[0].kv.v_head_dim, entries[0].kv.window) == (1, 24, 0, 19)
    assert entries[0].state is None and model.blocks[0].mixer.window == 11 and model.blocks[2].mixer.window == 19
    assert (entries[1].kv.num_kv_heads, entries[1].kv.head_dim, entries[1].kv.v_head_dim, entries[1].kv.window) == (2, 16, 8, None)
    assert set(entries[1].state) == {"right.memory"} and entries[1].state["right.memory"].shape == (3, 8, 12)
    assert entries[3].kv is None and entries[3].state["previous_token"].dtype == "int32"
    calls = [(c.layer, c.cache, c.writes_cache) for c in model.schedule]
    assert calls == [(0, 0, True), (1, 1, True), (2, 0, False), (3, 2, True)]
    assert model.blocks[3].ffn is None and model.logit_softcap == 9.0
    cache = CacheManager(entries, page_size=8, num_pages=8, max_slots=3, max_tokens_per_request=64, dtype="float32", device="cpu")
    assert cache.states[3]["previous_token"].shape == (3,)
    # In C two layers read layer 1's entry; the widest window among the three is what the entry keeps.
    c = load_model(make_karorax_folder(tmp_path, "C"), "float32", "cpu", max_positions=64)
    assert [(x.layer, x.cache, x.writes_cache) for x in c.schedule] == [(0, 0, True), (1, 1, True), (2, 1, False), (3, 1, False)]
    assert c.cache_entries()[1].kv.window == 21 and c.cache_entries()[0].kv.window == 1
    only_parallel = load_model(make_karorax_folder(tmp_path, "D"), "float32", "cpu", max_positions=64)
    assert all(e.kv is None or e.kv.num_kv_heads > 0 for e in only_parallel.cache_entries())


# ---- mechanisms alone ---------------------------------------------------------------------------------------------------
def _context(batch=None, kv=None, state=None):
    from kvcache_b200.engine.workspace import Workspace
    from kvcache_b200.parts.base import LayerContext
    return LayerContext(batch=batch, kernels=TorchKernels(wide=True), workspace=Workspace("cpu"), kv=kv, state=state)


def _weights(specs, seed, std=0.3):
    g = torch.Generator().manual_seed(seed)
    return {name: (torch.randn(spec.shape, generator=g) * std + (1.0 if name.endswith("norm") else 0.0)).to(torch.bfloat16)
            for name, spec in specs.items()}


def _scenario(segments, spec, page_size=4):
    from helpers import paged_scenario
    from kvcache_b200.parts.base import PagedKVView
    batch, kv = paged_scenario(segments, num_kv_heads=spec.num_kv_heads if spec else 1, head_dim=spec.head_dim if spec else 4,
                               page_size=page_size, dtype=torch.float32, device="cpu", fill_history=False, window=spec.window if spec else None)
    if spec is not None:
        kv = PagedKVView(spec=spec, k_pages=kv.k_pages, v_pages=torch.zeros(*kv.k_pages.shape[:-1], spec.v_head_dim),
                         block_table=kv.block_table, page_size=page_size, writes=True)
    return batch, kv


def test_norm_with_a_weight_around_zero_and_a_scale_on_the_result():
    """RMSNorm(offset=1) multiplies by 1 + w; a block with layer scales adds scale * sublayer(norm(h)), channel by channel."""
    from kvcache_b200.parts.base import ScaledDelta
    from kvcache_b200.parts.norm import RMSNorm
    W, eps = 24, 1e-5
    g = torch.Generator().manual_seed(1)
    norm = RMSNorm(W, eps, "n", offset=1.0)
    w = {"n": (torch.randn(W, generator=g) * 0.2).to(torch.bfloat16)}
    norm.bind(w, torch.device("cpu"))
    h = torch.randn(5, W, generator=g)
    delta, scale = torch.randn(5, W, generator=g), torch.randn(W, generator=g)
    out = torch.zeros(5, W)
    before = h.clone()
    norm.add_norm(h, ScaledDelta(delta, scale), out, _context())
    assert_close(h, before.double() + scale.double() * delta.double(), 1e-6, "the add")
    assert_close(out, plain.offset_norm(h.double(), w["n"].double(), eps), 1e-6, "the norm")
    assert norm.init_kinds() == {"n": "normal"}


@pytest.mark.parametrize("sizes", [dict(heads=3, dim=8, rot_dim=4, vdim=12, kv_rank=20, window=7, dims=4),
                                   dict(heads=1, dim=6, rot_dim=6, vdim=4, kv_rank=10, window=None, dims=4),
                                   dict(heads=4, dim=4, rot_dim=2, vdim=6, kv_rank=8, window=1, dims=2)])
def test_latent_attention_part_alone(sizes):
    """Sharp scores, whole and cut in two: neighbour pairs rotated (only part of the rotated numbers in one case), the window's
    first and last key, the sink in the denominator, one gate number per head."""
    from kvcache_b200.parts.latent_attention import LatentAttention
    from kvcache_b200.parts.position import RotaryHalf
    T, W, eps, scale = 29, 40, 1e-5, 6.0
    rot = {"base": 777.0, "dims": sizes["dims"]}
    part = LatentAttention(W, sizes["heads"], sizes["dim"], sizes["rot_dim"], sizes["vdim"], sizes["kv_rank"], None, scale=scale, eps=eps,
                           position=RotaryHalf(rot["dims"], rot["base"], 64), prefix="m.", dtype="float32", window=sizes["window"],
                           sink="learned", gate="head", rotary_layout="interleaved")
    w = _weights(part.tensor_specs(), 3)
    part.bind(w, torch.device("cpu"))
    assert set(w) == {"m.q", "m.dkv", "m.dkv.norm", "m.uk", "m.uv", "m.g", "m.o", "m.sink"} and w["m.g"].shape == (sizes["heads"], W)
    x = torch.randn(T, W, generator=torch.Generator().manual_seed(4))
    m = dict(heads=sizes["heads"], dim=sizes["dim"], rot_dim=sizes["rot_dim"], vdim=sizes["vdim"], kv_rank=sizes["kv_rank"], scale=scale, rot=rot)
    if sizes["window"]:
        m["mask"] = {"size": sizes["window"]}
    wd = {k: v.double() for k, v in w.items()}
    pos = torch.arange(T)
    want, _ = plain.latent_attention(m, wd, "m.", x.double(), pos, eps)
    if sizes["window"] and sizes["window"] > 1:   # one key more or one key less would show: the scores are sharp
        for other in (sizes["window"] + 1, sizes["window"] - 1):
            differs, _ = plain.latent_attention(dict(m, mask={"size": other}), wd, "m.", x.double(), pos, eps)
            assert (differs - want).abs().max() > 0.02 * want.abs().max()
    no_sink, _ = plain.latent_attention(m, dict(wd, **{"m.sink": torch.full((sizes["heads"],), -1e9, dtype=torch.float64)}), "m.", x.double(), pos, eps)
    assert (no_sink - want).abs().max() > 0.005 * want.abs().max()
    batch, kv = _scenario([(0, T)], part.cache_spec())
    assert_close(part.forward(x, _context(batch, kv)), want, 1e-5)
    second, kv = _scenario([(11, T - 11)], part.cache_spec())
    first, _ = _scenario([(0, 11)], part.cache_spec())
    got = [part.forward(x[:11], _context(first, kv)).clone(), part.forward(x[11:], _context(second, kv))]
    assert_close(torch.cat(got), want, 1e-5, "cut in two")


def test_a_layer_reads_the_latent_another_layer_cached():
    """The reader has no projection of its own: same cache rows, its own expansions, queries, window and sink."""
    from kvcache_b200.parts.base import PagedKVView
    from kvcache_b200.parts.latent_attention import LatentAttention
    from kvcache_b200.parts.position import RotaryHalf
    T, W, eps = 23, 32, 1e-5
    rope = RotaryHalf(4, 50.0, 64)
    common = dict(eps=eps, position=rope, dtype="float32", sink="learned", gate="head", rotary_layout="interleaved")
    owner = LatentAttention(W, 2, 8, 4, 6, 12, None, scale=3.0, prefix="a.", window=5, **common)
    reader = LatentAttention(W, 3, 6, 4, 10, 12, None, scale=4.0, prefix="b.", window=9, own_latent=False, **common)
    owner.keep_for_window(reader.window)
    assert owner.cache_spec().window == 9 and reader.cache_spec() is None and "b.dkv" not in reader.tensor_specs()
    w = {**_weights(owner.tensor_specs(), 1), **_weights(reader.tensor_specs(), 2)}
    owner.bind(w, torch.device("cpu"))
    reader.bind(w, torch.device("cpu"))
    wd = {k: v.double() for k, v in w.items()}
    x1, x2 = (torch.randn(T, W, generator=torch.Generator().manual_seed(s)) for s in (5, 6))
    pos = torch.arange(T)
    rot = {"base": 50.0, "dims": 4}
    m1 = dict(heads=2, dim=8, rot_dim=4, vdim=6, kv_rank=12, scale=3.0, rot=rot, mask={"size": 5})
    m2 = dict(heads=3, dim=6, rot_dim=4, vdim=10, kv_rank=12, scale=4.0, rot=rot, mask={"size": 9}, kv_from=0)
    want1, kept = plain.latent_attention(m1, wd, "a.", x1.double(), pos, eps)
    want2, _ = plain.latent_attention(m2, wd, "b.", x2.double(), pos, eps, kept)
    got1, got2, at = [], [], 0
    _, kv = _scenario([(0, T)], owner.cache_spec())
    for n in (9, 1, 13):
        batch, _ = _scenario([(at, n)], owner.cache_spec())
        reading = PagedKVView(spec=kv.spec, k_pages=kv.k_pages, v_pages=kv.v_pages, block_table=kv.block_table, page_size=kv.page_size, writes=False)
        got1.append(owner.forward(x1[at:at + n], _context(batch, kv)).clone())
        got2.append(reader.forward(x2[at:at + n], _context(batch, reading)).clone())
        at += n
    assert_close(torch.cat(got1), want1, 1e-5, "the owner, with its narrower window over the wider entry")
    assert_close(torch.cat(got2), want2, 1e-5, "the reader")


@pytest.mark.parametrize("sizes", [dict(heads=4, kv_heads=2, dim=16, vdim=8, softcap=2.0, q_temp=(0.5, 3)),
                                   dict(heads=3, kv_heads=3, dim=6, vdim=10, softcap=None, q_temp=None),
                                   dict(heads=5, kv_heads=1, dim=8, vdim=8, softcap=30.0, q_temp=(2.0, 1))])
def test_biased_attention_part_alone(sizes):
    """Query temperature by position, the cap (small enough to bend the scores), the bias that grows with the distance (its
    form slope * (i - j), per head), all keys visible; whole and cut in two."""
    from kvcache_b200.parts.attention import GQAAttention
    T, W, scale = 27, 40, 1.5
    part = GQAAttention(W, sizes["heads"], sizes["kv_heads"], sizes["dim"], qkv_bias=False, out_bias=False, position=None, window=None,
                        prefix="m.", dtype="float32", scale=scale, value_dim=sizes["vdim"], names=("q", "k", "v", "o"),
                        q_temperature=sizes["q_temp"], score_cap=sizes["softcap"], distance_bias="geometric", pad_values=True)
    w = _weights(part.tensor_specs(), 3)
    part.bind(w, torch.device("cpu"))
    assert_close(part.slopes, plain.distance_slopes(sizes["heads"]), 1e-6)
    x = torch.randn(T, W, generator=torch.Generator().manual_seed(4))
    m = dict(heads=sizes["heads"], kv_heads=sizes["kv_heads"], dim=sizes["dim"], vdim=sizes["vdim"], scale=scale)
    if sizes["softcap"]:
        m["softcap"] = sizes["softcap"]
    if sizes["q_temp"]:
        m["q_temp"] = {"coef": sizes["q_temp"][0], "every": sizes["q_temp"][1]}
    wd = {k: v.double() for k, v in w.items()}
    pos = torch.arange(T)
    want = plain.biased_attention(m, wd, "m.", x.double(), pos)
    for change in ({"softcap": 1000.0}, {"q_temp": {"coef": 0.0, "every": 1}}):
        if (sizes["softcap"] and "softcap" in change) or (sizes["q_temp"] and "q_temp" in change):
            assert (plain.biased_attention(dict(m, **change), wd, "m.", x.double(), pos) - want).abs().max() > 0.01 * want.abs().max()
    batch, kv = _scenario([(0, T)], part.cache_spec())
    out = torch.zeros(T, W)
    assert_close(part.forward(x, _context(batch, kv)), want, 1e-5)
    second, kv = _scenario([(10, T - 10)], part.cache_spec())
    first, _ = _scenario([(0, 10)], part.cache_spec())
    got = [part.forward(x[:10], _context(first, kv)).clone(), part.forward(x[10:], _context(second, kv))]
    assert_close(torch.cat(got), want, 1e-5, "cut in two")


@pytest.mark.parametrize("sizes", [dict(heads=3, dim=8, vdim=16, decay=(0.5, 0.97, 1.0)), dict(heads=1, dim=40, vdim=3, decay=(0.0,)),
                                   dict(heads=2, dim=33, vdim=70, decay=(0.998, 0.3))])
def test_lightning_attention_part_alone(sizes):
    """Whole, and cut into pieces that carry the state in a slot, against the plain recurrence; the norm runs over all heads at
    once; a state left in another slot does not leak."""
    from kvcache_b200.parts.recurrent import LightningAttention
    T, W, eps = 23, 48, 1e-5
    part = LightningAttention(W, sizes["heads"], sizes["dim"], sizes["vdim"], sizes["decay"], eps=eps, prefix="m.", dtype="float32")
    w = _weights(part.tensor_specs(), 5)
    part.bind(w, torch.device("cpu"))
    assert w["m.norm"].shape == (sizes["heads"] * sizes["vdim"],)
    x = torch.randn(T, W, generator=torch.Generator().manual_seed(7))
    m = dict(heads=sizes["heads"], dim=sizes["dim"], vdim=sizes["vdim"], decay=list(sizes["decay"]))
    want, _ = plain.lightning_attention(m, {k: v.double() for k, v in w.items()}, "m.", x.double(), eps)
    states = {"memory": torch.zeros(3, sizes["heads"], sizes["dim"], sizes["vdim"])}
    states["memory"][0].fill_(7.0)                                    # another request's state
    batch, _ = _scenario([(0, T)], None)
    batch.seg_slot[0] = 1
    assert_close(part.forward(x, _context(batch, state=states)), want, 1e-5)
    assert bool((states["memory"][0] == 7.0).all()) and float(states["memory"][1].abs().max()) > 0
    states, got, at = {"memory": torch.zeros(3, sizes["heads"], sizes["dim"], sizes["vdim"])}, [], 0
    for n in (1, 2, 9, 1, 10):
        batch, _ = _scenario([(at, n)], None)
        batch.seg_slot[0] = 2
        got.append(part.forward(x[at:at + n], _context(batch, state=states)).clone())
        at += n
    assert_close(torch.cat(got), want, 1e-5, "in pieces")


@pytest.mark.parametrize("E,top,shared", [(5, 2, 24), (3, 1, None), (4, 4, 8)])
def test_routed_feed_forward_part_alone(E, top, shared):
    """The router's bias decides choices; weights are the softmax over the chosen logits alone (they sum to 1); the experts
    are the plain gated form; a shared expert of its own size is added."""
    from kvcache_b200.parts.feedforward import GatedMLP, RoutedMLP
    T, W, F = 9, 40, 24
    sh = None if shared is None else GatedMLP(W, shared, activation="silu", prefix="f.shared.", dtype="float32", names=("gate", "up", "down"))
    part = RoutedMLP(W, F, E, top, activation="swiglu", scores="chosen", prefix="f.", dtype="float32", shared=sh, router_bias="router.b")
    w = _weights(part.tensor_specs(), 5)
    w["f.router.b"] = (torch.randn(E, generator=torch.Generator().manual_seed(8)) * 3).to(torch.bfloat16)
    part.bind(w, torch.device("cpu"))
    x = torch.randn(T, W, generator=torch.Generator().manual_seed(6))
    wd = {k: v.double() for k, v in w.items()}
    mlp = {"kind": "moe", "router": {"experts": E, "top": top}, "expert": {"ff": F}}
    if shared is not None:
        mlp["shared"] = {"ff": shared}
    assert_close(part.forward(x, _context()), plain.feed_forward(mlp, wd, "f.", x.double()), 1e-5)
    which, weight = plain.route(mlp, wd, "f.", x.double())
    assert torch.allclose(weight.sum(dim=-1), torch.ones(T, dtype=torch.float64))
    if top < E:
        unbiased, _ = plain.route(mlp, dict(wd, **{"f.router.b": torch.zeros(E, dtype=torch.float64)}), "f.", x.double())
        assert not torch.equal(which, unbiased)


def test_the_logits_are_capped(tmp_path):
    runner, config, weights = _runner(tmp_path, "A")
    tokens = random_tokens(config["vocab"], 12, 9)
    got = replay_modes.whole(runner, tokens)
    uncapped = plain.forward(dict(config, logit_softcap=None), weights, tokens)
    assert_close(got, config["logit_softcap"] * torch.tanh(uncapped / config["logit_softcap"]), REL)
    assert float((uncapped - got.double()).abs().max()) > 1e-3


def test_residual_stream_after_every_layer(tmp_path):
    """Layer by layer: a model cut after k layers (its final norm and head replaced by the identity) gives the plain
    implementation's residual stream after layer k."""
    folder = make_karorax_folder(tmp_path, "A")
    config, weights = plain.read_folder(folder)
    tokens = random_tokens(config["vocab"], 19, 3)
    streams = []
    plain.forward(config, weights, tokens, streams)
    from kvcache_b200.cache import CacheManager
    from kvcache_b200.engine.loading import load_model
    from kvcache_b200.engine.runner import ModelRunner, StepEntry
    for k in range(1, len(streams) + 1):
        model = load_model(folder, "float32", "cpu", max_positions=64)
        model.schedule = model.schedule[:k]
        model._writers = {c.cache: c.layer for c in model.schedule if c.writes_cache}
        model.final_norm.weight = torch.ones(model.width)
        model.final_norm.eps = 0.0
        model.head = torch.eye(model.width)
        model.vocab_size = model.width
        model.logit_softcap = None
        cache = CacheManager(model.cache_entries(), page_size=8, num_pages=16, max_slots=1, max_tokens_per_request=64, dtype="float32", device="cpu")
        runner = ModelRunner(model, cache, TorchKernels(wide=True), max_tokens_per_step=64)
        got = runner.step([StepEntry(cache.admit(), tokens, list(range(len(tokens))))]).double()
        want = streams[k - 1]
        want = want / torch.sqrt((want * want).mean(dim=-1, keepdim=True))
        assert_close(got, want, 1e-5, f"after layer {k}")


# ---- the model in the engine ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt_and_its_first_tokens(tmp_path, name):
    runner, config, weights = _runner(tmp_path, name)
    tokens = random_tokens(config["vocab"], 75, 1)
    want = plain.forward(config, weights, tokens)
    assert_close(replay_modes.whole(runner, tokens), want, REL)
    assert runner.cache.used_pages() == 0
    for n in (1, 2, 3):                 # a sequence's first tokens alone: the pair table's last row, empty states, the sink nearly alone
        assert_close(replay_modes.whole(runner, tokens[:n]), want[:n], REL, f"first {n}")


@pytest.mark.parametrize("name", list(CONFIGS))
def test_prefill_against_token_by_token_decoding(tmp_path, name):
    runner, config, weights = _runner(tmp_path, name)
    tokens = random_tokens(config["vocab"], 70, 2)
    want = plain.forward(config, weights, tokens)
    assert_close(replay_modes.last_32_one_by_one(runner, tokens), want[-33:], REL)
    assert_close(replay_modes.portions(runner, tokens, [1] * 70), want, REL, "every token alone")


@pytest.mark.parametrize("name", list(CONFIGS))
def test_portions_down_to_two_tokens(tmp_path, name):
    runner, config, weights = _runner(tmp_path, name)
    tokens = random_tokens(config["vocab"], 101, 3)
    want = plain.forward(config, weights, tokens)
    assert_close(replay_modes.portions(runner, tokens, [2, 17, 3, 31, 2, 16, 8, 22]), want, REL)
    assert_close(replay_modes.portions(runner, tokens, [40, 2, 2, 5, 52]), want, REL)


@pytest.mark.parametrize("name", list(CONFIGS))
def test_mixed_batches_with_pages_and_slots_used_again(tmp_path, name):
    """Unequal requests beside one another against each alone; a and b end and d and e take their slots, whose states
    (matrices, previous tokens) must start from nothing, and their pages, which hold other requests' rows."""
    page = PAGE_SIZE[name]
    runner, config, weights = _runner(tmp_path, name, num_pages=replay_modes.mixed_pool_tokens() // page)
    seqs = {k: random_tokens(config["vocab"], n, 10 + i) for i, (k, n) in enumerate(replay_modes.MIXED_LENGTHS)}
    got = replay_modes.mixed(runner, seqs)
    for k, tokens in seqs.items():
        assert_close(got[k], plain.forward(config, weights, tokens), REL, k)


@pytest.mark.parametrize("name", ["A", "C"])
def test_sharp_attention_at_the_windows_edges_in_prompts_and_decoding(tmp_path, name):
    """With the score scale multiplied, the softmax of most heads rests on single keys: a window one token too wide or too
    narrow (of the layer that owns the latent, or of one that reads it), or a key lost at a page border or at the start of a
    portion, changes the logits by far more than the tolerance."""
    runner, config, weights = _runner(tmp_path, name, sharpen=40.0, max_tokens_per_step=256, max_tokens_per_request=256)
    tokens = random_tokens(config["vocab"], 150, 5)
    want = plain.forward(config, weights, tokens)
    for index, layer in enumerate(config["layers"]):
        if layer["type"] != "latent_attention" or layer["mixer"]["mask"]["size"] < 2:
            continue
        for delta in (-1, 1):
            other = copy.deepcopy(config)
            other["layers"][index]["mixer"]["mask"]["size"] += delta
            assert (plain.forward(other, weights, tokens) - want).abs().max() > 0.01 * want.abs().max(), (index, delta)
    assert_close(replay_modes.portions(runner, tokens, [7, 2, 57, 64, 3, 17]), want, 1e-3)
    assert_close(replay_modes.last_32_one_by_one(runner, tokens), want[-33:], 1e-3)
    assert_close(replay_modes.portions(runner, tokens, [100] + [1] * 50), want, 1e-3, "the windows pass over decoded tokens")


def far_key_case(part, W, T, strength=40.0, seed=3):
    """Weights and inputs of a biased-attention part in which every query scores the sequence's FIRST key far above all
    others - although that key is the one the distance bias costs most: channel 0 of the input is 1 in the first row only
    and drives the keys along one direction, channel 1 is 1 in every row and drives the queries along the same direction."""
    g = torch.Generator().manual_seed(seed)
    w = {name: (torch.randn(spec.shape, generator=g) * 0.05).to(torch.bfloat16) for name, spec in part.tensor_specs().items()}
    D = part.head_dim
    u = torch.zeros(D)
    u[0] = 1.0
    q, k = w["m.q"].float(), w["m.k"].float()
    q[:, :2], k[:, :2] = 0.0, 0.0
    for h in range(part.num_heads):
        q[h * D:(h + 1) * D, 1] = u * strength
    for h in range(part.num_kv_heads):
        k[h * D:(h + 1) * D, 0] = u * strength
    w["m.q"], w["m.k"] = q.to(torch.bfloat16), k.to(torch.bfloat16)
    x = torch.randn(T, W, generator=g) * 0.1
    x[:, 0], x[:, 1] = 0.0, 1.0
    x[0, 0] = 1.0
    return w, x


def test_a_far_key_takes_all_the_weight_through_the_distance_bias():
    """Random weights would hide a lost far key among hundreds: here one key, hundreds of tokens and many pages back, takes all
    the weight, so every row's result is that key's value - in a prompt, in portions and for single tokens."""
    from kvcache_b200.parts.attention import GQAAttention
    T, W = 300, 24
    part = GQAAttention(W, 4, 2, 8, qkv_bias=False, out_bias=False, position=None, window=None, prefix="m.", dtype="float32", scale=1.0,
                        value_dim=6, names=("q", "k", "v", "o"), q_temperature=(0.4, 50), score_cap=None, distance_bias="geometric")
    w, x = far_key_case(part, W, T)
    part.bind(w, torch.device("cpu"))
    wd = {k: v.double() for k, v in w.items()}
    m = dict(heads=4, kv_heads=2, dim=8, vdim=6, scale=1.0, q_temp={"coef": 0.4, "every": 50})
    want = plain.biased_attention(m, wd, "m.", x.double(), torch.arange(T))
    first_value = plain.linear(x[:1].double(), wd["m.v"]).view(2, 6).repeat_interleave(2, dim=0).reshape(1, -1)
    assert_close(want[200:], plain.linear(first_value, wd["m.o"]).expand(T - 200, -1), 1e-3, "the first key takes all the weight")
    _, kv = _scenario([(0, T)], part.cache_spec(), page_size=16)
    got, at = [], 0
    for n in [130, 2, 100, 60] + [1] * 8:
        batch, _ = _scenario([(at, n)], part.cache_spec(), page_size=16)
        got.append(part.forward(x[at:at + n], _context(batch, kv)).clone())
        at += n
    assert_close(torch.cat(got), want, 1e-5)


def test_long_decoding_keeps_the_states_in_range(tmp_path):
    runner, config, weights = _runner(tmp_path, "A", max_tokens_per_step=512, max_tokens_per_request=512)
    tokens = random_tokens(config["vocab"], 300, 6)
    got = replay_modes.portions(runner, tokens, [20] + [1] * 280)
    assert_close(got, plain.forward(config, weights, tokens), REL)


def test_pages_behind_every_window_are_given_back(tmp_path):
    """C has only windowed latent layers: a long request never holds more pages than its widest window and a portion span."""
    runner, config, weights = _runner(tmp_path, "C", num_pages=24, max_tokens_per_step=64, max_tokens_per_request=512)
    from kvcache_b200.engine.runner import StepEntry
    tokens = random_tokens(config["vocab"], 200, 8)
    want = plain.forward(config, weights, tokens)
    slot, at, most = runner.cache.admit(), 0, 0
    got = []
    for n in [16] * 5 + [1] * 120:
        got.append(runner.step([StepEntry(slot, tokens[at:at + n], list(range(n)))]).clone())
        at += n
        most = max(most, runner.cache.used_pages())
    assert_close(torch.cat(got), want, REL)
    assert most <= 2 * ((21 - 1 + 16) // 4 + 2)                  # two groups (windows 1 and 21), pages of 4 tokens
    runner.cache.release(slot)
    assert runner.cache.used_pages() == 0


# ---- generation through the entry point and the scheduler -------------------------------------------------------------
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_greedy_generation_matches_plain(tmp_path, name):
    from kvcache_b200 import LLM, SamplingParams
    folder = make_karorax_folder(tmp_path, name)
    config, weights = plain.read_folder(folder)
    prompts = [random_tokens(config["vocab"], n, 40 + n) for n in (1, 9, 24, 40)]
    llm = LLM(folder, kernels=TorchKernels(), dtype="float32", device="cpu", page_size=PAGE_SIZE[name], num_pages=40, max_running=3,
              max_tokens_per_step=48, chunk_size=16, use_graphs=False)
    got = llm.generate(prompts, SamplingParams(max_new_tokens=6, ignore_eos=True))
    for prompt, out in zip(prompts, got):
        assert out == plain.greedy(config, weights, prompt, 6)
    assert llm.core.cache.used_pages() == 0 and llm.last_stats.finished == len(prompts)
