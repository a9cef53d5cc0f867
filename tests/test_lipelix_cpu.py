"""The Lipelix model in the engine (step function, cache and state manager, scheduler) on the CPU stand-in kernels
against the plain implementation; its parts alone against the plain functions; its configuration."""
import copy

import pytest
import torch

import plain_lipelix as plain
import replay_modes
from helpers import assert_close, make_runner, random_tokens
from lipelix_configs import CONFIGS, PAGE_SIZE, config_dict, make_lipelix_folder
from torch_kernels import TorchKernels

REL = 1e-4


def _runner(tmp_path, name, num_pages=64, sharpen=1.0, data=None, **kw):
    folder = make_lipelix_folder(tmp_path, name, sharpen=sharpen, data=data)
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
    assert [l.type for l in c.layers] == ["general_delta", "attention_2", "attention", "attention_2", "general_delta"]
    assert c.layers[2].mlp is None and c.layers[0].mlp.ff == 40 and c.residual_mult == 0.4 and c.embedding_scale == 0.7
    w = c.layers[1].mixer
    assert (w.heads, w.kv_heads, w.dim, w.vdim, w.window, w.keep_first, w.rot.dims, w.v_mix) == (4, 2, 12, 16, 11, 3, 8, True)
    assert c.layers[2].mixer.window is None and c.layers[0].mixer.heads == 3 and c.layers[0].mixer.dim == 8
    b = config_from_dict(config_dict("B"))
    assert b.layers[1].mixer.rot is None and not b.layers[0].mixer.v_mix and b.layers[3].mixer.keep_first == 0


def test_config_faults_are_all_reported():
    from kvcache_b200.config import ConfigError, config_from_dict
    bad = config_dict("A")
    bad["layers"][0]["mixer"].pop("dim")
    bad["layers"][1]["mixer"]["kv_heads"] = 3
    bad["layers"][2]["type"] = "convolution"
    bad["layers"][3]["mixer"]["rot"]["dims"] = 10
    bad["layers"][3]["mixer"]["vdim"] = 8            # no longer as many values as the layer it mixes with
    bad["layers"][4]["mlp"] = {"kind": "sparse"}
    del bad["norm"]
    with pytest.raises(ConfigError) as info:
        config_from_dict(bad)
    text = str(info.value)
    for piece in ("dim", "not a multiple of kv_heads", "convolution", "exceeds dim", "v_mix needs", "sparse", "norm"):
        assert piece in text, piece


def test_model_as_data(tmp_path):
    """Cache entries: pages for the attention layers (a group per window and kept count), a float32 matrix per head for
    the delta-rule layers, and in every layer the row that the token shift carries from step to step."""
    from kvcache_b200.cache import CacheManager
    from kvcache_b200.engine.loading import load_model
    model = load_model(make_lipelix_folder(tmp_path, "A"), "float32", "cpu", max_positions=64)
    entries = model.cache_entries()
    assert len(entries) == 5 and all("shift.previous" in e.state and e.state["shift.previous"].shape == (64,) for e in entries)
    assert entries[0].kv is None and entries[0].state["inner.memory"].shape == (3, 8, 8) and entries[4].state["inner.memory"].shape == (2, 20, 20)
    kv = entries[1].kv
    assert (kv.num_kv_heads, kv.head_dim, kv.v_head_dim, kv.window, kv.keep_first) == (2, 12, 16, 11, 3)
    assert (entries[2].kv.window, entries[2].kv.keep_first) == (None, 0) and (entries[3].kv.window, entries[3].kv.keep_first) == (5, 9)
    cache = CacheManager(entries, page_size=8, num_pages=8, max_slots=3, max_tokens_per_request=64, dtype="float32", device="cpu")
    assert len(cache.groups) == 3 and cache.states[0]["inner.memory"].shape == (3, 3, 8, 8)
    only_delta = load_model(make_lipelix_folder(tmp_path, "C"), "float32", "cpu", max_positions=64)
    assert all(e.kv is None for e in only_delta.cache_entries())
    roles = [b.mixer.inner.value_mix for b in model.blocks if hasattr(b.mixer.inner, "value_mix")]
    assert roles == ["source", "mix", "mix"]
    b = load_model(make_lipelix_folder(tmp_path, "B"), "float32", "cpu", max_positions=64)
    assert [blk.mixer.inner.value_mix for blk in b.blocks] == [None, "source", "mix", "mix"]


def test_decay_rank_comes_from_the_checkpoint(tmp_path):
    """The inner size of the decay's two matrices is no key a checkpoint's configuration must have: the tensors decide."""
    import json
    import os
    from kvcache_b200.engine.loading import load_model
    folder = make_lipelix_folder(tmp_path, "C")
    path = os.path.join(folder, "config.json")
    with open(path) as fh:
        data = json.load(fh)
    for layer in data["layers"]:
        layer["mixer"].pop("decay_rank")
    with open(path, "w") as fh:
        json.dump(data, fh)
    model = load_model(folder, "float32", "cpu", max_positions=32)
    assert [b.mixer.inner.w_w1.shape[0] for b in model.blocks] == [7, 2, 16]


# ---- mechanisms alone ---------------------------------------------------------------------------------------------------
def _context(batch=None, kv=None, state=None, workspace=None):
    from kvcache_b200.engine.workspace import Workspace
    from kvcache_b200.parts.base import LayerContext
    return LayerContext(batch=batch, kernels=TorchKernels(wide=True), workspace=workspace or Workspace("cpu"), kv=kv, state=state)


def _weights(specs, seed, std=0.3):
    g = torch.Generator().manual_seed(seed)
    return {name: (torch.randn(spec.shape, generator=g) * std + (1.0 if name.endswith("norm") else 0.0)).to(torch.bfloat16)
            for name, spec in specs.items()}


def _states(part, slots=3):
    return {name: torch.zeros((slots, *spec.shape), dtype=torch.float32) for name, spec in part.state_spec().items()}


def _scenario(segments, part=None, page_size=4):
    """A step's rows and, for a part that keeps pages, a cache of the part's own geometry over all of the requests' pages."""
    from helpers import paged_scenario
    from kvcache_b200.parts.base import PagedKVView
    spec = part.cache_spec() if part is not None and hasattr(part, "cache_spec") else None
    batch, kv = paged_scenario(segments, num_kv_heads=spec.num_kv_heads if spec else 1, head_dim=spec.head_dim if spec else 4,
                               page_size=page_size, dtype=torch.float32, device="cpu", fill_history=False)
    if spec is not None:
        kv = PagedKVView(spec=spec, k_pages=kv.k_pages, v_pages=torch.zeros(*kv.k_pages.shape[:-1], spec.v_head_dim),
                         block_table=kv.block_table, page_size=page_size, writes=True)
    return batch, kv


def _in_pieces(part, x, sizes, slot, states=None, with_pages=False, workspace=None, before=None):
    """The rows of one request through `part` in steps of `sizes` tokens, over one cache and one state slot."""
    T = x.shape[0]
    _, kv = _scenario([(0, T)], part) if with_pages else (None, None)
    got, at = [], 0
    for n in sizes:
        batch, _ = _scenario([(at, n)], part if with_pages else None)
        batch.seg_slot[0] = slot
        ctx = _context(batch, kv, states, workspace)
        if before is not None:
            before(ctx, at, n)
        got.append(part.forward(x[at:at + n], ctx).clone())
        at += n
    assert at == T
    return torch.cat(got)


class _Identity:
    """A mixer that hands its rows back: shows what the token shift gives the mixer it wraps."""
    def tensor_specs(self): return {}
    def init_kinds(self): return {}
    def bind(self, tensors, device): pass
    def weight_bytes(self): return 0
    def cache_spec(self): return None
    def state_spec(self): return None
    def step_planners(self, kernels): return ()
    def forward(self, x, ctx): return x.clone()


def test_token_shift_alone_carries_the_last_row_in_the_slot():
    from kvcache_b200.parts.token_shift import TokenShiftMixer
    T, W = 19, 10
    part = TokenShiftMixer(W, _Identity(), "shift", "float32")
    shift = torch.rand(W, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16)
    part.bind({"shift": shift}, torch.device("cpu"))
    x = torch.randn(T, W, generator=torch.Generator().manual_seed(2))
    want = plain.token_shift(x.double(), shift.double())
    assert torch.equal(want[0], (x[0].double() * (1 - shift.double())))            # the first token blends with zeros
    states = _states(part)
    states["shift.previous"][0].fill_(5.0)                                         # another request's row
    states["shift.previous"][1].fill_(-3.0)                                        # what an earlier request left in this slot
    assert_close(_in_pieces(part, x, [T], 1, states), want, 1e-6)
    assert bool((states["shift.previous"][0] == 5.0).all()) and torch.equal(states["shift.previous"][1], x[-1])
    states["shift.previous"][2].fill_(9.0)
    assert_close(_in_pieces(part, x, [1, 2, 1, 7, 2, 6], 2, states), want, 1e-6, "in pieces")
    # Two requests in one step, the second one continuing: each finds its own predecessor.
    batch, _ = _scenario([(0, 4), (7, 3)])
    batch.seg_slot.copy_(torch.tensor([0, 1], dtype=torch.int32))
    states = _states(part)
    states["shift.previous"][1] = x[6]
    got = part.forward(torch.cat([x[:4], x[7:10]]), _context(batch, state=states))
    assert_close(got, torch.cat([want[:4], want[7:10]]), 1e-6, "two requests")


def _double(w):
    return {k: v.double() for k, v in w.items()}


def _attention_part(kind, sizes, W, eps, scale, value_mix=None):
    from kvcache_b200.parts.attention import GQAAttention
    from kvcache_b200.parts.position import RotaryHalf
    rope = None if sizes.get("dims") is None else RotaryHalf(sizes["dims"], sizes.get("base", 777.0), 128)
    common = dict(qkv_bias=False, out_bias=False, position=rope, prefix="m.", dtype="float32", scale=scale, value_dim=sizes["vdim"],
                  qk_norm_eps=eps, names=("q", "k", "v", "o"), value_mix=value_mix)
    if kind == "attention":
        return GQAAttention(W, sizes["heads"], sizes["kv_heads"], sizes["dim"], window=None, qk_norm_scope="all", sink="learned", **common)
    return GQAAttention(W, sizes["heads"], sizes["kv_heads"], sizes["dim"], window=sizes["window"], keep_first=sizes["keep"],
                        qk_norm_weight=False, qk_norm_after_rotation=True, sink=0.0, **common)


def _mixer_dict(sizes, scale, v_mix=False):
    m = dict(heads=sizes["heads"], kv_heads=sizes["kv_heads"], dim=sizes["dim"], vdim=sizes["vdim"], scale=scale, v_mix=v_mix)
    if sizes.get("dims") is not None:
        m["rot"] = {"base": sizes.get("base", 777.0), "dims": sizes["dims"]}
    if sizes.get("window") is not None:
        m["mask"] = {"size": sizes["window"], "keep_first": sizes["keep"]}
    return m


@pytest.mark.parametrize("sizes", [dict(heads=4, kv_heads=2, dim=16, vdim=24, dims=8), dict(heads=3, kv_heads=3, dim=6, vdim=2, dims=6),
                                   dict(heads=2, kv_heads=1, dim=8, vdim=8, dims=None)])
def test_sink_attention_part_alone(sizes):
    """Norms over the whole query and key projections (not per head), rotation of part of a head, a learned sink per
    head that takes a good share of the weight: whole, cut in two, and token by token."""
    T, W, eps, scale = 27, 40, 1e-5, 2.5
    part = _attention_part("attention", sizes, W, eps, scale)
    w = _weights(part.tensor_specs(), 3)
    w["m.sink"] = torch.linspace(-1.0, 3.0, sizes["heads"]).to(torch.bfloat16)
    part.bind(w, torch.device("cpu"))
    x = torch.randn(T, W, generator=torch.Generator().manual_seed(4))
    m = _mixer_dict(sizes, scale)
    want, _ = plain.attention(x.double(), _double(w), "m.", m, eps, None)
    # The sink shows: without it (a sink far below every score) the result is another one.
    no_sink = dict(_double(w), **{"m.sink": torch.full((sizes["heads"],), -80.0, dtype=torch.float64)})
    assert (plain.attention(x.double(), no_sink, "m.", m, eps, None)[0] - want).abs().max() > 0.05 * want.abs().max()
    if sizes["heads"] > 1:      # and so does a norm taken head by head instead of over the whole row
        per_head = plain.linear(x.double(), w["m.q"].double()).view(T, sizes["heads"], sizes["dim"])
        assert not torch.allclose(plain.unit(per_head, eps).reshape(T, -1), plain.unit(per_head.reshape(T, -1), eps), atol=1e-3)
    assert_close(_in_pieces(part, x, [T], 0, with_pages=True), want, 1e-5)
    assert_close(_in_pieces(part, x, [11, T - 11], 0, with_pages=True), want, 1e-5, "cut in two")
    assert_close(_in_pieces(part, x, [1] * T, 0, with_pages=True), want, 1e-5, "token by token")


@pytest.mark.parametrize("sizes", [dict(heads=4, kv_heads=2, dim=16, vdim=24, dims=8, window=7, keep=3),
                                   dict(heads=3, kv_heads=3, dim=6, vdim=2, dims=6, window=1, keep=1),
                                   dict(heads=2, kv_heads=1, dim=8, vdim=8, dims=None, window=4, keep=9),
                                   dict(heads=2, kv_heads=2, dim=12, vdim=8, dims=4, window=6, keep=0)])
def test_window_attention_with_kept_first_tokens_alone(sizes):
    """Rotation first, then each head divided by its root mean square; the window's edge and the edge of the kept first
    tokens with sharp scores (one key more or less on either edge changes the result); one added to the denominator."""
    T, W, eps, scale = 31, 40, 1e-5, 3.0
    part = _attention_part("attention_2", sizes, W, eps, scale)
    w = _weights(part.tensor_specs(), 5)
    part.bind(w, torch.device("cpu"))
    x = torch.randn(T, W, generator=torch.Generator().manual_seed(6))
    m = _mixer_dict(sizes, scale)
    wd = _double(w)
    want, _ = plain.attention_2(x.double(), wd, "m.", m, eps, None)
    for key, delta in (("size", 1), ("size", -1), ("keep_first", 1), ("keep_first", -1)):
        if m["mask"][key] + delta < (1 if key == "size" else 0):
            continue
        other = dict(m, mask=dict(m["mask"], **{key: m["mask"][key] + delta}))
        assert (plain.attention_2(x.double(), wd, "m.", other, eps, None)[0] - want).abs().max() > 0.01 * want.abs().max(), (key, delta)
    # One in the denominator: the weights of a row do not sum to one.
    q = plain.unit(plain.rotate(plain.linear(x.double(), wd["m.q"]).view(T, sizes["heads"], sizes["dim"]), m.get("rot")), eps)
    assert float((q * q).mean(dim=-1).min()) > 0.99
    assert_close(_in_pieces(part, x, [T], 0, with_pages=True), want, 1e-5)
    assert_close(_in_pieces(part, x, [2, 9, 1, 5, T - 17], 0, with_pages=True), want, 1e-5, "in pieces")
    assert_close(_in_pieces(part, x, [1] * T, 0, with_pages=True), want, 1e-5, "token by token")


def test_one_kept_key_far_back_takes_all_the_weight():
    """A kept first token whose key is made to match every later query stands out among the window's keys at any distance;
    the first token after the kept ones, made as strong, must not be seen once it has left the window."""
    from kvcache_b200.parts.attention import GQAAttention
    T, W, keep, window = 90, 16, 2, 5
    part = GQAAttention(W, 1, 1, 16, qkv_bias=False, out_bias=False, position=None, window=window, keep_first=keep, prefix="m.",
                        dtype="float32", scale=4.0, value_dim=16, qk_norm_eps=1e-6, names=("q", "k", "v", "o"),
                        qk_norm_weight=False, qk_norm_after_rotation=True, sink=0.0)
    eye = torch.eye(W)
    swap = eye.clone()
    swap[[0, 3]] = swap[[3, 0]]             # a key's channel 0 is the row's channel 3
    w = {"m.q": eye, "m.k": swap, "m.v": eye, "m.o": eye}
    part.bind(w, torch.device("cpu"))
    x = torch.randn(T, W, generator=torch.Generator().manual_seed(1)) * 0.05
    x[:, 0] += 1.0                         # every query points along channel 0; ordinary keys do not
    x[1, 3], x[keep, 3] = 30.0, 30.0        # key 1 (kept) and key `keep` (the first one not kept) point there sharply
    x[1, 1], x[keep, 2] = 7.0, 7.0          # and their values say which of them was read
    got = _in_pieces(part, x, [40, 3, 1, 1, 1, 44], 0, with_pages=True)
    m = dict(heads=1, kv_heads=1, dim=16, vdim=16, scale=4.0, mask={"size": window, "keep_first": keep})
    want, _ = plain.attention_2(x.double(), _double(w), "m.", m, 1e-6, None)
    assert_close(got, want, 1e-5)
    late = got[keep + window + 3:]
    assert float(late[:, 1].min()) > 6.0 and float(late[:, 2].abs().max()) < 0.5
    assert float(got[keep + 1:keep + window, 2].min()) > 2.0          # while it is in the window, the other strong key is read too


def test_value_mixing_blends_with_the_source_layers_values_of_the_same_token():
    """A source layer leaves its values of the step's tokens; a mixing layer blends its own with them before they are
    cached, so that later steps read mixed values from the pages."""
    T, W, eps = 21, 32, 1e-6
    a = dict(heads=2, kv_heads=2, dim=8, vdim=12, dims=4, window=6, keep=2)
    b = dict(heads=4, kv_heads=1, dim=6, vdim=24, dims=None)
    source = _attention_part("attention_2", a, W, eps, 1.5, value_mix="source")
    mixing = _attention_part("attention", b, W, eps, 1.5, value_mix="mix")
    assert "m.vmix" in mixing.tensor_specs() and source.tensor_specs()["m.vmix"].optional
    ws_, wm = _weights(source.tensor_specs(), 7), _weights(mixing.tensor_specs(), 8)
    ws_.pop("m.vmix", None)
    wm["m.vmix"] = torch.tensor(0.7).to(torch.bfloat16)
    wm["m.sink"] = torch.zeros(4).to(torch.bfloat16)
    source.bind(ws_, torch.device("cpu"))
    mixing.bind(wm, torch.device("cpu"))
    x1 = torch.randn(T, W, generator=torch.Generator().manual_seed(9))
    x2 = torch.randn(T, W, generator=torch.Generator().manual_seed(10))
    want1, v_first = plain.attention_2(x1.double(), _double(ws_), "m.", _mixer_dict(a, 1.5, True), eps, None)
    want2, v2 = plain.attention(x2.double(), _double(wm), "m.", _mixer_dict(b, 1.5, True), eps, v_first)
    unmixed, _ = plain.attention(x2.double(), _double(wm), "m.", _mixer_dict(b, 1.5, False), eps, None)
    assert (unmixed - want2).abs().max() > 0.05 * want2.abs().max()
    from kvcache_b200.engine.workspace import Workspace
    for sizes in ([T], [3, 1, 2, 15]):
        workspace = Workspace("cpu")
        _, kv1 = _scenario([(0, T)], source)
        _, kv2 = _scenario([(0, T)], mixing)
        got1, got2, at = [], [], 0
        for n in sizes:
            batch, _ = _scenario([(at, n)], source)
            got1.append(source.forward(x1[at:at + n], _context(batch, kv1, None, workspace)).clone())
            got2.append(mixing.forward(x2[at:at + n], _context(batch, kv2, None, workspace)).clone())
            at += n
        assert_close(torch.cat(got1), want1, 1e-5, f"source {sizes}")
        assert_close(torch.cat(got2), want2, 1e-5, f"mixing {sizes}")


@pytest.mark.parametrize("sizes", [dict(heads=3, dim=8, rank=6), dict(heads=1, dim=40, rank=1), dict(heads=2, dim=33, rank=5)])
def test_delta_rule_part_alone(sizes):
    """Whole, and cut into pieces that carry the state in a slot, against the plain recurrence; a state left in another
    slot does not leak; removal and decay biases wide enough that both the strong and the weak ends occur."""
    from kvcache_b200.parts.recurrent import DeltaRuleMixer
    T, W, eps = 23, 48, 1e-5
    part = DeltaRuleMixer(W, sizes["heads"], sizes["dim"], sizes["rank"], eps=eps, prefix="m.", dtype="float32")
    w = _weights(part.tensor_specs(), 5)
    g = torch.Generator().manual_seed(6)
    n = sizes["heads"] * sizes["dim"]
    w["m.a.b"], w["m.w0"] = (torch.randn(n, generator=g) * 3).to(torch.bfloat16), (torch.randn(n, generator=g) * 3).to(torch.bfloat16)
    part.bind(w, torch.device("cpu"))
    x = torch.randn(T, W, generator=torch.Generator().manual_seed(7))
    want = plain.general_delta(x.double(), _double(w), "m.", dict(heads=sizes["heads"], dim=sizes["dim"]), eps)
    states = _states(part)
    states["memory"][0].fill_(7.0)                                    # another request's state
    assert_close(_in_pieces(part, x, [T], 1, states), want, 1e-5)
    assert bool((states["memory"][0] == 7.0).all()) and float(states["memory"][1].abs().max()) > 0
    assert_close(_in_pieces(part, x, [1, 2, 9, 1, 10], 2, _states(part)), want, 1e-5, "in pieces")
    assert_close(_in_pieces(part, x, [1] * T, 0, _states(part)), want, 1e-5, "token by token")


def test_delta_rule_reads_the_old_state_in_both_terms():
    """With removal rate 1 and no decay, writing key k twice replaces the first value: what u^T S reads is the state before
    this token's own k v^T is added (reading it after would remove part of the new value as well)."""
    D = 4
    k = torch.zeros(3, 1, D, dtype=torch.float64)
    k[:, 0, 1] = 1.0
    v = torch.tensor([[1.0, 2.0, 3.0, 4.0], [5.0, 6.0, 7.0, 8.0], [-1.0, 0.0, 1.0, 0.0]], dtype=torch.float64)[:, None, :]
    ones = torch.ones(3, 1, D, dtype=torch.float64)
    o, S = plain.delta_rule_scan(k.clone(), k, v, ones, ones)
    assert torch.allclose(o[:, 0], v[:, 0], atol=1e-5) and torch.allclose(S[0, 1], v[2, 0], atol=1e-5)
    from kvcache_b200.parts.base import StepBatch  # noqa: F401  (the engine's scan on the same rows)
    kernels = TorchKernels(wide=True)
    proj = torch.cat([k.reshape(3, D), k.reshape(3, D), v.reshape(3, D), torch.full((3, D), 30.0, dtype=torch.float64)], dim=1).float()
    z = torch.full((3, D), -40.0)                 # sigmoid ~ 0: the decay is 1
    batch, _ = _scenario([(0, 3)])
    memory, out = torch.zeros(1, 1, D, D), torch.zeros(3, D)
    from kvcache_b200.engine.workspace import Workspace
    kernels.delta_rule_scan(proj, (0, D, 2 * D, 3 * D), z, plain.DECAY_RATE, plain.UNIT_KEY_EPS, batch, memory, out, 1, D, Workspace("cpu"))
    assert_close(out, v.reshape(3, D), 1e-5)


def test_relu_squared_feed_forward_alone():
    from kvcache_b200.parts.feedforward import ReluSquaredMLP
    part = ReluSquaredMLP(24, 56, prefix="f.", dtype="float32")
    w = _weights(part.tensor_specs(), 2)
    part.bind(w, torch.device("cpu"))
    x = torch.randn(9, 24, generator=torch.Generator().manual_seed(3))
    want = plain.feed_forward(x.double(), _double(w), "f.", {"kind": "dense", "ff": 56})
    assert_close(part.forward(x, _context()), want, 1e-5)
    assert float((plain.linear(x.double(), w["f.up"].double()) < 0).double().mean()) > 0.2      # the relu cuts


def test_gated_normalised_add_alone():
    """h += m * unit(delta * sigmoid(W a + b)) * w: the gate reads the rows the norm before the sublayer made and acts
    before the result's norm; the multiplier sits in the norm's weight."""
    from kvcache_b200.parts.base import NormedDelta
    from kvcache_b200.parts.block import ResidualGate
    from kvcache_b200.parts.norm import RMSNorm
    T, W, eps, mult = 7, 24, 1e-5, 0.3
    g = torch.Generator().manual_seed(4)
    gate, post, pre = ResidualGate(W, "rg", "rg.b", "float32"), RMSNorm(W, eps, "post", gain=mult), RMSNorm(W, eps, "pre")
    w = {"rg": (torch.randn(W, W, generator=g) * 0.5).to(torch.bfloat16), "rg.b": torch.randn(W, generator=g).to(torch.bfloat16),
         "post": (1 + 0.3 * torch.randn(W, generator=g)).to(torch.bfloat16), "pre": (1 + 0.3 * torch.randn(W, generator=g)).to(torch.bfloat16)}
    for part in (gate, post, pre):
        part.bind(w, torch.device("cpu"))
    h, a, delta = (torch.randn(T, W, generator=g) for _ in range(3))
    wd = _double(w)
    want_h = h.double() + mult * plain.unit(delta.double() * plain.residual_gate(a.double(), wd["rg"], wd["rg.b"]), eps) * wd["post"]
    ctx = _context()
    out = torch.zeros(T, W)
    pre.add_norm(h, NormedDelta(delta, post, gate.forward(a, ctx, "gate")), out, ctx)
    assert_close(h, want_h, 1e-5, "the residual stream")
    assert_close(out, plain.unit(want_h, eps) * wd["pre"], 1e-5, "the rows the next sublayer reads")


def test_residual_stream_after_every_layer(tmp_path):
    """Layer by layer: a model cut after k layers (its final norm and head replaced by the identity) gives the plain
    implementation's residual stream after layer k, up to the norm that the cut model still applies."""
    for name in ("A", "B"):
        folder = make_lipelix_folder(tmp_path, name)
        config, weights = plain.read_folder(folder)
        tokens = random_tokens(config["vocab"], 19, 3)
        streams = plain.residual_streams(config, weights, tokens)[1:]
        from kvcache_b200.cache import CacheManager
        from kvcache_b200.engine.loading import load_model
        from kvcache_b200.engine.runner import ModelRunner, StepEntry
        for k in range(1, len(streams) + 1):
            model = load_model(folder, "float32", "cpu", max_positions=64)
            model.schedule = model.schedule[:k]
            model._writers = {c.cache: c.layer for c in model.schedule}
            model.final_norm.weight = torch.ones(model.width)
            model.final_norm.eps = 0.0
            model.head = torch.eye(model.width)
            model.vocab_size = model.width
            cache = CacheManager(model.cache_entries(), page_size=8, num_pages=16, max_slots=1, max_tokens_per_request=64, dtype="float32", device="cpu")
            runner = ModelRunner(model, cache, TorchKernels(wide=True), max_tokens_per_step=64)
            got = runner.step([StepEntry(cache.admit(), tokens, list(range(len(tokens))))]).double()
            want = streams[k - 1]
            want = want / torch.sqrt((want * want).mean(dim=-1, keepdim=True))
            assert_close(got, want, 1e-5, f"{name} after layer {k}")


# ---- the model in the engine ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt_and_its_first_tokens(tmp_path, name):
    runner, config, weights = _runner(tmp_path, name)
    tokens = random_tokens(config["vocab"], 75, 1)
    want = plain.logits_of(config, weights, tokens)
    assert_close(replay_modes.whole(runner, tokens), want, REL)
    assert runner.cache.used_pages() == 0
    for n in (1, 2, 3):                 # a sequence's first tokens alone: the shift blends with zeros, the states are empty
        assert_close(replay_modes.whole(runner, tokens[:n]), want[:n], REL, f"first {n}")


@pytest.mark.parametrize("name", list(CONFIGS))
def test_prefill_against_token_by_token_decoding(tmp_path, name):
    runner, config, weights = _runner(tmp_path, name)
    tokens = random_tokens(config["vocab"], 70, 2)
    want = plain.logits_of(config, weights, tokens)
    assert_close(replay_modes.last_32_one_by_one(runner, tokens), want[-33:], REL)
    assert_close(replay_modes.portions(runner, tokens, [1] * 70), want, REL, "every token alone")


@pytest.mark.parametrize("name", list(CONFIGS))
def test_portions_down_to_two_tokens(tmp_path, name):
    runner, config, weights = _runner(tmp_path, name)
    tokens = random_tokens(config["vocab"], 101, 3)
    want = plain.logits_of(config, weights, tokens)
    assert_close(replay_modes.portions(runner, tokens, [2, 17, 3, 31, 2, 16, 8, 22]), want, REL)
    assert_close(replay_modes.portions(runner, tokens, [40, 2, 2, 5, 52]), want, REL)


@pytest.mark.parametrize("name", list(CONFIGS))
def test_mixed_batches_with_pages_and_slots_used_again(tmp_path, name):
    """Unequal requests beside one another against each alone; a and b end and d and e take their slots, whose states
    (delta-rule matrices, the token shift's previous rows) must start from nothing, and their pages."""
    page = PAGE_SIZE[name]
    runner, config, weights = _runner(tmp_path, name, num_pages=replay_modes.mixed_pool_tokens() // page)
    seqs = {k: random_tokens(config["vocab"], n, 10 + i) for i, (k, n) in enumerate(replay_modes.MIXED_LENGTHS)}
    got = replay_modes.mixed(runner, seqs)
    for k, tokens in seqs.items():
        assert_close(got[k], plain.logits_of(config, weights, tokens), REL, k)


@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_sharp_attention_at_the_edges_in_prompts_and_decoding(tmp_path, name):
    """With the score scale multiplied, the softmax of most heads rests on single keys: a window or a run of kept tokens
    one too wide or too narrow, or a key lost at a page border or at the start of a portion, changes the logits by far
    more than the tolerance."""
    runner, config, weights = _runner(tmp_path, name, sharpen=25.0, max_tokens_per_step=256, max_tokens_per_request=256)
    tokens = random_tokens(config["vocab"], 150, 5)
    want = plain.logits_of(config, weights, tokens)
    for key, delta in (("size", -1), ("size", 1), ("keep_first", -1), ("keep_first", 1)):
        other = copy.deepcopy(config)
        changed = False
        for layer in other["layers"]:
            if layer["type"] == "attention_2" and layer["mixer"]["mask"][key] + delta >= (1 if key == "size" else 0):
                layer["mixer"]["mask"][key] += delta
                changed = True
        if changed:
            assert (plain.logits_of(other, weights, tokens) - want).abs().max() > 0.02 * want.abs().max(), (key, delta)
    assert_close(replay_modes.portions(runner, tokens, [7, 2, 57, 64, 3, 17]), want, 1e-3)
    assert_close(replay_modes.last_32_one_by_one(runner, tokens), want[-33:], 1e-3)
    assert_close(replay_modes.portions(runner, tokens, [100] + [1] * 50), want, 1e-3, "the window passes over decoded tokens")


def test_long_decoding_keeps_the_states_in_range(tmp_path):
    runner, config, weights = _runner(tmp_path, "A", max_tokens_per_step=512, max_tokens_per_request=512)
    tokens = random_tokens(config["vocab"], 300, 6)
    got = replay_modes.portions(runner, tokens, [20] + [1] * 280)
    assert_close(got, plain.logits_of(config, weights, tokens), REL)


def test_pages_behind_the_window_are_given_back_but_the_kept_first_ones_stay(tmp_path):
    """A window layer's pages pass out of the window as a request grows and go back to the pool, except those that hold
    kept first tokens; a pool too small for the whole request is enough."""
    data = config_dict("D")
    data["layers"] = data["layers"][:2]                     # windows of 37 (6 kept) and 3 (7 kept); pages of 4
    runner, config, weights = _runner(tmp_path, "D", num_pages=2 * 16, data=data, max_tokens_per_step=256, max_tokens_per_request=256)
    tokens = random_tokens(config["vocab"], 200, 7)
    slot = runner.cache.admit()
    from kvcache_b200.engine.runner import StepEntry
    got = [runner.step([StepEntry(slot, tokens[:90], list(range(90)))]).clone()]
    for i in range(90, 200):
        got.append(runner.step([StepEntry(slot, tokens[i:i + 1], [0])]).clone())
    assert runner.cache.used_pages() <= (37 + 4 + 8) // 4 + 2 + (3 + 4 + 8) // 4 + 2 + 2
    runner.cache.release(slot)
    assert runner.cache.used_pages() == 0
    assert_close(torch.cat(got), plain.logits_of(config, weights, tokens), REL)


# ---- generation through the entry point and the scheduler -------------------------------------------------------------
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_greedy_generation_matches_plain(tmp_path, name):
    from kvcache_b200 import LLM, SamplingParams
    folder = make_lipelix_folder(tmp_path, name)
    config, weights = plain.read_folder(folder)
    prompts = [random_tokens(config["vocab"], n, 40 + n) for n in (1, 9, 24, 40)]
    llm = LLM(folder, kernels=TorchKernels(), dtype="float32", device="cpu", page_size=PAGE_SIZE[name], num_pages=40, max_running=3,
              max_tokens_per_step=48, chunk_size=16, use_graphs=False)
    got = llm.generate(prompts, SamplingParams(max_new_tokens=6, ignore_eos=True))
    for prompt, out in zip(prompts, got):
        assert out == plain.greedy_generate(config, weights, prompt, 6)
    assert llm.core.cache.used_pages() == 0 and llm.last_stats.finished == len(prompts)
