"""The Lipelix model through the engine on the GPU, in float32 and bfloat16, against the plain implementation, and every
CUDA operator it brought alone against the plain PyTorch statement of the same operator (tests/torch_kernels.py)."""
import copy
import dataclasses
import json
import os
import subprocess
import sys

import numpy as np

import pytest
import torch

import plain_lipelix as plain
import replay_modes
from helpers import assert_close, batch_to, clone_kv, make_runner, paged_scenario, random_tokens
from lipelix_configs import CONFIGS, PAGE_SIZE, config_dict, make_lipelix_folder
from torch_kernels import TorchKernels

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REL = {"float32": 1e-4, "bfloat16": 3e-2}
TOL = {torch.float32: 2e-5, torch.bfloat16: 2e-2}


def _spread(config, weights, tokens, want):
    """What rounding alone does to each position's logits: the plain implementation with every product's rows and
    results rounded to bfloat16, against itself without."""
    with plain.rounding(torch.bfloat16):
        return (plain.logits_of(config, weights, tokens) - want).abs().max(dim=1).values


def assert_model_close(got, want, dtype, what="", spread=None, rel=None):
    """float32: within `rel` of the largest logit.  bfloat16: a layer of this design divides what a sublayer returns by
    its root mean square, so a position where a sublayer's sums nearly cancel magnifies rounding however it is computed.
    The errors are therefore held, as a distribution, to 4 times what rounding alone does in the plain implementation
    (`spread`: its per-position errors over the whole sequence): the k-th largest error against the k-th largest of the
    spread (floor: 1 % of the largest logit) except for the largest 2 % of them (at least one), the median position
    within 2 %, and no position beyond 30 % - a lost key, state or token moves many positions by as much as the logits
    themselves."""
    if dtype == "float32":
        return assert_close(got, want, rel or REL[dtype], what)
    got, want = got.detach().double().cpu(), want.double()
    assert got.shape == want.shape and torch.isfinite(got).all(), what
    scale = float(want.abs().max())
    floor = 0.01 * scale
    err = (got - want).abs().max(dim=1).values
    assert float(err.max()) <= 0.3 * scale, f"{what}: error {float(err.max()):.3e} of {scale:.3e}"
    if len(err) < 16:
        limit = max(4.0 * float(spread.max()), 4.0 * floor)
        assert float(err.max()) <= limit, f"{what}: error {float(err.max()):.3e}, spread {float(spread.max()):.3e}"
        return
    e, sp = torch.sort(err, descending=True).values, torch.sort(spread, descending=True).values
    like = sp[(torch.arange(len(e)) * len(sp) // len(e))]
    over = e > 4.0 * torch.clamp(like, min=floor)
    over[:max(1, len(e) // 50)] = False
    assert not bool(over.any()), f"{what}: the {int(over.nonzero()[0])}-th largest error {float(e[over][0]):.3e} against {float(like[over][0]):.3e}"
    assert float(err.median()) <= 0.02 * scale, f"{what}: median error {float(err.median()):.3e} of {scale:.3e}"


@pytest.fixture(scope="module")
def kernels():
    from kvcache_b200.kernels.api import CudaKernels
    return CudaKernels(DEV)


def _rand(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


def _segments_batch(segments, slots):
    batch, _ = paged_scenario(segments, num_kv_heads=1, head_dim=4, page_size=4, dtype=torch.float32, device="cpu", fill_history=False)
    batch.seg_slot.copy_(torch.tensor(slots, dtype=torch.int32))
    return batch


# ---- operators alone ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W", [10, 64, 200, 1024])
def test_token_shift(kernels, dtype, W):
    """Prompts from position 0 (blend with zeros whatever the slot holds), a portion and single tokens that continue (blend
    with the slot's row), the slots' rows afterwards, other slots untouched."""
    segments, slots = [(0, 19), (50, 1), (7, 6), (0, 1)], [2, 0, 3, 5]
    batch = _segments_batch(segments, slots)
    T = batch.num_tokens
    x, weight = _rand(T, W, dtype=dtype, seed=1), torch.rand(W, generator=torch.Generator().manual_seed(2))
    previous = _rand(6, W, seed=3)
    ref_prev, ref = previous.clone(), torch.zeros(T, W, dtype=dtype)
    TorchKernels(wide=True).token_shift(x, weight, ref_prev, batch, ref)
    got_prev, got = previous.clone().to(DEV), torch.zeros(T, W, dtype=dtype, device=DEV)
    kernels.token_shift(x.to(DEV), weight.to(DEV), got_prev, batch_to(batch, DEV), got)
    assert_close(got, ref, TOL[dtype])
    assert torch.equal(got_prev.cpu(), ref_prev) and torch.equal(got_prev[1].cpu(), previous[1]) and torch.equal(got_prev[4].cpu(), previous[4])
    assert torch.equal(got_prev[2].cpu(), x[18].float())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kind", ["tanh", "relu2"])
def test_plain_activations(kernels, dtype, kind):
    x = _rand(37, 129, dtype=dtype, seed=4, scale=2.0)
    ref, got = x.clone(), x.clone().to(DEV)
    TorchKernels(wide=True).activation_(ref, kind)
    kernels.activation_(got, kind)
    assert_close(got, ref, TOL[dtype])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_with_a_scale(kernels, dtype):
    table = _rand(50, 72, dtype=dtype, seed=5)
    ids = torch.tensor([3, 49, 0, 17, 3], dtype=torch.int32)
    out = torch.zeros(5, 72, device=DEV)
    kernels.embed(table.to(DEV), ids.to(DEV), out, scale=0.37)
    assert_close(out, table[ids.long()].float() * 0.37, 1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W", [24, 200, 896])
def test_gated_normalised_add(kernels, dtype, W):
    """h += rmsnorm(delta * sigmoid(gate); w_post); out = rmsnorm(h; w_pre): with and without the norm of the delta, with
    rows gathered (the final norm's form)."""
    T = 13
    h, delta, gate = _rand(T, W, seed=6), _rand(T, W, dtype=dtype, seed=7), _rand(T, W, dtype=dtype, seed=8, scale=2.0)
    w_post, w_pre = 1 + 0.3 * _rand(W, seed=9), 1 + 0.3 * _rand(W, seed=10)
    for post in (w_post, None):
        ref_h, ref = h.clone(), torch.zeros(T, W, dtype=dtype)
        TorchKernels(wide=True).norm_add_rmsnorm(ref_h, delta, post, 1e-5, w_pre, 1e-6, ref, delta_gate=gate)
        got_h, got = h.clone().to(DEV), torch.zeros(T, W, dtype=dtype, device=DEV)
        kernels.norm_add_rmsnorm(got_h, delta.to(DEV), None if post is None else post.to(DEV), 1e-5, w_pre.to(DEV), 1e-6, got, delta_gate=gate.to(DEV))
        assert_close(got_h, ref_h, 2e-6 if dtype == torch.float32 else 1e-5, "the residual stream")
        assert_close(got, ref, TOL[dtype])
    rows = torch.tensor([12, 0, 5], dtype=torch.int32)
    ref_h, ref = h.clone(), torch.zeros(3, W, dtype=dtype)
    TorchKernels(wide=True).norm_add_rmsnorm(ref_h, delta, w_post, 1e-5, w_pre, 1e-6, ref, rows=rows, delta_gate=gate)
    got_h, got = h.clone().to(DEV), torch.zeros(3, W, dtype=dtype, device=DEV)
    kernels.norm_add_rmsnorm(got_h, delta.to(DEV), w_post.to(DEV), 1e-5, w_pre.to(DEV), 1e-6, got, rows=rows.to(DEV), delta_gate=gate.to(DEV))
    assert_close(got, ref, TOL[dtype], "gathered rows")
    assert torch.equal(got_h.cpu(), h)


def _kv_scenario(segments, Hkv, D, Dv, page, dtype, window=None, keep_first=0, seed=2, fill=True):
    from kvcache_b200.parts.base import PagedKVSpec, PagedKVView
    batch, kv = paged_scenario(segments, num_kv_heads=Hkv, head_dim=D, page_size=page, dtype=dtype, device="cpu", seed=seed, window=window,
                               fill_history=fill)
    values = _rand(*kv.k_pages.shape[:-1], Dv, dtype=dtype, seed=seed + 1) if fill else torch.zeros(*kv.k_pages.shape[:-1], Dv, dtype=dtype)
    return batch, PagedKVView(spec=PagedKVSpec(Hkv, D, window, None if Dv == D else Dv, keep_first), k_pages=kv.k_pages, v_pages=values,
                              block_table=kv.block_table, page_size=page, writes=True)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("Hq,Hkv,D,Dv,rot", [(4, 2, 16, 24, 8), (3, 3, 6, 2, 6), (6, 3, 80, 160, 40), (5, 1, 40, 40, 0), (2, 2, 128, 64, 128), (1, 1, 64, 64, 32)])
def test_append_with_whole_row_norms_norms_after_rotation_and_mixed_values(kernels, dtype, Hq, Hkv, D, Dv, rot):
    """The root mean square over a row's whole query (key) projection with weights of that size, before the rotation;
    per head without weights, after it; the values kept for later layers, and blended with kept ones before the cache."""
    segments = [(0, 5), (37, 1), (14, 20)]
    batch, kv = _kv_scenario(segments, Hkv, D, Dv, 8, dtype, seed=3)
    T = batch.num_tokens
    qkv = _rand(T, (Hq + Hkv) * D + Hkv * Dv + 3, dtype=dtype, seed=7, scale=2.0)
    qw, kw = 1 + _rand(Hq * D, seed=8, scale=0.3), 1 + _rand(Hkv * D, seed=9, scale=0.3)
    cos = sin = None
    if rot:
        ang = torch.arange(64, dtype=torch.float64)[:, None] * torch.logspace(0, -3, rot // 2, dtype=torch.float64)[None, :]
        cos, sin = torch.cos(ang).float(), torch.sin(ang).float()
    dev = lambda t: None if t is None else t.to(DEV)
    kept_source = _rand(T, Hkv * Dv, dtype=dtype, seed=10)
    lam = torch.tensor([0.37])
    cases = [dict(q_norm=qw, k_norm=kw, norm_eps=1e-5, norm_scope="all"), dict(norm_eps=1e-5, norm_after_rotation=True),
             dict(q_norm=qw, k_norm=kw, norm_eps=1e-5, norm_scope="all", value_mix="keep"), dict(norm_eps=1e-5, norm_after_rotation=True, value_mix="mix"),
             dict(value_mix="mix")]
    for case in cases:
        mix = case.pop("value_mix", None)
        ref_kept = torch.zeros(T, Hkv * Dv, dtype=dtype) if mix == "keep" else kept_source.clone()
        got_kept = ref_kept.clone().to(DEV)
        ref_kv, ref_q = clone_kv(kv), torch.zeros(T, Hq * D, dtype=dtype)
        got_kv, got_q = clone_kv(kv, DEV), torch.zeros(T, Hq * D, dtype=dtype, device=DEV)
        ref_mix = None if mix is None else (ref_kept, None if mix == "keep" else lam)
        got_mix = None if mix is None else (got_kept, None if mix == "keep" else lam.to(DEV))
        TorchKernels(wide=True).qkv_rope_append(qkv, None, cos, sin, batch, ref_kv, ref_q, Hq, value_mix=ref_mix, **case)
        kernels.qkv_rope_append(qkv.to(DEV), None, dev(cos), dev(sin), batch_to(batch, DEV), got_kv, got_q, Hq, value_mix=got_mix,
                                **{k: dev(v) if isinstance(v, torch.Tensor) else v for k, v in case.items()})
        kernels.check_errors()
        what = f"{sorted(case)} {mix}"
        assert_close(got_q, ref_q, TOL[dtype], "queries " + what)
        assert_close(got_kv.k_pages, ref_kv.k_pages, TOL[dtype], "key pages " + what)
        assert_close(got_kv.v_pages, ref_kv.v_pages, TOL[dtype], "value pages " + what)
        if mix == "keep":
            assert torch.equal(got_kept.cpu(), qkv[:, (Hq + Hkv) * D:(Hq + Hkv) * D + Hkv * Dv].contiguous())
        untouched = ref_kv.v_pages == kv.v_pages
        assert torch.equal(got_kv.v_pages.cpu()[untouched], kv.v_pages[untouched])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("Hq,Hkv,D,Dv,window,keep", [(4, 2, 16, 24, 11, 3), (3, 3, 6, 2, None, 0), (6, 3, 80, 160, 70, 13), (5, 1, 40, 72, 16, 0),
                                                      (2, 1, 64, 32, 1, 1), (4, 4, 32, 32, 5, 20), (8, 2, 64, 64, None, 0), (2, 2, 128, 128, 33, 9)])
def test_attention_with_a_sink_and_kept_first_keys(kernels, dtype, Hq, Hkv, D, Dv, window, keep):
    """Prompts from position 0, portions that continue, single decoded tokens; a sink logit per head (large, small and
    zero), none with kept keys alone; kept keys inside the window, just behind it and far behind it."""
    from kvcache_b200.engine.workspace import Workspace
    batch, kv = _kv_scenario([(0, 45), (130, 1), (30, 20), (16, 1), (0, 1)], Hkv, D, Dv, 8, dtype, window, keep)
    T = batch.num_tokens
    q = _rand(T, Hq * D, dtype=dtype, seed=5, scale=0.5)
    sink = _rand(Hq, seed=6, scale=3.0)
    sink[0] = 0.0
    for s in (sink, torch.zeros(Hq)) + ((None,) if window and keep else ()):
        ref, got = torch.zeros(T, Hq * Dv, dtype=dtype), torch.zeros(T, Hq * Dv, dtype=dtype, device=DEV)
        TorchKernels(wide=True).paged_attention(q, batch, kv, ref, Hq, 0.4, sink=s)
        kernels.paged_attention(q.to(DEV), batch_to(batch, DEV), clone_kv(kv, DEV), got, Hq, 0.4, Workspace(DEV), sink=None if s is None else s.to(DEV))
        kernels.check_errors()
        assert_close(got, ref, TOL[dtype])


@pytest.mark.parametrize("path", ["default", "mma prefill, scratch decode", "tensor memory from 128 rows, tiles shared out"])
@pytest.mark.parametrize("Hq,Hkv,D,window,keep", [(4, 2, 64, None, 0), (4, 2, 64, 200, 5), (2, 1, 64, 100, 70), (6, 2, 64, 1000, 300),
                                                   (2, 2, 64, 64, 64), (3, 1, 128, 300, 129), (4, 4, 128, None, 0), (2, 1, 32, 150, 40),
                                                   (2, 2, 48, 70, 3), (4, 2, 64, 1, 1), (2, 2, 64, 700, 0), (4, 2, 80, 130, 65),
                                                   (6, 1, 96, 257, 1), (4, 4, 32, 5, 20), (16, 1, 64, 90, 33)])
def test_tensor_core_attention_with_a_sink_and_kept_first_keys(kernels, path, Hq, Hkv, D, window, keep):
    """bfloat16 with values as wide as keys: the tensor-core kernels for portions (tensor memory and mma.sync) and for
    single tokens (TMA clusters and the one whose splits meet in scratch), over many key tiles and several units a tile.
    Kept keys within the window's first tile, in tiles of their own far behind it, and more of them than a stage of the
    decode kernel holds; portions that start at 0 and that continue; short requests beside long ones."""
    from kvcache_b200.engine.workspace import Workspace
    from kvcache_b200.kernels.api import CudaKernels
    k = kernels
    min_tiles = 16
    if path != "default":
        k = CudaKernels(DEV)
        if path.startswith("mma"):
            k.tc_attention_min_rows, k.decode_merge = None, "ticket"
        else:
            k.tc_attention_min_rows, min_tiles = 128, 2
    dtype = torch.bfloat16
    batch, kv = paged_scenario([(0, 700), (2500, 1), (1500, 300), (900, 1), (63, 1), (0, 1), (3, 2), (1100, 130)], num_kv_heads=Hkv, head_dim=D,
                               page_size=16, dtype=dtype, device="cpu", seed=11, window=window, tc_min_key_tiles=min_tiles)
    kv = dataclasses.replace(kv, spec=dataclasses.replace(kv.spec, keep_first=keep))
    T = batch.num_tokens
    q = _rand(T, Hq * D, dtype=dtype, seed=5, scale=0.5)
    sink = _rand(Hq, seed=6, scale=3.0)
    sink[0] = 0.0
    for s in (sink, torch.zeros(Hq)) + ((None,) if window and keep else ()):
        ref, got = torch.zeros(T, Hq * D, dtype=dtype), torch.zeros(T, Hq * D, dtype=dtype, device=DEV)
        TorchKernels(wide=True).paged_attention(q, batch, kv, ref, Hq, 0.2, sink=s)
        before = dict(k.launch_counts)
        k.paged_attention(q.to(DEV), batch_to(batch, DEV), clone_kv(kv, DEV), got, Hq, 0.2, Workspace(DEV), sink=None if s is None else s.to(DEV))
        k.check_errors()
        used = {name for name, count in k.launch_counts.items() if count > before.get(name, 0)}
        assert not used & {"attention_sink", "attention_generic"}, used
        assert_close(got, ref, TOL[dtype])


@pytest.mark.parametrize("Hq,Hkv,D,window,keep", [(2, 1, 64, None, 0), (2, 1, 64, 5000, 700), (4, 1, 128, 2000, 100), (2, 1, 64, 300, 2000)])
def test_single_tokens_of_few_long_requests_with_a_sink_and_kept_first_keys(kernels, Hq, Hkv, D, window, keep):
    """One or two requests with many cached keys: the TMA decode kernel gives each several clusters whose partial sums meet
    in scratch; the sink must be counted once, the kept keys must be read by exactly one cluster."""
    from kvcache_b200.engine.workspace import Workspace
    dtype = torch.bfloat16
    for segments in ([(9000, 1)], [(12000, 1), (8200, 1)]):
        batch, kv = paged_scenario(segments, num_kv_heads=Hkv, head_dim=D, page_size=16, dtype=dtype, device="cpu", seed=13, window=window)
        kv = dataclasses.replace(kv, spec=dataclasses.replace(kv.spec, keep_first=keep))
        T = batch.num_tokens
        q = _rand(T, Hq * D, dtype=dtype, seed=5, scale=0.5)
        sink = _rand(Hq, seed=6, scale=3.0)
        ref, got = torch.zeros(T, Hq * D, dtype=dtype), torch.zeros(T, Hq * D, dtype=dtype, device=DEV)
        TorchKernels(wide=True).paged_attention(q, batch, kv, ref, Hq, 0.2, sink=sink)
        before = dict(kernels.launch_counts)
        kernels.paged_attention(q.to(DEV), batch_to(batch, DEV), clone_kv(kv, DEV), got, Hq, 0.2, Workspace(DEV), sink=sink.to(DEV))
        kernels.check_errors()
        used = {name for name, count in kernels.launch_counts.items() if count > before.get(name, 0)}
        assert used == {"flash_decode_tma"}, used
        assert_close(got, ref, TOL[dtype])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_the_sink_alone_in_the_denominator_halves_a_single_keys_weight(kernels, dtype):
    """One token, one key: without a sink the result is the value; with a sink whose logit equals the score it is half of
    it; with a sink far above the score, nothing."""
    from kvcache_b200.engine.workspace import Workspace
    Hq, D, Dv = 2, 16, 8
    batch, kv = _kv_scenario([(0, 1)], 1, D, Dv, 4, dtype, seed=4)
    page = int(kv.block_table[0, 0])
    kv.k_pages[page, 0, 0] = 1.0
    q = torch.full((1, Hq * D), 0.25, dtype=dtype)                       # score = 16 * 0.25 * 0.5 = 2
    got = torch.zeros(1, Hq * Dv, dtype=dtype, device=DEV)
    kernels.paged_attention(q.to(DEV), batch_to(batch, DEV), clone_kv(kv, DEV), got, Hq, 0.5, Workspace(DEV), sink=torch.tensor([2.0, 40.0], device=DEV))
    value = kv.v_pages[page, 0, 0].float()
    assert_close(got.view(Hq, Dv)[0], 0.5 * value, TOL[dtype])
    assert float(got.view(Hq, Dv)[1].float().abs().max()) < 1e-12


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("decoded", [True, False])
@pytest.mark.parametrize("shape", [(32, 48, 8, 25, 16, 200, 11), (64, 64, 16, 300, 144, 2000, 11), (64, 64, 16, 300, 144, 2000, 400),
                                   (128, 128, 32, 100, 64, 1500, 130), (64, 64, 16, 1000, 16, 1100, 1)])
def test_one_key_at_an_edge_takes_all_the_weight(kernels, dtype, decoded, shape):
    """The query of one head matches one key and nothing else, and the head's result is that key's value (against a sink
    of 0): the window's first key; the last kept key, far behind the window, at a page's last row.  Then a key just
    outside each edge matches still more strongly (the one behind the window, the first one after the kept keys): the
    result must not move."""
    from kvcache_b200.engine.workspace import Workspace
    Hq, Hkv = 4, 2
    D, Dv, page, window, keep, last, portion = shape      # in bfloat16 the shapes with values as wide as keys take the tensor-core kernels
    if portion == 1 and not decoded:
        pytest.skip("the decoded case has it")
    segments = [(last, 1), (5, 1)] if decoded else [(last - portion + 1, portion), (0, 6)]
    row, pos = (0, last) if decoded else (portion - 2, last - 1)
    edges = {"window": (pos - window + 1, pos - window), "kept": (keep - 1, keep)}
    assert edges["kept"][0] % page == page - 1
    for edge, (inside, outside) in edges.items():
        batch, kv = _kv_scenario(segments, Hkv, D, Dv, page, dtype, window, keep, seed=6)
        T = batch.num_tokens
        key = lambda p, hk: kv.k_pages[int(kv.block_table[0, p // page]), hk, p % page]
        val = lambda p, hk: kv.v_pages[int(kv.block_table[0, p // page]), hk, p % page]
        for head, strong_outside in ((1, False), (2, True)):
            q = (_rand(T, Hq * D, seed=7) * 0.01).to(dtype)
            hk = head // (Hq // Hkv)
            q.view(T, Hq, D)[row, head] = (key(inside, hk).float() * 2.0).to(dtype)
            if strong_outside:
                key(outside, hk).copy_((key(inside, hk).float() * 1.5).to(dtype))
            got = torch.zeros(T, Hq * Dv, dtype=dtype, device=DEV)
            kernels.paged_attention(q.to(DEV), batch_to(batch, DEV), clone_kv(kv, DEV), got, Hq, 1.0, Workspace(DEV), sink=torch.zeros(Hq, device=DEV))
            assert_close(got.view(T, Hq, Dv)[row, head], val(inside, hk), 2e-2 if dtype == torch.bfloat16 else 1e-4, f"{edge}, head {head}")


@pytest.mark.parametrize("H,D", [(3, 8), (1, 33), (2, 40), (4, 64), (2, 128), (1, 200), (5, 6)])
def test_delta_rule_scan(kernels, H, D):
    """Prompts, a portion that continues a state, single tokens, states of other slots untouched; then every row alone,
    which must give the same bits as the rows together."""
    from kvcache_b200.engine.workspace import Workspace
    segments, slots = [(0, 19), (50, 1), (7, 6), (3, 1)], [2, 0, 3, 5]
    batch = _segments_batch(segments, slots)
    T = batch.num_tokens
    cols = (3, 3 + H * D, 3 + 2 * H * D, 5 + 3 * H * D)
    proj, z = _rand(T, 4 * H * D + 7, seed=1), _rand(T, H * D, seed=2, scale=2.0)
    memory = _rand(6, H, D, D, seed=3)
    memory[2].zero_()
    ref_mem, ref_out = memory.clone(), torch.zeros(T, H * D)
    TorchKernels(wide=True).delta_rule_scan(proj, cols, z, 0.6, 1e-6, batch, ref_mem, ref_out, H, D)
    ws = Workspace(DEV)
    got_mem, got_out = memory.clone().to(DEV), torch.zeros(T, H * D, device=DEV)
    kernels.delta_rule_scan(proj.to(DEV), cols, z.to(DEV), 0.6, 1e-6, batch_to(batch, DEV), got_mem, got_out, H, D, ws)
    assert_close(got_out, ref_out, 2e-5, "read-out")
    assert_close(got_mem, ref_mem, 2e-5, "states")
    assert torch.equal(got_mem[1].cpu(), memory[1]) and torch.equal(got_mem[4].cpu(), memory[4])
    one_mem, one_out = memory.clone().to(DEV), torch.zeros(T, H * D, device=DEV)
    at = 0
    for (start, n), slot in zip(segments, slots):
        for i in range(n):
            single = _segments_batch([(start + i, 1)], [slot])
            kernels.delta_rule_scan(proj[at:at + 1].to(DEV).contiguous(), cols, z[at:at + 1].to(DEV).contiguous(), 0.6, 1e-6, batch_to(single, DEV),
                                    one_mem, one_out[at:at + 1], H, D, ws)
            at += 1
    assert torch.equal(one_out, got_out) and torch.equal(one_mem, got_mem)


@pytest.mark.parametrize("H,D", [(2, 64), (1, 33), (2, 128), (3, 8), (1, 200)])
def test_delta_rule_scan_of_long_portions_in_chunks(kernels, H, D):
    """Portions long enough to be cut into chunks that run side by side (each leaves its end state and the product of its
    tokens' transitions; the start states follow from those): from an empty state and from a filled one, lengths that are
    no multiple of the chunk, beside single tokens and a short portion; against the plain recurrence and against the
    same kernel in one piece."""
    from kvcache_b200.engine.workspace import Workspace
    segments, slots = [(0, 300), (50, 1), (100, 257), (3, 1), (0, 64)], [2, 0, 3, 5, 1]
    batch = _segments_batch(segments, slots)
    assert batch.max_q_len >= kernels.SCAN_CHUNK_MIN_ROWS
    T = batch.num_tokens
    cols = (3, 3 + H * D, 3 + 2 * H * D, 5 + 3 * H * D)
    proj, z = _rand(T, 4 * H * D + 7, seed=1), _rand(T, H * D, seed=2, scale=2.0)
    memory = _rand(6, H, D, D, seed=3)
    memory[2].zero_()
    ref_mem, ref_out = memory.clone(), torch.zeros(T, H * D)
    TorchKernels(wide=True).delta_rule_scan(proj, cols, z, 0.6, 1e-6, batch, ref_mem, ref_out, H, D)
    ws = Workspace(DEV)
    got_mem, got_out = memory.clone().to(DEV), torch.zeros(T, H * D, device=DEV)
    before = kernels.launches
    kernels.delta_rule_scan(proj.to(DEV), cols, z.to(DEV), 0.6, 1e-6, batch_to(batch, DEV), got_mem, got_out, H, D, ws)
    kernels.check_errors()
    assert kernels.launches - before == 4, "inputs, local scan, chunk starts, scan from the starts"
    assert_close(got_out, ref_out, 1e-4, "read-out")
    assert_close(got_mem, ref_mem, 1e-4, "states")
    assert torch.equal(got_mem[4].cpu(), memory[4])
    whole_mem, whole_out = memory.clone().to(DEV), torch.zeros(T, H * D, device=DEV)
    chunk, kernels.SCAN_CHUNK = kernels.SCAN_CHUNK, 0
    try:
        kernels.delta_rule_scan(proj.to(DEV), cols, z.to(DEV), 0.6, 1e-6, batch_to(batch, DEV), whole_mem, whole_out, H, D, ws)
    finally:
        kernels.SCAN_CHUNK = chunk
    assert_close(got_out, whole_out, 1e-4, "read-out, chunks against one piece")
    assert_close(got_mem, whole_mem, 1e-4, "states, chunks against one piece")


def test_delta_rule_scan_of_a_very_long_portion_takes_longer_chunks(kernels):
    """A portion long enough for the longer chunks, beside a shorter one and a single token, against the plain recurrence."""
    from kvcache_b200.engine.workspace import Workspace
    H, D = 2, 64
    segments, slots = [(10, kernels.DELTA_LONG_ROWS + 77), (0, 130), (5, 1)], [1, 0, 2]
    batch = _segments_batch(segments, slots)
    T = batch.num_tokens
    cols = (0, H * D, 2 * H * D, 3 * H * D)
    proj, z = _rand(T, 4 * H * D, seed=1), _rand(T, H * D, seed=2, scale=2.0)
    memory = _rand(3, H, D, D, seed=3)
    ref_mem, ref_out = memory.clone(), torch.zeros(T, H * D)
    TorchKernels(wide=True).delta_rule_scan(proj, cols, z, 0.6, 1e-6, batch, ref_mem, ref_out, H, D)
    got_mem, got_out = memory.clone().to(DEV), torch.zeros(T, H * D, device=DEV)
    kernels.delta_rule_scan(proj.to(DEV), cols, z.to(DEV), 0.6, 1e-6, batch_to(batch, DEV), got_mem, got_out, H, D, Workspace(DEV))
    kernels.check_errors()
    assert_close(got_out, ref_out, 1e-4, "read-out")
    assert_close(got_mem, ref_mem, 1e-4, "states")


def test_delta_rule_scan_removes_along_the_unit_key_from_the_old_state(kernels):
    """One head, no decay (the decay's logit far below zero), removal rate 1 (its logit far above): writing the same key
    twice leaves k v2^T plus what the decay kept, not k (v1 + v2)^T - the first value is taken out along the unit key."""
    from kvcache_b200.engine.workspace import Workspace
    H, D = 1, 16
    batch = _segments_batch([(0, 2)], [0])
    k = _rand(D, seed=1)
    v1, v2 = _rand(D, seed=2), _rand(D, seed=3)
    proj = torch.zeros(2, 4 * D)
    proj[:, D:2 * D] = k
    proj[0, 2 * D:3 * D], proj[1, 2 * D:3 * D] = v1, v2
    proj[:, 3 * D:] = 40.0
    proj[:, :D] = k / (k * k).sum()
    z = torch.full((2, D), -40.0)
    memory, out = torch.zeros(1, H, D, D, device=DEV), torch.zeros(2, D, device=DEV)
    kernels.delta_rule_scan(proj.to(DEV), (0, D, 2 * D, 3 * D), z.to(DEV), 0.6, 0.0, batch_to(batch, DEV), memory, out, H, D, Workspace(DEV))
    assert_close(out[0], v1, 1e-5)
    assert_close(out[1], v2, 1e-5, "the first value was removed")


# ---- the model in the engine ------------------------------------------------------------------------------------------
def _runner(tmp_path, kernels, name, dtype, num_pages=64, sharpen=1.0, data=None, **kw):
    folder = make_lipelix_folder(tmp_path, name, sharpen=sharpen, dtype=torch.bfloat16, data=data)
    runner = make_runner(folder, kernels, dtype=dtype, device=DEV, page_size=PAGE_SIZE[name], num_pages=num_pages, **kw)
    config, weights = plain.read_folder(folder)
    return runner, config, weights


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_four_ways_of_cutting(tmp_path, kernels, name, dtype):
    page = PAGE_SIZE[name]
    runner, config, weights = _runner(tmp_path, kernels, name, dtype, num_pages=max(replay_modes.mixed_pool_tokens(), 128) // page)
    tokens = random_tokens(config["vocab"], 101, 3)
    want = plain.logits_of(config, weights, tokens)
    spread = _spread(config, weights, tokens, want)
    assert_model_close(replay_modes.whole(runner, tokens), want, dtype, "whole", spread)
    for n in (1, 2, 3):
        assert_model_close(replay_modes.whole(runner, tokens[:n]), want[:n], dtype, f"first {n}", spread)
    assert_model_close(replay_modes.last_32_one_by_one(runner, tokens), want[-33:], dtype, "decode", spread)
    assert_model_close(replay_modes.portions(runner, tokens, [2, 17, 3, 31, 2, 16, 8, 22]), want, dtype, "portions", spread)
    seqs = {k: random_tokens(config["vocab"], n, 10 + i) for i, (k, n) in enumerate(replay_modes.MIXED_LENGTHS)}
    got = replay_modes.mixed(runner, seqs)
    for k, toks in seqs.items():
        alone = plain.logits_of(config, weights, toks)
        assert_model_close(got[k], alone, dtype, f"mixed {k}", _spread(config, weights, toks, alone))
    assert runner.cache.used_pages() == 0
    kernels.check_errors()


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_float32_rows_do_not_depend_on_the_batch_or_the_cut(tmp_path, kernels, name):
    """In float32 a position's logits are bit for bit the same alone, beside other requests, and in portions."""
    runner, config, _ = _runner(tmp_path, kernels, name, "float32")
    from kvcache_b200.engine.runner import StepEntry
    a, b = random_tokens(config["vocab"], 40, 1), random_tokens(config["vocab"], 23, 2)
    alone = replay_modes.whole(runner, a)
    sa, sb = runner.cache.admit(), runner.cache.admit()
    first = runner.step([StepEntry(sb, b[:20], []), StepEntry(sa, a[:17], list(range(17)))]).clone()
    second = runner.step([StepEntry(sa, a[17:], list(range(23))), StepEntry(sb, b[20:21], [0])]).clone()
    assert torch.equal(torch.cat([first, second[:23]]), alone)


@pytest.mark.parametrize("name", ["A", "C", "E"])
def test_long_prompts(tmp_path, kernels, name):
    """float32: a prompt of several hundred tokens whole, in two long portions and beside another request; then decoded
    tokens behind it."""
    runner, config, weights = _runner(tmp_path, kernels, name, "float32", num_pages=160, max_tokens_per_step=700, max_tokens_per_request=700)
    from kvcache_b200.engine.runner import StepEntry
    tokens, other = random_tokens(config["vocab"], 600, 11), random_tokens(config["vocab"], 90, 12)
    want = plain.logits_of(config, weights, tokens)
    assert_close(replay_modes.whole(runner, tokens), want, 2e-4, "whole")
    assert_close(replay_modes.portions(runner, tokens, [290, 310]), want, 2e-4, "two portions")
    assert_close(replay_modes.portions(runner, tokens, [560] + [1] * 40), want, 2e-4, "decoded behind a long prompt")
    sa, sb = runner.cache.admit(), runner.cache.admit()
    got = runner.step([StepEntry(sb, other[:60], []), StepEntry(sa, tokens[:333], list(range(333)))]).clone()
    more = runner.step([StepEntry(sa, tokens[333:], list(range(267))), StepEntry(sb, other[60:], [29])]).clone()
    assert_close(torch.cat([got, more[:267]]), want, 2e-4, "beside another request")
    assert_close(more[267:], plain.logits_of(config, weights, other)[-1:], 2e-4, "the other request")
    kernels.check_errors()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_sharp_attention_at_the_edges(tmp_path, kernels, name, dtype):
    """Sharpened scores make single keys carry the softmax: a window or a run of kept tokens one token off, or a key lost
    at a page border, in a portion's first rows or behind decoded tokens, shows.  bfloat16, whose rounding of much larger
    scores would itself change which key wins, is sharpened less (its single keys are met at kernel level)."""
    sharpen, rel = (25.0, 1e-3) if dtype == "float32" else (4.0, None)
    runner, config, weights = _runner(tmp_path, kernels, name, dtype, sharpen=sharpen, num_pages=96, max_tokens_per_step=320, max_tokens_per_request=320)
    tokens = random_tokens(config["vocab"], 300, 5)
    want = plain.logits_of(config, weights, tokens)
    if dtype == "float32":
        for key, delta in (("size", -1), ("size", 1), ("keep_first", -1), ("keep_first", 1)):
            other, changed = copy.deepcopy(config), False
            for layer in other["layers"]:
                if layer["type"] == "attention_2" and layer["mixer"]["mask"][key] + delta >= (1 if key == "size" else 0):
                    layer["mixer"]["mask"][key] += delta
                    changed = True
            if changed:
                assert (plain.logits_of(other, weights, tokens) - want).abs().max() > 10 * rel * want.abs().max(), (key, delta)
    spread = _spread(config, weights, tokens, want) if dtype == "bfloat16" else None
    assert_model_close(replay_modes.portions(runner, tokens, [7, 2, 57, 64, 3, 135, 32]), want, dtype, "portions", spread, rel)
    assert_model_close(replay_modes.portions(runner, tokens, [230] + [1] * 70), want, dtype, "the window passes over decoded tokens", spread, rel)
    kernels.check_errors()


def test_pages_behind_the_window_are_given_back_but_the_kept_first_ones_stay(tmp_path, kernels):
    """A pool too small for the whole request is enough: pages behind the window go back and are used again, those that
    hold kept first tokens stay, and the logits are the whole prompt's."""
    data = config_dict("D")
    data["layers"] = data["layers"][:2]
    runner, config, weights = _runner(tmp_path, kernels, "D", "float32", num_pages=2 * 16, data=data, max_tokens_per_step=256, max_tokens_per_request=256)
    from kvcache_b200.engine.runner import StepEntry
    tokens = random_tokens(config["vocab"], 200, 7)
    slot = runner.cache.admit()
    got = [runner.step([StepEntry(slot, tokens[:90], list(range(90)))]).clone()]
    for i in range(90, 200):
        got.append(runner.step([StepEntry(slot, tokens[i:i + 1], [0])]).clone())
    runner.cache.release(slot)
    assert runner.cache.used_pages() == 0
    assert_close(torch.cat(got), plain.logits_of(config, weights, tokens), 1e-4)
    kernels.check_errors()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "E"])
def test_long_decoding_under_graphs_matches_plain(tmp_path, kernels, name, dtype):
    """200 tokens decoded one by one, two requests at a time, replayed from CUDA graphs: every state (delta-rule matrices,
    the token shift's previous rows, pages, kept values) moves exactly once a step."""
    from kvcache_b200.engine.runner import StepEntry
    runner, config, weights = _runner(tmp_path, kernels, name, dtype, num_pages=80, max_slots=2)
    runner.use_graphs = True
    seqs = [random_tokens(config["vocab"], 230, 7), random_tokens(config["vocab"], 215, 8)]
    slots = [runner.cache.admit(), runner.cache.admit()]
    runner.step([StepEntry(slots[0], seqs[0][:30], []), StepEntry(slots[1], seqs[1][:15], [])])
    last = None
    for i in range(200):
        entries = [StepEntry(slots[0], [seqs[0][30 + i]], [0], (0.0, 0, i)), StepEntry(slots[1], [seqs[1][15 + i]], [0], (0.0, 0, i))]
        last, tokens = runner.step(entries, sample=True)
    assert runner.graph_replays >= 190
    kernels.check_errors()
    for r in range(2):
        want = plain.logits_of(config, weights, seqs[r])
        assert_model_close(last[r:r + 1], want[-1:], dtype, f"request {r}", _spread(config, weights, seqs[r], want))
        assert int(tokens[r]) == int(torch.argmax(last[r]))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(tmp_path, kernels, dtype):
    """Through `LLM`, the scheduler and CUDA graphs: prompts cut into chunks beside decoding requests, more requests than
    run at once."""
    from kvcache_b200 import LLM, SamplingParams
    folder = make_lipelix_folder(tmp_path, "A", dtype=torch.bfloat16)
    config, weights = plain.read_folder(folder)
    prompts = [random_tokens(config["vocab"], n, 40 + n) for n in (1, 9, 24, 40, 63)]
    llm = LLM(folder, kernels=kernels, dtype=dtype, device=DEV, page_size=8, num_pages=80, max_running=3, max_tokens_per_step=48,
              chunk_size=16, use_graphs=True)
    got = llm.generate(prompts, SamplingParams(max_new_tokens=8, ignore_eos=True))
    assert llm.core.cache.used_pages() == 0
    for prompt, out in zip(prompts, got):
        logits = plain.logits_of(config, weights, list(prompt) + out)
        for i, token in enumerate(out):
            row = logits[len(prompt) - 1 + i]
            best = torch.topk(row, 2).values
            if float(best[0] - best[1]) > (1e-3 if dtype == "float32" else 0.05) * float(row.abs().max()):
                assert token == int(torch.argmax(row)), (len(prompt), i)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_program(tmp_path, dtype):
    """bin/trace_run as a user runs it, on a Lipelix folder: mixed steps, requests that pause, pages and slots used again."""
    folder = make_lipelix_folder(tmp_path, "A", dtype=torch.bfloat16)
    config, weights = plain.read_folder(folder)
    seqs = {k: random_tokens(config["vocab"], n, 20 + i) for i, (k, n) in enumerate([("a", 70), ("b", 33), ("c", 64), ("d", 50)])}
    plan = [([("a", 40), ("b", 2)], []), ([("b", 1), ("c", 64)], ["c"]), ([("a", 1), ("b", 30)], ["b"]), ([("d", 50), ("a", 29)], ["a", "d"])]
    done = {k: 0 for k in seqs}
    lines, expected = [], []
    for step, (parts, end) in enumerate(plan):
        entries = []
        for k, n in parts:
            entries.append({"id": k, "tokens": seqs[k][done[k]:done[k] + n], "want": list(range(n))})
            expected.append((step, k, done[k], n))
            done[k] += n
        lines.append(json.dumps({"step": step, "entries": entries, "end": end}))
    out = os.path.join(str(tmp_path), "out")
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", out,
                           "--max-tokens", "192", "--max-live", "3"], input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(len(plan))]
    want = {k: plain.logits_of(config, weights, seqs[k]) for k in seqs}
    spread = {k: _spread(config, weights, seqs[k], want[k]) for k in seqs}
    for step in range(len(plan)):
        got = torch.from_numpy(np.fromfile(os.path.join(out, f"{step}.f32"), dtype="<f4").reshape(-1, config["vocab"]))
        at = 0
        for s, k, lo, n in expected:
            if s == step:
                assert_model_close(got[at:at + n], want[k][lo:lo + n], dtype, f"step {step} {k}", spread[k])
                at += n
