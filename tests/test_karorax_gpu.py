"""The Karorax model through the engine on the GPU, in float32 and bfloat16, against the plain implementation, and every
CUDA operator (or operator option) it brought alone against the plain PyTorch statement of the same operator
(tests/torch_kernels.py)."""
import copy
import dataclasses
import json
import os
import subprocess
import sys

import numpy as np

import pytest
import torch

import plain_karorax as plain
import replay_modes
from helpers import assert_close, batch_to, clone_kv, make_runner, paged_scenario, random_tokens
from karorax_configs import CONFIGS, PAGE_SIZE, config_dict, make_karorax_folder
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
        return (plain.forward(config, weights, tokens) - want).abs().max(dim=1).values


def assert_model_close(got, want, dtype, what="", spread=None, rel=None):
    """float32: within `rel` of the largest logit.  bfloat16: the errors are held, as a distribution, to 4 times what
    rounding alone does in the plain implementation (`spread`: its per-position errors over the whole sequence): the k-th
    largest error against the k-th largest of the spread (floor: 1 % of the largest logit) except for the largest 2 % of
    them (at least one), the median position within 2 %, and no position beyond 30 % - a lost key, state or token moves
    many positions by as much as the logits themselves."""
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


def _used(k, before):
    return {name for name, count in k.launch_counts.items() if count > before.get(name, 0)}


# ---- operators alone ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W,T", [(24, 5), (200, 9), (896, 300), (2050, 3)])
def test_add_with_a_scale_per_channel(kernels, dtype, W, T):
    """h += scale * delta inside the launch that normalises the next rows: the scalar, the vector and the warp-per-row forms,
    in place and for gathered rows."""
    h, delta, scale, weight = _rand(T, W, seed=1), _rand(T, W, dtype=dtype, seed=2), _rand(W, seed=3), _rand(W, seed=4) + 1.0
    for rows in (None, torch.tensor([T - 1, 0, T // 2], dtype=torch.int32)):
        n = T if rows is None else len(rows)
        h_ref, out_ref = h.clone(), torch.zeros(n, W, dtype=dtype)
        TorchKernels().add_rmsnorm(h_ref, delta, weight, 1e-5, out_ref, rows, delta_scale=scale)
        h_dev, out = h.clone().to(DEV), torch.zeros(n, W, dtype=dtype, device=DEV)
        kernels.add_rmsnorm(h_dev, delta.to(DEV), weight.to(DEV), 1e-5, out, None if rows is None else rows.to(DEV), delta_scale=scale.to(DEV))
        assert_close(h_dev, h_ref, 1e-6, "the stream")
        assert_close(out, out_ref, TOL[dtype], "the normalised rows")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_capped_logits(kernels, dtype):
    x = _rand(7, 333, dtype=dtype, seed=1, scale=20.0)
    got = x.clone().to(DEV)
    kernels.activation_(got, "softcap", 11.0)
    assert_close(got, 11.0 * torch.tanh(x.double() / 11.0), TOL[dtype])


def _latent_scenario(segments, key_dim, page, dtype, window=None, seed=2, drop_behind=None):
    """A cache of shared key rows.  `drop_behind`: pages that lie wholly before the first key that this window lets the
    step's first row see are taken out of the block table, as a windowed cache entry gives them back."""
    from kvcache_b200.parts.base import PagedKVSpec, PagedKVView
    batch, kv = paged_scenario(segments, num_kv_heads=1, head_dim=key_dim, page_size=page, dtype=dtype, device="cpu", seed=seed, window=window)
    table = kv.block_table.clone()
    if drop_behind:
        for i, (start, _) in enumerate(segments):
            table[i, :max(0, start - drop_behind + 1) // page] = -1
    return batch, PagedKVView(spec=PagedKVSpec(1, key_dim, window, value_dim=0), k_pages=kv.k_pages, v_pages=kv.k_pages[..., :0].contiguous(),
                              block_table=table, page_size=page, writes=True)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,kv_rank,rot_dim,dims,window,own", [(3, 20, 4, 4, 11, 11), (7, 64, 32, 32, 150, 200), (4, 48, 16, 8, None, None),
                                                              (16, 128, 64, 64, 70, 70), (2, 40, 8, 8, 1, 33), (5, 24, 8, 8, 300, 300)])
def test_latent_attention_with_a_window_and_a_sink(kernels, dtype, H, kv_rank, rot_dim, dims, window, own):
    """Attention over shared key rows with a sink per head and a window that may be narrower than what the cache entry keeps
    (`own`: the entry's), pages behind the entry's window gone from the block table: whole prompts, portions that continue,
    single tokens of long and short requests.  bfloat16 rows in steps of 8 take the tensor-core kernel with the windowed
    work list; float32 the generic one."""
    from kvcache_b200.engine.workspace import Workspace
    from kvcache_b200.parts.base import StepPlan
    key_dim = kv_rank + rot_dim
    segments = [(0, 150), (700, 1), (400, 90), (63, 1), (0, 1), (3, 2), (1100, 65)]
    batch, kv = _latent_scenario(segments, key_dim, 16, dtype, own, drop_behind=own)
    T = batch.num_tokens
    q = _rand(T, H * key_dim, dtype=dtype, seed=5, scale=0.3)
    sink = _rand(H, seed=6, scale=2.0)
    planner = kernels.latent_attention_planner(H, key_dim, kv_rank, window)
    arrays, counts = planner.plan(np.asarray([s for s, _ in segments]), np.asarray([n for _, n in segments]))
    batch.plans[planner.name] = StepPlan({k: torch.tensor(np.array(v), dtype=torch.int32) for k, v in arrays.items()}, counts)
    for s in (sink, None):
        ref, got = torch.zeros(T, H * kv_rank, dtype=dtype), torch.zeros(T, H * kv_rank, dtype=dtype, device=DEV)
        TorchKernels(wide=True).latent_attention(q, batch, kv, ref, H, kv_rank, 0.3, window=window, sink=s)
        before = dict(kernels.launch_counts)
        kernels.latent_attention(q.to(DEV), batch_to(batch, DEV), clone_kv(kv, DEV), got, H, kv_rank, 0.3, Workspace(DEV), window=window,
                                 sink=None if s is None else s.to(DEV))
        kernels.check_errors()
        if dtype == torch.bfloat16:
            assert _used(kernels, before) == {"latent_flash"}, _used(kernels, before)
        assert_close(got, ref, TOL[dtype])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("decoded", [True, False])
def test_one_key_at_the_windows_edge_takes_all_the_weight_of_a_latent_head(kernels, dtype, decoded):
    """One head's query matches the window's first key and nothing else: the head's result is that row's latent (against a
    sink far below).  Then the key just behind the window matches still more strongly: the result must not move."""
    from kvcache_b200.engine.workspace import Workspace
    from kvcache_b200.parts.base import StepPlan
    H, kv_rank, rot_dim, window, page, last, portion = 4, 48, 16, 150, 16, 900, 70
    key_dim = kv_rank + rot_dim
    segments = [(last, 1), (5, 1)] if decoded else [(last - portion + 1, portion), (0, 6)]
    row, pos = (0, last) if decoded else (portion - 2, last - 1)
    inside, outside = pos - window + 1, pos - window
    planner = kernels.latent_attention_planner(H, key_dim, kv_rank, window)
    for strong_outside in (False, True):
        batch, kv = _latent_scenario(segments, key_dim, page, dtype, window, seed=6)
        arrays, counts = planner.plan(np.asarray([s for s, _ in segments]), np.asarray([n for _, n in segments]))
        batch.plans[planner.name] = StepPlan({k: torch.tensor(np.array(v), dtype=torch.int32) for k, v in arrays.items()}, counts)
        key = lambda p: kv.k_pages[int(kv.block_table[0, p // page]), 0, p % page]
        T = batch.num_tokens
        q = (_rand(T, H * key_dim, seed=7) * 0.01).to(dtype)
        q.view(T, H, key_dim)[row, 2] = (key(inside).float() * 2.0).to(dtype)
        if strong_outside:
            key(outside).copy_((key(inside).float() * 1.5).to(dtype))
        got = torch.zeros(T, H * kv_rank, dtype=dtype, device=DEV)
        kernels.latent_attention(q.to(DEV), batch_to(batch, DEV), clone_kv(kv, DEV), got, H, kv_rank, 1.0, Workspace(DEV), window=window,
                                 sink=torch.full((H,), -5.0, device=DEV))
        assert_close(got.view(T, H, kv_rank)[row, 2], key(inside)[:kv_rank], 2e-2 if dtype == torch.bfloat16 else 1e-4, f"outside strong: {strong_outside}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,dim,rot_dim,dims,kv_rank,vdim", [(3, 8, 4, 4, 20, 12), (6, 64, 32, 32, 96, 48), (2, 16, 8, 6, 24, 16), (5, 24, 10, 10, 33, 7)])
def test_latent_projections_from_columns_of_wider_rows(kernels, dtype, H, dim, rot_dim, dims, kv_rank, vdim):
    """The key/value latent at a column of its own (no query latent), the heads' queries as columns of the same rows taken to
    the latent's space with their rotated part turned, and one gate number per head on the way out."""
    T = 37
    q_width, key_dim = H * (dim + rot_dim), kv_rank + rot_dim
    P = -(-(q_width + key_dim + H) // 8) * 8
    proj = _rand(T, P, dtype=dtype, seed=1)
    segments = [(5, 20), (0, 17)]
    batch, kv = _latent_scenario(segments, key_dim, 8, dtype, None, seed=3)
    kv.k_pages.zero_()
    half = dims // 2
    angles = torch.arange(64, dtype=torch.float64)[:, None] * (100.0 ** (-torch.arange(half, dtype=torch.float64) * 2.0 / dims))[None, :]
    cos, sin = torch.cos(angles).float(), torch.sin(angles).float()
    weight = _rand(kv_rank, seed=4) + 1.0
    ref_kv, dev_kv = clone_kv(kv), clone_kv(kv, DEV)
    TorchKernels().latent_norm_rope_append(proj, 0, kv_rank, rot_dim, None, weight, 1e-5, cos, sin, batch, ref_kv, None, kv_col=q_width)
    kernels.latent_norm_rope_append(proj.to(DEV), 0, kv_rank, rot_dim, None, weight.to(DEV), 1e-5, cos.to(DEV), sin.to(DEV), batch_to(batch, DEV),
                                    dev_kv, None, kv_col=q_width)
    assert_close(dev_kv.k_pages, ref_kv.k_pages, TOL[dtype], "cache rows")
    w_uk_t, w_uv = _rand(H, kv_rank, dim, dtype=dtype, seed=5, scale=0.2), _rand(H, vdim, kv_rank, dtype=dtype, seed=6, scale=0.2)
    ref, got = torch.zeros(T, H * key_dim, dtype=dtype), torch.zeros(T, H * key_dim, dtype=dtype, device=DEV)
    TorchKernels().head_linear(proj, w_uk_t, ref, rotate=(cos, sin, batch.positions), x_col=0)
    kernels.head_linear(proj.to(DEV), w_uk_t.to(DEV), got, rotate=(cos.to(DEV), sin.to(DEV), batch.positions.to(DEV)), x_col=0)
    assert_close(got, ref, TOL[dtype], "queries in the latent's space")
    o_lat = _rand(T, H * kv_rank, dtype=dtype, seed=7)
    ref, got = torch.zeros(T, H * vdim, dtype=dtype), torch.zeros(T, H * vdim, dtype=dtype, device=DEV)
    TorchKernels().head_linear(o_lat, w_uv, ref, gate=(proj, q_width + key_dim), gate_per_head=True)
    kernels.head_linear(o_lat.to(DEV), w_uv.to(DEV), got, gate=(proj.to(DEV), q_width + key_dim), gate_per_head=True)
    kernels.check_errors()
    assert_close(got, ref, TOL[dtype], "gated heads")


def _kv_scenario(segments, Hkv, D, Dv, page, dtype, window=None, seed=2, fill=True):
    from kvcache_b200.parts.base import PagedKVSpec, PagedKVView
    batch, kv = paged_scenario(segments, num_kv_heads=Hkv, head_dim=D, page_size=page, dtype=dtype, device="cpu", seed=seed, window=window,
                               fill_history=fill)
    values = _rand(*kv.k_pages.shape[:-1], Dv, dtype=dtype, seed=seed + 1) if fill else torch.zeros(*kv.k_pages.shape[:-1], Dv, dtype=dtype)
    return batch, PagedKVView(spec=PagedKVSpec(Hkv, D, window, None if Dv == D else Dv), k_pages=kv.k_pages, v_pages=values,
                              block_table=kv.block_table, page_size=page, writes=True)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("Hq,Hkv,D,Dv,store", [(4, 2, 16, 8, 16), (3, 3, 6, 10, 10), (8, 2, 64, 48, 64), (5, 1, 40, 40, 40)])
def test_append_with_a_query_temperature_and_values_stored_wider(kernels, dtype, Hq, Hkv, D, Dv, store):
    """Queries times 1 + coef ln(floor((p + 1) / every) + 1) by the row's position; values written `store` wide with zeros
    after their numbers."""
    segments = [(0, 9), (130, 3), (63, 2)]
    batch, kv = _kv_scenario(segments, Hkv, D, store, 8, dtype, fill=False)
    kv.v_pages.fill_(7.0)                                        # stale rows: the zeros after a value must be written
    T = batch.num_tokens
    qkv = _rand(T, (Hq + Hkv) * D + Hkv * Dv + 3, dtype=dtype, seed=3)
    for temperature in ((0.4, 32), (1.5, 1), None):
        ref_kv, dev_kv = clone_kv(kv), clone_kv(kv, DEV)
        ref_q, got_q = torch.zeros(T, Hq * D, dtype=dtype), torch.zeros(T, Hq * D, dtype=dtype, device=DEV)
        extra = {} if temperature is None else {"q_temperature": temperature}
        TorchKernels().qkv_rope_append(qkv, None, None, None, batch, ref_kv, ref_q, Hq, key_dim=D, value_dim=Dv, **extra)
        kernels.qkv_rope_append(qkv.to(DEV), None, None, None, batch_to(batch, DEV), dev_kv, got_q, Hq, key_dim=D, value_dim=Dv, **extra)
        kernels.check_errors()
        assert_close(got_q, ref_q, TOL[dtype], "queries")
        assert_close(dev_kv.k_pages, ref_kv.k_pages, TOL[dtype], "keys")
        assert_close(dev_kv.v_pages, ref_kv.v_pages, TOL[dtype], "values")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("Hq,Hkv,D,Dv,cap", [(4, 2, 16, 8, 2.0), (3, 3, 6, 10, None), (8, 2, 64, 48, 40.0), (5, 1, 40, 72, 1.0), (2, 2, 200, 200, 7.0)])
def test_attention_with_a_cap_and_a_distance_bias(kernels, dtype, Hq, Hkv, D, Dv, cap):
    """The generic kernel (float32, and sizes the tensor-core kernels do not take): score <- cap tanh(score / cap), then minus
    slope_h (i - j); prompts, portions, single tokens, short and long requests."""
    from kvcache_b200.engine.workspace import Workspace
    batch, kv = _kv_scenario([(0, 70), (300, 1), (150, 30), (63, 1), (0, 1), (3, 2)], Hkv, D, Dv, 8, dtype)
    T = batch.num_tokens
    q = _rand(T, Hq * D, dtype=dtype, seed=5, scale=0.6)
    slopes = plain.distance_slopes(Hq).float()
    ref, got = torch.zeros(T, Hq * Dv, dtype=dtype), torch.zeros(T, Hq * Dv, dtype=dtype, device=DEV)
    TorchKernels(wide=True).paged_attention(q, batch, kv, ref, Hq, 0.4, score_cap=cap, slopes=slopes)
    kernels.paged_attention(q.to(DEV), batch_to(batch, DEV), clone_kv(kv, DEV), got, Hq, 0.4, Workspace(DEV), score_cap=cap, slopes=slopes.to(DEV))
    kernels.check_errors()
    assert_close(got, ref, TOL[dtype])
    plain_ref = torch.zeros_like(ref)
    TorchKernels(wide=True).paged_attention(q, batch, kv, plain_ref, Hq, 0.4)
    assert float((plain_ref.double() - ref.double()).abs().max()) > 0.05 * float(ref.double().abs().max())     # the options matter here


@pytest.mark.parametrize("path", ["default", "scratch decode", "tensor memory from 128 rows, tiles shared out"])
@pytest.mark.parametrize("Hq,Hkv,D,cap", [(4, 2, 64, 40.0), (8, 2, 64, 3.0), (2, 1, 128, None), (6, 2, 32, 20.0), (16, 1, 64, 1.0), (4, 4, 48, 8.0),
                                          (3, 1, 96, 30.0)])
def test_tensor_core_attention_with_a_cap_and_a_distance_bias(kernels, path, Hq, Hkv, D, cap):
    """bfloat16 with values as wide as keys: the tensor-memory and mma.sync kernels for portions and the TMA-cluster and
    scratch-merge kernels for single tokens make the whole score in their softmax step - over many key tiles, several units a
    tile, short requests beside long ones; no generic kernel may run."""
    from kvcache_b200.engine.workspace import Workspace
    from kvcache_b200.kernels.api import CudaKernels
    k = kernels
    min_tiles = 16
    if path == "scratch decode":
        k = CudaKernels(DEV)
        k.tc_attention_min_rows, k.decode_merge = None, "ticket"
    elif path != "default":
        k = CudaKernels(DEV)
        k.tc_attention_min_rows, min_tiles = 128, 2
    dtype = torch.bfloat16
    batch, kv = paged_scenario([(0, 700), (2500, 1), (1500, 300), (900, 1), (63, 1), (0, 1), (3, 2), (1100, 130)], num_kv_heads=Hkv, head_dim=D,
                               page_size=16, dtype=dtype, device="cpu", seed=11, tc_min_key_tiles=min_tiles)
    T = batch.num_tokens
    q = _rand(T, Hq * D, dtype=dtype, seed=5, scale=0.5)
    for slopes in (plain.distance_slopes(Hq).float(), None):
        if slopes is None and cap is None:
            continue
        ref, got = torch.zeros(T, Hq * D, dtype=dtype), torch.zeros(T, Hq * D, dtype=dtype, device=DEV)
        TorchKernels(wide=True).paged_attention(q, batch, kv, ref, Hq, 0.2, score_cap=cap, slopes=slopes)
        before = dict(k.launch_counts)
        k.paged_attention(q.to(DEV), batch_to(batch, DEV), clone_kv(kv, DEV), got, Hq, 0.2, Workspace(DEV), score_cap=cap,
                          slopes=None if slopes is None else slopes.to(DEV))
        k.check_errors()
        used = _used(k, before)
        assert not used & {"attention_sink", "attention_generic"}, used
        if D in (64, 128) and path != "scratch decode":
            assert "attention_tc" in used, used
        assert_close(got, ref, TOL[dtype])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("decoded", [True, False])
def test_one_far_key_takes_all_the_weight_through_the_distance_bias(kernels, dtype, decoded):
    """One head's query matches the request's first key, hundreds of pages back, strongly enough to pay the distance bias:
    the head's result is that key's value.  With the bias too large for the match, the nearest keys take over."""
    from kvcache_b200.engine.workspace import Workspace
    Hq, Hkv, D, page, last, portion = 4, 2, 64, 16, 3000, 200
    segments = [(last, 1), (5, 1)] if decoded else [(last - portion + 1, portion), (0, 6)]
    row, pos = (0, last) if decoded else (portion - 2, last - 1)
    batch, kv = _kv_scenario(segments, Hkv, D, D, page, dtype, seed=6)
    T = batch.num_tokens
    key0 = kv.k_pages[int(kv.block_table[0, 0]), 1, 0]
    val0 = kv.v_pages[int(kv.block_table[0, 0]), 1, 0]
    q = (_rand(T, Hq * D, seed=7) * 0.01).to(dtype)
    q.view(T, Hq, D)[row, 3] = (key0.float() * 3.0).to(dtype)                    # score about 3 |k|^2 = 190
    for slope, taken in ((0.03, True), (0.2, False)):                             # the bias costs 90, or 600
        slopes = torch.full((Hq,), slope)
        got = torch.zeros(T, Hq * D, dtype=dtype, device=DEV)
        kernels.paged_attention(q.to(DEV), batch_to(batch, DEV), clone_kv(kv, DEV), got, Hq, 1.0, Workspace(DEV), slopes=slopes.to(DEV))
        kernels.check_errors()
        err = float((got.view(T, Hq, D)[row, 3].double().cpu() - val0.double()).abs().max())
        assert (err < 0.05) == taken, (slope, err)


@pytest.mark.parametrize("H,D,Dv", [(3, 8, 16), (1, 33, 5), (2, 64, 32), (2, 128, 64), (1, 200, 40), (4, 16, 8)])
def test_lightning_scan(kernels, H, D, Dv):
    """silu on q, k, v, a constant decay per head, states from and into slots; rows alone and together are the same bits."""
    from kvcache_b200.engine.workspace import Workspace
    segments, slots = [(0, 20), (40, 1), (7, 37), (3, 2)], [2, 0, 3, 1]
    batch = _segments_batch(segments, slots)
    T = batch.num_tokens
    P = 2 * H * D + H * Dv + 5
    proj = _rand(T, P, seed=1)
    decay = torch.tensor([0.5, 0.97, 1.0, 0.0][:H])
    memory = _rand(4, H, D, Dv, seed=2, scale=0.3)
    cols = (3, 3 + H * D, 3 + 2 * H * D)
    ref_proj, ref_mem, ref = proj.clone(), memory.clone(), torch.zeros(T, H * Dv)
    TorchKernels(wide=True).lightning_scan(ref_proj, cols, decay, batch, ref_mem, ref, H, D, Dv)
    dev_mem, got = memory.clone().to(DEV), torch.zeros(T, H * Dv, device=DEV)
    kernels.lightning_scan(proj.clone().to(DEV), cols, decay.to(DEV), batch_to(batch, DEV), dev_mem, got, H, D, Dv, Workspace(DEV))
    assert_close(got, ref, 2e-5)
    assert_close(dev_mem, ref_mem, 2e-5, "states")
    alone = _segments_batch([segments[2]], [slots[2]])
    lo = 21
    mem2, got2 = memory.clone().to(DEV), torch.zeros(37, H * Dv, device=DEV)
    kernels.lightning_scan(proj[lo:lo + 37].clone().to(DEV), cols, decay.to(DEV), batch_to(alone, DEV), mem2, got2, H, D, Dv, Workspace(DEV))
    assert torch.equal(got2, got[lo:lo + 37]) and torch.equal(mem2[3], dev_mem[3])


@pytest.mark.parametrize("H,D,Dv", [(2, 64, 32), (1, 33, 5), (2, 128, 64)])
def test_lightning_scan_of_long_portions_in_chunks(kernels, H, D, Dv):
    from kvcache_b200.engine.workspace import Workspace
    segments, slots = [(0, 700), (40, 1), (100, 300)], [1, 0, 2]
    batch = _segments_batch(segments, slots)
    T = batch.num_tokens
    proj = _rand(T, 2 * H * D + H * Dv, seed=1, scale=0.7)
    decay = torch.tensor([0.998, 0.9][:H])
    memory = _rand(3, H, D, Dv, seed=2, scale=0.3)
    cols = (0, H * D, 2 * H * D)
    ref_mem, ref = memory.clone(), torch.zeros(T, H * Dv)
    TorchKernels(wide=True).lightning_scan(proj.clone(), cols, decay, batch, ref_mem, ref, H, D, Dv)
    dev_mem, got = memory.clone().to(DEV), torch.zeros(T, H * Dv, device=DEV)
    before = kernels.launches
    kernels.lightning_scan(proj.clone().to(DEV), cols, decay.to(DEV), batch_to(batch, DEV), dev_mem, got, H, D, Dv, Workspace(DEV))
    assert kernels.launches - before >= 4                           # inputs, local pass, chunk starts, pass with read-outs
    assert_close(got, ref, 1e-4)
    assert_close(dev_mem, ref_mem, 1e-4, "states")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,Dv", [(3, 16), (1, 5), (2, 32), (8, 128)])
def test_norm_over_all_heads_and_heads_with_unused_columns(kernels, dtype, H, Dv):
    T = 11
    o, gate, weight = _rand(T, H * Dv, seed=1), _rand(T, H * Dv + 6, seed=2), _rand(H * Dv, seed=3) + 1.0
    ref, got = torch.zeros(T, H * Dv + 4, dtype=dtype), torch.zeros(T, H * Dv + 4, dtype=dtype, device=DEV)
    TorchKernels().head_norm_gate(o, weight, 1e-5, (gate, 3), "sigmoid", 0.9, ref, 4, H, Dv, scope="all")
    kernels.head_norm_gate(o.to(DEV), weight.to(DEV), 1e-5, (gate.to(DEV), 3), "sigmoid", 0.9, got, 4, H, Dv, scope="all")
    assert_close(got, ref, TOL[dtype], "norm over all heads")
    per_head = torch.zeros_like(ref)
    TorchKernels().head_norm_gate(o, weight, 1e-5, (gate, 3), "sigmoid", 0.9, per_head, 4, H, Dv)
    if H > 1:
        assert float((per_head.double() - ref.double()).abs().max()) > 1e-2
    stride = Dv + 8
    x = _rand(T, H * stride, dtype=dtype, seed=4)
    ref, got = torch.zeros(T, H * Dv + 2, dtype=dtype), torch.zeros(T, H * Dv + 2, dtype=dtype, device=DEV)
    TorchKernels().head_gate(x, None, H, Dv, 1.2, ref, 2, x_head_stride=stride)
    kernels.head_gate(x.to(DEV), None, H, Dv, 1.2, got, 2, x_head_stride=stride)
    assert_close(got, ref, TOL[dtype], "heads with columns left out")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,E,top,W,F", [(9, 5, 2, 40, 24), (70, 16, 2, 192, 64), (400, 8, 3, 128, 32), (3, 3, 3, 64, 16)])
def test_routed_experts_with_the_plain_gated_activation(kernels, dtype, T, E, top, W, F):
    """silu(gate) * up in the grouped products' epilogues: CUDA cores (float32), mma.sync tiles, and from 1,024 pairs the
    tensor-memory kernel; with a shared expert's result as the base."""
    from kvcache_b200.engine.workspace import Workspace
    x = _rand(T, W, dtype=dtype, seed=1)
    w_up, w_down = _rand(E, 2 * F, W, dtype=dtype, seed=2, scale=0.2), _rand(E, W, F, dtype=dtype, seed=3, scale=0.2)
    logits = _rand(T, E, seed=4)
    base = _rand(T, W, dtype=dtype, seed=5)
    chosen, share = torch.zeros(T, top, dtype=torch.int32), torch.zeros(T, top)
    TorchKernels().route_top(logits, chosen, share)
    ref, got = torch.zeros(T, W, dtype=dtype), torch.zeros(T, W, dtype=dtype, device=DEV)
    TorchKernels(wide=True).routed_experts(x, w_up, w_down, chosen, share, ref, "swiglu", base=base)
    kernels.routed_experts(x.to(DEV), w_up.to(DEV), w_down.to(DEV), chosen.to(DEV), share.to(DEV), got, "swiglu", Workspace(DEV), base=base.to(DEV))
    kernels.check_errors()
    assert_close(got, ref, TOL[dtype] * 2)


# ---- the model in the engine ------------------------------------------------------------------------------------------
def _runner(tmp_path, kernels, name, dtype, num_pages=64, sharpen=1.0, data=None, **kw):
    folder = make_karorax_folder(tmp_path, name, sharpen=sharpen, dtype=torch.bfloat16, data=data, all_experts=dtype == "bfloat16")
    runner = make_runner(folder, kernels, dtype=dtype, device=DEV, page_size=PAGE_SIZE[name], num_pages=num_pages, **kw)
    config, weights = plain.read_folder(folder)
    return runner, config, weights


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_four_ways_of_cutting(tmp_path, kernels, name, dtype):
    page = PAGE_SIZE[name]
    runner, config, weights = _runner(tmp_path, kernels, name, dtype, num_pages=max(replay_modes.mixed_pool_tokens(), 128) // page)
    tokens = random_tokens(config["vocab"], 101, 3)
    want = plain.forward(config, weights, tokens)
    spread = _spread(config, weights, tokens, want)
    assert_model_close(replay_modes.whole(runner, tokens), want, dtype, "whole", spread)
    for n in (1, 2, 3):
        assert_model_close(replay_modes.whole(runner, tokens[:n]), want[:n], dtype, f"first {n}", spread)
    assert_model_close(replay_modes.last_32_one_by_one(runner, tokens), want[-33:], dtype, "decode", spread)
    assert_model_close(replay_modes.portions(runner, tokens, [2, 17, 3, 31, 2, 16, 8, 22]), want, dtype, "portions", spread)
    seqs = {k: random_tokens(config["vocab"], n, 10 + i) for i, (k, n) in enumerate(replay_modes.MIXED_LENGTHS)}
    got = replay_modes.mixed(runner, seqs)
    for k, toks in seqs.items():
        alone = plain.forward(config, weights, toks)
        assert_model_close(got[k], alone, dtype, f"mixed {k}", _spread(config, weights, toks, alone))
    assert runner.cache.used_pages() == 0
    kernels.check_errors()


def test_the_tensor_core_kernels_serve_sizes_in_steps_of_16(tmp_path, kernels):
    """Configuration E in bfloat16: no attention call of a step goes through a generic kernel."""
    runner, config, weights = _runner(tmp_path, kernels, "E", "bfloat16", num_pages=64)
    tokens = random_tokens(config["vocab"], 120, 3)
    before = dict(kernels.launch_counts)
    replay_modes.portions(runner, tokens, [80, 39, 1])
    used = _used(kernels, before)
    assert {"latent_flash", "flash_prefill"} <= used and not used & {"attention_generic", "attention_sink"}, used


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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "D", "E"])
def test_long_prompts(tmp_path, kernels, name, dtype):
    """A prompt of several hundred tokens whole (chunked scans, many key tiles), in two long portions and beside another
    request; then decoded tokens behind it."""
    runner, config, weights = _runner(tmp_path, kernels, name, dtype, num_pages=200, max_tokens_per_step=700, max_tokens_per_request=700)
    from kvcache_b200.engine.runner import StepEntry
    tokens, other = random_tokens(config["vocab"], 600, 11), random_tokens(config["vocab"], 90, 12)
    want = plain.forward(config, weights, tokens)
    spread = _spread(config, weights, tokens, want) if dtype == "bfloat16" else None
    assert_model_close(replay_modes.whole(runner, tokens), want, dtype, "whole", spread, 2e-4)
    assert_model_close(replay_modes.portions(runner, tokens, [290, 310]), want, dtype, "two portions", spread, 2e-4)
    assert_model_close(replay_modes.portions(runner, tokens, [560] + [1] * 40), want, dtype, "decoded behind a long prompt", spread, 2e-4)
    sa, sb = runner.cache.admit(), runner.cache.admit()
    got = runner.step([StepEntry(sb, other[:60], []), StepEntry(sa, tokens[:333], list(range(333)))]).clone()
    more = runner.step([StepEntry(sa, tokens[333:], list(range(267))), StepEntry(sb, other[60:], [29])]).clone()
    assert_model_close(torch.cat([got, more[:267]]), want, dtype, "beside another request", spread, 2e-4)
    kernels.check_errors()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C", "E"])
def test_sharp_attention_at_the_edges(tmp_path, kernels, name, dtype):
    """Sharpened scores make single keys carry the softmax: a window one token off (of the layer that owns a latent or of one
    that reads it), or a key lost at a page border, in a portion's first rows or behind decoded tokens, shows.  bfloat16, whose
    rounding of much larger scores would itself change which key wins, is sharpened less (its single keys are met at kernel level)."""
    sharpen, rel = (25.0, 1e-3) if dtype == "float32" else (4.0, None)
    runner, config, weights = _runner(tmp_path, kernels, name, dtype, sharpen=sharpen, num_pages=96, max_tokens_per_step=320, max_tokens_per_request=320)
    tokens = random_tokens(config["vocab"], 300, 5)
    want = plain.forward(config, weights, tokens)
    if dtype == "float32":
        for index, layer in enumerate(config["layers"]):
            if layer["type"] != "latent_attention" or layer["mixer"]["mask"]["size"] < 2:
                continue
            for delta in (-1, 1):
                other = copy.deepcopy(config)
                other["layers"][index]["mixer"]["mask"]["size"] += delta
                assert (plain.forward(other, weights, tokens) - want).abs().max() > 10 * rel * want.abs().max(), (index, delta)
    spread = _spread(config, weights, tokens, want) if dtype == "bfloat16" else None
    assert_model_close(replay_modes.portions(runner, tokens, [7, 2, 57, 64, 3, 135, 32]), want, dtype, "portions", spread, rel)
    assert_model_close(replay_modes.portions(runner, tokens, [230] + [1] * 70), want, dtype, "the windows pass over decoded tokens", spread, rel)
    kernels.check_errors()


def test_pages_behind_the_windows_are_given_back(tmp_path, kernels):
    """A pool too small for the whole request is enough for a model of windowed latent layers: pages behind the widest window
    that reads an entry go back and are used again, and the logits are the whole prompt's."""
    runner, config, weights = _runner(tmp_path, kernels, "C", "float32", num_pages=40, max_tokens_per_step=128, max_tokens_per_request=512)
    from kvcache_b200.engine.runner import StepEntry
    tokens = random_tokens(config["vocab"], 300, 7)
    slot = runner.cache.admit()
    got = [runner.step([StepEntry(slot, tokens[:50], list(range(50)))]).clone()]
    for i in range(50, 300):
        got.append(runner.step([StepEntry(slot, tokens[i:i + 1], [0])]).clone())
    runner.cache.release(slot)
    assert runner.cache.used_pages() == 0
    assert_close(torch.cat(got), plain.forward(config, weights, tokens), 1e-4)
    kernels.check_errors()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "E"])
def test_long_decoding_under_graphs_matches_plain(tmp_path, kernels, name, dtype):
    """200 tokens decoded one by one, two requests at a time, replayed from CUDA graphs: every state (lightning matrices,
    previous tokens, pages) moves exactly once a step."""
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
        want = plain.forward(config, weights, seqs[r])
        assert_model_close(last[r:r + 1], want[-1:], dtype, f"request {r}", _spread(config, weights, seqs[r], want))
        assert int(tokens[r]) == int(torch.argmax(last[r]))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(tmp_path, kernels, dtype):
    """Through `LLM`, the scheduler and CUDA graphs: prompts cut into chunks beside decoding requests, more requests than
    run at once."""
    from kvcache_b200 import LLM, SamplingParams
    folder = make_karorax_folder(tmp_path, "A", dtype=torch.bfloat16, all_experts=dtype == "bfloat16")
    config, weights = plain.read_folder(folder)
    prompts = [random_tokens(config["vocab"], n, 40 + n) for n in (1, 9, 24, 40, 63)]
    llm = LLM(folder, kernels=kernels, dtype=dtype, device=DEV, page_size=8, num_pages=80, max_running=3, max_tokens_per_step=48,
              chunk_size=16, use_graphs=True)
    got = llm.generate(prompts, SamplingParams(max_new_tokens=8, ignore_eos=True))
    assert llm.core.cache.used_pages() == 0
    for prompt, out in zip(prompts, got):
        logits = plain.forward(config, weights, list(prompt) + out)
        for i, token in enumerate(out):
            row = logits[len(prompt) - 1 + i]
            best = torch.topk(row, 2).values
            if float(best[0] - best[1]) > (1e-3 if dtype == "float32" else 0.05) * float(row.abs().max()):
                assert token == int(torch.argmax(row)), (len(prompt), i)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_program(tmp_path, dtype):
    """bin/trace_run as a user runs it, on a Karorax folder: mixed steps, requests that pause, pages and slots used again."""
    folder = make_karorax_folder(tmp_path, "A", dtype=torch.bfloat16, all_experts=dtype == "bfloat16")
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
    want = {k: plain.forward(config, weights, seqs[k]) for k in seqs}
    spread = {k: _spread(config, weights, seqs[k], want[k]) for k in seqs}
    for step in range(len(plan)):
        got = torch.from_numpy(np.fromfile(os.path.join(out, f"{step}.f32"), dtype="<f4").reshape(-1, config["vocab"]))
        at = 0
        for s, k, lo, n in expected:
            if s == step:
                assert_model_close(got[at:at + n], want[k][lo:lo + n], dtype, f"step {step} {k}", spread[k])
                at += n
