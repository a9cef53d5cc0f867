"""The kernel set: the contract every operator of a step goes through, and its CUDA form.

`KernelSet` states what each operator computes; `CudaKernels` launches the
hand-written sm_100a kernels of `kvcache_b200/csrc` through ctypes on the
current CUDA stream.  The parts of a model call nothing else for device work
(matrix products included: `linear`).  There is no CPU implementation in the
package; `CudaKernels` raises if the device or the compiler is missing.
"""
from __future__ import annotations

import contextlib
import ctypes
from collections import Counter
from typing import Dict, Optional, Sequence

import torch

from ..parts.base import PagedKVView, StepBatch
from . import build
from .attention_plan import PagedAttentionPlanner
from .latent_plan import LatentAttentionPlanner

_c_int, _c_float, _c_void_p, _c_longlong = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_longlong

DEVICE_ERRORS = {8: "a wait inside a kernel ran out (a pipeline stalled); the step's results are not valid",
                 1: "a token id outside the vocabulary",
                 2: "a key or value was needed from a page the block table does not hold",
                 4: "a position beyond the rotation table (longer than the model's maximum length)"}


class KernelError(RuntimeError):
    pass


class KernelSet:
    """Operators of a step.  Shapes: T rows, H width, all tensors contiguous.

    embed(table[V,H], ids[T], src[T], last) -> h[T,H] float32; row r takes last[src[r]] instead of ids[r] where src[r] >= 0
    add_rmsnorm(h, delta, weight, eps, out, rows):
        rows is None: h[r] += delta[r] (if delta is given); out[r] = h[r] * rsqrt(mean(h[r]^2) + eps) * weight
        rows given:   v = h[rows[i]] + delta[rows[i]];      out[i] = v * rsqrt(mean(v^2) + eps) * weight
    linear(x[M,K], w[N,K], out[M,N], bias[N] float32 or None): out = x . w^T + bias
    qkv_rope_append(qkv[T,(Hq+2Hkv)D], bias, cos, sin, batch, kv, q_out[T,Hq*D]):
        adds the bias, rotates queries and keys by the row's position, writes the queries to
        q_out and, if kv.writes, keys and values into their cache pages
    paged_attention(q[T,Hq*D], batch, kv, out[T,Hq*D], scale): causal (windowed if kv.spec.window)
        softmax(scale * q.k) v over the keys of the row's request, from the pages
    rope_append_attention(qkv, bias, cos, sin, batch, kv, out, num_heads, scale, workspace) -> bool   (optional)
        both of the above in one launch where the set has a kernel for the step at hand; False: nothing was
        done and the caller makes the two calls
    silu_mul(gate_up[T,2I], out[T,I]): out = silu(gate_up[:, :I]) * gate_up[:, I:]
    sample(logits[R,V], temperature[R], seeds[R], counters[R]) -> tokens[R] int32
    """

    def check_errors(self) -> None:
        """Raises if a kernel has flagged bad input since the last check (synchronises)."""


def _dtype_code(t: torch.dtype) -> int:
    if t == torch.float32:
        return 0
    if t == torch.bfloat16:
        return 1
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {t}")


def _ptr(t: Optional[torch.Tensor]) -> _c_void_p:
    if t is None:
        return _c_void_p(0)
    if not t.is_contiguous():
        raise KernelError("kernels take contiguous tensors")
    if not t.is_cuda:
        raise KernelError("kernels take tensors on the device; a host tensor's address means nothing there")
    return _c_void_p(t.data_ptr())


_RETURN_CODES = {-1: "unsupported dtype", -2: "unsupported shape", -3: "misaligned operand", -4: "size beyond the kernel's limit"}


def _check(code: int, what: str) -> None:
    if code == 0:
        return
    if code < 0:
        raise KernelError(f"{what}: refused ({_RETURN_CODES.get(code, code)})")
    raise KernelError(f"{what}: CUDA error {code} at launch")


_SIGNATURES = {
    "elementwise": {
        "kvb_embed": [_c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_float, _c_void_p,
                      _c_void_p],
        "kvb_token_shift": [_c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                            _c_int, _c_int, _c_void_p],
        "kvb_activation": [_c_int, _c_void_p, _c_longlong, _c_int, _c_float, _c_void_p],
        "kvb_add_rmsnorm": [_c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_float, _c_void_p],
        "kvb_silu_mul": [_c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p],
        "kvb_gated_act": [_c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_float, _c_void_p],
    },
    "rope_append": {
        "kvb_qkv_rope_append": [_c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_void_p,
                                _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int,
                                _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p],
        "kvb_qkv_norm_rope_append": [_c_int, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_float, _c_int, _c_void_p, _c_void_p,
                                     _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int,
                                     _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_int,
                                     _c_float, _c_int, _c_void_p, _c_void_p],
    },
    "recurrent": {
        "kvb_matrix_state_scan": [_c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_float,
                                  _c_float, _c_float, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                                  _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p],
        "kvb_delta_rule_scan": [_c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_float, _c_float, _c_void_p, _c_void_p,
                                _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p,
                                _c_void_p],
        "kvb_delta_rule_set_lanes": [_c_int],
        "kvb_head_norm_gate": [_c_int, _c_void_p, _c_void_p, _c_int, _c_float, _c_void_p, _c_int, _c_int, _c_int, _c_float, _c_void_p,
                               _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p],
        "kvb_head_gate": [_c_int, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_float, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int,
                          _c_void_p],
        "kvb_lightning_scan": [_c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                               _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p],
        "kvb_bigram_embed": [_c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                             _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p],
    },
    "attention_generic": {
        "kvb_paged_attention_kv": [_c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int,
                                   _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_void_p, _c_void_p],
        "kvb_paged_attention_sink": [_c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int,
                                     _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_float, _c_void_p, _c_void_p],
        "kvb_paged_attention_ext": [_c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int,
                                    _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_float, _c_float, _c_void_p,
                                    _c_void_p, _c_void_p],
        "kvb_paged_attention_generic": [_c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p,
                                        _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                                        _c_float, _c_void_p, _c_void_p],
        "kvb_paged_attention_shared": [_c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p,
                                       _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_void_p, _c_void_p],
    },
    "latent": {
        "kvb_norm_add_rmsnorm": [_c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_float, _c_void_p, _c_float, _c_void_p, _c_void_p,
                                 _c_void_p, _c_int, _c_int, _c_void_p],
        "kvb_latent_norm_rope_append": [_c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_float,
                                        _c_void_p, _c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int,
                                        _c_void_p, _c_int, _c_int, _c_void_p, _c_int, _c_void_p, _c_void_p],
        "kvb_head_linear": [_c_int, _c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p,
                            _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p],
    },
    "latent_flash": {
        "kvb_latent_flash_supports": [_c_int, _c_int, _c_int],
        "kvb_latent_flash": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_void_p, _c_void_p,
                             _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int,
                             _c_void_p, _c_void_p, _c_void_p],
    },
    "gemm_grouped": {
        "kvb_gather_rows": [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p],
        "kvb_grouped_gemm_tcgen05": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int,
                                     _c_int, _c_void_p, _c_void_p],
        "kvb_grouped_gemm_tcgen05_act": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int,
                                         _c_int, _c_float, _c_void_p, _c_void_p],
    },
    "moe": {
        "kvb_route_top": [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p],
        "kvb_route_top_scores": [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p],
        "kvb_grouped_gemm_act": [_c_int, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int,
                                 _c_int, _c_int, _c_int, _c_float, _c_void_p],
        "kvb_routed_combine_base": [_c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p],
        "kvb_routed_plan": [_c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p],
        "kvb_grouped_gemm": [_c_int, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int,
                             _c_int, _c_int, _c_int, _c_void_p],
        "kvb_routed_combine": [_c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p],
    },
    "gemm_simt": {
        "kvb_gemm_simt": [_c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p],
    },
    "gemm_skinny": {
        "kvb_gemm_skinny": [_c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p],
        "kvb_gemm_skinny_gated": [_c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_float, _c_void_p],
        "kvb_gemm_skinny_norm_act": [_c_void_p, _c_void_p, _c_void_p, _c_float, _c_void_p, _c_int, _c_int, _c_int, _c_void_p],
        "kvb_gemm_skinny_residual": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p],
        "kvb_gemm_skinny_qkv": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_float, _c_void_p, _c_void_p, _c_int, _c_void_p,
                                _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int,
                                _c_int, _c_int, _c_int, _c_void_p, _c_void_p],
    },
    "gemm_wstream": {
        "kvb_gemm_wstream": [_c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_void_p],
        "kvb_gemm_wstream_gated": [_c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_float, _c_void_p, _c_void_p],
    },
    "gemm_tcgen05": {
        "kvb_gemm_tcgen05": [_c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_void_p],
    },
    "attention_flash": {
        "kvb_flash_head_dim": [],
        "kvb_flash_decode": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p,
                             _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float,
                             _c_void_p, _c_int, _c_void_p, _c_float, _c_void_p],
        "kvb_flash_decode_cluster": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int,
                                     _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float,
                                     _c_void_p],
        "kvb_flash_decode_tma_max_clusters": [_c_int],
        "kvb_flash_decode_tma": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_int,
                                 _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float,
                                 _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_void_p,
                                 _c_void_p, _c_int, _c_void_p, _c_float, _c_void_p, _c_void_p],
        "kvb_flash_prefill": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p,
                              _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_float, _c_void_p,
                              _c_int, _c_void_p, _c_float, _c_void_p],
    },
    "attention_tc": {
        "kvb_attention_tc_head_dim": [],
        "kvb_attention_tc": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p,
                             _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float,
                             _c_void_p, _c_int, _c_void_p, _c_float, _c_void_p, _c_void_p],
    },
    "primitive_costs": {
        "kvb_primitive_costs_count": [],
        "kvb_primitive_costs": [_c_void_p, _c_void_p, _c_void_p, _c_void_p],
    },
    "wait_probe": {
        "kvb_wait_probe": [_c_void_p, _c_void_p, _c_void_p],
    },
    "sampling": {
        "kvb_sample_parts": [_c_int],
        "kvb_sample": [_c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p],
    },
}


_OPTIONAL = {"kvb_flash_decode_tma", "kvb_flash_decode_tma_max_clusters"}      # only in attention_flash variants for head sizes 64 and 128


class _Library:
    """A lazily built and loaded kernel module with typed entry points."""

    def __init__(self, module: str, variant: str = "", flags: Sequence[str] = ()):
        self.module, self.variant, self.flags = module, variant, tuple(flags)
        self._lib = None

    def __getattr__(self, name: str):
        if self._lib is None:
            lib = build.load_module(self.module, self.variant, self.flags)
            for fname, argtypes in _SIGNATURES[self.module].items():
                try:
                    fn = getattr(lib, fname)
                except AttributeError:
                    if fname in _OPTIONAL:
                        continue              # a variant compiled for a size that has no such entry point
                    raise
                fn.argtypes = argtypes
                fn.restype = _c_int
            self._lib = lib
        return getattr(self._lib, name)


class CudaKernels(KernelSet):
    def __init__(self, device: torch.device | str = "cuda:0", bf16_gemm: str = "auto"):
        """`bf16_gemm`: which kernel multiplies bfloat16 matrices of more than SKINNY_MAX_ROWS rows:
        "tcgen05" (the tensor-memory kernel of csrc/gemm_tcgen05.cu), "cublas" (the library, as the
        reference uses it), "simt" (CUDA cores), or "auto": the tensor-memory kernel for the gate/up
        projection with its fused activation where 256 x 256 two-SM tiles fill the machine (measured
        30.8 us against 28.4 + 13.6 us for library product + activation kernel at 2,048 x 9,728 x 896),
        the library for plain products, where it is still ahead (28.4 against 33.7 us at that size)."""
        self.device = torch.device(device)
        if self.device.type != "cuda" or not torch.cuda.is_available():
            raise KernelError("kvcache_b200 runs on a CUDA device (sm_100a) only; no device is available")
        major, minor = torch.cuda.get_device_capability(self.device)
        if major != 10:
            raise KernelError(f"kernels are built for sm_100a; device {self.device} is sm_{major}{minor}")
        if bf16_gemm not in ("auto", "tcgen05", "cublas", "simt"):
            raise KernelError(f"unknown bf16_gemm '{bf16_gemm}'")
        self.bf16_gemm = bf16_gemm
        self._elementwise = _Library("elementwise")
        self._rope = _Library("rope_append")
        self._attn_generic = _Library("attention_generic")
        self._gemm_simt = _Library("gemm_simt")
        self._latent = _Library("latent")
        self._recurrent = _Library("recurrent")
        self._moe = _Library("moe")
        self._latent_flash = _Library("latent_flash")
        self._gemm_grouped = _Library("gemm_grouped")
        # Steps with at least this many (row, choice) pairs run the routed feed-forward's products through the tensor-memory
        # kernel (bfloat16, widths in steps of 8): tiles of 128 rows per expert only pay when experts have that many rows.
        self.routed_tcgen05_min_pairs: Optional[int] = 1024
        self.latent_flash = True             # bfloat16, key rows in steps of 8 numbers: the tensor-core kernel over shared key rows
        self._latent_planners: Dict[tuple, "LatentAttentionPlanner"] = {}
        self._zero_slopes: Dict[int, torch.Tensor] = {}
        self._sampling = _Library("sampling")
        self._gemm_skinny = _Library("gemm_skinny")
        self._gemm_tc = _Library("gemm_tcgen05")
        self._gemm_ws = _Library("gemm_wstream")
        self.wstream_gemm = True             # bfloat16, 16 < M <= WSTREAM_MAX_ROWS, K % 8 == 0: weights streamed through tcgen05
        self.skinny_gemm = True              # bfloat16, M <= 64, K % 32 == 0: weight-streaming kernel
        self._flash: Dict[int, _Library] = {}
        self._attn_tc: Dict[int, _Library] = {}
        # Portions of prompts with at least this many rows go through the tensor-memory attention kernel
        # (bfloat16, head size 64 or 128, pages of 8..64 tokens); None turns it off.  Measured on 24 layers of the
        # 0.5B shape: the mma.sync kernel is ahead at 128 and 256 rows (1.09 / 1.24 ms a step against 1.14 / 1.28),
        # the tensor-memory kernel from 512 rows on (1.56 against 1.69 ms).
        self.tc_attention_min_rows: Optional[int] = 384
        self.flash_attention = True          # bfloat16, head sizes 16..128: tensor-core kernels
        # Decode steps of at least this many requests: bias, rotation and append inside the TMA decode kernel (None: never).
        # Measured on 24 layers of the 0.5B shape at 4,096 tokens of context, a step with the kernel against a step with
        # the separate rotation kernel: 1 % slower at 1 and 8 requests (the queries reach the tensor cores a trip through
        # shared memory later, which costs what the saved launch gains), 1.4 % faster at 16, 3 % at 64.
        self.fused_rope_min_requests: Optional[int] = 16
        # Decode attention splits the keys of a request over blocks.  "cluster": the splits (at most 8) are a
        # thread-block cluster and merge through distributed shared memory; "tma": the same with keys and values
        # brought by TMA (head sizes 64 and 128, pages of 8..64 tokens; otherwise it falls back to "cluster");
        # "ticket": up to 32 splits leave partial results in scratch and the last one to finish merges them.
        self.decode_merge = "tma"
        self.decode_cluster_max = 8          # the kernel's limit
        self.decode_pow2_splits = True
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.decode_ctas_wanted = 2 * self.sm_count    # the split over the keys aims at this many blocks in flight
        self.decode_min_tiles = 4            # ... but gives a split at least this many 64-key tiles
        # Most clusters one (request, kv head) is given by the TMA kernel (0: always one).  The clusters meet through memory,
        # which costs about 5 us; it pays where there are fewer blocks than SMs and each block still keeps eight 64-key tiles -
        # one request: 10.5 -> 8.9 us a layer at 8,192 tokens, 18.0 -> 10.9 at 16,000, 34.6 -> 11.8 at 32,000 - and not where
        # the blocks fill the GPU already (8 requests at 8,192 tokens: 11.7 -> 17.3 us).
        self.decode_superclusters = 16
        self.decode_super_min_tiles = 8
        self.error_word = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.launches = 0
        self.launch_counts: Counter = Counter()      # launches by kernel, as issued from the host (a replayed graph adds none)
        self._pinned_stream: Optional[_c_void_p] = None
        self._tma_cluster_capacity: Dict[tuple, int] = {}
        self._timing = None
        self._attention_planner: Optional[PagedAttentionPlanner] = None

    # ---- helpers -----------------------------------------------------------
    def _count(self, kernel: str) -> None:
        """One launch of `kernel` (while a graph is being recorded: one launch of every later replay)."""
        self.launches += 1
        self.launch_counts[kernel] += 1

    def _stream(self) -> _c_void_p:
        if self._pinned_stream is not None:
            return self._pinned_stream
        return _c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    @contextlib.contextmanager
    def on_current_stream(self):
        """Within the block every launch goes to the stream that is current now (asked for once, not per launch)."""
        saved = self._pinned_stream
        self._pinned_stream = _c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        try:
            yield
        finally:
            self._pinned_stream = saved

    def start_timing(self, hold_ms: float = 4.0) -> None:
        """From now on every operator is bracketed by CUDA events and filed under its class (kernels/timing.py).
        For steps launched kernel by kernel: graphs cannot hold the events.  `hold_ms`: how long the GPU is kept busy
        before each step so that the host can queue the step's launches (0: not at all)."""
        from .timing import KernelTiming
        if self._timing is None:
            self._timing = KernelTiming(self, hold_ms)
            self._timing.start()

    def stop_timing(self) -> Dict[str, dict]:
        """Ends timing; returns {class: {"us", "bytes", "calls", "launches"}} summed over the calls since `start_timing`."""
        timing, self._timing = self._timing, None
        return timing.stop() if timing is not None else {}

    def check_errors(self) -> None:
        word = int(self.error_word.item())
        if word:
            self.error_word.zero_()
            reasons = [text for bit, text in DEVICE_ERRORS.items() if word & bit]
            raise KernelError("a kernel flagged bad input: " + "; ".join(reasons))

    def probe_wait_timeout(self) -> int:
        """Runs a kernel whose only wait cannot end (csrc/wait_probe.cu: the bounded mbarrier wait of the TMA and tcgen05
        kernels, on a barrier nothing arrives on, with a short poll limit).  The kernel gives up, sets the time-out bit of
        the error word and returns; the next `check_errors()` raises.  Returns the number of polls it made."""
        outcome = torch.zeros(2, dtype=torch.int32, device=self.device)
        self._count("wait_probe")
        _check(_Library("wait_probe").kvb_wait_probe(_ptr(self.error_word), _ptr(outcome), self._stream()), "wait_probe")
        gave_up, polls = (int(v) for v in outcome.tolist())
        if gave_up != 2:
            raise KernelError("the wait of the probe kernel ended although nothing arrived on its barrier")
        return polls

    PRIMITIVE_NAMES = ("wait on a completed mbarrier, all lanes", "the same, one lane asks and the warp meets again", "shuffle",
                       "vote and population count", "expect_tx by one lane and the warp meets again",
                       "tcgen05.mma 128 x 64 x 16, operands in shared memory", "tcgen05.mma 128 x 128 x 16, operands in shared memory",
                       "tcgen05.mma 128 x 64 x 16, A in tensor memory", "tcgen05.commit", "TMA copy of one page (16 rows of 128 bytes)",
                       "tcgen05.ld of 32 columns and its wait", "mma.sync m16n8k16 (bfloat16), eight accumulators in turn",
                       "mma.sync m16n8k16, each needing the one before")

    def primitive_costs(self) -> Dict[str, float]:
        """Clocks per primitive of the warp-specialised kernels on an otherwise idle SM (csrc/primitive_costs.cu)."""
        lib = _Library("primitive_costs")
        count = lib.kvb_primitive_costs_count()
        zeros = torch.zeros(4 << 20, dtype=torch.uint8, device=self.device)
        out = torch.zeros(count + 1, dtype=torch.float32, device=self.device)
        for _ in range(2):          # the second run finds the code and the tensor map cached
            self._count("primitive_costs")
            _check(lib.kvb_primitive_costs(_ptr(zeros), _ptr(out), _ptr(self.error_word), self._stream()), "primitive_costs")
        self.check_errors()
        return dict(zip(self.PRIMITIVE_NAMES, out[:count].tolist()))

    def paged_attention_planner(self) -> PagedAttentionPlanner:
        """The work lists `paged_attention` and `rope_append_attention` read from `StepBatch.plans` (one planner for all layers)."""
        if self._attention_planner is None:
            self._attention_planner = PagedAttentionPlanner()
        return self._attention_planner

    # Tiles of 32 rows where 64 rows leave room for one key stage only: measured slower (a prompt of 2,048 tokens, 16 heads, rows
    # of 576: 537 us with two stages beside 32 rows, 448 us with one stage beside 64 - a key tile then serves half the rows).
    latent_small_large_tile = False

    def _latent_plan_shape(self, key_dim: int, value_dim: int) -> tuple:
        """(blocks wanted, rows of a large tile) of the attention over shared key rows at these sizes."""
        dk_pad = -(-key_dim // 32) * 32
        row = max(dk_pad, 64 * (1 if value_dim <= 64 else 2 if value_dim <= 128 else 4 if value_dim <= 256 else 8)) + 8
        fits = lambda bm, stages: bm * (dk_pad + 8) * 2 + stages * 64 * row * 2 + bm * 72 * 4 + bm * 72 * 2 + bm * 16 <= 220 * 1024
        tile = 32 if self.latent_small_large_tile and not fits(64, 2) and fits(32, 2) else 64
        return self._latent_blocks_wanted(key_dim, value_dim), tile

    def _latent_blocks_wanted(self, key_dim: int, value_dim: int) -> int:
        """As many blocks as the GPU holds at once of the kernel's form for decoded tokens (tiles of 16 rows, two key stages):
        two an SM while their shared memory allows (csrc/latent_flash.cu, make_layout), else one - a second wave of blocks
        costs more than longer runs of keys per block (8 requests of 4,096 tokens, rows of 576: 20.0 us with 144 blocks, 22.9 with 256)."""
        dk_pad = -(-key_dim // 32) * 32
        row = max(dk_pad, 64 * (1 if value_dim <= 64 else 2 if value_dim <= 128 else 4 if value_dim <= 256 else 8)) + 8
        smem = 16 * (dk_pad + 8) * 2 + 2 * 64 * row * 2 + 16 * 68 * 4 + 16 * 72 * 2 + 256
        return (2 if 2 * smem <= 220 * 1024 else 1) * self.sm_count

    def latent_attention_planner(self, heads: int, key_dim: int, value_dim: int, window: Optional[int] = None) -> LatentAttentionPlanner:
        """The work list `latent_attention` reads from `StepBatch.plans` for mixers of these sizes and this window (one
        planner for all of them)."""
        key = (heads, *self._latent_plan_shape(key_dim, value_dim), int(window or 0))
        found = self._latent_planners.get(key)
        if found is None:
            found = self._latent_planners[key] = LatentAttentionPlanner(*key)
        return found

    # ---- operators ---------------------------------------------------------
    def embed(self, table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, src: Optional[torch.Tensor] = None,
              last: Optional[torch.Tensor] = None, out16: Optional[torch.Tensor] = None, scale: float = 1.0) -> None:
        """out[r] = table[ids[r]] * scale, or table[last[src[r]]] * scale where src[r] >= 0 (a token still on the device);
        `out16`: the same rows in bfloat16 as well."""
        T, H = out.shape
        self._count("embed")
        _check(self._elementwise.kvb_embed(_dtype_code(table.dtype), _ptr(table), _ptr(ids), _ptr(src), _ptr(last), _ptr(out),
                                           _ptr(out16), T, H, table.shape[0], float(scale), _ptr(self.error_word), self._stream()),
               "embed")

    def token_shift(self, x: torch.Tensor, weight: torch.Tensor, previous: torch.Tensor, batch: StepBatch, out: torch.Tensor) -> None:
        """out[r] = x[r] + (before - x[r]) * weight: `before` is the row above r in r's segment, or previous[slot] for the
        segment's first row (zeros at position 0); previous[slot] (float32 [slots, H]) then becomes the segment's last row."""
        T, H = x.shape
        if previous.dtype != torch.float32 or weight.dtype != torch.float32 or out.dtype != x.dtype:
            raise KernelError("token_shift: float32 weight and state, rows and result of one type")
        self._count("token_shift")
        _check(self._elementwise.kvb_token_shift(_dtype_code(x.dtype), _ptr(x), _ptr(weight), _ptr(previous), _ptr(batch.positions),
                                                 _ptr(batch.row_segment), _ptr(batch.seg_q_start), _ptr(batch.seg_q_len),
                                                 _ptr(batch.seg_slot), _ptr(out), T, H, self._stream()), "token_shift")

    ACTIVATIONS = {"tanh": 0, "relu2": 1, "softcap": 2}

    def activation_(self, x: torch.Tensor, kind: str, cap: float = 0.0) -> None:
        """x = tanh(x), relu(x)^2 or cap * tanh(x / cap) ("softcap"), in place."""
        if kind not in self.ACTIVATIONS:
            raise KernelError(f"activation_: '{kind}' is not built")
        self._count("activation")
        _check(self._elementwise.kvb_activation(_dtype_code(x.dtype), _ptr(x), x.numel(), self.ACTIVATIONS[kind], float(cap),
                                                self._stream()), "activation")

    # ---- the folded chain of a decode layer ------------------------------------------------------------------
    # For steps of few rows a layer can run as five launches instead of eight: the norm before a product inside that
    # product (x holds the residual stream in bfloat16, not normalised), the add after a product inside it
    # (`linear_into_residual`), and bias, rotation and cache append inside the q/k/v projection.  Off by default: measured
    # on 24 layers of the 0.5B shape at 8 requests and 4,096 tokens of context the folded chain takes 32 us a layer against
    # 26 - each folded product takes as long as the kernels it replaces together (q/k/v 5.6 us against 2.5 + 1.9 + 1.4),
    # and the products that add into the residual stream 5.0 us against 2.5, because the kernel after them, which streams
    # many megabytes of weights before its own wait, now crowds their loads instead of a norm kernel's that has few.
    fold_norms = False

    @property
    def fold_key(self) -> tuple:
        """The switches `can_fold` depends on (a model caches its answer per value of this)."""
        return (self.fold_norms, self.skinny_gemm, self.wstream_gemm, self.bf16_gemm)

    def can_fold(self, dtype: torch.dtype, rows: int, K: int, N: int) -> bool:
        """Whether a product of `rows` rows with a [N, K] weight can take the folded forms (the register kernel's)."""
        return self.fold_norms and self._skinny(dtype, rows, K, N)

    def norm_gate_up_act(self, x16: torch.Tensor, w_gate_up: torch.Tensor, norm_w: torch.Tensor, eps: float, out: torch.Tensor) -> None:
        """out[M, I] = silu(g) * u with [g | u] = rmsnorm(x16; norm_w, eps) . w_gate_up^T (rows interleaved in eights)."""
        M, K = x16.shape
        self._count("gemm_skinny_norm_act")
        _check(self._gemm_skinny.kvb_gemm_skinny_norm_act(_ptr(x16), _ptr(w_gate_up), _ptr(norm_w), float(eps), _ptr(out), M,
                                                          w_gate_up.shape[0], K, self._stream()), "norm_gate_up_act")

    def linear_into_residual(self, x: torch.Tensor, w: torch.Tensor, h: torch.Tensor, h16: torch.Tensor,
                             bias: Optional[torch.Tensor] = None) -> None:
        """h += x . w^T + bias (float32, in place); h16 = bfloat16(h)."""
        M, K = x.shape
        self._count("gemm_skinny_residual")
        _check(self._gemm_skinny.kvb_gemm_skinny_residual(_ptr(x), _ptr(w), _ptr(bias), _ptr(h), _ptr(h16), M, w.shape[0], K,
                                                          self._stream()), "linear_into_residual")

    def norm_qkv_rope_append(self, x16: torch.Tensor, w_paired: torch.Tensor, bias_paired: Optional[torch.Tensor],
                             norm_w: torch.Tensor, eps: float, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                             batch: StepBatch, kv: PagedKVView, q_out: torch.Tensor, num_heads: int) -> None:
        """The q/k/v projection of rmsnorm(x16) with bias, rotation and append: `qkv_rope_append` after `linear` after the
        norm, in one launch.  `w_paired` / `bias_paired`: rows permuted within each head so that rows 16 j + i and
        16 j + 8 + i (i < 8) are dimensions 8 j + i and D / 2 + 8 j + i (see `pair_rotation_rows`)."""
        M, K = x16.shape
        spec = kv.spec
        if cos is not None and cos.shape[1] * 2 != spec.head_dim:
            raise KernelError("the folded q/k/v projection rotates whole heads only")
        self._count("gemm_skinny_qkv")
        _check(self._gemm_skinny.kvb_gemm_skinny_qkv(
            _ptr(x16), _ptr(w_paired), _ptr(bias_paired), _ptr(norm_w), float(eps), _ptr(cos), _ptr(sin),
            0 if cos is None else cos.shape[0], _ptr(batch.positions), _ptr(batch.row_segment), _ptr(kv.block_table),
            kv.block_table.shape[1], _ptr(kv.k_pages), _ptr(kv.v_pages), _ptr(q_out), M, K, num_heads, spec.num_kv_heads,
            spec.head_dim, kv.page_size, 1 if kv.writes else 0, _ptr(self.error_word), self._stream()), "norm_qkv_rope_append")

    @staticmethod
    def pair_rotation_rows(num_heads_total: int, head_dim: int) -> torch.Tensor:
        """The row order `norm_qkv_rope_append` wants: for every head, tiles of 16 rows holding dimensions
        8 j .. 8 j + 7 and D / 2 + 8 j .. D / 2 + 8 j + 7.  Returns the source row of each row of the permuted matrix."""
        half = head_dim // 2
        within = torch.cat([torch.cat([torch.arange(8 * j, 8 * j + 8), torch.arange(half + 8 * j, half + 8 * j + 8)])
                            for j in range(head_dim // 16)])
        return (torch.arange(num_heads_total)[:, None] * head_dim + within[None, :]).reshape(-1)

    def add_rmsnorm(self, h: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                    out: torch.Tensor, rows: Optional[torch.Tensor] = None, delta_scale: Optional[torch.Tensor] = None) -> None:
        """`delta_scale` (float32 [H]): delta is multiplied by it, channel by channel, before the add."""
        n_out, H = out.shape
        if delta_scale is not None and (delta_scale.dtype != torch.float32 or delta_scale.numel() != H):
            raise KernelError("add_rmsnorm: the delta's scale is one float32 number per channel")
        self._count("add_rmsnorm")
        _check(self._elementwise.kvb_add_rmsnorm(_dtype_code(out.dtype), _ptr(h), _ptr(delta), _ptr(delta_scale if delta is not None else None),
                                                 _ptr(weight), _ptr(out), _ptr(rows), n_out, H, float(eps), self._stream()),
               "add_rmsnorm")

    GATED_ACTIVATIONS = {"silu": 0, "clamped_swiglu": 1}

    def silu_mul(self, gate_up: torch.Tensor, out: torch.Tensor, interleaved: bool = False, activation: str = "silu",
                 limit: float = 0.0) -> None:
        """out = act(gate, up) of the two halves (or interleaved eights) of `gate_up`: "silu": silu(g) u;
        "clamped_swiglu": g' sigmoid(1.702 g') (u' + 1), g' = min(g, limit), u' = clamp(u, -limit, limit)."""
        T, I = out.shape
        self._count("silu_mul")
        if activation == "silu":
            _check(self._elementwise.kvb_silu_mul(_dtype_code(out.dtype), _ptr(gate_up), _ptr(out), T, I,
                                                  1 if interleaved else 0, self._stream()), "silu_mul")
            return
        if activation not in self.GATED_ACTIVATIONS:
            raise KernelError(f"silu_mul: activation '{activation}' is not built")
        _check(self._elementwise.kvb_gated_act(_dtype_code(out.dtype), _ptr(gate_up), _ptr(out), T, I, 1 if interleaved else 0,
                                               self.GATED_ACTIVATIONS[activation], float(limit), self._stream()), "gated_act")

    def gate_up_act(self, x: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor, workspace, interleaved: bool,
                    activation: str = "silu", limit: float = 0.0) -> None:
        """out[M, I] = act(x Wg^T, x Wu^T) (see `silu_mul`); `w_gate_up` [2 I, K] holds gate and up rows one after the
        other, or interleaved in eights (see csrc/gemm_skinny.cu).  The clamped activation is in the epilogue of the two
        weight-streaming products (steps of few rows); with more rows it takes the product and the activation kernel."""
        M, K = x.shape
        I = out.shape[1]
        if activation != "silu":
            if activation != "clamped_swiglu" or not limit > 0.0:
                raise KernelError(f"gate_up_act: activation '{activation}' (limit {limit}) is not built")
            if interleaved and self._skinny(x.dtype, M, K, 2 * I):
                self._count("gemm_skinny")
                _check(self._gemm_skinny.kvb_gemm_skinny_gated(_dtype_code(out.dtype), _ptr(x), _ptr(w_gate_up), _ptr(out), M, 2 * I, K,
                                                               float(limit), self._stream()), "gate_up_act (skinny, clamped)")
                return
            if interleaved and self._wstream(x.dtype, M, K):
                self._count("gemm_wstream")
                _check(self._gemm_ws.kvb_gemm_wstream_gated(_dtype_code(out.dtype), _ptr(x), _ptr(w_gate_up), _ptr(out), M, 2 * I, K,
                                                            float(limit), _ptr(self.error_word), self._stream()),
                       "gate_up_act (wstream, clamped)")
                return
            gate_up = workspace.buffer("ffn.gate_up", (M, 2 * I), out.dtype)
            self.linear(x, w_gate_up, gate_up)
            self.silu_mul(gate_up, out, interleaved, activation, limit)
            return
        if interleaved and self._skinny(x.dtype, M, K, 2 * I):
            self._count("gemm_skinny")
            _check(self._gemm_skinny.kvb_gemm_skinny(_dtype_code(out.dtype), 1, _ptr(x), _ptr(w_gate_up), _ptr(None),
                                                     _ptr(out), M, 2 * I, K, self._stream()), "gate_up_act (skinny)")
            return
        if interleaved and self._wstream(x.dtype, M, K):
            self._count("gemm_wstream")
            _check(self._gemm_ws.kvb_gemm_wstream(_dtype_code(out.dtype), 1, _ptr(x), _ptr(w_gate_up), _ptr(None), _ptr(out), M,
                                                  2 * I, K, _ptr(self.error_word), self._stream()), "gate_up_act (wstream)")
            return
        if interleaved and self._tcgen05(x, w_gate_up, out, fused=True):
            self._count("gemm_tcgen05")
            _check(self._gemm_tc.kvb_gemm_tcgen05(_dtype_code(out.dtype), 1, _ptr(x), _ptr(w_gate_up), _ptr(None), _ptr(out), M,
                                                  2 * I, K, _ptr(self.error_word), self._stream()), "gate_up_act (tcgen05)")
            return
        gate_up = workspace.buffer("ffn.gate_up", (M, 2 * I), out.dtype)
        self.linear(x, w_gate_up, gate_up)
        self.silu_mul(gate_up, out, interleaved)

    SKINNY_MAX_ROWS = 16     # above this the weight-streaming tcgen05 product takes over
    WSTREAM_MAX_ROWS = 32    # measured on 24 layers of the 0.5B shape: 11 % faster steps than the library at 17 and 32 rows, equal at 40, slower at 128

    # Products with K >= 4 N (the feed-forward's way down) up to this many rows: the library splits K too little for
    # them - 8.4 us against 5.8 at 64 x 896 x 4864; steps of 40, 48 and 64 requests are 4 % faster for it.
    WSTREAM_DEEP_MAX_ROWS = 64

    def _wstream(self, dtype: torch.dtype, M: int, K: int, N: int = 0) -> bool:
        rows = self.WSTREAM_DEEP_MAX_ROWS if K >= 4 * N > 0 else self.WSTREAM_MAX_ROWS
        return self.wstream_gemm and dtype == torch.bfloat16 and self.bf16_gemm == "auto" and M <= rows and K % 8 == 0

    # Weights of at least this many bytes go through the weight-streaming tcgen05 kernel at any number of rows up to its
    # limit: TMA keeps more bytes in flight per SM than register loads do.  Measured at 8 rows: the 7B model's gate/up
    # (272 MB) 45 against 64 us, its way down (136 MB) 25 against 40 us, output heads (272 MB .. 1.1 GB) at 6.6-7.0
    # against 5.1-6.0 TB/s; below it the register kernel is ahead (1.5B gate/up, 55 MB: 10.5 against 13.2 us).
    WSTREAM_MIN_WEIGHT_BYTES = 96 << 20

    def _skinny(self, dtype: torch.dtype, M: int, K: int, N: int = 0) -> bool:
        if 2 * N * K >= self.WSTREAM_MIN_WEIGHT_BYTES and self._wstream(dtype, M, K, N):
            return False
        return self.skinny_gemm and dtype == torch.bfloat16 and M <= self.SKINNY_MAX_ROWS and K % 32 == 0

    def _tcgen05(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, fused: bool = False) -> bool:
        """The tensor-memory kernel takes bfloat16 operands whose rows are multiples of 16 bytes."""
        if x.dtype != torch.bfloat16 or w.shape[1] % 8 != 0 or (x.data_ptr() | w.data_ptr() | out.data_ptr()) % 16 != 0:
            return False
        if self.bf16_gemm == "auto":
            return fused and -(-x.shape[0] // 256) * -(-w.shape[0] // 256) >= self.sm_count
        return self.bf16_gemm == "tcgen05"

    def linear(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None) -> None:
        """out = x . w^T + bias."""
        M = x.shape[0]
        N, K = w.shape
        if x.shape[1] != K or tuple(out.shape) != (M, N):
            raise KernelError(f"linear: shapes x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)} do not fit")
        if self._skinny(x.dtype, M, K, N):
            self._count("gemm_skinny")
            _check(self._gemm_skinny.kvb_gemm_skinny(_dtype_code(out.dtype), 0, _ptr(x), _ptr(w), _ptr(bias),
                                                     _ptr(out), M, N, K, self._stream()), "linear (skinny)")
            return
        if self._wstream(x.dtype, M, K, N):
            self._count("gemm_wstream")
            _check(self._gemm_ws.kvb_gemm_wstream(_dtype_code(out.dtype), 0, _ptr(x), _ptr(w), _ptr(bias), _ptr(out), M, N, K,
                                                  _ptr(self.error_word), self._stream()), "linear (wstream)")
            return
        if self._tcgen05(x, w, out):
            self._count("gemm_tcgen05")
            _check(self._gemm_tc.kvb_gemm_tcgen05(_dtype_code(out.dtype), 0, _ptr(x), _ptr(w), _ptr(bias), _ptr(out), M, N, K,
                                                  _ptr(self.error_word), self._stream()), "linear (tcgen05)")
            return
        if x.dtype == torch.bfloat16 and self.bf16_gemm != "simt":
            # Library matrix product, as the reference's cublasGemmEx (apps/qwen_serve.cu:27-39).
            self._count("gemm_library")
            if out.dtype == torch.bfloat16:
                torch.matmul(x, w.t(), out=out)
            else:
                torch.mm(x, w.t(), out_dtype=torch.float32, out=out)
            if bias is not None:
                out.add_(bias)
            return
        self._count("gemm_simt")
        _check(self._gemm_simt.kvb_gemm_simt(_dtype_code(x.dtype), _dtype_code(out.dtype), _ptr(x), _ptr(w),
                                             _ptr(bias), _ptr(out), M, N, K, self._stream()), "linear")

    def qkv_rope_append(self, qkv: torch.Tensor, bias: Optional[torch.Tensor], cos: Optional[torch.Tensor],
                        sin: Optional[torch.Tensor], batch: StepBatch, kv: PagedKVView, q_out: torch.Tensor,
                        num_heads: int, q_norm: Optional[torch.Tensor] = None, k_norm: Optional[torch.Tensor] = None,
                        norm_eps: float = 0.0, key_dim: Optional[int] = None, norm_scope: str = "head",
                        norm_after_rotation: bool = False, value_mix=None, q_temperature=None, value_dim: Optional[int] = None) -> None:
        """`q_norm` / `k_norm` (float32 [key_dim]): queries and keys are divided by their root mean square per head and
        multiplied by these before the rotation.  `norm_eps` > 0 without weights: the division alone.  `norm_scope` "all":
        the root mean square runs over a row's whole query (key) projection and the weights have that size.
        `norm_after_rotation`: the norm follows the rotation (per head only).  `value_mix` = (kept [T, Hkv * Dv], lam):
        lam None - the row's values are also written to `kept`; else v = (1 - lam[0]) v + lam[0] kept[r] before the cache.  Values may have another size than keys (`kv.spec.v_head_dim`), and rows
        of `qkv` may carry further columns after [q | k | v].  `key_dim` < `kv.spec.head_dim`: queries and keys have
        `key_dim` numbers in `qkv` and are stored `kv.spec.head_dim` wide, with zeros after them.  `value_dim` <
        `kv.spec.v_head_dim`: likewise for the values.  `q_temperature` = (coef, every): the queries of a row at position p are
        multiplied by 1 + coef ln(floor((p + 1) / every) + 1)."""
        T = qkv.shape[0]
        spec = kv.spec
        rot_half = 0 if cos is None else cos.shape[1]
        table_len = 0 if cos is None else cos.shape[0]
        D = spec.head_dim if key_dim is None else int(key_dim)
        normed = q_norm is not None or norm_eps > 0.0
        Dv = spec.v_head_dim if value_dim is None else int(value_dim)
        qt_coef, qt_every = q_temperature if q_temperature is not None else (0.0, 0)
        if (normed or value_mix is not None or spec.v_head_dim != spec.head_dim or D != spec.head_dim or Dv != spec.v_head_dim
                or q_temperature is not None or qkv.shape[1] != (num_heads + 2 * spec.num_kv_heads) * spec.head_dim):
            flags = (1 if normed else 0) | (2 if normed and norm_scope == "all" else 0) | (4 if normed and norm_after_rotation else 0)
            kept, lam = value_mix if value_mix is not None else (None, None)
            mix_mode = 0 if value_mix is None else (1 if lam is None else 2)
            if kept is not None and (kept.dtype != qkv.dtype or kept.shape != (T, spec.num_kv_heads * Dv)):
                raise KernelError("qkv_rope_append: the kept values do not fit the step's rows")
            self._count("norm_rope_append")
            _check(self._rope.kvb_qkv_norm_rope_append(
                _dtype_code(qkv.dtype), _ptr(qkv), qkv.shape[1], _ptr(bias), _ptr(q_norm), _ptr(k_norm), float(norm_eps), flags,
                _ptr(cos), _ptr(sin), rot_half, table_len, _ptr(batch.positions), _ptr(batch.row_segment), _ptr(kv.block_table),
                kv.block_table.shape[1], _ptr(kv.k_pages), _ptr(kv.v_pages), _ptr(q_out), T, num_heads, spec.num_kv_heads,
                D, Dv, spec.head_dim, kv.page_size, 1 if kv.writes else 0, mix_mode, _ptr(kept), _ptr(lam), spec.v_head_dim,
                float(qt_coef), int(qt_every), _ptr(self.error_word), self._stream()), "qkv_norm_rope_append")
            return
        self._count("rope_append")
        _check(self._rope.kvb_qkv_rope_append(
            _dtype_code(qkv.dtype), _ptr(qkv), _ptr(bias), _ptr(cos), _ptr(sin), rot_half, table_len,
            _ptr(batch.positions), _ptr(batch.row_segment), _ptr(kv.block_table), kv.block_table.shape[1],
            _ptr(kv.k_pages), _ptr(kv.v_pages), _ptr(q_out), T, num_heads, spec.num_kv_heads, spec.head_dim,
            kv.page_size, 1 if kv.writes else 0, _ptr(self.error_word), self._stream()), "qkv_rope_append")

    def _tma_clusters(self, lib, head_dim: int, nsplit: int) -> int:
        key = (head_dim, nsplit)
        found = self._tma_cluster_capacity.get(key)
        if found is None:
            found = int(lib.kvb_flash_decode_tma_max_clusters(nsplit)) or 1 << 30     # unknown: no limit
            self._tma_cluster_capacity[key] = found
        return found

    def _flash_library(self, head_dim: int) -> _Library:
        lib = self._flash.get(head_dim)
        if lib is None:
            lib = _Library("attention_flash", f"d{head_dim}", [f"-DKVB_HEAD_DIM={head_dim}"])
            self._flash[head_dim] = lib
        return lib

    def _cluster_splits(self, n: int, Hkv: int, tiles: int) -> int:
        nsplit = max(1, min(self.decode_cluster_max, self.decode_ctas_wanted // (n * Hkv), tiles // self.decode_min_tiles))
        if self.decode_pow2_splits:
            nsplit = 1 << (nsplit.bit_length() - 1)     # clusters of 3, 5, 6, 7 blocks place badly
        return nsplit

    def _tma_decode(self, D: int, kv: PagedKVView) -> bool:
        return self.decode_merge == "tma" and D % 64 == 0 and 8 <= kv.page_size <= 64

    def _fit_clusters(self, lib, D: int, clusters: int, nsplit: int) -> int:
        # All clusters at once: a grid with more clusters than the GPU holds runs in waves.
        while nsplit > 1 and clusters > self._tma_clusters(lib, D, nsplit):
            nsplit //= 2
        return nsplit

    def rope_append_attention(self, qkv: torch.Tensor, bias: Optional[torch.Tensor], cos: Optional[torch.Tensor],
                              sin: Optional[torch.Tensor], batch: StepBatch, kv: PagedKVView, out: torch.Tensor,
                              num_heads: int, scale: float, workspace=None) -> bool:
        """`qkv_rope_append` and `paged_attention` in one launch, where one kernel does both: a step in which every
        request brings one token, bfloat16, through the TMA decode kernel, into a cache that this call writes.  Returns
        False (and does nothing) otherwise; the caller then makes the two calls."""
        spec = kv.spec
        D, Hkv, n = spec.head_dim, spec.num_kv_heads, batch.num_segments
        plan = batch.plans.get(PagedAttentionPlanner.name)
        if not (self.fused_rope_min_requests is not None and n >= self.fused_rope_min_requests
                and self.flash_attention and qkv.dtype == torch.bfloat16 and kv.writes and plan is not None
                and batch.num_tokens == n and plan.counts["decode_items"] == n and num_heads // Hkv <= 16
                and self._tma_decode(D, kv) and (cos is None or cos.shape[1] <= D // 2)
                and not (spec.window and spec.keep_first) and spec.v_head_dim == D):
            return False
        lib = self._flash_library(D)
        tiles = -(-(kv.block_table.shape[1] * kv.page_size) // 64)
        nsplit = self._fit_clusters(lib, D, n * Hkv, self._cluster_splits(n, Hkv, tiles))
        self._count("flash_decode_tma_fused")
        _check(lib.kvb_flash_decode_tma(
            None, _ptr(out), _ptr(kv.k_pages), _ptr(kv.v_pages), kv.k_pages.shape[0], _ptr(kv.block_table),
            kv.block_table.shape[1], None, n, _ptr(batch.seg_q_start), _ptr(batch.seg_q_len), _ptr(batch.seg_kv_len),
            num_heads, Hkv, kv.page_size, spec.window or 0, nsplit, float(scale), _ptr(qkv), _ptr(bias), _ptr(cos), _ptr(sin),
            0 if cos is None else cos.shape[1], 0 if cos is None else cos.shape[0], 1, None, None, None, 0, None, 0.0, _ptr(self.error_word),
            self._stream()), "flash_decode_tma (rotation and append fused)")
        return True

    def paged_attention(self, q: torch.Tensor, batch: StepBatch, kv: PagedKVView, out: torch.Tensor,
                        num_heads: int, scale: float, workspace=None, sink: Optional[torch.Tensor] = None,
                        score_cap: Optional[float] = None, slopes: Optional[torch.Tensor] = None) -> None:
        """`sink` (float32 [num_heads]): the softmax's denominator also holds exp(sink[h]), a key without a value.
        `kv.spec.keep_first` (with a window): the request's first keys stay visible to every later query.
        `score_cap`: a score (after the scale) becomes cap tanh(score / cap).  `slopes` (float32 [num_heads]): a key i - j
        tokens back then loses slopes[h] (i - j)."""
        T = q.shape[0]
        spec = kv.spec
        D, Hkv = spec.head_dim, spec.num_kv_heads
        plan = batch.plans.get(PagedAttentionPlanner.name)
        keep = spec.keep_first if spec.window else 0
        fast = (self.flash_attention and q.dtype == torch.bfloat16 and spec.v_head_dim == D and D % 16 == 0 and D <= 128
                and num_heads // Hkv <= 16 and workspace is not None and plan is not None)
        # Capped or biased scores: the tensor-core kernels (all but the cluster decode kernel without TMA) make the whole score
        # in their softmax step where a row's heads have slopes; a cap alone comes with slopes of zero.
        biased = score_cap is not None or slopes is not None
        cap = float(score_cap or 0.0)
        if biased and slopes is None:
            slopes = self._zero_slopes.get(num_heads)
            if slopes is None:
                slopes = self._zero_slopes[num_heads] = torch.zeros(num_heads, dtype=torch.float32, device=self.device)
        if biased and not fast:
            self._count("attention_generic")
            _check(self._attn_generic.kvb_paged_attention_ext(
                _dtype_code(q.dtype), _ptr(q), _ptr(kv.k_pages), _ptr(kv.v_pages), _ptr(kv.block_table), kv.block_table.shape[1],
                _ptr(batch.positions), _ptr(batch.row_segment), _ptr(out), T, num_heads, Hkv, D, spec.v_head_dim, kv.page_size,
                spec.window or 0, keep, _ptr(sink), float(scale), cap, _ptr(slopes), _ptr(self.error_word), self._stream()),
                "paged_attention")
            return
        # The cluster decode kernel knows neither a sink nor kept first keys nor biased scores: with them, and where the TMA
        # kernel does not apply, single tokens go through the kernel whose splits meet in scratch.
        plain_decode = self.decode_merge not in ("cluster", "tma") or ((sink is not None or keep or biased) and not self._tma_decode(D, kv))
        if (sink is not None or keep) and not fast:
            self._count("attention_sink")
            _check(self._attn_generic.kvb_paged_attention_sink(
                _dtype_code(q.dtype), _ptr(q), _ptr(kv.k_pages), _ptr(kv.v_pages), _ptr(kv.block_table), kv.block_table.shape[1],
                _ptr(batch.positions), _ptr(batch.row_segment), _ptr(out), T, num_heads, Hkv, D, spec.v_head_dim, kv.page_size,
                spec.window or 0, spec.keep_first if spec.window else 0, _ptr(sink), float(scale), _ptr(self.error_word),
                self._stream()), "paged_attention")
            return
        if spec.v_head_dim != D:
            # Values of another size than keys: the generic kernel, which takes any two sizes.
            self._count("attention_generic")
            _check(self._attn_generic.kvb_paged_attention_kv(
                _dtype_code(q.dtype), _ptr(q), _ptr(kv.k_pages), _ptr(kv.v_pages), _ptr(kv.block_table), kv.block_table.shape[1],
                _ptr(batch.positions), _ptr(batch.row_segment), _ptr(out), T, num_heads, Hkv, D, spec.v_head_dim, kv.page_size,
                spec.window or 0, float(scale), _ptr(self.error_word), self._stream()), "paged_attention")
            return
        if fast:
            lib = self._flash_library(D)
            counts, lists = plan.counts, plan.arrays
            if (counts["tc_units"] and self.tc_attention_min_rows is not None and D in (64, 128)
                    and 8 <= kv.page_size <= 64 and batch.max_q_len >= self.tc_attention_min_rows):
                tc = self._attn_tc.get(D)
                if tc is None:
                    tc = self._attn_tc[D] = _Library("attention_tc", f"d{D}", [f"-DKVB_HEAD_DIM={D}"])
                units = counts["tc_units"]
                scratch = workspace.buffer("attn.tc_scratch", (units * num_heads * 128 * (D + 2),), torch.float32)
                # Two counters of the kernel's work queue, then a ticket per (tile, head); the kernel leaves all of them zero.
                tickets = workspace.zeros("attn.tc_tickets", (2 + max(counts["tc_tiles"], 1) * num_heads,), torch.int32)
                self._count("attention_tc")
                _check(tc.kvb_attention_tc(
                    _ptr(q), _ptr(out), _ptr(kv.k_pages), _ptr(kv.v_pages), kv.k_pages.shape[0], _ptr(kv.block_table),
                    kv.block_table.shape[1], _ptr(lists["tc_units"]), units, _ptr(scratch), _ptr(tickets),
                    _ptr(batch.seg_q_start), _ptr(batch.seg_q_len), _ptr(batch.seg_kv_len), T, num_heads, Hkv, kv.page_size,
                    spec.window or 0, float(scale), _ptr(sink), keep, _ptr(slopes), cap, _ptr(self.error_word), self._stream()),
                    "attention_tc")
            elif counts["prefill_units"]:
                units = counts["prefill_units"]
                scratch = workspace.buffer("attn.prefill_scratch", (units * num_heads * 64 * (D + 2),), torch.float32)
                tickets = workspace.zeros("attn.prefill_tickets", (max(counts["prefill_tiles"], 1) * num_heads,), torch.int32)
                self._count("flash_prefill")
                _check(lib.kvb_flash_prefill(
                    _ptr(q), _ptr(out), _ptr(kv.k_pages), _ptr(kv.v_pages), _ptr(kv.block_table), kv.block_table.shape[1],
                    _ptr(lists["prefill_units"]), units, _ptr(batch.seg_q_start), _ptr(batch.seg_q_len),
                    _ptr(batch.seg_kv_len), _ptr(scratch), _ptr(tickets), num_heads, Hkv, kv.page_size, spec.window or 0,
                    float(scale), _ptr(sink), keep, _ptr(slopes), cap, self._stream()), "flash_prefill")
            n = counts["decode_items"]
            items = lists["decode_items"]
            if n:
                # Sized by the longest request the block table allows, not by this step's lengths, so that the
                # split (and with it the rounding) is the same in every step and under a CUDA graph.
                tiles = -(-(kv.block_table.shape[1] * kv.page_size) // 64)
                if not plain_decode:
                    nsplit = self._cluster_splits(n, Hkv, tiles)
                    if self._tma_decode(D, kv):
                        self._count("flash_decode_tma")
                        # Few requests with many keys: several clusters for each (request, kv head), each with a run of
                        # the keys, so that the whole GPU streams them; their sums meet in scratch, the last to finish
                        # adds them in cluster order.  Like the split itself this follows from the block table's
                        # capacity and the number of requests, never from the lengths of the moment.
                        nsuper = 1
                        if nsplit > 1 and self.decode_superclusters:
                            nsuper = max(1, min(self.decode_superclusters, self.sm_count // (n * Hkv * nsplit),
                                                tiles // (max(self.decode_min_tiles, self.decode_super_min_tiles) * nsplit)))
                            while nsuper > 1 and n * Hkv * nsuper > self._tma_clusters(lib, D, nsplit):
                                nsuper -= 1
                        nsplit = self._fit_clusters(lib, D, n * Hkv * nsuper, nsplit)
                        if nsplit == 1:
                            nsuper = 1
                        scratch = tickets = None
                        if nsuper > 1:
                            scratch = workspace.buffer("attn.decode_super", (n * Hkv * nsuper * 16 * (D + 2),), torch.float32)
                            tickets = workspace.zeros("attn.decode_super_tickets", (n * Hkv * 8,), torch.int32)
                        _check(lib.kvb_flash_decode_tma(
                            _ptr(q), _ptr(out), _ptr(kv.k_pages), _ptr(kv.v_pages), kv.k_pages.shape[0],
                            _ptr(kv.block_table), kv.block_table.shape[1],
                            _ptr(None if n == batch.num_segments else items), n,   # every segment, in order: no list
                            _ptr(batch.seg_q_start), _ptr(batch.seg_q_len), _ptr(batch.seg_kv_len), num_heads, Hkv,
                            kv.page_size, spec.window or 0, nsplit, float(scale), None, None, None, None, 0, 0,
                            nsuper, _ptr(scratch), _ptr(tickets), _ptr(sink), keep, _ptr(slopes), cap, _ptr(self.error_word),
                            self._stream()), "flash_decode_tma")
                        return
                    self._count("flash_decode_cluster")
                    _check(lib.kvb_flash_decode_cluster(
                        _ptr(q), _ptr(out), _ptr(kv.k_pages), _ptr(kv.v_pages), _ptr(kv.block_table),
                        kv.block_table.shape[1], _ptr(items), n, _ptr(batch.seg_q_start),
                        _ptr(batch.seg_q_len), _ptr(batch.seg_kv_len), num_heads, Hkv, kv.page_size, spec.window or 0,
                        nsplit, float(scale), self._stream()), "flash_decode_cluster")
                    return
                nsplit = max(1, min(32, 2 * self.decode_ctas_wanted // (n * Hkv), tiles // self.decode_min_tiles))
                scratch = workspace.buffer("attn.decode_scratch", (n * Hkv * nsplit * 16 * (D + 2),), torch.float32)
                tickets = workspace.zeros("attn.decode_tickets", (n * Hkv,), torch.int32)
                self._count("flash_decode_ticket")
                _check(lib.kvb_flash_decode(
                    _ptr(q), _ptr(out), _ptr(kv.k_pages), _ptr(kv.v_pages), _ptr(kv.block_table), kv.block_table.shape[1],
                    _ptr(items), n, _ptr(batch.seg_q_start), _ptr(batch.seg_q_len), _ptr(batch.seg_kv_len),
                    _ptr(scratch), _ptr(tickets), num_heads, Hkv, kv.page_size, spec.window or 0, nsplit, float(scale),
                    _ptr(sink), keep, _ptr(slopes), cap, self._stream()), "flash_decode")
            return
        self._count("attention_generic")
        _check(self._attn_generic.kvb_paged_attention_generic(
            _dtype_code(q.dtype), _ptr(q), _ptr(kv.k_pages), _ptr(kv.v_pages), _ptr(kv.block_table),
            kv.block_table.shape[1], _ptr(batch.positions), _ptr(batch.row_segment), _ptr(out), T, num_heads,
            spec.num_kv_heads, spec.head_dim, kv.page_size, spec.window or 0, float(scale),
            _ptr(self.error_word), self._stream()), "paged_attention")

    # ---- latent attention, normalised adds, routed feed-forward ----------------------------------------------
    def norm_add_rmsnorm(self, h: torch.Tensor, delta: Optional[torch.Tensor], delta_weight: Optional[torch.Tensor],
                         delta_eps: float, weight: Optional[torch.Tensor], eps: float, out: Optional[torch.Tensor],
                         rows: Optional[torch.Tensor] = None, tail: Optional[torch.Tensor] = None,
                         delta_gate: Optional[torch.Tensor] = None) -> None:
        """v = h + (delta_weight given: rmsnorm(delta; delta_weight, delta_eps), else delta); without `rows`, h = v.
        `delta_gate` (rows like delta): delta is first multiplied by sigmoid(delta_gate), element by element.
        out[:, :H] = rmsnorm(v; weight, eps), or v itself if `weight` is None; out[:, H:] = tail (float32 rows like h)
        in out's type.  `rows`: only these rows, gathered into out, h untouched.  `out` None: only the add."""
        if delta is None and out is None:
            return
        n, H = (out.shape[0] if out is not None else h.shape[0]), h.shape[1]
        if out is not None and out.shape[1] != (2 * H if tail is not None else H):
            raise KernelError(f"norm_add_rmsnorm: out{tuple(out.shape)} does not fit rows of {H}")
        dtype = out.dtype if out is not None else delta.dtype
        if delta is not None and delta.dtype != dtype:
            raise KernelError("norm_add_rmsnorm: delta and out differ in type")
        if delta_gate is not None and (delta is None or delta_gate.dtype != delta.dtype or delta_gate.shape != delta.shape):
            raise KernelError("norm_add_rmsnorm: the gate does not fit the delta")
        self._count("norm_add_rmsnorm")
        _check(self._latent.kvb_norm_add_rmsnorm(_dtype_code(dtype), _ptr(h), _ptr(delta), _ptr(delta_gate), _ptr(delta_weight), float(delta_eps),
                                                 _ptr(weight), float(eps), _ptr(out), _ptr(rows), _ptr(tail), n, H, self._stream()),
               "norm_add_rmsnorm")

    def latent_norm_rope_append(self, proj: torch.Tensor, q_rank: int, kv_rank: int, rot_dim: int, q_weight: Optional[torch.Tensor],
                                kv_weight: torch.Tensor, eps: float, cos: torch.Tensor, sin: torch.Tensor, batch: StepBatch,
                                kv: PagedKVView, cq_out: Optional[torch.Tensor], kv_col: Optional[int] = None) -> None:
        """cq_out = rmsnorm(proj[:, :q_rank]; q_weight) (q_rank 0: no query latent); if kv.writes, the cache row of every
        row's (request, position) = [rmsnorm(proj[:, kv_col:kv_col + kv_rank]; kv_weight) | the next rot_dim columns rotated
        by the position]; `kv_col` None: right after the query latent."""
        T, P = proj.shape
        kv_col = q_rank if kv_col is None else int(kv_col)
        if kv.spec.head_dim != kv_rank + rot_dim or kv.spec.num_kv_heads != 1:
            raise KernelError("latent_norm_rope_append: the cache entry is not one row of kv_rank + rot_dim numbers per token")
        self._count("latent_norm_rope_append")
        _check(self._latent.kvb_latent_norm_rope_append(
            _dtype_code(proj.dtype), _ptr(proj), P, q_rank, kv_col, kv_rank, rot_dim, _ptr(q_weight), _ptr(kv_weight), float(eps),
            _ptr(cos), _ptr(sin), cos.shape[1], cos.shape[0], _ptr(batch.positions), _ptr(batch.row_segment),
            _ptr(kv.block_table), kv.block_table.shape[1], _ptr(kv.k_pages), kv.page_size, 1 if kv.writes else 0, _ptr(cq_out),
            T, _ptr(self.error_word), self._stream()), "latent_norm_rope_append")

    def head_linear(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, rotate=None, gate=None, x_col: Optional[int] = None,
                    gate_per_head: bool = False) -> None:
        """One product per head: with H, N, K = w.shape, xs = x.shape[1] / H, os = out.shape[1] / H,
        out[t, h * os + n] = sum_k x[t, h * xs + k] * w[h, n, k].
        `rotate` = (cos, sin, positions): the xs - K trailing columns of each head of x, rotated by the row's position
        (first 2 * cos.shape[1] of them, pair (i, i + cos.shape[1])), go to out[t, h * os + N:].
        `gate` = (g, col): out *= sigmoid(g[t, col + h * os + n]), or, with `gate_per_head`, sigmoid(g[t, col + h]).
        `x_col`: the heads' inputs are the columns x_col .. x_col + H * xs of the wider rows of `x` (xs = K, plus the
        rotated columns if `rotate`)."""
        T = x.shape[0]
        H, N, K = w.shape
        os_ = out.shape[1] // H
        if x_col is None:
            xs, x_col = x.shape[1] // H, 0
            fits = xs * H == x.shape[1]
        else:
            xs = K + (os_ - N if rotate is not None else 0)
            fits = 0 <= x_col and x_col + H * xs <= x.shape[1]
        rot = xs - K if rotate is not None else 0
        if not fits or os_ * H != out.shape[1] or out.shape[0] != T or os_ != N + rot or xs < K:
            raise KernelError(f"head_linear: shapes x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)} do not fit")
        cos, sin, positions = rotate if rotate is not None else (None, None, None)
        g, col = gate if gate is not None else (None, 0)
        if g is not None and (g.shape[0] != T or col + (H if gate_per_head else H * os_) > g.shape[1] or g.dtype != x.dtype):
            raise KernelError("head_linear: the gate does not fit")
        self._count("head_linear")
        x_first = _c_void_p(x.data_ptr() + x_col * x.element_size()) if x_col else _ptr(x)
        _ptr(x)                                                    # the checks of a device tensor
        _check(self._latent.kvb_head_linear(
            _dtype_code(x.dtype), x_first, xs, x.shape[1], _ptr(w), _ptr(out), os_, T, N, K, H, _ptr(g), 0 if g is None else g.shape[1],
            col, 1 if gate_per_head else 0, rot, 0 if cos is None else cos.shape[1], _ptr(cos), _ptr(sin),
            0 if cos is None else cos.shape[0], _ptr(positions), _ptr(self.error_word), self._stream()), "head_linear")

    def latent_attention(self, q: torch.Tensor, batch: StepBatch, kv: PagedKVView, out: torch.Tensor, num_heads: int,
                         value_dim: int, scale: float, workspace=None, window: Optional[int] = -1,
                         sink: Optional[torch.Tensor] = None) -> None:
        """Causal softmax(scale * q . key) over the rows of a cache entry with one key row per token that all heads
        share; a row's value is the first `value_dim` numbers of its key.  q [T, H * key_dim], out [T, H * value_dim].
        `window` (-1: the cache entry's own): a query sees its own key and the window - 1 before it; a layer that reads
        another's cache entry may see less than the entry keeps.  `sink` (float32 [H]): the softmax's denominator also holds
        exp(sink[h]), a key without a value."""
        T = q.shape[0]
        spec = kv.spec
        window = spec.window if window == -1 else window
        if spec.window and (not window or window > spec.window):
            raise KernelError(f"latent_attention: a window of {window} over a cache entry that keeps {spec.window} keys")
        plan = batch.plans.get(LatentAttentionPlanner.plan_name(num_heads, *self._latent_plan_shape(spec.head_dim, value_dim),
                                                                int(window or 0)))
        if (self.latent_flash and q.dtype == torch.bfloat16 and plan is not None and workspace is not None and spec.num_kv_heads == 1
                and self._latent_flash.kvb_latent_flash_supports(spec.head_dim, value_dim, plan.counts["bm"]) == 0):
            n, tiles, nsplit, bm = (plan.counts[k] for k in ("items", "tiles", "nsplit", "bm"))
            part_o = part_ml = None
            if nsplit > 1:
                part_o = workspace.buffer("latent.part_o", (n * bm * value_dim,), torch.float32)
                part_ml = workspace.buffer("latent.part_ml", (n * bm * 2,), torch.float32)
            self._count("latent_flash")
            _check(self._latent_flash.kvb_latent_flash(
                _ptr(q), _ptr(out), _ptr(kv.k_pages), _ptr(kv.block_table), kv.block_table.shape[1], _ptr(plan.arrays["items"]), n,
                tiles, _ptr(batch.seg_q_start), _ptr(batch.seg_q_len), _ptr(batch.seg_kv_len), _ptr(part_o), _ptr(part_ml),
                num_heads, spec.head_dim, value_dim, bm, kv.page_size, window or 0, float(scale), nsplit, _ptr(sink),
                _ptr(self.error_word), self._stream()), "latent_flash")
            return
        self._count("attention_generic")
        _check(self._attn_generic.kvb_paged_attention_ext(
            _dtype_code(q.dtype), _ptr(q), _ptr(kv.k_pages), None, _ptr(kv.block_table), kv.block_table.shape[1],
            _ptr(batch.positions), _ptr(batch.row_segment), _ptr(out), T, num_heads, spec.num_kv_heads, spec.head_dim, value_dim,
            kv.page_size, window or 0, 0, _ptr(sink), float(scale), 0.0, None, _ptr(self.error_word), self._stream()),
            "latent_attention")

    def route_top(self, logits: torch.Tensor, chosen: torch.Tensor, share: torch.Tensor, scores: str = "chosen") -> None:
        """chosen[t] = the chosen.shape[1] experts with the largest logits[t] (float32); share[t] = softmax over those
        (`scores` "chosen"), or the softmax over all experts at the chosen ones, as it is ("all")."""
        T, E = logits.shape
        self._count("route_top")
        if scores == "chosen":
            _check(self._moe.kvb_route_top(_ptr(logits), _ptr(chosen), _ptr(share), T, E, chosen.shape[1], self._stream()), "route_top")
        elif scores == "all":
            _check(self._moe.kvb_route_top_scores(_ptr(logits), _ptr(chosen), _ptr(share), T, E, chosen.shape[1], 1, self._stream()),
                   "route_top")
        else:
            raise KernelError(f"route_top: scores '{scores}' (chosen, all)")

    ROUTED_SMALL_PAIRS = 256      # up to this many (row, choice) pairs the grouped products use tiles of 16 rows, else of 64

    def routed_experts(self, x: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, chosen: torch.Tensor,
                       share: torch.Tensor, out: torch.Tensor, activation: str, workspace, limit: float = 0.0,
                       base: Optional[torch.Tensor] = None) -> None:
        """out[t] = base[t] + sum_s share[t, s] * w_down[e] . act(w_up[e] . x[t]), e = chosen[t, s]; w_down [E, H, F].
        "relu2": w_up [E, F, H], act = relu(.)^2.  "clamped_swiglu": w_up [E, 2 F, H] with gate row i at 2 i and up row i
        at 2 i + 1, act = g' sigmoid(1.702 g') (u' + 1) with g' = min(g, limit), u' = clamp(u, -limit, limit).  "swiglu":
        the same layout, act = silu(g) u (the kernels' gated epilogue with no limit)."""
        if activation not in ("relu2", "clamped_swiglu", "swiglu"):
            raise KernelError(f"routed_experts: activation '{activation}' is not built")
        if activation == "clamped_swiglu" and not limit > 0.0:
            raise KernelError("routed_experts: the clamped activation needs a positive limit")
        T, H = x.shape
        E, F, _ = w_up.shape
        top = chosen.shape[1]
        if activation != "relu2" or base is not None:
            self._routed_general(x, w_up, w_down, chosen, share, out, 1 if activation == "relu2" else 2,
                                 float(limit) if activation == "clamped_swiglu" else 0.0, base, workspace)
            return
        pairs = T * top
        ws, i32 = workspace, torch.int32
        code, stream = _dtype_code(x.dtype), self._stream()
        place = ws.buffer("moe.place", (pairs,), i32)
        order = ws.buffer("moe.order", (pairs,), i32)
        plan = ws.buffer("moe.plan", (4,), i32)
        if (self.routed_tcgen05_min_pairs is not None and pairs >= self.routed_tcgen05_min_pairs and x.dtype == torch.bfloat16
                and H % 8 == 0 and F % 8 == 0):
            # Many rows: runs padded to tiles of 128 rows, the step's rows gathered into that order, both products on tcgen05.
            BM = 128
            max_tiles = -(-pairs // BM) + E
            capacity = max_tiles * BM
            tiles = ws.buffer("moe.tiles", (max_tiles * 3,), i32)
            xs = ws.buffer("moe.xs", (capacity, H), x.dtype)
            act = ws.buffer("moe.act", (capacity, F), x.dtype)
            y = ws.buffer("moe.y", (capacity, H), x.dtype)
            self._count("routed_plan")
            _check(self._moe.kvb_routed_plan(_ptr(chosen), pairs, E, BM, 1, _ptr(place), _ptr(order), _ptr(plan), _ptr(tiles), stream),
                   "routed_plan")
            self._count("gather_rows")
            _check(self._gemm_grouped.kvb_gather_rows(_ptr(x), _ptr(place), _ptr(xs), pairs, top, H, stream), "gather_rows")
            for a, w, out_, n, k, act_code, what in ((xs, w_up, act, F, H, 1, "up"), (act, w_down, y, H, F, 0, "down")):
                self._count("grouped_gemm_tcgen05")
                _check(self._gemm_grouped.kvb_grouped_gemm_tcgen05(_ptr(a), _ptr(w), _ptr(out_), _ptr(plan), _ptr(tiles), max_tiles,
                                                                   capacity, E, n, k, act_code, _ptr(self.error_word), stream),
                       f"grouped_gemm_tcgen05 ({what})")
            self._count("routed_combine")
            _check(self._moe.kvb_routed_combine(code, _ptr(y), _ptr(place), _ptr(share), _ptr(out), T, top, H, stream), "routed_combine")
            return
        BM = 16 if pairs <= self.ROUTED_SMALL_PAIRS else 64
        max_tiles = -(-pairs // BM) + E
        tiles = ws.buffer("moe.tiles", (max_tiles * 3,), i32)
        act = ws.buffer("moe.act", (pairs, F), x.dtype)
        y = ws.buffer("moe.y", (pairs, H), x.dtype)
        self._count("routed_plan")
        _check(self._moe.kvb_routed_plan(_ptr(chosen), pairs, E, BM, 0, _ptr(place), _ptr(order), _ptr(plan), _ptr(tiles), stream),
               "routed_plan")
        self._count("grouped_gemm")
        _check(self._moe.kvb_grouped_gemm(code, _ptr(x), _ptr(order), top, _ptr(w_up), _ptr(act), _ptr(plan), _ptr(tiles),
                                          max_tiles, BM, F, H, 1, stream), "grouped_gemm (up)")
        self._count("grouped_gemm")
        _check(self._moe.kvb_grouped_gemm(code, _ptr(act), _ptr(order), 0, _ptr(w_down), _ptr(y), _ptr(plan), _ptr(tiles),
                                          max_tiles, BM, H, F, 0, stream), "grouped_gemm (down)")
        self._count("routed_combine")
        _check(self._moe.kvb_routed_combine(code, _ptr(y), _ptr(place), _ptr(share), _ptr(out), T, top, H, stream), "routed_combine")

    def _routed_general(self, x, w_up, w_down, chosen, share, out, act: int, limit: float, base, ws) -> None:
        """The routed feed-forward with any of the grouped product's activations and an optional base: plan, product up
        (rows gathered, activation in the epilogue), product down, combine - float32 on CUDA cores, bfloat16 on `mma.sync`,
        and from `routed_tcgen05_min_pairs` pairs on through the tensor-memory kernel."""
        T, H = x.shape
        E, N, _ = w_up.shape
        F = N // 2 if act == 2 else N
        top = chosen.shape[1]
        pairs = T * top
        i32 = torch.int32
        code, stream = _dtype_code(x.dtype), self._stream()
        place = ws.buffer("moe.place", (pairs,), i32)
        order = ws.buffer("moe.order", (pairs,), i32)
        plan = ws.buffer("moe.plan", (4,), i32)
        if (self.routed_tcgen05_min_pairs is not None and pairs >= self.routed_tcgen05_min_pairs and x.dtype == torch.bfloat16
                and H % 8 == 0 and F % 8 == 0 and N % 16 == 0):
            # Many rows: runs padded to tiles of 128 rows, the step's rows gathered into that order, both products on tcgen05.
            BM = 128
            max_tiles = -(-pairs // BM) + E
            capacity = max_tiles * BM
            tiles = ws.buffer("moe.tiles", (max_tiles * 3,), i32)
            xs = ws.buffer("moe.xs", (capacity, H), x.dtype)
            hidden = ws.buffer("moe.act", (capacity, F), x.dtype)
            y = ws.buffer("moe.y", (capacity, H), x.dtype)
            self._count("routed_plan")
            _check(self._moe.kvb_routed_plan(_ptr(chosen), pairs, E, BM, 1, _ptr(place), _ptr(order), _ptr(plan), _ptr(tiles), stream),
                   "routed_plan")
            self._count("gather_rows")
            _check(self._gemm_grouped.kvb_gather_rows(_ptr(x), _ptr(place), _ptr(xs), pairs, top, H, stream), "gather_rows")
            for a, w, out_, n, k, act_code, what in ((xs, w_up, hidden, N, H, act, "up"), (hidden, w_down, y, H, F, 0, "down")):
                self._count("grouped_gemm_tcgen05")
                _check(self._gemm_grouped.kvb_grouped_gemm_tcgen05_act(_ptr(a), _ptr(w), _ptr(out_), _ptr(plan), _ptr(tiles), max_tiles,
                                                                       capacity, E, n, k, act_code, limit, _ptr(self.error_word),
                                                                       stream), f"grouped_gemm_tcgen05 ({what})")
            self._count("routed_combine")
            _check(self._moe.kvb_routed_combine_base(code, _ptr(y), _ptr(place), _ptr(share), _ptr(base), _ptr(out), T, top, H, stream),
                   "routed_combine")
            return
        BM = 16 if pairs <= self.ROUTED_SMALL_PAIRS else 64
        max_tiles = -(-pairs // BM) + E
        tiles = ws.buffer("moe.tiles", (max_tiles * 3,), i32)
        hidden = ws.buffer("moe.act", (pairs, F), x.dtype)
        y = ws.buffer("moe.y", (pairs, H), x.dtype)
        self._count("routed_plan")
        _check(self._moe.kvb_routed_plan(_ptr(chosen), pairs, E, BM, 0, _ptr(place), _ptr(order), _ptr(plan), _ptr(tiles), stream),
               "routed_plan")
        self._count("grouped_gemm")
        _check(self._moe.kvb_grouped_gemm_act(code, _ptr(x), _ptr(order), top, _ptr(w_up), _ptr(hidden), _ptr(plan), _ptr(tiles),
                                              max_tiles, BM, N, H, act, limit, stream), "grouped_gemm (up)")
        self._count("grouped_gemm")
        _check(self._moe.kvb_grouped_gemm_act(code, _ptr(hidden), _ptr(order), 0, _ptr(w_down), _ptr(y), _ptr(plan), _ptr(tiles),
                                              max_tiles, BM, H, F, 0, 0.0, stream), "grouped_gemm (down)")
        self._count("routed_combine")
        _check(self._moe.kvb_routed_combine_base(code, _ptr(y), _ptr(place), _ptr(share), _ptr(base), _ptr(out), T, top, H, stream),
               "routed_combine")

    # ---- hashed pair embedding, gated heads, matrix-state mixers ---------------------------------------------
    def bigram_embed(self, table: torch.Tensor, batch: StepBatch, previous: torch.Tensor, h: torch.Tensor, buckets: int,
                     mul_prev: int, mul_cur: int, vocab: int) -> None:
        """h[r] += table[(previous token * mul_prev + token * mul_cur) mod buckets], or table[buckets] at position 0; the
        token before a segment's first row is previous[slot], which then becomes the segment's last token."""
        T, W = h.shape
        self._count("bigram_embed")
        self.launches += 1
        _check(self._recurrent.kvb_bigram_embed(
            _dtype_code(table.dtype), _ptr(table), _ptr(batch.token_ids), _ptr(batch.token_src), _ptr(batch.last_tokens),
            _ptr(batch.positions), _ptr(batch.row_segment), _ptr(batch.seg_q_start), _ptr(batch.seg_q_len), _ptr(batch.seg_slot),
            _ptr(previous), _ptr(h), T, batch.num_segments, W, int(buckets), int(mul_prev), int(mul_cur), int(vocab),
            self._stream()), "bigram_embed")

    def head_gate(self, x: torch.Tensor, gate, num_heads: int, value_dim: int, scale: float, out: torch.Tensor,
                  out_col: int = 0, x_head_stride: Optional[int] = None) -> None:
        """out[t, out_col + h * Dv + d] = x[t, h * xs + d] * sigmoid(g[t, col + h]) * scale; `gate` = (g, col) or None;
        xs = `x_head_stride` (None: Dv): a head of x may carry columns after its Dv numbers, which are left out."""
        T = x.shape[0]
        xs = value_dim if x_head_stride is None else int(x_head_stride)
        if x.shape[1] != num_heads * xs:
            raise KernelError("head_gate: the rows do not hold num_heads heads of that stride")
        g, col = gate if gate is not None else (None, 0)
        if g is not None and g.dtype != x.dtype:
            raise KernelError("head_gate: the gate and the rows differ in type")
        self._count("head_gate")
        _check(self._recurrent.kvb_head_gate(_dtype_code(x.dtype), _ptr(x), xs, _ptr(g), 0 if g is None else g.shape[1], col, float(scale),
                                             _ptr(out), out.shape[1], out_col, T, num_heads, value_dim, self._stream()), "head_gate")

    def head_norm_gate(self, o: torch.Tensor, weight: torch.Tensor, eps: float, gate, activation: str, scale: float,
                       out: torch.Tensor, out_col: int, num_heads: int, value_dim: int, scope: str = "head") -> None:
        """out[t, out_col + h * Dv + d] = o[t, h, d] / sqrt(mean_d o[t, h, :]^2 + eps) * w * act(g[t, col + h * Dv + d]) * scale;
        o and g float32, `weight` of Dv numbers (all heads) or H * Dv, act "silu" or "sigmoid", `gate` = (g, col).
        `scope` "all": the mean runs over all H * Dv numbers of a row at once (`weight` of H * Dv numbers)."""
        T = o.shape[0]
        g, col = gate
        if o.dtype != torch.float32 or g.dtype != torch.float32:
            raise KernelError("head_norm_gate takes float32 rows")
        if weight.numel() not in (value_dim, num_heads * value_dim):
            raise KernelError("head_norm_gate: the weight fits neither one head nor all")
        if scope not in ("head", "all") or (scope == "all" and weight.numel() != num_heads * value_dim):
            raise KernelError("head_norm_gate: scope 'head' or 'all' (with a weight over all heads' channels)")
        self._count("head_norm_gate")
        mode = 2 if scope == "all" else (1 if weight.numel() != value_dim else 0)
        _check(self._recurrent.kvb_head_norm_gate(
            _dtype_code(out.dtype), _ptr(o), _ptr(weight), mode, float(eps), _ptr(g), g.shape[1],
            col, {"silu": 0, "sigmoid": 1}[activation], float(scale), _ptr(out), out.shape[1], out_col, T, num_heads, value_dim,
            self._stream()), "head_norm_gate")

    # A step whose longest segment has at least SCAN_CHUNK_MIN_ROWS tokens scans its segments in chunks of SCAN_CHUNK tokens
    # that run side by side (three launches, see csrc/recurrent.cu); below that a segment is one piece, and a token's
    # result is bit for bit the same however the request was cut.
    SCAN_CHUNK = 64
    SCAN_CHUNK_MIN_ROWS = 256
    DELTA_LONG_ROWS = 1536           # the delta rule: steps whose longest portion has at least this many rows ...
    DELTA_LONG_CHUNK = 128           # ... are cut into chunks of this many tokens

    def _scan(self, mode: int, proj, q_col, k_col, v_col, gate, g0, g1, p0, q_scale, floor, batch, memory, normalizer, maximum, out,
              H, D, Dv, workspace=None) -> None:
        if proj.dtype != torch.float32 or gate.dtype != torch.float32 or out.dtype != torch.float32 or memory.dtype != torch.float32:
            raise KernelError("the matrix-state scan takes float32 rows and states")
        if tuple(memory.shape[1:]) != (H, D, Dv):
            raise KernelError(f"the matrix-state scan wants states [slots, {H}, {D}, {Dv}], got {tuple(memory.shape)}")
        max_chunks, scratch = 0, None
        if workspace is not None and self.SCAN_CHUNK and batch.max_q_len >= self.SCAN_CHUNK_MIN_ROWS:
            # Sized by the step's rows and segments alone, so that a recorded step finds the same launches.
            max_chunks = -(-batch.num_tokens // self.SCAN_CHUNK) + batch.num_segments
            scratch = workspace.buffer("recurrent.chunks", (max_chunks * H * (2 * Dv * D + 2 * D + 3),), torch.float32)
            self.launches += 2
        self._count("matrix_state_scan")
        _check(self._recurrent.kvb_matrix_state_scan(
            mode, _ptr(proj), proj.shape[1], q_col, k_col, v_col, _ptr(gate), gate.shape[1], g0, g1, float(p0), float(q_scale),
            float(floor), _ptr(batch.seg_q_start), _ptr(batch.seg_q_len), _ptr(batch.seg_slot), _ptr(memory), _ptr(normalizer),
            _ptr(maximum), _ptr(out), proj.shape[0], batch.num_segments, H, D, Dv, self.SCAN_CHUNK, max_chunks, _ptr(scratch),
            self._stream()), "matrix_state_scan")

    def gated_linear_scan(self, proj: torch.Tensor, cols, z: torch.Tensor, tau: float, q_scale: float, batch: StepBatch,
                          memory: torch.Tensor, out: torch.Tensor, H: int, D: int, Dv: int, workspace=None) -> None:
        """Per segment, from and into memory[slot] ([H, D, Dv], float32): S = diag(a_t) S + k_t v_t^T, out_t = S^T (q_t q_scale),
        a_t = sigmoid(z_t)^(1 / tau) per key channel; q, k, v at columns `cols` of the float32 rows `proj`.  `z` [T, H * D] is
        overwritten by the decays."""
        self.launches += 1
        self._scan(0, proj, cols[0], cols[1], cols[2], z, 0, 0, tau, q_scale, 0.0, batch, memory, None, None, out, H, D, Dv, workspace)

    def lightning_scan(self, proj: torch.Tensor, cols, decay: torch.Tensor, batch: StepBatch, memory: torch.Tensor,
                       out: torch.Tensor, H: int, D: int, Dv: int, workspace) -> None:
        """Per segment, from and into memory[slot] ([H, D, Dv], float32): S = decay[h] S + k_t v_t^T, out_t = S^T q_t with
        q, k, v = silu of the columns `cols` of the float32 rows `proj`, which are overwritten by them; `decay` float32 [H]."""
        if proj.dtype != torch.float32 or out.dtype != torch.float32 or memory.dtype != torch.float32 or decay.dtype != torch.float32:
            raise KernelError("the lightning scan takes float32 rows, decays and states")
        if tuple(memory.shape[1:]) != (H, D, Dv) or decay.numel() != H:
            raise KernelError(f"the lightning scan wants states [slots, {H}, {D}, {Dv}] and {H} decays")
        T = proj.shape[0]
        decays = workspace.buffer("recurrent.decays", (T, H * D), torch.float32)
        max_chunks, scratch = 0, None
        if self.SCAN_CHUNK and batch.max_q_len >= self.SCAN_CHUNK_MIN_ROWS:
            max_chunks = -(-batch.num_tokens // self.SCAN_CHUNK) + batch.num_segments       # as in `_scan`
            scratch = workspace.buffer("recurrent.chunks", (max_chunks * H * (2 * Dv * D + 2 * D + 3),), torch.float32)
            self.launches += 2
        self.launches += 1
        self._count("lightning_scan")
        _check(self._recurrent.kvb_lightning_scan(
            _ptr(proj), proj.shape[1], cols[0], cols[1], cols[2], _ptr(decay), _ptr(decays), _ptr(batch.seg_q_start),
            _ptr(batch.seg_q_len), _ptr(batch.seg_slot), _ptr(memory), _ptr(out), T, batch.num_segments, H, D, Dv, self.SCAN_CHUNK,
            max_chunks, _ptr(scratch), self._stream()), "lightning_scan")

    def matrix_memory_scan(self, proj: torch.Tensor, cols, cap: float, q_scale: float, floor: float, batch: StepBatch,
                           memory: torch.Tensor, normalizer: torch.Tensor, maximum: torch.Tensor, out: torch.Tensor, H: int, D: int,
                           Dv: int, workspace=None) -> None:
        """Per segment, from and into (memory, normalizer, maximum)[slot]: i = cap tanh(x_i / cap), f = logsigmoid(cap tanh(x_f / cap)),
        m' = max(f + m, i), S = e^{f + m - m'} S + e^{i - m'} k v^T, n likewise with k, out = S^T q / (max(|n . q|, e^{-m'}) + floor);
        q, k, v and the gates' pre-activations x_i, x_f (one per head) at columns `cols` of `proj`."""
        self._scan(1, proj, cols[0], cols[1], cols[2], proj, cols[3], cols[4], cap, q_scale, floor, batch, memory, normalizer, maximum,
                   out, H, D, Dv, workspace)

    def delta_rule_scan(self, proj: torch.Tensor, cols, z: torch.Tensor, rate: float, unit_eps: float, batch: StepBatch,
                        memory: torch.Tensor, out: torch.Tensor, H: int, D: int, workspace) -> None:
        """Per segment, from and into memory[slot] ([H, D, D], float32): w = exp(-rate sigmoid(z)) per key channel,
        u = k / sqrt(sum k^2 + unit_eps) per head, a = sigmoid(removal logits); S = diag(w) S - (a u)(u^T S) + k v^T (both
        terms read the old state), out = S^T r; r, k, v and the removal logits at columns `cols` of the float32 rows `proj`."""
        if proj.dtype != torch.float32 or z.dtype != torch.float32 or out.dtype != torch.float32 or memory.dtype != torch.float32:
            raise KernelError("the delta-rule scan takes float32 rows and states")
        if tuple(memory.shape[1:]) != (H, D, D) or z.shape[1] != H * D:
            raise KernelError(f"the delta-rule scan wants states [slots, {H}, {D}, {D}], got {tuple(memory.shape)}")
        T = proj.shape[0]
        aux = workspace.buffer("recurrent.delta_inputs", (T, 3 * H * D), torch.float32)
        max_chunks, scratch = 0, None
        # Long portions take longer chunks: every chunk costs a product with its transition in the launch that walks the start
        # states (measured at 14 heads of 64 / 16 heads of 128 channels, chunks of 64 against 128 tokens: 143 / 328 us against
        # 223 / 349 us at 512 rows, 389 / 1,020 us against 279 / 731 us at 2,048 rows).
        chunk = self.SCAN_CHUNK if batch.max_q_len < self.DELTA_LONG_ROWS else max(self.SCAN_CHUNK, self.DELTA_LONG_CHUNK)
        if self.SCAN_CHUNK and batch.max_q_len >= self.SCAN_CHUNK_MIN_ROWS:
            # As in `_scan`; a chunk also leaves its transition, a matrix over the key channels.
            max_chunks = -(-batch.num_tokens // chunk) + batch.num_segments
            scratch = workspace.buffer("recurrent.delta_chunks", (max_chunks * H * (3 * D * D + 2 * D + 3),), torch.float32)
            self.launches += 2
        self.launches += 1
        self._count("delta_rule_scan")
        _check(self._recurrent.kvb_delta_rule_scan(
            _ptr(proj), proj.shape[1], cols[0], cols[1], cols[2], cols[3], _ptr(z), float(rate), float(unit_eps), _ptr(aux),
            _ptr(batch.seg_q_start), _ptr(batch.seg_q_len), _ptr(batch.seg_slot), _ptr(memory), _ptr(out), T, batch.num_segments,
            H, D, chunk, max_chunks, _ptr(scratch), self._stream()), "delta_rule_scan")

    def sample(self, logits: torch.Tensor, temperature: torch.Tensor, seeds: torch.Tensor, counters: torch.Tensor,
               out: torch.Tensor, scratch_val: torch.Tensor, scratch_idx: torch.Tensor) -> None:
        R, V = logits.shape
        self._count("sample")
        _check(self._sampling.kvb_sample(_ptr(logits), R, V, _ptr(temperature), _ptr(seeds), _ptr(counters),
                                         _ptr(scratch_val), _ptr(scratch_idx), _ptr(out), self._stream()), "sample")

    def sample_parts(self, vocab: int) -> int:
        return int(self._sampling.kvb_sample_parts(vocab))
