"""Time per class of kernel, behind a flag: CUDA events around every operator of the kernel set.

The reference times whole decode steps by wall clock (apps/qwen_infer.cu:30-38) and has no
per-kernel figures.  `KernelTiming` wraps the operators of a `CudaKernels` object while it is
switched on: each call is bracketed by two events on the launching stream and filed under a
class - the operator's name, and for matrix products the weight's shape, since one operator
serves the q/k/v, output, feed-forward and head products.  With each class go the bytes its
calls had to move (weights, activations, the keys and values of the step's requests), so that a
report can state microseconds, GB/s and launches per class.

A kernel between two events neither starts before its predecessor has ended nor overlaps its
successor, which the engine's launch chain otherwise allows; the classes therefore add up to
more than a step takes.  CUDA graphs cannot hold these events: switch graphs off while timing.

Launched one by one, the kernels of a decode step take the host longer to launch (about 12 us
each) than the GPU to run, and an event pair around an idle GPU measures the host.  So the
first operator of every step (`embed`) is preceded by a kernel that only spins for `hold_ms`
milliseconds: while it runs the host queues the step's launches, and the events then see the
kernels back to back.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Tuple

import torch


def _numel_bytes(t) -> int:
    return 0 if t is None else t.numel() * t.element_size()


def _attention_bytes(batch, kv, num_heads: int) -> int:
    """Keys and values of the step's requests (every key once per kv head), queries in, results out."""
    spec = kv.spec
    element = kv.k_pages.element_size()
    host = batch.host
    if "starts" in host and "counts" in host:
        keys = int((host["starts"] + host["counts"]).sum())
        if spec.window:
            keys = int(sum(min(int(s + c), spec.window + int(c) - 1) for s, c in zip(host["starts"], host["counts"])))
    else:
        keys = batch.max_kv_len * batch.num_segments
    rows = batch.num_tokens * num_heads * spec.head_dim * element
    return 2 * keys * spec.num_kv_heads * spec.head_dim * element + 2 * rows


class KernelTiming:
    OPERATORS = ("embed", "add_rmsnorm", "silu_mul", "gate_up_act", "linear", "qkv_rope_append", "rope_append_attention",
                 "paged_attention", "sample", "norm_add_rmsnorm", "latent_norm_rope_append", "head_linear", "latent_attention",
                 "route_top", "routed_experts", "bigram_embed", "head_gate", "head_norm_gate", "gated_linear_scan",
                 "matrix_memory_scan", "token_shift", "activation_", "delta_rule_scan", "lightning_scan")

    def __init__(self, kernels, hold_ms: float = 4.0):
        self.kernels = kernels
        self.hold_cycles = int(hold_ms * 1e-3 * getattr(torch.cuda.get_device_properties(kernels.device), "clock_rate", 1_900_000) * 1e3) if hold_ms > 0 else 0
        self.records: List[tuple] = []      # (class, bytes, begin event, end event, launches, flops)
        self._saved: Dict[str, Callable] = {}
        self._depth = 0

    # ---- which class a call belongs to and what it has to move -----------------------------------
    @staticmethod
    def _describe(name: str, args, kwargs) -> Tuple[str, int]:
        if name == "linear":
            x, w, out = args[0], args[1], args[2]
            return f"linear {w.shape[0]}x{w.shape[1]}", _numel_bytes(w) + _numel_bytes(x) + _numel_bytes(out)
        if name == "gate_up_act":
            x, w, out = args[0], args[1], args[2]
            return f"gate_up_act {w.shape[0]}x{w.shape[1]}", _numel_bytes(w) + _numel_bytes(x) + _numel_bytes(out)
        if name == "embed":
            out = args[2]
            return name, out.numel() * (4 + args[0].element_size())
        if name == "add_rmsnorm":
            h, delta, out = args[0], args[1], args[4]
            rows, width = out.shape
            return name, rows * width * (8 + out.element_size() + (delta.element_size() if delta is not None else 0))
        if name == "silu_mul":
            return name, _numel_bytes(args[0]) + _numel_bytes(args[1])
        if name == "qkv_rope_append":
            return name, 2 * _numel_bytes(args[0])
        if name == "rope_append_attention":
            qkv, batch, kv, num_heads = args[0], args[4], args[5], args[7]
            return name, _attention_bytes(batch, kv, num_heads) + _numel_bytes(qkv)
        if name == "paged_attention":
            batch, kv, num_heads = args[1], args[2], args[4]
            return name, _attention_bytes(batch, kv, num_heads)
        if name == "sample":
            return name, _numel_bytes(args[0])
        if name == "norm_add_rmsnorm":
            h, delta, out, tail = args[0], args[1], args[6], (args[8] if len(args) > 8 else kwargs.get("tail"))
            return name, _numel_bytes(delta) + (2 * _numel_bytes(h) if delta is not None else _numel_bytes(h)) + _numel_bytes(out) + _numel_bytes(tail)
        if name == "latent_norm_rope_append":
            proj, q_rank, kv_rank, rot_dim = args[0], args[1], args[2], args[3]
            return name, proj.shape[0] * (2 * q_rank + 2 * (kv_rank + rot_dim)) * proj.element_size()
        if name == "head_linear":
            x, w, out = args[0], args[1], args[2]
            return f"head_linear {w.shape[0]}x{w.shape[1]}x{w.shape[2]}", _numel_bytes(w) + _numel_bytes(x) + _numel_bytes(out)
        if name == "latent_attention":
            q, batch, kv, out = args[0], args[1], args[2], args[3]
            host = batch.host
            window = kwargs.get("window", -1)
            window = kv.spec.window if window == -1 else window
            keys = int((host["starts"] + host["counts"]).sum()) if "starts" in host else batch.max_kv_len * batch.num_segments
            if window and "starts" in host:
                keys = int(sum(min(int(s + c), window + int(c) - 1) for s, c in zip(host["starts"], host["counts"])))
            return name, keys * kv.spec.head_dim * kv.k_pages.element_size() + _numel_bytes(q) + _numel_bytes(out)
        if name == "route_top":
            return name, _numel_bytes(args[0])
        if name == "routed_experts":
            x, w_up, w_down, chosen, out = args[0], args[1], args[2], args[3], args[5]
            used = min(w_up.shape[0], chosen.numel())          # experts a step can touch at most
            per_expert = (w_up[0].numel() + w_down[0].numel()) * w_up.element_size()
            return f"routed_experts {w_up.shape[0]}x{w_up.shape[1]}x{w_up.shape[2]}", used * per_expert + _numel_bytes(x) + _numel_bytes(out)
        if name == "bigram_embed":
            h, table = args[3], args[0]
            return name, h.numel() * (8 + table.element_size())
        if name == "head_gate":
            return name, 2 * _numel_bytes(args[0])
        if name == "head_norm_gate":
            o, out, H, Dv = args[0], args[6], args[8], args[9]
            return name, 2 * _numel_bytes(o) + o.shape[0] * H * Dv * out.element_size()
        if name in ("gated_linear_scan", "matrix_memory_scan"):
            # The rows' q, k, decay (or gates) and v in, the read-outs out, and every segment's state in and out.
            if name == "gated_linear_scan":
                proj, batch, memory, out, H, D, Dv = args[0], args[5], args[6], args[7], args[8], args[9], args[10]
                per_row = 3 * H * D + 2 * H * Dv
            else:
                proj, batch, memory, out, H, D, Dv = args[0], args[5], args[6], args[9], args[10], args[11], args[12]
                per_row = 2 * H * D + 2 * H * Dv + 2 * H
            return f"{name} {H}x{D}x{Dv}", 4 * (proj.shape[0] * per_row + 2 * batch.num_segments * H * D * Dv)
        if name == "lightning_scan":
            # The rows' q, k and v in, the read-outs out, and every segment's state in and out (the decays are constants).
            proj, batch, H, D, Dv = args[0], args[3], args[6], args[7], args[8]
            return f"{name} {H}x{D}x{Dv}", 4 * (proj.shape[0] * (2 * H * D + 2 * H * Dv) + 2 * batch.num_segments * H * D * Dv)
        if name == "delta_rule_scan":
            # The rows' r, k, v, removal and decay logits in, the read-outs out, and every segment's state in and out.
            proj, batch, H, D = args[0], args[5], args[8], args[9]
            return f"{name} {H}x{D}x{D}", 4 * (proj.shape[0] * 6 * H * D + 2 * batch.num_segments * H * D * D)
        if name == "token_shift":
            x, out = args[0], args[4]
            return name, _numel_bytes(x) + _numel_bytes(out)
        if name == "activation_":
            return name, 2 * _numel_bytes(args[0])
        return name, 0

    @staticmethod
    def _keys_seen(batch, spec=None) -> int:
        """Sum over the step's rows of the keys a row sees (its own included): all up to its position, or with a window
        the window's keys and the kept first ones behind it."""
        host = batch.host
        if "starts" not in host:
            return batch.num_tokens * batch.max_kv_len
        window = getattr(spec, "window", None)
        if not window:
            return int(sum(int(c) * int(s) + int(c) * (int(c) + 1) // 2 for s, c in zip(host["starts"], host["counts"])))
        keep, total = int(getattr(spec, "keep_first", 0) or 0), 0
        for s, c in zip(host["starts"], host["counts"]):
            for p in range(int(s), int(s) + int(c)):
                total += min(p + 1, window) + max(0, min(keep, p + 1 - window))
        return total

    @classmethod
    def _flops(cls, name: str, args, kwargs) -> int:
        """Multiply-adds times two that the call's matrix products need (0 for classes that are only moved bytes)."""
        if name == "linear":
            return 2 * args[0].shape[0] * args[1].shape[0] * args[1].shape[1]
        if name == "gate_up_act":
            return 2 * args[0].shape[0] * args[1].shape[0] * args[1].shape[1]
        if name == "head_linear":
            w = args[1]
            return 2 * args[0].shape[0] * w.shape[0] * w.shape[1] * w.shape[2]
        if name == "latent_attention":
            batch, kv, heads, value_dim = args[1], args[2], args[4], args[5]
            window = kwargs.get("window", -1)

            class _Reach:
                pass
            reach = _Reach()
            reach.window, reach.keep_first = (kv.spec.window if window == -1 else window), 0
            return 2 * heads * (kv.spec.head_dim + value_dim) * cls._keys_seen(batch, reach)
        if name == "paged_attention":
            batch, kv, heads = args[1], args[2], args[4]
            return 2 * heads * (kv.spec.head_dim + kv.spec.v_head_dim) * cls._keys_seen(batch, kv.spec)
        if name == "rope_append_attention":
            batch, kv, heads = args[4], args[5], args[7]
            return 2 * heads * (kv.spec.head_dim + kv.spec.v_head_dim) * cls._keys_seen(batch, kv.spec)
        if name == "routed_experts":
            x, w_up, w_down, chosen = args[0], args[1], args[2], args[3]
            return 2 * chosen.numel() * (w_up.shape[1] * w_up.shape[2] + w_down.shape[1] * w_down.shape[2])
        if name == "gated_linear_scan":
            return 4 * args[0].shape[0] * args[8] * args[9] * args[10]          # per row and state element: decay-and-add, read-out
        if name == "matrix_memory_scan":
            return 4 * args[0].shape[0] * args[10] * args[11] * args[12]
        if name == "lightning_scan":
            return 4 * args[0].shape[0] * args[6] * args[7] * args[8]
        if name == "delta_rule_scan":
            # per row and state element: decay, the read along the unit key, its removal, the new outer product, read-out
            return 9 * args[0].shape[0] * args[8] * args[9] * args[9]
        return 0

    # ---- switching on and off -------------------------------------------------------------------------
    def start(self) -> None:
        for name in self.OPERATORS:
            original = getattr(self.kernels, name, None)
            if original is None:
                continue
            self._saved[name] = original
            setattr(self.kernels, name, self._wrap(name, original))

    def _wrap(self, name: str, original: Callable) -> Callable:
        def timed(*args, **kwargs):
            if self._depth:                              # called by an operator that is being timed: part of its class
                return original(*args, **kwargs)
            label, nbytes = self._describe(name, args, kwargs)
            flops = self._flops(name, args, kwargs)
            if name == "embed" and self.hold_cycles:
                torch.cuda._sleep(self.hold_cycles)      # keeps the GPU busy while the host queues this step
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            launches = self.kernels.launches
            begin.record()
            self._depth += 1
            try:
                result = original(*args, **kwargs)
            finally:
                self._depth -= 1
            end.record()
            if name == "rope_append_attention" and result is False:
                return result                            # nothing ran: the caller makes the two calls
            self.records.append((label, nbytes, begin, end, self.kernels.launches - launches, flops))
            return result
        return timed

    def stop(self) -> Dict[str, dict]:
        """Restores the operators; returns {class: {"us", "bytes", "calls", "launches", "flops"}} summed over all calls."""
        for name in self._saved:
            try:
                delattr(self.kernels, name)              # the wrapper lives on the instance; the class method is back
            except AttributeError:
                pass
        self._saved.clear()
        torch.cuda.synchronize(self.kernels.device)
        report: Dict[str, dict] = {}
        for label, nbytes, begin, end, launches, flops in self.records:
            entry = report.setdefault(label, {"us": 0.0, "bytes": 0, "calls": 0, "launches": 0, "flops": 0})
            entry["flops"] += flops
            entry["us"] += begin.elapsed_time(end) * 1e3
            entry["bytes"] += nbytes
            entry["calls"] += 1
            entry["launches"] += launches
        self.records.clear()
        return report


def format_report(report: Dict[str, dict], steps: int = 1) -> str:
    """A table of the classes, slowest first: microseconds a step, share, GB/s."""
    total = sum(e["us"] for e in report.values()) or 1.0
    lines = [f"{'class':<34}{'us/step':>10}{'share':>8}{'calls':>7}{'GB/s':>9}"]
    for label, e in sorted(report.items(), key=lambda kv: -kv[1]["us"]):
        gbs = e["bytes"] / (e["us"] * 1e-6) / 1e9 if e["us"] > 0 and e["bytes"] else 0.0
        lines.append(f"{label:<34}{e['us'] / steps:>10.1f}{100 * e['us'] / total:>7.1f}%{e['calls'] // max(steps, 1):>7}{gbs:>9.0f}")
    return "\n".join(lines)
