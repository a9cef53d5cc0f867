"""Plain PyTorch statement of every operator of the kernel set, over the same paged
layouts.  Two uses: the per-kernel reference that each CUDA kernel is compared with, and
a stand-in kernel set that lets the engine's host logic (cache, step function, scheduler)
run in tests on a machine without a GPU.  It is test code: the package has no CPU path.
"""
from __future__ import annotations

from typing import Optional

import torch

from plain_qwen2 import gumbel_scores


class TorchKernels:
    """Same operator signatures as kvcache_b200.kernels.api.CudaKernels; math in float32
    (or float64 when `wide` is set), stores in the tensors' own types."""

    def __init__(self, wide: bool = False):
        self.f = torch.float64 if wide else torch.float32
        self.launches = 0

    def check_errors(self) -> None:
        pass

    def embed(self, table, ids, out, src=None, last=None, scale=1.0):
        ids = ids.long()
        if src is not None:
            ids = torch.where(src >= 0, last[src.clamp(min=0).long()].long(), ids)
        out.copy_(table[ids].to(torch.float32) * scale)

    def add_rmsnorm(self, h, delta, weight, eps, out, rows=None, delta_scale=None):
        f = self.f
        if delta is not None and delta_scale is not None:
            delta = delta.to(torch.float32) * delta_scale
        if rows is None:
            if delta is not None:
                h.add_(delta.to(torch.float32))
            v = h.to(f)
        else:
            v = h[rows.long()].to(f)
            if delta is not None:
                v = (h[rows.long()] + delta[rows.long()].to(torch.float32)).to(f)
        inv = torch.rsqrt((v * v).mean(dim=-1, keepdim=True) + eps)
        out.copy_((v * inv * weight.to(f)).to(out.dtype))

    def linear(self, x, w, out, bias=None):
        y = x.to(self.f) @ w.to(self.f).t()
        if bias is not None:
            y = y + bias.to(self.f)
        out.copy_(y.to(out.dtype))

    def qkv_rope_append(self, qkv, bias, cos, sin, batch, kv, q_out, num_heads, q_norm=None, k_norm=None, norm_eps=0.0, key_dim=None,
                        norm_scope="head", norm_after_rotation=False, value_mix=None, q_temperature=None, value_dim=None):
        f = self.f
        T = qkv.shape[0]
        Hq, Hkv, D = num_heads, kv.spec.num_kv_heads, kv.spec.head_dim
        x = qkv.to(f)
        if bias is not None:
            x = x + bias.to(f)
        if (q_norm is not None or kv.spec.v_head_dim != D or x.shape[1] != (Hq + 2 * Hkv) * D or (key_dim or D) != D
                or norm_eps > 0.0 or value_mix is not None or q_temperature is not None or value_dim is not None):
            return self._qkv_norm_rope_append(x, cos, sin, batch, kv, q_out, Hq, q_norm, k_norm, norm_eps, key_dim or D,
                                              norm_scope, norm_after_rotation, value_mix, q_temperature, value_dim)
        x = x.view(T, Hq + 2 * Hkv, D).clone()
        pos = batch.positions.long()
        if cos is not None:
            half = cos.shape[1]
            c, s = cos[pos].to(f)[:, None, :], sin[pos].to(f)[:, None, :]
            qk = x[:, :Hq + Hkv, :]
            x1, x2 = qk[..., :half].clone(), qk[..., half:2 * half].clone()
            qk[..., :half] = x1 * c - x2 * s
            qk[..., half:2 * half] = x2 * c + x1 * s
        q_out.copy_(x[:, :Hq, :].reshape(T, Hq * D).to(q_out.dtype))
        if kv.writes:
            seg = batch.row_segment.long()
            page = kv.block_table[seg, pos // kv.page_size].long()
            assert bool((page >= 0).all()), "append into a page the block table does not hold"
            slot = pos % kv.page_size
            kv.k_pages[page, :, slot, :] = x[:, Hq:Hq + Hkv, :].to(kv.k_pages.dtype)
            kv.v_pages[page, :, slot, :] = x[:, Hq + Hkv:, :].to(kv.v_pages.dtype)

    def _qkv_norm_rope_append(self, x, cos, sin, batch, kv, q_out, Hq, q_norm, k_norm, eps, D, scope="head", after=False,
                              value_mix=None, q_temperature=None, value_dim=None):
        """Rows [q heads of D | k heads of D | v heads of Dv | columns that are not this operator's]; queries and keys are
        stored kv.spec.head_dim wide, with zeros after their D numbers.  The norm (eps > 0 or weights given): per head or
        over all of a row's heads at once (`scope`), before or `after` the rotation, with or without weights.
        `value_mix` = (kept, lam): lam None - the values are also copied to `kept`; else v = (1 - lam) v + lam kept."""
        f = self.f
        T = x.shape[0]
        Hkv, Dv, wide = kv.spec.num_kv_heads, kv.spec.v_head_dim, kv.spec.head_dim
        v_wide = Dv                        # `value_dim`: values have that many numbers and are stored v_wide wide, zeros after them
        if value_dim is not None:
            Dv = value_dim
        q = x[:, :Hq * D].reshape(T, Hq, D).clone()
        k = x[:, Hq * D:(Hq + Hkv) * D].reshape(T, Hkv, D).clone()
        v = x[:, (Hq + Hkv) * D:(Hq + Hkv) * D + Hkv * Dv].reshape(T, Hkv, Dv)
        if value_mix is not None:
            kept, lam = value_mix
            if lam is None:
                kept.copy_(v.reshape(T, -1).to(kept.dtype))
            else:
                v = (1.0 - lam.to(f)) * v + lam.to(f) * kept.to(f).view(T, Hkv, Dv)

        def normalise(t, weight):
            if scope == "all":
                flat = t.reshape(T, -1)
                flat = flat * torch.rsqrt((flat * flat).mean(dim=-1, keepdim=True) + eps)
                return (flat if weight is None else flat * weight.to(f)).view(t.shape)
            t = t * torch.rsqrt((t * t).mean(dim=-1, keepdim=True) + eps)
            return t if weight is None else t * weight.to(f)

        normed = q_norm is not None or eps > 0.0
        if normed and not after:
            q, k = normalise(q, q_norm), normalise(k, k_norm)
        pos = batch.positions.long()
        if cos is not None:
            half = cos.shape[1]
            c, s = cos[pos].to(f)[:, None, :], sin[pos].to(f)[:, None, :]
            for t in (q, k):
                u, w = t[..., :half].clone(), t[..., half:2 * half].clone()
                t[..., :half], t[..., half:2 * half] = u * c - w * s, w * c + u * s
        if normed and after:
            q, k = normalise(q, q_norm), normalise(k, k_norm)
        if q_temperature is not None:
            coef, every = q_temperature
            q = q * (1.0 + coef * torch.log(torch.div(pos + 1, every, rounding_mode="floor").to(f) + 1.0))[:, None, None]
        if v_wide > Dv:
            v = torch.cat([v, torch.zeros(T, Hkv, v_wide - Dv, dtype=f)], dim=-1)
        if wide > D:
            q = torch.cat([q, torch.zeros(T, Hq, wide - D, dtype=f)], dim=-1)
            k = torch.cat([k, torch.zeros(T, Hkv, wide - D, dtype=f)], dim=-1)
        q_out.copy_(q.reshape(T, Hq * wide).to(q_out.dtype))
        if kv.writes:
            page = kv.block_table[batch.row_segment.long(), pos // kv.page_size].long()
            assert bool((page >= 0).all()), "append into a page the block table does not hold"
            kv.k_pages[page, :, pos % kv.page_size, :] = k.to(kv.k_pages.dtype)
            kv.v_pages[page, :, pos % kv.page_size, :] = v.to(kv.v_pages.dtype)

    def paged_attention(self, q, batch, kv, out, num_heads, scale, workspace=None, sink=None, score_cap=None, slopes=None):
        """`sink` [Hq]: the softmax's denominator also holds exp(sink[h]).  kv.spec.keep_first: with a window, the
        request's first keys stay visible.  `score_cap`: s <- cap tanh(s / cap); `slopes` [Hq]: s <- s - slopes[h] (i - j)."""
        f = self.f
        T = q.shape[0]
        Hq, Hkv, D = num_heads, kv.spec.num_kv_heads, kv.spec.head_dim
        group = Hq // Hkv
        window = kv.spec.window
        qf = q.to(f).view(T, Hq, D)
        result = torch.zeros(T, Hq, kv.spec.v_head_dim, dtype=f, device=q.device)
        for r in range(T):
            p = int(batch.positions[r])
            seg = int(batch.row_segment[r])
            lo = max(0, p - window + 1) if window else 0
            js = torch.arange(lo, p + 1, device=q.device)
            if window and kv.spec.keep_first:
                js = torch.cat([torch.arange(0, min(lo, kv.spec.keep_first), device=q.device), js])
            pages = kv.block_table[seg, js // kv.page_size].long()
            assert bool((pages >= 0).all()), "a needed key lies in a page the block table does not hold"
            keys = kv.k_pages[pages, :, js % kv.page_size, :].to(f)     # [n, Hkv, D]
            vals = kv.v_pages[pages, :, js % kv.page_size, :].to(f)
            for h in range(Hq):
                s = (keys[:, h // group, :] @ qf[r, h]) * scale
                if score_cap is not None:
                    s = score_cap * torch.tanh(s / score_cap)
                if slopes is not None:
                    s = s - slopes[h].to(f) * (p - js).to(f)
                if sink is None:
                    result[r, h] = torch.softmax(s, dim=0) @ vals[:, h // group, :]
                else:
                    top = torch.maximum(s.max(), sink[h].to(f))
                    e = torch.exp(s - top)
                    result[r, h] = (e / (e.sum() + torch.exp(sink[h].to(f) - top))) @ vals[:, h // group, :]
        out.copy_(result.view(T, -1).to(out.dtype))

    @staticmethod
    def _gated(g, u, activation, limit):
        if activation == "silu":
            return g / (1.0 + torch.exp(-g)) * u
        assert activation == "clamped_swiglu"
        g, u = torch.clamp(g, max=limit), torch.clamp(u, min=-limit, max=limit)
        return g * torch.sigmoid(1.702 * g) * (u + 1.0)

    def silu_mul(self, gate_up, out, interleaved=False, activation="silu", limit=0.0):
        I = out.shape[1]
        if interleaved:
            pairs = gate_up.view(gate_up.shape[0], I // 8, 2, 8)
            g, u = pairs[:, :, 0, :].reshape(-1, I).to(self.f), pairs[:, :, 1, :].reshape(-1, I).to(self.f)
        else:
            g, u = gate_up[:, :I].to(self.f), gate_up[:, I:].to(self.f)
        out.copy_(self._gated(g, u, activation, limit).to(out.dtype))

    def gate_up_act(self, x, w_gate_up, out, workspace, interleaved, activation="silu", limit=0.0):
        gate_up = torch.empty(x.shape[0], w_gate_up.shape[0], dtype=out.dtype, device=out.device)
        self.linear(x, w_gate_up, gate_up)
        self.silu_mul(gate_up, out, interleaved, activation, limit)

    def sample_parts(self, vocab):
        return 1

    def sample(self, logits, temperature, seeds, counters, out, scratch_val=None, scratch_idx=None):
        for r in range(logits.shape[0]):
            t = float(temperature[r])
            if t > 0:
                scores = gumbel_scores(logits[r].cpu(), t, int(seeds[r]), int(counters[r]))
                out[r] = int(torch.argmax(scores))
            else:
                out[r] = int(torch.argmax(logits[r]))

    # ---- operators of the latent-attention and routed feed-forward parts ------------------------------------------
    def norm_add_rmsnorm(self, h, delta, delta_weight, delta_eps, weight, eps, out, rows=None, tail=None, delta_gate=None):
        f = self.f
        pick = (lambda t: t) if rows is None else (lambda t: t[rows.long()])
        v = pick(h).to(f)
        if delta is not None:
            d = pick(delta).to(f)
            if delta_gate is not None:
                d = d * torch.sigmoid(pick(delta_gate).to(f))
            if delta_weight is not None:
                d = d * torch.rsqrt((d * d).mean(dim=-1, keepdim=True) + delta_eps) * delta_weight.to(f)
            v = (pick(h) + d.to(torch.float32)).to(f) if f == torch.float32 else v + d
        if rows is None and delta is not None:
            h.copy_(v.to(torch.float32))
        if out is None:
            return
        H = h.shape[1]
        y = v if weight is None else v * torch.rsqrt((v * v).mean(dim=-1, keepdim=True) + eps) * weight.to(f)
        out[:, :H] = y.to(out.dtype)
        if tail is not None:
            out[:, H:] = pick(tail).to(out.dtype)

    def latent_norm_rope_append(self, proj, q_rank, kv_rank, rot_dim, q_weight, kv_weight, eps, cos, sin, batch, kv, cq_out,
                                kv_col=None):
        f = self.f
        norm = lambda v, w: v * torch.rsqrt((v * v).mean(dim=-1, keepdim=True) + eps) * w.to(f)
        if q_rank > 0:
            cq_out.copy_(norm(proj[:, :q_rank].to(f), q_weight).to(cq_out.dtype))
        if not kv.writes:
            return
        at = q_rank if kv_col is None else kv_col
        pos = batch.positions.long()
        c = norm(proj[:, at:at + kv_rank].to(f), kv_weight)
        kr = proj[:, at + kv_rank:at + kv_rank + rot_dim].to(f).clone()
        half = cos.shape[1]
        co, si = cos[pos].to(f), sin[pos].to(f)
        u, v = kr[:, :half].clone(), kr[:, half:2 * half].clone()
        kr[:, :half], kr[:, half:2 * half] = u * co - v * si, v * co + u * si
        page = kv.block_table[batch.row_segment.long(), pos // kv.page_size].long()
        assert bool((page >= 0).all()), "append into a page the block table does not hold"
        kv.k_pages[page, 0, pos % kv.page_size, :] = torch.cat([c, kr], dim=1).to(kv.k_pages.dtype)

    def head_linear(self, x, w, out, rotate=None, gate=None, x_col=None, gate_per_head=False):
        f = self.f
        T = x.shape[0]
        H, N, K = w.shape
        os_ = out.shape[1] // H
        if x_col is not None:                  # the heads' inputs are columns x_col .. of wider rows
            xs = K + (os_ - N if rotate is not None else 0)
            x = x[:, x_col:x_col + H * xs]
        xs = x.shape[1] // H
        xv = x.reshape(T, H, xs).to(f)
        y = torch.einsum("thk,hnk->thn", xv[:, :, :K], w.to(f))
        if gate is not None and gate_per_head:
            g, col = gate
            y = y * torch.sigmoid(g[:, col:col + H].to(f))[:, :, None]
        elif gate is not None:
            g, col = gate
            y = y * torch.sigmoid(g[:, col:col + H * N].to(f).view(T, H, N))
        res = out.view(T, H, os_)
        res[:, :, :N] = y.to(out.dtype)
        if rotate is not None:
            cos, sin, positions = rotate
            assert os_ - N == xs - K
            half = cos.shape[1]
            t = xv[:, :, K:].clone()
            co, si = cos[positions.long()].to(f)[:, None, :], sin[positions.long()].to(f)[:, None, :]
            u, v = t[..., :half].clone(), t[..., half:2 * half].clone()
            t[..., :half], t[..., half:2 * half] = u * co - v * si, v * co + u * si
            res[:, :, N:] = t.to(out.dtype)

    def latent_attention(self, q, batch, kv, out, num_heads, value_dim, scale, workspace=None, window=-1, sink=None):
        """`window` -1: the cache entry's own; `sink` [H]: the softmax's denominator also holds exp(sink[h])."""
        f = self.f
        T, D = q.shape[0], kv.spec.head_dim
        qf = q.to(f).view(T, num_heads, D)
        window = kv.spec.window if window == -1 else window
        result = torch.zeros(T, num_heads, value_dim, dtype=f, device=q.device)
        for r in range(T):
            p, seg = int(batch.positions[r]), int(batch.row_segment[r])
            lo = max(0, p - window + 1) if window else 0
            js = torch.arange(lo, p + 1, device=q.device)
            pages = kv.block_table[seg, js // kv.page_size].long()
            assert bool((pages >= 0).all()), "a needed key lies in a page the block table does not hold"
            keys = kv.k_pages[pages, 0, js % kv.page_size, :].to(f)      # [n, D]
            scores = (qf[r] @ keys.t()) * scale                           # [H, n]
            if sink is None:
                weights = torch.softmax(scores, dim=-1)
            else:
                top = torch.maximum(scores.max(dim=-1).values, sink.to(f))
                e = torch.exp(scores - top[:, None])
                weights = e / (e.sum(dim=-1) + torch.exp(sink.to(f) - top))[:, None]
            result[r] = weights @ keys[:, :value_dim]
        out.copy_(result.view(T, num_heads * value_dim).to(out.dtype))

    def route_top(self, logits, chosen, share, scores="chosen"):
        z = logits.to(self.f)
        best, which = torch.topk(z, chosen.shape[1], dim=-1)
        chosen.copy_(which.to(torch.int32))
        if scores == "all":
            share.copy_(torch.gather(torch.softmax(z, dim=-1), 1, which).to(torch.float32))
        else:
            share.copy_(torch.softmax(best, dim=-1).to(torch.float32))

    def routed_experts(self, x, w_up, w_down, chosen, share, out, activation, workspace=None, limit=0.0, base=None):
        f = self.f
        result = torch.zeros(x.shape[0], w_down.shape[1], dtype=f) if base is None else base.to(f).clone()
        for r in range(x.shape[0]):
            for s in range(chosen.shape[1]):
                e = int(chosen[r, s])
                up = w_up[e].to(f) @ x[r].to(f)
                if activation == "relu2":
                    a = torch.relu(up) ** 2
                elif activation == "swiglu":
                    a = self._gated(up[0::2], up[1::2], "silu", 0.0)
                else:
                    a = self._gated(up[0::2], up[1::2], activation, limit)     # gate and up rows in turn
                result[r] += share[r, s].to(f) * (w_down[e].to(f) @ a.to(x.dtype).to(f))
        out.copy_(result.to(out.dtype))

    # ---- operators of the hashed pair embedding, gated heads and the matrix-state mixers ----------------------------
    def bigram_embed(self, table, batch, previous, h, buckets, mul_prev, mul_cur, vocab):
        ids = batch.token_ids.long()
        if batch.token_src is not None:
            ids = torch.where(batch.token_src >= 0, batch.last_tokens[batch.token_src.clamp(min=0).long()].long(), ids)
        for s in range(batch.num_segments):
            lo, n, slot = int(batch.seg_q_start[s]), int(batch.seg_q_len[s]), int(batch.seg_slot[s])
            for r in range(lo, lo + n):
                if int(batch.positions[r]) == 0:
                    row = buckets
                else:
                    before = int(ids[r - 1]) if r > lo else int(previous[slot])
                    row = (before * mul_prev + int(ids[r]) * mul_cur) % buckets
                h[r] += table[row].to(torch.float32)
            previous[slot] = int(ids[lo + n - 1])

    def head_gate(self, x, gate, num_heads, value_dim, scale, out, out_col=0, x_head_stride=None):
        f = self.f
        T = x.shape[0]
        y = x.to(f).view(T, num_heads, x_head_stride or value_dim)[:, :, :value_dim]
        if gate is not None:
            src, col = gate
            y = y * torch.sigmoid(src[:, col:col + num_heads].to(f))[:, :, None]
        out[:, out_col:out_col + num_heads * value_dim] = (y * scale).reshape(T, -1).to(out.dtype)

    def head_norm_gate(self, o, weight, eps, gate, activation, scale, out, out_col, num_heads, value_dim, scope="head"):
        f = self.f
        T = o.shape[0]
        y = o.to(f).view(T, num_heads, value_dim)
        if scope == "all":
            y = y * torch.rsqrt((y * y).mean(dim=(-2, -1), keepdim=True) + eps)
        else:
            y = y * torch.rsqrt((y * y).mean(dim=-1, keepdim=True) + eps)
        y = y * (weight.to(f).view(num_heads, value_dim) if weight.numel() == num_heads * value_dim else weight.to(f))
        src, col = gate
        g = src[:, col:col + num_heads * value_dim].to(f)
        g = g * torch.sigmoid(g) if activation == "silu" else torch.sigmoid(g)
        out[:, out_col:out_col + num_heads * value_dim] = (y.reshape(T, -1) * g * scale).to(out.dtype)

    def _segments(self, batch):
        for s in range(batch.num_segments):
            yield int(batch.seg_q_start[s]), int(batch.seg_q_len[s]), int(batch.seg_slot[s])

    def gated_linear_scan(self, proj, cols, z, tau, q_scale, batch, memory, out, H, D, Dv, workspace=None):
        f = self.f
        qc, kc, vc = cols
        for lo, n, slot in self._segments(batch):
            S = memory[slot].to(f)                                   # [H, D, Dv]
            for r in range(lo, lo + n):
                q = proj[r, qc:qc + H * D].to(f).view(H, D) * q_scale
                k = proj[r, kc:kc + H * D].to(f).view(H, D)
                v = proj[r, vc:vc + H * Dv].to(f).view(H, Dv)
                decay = torch.exp(torch.nn.functional.logsigmoid(z[r].to(f)).view(H, D) / tau)
                S = decay[:, :, None] * S + k[:, :, None] * v[:, None, :]
                out[r] = torch.einsum("hdv,hd->hv", S, q).reshape(-1).to(out.dtype)
            memory[slot] = S.to(memory.dtype)

    def lightning_scan(self, proj, cols, decay, batch, memory, out, H, D, Dv, workspace=None):
        """q, k, v = silu of the columns `cols` of `proj` (which are overwritten by them); S = decay[h] S + k v^T, out = S^T q."""
        f = self.f
        qc, kc, vc = cols
        for c, n in ((qc, H * D), (kc, H * D), (vc, H * Dv)):
            z = proj[:, c:c + n].to(f)
            proj[:, c:c + n] = (z * torch.sigmoid(z)).to(proj.dtype)
        for lo, n, slot in self._segments(batch):
            S = memory[slot].to(f)
            for r in range(lo, lo + n):
                q = proj[r, qc:qc + H * D].to(f).view(H, D)
                k = proj[r, kc:kc + H * D].to(f).view(H, D)
                v = proj[r, vc:vc + H * Dv].to(f).view(H, Dv)
                S = decay.to(f)[:, None, None] * S + k[:, :, None] * v[:, None, :]
                out[r] = torch.einsum("hdv,hd->hv", S, q).reshape(-1).to(out.dtype)
            memory[slot] = S.to(memory.dtype)

    def matrix_memory_scan(self, proj, cols, cap, q_scale, floor, batch, memory, normalizer, maximum, out, H, D, Dv, workspace=None):
        f = self.f
        qc, kc, vc, ic, fc = cols
        for lo, n, slot in self._segments(batch):
            S, nz, m = memory[slot].to(f), normalizer[slot].to(f), maximum[slot].to(f)
            for r in range(lo, lo + n):
                q = proj[r, qc:qc + H * D].to(f).view(H, D) * q_scale
                k = proj[r, kc:kc + H * D].to(f).view(H, D)
                v = proj[r, vc:vc + H * Dv].to(f).view(H, Dv)
                gi = cap * torch.tanh(proj[r, ic:ic + H].to(f) / cap)
                gf = torch.nn.functional.logsigmoid(cap * torch.tanh(proj[r, fc:fc + H].to(f) / cap))
                m_new = torch.maximum(gf + m, gi)
                keep, take = torch.exp(gf + m - m_new), torch.exp(gi - m_new)
                S = keep[:, None, None] * S + take[:, None, None] * k[:, :, None] * v[:, None, :]
                nz = keep[:, None] * nz + take[:, None] * k
                m = m_new
                denom = torch.maximum((nz * q).sum(dim=-1).abs(), torch.exp(-m)) + floor
                out[r] = (torch.einsum("hdv,hd->hv", S, q) / denom[:, None]).reshape(-1).to(out.dtype)
            memory[slot], normalizer[slot], maximum[slot] = S.to(memory.dtype), nz.to(normalizer.dtype), m.to(maximum.dtype)

    # ---- operators of token shift, plain activations and the delta-rule mixer --------------------------------------------
    def token_shift(self, x, weight, previous, batch, out):
        """out[r] = x[r] + (before - x[r]) * weight, before = the segment's row before r, or previous[slot] for its first
        row (zeros at position 0); previous[slot] then becomes the segment's last row."""
        f = self.f
        for lo, n, slot in self._segments(batch):
            rows = x[lo:lo + n].to(f)
            first = previous[slot].to(f) if int(batch.positions[lo]) > 0 else torch.zeros_like(rows[0])
            before = torch.cat([first[None, :], rows[:-1]], dim=0)
            out[lo:lo + n] = (rows + (before - rows) * weight.to(f)).to(out.dtype)
            previous[slot] = rows[-1].to(previous.dtype)

    def activation_(self, x, kind, cap=0.0):
        v = x.to(self.f)
        x.copy_((torch.tanh(v) if kind == "tanh" else torch.relu(v) ** 2 if kind == "relu2" else cap * torch.tanh(v / cap)).to(x.dtype))

    def delta_rule_scan(self, proj, cols, z, rate, unit_eps, batch, memory, out, H, D, workspace=None):
        """Per segment, from and into memory[slot] ([H, D, D]): w = exp(-rate sigmoid(z)), a = sigmoid(proj[a_col]),
        u = k / sqrt(sum k^2 + unit_eps); S = diag(w) S - (a u)(u^T S) + k v^T; out = S^T r."""
        f = self.f
        rc, kc, vc, ac = cols
        for lo, n, slot in self._segments(batch):
            S = memory[slot].to(f)
            for t in range(lo, lo + n):
                r, k, v, a = (proj[t, c:c + H * D].to(f).view(H, D) for c in (rc, kc, vc, ac))
                w = torch.exp(-rate * torch.sigmoid(z[t].to(f))).view(H, D)
                u = k / torch.sqrt((k * k).sum(dim=-1, keepdim=True) + unit_eps)
                read = torch.einsum("hk,hkv->hv", u, S)
                S = w[:, :, None] * S - (torch.sigmoid(a) * u)[:, :, None] * read[:, None, :] + k[:, :, None] * v[:, None, :]
                out[t] = torch.einsum("hkv,hk->hv", S, r).reshape(-1).to(out.dtype)
            memory[slot] = S.to(memory.dtype)
