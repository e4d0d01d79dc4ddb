"""Plain PyTorch statement of every kernel's contract (same call signatures as
``dlm_b200.ops.native.NativeOps``).  Two uses, both in tests only:

* the reference each kernel is compared with, alone, at sizes of the test's choosing;
* a stand-in backend that lets the host-side logic (cache, step function, scheduler,
  replay) run on a machine without a GPU.

It is not part of the package and the package never falls back to it.
"""
from __future__ import annotations

import torch


def _f(t):
    return t.to(torch.float32)


class _InOrder:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False

    def join(self):
        pass


class PlainOps:
    def check_errors(self):
        pass

    def branch(self, rows):
        return _InOrder()

    # ----------------------------------------------------------------- basic
    def embed(self, tokens, table):
        return _f(table[tokens.long()])

    def rmsnorm(self, x, w, eps, out_dtype, rows=None):
        if rows is not None:
            x = x[rows.long()]
        ms = (x * x).sum(-1, keepdim=True) / x.shape[-1]
        return ((x * (1.0 / torch.sqrt(ms + eps))) * w).to(out_dtype)

    # -------------------------------------------------------------- products
    def linear(self, a, w, bias, out_dtype):
        out = _f(a) @ _f(w).T
        if bias is not None:
            out = out + bias
        return out.to(out_dtype)

    def linear_add(self, a, w, resid):
        resid += _f(a) @ _f(w).T

    @staticmethod
    def _swiglu(acc, dtype):
        g, u = acc[:, 0::2], acc[:, 1::2]
        return ((g / (1.0 + torch.exp(-g))) * u).to(dtype)

    def linear_swiglu(self, a, w_gate_up):
        return self._swiglu(_f(a) @ _f(w_gate_up).T, a.dtype)

    def grouped_swiglu(self, a, w_gate_up, offsets, rows):
        E, N, K = w_gate_up.shape
        out = torch.zeros((rows.numel(), N // 2), dtype=a.dtype, device=a.device)
        off = offsets.tolist()
        for e in range(E):
            if off[e + 1] > off[e]:
                x = _f(a[rows[off[e]:off[e + 1]].long()])
                out[off[e]:off[e + 1]] = self._swiglu(x @ _f(w_gate_up[e]).T, a.dtype)
        return out

    def grouped_linear(self, a, w, offsets):
        E, N, K = w.shape
        out = torch.zeros((a.shape[0], N), dtype=torch.float32, device=a.device)
        off = offsets.tolist()
        for e in range(E):
            if off[e + 1] > off[e]:
                out[off[e]:off[e + 1]] = _f(a[off[e]:off[e + 1]]) @ _f(w[e]).T
        return out

    # ------------------------------------------------------------- attention
    def rope_kv_write(self, qkv, positions, inv_freq, rotary_dim, slots, k_cache, v_cache, nh, nkv, hd, out_dtype,
                      interleaved=False):
        T = qkv.shape[0]
        Q, KV = nh * hd, nkv * hd
        q = qkv[:, :Q].reshape(T, nh, hd).clone()
        k = qkv[:, Q:Q + KV].reshape(T, nkv, hd).clone()
        v = qkv[:, Q + KV:].reshape(T, nkv, hd)
        if inv_freq is not None:
            half = rotary_dim // 2
            ang = positions.to(torch.float32)[:, None] * inv_freq[None, :]
            sin, cos = torch.sin(ang)[:, None, :], torch.cos(ang)[:, None, :]
            for x in (q, k):
                if interleaved:
                    a, b = x[..., 0:rotary_dim:2].clone(), x[..., 1:rotary_dim:2].clone()
                    x[..., 0:rotary_dim:2] = a * cos - b * sin
                    x[..., 1:rotary_dim:2] = a * sin + b * cos
                else:
                    a, b = x[..., :half].clone(), x[..., half:rotary_dim].clone()
                    x[..., :half] = a * cos - b * sin
                    x[..., half:rotary_dim] = a * sin + b * cos
        if slots is not None:
            ps = k_cache.shape[2]
            sl = slots.long()
            ok = sl >= 0
            page, off = sl[ok] // ps, sl[ok] % ps
            k_cache[page, :, off, :] = k[ok].to(k_cache.dtype)
            v_cache[page, :, off, :] = v[ok].to(v_cache.dtype)
        return q.reshape(T, Q).to(out_dtype)

    def attention(self, q, k_cache, v_cache, block_table, cu_q, kv_len, window, scale, nh, nkv, hd, max_q_len,
                  max_kv_len, num_single=0):
        T = q.shape[0]
        ps = k_cache.shape[2]
        out = torch.zeros((T, nh * hd), dtype=torch.float32, device=q.device)
        cu, lens = cu_q.tolist(), kv_len.tolist()
        group = nh // nkv
        for r in range(block_table.shape[0]):
            q_len, n = cu[r + 1] - cu[r], lens[r]
            if q_len == 0:
                continue
            first = n - q_len
            lo = max(0, first - window + 1) if window > 0 else 0
            pos = torch.arange(lo, n, device=q.device)
            pages = block_table[r, (pos // ps).long()].long()
            assert int(pages.min()) >= 0, "a visible key has no page"
            k = _f(k_cache[pages, :, pos % ps, :])          # [n - lo, nkv, hd]
            v = _f(v_cache[pages, :, pos % ps, :])
            qs = _f(q[cu[r]:cu[r + 1]]).reshape(q_len, nh, hd)
            qpos = torch.arange(first, n, device=q.device)
            ok = pos[None, :] <= qpos[:, None]
            if window > 0:
                ok &= (qpos[:, None] - pos[None, :]) < window
            for h in range(nh):
                s = (qs[:, h, :] @ k[:, h // group, :].T) * scale
                s = s.masked_fill(~ok, float("-inf"))
                p = torch.softmax(s, dim=-1)
                out[cu[r]:cu[r + 1], h * hd:(h + 1) * hd] = p @ v[:, h // group, :]
        return out.to(q.dtype)

    # ------------------------------------------------------------------- moe
    def router_topk(self, h, w, E, k, norm, has_gate, norm_weight=None, eps=0.0, score="softmax", scale=1.0,
                    select_bias=None):
        if norm_weight is not None:
            h = self.rmsnorm(h, norm_weight, eps, torch.float32)
        logits = _f(h) @ _f(w).T
        gate = None
        if has_gate:
            gate = 1.0 / (1.0 + torch.exp(-logits[:, E]))
            logits = logits[:, :E]
        probs = torch.softmax(logits, dim=-1) if score == "softmax" else 1.0 / (1.0 + torch.exp(-logits))
        pick = probs if select_bias is None else probs + select_bias[None, :].to(probs.dtype)
        ids = torch.sort(pick, dim=-1, descending=True, stable=True).indices[:, :k]
        wts = torch.gather(probs, 1, ids)
        if norm:
            s = wts.sum(-1, keepdim=True)
            wts = torch.where(s > 0, wts / s, wts)
        return ids.to(torch.int32), wts * scale, gate

    def route(self, h, w, E, k, norm, has_gate, input_settled=False, **kw):
        ids, wts, gate = self.router_topk(h, w, E, k, norm, has_gate, **kw)
        return (ids, wts, gate) + tuple(self.moe_permute(ids, E))

    def moe_permute(self, ids, E):
        T, k = ids.shape
        flat = ids.reshape(-1).long()
        order = torch.sort(flat, stable=True).indices
        counts = torch.bincount(flat, minlength=E)
        offsets = torch.zeros(E + 1, dtype=torch.int32, device=ids.device)
        offsets[1:] = torch.cumsum(counts, 0).to(torch.int32)
        rows = (order // k).to(torch.int32)
        dest = torch.empty(T * k, dtype=torch.int32, device=ids.device)
        dest[order] = torch.arange(T * k, dtype=torch.int32, device=ids.device)
        return offsets, rows, dest.reshape(T, k)

    def moe_combine(self, y, dest, wts, shared, gate, resid):
        T, k = dest.shape
        acc = torch.zeros_like(resid)
        for j in range(k):
            acc = acc + wts[:, j:j + 1] * y[dest[:, j].long()]
        if shared is not None:
            g = gate[:, None] if gate is not None else 1.0
            acc = acc + g * shared
        resid += acc

    # -------------------------------------------------------------- sampling
    def argmax(self, logits):
        # the first maximum
        mx = logits.max(dim=-1, keepdim=True).values
        first = torch.argmax((logits == mx).to(torch.int32), dim=-1)
        return first.to(torch.int32)

    def sample(self, logits, params, top_k, u, seen_offsets, seen_tokens):
        """Same candidate order and cuts as the kernel, in double precision."""
        N, V = logits.shape
        out = torch.zeros(N, dtype=torch.int32, device=logits.device)
        for i in range(N):
            temp, top_p, min_p, pen = [float(x) for x in params[i]]
            z = logits[i].clone()
            if pen != 1.0 and seen_offsets is not None:
                seen = seen_tokens[int(seen_offsets[i]):int(seen_offsets[i + 1])].long()
                z[seen] = torch.where(z[seen] > 0, z[seen] / pen, z[seen] * pen)
            if not temp > 0:
                out[i] = int(self.argmax(z[None])[0])
                continue
            order = torch.sort(z, descending=True, stable=True).indices
            k = int(top_k[i])
            if 0 < k < V:
                order = order[:k]
            p = torch.exp((z[order] - z[order[0]]).double() / temp)
            if 0.0 < top_p < 1.0:
                cum = torch.cumsum(p, 0)
                cut = int(torch.nonzero(cum >= top_p * cum[-1])[0]) + 1
                order, p = order[:cut], p[:cut]
            if min_p > 0:
                keep = max(int((p >= min(min_p, 1.0)).sum()), 1)
                order, p = order[:keep], p[:keep]
            cum = torch.cumsum(p, 0)
            hit = torch.nonzero(cum > float(u[i]) * cum[-1])
            out[i] = int(order[int(hit[0])]) if hit.numel() else int(order[-1])
        return out
