"""Plain torch statements of what each CUDA kernel computes, for tests only.

Two uses.  The ``-m gpu`` tests call each kernel alone and compare it with the function of
the same name here, computed in float32 (or float64) on the CPU.  The CPU tests put an
instance of :class:`ReferenceKernels` in the place of the CUDA kernel set, so that the
step function, the cache manager and the scheduler can be exercised on a machine
without a GPU; the package itself never does that and fails if its CUDA libraries
cannot be loaded.

Every function takes the same arguments as the method of the same name of
``infurnace_b200.kernels.cuda.CudaKernels``.
"""
from __future__ import annotations

import torch


class ReferenceKernels:
    name = "reference"

    def __init__(self, compute_dtype=torch.float32, fold=True):
        self.cd = compute_dtype
        self.fold = fold          # offer the folded norm (for few rows, as the CUDA kernels do)

    # ------------------------------------------------------------------ embedding
    def embed(self, table, ids, out):
        out.copy_(table[ids.long()].to(out.dtype))

    def random_normal(self, out, seed64, mean, std):
        """out[i] = mean + std * z_i, the counter-based values of weights/random_init.py."""
        from infurnace_b200.weights.random_init import normal_values
        out.copy_(normal_values(seed64, out.numel(), mean, std).view(out.shape).to(out.dtype))

    # ------------------------------------------------------------------ norm
    def rmsnorm(self, x, weight, eps, out, delta=None, rows=None):
        """x is the float32 residual stream [N, H]; delta ([N, H] or [S, N, H], summed over S)
        is what the previous part adds to it.  Without ``rows``: x += delta in place and
        out[n] = norm(x[n]).  With ``rows`` (int32 [M]): x is left as it is and
        out[m] = norm(x[rows[m]] + delta[rows[m]]).  norm(v) = v * rsqrt(mean(v^2) + eps) *
        weight, statistics in 32-bit, rounded to out's dtype."""
        d = None
        if delta is not None:
            d = delta.to(torch.float32)
            if d.dim() == 3:
                d = d.sum(0)
        if rows is None:
            if d is not None:
                x.add_(d)
            src = x
        else:
            src = x[rows.long()]
            if d is not None:
                src = src + d[rows.long()]
        s = src.to(self.cd)
        y = s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + eps) * weight.to(self.cd)
        out.copy_(y.to(out.dtype))

    # ------------------------------------------------------------------ matrix products
    def linear(self, x, w, out, epilogue="none", row_scale=None):
        """out = x @ w^T (w is [out_features, in_features]); accumulation in 32-bit.
        epilogue "silu_gate": w is [2I, K] with the gate rows first; out[n, j] =
        silu(y[n, j]) * y[n, I + j].  row_scale (partials, parts, eps, width): row n of the
        product is multiplied by rsqrt(sum_p partials[p, n] / width + eps) first."""
        y = x.to(self.cd) @ w.to(self.cd).t()
        if row_scale is not None:
            partials, parts, eps, width = row_scale
            r = torch.rsqrt(partials[:parts].to(self.cd).sum(dim=0) / width + eps)
            y = y * r[:, None]
        if epilogue == "silu_gate":
            half = y.shape[1] // 2
            g, u = y[:, :half], y[:, half:]
            y = g * torch.sigmoid(g) * u
        elif epilogue == "relu2":
            y = torch.relu(y) ** 2
        elif epilogue == "silu":
            y = y * torch.sigmoid(y)
        elif epilogue == "sigmoid":
            y = torch.sigmoid(y)
        elif epilogue == "gelu_tanh":
            y = 0.5 * y * (1 + torch.tanh(0.7978845608028654 * (y + 0.044715 * y ** 3)))
        elif epilogue == "tanh":
            y = torch.tanh(y)
        elif epilogue != "none":
            raise ValueError(epilogue)
        out.copy_(y.to(out.dtype))

    def can_fold_norm(self, n, dtype, w, epilogue="none"):
        return bool(self.fold) and 0 < n <= 64

    def fold_parts(self, out_features, n=None, w=None):
        return -(-out_features // 16)

    def linear_residual_norm(self, a, w, x, norm_weight, out, partials):
        """x += a @ w^T; out = x * norm_weight; partials[p, n] = sum of x[n, 16p:16p+16]^2."""
        x.add_((a.to(self.cd) @ w.to(self.cd).t()).to(x.dtype))
        v = x.to(self.cd)
        out.copy_((v * norm_weight.to(self.cd)[None, :]).to(out.dtype))
        o = v.shape[1]
        parts = self.fold_parts(o)
        sq = torch.zeros(v.shape[0], parts * 16, dtype=self.cd)
        sq[:, :o] = v * v
        partials[:parts].copy_(sq.view(v.shape[0], parts, 16).sum(dim=2).t().to(partials.dtype))

    # ------------------------------------------------------------------ q/k norm, rotation, store
    def rope_table(self, positions, inv_freq, out, gain=1.0):
        """out[tok] = gain * (cos, sin) pairs of positions[tok] * inv_freq[i], interleaved: [tokens, 2 * len(inv_freq)]."""
        ang = positions.to(torch.float32)[:, None] * inv_freq.to(torch.float32)[None, :]
        out.copy_(torch.stack((ang.cos() * gain, ang.sin() * gain), dim=-1).flatten(-2))

    def qk_norm_rope_store(self, qkv, num_heads, num_kv_heads, head_dim, q_weight, k_weight, eps,
                           inv_freq, rotary_dim, interleaved, positions, slot_mapping, kv_pages, rope_table=None):
        """In place on qkv [N, (nq + 2 nkv) d]: per-head RMSNorm of the q and k heads (when
        the weights are given), rotation of q and k by the token's position (when inv_freq
        is given), then k and v are written to the pages at ``slot_mapping`` (slot =
        page * page_size + offset; -1: not stored).  kv_pages: [pages, 2, nkv, page_size, d]."""
        N = qkv.shape[0]
        nq, nkv, d = num_heads, num_kv_heads, head_dim
        q = qkv[:, : nq * d].to(self.cd).reshape(N, nq, d).clone()
        k = qkv[:, nq * d: (nq + nkv) * d].to(self.cd).reshape(N, nkv, d).clone()
        v = qkv[:, (nq + nkv) * d:].view(N, nkv, d)

        def norm(t, w):
            return t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps) * w.to(self.cd)

        if q_weight is not None:
            q = norm(q, q_weight)
        if k_weight is not None:
            k = norm(k, k_weight)
        if inv_freq is not None:
            if rope_table is not None:
                pairs = rope_table.view(N, rotary_dim // 2, 2)
                cos, sin = pairs[..., 0].to(self.cd)[:, None, :], pairs[..., 1].to(self.cd)[:, None, :]
            else:
                ang = positions.to(torch.float32)[:, None] * inv_freq.to(torch.float32)[None, :]
                cos, sin = ang.cos().to(self.cd)[:, None, :], ang.sin().to(self.cd)[:, None, :]

            def rot(t):
                r, rest = t[..., :rotary_dim], t[..., rotary_dim:]
                if interleaved:
                    a, b = r[..., 0::2], r[..., 1::2]
                    o = torch.stack((a * cos - b * sin, b * cos + a * sin), dim=-1).flatten(-2)
                else:
                    a, b = r[..., : rotary_dim // 2], r[..., rotary_dim // 2:]
                    o = torch.cat((a * cos - b * sin, b * cos + a * sin), dim=-1)
                return torch.cat((o, rest), dim=-1)

            q, k = rot(q), rot(k)
        qkv[:, : nq * d] = q.reshape(N, nq * d).to(qkv.dtype)
        qkv[:, nq * d: (nq + nkv) * d] = k.reshape(N, nkv * d).to(qkv.dtype)
        if slot_mapping is not None:
            ps = kv_pages.shape[3]
            kk = k.to(kv_pages.dtype)
            for n in range(N):
                s = int(slot_mapping[n])
                if s < 0:
                    continue
                kv_pages[s // ps, 0, :, s % ps, :] = kk[n]
                kv_pages[s // ps, 1, :, s % ps, :] = v[n].to(kv_pages.dtype)

    # ------------------------------------------------------------------ attention over pages
    def paged_attention(self, qkv, num_heads, num_kv_heads, head_dim, kv_pages, block_tables, cu_q,
                        seq_lens, out, scale, window, max_q_len, max_seq_len, min_q_len=1, weight_terms=1):
        """For request r the query tokens are rows cu_q[r] .. cu_q[r+1]-1 of qkv (their q
        heads are the first nq*d columns); the last of them stands at position
        seq_lens[r]-1.  A query at position p attends to the keys at positions
        max(0, p-window+1) .. p (window 0: from 0), read from the pages that
        block_tables[r] names.  Softmax in 32-bit.  A query with no visible key gives 0."""
        nq, nkv, d = num_heads, num_kv_heads, head_dim
        ps = kv_pages.shape[3]
        R = cu_q.numel() - 1
        g = nq // nkv
        for r in range(R):
            q0, q1 = int(cu_q[r]), int(cu_q[r + 1])
            n, L = q1 - q0, int(seq_lens[r])
            if n == 0:
                continue
            if L <= 0:
                out[q0:q1] = 0
                continue
            first = 0
            if window:
                first = max(0, (L - n) - window + 1)
            pos = torch.arange(first, L)
            pages = block_tables[r].long()[pos // ps]
            k = kv_pages[pages, 0, :, pos % ps, :].to(self.cd)      # [keys, nkv, d]
            v = kv_pages[pages, 1, :, pos % ps, :].to(self.cd)
            q = qkv[q0:q1, : nq * d].to(self.cd).view(n, nq, d)
            k = k.repeat_interleave(g, dim=1)
            v = v.repeat_interleave(g, dim=1)
            s = torch.einsum("nhd,khd->hnk", q, k) * scale
            qpos = torch.arange(L - n, L)
            vis = pos[None, :] <= qpos[:, None]
            if window:
                vis &= (qpos[:, None] - pos[None, :]) < window
            s = s.masked_fill(~vis[None], float("-inf"))
            p = torch.softmax(s.float(), dim=-1).to(self.cd)
            o = torch.einsum("hnk,khd->nhd", p, v)
            out[q0:q1] = o.reshape(n, nq * d).to(out.dtype)

    # ------------------------------------------------------------------ post-norm sublayers, recurrence, talking attention
    def embed_sinusoid(self, table, ids, positions, inv_freq, out, half=None):
        """out[n] = table[ids[n]] + e, e[2i] = sin(positions[n] * inv_freq[i]), e[2i+1] = cos of that angle."""
        ang = positions.to(torch.float64)[:, None] * inv_freq.to(torch.float64)[None, :]
        e = torch.stack((ang.sin(), ang.cos()), dim=-1).flatten(-2)[:, : out.shape[1]]
        out.copy_((table[ids.long()].to(torch.float64) + e).to(out.dtype))
        if half is not None:
            half.copy_(out.to(half.dtype))

    def residual_postnorm(self, x, y, g, scale, eps, half=None):
        """x += y / sqrt(mean(y^2) + eps) * g * scale."""
        v = y.to(self.cd)
        x.add_((v / torch.sqrt(v.pow(2).mean(-1, keepdim=True) + eps) * g.to(self.cd).reshape(()) * scale.to(self.cd)).to(x.dtype))
        if half is not None:
            half.copy_(x.to(half.dtype))

    def cast_rows(self, x, out):
        out.copy_(x.to(out.dtype))

    def wide_norm_store(self, proj, q_width, k_width, v_col, head_dim, q_weight, k_weight, eps, q_out, slot_mapping, kv_pages):
        """q_out = whole-row RMSNorm of proj[:, :q_width] times q_weight; key page = the same of the next k_width
        columns; value page = those columns as they are (v_col < 0) or proj[:, v_col : v_col + k_width]."""
        def norm(t, w):
            return t if w is None else t / torch.sqrt(t.pow(2).mean(-1, keepdim=True) + eps) * w.to(self.cd)
        q = proj[:, :q_width].to(self.cd)
        k = proj[:, q_width: q_width + k_width].to(self.cd)
        v = k if v_col < 0 else proj[:, v_col: v_col + k_width].to(self.cd)
        q_out.copy_(norm(q, q_weight).to(q_out.dtype))
        if slot_mapping is None:
            return
        ps, g = kv_pages.shape[3], k_width // head_dim
        kn = norm(k, k_weight).to(kv_pages.dtype).view(-1, g, head_dim)
        vv = v.to(kv_pages.dtype).view(-1, g, head_dim)
        for n in range(proj.shape[0]):
            s = int(slot_mapping[n])
            if s >= 0:
                kv_pages[s // ps, 0, :, s % ps, :] = kn[n]
                kv_pages[s // ps, 1, :, s % ps, :] = vv[n]

    def gated_scan_slabs(self, dim, vdim):
        return 1

    def gated_scan(self, proj, q_col, f_col, v_col, bias, lower, norm_weight, eps, state, state_slots, cu_q, seq_lens, out,
                   heads, dim, vdim, raw=None, max_q_len=1):
        """Token by token for each request r (rows cu_q[r] .. cu_q[r+1]-1; seq_lens[r] == 0: padding, skipped), on the
        state rows state[state_slots[r]]: S = f[:, None] * S + (1 - f)[:, None] * v[None, :], o = S^T q, with
        q = silu(q_raw), f = lower + (1 - lower) * sigmoid(f_raw + bias); out = o / rms(o) * norm_weight per head."""
        hd, hv = heads * dim, heads * vdim
        lo, b, nw = lower.to(self.cd), bias.to(self.cd), norm_weight.to(self.cd)
        for r in range(seq_lens.numel()):
            if int(seq_lens[r]) <= 0:
                continue
            S = state[int(state_slots[r])].to(self.cd)
            for t in range(int(cu_q[r]), int(cu_q[r + 1])):
                qr = proj[t, q_col: q_col + hd].to(self.cd)
                q = (qr * torch.sigmoid(qr)).view(heads, dim)
                f = (lo + (1 - lo) * torch.sigmoid(proj[t, f_col: f_col + hd].to(self.cd) + b)).view(heads, dim)
                v = proj[t, v_col: v_col + hv].to(self.cd).view(heads, vdim)
                S = f[:, :, None] * S + (1 - f)[:, :, None] * v[:, None, :]
                o = torch.einsum("hde,hd->he", S, q)
                o = o / torch.sqrt(o.pow(2).mean(-1, keepdim=True) + eps) * nw
                out[t] = o.reshape(hv).to(out.dtype)
            state[int(state_slots[r])] = S.to(state.dtype)

    def attention_talk(self, q, num_heads, num_kv_heads, head_dim, kv_pages, block_tables, cu_q, seq_lens, out, scale,
                       chunk=0, slope_exponent=0.0, talk=None, gate=None, gate_col=0, max_q_len=0, max_seq_len=0):
        """Per request, the query at position p sees keys (p // chunk) * chunk .. p (chunk 0: 0 .. p) from the pages:
        a[j] = scale * q_j . k - slope_j * (p - s); b = talk @ a over the heads; softmax over the keys; o = P V;
        out = o * sigmoid(gate)."""
        H, G, d = num_heads, num_kv_heads, head_dim
        ps = kv_pages.shape[3]
        slopes = torch.tensor([2.0 ** (-slope_exponent * (j + 1) / H) if slope_exponent else 0.0 for j in range(H)], dtype=self.cd)
        for r in range(seq_lens.numel()):
            q0, q1, L = int(cu_q[r]), int(cu_q[r + 1]), int(seq_lens[r])
            if L <= 0:
                out[q0:q1] = 0
                continue
            for t in range(q0, q1):
                p = L - (q1 - q0) + (t - q0)
                first = (p // chunk) * chunk if chunk else 0
                pos = torch.arange(first, p + 1)
                pages = block_tables[r].long()[pos // ps]
                k = kv_pages[pages, 0, :, pos % ps, :].to(self.cd).repeat_interleave(H // G, dim=1)      # [keys, H, d]
                v = kv_pages[pages, 1, :, pos % ps, :].to(self.cd).repeat_interleave(H // G, dim=1)
                a = torch.einsum("hd,shd->hs", q[t].to(self.cd).view(H, d), k) * scale - slopes[:, None] * (p - pos).to(self.cd)[None]
                if talk is not None:
                    a = talk.to(self.cd) @ a
                o = torch.einsum("hs,shd->hd", torch.softmax(a, dim=-1), v).reshape(H * d)
                if gate is not None:
                    o = o * torch.sigmoid(gate[t, gate_col: gate_col + H * d].to(self.cd))
                out[t] = o.to(out.dtype)

    # ------------------------------------------------------------------ sandwich-norm blocks, loops, token side input
    def residual_norm_update(self, x, y, post_weight, eps, out=None, next_weight=None, y2=None, scale=1.0, scale2=1.0):
        """x += y / sqrt(mean(y^2) + eps) * post_weight (float32, in place); with y2, y stands for scale * y + scale2 * y2.  ``out``: the updated rows for the next
        product, x / sqrt(mean(x^2) + eps) * next_weight, or x itself when next_weight is None, in out's dtype."""
        v = y.to(self.cd) * scale
        if y2 is not None:
            v = v + y2.to(self.cd) * scale2
        x.add_((v / torch.sqrt(v.pow(2).mean(-1, keepdim=True) + eps) * post_weight.to(self.cd)).to(x.dtype))
        if out is not None:
            u = x.to(self.cd)
            if next_weight is not None:
                u = u / torch.sqrt(u.pow(2).mean(-1, keepdim=True) + eps) * next_weight.to(self.cd)
            out.copy_(u.to(out.dtype))

    def add_rows(self, x, rows=None, vec=None, accumulate=True):
        """x (+)= rows + vec: rows float32 of x's shape, vec one row for all."""
        t = torch.zeros_like(x, dtype=self.cd)
        if accumulate:
            t = t + x.to(self.cd)
        if rows is not None:
            t = t + rows.to(self.cd)
        if vec is not None:
            t = t + vec.to(self.cd)[None, :]
        x.copy_(t.to(x.dtype))

    def scaled_sum(self, total, d, scale, accumulate=True, copy=None):
        """total (+)= scale * d; ``copy`` also gets the new total."""
        t = d.to(self.cd) * scale
        if accumulate:
            t = t + total.to(self.cd)
        total.copy_(t.to(total.dtype))
        if copy is not None:
            copy.copy_(total.to(copy.dtype))

    def token_side_gate(self, z, table, ids, offset, activation, out):
        """out[n, j] = act(z[n, j]) * table[ids[n], offset + j]."""
        y = z.to(self.cd)
        if activation == "gelu_tanh":
            y = 0.5 * y * (1 + torch.tanh(0.7978845608028654 * (y + 0.044715 * y ** 3)))
        elif activation == "silu":
            y = y * torch.sigmoid(y)
        else:
            raise ValueError(activation)
        out.copy_((y * table[ids.long(), offset: offset + z.shape[1]].to(self.cd)).to(out.dtype))

    def softcap(self, logits, cap):
        logits.copy_((cap * torch.tanh(logits.to(self.cd) / cap)).to(logits.dtype))

    # ------------------------------------------------------------------ recurrences with state slots
    def token_shift_mix(self, h, last, state_slots, cu_q, seq_lens, mu, out):
        """out[s, t] = h[t] + (h'[t] - h[t]) * mu[s], h' the row before t in its request, or for a request's first
        row of the step last[slot] (which then becomes the request's last row of the step)."""
        for r in range(seq_lens.numel()):
            if int(seq_lens[r]) <= 0:
                continue
            a, b, slot = int(cu_q[r]), int(cu_q[r + 1]), int(state_slots[r])
            cur = h[a:b].to(self.cd)
            prev = torch.cat((last[slot].to(self.cd)[None, :], cur[:-1]), dim=0)
            for s_ in range(mu.shape[0]):
                out[s_, a:b] = (cur + (prev - cur) * mu[s_].to(self.cd)).to(out.dtype)
            last[slot] = cur[-1].to(last.dtype)

    def linear_scan(self, q, k, v, w, heads, dim, vdim, state, state_slots, cu_q, seq_lens, out, eps, decay=None, w_bias=None,
                    key_scale=1.0, bonus=None, norm_weight=None, gate=None, max_q_len=1):
        """Per request and head, token by token on state[slot] [heads, dim, vdim] (float32): with the decay
        d = decay[head] (constant) or exp(-exp(w + w_bias)) per key channel, kk = k * key_scale:
        without bonus  S = d S + kk v^T, o = S^T q;  with bonus u  o = (S + u kk v^T)^T q, then S = d S + kk v^T.
        out = o / rms(o) per head (* norm_weight [heads * vdim]) (* silu(gate))."""
        for r in range(seq_lens.numel()):
            if int(seq_lens[r]) <= 0:
                continue
            slot = int(state_slots[r])
            S = state[slot].to(self.cd)
            for t in range(int(cu_q[r]), int(cu_q[r + 1])):
                qt = q[t].to(self.cd).view(heads, dim)
                kt = k[t].to(self.cd).view(heads, dim) * key_scale
                vt = v[t].to(self.cd).view(heads, vdim)
                if decay is not None:
                    d = decay.to(self.cd)[:, None].expand(heads, dim)
                else:
                    d = torch.exp(-torch.exp(w[t].to(self.cd) + w_bias.to(self.cd))).view(heads, dim)
                kv = kt[:, :, None] * vt[:, None, :]
                if bonus is not None:
                    o = torch.einsum("hde,hd->he", S + bonus.to(self.cd).view(heads, dim)[:, :, None] * kv, qt)
                    S = d[:, :, None] * S + kv
                else:
                    S = d[:, :, None] * S + kv
                    o = torch.einsum("hde,hd->he", S, qt)
                o = (o / torch.sqrt(o.pow(2).mean(-1, keepdim=True) + eps)).reshape(heads * vdim)
                if norm_weight is not None:
                    o = o * norm_weight.to(self.cd)
                if gate is not None:
                    g = gate[t].to(self.cd)
                    o = o * g * torch.sigmoid(g)
                out[t] = o.to(out.dtype)
            state[slot] = S.to(state.dtype)

    def gated_unit_scan(self, proj, z_bias, x_bias, state, state_slots, cu_q, seq_lens, out, max_q_len=1):
        """proj [n, 3 width] holds z_raw | x_raw | g.  z = sigmoid(z_raw + z_bias), u = x_raw + x_bias,
        c = u + 1/2 where u >= 0 else sigmoid(u); S = (1 - z) S + z c on state[slot] [width]; out = S * silu(g)."""
        n = state.shape[1]
        for r in range(seq_lens.numel()):
            if int(seq_lens[r]) <= 0:
                continue
            slot = int(state_slots[r])
            S = state[slot].to(self.cd)
            for t in range(int(cu_q[r]), int(cu_q[r + 1])):
                row = proj[t].to(self.cd)
                z = torch.sigmoid(row[:n] + z_bias.to(self.cd))
                u = row[n:2 * n] + x_bias.to(self.cd)
                c = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
                S = (1 - z) * S + z * c
                g = row[2 * n:]
                out[t] = (S * g * torch.sigmoid(g)).to(out.dtype)
            state[slot] = S.to(state.dtype)

    # ------------------------------------------------------------------ the real-gated linear recurrent unit
    def rglru_conv(self, proj, x_col, x_bias, conv_weight, conv_bias, state, state_slots, cu_q, seq_lens, req_index, u, u_blocks,
                   offsets, tile_block=None, tile=0):
        """u_t = conv_bias + sum_j conv_weight[:, j] * xin_(t - taps + 1 + j), xin = proj[:, x_col:x_col + width] + x_bias, per
        request from the inputs its slot kept; u token-major float32 and block-major in u_blocks [blocks, seg, bs]."""
        n, width = u.shape
        blocks, seg, rowlen = u_blocks.shape
        bs = width // blocks
        taps = conv_weight.shape[1]
        K = taps - 1
        xin = proj[:, x_col:x_col + width].to(self.cd) + x_bias.to(self.cd)
        w, b = conv_weight.to(self.cd), conv_bias.to(self.cd)
        offsets.copy_(torch.arange(blocks + 1, dtype=offsets.dtype) * seg)
        if tile_block is not None:
            tile_block.copy_((torch.arange(tile_block.numel()) // (seg // tile)).to(tile_block.dtype))
        for r in range(seq_lens.numel()):
            a, e = int(cu_q[r]), int(cu_q[r + 1])
            if e == a:
                continue
            if int(seq_lens[r]) <= 0:
                u[a:e] = 0
                continue
            st = state[int(state_slots[r])]
            hist = torch.cat((st[:K].to(self.cd), xin[a:e]), dim=0) if K else xin[a:e]
            acc = b.expand(e - a, width).clone()
            for j in range(taps):
                acc = acc + w[:, j] * hist[j:j + e - a]
            u[a:e] = acc.to(u.dtype)
            if K:
                st[:K] = hist[hist.shape[0] - K:].to(st.dtype)
        first = u.view(n, blocks, bs).transpose(0, 1).to(u_blocks.dtype)
        u_blocks[:, :n, :bs] = first
        if rowlen == 2 * bs:           # two terms: the roundings, then what each rounding left out
            u_blocks[:, :n, bs:] = (u.view(n, blocks, bs).transpose(0, 1).to(self.cd) - first.to(self.cd)).to(u_blocks.dtype)

    def rglru_scan(self, gates, a_bias, i_bias, decay, decay_scale, u, proj, y_col, y_bias, state, state_slots, cu_q, seq_lens, out,
                   max_q_len=1):
        """r = sigmoid(gates_r + a_bias), i = sigmoid(gates_i + i_bias), a = exp(-decay_scale * r * softplus(decay)),
        S <- a S + sqrt(1 - a^2) * i * u from the slot's state; out = S * gelu_tanh(proj[:, y_col:y_col + width] + y_bias)."""
        n, width = out.shape
        blocks, seg, two_bs = gates.shape
        bs = two_bs // 2
        g = gates[:, :n].to(self.cd)
        r = torch.sigmoid(g[..., :bs].transpose(0, 1).reshape(n, width) + a_bias.to(self.cd))
        i = torch.sigmoid(g[..., bs:].transpose(0, 1).reshape(n, width) + i_bias.to(self.cd))
        loga = -decay_scale * r * torch.nn.functional.softplus(decay.to(self.cd))
        a = torch.exp(loga)
        term = torch.sqrt(torch.clamp(-torch.expm1(2 * loga), min=0)) * i * u.to(self.cd)
        y = torch.nn.functional.gelu(proj[:, y_col:y_col + width].to(self.cd) + y_bias.to(self.cd), approximate="tanh")
        for q in range(seq_lens.numel()):
            lo, hi = int(cu_q[q]), int(cu_q[q + 1])
            if int(seq_lens[q]) <= 0:
                out[lo:hi] = 0
                continue
            S = state[int(state_slots[q])].to(self.cd)
            for t in range(lo, hi):
                S = a[t] * S + term[t]
                out[t] = (S * y[t]).to(out.dtype)
            if hi > lo:
                state[int(state_slots[q])] = S.to(state.dtype)

    # ------------------------------------------------------------------ attention with rotated values
    @staticmethod
    def _turn(t, cos, sin, dims, interleaved):
        """Rotate the first ``dims`` entries of the last axis of t [n, heads, d]; cos, sin [n, 1, dims / 2]."""
        out = t.clone()
        if interleaved:
            a, b = t[..., 0:dims:2], t[..., 1:dims:2]
            out[..., 0:dims:2], out[..., 1:dims:2] = a * cos - b * sin, b * cos + a * sin
        else:
            a, b = t[..., : dims // 2], t[..., dims // 2: dims]
            out[..., : dims // 2], out[..., dims // 2: dims] = a * cos - b * sin, b * cos + a * sin
        return out

    def _table(self, table):
        pairs = table.view(table.shape[0], -1, 2).to(self.cd)
        return pairs[..., 0][:, None, :], pairs[..., 1][:, None, :]

    def rotary_store(self, qkv, num_heads, num_kv_heads, head_dim, value_head_dim, qk_table, rotary_dim, interleaved, value_eps,
                     v_table, v_interleaved, q_out, k_pages, v_pages, slot_mapping, values_are_keys=False):
        """qkv [n, H d + G d + G dv] ([n, H d + G d] with ``values_are_keys``: a value head is its key head before rotation).  q and k are rotated by the angles of qk_table ([n, rotary_dim] (cos, sin)
        pairs; None: not rotated); each value head is divided by its root mean square (value_eps None: not) and
        rotated over its whole width by v_table (None: not).  q_out gets q; k and v go to their pages
        [pages, G, page_size, width] at slot_mapping (None: nothing is stored)."""
        n, H, G, d, dv = qkv.shape[0], num_heads, num_kv_heads, head_dim, value_head_dim
        q = qkv[:, : H * d].to(self.cd).reshape(n, H, d)
        k = qkv[:, H * d: (H + G) * d].to(self.cd).reshape(n, G, d)
        v = k.clone() if values_are_keys else qkv[:, (H + G) * d:].to(self.cd).reshape(n, G, dv)
        if qk_table is not None:
            c, s_ = self._table(qk_table)
            q, k = self._turn(q, c, s_, rotary_dim, interleaved), self._turn(k, c, s_, rotary_dim, interleaved)
        if value_eps is not None:
            v = v / torch.sqrt(v.pow(2).mean(-1, keepdim=True) + value_eps)
        if v_table is not None:
            c, s_ = self._table(v_table)
            v = self._turn(v, c, s_, dv, v_interleaved)
        q_out.copy_(q.reshape(n, H * d).to(q_out.dtype))
        if slot_mapping is not None:
            ps = k_pages.shape[2]
            for t in range(n):
                s_ = int(slot_mapping[t])
                if s_ >= 0:
                    k_pages[s_ // ps, :, s_ % ps, :] = k[t].to(k_pages.dtype)
                    v_pages[s_ // ps, :, s_ % ps, :] = v[t].to(v_pages.dtype)

    def rotate_rows(self, rows, table, heads, width, dims, interleaved, back=False):
        """rows [n, heads * width] in place: every head's first ``dims`` entries turned by the token's angles, forward or back."""
        c, s_ = self._table(table)
        t = self._turn(rows.to(self.cd).view(rows.shape[0], heads, width), c, -s_ if back else s_, dims, interleaved)
        rows.copy_(t.reshape(rows.shape).to(rows.dtype))

    def paged_attention_streams(self, q, num_heads, num_kv_heads, head_dim, value_head_dim, k_pages, v_pages, block_tables, cu_q,
                                seq_lens, out, scale, window, out_table, out_interleaved, max_q_len=0, max_seq_len=0):
        """Causal softmax attention of q [n, H d] over the keys and values of the request's pages (streams
        [pages, G, page_size, width]); the output of every head is then rotated BACK by the angles of out_table (the
        query token's row; None: not)."""
        H, G, d, dv = num_heads, num_kv_heads, head_dim, value_head_dim
        ps = k_pages.shape[2]
        for r in range(seq_lens.numel()):
            q0, q1, L = int(cu_q[r]), int(cu_q[r + 1]), int(seq_lens[r])
            if L <= 0:
                out[q0:q1] = 0
                continue
            for t in range(q0, q1):
                p = L - (q1 - q0) + (t - q0)
                first = max(0, p - window + 1) if window else 0
                pos = torch.arange(first, p + 1)
                pages = block_tables[r].long()[pos // ps]
                kk = k_pages[pages, :, pos % ps, :].to(self.cd).repeat_interleave(H // G, dim=1)
                vv = v_pages[pages, :, pos % ps, :].to(self.cd).repeat_interleave(H // G, dim=1)
                a = torch.einsum("hd,shd->hs", q[t].to(self.cd).view(H, d), kk) * scale
                o = torch.einsum("hs,shd->hd", torch.softmax(a, dim=-1), vv)[None]
                if out_table is not None:
                    c, s_ = self._table(out_table[t:t + 1])
                    o = self._turn(o, c, -s_, dv, out_interleaved)
                out[t] = o.reshape(H * dv).to(out.dtype)

    # ------------------------------------------------------------------ routed experts
    def moe_route(self, logits, top, ids, gates, experts=None, scoring="chosen", groups=None, weight_scale=1.0):
        """ids[n] = the ``top`` largest scores' indices, largest first (the lower index among equals).  scoring "chosen":
        scores are the logits, gates[n] = softmax over the chosen logits.  scoring "all": scores are the softmax over all
        experts, limited to the ``keep`` groups of neighbours with the largest best score when ``groups`` = (count, keep);
        gates[n] = score * weight_scale.  Only the first ``experts`` columns of ``logits`` are the router's."""
        z = logits[:, :experts if experts is not None else logits.shape[1]].to(self.cd)
        if scoring == "sigmoid":         # sigmoid(z) per expert; the order of the logits is the order of the scores
            val, idx = torch.sort(z, dim=-1, descending=True, stable=True)
            ids.copy_(idx[:, :top].to(ids.dtype))
            gates.copy_((torch.sigmoid(val[:, :top]) * weight_scale).to(gates.dtype))
            return
        if scoring == "chosen":
            val, idx = torch.sort(z, dim=-1, descending=True, stable=True)
            ids.copy_(idx[:, :top].to(ids.dtype))
            gates.copy_(torch.softmax(val[:, :top], dim=-1).to(gates.dtype))
            return
        score = torch.softmax(z, dim=-1)
        masked = score.clone()
        if groups is not None and groups[1] < groups[0]:
            count, keep = groups
            n, E = score.shape
            best = score.view(n, count, E // count).max(dim=-1).values
            order = torch.sort(best, dim=-1, descending=True, stable=True).indices[:, :keep]
            allowed = torch.zeros(n, count, dtype=torch.bool)
            allowed.scatter_(1, order, True)
            masked[~allowed.repeat_interleave(E // count, dim=1)] = -1.0
        idx = torch.sort(masked, dim=-1, descending=True, stable=True).indices[:, :top]
        ids.copy_(idx.to(ids.dtype))
        gates.copy_((torch.gather(score, 1, idx) * weight_scale).to(gates.dtype))

    def moe_route_plan(self, logits, top, ids, gates, offsets, perm, pos, experts=None, scoring="chosen", groups=None,
                       weight_scale=1.0):
        """moe_route, then moe_plan."""
        self.moe_route(logits, top, ids, gates, experts=experts, scoring=scoring, groups=groups, weight_scale=weight_scale)
        self.moe_plan(ids, experts if experts is not None else logits.shape[1], offsets, perm, pos)

    def moe_plan(self, ids, num_experts, offsets, perm, pos):
        """The pairs (token, choice), numbered token * top + choice, listed by expert in ascending pair number:
        offsets[e] .. offsets[e + 1] are expert e's places in ``perm``; pos[pair] is the pair's place."""
        flat = ids.reshape(-1).long()
        order = torch.sort(flat, stable=True).indices
        perm.copy_(order.to(perm.dtype))
        pos[order] = torch.arange(flat.numel(), dtype=pos.dtype)
        counts = torch.bincount(flat, minlength=num_experts)
        offsets[0] = 0
        offsets[1:] = torch.cumsum(counts, 0).to(offsets.dtype)

    def moe_linear(self, x, w, offsets, perm, top, out, epilogue="none"):
        """Row i of ``out`` belongs to the expert e with offsets[e] <= i < offsets[e + 1] and is
        x[perm[i] // top] @ w[e]^T (perm None: x[i]); epilogue "silu_gate" as in ``linear``."""
        for e in range(w.shape[0]):
            a, b = int(offsets[e]), int(offsets[e + 1])
            if a == b:
                continue
            rows = x[(perm[a:b].long() // top)] if perm is not None else x[a:b]
            y = rows.to(self.cd) @ w[e].to(self.cd).t()
            if epilogue == "silu_gate":
                half = y.shape[1] // 2
                y = y[:, :half] * torch.sigmoid(y[:, :half]) * y[:, half:]
            elif epilogue != "none":
                raise ValueError(epilogue)
            out[a:b] = y.to(out.dtype)

    def moe_gather_scaled(self, x, perm, top, gates, out, tile_expert=None):
        """out[place] = gates[perm[place]] * x[perm[place] // top], zeros where perm[place] < 0."""
        p = perm.long()
        live = p >= 0
        rows = torch.zeros(out.shape, dtype=self.cd)
        rows[live] = x[p[live] // top].to(self.cd) * gates.reshape(-1)[p[live]].to(self.cd)[:, None]
        out.copy_(rows.to(out.dtype))

    def moe_combine(self, y, pos, gates, out, shared=None, shared_logit=None):
        """out[n] = sum_j gates[n, j] * y[pos[n * top + j]], j ascending (gates None: weights of 1); + shared[n] (times
        sigmoid(shared_logit[n]))."""
        if gates is None:
            gates = torch.ones(out.shape[0], pos.numel() // max(out.shape[0], 1), dtype=self.cd)
        n, top = gates.shape
        acc = torch.zeros(n, y.shape[1], dtype=self.cd)
        for j in range(top):
            acc = acc + gates[:, j].to(self.cd)[:, None] * y[pos.view(n, top)[:, j].long()].to(self.cd)
        if shared is not None:
            g = torch.sigmoid(shared_logit.to(self.cd))[:, None] if shared_logit is not None else 1.0
            acc = acc + g * shared.to(self.cd)
        out.copy_(acc.to(out.dtype))

    # ------------------------------------------------------------------ decoders with latent attention
    def _group_norm(self, v, weight, groups, eps):
        n, W = v.shape
        p = v.to(self.cd).view(n, groups, W // groups)
        p = p * torch.rsqrt(p.pow(2).mean(-1, keepdim=True) + eps)
        return p.reshape(n, W) * weight.to(self.cd)

    def group_rmsnorm(self, x, weight, groups, eps, out, delta=None, mult=1.0, rows=None, keep=None):
        """x += mult * delta (in place unless ``rows``); keep = the updated rows; out = the norm in groups of them."""
        if rows is None:
            if delta is not None:
                x.add_(mult * delta.to(torch.float32))
            src = x
        else:
            src = x[rows.long()]
            if delta is not None:
                src = src + mult * delta[rows.long()].to(torch.float32)
        if keep is not None:
            keep.copy_(src)
        out.copy_(self._group_norm(src, weight, groups, eps).to(out.dtype))

    def depth_average(self, x, delta, mult, hist, depth, coeff, out=None, next_weight=None, groups=1, eps=0.0):
        """hist[:, depth] = x + mult * delta; x = sum_(j <= depth) coeff[j] * hist[:, j]; out = the next norm of x."""
        v = x if delta is None else x + mult * delta.to(torch.float32)
        hist[:, depth] = v
        x.copy_((hist[:, :depth + 1].to(self.cd) * coeff.to(self.cd)[None, :, None]).sum(1).to(torch.float32))
        if out is not None:
            out.copy_(self._group_norm(x, next_weight, groups, eps).to(out.dtype))

    def causal_conv(self, h, weight, state, state_slots, cu_q, seq_lens, req_index, out):
        """out_t = h_t + sum_j weight[:, j] * h_(t - taps + 1 + j) per request; state[slot] holds the taps - 1 inputs before
        the portion (oldest first) and takes the portion's last inputs."""
        taps = weight.shape[1]
        K = taps - 1
        w = weight.to(self.cd)
        for r in range(cu_q.numel() - 1):
            a, b = int(cu_q[r]), int(cu_q[r + 1])
            if int(seq_lens[r]) <= 0 or a == b:
                out[a:b] = h[a:b]
                continue
            slot = int(state_slots[r])
            seq = torch.cat((state[slot, :K].to(self.cd), h[a:b].to(self.cd)), dim=0)        # inputs -K .. len - 1
            y = h[a:b].to(self.cd).clone()
            for j in range(taps):
                y = y + w[:, j] * seq[j:j + (b - a)]
            out[a:b] = y.to(out.dtype)
            if K:
                state[slot, :K] = seq[seq.shape[0] - K:].to(state.dtype)

    def latent_prepare(self, proj, heads, dim, rot, rank, down_col, norm_weight, eps, table, dims, q_plain, q_rot, latent_pages,
                       rot_pages, slot_mapping, offsets, tile_head=None, tile=0, q=None, interleaved=False):
        """Queries head-major, rotated parts turned, the normalised latent and the turned shared key part into the pages."""
        n = proj.shape[0]
        seg = q_plain.shape[1]
        p = proj.to(self.cd)
        q = (p[:, :heads * (dim + rot)] if q is None else q.to(self.cd)).reshape(n, heads, dim + rot)
        q_plain[:, :n] = q[..., :dim].transpose(0, 1).to(q_plain.dtype)
        offsets.copy_(torch.arange(heads + 1, dtype=offsets.dtype) * seg)
        if tile_head is not None:
            tile_head.copy_((torch.arange(tile_head.numel()) // (seg // tile)).to(tile_head.dtype))

        def turn(v):                     # v [n, ..., rot]
            if table is None:
                return v
            cs = table.to(self.cd).view(n, dims // 2, 2)
            while cs.dim() < v.dim() + 1:
                cs = cs.unsqueeze(1)
            c, s = cs[..., 0], cs[..., 1]
            if interleaved:
                a, b = v[..., 0:dims:2], v[..., 1:dims:2]
                w = v.clone()
                w[..., 0:dims:2], w[..., 1:dims:2] = a * c - b * s, b * c + a * s
                return w
            a, b = v[..., :dims // 2], v[..., dims // 2:dims]
            return torch.cat((a * c - b * s, b * c + a * s, v[..., dims:]), dim=-1)

        if rot:
            q_rot.copy_(turn(q[..., dim:]).to(q_rot.dtype))
        if slot_mapping is None:
            return
        lat = p[:, down_col:down_col + rank]
        lat = lat * torch.rsqrt(lat.pow(2).mean(-1, keepdim=True) + eps) * norm_weight.to(self.cd)
        slots = slot_mapping[:n].long()
        live = slots >= 0
        latent_pages.view(-1, rank)[slots[live]] = lat[live].to(latent_pages.dtype)
        if rot:
            kr = turn(p[:, down_col + rank:down_col + rank + rot])
            rot_pages.view(-1, rot)[slots[live]] = kr[live].to(rot_pages.dtype)

    def latent_attention(self, q_lat, q_rot, latent_pages, rot_pages, block_tables, cu_q, seq_lens, req_index, sink, out, scale,
                         window, tokens, max_q_len=None, max_seq_len=None, exact=False, weight_terms=1):
        """Every head of a token attends over its request's cached latents (and the shared rotated key part)."""
        heads, seg, rank = q_lat.shape
        ps = latent_pages.shape[2]
        lat = latent_pages.view(-1, rank)
        rk = rot_pages.view(-1, rot_pages.shape[3]) if rot_pages is not None else None
        for r in range(cu_q.numel() - 1):
            a, b, L = int(cu_q[r]), int(cu_q[r + 1]), int(seq_lens[r])
            for t in range(a, b):
                if L <= 0:
                    out[:, t] = 0
                    continue
                p = L - (b - a) + (t - a)
                first = max(0, p - window + 1) if window else 0
                js = torch.arange(first, p + 1)
                slots = block_tables[r][(js // ps).long()].long() * ps + js % ps
                c = lat[slots].to(self.cd)                                             # [keys, rank]
                s = q_lat[:, t].to(self.cd) @ c.t()                                    # [heads, keys]
                if rk is not None:
                    s = s + q_rot[t].to(self.cd) @ rk[slots].to(self.cd).t()
                s = s * scale
                m = s.max(dim=1).values
                if sink is not None:
                    m = torch.maximum(m, sink.to(self.cd))
                e = torch.exp(s - m[:, None])
                den = e.sum(1)
                if sink is not None:
                    den = den + torch.exp(sink.to(self.cd) - m)
                out[:, t] = ((e / den[:, None]) @ c).to(out.dtype)

    def gate_heads(self, y, gate, out, tokens, per_head=False):
        """out[t, h * vdim + v] = y[h, t, v] * sigmoid(gate[t, h * vdim + v]) (``per_head``: gate[t, h])."""
        heads, seg, vdim = y.shape
        v = y[:, :tokens].to(self.cd).transpose(0, 1).reshape(tokens, heads * vdim)
        if gate is not None:
            g = torch.sigmoid(gate.to(self.cd))
            v = v * (g.repeat_interleave(vdim, dim=1) if per_head else g)
        out.copy_(v.to(out.dtype))

    # ------------------------------------------------------------------ sampling
    def sample(self, logits, temperature, uniform, out):
        """Row m: temperature[m] == 0 -> the index of the largest logit (the lowest such
        index); else the smallest index i with cumsum(softmax(logits/temperature))[i] >
        uniform[m] (the last index with non-zero probability if rounding leaves none)."""
        for m in range(logits.shape[0]):
            t = 0.0 if temperature is None else float(temperature[m])
            row = logits[m].double()
            if t == 0.0:
                out[m] = int(torch.argmax(row))
            else:
                p = torch.softmax(row / t, dim=-1)
                c = torch.cumsum(p, 0)
                idx = int(torch.searchsorted(c, torch.tensor(float(uniform[m]), dtype=torch.float64), right=True))
                out[m] = min(idx, row.numel() - 1)
