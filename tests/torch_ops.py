"""A kernel set written with plain torch, for tests that run the engine's step function,
cache and parts without a GPU.  It is a test double: the product path has no such set and
refuses to run without its CUDA extension.  It follows the same calling conventions and
cache layout as the CUDA kernel set, and shares nothing with ``plain_gpt``.
"""

from __future__ import annotations

import math

import torch


class TorchOps:
    name = "torch-test-double"

    def embed(self, token_ids, positions, tok_emb, pos_table, scale=1.0):
        x = tok_emb.float()[token_ids.long()] * scale
        if pos_table is not None:
            x = x + pos_table.float()[positions.long()]
        return x

    def layernorm(self, x32, gain, shift, eps, out_dtype):
        mean = x32.mean(-1, keepdim=True)
        var = ((x32 - mean) ** 2).mean(-1, keepdim=True)
        y = (x32 - mean) * torch.rsqrt(var + eps) * gain
        if shift is not None:
            y = y + shift
        return y.to(out_dtype)

    def linear(self, x, weight, bias, activation, out_dtype, out=None):
        if out is not None:
            out.copy_(self.linear(x, weight, bias, activation, out_dtype))
            return out
        y = x.float() @ weight.float().T
        if bias is not None:
            y = y + bias
        if activation == "gelu_tanh":
            y = 0.5 * y * (1 + torch.tanh(math.sqrt(2 / math.pi) * (y + 0.044715 * y ** 3)))
        elif activation == "relu_sq":
            y = torch.relu(y) ** 2
        elif activation != "none":
            raise ValueError(activation)
        return y.to(out_dtype)

    def linear_residual(self, x, weight, bias, residual32):
        y = x.float() @ weight.float().T
        if bias is not None:
            y = y + bias
        residual32 += y

    def kv_store(self, qkv, n_head, n_kv_head, head_dim, cache, slot_mapping):
        N = qkv.shape[0]
        k = qkv[:, n_head * head_dim: (n_head + n_kv_head) * head_dim].reshape(N, n_kv_head, head_dim)
        v = qkv[:, (n_head + n_kv_head) * head_dim:].reshape(N, n_kv_head, head_dim)
        slots = slot_mapping.long()
        page, off = slots // cache.page_tokens, slots % cache.page_tokens
        cache.k_pages[page, :, off] = k.to(cache.k_pages.dtype)
        cache.v_pages[page, :, off] = v.to(cache.v_pages.dtype)

    def paged_attention(self, qkv, n_head, n_kv_head, head_dim, scale, cache, ctx):
        N = qkv.shape[0]
        q = qkv[:, : n_head * head_dim].reshape(N, n_head, head_dim).float()
        out = torch.zeros(N, n_head, head_dim)
        table = ctx.block_tables[cache.group].long()
        pt = cache.page_tokens
        for i in range(N):
            r = int(ctx.token_request[i])
            p = int(ctx.positions[i])
            lo = 0 if cache.window is None else max(0, p - cache.window + 1)
            keys = torch.arange(lo, p + 1)
            pages = table[r, keys // pt]
            assert (pages >= 0).all(), "attention reads a page that is not there"
            k = cache.k_pages[pages, :, keys % pt].float()      # [keys, Hkv, D]
            v = k[..., :v_dim] if getattr(cache, "values_in_keys", False) else cache.v_pages[pages, :, keys % pt].float()
            for h in range(n_head):
                kh = h // (n_head // n_kv_head)
                s = (k[:, kh] @ q[i, h]) * scale
                out[i, h] = torch.softmax(s, dim=0) @ v[:, kh]
        return out.reshape(N, n_head * head_dim).to(qkv.dtype)

    def gather_rows(self, x32, rows):
        return x32[rows.long()]

    def logits(self, y, tok_emb, scale=1.0):
        return (y.float() @ tok_emb.float().T) * scale

    # ---- what the second architecture adds (same conventions as the CUDA kernel set) ---------------
    def head_prepare(self, proj, n_head, n_kv_head, head_dim, v_dim, q_off, k_off, v_off, unit_norm, eps,
                     cache, slots, positions, v_other=None, blend=None, q_gain=None, k_gain=None):
        n = proj.shape[0]
        live = positions >= 0

        def unit(x, gain=None):
            x = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) if unit_norm else x
            return x if gain is None else x * gain

        q = proj[:, q_off: q_off + n_head * head_dim].float().reshape(n, n_head, head_dim)
        v = proj[:, v_off: v_off + n_kv_head * v_dim].float()
        k = unit(proj[:, k_off: k_off + n_kv_head * head_dim].float().reshape(n, n_kv_head, head_dim), k_gain)
        if v_other is not None:
            v = (1.0 - blend[0]) * v + blend[0] * v_other.float()
        v = v.reshape(n, n_kv_head, v_dim)
        proj[live, q_off: q_off + n_head * head_dim] = unit(q, q_gain)[live].reshape(int(live.sum()), -1).to(proj.dtype)
        if cache is not None and cache.writes:
            keep = live & (slots >= 0)
            page, off = slots[keep].long() // cache.page_tokens, slots[keep].long() % cache.page_tokens
            cache.k_pages[page, :, off] = k[keep].to(cache.k_pages.dtype)
            cache.v_pages[page, :, off] = v[keep].to(cache.v_pages.dtype)

    def paged_attention_general(self, q, n_head, n_kv_head, head_dim, v_dim, scale, cache, ctx, gate=None,
                                slopes=None, block=None, softcap=None, sinks=None):
        n = q.shape[0]
        qh = q[:, : n_head * head_dim].reshape(n, n_head, head_dim).float()
        out = torch.zeros(n, n_head, v_dim)
        table = ctx.block_tables[cache.group].long()
        pt = cache.page_tokens
        for i in range(n):
            r, p = int(ctx.token_request[i]), int(ctx.positions[i])
            if p < 0:
                continue
            lo = 0 if cache.window is None else max(0, p - cache.window + 1)
            if block:
                lo = max(lo, p // block * block)
            keys = torch.arange(lo, p + 1)
            pages = table[r, keys // pt]
            assert (pages >= 0).all(), "attention reads a page that is not there"
            k = cache.k_pages[pages, :, keys % pt].float()
            v = k[..., :v_dim] if getattr(cache, "values_in_keys", False) else cache.v_pages[pages, :, keys % pt].float()
            for h in range(n_head):
                kh = h // (n_head // n_kv_head)
                scores = (k[:, kh] @ qh[i, h]) * scale
                if slopes is not None:
                    scores = scores - slopes[h] * (p - keys).float()
                if softcap:
                    scores = softcap * torch.tanh(scores / softcap)
                if sinks is not None:
                    # one more term in the denominator, with no value: a key whose value is zero
                    weights = torch.softmax(torch.cat([scores, sinks[h].float().view(1)]), dim=0)[:-1]
                else:
                    weights = torch.softmax(scores, dim=0)
                out[i, h] = weights @ v[:, kh]
        out = out.reshape(n, n_head * v_dim)
        if gate is not None:
            out = out * torch.sigmoid(gate.float())
        return out.to(q.dtype)

    def moe_route(self, y, router_weight, gate_weight, positions, top):
        z = y.float() @ router_weight.float().T
        vals, ids = torch.topk(z, top, dim=-1)
        weights = torch.softmax(vals, dim=-1)
        ids = ids.to(torch.int32)
        ids[positions < 0] = -1
        gate = torch.sigmoid(y.float() @ gate_weight.float()) if gate_weight is not None else None
        return ids, weights, gate

    @staticmethod
    def _gated(a, u, activation, limit):
        if activation == "silu":
            return a * torch.sigmoid(a) * u
        if activation == "gelu_tanh":
            return 0.5 * a * (1 + torch.tanh(math.sqrt(2 / math.pi) * (a + 0.044715 * a ** 3))) * u
        if activation == "clamped_swish":
            a, u = a.clamp(max=limit), u.clamp(-limit, limit)
            return a * torch.sigmoid(1.702 * a) * (u + 1.0)
        raise ValueError(activation)

    def moe_experts_residual(self, y, ids, weights, w_in, w_out, residual32, activation="silu", limit=0.0):
        inner = w_in.shape[1] // 2
        for t in range(y.shape[0]):
            for k in range(ids.shape[1]):
                e = int(ids[t, k])
                if e < 0:
                    continue
                a = w_in[e].float() @ y[t].float()
                hidden = self._gated(a[:inner], a[inner:], activation, limit).to(y.dtype).float()
                residual32[t] += weights[t, k] * (w_out[e].float() @ hidden)

    def moe_route_scored(self, y, router_weight, gate_weight, positions, top, scoring, correction, groups, scale):
        z = y.float() @ router_weight.float().T
        n, experts = z.shape
        s = torch.sigmoid(z) if scoring == "sigmoid" else z
        choice = s if correction is None else s + correction
        if groups is not None:
            count, keep = groups
            per = experts // count
            grouped = choice.view(n, count, per)
            score = grouped.topk(min(2, per), dim=-1).values.sum(-1)
            allowed = torch.zeros(n, count, dtype=torch.bool).scatter_(1, score.topk(keep, dim=-1).indices, True)
            choice = grouped.masked_fill(~allowed[:, :, None], -math.inf).reshape(n, experts)
        ids = choice.topk(top, dim=-1).indices
        picked = s.gather(1, ids)
        weights = (picked if scoring == "sigmoid" else torch.softmax(picked, dim=-1)) * scale
        ids = ids.to(torch.int32)
        ids[positions < 0] = -1
        gate = torch.sigmoid(y.float() @ gate_weight.float()) if gate_weight is not None else None
        return ids, weights, gate

    def scale_(self, x32, scale):
        x32 *= scale
        return x32

    def clone(self, x):
        return x.clone()

    def embed_pairs(self, ctx, tok_emb, pair_emb, pos_table, buckets, mul_prev, mul_cur, state, source=None,
                    previous=None):
        ids = ctx.token_ids.long()
        x = tok_emb.float()[ids] + pos_table.float()[ctx.positions.long().clamp(min=0)]
        for r in range(ctx.num_requests):
            start, count = int(ctx.req_q_start[r]), int(ctx.req_q_len[r])
            slot = int(ctx.req_state_slot[r])
            if count == 0:
                continue
            before = None if int(ctx.req_ctx_before[r]) == 0 else int(state[slot, 0])
            for i in range(start, start + count):
                row = buckets if before is None else (before * mul_prev + int(ids[i]) * mul_cur) % buckets
                x[i] += pair_emb[row].float()
                before = int(ids[i])
            state[slot, 0] = before
        return x

    def rmsnorm(self, x32, weight, eps, offset, out_dtype):
        return (x32 / torch.sqrt((x32 * x32).mean(-1, keepdim=True) + eps) * (offset + weight)).to(out_dtype)

    def concat_cast(self, a32, b32, out_dtype):
        return torch.cat([a32, b32], dim=-1).to(out_dtype)

    def matrix_memory_scan(self, ctx, mode, proj, q_off, k_off, v_off, n_head, head_dim, v_dim, gates, constant, state,
                           state_offset=0, qk_group=1, head_consts=None):
        if mode in ("retention", "wkv"):
            return self._fixed_or_bonus_scan(ctx, mode, proj, q_off, k_off, v_off, n_head, head_dim, v_dim, gates, state,
                                             state_offset, head_consts), None
        n = proj.shape[0]
        if mode == "ssd":
            return self._state_space_scan(ctx, proj, q_off, k_off, v_off, n_head, head_dim, v_dim, gates, state,
                                          state_offset, qk_group, head_consts), None
        q = proj[:, q_off: q_off + n_head * head_dim].float().reshape(n, n_head, head_dim) * head_dim ** -0.5
        k = proj[:, k_off: k_off + n_head * head_dim].float().reshape(n, n_head, head_dim)
        v = proj[:, v_off: v_off + n_head * v_dim].float().reshape(n, n_head, v_dim)
        out = torch.zeros(n, n_head, v_dim)
        aux = torch.zeros(n, n_head, 2) if mode == "mlstm" else None
        cols = v_dim + (1 if mode == "mlstm" else 0)
        for r in range(ctx.num_requests):
            start, count = int(ctx.req_q_start[r]), int(ctx.req_q_len[r])
            if count == 0:
                continue
            slot = int(ctx.req_state_slot[r])
            flat = state[slot]
            S = flat[: n_head * cols * head_dim].view(n_head, cols, head_dim).clone()
            m = flat[n_head * cols * head_dim:].clone() if mode == "mlstm" else None
            if int(ctx.req_ctx_before[r]) == 0:
                S.zero_()
                if m is not None:
                    m.zero_()
            for i in range(start, start + count):
                if mode == "gla":
                    decay = torch.exp(torch.nn.functional.logsigmoid(gates[i].float()) / constant).view(n_head, head_dim)
                    S = decay[:, None, :] * S + v[i][:, :, None] * k[i][:, None, :]
                    out[i] = torch.einsum("hvd,hd->hv", S, q[i])
                else:
                    cap = constant
                    gi = cap * torch.tanh(gates[i, :n_head].float() / cap)
                    gf = torch.nn.functional.logsigmoid(cap * torch.tanh(gates[i, n_head:].float() / cap))
                    m_new = torch.maximum(gf + m, gi)
                    keep, take = torch.exp(gf + m - m_new), torch.exp(gi - m_new)
                    v1 = torch.cat([v[i], torch.ones(n_head, 1)], dim=1)
                    S = keep[:, None, None] * S + take[:, None, None] * v1[:, :, None] * k[i][:, None, :]
                    m = m_new
                    full = torch.einsum("hvd,hd->hv", S, q[i])
                    out[i] = full[:, :v_dim]
                    aux[i, :, 0], aux[i, :, 1] = full[:, v_dim], m
            flat[: n_head * cols * head_dim] = S.reshape(-1)
            if m is not None:
                flat[n_head * cols * head_dim:] = m
        return out.reshape(n, n_head * v_dim), aux

    def _fixed_or_bonus_scan(self, ctx, mode, proj, q_off, k_off, v_off, n_head, head_dim, v_dim, gates, state, state_offset,
                             head_consts):
        """Retention (a fixed decay per head, keys scaled) and the wkv form (the read before the update, with a bonus
        on the token itself); ``proj`` may be planes ``[planes, tokens, columns]`` with offsets that name a plane."""
        n, ld = proj.shape[-2], proj.shape[-1]
        flat_rows = proj.reshape(-1, ld)

        def take(off, size):
            plane, col = divmod(int(off), n * ld) if proj.dim() == 3 else (0, int(off))
            return flat_rows[plane * n: (plane + 1) * n, col: col + size].float()
        q = take(q_off, n_head * head_dim).reshape(n, n_head, head_dim)
        k = take(k_off, n_head * head_dim).reshape(n, n_head, head_dim)
        v = take(v_off, n_head * v_dim).reshape(n, n_head, v_dim)
        if mode == "retention":
            k = k * head_dim ** -0.5
        out = torch.zeros(n, n_head, v_dim)
        size = n_head * v_dim * head_dim
        for r in range(ctx.num_requests):
            start, count = int(ctx.req_q_start[r]), int(ctx.req_q_len[r])
            if count == 0:
                continue
            flat = state[int(ctx.req_state_slot[r])]
            S = flat[state_offset: state_offset + size].view(n_head, v_dim, head_dim).clone()
            if int(ctx.req_ctx_before[r]) == 0:
                S.zero_()
            for i in range(start, start + count):
                kv = v[i][:, :, None] * k[i][:, None, :]
                if mode == "retention":
                    S = head_consts.float()[:, None, None] * S + kv
                    out[i] = torch.einsum("hvd,hd->hv", S, q[i])
                else:
                    bonus = head_consts.float().view(n_head, 1, head_dim)
                    out[i] = torch.einsum("hvd,hd->hv", S + bonus * kv, q[i])
                    decay = torch.exp(-torch.exp(gates[i].float())).view(n_head, 1, head_dim)
                    S = decay * S + kv
            flat[state_offset: state_offset + size] = S.reshape(-1)
        return out.reshape(n, n_head * v_dim)

    def _state_space_scan(self, ctx, proj, q_off, k_off, v_off, n_head, n_state, v_dim, steps, state, state_offset,
                          qk_group, head_consts):
        n, groups = proj.shape[0], n_head // qk_group
        c = proj[:, q_off: q_off + groups * n_state].float().reshape(n, groups, n_state).repeat_interleave(qk_group, 1)
        b = proj[:, k_off: k_off + groups * n_state].float().reshape(n, groups, n_state).repeat_interleave(qk_group, 1)
        x = proj[:, v_off: v_off + n_head * v_dim].float().reshape(n, n_head, v_dim)
        a, d = head_consts[:n_head], head_consts[n_head:]
        out = torch.zeros(n, n_head, v_dim)
        size = n_head * v_dim * n_state
        for r in range(ctx.num_requests):
            start, count = int(ctx.req_q_start[r]), int(ctx.req_q_len[r])
            if count == 0:
                continue
            flat = state[int(ctx.req_state_slot[r])]
            S = flat[state_offset: state_offset + size].view(n_head, v_dim, n_state).clone()
            if int(ctx.req_ctx_before[r]) == 0:
                S.zero_()
            for i in range(start, start + count):
                dt = torch.nn.functional.softplus(steps[i].float(), threshold=1e9)
                S = torch.exp(-torch.exp(a) * dt)[:, None, None] * S + dt[:, None, None] * x[i][:, :, None] * b[i][:, None, :]
                out[i] = torch.einsum("hvn,hn->hv", S, c[i]) + d[:, None] * x[i]
            flat[state_offset: state_offset + size] = S.reshape(-1)
        return out.reshape(n, n_head * v_dim)

    def head_norm_gate(self, out32, aux, gate, gain, n_head, v_dim, eps, per_head_gain, gate_activation, out_dtype,
                       positions=None):
        n = out32.shape[0]
        o = out32.view(n, n_head, v_dim)
        if aux is not None:
            o = o / (torch.maximum(aux[:, :, 0].abs(), torch.exp(-aux[:, :, 1])) + 1e-6)[:, :, None]
        o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps)
        if gain is not None:
            o = o * (gain.view(n_head, v_dim) if per_head_gain else gain)
        g = gate.float().reshape(n, n_head, v_dim)
        g = g * torch.sigmoid(g) if gate_activation == "silu" else torch.sigmoid(g)
        return (o * g).reshape(n, n_head * v_dim).to(out_dtype)

    def glu(self, gate_up, row_scale=None, activation="silu", limit=0.0):
        inner = gate_up.shape[1] // 2
        a, u = gate_up[:, :inner].float(), gate_up[:, inner:].float()
        out = self._gated(a, u, activation, limit)
        if row_scale is not None:
            out = out * row_scale[:, None]
        return out.to(gate_up.dtype)

    def argmax(self, logits, vocab_limit=None, out=None):
        v = logits if vocab_limit is None else logits[:, :vocab_limit]
        ids = v.argmax(-1).to(torch.int32)
        if out is None:
            return ids
        out.copy_(ids)
        return out

    # ---- what the fourth architecture adds -----------------------------------------------------------
    def streams_spread(self, x32, streams):
        return x32[None].repeat(int(streams), 1, 1)

    def streams_read(self, streams32, weights, want_zeros=False):
        u = torch.einsum("s,stc->tc", weights.float(), streams32)
        return (u, torch.zeros_like(u)) if want_zeros else u

    def streams_sum(self, streams32):
        return streams32.sum(0)

    def streams_write(self, streams32, mix, weights, y32, next_read=None):
        new = torch.einsum("sr,stc->rtc", mix.float(), streams32) + weights.float()[:, None, None] * y32[None]
        streams32.copy_(new)
        return self.streams_read(streams32, next_read, want_zeros=True) if next_read is not None else None

    @staticmethod
    def _turn(x, positions, rot_dims, freq):
        """x: [tokens, heads, features]; the first rot_dims features of each head by position * freq."""
        if not rot_dims:
            return x
        half = rot_dims // 2
        angle = positions.clamp(min=0).float()[:, None] * freq.float()[None, :]
        cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
        u, v = x[..., :half], x[..., half:rot_dims]
        return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., rot_dims:]], dim=-1)

    def qk_norm_rotary(self, proj, n_head, n_kv_head, head_dim, v_dim, q_off, k_off, v_off, norm, eps, rot_dims, freq,
                       cache, slots, positions, q_gain=None, k_gain=None, v_unit_norm=False, v_freq=None):
        n = proj.shape[0]
        live = positions >= 0

        def whole(x, gain):
            return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * gain if norm else x

        q = whole(proj[:, q_off: q_off + n_head * head_dim].float(), q_gain).reshape(n, n_head, head_dim)
        k = whole(proj[:, k_off: k_off + n_kv_head * head_dim].float(), k_gain).reshape(n, n_kv_head, head_dim)
        q, k = self._turn(q, positions, rot_dims, freq), self._turn(k, positions, rot_dims, freq)
        v = proj[:, v_off: v_off + n_kv_head * v_dim].float().reshape(n, n_kv_head, v_dim)
        if v_unit_norm:
            v = v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)
        if v_freq is not None:
            v = self._turn(v, positions, v_dim, v_freq)
        proj[live, q_off: q_off + n_head * head_dim] = q[live].reshape(int(live.sum()), -1).to(proj.dtype)
        if cache is not None and cache.writes:
            keep = live & (slots >= 0)
            page, off = slots[keep].long() // cache.page_tokens, slots[keep].long() % cache.page_tokens
            cache.k_pages[page, :, off] = k[keep].to(cache.k_pages.dtype)
            cache.v_pages[page, :, off] = v[keep].to(cache.v_pages.dtype)

    def latent_prepare(self, proj, n_head, q_off, q_dim, rot_dim, low_off, rank, gain, eps, freq, cache, slots, positions):
        n = proj.shape[0]
        q_in = proj[:, q_off: q_off + n_head * (q_dim + rot_dim)].float().reshape(n, n_head, q_dim + rot_dim)
        q = torch.zeros(n, n_head, rank + rot_dim)
        q[..., rank:] = self._turn(q_in[..., q_dim:], positions, rot_dim, freq)
        if cache is not None and cache.writes:
            c = proj[:, low_off: low_off + rank].float()
            c = c / torch.sqrt((c * c).mean(-1, keepdim=True) + eps) * gain
            shared = self._turn(proj[:, None, low_off + rank: low_off + rank + rot_dim].float(), positions, rot_dim, freq)[:, 0]
            keep = (positions >= 0) & (slots >= 0)
            page, off = slots[keep].long() // cache.page_tokens, slots[keep].long() % cache.page_tokens
            cache.k_pages[page, 0, off] = torch.cat([c, shared], dim=-1)[keep].to(cache.k_pages.dtype)
        return q.reshape(n, -1).to(proj.dtype)

    def head_linear(self, x, x_off, x_head, weight, rows_are_inputs, n_head, n_in, n_out, gate=None, out=None, out_off=0,
                    out_head=None):
        n = x.shape[0]
        cols = x_off + x_head * torch.arange(n_head)[:, None] + torch.arange(n_in)[None, :]
        xs = x[:, cols.reshape(-1)].float().reshape(n, n_head, n_in)
        w = weight.float().reshape(n_head, n_in, n_out) if rows_are_inputs else weight.float().reshape(n_head, n_out, n_in).transpose(1, 2)
        y = torch.einsum("nhi,hio->nho", xs, w)
        if gate is not None:
            y = y * torch.sigmoid(gate.float().reshape(n, n_head, n_out))
        if out is None:
            return y.reshape(n, n_head * n_out).to(x.dtype)
        out_head = n_out if out_head is None else out_head
        where = out_off + out_head * torch.arange(n_head)[:, None] + torch.arange(n_out)[None, :]
        out[:, where.reshape(-1)] = y.reshape(n, -1).to(out.dtype)
        return out

    def causal_conv_silu(self, ctx, x, x_off, channels, taps, bias, state):
        n, width = x.shape[0], taps.shape[1]
        out = torch.zeros(n, channels)
        for r in range(ctx.num_requests):
            start, count = int(ctx.req_q_start[r]), int(ctx.req_q_len[r])
            if count == 0:
                continue
            before = state[int(ctx.req_state_slot[r]), : (width - 1) * channels].view(width - 1, channels).clone()
            if int(ctx.req_ctx_before[r]) == 0:
                before.zero_()
            elif int(ctx.req_ctx_before[r]) < width - 1:       # rows before the sequence's start are zeros
                before[: width - 1 - int(ctx.req_ctx_before[r])] = 0
            rows = torch.cat([before, x[start: start + count, x_off: x_off + channels].float()], dim=0)
            y = bias.float()[None, :].repeat(count, 1) if bias is not None else torch.zeros(count, channels)
            for j in range(width):
                y = y + rows[j: j + count] * taps[:, j].float()[None, :]
            out[start: start + count] = y * torch.sigmoid(y)
        return out.to(x.dtype)

    def conv_state_update(self, ctx, x, x_off, channels, n_taps, state):
        keep = n_taps - 1
        if keep <= 0:
            return
        for r in range(ctx.num_requests):
            start, count = int(ctx.req_q_start[r]), int(ctx.req_q_len[r])
            if count == 0:
                continue
            slot = int(ctx.req_state_slot[r])
            before = state[slot, : keep * channels].view(keep, channels).clone()
            if int(ctx.req_ctx_before[r]) == 0:
                before.zero_()
            rows = torch.cat([before, x[start: start + count, x_off: x_off + channels].float()], dim=0)
            state[slot, : keep * channels] = rows[-keep:].reshape(-1)

    def gated_group_norm(self, out32, gate, gain, parts, eps, out_dtype, positions=None):
        n, width = out32.shape
        g = gate.float()
        y = (out32 * g * torch.sigmoid(g)).view(n, parts, width // parts)
        y = y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps)
        return (y.reshape(n, width) * gain).to(out_dtype)

    def rotate_heads(self, heads, n_head, v_dim, freq, positions, sign=-1.0):
        n = heads.shape[0]
        turned = self._turn(heads.float().reshape(n, n_head, v_dim), positions, v_dim, sign * freq.float())
        live = positions >= 0
        heads[live] = turned.reshape(n, -1)[live].to(heads.dtype)
        return heads

    def gated_recurrence(self, ctx, pre, z_off, u_off, g_off, width, state, state_offset, out_dtype):
        n = pre.shape[0]
        z = torch.sigmoid(pre[:, z_off: z_off + width])
        u = pre[:, u_off: u_off + width]
        cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
        g = pre[:, g_off: g_off + width]
        out = torch.zeros(n, width)
        for r in range(ctx.num_requests):
            start, count = int(ctx.req_q_start[r]), int(ctx.req_q_len[r])
            if count == 0:
                continue
            slot = int(ctx.req_state_slot[r])
            s = state[slot, state_offset: state_offset + width].clone()
            if int(ctx.req_ctx_before[r]) == 0:
                s.zero_()
            for i in range(start, start + count):
                s = (1 - z[i]) * s + z[i] * cand[i]
                out[i] = s * g[i] * torch.sigmoid(g[i])
            state[slot, state_offset: state_offset + width] = s
        return out.to(out_dtype)

    def token_shift_mix(self, ctx, x, mu, state):
        n, width = x.shape
        before = torch.zeros(n, width)
        for r in range(ctx.num_requests):
            start, count = int(ctx.req_q_start[r]), int(ctx.req_q_len[r])
            if count == 0:
                continue
            if int(ctx.req_ctx_before[r]) > 0:
                before[start] = state[int(ctx.req_state_slot[r]), :width]
            before[start + 1: start + count] = x[start: start + count - 1].float()
        cur = x.float()
        return (cur[None] + (before - cur)[None] * mu.float()[:, None, :]).to(x.dtype)

    def zeros32(self, rows, width, ctx=None, index=0):
        shared = getattr(ctx, "shared", None)
        key = ("zeros32", rows, width, index)
        if shared is not None and key in shared:
            assert not bool(shared[key].any()), "a buffer of zeros was handed back with something in it"
            return shared[key]
        out = torch.zeros(rows, width)
        if shared is not None:
            shared[key] = out
        return out

    def rmsnorm_add(self, residual32, y32, weight, eps, offset=0.0, other32=None, scale=1.0, other_scale=1.0, clear=False):
        y = scale * y32 if other32 is None else scale * y32 + other_scale * other32
        residual32 += y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps) * (offset + weight)
        if clear:
            y32.zero_()
            if other32 is not None:
                other32.zero_()
        return residual32

    def add_rows(self, x32, rows32, vector):
        x32 += vector if rows32 is None else rows32 + vector
        return x32

    def scaled_sum_(self, x32, a32, scale_a, b32, scale_b, clear=False):
        x32 += scale_a * a32 + scale_b * b32
        if clear:
            a32.zero_()
            b32.zero_()
        return x32

    def softcap_(self, x32, cap):
        x32.copy_(cap * torch.tanh(x32 / cap))
        return x32

    def cast(self, x32, out_dtype):
        return x32.to(out_dtype)

    def tanh_cast(self, x32, out_dtype):
        return torch.tanh(x32).to(out_dtype)

    def token_side_residual(self, ctx, residual32, gate_weight, proj_weight, norm_weight, table, offset, eps, act_dtype):
        gate = self.linear(self.cast(residual32, act_dtype), gate_weight, None, "none", torch.float32)
        gated = self.token_gate(ctx, gate, table, offset, act_dtype)
        y = self.linear(gated, proj_weight, None, "none", torch.float32)
        return self.rmsnorm_add(residual32, y, norm_weight, eps)

    def token_gate(self, ctx, gate32, table, offset, out_dtype):
        dim = gate32.shape[1]
        e = table.float()[ctx.token_ids.long().clamp(min=0), offset: offset + dim]
        z = gate32
        act = 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))
        return (act * e).to(out_dtype)
