"""A stand-in for the kernel library, in plain tensor code, for tests only.

It has the interface of `paged_llm_b200.kernels.ops.CudaOps` so that the engine's
host logic (runner, cache, scheduler, replay) can be exercised on a machine
without a GPU.  The product never imports it; on the product path a missing
extension is an error.
"""

from __future__ import annotations

import numpy as np
import torch

from paged_llm_b200.kernels.plan import plan_attention


class TorchOps:
    supports_graphs = False

    def __init__(self, device="cpu"):
        self.device = torch.device(device)
        self.compute_dtype = torch.float32
        self.calls: dict[str, int] = {}

    def _count(self, name):
        self.calls[name] = self.calls.get(name, 0) + 1

    def set_compute_dtype(self, dtype):
        self.compute_dtype = dtype

    # ---- elementwise / norms ---------------------------------------------------
    def embedding(self, table, ids, scale=1.0, copies=1):
        self._count("embedding")
        return (table[ids.long()].float() * scale).repeat(1, copies)

    def stream_norm(self, x, streams, branch, mix, out, w_in, norm_w, groups, eps, branch2=None, scales=None, biases=None):
        self._count("stream_norm")
        rows, width = x.shape[0], x.shape[1] // streams
        xs = x.view(rows, streams, width)
        if branch is not None:
            y = branch.float()
            if branch2 is not None:
                (sa, sb), (ba, bb) = scales, biases
                y = sa * (y + (ba.float() if ba is not None else 0.0)) + sb * (branch2.float() + (bb.float() if bb is not None else 0.0))
            if mix is None:
                xs += y[:, None, :]
            else:
                xs.copy_(torch.einsum("st,rsw->rtw", mix.float(), xs) + out.float()[None, :, None] * y[:, None, :])
        u = xs.sum(1) if w_in is None else torch.einsum("s,rsw->rw", w_in.float(), xs)
        p = u.view(rows, groups, width // groups)
        p = p * torch.rsqrt((p * p).mean(-1, keepdim=True) + eps)
        return (p.reshape(rows, width) * norm_w.float()).to(self.compute_dtype)

    def poly_norm(self, z, coef, eps):
        self._count("poly_norm")
        z = z.float()

        def unit(t):
            return t * torch.rsqrt((t * t).mean(-1, keepdim=True) + eps)

        a, b, c, e = coef.float()
        return (a * unit(z) + b * unit(z * z) + c * unit(z * z * z) + e).to(self.compute_dtype)

    def add_bias(self, y, bias):
        y += bias.to(y.dtype)
        return y

    def scaled_sum(self, a, scale_a, bias_a, b, scale_b, bias_b):
        self._count("scaled_sum")
        a, b = a.float(), b.float()
        if bias_a is not None:
            a = a + bias_a
        if bias_b is not None:
            b = b + bias_b
        return scale_a * a + scale_b * b

    def dyt(self, x, branch, post, pre, out_dtype=None):
        self._count("dyt")
        v = None
        if branch is not None:
            v = branch.float()
            if post is not None:
                v = torch.tanh(post[0] * v) * post[1] + post[2]
        if x is not None:
            if v is not None:
                x += v
            v = x
        if pre is None:
            return None
        return (torch.tanh(pre[0] * v) * pre[1] + pre[2]).to(out_dtype or self.compute_dtype)

    def rms_norm(self, x, w, eps):
        self._count("rms_norm")
        xf = x.float()
        y = xf * torch.rsqrt((xf * xf).mean(-1, keepdim=True) + eps) * w.float()
        return y.to(self.compute_dtype)

    def add_rms_norm(self, x, branch, w, eps):
        x += branch.float()
        return self.rms_norm(x, w, eps)

    def linear(self, h, w, out_float32=False):
        self._count("linear")
        y = h.float() @ w.float().T
        return y if out_float32 else y.to(self.compute_dtype)

    def silu_mul(self, gate_up):
        return self.act_mul(gate_up, "silu")

    def act_mul(self, gate_up, activation="silu", limit=0.0):
        self._count("silu_mul")
        i = gate_up.shape[1] // 2
        g, u = gate_up[:, :i].float(), gate_up[:, i:].float()
        if activation == "swish_clamped":
            g, u = g.clamp(max=limit), u.clamp(-limit, limit)
            return (g * torch.sigmoid(1.702 * g) * (u + 1.0)).to(self.compute_dtype)
        a = g * torch.sigmoid(g) if activation == "silu" else torch.nn.functional.gelu(g, approximate="tanh")
        return (a * u).to(self.compute_dtype)

    def add_rows(self, x, branch=None, extra=None):
        if branch is not None:
            x += branch.float()
        if extra is not None:
            x += extra
        return x

    def gated_act_linear(self, h, w_gate_up, activation="silu"):
        return self.act_mul(self.linear(h, w_gate_up), activation)

    def routed_experts(self, h, w_router, w_gate_up, w_down, top_k, activation="silu", shared=None,
                       shared_activation="silu", activation_limit=0.0, scoring="softmax_top", groups=None):
        self._count("routed_experts")
        E = w_gate_up.shape[0]
        z = h.float() @ w_router.float().T              # (rows behind the experts' and the gate's are padding)
        if scoring == "sigmoid":
            sc = torch.sigmoid(z[:, :E])
            pick = sc
            if groups is not None:
                count, keep, best = groups
                per = sc.view(-1, count, E // count)
                group_score = per.topk(min(best, E // count), dim=-1).values.sum(-1)
                kept = torch.zeros_like(group_score, dtype=torch.bool).scatter_(1, group_score.topk(keep, dim=-1).indices, True)
                pick = sc.masked_fill(~kept[:, :, None].expand_as(per).reshape(-1, E), -1.0)
            idx = torch.topk(pick, top_k, dim=-1).indices
            wt = sc.gather(1, idx)
        else:
            top, idx = torch.topk(z[:, :E], top_k, dim=-1)
            wt = torch.softmax(top, dim=-1)
        y = torch.zeros(h.shape[0], w_down.shape[1], dtype=torch.float32, device=h.device)
        for t in range(h.shape[0]):
            for j in range(top_k):
                e = int(idx[t, j])
                inter = self.act_mul(self.linear(h[t:t + 1], w_gate_up[e]), activation, activation_limit)
                y[t] += wt[t, j] * self.linear(inter, w_down[e]).float()[0]
        if shared is not None:
            s = self.linear(self.gated_act_linear(h, shared[0], shared_activation), shared[1]).float()
            y += torch.sigmoid(z[:, E:E + 1]) * s
        return y

    def materialize(self, h):
        return h

    def linear_add_rms_norm(self, h, w, x, norm_w, eps):
        return self.add_rms_norm(x, self.linear(h, w), norm_w, eps)

    def gated_silu_linear(self, h, w_gate_up):
        return self.silu_mul(self.linear(h, w_gate_up))

    def qkv_rope_write(self, h, w_qkv, nh, nkv, d, position, ctx, kv, block_table, write=True, value_from_key=False):
        qkv = self.linear(h, w_qkv)
        self.rope_kv_write(qkv, nh, nkv, d, position, ctx, kv, block_table, write=write, value_from_key=value_from_key)
        return qkv

    def qkv_attention(self, h, w_qkv, nh, nkv, d, position, ctx, kv, block_table, scale, window, write=True,
                      softcap=None, slopes=None, chunk=None, value_from_key=False):
        qkv = self.qkv_rope_write(h, w_qkv, nh, nkv, d, position, ctx, kv, block_table, write=write,
                                  value_from_key=value_from_key)
        return self.paged_attention(qkv, nh, nkv, d, kv, block_table, ctx, scale, window, softcap=softcap, slopes=slopes,
                                    chunk=chunk)

    def gather_rows(self, x, idx):
        return x[idx.long()].clone()

    # ---- positions -------------------------------------------------------------
    def rope_table(self, inv_freq, max_positions, magnitude=1.0):
        ang = torch.outer(torch.arange(max_positions, dtype=torch.float32), inv_freq.float().cpu())
        return (torch.stack([ang.cos(), ang.sin()], dim=-1) * magnitude).to(self.device)

    def rope_kv_write(self, qkv, nh, nkv, d, position, ctx, kv, block_table, write=True, value_from_key=False):
        self._count("rope_kv_write")
        T = ctx.num_tokens
        q = qkv[:, :nh * d].view(T, nh, d)
        k = qkv[:, nh * d:(nh + nkv) * d].view(T, nkv, d)
        v = k.clone() if value_from_key else qkv[:, (nh + nkv) * d:].view(T, nkv, d)
        pos = ctx.positions.long()
        if position is not None:
            rd = position.rotary_dim
            cs = position.table[pos]                 # [T, rd/2, 2]
            cos, sin = cs[..., 0][:, None, :], cs[..., 1][:, None, :]
            for x in (q, k):
                xf = x[..., :rd].float()
                if position.pairing == "half":
                    a, b = xf[..., :rd // 2], xf[..., rd // 2:]
                    out = torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)
                else:
                    a, b = xf[..., 0::2], xf[..., 1::2]
                    out = torch.stack([a * cos - b * sin, b * cos + a * sin], dim=-1).flatten(-2)
                x[..., :rd] = out.to(x.dtype)
        if write:
            ps = kv.shape[3]
            seq = ctx.token_seq.long()
            for t in range(T):
                if seq[t] < 0:
                    continue
                p = int(pos[t])
                page = int(block_table[seq[t], p // ps])
                assert page >= 0, "write into a page that was given back"
                kv[page, 0, :, p % ps, :] = k[t].to(kv.dtype)
                kv[page, 1, :, p % ps, :] = v[t].to(kv.dtype)

    # ---- attention -------------------------------------------------------------
    def plan_attention(self, q_lens, k_lens, group_size, num_kv_heads, window, head_dim, chunk=None, pad_requests=None,
                       fixed_capacity=False, pad_tokens=None):
        return plan_attention(q_lens, k_lens, group_size, num_kv_heads, window, chunk=chunk, small_rows=16, large_rows=64,
                              min_split_keys=128, num_sms=4, pad_requests=pad_requests, fixed_capacity=fixed_capacity,
                              pad_tokens=pad_tokens)

    def paged_attention(self, qkv, nh, nkv, d, kv, block_table, ctx, scale, window, softcap=None, slopes=None,
                        chunk=None, dist_bias=None, sink=None):
        self._count("paged_attention")
        T = ctx.num_tokens
        q = qkv[:, :nh * d].view(T, nh, d).float()
        out = torch.zeros(T, nh * d, dtype=self.compute_dtype, device=qkv.device)
        ps = kv.shape[3]
        g = nh // nkv
        cu = ctx.host.cu
        for s, (nq, lk) in enumerate(zip(ctx.host.q_lens, ctx.host.k_lens)):
            first = lk - nq
            lo = max(0, first - window + 1) if window else 0
            if chunk:
                lo = max(lo, first - first % chunk)
            idx = torch.arange(lo, lk)
            pages = block_table[s, (idx // ps)].long()
            assert (pages >= 0).all(), "read of a page that was given back"
            k = kv[pages, 0, :, idx % ps, :].float()       # [n, nkv, d]
            v = kv[pages, 1, :, idx % ps, :].float()
            k = k.repeat_interleave(g, dim=1)
            v = v.repeat_interleave(g, dim=1)
            qs = q[cu[s]:cu[s + 1]]
            scores = torch.einsum("qhd,khd->hqk", qs, k) * scale
            qpos = torch.arange(first, lk)
            if softcap:
                scores = softcap * torch.tanh(scores / softcap)
            if slopes is not None:
                scores = scores + slopes.float().cpu()[:, None, None] * (idx[None, None, :] - qpos[None, :, None])
            if dist_bias is not None:
                dist = (qpos[:, None] - idx[None, :]).clamp(0, dist_bias.shape[1] - 1)
                scores = scores + dist_bias.float().cpu()[:, dist]
            hidden = idx[None, :] > qpos[:, None]
            if window:
                hidden |= idx[None, :] <= qpos[:, None] - window
            if chunk:
                hidden |= idx[None, :] < (qpos - qpos % chunk)[:, None]
            scores = scores.masked_fill(hidden[None], float("-inf"))
            if sink is not None:
                # one more term in the denominator, without a value
                scores = torch.cat([scores, sink.float().cpu()[:, None, None].expand(nh, nq, 1)], dim=-1)
                o = torch.einsum("hqk,khd->qhd", scores.softmax(-1)[..., :-1], v)
            else:
                o = torch.einsum("hqk,khd->qhd", scores.softmax(-1), v)
            out[cu[s]:cu[s + 1]] = o.reshape(nq, nh * d).to(self.compute_dtype)
        return out

    # ---- mixers that are not plain grouped-query attention -----------------------
    def _write_slots(self, ctx, kv, block_table, k, v):
        """k, v: [T, heads, D] into the page slots of the step's tokens."""
        ps = kv.shape[3]
        seq, pos = ctx.token_seq.long(), ctx.positions.long()
        for t in range(k.shape[0]):
            if seq[t] < 0:
                continue
            p = int(pos[t])
            page = int(block_table[seq[t], p // ps])
            assert page >= 0, "write into a page that was given back"
            kv[page, 0, :, p % ps, :] = k[t].to(kv.dtype)
            kv[page, 1, :, p % ps, :] = v[t].to(kv.dtype)

    def heads_linear(self, x, col0, head_stride, w, out_float32=False):
        self._count("heads_linear")
        nh, N, K = w.shape
        xs = torch.stack([x[:, col0 + h * head_stride:col0 + h * head_stride + K] for h in range(nh)], dim=1).float()
        y = torch.einsum("thk,hnk->thn", xs, w.float()).reshape(x.shape[0], nh * N)
        return y if out_float32 else y.to(self.compute_dtype)

    @staticmethod
    def _turn(x, position, pos, back=False):
        """x [T, heads, n]: the first rotary_dim elements of each head turned by the table's angles at `pos`
        (`back`: by minus those angles), pairs as the table says."""
        rd = position.rotary_dim
        cs = position.table[pos]                            # [T, rd/2, 2]
        cos, sin = cs[..., 0][:, None, :], cs[..., 1][:, None, :]
        if back:
            sin = -sin
        out = x.clone()
        if position.pairing == "half":
            a, b = x[..., :rd // 2], x[..., rd // 2:rd]
            out[..., :rd // 2], out[..., rd // 2:rd] = a * cos - b * sin, b * cos + a * sin
        else:
            a, b = x[..., 0:rd:2], x[..., 1:rd:2]
            out[..., 0:rd:2], out[..., 1:rd:2] = a * cos - b * sin, b * cos + a * sin
        return out

    def rotated_qkv_write(self, proj, bias, nh, nkv, d, dv, D, position, value_position, ctx, kv, block_table, write=True):
        self._count("rotated_qkv_write")
        T = proj.shape[0]
        n = nh * d + nkv * (d + dv)
        pf = proj[:, :n].float()
        if bias is not None:
            pf = pf + bias.float()
        pos = ctx.positions.long()
        q = pf[:, :nh * d].view(T, nh, d)
        k = pf[:, nh * d:(nh + nkv) * d].view(T, nkv, d)
        v = pf[:, (nh + nkv) * d:].view(T, nkv, dv)
        if position is not None:
            q, k = self._turn(q, position, pos), self._turn(k, position, pos)
        if value_position is not None:
            v = self._turn(v, value_position, pos)
        qp = torch.zeros(T, nh, D)
        qp[:, :, :d] = q
        if write:
            kp, vp = torch.zeros(T, nkv, D), torch.zeros(T, nkv, D)
            kp[:, :, :d], vp[:, :, :dv] = k, v
            self._write_slots(ctx, kv, block_table, kp, vp)
        return qp.reshape(T, nh * D).to(self.compute_dtype)

    def head_unrotate_gate(self, o, nh, D, dv, value_position, ctx, gate=None):
        self._count("head_unrotate_gate")
        T = o.shape[0]
        out = o.float().view(T, nh, D)[:, :, :dv]
        if value_position is not None:
            out = self._turn(out, value_position, ctx.positions.long(), back=True)
        if gate is not None:
            out = out * torch.sigmoid(gate.float())[:, :, None]
        return out.reshape(T, nh * dv).to(self.compute_dtype)

    def causal_conv(self, yx, col0, C, b_in, conv_w, conv_b, state, ctx, activation=None, low=True):
        self._count("causal_conv")
        taps = conv_w.shape[1]
        hist = taps - 1
        x = yx[:, col0:col0 + C].float()
        if b_in is not None:
            x = x + b_in[col0:col0 + C]
        if conv_b is None:
            conv_b = torch.zeros(C)
        out = torch.zeros(yx.shape[0], C)
        cu = ctx.host.cu
        for s, slot in enumerate(ctx.host.state_slots):
            assert slot >= 0, "a request of a model with state must own a slot"
            nq = cu[s + 1] - cu[s]
            seq = torch.cat([state[slot][:hist * C].view(hist, C), x[cu[s]:cu[s + 1]]], dim=0)
            u = conv_b[None, :].expand(nq, C).clone()
            for j in range(taps):
                u = u + seq[j:j + nq] * conv_w[:, j][None, :]
            out[cu[s]:cu[s + 1]] = u
            if hist:
                state[slot][:hist * C] = seq[nq:].reshape(-1)
        if activation == "silu":
            out = out * torch.sigmoid(out)
        if not low:
            return out, None
        low = out.to(self.compute_dtype)
        return out, (out if low.dtype == torch.float32 else low)

    def delta_rule_scan(self, u, proj, gate_col0, decay_rate, decay_bias, H, G, d, dv, unit_eps, q_scale, state_off, state, ctx):
        """u float32 [T, q: G*d | k: G*d | v: H*dv] (convolved, activated); proj columns gate_col0.. hold [beta: H | a: H]."""
        self._count("delta_rule_scan")
        T = u.shape[0]
        q, k = u[:, :G * d].view(T, G, d), u[:, G * d:2 * G * d].view(T, G, d)
        v = u[:, 2 * G * d:].view(T, H, dv)
        q = q * torch.rsqrt((q * q).sum(-1, keepdim=True) + unit_eps) * q_scale
        k = k * torch.rsqrt((k * k).sum(-1, keepdim=True) + unit_eps)
        beta = torch.sigmoid(proj[:, gate_col0:gate_col0 + H].float())
        g = torch.exp(decay_rate * torch.nn.functional.softplus(proj[:, gate_col0 + H:gate_col0 + 2 * H].float() + decay_bias))
        out = torch.zeros(T, H, dv)
        cu = ctx.host.cu
        rep = H // G
        for s, slot in enumerate(ctx.host.state_slots):
            assert slot >= 0, "a request of a model with state must own a slot"
            S = state[slot][state_off:state_off + H * dv * d].view(H, dv, d)          # column j of head h: S[h, j, :]
            for t in range(cu[s], cu[s + 1]):
                for h in range(H):
                    kt, qt = k[t, h // rep], q[t, h // rep]
                    Sh = S[h] * g[t, h]
                    w = beta[t, h] * (v[t, h] - Sh @ kt)
                    Sh = Sh + w[:, None] * kt[None, :]
                    S[h] = Sh
                    out[t, h] = Sh @ qt
        return out.reshape(T, H * dv)

    def normed_pair_sum(self, a, b, wa, wb, sa, sb, eps):
        self._count("normed_pair_sum")

        def normed(x, w):
            x = x.float()
            return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * w.float()

        return sa * normed(a, wa) + sb * normed(b, wb)

    def normed_pair_add_rms_norm(self, x, a, b, wa, wb, sa, sb, pair_eps, norm_w, eps):
        x += self.normed_pair_sum(a, b, wa, wb, sa, sb, pair_eps)
        return self.rms_norm(x, norm_w, eps)

    def gated_recurrence(self, gates, b_gates, u, yx, b_in, rate, blocks, taps, state, ctx):
        self._count("gated_recurrence")
        T, C = u.shape
        bw, hist = C // blocks, taps - 1
        g = gates.view(T, blocks, 2 * bw) + b_gates[None]
        r = torch.sigmoid(g[:, :, :bw]).reshape(T, C)
        i = torch.sigmoid(g[:, :, bw:]).reshape(T, C)
        a = torch.exp(rate[None, :] * r)
        drive = torch.sqrt(1.0 - a * a) * i * u
        y = torch.nn.functional.gelu(yx[:, :C].float() + b_in[:C], approximate="tanh")
        out = torch.zeros(T, C)
        cu = ctx.host.cu
        for s, slot in enumerate(ctx.host.state_slots):
            st = state[slot]
            S = st[hist * C:]
            for t in range(cu[s], cu[s + 1]):
                S.mul_(a[t]).add_(drive[t])
                out[t] = S * y[t]
        return out.to(self.compute_dtype)          # (the convolution has replaced its inputs in the state already)

    def linear_attention_scan(self, proj, z, z_bias, H, d, dv, tau, q_scale, state, ctx):
        self._count("linear_attention_scan")
        T = proj.shape[0]
        pf = proj.float()
        q = pf[:, :H * d].view(T, H, d) * q_scale
        k = pf[:, H * d:2 * H * d].view(T, H, d)
        v = pf[:, 2 * H * d:2 * H * d + H * dv].view(T, H, dv)
        alpha = torch.exp(torch.nn.functional.logsigmoid(z.float() + z_bias) / tau).view(T, H, d)
        out = torch.zeros(T, H * dv)
        cu = ctx.host.cu
        for s, slot in enumerate(ctx.host.state_slots):
            assert slot >= 0, "a request of a model with state must own a slot"
            S = state[slot].view(H, dv, d)
            for t in range(cu[s], cu[s + 1]):
                S.mul_(alpha[t][:, None, :]).add_(v[t][:, :, None] * k[t][:, None, :])
                out[t] = torch.einsum("hvd,hd->hv", S, q[t]).reshape(H * dv)
        return out

    def head_norm_gate(self, o, proj, g_col0, H, dv, norm_w, eps):
        self._count("head_norm_gate")
        T = o.shape[0]
        v = o.view(T, H, dv)
        v = v * torch.rsqrt((v * v).mean(-1, keepdim=True) + eps) * norm_w[None, None, :]
        g = proj[:, g_col0:g_col0 + H * dv].float()
        return (v.reshape(T, H * dv) * (g * torch.sigmoid(g))).to(self.compute_dtype)

    def normed_qkv_write(self, proj, nh, nkv, d, dv, D, q_weight, k_weight, eps, ctx, kv, block_table, has_kv=True,
                         write=True, position=None, query_temperature=None):
        self._count("normed_qkv_write")
        T = proj.shape[0]
        pf = proj.float()
        pos = ctx.positions.long()

        def normed(x, w):
            return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * w

        qn = normed(pf[:, :nh * d], q_weight).view(T, nh, d)
        if position is not None:
            qn = self._turn(qn, position, pos.clamp(min=0))
        if query_temperature is not None:
            coef, every = query_temperature
            qn = qn * (1.0 + coef * torch.log(torch.floor((pos.float() + 1.0) / every) + 1.0))[:, None, None]
        q = torch.zeros(T, nh, D)
        q[:, :, :d] = qn
        if has_kv and write:
            k = torch.zeros(T, nkv, D)
            v = torch.zeros(T, nkv, D)
            kn = normed(pf[:, nh * d:(nh + nkv) * d], k_weight).view(T, nkv, d)
            k[:, :, :d] = self._turn(kn, position, pos.clamp(min=0)) if position is not None else kn
            v[:, :, :dv] = pf[:, (nh + nkv) * d:(nh + nkv) * d + nkv * dv].view(T, nkv, dv)
            self._write_slots(ctx, kv, block_table, k, v)
        return q.reshape(T, nh * D).to(self.compute_dtype)

    def head_gate(self, o, nh, D, dv, gate=None):
        self._count("head_gate")
        T = o.shape[0]
        out = o.float().view(T, nh, D)[:, :, :dv].reshape(T, nh * dv)
        if gate is not None:
            out = out * torch.sigmoid(gate.float())
        return out.to(self.compute_dtype)

    @staticmethod
    def _rotate_pairs(x, position, pos):
        """x [T, ..., n]: pairs (2i, 2i+1) of the first rotary_dim elements."""
        if position is None:
            return x
        rd = position.rotary_dim
        cs = position.table[pos]                            # [T, rd/2, 2]
        shape = [cs.shape[0]] + [1] * (x.dim() - 2) + [rd // 2]
        cos, sin = cs[..., 0].view(shape), cs[..., 1].view(shape)
        a, b = x[..., 0:rd:2], x[..., 1:rd:2]
        out = x.clone()
        out[..., 0:rd:2] = a * cos - b * sin
        out[..., 1:rd:2] = b * cos + a * sin
        return out

    def _rotate_part(self, x, position, pos):
        """x [T, heads, n]: the table's pairing over its rotary_dim leading elements."""
        if position is None:
            return x
        return self._turn(x, position, pos) if position.pairing == "half" else self._rotate_pairs(x, position, pos)

    def latent_kv_write(self, down, q_rank, kv_rank, rot_dim, D, q_weight, c_weight, eps, position, ctx, kv, block_table,
                        write=True, norm_q=True):
        self._count("latent_kv_write")
        T = down.shape[0]
        df = down.float()

        def normed(x, w):
            return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * w

        cq = normed(df[:, :q_rank], q_weight).to(self.compute_dtype) if norm_q else None
        if write:
            c = normed(df[:, q_rank:q_rank + kv_rank], c_weight).to(self.compute_dtype).float()
            kr = self._rotate_part(df[:, None, q_rank + kv_rank:q_rank + kv_rank + rot_dim], position, ctx.positions.long())[:, 0]
            k = torch.zeros(T, 1, D)
            v = torch.zeros(T, 1, D)
            k[:, 0, :kv_rank] = c
            k[:, 0, kv_rank:kv_rank + rot_dim] = kr
            v[:, 0, :kv_rank] = c
            self._write_slots(ctx, kv, block_table, k, v)
        return cq

    def latent_queries(self, q_abs, q, nh, d, rot_dim, kv_rank, D, position, ctx):
        self._count("latent_queries")
        T = q.shape[0]
        out = torch.zeros(T, nh, D)
        out[:, :, :kv_rank] = q_abs.float().view(T, nh, kv_rank)
        qr = q[:, :nh * (d + rot_dim)].float().view(T, nh, d + rot_dim)[:, :, d:]
        out[:, :, kv_rank:kv_rank + rot_dim] = self._rotate_part(qr, position, ctx.positions.long())
        return out.reshape(T, nh * D).to(self.compute_dtype)

    def ssm_mix(self, zx, inner, groups, state_size, heads, head_dim, conv_w, conv_b, dt_bias, a_log, d_skip, norm_w,
                norm_groups, eps, state, ctx):
        self._count("ssm_mix")
        G, N, H, P = groups, state_size, heads, head_dim
        C = inner + 2 * G * N
        taps = conv_w.shape[1]
        hist = taps - 1
        zf = zx.float()
        out = torch.zeros(zx.shape[0], inner)
        cu = ctx.host.cu
        for s, slot in enumerate(ctx.host.state_slots):
            assert slot >= 0, "a request of a model with state must own a slot"
            rows = zf[cu[s]:cu[s + 1]]
            nq = rows.shape[0]
            st = state[slot]
            old = st[:hist * C].view(hist, C)
            S = st[hist * C:].view(H, P, N)
            seq = torch.cat([old, rows[:, inner:inner + C]], dim=0)           # [hist + nq, C]
            xbc = conv_b[None, :].expand(nq, C).clone()
            for k in range(taps):
                xbc = xbc + seq[k:k + nq] * conv_w[:, k][None, :]
            xbc = xbc * torch.sigmoid(xbc)
            old.copy_(seq[nq:nq + hist].clone())
            dt = torch.nn.functional.softplus(rows[:, 2 * inner + 2 * G * N:] + dt_bias[None, :])
            decay = torch.exp(-torch.exp(a_log)[None, :] * dt)
            x = xbc[:, :inner].view(nq, H, P)
            B = xbc[:, inner:inner + G * N].view(nq, G, N).repeat_interleave(H // G, dim=1)
            Cm = xbc[:, inner + G * N:].view(nq, G, N).repeat_interleave(H // G, dim=1)
            y = torch.zeros(nq, H, P)
            for t in range(nq):
                S.mul_(decay[t][:, None, None]).add_(dt[t][:, None, None] * x[t][:, :, None] * B[t][:, None, :])
                y[t] = torch.einsum("hpn,hn->hp", S, Cm[t]) + d_skip[:, None] * x[t]
            v = y.view(nq, inner) * (rows[:, :inner] * torch.sigmoid(rows[:, :inner]))
            v = v.view(nq, norm_groups, inner // norm_groups)
            v = v * torch.rsqrt((v * v).mean(-1, keepdim=True) + eps)
            out[cu[s]:cu[s + 1]] = v.reshape(nq, inner) * norm_w[None, :]
        return out.to(self.compute_dtype)

    def copy_pages(self, pool, pairs):
        self._count("copy_pages")
        for src, dst in pairs:
            pool[:, dst] = pool[:, src]

    # ---- sampling --------------------------------------------------------------
    def argmax(self, logits):
        return logits.argmax(-1)

    def sample(self, logits, temps, top_k, top_p, seeds, counters):
        from tests.plain_sampling import sample_rows
        return torch.tensor(sample_rows(logits.float().cpu().numpy(), temps, top_k, top_p, seeds, counters))
