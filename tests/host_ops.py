"""A stand-in for the CUDA kernel set, for tests of the engine's HOST logic on a machine
without a GPU (batch metadata, cache bookkeeping, scheduling).  It follows the kernels'
calling conventions and cache layout with elementary torch arithmetic on the CPU.  It is
test equipment: the package never imports it, and the `-m gpu` tests never use it.
"""
from __future__ import annotations

import math

import torch


class HostOps:
    def __init__(self):
        self.launches = 0

    def require(self, *names):
        return None

    def choose_kernels(self, kernels):
        return None

    def compile(self, plan):
        return HostPlan(self, plan)

    def embedding(self, ids, table, out):
        out.copy_(table[ids.long()].float())
        return out

    def rmsnorm(self, x, gain, eps, out, delta=None, rows=None):
        if delta is not None:
            if rows is None:
                x += delta.float()
            else:
                x[rows.long()] += delta.float()[rows.long()]
        src = x if rows is None else x[rows.long()]
        ms = (src * src).sum(-1, keepdim=True) / src.shape[-1]
        out.copy_(((src * (1.0 / torch.sqrt(ms + eps))) * gain.float()).to(out.dtype))
        return out

    def qkv_post(self, *, q_in, k_in, v_in, num_heads, num_kv_heads, head_dim, q_gain=None, k_gain=None, eps=0.0,
                 cos_sin=None, positions=None, q_out=None, k_out=None, cache=None, slot_mapping=None, page_size=0):
        hd, half = head_dim, head_dim // 2

        def post(x, heads, gain):
            x = x.float().reshape(x.shape[0], heads, hd)
            if gain is not None:
                ms = (x * x).sum(-1, keepdim=True) / hd
                x = (x * (1.0 / torch.sqrt(ms + eps))) * gain.float()
            if cos_sin is not None:
                cs = cos_sin[positions.long()]
                c, s = cs[:, None, :half], cs[:, None, half:]
                a, b = x[..., :half], x[..., half:]
                x = torch.cat([a * c - b * s, a * s + b * c], -1)
            return x

        def store(which, x):  # x [T, nkv, hd] -> cache[page, which, kvh, off, :]
            for t in range(x.shape[0]):
                slot = int(slot_mapping[t])
                if slot < 0:
                    continue
                cache[slot // page_size, which, :, slot % page_size, :] = x[t].to(cache.dtype)

        if q_in is not None:
            q = post(q_in, num_heads, q_gain)
            if q_out is not None:
                q_out.copy_(q.reshape(q.shape[0], -1).to(q_out.dtype))
        if k_in is not None:
            k = post(k_in, num_kv_heads, k_gain)
            if k_out is not None:
                k_out.copy_(k.reshape(k.shape[0], -1).to(k_out.dtype))
            if cache is not None:
                store(0, k)
        if v_in is not None and cache is not None:
            store(1, v_in.float().reshape(v_in.shape[0], num_kv_heads, hd))

    def attention_plain(self, *, q, cache, out, positions, token_request, block_tables, num_heads, num_kv_heads,
                        head_dim, page_size, window, scale):
        T = q.shape[0]
        g = num_heads // num_kv_heads
        qf = q.float().reshape(T, num_heads, head_dim)
        for t in range(T):
            p = int(positions[t])
            lo = max(0, p - window + 1) if window > 0 else 0
            bt = block_tables[int(token_request[t])]
            js = torch.arange(lo, p + 1)
            pages = bt[(js // page_size).long()].long()
            assert (pages >= 0).all(), "attention would read a page that is not held"
            k = cache[pages, 0, :, (js % page_size).long(), :].float()      # [n, nkv, hd]
            v = cache[pages, 1, :, (js % page_size).long(), :].float()
            for h in range(num_heads):
                s = (k[:, h // g] @ qf[t, h]) * scale
                w = torch.softmax(s, 0)
                out[t, h * head_dim:(h + 1) * head_dim] = (w @ v[:, h // g]).to(out.dtype)
        return out

    # the fast kernels share the plain one's semantics
    attention = attention_plain

    def swiglu(self, gate_up, out):
        inter = out.shape[1]
        g, u = gate_up[:, :inter].float(), gate_up[:, inter:].float()
        out.copy_(((g / (1.0 + torch.exp(-g))) * u).to(out.dtype))
        return out

    def linear(self, x, w, out):
        out.copy_((x.float() @ w.float().t()).to(out.dtype))
        return out

    def repetition_penalty(self, logits, rows, tokens, counts, penalty):
        for r, t, c in zip(rows.tolist(), tokens.tolist(), counts.tolist()):
            p = float(penalty[r])
            for _ in range(c):
                logits[r, t] = logits[r, t] / p if logits[r, t] > 0 else logits[r, t] * p

    def sample(self, logits, *, greedy, temperature, top_k, top_p, u, out):
        from plain_model import plain_sample
        for r in range(logits.shape[0]):
            out[r] = plain_sample(logits[r], greedy=bool(greedy[r]), temperature=float(temperature[r]),
                                  top_k=int(top_k[r]), top_p=float(top_p[r]), u=float(u[r]))
        return out


class HostPlan:
    """A plan interpreted on the CPU: every record runs on the first rows of its buffers, as the native
    executor runs it on the device."""

    def __init__(self, ops, plan):
        self.ops, self.plan = ops, plan

    def run(self, batch, first=0, count=-1):
        o = self.ops
        T, NL = batch.num_tokens, batch.logit_rows.numel()
        last = len(self.plan.ops) if count < 0 else first + count

        def n_rows(kind):
            return NL if kind == "logits" else T

        def cut(t, n=T):
            return None if t is None else t[:n]
        for op in self.plan.ops[first:last]:
            a, k = op.a, op.kind
            if k == "embedding":
                o.embedding(batch.token_ids, a["table"], a["out"][:T])
            elif k == "rmsnorm":
                some = a["rows"] == "logits"
                o.rmsnorm(a["x"][:T], a["gain"], a["eps"], a["out"][:n_rows(a["rows"])], delta=cut(a["delta"]),
                          rows=batch.logit_rows if some else None)
            elif k == "linear":
                n = n_rows(a["rows"])
                if n:
                    o.linear(a["x"][:n], a["w"], batch.logits if a["out"] is None else a["out"][:n])
            elif k == "linear_swiglu":
                o.linear(a["x"][:T], a["w_gate_up"], a["gate_up"][:T])
                o.swiglu(a["gate_up"][:T], a["out"][:T])
            elif k == "qkv_post":
                self._qkv_post(a, batch, T)
            elif k == "attend":
                self._attend(a, batch, T)
            elif k == "attention":
                nh, nkv, hd = a["num_heads"], a["num_kv_heads"], a["head_dim"]
                qs, kvs = nh * hd, nkv * hd
                qkv, w = a["qkv"], a["writes"]
                self._qkv_post(dict(a, q_in=qkv[:, :qs], k_in=qkv[:, qs:qs + kvs] if w else None,
                                    v_in=qkv[:, qs + kvs:] if w else None, q_out=a["q"], k_out=None,
                                    cache=a["cache"] if w else None), batch, T)
                self._attend(a, batch, T)
            elif k == "call":
                a["fn"](batch)
            else:
                raise ValueError(k)

    def _qkv_post(self, a, batch, T):
        cut = lambda t: None if t is None else t[:T]
        g = batch.groups[a["group"]] if a.get("cache") is not None else None
        self.ops.qkv_post(q_in=cut(a.get("q_in")), k_in=cut(a.get("k_in")), v_in=cut(a.get("v_in")), num_heads=a["num_heads"],
                          num_kv_heads=a["num_kv_heads"], head_dim=a["head_dim"], q_gain=a.get("q_gain"), k_gain=a.get("k_gain"),
                          eps=a.get("eps", 0.0), cos_sin=a.get("cos_sin"), positions=batch.positions, q_out=cut(a.get("q_out")),
                          k_out=cut(a.get("k_out")), cache=a.get("cache"), slot_mapping=g.slot_mapping if g else None,
                          page_size=g.page_size if g else 0)

    def _attend(self, a, batch, T):
        g = batch.groups[a["group"]]
        self.ops.attention_plain(q=a["q"][:T], cache=a["cache"], out=a["out"][:T], positions=batch.positions,
                                 token_request=batch.token_request, block_tables=g.block_tables, num_heads=a["num_heads"],
                                 num_kv_heads=a["num_kv_heads"], head_dim=a["head_dim"], page_size=g.page_size,
                                 window=a["window"], scale=a["scale"])
