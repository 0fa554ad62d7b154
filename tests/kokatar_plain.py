"""A plain, slow float64 restatement of the Kokatar design, one function per mechanism, reading raw checkpoint tensors by
name.  It shares no code with ssd_b200: the tests compare libssdk against it.

Notation: x residual row, n(x) = x / sqrt(mean(x^2) + eps) * w, h = n(x), s(.) the logistic function.
    layer     x <- x + s(G1 h + b1) * mixer(h + conv1(h)) + s(G2 h + b2) * ff(h + conv2(h))
    conv      per channel over time: y_t = sum_j w[:, j] u_(t - taps + 1 + j), u = 0 before the sequence starts
Every function that looks back in time takes `state` (what earlier portions of the sequence left) and the position p0 of
its first row, so that a sequence can be run whole, in portions or token by token."""
from __future__ import annotations

import torch

F64 = torch.float64


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return unit_rms(x, eps) * w


def short_conv(u, w, state, key):
    """u [n, C] rows of this portion, w [C, taps]; state[key] keeps the last taps - 1 rows of u seen so far."""
    taps = w.shape[1]
    prev = state.get(key)
    if prev is None:
        prev = torch.zeros(taps - 1, u.shape[1], dtype=F64)
    full = torch.cat([prev, u])
    state[key] = full[full.shape[0] - (taps - 1):].clone()
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + w[:, j] * full[j:j + u.shape[0]]
    return y


def rotate_half(x, pos, dims, base):
    """x [n, heads, D]; entry i < dims/2 turns with entry i + dims/2 by the angle pos * base^(-2i/dims); the rest stays."""
    if dims < 2:
        return x
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    a = torch.tensor(pos, dtype=F64)[:, None] * f[None, :]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    lo, hi = x[..., :half], x[..., half:dims]
    return torch.cat([lo * c - hi * s, hi * c + lo * s, x[..., dims:]], -1)


def first_visible(i, window):
    """The oldest key a query at position i reads: a window keeps the last `window` positions, i included (0: all of them)."""
    return max(0, i - window + 1) if window else 0


def windowed_softmax_attention(q, k, v, p0, scale, window, sink=None):
    """q [n, D] at positions p0 .., k [p0 + n, D], v [p0 + n, V] from position 0.  A sink is a logit that joins the
    denominator once, unscaled, and carries no value."""
    out = torch.zeros(q.shape[0], v.shape[1], dtype=F64)
    for r in range(q.shape[0]):
        i = p0 + r
        lo = first_visible(i, window)
        sc = (k[lo:i + 1] @ q[r]) * scale
        mx = sc.max() if sink is None else torch.maximum(sc.max(), sink)
        e = torch.exp(sc - mx)
        den = e.sum() + (torch.exp(sink - mx) if sink is not None else 0.0)
        out[r] = (e / den) @ v[lo:i + 1]
    return out


def attention_mixer(h, W, p, m, state, p0):
    n = h.shape[0]
    H, G, D, V = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m.get("vdim", m["dim"])
    rot = m.get("rot") or {}
    dims, base = int(rot.get("dims", 0)), float(rot.get("base", 10000.0))
    proj = {}
    for s in "qkv":
        z = h @ W[f"{p}.{s}"].T + W[f"{p}.{s}.b"]
        proj[s] = short_conv(z, W[f"{p}.{s}.conv"], state, "conv_" + s) if f"{p}.{s}.conv" in W else z
    pos = list(range(p0, p0 + n))
    q = rotate_half(proj["q"].view(n, H, D), pos, dims, base)
    k = rotate_half(proj["k"].view(n, G, D), pos, dims, base)
    v = proj["v"].view(n, G, V)
    state["k"] = torch.cat([state["k"], k]) if "k" in state else k
    state["v"] = torch.cat([state["v"], v]) if "v" in state else v
    window = int((m.get("mask") or {}).get("size", 0))
    heads = [windowed_softmax_attention(q[:, hd], state["k"][:, hd // (H // G)], state["v"][:, hd // (H // G)], p0, m["scale"], window,
                                        W[p + ".sink"][hd]) for hd in range(H)]
    return torch.cat(heads, -1) @ W[p + ".o"].T


def latent_attention_mixer(h, W, p, m, eps, state, p0):
    n = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = (h @ W[p + ".q"].T).view(n, H, D)
    c = rms_norm(h @ W[p + ".dkv"].T, W[p + ".dkv.norm"], eps)
    state["c"] = torch.cat([state["c"], c]) if "c" in state else c
    k = (state["c"] @ W[p + ".uk"].T).view(-1, H, D)
    v = (state["c"] @ W[p + ".uv"].T).view(-1, H, V)
    window = int((m.get("mask") or {}).get("size", 0))
    heads = [windowed_softmax_attention(q[:, hd], k[:, hd], v[:, hd], p0, m["scale"], window) for hd in range(H)]
    return torch.cat(heads, -1) @ W[p + ".o"].T


def polynorm(z, coef, eps):
    return coef[0] * unit_rms(z, eps) + coef[1] * unit_rms(z ** 2, eps) + coef[2] * unit_rms(z ** 3, eps) + coef[3]


def dense_ff(h, W, p, eps):
    return polynorm(h @ W[p + ".up"].T, W[p + ".act"], eps) @ W[p + ".down"].T


def relu2_expert(h, up, down):
    return torch.relu(h @ up.T) ** 2 @ down.T


def route_top(z, top):
    """The `top` largest logits (ties to the lower index) and the softmax over just those."""
    order = sorted(range(z.shape[0]), key=lambda e: (-float(z[e]), e))[:top]
    return order, torch.softmax(z[order], -1)


def moe_ff(h, W, p, m):
    z = h @ W[p + ".router"].T
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        chosen, wts = route_top(z[t], m["router"]["top"])
        for e, wt in zip(chosen, wts):
            out[t] += wt * relu2_expert(h[t:t + 1], W[f"{p}.e{e}.up"], W[f"{p}.e{e}.down"])[0]
    if m.get("shared"):
        g = torch.sigmoid(h @ W[p + ".shared.sg"].reshape(-1))[:, None]
        out = out + g * relu2_expert(h, W[p + ".shared.up"], W[p + ".shared.down"])
    return out


class PlainModel:
    def __init__(self, cfg: dict, tensors: dict):
        self.cfg = cfg
        self.W = {k: v.to(F64) for k, v in tensors.items()}

    def new_state(self):
        return [dict() for _ in self.cfg["layers"]]

    def sublayer_input(self, h, i, which, state):
        key = f"l{i}.canon{which}"
        return h + short_conv(h, self.W[key], state, "canon" + which) if key in self.W else h

    def run(self, tokens, state=None, p0=0, layers_out=None):
        """Logits [n, vocab] of `tokens` continuing a sequence at position p0 with `state` (None: a new sequence)."""
        cfg, W = self.cfg, self.W
        eps = cfg["norm"]["eps"]
        state = state if state is not None else self.new_state()
        x = W["embed"][torch.tensor(list(tokens))]
        for i, lc in enumerate(cfg["layers"]):
            p, st = f"l{i}", state[i]
            h = rms_norm(x, W[p + ".norm1"], eps)
            hm = self.sublayer_input(h, i, "1", st)
            if lc["type"] == "attention":
                y = attention_mixer(hm, W, p + ".mix", lc["mixer"], st, p0)
            else:
                y = latent_attention_mixer(hm, W, p + ".mix", lc["mixer"], eps, st, p0)
            y = y * torch.sigmoid(h @ W[p + ".rg1"].T + W[p + ".rg1.b"])
            mlp = lc.get("mlp")
            if mlp:
                hf = self.sublayer_input(h, i, "2", st)
                f = dense_ff(hf, W, p + ".mlp", eps) if mlp["kind"] == "dense" else moe_ff(hf, W, p + ".mlp", mlp)
                y = y + f * torch.sigmoid(h @ W[p + ".rg2"].T + W[p + ".rg2.b"])
            x = x + y
            if layers_out is not None:
                layers_out.append(x.clone())
        return rms_norm(x, W["final.norm"], eps) @ W["head"].T

    def greedy(self, prompt, n_new):
        state = self.new_state()
        logits = self.run(prompt, state, 0)
        out, pos = [], len(prompt)
        for _ in range(n_new):
            tok = int(torch.argmax(logits[-1]))
            out.append(tok)
            logits = self.run([tok], state, pos)
            pos += 1
        return out
