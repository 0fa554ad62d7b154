"""Plain, slow restatement of the Lisenex design in float64 on the CPU — the oracle of tests/test_lisenex_*.py.
One function per mechanism, written from the design's equations; it shares no code with ssd_b200 (it reads the raw
checkpoint tensors by name, not the packed layout, and keeps its own per-layer cache lists).

The design: x0 = embed[token] * s_e; every layer is a parallel block with two norms,
    x <- x + mixer(n1(x)) + ff(n2(x)),      n(x) = x / sqrt(mean(x^2) + eps) * w,
the mixer is latent attention (full-rank queries, a cached latent c_t plus ONE rotated key part per token, interleaved
rotation, plain causal softmax, sigmoid output gate; a layer may read another layer's cache instead of making its own),
the feed-forward is none, dense (squared relu, biases) or a mixture of silu-GLU experts behind a softmax router with a
selection bias, group limits and identity experts, plus an always-on shared expert.  Logits = embed . n_f(x)."""
from __future__ import annotations

import torch

F64 = torch.float64


def unit_rms(v: torch.Tensor, eps: float) -> torch.Tensor:
    return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)


def rms_norm(x, weight, eps):
    return unit_rms(x, eps) * weight


def rotate_interleaved(vec, pos, dims, base):
    """vec [..., R]: entries (2i, 2i+1), i < dims/2, are turned by the angle pos * base^(-2i/dims); the rest pass."""
    half = dims // 2
    ang = pos * base ** (-2.0 * torch.arange(half, dtype=F64) / dims)
    u, v = vec[..., 0:dims:2], vec[..., 1:dims:2]
    out = vec.clone()
    out[..., 0:dims:2] = u * torch.cos(ang) - v * torch.sin(ang)
    out[..., 1:dims:2] = v * torch.cos(ang) + u * torch.sin(ang)
    return out


def latent_attention_mixer(h, W, p, mx, eps, cache, p0):
    """h [n, width] rows of one sequence from position p0; cache = {"c": [...], "kr": [...]} of the layer whose latents
    this layer reads (its own, or the one `kv_from` names — then that layer has already appended these rows)."""
    H, D, R, V, KR = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
    dims, base = mx["rot"]["dims"], mx["rot"]["base"]
    own = mx.get("kv_from") is None
    lat, rot = cache.setdefault("c", []), cache.setdefault("kr", [])
    out = []
    for t in range(h.shape[0]):
        pos, cur = p0 + t, h[t]
        q = (W[p + ".q"] @ cur).view(H, D + R)
        if own:
            down = W[p + ".dkv"] @ cur
            lat.append(rms_norm(down[:KR], W[p + ".dkv.norm"], eps))
            rot.append(rotate_interleaved(down[KR:], pos, dims, base))
        C, KRm = torch.stack(lat[:pos + 1]), torch.stack(rot[:pos + 1])      # [ctx, KR], [ctx, R]
        keys = (C @ W[p + ".uk"].T).view(-1, H, D)
        vals = (C @ W[p + ".uv"].T).view(-1, H, V)
        o = torch.zeros(H, V, dtype=F64)
        for hd in range(H):
            qr = rotate_interleaved(q[hd, D:], pos, dims, base)
            s = (keys[:, hd] @ q[hd, :D] + KRm @ qr) * mx["scale"]
            o[hd] = torch.softmax(s, 0) @ vals[:, hd]
        gate = torch.sigmoid(W[p + ".g"] @ cur)
        out.append(W[p + ".o"] @ (o.reshape(-1) * gate))
    return torch.stack(out)


def dense_ff(h, W, p):
    a = torch.relu(h @ W[p + ".up"].T + W[p + ".up.b"]) ** 2
    return a @ W[p + ".down"].T + W[p + ".down.b"]


def silu_expert(h, gate, up, down):
    return (torch.nn.functional.silu(h @ gate.T) * (h @ up.T)) @ down.T


def route(scores, correction, top, groups, keep):
    """scores [E + I] of one token (softmax over all router outputs) -> (chosen outputs, their weights).  The choice is
    made on scores + correction inside the `keep` groups whose best choice score is largest; the weights are the plain
    scores, not renormalised."""
    n = scores.numel()
    per = n // groups
    choice = (scores + correction).tolist()
    gscore = [max(choice[g * per:(g + 1) * per]) for g in range(groups)]
    kept = sorted(range(groups), key=lambda g: (-gscore[g], g))[:keep]
    allowed = [e for g in kept for e in range(g * per, (g + 1) * per)]
    chosen = sorted(allowed, key=lambda e: (-choice[e], e))[:top]
    return chosen, [scores[e] for e in chosen]


def moe_ff(h, W, p, m):
    r = m["router"]
    grp = r.get("groups") or {}
    groups = grp.get("count", 1)
    keep = grp.get("keep", groups)
    E, ident = r["experts"], r.get("identity", 0)
    scores = torch.softmax(h @ W[p + ".router"].T, -1)
    corr = W[p + ".correction"] if (p + ".correction") in W else torch.zeros(E + ident, dtype=F64)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        chosen, wts = route(scores[t], corr, r["top"], groups, keep)
        for e, wt in zip(chosen, wts):
            if e >= E:      # identity expert: the input itself
                out[t] += wt * h[t]
            else:
                q = f"{p}.e{e}"
                out[t] += wt * silu_expert(h[t:t + 1], W[q + ".gate"], W[q + ".up"], W[q + ".down"])[0]
    if m.get("shared"):
        q = p + ".shared"
        out = out + silu_expert(h, W[q + ".gate"], W[q + ".up"], W[q + ".down"])
    return out


class PlainModel:
    def __init__(self, cfg: dict, tensors: dict):
        self.cfg = cfg
        self.W = {k: v.to(F64) for k, v in tensors.items()}

    def new_state(self):
        return [dict() for _ in self.cfg["layers"]]

    def run(self, tokens, state=None, p0=0, layers_out=None):
        """Logits [n, vocab] of `tokens` continuing a sequence at position p0 with `state` (None: a new sequence)."""
        cfg, W = self.cfg, self.W
        eps = cfg["norm"]["eps"]
        state = state if state is not None else self.new_state()
        x = W["embed"][torch.tensor(list(tokens))] * (cfg.get("embedding") or {}).get("scale", 1.0)
        for i, lc in enumerate(cfg["layers"]):
            p, mx = f"l{i}", lc["mixer"]
            src = mx.get("kv_from")
            y = latent_attention_mixer(rms_norm(x, W[p + ".norm1"], eps), W, p + ".mix", mx, eps,
                                       state[i if src is None else src], p0)
            mlp = lc.get("mlp")
            if mlp:
                h2 = rms_norm(x, W[p + ".norm2"], eps)
                y = y + (dense_ff(h2, W, p + ".mlp") if mlp["kind"] == "dense" else moe_ff(h2, W, p + ".mlp", mlp))
            x = x + y
            if layers_out is not None:
                layers_out.append(x.clone())
        return rms_norm(x, W["final.norm"], eps) @ W["embed"].T

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
