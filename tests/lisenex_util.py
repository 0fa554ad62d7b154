"""Small random Lisenex checkpoints for the tests: configuration builders and seeded weights (values representable in
bfloat16, so that both storage types and the float64 oracle read the same numbers).  The safetensors writer is the one of
tests/pikavik_util.py."""
from __future__ import annotations

import torch

from tests.pikavik_util import rel_err, write_checkpoint  # noqa: F401  (re-exported)


def dense(ff=28):
    return {"kind": "dense", "ff": ff}


def moe(experts=6, identity=2, top=3, groups=4, keep=2, ff=20, shared_ff=12):
    """experts + identity router outputs in `groups` equal groups."""
    return {"kind": "moe", "expert": {"ff": ff},
            "router": {"experts": experts, "identity": identity, "groups": {"count": groups, "keep": keep}, "top": top},
            "shared": {"ff": shared_ff} if shared_ff else None}


def latent(heads=3, dim=10, rot_dim=8, vdim=14, kv_rank=20, scale=0.3, base=10000.0, dims=None, kv_from=None, mlp=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
         "rot": {"base": base, "dims": rot_dim if dims is None else dims}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def config(layers, width=40, vocab=50, eps=1e-6, embed_scale=3.0):
    return {"architecture": "Lisenex", "embedding": {"scale": embed_scale}, "layers": layers, "norm": {"eps": eps},
            "vocab": vocab, "width": width}


def random_tensors(cfg: dict, seed: int = 0, correction: float = 0.3) -> dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]

    def lin(o, i, gain=1.0):
        return torch.randn(o, i, generator=g) * gain / i ** 0.5

    def vec(n, mean=0.0, std=0.1):
        return mean + std * torch.randn(n, generator=g)

    t = {"embed": torch.randn(cfg["vocab"], W, generator=g) / cfg["embedding"]["scale"], "final.norm": vec(W, 1.0, 0.2)}
    for i, lc in enumerate(cfg["layers"]):
        p, mx, m = f"l{i}.", f"l{i}.mix.", lc["mixer"]
        H, D, R, V, KR = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
        t[p + "norm1"] = vec(W, 1.0, 0.2)
        t[mx + "q"], t[mx + "g"], t[mx + "o"] = lin(H * (D + R), W), lin(H * V, W, 2.0), lin(W, H * V)
        if m.get("kv_from") is None:
            t[mx + "dkv"], t[mx + "dkv.norm"] = lin(KR + R, W), vec(KR, 1.0, 0.2)
        t[mx + "uk"], t[mx + "uv"] = lin(H * D, KR), lin(H * V, KR)
        mlp = lc.get("mlp")
        if not mlp:
            continue
        q = p + "mlp."
        t[p + "norm2"] = vec(W, 1.0, 0.2)
        if mlp["kind"] == "dense":
            ff = mlp["ff"]
            t[q + "up"], t[q + "up.b"], t[q + "down"], t[q + "down.b"] = lin(ff, W), vec(ff, 0.0, 0.3), lin(W, ff), vec(W, 0.0, 0.3)
            continue
        r, ff = mlp["router"], mlp["expert"]["ff"]
        n_out = r["experts"] + r.get("identity", 0)
        t[q + "router"] = lin(n_out, W, 3.0)
        # selection biases of both signs and of the size of the scores themselves: choice scores can be negative
        t[q + "correction"] = correction * torch.randn(n_out, generator=g)
        for e in range(r["experts"]):
            t[f"{q}e{e}.gate"], t[f"{q}e{e}.up"], t[f"{q}e{e}.down"] = lin(ff, W, 2.0), lin(ff, W, 2.0), lin(W, ff)
        if mlp.get("shared"):
            sff = mlp["shared"]["ff"]
            t[q + "shared.gate"], t[q + "shared.up"], t[q + "shared.down"] = lin(sff, W, 2.0), lin(sff, W, 2.0), lin(W, sff)
    return {k: v.to(torch.bfloat16).to(torch.float32) for k, v in t.items()}
