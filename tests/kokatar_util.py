"""Small random Kokatar checkpoints for the tests: configuration builders and seeded weights (values representable in
bfloat16, so that both storage types and the float64 oracle read the same numbers).  The safetensors writer is the one of
tests/pikavik_util.py."""
from __future__ import annotations

import torch

from tests.pikavik_util import rel_err, write_checkpoint  # noqa: F401  (re-exported)


def dense(ff=28):
    return {"kind": "dense", "ff": ff}


def moe(experts=6, top=2, ff=20, shared_ff=12):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top},
            "shared": {"ff": shared_ff} if shared_ff else None}


def attention(heads=6, kv_heads=2, dim=10, vdim=6, conv=3, window=24, scale=0.4, dims=6, base=300.0, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "mask": {"size": window}, "scale": scale}
    if dims:
        m["rot"] = {"base": base, "dims": dims}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def latent(heads=3, dim=10, vdim=14, kv_rank=20, window=17, scale=0.3, mlp=None):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "mask": {"size": window}, "scale": scale}, "mlp": mlp}


def config(layers, width=40, vocab=50, eps=1e-6, taps=2):
    return {"architecture": "Kokatar", "canon": {"taps": taps}, "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}


def random_tensors(cfg: dict, seed: int = 0) -> dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    W, taps = cfg["width"], cfg["canon"]["taps"]

    def lin(o, i, gain=1.0):
        return torch.randn(o, i, generator=g) * gain / i ** 0.5

    def vec(n, mean=0.0, std=0.1):
        return mean + std * torch.randn(n, generator=g)

    t = {"embed": torch.randn(cfg["vocab"], W, generator=g), "head": lin(cfg["vocab"], W), "final.norm": vec(W, 1.0, 0.2)}
    for i, lc in enumerate(cfg["layers"]):
        p, mx, m = f"l{i}.", f"l{i}.mix.", lc["mixer"]
        H, D, V = m["heads"], m["dim"], m["vdim"]
        t[p + "norm1"] = vec(W, 1.0, 0.2)
        t[p + "canon1"] = 0.5 * torch.randn(W, taps, generator=g)
        t[p + "rg1"], t[p + "rg1.b"] = lin(W, W, 2.0), vec(W, 0.5, 0.5)
        if lc["type"] == "attention":
            G = m["kv_heads"]
            for s, rows in (("q", H * D), ("k", G * D), ("v", G * V)):
                t[mx + s], t[mx + s + ".b"] = lin(rows, W), vec(rows, 0.0, 0.3)
                t[mx + s + ".conv"] = 0.6 * torch.randn(rows, m["conv"], generator=g)
            t[mx + "sink"], t[mx + "o"] = vec(H, 0.0, 1.0), lin(W, H * V)
        else:
            KR = m["kv_rank"]
            t[mx + "q"], t[mx + "dkv"], t[mx + "dkv.norm"] = lin(H * D, W), lin(KR, W), vec(KR, 1.0, 0.2)
            t[mx + "uk"], t[mx + "uv"], t[mx + "o"] = lin(H * D, KR), lin(H * V, KR), lin(W, H * V)
        mlp = lc.get("mlp")
        if not mlp:
            continue
        q = p + "mlp."
        t[p + "canon2"] = 0.5 * torch.randn(W, taps, generator=g)
        t[p + "rg2"], t[p + "rg2.b"] = lin(W, W, 2.0), vec(W, 0.5, 0.5)
        if mlp["kind"] == "dense":
            ff = mlp["ff"]
            t[q + "up"], t[q + "down"] = lin(ff, W), lin(W, ff)
            t[q + "act"] = torch.tensor([0.6, 0.4, -0.3, 0.1]) + 0.1 * torch.randn(4, generator=g)
            continue
        ff = mlp["expert"]["ff"]
        t[q + "router"] = lin(mlp["router"]["experts"], W, 3.0)
        for e in range(mlp["router"]["experts"]):
            t[f"{q}e{e}.up"], t[f"{q}e{e}.down"] = lin(ff, W, 1.5), lin(W, ff)
        if mlp.get("shared"):
            sff = mlp["shared"]["ff"]
            t[q + "shared.up"], t[q + "shared.down"], t[q + "shared.sg"] = lin(sff, W, 1.5), lin(W, sff), lin(1, W, 2.0)
    return {k: v.to(torch.bfloat16).to(torch.float32) for k, v in t.items()}
