"""Layered ("hybrid") models: a program of layers, each one token mixer + an optional feed-forward.  Four designs are
served through this module, told apart by config.json's `"architecture"`:

    Pikavik   parallel pre-norm blocks (mixer and mixture-of-experts feed-forward read the same normed input, unit-offset
              norm weights, layer scales); mixers mLSTM, RWKV-style wkv and latent attention
    Kefurax   serial post-norm blocks (x += m * norm(sublayer(x)): the sublayers read x itself, plain norm weights, scaled
              embedding); mixers rglru (gated diagonal recurrence behind a short convolution), mamba1 (selective scan)
              and `parallel` (grouped-query sink attention with YaRN-scaled interleaved rotation beside a gated delta
              rule); dense gelu-GLU feed-forward
    Lisenex   parallel blocks with two norms (x += mixer(norm1 x) + ff(norm2 x), plain norm weights, scaled embedding,
              head tied to the embedding); latent attention with full-rank queries, interleaved rotation, plain
              softmax, a sigmoid output gate and layers that read another layer's latent cache (`kv_from`);
              feed-forward dense (squared relu, biases) or a mixture of silu-GLU experts behind a softmax router
              with a selection bias, group limits, identity experts and an ungated shared expert
    Kokatar   parallel blocks with ONE norm: mixer and feed-forward each read h + conv(h) (a short causal convolution
              over time of the normed rows, taps of their own) and each result is multiplied by sigmoid(W_g h + b) before
              it joins the residual; mixers `attention` (grouped-query, biased q | k | v behind a short convolution,
              rotate-half rotation of the first dims, sliding window, a learned sink logit per head) and latent attention
              without positions (sliding window, plain softmax); feed-forward dense with a PolyNorm activation or a
              mixture of squared-relu experts whose weights are the softmax over the chosen logits, plus a gated shared
              expert

    HybridSpec     what config.json (and, for sizes it does not list, the checkpoint's tensor shapes) says
    load_hybrid_weights   safetensors -> device tensors in the packed layout libssdk's ssdk_hyb_bind expects
    HybridRunner   owner of the device state behind one ssdk_hyb handle (weights, paged latent cache, recurrent-state
                   slots, workspace); `forward` runs one ragged batch — prompt portions beside single decode tokens

PyTorch is plumbing only (allocation, host->device copies of weights); every FLOP runs in libssdk.  The reference has no
model of this family, so nothing here cites it; the runner mirrors PairRunner's conventions (runner.py)."""
from __future__ import annotations

import ctypes as C
import json
import os
import struct
from dataclasses import dataclass, field

import numpy as np
import torch

from . import lib as L

MIXERS = {"wkv": L.MIX_WKV, "mlstm": L.MIX_MLSTM, "latent_attention": L.MIX_LATENT_ATTN, "rglru": L.MIX_RGLRU,
          "mamba1": L.MIX_SELECTIVE, "parallel": L.MIX_ATTN_DELTA, "attention": L.MIX_ATTENTION}
# which mixers and feed-forwards a design may list, and how its blocks join the residual stream
DESIGNS = {
    "Pikavik": {"mixers": ("wkv", "mlstm", "latent_attention"), "mlp": ("moe",), "block": L.BLOCK_PARALLEL_PRENORM,
                "norm_offset": 1.0},
    "Kefurax": {"mixers": ("rglru", "mamba1", "parallel"), "mlp": ("dense",), "block": L.BLOCK_SERIAL_POSTNORM,
                "norm_offset": 0.0},
    # constants the design fixes, as the arguments the shared mechanisms take
    "Lisenex": {"mixers": ("latent_attention",), "mlp": ("dense", "moe"), "block": L.BLOCK_PARALLEL_TWO_NORMS,
                "norm_offset": 0.0, "dense": "ffn", "tied_head": True,
                "latent": {"rot_interleaved": 1, "out_gate": 1, "learned_sink": 0},
                "moe": {"route_softmax": 1, "route_bias": 1, "group_best": 1, "route_renorm": 0, "expert_act": L.ACT_SILU,
                        "shared_gate": 0},
                "ffn": {"ff_act": L.ACT_RELU2}},
    "Kokatar": {"mixers": ("attention", "latent_attention"), "mlp": ("dense", "moe"), "block": L.BLOCK_PARALLEL_ONE_NORM,
                "norm_offset": 0.0, "dense": "ffn", "gated_residual": True,
                "attention": {"rot_half": 1, "learned_sink": 1},
                "latent": {"rot_interleaved": 0, "out_gate": 0, "learned_sink": 0},
                "moe": {"route_top_softmax": 1, "group_best": 1, "expert_act": L.ACT_RELU2, "expert_glu": 0, "shared_gate": 1},
                "ffn": {"ff_act": L.ACT_POLYNORM}},
}
RGLRU_DECAY_MULT = 8.0  # log a = -8 r softplus(lam)


@dataclass
class LayerSpec:
    mixer: str
    heads: int
    dim: int
    vdim: int = 0
    rot_dim: int = 0
    rot_dims: int = 0
    rot_base: float = 10000.0
    kv_rank: int = 0
    q_rank: int = 0
    attn_scale: float = 1.0
    gate_cap: float = 0.0
    decay_rank: int = 0
    # feed-forward (None = the layer has none)
    mlp: str | None = None
    experts: int = 0
    top: int = 0
    groups: int = 1
    keep: int = 1
    route_scale: float = 1.0
    ff: int = 0
    limit: float = 0.0
    shared_ff: int = 0
    shared_limit: float = 0.0
    # grouped-query attention of the `parallel` mixer (heads / dim / vdim / rot_dims / rot_base / attn_scale above)
    kv_heads: int = 0
    qk_norm: int = 0
    sink: float = 0.0
    yarn_factor: float = 0.0
    yarn_original: float = 0.0
    yarn_fast: float = 0.0
    yarn_slow: float = 0.0
    # short convolution; rglru (inner channels, blocks); selective scan (inner, state, dt_rank)
    conv: int = 0
    inner: int = 0
    blocks: int = 0
    state: int = 0
    dt_rank: int = 0
    decay_mult: float = 0.0
    # gated delta rule of the `parallel` mixer
    d_heads: int = 0
    d_kv_heads: int = 0
    d_dim: int = 0
    d_vdim: int = 0
    left_scale: float = 1.0
    right_scale: float = 1.0
    # latent attention variants (the defaults are Pikavik's: rotate-half, own cache, no output gate, learned sink)
    rot_interleaved: int = 0
    kv_from: int = -1
    out_gate: int = 0
    learned_sink: int = 1
    # router / expert variants (the defaults are Pikavik's: sigmoid scores, group score = two best, renormalised weights,
    # clamped GLU, gated shared expert)
    identity: int = 0
    route_softmax: int = 0
    route_bias: int = 0
    group_best: int = 2
    route_renorm: int = 1
    expert_act: int = L.ACT_CLAMPED
    shared_gate: int = 1
    ff_act: int = L.ACT_RELU2
    # attention window (0: none), pairing of the `attention` mixer's rotation, experts with or without a gate matrix,
    # weights = softmax over the chosen logits
    window: int = 0
    rot_half: int = 0
    expert_glu: int = 1
    route_top_softmax: int = 0

    def cfg(self) -> L.HybLayerCfg:
        mlp = {"moe": L.MLP_MOE, "dense": L.MLP_GLU, "ffn": L.MLP_FFN, None: L.MLP_NONE}[self.mlp]
        return L.HybLayerCfg(MIXERS[self.mixer], self.heads, self.dim, self.vdim, self.rot_dim, self.rot_dims, self.kv_rank,
                             self.q_rank, self.decay_rank, self.rot_base, self.attn_scale, self.gate_cap,
                             mlp, self.experts, self.top, self.groups, self.keep,
                             self.ff, self.shared_ff, self.route_scale, self.limit, self.shared_limit,
                             self.kv_heads, self.qk_norm, self.sink, self.yarn_factor, self.yarn_original, self.yarn_fast,
                             self.yarn_slow, self.conv, self.inner, self.blocks, self.state, self.dt_rank, self.decay_mult,
                             self.d_heads, self.d_kv_heads, self.d_dim, self.d_vdim, self.left_scale, self.right_scale,
                             self.rot_interleaved, self.kv_from, self.out_gate, self.learned_sink, self.identity,
                             self.route_softmax, self.route_bias, self.group_best, self.route_renorm, self.expert_act,
                             self.shared_gate, self.ff_act, self.window, self.rot_half, self.expert_glu,
                             self.route_top_softmax)


@dataclass
class HybridSpec:
    width: int
    vocab: int
    eps: float
    layers: list[LayerSpec] = field(default_factory=list)
    architecture: str = "Pikavik"
    embed_scale: float = 1.0
    residual_mult: float = 1.0
    canon_taps: int = 0       # one-norm blocks: taps of the sublayers' input convolutions (0: none)

    @property
    def gated_residual(self) -> bool:
        return bool(DESIGNS[self.architecture].get("gated_residual"))

    @property
    def block(self) -> int:
        return DESIGNS[self.architecture]["block"]

    @property
    def norm_offset(self) -> float:
        return DESIGNS[self.architecture]["norm_offset"]

    @property
    def tied_head(self) -> bool:
        return bool(DESIGNS[self.architecture].get("tied_head"))

    @property
    def has_cache(self) -> bool:
        """Some layer keeps per-token rows in the paged cache (latent or grouped-query attention)."""
        return any(l.mixer in ("latent_attention", "parallel", "attention") for l in self.layers)

    has_latent = has_cache

    @property
    def has_state(self) -> bool:
        return self.canon_taps > 1 or any(l.mixer != "latent_attention" for l in self.layers)

    @classmethod
    def from_config(cls, cfg: dict, shapes: dict[str, list[int]] | None = None) -> "HybridSpec":
        """cfg: the parsed config.json.  shapes: tensor name -> shape of the checkpoint, for the sizes that only a
        tensor gives (the rank of the wkv decay bottleneck)."""
        arch = cfg.get("architecture", "Pikavik")
        if arch not in DESIGNS:
            raise ValueError(f"unknown layered design {arch!r}")
        design = DESIGNS[arch]
        layers = []
        for i, lc in enumerate(cfg["layers"]):
            kind, m = lc["type"], lc["mixer"]
            if kind not in design["mixers"]:
                raise ValueError(f"layer {i}: {arch} has no mixer type {kind!r}")
            if kind == "rglru":
                ls = LayerSpec(mixer=kind, heads=1, dim=1, inner=int(m["width"]), blocks=int(m["blocks"]), conv=int(m["conv"]),
                               decay_mult=RGLRU_DECAY_MULT)
            elif kind == "mamba1":
                ls = LayerSpec(mixer=kind, heads=1, dim=1, inner=int(m["inner"]), state=int(m["state"]),
                               dt_rank=int(m["dt_rank"]), conv=int(m["conv"]))
            elif kind == "parallel":
                a, d = m["left"], m["right"]
                rot = a.get("rot") or {}
                sc = rot.get("scaling") or {}
                ls = LayerSpec(mixer=kind, heads=int(a["heads"]), kv_heads=int(a["kv_heads"]), dim=int(a["dim"]),
                               vdim=int(a["vdim"]), attn_scale=float(a["scale"]), qk_norm=1, sink=1.0,
                               rot_dims=int(rot.get("dims", 0)), rot_base=float(rot.get("base", 10000.0)),
                               yarn_factor=float(sc.get("factor", 0.0)), yarn_original=float(sc.get("original", 0.0)),
                               yarn_fast=float(sc.get("fast", 0.0)), yarn_slow=float(sc.get("slow", 0.0)),
                               d_heads=int(d["heads"]), d_kv_heads=int(d["kv_heads"]), d_dim=int(d["dim"]),
                               d_vdim=int(d["vdim"]), conv=int(d["conv"]), left_scale=float(m["left_scale"]),
                               right_scale=float(m["right_scale"]))
            elif kind == "attention":
                rot = m.get("rot") or {}
                ls = LayerSpec(mixer=kind, heads=int(m["heads"]), kv_heads=int(m.get("kv_heads", m["heads"])), dim=int(m["dim"]),
                               vdim=int(m.get("vdim", m["dim"])), attn_scale=float(m["scale"]), conv=int(m.get("conv") or 1),
                               rot_dims=int(rot.get("dims", 0)), rot_base=float(rot.get("base", 10000.0)),
                               window=int((m.get("mask") or {}).get("size", 0)))
                for key, val in (design.get("attention") or {}).items():
                    setattr(ls, key, val)
            else:
                ls = LayerSpec(mixer=kind, heads=int(m["heads"]), dim=int(m["dim"]))
            if kind == "wkv":
                ls.vdim = ls.dim
                if shapes is not None:
                    ls.decay_rank = int(shapes[f"l{i}.mix.w1"][0])
                else:
                    ls.decay_rank = int(m.get("decay_rank", 0))
                if ls.decay_rank < 1:
                    raise ValueError(f"layer {i}: the decay bottleneck's rank is unknown")
            elif kind == "mlstm":
                ls.vdim, ls.gate_cap = int(m["vdim"]), float(m["gate_cap"])
            elif kind == "latent_attention":
                rot = m.get("rot") or {}
                ls.vdim, ls.rot_dim = int(m["vdim"]), int(m.get("rot_dim", 0))
                ls.window = int((m.get("mask") or {}).get("size", 0))
                ls.rot_dims, ls.rot_base = int(rot.get("dims", ls.rot_dim)), float(rot.get("base", 10000.0))
                ls.kv_rank, ls.q_rank, ls.attn_scale = int(m["kv_rank"]), int(m.get("q_rank", 0)), float(m["scale"])
                src = m.get("kv_from")
                ls.kv_from = -1 if src is None else int(src)
                for key, val in (design.get("latent") or {}).items():
                    setattr(ls, key, val)
            mlp = lc.get("mlp")
            if mlp:
                mk = mlp.get("kind", design["mlp"][0])
                if mk not in design["mlp"]:
                    raise ValueError(f"layer {i}: unknown feed-forward kind {mk!r}")
                if mk == "dense":
                    ls.mlp, ls.ff = design.get("dense", "dense"), int(mlp["ff"])
                    for key, val in (design.get("ffn") or {}).items():
                        setattr(ls, key, val)
                else:
                    r, ex, sh = mlp["router"], mlp["expert"], mlp.get("shared")
                    g = r.get("groups") or {}
                    ls.mlp, ls.experts, ls.top = "moe", int(r["experts"]), int(r["top"])
                    ls.groups, ls.keep = int(g.get("count", 1)), int(g.get("keep", g.get("count", 1)))
                    ls.route_scale, ls.ff, ls.limit = float(r.get("scale", 1.0)), int(ex["ff"]), float(ex.get("limit", 0.0))
                    ls.identity = int(r.get("identity", 0))
                    if sh:
                        ls.shared_ff, ls.shared_limit = int(sh["ff"]), float(sh.get("limit", 0.0))
                    for key, val in (design.get("moe") or {}).items():
                        setattr(ls, key, val)
            layers.append(ls)
        return cls(width=int(cfg["width"]), vocab=int(cfg["vocab"]), eps=float(cfg["norm"]["eps"]), layers=layers,
                   architecture=arch, embed_scale=float((cfg.get("embedding") or {}).get("scale", 1.0)),
                   residual_mult=float(cfg.get("residual_mult", 1.0)),
                   canon_taps=int((cfg.get("canon") or {}).get("taps", 0)) if design["block"] == L.BLOCK_PARALLEL_ONE_NORM else 0)

    @classmethod
    def from_dir(cls, path: str) -> "HybridSpec":
        with open(os.path.join(path, "config.json")) as f:
            cfg = json.load(f)
        return cls.from_config(cfg, safetensors_shapes(os.path.join(path, "model.safetensors")))


def safetensors_header(path: str) -> tuple[dict, int]:
    """(name -> {dtype, shape, data_offsets}, offset of the data section): 8-byte little-endian length, then JSON."""
    with open(path, "rb") as f:
        n = struct.unpack("<Q", f.read(8))[0]
        header = json.loads(f.read(n))
    header.pop("__metadata__", None)
    return header, 8 + n


def safetensors_shapes(path: str) -> dict[str, list[int]]:
    return {k: v["shape"] for k, v in safetensors_header(path)[0].items()}


_ST_DTYPES = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32, "I64": torch.int64,
              "F64": torch.float64}


def read_safetensors(path: str) -> dict[str, torch.Tensor]:
    header, base = safetensors_header(path)
    raw = np.fromfile(path, dtype=np.uint8)
    out = {}
    for name, info in header.items():
        lo, hi = info["data_offsets"]
        buf = torch.from_numpy(raw[base + lo:base + hi].copy())
        out[name] = buf.view(_ST_DTYPES[info["dtype"]]).reshape(info["shape"])
    return out


def pack_hybrid_weights(spec: HybridSpec, raw: dict[str, torch.Tensor], dtype: torch.dtype, device) -> dict:
    """Checkpoint tensors -> the packed per-layer tensors of ssdk_hyb_bind (include/ssdk.h, SSDK_HT_*): projections that
    read the same input are stacked by output rows, per-expert matrices are stacked by expert, W_uk is transposed per
    head for the query absorption."""
    def t(name):
        return raw[name].to(torch.float32)

    def dev(x):
        return x.to(dtype).contiguous().to(device)

    w = {"EMBED": dev(t("embed")), "FINAL_NORM": dev(t("final.norm")), "layers": []}
    w["HEAD"] = w["EMBED"] if spec.tied_head else dev(t("head"))   # a tied head reads the table itself (without its scale)
    two_norms = spec.block == L.BLOCK_PARALLEL_TWO_NORMS
    one_norm = spec.block == L.BLOCK_PARALLEL_ONE_NORM
    scales = not two_norms and not one_norm
    for i, ls in enumerate(spec.layers):
        p, mx = f"l{i}.", f"l{i}.mix."
        lw = {"NORM": dev(t(p + "norm1"))}
        if one_norm:   # per sublayer: taps of its input convolution, rows and bias of its residual gate
            subs = ("1", "2") if ls.mlp else ("1",)
            if spec.canon_taps > 0:
                lw["CANON_W"] = dev(torch.stack([t(p + "canon" + k) for k in subs]))
            if spec.gated_residual:
                lw["RES_GATE"] = dev(torch.cat([t(p + "rg" + k) for k in subs]))
                lw["RES_GATE_B"] = dev(torch.cat([t(p + "rg" + k + ".b") for k in subs]))
        if ls.mixer in ("wkv", "mlstm", "latent_attention"):
            lw["MIX_OUT"] = dev(t(mx + "o"))
            if scales:
                lw["LS_MIX"] = dev(t(p + "ls1"))
        if two_norms and ls.mlp:
            lw["NORM2"] = dev(t(p + "norm2"))
        if ls.mixer == "rglru":
            lw["RGLRU_IN"] = dev(torch.cat([t(mx + "y"), t(mx + "x")]))
            lw["RGLRU_IN_B"] = dev(torch.cat([t(mx + "y.b"), t(mx + "x.b")]))
            lw["CONV_W"], lw["CONV_B"] = dev(t(mx + "conv")), dev(t(mx + "conv.b"))
            lw["RGLRU_GATE"] = dev(torch.cat([t(mx + "ra"), t(mx + "ri")], dim=1))      # [blocks, 2 bs, bs]
            lw["RGLRU_GATE_B"] = dev(torch.cat([t(mx + "ra.b"), t(mx + "ri.b")], dim=1))  # [blocks, 2 bs]
            lw["RGLRU_LAM"], lw["MIX_OUT"] = dev(t(mx + "lam")), dev(t(mx + "o"))
        elif ls.mixer == "mamba1":
            lw["SEL_IN"], lw["CONV_W"], lw["CONV_B"] = dev(t(mx + "in")), dev(t(mx + "conv")), dev(t(mx + "conv.b"))
            lw["SEL_X"], lw["SEL_DT"], lw["SEL_DT_B"] = dev(t(mx + "x")), dev(t(mx + "dt")), dev(t(mx + "dt.b"))
            lw["SEL_ALOG"], lw["SEL_D"], lw["MIX_OUT"] = dev(t(mx + "A_log")), dev(t(mx + "D")), dev(t(mx + "o"))
        elif ls.mixer == "parallel":
            a, d = mx + "left.", mx + "right."
            lw["PAIR_IN"] = dev(torch.cat([t(a + "q"), t(a + "k"), t(a + "v"), t(a + "g"),
                                           t(d + "q"), t(d + "k"), t(d + "v"), t(d + "g"), t(d + "b"), t(d + "a")]))
            lw["ATTN_OUT"], lw["MIX_OUT"] = dev(t(a + "o")), dev(t(d + "o"))
            lw["CONV_W"] = dev(torch.cat([t(d + "q.conv"), t(d + "k.conv"), t(d + "v.conv")]))
            lw["DELTA_ALOG"], lw["DELTA_DT_B"] = dev(t(d + "A_log")), dev(t(d + "dt_bias"))
            lw["MIX_NORM"] = dev(t(d + "norm").repeat(ls.d_heads))  # one weight per value channel, the same for every head
        elif ls.mixer == "attention":
            lw["ATTN_IN"] = dev(torch.cat([t(mx + "q"), t(mx + "k"), t(mx + "v")]))
            if mx + "q.b" in raw:
                lw["ATTN_IN_B"] = dev(torch.cat([t(mx + "q.b"), t(mx + "k.b"), t(mx + "v.b")]))
            if mx + "q.conv" in raw:
                lw["CONV_W"] = dev(torch.cat([t(mx + "q.conv"), t(mx + "k.conv"), t(mx + "v.conv")]))
            else:   # no convolution: one tap of weight 1
                lw["CONV_W"] = dev(torch.ones(lw["ATTN_IN"].shape[0], 1))
            if ls.learned_sink:
                lw["ATTN_SINK"] = dev(t(mx + "sink"))
            lw["MIX_OUT"] = dev(t(mx + "o"))
        elif ls.mixer == "wkv":
            lw["WKV_MU"] = dev(torch.stack([t(mx + "mu." + s) for s in "rkvgw"]))
            for s in "rkvg":
                lw["WKV_" + s.upper()] = dev(t(mx + s))
            lw["WKV_W1"], lw["WKV_W2"], lw["WKV_W0"] = dev(t(mx + "w1")), dev(t(mx + "w2")), dev(t(mx + "w0"))
            lw["WKV_U"], lw["MIX_NORM"] = dev(t(mx + "u")), dev(t(mx + "norm"))
        elif ls.mixer == "mlstm":
            lw["MLSTM_IN"] = dev(torch.cat([t(mx + s) for s in ("q", "k", "v", "g", "i", "f")]))
            lw["MLSTM_IB"], lw["MLSTM_FB"], lw["MIX_NORM"] = dev(t(mx + "i.b")), dev(t(mx + "f.b")), dev(t(mx + "norm"))
        else:
            if ls.q_rank > 0:
                lw["LAT_DOWN"] = dev(torch.cat([t(mx + "dq"), t(mx + "dkv")]))
                lw["LAT_QNORM"], lw["LAT_UQ"] = dev(t(mx + "dq.norm")), dev(t(mx + "uq"))
            else:   # full-rank queries: everything that reads the mixer's input is one matrix
                rows = [t(mx + "q")] + ([t(mx + "dkv")] if ls.kv_from < 0 else []) + ([t(mx + "g")] if ls.out_gate else [])
                lw["LAT_IN"] = dev(torch.cat(rows))
            if ls.kv_from < 0:
                lw["LAT_KVNORM"] = dev(t(mx + "dkv.norm"))
            if ls.learned_sink:
                lw["LAT_SINK"] = dev(t(mx + "sink"))
            lw["LAT_UV"] = dev(t(mx + "uv"))
            lw["LAT_UKT"] = dev(t(mx + "uk").view(ls.heads, ls.dim, ls.kv_rank).transpose(1, 2))
        if ls.mlp == "ffn":
            q = p + "mlp."
            lw["FFN_IN"], lw["FFN_OUT"] = dev(t(q + "up")), dev(t(q + "down"))
            if q + "up.b" in raw:
                lw["FFN_IN_B"] = dev(t(q + "up.b"))
            if q + "down.b" in raw:
                lw["FFN_OUT_B"] = dev(t(q + "down.b"))
            if ls.ff_act == L.ACT_POLYNORM:
                lw["FFN_ACT"] = dev(t(q + "act"))
        if ls.mlp == "dense":
            q = p + "mlp."
            lw["NORM2"] = dev(t(p + "norm2"))
            lw["GLU_IN"], lw["GLU_OUT"] = dev(torch.cat([t(q + "gate"), t(q + "up")])), dev(t(q + "down"))
        if ls.mlp == "moe":
            q = p + "mlp."
            lw["ROUTER"] = dev(t(q + "router"))
            if scales:
                lw["LS_MLP"] = dev(t(p + "ls2"))
            if ls.route_bias:
                lw["ROUTER_BIAS"] = dev(t(q + "correction"))
            mats = ("gate", "up") if ls.expert_glu else ("up",)   # an expert's input matrices, stacked by rows
            lw["EXPERT_IN"] = dev(torch.stack([torch.cat([t(f"{q}e{e}.{k}") for k in mats]) for e in range(ls.experts)]))
            lw["EXPERT_OUT"] = dev(torch.stack([t(f"{q}e{e}.down") for e in range(ls.experts)]))
            if ls.shared_ff:
                lw["SHARED_IN"] = dev(torch.cat([t(q + "shared." + k) for k in mats] +
                                                ([t(q + "shared.sg").reshape(1, -1)] if ls.shared_gate else [])))
                lw["SHARED_OUT"] = dev(t(q + "shared.down"))
        w["layers"].append(lw)
    return w


def load_hybrid_weights(path: str, spec: HybridSpec, dtype: torch.dtype, device) -> dict:
    return pack_hybrid_weights(spec, read_safetensors(os.path.join(path, "model.safetensors")), dtype, device)


def random_hybrid_weights(spec: HybridSpec, dtype: torch.dtype, device, seed: int = 0) -> dict:
    """Random weights in the packed layout, generated on the device (benchmarks: there are no checkpoints to load).
    Scales keep activations O(1): linear layers N(0, 1/in), norm offsets small, decays spread over (0.2, 0.9)."""
    g = torch.Generator(device=device).manual_seed(seed)
    W = spec.width

    def lin(*shape):
        return (torch.randn(*shape, generator=g, device=device) / shape[-1] ** 0.5).to(dtype)

    def vec(n, mean=0.0, std=0.1):
        return (mean + std * torch.randn(n, generator=g, device=device)).to(dtype)

    w = {"EMBED": torch.randn(spec.vocab, W, generator=g, device=device).to(dtype), "HEAD": lin(spec.vocab, W),
         "FINAL_NORM": vec(W), "layers": []}
    def uni(lo, hi, *shape):
        return (lo + (hi - lo) * torch.rand(*shape, generator=g, device=device)).to(dtype)

    if spec.block == L.BLOCK_SERIAL_POSTNORM:
        w["FINAL_NORM"] = vec(W, 1.0)
    if spec.block == L.BLOCK_PARALLEL_ONE_NORM:
        w["FINAL_NORM"] = vec(W, 1.0)
    if spec.block == L.BLOCK_PARALLEL_TWO_NORMS:
        w["FINAL_NORM"] = vec(W, 1.0)
        if spec.tied_head:   # the table is read as it is by the head: unit-size logits, the embedding's scale restores O(1) rows
            w["EMBED"] = (torch.randn(spec.vocab, W, generator=g, device=device) / W ** 0.5).to(dtype)
            w["HEAD"] = w["EMBED"]
    for ls in spec.layers:
        H, D, V = ls.heads, ls.dim, ls.vdim
        if spec.block == L.BLOCK_PARALLEL_ONE_NORM:
            subs = 2 if ls.mlp else 1
            lw = {"NORM": vec(W, 1.0), "MIX_OUT": lin(W, H * V)}
            if spec.canon_taps > 0:
                lw["CANON_W"] = (torch.randn(subs, W, spec.canon_taps, generator=g, device=device) * 0.3).to(dtype)
            if spec.gated_residual:
                lw["RES_GATE"], lw["RES_GATE_B"] = lin(subs * W, W), vec(subs * W, 0.5, 0.5)
            if ls.mixer == "attention":
                n_in = H * D + ls.kv_heads * (D + V)
                lw["ATTN_IN"], lw["ATTN_IN_B"] = lin(n_in, W), vec(n_in, 0.0, 0.3)
                lw["CONV_W"] = (torch.randn(n_in, ls.conv, generator=g, device=device) * 0.5).to(dtype)
                if ls.learned_sink:
                    lw["ATTN_SINK"] = vec(H, 0.0, 1.0)
            elif ls.mixer == "latent_attention" and not ls.q_rank and ls.kv_from < 0:
                KR, R = ls.kv_rank, ls.rot_dim
                lw["LAT_IN"], lw["LAT_KVNORM"] = lin(H * (D + R) + KR + R + (H * V if ls.out_gate else 0), W), vec(KR, 1.0)
                lw["LAT_UV"], lw["LAT_UKT"] = lin(H * V, KR), (lin(H, KR, D) * (D / KR) ** 0.5).contiguous()
                if ls.learned_sink:
                    lw["LAT_SINK"] = vec(H, 0.0, 1.0)
            else:
                raise ValueError("random weights of one-norm blocks are made for attention and latent attention with full-rank queries")
            mats = 2 if ls.expert_glu else 1
            if ls.mlp == "ffn":
                lw["FFN_IN"], lw["FFN_OUT"] = lin(ls.ff, W), lin(W, ls.ff)
                if ls.ff_act == L.ACT_POLYNORM:
                    lw["FFN_ACT"] = torch.tensor([0.6, 0.4, -0.3, 0.1], device=device).to(dtype)
            elif ls.mlp == "moe":
                lw["ROUTER"] = lin(ls.experts + ls.identity, W)
                lw["EXPERT_IN"], lw["EXPERT_OUT"] = lin(ls.experts, mats * ls.ff, W), lin(ls.experts, W, ls.ff)
                if ls.shared_ff:
                    lw["SHARED_IN"] = lin(mats * ls.shared_ff + (1 if ls.shared_gate else 0), W)
                    lw["SHARED_OUT"] = lin(W, ls.shared_ff)
            w["layers"].append(lw)
            continue
        if spec.block == L.BLOCK_PARALLEL_TWO_NORMS:
            if ls.mixer != "latent_attention" or ls.q_rank:
                raise ValueError("random weights of two-norm blocks are made for latent attention with full-rank queries")
            R, KR, own = ls.rot_dim, ls.kv_rank, ls.kv_from < 0
            lw = {"NORM": vec(W, 1.0), "MIX_OUT": lin(W, H * V), "LAT_UV": lin(H * V, KR),
                  "LAT_IN": lin(H * (D + R) + (KR + R if own else 0) + (H * V if ls.out_gate else 0), W),
                  "LAT_UKT": (lin(H, KR, D) * (D / KR) ** 0.5).contiguous()}
            if own:
                lw["LAT_KVNORM"] = vec(KR, 1.0)
            if ls.learned_sink:
                lw["LAT_SINK"] = vec(H, 0.0, 1.0)
            if ls.mlp:
                lw["NORM2"] = vec(W, 1.0)
            if ls.mlp == "ffn":
                lw["FFN_IN"], lw["FFN_IN_B"], lw["FFN_OUT"], lw["FFN_OUT_B"] = lin(ls.ff, W), vec(ls.ff), lin(W, ls.ff), vec(W)
            elif ls.mlp == "moe":
                lw["ROUTER"] = lin(ls.experts + ls.identity, W)
                if ls.route_bias:
                    lw["ROUTER_BIAS"] = vec(ls.experts + ls.identity, 0.0, 0.02)
                lw["EXPERT_IN"], lw["EXPERT_OUT"] = lin(ls.experts, 2 * ls.ff, W), lin(ls.experts, W, ls.ff)
                if ls.shared_ff:
                    lw["SHARED_IN"] = lin(2 * ls.shared_ff + (1 if ls.shared_gate else 0), W)
                    lw["SHARED_OUT"] = lin(W, ls.shared_ff)
            w["layers"].append(lw)
            continue
        if ls.mixer in ("rglru", "mamba1", "parallel"):
            lw = {"NORM": vec(W, 1.0)}
            taps = ls.conv
            if ls.mixer == "rglru":
                R, bs = ls.inner, ls.inner // ls.blocks
                lw["RGLRU_IN"], lw["RGLRU_IN_B"] = lin(2 * R, W), vec(2 * R, 0.0, 0.3)
                lw["CONV_W"], lw["CONV_B"] = (torch.randn(R, taps, generator=g, device=device) * 0.5).to(dtype), vec(R, 0.0, 0.2)
                lw["RGLRU_GATE"], lw["RGLRU_GATE_B"] = lin(ls.blocks, 2 * bs, bs), vec(ls.blocks * 2 * bs, 0.0, 0.5).view(ls.blocks, 2 * bs)
                lw["RGLRU_LAM"], lw["MIX_OUT"] = uni(-4.0, 0.5, R), lin(W, R)
            elif ls.mixer == "mamba1":
                I, N, Rk = ls.inner, ls.state, ls.dt_rank
                lw["SEL_IN"], lw["CONV_B"] = lin(2 * I, W), vec(I, 0.0, 0.2)
                lw["CONV_W"] = (torch.randn(I, taps, generator=g, device=device) * 0.5).to(dtype)
                lw["SEL_X"], lw["SEL_DT"], lw["SEL_DT_B"] = lin(Rk + 2 * N, I), lin(I, Rk), uni(-3.0, -0.5, I)
                lw["SEL_ALOG"], lw["SEL_D"], lw["MIX_OUT"] = torch.log(uni(0.3, 4.0, I, N).float()).to(dtype), vec(I, 1.0, 0.2), lin(W, I)
            else:
                G, Hd, Gd, Dd, Vd = ls.kv_heads, ls.d_heads, ls.d_kv_heads, ls.d_dim, ls.d_vdim
                Cd = 2 * Gd * Dd + Hd * Vd
                lw["PAIR_IN"] = lin(H * D + G * D + G * V + H * V + Cd + Hd * Vd + 2 * Hd, W)
                lw["ATTN_OUT"], lw["MIX_OUT"] = lin(W, H * V), lin(W, Hd * Vd)
                lw["CONV_W"] = (torch.randn(Cd, taps, generator=g, device=device) * 0.6).to(dtype)
                lw["DELTA_ALOG"], lw["DELTA_DT_B"], lw["MIX_NORM"] = uni(-2.0, 0.5, Hd), uni(-2.0, 1.0, Hd), vec(Hd * Vd, 1.0)
            if ls.mlp == "dense":
                lw["NORM2"], lw["GLU_IN"], lw["GLU_OUT"] = vec(W, 1.0), lin(2 * ls.ff, W), lin(W, ls.ff)
            w["layers"].append(lw)
            continue
        lw = {"NORM": vec(W), "LS_MIX": vec(W, 1.0), "MIX_OUT": lin(W, H * V)}
        if ls.mixer == "wkv":
            lw["WKV_MU"] = torch.rand(5, W, generator=g, device=device).to(dtype)
            for s_ in "RKVG":
                lw["WKV_" + s_] = lin(H * D, W)
            lw["WKV_W1"], lw["WKV_W2"] = lin(ls.decay_rank, W), lin(H * D, ls.decay_rank)
            lw["WKV_W0"] = (torch.rand(H * D, generator=g, device=device) * 3.0 - 2.5).to(dtype)
            lw["WKV_U"], lw["MIX_NORM"] = vec(H * D, 0.0, 0.5).view(H, D), vec(H * D, 1.0)
        elif ls.mixer == "mlstm":
            lw["MLSTM_IN"] = lin(2 * H * D + 2 * H * V + 2 * H, W)
            lw["MLSTM_IB"], lw["MLSTM_FB"], lw["MIX_NORM"] = vec(H, 0.0, 1.0), vec(H, 2.5, 0.5), vec(H * V, 1.0)
        else:
            lw["LAT_DOWN"] = lin(ls.q_rank + ls.kv_rank + ls.rot_dim, W)
            lw["LAT_QNORM"], lw["LAT_KVNORM"] = vec(ls.q_rank, 1.0), vec(ls.kv_rank, 1.0)
            lw["LAT_UQ"], lw["LAT_UV"] = lin(H * (D + ls.rot_dim), ls.q_rank), lin(H * V, ls.kv_rank)
            lw["LAT_UKT"], lw["LAT_SINK"] = (lin(H, ls.kv_rank, D) * (D / ls.kv_rank) ** 0.5).contiguous(), vec(H, 0.0, 1.0)
        if ls.mlp == "moe":
            lw["LS_MLP"], lw["ROUTER"] = vec(W, 1.0), lin(ls.experts, W)
            lw["EXPERT_IN"], lw["EXPERT_OUT"] = lin(ls.experts, 2 * ls.ff, W), lin(ls.experts, W, ls.ff)
            if ls.shared_ff:
                lw["SHARED_IN"], lw["SHARED_OUT"] = lin(2 * ls.shared_ff + 1, W), lin(W, ls.shared_ff)
        w["layers"].append(lw)
    return w


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


class HybridRunner:
    """Device state of one hybrid model + the one forward call every path uses (generation, trace replay, tests).

    max_tokens      rows one library call carries (longer batches are cut into several calls by `forward`)
    num_blocks      pages of the latent cache (block_size tokens each), shared by all latent-attention layers' pools
    n_slots         recurrent-state slots (one per live sequence)"""

    def __init__(self, spec: HybridSpec, weights: dict, *, dtype: str = "bfloat16", max_tokens: int = 2048, max_seqs: int = 8,
                 block_size: int = 64, num_blocks: int = 64, n_slots: int = 8, max_model_len: int = 4096,
                 max_logit_rows: int | None = None, device: str | torch.device = "cuda:0"):
        if not torch.cuda.is_available():
            raise RuntimeError("HybridRunner needs a CUDA device: libssdk has no CPU path")
        self.lib = L.load()
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        self.spec, self.block_size, self.num_blocks, self.n_slots = spec, block_size, num_blocks, n_slots
        self.max_tokens, self.max_seqs = max_tokens, max_seqs
        self.max_blocks = -(-max_model_len // block_size)
        self.max_model_len = max_model_len
        self.dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype]
        # logits of one call live on the device as fp32 + bf16: all rows of a call unless that exceeds ~6 GB
        self.max_logit_rows = max_logit_rows or max(1, min(max_tokens, (1 << 30) // spec.vocab))
        cfg = L.HybCfg(spec.width, spec.vocab, len(spec.layers), L.DT_BF16 if self.dtype == torch.bfloat16 else L.DT_F32,
                       spec.eps, max_tokens, max_seqs, self.max_logit_rows, block_size, self.max_blocks, spec.block, spec.norm_offset,
                       spec.embed_scale, spec.residual_mult, spec.canon_taps, int(spec.gated_residual))
        layer_cfgs = (L.HybLayerCfg * len(spec.layers))(*[l.cfg() for l in spec.layers])
        h = C.c_void_p()
        L.check(self.lib.ssdk_hyb_create(C.byref(cfg), layer_cfgs, C.byref(h)), "ssdk_hyb_create")
        self.h = h
        self.weights = weights
        self._bind_weights(weights)
        nb_c = max(0, self.lib.ssdk_hyb_cache_bytes(self.h, num_blocks))
        nb_s = max(0, self.lib.ssdk_hyb_state_bytes(self.h, n_slots))
        nb_w = self.lib.ssdk_hyb_workspace_bytes(self.h)
        self.cache = torch.zeros(max(nb_c, 16), dtype=torch.uint8, device=self.device)
        self.state = torch.zeros(max(nb_s, 16), dtype=torch.uint8, device=self.device)
        self.workspace = torch.zeros(nb_w + 512, dtype=torch.uint8, device=self.device)
        off = (-self.workspace.data_ptr()) % 256
        L.check(self.lib.ssdk_hyb_bind_pools(self.h, self.cache.data_ptr(), num_blocks, self.state.data_ptr(), n_slots,
                                             self.workspace.data_ptr() + off, nb_w), "ssdk_hyb_bind_pools")
        self.step_id = 0

    def _bind_weights(self, w: dict) -> None:
        def bind(layer, name, t):
            if t.dtype != self.dtype or not t.is_cuda or not t.is_contiguous():
                raise ValueError(f"{name}: weights must be contiguous {self.dtype} CUDA tensors")
            rows, cols = (t.shape[0], t.numel() // t.shape[0]) if t.dim() >= 2 else (t.shape[0], 1)
            L.check(self.lib.ssdk_hyb_bind(self.h, layer, L.HT[name], t.data_ptr(), rows, cols), f"bind {name} layer {layer}")

        for name in ("EMBED", "HEAD", "FINAL_NORM"):
            bind(-1, name, w[name])
        for i, lw in enumerate(w["layers"]):
            for name, t in lw.items():
                bind(i, name, t)

    # ------------------------------------------------------------------ the step function
    def forward(self, entries, *, want_logits: bool = True, temps=None, seed: int = 0, residual: bool = False):
        """entries: list of (tokens, pos0, slot, block_table, want) — `tokens` continue a sequence at position pos0 whose
        state lives in `slot` and whose latent rows live in the pages `block_table`; `want` lists the places among
        `tokens` whose logits (and, with `temps`, sampled tokens) are asked for.  Returns (logits [n_want, vocab] float32
        or None, tokens list or None[, residual [layers, rows, width]]), rows in the order of the entries."""
        total = sum(len(e[0]) for e in entries)
        if total > self.max_tokens or len(entries) > self.max_seqs or sum(len(e[4]) for e in entries) > self.max_logit_rows:
            return self._forward_split(entries, want_logits, temps, seed, residual)
        ids, cu, pos0, slots, want_rows = [], [0], [], [], []
        tables = np.full((len(entries), self.max_blocks), -1, dtype=np.int32)
        for s, (toks, p0, slot, table, want) in enumerate(entries):
            if p0 + len(toks) > self.max_model_len:
                raise ValueError("sequence longer than max_model_len")
            want_rows += [cu[-1] + int(k) for k in want]
            ids += list(toks)
            cu.append(cu[-1] + len(toks))
            pos0.append(p0)
            slots.append(slot)
            tables[s, :len(table)] = table
        n_want = len(want_rows)
        logits = np.empty((n_want, self.spec.vocab), dtype=np.float32) if (want_logits and n_want) else None
        toks_out = np.zeros(max(n_want, 1), dtype=np.int64)
        temps_a = np.ascontiguousarray(temps, dtype=np.float32) if temps is not None else None
        if temps_a is not None and len(temps_a) != n_want:
            raise ValueError("one temperature per wanted row")
        res = np.empty((len(self.spec.layers), total, self.spec.width), dtype=np.float32) if residual else None
        ids_a, cu_a, pos_a, slot_a, want_a = _i32(ids), _i32(cu), _i32(pos0), _i32(slots), _i32(want_rows or [0])
        L.check(self.lib.ssdk_hyb_forward(
            self.h, len(entries), total, ids_a.ctypes.data_as(L.c_i32p), cu_a.ctypes.data_as(L.c_i32p),
            pos_a.ctypes.data_as(L.c_i32p), slot_a.ctypes.data_as(L.c_i32p), tables.ctypes.data_as(L.c_i32p), n_want,
            want_a.ctypes.data_as(L.c_i32p), logits.ctypes.data_as(L.c_f32p) if logits is not None else None,
            temps_a.ctypes.data_as(L.c_f32p) if temps_a is not None else None, seed, self.step_id,
            toks_out.ctypes.data_as(L.c_i64p), res.ctypes.data_as(L.c_f32p) if res is not None else None,
            torch.cuda.current_stream().cuda_stream), "ssdk_hyb_forward")
        self.step_id += 1
        out = (logits, toks_out[:n_want].tolist() if temps_a is not None else None)
        return out + (res,) if residual else out

    def _forward_split(self, entries, want_logits, temps, seed, residual):
        """A batch over the per-call limits runs as several calls: sequences are taken in order and a long portion is
        cut, which the carried state and cache make equivalent to one call."""
        if residual:
            raise ValueError("the residual tap covers single calls only")
        calls, cur, room, lroom = [], [], self.max_tokens, self.max_logit_rows
        first = np.cumsum([0] + [len(e[4]) for e in entries])  # first output row of every entry
        for i, (toks, p0, slot, table, want) in enumerate(entries):
            if list(want) != sorted(want):
                raise ValueError("wanted places must ascend")
            lo = 0
            while lo < len(toks):
                if room == 0 or lroom == 0 or len(cur) == self.max_seqs:
                    calls.append(cur)
                    cur, room, lroom = [], self.max_tokens, self.max_logit_rows
                n = min(room, len(toks) - lo)
                js = [j for j, k in enumerate(want) if lo <= k < lo + n]
                if len(js) > lroom:  # cut the piece after the last wanted place that still fits this call
                    js = js[:lroom]
                    n = want[js[-1]] - lo + 1
                cur.append(([first[i] + j for j in js], (toks[lo:lo + n], p0 + lo, slot, table, [want[j] - lo for j in js])))
                lo += n
                room -= n
                lroom -= len(js)
        calls.append(cur)
        n_out = int(first[-1])
        logits = np.empty((n_out, self.spec.vocab), dtype=np.float32) if (want_logits and n_out) else None
        tokens = [0] * n_out
        for call in calls:
            rows = [r for rs, _ in call for r in rs]
            lg, tk = self.forward([e for _, e in call], want_logits=want_logits,
                                  temps=[temps[r] for r in rows] if temps is not None else None, seed=seed)
            for k, r in enumerate(rows):
                if lg is not None:
                    logits[r] = lg[k]
                if tk is not None:
                    tokens[r] = tk[k]
        return logits, (tokens if temps is not None else None)

    @property
    def launch_count(self) -> int:
        return int(self.lib.ssdk_hyb_launch_count(self.h))

    def close(self) -> None:
        if getattr(self, "h", None):
            self.lib.ssdk_hyb_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
