"""Throughput of the hybrid families (bench.py --arch pikavik | kefurax | lisenex | kokatar).

--arch pikavik: a Pikavik stack beside the closest dense model of the framework (below).
--arch kefurax: a Kefurax stack (attention + delta-rule pair with a dense feed-forward, selective scan, rglru, ...) beside
the closest existing model of the framework, a Pikavik stack of the same width, depth and active feed-forward size.
--arch lisenex: a Lisenex stack (latent attention with full-rank queries in every layer, every second layer reading the
layer before's latent pool; a dense squared-relu feed-forward first, then softmax-routed experts with identity experts and a
shared expert) beside the same Pikavik stack.
--arch kokatar: a Kokatar stack (one-norm blocks with input convolutions and residual gates; windowed grouped-query
attention with a learned sink and windowed latent attention without positions; a dense PolyNorm feed-forward or
squared-relu experts with a gated shared expert) beside the closest existing model of the framework, a Lisenex stack of the
same width, depth, vocabulary and feed-forward / expert sizes.

For every size: a Pikavik stack (mLSTM, wkv, wkv, latent attention, ... each with a grouped mixture of experts and a
shared expert) with random weights, and a Llama stack of the same width, depth and ACTIVE feed-forward size
(top * ff + shared ff) through PairRunner.  Prefill = one prompt, tokens / s over the whole prompt; decode = `batch`
sequences at that context, one token each per step.  CUDA events on the launching stream after warm-up; every timed
iteration reads weights larger than... see `l2_note` in the output (a stack of this size streams more than the 126 MB
L2 per pass, so no explicit flush is needed)."""
from __future__ import annotations

import time

import numpy as np
import torch

SIZES = {
    # name: (width, layers, heads x dim of the recurrent mixers, latent heads/dim/rot/kv_rank/q_rank, experts, top, ff, shared)
    "s": dict(width=1024, layers=8, rh=16, rd=64, lh=16, ld=64, rot=64, kvr=256, qr=384, experts=16, top=2, groups=4, keep=2, ff=512, sff=1024, vocab=32768),
    "m": dict(width=2048, layers=8, rh=32, rd=64, lh=16, ld=128, rot=64, kvr=512, qr=768, experts=32, top=4, groups=8, keep=4, ff=1024, sff=2048, vocab=32768),
}


def pikavik_spec(z):
    from .hybrid import HybridSpec, LayerSpec
    mlp = dict(mlp="moe", experts=z["experts"], top=z["top"], groups=z["groups"], keep=z["keep"], route_scale=2.0,
               ff=z["ff"], limit=7.0, shared_ff=z["sff"], shared_limit=7.0)
    layers = []
    for i in range(z["layers"]):
        kind = ("mlstm", "wkv", "wkv", "latent_attention")[i % 4]
        if kind == "wkv":
            layers.append(LayerSpec("wkv", z["rh"], z["rd"], z["rd"], decay_rank=64, **mlp))
        elif kind == "mlstm":
            layers.append(LayerSpec("mlstm", z["rh"], z["rd"], z["rd"], gate_cap=15.0, **mlp))
        else:
            layers.append(LayerSpec("latent_attention", z["lh"], z["ld"], z["ld"], rot_dim=z["rot"], rot_dims=z["rot"],
                                    kv_rank=z["kvr"], q_rank=z["qr"], attn_scale=(z["ld"] + z["rot"]) ** -0.5, **mlp))
    return HybridSpec(z["width"], z["vocab"], 1e-6, layers)


def kefurax_spec(z):
    """Layers that resemble a real model's: 128-wide heads, four query heads per key/value head, a delta rule with
    128 x 128 heads, a selective scan of twice the width with 16 states, a recurrence as wide as the model."""
    from .hybrid import RGLRU_DECAY_MULT, HybridSpec, LayerSpec
    W = z["width"]
    heads, ff = W // 128, z["top"] * z["ff"] + z["sff"]
    layers = []
    for i in range(z["layers"]):
        kind = ("parallel", "mamba1", "rglru", "parallel")[i % 4]
        if kind == "parallel":
            layers.append(LayerSpec("parallel", heads, 128, 128, rot_dims=64, rot_base=10000.0, attn_scale=128 ** -0.5,
                                    kv_heads=max(1, heads // 4), qk_norm=1, sink=1.0, yarn_factor=4.0, yarn_original=4096.0,
                                    yarn_fast=16.0, yarn_slow=2.0, conv=4, d_heads=heads, d_kv_heads=max(1, heads // 2), d_dim=128,
                                    d_vdim=128, left_scale=1.0, right_scale=1.0, mlp="dense", ff=ff))
        elif kind == "mamba1":
            layers.append(LayerSpec("mamba1", 1, 1, inner=2 * W, state=16, dt_rank=W // 16, conv=4, mlp="dense", ff=ff))
        else:
            layers.append(LayerSpec("rglru", 1, 1, inner=W, blocks=heads, conv=4, decay_mult=RGLRU_DECAY_MULT, mlp="dense", ff=ff))
    return HybridSpec(W, z["vocab"], 1e-6, layers, architecture="Kefurax", embed_scale=1.0, residual_mult=0.7)


def lisenex_spec(z):
    """Layers that resemble a real model's: 16 heads of 64 / 128 unrotated + 64 rotated query dimensions over a latent of
    256 / 512, values as wide as the keys; layer 2k+1 reads layer 2k's latent pool; the first feed-forward is dense (as wide
    as a token's active experts), the others route over `experts` outputs, two of them identity experts."""
    from . import lib as L
    from .hybrid import DESIGNS, HybridSpec, LayerSpec
    d = DESIGNS["Lisenex"]
    layers = []
    for i in range(z["layers"]):
        ls = LayerSpec("latent_attention", z["lh"], z["ld"], z["ld"], rot_dim=z["rot"], rot_dims=z["rot"], rot_base=10000.0,
                       kv_rank=z["kvr"], q_rank=0, attn_scale=(z["ld"] + z["rot"]) ** -0.5, kv_from=(i - 1 if i % 2 else -1),
                       **d["latent"])
        if i == 0:
            ls.mlp, ls.ff, ls.ff_act = "ffn", z["top"] * z["ff"] + z["sff"], d["ffn"]["ff_act"]
        else:
            ls.mlp, ls.experts, ls.identity, ls.top, ls.groups, ls.keep = "moe", z["experts"] - 2, 2, z["top"], z["groups"], z["keep"]
            ls.ff, ls.shared_ff = z["ff"], z["sff"]
            for k, v in d["moe"].items():
                setattr(ls, k, v)
        layers.append(ls)
    return HybridSpec(z["width"], z["vocab"], 1e-6, layers, architecture="Lisenex", embed_scale=float(z["width"]) ** 0.5)


def kokatar_spec(z, window=1024):
    """Layers that resemble a real model's: attention with 128-wide heads, four query heads per key/value head, half of a
    head rotated, 4 taps on q | k | v; latent attention with 16 heads of 64 / 128 over a latent of 256 / 512; every layer
    looks back `window` tokens; 4 taps on the sublayers' inputs; feed-forwards alternate between a dense one as wide as a
    token's active experts and `experts` routed experts with a shared one."""
    from .hybrid import DESIGNS, HybridSpec, LayerSpec
    d = DESIGNS["Kokatar"]
    W = z["width"]
    heads = W // 128
    layers = []
    for i in range(z["layers"]):
        if i % 3 == 0:
            ls = LayerSpec("attention", heads, 128, 128, rot_dims=64, rot_base=10000.0, attn_scale=128 ** -0.5,
                           kv_heads=max(1, heads // 4), conv=4, window=window, **d["attention"])
        else:
            ls = LayerSpec("latent_attention", z["lh"], z["ld"], z["ld"], kv_rank=z["kvr"], attn_scale=z["ld"] ** -0.5, window=window,
                           **d["latent"])
        if i % 2 == 0:
            ls.mlp, ls.ff, ls.ff_act = "ffn", z["top"] * z["ff"] + z["sff"], d["ffn"]["ff_act"]
        else:
            ls.mlp, ls.experts, ls.top, ls.ff, ls.shared_ff = "moe", z["experts"], z["top"], z["ff"], z["sff"]
            for k, v in d["moe"].items():
                setattr(ls, k, v)
        layers.append(ls)
    return HybridSpec(W, z["vocab"], 1e-6, layers, architecture="Kokatar", canon_taps=4)


def _events(fn, warmup, steps):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    t = []
    for _ in range(steps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        t.append(a.elapsed_time(b))
    return float(np.median(t))


def run_pikavik(z, prompt, batch, warmup, steps, dtype="bfloat16", spec_fn=pikavik_spec):
    from .hybrid import HybridRunner, random_hybrid_weights
    spec = spec_fn(z)
    tdt = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    w = random_hybrid_weights(spec, tdt, "cuda:0")
    bs = 64
    pages = -(-(prompt + 8) // bs)
    r = HybridRunner(spec, w, dtype=dtype, max_tokens=max(prompt, batch), max_seqs=batch, block_size=bs,
                     num_blocks=pages * batch, n_slots=batch, max_model_len=pages * bs, max_logit_rows=batch)
    g = torch.Generator().manual_seed(0)
    toks = torch.randint(0, spec.vocab, (prompt,), generator=g).tolist()
    tables = [list(range(i * pages, (i + 1) * pages)) for i in range(batch)]
    n0 = r.launch_count
    pre = _events(lambda: r.forward([(toks, 0, 0, tables[0], [prompt - 1])], want_logits=False, temps=[0.0]), warmup, steps)
    launches_prefill = (r.launch_count - n0) // (warmup + steps)
    for i in range(batch):  # every sequence gets a context (states and latent rows of its own)
        r.forward([(toks, 0, i, tables[i], [prompt - 1])], want_logits=False, temps=[0.0])
    n0 = r.launch_count
    dec = _events(lambda: r.forward([([toks[i]], prompt, i, tables[i], [0]) for i in range(batch)], want_logits=False,
                                    temps=[0.0] * batch), warmup, steps)
    launches_decode = (r.launch_count - n0) // (warmup + steps)
    params = sum(t.numel() for lw in w["layers"] for t in lw.values()) + w["HEAD"].numel()
    active = params - sum((lw["EXPERT_IN"].numel() + lw["EXPERT_OUT"].numel()) * (1 - min(1.0, ls.top / ls.experts))
                          for lw, ls in zip(w["layers"], spec.layers) if "EXPERT_IN" in lw)
    r.close()
    return {"prefill_ms": pre, "prefill_tok_s": prompt / pre * 1e3, "decode_ms": dec, "decode_tok_s": batch / dec * 1e3,
            "launches_prefill": launches_prefill, "launches_decode": launches_decode, "params": int(params),
            "active_params": int(active)}


def run_llama(z, prompt, batch, warmup, steps):
    """The dense arm: same width, depth and active feed-forward size; 128-wide heads, 4 query heads per KV head."""
    from . import lib as L
    from .runner import ModelSpec, PairRunner
    heads = z["width"] // 128
    ffn = z["top"] * z["ff"] + z["sff"]
    spec = ModelSpec(hidden=z["width"], layers=z["layers"], heads=heads, kv_heads=max(1, heads // 4), head_dim=128, ffn=ffn,
                     vocab=z["vocab"], rms_eps=1e-6, rope_theta=10000.0, max_pos=8192)
    bs = 256
    mb = -(-(prompt + 8) // bs)
    r = PairRunner(spec, None, spec_k=0, max_batch=batch, block_size=bs, max_model_len=mb * bs, use_graph=False)
    g = torch.Generator(device="cuda:0").manual_seed(0)
    bf = torch.bfloat16

    def lin(o, i):
        return (torch.randn(o, i, generator=g, device="cuda:0") / i ** 0.5).to(bf)

    d, hd, kv = spec.hidden, spec.head_dim, spec.kv_heads
    w = {"embed": torch.randn(spec.vocab, d, generator=g, device="cuda:0").to(bf), "lm_head": lin(spec.vocab, d),
         "final_norm": torch.ones(d, dtype=bf, device="cuda:0"), "layers": []}
    for _ in range(spec.layers):
        w["layers"].append({"input_norm": torch.ones(d, dtype=bf, device="cuda:0"), "post_norm": torch.ones(d, dtype=bf, device="cuda:0"),
                            "qkv": lin((heads + 2 * kv) * hd, d), "o": lin(d, heads * hd), "gate_up": lin(2 * ffn, d), "down": lin(d, ffn)})
    r.bind_weights(L.TARGET, w)
    r.finalize()
    toks = torch.randint(0, spec.vocab, (prompt,), generator=torch.Generator().manual_seed(0)).tolist()
    tables = [list(range(i * mb, (i + 1) * mb)) for i in range(batch)]
    n0 = r.launch_count
    pre = _events(lambda: r.prefill(L.TARGET, toks, tables[0]), warmup, steps)
    launches_prefill = (r.launch_count - n0) // (warmup + steps)
    for i in range(batch):
        r.prefill(L.TARGET, toks, tables[i])
    n0 = r.launch_count
    dec = _events(lambda: r.forward_tokens(L.TARGET, [[toks[i]] for i in range(batch)], [prompt] * batch, tables, [0.0] * batch),
                  warmup, steps)
    launches_decode = (r.launch_count - n0) // (warmup + steps)
    params = sum(t.numel() for lw in w["layers"] for t in lw.values()) + w["lm_head"].numel()
    r.close()
    return {"prefill_ms": pre, "prefill_tok_s": prompt / pre * 1e3, "decode_ms": dec, "decode_tok_s": batch / dec * 1e3,
            "launches_prefill": launches_prefill, "launches_decode": launches_decode, "params": int(params),
            "active_params": int(params)}


def run_kefurax(args):
    out = {"metric": "prefill and decode tokens/s, Kefurax beside Pikavik at equal width / depth / active feed-forward",
           "dtype": "bf16", "data": "synthetic (random weights, random token ids)", "n_gpus": 1, "steps": args.steps,
           "warmup": args.warmup, "timing": "CUDA events around the public forward call, median; every pass streams the stack's "
           "weights (> 126 MB L2 for size m; size s partly L2-resident, stated here)", "sizes": {}}
    names = [args.hybrid_size] if args.hybrid_size != "all" else list(SIZES)
    for name in names:
        z = SIZES[name]
        row = {"config": {k: z[k] for k in ("width", "layers", "vocab")}, "prompt": args.prompt_len_hybrid, "decode_batch": args.hybrid_batch}
        row["kefurax"] = run_pikavik(z, args.prompt_len_hybrid, args.hybrid_batch, args.warmup, args.steps, spec_fn=kefurax_spec)
        if not args.no_dense_arm:
            row["pikavik"] = run_pikavik(z, args.prompt_len_hybrid, args.hybrid_batch, args.warmup, args.steps)
        if args.hybrid_fp32:
            row["kefurax_fp32"] = run_pikavik(z, args.prompt_len_hybrid, args.hybrid_batch, args.warmup, args.steps, "float32", kefurax_spec)
        out["sizes"][name] = row
    return out


def run_lisenex(args):
    out = {"metric": "prefill and decode tokens/s, Lisenex beside Pikavik at equal width / depth / active feed-forward",
           "dtype": "bf16", "data": "synthetic (random weights, random token ids)", "n_gpus": 1, "steps": args.steps,
           "warmup": args.warmup, "timing": "CUDA events around the public forward call, median; every pass streams the stack's "
           "weights (> 126 MB L2 for size m; size s partly L2-resident, stated here)", "sizes": {}}
    names = [args.hybrid_size] if args.hybrid_size != "all" else list(SIZES)
    for name in names:
        z = SIZES[name]
        row = {"config": {k: z[k] for k in ("width", "layers", "experts", "top", "ff", "sff", "vocab")}, "prompt": args.prompt_len_hybrid,
               "decode_batch": args.hybrid_batch}
        row["lisenex"] = run_pikavik(z, args.prompt_len_hybrid, args.hybrid_batch, args.warmup, args.steps, spec_fn=lisenex_spec)
        if not args.no_dense_arm:
            row["pikavik"] = run_pikavik(z, args.prompt_len_hybrid, args.hybrid_batch, args.warmup, args.steps)
        if args.hybrid_fp32:
            row["lisenex_fp32"] = run_pikavik(z, args.prompt_len_hybrid, args.hybrid_batch, args.warmup, args.steps, "float32", lisenex_spec)
        out["sizes"][name] = row
    return out


def run_kokatar(args):
    out = {"metric": "prefill and decode tokens/s, Kokatar beside Lisenex at equal width / depth / feed-forward and expert sizes",
           "dtype": "bf16", "data": "synthetic (random weights, random token ids)", "n_gpus": 1, "steps": args.steps,
           "warmup": args.warmup, "timing": "CUDA events around the public forward call, median; every pass streams the stack's "
           "weights (> 126 MB L2 for size m; size s partly L2-resident, stated here)", "sizes": {}}
    names = [args.hybrid_size] if args.hybrid_size != "all" else list(SIZES)
    for name in names:
        z = SIZES[name]
        row = {"config": {k: z[k] for k in ("width", "layers", "experts", "top", "ff", "sff", "vocab")}, "prompt": args.prompt_len_hybrid,
               "decode_batch": args.hybrid_batch, "window": 1024}
        row["kokatar"] = run_pikavik(z, args.prompt_len_hybrid, args.hybrid_batch, args.warmup, args.steps, spec_fn=kokatar_spec)
        if not args.no_dense_arm:
            row["lisenex"] = run_pikavik(z, args.prompt_len_hybrid, args.hybrid_batch, args.warmup, args.steps, spec_fn=lisenex_spec)
        if args.hybrid_fp32:
            row["kokatar_fp32"] = run_pikavik(z, args.prompt_len_hybrid, args.hybrid_batch, args.warmup, args.steps, "float32", kokatar_spec)
        out["sizes"][name] = row
    return out


def run(args):
    if getattr(args, "arch", "pikavik") == "kokatar":
        return run_kokatar(args)
    if getattr(args, "arch", "pikavik") == "kefurax":
        return run_kefurax(args)
    if getattr(args, "arch", "pikavik") == "lisenex":
        return run_lisenex(args)
    out = {"metric": "prefill and decode tokens/s, Pikavik beside Llama at equal width / depth / active feed-forward",
           "dtype": "bf16", "data": "synthetic (random weights, random token ids)", "n_gpus": 1, "steps": args.steps,
           "warmup": args.warmup, "timing": "CUDA events around the public forward call, median; every pass streams the stack's "
           "weights (> 126 MB L2 for size m; size s partly L2-resident, stated here)", "sizes": {}}
    names = [args.hybrid_size] if args.hybrid_size != "all" else list(SIZES)
    for name in names:
        z = SIZES[name]
        row = {"config": {k: z[k] for k in ("width", "layers", "experts", "top", "ff", "sff", "vocab")}, "prompt": args.prompt_len_hybrid,
               "decode_batch": args.hybrid_batch}
        row["pikavik"] = run_pikavik(z, args.prompt_len_hybrid, args.hybrid_batch, args.warmup, args.steps)
        if not args.no_dense_arm:
            row["llama"] = run_llama(z, args.prompt_len_hybrid, args.hybrid_batch, args.warmup, args.steps)
        if args.hybrid_fp32:
            row["pikavik_fp32"] = run_pikavik(z, args.prompt_len_hybrid, args.hybrid_batch, args.warmup, args.steps, "float32")
        out["sizes"][name] = row
    return out
