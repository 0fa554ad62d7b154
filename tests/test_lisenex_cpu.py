"""Host side of the Lisenex design, no GPU: registry and configuration reading, checkpoint packing, and the float64
oracle's own consistency (portions == whole, routing rules, rotation)."""
import os

import pytest
import torch

from tests import lisenex_util as U
from tests import lisenex_plain as P


def _ckpt(tmp_path, layers, seed=0, **kw):
    cfg = U.config(layers, **kw)
    tensors = U.random_tensors(cfg, seed)
    return cfg, tensors, U.write_checkpoint(str(tmp_path / "ckpt"), cfg, tensors)


LAYERS = [U.latent(mlp=U.dense()), U.latent(kv_from=0, heads=2, dim=6, vdim=5, mlp=U.moe()),
          U.latent(heads=1, dim=4, rot_dim=6, vdim=9, kv_rank=11, scale=0.7, base=50.0, dims=4),
          U.latent(kv_from=0, mlp=U.moe(experts=5, identity=0, top=1, groups=1, keep=1, shared_ff=0))]


def test_registry_and_spec(tmp_path):
    from ssd_b200 import lib as L
    from ssd_b200.config import load_hf_config
    from ssd_b200.hybrid import HybridSpec
    _, _, path = _ckpt(tmp_path, LAYERS, width=24, vocab=31, eps=1e-5, embed_scale=7.0)
    hf = load_hf_config(path)
    assert hf.family.name == "lisenex" and hf.family.kind == "hybrid" and hf.vocab_size == 31
    s = HybridSpec.from_dir(path)
    assert (s.width, s.vocab, s.eps, s.embed_scale, len(s.layers)) == (24, 31, 1e-5, 7.0, 4)
    assert s.block == L.BLOCK_PARALLEL_TWO_NORMS and s.norm_offset == 0.0 and s.tied_head and s.has_cache and not s.has_state
    a, b, c, d = s.layers
    assert (a.mlp, a.ff, a.ff_act, a.kv_from, a.q_rank, a.rot_interleaved, a.out_gate, a.learned_sink) == ("ffn", 28, L.ACT_RELU2, -1, 0, 1, 1, 0)
    assert (b.kv_from, b.heads, b.dim, b.vdim, b.experts, b.identity, b.top, b.groups, b.keep, b.ff, b.shared_ff) == (0, 2, 6, 5, 6, 2, 3, 4, 2, 20, 12)
    assert (b.route_softmax, b.route_bias, b.group_best, b.route_renorm, b.expert_act, b.shared_gate) == (1, 1, 1, 0, L.ACT_SILU, 0)
    assert (c.heads, c.dim, c.rot_dim, c.rot_dims, c.vdim, c.kv_rank, c.attn_scale, c.rot_base, c.mlp) == (1, 4, 6, 4, 9, 11, 0.7, 50.0, None)
    assert (d.kv_from, d.experts, d.identity, d.top, d.groups, d.keep, d.shared_ff) == (0, 5, 0, 1, 1, 1, 0)
    with pytest.raises(ValueError):
        HybridSpec.from_config({**U.config([{"type": "wkv", "mixer": {"heads": 1, "dim": 4}, "mlp": None}])})


def test_packing_matches_the_bound_layout(tmp_path):
    from ssd_b200.hybrid import HybridSpec, pack_hybrid_weights, read_safetensors
    cfg, tensors, path = _ckpt(tmp_path, LAYERS)
    raw = read_safetensors(os.path.join(path, "model.safetensors"))
    assert set(raw) == set(tensors) and "head" not in raw and "l1.mix.dkv" not in raw
    w = pack_hybrid_weights(HybridSpec.from_dir(path), raw, torch.float32, "cpu")
    assert w["HEAD"] is w["EMBED"]
    l0, l1, l2, l3 = w["layers"]
    nq0 = 3 * (10 + 8)
    assert l0["LAT_IN"].shape == (nq0 + 28 + 3 * 14, 40)
    assert torch.equal(l0["LAT_IN"][nq0:nq0 + 28], tensors["l0.mix.dkv"]) and torch.equal(l0["LAT_IN"][nq0 + 28:], tensors["l0.mix.g"])
    assert l1["LAT_IN"].shape == (2 * (6 + 8) + 2 * 5, 40) and "LAT_KVNORM" not in l1 and "LAT_SINK" not in l0
    assert torch.equal(l1["LAT_IN"][28:], tensors["l1.mix.g"])
    uk = tensors["l0.mix.uk"].view(3, 10, 20)
    assert l0["LAT_UKT"].shape == (3, 20, 10) and torch.equal(l0["LAT_UKT"][2], uk[2].T)
    assert torch.equal(l0["FFN_IN_B"], tensors["l0.mlp.up.b"]) and torch.equal(l0["FFN_OUT_B"], tensors["l0.mlp.down.b"])
    assert l1["ROUTER"].shape == (8, 40) and torch.equal(l1["ROUTER_BIAS"], tensors["l1.mlp.correction"])
    assert l1["EXPERT_IN"].shape == (6, 40, 40) and torch.equal(l1["EXPERT_IN"][4, :20], tensors["l1.mlp.e4.gate"])
    assert l1["SHARED_IN"].shape == (24, 40) and "SHARED_IN" not in l3 and "NORM2" not in l2 and "LS_MIX" not in l0


def test_oracle_portions_equal_whole(tmp_path):
    cfg, tensors, _ = _ckpt(tmp_path, LAYERS)
    m = P.PlainModel(cfg, tensors)
    toks = torch.randint(0, 50, (30,), generator=torch.Generator().manual_seed(1)).tolist()
    whole = m.run(toks)
    st, out, pos = m.new_state(), [], 0
    for c in (7, 2, 1, 13, 7):
        out.append(m.run(toks[pos:pos + c], st, pos))
        pos += c
    assert torch.allclose(torch.cat(out), whole, rtol=1e-10, atol=1e-10)


def test_oracle_routing_rules():
    s = torch.tensor([0.05, 0.10, 0.30, 0.05, 0.20, 0.10, 0.15, 0.05], dtype=P.F64)
    # all choice scores negative: the shut-out groups must lose to negative scores (they count as -inf, not as 0)
    corr = torch.tensor([-1.0, -1.0, -1.0, -1.0, -0.5, -0.9, -0.9, -0.9], dtype=P.F64)
    chosen, w = P.route(s, corr, top=2, groups=4, keep=1)
    assert chosen == [4, 5] and [float(x) for x in w] == [0.20, 0.10]          # group 2 wins by its best (-0.3); plain scores as weights
    chosen, _ = P.route(s, torch.zeros(8, dtype=P.F64), top=3, groups=2, keep=1)
    assert chosen == [2, 1, 0]                                                    # ties go to the lower index
    chosen, w = P.route(s, torch.zeros(8, dtype=P.F64), top=8, groups=2, keep=2)
    assert sorted(chosen) == list(range(8)) and abs(float(sum(w)) - 1.0) < 1e-12


def test_oracle_identity_expert_and_rotation(tmp_path):
    cfg = U.config([U.latent(mlp=U.moe(experts=2, identity=2, top=1, groups=1, keep=1, shared_ff=0))])
    t = U.random_tensors(cfg, 2)
    t["l0.mlp.correction"] = torch.tensor([-9.0, -9.0, 0.0, 9.0])             # the last output, an identity expert, always wins
    W = {k: v.to(P.F64) for k, v in t.items()}
    h = torch.randn(5, 40, dtype=P.F64)
    s = torch.softmax(h @ W["l0.mlp.router"].T, -1)[:, 3:4]
    assert torch.allclose(P.moe_ff(h, W, "l0.mlp", cfg["layers"][0]["mlp"]), s * h)
    # rotation: pairs (2i, 2i+1) turn, lengths stay, the product of two rotated vectors depends on the distance only
    a, b = torch.randn(10, dtype=P.F64), torch.randn(10, dtype=P.F64)
    ra, rb = P.rotate_interleaved(a, 17, 6, 100.0), P.rotate_interleaved(b, 12, 6, 100.0)
    assert torch.equal(ra[6:], a[6:]) and abs(float(ra[:2].norm() - a[:2].norm())) < 1e-12
    rc, rd = P.rotate_interleaved(a, 105, 6, 100.0), P.rotate_interleaved(b, 100, 6, 100.0)
    assert abs(float(ra @ rb - rc @ rd)) < 1e-9
