"""Host side of the Kokatar design, no GPU: registry and configuration reading, checkpoint packing, and the float64
oracle's own consistency (portions == whole, window, sink, routing, activation, rotation)."""
import os

import pytest
import torch

from tests import kokatar_util as U
from tests import kokatar_plain as P


def _ckpt(tmp_path, layers, seed=0, **kw):
    cfg = U.config(layers, **kw)
    tensors = U.random_tensors(cfg, seed)
    return cfg, tensors, U.write_checkpoint(str(tmp_path / "ckpt"), cfg, tensors)


LAYERS = [U.attention(mlp=U.dense()), U.latent(mlp=U.moe()),
          U.attention(heads=4, kv_heads=4, dim=8, vdim=12, conv=1, window=40, scale=0.5, dims=0),
          U.latent(heads=1, dim=4, vdim=9, kv_rank=11, window=3, scale=0.7, mlp=U.moe(experts=5, top=1, ff=12, shared_ff=0))]


def test_registry_and_spec(tmp_path):
    from ssd_b200 import lib as L
    from ssd_b200.config import load_hf_config
    from ssd_b200.hybrid import HybridSpec
    _, _, path = _ckpt(tmp_path, LAYERS, width=24, vocab=31, eps=1e-5, taps=3)
    hf = load_hf_config(path)
    assert hf.family.name == "kokatar" and hf.family.kind == "hybrid" and hf.vocab_size == 31
    s = HybridSpec.from_dir(path)
    assert (s.width, s.vocab, s.eps, s.canon_taps, len(s.layers)) == (24, 31, 1e-5, 3, 4)
    assert s.block == L.BLOCK_PARALLEL_ONE_NORM and s.norm_offset == 0.0 and s.gated_residual and not s.tied_head
    assert s.has_cache and s.has_state
    a, b, c, d = s.layers
    assert (a.mixer, a.heads, a.kv_heads, a.dim, a.vdim, a.conv, a.window, a.attn_scale) == ("attention", 6, 2, 10, 6, 3, 24, 0.4)
    assert (a.rot_dims, a.rot_base, a.rot_half, a.learned_sink, a.mlp, a.ff, a.ff_act) == (6, 300.0, 1, 1, "ffn", 28, L.ACT_POLYNORM)
    assert (b.mixer, b.heads, b.dim, b.vdim, b.kv_rank, b.rot_dim, b.q_rank, b.window, b.learned_sink, b.out_gate) == ("latent_attention", 3, 10, 14, 20, 0, 0, 17, 0, 0)
    assert (b.mlp, b.experts, b.top, b.ff, b.shared_ff, b.route_top_softmax, b.expert_glu, b.expert_act, b.shared_gate) == ("moe", 6, 2, 20, 12, 1, 0, L.ACT_RELU2, 1)
    assert (c.kv_heads, c.conv, c.rot_dims, c.window, c.mlp) == (4, 1, 0, 40, None)
    assert (d.window, d.top, d.shared_ff) == (3, 1, 0)
    with pytest.raises(ValueError):
        HybridSpec.from_config(U.config([{"type": "wkv", "mixer": {"heads": 1, "dim": 4}, "mlp": None}]))
    # a model of the design without input convolutions: no history rows; latent layers alone then keep no state at all
    bare = U.config([U.latent()])
    del bare["canon"]
    sb = HybridSpec.from_config(bare)
    assert sb.canon_taps == 0 and not sb.has_state


def test_packing_matches_the_bound_layout(tmp_path):
    from ssd_b200.hybrid import HybridSpec, pack_hybrid_weights, read_safetensors
    cfg, tensors, path = _ckpt(tmp_path, LAYERS, taps=3)
    raw = read_safetensors(os.path.join(path, "model.safetensors"))
    assert set(raw) == set(tensors)
    w = pack_hybrid_weights(HybridSpec.from_dir(path), raw, torch.float32, "cpu")
    assert w["HEAD"] is not w["EMBED"] and torch.equal(w["HEAD"], tensors["head"])
    l0, l1, l2, l3 = w["layers"]
    # one stacked projection q | k | v with its bias and the taps of its convolution in the same row order
    assert l0["ATTN_IN"].shape == (6 * 10 + 2 * 10 + 2 * 6, 40) and torch.equal(l0["ATTN_IN"][60:80], tensors["l0.mix.k"])
    assert torch.equal(l0["ATTN_IN_B"][80:], tensors["l0.mix.v.b"]) and torch.equal(l0["CONV_W"][:60], tensors["l0.mix.q.conv"])
    assert l0["CONV_W"].shape == (92, 3) and l2["CONV_W"].shape == (4 * 8 + 4 * 8 + 4 * 12, 1)
    assert torch.equal(l0["ATTN_SINK"], tensors["l0.mix.sink"]) and "LAT_SINK" not in l1
    # input convolutions and residual gates: the mixer's first, the feed-forward's second; a layer without one has only the first
    assert l0["CANON_W"].shape == (2, 40, 3) and torch.equal(l0["CANON_W"][1], tensors["l0.canon2"])
    assert l2["CANON_W"].shape == (1, 40, 3) and l2["RES_GATE"].shape == (40, 40) and l2["RES_GATE_B"].shape == (40,)
    assert l1["RES_GATE"].shape == (80, 40) and torch.equal(l1["RES_GATE"][40:], tensors["l1.rg2"]) and torch.equal(l1["RES_GATE_B"][:40], tensors["l1.rg1.b"])
    # latent attention without a rotated part: q | dkv in one matrix, W_uk transposed per head
    assert l1["LAT_IN"].shape == (3 * 10 + 20, 40) and torch.equal(l1["LAT_IN"][30:], tensors["l1.mix.dkv"])
    assert l1["LAT_UKT"].shape == (3, 20, 10) and torch.equal(l1["LAT_UKT"][2], tensors["l1.mix.uk"].view(3, 10, 20)[2].T)
    # un-gated experts: one input matrix each; the shared expert's gate row behind its input matrix
    assert l1["EXPERT_IN"].shape == (6, 20, 40) and torch.equal(l1["EXPERT_IN"][4], tensors["l1.mlp.e4.up"])
    assert l1["SHARED_IN"].shape == (13, 40) and torch.equal(l1["SHARED_IN"][12], tensors["l1.mlp.shared.sg"][0]) and "SHARED_IN" not in l3
    assert torch.equal(l0["FFN_ACT"], tensors["l0.mlp.act"]) and "FFN_IN_B" not in l0 and "LS_MIX" not in l0 and "NORM2" not in l0


def test_oracle_portions_equal_whole(tmp_path):
    cfg, tensors, _ = _ckpt(tmp_path, LAYERS, taps=4)
    m = P.PlainModel(cfg, tensors)
    toks = torch.randint(0, 50, (60,), generator=torch.Generator().manual_seed(1)).tolist()
    whole = m.run(toks)
    st, out, pos = m.new_state(), [], 0
    for c in (7, 2, 1, 13, 7, 30):
        out.append(m.run(toks[pos:pos + c], st, pos))
        pos += c
    assert torch.allclose(torch.cat(out), whole, rtol=1e-10, atol=1e-10)


def test_oracle_window_and_sink():
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(9, 5, generator=g, dtype=P.F64) for _ in range(3))
    # window 1: every position sees itself only; without a sink the output is its own value row
    assert torch.allclose(P.windowed_softmax_attention(q, k, v, 0, 0.7, 1), v)
    # a key that dominates: read while it is among the query's last `window` positions, gone one position later
    k2 = k.clone(); k2[2] = 50.0 * q[6] / (q[6] @ q[6])
    o4 = P.windowed_softmax_attention(q, k2, v, 0, 5.0, 5)
    o3 = P.windowed_softmax_attention(q, k2, v, 0, 5.0, 4)
    assert torch.allclose(o4[6], v[2], atol=1e-6) and not torch.allclose(o3[6], v[2], atol=1e-2)
    assert [P.first_visible(i, 4) for i in (0, 3, 4, 10)] == [0, 0, 1, 7] and P.first_visible(10, 0) == 0
    # the sink joins the denominator once and carries no value: a huge sink empties the output, a tiny one changes nothing
    big = P.windowed_softmax_attention(q, k, v, 0, 0.7, 4, torch.tensor(40.0, dtype=P.F64))
    none = P.windowed_softmax_attention(q, k, v, 0, 0.7, 4, torch.tensor(-40.0, dtype=P.F64))
    assert big.abs().max() < 1e-9 and torch.allclose(none, P.windowed_softmax_attention(q, k, v, 0, 0.7, 4))
    zero = P.windowed_softmax_attention(q[:1], k[:1], v[:1], 0, 1.0, 4, (q[0] @ k[0]).clone())
    assert torch.allclose(zero[0], 0.5 * v[0])          # one key whose score equals the sink: half the weight each


def test_oracle_routing_activation_rotation_convolution():
    z = torch.tensor([0.5, 2.0, -1.0, 2.0, 1.0], dtype=P.F64)
    chosen, w = P.route_top(z, 3)
    assert chosen == [1, 3, 4] and abs(float(w.sum()) - 1.0) < 1e-12 and abs(float(w[0] / w[2]) - torch.e) < 1e-9   # ties to the lower index
    assert P.route_top(z, 1)[1].tolist() == [1.0]
    # PolyNorm: each power is brought to unit RMS before its coefficient; the constant is added last
    x = torch.randn(3, 16, dtype=P.F64)
    y = P.polynorm(x, torch.tensor([0.0, 1.0, 0.0, 0.25], dtype=P.F64), 0.0)
    assert torch.allclose(((y - 0.25) ** 2).mean(-1), torch.ones(3, dtype=P.F64)) and torch.allclose(P.polynorm(3 * x, torch.tensor([1.0, 1.0, 1.0, 0.0], dtype=P.F64), 0.0),
                                                                                                      P.polynorm(x, torch.tensor([1.0, 1.0, 1.0, 0.0], dtype=P.F64), 0.0))
    assert torch.equal(P.relu2_expert(torch.tensor([[-1.0, 2.0]], dtype=P.F64), torch.eye(2, dtype=P.F64), torch.eye(2, dtype=P.F64)), torch.tensor([[0.0, 4.0]], dtype=P.F64))
    # rotation: entry i turns with entry i + dims/2, lengths stay, products of rotated vectors depend on the distance only
    a, b = torch.randn(1, 1, 10, dtype=P.F64), torch.randn(1, 1, 10, dtype=P.F64)
    ra, rb = P.rotate_half(a, [17], 6, 100.0), P.rotate_half(b, [12], 6, 100.0)
    assert torch.equal(ra[..., 6:], a[..., 6:]) and abs(float(ra[0, 0, [0, 3]].norm() - a[0, 0, [0, 3]].norm())) < 1e-12
    rc, rd = P.rotate_half(a, [105], 6, 100.0), P.rotate_half(b, [100], 6, 100.0)
    assert abs(float((ra * rb).sum() - (rc * rd).sum())) < 1e-9
    # convolution: the last tap multiplies the current row; rows before the sequence are zeros; the history carries over
    u = torch.arange(1.0, 7.0, dtype=P.F64)[:, None]
    w = torch.tensor([[100.0, 10.0, 1.0]], dtype=P.F64)
    st = {}
    first = P.short_conv(u[:2], w, st, "h")
    rest = P.short_conv(u[2:], w, st, "h")
    assert torch.cat([first, rest])[:, 0].tolist() == [1.0, 12.0, 123.0, 234.0, 345.0, 456.0] and st["h"][:, 0].tolist() == [5.0, 6.0]
