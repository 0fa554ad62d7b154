"""Kokatar through libssdk (HybridRunner / LLM) against the plain float64 oracle of tests/kokatar_plain.py, on small
random checkpoints of sizes of their own.  float32 storage is the sharp comparison (a wrong key, a window that is one
position off, a lost convolution row or a missing sink shows as an error of 1e-2 .. 1, rounding as 1e-6); bfloat16 runs
are compared where no discrete choice (expert routing) can flip."""
import copy

import numpy as np
import pytest
import torch

from tests import kokatar_util as U
from tests.kokatar_plain import PlainModel

pytestmark = pytest.mark.gpu

F32_TOL = 3e-4
BF16_TOL = 6e-2


def _load(path, dtype="float32", **kw):
    from ssd_b200.hybrid import HybridRunner, HybridSpec, load_hybrid_weights
    spec = HybridSpec.from_dir(path)
    w = load_hybrid_weights(path, spec, {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype], "cuda:0")
    args = dict(dtype=dtype, max_tokens=512, max_seqs=4, block_size=16, num_blocks=40, n_slots=4, max_model_len=512)
    args.update(kw)
    return HybridRunner(spec, w, **args)


def _runner(tmp_path, cfg, seed=0, dtype="float32", tensors=None, **kw):
    tensors = tensors if tensors is not None else U.random_tensors(cfg, seed)
    path = U.write_checkpoint(str(tmp_path / f"ckpt{seed}"), cfg, tensors)
    return _load(path, dtype, **kw), PlainModel(cfg, tensors), path


def _tokens(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def _pages(n, block, first=0):
    return list(range(first, first + -(-n // block)))


def _per_pos(got, ref):
    return np.sqrt(((got - ref) ** 2).mean(-1)) / np.sqrt((ref ** 2).mean())


# both mixers, every feed-forward kind and none, all sizes unequal: windows shorter and longer than a page and than the
# portions, 1 .. 5 taps, grouped heads 6:2, 4:4 and 5:1, full, partial and no rotation, value size above and below the key size
FULL = [U.attention(mlp=U.dense()),
        U.latent(mlp=U.moe()),
        U.attention(heads=4, kv_heads=4, dim=8, vdim=12, conv=1, window=40, scale=0.5, dims=8, mlp=U.moe(experts=5, top=1, ff=12, shared_ff=0)),
        U.latent(heads=1, dim=4, vdim=9, kv_rank=11, window=3, scale=0.7),
        U.attention(heads=5, kv_heads=1, dim=6, vdim=3, conv=5, window=9, scale=0.6, dims=0, mlp=U.moe(experts=7, top=4, ff=12, shared_ff=20)),
        U.latent(heads=5, dim=3, vdim=4, kv_rank=7, window=64, scale=1.0, mlp=U.dense(ff=33))]


@pytest.mark.parametrize("layer,taps", [(U.attention(), 2), (U.attention(heads=3, kv_heads=3, dim=12, vdim=12, conv=1, window=1000, dims=12), 4),
                                        (U.attention(heads=8, kv_heads=2, dim=4, vdim=7, conv=6, window=1, dims=2), 1),
                                        (U.attention(heads=2, kv_heads=1, dim=33, vdim=40, conv=2, window=16, dims=0), 3),
                                        (U.latent(), 2), (U.latent(heads=1, dim=33, vdim=7, kv_rank=5, window=16), 5),
                                        (U.latent(heads=5, dim=4, vdim=3, kv_rank=7, window=1000, scale=1.0), 1)],
                         ids=["attention", "attention-no-groups-full-rotation-wide-window", "attention-window-of-one", "attention-no-rotation-wide-values",
                              "latent", "latent-one-head-window-of-a-page", "latent-wide-window"])
def test_mixer_alone(tmp_path, layer, taps):
    """One layer without a feed-forward: norm, input convolution, mixer, residual gate."""
    cfg = U.config([layer], taps=taps)
    r, plain, _ = _runner(tmp_path, cfg)
    toks = _tokens(37, cfg["vocab"], 1)
    lg, _, res = r.forward([(toks, 0, 2, _pages(37, 16, 5), list(range(37)))], residual=True)
    lo = []
    ref = plain.run(toks, layers_out=lo)
    assert U.rel_err(res[0], lo[0].numpy()) < F32_TOL
    assert U.rel_err(lg, ref.numpy()) < F32_TOL


@pytest.mark.parametrize("mlp,taps", [(U.dense(), 2), (U.dense(ff=64), 4), (U.moe(), 2), (U.moe(experts=4, top=1, shared_ff=0), 1),
                                      (U.moe(experts=9, top=9, ff=12, shared_ff=20), 3), (U.moe(experts=2, top=2, ff=70, shared_ff=5), 2)],
                         ids=["dense", "dense-wide", "moe", "top1-no-shared", "all-chosen", "two-experts"])
def test_feed_forward_alone(tmp_path, mlp, taps):
    """The mixer is switched off by a zero output projection; what is left of the layer is x + gate * ff(h + conv(h))."""
    cfg = U.config([U.latent(mlp=mlp)], taps=taps)
    tensors = U.random_tensors(cfg, 3)
    tensors["l0.mix.o"].zero_()
    r, plain, _ = _runner(tmp_path, cfg, tensors=tensors, max_tokens=256, num_blocks=8, max_model_len=128)
    toks = _tokens(90, cfg["vocab"], 4)
    _, _, res = r.forward([(toks, 0, 0, _pages(90, 16), list(range(90)))], residual=True)
    lo = []
    plain.run(toks, layers_out=lo)
    assert U.rel_err(res[0], lo[0].numpy()) < F32_TOL


def test_gates_convolutions_and_sink_carry_weight(tmp_path):
    """The comparison rests on every part of the layer: an oracle without the residual gates, without the input
    convolutions, without the q/k/v convolution or with the sink pushed out of the denominator is far from the engine."""
    cfg = U.config([U.attention(mlp=U.dense())], taps=3)
    tensors = U.random_tensors(cfg, 6)
    tensors["l0.mix.sink"] += 2.0
    r, plain, _ = _runner(tmp_path, cfg, tensors=tensors)
    toks = _tokens(60, cfg["vocab"], 2)
    lg, _ = r.forward([(toks, 0, 0, _pages(60, 16), list(range(60)))])
    assert U.rel_err(lg, plain.run(toks).numpy()) < F32_TOL
    for name, change in (("gate", lambda t: (t["l0.rg1"].zero_(), t["l0.rg1.b"].fill_(30.0))),
                         ("feed-forward gate", lambda t: (t["l0.rg2"].zero_(), t["l0.rg2.b"].fill_(30.0))),
                         ("input convolution", lambda t: t["l0.canon1"].zero_()),
                         ("feed-forward input convolution", lambda t: t["l0.canon2"].zero_()),
                         ("key convolution", lambda t: (t["l0.mix.k.conv"].zero_(), t["l0.mix.k.conv"][:, -1].fill_(1.0))),
                         ("sink", lambda t: t["l0.mix.sink"].fill_(-40.0))):
        other = {k: v.clone() for k, v in tensors.items()}
        change(other)
        assert U.rel_err(lg, PlainModel(cfg, other).run(toks).numpy()) > 30 * F32_TOL, name


def test_prefill_portions_and_token_by_token(tmp_path):
    cfg = U.config(FULL, taps=3)
    r, plain, _ = _runner(tmp_path, cfg)
    n = 150
    toks = _tokens(n, cfg["vocab"], 5)
    ref = plain.run(toks).numpy()
    whole, _ = r.forward([(toks, 0, 0, _pages(n, 16), list(range(n)))])
    assert U.rel_err(whole, ref) < F32_TOL
    # portions of several sizes, down to two tokens (shorter than the taps), cut inside pages and windows; then single tokens
    for sizes, slot, first in (([2, 3, 16, 5, 2, 31, 2, 17, 64], 1, 10), ([1] * n, 2, 20), ([47, 2, 2, 2], 3, 30)):
        out, pos, k = [], 0, 0
        while pos < n:
            c = min(sizes[k % len(sizes)], n - pos)
            lg, _ = r.forward([(toks[pos:pos + c], pos, slot, _pages(n, 16, first), list(range(c)))])
            out.append(lg)
            pos, k = pos + c, k + 1
        got = np.concatenate(out)
        assert U.rel_err(got, ref) < F32_TOL
        assert np.abs(got - whole).max() < 1e-4 * np.abs(whole).max()


def test_batch_of_unequal_requests_equals_each_alone(tmp_path):
    cfg = U.config(FULL)
    r, plain, _ = _runner(tmp_path, cfg)
    lens = [70, 9, 33, 1]
    seqs = [_tokens(n, cfg["vocab"], 10 + i) for i, n in enumerate(lens)]
    alone = [r.forward([(s, 0, 0, _pages(len(s), 16), list(range(len(s))))])[0] for s in seqs]
    # step 1: portions of requests 0, 1 and 2 + the whole of request 3; step 2: the rests, one of them a single token
    cut = [40, 8, 20, 1]
    pages = [_pages(n, 16, 8 * i) for i, n in enumerate(lens)]
    a, _ = r.forward([(seqs[i][:cut[i]], 0, i, pages[i], list(range(cut[i]))) for i in range(4)])
    b, _ = r.forward([(seqs[i][cut[i]:], cut[i], i, pages[i], list(range(lens[i] - cut[i]))) for i in (2, 1, 0)])
    got = {0: [], 1: [], 2: [], 3: []}
    o = 0
    for i in range(4):
        got[i].append(a[o:o + cut[i]]); o += cut[i]
    o = 0
    for i in (2, 1, 0):
        got[i].append(b[o:o + lens[i] - cut[i]]); o += lens[i] - cut[i]
    for i in range(4):
        g = np.concatenate(got[i])
        assert np.abs(g - alone[i]).max() < 1e-5 * np.abs(alone[i]).max(), f"request {i} depends on its batch"
        assert U.rel_err(g, plain.run(seqs[i]).numpy()) < F32_TOL


def test_pages_and_slots_are_reused(tmp_path, monkeypatch):
    """Requests come and go through the engine's managers: a later request gets the pages and the slot (convolution
    histories of every layer) that an earlier one dirtied, in another order."""
    from ssd_b200.engine.block_manager import BlockManager
    from ssd_b200.engine.sequence import Sequence
    from ssd_b200.engine.state_manager import StateSlotManager
    cfg = U.config(FULL, taps=4)
    r, plain, _ = _runner(tmp_path, cfg, num_blocks=8, n_slots=2)
    monkeypatch.setattr(Sequence, "block_size", 16)
    bm, sm = BlockManager(8, 16, prefix_reuse=False), StateSlotManager(2)
    prompts = [_tokens(n, cfg["vocab"], 20 + i) for i, n in enumerate([50, 40, 45, 30])]
    used_pages, used_slots = [], []
    live = []
    for k, toks in enumerate(prompts):
        if len(live) == 2:  # the pools are full: the older request ends
            old = live.pop(0)
            bm.deallocate(old); sm.free(old)
        s = Sequence(toks)
        bm.allocate(s); sm.allocate(s)
        live.append(s)
        used_pages.append(tuple(s.block_table)); used_slots.append(s.state_slot)
        half = len(toks) // 2
        a, _ = r.forward([(toks[:half], 0, s.state_slot, s.block_table, list(range(half)))])
        b, _ = r.forward([(toks[half:], half, s.state_slot, s.block_table, list(range(len(toks) - half)))])
        assert U.rel_err(np.concatenate([a, b]), plain.run(toks).numpy()) < F32_TOL, f"request {k}"
    assert len(set(used_slots)) < len(used_slots) and len({p for t in used_pages for p in t}) <= 8


@pytest.mark.parametrize("window", [23, 32, 150], ids=["inside-a-page-pair", "two-pages", "hundreds-of-keys"])
def test_window_edges_with_sharp_attention(tmp_path, window):
    """Attention made sharp: a large score scale puts nearly all weight on ONE key of the window, wherever it lies — also
    on the oldest key the window keeps, and never on the one just outside.  In a prompt, in portions that start inside a
    window and while decoding over page borders; in both mixers.  The oracle with a window of one more or one less key is
    far from the engine, so the comparison does rest on the edge."""
    layers = [U.attention(heads=4, kv_heads=2, dim=8, vdim=8, conv=2, window=window, scale=5.0, dims=4),
              U.latent(heads=4, dim=8, vdim=8, kv_rank=12, window=window + 5, scale=6.0, mlp=U.moe())]
    cfg = U.config(layers)
    tensors = U.random_tensors(cfg, 7)
    r, plain, _ = _runner(tmp_path, cfg, seed=7, tensors=tensors, num_blocks=24, n_slots=2, max_model_len=384)
    n, tail = 330, 70
    toks = _tokens(n, cfg["vocab"], 8)
    ref = plain.run(toks).numpy()
    pages = list(range(23, 23 - 21, -1))
    out = [r.forward([(toks[:n - tail], 0, 0, pages, list(range(n - tail)))])[0]]
    for p in range(n - tail, n):  # decoding walks over four page borders
        out.append(r.forward([([toks[p]], p, 0, pages, [0])])[0])
    got = np.concatenate(out)
    assert _per_pos(got, ref).max() < 2e-3, f"worst position {int(_per_pos(got, ref).argmax())}"
    # portions that start in the middle of a window (their first rows see keys of earlier calls only up to the edge)
    out, pos = [], 0
    for c in [window + 3, 2, window - 1, 5, 64, 2, 400]:
        c = min(c, n - pos)
        if c:
            out.append(r.forward([(toks[pos:pos + c], pos, 1, pages, list(range(c)))])[0])
        pos += c
    assert pos == n and _per_pos(np.concatenate(out), ref).max() < 2e-3
    for li in (0, 1):
        for d in (-1, 1):
            other = copy.deepcopy(cfg)
            other["layers"][li]["mixer"]["mask"]["size"] += d
            moved = _per_pos(PlainModel(other, tensors).run(toks).numpy(), ref)
            far = moved > 0.02   # ten times the tolerance
            assert far[window:].sum() >= 3, (li, d)
            if window < 100:
                assert far[window:n - tail].sum() >= 3 and far[n - tail:].sum() >= 1, (li, d)


def test_decoding_sequences_of_unequal_context_share_a_step(tmp_path):
    """Three sequences decode together at contexts of a few, ~150 and ~300 tokens beside a prompt portion of a fourth: the
    single-token rows take the split-context attention over their windows (one shorter than its window, two longer; some
    splits hold no key at all), the portion the GEMM path, in one call."""
    cfg = U.config([U.attention(heads=6, kv_heads=3, dim=8, vdim=10, window=200, scale=2.0, mlp=U.moe()),
                    U.latent(heads=5, dim=6, vdim=6, kv_rank=12, window=140, scale=2.0, mlp=U.dense()),
                    U.attention(heads=2, kv_heads=2, dim=6, vdim=6, conv=4, window=8, scale=2.0, dims=6)], taps=4)
    r, plain, _ = _runner(tmp_path, cfg, seed=5, num_blocks=64)
    lens, steps = [3, 150, 300, 90], 6
    seqs = [_tokens(n + steps, cfg["vocab"], 90 + i) for i, n in enumerate(lens)]
    refs = [plain.run(s).numpy() for s in seqs]
    pages = [_pages(len(s), 16, first) for s, first in zip(seqs, (58, 40, 5, 30))]
    for i in range(3):  # prompts of the decoding sequences, each alone
        r.forward([(seqs[i][:lens[i]], 0, i, pages[i], [lens[i] - 1])])
    got = [[] for _ in seqs]
    for t in range(steps):
        ents = [([seqs[i][lens[i] + t]], lens[i] + t, i, pages[i], [0]) for i in range(3)]
        lo, hi = 16 * t, (16 * (t + 1) if t < steps - 1 else len(seqs[3]))
        ents.insert(1, (seqs[3][lo:hi], lo, 3, pages[3], list(range(hi - lo))))
        lg, _ = r.forward(ents)
        got[0].append(lg[0:1]); got[3].append(lg[1:1 + hi - lo]); got[1].append(lg[1 + hi - lo:2 + hi - lo]); got[2].append(lg[2 + hi - lo:])
    for i in range(3):
        assert U.rel_err(np.concatenate(got[i]), refs[i][lens[i]:]) < 2e-3, f"decoding sequence {i}"
    assert U.rel_err(np.concatenate(got[3]), refs[3]) < 2e-3


def test_first_tokens_and_long_decoding(tmp_path):
    cfg = U.config(FULL, taps=5)
    r, plain, _ = _runner(tmp_path, cfg, seed=2)
    for n in (1, 2, 3):   # fewer tokens than taps: the rest of the convolutions' reach is zeros, whatever the slot holds
        toks = _tokens(n, cfg["vocab"], 30 + n)
        lg, _ = r.forward([(toks, 0, 1, [4], list(range(n)))])
        assert U.rel_err(lg, plain.run(toks).numpy()) < F32_TOL
    toks = _tokens(260, cfg["vocab"], 40)
    ref = plain.run(toks).numpy()
    out = [r.forward([(toks[:4], 0, 1, _pages(260, 16), [0, 1, 2, 3])])[0]]
    for p in range(4, 260):
        out.append(r.forward([([toks[p]], p, 1, _pages(260, 16), [0])])[0])
    got = np.concatenate(out)
    assert _per_pos(got, ref).max() < 5 * F32_TOL, f"worst position {int(_per_pos(got, ref).argmax())}"


def test_long_batches_are_split_into_calls(tmp_path):
    cfg = U.config(FULL[:4])
    r, plain, _ = _runner(tmp_path, cfg, max_tokens=48, max_seqs=2, max_logit_rows=48)
    seqs = [_tokens(n, cfg["vocab"], 50 + i) for i, n in enumerate([100, 7, 30])]
    lg, _ = r.forward([(s, 0, i, _pages(len(s), 16, 8 * i), [0, len(s) - 1]) for i, s in enumerate(seqs)])
    for i, s in enumerate(seqs):
        ref = plain.run(s).numpy()
        assert U.rel_err(lg[2 * i:2 * i + 2], ref[[0, len(s) - 1]]) < F32_TOL


def test_engine_rejects_what_it_cannot_serve(tmp_path):
    bad = U.attention(heads=5, kv_heads=2)
    cfg = U.config([bad])
    cfg["layers"][0]["mixer"]["kv_heads"] = 5
    tensors = U.random_tensors(cfg, 0)
    cfg["layers"][0]["mixer"]["kv_heads"] = 2      # 5 query heads do not split over 2 key/value heads
    path = U.write_checkpoint(str(tmp_path / "bad"), cfg, tensors)
    with pytest.raises(RuntimeError):
        _load(path)


@pytest.mark.parametrize("width", [40, 128, 36], ids=["rows-16B-aligned", "tcgen05-shapes", "unaligned"])
def test_bfloat16_storage(tmp_path, width):
    """bf16 weights / activations / cache with fp32 accumulation, residual, norms, router, scores and gates.  Every expert
    is chosen (top == experts), so no routing decision can flip between the oracle and the rounded run.  The width picks
    the product kernel: 128 puts the dense projections on the tcgen05 GEMM, 40 on the mma.sync tile, 36 on the FMA tile."""
    every = dict(experts=4, top=4)
    cfg = U.config([U.attention(heads=4, kv_heads=2, dim=16, vdim=16, window=50, dims=8, mlp=U.dense(ff=64)), U.latent(mlp=U.moe(**every)),
                    U.latent(heads=2, dim=32, vdim=32, kv_rank=64, window=70, mlp=U.moe(**every)),
                    U.attention(heads=4, kv_heads=1, dim=16, vdim=24, conv=4, window=20, dims=16)], width=width, taps=4)
    r, plain, _ = _runner(tmp_path, cfg, dtype="bfloat16")
    n = 120
    toks = _tokens(n, cfg["vocab"], 60)
    ref = plain.run(toks).numpy()
    whole, _ = r.forward([(toks, 0, 0, _pages(n, 16), list(range(n)))])
    assert U.rel_err(whole, ref) < BF16_TOL
    out, pos = [], 0
    for c in [2, 30, 3, 64, 2] + [1] * 19:
        out.append(r.forward([(toks[pos:pos + c], pos, 1, _pages(n, 16, 9), list(range(c)))])[0])
        pos += c
    # single-token rows take the fused decode attention, which keeps its weights in fp32: equal up to bf16 rounding
    assert U.rel_err(np.concatenate(out), whole) < 1.5e-2


def test_bfloat16_calls_of_many_rows(tmp_path, monkeypatch):
    """More rows than one tile of the tcgen05 GEMM holds (256) and enough routed rows for the grouped tcgen05 expert GEMM
    (un-gated experts: one input matrix each); windows shorter than the prompt, so that the portion path runs in several
    query blocks over shifted key ranges.  Two prompts of unequal length in one call, against the oracle, against portions,
    and against the mma.sync tile on the same checkpoint."""
    every = dict(experts=3, top=3, ff=64, shared_ff=64)
    cfg = U.config([U.latent(heads=2, dim=32, vdim=32, kv_rank=64, window=100, mlp=U.moe(**every)),
                    U.attention(heads=4, kv_heads=2, dim=16, vdim=16, window=130, dims=16, mlp=U.dense(ff=192)),
                    U.latent(heads=4, dim=16, vdim=16, kv_rank=64, window=300, mlp=U.moe(**every))], width=128, vocab=96, taps=4)
    tensors = U.random_tensors(cfg, 0)
    path = U.write_checkpoint(str(tmp_path / "rows"), cfg, tensors)
    plain = PlainModel(cfg, tensors)
    seqs = [_tokens(330, cfg["vocab"], 80), _tokens(271, cfg["vocab"], 81)]
    refs = [plain.run(s).numpy() for s in seqs]
    got = {}
    for tc in ("1", "0"):
        monkeypatch.setenv("SSDK_HYB_TC_EXPERTS", tc)
        r = _load(path, "bfloat16", max_tokens=1024, num_blocks=64)
        lg, _ = r.forward([(s, 0, i, _pages(len(s), 16, 30 * i), list(range(len(s)))) for i, s in enumerate(seqs)])
        got[tc] = [lg[:330], lg[330:]]
        for g, ref in zip(got[tc], refs):
            assert U.rel_err(g, ref) < BF16_TOL
        if tc == "1":
            out, pos = [], 0
            for c in [200, 100, 30]:
                out.append(r.forward([(seqs[0][pos:pos + c], pos, 2, _pages(330, 16, 30), list(range(c)))])[0])
                pos += c
            assert U.rel_err(np.concatenate(out), got[tc][0]) < 2e-2
        r.close()
    assert U.rel_err(got["1"][0], got["0"][0]) < 5e-3


def test_greedy_generation_through_llm(tmp_path):
    """The public entry point: LLM.generate with the engine's scheduler (three prompts, two sequences at a time: the third
    waits and gets used pages and a used slot), temperature 0, against the oracle's greedy continuation."""
    from ssd_b200 import LLM, SamplingParams
    cfg = U.config(FULL[:4], vocab=64, taps=3)
    tensors = U.random_tensors(cfg, 11)
    path = U.write_checkpoint(str(tmp_path / "gen"), cfg, tensors)
    plain = PlainModel(cfg, tensors)
    prompts = [_tokens(n, cfg["vocab"], 70 + i) for i, n in enumerate([21, 5, 40])]
    llm = LLM(path, dtype="float32", kvcache_block_size=16, max_model_len=128, max_num_batched_tokens=128, max_num_seqs=2)
    try:
        outs, _ = llm.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=12, ignore_eos=True), use_tqdm=False)
    finally:
        llm.exit()
    for p, o in zip(prompts, outs):
        assert o["token_ids"] == plain.greedy(p, 12)
