"""Lisenex through libssdk (HybridRunner / LLM) against the plain float64 oracle of tests/lisenex_plain.py, on small
random checkpoints of sizes of their own.  float32 storage is the sharp comparison (a wrong key, edge, cache row or
router rule shows as an error of 1e-2 .. 1, rounding as 1e-6); bfloat16 runs are compared where no discrete choice
(expert routing) can flip."""
import numpy as np
import pytest
import torch

from tests import lisenex_util as U
from tests.lisenex_plain import PlainModel

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


# own caches and shared ones (adjacent, distant, two readers of one source), every feed-forward kind, sizes all unequal
FULL = [U.latent(mlp=U.dense()),
        U.latent(kv_from=0, heads=2, dim=6, vdim=5, scale=0.5, mlp=U.moe()),
        U.latent(heads=1, dim=4, rot_dim=6, vdim=9, kv_rank=11, scale=0.7, base=50.0, dims=4, mlp=U.moe(experts=4, identity=0, top=1, groups=1, keep=1, shared_ff=0)),
        U.latent(kv_from=0, heads=5, dim=3, vdim=4, mlp=U.moe(experts=7, identity=1, top=4, groups=2, keep=2, ff=12, shared_ff=20)),
        U.latent(kv_from=2, heads=2, dim=7, rot_dim=6, vdim=3, kv_rank=11, base=50.0, dims=4),
        U.latent(heads=4, dim=8, rot_dim=4, vdim=8, kv_rank=16, scale=0.25, mlp=U.moe(experts=3, identity=3, top=2, groups=3, keep=2, shared_ff=7))]


@pytest.mark.parametrize("layers", [[U.latent()], [U.latent(heads=5, dim=4, rot_dim=12, vdim=3, kv_rank=7, scale=1.0)],
                                    [U.latent(heads=1, dim=33, rot_dim=2, vdim=7, kv_rank=5)], [U.latent(rot_dim=10, dims=6)],
                                    [U.latent(), U.latent(kv_from=0, heads=2, dim=5, vdim=3)],
                                    [U.latent(), U.latent(rot_dim=4, kv_rank=9), U.latent(kv_from=0), U.latent(kv_from=1, rot_dim=4, kv_rank=9, heads=1)]],
                         ids=["latent", "odd-sizes", "one-head", "part-rot", "shared-cache", "shared-cache-distant"])
def test_latent_attention_alone(tmp_path, layers):
    cfg = U.config(layers)
    r, plain, _ = _runner(tmp_path, cfg)
    toks = _tokens(37, cfg["vocab"], 1)
    lg, _, res = r.forward([(toks, 0, 2, _pages(37, 16, 5), list(range(37)))], residual=True)
    lo = []
    ref = plain.run(toks, layers_out=lo)
    for i in range(len(layers)):
        assert U.rel_err(res[i], lo[i].numpy()) < F32_TOL, f"layer {i}"
    assert U.rel_err(lg, ref.numpy()) < F32_TOL


@pytest.mark.parametrize("mlp,correction", [(U.dense(), 0.3), (U.dense(ff=64), 0.3), (U.moe(), 0.3), (U.moe(), 3.0),
                                            (U.moe(experts=4, identity=0, top=1, groups=1, keep=1, shared_ff=0), 0.3),
                                            (U.moe(experts=5, identity=1, top=2, groups=6, keep=3, ff=12, shared_ff=20), 0.5),
                                            (U.moe(experts=2, identity=6, top=4, groups=2, keep=2, shared_ff=5), 0.3),
                                            (U.moe(experts=8, identity=4, top=3, groups=3, keep=1, shared_ff=0), 1.0)],
                         ids=["dense", "dense-wide", "grouped", "negative-choice-scores", "top1-plain", "one-output-groups",
                              "mostly-identity", "one-group-kept"])
def test_feed_forward_alone(tmp_path, mlp, correction):
    """The mixer is switched off by a zero output projection; what is left of the layer is x + ff(norm2(x)).  With large
    selection biases the choice scores of whole groups are negative: a shut-out group counted as 0 would win."""
    cfg = U.config([U.latent(mlp=mlp)])
    tensors = U.random_tensors(cfg, 3, correction=correction)
    tensors["l0.mix.o"].zero_()
    r, plain, _ = _runner(tmp_path, cfg, tensors=tensors, max_tokens=256, num_blocks=8, max_model_len=128)
    toks = _tokens(90, cfg["vocab"], 4)
    _, _, res = r.forward([(toks, 0, 0, _pages(90, 16), list(range(90)))], residual=True)
    lo = []
    plain.run(toks, layers_out=lo)
    assert U.rel_err(res[0], lo[0].numpy()) < F32_TOL
    if mlp["kind"] == "moe" and mlp["router"].get("identity"):
        # the comparison does rest on the identity experts: some token chooses one
        import tests.lisenex_plain as P
        W = plain.W
        x = W["embed"][torch.tensor(toks)] * cfg["embedding"]["scale"]
        h = P.rms_norm(x, W["l0.norm2"], 1e-6)
        s = torch.softmax(h @ W["l0.mlp.router"].T, -1)
        rt = mlp["router"]
        picks = [P.route(s[t], W["l0.mlp.correction"], rt["top"], rt["groups"]["count"], rt["groups"]["keep"])[0] for t in range(len(toks))]
        assert any(e >= rt["experts"] for p in picks for e in p)


def test_prefill_portions_and_token_by_token(tmp_path):
    cfg = U.config(FULL)
    r, plain, _ = _runner(tmp_path, cfg)
    n = 150
    toks = _tokens(n, cfg["vocab"], 5)
    ref = plain.run(toks).numpy()
    whole, _ = r.forward([(toks, 0, 0, _pages(n, 16), list(range(n)))])
    assert U.rel_err(whole, ref) < F32_TOL
    # portions of several sizes, down to two tokens, cut inside pages; then single tokens
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
    """Requests come and go through the engine's managers: a later request gets the pages and the slot that an earlier
    one dirtied, in another order; the layers that read another layer's pool follow the same page table."""
    from ssd_b200.engine.block_manager import BlockManager
    from ssd_b200.engine.sequence import Sequence
    from ssd_b200.engine.state_manager import StateSlotManager
    cfg = U.config(FULL)
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


def test_far_keys_and_page_borders(tmp_path):
    """Attention made sharp: a large score scale puts nearly all weight on ONE key, wherever it lies (hundreds of tokens
    back, on either side of a page border), in a layer with its own pool and in one that reads it."""
    cfg = U.config([U.latent(heads=4, dim=8, rot_dim=8, vdim=8, kv_rank=12, scale=6.0),
                    U.latent(kv_from=0, heads=2, dim=6, rot_dim=8, vdim=6, kv_rank=12, scale=4.0, mlp=U.moe())])
    r, plain, _ = _runner(tmp_path, cfg, seed=7, num_blocks=24, n_slots=1, max_model_len=384)
    n, tail = 330, 70
    toks = _tokens(n, cfg["vocab"], 8)
    ref = plain.run(toks).numpy()
    pages = list(range(23, 23 - 21, -1))
    out = [r.forward([(toks[:n - tail], 0, 0, pages, list(range(n - tail)))])[0]]
    for p in range(n - tail, n):  # decoding walks over four page borders
        out.append(r.forward([([toks[p]], p, 0, pages, [0])])[0])
    got = np.concatenate(out)
    per_pos = np.sqrt(((got - ref) ** 2).mean(-1)) / np.sqrt((ref ** 2).mean())
    assert per_pos.max() < 2e-3, f"worst position {int(per_pos.argmax())}"
    # the comparison does rest on far keys: another token at position 3 moves the logits hundreds of positions later
    toks2 = list(toks)
    toks2[3] = (toks[3] + 1) % cfg["vocab"]
    ref2 = plain.run(toks2).numpy()
    moved = np.sqrt(((ref2 - ref) ** 2).mean(-1))[200:] / np.sqrt((ref ** 2).mean())
    assert moved.max() > 50 * 2e-3
    got2, _ = r.forward([(toks2, 0, 0, pages, list(range(n)))])
    assert U.rel_err(got2, ref2) < 2e-3


def test_decoding_sequences_of_unequal_context_share_a_step(tmp_path):
    """Three sequences decode together at contexts of a few, ~150 and ~300 tokens beside a prompt portion of a fourth: the
    single-token rows take the split-context attention (some splits of the short sequence hold no key at all, and there is
    no sink to fill the denominator), the portion the GEMM path, in one call."""
    cfg = U.config([U.latent(heads=3, dim=8, rot_dim=8, vdim=10, kv_rank=12, scale=4.0, mlp=U.moe()),
                    U.latent(kv_from=0, heads=5, dim=6, rot_dim=8, vdim=6, kv_rank=12, scale=2.0, mlp=U.dense()),
                    U.latent(heads=2, dim=6, rot_dim=4, vdim=6, kv_rank=9, scale=2.0)])
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
    cfg = U.config(FULL)
    r, plain, _ = _runner(tmp_path, cfg, seed=2)
    for n in (1, 2, 3):
        toks = _tokens(n, cfg["vocab"], 30 + n)
        lg, _ = r.forward([(toks, 0, 1, [4], list(range(n)))])
        assert U.rel_err(lg, plain.run(toks).numpy()) < F32_TOL
    toks = _tokens(260, cfg["vocab"], 40)
    ref = plain.run(toks).numpy()
    out = [r.forward([(toks[:4], 0, 0, _pages(260, 16), [0, 1, 2, 3])])[0]]
    for p in range(4, 260):
        out.append(r.forward([([toks[p]], p, 0, _pages(260, 16), [0])])[0])
    got = np.concatenate(out)
    per_pos = np.sqrt(((got - ref) ** 2).mean(-1)) / np.sqrt((ref ** 2).mean())
    assert per_pos.max() < 5 * F32_TOL, f"worst position {int(per_pos.argmax())}"


def test_long_batches_are_split_into_calls(tmp_path):
    cfg = U.config(FULL[:4])
    r, plain, _ = _runner(tmp_path, cfg, max_tokens=48, max_seqs=2, max_logit_rows=48)
    seqs = [_tokens(n, cfg["vocab"], 50 + i) for i, n in enumerate([100, 7, 30])]
    lg, _ = r.forward([(s, 0, i, _pages(len(s), 16, 8 * i), [0, len(s) - 1]) for i, s in enumerate(seqs)])
    for i, s in enumerate(seqs):
        ref = plain.run(s).numpy()
        assert U.rel_err(lg[2 * i:2 * i + 2], ref[[0, len(s) - 1]]) < F32_TOL


def test_engine_rejects_a_cache_source_that_cannot_serve(tmp_path):
    """A layer may read only the pool of an EARLIER latent layer that fills its own with rows of the same layout."""
    for layers in ([U.latent(kv_from=1), U.latent()], [U.latent(), U.latent(kv_from=0), U.latent(kv_from=1)],
                   [U.latent(), U.latent(kv_from=0, kv_rank=12)]):
        cfg = U.config(layers)
        tensors = U.random_tensors(cfg, 0)
        path = U.write_checkpoint(str(tmp_path / f"bad{len(layers)}{layers[-1]['mixer']['kv_rank']}"), cfg, tensors)
        with pytest.raises(RuntimeError):
            _load(path)


@pytest.mark.parametrize("width", [40, 128, 36], ids=["rows-16B-aligned", "tcgen05-shapes", "unaligned"])
def test_bfloat16_storage(tmp_path, width):
    """bf16 weights / activations / cache with fp32 accumulation, residual, router and scores.  Every router output is
    chosen (top == outputs), so no routing decision can flip between the oracle and the rounded run.  The width picks the
    product kernel: 128 puts the dense projections on the tcgen05 GEMM, 40 on the mma.sync tile, 36 on the FMA tile."""
    every = dict(experts=3, identity=1, top=4, groups=2, keep=2)
    cfg = U.config([U.latent(mlp=U.dense(ff=64)), U.latent(kv_from=0, mlp=U.moe(**every)), U.latent(heads=2, dim=32, rot_dim=16, vdim=32, kv_rank=64, mlp=U.moe(**every)),
                    U.latent(kv_from=2, heads=4, dim=16, rot_dim=16, vdim=16, kv_rank=64)], width=width)
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
    assert U.rel_err(np.concatenate(out), whole) < 1e-2


def test_bfloat16_decode_attention_on_tensor_cores(tmp_path, monkeypatch):
    """Single-token rows of bf16 models whose cached rows start on 16-byte boundaries take the tensor-core form of the
    split-context attention: more than 16 heads (two head groups), latent sizes that end inside an n-tile pair, a column
    count that is no multiple of 16 (zero padding), three instantiations, contexts from a few keys (empty splits, a partly
    filled tile) to hundreds.  Against the oracle, and against the CUDA-core form of the same pass."""
    cfg = U.config([U.latent(heads=20, dim=16, rot_dim=16, vdim=8, kv_rank=40, scale=1.5, mlp=U.dense(ff=64)),
                    U.latent(kv_from=0, heads=3, dim=8, rot_dim=16, vdim=24, kv_rank=40, scale=1.0),
                    U.latent(heads=6, dim=16, rot_dim=64, vdim=16, kv_rank=128, scale=0.5),
                    U.latent(heads=2, dim=24, rot_dim=8, vdim=16, kv_rank=136, scale=0.5)], width=64)
    tensors = U.random_tensors(cfg, 9)
    path = U.write_checkpoint(str(tmp_path / "dec"), cfg, tensors)
    plain = PlainModel(cfg, tensors)
    lens, steps = [5, 70, 333], 5
    seqs = [_tokens(n + steps, cfg["vocab"], 100 + i) for i, n in enumerate(lens)]
    refs = [plain.run(s).numpy() for s in seqs]
    pages = [_pages(len(s), 16, first) for s, first in zip(seqs, (0, 3, 10))]
    got = {}
    for mma in ("1", "0"):
        monkeypatch.setenv("SSDK_HYB_DECODE_MMA", mma)
        r = _load(path, "bfloat16", num_blocks=40)
        for i in range(3):
            r.forward([(seqs[i][:lens[i]], 0, i, pages[i], [lens[i] - 1])])
        out = [[] for _ in seqs]
        for t in range(steps):
            lg, _ = r.forward([([seqs[i][lens[i] + t]], lens[i] + t, i, pages[i], [0]) for i in range(3)])
            for i in range(3):
                out[i].append(lg[i:i + 1])
        got[mma] = [np.concatenate(o) for o in out]
        r.close()
    for i in range(3):
        assert U.rel_err(got["1"][i], refs[i][lens[i]:]) < BF16_TOL, f"sequence {i}"
        assert U.rel_err(got["1"][i], got["0"][i]) < 1e-2, f"sequence {i}: the two forms of the pass disagree"


def test_bfloat16_calls_of_many_rows(tmp_path):
    """More rows than one tile of the tcgen05 GEMM holds (256): the dense projections run as row chunks of one launch, the
    last chunk partly filled; two prompts of unequal length in one call, against the oracle and against portions."""
    every = dict(experts=3, identity=1, top=4, groups=2, keep=2, ff=64, shared_ff=64)
    cfg = U.config([U.latent(heads=2, dim=32, rot_dim=16, vdim=32, kv_rank=64, mlp=U.moe(**every)),
                    U.latent(kv_from=0, heads=4, dim=16, rot_dim=16, vdim=16, kv_rank=64, mlp=U.dense(ff=192))], width=128, vocab=96)
    r, plain, _ = _runner(tmp_path, cfg, dtype="bfloat16", max_tokens=1024, num_blocks=64)
    seqs = [_tokens(330, cfg["vocab"], 80), _tokens(271, cfg["vocab"], 81)]
    refs = [plain.run(s).numpy() for s in seqs]
    lg, _ = r.forward([(s, 0, i, _pages(len(s), 16, 30 * i), list(range(len(s)))) for i, s in enumerate(seqs)])
    got = [lg[:330], lg[330:]]
    for g, ref in zip(got, refs):
        assert U.rel_err(g, ref) < BF16_TOL
    out, pos = [], 0
    for c in [200, 100, 30]:
        out.append(r.forward([(seqs[0][pos:pos + c], pos, 2, _pages(330, 16, 30), list(range(c)))])[0])
        pos += c
    assert U.rel_err(np.concatenate(out), got[0]) < 2e-2


def test_bfloat16_experts_on_the_grouped_tensor_core_gemm(tmp_path, monkeypatch):
    """Calls with many routed rows take the grouped tcgen05 GEMM (rows gathered per expert, a tile list per expert on the
    device): experts with few or no rows, identity outputs sorted behind the real ones, an output width that ends inside a
    tile (the next expert's rows are read and dropped).  Against the mma.sync tile on the same checkpoint (the routing is the
    same code, so the two agree to rounding) and, with every output chosen, against the oracle."""
    for name, mlp, oracle in (("few", U.moe(experts=9, identity=1, top=2, groups=5, keep=2, ff=64, shared_ff=0), False),
                              ("all", U.moe(experts=5, identity=1, top=6, groups=3, keep=3, ff=192, shared_ff=64), True)):
        cfg = U.config([U.latent(heads=2, dim=16, rot_dim=16, vdim=16, kv_rank=48, mlp=mlp),
                        U.latent(kv_from=0, heads=3, dim=8, rot_dim=16, vdim=8, kv_rank=48, mlp=mlp)], width=192)
        tensors = U.random_tensors(cfg, 13, correction=1.0)
        path = U.write_checkpoint(str(tmp_path / name), cfg, tensors)
        toks = _tokens(300, cfg["vocab"], 120)
        got = {}
        for tc in ("1", "0"):
            monkeypatch.setenv("SSDK_HYB_TC_EXPERTS", tc)
            r = _load(path, "bfloat16", num_blocks=24)
            got[tc], _ = r.forward([(toks, 0, 0, _pages(300, 16), list(range(300)))])
            r.close()
        assert U.rel_err(got["1"], got["0"]) < 2e-3, name
        if oracle:
            assert U.rel_err(got["1"], PlainModel(cfg, tensors).run(toks).numpy()) < BF16_TOL


def test_greedy_generation_through_llm(tmp_path):
    """The public entry point: LLM.generate with the engine's scheduler (three prompts, two sequences at a time: the third
    waits and gets used pages), temperature 0, against the oracle's greedy continuation."""
    from ssd_b200 import LLM, SamplingParams
    cfg = U.config(FULL[:4], vocab=64)
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
