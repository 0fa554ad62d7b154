// hybrid_engine.cuh — host side of the layered (hybrid) model family: the layer program, the pools it addresses
// (paged latent cache, recurrent-state slots, workspace) and the ragged forward that prefill portions and single decode
// tokens share.  Included by engine.cu; uses its Launcher / error helpers.  Kernels: layer_ops.cuh, linear.cuh,
// recurrent.cuh, latent_attention.cuh, moe.cuh; the sampler is sample_kernel of sampling.cuh.
#pragma once
#include "conv_scan.cuh"
#include "gqa_attention.cuh"
#include "latent_attention.cuh"
#include "layer_ops.cuh"
#include "linear.cuh"
#include "moe.cuh"
#include "recurrent.cuh"

struct HybTensor {
  const void* p = nullptr;
  int64_t rows = 0, cols = 0;
};
struct HybLayer {
  ssdk_hyb_layer_cfg c;
  HybTensor t[SSDK_HT_COUNT];
  size_t state_off = 0;      // floats from the start of a slot
  size_t canon_off = 0;      // one-norm blocks: the input convolutions' history [canon_taps - 1, width], floats from the start of a slot
  size_t cache_row = 0;      // row width (elements) of this layer's latent pool
  size_t cache_rows_before = 0;  // sum of the row widths of the latent layers before this one
  float* inv_freq = nullptr; // device, [rot_dims / 2]
  float rot_mult = 1.0f;     // factor on cos and sin (frequency scaling)
};

struct ssdk_hyb_engine {
  ssdk_hyb_cfg cfg;
  std::vector<HybLayer> layers;
  HybTensor embed, head, final_norm;
  size_t esz = 2;            // sizeof(T)
  size_t slot_floats = 0, cache_row_total = 0;
  uint8_t* cache = nullptr; int64_t num_blocks = 0;
  float* state = nullptr; int64_t n_slots = 0;
  // workspace carve
  int64_t ws_bytes = 0;
  float *x = nullptr, *p0 = nullptr, *p1 = nullptr, *p2 = nullptr, *mix_out = nullptr, *mix2 = nullptr;
  void *h = nullptr, *h2 = nullptr, *hc = nullptr, *mixes = nullptr, *t0 = nullptr, *t1 = nullptr;
  float* gz = nullptr;       // one-norm blocks: pre-activations of the two residual gates [rows, 2 width]
  // latent attention: concatenated queries, one sequence's gathered keys / transposed latents, score and weight blocks
  void *qcat = nullptr, *keys = nullptr, *lat_t = nullptr, *att_p = nullptr; float* att_s = nullptr;
  float* att_o = nullptr;    // fp32 P C of the latent-attention portions when it runs on the tcgen05 GEMM (rounded to T afterwards)
  int w_lat_o = 0;           // heads x kv_rank of the widest latent layer
  size_t att_elems = 0; int w_qcat = 0, w_key = 0, w_kr = 0, w_lh = 0;
  float *rz = nullptr, *wts = nullptr, *eg = nullptr, *eo = nullptr, *sz = nullptr, *so = nullptr;
  void *ey = nullptr, *sy = nullptr, *xs = nullptr;   // xs: routed rows gathered per expert (grouped tcgen05 GEMM)
  int *sel = nullptr, *apos = nullptr, *arow = nullptr, *tile_expert = nullptr, *tile_row0 = nullptr, *tile_rows = nullptr,
      *n_tiles = nullptr, *n_rows = nullptr;
  void* hn = nullptr; float* logits = nullptr; bf16* logits16 = nullptr; int64_t* tokens = nullptr; float* temps = nullptr;
  int* meta = nullptr; size_t meta_ints = 0;
  int max_tiles = 0;
  // widths of the shared buffers (elements per row)
  int w_p0 = 0, w_p1 = 0, w_p2 = 0, w_t0 = 0, w_t1 = 0, w_e = 0, w_top = 0, w_ff2 = 0, w_ff = 0, w_sff2 = 0, w_sff = 0;
  bool any_wkv = false, any_pair = false, any_ffn = false;
  int* h_meta = nullptr;     // pinned staging of the step's integers
  // tcgen05 path of the dense bf16 products: TMA descriptors by (pointer, rows, K, box rows), split-K partials
  bool use_tc = true;
  bool use_decode_attn = true;  // fused single-token latent attention (SSDK_HYB_DECODE_ATTN=0: GEMM path for every row)
  bool use_tc_experts = true;   // routed experts of calls with many rows on the grouped tcgen05 GEMM (SSDK_HYB_TC_EXPERTS=0: mma.sync tile)
  bool use_tc_scores = true;    // score GEMM of latent-attention portions on the tcgen05 GEMM (SSDK_HYB_TC_SCORES=0: mma.sync tile)
  bool use_decode_mma = true;   // its tensor-core form for bf16 storage (SSDK_HYB_DECODE_MMA=0: the CUDA-core form)
  std::map<std::tuple<const void*, int64_t, int, int, int>, CUtensorMap> tmaps;
  float* partials = nullptr; size_t partial_floats = 0;
  int tmap(const void* ptr, int64_t rows, int K, int box_rows, const CUtensorMap** out, int ld = 0) {
    auto key = std::make_tuple(ptr, rows, K, box_rows, ld);
    auto it = tmaps.find(key);
    if (it == tmaps.end()) {
      if (tmaps.size() >= 8192) tmaps.clear();   // activations at changing offsets / row counts: keep the table bounded
      CUtensorMap tm;
      CKI(make_tmap(&tm, ptr, rows, K, box_rows, ld));
      it = tmaps.emplace(key, tm).first;
    }
    *out = &it->second;
    return 0;
  }
  int64_t launches = 0;
  bool smem_attr_done = false;
};

// delta rule: rows of a state column per thread (DR) and row groups (NG); DR = 0: the shared-memory walk
static void delta_shape(int D, int Vr, int* DR, int* NG) {
  *DR = 0; *NG = 1;
  if (D <= 16) { *DR = 16; return; }
  for (int dr : {32, 64}) {  // (16 rows per thread in eight row groups measured 5 % slower: the barriers outweigh the extra warps)
    const int g = (D + dr - 1) / dr;
    if (Vr * g <= 512 && g <= 8) { *DR = dr; *NG = g; return; }  // 512 threads: the register file holds DR + ~40 each
  }
}

static int hyb_derive(ssdk_hyb_engine* e) {
  const ssdk_hyb_cfg& g = e->cfg;
  size_t soff = 0, crow = 0;
  auto up = [](int& a, long long b) { if (b > a) a = (int)b; };
  for (size_t li = 0; li < e->layers.size(); ++li) {
    HybLayer& L = e->layers[li];
    const ssdk_hyb_layer_cfg& c = L.c;
    const int H = c.heads, D = c.dim, V = c.vdim;
    if (H < 1 || D < 1) return fail("hybrid layer: heads / dim must be positive");
    if (c.window < 0) return fail("hybrid layer: window %d", c.window);
    if (g.block == SSDK_BLOCK_PARALLEL_ONE_NORM) {
      if (c.mixer != SSDK_MIX_ATTENTION && c.mixer != SSDK_MIX_LATENT_ATTN && c.mixer != SSDK_MIX_RGLRU && c.mixer != SSDK_MIX_SELECTIVE)
        return fail("one-norm blocks are built for the attention, latent-attention, rglru and selective-scan mixers");
      L.canon_off = soff;
      if (g.canon_taps > 1) soff += (size_t)(g.canon_taps - 1) * g.width;
    }
    L.state_off = soff;
    if (c.mixer == SSDK_MIX_WKV) {
      if (D > 1024 || (size_t)(D * D + 5 * D + 1024) * 4 > 200 * 1024) return fail("wkv: head dim %d too large for the resident-state scan", D);
      soff += (size_t)H * D * D + g.width;
      up(e->w_p0, 5LL * H * D); up(e->w_p1, c.decay_rank); up(e->w_p2, (long long)H * D);
      up(e->w_t0, c.decay_rank); up(e->w_t1, (long long)H * D);
      e->any_wkv = true;
    } else if (c.mixer == SSDK_MIX_MLSTM) {
      if (V < 1 || std::max(D, V) > 1024 || (size_t)(D * V + 3 * D + 1024) * 4 > 200 * 1024) return fail("mlstm: head sizes %d x %d too large", D, V);
      soff += (size_t)H * D * V + (size_t)H * D + H;
      up(e->w_p0, 2LL * H * D + 2LL * H * V + 2 * H); up(e->w_p2, (long long)H * V); up(e->w_t1, (long long)H * V);
    } else if (c.mixer == SSDK_MIX_LATENT_ATTN) {
      if (c.rot_dims > c.rot_dim || (c.rot_dims & 1)) return fail("latent attention: rot dims %d of %d", c.rot_dims, c.rot_dim);
      if (V < 1 || c.kv_rank < 1 || c.rot_dim < 0 || c.q_rank < 0) return fail("latent attention: bad sizes");
      if (c.q_rank > 0 && (c.kv_from >= 0 || c.out_gate)) return fail("latent attention: a shared cache and an output gate are built for full-rank queries");
      if (c.kv_from >= 0) {
        // the layer reads the pool of an earlier latent layer that fills its own (same row layout and rotation)
        if ((size_t)c.kv_from >= li) return fail("latent attention: layer %d reads the cache of layer %d, which does not run before it", (int)li, c.kv_from);
        const HybLayer& src = e->layers[c.kv_from];
        if (src.c.mixer != SSDK_MIX_LATENT_ATTN || src.c.kv_from >= 0) return fail("latent attention: layer %d has no latent cache of its own", c.kv_from);
        if (src.c.kv_rank != c.kv_rank || src.c.rot_dim != c.rot_dim || src.c.rot_dims != c.rot_dims || src.c.rot_base != c.rot_base ||
            src.c.rot_interleaved != c.rot_interleaved)
          return fail("latent attention: layers %d and %d disagree on the cached row", (int)li, c.kv_from);
        L.cache_row = 0;
        L.cache_rows_before = src.cache_rows_before;
      } else {
        L.cache_row = (size_t)c.kv_rank + c.rot_dim;
        L.cache_rows_before = crow;
        crow += L.cache_row;
      }
      if (c.q_rank > 0) {
        up(e->w_p0, (long long)c.q_rank + c.kv_rank + c.rot_dim); up(e->w_p1, (long long)H * (D + c.rot_dim));
      } else {
        up(e->w_p0, (long long)H * (D + c.rot_dim) + (c.kv_from < 0 ? c.kv_rank + c.rot_dim : 0) + (c.out_gate ? (long long)H * V : 0));
        up(e->w_p1, (long long)H * V);
      }
      up(e->w_qcat, (long long)H * (c.kv_rank + c.rot_dim)); up(e->w_key, (long long)c.kv_rank + c.rot_dim);
      up(e->w_kr, c.kv_rank); up(e->w_lh, H); up(e->w_lat_o, (long long)H * c.kv_rank);
      up(e->w_t0, std::max((long long)c.q_rank, (long long)H * c.kv_rank)); up(e->w_t1, std::max((long long)H * D, (long long)H * V));
    } else if (c.mixer == SSDK_MIX_RGLRU) {
      const int R = c.inner;
      if (R < 1 || c.blocks < 1 || R % c.blocks || c.conv < 1) return fail("rglru: %d channels in %d blocks, %d taps", R, c.blocks, c.conv);
      soff += (size_t)R + (size_t)(c.conv - 1) * R;
      up(e->w_p0, 2LL * R); up(e->w_p1, R); up(e->w_p2, 2LL * R); up(e->w_t0, R); up(e->w_t1, R);
    } else if (c.mixer == SSDK_MIX_SELECTIVE) {
      const int I = c.inner, N = c.state, Rk = c.dt_rank;
      if (I < 1 || N < 1 || Rk < 1 || c.conv < 1) return fail("selective scan: inner %d, state %d, dt rank %d, %d taps", I, N, Rk, c.conv);
      soff += (size_t)I * N + (size_t)(c.conv - 1) * I;
      up(e->w_p0, 2LL * I); up(e->w_p1, I); up(e->w_p2, (long long)Rk + 2 * N + I); up(e->w_t0, I); up(e->w_t1, std::max(I, Rk));
    } else if (c.mixer == SSDK_MIX_ATTN_DELTA) {
      const int G = c.kv_heads, Hd = c.d_heads, Gd = c.d_kv_heads, Dd = c.d_dim, Vd = c.d_vdim;
      if (V < 1 || G < 1 || H % G) return fail("attention: %d query heads on %d key/value heads", H, G);
      if (c.rot_dims < 0 || c.rot_dims > D || (c.rot_dims & 1)) return fail("attention: rot dims %d of %d", c.rot_dims, D);
      if (V > 256 * 4) return fail("attention: value size %d too large", V);
      if (Hd < 1 || Gd < 1 || Hd % Gd || Dd < 1 || Vd < 1 || Vd > 1024 || c.conv < 1)
        return fail("delta rule: %d heads on %d query/key heads, %d x %d, %d taps", Hd, Gd, Dd, Vd, c.conv);
      {
        const int Vr = (Vd + 31) / 32 * 32;
        int dr = 0, ng = 1;
        delta_shape(Dd, Vr, &dr, &ng);
        if (dr == 0 && ssdk::delta_scan_smem(Dd, Vr, 0, 1) > 200 * 1024) return fail("delta rule: head %d x %d too large", Dd, Vd);
      }
      const long long Cd = 2LL * Gd * Dd + (long long)Hd * Vd;
      soff += (size_t)Hd * Dd * Vd + (size_t)(c.conv - 1) * Cd;
      L.cache_row = (size_t)G * (D + V);
      L.cache_rows_before = crow;
      crow += L.cache_row;
      up(e->w_p0, (long long)H * D + (long long)G * D + (long long)G * V + (long long)H * V + Cd + (long long)Hd * Vd + 2 * Hd);
      up(e->w_p1, std::max((long long)H * V, (long long)Hd * Vd)); up(e->w_p2, Cd + 2 * Hd);
      up(e->w_t0, (long long)H * V); up(e->w_t1, (long long)Hd * Vd);
      up(e->w_qcat, (long long)H * D); up(e->w_key, (long long)G * D); up(e->w_kr, (long long)G * V); up(e->w_lh, H);
      e->any_pair = true;
    } else if (c.mixer == SSDK_MIX_ATTENTION) {
      const int G = c.kv_heads;
      if (V < 1 || G < 1 || H % G) return fail("attention: %d query heads on %d key/value heads", H, G);
      if (c.rot_dims < 0 || c.rot_dims > D || (c.rot_dims & 1)) return fail("attention: rot dims %d of %d", c.rot_dims, D);
      if (V > 256 * 4) return fail("attention: value size %d too large", V);
      if (c.conv < 1) return fail("attention: %d taps", c.conv);
      const long long Nqkv = (long long)H * D + (long long)G * D + (long long)G * V;
      soff += (size_t)(c.conv - 1) * Nqkv;
      L.cache_row = (size_t)G * (D + V);
      L.cache_rows_before = crow;
      crow += L.cache_row;
      up(e->w_p0, Nqkv); up(e->w_p1, Nqkv); up(e->w_p2, (long long)H * V); up(e->w_t0, (long long)H * V);
      up(e->w_qcat, (long long)H * D); up(e->w_key, (long long)G * D); up(e->w_kr, (long long)G * V); up(e->w_lh, H);
    } else {
      return fail("hybrid layer: unknown mixer %d", c.mixer);
    }
    if (c.mlp == SSDK_MLP_GLU) {
      if (c.ff < 1) return fail("dense feed-forward: ff %d", c.ff);
      if (e->cfg.block != SSDK_BLOCK_SERIAL_POSTNORM) return fail("the dense feed-forward is built for serial blocks");
      up(e->w_p0, 2LL * c.ff); up(e->w_t0, c.ff);
    } else if (c.mlp == SSDK_MLP_FFN) {
      if (c.ff < 1) return fail("dense feed-forward: ff %d", c.ff);
      if (e->cfg.block == SSDK_BLOCK_SERIAL_POSTNORM) return fail("the ungated feed-forward is built for parallel blocks");
      if (c.ff_act != SSDK_ACT_RELU2 && c.ff_act != SSDK_ACT_GELU_TANH && c.ff_act != SSDK_ACT_SILU && c.ff_act != SSDK_ACT_POLYNORM)
        return fail("dense feed-forward: unknown activation %d", c.ff_act);
      up(e->w_sff2, c.ff); up(e->w_sff, c.ff);   // it shares the shared expert's buffers: no layer has both
      e->any_ffn = true;
    } else if (c.mlp == SSDK_MLP_MOE) {
      const int Et = c.experts + c.identity;   // router outputs: real experts, then identity experts
      if (e->cfg.block == SSDK_BLOCK_SERIAL_POSTNORM) return fail("the mixture of experts is built for parallel blocks");
      if (c.experts < 1 || c.identity < 0 || Et > kRouterMaxE) return fail("moe: 1 <= experts (+ identity) <= %d", kRouterMaxE);
      if (c.groups < 1 || Et % c.groups) return fail("moe: %d router outputs do not form %d equal groups", Et, c.groups);
      if (c.keep < 1 || c.keep > c.groups) return fail("moe: keep %d of %d groups", c.keep, c.groups);
      if (c.top < 1 || c.top > 32 || c.top > c.keep * (Et / c.groups)) return fail("moe: top %d does not fit the kept groups", c.top);
      if (c.group_best != 1 && c.group_best != 2) return fail("moe: a group scores its 1 or 2 best, not %d", c.group_best);
      if (c.expert_glu) {
        if (c.expert_act != SSDK_ACT_CLAMPED && c.expert_act != SSDK_ACT_SILU) return fail("moe: unknown gated expert activation %d", c.expert_act);
      } else if (c.expert_act != SSDK_ACT_RELU2 && c.expert_act != SSDK_ACT_SILU && c.expert_act != SSDK_ACT_GELU_TANH) {
        return fail("moe: unknown expert activation %d", c.expert_act);
      }
      const long long mats = c.expert_glu ? 2 : 1;   // stacked input matrices of an expert
      up(e->w_e, Et); up(e->w_top, c.top); up(e->w_ff2, mats * c.ff); up(e->w_ff, c.ff);
      if (c.shared_ff > 0) { up(e->w_sff2, mats * c.shared_ff + 1); up(e->w_sff, c.shared_ff); }
    } else if (c.mlp != SSDK_MLP_NONE) {
      return fail("hybrid layer: unknown feed-forward kind %d", c.mlp);
    }
  }
  e->slot_floats = soff;
  e->cache_row_total = crow;
  return 0;
}

// workspace carve: base == nullptr only sizes it
static int64_t hyb_carve(ssdk_hyb_engine* e, uint8_t* base) {
  const ssdk_hyb_cfg& g = e->cfg;
  const size_t cap = g.max_tokens, A = cap * (size_t)std::max(1, e->w_top), es = e->esz;
  size_t off = 0;
  auto take = [&](size_t bytes) { uint8_t* p = base ? base + off : nullptr; off = align_up(off + bytes, 256); return p; };
  e->x = (float*)take(cap * g.width * 4);
  e->h = take(cap * g.width * es);
  const bool one_norm = g.block == SSDK_BLOCK_PARALLEL_ONE_NORM;
  e->h2 = take(g.block == SSDK_BLOCK_PARALLEL_TWO_NORMS || (one_norm && g.canon_taps > 0) ? cap * g.width * es : 0);
  e->hc = take(one_norm && g.canon_taps > 0 ? cap * g.width * es : 0);
  e->gz = (float*)take(one_norm && g.gated_residual ? cap * 2 * g.width * 4 : 0);
  e->mixes = take(e->any_wkv ? 5 * cap * g.width * es : 0);
  e->p0 = (float*)take(cap * e->w_p0 * 4);
  e->p1 = (float*)take(cap * e->w_p1 * 4);
  e->p2 = (float*)take(cap * e->w_p2 * 4);
  e->t0 = take(cap * e->w_t0 * es);
  e->t1 = take(cap * e->w_t1 * es);
  e->mix_out = (float*)take(cap * g.width * 4);
  e->mix2 = (float*)take(e->any_pair ? cap * g.width * 4 : 0);
  {
    const size_t ctx_pad = align_up((size_t)g.max_blocks_per_seq * g.block_size, 64);
    e->qcat = take(cap * e->w_qcat * es);
    e->keys = take(e->w_key ? ctx_pad * e->w_key * es : 0);
    e->lat_t = take(e->w_kr ? ctx_pad * e->w_kr * es : 0);
    // one query block's scores (fp32) and weights (T): as many queries as fit 24 M elements, at least one
    e->att_elems = e->w_lh ? std::max((size_t)e->w_lh * ctx_pad, std::min(cap * e->w_lh * ctx_pad, (size_t)24 << 20)) : 0;
    e->att_s = (float*)take(e->att_elems * 4);
    e->att_p = take(e->att_elems * es);
    e->att_o = (float*)take(es == 2 ? cap * e->w_lat_o * 4 : 0);
  }
  e->rz = (float*)take(cap * e->w_e * 4);
  e->wts = (float*)take(A * 4);
  e->sel = (int*)take(A * 4); e->apos = (int*)take(A * 4); e->arow = (int*)take(A * 4);
  e->max_tiles = (int)(A / kLinBM + e->w_e + 1);
  e->tile_expert = (int*)take(e->max_tiles * 4); e->tile_row0 = (int*)take(e->max_tiles * 4);
  e->tile_rows = (int*)take(e->max_tiles * 4);
  e->n_tiles = (int*)take(4); e->n_rows = (int*)take(4);
  e->eg = (float*)take(A * e->w_ff2 * 4);
  e->ey = take(A * e->w_ff * es);
  e->xs = take(es == 2 && e->w_e ? A * g.width * es : 0);
  e->eo = (float*)take(e->w_e ? A * g.width * 4 : 0);
  e->sz = (float*)take(cap * e->w_sff2 * 4);
  e->sy = take(cap * e->w_sff * es);
  e->so = (float*)take(e->w_sff ? cap * g.width * 4 : 0);
  const size_t lr = g.max_logit_rows;
  e->hn = take(lr * g.width * es);
  e->logits = (float*)take(lr * g.vocab * 4);
  e->logits16 = (bf16*)take(lr * g.vocab * 2);
  e->tokens = (int64_t*)take(lr * 8);
  e->temps = (float*)take(lr * 4);
  e->meta_ints = 2 * cap + 3 * (size_t)g.max_seqs + 1 + (size_t)g.max_seqs * g.max_blocks_per_seq + lr;
  e->meta = (int*)take(e->meta_ints * 4);
  // split-K partials of the tcgen05 GEMM: up to 8 splits of a 256-row call of the widest output, bounded at 64 MB
  size_t widest = std::max<size_t>(g.vocab, g.width);
  for (int w : {e->w_p0, e->w_p1, e->w_sff2, one_norm ? 2 * g.width : 0}) widest = std::max<size_t>(widest, (size_t)w);
  e->partial_floats = es == 2 ? std::min<size_t>(8 * std::min<size_t>(cap, 256) * widest, 16u << 20) : 0;
  e->partials = (float*)take(e->partial_floats * 4);
  return (int64_t)off;
}

constexpr size_t kScanSmemMax = 200 * 1024;  // dynamic shared memory the scans may ask for

template <typename T>
struct HybRun {
  ssdk_hyb_engine* e;
  Launcher L;
  ssdk::Ragged rg;
  const int32_t *h_cu = nullptr, *h_pos0 = nullptr;  // host copies of the row offsets and first positions
  int M;

  template <typename OutT>
  int lin_args(const ssdk::LinearArgs& a, int rows_hint, int batch) {
    dim3 grid((a.N + ssdk::kLinBN - 1) / ssdk::kLinBN, a.tile_expert ? e->max_tiles : (rows_hint + ssdk::kLinBM - 1) / ssdk::kLinBM, batch);
    if constexpr (std::is_same<T, bf16>::value) {
      const bool vec = a.K % 8 == 0 && a.lda % 8 == 0 && a.ldw % 8 == 0 && a.sA % 8 == 0 && a.sW % 8 == 0 && a.sW_expert % 8 == 0 &&
                       ((uintptr_t)a.A & 15) == 0 && ((uintptr_t)a.W & 15) == 0;
      if (vec) return L.go(ssdk::linear_mma_kernel<OutT>, grid, dim3(ssdk::kMmaThreads), 0, a);
    }
    return L.go(ssdk::linear_kernel<T, OutT>, grid, dim3(ssdk::kLinThreads), 0, a);
  }
  // dense bf16 product on the tcgen05 GEMM of gemm.cuh (swap-AB, TMA-fed, fp32 out): K a multiple of 64, dense rows
  bool tc_ok(const void* A, int lda, const void* W, int ldw, int ldc, int N, int K) const {
    return std::is_same<T, bf16>::value && e->use_tc && K % kBlockK == 0 && lda == K && ldw >= K && ldw % 8 == 0 && ldc == N &&
           ((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0;
  }
  int lin_tc(const void* A, const void* W, float* C, int m_total, int N, int K, int ldw) {
    const CUtensorMap* tm;   // (copied: a later lookup may empty the table)
    CKI(e->tmap(W, N, K, 64, &tm, ldw == K ? 0 : ldw));
    const CUtensorMap tmW = *tm;
    // one launch for all rows: chunks of `un` tokens along gridDim.z share the weight tiles through L2
    const int un = umma_n_for(std::min(m_total, kMaxTokens)), chunks = (m_total + un - 1) / un;
    CKI(e->tmap(A, m_total, K, un, &tm));
    const CUtensorMap tmX = *tm;
    const int tiles = (N + kTileRows - 1) / kTileRows, num_kb = K / kBlockK;
    // narrow outputs (a head projection is 8 .. 32 tiles) with few row chunks fill the machine by splitting K
    int S = auto_splits(tiles * chunks, num_kb, un <= 64 ? 2 : 1);
    while (S > 1 && (size_t)S * m_total * N > e->partial_floats) --S;
    GemmParams p;
    p.M = m_total; p.N = N; p.ldo = N; p.num_kb = num_kb; p.tile_rows = kTileRows; p.hi_row_offset = 64;
    p.sk_partials = nullptr; p.sk_counters = nullptr; p.sk_width = 0;
    p.kb_per_split = (num_kb + S - 1) / S;
    S = (num_kb + p.kb_per_split - 1) / p.kb_per_split;
    p.out = S == 1 ? C : e->partials;
    CKI(launch_gemm(L, un, EPI_PARTIAL, tmW, tmX, p, tiles, S, chunks));
    if (S > 1) {
      const size_t n = (size_t)m_total * N;
      CKI(L.go(ssdk::splitk_sum_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, (const float*)e->partials, C, S, n));
    }
    return 0;
  }
  // grouped form: rows of X sorted by expert, tile list on the device (expert_plan_kernel with tiles of `un` rows);
  // C[r, :] = X[r, :] Wm[expert(r)]^T with Wm the experts' [N, K] matrices stacked by rows
  int lin_tc_grouped(const void* X, const void* Wm, float* C, int rows, int N, int K, int n_experts, int un, int max_tiles) {
    const CUtensorMap* tm;
    CKI(e->tmap(Wm, (int64_t)n_experts * N, K, 64, &tm));
    const CUtensorMap tmW = *tm;
    CKI(e->tmap(X, rows, K, un, &tm));
    const CUtensorMap tmX = *tm;
    GemmParams p;
    p.M = rows; p.N = N; p.ldo = N; p.num_kb = K / kBlockK; p.kb_per_split = p.num_kb; p.tile_rows = kTileRows; p.hi_row_offset = 64;
    p.sk_partials = nullptr; p.sk_counters = nullptr; p.sk_width = 0; p.out = C;
    p.g_tile_expert = e->tile_expert; p.g_tile_row0 = e->tile_row0; p.g_tile_rows = e->tile_rows; p.g_n_tiles = e->n_tiles;
    p.g_expert_rows = N;
    return launch_gemm(L, un, EPI_PARTIAL, tmW, tmX, p, (N + kTileRows - 1) / kTileRows, 1, max_tiles);
  }
  // C[M, N] (fp32 unless out_t) = A[M, K] W[N, K]^T
  int lin(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int m, int N, int K, bool out_t = false,
          int batch = 1, long long sA = 0, long long sW = 0, long long sC = 0, bool allow_tc = true) {
    if (allow_tc && !out_t && batch == 1 && tc_ok(A, lda, W, ldw, ldc, N, K)) return lin_tc(A, W, (float*)C, m, N, K, ldw);
    ssdk::LinearArgs a = {};
    a.A = A; a.W = W; a.C = C; a.M = m; a.N = N; a.K = K; a.lda = lda; a.ldw = ldw; a.ldc = ldc;
    a.sA = sA; a.sW = sW; a.sC = sC;
    return out_t ? lin_args<T>(a, m, batch) : lin_args<float>(a, m, batch);
  }
  int check_tensor(const HybLayer& Lr, int id, int64_t rows, int64_t cols, const char* name) {
    const HybTensor& t = Lr.t[id];
    if (!t.p) return fail("hybrid: tensor %s not bound", name);
    if (t.rows * t.cols != rows * cols) return fail("hybrid: tensor %s has %lld x %lld elements, expected %lld x %lld", name,
                                                     (long long)t.rows, (long long)t.cols, (long long)rows, (long long)cols);
    return 0;
  }

  // scan CTA: V columns (padded to a warp) x G row groups of >= 8 rows, at most 512 threads
  static ssdk::ScanShape scan_shape(int D, int V) {
    ssdk::ScanShape sh;
    sh.Vr = (V + 31) / 32 * 32;
    sh.G = std::max(1, std::min({8, 512 / sh.Vr, D / 8}));
    sh.Dg = (D + sh.G - 1) / sh.G;
    return sh;
  }

  // register-resident scan: the fewest rows per thread (8, 16 or 32) whose row groups fit 512 threads; *dg = 0 if none
  static ssdk::ScanShape reg_scan_shape(int D, int V, int* dg) {
    ssdk::ScanShape sh;
    sh.Vr = (V + 31) / 32 * 32;
    *dg = 0;
    if (env_int("SSDK_HYB_SCAN_SMEM", 0)) return sh;
    for (int d : {8, 16, 32}) {
      const int G = (D + d - 1) / d;
      if (sh.Vr * G <= 512) { *dg = d; sh.G = G; sh.Dg = d; break; }
    }
    return sh;
  }

  int wkv(HybLayer& Lr) {
    const ssdk_hyb_layer_cfg& c = Lr.c;
    const int H = c.heads, D = c.dim, HD = H * D, W = e->cfg.width;
    CKI(check_tensor(Lr, SSDK_HT_WKV_MU, 5, W, "wkv.mu")); CKI(check_tensor(Lr, SSDK_HT_WKV_R, HD, W, "wkv.r"));
    CKI(check_tensor(Lr, SSDK_HT_WKV_K, HD, W, "wkv.k")); CKI(check_tensor(Lr, SSDK_HT_WKV_V, HD, W, "wkv.v"));
    CKI(check_tensor(Lr, SSDK_HT_WKV_G, HD, W, "wkv.g")); CKI(check_tensor(Lr, SSDK_HT_WKV_W1, c.decay_rank, W, "wkv.w1"));
    CKI(check_tensor(Lr, SSDK_HT_WKV_W2, HD, c.decay_rank, "wkv.w2")); CKI(check_tensor(Lr, SSDK_HT_WKV_W0, HD, 1, "wkv.w0"));
    CKI(check_tensor(Lr, SSDK_HT_WKV_U, H, D, "wkv.u")); CKI(check_tensor(Lr, SSDK_HT_MIX_NORM, HD, 1, "mix.norm"));
    CKI(check_tensor(Lr, SSDK_HT_MIX_OUT, W, HD, "mix.o"));
    float* st = e->state + Lr.state_off;
    float* h_prev = st + (size_t)H * D * D;
    const T* mixes = (const T*)e->mixes;
    CKI(L.go(ssdk::token_shift_kernel<T>, dim3(M), dim3(256), 0, (const T*)e->h, (const T*)Lr.t[SSDK_HT_WKV_MU].p,
             (const float*)h_prev, e->slot_floats, (T*)e->mixes, rg, W, 5));
    float* pr = e->p0;
    float* pk = pr + (size_t)M * HD;
    float* pv = pk + (size_t)M * HD;
    float* pg = pv + (size_t)M * HD;
    float* pw = pg + (size_t)M * HD;
    const size_t ms = (size_t)M * W;
    CKI(lin(mixes + 0 * ms, W, Lr.t[SSDK_HT_WKV_R].p, W, pr, HD, M, HD, W));
    CKI(lin(mixes + 1 * ms, W, Lr.t[SSDK_HT_WKV_K].p, W, pk, HD, M, HD, W));
    CKI(lin(mixes + 2 * ms, W, Lr.t[SSDK_HT_WKV_V].p, W, pv, HD, M, HD, W));
    CKI(lin(mixes + 3 * ms, W, Lr.t[SSDK_HT_WKV_G].p, W, pg, HD, M, HD, W));
    CKI(lin(mixes + 4 * ms, W, Lr.t[SSDK_HT_WKV_W1].p, W, e->p1, c.decay_rank, M, c.decay_rank, W));
    const size_t nt = (size_t)M * c.decay_rank;
    CKI(L.go(ssdk::tanh_rows_kernel<T>, dim3((unsigned)std::min<size_t>((nt + 255) / 256, 4096)), dim3(256), 0,
             (const float*)e->p1, (T*)e->t0, nt));
    CKI(lin(e->t0, c.decay_rank, Lr.t[SSDK_HT_WKV_W2].p, c.decay_rank, pw, HD, M, HD, c.decay_rank));
    ssdk::WkvArgs a;
    a.r = pr; a.k = pk; a.v = pv; a.zw = pw; a.ld = HD; a.w0 = Lr.t[SSDK_HT_WKV_W0].p; a.u = Lr.t[SSDK_HT_WKV_U].p;
    a.o = e->p2; a.state = st; a.slot_stride = e->slot_floats; a.h = e->h; a.h_prev = h_prev; a.width = W; a.H = H; a.D = D;
    int dg = 0;
    ssdk::ScanShape sh = reg_scan_shape(D, D, &dg);
    const size_t reg_smem = dg ? ssdk::wkv_scan_reg_smem(D, sh, dg) : 0;
    if (dg && reg_smem <= kScanSmemMax) {
      const size_t smem = reg_smem;
      const dim3 grid(rg.n_seqs, H), block(sh.Vr * sh.G);
      if (dg == 8) CKI(L.go(ssdk::wkv_scan_reg_kernel<T, 8>, grid, block, smem, a, rg, sh));
      else if (dg == 16) CKI(L.go(ssdk::wkv_scan_reg_kernel<T, 16>, grid, block, smem, a, rg, sh));
      else CKI(L.go(ssdk::wkv_scan_reg_kernel<T, 32>, grid, block, smem, a, rg, sh));
    } else {
      sh = scan_shape(D, D);
      const size_t smem = (size_t)(D * D + 5 * D + sh.G * sh.Vr) * 4;
      CKI(L.go(ssdk::wkv_scan_kernel<T>, dim3(rg.n_seqs, H), dim3(sh.Vr * sh.G), smem, a, rg, sh));
    }
    CKI(L.go(ssdk::head_rmsnorm_gate_kernel<T, 0>, dim3(M, H), dim3(std::min(256, (D + 31) / 32 * 32)), 0, (const float*)e->p2,
             (const float*)pg, HD, (const T*)Lr.t[SSDK_HT_MIX_NORM].p, (T*)e->t1, H, D, e->cfg.eps));
    return lin(e->t1, HD, Lr.t[SSDK_HT_MIX_OUT].p, HD, e->mix_out, W, M, W, HD);
  }

  int mlstm(HybLayer& Lr) {
    const ssdk_hyb_layer_cfg& c = Lr.c;
    const int H = c.heads, D = c.dim, V = c.vdim, W = e->cfg.width;
    const int N = 2 * H * D + 2 * H * V + 2 * H;
    CKI(check_tensor(Lr, SSDK_HT_MLSTM_IN, N, W, "mlstm.in")); CKI(check_tensor(Lr, SSDK_HT_MLSTM_IB, H, 1, "mlstm.i.b"));
    CKI(check_tensor(Lr, SSDK_HT_MLSTM_FB, H, 1, "mlstm.f.b")); CKI(check_tensor(Lr, SSDK_HT_MIX_NORM, H * V, 1, "mix.norm"));
    CKI(check_tensor(Lr, SSDK_HT_MIX_OUT, W, H * V, "mix.o"));
    CKI(lin(e->h, W, Lr.t[SSDK_HT_MLSTM_IN].p, W, e->p0, N, M, N, W));
    ssdk::MlstmArgs a;
    a.q = e->p0; a.k = a.q + H * D; a.v = a.k + H * D;
    const float* g = a.v + H * V;
    a.ig = g + H * V; a.fg = a.ig + H; a.ld = N;
    a.ib = Lr.t[SSDK_HT_MLSTM_IB].p; a.fb = Lr.t[SSDK_HT_MLSTM_FB].p; a.o = e->p2;
    float* st = e->state + Lr.state_off;
    a.S = st; a.n = st + (size_t)H * D * V; a.m = a.n + (size_t)H * D; a.slot_stride = e->slot_floats;
    a.H = H; a.D = D; a.V = V; a.cap = c.gate_cap; a.q_scale = 1.0f / sqrtf((float)D);
    int dg = 0;
    ssdk::ScanShape sh = reg_scan_shape(D, V, &dg);
    const size_t reg_smem = dg ? ssdk::mlstm_scan_reg_smem(D, V, sh, dg) : 0;
    if (dg && reg_smem <= kScanSmemMax) {
      const size_t smem = reg_smem;
      const dim3 grid(rg.n_seqs, H), block(sh.Vr * sh.G);
      if (dg == 8) CKI(L.go(ssdk::mlstm_scan_reg_kernel<T, 8>, grid, block, smem, a, rg, sh));
      else if (dg == 16) CKI(L.go(ssdk::mlstm_scan_reg_kernel<T, 16>, grid, block, smem, a, rg, sh));
      else CKI(L.go(ssdk::mlstm_scan_reg_kernel<T, 32>, grid, block, smem, a, rg, sh));
    } else {
      sh = scan_shape(D, V);
      const size_t smem = (size_t)(D * V + 3 * D + sh.G * sh.Vr + sh.G) * 4;
      CKI(L.go(ssdk::mlstm_scan_kernel<T>, dim3(rg.n_seqs, H), dim3(sh.Vr * sh.G), smem, a, rg, sh));
    }
    CKI(L.go(ssdk::head_rmsnorm_gate_kernel<T, 1>, dim3(M, H), dim3(std::min(256, (V + 31) / 32 * 32)), 0, (const float*)e->p2, g, N,
             (const T*)Lr.t[SSDK_HT_MIX_NORM].p, (T*)e->t1, H, V, e->cfg.eps));
    return lin(e->t1, H * V, Lr.t[SSDK_HT_MIX_OUT].p, H * V, e->mix_out, W, M, W, H * V);
  }

  // query rows per block of a windowed attention's portion path
  static int window_block(int win) { return std::max(128, (win + 63) / 64 * 64); }

  int latent(HybLayer& Lr) {
    const ssdk_hyb_layer_cfg& c = Lr.c;
    const int H = c.heads, D = c.dim, V = c.vdim, R = c.rot_dim, KR = c.kv_rank, QR = c.q_rank, W = e->cfg.width;
    const bool own = c.kv_from < 0;   // the layer fills a pool of its own (else it reads an earlier layer's rows of this step and before)
    const int Nq = H * (D + R), Nkv = own ? KR + R : 0, win = c.window;
    CKI(check_tensor(Lr, SSDK_HT_LAT_UKT, (int64_t)H * KR, D, "uk^T")); CKI(check_tensor(Lr, SSDK_HT_LAT_UV, (int64_t)H * V, KR, "uv"));
    CKI(check_tensor(Lr, SSDK_HT_MIX_OUT, W, (int64_t)H * V, "mix.o"));
    if (own) CKI(check_tensor(Lr, SSDK_HT_LAT_KVNORM, KR, 1, "dkv.norm"));
    if (c.learned_sink) CKI(check_tensor(Lr, SSDK_HT_LAT_SINK, H, 1, "sink"));
    if (!e->cache) return fail("hybrid: latent cache not bound");
    uint8_t* pool = e->cache + (size_t)e->num_blocks * e->cfg.block_size * Lr.cache_rows_before * e->esz;
    const void* sink = c.learned_sink ? Lr.t[SSDK_HT_LAT_SINK].p : nullptr;
    const float* q = nullptr;       // fp32 query rows [H, D + R] with leading dimension ldq
    const float* gate = nullptr;    // fp32 pre-activations of the output gate [H V], leading dimension ldq
    int ldq = 0;
    ssdk::LatentPrepArgs pa;
    pa.qn_w = nullptr; pa.kvn_w = own ? Lr.t[SSDK_HT_LAT_KVNORM].p : nullptr; pa.cq = e->t0;
    pa.cache = pool; pa.inv_freq = Lr.inv_freq; pa.q_rank = QR; pa.kv_rank = KR; pa.rot_dim = R; pa.rot_dims = c.rot_dims;
    pa.interleaved = c.rot_interleaved; pa.eps = e->cfg.eps;
    if (QR > 0) {
      // low-rank queries: down projection (query latent | kv latent | key rot part), norms, then the query up projection
      const int Nd = QR + KR + R;
      CKI(check_tensor(Lr, SSDK_HT_LAT_DOWN, Nd, W, "latent.down")); CKI(check_tensor(Lr, SSDK_HT_LAT_QNORM, QR, 1, "dq.norm"));
      CKI(check_tensor(Lr, SSDK_HT_LAT_UQ, (int64_t)Nq, QR, "uq"));
      CKI(lin(hin, W, Lr.t[SSDK_HT_LAT_DOWN].p, W, e->p0, Nd, M, Nd, W));
      pa.z = e->p0; pa.ldz = Nd; pa.qn_w = Lr.t[SSDK_HT_LAT_QNORM].p;
      CKI(L.go(ssdk::latent_prep_kernel<T>, dim3(M), dim3(128), 0, pa, rg));
      CKI(lin(e->t0, QR, Lr.t[SSDK_HT_LAT_UQ].p, QR, e->p1, Nq, M, Nq, QR));
      q = e->p1; ldq = Nq;
    } else {
      // full-rank queries: ONE stacked projection q | kv latent, key rot part (own pool only) | output gate
      const int Nin = Nq + Nkv + (c.out_gate ? H * V : 0);
      CKI(check_tensor(Lr, SSDK_HT_LAT_IN, Nin, W, "latent.in"));
      CKI(lin(hin, W, Lr.t[SSDK_HT_LAT_IN].p, W, e->p0, Nin, M, Nin, W));
      q = e->p0; ldq = Nin;
      if (c.out_gate) gate = e->p0 + Nq + Nkv;
      if (own) {
        pa.z = e->p0 + Nq; pa.ldz = Nin;
        CKI(L.go(ssdk::latent_prep_kernel<T>, dim3(M), dim3(128), 0, pa, rg));
      }
    }
    const int Wd = KR + R;
    CKI(L.go(ssdk::latent_q_kernel<T>, dim3(M, H), dim3(64), 0, q, ldq, (T*)e->t1, (T*)e->qcat, (const float*)Lr.inv_freq, rg,
             H, D, R, KR, c.rot_dims, c.rot_interleaved));
    // absorption: qcat[m, h, :kv_rank] = W_uk,h^T qn[m, h, :]
    CKI(lin(e->t1, H * D, Lr.t[SSDK_HT_LAT_UKT].p, D, e->qcat, H * Wd, M, KR, D, true, H, D, (long long)KR * D, Wd));
    // single-token sequences (decode) share ONE fused launch + a merge; the others take the GEMM path below
    bool fused_decode = false;
    {
      int n_dec = 0, ctx_max = 0;
      for (int s = 0; s < rg.n_seqs; ++s)
        if (h_cu[s + 1] - h_cu[s] == 1) { ++n_dec; ctx_max = std::max(ctx_max, h_pos0[s] + 1); }
      if (win > 0) ctx_max = std::min(ctx_max, win);
      const size_t smem = ssdk::latent_decode_smem(H, KR, Wd, sizeof(T));
      const bool pool_aligned = ((uintptr_t)pool & 15) == 0;
      // bf16 rows that start on 16-byte boundaries go through the tensor cores: k-steps of 16 columns and n-tiles of 8
      // latent columns per warp pick the instantiation; the CUDA-core form holds all heads' queries and sums in shared memory
      const int ks_per = ((Wd + 15) / 16 + 3) / 4, nt_per = ((KR + 7) / 8 + 3) / 4;
      const bool mma = !kF32 && e->use_decode_mma && pool_aligned && Wd % 8 == 0 && KR % 8 == 0 && ks_per <= 9 && nt_per <= 16;
      if (n_dec > 0 && (mma || smem <= 200 * 1024) && e->use_decode_attn) {
        // ~2 CTAs per SM over all sequences, at least 64 keys per split, partials within the score buffer
        int splits = std::max(1, std::min({ssdk::kDecMaxSplits, 2 * num_sms() / n_dec, (ctx_max + 63) / 64}));
        const size_t per_split = (size_t)rg.n_seqs * H * (KR + 2);
        splits = (int)std::min<size_t>(splits, e->att_elems / per_split);
        if (splits >= 1) {
          ssdk::LatentDecodeArgs da;
          da.qcat = e->qcat; da.cache = pool; da.sink = sink; da.part = e->att_s; da.out = e->t0;
          da.H = H; da.KR = KR; da.W = Wd; da.splits = splits; da.scale = c.attn_scale; da.pool_aligned = pool_aligned; da.window = win;
          if (mma) {
            const dim3 grid(rg.n_seqs, splits, (H + 15) / 16), block(ssdk::kDmThreads);
            const size_t sm = ssdk::latent_decode_mma_smem(Wd);
            if (ks_per <= 3 && nt_per <= 4) CKI(L.go(ssdk::latent_decode_mma_kernel<3, 4>, grid, block, sm, da, rg));
            else if (ks_per <= 5 && nt_per <= 8) CKI(L.go(ssdk::latent_decode_mma_kernel<5, 8>, grid, block, sm, da, rg));
            else CKI(L.go(ssdk::latent_decode_mma_kernel<9, 16>, grid, block, sm, da, rg));
          } else {
            CKI(L.go(ssdk::latent_decode_partial_kernel<T>, dim3(rg.n_seqs, splits), dim3(ssdk::kDecThreads), smem, da, rg));
          }
          CKI(L.go(ssdk::latent_decode_merge_kernel<T>, dim3(rg.n_seqs, H, (KR + 127) / 128), dim3(128), 0, da, rg));
          fused_decode = true;
        }
      }
    }
    // both attention GEMMs of a portion run on the tcgen05 GEMM when the operands are whole k-blocks: the key count is then
    // padded to 64 (zero keys, zero weights) instead of 8
    const bool tc_attn = !kF32 && e->use_tc && e->use_tc_scores;
    const int kpad = tc_attn ? 64 : 8;
    for (int s = 0; s < rg.n_seqs; ++s) {
      const int r0 = h_cu[s], n = h_cu[s + 1] - r0, p0 = h_pos0[s];
      if (fused_decode && n == 1) continue;
      // the portion's keys: positions lo .. p0 + n - 1 (a window hides the positions before lo from every row of the portion)
      const int lo = win > 0 ? std::max(0, p0 - win + 1) : 0, ctx = p0 + n - lo, ctx_pad = (ctx + kpad - 1) / kpad * kpad;
      CKI(L.go(ssdk::latent_gather_kernel<T>, dim3(ctx_pad), dim3(128), 0, (const T*)pool, (T*)e->keys, (T*)e->lat_t, rg, s, lo, ctx, ctx_pad,
               KR, Wd));
      int qb = (int)std::max<size_t>(1, e->att_elems / ((size_t)H * ctx_pad));
      if (win > 0) qb = std::min(qb, window_block(win));   // short query blocks: a block's scores span its rows + the window
      for (int q0 = 0; q0 < n; q0 += qb) {
        // gathered keys kb .. kb + cb - 1 are what this block can see (whole pads, so that the operands stay aligned)
        const int nq = std::min(qb, n - q0), rows = nq * H, kb = win > 0 ? std::max(0, p0 + q0 - win + 1 - lo) / kpad * kpad : 0;
        const int cb = (p0 + q0 + nq - lo - kb + kpad - 1) / kpad * kpad;
        const T* qrows = (const T*)e->qcat + (size_t)(r0 + q0) * H * Wd;
        const T* krows = (const T*)e->keys + (size_t)kb * Wd;
        const T* lat_t = (const T*)e->lat_t + kb;
        // scores: keys are the 128-row operand, (query, head) rows the tokens
        CKI(lin(qrows, Wd, krows, Wd, e->att_s, cb, rows, cb, Wd, false, 1, 0, 0, 0, tc_attn));
        CKI(L.go(ssdk::sink_softmax_kernel<T>, dim3(rows), dim3(256), 0, (const float*)e->att_s, (T*)e->att_p,
                 (const T*)sink, H, cb, p0 + q0, c.attn_scale, rows, 0.f, lo + kb, win));
        T* o_rows = (T*)e->t0 + (size_t)(r0 + q0) * H * KR;
        if (tc_attn && tc_ok(e->att_p, cb, lat_t, ctx_pad, KR, KR, cb)) {
          // P C: the transposed latents [kv_rank, ctx_pad] are the 128-row operand, read with the row stride of the gather
          CKI(lin_tc(e->att_p, lat_t, e->att_o, rows, KR, cb, ctx_pad));
          CKI(L.go(ssdk::cast_cols_kernel<T>, dim3(rows), dim3(128), 0, (const float*)e->att_o, KR, o_rows, KR, KR));
        } else {
          CKI(lin(e->att_p, cb, lat_t, ctx_pad, o_rows, KR, rows, KR, cb, true, 1, 0, 0, 0, false));
        }
      }
    }
    // per-head value projection of the latent output, rounded to T for the output projection (after the sigmoid gate on
    // the concatenated heads, if the layer has one: the product stays fp32 up to the gate)
    if (gate) {
      CKI(lin(e->t0, H * KR, Lr.t[SSDK_HT_LAT_UV].p, KR, e->p1, H * V, M, V, KR, false, H, KR, (long long)V * KR, V));
      CKI(L.go(ssdk::attn_gate_kernel<T>, dim3(M), dim3(256), 0, (const float*)e->p1, gate, ldq, (T*)e->t1, M, H, 1, V));
    } else {
      CKI(lin(e->t0, H * KR, Lr.t[SSDK_HT_LAT_UV].p, KR, e->t1, H * V, M, V, KR, true, H, KR, (long long)V * KR, V));
    }
    return lin(e->t1, H * V, Lr.t[SSDK_HT_MIX_OUT].p, H * V, e->mix_out, W, M, W, H * V);
  }

  const void* fin = nullptr;   // the feed-forward's input in the storage type (the mixer's input, or the second norm's rows)

  // an expert's activation over `rows` rows of z [rows, ldz] -> y [rows, ff]: gated (z = gate | up columns) or not (z = up columns)
  int expert_act(const ssdk_hyb_layer_cfg& c, const float* z, int ldz, T* y, int ff, float limit, int rows, const int* n_rows) {
    const dim3 grid(rows), block(128);
    if (c.expert_glu) {
      if (c.expert_act == SSDK_ACT_SILU) return L.go(ssdk::glu_act_kernel<T, SSDK_ACT_SILU>, grid, block, 0, z, ldz, y, ff, n_rows);
      return L.go(ssdk::clamped_glu_kernel<T>, grid, block, 0, z, ldz, y, ff, limit, n_rows);
    }
    if (c.expert_act == SSDK_ACT_SILU) return L.go(ssdk::act_cols_kernel<T, SSDK_ACT_SILU>, grid, block, 0, z, ldz, y, ff, n_rows);
    if (c.expert_act == SSDK_ACT_GELU_TANH) return L.go(ssdk::act_cols_kernel<T, SSDK_ACT_GELU_TANH>, grid, block, 0, z, ldz, y, ff, n_rows);
    return L.go(ssdk::act_cols_kernel<T, SSDK_ACT_RELU2>, grid, block, 0, z, ldz, y, ff, n_rows);
  }

  int moe(HybLayer& Lr) {
    const ssdk_hyb_layer_cfg& c = Lr.c;
    const int W = e->cfg.width, E = c.experts, Et = E + c.identity, ff = c.ff, top = c.top, A = M * top;
    const int Nin = c.expert_glu ? 2 * ff : ff;   // rows of an expert's stacked input matrices
    CKI(check_tensor(Lr, SSDK_HT_ROUTER, Et, W, "router")); CKI(check_tensor(Lr, SSDK_HT_EXPERT_IN, (int64_t)E * Nin, W, "experts.in"));
    CKI(check_tensor(Lr, SSDK_HT_EXPERT_OUT, (int64_t)E * W, ff, "experts.out"));
    if (c.route_bias) CKI(check_tensor(Lr, SSDK_HT_ROUTER_BIAS, Et, 1, "router.bias"));
    CKI(lin(fin, W, Lr.t[SSDK_HT_ROUTER].p, W, e->rz, Et, M, Et, W));
    ssdk::RouterArgs ra;
    ra.z = e->rz; ra.bias = c.route_bias ? Lr.t[SSDK_HT_ROUTER_BIAS].p : nullptr; ra.sel = e->sel; ra.wts = e->wts; ra.M = M; ra.E = Et;
    ra.top = top; ra.groups = c.groups; ra.keep = c.keep; ra.softmax = c.route_top_softmax ? 2 : c.route_softmax; ra.group_best = c.group_best;
    ra.renorm = c.route_renorm; ra.route_scale = c.route_scale;
    CKI(L.go(ssdk::group_topk_router_kernel<T>, dim3((M + ssdk::kRouterWarps - 1) / ssdk::kRouterWarps), dim3(ssdk::kRouterWarps * 32), 0, ra));
    // many rows in bf16 with whole k-blocks: the grouped tcgen05 GEMM over rows gathered per expert (tiles of 128 rows);
    // else the mma.sync / FMA tile, which gathers by index itself (tiles of kLinBM rows)
    const bool tc_moe = !kF32 && e->use_tc && e->use_tc_experts && A >= 256 && W % kBlockK == 0 && ff % kBlockK == 0 &&
                        (((uintptr_t)Lr.t[SSDK_HT_EXPERT_IN].p | (uintptr_t)Lr.t[SSDK_HT_EXPERT_OUT].p) & 15) == 0;
    const int tile = tc_moe ? 128 : ssdk::kLinBM;
    ssdk::PlanArgs pa;
    pa.sel = e->sel; pa.apos = e->apos; pa.arow = e->arow; pa.tile_expert = e->tile_expert; pa.tile_row0 = e->tile_row0;
    pa.tile_rows = e->tile_rows; pa.n_tiles = e->n_tiles; pa.n_rows = e->n_rows; pa.A = A; pa.E = Et; pa.top = top; pa.tile = tile;
    pa.E_real = E;
    CKI(L.go(ssdk::expert_plan_kernel, dim3(1), dim3(1024), 0, pa));
    const int* n_real_rows = c.identity > 0 ? e->n_rows : nullptr;   // rows behind them belong to identity experts: nothing to compute
    ssdk::LinearArgs a = {};
    if (tc_moe) {
      CKI(L.go(ssdk::gather_rows_kernel<T>, dim3(A), dim3(128), 0, (const T*)fin, (const int*)e->arow, (const int*)e->n_rows, (T*)e->xs, W));
      CKI(lin_tc_grouped(e->xs, Lr.t[SSDK_HT_EXPERT_IN].p, e->eg, A, Nin, W, E, tile, A / tile + E + 1));
    } else {
      a.A = fin; a.W = Lr.t[SSDK_HT_EXPERT_IN].p; a.C = e->eg; a.M = A; a.N = Nin; a.K = W; a.lda = W; a.ldw = W; a.ldc = Nin;
      a.a_rows = e->arow; a.tile_expert = e->tile_expert; a.tile_row0 = e->tile_row0; a.tile_rows = e->tile_rows; a.n_tiles = e->n_tiles;
      a.sW_expert = (long long)Nin * W;
      CKI(lin_args<float>(a, A, 1));
    }
    CKI(expert_act(c, (const float*)e->eg, Nin, (T*)e->ey, ff, c.limit, A, n_real_rows));
    if (tc_moe) {
      CKI(lin_tc_grouped(e->ey, Lr.t[SSDK_HT_EXPERT_OUT].p, e->eo, A, W, ff, E, tile, A / tile + E + 1));
    } else {
      a.A = e->ey; a.W = Lr.t[SSDK_HT_EXPERT_OUT].p; a.C = e->eo; a.N = W; a.K = ff; a.lda = ff; a.ldw = ff; a.ldc = W; a.a_rows = nullptr;
      a.tile_expert = e->tile_expert; a.tile_row0 = e->tile_row0; a.tile_rows = e->tile_rows; a.n_tiles = e->n_tiles;
      a.M = A; a.sW_expert = (long long)W * ff;
      CKI(lin_args<float>(a, A, 1));
    }
    if (c.shared_ff > 0) {
      const int sff = c.shared_ff, Ns = (c.expert_glu ? 2 : 1) * sff + (c.shared_gate ? 1 : 0);
      CKI(check_tensor(Lr, SSDK_HT_SHARED_IN, Ns, W, "shared.in")); CKI(check_tensor(Lr, SSDK_HT_SHARED_OUT, W, sff, "shared.out"));
      CKI(lin(fin, W, Lr.t[SSDK_HT_SHARED_IN].p, W, e->sz, Ns, M, Ns, W));
      CKI(expert_act(c, (const float*)e->sz, Ns, (T*)e->sy, sff, c.shared_limit, M, (const int*)nullptr));
      CKI(lin(e->sy, sff, Lr.t[SSDK_HT_SHARED_OUT].p, sff, e->so, W, M, W, sff));
    }
    return 0;
  }

  // dense feed-forward without a gate: so = W_down act(W_up h + b_up); b_down joins in the block's combine
  int ffn(HybLayer& Lr) {
    const int W = e->cfg.width, ff = Lr.c.ff;
    CKI(check_tensor(Lr, SSDK_HT_FFN_IN, ff, W, "mlp.up")); CKI(check_tensor(Lr, SSDK_HT_FFN_OUT, W, ff, "mlp.down"));
    const T* b_up = (const T*)Lr.t[SSDK_HT_FFN_IN_B].p;
    if (b_up) CKI(check_tensor(Lr, SSDK_HT_FFN_IN_B, ff, 1, "mlp.up.b"));
    if (Lr.t[SSDK_HT_FFN_OUT_B].p) CKI(check_tensor(Lr, SSDK_HT_FFN_OUT_B, W, 1, "mlp.down.b"));
    CKI(lin(fin, W, Lr.t[SSDK_HT_FFN_IN].p, W, e->sz, ff, M, ff, W));
    const dim3 grid(M), block(256);
    if (Lr.c.ff_act == SSDK_ACT_POLYNORM) {
      if (b_up) return fail("the PolyNorm feed-forward has no input bias");
      CKI(check_tensor(Lr, SSDK_HT_FFN_ACT, 4, 1, "mlp.act"));
      CKI(L.go(ssdk::polynorm_kernel<T>, grid, block, 0, (const float*)e->sz, (const T*)Lr.t[SSDK_HT_FFN_ACT].p, (T*)e->sy, ff, e->cfg.eps));
    } else if (Lr.c.ff_act == SSDK_ACT_RELU2) CKI(L.go(ssdk::bias_act_kernel<T, SSDK_ACT_RELU2>, grid, block, 0, (const float*)e->sz, b_up, (T*)e->sy, ff));
    else if (Lr.c.ff_act == SSDK_ACT_SILU) CKI(L.go(ssdk::bias_act_kernel<T, SSDK_ACT_SILU>, grid, block, 0, (const float*)e->sz, b_up, (T*)e->sy, ff));
    else CKI(L.go(ssdk::bias_act_kernel<T, SSDK_ACT_GELU_TANH>, grid, block, 0, (const float*)e->sz, b_up, (T*)e->sy, ff));
    return lin(e->sy, ff, Lr.t[SSDK_HT_FFN_OUT].p, ff, e->so, W, M, W, ff);
  }

  // ---- mixers of the serial post-norm designs (usable in either block kind: they read `hin`) ----
  const void* hin = nullptr;   // the sublayer's input in the storage type: normed rows (parallel blocks) or x itself
  static constexpr bool kF32 = std::is_same<T, float>::value;
  const T* w_at(const HybTensor& t, size_t off) const { return (const T*)t.p + off; }

  int glu(HybLayer& Lr) {
    const int W = e->cfg.width, ff = Lr.c.ff;
    CKI(check_tensor(Lr, SSDK_HT_GLU_IN, 2 * ff, W, "mlp.gate|up")); CKI(check_tensor(Lr, SSDK_HT_GLU_OUT, W, ff, "mlp.down"));
    CKI(lin(hin, W, Lr.t[SSDK_HT_GLU_IN].p, W, e->p0, 2 * ff, M, 2 * ff, W));
    CKI(L.go(ssdk::glu_act_kernel<T, SSDK_ACT_GELU_TANH>, dim3(M), dim3(256), 0, (const float*)e->p0, 2 * ff, (T*)e->t0, ff, (const int*)nullptr));
    return lin(e->t0, ff, Lr.t[SSDK_HT_GLU_OUT].p, ff, e->mix_out, W, M, W, ff);
  }

  int rglru(HybLayer& Lr) {
    const ssdk_hyb_layer_cfg& c = Lr.c;
    const int W = e->cfg.width, R = c.inner, nb = c.blocks, bs = R / nb, taps = c.conv;
    CKI(check_tensor(Lr, SSDK_HT_RGLRU_IN, 2 * R, W, "rglru.y|x")); CKI(check_tensor(Lr, SSDK_HT_RGLRU_IN_B, 2 * R, 1, "rglru.y.b|x.b"));
    CKI(check_tensor(Lr, SSDK_HT_CONV_W, R, taps, "conv")); CKI(check_tensor(Lr, SSDK_HT_CONV_B, R, 1, "conv.b"));
    CKI(check_tensor(Lr, SSDK_HT_RGLRU_GATE, (int64_t)nb * 2 * bs, bs, "rglru.ra|ri"));
    CKI(check_tensor(Lr, SSDK_HT_RGLRU_GATE_B, (int64_t)nb * 2 * bs, 1, "rglru.ra.b|ri.b"));
    CKI(check_tensor(Lr, SSDK_HT_RGLRU_LAM, R, 1, "rglru.lam")); CKI(check_tensor(Lr, SSDK_HT_MIX_OUT, W, R, "mix.o"));
    CKI(lin(hin, W, Lr.t[SSDK_HT_RGLRU_IN].p, W, e->p0, 2 * R, M, 2 * R, W));   // y pre-activations | x branch
    float* st = e->state + Lr.state_off;
    ssdk::ConvArgs ca = {};
    ca.in = e->p0 + R; ca.ld_in = 2 * R; ca.in_bias = w_at(Lr.t[SSDK_HT_RGLRU_IN_B], R); ca.w = Lr.t[SSDK_HT_CONV_W].p;
    ca.bias = Lr.t[SSDK_HT_CONV_B].p; ca.out = e->p1; ca.ld_out = R; ca.out_t = kF32 ? nullptr : e->t0; ca.ld_t = R;
    ca.hist = st + R; ca.slot_stride = e->slot_floats; ca.C = R; ca.taps = taps;
    const dim3 cgrid(M, (R + 255) / 256), sgrid(rg.n_seqs, (R + 255) / 256);
    CKI(L.go(ssdk::short_conv_kernel<T, 0>, cgrid, dim3(256), 0, ca, rg));
    CKI(L.go(ssdk::conv_state_kernel<T>, sgrid, dim3(256), 0, ca, rg));
    // block-diagonal gates: per block one [2 bs, bs] product, all blocks in one batched launch
    const void* u_t = kF32 ? (const void*)e->p1 : (const void*)e->t0;
    CKI(lin(u_t, R, Lr.t[SSDK_HT_RGLRU_GATE].p, bs, e->p2, 2 * R, M, 2 * bs, bs, false, nb, bs, 2LL * bs * bs, 2 * bs));
    ssdk::RglruArgs a;
    a.u = e->p1; a.ld_u = R; a.gates = e->p2; a.ld_g = 2 * R; a.gate_bias = Lr.t[SSDK_HT_RGLRU_GATE_B].p; a.lam = Lr.t[SSDK_HT_RGLRU_LAM].p;
    a.y = e->p0; a.ld_y = 2 * R; a.y_bias = Lr.t[SSDK_HT_RGLRU_IN_B].p; a.out = e->t1; a.S = st; a.slot_stride = e->slot_floats;
    a.R = R; a.bs = bs; a.decay_mult = c.decay_mult;
    CKI(L.go(ssdk::rglru_gate_kernel<T>, dim3(M, (R + 255) / 256), dim3(256), 0, a, e->p2, e->p0));
    const int rt = rg.n_seqs * ((R + 127) / 128) >= num_sms() ? 128 : 32;  // few sequences: one warp per CTA spreads the channels over the SMs
    CKI(L.go(ssdk::rglru_scan_kernel<T>, dim3(rg.n_seqs, (R + rt - 1) / rt), dim3(rt), 0, a, rg));
    return lin(e->t1, R, Lr.t[SSDK_HT_MIX_OUT].p, R, e->mix_out, W, M, W, R);
  }

  int selective(HybLayer& Lr) {
    const ssdk_hyb_layer_cfg& c = Lr.c;
    const int W = e->cfg.width, I = c.inner, N = c.state, Rk = c.dt_rank, taps = c.conv, Nx = Rk + 2 * N;
    CKI(check_tensor(Lr, SSDK_HT_SEL_IN, 2 * I, W, "mamba.in")); CKI(check_tensor(Lr, SSDK_HT_CONV_W, I, taps, "conv"));
    CKI(check_tensor(Lr, SSDK_HT_CONV_B, I, 1, "conv.b")); CKI(check_tensor(Lr, SSDK_HT_SEL_X, Nx, I, "mamba.x"));
    CKI(check_tensor(Lr, SSDK_HT_SEL_DT, I, Rk, "mamba.dt")); CKI(check_tensor(Lr, SSDK_HT_SEL_DT_B, I, 1, "mamba.dt.b"));
    CKI(check_tensor(Lr, SSDK_HT_SEL_ALOG, I, N, "mamba.A_log")); CKI(check_tensor(Lr, SSDK_HT_SEL_D, I, 1, "mamba.D"));
    CKI(check_tensor(Lr, SSDK_HT_MIX_OUT, W, I, "mix.o"));
    CKI(lin(hin, W, Lr.t[SSDK_HT_SEL_IN].p, W, e->p0, 2 * I, M, 2 * I, W));   // x | z
    float* st = e->state + Lr.state_off;
    ssdk::ConvArgs ca = {};
    ca.in = e->p0; ca.ld_in = 2 * I; ca.w = Lr.t[SSDK_HT_CONV_W].p; ca.bias = Lr.t[SSDK_HT_CONV_B].p; ca.out = e->p1; ca.ld_out = I;
    ca.out_t = kF32 ? nullptr : e->t0; ca.ld_t = I; ca.hist = st + (size_t)I * N; ca.slot_stride = e->slot_floats; ca.C = I; ca.taps = taps;
    CKI(L.go(ssdk::short_conv_kernel<T, 1>, dim3(M, (I + 255) / 256), dim3(256), 0, ca, rg));
    CKI(L.go(ssdk::conv_state_kernel<T>, dim3(rg.n_seqs, (I + 255) / 256), dim3(256), 0, ca, rg));
    const void* x_t = kF32 ? (const void*)e->p1 : (const void*)e->t0;
    CKI(lin(x_t, I, Lr.t[SSDK_HT_SEL_X].p, I, e->p2, Nx, M, Nx, I));          // dt (low rank) | B | C
    float* dtz = e->p2 + (size_t)M * Nx;
    if (kF32) {
      CKI(lin(e->p2, Nx, Lr.t[SSDK_HT_SEL_DT].p, Rk, dtz, I, M, I, Rk));
    } else {
      CKI(L.go(ssdk::cast_cols_kernel<T>, dim3(M), dim3(128), 0, (const float*)e->p2, Nx, (T*)e->t1, Rk, Rk));
      CKI(lin(e->t1, Rk, Lr.t[SSDK_HT_SEL_DT].p, Rk, dtz, I, M, I, Rk));
    }
    ssdk::SelScanArgs a;
    a.x = e->p1; a.ld_x = I; a.dtz = dtz; a.ld_dt = I; a.bc = e->p2 + Rk; a.ld_bc = Nx;
    a.A_log = Lr.t[SSDK_HT_SEL_ALOG].p; a.Dw = Lr.t[SSDK_HT_SEL_D].p; a.z = e->p0 + I; a.ld_z = 2 * I; a.out = e->t1;
    a.S = st; a.slot_stride = e->slot_floats; a.inner = I; a.N = N;
    const size_t smem = (size_t)ssdk::kSelRows * 2 * N * 4;
    CKI(L.go(ssdk::selective_gate_kernel<T>, dim3(M, (I + 255) / 256), dim3(256), 0, dtz, I, (const T*)Lr.t[SSDK_HT_SEL_DT_B].p, e->p0 + I, 2 * I, I));
    if (N <= 128) {
      // NT states per lane, the lanes of a channel side by side in one warp: the fewest lanes that still give every SM
      // eight warps (a long prompt of one sequence), never more than a warp per channel
      int nt = 4;
      auto lanes = [&](int t) { int l = 1; while (l * t < N) l *= 2; return l; };
      while (nt > 1 && (lanes(nt) > 32 || (long long)rg.n_seqs * I * lanes(nt) / 32 < 8LL * num_sms()) && lanes(nt / 2) <= 32) nt /= 2;
      if (lanes(nt) > 32) nt = 4;
      const int lpc = lanes(nt), cpb = 128 / lpc;
      const dim3 grid(rg.n_seqs, (I + cpb - 1) / cpb), block(lpc, cpb);
      if (nt == 4) CKI(L.go(ssdk::selective_scan_kernel<T, 4>, grid, block, smem, a, rg));
      else if (nt == 2) CKI(L.go(ssdk::selective_scan_kernel<T, 2>, grid, block, smem, a, rg));
      else CKI(L.go(ssdk::selective_scan_kernel<T, 1>, grid, block, smem, a, rg));
    } else {
      CKI(L.go(ssdk::selective_scan_kernel<T, 0>, dim3(rg.n_seqs, (I + 127) / 128), dim3(1, 128), smem, a, rg));
    }
    return lin(e->t1, I, Lr.t[SSDK_HT_MIX_OUT].p, I, e->mix_out, W, M, W, I);
  }

  // grouped-query sink attention over the layer's page pool: z holds q | k | v (fp32); og [G, M, H/G, V] fp32
  int gqa_attention(HybLayer& Lr, const float* z, int ldz, float* og, const void* sinks = nullptr) {
    const ssdk_hyb_layer_cfg& c = Lr.c;
    const int H = c.heads, G = c.kv_heads, D = c.dim, V = c.vdim, hpg = H / G, win = c.window;
    const float sink_const = sinks ? 0.f : c.sink;
    if (!e->cache) return fail("hybrid: attention cache not bound");
    uint8_t* pool = e->cache + (size_t)e->num_blocks * e->cfg.block_size * Lr.cache_rows_before * e->esz;
    ssdk::GqaPrepArgs pa;
    pa.z = z; pa.ldz = ldz; pa.q = e->qcat; pa.cache = pool; pa.inv_freq = c.rot_dims >= 2 ? Lr.inv_freq : nullptr;
    pa.H = H; pa.G = G; pa.D = D; pa.V = V; pa.rot_dims = c.rot_dims; pa.qk_norm = c.qk_norm; pa.rot_mult = Lr.rot_mult; pa.eps = e->cfg.eps;
    pa.rot_half = c.rot_half;
    CKI(L.go(ssdk::gqa_prep_kernel<T>, dim3(M, H + G), dim3(32), 0, pa, rg));
    bool fused_decode = false;
    {
      int n_dec = 0, ctx_max = 0;
      for (int s = 0; s < rg.n_seqs; ++s)
        if (h_cu[s + 1] - h_cu[s] == 1) { ++n_dec; ctx_max = std::max(ctx_max, h_pos0[s] + 1); }
      if (win > 0) ctx_max = std::min(ctx_max, win);
      const int vpl = (V + 31) / 32;
      if (n_dec > 0 && vpl <= 8 && e->use_decode_attn) {
        int splits = std::max(1, std::min({32, 8 * num_sms() / std::max(1, n_dec * H), (ctx_max + 127) / 128}));  // ~8 four-warp CTAs per SM
        const size_t per_split = (size_t)rg.n_seqs * H * (V + 2);
        splits = (int)std::min<size_t>(splits, e->att_elems / per_split);
        if (splits >= 1) {
          ssdk::GqaDecodeArgs da;
          da.q = e->qcat; da.cache = pool; da.part = e->att_s; da.out = og; da.H = H; da.G = G; da.D = D; da.V = V; da.splits = splits;
          da.scale = c.attn_scale; da.sink = sink_const; da.sinks = sinks; da.window = win;
          const dim3 grid(rg.n_seqs, H, splits), block(ssdk::kGqaDecWarps * 32);
          const size_t smem = ssdk::gqa_decode_smem(D, V);
          if (vpl <= 1) CKI(L.go(ssdk::gqa_decode_partial_kernel<T, 1>, grid, block, smem, da, rg));
          else if (vpl <= 2) CKI(L.go(ssdk::gqa_decode_partial_kernel<T, 2>, grid, block, smem, da, rg));
          else if (vpl <= 4) CKI(L.go(ssdk::gqa_decode_partial_kernel<T, 4>, grid, block, smem, da, rg));
          else CKI(L.go(ssdk::gqa_decode_partial_kernel<T, 8>, grid, block, smem, da, rg));
          CKI(L.go(ssdk::gqa_decode_merge_kernel<T>, dim3(rg.n_seqs, H), dim3(64), 0, da, rg));
          fused_decode = true;
        }
      }
    }
    for (int s = 0; s < rg.n_seqs; ++s) {
      const int r0 = h_cu[s], n = h_cu[s + 1] - r0, p0 = h_pos0[s];
      if (fused_decode && n == 1) continue;
      const int lo = win > 0 ? std::max(0, p0 - win + 1) : 0, ctx = p0 + n - lo, ctx_pad = (ctx + 7) / 8 * 8;   // keys lo .. p0 + n - 1
      CKI(L.go(ssdk::kv_gather_kernel<T>, dim3(ctx_pad), dim3(128), 0, (const T*)pool, (T*)e->keys, (T*)e->lat_t, rg, s, lo, ctx, ctx_pad, G, D, V));
      int qb = (int)std::max<size_t>(1, e->att_elems / ((size_t)H * ctx_pad));
      if (win > 0) qb = std::min(qb, window_block(win));
      for (int q0 = 0; q0 < n; q0 += qb) {
        const int nq = std::min(qb, n - q0), rows = nq * hpg, kb = win > 0 ? std::max(0, p0 + q0 - win + 1 - lo) / 8 * 8 : 0;
        const int cb = (p0 + q0 + nq - lo - kb + 7) / 8 * 8;   // gathered keys kb .. kb + cb - 1 are what this block can see
        const T* qrows = (const T*)e->qcat + (size_t)(r0 + q0) * hpg * D;
        CKI(lin(qrows, D, (const T*)e->keys + (size_t)kb * D, D, e->att_s, cb, rows, cb, D, false, G, (long long)M * hpg * D, (long long)ctx_pad * D,
                (long long)rows * cb, false));
        CKI(L.go(ssdk::sink_softmax_kernel<T>, dim3(G * rows), dim3(256), 0, (const float*)e->att_s, (T*)e->att_p, (const T*)sinks, hpg, cb,
                 p0 + q0, c.attn_scale, rows, sink_const, lo + kb, win));
        CKI(lin(e->att_p, cb, (const T*)e->lat_t + kb, ctx_pad, og + (size_t)(r0 + q0) * hpg * V, V, rows, V, cb, false, G, (long long)rows * cb,
                (long long)V * ctx_pad, (long long)M * hpg * V, false));
      }
    }
    return 0;
  }

  // grouped-query attention alone: stacked q | k | v projection, its bias, a short convolution over time on every channel
  // (history in the state slot), rotation, window, learned sink, output projection
  int attention(HybLayer& Lr) {
    const ssdk_hyb_layer_cfg& c = Lr.c;
    const int W = e->cfg.width, H = c.heads, G = c.kv_heads, D = c.dim, V = c.vdim, taps = c.conv, Nqkv = H * D + G * D + G * V;
    CKI(check_tensor(Lr, SSDK_HT_ATTN_IN, Nqkv, W, "attention.in")); CKI(check_tensor(Lr, SSDK_HT_CONV_W, Nqkv, taps, "attention.conv"));
    CKI(check_tensor(Lr, SSDK_HT_MIX_OUT, W, (int64_t)H * V, "mix.o"));
    if (Lr.t[SSDK_HT_ATTN_IN_B].p) CKI(check_tensor(Lr, SSDK_HT_ATTN_IN_B, Nqkv, 1, "attention.in.b"));
    if (c.learned_sink) CKI(check_tensor(Lr, SSDK_HT_ATTN_SINK, H, 1, "sink"));
    CKI(lin(hin, W, Lr.t[SSDK_HT_ATTN_IN].p, W, e->p0, Nqkv, M, Nqkv, W));
    ssdk::ConvArgs ca = {};
    ca.in = e->p0; ca.ld_in = Nqkv; ca.in_bias = Lr.t[SSDK_HT_ATTN_IN_B].p; ca.w = Lr.t[SSDK_HT_CONV_W].p; ca.out = e->p1; ca.ld_out = Nqkv;
    ca.hist = e->state + Lr.state_off; ca.slot_stride = e->slot_floats; ca.C = Nqkv; ca.taps = taps;
    CKI(L.go(ssdk::short_conv_kernel<T, 0>, dim3(M, (Nqkv + 255) / 256), dim3(256), 0, ca, rg));
    if (taps > 1) CKI(L.go(ssdk::conv_state_kernel<T>, dim3(rg.n_seqs, (Nqkv + 255) / 256), dim3(256), 0, ca, rg));
    CKI(gqa_attention(Lr, e->p1, Nqkv, e->p2, c.learned_sink ? Lr.t[SSDK_HT_ATTN_SINK].p : nullptr));
    CKI(L.go(ssdk::attn_gate_kernel<T>, dim3(M), dim3(256), 0, (const float*)e->p2, (const float*)nullptr, 0, (T*)e->t0, M, H, G, V));
    return lin(e->t0, H * V, Lr.t[SSDK_HT_MIX_OUT].p, H * V, e->mix_out, W, M, W, H * V);
  }

  int attn_delta(HybLayer& Lr) {
    const ssdk_hyb_layer_cfg& c = Lr.c;
    const int W = e->cfg.width, H = c.heads, G = c.kv_heads, D = c.dim, V = c.vdim, taps = c.conv;
    const int Hd = c.d_heads, Gd = c.d_kv_heads, Dd = c.d_dim, Vd = c.d_vdim;
    const int HV = H * V, dGD = Gd * Dd, dHV = Hd * Vd, Cd = 2 * dGD + dHV;
    const int o_g = H * D + G * D + G * V, o_dq = o_g + HV, o_dg = o_dq + Cd, o_b = o_dg + dHV, Ntot = o_b + 2 * Hd;
    CKI(check_tensor(Lr, SSDK_HT_PAIR_IN, Ntot, W, "pair.in")); CKI(check_tensor(Lr, SSDK_HT_ATTN_OUT, W, HV, "left.o"));
    CKI(check_tensor(Lr, SSDK_HT_MIX_OUT, W, dHV, "right.o")); CKI(check_tensor(Lr, SSDK_HT_CONV_W, Cd, taps, "right.conv"));
    CKI(check_tensor(Lr, SSDK_HT_DELTA_ALOG, Hd, 1, "right.A_log")); CKI(check_tensor(Lr, SSDK_HT_DELTA_DT_B, Hd, 1, "right.dt_bias"));
    CKI(check_tensor(Lr, SSDK_HT_MIX_NORM, dHV, 1, "right.norm"));
    CKI(lin(hin, W, Lr.t[SSDK_HT_PAIR_IN].p, W, e->p0, Ntot, M, Ntot, W));
    // left: attention
    CKI(gqa_attention(Lr, e->p0, Ntot, e->p1));
    CKI(L.go(ssdk::attn_gate_kernel<T>, dim3(M), dim3(256), 0, (const float*)e->p1, (const float*)(e->p0 + o_g), Ntot, (T*)e->t0, M, H, G, V));
    CKI(lin(e->t0, HV, Lr.t[SSDK_HT_ATTN_OUT].p, HV, e->mix_out, W, M, W, HV));
    // right: gated delta rule
    float* st = e->state + Lr.state_off;
    ssdk::DeltaPrepArgs dp = {};
    dp.conv.in = e->p0 + o_dq; dp.conv.ld_in = Ntot; dp.conv.w = Lr.t[SSDK_HT_CONV_W].p; dp.conv.hist = st + (size_t)Hd * Dd * Vd;
    dp.conv.slot_stride = e->slot_floats; dp.conv.C = Cd; dp.conv.taps = taps;
    dp.ba = e->p0 + o_b; dp.ld_ba = Ntot; dp.A_log = Lr.t[SSDK_HT_DELTA_ALOG].p; dp.dt_bias = Lr.t[SSDK_HT_DELTA_DT_B].p;
    dp.q = e->p2; dp.k = dp.q + (size_t)M * dGD; dp.v = dp.k + (size_t)M * dGD; dp.beta = dp.v + (size_t)M * dHV; dp.decay = dp.beta + (size_t)M * Hd;
    dp.H = Hd; dp.G = Gd; dp.D = Dd; dp.V = Vd; dp.q_scale = 1.0f / sqrtf((float)Dd); dp.unit_eps = 1e-6f;
    CKI(L.go(ssdk::delta_prep_kernel<T>, dim3(M, 2 * Gd + Hd), dim3(std::min(256, (std::max(Dd, Vd) + 31) / 32 * 32)),
             (size_t)std::max(Dd, Vd) * 4, dp, rg));
    CKI(L.go(ssdk::conv_state_kernel<T>, dim3(rg.n_seqs, (Cd + 255) / 256), dim3(256), 0, dp.conv, rg));
    ssdk::DeltaArgs da;
    da.q = dp.q; da.k = dp.k; da.v = dp.v; da.beta = dp.beta; da.decay = dp.decay; da.o = e->p1; da.S = st; da.slot_stride = e->slot_floats;
    da.H = Hd; da.G = Gd; da.D = Dd; da.V = Vd;
    const int Vall = (Vd + 31) / 32 * 32;
    int Vr = Vall, DR = 0, NG = 1;
    delta_shape(Dd, Vr, &DR, &NG);
    // the state's columns are independent: few (sequence, head) pairs spread a head's columns over several CTAs
    while (DR > 0 && Vr % 64 == 0 && rg.n_seqs * Hd * (Vall / Vr) < num_sms()) {
      Vr /= 2;
      delta_shape(Dd, Vr, &DR, &NG);
    }
    const dim3 grid(rg.n_seqs, Hd, (Vall + Vr - 1) / Vr), block(Vr, NG);
    const size_t smem = ssdk::delta_scan_smem(Dd, Vr, DR, NG);
    if (DR == 16) CKI(L.go(ssdk::delta_scan_kernel<16>, grid, block, smem, da, rg));
    else if (DR == 32) CKI(L.go(ssdk::delta_scan_kernel<32>, grid, block, smem, da, rg));
    else if (DR == 64) CKI(L.go(ssdk::delta_scan_kernel<64>, grid, block, smem, da, rg));
    else CKI(L.go(ssdk::delta_scan_kernel<0>, grid, block, smem, da, rg));
    CKI(L.go(ssdk::head_rmsnorm_gate_kernel<T, 0>, dim3(M, Hd), dim3(std::min(256, Vall)), 0, (const float*)e->p1, (const float*)(e->p0 + o_dg), Ntot,
             (const T*)Lr.t[SSDK_HT_MIX_NORM].p, (T*)e->t1, Hd, Vd, e->cfg.eps));
    return lin(e->t1, dHV, Lr.t[SSDK_HT_MIX_OUT].p, dHV, e->mix2, W, M, W, dHV);
  }

  int run_mixer(HybLayer& Lr) {
    switch (Lr.c.mixer) {
      case SSDK_MIX_WKV: return wkv(Lr);
      case SSDK_MIX_MLSTM: return mlstm(Lr);
      case SSDK_MIX_LATENT_ATTN: return latent(Lr);
      case SSDK_MIX_RGLRU: return rglru(Lr);
      case SSDK_MIX_SELECTIVE: return selective(Lr);
      case SSDK_MIX_ATTENTION: return attention(Lr);
      default: return attn_delta(Lr);
    }
  }

  // x += m * norm1(mixer(x)); x += m * norm2(ff(x)): both sublayers read the residual stream itself
  int serial_layer(HybLayer& Lr) {
    const ssdk_hyb_cfg& g = e->cfg;
    const int W = g.width;
    T* xt = kF32 ? nullptr : (T*)e->h;
    hin = kF32 ? (const void*)e->x : (const void*)e->h;
    CKI(check_tensor(Lr, SSDK_HT_NORM, W, 1, "norm1"));
    if (Lr.c.mixer == SSDK_MIX_WKV || Lr.c.mixer == SSDK_MIX_MLSTM || Lr.c.mixer == SSDK_MIX_LATENT_ATTN)
      return fail("wkv, mlstm and latent attention are built for parallel blocks");
    CKI(run_mixer(Lr));
    const bool pair = Lr.c.mixer == SSDK_MIX_ATTN_DELTA;
    CKI(L.go(ssdk::postnorm_residual_kernel<T>, dim3(M), dim3(256), 0, e->x, (const float*)e->mix_out, pair ? Lr.c.left_scale : 1.0f,
             (const float*)(pair ? e->mix2 : nullptr), pair ? Lr.c.right_scale : 0.f, (const T*)Lr.t[SSDK_HT_NORM].p, W, g.eps, g.norm_offset,
             g.residual_mult, xt));
    if (Lr.c.mlp == SSDK_MLP_GLU) {
      CKI(check_tensor(Lr, SSDK_HT_NORM2, W, 1, "norm2"));
      CKI(glu(Lr));
      CKI(L.go(ssdk::postnorm_residual_kernel<T>, dim3(M), dim3(256), 0, e->x, (const float*)e->mix_out, 1.0f, (const float*)nullptr, 0.f,
               (const T*)Lr.t[SSDK_HT_NORM2].p, W, g.eps, g.norm_offset, g.residual_mult, xt));
    }
    return 0;
  }

  int layer(HybLayer& Lr, int li) {
    if (e->cfg.block == SSDK_BLOCK_SERIAL_POSTNORM) return serial_layer(Lr);
    const int W = e->cfg.width;
    const bool two = e->cfg.block == SSDK_BLOCK_PARALLEL_TWO_NORMS;   // norm1 feeds the mixer, norm2 the feed-forward; no layer scales
    const bool one = e->cfg.block == SSDK_BLOCK_PARALLEL_ONE_NORM;    // one norm; input convolutions and residual gates; no layer scales
    const bool scales = !two && !one;
    const bool ff2 = two && Lr.c.mlp != SSDK_MLP_NONE;
    hin = e->h;
    fin = ff2 ? e->h2 : e->h;
    CKI(check_tensor(Lr, SSDK_HT_NORM, W, 1, "norm1"));
    if (scales) CKI(check_tensor(Lr, SSDK_HT_LS_MIX, W, 1, "ls1"));
    if (ff2) CKI(check_tensor(Lr, SSDK_HT_NORM2, W, 1, "norm2"));
    CKI(L.go(ssdk::offset_rmsnorm_kernel<T>, dim3(M), dim3(256), 0, (const float*)e->x, (const T*)Lr.t[SSDK_HT_NORM].p, (T*)e->h,
             (const int*)nullptr, W, e->cfg.eps, e->cfg.norm_offset, ff2 ? (const T*)Lr.t[SSDK_HT_NORM2].p : (const T*)nullptr,
             ff2 ? (T*)e->h2 : (T*)nullptr));
    ssdk::CombineArgs ca = {};
    if (one) {
      const bool has_ff = Lr.c.mlp != SSDK_MLP_NONE;
      const int taps = e->cfg.canon_taps, sub = has_ff ? 2 : 1;   // sublayers that have an input convolution and a gate
      if (taps > 0) {
        // each sublayer reads h + conv(h) with its own taps; the last taps - 1 rows of h live in the state slot
        CKI(check_tensor(Lr, SSDK_HT_CANON_W, (int64_t)sub * W, taps, "canon"));
        ssdk::InputConvArgs ia;
        ia.h = e->h; ia.w = Lr.t[SSDK_HT_CANON_W].p; ia.y1 = e->hc; ia.y2 = has_ff ? e->h2 : nullptr;
        ia.hist = e->state + Lr.canon_off; ia.slot_stride = e->slot_floats; ia.C = W; ia.taps = taps;
        // 16 bytes of channels per thread when rows, taps and history rows start on 16-byte boundaries (2 .. 4 taps)
        constexpr int kVec = 16 / (int)sizeof(T);
        const bool vec = W % kVec == 0 && taps >= 2 && taps <= 4 && (((uintptr_t)ia.h | (uintptr_t)ia.w | (uintptr_t)ia.y1 | (uintptr_t)ia.y2) & 15) == 0 &&
                         ((uintptr_t)ia.hist & 15) == 0 && e->slot_floats % 4 == 0 && W % 4 == 0;
        const dim3 vgrid(M, (W / kVec + 127) / 128), vblock(128);
        if (vec && taps == 4) CKI(L.go(ssdk::input_conv_vec_kernel<T, 4>, vgrid, vblock, 0, ia, rg));
        else if (vec && taps == 3) CKI(L.go(ssdk::input_conv_vec_kernel<T, 3>, vgrid, vblock, 0, ia, rg));
        else if (vec && taps == 2) CKI(L.go(ssdk::input_conv_vec_kernel<T, 2>, vgrid, vblock, 0, ia, rg));
        else CKI(L.go(ssdk::input_conv_kernel<T>, dim3(M, (W + 255) / 256), dim3(256), 0, ia, rg));
        if (taps > 1) CKI(L.go(ssdk::input_conv_state_kernel<T>, dim3(rg.n_seqs, (W + 255) / 256), dim3(256), 0, ia, rg));
        hin = e->hc;
        fin = e->h2;
      }
      if (e->cfg.gated_residual) {
        // the gates read the normed rows themselves (before the input convolutions): one stacked product for both sublayers
        CKI(check_tensor(Lr, SSDK_HT_RES_GATE, (int64_t)sub * W, W, "residual gates")); CKI(check_tensor(Lr, SSDK_HT_RES_GATE_B, (int64_t)sub * W, 1, "residual gates' bias"));
        CKI(lin(e->h, W, Lr.t[SSDK_HT_RES_GATE].p, W, e->gz, sub * W, M, sub * W, W));
        ca.gz = e->gz; ca.ld_gz = sub * W; ca.gz_bias = Lr.t[SSDK_HT_RES_GATE_B].p;
      }
    }
    if (Lr.c.mixer == SSDK_MIX_ATTN_DELTA) return fail("the attention pair is built for serial blocks");
    if (Lr.c.mixer == SSDK_MIX_ATTENTION && !one) return fail("the attention mixer is built for one-norm blocks");
    CKI(run_mixer(Lr));
    ca.x = e->x; ca.mix = e->mix_out; ca.ls1 = scales ? Lr.t[SSDK_HT_LS_MIX].p : nullptr; ca.width = W;
    if (Lr.c.mlp == SSDK_MLP_MOE) {
      if (scales) CKI(check_tensor(Lr, SSDK_HT_LS_MLP, W, 1, "ls2"));
      CKI(moe(Lr));
      ca.ls2 = scales ? Lr.t[SSDK_HT_LS_MLP].p : nullptr; ca.routed = e->eo; ca.apos = e->apos; ca.wts = e->wts; ca.top = Lr.c.top;
      if (Lr.c.identity > 0) { ca.sel = e->sel; ca.n_real = Lr.c.experts; ca.fin = fin; }
      if (Lr.c.shared_ff > 0) {
        ca.shared = e->so;
        const int ld = (Lr.c.expert_glu ? 2 : 1) * Lr.c.shared_ff;
        if (Lr.c.shared_gate) { ca.sg = e->sz + ld; ca.ld_sg = ld + 1; }
      }
    } else if (Lr.c.mlp == SSDK_MLP_FFN) {
      CKI(ffn(Lr));
      ca.shared = e->so; ca.ff_bias = Lr.t[SSDK_HT_FFN_OUT_B].p;
    } else if (Lr.c.mlp != SSDK_MLP_NONE) {
      return fail("the gated dense feed-forward is built for serial blocks");
    }
    return L.go(ssdk::block_combine_kernel<T>, dim3(M), dim3(256), 0, ca);
  }
};

static int hyb_smem_attrs(ssdk_hyb_engine* e) {
  if (e->smem_attr_done) return 0;
  const int big = 200 * 1024;
  CK(cudaFuncSetAttribute(ssdk::wkv_scan_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, big));
  CK(cudaFuncSetAttribute(ssdk::wkv_scan_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, big));
  CK(cudaFuncSetAttribute(ssdk::mlstm_scan_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, big));
  CK(cudaFuncSetAttribute(ssdk::mlstm_scan_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, big));
#define SSDK_SCAN_ATTR(DG) \
  CK(cudaFuncSetAttribute(ssdk::wkv_scan_reg_kernel<bf16, DG>, cudaFuncAttributeMaxDynamicSharedMemorySize, big)); \
  CK(cudaFuncSetAttribute(ssdk::wkv_scan_reg_kernel<float, DG>, cudaFuncAttributeMaxDynamicSharedMemorySize, big)); \
  CK(cudaFuncSetAttribute(ssdk::mlstm_scan_reg_kernel<bf16, DG>, cudaFuncAttributeMaxDynamicSharedMemorySize, big)); \
  CK(cudaFuncSetAttribute(ssdk::mlstm_scan_reg_kernel<float, DG>, cudaFuncAttributeMaxDynamicSharedMemorySize, big));
  SSDK_SCAN_ATTR(8) SSDK_SCAN_ATTR(16) SSDK_SCAN_ATTR(32)
#undef SSDK_SCAN_ATTR
  CK(cudaFuncSetAttribute(ssdk::latent_decode_partial_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, big));
  CK(cudaFuncSetAttribute(ssdk::latent_decode_partial_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, big));
  CK(cudaFuncSetAttribute(ssdk::latent_decode_mma_kernel<3, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, big));
  CK(cudaFuncSetAttribute(ssdk::latent_decode_mma_kernel<5, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, big));
  CK(cudaFuncSetAttribute(ssdk::latent_decode_mma_kernel<9, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, big));
  CK(cudaFuncSetAttribute(ssdk::delta_scan_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, big));
  CK(cudaFuncSetAttribute(ssdk::delta_scan_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, big));
  CK(cudaFuncSetAttribute(ssdk::delta_scan_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, big));
  CK(cudaFuncSetAttribute(ssdk::delta_scan_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, big));
  CK(cudaFuncSetAttribute(ssdk::delta_prep_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, big));
  CK(cudaFuncSetAttribute(ssdk::delta_prep_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, big));
  e->smem_attr_done = true;
  return 0;
}

template <typename T>
static int hyb_forward_t(ssdk_hyb_engine* e, int n_seqs, int M, const int32_t* ids, const int32_t* cu, const int32_t* pos0,
                         const int32_t* slot, const int32_t* tables, int n_want, const int32_t* want_rows, float* logits_host,
                         const float* temps, uint64_t seed, uint64_t step_id, int64_t* out_tokens, float* residual_host,
                         cudaStream_t st) {
  const ssdk_hyb_cfg& g = e->cfg;
  CKI(hyb_smem_attrs(e));
  // stage the step's integers: ids | tok_seq | cu | pos0 | slot | tables | want_rows
  int* hm = e->h_meta;
  int* d = e->meta;
  size_t o = 0;
  const size_t o_ids = o; memcpy(hm + o, ids, (size_t)M * 4); o += M;
  const size_t o_seq = o;
  for (int s = 0; s < n_seqs; ++s)
    for (int r = cu[s]; r < cu[s + 1]; ++r) hm[o_seq + r] = s;
  o += M;
  const size_t o_cu = o; memcpy(hm + o, cu, (size_t)(n_seqs + 1) * 4); o += n_seqs + 1;
  const size_t o_pos = o; memcpy(hm + o, pos0, (size_t)n_seqs * 4); o += n_seqs;
  const size_t o_slot = o; memcpy(hm + o, slot, (size_t)n_seqs * 4); o += n_seqs;
  const size_t o_tab = o; memcpy(hm + o, tables, (size_t)n_seqs * g.max_blocks_per_seq * 4); o += (size_t)n_seqs * g.max_blocks_per_seq;
  const size_t o_want = o; if (n_want) memcpy(hm + o, want_rows, (size_t)n_want * 4); o += n_want;
  CK(cudaMemcpyAsync(d, hm, o * 4, cudaMemcpyHostToDevice, st));
  HybRun<T> run;
  run.e = e; run.L.st = st; run.L.pdl = false; run.M = M; run.h_cu = cu; run.h_pos0 = pos0;
  run.rg.cu = d + o_cu; run.rg.pos0 = d + o_pos; run.rg.slot = d + o_slot; run.rg.tok_seq = d + o_seq; run.rg.tables = d + o_tab;
  run.rg.n_seqs = n_seqs; run.rg.M = M; run.rg.max_blocks = g.max_blocks_per_seq; run.rg.block_size = g.block_size;
  CKI(run.L.go(ssdk::embed_rows_kernel<T>, dim3(M), dim3(128), 0, (const int*)(d + o_ids), (const T*)e->embed.p, e->x, g.width, g.vocab,
               g.embed_scale, (g.block == SSDK_BLOCK_SERIAL_POSTNORM && !std::is_same<T, float>::value) ? (T*)e->h : (T*)nullptr));
  for (int li = 0; li < g.n_layers; ++li) {
    CKI(run.layer(e->layers[li], li));
    if (residual_host)
      CK(cudaMemcpyAsync(residual_host + (size_t)li * M * g.width, e->x, (size_t)M * g.width * 4, cudaMemcpyDeviceToHost, st));
  }
  if (n_want > 0) {
    CKI(run.L.go(ssdk::offset_rmsnorm_kernel<T>, dim3(n_want), dim3(256), 0, (const float*)e->x, (const T*)e->final_norm.p, (T*)e->hn,
                 (const int*)(d + o_want), g.width, g.eps, g.norm_offset, (const T*)nullptr, (T*)nullptr));
    CKI(run.lin(e->hn, g.width, e->head.p, g.width, e->logits, g.vocab, n_want, g.vocab, g.width));
    if (logits_host) CK(cudaMemcpyAsync(logits_host, e->logits, (size_t)n_want * g.vocab * 4, cudaMemcpyDeviceToHost, st));
    if (temps && out_tokens) {
      const size_t n = (size_t)n_want * g.vocab;
      CKI(run.L.go(ssdk::f32_to_bf16_kernel, dim3((unsigned)std::min<size_t>((n + 255) / 256, 8192)), dim3(256), 0, (const float*)e->logits,
                   e->logits16, n));
      CK(cudaMemcpyAsync(e->temps, temps, (size_t)n_want * 4, cudaMemcpyHostToDevice, st));
      void* scr = nullptr;
      CKI(op_scratch(&scr, st));
      for (int r0 = 0; r0 < n_want; r0 += 256) {
        const int nb = std::min(256, n_want - r0);
        SampleParams sp;
        sp.logits = e->logits16 + (size_t)r0 * g.vocab; sp.ld = g.vocab; sp.temps = e->temps + r0; sp.V = g.vocab; sp.seed = seed;
        sp.call_id = step_id; sp.out = e->tokens + r0; sp.out_stride = 1; sp.counters = (unsigned*)scr;
        sp.partial = (ArgMax*)((uint8_t*)scr + 4096); sp.dyn = nullptr; sp.sub = 0;
        CKI(run.L.go(sample_kernel, dim3(kSampleChunks, nb), dim3(256), 0, sp));
      }
      CK(cudaMemcpyAsync(out_tokens, e->tokens, (size_t)n_want * 8, cudaMemcpyDeviceToHost, st));
    }
  }
  e->launches += run.L.count;
  CK(cudaStreamSynchronize(st));
  return 0;
}

extern "C" {

int ssdk_hyb_create(const ssdk_hyb_cfg* cfg, const ssdk_hyb_layer_cfg* layers, ssdk_hyb_handle* out) {
  if (!cfg || !layers || !out) return fail("ssdk_hyb_create: null argument");
  if (cfg->width < 1 || cfg->vocab < 1 || cfg->n_layers < 1) return fail("ssdk_hyb_create: bad sizes");
  if (cfg->dtype != SSDK_DT_F32 && cfg->dtype != SSDK_DT_BF16) return fail("ssdk_hyb_create: unknown dtype %d", cfg->dtype);
  if (cfg->block != SSDK_BLOCK_PARALLEL_PRENORM && cfg->block != SSDK_BLOCK_SERIAL_POSTNORM && cfg->block != SSDK_BLOCK_PARALLEL_TWO_NORMS &&
      cfg->block != SSDK_BLOCK_PARALLEL_ONE_NORM) return fail("ssdk_hyb_create: unknown block kind %d", cfg->block);
  if (cfg->canon_taps < 0 || (cfg->block != SSDK_BLOCK_PARALLEL_ONE_NORM && (cfg->canon_taps || cfg->gated_residual)))
    return fail("ssdk_hyb_create: input convolutions and residual gates belong to one-norm blocks");
  if (cfg->max_tokens < 1 || cfg->max_seqs < 1 || cfg->max_logit_rows < 1 || cfg->block_size < 1 || cfg->max_blocks_per_seq < 1)
    return fail("ssdk_hyb_create: bad runtime limits");
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev < 1) return fail("ssdk_hyb_create: no CUDA device (there is no CPU path)");
  auto* e = new ssdk_hyb_engine();
  e->cfg = *cfg;
  e->esz = cfg->dtype == SSDK_DT_BF16 ? 2 : 4;
  e->use_tc = env_int("SSDK_HYB_TCGEN05", 1) != 0;
  e->use_decode_attn = env_int("SSDK_HYB_DECODE_ATTN", 1) != 0;
  e->use_decode_mma = env_int("SSDK_HYB_DECODE_MMA", 1) != 0;
  e->use_tc_scores = env_int("SSDK_HYB_TC_SCORES", 1) != 0;
  e->use_tc_experts = env_int("SSDK_HYB_TC_EXPERTS", 1) != 0;
  e->layers.resize(cfg->n_layers);
  for (int i = 0; i < cfg->n_layers; ++i) e->layers[i].c = layers[i];
  if (hyb_derive(e) != 0) { delete e; return -1; }
  for (auto& L : e->layers) {
    if ((L.c.mixer != SSDK_MIX_LATENT_ATTN && L.c.mixer != SSDK_MIX_ATTN_DELTA && L.c.mixer != SSDK_MIX_ATTENTION) || L.c.rot_dims < 2) continue;
    const int half = L.c.rot_dims / 2;
    std::vector<float> f(half);
    const double dims = (double)L.c.rot_dims, base = (double)L.c.rot_base;
    for (int i = 0; i < half; ++i) f[i] = (float)pow(base, -2.0 * i / dims);
    if (L.c.mixer == SSDK_MIX_ATTN_DELTA && L.c.yarn_factor > 0.f) {
      // YaRN: dimensions that turn fewer than `slow` times over the original length are slowed by `factor`, those that
      // turn more than `fast` times are kept, a linear ramp in between; cos and sin grow by 0.1 ln(factor) + 1
      const double kPi = 3.14159265358979323846, factor = (double)L.c.yarn_factor, orig = (double)L.c.yarn_original;
      auto dim_of = [&](double turns) { return dims * log(orig / (2.0 * kPi * turns)) / (2.0 * log(base)); };
      const double lo = std::max(floor(dim_of((double)L.c.yarn_fast)), 0.0), hi = std::min(ceil(dim_of((double)L.c.yarn_slow)), dims - 1.0);
      for (int i = 0; i < half; ++i) {
        const double fi = pow(base, -2.0 * i / dims);
        const double ramp = std::min(std::max(((double)i - lo) / std::max(hi - lo, 0.001), 0.0), 1.0);
        f[i] = (float)(fi / factor * ramp + fi * (1.0 - ramp));
      }
      L.rot_mult = (float)(0.1 * log(factor) + 1.0);
    }
    if (cudaMalloc(&L.inv_freq, half * 4) != cudaSuccess ||
        cudaMemcpy(L.inv_freq, f.data(), half * 4, cudaMemcpyHostToDevice) != cudaSuccess) {
      delete e;
      return fail("ssdk_hyb_create: could not place the rotation frequencies on the device");
    }
  }
  e->ws_bytes = hyb_carve(e, nullptr);
  if (cudaMallocHost(&e->h_meta, e->meta_ints * 4) != cudaSuccess) { delete e; return fail("ssdk_hyb_create: pinned staging allocation failed"); }
  *out = e;
  return 0;
}

int ssdk_hyb_destroy(ssdk_hyb_handle e) {
  if (!e) return 0;
  for (auto& L : e->layers)
    if (L.inv_freq) cudaFree(L.inv_freq);
  if (e->h_meta) cudaFreeHost(e->h_meta);
  delete e;
  return 0;
}

int ssdk_hyb_bind(ssdk_hyb_handle e, int layer, int tensor, const void* dev_ptr, int64_t rows, int64_t cols) {
  if (!e || !dev_ptr) return fail("ssdk_hyb_bind: null argument");
  if (tensor < 0 || tensor >= SSDK_HT_COUNT) return fail("ssdk_hyb_bind: unknown tensor %d", tensor);
  HybTensor t;
  t.p = dev_ptr; t.rows = rows; t.cols = cols;
  if (tensor == SSDK_HT_EMBED || tensor == SSDK_HT_HEAD || tensor == SSDK_HT_FINAL_NORM) {
    const int64_t want = tensor == SSDK_HT_FINAL_NORM ? e->cfg.width : (int64_t)e->cfg.vocab * e->cfg.width;
    if (rows * cols != want) return fail("ssdk_hyb_bind: tensor %d has %lld elements, expected %lld", tensor, (long long)(rows * cols), (long long)want);
    (tensor == SSDK_HT_EMBED ? e->embed : tensor == SSDK_HT_HEAD ? e->head : e->final_norm) = t;
    return 0;
  }
  if (layer < 0 || layer >= e->cfg.n_layers) return fail("ssdk_hyb_bind: layer %d out of range", layer);
  e->layers[layer].t[tensor] = t;
  return 0;
}

int64_t ssdk_hyb_cache_bytes(ssdk_hyb_handle e, int64_t num_blocks) {
  if (!e) return -1;
  return (int64_t)(num_blocks * e->cfg.block_size * e->cache_row_total * e->esz);
}
int64_t ssdk_hyb_state_bytes(ssdk_hyb_handle e, int64_t n_slots) {
  if (!e) return -1;
  return (int64_t)(n_slots * e->slot_floats * 4);
}
int64_t ssdk_hyb_workspace_bytes(ssdk_hyb_handle e) { return e ? e->ws_bytes : -1; }

int ssdk_hyb_bind_pools(ssdk_hyb_handle e, void* cache, int64_t num_blocks, void* state, int64_t n_slots, void* workspace,
                        int64_t workspace_bytes) {
  if (!e) return fail("ssdk_hyb_bind_pools: null handle");
  if (e->cache_row_total && (!cache || num_blocks < 1)) return fail("ssdk_hyb_bind_pools: the model has attention layers but no cache was given");
  if (e->slot_floats && (!state || n_slots < 1)) return fail("ssdk_hyb_bind_pools: the model has recurrent layers but no state pool was given");
  if (!workspace || workspace_bytes < e->ws_bytes) return fail("ssdk_hyb_bind_pools: workspace too small");
  if (((uintptr_t)workspace & 255) || ((uintptr_t)cache & 15) || ((uintptr_t)state & 15)) return fail("ssdk_hyb_bind_pools: misaligned pool");
  e->cache = (uint8_t*)cache; e->num_blocks = num_blocks; e->state = (float*)state; e->n_slots = n_slots;
  hyb_carve(e, (uint8_t*)workspace);
  return 0;
}

int ssdk_hyb_forward(ssdk_hyb_handle e, int n_seqs, int n_tokens, const int32_t* ids, const int32_t* cu, const int32_t* pos0,
                     const int32_t* slot, const int32_t* tables, int n_want, const int32_t* want_rows, float* logits_host,
                     const float* temps, uint64_t seed, uint64_t step_id, int64_t* out_tokens, float* residual_host, void* stream) {
  if (!e || !e->x) return fail("ssdk_hyb_forward: pools not bound");
  const ssdk_hyb_cfg& g = e->cfg;
  if (n_seqs < 1 || n_seqs > g.max_seqs) return fail("ssdk_hyb_forward: %d sequences (1..%d)", n_seqs, g.max_seqs);
  if (n_tokens < 1 || n_tokens > g.max_tokens) return fail("ssdk_hyb_forward: %d rows (1..%d)", n_tokens, g.max_tokens);
  if (n_want < 0 || n_want > g.max_logit_rows) return fail("ssdk_hyb_forward: %d logit rows (0..%d)", n_want, g.max_logit_rows);
  if (!e->embed.p || !e->head.p || !e->final_norm.p) return fail("ssdk_hyb_forward: embedding / head / final norm not bound");
  if (cu[0] != 0 || cu[n_seqs] != n_tokens) return fail("ssdk_hyb_forward: row offsets do not cover the batch");
  for (int s = 0; s < n_seqs; ++s) {
    if (cu[s + 1] <= cu[s]) return fail("ssdk_hyb_forward: sequence %d brings no rows", s);
    if (pos0[s] < 0) return fail("ssdk_hyb_forward: negative position");
    if (e->slot_floats && (slot[s] < 0 || slot[s] >= e->n_slots)) return fail("ssdk_hyb_forward: state slot %d out of range", slot[s]);
    for (int s2 = 0; s2 < s; ++s2)
      if (e->slot_floats && slot[s2] == slot[s]) return fail("ssdk_hyb_forward: two sequences share state slot %d", slot[s]);
    if (e->cache_row_total) {
      const int last = pos0[s] + (cu[s + 1] - cu[s]) - 1;
      if (last / g.block_size >= g.max_blocks_per_seq) return fail("ssdk_hyb_forward: sequence %d outgrows its page table", s);
      for (int b = 0; b <= last / g.block_size; ++b) {
        const int pg = tables[(size_t)s * g.max_blocks_per_seq + b];
        if (pg < 0 || pg >= e->num_blocks) return fail("ssdk_hyb_forward: page %d of sequence %d out of range", pg, s);
      }
    }
  }
  for (int i = 0; i < n_want; ++i)
    if (want_rows[i] < 0 || want_rows[i] >= n_tokens) return fail("ssdk_hyb_forward: logit row out of range");
  cudaStream_t st = (cudaStream_t)stream;
  if (g.dtype == SSDK_DT_BF16)
    return hyb_forward_t<bf16>(e, n_seqs, n_tokens, ids, cu, pos0, slot, tables, n_want, want_rows, logits_host, temps, seed, step_id,
                               out_tokens, residual_host, st);
  return hyb_forward_t<float>(e, n_seqs, n_tokens, ids, cu, pos0, slot, tables, n_want, want_rows, logits_host, temps, seed, step_id,
                              out_tokens, residual_host, st);
}

int64_t ssdk_hyb_launch_count(ssdk_hyb_handle e) { return e ? e->launches : -1; }

}  // extern "C"
