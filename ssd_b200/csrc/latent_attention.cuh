// latent_attention.cuh — attention over a compressed (latent) KV cache, with or without a learned softmax sink.
//
// What is cached per token and layer is one row [kv_rank + rot_dim] of storage type T in a paged pool: the RMS-normed
// latent c and the ONE rotated key part shared by all heads.  Keys and values are never materialised: with
//   k_h = W_uk,h c,   v_h = W_uv,h c       the score is   q_h . k_h = (W_uk,h^T q_h) . c
// so the queries are taken into latent space once per token (a per-head GEMM against W_uk^T, "absorption"), attention
// runs multi-query style over the latent rows (every head reads the same row), and the per-head value projection is
// applied to the attention's latent output (a per-head GEMM against W_uv).
//
//   latent_prep_kernel   splits the fused down-projection: RMS-norm -> query latent (T; skipped when the queries are
//                        full-rank); RMS-norm -> c and RoPE (fp32 angles; rotate-half or interleaved pairs) -> rotated
//                        key part, both scattered into the page slot.  A layer that reads another layer's pool skips it.
//   latent_q_kernel      per head: unrotated query part -> T (operand of the absorption GEMM), rotated part -> RoPE;
//                        absorbed and rotated parts share one row [kv_rank + rot_dim] per (token, head)
//   attention proper     per sequence and query block, as two tensor-core GEMMs around a softmax (HybRun::latent):
//                        latent_gather_kernel (pages -> contiguous keys and transposed latents), scores = Q K^T with the
//                        (token, head) pairs as rows (every head meets the same keys: multi-query), sink_softmax_kernel
//                        (fp32: causal edge per row; the per-head sink logit only enlarges the denominator, it
//                        contributes nothing to the output), output = P C.  Accumulation runs over keys in index order, whatever the portion.
//   single-token rows    (decode) skip the gather and the GEMMs: latent_decode_partial_kernel walks the pages of ALL such
//                        sequences in one launch, split along the context (scores, running maximum and P C per split,
//                        fp32), latent_decode_merge_kernel joins the splits and adds the sink to the denominator.
#pragma once
#include "layer_ops.cuh"

namespace ssdk {

SSDK_DEVINL size_t page_row(const Ragged& rg, int s, int pos) {
  const int page = rg.tables[(size_t)s * rg.max_blocks + pos / rg.block_size];
  return (size_t)page * rg.block_size + pos % rg.block_size;
}

struct LatentPrepArgs {
  const float* z;     // [M, ldz]: q latent [q_rank] | kv latent [kv_rank] | key rot part [rot_dim]
  int ldz;
  const void* qn_w;   // [q_rank] T
  const void* kvn_w;  // [kv_rank] T
  void* cq;           // [M, q_rank] T
  void* cache;        // [rows, kv_rank + rot_dim] T (this layer's pool)
  const float* inv_freq;  // [rot_dims / 2]
  int q_rank, kv_rank, rot_dim, rot_dims;
  int interleaved;    // 0: entry i turns with entry i + rot_dims/2; 1: entry 2i with entry 2i + 1
  float eps;
};

// entry c of a rotated vector zr at position pos: (u, v) -> (u cos a - v sin a, v cos a + u sin a), a = pos * f_i
SSDK_DEVINL float rope_entry(const float* zr, int c, int rot_dims, int interleaved, int pos, const float* inv_freq) {
  if (c >= rot_dims) return zr[c];
  const int half = rot_dims / 2;
  const bool first = interleaved ? !(c & 1) : c < half;
  const int i = interleaved ? c >> 1 : (first ? c : c - half);
  const int other = interleaved ? (c ^ 1) : (first ? c + half : c - half);
  float sn, cs;
  sincosf((float)pos * inv_freq[i], &sn, &cs);
  return first ? zr[c] * cs - zr[other] * sn : zr[c] * cs + zr[other] * sn;
}

template <typename T>
__global__ void latent_prep_kernel(const LatentPrepArgs p, const Ragged rg) {
  __shared__ float red[33];
  const int m = blockIdx.x, s = rg.tok_seq[m];
  const int pos = rg.pos0[s] + (m - rg.cu[s]);
  const float* z = p.z + (size_t)m * p.ldz;
  float ss = 0.f, inv;
  if (p.q_rank > 0) {
    for (int c = threadIdx.x; c < p.q_rank; c += blockDim.x) ss = fmaf(z[c], z[c], ss);
    ss = block_sum(ss, red);
    inv = 1.0f / sqrtf(ss / (float)p.q_rank + p.eps);
    for (int c = threadIdx.x; c < p.q_rank; c += blockDim.x)
      st_f<T>((T*)p.cq + (size_t)m * p.q_rank + c, z[c] * inv * ld_f<T>((const T*)p.qn_w + c));
  }
  const float* zk = z + p.q_rank;
  ss = 0.f;
  for (int c = threadIdx.x; c < p.kv_rank; c += blockDim.x) ss = fmaf(zk[c], zk[c], ss);
  ss = block_sum(ss, red);
  inv = 1.0f / sqrtf(ss / (float)p.kv_rank + p.eps);
  T* row = (T*)p.cache + page_row(rg, s, pos) * (size_t)(p.kv_rank + p.rot_dim);
  for (int c = threadIdx.x; c < p.kv_rank; c += blockDim.x) st_f<T>(row + c, zk[c] * inv * ld_f<T>((const T*)p.kvn_w + c));
  const float* zr = zk + p.kv_rank;
  for (int c = threadIdx.x; c < p.rot_dim; c += blockDim.x)
    st_f<T>(row + p.kv_rank + c, rope_entry(zr, c, p.rot_dims, p.interleaved, pos, p.inv_freq));
}

// q rows [ldq] fp32 holding [H, D + R] -> qn [M, H, D] (T, operand of the absorption GEMM) and the rotated part (T) into
// columns [kv_rank, kv_rank + R) of the concatenated query rows qcat [M, H, kv_rank + R]; the absorption GEMM fills the rest
template <typename T>
__global__ void latent_q_kernel(const float* __restrict__ q, int ldq, T* __restrict__ qn, T* __restrict__ qcat,
                                const float* __restrict__ inv_freq, const Ragged rg, int H, int D, int R, int KR, int rot_dims,
                                int interleaved) {
  const int m = blockIdx.x, hd = blockIdx.y, s = rg.tok_seq[m];
  const int pos = rg.pos0[s] + (m - rg.cu[s]);
  const float* src = q + (size_t)m * ldq + (size_t)hd * (D + R);
  for (int c = threadIdx.x; c < D; c += blockDim.x) st_f<T>(qn + ((size_t)m * H + hd) * D + c, src[c]);
  const float* zr = src + D;
  for (int c = threadIdx.x; c < R; c += blockDim.x)
    st_f<T>(qcat + ((size_t)m * H + hd) * (KR + R) + KR + c, rope_entry(zr, c, rot_dims, interleaved, pos, inv_freq));
}

// One sequence's cached rows of positions lo .. lo + ctx - 1, made contiguous for the two attention GEMMs: keys [ctx_pad, W]
// (W = kv_rank + R) and the latents transposed, lat_t [kv_rank, ctx_pad]; rows / columns from ctx up to ctx_pad (a multiple
// of 8) are zero.  lo > 0 when a sliding window hides the sequence's first positions from the whole portion.
template <typename T>
__global__ void latent_gather_kernel(const T* __restrict__ cache, T* __restrict__ keys, T* __restrict__ lat_t, const Ragged rg,
                                     int s, int lo, int ctx, int ctx_pad, int KR, int W) {
  const int j = blockIdx.x;
  const T* row = j < ctx ? cache + page_row(rg, s, lo + j) * (size_t)W : nullptr;
  for (int d = threadIdx.x; d < W; d += blockDim.x) {
    const float v = row ? ld_f<T>(row + d) : 0.f;
    st_f<T>(keys + (size_t)j * W + d, v);
    if (d < KR) st_f<T>(lat_t + (size_t)d * ctx_pad + j, v);
  }
}

// Softmax with a sink over the score rows of one query block.  The rows come in `batches` of rows_per_batch (one batch
// per key/value head of grouped-query attention; a single batch for latent attention); inside a batch row r is
// (query q0 + r / H, head r % H) with H the heads that share the batch's keys.  Column j of a row is the key at position
// key_first + j; the query at position pos sees the keys at max(0, pos - window + 1) .. pos (window = 0: at 0 .. pos).
// sc [rows, ld] fp32 raw dot products -> pr [rows, ld] (T) weights, zero outside the visible range and in the padding.
// The sink is a learned per-head logit (`sink`, indexed batch * H + head) or, without one, the constant sink_const added
// to the denominator (0: plain softmax); it joins the maximum, is not scaled and contributes nothing to the output.
template <typename T>
__global__ void sink_softmax_kernel(const float* __restrict__ sc, T* __restrict__ pr, const T* __restrict__ sink, int H, int ld,
                                    int pos_first, float scale, int rows_per_batch, float sink_const, int key_first, int window) {
  __shared__ float red[33];
  const int r = blockIdx.x, batch = r / rows_per_batch, rb = r - batch * rows_per_batch;
  const int h = rb % H, pos = pos_first + rb / H;
  const int n = pos - key_first + 1;                                             // columns [j0, n) are the keys this row sees
  const int j0 = window > 0 ? max(0, pos - window + 1 - key_first) : 0;
  const float* srow = sc + (size_t)r * ld;
  const float sk = sink ? ld_f<T>(sink + batch * H + h) : (sink_const > 0.f ? logf(sink_const) : -INFINITY);
  float mx = sk;
  for (int j = j0 + threadIdx.x; j < n; j += blockDim.x) mx = fmaxf(mx, srow[j] * scale);
  __syncthreads();
  mx = warp_max(mx);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
  __syncthreads();
  mx = red[0];
  for (int w = 1; w < (int)(blockDim.x >> 5); ++w) mx = fmaxf(mx, red[w]);
  float sum = 0.f;
  for (int j = j0 + threadIdx.x; j < n; j += blockDim.x) sum += expf(srow[j] * scale - mx);
  sum = block_sum(sum, red) + expf(sk - mx);
  const float inv = 1.0f / sum;
  for (int j = threadIdx.x; j < ld; j += blockDim.x)
    st_f<T>(pr + (size_t)r * ld + j, (j >= j0 && j < n) ? expf(srow[j] * scale - mx) * inv : 0.f);
}

// ---- single-token (decode) rows: one launch over all such sequences, the context split flash-decoding style ----
struct LatentDecodeArgs {
  const void* qcat;   // [M, H, W] T: latent-space query | rotated part
  const void* cache;  // [rows, W] T (this layer's pool)
  const void* sink;   // [H] T, or nullptr: plain softmax
  float* part;        // [n_seqs, splits, H, KR + 2] fp32: unnormalised P C | running maximum | running sum
  void* out;          // [M, H, KR] T
  int H, KR, W, splits;
  int pool_aligned;   // the pool starts on a 16-byte boundary
  float scale;
  int window;         // the token at position p sees the keys at max(0, p - window + 1) .. p; 0: all of 0 .. p
};

// keys [k_lo, k_hi) of split j (of `splits`) for a single token at position ctx - 1
SSDK_DEVINL void decode_split(int ctx, int window, int j, int splits, int* k_lo, int* k_hi) {
  const int first = window > 0 ? max(0, ctx - window) : 0, per = (ctx - first + splits - 1) / splits;
  *k_lo = first + j * per;
  *k_hi = min(ctx, *k_lo + per);
}

constexpr int kDecTile = 16, kDecThreads = 256;

inline size_t latent_decode_smem(int H, int KR, int W, size_t esz) {
  const size_t Hp = (size_t)(H + 3) / 4 * 4;
  return (kDecTile * Hp + (size_t)H * W + (size_t)H * KR + 3 * (size_t)H) * 4 + (size_t)kDecTile * W * esz + 16;
}

template <typename T> SSDK_DEVINL float2 ld_pair(const T* p);
template <> SSDK_DEVINL float2 ld_pair<float>(const float* p) { return make_float2(p[0], p[1]); }
template <> SSDK_DEVINL float2 ld_pair<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}

// grid (n_seqs, splits); a sequence that brings more than one row is left to the GEMM path.  Both products are
// register-blocked over heads so that one shared-memory load feeds several FMAs: a warp scores one key against four
// heads at a time (two dimensions per lane and step), a thread accumulates one latent column for eight heads at a time.
template <typename T>
__global__ void __launch_bounds__(kDecThreads) latent_decode_partial_kernel(const LatentDecodeArgs p, const Ragged rg) {
  const int s = blockIdx.x, j = blockIdx.y;
  const int row = rg.cu[s];
  if (rg.cu[s + 1] - row != 1) return;
  const int H = p.H, KR = p.KR, W = p.W, Hp = (H + 3) / 4 * 4;
  extern __shared__ __align__(16) uint8_t dec_smem[];
  float* ps = (float*)dec_smem;            // [kDecTile, Hp] scores, then weights (columns H .. Hp stay zero)
  float* qs = ps + kDecTile * Hp;          // [H, W] query times scale
  float* acc = qs + (size_t)H * W;         // [H, KR]
  float* mx = acc + (size_t)H * KR;        // [H] running maximum
  float* ls = mx + H;                      // [H] running sum
  float* rs = ls + H;                      // [H] rescale of this tile
  T* ct = (T*)(rs + H);                    // [kDecTile, W] key rows
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int k_lo, k_hi;
  decode_split(rg.pos0[s] + 1, p.window, j, p.splits, &k_lo, &k_hi);
  const T* q = (const T*)p.qcat + (size_t)row * H * W;
  constexpr int kPerVec = 16 / (int)sizeof(T);
  const size_t ct_off = ((size_t)kDecTile * Hp + (size_t)H * W + (size_t)H * KR + 3 * (size_t)H) * 4;
  // rows of the pool start on 16-byte boundaries when W is a multiple of a vector (the pool itself is 16-byte aligned)
  const bool vec = p.pool_aligned && W % kPerVec == 0 && ct_off % 16 == 0;
  const bool pairs = W % 2 == 0;  // (the key tile starts on a 4-byte boundary, which a bf16 pair needs)
  for (int i = tid; i < H * W; i += kDecThreads) qs[i] = ld_f<T>(q + i) * p.scale;
  for (int i = tid; i < H * KR; i += kDecThreads) acc[i] = 0.f;
  for (int i = tid; i < kDecTile * Hp; i += kDecThreads) ps[i] = 0.f;
  for (int i = tid; i < H; i += kDecThreads) { mx[i] = -INFINITY; ls[i] = 0.f; }
  __syncthreads();
  const int hq = Hp / 4;
  for (int k0 = k_lo; k0 < k_hi; k0 += kDecTile) {
    const int nk = min(kDecTile, k_hi - k0);
    if (vec) {  // 16-byte loads, every thread several in flight
      const int vpr = W / kPerVec;
#pragma unroll 4
      for (int i = tid; i < nk * vpr; i += kDecThreads) {
        const int k = i / vpr, v = i - k * vpr;
        const uint4* src = (const uint4*)((const T*)p.cache + page_row(rg, s, k0 + k) * (size_t)W);
        ((uint4*)ct)[i] = __ldg(src + v);
      }
    } else {
      for (int k = warp; k < nk; k += kDecThreads / 32) {
        const T* src = (const T*)p.cache + page_row(rg, s, k0 + k) * (size_t)W;
        for (int d = lane; d < W; d += 32) ct[k * W + d] = src[d];
      }
    }
    __syncthreads();
    for (int pr = warp; pr < kDecTile * hq; pr += kDecThreads / 32) {
      const int k = pr % kDecTile, h0 = (pr / kDecTile) * 4;
      float a[4] = {0.f, 0.f, 0.f, 0.f};
      if (k < nk) {
        const T* kr = ct + k * W;
        if (pairs) {
          for (int d = 2 * lane; d < W; d += 64) {
            const float2 x = ld_pair<T>(kr + d);
#pragma unroll
            for (int hh = 0; hh < 4; ++hh)
              if (h0 + hh < H) {
                const float2 qv = *reinterpret_cast<const float2*>(qs + (size_t)(h0 + hh) * W + d);
                a[hh] = fmaf(qv.x, x.x, fmaf(qv.y, x.y, a[hh]));
              }
          }
        } else {
          for (int d = lane; d < W; d += 32) {
            const float x = ld_f<T>(kr + d);
#pragma unroll
            for (int hh = 0; hh < 4; ++hh)
              if (h0 + hh < H) a[hh] = fmaf(qs[(size_t)(h0 + hh) * W + d], x, a[hh]);
          }
        }
      }
#pragma unroll
      for (int hh = 0; hh < 4; ++hh) {
        const float v = warp_sum(a[hh]);
        if (lane == 0 && h0 + hh < H) ps[k * Hp + h0 + hh] = k < nk ? v : -INFINITY;
      }
    }
    __syncthreads();
    for (int h = tid; h < H; h += kDecThreads) {
      float m_new = mx[h];
      for (int k = 0; k < nk; ++k) m_new = fmaxf(m_new, ps[k * Hp + h]);
      const float r = mx[h] == -INFINITY ? 0.f : expf(mx[h] - m_new);
      float sum = ls[h] * r;
      for (int k = 0; k < kDecTile; ++k) {
        const float w = k < nk ? expf(ps[k * Hp + h] - m_new) : 0.f;
        ps[k * Hp + h] = w;
        sum += w;
      }
      mx[h] = m_new; ls[h] = sum; rs[h] = r;
    }
    __syncthreads();
    for (int c = tid; c < KR; c += kDecThreads) {
      for (int h0 = 0; h0 < H; h0 += 8) {
        float a[8];
#pragma unroll
        for (int hh = 0; hh < 8; ++hh) a[hh] = h0 + hh < H ? acc[(size_t)(h0 + hh) * KR + c] * rs[h0 + hh] : 0.f;
        const bool second = h0 + 4 < Hp;
        for (int k = 0; k < nk; ++k) {
          const float x = ld_f<T>(ct + k * W + c);
          const float4 p0 = *reinterpret_cast<const float4*>(ps + k * Hp + h0);
          const float4 p1 = second ? *reinterpret_cast<const float4*>(ps + k * Hp + h0 + 4) : make_float4(0.f, 0.f, 0.f, 0.f);
          a[0] = fmaf(p0.x, x, a[0]); a[1] = fmaf(p0.y, x, a[1]); a[2] = fmaf(p0.z, x, a[2]); a[3] = fmaf(p0.w, x, a[3]);
          a[4] = fmaf(p1.x, x, a[4]); a[5] = fmaf(p1.y, x, a[5]); a[6] = fmaf(p1.z, x, a[6]); a[7] = fmaf(p1.w, x, a[7]);
        }
#pragma unroll
        for (int hh = 0; hh < 8; ++hh)
          if (h0 + hh < H) acc[(size_t)(h0 + hh) * KR + c] = a[hh];
      }
    }
    __syncthreads();
  }
  float* dst = p.part + ((size_t)s * p.splits + j) * H * (KR + 2);
  for (int o = tid; o < H * KR; o += kDecThreads) dst[(size_t)(o / KR) * (KR + 2) + o % KR] = acc[o];
  for (int h = tid; h < H; h += kDecThreads) { dst[(size_t)h * (KR + 2) + KR] = mx[h]; dst[(size_t)h * (KR + 2) + KR + 1] = ls[h]; }
}

// ---- the same split-context pass on the tensor cores (bf16 storage, rows of the pool 16-byte aligned) ----
// grid (n_seqs, splits, head groups of 16), four warps.  The queries of up to 16 heads are the 16 rows of an m16n8k16
// tile: a warp keeps the A fragments of ITS quarter of the W = kv_rank + rot_dim columns in registers for the whole
// pass, so a tile of 32 keys (cp.async, double buffered, rows beyond the split zero-filled) is read from shared memory
// once for the scores — the four warps' partial products are summed through shared memory — and once more, transposed
// by ldmatrix, as the B operand of P C, where every warp owns a quarter of the latent columns (NT n-tiles of 8).
// Scores, maximum, sum and the rescaling stay fp32; P is rounded to bf16 for the product like on the GEMM path.
// Writes the same partials as latent_decode_partial_kernel, so latent_decode_merge_kernel joins them.
constexpr int kDmKeys = 32, kDmThreads = 128;

inline int latent_decode_mma_ldk(int W) { return (W + 15) / 16 * 16 + 8; }   // padded row (elements) of queries and keys in shared memory
inline size_t latent_decode_mma_smem(int W) {
  return (size_t)(2 * kDmKeys + 16) * latent_decode_mma_ldk(W) * 2 + (size_t)4 * 16 * (kDmKeys + 1) * 4 + (size_t)16 * (kDmKeys + 8) * 2 + 3 * 16 * 4;
}

template <int KS, int NT>
__global__ void __launch_bounds__(kDmThreads) latent_decode_mma_kernel(const LatentDecodeArgs p, const Ragged rg) {
  const int s = blockIdx.x, j = blockIdx.y, h0 = blockIdx.z * 16;
  const int row = rg.cu[s];
  if (rg.cu[s + 1] - row != 1) return;
  const int H = p.H, KR = p.KR, W = p.W, LDK = (W + 15) / 16 * 16 + 8, nh = min(16, H - h0);
  extern __shared__ __align__(16) uint8_t dm_smem[];
  __nv_bfloat16* kt = (__nv_bfloat16*)dm_smem;                 // [2][kDmKeys][LDK] key tiles
  __nv_bfloat16* qs = kt + (size_t)2 * kDmKeys * LDK;          // [16][LDK] queries (rows beyond the heads are zero)
  float* sp = (float*)(qs + (size_t)16 * LDK);                 // [4][16][kDmKeys + 1] partial scores per warp
  __nv_bfloat16* pb = (__nv_bfloat16*)(sp + 4 * 16 * (kDmKeys + 1));   // [16][kDmKeys + 8] weights
  float* mx = (float*)(pb + 16 * (kDmKeys + 8));               // [16] running maximum
  float* ls = mx + 16;                                         // [16] running sum
  float* rs = ls + 16;                                         // [16] rescale of this tile
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t4 = lane & 3;
  int k_lo, k_hi;
  decode_split(rg.pos0[s] + 1, p.window, j, p.splits, &k_lo, &k_hi);
  const int vpr = W / 8;   // 16-byte vectors per row
  const __nv_bfloat16* cache = (const __nv_bfloat16*)p.cache;
  auto load_tile = [&](int k0, int buf) {
    __nv_bfloat16* dst = kt + (size_t)buf * kDmKeys * LDK;
    for (int i = tid; i < kDmKeys * vpr; i += kDmThreads) {
      const int k = i / vpr, v = i - k * vpr;
      const bool ok = k0 + k < k_hi;
      const __nv_bfloat16* src = ok ? cache + page_row(rg, s, k0 + k) * (size_t)W + v * 8 : cache;
      cp_async16(dst + (size_t)k * LDK + v * 8, src, ok);
    }
    cp_async_commit();
  };
  if (k_lo < k_hi) load_tile(k_lo, 0);
  // queries, padding columns of all three buffers, running statistics
  const __nv_bfloat16* q = (const __nv_bfloat16*)p.qcat + ((size_t)row * H + h0) * W;
  for (int i = tid; i < 16 * LDK; i += kDmThreads) {
    const int r = i / LDK, c = i - r * LDK;
    qs[i] = (r < nh && c < W) ? q[(size_t)r * W + c] : __float2bfloat16_rn(0.f);
  }
  for (int i = tid; i < 2 * kDmKeys * (LDK - W); i += kDmThreads) {
    const int r = i / (LDK - W), c = W + i % (LDK - W);
    kt[(size_t)r * LDK + c] = __float2bfloat16_rn(0.f);
  }
  if (tid < 16) { mx[tid] = -INFINITY; ls[tid] = 0.f; }
  __syncthreads();
  const int nks = (W + 15) / 16, ks_per = (nks + 3) / 4, ks0 = warp * ks_per, my_ks = max(0, min(ks_per, nks - ks0));
  uint32_t qa[KS][4];
#pragma unroll
  for (int i = 0; i < KS; ++i)
    if (i < my_ks) ldmatrix_x4(qa[i], qs + (size_t)(lane & 15) * LDK + (ks0 + i) * 16 + (lane >> 4) * 8);
  float acc[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
  const int ntiles = (KR + 7) / 8, nt0 = warp * NT;   // this warp's latent columns: n-tiles nt0 .. nt0 + NT - 1
  int buf = 0;
  for (int k0 = k_lo; k0 < k_hi; k0 += kDmKeys, buf ^= 1) {
    cp_async_wait<0>();
    __syncthreads();   // the tile has landed; everyone is done with the other buffer
    if (k0 + kDmKeys < k_hi) load_tile(k0 + kDmKeys, buf ^ 1);
    const __nv_bfloat16* tile = kt + (size_t)buf * kDmKeys * LDK;
    float sc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.f;
#pragma unroll
    for (int i = 0; i < KS; ++i)
      if (i < my_ks) {
        const int kk = (ks0 + i) * 16;
#pragma unroll
        for (int nj = 0; nj < 2; ++nj) {
          uint32_t b[4];
          ldmatrix_x4(b, tile + (size_t)(nj * 16 + (lane >> 4) * 8 + (lane & 7)) * LDK + kk + ((lane >> 3) & 1) * 8);
          mma_bf16_16816(sc[2 * nj], qa[i], b[0], b[1]);
          mma_bf16_16816(sc[2 * nj + 1], qa[i], b[2], b[3]);
        }
      }
    float* spw = sp + warp * 16 * (kDmKeys + 1);
#pragma unroll
    for (int ni = 0; ni < 4; ++ni) {
      spw[g * (kDmKeys + 1) + ni * 8 + 2 * t4] = sc[ni][0];
      spw[g * (kDmKeys + 1) + ni * 8 + 2 * t4 + 1] = sc[ni][1];
      spw[(g + 8) * (kDmKeys + 1) + ni * 8 + 2 * t4] = sc[ni][2];
      spw[(g + 8) * (kDmKeys + 1) + ni * 8 + 2 * t4 + 1] = sc[ni][3];
    }
    __syncthreads();
    {
      // row r of the tile: eight threads, four keys each (fp32 softmax step)
      const int r = tid >> 3, sub = tid & 7, nk = min(kDmKeys, k_hi - k0);
      float v[4], m_new = mx[r];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int k = sub * 4 + c;
        float a = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) a += sp[(w * 16 + r) * (kDmKeys + 1) + k];
        v[c] = k < nk ? a * p.scale : -INFINITY;
        m_new = fmaxf(m_new, v[c]);
      }
#pragma unroll
      for (int o = 4; o > 0; o >>= 1) m_new = fmaxf(m_new, __shfl_xor_sync(0xffffffffu, m_new, o));
      float sum = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float w = v[c] == -INFINITY ? 0.f : expf(v[c] - m_new);
        pb[r * (kDmKeys + 8) + sub * 4 + c] = __float2bfloat16_rn(w);
        sum += w;
      }
#pragma unroll
      for (int o = 4; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      const float m_old = mx[r];
      const float resc = m_old == -INFINITY ? 0.f : expf(m_old - m_new);
      __syncwarp();
      if (sub == 0) { mx[r] = m_new; ls[r] = ls[r] * resc + sum; rs[r] = resc; }
    }
    __syncthreads();
    const float r_lo = rs[g], r_hi = rs[g + 8];
#pragma unroll
    for (int i = 0; i < NT; ++i) { acc[i][0] *= r_lo; acc[i][1] *= r_lo; acc[i][2] *= r_hi; acc[i][3] *= r_hi; }
#pragma unroll
    for (int kk = 0; kk < kDmKeys; kk += 16) {
      uint32_t pa[4];
      ldmatrix_x4(pa, pb + (size_t)(lane & 15) * (kDmKeys + 8) + kk + (lane >> 4) * 8);
#pragma unroll
      for (int i = 0; i < NT; i += 2) {
        if (nt0 + i >= ntiles) continue;
        uint32_t vb[4];
        const int mi = lane >> 3, rr = lane & 7;
        // (a second n-tile beyond the latent columns reads the rotated part or the zero padding: its result is dropped)
        ldmatrix_x4_trans(vb, tile + (size_t)(kk + (mi & 1) * 8 + rr) * LDK + (nt0 + i) * 8 + (mi >> 1) * 8);
        mma_bf16_16816(acc[i], pa, vb[0], vb[1]);
        if (i + 1 < NT) mma_bf16_16816(acc[i + 1], pa, vb[2], vb[3]);
      }
    }
  }
  __syncthreads();
  float* dst = p.part + (((size_t)s * p.splits + j) * H + h0) * (KR + 2);
#pragma unroll
  for (int i = 0; i < NT; ++i) {
    const int c = (nt0 + i) * 8 + 2 * t4;
    if (nt0 + i >= ntiles) continue;
    if (g < nh) {
      if (c < KR) dst[(size_t)g * (KR + 2) + c] = acc[i][0];
      if (c + 1 < KR) dst[(size_t)g * (KR + 2) + c + 1] = acc[i][1];
    }
    if (g + 8 < nh) {
      if (c < KR) dst[(size_t)(g + 8) * (KR + 2) + c] = acc[i][2];
      if (c + 1 < KR) dst[(size_t)(g + 8) * (KR + 2) + c + 1] = acc[i][3];
    }
  }
  if (tid < nh) { dst[(size_t)tid * (KR + 2) + KR] = mx[tid]; dst[(size_t)tid * (KR + 2) + KR + 1] = ls[tid]; }
}

// grid (n_seqs, H, column chunks of the block size): out = sum_j e^(m_j - m) acc_j / (e^(sink - m) + sum_j e^(m_j - m) l_j), m = max(sink, max_j m_j)
constexpr int kDecMaxSplits = 32;   // the host never asks for more context splits

template <typename T>
__global__ void latent_decode_merge_kernel(const LatentDecodeArgs p, const Ragged rg) {
  __shared__ float wj[kDecMaxSplits];   // e^(m_j - m) / denominator per split (0 for a split without keys)
  const int s = blockIdx.x, h = blockIdx.y;
  const int row = rg.cu[s];
  if (rg.cu[s + 1] - row != 1) return;
  const int KR = p.KR;
  const float* part = p.part + ((size_t)s * p.splits * p.H + h) * (KR + 2);
  const size_t js = (size_t)p.H * (KR + 2);  // floats between two splits of one head
  if (threadIdx.x < 32) {
    const int j = threadIdx.x;
    const float sk = p.sink ? ld_f<T>((const T*)p.sink + h) : -INFINITY;
    const float mj = j < p.splits ? part[j * js + KR] : -INFINITY;
    const float m = fmaxf(sk, warp_max(mj));
    const float w = mj == -INFINITY ? 0.f : expf(mj - m);
    const float den = warp_sum(j < p.splits ? w * part[j * js + KR + 1] : 0.f) + (sk == -INFINITY ? 0.f : expf(sk - m));
    if (j < p.splits) wj[j] = w / den;
  }
  __syncthreads();
  T* out = (T*)p.out + ((size_t)row * p.H + h) * KR;
  // a thread per latent column (blockIdx.z picks the chunk of columns), four independent sums so that the loads overlap
  const int c = blockIdx.z * blockDim.x + threadIdx.x;
  if (c >= KR) return;
  float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
  int j = 0;
  for (; j + 4 <= p.splits; j += 4) {
    a0 = fmaf(wj[j], part[j * js + c], a0);
    a1 = fmaf(wj[j + 1], part[(j + 1) * js + c], a1);
    a2 = fmaf(wj[j + 2], part[(j + 2) * js + c], a2);
    a3 = fmaf(wj[j + 3], part[(j + 3) * js + c], a3);
  }
  for (; j < p.splits; ++j) a0 = fmaf(wj[j], part[j * js + c], a0);
  st_f<T>(out + c, (a0 + a1) + (a2 + a3));
}

}  // namespace ssdk
