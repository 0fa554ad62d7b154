// gqa_attention.cuh — grouped-query causal softmax attention over a paged key/value cache, for the layered (hybrid)
// models.  H query heads share G key/value heads (query head h reads head h / (H / G)); key size D and value size V are
// independent.  A page row holds, for one token, the keys of all G heads (rotated, optionally unit-RMS) and then their
// values: [G D | G V] of storage type T.  The softmax denominator may carry a constant (`sink`: 1 = a sink of score 0
// that has no value) or a learned logit per query head; a sliding window limits a query to its last `window` positions.
//
//   gqa_prep_kernel      per (token, head): rotation of the first rot_dims dimensions in adjacent or half-apart pairs (angle = position *
//                        frequency in fp32, cos and sin times a constant), optional unit RMS over D; queries go to a
//                        group-major buffer [G, M, H/G, D] (T), keys and raw values into the token's page row
//   kv_gather_kernel     one sequence's pages -> contiguous keys [G, ctx_pad, D] and transposed values [G, V, ctx_pad]
//   portions (>= 2 rows) two batched GEMMs per query block around sink_softmax_kernel (HybRun::gqa_attention)
//   single-token rows    gqa_decode_partial_kernel (all decoding sequences in one launch, context split flash-decoding
//                        style, fp32 weights) + gqa_decode_merge_kernel
//   attn_gate_kernel     group-major fp32 output x sigmoid(gate pre-activation) -> [M, H V] (T) for the output projection
#pragma once
#include "latent_attention.cuh"

namespace ssdk {

struct GqaPrepArgs {
  const float* z; int ldz;     // [M, ldz]: q [H D] | k [G D] | v [G V] (fp32 projections)
  void* q;                     // [G, M, H/G, D] T
  void* cache;                 // [rows, G (D + V)] T (this layer's pool)
  const float* inv_freq;       // [rot_dims / 2] or nullptr
  int H, G, D, V, rot_dims, qk_norm;
  float rot_mult, eps;
  int rot_half;                // 0: entry 2i turns with 2i + 1; 1: entry i turns with i + rot_dims / 2
};

// grid (M, H + G), one warp: units 0 .. H-1 are query heads, H .. H+G-1 key heads (which also copy their value head)
template <typename T>
__global__ void gqa_prep_kernel(const GqaPrepArgs p, const Ragged rg) {
  const int m = blockIdx.x, unit = blockIdx.y, lane = threadIdx.x, s = rg.tok_seq[m];
  const int pos = rg.pos0[s] + (m - rg.cu[s]);
  const int H = p.H, G = p.G, D = p.D, V = p.V;
  const bool is_q = unit < H;
  const int hd = is_q ? unit : unit - H;
  const float* src = p.z + (size_t)m * p.ldz + (is_q ? (size_t)hd * D : (size_t)H * D + (size_t)hd * D);
  T* dst;
  if (is_q) {
    const int hpg = H / G, g = hd / hpg;
    dst = (T*)p.q + (((size_t)g * rg.M + m) * hpg + (hd - g * hpg)) * D;
  } else {
    dst = (T*)p.cache + page_row(rg, s, pos) * (size_t)(G * (D + V)) + (size_t)hd * D;
  }
  // pass 1: rotate pairs, accumulate the square sum; pass 2: scale and store (the pair values are recomputed)
  float ss = 0.f;
  const int rd = p.inv_freq ? p.rot_dims : 0;
  auto value = [&](int d) -> float {
    if (d >= rd) return src[d];
    if (p.rot_half) {
      const int half = rd >> 1, i = d < half ? d : d - half;
      float sn, cs;
      sincosf((float)pos * p.inv_freq[i], &sn, &cs);
      sn *= p.rot_mult; cs *= p.rot_mult;
      return d < half ? src[d] * cs - src[d + half] * sn : src[d] * cs + src[d - half] * sn;
    }
    const int i = d >> 1;
    float sn, cs;
    sincosf((float)pos * p.inv_freq[i], &sn, &cs);
    sn *= p.rot_mult; cs *= p.rot_mult;
    const float a = src[2 * i], b = src[2 * i + 1];
    return (d & 1) ? b * cs + a * sn : a * cs - b * sn;
  };
  float inv = 1.0f;
  if (p.qk_norm) {
    for (int d = lane; d < D; d += 32) { const float v = value(d); ss = fmaf(v, v, ss); }
    ss = warp_sum(ss);
    inv = 1.0f / sqrtf(ss / (float)D + p.eps);
  }
  for (int d = lane; d < D; d += 32) st_f<T>(dst + d, value(d) * inv);
  if (!is_q) {
    const float* vsrc = p.z + (size_t)m * p.ldz + (size_t)(H + G) * D + (size_t)hd * V;
    T* vdst = (T*)p.cache + page_row(rg, s, pos) * (size_t)(G * (D + V)) + (size_t)G * D + (size_t)hd * V;
    for (int d = lane; d < V; d += 32) st_f<T>(vdst + d, vsrc[d]);
  }
}

// grid (ctx_pad): position lo + j of sequence s -> keys[g][j][:] and vt[g][:][j]; zero from ctx up to ctx_pad
template <typename T>
__global__ void kv_gather_kernel(const T* __restrict__ cache, T* __restrict__ keys, T* __restrict__ vt, const Ragged rg, int s,
                                 int lo, int ctx, int ctx_pad, int G, int D, int V) {
  const int j = blockIdx.x;
  const T* row = j < ctx ? cache + page_row(rg, s, lo + j) * (size_t)(G * (D + V)) : nullptr;
  for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
    const int g = i / D, d = i - g * D;
    keys[((size_t)g * ctx_pad + j) * D + d] = row ? row[i] : T(0.f);
  }
  for (int i = threadIdx.x; i < G * V; i += blockDim.x) vt[(size_t)i * ctx_pad + j] = row ? row[(size_t)G * D + i] : T(0.f);
}

struct GqaDecodeArgs {
  const void* q;      // [G, M, H/G, D] T
  const void* cache;  // [rows, G (D + V)] T
  float* part;        // [n_seqs, H, splits, V + 2] fp32: unnormalised P V | running maximum | running sum
  float* out;         // [G, M, H/G, V] fp32
  int H, G, D, V, splits;
  float scale, sink;
  const void* sinks;  // [H] T learned sink logits (they replace the constant), or nullptr
  int window;         // as LatentDecodeArgs::window
};

constexpr int kGqaDecWarps = 4;

inline size_t gqa_decode_smem(int D, int V) { return ((size_t)(D + 3) / 4 * 4 + (size_t)kGqaDecWarps * (V + 2)) * 4; }

// grid (n_seqs, H, splits), kGqaDecWarps warps.  A warp takes 32 keys at a time: first every lane scores ONE key (a
// thread-local dot product over D, the key row read in 16-byte pieces where its alignment allows), then every lane owns
// the VPL = ceil(V / 32) value columns lane VPL .. lane VPL + VPL - 1 (one vector load per key) and the 32 weights are
// passed around by shuffle.
template <typename T, int VPL>
__global__ void __launch_bounds__(kGqaDecWarps * 32) gqa_decode_partial_kernel(const GqaDecodeArgs p, const Ragged rg) {
  extern __shared__ __align__(16) float gd_sm[];
  const int s = blockIdx.x, hd = blockIdx.y, sp = blockIdx.z;
  const int row = rg.cu[s];
  if (rg.cu[s + 1] - row != 1) return;
  const int H = p.H, G = p.G, D = p.D, V = p.V, hpg = H / G, g = hd / hpg;
  const int Dp = (D + 3) / 4 * 4;
  float* qs = gd_sm;                      // [Dp] query times scale
  float* wp = gd_sm + Dp;                 // [warps][V + 2]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const T* q = (const T*)p.q + (((size_t)g * rg.M + row) * hpg + (hd - g * hpg)) * D;
  for (int d = tid; d < Dp; d += blockDim.x) qs[d] = d < D ? ld_f<T>(q + d) * p.scale : 0.f;
  __syncthreads();
  int k_lo, k_hi;
  decode_split(rg.pos0[s] + 1, p.window, sp, p.splits, &k_lo, &k_hi);
  const size_t roww = (size_t)G * (D + V);
  constexpr int kPer = 16 / (int)sizeof(T);
  const bool pool16 = ((uintptr_t)p.cache & 15) == 0;
  const bool vec_k = pool16 && D % kPer == 0 && roww % kPer == 0;
  constexpr int kVecBytes = VPL * (int)sizeof(T) >= 16 ? 16 : VPL * (int)sizeof(T);
  constexpr int kVecElems = kVecBytes / (int)sizeof(T);
  const bool vec_v = pool16 && V % VPL == 0 && roww % kVecElems == 0 && ((size_t)G * D) % kVecElems == 0 && V % kVecElems == 0;
  float mx = -INFINITY, sum = 0.f, acc[VPL];
#pragma unroll
  for (int i = 0; i < VPL; ++i) acc[i] = 0.f;
  const int c0 = lane * VPL;  // first value column of this lane
  for (int k0 = k_lo + warp * 32; k0 < k_hi; k0 += kGqaDecWarps * 32) {
    const int key = k0 + lane;
    const bool ok = key < k_hi;
    const size_t prow = ok ? page_row(rg, s, key) : 0;
    float sc = -INFINITY;
    if (ok) {
      const T* kr = (const T*)p.cache + prow * roww + (size_t)g * D;
      float a0 = 0.f, a1 = 0.f;
      if (vec_k) {
#pragma unroll 4
        for (int d = 0; d < D; d += kPer) {
          float f[kPer];
          ld_contig<T, kPer>(kr + d, f);
#pragma unroll
          for (int e = 0; e < kPer; e += 4) {
            const float4 q4 = *reinterpret_cast<const float4*>(qs + d + e);
            a0 = fmaf(q4.x, f[e], a0); a1 = fmaf(q4.y, f[e + 1], a1); a0 = fmaf(q4.z, f[e + 2], a0); a1 = fmaf(q4.w, f[e + 3], a1);
          }
        }
      } else {
        int d = 0;
        for (; d + 1 < D; d += 2) { a0 = fmaf(qs[d], ld_f<T>(kr + d), a0); a1 = fmaf(qs[d + 1], ld_f<T>(kr + d + 1), a1); }
        if (d < D) a0 = fmaf(qs[d], ld_f<T>(kr + d), a0);
      }
      sc = a0 + a1;
    }
    const float m_new = fmaxf(mx, warp_max(sc));
    const float r = mx == -INFINITY ? 0.f : expf(mx - m_new);
    const float w = ok ? expf(sc - m_new) : 0.f;
    sum = sum * r + warp_sum(w);
#pragma unroll
    for (int i = 0; i < VPL; ++i) acc[i] *= r;
    mx = m_new;
    const int nk = min(32, k_hi - k0);
    // eight keys' value rows are requested before any of them is used
    for (int kk0 = 0; kk0 < nk; kk0 += 8) {
      float f[8][VPL], wk[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int kk = kk0 + u;  // (a lane index below 32 in every case: nk <= 32 and kk0 is a multiple of 8)
        wk[u] = __shfl_sync(0xffffffffu, w, kk);
        const unsigned long long pr = __shfl_sync(0xffffffffu, (unsigned long long)prow, kk);
        const T* vr = (const T*)p.cache + (size_t)pr * roww + (size_t)G * D + (size_t)g * V + c0;
        const bool live = kk < nk && c0 < V;
        if (live && vec_v) {
          ld_contig<T, VPL>(vr, f[u]);
        } else {
#pragma unroll
          for (int i = 0; i < VPL; ++i) f[u][i] = (live && c0 + i < V) ? ld_f<T>(vr + i) : 0.f;
        }
      }
#pragma unroll
      for (int u = 0; u < 8; ++u)
#pragma unroll
        for (int i = 0; i < VPL; ++i) acc[i] = fmaf(wk[u], f[u][i], acc[i]);
    }
  }
  float* mine = wp + (size_t)warp * (V + 2);
#pragma unroll
  for (int i = 0; i < VPL; ++i)
    if (c0 + i < V) mine[c0 + i] = acc[i];
  if (lane == 0) { mine[V] = mx; mine[V + 1] = sum; }
  __syncthreads();
  // the warps' parts are joined in warp order
  float m = -INFINITY;
  for (int w = 0; w < kGqaDecWarps; ++w) m = fmaxf(m, wp[(size_t)w * (V + 2) + V]);
  float* dst = p.part + (((size_t)s * H + hd) * p.splits + sp) * (V + 2);
  for (int c = tid; c < V + 1; c += blockDim.x) {
    float a = 0.f;
    for (int w = 0; w < kGqaDecWarps; ++w) {
      const float mw = wp[(size_t)w * (V + 2) + V];
      if (mw != -INFINITY) a = fmaf(expf(mw - m), wp[(size_t)w * (V + 2) + (c < V ? c : V + 1)], a);
    }
    dst[c < V ? c : V + 1] = a;
  }
  if (tid == 0) dst[V] = m;
}

// grid (n_seqs, H): out = sum_j e^(m_j - m) acc_j / (e^(s - m) + sum_j e^(m_j - m) l_j), s the sink's logit (ln of the
// constant, or the head's learned one)
template <typename T>
__global__ void gqa_decode_merge_kernel(const GqaDecodeArgs p, const Ragged rg) {
  const int s = blockIdx.x, hd = blockIdx.y;
  const int row = rg.cu[s];
  if (rg.cu[s + 1] - row != 1) return;
  const int V = p.V, hpg = p.H / p.G, g = hd / hpg;
  const float* part = p.part + ((size_t)s * p.H + hd) * p.splits * (V + 2);
  const float sk = p.sinks ? ld_f<T>((const T*)p.sinks + hd) : (p.sink > 0.f ? logf(p.sink) : -INFINITY);
  float m = sk;
  for (int j = 0; j < p.splits; ++j) m = fmaxf(m, part[(size_t)j * (V + 2) + V]);
  float den = sk == -INFINITY ? 0.f : expf(sk - m);
  for (int j = 0; j < p.splits; ++j) {
    const float mj = part[(size_t)j * (V + 2) + V];
    if (mj != -INFINITY) den += expf(mj - m) * part[(size_t)j * (V + 2) + V + 1];
  }
  const float inv = 1.0f / den;
  float* out = p.out + (((size_t)g * rg.M + row) * hpg + (hd - g * hpg)) * V;
  for (int c = threadIdx.x; c < V; c += blockDim.x) {
    float a = 0.f;
    for (int j = 0; j < p.splits; ++j) {
      const float mj = part[(size_t)j * (V + 2) + V];
      if (mj != -INFINITY) a = fmaf(expf(mj - m), part[(size_t)j * (V + 2) + c], a);
    }
    out[c] = a * inv;
  }
}

// o [G, M, H/G, V] fp32 (group-major) and gate pre-activations gz[m * ldg + h * V + v] -> y [M, H V] (T) = o * sigmoid(gz)
template <typename T>
__global__ void attn_gate_kernel(const float* __restrict__ o, const float* __restrict__ gz, int ldg, T* __restrict__ y, int M, int H,
                                 int G, int V) {
  const int m = blockIdx.x, hpg = H / G;
  for (int i = threadIdx.x; i < H * V; i += blockDim.x) {
    const int hd = i / V, v = i - hd * V, g = hd / hpg;
    const float ov = o[(((size_t)g * M + m) * hpg + (hd - g * hpg)) * V + v];
    st_f<T>(y + (size_t)m * H * V + i, gz ? ov * sigmoid_f(gz[(size_t)m * ldg + i]) : ov);
  }
}

}  // namespace ssdk
