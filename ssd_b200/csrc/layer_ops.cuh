// layer_ops.cuh — the element-wise steps of a layered (hybrid) model's block.  The residual stream, every norm
// statistic and every gate are fp32; T (bf16 or float) is the storage type of the activations that feed a linear layer.
//   embed_rows_kernel         x = embed[token] * scale                          (fp32 residual; optional T copy)
//   offset_rmsnorm_kernel     y = x / sqrt(mean(x^2) + eps) * (offset + w)       (offset 1: unit-offset weight, 0: plain);
//                             optionally a second output with a second weight from the same statistic (two-norm blocks)
//   postnorm_residual_kernel  x += mult * norm(s1 y1 + s2 y2): the norm sits on a sublayer's OUTPUT (serial blocks)
//   glu_act_kernel            y = act(g) * u, act = gelu_tanh | silu
//   bias_act_kernel           y = act(z + b), act = relu^2 | gelu_tanh | silu     (feed-forward without a gate)
//   act_cols_kernel           the same without a bias on rows of any leading dimension (experts without a gate)
//   polynorm_kernel           y = k1 u1 + k2 u2 + k3 u3 + k0, u_p = z^p / rms(z^p) over the row (feed-forward without a gate)
//   token_shift_kernel        RWKV token shift: S mixes h + (h_prev - h) * mu_s, h_prev carried in the state slot
//   head_rmsnorm_gate_kernel  per-head unit RMS, times a channel weight, times silu / sigmoid of a gate pre-activation
//   clamped_glu_kernel        y = g * sigmoid(1.702 g) * (u + 1) with g = min(g, lim), u = clamp(u, -lim, lim)
//   unary_kernel              tanh (decay low-rank bottleneck)
//   block_combine_kernel      parallel block: x += ls1 * g1 * mixer + ls2 * g2 * (sum_k w_k expert_k + sigmoid(sg) * shared + b);
//                             ls1, ls2, sg, b are optional (1, 1, no gate, 0), and so are the per-token, per-channel residual
//                             gates g = sigmoid(pre-activation + bias); an identity expert's output is the feed-forward's
//                             input row itself
#pragma once
#include "common.cuh"
#include "linear.cuh"

namespace ssdk {

// per-step description of a ragged batch, all on the device
struct Ragged {
  const int* cu;        // [n_seqs + 1] first row of every sequence's portion
  const int* pos0;      // [n_seqs] tokens of the sequence that earlier steps already ran
  const int* slot;      // [n_seqs] recurrent-state slot
  const int* tok_seq;   // [M] sequence of a row
  const int* tables;    // [n_seqs, max_blocks] page table
  int n_seqs, M, max_blocks, block_size;
};

// N contiguous elements of storage type T -> floats, with the widest loads their size allows (the caller guarantees that
// p is aligned to min(16, N * sizeof(T)) bytes)
template <typename T, int N>
SSDK_DEVINL void ld_contig(const T* p, float* f) {
  constexpr int kBytes = N * (int)sizeof(T);
  if constexpr (kBytes % 16 == 0) {
    uint32_t w[kBytes / 4];
#pragma unroll
    for (int i = 0; i < kBytes / 16; ++i) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(p) + i);
      w[4 * i] = v.x; w[4 * i + 1] = v.y; w[4 * i + 2] = v.z; w[4 * i + 3] = v.w;
    }
#pragma unroll
    for (int i = 0; i < N; ++i) {
      if constexpr (sizeof(T) == 4) f[i] = __uint_as_float(w[i]);
      else f[i] = __uint_as_float((i & 1) ? (w[i >> 1] & 0xffff0000u) : (w[i >> 1] << 16));
    }
  } else if constexpr (kBytes == 8) {
    const uint2 v = __ldg(reinterpret_cast<const uint2*>(p));
    if constexpr (sizeof(T) == 4) { f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y); }
    else { f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xffff0000u); f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xffff0000u); }
  } else if constexpr (kBytes == 4 && sizeof(T) == 2) {
    const uint32_t v = __ldg(reinterpret_cast<const uint32_t*>(p));
    f[0] = __uint_as_float(v << 16); f[1] = __uint_as_float(v & 0xffff0000u);
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i) f[i] = ld_f<T>(p + i);
  }
}

// N floats -> N contiguous elements of storage type T (p aligned to min(16, N * sizeof(T)) bytes, N * sizeof(T) a multiple of 16)
template <typename T, int N>
SSDK_DEVINL void st_contig(T* p, const float* f) {
  constexpr int kBytes = N * (int)sizeof(T);
  static_assert(kBytes % 16 == 0, "st_contig writes whole 16-byte pieces");
  uint32_t w[kBytes / 4];
#pragma unroll
  for (int i = 0; i < kBytes / 4; ++i) {
    if constexpr (sizeof(T) == 4) {
      w[i] = __float_as_uint(f[i]);
    } else {
      const __nv_bfloat162 v = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&v);
    }
  }
#pragma unroll
  for (int i = 0; i < kBytes / 16; ++i) reinterpret_cast<uint4*>(p)[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
}

template <typename T>
__global__ void embed_rows_kernel(const int* __restrict__ ids, const T* __restrict__ embed, float* __restrict__ x, int width,
                                  int vocab, float scale, T* __restrict__ xt) {
  const int m = blockIdx.x;
  int id = ids[m];
  id = min(max(id, 0), vocab - 1);
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float v = ld_f<T>(embed + (size_t)id * width + c) * scale;
    x[(size_t)m * width + c] = v;
    if (xt) st_f<T>(xt + (size_t)m * width + c, v);
  }
}

// rows: optional gather (row r of the output reads x[rows[r]]).  w2 / y2 (optional): a second norm of the same row
// with its own weight — the statistic is shared, so a block whose mixer and feed-forward each have a norm reads x once.
template <typename T>
__global__ void offset_rmsnorm_kernel(const float* __restrict__ x, const T* __restrict__ w, T* __restrict__ y,
                                      const int* __restrict__ rows, int width, float eps, float offset,
                                      const T* __restrict__ w2, T* __restrict__ y2) {
  __shared__ float red[33];
  const int r = blockIdx.x;
  const float* xr = x + (size_t)(rows ? rows[r] : r) * width;
  float ss = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) { const float v = xr[c]; ss = fmaf(v, v, ss); }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)width + eps);
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float v = xr[c] * inv;
    st_f<T>(y + (size_t)r * width + c, v * (offset + ld_f<T>(w + c)));
    if (y2) st_f<T>(y2 + (size_t)r * width + c, v * (offset + ld_f<T>(w2 + c)));
  }
}

// Serial post-norm block: x[m] += mult * (y / sqrt(mean(y^2) + eps)) * (offset + w) with y = s1 y1[m] (+ s2 y2[m]); the
// updated row is also written in the storage type (xt, may be null) for the next sublayer's projections.
template <typename T>
__global__ void postnorm_residual_kernel(float* __restrict__ x, const float* __restrict__ y1, float s1, const float* __restrict__ y2,
                                         float s2, const T* __restrict__ w, int width, float eps, float offset, float mult,
                                         T* __restrict__ xt) {
  __shared__ float red[33];
  const size_t base = (size_t)blockIdx.x * width;
  float ss = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float v = y2 ? fmaf(s2, y2[base + c], s1 * y1[base + c]) : s1 * y1[base + c];
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)width + eps);
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float v = y2 ? fmaf(s2, y2[base + c], s1 * y1[base + c]) : s1 * y1[base + c];
    const float xn = fmaf(mult, v * inv * (offset + ld_f<T>(w + c)), x[base + c]);
    x[base + c] = xn;
    if (xt) st_f<T>(xt + base + c, xn);
  }
}

SSDK_DEVINL float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }

// ACT: the SSDK_ACT_* values of the C ABI (1 silu, 2 gelu_tanh, 3 squared relu)
template <int ACT>
SSDK_DEVINL float act_f(float g) {
  if (ACT == 1) return g * sigmoid_f(g);
  if (ACT == 2) return 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
  const float r = fmaxf(g, 0.f);
  return r * r;
}

// z [rows, ldz] fp32 with gate columns [0, ff) and up columns [ff, 2 ff) -> y [rows, ff] (T) = act(gate) * up; rows at
// and beyond *n_rows (optional, on the device) are skipped
template <typename T, int ACT>
__global__ void glu_act_kernel(const float* __restrict__ z, int ldz, T* __restrict__ y, int ff, const int* __restrict__ n_rows) {
  const int r = blockIdx.x;
  if (n_rows && r >= *n_rows) return;
  for (int c = threadIdx.x; c < ff; c += blockDim.x)
    st_f<T>(y + (size_t)r * ff + c, act_f<ACT>(z[(size_t)r * ldz + c]) * z[(size_t)r * ldz + ff + c]);
}

// z [rows, ff] fp32, b [ff] (T, optional) -> y [rows, ff] (T) = act(z + b)
template <typename T, int ACT>
__global__ void bias_act_kernel(const float* __restrict__ z, const T* __restrict__ b, T* __restrict__ y, int ff) {
  const int r = blockIdx.x;
  for (int c = threadIdx.x; c < ff; c += blockDim.x)
    st_f<T>(y + (size_t)r * ff + c, act_f<ACT>(z[(size_t)r * ff + c] + (b ? ld_f<T>(b + c) : 0.f)));
}

// z [rows, ldz] fp32 -> y [rows, ff] (T) = act(z); rows at and beyond *n_rows (optional, on the device) are skipped
template <typename T, int ACT>
__global__ void act_cols_kernel(const float* __restrict__ z, int ldz, T* __restrict__ y, int ff, const int* __restrict__ n_rows) {
  const int r = blockIdx.x;
  if (n_rows && r >= *n_rows) return;
  for (int c = threadIdx.x; c < ff; c += blockDim.x) st_f<T>(y + (size_t)r * ff + c, act_f<ACT>(z[(size_t)r * ldz + c]));
}

// z [rows, ff] fp32, coef [4] (T) = k1, k2, k3, k0 -> y [rows, ff] (T) = k1 z / r1 + k2 z^2 / r2 + k3 z^3 / r3 + k0 with
// r_p = sqrt(mean over the row of z^(2p) + eps): three unit-RMS powers of the row, all in fp32
template <typename T>
__global__ void polynorm_kernel(const float* __restrict__ z, const T* __restrict__ coef, T* __restrict__ y, int ff, float eps) {
  __shared__ float red[33];
  const float* zr = z + (size_t)blockIdx.x * ff;
  float s1 = 0.f, s2 = 0.f, s3 = 0.f;
  for (int c = threadIdx.x; c < ff; c += blockDim.x) {
    const float v = zr[c], v2 = v * v;
    s1 += v2; s2 = fmaf(v2, v2, s2); s3 = fmaf(v2 * v, v2 * v, s3);
  }
  s1 = block_sum(s1, red); s2 = block_sum(s2, red); s3 = block_sum(s3, red);
  const float a = ld_f<T>(coef) / sqrtf(s1 / (float)ff + eps), b = ld_f<T>(coef + 1) / sqrtf(s2 / (float)ff + eps),
              g = ld_f<T>(coef + 2) / sqrtf(s3 / (float)ff + eps), e = ld_f<T>(coef + 3);
  for (int c = threadIdx.x; c < ff; c += blockDim.x) {
    const float v = zr[c];
    st_f<T>(y + (size_t)blockIdx.x * ff + c, fmaf(v, fmaf(v, fmaf(v, g, b), a), e));
  }
}

// mixes[s][m][c] = h[m][c] + (prev[m][c] - h[m][c]) * mu[s][c]; prev of a portion's first row comes from the slot
// (zero at position 0).  h_prev is NOT written here: the scan kernel of the same layer saves the portion's last row after
// every row of this kernel has read the old one (stream order).
template <typename T>
__global__ void token_shift_kernel(const T* __restrict__ h, const T* __restrict__ mu, const float* __restrict__ h_prev,
                                   size_t slot_stride, T* __restrict__ mixes, Ragged rg, int width, int n_mix) {
  const int m = blockIdx.x, s = rg.tok_seq[m];
  const bool first = m == rg.cu[s];
  const float* prev_state = (first && rg.pos0[s] > 0) ? h_prev + (size_t)rg.slot[s] * slot_stride : nullptr;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float cur = ld_f<T>(h + (size_t)m * width + c);
    const float prev = first ? (prev_state ? prev_state[c] : 0.f) : ld_f<T>(h + (size_t)(m - 1) * width + c);
    const float d = prev - cur;
    for (int k = 0; k < n_mix; ++k)
      st_f<T>(mixes + ((size_t)k * rg.M + m) * width + c, fmaf(d, ld_f<T>(mu + (size_t)k * width + c), cur));
  }
}

// o [M, H, V] fp32 -> y [M, H*V] (T): o / rms(o) * w * act(g);  GATE: 0 = silu, 1 = sigmoid
template <typename T, int GATE>
__global__ void head_rmsnorm_gate_kernel(const float* __restrict__ o, const float* __restrict__ g, int ldg,
                                         const T* __restrict__ w, T* __restrict__ y, int H, int V, float eps) {
  __shared__ float red[33];
  const int m = blockIdx.x, hd = blockIdx.y;
  const float* orow = o + ((size_t)m * H + hd) * V;
  float ss = 0.f;
  for (int j = threadIdx.x; j < V; j += blockDim.x) ss = fmaf(orow[j], orow[j], ss);
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)V + eps);
  for (int j = threadIdx.x; j < V; j += blockDim.x) {
    const float gz = g[(size_t)m * ldg + hd * V + j];
    const float ga = GATE == 0 ? gz * sigmoid_f(gz) : sigmoid_f(gz);
    st_f<T>(y + (size_t)m * H * V + hd * V + j, orow[j] * inv * ld_f<T>(w + hd * V + j) * ga);
  }
}

// z [rows, ldz] fp32 with gate columns [0, ff) and up columns [ff, 2 ff) -> y [rows, ff] (T)
template <typename T>
__global__ void clamped_glu_kernel(const float* __restrict__ z, int ldz, T* __restrict__ y, int ff, float limit,
                                   const int* __restrict__ n_rows) {
  const int r = blockIdx.x;
  if (n_rows && r >= *n_rows) return;
  for (int c = threadIdx.x; c < ff; c += blockDim.x) {
    const float g = fminf(z[(size_t)r * ldz + c], limit);
    const float u = fminf(fmaxf(z[(size_t)r * ldz + ff + c], -limit), limit);
    st_f<T>(y + (size_t)r * ff + c, g * sigmoid_f(1.702f * g) * (u + 1.0f));
  }
}

template <typename T>
__global__ void tanh_rows_kernel(const float* __restrict__ z, T* __restrict__ y, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    st_f<T>(y + i, tanhf(z[i]));
}

__global__ void f32_to_bf16_kernel(const float* __restrict__ z, __nv_bfloat16* __restrict__ y, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    y[i] = __float2bfloat16_rn(z[i]);
}

// out[i] = sum over s of partials[s][i] in the fixed order s = 0 .. S-1 (split-K of the tcgen05 GEMM, fp32)
__global__ void splitk_sum_kernel(const float* __restrict__ partials, float* __restrict__ out, int S, size_t n) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float a = partials[i];
  for (int s = 1; s < S; ++s) a += partials[(size_t)s * n + i];
  out[i] = a;
}

struct CombineArgs {
  float* x;              // [M, width] residual, updated in place
  const float* mix;      // [M, width] mixer output (after its output projection)
  const void* ls1;       // [width] T or nullptr (no layer scale)
  const void* ls2;       // [width] T or nullptr (no layer scale on the feed-forward)
  const float* routed;   // [M * top, width] expert outputs in assignment order, or nullptr
  const int* apos;       // [M * top] row of (token, k) in `routed`
  const float* wts;      // [M * top] routing weights
  int top;
  const float* shared;   // [M, width] output of the shared expert or of a dense feed-forward, or nullptr
  const float* sg;       // shared gate pre-activation: sg[m * ld_sg], or nullptr (no gate)
  int ld_sg;
  int width;
  const void* ff_bias;   // [width] T bias of the feed-forward's output, or nullptr
  const int* sel;        // [M * top] chosen router output; outputs >= n_real are identity experts (nullptr: there are none)
  int n_real;
  const void* fin;       // [M, width] T the feed-forward's input (what an identity expert returns)
  const float* gz;       // [M, ld_gz] pre-activations of the residual gates: mixer's in columns [0, width), feed-forward's in
  int ld_gz;             //   [width, 2 width); nullptr: no gates
  const void* gz_bias;   // [2 width] T
};
template <typename T>
__global__ void block_combine_kernel(const CombineArgs p) {
  const int m = blockIdx.x;
  const float sgate = (p.shared && p.sg) ? sigmoid_f(p.sg[(size_t)m * p.ld_sg]) : 1.f;
  for (int c = threadIdx.x; c < p.width; c += blockDim.x) {
    float y = p.mix[(size_t)m * p.width + c];
    if (p.ls1) y *= ld_f<T>((const T*)p.ls1 + c);
    if (p.gz) y *= sigmoid_f(p.gz[(size_t)m * p.ld_gz + c] + ld_f<T>((const T*)p.gz_bias + c));
    if (p.routed || p.shared) {
      float f = 0.f;
      if (p.routed)
        for (int k = 0; k < p.top; ++k) {
          const size_t a = (size_t)m * p.top + k;
          const float v = (p.sel && p.sel[a] >= p.n_real) ? ld_f<T>((const T*)p.fin + (size_t)m * p.width + c)
                                                          : p.routed[(size_t)p.apos[a] * p.width + c];
          f = fmaf(p.wts[a], v, f);
        }
      if (p.shared) f = fmaf(sgate, p.shared[(size_t)m * p.width + c], f);
      if (p.ff_bias) f += ld_f<T>((const T*)p.ff_bias + c);
      if (p.gz) f *= sigmoid_f(p.gz[(size_t)m * p.ld_gz + p.width + c] + ld_f<T>((const T*)p.gz_bias + p.width + c));
      y = p.ls2 ? fmaf(ld_f<T>((const T*)p.ls2 + c), f, y) : y + f;
    }
    p.x[(size_t)m * p.width + c] += y;
  }
}

}  // namespace ssdk
