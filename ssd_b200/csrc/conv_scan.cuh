// conv_scan.cuh — recurrent mixers that sit behind a short causal convolution, for the layered (hybrid) models.
// Everything here is fp32: the convolution, its activation, gates, decays, step sizes and the carried state; T (bf16 or
// float) is only the storage type of weights and of the rows handed to the next linear layer.
//
//   short_conv_kernel     per-channel causal convolution over time (taps from the checkpoint, last tap = current token),
//                         optional input bias / output bias / SiLU; rows before the portion come from the state slot,
//                         zeros before the sequence
//   conv_state_kernel     saves the last taps - 1 inputs of every sequence's portion into its slot (runs after the readers)
//   input_conv_kernel     a block's input convolutions: y_k = h + conv_k(h) for up to two tap sets over the same rows h (T),
//                         no bias; input_conv_state_kernel saves the last taps - 1 rows of h
//   rglru_scan_kernel     S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t,  a_t = exp(-c r_t softplus(lam)),  out = S_t gelu(y_t)
//   selective_scan_kernel S[c,n] = exp(dt_c A[c,n]) S[c,n] + dt_c x_c B_n,  y_c = sum_n S[c,n] C_n + D_c x_c,  out = y silu(z)
//   delta_prep_kernel     convolution + SiLU of q | k | v, unit vectors per head for q and k, beta and the head decay
//   delta_scan_kernel     gated delta rule: S = g S; u = beta (v - S^T k); S += k u^T; o = S^T q
//
// A state slot is never cleared: a sequence whose portion starts at position 0 ignores what the slot holds.
#pragma once
#include "layer_ops.cuh"
#include "recurrent.cuh"  // cp_async4

namespace ssdk {

SSDK_DEVINL float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }
SSDK_DEVINL float silu_f(float z) { return z * sigmoid_f(z); }
SSDK_DEVINL float gelu_tanh_f(float z) { return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z))); }

struct ConvArgs {
  const float* in;      // [M, ld_in] rows before the convolution; channel c is column c
  int ld_in;
  const void* in_bias;  // [C] T added to every input row (not to the zeros before the sequence), or nullptr
  const void* w;        // [C, taps] T
  const void* bias;     // [C] T added to the result, or nullptr
  float* out;           // [M, ld_out] fp32, or nullptr
  int ld_out;
  void* out_t;          // [M, ld_t] T copy for a following linear layer, or nullptr
  int ld_t;
  float* hist;          // state: [taps - 1, C] per slot (with the input bias already added), oldest first
  size_t slot_stride;
  int C, taps;
};

// value of channel c at row m (row t of sequence s) after the convolution, before any activation
template <typename T>
SSDK_DEVINL float conv_at(const ConvArgs& p, const Ragged& rg, int m, int s, int t, int c) {
  float acc = p.bias ? ld_f<T>((const T*)p.bias + c) : 0.f;
  const float ib = p.in_bias ? ld_f<T>((const T*)p.in_bias + c) : 0.f;
  const bool carried = rg.pos0[s] > 0;
  const float* hist = p.hist + (size_t)rg.slot[s] * p.slot_stride;
  for (int j = 0; j < p.taps; ++j) {
    const int back = p.taps - 1 - j;
    float v;
    if (back <= t) v = p.in[(size_t)(m - back) * p.ld_in + c] + ib;
    else v = carried ? hist[(size_t)(p.taps - 1 - (back - t)) * p.C + c] : 0.f;
    acc = fmaf(ld_f<T>((const T*)p.w + (size_t)c * p.taps + j), v, acc);
  }
  return acc;
}

// ACT: 0 none, 1 SiLU.  grid (M, ceil(C / blockDim))
template <typename T, int ACT>
__global__ void short_conv_kernel(const ConvArgs p, const Ragged rg) {
  const int m = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= p.C) return;
  const int s = rg.tok_seq[m];
  float v = conv_at<T>(p, rg, m, s, m - rg.cu[s], c);
  if (ACT == 1) v = silu_f(v);
  if (p.out) p.out[(size_t)m * p.ld_out + c] = v;
  if (p.out_t) st_f<T>((T*)p.out_t + (size_t)m * p.ld_t + c, v);
}

// grid (n_seqs, ceil(C / blockDim)).  New history = the last taps - 1 entries of (old history ++ this portion's inputs);
// entry j is read from an index above j, so one thread per channel may work in place in ascending order.
template <typename T>
__global__ void conv_state_kernel(const ConvArgs p, const Ragged rg) {
  const int s = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= p.C) return;
  const int r0 = rg.cu[s], n = rg.cu[s + 1] - r0, keep = p.taps - 1;
  const bool carried = rg.pos0[s] > 0;
  const float ib = p.in_bias ? ld_f<T>((const T*)p.in_bias + c) : 0.f;
  float* hist = p.hist + (size_t)rg.slot[s] * p.slot_stride;
  for (int j = 0; j < keep; ++j) {
    const int idx = n + j;
    float v;
    if (idx < keep) v = carried ? hist[(size_t)idx * p.C + c] : 0.f;
    else v = p.in[(size_t)(r0 + idx - keep) * p.ld_in + c] + ib;
    hist[(size_t)j * p.C + c] = v;
  }
}

// Residual input convolution of a block's sublayers.  h [M, C] (T) are the rows both sublayers read; sublayer k gets
// y_k[m, c] = h[m, c] + sum_j w_k[c, j] h[row of position t - taps + 1 + j, c] with zeros before the sequence's start and the
// rows before the portion taken from the state slot (hist [taps - 1, C] fp32 per slot, oldest first).  Sums in fp32.
struct InputConvArgs {
  const void* h;        // [M, C] T
  const void* w;        // [2, C, taps] T: taps of y1, then of y2
  void* y1;             // [M, C] T
  void* y2;             // [M, C] T or nullptr
  float* hist; size_t slot_stride;
  int C, taps;
};

// grid (M, ceil(C / blockDim)): one channel per thread, any number of taps
template <typename T>
__global__ void input_conv_kernel(const InputConvArgs p, const Ragged rg) {
  const int m = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= p.C) return;
  const int s = rg.tok_seq[m], t = m - rg.cu[s];
  const bool carried = rg.pos0[s] > 0;
  const float* hist = p.hist + (size_t)rg.slot[s] * p.slot_stride;
  const T* h = (const T*)p.h;
  const T* w1 = (const T*)p.w + (size_t)c * p.taps;
  const T* w2 = w1 + (size_t)p.C * p.taps;
  const float cur = ld_f<T>(h + (size_t)m * p.C + c);
  float a1 = 0.f, a2 = 0.f;
  for (int j = 0; j < p.taps; ++j) {
    const int back = p.taps - 1 - j;
    float v;
    if (back == 0) v = cur;
    else if (back <= t) v = ld_f<T>(h + (size_t)(m - back) * p.C + c);
    else v = carried ? hist[(size_t)(p.taps - 1 - (back - t)) * p.C + c] : 0.f;
    a1 = fmaf(ld_f<T>(w1 + j), v, a1);
    if (p.y2) a2 = fmaf(ld_f<T>(w2 + j), v, a2);
  }
  st_f<T>((T*)p.y1 + (size_t)m * p.C + c, cur + a1);
  if (p.y2) st_f<T>((T*)p.y2 + (size_t)m * p.C + c, cur + a2);
}

// The same with 16 bytes of channels per thread (8 bf16 or 4 floats) and the taps in registers: C a multiple of that,
// rows and taps 16-byte aligned.  grid (M, ceil(C / VEC / blockDim)).  Same sums in the same order as the scalar form.
template <typename T, int TAPS>
__global__ void input_conv_vec_kernel(const InputConvArgs p, const Ragged rg) {
  constexpr int VEC = 16 / (int)sizeof(T);
  const int m = blockIdx.x, c = (blockIdx.y * blockDim.x + threadIdx.x) * VEC;
  if (c >= p.C) return;
  const int s = rg.tok_seq[m], t = m - rg.cu[s];
  const bool carried = rg.pos0[s] > 0;
  const float* hist = p.hist + (size_t)rg.slot[s] * p.slot_stride;
  const T* h = (const T*)p.h;
  float w1[VEC * TAPS], w2[VEC * TAPS];   // entry e * TAPS + j: channel c + e, tap j
  ld_contig<T, VEC * TAPS>((const T*)p.w + (size_t)c * TAPS, w1);
  if (p.y2) ld_contig<T, VEC * TAPS>((const T*)p.w + ((size_t)p.C + c) * TAPS, w2);
  float cur[VEC], a1[VEC], a2[VEC];
  ld_contig<T, VEC>(h + (size_t)m * p.C + c, cur);
#pragma unroll
  for (int e = 0; e < VEC; ++e) a1[e] = a2[e] = 0.f;
#pragma unroll
  for (int j = 0; j < TAPS; ++j) {
    const int back = TAPS - 1 - j;
    float v[VEC];
    if (back == 0) {
#pragma unroll
      for (int e = 0; e < VEC; ++e) v[e] = cur[e];
    } else if (back <= t) {
      ld_contig<T, VEC>(h + (size_t)(m - back) * p.C + c, v);
    } else if (carried) {
      ld_contig<float, VEC>(hist + (size_t)(TAPS - 1 - (back - t)) * p.C + c, v);
    } else {
#pragma unroll
      for (int e = 0; e < VEC; ++e) v[e] = 0.f;
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      a1[e] = fmaf(w1[e * TAPS + j], v[e], a1[e]);
      if (p.y2) a2[e] = fmaf(w2[e * TAPS + j], v[e], a2[e]);
    }
  }
#pragma unroll
  for (int e = 0; e < VEC; ++e) { a1[e] += cur[e]; a2[e] += cur[e]; }
  st_contig<T, VEC>((T*)p.y1 + (size_t)m * p.C + c, a1);
  if (p.y2) st_contig<T, VEC>((T*)p.y2 + (size_t)m * p.C + c, a2);
}

// grid (n_seqs, ceil(C / blockDim)); runs after input_conv_kernel.  As conv_state_kernel: entry j is read from an index
// above j, so one thread per channel works in place in ascending order.
template <typename T>
__global__ void input_conv_state_kernel(const InputConvArgs p, const Ragged rg) {
  const int s = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= p.C) return;
  const int r0 = rg.cu[s], n = rg.cu[s + 1] - r0, keep = p.taps - 1;
  const bool carried = rg.pos0[s] > 0;
  float* hist = p.hist + (size_t)rg.slot[s] * p.slot_stride;
  for (int j = 0; j < keep; ++j) {
    const int idx = n + j;
    float v;
    if (idx < keep) v = carried ? hist[(size_t)idx * p.C + c] : 0.f;
    else v = ld_f<T>((const T*)p.h + (size_t)(r0 + idx - keep) * p.C + c);
    hist[(size_t)j * p.C + c] = v;
  }
}

// fp32 columns -> T columns (operand of a following linear layer)
template <typename T>
__global__ void cast_cols_kernel(const float* __restrict__ src, int ld_src, T* __restrict__ dst, int ld_dst, int cols) {
  const int m = blockIdx.x;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) st_f<T>(dst + (size_t)m * ld_dst + c, src[(size_t)m * ld_src + c]);
}

// ---------------------------------------------------------------------------------------------- rglru
struct RglruArgs {
  const float* u; int ld_u;          // [M, R] convolved x branch
  const float* gates; int ld_g;      // [M, blocks * 2 bs]: per block recurrence-gate slots, then input-gate slots
                                     // (pre-activations before rglru_gate_kernel, decay a and input term b after it)
  const void* gate_bias;             // [blocks, 2 bs] T
  const void* lam;                   // [R] T
  const float* y; int ld_y;          // [M, ...] y branch (pre-activation before rglru_gate_kernel, gelu after)
  const void* y_bias;                // [R] T
  void* out;                         // [M, R] T: S * gelu_tanh(y)
  float* S; size_t slot_stride;      // [R] per slot
  int R, bs;
  float decay_mult;
};

// grid (M, ceil(R / blockDim)): everything of a row that does not depend on the state, for all rows at once and in place:
// gates[m][recurrence slot] <- a = exp(-c r softplus(lam)), gates[m][input slot] <- sqrt(1 - a^2) i u,
// y[m] <- gelu_tanh(y[m] + bias)
template <typename T>
__global__ void rglru_gate_kernel(const RglruArgs p, float* __restrict__ gates, float* __restrict__ y) {
  const int m = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= p.R) return;
  const int b = c / p.bs, cb = c - b * p.bs;
  const int gr = b * 2 * p.bs + cb, gi = gr + p.bs;
  const float sp = softplus_f(ld_f<T>((const T*)p.lam + c)) * p.decay_mult;
  float* grow = gates + (size_t)m * p.ld_g;
  const float log_a = -sigmoid_f(grow[gr] + ld_f<T>((const T*)p.gate_bias + gr)) * sp;
  const float i = sigmoid_f(grow[gi] + ld_f<T>((const T*)p.gate_bias + gi));
  grow[gr] = expf(log_a);
  // 1 - a^2 through expm1: exact also where a is within an ulp of 1
  grow[gi] = sqrtf(-expm1f(2.0f * log_a)) * i * p.u[(size_t)m * p.ld_u + c];
  float* yp = y + (size_t)m * p.ld_y + c;
  *yp = gelu_tanh_f(*yp + ld_f<T>((const T*)p.y_bias + c));
}

constexpr int kRglruRows = 16;  // rows whose operands are requested together

// grid (n_seqs, ceil(R / blockDim)): one thread per channel walks its sequence's rows, S = a S + b, out = S y, with the
// operands rglru_gate_kernel left (sixteen rows' loads in flight at a time).
template <typename T>
__global__ void rglru_scan_kernel(const RglruArgs p, const Ragged rg) {
  const int s = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= p.R) return;
  const int b = c / p.bs, cb = c - b * p.bs;
  const int gr = b * 2 * p.bs + cb, gi = gr + p.bs;
  float* Sp = p.S + (size_t)rg.slot[s] * p.slot_stride + c;
  float S = rg.pos0[s] > 0 ? *Sp : 0.f;
  const int r0 = rg.cu[s], r1 = rg.cu[s + 1];
  for (int m0 = r0; m0 < r1; m0 += kRglruRows) {
    float a[kRglruRows], bb[kRglruRows], y[kRglruRows];
#pragma unroll
    for (int k = 0; k < kRglruRows; ++k) {
      const int m = min(m0 + k, r1 - 1);
      a[k] = p.gates[(size_t)m * p.ld_g + gr]; bb[k] = p.gates[(size_t)m * p.ld_g + gi]; y[k] = p.y[(size_t)m * p.ld_y + c];
    }
#pragma unroll
    for (int k = 0; k < kRglruRows; ++k) {
      if (m0 + k < r1) {
        S = fmaf(a[k], S, bb[k]);
        st_f<T>((T*)p.out + (size_t)(m0 + k) * p.R + c, S * y[k]);
      }
    }
  }
  *Sp = S;
}

// ---------------------------------------------------------------------------------------------- selective scan
struct SelScanArgs {
  const float* x; int ld_x;          // [M, inner] convolved, SiLU'd input
  const float* dtz; int ld_dt;       // [M, inner] step sizes (after softplus)
  const float* bc; int ld_bc;        // [M, ...]: B in columns [0, N), C in [N, 2N)
  const void* A_log;                 // [inner, N] T
  const void* Dw;                    // [inner] T
  const float* z; int ld_z;          // [M, inner] gate values silu(z)
  void* out;                         // [M, inner] T: y * silu(z)
  float* S; size_t slot_stride;      // [inner, N] per slot
  int inner, N;
};

// grid (M, ceil(inner / blockDim)): the state-independent part of a row, in place: dtz <- softplus(dtz + bias), z <- silu(z)
template <typename T>
__global__ void selective_gate_kernel(float* __restrict__ dtz, int ld_dt, const T* __restrict__ dt_bias, float* __restrict__ z, int ld_z,
                                      int inner) {
  const int m = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= inner) return;
  float* d = dtz + (size_t)m * ld_dt + c;
  *d = softplus_f(*d + ld_f<T>(dt_bias + c));
  float* zp = z + (size_t)m * ld_z + c;
  *zp = silu_f(*zp);
}

constexpr int kSelRows = 8;  // rows whose inputs are requested (and whose B | C are staged) together

// A channel's N states are spread over LPC = blockDim.x lanes of a warp (a power of two), NT states per lane in
// registers (N <= NT * LPC); blockDim.y channels per CTA, grid (n_seqs, ceil(inner / blockDim.y)).  Per row a lane
// advances its states and the lanes' parts of y = sum_n S[n] C[n] meet by shuffle (a fixed tree).  exp(dt A) is taken as
// exp2(dt (A log2 e)).  dtz holds the step sizes and z the gate values selective_gate_kernel left.  NT == 0: any N, one
// lane per channel, the state stays in its slot (global memory).  dynamic shared memory: kSelRows * 2 N floats.
template <typename T, int NT>
__global__ void selective_scan_kernel(const SelScanArgs p, const Ragged rg) {
  extern __shared__ float sel_sm[];
  const int s = blockIdx.x, lpc = blockDim.x, ln = threadIdx.x, N = p.N;
  const int c = blockIdx.y * blockDim.y + threadIdx.y, tid = threadIdx.y * lpc + ln, nthr = lpc * blockDim.y;
  const bool live = c < p.inner;
  const bool carried = rg.pos0[s] > 0;
  const int n0 = ln * NT;  // first state of this lane
  float A2[NT > 0 ? NT : 1], S[NT > 0 ? NT : 1];
  float* Sg = p.S + (size_t)rg.slot[s] * p.slot_stride + (size_t)(live ? c : 0) * N;
  if (NT > 0) {
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      const bool ok = live && n0 + n < N;
      A2[n] = ok ? -expf(ld_f<T>((const T*)p.A_log + (size_t)c * N + n0 + n)) * 1.4426950408889634f : 0.f;
      S[n] = (ok && carried) ? Sg[n0 + n] : 0.f;
    }
  } else if (live && !carried) {
    for (int n = 0; n < N; ++n) Sg[n] = 0.f;
  }
  const float Dc = live ? ld_f<T>((const T*)p.Dw + c) : 0.f;
  const int r0 = rg.cu[s], r1 = rg.cu[s + 1], cc = live ? c : 0;
  for (int m0 = r0; m0 < r1; m0 += kSelRows) {
    const int nr = min(kSelRows, r1 - m0);
    float dt[kSelRows], xv[kSelRows], zv[kSelRows];
#pragma unroll
    for (int r = 0; r < kSelRows; ++r) {
      const int m = min(m0 + r, r1 - 1);
      dt[r] = p.dtz[(size_t)m * p.ld_dt + cc]; xv[r] = p.x[(size_t)m * p.ld_x + cc]; zv[r] = p.z[(size_t)m * p.ld_z + cc];
    }
    __syncthreads();
    for (int i = tid; i < nr * 2 * N; i += nthr) {
      const int r = i / (2 * N), k = i - r * 2 * N;
      sel_sm[i] = p.bc[(size_t)(m0 + r) * p.ld_bc + k];
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < kSelRows; ++r) {
      if (r < nr) {
        const int m = m0 + r;
        const float dx = dt[r] * xv[r];
        const float* B = sel_sm + r * 2 * N;
        const float* Cm = B + N;
        float y = 0.f;
        if (NT > 0) {
#pragma unroll
          for (int n = 0; n < NT; ++n) {
            if (n0 + n < N) {
              S[n] = fmaf(exp2f(dt[r] * A2[n]), S[n], dx * B[n0 + n]);
              y = fmaf(S[n], Cm[n0 + n], y);
            }
          }
          for (int o = lpc >> 1; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
        } else if (live) {
          for (int n = 0; n < N; ++n) {
            const float a = -expf(ld_f<T>((const T*)p.A_log + (size_t)c * N + n));
            const float sn = fmaf(expf(dt[r] * a), Sg[n], dx * B[n]);
            Sg[n] = sn;
            y = fmaf(sn, Cm[n], y);
          }
        }
        if (live && ln == 0) st_f<T>((T*)p.out + (size_t)m * p.inner + c, fmaf(Dc, xv[r], y) * zv[r]);
      }
    }
  }
  if (NT > 0 && live) {
#pragma unroll
    for (int n = 0; n < NT; ++n)
      if (n0 + n < N) Sg[n0 + n] = S[n];
  }
}

// ---------------------------------------------------------------------------------------------- gated delta rule
struct DeltaPrepArgs {
  ConvArgs conv;          // over the q | k | v columns (C = 2 G D + H V); out / out_t unused
  const float* ba; int ld_ba;  // [M, ...]: beta pre-activations in columns [0, H), decay pre-activations in [H, 2H)
  const void* A_log;      // [H] T
  const void* dt_bias;    // [H] T
  float* q;               // [M, G D] unit vectors * q_scale
  float* k;               // [M, G D] unit vectors
  float* v;               // [M, H V]
  float* beta;            // [M, H]
  float* decay;           // [M, H]
  int H, G, D, V;
  float q_scale, unit_eps;
};

// grid (M, 2 G + H): unit u < G is a query head, u < 2 G a key head, the rest value heads; one CTA convolves the unit's
// channels (SiLU), and makes a query or key head a unit vector.  dynamic shared memory: max(D, V) floats.
template <typename T>
__global__ void delta_prep_kernel(const DeltaPrepArgs p, const Ragged rg) {
  extern __shared__ float dp_sm[];
  __shared__ float red[33];
  const int m = blockIdx.x, unit = blockIdx.y, s = rg.tok_seq[m], t = m - rg.cu[s];
  const int GD = p.G * p.D, HV = p.H * p.V;
  if (unit == 0) {
    for (int h = threadIdx.x; h < p.H; h += blockDim.x) {
      p.beta[(size_t)m * p.H + h] = sigmoid_f(p.ba[(size_t)m * p.ld_ba + h]);
      const float sp = softplus_f(p.ba[(size_t)m * p.ld_ba + p.H + h] + ld_f<T>((const T*)p.dt_bias + h));
      p.decay[(size_t)m * p.H + h] = expf(-expf(ld_f<T>((const T*)p.A_log + h)) * sp);
    }
  }
  if (unit >= 2 * p.G) {  // a value head: convolution and SiLU only
    const int c0 = 2 * GD + (unit - 2 * p.G) * p.V;
    for (int d = threadIdx.x; d < p.V; d += blockDim.x)
      p.v[(size_t)m * HV + (size_t)(unit - 2 * p.G) * p.V + d] = silu_f(conv_at<T>(p.conv, rg, m, s, t, c0 + d));
    return;
  }
  const int c0 = unit * p.D;  // q heads, then k heads, in the order of the convolution's channels
  float ss = 0.f;
  for (int d = threadIdx.x; d < p.D; d += blockDim.x) {
    const float v = silu_f(conv_at<T>(p.conv, rg, m, s, t, c0 + d));
    dp_sm[d] = v;
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, red);
  const bool is_q = unit < p.G;
  const float inv = (is_q ? p.q_scale : 1.0f) / sqrtf(ss + p.unit_eps);
  float* dst = (is_q ? p.q : p.k) + (size_t)m * GD + (size_t)(is_q ? unit : unit - p.G) * p.D;
  for (int d = threadIdx.x; d < p.D; d += blockDim.x) dst[d] = dp_sm[d] * inv;
}

struct DeltaArgs {
  const float* q; const float* k;    // [M, G D]
  const float* v;                    // [M, H V]
  const float* beta; const float* decay;  // [M, H]
  float* o;                          // [M, H V]
  float* S; size_t slot_stride;      // [H, D, V] per slot
  int H, G, D, V;
};

constexpr int kDeltaRows = 16;  // rows staged together (two such buffers: the next chunk arrives under the current one's walk)

// shared memory of delta_scan_kernel<DR> with G row groups (DR == 0: G = 1 and the state itself lives there)
inline size_t delta_scan_smem(int D, int Vr, int DR, int G) {
  const int DP = DR > 0 ? DR * G : D;
  return ((size_t)(DR > 0 ? 0 : D * Vr) + (size_t)2 * kDeltaRows * (2 * DP + Vr + 2) + (size_t)2 * G * Vr) * 4;
}

// grid (n_seqs, H, column splits), block (Vr, G) with Vr a multiple of 32 columns per CTA (the columns of the state are
// independent of one another, so a head may be spread over several CTAs): thread (j, gi) owns rows [gi DR, (gi + 1) DR)
// of one column of the head's D x V state, in registers.  The rows' k, q, v, beta and decay arrive by cp.async, sixteen
// rows at a time, under the walk of the previous sixteen; k and q are read from shared memory four rows at a time.
// Both contractions over D (S^T k and S^T q) are thread-local sums over the thread's rows; with G > 1 the row groups'
// partial sums meet in shared memory and are added in group order (two CTA barriers per row, none with G == 1).
// Padded rows meet k = q = 0.  DR == 0: any D, one group, the column lives in shared memory.  Everything is fp32
// whatever the model's storage type.
template <int DR>
__global__ void delta_scan_kernel(const DeltaArgs p, const Ragged rg) {
  extern __shared__ __align__(16) float ds_sm[];
  const int s = blockIdx.x, hd = blockIdx.y, g = hd / (p.H / p.G);
  const int jl = threadIdx.x, gi = threadIdx.y, Vr = blockDim.x, NG = blockDim.y, tid = gi * Vr + jl, nthr = Vr * NG;
  const int j = blockIdx.z * Vr + jl;  // column of the head's state
  const int D = p.D, V = p.V, DP = DR > 0 ? DR * NG : D;
  float* Ssm = ds_sm;                                     // [D][Vr] (DR == 0)
  constexpr int kR = kDeltaRows;
  const int stage = kR * (2 * DP + Vr + 2);               // floats of one staging buffer
  float* st0 = ds_sm + (DR > 0 ? 0 : (size_t)D * Vr);     // two buffers: [rows][2 DP] k then q | [rows][Vr] v | [rows][2] beta, decay
  float* part = st0 + 2 * stage;                          // [2][NG][Vr] partial contractions
  float Sr[DR > 0 ? DR : 1];
  const bool col = j < V, carried = rg.pos0[s] > 0;
  const int d0 = gi * DR;
  float* Sg = p.S + (size_t)rg.slot[s] * p.slot_stride + (size_t)hd * D * V + (col ? j : 0);
  if (DR > 0) {
#pragma unroll
    for (int d = 0; d < DR; ++d) Sr[d] = (col && carried && d0 + d < D) ? Sg[(size_t)(d0 + d) * V] : 0.f;
  } else {
    for (int d = 0; d < D; ++d) Ssm[(size_t)d * Vr + jl] = (col && carried) ? Sg[(size_t)d * V] : 0.f;
  }
  // padding (rows of k and q from D up to DP, value columns beyond V) is zero in both buffers and never written again
  for (int i = tid; i < 2 * stage; i += nthr) st0[i] = 0.f;
  __syncthreads();
  const int r0 = rg.cu[s], r1 = rg.cu[s + 1], GD = p.G * D, HV = p.H * V;
  const int vcols = max(0, min(Vr, V - (int)blockIdx.z * Vr));
  auto issue = [&](int m0, float* buf) {  // 4-byte asynchronous copies: no alignment rule beyond the element's own
    const int nr = min(kR, r1 - m0);
    float* kq = buf;
    float* vs = kq + kR * 2 * DP;
    float* bg = vs + kR * Vr;
    for (int i = tid; i < nr * D; i += nthr) {
      const int r = i / D, d = i - r * D;
      cp_async4(kq + r * 2 * DP + d, p.k + (size_t)(m0 + r) * GD + g * D + d);
      cp_async4(kq + r * 2 * DP + DP + d, p.q + (size_t)(m0 + r) * GD + g * D + d);
    }
    for (int i = tid; i < nr * vcols; i += nthr) {
      const int r = i / vcols, c = i - r * vcols;
      cp_async4(vs + r * Vr + c, p.v + (size_t)(m0 + r) * HV + hd * V + blockIdx.z * Vr + c);
    }
    if (tid < nr) {
      cp_async4(bg + 2 * tid, p.beta + (size_t)(m0 + tid) * p.H + hd);
      cp_async4(bg + 2 * tid + 1, p.decay + (size_t)(m0 + tid) * p.H + hd);
    }
    cp_async_commit();
  };
  issue(r0, st0);
  int cur = 0;
  for (int m0 = r0; m0 < r1; m0 += kR, cur ^= 1) {
    const int nr = min(kR, r1 - m0);
    if (m0 + kR < r1) {
      issue(m0 + kR, st0 + (cur ^ 1) * stage);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const float* kq = st0 + cur * stage;
    const float* vs = kq + kR * 2 * DP;
    const float* bg = vs + kR * Vr;
    for (int r = 0; r < nr; ++r) {
      const float* kr = kq + r * 2 * DP + d0;
      const float* qr = kr + DP;
      const float beta = bg[2 * r], dec = bg[2 * r + 1];
      float o = 0.f;
      if (DR > 0) {
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
        for (int d = 0; d < DR; d += 4) {
          const float4 k4 = *reinterpret_cast<const float4*>(kr + d);
          Sr[d] *= dec; Sr[d + 1] *= dec; Sr[d + 2] *= dec; Sr[d + 3] *= dec;
          a0 = fmaf(Sr[d], k4.x, a0); a1 = fmaf(Sr[d + 1], k4.y, a1);
          a2 = fmaf(Sr[d + 2], k4.z, a2); a3 = fmaf(Sr[d + 3], k4.w, a3);
        }
        float dot = (a0 + a1) + (a2 + a3);
        if (NG > 1) {
          part[gi * Vr + jl] = dot;
          __syncthreads();
          dot = part[jl];
          for (int w = 1; w < NG; ++w) dot += part[w * Vr + jl];
        }
        const float u = beta * (vs[r * Vr + jl] - dot);
        a0 = a1 = a2 = a3 = 0.f;
#pragma unroll
        for (int d = 0; d < DR; d += 4) {
          const float4 k4 = *reinterpret_cast<const float4*>(kr + d);
          const float4 q4 = *reinterpret_cast<const float4*>(qr + d);
          Sr[d] = fmaf(k4.x, u, Sr[d]); Sr[d + 1] = fmaf(k4.y, u, Sr[d + 1]);
          Sr[d + 2] = fmaf(k4.z, u, Sr[d + 2]); Sr[d + 3] = fmaf(k4.w, u, Sr[d + 3]);
          a0 = fmaf(Sr[d], q4.x, a0); a1 = fmaf(Sr[d + 1], q4.y, a1);
          a2 = fmaf(Sr[d + 2], q4.z, a2); a3 = fmaf(Sr[d + 3], q4.w, a3);
        }
        o = (a0 + a1) + (a2 + a3);
        if (NG > 1) {
          part[(NG + gi) * Vr + jl] = o;
          __syncthreads();
          if (gi == 0) {
            o = part[NG * Vr + jl];
            for (int w = 1; w < NG; ++w) o += part[(NG + w) * Vr + jl];
          }
        }
      } else {
        float dot = 0.f;
        for (int d = 0; d < D; ++d) {
          const float sv = Ssm[(size_t)d * Vr + jl] * dec;
          Ssm[(size_t)d * Vr + jl] = sv;
          dot = fmaf(sv, kr[d], dot);
        }
        const float u = beta * (vs[r * Vr + jl] - dot);
        for (int d = 0; d < D; ++d) {
          const float sv = fmaf(kr[d], u, Ssm[(size_t)d * Vr + jl]);
          Ssm[(size_t)d * Vr + jl] = sv;
          o = fmaf(sv, qr[d], o);
        }
      }
      if (col && gi == 0) p.o[(size_t)(m0 + r) * HV + hd * V + j] = o;
    }
    __syncthreads();  // every thread is done with this buffer before the chunk after next is copied into it
  }
  if (col) {
    if (DR > 0) {
#pragma unroll
      for (int d = 0; d < DR; ++d)
        if (d0 + d < D) Sg[(size_t)(d0 + d) * V] = Sr[d];
    } else {
      for (int d = 0; d < D; ++d) Sg[(size_t)d * V] = Ssm[(size_t)d * Vr + jl];
    }
  }
}

}  // namespace ssdk
