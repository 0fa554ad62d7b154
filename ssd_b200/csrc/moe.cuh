// moe.cuh — routing of a group-limited mixture of experts.
//
//   group_topk_router_kernel  one warp per token, all fp32.  scores = sigmoid(logits) or softmax(logits) over all E
//       router outputs, or the logits themselves with a softmax over the chosen ones as weights.  The CHOICE is made on choice scores = scores (+ a per-output selection bias): the outputs form
//       `groups` equal, contiguous groups; a group scores the sum of its `group_best` (1 or 2) best choice scores; only
//       outputs of the `keep` best groups compete (the others are shut out whatever their sign); the `top` best of
//       those are chosen.  The WEIGHTS are the chosen outputs' plain scores (without the bias), optionally divided by
//       their sum (+ 1e-20), times `route_scale`.  Ties go to the lower index.  Outputs at and beyond the number of
//       real experts are identity experts: they are routed like any other and resolved by the combine kernel.
//   expert_plan_kernel        one CTA: counting sort of the (token, k) assignments by router output -> for every
//       assignment its row in expert order (apos) and the token each sorted row reads (arow), plus the list of row tiles
//       (expert, first row, rows) that the grouped linear kernel walks — tiles are made for the first E_real outputs
//       only; *n_rows = rows that belong to real experts (they come first).  The order of rows inside one expert is
//       arbitrary; every row is computed independently, so results do not depend on it.
// The expert matrices themselves run through the grouped mode of the tcgen05 GEMM (bf16, many rows, whole k-blocks: rows first
// made contiguous per expert by gather_rows_kernel) or of linear_kernel / linear_mma_kernel (linear.cuh), and a GLU kernel.
#pragma once
#include "layer_ops.cuh"

namespace ssdk {

struct RouterArgs {
  const float* z;   // [M, E] router logits
  const void* bias; // [E] T selection bias or nullptr
  int* sel;         // [M, top]
  float* wts;       // [M, top]
  int M, E, top, groups, keep;
  int softmax;      // 0: sigmoid scores, 1: softmax over the E outputs, 2: the raw logits choose and the weights are the
                    //    softmax over the CHOSEN logits only (renorm is then implied)
  int group_best;   // 1 or 2
  int renorm;
  float route_scale;
};
constexpr int kRouterMaxE = 512;
constexpr int kRouterWarps = 4;

template <typename T>
__global__ void __launch_bounds__(kRouterWarps * 32) group_topk_router_kernel(const RouterArgs p) {
  __shared__ float s_score[kRouterWarps][kRouterMaxE];    // plain scores
  __shared__ float s_choice[kRouterWarps][kRouterMaxE];   // choice scores; -inf once taken or shut out
  __shared__ float s_group[kRouterWarps][kRouterMaxE];
  __shared__ unsigned char s_kept[kRouterWarps][kRouterMaxE];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m = blockIdx.x * kRouterWarps + warp;
  if (m >= p.M) return;
  float* sc = s_score[warp];
  float* ch = s_choice[warp];
  float* gs = s_group[warp];
  unsigned char* kept = s_kept[warp];
  const int E = p.E, G = p.groups, per = E / G;
  const float* z = p.z + (size_t)m * E;
  if (p.softmax == 2) {
    for (int e = lane; e < E; e += 32) sc[e] = z[e];
  } else if (p.softmax) {
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[e]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) { const float v = expf(z[e] - mx); sc[e] = v; sum += v; }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
    for (int e = lane; e < E; e += 32) sc[e] *= inv;
  } else {
    for (int e = lane; e < E; e += 32) sc[e] = sigmoid_f(z[e]);
  }
  for (int e = lane; e < E; e += 32) ch[e] = sc[e] + (p.bias ? ld_f<T>((const T*)p.bias + e) : 0.f);
  __syncwarp();
  for (int g = lane; g < G; g += 32) {
    float b1 = -INFINITY, b2 = -INFINITY;
    for (int e = g * per; e < (g + 1) * per; ++e) {
      const float v = ch[e];
      if (v > b1) { b2 = b1; b1 = v; } else if (v > b2) { b2 = v; }
    }
    gs[g] = (p.group_best >= 2 && per >= 2) ? b1 + b2 : b1;
    kept[g] = 0;
  }
  __syncwarp();
  // keep the `keep` best groups, then shut out the outputs of all others
  for (int r = 0; r < p.keep; ++r) {
    ArgMax a{-INFINITY, 0x7fffffff};
    for (int g = lane; g < G; g += 32)
      if (!kept[g]) a = argmax_better(a, ArgMax{gs[g], g});
    a = warp_argmax(a);
    __syncwarp();
    if (lane == 0 && a.i < G) kept[a.i] = 1;
    __syncwarp();
  }
  for (int e = lane; e < E; e += 32)
    if (!kept[e / per]) ch[e] = -INFINITY;
  __syncwarp();
  float mine = 0.f, total = 0.f, first = 0.f;   // lane r keeps the r-th chosen score (top <= 32)
  int mine_i = 0;
  for (int r = 0; r < p.top; ++r) {
    ArgMax a{-INFINITY, 0x7fffffff};
    for (int e = lane; e < E; e += 32) a = argmax_better(a, ArgMax{ch[e], e});
    a = warp_argmax(a);
    if (a.i >= E) a.i = 0;   // (cannot happen with finite logits: top fits the kept groups)
    __syncwarp();
    if (lane == 0) ch[a.i] = -INFINITY;
    __syncwarp();
    float w = sc[a.i];
    if (p.softmax == 2) {   // the first chosen logit is the largest: exponentials relative to it
      if (r == 0) first = w;
      w = expf(w - first);
    }
    if (lane == r) { mine = w; mine_i = a.i; }
    total += w;
  }
  if (lane < p.top) {
    p.sel[(size_t)m * p.top + lane] = mine_i;
    p.wts[(size_t)m * p.top + lane] = ((p.renorm || p.softmax == 2) ? mine / (total + 1e-20f) : mine) * p.route_scale;
  }
}

struct PlanArgs {
  const int* sel;    // [A] expert of assignment a = token * top + k
  int* apos;         // [A] row of assignment a in expert order
  int* arow;         // [A] token of sorted row
  int* tile_expert; int* tile_row0; int* tile_rows; int* n_tiles;
  int* n_rows;       // rows of real experts (device copy for kernels that bound their work by it)
  int A, E, top, tile;
  int E_real;        // outputs >= E_real are identity experts: sorted behind the real ones, no tiles
};

__global__ void __launch_bounds__(1024) expert_plan_kernel(const PlanArgs p) {
  __shared__ int s_cnt[kRouterMaxE];
  __shared__ int s_off[kRouterMaxE + 1];
  for (int e = threadIdx.x; e < p.E; e += blockDim.x) s_cnt[e] = 0;
  __syncthreads();
  for (int a = threadIdx.x; a < p.A; a += blockDim.x) atomicAdd(&s_cnt[p.sel[a]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int off = 0, nt = 0;
    for (int e = 0; e < p.E; ++e) {
      s_off[e] = off;
      if (e == p.E_real) *p.n_rows = off;
      for (int r0 = 0; e < p.E_real && r0 < s_cnt[e]; r0 += p.tile) {
        p.tile_expert[nt] = e;
        p.tile_row0[nt] = off + r0;
        p.tile_rows[nt] = min(p.tile, s_cnt[e] - r0);
        ++nt;
      }
      off += s_cnt[e];
    }
    s_off[p.E] = off;
    *p.n_tiles = nt;
    if (p.E_real >= p.E) *p.n_rows = p.A;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < p.E; e += blockDim.x) s_cnt[e] = 0;
  __syncthreads();
  for (int a = threadIdx.x; a < p.A; a += blockDim.x) {
    const int e = p.sel[a];
    const int row = s_off[e] + atomicAdd(&s_cnt[e], 1);
    p.apos[a] = row;
    p.arow[row] = a / p.top;
  }
}

// dst[r, :] = src[rows[r], :] for r < *n_rows: the routed rows made contiguous per expert (operand of the grouped tcgen05 GEMM,
// whose TMA boxes cannot follow an index list)
template <typename T>
__global__ void gather_rows_kernel(const T* __restrict__ src, const int* __restrict__ rows, const int* __restrict__ n_rows,
                                   T* __restrict__ dst, int width) {
  const int r = blockIdx.x;
  if (r >= *n_rows) return;
  const T* s = src + (size_t)rows[r] * width;
  T* d = dst + (size_t)r * width;
  if (sizeof(T) == 2 && width % 8 == 0 && (((uintptr_t)src | (uintptr_t)dst) & 15) == 0) {
    for (int c = threadIdx.x; c < width / 8; c += blockDim.x) ((uint4*)d)[c] = ((const uint4*)s)[c];
  } else {
    for (int c = threadIdx.x; c < width; c += blockDim.x) d[c] = s[c];
  }
}

}  // namespace ssdk
