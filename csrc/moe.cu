// Mixture-of-experts routing for the hybrid decoder family: choosing experts per token, ordering the (token, choice) pairs
// by expert for the grouped linear kernels (seq_linear.cu), and the weighted sum of the experts' outputs.
//
//   route    one warp per token: scores (sigmoid or softmax of the fp32 router logits), choice scores (scores plus an optional
//            per-expert bias that only the choice sees), optional restriction to the best groups of neighbouring experts, the
//            `top` largest choice scores of what is left, weights = chosen scores over their sum (when normalised) times a
//            constant.  The last E - n_real router outputs can be identity experts (no matrices: their output is the input):
//            a chosen one is reported as expert -1 and its weight is summed per token.  Everything in fp32.
//   sort     one CTA: counts per expert, segments rounded up to whole row tiles, the sorted position of every pair, the
//            source token of every sorted row and the expert of every tile.
//   combine  y[m, :] = sum_k weight[m, k] * z[pos[m, k], :]  (+ sigmoid(gate logit[m]) * shared[m, :]).
#include <stdint.h>

#include "jllama_b200.h"
#include "seq_types.cuh"

namespace jl {

enum { SCORE_SIGMOID = 0, SCORE_SOFTMAX = 1 };

struct RouteParams {
  const float* z; int ldz;          // router logits: columns 0 .. E-1 of row m
  int M, E, top;
  int groups, keep, group_top;      // groups <= 1: every expert can be chosen; group score = sum of its group_top largest
  int score, normalise;
  float scale;
  int* idx; float* wt;              // [M][top]
  const float* bias;                // [E] fp32 added to the logits, or nullptr
  const float* choice_bias;         // [E] fp32 added to the scores for the choice (groups and top) only, or nullptr
  int n_real;                       // experts 0 .. n_real-1 have matrices; n_real .. E-1 are identity experts
  float* ident_w;                   // [M]: sum of the weights of the identity experts a token chose (n_real < E)
};

constexpr int RT_WARPS = 4;

__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
  }
}

__global__ void __launch_bounds__(RT_WARPS * 32) moe_route_kernel(RouteParams p) {
  pdl_wait();                      // programmatic dependent launch: nothing is read before the predecessor is done
  pdl_launch_dependents();
  extern __shared__ float sm[];                                  // per warp: scores [E], work copy [E], group scores [groups]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m = blockIdx.x * RT_WARPS + warp;
  if (m >= p.M) return;
  const int ng = p.groups > 1 ? p.groups : 0;
  float* s = sm + (size_t)warp * (2 * p.E + ng);
  float* work = s + p.E;
  float* gs = work + p.E;
  const float* zr = p.z + (size_t)m * p.ldz;
  auto logit = [&](int e) { return p.bias ? zr[e] + p.bias[e] : zr[e]; };
  if (p.score == SCORE_SOFTMAX) {
    float mx = -INFINITY;
    for (int e = lane; e < p.E; e += 32) mx = fmaxf(mx, logit(e));
    mx = warp_max(mx);
    float sum = 0.0f;
    for (int e = lane; e < p.E; e += 32) { const float v = expf(logit(e) - mx); s[e] = v; sum += v; }
    sum = warp_sum(sum);
    for (int e = lane; e < p.E; e += 32) s[e] = s[e] / sum;
  } else {
    for (int e = lane; e < p.E; e += 32) s[e] = sigmoid_f(logit(e));
  }
  __syncwarp();
  for (int e = lane; e < p.E; e += 32) work[e] = p.choice_bias ? s[e] + p.choice_bias[e] : s[e];
  __syncwarp();
  if (ng) {
    const int per = p.E / ng;
    for (int g = lane; g < ng; g += 32) {                        // sum of the group's group_top largest scores
      float acc = 0.0f;
      float last = INFINITY; int last_i = -1;
      for (int t = 0; t < p.group_top && t < per; ++t) {         // t-th largest: the largest that comes after (last, last_i)
        float best = -INFINITY; int bi = -1;
        for (int j = 0; j < per; ++j) {
          const float v = work[g * per + j];
          const bool after = v < last || (v == last && j > last_i);
          if (after && (v > best || bi < 0)) { best = v; bi = j; }
        }
        if (bi < 0) break;
        acc += best; last = best; last_i = bi;
      }
      gs[g] = acc;
    }
    __syncwarp();
    for (int t = 0; t < p.keep; ++t) {                           // mark the keep best groups with -inf
      float v = -INFINITY; int gi = 0x7fffffff;
      for (int g = lane; g < ng; g += 32)
        if (gs[g] > v && gs[g] != -INFINITY) { v = gs[g]; gi = g; }
      warp_argmax(v, gi);
      __syncwarp();
      if (lane == 0 && gi != 0x7fffffff) gs[gi] = -INFINITY;
      __syncwarp();
    }
    for (int e = lane; e < p.E; e += 32)
      if (gs[e / per] != -INFINITY) work[e] = -INFINITY;           // experts outside the kept groups cannot be chosen
  }
  __syncwarp();
  float sum = 0.0f, mine = 0.0f, ident = 0.0f; int mine_i = 0;
  for (int t = 0; t < p.top; ++t) {
    float v = -INFINITY; int ei = 0x7fffffff;
    for (int e = lane; e < p.E; e += 32)
      if (work[e] > v) { v = work[e]; ei = e; }
    warp_argmax(v, ei);
    if (ei == 0x7fffffff) ei = 0;
    const float sc = s[ei];
    sum += sc;
    const int eo = ei < p.n_real ? ei : -1;                      // an identity expert has no matrices to run
    if (eo < 0) ident += sc;
    if (lane == t % 32 && t < 32) { mine = sc; mine_i = eo; }
    if (t >= 32 && lane == 0) { p.idx[(size_t)m * p.top + t] = eo; p.wt[(size_t)m * p.top + t] = sc; }    // weights scaled below
    __syncwarp();
    if (lane == 0) work[ei] = -INFINITY;
    __syncwarp();
  }
  const float mul = (p.normalise ? 1.0f / (sum + 1e-20f) : 1.0f) * p.scale;
  if (lane < p.top) { p.idx[(size_t)m * p.top + lane] = mine_i; p.wt[(size_t)m * p.top + lane] = mine * mul; }
  if (p.top > 32 && lane == 0)
    for (int t = 32; t < p.top; ++t) p.wt[(size_t)m * p.top + t] *= mul;
  if (p.ident_w && lane == 0) p.ident_w[m] = ident * mul;
}

// One CTA orders the n = M * top pairs by expert.  counts / offsets live in shared memory (E + 1 ints each).
__global__ void __launch_bounds__(1024) moe_sort_kernel(const int* __restrict__ idx, int n, int top, int E, int tile, int cap,
                                                        int* __restrict__ pos, int* __restrict__ row_src,
                                                        int* __restrict__ tile_group, int* __restrict__ tiles_used) {
  pdl_wait();                      // programmatic dependent launch: nothing is read before the predecessor is done
  pdl_launch_dependents();
  extern __shared__ int si[];
  int* count = si;                 // [E]
  int* start = si + E;             // [E + 1], in rows
  for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
  for (int i = threadIdx.x; i < cap; i += blockDim.x) row_src[i] = -1;
  for (int i = threadIdx.x; i < cap / tile; i += blockDim.x) tile_group[i] = -1;
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x)               // rank within its expert (expert < 0: a pair that runs no expert)
    pos[i] = idx[i] >= 0 ? atomicAdd(&count[idx[i]], 1) : -1;
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0;
    for (int e = 0; e < E; ++e) { start[e] = at; at += (count[e] + tile - 1) / tile * tile; }
    start[E] = at;
    if (tiles_used) *tiles_used = at / tile;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x)
    for (int t = start[e] / tile; t < start[e + 1] / tile; ++t) tile_group[t] = e;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    if (idx[i] < 0) continue;                                      // pos stays -1: the combine pass skips the pair
    const int at = start[idx[i]] + pos[i];
    pos[i] = at;
    row_src[at] = i / top;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) moe_combine_kernel(const float* __restrict__ z, int ldz, const int* __restrict__ pos,
                                                          const float* __restrict__ wt, int top, const float* __restrict__ shared,
                                                          int lds, const float* __restrict__ gate, int ldg,
                                                          float* __restrict__ out, int W, const int* __restrict__ idx,
                                                          const float* __restrict__ ident_w, const T* __restrict__ x, int ldx) {
  pdl_wait();                      // programmatic dependent launch: nothing is read before the predecessor is done
  pdl_launch_dependents();
  const size_t m = blockIdx.x;
  const float g = shared ? (gate ? sigmoid_f(gate[m * ldg]) : 1.0f) : 0.0f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float acc = 0.0f;
    for (int k = 0; k < top; ++k) {
      if (idx && idx[m * top + k] < 0) continue;                   // an identity expert: its share comes with ident_w below
      const size_t r = pos ? (size_t)pos[m * top + k] : m * top + k;
      acc = fmaf(wt[m * top + k], z[r * ldz + i], acc);
    }
    if (ident_w) acc = fmaf(ident_w[m], to_f(x[m * ldx + i]), acc);
    if (shared) acc = fmaf(g, shared[m * lds + i], acc);
    out[m * W + i] = acc;
  }
}

// xs[p, :] = x[row_src[p], :] (row_src[p] < 0: zeros): the rows of a step in sorted order, for kernels that cannot gather.
template <typename T>
__global__ void __launch_bounds__(128) moe_gather_kernel(const T* __restrict__ x, int ldx, const int* __restrict__ row_src,
                                                         T* __restrict__ xs, int W) {
  pdl_wait();                      // programmatic dependent launch: nothing is read before the predecessor is done
  pdl_launch_dependents();
  const size_t p = blockIdx.x;
  const int src = row_src[p];
  constexpr int VN = 16 / sizeof(T);
  if (W % VN == 0 && ldx % VN == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)xs & 15) == 0) {
    const uint4* in = src >= 0 ? reinterpret_cast<const uint4*>(x + (size_t)src * ldx) : nullptr;
    uint4* out = reinterpret_cast<uint4*>(xs + p * W);
    for (int i = threadIdx.x; i < W / VN; i += blockDim.x) out[i] = in ? in[i] : make_uint4(0, 0, 0, 0);
    return;
  }
  for (int i = threadIdx.x; i < W; i += blockDim.x) xs[p * W + i] = src >= 0 ? x[(size_t)src * ldx + i] : from_f<T>(0.0f);
}

}  // namespace jl

using namespace jl;

static int moe_route_launch(const float* z, int ldz, int M, int E, int top, int groups, int keep, int group_top, int score,
                            int normalise, float scale, const float* bias, const float* choice_bias, int n_real, float* ident_w,
                            int* idx, float* wt, void* stream) {
  JL_CHECK_ARG(M >= 1 && E >= 1 && top >= 1 && top <= E && ldz >= E, "jl_moe_route: bad shape M=%d E=%d top=%d ldz=%d", M, E, top, ldz);
  JL_CHECK_ARG(groups <= 1 || (E % groups == 0 && keep >= 1 && keep <= groups && group_top >= 1 && keep * (E / groups) >= top),
               "jl_moe_route: %d groups of %d experts, keep %d, cannot give %d choices", groups, groups > 0 ? E / groups : 0, keep, top);
  JL_CHECK_ARG(score == SCORE_SIGMOID || score == SCORE_SOFTMAX, "jl_moe_route: score function %d", score);
  JL_CHECK_ARG(n_real >= 1 && n_real <= E && (n_real == E || ident_w != nullptr), "jl_moe_route: %d of %d experts with matrices", n_real, E);
  RouteParams p{z, ldz, M, E, top, groups, keep, group_top, score, normalise, scale, idx, wt, bias, choice_bias, n_real, ident_w};
  const size_t smem = (size_t)RT_WARPS * (2 * E + (groups > 1 ? groups : 0)) * sizeof(float);
  JL_CHECK_ARG(smem <= 200 * 1024, "jl_moe_route: %d experts do not fit shared memory", E);
  if (smem > 48 * 1024) JL_CUDA(cudaFuncSetAttribute(moe_route_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  JL_LAUNCH_PDL(moe_route_kernel, dim3((M + RT_WARPS - 1) / RT_WARPS), dim3(RT_WARPS * 32), smem, stream, p);
  JL_CUDA(cudaGetLastError());
  return JL_OK;
}

extern "C" JL_API int jl_moe_route(const float* z, int ldz, int M, int E, int top, int groups, int keep, int group_top, int score,
                                   int normalise, float scale, const float* bias, int* idx, float* wt, void* stream) {
  return moe_route_launch(z, ldz, M, E, top, groups, keep, group_top, score, normalise, scale, bias, nullptr, E, nullptr, idx, wt, stream);
}

// The same with a choice bias (added to the scores for groups and top only) and identity experts: router outputs n_real .. E-1
// have no matrices; a chosen one is reported as expert -1 and its weight is added to ident_w[m].
extern "C" JL_API int jl_moe_route_ex(const float* z, int ldz, int M, int E, int top, int groups, int keep, int group_top, int score,
                                      int normalise, float scale, const float* bias, const float* choice_bias, int n_real,
                                      float* ident_w, int* idx, float* wt, void* stream) {
  return moe_route_launch(z, ldz, M, E, top, groups, keep, group_top, score, normalise, scale, bias, choice_bias, n_real, ident_w, idx,
                          wt, stream);
}

// Rows of the sorted layout for n pairs over E experts with row tiles of `tile`: every expert's segment is rounded up.
extern "C" JL_API int jl_moe_sorted_rows(int n, int E, int tile) { return (n + E * (tile - 1) + tile - 1) / tile * tile; }

extern "C" JL_API int jl_moe_sort(const int* idx, int M, int top, int E, int tile, int cap, int* pos, int* row_src, int* tile_group,
                                  int* tiles_used, void* stream) {
  JL_CHECK_ARG(M >= 1 && top >= 1 && E >= 1 && tile >= 1, "jl_moe_sort: bad shape");
  JL_CHECK_ARG(cap % tile == 0 && cap >= jl_moe_sorted_rows(M * top, E, tile), "jl_moe_sort: %d rows are too few", cap);
  const size_t smem = (size_t)(2 * E + 1) * sizeof(int);
  JL_CHECK_ARG(smem <= 48 * 1024, "jl_moe_sort: %d experts do not fit shared memory", E);
  JL_LAUNCH_PDL(moe_sort_kernel, dim3(1), dim3(1024), smem, stream, idx, M * top, top, E, tile, cap, pos, row_src, tile_group, tiles_used);
  JL_CUDA(cudaGetLastError());
  return JL_OK;
}

extern "C" JL_API int jl_moe_combine(const float* z, int ldz, const int* pos, const float* wt, int top, const float* shared, int lds,
                                     const float* gate, int ldg, float* out, int M, int W, void* stream) {
  JL_CHECK_ARG(M >= 1 && W >= 1 && top >= 1 && ldz >= W, "jl_moe_combine: bad shape");
  JL_LAUNCH_PDL(moe_combine_kernel<float>, dim3(M), dim3(256), 0, stream, z, ldz, pos, wt, top, shared, lds, gate, ldg, out, W,
                (const int*)nullptr, (const float*)nullptr, (const float*)nullptr, 0);
  JL_CUDA(cudaGetLastError());
  return JL_OK;
}

// The same for a router with identity experts: pairs with idx < 0 ran no expert (their rows of z are not read); ident_w[m] · x[m, :]
// (x in `dtype`, row pitch ldx) is added instead.
extern "C" JL_API int jl_moe_combine_ex(const float* z, int ldz, const int* pos, const float* wt, int top, const float* shared, int lds,
                                        const float* gate, int ldg, float* out, int M, int W, const int* idx, const float* ident_w,
                                        const void* x, int ldx, int dtype, void* stream) {
  JL_CHECK_ARG(M >= 1 && W >= 1 && top >= 1 && ldz >= W, "jl_moe_combine: bad shape");
  JL_CHECK_ARG(ident_w == nullptr || (x != nullptr && ldx >= W), "jl_moe_combine: identity weights without the input rows");
  JL_DISPATCH_DTYPE(dtype, JL_LAUNCH_PDL(moe_combine_kernel<T>, dim3(M), dim3(256), 0, stream, z, ldz, pos, wt, top, shared, lds, gate,
                                         ldg, out, W, idx, ident_w, (const T*)x, ldx));
  JL_CUDA(cudaGetLastError());
  return JL_OK;
}

extern "C" JL_API int jl_moe_gather(const void* x, int ldx, const int* row_src, void* xs, int rows, int W, int dtype, void* stream) {
  JL_CHECK_ARG(rows >= 1 && W >= 1 && ldx >= W, "jl_moe_gather: bad shape");
  JL_DISPATCH_DTYPE(dtype, JL_LAUNCH_PDL(moe_gather_kernel<T>, dim3(rows), dim3(128), 0, stream, (const T*)x, ldx, row_src, (T*)xs, W));
  JL_CUDA(cudaGetLastError());
  return JL_OK;
}
