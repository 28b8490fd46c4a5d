// Inputs that depend on the token itself or on its place in the sequence, in bfloat16 or true float32 (sums in fp32):
//
//  * embed_pos_kernel  — token embedding plus a learned position row: x = E[token] + P[position], into the fp32 stream.
//  * side_gate_kernel  — the gate of a per-layer token input: g = gelu_tanh(t) * Es[token, col0 .. col0 + n), t the fp32
//    product of a small projection with the stream, Es a second embedding table whose row holds one slice per layer.
//  * side_gate_rows_kernel — the same gate for a few rows (decoding) with the small projection inside: a CTA per four gate
//    channels streams their rows of the projection against the fp32 stream rows of all tokens (the stream is not rounded first).
//  * branch_add_cast_kernel — the residual step of a block (both branches added to the fp32 stream) with a copy of the updated
//    stream in the operand type, which the token input's first GEMM reads.
//
// Token (b, s) of a call sits at slot *cache_len + s and position slot - pad_left[b]; negative positions are padding.
#include <stdint.h>

#include "jllama_b200.h"
#include "seq_types.cuh"

namespace jl {

template <typename T>
__global__ void __launch_bounds__(128) embed_pos_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                                                        const T* __restrict__ pos_table, float* __restrict__ out,
                                                        const int* __restrict__ cache_len, const int* __restrict__ pad_left, int S,
                                                        int W, int V, int P) {
  pdl_wait();                      // programmatic dependent launch: nothing is read before the predecessor is done
  pdl_launch_dependents();
  const int m = blockIdx.x, b = m / S, s = m % S;
  int pos = (cache_len ? *cache_len : 0) + s - (pad_left ? pad_left[b] : 0);
  float* orow = out + (size_t)m * W;
  if (pos < 0) {                                         // padding: a zero row (nothing reads what the layers make of it)
    for (int i = threadIdx.x; i < W; i += blockDim.x) orow[i] = 0.0f;
    return;
  }
  pos = pos >= P ? P - 1 : pos;
  int tok = ids[m];
  tok = tok < 0 ? 0 : (tok >= V ? V - 1 : tok);
  const T* e = table + (size_t)tok * W;
  const T* pr = pos_table + (size_t)pos * W;
  for (int i = threadIdx.x; i < W; i += blockDim.x) orow[i] = to_f(e[i]) + to_f(pr[i]);
}

template <typename T>
__global__ void __launch_bounds__(256) side_gate_kernel(const float* __restrict__ t, int ldt, const int* __restrict__ ids,
                                                        const T* __restrict__ side, int lds, int col0, T* __restrict__ out, int ldo,
                                                        int M, int n, int V) {
  pdl_wait();                      // programmatic dependent launch: nothing is read before the predecessor is done
  pdl_launch_dependents();
  const size_t total = (size_t)M * n;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int m = (int)(i / n), c = (int)(i % n);
    int tok = ids[m];
    tok = tok < 0 ? 0 : (tok >= V ? V - 1 : tok);
    out[(size_t)m * ldo + c] = from_f<T>(apply_act(t[(size_t)m * ldt + c], ACT_GELU_TANH, 0.0f, 0.0f) *
                                         to_f(side[(size_t)tok * lds + col0 + c]));
  }
}

constexpr int SG_WARPS = 8, SG_CH = 4, SG_MAXM = 8;

// A few rows (decoding): a CTA owns SG_CH gate channels, its warps split the width; a lane reads four elements of every channel's
// row of the gate projection per step (all loads of a step issued before the first use) against the fp32 stream rows of all M
// tokens, which are read as they are (no rounding to the operand type).  The warps' sums meet in shared memory in a fixed
// order; then gelu_tanh and the token's table entry.
template <typename T, int M>
__global__ void __launch_bounds__(SG_WARPS * 32) side_gate_rows_kernel(const float* __restrict__ x, int ldx, const int* __restrict__ ids,
                                                                       const T* __restrict__ side, int lds, int col0,
                                                                       const T* __restrict__ wg, T* __restrict__ out, int ldo,
                                                                       int W, int n, int V, int vec_ok) {
  pdl_wait();                      // programmatic dependent launch: nothing is read before the predecessor is done
  pdl_launch_dependents();
  __shared__ float red[SG_WARPS][SG_CH][M];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c0 = blockIdx.x * SG_CH;
  float acc[SG_CH][M];
#pragma unroll
  for (int r = 0; r < SG_CH; ++r)
#pragma unroll
    for (int m = 0; m < M; ++m) acc[r][m] = 0.0f;
  int done = 0;
  if (vec_ok) {
    const int kv = W / 4 * 4;
    for (int k = (warp * 32 + lane) * 4; k < kv; k += SG_WARPS * 128) {
      float wv[SG_CH][4];
#pragma unroll
      for (int r = 0; r < SG_CH; ++r) load4(wg + (size_t)min(c0 + r, n - 1) * W + k, wv[r]);
#pragma unroll
      for (int m = 0; m < M; ++m) {
        float xv[4];
        load4(x + (size_t)m * ldx + k, xv);
#pragma unroll
        for (int r = 0; r < SG_CH; ++r)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[r][m] = fmaf(wv[r][j], xv[j], acc[r][m]);
      }
    }
    done = kv;
  }
  for (int k = done + warp * 32 + lane; k < W; k += SG_WARPS * 32) {
#pragma unroll
    for (int r = 0; r < SG_CH; ++r) {
      const float wv = to_f(wg[(size_t)min(c0 + r, n - 1) * W + k]);
#pragma unroll
      for (int m = 0; m < M; ++m) acc[r][m] = fmaf(wv, x[(size_t)m * ldx + k], acc[r][m]);
    }
  }
#pragma unroll
  for (int r = 0; r < SG_CH; ++r)
#pragma unroll
    for (int m = 0; m < M; ++m) {
      const float d = warp_sum(acc[r][m]);
      if (lane == 0) red[warp][r][m] = d;
    }
  __syncthreads();
  if (threadIdx.x < SG_CH * M) {
    const int r = threadIdx.x / M, m = threadIdx.x % M, c = c0 + r;
    float d = 0.0f;
#pragma unroll
    for (int w = 0; w < SG_WARPS; ++w) d += red[w][r][m];
    if (c < n) {
      int tok = ids[m];
      tok = tok < 0 ? 0 : (tok >= V ? V - 1 : tok);
      out[(size_t)m * ldo + c] = from_f<T>(apply_act(d, ACT_GELU_TANH, 0.0f, 0.0f) * to_f(side[(size_t)tok * lds + col0 + c]));
    }
  }
}

// x[m, :] += mult * (y1[m, :] + y2[m, :]) in place (fp32; either branch may be absent) and a copy of the updated row in the
// operand type: the residual step of a block whose token input reads the stream itself through a GEMM.
template <typename T>
__global__ void __launch_bounds__(256) branch_add_cast_kernel(const float* __restrict__ y1, int ld1, const float* __restrict__ y2,
                                                              int ld2, float mult, float* __restrict__ x, T* __restrict__ xc, int W,
                                                              int vec) {
  pdl_wait();                      // programmatic dependent launch: nothing is read before the predecessor is done
  pdl_launch_dependents();
  const size_t m = blockIdx.x;
  float* xr = x + m * W;
  const float* a = y1 ? y1 + m * ld1 : nullptr;
  const float* b = y2 ? y2 + m * ld2 : nullptr;
  if (vec) {
    for (int i = threadIdx.x * 4; i < W; i += blockDim.x * 4) {
      float v[4], s[4] = {0.f, 0.f, 0.f, 0.f}, t[4];
      load4(xr + i, v);
      if (a) load4(a + i, s);
      if (b) { load4(b + i, t);
#pragma unroll
        for (int j = 0; j < 4; ++j) s[j] += t[j]; }
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = fmaf(mult, s[j], v[j]);
      store4(xr + i, v);
      store4(xc + m * W + i, v);
    }
    return;
  }
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float v = fmaf(mult, (a ? a[i] : 0.0f) + (b ? b[i] : 0.0f), xr[i]);
    xr[i] = v;
    xc[m * W + i] = from_f<T>(v);
  }
}

}  // namespace jl

using namespace jl;

extern "C" JL_API int jl_embed_pos(const int* ids, const void* table, const void* pos_table, float* out, const int* cache_len,
                                   const int* pad_left, int B, int S, int W, int V, int P, int dtype, void* stream) {
  JL_CHECK_ARG(B >= 1 && S >= 1 && W >= 1 && V >= 1 && P >= 1, "jl_embed_pos: bad shape B=%d S=%d W=%d V=%d P=%d", B, S, W, V, P);
  JL_DISPATCH_DTYPE(dtype, JL_LAUNCH_PDL(embed_pos_kernel<T>, dim3(B * S), dim3(128), 0, (cudaStream_t)stream, ids, (const T*)table,
                                         (const T*)pos_table, out, cache_len, pad_left, S, W, V, P));
  JL_CUDA(cudaGetLastError());
  return JL_OK;
}

extern "C" JL_API int jl_side_gate(const float* t, int ldt, const int* ids, const void* side, int lds, int col0, void* out, int ldo,
                                   int M, int n, int V, int dtype, void* stream) {
  JL_CHECK_ARG(M >= 1 && n >= 1 && V >= 1 && ldt >= n && ldo >= n && col0 >= 0 && lds >= col0 + n,
               "jl_side_gate: bad shape M=%d n=%d ldt=%d ldo=%d col0=%d lds=%d", M, n, ldt, ldo, col0, lds);
  const size_t total = (size_t)M * n;
  const int blocks = (int)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
  JL_DISPATCH_DTYPE(dtype, JL_LAUNCH_PDL(side_gate_kernel<T>, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, t, ldt, ids,
                                         (const T*)side, lds, col0, (T*)out, ldo, M, n, V));
  JL_CUDA(cudaGetLastError());
  return JL_OK;
}

extern "C" JL_API int jl_side_gate_rows(const float* x, int ldx, const int* ids, const void* side, int lds, int col0, const void* w_gate,
                                        void* out, int ldo, int M, int W, int n, int V, int dtype, void* stream) {
  JL_CHECK_ARG(M >= 1 && M <= SG_MAXM && W >= 1 && n >= 1 && V >= 1 && ldx >= W && ldo >= n && col0 >= 0 && lds >= col0 + n,
               "jl_side_gate_rows: bad shape M=%d W=%d n=%d ldx=%d ldo=%d", M, W, n, ldx, ldo);
  const int vec_ok = W % 4 == 0 && ldx % 4 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)w_gate % 16 == 0;
  const dim3 grid((n + SG_CH - 1) / SG_CH);
#define JL_SG(MM)                                                                                                            \
  case MM:                                                                                                                   \
    JL_DISPATCH_DTYPE(dtype, JL_LAUNCH_PDL((side_gate_rows_kernel<T, MM>), dim3(grid), dim3(SG_WARPS * 32), 0, (cudaStream_t)stream, x, ldx, \
                                           ids, (const T*)side, lds, col0, (const T*)w_gate, (T*)out, ldo, W, n, V, vec_ok));   \
    break;
  switch (M) { JL_SG(1) JL_SG(2) JL_SG(3) JL_SG(4) JL_SG(5) JL_SG(6) JL_SG(7) JL_SG(8) }
#undef JL_SG
  JL_CUDA(cudaGetLastError());
  return JL_OK;
}

extern "C" JL_API int jl_branch_add_cast(const float* y1, int ld1, const float* y2, int ld2, float mult, float* x, void* xc, int M, int W,
                                         int dtype, void* stream) {
  JL_CHECK_ARG(M >= 1 && W >= 1 && xc != nullptr, "jl_branch_add_cast: bad shape M=%d W=%d", M, W);
  JL_CHECK_ARG((y1 == nullptr || ld1 >= W) && (y2 == nullptr || ld2 >= W), "jl_branch_add_cast: row pitch below W=%d", W);
  const int vec = W % 4 == 0 && (y1 == nullptr || ld1 % 4 == 0) && (y2 == nullptr || ld2 % 4 == 0) && (uintptr_t)y1 % 16 == 0 &&
                  (uintptr_t)y2 % 16 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)xc % 16 == 0;
  JL_DISPATCH_DTYPE(dtype, JL_LAUNCH_PDL(branch_add_cast_kernel<T>, dim3(M), dim3(256), 0, (cudaStream_t)stream, y1, ld1, y2, ld2, mult, x,
                                         (T*)xc, W, vec));
  JL_CUDA(cudaGetLastError());
  return JL_OK;
}
