// Inputs that depend on the token itself or on its place in the sequence, in bfloat16 or true float32 (sums in fp32):
//
//  * embed_pos_kernel  — token embedding plus a learned position row: x = E[token] + P[position], into the fp32 stream.
//  * side_gate_kernel  — the gate of a per-layer token input: g = gelu_tanh(t) * Es[token, col0 .. col0 + n), t the fp32
//    product of a small projection with the stream, Es a second embedding table whose row holds one slice per layer.
//  * side_gate_rows_kernel — the same gate for a few rows (decoding) with the small projection inside: a warp per gate channel
//    streams its row of the projection against the fp32 stream rows of all tokens (the stream is not rounded first).
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

constexpr int SG_WARPS = 4, SG_MAXM = 8;

// A few rows (decoding): a warp per gate channel c streams row c of the gate projection once (16-byte loads) against the fp32
// stream rows of all M tokens, then applies gelu_tanh and the token's table entry.  The stream is read as it is (no rounding
// to the operand type); n / SG_WARPS CTAs share the weight matrix between them.
template <typename T, int M>
__global__ void __launch_bounds__(SG_WARPS * 32) side_gate_rows_kernel(const float* __restrict__ x, int ldx, const int* __restrict__ ids,
                                                                       const T* __restrict__ side, int lds, int col0,
                                                                       const T* __restrict__ wg, T* __restrict__ out, int ldo,
                                                                       int W, int n, int V, int vec_ok) {
  pdl_wait();                      // programmatic dependent launch: nothing is read before the predecessor is done
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c = blockIdx.x * SG_WARPS + warp;
  if (c >= n) return;
  const T* wr = wg + (size_t)c * W;
  float acc[M];
#pragma unroll
  for (int m = 0; m < M; ++m) acc[m] = 0.0f;
  int done = 0;
  if (vec_ok) {
    const int kv = W / 4 * 4;
    for (int k = lane * 4; k < kv; k += 128) {
      float wv[4];
      load4(wr + k, wv);
#pragma unroll
      for (int m = 0; m < M; ++m) {
        float xv[4];
        load4(x + (size_t)m * ldx + k, xv);
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[m] = fmaf(wv[j], xv[j], acc[m]);
      }
    }
    done = kv;
  }
  for (int k = done + lane; k < W; k += 32) {
    const float wv = to_f(wr[k]);
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = fmaf(wv, x[(size_t)m * ldx + k], acc[m]);
  }
#pragma unroll
  for (int m = 0; m < M; ++m) {
    const float d = warp_sum(acc[m]);
    if (lane == 0) {
      int tok = ids[m];
      tok = tok < 0 ? 0 : (tok >= V ? V - 1 : tok);
      out[(size_t)m * ldo + c] = from_f<T>(apply_act(d, ACT_GELU_TANH, 0.0f, 0.0f) * to_f(side[(size_t)tok * lds + col0 + c]));
    }
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
  const dim3 grid((n + SG_WARPS - 1) / SG_WARPS);
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
