// Inputs that depend on the token itself or on its place in the sequence, in bfloat16 or true float32 (sums in fp32):
//
//  * embed_pos_kernel  — token embedding plus a learned position row: x = E[token] + P[position], into the fp32 stream.
//  * side_gate_kernel  — the gate of a per-layer token input: g = gelu_tanh(t) * Es[token, col0 .. col0 + n), t the fp32
//    product of a small projection with the stream, Es a second embedding table whose row holds one slice per layer.
//  * token_side_kernel — the whole per-layer token input for a few rows (decoding), one CTA per row:
//    y = Wp (gelu_tanh(Wg x) * Es[token, slice]);  x += y / rms(y) * w_side;  h = x / rms(x) * w_next.
//    The stream row stays fp32 throughout (the projections read it as it is; only the weights are in the operand type).
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

constexpr int TS_THREADS = 256;

// One CTA per row.  Shared memory: the stream row [W] | the gate vector [n] | reduction scratch.
template <typename T>
__global__ void __launch_bounds__(TS_THREADS) token_side_kernel(float* __restrict__ x, const int* __restrict__ ids,
                                                                const T* __restrict__ side, int lds, int col0,
                                                                const T* __restrict__ wg, const T* __restrict__ wp,
                                                                const T* __restrict__ w_side, const T* __restrict__ w_next,
                                                                T* __restrict__ h, int W, int n, int V, float eps) {
  pdl_wait();                      // programmatic dependent launch: nothing is read before the predecessor is done
  pdl_launch_dependents();
  extern __shared__ float sm[];
  __shared__ float red[33];
  float* xs = sm;                  // [W]
  float* gs = sm + W;              // [n]
  const int m = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* xr = x + (size_t)m * W;
  for (int i = threadIdx.x; i < W; i += blockDim.x) xs[i] = xr[i];
  __syncthreads();
  int tok = ids[m];
  tok = tok < 0 ? 0 : (tok >= V ? V - 1 : tok);
  for (int c = warp; c < n; c += TS_THREADS / 32) {      // a warp per gate channel: Wg[c, :] . x
    const T* wr = wg + (size_t)c * W;
    float d = 0.0f;
    for (int i = lane; i < W; i += 32) d = fmaf(to_f(wr[i]), xs[i], d);
    d = warp_sum(d);
    if (lane == 0) gs[c] = apply_act(d, ACT_GELU_TANH, 0.0f, 0.0f) * to_f(side[(size_t)tok * lds + col0 + c]);
  }
  __syncthreads();
  float ss = 0.0f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {    // a thread per output channel: Wp[i, :] . g (y)
    const T* wr = wp + (size_t)i * n;
    float d = 0.0f;
    for (int c = 0; c < n; ++c) d = fmaf(to_f(wr[c]), gs[c], d);
    xr[i] = d;                                           // parked in the row's own slot until the norm is known (xs holds x)
    ss += d * d;
  }
  const float r = 1.0f / sqrtf(block_sum(ss, red) / (float)W + eps);
  float s2 = 0.0f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {    // each thread re-reads the elements it wrote itself
    const float v = xs[i] + xr[i] * r * to_f(w_side[i]);
    xr[i] = v;
    xs[i] = v;
    s2 += v * v;
  }
  if (w_next == nullptr) return;
  const float r2 = 1.0f / sqrtf(block_sum(s2, red) / (float)W + eps);
  for (int i = threadIdx.x; i < W; i += blockDim.x) h[(size_t)m * W + i] = from_f<T>(xs[i] * r2 * to_f(w_next[i]));
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

extern "C" JL_API int jl_token_side(float* x, const int* ids, const void* side, int lds, int col0, const void* w_gate, const void* w_proj,
                                    const void* w_side, const void* w_next, void* h, int M, int W, int n, int V, float eps, int dtype,
                                    void* stream) {
  JL_CHECK_ARG(M >= 1 && W >= 1 && n >= 1 && V >= 1 && col0 >= 0 && lds >= col0 + n, "jl_token_side: bad shape M=%d W=%d n=%d", M, W, n);
  JL_CHECK_ARG((w_next == nullptr) == (h == nullptr), "jl_token_side: w_next and h come together");
  const size_t smem = (size_t)(W + n) * sizeof(float);
  JL_CHECK_ARG(smem <= 200 * 1024, "jl_token_side: a row of %d + %d floats does not fit shared memory", W, n);
  JL_DISPATCH_DTYPE(dtype, {
    if (smem > 48 * 1024)
      JL_CUDA(cudaFuncSetAttribute(token_side_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    JL_LAUNCH_PDL(token_side_kernel<T>, dim3(M), dim3(TS_THREADS), smem, (cudaStream_t)stream, x, ids, (const T*)side, lds, col0,
                  (const T*)w_gate, (const T*)w_proj, (const T*)w_side, (const T*)w_next, (T*)h, W, n, V, eps);
  });
  JL_CUDA(cudaGetLastError());
  return JL_OK;
}
