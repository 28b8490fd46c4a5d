// Pieces that newer hybrid decoders put around their mixers, in bfloat16 or true float32 (statistics always fp32):
//
//  * embed_pair_norm_kernel — token embedding plus one row of a hashed pair table chosen by (previous token, token), then
//    the model norm; the previous token of every row of the batch is state that the kernel reads and replaces.
//  * causal_conv_kernel     — short causal convolution over time per channel with an activation; the last taps-1 inputs
//    of every row are state.
//  * norm_mean2_kernel      — c * (norm(a) * wa + norm(b) * wb): two mixers that run side by side on the same input.
//  * gated_groupnorm_kernel — (o + skip * x) * act(z), then an RMS norm over equal parts of the row, times a weight.
//  * glu_act_kernel         — gated activations of a fused gate | up product (act(g) * u; the clamped sigmoid form).
//  * talk_mix_kernel        — attention weights mixed across heads, applied to the per-(head, value head) weighted sums.
//  * ssd_gates_kernel       — step size, decay and value scale of a selective state space layer.
//
// Token (b, s) of a call sits at slot *cache_len + s and position slot - pad_left[b]; negative positions are padding.
#include <stdint.h>

#include "jllama_b200.h"
#include "seq_types.cuh"

namespace jl {

__device__ __forceinline__ float softplus_f(float z) { return z > 20.0f ? z : log1pf(expf(z)); }

template <typename T>
__global__ void __launch_bounds__(128) embed_pair_norm_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                                                              const T* __restrict__ pair, const T* __restrict__ norm_w,
                                                              float* __restrict__ out, int* __restrict__ prev_tok,
                                                              const int* __restrict__ cache_len, const int* __restrict__ pad_left,
                                                              int S, int W, int V, int buckets, long long mul_prev,
                                                              long long mul_cur, float eps) {
  pdl_wait();                      // programmatic dependent launch: nothing is read before the predecessor is done
  pdl_launch_dependents();
  __shared__ float red[33];
  __shared__ int prev_s;
  const int m = blockIdx.x, b = m / S, s = m % S;
  const int pos = (cache_len ? *cache_len : 0) + s - (pad_left ? pad_left[b] : 0);
  if (threadIdx.x == 0) prev_s = s > 0 ? ids[m - 1] : prev_tok[b];
  __syncthreads();
  // the block of a row's first token is the only one that touches the row's previous-token slot: it has read it above
  if (s == 0 && threadIdx.x == 0) prev_tok[b] = ids[(size_t)b * S + S - 1];
  float* orow = out + (size_t)m * W;
  if (pos < 0) {
    for (int i = threadIdx.x; i < W; i += blockDim.x) orow[i] = 0.0f;
    return;
  }
  int tok = ids[m];
  tok = tok < 0 ? 0 : (tok >= V ? V - 1 : tok);
  long long r = buckets;
  if (pos > 0) {
    r = ((long long)prev_s * mul_prev + (long long)tok * mul_cur) % (long long)buckets;
    if (r < 0) r += buckets;
  }
  const T* e = table + (size_t)tok * W;
  const T* g = pair + (size_t)r * W;
  float ss = 0.0f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float v = to_f(e[i]) + to_f(g[i]);
    orow[i] = v;
    ss += v * v;
  }
  if (norm_w == nullptr) return;
  const float rn = 1.0f / sqrtf(block_sum(ss, red) / (float)W + eps);
  for (int i = threadIdx.x; i < W; i += blockDim.x) orow[i] = orow[i] * rn * to_f(norm_w[i]);     // own elements only
}

constexpr int CC_MAX_TAPS = 8;
constexpr int CC_CHUNK = 64;       // tokens per CTA along time

// grid (channel blocks, rows, time chunks); a thread owns one channel and walks its chunk with the last taps-1 inputs in
// registers.  Only the first chunk reads the state (chunks are at least taps-1 tokens long) and it is also the one that
// replaces it, from the read-only inputs and the old values it holds in registers.
template <typename T>
__global__ void __launch_bounds__(128) causal_conv_kernel(const float* __restrict__ y, int ldy, int col0, int C,
                                                          const T* __restrict__ w, const T* __restrict__ bias,
                                                          float* __restrict__ state, float* __restrict__ out, int ldo,
                                                          const int* __restrict__ cache_len, const int* __restrict__ pad_left,
                                                          int S, int taps, int act, int chunk) {
  pdl_wait();                      // programmatic dependent launch: nothing is read before the predecessor is done
  pdl_launch_dependents();
  const int c = blockIdx.x * blockDim.x + threadIdx.x, b = blockIdx.y;
  if (c >= C) return;
  const int s0 = blockIdx.z * chunk, s1 = min(S, s0 + chunk);
  const int first = (pad_left ? pad_left[b] : 0) - (cache_len ? *cache_len : 0);      // tokens before it are padding
  const int nh = taps - 1;
  float wv[CC_MAX_TAPS], hist[CC_MAX_TAPS];        // hist[j]: the input j + 1 tokens back
#pragma unroll
  for (int j = 0; j < CC_MAX_TAPS; ++j) { wv[j] = j < taps ? to_f(w[(size_t)c * taps + j]) : 0.0f; hist[j] = 0.0f; }
  const float bv = bias ? to_f(bias[c]) : 0.0f;
  float* st = state + (size_t)b * nh * C + c;      // st[i * C]: the input taps-1-i tokens before this call's first
  auto input = [&](int s) { return s >= first ? y[(size_t)(b * S + s) * ldy + col0 + c] : 0.0f; };
#pragma unroll
  for (int j = 0; j < CC_MAX_TAPS; ++j) {
    if (j >= nh) break;
    const int s = s0 - 1 - j;
    hist[j] = s >= 0 ? input(s) : st[(size_t)(nh + s) * C];
  }
  if (blockIdx.z == 0) {                           // s0 == 0: hist holds the whole old state; write the new one
#pragma unroll
    for (int i = 0; i < CC_MAX_TAPS; ++i) {
      if (i >= nh) break;
      const int s = S - nh + i;                    // the token this state slot holds after the call
      float v;
      if (s >= 0) v = input(s);
      else {                                       // still a token of an earlier call: old slot i + S, i.e. -s - 1 tokens back
        v = 0.0f;
#pragma unroll
        for (int j = 0; j < CC_MAX_TAPS; ++j) if (j == -s - 1) v = hist[j];
      }
      st[(size_t)i * C] = v;
    }
  }
  for (int s = s0; s < s1; ++s) {
    const float xin = input(s);
    float acc = fmaf(wv[taps - 1], xin, bv);
#pragma unroll
    for (int j = 0; j < CC_MAX_TAPS; ++j) if (j < nh) acc = fmaf(wv[nh - 1 - j], hist[j], acc);
    out[(size_t)(b * S + s) * ldo + c] = s >= first ? apply_act(acc, act, 0.0f, 0.0f) : 0.0f;
#pragma unroll
    for (int j = CC_MAX_TAPS - 1; j > 0; --j) hist[j] = hist[j - 1];
    hist[0] = xin;
  }
}

// One CTA per row; on the vector path (W a multiple of 4, 16-byte pitches, W <= 256 * 4 * VPT) both rows stay in registers
// between the sums of squares and the output.
template <typename T, int VPT>
__global__ void __launch_bounds__(256) norm_mean2_kernel(const float* __restrict__ a, int lda, const T* __restrict__ wa,
                                                         const float* __restrict__ b, int ldb, const T* __restrict__ wb, float c,
                                                         float* __restrict__ out, int W, float eps, int vec) {
  pdl_wait();                      // programmatic dependent launch: nothing is read before the predecessor is done
  pdl_launch_dependents();
  __shared__ float red[33];
  const size_t m = blockIdx.x;
  const float* ar = a + m * lda;
  const float* br = b ? b + m * ldb : nullptr;
  float sa = 0.0f, sb = 0.0f;
  if (vec) {
    const int nv = W / 4;
    float av[VPT][4], bv[VPT][4];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = threadIdx.x + i * 256;
      if (idx < nv) {
        load4(ar + 4 * idx, av[i]);
        if (br) load4(br + 4 * idx, bv[i]);
#pragma unroll
        for (int j = 0; j < 4; ++j) { sa += av[i][j] * av[i][j]; if (br) sb += bv[i][j] * bv[i][j]; }
      }
    }
    const float ra = 1.0f / sqrtf(block_sum(sa, red) / (float)W + eps);
    const float rb = br ? 1.0f / sqrtf(block_sum(sb, red) / (float)W + eps) : 0.0f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = threadIdx.x + i * 256;
      if (idx < nv) {
        float w4[4], o4[4];
        load4(wa + 4 * idx, w4);
#pragma unroll
        for (int j = 0; j < 4; ++j) o4[j] = av[i][j] * ra * w4[j];
        if (br) {
          load4(wb + 4 * idx, w4);
#pragma unroll
          for (int j = 0; j < 4; ++j) o4[j] += bv[i][j] * rb * w4[j];
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) o4[j] *= c;
        store4(out + m * W + 4 * idx, o4);
      }
    }
    return;
  }
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float u = ar[i];
    sa += u * u;
    if (br) { const float v = br[i]; sb += v * v; }
  }
  const float ra = 1.0f / sqrtf(block_sum(sa, red) / (float)W + eps);
  const float rb = br ? 1.0f / sqrtf(block_sum(sb, red) / (float)W + eps) : 0.0f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float v = ar[i] * ra * to_f(wa[i]);
    if (br) v += br[i] * rb * to_f(wb[i]);
    out[m * W + i] = c * v;
  }
}

// grid (rows, groups): one CTA per part of a row
template <typename T>
__global__ void __launch_bounds__(128) gated_groupnorm_kernel(const float* __restrict__ o, const float* __restrict__ x, int ldx,
                                                              const T* __restrict__ skip, int P, const float* __restrict__ z,
                                                              int ldz, const T* __restrict__ w, T* __restrict__ out, int N,
                                                              int groups, float eps, int gate_act) {
  pdl_wait();                      // programmatic dependent launch: nothing is read before the predecessor is done
  pdl_launch_dependents();
  __shared__ float red[33];
  const size_t m = blockIdx.x;
  const int n = N / groups, i0 = blockIdx.y * n;
  auto value = [&](int i) {
    float v = o[m * N + i];
    if (x) v = fmaf(skip ? to_f(skip[i / P]) : 1.0f, x[m * ldx + i], v);
    return v * apply_act(z[m * ldz + i], gate_act, 0.0f, 0.0f);
  };
  float ss = 0.0f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) { const float v = value(i0 + i); ss += v * v; }
  const float r = 1.0f / sqrtf(block_sum(ss, red) / (float)n + eps);
  for (int i = threadIdx.x; i < n; i += blockDim.x) out[m * N + i0 + i] = from_f<T>(value(i0 + i) * r * to_f(w[i0 + i]));
}

template <typename T>
__global__ void __launch_bounds__(256) glu_act_kernel(const float* __restrict__ in, int ldi, int g_off, int u_off, T* __restrict__ out,
                                                      int ldo, int M, int F, int kind, int act, float limit, float alpha,
                                                      const int* __restrict__ rows_used, int rows_mult) {
  pdl_wait();                      // programmatic dependent launch: nothing is read before the predecessor is done
  pdl_launch_dependents();
  const size_t rows = rows_used ? (size_t)min(M, *rows_used * rows_mult) : (size_t)M;
  const size_t total = rows * F;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t m = idx / F, j = idx % F;
    float g = in[m * ldi + g_off + j], u = in[m * ldi + u_off + j], v;
    if (kind == 1) {
      g = fminf(g, limit);
      u = fminf(fmaxf(u, -limit), limit);
      v = g * sigmoid_f(alpha * g) * (u + 1.0f);
    } else {
      v = apply_act(g, act, 0.0f, 0.0f) * u;
    }
    out[m * ldo + j] = from_f<T>(v);
  }
}

template <typename T>
__global__ void __launch_bounds__(128) talk_mix_kernel(const float* __restrict__ o, const T* __restrict__ mix, T* __restrict__ out,
                                                       int H, int G, int Gc, int c0, int Dv) {
  pdl_wait();                      // programmatic dependent launch: nothing is read before the predecessor is done
  pdl_launch_dependents();
  const size_t m = blockIdx.x;
  const int h = blockIdx.y, c = h / (H / G) - c0;          // grid (tokens, heads)
  if (c < 0 || c >= Gc) return;
  const float* orow = o + m * H * Gc * Dv;
  for (int d = threadIdx.x; d < Dv; d += blockDim.x) {
    float acc = 0.0f;
    for (int g = 0; g < H; ++g) acc = fmaf(to_f(mix[h * H + g]), orow[((size_t)g * Gc + c) * Dv + d], acc);
    out[(m * H + h) * Dv + d] = from_f<T>(acc);
  }
}

template <typename T>
__global__ void ssd_gates_kernel(const float* __restrict__ y, int ldy, int dt_off, const T* __restrict__ dt_bias,
                                 const T* __restrict__ a_log, float* __restrict__ aux, int M, int H) {
  pdl_wait();                      // programmatic dependent launch: nothing is read before the predecessor is done
  pdl_launch_dependents();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= M * H) return;
  const int m = i / H, h = i % H;
  const float dt = softplus_f(y[(size_t)m * ldy + dt_off + h] + to_f(dt_bias[h]));
  aux[(size_t)m * 2 * H + h] = expf(-expf(to_f(a_log[h])) * dt);
  aux[(size_t)m * 2 * H + H + h] = dt;
}

}  // namespace jl

using namespace jl;

extern "C" JL_API int jl_embed_pair_norm(const int* ids, const void* table, const void* pair, const void* norm_w, float* out,
                                         int* prev_tok, const int* cache_len, const int* pad_left, int B, int S, int W, int V,
                                         int buckets, long long mul_prev, long long mul_cur, float eps, int dtype, void* stream) {
  JL_CHECK_ARG(B >= 1 && S >= 1 && W >= 1 && V >= 1 && buckets >= 1 && prev_tok != nullptr, "jl_embed_pair_norm: bad shape");
  JL_DISPATCH_DTYPE(dtype, JL_LAUNCH_PDL(embed_pair_norm_kernel<T>, dim3(B * S), dim3(128), 0, stream, ids, (const T*)table,
                                         (const T*)pair, (const T*)norm_w, out, prev_tok, cache_len, pad_left, S, W, V, buckets,
                                         mul_prev, mul_cur, eps));
  JL_CUDA(cudaGetLastError());
  return JL_OK;
}

extern "C" JL_API int jl_causal_conv(const float* y, int ldy, int col0, int C, const void* w, const void* bias, float* state,
                                     float* out, int ldo, const int* cache_len, const int* pad_left, int B, int S, int taps,
                                     int act, int dtype, void* stream) {
  JL_CHECK_ARG(B >= 1 && S >= 1 && C >= 1 && ldo >= C, "jl_causal_conv: bad shape");
  JL_CHECK_ARG(taps >= 1 && taps <= CC_MAX_TAPS, "jl_causal_conv: %d taps (1 .. %d)", taps, CC_MAX_TAPS);
  JL_CHECK_ARG(taps == 1 || state != nullptr, "jl_causal_conv: no state for %d taps", taps);
  const int chunk = CC_CHUNK;
  dim3 grid((C + 127) / 128, B, (S + chunk - 1) / chunk);
  JL_DISPATCH_DTYPE(dtype, JL_LAUNCH_PDL(causal_conv_kernel<T>, dim3(grid), dim3(128), 0, stream, y, ldy, col0, C, (const T*)w,
                                         (const T*)bias, state, out, ldo, cache_len, pad_left, S, taps, act, chunk));
  JL_CUDA(cudaGetLastError());
  return JL_OK;
}

extern "C" JL_API int jl_norm_mean2(const float* a, int lda, const void* wa, const float* b, int ldb, const void* wb, float c,
                                    float* out, int M, int W, float eps, int dtype, void* stream) {
  JL_CHECK_ARG(M >= 1 && W >= 1 && a != nullptr && wa != nullptr && (b == nullptr || wb != nullptr), "jl_norm_mean2: bad arguments");
  const int vec = W % 4 == 0 && lda % 4 == 0 && ldb % 4 == 0 && ((uintptr_t)a | (uintptr_t)b | (uintptr_t)out) % 16 == 0 &&
                  ((uintptr_t)wa | (uintptr_t)wb) % 16 == 0 && W <= 256 * 4 * 8;
  if (vec && W <= 256 * 4 * 2)
    JL_DISPATCH_DTYPE(dtype, JL_LAUNCH_PDL((norm_mean2_kernel<T, 2>), dim3(M), dim3(256), 0, stream, a, lda, (const T*)wa, b, ldb,
                                           (const T*)wb, c, out, W, eps, 1));
  else
    JL_DISPATCH_DTYPE(dtype, JL_LAUNCH_PDL((norm_mean2_kernel<T, 8>), dim3(M), dim3(256), 0, stream, a, lda, (const T*)wa, b, ldb,
                                           (const T*)wb, c, out, W, eps, vec));
  JL_CUDA(cudaGetLastError());
  return JL_OK;
}

extern "C" JL_API int jl_gated_groupnorm(const float* o, const float* x, int ldx, const void* skip, int P, const float* z, int ldz,
                                         const void* w, void* out, int M, int N, int groups, float eps, int gate_act, int dtype,
                                         void* stream) {
  JL_CHECK_ARG(M >= 1 && N >= 1 && groups >= 1 && N % groups == 0 && P >= 1, "jl_gated_groupnorm: %d columns in %d groups", N, groups);
  JL_DISPATCH_DTYPE(dtype, JL_LAUNCH_PDL(gated_groupnorm_kernel<T>, dim3(M, groups), dim3(128), 0, stream, o, x, ldx, (const T*)skip,
                                         P, z, ldz, (const T*)w, (T*)out, N, groups, eps, gate_act));
  JL_CUDA(cudaGetLastError());
  return JL_OK;
}

extern "C" JL_API int jl_glu_act(const float* in, int ldi, int g_off, int u_off, void* out, int ldo, int M, int F, int kind,
                                 int act, float limit, float alpha, const int* rows_used, int rows_mult, int dtype, void* stream) {
  JL_CHECK_ARG(M >= 1 && F >= 1 && (kind == 0 || kind == 1), "jl_glu_act: bad arguments");
  const size_t total = (size_t)M * F;
  const int blocks = (int)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
  JL_DISPATCH_DTYPE(dtype, JL_LAUNCH_PDL(glu_act_kernel<T>, dim3(blocks), dim3(256), 0, stream, in, ldi, g_off, u_off, (T*)out, ldo,
                                         M, F, kind, act, limit, alpha, rows_used, rows_mult));
  JL_CUDA(cudaGetLastError());
  return JL_OK;
}

extern "C" JL_API int jl_talk_mix(const float* o, const void* mix, void* out, int M, int H, int G, int Gc, int c0, int Dv,
                                  int dtype, void* stream) {
  JL_CHECK_ARG(M >= 1 && H >= 1 && G >= 1 && H % G == 0 && Gc >= 1 && c0 >= 0 && c0 + Gc <= G && Dv >= 1, "jl_talk_mix: bad shape");
  JL_DISPATCH_DTYPE(dtype, JL_LAUNCH_PDL(talk_mix_kernel<T>, dim3(M, H), dim3(128), 0, stream, o, (const T*)mix, (T*)out, H, G, Gc, c0, Dv));
  JL_CUDA(cudaGetLastError());
  return JL_OK;
}

extern "C" JL_API int jl_ssd_gates(const float* y, int ldy, int dt_off, const void* dt_bias, const void* a_log, float* aux, int M,
                                   int H, int dtype, void* stream) {
  JL_CHECK_ARG(M >= 1 && H >= 1, "jl_ssd_gates: bad shape");
  JL_DISPATCH_DTYPE(dtype, JL_LAUNCH_PDL(ssd_gates_kernel<T>, dim3((M * H + 127) / 128), dim3(128), 0, stream, y, ldy, dt_off,
                                         (const T*)dt_bias, (const T*)a_log, aux, M, H));
  JL_CUDA(cudaGetLastError());
  return JL_OK;
}
