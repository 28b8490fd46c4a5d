// Row-wise kernels of the models whose residual stream is float32: embedding into fp32, RMS norm with a weight offset
// (weight stored around zero: offset 1; plain weight: offset 0), the "norm after the sublayer + residual add + norm
// before the next sublayer" fusion, per-head norm with an output gate, and the activation / cast pass that follows a
// tensor-core GEMM.  All statistics in fp32, exact math (no fast-math for this file).
#include "jllama_b200.h"
#include "seq_types.cuh"

namespace jl {

template <typename T>
__global__ void embed_f32_kernel(const int* __restrict__ ids, const T* __restrict__ table, float* __restrict__ out, int W,
                                 int V) {
  pdl_wait();                      // programmatic dependent launch: nothing is read before the predecessor is done
  pdl_launch_dependents();
  const int m = blockIdx.x;
  int id = ids[m];
  id = id < 0 ? 0 : (id >= V ? V - 1 : id);
  const T* row = table + (size_t)id * W;
  for (int i = threadIdx.x; i < W; i += blockDim.x) out[(size_t)m * W + i] = to_f(row[i]);
}

// out[m, :] = x[m, :] / sqrt(mean(x^2) + eps) * (offset + w)
template <typename T>
__global__ void norm_f32_kernel(const float* __restrict__ x, const T* __restrict__ w, T* __restrict__ out, int W, float eps,
                                float offset) {
  pdl_wait();                      // programmatic dependent launch: nothing is read before the predecessor is done
  pdl_launch_dependents();
  __shared__ float red[33];
  const float* xr = x + (size_t)blockIdx.x * W;
  float ss = 0.0f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) { float v = xr[i]; ss += v * v; }
  const float r = 1.0f / sqrtf(block_sum(ss, red) / (float)W + eps);
  for (int i = threadIdx.x; i < W; i += blockDim.x)
    out[(size_t)blockIdx.x * W + i] = from_f<T>(xr[i] * r * (offset + to_f(w[i])));
}

// x[m, :] += norm(y[m, :]) * (offset + w_post);  if w_next: h[m, :] = norm(x[m, :]) * (offset + w_next)
template <typename T>
__global__ void postnorm_add_kernel(const float* __restrict__ y, int ldy, const T* __restrict__ w_post, float* __restrict__ x,
                                    const T* __restrict__ w_next, T* __restrict__ h, int W, float eps, float offset) {
  pdl_wait();                      // programmatic dependent launch: nothing is read before the predecessor is done
  pdl_launch_dependents();
  __shared__ float red[33];
  const float* yr = y + (size_t)blockIdx.x * ldy;
  float* xr = x + (size_t)blockIdx.x * W;
  float ss = 0.0f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) { float v = yr[i]; ss += v * v; }
  const float r = 1.0f / sqrtf(block_sum(ss, red) / (float)W + eps);
  float s2 = 0.0f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float v = xr[i] + yr[i] * r * (offset + to_f(w_post[i]));
    xr[i] = v;
    s2 += v * v;
  }
  if (w_next == nullptr) return;
  const float r2 = 1.0f / sqrtf(block_sum(s2, red) / (float)W + eps);
  for (int i = threadIdx.x; i < W; i += blockDim.x)          // each thread re-reads the elements it wrote itself
    h[(size_t)blockIdx.x * W + i] = from_f<T>(xr[i] * r2 * (offset + to_f(w_next[i])));
}

// The same step with the row held in registers: 16-byte loads, x and y read once, x and h written once.
// W % 4 == 0, ldy % 4 == 0, W <= 256 * 4 * VPT.
template <typename T, int VPT>
__global__ void __launch_bounds__(256) postnorm_add_vec_kernel(const float* __restrict__ y, int ldy, const T* __restrict__ w_post,
                                                               float* __restrict__ x, const T* __restrict__ w_next,
                                                               T* __restrict__ h, int W, float eps, float offset) {
  pdl_wait();                      // programmatic dependent launch: nothing is read before the predecessor is done
  pdl_launch_dependents();
  __shared__ float red[33];
  const float* yr = y + (size_t)blockIdx.x * ldy;
  float* xr = x + (size_t)blockIdx.x * W;
  const int nv = W / 4;
  float yv[VPT][4], xv[VPT][4];
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * 256;
    if (idx < nv) {
      load4(yr + 4 * idx, yv[i]);
      load4(xr + 4 * idx, xv[i]);
#pragma unroll
      for (int j = 0; j < 4; ++j) ss += yv[i][j] * yv[i][j];
    }
  }
  const float r = 1.0f / sqrtf(block_sum(ss, red) / (float)W + eps);
  float s2 = 0.0f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * 256;
    if (idx < nv) {
      float wv[4];
      load4(w_post + 4 * idx, wv);
#pragma unroll
      for (int j = 0; j < 4; ++j) { xv[i][j] += yv[i][j] * r * (offset + wv[j]); s2 += xv[i][j] * xv[i][j]; }
      store4(xr + 4 * idx, xv[i]);
    }
  }
  if (w_next == nullptr) return;
  const float r2 = 1.0f / sqrtf(block_sum(s2, red) / (float)W + eps);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * 256;
    if (idx < nv) {
      float wv[4], hv[4];
      load4(w_next + 4 * idx, wv);
#pragma unroll
      for (int j = 0; j < 4; ++j) hv[j] = xv[i][j] * r2 * (offset + wv[j]);
      store4(h + (size_t)blockIdx.x * W + 4 * idx, hv);
    }
  }
}

// Residual step of a block whose branches read the same input: x[m, :] += mult * (y1[m, :] + y2[m, :]) (y1 / y2 may be
// absent), then up to two norms of the updated row with plain weights: h1 = norm(x) * w1, h2 = norm(x) * w2 (the inputs of
// the next block's two branches).  With y1 == y2 == nullptr it only forms the norms.  The row is kept in registers:
// 4 floats per thread and step, W <= 256 * 4 * VPT on the vector path.
template <typename T, int VPT>
__global__ void __launch_bounds__(256) branch_add_norm_kernel(const float* __restrict__ y1, int ld1, const float* __restrict__ y2,
                                                              int ld2, float mult, float* __restrict__ x,
                                                              const T* __restrict__ w1, T* __restrict__ h1,
                                                              const T* __restrict__ w2, T* __restrict__ h2, int W, float eps,
                                                              int vec) {
  pdl_wait();                      // programmatic dependent launch: nothing is read before the predecessor is done
  pdl_launch_dependents();
  __shared__ float red[33];
  const size_t m = blockIdx.x;
  float* xr = x + m * W;
  const float* a = y1 ? y1 + m * ld1 : nullptr;
  const float* b = y2 ? y2 + m * ld2 : nullptr;
  float ss = 0.0f;
  if (vec) {
    const int nv = W / 4;
    float xv[VPT][4];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = threadIdx.x + i * 256;
      if (idx < nv) {
        load4(xr + 4 * idx, xv[i]);
        if (a || b) {
          float s[4] = {0.f, 0.f, 0.f, 0.f}, t[4];
          if (a) load4(a + 4 * idx, s);
          if (b) { load4(b + 4 * idx, t);
#pragma unroll
            for (int j = 0; j < 4; ++j) s[j] += t[j]; }
#pragma unroll
          for (int j = 0; j < 4; ++j) xv[i][j] = fmaf(mult, s[j], xv[i][j]);
          store4(xr + 4 * idx, xv[i]);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) ss += xv[i][j] * xv[i][j];
      }
    }
    if (w1 == nullptr && w2 == nullptr) return;
    const float r = 1.0f / sqrtf(block_sum(ss, red) / (float)W + eps);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = threadIdx.x + i * 256;
      if (idx < nv) {
        float wv[4], hv[4];
        if (w1) {
          load4(w1 + 4 * idx, wv);
#pragma unroll
          for (int j = 0; j < 4; ++j) hv[j] = xv[i][j] * r * wv[j];
          store4(h1 + m * W + 4 * idx, hv);
        }
        if (w2) {
          load4(w2 + 4 * idx, wv);
#pragma unroll
          for (int j = 0; j < 4; ++j) hv[j] = xv[i][j] * r * wv[j];
          store4(h2 + m * W + 4 * idx, hv);
        }
      }
    }
    return;
  }
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float v = xr[i];
    if (a || b) {
      const float s = (a ? a[i] : 0.0f) + (b ? b[i] : 0.0f);
      v = fmaf(mult, s, v);
      xr[i] = v;
    }
    ss += v * v;
  }
  if (w1 == nullptr && w2 == nullptr) return;
  const float r = 1.0f / sqrtf(block_sum(ss, red) / (float)W + eps);
  for (int i = threadIdx.x; i < W; i += blockDim.x) {       // each thread re-reads the elements it wrote itself
    const float v = xr[i] * r;
    if (w1) h1[m * W + i] = from_f<T>(v * to_f(w1[i]));
    if (w2) h2[m * W + i] = from_f<T>(v * to_f(w2[i]));
  }
}

// One warp per (token, head): out = o / sqrt(mean_v(o^2) + eps) * w[v] * act(gate)   (w == nullptr: no weight)
template <typename T>
__global__ void headnorm_gate_kernel(const float* __restrict__ o, const T* __restrict__ w, const float* __restrict__ gate,
                                     int ldg, T* __restrict__ out, int M, int H, int V, float eps, int gate_act) {
  pdl_wait();                      // programmatic dependent launch: nothing is read before the predecessor is done
  pdl_launch_dependents();
  const int wid = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (wid >= M * H) return;
  const int m = wid / H, hh = wid % H;
  const float* orow = o + ((size_t)m * H + hh) * V;
  float ss = 0.0f;
  for (int i = lane; i < V; i += 32) { float v = orow[i]; ss += v * v; }
  const float r = 1.0f / sqrtf(warp_sum(ss) / (float)V + eps);
  const float* grow = gate + (size_t)m * ldg + (size_t)hh * V;
  for (int i = lane; i < V; i += 32)
    out[((size_t)m * H + hh) * V + i] = from_f<T>(orow[i] * r * (w ? to_f(w[i]) : 1.0f) * apply_act(grow[i], gate_act, 0.f, 0.f));
}

// out[m, n] = act(in[m, n]) for an fp32 [M, N] block with row pitch ldi; out has pitch ldo (may alias in for OutT = float)
template <typename OutT>
__global__ void act_cast_kernel(const float* __restrict__ in, int ldi, OutT* __restrict__ out, int ldo, int M, int N, int act,
                                float p0, float p1) {
  pdl_wait();                      // programmatic dependent launch: nothing is read before the predecessor is done
  pdl_launch_dependents();
  const size_t total = (size_t)M * N;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t m = idx / N, n = idx % N;
    out[m * ldo + n] = from_f<OutT>(apply_act(in[m * ldi + n], act, p0, p1));
  }
}

// data[m, n] = act(data[m, n]) in place, 16 bytes per thread and step where the pitch allows
template <typename T>
__global__ void act_inplace_kernel(T* __restrict__ data, int ld, int M, int N, int act, float p0, float p1, int vec) {
  pdl_wait();                      // programmatic dependent launch: nothing is read before the predecessor is done
  pdl_launch_dependents();
  constexpr int VN = 16 / sizeof(T);
  if (vec) {
    const size_t per_row = N / VN, total = (size_t)M * per_row;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
      T* ptr = data + (idx / per_row) * ld + (idx % per_row) * VN;
      uint4 raw = *reinterpret_cast<uint4*>(ptr);
      T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
      for (int j = 0; j < VN; ++j) e[j] = from_f<T>(apply_act(to_f(e[j]), act, p0, p1));
      *reinterpret_cast<uint4*>(ptr) = raw;
    }
    return;
  }
  const size_t total = (size_t)M * N;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    T* ptr = data + (idx / N) * ld + idx % N;
    *ptr = from_f<T>(apply_act(to_f(*ptr), act, p0, p1));
  }
}

}  // namespace jl

using namespace jl;

extern "C" JL_API int jl_act_inplace(void* data, int ld, int M, int N, int act, float p0, float p1, int dtype, void* stream) {
  JL_CHECK_ARG(M >= 1 && N >= 1 && ld >= N, "jl_act_inplace: bad shape M=%d N=%d ld=%d", M, N, ld);
  const int vn = dtype == DT_BF16 ? 8 : 4;
  const int vec = N % vn == 0 && ld % vn == 0 && (uintptr_t)data % 16 == 0;
  const size_t work = (size_t)M * N / (vec ? vn : 1);
  const int blocks = (int)((work + 255) / 256 < 148 * 8 ? (work + 255) / 256 : 148 * 8);
  JL_DISPATCH_DTYPE(dtype, JL_LAUNCH_PDL(act_inplace_kernel<T>, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, (T*)data, ld, M, N, act, p0, p1, vec));
  JL_CUDA(cudaGetLastError());
  return JL_OK;
}

extern "C" JL_API int jl_embed_f32(const int* ids, const void* table, float* out, int M, int W, int V, int dtype, void* stream) {
  JL_CHECK_ARG(M >= 1 && W >= 1 && V >= 1, "jl_embed_f32: bad shape M=%d W=%d V=%d", M, W, V);
  JL_DISPATCH_DTYPE(dtype, JL_LAUNCH_PDL(embed_f32_kernel<T>, dim3(M), dim3(128), 0, (cudaStream_t)stream, ids, (const T*)table, out, W, V));
  JL_CUDA(cudaGetLastError());
  return JL_OK;
}

extern "C" JL_API int jl_norm_f32(const float* x, const void* w, void* out, int M, int W, float eps, float offset, int dtype,
                                  void* stream) {
  JL_CHECK_ARG(M >= 1 && W >= 1, "jl_norm_f32: bad shape M=%d W=%d", M, W);
  JL_DISPATCH_DTYPE(dtype, JL_LAUNCH_PDL(norm_f32_kernel<T>, dim3(M), dim3(256), 0, (cudaStream_t)stream, x, (const T*)w, (T*)out, W, eps, offset));
  JL_CUDA(cudaGetLastError());
  return JL_OK;
}

extern "C" JL_API int jl_postnorm_add(const float* y, int ldy, const void* w_post, float* x, const void* w_next, void* h, int M,
                                      int W, float eps, float offset, int dtype, void* stream) {
  JL_CHECK_ARG(M >= 1 && W >= 1 && ldy >= W, "jl_postnorm_add: bad shape M=%d W=%d ldy=%d", M, W, ldy);
  JL_CHECK_ARG((w_next == nullptr) == (h == nullptr), "jl_postnorm_add: w_next and h come together");
  const bool vec = W % 4 == 0 && ldy % 4 == 0 && W <= 256 * 4 * 16 && (uintptr_t)y % 16 == 0 && (uintptr_t)x % 16 == 0 &&
                   (uintptr_t)w_post % 16 == 0 && (uintptr_t)w_next % 16 == 0 && (uintptr_t)h % 16 == 0;
  if (vec) {
    const int vpt = (W / 4 + 255) / 256;
#define JL_PN(V)                                                                                                         \
  JL_DISPATCH_DTYPE(dtype, JL_LAUNCH_PDL((postnorm_add_vec_kernel<T, V>), dim3(M), dim3(256), 0, (cudaStream_t)stream, y, ldy, (const T*)w_post, x, \
                                                                                               (const T*)w_next, (T*)h, W, eps, offset))
    if (vpt <= 1) JL_PN(1); else if (vpt <= 2) JL_PN(2); else if (vpt <= 4) JL_PN(4); else if (vpt <= 8) JL_PN(8); else JL_PN(16);
#undef JL_PN
    JL_CUDA(cudaGetLastError());
    return JL_OK;
  }
  JL_DISPATCH_DTYPE(dtype, JL_LAUNCH_PDL(postnorm_add_kernel<T>, dim3(M), dim3(256), 0, (cudaStream_t)stream, y, ldy, (const T*)w_post, x,
                                                                                        (const T*)w_next, (T*)h, W, eps, offset));
  JL_CUDA(cudaGetLastError());
  return JL_OK;
}

extern "C" JL_API int jl_branch_add_norm(const float* y1, int ld1, const float* y2, int ld2, float mult, float* x, const void* w1,
                                         void* h1, const void* w2, void* h2, int M, int W, float eps, int dtype, void* stream) {
  JL_CHECK_ARG(M >= 1 && W >= 1, "jl_branch_add_norm: bad shape M=%d W=%d", M, W);
  JL_CHECK_ARG((w1 == nullptr) == (h1 == nullptr) && (w2 == nullptr) == (h2 == nullptr), "jl_branch_add_norm: a weight and its output come together");
  JL_CHECK_ARG((y1 == nullptr || ld1 >= W) && (y2 == nullptr || ld2 >= W), "jl_branch_add_norm: row pitch below W=%d", W);
  const bool vec = W % 4 == 0 && (y1 == nullptr || ld1 % 4 == 0) && (y2 == nullptr || ld2 % 4 == 0) && W <= 256 * 4 * 16 &&
                   (uintptr_t)y1 % 16 == 0 && (uintptr_t)y2 % 16 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)w1 % 16 == 0 &&
                   (uintptr_t)w2 % 16 == 0 && (uintptr_t)h1 % 16 == 0 && (uintptr_t)h2 % 16 == 0;
  const int vpt = vec ? (W / 4 + 255) / 256 : 1;
#define JL_BA(V)                                                                                                              \
  JL_DISPATCH_DTYPE(dtype, JL_LAUNCH_PDL((branch_add_norm_kernel<T, V>), dim3(M), dim3(256), 0, (cudaStream_t)stream, y1, ld1, y2, ld2, \
                                         mult, x, (const T*)w1, (T*)h1, (const T*)w2, (T*)h2, W, eps, (int)vec))
  if (vpt <= 1) JL_BA(1); else if (vpt <= 2) JL_BA(2); else if (vpt <= 4) JL_BA(4); else if (vpt <= 8) JL_BA(8); else JL_BA(16);
#undef JL_BA
  JL_CUDA(cudaGetLastError());
  return JL_OK;
}

extern "C" JL_API int jl_headnorm_gate(const float* o, const void* w, const float* gate, int ldg, void* out, int M, int H, int V,
                                       float eps, int gate_act, int dtype, void* stream) {
  JL_CHECK_ARG(M >= 1 && H >= 1 && V >= 1, "jl_headnorm_gate: bad shape M=%d H=%d V=%d", M, H, V);
  const int warps = 4, blocks = (M * H + warps - 1) / warps;
  JL_DISPATCH_DTYPE(dtype, JL_LAUNCH_PDL(headnorm_gate_kernel<T>, dim3(blocks), dim3(warps * 32), 0, (cudaStream_t)stream, 
                               o, (const T*)w, gate, ldg, (T*)out, M, H, V, eps, gate_act));
  JL_CUDA(cudaGetLastError());
  return JL_OK;
}

extern "C" JL_API int jl_act_cast(const float* in, int ldi, void* out, int ldo, int M, int N, int act, float p0, float p1,
                                  int out_dtype, void* stream) {
  JL_CHECK_ARG(M >= 1 && N >= 1 && ldi >= N && ldo >= N, "jl_act_cast: bad shape M=%d N=%d ldi=%d ldo=%d", M, N, ldi, ldo);
  const size_t total = (size_t)M * N;
  const int blocks = (int)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
  JL_DISPATCH_DTYPE(out_dtype, JL_LAUNCH_PDL(act_cast_kernel<T>, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, in, ldi, (T*)out, ldo, M, N, act, p0, p1));
  JL_CUDA(cudaGetLastError());
  return JL_OK;
}
