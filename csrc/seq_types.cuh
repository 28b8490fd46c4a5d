// Element-type plumbing of the kernels that run in either bfloat16 or true float32 (the hybrid
// attention / linear-recurrence models).  dtype codes of the C ABI: 0 = bfloat16, 1 = float32.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>

#include "common.cuh"

namespace jl {

enum { DT_BF16 = 0, DT_F32 = 1 };
// epilogue / activation codes shared by the generic linears and jl_act_cast
// ACT_XIELU: z > 0: p0 z^2 + z/2;  z <= 0: p1 (e^z - 1 - z) + z/2  (p0, p1 positive, formed by the caller from the layer's two numbers)
enum { ACT_NONE = 0, ACT_RELU2 = 1, ACT_GELU_TANH = 2, ACT_SILU = 3, ACT_SCALE_SOFTCAP = 4, ACT_SIGMOID = 5, ACT_XIELU = 6, ACT_LAST = ACT_XIELU };

__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// exact-math activations (this file's users are compiled without fast-math)
__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float apply_act(float z, int act, float p0, float p1) {
  switch (act) {
    case ACT_RELU2: { float r = fmaxf(z, 0.0f); return r * r; }
    case ACT_GELU_TANH: return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    case ACT_SILU: return z * sigmoid_f(z);
    case ACT_SIGMOID: return sigmoid_f(z);
    case ACT_XIELU: return z > 0.0f ? fmaf(p0 * z, z, 0.5f * z) : fmaf(p1, expm1f(z) - z, 0.5f * z);
    case ACT_SCALE_SOFTCAP: { float s = z * p0; return p1 > 0.0f ? p1 * tanhf(s / p1) : s; }
    default: return z;
  }
}

// Channel d of a head after the rotary embedding of its first `rot` channels (even): the pair (u, v) turns into
// (u cos - v sin, v cos + u sin).  layout 0 pairs channel 2i with 2i+1, layout 1 pairs channel i with i + rot/2; ct / st are
// the cos / sin of the token's position for the rot/2 pairs (any factor on them is already in the table).
template <typename S>
__device__ __forceinline__ float rotary_channel(const S* __restrict__ src, int d, int rot, int layout, const float* __restrict__ ct,
                                                const float* __restrict__ st) {
  if (d >= rot) return to_f(src[d]);
  if (layout == 0) {
    const int i = d >> 1;
    return (d & 1) ? to_f(src[d]) * ct[i] + to_f(src[d - 1]) * st[i] : to_f(src[d]) * ct[i] - to_f(src[d + 1]) * st[i];
  }
  const int half = rot >> 1;
  return d < half ? to_f(src[d]) * ct[d] - to_f(src[d + half]) * st[d]
                  : to_f(src[d]) * ct[d - half] + to_f(src[d - half]) * st[d - half];
}

// four consecutive elements as floats (16-byte / 8-byte accesses: the address has to be aligned accordingly)
__device__ __forceinline__ void load4(const float* p, float (&v)[4]) {
  const float4 t = *reinterpret_cast<const float4*>(p);
  v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 t = *reinterpret_cast<const uint2*>(p);
  v[0] = bf16_lo(t.x); v[1] = bf16_hi(t.x); v[2] = bf16_lo(t.y); v[3] = bf16_hi(t.y);
}
__device__ __forceinline__ void store4(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, const float (&v)[4]) {
  *reinterpret_cast<uint2*>(p) = make_uint2(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]));
}

__device__ __forceinline__ float block_sum(float v, float* red /* >= 33 floats of shared memory */) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  __syncthreads();                      // red may still be read from a previous call
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nw ? red[lane] : 0.0f;
    t = warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

// Launch with programmatic dependent launch enabled (common.cuh launch_pdl counts the launch).  A kernel name with template
// commas goes in parentheses.  The launch error, if any, is read by the caller with cudaGetLastError().
#define JL_LAUNCH_PDL(kernel, grid, block, smem, stream, ...) \
  (void)jl::launch_pdl(kernel, grid, block, (size_t)(smem), (cudaStream_t)(stream), __VA_ARGS__)

#define JL_DISPATCH_DTYPE(dt, ...)                                   \
  do {                                                               \
    if ((dt) == jl::DT_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
    else { using T = float; __VA_ARGS__; }                           \
  } while (0)

}  // namespace jl
