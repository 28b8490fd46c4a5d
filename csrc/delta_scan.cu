// Gated delta rule with one decay per key channel: per head a matrix state S [D x Dv] that every token first decays, then
// corrects towards its value along its key, then reads with its query:
//     S <- diag(a_t) S;   e_t = beta_t (v_t - S^T k_t);   S <- S + k_t e_t^T;   o_t = S^T q_t.
// The update is not a plain linear recurrence in S (the correction multiplies S by I - beta k k^T), so the tokens of a row
// run in order; the Dv columns of S are independent of one another and spread over threads and CTAs.
//
// Two launches.  delta_prep_kernel is token-parallel: unit-length q and k per head (q also times D^(-1/2)), their dot
// product, beta = sigmoid(.), and the decays a = exp(-exp(A_log_h) softplus(A2 z + bias)) from the rank-R input z — all
// fp32 — written as one record per (token, head) in the layout the scan stages in shared memory.  delta_scan_kernel walks
// the tokens: a thread owns 32 key channels of one value column in registers, the P = ceil(D / 32) lanes of a column are
// adjacent.  With c = a ⊙ s the two dot products k·c and q·c are formed in one pass and reduced together, and
// o = q·c + (q·k) e needs no second reduction; the second pass adds k e to the state.
#include "jllama_b200.h"
#include "seq_types.cuh"

namespace jl {

constexpr int DS_DP = 32;            // key channels per thread
constexpr int DS_PITCH = DS_DP + 4;  // floats per 32 channels in a record: 16-byte rows, distinct banks per lane group
constexpr int DS_TC = 16;            // tokens staged per chunk
constexpr int DS_THREADS = 128;

__device__ __forceinline__ float delta_softplus(float z) { return z > 20.0f ? z : log1pf(expf(z)); }
__host__ __device__ inline int delta_record_floats(int P, int Dv) { return 3 * P * DS_PITCH + ((Dv + 3) & ~3) + 4; }

struct DeltaParams {
  const float* u; int ldu;           // q | k | v after their convolutions
  int q_off, k_off, v_off, G;        // G q / k heads shared by H / G heads each
  const float* y; int ldy;           // projection row: beta logits and the rank-R decay input
  int b_off, a_off;
  int B, S, H, D, Dv, R, P;
  const int* cache_len; const int* pad_left;
  float* state;                      // [B][H][D][Dv]
  float* o;                          // [B*S][H][Dv]
  float* rec;                        // [B*S][H][record]
};

// one CTA per token; a warp per head for the unit vectors, then all threads for the decays and the values
template <typename T>
__global__ void __launch_bounds__(128) delta_prep_kernel(DeltaParams p, const T* __restrict__ a2, const T* __restrict__ a_bias,
                                                         const T* __restrict__ a_log) {
  pdl_wait();                      // programmatic dependent launch: nothing is read before the predecessor is done
  pdl_launch_dependents();
  extern __shared__ float sm[];                                // [R] decay input | [G][3] 1/|q| * D^-1/2, 1/|k|, q·k
  float* zs = sm;
  float* hs = sm + p.R;
  const int m = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const float* ur = p.u + (size_t)m * p.ldu;
  const float* yr = p.y + (size_t)m * p.ldy;
  for (int r = threadIdx.x; r < p.R; r += blockDim.x) zs[r] = yr[p.a_off + r];
  for (int g = warp; g < p.G; g += nw) {
    const float* q = ur + p.q_off + g * p.D;
    const float* k = ur + p.k_off + g * p.D;
    float qq = 0.0f, kk = 0.0f, qk = 0.0f;
    for (int d = lane; d < p.D; d += 32) { qq = fmaf(q[d], q[d], qq); kk = fmaf(k[d], k[d], kk); qk = fmaf(q[d], k[d], qk); }
    qq = warp_sum(qq); kk = warp_sum(kk); qk = warp_sum(qk);
    if (lane == 0) {
      const float rq = 1.0f / sqrtf(qq + 1e-6f) / sqrtf((float)p.D), rk = 1.0f / sqrtf(kk + 1e-6f);
      hs[3 * g] = rq; hs[3 * g + 1] = rk; hs[3 * g + 2] = qk * rq * rk;
    }
  }
  __syncthreads();
  const int P = p.P, RF = delta_record_floats(P, p.Dv), per = p.H / p.G, chans = P * DS_DP;
  float* out = p.rec + (size_t)m * p.H * RF;
  for (int i = threadIdx.x; i < p.H * chans; i += blockDim.x) {
    const int h = i / chans, d = i % chans, g = h / per;
    float qv = 0.0f, kv = 0.0f, av = 1.0f;
    if (d < p.D) {
      qv = ur[p.q_off + g * p.D + d] * hs[3 * g];
      kv = ur[p.k_off + g * p.D + d] * hs[3 * g + 1];
      const int n = h * p.D + d;
      float z = to_f(a_bias[n]);
      for (int r = 0; r < p.R; ++r) z = fmaf(to_f(a2[(size_t)n * p.R + r]), zs[r], z);
      av = expf(-expf(to_f(a_log[h])) * delta_softplus(z));
    }
    float* o = out + (size_t)h * RF + (d / DS_DP) * DS_PITCH + d % DS_DP;
    o[0] = qv; o[P * DS_PITCH] = kv; o[2 * P * DS_PITCH] = av;
  }
  const int dvp = (p.Dv + 3) & ~3;
  for (int i = threadIdx.x; i < p.H * (dvp + 4); i += blockDim.x) {
    const int h = i / (dvp + 4), c = i % (dvp + 4);
    float v = 0.0f;
    if (c < p.Dv) v = ur[p.v_off + h * p.Dv + c];
    else if (c == dvp) v = sigmoid_f(yr[p.b_off + h]);
    else if (c == dvp + 1) v = hs[3 * (h / per) + 2];
    out[(size_t)h * RF + 3 * P * DS_PITCH + c] = v;
  }
}

// grid (value-column slices, heads, rows)
__global__ void __launch_bounds__(DS_THREADS) delta_scan_kernel(DeltaParams p) {
  pdl_wait();                      // programmatic dependent launch: nothing is read before the predecessor is done
  pdl_launch_dependents();
  extern __shared__ float4 smem4[];
  float* smem = reinterpret_cast<float*>(smem4);
  const int P = p.P, cols = DS_THREADS / P;
  const int tid = threadIdx.x, part = tid % P, lcol = tid / P, col = blockIdx.x * cols + lcol;
  const int h = blockIdx.y, b = blockIdx.z;
  const int QKA = 3 * P * DS_PITCH, dvp = (p.Dv + 3) & ~3, RF = delta_record_floats(P, p.Dv);
  const int SF = QKA + cols + 4;                                // floats per staged token: q | k | a, this CTA's values, beta, q·k
  float st[DS_DP];
  const int d0 = part * DS_DP;
  float* sbase = p.state + (((size_t)b * p.H + h) * p.D) * p.Dv;
#pragma unroll
  for (int r = 0; r < DS_DP; ++r) st[r] = (col < p.Dv && d0 + r < p.D) ? sbase[(size_t)(d0 + r) * p.Dv + col] : 0.0f;
  const int first = max(0, (p.pad_left ? p.pad_left[b] : 0) - (p.cache_len ? *p.cache_len : 0));
  if (part == 0 && col < p.Dv)
    for (int s = 0; s < min(first, p.S); ++s) p.o[((size_t)(b * p.S + s) * p.H + h) * p.Dv + col] = 0.0f;
  for (int s0 = first; s0 < p.S; s0 += DS_TC) {
    const int nt = min(DS_TC, p.S - s0);
    __syncthreads();
    for (int i = tid; i < nt * (QKA / 4); i += DS_THREADS) {
      const int t = i / (QKA / 4), c = i % (QKA / 4);
      const float* src = p.rec + ((size_t)(b * p.S + s0 + t) * p.H + h) * RF;
      reinterpret_cast<float4*>(smem + t * SF)[c] = reinterpret_cast<const float4*>(src)[c];
    }
    for (int i = tid; i < nt * (cols + 4); i += DS_THREADS) {
      const int t = i / (cols + 4), c = i % (cols + 4);
      const float* src = p.rec + ((size_t)(b * p.S + s0 + t) * p.H + h) * RF + QKA;
      float v = 0.0f;
      if (c < cols) { const int gc = blockIdx.x * cols + c; if (gc < p.Dv) v = src[gc]; }
      else v = src[dvp + (c - cols)];
      smem[t * SF + QKA + c] = v;
    }
    __syncthreads();
    for (int t = 0; t < nt; ++t) {
      const float* tk = smem + t * SF;
      const float v = tk[QKA + lcol], beta = tk[QKA + cols], qk = tk[QKA + cols + 1];
      const float4* qt = reinterpret_cast<const float4*>(tk + part * DS_PITCH);
      const float4* kt = reinterpret_cast<const float4*>(tk + (P + part) * DS_PITCH);
      const float4* at = reinterpret_cast<const float4*>(tk + (2 * P + part) * DS_PITCH);
      float ks0 = 0.0f, ks1 = 0.0f, qs0 = 0.0f, qs1 = 0.0f;
#pragma unroll
      for (int r = 0; r < DS_DP / 4; ++r) {
        const float4 al = at[r], kk = kt[r], qq = qt[r];
        st[4 * r + 0] *= al.x; ks0 = fmaf(kk.x, st[4 * r + 0], ks0); qs0 = fmaf(qq.x, st[4 * r + 0], qs0);
        st[4 * r + 1] *= al.y; ks1 = fmaf(kk.y, st[4 * r + 1], ks1); qs1 = fmaf(qq.y, st[4 * r + 1], qs1);
        st[4 * r + 2] *= al.z; ks0 = fmaf(kk.z, st[4 * r + 2], ks0); qs0 = fmaf(qq.z, st[4 * r + 2], qs0);
        st[4 * r + 3] *= al.w; ks1 = fmaf(kk.w, st[4 * r + 3], ks1); qs1 = fmaf(qq.w, st[4 * r + 3], qs1);
      }
      float ks = ks0 + ks1, qs = qs0 + qs1;
      for (int off = P >> 1; off > 0; off >>= 1) {
        ks += __shfl_xor_sync(0xffffffffu, ks, off);
        qs += __shfl_xor_sync(0xffffffffu, qs, off);
      }
      const float e = beta * (v - ks);
#pragma unroll
      for (int r = 0; r < DS_DP / 4; ++r) {
        const float4 kk = kt[r];
        st[4 * r + 0] = fmaf(kk.x, e, st[4 * r + 0]);
        st[4 * r + 1] = fmaf(kk.y, e, st[4 * r + 1]);
        st[4 * r + 2] = fmaf(kk.z, e, st[4 * r + 2]);
        st[4 * r + 3] = fmaf(kk.w, e, st[4 * r + 3]);
      }
      if (part == 0 && col < p.Dv) p.o[((size_t)(b * p.S + s0 + t) * p.H + h) * p.Dv + col] = fmaf(qk, e, qs);
    }
  }
#pragma unroll
  for (int r = 0; r < DS_DP; ++r)
    if (col < p.Dv && d0 + r < p.D) sbase[(size_t)(d0 + r) * p.Dv + col] = st[r];
}

}  // namespace jl

using namespace jl;

static int delta_lanes(int D) {
  int P = 1;
  while (P * DS_DP < D) P *= 2;
  return P;
}

extern "C" JL_API size_t jl_delta_scan_ws_floats(int B, int S, int H, int D, int Dv) {
  return (size_t)B * S * H * delta_record_floats(delta_lanes(D), Dv);
}

extern "C" JL_API int jl_delta_scan(const float* u, int ldu, int q_off, int k_off, int v_off, int G, const float* y, int ldy,
                                    int b_off, int a_off, const void* a2, const void* a_bias, const void* a_log, float* state,
                                    float* o, const int* cache_len, const int* pad_left, int B, int S, int H, int D, int Dv, int R,
                                    float* ws, int dtype, void* stream) {
  JL_CHECK_ARG(B >= 1 && S >= 1 && H >= 1 && D >= 1 && Dv >= 1 && R >= 1 && ws != nullptr, "jl_delta_scan: bad shape");
  JL_CHECK_ARG(G >= 1 && H % G == 0, "jl_delta_scan: %d heads over %d q / k heads", H, G);
  const int P = delta_lanes(D);
  JL_CHECK_ARG(P <= 32, "jl_delta_scan: key size %d above %d", D, 32 * DS_DP);
  DeltaParams p{u, ldu, q_off, k_off, v_off, G, y, ldy, b_off, a_off, B, S, H, D, Dv, R, P, cache_len, pad_left, state, o, ws};
  const size_t smem1 = (size_t)(R + 3 * G) * sizeof(float);
  JL_CHECK_ARG(smem1 <= 48 * 1024, "jl_delta_scan: rank %d with %d q / k heads does not fit", R, G);
  JL_DISPATCH_DTYPE(dtype, JL_LAUNCH_PDL(delta_prep_kernel<T>, dim3(B * S), dim3(128), smem1, stream, p, (const T*)a2,
                                         (const T*)a_bias, (const T*)a_log));
  JL_CUDA(cudaGetLastError());
  const int cols = DS_THREADS / P;
  const size_t smem2 = (size_t)DS_TC * (3 * P * DS_PITCH + cols + 4) * sizeof(float);
  JL_CHECK_ARG(smem2 <= 200 * 1024, "jl_delta_scan: key size %d does not fit the staging buffer", D);
  if (smem2 > 48 * 1024) JL_CUDA(cudaFuncSetAttribute(delta_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2));
  JL_LAUNCH_PDL(delta_scan_kernel, dim3((Dv + cols - 1) / cols, H, B), dim3(DS_THREADS), smem2, stream, p);
  JL_CUDA(cudaGetLastError());
  return JL_OK;
}
