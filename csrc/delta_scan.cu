// Gated delta rule with one decay per key channel: per head a matrix state S [D x Dv] that every token first decays, then
// corrects towards its value along its key, then reads with its query:
//     S <- diag(a_t) S;   e_t = beta_t (v_t - S^T k_t);   S <- S + k_t e_t^T;   o_t = S^T q_t.
// The update is not a plain linear recurrence in S (the correction multiplies S by I - beta k k^T), so the tokens of a row
// run in order; the Dv columns of S are independent of one another and spread over threads and CTAs.
//
// Prompts take two launches.  delta_prep_kernel is token-parallel: unit-length q and k per head (q also times D^(-1/2)),
// their dot product, beta = sigmoid(.), and the decays a = exp(-exp(A_log_h) softplus(A2 z + bias)) from the rank-R input
// z — all fp32 — written as one record per (token, head) in the layout the scan stages in shared memory; the scan copies
// them with cp.async two stages deep.  A few tokens per row (decoding) take one launch: the scan forms its head's records
// itself.  delta_scan_kernel walks the tokens: a thread owns DP key channels of one value column in registers, the
// P = ceil(D / DP) lanes of a column are adjacent.  With c = a ⊙ s the two dot products k·c and q·c are formed in one pass and reduced together, and
// o = q·c + (q·k) e needs no second reduction; the second pass adds k e to the state.
#include "jllama_b200.h"
#include "seq_types.cuh"

namespace jl {

// Key channels per thread, DP: 8 for keys up to 256 channels, 32 above.  The walk over the tokens of a row is a chain of
// dependent instructions issued by few warps (one instruction every three cycles per warp, measured): what a token costs is
// the number of instructions a thread spends on it, so a column's channels are spread over more lanes (three shuffle levels
// at 64 channels) rather than kept in one thread.  A record holds q | k | a in rows of DP + 4 floats per lane: 16-byte rows,
// distinct banks for the lanes of a column.
constexpr int DS_TC = 32;            // tokens per pipeline stage (fewer when two stages of wide keys would not fit)
constexpr int DS_THREADS = 128;

__device__ __forceinline__ float delta_softplus(float z) { return z > 20.0f ? z : log1pf(expf(z)); }
__host__ __device__ inline int delta_record_floats(int P, int DP, int Dv) { return 3 * P * (DP + 4) + ((Dv + 3) & ~3) + 4; }

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

// The record of one (token, head), formed by a whole CTA: q | k | a in the scan's padded layout at dst, the value columns
// [v0, v0 + nv) at dst + v_at and beta, q·k at dst + s_at.  zs (R floats) and hs (3 floats) are shared-memory scratch.
template <typename T, int DP>
__device__ __forceinline__ void delta_record(const DeltaParams& p, size_t m, int h, const T* __restrict__ a2,
                                             const T* __restrict__ a_bias, const T* __restrict__ a_log, float* dst, int v0, int nv,
                                             int v_at, int s_at, float* zs, float* hs) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float* ur = p.u + m * p.ldu;
  const float* yr = p.y + m * p.ldy;
  const int g = h / (p.H / p.G);
  __syncthreads();                                       // scratch of the previous record is no longer read
  for (int r = threadIdx.x; r < p.R; r += blockDim.x) zs[r] = yr[p.a_off + r];
  if (warp == 0) {
    const float* q = ur + p.q_off + g * p.D;
    const float* k = ur + p.k_off + g * p.D;
    float qq = 0.0f, kk = 0.0f, qk = 0.0f;
    for (int d = lane; d < p.D; d += 32) { qq = fmaf(q[d], q[d], qq); kk = fmaf(k[d], k[d], kk); qk = fmaf(q[d], k[d], qk); }
    qq = warp_sum(qq); kk = warp_sum(kk); qk = warp_sum(qk);
    if (lane == 0) {
      const float rq = 1.0f / sqrtf(qq + 1e-6f) / sqrtf((float)p.D), rk = 1.0f / sqrtf(kk + 1e-6f);
      hs[0] = rq; hs[1] = rk; hs[2] = qk * rq * rk;
    }
  }
  __syncthreads();
  constexpr int PITCH = DP + 4;
  const int P = p.P, chans = P * DP;
  const float decay_rate = -expf(to_f(a_log[h]));
  for (int d = threadIdx.x; d < chans; d += blockDim.x) {
    float qv = 0.0f, kv = 0.0f, av = 1.0f;
    if (d < p.D) {
      qv = ur[p.q_off + g * p.D + d] * hs[0];
      kv = ur[p.k_off + g * p.D + d] * hs[1];
      const int n = h * p.D + d;
      float z = to_f(a_bias[n]);
      for (int r = 0; r < p.R; ++r) z = fmaf(to_f(a2[(size_t)n * p.R + r]), zs[r], z);
      av = expf(decay_rate * delta_softplus(z));
    }
    float* o = dst + (d / DP) * PITCH + d % DP;
    o[0] = qv; o[P * PITCH] = kv; o[2 * P * PITCH] = av;
  }
  for (int c = threadIdx.x; c < nv; c += blockDim.x) dst[v_at + c] = v0 + c < p.Dv ? ur[p.v_off + h * p.Dv + v0 + c] : 0.0f;
  if (threadIdx.x == 0) { dst[s_at] = sigmoid_f(yr[p.b_off + h]); dst[s_at + 1] = hs[2]; dst[s_at + 2] = 0.0f; dst[s_at + 3] = 0.0f; }
}

// grid (heads, tokens): one record each
template <typename T, int DP>
__global__ void __launch_bounds__(128) delta_prep_kernel(DeltaParams p, const T* __restrict__ a2, const T* __restrict__ a_bias,
                                                         const T* __restrict__ a_log) {
  pdl_wait();                      // programmatic dependent launch: nothing is read before the predecessor is done
  pdl_launch_dependents();
  extern __shared__ float sm[];                                // [R] decay input | 3 scalars
  const int h = blockIdx.x;
  const size_t m = blockIdx.y;
  const int dvp = (p.Dv + 3) & ~3, RF = delta_record_floats(p.P, DP, p.Dv), QKA = 3 * p.P * (DP + 4);
  delta_record<T, DP>(p, m, h, a2, a_bias, a_log, p.rec + (m * p.H + h) * RF, 0, dvp, QKA, QKA + dvp, sm, sm + p.R);
}

__device__ __forceinline__ void ds_cp_async16(void* smem_dst, const void* gsrc) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void ds_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void ds_cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// grid (value-column slices, heads, rows).  FUSED (a few tokens per row: decoding): the CTA forms its head's records itself
// in shared memory, one launch; otherwise the records of `tc` tokens per stage are copied with cp.async, two stages deep,
// so that the copy of the next tokens runs under the arithmetic of the current ones.
template <typename T, int DP, bool FUSED>
__global__ void __launch_bounds__(DS_THREADS) delta_scan_kernel(DeltaParams p, int tc, const T* __restrict__ a2,
                                                                const T* __restrict__ a_bias, const T* __restrict__ a_log) {
  pdl_wait();                      // programmatic dependent launch: nothing is read before the predecessor is done
  pdl_launch_dependents();
  extern __shared__ float4 smem4[];
  float* smem = reinterpret_cast<float*>(smem4);
  const int P = p.P, NT = blockDim.x, cols = NT / P;            // NT: 32, 64 or 128 threads, chosen by the host
  const int tid = threadIdx.x, part = tid % P, lcol = tid / P, col = blockIdx.x * cols + lcol;
  const int h = blockIdx.y, b = blockIdx.z;
  constexpr int PITCH = DP + 4;
  const int QKA = 3 * P * PITCH, dvp = (p.Dv + 3) & ~3, RF = delta_record_floats(P, DP, p.Dv);
  const int SF = QKA + cols + 4;                                // floats per staged token: q | k | a, this CTA's values, beta, q·k
  float st[DP];
  const int d0 = part * DP;
  float* sbase = p.state + (((size_t)b * p.H + h) * p.D) * p.Dv;
#pragma unroll
  for (int r = 0; r < DP; ++r) st[r] = (col < p.Dv && d0 + r < p.D) ? sbase[(size_t)(d0 + r) * p.Dv + col] : 0.0f;
  const int first = max(0, (p.pad_left ? p.pad_left[b] : 0) - (p.cache_len ? *p.cache_len : 0));
  if (part == 0 && col < p.Dv)
    for (int s = 0; s < min(first, p.S); ++s) p.o[((size_t)(b * p.S + s) * p.H + h) * p.Dv + col] = 0.0f;
  auto issue = [&](int s0, int stage) {
    const int nt = min(tc, p.S - s0), per = QKA / 4 + cols / 4 + 1;
    float* dst = smem + (size_t)stage * tc * SF;
    const float* src = p.rec + ((size_t)(b * p.S + s0) * p.H + h) * RF;
    for (int t = 0; t < nt; ++t, dst += SF, src += (size_t)p.H * RF)
      for (int c = tid; c < per; c += NT) {
        if (c < QKA / 4) ds_cp_async16(dst + 4 * c, src + 4 * c);
        else if (c < per - 1) {
          const int vc = (int)(blockIdx.x * cols) + 4 * (c - QKA / 4);
          if (vc < dvp) ds_cp_async16(dst + QKA + 4 * (c - QKA / 4), src + QKA + vc);
        } else ds_cp_async16(dst + QKA + cols, src + QKA + dvp);
      }
    ds_cp_async_commit();
  };
  int stage = 0;
  if (!FUSED && first < p.S) issue(first, 0);
  for (int s0 = first; s0 < p.S; s0 += tc, stage ^= 1) {
    const int nt = min(tc, p.S - s0);
    if (FUSED) {
      float* scratch = smem + (size_t)tc * SF;                  // [R + 3] behind the single stage
      for (int t = 0; t < nt; ++t)
        delta_record<T, DP>(p, (size_t)(b * p.S + s0 + t), h, a2, a_bias, a_log, smem + t * SF, blockIdx.x * cols, cols, QKA, QKA + cols,
                        scratch, scratch + p.R);
      stage = 0;
    } else if (s0 + tc < p.S) { issue(s0 + tc, stage ^ 1); ds_cp_async_wait<1>(); } else { ds_cp_async_wait<0>(); }
    __syncthreads();
    const float* base = smem + (size_t)stage * tc * SF;
    for (int t = 0; t < nt; ++t) {
      const float* tk = base + t * SF;
      const float v = tk[QKA + lcol], beta = tk[QKA + cols], qk = tk[QKA + cols + 1];
      const float4* qt = reinterpret_cast<const float4*>(tk + part * PITCH);
      const float4* kt = reinterpret_cast<const float4*>(tk + (P + part) * PITCH);
      const float4* at = reinterpret_cast<const float4*>(tk + (2 * P + part) * PITCH);
      float ks0 = 0.0f, ks1 = 0.0f, qs0 = 0.0f, qs1 = 0.0f;
#pragma unroll
      for (int r = 0; r < DP / 4; ++r) {
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
      for (int r = 0; r < DP / 4; ++r) {
        const float4 kk = kt[r];
        st[4 * r + 0] = fmaf(kk.x, e, st[4 * r + 0]);
        st[4 * r + 1] = fmaf(kk.y, e, st[4 * r + 1]);
        st[4 * r + 2] = fmaf(kk.z, e, st[4 * r + 2]);
        st[4 * r + 3] = fmaf(kk.w, e, st[4 * r + 3]);
      }
      if (part == 0 && col < p.Dv) p.o[((size_t)(b * p.S + s0 + t) * p.H + h) * p.Dv + col] = fmaf(qk, e, qs);
    }
    __syncthreads();                                            // the stage is free for the copy after next
  }
#pragma unroll
  for (int r = 0; r < DP; ++r)
    if (col < p.Dv && d0 + r < p.D) sbase[(size_t)(d0 + r) * p.Dv + col] = st[r];
}

}  // namespace jl

using namespace jl;

// DP: 8 channels per thread while that leaves the GPU short of eight warps per SM (the walk is bound by the latency of one
// token: measured 0.99 against 1.26 ms for 2048 tokens x 16 heads of 64 x 128), 32 when rows and heads fill it anyway (there
// the extra shuffle levels only add instructions: 8 rows of the same shape 112 against 103 ms per prompt batch).
static int delta_channels(int B, int H, int D, int Dv) {
  if (D > 256) return 32;
  int P = 1;
  while (P * 8 < D) P *= 2;
  return (long)B * H * Dv * P / 32 >= 148 * 8 ? 32 : 8;
}
static int delta_lanes(int D, int DP) {
  int P = 1;
  while (P * DP < D) P *= 2;
  return P;
}

extern "C" JL_API size_t jl_delta_scan_ws_floats(int B, int S, int H, int D, int Dv) {
  const int DP = delta_channels(B, H, D, Dv);
  return (size_t)B * S * H * delta_record_floats(delta_lanes(D, DP), DP, Dv);
}

constexpr int DS_FUSED_MAX_TOKENS = 8;      // up to this many tokens per row the records are formed inside the scan (one launch)

template <typename T, int DP>
static int delta_launch(DeltaParams p, const void* a2, const void* a_bias, const void* a_log, void* stream) {
  const int P = p.P, S = p.S, R = p.R;
  // Threads per CTA: while the grid is short of one CTA per SM the value columns are spread over more, smaller CTAs; the
  // value part of a stage needs at least four columns per CTA (16-byte copies).
  int NT = DS_THREADS;
  while (NT / 2 >= 32 && NT / 2 >= 4 * P && (long)((p.Dv + NT / P - 1) / (NT / P)) * p.H * p.B < 148) NT /= 2;
  const int cols = NT / P, SF = 3 * P * (DP + 4) + cols + 4;
  dim3 grid((p.Dv + cols - 1) / cols, p.H, p.B);
  if (S <= DS_FUSED_MAX_TOKENS) {
    const size_t smem = (size_t)(S * SF + R + 4) * sizeof(float);
    JL_CHECK_ARG(smem <= 200 * 1024, "jl_delta_scan: key size %d with rank %d does not fit the staging buffer", p.D, R);
    if (smem > 48 * 1024)
      JL_CUDA(cudaFuncSetAttribute(delta_scan_kernel<T, DP, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    JL_LAUNCH_PDL((delta_scan_kernel<T, DP, true>), dim3(grid), dim3(NT), smem, stream, p, S, (const T*)a2, (const T*)a_bias,
                  (const T*)a_log);
    JL_CUDA(cudaGetLastError());
    return JL_OK;
  }
  JL_CHECK_ARG(p.rec != nullptr, "jl_delta_scan: %d tokens per row need the record workspace", S);
  JL_CHECK_ARG(cols >= 4, "jl_delta_scan: key size %d leaves %d value columns per CTA", p.D, cols);
  const size_t smem1 = (size_t)(R + 4) * sizeof(float);
  JL_CHECK_ARG(smem1 <= 48 * 1024, "jl_delta_scan: rank %d does not fit", R);
  JL_LAUNCH_PDL((delta_prep_kernel<T, DP>), dim3(p.H, p.B * S), dim3(128), smem1, stream, p, (const T*)a2, (const T*)a_bias,
                (const T*)a_log);
  JL_CUDA(cudaGetLastError());
  int tc = DS_TC;                                               // tokens per pipeline stage: two stages have to fit
  while (tc > 1 && (size_t)2 * tc * SF * sizeof(float) > 160 * 1024) tc /= 2;
  const size_t smem2 = (size_t)2 * tc * SF * sizeof(float);
  JL_CHECK_ARG(smem2 <= 200 * 1024, "jl_delta_scan: key size %d does not fit the pipeline stages", p.D);
  if (smem2 > 48 * 1024)
    JL_CUDA(cudaFuncSetAttribute(delta_scan_kernel<T, DP, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2));
  JL_LAUNCH_PDL((delta_scan_kernel<T, DP, false>), dim3(grid), dim3(NT), smem2, stream, p, tc, (const T*)a2, (const T*)a_bias,
                (const T*)a_log);
  JL_CUDA(cudaGetLastError());
  return JL_OK;
}

extern "C" JL_API int jl_delta_scan(const float* u, int ldu, int q_off, int k_off, int v_off, int G, const float* y, int ldy,
                                    int b_off, int a_off, const void* a2, const void* a_bias, const void* a_log, float* state,
                                    float* o, const int* cache_len, const int* pad_left, int B, int S, int H, int D, int Dv, int R,
                                    float* ws, int dtype, void* stream) {
  JL_CHECK_ARG(B >= 1 && S >= 1 && H >= 1 && D >= 1 && Dv >= 1 && R >= 1, "jl_delta_scan: bad shape");
  JL_CHECK_ARG(G >= 1 && H % G == 0, "jl_delta_scan: %d heads over %d q / k heads", H, G);
  const int DP = delta_channels(B, H, D, Dv), P = delta_lanes(D, DP);
  JL_CHECK_ARG(P <= 32, "jl_delta_scan: key size %d above 1024", D);
  DeltaParams p{u, ldu, q_off, k_off, v_off, G, y, ldy, b_off, a_off, B, S, H, D, Dv, R, P, cache_len, pad_left, state, o, ws};
  if (DP == 8) JL_DISPATCH_DTYPE(dtype, return (delta_launch<T, 8>(p, a2, a_bias, a_log, stream)));
  JL_DISPATCH_DTYPE(dtype, return (delta_launch<T, 32>(p, a2, a_bias, a_log, stream)));
  return JL_OK;
}
