// Linear layers for any shape and for bfloat16 or true float32 operands: y = act(x W^T) with W [N, K] (out, in).
//
//  * linear_rows_kernel  (M <= 8: decode)  — weight-streaming: a CTA owns ROWS output features, its 8 warps split K, each
//    lane reads 16 bytes of every row per step (all loads issued before the first use) and keeps ROWS x M fp32
//    accumulators; activations come from L1; the warps' sums meet in shared memory in a fixed order.
//  * linear_tiled_kernel (any M)           — 64 x 64 x 16 shared-memory tiles, 4 x 4 outputs per thread, fp32 FMA.  This is
//    the exact float32 path and the fall-back for pitches the tensor-core GEMM does not take.
//
// Products and sums are fp32 (fmaf), never TF32.  The output is fp32 or the operand type, written at a column offset
// of a wider row (ldo) so that projections that share an input can share an output buffer.
#include "jllama_b200.h"
#include "seq_types.cuh"

namespace jl {

// Many small products in one launch.  Plain batches: batch z reads x + (z / x_div) * x_bs, weights
// w + (w_index ? w_index[z] : z) * w_bs (w_index[z] < 0: the batch is skipped) and writes out + z * o_bs (per-head matrices; one expert per (token, choice) pair when
// decoding a mixture of experts: x_div = choices per token, so that the pairs of a token read the same input row).
// Sorted rows (tiled kernel only): the rows come in tiles of LT_BM that each belong to one weight matrix, tile_group[tile]
// (< 0: empty tile); row position p reads input row row_src[p] (< 0: padding, read as zero; nullptr: p itself) and writes
// output row p — the prompt path of a mixture of experts after its tokens were sorted by expert.
struct LinearGroup {
  long long x_bs, w_bs, o_bs;
  int x_div;
  const int* w_index;
  const int* tile_group;
  const int* row_src;
};

constexpr int LR_ROWS = 4;      // output features per warp
constexpr int LR_MAXM = 8;

template <typename T> struct Vec;                    // 16-byte vector of T
template <> struct Vec<float> { static constexpr int N = 4; };
template <> struct Vec<__nv_bfloat16> { static constexpr int N = 8; };

template <typename T> __device__ __forceinline__ void load_vec(const T* p, float (&v)[Vec<T>::N]);
template <> __device__ __forceinline__ void load_vec<float>(const float* p, float (&v)[4]) {
  float4 t = *reinterpret_cast<const float4*>(p);
  v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
template <> __device__ __forceinline__ void load_vec<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  uint4 t = *reinterpret_cast<const uint4*>(p);
  v[0] = bf16_lo(t.x); v[1] = bf16_hi(t.x); v[2] = bf16_lo(t.y); v[3] = bf16_hi(t.y);
  v[4] = bf16_lo(t.z); v[5] = bf16_hi(t.z); v[6] = bf16_lo(t.w); v[7] = bf16_hi(t.w);
}

constexpr int LR_WARPS = 8;     // warps of a CTA: they split K for the same LR_ROWS output features

template <typename T, typename OutT, int M>
__global__ void __launch_bounds__(LR_WARPS * 32) linear_rows_kernel(const T* __restrict__ x, int ldx, const T* __restrict__ w,
                                                                    OutT* __restrict__ out, int ldo, int N, int K, int act,
                                                                    float p0, float p1, int vec_ok, LinearGroup g) {
  pdl_wait();                      // programmatic dependent launch: nothing is read before the predecessor is done
  pdl_launch_dependents();
  __shared__ float red[LR_WARPS][LR_ROWS][M];
  if (g.w_index && g.w_index[blockIdx.y] < 0) return;            // a batch without a matrix (uniform for the CTA): nothing is written
  {
    const long long z = blockIdx.y;
    x += (z / g.x_div) * g.x_bs;
    w += (g.w_index ? (long long)g.w_index[z] : z) * g.w_bs;
    out += z * g.o_bs;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n0 = blockIdx.x * LR_ROWS;
  float acc[LR_ROWS][M];
#pragma unroll
  for (int r = 0; r < LR_ROWS; ++r)
#pragma unroll
    for (int m = 0; m < M; ++m) acc[r][m] = 0.0f;
  constexpr int VN = Vec<T>::N;
  int k_done = 0;
  if (vec_ok) {
    const int kv = K / VN * VN;
    for (int k = (warp * 32 + lane) * VN; k < kv; k += LR_WARPS * 32 * VN) {
      float wv[LR_ROWS][VN];
#pragma unroll
      for (int r = 0; r < LR_ROWS; ++r) {          // all weight loads of this step are in flight before any is used
        const int n = min(n0 + r, N - 1);
        load_vec<T>(w + (size_t)n * K + k, wv[r]);
      }
#pragma unroll
      for (int m = 0; m < M; ++m) {
        float xv[VN];
        load_vec<T>(x + (size_t)m * ldx + k, xv);
#pragma unroll
        for (int r = 0; r < LR_ROWS; ++r)
#pragma unroll
          for (int j = 0; j < VN; ++j) acc[r][m] = fmaf(wv[r][j], xv[j], acc[r][m]);
      }
    }
    k_done = kv;
  }
  for (int k = k_done + warp * 32 + lane; k < K; k += LR_WARPS * 32) {
#pragma unroll
    for (int r = 0; r < LR_ROWS; ++r) {
      const float wv = to_f(w[(size_t)min(n0 + r, N - 1) * K + k]);
#pragma unroll
      for (int m = 0; m < M; ++m) acc[r][m] = fmaf(wv, to_f(x[(size_t)m * ldx + k]), acc[r][m]);
    }
  }
#pragma unroll
  for (int r = 0; r < LR_ROWS; ++r)
#pragma unroll
    for (int m = 0; m < M; ++m) {
      const float s = warp_sum(acc[r][m]);
      if (lane == 0) red[warp][r][m] = s;
    }
  __syncthreads();
  if (threadIdx.x < LR_ROWS * M) {
    const int r = threadIdx.x / M, m = threadIdx.x % M;
    float s = 0.0f;
#pragma unroll
    for (int wq = 0; wq < LR_WARPS; ++wq) s += red[wq][r][m];
    if (n0 + r < N) out[(size_t)m * ldo + n0 + r] = from_f<OutT>(apply_act(s, act, p0, p1));
  }
}

constexpr int LT_BM = 64, LT_BN = 64, LT_BK = 16;

template <typename T, typename OutT>
__global__ void __launch_bounds__(256) linear_tiled_kernel(const T* __restrict__ x, int ldx, const T* __restrict__ w,
                                                           OutT* __restrict__ out, int ldo, int M, int N, int K, int act,
                                                           float p0, float p1, LinearGroup g) {
  pdl_wait();                      // programmatic dependent launch: nothing is read before the predecessor is done
  pdl_launch_dependents();
  __shared__ float xs[LT_BK][LT_BM + 4];
  __shared__ float ws[LT_BK][LT_BN + 4];
  __shared__ int srow[LT_BM];
  const int m0 = blockIdx.y * LT_BM, n0 = blockIdx.x * LT_BN;
  if (g.tile_group) {
    const int e = g.tile_group[blockIdx.y];
    if (e < 0) return;                                             // uniform for the CTA
    w += (long long)e * g.w_bs;
  } else {
    const long long z = blockIdx.z;
    if (g.w_index && g.w_index[z] < 0) return;                     // a batch without a matrix (uniform for the CTA)
    x += (z / g.x_div) * g.x_bs;
    w += (g.w_index ? (long long)g.w_index[z] : z) * g.w_bs;
    out += z * g.o_bs;
  }
  if (threadIdx.x < LT_BM) {
    const int gm = m0 + threadIdx.x;
    srow[threadIdx.x] = gm < M ? ((g.tile_group && g.row_src) ? g.row_src[gm] : gm) : -1;
  }
  __syncthreads();
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;         // 16 x 16 threads, 4 x 4 outputs each
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += LT_BK) {
    for (int i = threadIdx.x; i < LT_BM * LT_BK; i += 256) {
      const int r = i / LT_BK, c = i % LT_BK;
      const int gn = n0 + r, gk = k0 + c;
      xs[c][r] = (srow[r] >= 0 && gk < K) ? to_f(x[(size_t)srow[r] * ldx + gk]) : 0.0f;
      ws[c][r] = (gn < N && gk < K) ? to_f(w[(size_t)gn * K + gk]) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int c = 0; c < LT_BK; ++c) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { a[i] = xs[c][ty * 4 + i]; b[i] = ws[c][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn < N) out[(size_t)gm * ldo + gn] = from_f<OutT>(apply_act(acc[i][j], act, p0, p1));
    }
  }
}

template <typename T, typename OutT>
static int launch_linear(const void* x, int ldx, const void* w, void* out, int ldo, int M, int N, int K, int act, float p0,
                         float p1, cudaStream_t st, LinearGroup g = LinearGroup{0, 0, 0, 1, nullptr, nullptr, nullptr}, int nbatch = 1) {
  if (M <= LR_MAXM && g.tile_group == nullptr) {
    constexpr int VN = Vec<T>::N;
    const int vec_ok = (K % VN == 0) && (ldx % VN == 0) && ((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0) &&
                       (g.x_bs % VN == 0) && (g.w_bs % VN == 0);
    const dim3 blocks((N + LR_ROWS - 1) / LR_ROWS, nbatch);
#define JL_LR(MM)                                                                                                       \
  case MM:                                                                                                              \
    JL_LAUNCH_PDL((linear_rows_kernel<T, OutT, MM>), dim3(blocks), dim3(LR_WARPS * 32), 0, st, (const T*)x, ldx, (const T*)w, (OutT*)out, ldo, N, K, act, \
                                                                   p0, p1, vec_ok, g);                                  \
    break;
    switch (M) { JL_LR(1) JL_LR(2) JL_LR(3) JL_LR(4) JL_LR(5) JL_LR(6) JL_LR(7) JL_LR(8) }
#undef JL_LR
  } else {
    dim3 grid((N + LT_BN - 1) / LT_BN, (M + LT_BM - 1) / LT_BM, g.tile_group ? 1 : nbatch);
    JL_LAUNCH_PDL((linear_tiled_kernel<T, OutT>), dim3(grid), dim3(256), 0, st, (const T*)x, ldx, (const T*)w, (OutT*)out, ldo, M, N, K, act, p0, p1, g);
  }
  return cudaGetLastError() == cudaSuccess ? JL_OK : JL_ERR_CUDA;
}

}  // namespace jl

using namespace jl;

extern "C" JL_API int jl_linear_any(const void* x, int ldx, const void* w, void* out, int ldo, int M, int N, int K, int act,
                                    float p0, float p1, int dtype, int out_f32, void* stream) {
  JL_CHECK_ARG(M >= 1 && N >= 1 && K >= 1 && ldx >= K && ldo >= N, "jl_linear_any: bad shape M=%d N=%d K=%d ldx=%d ldo=%d", M, N,
               K, ldx, ldo);
  JL_CHECK_ARG(act >= 0 && act <= ACT_LAST, "jl_linear_any: bad activation %d", act);
  cudaStream_t st = (cudaStream_t)stream;
  int rc;
  if (dtype == DT_BF16)
    rc = out_f32 ? launch_linear<__nv_bfloat16, float>(x, ldx, w, out, ldo, M, N, K, act, p0, p1, st)
                 : launch_linear<__nv_bfloat16, __nv_bfloat16>(x, ldx, w, out, ldo, M, N, K, act, p0, p1, st);
  else
    rc = launch_linear<float, float>(x, ldx, w, out, ldo, M, N, K, act, p0, p1, st);
  if (rc != JL_OK) return cuda_fail(cudaGetLastError(), "jl_linear_any launch");
  return JL_OK;
}

extern "C" JL_API int jl_linear_tile_rows(void) { return LT_BM; }

extern "C" JL_API int jl_linear_grouped(const void* x, int ldx, long long x_bs, const void* w, long long w_bs, void* out, int ldo,
                                        long long o_bs, int nbatch, int x_div, int M, int N, int K, int act, float p0,
                                        float p1, const int* w_index, const int* tile_group, const int* row_src, int dtype, int out_f32,
                                        void* stream) {
  JL_CHECK_ARG(M >= 1 && N >= 1 && K >= 1 && ldx >= K && ldo >= N && nbatch >= 1 && x_div >= 1, "jl_linear_grouped: bad shape M=%d N=%d K=%d ldx=%d ldo=%d",
               M, N, K, ldx, ldo);
  JL_CHECK_ARG(act >= 0 && act <= ACT_LAST, "jl_linear_grouped: bad activation %d", act);
  JL_CHECK_ARG(tile_group == nullptr || M % LT_BM == 0, "jl_linear_grouped: sorted rows come in tiles of %d, M=%d", LT_BM, M);
  JL_CHECK_ARG(nbatch <= 65535, "jl_linear_grouped: %d batches above the grid limit", nbatch);
  cudaStream_t st = (cudaStream_t)stream;
  const LinearGroup g{x_bs, w_bs, o_bs, x_div, w_index, tile_group, row_src};
  int rc;
  if (dtype == DT_BF16)
    rc = out_f32 ? launch_linear<__nv_bfloat16, float>(x, ldx, w, out, ldo, M, N, K, act, p0, p1, st, g, nbatch)
                 : launch_linear<__nv_bfloat16, __nv_bfloat16>(x, ldx, w, out, ldo, M, N, K, act, p0, p1, st, g, nbatch);
  else
    rc = launch_linear<float, float>(x, ldx, w, out, ldo, M, N, K, act, p0, p1, st, g, nbatch);
  if (rc != JL_OK) return cuda_fail(cudaGetLastError(), "jl_linear_grouped launch");
  return JL_OK;
}
