// Gated linear attention: the per-head matrix state S [D x Dv] with one decay per key channel,
//     S_t = diag(alpha_t) S_(t-1) + k_t v_t^T,     o_t = S_t^T q_t,
// advanced token by token in fp32, for prompts (S tokens per row) and for decoding (S = 1) alike.
//
// The decay comes from a low-rank projection: z = A2 (A1 h) + bias, alpha = sigmoid(z)^(1/tau) = exp(logsigmoid(z) / tau).
// The rank-R product A1 h arrives as R fp32 columns of the fused projection buffer; the A2 product, the bias, the
// log-sigmoid and the exponential are done here in fp32 for a chunk of tokens at a time.
//
// Work split: grid (value-column slices, heads, batch rows); a thread owns GS_DP = 32 key channels of one value column of
// the state in registers, P = ceil(D / 32) (rounded to a power of two) adjacent lanes share a column and add their
// partial o with shuffles.  q, k and alpha of a chunk of tokens are staged in shared memory, one row of 36 floats per
// 32 channels (16-byte loads; the P lanes of a column read different banks).  Padding tokens (slot < pad_left[b]) are skipped:
// the state of a left-padded row starts at its first real token.
#include <stdlib.h>

#include "jllama_b200.h"
#include "seq_types.cuh"

namespace jl {

constexpr int GS_DP = 32;        // state rows per thread
constexpr int GS_TC = 8;         // tokens staged per chunk
constexpr int GS_THREADS = 128;
constexpr int GS_PITCH = GS_DP + 4;   // floats per 32 channels in shared memory: 16-byte aligned rows, distinct banks per lane group

__device__ __forceinline__ float log_sigmoid(float z) {
  return z >= 0.0f ? -log1pf(expf(-z)) : z - log1pf(expf(z));
}

struct GlaParams {
  const float* y; int ldy;
  int q_off, k_off, v_off, a_off;      // columns of y: q [H*D], k [H*D], v [H*Dv], low-rank decay input [R]
  int B, S, H, D, Dv, R, P;
  float q_scale, inv_tau;
  const int* cache_len; const int* pad_left;
  float* state;                        // [B][H][D][Dv] fp32, read and written
  float* o;                            // [B*S][H][Dv] fp32
  // time chunks of the prompt scan (gla_stream_kernel): NC chunks of L tokens per row
  int NC, L, mode;                     // mode 0: one chunk, state in / out; 1: local scan from zero, no read-out; 3: read-out pass
  float* cstate;                       // [B][NC][H][D][Dv]: local end states (after mode 1), incoming states (after the combine)
  float* cdecay;                       // [B][NC][H][D]: product of the chunk's decays per key channel
  // retention (jl_retention_scan): one fixed decay per head instead of the projected one, rotary embedding of q and k at the
  // token's position, k scaled after the rotation
  const float* head_decay;             // [H] fp32, or nullptr: alpha from the low-rank projection
  const float* cos_t; const float* sin_t; int rot, layout, max_pos;      // tables [max_pos][rot/2]; rot == 0: no rotation
  float k_scale;
  // state space scan (jl_ssd_scan): q / k are shared by the qk_div heads of a group; the decay of (token, head) is
  // aux[m * ld_aux + h] and the value row is scaled by aux[m * ld_aux + H + h]
  int qk_div;                          // heads per q / k head (1: every head has its own)
  const float* aux; int ld_aux;
};

__device__ __forceinline__ float scan_value_scale(const GlaParams& p, size_t m, int h) {
  return p.aux ? p.aux[m * p.ld_aux + p.H + h] : 1.0f;
}

// q, k and alpha of channel d of head h for the token whose projection row is yr (position pos).
template <typename T>
__device__ __forceinline__ void scan_channel(const GlaParams& p, size_t m, int h, int d, int pos,
                                             const float* __restrict__ zs, const T* __restrict__ a2, const T* __restrict__ a2b,
                                             float& qv, float& kv, float& av) {
  const float* yr = p.y + m * p.ldy;
  const int hq = p.qk_div > 1 ? h / p.qk_div : h;
  const float* qh = yr + p.q_off + hq * p.D;
  const float* kh = yr + p.k_off + hq * p.D;
  if (p.rot > 0) {
    const float* ct = p.cos_t + (size_t)pos * (p.rot / 2);
    const float* st = p.sin_t + (size_t)pos * (p.rot / 2);
    qv = rotary_channel(qh, d, p.rot, p.layout, ct, st) * p.q_scale;
    kv = rotary_channel(kh, d, p.rot, p.layout, ct, st) * p.k_scale;
  } else {
    qv = qh[d] * p.q_scale;
    kv = kh[d] * p.k_scale;
  }
  if (p.aux) { av = p.aux[m * p.ld_aux + h]; return; }
  if (p.head_decay) { av = p.head_decay[h]; return; }
  const int n = h * p.D + d;
  float z = to_f(a2b[n]);
  for (int r = 0; r < p.R; ++r) z = fmaf(to_f(a2[(size_t)n * p.R + r]), zs[r], z);
  av = expf(log_sigmoid(z) * p.inv_tau);
}

__device__ __forceinline__ int scan_position(const GlaParams& p, int b, int s) {
  if (p.rot <= 0) return 0;
  const int pos = (p.cache_len ? *p.cache_len : 0) + s - (p.pad_left ? p.pad_left[b] : 0);
  return pos < 0 ? 0 : (pos >= p.max_pos ? p.max_pos - 1 : pos);
}


template <typename T>
__global__ void __launch_bounds__(GS_THREADS, 3) gla_scan_kernel(GlaParams p, const T* __restrict__ a2, const T* __restrict__ a2b) {
  pdl_wait();                      // programmatic dependent launch: nothing is read before the predecessor is done
  pdl_launch_dependents();
  extern __shared__ float4 smem4[];
  float* smem = reinterpret_cast<float*>(smem4);
  const int P = p.P;                                         // lanes per value column (power of two, adjacent lanes of a warp)
  const int cols = GS_THREADS / P;                           // value columns per CTA
  const int tid = threadIdx.x;
  const int part = tid % P, lcol = tid / P, col = blockIdx.x * cols + lcol;
  const int h = blockIdx.y, b = blockIdx.z;
  const int DS = P * GS_PITCH;                               // padded channel pitch of one token's q / k / alpha
  float* qs = smem;                                          // [TC][DS]
  float* ks = qs + GS_TC * DS;
  float* as = ks + GS_TC * DS;
  float* vs = as + GS_TC * DS;                               // [TC][cols]
  float* zs = vs + GS_TC * cols;                             // [TC][R]

  float st[GS_DP];
  const int d0 = part * GS_DP;
  float* sbase = p.state + (((size_t)b * p.H + h) * p.D) * p.Dv;
#pragma unroll
  for (int r = 0; r < GS_DP; ++r) st[r] = (col < p.Dv && d0 + r < p.D) ? sbase[(size_t)(d0 + r) * p.Dv + col] : 0.0f;

  const int first = max(0, (p.pad_left ? p.pad_left[b] : 0) - (p.cache_len ? *p.cache_len : 0));   // first real token of this call
  if (part == 0 && col < p.Dv)                               // padding tokens: defined (zero) output rows
    for (int s = 0; s < min(first, p.S); ++s) p.o[((size_t)(b * p.S + s) * p.H + h) * p.Dv + col] = 0.0f;
  for (int s0 = first; s0 < p.S; s0 += GS_TC) {
    const int nt = min(GS_TC, p.S - s0);
    __syncthreads();
    for (int i = tid; i < nt * p.R; i += GS_THREADS) {
      const int t = i / p.R, r = i % p.R;
      zs[t * p.R + r] = p.y[(size_t)(b * p.S + s0 + t) * p.ldy + p.a_off + r];
    }
    for (int i = tid; i < nt * cols; i += GS_THREADS) {
      const int t = i / cols, c = blockIdx.x * cols + i % cols;
      const size_t mt = (size_t)(b * p.S + s0 + t);
      vs[i] = c < p.Dv ? p.y[mt * p.ldy + p.v_off + h * p.Dv + c] * scan_value_scale(p, mt, h) : 0.0f;
    }
    __syncthreads();
    for (int i = tid; i < nt * P * GS_DP; i += GS_THREADS) {
      const int t = i / (P * GS_DP), d = i % (P * GS_DP);
      const int at = t * DS + (d / GS_DP) * GS_PITCH + d % GS_DP;
      float qv = 0.0f, kv = 0.0f, av = 1.0f;
      if (d < p.D)
        scan_channel<T>(p, (size_t)(b * p.S + s0 + t), h, d, scan_position(p, b, s0 + t), zs + t * p.R, a2, a2b, qv, kv, av);
      qs[at] = qv; ks[at] = kv; as[at] = av;
    }
    __syncthreads();
    for (int t = 0; t < nt; ++t) {
      const float v = vs[t * cols + lcol];
      const float4* qt = reinterpret_cast<const float4*>(qs + t * DS + part * GS_PITCH);
      const float4* kt = reinterpret_cast<const float4*>(ks + t * DS + part * GS_PITCH);
      const float4* at = reinterpret_cast<const float4*>(as + t * DS + part * GS_PITCH);
      float a0 = 0.0f, a1 = 0.0f, a2v = 0.0f, a3 = 0.0f;
#pragma unroll
      for (int r = 0; r < GS_DP / 4; ++r) {
        const float4 al = at[r], kk = kt[r], qq = qt[r];
        st[4 * r + 0] = fmaf(al.x, st[4 * r + 0], kk.x * v); a0 = fmaf(qq.x, st[4 * r + 0], a0);
        st[4 * r + 1] = fmaf(al.y, st[4 * r + 1], kk.y * v); a1 = fmaf(qq.y, st[4 * r + 1], a1);
        st[4 * r + 2] = fmaf(al.z, st[4 * r + 2], kk.z * v); a2v = fmaf(qq.z, st[4 * r + 2], a2v);
        st[4 * r + 3] = fmaf(al.w, st[4 * r + 3], kk.w * v); a3 = fmaf(qq.w, st[4 * r + 3], a3);
      }
      float acc = (a0 + a1) + (a2v + a3);
      for (int off = P >> 1; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
      if (part == 0 && col < p.Dv) p.o[((size_t)(b * p.S + s0 + t) * p.H + h) * p.Dv + col] = acc;
    }
  }
#pragma unroll
  for (int r = 0; r < GS_DP; ++r)
    if (col < p.Dv && d0 + r < p.D) sbase[(size_t)(d0 + r) * p.Dv + col] = st[r];
}


// ---------------------------------------------------------------------------------------------------------------------
// Prompts: the same recurrence in two launches.  gla_prep_kernel is token-parallel: it forms alpha (low-rank product,
// bias, log-sigmoid, exponential — fp32), scales q, and writes q | k | alpha | v of every (token, head) as one
// contiguous fp32 record laid out exactly like the scan's shared-memory stage ([3][P][DP + 4] then the value row,
// padded to 16 bytes).  gla_stream_kernel then only copies records with cp.async, two stages deep (the copy of the next
// GS_TS tokens runs under the arithmetic of the current ones), and advances the state.  The fused kernel above pays two
// dependent DRAM round trips and the transcendental math per 8 tokens on the critical path of a sequential loop; here
// the loop sees shared memory only.
//
// A thread of the streaming kernel owns a DP x C tile of the state: DP key channels of C adjacent value columns.  The
// loop is bound by shared-memory reads of q, k and alpha (every thread needs them for its channels), so the tile is
// wide in columns (C = 4: the reads are shared by four columns) and short in channels (DP = 8), and the P = D / DP
// lanes of a column group add their partial read-outs with shuffles.  Key sizes above 256 take DP = 32, C = 1.
constexpr int GS_TS = 16;        // tokens per pipeline stage

struct GlaTile { int DP, C, P; };
static GlaTile gla_tile(int D) {
  // measured (2048 tokens, D 64, Dv 128): 0.80 ms with the 32 x 1 tile, 1.22 ms with 8 x 4 (its three shuffle levels per
  // token lengthen the dependent chain, and the loop is bound by latency, not by shared-memory bandwidth);
  // JLLAMA_GLA_TILE=8 selects the wide tile for A/B
  static const bool wide = [] { const char* e = getenv("JLLAMA_GLA_TILE"); return e && e[0] == '8'; }();
  GlaTile t{32, 1, 1};
  if (wide && D <= 256) t = GlaTile{8, 4, 1};
  while (t.P * t.DP < D) t.P *= 2;
  return t;
}
__host__ __device__ inline int gla_record_floats(int P, int DP, int Dv) { return 3 * P * (DP + 4) + ((Dv + 3) & ~3); }

template <typename T>
__global__ void __launch_bounds__(128) gla_prep_kernel(GlaParams p, const T* __restrict__ a2, const T* __restrict__ a2b,
                                                       float* __restrict__ rec, int DP) {
  pdl_wait();                      // programmatic dependent launch: nothing is read before the predecessor is done
  pdl_launch_dependents();
  extern __shared__ float zs[];                                 // [R]
  const int m = blockIdx.x;
  const float* yr = p.y + (size_t)m * p.ldy;
  const int pos = scan_position(p, m / p.S, m % p.S);
  for (int r = threadIdx.x; r < p.R; r += blockDim.x) zs[r] = yr[p.a_off + r];
  __syncthreads();
  const int P = p.P, pitch = DP + 4, RF = gla_record_floats(P, DP, p.Dv);
  float* out = rec + (size_t)m * p.H * RF;
  const int per_head = P * DP;
  for (int i = threadIdx.x; i < p.H * per_head; i += blockDim.x) {
    const int h = i / per_head, d = i % per_head;
    float qv = 0.0f, kv = 0.0f, av = 1.0f;
    if (d < p.D) scan_channel<T>(p, (size_t)m, h, d, pos, zs, a2, a2b, qv, kv, av);
    float* o = out + (size_t)h * RF + (d / DP) * pitch + d % DP;
    o[0] = qv; o[P * pitch] = kv; o[2 * P * pitch] = av;
  }
  const int dvp = (p.Dv + 3) & ~3;
  for (int i = threadIdx.x; i < p.H * dvp; i += blockDim.x) {
    const int h = i / dvp, c = i % dvp;
    out[(size_t)h * RF + 3 * P * pitch + c] = c < p.Dv ? yr[p.v_off + h * p.Dv + c] * scan_value_scale(p, (size_t)m, h) : 0.0f;
  }
}

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int DP, int C>
__global__ void __launch_bounds__(GS_THREADS, 2) gla_stream_kernel(GlaParams p, const float* __restrict__ rec) {
  pdl_wait();                      // programmatic dependent launch: nothing is read before the predecessor is done
  pdl_launch_dependents();
  extern __shared__ float4 smem4[];
  float* smem = reinterpret_cast<float*>(smem4);
  constexpr int PITCH = DP + 4;
  const int P = p.P, groups = GS_THREADS / P, cols = groups * C;        // value columns per CTA
  const int tid = threadIdx.x, part = tid % P, grp = tid / P;
  const int col0 = blockIdx.x * cols + grp * C;                         // first of this thread's C columns
  const int h = blockIdx.y, b = blockIdx.z / p.NC, chunk = blockIdx.z % p.NC;
  const int QKA = 3 * P * PITCH;                                        // floats of q | k | alpha per token
  const int SF = QKA + cols;                                            // floats per token in a stage
  const int RF = gla_record_floats(P, DP, p.Dv);
  float st[DP][C];
  const int d0 = part * DP;
  float* sbase = p.mode == 0 ? p.state + (((size_t)b * p.H + h) * p.D) * p.Dv
                             : p.cstate + ((((size_t)b * p.NC + chunk) * p.H + h) * p.D) * p.Dv;
  float ap[DP];                                                         // mode 1: product of this chunk's decays
#pragma unroll
  for (int r = 0; r < DP; ++r) {
    ap[r] = 1.0f;
#pragma unroll
    for (int c = 0; c < C; ++c)
      st[r][c] = (p.mode != 1 && col0 + c < p.Dv && d0 + r < p.D) ? sbase[(size_t)(d0 + r) * p.Dv + col0 + c] : 0.0f;
  }
  const int t_begin = chunk * p.L, t_end = min(p.S, t_begin + p.L);     // this CTA's tokens of row b
  const int first = max(t_begin, (p.pad_left ? p.pad_left[b] : 0) - (p.cache_len ? *p.cache_len : 0));
  if (part == 0 && p.mode != 1)
    for (int s = t_begin; s < min(first, t_end); ++s)
      for (int c = 0; c < C; ++c)
        if (col0 + c < p.Dv) p.o[((size_t)(b * p.S + s) * p.H + h) * p.Dv + col0 + c] = 0.0f;
  const int vcols4 = cols / 4, q4 = QKA / 4, dvp = (p.Dv + 3) & ~3;
  auto issue = [&](int s0, int stage) {
    const int nt = min(GS_TS, t_end - s0);
    float* dst = smem + (size_t)stage * GS_TS * SF;
    for (int i = tid; i < nt * (q4 + vcols4); i += GS_THREADS) {
      const int t = i / (q4 + vcols4), c = i % (q4 + vcols4);
      const float* src = rec + ((size_t)(b * p.S + s0 + t) * p.H + h) * RF;
      if (c < q4) cp_async16(dst + t * SF + 4 * c, src + 4 * c);
      else if ((int)(blockIdx.x * cols) + 4 * (c - q4) < dvp)
        cp_async16(dst + t * SF + QKA + 4 * (c - q4), src + QKA + blockIdx.x * cols + 4 * (c - q4));
    }
    cp_async_commit();
  };
  int stage = 0;
  if (first < t_end) issue(first, 0);
  for (int s0 = first; s0 < t_end; s0 += GS_TS, stage ^= 1) {
    if (s0 + GS_TS < t_end) { issue(s0 + GS_TS, stage ^ 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
    __syncthreads();
    const int nt = min(GS_TS, t_end - s0);
    const float* base = smem + (size_t)stage * GS_TS * SF;
    for (int t = 0; t < nt; ++t) {
      const float* tk = base + t * SF;
      float v[C];
      if constexpr (C == 4) {
        const float4 vv = *reinterpret_cast<const float4*>(tk + QKA + grp * C);
        v[0] = vv.x; v[1] = vv.y; v[2] = vv.z; v[3] = vv.w;
      } else {
#pragma unroll
        for (int c = 0; c < C; ++c) v[c] = tk[QKA + grp * C + c];
      }
      const float4* qt = reinterpret_cast<const float4*>(tk + part * PITCH);
      const float4* kt = reinterpret_cast<const float4*>(tk + (P + part) * PITCH);
      const float4* at = reinterpret_cast<const float4*>(tk + (2 * P + part) * PITCH);
      float acc[C][2];
#pragma unroll
      for (int c = 0; c < C; ++c) acc[c][0] = acc[c][1] = 0.0f;
#pragma unroll
      for (int r = 0; r < DP / 4; ++r) {
        const float4 al = at[r], kk = kt[r], qq = qt[r];
        const float a4[4] = {al.x, al.y, al.z, al.w}, k4[4] = {kk.x, kk.y, kk.z, kk.w}, q4v[4] = {qq.x, qq.y, qq.z, qq.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          ap[4 * r + j] *= a4[j];
#pragma unroll
          for (int c = 0; c < C; ++c) {
            st[4 * r + j][c] = fmaf(a4[j], st[4 * r + j][c], k4[j] * v[c]);
            acc[c][j & 1] = fmaf(q4v[j], st[4 * r + j][c], acc[c][j & 1]);
          }
        }
      }
      if (p.mode == 1) continue;                              // local scan: the read-outs come in the second pass
      float o[C];
#pragma unroll
      for (int c = 0; c < C; ++c) {
        o[c] = acc[c][0] + acc[c][1];
        for (int off = P >> 1; off > 0; off >>= 1) o[c] += __shfl_xor_sync(0xffffffffu, o[c], off);
      }
      if (part == 0) {
        float* dst = p.o + ((size_t)(b * p.S + s0 + t) * p.H + h) * p.Dv + col0;
        if (C == 4 && col0 + 3 < p.Dv && (p.Dv & 3) == 0) {
          *reinterpret_cast<float4*>(dst) = make_float4(o[0], o[1], o[2], o[3]);
        } else {
#pragma unroll
          for (int c = 0; c < C; ++c) if (col0 + c < p.Dv) dst[c] = o[c];
        }
      }
    }
    __syncthreads();                                          // the stage is free for the copy after next
  }
  if (p.mode == 3) return;
#pragma unroll
  for (int r = 0; r < DP; ++r) {
#pragma unroll
    for (int c = 0; c < C; ++c)
      if (col0 + c < p.Dv && d0 + r < p.D) sbase[(size_t)(d0 + r) * p.Dv + col0 + c] = st[r][c];
    if (p.mode == 1 && blockIdx.x == 0 && grp == 0 && d0 + r < p.D)
      p.cdecay[(((size_t)b * p.NC + chunk) * p.H + h) * p.D + d0 + r] = ap[r];
  }
}

// Between the two passes: walk the chunks of a row in order.  cstate[c] holds the chunk's local end state on entry and the
// state the chunk starts from on exit; the row's state is advanced to the end of the prompt.
__global__ void gla_combine_kernel(GlaParams p) {
  pdl_wait();                      // programmatic dependent launch: nothing is read before the predecessor is done
  pdl_launch_dependents();
  const size_t per_row = (size_t)p.H * p.D * p.Dv, total = (size_t)p.B * per_row;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t b = i / per_row, e = i % per_row, hd = e / p.Dv;           // hd = h * D + d
    float s = p.state[i];
    for (int c = 0; c < p.NC; ++c) {
      float* slot = p.cstate + ((size_t)b * p.NC + c) * per_row + e;
      const float local = *slot;
      *slot = s;
      s = fmaf(p.cdecay[((size_t)b * p.NC + c) * p.H * p.D + hd], s, local);
    }
    p.state[i] = s;
  }
}

}  // namespace jl

using namespace jl;

// Time chunks of a prompt scan.  One token costs a few hundred nanoseconds of dependent latency however many heads and
// rows run beside it (measured: 2048 tokens take 0.76 ms for 1 head and 0.94 ms for 64), so while the grid is short
// of one resident wave (two CTAs per SM) the prompt is cut into chunks that run side by side, in two passes.  Beyond
// a wave the second pass is pure cost (8 rows x 16 heads: 1.21 ms unchunked, 1.84 ms in 4 chunks).
static int gla_chunks(int B, int S, int H, int D, int Dv) {
  static const int forced = [] { const char* e = getenv("JLLAMA_GLA_CHUNKS"); return e ? atoi(e) : 0; }();
  const GlaTile t = gla_tile(D);
  const int tcols = GS_THREADS / t.P * t.C;
  const long ctas = (long)B * H * ((Dv + tcols - 1) / tcols);
  int nc = (int)(296 / (ctas > 0 ? ctas : 1));
  if (forced > 0) nc = forced;
  if (nc > S / 64) nc = S / 64;
  if (nc > 64) nc = 64;
  return nc < 2 ? 1 : nc;
}

extern "C" JL_API size_t jl_gla_scan_ws_floats(int B, int S, int H, int D, int Dv) {
  const GlaTile t = gla_tile(D);
  const int nc = gla_chunks(B, S, H, D, Dv);
  size_t n = (size_t)B * S * H * gla_record_floats(t.P, t.DP, Dv);
  if (nc > 1) n += (size_t)B * nc * H * D * Dv + (size_t)B * nc * H * D;
  return n;
}

// Both scans (projected decays; fixed decays with rotary q / k) share the kernels: what differs is in p.
static int launch_scan(GlaParams p, const void* a2, const void* a2_bias, float* ws, int dtype, void* stream) {
  const int B = p.B, S = p.S, H = p.H, D = p.D, Dv = p.Dv, R = p.R;
  int P = 1;
  while (P * GS_DP < D) P *= 2;
  JL_CHECK_ARG(P <= 32, "jl_gla_scan: key size %d above %d", D, 32 * GS_DP);
  const int cols = GS_THREADS / P;
  p.P = P;
  const size_t smem = (size_t)(3 * GS_TC * P * GS_PITCH + GS_TC * cols + GS_TC * R) * sizeof(float);
  JL_CHECK_ARG(smem <= 200 * 1024, "jl_gla_scan: key size %d with rank %d does not fit the staging buffer", D, R);
  dim3 grid((Dv + cols - 1) / cols, H, B), block(GS_THREADS);
  if (ws != nullptr && D <= 256) {                           // (wider keys: the fused kernel below)                           // prompts: token-parallel preparation, then the pipelined scan
    cudaStream_t st = (cudaStream_t)stream;
    const GlaTile t = gla_tile(D);
    JL_CHECK_ARG(t.P <= 32, "jl_gla_scan: key size %d above %d", D, 32 * t.DP);
    p.P = t.P;
    const int tcols = GS_THREADS / t.P * t.C;
      JL_DISPATCH_DTYPE(dtype, JL_LAUNCH_PDL(gla_prep_kernel<T>, dim3(B * S), dim3(128), R * sizeof(float), st, p, (const T*)a2, (const T*)a2_bias, ws, t.DP));
    JL_CUDA(cudaGetLastError());
    const size_t smem2 = (size_t)2 * GS_TS * (3 * t.P * (t.DP + 4) + tcols) * sizeof(float);
    JL_CHECK_ARG(smem2 <= 200 * 1024, "jl_gla_scan: key size %d does not fit the pipeline stages", D);
    const int nc = gla_chunks(B, S, H, D, Dv);
    p.NC = nc;
    p.L = nc > 1 ? ((S + nc - 1) / nc + GS_TS - 1) / GS_TS * GS_TS : S;
    p.cstate = ws + (size_t)B * S * H * gla_record_floats(t.P, t.DP, Dv);
    p.cdecay = p.cstate + (size_t)B * nc * H * D * Dv;
    dim3 grid2((Dv + tcols - 1) / tcols, H, B * nc);
    if (t.DP == 8 && smem2 > 48 * 1024)
      JL_CUDA(cudaFuncSetAttribute(gla_stream_kernel<8, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2));
    if (t.DP == 32 && smem2 > 48 * 1024)
      JL_CUDA(cudaFuncSetAttribute(gla_stream_kernel<32, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2));
    for (int pass = 0; pass < (nc > 1 ? 2 : 1); ++pass) {
      p.mode = nc > 1 ? (pass == 0 ? 1 : 3) : 0;
          if (t.DP == 8) JL_LAUNCH_PDL((gla_stream_kernel<8, 4>), dim3(grid2), dim3(block), smem2, st, p, ws);
      else JL_LAUNCH_PDL((gla_stream_kernel<32, 1>), dim3(grid2), dim3(block), smem2, st, p, ws);
      JL_CUDA(cudaGetLastError());
      if (pass == 0 && nc > 1) {
        const size_t total = (size_t)B * H * D * Dv;
              JL_LAUNCH_PDL(gla_combine_kernel, dim3((unsigned)((total + 255) / 256 < 1184 ? (total + 255) / 256 : 1184)), dim3(256), 0, st, p);
        JL_CUDA(cudaGetLastError());
      }
    }
    return JL_OK;
  }
  if (smem > 48 * 1024) {
    if (dtype == DT_BF16) JL_CUDA(cudaFuncSetAttribute(gla_scan_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    else JL_CUDA(cudaFuncSetAttribute(gla_scan_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  }
  JL_DISPATCH_DTYPE(dtype, JL_LAUNCH_PDL(gla_scan_kernel<T>, dim3(grid), dim3(block), smem, (cudaStream_t)stream, p, (const T*)a2, (const T*)a2_bias));
  JL_CUDA(cudaGetLastError());
  return JL_OK;
}

extern "C" JL_API int jl_gla_scan(const float* y, int ldy, int q_off, int k_off, int v_off, int a_off, const void* a2,
                                  const void* a2_bias, float* state, float* o, const int* cache_len, const int* pad_left, int B,
                                  int S, int H, int D, int Dv, int R, float q_scale, float tau, float* ws, int dtype,
                                  void* stream) {
  JL_CHECK_ARG(B >= 1 && S >= 1 && H >= 1 && D >= 1 && Dv >= 1 && R >= 1, "jl_gla_scan: bad shape");
  JL_CHECK_ARG(tau > 0.0f, "jl_gla_scan: tau=%f must be positive", tau);
  GlaParams p{y, ldy, q_off, k_off, v_off, a_off, B, S, H, D, Dv, R, 1, q_scale, 1.0f / tau, cache_len, pad_left, state, o};
  p.k_scale = 1.0f;
  return launch_scan(p, a2, a2_bias, ws, dtype, stream);
}

extern "C" JL_API int jl_retention_scan(const float* y, int ldy, int q_off, int k_off, int v_off, const float* head_decay,
                                        const float* cos_t, const float* sin_t, int max_pos, int rot, int layout, float q_scale,
                                        float k_scale, float* state, float* o, const int* cache_len, const int* pad_left, int B,
                                        int S, int H, int D, int Dv, float* ws, void* stream) {
  JL_CHECK_ARG(B >= 1 && S >= 1 && H >= 1 && D >= 1 && Dv >= 1 && head_decay != nullptr, "jl_retention_scan: bad shape");
  JL_CHECK_ARG(rot >= 0 && rot <= D && rot % 2 == 0 && (layout == 0 || layout == 1), "jl_retention_scan: rot=%d of D=%d, layout %d",
               rot, D, layout);
  GlaParams p{y, ldy, q_off, k_off, v_off, 0, B, S, H, D, Dv, 0, 1, q_scale, 1.0f, cache_len, pad_left, state, o};
  p.head_decay = head_decay; p.cos_t = cos_t; p.sin_t = sin_t; p.rot = rot; p.layout = layout; p.max_pos = max_pos;
  p.k_scale = k_scale;
  return launch_scan(p, nullptr, nullptr, ws, DT_F32, stream);
}

extern "C" JL_API int jl_ssd_scan(const float* u, int ldu, int q_off, int k_off, int v_off, int G, const float* aux, float* state,
                                  float* o, const int* cache_len, const int* pad_left, int B, int S, int H, int D, int Dv,
                                  float* ws, void* stream) {
  JL_CHECK_ARG(B >= 1 && S >= 1 && H >= 1 && D >= 1 && Dv >= 1 && aux != nullptr, "jl_ssd_scan: bad shape");
  JL_CHECK_ARG(G >= 1 && H % G == 0, "jl_ssd_scan: %d heads in %d groups", H, G);
  GlaParams p{u, ldu, q_off, k_off, v_off, 0, B, S, H, D, Dv, 0, 1, 1.0f, 1.0f, cache_len, pad_left, state, o};
  p.k_scale = 1.0f;
  p.qk_div = H / G; p.aux = aux; p.ld_aux = 2 * H;
  return launch_scan(p, nullptr, nullptr, ws, DT_F32, stream);
}
