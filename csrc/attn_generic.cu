// Softmax attention for any head sizes (query/key size D, value size Dv, D != Dv allowed), grouped key/value heads, in
// bfloat16 or true float32, with the pieces newer decoder designs put around it:
//
//  * attn_prep_kernel   — interleaved-pair rotary embedding on the first `rot` channels of each head (pair 2i, 2i+1;
//    the rest pass through), then optional weight-free unit-RMS scaling of q and k per head, append of k / v to the
//    cache [B][G][T][D] / [B][G][T][Dv].  Token (b, s) goes to slot *cache_len + s at position slot - pad_left[b].
//    A layer that reads another layer's keys and values runs it for the queries only.
//  * attn_rows_kernel   — 16 queries of one head per CTA against key / value tiles of 32 rows staged in shared memory
//    (one key per lane for the scores, one value column per lane for the output), online softmax in fp32, causal over
//    slots [pad_left[b], slot], optional per-head output gate sigmoid(g).  Prompts of any length; exact path for
//    float32 and for head sizes the tensor-core kernels are not built for.
//  * attn_decode_kernel — one CTA per (row, head) for a single new token: its warps take interleaved blocks of 32 keys
//    and merge their (max, sum, output) triples in shared memory (what runs when the caller brings no scratch).
//  * attn_split_kernel + attn_merge_kernel — a single new token with the keys split over CTAs: a CTA stages 32-key tiles
//    once for up to 16 query heads of a key/value head and a second launch merges the splits.
//  * latent_prep_kernel, rotary_slice_kernel — what latent attention puts around the attention proper: norms of the
//    query and key/value latents, rotation of the key part shared by the heads, append of one row per token; rotation
//    of a slice of every head into another head layout.
//
// Keys and values are addressed by a row pitch and batch / head strides, so that the kernels read [B][G][T][d] caches,
// one cached row per token shared by all heads (values = leading columns of the keys), or token-major projections; a
// window limits a query to the last `window` slots up to its own.
//
// Input q / k / v / gate are columns of one fp32 projection buffer (row pitch ldy), as the fused projection writes them.
#include "jllama_b200.h"
#include "seq_types.cuh"

namespace jl {

struct PrepParams {
  const float* y; int ldy;
  int q_off, k_off, v_off;          // column offsets in y; k_off < 0: queries only
  int B, S, H, G, D, Dv, T;
  int rot;                          // rotated channels per head (even, <= D)
  const float* cos_t; const float* sin_t; int max_pos;      // [max_pos][rot/2]
  int unit_norm; float eps;
  const int* cache_len; const int* pad_left;
  const float* bias;                // fp32, indexed like the columns of y (added before anything else), or nullptr
  int v_norm;                       // values scaled to unit RMS per head (no weight) before they are cached
  int v_token_major;                // value cache [B][T][G*Dv] (all heads of a token in one row) instead of [B][G][T][Dv]
  int layout;                       // pairing of the rotated q / k channels: 0 = (2i, 2i+1), 1 = (i, i + rot/2)
  const void* qw; const void* kw;   // [D] weights (element type of the caches) of an RMS norm of every q / k head BEFORE the
                                    // rotation, shared by the heads; nullptr: none
  const float* vcos; const float* vsin; int v_max_pos, v_layout;   // [v_max_pos][Dv/2]: values are rotated at their own position over all
                                    // Dv channels before they are cached (pairs as v_layout says); nullptr: cached as they are
};

constexpr int AP_WARPS = 4;      // heads per CTA of the preparation kernel (one warp each)

template <typename T>
__global__ void __launch_bounds__(AP_WARPS * 32) attn_prep_kernel(PrepParams p, T* __restrict__ q_out, T* __restrict__ kc,
                                                                  T* __restrict__ vc, int n_heads, int pair_loads) {
  pdl_wait();                      // programmatic dependent launch: nothing is read before the predecessor is done
  pdl_launch_dependents();
  const int m = blockIdx.x, head = blockIdx.y * AP_WARPS + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (head >= n_heads) return;
  const int b = m / p.S, s = m % p.S;
  const int slot = (p.cache_len ? *p.cache_len : 0) + s;
  int pos = slot - (p.pad_left ? p.pad_left[b] : 0);
  pos = pos < 0 ? 0 : (pos >= p.max_pos ? p.max_pos - 1 : pos);
  const float* yr = p.y + (size_t)m * p.ldy;
  if (head >= p.H + p.G) {                               // value head: plain copy into the cache
    const int g = head - p.H - p.G;
    T* dst = p.v_token_major ? vc + (((size_t)b * p.T + slot) * p.G + g) * p.Dv : vc + (((size_t)b * p.G + g) * p.T + slot) * p.Dv;
    const float* vb = p.bias ? p.bias + p.v_off + g * p.Dv : nullptr;
    float r = 1.0f;
    if (p.v_norm) {
      float ss = 0.0f;
      for (int i = lane; i < p.Dv; i += 32) { const float v = yr[p.v_off + g * p.Dv + i] + (vb ? vb[i] : 0.0f); ss += v * v; }
      r = 1.0f / sqrtf(warp_sum(ss) / (float)p.Dv + p.eps);
    }
    if (p.vcos) {                                          // value turned by its own position (undone on the head's sum later)
      int vpos = slot - (p.pad_left ? p.pad_left[b] : 0);
      vpos = vpos < 0 ? 0 : (vpos >= p.v_max_pos ? p.v_max_pos - 1 : vpos);
      const float* ct = p.vcos + (size_t)vpos * (p.Dv / 2);
      const float* st = p.vsin + (size_t)vpos * (p.Dv / 2);
      const float* vs = yr + p.v_off + g * p.Dv;
      const int half = p.Dv / 2;
      for (int i = lane; i < half; i += 32) {
        const int c0 = p.v_layout ? i : 2 * i, c1 = p.v_layout ? i + half : 2 * i + 1;
        const float u = (vs[c0] + (vb ? vb[c0] : 0.0f)) * r, v = (vs[c1] + (vb ? vb[c1] : 0.0f)) * r;
        dst[c0] = from_f<T>(u * ct[i] - v * st[i]);
        dst[c1] = from_f<T>(v * ct[i] + u * st[i]);
      }
      return;
    }
    for (int i = lane; i < p.Dv; i += 32) dst[i] = from_f<T>((yr[p.v_off + g * p.Dv + i] + (vb ? vb[i] : 0.0f)) * r);
    return;
  }
  const bool is_q = head < p.H;
  const int col = is_q ? p.q_off + head * p.D : p.k_off + (head - p.H) * p.D;
  const float* src = yr + col;
  const float* bs = p.bias ? p.bias + col : nullptr;
  T* dst = is_q ? q_out + ((size_t)m * p.H + head) * p.D
                : kc + (((size_t)b * p.G + (head - p.H)) * p.T + slot) * p.D;
  const float* ct = p.cos_t + (size_t)pos * (p.rot / 2);
  const float* st = p.sin_t + (size_t)pos * (p.rot / 2);
  if (p.qw != nullptr || p.layout != 0) {
    // general form: optional RMS norm with a weight first, then the rotation in either pairing
    const T* w = reinterpret_cast<const T*>(is_q ? p.qw : p.kw);
    float r = 1.0f;
    if (w) {
      float ss = 0.0f;
      for (int c = lane; c < p.D; c += 32) { const float v = src[c] + (bs ? bs[c] : 0.0f); ss += v * v; }
      r = 1.0f / sqrtf(warp_sum(ss) / (float)p.D + p.eps);
    }
    auto val = [&](int c) { const float v = src[c] + (bs ? bs[c] : 0.0f); return w ? v * r * to_f(w[c]) : v; };
    const int half = p.rot / 2;
    for (int i = lane; i < half; i += 32) {
      const int c0 = p.layout ? i : 2 * i, c1 = p.layout ? i + half : 2 * i + 1;
      const float u = val(c0), v = val(c1);
      dst[c0] = from_f<T>(u * ct[i] - v * st[i]);
      dst[c1] = from_f<T>(v * ct[i] + u * st[i]);
    }
    for (int c = p.rot + lane; c < p.D; c += 32) dst[c] = from_f<T>(val(c));
    return;
  }
  const int npairs = p.D / 2 + (p.D & 1);
  // pass 1 rotates and sums the squares, pass 2 rotates again (L1 hits) and writes the scaled values
  float r = 1.0f;
  for (int pass = p.unit_norm ? 0 : 1; pass < 2; ++pass) {
    float ss = 0.0f;
    for (int i = lane; i < npairs; i += 32) {
      const int c0 = 2 * i, c1 = 2 * i + 1;
      float u, v;
      if (pair_loads) { const float2 t = *reinterpret_cast<const float2*>(src + c0); u = t.x; v = t.y; }
      else { u = src[c0]; v = c1 < p.D ? src[c1] : 0.0f; }
      if (bs) { u += bs[c0]; if (c1 < p.D) v += bs[c1]; }
      if (c1 < p.rot) { const float c = ct[i], sn = st[i]; const float ru = u * c - v * sn, rv = v * c + u * sn; u = ru; v = rv; }
      if (pass == 0) {
        ss += u * u + v * v;
      } else {
        dst[c0] = from_f<T>(u * r);
        if (c1 < p.D) dst[c1] = from_f<T>(v * r);
      }
    }
    if (pass == 0) r = 1.0f / sqrtf(warp_sum(ss) / (float)p.D + p.eps);
  }
}

// Latent attention, preparation: the fused down-projection row y holds the query latent (q_rank columns at q_off) and the
// key/value latent followed by one rotated key part shared by all heads (kv_rank + rot_dim columns at kv_off).  Both latents
// are RMS-normed with a plain weight; the key part gets the rotary embedding of the token's position on its first `rot`
// channels.  The normed query latent goes to cq [M][q_rank]; the normed key/value latent and the rotated key part are
// appended as ONE cache row [kv_rank | rot_dim] at slot *cache_len + s — all that this kind of layer keeps per token.
struct LatentPrepParams {
  const float* y; int ldy;
  int q_off, q_rank, kv_off, kv_rank, rot_dim, rot, layout;
  const float* cos_t; const float* sin_t; int max_pos;
  float eps;
  int B, S, T;
  const int* cache_len; const int* pad_left;
  void* c_out; void* kr_out;        // optional token-major copies of what was appended: latent [M][kv_rank], key part [M][rot_dim]
};

template <typename T>
__global__ void __launch_bounds__(128) latent_prep_kernel(LatentPrepParams p, const T* __restrict__ wq, const T* __restrict__ wkv,
                                                          T* __restrict__ cq, T* __restrict__ cache) {
  pdl_wait();                      // programmatic dependent launch: nothing is read before the predecessor is done
  pdl_launch_dependents();
  __shared__ float red[33];
  const int m = blockIdx.x, b = m / p.S, s = m % p.S;
  const int slot = (p.cache_len ? *p.cache_len : 0) + s;
  int pos = slot - (p.pad_left ? p.pad_left[b] : 0);
  pos = pos < 0 ? 0 : (pos >= p.max_pos ? p.max_pos - 1 : pos);
  const float* yr = p.y + (size_t)m * p.ldy;
  if (p.q_rank > 0) {
    float ss = 0.0f;
    for (int i = threadIdx.x; i < p.q_rank; i += blockDim.x) { const float v = yr[p.q_off + i]; ss += v * v; }
    const float r = 1.0f / sqrtf(block_sum(ss, red) / (float)p.q_rank + p.eps);
    for (int i = threadIdx.x; i < p.q_rank; i += blockDim.x)
      cq[(size_t)m * p.q_rank + i] = from_f<T>(yr[p.q_off + i] * r * to_f(wq[i]));
  }
  T* row = cache + ((size_t)b * p.T + slot) * (p.kv_rank + p.rot_dim);
  float ss = 0.0f;
  for (int i = threadIdx.x; i < p.kv_rank; i += blockDim.x) { const float v = yr[p.kv_off + i]; ss += v * v; }
  const float r = 1.0f / sqrtf(block_sum(ss, red) / (float)p.kv_rank + p.eps);
  T* c_out = p.c_out ? (T*)p.c_out + (size_t)m * p.kv_rank : nullptr;
  T* kr_out = p.kr_out ? (T*)p.kr_out + (size_t)m * p.rot_dim : nullptr;
  for (int i = threadIdx.x; i < p.kv_rank; i += blockDim.x) {
    const T v = from_f<T>(yr[p.kv_off + i] * r * to_f(wkv[i]));
    row[i] = v;
    if (c_out) c_out[i] = v;
  }
  const float* src = yr + p.kv_off + p.kv_rank;
  const float* ct = p.cos_t + (size_t)pos * (p.rot / 2);
  const float* st = p.sin_t + (size_t)pos * (p.rot / 2);
  for (int d = threadIdx.x; d < p.rot_dim; d += blockDim.x) {
    const T v = from_f<T>(rotary_channel(src, d, p.rot, p.layout, ct, st));
    row[p.kv_rank + d] = v;
    if (kr_out) kr_out[d] = v;
  }
}

// out[m, h, out_off + d] = rotary(in[m, h, in_off + d]), d < n: a slice of every head rotated at the token's position and
// copied into another head layout (in / out head pitches in_hs / out_hs, row pitches ldi / ldo).
template <typename T>
__global__ void __launch_bounds__(128) rotary_slice_kernel(const T* __restrict__ in, int ldi, int in_hs, int in_off,
                                                           T* __restrict__ out, int ldo, int out_hs, int out_off, int H, int n,
                                                           int rot, int layout, const float* __restrict__ cos_t,
                                                           const float* __restrict__ sin_t, int max_pos,
                                                           const int* __restrict__ cache_len, const int* __restrict__ pad_left,
                                                           int S) {
  pdl_wait();                      // programmatic dependent launch: nothing is read before the predecessor is done
  pdl_launch_dependents();
  const int m = blockIdx.x, b = m / S, s = m % S;
  int pos = (cache_len ? *cache_len : 0) + s - (pad_left ? pad_left[b] : 0);
  pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
  const float* ct = cos_t + (size_t)pos * (rot / 2);
  const float* st = sin_t + (size_t)pos * (rot / 2);
  for (int i = threadIdx.x; i < H * n; i += blockDim.x) {
    const int h = i / n, d = i % n;
    out[(size_t)m * ldo + (size_t)h * out_hs + out_off + d] =
        from_f<T>(rotary_channel(in + (size_t)m * ldi + (size_t)h * in_hs + in_off, d, rot, layout, ct, st));
  }
}

struct AttnParams {
  int B, S, H, G, D, Dv, T;
  int ldk, ldv;                     // row pitch of the key / value cache in elements (>= D / Dv: the two may be columns of one row)
  long long k_bs, k_hs, v_bs, v_hs; // batch-row and key/value-head strides in elements: [B][G][T][ld] caches have bs = G*T*ld, hs = T*ld;
                                    // token-major projections [B*T][G][ld'] have bs = T*G*ld', hs = ld' and a row pitch of G*ld'
  int window;                       // > 0: a query at slot i sees slots i - window + 1 .. i only; 0: everything before it
  float scale;
  const int* cache_len;             // slots already filled BEFORE this call's tokens (device scalar); nullptr = 0
  const int* pad_left;
  const float* gate; int ldg;       // fp32 pre-activation of the per-head output gate (column h of row m), or nullptr
  int sink;                         // 1: the softmax denominator has one more term exp(0) (a key with score 0 and no value)
  float* out32;                     // fp32 output [M][H][Dv] instead of `out` (what a later fp32 step reads), or nullptr
  int chunk;                        // > 0: positions (slot - pad_left) form blocks of `chunk`; a query sees the keys of its own block only
  const float* sink_logit;          // [H] fp32: the extra term of the denominator is exp(sink_logit[h]) instead of exp(0) (with sink = 1)
  const float* vcos; const float* vsin; int v_max_pos, v_layout;   // [v_max_pos][Dv/2]: the cached values were rotated at their own
                                    // positions; every head's sum is rotated back by the query's position (pairs as v_layout)
};

// first slot a query at slot hi_q of a row whose sequence starts at slot lo may see
__device__ __forceinline__ int attn_first_visible(const AttnParams& p, int lo, int hi_q) {
  int first = lo;
  if (p.window > 0) first = max(first, hi_q - p.window + 1);
  if (p.chunk > 0 && hi_q >= lo) first = max(first, lo + (hi_q - lo) / p.chunk * p.chunk);
  return first;
}

// the denominator of a row whose running maximum is m and whose visible keys sum to l (l == 0: nothing visible, the row is zero)
__device__ __forceinline__ float attn_inv_denominator(const AttnParams& p, float m, float l, int h) {
  if (!(l > 0.0f)) return 0.0f;
  return 1.0f / (p.sink ? l + expf((p.sink_logit ? p.sink_logit[h] : 0.0f) - m) : l);
}
template <typename T>
__device__ __forceinline__ void attn_store(const AttnParams& p, T* out, size_t at, float v) {
  if (p.out32) p.out32[at] = v; else out[at] = from_f<T>(v);
}

// A head's normalised sum `o` (Dv floats in shared memory, complete and visible to the calling threads) → rotated back by the
// query's position when the values were cached rotated, times gmul, stored.  Threads tid, tid + nthreads, ... take the columns.
template <typename T>
__device__ __forceinline__ void attn_finish_row(const AttnParams& p, T* out, size_t at, const float* o, int pos, float gmul, int tid,
                                                int nthreads) {
  if (p.vcos == nullptr) {
    for (int c = tid; c < p.Dv; c += nthreads) attn_store<T>(p, out, at + c, o[c] * gmul);
    return;
  }
  pos = pos < 0 ? 0 : (pos >= p.v_max_pos ? p.v_max_pos - 1 : pos);
  const int half = p.Dv / 2;
  const float* ct = p.vcos + (size_t)pos * half;
  const float* st = p.vsin + (size_t)pos * half;
  for (int i = tid; i < half; i += nthreads) {
    const int c0 = p.v_layout ? i : 2 * i, c1 = p.v_layout ? i + half : 2 * i + 1;
    const float u = o[c0], v = o[c1];
    attn_store<T>(p, out, at + c0, (u * ct[i] + v * st[i]) * gmul);           // the turn by -pos
    attn_store<T>(p, out, at + c1, (v * ct[i] - u * st[i]) * gmul);
  }
}

constexpr int AT_MAXV = 16;         // value columns per lane: Dv <= 512

// scores of one block of 32 keys (lane = key), then the block's contribution to the output (lane = value column)
template <typename T>
__device__ __forceinline__ void attn_block(const float* __restrict__ qs, const T* __restrict__ kbase, const T* __restrict__ vbase,
                                           int j0, int lo, int hi, int D, int Dv, int ldk, int ldv, float scale, float& mrun,
                                           float& lrun, float (&acc)[AT_MAXV]) {
  const int lane = threadIdx.x & 31;
  const int j = j0 + lane;
  float sc = -INFINITY;
  if (j >= lo && j <= hi) {
    const T* kr = kbase + (size_t)j * ldk;
    float d = 0.0f;
    for (int c = 0; c < D; ++c) d = fmaf(qs[c], to_f(kr[c]), d);
    sc = d * scale;
  }
  const float mnew = fmaxf(mrun, warp_max(sc));
  if (mnew == -INFINITY) return;                       // nothing visible in this block (uniform across the warp)
  const float corr = mrun == -INFINITY ? 0.0f : expf(mrun - mnew);
  const float pj = sc == -INFINITY ? 0.0f : expf(sc - mnew);
  lrun = lrun * corr + warp_sum(pj);
  mrun = mnew;
#pragma unroll
  for (int i = 0; i < AT_MAXV; ++i) acc[i] *= corr;
  const int jend = min(32, hi - j0 + 1);
  for (int t = 0; t < jend; ++t) {
    const float pt = __shfl_sync(0xffffffffu, pj, t);
    if (pt == 0.0f) continue;
    const T* vr = vbase + (size_t)(j0 + t) * ldv;
#pragma unroll
    for (int i = 0; i < AT_MAXV; ++i) {
      const int c = lane + 32 * i;
      if (c < Dv) acc[i] = fmaf(pt, to_f(vr[c]), acc[i]);
    }
  }
}

// Rows j0 .. j0+31 of a cache head (row length n, row pitch ld, rows beyond jmax read as zero) into shared memory as fp32 with row
// pitch `pitch`; 16-byte global loads when a row is a whole number of them, else element by element (which also zeroes
// the columns between n and the next multiple of four, the part of the pitch the dot products read).
template <typename T>
__device__ __forceinline__ void stage_rows(float* dst, int pitch, const T* __restrict__ src, int n, int ld, int j0, int jmax) {
  constexpr int VN = 16 / sizeof(T);
  if (n % VN == 0 && ld % VN == 0 && ((uintptr_t)src & 15) == 0) {
    const int per_row = n / VN, total = 32 * per_row;
    constexpr int U = 4;                                   // loads in flight per thread: the tile is latency-bound otherwise
    for (int i0 = threadIdx.x; i0 < total; i0 += U * blockDim.x) {
      uint4 raw[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int i = i0 + u * blockDim.x;
        const int r = i / per_row, cv = i % per_row, j = j0 + r;
        raw[u] = (i < total && j <= jmax) ? *reinterpret_cast<const uint4*>(src + (size_t)j * ld + cv * VN) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int i = i0 + u * blockDim.x;
        if (i >= total) break;
        float* d = dst + (i / per_row) * pitch + (i % per_row) * VN;
        if constexpr (sizeof(T) == 2) {                      // zero bits are 0.0f in both types
          *reinterpret_cast<float4*>(d) = make_float4(bf16_lo(raw[u].x), bf16_hi(raw[u].x), bf16_lo(raw[u].y), bf16_hi(raw[u].y));
          *reinterpret_cast<float4*>(d + 4) = make_float4(bf16_lo(raw[u].z), bf16_hi(raw[u].z), bf16_lo(raw[u].w), bf16_hi(raw[u].w));
        } else {
          *reinterpret_cast<uint4*>(d) = raw[u];
        }
      }
    }
    return;
  }
  const int np = (n + 3) & ~3;
  for (int i = threadIdx.x; i < 32 * np; i += blockDim.x) {
    const int r = i / np, c = i % np, j = j0 + r;
    dst[r * pitch + c] = (j <= jmax && c < n) ? to_f(src[(size_t)j * ld + c]) : 0.0f;
  }
}

// Prompt attention, tiled: a CTA owns AR_QB consecutive queries of one head (AR_QW per warp) and walks the visible keys
// in tiles of 32.  The K and V rows of a tile are brought into shared memory once, with coalesced loads, converted to
// fp32, and serve all the CTA's queries; a lane scores one key (16-byte shared-memory reads of its K row against the
// query held in shared memory), then owns value columns lane, lane + 32, ... for the weighted sum.
constexpr int AR_WARPS = 4, AR_QW = 4, AR_QB = AR_WARPS * AR_QW;

template <typename T, int NV>
__global__ void __launch_bounds__(AR_WARPS * 32) attn_rows_kernel(AttnParams p, const T* __restrict__ q, const T* __restrict__ kc,
                                                                  const T* __restrict__ vc, T* __restrict__ out) {
  pdl_wait();                      // programmatic dependent launch: nothing is read before the predecessor is done
  pdl_launch_dependents();
  extern __shared__ float4 smem4[];
  float* smem = reinterpret_cast<float*>(smem4);
  const int DP = ((p.D + 3) & ~3) + 4;                   // fp32 pitch of a K / q row: 16-byte rows, banks spread
  float* Qs = smem;                                      // [AR_QB][DP]
  float* Ks = Qs + AR_QB * DP;                           // [32][DP]
  float* Vs = Ks + 32 * DP;                              // [32][DVP]
  const int DVP = (p.Dv + 3) & ~3;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y, b = blockIdx.z, q0 = blockIdx.x * AR_QB;
  const int g = h / (p.H / p.G);
  const int base = p.cache_len ? *p.cache_len : 0;
  const int lo = p.pad_left ? p.pad_left[b] : 0;
  const int hi_cta = base + min(q0 + AR_QB, p.S) - 1;    // last key any query of this CTA sees
  const int lo_cta = attn_first_visible(p, lo, base + q0);      // first key any query of this CTA sees (its first query's)
  for (int i = threadIdx.x; i < AR_QB * DP; i += blockDim.x) {
    const int r = i / DP, c = i % DP, s = q0 + r;
    Qs[i] = (s < p.S && c < p.D) ? to_f(q[((size_t)(b * p.S + s) * p.H + h) * p.D + c]) : 0.0f;
  }
  const T* kbase = kc + (size_t)b * p.k_bs + (size_t)g * p.k_hs;
  const T* vbase = vc + (size_t)b * p.v_bs + (size_t)g * p.v_hs;
  float mrun[AR_QW], lrun[AR_QW], acc[AR_QW][NV];
#pragma unroll
  for (int qi = 0; qi < AR_QW; ++qi) {
    mrun[qi] = -INFINITY; lrun[qi] = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; ++i) acc[qi][i] = 0.0f;
  }
  for (int j0 = lo_cta & ~31; j0 <= hi_cta; j0 += 32) {
    __syncthreads();                                     // the previous tile is no longer read
    stage_rows<T>(Ks, DP, kbase, p.D, p.ldk, j0, hi_cta);
    stage_rows<T>(Vs, DVP, vbase, p.Dv, p.ldv, j0, hi_cta);
    __syncthreads();
    // the warp's AR_QW queries against the tile (lane = key): every key and value channel is read once for all of them
    int hi_q[AR_QW], lo_q[AR_QW], jend = 0;
    bool on[AR_QW];
#pragma unroll
    for (int qi = 0; qi < AR_QW; ++qi) {
      const int s = q0 + warp * AR_QW + qi;
      hi_q[qi] = base + s;
      lo_q[qi] = attn_first_visible(p, lo, hi_q[qi]);
      on[qi] = s < p.S && j0 <= hi_q[qi] && j0 + 31 >= lo_q[qi];         // warp-uniform
      if (on[qi]) jend = max(jend, min(32, hi_q[qi] - j0 + 1));
    }
    if (jend == 0) continue;                               // no query of this warp sees the tile (the CTA's barriers are above)
    float d0[AR_QW], d1[AR_QW], pj[AR_QW];
#pragma unroll
    for (int qi = 0; qi < AR_QW; ++qi) d0[qi] = d1[qi] = 0.0f;
    {
      const float4* kr = reinterpret_cast<const float4*>(Ks + lane * DP);
      const float4* qr = reinterpret_cast<const float4*>(Qs + warp * AR_QW * DP);
      for (int c = 0; c < (DP - 4) / 4; ++c) {
        const float4 k4 = kr[c];
#pragma unroll
        for (int qi = 0; qi < AR_QW; ++qi) {
          const float4 a = qr[qi * (DP / 4) + c];
          d0[qi] = fmaf(a.x, k4.x, d0[qi]); d1[qi] = fmaf(a.y, k4.y, d1[qi]);
          d0[qi] = fmaf(a.z, k4.z, d0[qi]); d1[qi] = fmaf(a.w, k4.w, d1[qi]);
        }
      }
    }
    const int j = j0 + lane;
#pragma unroll
    for (int qi = 0; qi < AR_QW; ++qi) {
      pj[qi] = 0.0f;
      if (!on[qi]) continue;
      const float sc = (j >= lo_q[qi] && j <= hi_q[qi]) ? (d0[qi] + d1[qi]) * p.scale : -INFINITY;
      const float mnew = fmaxf(mrun[qi], warp_max(sc));
      if (mnew == -INFINITY) continue;
      const float corr = mrun[qi] == -INFINITY ? 0.0f : expf(mrun[qi] - mnew);
      pj[qi] = sc == -INFINITY ? 0.0f : expf(sc - mnew);
      lrun[qi] = lrun[qi] * corr + warp_sum(pj[qi]);
      mrun[qi] = mnew;
#pragma unroll
      for (int i = 0; i < NV; ++i) acc[qi][i] *= corr;
    }
    for (int t = 0; t < jend; ++t) {
      float pt[AR_QW];
#pragma unroll
      for (int qi = 0; qi < AR_QW; ++qi) pt[qi] = __shfl_sync(0xffffffffu, pj[qi], t);
      const float* vr = Vs + t * DVP;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int c = lane + 32 * i;
        if (c < p.Dv) {
          const float v = vr[c];
#pragma unroll
          for (int qi = 0; qi < AR_QW; ++qi) acc[qi][i] = fmaf(pt[qi], v, acc[qi][i]);
        }
      }
    }
  }
  if (p.vcos) __syncthreads();                             // every warp is done with the last value tile: its rows are reused below
#pragma unroll
  for (int qi = 0; qi < AR_QW; ++qi) {
    const int s = q0 + warp * AR_QW + qi;
    if (s >= p.S) continue;
    const int m = b * p.S + s;
    float gmul = attn_inv_denominator(p, mrun[qi], lrun[qi], h);  // a padding query sees nothing: its row is zero
    if (p.vcos) {                                          // the normalised sum meets in the warp's row of shared memory first
      float* orow = Vs + warp * DVP;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int c = lane + 32 * i;
        if (c < p.Dv) orow[c] = acc[qi][i] * gmul;
      }
      __syncwarp();
      const float gate = p.gate ? sigmoid_f(p.gate[(size_t)m * p.ldg + h]) : 1.0f;
      attn_finish_row<T>(p, out, ((size_t)m * p.H + h) * p.Dv, orow, base + s - lo, gate, lane, 32);
      __syncwarp();
      continue;
    }
    if (p.gate) gmul *= sigmoid_f(p.gate[(size_t)m * p.ldg + h]);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = lane + 32 * i;
      if (c < p.Dv) attn_store<T>(p, out, ((size_t)m * p.H + h) * p.Dv + c, acc[qi][i] * gmul);
    }
  }
}

constexpr int AD_WARPS = 8;

template <typename T>
__global__ void __launch_bounds__(AD_WARPS * 32) attn_decode_kernel(AttnParams p, const T* __restrict__ q, const T* __restrict__ kc,
                                                                    const T* __restrict__ vc, T* __restrict__ out) {
  pdl_wait();                      // programmatic dependent launch: nothing is read before the predecessor is done
  pdl_launch_dependents();
  extern __shared__ float smem[];                       // [D] query | [warps][2] (max, sum) | [warps][Dv] partial outputs
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.x, b = blockIdx.y;             // S == 1: row m = b
  const int g = h / (p.H / p.G);
  float* qs = smem;
  float* ml = smem + p.D;
  float* part = ml + 2 * AD_WARPS;
  const T* qr = q + ((size_t)b * p.H + h) * p.D;
  for (int c = threadIdx.x; c < p.D; c += blockDim.x) qs[c] = to_f(qr[c]);
  __syncthreads();
  const int hi = p.cache_len ? *p.cache_len : 0;
  const int lo_seq = p.pad_left ? p.pad_left[b] : 0;     // where the row's sequence starts
  const int lo = attn_first_visible(p, lo_seq, hi);
  const T* kbase = kc + (size_t)b * p.k_bs + (size_t)g * p.k_hs;
  const T* vbase = vc + (size_t)b * p.v_bs + (size_t)g * p.v_hs;
  float mrun = -INFINITY, lrun = 0.0f, acc[AT_MAXV] = {};
  for (int j0 = (lo & ~31) + 32 * warp; j0 <= hi; j0 += 32 * AD_WARPS)
    attn_block<T>(qs, kbase, vbase, j0, lo, hi, p.D, p.Dv, p.ldk, p.ldv, p.scale, mrun, lrun, acc);
  if (lane == 0) { ml[2 * warp] = mrun; ml[2 * warp + 1] = lrun; }
#pragma unroll
  for (int i = 0; i < AT_MAXV; ++i) {
    const int c = lane + 32 * i;
    if (c < p.Dv) part[warp * p.Dv + c] = acc[i];
  }
  __syncthreads();
  float mall = -INFINITY;
  for (int w = 0; w < AD_WARPS; ++w) mall = fmaxf(mall, ml[2 * w]);
  float lall = 0.0f;
  for (int w = 0; w < AD_WARPS; ++w) if (ml[2 * w] != -INFINITY) lall += ml[2 * w + 1] * expf(ml[2 * w] - mall);
  float gmul = attn_inv_denominator(p, mall, lall, h);
  if (p.vcos) {                                            // the normalised sum meets in shared memory, then turns back
    float o[(32 * AT_MAXV + AD_WARPS * 32 - 1) / (AD_WARPS * 32)];
    for (int c = threadIdx.x, i = 0; c < p.Dv; c += blockDim.x, ++i) {
      o[i] = 0.0f;
      for (int w = 0; w < AD_WARPS; ++w) if (ml[2 * w] != -INFINITY) o[i] += part[w * p.Dv + c] * expf(ml[2 * w] - mall);
    }
    __syncthreads();
    for (int c = threadIdx.x, i = 0; c < p.Dv; c += blockDim.x, ++i) part[c] = o[i] * gmul;
    __syncthreads();
    const float gate = p.gate ? sigmoid_f(p.gate[(size_t)b * p.ldg + h]) : 1.0f;
    attn_finish_row<T>(p, out, ((size_t)b * p.H + h) * p.Dv, part, hi - lo_seq, gate, threadIdx.x, blockDim.x);
    return;
  }
  if (p.gate) gmul *= sigmoid_f(p.gate[(size_t)b * p.ldg + h]);
  for (int c = threadIdx.x; c < p.Dv; c += blockDim.x) {
    float o = 0.0f;
    for (int w = 0; w < AD_WARPS; ++w) if (ml[2 * w] != -INFINITY) o += part[w * p.Dv + c] * expf(ml[2 * w] - mall);
    attn_store<T>(p, out, ((size_t)b * p.H + h) * p.Dv + c, o * gmul);
  }
}

// One new token, split over the keys: a CTA owns one key/value head of one row and every `splits`-th tile of 32 keys;
// the tile is staged in shared memory once and serves all query heads of the group (a warp takes up to AS_RW of them).
// Each CTA leaves an unnormalised (max, sum, output) triple per query head; attn_merge_kernel joins the splits,
// normalises, applies the output gate and stores.  Contexts of thousands of keys thus spread over the whole GPU.
constexpr int AS_WARPS = 4, AS_RW = 4;             // query heads per group <= AS_WARPS * AS_RW

template <typename T, int NV>
__global__ void __launch_bounds__(AS_WARPS * 32) attn_split_kernel(AttnParams p, const T* __restrict__ q, const T* __restrict__ kc,
                                                                   const T* __restrict__ vc, float* __restrict__ part, int splits) {
  pdl_wait();                      // programmatic dependent launch: nothing is read before the predecessor is done
  pdl_launch_dependents();
  extern __shared__ float4 smem4[];
  float* smem = reinterpret_cast<float*>(smem4);
  constexpr int RB = AS_WARPS * AS_RW;                   // query heads a CTA takes; wider groups are cut into blocks of RB
  const int RG = p.H / p.G, nblk = (RG + RB - 1) / RB;
  const int g = blockIdx.y / nblk, r0 = (blockIdx.y % nblk) * RB;
  const int R = min(RB, RG - r0);
  const int DP = ((p.D + 3) & ~3) + 4;
  float* Qs = smem;                                      // [R][DP]
  float* Ks = Qs + R * DP;                               // [32][DP]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int z = blockIdx.x, b = blockIdx.z;
  const T* kbase = kc + (size_t)b * p.k_bs + (size_t)g * p.k_hs;
  const T* vbase = vc + (size_t)b * p.v_bs + (size_t)g * p.v_hs;
  // values that are the leading columns of the key rows (attention over cached latents) are staged once, with the keys
  const bool v_in_k = vbase == kbase && p.ldv == p.ldk && p.Dv <= p.D;
  float* Vs = v_in_k ? Ks : Ks + 32 * DP;                // [32][DVP]
  const int DVP = v_in_k ? DP : (p.Dv + 3) & ~3;
  const int hi = p.cache_len ? *p.cache_len : 0;         // the new token's own slot
  const int lo_seq = p.pad_left ? p.pad_left[b] : 0;     // where the row's sequence starts
  const int lo = attn_first_visible(p, lo_seq, hi);
  // the R query rows are consecutive: staged like a key tile (rows beyond R fall into the key buffer, which is filled later)
  stage_rows<T>(Qs, DP, q + ((size_t)b * p.H + (size_t)g * RG + r0) * p.D, p.D, p.D, 0, R - 1);
  float mrun[AS_RW], lrun[AS_RW], acc[AS_RW][NV];
#pragma unroll
  for (int qi = 0; qi < AS_RW; ++qi) {
    mrun[qi] = -INFINITY; lrun[qi] = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; ++i) acc[qi][i] = 0.0f;
  }
  for (int j0 = (lo & ~31) + 32 * z; j0 <= hi; j0 += 32 * splits) {
    __syncthreads();
    stage_rows<T>(Ks, DP, kbase, p.D, p.ldk, j0, hi);
    if (!v_in_k) stage_rows<T>(Vs, DVP, vbase, p.Dv, p.ldv, j0, hi);
    __syncthreads();
    const int j = j0 + lane;
    const bool vis = j >= lo && j <= hi;
    // scores of this warp's rows (lane = key): every key channel is read once for all of them; a row's sum runs in the
    // same order as in the prompt kernel
    float d0[AS_RW], d1[AS_RW], pj[AS_RW];
#pragma unroll
    for (int qi = 0; qi < AS_RW; ++qi) d0[qi] = d1[qi] = 0.0f;
    {
      const float4* kr = reinterpret_cast<const float4*>(Ks + lane * DP);
      for (int c = 0; c < (DP - 4) / 4; ++c) {
        const float4 k4 = kr[c];
#pragma unroll
        for (int qi = 0; qi < AS_RW; ++qi) {
          const int r = min(warp + AS_WARPS * qi, R - 1);          // rows beyond R repeat the last one and are dropped below
          const float4 a = reinterpret_cast<const float4*>(Qs + r * DP)[c];
          d0[qi] = fmaf(a.x, k4.x, d0[qi]); d1[qi] = fmaf(a.y, k4.y, d1[qi]);
          d0[qi] = fmaf(a.z, k4.z, d0[qi]); d1[qi] = fmaf(a.w, k4.w, d1[qi]);
        }
      }
    }
#pragma unroll
    for (int qi = 0; qi < AS_RW; ++qi) {
      pj[qi] = 0.0f;
      if (warp + AS_WARPS * qi >= R) continue;           // warp-uniform
      const float sc = vis ? (d0[qi] + d1[qi]) * p.scale : -INFINITY;
      const float mnew = fmaxf(mrun[qi], warp_max(sc));
      if (mnew == -INFINITY) continue;
      const float corr = mrun[qi] == -INFINITY ? 0.0f : expf(mrun[qi] - mnew);
      pj[qi] = sc == -INFINITY ? 0.0f : expf(sc - mnew);
      lrun[qi] = lrun[qi] * corr + warp_sum(pj[qi]);
      mrun[qi] = mnew;
#pragma unroll
      for (int i = 0; i < NV; ++i) acc[qi][i] *= corr;
    }
    const int jend = min(32, hi - j0 + 1);
    for (int t = 0; t < jend; ++t) {                     // every value channel is read once for all rows
      float pt[AS_RW];
#pragma unroll
      for (int qi = 0; qi < AS_RW; ++qi) pt[qi] = __shfl_sync(0xffffffffu, pj[qi], t);
      const float* vr = Vs + t * DVP;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int c = lane + 32 * i;
        if (c < p.Dv) {
          const float v = vr[c];
#pragma unroll
          for (int qi = 0; qi < AS_RW; ++qi) acc[qi][i] = fmaf(pt[qi], v, acc[qi][i]);
        }
      }
    }
  }
#pragma unroll
  for (int qi = 0; qi < AS_RW; ++qi) {
    const int r = warp + AS_WARPS * qi;
    if (r >= R) continue;
    float* dst = part + (((size_t)b * p.H + (size_t)g * RG + r0 + r) * splits + z) * (p.Dv + 2);
    if (lane == 0) { dst[0] = mrun[qi]; dst[1] = lrun[qi]; }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = lane + 32 * i;
      if (c < p.Dv) dst[2 + c] = acc[qi][i];
    }
  }
}

template <typename T>
__global__ void attn_merge_kernel(AttnParams p, const float* __restrict__ part, int splits, T* __restrict__ out) {
  pdl_wait();                      // programmatic dependent launch: nothing is read before the predecessor is done
  pdl_launch_dependents();
  __shared__ float wz[64];                                 // weight of every split (splits <= 64)
  __shared__ float tot, top;
  const int h = blockIdx.x, b = blockIdx.y;
  const float* src = part + ((size_t)b * p.H + h) * splits * (p.Dv + 2);
  if (threadIdx.x < 32) {                                  // the splits' maxima and sums, all loads at once
    const int lane = threadIdx.x;
    const float m0 = lane < splits ? src[(size_t)lane * (p.Dv + 2)] : -INFINITY;
    const float m1 = lane + 32 < splits ? src[(size_t)(lane + 32) * (p.Dv + 2)] : -INFINITY;
    const float l0 = lane < splits ? src[(size_t)lane * (p.Dv + 2) + 1] : 0.0f;
    const float l1 = lane + 32 < splits ? src[(size_t)(lane + 32) * (p.Dv + 2) + 1] : 0.0f;
    const float mall = warp_max(fmaxf(m0, m1));
    const float w0 = m0 == -INFINITY ? 0.0f : expf(m0 - mall), w1 = m1 == -INFINITY ? 0.0f : expf(m1 - mall);
    wz[lane] = w0; wz[lane + 32] = w1;
    float lall = 0.0f;                                     // summed in split order, as the columns below are
    for (int zz = 0; zz < splits; ++zz)
      lall += zz < 32 ? __shfl_sync(0xffffffffu, l0 * w0, zz) : __shfl_sync(0xffffffffu, l1 * w1, zz - 32);
    if (lane == 0) { tot = lall; top = mall; }
  }
  __syncthreads();
  const float lall = tot;
  float gmul = attn_inv_denominator(p, top, lall, h);
  if (p.vcos) {                                            // the normalised sum meets in shared memory, then turns back
    __shared__ float orow[32 * AT_MAXV];
    for (int c = threadIdx.x; c < p.Dv; c += blockDim.x) {
      float o = 0.0f;
#pragma unroll 8
      for (int zz = 0; zz < splits; ++zz) o = fmaf(src[(size_t)zz * (p.Dv + 2) + 2 + c], wz[zz], o);
      orow[c] = o * gmul;
    }
    __syncthreads();
    const float gate = p.gate ? sigmoid_f(p.gate[(size_t)b * p.ldg + h]) : 1.0f;
    const int hi = p.cache_len ? *p.cache_len : 0;
    attn_finish_row<T>(p, out, ((size_t)b * p.H + h) * p.Dv, orow, hi - (p.pad_left ? p.pad_left[b] : 0), gate, threadIdx.x, blockDim.x);
    return;
  }
  if (p.gate) gmul *= sigmoid_f(p.gate[(size_t)b * p.ldg + h]);
  for (int c = threadIdx.x; c < p.Dv; c += blockDim.x) {
    float o = 0.0f;
#pragma unroll 8
    for (int zz = 0; zz < splits; ++zz) o = fmaf(src[(size_t)zz * (p.Dv + 2) + 2 + c], wz[zz], o);
    attn_store<T>(p, out, ((size_t)b * p.H + h) * p.Dv + c, o * gmul);
  }
}

// out[m, h, :] *= sigmoid(gate[m, h]) for attention kernels that have no gate input (the tcgen05 prefill kernel)
template <typename T>
__global__ void head_gate_kernel(T* __restrict__ out, const float* __restrict__ gate, int ldg, int M, int H, int Dv) {
  pdl_wait();                      // programmatic dependent launch: nothing is read before the predecessor is done
  pdl_launch_dependents();
  const size_t total = (size_t)M * H * Dv;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t mh = i / Dv;
    out[i] = from_f<T>(to_f(out[i]) * sigmoid_f(gate[(mh / H) * ldg + mh % H]));
  }
}

}  // namespace jl

using namespace jl;

static int attn_prep_launch(PrepParams p, void* q_out, void* k_cache, void* v_cache, int dtype, void* stream) {
  JL_CHECK_ARG(p.B >= 1 && p.S >= 1 && p.H >= 1 && p.G >= 1 && p.D >= 1 && p.Dv >= 1, "jl_attn_prep: bad shape");
  JL_CHECK_ARG(p.rot >= 0 && p.rot <= p.D && p.rot % 2 == 0, "jl_attn_prep: rot=%d must be even and <= D=%d", p.rot, p.D);
  JL_CHECK_ARG(p.k_off >= 0 || (k_cache == nullptr && v_cache == nullptr), "jl_attn_prep: queries-only call takes no caches");
  JL_CHECK_ARG(p.layout == 0 || p.layout == 1, "jl_attn_prep: layout %d", p.layout);
  JL_CHECK_ARG((p.qw == nullptr) == (p.kw == nullptr), "jl_attn_prep: the q and k norm weights come together");
  JL_CHECK_ARG(!(p.unit_norm && (p.qw != nullptr || p.layout != 0)),
               "jl_attn_prep: unit-RMS scaling after the rotation goes with interleaved pairs and no weighted norm");
  JL_CHECK_ARG(p.vcos == nullptr || (p.vsin != nullptr && p.Dv % 2 == 0 && p.v_max_pos >= 1 && !p.v_token_major),
               "jl_attn_prep: rotated values need an even Dv=%d and head-major caches", p.Dv);
  const int n_heads = p.k_off >= 0 ? p.H + 2 * p.G : p.H;
  const int pair_loads = p.D % 2 == 0 && p.ldy % 2 == 0 && p.q_off % 2 == 0 && (p.k_off < 0 || p.k_off % 2 == 0) && (uintptr_t)p.y % 8 == 0;
  dim3 grid(p.B * p.S, (n_heads + AP_WARPS - 1) / AP_WARPS);
  JL_DISPATCH_DTYPE(dtype, JL_LAUNCH_PDL(attn_prep_kernel<T>, dim3(grid), dim3(AP_WARPS * 32), 0, (cudaStream_t)stream, p, (T*)q_out, (T*)k_cache,
                                                                                                (T*)v_cache, n_heads, pair_loads));
  JL_CUDA(cudaGetLastError());
  return JL_OK;
}

extern "C" JL_API int jl_attn_prep(const float* y, int ldy, int q_off, int k_off, int v_off, void* q_out, void* k_cache,
                                   void* v_cache, const float* cos_t, const float* sin_t, int max_pos, int rot, int unit_norm,
                                   float eps, const int* cache_len, const int* pad_left, int B, int S, int H, int G, int D, int Dv,
                                   int T_cap, const float* bias, int v_norm, int v_token_major, int dtype, void* stream) {
  PrepParams p{y, ldy, q_off, k_off, v_off, B, S, H, G, D, Dv, T_cap, rot, cos_t, sin_t, max_pos, unit_norm, eps, cache_len, pad_left,
               bias, v_norm, v_token_major, 0, nullptr, nullptr, nullptr, nullptr, 0, 0};
  return attn_prep_launch(p, q_out, k_cache, v_cache, dtype, stream);
}

// The same with the newer pieces: `layout` of the rotated q / k pairs, an RMS norm with weights q_norm_w / k_norm_w [D] before the
// rotation, and values rotated at their own position with the tables v_cos / v_sin [v_max_pos][Dv/2] (pairs as v_layout).
extern "C" JL_API int jl_attn_prep_ex(const float* y, int ldy, int q_off, int k_off, int v_off, void* q_out, void* k_cache,
                                      void* v_cache, const float* cos_t, const float* sin_t, int max_pos, int rot, int layout,
                                      int unit_norm, const void* q_norm_w, const void* k_norm_w, float eps, const float* v_cos,
                                      const float* v_sin, int v_max_pos, int v_layout, const int* cache_len, const int* pad_left,
                                      int B, int S, int H, int G, int D, int Dv, int T_cap, const float* bias, int v_norm,
                                      int v_token_major, int dtype, void* stream) {
  PrepParams p{y, ldy, q_off, k_off, v_off, B, S, H, G, D, Dv, T_cap, rot, cos_t, sin_t, max_pos, unit_norm, eps, cache_len, pad_left,
               bias, v_norm, v_token_major, layout, q_norm_w, k_norm_w, v_cos, v_sin, v_max_pos, v_layout};
  return attn_prep_launch(p, q_out, k_cache, v_cache, dtype, stream);
}

extern "C" JL_API int jl_attn_generic_splits(int B, int H, int G, int T_cap) {
  if (G <= 0) return 0;
  const int nblk = (H / G + AS_WARPS * AS_RW - 1) / (AS_WARPS * AS_RW);      // blocks of query heads per key/value head
  int s = 296 / (B * G * nblk > 0 ? B * G * nblk : 1);   // about one resident wave of CTAs
  const int tiles = (T_cap + 31) / 32;                   // a split is at least one 32-key tile at full capacity
  if (s > tiles) s = tiles;
  if (s > 64) s = 64;
  return s < 1 ? 1 : s;
}

static int attn_launch(const void* q, const void* k_cache, const void* v_cache, void* out, const float* gate, int ldg,
                       const int* cache_len, const int* pad_left, int B, int S, int H, int G, int D, int Dv, int T_cap, int ldk,
                       int ldv, int window, float scale, float* scratch, int splits, int dtype, void* stream,
                       long long k_bs = 0, long long k_hs = 0, long long v_bs = 0, long long v_hs = 0, int sink = 0,
                       float* out32 = nullptr, int chunk = 0, const float* sink_logit = nullptr, const float* vcos = nullptr,
                       const float* vsin = nullptr, int v_max_pos = 0, int v_layout = 0) {
  JL_CHECK_ARG(B >= 1 && S >= 1 && G >= 1 && H % G == 0, "jl_attn_generic: H=%d not a multiple of G=%d", H, G);
  JL_CHECK_ARG(Dv <= 32 * AT_MAXV, "jl_attn_generic: value size %d above %d", Dv, 32 * AT_MAXV);
  JL_CHECK_ARG(ldk >= D && ldv >= Dv && window >= 0, "jl_attn_generic: bad pitch %d / %d or window %d", ldk, ldv, window);
  if (k_bs == 0 && k_hs == 0) { k_hs = (long long)T_cap * ldk; k_bs = k_hs * G; }
  if (v_bs == 0 && v_hs == 0) { v_hs = (long long)T_cap * ldv; v_bs = v_hs * G; }
  JL_CHECK_ARG(chunk >= 0 && (sink_logit == nullptr || sink), "jl_attn_generic: chunk %d, a sink logit without a sink", chunk);
  JL_CHECK_ARG(vcos == nullptr || (vsin != nullptr && Dv % 2 == 0 && v_max_pos >= 1 && (v_layout == 0 || v_layout == 1)),
               "jl_attn_generic: rotated values need both tables and an even Dv=%d", Dv);
  AttnParams p{B, S, H, G, D, Dv, T_cap, ldk, ldv, k_bs, k_hs, v_bs, v_hs, window, scale, cache_len, pad_left, gate, ldg, sink, out32,
               chunk, sink_logit, vcos, vsin, v_max_pos, v_layout};
  cudaStream_t st = (cudaStream_t)stream;
  if (S == 1 && scratch != nullptr && splits >= 1 && splits <= 64) {
    const int dp = ((D + 3) & ~3) + 4;
    const int rb = H / G < AS_WARPS * AS_RW ? H / G : AS_WARPS * AS_RW, nblk = (H / G + rb - 1) / rb;
    const size_t smem = (size_t)((rb + 32) * dp + 32 * ((Dv + 3) & ~3)) * sizeof(float);
    JL_CHECK_ARG(smem <= 200 * 1024, "jl_attn_generic: head sizes %d / %d do not fit the key tile", D, Dv);
#define JL_AS(NV_)                                                                                                   \
  JL_DISPATCH_DTYPE(dtype, {                                                                                         \
    if (smem > 48 * 1024)                                                                                            \
      JL_CUDA(cudaFuncSetAttribute(attn_split_kernel<T, NV_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    JL_LAUNCH_PDL((attn_split_kernel<T, NV_>), dim3(dim3(splits, G * nblk, B)), dim3(AS_WARPS * 32), smem, st, p, (const T*)q, (const T*)k_cache,   \
                                                                               (const T*)v_cache, scratch, splits);  \
  })
    const int nv = (Dv + 31) / 32;
    if (nv <= 1) JL_AS(1); else if (nv <= 2) JL_AS(2); else if (nv <= 4) JL_AS(4); else if (nv <= 8) JL_AS(8); else JL_AS(16);
#undef JL_AS
    JL_CUDA(cudaGetLastError());
      JL_DISPATCH_DTYPE(dtype, JL_LAUNCH_PDL(attn_merge_kernel<T>, dim3(dim3(H, B)), dim3(128), 0, st, p, scratch, splits, (T*)out));
  } else if (S == 1) {
    const size_t smem = (size_t)(D + 2 * AD_WARPS + AD_WARPS * Dv) * sizeof(float);
    JL_DISPATCH_DTYPE(dtype, JL_LAUNCH_PDL(attn_decode_kernel<T>, dim3(dim3(H, B)), dim3(AD_WARPS * 32), smem, st, p, (const T*)q, (const T*)k_cache,
                                                                                         (const T*)v_cache, (T*)out));
  } else {
    const int dp = ((D + 3) & ~3) + 4;
    const size_t smem = (size_t)((AR_QB + 32) * dp + 32 * ((Dv + 3) & ~3)) * sizeof(float);
    JL_CHECK_ARG(smem <= 200 * 1024, "jl_attn_generic: head sizes %d / %d do not fit the key tile", D, Dv);
#define JL_AR(NV_)                                                                                                  \
  JL_DISPATCH_DTYPE(dtype, {                                                                                        \
    if (smem > 48 * 1024)                                                                                           \
      JL_CUDA(cudaFuncSetAttribute(attn_rows_kernel<T, NV_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    JL_LAUNCH_PDL((attn_rows_kernel<T, NV_>), dim3(dim3((S + AR_QB - 1) / AR_QB, H, B)), dim3(AR_WARPS * 32), smem, st,                     \
        p, (const T*)q, (const T*)k_cache, (const T*)v_cache, (T*)out);                                             \
  })
    const int nv = (Dv + 31) / 32;
    if (nv <= 1) JL_AR(1); else if (nv <= 2) JL_AR(2); else if (nv <= 4) JL_AR(4); else if (nv <= 8) JL_AR(8); else JL_AR(16);
#undef JL_AR
  }
  JL_CUDA(cudaGetLastError());
  return JL_OK;
}

extern "C" JL_API int jl_attn_generic(const void* q, const void* k_cache, const void* v_cache, void* out, const float* gate, int ldg,
                                      const int* cache_len, const int* pad_left, int B, int S, int H, int G, int D, int Dv,
                                      int T_cap, float scale, float* scratch, int splits, int dtype, void* stream) {
  return attn_launch(q, k_cache, v_cache, out, gate, ldg, cache_len, pad_left, B, S, H, G, D, Dv, T_cap, D, Dv, 0, scale, scratch,
                     splits, dtype, stream);
}

extern "C" JL_API int jl_attn_windowed(const void* q, const void* k_cache, const void* v_cache, void* out, const int* cache_len,
                                       const int* pad_left, int B, int S, int H, int G, int D, int Dv, int T_cap, int ldk, int ldv,
                                       long long k_bs, long long k_hs, long long v_bs, long long v_hs, int window, float scale,
                                       float* scratch, int splits, int sink, float* out32, int dtype, void* stream) {
  JL_CHECK_ARG(out != nullptr || out32 != nullptr, "jl_attn_windowed: no output");
  return attn_launch(q, k_cache, v_cache, out, nullptr, 0, cache_len, pad_left, B, S, H, G, D, Dv, T_cap, ldk, ldv, window, scale,
                     scratch, splits, dtype, stream, k_bs, k_hs, v_bs, v_hs, sink, out32);
}

// Everything the attention kernels take: gate (fp32 pre-activation, column h of row m, pitch ldg), window, blocks of `chunk`
// positions, a sink (score 0, or sink_logit[h]), values cached rotated (v_cos / v_sin [v_max_pos][Dv/2], pairs as v_layout).
extern "C" JL_API int jl_attn_masked(const void* q, const void* k_cache, const void* v_cache, void* out, const float* gate, int ldg,
                                     const int* cache_len, const int* pad_left, int B, int S, int H, int G, int D, int Dv, int T_cap,
                                     int ldk, int ldv, long long k_bs, long long k_hs, long long v_bs, long long v_hs, int window,
                                     int chunk, float scale, float* scratch, int splits, int sink, const float* sink_logit,
                                     const float* v_cos, const float* v_sin, int v_max_pos, int v_layout, float* out32, int dtype,
                                     void* stream) {
  JL_CHECK_ARG(out != nullptr || out32 != nullptr, "jl_attn_masked: no output");
  return attn_launch(q, k_cache, v_cache, out, gate, ldg, cache_len, pad_left, B, S, H, G, D, Dv, T_cap, ldk, ldv, window, scale,
                     scratch, splits, dtype, stream, k_bs, k_hs, v_bs, v_hs, sink, out32, chunk, sink_logit, v_cos, v_sin, v_max_pos,
                     v_layout);
}

extern "C" JL_API int jl_latent_prep(const float* y, int ldy, int q_off, int q_rank, int kv_off, int kv_rank, int rot_dim, int rot,
                                     int layout, const void* wq_norm, const void* wkv_norm, void* cq, void* cache,
                                     const float* cos_t, const float* sin_t, int max_pos, float eps, const int* cache_len,
                                     const int* pad_left, int B, int S, int T_cap, void* c_out, void* kr_out, int dtype,
                                     void* stream) {
  JL_CHECK_ARG(B >= 1 && S >= 1 && q_rank >= 0 && kv_rank >= 1 && rot_dim >= 0, "jl_latent_prep: bad shape");
  JL_CHECK_ARG(rot >= 0 && rot <= rot_dim && rot % 2 == 0, "jl_latent_prep: rot=%d must be even and <= rot_dim=%d", rot, rot_dim);
  JL_CHECK_ARG(layout == 0 || layout == 1, "jl_latent_prep: layout %d", layout);
  LatentPrepParams p{y, ldy, q_off, q_rank, kv_off, kv_rank, rot_dim, rot, layout, cos_t, sin_t, max_pos, eps, B, S, T_cap,
                     cache_len, pad_left, c_out, kr_out};
  JL_DISPATCH_DTYPE(dtype, JL_LAUNCH_PDL(latent_prep_kernel<T>, dim3(B * S), dim3(128), 0, (cudaStream_t)stream, p, (const T*)wq_norm,
                                         (const T*)wkv_norm, (T*)cq, (T*)cache));
  JL_CUDA(cudaGetLastError());
  return JL_OK;
}

extern "C" JL_API int jl_rotary_slice(const void* in, int ldi, int in_hs, int in_off, void* out, int ldo, int out_hs, int out_off,
                                      int H, int n, int rot, int layout, const float* cos_t, const float* sin_t, int max_pos,
                                      const int* cache_len, const int* pad_left, int B, int S, int dtype, void* stream) {
  JL_CHECK_ARG(B >= 1 && S >= 1 && H >= 1 && n >= 1, "jl_rotary_slice: bad shape");
  JL_CHECK_ARG(rot >= 0 && rot <= n && rot % 2 == 0 && (layout == 0 || layout == 1), "jl_rotary_slice: rot=%d of n=%d, layout %d", rot,
               n, layout);
  JL_DISPATCH_DTYPE(dtype, JL_LAUNCH_PDL(rotary_slice_kernel<T>, dim3(B * S), dim3(128), 0, (cudaStream_t)stream, (const T*)in, ldi,
                                         in_hs, in_off, (T*)out, ldo, out_hs, out_off, H, n, rot, layout, cos_t, sin_t, max_pos,
                                         cache_len, pad_left, S));
  JL_CUDA(cudaGetLastError());
  return JL_OK;
}

extern "C" JL_API int jl_head_gate(void* out, const float* gate, int ldg, int M, int H, int Dv, int dtype, void* stream) {
  JL_CHECK_ARG(M >= 1 && H >= 1 && Dv >= 1, "jl_head_gate: bad shape");
  const size_t total = (size_t)M * H * Dv;
  const int blocks = (int)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
  JL_DISPATCH_DTYPE(dtype, JL_LAUNCH_PDL(head_gate_kernel<T>, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, (T*)out, gate, ldg, M, H, Dv));
  JL_CUDA(cudaGetLastError());
  return JL_OK;
}
