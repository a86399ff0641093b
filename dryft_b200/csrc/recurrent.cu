// Mixers whose memory is a fixed-size 32-bit state per sequence instead of cached keys: a step runs the tokens it is
// given from the state the step before left, and leaves the state for the next (one token, a prompt, or a piece of one).
//
// retention_scan     linear attention with one fixed decay per head, no softmax and no denominator.  Per head, with the
//                    rotated query q_t, the rotated key k_t times k_scale, and the value v_t of token t:
//                        S_t = decay * S_(t-1) + k_t v_t^T          S [dim, vdim], 32-bit
//                        o_t = S_t^T q_t ;  o_t <- o_t / sqrt(mean(o_t^2) + eps) ;  out = T( o_t * silu(g_t) )
//                    One block per (sequence, head) walks the sequence's tokens in order with S in shared memory.
//                    q | k | v | g are columns of one projection row (offsets given); the rotation pairs entry i with
//                    entry i + R/2 of the first R entries (angle = position * inv_freq[i]; see sincos_split below).
//
// rglru_gates        the input side of a real-gated linear recurrent unit over C channels in `blocks` equal groups:
//                        x_t  = xproj_t + x_bias                                   (a column range of the projection row)
//                        u_t  = conv_b + sum_j conv_w[c][j] * x_(t - (taps-1) + j)    (causal, per channel; inputs before
//                               the step come from the sequence's stored tail, zeros before the sequence's start)
//                        r_t  = sigmoid(Wa[b] u_t,b + ba) ;  i_t = sigmoid(Wi[b] u_t,b + bi)     (per group b, 32-bit)
//                        log a_t = -c * r_t * softplus(lam) ;  a_t = exp(log a_t)
//                        b_t  = sqrt(1 - a_t^2) * i_t * u_t          (1 - a^2 as -expm1(2 log a): no cancellation)
//                    leaves e_t = a_t - 1 (as expm1(log a_t): a decay of 0.9999 keeps its distance from one, which a
//                    32-bit a_t would round to one part in 2,000) and b_t, [tokens, C] in 32-bit.
// rglru_scan         S_t = S_(t-1) + (e_t * S_(t-1) + b_t) per channel, out_t = T( S_t * gelu_tanh(yproj_t + y_bias) ), then the new
//                    state and the new tail (the last taps-1 inputs) are stored.  Time is walked by eight warps at once,
//                    each folding its own steps first (see the kernel).
//
// Everything that enters a recurrence is 32-bit whatever the activation type T.  Sizes are runtime arguments of any value
// (shared memory permitting).  No block waits on another.
#include "common.cuh"
#include <math.h>

namespace {
constexpr int RT_THREADS = 256;

// sin and cos of  pos * (f_hi + f_lo)  for a rotary position: the product is formed in 32-bit, and what its rounding
// drops (recovered exactly with one fused multiply-add) plus the low half of the frequency are applied as a first-order
// turn, so the angle is as good as the frequency pair instead of losing one part in 2^24 of a large angle.  f_lo = 0 gives
// the plain 32-bit angle to within that correction.
__device__ __forceinline__ void sincos_split(float pos, float f_hi, float f_lo, float* sn, float* cs) {
  const float a = pos * f_hi;
  const float e = fmaf(pos, f_hi, -a) + pos * f_lo;
  float s, c;
  sincosf(a, &s, &c);
  *sn = fmaf(e, c, s);
  *cs = fmaf(-e, s, c);
}


template <typename T>
__global__ void __launch_bounds__(RT_THREADS) retention_scan_kernel(
    const T* __restrict__ proj, int ld, int q_off, int k_off, int v_off, int g_off, const int* __restrict__ cu_q,
    const int* __restrict__ seq_slot, const int* __restrict__ tok_pos, const float* __restrict__ inv_freq,
    const float* __restrict__ inv_freq_lo, int rot, const double* __restrict__ decay, float* __restrict__ state,
    T* __restrict__ out, int H, int dim, int vdim, float k_scale, float eps) {
  extern __shared__ __align__(16) float smem[];
  const int b = blockIdx.x, hd = blockIdx.y;
  const int slot = seq_slot[b];
  if (slot < 0) return;
  const int n0 = cu_q[b], n1 = cu_q[b + 1];
  const int cols = vdim < RT_THREADS ? vdim : RT_THREADS;   // threads side by side over the value index
  const int groups = RT_THREADS / cols;                      // groups of them over the key index
  float* S = smem;                        // [dim][vdim]
  float* qs = S + (size_t)dim * vdim;     // [dim]
  float* ks = qs + dim;                   // [dim]
  float* vs = ks + dim;                   // [vdim]
  float* red = vs + vdim;                 // [groups][vdim]
  __shared__ float scratch[33];
  const int tid = threadIdx.x;
  float* Sg = state + ((size_t)slot * H + hd) * dim * vdim;
  for (int i = tid; i < dim * vdim; i += RT_THREADS) S[i] = Sg[i];
  // the decay as a 32-bit value and what that drops: compounded over hundreds of tokens, one part in 2^24 of it shows
  const float dec = (float)decay[hd], dec_lo = (float)(decay[hd] - (double)dec);
  const int half = rot >> 1;
  const int cv = tid % cols, rg = tid / cols;
  const bool active = rg < groups;
  for (int n = n0; n < n1; ++n) {
    const T* row = proj + (size_t)n * ld;
    const float pos = (float)tok_pos[n];
    __syncthreads();   // the token before is done with qs / ks / vs / red
    for (int i = tid; i < 2 * dim; i += RT_THREADS) {
      const bool is_k = i >= dim;
      const int d = is_k ? i - dim : i;
      const T* src = row + (is_k ? k_off : q_off) + hd * dim;
      float val = to_f32<T>(src[d]);
      if (d < rot) {
        const int j = d < half ? d : d - half;
        const float other = to_f32<T>(src[d < half ? d + half : d - half]);
        float sn, cs;
        sincos_split(pos, inv_freq[j], inv_freq_lo ? inv_freq_lo[j] : 0.f, &sn, &cs);
        val = d < half ? val * cs - other * sn : val * cs + other * sn;
      }
      if (is_k) ks[d] = val * k_scale; else qs[d] = val;
    }
    for (int i = tid; i < vdim; i += RT_THREADS) vs[i] = to_f32<T>(row[v_off + hd * vdim + i]);
    __syncthreads();
    if (active) {
      for (int v = cv; v < vdim; v += cols) {
        const float vv = vs[v];
        float acc = 0.f;
        for (int d = rg; d < dim; d += groups) {
          const float old = S[d * vdim + v];
          const float s = fmaf(dec, old, fmaf(dec_lo, old, ks[d] * vv));
          S[d * vdim + v] = s;
          acc = fmaf(s, qs[d], acc);
        }
        red[rg * vdim + v] = acc;
      }
    }
    __syncthreads();
    float ss = 0.f;
    for (int v = tid; v < vdim; v += RT_THREADS) {
      float o = 0.f;
      for (int g = 0; g < groups; ++g) o += red[g * vdim + v];
      vs[v] = o;          // vs is free again: every thread passed the barrier above
      ss = fmaf(o, o, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / (float)vdim + eps);
    for (int v = tid; v < vdim; v += RT_THREADS) {
      const float g = to_f32<T>(row[g_off + hd * vdim + v]);
      out[(size_t)n * H * vdim + hd * vdim + v] = from_f32<T>(vs[v] * inv * (g / (1.f + expf(-g))));
    }
  }
  __syncthreads();
  for (int i = tid; i < dim * vdim; i += RT_THREADS) Sg[i] = S[i];
}

// ---------------------------------------------------------------------------------------------------------------------
// The same retention for steps of many tokens, in chunks of CH tokens so that the work is matrix-shaped and spread over
// (chunk, head) blocks instead of walked token by token.  For chunk g of a sequence, L tokens long, with S_in the state
// before it (w = decay):
//     D_g   = sum_j w^(L-1-j) k_j v_j^T                                   retention_chunk_state   (every chunk at once)
//     S_in  of every chunk, by S <- w^L S + D_g in order                   retention_chunk_prefix  (elementwise; the
//                                                                          sequence's stored state is read and updated)
//     o_i   = w^(i+1) S_in^T q_i + sum_(j<=i) w^(i-j) (q_i . k_j) v_j       retention_chunk_out     (every chunk at once),
// then the same norm and gate as above.  Powers of the decay come from a table made in 64-bit.  Chunk g of the step is
// found from cu_q: sequence b has ceil(len_b / CH) chunks, numbered in sequence order after those of the sequences before.
constexpr int CH = 64;
constexpr int CK_THREADS = 256;

__device__ __forceinline__ bool locate_chunk(const int* __restrict__ cu_q, int n_seqs, int g, int* b_out, int* k_out) {
  int base = 0;
  for (int b = 0; b < n_seqs; ++b) {
    const int nc = (cu_q[b + 1] - cu_q[b] + CH - 1) / CH;
    if (g < base + nc) { *b_out = b; *k_out = g - base; return true; }
    base += nc;
  }
  return false;
}

// rows [L][ld] of shared memory <- the rotated (and scaled) head vectors of L tokens; columns dim..ld-1 are zeroed
template <typename T>
__device__ __forceinline__ void load_rotated(float* dst, int ld, const T* __restrict__ proj, int ldp, int col0, int n_first, int L,
                                             int dim, int rot, const float* __restrict__ inv_freq,
                                             const float* __restrict__ inv_freq_lo, const int* __restrict__ tok_pos, float scale) {
  const int half = rot >> 1;
  for (int idx = threadIdx.x; idx < L * ld; idx += CK_THREADS) {
    const int t = idx / ld, d = idx % ld;
    float val = 0.f;
    if (d < dim) {
      const T* src = proj + (size_t)(n_first + t) * ldp + col0;
      val = to_f32<T>(src[d]);
      if (d < rot) {
        const int j = d < half ? d : d - half;
        const float other = to_f32<T>(src[d < half ? d + half : d - half]);
        float sn, cs;
        sincos_split((float)tok_pos[n_first + t], inv_freq[j], inv_freq_lo ? inv_freq_lo[j] : 0.f, &sn, &cs);
        val = d < half ? val * cs - other * sn : val * cs + other * sn;
      }
      val *= scale;
    }
    dst[t * ld + d] = val;
  }
}

template <typename T>
__global__ void __launch_bounds__(CK_THREADS) retention_chunk_state_kernel(
    const T* __restrict__ proj, int ld, int k_off, int v_off, const int* __restrict__ cu_q, const int* __restrict__ seq_slot,
    int n_seqs, const int* __restrict__ tok_pos, const float* __restrict__ inv_freq, const float* __restrict__ inv_freq_lo,
    int rot, const double* __restrict__ decay, float* __restrict__ sbuf, int H, int dim, int vdim, float k_scale) {
  extern __shared__ __align__(16) float smem[];
  __shared__ int loc[3];
  const int g = blockIdx.x, hd = blockIdx.y;
  if (threadIdx.x == 0) {
    int b = 0, k = 0;
    loc[2] = locate_chunk(cu_q, n_seqs, g, &b, &k) && seq_slot[b] >= 0;
    loc[0] = b; loc[1] = k;
  }
  __syncthreads();
  if (!loc[2]) return;
  const int b = loc[0], n_first = cu_q[b] + loc[1] * CH, L = min(CH, cu_q[b + 1] - n_first);
  const int dP = (dim + 7) & ~7, vP = (vdim + 7) & ~7;
  float* ks = smem;                 // [CH][dP]
  float* vs = ks + CH * dP;         // [CH][vP]
  float* pw = vs + CH * vP;         // [CH + 1]
  for (int i = threadIdx.x; i <= CH; i += CK_THREADS) pw[i] = (float)pow(decay[hd], (double)i);
  load_rotated<T>(ks, dP, proj, ld, k_off + hd * dim, n_first, L, dim, rot, inv_freq, inv_freq_lo, tok_pos, k_scale);
  for (int idx = threadIdx.x; idx < L * vP; idx += CK_THREADS) {
    const int t = idx / vP, v = idx % vP;
    vs[idx] = v < vdim ? to_f32<T>(proj[(size_t)(n_first + t) * ld + v_off + hd * vdim + v]) : 0.f;
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < L * dP; idx += CK_THREADS) ks[idx] *= pw[L - 1 - idx / dP];
  __syncthreads();
  float* dst = sbuf + ((size_t)g * H + hd) * dim * vdim;
  const int tv = vP / 8, n_tiles = (dP / 8) * tv;
  for (int tile = threadIdx.x; tile < n_tiles; tile += CK_THREADS) {
    const int d0 = (tile / tv) * 8, v0 = (tile % tv) * 8;
    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int c = 0; c < 8; ++c) acc[i][c] = 0.f;
    for (int j = 0; j < L; ++j) {
      const float4 k0 = *reinterpret_cast<const float4*>(ks + j * dP + d0), k1 = *reinterpret_cast<const float4*>(ks + j * dP + d0 + 4);
      const float4 u0 = *reinterpret_cast<const float4*>(vs + j * vP + v0), u1 = *reinterpret_cast<const float4*>(vs + j * vP + v0 + 4);
      const float kv[8] = {k0.x, k0.y, k0.z, k0.w, k1.x, k1.y, k1.z, k1.w}, vv[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int c = 0; c < 8; ++c) acc[i][c] = fmaf(kv[i], vv[c], acc[i][c]);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int c = 0; c < 8; ++c)
        if (d0 + i < dim && v0 + c < vdim) dst[(size_t)(d0 + i) * vdim + v0 + c] = acc[i][c];
  }
}

__global__ void retention_chunk_prefix_kernel(const int* __restrict__ cu_q, const int* __restrict__ seq_slot,
                                              const double* __restrict__ decay, float* __restrict__ sbuf,
                                              float* __restrict__ state, int H, int per_head) {
  const int b = blockIdx.x, hd = blockIdx.y;
  const int e = blockIdx.z * blockDim.x + threadIdx.x;
  const int slot = seq_slot[b];
  if (slot < 0 || e >= per_head) return;
  int base = 0;
  for (int bb = 0; bb < b; ++bb) base += (cu_q[bb + 1] - cu_q[bb] + CH - 1) / CH;
  const int q = cu_q[b + 1] - cu_q[b];
  float* sp = state + ((size_t)slot * H + hd) * per_head + e;
  float S = *sp;
  const double w = decay[hd];
  const float w_full = (float)pow(w, (double)CH);
  const int n_chunks = (q + CH - 1) / CH;
  for (int k0 = 0; k0 < n_chunks; k0 += 8) {   // eight chunk sums asked for at once, then folded in order
    float delta[8];
#pragma unroll
    for (int u = 0; u < 8; ++u)
      if (k0 + u < n_chunks) delta[u] = __ldcs(sbuf + ((size_t)(base + k0 + u) * H + hd) * per_head + e);
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      if (k0 + u < n_chunks) {
        sbuf[((size_t)(base + k0 + u) * H + hd) * per_head + e] = S;   // the state the chunk starts from
        const int L = min(CH, q - (k0 + u) * CH);
        S = fmaf(L == CH ? w_full : (float)pow(w, (double)L), S, delta[u]);
      }
    }
  }
  *sp = S;
}

template <typename T>
__global__ void __launch_bounds__(CK_THREADS) retention_chunk_out_kernel(
    const T* __restrict__ proj, int ld, int q_off, int k_off, int v_off, int g_off, const int* __restrict__ cu_q,
    const int* __restrict__ seq_slot, int n_seqs, const int* __restrict__ tok_pos, const float* __restrict__ inv_freq,
    const float* __restrict__ inv_freq_lo, int rot, const double* __restrict__ decay, const float* __restrict__ sbuf,
    T* __restrict__ out, int H, int dim, int vdim, float k_scale, float eps) {
  extern __shared__ __align__(16) float smem[];
  __shared__ int loc[3];
  const int g = blockIdx.x, hd = blockIdx.y;
  if (threadIdx.x == 0) {
    int b = 0, k = 0;
    loc[2] = locate_chunk(cu_q, n_seqs, g, &b, &k) && seq_slot[b] >= 0;
    loc[0] = b; loc[1] = k;
  }
  __syncthreads();
  if (!loc[2]) return;
  const int b = loc[0], n_first = cu_q[b] + loc[1] * CH, L = min(CH, cu_q[b + 1] - n_first);
  const int dQ = ((dim + 3) & ~3) + 1;           // odd row length: rows of q and k fall on different banks
  const int vP = (vdim + 3) & ~3;
  const int stage = max(CH * dQ, CH * vP);       // the q rows' place also holds the outputs before the norm
  float* vs = smem;                  // [CH][vP]            (16-byte rows first)
  float* slab = vs + CH * vP;        // [SLAB][vP]          a slab of the state the chunk starts from
  float* qs = slab + 16 * vP;        // [CH][dQ], later o [CH][vP]
  float* ks = qs + stage;            // [CH][dQ]
  float* A = ks + CH * dQ;           // [CH][CH + 1]
  float* pw = A + CH * (CH + 1);     // [CH + 1]
  for (int i = threadIdx.x; i <= CH; i += CK_THREADS) pw[i] = (float)pow(decay[hd], (double)i);
  load_rotated<T>(qs, dQ, proj, ld, q_off + hd * dim, n_first, L, dim, rot, inv_freq, inv_freq_lo, tok_pos, 1.f);
  load_rotated<T>(ks, dQ, proj, ld, k_off + hd * dim, n_first, L, dim, rot, inv_freq, inv_freq_lo, tok_pos, k_scale);
  for (int idx = threadIdx.x; idx < CH * vP; idx += CK_THREADS) {
    const int t = idx / vP, v = idx % vP;
    vs[idx] = (t < L && v < vdim) ? to_f32<T>(proj[(size_t)(n_first + t) * ld + v_off + hd * vdim + v]) : 0.f;
  }
  for (int idx = threadIdx.x + L * dQ; idx < CH * dQ; idx += CK_THREADS) { qs[idx] = 0.f; ks[idx] = 0.f; }   // rows behind the chunk
  __syncthreads();
  // A[i][j] = w^(i-j) q_i . k_j  for j <= i, else 0: 4 x 4 outputs a thread
  for (int tile = threadIdx.x; tile < (CH / 4) * (CH / 4); tile += CK_THREADS) {
    const int i0 = (tile / (CH / 4)) * 4, j0 = (tile % (CH / 4)) * 4;
    float acc[4][4];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[r][c] = 0.f;
    if (j0 <= i0 + 3 && i0 < L) {
      for (int d = 0; d < dim; ++d) {
        float qv[4], kv[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) { qv[r] = qs[(i0 + r) * dQ + d]; kv[r] = ks[(j0 + r) * dQ + d]; }
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
          for (int c = 0; c < 4; ++c) acc[r][c] = fmaf(qv[r], kv[c], acc[r][c]);
      }
    }
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int i = i0 + r, j = j0 + c;
        A[i * (CH + 1) + j] = j <= i ? acc[r][c] * pw[i - j] : 0.f;
      }
  }
  __syncthreads();
  // o = w^(i+1) (q S_in) + A v : 8 rows x 4 columns a thread, kept in registers until every thread has read q.
  // S_in comes through shared memory in slabs of SLAB key rows; the next slab is asked for (into registers) before the
  // current one is multiplied, so its trip from L2 hides behind the products.
  const float* S_in = sbuf + ((size_t)g * H + hd) * dim * vdim;
  const int tv = vP / 4, n_tiles = (CH / 8) * tv;
  constexpr int MAX_TILES = 4;       // tiles a thread may hold (value sizes up to 512)
  constexpr int SLAB = 16, SLAB_LOADS = (SLAB * 512 / 4 + CK_THREADS - 1) / CK_THREADS;   // float4 pieces a thread fetches
  float acc[MAX_TILES][8][4];
#pragma unroll
  for (int t = 0; t < MAX_TILES; ++t)
#pragma unroll
    for (int r = 0; r < 8; ++r)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[t][r][c] = 0.f;
  const int slab_vec = SLAB * tv;    // float4 pieces of a slab [SLAB][vP]
  const bool rows_vec = (vdim & 3) == 0;
  float4 pre[SLAB_LOADS];
  auto fetch = [&](int d0) {
#pragma unroll
    for (int u = 0; u < SLAB_LOADS; ++u) {
      const int idx = threadIdx.x + u * CK_THREADS;
      pre[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (idx < slab_vec) {
        const int dd = d0 + idx / tv, v = (idx % tv) * 4;
        if (dd < dim) {
          const float* src = S_in + (size_t)dd * vdim + v;
          if (rows_vec) pre[u] = __ldg(reinterpret_cast<const float4*>(src));
          else pre[u] = make_float4(v < vdim ? __ldg(src) : 0.f, v + 1 < vdim ? __ldg(src + 1) : 0.f,
                                    v + 2 < vdim ? __ldg(src + 2) : 0.f, v + 3 < vdim ? __ldg(src + 3) : 0.f);
        }
      }
    }
  };
  fetch(0);
  for (int d0 = 0; d0 < dim; d0 += SLAB) {
    __syncthreads();   // the slab before is used up
#pragma unroll
    for (int u = 0; u < SLAB_LOADS; ++u) {
      const int idx = threadIdx.x + u * CK_THREADS;
      if (idx < slab_vec) *reinterpret_cast<float4*>(slab + (size_t)idx * 4) = pre[u];
    }
    __syncthreads();
    if (d0 + SLAB < dim) fetch(d0 + SLAB);
    const int d_end = min(SLAB, dim - d0);
    int n_mine = 0;
    for (int tile = threadIdx.x; tile < n_tiles && n_mine < MAX_TILES; tile += CK_THREADS, ++n_mine) {
      const int i0 = (tile / tv) * 8, v0 = (tile % tv) * 4;
      if (i0 >= L) continue;
      float (*a)[4] = acc[n_mine];
      for (int dd = 0; dd < d_end; ++dd) {
        const float4 sv = *reinterpret_cast<const float4*>(slab + (size_t)dd * vP + v0);
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          const float qv = qs[(i0 + r) * dQ + d0 + dd];
          a[r][0] = fmaf(qv, sv.x, a[r][0]); a[r][1] = fmaf(qv, sv.y, a[r][1]);
          a[r][2] = fmaf(qv, sv.z, a[r][2]); a[r][3] = fmaf(qv, sv.w, a[r][3]);
        }
      }
    }
  }
  {
    int n_mine = 0;
    for (int tile = threadIdx.x; tile < n_tiles && n_mine < MAX_TILES; tile += CK_THREADS, ++n_mine) {
      const int i0 = (tile / tv) * 8, v0 = (tile % tv) * 4;
      if (i0 >= L) continue;
      float (*a)[4] = acc[n_mine];
#pragma unroll
      for (int r = 0; r < 8; ++r)
#pragma unroll
        for (int c = 0; c < 4; ++c) a[r][c] *= pw[i0 + r + 1];
      const int j_end = min(L, i0 + 8);
      for (int j = 0; j < j_end; ++j) {
        const float4 vv = *reinterpret_cast<const float4*>(vs + (size_t)j * vP + v0);
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          const float av = A[(i0 + r) * (CH + 1) + j];
          a[r][0] = fmaf(av, vv.x, a[r][0]); a[r][1] = fmaf(av, vv.y, a[r][1]);
          a[r][2] = fmaf(av, vv.z, a[r][2]); a[r][3] = fmaf(av, vv.w, a[r][3]);
        }
      }
    }
  }
  __syncthreads();   // q is read by all: its place takes the outputs
  int n_mine = 0;
  for (int tile = threadIdx.x; tile < n_tiles && n_mine < MAX_TILES; tile += CK_THREADS, ++n_mine) {
    const int i0 = (tile / tv) * 8, v0 = (tile % tv) * 4;
#pragma unroll
    for (int r = 0; r < 8; ++r)
#pragma unroll
      for (int c = 0; c < 4; ++c) qs[(i0 + r) * vP + v0 + c] = acc[n_mine][r][c];
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = warp; i < L; i += CK_THREADS / 32) {
    float ss = 0.f;
    for (int v = lane; v < vdim; v += 32) { const float o = qs[i * vP + v]; ss = fmaf(o, o, ss); }
    ss = warp_sum(ss);
    const float inv = 1.f / sqrtf(ss / (float)vdim + eps);
    const size_t n = (size_t)(n_first + i);
    for (int v = lane; v < vdim; v += 32) {
      const float gv = to_f32<T>(proj[n * ld + g_off + hd * vdim + v]);
      out[n * H * vdim + hd * vdim + v] = from_f32<T>(qs[i * vP + v] * inv * (gv / (1.f + expf(-gv))));
    }
  }
}

constexpr int GT = 8;          // tokens per block of rglru_gates
constexpr int G_THREADS = 256;

template <typename T>
__global__ void __launch_bounds__(G_THREADS) rglru_gates_kernel(
    const T* __restrict__ proj, int ld, int x_off, const float* __restrict__ x_bias, const int* __restrict__ tok_slot,
    const float* __restrict__ conv_w, const float* __restrict__ conv_b, int taps, const float* __restrict__ tail,
    const float* __restrict__ w_gates, const float* __restrict__ b_a, const float* __restrict__ b_i,
    const float* __restrict__ sp_lam, float c_mult, float* __restrict__ a_out, float* __restrict__ b_out, int n_tokens,
    int C, int nb) {
  extern __shared__ __align__(16) float u_s[];   // [GT][nb]
  const int n0 = blockIdx.x * GT, blk = blockIdx.y, c0 = blk * nb;
  const int K1 = taps - 1;
  for (int idx = threadIdx.x; idx < GT * nb; idx += G_THREADS) {
    const int t = idx / nb, cc = idx % nb, n = n0 + t, c = c0 + cc;
    float u = 0.f;
    if (n < n_tokens) {
      const int slot = tok_slot[n];
      if (slot >= 0) {
        int avail = 0;   // tokens of the same sequence right before this one in the step, up to taps-1
        while (avail < K1 && n - avail - 1 >= 0 && tok_slot[n - avail - 1] == slot) ++avail;
        u = conv_b[c];
        for (int j = 0; j < taps; ++j) {
          const int back = K1 - j;
          float xv;
          if (back <= avail) xv = to_f32<T>(proj[(size_t)(n - back) * ld + x_off + c]) + x_bias[c];
          else xv = tail[((size_t)slot * K1 + (K1 - back + avail)) * C + c];
          u = fmaf(conv_w[(size_t)c * taps + j], xv, u);
        }
      }
    }
    u_s[t * nb + cc] = u;
  }
  __syncthreads();
  const float* wg = w_gates + (size_t)blk * nb * 2 * nb;   // [k][2][o]
  for (int o = threadIdx.x; o < nb; o += G_THREADS) {
    float ar[GT], ai[GT];
    const float ba = b_a[c0 + o], bi = b_i[c0 + o];
#pragma unroll
    for (int t = 0; t < GT; ++t) { ar[t] = ba; ai[t] = bi; }
    for (int k = 0; k < nb; ++k) {
      const float wr = wg[((size_t)k * 2) * nb + o], wi = wg[((size_t)k * 2 + 1) * nb + o];
#pragma unroll
      for (int t = 0; t < GT; ++t) {
        const float uv = u_s[t * nb + k];
        ar[t] = fmaf(wr, uv, ar[t]);
        ai[t] = fmaf(wi, uv, ai[t]);
      }
    }
    const float sp = sp_lam[c0 + o];
#pragma unroll
    for (int t = 0; t < GT; ++t) {
      const int n = n0 + t;
      if (n >= n_tokens) break;
      const float r = 1.f / (1.f + expf(-ar[t])), ig = 1.f / (1.f + expf(-ai[t]));
      const float log_a = -c_mult * r * sp;
      a_out[(size_t)n * C + c0 + o] = expm1f(log_a);   // a - 1: a decay close to one keeps its distance from one
      b_out[(size_t)n * C + c0 + o] = sqrtf(-expm1f(2.f * log_a)) * ig * u_s[t * nb + o];
    }
  }
}

__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// A block takes 32 channels (a lane each) of one sequence and walks time in pieces of SCAN_WARPS * SCAN_SEG steps: every
// warp folds its own SCAN_SEG steps into one (E, B) pair  S_out = S_in + (E * S_in + B),  the pairs of the warps before it give its
// S_in, and it walks its steps again for the outputs -- 2 * SCAN_SEG + SCAN_WARPS dependent steps a piece instead of
// SCAN_WARPS * SCAN_SEG, with every warp's loads in flight at once.
constexpr int SCAN_WARPS = 8, SCAN_SEG = 16;

template <typename T>
__global__ void __launch_bounds__(SCAN_WARPS * 32) rglru_scan_kernel(
    const T* __restrict__ proj, int ld, int y_off, const float* __restrict__ y_bias, int x_off,
    const float* __restrict__ x_bias, const int* __restrict__ cu_q, const int* __restrict__ seq_slot,
    const float* __restrict__ a_in, const float* __restrict__ b_in, float* __restrict__ state, float* __restrict__ tail,
    int taps, T* __restrict__ out, int C) {
  __shared__ float As[SCAN_WARPS][32], Bs[SCAN_WARPS][32], carry[32];
  const int b = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c = blockIdx.y * 32 + lane;
  const int slot = seq_slot[b];
  if (slot < 0) return;
  const bool on = c < C;
  const int n0 = cu_q[b], n1 = cu_q[b + 1];
  if (warp == 0) carry[lane] = on ? state[(size_t)slot * C + c] : 0.f;
  const float yb = on ? y_bias[c] : 0.f;
  __syncthreads();
  for (int t0 = n0; t0 < n1; t0 += SCAN_WARPS * SCAN_SEG) {
    const int first = t0 + warp * SCAN_SEG;
    float av[SCAN_SEG], bv[SCAN_SEG], yv[SCAN_SEG];
#pragma unroll
    for (int i = 0; i < SCAN_SEG; ++i) {
      const int n = first + i;
      const bool ok = on && n < n1;
      av[i] = ok ? a_in[(size_t)n * C + c] : 0.f;      // a - 1; steps behind the end change nothing
      bv[i] = ok ? b_in[(size_t)n * C + c] : 0.f;
      yv[i] = ok ? to_f32<T>(proj[(size_t)n * ld + y_off + c]) : 0.f;
    }
    // with e = a - 1:  S <- S + (e S + b);  two steps (E1, B1) then (e, b) compose to  E = E1 + e + E1 e,  B = B1 + (e B1 + b)
    float E = 0.f, B = 0.f;
#pragma unroll
    for (int i = 0; i < SCAN_SEG; ++i) { B += fmaf(av[i], B, bv[i]); E = fmaf(E, av[i], E + av[i]); }
    As[warp][lane] = E;
    Bs[warp][lane] = B;
    __syncthreads();
    float S = carry[lane];
    for (int w = 0; w < warp; ++w) S += fmaf(As[w][lane], S, Bs[w][lane]);
#pragma unroll
    for (int i = 0; i < SCAN_SEG; ++i) {
      const int n = first + i;
      S += fmaf(av[i], S, bv[i]);
      if (on && n < n1) out[(size_t)n * C + c] = from_f32<T>(S * gelu_tanh_f(yv[i] + yb));
    }
    __syncthreads();          // every warp has read the carry
    if (warp == SCAN_WARPS - 1) carry[lane] = S;
    __syncthreads();
  }
  if (warp != 0 || !on) return;
  state[(size_t)slot * C + c] = carry[lane];
  const int K1 = taps - 1, q = n1 - n0;
  const float xb = x_bias[c];
  for (int j = 0; j < K1; ++j) {   // ascending: an old entry is read before the entry below it is overwritten
    const int idx = q - K1 + j;
    float* dst = tail + ((size_t)slot * K1 + j) * C + c;
    if (idx >= 0) *dst = to_f32<T>(proj[(size_t)(n0 + idx) * ld + x_off + c]) + xb;
    else *dst = tail[((size_t)slot * K1 + j + q) * C + c];
  }
}

template <typename K> int opt_in_smem(K kernel, size_t bytes) {
  if (bytes > 200 * 1024) return DRYFT_ERR_UNSUPPORTED;
  if (bytes > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return (int)e;
  }
  return 0;
}
}  // namespace

DRYFT_API int dryft_retention_scan(int is_bf16, const void* proj, int ld, int q_off, int k_off, int v_off, int g_off,
                                   const int* cu_q, const int* seq_slot, const int* tok_pos, const float* inv_freq,
                                   const float* inv_freq_lo, int rot, const double* decay, float* state, void* out, int n_seqs, int H, int dim, int vdim,
                                   float k_scale, float eps, cudaStream_t st) {
  if (n_seqs <= 0) return 0;
  if (H <= 0 || dim <= 0 || vdim <= 0 || rot < 0 || rot > dim || (rot & 1) || H > 65535) return DRYFT_ERR_UNSUPPORTED;
  typedef __nv_bfloat16 bf;
  const int cols = vdim < RT_THREADS ? vdim : RT_THREADS, groups = RT_THREADS / cols;
  const size_t smem = sizeof(float) * ((size_t)dim * vdim + 2 * (size_t)dim + vdim + (size_t)groups * vdim);
  int rc = is_bf16 ? opt_in_smem(retention_scan_kernel<bf>, smem) : opt_in_smem(retention_scan_kernel<float>, smem);
  if (rc) return rc;
  dim3 grid(n_seqs, H);
  if (is_bf16)
    retention_scan_kernel<bf><<<grid, RT_THREADS, smem, st>>>((const bf*)proj, ld, q_off, k_off, v_off, g_off, cu_q, seq_slot, tok_pos,
                                                              inv_freq, inv_freq_lo, rot, decay, state, (bf*)out, H, dim, vdim, k_scale, eps);
  else
    retention_scan_kernel<float><<<grid, RT_THREADS, smem, st>>>((const float*)proj, ld, q_off, k_off, v_off, g_off, cu_q, seq_slot,
                                                                 tok_pos, inv_freq, inv_freq_lo, rot, decay, state, (float*)out, H, dim, vdim,
                                                                 k_scale, eps);
  return launch_status();
}

// The chunked form: `sbuf` holds (n_tokens / CH + n_seqs) * H * dim * vdim floats.  Three launches.
DRYFT_API int dryft_retention_chunked(int is_bf16, const void* proj, int ld, int q_off, int k_off, int v_off, int g_off,
                                      const int* cu_q, const int* seq_slot, const int* tok_pos, const float* inv_freq,
                                      const float* inv_freq_lo, int rot, const double* decay, float* state, float* sbuf,
                                      void* out, int n_tokens, int n_seqs, int H, int dim, int vdim, float k_scale, float eps,
                                      cudaStream_t st) {
  if (n_seqs <= 0 || n_tokens <= 0) return 0;
  if (H <= 0 || dim <= 0 || vdim <= 0 || vdim > 512 || rot < 0 || rot > dim || (rot & 1) || H > 65535 || n_seqs > 65535)
    return DRYFT_ERR_UNSUPPORTED;
  typedef __nv_bfloat16 bf;
  const int n_chunks = n_tokens / CH + n_seqs;       // an upper bound; blocks behind the last chunk leave at once
  const int dP = (dim + 7) & ~7, vP8 = (vdim + 7) & ~7;
  const size_t smem_a = sizeof(float) * ((size_t)CH * dP + (size_t)CH * vP8 + CH + 1);
  const int dQ = ((dim + 3) & ~3) + 1, vP = (vdim + 3) & ~3;
  const size_t stage = (size_t)CH * (dQ > vP ? dQ : vP);
  const size_t smem_c = sizeof(float) * (stage + (size_t)CH * dQ + (size_t)(CH + 16) * vP + (size_t)CH * (CH + 1) + CH + 1);
  int rc = is_bf16 ? opt_in_smem(retention_chunk_state_kernel<bf>, smem_a) : opt_in_smem(retention_chunk_state_kernel<float>, smem_a);
  if (rc) return rc;
  rc = is_bf16 ? opt_in_smem(retention_chunk_out_kernel<bf>, smem_c) : opt_in_smem(retention_chunk_out_kernel<float>, smem_c);
  if (rc) return rc;
  dim3 grid(n_chunks, H);
  if (is_bf16)
    retention_chunk_state_kernel<bf><<<grid, CK_THREADS, smem_a, st>>>((const bf*)proj, ld, k_off, v_off, cu_q, seq_slot, n_seqs, tok_pos,
                                                                       inv_freq, inv_freq_lo, rot, decay, sbuf, H, dim, vdim, k_scale);
  else
    retention_chunk_state_kernel<float><<<grid, CK_THREADS, smem_a, st>>>((const float*)proj, ld, k_off, v_off, cu_q, seq_slot, n_seqs,
                                                                          tok_pos, inv_freq, inv_freq_lo, rot, decay, sbuf, H, dim, vdim,
                                                                          k_scale);
  int e = launch_status();
  if (e) return e;
  const int per_head = dim * vdim;
  dim3 grid_b(n_seqs, H, (per_head + 255) / 256);
  retention_chunk_prefix_kernel<<<grid_b, 256, 0, st>>>(cu_q, seq_slot, decay, sbuf, state, H, per_head);
  e = launch_status();
  if (e) return e;
  if (is_bf16)
    retention_chunk_out_kernel<bf><<<grid, CK_THREADS, smem_c, st>>>((const bf*)proj, ld, q_off, k_off, v_off, g_off, cu_q, seq_slot, n_seqs,
                                                                     tok_pos, inv_freq, inv_freq_lo, rot, decay, sbuf, (bf*)out, H, dim,
                                                                     vdim, k_scale, eps);
  else
    retention_chunk_out_kernel<float><<<grid, CK_THREADS, smem_c, st>>>((const float*)proj, ld, q_off, k_off, v_off, g_off, cu_q, seq_slot,
                                                                        n_seqs, tok_pos, inv_freq, inv_freq_lo, rot, decay, sbuf,
                                                                        (float*)out, H, dim, vdim, k_scale, eps);
  return launch_status();
}

DRYFT_API int dryft_retention_chunk_tokens() { return CH; }

DRYFT_API int dryft_rglru_gates(int is_bf16, const void* proj, int ld, int x_off, const float* x_bias, const int* tok_slot,
                                const float* conv_w, const float* conv_b, int taps, const float* tail, const float* w_gates,
                                const float* b_a, const float* b_i, const float* sp_lam, float c_mult, float* a_out, float* b_out,
                                int n_tokens, int C, int n_blocks, cudaStream_t st) {
  if (n_tokens <= 0) return 0;
  if (taps < 1 || n_blocks < 1 || C % n_blocks || n_blocks > 65535) return DRYFT_ERR_UNSUPPORTED;
  typedef __nv_bfloat16 bf;
  const int nb = C / n_blocks;
  const size_t smem = sizeof(float) * (size_t)GT * nb;
  int rc = is_bf16 ? opt_in_smem(rglru_gates_kernel<bf>, smem) : opt_in_smem(rglru_gates_kernel<float>, smem);
  if (rc) return rc;
  dim3 grid((n_tokens + GT - 1) / GT, n_blocks);
  if (is_bf16)
    rglru_gates_kernel<bf><<<grid, G_THREADS, smem, st>>>((const bf*)proj, ld, x_off, x_bias, tok_slot, conv_w, conv_b, taps, tail,
                                                          w_gates, b_a, b_i, sp_lam, c_mult, a_out, b_out, n_tokens, C, nb);
  else
    rglru_gates_kernel<float><<<grid, G_THREADS, smem, st>>>((const float*)proj, ld, x_off, x_bias, tok_slot, conv_w, conv_b, taps,
                                                             tail, w_gates, b_a, b_i, sp_lam, c_mult, a_out, b_out, n_tokens, C, nb);
  return launch_status();
}

DRYFT_API int dryft_rglru_scan(int is_bf16, const void* proj, int ld, int y_off, const float* y_bias, int x_off,
                               const float* x_bias, const int* cu_q, const int* seq_slot, const float* a_in, const float* b_in,
                               float* state, float* tail, int taps, void* out, int n_seqs, int C, cudaStream_t st) {
  if (n_seqs <= 0) return 0;
  typedef __nv_bfloat16 bf;
  const int threads = SCAN_WARPS * 32;
  dim3 grid(n_seqs, (C + 31) / 32);
  if (grid.y > 65535) return DRYFT_ERR_UNSUPPORTED;
  if (is_bf16)
    rglru_scan_kernel<bf><<<grid, threads, 0, st>>>((const bf*)proj, ld, y_off, y_bias, x_off, x_bias, cu_q, seq_slot, a_in, b_in, state,
                                                    tail, taps, (bf*)out, C);
  else
    rglru_scan_kernel<float><<<grid, threads, 0, st>>>((const float*)proj, ld, y_off, y_bias, x_off, x_bias, cu_q, seq_slot, a_in, b_in,
                                                       state, tail, taps, (float*)out, C);
  return launch_status();
}
