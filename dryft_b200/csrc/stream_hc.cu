// A 32-bit residual stream that is kept as several copies ("streams") joined by small learned matrices
// (hyper-connections), the embedding that starts it, and the clamped gated activation of its feed-forward.
//
//   embed_pair_norm   x32[n] = norm( table[token] * scale + pair_table[row] ) * w,  row = (prev * mul_prev + token * mul_cur)
//                     mod buckets, or `buckets` (the table's last row) for a sequence's first token.  `prev` is the token
//                     before it in the step, or -- for the first token a sequence brings in a step -- the sequence's
//                     stored last token.  Both the pair table and the norm are optional.
//   seq_last_token    prev_state[slot] = the last token each sequence brought in this step
//   hc_step           with S streams x_1..x_S per row (32-bit), an optional pending sublayer output y and the next
//                     sublayer's input weights:
//                         x'_t = sum_s mix[s][t] * x_s + mult * out[t] * y          (all t at once from the old x)
//                         u    = sum_t in[t] * x'_t ;  h = T( u / sqrt(mean(u^2) + eps) * w )
//                     either half may be left out; the input may hold one stream that stands for all S (the start);
//                     with `rows` only the gathered rows are read and nothing is written back (the last norm).
//                     S = 1 with mix = out = in = 1 is the plain pre-norm residual  x += mult * y ; h = norm(x).
//   glu_clamp         out = g * sigmoid(alpha * g) * (u + up_offset),  g = min(gate, limit), u = clamp(up, -limit, limit)
//
// Sums, norms and the streams are 32-bit whatever the activation type T.  One block per row; widths are runtime
// arguments of any size.  No block waits on another.
#include "common.cuh"
#include <math.h>

namespace {
constexpr int THREADS = 256;
constexpr int MAX_STREAMS = 8;

template <typename TT>
__global__ void __launch_bounds__(THREADS) embed_pair_norm_kernel(
    const int* __restrict__ tokens, const int* __restrict__ tok_slot, const int* __restrict__ tok_pos,
    const int* __restrict__ prev_state, const TT* __restrict__ table, const TT* __restrict__ pair_table, int buckets,
    long long mul_prev, long long mul_cur, float scale, const float* __restrict__ norm_w, float eps,
    float* __restrict__ x32, int width, int vocab, int* __restrict__ err) {
  extern __shared__ __align__(16) float row[];
  __shared__ float scratch[33];
  const int n = blockIdx.x;
  const int slot = tok_slot[n];
  const int tok = tokens[n];
  const bool bad = tok < 0 || tok >= vocab;
  if (slot < 0 || bad) {  // a padding row, or an id outside the table: the row is zero
    if (slot >= 0 && threadIdx.x == 0 && err) atomicExch(err, 1);
    for (int c = threadIdx.x; c < width; c += THREADS) x32[(size_t)n * width + c] = 0.f;
    return;
  }
  const TT* pair = nullptr;
  if (pair_table) {
    long long r = buckets;
    if (n > 0 && tok_slot[n - 1] == slot) {
      r = ((long long)tokens[n - 1] * mul_prev + (long long)tok * mul_cur) % buckets;
    } else if (tok_pos[n] > 0) {
      r = ((long long)prev_state[slot] * mul_prev + (long long)tok * mul_cur) % buckets;
    }
    if (r < 0) r += buckets;
    pair = pair_table + (size_t)r * width;
  }
  const TT* src = table + (size_t)tok * width;
  float ss = 0.f;
  for (int c = threadIdx.x; c < width; c += THREADS) {
    float v = to_f32<TT>(src[c]) * scale;
    if (pair) v += to_f32<TT>(pair[c]);
    row[c] = v;
    ss = fmaf(v, v, ss);
  }
  if (!norm_w) {
    for (int c = threadIdx.x; c < width; c += THREADS) x32[(size_t)n * width + c] = row[c];
    return;
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(ss / (float)width + eps);
  for (int c = threadIdx.x; c < width; c += THREADS) x32[(size_t)n * width + c] = row[c] * inv * norm_w[c];
}

__global__ void seq_last_token_kernel(const int* __restrict__ tokens, const int* __restrict__ tok_slot, int n_tokens,
                                      int* __restrict__ prev_state) {
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= n_tokens) return;
  const int slot = tok_slot[n];
  if (slot < 0) return;
  if (n + 1 == n_tokens || tok_slot[n + 1] != slot) prev_state[slot] = tokens[n];
}

// four consecutive elements at once (8 or 16 bytes)
template <typename T> __device__ __forceinline__ float4 load4(const T* p);
template <> __device__ __forceinline__ float4 load4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <> __device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
template <typename T> __device__ __forceinline__ void store4(T* p, float4 v);
template <> __device__ __forceinline__ void store4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<unsigned*>(&a);
  raw.y = *reinterpret_cast<unsigned*>(&b);
  *reinterpret_cast<uint2*>(p) = raw;
}

// MS: the most streams this instantiation holds in registers (1, 2, 4 or MAX_STREAMS); fewer registers, more blocks an SM
template <typename T, int MS>
__global__ void __launch_bounds__(THREADS) hc_step_kernel(
    const float* __restrict__ x_in, int s_in, float* __restrict__ x_out, int S, const T* __restrict__ y,
    const float* __restrict__ mix, const float* __restrict__ outw, float mult, const float* __restrict__ inw,
    const float* __restrict__ norm_w, float eps, const int* __restrict__ rows, T* __restrict__ h, int width) {
  extern __shared__ __align__(16) float row[];
  __shared__ float scratch[33];
  __shared__ float c_mix[MS * MS], c_out[MS], c_in[MS];
  const int r = blockIdx.x;
  const size_t src = rows ? (size_t)rows[r] : (size_t)r;
  if (threadIdx.x < S * S) c_mix[threadIdx.x] = y ? mix[threadIdx.x] : 0.f;
  if (threadIdx.x < S) {
    c_out[threadIdx.x] = y ? mult * outw[threadIdx.x] : 0.f;
    c_in[threadIdx.x] = inw ? inw[threadIdx.x] : 0.f;
  }
  __syncthreads();
  float ss = 0.f;
  if ((width & 3) == 0) {
    // four columns a thread, 16-byte accesses to the streams: the pass is bound by bytes in flight
    for (int c = threadIdx.x * 4; c < width; c += THREADS * 4) {
      float4 x[MS];
#pragma unroll
      for (int s = 0; s < MS; ++s)
        if (s < S) x[s] = *reinterpret_cast<const float4*>(x_in + (src * s_in + (s_in == 1 ? 0 : s)) * width + c);
      if (y) {
        const float4 yv = load4<T>(y + src * width + c);
        float4 xn[MS];
#pragma unroll
        for (int t = 0; t < MS; ++t) {
          if (t < S) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int s = 0; s < MS; ++s)
              if (s < S) {
                const float m = c_mix[s * S + t];
                acc.x = fmaf(m, x[s].x, acc.x); acc.y = fmaf(m, x[s].y, acc.y); acc.z = fmaf(m, x[s].z, acc.z); acc.w = fmaf(m, x[s].w, acc.w);
              }
            const float o = c_out[t];
            xn[t] = make_float4(fmaf(o, yv.x, acc.x), fmaf(o, yv.y, acc.y), fmaf(o, yv.z, acc.z), fmaf(o, yv.w, acc.w));
          }
        }
#pragma unroll
        for (int t = 0; t < MS; ++t)
          if (t < S) x[t] = xn[t];
      }
      if (x_out) {
#pragma unroll
        for (int t = 0; t < MS; ++t)
          if (t < S) *reinterpret_cast<float4*>(x_out + (src * S + t) * width + c) = x[t];
      }
      if (inw) {
        float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int t = 0; t < MS; ++t)
          if (t < S) {
            const float w = c_in[t];
            u.x = fmaf(w, x[t].x, u.x); u.y = fmaf(w, x[t].y, u.y); u.z = fmaf(w, x[t].z, u.z); u.w = fmaf(w, x[t].w, u.w);
          }
        *reinterpret_cast<float4*>(row + c) = u;
        ss = fmaf(u.x, u.x, fmaf(u.y, u.y, fmaf(u.z, u.z, fmaf(u.w, u.w, ss))));
      }
    }
    if (!inw) return;
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / (float)width + eps);
    for (int c = threadIdx.x * 4; c < width; c += THREADS * 4) {
      const float4 u = *reinterpret_cast<const float4*>(row + c), w = *reinterpret_cast<const float4*>(norm_w + c);
      store4<T>(h + (size_t)r * width + c, make_float4(u.x * inv * w.x, u.y * inv * w.y, u.z * inv * w.z, u.w * inv * w.w));
    }
    return;
  }
  for (int c = threadIdx.x; c < width; c += THREADS) {
    float x[MS];
#pragma unroll
    for (int s = 0; s < MS; ++s)
      if (s < S) x[s] = x_in[(src * s_in + (s_in == 1 ? 0 : s)) * width + c];
    if (y) {
      const float yv = to_f32<T>(y[src * width + c]);
      float xn[MS];
#pragma unroll
      for (int t = 0; t < MS; ++t) {
        if (t < S) {
          float acc = 0.f;
#pragma unroll
          for (int s = 0; s < MS; ++s)
            if (s < S) acc = fmaf(c_mix[s * S + t], x[s], acc);
          xn[t] = fmaf(c_out[t], yv, acc);
        }
      }
#pragma unroll
      for (int t = 0; t < MS; ++t)
        if (t < S) x[t] = xn[t];
    }
    if (x_out) {
#pragma unroll
      for (int t = 0; t < MS; ++t)
        if (t < S) x_out[(src * S + t) * width + c] = x[t];
    }
    if (inw) {
      float u = 0.f;
#pragma unroll
      for (int t = 0; t < MS; ++t)
        if (t < S) u = fmaf(c_in[t], x[t], u);
      row[c] = u;
      ss = fmaf(u, u, ss);
    }
  }
  if (!inw) return;
  ss = block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(ss / (float)width + eps);
  for (int c = threadIdx.x; c < width; c += THREADS) h[(size_t)r * width + c] = from_f32<T>(row[c] * inv * norm_w[c]);
}

__device__ __forceinline__ float glu_one(float g, float u, float limit, int has_limit, float alpha, float up_offset) {
  if (has_limit) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
  }
  return g / (1.f + expf(-alpha * g)) * (u + up_offset);
}

// VEC = 4: four columns a thread (8- or 16-byte accesses; the width is then a multiple of four), VEC = 1: any width
template <typename T, int VEC>
__global__ void glu_clamp_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int rows, int inter, float limit,
                                 int has_limit, float alpha, float up_offset) {
  const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * VEC;
  if (i >= (size_t)rows * inter) return;
  const size_t r = i / inter, f = i % inter;
  const T* g = gate_up + r * 2 * inter + f;
  if (VEC == 4) {
    const float4 gv = load4<T>(g), uv = load4<T>(g + inter);
    store4<T>(out + i, make_float4(glu_one(gv.x, uv.x, limit, has_limit, alpha, up_offset), glu_one(gv.y, uv.y, limit, has_limit, alpha, up_offset),
                                   glu_one(gv.z, uv.z, limit, has_limit, alpha, up_offset), glu_one(gv.w, uv.w, limit, has_limit, alpha, up_offset)));
  } else {
    out[i] = from_f32<T>(glu_one(to_f32<T>(g[0]), to_f32<T>(g[inter]), limit, has_limit, alpha, up_offset));
  }
}

template <typename K> int row_smem(K kernel, int width) {
  const size_t bytes = sizeof(float) * (size_t)width;
  if (bytes > 200 * 1024) return DRYFT_ERR_UNSUPPORTED;
  if (bytes > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return (int)e;
  }
  return 0;
}
}  // namespace

DRYFT_API int dryft_embed_pair_norm(int table_bf16, const int* tokens, const int* tok_slot, const int* tok_pos,
                                    const int* prev_state, const void* table, const void* pair_table, int buckets,
                                    long long mul_prev, long long mul_cur, float scale, const float* norm_w, float eps, float* x32,
                                    int n, int width, int vocab, int* err, cudaStream_t st) {
  if (n <= 0) return 0;
  if (pair_table && (buckets <= 0 || !prev_state)) return DRYFT_ERR_UNSUPPORTED;
  typedef __nv_bfloat16 bf;
  const size_t smem = sizeof(float) * (size_t)width;
  int rc = table_bf16 ? row_smem(embed_pair_norm_kernel<bf>, width) : row_smem(embed_pair_norm_kernel<float>, width);
  if (rc) return rc;
  if (table_bf16)
    embed_pair_norm_kernel<bf><<<n, THREADS, smem, st>>>(tokens, tok_slot, tok_pos, prev_state, (const bf*)table, (const bf*)pair_table,
                                                         buckets, mul_prev, mul_cur, scale, norm_w, eps, x32, width, vocab, err);
  else
    embed_pair_norm_kernel<float><<<n, THREADS, smem, st>>>(tokens, tok_slot, tok_pos, prev_state, (const float*)table,
                                                            (const float*)pair_table, buckets, mul_prev, mul_cur, scale, norm_w, eps,
                                                            x32, width, vocab, err);
  return launch_status();
}

DRYFT_API int dryft_seq_last_token(const int* tokens, const int* tok_slot, int n, int* prev_state, cudaStream_t st) {
  if (n <= 0) return 0;
  seq_last_token_kernel<<<(n + 255) / 256, 256, 0, st>>>(tokens, tok_slot, n, prev_state);
  return launch_status();
}

DRYFT_API int dryft_hc_step(int is_bf16, const float* x_in, int s_in, float* x_out, int n_streams, const void* y, const float* mix,
                            const float* outw, float mult, const float* inw, const float* norm_w, float eps, const int* rows,
                            void* h, int n_rows, int width, cudaStream_t st) {
  if (n_rows <= 0) return 0;
  if (n_streams < 1 || n_streams > MAX_STREAMS || (s_in != 1 && s_in != n_streams)) return DRYFT_ERR_UNSUPPORTED;
  if (y && (!mix || !outw)) return DRYFT_ERR_UNSUPPORTED;
  if (inw && (!norm_w || !h)) return DRYFT_ERR_UNSUPPORTED;
  typedef __nv_bfloat16 bf;
  const size_t smem = sizeof(float) * (size_t)width;
#define DRYFT_HC_LAUNCH(TT, MS)                                                                                                  \
  do {                                                                                                                          \
    int rc = row_smem(hc_step_kernel<TT, MS>, width);                                                                           \
    if (rc) return rc;                                                                                                          \
    hc_step_kernel<TT, MS><<<n_rows, THREADS, smem, st>>>(x_in, s_in, x_out, n_streams, (const TT*)y, mix, outw, mult, inw, norm_w, \
                                                          eps, rows, (TT*)h, width);                                            \
  } while (0)
#define DRYFT_HC_BY_STREAMS(TT)                                                                                                  \
  do {                                                                                                                          \
    if (n_streams <= 1) DRYFT_HC_LAUNCH(TT, 1);                                                                                 \
    else if (n_streams <= 2) DRYFT_HC_LAUNCH(TT, 2);                                                                            \
    else if (n_streams <= 4) DRYFT_HC_LAUNCH(TT, 4);                                                                            \
    else DRYFT_HC_LAUNCH(TT, MAX_STREAMS);                                                                                      \
  } while (0)
  if (is_bf16) DRYFT_HC_BY_STREAMS(bf);
  else DRYFT_HC_BY_STREAMS(float);
#undef DRYFT_HC_BY_STREAMS
#undef DRYFT_HC_LAUNCH
  return launch_status();
}

DRYFT_API int dryft_glu_clamp(int is_bf16, const void* gate_up, void* out, int rows, int inter, float limit, int has_limit,
                              float alpha, float up_offset, cudaStream_t st) {
  if (rows <= 0 || inter <= 0) return 0;
  typedef __nv_bfloat16 bf;
  const size_t total = (size_t)rows * inter;
  if ((inter & 3) == 0) {
    const unsigned blocks = (unsigned)((total / 4 + 255) / 256);
    if (is_bf16) glu_clamp_kernel<bf, 4><<<blocks, 256, 0, st>>>((const bf*)gate_up, (bf*)out, rows, inter, limit, has_limit, alpha, up_offset);
    else glu_clamp_kernel<float, 4><<<blocks, 256, 0, st>>>((const float*)gate_up, (float*)out, rows, inter, limit, has_limit, alpha, up_offset);
  } else {
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (is_bf16) glu_clamp_kernel<bf, 1><<<blocks, 256, 0, st>>>((const bf*)gate_up, (bf*)out, rows, inter, limit, has_limit, alpha, up_offset);
    else glu_clamp_kernel<float, 1><<<blocks, 256, 0, st>>>((const float*)gate_up, (float*)out, rows, inter, limit, has_limit, alpha, up_offset);
  }
  return launch_status();
}
