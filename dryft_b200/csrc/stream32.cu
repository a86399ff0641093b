// Kernels around a residual stream that is kept in 32-bit whatever the activation type T is: a model whose
// layers add a normalised sublayer output to the stream (x += norm(f(x))) sums in 32-bit and hands each
// sublayer the stream rounded to T.
//
//   embed_sinusoid    x32[n] = table[token] * scale + s(pos),  s[2i] = sin(pos * f_i), s[2i+1] = cos(pos * f_i),
//                     f_i given by the host (32-bit, [ceil(width/2)]); h[n] = T(x32[n])
//   stream_norm_add   y = the sublayer's output row (or the weighted sum of `top` rows: y = sum_k wts[n,k] * y[n*top+k]);
//                     x32[n] += y / sqrt(mean(y^2) + eps) * (offset + w);  h[n] = T(x32[n])
//   stream_norm_rows  out[r] = T( x[src] / sqrt(mean(x[src]^2) + eps) * (offset + w) ),  src = rows ? rows[r] : r,
//                     x of 32-bit or of type T
//
// Angles, sums of squares, the norm and the stream's sum are 32-bit.  One block per row; widths are runtime
// arguments of any size (the row is staged in shared memory as floats, 4 * width bytes).  No block waits on another.
#include "common.cuh"
#include <math.h>

namespace {
constexpr int THREADS = 256;

template <typename TT, typename T>
__global__ void __launch_bounds__(THREADS) embed_sinusoid_kernel(
    const int* __restrict__ tokens, const int* __restrict__ tok_pos, const TT* __restrict__ table,
    const float* __restrict__ freq, float scale, float* __restrict__ x32, T* __restrict__ h, int width, int vocab,
    int* __restrict__ err) {
  const int n = blockIdx.x;
  const int tok = tokens[n];
  const bool bad = tok < 0 || tok >= vocab;
  if (bad && threadIdx.x == 0 && err) atomicExch(err, 1);
  const float pos = (float)tok_pos[n];
  const TT* src = table + (size_t)(bad ? 0 : tok) * width;
  for (int c = threadIdx.x; c < width; c += THREADS) {
    float v = 0.f;
    if (!bad) {
      const float ang = pos * freq[c >> 1];
      v = to_f32<TT>(src[c]) * scale + ((c & 1) ? cosf(ang) : sinf(ang));
    }
    x32[(size_t)n * width + c] = v;
    if (h) h[(size_t)n * width + c] = from_f32<T>(v);
  }
}

// four consecutive elements at once (8 or 16 bytes); rows whose width is not a multiple of four go element by element
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

template <typename T>
__global__ void __launch_bounds__(THREADS) stream_norm_add_kernel(
    const T* __restrict__ y, const float* __restrict__ wts, int top, const float* __restrict__ w, float offset, float eps,
    float* __restrict__ x32, T* __restrict__ h, int width) {
  extern __shared__ __align__(16) float row[];
  __shared__ float scratch[33];
  const int n = blockIdx.x;
  float ss = 0.f;
  if ((width & 3) == 0) {
    for (int c = threadIdx.x * 4; c < width; c += THREADS * 4) {
      float4 v;
      if (top > 0) {
        v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
        for (int k = 0; k < top; ++k) {
          const float wk = wts[(size_t)n * top + k];
          const float4 u = load4<T>(y + ((size_t)n * top + k) * width + c);
          v.x = fmaf(wk, u.x, v.x); v.y = fmaf(wk, u.y, v.y); v.z = fmaf(wk, u.z, v.z); v.w = fmaf(wk, u.w, v.w);
        }
      } else {
        v = load4<T>(y + (size_t)n * width + c);
      }
      *reinterpret_cast<float4*>(row + c) = v;
      ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / (float)width + eps);
    for (int c = threadIdx.x * 4; c < width; c += THREADS * 4) {
      const float4 r = *reinterpret_cast<const float4*>(row + c), ww = *reinterpret_cast<const float4*>(w + c);
      float4 v = *reinterpret_cast<const float4*>(x32 + (size_t)n * width + c);
      v.x += r.x * inv * (offset + ww.x); v.y += r.y * inv * (offset + ww.y);
      v.z += r.z * inv * (offset + ww.z); v.w += r.w * inv * (offset + ww.w);
      *reinterpret_cast<float4*>(x32 + (size_t)n * width + c) = v;
      if (h) store4<T>(h + (size_t)n * width + c, v);
    }
    return;
  }
  for (int c = threadIdx.x; c < width; c += THREADS) {
    float v;
    if (top > 0) {
      v = 0.f;
      for (int k = 0; k < top; ++k) v = fmaf(wts[(size_t)n * top + k], to_f32<T>(y[((size_t)n * top + k) * width + c]), v);
    } else {
      v = to_f32<T>(y[(size_t)n * width + c]);
    }
    row[c] = v;
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(ss / (float)width + eps);
  for (int c = threadIdx.x; c < width; c += THREADS) {
    const float v = x32[(size_t)n * width + c] + row[c] * inv * (offset + w[c]);
    x32[(size_t)n * width + c] = v;
    if (h) h[(size_t)n * width + c] = from_f32<T>(v);
  }
}

template <typename TI, typename T>
__global__ void __launch_bounds__(THREADS) stream_norm_rows_kernel(
    const TI* __restrict__ x, const int* __restrict__ rows, const float* __restrict__ w, float offset, float eps,
    T* __restrict__ out, int width) {
  extern __shared__ __align__(16) float row[];
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  const size_t src = rows ? (size_t)rows[r] : (size_t)r;
  float ss = 0.f;
  for (int c = threadIdx.x; c < width; c += THREADS) {
    const float v = to_f32<TI>(x[src * width + c]);
    row[c] = v;
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(ss / (float)width + eps);
  for (int c = threadIdx.x; c < width; c += THREADS) out[(size_t)r * width + c] = from_f32<T>(row[c] * inv * (offset + w[c]));
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

DRYFT_API int dryft_embed_sinusoid(int table_bf16, int act_bf16, const int* tokens, const int* tok_pos, const void* table,
                                   const float* freq, float scale, float* x32, void* h, int n, int width, int vocab, int* err,
                                   cudaStream_t st) {
  if (n <= 0) return 0;
  typedef __nv_bfloat16 bf;
  if (table_bf16 && act_bf16)
    embed_sinusoid_kernel<bf, bf><<<n, THREADS, 0, st>>>(tokens, tok_pos, (const bf*)table, freq, scale, x32, (bf*)h, width, vocab, err);
  else if (table_bf16)
    embed_sinusoid_kernel<bf, float><<<n, THREADS, 0, st>>>(tokens, tok_pos, (const bf*)table, freq, scale, x32, (float*)h, width, vocab, err);
  else if (act_bf16)
    embed_sinusoid_kernel<float, bf><<<n, THREADS, 0, st>>>(tokens, tok_pos, (const float*)table, freq, scale, x32, (bf*)h, width, vocab, err);
  else
    embed_sinusoid_kernel<float, float><<<n, THREADS, 0, st>>>(tokens, tok_pos, (const float*)table, freq, scale, x32, (float*)h, width, vocab, err);
  return launch_status();
}

DRYFT_API int dryft_stream_norm_add(int is_bf16, const void* y, const float* wts, int top, const float* w, float offset, float eps,
                                    float* x32, void* h, int n, int width, cudaStream_t st) {
  if (n <= 0) return 0;
  typedef __nv_bfloat16 bf;
  const size_t smem = sizeof(float) * (size_t)width;
  int rc = is_bf16 ? row_smem(stream_norm_add_kernel<bf>, width) : row_smem(stream_norm_add_kernel<float>, width);
  if (rc) return rc;
  if (is_bf16)
    stream_norm_add_kernel<bf><<<n, THREADS, smem, st>>>((const bf*)y, wts, top, w, offset, eps, x32, (bf*)h, width);
  else
    stream_norm_add_kernel<float><<<n, THREADS, smem, st>>>((const float*)y, wts, top, w, offset, eps, x32, (float*)h, width);
  return launch_status();
}

DRYFT_API int dryft_stream_norm_rows(int in_bf16, int out_bf16, const void* x, const int* rows, const float* w, float offset,
                                     float eps, void* out, int n, int width, cudaStream_t st) {
  if (n <= 0) return 0;
  typedef __nv_bfloat16 bf;
  const size_t smem = sizeof(float) * (size_t)width;
  int rc;
  if (in_bf16 && out_bf16) {
    if ((rc = row_smem(stream_norm_rows_kernel<bf, bf>, width))) return rc;
    stream_norm_rows_kernel<bf, bf><<<n, THREADS, smem, st>>>((const bf*)x, rows, w, offset, eps, (bf*)out, width);
  } else if (in_bf16) {
    if ((rc = row_smem(stream_norm_rows_kernel<bf, float>, width))) return rc;
    stream_norm_rows_kernel<bf, float><<<n, THREADS, smem, st>>>((const bf*)x, rows, w, offset, eps, (float*)out, width);
  } else if (out_bf16) {
    if ((rc = row_smem(stream_norm_rows_kernel<float, bf>, width))) return rc;
    stream_norm_rows_kernel<float, bf><<<n, THREADS, smem, st>>>((const float*)x, rows, w, offset, eps, (bf*)out, width);
  } else {
    if ((rc = row_smem(stream_norm_rows_kernel<float, float>, width))) return rc;
    stream_norm_rows_kernel<float, float><<<n, THREADS, smem, st>>>((const float*)x, rows, w, offset, eps, (float*)out, width);
  }
  return launch_status();
}
