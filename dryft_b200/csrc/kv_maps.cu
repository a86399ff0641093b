// Per-map query/key RMS norm and the K/V write into the paged cache, for attention whose heads carry several
// score maps and whose values have a size of their own (no rotation: positions do not enter the scores).
//
// A token's projected row is  [ q: nH x MAPS x D | k: nKV x MAPS x D | v: nKV x DV | anything behind ]  (row stride
// given; the k and v parts are absent when the layer reads another layer's cache).  Every (head, map) vector of q
// and k is normalised on its own,  y = w * x / sqrt(mean(x^2) + eps)  in 32-bit with one weight vector [D] for
// all query heads and maps and one for the keys, and rounded to T once.  The normalised queries go to
// q_out [N, nH, MAPS*D]; the keys to k_pages [pages, nKV, PAGE, MAPS*D] and the values to
// v_pages [pages, nKV, PAGE, DV] at the token's (slot, position).  Padding tokens (slot < 0) write nothing but
// zero queries.
//
// Blocks (token, share of the token's vectors), one warp per vector.  No block waits on another.
#include "common.cuh"
#include <math.h>

namespace {
constexpr int THREADS = 128;

__device__ __forceinline__ float2 load2(const float* p) { return *reinterpret_cast<const float2*>(p); }
__device__ __forceinline__ float2 load2(const __nv_bfloat16* p) { return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p)); }
__device__ __forceinline__ void store2(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
__device__ __forceinline__ void store2(__nv_bfloat16* p, float a, float b) { *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b); }

template <typename T>
__global__ void __launch_bounds__(THREADS) kv_maps_store_kernel(
    const T* __restrict__ proj, int stride, const float* __restrict__ q_w, const float* __restrict__ k_w,
    const int* __restrict__ tok_slot, const int* __restrict__ tok_pos, T* __restrict__ q_out, T* __restrict__ k_pages,
    T* __restrict__ v_pages, const int* __restrict__ page_table, int max_pages, int nH, int nKV, int maps, int D, int DV,
    int page_size, float eps, int write_kv) {
  const int n = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = THREADS / 32;
  const int slot = tok_slot[n];
  const T* row = proj + (size_t)n * stride;
  const int nq = nH * maps, nk = write_kv ? nKV * maps : 0, nv = write_kv ? nKV : 0;
  // pairs of elements where every vector starts on an even element (row stride, D and DV even)
  const bool pairs = ((stride | D | DV) & 1) == 0;
  T* krow = nullptr;
  T* vrow = nullptr;
  if (write_kv && slot >= 0) {
    const int pos = tok_pos[n];
    const int page = page_table[(size_t)slot * max_pages + pos / page_size];
    const int r = pos % page_size;
    krow = k_pages + (((size_t)page * nKV) * page_size + r) * (size_t)(maps * D);   // kv head g adds g * page_size * maps*D
    vrow = v_pages + (((size_t)page * nKV) * page_size + r) * (size_t)DV;
  }
  // a warp takes one vector; the grid's second dimension covers a token's vectors, so that a step of few tokens (decode)
  // is many short blocks instead of a few long ones
  for (int u = blockIdx.y * nwarp + warp; u < nq + nk + nv; u += gridDim.y * nwarp) {
    if (u < nq + nk) {
      const bool is_q = u < nq;
      const int v = is_q ? u : u - nq;                 // vector index: head * maps + map
      const T* src = row + (size_t)u * D;              // q and k vectors lie back to back in the row
      T* dst;
      if (is_q) {
        dst = q_out + ((size_t)n * nq + v) * D;
      } else {
        if (krow == nullptr) continue;
        const int g = v / maps, m = v % maps;
        dst = krow + (size_t)g * page_size * (maps * D) + (size_t)m * D;
      }
      if (slot < 0) {
        for (int c = lane; c < D; c += 32) dst[c] = from_f32<T>(0.f);
        continue;
      }
      const float* w = is_q ? q_w : k_w;
      if (pairs) {   // two elements a lane and trip; a vector of up to 128 stays in registers between the two passes
        float2 keep[2];
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int c = 2 * (lane + 32 * i);
          keep[i] = make_float2(0.f, 0.f);
          if (c < D) keep[i] = load2(src + c);
          ss = fmaf(keep[i].x, keep[i].x, fmaf(keep[i].y, keep[i].y, ss));
        }
        for (int c = 128 + 2 * lane; c < D; c += 64) {
          const float2 x = load2(src + c);
          ss = fmaf(x.x, x.x, fmaf(x.y, x.y, ss));
        }
        ss = warp_sum(ss);
        const float inv = 1.f / sqrtf(ss / (float)D + eps);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int c = 2 * (lane + 32 * i);
          if (c < D) store2(dst + c, keep[i].x * inv * (w ? w[c] : 1.f), keep[i].y * inv * (w ? w[c + 1] : 1.f));
        }
        for (int c = 128 + 2 * lane; c < D; c += 64) {
          const float2 x = load2(src + c);
          store2(dst + c, x.x * inv * (w ? w[c] : 1.f), x.y * inv * (w ? w[c + 1] : 1.f));
        }
        continue;
      }
      float ss = 0.f;
      for (int c = lane; c < D; c += 32) {
        const float x = to_f32<T>(src[c]);
        ss = fmaf(x, x, ss);
      }
      ss = warp_sum(ss);
      const float inv = 1.f / sqrtf(ss / (float)D + eps);
      for (int c = lane; c < D; c += 32) {
        const float x = to_f32<T>(src[c]) * inv;
        dst[c] = from_f32<T>(w ? x * w[c] : x);
      }
    } else {
      if (vrow == nullptr) continue;
      const int g = u - nq - nk;
      const T* src = row + (size_t)(nq + nk) * D + (size_t)g * DV;
      T* dst = vrow + (size_t)g * page_size * DV;
      if (pairs) {
        for (int c = 2 * lane; c < DV; c += 64) {
          const float2 x = load2(src + c);
          store2(dst + c, x.x, x.y);
        }
      } else {
        for (int c = lane; c < DV; c += 32) dst[c] = src[c];
      }
    }
  }
}

template <typename T>
int launch(const void* proj, int stride, const float* q_w, const float* k_w, const int* tok_slot, const int* tok_pos,
           void* q_out, void* k_pages, void* v_pages, const int* page_table, int max_pages, int n, int nH, int nKV, int maps,
           int D, int DV, int page_size, float eps, int write_kv, cudaStream_t st) {
  if (n <= 0) return 0;
  if (nH < 1 || nKV < 1 || maps < 1 || D < 1 || DV < 1) return DRYFT_ERR_UNSUPPORTED;
  if (write_kv && (page_size < 1 || !k_pages || !v_pages || !page_table)) return DRYFT_ERR_UNSUPPORTED;
  const int units = nH * maps + (write_kv ? nKV * maps + nKV : 0);
  dim3 grid(n, (unsigned)min(64, (units + THREADS / 32 - 1) / (THREADS / 32)));
  kv_maps_store_kernel<T><<<grid, THREADS, 0, st>>>((const T*)proj, stride, q_w, k_w, tok_slot, tok_pos, (T*)q_out, (T*)k_pages,
                                                 (T*)v_pages, page_table, max_pages, nH, nKV, maps, D, DV, page_size, eps, write_kv);
  return launch_status();
}
}  // namespace

DRYFT_API int dryft_kv_maps_store(int is_bf16, const void* proj, int stride, const float* q_w, const float* k_w,
                                  const int* tok_slot, const int* tok_pos, void* q_out, void* k_pages, void* v_pages,
                                  const int* page_table, int max_pages, int n, int nH, int nKV, int maps, int D, int DV,
                                  int page_size, float eps, int write_kv, cudaStream_t st) {
  return is_bf16 ? launch<__nv_bfloat16>(proj, stride, q_w, k_w, tok_slot, tok_pos, q_out, k_pages, v_pages, page_table, max_pages,
                                         n, nH, nKV, maps, D, DV, page_size, eps, write_kv, st)
                 : launch<float>(proj, stride, q_w, k_w, tok_slot, tok_pos, q_out, k_pages, v_pages, page_table, max_pages, n, nH,
                                 nKV, maps, D, DV, page_size, eps, write_kv, st);
}
