// Differential attention of independent query rows over the paged cache ("split-KV"): the decode kernel of both
// precisions, the prefill kernel of the 32-bit path (a prompt token is a row with its own position) and the general
// fallback.  Compiled per model with -DDRYFT_QK_DIM (size of one score map's queries and keys), -DDRYFT_V_DIM,
// -DDRYFT_GROUP, -DDRYFT_PAGE.
//
// A head has two score maps over the same values.  Keys lie in the cache as [pages, nKV, PAGE, 2*DQ] (map 1, then
// map 2), values as [pages, nKV, PAGE, DV]; queries come normalised as [N, nH, 2*DQ].  With a_1, a_2 the two maps'
// softmax-weighted sums of the values,
//     o = a_1 - lambda * a_2 ;   o <- o / sqrt(mean(o^2) + eps) * out_scale ;   o <- o * sigmoid(gate[n, h])
// (the gate is optional: one logit per token and head, read from a row of the projection output).
// Row n at position p of slot s sees the keys j <= p with
//     j >= p + 1 - window        (window > 0: the last `window` keys)
//     j >= floor(p / chunk) * chunk   (chunk > 0: only keys of the query's own block of `chunk` positions,
//                                      counted from position 0 of the sequence)
// Scores, maxima, sums, the combination and its norm are 32-bit.
//
// Grid (rows, kv heads, splits).  One block serves the GROUP query heads of a kv head (2*GROUP maps) for one row over
// a contiguous range of pages.  With one split the block finishes the row itself; otherwise it leaves un-normalised
// partials (acc, m, l) per map and `diff_attn_reduce_kernel` combines them and applies the epilogue.
// No block waits on another block; there is no spin anywhere in this file.
#include "common.cuh"
#include <math.h>

#if !defined(DRYFT_QK_DIM) || !defined(DRYFT_V_DIM) || !defined(DRYFT_GROUP) || !defined(DRYFT_PAGE)
#error "compile with -DDRYFT_QK_DIM=.. -DDRYFT_V_DIM=.. -DDRYFT_GROUP=.. -DDRYFT_PAGE=.."
#endif

namespace {
constexpr int DQ = DRYFT_QK_DIM;
constexpr int DV = DRYFT_V_DIM;
constexpr int G = DRYFT_GROUP;
constexpr int PAGE = DRYFT_PAGE;
constexpr int MAPS = 2;
constexpr int GM = G * MAPS;          // score maps a block serves
constexpr int KW = MAPS * DQ;         // elements of one cached key row
constexpr int THREADS = 128;
constexpr int NWARP = THREADS / 32;
constexpr int DIMS_PER_THREAD = (DV + THREADS - 1) / THREADS;
static_assert(PAGE % 32 == 0, "page size must be a multiple of 32");

template <typename T> struct Smem {
  // 16-byte copies where both row sizes allow them, else element by element
  static constexpr int VEC = ((KW * sizeof(T)) % 16 == 0 && (DV * sizeof(T)) % 16 == 0) ? (int)(16 / sizeof(T)) : 1;
  static constexpr int KSTRIDE = KW + (VEC > 1 ? VEC : 1);   // padded K row: conflict-free row-per-thread reads
  static constexpr size_t floats() { return (size_t)GM * DQ + (size_t)GM * PAGE + 3 * GM + (size_t)G * DV + G; }
  static constexpr size_t bytes() { return sizeof(float) * floats() + sizeof(T) * (size_t)(PAGE * KSTRIDE + PAGE * DV) + 32; }
};

template <typename T, int VEC> struct alignas(sizeof(T) * VEC) Chunk { T e[VEC]; };

__device__ __forceinline__ int first_visible(int pos, int window, int chunk) {
  int lo = 0;
  if (window > 0) lo = max(lo, pos + 1 - window);
  if (chunk > 0) lo = max(lo, pos - pos % chunk);
  return lo;
}

template <typename T>
__global__ void __launch_bounds__(THREADS) diff_attn_rows_kernel(
    const T* __restrict__ q,                                        // [N, nH, 2*DQ]
    const T* __restrict__ k_pages, const T* __restrict__ v_pages,   // [pages, nKV, PAGE, 2*DQ], [pages, nKV, PAGE, DV]
    const int* __restrict__ page_table, int max_pages,
    const int* __restrict__ tok_slot, const int* __restrict__ tok_pos,
    const T* __restrict__ gate, int gate_stride,                    // gate[n * gate_stride + h] (logits) or null
    T* __restrict__ out,                                            // [N, nH * DV]
    float* __restrict__ part_o, float* __restrict__ part_ml,        // [N, nH, 2, S, DV], [N, nH, 2, S, 2]
    int nKV, int n_splits, float scale, int window, int chunk, float lambda, float sub_eps, float out_scale) {
  using L = Smem<T>;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* kt = reinterpret_cast<T*>(smem_raw);                 // [PAGE][KSTRIDE]
  T* vt = kt + PAGE * L::KSTRIDE;                         // [PAGE][DV]
  float* qs = reinterpret_cast<float*>(smem_raw + ((sizeof(T) * (size_t)(PAGE * L::KSTRIDE + PAGE * DV) + 15) / 16) * 16);  // [GM][DQ]
  float* sc = qs + GM * DQ;                               // [GM][PAGE]
  float* m_s = sc + GM * PAGE;                            // [GM]
  float* l_s = m_s + GM;
  float* a_s = l_s + GM;
  float* ob = a_s + GM;                                   // [G][DV]
  float* ssq = ob + G * DV;                               // [G]

  const int n = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int nH = nKV * G;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int slot = tok_slot[n];

  if (slot < 0) {  // padding row: defined zeros, no cache access
    if (n_splits == 1) {
      for (int i = tid; i < G * DV; i += THREADS) out[(size_t)n * nH * DV + (size_t)kvh * G * DV + i] = from_f32<T>(0.f);
    } else {
      for (int gm = 0; gm < GM; ++gm) {
        const size_t pi = (((size_t)n * nH + kvh * G) * MAPS + gm) * n_splits + split;
        for (int d = tid; d < DV; d += THREADS) part_o[pi * DV + d] = 0.f;
        if (tid == 0) { part_ml[pi * 2] = -INFINITY; part_ml[pi * 2 + 1] = 0.f; }
      }
    }
    return;
  }

  const int pos = tok_pos[n];
  const int kv_hi = pos + 1;                                  // exclusive
  const int kv_lo = first_visible(pos, window, chunk);        // inclusive
  const int first_page = kv_lo / PAGE, last_page = (kv_hi - 1) / PAGE;
  const int n_pages = last_page - first_page + 1;
  const int per_split = (n_pages + n_splits - 1) / n_splits;
  const int pg_begin = first_page + split * per_split;
  const int pg_end = min(pg_begin + per_split, last_page + 1);

  // the block's GM query vectors: head g's map m is row g*MAPS + m, contiguous in q
  for (int i = tid; i < GM * DQ; i += THREADS) qs[i] = to_f32<T>(q[((size_t)n * nH + (size_t)kvh * G) * KW + i]);
  if (tid < GM) { m_s[tid] = -INFINITY; l_s[tid] = 0.f; a_s[tid] = 1.f; }
  float acc[DIMS_PER_THREAD][GM];
#pragma unroll
  for (int i = 0; i < DIMS_PER_THREAD; ++i)
#pragma unroll
    for (int g = 0; g < GM; ++g) acc[i][g] = 0.f;

  const int* pt = page_table + (size_t)slot * max_pages;
  constexpr int VEC = L::VEC;
  typedef Chunk<T, VEC> CK;
  constexpr int KVPR = KW / VEC, VVPR = DV / VEC;
  for (int pg = pg_begin; pg < pg_end; ++pg) {
    const int page = pt[pg];
    const int p0 = pg * PAGE;
    const T* kp = k_pages + ((size_t)page * nKV + kvh) * PAGE * KW;
    const T* vp = v_pages + ((size_t)page * nKV + kvh) * PAGE * DV;
    __syncthreads();  // previous tile fully consumed
    for (int i = tid; i < PAGE * KVPR; i += THREADS) {
      const int r = i / KVPR, c = i % KVPR;
      const int p = p0 + r;
      CK v;
#pragma unroll
      for (int t = 0; t < VEC; ++t) v.e[t] = from_f32<T>(0.f);
      if (p >= kv_lo && p < kv_hi) v = reinterpret_cast<const CK*>(kp + (size_t)r * KW)[c];
      *reinterpret_cast<CK*>(kt + r * L::KSTRIDE + c * VEC) = v;
    }
    for (int i = tid; i < PAGE * VVPR; i += THREADS) {
      const int r = i / VVPR, c = i % VVPR;
      const int p = p0 + r;
      CK v;
#pragma unroll
      for (int t = 0; t < VEC; ++t) v.e[t] = from_f32<T>(0.f);
      if (p >= kv_lo && p < kv_hi) v = reinterpret_cast<const CK*>(vp + (size_t)r * DV)[c];
      *reinterpret_cast<CK*>(vt + r * DV + c * VEC) = v;
    }
    __syncthreads();
    // scores: item -> (map gm, key r); consecutive threads take consecutive keys
    for (int item = tid; item < GM * PAGE; item += THREADS) {
      const int gm = item / PAGE, r = item % PAGE;
      const int p = p0 + r;
      float s = -INFINITY;
      if (p >= kv_lo && p < kv_hi) {
        const T* kr = kt + r * L::KSTRIDE + (gm % MAPS) * DQ;
        const float* qg = qs + gm * DQ;
        float dot = 0.f;
#pragma unroll 8
        for (int c = 0; c < DQ; ++c) dot = fmaf(qg[c], to_f32<T>(kr[c]), dot);
        s = dot * scale;
      }
      sc[item] = s;
    }
    __syncthreads();
    // online softmax, one warp per map
    for (int gm = warp; gm < GM; gm += NWARP) {
      float mx = -INFINITY;
      for (int r = lane; r < PAGE; r += 32) mx = fmaxf(mx, sc[gm * PAGE + r]);
      mx = warp_max(mx);
      const float m_old = m_s[gm];
      const float m_new = fmaxf(m_old, mx);
      float sum = 0.f;
      for (int r = lane; r < PAGE; r += 32) {
        const float s = sc[gm * PAGE + r];
        const float p = (s == -INFINITY) ? 0.f : expf(s - m_new);
        sc[gm * PAGE + r] = p;
        sum += p;
      }
      sum = warp_sum(sum);
      if (lane == 0) {
        const float alpha = (m_old == -INFINITY) ? 0.f : expf(m_old - m_new);
        a_s[gm] = alpha;
        m_s[gm] = m_new;
        l_s[gm] = l_s[gm] * alpha + sum;
      }
    }
    __syncthreads();
    // acc = acc*alpha + P V ; thread owns value dims tid, tid+THREADS, ...
#pragma unroll
    for (int i = 0; i < DIMS_PER_THREAD; ++i) {
      const int d = tid + i * THREADS;
      if (d < DV) {
#pragma unroll
        for (int g = 0; g < GM; ++g) acc[i][g] *= a_s[g];
        for (int r = 0; r < PAGE; ++r) {
          const float v = to_f32<T>(vt[r * DV + d]);
#pragma unroll
          for (int g = 0; g < GM; ++g) acc[i][g] = fmaf(sc[g * PAGE + r], v, acc[i][g]);
        }
      }
    }
  }
  __syncthreads();
  if (n_splits > 1) {
#pragma unroll
    for (int i = 0; i < DIMS_PER_THREAD; ++i) {
      const int d = tid + i * THREADS;
      if (d >= DV) continue;
#pragma unroll
      for (int gm = 0; gm < GM; ++gm)
        part_o[((((size_t)n * nH + kvh * G) * MAPS + gm) * n_splits + split) * DV + d] = acc[i][gm];
    }
    if (tid < GM) {
      const size_t pi = (((size_t)n * nH + kvh * G) * MAPS + tid) * n_splits + split;
      part_ml[pi * 2] = m_s[tid];
      part_ml[pi * 2 + 1] = l_s[tid];
    }
    return;
  }
  // one split: combine the two maps, normalise over the value dims, gate, store
#pragma unroll
  for (int i = 0; i < DIMS_PER_THREAD; ++i) {
    const int d = tid + i * THREADS;
    if (d >= DV) continue;
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float l1 = l_s[g * MAPS], l2 = l_s[g * MAPS + 1];
      const float a1 = l1 > 0.f ? acc[i][g * MAPS] / l1 : 0.f;
      const float a2 = l2 > 0.f ? acc[i][g * MAPS + 1] / l2 : 0.f;
      ob[g * DV + d] = a1 - lambda * a2;
    }
  }
  __syncthreads();
  for (int g = warp; g < G; g += NWARP) {
    float ss = 0.f;
    for (int d = lane; d < DV; d += 32) ss = fmaf(ob[g * DV + d], ob[g * DV + d], ss);
    ss = warp_sum(ss);
    if (lane == 0) {
      float f = out_scale / sqrtf(ss / (float)DV + sub_eps);
      if (gate) f *= 1.f / (1.f + expf(-to_f32<T>(gate[(size_t)n * gate_stride + kvh * G + g])));
      ssq[g] = f;
    }
  }
  __syncthreads();
  for (int i = tid; i < G * DV; i += THREADS)
    out[((size_t)n * nH + (size_t)kvh * G) * DV + i] = from_f32<T>(ob[i] * ssq[i / DV]);
}

// Combine the partials of one (row, head): per map  w_s = exp(m_s - max m) / sum_s' w_s' l_s',  a = sum w_s acc_s ; then
// the same epilogue as above.
template <typename T>
__global__ void __launch_bounds__(THREADS) diff_attn_reduce_kernel(
    const float* __restrict__ part_o, const float* __restrict__ part_ml, const int* __restrict__ tok_slot,
    const T* __restrict__ gate, int gate_stride, T* __restrict__ out, int nH, int n_splits, float lambda, float sub_eps,
    float out_scale) {
  __shared__ float o_s[DV];
  __shared__ float scratch[33];
  extern __shared__ float wgt[];   // [MAPS][n_splits]: each split's share exp(m_s - max m) / sum, worked out once
  const size_t rh = blockIdx.x;  // row * nH + head
  const int n = (int)(rh / nH), h = (int)(rh % nH);
  if (threadIdx.x < MAPS * 32) {   // one warp per map
    const int m = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float* ml = part_ml + (rh * MAPS + m) * n_splits * 2;
    float mx = -INFINITY;
    for (int s = lane; s < n_splits; s += 32) mx = fmaxf(mx, ml[s * 2]);
    mx = warp_max(mx);
    float denom = 0.f;
    for (int s = lane; s < n_splits; s += 32)
      if (ml[s * 2] != -INFINITY) denom += expf(ml[s * 2] - mx) * ml[s * 2 + 1];
    denom = warp_sum(denom);
    for (int s = lane; s < n_splits; s += 32)
      wgt[m * n_splits + s] = (ml[s * 2] != -INFINITY && denom > 0.f) ? expf(ml[s * 2] - mx) / denom : 0.f;
  }
  __syncthreads();
  float ss = 0.f;
  for (int d = threadIdx.x; d < DV; d += THREADS) {
    float a[MAPS];
#pragma unroll
    for (int m = 0; m < MAPS; ++m) {
      float num = 0.f;
#pragma unroll 4
      for (int s = 0; s < n_splits; ++s) num = fmaf(wgt[m * n_splits + s], part_o[((rh * MAPS + m) * n_splits + s) * DV + d], num);
      a[m] = num;
    }
    const float o = a[0] - lambda * a[1];
    o_s[d] = o;
    ss = fmaf(o, o, ss);
  }
  ss = block_sum(ss, scratch);
  float f = out_scale / sqrtf(ss / (float)DV + sub_eps);
  if (tok_slot[n] < 0) f = 0.f;
  else if (gate) f *= 1.f / (1.f + expf(-to_f32<T>(gate[(size_t)n * gate_stride + h])));
  for (int d = threadIdx.x; d < DV; d += THREADS) out[rh * DV + d] = from_f32<T>(o_s[d] * f);
}

template <typename T>
int launch(const void* q, const void* k_pages, const void* v_pages, const int* page_table, int max_pages,
           const int* tok_slot, const int* tok_pos, const void* gate, int gate_stride, void* out, float* part_o, float* part_ml,
           int n_rows, int nKV, int n_splits, float scale, int window, int chunk, float lambda, float sub_eps, float out_scale,
           cudaStream_t st) {
  if (n_rows <= 0) return 0;
  if (n_splits < 1 || nKV < 1 || nKV > 65535 || n_splits > 4096) return DRYFT_ERR_UNSUPPORTED;
  if (n_splits > 1 && (!part_o || !part_ml)) return DRYFT_ERR_UNSUPPORTED;
  const size_t smem = Smem<T>::bytes();
  if (smem > 227 * 1024) return DRYFT_ERR_UNSUPPORTED;
  static bool attr_set[64] = {false};   // per instantiation and device; set by the first (eager) launch
  if (smem > 48 * 1024) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return DRYFT_ERR_UNSUPPORTED;
    if (!attr_set[dev]) {
      e = cudaFuncSetAttribute(diff_attn_rows_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
      attr_set[dev] = true;
    }
  }
  dim3 grid(n_rows, nKV, n_splits);
  diff_attn_rows_kernel<T><<<grid, THREADS, smem, st>>>((const T*)q, (const T*)k_pages, (const T*)v_pages, page_table, max_pages,
                                                       tok_slot, tok_pos, (const T*)gate, gate_stride, (T*)out, part_o, part_ml,
                                                       nKV, n_splits, scale, window, chunk, lambda, sub_eps, out_scale);
  int rc = launch_status();
  if (rc || n_splits == 1) return rc;
  diff_attn_reduce_kernel<T><<<(unsigned)((size_t)n_rows * nKV * G), THREADS, sizeof(float) * MAPS * n_splits, st>>>(
      part_o, part_ml, tok_slot, (const T*)gate, gate_stride, (T*)out, nKV * G, n_splits, lambda, sub_eps, out_scale);
  return launch_status();
}
}  // namespace

DRYFT_API int dryft_diff_attn_rows_qk_dim() { return DQ; }
DRYFT_API int dryft_diff_attn_rows_v_dim() { return DV; }
DRYFT_API int dryft_diff_attn_rows_group() { return G; }
DRYFT_API int dryft_diff_attn_rows_page() { return PAGE; }

DRYFT_API int dryft_diff_attn_rows(int is_bf16, const void* q, const void* k_pages, const void* v_pages, const int* page_table,
                                   int max_pages, const int* tok_slot, const int* tok_pos, const void* gate, int gate_stride,
                                   void* out, float* part_o, float* part_ml, int n_rows, int nKV, int n_splits, float scale,
                                   int window, int chunk, float lambda, float sub_eps, float out_scale, cudaStream_t st) {
  return is_bf16 ? launch<__nv_bfloat16>(q, k_pages, v_pages, page_table, max_pages, tok_slot, tok_pos, gate, gate_stride, out,
                                         part_o, part_ml, n_rows, nKV, n_splits, scale, window, chunk, lambda, sub_eps, out_scale, st)
                 : launch<float>(q, k_pages, v_pages, page_table, max_pages, tok_slot, tok_pos, gate, gate_stride, out, part_o,
                                 part_ml, n_rows, nKV, n_splits, scale, window, chunk, lambda, sub_eps, out_scale, st);
}
