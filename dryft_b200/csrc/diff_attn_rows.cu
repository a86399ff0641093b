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
//     j >= floor(p / chunk) * chunk   (chunk > 0: only keys of the query's own block of `chunk` positions; blocks are
//                                      aligned to the sequence's start, whatever portions it was fed in)
// Scores, maxima, sums, the combination and its norm are 32-bit.
//
// Grid (rows, kv heads, splits).  One block serves the GROUP query heads of a kv head (2*GROUP maps) for one row over
// a contiguous range of pages.  With one split the block finishes the row itself; otherwise every block leaves its
// un-normalised partials (acc, m, l) per map and draws a ticket, and the block that draws the last ticket of its
// (row, kv head) combines the splits and applies the epilogue -- one launch either way.  In a step whose rows are each
// their sequence's one new token (decode) the same launch also takes the per-map q/k norm and the cache write of the new
// key and value (`fuse`), which prompts leave to kv_maps.cu.
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
    int* __restrict__ tickets,                                      // [N * nKV] zeros; left zero
    // fuse > 0 (a step in which every row is its sequence's one new token): the queries are normalised here from the
    // projection row [q | k | v | ..] instead of being read from q; fuse == 2: the row's new key and value are normalised,
    // written into the cache and used, by the block whose pages hold the row's own position
    const T* __restrict__ proj, int proj_stride, const float* __restrict__ q_w, const float* __restrict__ k_w, float qk_eps,
    int fuse, T* __restrict__ k_pages_w, T* __restrict__ v_pages_w,
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
  float* wgt = ssq + G;                                   // [GM][n_splits]: each split's share, for the block that combines
  __shared__ int s_last;

  const int n = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int nH = nKV * G;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int slot = tok_slot[n];

  if (slot < 0) {  // padding row: defined zeros, no cache access, no ticket (every split of the row comes here)
    if (split == 0)
      for (int i = tid; i < G * DV; i += THREADS) out[(size_t)n * nH * DV + (size_t)kvh * G * DV + i] = from_f32<T>(0.f);
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

  // the block's GM query vectors: head g's map m is row g*MAPS + m, contiguous in q (and in the projection row)
  if (fuse) {
    const T* prow = proj + (size_t)n * proj_stride;
    for (int gm = warp; gm < GM; gm += NWARP) {   // y = T(w * x / sqrt(mean(x^2) + eps)), as the separate kernel rounds it
      const T* src = prow + ((size_t)kvh * GM + gm) * DQ;
      float ss = 0.f;
      for (int c = lane; c < DQ; c += 32) {
        const float x = to_f32<T>(src[c]);
        ss = fmaf(x, x, ss);
      }
      ss = warp_sum(ss);
      const float inv = 1.f / sqrtf(ss / (float)DQ + qk_eps);
      for (int c = lane; c < DQ; c += 32) {
        const float x = to_f32<T>(src[c]) * inv;
        qs[gm * DQ + c] = rnd<T>(q_w ? x * q_w[c] : x);
      }
    }
  } else {
    for (int i = tid; i < GM * DQ; i += THREADS) qs[i] = to_f32<T>(q[((size_t)n * nH + (size_t)kvh * G) * KW + i]);
  }
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
    if (fuse == 2 && pg == last_page) {   // the row's own key and value: into the cache and into this tile
      const T* prow = proj + (size_t)n * proj_stride + (size_t)nH * KW;   // behind the queries: k (nKV x KW), then v (nKV x DV)
      const int r = pos - p0;
      T* kdst = k_pages_w + (((size_t)page * nKV + kvh) * PAGE + r) * KW;
      T* vdst = v_pages_w + (((size_t)page * nKV + kvh) * PAGE + r) * DV;
      for (int m = warp; m < MAPS; m += NWARP) {
        const T* src = prow + (size_t)kvh * KW + m * DQ;
        float ss = 0.f;
        for (int c = lane; c < DQ; c += 32) {
          const float x = to_f32<T>(src[c]);
          ss = fmaf(x, x, ss);
        }
        ss = warp_sum(ss);
        const float inv = 1.f / sqrtf(ss / (float)DQ + qk_eps);
        for (int c = lane; c < DQ; c += 32) {
          const float x = to_f32<T>(src[c]) * inv;
          const T y = from_f32<T>(k_w ? x * k_w[c] : x);
          kt[r * L::KSTRIDE + m * DQ + c] = y;
          kdst[m * DQ + c] = y;
        }
      }
      const T* vsrc = prow + (size_t)nKV * KW + (size_t)kvh * DV;
      for (int c = tid; c < DV; c += THREADS) {
        const T y = vsrc[c];
        vt[r * DV + c] = y;
        vdst[c] = y;
      }
      __syncthreads();
    }
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
    const size_t base = ((size_t)n * nH + kvh * G) * MAPS;   // first of this block's GM maps
#pragma unroll
    for (int i = 0; i < DIMS_PER_THREAD; ++i) {
      const int d = tid + i * THREADS;
      if (d >= DV) continue;
#pragma unroll
      for (int gm = 0; gm < GM; ++gm) part_o[((base + gm) * n_splits + split) * DV + d] = acc[i][gm];
    }
    if (tid < GM) {
      const size_t pi = (base + tid) * n_splits + split;
      part_ml[pi * 2] = m_s[tid];
      part_ml[pi * 2 + 1] = l_s[tid];
    }
    // The block that draws the last ticket of this (row, kv head) combines all splits; nobody waits.  Its reads of the
    // other blocks' partials go to L2 (ld.global.cg) behind the fences.
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      const int t = atomicAdd(&tickets[n * nKV + kvh], 1);
      s_last = (t == n_splits - 1);
      if (s_last) tickets[n * nKV + kvh] = 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    for (int gm = warp; gm < GM; gm += NWARP) {   // per map: w_s = exp(m_s - max m) / sum_s' exp(m_s' - max m) l_s'
      const float* ml = part_ml + (base + gm) * n_splits * 2;
      float mx = -INFINITY;
      for (int sp = lane; sp < n_splits; sp += 32) mx = fmaxf(mx, __ldcg(ml + sp * 2));
      mx = warp_max(mx);
      float denom = 0.f;
      for (int sp = lane; sp < n_splits; sp += 32) {
        const float m = __ldcg(ml + sp * 2);
        if (m != -INFINITY) denom += expf(m - mx) * __ldcg(ml + sp * 2 + 1);
      }
      denom = warp_sum(denom);
      for (int sp = lane; sp < n_splits; sp += 32) {
        const float m = __ldcg(ml + sp * 2);
        wgt[gm * n_splits + sp] = (m != -INFINITY && denom > 0.f) ? expf(m - mx) / denom : 0.f;
      }
    }
    __syncthreads();
    // a thread owns the outputs tid, tid + THREADS, ...; per split all their partials are requested before any is used
    constexpr int ITEMS = (G * DV + THREADS - 1) / THREADS;
    float a[ITEMS][MAPS];
#pragma unroll
    for (int i = 0; i < ITEMS; ++i)
#pragma unroll
      for (int m = 0; m < MAPS; ++m) a[i][m] = 0.f;
#pragma unroll 2
    for (int sp = 0; sp < n_splits; ++sp) {
      float v[ITEMS][MAPS];
#pragma unroll
      for (int i = 0; i < ITEMS; ++i) {
        const int item = min(tid + i * THREADS, G * DV - 1);
        const int g = item / DV, d = item % DV;
#pragma unroll
        for (int m = 0; m < MAPS; ++m) v[i][m] = __ldcg(part_o + ((base + g * MAPS + m) * n_splits + sp) * DV + d);
      }
#pragma unroll
      for (int i = 0; i < ITEMS; ++i) {
        const int g = min(tid + i * THREADS, G * DV - 1) / DV;
#pragma unroll
        for (int m = 0; m < MAPS; ++m) a[i][m] = fmaf(wgt[(g * MAPS + m) * n_splits + sp], v[i][m], a[i][m]);
      }
    }
#pragma unroll
    for (int i = 0; i < ITEMS; ++i)
      if (tid + i * THREADS < G * DV) ob[tid + i * THREADS] = a[i][0] - lambda * a[i][1];
  } else {
    // one split: this block holds everything
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
  }
  // the two maps are combined in ob: normalise over the value dims, gate, store
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

template <typename T>
int launch(const void* q, const void* k_pages, const void* v_pages, const int* page_table, int max_pages,
           const int* tok_slot, const int* tok_pos, const void* gate, int gate_stride, void* out, float* part_o, float* part_ml,
           int* tickets, const void* proj, int proj_stride, const float* q_w, const float* k_w, float qk_eps, int fuse, int n_rows, int nKV, int n_splits, float scale, int window, int chunk, float lambda, float sub_eps, float out_scale,
           cudaStream_t st) {
  if (n_rows <= 0) return 0;
  if (n_splits < 1 || nKV < 1 || nKV > 65535 || n_splits > 4096) return DRYFT_ERR_UNSUPPORTED;
  if (n_splits > 1 && (!part_o || !part_ml || !tickets)) return DRYFT_ERR_UNSUPPORTED;
  if (fuse < 0 || fuse > 2 || (fuse && !proj) || (!fuse && !q)) return DRYFT_ERR_UNSUPPORTED;
  const size_t smem = Smem<T>::bytes() + sizeof(float) * (size_t)GM * n_splits;
  if (smem > 224 * 1024) return DRYFT_ERR_UNSUPPORTED;   // the kernel's few static bytes count against the same 227 KB
  static bool attr_set[64] = {false};   // per instantiation and device; set by the first (eager) launch
  if (smem > 48 * 1024) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return DRYFT_ERR_UNSUPPORTED;
    if (!attr_set[dev]) {
      // the largest there is: the size grows with the split count, and the attribute is set once
      e = cudaFuncSetAttribute(diff_attn_rows_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024);
      if (e != cudaSuccess) return (int)e;
      attr_set[dev] = true;
    }
  }
  dim3 grid(n_rows, nKV, n_splits);
  diff_attn_rows_kernel<T><<<grid, THREADS, smem, st>>>((const T*)q, (const T*)k_pages, (const T*)v_pages, page_table, max_pages,
                                                       tok_slot, tok_pos, (const T*)gate, gate_stride, (T*)out, part_o, part_ml,
                                                       tickets, (const T*)proj, proj_stride, q_w, k_w, qk_eps, fuse, (T*)k_pages,
                                                       (T*)v_pages, nKV, n_splits, scale, window, chunk, lambda, sub_eps, out_scale);
  return launch_status();
}
}  // namespace

DRYFT_API int dryft_diff_attn_rows_qk_dim() { return DQ; }
DRYFT_API int dryft_diff_attn_rows_v_dim() { return DV; }
DRYFT_API int dryft_diff_attn_rows_group() { return G; }
DRYFT_API int dryft_diff_attn_rows_page() { return PAGE; }

DRYFT_API int dryft_diff_attn_rows(int is_bf16, const void* q, const void* k_pages, const void* v_pages, const int* page_table,
                                   int max_pages, const int* tok_slot, const int* tok_pos, const void* gate, int gate_stride,
                                   void* out, float* part_o, float* part_ml, int* tickets, const void* proj, int proj_stride,
                                   const float* q_w, const float* k_w, float qk_eps, int fuse, int n_rows, int nKV, int n_splits,
                                   float scale, int window, int chunk, float lambda, float sub_eps, float out_scale, cudaStream_t st) {
  return is_bf16 ? launch<__nv_bfloat16>(q, k_pages, v_pages, page_table, max_pages, tok_slot, tok_pos, gate, gate_stride, out,
                                         part_o, part_ml, tickets, proj, proj_stride, q_w, k_w, qk_eps, fuse, n_rows, nKV, n_splits,
                                         scale, window, chunk, lambda, sub_eps, out_scale, st)
                 : launch<float>(q, k_pages, v_pages, page_table, max_pages, tok_slot, tok_pos, gate, gate_stride, out, part_o,
                                 part_ml, tickets, proj, proj_stride, q_w, k_w, qk_eps, fuse, n_rows, nKV, n_splits, scale, window,
                                 chunk, lambda, sub_eps, out_scale, st);
}
