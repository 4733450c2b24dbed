// Grouped-query attention over a sliding window of tokens and, before the window, one pooled key and value for every
// whole block of `pool` tokens (the mean of the block's cached keys and of its values):
//   token j is seen from position i if 0 <= i - j < window (window 0: every j <= i, and no blocks);
//   block b (positions b pool .. b pool + pool - 1) is seen if b pool + pool - 1 <= i - window;
//   p_h[x] = exp(s_h[x]) / (sink + sum_x' exp(s_h[x']))     over the seen tokens and blocks x, s = scale q.k,
//            sink = 1 with a sink of score zero in the denominator, else 0;
//   w_h[x] = sum_g mix[h, g] p_g[x]                         (with a mixing matrix; else w = p);
//   o_h    = sum_x w_h[x] v_kv(h)[x],  times sigmoid(gate) if a gate is given.
// Scores, weights and sums are 32-bit in both precisions.
//
//   pool_blocks_kernel       for a step's tokens that end a block: the means over the block's cached rows, written to
//                            the block's row of the pooled pages (the step's keys and values are in their pages already)
//   pooled_attention_kernel  one CTA per token with all heads (mixing needs every head's weight of a key).  Two walks
//                            over the keys in chunks: the first leaves every head's maximum and denominator, the
//                            second forms the weights, mixes them over the heads and adds the weighted values.  The
//                            result does not depend on how a request's tokens are cut into steps.
#include "common.cuh"

namespace atom {

constexpr int kPaThreads = 256;
constexpr int kPaMaxAcc = 16;      // outputs per thread: heads * value size <= 16 * 256

// k_pages [pages, G, page, dk], v_pages [pages, G, page, dv]; pooled pages alike with a block where a token is.
template <typename T>
__global__ void pool_blocks_kernel(const T* __restrict__ k_pages, const T* __restrict__ v_pages, T* __restrict__ pk_pages,
                                   T* __restrict__ pv_pages, const int* __restrict__ block_table, int table_width,
                                   const int* __restrict__ pool_table, int pool_width, int page_size, int64_t num_pages,
                                   int64_t num_pool_pages, const int* __restrict__ positions,
                                   const int* __restrict__ seq_of_token, int G, int dk, int dv, int pool,
                                   int* __restrict__ status) {
  atom::pdl_trigger();
  atom::pdl_wait();
  const int t = blockIdx.x, c = blockIdx.y;
  const int s = seq_of_token[t];
  if (s < 0) return;
  const int pos = positions[t];
  if ((pos + 1) % pool != 0) return;
  const int b = pos / pool;
  const int dst_page = pool_table[(int64_t)s * pool_width + b / page_size];
  if (dst_page < 0 || dst_page >= num_pool_pages) {
    if (threadIdx.x == 0) atomicExch(status, 1);
    return;
  }
  const float inv = 1.f / (float)pool;
  for (int i = threadIdx.x; i < dk + dv; i += blockDim.x) {
    const bool is_k = i < dk;
    const int ch = is_k ? i : i - dk, d = is_k ? dk : dv;
    const T* src = is_k ? k_pages : v_pages;
    float sum = 0.f;
    for (int p = 0; p < pool; ++p) {
      const int j = b * pool + p;
      const int page = block_table[(int64_t)s * table_width + j / page_size];
      if (page < 0 || page >= num_pages) {
        atomicExch(status, 1);
        continue;
      }
      sum += to_float(src[(((int64_t)page * G + c) * page_size + j % page_size) * d + ch]);
    }
    T* dst = is_k ? pk_pages : pv_pages;
    dst[(((int64_t)dst_page * G + c) * page_size + b % page_size) * d + ch] = from_float<T>(sum * inv);
  }
}

struct PaArgs {
  const int* block_table; int table_width;
  const int* pool_table; int pool_width;
  int page_size;
  const int* positions; const int* seq_of_token;
  int H, G, dk, dv, window, pool, chunk;
  float scale; int sink;
  const float* mix;        // [H, H] or null
  int64_t ldq, ldg;
};

// The row of key x of the token's set (blocks first, then the window's tokens) in its pages, for kv head 0.
template <typename T>
__device__ __forceinline__ const T* pa_row(const T* tok_pages, const T* pool_pages, const PaArgs& a, int s, int x, int nb,
                                           int jlo, int d) {
  if (x < nb) {
    const int page = a.pool_table[(int64_t)s * a.pool_width + x / a.page_size];
    return pool_pages + (((int64_t)page * a.G) * a.page_size + x % a.page_size) * d;
  }
  const int j = jlo + (x - nb);
  const int page = a.block_table[(int64_t)s * a.table_width + j / a.page_size];
  return tok_pages + (((int64_t)page * a.G) * a.page_size + j % a.page_size) * d;
}

// Floats between the staged rows of two keys: odd, so that lanes that walk the keys meet different banks.
__host__ __device__ __forceinline__ int pa_stride(int G, int d) { return (G * (d + 1)) | 1; }

// Stages rows [x0, x0 + n) of all kv heads into kv_s [n][pa_stride] (a head's row d + 1 floats apart) as floats.
template <typename T>
__device__ __forceinline__ void pa_stage(float* kv_s, const T* tok_pages, const T* pool_pages, const PaArgs& a, int s,
                                         int x0, int n, int nb, int jlo, int d) {
  const int per = a.G * d;
  for (int e = threadIdx.x; e < n * per; e += kPaThreads) {
    const int x = e / per, rem = e - x * per;
    const int c = rem / d, i = rem - c * d;
    const T* row = pa_row(tok_pages, pool_pages, a, s, x0 + x, nb, jlo, d);
    kv_s[x * pa_stride(a.G, d) + c * (d + 1) + i] = to_float(row[(int64_t)c * a.page_size * d + i]);
  }
}

template <typename T>
__global__ void __launch_bounds__(kPaThreads)
pooled_attention_kernel(T* __restrict__ out, const T* __restrict__ q, const T* __restrict__ k_pages,
                        const T* __restrict__ v_pages, const T* __restrict__ pk_pages, const T* __restrict__ pv_pages,
                        const T* __restrict__ gate, PaArgs a) {
  atom::pdl_trigger();
  atom::pdl_wait();
  const int t = blockIdx.x;
  const int s = a.seq_of_token[t];
  if (s < 0) return;
  const int H = a.H, G = a.G, dk = a.dk, dv = a.dv, C = a.chunk, per = H / G;
  extern __shared__ __align__(16) float pa_smem[];
  float* q_s = pa_smem;                       // [H][dk], times scale
  float* mix_s = q_s + H * dk;                // [H][H]
  float* m_s = mix_s + H * H;                 // [H] running maximum
  float* l_s = m_s + H;                       // [H] denominator, then its inverse
  float* p_s = l_s + H;                       // [H][C] scores, then weights
  float* w_s = p_s + H * C;                   // [H][C] mixed weights
  float* kv_s = w_s + H * C;                  // [C][pa_stride(G, dmax)]
  const int i_pos = a.positions[t];
  const int jlo = a.window > 0 ? max(0, i_pos - a.window + 1) : 0;
  const int nb = (a.window > 0 && a.pool > 0 && i_pos - a.window + 1 > 0) ? (i_pos - a.window + 1) / a.pool : 0;
  const int n_keys = nb + (i_pos - jlo + 1);
  for (int e = threadIdx.x; e < H * dk; e += kPaThreads) q_s[e] = to_float(q[(int64_t)t * a.ldq + e]) * a.scale;
  for (int e = threadIdx.x; e < H * H; e += kPaThreads) mix_s[e] = a.mix ? a.mix[e] : 0.f;
  for (int e = threadIdx.x; e < H; e += kPaThreads) {
    m_s[e] = a.sink ? 0.f : -INFINITY;
    l_s[e] = a.sink ? 1.f : 0.f;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // scores of a staged chunk: thread per (head, key); keys run along the lanes
  auto scores = [&](int n) {
    for (int e = threadIdx.x; e < H * C; e += kPaThreads) {
      const int h = e / C, x = e - h * C;
      if (x < n) {
        const float* kr = kv_s + x * pa_stride(G, dk) + (h / per) * (dk + 1);
        const float* qr = q_s + h * dk;
        float acc = 0.f;
        for (int i = 0; i < dk; ++i) acc = fmaf(qr[i], kr[i], acc);
        p_s[e] = acc;
      }
    }
  };

  // first walk: every head's maximum and denominator
  for (int x0 = 0; x0 < n_keys; x0 += C) {
    const int n = min(C, n_keys - x0);
    pa_stage(kv_s, k_pages, pk_pages, a, s, x0, n, nb, jlo, dk);
    __syncthreads();
    scores(n);
    __syncthreads();
    for (int h = warp; h < H; h += kPaThreads / 32) {
      float mx = -INFINITY;
      for (int x = lane; x < n; x += 32) mx = fmaxf(mx, p_s[h * C + x]);
      mx = warp_max(mx);
      const float m_old = m_s[h], m_new = fmaxf(m_old, mx);
      float sum = 0.f;
      for (int x = lane; x < n; x += 32) sum += expf(p_s[h * C + x] - m_new);
      sum = warp_sum(sum);
      if (lane == 0) {
        l_s[h] = l_s[h] * (m_old == -INFINITY ? 0.f : expf(m_old - m_new)) + sum;
        m_s[h] = m_new;
      }
    }
    __syncthreads();
  }
  for (int e = threadIdx.x; e < H; e += kPaThreads) l_s[e] = 1.f / l_s[e];
  __syncthreads();

  // second walk: weights, mixed over the heads, times the values
  float acc[kPaMaxAcc];
#pragma unroll
  for (int u = 0; u < kPaMaxAcc; ++u) acc[u] = 0.f;
  for (int x0 = 0; x0 < n_keys; x0 += C) {
    const int n = min(C, n_keys - x0);
    pa_stage(kv_s, k_pages, pk_pages, a, s, x0, n, nb, jlo, dk);
    __syncthreads();
    scores(n);
    __syncthreads();
    for (int e = threadIdx.x; e < H * C; e += kPaThreads) {
      const int h = e / C, x = e - h * C;
      if (x < n) p_s[e] = expf(p_s[e] - m_s[h]) * l_s[h];
    }
    pa_stage(kv_s, v_pages, pv_pages, a, s, x0, n, nb, jlo, dv);      // (the keys have been read: scores are in p_s)
    __syncthreads();
    const float* wt = p_s;
    if (a.mix) {
      for (int e = threadIdx.x; e < H * C; e += kPaThreads) {
        const int h = e / C, x = e - h * C;
        if (x < n) {
          float sum = 0.f;
          for (int g = 0; g < H; ++g) sum = fmaf(mix_s[h * H + g], p_s[g * C + x], sum);
          w_s[e] = sum;
        }
      }
      __syncthreads();
      wt = w_s;
    }
#pragma unroll
    for (int u = 0; u < kPaMaxAcc; ++u) {
      const int e = threadIdx.x + u * kPaThreads;
      if (e < H * dv) {
        const int h = e / dv, jj = e - h * dv;
        const float* vr = kv_s + (h / per) * (dv + 1) + jj;
        const float* wr = wt + h * C;
        float sum = acc[u];
        const int rs = pa_stride(G, dv);
        for (int x = 0; x < n; ++x) sum = fmaf(wr[x], vr[x * rs], sum);
        acc[u] = sum;
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int u = 0; u < kPaMaxAcc; ++u) {
    const int e = threadIdx.x + u * kPaThreads;
    if (e < H * dv) {
      float o = acc[u];
      if (gate) o = o / (1.f + expf(-to_float(gate[(int64_t)t * a.ldg + e])));
      out[(int64_t)t * H * dv + e] = from_float<T>(o);
    }
  }
}

static inline size_t pa_smem_bytes(int H, int G, int dk, int dv, int C) {
  const int dmax = dk > dv ? dk : dv;
  return sizeof(float) * ((size_t)H * dk + (size_t)H * H + 2 * H + 2 * (size_t)H * C + (size_t)C * pa_stride(G, dmax));
}

static inline int pa_chunk(int H, int G, int dk, int dv) {
  for (int C = 64; C >= 8; C >>= 1)
    if (pa_smem_bytes(H, G, dk, dv, C) <= 96 * 1024) return C;
  for (int C = 64; C >= 4; C >>= 1)
    if (pa_smem_bytes(H, G, dk, dv, C) <= 200 * 1024) return C;
  return 0;
}

}  // namespace atom

ATOM_EXPORT int atom_pooled_attention_supports(int H, int G, int dk, int dv) {
  if (H <= 0 || G <= 0 || H % G || dk <= 0 || dv <= 0 || H * dv > atom::kPaMaxAcc * atom::kPaThreads) return 0;
  return atom::pa_chunk(H, G, dk, dv) > 0;
}

ATOM_EXPORT int atom_pool_blocks(const void* k_pages, const void* v_pages, void* pk_pages, void* pv_pages, int dtype,
                                 const int* block_table, int table_width, const int* pool_table, int pool_width,
                                 int page_size, int64_t num_pages, int64_t num_pool_pages, const int* positions,
                                 const int* seq_of_token, int T, int G, int dk, int dv, int pool, int* status,
                                 cudaStream_t stream) {
  if (T <= 0) return ATOM_OK;
  if (G <= 0 || G > 65535 || dk <= 0 || dv <= 0 || pool <= 0 || page_size <= 0) return ATOM_ERR_ARG;
  const int threads = dk + dv >= 256 ? 256 : 128;
  if (dtype == ATOM_F32)
    atom::launch_pdl(atom::pool_blocks_kernel<float>, dim3(T, G), dim3(threads), 0, stream, (const float*)k_pages,
                     (const float*)v_pages, (float*)pk_pages, (float*)pv_pages, block_table, table_width, pool_table,
                     pool_width, page_size, num_pages, num_pool_pages, positions, seq_of_token, G, dk, dv, pool, status);
  else if (dtype == ATOM_BF16)
    atom::launch_pdl(atom::pool_blocks_kernel<__nv_bfloat16>, dim3(T, G), dim3(threads), 0, stream,
                     (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, (__nv_bfloat16*)pk_pages,
                     (__nv_bfloat16*)pv_pages, block_table, table_width, pool_table, pool_width, page_size, num_pages,
                     num_pool_pages, positions, seq_of_token, G, dk, dv, pool, status);
  else
    return ATOM_ERR_ARG;
  return atom::check_launch();
}

// out [T, H dv]; q [T, .] rows ldq apart, heads in a row; gate (or null) rows ldg apart; mix [H, H] float or null.
ATOM_EXPORT int atom_pooled_attention(void* out, const void* q, int64_t ldq, const void* k_pages, const void* v_pages,
                                      const void* pk_pages, const void* pv_pages, int dtype, const int* block_table,
                                      int table_width, const int* pool_table, int pool_width, int page_size,
                                      const int* positions, const int* seq_of_token, int T, int H, int G, int dk, int dv,
                                      float scale, int window, int pool, int sink, const float* mix, const void* gate,
                                      int64_t ldg, cudaStream_t stream) {
  if (T <= 0) return ATOM_OK;
  if (!atom_pooled_attention_supports(H, G, dk, dv) || window < 0 || pool < 0 || page_size <= 0) return ATOM_ERR_ARG;
  if (pool > 0 && window > 0 && (!pk_pages || !pv_pages || !pool_table)) return ATOM_ERR_ARG;
  atom::PaArgs a;
  a.block_table = block_table; a.table_width = table_width;
  a.pool_table = pool_table; a.pool_width = pool_width;
  a.page_size = page_size; a.positions = positions; a.seq_of_token = seq_of_token;
  a.H = H; a.G = G; a.dk = dk; a.dv = dv; a.window = window; a.pool = pool;
  a.chunk = atom::pa_chunk(H, G, dk, dv);
  a.scale = scale; a.sink = sink; a.mix = mix; a.ldq = ldq; a.ldg = ldg;
  const size_t smem = atom::pa_smem_bytes(H, G, dk, dv, a.chunk);
  if (dtype == ATOM_F32) {
    auto kern = atom::pooled_attention_kernel<float>;
    if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return ATOM_ERR_LAUNCH;
    atom::launch_pdl(kern, dim3(T), dim3(atom::kPaThreads), smem, stream, (float*)out, (const float*)q,
                     (const float*)k_pages, (const float*)v_pages, (const float*)pk_pages, (const float*)pv_pages,
                     (const float*)gate, a);
  } else if (dtype == ATOM_BF16) {
    auto kern = atom::pooled_attention_kernel<__nv_bfloat16>;
    if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return ATOM_ERR_LAUNCH;
    atom::launch_pdl(kern, dim3(T), dim3(atom::kPaThreads), smem, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)q,
                     (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, (const __nv_bfloat16*)pk_pages,
                     (const __nv_bfloat16*)pv_pages, (const __nv_bfloat16*)gate, a);
  } else {
    return ATOM_ERR_ARG;
  }
  return atom::check_launch();
}
