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
//   pooled_attention_split_kernel, pooled_attention_merge_kernel
//                            for steps of few tokens (decoding): the keys of a token are shared out among CTAs, which
//                            cannot know a head's denominator before all have finished.  A share therefore keeps, for
//                            every head g and EVERY kv head c, the unnormalised sum U[g][c] = sum_x exp(s_g[x] - m_g) v_c[x]
//                            with its running maximum m_g and sum l_g (one walk, keys and values read once); the merge
//                            kernel puts the shares together, divides, and mixes over the heads:
//                            o_h = sum_g mix[h][g] U[g][kv(h)] / l_g, the sink as one more term of l_g.
#include "common.cuh"

namespace atom {

constexpr int kPaThreads = 256;
constexpr int kPaMaxAcc = 16;      // outputs per thread: heads * value size <= 16 * 256

// 16 bytes of a row as floats.
template <typename T, int V> struct PaVecLoad {
  __device__ static __forceinline__ void load(const T* p, float (&o)[V]) { o[0] = to_float(p[0]); }
};
template <> struct PaVecLoad<float, 4> {
  __device__ static __forceinline__ void load(const float* p, float (&o)[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
  }
};
template <> struct PaVecLoad<__nv_bfloat16, 8> {
  __device__ static __forceinline__ void load(const __nv_bfloat16* p, float (&o)[8]) {
    const uint4 q = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = __bfloat1622float2(h[e]);
      o[2 * e] = f.x;
      o[2 * e + 1] = f.y;
    }
  }
};

// k_pages [pages, G, page, dk], v_pages [pages, G, page, dv]; pooled pages alike with a block where a token is.  A
// thread owns V channels in a row (16 bytes of a cached row where the sizes allow, else one) and walks the block's
// positions in order, eight loads on their way together.
template <typename T, int V>
__global__ void pool_blocks_kernel(const T* __restrict__ k_pages, const T* __restrict__ v_pages, T* __restrict__ pk_pages,
                                   T* __restrict__ pv_pages, const int* __restrict__ block_table, int table_width,
                                   const int* __restrict__ pool_table, int pool_width, int page_size, int64_t num_pages,
                                   int64_t num_pool_pages, const int* __restrict__ positions,
                                   const int* __restrict__ seq_of_token, int G, int dk, int dv, int pool,
                                   int* __restrict__ status) {
  atom::pdl_trigger();
  atom::pdl_wait();
  const int t = blockIdx.x;
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
  const int nk = dk / V, nvv = dv / V;
  bool bad = false;
  for (int idx = threadIdx.x; idx < G * (nk + nvv); idx += blockDim.x) {
    const int c = idx / (nk + nvv), i = idx - c * (nk + nvv);
    const bool is_k = i < nk;
    const int ch = (is_k ? i : i - nk) * V, d = is_k ? dk : dv;
    const T* src = is_k ? k_pages : v_pages;
    float sum[V];
#pragma unroll
    for (int k = 0; k < V; ++k) sum[k] = 0.f;
    for (int p0 = 0; p0 < pool; p0 += 8) {
      float v[8][V];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
#pragma unroll
        for (int k = 0; k < V; ++k) v[u][k] = 0.f;
        const int j = b * pool + p0 + u;
        if (p0 + u < pool) {
          const int page = block_table[(int64_t)s * table_width + j / page_size];
          if (page < 0 || page >= num_pages) {
            bad = true;
          } else {
            const T* row = src + (((int64_t)page * G + c) * page_size + j % page_size) * d + ch;
            if (V == 1) v[u][0] = to_float(row[0]);
            else PaVecLoad<T, V>::load(row, v[u]);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 8; ++u)
#pragma unroll
        for (int k = 0; k < V; ++k) sum[k] += v[u][k];
    }
    T* dst = (is_k ? pk_pages : pv_pages) + (((int64_t)dst_page * G + c) * page_size + b % page_size) * d + ch;
#pragma unroll
    for (int k = 0; k < V; ++k) dst[k] = from_float<T>(sum[k] * inv);
  }
  if (bad) atomicExch(status, 1);
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

// The row of key x of the token's set (blocks first, then the window's tokens) in its pages, for kv head 0, counted in
// rows: >= 0 in the token pages, < 0 (as -1 - row) in the pooled pages.
__device__ __forceinline__ int pa_row(const PaArgs& a, int s, int x, int nb, int jlo) {
  if (x < nb) {
    const int page = a.pool_table[(int64_t)s * a.pool_width + x / a.page_size];
    return -1 - (page * a.G * a.page_size + x % a.page_size);
  }
  const int j = jlo + (x - nb);
  const int page = a.block_table[(int64_t)s * a.table_width + j / a.page_size];
  return page * a.G * a.page_size + j % a.page_size;
}

// Floats between the staged rows of two keys: odd, so that lanes that walk the keys meet different banks.
__host__ __device__ __forceinline__ int pa_stride(int G, int d) { return (G * (d + 1)) | 1; }

template <typename T> struct PaVec;
template <> struct PaVec<float> {
  static constexpr int N = 4;
  __device__ static __forceinline__ void load(const float* p, float (&o)[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
  }
};
template <> struct PaVec<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static __forceinline__ void load(const __nv_bfloat16* p, float (&o)[8]) {
    const uint4 q = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = __bfloat1622float2(h[e]);
      o[2 * e] = f.x;
      o[2 * e + 1] = f.y;
    }
  }
};

// Stages rows [x0, x0 + n) of all kv heads into kv_s [n][pa_stride] (a head's row d + 1 floats apart) as floats.  The
// rows' places are looked up first (row_s, unless `reuse` says that it holds this chunk's already), so that the copies
// do not wait for a table entry each and several of them, 16 bytes each, are on their way per thread.
template <typename T>
__device__ __forceinline__ void pa_stage(float* kv_s, int* row_s, const T* tok_pages, const T* pool_pages, const PaArgs& a,
                                         int s, int x0, int n, int nb, int jlo, int d, bool reuse) {
  if (!reuse) {
    for (int x = threadIdx.x; x < n; x += kPaThreads) row_s[x] = pa_row(a, s, x0 + x, nb, jlo);
    __syncthreads();
  }
  constexpr int V = PaVec<T>::N;
  const int rs = pa_stride(a.G, d);
  if (d % V == 0) {
    const int nv = d / V, per = a.G * nv;
#pragma unroll 4
    for (int e = threadIdx.x; e < n * per; e += kPaThreads) {
      const int x = e / per, rem = e - x * per;
      const int c = rem / nv, iv = rem - c * nv;
      const int row = row_s[x];
      const T* src = (row >= 0 ? tok_pages + (int64_t)row * d : pool_pages + (int64_t)(-1 - row) * d) +
                     (int64_t)c * a.page_size * d + iv * V;
      float o[V];
      PaVec<T>::load(src, o);
      float* dst = kv_s + x * rs + c * (d + 1) + iv * V;
#pragma unroll
      for (int k = 0; k < V; ++k) dst[k] = o[k];
    }
  } else {
    const int per = a.G * d;
#pragma unroll 4
    for (int e = threadIdx.x; e < n * per; e += kPaThreads) {
      const int x = e / per, rem = e - x * per;
      const int c = rem / d, i = rem - c * d;
      const int row = row_s[x];
      const T* src = (row >= 0 ? tok_pages + (int64_t)row * d : pool_pages + (int64_t)(-1 - row) * d) +
                     (int64_t)c * a.page_size * d;
      kv_s[x * rs + c * (d + 1) + i] = to_float(src[i]);
    }
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
  __shared__ int row_s[64];                   // where the chunk's keys lie
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
    pa_stage(kv_s, row_s, k_pages, pk_pages, a, s, x0, n, nb, jlo, dk, false);
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
    pa_stage(kv_s, row_s, k_pages, pk_pages, a, s, x0, n, nb, jlo, dk, false);
    __syncthreads();
    scores(n);
    __syncthreads();
    for (int e = threadIdx.x; e < H * C; e += kPaThreads) {
      const int h = e / C, x = e - h * C;
      if (x < n) p_s[e] = expf(p_s[e] - m_s[h]) * l_s[h];
    }
    pa_stage(kv_s, row_s, v_pages, pv_pages, a, s, x0, n, nb, jlo, dv, true);      // (the keys have been read: scores are in p_s)
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

constexpr int kPaMaxU = 32;        // sums per thread of the split kernel: (heads, padded) * columns of a thread

// part: [T, nsplit, 2 H + H G dv]: maxima, sums, then U[g][c][:].  A thread owns up to 32 / HP of the G dv value
// columns with the sums of all heads (HP: heads padded to a multiple of 4), so that a key costs it one load per column
// and HP / 4 loads of weights for HP multiply-adds per column.
template <typename T, int HP>
__global__ void __launch_bounds__(kPaThreads)
pooled_attention_split_kernel(float* __restrict__ part, const T* __restrict__ q, const T* __restrict__ k_pages,
                              const T* __restrict__ v_pages, const T* __restrict__ pk_pages, const T* __restrict__ pv_pages,
                              PaArgs a, int nsplit) {
  atom::pdl_trigger();
  atom::pdl_wait();
  constexpr int NC = kPaMaxU / HP;            // value columns per thread
  const int t = blockIdx.x, split = blockIdx.y;
  const int s = a.seq_of_token[t];
  if (s < 0) return;
  const int H = a.H, G = a.G, dk = a.dk, dv = a.dv, C = a.chunk, per = H / G;
  extern __shared__ __align__(16) float pa_smem[];
  float* p_s = pa_smem;                       // [C][HP] scores, then exp(s - m)
  float* q_s = p_s + C * HP;                  // [H][dk], times scale
  float* m_s = q_s + H * dk;                  // [HP] running maximum
  float* l_s = m_s + HP;                      // [HP] running sum
  float* c_s = l_s + HP;                      // [HP] correction of the sums so far
  float* kv_s = c_s + HP;                     // [C][pa_stride(G, dmax)]
  __shared__ int row_s[64];                   // where the chunk's keys lie
  const int i_pos = a.positions[t];
  const int jlo = a.window > 0 ? max(0, i_pos - a.window + 1) : 0;
  const int nb = (a.window > 0 && a.pool > 0 && i_pos - a.window + 1 > 0) ? (i_pos - a.window + 1) / a.pool : 0;
  const int n_keys = nb + (i_pos - jlo + 1);
  const int share = ((n_keys + nsplit - 1) / nsplit + C - 1) / C * C;
  const int x_lo = split * share, x_hi = min(n_keys, x_lo + share);
  for (int e = threadIdx.x; e < H * dk; e += kPaThreads) q_s[e] = to_float(q[(int64_t)t * a.ldq + e]) * a.scale;
  for (int e = threadIdx.x; e < HP; e += kPaThreads) {
    m_s[e] = -INFINITY;
    l_s[e] = 0.f;
    c_s[e] = 0.f;
  }
  for (int e = threadIdx.x; e < C * HP; e += kPaThreads) p_s[e] = 0.f;       // (the padding heads' weights stay zero)
  float U[NC][HP];
  int voff[NC];
#pragma unroll
  for (int nc = 0; nc < NC; ++nc) {
    const int col = threadIdx.x + nc * kPaThreads;
    voff[nc] = col < G * dv ? (col / dv) * (dv + 1) + col % dv : -1;
#pragma unroll
    for (int g = 0; g < HP; ++g) U[nc][g] = 0.f;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rs = pa_stride(G, dv);
  for (int x0 = x_lo; x0 < x_hi; x0 += C) {
    const int n = min(C, x_hi - x0);
    pa_stage(kv_s, row_s, k_pages, pk_pages, a, s, x0, n, nb, jlo, dk, false);
    __syncthreads();
    for (int e = threadIdx.x; e < H * C; e += kPaThreads) {
      const int h = e / C, x = e - h * C;
      if (x < n) {
        const float* kr = kv_s + x * pa_stride(G, dk) + (h / per) * (dk + 1);
        const float* qr = q_s + h * dk;
        float acc = 0.f;
        for (int i = 0; i < dk; ++i) acc = fmaf(qr[i], kr[i], acc);
        p_s[x * HP + h] = acc;
      }
    }
    __syncthreads();
    for (int h = warp; h < H; h += kPaThreads / 32) {
      float mx = -INFINITY;
      for (int x = lane; x < n; x += 32) mx = fmaxf(mx, p_s[x * HP + h]);
      mx = warp_max(mx);
      const float m_old = m_s[h], m_new = fmaxf(m_old, mx);
      float sum = 0.f;
      for (int x = lane; x < n; x += 32) {
        const float p = expf(p_s[x * HP + h] - m_new);
        p_s[x * HP + h] = p;
        sum += p;
      }
      sum = warp_sum(sum);
      if (lane == 0) {
        const float corr = m_old == -INFINITY ? 0.f : expf(m_old - m_new);
        c_s[h] = corr;
        l_s[h] = l_s[h] * corr + sum;
        m_s[h] = m_new;
      }
    }
    pa_stage(kv_s, row_s, v_pages, pv_pages, a, s, x0, n, nb, jlo, dv, true);      // (the keys have been read: scores are in p_s)
    __syncthreads();
#pragma unroll
    for (int nc = 0; nc < NC; ++nc)
#pragma unroll
      for (int g = 0; g < HP; ++g) U[nc][g] *= c_s[g];
    for (int x = 0; x < n; ++x) {
      float w[HP];
#pragma unroll
      for (int g4 = 0; g4 < HP / 4; ++g4) {
        const float4 w4 = *reinterpret_cast<const float4*>(p_s + x * HP + 4 * g4);
        w[4 * g4] = w4.x; w[4 * g4 + 1] = w4.y; w[4 * g4 + 2] = w4.z; w[4 * g4 + 3] = w4.w;
      }
#pragma unroll
      for (int nc = 0; nc < NC; ++nc) {
        const float v = voff[nc] >= 0 ? kv_s[x * rs + voff[nc]] : 0.f;
#pragma unroll
        for (int g = 0; g < HP; ++g) U[nc][g] = fmaf(w[g], v, U[nc][g]);
      }
    }
    __syncthreads();
  }
  const int n_out = H * G * dv;
  float* pt = part + ((int64_t)t * nsplit + split) * (2 * H + n_out);
  for (int e = threadIdx.x; e < H; e += kPaThreads) {
    pt[e] = m_s[e];
    pt[H + e] = l_s[e];
  }
#pragma unroll
  for (int nc = 0; nc < NC; ++nc) {
    const int col = threadIdx.x + nc * kPaThreads;          // = c * dv + jj
    if (col < G * dv) {
#pragma unroll
      for (int g = 0; g < HP; ++g)
        if (g < H) pt[2 * H + (int64_t)g * G * dv + col] = U[nc][g];
    }
  }
}

// A CTA per (token, kv head c, 32 value columns): f[split][g] = exp(m_split,g - M_g) / L_g; V[g][:] = sum_split f
// U_split[g][c][:] to shared memory (every load coalesced, the shares' loads of a thread on their way together); then
// out[t][h][:] = sum_g mix[h][g] V[g][:] for the heads h of c's group.
constexpr int kPaMergeCols = 32;

template <typename T>
__global__ void pooled_attention_merge_kernel(T* __restrict__ out, const float* __restrict__ part,
                                              const int* __restrict__ seq_of_token, int H, int G, int dv, int nsplit,
                                              int sink, const float* __restrict__ mix, const T* __restrict__ gate,
                                              int64_t ldg) {
  atom::pdl_trigger();
  atom::pdl_wait();
  const int t = blockIdx.x, c = blockIdx.y, j0 = blockIdx.z * kPaMergeCols;
  if (seq_of_token[t] < 0) return;
  extern __shared__ float f_s[];              // [nsplit][H], then mix [H][H], then V [H][32]
  float* mix_s = f_s + nsplit * H;
  float* V_s = mix_s + H * H;
  const int n_out = H * G * dv, per = H / G;
  const int nj = min(kPaMergeCols, dv - j0);
  const int64_t stride = 2 * H + n_out;
  const float* pt = part + (int64_t)t * nsplit * stride;
  for (int g = threadIdx.x; g < H; g += blockDim.x) {
    float M = sink ? 0.f : -INFINITY;
    for (int sp = 0; sp < nsplit; ++sp) M = fmaxf(M, pt[sp * stride + g]);
    float L = sink ? expf(-M) : 0.f;
    for (int sp = 0; sp < nsplit; ++sp) {
      const float m = pt[sp * stride + g];
      const float f = m == -INFINITY ? 0.f : expf(m - M);
      f_s[sp * H + g] = f;
      L = fmaf(pt[sp * stride + H + g], f, L);
    }
    const float inv = L > 0.f ? 1.f / L : 0.f;
    for (int sp = 0; sp < nsplit; ++sp) f_s[sp * H + g] *= inv;
  }
  for (int e = threadIdx.x; e < H * H; e += blockDim.x) mix_s[e] = mix ? mix[e] : ((e / H == e % H) ? 1.f : 0.f);
  __syncthreads();
  for (int e = threadIdx.x; e < H * kPaMergeCols; e += blockDim.x) {
    const int g = e / kPaMergeCols, jj = e - g * kPaMergeCols;
    float a = 0.f;
    if (jj < nj) {
      const float* u = pt + 2 * H + (g * G + c) * dv + j0 + jj;
      for (int sp0 = 0; sp0 < nsplit; sp0 += 8) {
        float v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = sp0 + k < nsplit ? u[(sp0 + k) * stride] : 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k)
          if (sp0 + k < nsplit) a = fmaf(f_s[(sp0 + k) * H + g], v[k], a);
      }
    }
    V_s[e] = a;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < per * kPaMergeCols; e += blockDim.x) {
    const int h = c * per + e / kPaMergeCols, jj = e % kPaMergeCols;
    if (jj >= nj) continue;
    float o = 0.f;
    for (int g = 0; g < H; ++g) o = fmaf(mix_s[h * H + g], V_s[g * kPaMergeCols + jj], o);
    const int col = h * dv + j0 + jj;
    if (gate) o = o / (1.f + expf(-to_float(gate[(int64_t)t * ldg + col])));
    out[(int64_t)t * H * dv + col] = from_float<T>(o);
  }
}

static inline int pa_heads_padded(int H) { return H <= 4 ? 4 : (H <= 8 ? 8 : (H <= 16 ? 16 : 32)); }

static inline size_t pa_split_smem_bytes(int H, int G, int dk, int dv, int C) {
  const int dmax = dk > dv ? dk : dv, HP = pa_heads_padded(H);
  return sizeof(float) * ((size_t)H * dk + 3 * HP + (size_t)HP * C + (size_t)C * pa_stride(G, dmax));
}

static inline int pa_split_chunk(int H, int G, int dk, int dv) {
  for (int C = 64; C >= 8; C >>= 1)
    if (pa_split_smem_bytes(H, G, dk, dv, C) <= 100 * 1024) return C;
  return 0;
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

ATOM_EXPORT int atom_pooled_attention_split_supports(int H, int G, int dk, int dv) {
  if (H <= 0 || H > 32 || G <= 0 || H % G || dk <= 0 || dv <= 0) return 0;
  if (G * dv > (atom::kPaMaxU / atom::pa_heads_padded(H)) * atom::kPaThreads) return 0;      // a thread's columns
  return atom::pa_split_chunk(H, G, dk, dv) > 0;
}

// The keys of every token shared out among nsplit CTAs; part holds T * nsplit * (2 H + H G dv) floats.
ATOM_EXPORT int atom_pooled_attention_split(void* out, float* part, const void* q, int64_t ldq, const void* k_pages,
                                            const void* v_pages, const void* pk_pages, const void* pv_pages, int dtype,
                                            const int* block_table, int table_width, const int* pool_table,
                                            int pool_width, int page_size, const int* positions,
                                            const int* seq_of_token, int T, int H, int G, int dk, int dv, float scale,
                                            int window, int pool, int sink, const float* mix, const void* gate,
                                            int64_t ldg, int nsplit, cudaStream_t stream) {
  if (T <= 0) return ATOM_OK;
  if (!atom_pooled_attention_split_supports(H, G, dk, dv) || window < 0 || pool < 0 || page_size <= 0 || nsplit < 1 ||
      nsplit > 256 || !part)
    return ATOM_ERR_ARG;
  if (pool > 0 && window > 0 && (!pk_pages || !pv_pages || !pool_table)) return ATOM_ERR_ARG;
  atom::PaArgs a;
  a.block_table = block_table; a.table_width = table_width;
  a.pool_table = pool_table; a.pool_width = pool_width;
  a.page_size = page_size; a.positions = positions; a.seq_of_token = seq_of_token;
  a.H = H; a.G = G; a.dk = dk; a.dv = dv; a.window = window; a.pool = pool;
  a.chunk = atom::pa_split_chunk(H, G, dk, dv);
  a.scale = scale; a.sink = sink; a.mix = mix; a.ldq = ldq; a.ldg = ldg;
  const size_t smem = atom::pa_split_smem_bytes(H, G, dk, dv, a.chunk);
  const size_t msmem = sizeof(float) * ((size_t)nsplit * H + (size_t)H * H + (size_t)H * atom::kPaMergeCols);
  const int mthreads = H * atom::kPaMergeCols >= 256 ? 256 : 128;
  if (msmem > 48 * 1024) return ATOM_ERR_ARG;
  const dim3 grid(T, nsplit), mgrid(T, G, (dv + atom::kPaMergeCols - 1) / atom::kPaMergeCols);
#define ATOM_PA_SPLIT(TT, HP)                                                                                         \
  {                                                                                                                   \
    auto kern = atom::pooled_attention_split_kernel<TT, HP>;                                                          \
    if (smem > 48 * 1024 &&                                                                                           \
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)            \
      return ATOM_ERR_LAUNCH;                                                                                         \
    atom::launch_pdl(kern, grid, dim3(atom::kPaThreads), smem, stream, part, (const TT*)q, (const TT*)k_pages,        \
                     (const TT*)v_pages, (const TT*)pk_pages, (const TT*)pv_pages, a, nsplit);                        \
    atom::launch_pdl(atom::pooled_attention_merge_kernel<TT>, mgrid, dim3(mthreads), msmem, stream, (TT*)out,         \
                     (const float*)part, seq_of_token, H, G, dv, nsplit, sink, mix, (const TT*)gate, ldg);            \
  }
#define ATOM_PA_SPLIT_BY_HEADS(TT)                       \
  switch (atom::pa_heads_padded(H)) {                    \
    case 4: ATOM_PA_SPLIT(TT, 4) break;                  \
    case 8: ATOM_PA_SPLIT(TT, 8) break;                  \
    case 16: ATOM_PA_SPLIT(TT, 16) break;                \
    default: ATOM_PA_SPLIT(TT, 32) break;                \
  }
  if (dtype == ATOM_F32) {
    ATOM_PA_SPLIT_BY_HEADS(float)
  } else if (dtype == ATOM_BF16) {
    ATOM_PA_SPLIT_BY_HEADS(__nv_bfloat16)
  } else {
    return ATOM_ERR_ARG;
  }
#undef ATOM_PA_SPLIT_BY_HEADS
#undef ATOM_PA_SPLIT
  return atom::check_launch();
}

ATOM_EXPORT int atom_pool_blocks(const void* k_pages, const void* v_pages, void* pk_pages, void* pv_pages, int dtype,
                                 const int* block_table, int table_width, const int* pool_table, int pool_width,
                                 int page_size, int64_t num_pages, int64_t num_pool_pages, const int* positions,
                                 const int* seq_of_token, int T, int G, int dk, int dv, int pool, int* status,
                                 cudaStream_t stream) {
  if (T <= 0) return ATOM_OK;
  if (G <= 0 || G > 65535 || dk <= 0 || dv <= 0 || pool <= 0 || page_size <= 0) return ATOM_ERR_ARG;
#define ATOM_POOL_BLOCKS(TT, VV)                                                                                      \
  {                                                                                                                   \
    const int work = G * (dk / VV + dv / VV);                                                                         \
    const int threads = work >= 256 ? 256 : (work >= 128 ? 128 : 64);                                                 \
    atom::launch_pdl(atom::pool_blocks_kernel<TT, VV>, dim3(T), dim3(threads), 0, stream, (const TT*)k_pages,         \
                     (const TT*)v_pages, (TT*)pk_pages, (TT*)pv_pages, block_table, table_width, pool_table, pool_width, \
                     page_size, num_pages, num_pool_pages, positions, seq_of_token, G, dk, dv, pool, status);          \
  }
  const bool al = ((uintptr_t)k_pages % 16 == 0) && ((uintptr_t)v_pages % 16 == 0);
  if (dtype == ATOM_F32) {
    if (al && dk % 4 == 0 && dv % 4 == 0) ATOM_POOL_BLOCKS(float, 4) else ATOM_POOL_BLOCKS(float, 1)
  } else if (dtype == ATOM_BF16) {
    if (al && dk % 8 == 0 && dv % 8 == 0) ATOM_POOL_BLOCKS(__nv_bfloat16, 8) else ATOM_POOL_BLOCKS(__nv_bfloat16, 1)
  } else {
    return ATOM_ERR_ARG;
  }
#undef ATOM_POOL_BLOCKS
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
