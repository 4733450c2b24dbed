// Attention over a cached latent: every token keeps one row [c | kr] in its page, c the normalised latent
// of R numbers from which every head's unrotated keys and its values are linear maps, kr the rotated key
// part of rd numbers that all heads share.  With the key map folded into the query, q'_h = W_uk,h^T q_h,
// the score of head h is  scale * (q'_h . c_j + qr_h . kr_j): all heads read the same row of R + rd
// numbers, and the weighted sum of the rows' first R numbers is the head's output before its value map.
//
//   latent_prepare_kernel   per token: RMSNorm of the query latent; RMSNorm of the first R numbers of the
//                           key/value projection, rotation of the last rd, both written to the page row
//   rotate_pairs_kernel     rotates vectors' leading dims numbers by position * frequency (pairs (i, i + dims/2)),
//                           copies what follows, into a strided 32-bit destination
//   latent_attention_kernel one CTA per (token, group of heads, share of the keys): sliding window, online
//                           softmax in 32-bit, a learned sink per head in the denominator
//   latent_merge_kernel     puts the shares of the keys together
// Angles, norms, scores, weights and sums are 32-bit in both precisions.
#include "common.cuh"

namespace atom {

__device__ __forceinline__ void rotate_pair(float u, float v, float angle, float mag, float& ou, float& ov) {
  float s, c;
  sincosf(angle, &s, &c);
  s *= mag;
  c *= mag;
  ou = u * c - v * s;
  ov = v * c + u * s;
}

// proj: [T, ld] rows hold the query latent at q_off (Rq numbers) and, if pages != null, [c raw | kr raw] at kv_off.
template <typename T>
__global__ void latent_prepare_kernel(T* __restrict__ cq, const T* __restrict__ proj, int64_t ld, int q_off, int Rq,
                                      const void* __restrict__ wq, int kv_off, int R, int rd, int dims,
                                      const void* __restrict__ wkv, int w_dtype, float eps,
                                      const float* __restrict__ freq, float mag, const int* __restrict__ positions,
                                      const int* __restrict__ seq_of_token, const int* __restrict__ block_table,
                                      int table_width, int page_size, T* __restrict__ pages, int64_t num_pages,
                                      int* __restrict__ status) {
  atom::pdl_trigger();
  atom::pdl_wait();
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  const int s = seq_of_token[t];
  if (s < 0) return;
  const T* row = proj + (int64_t)t * ld;
  if (Rq > 0) {       // (0: the queries pass no latent of their own)
    float ss = 0.f;
    for (int i = threadIdx.x; i < Rq; i += blockDim.x) {
      const float v = to_float(row[q_off + i]);
      ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float rq = rsqrtf(ss / (float)Rq + eps);
    for (int i = threadIdx.x; i < Rq; i += blockDim.x)
      cq[(int64_t)t * Rq + i] = from_float<T>(to_float(row[q_off + i]) * rq * load_as_float(wq, w_dtype, i));
  }
  if (pages == nullptr) return;
  const int pos = positions[t];
  const int page = block_table[(int64_t)s * table_width + pos / page_size];
  if (page < 0 || page >= num_pages) {
    if (threadIdx.x == 0) atomicExch(status, 1);
    return;
  }
  T* dst = pages + ((int64_t)page * page_size + pos % page_size) * (R + rd);
  float sk = 0.f;
  for (int i = threadIdx.x; i < R; i += blockDim.x) {
    const float v = to_float(row[kv_off + i]);
    sk = fmaf(v, v, sk);
  }
  sk = block_sum(sk, scratch);
  const float rk = rsqrtf(sk / (float)R + eps);
  for (int i = threadIdx.x; i < R; i += blockDim.x)
    dst[i] = from_float<T>(to_float(row[kv_off + i]) * rk * load_as_float(wkv, w_dtype, i));
  const int half = dims / 2;
  for (int i = threadIdx.x; i < rd; i += blockDim.x) {
    if (i < half) {
      float a, b;
      rotate_pair(to_float(row[kv_off + R + i]), to_float(row[kv_off + R + i + half]), (float)pos * freq[i], mag, a, b);
      dst[R + i] = from_float<T>(a);
      dst[R + i + half] = from_float<T>(b);
    } else if (i >= dims) {
      dst[R + i] = row[kv_off + R + i];
    }
  }
}

// For every token t and vector n < n_vec: src = in[t * in_ld + n * in_stride + in_off ...] (len numbers),
// dst = out[t * out_ld + n * out_stride + out_off ...]; the first dims numbers rotated, the rest copied.
template <typename TI, typename TO>
__global__ void rotate_pairs_kernel(TO* __restrict__ out, int64_t out_ld, int out_stride, int out_off,
                                    const TI* __restrict__ in, int64_t in_ld, int in_stride, int in_off, int n_vec,
                                    int len, int dims, const float* __restrict__ freq, float mag,
                                    const int* __restrict__ positions, const int* __restrict__ seq_of_token) {
  atom::pdl_trigger();
  atom::pdl_wait();
  const int t = blockIdx.x;
  if (seq_of_token[t] < 0) return;
  const float pos = (float)positions[t];
  const int half = dims / 2;
  for (int idx = threadIdx.x; idx < n_vec * len; idx += blockDim.x) {
    const int n = idx / len, i = idx - n * len;
    const TI* src = in + (int64_t)t * in_ld + (int64_t)n * in_stride + in_off;
    TO* dst = out + (int64_t)t * out_ld + (int64_t)n * out_stride + out_off;
    if (i < half) {
      float a, b;
      rotate_pair(to_float(src[i]), to_float(src[i + half]), pos * freq[i], mag, a, b);
      dst[i] = from_float<TO>(a);
      dst[i + half] = from_float<TO>(b);
    } else if (i >= dims) {
      dst[i] = from_float<TO>(to_float(src[i]));
    }
  }
}

constexpr int kLatKT = 32;        // keys per tile (one per lane in the softmax)
constexpr int kLatThreads = 256;
constexpr int kLatAcc = 16;       // outputs per thread: heads of a group * R <= kLatAcc * kLatThreads

// q: [T, H, Dk] float (Dk = R + rd: folded query, then the rotated query part); pages: [pages, page, Dk];
// out: [T, H, R] of the cache's type, or with nsplit > 1 partial sums in scratch
// [T, H, nsplit, R + 2] float (unnormalised sum, running maximum, sum of weights).
template <typename T>
__global__ void __launch_bounds__(kLatThreads)
latent_attention_kernel(T* __restrict__ out, float* __restrict__ scratch, const float* __restrict__ q,
                        const T* __restrict__ pages, const int* __restrict__ block_table, int table_width,
                        int page_size, const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                        int H, int HG, int R, int rd, float scale, int window, const float* __restrict__ sink,
                        int nsplit) {
  atom::pdl_trigger();
  atom::pdl_wait();
  extern __shared__ float smem[];
  const int Dk = R + rd, Dp = Dk + 1;
  float* qs = smem;                        // [HG][Dk]
  float* ks = qs + HG * Dk;                // [KT][Dp]
  float* ps = ks + kLatKT * Dp;            // [HG][KT]
  float* ms = ps + HG * kLatKT;            // [HG] running maximum
  float* ls = ms + HG;                     // [HG] running sum
  float* cs = ls + HG;                     // [HG] correction of this tile
  __shared__ int64_t rowoff[kLatKT];
  const int t = blockIdx.x;
  const int s = seq_of_token[t];
  if (s < 0) return;
  const int h0 = blockIdx.y * HG;
  const int hg = min(HG, H - h0);
  const int pos = positions[t];
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int n = pos - lo + 1;
  int per = (n + nsplit - 1) / nsplit;
  per = (per + kLatKT - 1) / kLatKT * kLatKT;
  const int k_begin = lo + blockIdx.z * per;
  const int k_end = min(pos + 1, k_begin + per);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  for (int i = tid; i < hg * Dk; i += kLatThreads) qs[i] = q[((int64_t)t * H + h0) * Dk + i];
  for (int i = tid; i < hg; i += kLatThreads) {
    ms[i] = -INFINITY;
    ls[i] = 0.f;
  }
  float acc[kLatAcc];
#pragma unroll
  for (int a = 0; a < kLatAcc; ++a) acc[a] = 0.f;
  const int n_out = hg * R;

  for (int k0 = k_begin; k0 < k_end; k0 += kLatKT) {
    const int kt = min(kLatKT, k_end - k0);
    __syncthreads();      // the tile before is used up (and q, m, l are in place)
    if (tid < kt) {
      const int j = k0 + tid;
      const int page = block_table[(int64_t)s * table_width + j / page_size];
      rowoff[tid] = ((int64_t)page * page_size + j % page_size) * Dk;
    }
    __syncthreads();
    for (int i = tid; i < kt * Dk; i += kLatThreads) {
      const int j = i / Dk, d = i - j * Dk;
      ks[j * Dp + d] = to_float(pages[rowoff[j] + d]);
    }
    __syncthreads();
    for (int pr = tid; pr < hg * kLatKT; pr += kLatThreads) {
      const int h = pr / kLatKT, j = pr - h * kLatKT;
      float sc = -INFINITY;
      if (j < kt) {
        const float* qv = qs + h * Dk;
        const float* kv = ks + j * Dp;
        float d0 = 0.f;
        for (int d = 0; d < Dk; ++d) d0 = fmaf(qv[d], kv[d], d0);
        sc = d0 * scale;
      }
      ps[pr] = sc;
    }
    __syncthreads();
    for (int h = warp; h < hg; h += kLatThreads / 32) {
      const float sc = ps[h * kLatKT + lane];
      const float m_old = ms[h];
      const float m_new = fmaxf(m_old, warp_max(sc));
      const float p = (sc == -INFINITY) ? 0.f : expf(sc - m_new);
      const float sum = warp_sum(p);
      ps[h * kLatKT + lane] = p;
      if (lane == 0) {
        const float corr = (m_old == -INFINITY) ? 0.f : expf(m_old - m_new);
        cs[h] = corr;
        ms[h] = m_new;
        ls[h] = ls[h] * corr + sum;
      }
    }
    __syncthreads();
#pragma unroll
    for (int a = 0; a < kLatAcc; ++a) {
      const int idx = tid + a * kLatThreads;
      if (idx < n_out) {
        const int h = idx / R, d = idx - h * R;
        float v = acc[a] * cs[h];
        const float* pv = ps + h * kLatKT;
        for (int j = 0; j < kt; ++j) v = fmaf(pv[j], ks[j * Dp + d], v);
        acc[a] = v;
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int a = 0; a < kLatAcc; ++a) {
    const int idx = tid + a * kLatThreads;
    if (idx < n_out) {
      const int h = idx / R, d = idx - h * R;
      if (nsplit == 1) {
        const float m = ms[h], sk = sink ? sink[h0 + h] : -INFINITY;
        const float top = fmaxf(m, sk);
        const float w = expf(m - top);
        const float den = ls[h] * w + (sink ? expf(sk - top) : 0.f);
        out[((int64_t)t * H + h0 + h) * R + d] = from_float<T>(acc[a] * w / den);
      } else {
        float* dst = scratch + (((int64_t)t * H + h0 + h) * nsplit + blockIdx.z) * (R + 2);
        dst[d] = acc[a];
        if (d == 0) {
          dst[R] = ms[h];
          dst[R + 1] = ls[h];
        }
      }
    }
  }
}

constexpr int kLatMergeShares = 64;   // shares whose weights the merge kernel keeps in shared memory

template <typename T>
__global__ void latent_merge_kernel(T* __restrict__ out, const float* __restrict__ scratch,
                                    const int* __restrict__ seq_of_token, int H, int R, int nsplit,
                                    const float* __restrict__ sink) {
  atom::pdl_trigger();
  atom::pdl_wait();
  __shared__ float ws[kLatMergeShares];
  const int t = blockIdx.x, h = blockIdx.y;
  if (seq_of_token[t] < 0) return;
  const float* src = scratch + ((int64_t)t * H + h) * nsplit * (R + 2);
  if (nsplit <= kLatMergeShares) {
    // warp 0: every share's weight exp(m_z - top) / denominator, once; then each thread sums its columns
    if (threadIdx.x < 32) {
      const int lane = threadIdx.x;
      float m[kLatMergeShares / 32], l[kLatMergeShares / 32];
      float top = sink ? sink[h] : -INFINITY;
#pragma unroll
      for (int i = 0; i < kLatMergeShares / 32; ++i) {
        const int z = lane + 32 * i;
        m[i] = z < nsplit ? src[z * (R + 2) + R] : -INFINITY;
        l[i] = z < nsplit ? src[z * (R + 2) + R + 1] : 0.f;
        top = fmaxf(top, m[i]);
      }
      top = warp_max(top);
      float den = 0.f;
#pragma unroll
      for (int i = 0; i < kLatMergeShares / 32; ++i) {
        m[i] = (m[i] == -INFINITY) ? 0.f : expf(m[i] - top);
        den = fmaf(l[i], m[i], den);
      }
      den = warp_sum(den) + (sink ? expf(sink[h] - top) : 0.f);
#pragma unroll
      for (int i = 0; i < kLatMergeShares / 32; ++i)
        if (lane + 32 * i < nsplit) ws[lane + 32 * i] = m[i] / den;
    }
    __syncthreads();
    for (int d = threadIdx.x; d < R; d += blockDim.x) {
      float v = 0.f;
#pragma unroll 8
      for (int z = 0; z < nsplit; ++z) v = fmaf(src[z * (R + 2) + d], ws[z], v);
      out[((int64_t)t * H + h) * R + d] = from_float<T>(v);
    }
    return;
  }
  float top = sink ? sink[h] : -INFINITY;
  for (int z = 0; z < nsplit; ++z) top = fmaxf(top, src[z * (R + 2) + R]);
  float den = sink ? expf(sink[h] - top) : 0.f;
  for (int z = 0; z < nsplit; ++z) {
    const float m = src[z * (R + 2) + R];
    if (m != -INFINITY) den += src[z * (R + 2) + R + 1] * expf(m - top);
  }
  for (int d = threadIdx.x; d < R; d += blockDim.x) {
    float v = 0.f;
    for (int z = 0; z < nsplit; ++z) {
      const float m = src[z * (R + 2) + R];
      if (m != -INFINITY) v = fmaf(src[z * (R + 2) + d], expf(m - top), v);
    }
    out[((int64_t)t * H + h) * R + d] = from_float<T>(v / den);
  }
}

// Heads a CTA takes together: as many as the accumulators and 64 KB of shared memory for the queries hold.
static inline int latent_head_group(int H, int R, int rd) {
  int hg = (kLatAcc * kLatThreads) / R;
  const int by_smem = (64 * 1024 / 4) / (R + rd);
  if (hg > by_smem) hg = by_smem;
  if (hg > H) hg = H;
  return hg;
}

static inline size_t latent_smem(int HG, int R, int rd) {
  const int Dk = R + rd;
  return sizeof(float) * ((size_t)HG * Dk + (size_t)kLatKT * (Dk + 1) + (size_t)HG * kLatKT + 3 * (size_t)HG);
}

}  // namespace atom

ATOM_EXPORT int atom_latent_prepare(void* cq, const void* proj, int dtype, int64_t ld, int q_off, int Rq,
                                    const void* wq, int kv_off, int R, int rd, int dims, const void* wkv, int w_dtype,
                                    float eps, const float* freq, float mag, const int* positions,
                                    const int* seq_of_token, const int* block_table, int table_width, int page_size,
                                    void* pages, int64_t num_pages, int* status, int T, cudaStream_t stream) {
  if (T <= 0) return ATOM_OK;
  if (Rq < 0 || (Rq > 0 && (!cq || !wq)) || dims < 0 || dims % 2 || (dims > 0 && !freq) || (pages && (R <= 0 || rd < dims || page_size <= 0))) return ATOM_ERR_ARG;
  if (w_dtype != ATOM_F32 && w_dtype != ATOM_BF16) return ATOM_ERR_ARG;
  const int threads = 128;
  if (dtype == ATOM_F32)
    atom::launch_pdl(atom::latent_prepare_kernel<float>, dim3(T), dim3(threads), 0, stream, (float*)cq,
                     (const float*)proj, ld, q_off, Rq, wq, kv_off, R, rd, dims, wkv, w_dtype, eps, freq, mag,
                     positions, seq_of_token, block_table, table_width, page_size, (float*)pages, num_pages, status);
  else if (dtype == ATOM_BF16)
    atom::launch_pdl(atom::latent_prepare_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream,
                     (__nv_bfloat16*)cq, (const __nv_bfloat16*)proj, ld, q_off, Rq, wq, kv_off, R, rd, dims, wkv,
                     w_dtype, eps, freq, mag, positions, seq_of_token, block_table, table_width, page_size,
                     (__nv_bfloat16*)pages, num_pages, status);
  else
    return ATOM_ERR_ARG;
  return atom::check_launch();
}

// in: the activation type; out: float32.
ATOM_EXPORT int atom_rotate_pairs(float* out, int64_t out_ld, int out_stride, int out_off, const void* in,
                                  int in_dtype, int64_t in_ld, int in_stride, int in_off, int n_vec, int len, int dims,
                                  const float* freq, float mag, const int* positions, const int* seq_of_token, int T,
                                  cudaStream_t stream) {
  if (T <= 0 || n_vec <= 0 || len <= 0) return ATOM_OK;
  if (dims < 0 || dims % 2 || dims > len) return ATOM_ERR_ARG;
  const int threads = n_vec * len >= 256 ? 256 : 64;
  if (in_dtype == ATOM_F32)
    atom::launch_pdl(atom::rotate_pairs_kernel<float, float>, dim3(T), dim3(threads), 0, stream, out, out_ld,
                     out_stride, out_off, (const float*)in, in_ld, in_stride, in_off, n_vec, len, dims, freq, mag,
                     positions, seq_of_token);
  else if (in_dtype == ATOM_BF16)
    atom::launch_pdl(atom::rotate_pairs_kernel<__nv_bfloat16, float>, dim3(T), dim3(threads), 0, stream, out, out_ld,
                     out_stride, out_off, (const __nv_bfloat16*)in, in_ld, in_stride, in_off, n_vec, len, dims, freq,
                     mag, positions, seq_of_token);
  else
    return ATOM_ERR_ARG;
  return atom::check_launch();
}

ATOM_EXPORT int atom_latent_attention_head_group(int H, int R, int rd) {
  if (H <= 0 || R <= 0 || rd < 0) return 0;
  return atom::latent_head_group(H, R, rd);
}

ATOM_EXPORT int atom_latent_attention_supports(int H, int R, int rd) {
  if (H <= 0 || R <= 0 || rd < 0) return 0;
  const int hg = atom::latent_head_group(H, R, rd);
  return hg >= 1 && atom::latent_smem(hg, R, rd) <= 200 * 1024;
}

// out[t, h, :] from the shares' partial sums in scratch [T, H, nsplit, R + 2] (either attention kernel leaves them).
ATOM_EXPORT int atom_latent_merge(void* out, const float* scratch, int dtype, const int* seq_of_token, int T, int H,
                                  int R, int nsplit, const float* sink, cudaStream_t stream) {
  if (T <= 0) return ATOM_OK;
  if (H <= 0 || H > 65535 || R <= 0 || nsplit < 1 || !scratch) return ATOM_ERR_ARG;
  const int threads = R >= 256 ? 256 : 64;
  if (dtype == ATOM_F32)
    atom::launch_pdl(atom::latent_merge_kernel<float>, dim3(T, H), dim3(threads), 0, stream, (float*)out, scratch,
                     seq_of_token, H, R, nsplit, sink);
  else if (dtype == ATOM_BF16)
    atom::launch_pdl(atom::latent_merge_kernel<__nv_bfloat16>, dim3(T, H), dim3(threads), 0, stream,
                     (__nv_bfloat16*)out, scratch, seq_of_token, H, R, nsplit, sink);
  else
    return ATOM_ERR_ARG;
  return atom::check_launch();
}

ATOM_EXPORT int atom_latent_attention(void* out, float* scratch, const float* q, const void* pages, int dtype,
                                      const int* block_table, int table_width, int page_size, const int* positions,
                                      const int* seq_of_token, int T, int H, int R, int rd, float scale, int window,
                                      const float* sink, int nsplit, cudaStream_t stream) {
  if (T <= 0) return ATOM_OK;
  if (!atom_latent_attention_supports(H, R, rd) || nsplit < 1 || nsplit > 65535 || (nsplit > 1 && !scratch) ||
      page_size <= 0 || window < 0)
    return ATOM_ERR_ARG;
  const int hg = atom::latent_head_group(H, R, rd);
  const size_t smem = atom::latent_smem(hg, R, rd);
  const dim3 grid(T, (H + hg - 1) / hg, nsplit);
  if (grid.y > 65535) return ATOM_ERR_ARG;
  if (dtype == ATOM_F32) {
    auto k = atom::latent_attention_kernel<float>;
    if (smem > 48 * 1024 && cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return ATOM_ERR_LAUNCH;
    atom::launch_pdl(k, grid, dim3(atom::kLatThreads), smem, stream, (float*)out, scratch, q, (const float*)pages,
                     block_table, table_width, page_size, positions, seq_of_token, H, hg, R, rd, scale, window, sink,
                     nsplit);
  } else if (dtype == ATOM_BF16) {
    auto k = atom::latent_attention_kernel<__nv_bfloat16>;
    if (smem > 48 * 1024 && cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return ATOM_ERR_LAUNCH;
    atom::launch_pdl(k, grid, dim3(atom::kLatThreads), smem, stream, (__nv_bfloat16*)out, scratch, q,
                     (const __nv_bfloat16*)pages, block_table, table_width, page_size, positions, seq_of_token, H, hg,
                     R, rd, scale, window, sink, nsplit);
  } else {
    return ATOM_ERR_ARG;
  }
  if (atom::check_launch() != ATOM_OK) return ATOM_ERR_LAUNCH;
  if (nsplit > 1) return atom_latent_merge(out, scratch, dtype, seq_of_token, T, H, R, nsplit, sink, stream);
  return ATOM_OK;
}
