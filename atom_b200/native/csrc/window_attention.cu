// Grouped-query attention behind a short causal convolution, with capped scores and a sliding window that
// always keeps a request's first tokens.  Key size and value size may differ.
//
//   conv_rope_write_kernel    per token: the convolution over time on every channel of [q | k | v]
//                               y_t[c] = sum_j w[c, j] * u_(t - taps + 1 + j)[c]        (zeros before the request's start)
//                             with rows before the step's first token of a request taken from the request's
//                             convolution state (its last taps - 1 projected rows); rotation of the first rot_dims
//                             numbers of every query and key head by position * frequency (pairs (i, i + rot_dims/2));
//                             q to a dense array, k and v to their pages (conv_rope_write_vec_kernel: the same
//                             for bfloat16 sizes in steps of 8, 16 bytes at a time)
//   conv_state_update_kernel  per request: the last taps - 1 projected rows after this step
//   window_attention_kernel   one CTA per (token, query head): keys j <= p with p - j < window or j < keep_first,
//                             s = scale * q.k, s <- cap * tanh(s / cap), online softmax in 32-bit; any sizes, both
//                             precisions
// Convolution sums, angles, scores, weights and sums are 32-bit in both precisions.
#include "common.cuh"

namespace atom {

// Row t' (an index into the step's rows, possibly before the request's first row of this step) of channel c.
template <typename T>
__device__ __forceinline__ float conv_input(const T* __restrict__ qkv, int64_t ld, const T* __restrict__ state_row,
                                            int C, int taps, int first, int tp, int c) {
  if (tp >= first) return to_float(qkv[(int64_t)tp * ld + c]);
  const int d = first - tp;                       // 1 .. taps - 1 rows before the step
  return state_row ? to_float(state_row[(int64_t)(taps - 1 - d) * C + c]) : 0.f;
}

template <typename T>
__device__ __forceinline__ float conv_at(const T* __restrict__ qkv, int64_t ld, const T* __restrict__ state_row, int C,
                                         int taps, const void* __restrict__ w, int w_dtype, int first, int t, int c) {
  if (taps <= 0) return to_float(qkv[(int64_t)t * ld + c]);
  float y = 0.f;
  for (int j = 0; j < taps; ++j)
    y += load_as_float(w, w_dtype, (int64_t)c * taps + j) * conv_input(qkv, ld, state_row, C, taps, first, t - taps + 1 + j, c);
  return y;
}

template <typename T>
__global__ void __launch_bounds__(256)
conv_rope_write_kernel(T* __restrict__ q_out, const T* __restrict__ qkv, int64_t ld, int H, int G, int dk, int dv,
                       const void* __restrict__ conv_w, int w_dtype, int taps, const T* __restrict__ conv_state,
                       const float* __restrict__ freq, int rot_dims, const int* __restrict__ positions,
                       const int* __restrict__ seq_of_token, const int* __restrict__ cu_q,
                       const int* __restrict__ state_slots, const int* __restrict__ block_table, int max_pages,
                       int page_size, T* __restrict__ k_pages, T* __restrict__ v_pages, int64_t num_pages,
                       int* __restrict__ status) {
  atom::pdl_trigger();
  atom::pdl_wait();
  const int t = blockIdx.x;
  const int s = seq_of_token[t];
  if (s < 0) return;
  const int p = positions[t];
  const int first = cu_q[s];
  const int C = H * dk + G * dk + G * dv;
  const T* state_row = (conv_state && taps > 1) ? conv_state + (int64_t)state_slots[s] * (taps - 1) * C : nullptr;
  const int lp = p / page_size;
  const int page = lp < max_pages ? block_table[(int64_t)s * max_pages + lp] : -1;
  const bool writes = k_pages != nullptr;
  if (writes && (page < 0 || page >= num_pages)) {
    if (threadIdx.x == 0) atomicExch(status, 1);
    return;
  }
  const int slot = p % page_size;
  const int half = rot_dims / 2;
  const float pos = (float)p;
  // queries and keys: H + G vectors of dk numbers
  for (int idx = threadIdx.x; idx < (H + G) * dk; idx += blockDim.x) {
    const int n = idx / dk, i = idx - n * dk;
    if (i >= half && i < rot_dims) continue;      // the second of a pair: written by the first
    const int c = n * dk + i;                      // (keys follow the queries in the row)
    T* dst;
    if (n < H) {
      dst = q_out + ((int64_t)t * H + n) * dk;
    } else {
      if (!writes) continue;
      dst = k_pages + (((int64_t)page * G + (n - H)) * page_size + slot) * dk;
    }
    const float a = conv_at(qkv, ld, state_row, C, taps, conv_w, w_dtype, first, t, c);
    if (i < half) {
      const float b = conv_at(qkv, ld, state_row, C, taps, conv_w, w_dtype, first, t, c + half);
      float sn, cs;
      sincosf(pos * freq[i], &sn, &cs);
      dst[i] = from_float<T>(a * cs - b * sn);
      dst[i + half] = from_float<T>(b * cs + a * sn);
    } else {
      dst[i] = from_float<T>(a);
    }
  }
  if (!writes) return;
  const int v0 = (H + G) * dk;
  for (int idx = threadIdx.x; idx < G * dv; idx += blockDim.x) {
    const int g = idx / dv, i = idx - g * dv;
    v_pages[(((int64_t)page * G + g) * page_size + slot) * dv + i] =
        from_float<T>(conv_at(qkv, ld, state_row, C, taps, conv_w, w_dtype, first, t, v0 + idx));
  }
}

// The same in bfloat16 for sizes in steps of 8 (key and value sizes, and half of rot_dims): a thread owns 8 channels
// in a row, so every row of inputs, the channels' taps and the outputs move 16 bytes at a time; the token's
// convolved channels pass through shared memory in 32-bit, where a rotated pair finds its other half.  The sums run
// over the taps in the same order as in the kernel above.
template <int TAPS>
__global__ void __launch_bounds__(256)
conv_rope_write_vec_kernel(__nv_bfloat16* __restrict__ q_out, const __nv_bfloat16* __restrict__ qkv, int64_t ld, int H,
                           int G, int dk, int dv, const __nv_bfloat16* __restrict__ conv_w,
                           const __nv_bfloat16* __restrict__ conv_state, const float* __restrict__ freq, int rot_dims,
                           const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                           const int* __restrict__ cu_q, const int* __restrict__ state_slots,
                           const int* __restrict__ block_table, int max_pages, int page_size,
                           __nv_bfloat16* __restrict__ k_pages, __nv_bfloat16* __restrict__ v_pages, int64_t num_pages,
                           int* __restrict__ status) {
  atom::pdl_trigger();
  atom::pdl_wait();
  extern __shared__ __align__(16) float cv_y[];      // [C]
  const int t = blockIdx.x;
  const int s = seq_of_token[t];
  if (s < 0) return;
  const int p = positions[t];
  const int first = cu_q[s];
  const int C = H * dk + G * dk + G * dv;
  const __nv_bfloat16* state_row =
      (conv_state && TAPS > 1) ? conv_state + (int64_t)state_slots[s] * (TAPS - 1) * C : nullptr;
  const int lp = p / page_size;
  const int page = lp < max_pages ? block_table[(int64_t)s * max_pages + lp] : -1;
  const bool writes = k_pages != nullptr;
  if (writes && (page < 0 || page >= num_pages)) {
    if (threadIdx.x == 0) atomicExch(status, 1);
    return;
  }
  const int slot = p % page_size;
  const int groups = C / 8;
  for (int g = threadIdx.x; g < groups; g += blockDim.x) {
    const int c = g * 8;
    float y[8];
    if (TAPS == 0) {
      const uint4 raw = *reinterpret_cast<const uint4*>(qkv + (int64_t)t * ld + c);
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h2[e]);
        y[2 * e] = f.x;
        y[2 * e + 1] = f.y;
      }
    } else {
      constexpr int NW = TAPS > 0 ? TAPS : 1;
      uint4 wraw[NW];                                  // the 8 channels' taps: 8 * TAPS numbers in a row
#pragma unroll
      for (int j = 0; j < NW; ++j) wraw[j] = *reinterpret_cast<const uint4*>(conv_w + (int64_t)c * TAPS + j * 8);
      const __nv_bfloat16* wv = reinterpret_cast<const __nv_bfloat16*>(wraw);
#pragma unroll
      for (int e = 0; e < 8; ++e) y[e] = 0.f;
#pragma unroll
      for (int j = 0; j < NW; ++j) {
        const int tp = t - TAPS + 1 + j;
        uint4 raw = make_uint4(0u, 0u, 0u, 0u);
        if (tp >= first)
          raw = *reinterpret_cast<const uint4*>(qkv + (int64_t)tp * ld + c);
        else if (state_row)
          raw = *reinterpret_cast<const uint4*>(state_row + (int64_t)(TAPS - 1 - (first - tp)) * C + c);
        const __nv_bfloat16* xv = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
        for (int e = 0; e < 8; ++e) y[e] += __bfloat162float(wv[e * TAPS + j]) * __bfloat162float(xv[e]);
      }
    }
    *reinterpret_cast<float4*>(cv_y + c) = make_float4(y[0], y[1], y[2], y[3]);
    *reinterpret_cast<float4*>(cv_y + c + 4) = make_float4(y[4], y[5], y[6], y[7]);
  }
  __syncthreads();
  const int half = rot_dims / 2;
  const float pos = (float)p;
  const int qk_end = (H + G) * dk;
  for (int g = threadIdx.x; g < groups; g += blockDim.x) {
    const int c = g * 8;
    __nv_bfloat16* dst;
    int i0 = 0;
    bool rotated = false;
    if (c < qk_end) {
      const int n = c / dk;
      i0 = c - n * dk;
      rotated = i0 < rot_dims;
      if (n < H) {
        dst = q_out + ((int64_t)t * H + n) * dk + i0;
      } else {
        if (!writes) continue;
        dst = k_pages + (((int64_t)page * G + (n - H)) * page_size + slot) * dk + i0;
      }
    } else {
      if (!writes) continue;
      const int idx = c - qk_end;
      const int gg = idx / dv;
      dst = v_pages + (((int64_t)page * G + gg) * page_size + slot) * dv + (idx - gg * dv);
    }
    float o[8];
    if (rotated) {
      const bool low = i0 < half;                      // the first of the pair: (a, b) = (own, + half); else (- half, own)
      const float* av = cv_y + (low ? c : c - half);
      const float* bv = cv_y + (low ? c + half : c);
      const float* fr = freq + (low ? i0 : i0 - half);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        float sn, cs;
        sincosf(pos * fr[e], &sn, &cs);
        const float a = av[e], b = bv[e];
        o[e] = low ? a * cs - b * sn : b * cs + a * sn;
      }
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = cv_y[c + e];
    }
    uint4 packed;
    __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
    for (int e = 0; e < 4; ++e) h2[e] = __floats2bfloat162_rn(o[2 * e], o[2 * e + 1]);
    *reinterpret_cast<uint4*>(dst) = packed;
  }
}

// state [slots, taps - 1, C]: row taps - 2 is the request's latest projected row.  A thread owns a channel and walks
// the rows upwards, so a row it still has to read (further up) has not been written.
template <typename T>
__global__ void conv_state_update_kernel(T* __restrict__ conv_state, const T* __restrict__ qkv, int64_t ld, int C,
                                         int taps, const int* __restrict__ cu_q, const int* __restrict__ state_slots) {
  atom::pdl_trigger();
  atom::pdl_wait();
  const int s = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int first = cu_q[s], len = cu_q[s + 1] - first;
  if (len <= 0) return;
  T* st = conv_state + (int64_t)state_slots[s] * (taps - 1) * C;
  for (int r = 0; r < taps - 1; ++r) {
    const int src = r + len - (taps - 1);          // row of the step (>= 0) or of the old state (< 0)
    st[(int64_t)r * C + c] = src >= 0 ? qkv[(int64_t)(first + src) * ld + c] : st[(int64_t)(r + len) * C + c];
  }
}

constexpr int kWinThreads = 128;
constexpr int kWinChunk = 256;

template <typename T>
__global__ void __launch_bounds__(kWinThreads)
window_attention_kernel(T* __restrict__ out, const T* __restrict__ q, const T* __restrict__ k_pages,
                        const T* __restrict__ v_pages, const int* __restrict__ block_table, int max_pages,
                        int page_size, const int* __restrict__ positions, const int* __restrict__ seq_of_token, int nh,
                        int nkv, int dk, int dv, float scale, float softcap, int window, int keep_first) {
  atom::pdl_trigger();
  atom::pdl_wait();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  int64_t* row_of = (int64_t*)smem_raw;            // [kWinChunk] (page * nkv + g) * page_size + slot of a key
  float* prob = (float*)(row_of + kWinChunk);      // [kWinChunk]
  float* qs = prob + kWinChunk;                    // [dk]
  __shared__ float scratch[32];

  const int t = blockIdx.x, h = blockIdx.y;
  if (seq_of_token[t] < 0) return;
  const int g = h / (nh / nkv);
  const int p = positions[t];
  const int* bt = block_table + (int64_t)seq_of_token[t] * max_pages;
  const T* qrow = q + ((int64_t)t * nh + h) * dk;
  for (int i = threadIdx.x; i < dk; i += blockDim.x) qs[i] = to_float(qrow[i]);

  int lo = 0;
  if (window > 0 && p - window + 1 > 0) lo = p - window + 1;
  const int n_first = min(keep_first, lo);         // kept first tokens that the window itself does not reach
  const int n_keys = n_first + (p - lo + 1);
  const float inv_cap = softcap > 0.f ? 1.f / softcap : 0.f;

  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  float m = -INFINITY, l = 0.f;
  __syncthreads();
  for (int c0 = 0; c0 < n_keys; c0 += kWinChunk) {
    const int n = min(kWinChunk, n_keys - c0);
    float cmax = -INFINITY;
    for (int jj = threadIdx.x; jj < n; jj += blockDim.x) {
      const int e = c0 + jj;
      const int j = e < n_first ? e : lo + (e - n_first);
      const int page = bt[j / page_size];
      const int64_t row = ((int64_t)page * nkv + g) * page_size + (j % page_size);
      row_of[jj] = row;
      const T* kr = k_pages + row * dk;
      float sc = 0.f;
      for (int i = 0; i < dk; ++i) sc += qs[i] * to_float(kr[i]);
      sc *= scale;
      if (softcap > 0.f) sc = softcap * tanhf(sc * inv_cap);
      prob[jj] = sc;
      cmax = fmaxf(cmax, sc);
    }
    cmax = block_max(cmax, scratch);
    const float m_new = fmaxf(m, cmax);
    const float corr = expf(m - m_new);
    float lsum = 0.f;
    for (int jj = threadIdx.x; jj < n; jj += blockDim.x) {
      const float e = expf(prob[jj] - m_new);
      prob[jj] = e;
      lsum += e;
    }
    lsum = block_sum(lsum, scratch);
    l = l * corr + lsum;
    m = m_new;
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      const int d = threadIdx.x + a * kWinThreads;
      if (d < dv) {
        float sum = acc[a] * corr;
        for (int jj = 0; jj < n; ++jj) sum += prob[jj] * to_float(v_pages[row_of[jj] * dv + d]);
        acc[a] = sum;
      }
    }
    __syncthreads();
  }
  T* orow = out + ((int64_t)t * nh + h) * dv;
  const float inv = 1.f / l;
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    const int d = threadIdx.x + a * kWinThreads;
    if (d < dv) orow[d] = from_float<T>(acc[a] * inv);
  }
}

// Puts together the shares that window_attention_tc.cu left in `part`: per token and share [m (nh) | l (nh) | o (nh dv)],
// a share's running maximum (natural logarithm), sum and unnormalised output.  One CTA per (token, head).
template <typename T>
__global__ void window_attention_merge_kernel(T* __restrict__ out, const float* __restrict__ part,
                                              const int* __restrict__ seq_of_token, int nh, int dv, int nsplit) {
  atom::pdl_trigger();
  atom::pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  if (seq_of_token[t] < 0) return;
  const int64_t stride = (int64_t)nh * dv + 2 * nh;
  const float* pt = part + (int64_t)t * nsplit * stride;
  float M = -INFINITY;
  for (int s = 0; s < nsplit; ++s) M = fmaxf(M, pt[s * stride + h]);
  for (int i = threadIdx.x; i < dv; i += blockDim.x) {
    float L = 0.f, o = 0.f;
    for (int s = 0; s < nsplit; ++s) {
      const float m = pt[s * stride + h];
      const float w = (m == -INFINITY) ? 0.f : expf(m - M);      // a share without keys weighs nothing
      L = fmaf(pt[s * stride + nh + h], w, L);
      o = fmaf(pt[s * stride + 2 * nh + (int64_t)h * dv + i], w, o);
    }
    out[((int64_t)t * nh + h) * dv + i] = from_float<T>(o / L);
  }
}

}  // namespace atom

// qkv: [T, >= C] rows of [q (H dk) | k (G dk) | v (G dv)], row stride ld; q_out [T, H dk] dense.  conv_w [C, taps]
// (taps 0: no convolution), conv_state [slots, taps - 1, C] (read only here).  k_pages null: nothing is written.
ATOM_EXPORT int atom_conv_rope_write(void* q_out, const void* qkv, int dtype, int64_t ld, int T, int H, int G, int dk,
                                     int dv, const void* conv_w, int w_dtype, int taps, const void* conv_state,
                                     const float* freq, int rot_dims, const int* positions, const int* seq_of_token,
                                     const int* cu_q, const int* state_slots, const int* block_table, int max_pages,
                                     int page_size, void* k_pages, void* v_pages, int64_t num_pages, int* status,
                                     cudaStream_t stream) {
  if (T <= 0) return ATOM_OK;
  if (H <= 0 || G <= 0 || dk <= 0 || dv <= 0 || rot_dims < 0 || rot_dims % 2 || rot_dims > dk || taps < 0 ||
      page_size <= 0 || (rot_dims > 0 && !freq) || (taps > 0 && !conv_w))
    return ATOM_ERR_ARG;
  if (dtype == ATOM_F32)
    atom::launch_pdl(atom::conv_rope_write_kernel<float>, dim3(T), dim3(256), 0, stream, (float*)q_out,
                     (const float*)qkv, ld, H, G, dk, dv, conv_w, w_dtype, taps, (const float*)conv_state, freq,
                     rot_dims, positions, seq_of_token, cu_q, state_slots, block_table, max_pages, page_size,
                     (float*)k_pages, (float*)v_pages, num_pages, status);
  else if (dtype == ATOM_BF16 && dk % 8 == 0 && dv % 8 == 0 && rot_dims % 16 == 0 && ld % 8 == 0 && taps <= 8 &&
           (taps == 0 || w_dtype == ATOM_BF16) && ((H + 2 * G) * dk + G * dv) * sizeof(float) <= 48 * 1024 &&
           ((uintptr_t)qkv % 16) == 0 && ((uintptr_t)conv_w % 16) == 0 && ((uintptr_t)conv_state % 16) == 0 &&
           ((uintptr_t)q_out % 16) == 0 && ((uintptr_t)k_pages % 16) == 0 && ((uintptr_t)v_pages % 16) == 0) {
    const int C = (H + G) * dk + G * dv;
    const int threads = C / 8 >= 256 ? 256 : ((C / 8 + 31) / 32) * 32;
#define ATOM_CV(TAPS)                                                                                               \
  atom::launch_pdl(atom::conv_rope_write_vec_kernel<TAPS>, dim3(T), dim3(threads), C * sizeof(float), stream,       \
                   (__nv_bfloat16*)q_out, (const __nv_bfloat16*)qkv, ld, H, G, dk, dv, (const __nv_bfloat16*)conv_w, \
                   (const __nv_bfloat16*)conv_state, freq, rot_dims, positions, seq_of_token, cu_q, state_slots,    \
                   block_table, max_pages, page_size, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, num_pages,  \
                   status)
    switch (taps) {
      case 0: ATOM_CV(0); break;
      case 1: ATOM_CV(1); break;
      case 2: ATOM_CV(2); break;
      case 3: ATOM_CV(3); break;
      case 4: ATOM_CV(4); break;
      case 5: ATOM_CV(5); break;
      case 6: ATOM_CV(6); break;
      case 7: ATOM_CV(7); break;
      default: ATOM_CV(8); break;
    }
#undef ATOM_CV
  } else if (dtype == ATOM_BF16)
    atom::launch_pdl(atom::conv_rope_write_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, stream,
                     (__nv_bfloat16*)q_out, (const __nv_bfloat16*)qkv, ld, H, G, dk, dv, conv_w, w_dtype, taps,
                     (const __nv_bfloat16*)conv_state, freq, rot_dims, positions, seq_of_token, cu_q, state_slots,
                     block_table, max_pages, page_size, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, num_pages,
                     status);
  else
    return ATOM_ERR_ARG;
  return atom::check_launch();
}

ATOM_EXPORT int atom_conv_state_update(void* conv_state, const void* qkv, int dtype, int64_t ld, int C, int taps,
                                       const int* cu_q, const int* state_slots, int num_seqs, cudaStream_t stream) {
  if (num_seqs <= 0 || taps <= 1) return ATOM_OK;
  if (C <= 0 || num_seqs > 65535) return ATOM_ERR_ARG;
  dim3 grid((C + 127) / 128, num_seqs);
  if (dtype == ATOM_F32)
    atom::launch_pdl(atom::conv_state_update_kernel<float>, grid, dim3(128), 0, stream, (float*)conv_state,
                     (const float*)qkv, ld, C, taps, cu_q, state_slots);
  else if (dtype == ATOM_BF16)
    atom::launch_pdl(atom::conv_state_update_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream,
                     (__nv_bfloat16*)conv_state, (const __nv_bfloat16*)qkv, ld, C, taps, cu_q, state_slots);
  else
    return ATOM_ERR_ARG;
  return atom::check_launch();
}

// out [T, nh dv]; q [T, nh dk] dense.  window <= 0: every earlier key; softcap <= 0: none.
ATOM_EXPORT int atom_window_attention(void* out, const void* q, int dtype, const void* k_pages, const void* v_pages,
                                      const int* block_table, int max_pages, int page_size, const int* positions,
                                      const int* seq_of_token, int T, int nh, int nkv, int dk, int dv, float scale,
                                      float softcap, int window, int keep_first, cudaStream_t stream) {
  if (T <= 0) return ATOM_OK;
  if (nh <= 0 || nkv <= 0 || nh % nkv != 0 || dk <= 0 || dv <= 0 || dv > 4 * atom::kWinThreads || dk > 4096 ||
      page_size <= 0 || nh > 65535 || keep_first < 0)
    return ATOM_ERR_ARG;
  const size_t smem = sizeof(float) * (dk + atom::kWinChunk) + sizeof(int64_t) * atom::kWinChunk;
  dim3 grid(T, nh);
  if (dtype == ATOM_F32)
    atom::launch_pdl(atom::window_attention_kernel<float>, grid, dim3(atom::kWinThreads), smem, stream, (float*)out,
                     (const float*)q, (const float*)k_pages, (const float*)v_pages, block_table, max_pages, page_size,
                     positions, seq_of_token, nh, nkv, dk, dv, scale, softcap, window, keep_first);
  else if (dtype == ATOM_BF16)
    atom::launch_pdl(atom::window_attention_kernel<__nv_bfloat16>, grid, dim3(atom::kWinThreads), smem, stream,
                     (__nv_bfloat16*)out, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pages,
                     (const __nv_bfloat16*)v_pages, block_table, max_pages, page_size, positions, seq_of_token, nh,
                     nkv, dk, dv, scale, softcap, window, keep_first);
  else
    return ATOM_ERR_ARG;
  return atom::check_launch();
}

ATOM_EXPORT int atom_window_attention_merge(void* out, int dtype, const float* part, const int* seq_of_token, int T, int nh,
                                            int dv, int nsplit, cudaStream_t stream) {
  if (T <= 0) return ATOM_OK;
  if (nsplit < 1 || part == nullptr || nh <= 0 || nh > 65535 || dv <= 0) return ATOM_ERR_ARG;
  const int threads = dv >= 128 ? 128 : (dv >= 64 ? 64 : 32);
  if (dtype == ATOM_F32)
    atom::launch_pdl(atom::window_attention_merge_kernel<float>, dim3(T, nh), dim3(threads), 0, stream, (float*)out, part,
                     seq_of_token, nh, dv, nsplit);
  else if (dtype == ATOM_BF16)
    atom::launch_pdl(atom::window_attention_merge_kernel<__nv_bfloat16>, dim3(T, nh), dim3(threads), 0, stream,
                     (__nv_bfloat16*)out, part, seq_of_token, nh, dv, nsplit);
  else
    return ATOM_ERR_ARG;
  return atom::check_launch();
}
