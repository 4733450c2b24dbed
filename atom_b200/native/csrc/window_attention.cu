// Grouped-query attention behind a short causal convolution, with capped scores and a sliding window that
// always keeps a request's first tokens.  Key size and value size may differ.
//
//   conv_rope_write_kernel    per token: the convolution over time on every channel of [q | k | v]
//                               y_t[c] = sum_j w[c, j] * u_(t - taps + 1 + j)[c]        (zeros before the request's start)
//                             with rows before the step's first token of a request taken from the request's
//                             convolution state (its last taps - 1 projected rows); rotation of the first rot_dims
//                             numbers of every query and key head by position * frequency (pairs (i, i + rot_dims/2));
//                             q to a dense array, k and v to their pages
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
  else if (dtype == ATOM_BF16)
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
