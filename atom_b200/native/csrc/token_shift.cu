// Token shift: every token is blended with the token before it in its own request,
//   out[m][t] = h[t] + (h[t-1] - h[t]) * mu[m]        for each of n_mix blend vectors mu[m],
// in 32-bit, rounded to the activation type.  For a request's first token of this step h[t-1] is what
// the step before left in the request's state row (zeros at the very first token), and the row then
// takes the h of the request's last token of this step.  One block per token; the block of a request's
// first token is the only one that touches the state row, each of its threads reading and then writing
// the columns it owns, so no other block has to wait for it.
#include "common.cuh"

namespace atom {

constexpr int kMaxMix = 8;

template <typename T>
__global__ void token_shift_mix_kernel(T* __restrict__ out, const T* __restrict__ h, const void* __restrict__ mu,
                                       int mu_dtype, T* __restrict__ state, const int* __restrict__ seq_of_token,
                                       const int* __restrict__ cu_q, const int* __restrict__ state_slots, int Tn,
                                       int W, int n_mix, int write_state) {
  atom::pdl_trigger();
  atom::pdl_wait();
  const int t = blockIdx.x;
  const int s = seq_of_token[t];
  if (s < 0) return;      // a padding row of a fixed-size batch
  const int first = cu_q[s], last = cu_q[s + 1] - 1;
  const bool head = (t == first);
  T* srow = state + (int64_t)state_slots[s] * W;
  const T* cur_row = h + (int64_t)t * W;
  const T* prev_row = head ? srow : h + (int64_t)(t - 1) * W;
  const T* last_row = h + (int64_t)last * W;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float cur = to_float(cur_row[i]);
    const float prev = to_float(prev_row[i]);
    if (head && write_state) srow[i] = last_row[i];
    const float d = prev - cur;
    for (int m = 0; m < n_mix; ++m) {
      const float w = load_as_float(mu, mu_dtype, (int64_t)m * W + i);
      out[((int64_t)m * Tn + t) * W + i] = from_float<T>(fmaf(d, w, cur));
    }
  }
}

// bfloat16 rows of a multiple of 8 numbers: a thread owns 8 columns in a row, every array moves 16 bytes at a time.
__global__ void token_shift_mix_bf16_vec_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ h,
                                                const void* __restrict__ mu, int mu_dtype, __nv_bfloat16* __restrict__ state,
                                                const int* __restrict__ seq_of_token, const int* __restrict__ cu_q,
                                                const int* __restrict__ state_slots, int Tn, int W, int n_mix,
                                                int write_state) {
  atom::pdl_trigger();
  atom::pdl_wait();
  const int t = blockIdx.x;
  const int s = seq_of_token[t];
  if (s < 0) return;
  const int first = cu_q[s], last = cu_q[s + 1] - 1;
  const bool head = (t == first);
  __nv_bfloat16* srow = state + (int64_t)state_slots[s] * W;
  const __nv_bfloat16* cur_row = h + (int64_t)t * W;
  const __nv_bfloat16* prev_row = head ? srow : h + (int64_t)(t - 1) * W;
  const __nv_bfloat16* last_row = h + (int64_t)last * W;
  for (int i = threadIdx.x * 8; i < W; i += blockDim.x * 8) {
    const uint4 cq = *reinterpret_cast<const uint4*>(cur_row + i);
    const uint4 pq = *reinterpret_cast<const uint4*>(prev_row + i);
    if (head && write_state) *reinterpret_cast<uint4*>(srow + i) = *reinterpret_cast<const uint4*>(last_row + i);
    const __nv_bfloat162* c2 = reinterpret_cast<const __nv_bfloat162*>(&cq);
    const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&pq);
    float cur[8], d[8];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 a = __bfloat1622float2(c2[e]), b = __bfloat1622float2(p2[e]);
      cur[2 * e] = a.x;
      cur[2 * e + 1] = a.y;
      d[2 * e] = b.x - a.x;
      d[2 * e + 1] = b.y - a.y;
    }
    for (int m = 0; m < n_mix; ++m) {
      uint4 oq;
      __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&oq);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float w0 = load_as_float(mu, mu_dtype, (int64_t)m * W + i + 2 * e);
        const float w1 = load_as_float(mu, mu_dtype, (int64_t)m * W + i + 2 * e + 1);
        o2[e] = __floats2bfloat162_rn(fmaf(d[2 * e], w0, cur[2 * e]), fmaf(d[2 * e + 1], w1, cur[2 * e + 1]));
      }
      *reinterpret_cast<uint4*>(out + ((int64_t)m * Tn + t) * W + i) = oq;
    }
  }
}

}  // namespace atom

// out: [n_mix, T, W]; h: [T, W]; mu: [n_mix, W]; state: [slots, W] of the activation type.
ATOM_EXPORT int atom_token_shift_mix(void* out, const void* h, int dtype, const void* mu, int mu_dtype, void* state,
                                     const int* seq_of_token, const int* cu_q, const int* state_slots, int T, int W,
                                     int n_mix, int write_state, cudaStream_t stream) {
  if (T <= 0) return ATOM_OK;
  if (W <= 0 || n_mix <= 0 || n_mix > atom::kMaxMix) return ATOM_ERR_ARG;
  const int threads = W >= 1024 ? 256 : 128;
  if (dtype == ATOM_F32) {
    atom::launch_pdl(atom::token_shift_mix_kernel<float>, dim3(T), dim3(threads), 0, stream, (float*)out,
                     (const float*)h, mu, mu_dtype, (float*)state, seq_of_token, cu_q, state_slots, T, W, n_mix,
                     write_state);
  } else if (dtype == ATOM_BF16 && W % 8 == 0 && ((uintptr_t)out % 16) == 0 && ((uintptr_t)h % 16) == 0 &&
             ((uintptr_t)state % 16) == 0) {
    const int vt = W / 8 >= 256 ? 256 : (W / 8 >= 128 ? 128 : (W / 8 >= 64 ? 64 : 32));
    atom::launch_pdl(atom::token_shift_mix_bf16_vec_kernel, dim3(T), dim3(vt), 0, stream, (__nv_bfloat16*)out,
                     (const __nv_bfloat16*)h, mu, mu_dtype, (__nv_bfloat16*)state, seq_of_token, cu_q, state_slots, T, W,
                     n_mix, write_state);
  } else if (dtype == ATOM_BF16) {
    atom::launch_pdl(atom::token_shift_mix_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream,
                     (__nv_bfloat16*)out, (const __nv_bfloat16*)h, mu, mu_dtype, (__nv_bfloat16*)state, seq_of_token,
                     cu_q, state_slots, T, W, n_mix, write_state);
  } else {
    return ATOM_ERR_ARG;
  }
  return atom::check_launch();
}
