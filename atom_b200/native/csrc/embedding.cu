// Embedding gather: residual[t, :] = table[ids[t], :] * scale, widened to 32-bit (scale 1 for most models).
// The residual stream is kept in 32-bit in both precisions, so the gather writes floats.
#include "common.cuh"

namespace atom {

template <typename T>
__global__ void embedding_kernel(float* __restrict__ out, const T* __restrict__ table,
                                 const int* __restrict__ ids, int H, int V, float scale) {
  atom::pdl_trigger();   // the next kernel may be scheduled at once: before its own wait it reads nothing a kernel of this step writes
  atom::pdl_wait();      // inputs written by the kernel before this one are visible from here on
  const int t = blockIdx.x;
  int id = ids[t];
  // Ids are validated on the host; the clamp only keeps a bad id from reading outside the table.
  id = id < 0 ? 0 : (id >= V ? V - 1 : id);
  const T* row = table + (int64_t)id * H;
  float* o = out + (int64_t)t * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = to_float(row[i]) * scale;
}

// bf16 table, H a multiple of 8: 16 bytes per load, all of a thread's loads asked for before the first is used
// (a row is one cold read from HBM: the kernel's time is round trips, not bytes).
__global__ void embedding_bf16_vec_kernel(float* __restrict__ out, const __nv_bfloat16* __restrict__ table,
                                          const int* __restrict__ ids, int H, int V, float scale) {
  atom::pdl_trigger();
  atom::pdl_wait();
  const int t = blockIdx.x;
  int id = ids[t];
  id = id < 0 ? 0 : (id >= V ? V - 1 : id);
  const uint4* row = reinterpret_cast<const uint4*>(table + (int64_t)id * H);
  float4* o = reinterpret_cast<float4*>(out + (int64_t)t * H);
  const int n = H >> 3;
  for (int i0 = threadIdx.x; i0 < n; i0 += 4 * blockDim.x) {
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = i0 + u * blockDim.x;
      v[u] = i < n ? __ldg(row + i) : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = i0 + u * blockDim.x;
      if (i < n) {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[u]);
        const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
        const float2 c = __bfloat1622float2(h[2]), d = __bfloat1622float2(h[3]);
        o[2 * i] = make_float4(a.x * scale, a.y * scale, b.x * scale, b.y * scale);
        o[2 * i + 1] = make_float4(c.x * scale, c.y * scale, d.x * scale, d.y * scale);
      }
    }
  }
}

}  // namespace atom

ATOM_EXPORT int atom_embedding(float* out, const void* table, int table_dtype, const int* ids, int T,
                               int H, int V, float scale, cudaStream_t stream) {
  if (T <= 0) return ATOM_OK;
  if (H <= 0 || V <= 0) return ATOM_ERR_ARG;
  const int threads = H >= 1024 ? 256 : 128;
  if (table_dtype == ATOM_F32) {
    atom::launch_pdl(atom::embedding_kernel<float>, dim3(T), dim3(threads), 0, stream, out, (const float*)table, ids, H, V, scale);
  } else if (table_dtype == ATOM_BF16 && H % 8 == 0 && ((uintptr_t)table % 16) == 0 && ((uintptr_t)out % 16) == 0) {
    const int vt = H >= 4096 ? 128 : (H >= 1024 ? 64 : 32);      // a thread takes up to four 16-byte pieces at a time
    atom::launch_pdl(atom::embedding_bf16_vec_kernel, dim3(T), dim3(vt), 0, stream, out, (const __nv_bfloat16*)table, ids,
                     H, V, scale);
  } else if (table_dtype == ATOM_BF16) {
    atom::launch_pdl(atom::embedding_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, out, (const __nv_bfloat16*)table, ids, H, V, scale);
  } else {
    return ATOM_ERR_ARG;
  }
  return atom::check_launch();
}

// ------------------------------------------------------------------ embedding with a table of token pairs
// residual[t] = table[id] * scale + pairs[row],  row = (previous id * mul_prev + id * mul_cur) mod buckets, and row
// `buckets` (the table's last) for a request's first token.  The previous id of a request's first token of this step is
// what the step before left in the request's state row; the row then takes the id of the request's last token of this
// step.  The block of a request's first token of the step is the only one that touches the state row.
namespace atom {

template <typename T>
__global__ void pair_embedding_kernel(float* __restrict__ out, const T* __restrict__ table, const T* __restrict__ pairs,
                                      const int* __restrict__ ids, const int* __restrict__ positions,
                                      const int* __restrict__ seq_of_token, const int* __restrict__ cu_q,
                                      const int* __restrict__ state_slots, int* __restrict__ prev_state, int H, int V,
                                      int buckets, unsigned long long mul_prev, unsigned long long mul_cur, float scale,
                                      int write_state) {
  atom::pdl_trigger();
  atom::pdl_wait();
  __shared__ int prev_s;
  const int t = blockIdx.x;
  const int s = seq_of_token[t];
  int id = ids[t];
  id = id < 0 ? 0 : (id >= V ? V - 1 : id);
  float* o = out + (int64_t)t * H;
  const T* row = table + (int64_t)id * H;
  if (s < 0) {      // a padding row of a fixed-size batch: any finite numbers
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = to_float(row[i]) * scale;
    return;
  }
  const int first = cu_q[s], last = cu_q[s + 1] - 1;
  if (threadIdx.x == 0) {
    int prev;
    if (t == first) {
      int* st = prev_state + state_slots[s];
      prev = *st;
      if (write_state) *st = ids[last];
    } else {
      prev = ids[t - 1];
    }
    prev_s = prev < 0 ? 0 : (prev >= V ? V - 1 : prev);
  }
  __syncthreads();
  const unsigned long long pr =
      positions[t] == 0 ? (unsigned long long)buckets
                        : ((unsigned long long)prev_s * mul_prev + (unsigned long long)id * mul_cur) % (unsigned long long)buckets;
  const T* prow = pairs + (int64_t)pr * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = fmaf(to_float(row[i]), scale, to_float(prow[i]));
}

}  // namespace atom

// table [V, H], pairs [buckets + 1, H] of one type; prev_state [slots] int32.
ATOM_EXPORT int atom_pair_embedding(float* out, const void* table, const void* pairs, int table_dtype, const int* ids,
                                    const int* positions, const int* seq_of_token, const int* cu_q,
                                    const int* state_slots, int* prev_state, int T, int H, int V, int buckets,
                                    int64_t mul_prev, int64_t mul_cur, float scale, int write_state, cudaStream_t stream) {
  if (T <= 0) return ATOM_OK;
  if (H <= 0 || V <= 0 || buckets <= 0 || mul_prev < 0 || mul_cur < 0) return ATOM_ERR_ARG;
  const int threads = H >= 1024 ? 256 : 128;
  if (table_dtype == ATOM_F32)
    atom::launch_pdl(atom::pair_embedding_kernel<float>, dim3(T), dim3(threads), 0, stream, out, (const float*)table,
                     (const float*)pairs, ids, positions, seq_of_token, cu_q, state_slots, prev_state, H, V, buckets,
                     (unsigned long long)mul_prev, (unsigned long long)mul_cur, scale, write_state);
  else if (table_dtype == ATOM_BF16)
    atom::launch_pdl(atom::pair_embedding_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, out,
                     (const __nv_bfloat16*)table, (const __nv_bfloat16*)pairs, ids, positions, seq_of_token, cu_q,
                     state_slots, prev_state, H, V, buckets, (unsigned long long)mul_prev, (unsigned long long)mul_cur,
                     scale, write_state);
  else
    return ATOM_ERR_ARG;
  return atom::check_launch();
}

// residual[t, :] += vec[:] (32-bit), for every row of the step.
namespace atom {
__global__ void add_row_kernel(float* __restrict__ residual, const void* __restrict__ vec, int vec_dtype, int H, int64_t n) {
  atom::pdl_trigger();
  atom::pdl_wait();
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (int64_t)gridDim.x * blockDim.x)
    residual[e] += load_as_float(vec, vec_dtype, e % H);
}
}  // namespace atom

ATOM_EXPORT int atom_add_row(float* residual, const void* vec, int vec_dtype, int T, int H, cudaStream_t stream) {
  if (T <= 0) return ATOM_OK;
  if (H <= 0) return ATOM_ERR_ARG;
  const int64_t n = (int64_t)T * H;
  const int blocks = (int)((n + 255) / 256 > 148 * 8 ? 148 * 8 : (n + 255) / 256);
  atom::launch_pdl(atom::add_row_kernel, dim3(blocks), dim3(256), 0, stream, residual, vec, vec_dtype, H, n);
  return atom::check_launch();
}
