// Lightning attention: a matrix state per head with one constant decay per head,
//   q = silu(.), k = silu(.), v = silu(.);   S_t = decay_h * S_(t-1) + k_t v_t^T;   o_t = S_t^T q_t
// over every request's rows of the step, the state (32-bit) carried in the request's slot.
//
// Every column of the state runs by itself, so a CTA owns (a run of a request's rows, a head, 32 value columns): a
// thread holds a quarter of one column's key channels in registers, the four quarters of a column sit in neighbouring
// lanes.  The recurrence is linear in S, so a request's rows are cut into runs of `run` rows:
//   mode 1  every run from S = 0: its sum B (S_end = decay^len S_begin + B) to the scratch array
//   prefix  per request and state element, over the runs in order: the scratch takes the run's S_begin, the slot
//           the state after the step
//   mode 2  every run from its S_begin: the outputs
// and a step of few rows walks each request once (mode 0: slot in, outputs, slot out).  The cut into runs depends on
// the step's rows alone and changes only the order of 32-bit roundings.
//
//   lightning_gate_norm_kernel   y = o / rms(o over all heads) * w * sigmoid(g)
#include "common.cuh"

namespace atom {

constexpr int kLtThreads = 128;
constexpr int kLtCols = 32;       // value columns per CTA
constexpr int kLtStage = 16;      // rows staged in shared memory at a time

__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }

// Finds the request and the run of run slot x: requests take ceil(len / run) slots one after another (a request
// without rows takes none).  Returns false when x lies beyond the step's runs.
__device__ __forceinline__ bool find_run(int x, const int* __restrict__ cu_q, int num_seqs, int run, int& s, int& r,
                                         int& n_runs) {
  int acc = 0;
  for (s = 0; s < num_seqs; ++s) {
    const int len = cu_q[s + 1] - cu_q[s];
    n_runs = (len + run - 1) / run;
    if (x < acc + n_runs) {
      r = x - acc;
      return true;
    }
    acc += n_runs;
  }
  return false;
}

// Key channel of register m of a thread of slice 0..3: with KPT a multiple of 4 a thread holds runs of four channels
// in a row (one 16-byte load of shared memory a run), else every fourth channel.
template <int KPT>
__device__ __forceinline__ int lt_channel(int slice, int m) {
  return KPT % 4 == 0 ? (slice + 4 * (m / 4)) * 4 + (m % 4) : slice + 4 * m;
}

// proj rows: [q (H dk) | k (H dk) | v (H dv) | ...], row stride ld.  out [T, H dv] float32.  state [slots, H, dk, dv].
// scratch [run slots, H, dk, dv].
template <typename T, int KPT, int MODE>
__global__ void __launch_bounds__(kLtThreads)
lightning_scan_kernel(float* __restrict__ out, const T* __restrict__ proj, int64_t ld, const float* __restrict__ decay,
                      float* __restrict__ state, float* __restrict__ scratch, const int* __restrict__ cu_q,
                      const int* __restrict__ state_slots, int num_seqs, int H, int dk, int dv, int run,
                      int write_state) {
  atom::pdl_trigger();
  atom::pdl_wait();
  extern __shared__ __align__(16) float lt_smem[];
  const int dkp = (dk + 3) & ~3;                // rows of k and q are padded with zeros to whole 16-byte loads
  float* ks = lt_smem;                          // [kLtStage][dkp]
  float* qs = ks + kLtStage * dkp;              // [kLtStage][dkp]
  float* vs = qs + kLtStage * dkp;              // [kLtStage][kLtCols]
  int s, r, n_runs;
  if (MODE == 0) {
    s = blockIdx.x;
    r = 0;
    n_runs = 1;
    if (s >= num_seqs) return;
  } else if (!find_run(blockIdx.x, cu_q, num_seqs, run, s, r, n_runs)) {
    return;
  }
  const int h = blockIdx.y;
  const int c0 = blockIdx.z * kLtCols;
  const int first = cu_q[s] + r * run;
  const int len = (MODE == 0) ? (cu_q[s + 1] - cu_q[s]) : min(run, cu_q[s + 1] - first);
  if (len <= 0) return;
  const int slice = threadIdx.x & 3, col = threadIdx.x >> 2;
  const int c = c0 + col;
  const bool live = c < dv;
  const float lam = decay[h];
  const int64_t mat = (int64_t)dk * dv;
  float S[KPT];
  if (MODE == 1) {
#pragma unroll
    for (int m = 0; m < KPT; ++m) S[m] = 0.f;
  } else {
    const float* src = (MODE == 0) ? state + ((int64_t)state_slots[s] * H + h) * mat
                                   : scratch + ((int64_t)blockIdx.x * H + h) * mat;
#pragma unroll
    for (int m = 0; m < KPT; ++m) {
      const int i = lt_channel<KPT>(slice, m);
      S[m] = (live && i < dk) ? src[(int64_t)i * dv + c] : 0.f;
    }
  }
  const int q_off = h * dk, k_off = H * dk + h * dk, v_off = 2 * H * dk + h * dv + c0;
  for (int t0 = 0; t0 < len; t0 += kLtStage) {
    const int n = min(kLtStage, len - t0);
    __syncthreads();
    for (int idx = threadIdx.x; idx < n * dkp; idx += kLtThreads) {
      const int tt = idx / dkp, i = idx - tt * dkp;
      const T* row = proj + (int64_t)(first + t0 + tt) * ld;
      ks[idx] = i < dk ? silu_f(to_float(row[k_off + i])) : 0.f;
      if (MODE != 1) qs[idx] = i < dk ? silu_f(to_float(row[q_off + i])) : 0.f;
    }
    for (int idx = threadIdx.x; idx < n * kLtCols; idx += kLtThreads) {
      const int tt = idx / kLtCols, j = idx - tt * kLtCols;
      vs[idx] = (c0 + j < dv) ? silu_f(to_float(proj[(int64_t)(first + t0 + tt) * ld + v_off + j])) : 0.f;
    }
    __syncthreads();
    for (int tt = 0; tt < n; ++tt) {
      const float v = vs[tt * kLtCols + col];
      const float* kr = ks + tt * dkp;
      const float* qr = qs + tt * dkp;
      float acc = 0.f;
      if (KPT % 4 == 0) {
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;      // four sums side by side: chains of KPT / 4 dependent FMAs
        // four channels in a row per load: the lanes of a slice read the same 16 bytes of shared memory
#pragma unroll
        for (int m4 = 0; m4 < KPT / 4; ++m4) {
          const int i = (slice + 4 * m4) * 4;
          if (i < dk) {          // (channels from dk up to the row's padded end are zeros)
            const float4 k4 = *reinterpret_cast<const float4*>(kr + i);
            S[4 * m4 + 0] = lam * S[4 * m4 + 0] + k4.x * v;
            S[4 * m4 + 1] = lam * S[4 * m4 + 1] + k4.y * v;
            S[4 * m4 + 2] = lam * S[4 * m4 + 2] + k4.z * v;
            S[4 * m4 + 3] = lam * S[4 * m4 + 3] + k4.w * v;
            if (MODE != 1) {
              const float4 q4 = *reinterpret_cast<const float4*>(qr + i);
              a0 = fmaf(S[4 * m4 + 0], q4.x, a0);
              a1 = fmaf(S[4 * m4 + 1], q4.y, a1);
              a2 = fmaf(S[4 * m4 + 2], q4.z, a2);
              a3 = fmaf(S[4 * m4 + 3], q4.w, a3);
            }
          }
        }
        acc = (a0 + a1) + (a2 + a3);
      } else {
#pragma unroll
        for (int m = 0; m < KPT; ++m) {
          const int i = slice + 4 * m;
          if (i < dk) {
            S[m] = lam * S[m] + kr[i] * v;
            if (MODE != 1) acc += S[m] * qr[i];
          }
        }
      }
      if (MODE != 1) {
        acc += __shfl_xor_sync(0xffffffffu, acc, 1);
        acc += __shfl_xor_sync(0xffffffffu, acc, 2);
        if (slice == 0 && live) out[(int64_t)(first + t0 + tt) * H * dv + h * dv + c] = acc;
      }
    }
  }
  if (MODE == 2 || (MODE == 0 && !write_state)) return;
  float* dst = (MODE == 0) ? state + ((int64_t)state_slots[s] * H + h) * mat
                           : scratch + ((int64_t)blockIdx.x * H + h) * mat;
#pragma unroll
  for (int m = 0; m < KPT; ++m) {
    const int i = lt_channel<KPT>(slice, m);
    if (live && i < dk) dst[(int64_t)i * dv + c] = S[m];
  }
}

// One thread per (request, head, state element): walks the request's runs in order.
__global__ void lightning_prefix_kernel(float* __restrict__ state, float* __restrict__ scratch,
                                        const float* __restrict__ decay, const int* __restrict__ cu_q,
                                        const int* __restrict__ state_slots, int H, int dk, int dv, int run,
                                        int write_state) {
  atom::pdl_trigger();
  atom::pdl_wait();
  const int s = blockIdx.z, h = blockIdx.y;
  const int64_t mat = (int64_t)dk * dv;
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= mat) return;
  int slot0 = 0;
  for (int j = 0; j < s; ++j) slot0 += (cu_q[j + 1] - cu_q[j] + run - 1) / run;
  const int len = cu_q[s + 1] - cu_q[s];
  const int n_runs = (len + run - 1) / run;
  if (n_runs <= 0) return;
  const float lam = decay[h];
  const float lam_run = powf(lam, (float)run);
  float* st = state + ((int64_t)state_slots[s] * H + h) * mat + e;
  float S = *st;
  // the runs' sums do not depend on S: sixteen loads are under way together before the chain of updates uses them
  constexpr int kAhead = 16;
  for (int r0 = 0; r0 < n_runs; r0 += kAhead) {
    float sums[kAhead];
#pragma unroll
    for (int j = 0; j < kAhead; ++j)
      sums[j] = (r0 + j < n_runs) ? scratch[((int64_t)(slot0 + r0 + j) * H + h) * mat + e] : 0.f;
#pragma unroll
    for (int j = 0; j < kAhead; ++j) {
      const int r = r0 + j;
      if (r < n_runs) {
        scratch[((int64_t)(slot0 + r) * H + h) * mat + e] = S;
        const int rl = min(run, len - r * run);
        S = (rl == run ? lam_run : powf(lam, (float)rl)) * S + sums[j];
      }
    }
  }
  if (write_state) *st = S;
}

// o [T, n] float32 (all heads of a row side by side); g: rows of the projection (stride ld); y [T, n].
template <typename T>
__global__ void lightning_gate_norm_kernel(T* __restrict__ y, const float* __restrict__ o, const T* __restrict__ g,
                                           int64_t ld, const void* __restrict__ w, int w_dtype, int n, float eps,
                                           const int* __restrict__ seq_of_token) {
  atom::pdl_trigger();
  atom::pdl_wait();
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  if (seq_of_token[t] < 0) return;
  const float* row = o + (int64_t)t * n;
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) ss += row[i] * row[i];
  ss = block_sum(ss, scratch);
  const float rstd = rsqrtf(ss / (float)n + eps);
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float gate = 1.f / (1.f + expf(-to_float(g[(int64_t)t * ld + i])));
    y[(int64_t)t * n + i] = from_float<T>(row[i] * rstd * load_as_float(w, w_dtype, i) * gate);
  }
}

template <typename T, int KPT>
static int lightning_launch(float* out, const T* proj, int64_t ld, const float* decay, float* state, float* scratch,
                            const int* cu_q, const int* state_slots, int num_seqs, int T_rows, int H, int dk, int dv,
                            int run, int write_state, cudaStream_t stream) {
  const size_t smem = sizeof(float) * kLtStage * (2 * ((dk + 3) & ~3) + kLtCols);
  const int tiles = (dv + kLtCols - 1) / kLtCols;
  if (run <= 0) {      // few rows: every request is walked once
    launch_pdl(lightning_scan_kernel<T, KPT, 0>, dim3(num_seqs, H, tiles), dim3(kLtThreads), smem, stream, out, proj,
               ld, decay, state, scratch, cu_q, state_slots, num_seqs, H, dk, dv, 0, write_state);
    return check_launch();
  }
  const int slots = (T_rows + run - 1) / run + num_seqs;
  launch_pdl(lightning_scan_kernel<T, KPT, 1>, dim3(slots, H, tiles), dim3(kLtThreads), smem, stream, out, proj, ld,
             decay, state, scratch, cu_q, state_slots, num_seqs, H, dk, dv, run, write_state);
  const int64_t mat = (int64_t)dk * dv;
  launch_pdl(lightning_prefix_kernel, dim3((unsigned)((mat + 255) / 256), H, num_seqs), dim3(256), 0, stream, state,
             scratch, decay, cu_q, state_slots, H, dk, dv, run, write_state);
  launch_pdl(lightning_scan_kernel<T, KPT, 2>, dim3(slots, H, tiles), dim3(kLtThreads), smem, stream, out, proj, ld,
             decay, state, scratch, cu_q, state_slots, num_seqs, H, dk, dv, run, write_state);
  return check_launch();
}

template <typename T>
static int lightning_dispatch(float* out, const T* proj, int64_t ld, const float* decay, float* state, float* scratch,
                              const int* cu_q, const int* state_slots, int num_seqs, int T_rows, int H, int dk, int dv,
                              int run, int write_state, cudaStream_t stream) {
#define ATOM_LT(K) \
  return lightning_launch<T, K>(out, proj, ld, decay, state, scratch, cu_q, state_slots, num_seqs, T_rows, H, dk, dv, \
                                run, write_state, stream)
  if (dk <= 32) ATOM_LT(8);
  if (dk <= 64) ATOM_LT(16);
  if (dk <= 128) ATOM_LT(32);
  ATOM_LT(64);
#undef ATOM_LT
}

}  // namespace atom

ATOM_EXPORT int atom_lightning_supports(int dk, int dv) { return dk > 0 && dk <= 256 && dv > 0 ? 1 : 0; }

// run <= 0: every request walked once (steps of few rows); else rows per run, with scratch of
// (ceil(T / run) + num_seqs) * H * dk * dv floats.
ATOM_EXPORT int atom_lightning_scan(float* out, const void* proj, int dtype, int64_t ld, const float* decay,
                                    float* state, float* scratch, const int* cu_q, const int* state_slots,
                                    int num_seqs, int T, int H, int dk, int dv, int run, int write_state,
                                    cudaStream_t stream) {
  if (T <= 0 || num_seqs <= 0) return ATOM_OK;
  if (H <= 0 || H > 65535 || num_seqs > 65535 || !atom_lightning_supports(dk, dv) || (run > 0 && !scratch))
    return ATOM_ERR_ARG;
  if (dtype == ATOM_F32)
    return atom::lightning_dispatch<float>(out, (const float*)proj, ld, decay, state, scratch, cu_q, state_slots,
                                           num_seqs, T, H, dk, dv, run, write_state, stream);
  if (dtype == ATOM_BF16)
    return atom::lightning_dispatch<__nv_bfloat16>(out, (const __nv_bfloat16*)proj, ld, decay, state, scratch, cu_q,
                                                   state_slots, num_seqs, T, H, dk, dv, run, write_state, stream);
  return ATOM_ERR_ARG;
}

ATOM_EXPORT int atom_lightning_gate_norm(void* y, const float* o, const void* g, int dtype, int64_t ld, const void* w,
                                         int w_dtype, int T, int n, float eps, const int* seq_of_token,
                                         cudaStream_t stream) {
  if (T <= 0) return ATOM_OK;
  if (n <= 0) return ATOM_ERR_ARG;
  const int threads = n >= 1024 ? 256 : 128;
  if (dtype == ATOM_F32)
    atom::launch_pdl(atom::lightning_gate_norm_kernel<float>, dim3(T), dim3(threads), 0, stream, (float*)y, o,
                     (const float*)g, ld, w, w_dtype, n, eps, seq_of_token);
  else if (dtype == ATOM_BF16)
    atom::launch_pdl(atom::lightning_gate_norm_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream,
                     (__nv_bfloat16*)y, o, (const __nv_bfloat16*)g, ld, w, w_dtype, n, eps, seq_of_token);
  else
    return ATOM_ERR_ARG;
  return atom::check_launch();
}
