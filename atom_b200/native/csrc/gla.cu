// Gated linear attention: a matrix state per head whose rows decay by a number per key channel that depends on the
// token,
//   a_t = sigmoid(z_t + b)^(1/tau) = exp(-softplus(-(z_t + b)) / tau)
//   S_t = diag(a_t) S_(t-1) + k_t v_t^T;   o_t = S_t^T (q_t * q_scale)
// over every request's rows of the step, the state (32-bit) carried in the request's slot.  The decay, the state and
// every sum are 32-bit; q, k, v come from matrix products in the activation type, z from one with a 32-bit result.
//
// Every column of the state runs by itself, so a CTA owns (a run of a request's rows, a head, 32 value columns): a
// thread holds a quarter of one column's key channels in registers, the four quarters of a column sit in neighbouring
// lanes.  The recurrence is linear in S, so a request's rows are cut into runs of `run` rows:
//   mode 1  every run from S = 0: its sum B and the product A of its decays (S_end = diag(A) S_begin + B) to scratch
//   prefix  per request and state element, over the runs in order: the scratch takes the run's S_begin, the slot the
//           state after the step
//   mode 2  every run from its S_begin: the outputs
// and a step of few rows walks each request once (mode 0: slot in, outputs, slot out).  The cut into runs depends on
// the step's rows alone and changes only the order of 32-bit roundings.  In steps that are cut into runs every CTA
// of both walks would form the same decays again, so a kernel of its own turns z into the decays in place first.
//
//   gla_gate_norm_kernel   y = o / rms(o over a head's columns) * w * silu(g), w shared by the heads
#include "common.cuh"

namespace atom {

constexpr int kGlaThreads = 128;
constexpr int kGlaCols = 32;       // value columns per CTA
constexpr int kGlaStage = 16;      // rows staged in shared memory at a time

// Run slot x -> request and run: requests take ceil(len / run) slots one after another.
__device__ __forceinline__ bool gla_find_run(int x, const int* __restrict__ cu_q, int num_seqs, int run, int& s, int& r) {
  int acc = 0;
  for (s = 0; s < num_seqs; ++s) {
    const int len = cu_q[s + 1] - cu_q[s];
    const int n_runs = (len + run - 1) / run;
    if (x < acc + n_runs) {
      r = x - acc;
      return true;
    }
    acc += n_runs;
  }
  return false;
}

// Key channel of register m of a thread of slice 0..3: runs of four channels in a row (one 16-byte load each).
__device__ __forceinline__ int gla_channel(int slice, int m) { return (slice + 4 * (m / 4)) * 4 + (m % 4); }

__device__ __forceinline__ float gla_decay(float z, float inv_tau) {
  // log sigmoid(z) = -softplus(-z) = min(z, 0) - log1p(exp(-|z|))
  const float ls = fminf(z, 0.f) - log1pf(expf(-fabsf(z)));
  return expf(ls * inv_tau);
}

// q, k rows: [H dk] at stride ld; v rows [H dv] at stride ld; z rows [H dk] float at stride ldz.  out [T, H dv] float.
// state [slots, H, dk, dv]; sB [run slots, H, dk, dv]; sA [run slots, H, dk].
template <typename T, int KPT, int MODE>
__global__ void __launch_bounds__(kGlaThreads)
gla_scan_kernel(float* __restrict__ out, const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                int64_t ld, const float* __restrict__ z, int64_t ldz, const void* __restrict__ zb, int zb_dtype,
                float inv_tau, float q_scale, float* __restrict__ state, float* __restrict__ sB, float* __restrict__ sA,
                const int* __restrict__ cu_q, const int* __restrict__ state_slots, int num_seqs, int H, int dk, int dv,
                int run, int write_state) {
  atom::pdl_trigger();
  atom::pdl_wait();
  constexpr int DKP = 4 * KPT;
  extern __shared__ __align__(16) float gla_smem[];
  float* q_s = gla_smem;                       // [stage][DKP]
  float* k_s = q_s + kGlaStage * DKP;
  float* a_s = k_s + kGlaStage * DKP;
  float* v_s = a_s + kGlaStage * DKP;          // [stage][cols]
  int s, r = 0;
  if (MODE == 0) {
    s = blockIdx.x;
    if (s >= num_seqs) return;
  } else if (!gla_find_run(blockIdx.x, cu_q, num_seqs, run, s, r)) {
    return;
  }
  const int hd = blockIdx.y, col0 = blockIdx.z * kGlaCols;
  const int t0 = cu_q[s] + r * run;
  const int t1 = MODE == 0 ? cu_q[s + 1] : min(cu_q[s + 1], t0 + run);
  if (t1 <= t0) return;
  const int col = threadIdx.x >> 2, slice = threadIdx.x & 3;
  const int j = col0 + col;
  const bool lead = MODE == 1 && blockIdx.z == 0 && col == 0;     // the threads that form the run's product of decays
  float* S_g = state + (((int64_t)state_slots[s] * H + hd) * dk) * dv;
  float* B_g = sB ? sB + (((int64_t)blockIdx.x * H + hd) * dk) * dv : nullptr;
  float S[KPT], A[KPT];
#pragma unroll
  for (int m = 0; m < KPT; ++m) {
    const int ch = gla_channel(slice, m);
    A[m] = 1.f;
    if (MODE == 1 || ch >= dk || j >= dv) S[m] = 0.f;
    else S[m] = MODE == 0 ? S_g[(int64_t)ch * dv + j] : B_g[(int64_t)ch * dv + j];
  }
  const int64_t ldo = (int64_t)H * dv;
  for (int c0 = t0; c0 < t1; c0 += kGlaStage) {
    const int n = min(kGlaStage, t1 - c0);
    for (int e = threadIdx.x; e < n * DKP; e += kGlaThreads) {
      const int row = e / DKP, i = e - row * DKP;
      float qq = 0.f, kk = 0.f, aa = 1.f;
      if (i < dk) {
        const int64_t off = (int64_t)(c0 + row) * ld + (int64_t)hd * dk + i;
        qq = to_float(q[off]) * q_scale;
        kk = to_float(k[off]);
        const float zz = z[(int64_t)(c0 + row) * ldz + (int64_t)hd * dk + i];
        // (zb null: z holds the decays already)
        aa = zb ? gla_decay(zz + load_as_float(zb, zb_dtype, (int64_t)hd * dk + i), inv_tau) : zz;
      }
      q_s[e] = qq;
      k_s[e] = kk;
      a_s[e] = aa;
    }
    for (int e = threadIdx.x; e < n * kGlaCols; e += kGlaThreads) {
      const int row = e / kGlaCols, c = e - row * kGlaCols;
      v_s[e] = col0 + c < dv ? to_float(v[(int64_t)(c0 + row) * ld + (int64_t)hd * dv + col0 + c]) : 0.f;
    }
    __syncthreads();
    for (int row = 0; row < n; ++row) {
      const float vj = v_s[row * kGlaCols + col];
      float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
      for (int m4 = 0; m4 < KPT / 4; ++m4) {
        const int at = row * DKP + (slice + 4 * m4) * 4;
        const float4 a4 = *reinterpret_cast<const float4*>(a_s + at);
        const float4 k4 = *reinterpret_cast<const float4*>(k_s + at);
        S[4 * m4] = fmaf(a4.x, S[4 * m4], k4.x * vj);
        S[4 * m4 + 1] = fmaf(a4.y, S[4 * m4 + 1], k4.y * vj);
        S[4 * m4 + 2] = fmaf(a4.z, S[4 * m4 + 2], k4.z * vj);
        S[4 * m4 + 3] = fmaf(a4.w, S[4 * m4 + 3], k4.w * vj);
        if (MODE == 1) {
          if (lead) {
            A[4 * m4] *= a4.x;
            A[4 * m4 + 1] *= a4.y;
            A[4 * m4 + 2] *= a4.z;
            A[4 * m4 + 3] *= a4.w;
          }
        } else {
          const float4 q4 = *reinterpret_cast<const float4*>(q_s + at);
          acc0 = fmaf(q4.x, S[4 * m4], acc0);
          acc1 = fmaf(q4.y, S[4 * m4 + 1], acc1);
          acc0 = fmaf(q4.z, S[4 * m4 + 2], acc0);
          acc1 = fmaf(q4.w, S[4 * m4 + 3], acc1);
        }
      }
      if (MODE != 1) {
        float acc = acc0 + acc1;
        acc += __shfl_xor_sync(0xffffffffu, acc, 1);
        acc += __shfl_xor_sync(0xffffffffu, acc, 2);
        if (slice == 0 && j < dv) out[(int64_t)(c0 + row) * ldo + (int64_t)hd * dv + j] = acc;
      }
    }
    __syncthreads();
  }
  if (MODE == 0 && !write_state) return;
  if (MODE == 2) return;
  float* dst = MODE == 0 ? S_g : B_g;
#pragma unroll
  for (int m = 0; m < KPT; ++m) {
    const int ch = gla_channel(slice, m);
    if (ch < dk && j < dv) dst[(int64_t)ch * dv + j] = S[m];
    if (lead && ch < dk) sA[((int64_t)blockIdx.x * H + hd) * dk + ch] = A[m];
  }
}

// z[t, i] <- sigmoid(z[t, i] + b[i])^(1/tau), in place.
__global__ void gla_decay_kernel(float* __restrict__ z, int64_t ldz, const void* __restrict__ zb, int zb_dtype,
                                 float inv_tau, int n, int64_t total) {
  atom::pdl_trigger();
  atom::pdl_wait();
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = e / n;
    const int i = (int)(e - t * n);
    float* p = z + t * ldz + i;
    *p = gla_decay(*p + load_as_float(zb, zb_dtype, i), inv_tau);
  }
}

// Per request and state element, over the request's runs in order: sB[run] <- the state the run begins with, and the
// slot takes the state after the last run.
__global__ void gla_prefix_kernel(float* __restrict__ state, float* __restrict__ sB, const float* __restrict__ sA,
                                  const int* __restrict__ cu_q, const int* __restrict__ state_slots, int H, int dk,
                                  int dv, int run, int write_state) {
  atom::pdl_trigger();
  atom::pdl_wait();
  const int s = blockIdx.x, hd = blockIdx.y;
  const int len = cu_q[s + 1] - cu_q[s];
  if (len <= 0) return;
  int x0 = 0;
  for (int p = 0; p < s; ++p) x0 += (cu_q[p + 1] - cu_q[p] + run - 1) / run;
  const int n_runs = (len + run - 1) / run;
  float* S_g = state + (((int64_t)state_slots[s] * H + hd) * dk) * dv;
  for (int e = blockIdx.z * blockDim.x + threadIdx.x; e < dk * dv; e += gridDim.z * blockDim.x) {
    const int ch = e / dv;
    float S = S_g[e];
    for (int r = 0; r < n_runs; ++r) {
      float* B = sB + (((int64_t)(x0 + r) * H + hd) * dk) * dv + e;
      const float b = *B;
      *B = S;
      S = fmaf(sA[((int64_t)(x0 + r) * H + hd) * dk + ch], S, b);
    }
    if (write_state) S_g[e] = S;
  }
}

// y[t, h, :] = o[t, h, :] / rms(o[t, h, :]) * w * silu(g[t, h, :]); a warp per (token, head).
template <typename T>
__global__ void gla_gate_norm_kernel(T* __restrict__ y, const float* __restrict__ o, const T* __restrict__ g, int64_t ldg,
                                     const void* __restrict__ w, int w_dtype, int H, int dv, float eps,
                                     const int* __restrict__ seq_of_token) {
  atom::pdl_trigger();
  atom::pdl_wait();
  const int t = blockIdx.x;
  if (seq_of_token[t] < 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int h = warp; h < H; h += nwarps) {
    const float* orow = o + ((int64_t)t * H + h) * dv;
    float ss = 0.f;
    for (int i = lane; i < dv; i += 32) ss = fmaf(orow[i], orow[i], ss);
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / (float)dv + eps);
    for (int i = lane; i < dv; i += 32) {
      const float gg = to_float(g[(int64_t)t * ldg + (int64_t)h * dv + i]);
      y[((int64_t)t * H + h) * dv + i] =
          from_float<T>(orow[i] * rstd * load_as_float(w, w_dtype, i) * (gg / (1.f + expf(-gg))));
    }
  }
}

template <typename T, int KPT>
static int launch_gla(float* out, const T* q, const T* k, const T* v, int64_t ld, float* z, int64_t ldz,
                      const void* zb, int zb_dtype, float inv_tau, float q_scale, float* state, float* sB, float* sA,
                      const int* cu_q, const int* state_slots, int num_seqs, int T_, int H, int dk, int dv, int run,
                      int write_state, cudaStream_t stream) {
  const size_t smem = sizeof(float) * (size_t)kGlaStage * (3 * 4 * KPT + kGlaCols);
  const int colb = (dv + kGlaCols - 1) / kGlaCols;
  if (smem > 48 * 1024) {
    cudaFuncSetAttribute(gla_scan_kernel<T, KPT, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaFuncSetAttribute(gla_scan_kernel<T, KPT, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaFuncSetAttribute(gla_scan_kernel<T, KPT, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  }
  if (run <= 0) {
    launch_pdl(gla_scan_kernel<T, KPT, 0>, dim3(num_seqs, H, colb), dim3(kGlaThreads), smem, stream, out, q, k, v, ld, z,
               ldz, zb, zb_dtype, inv_tau, q_scale, state, (float*)nullptr, (float*)nullptr, cu_q, state_slots, num_seqs,
               H, dk, dv, 0, write_state);
    return check_launch();
  }
  const int slots = (T_ + run - 1) / run + num_seqs;
  {
    const int64_t total = (int64_t)T_ * H * dk;
    const int blocks = (int)((total + 255) / 256 > 148 * 16 ? 148 * 16 : (total + 255) / 256);
    launch_pdl(gla_decay_kernel, dim3(blocks), dim3(256), 0, stream, z, ldz, zb, zb_dtype, inv_tau, H * dk, total);
    zb = nullptr;
  }
  launch_pdl(gla_scan_kernel<T, KPT, 1>, dim3(slots, H, colb), dim3(kGlaThreads), smem, stream, out, q, k, v, ld, z, ldz,
             zb, zb_dtype, inv_tau, q_scale, state, sB, sA, cu_q, state_slots, num_seqs, H, dk, dv, run, write_state);
  const int eb = (dk * dv + 255) / 256;
  launch_pdl(gla_prefix_kernel, dim3(num_seqs, H, eb > 64 ? 64 : eb), dim3(256), 0, stream, state, sB, (const float*)sA,
             cu_q, state_slots, H, dk, dv, run, write_state);
  launch_pdl(gla_scan_kernel<T, KPT, 2>, dim3(slots, H, colb), dim3(kGlaThreads), smem, stream, out, q, k, v, ld, z, ldz,
             zb, zb_dtype, inv_tau, q_scale, state, sB, sA, cu_q, state_slots, num_seqs, H, dk, dv, run, write_state);
  return check_launch();
}

template <typename T>
static int dispatch_gla(float* out, const T* q, const T* k, const T* v, int64_t ld, float* z, int64_t ldz,
                        const void* zb, int zb_dtype, float inv_tau, float q_scale, float* state, float* sB, float* sA,
                        const int* cu_q, const int* state_slots, int num_seqs, int T_, int H, int dk, int dv, int run,
                        int write_state, cudaStream_t stream) {
#define ATOM_GLA_CASE(N)                                                                                             \
  if (dk <= 4 * N)                                                                                                   \
    return launch_gla<T, N>(out, q, k, v, ld, z, ldz, zb, zb_dtype, inv_tau, q_scale, state, sB, sA, cu_q, state_slots, \
                            num_seqs, T_, H, dk, dv, run, write_state, stream);
  ATOM_GLA_CASE(4)
  ATOM_GLA_CASE(8)
  ATOM_GLA_CASE(16)
  ATOM_GLA_CASE(24)
  ATOM_GLA_CASE(32)
  ATOM_GLA_CASE(48)
  ATOM_GLA_CASE(64)
#undef ATOM_GLA_CASE
  return ATOM_ERR_ARG;
}

}  // namespace atom

ATOM_EXPORT int atom_gla_supports(int dk, int dv) { return dk > 0 && dk <= 256 && dv > 0 ? 1 : 0; }

// run 0: every request is walked once.  Otherwise z is overwritten with the decays, sB holds (ceil(T / run) + num_seqs) * H * dk * dv floats and sA
// (ceil(T / run) + num_seqs) * H * dk.
ATOM_EXPORT int atom_gla_scan(float* out, const void* q, const void* k, const void* v, int dtype, int64_t ld,
                              float* z, int64_t ldz, const void* zb, int zb_dtype, float tau, float q_scale,
                              float* state, float* sB, float* sA, const int* cu_q, const int* state_slots, int num_seqs,
                              int T, int H, int dk, int dv, int run, int write_state, cudaStream_t stream) {
  if (T <= 0 || num_seqs <= 0) return ATOM_OK;
  if (!atom_gla_supports(dk, dv) || H <= 0 || H > 65535 || !(tau > 0.f) || (run > 0 && (!sB || !sA))) return ATOM_ERR_ARG;
  if (zb_dtype != ATOM_F32 && zb_dtype != ATOM_BF16) return ATOM_ERR_ARG;
  if (dtype == ATOM_F32)
    return atom::dispatch_gla<float>(out, (const float*)q, (const float*)k, (const float*)v, ld, z, ldz, zb, zb_dtype,
                                     1.f / tau, q_scale, state, sB, sA, cu_q, state_slots, num_seqs, T, H, dk, dv, run,
                                     write_state, stream);
  if (dtype == ATOM_BF16)
    return atom::dispatch_gla<__nv_bfloat16>(out, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k,
                                             (const __nv_bfloat16*)v, ld, z, ldz, zb, zb_dtype, 1.f / tau, q_scale, state,
                                             sB, sA, cu_q, state_slots, num_seqs, T, H, dk, dv, run, write_state, stream);
  return ATOM_ERR_ARG;
}

ATOM_EXPORT int atom_gla_gate_norm(void* y, const float* o, const void* g, int dtype, int64_t ldg, const void* w,
                                   int w_dtype, int T, int H, int dv, float eps, const int* seq_of_token,
                                   cudaStream_t stream) {
  if (T <= 0) return ATOM_OK;
  if (H <= 0 || dv <= 0 || (w_dtype != ATOM_F32 && w_dtype != ATOM_BF16)) return ATOM_ERR_ARG;
  const int threads = H >= 8 ? 256 : 32 * H;
  if (dtype == ATOM_F32)
    atom::launch_pdl(atom::gla_gate_norm_kernel<float>, dim3(T), dim3(threads), 0, stream, (float*)y, o, (const float*)g,
                     ldg, w, w_dtype, H, dv, eps, seq_of_token);
  else if (dtype == ATOM_BF16)
    atom::launch_pdl(atom::gla_gate_norm_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, (__nv_bfloat16*)y, o,
                     (const __nv_bfloat16*)g, ldg, w, w_dtype, H, dv, eps, seq_of_token);
  else
    return ATOM_ERR_ARG;
  return atom::check_launch();
}
