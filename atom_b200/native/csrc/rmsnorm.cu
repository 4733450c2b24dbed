// Fused residual add + RMSNorm.
//   r = residual[row] (+ dscale * delta[row]);  residual[row] = r  (unless rows are picked);
//   out[i] = r * rsqrt(mean(r^2) + eps) * w
// The residual stream and all arithmetic are 32-bit; `delta` (the previous block's
// output) and `out` (the next matrix product's input) have the activation type.
// With `rows` given, only those rows are normalised and written densely: this is
// the gather of the rows whose logits are wanted, fused into the final norm.
#include "common.cuh"

namespace atom {

template <typename TA>
__global__ void add_rmsnorm_kernel(TA* __restrict__ out, float* __restrict__ residual,
                                   const TA* __restrict__ delta, const void* __restrict__ w,
                                   int w_dtype, float eps, const int* __restrict__ rows, int H, float dscale) {
  atom::pdl_trigger();   // the next kernel may be scheduled at once: before its own wait it reads nothing a kernel of this step writes
  atom::pdl_wait();      // inputs written by the kernel before this one are visible from here on
  __shared__ float scratch[32];
  const int r = blockIdx.x;
  const int64_t src = rows ? rows[r] : r;
  float* res = residual + src * H;
  const TA* d = delta ? delta + src * H : nullptr;
  TA* o = out + (int64_t)r * H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = res[i];
    if (d) {
      v = fmaf(dscale, to_float(d[i]), v);
      // Picked rows are not carried further: their sum is formed again in the second pass
      // instead of being written back.
      if (!rows) res[i] = v;
    }
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float rstd = rsqrtf(ss / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = res[i];
    if (d && rows) v = fmaf(dscale, to_float(d[i]), v);
    o[i] = from_float<TA>(v * rstd * load_as_float(w, w_dtype, i));
  }
}

// Plain RMSNorm over the last dimension of a dense [rows, H] array of the activation type.
template <typename TA>
__global__ void rmsnorm_kernel(TA* __restrict__ out, const TA* __restrict__ x,
                               const void* __restrict__ w, int w_dtype, float eps, int H) {
  atom::pdl_trigger();   // the next kernel may be scheduled at once: before its own wait it reads nothing a kernel of this step writes
  atom::pdl_wait();      // inputs written by the kernel before this one are visible from here on
  __shared__ float scratch[32];
  const TA* xi = x + (int64_t)blockIdx.x * H;
  TA* o = out + (int64_t)blockIdx.x * H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = to_float(xi[i]);
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float rstd = rsqrtf(ss / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x)
    o[i] = from_float<TA>(to_float(xi[i]) * rstd * load_as_float(w, w_dtype, i));
}

static inline int norm_threads(int H) { return H >= 2048 ? 512 : (H >= 512 ? 256 : 128); }

// bf16 activations, H a multiple of 8, at most 8 * NV * blockDim: every thread keeps its
// 8 * NV elements in registers, so the row is read once and written once, 16 bytes at a time.
template <int NV>
__global__ void add_rmsnorm_bf16_vec_kernel(__nv_bfloat16* __restrict__ out, float* __restrict__ residual,
                                            const __nv_bfloat16* __restrict__ delta,
                                            const void* __restrict__ w, int w_dtype, float eps,
                                            const int* __restrict__ rows, int H, float dscale) {
  atom::pdl_trigger();   // the next kernel may be scheduled at once: before its own wait it reads nothing a kernel of this step writes
  __shared__ float scratch[32];
  const int r = blockIdx.x;
  const int64_t src = rows ? rows[r] : r;
  // The norm weights do not depend on the kernel in front of this one: they are on their way before the wait.
  float wv[NV][8];
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = (threadIdx.x + k * blockDim.x) * 8;
    if (i < H) {
      if (w_dtype == ATOM_F32) {
        const float4 a = *reinterpret_cast<const float4*>((const float*)w + i);
        const float4 b = *reinterpret_cast<const float4*>((const float*)w + i + 4);
        wv[k][0] = a.x; wv[k][1] = a.y; wv[k][2] = a.z; wv[k][3] = a.w;
        wv[k][4] = b.x; wv[k][5] = b.y; wv[k][6] = b.z; wv[k][7] = b.w;
      } else {
        const uint4 q = *reinterpret_cast<const uint4*>((const __nv_bfloat16*)w + i);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(h[e]);
          wv[k][2 * e] = f.x;
          wv[k][2 * e + 1] = f.y;
        }
      }
    }
  }
  atom::pdl_wait();      // inputs written by the kernel before this one are visible from here on
  float* res = residual + src * H;
  const __nv_bfloat16* d = delta ? delta + src * H : nullptr;
  float v[NV][8];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = (threadIdx.x + k * blockDim.x) * 8;
    if (i < H) {
      const float4 a = *reinterpret_cast<const float4*>(res + i);
      const float4 b = *reinterpret_cast<const float4*>(res + i + 4);
      v[k][0] = a.x; v[k][1] = a.y; v[k][2] = a.z; v[k][3] = a.w;
      v[k][4] = b.x; v[k][5] = b.y; v[k][6] = b.z; v[k][7] = b.w;
      if (d) {
        const uint4 q = *reinterpret_cast<const uint4*>(d + i);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(h[e]);
          v[k][2 * e] = fmaf(dscale, f.x, v[k][2 * e]);
          v[k][2 * e + 1] = fmaf(dscale, f.y, v[k][2 * e + 1]);
        }
        if (!rows) {
          *reinterpret_cast<float4*>(res + i) = make_float4(v[k][0], v[k][1], v[k][2], v[k][3]);
          *reinterpret_cast<float4*>(res + i + 4) = make_float4(v[k][4], v[k][5], v[k][6], v[k][7]);
        }
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += v[k][e] * v[k][e];
    }
  }
  ss = block_sum(ss, scratch);
  const float rstd = rsqrtf(ss / (float)H + eps);
  __nv_bfloat16* o = out + (int64_t)r * H;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = (threadIdx.x + k * blockDim.x) * 8;
    if (i < H) {
      uint4 q;
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
      for (int e = 0; e < 4; ++e)
        h[e] = __floats2bfloat162_rn(v[k][2 * e] * rstd * wv[k][2 * e], v[k][2 * e + 1] * rstd * wv[k][2 * e + 1]);
      *reinterpret_cast<uint4*>(o + i) = q;
    }
  }
}

// Two branches that end in an RMSNorm of their own, averaged into the residual stream, with an optional
// third addend:   residual[row] += 0.5 * (rmsnorm(a; wa) + rmsnorm(b; wb)) (+ c),   all in 32-bit.
// With b null there is one branch and no halving: residual[row] += rmsnorm(a; wa) (+ c); with wa null as
// well a is added as it is: residual[row] += a (+ c).
template <typename TA>
__global__ void pair_rmsnorm_add_kernel(float* __restrict__ residual, const TA* __restrict__ a,
                                        const void* __restrict__ wa, const TA* __restrict__ b,
                                        const void* __restrict__ wb, int w_dtype, const TA* __restrict__ c,
                                        float eps, int H) {
  atom::pdl_trigger();
  atom::pdl_wait();
  __shared__ float scratch[32];
  const int64_t r = blockIdx.x;
  const TA* ar = a + r * H;
  const TA* br = b ? b + r * H : nullptr;
  float sa = 0.f, sb = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float x = to_float(ar[i]);
    sa = fmaf(x, x, sa);
    if (br) {
      const float y = to_float(br[i]);
      sb = fmaf(y, y, sb);
    }
  }
  sa = block_sum(sa, scratch);
  sb = block_sum(sb, scratch);
  const float ra = rsqrtf(sa / (float)H + eps), rb = rsqrtf(sb / (float)H + eps);
  float* res = residual + r * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = to_float(ar[i]);
    if (wa) v = v * ra * load_as_float(wa, w_dtype, i);
    if (br) v = 0.5f * (v + to_float(br[i]) * rb * load_as_float(wb, w_dtype, i));
    if (c) v += to_float(c[r * H + i]);
    res[i] += v;
  }
}

}  // namespace atom

ATOM_EXPORT int atom_pair_rmsnorm_add(float* residual, const void* a, const void* wa, const void* b, const void* wb,
                                      int w_dtype, const void* c, int act_dtype, float eps, int n_rows, int H,
                                      cudaStream_t stream) {
  if (n_rows <= 0) return ATOM_OK;
  if (H <= 0 || (w_dtype != ATOM_F32 && w_dtype != ATOM_BF16)) return ATOM_ERR_ARG;
  const int threads = atom::norm_threads(H);
  if (act_dtype == ATOM_F32)
    atom::launch_pdl(atom::pair_rmsnorm_add_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, residual, (const float*)a, wa, (const float*)b, wb, w_dtype, (const float*)c, eps, H);
  else if (act_dtype == ATOM_BF16)
    atom::launch_pdl(atom::pair_rmsnorm_add_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, stream, residual, (const __nv_bfloat16*)a, wa, (const __nv_bfloat16*)b, wb, w_dtype, (const __nv_bfloat16*)c, eps, H);
  else
    return ATOM_ERR_ARG;
  return atom::check_launch();
}

ATOM_EXPORT int atom_add_rmsnorm(void* out, int act_dtype, float* residual, const void* delta,
                                 const void* w, int w_dtype, float eps, const int* rows, int n_rows,
                                 int H, float dscale, cudaStream_t stream) {
  if (n_rows <= 0) return ATOM_OK;
  if (H <= 0 || (w_dtype != ATOM_F32 && w_dtype != ATOM_BF16)) return ATOM_ERR_ARG;
  const int threads = atom::norm_threads(H);
  const bool aligned = ((uintptr_t)out % 16 == 0) && ((uintptr_t)residual % 16 == 0) &&
                       ((uintptr_t)delta % 16 == 0) && ((uintptr_t)w % 16 == 0);
  if (act_dtype == ATOM_BF16 && H % 8 == 0 && H <= 8 * 2 * 1024 && aligned) {
    // one pass over the row, 16-byte accesses: 128 to 1024 threads, one or two vectors each
    const int vecs = H / 8;
    int nv = 1, th = ((vecs + 31) / 32) * 32;
    if (th > 1024) {
      nv = 2;
      th = (((vecs + 1) / 2 + 31) / 32) * 32;
    }
    if (th < 64) th = 64;
    if (nv == 1)
      atom::launch_pdl(atom::add_rmsnorm_bf16_vec_kernel<1>, dim3(n_rows), dim3(th), 0, stream, (__nv_bfloat16*)out, residual, (const __nv_bfloat16*)delta, w, w_dtype, eps, rows, H, dscale);
    else
      atom::launch_pdl(atom::add_rmsnorm_bf16_vec_kernel<2>, dim3(n_rows), dim3(th), 0, stream, (__nv_bfloat16*)out, residual, (const __nv_bfloat16*)delta, w, w_dtype, eps, rows, H, dscale);
    return atom::check_launch();
  }
  if (act_dtype == ATOM_F32) {
    atom::launch_pdl(atom::add_rmsnorm_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, (float*)out, residual, (const float*)delta, w, w_dtype, eps, rows, H, dscale);
  } else if (act_dtype == ATOM_BF16) {
    atom::launch_pdl(atom::add_rmsnorm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, stream, (__nv_bfloat16*)out, residual, (const __nv_bfloat16*)delta, w, w_dtype, eps, rows, H, dscale);
  } else {
    return ATOM_ERR_ARG;
  }
  return atom::check_launch();
}

ATOM_EXPORT int atom_rmsnorm(void* out, const void* x, int act_dtype, const void* w, int w_dtype,
                             float eps, int n_rows, int H, cudaStream_t stream) {
  if (n_rows <= 0) return ATOM_OK;
  if (H <= 0 || (w_dtype != ATOM_F32 && w_dtype != ATOM_BF16)) return ATOM_ERR_ARG;
  const int threads = atom::norm_threads(H);
  if (act_dtype == ATOM_F32) {
    atom::launch_pdl(atom::rmsnorm_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, (float*)out, (const float*)x, w, w_dtype, eps, H);
  } else if (act_dtype == ATOM_BF16) {
    atom::launch_pdl(atom::rmsnorm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)x, w, w_dtype, eps, H);
  } else {
    return ATOM_ERR_ARG;
  }
  return atom::check_launch();
}

// A sub-block whose output passes an RMSNorm of its own before it enters the residual stream, fused with the norm
// that reads the stream next:
//   r = residual[row] + rmsnorm(delta[row]; wd, eps_d);   residual[row] = r (unless rows are picked);
//   out = rmsnorm(r; w, eps)
// all in 32-bit; the row's numbers wait in shared memory between the passes.
namespace atom {

template <typename TA>
__global__ void normed_add_rmsnorm_kernel(TA* __restrict__ out, float* __restrict__ residual,
                                          const TA* __restrict__ delta, const void* __restrict__ wd, float eps_d,
                                          const void* __restrict__ w, int w_dtype, float eps,
                                          const int* __restrict__ rows, int H) {
  atom::pdl_trigger();
  atom::pdl_wait();
  extern __shared__ float row_s[];
  __shared__ float scratch[32];
  const int r = blockIdx.x;
  const int64_t src = rows ? rows[r] : r;
  float* res = residual + src * H;
  const TA* d = delta + src * H;
  float sd = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float v = to_float(d[i]);
    row_s[i] = v;
    sd = fmaf(v, v, sd);
  }
  sd = block_sum(sd, scratch);
  const float rd = rsqrtf(sd / (float)H + eps_d);
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float v = res[i] + row_s[i] * rd * load_as_float(wd, w_dtype, i);
    row_s[i] = v;
    if (!rows) res[i] = v;
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float rstd = rsqrtf(ss / (float)H + eps);
  TA* o = out + (int64_t)r * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x)
    o[i] = from_float<TA>(row_s[i] * rstd * load_as_float(w, w_dtype, i));
}

// The same for bfloat16 rows of a multiple of 8 numbers, at most 8 * NV * blockDim: a thread keeps its 8 * NV numbers in
// registers, so that every array is read once and written once, 16 bytes at a time.
__device__ __forceinline__ void load8(const void* w, int w_dtype, int i, float (&o)[8]) {
  if (w_dtype == ATOM_F32) {
    const float4 a = *reinterpret_cast<const float4*>((const float*)w + i);
    const float4 b = *reinterpret_cast<const float4*>((const float*)w + i + 4);
    o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
  } else {
    const uint4 q = *reinterpret_cast<const uint4*>((const __nv_bfloat16*)w + i);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = __bfloat1622float2(h[e]);
      o[2 * e] = f.x;
      o[2 * e + 1] = f.y;
    }
  }
}

template <int NV>
__global__ void normed_add_rmsnorm_bf16_vec_kernel(__nv_bfloat16* __restrict__ out, float* __restrict__ residual,
                                                   const __nv_bfloat16* __restrict__ delta, const void* __restrict__ wd,
                                                   float eps_d, const void* __restrict__ w, int w_dtype, float eps,
                                                   const int* __restrict__ rows, int H) {
  atom::pdl_trigger();
  atom::pdl_wait();
  __shared__ float scratch[32];
  const int r = blockIdx.x;
  const int64_t src = rows ? rows[r] : r;
  float v[NV][8];
  float sd = 0.f;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = (threadIdx.x + k * blockDim.x) * 8;
    if (i < H) {
      load8(delta + src * H, ATOM_BF16, i, v[k]);
#pragma unroll
      for (int e = 0; e < 8; ++e) sd = fmaf(v[k][e], v[k][e], sd);
    }
  }
  sd = block_sum(sd, scratch);
  const float rd = rsqrtf(sd / (float)H + eps_d);
  float* res = residual + src * H;
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = (threadIdx.x + k * blockDim.x) * 8;
    if (i < H) {
      float wv[8], rv[8];
      load8(wd, w_dtype, i, wv);
      load8(res, ATOM_F32, i, rv);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        v[k][e] = rv[e] + v[k][e] * rd * wv[e];
        ss = fmaf(v[k][e], v[k][e], ss);
      }
      if (!rows) {
        *reinterpret_cast<float4*>(res + i) = make_float4(v[k][0], v[k][1], v[k][2], v[k][3]);
        *reinterpret_cast<float4*>(res + i + 4) = make_float4(v[k][4], v[k][5], v[k][6], v[k][7]);
      }
    }
  }
  ss = block_sum(ss, scratch);
  const float rstd = rsqrtf(ss / (float)H + eps);
  __nv_bfloat16* o = out + (int64_t)r * H;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = (threadIdx.x + k * blockDim.x) * 8;
    if (i < H) {
      float wv[8];
      load8(w, w_dtype, i, wv);
      uint4 q;
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
      for (int e = 0; e < 4; ++e)
        h[e] = __floats2bfloat162_rn(v[k][2 * e] * rstd * wv[2 * e], v[k][2 * e + 1] * rstd * wv[2 * e + 1]);
      *reinterpret_cast<uint4*>(o + i) = q;
    }
  }
}

}  // namespace atom

// wd and w have one type (w_dtype).
ATOM_EXPORT int atom_normed_add_rmsnorm(void* out, int act_dtype, float* residual, const void* delta, const void* wd,
                                        float eps_d, const void* w, int w_dtype, float eps, const int* rows, int n_rows,
                                        int H, cudaStream_t stream) {
  if (n_rows <= 0) return ATOM_OK;
  if (H <= 0 || H > 48 * 256 || !delta || !wd || (w_dtype != ATOM_F32 && w_dtype != ATOM_BF16)) return ATOM_ERR_ARG;
  const int threads = atom::norm_threads(H);
  const size_t smem = sizeof(float) * (size_t)H;
  const bool aligned = ((uintptr_t)out % 16 == 0) && ((uintptr_t)residual % 16 == 0) && ((uintptr_t)delta % 16 == 0) &&
                       ((uintptr_t)w % 16 == 0) && ((uintptr_t)wd % 16 == 0);
  if (act_dtype == ATOM_BF16 && H % 8 == 0 && H <= 8 * 2 * 1024 && aligned) {
    const int vecs = H / 8;
    int nv = 1, th = ((vecs + 31) / 32) * 32;
    if (th > 1024) {
      nv = 2;
      th = (((vecs + 1) / 2 + 31) / 32) * 32;
    }
    if (th < 64) th = 64;
    if (nv == 1)
      atom::launch_pdl(atom::normed_add_rmsnorm_bf16_vec_kernel<1>, dim3(n_rows), dim3(th), 0, stream, (__nv_bfloat16*)out,
                       residual, (const __nv_bfloat16*)delta, wd, eps_d, w, w_dtype, eps, rows, H);
    else
      atom::launch_pdl(atom::normed_add_rmsnorm_bf16_vec_kernel<2>, dim3(n_rows), dim3(th), 0, stream, (__nv_bfloat16*)out,
                       residual, (const __nv_bfloat16*)delta, wd, eps_d, w, w_dtype, eps, rows, H);
    return atom::check_launch();
  }
  if (act_dtype == ATOM_F32)
    atom::launch_pdl(atom::normed_add_rmsnorm_kernel<float>, dim3(n_rows), dim3(threads), smem, stream, (float*)out,
                     residual, (const float*)delta, wd, eps_d, w, w_dtype, eps, rows, H);
  else if (act_dtype == ATOM_BF16)
    atom::launch_pdl(atom::normed_add_rmsnorm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), smem, stream,
                     (__nv_bfloat16*)out, residual, (const __nv_bfloat16*)delta, wd, eps_d, w, w_dtype, eps, rows, H);
  else
    return ATOM_ERR_ARG;
  return atom::check_launch();
}
