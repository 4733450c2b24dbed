// Activations of the feed-forwards.  SiLU-gated product: out[t, i] = silu(gu[t, i]) * gu[t, I + i],
// computed in 32-bit (silu(x) = x / (1 + exp(-x))).
#include "common.cuh"

namespace atom {

template <typename T>
__global__ void silu_mul_kernel(T* __restrict__ out, const T* __restrict__ gu, int64_t n, int I) {
  atom::pdl_trigger();   // the next kernel may be scheduled at once: before its own wait it reads nothing a kernel of this step writes
  atom::pdl_wait();      // inputs written by the kernel before this one are visible from here on
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += stride) {
    const int64_t t = idx / I;
    const int i = (int)(idx - t * I);
    const float g = to_float(gu[t * 2 * I + i]);
    const float u = to_float(gu[t * 2 * I + I + i]);
    out[idx] = from_float<T>(g / (1.f + expf(-g)) * u);
  }
}

// silu(x) = x / (1 + e^-x) = x * (0.5 + 0.5 * tanh(x / 2)): one special-function operation instead of two
// (the result is rounded to bfloat16, eight times coarser than tanh.approx's error).
__device__ __forceinline__ float silu_fast(float x) {
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * x));
  return x * fmaf(0.5f, t, 0.5f);
}

// bf16, I a multiple of 8: 16 bytes of gate and of up per thread.
__global__ void silu_mul_bf16_vec_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ gu,
                                         int64_t nvec, int I8) {
  atom::pdl_trigger();   // the next kernel may be scheduled at once: before its own wait it reads nothing a kernel of this step writes
  atom::pdl_wait();      // inputs written by the kernel before this one are visible from here on
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < nvec; idx += stride) {
    const int64_t t = idx / I8;
    const int i = (int)(idx - t * I8);
    const uint4 g4 = *reinterpret_cast<const uint4*>(gu + (t * 2 * I8 + i) * 8);
    const uint4 u4 = *reinterpret_cast<const uint4*>(gu + (t * 2 * I8 + I8 + i) * 8);
    const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&g4);
    const __nv_bfloat162* uh = reinterpret_cast<const __nv_bfloat162*>(&u4);
    uint4 o4;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 g = __bfloat1622float2(gh[e]), u = __bfloat1622float2(uh[e]);
      oh[e] = __floats2bfloat162_rn(silu_fast(g.x) * u.x, silu_fast(g.y) * u.y);
    }
    *reinterpret_cast<uint4*>(out + idx * 8) = o4;
  }
}

// xIELU, an activation with two shape numbers (given here already passed through softplus, ap and aq):
//   z > 0:  ap * z^2 + z / 2;      z <= 0:  (1/2 + aq) * (exp(z) - 1 - z) + z / 2,
// computed in 32-bit.  expm1f keeps the small-|z| branch exact.
template <typename T>
__global__ void xielu_kernel(T* __restrict__ out, const T* __restrict__ x, int64_t n, float ap, float aq) {
  atom::pdl_trigger();
  atom::pdl_wait();
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += stride) {
    const float z = to_float(x[idx]);
    const float y = z > 0.f ? fmaf(ap * z, z, 0.5f * z) : fmaf(0.5f + aq, expm1f(z) - z, 0.5f * z);
    out[idx] = from_float<T>(y);
  }
}

// tanh in place, in 32-bit (the hidden layer of a low-rank projection).
template <typename T>
__global__ void tanh_kernel(T* __restrict__ x, int64_t n) {
  atom::pdl_trigger();
  atom::pdl_wait();
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += stride)
    x[idx] = from_float<T>(tanhf(to_float(x[idx])));
}

// relu(x)^2 in place.
template <typename T>
__global__ void relu2_kernel(T* __restrict__ x, int64_t n) {
  atom::pdl_trigger();
  atom::pdl_wait();
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += stride) {
    const float z = fmaxf(to_float(x[idx]), 0.f);
    x[idx] = from_float<T>(z * z);
  }
}

// bfloat16, eight numbers per load and store.
__global__ void relu2_bf16_vec_kernel(uint4* __restrict__ x, int64_t nvec) {
  atom::pdl_trigger();
  atom::pdl_wait();
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < nvec; idx += stride) {
    uint4 v = x[idx];
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __bfloat1622float2(h[i]);
      f.x = fmaxf(f.x, 0.f);
      f.y = fmaxf(f.y, 0.f);
      h[i] = __floats2bfloat162_rn(f.x * f.x, f.y * f.y);
    }
    x[idx] = v;
  }
}

}  // namespace atom

ATOM_EXPORT int atom_tanh(void* x, int dtype, int64_t n, cudaStream_t stream) {
  if (n <= 0) return ATOM_OK;
  int64_t blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (dtype == ATOM_F32)
    atom::launch_pdl(atom::tanh_kernel<float>, dim3((int)blocks), dim3(256), 0, stream, (float*)x, n);
  else if (dtype == ATOM_BF16)
    atom::launch_pdl(atom::tanh_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(256), 0, stream, (__nv_bfloat16*)x, n);
  else
    return ATOM_ERR_ARG;
  return atom::check_launch();
}

ATOM_EXPORT int atom_xielu(void* out, const void* x, int dtype, int64_t n, float ap, float aq, cudaStream_t stream) {
  if (n <= 0) return ATOM_OK;
  const int threads = 256;
  int64_t blocks = (n + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (dtype == ATOM_F32)
    atom::launch_pdl(atom::xielu_kernel<float>, dim3((int)blocks), dim3(threads), 0, stream, (float*)out, (const float*)x, n, ap, aq);
  else if (dtype == ATOM_BF16)
    atom::launch_pdl(atom::xielu_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(threads), 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)x, n, ap, aq);
  else
    return ATOM_ERR_ARG;
  return atom::check_launch();
}

ATOM_EXPORT int atom_silu_mul(void* out, const void* gu, int dtype, int T, int I,
                              cudaStream_t stream) {
  if (T <= 0) return ATOM_OK;
  if (I <= 0) return ATOM_ERR_ARG;
  const int64_t n = (int64_t)T * I;
  const int threads = 256;
  int64_t blocks = (n + threads - 1) / threads;
  if (dtype == ATOM_BF16 && I % 8 == 0 && (uintptr_t)out % 16 == 0 && (uintptr_t)gu % 16 == 0) {
    const int64_t nvec = n / 8;
    int64_t vb = (nvec + threads - 1) / threads;
    if (vb > 148 * 32) vb = 148 * 32;
    atom::launch_pdl(atom::silu_mul_bf16_vec_kernel, dim3((int)vb), dim3(threads), 0, stream, (__nv_bfloat16*)out,
                                                                    (const __nv_bfloat16*)gu, nvec, I / 8);
    return atom::check_launch();
  }
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (dtype == ATOM_F32) {
    atom::launch_pdl(atom::silu_mul_kernel<float>, dim3((int)blocks), dim3(threads), 0, stream, (float*)out, (const float*)gu, n, I);
  } else if (dtype == ATOM_BF16) {
    atom::launch_pdl(atom::silu_mul_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(threads), 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)gu, n, I);
  } else {
    return ATOM_ERR_ARG;
  }
  return atom::check_launch();
}

ATOM_EXPORT int atom_relu2(void* x, int dtype, int64_t n, cudaStream_t stream) {
  if (n <= 0) return ATOM_OK;
  const int threads = 256;
  if (dtype == ATOM_BF16 && n % 8 == 0 && (uintptr_t)x % 16 == 0) {
    int64_t vb = (n / 8 + threads - 1) / threads;
    if (vb > 148 * 32) vb = 148 * 32;
    atom::launch_pdl(atom::relu2_bf16_vec_kernel, dim3((int)vb), dim3(threads), 0, stream, (uint4*)x, n / 8);
    return atom::check_launch();
  }
  int64_t blocks = (n + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (dtype == ATOM_F32)
    atom::launch_pdl(atom::relu2_kernel<float>, dim3((int)blocks), dim3(threads), 0, stream, (float*)x, n);
  else if (dtype == ATOM_BF16)
    atom::launch_pdl(atom::relu2_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(threads), 0, stream, (__nv_bfloat16*)x, n);
  else
    return ATOM_ERR_ARG;
  return atom::check_launch();
}

// x[t, h, :] *= sigmoid(g[t, h]): one gate number per head.  x [T, H, n] dense; g rows ldg apart.
namespace atom {
template <typename T>
__global__ void head_gate_kernel(T* __restrict__ x, const T* __restrict__ g, int64_t ldg, int H, int n, int64_t total) {
  atom::pdl_trigger();
  atom::pdl_wait();
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
    const int64_t th = e / n;
    const int64_t t = th / H;
    const int h = (int)(th - t * H);
    const float z = to_float(g[t * ldg + h]);
    x[e] = from_float<T>(to_float(x[e]) / (1.f + expf(-z)));
  }
}
}  // namespace atom

ATOM_EXPORT int atom_head_gate(void* x, const void* g, int dtype, int64_t ldg, int T, int H, int n, cudaStream_t stream) {
  if (T <= 0) return ATOM_OK;
  if (H <= 0 || n <= 0) return ATOM_ERR_ARG;
  const int64_t total = (int64_t)T * H * n;
  const int blocks = (int)((total + 255) / 256 > 148 * 8 ? 148 * 8 : (total + 255) / 256);
  if (dtype == ATOM_F32)
    atom::launch_pdl(atom::head_gate_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)x, (const float*)g, ldg, H, n, total);
  else if (dtype == ATOM_BF16)
    atom::launch_pdl(atom::head_gate_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (__nv_bfloat16*)x,
                     (const __nv_bfloat16*)g, ldg, H, n, total);
  else
    return ATOM_ERR_ARG;
  return atom::check_launch();
}
