// Routed experts: every row goes to the `top` experts with the largest router scores.
//
//   moe_route_kernel    per row (a warp): score = sigmoid(logit) or softmax over the experts, the top experts by
//                       score (ties: the lower index), their weights (optionally divided by their sum), and the
//                       experts' row counts
//   moe_place_kernel    one CTA: the experts' first rows (a running sum of the counts) and a place for every
//                       (row, choice) pair among its expert's rows; the counts go back to zero
//   moe_gemm_kernel     out[r] = A[r] W_e^T for the rows r of every expert e, tile by tile.  A[r] is either a dense
//                       row or weight_r * x[token_r] (the weight on the expert's INPUT); with GATED, W_e is
//                       [gate ; up] and the output is silu(gate) * up.  32-bit sums, each output summed over k in
//                       order, so a row's result does not depend on the rows beside it; in bfloat16 on the tensor
//                       cores (moe_gemm_tc_kernel), in 32-bit and for odd sizes with plain FMAs
//   moe_combine_kernel  out[t] = sum over t's choices of (weight *) y[place] (+ sigmoid(gate logit_t) * shared[t])
#include "common.cuh"

namespace atom {

// logits [T, ld] float32.  ids, wts [T, top]; counts [E] (zero on entry).
__global__ void moe_route_kernel(const float* __restrict__ logits, int64_t ld, int E, int top, int softmax_scores,
                                 int renormalize, const int* __restrict__ seq_of_token, int T, int* __restrict__ ids,
                                 float* __restrict__ wts, int* __restrict__ counts) {
  atom::pdl_trigger();
  atom::pdl_wait();
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  if (seq_of_token[t] < 0) {
    for (int k = lane; k < top; k += 32) ids[(int64_t)t * top + k] = -1;
    return;
  }
  const float* z = logits + (int64_t)t * ld;
  float zmax = -INFINITY, denom = 1.f;
  if (softmax_scores) {
    for (int e = lane; e < E; e += 32) zmax = fmaxf(zmax, z[e]);
    zmax = warp_max(zmax);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) sum += expf(z[e] - zmax);
    denom = warp_sum(sum);
  }
  uint32_t taken = 0;                       // bit m: expert lane + 32 m has been chosen (E <= 1024)
  float wsum = 0.f, mine = 0.f;             // lane k keeps the weight of choice k (top <= 32)
  int mine_id = -1;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
    for (int e = lane, m = 0; e < E; e += 32, ++m) {
      if ((taken >> m) & 1u) continue;
      const float v = z[e];
      if (v > best) {               // ascending e: the lower index wins a tie
        best = v;
        best_e = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) {
        best = ob;
        best_e = oe;
      }
    }
    if ((best_e & 31) == lane) taken |= 1u << (best_e >> 5);
    const float w = softmax_scores ? expf(best - zmax) / denom : 1.f / (1.f + expf(-best));
    wsum += w;
    if (lane == k) {
      mine = w;
      mine_id = best_e;
    }
  }
  if (lane < top) {
    ids[(int64_t)t * top + lane] = mine_id;
    wts[(int64_t)t * top + lane] = renormalize ? mine / wsum : mine;
    atomicAdd(&counts[mine_id], 1);
  }
}

// offsets [E + 1]; row_token, row_w [pairs]; pair_pos [pairs] (-1: a padding row's pair).
__global__ void __launch_bounds__(1024)
moe_place_kernel(const int* __restrict__ ids, const float* __restrict__ wts, int pairs, int top, int E,
                 int* __restrict__ counts, int* __restrict__ offsets, int* __restrict__ row_token,
                 float* __restrict__ row_w, int* __restrict__ pair_pos) {
  atom::pdl_trigger();
  atom::pdl_wait();
  __shared__ int first[1025];
  __shared__ int cursor[1024];
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < E; ++e) {
      first[e] = acc;
      acc += counts[e];
    }
    first[E] = acc;
  }
  for (int e = threadIdx.x; e < E; e += blockDim.x) cursor[e] = 0;
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) offsets[e] = first[e];
  for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int e = ids[i];
    if (e < 0) {
      pair_pos[i] = -1;
      continue;
    }
    const int pos = first[e] + atomicAdd(&cursor[e], 1);
    row_token[pos] = i / top;
    row_w[pos] = wts[i];
    pair_pos[i] = pos;
  }
}

constexpr int kMoeBM = 32, kMoeBN = 32, kMoeBK = 32;

// Finds the expert and the first row of row tile x: expert e takes ceil(rows_e / BM) tiles, one after another.
__device__ __forceinline__ bool moe_find_tile(int x, const int* __restrict__ offsets, int E, int bm, int& e, int& row0,
                                              int& rows) {
  int acc = 0;
  for (e = 0; e < E; ++e) {
    const int n = offsets[e + 1] - offsets[e];
    const int tiles = (n + bm - 1) / bm;
    if (x < acc + tiles) {
      row0 = offsets[e] + (x - acc) * bm;
      rows = min(bm, offsets[e + 1] - row0);
      return true;
    }
    acc += tiles;
  }
  return false;
}

// A: GATHER: x [T, K] rows (stride lda) picked by row_token and multiplied by row_w; else dense rows [R, K] (stride lda).
// W: [E, N (2 N if GATED), K].  out [R, N] dense.
template <typename T, bool GATED, bool GATHER>
__global__ void __launch_bounds__(256)
moe_gemm_kernel(T* __restrict__ out, const T* __restrict__ A, int64_t lda, const T* __restrict__ W,
                const int* __restrict__ offsets, const int* __restrict__ row_token, const float* __restrict__ row_w,
                int E, int N, int K) {
  atom::pdl_trigger();
  atom::pdl_wait();
  __shared__ float As[kMoeBK][kMoeBM + 1];
  __shared__ float Wg[kMoeBK][kMoeBN + 1];
  __shared__ float Wu[GATED ? kMoeBK : 1][kMoeBN + 1];
  __shared__ int64_t a_row[kMoeBM];
  __shared__ float a_mul[kMoeBM];
  int e, row0, rows;
  if (!moe_find_tile(blockIdx.x, offsets, E, kMoeBM, e, row0, rows)) return;
  const int n0 = blockIdx.y * kMoeBN;
  const T* We = W + (int64_t)e * (GATED ? 2 : 1) * N * K;
  if (threadIdx.x < kMoeBM) {
    const int r = threadIdx.x;
    if (r < rows) {
      a_row[r] = (GATHER ? (int64_t)row_token[row0 + r] : (int64_t)(row0 + r)) * lda;
      a_mul[r] = GATHER ? row_w[row0 + r] : 1.f;
    } else {
      a_row[r] = -1;
      a_mul[r] = 0.f;
    }
  }
  __syncthreads();
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;      // outputs (ty, ty + 16) x (tx, tx + 16)
  float g00 = 0.f, g01 = 0.f, g10 = 0.f, g11 = 0.f, u00 = 0.f, u01 = 0.f, u10 = 0.f, u11 = 0.f;
  for (int k0 = 0; k0 < K; k0 += kMoeBK) {
    for (int idx = threadIdx.x; idx < kMoeBM * kMoeBK; idx += 256) {
      const int r = idx / kMoeBK, kk = idx - r * kMoeBK;
      float v = 0.f;
      if (a_row[r] >= 0 && k0 + kk < K) {
        v = to_float(A[a_row[r] + k0 + kk]);
        // the weighted row is rounded to the activation type, as a row that a kernel of its own had written
        if (GATHER) v = to_float(from_float<T>(v * a_mul[r]));
      }
      As[kk][r] = v;
    }
    for (int idx = threadIdx.x; idx < kMoeBN * kMoeBK; idx += 256) {
      const int n = idx / kMoeBK, kk = idx - n * kMoeBK;
      const bool in = n0 + n < N && k0 + kk < K;
      Wg[kk][n] = in ? to_float(We[(int64_t)(n0 + n) * K + k0 + kk]) : 0.f;
      if (GATED) Wu[kk][n] = in ? to_float(We[(int64_t)(N + n0 + n) * K + k0 + kk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kMoeBK; ++kk) {
      const float a0 = As[kk][ty], a1 = As[kk][ty + 16];
      const float w0 = Wg[kk][tx], w1 = Wg[kk][tx + 16];
      g00 += a0 * w0;
      g01 += a0 * w1;
      g10 += a1 * w0;
      g11 += a1 * w1;
      if (GATED) {
        const float v0 = Wu[kk][tx], v1 = Wu[kk][tx + 16];
        u00 += a0 * v0;
        u01 += a0 * v1;
        u10 += a1 * v0;
        u11 += a1 * v1;
      }
    }
    __syncthreads();
  }
  auto put = [&](int r, int n, float g, float u) {
    if (r < rows && n0 + n < N) {
      float v = g;
      if (GATED) {
        // gate and up are rounded to the activation type first, as the unfused product hands them on
        const float gr = to_float(from_float<T>(g)), ur = to_float(from_float<T>(u));
        v = gr / (1.f + expf(-gr)) * ur;
      }
      out[(int64_t)(row0 + r) * N + n0 + n] = from_float<T>(v);
    }
  };
  put(ty, tx, g00, u00);
  put(ty, tx + 16, g01, u01);
  put(ty + 16, tx, g10, u10);
  put(ty + 16, tx + 16, g11, u11);
}

// y [R, n] expert outputs by place; shared [T, n] or null; gate: logits + gate_col, one per row (stride ld), or null.
template <typename T>
__global__ void moe_combine_kernel(T* __restrict__ out, const T* __restrict__ y, const int* __restrict__ pair_pos,
                                   const float* __restrict__ pair_w, int top, const T* __restrict__ shared_out,
                                   const float* __restrict__ gate, int64_t gate_ld, int n,
                                   const int* __restrict__ seq_of_token) {
  atom::pdl_trigger();
  atom::pdl_wait();
  const int t = blockIdx.x;
  if (seq_of_token[t] < 0) return;
  const float sg = (shared_out && gate) ? 1.f / (1.f + expf(-gate[(int64_t)t * gate_ld])) : 1.f;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < n; i += gridDim.y * blockDim.x) {
    float sum = 0.f;
    for (int k = 0; k < top; ++k) {
      const int pos = pair_pos[(int64_t)t * top + k];
      if (pos >= 0) sum += (pair_w ? pair_w[(int64_t)t * top + k] : 1.f) * to_float(y[(int64_t)pos * n + i]);
    }
    if (shared_out) sum += sg * to_float(shared_out[(int64_t)t * n + i]);
    out[(int64_t)t * n + i] = from_float<T>(sum);
  }
}

// ---- the same product in bfloat16 on the tensor cores -----------------------------------------------------------
// A CTA of 4 warps takes BM rows of one expert (64, or 16 in steps of few rows, where the warps share out the
// columns instead of the rows) and 64 output columns (with GATED the 64 gate rows and the 64 up rows of W_e), and
// walks K in steps of 32, three steps deep (of 64, four deep, with 16 rows: an expert's few rows stream its whole
// matrix, so the bytes in flight count): tiles of A and W_e come into shared memory with cp.async (gathered rows
// pass through registers, where they are weighted and rounded); mma.sync m16n8k16 with 32-bit sums.  Every output is
// summed over k in the same order whatever the tile, so a row's result does not depend on the rows beside it.
constexpr int kTcBN = 64, kTcThreads = 128;

__device__ __forceinline__ void moe_ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void moe_mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void moe_cp_async16(void* smem, const void* gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(n));
}

constexpr size_t moe_tc_smem(int bm, bool gated, int bk, int stages) {
  return sizeof(__nv_bfloat16) * stages * ((size_t)bm + (gated ? 2 : 1) * kTcBN) * (bk + 8);
}

template <bool GATED, bool GATHER, int BM, int MI, int kTcBK, int kTcStages>
__global__ void __launch_bounds__(kTcThreads)
moe_gemm_tc_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ A, int64_t lda,
                   const __nv_bfloat16* __restrict__ W, const int* __restrict__ offsets,
                   const int* __restrict__ row_token, const float* __restrict__ row_w, int E, int N, int K) {
  atom::pdl_trigger();
  atom::pdl_wait();
  constexpr int kTcLD = kTcBK + 8;                         // bf16 elements per row in shared memory
  constexpr int WM = BM / (16 * MI), WN = 4 / WM;          // warps along the rows (MI tiles of 16 rows each) and the columns
  constexpr int NT = kTcBN / WN / 8;                        // 8-column tiles of a warp
  constexpr int BROWS = (GATED ? 2 : 1) * kTcBN;
  constexpr int STAGE = (BM + BROWS) * kTcLD;
  extern __shared__ __align__(16) unsigned char moe_smem[];
  __nv_bfloat16* sm = reinterpret_cast<__nv_bfloat16*>(moe_smem);
  __shared__ int64_t a_row[BM];
  __shared__ float a_mul[BM];
  int e, row0, rows;
  if (!moe_find_tile(blockIdx.x, offsets, E, BM, e, row0, rows)) return;
  const int n0 = blockIdx.y * kTcBN;
  const __nv_bfloat16* We = W + (int64_t)e * (GATED ? 2 : 1) * N * K;
  if (threadIdx.x < BM) {
    const int r = threadIdx.x;
    if (r < rows) {
      a_row[r] = (GATHER ? (int64_t)row_token[row0 + r] : (int64_t)(row0 + r)) * lda;
      a_mul[r] = GATHER ? row_w[row0 + r] : 1.f;
    } else {
      a_row[r] = -1;
      a_mul[r] = 0.f;
    }
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wm = warp % WM, wn = warp / WM;

  auto load = [&](int stage, int k0) {
    __nv_bfloat16* As = sm + stage * STAGE;
    __nv_bfloat16* Bs = As + BM * kTcLD;
    constexpr int KC = kTcBK / 8;
    for (int idx = threadIdx.x; idx < BM * KC; idx += kTcThreads) {
      const int r = idx / KC, c = idx - r * KC;
      const bool valid = a_row[r] >= 0 && k0 + c * 8 < K;
      __nv_bfloat16* dst = As + r * kTcLD + c * 8;
      if (GATHER) {
        uint4 raw = make_uint4(0u, 0u, 0u, 0u);
        if (valid) {
          raw = *reinterpret_cast<const uint4*>(A + a_row[r] + k0 + c * 8);
          __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&raw);
          const float m = a_mul[r];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            // the weighted row is rounded to the activation type, as a row that a kernel of its own had written
            const float2 f = __bfloat1622float2(h2[i]);
            h2[i] = __floats2bfloat162_rn(f.x * m, f.y * m);
          }
        }
        *reinterpret_cast<uint4*>(dst) = raw;
      } else {
        moe_cp_async16(dst, A + (valid ? a_row[r] + k0 + c * 8 : 0), valid);
      }
    }
    for (int idx = threadIdx.x; idx < BROWS * KC; idx += kTcThreads) {
      const int r = idx / KC, c = idx - r * KC;
      const int n = n0 + (r % kTcBN);
      const bool valid = n < N && k0 + c * 8 < K;
      const int64_t wrow = (GATED && r >= kTcBN) ? (int64_t)N + n : (int64_t)n;
      moe_cp_async16(Bs + r * kTcLD + c * 8, We + (valid ? wrow * K + k0 + c * 8 : 0), valid);
    }
  };

  float g[MI][NT][4], u[MI][GATED ? NT : 1][4];
#pragma unroll
  for (int mi = 0; mi < MI; ++mi) {
#pragma unroll
    for (int i = 0; i < NT; ++i) g[mi][i][0] = g[mi][i][1] = g[mi][i][2] = g[mi][i][3] = 0.f;
#pragma unroll
    for (int i = 0; i < (GATED ? NT : 1); ++i) u[mi][i][0] = u[mi][i][1] = u[mi][i][2] = u[mi][i][3] = 0.f;
  }

  const int steps = (K + kTcBK - 1) / kTcBK;
#pragma unroll
  for (int s = 0; s < kTcStages - 1; ++s) {
    if (s < steps) load(s, s * kTcBK);
    asm volatile("cp.async.commit_group;\n" ::);
  }
  for (int it = 0; it < steps; ++it) {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(kTcStages - 2));
    __syncthreads();                                  // step `it` has landed, and the stage loaded below is free
    if (it + kTcStages - 1 < steps) load((it + kTcStages - 1) % kTcStages, (it + kTcStages - 1) * kTcBK);
    asm volatile("cp.async.commit_group;\n" ::);
    const __nv_bfloat16* As = sm + (it % kTcStages) * STAGE;
    const __nv_bfloat16* Bs = As + BM * kTcLD;
#pragma unroll
    for (int kk = 0; kk < kTcBK / 16; ++kk) {
      uint32_t a[MI][4];
#pragma unroll
      for (int mi = 0; mi < MI; ++mi)
        moe_ldmatrix_x4(a[mi], As + ((wm * MI + mi) * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * kTcLD + kk * 16 +
                                   (lane >> 4) * 8);
#pragma unroll
      for (int np = 0; np < NT / 2; ++np) {
        const int brow = wn * (kTcBN / WN) + np * 16 + (lane >> 4) * 8 + (lane & 7);
        uint32_t b[4];
        moe_ldmatrix_x4(b, Bs + brow * kTcLD + kk * 16 + ((lane >> 3) & 1) * 8);
#pragma unroll
        for (int mi = 0; mi < MI; ++mi) {
          moe_mma_bf16(g[mi][2 * np], a[mi], b[0], b[1]);
          moe_mma_bf16(g[mi][2 * np + 1], a[mi], b[2], b[3]);
        }
        if (GATED) {
          moe_ldmatrix_x4(b, Bs + (kTcBN + brow) * kTcLD + kk * 16 + ((lane >> 3) & 1) * 8);
#pragma unroll
          for (int mi = 0; mi < MI; ++mi) {
            moe_mma_bf16(u[mi][2 * np], a[mi], b[0], b[1]);
            moe_mma_bf16(u[mi][2 * np + 1], a[mi], b[2], b[3]);
          }
        }
      }
    }
  }
  asm volatile("cp.async.wait_group 0;\n" ::);
#pragma unroll
  for (int mi = 0; mi < MI; ++mi) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = (wm * MI + mi) * 16 + (lane >> 2) + (i >> 1) * 8;
        const int n = n0 + wn * (kTcBN / WN) + nt * 8 + (lane & 3) * 2 + (i & 1);
        if (r < rows && n < N) {
          float v = g[mi][nt][i];
          if (GATED) {
            // gate and up are rounded to the activation type first, as the unfused product hands them on
            const float gr = __bfloat162float(__float2bfloat16_rn(v));
            const float ur = __bfloat162float(__float2bfloat16_rn(u[mi][GATED ? nt : 0][i]));
            v = gr / (1.f + expf(-gr)) * ur;
          }
          out[(int64_t)(row0 + r) * N + n] = __float2bfloat16_rn(v);
        }
      }
    }
  }
}

template <bool GATED, bool GATHER, int BM, int MI, int BK, int STAGES>
static int moe_gemm_tc_launch_one(__nv_bfloat16* out, const __nv_bfloat16* A, int64_t lda, const __nv_bfloat16* W,
                                   const int* offsets, const int* row_token, const float* row_w, int R, int E, int N,
                                   int K, cudaStream_t stream) {
  dim3 grid((R + BM - 1) / BM + E, (N + kTcBN - 1) / kTcBN);
  constexpr size_t smem = moe_tc_smem(BM, GATED, BK, STAGES);
  if (smem > 48 * 1024) {
    static bool attr_set = false;
    if (!attr_set) {
      if (cudaFuncSetAttribute(moe_gemm_tc_kernel<GATED, GATHER, BM, MI, BK, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               (int)smem) != cudaSuccess)
        return ATOM_ERR_LAUNCH;
      attr_set = true;
    }
  }
  launch_pdl(moe_gemm_tc_kernel<GATED, GATHER, BM, MI, BK, STAGES>, grid, dim3(kTcThreads), smem, stream, out, A, lda, W, offsets,
             row_token, row_w, E, N, K);
  return ATOM_OK;
}

// Rows per tile: 16 while the step's rows are few (decoding: an expert gets a handful), else 64.  (Tiles of 128 rows,
// a warp 32 rows so that every piece of W_e read from shared memory serves two tiles of rows, were slower: 168
// registers a thread and 60 KB a CTA leave an SM too few warps.)
static int moe_gemm_tc_launch(__nv_bfloat16* out, const __nv_bfloat16* A, int64_t lda, const __nv_bfloat16* W,
                              const int* offsets, const int* row_token, const float* row_w, int R, int E, int N, int K,
                              int gated, int gather, cudaStream_t stream) {
  const bool small = R <= 16 * E;
  int rc = ATOM_OK;
#define ATOM_MOE_TC(G, H)                                                                                                 \
  do {                                                                                                                    \
    if (small) rc = moe_gemm_tc_launch_one<G, H, 16, 1, 64, 4>(out, A, lda, W, offsets, row_token, row_w, R, E, N, K, stream); \
    else rc = moe_gemm_tc_launch_one<G, H, 64, 1, 32, 3>(out, A, lda, W, offsets, row_token, row_w, R, E, N, K, stream);      \
  } while (0)
  if (gated && gather) ATOM_MOE_TC(true, true);
  else if (gated) ATOM_MOE_TC(true, false);
  else if (gather) ATOM_MOE_TC(false, true);
  else ATOM_MOE_TC(false, false);
#undef ATOM_MOE_TC
  if (rc != ATOM_OK) return rc;
  return check_launch();
}

template <typename T>
static int moe_gemm_launch(T* out, const T* A, int64_t lda, const T* W, const int* offsets, const int* row_token,
                           const float* row_w, int R, int E, int N, int K, int gated, int gather, cudaStream_t stream) {
  dim3 grid((R + kMoeBM - 1) / kMoeBM + E, (N + kMoeBN - 1) / kMoeBN);
#define ATOM_MOE(G, H) \
  launch_pdl(moe_gemm_kernel<T, G, H>, grid, dim3(256), 0, stream, out, A, lda, W, offsets, row_token, row_w, E, N, K)
  if (gated && gather) ATOM_MOE(true, true);
  else if (gated) ATOM_MOE(true, false);
  else if (gather) ATOM_MOE(false, true);
  else ATOM_MOE(false, false);
#undef ATOM_MOE
  return check_launch();
}

}  // namespace atom

ATOM_EXPORT int atom_moe_route(const float* logits, int64_t ld, int T, int E, int top, int softmax_scores,
                               int renormalize, const int* seq_of_token, int* ids, float* wts, int* counts,
                               cudaStream_t stream) {
  if (T <= 0) return ATOM_OK;
  if (E <= 0 || E > 1024 || top <= 0 || top > 32 || top > E) return ATOM_ERR_ARG;
  atom::launch_pdl(atom::moe_route_kernel, dim3((T + 3) / 4), dim3(128), 0, stream, logits, ld, E, top, softmax_scores,
                   renormalize, seq_of_token, T, ids, wts, counts);
  return atom::check_launch();
}

ATOM_EXPORT int atom_moe_place(const int* ids, const float* wts, int pairs, int top, int E, int* counts, int* offsets,
                               int* row_token, float* row_w, int* pair_pos, cudaStream_t stream) {
  if (pairs <= 0) return ATOM_OK;
  if (E <= 0 || E > 1024 || top <= 0) return ATOM_ERR_ARG;
  atom::launch_pdl(atom::moe_place_kernel, dim3(1), dim3(1024), 0, stream, ids, wts, pairs, top, E, counts, offsets,
                   row_token, row_w, pair_pos);
  return atom::check_launch();
}

// R: the most rows there can be (rows of the step x top); the kernel finds the real ones from `offsets`.
ATOM_EXPORT int atom_moe_gemm(void* out, const void* A, int dtype, int64_t lda, const void* W, const int* offsets,
                              const int* row_token, const float* row_w, int R, int E, int N, int K, int gated,
                              int gather, int tc, cudaStream_t stream) {
  if (R <= 0) return ATOM_OK;
  if (E <= 0 || N <= 0 || K <= 0 || (gather && (!row_token || !row_w))) return ATOM_ERR_ARG;
  if (dtype == ATOM_F32)
    return atom::moe_gemm_launch<float>((float*)out, (const float*)A, lda, (const float*)W, offsets, row_token, row_w,
                                        R, E, N, K, gated, gather, stream);
  if (dtype == ATOM_BF16 && tc && K % 8 == 0 && lda % 8 == 0 && ((uintptr_t)A % 16) == 0 && ((uintptr_t)W % 16) == 0)
    return atom::moe_gemm_tc_launch((__nv_bfloat16*)out, (const __nv_bfloat16*)A, lda, (const __nv_bfloat16*)W, offsets,
                                    row_token, row_w, R, E, N, K, gated, gather, stream);
  if (dtype == ATOM_BF16)
    return atom::moe_gemm_launch<__nv_bfloat16>((__nv_bfloat16*)out, (const __nv_bfloat16*)A, lda,
                                                (const __nv_bfloat16*)W, offsets, row_token, row_w, R, E, N, K, gated,
                                                gather, stream);
  return ATOM_ERR_ARG;
}

ATOM_EXPORT int atom_moe_combine(void* out, const void* y, int dtype, const int* pair_pos, const float* pair_w, int top,
                                 const void* shared_out, const float* gate, int64_t gate_ld, int T, int n,
                                 const int* seq_of_token, cudaStream_t stream) {
  if (T <= 0) return ATOM_OK;
  if (n <= 0 || top <= 0) return ATOM_ERR_ARG;
  // few rows: the columns are shared out among CTAs too (a row's sums are chains of dependent loads)
  const dim3 grid(T, T >= 512 ? 1 : (unsigned)min(8, (n + 255) / 256));
  if (dtype == ATOM_F32)
    atom::launch_pdl(atom::moe_combine_kernel<float>, grid, dim3(256), 0, stream, (float*)out, (const float*)y,
                     pair_pos, pair_w, top, (const float*)shared_out, gate, gate_ld, n, seq_of_token);
  else if (dtype == ATOM_BF16)
    atom::launch_pdl(atom::moe_combine_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, (__nv_bfloat16*)out,
                     (const __nv_bfloat16*)y, pair_pos, pair_w, top, (const __nv_bfloat16*)shared_out, gate, gate_ld, n,
                     seq_of_token);
  else
    return ATOM_ERR_ARG;
  return atom::check_launch();
}
