// Causal paged attention with capped scores and a sliding window that keeps a request's first tokens
// (the formulas stand in window_attention.cu), in bfloat16 on the tensor cores, compiled for one pair of sizes:
//   -DATOM_WA_DK (key size) -DATOM_WA_DV (value size), both multiples of 16.
//
// A CTA of 4 warps takes a tile of up to 64 consecutive tokens of one request and one query head (a warp 16 rows)
// and walks the keys it can see in tiles of 64: first the tiles of the kept first tokens that lie before the window,
// then the window's.  Keys and values of a tile come into shared memory with cp.async, the next tile under way
// while this one is used.  S = Q K^T on mma.sync m16n8k16 with 32-bit sums; scale, cap (cap * tanh(s / cap)), the
// mask by positions, the running maximum and sum per row stay in 32-bit registers (a row's numbers sit in the four
// lanes of a quad); the weights exp(s - m) enter the product with the values as TWO bfloat16 numbers, p = hi + lo,
// so that the product sees 16 bits of their mantissa; the 16 x DV output of a warp stays in registers over all tiles.
// With few tokens in the step the key tiles of a unit are shared out among `nsplit` CTAs, which leave maximum, sum
// and unnormalised output per (token, head) in a scratch array that window_attention.cu's merge kernel puts together.
// In a step of single tokens a CTA's rows are the query heads that share one key head, so a request's keys and values
// are read once per key head.
#include "common.cuh"

#if !defined(ATOM_WA_DK) || !defined(ATOM_WA_DV)
#error "compile with -DATOM_WA_DK= -DATOM_WA_DV="
#endif

namespace atom {
namespace watc {

constexpr int DK = ATOM_WA_DK, DV = ATOM_WA_DV;
constexpr int BM = 64, BN = 64, WARPS = 4, THREADS = WARPS * 32;
constexpr int LDK = DK + 8, LDV = DV + 8;                 // bf16 elements per row in shared memory (16 bytes of padding)
static_assert(DK % 16 == 0 && DV % 16 == 0 && DK <= 256 && DV <= 128, "sizes");

constexpr size_t kSmemBytes = sizeof(__nv_bfloat16) * ((size_t)BM * LDK + 2 * ((size_t)BN * LDK + (size_t)BN * LDV));

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 16 bytes global -> shared without passing through registers; !valid: 16 zero bytes, nothing is read.
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ uint32_t pack_bf16(__nv_bfloat16 a, __nv_bfloat16 b) {
  return (uint32_t)__bfloat16_as_ushort(a) | ((uint32_t)__bfloat16_as_ushort(b) << 16);
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
constexpr float kLog2e = 1.4426950408889634f, kLn2 = 0.6931471805599453f;
// tanh(x) = 1 - 2 / (exp(2x) + 1): absolute error of a few 1e-7, exact limits at both ends.
__device__ __forceinline__ float tanh_fast(float x) { return 1.f - __fdividef(2.f, ex2(x * (2.f * kLog2e)) + 1.f); }

// Finds request s and tile r of unit x: requests take ceil(rows / BM) units one after another.
__device__ __forceinline__ bool find_tile(int x, const int* __restrict__ cu_q, int num_seqs, int& s, int& r) {
  int acc = 0;
  for (s = 0; s < num_seqs; ++s) {
    const int n = (cu_q[s + 1] - cu_q[s] + BM - 1) / BM;
    if (x < acc + n) {
      r = n - 1 - (x - acc);          // a request's last tiles see the most keys: they start first
      return true;
    }
    acc += n;
  }
  return false;
}

struct Params {
  __nv_bfloat16* out;
  const __nv_bfloat16* q;
  int64_t q_stride;
  const __nv_bfloat16* k_pages;
  const __nv_bfloat16* v_pages;
  const int* block_table;
  int max_pages, page_size;
  int64_t num_pages;
  const int* positions;
  const int* seq_of_token;
  const int* cu_q;
  int num_seqs, nh, nkv;
  float scale, cap;
  int window, keep;
  int nsplit;
  float* part;
};

// Two threads per key row: the page is looked up once per row and tile, the row's 16-byte pieces alternate between them.
__device__ __forceinline__ void load_kv_tile(__nv_bfloat16* Ks, __nv_bfloat16* Vs, const Params& p, const int* bt, int g,
                                             int j0, int p_last) {
  constexpr int KC = DK / 8, VC = DV / 8;
  static_assert(THREADS == 2 * BN, "two threads per key row");
  const int r = threadIdx.x >> 1, half = threadIdx.x & 1;
  const int j = j0 + r;
  int page = -1;
  if (j <= p_last) {
    const int lp = j / p.page_size;
    if (lp < p.max_pages) page = bt[lp];
  }
  const bool valid = page >= 0 && page < p.num_pages;
  const int64_t row = valid ? ((int64_t)page * p.nkv + g) * p.page_size + (j % p.page_size) : 0;
  const __nv_bfloat16* ksrc = p.k_pages + row * DK;
  const __nv_bfloat16* vsrc = p.v_pages + row * DV;
#pragma unroll
  for (int c = 0; c < KC / 2; ++c) cp_async16(Ks + r * LDK + (2 * c + half) * 8, ksrc + (2 * c + half) * 8, valid);
#pragma unroll
  for (int c = 0; c < VC / 2; ++c) cp_async16(Vs + r * LDV + (2 * c + half) * 8, vsrc + (2 * c + half) * 8, valid);
}

// HEADS: a step of single tokens.  A CTA's rows are the query heads of ONE key head for one token (they share the
// keys and values, which are then read once for the group), blockIdx = (token, key head, share).
template <bool HEADS>
__global__ void __launch_bounds__(THREADS, 2) window_attention_tc_kernel(const Params p) {
  atom::pdl_trigger();
  atom::pdl_wait();
  extern __shared__ __align__(16) unsigned char wa_smem[];
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(wa_smem);
  __nv_bfloat16* KVs = Qs + BM * LDK;                          // two stages of [K tile | V tile]
  constexpr int STAGE = BN * LDK + BN * LDV;

  int s, r, h, g, t0, rows;
  const int z = blockIdx.z;
  if (HEADS) {
    t0 = blockIdx.x;
    s = p.seq_of_token[t0];
    if (s < 0) return;
    g = blockIdx.y;
    rows = p.nh / p.nkv;
    h = g * rows;                                               // the group's first head; row r is head h + r
  } else {
    if (!find_tile(blockIdx.x, p.cu_q, p.num_seqs, s, r)) return;
    h = blockIdx.y;
    g = h / (p.nh / p.nkv);
    t0 = p.cu_q[s] + r * BM;
    rows = min(BM, p.cu_q[s + 1] - t0);
  }
  const int p0 = p.positions[t0];
  const int p_last = HEADS ? p0 : p0 + rows - 1;
  const int* bt = p.block_table + (int64_t)s * p.max_pages;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // key tiles: the kept first tokens' that lie before the window's first tile, then the window's
  const int lo = p.window > 0 ? max(0, p0 - p.window + 1) : 0;
  const int jt_lo = lo / BN, n_tiles = p_last / BN + 1;
  const int nk = p.window > 0 ? min((p.keep + BN - 1) / BN, jt_lo) : 0;
  const int n = nk + n_tiles - jt_lo;
  const int per = (n + p.nsplit - 1) / p.nsplit;
  const int i_begin = z * per, i_end = min(n, i_begin + per);
  auto tile_of = [&](int i) { return i < nk ? i : jt_lo + (i - nk); };

  // the queries of the tile, and the first key tile
  constexpr int KC = DK / 8;
  for (int idx = threadIdx.x; idx < BM * KC; idx += THREADS) {
    const int rr = idx / KC, c = idx - rr * KC;
    const bool valid = rr < rows;
    const int qt = HEADS ? t0 : t0 + (valid ? rr : 0), qh = HEADS ? h + (valid ? rr : 0) : h;
    cp_async16(Qs + rr * LDK + c * 8, p.q + (int64_t)qt * p.q_stride + (int64_t)qh * DK + c * 8, valid);
  }
  if (i_begin < i_end) load_kv_tile(KVs, KVs + BN * LDK, p, bt, g, tile_of(i_begin) * BN, p_last);
  cp_async_commit();

  float o[DV / 8][4];
#pragma unroll
  for (int i = 0; i < DV / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const bool active = warp * 16 < rows;                        // a warp without rows only helps to load
  const int row_a = warp * 16 + (lane >> 2), row_b = row_a + 8;
  // with a cap: score = cap2 * tanh(sum * in_mul); without: sum * in_mul; both in units of log 2
  const float in_mul = p.cap > 0.f ? p.scale / p.cap : p.scale * kLog2e;
  const float cap2 = p.cap * kLog2e;

  for (int i = i_begin; i < i_end; ++i) {
    const int stage = (i - i_begin) & 1;
    __nv_bfloat16* Ks = KVs + stage * STAGE;
    __nv_bfloat16* Vs = Ks + BN * LDK;
    if (i + 1 < i_end) {
      __nv_bfloat16* Kn = KVs + (stage ^ 1) * STAGE;
      load_kv_tile(Kn, Kn + BN * LDK, p, bt, g, tile_of(i + 1) * BN, p_last);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (active) {
      const int j0 = tile_of(i) * BN;
      float sc[BN / 8][4];
#pragma unroll
      for (int nt = 0; nt < BN / 8; ++nt) sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < DK / 16; ++kk) {
        uint32_t a[4];
        ldmatrix_x4(a, Qs + (warp * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * LDK + kk * 16 + (lane >> 4) * 8);
#pragma unroll
        for (int np = 0; np < BN / 16; ++np) {
          uint32_t b[4];
          ldmatrix_x4(b, Ks + (np * 16 + (lane >> 4) * 8 + (lane & 7)) * LDK + kk * 16 + ((lane >> 3) & 1) * 8);
          mma_bf16(sc[2 * np], a, b[0], b[1]);
          mma_bf16(sc[2 * np + 1], a, b[2], b[3]);
        }
      }
      // scale and cap, in units of log 2 (the weights are powers of two of score differences); the mask, which only
      // tiles at an edge need (the diagonal, the window's far end, the end of the kept tokens, a tile of few rows);
      // the tile's maximum per row
      const bool interior = !HEADS && rows == BM && j0 + BN - 1 <= p0 &&
                            (p.window <= 0 || p_last - j0 < p.window || j0 + BN <= p.keep);
#pragma unroll
      for (int nt = 0; nt < BN / 8; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          sc[nt][e] = p.cap > 0.f ? cap2 * tanh_fast(sc[nt][e] * in_mul) : sc[nt][e] * in_mul;
      }
      if (!interior) {
#pragma unroll
        for (int nt = 0; nt < BN / 8; ++nt) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int j = j0 + nt * 8 + (lane & 3) * 2 + (e & 1);
            const int row = (e < 2) ? row_a : row_b;
            const int pi = HEADS ? p0 : p0 + row;
            const bool seen = row < rows && j <= pi && (p.window <= 0 || pi - j < p.window || j < p.keep);
            if (!seen) sc[nt][e] = -INFINITY;
          }
        }
      }
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nt = 0; nt < BN / 8; ++nt) {
        mx[0] = fmaxf(mx[0], fmaxf(sc[nt][0], sc[nt][1]));
        mx[1] = fmaxf(mx[1], fmaxf(sc[nt][2], sc[nt][3]));
      }
      float corr[2], m_use[2];
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        mx[k] = fmaxf(mx[k], __shfl_xor_sync(0xffffffffu, mx[k], 1));
        mx[k] = fmaxf(mx[k], __shfl_xor_sync(0xffffffffu, mx[k], 2));
        const float m_new = fmaxf(m_run[k], mx[k]);
        m_use[k] = (m_new == -INFINITY) ? 0.f : m_new;
        corr[k] = (m_run[k] == -INFINITY) ? 0.f : ex2(m_run[k] - m_use[k]);
        m_run[k] = m_new;
      }
      float sum[2] = {0.f, 0.f};
      uint32_t phi[BN / 16][4], plo[BN / 16][4];
#pragma unroll
      for (int nt = 0; nt < BN / 8; ++nt) {
        __nv_bfloat16 hi[4], lw[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float pe = ex2(sc[nt][e] - m_use[e >> 1]);           // 2^(-inf) = 0 for what is not seen
          sum[e >> 1] += pe;
          hi[e] = __float2bfloat16_rn(pe);
          lw[e] = __float2bfloat16_rn(pe - __bfloat162float(hi[e]));
        }
        const int ks = nt >> 1, half = (nt & 1) * 2;
        phi[ks][half] = pack_bf16(hi[0], hi[1]);
        phi[ks][half + 1] = pack_bf16(hi[2], hi[3]);
        plo[ks][half] = pack_bf16(lw[0], lw[1]);
        plo[ks][half + 1] = pack_bf16(lw[2], lw[3]);
      }
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        sum[k] += __shfl_xor_sync(0xffffffffu, sum[k], 1);
        sum[k] += __shfl_xor_sync(0xffffffffu, sum[k], 2);
        l_run[k] = l_run[k] * corr[k] + sum[k];
      }
#pragma unroll
      for (int nt = 0; nt < DV / 8; ++nt) {
        o[nt][0] *= corr[0];
        o[nt][1] *= corr[0];
        o[nt][2] *= corr[1];
        o[nt][3] *= corr[1];
      }
#pragma unroll
      for (int ks = 0; ks < BN / 16; ++ks) {
#pragma unroll
        for (int np = 0; np < DV / 16; ++np) {
          uint32_t b[4];
          ldmatrix_x4_trans(b, Vs + (ks * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * LDV + np * 16 + (lane >> 4) * 8);
          mma_bf16(o[2 * np], phi[ks], b[0], b[1]);
          mma_bf16(o[2 * np + 1], phi[ks], b[2], b[3]);
          mma_bf16(o[2 * np], plo[ks], b[0], b[1]);
          mma_bf16(o[2 * np + 1], plo[ks], b[2], b[3]);
        }
      }
    }
    __syncthreads();                                            // the stage is free for the tile after the next
  }
  if (i_begin >= i_end) cp_async_wait<0>();
  if (!active) return;

  const int col = (lane & 3) * 2;
  if (p.nsplit == 1) {
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int row = k ? row_b : row_a;
      if (row >= rows) continue;
      const float inv = l_run[k] > 0.f ? 1.f / l_run[k] : 0.f;
      __nv_bfloat16* dst = p.out + (int64_t)(HEADS ? t0 : t0 + row) * p.nh * DV + (int64_t)(HEADS ? h + row : h) * DV;
#pragma unroll
      for (int nt = 0; nt < DV / 8; ++nt)
        *reinterpret_cast<__nv_bfloat162*>(dst + nt * 8 + col) =
            __floats2bfloat162_rn(o[nt][2 * k] * inv, o[nt][2 * k + 1] * inv);
    }
  } else {
    const int stride = p.nh * DV + 2 * p.nh;
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int row = k ? row_b : row_a;
      if (row >= rows) continue;
      float* dst = p.part + ((int64_t)(HEADS ? t0 : t0 + row) * p.nsplit + z) * stride;
      const int hh = HEADS ? h + row : h;
      if ((lane & 3) == 0) {
        dst[hh] = m_run[k] * kLn2;                               // the merge kernel takes natural logarithms
        dst[p.nh + hh] = l_run[k];
      }
      float* od = dst + 2 * p.nh + (int64_t)hh * DV;
#pragma unroll
      for (int nt = 0; nt < DV / 8; ++nt)
        *reinterpret_cast<float2*>(od + nt * 8 + col) = make_float2(o[nt][2 * k], o[nt][2 * k + 1]);
    }
  }
}

}  // namespace watc
}  // namespace atom

ATOM_EXPORT void atom_watc_sizes(int* dk, int* dv) {
  *dk = atom::watc::DK;
  *dv = atom::watc::DV;
}

// out [T, nh * DV]; q: row t at q + t * q_stride, heads packed [nh, DK]; k_pages [pages, nkv, page, DK]; v_pages
// [pages, nkv, page, DV]; units: an upper bound of the step's tiles (ceil(T / 64) + num_seqs), or with heads_rows (a
// step of single tokens: a CTA's rows are the query heads of one key head) the step's tokens.  nsplit > 1: part holds
// T * nsplit * nh * (DV + 2) floats, which attention_mixed.cu's merge kernel puts together.
ATOM_EXPORT int atom_window_attention_tc(void* out, const void* q, int64_t q_stride, const void* k_pages,
                                         const void* v_pages, int64_t num_pages, const int* block_table, int max_pages,
                                         int page_size, const int* positions, const int* seq_of_token, const int* cu_q,
                                         int num_seqs, int units, int nh, int nkv, float scale, float cap, int window,
                                         int keep, int nsplit, float* part, int heads_rows, cudaStream_t stream) {
  using namespace atom::watc;
  if (units <= 0) return ATOM_OK;
  if (nh <= 0 || nkv <= 0 || nh % nkv || page_size <= 0 || nsplit < 1 || nsplit > 65535 || nh > 65535 ||
      (nsplit > 1 && part == nullptr) || (q_stride % 8) != 0 || (heads_rows && nh / nkv > BM))
    return ATOM_ERR_ARG;
  Params p;
  p.out = (__nv_bfloat16*)out;
  p.q = (const __nv_bfloat16*)q;
  p.q_stride = q_stride;
  p.k_pages = (const __nv_bfloat16*)k_pages;
  p.v_pages = (const __nv_bfloat16*)v_pages;
  p.block_table = block_table;
  p.max_pages = max_pages;
  p.page_size = page_size;
  p.num_pages = num_pages;
  p.positions = positions;
  p.seq_of_token = seq_of_token;
  p.cu_q = cu_q;
  p.num_seqs = num_seqs;
  p.nh = nh;
  p.nkv = nkv;
  p.scale = scale;
  p.cap = cap;
  p.window = window;
  p.keep = window > 0 ? keep : 0;
  p.nsplit = nsplit;
  p.part = part;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(window_attention_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)kSmemBytes) != cudaSuccess ||
        cudaFuncSetAttribute(window_attention_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)kSmemBytes) != cudaSuccess)
      return ATOM_ERR_LAUNCH;
    attr_set = true;
  }
  if (heads_rows)      // units: the step's tokens
    atom::launch_pdl(window_attention_tc_kernel<true>, dim3(units, nkv, nsplit), dim3(THREADS), kSmemBytes, stream, p);
  else
    atom::launch_pdl(window_attention_tc_kernel<false>, dim3(units, nh, nsplit), dim3(THREADS), kSmemBytes, stream, p);
  return atom::check_launch();
}
