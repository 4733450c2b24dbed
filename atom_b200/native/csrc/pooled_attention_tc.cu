// Attention over a sliding window and pooled blocks before it (the formulas stand in pooled_attention.cu), in bfloat16
// on the tensor cores, compiled for one set of sizes:
//   -DATOM_PW_NH (query heads) -DATOM_PW_NKV (kv heads) -DATOM_PW_DK (key size) -DATOM_PW_DV (value size).
//
// A CTA of 16 warps takes a tile of 16 consecutive tokens of one request with ALL heads, because mixing the heads'
// weights needs every head's weight of a (query, key) pair at once.  Its keys are the pooled blocks that its last row
// sees, then the tokens from the first row's window on; it walks them in chunks of 64, twice:
//   first walk   per kv head: its 64 keys go to shared memory (cp.async, the next load under way while this one is
//                used); S_h = Q_h K^T for the heads of its group on mma.sync (m16n8k16, 32-bit sums) to shared memory
//                in 32-bit; warp r owns row r and keeps the running maximum and denominator per (head, row), with the
//                sink of score zero as the denominator's first term;
//   second walk  the scores again; warp r turns its row's scores into weights exp(s - m) / l, forms every head's mixed
//                weight as a 32-bit sum over heads and leaves it in shared memory as TWO bfloat16 numbers, w = hi + lo,
//                so that the product with the values sees 16 bits of its mantissa; per kv head: its 64 values go to
//                shared memory; O_h += (W_hi + W_lo) V on mma.sync.  The output tiles (head, 16 columns) of a kv head's
//                group are dealt out to the warps, which keep them in registers over all chunks.
// The weights are final when they are mixed, so nothing is rescaled and the result does not depend on how a request's
// tokens are cut into steps beyond the order of 32-bit sums.  The output gate is the epilogue.
#include "common.cuh"

#if !defined(ATOM_PW_NH) || !defined(ATOM_PW_NKV) || !defined(ATOM_PW_DK) || !defined(ATOM_PW_DV)
#error "compile with -DATOM_PW_NH= -DATOM_PW_NKV= -DATOM_PW_DK= -DATOM_PW_DV="
#endif

namespace atom {
namespace pwtc {

constexpr int NH = ATOM_PW_NH, NKV = ATOM_PW_NKV, DK = ATOM_PW_DK, DV = ATOM_PW_DV;
constexpr int GROUP = NH / NKV;
constexpr int BM = 16, BN = 64, WARPS = 16, THREADS = WARPS * 32;
constexpr int LDQ = DK + 8;                              // bf16 elements per row of Q in shared memory
constexpr int LDKV = (DK > DV ? DK : DV) + 8;            // ... of the keys' / values' buffer
constexpr int LDR = 72;                                  // floats per (head, row) of scores = 288 bytes,
                                                         // later 72 bf16 of W_hi and 72 bf16 of W_lo
constexpr int QK_UNITS = GROUP * (BN / 16);              // (head of the group, 16 keys) per kv head
constexpr int PV_UNITS = GROUP * (DV / 16);              // (head of the group, 16 value columns) per kv head
constexpr int TPG = (PV_UNITS + WARPS - 1) / WARPS;      // output tiles of a warp per kv head
static_assert(NH % NKV == 0 && DK % 16 == 0 && DV % 16 == 0, "sizes");
static_assert(NKV * TPG * 8 <= 64, "output tiles of a warp exceed its registers");
static_assert(NH <= 16, "at most 16 heads");

constexpr size_t smem_bytes() {
  return sizeof(__nv_bfloat16) * ((size_t)NH * BM * LDQ + (size_t)2 * BN * LDKV) + sizeof(float) * ((size_t)NH * BM * LDR) +
         sizeof(float) * (NH * NH) + sizeof(float) * (2 * NH * BM) + sizeof(int) * (2 * BN);
}

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

// Reduces N values per lane (N a power of two up to 16) over the warp with N - 1 + (5 - log2 N) shuffles instead of
// 5 N: in every halving step a lane hands over the half of its values that its partner keeps.  Afterwards lane L
// holds, in v[0], the warp's total of element (L >> (5 - log2 N)) & (N - 1).
template <int N, bool IS_MAX>
__device__ __forceinline__ float reduce_many(float (&v)[N], int lane) {
  int off = 16;
#pragma unroll
  for (int n = N; n > 1; n >>= 1) {
    const bool upper = (lane & off) != 0;
#pragma unroll
    for (int i = 0; i < n / 2; ++i) {
      const float send = upper ? v[i] : v[i + n / 2];
      const float keep = upper ? v[i + n / 2] : v[i];
      const float got = __shfl_xor_sync(0xffffffffu, send, off);
      v[i] = IS_MAX ? fmaxf(keep, got) : keep + got;
    }
    off >>= 1;
  }
  float t = v[0];
  for (; off > 0; off >>= 1) {
    const float got = __shfl_xor_sync(0xffffffffu, t, off);
    t = IS_MAX ? fmaxf(t, got) : t + got;
  }
  return t;
}

constexpr int NHP = NH <= 1 ? 1 : (NH <= 2 ? 2 : (NH <= 4 ? 4 : (NH <= 8 ? 8 : 16)));      // heads, rounded up to a power of two
constexpr int LOG_NHP = NHP == 1 ? 0 : (NHP == 2 ? 1 : (NHP == 4 ? 2 : (NHP == 8 ? 3 : 4)));

__global__ void __launch_bounds__(THREADS, 1)
pooled_attention_tc_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ q, int64_t q_stride,
                           const __nv_bfloat16* __restrict__ k_pages, const __nv_bfloat16* __restrict__ v_pages,
                           const __nv_bfloat16* __restrict__ pk_pages, const __nv_bfloat16* __restrict__ pv_pages,
                           const int* __restrict__ block_table, int max_pages, const int* __restrict__ pool_table,
                           int pool_width, int page_size, const int* __restrict__ positions,
                           const int* __restrict__ cu_q, int num_seqs, float scale, int window, int pool, int sink,
                           const float* __restrict__ mix, const __nv_bfloat16* __restrict__ gate, int64_t gate_stride) {
  atom::pdl_trigger();
  atom::pdl_wait();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* Qs = (__nv_bfloat16*)smem_raw;                  // [NH][16][LDQ]
  __nv_bfloat16* KVs = Qs + NH * BM * LDQ;                       // [2][64][LDKV]: one kv head's keys or values, twice
  float* raw = (float*)(KVs + 2 * BN * LDKV);                    // [NH][16][LDR]
  float* mix_s = raw + NH * BM * LDR;                            // [NH][NH]
  float* m_s = mix_s + NH * NH;                                  // [NH][16] running maximum
  float* l_s = m_s + NH * BM;                                    // [NH][16] denominator, then its inverse
  int* off_s = (int*)(l_s + NH * BM);                            // [2][64] row of a key in its pages, kv head 0
  __shared__ int tile_s[3];

  if (threadIdx.x == 0) {          // which tile this CTA has: tiles are numbered request by request
    int b = blockIdx.x, found = -1, first = 0, rows = 0;
    for (int s = 0; s < num_seqs; ++s) {
      const int a = cu_q[s], n = cu_q[s + 1] - a;
      const int nt = (n + BM - 1) / BM;
      if (b < nt) {
        found = s;
        first = a + b * BM;
        rows = min(BM, n - b * BM);
        break;
      }
      b -= nt;
    }
    tile_s[0] = found;
    tile_s[1] = first;
    tile_s[2] = rows;
  }
  __syncthreads();
  const int seq = tile_s[0], t0 = tile_s[1], nrows = tile_s[2];
  if (seq < 0) return;
  const int p0 = positions[t0];                                   // the tile's rows have positions p0, p0 + 1, ...
  const int* bt = block_table + (int64_t)seq * max_pages;
  const int* pbt = pool_table ? pool_table + (int64_t)seq * pool_width : nullptr;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int mat = lane >> 3, r8 = lane & 7;

  // The tile's keys: the blocks its last row sees (key x < nb is block x), then the tokens jlo, jlo + 1, ... up to
  // its last row's own (key x >= nb is token jlo + x - nb).
  const int p_last = p0 + nrows - 1;
  const int nb = (window > 0 && pool > 0 && pbt && p_last - window + 1 > 0) ? (p_last - window + 1) / pool : 0;
  const int jlo = (window > 0 && p0 - window + 1 > 0) ? p0 - window + 1 : 0;
  const int hi = nb + (p_last + 1 - jlo);

  // ---- prologue: Q, the mixing matrix, running maximum and denominator
  for (int e = threadIdx.x; e < NH * BM * (DK / 8); e += THREADS) {
    const int seg = e % (DK / 8), hr = e / (DK / 8);
    const int r = hr % BM, h = hr / BM;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < nrows) v = *reinterpret_cast<const uint4*>(q + (int64_t)(t0 + r) * q_stride + h * DK + seg * 8);
    *reinterpret_cast<uint4*>(Qs + (h * BM + r) * LDQ + seg * 8) = v;
  }
  for (int e = threadIdx.x; e < NH * NH; e += THREADS) mix_s[e] = mix ? mix[e] : ((e / NH == e % NH) ? 1.f : 0.f);
  for (int e = threadIdx.x; e < NH * BM; e += THREADS) {
    m_s[e] = sink ? 0.f : -INFINITY;          // the sink: a key of score zero without a value
    l_s[e] = sink ? 1.f : 0.f;
  }
  float O[NKV][TPG][2][4];
#pragma unroll
  for (int g = 0; g < NKV; ++g)
#pragma unroll
    for (int s = 0; s < TPG; ++s)
#pragma unroll
      for (int n = 0; n < 2; ++n) O[g][s][n][0] = O[g][s][n][1] = O[g][s][n][2] = O[g][s][n][3] = 0.f;
  __syncthreads();

  // The keys and values of a chunk come as loads of one kv head's 64 rows each, through two buffers: while the warps
  // work on one load, the next is on its way.  A row's place: >= 0 in the token pages, <= -2 (as -2 - place) in the
  // pooled pages, -1 none.
  int issued = 0, used = 0;
  auto key_rows = [&](int c0_, int* offs) {      // threads 0..63: where chunk c0_'s keys lie
    const int x = c0_ + threadIdx.x;
    int off = -1;
    if (x < nb) {
      const int pg = pbt[x / page_size];
      if (pg >= 0) off = -2 - (pg * NKV * page_size + (x % page_size));
    } else if (x < hi) {
      const int j = jlo + (x - nb);
      const int pg = bt[j / page_size];
      if (pg >= 0) off = pg * NKV * page_size + (j % page_size);
    }
    offs[threadIdx.x] = off;
  };
  auto issue = [&](int c0_, int i, const int* offs) {     // i < NKV: keys of kv head i; else values of kv head i - NKV
    __nv_bfloat16* dst = KVs + (issued & 1) * BN * LDKV;
    if (c0_ < hi) {
      if (i < NKV) {
        for (int e = threadIdx.x; e < BN * (DK / 8); e += THREADS) {
          const int seg = e % (DK / 8), key = e / (DK / 8);
          const int off = offs[key];
          const __nv_bfloat16* base = off >= 0 ? k_pages : pk_pages;
          const int64_t at = off >= 0 ? off : -2 - off;
          cp_async16(dst + key * LDKV + seg * 8,
                     off != -1 ? base + (at + (int64_t)i * page_size) * DK + seg * 8 : k_pages, off != -1);
        }
      } else {
        for (int e = threadIdx.x; e < BN * (DV / 8); e += THREADS) {
          const int seg = e % (DV / 8), key = e / (DV / 8);
          const int off = offs[key];
          const __nv_bfloat16* base = off >= 0 ? v_pages : pv_pages;
          const int64_t at = off >= 0 ? off : -2 - off;
          cp_async16(dst + key * LDKV + seg * 8,
                     off != -1 ? base + (at + (int64_t)(i - NKV) * page_size) * DV + seg * 8 : v_pages, off != -1);
        }
      }
    }
    cp_async_commit();
    ++issued;
  };
  // S_h = Q_h K^T of kv head g's group for the staged keys, to raw[h][row][key] (unscaled)
  auto scores = [&](int g, const __nv_bfloat16* Ks) {
    for (int u = warp; u < QK_UNITS; u += WARPS) {
      const int hq = u / (BN / 16), kb = u % (BN / 16);
      const int h = g * GROUP + hq;
      float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      const __nv_bfloat16* qbase = Qs + (h * BM + (mat & 1) * 8 + r8) * LDQ + (mat >> 1) * 8;
      const __nv_bfloat16* kbase = Ks + (kb * 16 + (mat >> 1) * 8 + r8) * LDKV + (mat & 1) * 8;
#pragma unroll
      for (int ks = 0; ks < DK / 16; ++ks) {
        uint32_t a[4], b[4];
        ldmatrix_x4(a, qbase + ks * 16);
        ldmatrix_x4(b, kbase + ks * 16);
        mma_bf16(s[0], a, b[0], b[1]);
        mma_bf16(s[1], a, b[2], b[3]);
      }
#pragma unroll
      for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int row = (lane >> 2) + (e >= 2 ? 8 : 0);
          const int col = kb * 16 + n * 8 + 2 * (lane & 3) + (e & 1);
          raw[(h * BM + row) * LDR + col] = s[n][e];
        }
    }
  };
  // whether row r (position pr) sees key x of the tile's set
  auto sees = [&](int r, int x) -> bool {
    if (r >= nrows || x >= hi) return false;
    const int pr = p0 + r;
    if (x < nb) return (x + 1) * pool <= pr - window + 1;
    const int j = jlo + (x - nb);
    return j <= pr && (window <= 0 || j > pr - window);
  };
  constexpr int OWNER_SHIFT = 5 - LOG_NHP;                    // lane L answers for head (L >> OWNER_SHIFT) & (NHP - 1)

  // ================================================================ first walk: maximum and denominator
  if (threadIdx.x < BN) key_rows(0, off_s);
  __syncthreads();
  issue(0, 0, off_s);
  int ci = 0;
  for (int c0 = 0; c0 < hi; c0 += BN, ++ci) {
    const int* cur = off_s + (ci & 1) * BN;
    int* nxt = off_s + ((ci + 1) & 1) * BN;
    if (threadIdx.x < BN) key_rows(c0 + BN, nxt);
    __syncthreads();
#pragma unroll 1
    for (int g = 0; g < NKV; ++g) {
      if (g + 1 < NKV)
        issue(c0, g + 1, cur);                                    // the next kv head's keys
      else
        issue(c0 + BN, 0, nxt);                                   // the next chunk's first keys
      cp_async_wait<1>();
      __syncthreads();
      scores(g, KVs + (used & 1) * BN * LDKV);
      ++used;
      __syncthreads();
    }
    {
      const int r = warp;
      const bool ok0 = sees(r, c0 + lane), ok1 = sees(r, c0 + lane + 32);
      float x0[NH], x1[NH], mx[NHP];
#pragma unroll
      for (int h = 0; h < NHP; ++h) {
        mx[h] = -INFINITY;
        if (h < NH) {
          x0[h] = ok0 ? raw[(h * BM + r) * LDR + lane] * scale : -INFINITY;
          x1[h] = ok1 ? raw[(h * BM + r) * LDR + lane + 32] * scale : -INFINITY;
          mx[h] = fmaxf(x0[h], x1[h]);
        }
      }
      const float row_max = reduce_many<NHP, true>(mx, lane);
      const int own = (lane >> OWNER_SHIFT) & (NHP - 1);          // the head this lane answers for
      const bool owner = own < NH && (lane & ((1 << OWNER_SHIFT) - 1)) == 0;
      float m_old_own = 0.f, m_use_own = 0.f;
      if (owner) {
        m_old_own = m_s[own * BM + r];
        const float m_new = fmaxf(m_old_own, row_max);
        m_use_own = (m_new == -INFINITY) ? 0.f : m_new;
        m_s[own * BM + r] = m_new;
      }
      __syncwarp();
      float psum[NHP];
#pragma unroll
      for (int h = 0; h < NHP; ++h) {
        psum[h] = 0.f;
        if (h < NH) {
          const float m_new = m_s[h * BM + r];
          const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
          psum[h] = expf(x0[h] - m_use) + expf(x1[h] - m_use);     // exp(-inf) = 0 for keys that are not seen
        }
      }
      const float row_sum = reduce_many<NHP, false>(psum, lane);
      if (owner) l_s[own * BM + r] = l_s[own * BM + r] * expf(m_old_own - m_use_own) + row_sum;
    }
    __syncthreads();
  }
  for (int e = threadIdx.x; e < NH * BM; e += THREADS) {
    const float l = l_s[e];
    l_s[e] = l > 0.f ? 1.f / l : 0.f;
    if (m_s[e] == -INFINITY) m_s[e] = 0.f;
  }
  // (the load issued last asked for nothing: its chunk lies beyond the keys)
  cp_async_wait<0>();
  __syncthreads();

  // ================================================================ second walk: weights, mixed, times the values
  issued = used = 0;
  if (threadIdx.x < BN) key_rows(0, off_s);
  __syncthreads();
  issue(0, 0, off_s);
  ci = 0;
  for (int c0 = 0; c0 < hi; c0 += BN, ++ci) {
    const int* cur = off_s + (ci & 1) * BN;
    int* nxt = off_s + ((ci + 1) & 1) * BN;
    if (threadIdx.x < BN) key_rows(c0 + BN, nxt);
    __syncthreads();
#pragma unroll 1
    for (int g = 0; g < NKV; ++g) {
      issue(c0, g + 1, cur);                                      // the next kv head's keys, or the first one's values
      cp_async_wait<1>();
      __syncthreads();
      scores(g, KVs + (used & 1) * BN * LDKV);
      ++used;
      __syncthreads();
    }
    {
      const int r = warp;
      const bool ok0 = sees(r, c0 + lane), ok1 = sees(r, c0 + lane + 32);
      float x0[NH], x1[NH];
#pragma unroll
      for (int g = 0; g < NH; ++g) {
        const float m = m_s[g * BM + r], il = l_s[g * BM + r];
        x0[g] = ok0 ? expf(raw[(g * BM + r) * LDR + lane] * scale - m) * il : 0.f;
        x1[g] = ok1 ? expf(raw[(g * BM + r) * LDR + lane + 32] * scale - m) * il : 0.f;
      }
      __syncwarp();                                                // (all lanes have read the row's scores)
#pragma unroll
      for (int h = 0; h < NH; ++h) {
        float w0 = 0.f, w1 = 0.f;
#pragma unroll
        for (int g = 0; g < NH; ++g) {
          const float w = mix_s[h * NH + g];
          w0 = fmaf(w, x0[g], w0);
          w1 = fmaf(w, x1[g], w1);
        }
        __nv_bfloat16* ph = reinterpret_cast<__nv_bfloat16*>(raw + (h * BM + r) * LDR);
        const __nv_bfloat16 h0 = __float2bfloat16_rn(w0), h1 = __float2bfloat16_rn(w1);
        ph[lane] = h0;
        ph[lane + 32] = h1;
        ph[LDR + lane] = __float2bfloat16_rn(w0 - __bfloat162float(h0));
        ph[LDR + lane + 32] = __float2bfloat16_rn(w1 - __bfloat162float(h1));
      }
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < NKV; ++g) {
      if (g + 1 < NKV)
        issue(c0, NKV + g + 1, cur);                              // the next kv head's values
      else
        issue(c0 + BN, 0, nxt);                                   // the next chunk's first keys
      cp_async_wait<1>();
      __syncthreads();
      const __nv_bfloat16* Vs = KVs + (used & 1) * BN * LDKV;
      ++used;
#pragma unroll
      for (int s = 0; s < TPG; ++s) {
        const int u = warp + WARPS * s;
        if (u < PV_UNITS) {
          const int hq = u / (DV / 16), db = u % (DV / 16);
          const int h = g * GROUP + hq;
          const __nv_bfloat16* pbase = reinterpret_cast<const __nv_bfloat16*>(raw + (h * BM + (mat & 1) * 8 + r8) * LDR) + (mat >> 1) * 8;
          const __nv_bfloat16* vbase = Vs + ((mat & 1) * 8 + r8) * LDKV + (mat >> 1) * 8 + db * 16;
#pragma unroll
          for (int kk = 0; kk < BN / 16; ++kk) {
            uint32_t ah[4], al[4], b[4];
            ldmatrix_x4(ah, pbase + kk * 16);
            ldmatrix_x4(al, pbase + LDR + kk * 16);
            ldmatrix_x4_trans(b, vbase + kk * 16 * LDKV);
            mma_bf16(O[g][s][0], ah, b[0], b[1]);
            mma_bf16(O[g][s][1], ah, b[2], b[3]);
            mma_bf16(O[g][s][0], al, b[0], b[1]);
            mma_bf16(O[g][s][1], al, b[2], b[3]);
          }
        }
      }
      __syncthreads();
    }
  }
  cp_async_wait<0>();

  // ---- epilogue: the gate, and out
  constexpr int n_out = NH * DV;
#pragma unroll
  for (int g = 0; g < NKV; ++g)
#pragma unroll
    for (int s = 0; s < TPG; ++s) {
      const int u = warp + WARPS * s;
      if (u < PV_UNITS) {
        const int hq = u / (DV / 16), db = u % (DV / 16);
        const int h = g * GROUP + hq;
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
          for (int half_ = 0; half_ < 2; ++half_) {
            const int row = (lane >> 2) + half_ * 8;
            const int col = h * DV + db * 16 + n * 8 + 2 * (lane & 3);
            if (row < nrows) {
              float a = O[g][s][n][2 * half_], b = O[g][s][n][2 * half_ + 1];
              if (gate) {
                const float2 gg = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gate + (int64_t)(t0 + row) * gate_stride + col));
                a = a / (1.f + expf(-gg.x));
                b = b / (1.f + expf(-gg.y));
              }
              *reinterpret_cast<__nv_bfloat162*>(out + (int64_t)(t0 + row) * n_out + col) = __floats2bfloat162_rn(a, b);
            }
          }
      }
    }
}

}  // namespace pwtc
}  // namespace atom

ATOM_EXPORT int atom_pwtc_sizes(int* nh, int* nkv, int* dk, int* dv) {
  *nh = atom::pwtc::NH;
  *nkv = atom::pwtc::NKV;
  *dk = atom::pwtc::DK;
  *dv = atom::pwtc::DV;
  return ATOM_OK;
}

ATOM_EXPORT int atom_pwtc_set_option(int key, int value) { return atom::set_option(key, value); }

// Shapes as atom_pooled_attention (pooled_attention.cu), all bfloat16; cu_q: [num_seqs + 1] first token row of every
// request; tiles: an upper bound on the number of 16-row tiles, e.g. ceil(T / 16) + num_seqs.
ATOM_EXPORT int atom_pooled_attention_tc(void* out, const void* q, int64_t q_stride, const void* k_pages,
                                         const void* v_pages, const void* pk_pages, const void* pv_pages,
                                         const int* block_table, int max_pages, const int* pool_table, int pool_width,
                                         int page_size, const int* positions, const int* cu_q, int num_seqs, int tiles,
                                         float scale, int window, int pool, int sink, const float* mix, const void* gate,
                                         int64_t gate_stride, cudaStream_t stream) {
  using namespace atom::pwtc;
  if (tiles <= 0) return ATOM_OK;
  if (page_size <= 0 || window < 0 || pool < 0 || (q_stride % 8) != 0 || ((uintptr_t)q % 16) != 0 ||
      ((uintptr_t)k_pages % 16) != 0 || ((uintptr_t)v_pages % 16) != 0 || ((uintptr_t)pk_pages % 16) != 0 ||
      ((uintptr_t)pv_pages % 16) != 0 || (gate && ((gate_stride % 2) != 0 || ((uintptr_t)gate % 4) != 0)))
    return ATOM_ERR_ARG;
  if (pool > 0 && window > 0 && (!pk_pages || !pv_pages || !pool_table)) return ATOM_ERR_ARG;
  const size_t smem = smem_bytes();
  if (smem > 226 * 1024) return ATOM_ERR_ARG;      // (the kernel has a few static bytes of its own)
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(pooled_attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return ATOM_ERR_LAUNCH;
    attr_set = true;
  }
  atom::launch_pdl(pooled_attention_tc_kernel, dim3(tiles), dim3(THREADS), smem, stream, (__nv_bfloat16*)out,
                   (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages,
                   (const __nv_bfloat16*)pk_pages, (const __nv_bfloat16*)pv_pages, block_table, max_pages, pool_table,
                   pool_width, page_size, positions, cu_q, num_seqs, scale, window, pool, sink, mix,
                   (const __nv_bfloat16*)gate, gate_stride);
  return atom::check_launch();
}
