// Kernels of latent attention, routed experts and table-sum embeddings.
//
//   hashed_pair_add   x[t] += table[row(previous token, token)], the previous token kept per request
//   sinusoid_add      x[t, 2i] += sin(p f_i), x[t, 2i+1] += cos(p f_i)
//   latent_write      RMS norm of a projected latent row, written into the token's page
//   rows_gemm         float32-accumulating products on the CUDA cores whose rows may be gathered
//                     and scaled and whose weights are chosen per head (batched over heads) or per
//                     tile (experts); each output element is one thread's in-order sum over k, so
//                     a row's result does not depend on the batch it is in
//   moe_route         a router's logits (+ bias), the top-k experts per token with sigmoid scores or
//                     a softmax over the chosen logits, a shared gate
//   moe_sort          tokens' expert choices sorted by expert, as tiles of rows for rows_gemm
//   moe_combine       per token: the sum of its experts' rows (+ gate * shared expert), into x
#include "common.cuh"
#include "kernels.h"

namespace lse {

// ------------------------------------------------------------------------------------ embeddings
constexpr int EMB_SLICE = 256;  // columns per block of the sinusoid: two per thread

template <typename T>
__global__ void __launch_bounds__(128)
hashed_pair_add_kernel(float* __restrict__ x, const T* __restrict__ table, int* __restrict__ state,
                       const int* __restrict__ ids, const int* __restrict__ positions,
                       const int* __restrict__ token_seq, const int* __restrict__ cu_q,
                       const int* __restrict__ slots, int W, long long buckets, long long mul_prev,
                       long long mul_cur) {
  pdl_trigger();
  pdl_wait();  // everything below reads what kernels before this one wrote
  const int t = blockIdx.x;
  const int seq = token_seq[t];
  const int first = cu_q[seq];
  const int cur = ids[t];
  long long row = buckets;  // a sequence's first token
  if (positions[t] > 0) {
    const int prev = (t == first) ? state[slots[seq]] : ids[t - 1];
    row = ((long long)prev * mul_prev + (long long)cur * mul_cur) % buckets;
  }
  __syncthreads();  // the state was read before it is written below
  // the block of a sequence's first row is the only one that touches the sequence's state
  if (t == first && threadIdx.x == 0) state[slots[seq]] = ids[cu_q[seq + 1] - 1];
  const T* src = table + (size_t)row * W;
  float* dst = x + (size_t)t * W;
#pragma unroll 4
  for (int i = threadIdx.x; i < W; i += 128) dst[i] += Num<T>::to_float(src[i]);
}

__global__ void __launch_bounds__(128)
sinusoid_add_kernel(float* __restrict__ x, const int* __restrict__ positions,
                    const float* __restrict__ freq, int W) {
  pdl_trigger();
  pdl_wait();  // everything below reads what kernels before this one wrote
  const int t = blockIdx.x;
  const float p = (float)positions[t];
  float* dst = x + (size_t)t * W;
  const int i0 = blockIdx.y * EMB_SLICE + threadIdx.x;
#pragma unroll
  for (int j = 0; j < EMB_SLICE / 128; ++j) {
    const int i = i0 + j * 128;
    if (i < W) {
      const float ang = p * freq[i >> 1];  // the angle is a float32 product, as positions are float32
      dst[i] += (i & 1) ? cosf(ang) : sinf(ang);
    }
  }
}

// ------------------------------------------------------------------------------------ latent rows
template <typename TIn, typename T>
__global__ void __launch_bounds__(128)
latent_write_kernel(const TIn* __restrict__ proj, long long stride, int col0, int R, int Rp,
                    const float* __restrict__ weight, float eps, T* __restrict__ pages,
                    const int* __restrict__ positions, const int* __restrict__ token_seq,
                    const int* __restrict__ block_tables, int table_stride, int page_tokens) {
  pdl_trigger();
  pdl_wait();  // everything below reads what kernels before this one wrote
  __shared__ float red[32];
  const int t = blockIdx.x;
  const TIn* src = proj + (size_t)t * stride + col0;
  float ss = 0.f;
  for (int i = threadIdx.x; i < R; i += blockDim.x) {
    const float v = Num<TIn>::to_float(src[i]);
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float r = rsqrtf(ss / (float)R + eps);
  const int pos = positions[t];
  const int page = block_tables[(size_t)token_seq[t] * table_stride + pos / page_tokens];
  T* dst = pages + ((size_t)page * page_tokens + pos % page_tokens) * Rp;
  for (int i = threadIdx.x; i < Rp; i += blockDim.x)
    dst[i] = Num<T>::from_float(i < R ? Num<TIn>::to_float(src[i]) * r * weight[i] : 0.f);
}

// ------------------------------------------------------------------------------------ rows_gemm
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;  // 256 threads, 4x4 outputs each

struct RowsGemm {
  const void* a;            // [rows, a_stride] (+ a_col0 + batch * a_batch_cols)
  long long a_stride;
  long long a_col0, a_batch_cols;
  const int* a_rows;        // null, or logical row r reads row a_rows[r] / a_div ...
  int a_div;
  const float* a_scale;     // ... multiplied by a_scale[a_rows[r]] (null: not scaled)
  const void* w;            // [N, K] at w + batch * w_batch_stride
  long long w_batch_stride;
  void* out;                // [rows, out_stride] (+ batch * out_batch_cols)
  long long out_stride, out_batch_cols;
  // tiles of rows that belong to one batch entry each (null: all rows, batch = blockIdx.z)
  const int* tile_batch;
  const int* tile_row0;
  const int* offsets;       // [batches + 1] row ranges of the batch entries
  const int* num_tiles;
  int T, N, K;
};

template <typename TA, typename TW, typename TO>
__global__ void __launch_bounds__(256) rows_gemm_kernel(const RowsGemm g) {
  pdl_trigger();
  pdl_wait();  // everything below reads what kernels before this one wrote
  __shared__ float as[BK][BM + 4];
  __shared__ float ws[BK][BN + 4];
  __shared__ int srow[BM];
  __shared__ float sscale[BM];
  const int tid = threadIdx.x;
  int batch, m0, m_end;
  if (g.tile_batch) {
    if ((int)blockIdx.y >= *g.num_tiles) return;
    batch = g.tile_batch[blockIdx.y];
    m0 = g.tile_row0[blockIdx.y];
    m_end = min(g.offsets[batch + 1], m0 + BM);
  } else {
    batch = blockIdx.z;
    m0 = blockIdx.y * BM;
    m_end = min(g.T, m0 + BM);
  }
  if (tid < BM) {
    const int r = m0 + tid;
    int row = -1;
    float sc = 1.f;
    if (r < m_end) {
      const int idx = g.a_rows ? g.a_rows[r] : r;
      row = g.a_rows ? idx / g.a_div : r;
      if (g.a_scale) sc = g.a_scale[idx];
    }
    srow[tid] = row;
    sscale[tid] = sc;
  }
  __syncthreads();
  const int N = g.N, K = g.K;
  const int n0 = blockIdx.x * BN;
  const TA* a = (const TA*)g.a + g.a_col0 + (long long)batch * g.a_batch_cols;
  const TW* w = (const TW*)g.w + (long long)batch * g.w_batch_stride;
  const int tm = (tid / 16) * TM, tn = (tid % 16) * TN;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;
  const int lr = tid / 4, lk = (tid % 4) * 4;
  const int arow = srow[lr];
  const float asc = sscale[lr];
  const int gn = n0 + lr;
  for (int k0 = 0; k0 < K; k0 += BK) {
    float av[4] = {0.f, 0.f, 0.f, 0.f}, wv[4] = {0.f, 0.f, 0.f, 0.f};
    const int gk = k0 + lk;
    if (arow >= 0) {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (gk + j < K) av[j] = Num<TA>::to_float(a[(size_t)arow * g.a_stride + gk + j]) * asc;
    }
    if (gn < N) {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (gk + j < K) wv[j] = Num<TW>::to_float(w[(size_t)gn * K + gk + j]);
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      as[lk + j][lr] = av[j];
      ws[lk + j][lr] = wv[j];
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float ar[TM], wr[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) ar[i] = as[kk][tm + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) wr[j] = ws[kk][tn + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(ar[i], wr[j], acc[i][j]);
    }
  }
  TO* out = (TO*)g.out + (long long)batch * g.out_batch_cols;
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int r = m0 + tm + i;
    if (r >= m_end) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tn + j;
      if (n < N) out[(size_t)r * g.out_stride + n] = Num<TO>::from_float(acc[i][j]);
    }
  }
}

// ------------------------------------------------------------------------------------ rows_gemm, bfloat16
// The same products for bfloat16 operands whose rows are whole 16-byte vectors (K, the row
// strides and the column offsets multiples of 8). out_scale: the result of logical row r is
// multiplied by a_scale[a_rows[r]] (a product is linear in its input, so scaling the input row
// is scaling the result; here it is done in float32 on the sums).
//
// rows_gemm_mma: 64 rows x 128 columns per block on mma.sync tensor cores (m16n8k16, float32
// accumulation), 8 warps of 32 x 32, operand tiles of 32 k brought by cp.async into two buffers.
constexpr int MM_BN = 128, MM_BK = 32, MM_LD = MM_BK + 8, MM_THREADS = 256;

__device__ __forceinline__ void rg_ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void rg_mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void rg_cp_async16(void* smem, const void* gmem, bool valid) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;  // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(addr), "l"(gmem), "r"(bytes));
}

// Which rows a block works on (shared by the kernels of this file): tile or grid position.
__device__ __forceinline__ bool rows_of_block(const RowsGemm& g, int& batch, int& m0, int& m_end) {
  if (g.tile_batch) {
    if ((int)blockIdx.y >= *g.num_tiles) return false;
    batch = g.tile_batch[blockIdx.y];
    m0 = g.tile_row0[blockIdx.y];
    m_end = min(g.offsets[batch + 1], m0 + BM);
  } else {
    batch = blockIdx.z;
    m0 = blockIdx.y * BM;
    m_end = min(g.T, m0 + BM);
  }
  return true;
}

template <typename TO>
__global__ void __launch_bounds__(MM_THREADS) rows_gemm_mma_kernel(const RowsGemm g) {
  pdl_trigger();
  pdl_wait();  // everything below reads what kernels before this one wrote
  __shared__ __align__(16) bf16 As[2][BM][MM_LD];
  __shared__ __align__(16) bf16 Bs[2][MM_BN][MM_LD];
  __shared__ int srow[BM];
  __shared__ float sscale[BM];
  const int tid = threadIdx.x;
  int batch, m0, m_end;
  if (!rows_of_block(g, batch, m0, m_end)) return;
  if (tid < BM) {
    const int r = m0 + tid;
    int row = -1;
    float sc = 1.f;
    if (r < m_end) {
      const int idx = g.a_rows ? g.a_rows[r] : r;
      row = g.a_rows ? idx / g.a_div : r;
      if (g.a_scale) sc = g.a_scale[idx];
    }
    srow[tid] = row;
    sscale[tid] = sc;
  }
  __syncthreads();
  const int N = g.N, K = g.K;
  const int n0 = blockIdx.x * MM_BN;
  const bf16* a = (const bf16*)g.a + g.a_col0 + (long long)batch * g.a_batch_cols;
  const bf16* w = (const bf16*)g.w + (long long)batch * g.w_batch_stride;
  const int warp = tid >> 5, lane = tid & 31, gq = lane >> 2, t4 = lane & 3;
  const int wm = (warp >> 2) * 32, wn = (warp & 3) * 32;

  auto load_tiles = [&](int buf, int k0) {
    // A: 64 rows x 4 vectors; B: 128 rows x 4 vectors
    {
      const int r = tid >> 2, c = (tid & 3) * 8;
      const int row = srow[r];
      const bool ok = row >= 0 && k0 + c < K;
      rg_cp_async16(&As[buf][r][c], a + (ok ? (size_t)row * g.a_stride + k0 + c : 0), ok);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int idx = tid + i * MM_THREADS;
      const int r = idx >> 2, c = (idx & 3) * 8;
      const bool ok = n0 + r < N && k0 + c < K;
      rg_cp_async16(&Bs[buf][r][c], w + (ok ? (size_t)(n0 + r) * K + k0 + c : 0), ok);
    }
    asm volatile("cp.async.commit_group;\n" ::);
  };

  float acc[2][4][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;

  load_tiles(0, 0);
  int buf = 0;
  for (int k0 = 0; k0 < K; k0 += MM_BK, buf ^= 1) {
    if (k0 + MM_BK < K) {
      load_tiles(buf ^ 1, k0 + MM_BK);
      asm volatile("cp.async.wait_group 1;\n" ::);
    } else {
      asm volatile("cp.async.wait_group 0;\n" ::);
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < MM_BK / 16; ++kk) {
      uint32_t af[2][4];
#pragma unroll
      for (int mi = 0; mi < 2; ++mi)
        rg_ldmatrix_x4(af[mi], &As[buf][wm + mi * 16 + (lane & 15)][kk * 16 + ((lane >> 4) << 3)]);
#pragma unroll
      for (int nb = 0; nb < 4; nb += 2) {
        uint32_t b[4];
        rg_ldmatrix_x4(b, &Bs[buf][wn + nb * 8 + (lane & 7) + ((lane >> 4) << 3)][kk * 16 + (((lane >> 3) & 1) << 3)]);
#pragma unroll
        for (int mi = 0; mi < 2; ++mi) {
          rg_mma_bf16(acc[mi][nb], af[mi], b[0], b[1]);
          rg_mma_bf16(acc[mi][nb + 1], af[mi], b[2], b[3]);
        }
      }
    }
    __syncthreads();  // all warps are done with this buffer before it is filled again
  }
  TO* out = (TO*)g.out + (long long)batch * g.out_batch_cols;
#pragma unroll
  for (int mi = 0; mi < 2; ++mi)
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
      const int lr = wm + mi * 16 + gq + rr * 8;
      const int r = m0 + lr;
      if (r >= m_end) continue;
      const float sc = sscale[lr];
#pragma unroll
      for (int nb = 0; nb < 4; ++nb)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int n = n0 + wn + nb * 8 + t4 * 2 + e;
          if (n < N) out[(size_t)r * g.out_stride + n] = Num<TO>::from_float(acc[mi][nb][rr * 2 + e] * sc);
        }
    }
}

// rows_gemv: few rows per tile (single tokens). A warp streams four weight rows at a time in
// 16-byte pieces, two steps of k in flight (eight loads per lane), and multiplies them with up to
// RN rows of the tile (RN = 1, 2 or 4 by the tile's row count; more rows take further passes over
// the weights, which then come from L2); the rows come from L1. The lanes' partial sums are added
// in a fixed order, so a row's result does not depend on the batch.
constexpr int GV_WARPS = 8, GV_ROWS = 4, GV_CPW = 4, GV_COLS = GV_WARPS * GV_CPW;  // columns per block

template <typename TO, int RN>
__device__ __forceinline__ void gemv_rows(const RowsGemm& g, const bf16* a, const bf16* w, TO* out,
                                          const int* srow, const float* sscale, int m0, int r0, int rows,
                                          int n, int lane) {
  const int K = g.K, N = g.N;
  const bf16* wr[GV_CPW];
#pragma unroll
  for (int c = 0; c < GV_CPW; ++c) wr[c] = w + (size_t)min(n + c, N - 1) * K;
  const bf16* ar[RN];
#pragma unroll
  for (int r = 0; r < RN; ++r) ar[r] = a + (size_t)srow[min(r0 + r, rows - 1)] * g.a_stride;
  float acc[GV_CPW][RN];
#pragma unroll
  for (int c = 0; c < GV_CPW; ++c)
#pragma unroll
    for (int r = 0; r < RN; ++r) acc[c][r] = 0.f;
  for (int k = lane * 8; k < K; k += 2 * 32 * 8) {
    const int k2 = k + 32 * 8;
    const bool more = k2 < K;
    Vec16<bf16> wv[2][GV_CPW];
#pragma unroll
    for (int c = 0; c < GV_CPW; ++c) {
      wv[0][c] = load16(wr[c] + k);
      wv[1][c] = load16(wr[c] + (more ? k2 : k));
    }
#pragma unroll
    for (int r = 0; r < RN; ++r) {
      const Vec16<bf16> a0 = load16(ar[r] + k), a1 = load16(ar[r] + (more ? k2 : k));
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float x0 = __bfloat162float(a0.v[e]);
        const float x1 = more ? __bfloat162float(a1.v[e]) : 0.f;
#pragma unroll
        for (int c = 0; c < GV_CPW; ++c) {
          acc[c][r] = fmaf(x0, __bfloat162float(wv[0][c].v[e]), acc[c][r]);
          acc[c][r] = fmaf(x1, __bfloat162float(wv[1][c].v[e]), acc[c][r]);
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < RN; ++r)
#pragma unroll
    for (int c = 0; c < GV_CPW; ++c) {
      const float sum = warp_sum(acc[c][r]);
      if (lane == 0 && r0 + r < rows && n + c < N)
        out[(size_t)(m0 + r0 + r) * g.out_stride + n + c] = Num<TO>::from_float(sum * sscale[r0 + r]);
    }
}

template <typename TO>
__global__ void __launch_bounds__(GV_WARPS * 32, 2) rows_gemv_kernel(const RowsGemm g) {
  pdl_trigger();
  pdl_wait();  // everything below reads what kernels before this one wrote
  __shared__ int srow[BM];
  __shared__ float sscale[BM];
  const int tid = threadIdx.x;
  int batch, m0, m_end;
  if (!rows_of_block(g, batch, m0, m_end)) return;
  if (tid < BM) {
    const int r = m0 + tid;
    int row = 0;
    float sc = 1.f;
    if (r < m_end) {
      const int idx = g.a_rows ? g.a_rows[r] : r;
      row = g.a_rows ? idx / g.a_div : r;
      if (g.a_scale) sc = g.a_scale[idx];
    }
    srow[tid] = row;
    sscale[tid] = sc;
  }
  __syncthreads();
  const int rows = m_end - m0;
  if (rows <= 0) return;
  const bf16* a = (const bf16*)g.a + g.a_col0 + (long long)batch * g.a_batch_cols;
  const bf16* w = (const bf16*)g.w + (long long)batch * g.w_batch_stride;
  TO* out = (TO*)g.out + (long long)batch * g.out_batch_cols;
  const int warp = tid >> 5, lane = tid & 31;
  const int n = blockIdx.x * GV_COLS + warp * GV_CPW;
  if (n >= g.N) return;
  for (int r0 = 0; r0 < rows; r0 += GV_ROWS) {
    const int left = rows - r0;
    if (left == 1) gemv_rows<TO, 1>(g, a, w, out, srow, sscale, m0, r0, rows, n, lane);
    else if (left == 2) gemv_rows<TO, 2>(g, a, w, out, srow, sscale, m0, r0, rows, n, lane);
    else gemv_rows<TO, GV_ROWS>(g, a, w, out, srow, sscale, m0, r0, rows, n, lane);
  }
}

// ------------------------------------------------------------------------------------ routing
// One block of eight warps per token. Every router row is shared by the eight warps (warp w takes
// the columns w * 32 + lane, + 256, ...); the warps' partial sums are added in the order of the
// warps, so a score depends on nothing but the width. z = router . h (+ bias) in float32; then the
// first warp picks the `top` largest (the lower index on a tie). Their weights: sigmoid(z) (mode 0;
// the sigmoid is monotone, so the order is that of z) or the softmax over the chosen z alone
// (mode 1). Row E of the router, if there is one, is the shared expert's gate.
constexpr int ROUTE_WARPS = 8;

template <typename TH>
__global__ void __launch_bounds__(ROUTE_WARPS * 32)
moe_route_kernel(const TH* __restrict__ h, const float* __restrict__ router, int W, int E,
                 int has_gate, int top, int* __restrict__ idx, float* __restrict__ wts,
                 float* __restrict__ gate, const float* __restrict__ bias, int mode) {
  pdl_trigger();
  pdl_wait();  // everything below reads what kernels before this one wrote
  extern __shared__ float s[];  // [E + 1] scores, then [E + 1][ROUTE_WARPS] partial sums
  float* part = s + E + 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const size_t t = blockIdx.x;
  const TH* row = h + t * W;
  const int rows = E + has_gate;
  for (int e = 0; e < rows; ++e) {
    const float* r = router + (size_t)e * W;
    float d = 0.f;
    for (int i = threadIdx.x; i < W; i += ROUTE_WARPS * 32) d = fmaf(Num<TH>::to_float(row[i]), r[i], d);
    d = warp_sum(d);
    if (lane == 0) part[e * ROUTE_WARPS + warp] = d;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < rows; e += ROUTE_WARPS * 32) {
    float d = 0.f;
#pragma unroll
    for (int w = 0; w < ROUTE_WARPS; ++w) d += part[e * ROUTE_WARPS + w];
    if (e < E) s[e] = d + (bias ? bias[e] : 0.f);
    else gate[t] = 1.f / (1.f + expf(-d));
  }
  __syncthreads();
  if (warp != 0) return;
  float first = 0.f, total = 0.f;  // mode 1: the largest chosen logit, the sum of the exponentials
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32)
      if (s[e] > best || (bi == 0x7fffffff && s[e] == best)) {
        best = s[e];
        bi = e;
      }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) {
        best = ob;
        bi = oi;
      }
    }
    if (bi == 0x7fffffff) bi = 0;  // only if every logit left is NaN
    if (k == 0) first = best;
    const float wk = mode == 0 ? 1.f / (1.f + expf(-best)) : expf(best - first);
    total += wk;
    if (lane == 0) {
      idx[t * top + k] = bi;
      wts[t * top + k] = wk;
      s[bi] = -INFINITY;  // taken
    }
    __syncwarp();
  }
  if (mode == 1)
    for (int k = lane; k < top; k += 32) wts[t * top + k] /= total;
}

// One block. n choices idx[i] in [0, E): offsets[e] .. offsets[e+1] are expert e's rows in the
// sorted order, perm[r] the choice at sorted row r, pos_of[i] the sorted row of choice i, and the
// rows as tiles of at most tile_rows rows of one expert (tile_batch, tile_row0, num_tiles).
__global__ void __launch_bounds__(1024)
moe_sort_kernel(const int* __restrict__ idx, int n, int E, int tile_rows, int* __restrict__ offsets,
                int* __restrict__ perm, int* __restrict__ pos_of, int* __restrict__ tile_batch,
                int* __restrict__ tile_row0, int* __restrict__ num_tiles) {
  pdl_trigger();
  pdl_wait();  // everything below reads what kernels before this one wrote
  extern __shared__ int sm_sort[];  // counts[E], start[E + 1], tile_start[E + 1]
  int* counts = sm_sort;
  int* start = counts + E;
  int* tstart = start + E + 1;
  for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) atomicAdd(&counts[idx[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0, tiles = 0;
    for (int e = 0; e < E; ++e) {
      start[e] = run;
      tstart[e] = tiles;
      run += counts[e];
      tiles += (counts[e] + tile_rows - 1) / tile_rows;
    }
    start[E] = run;
    tstart[E] = tiles;
    *num_tiles = tiles;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) offsets[e] = start[e];
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int nt = tstart[e + 1] - tstart[e];
    for (int k = 0; k < nt; ++k) {
      tile_batch[tstart[e] + k] = e;
      tile_row0[tstart[e] + k] = start[e] + k * tile_rows;
    }
    counts[e] = 0;  // now the cursor of expert e
  }
  __syncthreads();
  // the order of an expert's rows among themselves is free: every row's result stands alone
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int e = idx[i];
    const int r = start[e] + atomicAdd(&counts[e], 1);
    perm[r] = i;
    pos_of[i] = r;
  }
}

// out[r] = a[perm[r] / top]: the tokens' rows in sorted order, in 16-byte pieces (K a multiple of 8)
__global__ void __launch_bounds__(256)
moe_gather_rows_kernel(const bf16* __restrict__ a, const int* __restrict__ perm, int top,
                       bf16* __restrict__ out, int n, int K) {
  pdl_trigger();
  pdl_wait();  // everything below reads what kernels before this one wrote
  const int per_row = K / 8;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)n * per_row) return;
  const int r = (int)(i / per_row), c = (int)(i - (long long)r * per_row);
  store16(out + (size_t)r * K + c * 8, load16(a + (size_t)(perm[r] / top) * K + c * 8));
}

// x[t] (or out[t]) (+)= sum_k wts[t * top + k] * y[pos_of[t * top + k]] + gate[t] * shared[t] (a
// null wts or gate counts as ones); a block per token and
// slice of 512 columns, four columns per thread (the experts' rows are added in the order k = 0, 1, ...)
constexpr int COMBINE_SLICE = 512;

__global__ void __launch_bounds__(128)
moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ pos_of, int top,
                   const float* __restrict__ shared_out, const float* __restrict__ gate,
                   float* __restrict__ out, int accumulate, int W, const float* __restrict__ wts) {
  pdl_trigger();
  pdl_wait();  // everything below reads what kernels before this one wrote
  const int t = blockIdx.x;
  const float g = gate ? gate[t] : 1.f;
  const int i0 = blockIdx.y * COMBINE_SLICE + threadIdx.x;
  float v[COMBINE_SLICE / 128];
#pragma unroll
  for (int j = 0; j < COMBINE_SLICE / 128; ++j) v[j] = 0.f;
  for (int k = 0; k < top; ++k) {
    const float* row = y + (size_t)pos_of[(size_t)t * top + k] * W;
    const float wk = wts ? wts[(size_t)t * top + k] : 1.f;
#pragma unroll
    for (int j = 0; j < COMBINE_SLICE / 128; ++j) {
      const int i = i0 + j * 128;
      if (i < W) v[j] = fmaf(wk, row[i], v[j]);
    }
  }
#pragma unroll
  for (int j = 0; j < COMBINE_SLICE / 128; ++j) {
    const int i = i0 + j * 128;
    if (i >= W) continue;
    float r = v[j];
    if (shared_out) r += g * shared_out[(size_t)t * W + i];
    float* o = out + (size_t)t * W + i;
    *o = accumulate ? *o + r : r;
  }
}

}  // namespace lse

using namespace lse;

#define LSE_CHECK_LAUNCH() (cudaPeekAtLastError() == cudaSuccess ? LSE_OK : LSE_LAUNCH_FAILED)

extern "C" int lse_hashed_pair_add(float* x, const void* table, int table_dtype, int* state,
                                   const int* ids, const int* positions, const int* token_seq,
                                   const int* cu_q, const int* slots, int T, int num_seqs, int W,
                                   long long buckets, long long mul_prev, long long mul_cur,
                                   cudaStream_t stream) {
  if (T <= 0) return LSE_OK;
  if (buckets <= 0 || W <= 0 || num_seqs <= 0) return LSE_BAD_ARGUMENT;
  if (table_dtype == LSE_F32)
    launch(hashed_pair_add_kernel<float>, T, 128, 0, stream, x, (const float*)table, state, ids, positions, token_seq,
                                                         cu_q, slots, W, buckets, mul_prev, mul_cur);
  else if (table_dtype == LSE_BF16)
    launch(hashed_pair_add_kernel<bf16>, T, 128, 0, stream, x, (const bf16*)table, state, ids, positions, token_seq,
                                                        cu_q, slots, W, buckets, mul_prev, mul_cur);
  else
    return LSE_BAD_ARGUMENT;
  return LSE_CHECK_LAUNCH();
}

extern "C" int lse_sinusoid_add(float* x, const int* positions, const float* freq, int T, int W,
                                cudaStream_t stream) {
  if (T <= 0) return LSE_OK;
  launch(sinusoid_add_kernel, dim3(T, (W + EMB_SLICE - 1) / EMB_SLICE), 128, 0, stream, x, positions, freq, W);
  return LSE_CHECK_LAUNCH();
}

extern "C" int lse_latent_write(const void* proj, int in_dtype, long long stride, int col0, int R,
                                int Rp, const float* weight, float eps, void* pages, int dtype,
                                const int* positions, const int* token_seq, const int* block_tables,
                                int table_stride, int page_tokens, int T, cudaStream_t stream) {
  if (T <= 0) return LSE_OK;
  if (R <= 0 || Rp < R || page_tokens <= 0) return LSE_BAD_ARGUMENT;
#define LSE_LATENT(TIn, T_) \
  launch(latent_write_kernel<TIn, T_>, T, 128, 0, stream, (const TIn*)proj, stride, col0, R, Rp, weight, eps, \
      (T_*)pages, positions, token_seq, block_tables, table_stride, page_tokens)
  if (in_dtype == LSE_F32 && dtype == LSE_F32) LSE_LATENT(float, float);
  else if (in_dtype == LSE_F32 && dtype == LSE_BF16) LSE_LATENT(float, bf16);
  else if (in_dtype == LSE_BF16 && dtype == LSE_BF16) LSE_LATENT(bf16, bf16);
  else return LSE_BAD_ARGUMENT;
#undef LSE_LATENT
  return LSE_CHECK_LAUNCH();
}

// kind: 0 = CUDA cores (any operands), 1 = mma.sync tiles, 2 = few rows per tile (1 and 2: bfloat16
// operands of whole 16-byte vectors; they multiply the result by a_scale instead of the input)
static bool vectors_ok(const RowsGemm& g) {
  return g.K % 8 == 0 && g.a_stride % 8 == 0 && g.a_col0 % 8 == 0 && g.a_batch_cols % 8 == 0 &&
         reinterpret_cast<uintptr_t>(g.a) % 16 == 0 && reinterpret_cast<uintptr_t>(g.w) % 16 == 0;
}

static int launch_rows_gemm(const RowsGemm& g, int a_dtype, int w_dtype, int out_dtype, dim3 grid,
                            cudaStream_t stream, int kind = 0) {
  if (grid.y > 65535 || grid.z > 65535) return LSE_BAD_ARGUMENT;
  if (kind != 0 && a_dtype == LSE_BF16 && w_dtype == LSE_BF16 && vectors_ok(g)) {
    if (kind == 1) {
      grid.x = (g.N + MM_BN - 1) / MM_BN;
      if (out_dtype == LSE_F32) launch(rows_gemm_mma_kernel<float>, grid, MM_THREADS, 0, stream, g);
      else launch(rows_gemm_mma_kernel<bf16>, grid, MM_THREADS, 0, stream, g);
    } else {
      grid.x = (g.N + GV_COLS - 1) / GV_COLS;
      if (out_dtype == LSE_F32) launch(rows_gemv_kernel<float>, grid, GV_WARPS * 32, 0, stream, g);
      else launch(rows_gemv_kernel<bf16>, grid, GV_WARPS * 32, 0, stream, g);
    }
    return LSE_CHECK_LAUNCH();
  }
#define LSE_RG(TA, TW, TO) launch(rows_gemm_kernel<TA, TW, TO>, grid, 256, 0, stream, g)
  if (a_dtype == LSE_F32 && w_dtype == LSE_F32 && out_dtype == LSE_F32) LSE_RG(float, float, float);
  else if (a_dtype == LSE_F32 && w_dtype == LSE_BF16 && out_dtype == LSE_BF16) LSE_RG(float, bf16, bf16);
  else if (a_dtype == LSE_F32 && w_dtype == LSE_BF16 && out_dtype == LSE_F32) LSE_RG(float, bf16, float);
  else if (a_dtype == LSE_BF16 && w_dtype == LSE_BF16 && out_dtype == LSE_BF16) LSE_RG(bf16, bf16, bf16);
  else if (a_dtype == LSE_BF16 && w_dtype == LSE_BF16 && out_dtype == LSE_F32) LSE_RG(bf16, bf16, float);
  else return LSE_BAD_ARGUMENT;
#undef LSE_RG
  return LSE_CHECK_LAUNCH();
}

extern "C" int lse_head_linear(const void* a, int a_dtype, long long a_stride, long long a_col0,
                               const void* w, int w_dtype, void* out, int out_dtype, int T, int H,
                               int N, int K, int kind, cudaStream_t stream, long long a_head_cols,
                               long long out_head_cols, long long out_stride) {
  if (T <= 0 || H <= 0 || N <= 0) return LSE_OK;
  if (K <= 0) return LSE_BAD_ARGUMENT;
  if (a_head_cols <= 0) a_head_cols = K;
  if (out_head_cols <= 0) out_head_cols = N;
  if (out_stride <= 0) out_stride = (long long)H * out_head_cols;
  if (a_head_cols < K || out_head_cols < N) return LSE_BAD_ARGUMENT;
  RowsGemm g = {};
  g.a = a; g.a_stride = a_stride; g.a_col0 = a_col0; g.a_batch_cols = a_head_cols; g.a_div = 1;
  g.w = w; g.w_batch_stride = (long long)N * K;
  g.out = out; g.out_stride = out_stride; g.out_batch_cols = out_head_cols;
  g.T = T; g.N = N; g.K = K;
  return launch_rows_gemm(g, a_dtype, w_dtype, out_dtype, dim3((N + BN - 1) / BN, (T + BM - 1) / BM, H), stream,
                          kind);
}

extern "C" int lse_moe_tile_rows(void) { return BM; }

extern "C" int lse_expert_linear(const void* a, int a_dtype, long long a_stride, const int* a_rows,
                                 int a_div, const float* a_scale, const void* w, int w_dtype,
                                 float* out, int rows, int N, int K, const int* offsets,
                                 const int* tile_batch, const int* tile_row0, const int* num_tiles,
                                 int max_tiles, int kind, cudaStream_t stream) {
  if (rows <= 0 || N <= 0 || max_tiles <= 0) return LSE_OK;
  if (K <= 0 || a_div <= 0 || !offsets || !tile_batch || !tile_row0 || !num_tiles) return LSE_BAD_ARGUMENT;
  RowsGemm g = {};
  g.a = a; g.a_stride = a_stride; g.a_rows = a_rows; g.a_div = a_div; g.a_scale = a_scale;
  g.w = w; g.w_batch_stride = (long long)N * K;
  g.out = out; g.out_stride = N;
  g.tile_batch = tile_batch; g.tile_row0 = tile_row0; g.offsets = offsets; g.num_tiles = num_tiles;
  g.T = rows; g.N = N; g.K = K;
  return launch_rows_gemm(g, a_dtype, w_dtype, LSE_F32, dim3((N + BN - 1) / BN, max_tiles, 1), stream, kind);
}

extern "C" int lse_moe_route(const void* h, int h_dtype, const float* router, int T, int W, int E,
                             int has_gate, int top, int* idx, float* wts, float* gate,
                             cudaStream_t stream, const float* bias, int mode) {
  if (T <= 0) return LSE_OK;
  if (E <= 0 || top <= 0 || top > E || E > 1024 || (has_gate && !gate) || mode < 0 || mode > 1) return LSE_BAD_ARGUMENT;
  const size_t smem = (size_t)(E + 1) * (1 + ROUTE_WARPS) * sizeof(float);
  if (h_dtype == LSE_F32)
    launch(moe_route_kernel<float>, T, ROUTE_WARPS * 32, smem, stream, (const float*)h, router, W, E, has_gate, top,
                                                                   idx, wts, gate, bias, mode);
  else if (h_dtype == LSE_BF16)
    launch(moe_route_kernel<bf16>, T, ROUTE_WARPS * 32, smem, stream, (const bf16*)h, router, W, E, has_gate, top,
                                                                  idx, wts, gate, bias, mode);
  else
    return LSE_BAD_ARGUMENT;
  return LSE_CHECK_LAUNCH();
}

extern "C" int lse_moe_sort(const int* idx, int n, int E, int tile_rows, int* offsets, int* perm, int* pos_of,
                            int* tile_batch, int* tile_row0, int* num_tiles, cudaStream_t stream) {
  if (n <= 0) return LSE_OK;
  if (E <= 0 || E > 2048 || tile_rows <= 0) return LSE_BAD_ARGUMENT;
  const size_t smem = (size_t)(3 * E + 2) * sizeof(int);
  launch(moe_sort_kernel, 1, 1024, smem, stream, idx, n, E, tile_rows, offsets, perm, pos_of, tile_batch, tile_row0,
                                             num_tiles);
  return LSE_CHECK_LAUNCH();
}

extern "C" int lse_moe_gather_rows(const void* a, const int* perm, int top, void* out, int n, int K,
                                   cudaStream_t stream) {
  if (n <= 0) return LSE_OK;
  if (K <= 0 || K % 8 || top <= 0) return LSE_BAD_ARGUMENT;
  const long long items = (long long)n * (K / 8);
  launch(moe_gather_rows_kernel, (unsigned)((items + 255) / 256), 256, 0, stream, (const bf16*)a, perm, top, (bf16*)out,
                                                                              n, K);
  return LSE_CHECK_LAUNCH();
}

extern "C" int lse_moe_combine(const float* y, const int* pos_of, int top, const float* shared_out,
                               const float* gate, float* out, int accumulate, int T, int W,
                               cudaStream_t stream, const float* wts) {
  if (T <= 0) return LSE_OK;
  launch(moe_combine_kernel, dim3(T, (W + COMBINE_SLICE - 1) / COMBINE_SLICE), 128, 0, stream, y, pos_of, top,
         shared_out, gate, out, accumulate, W, wts);
  return LSE_CHECK_LAUNCH();
}
