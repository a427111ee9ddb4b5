// Kernels of blocks that carry several residual streams, of attention whose queries and keys are
// prepared a whole token at a time, and of differential attention.
//
//   streams_spread        every stream of a token starts as its embedded row times a constant
//   streams_read_norm     u = sum_s read[s] x_s, then u / rms(u) * w, per token (or per listed row)
//   streams_write         x_t <- sum_s mix[s, t] x_s + out[t] * scale * y for all streams t of a
//                         token at once; optionally followed, while the block holds the token's
//                         streams, by the read and norm that the next sublayer needs
//   qkv_norm_rope_write   per token: RMS norm over all query rows (and over all key rows) with
//                         weights of that size, a query factor that grows with the position, the
//                         first `rot` dims of each head turned, heads filled up with zeros to the
//                         attention kernels' head size, keys and values written into their pages
//                         (each value head into the pages of `repeat` key heads)
//   differential_combine  o = a1 - lam * a2 of a head's two attention maps, divided by its root
//                         mean square, scaled and gated by a sigmoid per head
//
// The streams, the sums, the norms, the angles and the gates are float32 arithmetic whatever the
// types of the tensors are; values are rounded once when they are stored in the compute dtype.
#include "common.cuh"
#include "kernels.h"

namespace lse {

#define LSE_CHECK_LAUNCH() (cudaPeekAtLastError() == cudaSuccess ? LSE_OK : LSE_LAUNCH_FAILED)

constexpr int SM_MAX_STREAMS = 16;
constexpr int SM_THREADS = 256;

// ------------------------------------------------------------------------------------ spread
__global__ void streams_spread_kernel(const float* __restrict__ x, float* __restrict__ out, int W, int S,
                                      float scale, long long n) {
  pdl_trigger();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const long long t = i / W;
  const int c = (int)(i - t * W);
  const float v = x[i] * scale;
  float* dst = out + t * (long long)S * W + c;
  for (int s = 0; s < S; ++s) dst[(size_t)s * W] = v;
}

template <typename T, int V>
__device__ __forceinline__ void ld_vec(const T* p, float (&v)[V]) {
  if constexpr (V == 4) load4<T>(p, v);
  else v[0] = Num<T>::to_float(p[0]);
}
template <typename T, int V>
__device__ __forceinline__ void st_vec(T* p, const float (&v)[V]) {
  if constexpr (V == 4) store4<T>(p, v);
  else p[0] = Num<T>::from_float(v[0]);
}

// ------------------------------------------------------------------------------------ read + norm
// One block per output row; u is kept in shared memory between the two visits.
template <typename TO, int V>
__global__ void __launch_bounds__(SM_THREADS)
streams_read_norm_kernel(const float* __restrict__ x, const float* __restrict__ read,
                         const float* __restrict__ w, float eps, TO* __restrict__ out,
                         const int* __restrict__ rows, int W, int S) {
  extern __shared__ __align__(16) float u_row[];  // [W]
  __shared__ float scratch[32];
  __shared__ float rd[SM_MAX_STREAMS];
  pdl_trigger();
  if (threadIdx.x < S) rd[threadIdx.x] = read[threadIdx.x];
  __syncthreads();
  pdl_wait();
  const size_t t = rows ? (size_t)rows[blockIdx.x] : (size_t)blockIdx.x;
  const float* xr = x + t * (size_t)S * W;
  float ss = 0.f;
  for (int i = threadIdx.x * V; i < W; i += SM_THREADS * V) {
    float u[V];
#pragma unroll
    for (int j = 0; j < V; ++j) u[j] = 0.f;
    for (int s = 0; s < S; ++s) {
      float xv[V];
      ld_vec<float, V>(xr + (size_t)s * W + i, xv);
#pragma unroll
      for (int j = 0; j < V; ++j) u[j] = fmaf(rd[s], xv[j], u[j]);
    }
#pragma unroll
    for (int j = 0; j < V; ++j) {
      ss += u[j] * u[j];
      u_row[i + j] = u[j];
    }
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)W + eps);
  TO* o = out + (size_t)blockIdx.x * W;
  for (int i = threadIdx.x * V; i < W; i += SM_THREADS * V) {
    float u[V], wv[V];
    ld_vec<float, V>(u_row + i, u);  // this thread's own writes
    ld_vec<float, V>(w + i, wv);
#pragma unroll
    for (int j = 0; j < V; ++j) u[j] *= inv * wv[j];
    st_vec<TO, V>(o + i, u);
  }
}

// ------------------------------------------------------------------------------------ write (+ read + norm)
// One block per token. TY: the sublayer's result as float32, bfloat16, or the fixed-point sums of
// a few-rows product (taken: zeros are left behind).
// MS: the most streams this instantiation holds in registers (S <= MS).
template <typename TY, typename TO, int V, int MS>
__global__ void __launch_bounds__(SM_THREADS)
streams_write_kernel(float* __restrict__ x, const TY* y, const float* __restrict__ scale,
                     const float* __restrict__ mix, const float* __restrict__ outw, int W, int S,
                     const float* __restrict__ then_read, const float* __restrict__ then_w, float then_eps,
                     TO* __restrict__ out) {
  extern __shared__ __align__(16) float u_row[];  // [W], only with then_read
  __shared__ float scratch[32];
  __shared__ float m[SM_MAX_STREAMS * SM_MAX_STREAMS], ow[SM_MAX_STREAMS], rd[SM_MAX_STREAMS];
  pdl_trigger();
  if (threadIdx.x < S * S) m[threadIdx.x] = mix[threadIdx.x];
  if (threadIdx.x < S) {
    ow[threadIdx.x] = outw[threadIdx.x];
    rd[threadIdx.x] = then_read ? then_read[threadIdx.x] : 0.f;
  }
  __syncthreads();
  pdl_wait();
  const size_t t = blockIdx.x;
  float* xr = x + t * (size_t)S * W;
  const TY* yr = y + t * (size_t)W;
  float ss = 0.f;
  for (int i = threadIdx.x * V; i < W; i += SM_THREADS * V) {
    float xs[MS][V], yv[V];
#pragma unroll
    for (int s = 0; s < MS; ++s)
      if (s < S) ld_vec<float, V>(xr + (size_t)s * W + i, xs[s]);
    ld_vec<TY, V>(yr + i, yv);
    if (scale) {
      float sv[V];
      ld_vec<float, V>(scale + i, sv);
#pragma unroll
      for (int j = 0; j < V; ++j) yv[j] *= sv[j];
    }
    float u[V];
#pragma unroll
    for (int j = 0; j < V; ++j) u[j] = 0.f;
#pragma unroll
    for (int r = 0; r < MS; ++r) {
      if (r < S) {
        float nv[V];
#pragma unroll
        for (int j = 0; j < V; ++j) nv[j] = ow[r] * yv[j];
#pragma unroll
        for (int s = 0; s < MS; ++s)
          if (s < S) {
#pragma unroll
            for (int j = 0; j < V; ++j) nv[j] = fmaf(m[s * S + r], xs[s][j], nv[j]);
          }
        st_vec<float, V>(xr + (size_t)r * W + i, nv);
#pragma unroll
        for (int j = 0; j < V; ++j) u[j] = fmaf(rd[r], nv[j], u[j]);
      }
    }
    if (then_read) {
#pragma unroll
      for (int j = 0; j < V; ++j) {
        ss += u[j] * u[j];
        u_row[i + j] = u[j];
      }
    }
  }
  if (!then_read) return;
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)W + then_eps);
  TO* o = out + t * (size_t)W;
  for (int i = threadIdx.x * V; i < W; i += SM_THREADS * V) {
    float u[V], wv[V];
    ld_vec<float, V>(u_row + i, u);
    ld_vec<float, V>(then_w + i, wv);
#pragma unroll
    for (int j = 0; j < V; ++j) u[j] *= inv * wv[j];
    st_vec<TO, V>(o + i, u);
  }
}

// ------------------------------------------------------------------------------------ q, k, v of a token
struct QkvRowsArgs {
  const float* proj;  // [T, stride]: q heads (nq x D), k heads (nk x D), then nv value heads of Dv
  long long stride;
  int nq, nk, nv;     // nv == 0: a key head's value is the key as projected
  int D, Dv, Dp;      // sizes in the projection, and of a head in q_out and in the pages
  const float* qw;    // [nq * D], [nk * D] or both null
  const float* kw;
  float eps;
  float temp_coef;    // q *= 1 + temp_coef * ln(floor((pos + 1) / temp_every) + 1), if temp_every > 0
  int temp_every;
  const int* positions;
  const int* token_seq;
  const float* cos;   // [positions, rot / 2] or null
  const float* sin;
  int rot;
  void* q_out;        // [T, nq * Dp]
  void* k_pages;      // [pages, nk, page_tokens, Dp], or both null
  void* v_pages;
  const int* block_tables;
  int table_stride, page_tokens;
};

// One token per blockIdx.x; the token's heads are shared by the gridDim.y blocks of that token (few
// tokens: many blocks each), every one of which forms the two sums of squares itself. A thread's
// unit of work is VEC consecutive dims of one head (4: every row, head and rotated half holds
// whole 16-byte vectors; 1: any sizes). STAGED: the token's query and key rows are brought into
// shared memory once, while their squares are summed, and everything after (values, rotation
// partners, the values that are keys) is read from there; otherwise the rows are read for the
// sums and read again from cache (rows beyond the shared memory's size). Keeping a thread's
// values in registers between the two visits instead (eight vectors, 78 registers, three blocks
// an SM instead of six) was slower than reading twice: 135 against 108 us on 8192 tokens.
template <typename T, int VEC, bool STAGED>
__global__ void __launch_bounds__(SM_THREADS) qkv_norm_rope_write_kernel(const QkvRowsArgs a) {
  extern __shared__ __align__(16) float staged_rows[];  // STAGED: (nq + nk) * D values (nq * D without pages)
  __shared__ float scratch[32];
  pdl_trigger();
  const int t = blockIdx.x;
  const int pos = a.positions[t];
  const int D = a.D, Dp = a.Dp, nq = a.nq, nk = a.nk;
  size_t page_row = 0;  // of key head 0 of this token, in units of Dp
  if (a.k_pages) {
    const int pi = pos / a.page_tokens, off = pos - pi * a.page_tokens;
    const int page = a.block_tables[(size_t)a.token_seq[t] * a.table_stride + pi];
    page_row = (size_t)page * nk * a.page_tokens + off;
  }
  pdl_wait();
  const float* row = a.proj + (size_t)t * a.stride;
  const float* qk = STAGED ? staged_rows : row;  // where the query and key rows are read from
  float inv_q = 1.f, inv_k = 1.f;
  if constexpr (STAGED) {
    float sq = 0.f, sk = 0.f;
    const int n_q = nq * D, n_all = (a.k_pages ? nq + nk : nq) * D;
    for (int i = threadIdx.x * VEC; i < n_all; i += SM_THREADS * VEC) {
      float v[VEC];
      ld_vec<float, VEC>(row + i, v);
      st_vec<float, VEC>(staged_rows + i, v);
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < VEC; ++j) ss += v[j] * v[j];
      if (i < n_q) sq += ss;  // a vector lies in the query rows or in the key rows, never across
      else sk += ss;
    }
    if (a.qw) {
      sq = block_sum(sq, scratch);
      sk = block_sum(sk, scratch);
      inv_q = rsqrtf(sq / (float)(nq * D) + a.eps);
      inv_k = rsqrtf(sk / (float)(nk * D) + a.eps);
    } else {
      __syncthreads();
    }
  } else if (a.qw) {
    float sq = 0.f, sk = 0.f;
    for (int i = threadIdx.x * VEC; i < nq * D; i += SM_THREADS * VEC) {
      float v[VEC];
      ld_vec<float, VEC>(row + i, v);
#pragma unroll
      for (int j = 0; j < VEC; ++j) sq += v[j] * v[j];
    }
    for (int i = threadIdx.x * VEC; i < nk * D; i += SM_THREADS * VEC) {
      float v[VEC];
      ld_vec<float, VEC>(row + nq * D + i, v);
#pragma unroll
      for (int j = 0; j < VEC; ++j) sk += v[j] * v[j];
    }
    sq = block_sum(sq, scratch);
    sk = block_sum(sk, scratch);
    inv_q = rsqrtf(sq / (float)(nq * D) + a.eps);
    inv_k = rsqrtf(sk / (float)(nk * D) + a.eps);
  }
  if (a.temp_every > 0) inv_q *= 1.f + a.temp_coef * logf((float)((pos + 1) / a.temp_every) + 1.f);
  const int half = a.rot / 2;
  const float* cr = a.cos ? a.cos + (size_t)pos * half : nullptr;
  const float* sr = a.cos ? a.sin + (size_t)pos * half : nullptr;
  T* q_out = (T*)a.q_out + (size_t)t * nq * Dp;
  T* k_pages = (T*)a.k_pages;
  T* v_pages = (T*)a.v_pages;
  const int per_head = Dp / VEC;
  const int qk_units = (a.k_pages ? nq + nk : nq) * per_head;
  const int units = qk_units + (a.v_pages ? nk * per_head : 0);
  const int repeat = a.nv > 0 ? nk / a.nv : 1;
  for (int u = blockIdx.y * SM_THREADS + threadIdx.x; u < units; u += gridDim.y * SM_THREADS) {
    float v[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) v[j] = 0.f;
    if (u < qk_units) {
      const int h = u / per_head, i = (u - h * per_head) * VEC;
      const bool is_q = h < nq;
      if (i < D) {
        const float* src = qk + (size_t)h * D;  // the key heads follow the query heads
        const float* w = a.qw ? (is_q ? a.qw + (size_t)h * D : a.kw + (size_t)(h - nq) * D) : nullptr;
        const float inv = is_q ? inv_q : inv_k;
        ld_vec<float, VEC>(src + i, v);
        if (w) {
          float wv[VEC];
          ld_vec<float, VEC>(w + i, wv);
#pragma unroll
          for (int j = 0; j < VEC; ++j) v[j] *= wv[j];
        }
#pragma unroll
        for (int j = 0; j < VEC; ++j) v[j] *= inv;
        if (i < a.rot) {
          const int ip = i < half ? i + half : i - half, f = i < half ? i : i - half;
          float vp[VEC], c[VEC], sn[VEC];
          ld_vec<float, VEC>(src + ip, vp);
          if (w) {
            float wv[VEC];
            ld_vec<float, VEC>(w + ip, wv);
#pragma unroll
            for (int j = 0; j < VEC; ++j) vp[j] *= wv[j];
          }
          ld_vec<float, VEC>(cr + f, c);
          ld_vec<float, VEC>(sr + f, sn);
#pragma unroll
          for (int j = 0; j < VEC; ++j) {
            const float p = vp[j] * inv;
            v[j] = i < half ? v[j] * c[j] - p * sn[j] : v[j] * c[j] + p * sn[j];
          }
        }
      }
      T* dst = is_q ? q_out + (size_t)h * Dp + i : k_pages + (page_row + (size_t)(h - nq) * a.page_tokens) * Dp + i;
      st_vec<T, VEC>(dst, v);
    } else {
      const int uv = u - qk_units;
      const int h = uv / per_head, i = (uv - h * per_head) * VEC;
      if (a.nv == 0) {
        if (i < D) ld_vec<float, VEC>(qk + (size_t)(nq + h) * D + i, v);
      } else if (i < a.Dv) {
        ld_vec<float, VEC>(row + (size_t)(nq + nk) * D + (size_t)(h / repeat) * a.Dv + i, v);
      }
      st_vec<T, VEC>(v_pages + (page_row + (size_t)h * a.page_tokens) * Dp + i, v);
    }
  }
}

// ------------------------------------------------------------------------------------ differential combine
// One warp per (token, head). a [T, 2H * Dp] holds, for key group g (n heads each), the n heads'
// first maps and then their second maps; out [T, H * Dv].
constexpr int DC_WARPS = 4;
template <typename TA, typename TO>
__global__ void differential_combine_kernel(const TA* __restrict__ a, const float* __restrict__ gate,
                                            long long gate_stride, int H, int n, int Dp, int Dv, float lam,
                                            float eps, float out_scale, TO* __restrict__ out, int T) {
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long th = (long long)blockIdx.x * DC_WARPS + warp;
  if (th >= (long long)T * H) return;
  const int t = (int)(th / H), h = (int)(th - (long long)t * H);
  const int g = h / n, r = h - g * n;
  const TA* a1 = a + ((size_t)t * 2 * H + (size_t)(2 * g) * n + r) * Dp;
  const TA* a2 = a1 + (size_t)n * Dp;
  float o[8];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const int i = lane + 32 * c;
    o[c] = i < Dv ? Num<TA>::to_float(a1[i]) - lam * Num<TA>::to_float(a2[i]) : 0.f;
    ss += o[c] * o[c];
  }
  ss = warp_sum(ss);
  const float z = gate[(size_t)t * gate_stride + h];
  const float f = rsqrtf(ss / (float)Dv + eps) * out_scale / (1.f + expf(-z));
  TO* dst = out + ((size_t)t * H + h) * Dv;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const int i = lane + 32 * c;
    if (i < Dv) dst[i] = Num<TO>::from_float(o[c] * f);
  }
}

}  // namespace lse

using namespace lse;

extern "C" int lse_streams_spread(const float* x, float* out, int T, int W, int S, float scale,
                                  cudaStream_t stream) {
  if (T <= 0) return LSE_OK;
  if (W <= 0 || S <= 0) return LSE_BAD_ARGUMENT;
  const long long n = (long long)T * W;
  launch(streams_spread_kernel, (unsigned)((n + 255) / 256), 256, 0, stream, x, out, W, S, scale, n);
  return LSE_CHECK_LAUNCH();
}

// Rows of up to this many floats are kept in shared memory between a block's two visits.
static const int kStreamsMaxWidth = 48 * 1024;

template <typename K>
static int allow_row(K kernel, size_t bytes) {
  if (bytes <= 48 * 1024) return LSE_OK;
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 192 * 1024) == cudaSuccess
             ? LSE_OK
             : LSE_LAUNCH_FAILED;
}

extern "C" int lse_streams_read_norm(const float* x, const float* read, const float* w, float eps, void* out,
                                     int out_dtype, const int* rows, int n_rows, int W, int S,
                                     cudaStream_t stream) {
  if (n_rows <= 0) return LSE_OK;
  if (W <= 0 || W > kStreamsMaxWidth || S <= 0 || S > SM_MAX_STREAMS) return LSE_BAD_ARGUMENT;
  const size_t smem = (size_t)W * sizeof(float);
  const bool wide = W % 4 == 0;
#define LSE_RN(TO, V)                                                                                   \
  do {                                                                                                  \
    if (allow_row(streams_read_norm_kernel<TO, V>, smem) != LSE_OK) return LSE_LAUNCH_FAILED;           \
    launch(streams_read_norm_kernel<TO, V>, n_rows, SM_THREADS, smem, stream, x, read, w, eps, (TO*)out, \
           rows, W, S);                                                                                 \
  } while (0)
  if (out_dtype == LSE_BF16) {
    if (wide) LSE_RN(bf16, 4); else LSE_RN(bf16, 1);
  } else if (out_dtype == LSE_F32) {
    if (wide) LSE_RN(float, 4); else LSE_RN(float, 1);
  } else {
    return LSE_BAD_ARGUMENT;
  }
#undef LSE_RN
  return LSE_CHECK_LAUNCH();
}

extern "C" int lse_streams_write(float* x, const void* y, int y_dtype, const float* scale, const float* mix,
                                 const float* outw, int T, int W, int S, const float* then_read,
                                 const float* then_w, float then_eps, void* out, int out_dtype,
                                 cudaStream_t stream) {
  if (T <= 0) return LSE_OK;
  if (W <= 0 || W > kStreamsMaxWidth || S <= 0 || S > SM_MAX_STREAMS || (then_read && (!then_w || !out)))
    return LSE_BAD_ARGUMENT;
  // more than eight streams: an element per thread (sixteen 16-byte vectors would not fit the registers)
  const bool wide = W % 4 == 0 && (S <= 8 || y_dtype == LSE_FIXED64);
  if (y_dtype == LSE_FIXED64 && W % 4 != 0) return LSE_BAD_ARGUMENT;
  const size_t smem = then_read ? (size_t)W * sizeof(float) : 0;
  if (!then_read) out_dtype = LSE_F32;
#define LSE_SW_MS(TY, TO, V, MS)                                                                                \
  do {                                                                                                          \
    if (allow_row(streams_write_kernel<TY, TO, V, MS>, smem) != LSE_OK) return LSE_LAUNCH_FAILED;               \
    launch(streams_write_kernel<TY, TO, V, MS>, T, SM_THREADS, smem, stream, x, (const TY*)y, scale, mix, outw, \
           W, S, then_read, then_w, then_eps, (TO*)out);                                                        \
  } while (0)
#define LSE_SW(TY, TO, V)                                   \
  do {                                                      \
    if (V == 4 && S <= 2) LSE_SW_MS(TY, TO, V, 2);          \
    else if (V == 4 && S <= 4) LSE_SW_MS(TY, TO, V, 4);     \
    else if (S <= 8) LSE_SW_MS(TY, TO, V, 8);               \
    else LSE_SW_MS(TY, TO, V, SM_MAX_STREAMS);              \
  } while (0)
#define LSE_SW_OUT(TY, V)                              \
  do {                                                 \
    if (out_dtype == LSE_BF16) LSE_SW(TY, bf16, V);    \
    else if (out_dtype == LSE_F32) LSE_SW(TY, float, V); \
    else return LSE_BAD_ARGUMENT;                      \
  } while (0)
  if (y_dtype == LSE_F32) {
    if (wide) LSE_SW_OUT(float, 4); else LSE_SW_OUT(float, 1);
  } else if (y_dtype == LSE_BF16) {
    if (wide) LSE_SW_OUT(bf16, 4); else LSE_SW_OUT(bf16, 1);
  } else if (y_dtype == LSE_FIXED64) {
    LSE_SW_OUT(fixed64, 4);
  } else {
    return LSE_BAD_ARGUMENT;
  }
#undef LSE_SW_OUT
#undef LSE_SW
#undef LSE_SW_MS
  return LSE_CHECK_LAUNCH();
}

extern "C" int lse_qkv_norm_rope_write(const float* proj, long long stride, int T, int nq, int nk, int nv,
                                       int D, int Dv, int Dp, const float* qw, const float* kw, float eps,
                                       float temp_coef, int temp_every, const int* positions,
                                       const int* token_seq, const float* cos, const float* sin, int rot,
                                       void* q_out, void* k_pages, void* v_pages, int dtype,
                                       const int* block_tables, int table_stride, int page_tokens,
                                       cudaStream_t stream) {
  if (T <= 0) return LSE_OK;
  if (nq <= 0 || nk <= 0 || nv < 0 || (nv > 0 && nk % nv) || D <= 0 || Dp < D || (nv > 0 && (Dv <= 0 || Dp < Dv)) ||
      (!qw != !kw) || (!cos != !sin) || (!k_pages != !v_pages) || rot < 0 || rot > D || rot % 2 || (rot && !cos) ||
      page_tokens <= 0 || temp_every < 0 || stride < (long long)(nq + nk) * D + (long long)nv * Dv)
    return LSE_BAD_ARGUMENT;
  QkvRowsArgs a;
  a.proj = proj; a.stride = stride; a.nq = nq; a.nk = nk; a.nv = nv; a.D = D; a.Dv = Dv; a.Dp = Dp;
  a.qw = qw; a.kw = kw; a.eps = eps; a.temp_coef = temp_coef; a.temp_every = temp_every;
  a.positions = positions; a.token_seq = token_seq; a.cos = cos; a.sin = sin; a.rot = cos ? rot : 0;
  a.q_out = q_out; a.k_pages = k_pages; a.v_pages = v_pages; a.block_tables = block_tables;
  a.table_stride = table_stride; a.page_tokens = page_tokens;
  // whole 16-byte vectors everywhere: rows, heads, value heads, rotated halves, cos/sin rows
  const bool wide = stride % 4 == 0 && D % 4 == 0 && Dp % 4 == 0 && (nv == 0 || Dv % 4 == 0) && a.rot % 8 == 0;
  const int units = ((k_pages ? nq + nk : nq) + (v_pages ? nk : 0)) * (Dp / (wide ? 4 : 1));
  // few tokens: a token's heads are shared by several blocks, up to about four blocks per SM in all
  int parts = (600 + T - 1) / T;
  const int most = (units + SM_THREADS - 1) / SM_THREADS;
  if (parts > most) parts = most;
  if (parts < 1) parts = 1;
  const dim3 grid(T, parts);
  // the token's query and key rows in shared memory, where they fit beside five more blocks of an SM
  const size_t smem = (size_t)(k_pages ? nq + nk : nq) * D * sizeof(float);
  const bool staged = smem <= 36 * 1024;
#define LSE_QKV(TT, V)                                                                                       \
  do {                                                                                                       \
    if (staged) launch(qkv_norm_rope_write_kernel<TT, V, true>, grid, SM_THREADS, smem, stream, a);          \
    else launch(qkv_norm_rope_write_kernel<TT, V, false>, grid, SM_THREADS, 0, stream, a);                   \
  } while (0)
  if (dtype == LSE_BF16) {
    if (wide) LSE_QKV(bf16, 4); else LSE_QKV(bf16, 1);
  } else if (dtype == LSE_F32) {
    if (wide) LSE_QKV(float, 4); else LSE_QKV(float, 1);
  } else {
    return LSE_BAD_ARGUMENT;
  }
#undef LSE_QKV
  return LSE_CHECK_LAUNCH();
}

extern "C" int lse_differential_combine(const void* a, int a_dtype, const float* gate, long long gate_stride,
                                        int T, int H, int n, int Dp, int Dv, float lam, float eps,
                                        float out_scale, void* out, int out_dtype, cudaStream_t stream) {
  if (T <= 0) return LSE_OK;
  if (H <= 0 || n <= 0 || H % n || Dv <= 0 || Dv > 256 || Dp < Dv) return LSE_BAD_ARGUMENT;
  const unsigned blocks = (unsigned)(((long long)T * H + DC_WARPS - 1) / DC_WARPS);
#define LSE_DC(TA, TO)                                                                                        \
  launch(differential_combine_kernel<TA, TO>, blocks, DC_WARPS * 32, 0, stream, (const TA*)a, gate, gate_stride, \
         H, n, Dp, Dv, lam, eps, out_scale, (TO*)out, T)
  if (a_dtype == LSE_BF16 && out_dtype == LSE_BF16) LSE_DC(bf16, bf16);
  else if (a_dtype == LSE_F32 && out_dtype == LSE_F32) LSE_DC(float, float);
  else if (a_dtype == LSE_F32 && out_dtype == LSE_BF16) LSE_DC(float, bf16);
  else return LSE_BAD_ARGUMENT;
#undef LSE_DC
  return LSE_CHECK_LAUNCH();
}
