// Kernels of latent attention whose keys carry a rotated part, of output gates and of plain
// (ungated) activations.
//
//   latent_rope_write   per token: the key/value latent RMS-normed and, behind it, the key part
//                       that all heads share, turned by the token's position (neighbouring dims
//                       are a pair), both into the token's row of its page; and the query latent
//                       RMS-normed into a dense tensor
//   latent_query_rope   per token and head: the head's rotated query dims turned by the position
//                       and placed behind the head's latent-space query; the row's padding zeroed
//   sigmoid_gate_mul    o[t, i] *= sigmoid(g[t, col0 + i / group])
//   act_rows            out = act(in) element by element (act: the square of relu, relu, gelu_tanh, silu)
//
// Norms, angles, rotations, sigmoids and activations are float32 arithmetic whatever the types
// of the tensors are.
#include <type_traits>

#include "common.cuh"
#include "kernels.h"

namespace lse {

// Turn the pair (u, v) = (x[2i], x[2i+1]) by the angle of (pos, i): cos/sin [positions, rot/2].
__device__ __forceinline__ float rotated_neighbour(const float* x, int i, int rot, const float* cr,
                                                   const float* sr) {
  if (i >= rot) return x[i];
  const int p = i >> 1;
  return (i & 1) ? x[i] * cr[p] + x[i - 1] * sr[p] : x[i] * cr[p] - x[i + 1] * sr[p];
}

constexpr int LRW_THREADS = 128;

// One block per token. proj row: [.. q latent at q_col0 (Rq dims) .. kv latent at kv_col0 (R dims)
// followed by the shared key part (Dr dims) ..]. Rq = 0: no query latent; R = 0: no key/value side
// (a layer that reads rows another layer wrote).
template <typename TIn, typename T>
__global__ void __launch_bounds__(LRW_THREADS)
latent_rope_write_kernel(const TIn* __restrict__ proj, long long stride, int q_col0, int Rq,
                         const float* __restrict__ q_weight, T* __restrict__ cq, int kv_col0, int R,
                         int Dr, int rot, const float* __restrict__ kv_weight, float eps,
                         const float* __restrict__ cos, const float* __restrict__ sin,
                         T* __restrict__ pages, int Rp, const int* __restrict__ positions,
                         const int* __restrict__ token_seq, const int* __restrict__ block_tables,
                         int table_stride, int page_tokens) {
  pdl_trigger();
  pdl_wait();  // everything below reads what kernels before this one wrote
  __shared__ float red[32];
  extern __shared__ float kr[];  // [Dr] the key part as projected
  const int t = blockIdx.x;
  const TIn* row = proj + (size_t)t * stride;
  if (Rq > 0) {
    const TIn* src = row + q_col0;
    float ss = 0.f;
    for (int i = threadIdx.x; i < Rq; i += LRW_THREADS) {
      const float v = Num<TIn>::to_float(src[i]);
      ss += v * v;
    }
    ss = block_sum(ss, red);
    const float r = rsqrtf(ss / (float)Rq + eps);
    T* dst = cq + (size_t)t * Rq;
    for (int i = threadIdx.x; i < Rq; i += LRW_THREADS)
      dst[i] = Num<T>::from_float(Num<TIn>::to_float(src[i]) * r * q_weight[i]);
  }
  if (R <= 0) return;
  const TIn* src = row + kv_col0;
  float ss = 0.f;
  for (int i = threadIdx.x; i < R; i += LRW_THREADS) {
    const float v = Num<TIn>::to_float(src[i]);
    ss += v * v;
  }
  for (int i = threadIdx.x; i < Dr; i += LRW_THREADS) kr[i] = Num<TIn>::to_float(src[R + i]);
  ss = block_sum(ss, red);  // its barriers also publish kr
  const float r = rsqrtf(ss / (float)R + eps);
  const int pos = positions[t];
  const int page = block_tables[(size_t)token_seq[t] * table_stride + pos / page_tokens];
  T* dst = pages + ((size_t)page * page_tokens + pos % page_tokens) * Rp;
  const float* cr = cos + (size_t)pos * (rot / 2);
  const float* sr = sin + (size_t)pos * (rot / 2);
  for (int i = threadIdx.x; i < Rp; i += LRW_THREADS) {
    float v = 0.f;
    if (i < R) v = Num<TIn>::to_float(src[i]) * r * kv_weight[i];
    else if (i < R + Dr) v = rotated_neighbour(kr, i - R, rot, cr, sr);
    dst[i] = Num<T>::from_float(v);
  }
}

// A token per blockIdx.x; one thread per (head, two neighbouring dims behind the head's
// latent-space query). q row: heads of (D + Dr) dims, the last Dr to be rotated. out row: heads of
// Rp dims; dims [R, R + Dr) receive the rotated part, [R + Dr, Rp) zeros. Dims [0, R) are written
// by the per-head product that runs beside this kernel. PAIRS: D, Dr, R and Rp are even, so that a
// pair is one aligned 4- or 8-byte access on both sides.
template <typename T, bool PAIRS>
__global__ void __launch_bounds__(256)
latent_query_rope_kernel(const T* __restrict__ q, int H, int D, int Dr, int rot,
                         const float* __restrict__ cos, const float* __restrict__ sin,
                         const int* __restrict__ positions, T* __restrict__ out, int R, int Rp,
                         int pairs) {
  pdl_trigger();
  pdl_wait();  // everything below reads what kernels before this one wrote
  const int idx = blockIdx.y * blockDim.x + threadIdx.x;
  if (idx >= H * pairs) return;
  const int h = idx / pairs, p = idx - h * pairs;
  const size_t th = (size_t)blockIdx.x * H + h;
  const int i = 2 * p, n = Rp - R;
  const T* src = q + th * (D + Dr) + D + i;
  T* dst = out + th * Rp + R + i;
  float u = 0.f, v = 0.f;
  if (PAIRS) {
    if (i < Dr) {  // Dr is even: the pair's second dim is inside too
      if constexpr (sizeof(T) == 2) {
        const __nv_bfloat162 t = *reinterpret_cast<const __nv_bfloat162*>(src);
        u = __low2float(t);
        v = __high2float(t);
      } else {
        const float2 t = *reinterpret_cast<const float2*>(src);
        u = t.x;
        v = t.y;
      }
    }
  } else {
    if (i < Dr) u = Num<T>::to_float(src[0]);
    if (i + 1 < Dr) v = Num<T>::to_float(src[1]);
  }
  if (i < rot) {  // rot is even and at most Dr
    const size_t at = (size_t)positions[blockIdx.x] * (rot / 2) + p;
    const float c = cos[at], sn = sin[at];
    const float ru = u * c - v * sn;
    v = v * c + u * sn;
    u = ru;
  }
  if (PAIRS) {
    if constexpr (sizeof(T) == 2) *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(u, v);
    else *reinterpret_cast<float2*>(dst) = make_float2(u, v);
  } else {
    dst[0] = Num<T>::from_float(u);
    if (i + 1 < n) dst[1] = Num<T>::from_float(v);
  }
}

// The same for bfloat16 rows whose pieces (D, Dr, rot, R, Rp) are all multiples of 8: one thread per
// (head, 16-byte vector of eight dims), which is rotated whole, copied whole or zero.
__global__ void __launch_bounds__(256)
latent_query_rope_wide_kernel(const bf16* __restrict__ q, int H, int D, int Dr, int rot,
                              const float* __restrict__ cos, const float* __restrict__ sin,
                              const int* __restrict__ positions, bf16* __restrict__ out, int R, int Rp,
                              int vectors) {
  pdl_trigger();
  pdl_wait();  // everything below reads what kernels before this one wrote
  const int idx = blockIdx.y * blockDim.x + threadIdx.x;
  if (idx >= H * vectors) return;
  const int h = idx / vectors, i = 8 * (idx - h * vectors);
  const size_t th = (size_t)blockIdx.x * H + h;
  Vec16<bf16> v;
  if (i < Dr) {
    v = load16(q + th * (D + Dr) + D + i);
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) v.v[j] = __float2bfloat16_rn(0.f);
  }
  if (i < rot) {
    const size_t at = (size_t)positions[blockIdx.x] * (rot / 2) + i / 2;
    float c[4], sn[4];
    load4<float>(cos + at, c);
    load4<float>(sin + at, sn);
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      const float u = __bfloat162float(v.v[2 * p]), w = __bfloat162float(v.v[2 * p + 1]);
      v.v[2 * p] = __float2bfloat16_rn(u * c[p] - w * sn[p]);
      v.v[2 * p + 1] = __float2bfloat16_rn(w * c[p] + u * sn[p]);
    }
  }
  store16(out + th * Rp + R + i, v);
}

// A row per blockIdx.x, the row's columns over blockIdx.y and the threads. VEC4: four neighbouring
// columns per thread (N a multiple of 4, o 16-byte aligned).
template <typename T, typename TG, bool VEC4>
__global__ void __launch_bounds__(256)
sigmoid_gate_mul_kernel(T* __restrict__ o, const TG* __restrict__ g, long long g_stride, int col0,
                        int group, int N) {
  pdl_trigger();
  pdl_wait();  // everything below reads what kernels before this one wrote
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * (VEC4 ? 4 : 1);
  if (c >= N) return;
  const size_t t = blockIdx.x;
  const TG* gr = g + t * g_stride + col0;
  T* op = o + t * N + c;
  int gi = c / group;
  if (VEC4) {
    float v[4];
    load4<T>(op, v);
    int left = group - (c - gi * group);  // columns of this thread's first gate that are still to come
    float sg = 1.f / (1.f + expf(-Num<TG>::to_float(gr[gi])));
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (left == 0) {
        sg = 1.f / (1.f + expf(-Num<TG>::to_float(gr[++gi])));
        left = group;
      }
      v[j] *= sg;
      --left;
    }
    store4<T>(op, v);
  } else {
    const float z = Num<TG>::to_float(gr[gi]);
    *op = Num<T>::from_float(Num<T>::to_float(*op) / (1.f + expf(-z)));
  }
}

__device__ __forceinline__ float plain_activation(float z, int act) {
  switch (act) {
    case 0: {  // the square of relu
      const float r = fmaxf(z, 0.f);
      return r * r;
    }
    case 1: return fmaxf(z, 0.f);
    case 2: return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    default: return z / (1.f + expf(-z));
  }
}

// VEC4: four elements per thread (total a multiple of 4, both tensors 16-byte aligned). Fixed-point
// sums are taken as they are read: zeros are left behind for the next sums.
template <typename TIn, typename T, bool VEC4>
__global__ void __launch_bounds__(256)
act_rows_kernel(const TIn* __restrict__ in, T* __restrict__ out, long long total, int act) {
  pdl_trigger();
  pdl_wait();  // everything below reads what kernels before this one wrote
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * (VEC4 ? 4 : 1);
  if (i >= total) return;
  if (VEC4) {
    float v[4];
    load4<TIn>(in + i, v);
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = plain_activation(v[j], act);
    store4<T>(out + i, v);
  } else {
    out[i] = Num<T>::from_float(plain_activation(Num<TIn>::to_float(in[i]), act));
    if (std::is_same<TIn, fixed64>::value) const_cast<TIn*>(in)[i] = Num<TIn>::from_float(0.f);
  }
}

}  // namespace lse

using namespace lse;

#define LSE_CHECK_LAUNCH() (cudaPeekAtLastError() == cudaSuccess ? LSE_OK : LSE_LAUNCH_FAILED)

extern "C" int lse_latent_rope_write(const void* proj, int in_dtype, long long stride, int q_col0, int Rq,
                                     const float* q_weight, void* cq, int kv_col0, int R, int Dr, int rot,
                                     const float* kv_weight, float eps, const float* cos, const float* sin,
                                     void* pages, int Rp, int dtype, const int* positions,
                                     const int* token_seq, const int* block_tables, int table_stride,
                                     int page_tokens, int T, cudaStream_t stream) {
  if (T <= 0) return LSE_OK;
  if (Rq < 0 || R < 0 || (Rq == 0 && R == 0)) return LSE_BAD_ARGUMENT;
  if (Rq > 0 && (!q_weight || !cq)) return LSE_BAD_ARGUMENT;
  if (R > 0 && (Dr < 0 || rot < 0 || rot > Dr || rot % 2 || Rp < R + Dr || page_tokens <= 0 || !pages ||
                !kv_weight || (rot > 0 && (!cos || !sin))))
    return LSE_BAD_ARGUMENT;
  const size_t smem = (size_t)(Dr > 0 ? Dr : 1) * sizeof(float);
#define LSE_LRW(TIn, T_) \
  launch(latent_rope_write_kernel<TIn, T_>, T, LRW_THREADS, smem, stream, (const TIn*)proj, stride, q_col0, Rq, \
         q_weight, (T_*)cq, kv_col0, R, Dr, rot, kv_weight, eps, cos, sin, (T_*)pages, Rp, positions, token_seq, \
         block_tables, table_stride, page_tokens)
  if (in_dtype == LSE_F32 && dtype == LSE_F32) LSE_LRW(float, float);
  else if (in_dtype == LSE_F32 && dtype == LSE_BF16) LSE_LRW(float, bf16);
  else if (in_dtype == LSE_BF16 && dtype == LSE_BF16) LSE_LRW(bf16, bf16);
  else return LSE_BAD_ARGUMENT;
#undef LSE_LRW
  return LSE_CHECK_LAUNCH();
}

extern "C" int lse_latent_query_rope(const void* q, int dtype, int T, int H, int D, int Dr, int rot,
                                     const float* cos, const float* sin, const int* positions, void* out,
                                     int R, int Rp, cudaStream_t stream) {
  if (T <= 0 || H <= 0) return LSE_OK;
  if (D < 0 || Dr < 0 || rot < 0 || rot > Dr || rot % 2 || Rp < R + Dr || (rot > 0 && (!cos || !sin)))
    return LSE_BAD_ARGUMENT;
  if (Rp == R) return LSE_OK;
  const int pairs = (Rp - R + 1) / 2;
  const dim3 grid(T, (H * pairs + 255) / 256);
  if (grid.y > 65535) return LSE_BAD_ARGUMENT;
  const bool even = D % 2 == 0 && Dr % 2 == 0 && R % 2 == 0 && Rp % 2 == 0 &&
                    reinterpret_cast<uintptr_t>(q) % 8 == 0 && reinterpret_cast<uintptr_t>(out) % 8 == 0;
  auto aligned16 = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  if (dtype == LSE_BF16 && D % 8 == 0 && Dr % 8 == 0 && rot % 8 == 0 && R % 8 == 0 && Rp % 8 == 0 &&
      aligned16(q) && aligned16(out) && aligned16(cos) && aligned16(sin)) {
    const int vectors = (Rp - R) / 8;
    const dim3 wide(T, (H * vectors + 255) / 256);
    if (wide.y > 65535) return LSE_BAD_ARGUMENT;
    launch(latent_query_rope_wide_kernel, wide, 256, 0, stream, (const bf16*)q, H, D, Dr, rot, cos, sin, positions,
           (bf16*)out, R, Rp, vectors);
    return LSE_CHECK_LAUNCH();
  }
#define LSE_LQR(T_, P) \
  launch(latent_query_rope_kernel<T_, P>, grid, 256, 0, stream, (const T_*)q, H, D, Dr, rot, cos, sin, positions, \
         (T_*)out, R, Rp, pairs)
  if (dtype == LSE_F32) {
    if (even) LSE_LQR(float, true); else LSE_LQR(float, false);
  } else if (dtype == LSE_BF16) {
    if (even) LSE_LQR(bf16, true); else LSE_LQR(bf16, false);
  } else {
    return LSE_BAD_ARGUMENT;
  }
#undef LSE_LQR
  return LSE_CHECK_LAUNCH();
}

extern "C" int lse_sigmoid_gate_mul(void* o, int dtype, const void* g, int g_dtype, long long g_stride,
                                    int col0, int group, int T, int N, cudaStream_t stream) {
  if (T <= 0 || N <= 0) return LSE_OK;
  if (group <= 0 || col0 < 0) return LSE_BAD_ARGUMENT;
  const bool vec = N % 4 == 0 && reinterpret_cast<uintptr_t>(o) % 16 == 0;
  const int per_block = 256 * (vec ? 4 : 1);
  const dim3 blocks(T, (N + per_block - 1) / per_block);
  if (blocks.y > 65535) return LSE_BAD_ARGUMENT;
#define LSE_SGM_V(T_, TG, V) \
  launch(sigmoid_gate_mul_kernel<T_, TG, V>, blocks, 256, 0, stream, (T_*)o, (const TG*)g, g_stride, col0, group, N)
#define LSE_SGM(T_, TG) \
  do { \
    if (vec) LSE_SGM_V(T_, TG, true); \
    else LSE_SGM_V(T_, TG, false); \
  } while (0)
  if (dtype == LSE_F32 && g_dtype == LSE_F32) LSE_SGM(float, float);
  else if (dtype == LSE_BF16 && g_dtype == LSE_F32) LSE_SGM(bf16, float);
  else if (dtype == LSE_BF16 && g_dtype == LSE_BF16) LSE_SGM(bf16, bf16);
  else return LSE_BAD_ARGUMENT;
#undef LSE_SGM
#undef LSE_SGM_V
  return LSE_CHECK_LAUNCH();
}

extern "C" int lse_act_rows(const void* in, int in_dtype, void* out, int dtype, long long total, int act,
                            cudaStream_t stream) {
  if (total <= 0) return LSE_OK;
  if (act < 0 || act > 3) return LSE_BAD_ARGUMENT;
  const bool vec = total % 4 == 0 && reinterpret_cast<uintptr_t>(in) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(out) % 16 == 0;
  const long long nblocks = ((vec ? total / 4 : total) + 255) / 256;
  if (nblocks > 0x7fffffffLL) return LSE_BAD_ARGUMENT;
  const unsigned blocks = (unsigned)nblocks;
#define LSE_ACT_V(TIn, T_, V) \
  launch(act_rows_kernel<TIn, T_, V>, blocks, 256, 0, stream, (const TIn*)in, (T_*)out, total, act)
#define LSE_ACT(TIn, T_) \
  do { \
    if (vec) LSE_ACT_V(TIn, T_, true); \
    else LSE_ACT_V(TIn, T_, false); \
  } while (0)
  if (in_dtype == LSE_F32 && dtype == LSE_F32) LSE_ACT(float, float);
  else if (in_dtype == LSE_F32 && dtype == LSE_BF16) LSE_ACT(float, bf16);
  else if (in_dtype == LSE_BF16 && dtype == LSE_BF16) LSE_ACT(bf16, bf16);
  else if (in_dtype == LSE_FIXED64 && dtype == LSE_BF16) LSE_ACT(fixed64, bf16);
  else return LSE_BAD_ARGUMENT;
#undef LSE_ACT
#undef LSE_ACT_V
  return LSE_CHECK_LAUNCH();
}
