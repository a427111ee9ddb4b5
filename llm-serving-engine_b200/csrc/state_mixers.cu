// Kernels of the parts that keep a running state per request, and of blocks that norm a branch's
// output: token shift, linear attention with a decay per head, the grouped norm with a gate that
// follows it, query/key norm with the key/value page write, and "x += norm(branch)".
// All arithmetic is float32; values are rounded once when they are stored in the compute dtype.
//
// A request's state lives in row state_slots[seq] of a [slots, ...] float32 tensor. A sequence
// whose first row of this step is at position 0 starts from zeros, whatever its slot holds.
#include "common.cuh"
#include "kernels.h"

namespace lse {

#define LSE_CHECK_LAUNCH() (cudaPeekAtLastError() == cudaSuccess ? LSE_OK : LSE_LAUNCH_FAILED)

__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }

// ------------------------------------------------------------------------------------ cast
template <typename TO>
__global__ void cast_kernel(const float* __restrict__ x, TO* __restrict__ out, long long n) {
  pdl_trigger();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = Num<TO>::from_float(x[i]);
}

// ------------------------------------------------------------------------------------ token shift
// One block per row. The block of a sequence's first row is the only one that touches the
// sequence's state: each of its threads reads the old value of its elements and then stores the
// sequence's last row of this step there.
template <typename TO>
__global__ void token_shift_kernel(const float* __restrict__ x, const float* __restrict__ mix,
                                   float* state, TO* __restrict__ out,
                                   const int* __restrict__ token_seq, const int* __restrict__ cu_q,
                                   const int* __restrict__ ctx_lens, const int* __restrict__ slots,
                                   int W) {
  pdl_trigger();
  const int t = blockIdx.x;
  const int s = token_seq[t];
  const int r0 = cu_q[s], r1 = cu_q[s + 1];
  const bool first = (t == r0);
  const bool from_zero = first && (ctx_lens[s] - (r1 - r0) == 0);
  float* st = state + (size_t)slots[s] * W;
  pdl_wait();
  const float* cur = x + (size_t)t * W;
  const float* prev = first ? st : cur - W;
  const float* last = x + (size_t)(r1 - 1) * W;
  TO* o = out + (size_t)t * W;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float c = cur[i];
    const float p = from_zero ? 0.f : prev[i];
    if (first) st[i] = last[i];
    o[i] = Num<TO>::from_float(c + (p - c) * mix[i]);
  }
}

// ------------------------------------------------------------------------------------ x += norm(branch)
// One block per row. y = a, or, with inner weights, ca * wa * a / rms(a) (+ cb * wb * b / rms(b));
// then x += w * y / rms(y). out (if given) = the new x in the compute dtype, or, with then_w, the
// next norm of the new x: then_w * x / rms(x), while the block still holds the row. y is
// recomputed in the last pass rather than kept: the row's second read comes from cache, and a
// thread reads back only what it wrote itself. SUMS: a (and b) are the fixed-point sums of a
// few-rows product; they are taken once (converted into shared memory, zeros left behind) and read
// from there. V: elements per thread and visit (4: H a multiple of 4, every row 16-byte aligned).
// K > 0: a thread visits at most K places of the row and keeps y and the new x of each in
// registers, so that a and x are read once and x's old values are already on their way while the
// block sums the squares; K = 0: any row length, y recomputed and x read back.
template <typename TO, bool SUMS, int V, int K>
__global__ void rmsnorm_add_kernel(float* __restrict__ x, const void* a, const void* b,
                                   const float* __restrict__ wa,
                                   const float* __restrict__ wb, float ca, float cb, float eps_in,
                                   const float* __restrict__ w, float eps, TO* __restrict__ out,
                                   const float* __restrict__ then_w, float then_eps, int H) {
  __shared__ float scratch[32];
  extern __shared__ __align__(16) float taken[];  // SUMS: [H] for a, then [H] for b
  pdl_trigger();
  pdl_wait();
  const size_t row = (size_t)blockIdx.x * H;
  const int first = threadIdx.x * V, step = blockDim.x * V;
  auto ld = [](const float* p, float (&v)[V]) {
    if constexpr (V == 4) load4<float>(p, v);
    else v[0] = p[0];
  };
  const float* ar;
  const float* br = nullptr;
  if (SUMS) {
    fixed64* as = reinterpret_cast<fixed64*>(const_cast<void*>(a)) + row;
    fixed64* bs = b ? reinterpret_cast<fixed64*>(const_cast<void*>(b)) + row : nullptr;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      taken[i] = fixed_to_float(as[i]);
      as[i] = 0;
      if (bs) {
        taken[H + i] = fixed_to_float(bs[i]);
        bs[i] = 0;
      }
    }
    __syncthreads();
    ar = taken;
    if (bs) br = taken + H;
  } else {
    ar = reinterpret_cast<const float*>(a) + row;
    if (b) br = reinterpret_cast<const float*>(b) + row;
  }
  float inv_a = 1.f, inv_b = 1.f;
  if (wa) {
    float sa = 0.f, sb = 0.f;
    for (int i = first; i < H; i += step) {
      float va[V];
      ld(ar + i, va);
#pragma unroll
      for (int j = 0; j < V; ++j) sa += va[j] * va[j];
      if (br) {
        float vb[V];
        ld(br + i, vb);
#pragma unroll
        for (int j = 0; j < V; ++j) sb += vb[j] * vb[j];
      }
    }
    sa = block_sum(sa, scratch);
    inv_a = ca * rsqrtf(sa / (float)H + eps_in);
    if (br) {
      sb = block_sum(sb, scratch);
      inv_b = cb * rsqrtf(sb / (float)H + eps_in);
    }
  }
  auto y_at = [&](int i, float (&y)[V]) {
    ld(ar + i, y);
    if (!wa) return;
    float wv[V];
    ld(wa + i, wv);
#pragma unroll
    for (int j = 0; j < V; ++j) y[j] *= inv_a * wv[j];
    if (br) {
      float vb[V];
      ld(br + i, vb);
      ld(wb + i, wv);
#pragma unroll
      for (int j = 0; j < V; ++j) y[j] += vb[j] * inv_b * wv[j];
    }
  };
  auto put = [&](int i, const float (&v)[V]) {
    if constexpr (V == 4) store4<TO>(out + row + i, v);
    else out[row + i] = Num<TO>::from_float(v[0]);
  };
  float* xr = x + row;
  if constexpr (K > 0) {
    float yk[K][V], xk[K][V];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int i = first + k * step;
      if (i < H) {
        y_at(i, yk[k]);
        ld(xr + i, xk[k]);
#pragma unroll
        for (int j = 0; j < V; ++j) ss += yk[k][j] * yk[k][j];
      }
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)H + eps);
    float s2 = 0.f;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int i = first + k * step;
      if (i < H) {
        float wv[V];
        ld(w + i, wv);
#pragma unroll
        for (int j = 0; j < V; ++j) {
          xk[k][j] += yk[k][j] * inv * wv[j];
          s2 += xk[k][j] * xk[k][j];
        }
        if constexpr (V == 4) store4<float>(xr + i, xk[k]);
        else xr[i] = xk[k][0];
        if (out && !then_w) put(i, xk[k]);
      }
    }
    if (!out || !then_w) return;
    s2 = block_sum(s2, scratch);
    const float inv2 = rsqrtf(s2 / (float)H + then_eps);
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int i = first + k * step;
      if (i < H) {
        float wv[V];
        ld(then_w + i, wv);
#pragma unroll
        for (int j = 0; j < V; ++j) xk[k][j] *= inv2 * wv[j];
        put(i, xk[k]);
      }
    }
    return;
  }
  float ss = 0.f;
  for (int i = first; i < H; i += step) {
    float y[V];
    y_at(i, y);
#pragma unroll
    for (int j = 0; j < V; ++j) ss += y[j] * y[j];
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)H + eps);
  float s2 = 0.f;
  for (int i = first; i < H; i += step) {
    float y[V], xv[V], wv[V];
    y_at(i, y);
    ld(xr + i, xv);
    ld(w + i, wv);
#pragma unroll
    for (int j = 0; j < V; ++j) {
      xv[j] += y[j] * inv * wv[j];
      s2 += xv[j] * xv[j];
    }
    if constexpr (V == 4) store4<float>(xr + i, xv);
    else xr[i] = xv[0];
    if (out && !then_w) put(i, xv);
  }
  if (!out || !then_w) return;
  s2 = block_sum(s2, scratch);
  const float inv2 = rsqrtf(s2 / (float)H + then_eps);
  for (int i = first; i < H; i += step) {
    float xv[V], wv[V];
    ld(xr + i, xv);  // this thread's own writes
    ld(then_w + i, wv);
#pragma unroll
    for (int j = 0; j < V; ++j) xv[j] *= inv2 * wv[j];
    put(i, xv);
  }
}

// out = ca * wa * a / rms(a) + cb * wb * b / rms(b)   (b may be null)
__global__ void mix_normed_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                  const float* __restrict__ wa, const float* __restrict__ wb,
                                  float ca, float cb, float eps, float* __restrict__ out, int H) {
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const size_t row = (size_t)blockIdx.x * H;
  float sa = 0.f, sb = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    sa += a[row + i] * a[row + i];
    if (b) sb += b[row + i] * b[row + i];
  }
  sa = block_sum(sa, scratch);
  const float inv_a = ca * rsqrtf(sa / (float)H + eps);
  float inv_b = 0.f;
  if (b) {
    sb = block_sum(sb, scratch);
    inv_b = cb * rsqrtf(sb / (float)H + eps);
  }
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float y = a[row + i] * inv_a * wa[i];
    if (b) y += b[row + i] * inv_b * wb[i];
    out[row + i] = y;
  }
}

// ------------------------------------------------------------------------------------ grouped norm with a gate
// out[t, g*group + i] = o / rms(o over the group) * weight * act(gate); one block per (row, group).
template <typename TO>
__global__ void gated_group_norm_kernel(const float* __restrict__ o, const float* __restrict__ gate,
                                        long long gate_stride, int N, int group,
                                        const float* __restrict__ weight, float eps, int sigmoid,
                                        TO* __restrict__ out) {
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, g = blockIdx.y;
  const float* orow = o + (size_t)t * N + (size_t)g * group;
  const float* grow = gate + (size_t)t * gate_stride + (size_t)g * group;
  float ss = 0.f;
  for (int i = threadIdx.x; i < group; i += blockDim.x) ss += orow[i] * orow[i];
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)group + eps);
  for (int i = threadIdx.x; i < group; i += blockDim.x) {
    float y = orow[i] * inv;
    if (weight) y *= weight[g * group + i];
    const float z = grow[i];
    y *= sigmoid ? sigmoid_f(z) : silu_f(z);
    out[(size_t)t * N + (size_t)g * group + i] = Num<TO>::from_float(y);
  }
}

// ------------------------------------------------------------------------------------ q/k norm, rotation, page write
// One warp per (token, head) of the projection's heads: nq query heads, nk key heads, then nk
// value heads unless the values are the keys as projected. D <= 256.
constexpr int NRW_WARPS = 4;
template <typename T>
__global__ void norm_rope_kv_write_kernel(const float* __restrict__ qkv, T* __restrict__ q_out,
                                          int nq, int nk, int D, int v_from_k,
                                          const float* __restrict__ qw, const float* __restrict__ kw,
                                          float eps, const int* __restrict__ positions,
                                          const int* __restrict__ token_seq,
                                          const float* __restrict__ cos, const float* __restrict__ sin,
                                          T* __restrict__ k_pages, T* __restrict__ v_pages,
                                          const int* __restrict__ block_tables, int table_stride,
                                          int page_tokens, int norm_dim, long long row_stride) {
  __shared__ float buf[NRW_WARPS][256];
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int nv = v_from_k ? 0 : nk;
  const int hs = blockIdx.y * NRW_WARPS + warp;
  if (hs >= nq + nk + nv) return;
  const float* src = qkv + (size_t)t * row_stride + (size_t)hs * D;
  const int pos = positions[t];
  size_t page_base = 0;
  if (hs >= nq) {
    const int pi = pos / page_tokens, off = pos - pi * page_tokens;
    const int page = block_tables[(size_t)token_seq[t] * table_stride + pi];
    const int kvh = hs < nq + nk ? hs - nq : hs - nq - nk;
    page_base = (((size_t)page * nk + kvh) * page_tokens + off) * D;
  }
  float v[8];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const int i = lane + 32 * c;
    v[c] = i < D ? src[i] : 0.f;
    ss += v[c] * v[c];
  }
  if (hs >= nq + nk) {  // a value head: stored as projected
    if (v_pages)
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const int i = lane + 32 * c;
        if (i < D) v_pages[page_base + i] = Num<T>::from_float(v[c]);
      }
    return;
  }
  const bool is_q = hs < nq;
  if (!is_q && v_from_k && v_pages) {
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const int i = lane + 32 * c;
      if (i < D) v_pages[page_base + i] = Num<T>::from_float(v[c]);
    }
  }
  const float* w = is_q ? qw : kw;
  if (w) {
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)norm_dim + eps);
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const int i = lane + 32 * c;
      if (i < D) v[c] = v[c] * inv * w[i];
    }
  }
  if (cos) {
    const int half = D / 2;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const int i = lane + 32 * c;
      if (i < D) buf[warp][i] = v[c];
    }
    __syncwarp();
    const float* cr = cos + (size_t)pos * half;
    const float* sr = sin + (size_t)pos * half;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const int i = lane + 32 * c;
      if (i < half) v[c] = v[c] * cr[i] - buf[warp][i + half] * sr[i];
      else if (i < D) v[c] = v[c] * cr[i - half] + buf[warp][i - half] * sr[i - half];
    }
  }
  T* dst = is_q ? q_out + (size_t)t * nq * D + (size_t)hs * D : (k_pages ? k_pages + page_base : nullptr);
  if (dst)
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const int i = lane + 32 * c;
      if (i < D) dst[i] = Num<T>::from_float(v[c]);
    }
}

// ------------------------------------------------------------------------------------ linear attention with decay
// S_t = decay * S_{t-1} + k_t v_t^T,  o_t = S_t^T q_t, in float32 on the CUDA cores.
// One block per (head, slice of CB value columns, chunk of the portion, sequence); 256 threads.
// A pair of neighbouring columns of S (key_dim values each) is shared by P neighbouring lanes,
// RPT = 8 rows of both columns each (so a thread's q and k values serve two columns), held in
// registers while the block steps through its tokens; the P partial dot products of o are added
// with shuffles. Columns are independent of one another, so slices of a head's columns run as
// separate blocks. q, k (after activation, rotation and scaling) and v of TT tokens are staged in
// shared memory per pass. The state is stored transposed, [slot][head][value_dim][key_dim]: a
// thread's rows are contiguous there.
//
// A portion longer than L tokens is cut into chunks of L that run side by side, in three launches:
//   A  every chunk steps through its tokens from a zero state (the first chunk from the request's
//      state) and leaves its outputs and its final state (chunk c: E_c) in a scratch;
//   B  the chunks' states are chained, element by element: F_0 = E_0, F_c = decay^len_c F_{c-1} + E_c;
//      the last one is the request's new state;
//   C  chunk c >= 1 adds what the state before it contributes: o_t += decay^(t - t_c + 1) F_{c-1}^T q_t.
// A portion of at most L tokens (a single token, above all) is one chunk: launch A alone, which
// then reads and writes the request's state itself.
constexpr int LA_RPT = 8, LA_TT = 16, LA_THREADS = 256, LA_PAD = 4;
constexpr int LA_TT_GATED = 8;  // tokens per tile with decays per channel: a third array is staged beside q and k

struct LinAttnArgs {
  const float* proj;      // [T, stride]: q | k | v | ... per row, heads concatenated
  long long stride;
  float* out;             // [T, H * dv]
  float* state;           // [slots, H, dv, dk]
  float* chunks;          // scratch [chunks of all chunked sequences, H, dv, dk], or null
  const float* decay;     // [H]
  const int* cu_q;
  const int* ctx_lens;
  const int* slots;
  const float* cos;       // [positions, rot/2] or null
  const float* sin;
  int H, dk, dv, rot, silu;
  float key_scale;
  int P, CB;              // lanes per column; columns per block
  int L;                  // chunk length
  int phase;              // 0: launch A, 2: launch C
  // a decay per key channel and token instead of decay[h]: alpha = sigmoid(z)^inv_root
  const float* gate_z;    // [T, gate_stride], heads x dk logits per row; null: the fixed decays
  long long gate_stride;
  float inv_root;
  float query_scale;      // the outputs are multiplied by this (a factor on q)
  int gate_is_logit;      // 1: gate_z holds logits; 0: it holds the decays themselves
  float* chunk_decay;     // scratch [chunks of all chunked sequences, H, dk]: the product of a chunk's alphas
};

__device__ __forceinline__ float root_of_sigmoid(float z, float inv_root) {
  // log sigmoid(z) = -(max(-z, 0) + log1p(exp(-|z|)))
  return expf(-(fmaxf(-z, 0.f) + log1pf(expf(-fabsf(z)))) * inv_root);
}

// Index of a sequence's first chunk in the scratch: only sequences of more than one chunk have any.
__device__ __forceinline__ int chunk_base(const int* cu_q, int seq, int L) {
  int base = 0;
  for (int s = 0; s < seq; ++s) {
    const int nc = (cu_q[s + 1] - cu_q[s] + L - 1) / L;
    base += nc > 1 ? nc : 0;
  }
  return base;
}

__device__ __forceinline__ void la_copy(float* smem, const float* gmem, bool wide) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem);
  if (wide) asm volatile("cp.async.ca.shared.global [%0], [%1], 16;\n" ::"r"(addr), "l"(gmem));
  else asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(addr), "l"(gmem));
}

// The rows of a tile go from global to shared memory as they are (cp.async, the next tile while
// this one is computed: two buffers); activation, rotation and the key's scale are then applied
// in place. Row i of a token's q (or k) lies at (i / RPT) * (RPT + PAD) + i % RPT: the pad keeps
// the 16-byte reads of the P lanes of a column on different banks.
// MODE 0: a fixed decay per head (launch A or C by a.phase). MODE 1 and 2: launches A and C with a
// decay per row and token, alpha_t[i]: its logits are staged like q and k and turned into alphas
// in place; launch C carries the running product of the chunk's alphas per row instead of a power
// of the decay. The product of each chunk's alphas, which launch B needs, is made by
// chunk_decay_kernel.
template <int P, int MODE>
__global__ void __launch_bounds__(LA_THREADS, MODE == 0 ? 0 : 3) decay_linear_attention_kernel(const LinAttnArgs a) {
  constexpr bool GATED = MODE != 0;
  constexpr int TT = GATED ? LA_TT_GATED : LA_TT;
  extern __shared__ __align__(16) float la_smem[];
  pdl_trigger();
  constexpr int CB = 2 * LA_THREADS / P;
  const int dk = a.dk, dv = a.dv, H = a.H, L = a.L;
  const int slices = (dv + CB - 1) / CB;
  const int h = blockIdx.x / slices, cb = blockIdx.x - h * slices;
  const int seq = blockIdx.z;
  const int r0 = a.cu_q[seq], n = a.cu_q[seq + 1] - r0;
  const int num_chunks = (n + L - 1) / L;
  const bool add_pass = MODE == 0 ? a.phase == 2 : MODE == 2;
  const int c = blockIdx.y + (add_pass ? 1 : 0);
  if (c >= num_chunks) {
    pdl_wait();  // no block leaves before the kernels before this one are done: the next kernel counts on it
    return;
  }
  const int pos0 = a.ctx_lens[seq] - n;
  const int t_begin = c * L, t_end = min(n, t_begin + L);
  const int p = threadIdx.x % P, jl = 2 * (threadIdx.x / P);
  const int j = cb * CB + jl;  // this thread's columns: j and j + 1
  constexpr int ldq = P * (LA_RPT + LA_PAD);
  // q [TT][ldq], k [TT][ldq], v [TT][CB], and with GATED the alphas [TT][ldq]
  constexpr int per_buf = (GATED ? 3 : 2) * TT * ldq + TT * CB;
  const float decay = GATED ? 1.f : a.decay[h];
  float S[LA_RPT], S1[LA_RPT];
  const bool has0 = j < dv, has1 = j + 1 < dv;
  const size_t column = ((size_t)h * dv + (has0 ? j : 0)) * dk + p * LA_RPT;
  const size_t per_state = (size_t)H * dv * dk;
  float* st = a.state + (size_t)a.slots[seq] * per_state + column;
  float* chunk_states = nullptr;
  const int first_chunk = num_chunks > 1 ? chunk_base(a.cu_q, seq, L) : 0;
  if (num_chunks > 1) chunk_states = a.chunks + (size_t)first_chunk * per_state + column;
  // rows beyond key_dim and columns beyond value_dim stay zero in both buffers (nothing else is
  // ever read that the copies below do not write)
  const int cols = min(CB, dv - cb * CB);  // value columns of this block
  if (dk != P * LA_RPT || cols != CB)
    for (int i = threadIdx.x; i < 2 * per_buf; i += LA_THREADS) la_smem[i] = 0.f;
  const bool wide_qk = (dk % 4 == 0) && (a.stride % 4 == 0) && (!GATED || a.gate_stride % 4 == 0);
  const bool wide_v = wide_qk && (dv % 4 == 0) && (CB % 4 == 0);
  const int qk_step = wide_qk ? 4 : 1, v_step = wide_v ? 4 : 1;
  const int qk_units = dk / qk_step, v_units = (cols + v_step - 1) / v_step;  // cols % 4 == 0 when wide
  __syncthreads();
  pdl_wait();
  auto issue = [&](int buf, int t0) {
    float* qs = la_smem + buf * per_buf;
    float* ks = qs + TT * ldq;
    float* vs = ks + TT * ldq;
    const int tn = min(TT, t_end - t0);
    for (int idx = threadIdx.x; idx < tn * qk_units; idx += LA_THREADS) {
      const int tt = idx / qk_units, i = (idx - tt * qk_units) * qk_step;
      const float* row = a.proj + (size_t)(r0 + t0 + tt) * a.stride + (size_t)h * dk + i;
      const int at = tt * ldq + (i / LA_RPT) * (LA_RPT + LA_PAD) + (i % LA_RPT);
      la_copy(qs + at, row, wide_qk);
      if (!add_pass) la_copy(ks + at, row + (size_t)H * dk, wide_qk);
      if constexpr (GATED)
        la_copy(vs + TT * CB + at, a.gate_z + (size_t)(r0 + t0 + tt) * a.gate_stride + (size_t)h * dk + i, wide_qk);
    }
    if (!add_pass)
      for (int idx = threadIdx.x; idx < tn * v_units; idx += LA_THREADS) {
        const int tt = idx / v_units, cc = (idx - tt * v_units) * v_step;
        la_copy(vs + tt * CB + cc,
                a.proj + (size_t)(r0 + t0 + tt) * a.stride + (size_t)2 * H * dk + (size_t)h * dv + cb * CB + cc,
                wide_v);
      }
    asm volatile("cp.async.commit_group;\n" ::);
  };
  issue(0, t_begin);
  {
    const float* from = add_pass ? chunk_states + (size_t)(c - 1) * per_state : st;
    const bool read = add_pass || (c == 0 && pos0 > 0);
    auto load_column = [&](float (&dst)[LA_RPT], const float* src, bool on) {
      if (on && dk % 4 == 0) {  // a thread's rows are contiguous: 16-byte loads
#pragma unroll
        for (int r4 = 0; r4 < LA_RPT / 4; ++r4) {
          float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
          if (p * LA_RPT + 4 * r4 < dk) v = __ldcg(reinterpret_cast<const float4*>(src) + r4);
          dst[4 * r4 + 0] = v.x; dst[4 * r4 + 1] = v.y; dst[4 * r4 + 2] = v.z; dst[4 * r4 + 3] = v.w;
        }
      } else {
#pragma unroll
        for (int r = 0; r < LA_RPT; ++r) dst[r] = (on && p * LA_RPT + r < dk) ? src[r] : 0.f;
      }
    };
    load_column(S, from, read && has0);
    load_column(S1, from + dk, read && has1);
  }
  const int half = a.rot / 2;
  const int work = dk - half;  // a rotated pair is one piece of work, every other row one
  float carried = 1.f;  // launch C: decay^(tokens of the chunk so far)
  float run[GATED ? LA_RPT : 1];  // GATED: the product of the chunk's alphas so far, row by row
#pragma unroll
  for (int r = 0; r < (GATED ? LA_RPT : 1); ++r) run[r] = 1.f;
  const bool keeps_run = MODE == 2;
  int buf = 0;
  for (int t0 = t_begin; t0 < t_end; t0 += TT, buf ^= 1) {
    const int tn = min(TT, t_end - t0);
    if (t0 + TT < t_end) {
      issue(buf ^ 1, t0 + TT);
      asm volatile("cp.async.wait_group 1;\n" ::);
    } else {
      asm volatile("cp.async.wait_group 0;\n" ::);
    }
    __syncthreads();
    float* qs = la_smem + buf * per_buf;
    float* ks = qs + TT * ldq;
    float* vs = ks + TT * ldq;
    float* gs = vs + TT * CB;
    if (a.silu || a.rot || a.key_scale != 1.f || (GATED && a.gate_is_logit)) {
      for (int idx = threadIdx.x; idx < tn * work; idx += LA_THREADS) {
        const int tt = idx / work, w = idx - tt * work;
        const int i = w < half ? w : w + half;  // rows [half, rot) are done with their partners
        const int at = tt * ldq + (i / LA_RPT) * (LA_RPT + LA_PAD) + (i % LA_RPT);
        float q = qs[at], k = ks[at];
        if (a.silu) {
          q = silu_f(q);
          k = silu_f(k);
        }
        if (w < half) {
          const int ip = i + half;
          const int atp = tt * ldq + (ip / LA_RPT) * (LA_RPT + LA_PAD) + (ip % LA_RPT);
          float qp = qs[atp], kp = ks[atp];
          if (a.silu) {
            qp = silu_f(qp);
            kp = silu_f(kp);
          }
          const size_t tab = (size_t)(pos0 + t0 + tt) * half + i;
          const float cs = a.cos[tab], sn = a.sin[tab];
          qs[atp] = qp * cs + q * sn;
          ks[atp] = (kp * cs + k * sn) * a.key_scale;
          if constexpr (GATED) {
            if (a.gate_is_logit) gs[atp] = root_of_sigmoid(gs[atp], a.inv_root);
          }
          const float q2 = q * cs - qp * sn, k2 = k * cs - kp * sn;
          q = q2;
          k = k2;
        }
        qs[at] = q;
        ks[at] = k * a.key_scale;
        if constexpr (GATED) {
          if (a.gate_is_logit) gs[at] = root_of_sigmoid(gs[at], a.inv_root);
        }
      }
      if (a.silu && !add_pass)
        for (int idx = threadIdx.x; idx < tn * cols; idx += LA_THREADS) {
          const int tt = idx / cols, cc = idx - tt * cols;
          vs[tt * CB + cc] = silu_f(vs[tt * CB + cc]);
        }
      __syncthreads();
    }
    const float4* q4 = reinterpret_cast<const float4*>(qs + p * (LA_RPT + LA_PAD));
    const float4* k4 = reinterpret_cast<const float4*>(ks + p * (LA_RPT + LA_PAD));
    const float4* g4 = reinterpret_cast<const float4*>(gs + p * (LA_RPT + LA_PAD));
    const float* vcol = vs + jl;
    // after the reduction lane p == 0 holds column j's sum and lane p == 1 column j + 1's
    const int mine = P > 1 ? (p & 1) : 0;
    float* dst = a.out + (size_t)(r0 + t0) * ((size_t)H * dv) + (size_t)h * dv + j + mine;
    const size_t out_stride = (size_t)H * dv;
    const bool writes = P > 1 ? (p < 2 && j + mine < dv) : has0;
#pragma unroll 2
    for (int tt = 0; tt < tn; ++tt, q4 += ldq / 4, k4 += ldq / 4, g4 += ldq / 4, vcol += CB, dst += out_stride) {
      float acc0 = 0.f, acc1 = 0.f;
      if (!add_pass) {
        const float2 vj = *reinterpret_cast<const float2*>(vcol);
#pragma unroll
        for (int r4 = 0; r4 < LA_RPT / 4; ++r4) {
          const float4 q = q4[r4], k = k4[r4];
          const float qv[4] = {q.x, q.y, q.z, q.w}, kv[4] = {k.x, k.y, k.z, k.w};
          float gv[4] = {decay, decay, decay, decay};
          if constexpr (GATED) {
            const float4 g = g4[r4];
            gv[0] = g.x; gv[1] = g.y; gv[2] = g.z; gv[3] = g.w;
            if (keeps_run) {
#pragma unroll
              for (int e = 0; e < 4; ++e) run[4 * r4 + e] *= gv[e];
            }
          }
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            S[4 * r4 + e] = fmaf(gv[e], S[4 * r4 + e], kv[e] * vj.x);
            S1[4 * r4 + e] = fmaf(gv[e], S1[4 * r4 + e], kv[e] * vj.y);
            acc0 = fmaf(S[4 * r4 + e], qv[e], acc0);
            acc1 = fmaf(S1[4 * r4 + e], qv[e], acc1);
          }
        }
      } else {
#pragma unroll
        for (int r4 = 0; r4 < LA_RPT / 4; ++r4) {
          const float4 q = q4[r4];
          float qv[4] = {q.x, q.y, q.z, q.w};
          if constexpr (GATED) {  // what is left of the state before the chunk, row by row
            const float4 g = g4[r4];
            const float gv[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              run[4 * r4 + e] *= gv[e];
              qv[e] *= run[4 * r4 + e];
            }
          }
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            acc0 = fmaf(S[4 * r4 + e], qv[e], acc0);
            acc1 = fmaf(S1[4 * r4 + e], qv[e], acc1);
          }
        }
        carried *= decay;
      }
      float acc = acc0;
      if (P > 1) {
        // the first step halves the data: a lane hands over the sum of the column it does not keep
        const float give = mine ? acc0 : acc1, keep = mine ? acc1 : acc0;
        acc = keep + __shfl_xor_sync(0xffffffffu, give, 1);
#pragma unroll
        for (int o = P >> 1; o > 1; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      }
      if (writes) {
        // launch C adds into what launch A stored: a reduction without a return value, so that
        // the warp does not wait for the old value (one thread per element: the order is fixed)
        if (add_pass) atomicAdd(dst, carried * acc * a.query_scale);
        else *dst = acc * a.query_scale;
      }
      if (P == 1 && has1) {
        if (add_pass) atomicAdd(dst + 1, carried * acc1 * a.query_scale);
        else dst[1] = acc1 * a.query_scale;
      }
    }
    __syncthreads();  // the buffer is free for the tile after the next
  }
  if (add_pass) return;
  float* to = num_chunks > 1 ? chunk_states + (size_t)c * per_state : st;
  auto store_column = [&](const float (&src)[LA_RPT], float* dst) {
    if (dk % 4 == 0) {
#pragma unroll
      for (int r4 = 0; r4 < LA_RPT / 4; ++r4)
        if (p * LA_RPT + 4 * r4 < dk)
          reinterpret_cast<float4*>(dst)[r4] =
              make_float4(src[4 * r4], src[4 * r4 + 1], src[4 * r4 + 2], src[4 * r4 + 3]);
    } else {
#pragma unroll
      for (int r = 0; r < LA_RPT; ++r)
        if (p * LA_RPT + r < dk) dst[r] = src[r];
    }
  };
  if (has0) store_column(S, to);
  if (has1) store_column(S1, to + dk);
}

// Logits of decays turned into the decays themselves, in place: sigmoid(z)^inv_root. Rows of
// `cols` values, `stride` apart.
__global__ void decay_from_logits_kernel(float* __restrict__ z, long long stride, int cols, long long n,
                                         float inv_root) {
  pdl_trigger();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const long long t = i / cols;
  float* p = z + t * stride + (i - t * cols);
  *p = root_of_sigmoid(*p, inv_root);
}

// The product of the alphas of each chunk of every sequence of more than one chunk, per head and
// key channel: chunk_decay[first chunk of the sequence + c][h * dk + i]. One thread per channel.
__global__ void chunk_decay_kernel(const float* __restrict__ gate_z, long long gate_stride, float inv_root,
                                   int is_logit, float* __restrict__ chunk_decay,
                                   const int* __restrict__ cu_q, int HK, int L) {
  pdl_trigger();
  const int seq = blockIdx.z, c = blockIdx.y;
  const int r0 = cu_q[seq], n = cu_q[seq + 1] - r0;
  const int num_chunks = (n + L - 1) / L;
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  pdl_wait();
  if (num_chunks <= 1 || c >= num_chunks || e >= HK) return;
  const int t_end = min(n, (c + 1) * L);
  float prod = 1.f;
  for (int t = c * L; t < t_end; ++t) {
    const float g = gate_z[(size_t)(r0 + t) * gate_stride + e];
    prod *= is_logit ? root_of_sigmoid(g, inv_root) : g;
  }
  chunk_decay[(size_t)(chunk_base(cu_q, seq, L) + c) * HK + e] = prod;
}

// Launch B: one thread per element of the state and sequence of more than one chunk.
__global__ void chain_chunk_states_kernel(float* __restrict__ chunks, float* __restrict__ state,
                                          const float* __restrict__ decay, const int* __restrict__ cu_q,
                                          const int* __restrict__ slots, int H, int dv, int dk, int L,
                                          const float* chunk_decay) {
  pdl_trigger();
  const int seq = blockIdx.y;
  const int n = cu_q[seq + 1] - cu_q[seq];
  const int num_chunks = (n + L - 1) / L;
  const size_t per_state = (size_t)H * dv * dk;
  const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (num_chunks <= 1 || e >= per_state) {
    pdl_wait();  // as above
    return;
  }
  const int first_chunk = chunk_base(cu_q, seq, L);
  float* mine = chunks + (size_t)first_chunk * per_state + e;
  const int head = (int)(e / ((size_t)dv * dk));
  const float d = chunk_decay ? 1.f : decay[head];
  const float whole = powf(d, (float)L);
  // with a decay per channel and token: the product of chunk c's alphas of this element's row
  const float* across = chunk_decay ? chunk_decay + ((size_t)first_chunk * H + head) * dk + e % dk : nullptr;
  pdl_wait();
  float S = mine[0];
  for (int c0 = 1; c0 < num_chunks; c0 += 8) {  // a round's loads are all in flight before its chain
    float E[8], A[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      E[u] = c0 + u < num_chunks ? __ldcg(mine + (size_t)(c0 + u) * per_state) : 0.f;
      A[u] = (across && c0 + u < num_chunks) ? __ldcg(across + (size_t)(c0 + u) * H * dk) : 0.f;
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int c = c0 + u;
      if (c < num_chunks) {
        const int len = min(L, n - c * L);
        S = fmaf(across ? A[u] : (len == L ? whole : powf(d, (float)len)), S, E[u]);
        mine[(size_t)c * per_state] = S;
      }
    }
  }
  state[(size_t)slots[seq] * per_state + e] = S;
}

static int pow2_at_least(int n) {
  int p = 1;
  while (p < n) p <<= 1;
  return p;
}

}  // namespace lse

using namespace lse;

extern "C" int lse_cast(const float* x, void* out, int out_dtype, long long n, cudaStream_t stream) {
  if (n <= 0) return LSE_OK;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  if (out_dtype == LSE_BF16) launch(cast_kernel<bf16>, blocks, 256, 0, stream, x, (bf16*)out, n);
  else if (out_dtype == LSE_F32) launch(cast_kernel<float>, blocks, 256, 0, stream, x, (float*)out, n);
  else return LSE_BAD_ARGUMENT;
  return LSE_CHECK_LAUNCH();
}

extern "C" int lse_token_shift(const float* x, const float* mix, float* state, void* out, int out_dtype,
                               const int* token_seq, const int* cu_q, const int* ctx_lens,
                               const int* slots, int T, int W, cudaStream_t stream) {
  if (T <= 0) return LSE_OK;
  const int threads = W >= 1024 ? 256 : 128;
  if (out_dtype == LSE_BF16)
    launch(token_shift_kernel<bf16>, T, threads, 0, stream, x, mix, state, (bf16*)out, token_seq, cu_q,
           ctx_lens, slots, W);
  else if (out_dtype == LSE_F32)
    launch(token_shift_kernel<float>, T, threads, 0, stream, x, mix, state, (float*)out, token_seq, cu_q,
           ctx_lens, slots, W);
  else return LSE_BAD_ARGUMENT;
  return LSE_CHECK_LAUNCH();
}

extern "C" int lse_rmsnorm_add(float* x, const void* a, const void* b, int branch_dtype, const float* wa,
                               const float* wb, float ca, float cb, float eps_in, const float* w, float eps,
                               void* out, int out_dtype, const float* then_w, float then_eps, int T, int H,
                               cudaStream_t stream) {
  if (T <= 0) return LSE_OK;
  if (!x || !a || !w || (b && !wa) || (wa && b && !wb)) return LSE_BAD_ARGUMENT;
  if (branch_dtype != LSE_F32 && branch_dtype != LSE_FIXED64) return LSE_BAD_ARGUMENT;
  const bool sums = branch_dtype == LSE_FIXED64;
  const size_t smem = sums ? (size_t)H * (b ? 2 : 1) * sizeof(float) : 0;
  if (smem > 48 * 1024) return LSE_BAD_ARGUMENT;
  if (then_w && !out) return LSE_BAD_ARGUMENT;
  const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
  const bool to_bf16 = out && out_dtype == LSE_BF16;
  if (!to_bf16 && out && out_dtype != LSE_F32) return LSE_BAD_ARGUMENT;
  auto aligned = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  const bool vec = H % 4 == 0 && aligned(x) && aligned(w) && aligned(out) && aligned(wa) && aligned(wb) &&
                   aligned(then_w) && (sums || (aligned(a) && aligned(b)));
  const int per_visit = threads * (vec ? 4 : 1);
  const int visits = (H + per_visit - 1) / per_visit;  // places of the row per thread
#define LSE_RNA_V(TO, S, V, K) \
  launch(rmsnorm_add_kernel<TO, S, V, K>, T, threads, smem, stream, x, a, b, wa, wb, ca, cb, eps_in, w, eps, \
         (TO*)out, then_w, then_eps, H)
#define LSE_RNA(TO, S) \
  do { \
    if (vec && visits == 1) LSE_RNA_V(TO, S, 4, 1); \
    else if (vec && visits == 2) LSE_RNA_V(TO, S, 4, 2); \
    else if (vec) LSE_RNA_V(TO, S, 4, 0); \
    else if (visits == 1) LSE_RNA_V(TO, S, 1, 1); \
    else LSE_RNA_V(TO, S, 1, 0); \
  } while (0)
  if (to_bf16) {
    if (sums) LSE_RNA(bf16, true); else LSE_RNA(bf16, false);
  } else {
    if (sums) LSE_RNA(float, true); else LSE_RNA(float, false);
  }
#undef LSE_RNA_V
#undef LSE_RNA
  return LSE_CHECK_LAUNCH();
}

extern "C" int lse_mix_normed(const float* a, const float* b, const float* wa, const float* wb, float ca,
                              float cb, float eps, float* out, int T, int H, cudaStream_t stream) {
  if (T <= 0) return LSE_OK;
  if (!a || !wa || (b && !wb) || !out) return LSE_BAD_ARGUMENT;
  const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
  launch(mix_normed_kernel, T, threads, 0, stream, a, b, wa, wb, ca, cb, eps, out, H);
  return LSE_CHECK_LAUNCH();
}

extern "C" int lse_gated_group_norm(const float* o, const float* gate, long long gate_stride, int T, int N,
                                    int group, const float* weight, float eps, int sigmoid, void* out,
                                    int out_dtype, cudaStream_t stream) {
  if (T <= 0) return LSE_OK;
  if (group <= 0 || N % group || N / group > 65535) return LSE_BAD_ARGUMENT;
  const int threads = group >= 1024 ? 256 : (group >= 128 ? 128 : (group > 32 ? 64 : 32));
  dim3 grid(T, N / group);
  if (out_dtype == LSE_BF16)
    launch(gated_group_norm_kernel<bf16>, grid, threads, 0, stream, o, gate, gate_stride, N, group, weight,
           eps, sigmoid, (bf16*)out);
  else if (out_dtype == LSE_F32)
    launch(gated_group_norm_kernel<float>, grid, threads, 0, stream, o, gate, gate_stride, N, group, weight,
           eps, sigmoid, (float*)out);
  else return LSE_BAD_ARGUMENT;
  return LSE_CHECK_LAUNCH();
}

extern "C" int lse_norm_rope_kv_write(const float* qkv, void* q_out, int dtype, int T, int nq, int nk, int D,
                                      int v_from_k, const float* qw, const float* kw, float eps,
                                      const int* positions, const int* token_seq, const float* cos,
                                      const float* sin, void* k_pages, void* v_pages,
                                      const int* block_tables, int table_stride, int page_tokens,
                                      int norm_dim, cudaStream_t stream, long long row_stride) {
  if (row_stride <= 0) row_stride = (long long)(nq + nk + (v_from_k ? 0 : nk)) * D;
  if (T <= 0) return LSE_OK;
  if (D <= 0 || D > 256 || (cos && D % 2) || (!qw != !kw) || (!cos != !sin) || (!k_pages != !v_pages) ||
      page_tokens <= 0)
    return LSE_BAD_ARGUMENT;
  const int heads = nq + nk + (v_from_k ? 0 : nk);
  dim3 grid(T, (heads + NRW_WARPS - 1) / NRW_WARPS);
  if (grid.y > 65535) return LSE_BAD_ARGUMENT;
  if (dtype == LSE_BF16)
    launch(norm_rope_kv_write_kernel<bf16>, grid, NRW_WARPS * 32, 0, stream, qkv, (bf16*)q_out, nq, nk, D,
           v_from_k, qw, kw, eps, positions, token_seq, cos, sin, (bf16*)k_pages, (bf16*)v_pages,
           block_tables, table_stride, page_tokens, norm_dim, row_stride);
  else if (dtype == LSE_F32)
    launch(norm_rope_kv_write_kernel<float>, grid, NRW_WARPS * 32, 0, stream, qkv, (float*)q_out, nq, nk, D,
           v_from_k, qw, kw, eps, positions, token_seq, cos, sin, (float*)k_pages, (float*)v_pages,
           block_tables, table_stride, page_tokens, norm_dim, row_stride);
  else return LSE_BAD_ARGUMENT;
  return LSE_CHECK_LAUNCH();
}

extern "C" int lse_linear_attention_chunk(void) { return 64; }

extern "C" int lse_decay_linear_attention(const float* proj, long long stride, float* out, float* state,
                                          const float* decay, const int* cu_q, const int* ctx_lens,
                                          const int* slots, int num_seqs, int H, int dk, int dv,
                                          const float* cos, const float* sin, int rot, int silu,
                                          float key_scale, int max_chunks, float* chunks,
                                          cudaStream_t stream, const float* gate_z, long long gate_stride,
                                          float decay_root, float query_scale, float* chunk_decay,
                                          int total_rows) {
  if (num_seqs <= 0) return LSE_OK;
  if ((!gate_z && !decay) || (gate_z && (decay_root <= 0.f || gate_stride < (long long)H * dk)) ||
      (gate_z && max_chunks > 1 && !chunk_decay))
    return LSE_BAD_ARGUMENT;
  if (H <= 0 || dk <= 0 || dv <= 0 || dk > 256 || rot < 0 || rot > dk || rot % 2 || (rot && (!cos || !sin)) ||
      num_seqs > 65535 || max_chunks < 1 || max_chunks > 65535 || (max_chunks > 1 && !chunks))
    return LSE_BAD_ARGUMENT;
  LinAttnArgs a;
  a.proj = proj; a.stride = stride; a.out = out; a.state = state; a.chunks = chunks; a.decay = decay;
  a.cu_q = cu_q; a.ctx_lens = ctx_lens; a.slots = slots; a.cos = cos; a.sin = sin; a.H = H; a.dk = dk;
  a.dv = dv; a.rot = rot; a.silu = silu; a.key_scale = key_scale;
  a.gate_z = gate_z; a.gate_stride = gate_stride; a.inv_root = gate_z ? 1.f / decay_root : 1.f;
  a.query_scale = query_scale; a.chunk_decay = chunk_decay;
  const bool gated = gate_z != nullptr;
  // Long portions: many blocks (chunks, slices of a head's columns) read the same logits, so the
  // decays are made once, in place, by a kernel of their own. Steps of short portions and single
  // tokens turn the logits into decays as they stage them (one launch fewer).
  a.gate_is_logit = 1;
  if (gated && max_chunks > 1 && total_rows > 0) {
    const long long n = (long long)total_rows * H * dk;
    launch(decay_from_logits_kernel, (unsigned)((n + 255) / 256), 256, 0, stream, const_cast<float*>(gate_z),
           gate_stride, H * dk, n, a.inv_root);
    a.gate_is_logit = 0;
  }
  a.P = pow2_at_least((dk + LA_RPT - 1) / LA_RPT);
  a.CB = 2 * LA_THREADS / a.P;
#define LSE_LA_KERNEL(MODE)                                          \
  (a.P == 1 ? decay_linear_attention_kernel<1, MODE>                 \
   : a.P == 2 ? decay_linear_attention_kernel<2, MODE>               \
   : a.P == 4 ? decay_linear_attention_kernel<4, MODE>               \
   : a.P == 8 ? decay_linear_attention_kernel<8, MODE>               \
   : a.P == 16 ? decay_linear_attention_kernel<16, MODE>             \
               : decay_linear_attention_kernel<32, MODE>)
  void (*kernel)(LinAttnArgs) = gated ? LSE_LA_KERNEL(1) : LSE_LA_KERNEL(0);
  void (*kernel_add)(LinAttnArgs) = gated ? LSE_LA_KERNEL(2) : kernel;
#undef LSE_LA_KERNEL
  a.L = lse_linear_attention_chunk();
  a.phase = 0;
  const int slices = (dv + a.CB - 1) / a.CB;
  const int tile = gated ? LA_TT_GATED : LA_TT;
  const size_t smem =
      2 * ((size_t)(gated ? 3 : 2) * tile * a.P * (LA_RPT + LA_PAD) + (size_t)tile * a.CB) * sizeof(float);
  static bool configured[2][33] = {};
  if (!configured[gated][a.P]) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024) != cudaSuccess ||
        (kernel_add != kernel &&
         cudaFuncSetAttribute(kernel_add, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024) != cudaSuccess))
      return LSE_LAUNCH_FAILED;
    configured[gated][a.P] = true;
  }
  launch(kernel, dim3(H * slices, max_chunks, num_seqs), LA_THREADS, smem, stream, a);
  if (max_chunks > 1) {
    const size_t per_state = (size_t)H * dv * dk;
    if (gated)
      launch(chunk_decay_kernel, dim3((unsigned)((H * dk + 127) / 128), max_chunks, num_seqs), 128, 0, stream, gate_z,
             gate_stride, a.inv_root, a.gate_is_logit, chunk_decay, cu_q, H * dk, a.L);
    launch(chain_chunk_states_kernel, dim3((unsigned)((per_state + 255) / 256), num_seqs), 256, 0, stream,
           chunks, state, decay, cu_q, slots, H, dv, dk, a.L, (const float*)(gated ? chunk_decay : nullptr));
    a.phase = 2;
    launch(kernel_add, dim3(H * slices, max_chunks - 1, num_seqs), LA_THREADS, smem, stream, a);
  }
  return LSE_CHECK_LAUNCH();
}
