// Python binding of the engine's CUDA kernels. Every function checks device, dtype, shape and
// contiguity of what it is given and raises on anything it cannot serve; work is enqueued on
// PyTorch's current CUDA stream. Attention kernels live in one shared library per head size,
// loaded here with dlopen.
#include <ATen/cuda/CUDAContext.h>
#include <dlfcn.h>
#include <torch/extension.h>

#include <map>
#include <optional>
#include <string>

#include "attention_args.h"
#include "kernels.h"

namespace {

using torch::Tensor;
using OptTensor = std::optional<Tensor>;

// Numbers go into messages as strings made here: streaming an integer or a double into an error
// message (operator<< of an ostream) has crashed the interpreter in builds of this extension on
// some hosts, and an error path must never do that.
template <typename N>
std::string num(N v) { return std::to_string(v); }

int dtype_code(const Tensor& t, const char* what) {
  if (t.scalar_type() == torch::kFloat32) return LSE_F32;
  if (t.scalar_type() == torch::kBFloat16) return LSE_BF16;
  if (t.scalar_type() == torch::kInt64) return LSE_FIXED64;  // fixed-point sums of the few-rows product
  TORCH_CHECK(false, what, ": dtype must be float32 or bfloat16, got ", c10::toString(t.scalar_type()));
}

void check_cuda(const Tensor& t, const char* what) {
  TORCH_CHECK(t.is_cuda(), what, " must be a CUDA tensor");
  TORCH_CHECK(t.is_contiguous(), what, " must be contiguous");
  // the kernels read and write 16-byte vectors wherever a row holds whole ones
  TORCH_CHECK(t.numel() == 0 || reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0, what,
              " must start on a 16-byte boundary");
}

void check_i32(const Tensor& t, const char* what) {
  check_cuda(t, what);
  TORCH_CHECK(t.scalar_type() == torch::kInt32, what, " must be int32");
}

void check_f32(const Tensor& t, const char* what) {
  check_cuda(t, what);
  TORCH_CHECK(t.scalar_type() == torch::kFloat32, what, " must be float32");
}

// A per-request state is a slice of a [layers, slots, ...] tensor: its start follows from the
// state's size, so only what the kernels need of it is asked (they read states element by
// element unless every row of a state is a whole number of 16-byte vectors).
void check_state(const Tensor& t, const char* what, int64_t vector_rows) {
  TORCH_CHECK(t.is_cuda() && t.is_contiguous() && t.scalar_type() == torch::kFloat32, what,
              " must be a contiguous float32 CUDA tensor");
  TORCH_CHECK(vector_rows % 4 != 0 || reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0, what,
              " must start on a 16-byte boundary");
}

cudaStream_t stream() { return at::cuda::getCurrentCUDAStream().stream(); }

void done(int code, const char* what) {
  TORCH_CHECK(code != LSE_BAD_ARGUMENT, what, ": the kernel refused these arguments");
  if (code != LSE_OK) {
    cudaError_t e = cudaGetLastError();
    TORCH_CHECK(false, what, ": launch failed: ", cudaGetErrorString(e));
  }
  // a capture that something has invalidated is reported where it is first seen, not at its end
  cudaStreamCaptureStatus status = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream(), &status) != cudaSuccess ||
      status == cudaStreamCaptureStatusInvalidated) {
    cudaGetLastError();
    TORCH_CHECK(false, what, ": the stream's graph capture is invalid after this call");
  }
}

void embedding(const Tensor& ids, const Tensor& table, Tensor& out) {
  check_i32(ids, "ids");
  check_cuda(table, "table");
  check_f32(out, "out");
  TORCH_CHECK(table.dim() == 2 && out.dim() == 2 && ids.dim() == 1, "embedding: bad ranks");
  TORCH_CHECK(out.size(0) == ids.size(0) && out.size(1) == table.size(1), "embedding: bad shapes");
  done(lse_embedding(ids.data_ptr<int>(), table.data_ptr(), dtype_code(table, "table"),
                     out.data_ptr<float>(), (int)ids.size(0), (int)table.size(1), stream()),
       "embedding");
}

void add_rmsnorm(Tensor& x, const OptTensor& residual, const Tensor& weight, double eps,
                 Tensor& out, const OptTensor& rows) {
  check_f32(x, "x");
  check_f32(weight, "weight");
  check_cuda(out, "out");
  TORCH_CHECK(x.dim() == 2 && out.dim() == 2 && weight.dim() == 1, "add_rmsnorm: bad ranks");
  const int H = (int)x.size(1);
  TORCH_CHECK(weight.size(0) == H && out.size(1) == H, "add_rmsnorm: widths differ");
  int rcode = LSE_F32;
  const void* rptr = nullptr;
  if (residual) {
    check_cuda(*residual, "residual");
    TORCH_CHECK(residual->sizes() == x.sizes(), "add_rmsnorm: residual shape differs from x");
    rcode = dtype_code(*residual, "residual");
    rptr = residual->data_ptr();
  }
  const int* rows_ptr = nullptr;
  int T = (int)x.size(0);
  if (rows) {
    check_i32(*rows, "rows");
    rows_ptr = rows->data_ptr<int>();
    T = (int)rows->size(0);
  }
  TORCH_CHECK(out.size(0) == T, "add_rmsnorm: out has ", num(out.size(0)), " rows, expected ", num(T));
  done(lse_add_rmsnorm(x.data_ptr<float>(), rptr, rcode, weight.data_ptr<float>(), (float)eps,
                       out.data_ptr(), dtype_code(out, "out"), rows_ptr, T, H, stream()),
       "add_rmsnorm");
}

// Returns the rotated queries: a view of qkv's first nq*D columns when qkv already has the pages'
// dtype, or a new [T, nq*D] tensor of `q_dtype` when qkv holds float32 sums.
Tensor rope_kv_write(Tensor& qkv, int64_t nq, int64_t nk, int64_t D, const Tensor& positions,
                     const Tensor& token_seq, const OptTensor& cos, const OptTensor& sin,
                     const OptTensor& k_pages, const OptTensor& v_pages, const Tensor& block_tables,
                     int64_t page_tokens, bool q_bf16) {
  check_cuda(qkv, "qkv");
  check_i32(positions, "positions");
  check_i32(token_seq, "token_seq");
  check_i32(block_tables, "block_tables");
  TORCH_CHECK(qkv.dim() == 2 && qkv.size(1) == (nq + 2 * nk) * D, "rope_kv_write: qkv width");
  const int T = (int)qkv.size(0);
  TORCH_CHECK(positions.size(0) == T && token_seq.size(0) == T, "rope_kv_write: lengths differ");
  TORCH_CHECK(block_tables.dim() == 2, "rope_kv_write: block_tables must be [sequences, blocks]");
  const int in_code = dtype_code(qkv, "qkv");
  const int out_code = q_bf16 ? LSE_BF16 : LSE_F32;
  TORCH_CHECK(in_code == out_code || in_code == LSE_F32 || (in_code == LSE_FIXED64 && q_bf16),
              "rope_kv_write: this qkv dtype cannot give this q dtype");
  const float *c = nullptr, *s = nullptr;
  if (cos) {
    TORCH_CHECK(sin.has_value(), "rope_kv_write: cos without sin");
    check_f32(*cos, "cos");
    check_f32(*sin, "sin");
    TORCH_CHECK(cos->dim() == 2 && cos->size(1) == D / 2 && sin->sizes() == cos->sizes(),
                "rope_kv_write: tables must be [positions, head_dim/2]");
    c = cos->data_ptr<float>();
    s = sin->data_ptr<float>();
  }
  void *kp = nullptr, *vp = nullptr;
  if (k_pages) {
    TORCH_CHECK(v_pages.has_value(), "rope_kv_write: k_pages without v_pages");
    check_cuda(*k_pages, "k_pages");
    check_cuda(*v_pages, "v_pages");
    TORCH_CHECK(dtype_code(*k_pages, "k_pages") == out_code && dtype_code(*v_pages, "v_pages") == out_code,
                "rope_kv_write: pages and q differ in dtype");
    TORCH_CHECK(k_pages->dim() == 4 && k_pages->size(1) == nk && k_pages->size(2) == page_tokens &&
                    k_pages->size(3) == D && v_pages->sizes() == k_pages->sizes(),
                "rope_kv_write: pages must be [pages, kv_heads, page_tokens, head_dim]");
    kp = k_pages->data_ptr();
    vp = v_pages->data_ptr();
  }
  Tensor q = in_code == out_code
                 ? qkv.narrow(1, 0, nq * D)
                 : torch::empty({T, nq * D}, qkv.options().dtype(torch::kBFloat16));
  done(lse_rope_kv_write(qkv.data_ptr(), in_code, q.data_ptr(), out_code, T, (int)nq, (int)nk, (int)D,
                         positions.data_ptr<int>(), token_seq.data_ptr<int>(), c, s, kp, vp,
                         block_tables.data_ptr<int>(), (int)block_tables.size(1), (int)page_tokens,
                         stream()),
       "rope_kv_write");
  return q;
}

void silu_mul(const Tensor& gu, Tensor& out, int64_t act) {
  check_cuda(gu, "gu");
  check_cuda(out, "out");
  TORCH_CHECK(gu.dim() == 2 && out.dim() == 2 && gu.size(1) == 2 * out.size(1) &&
                  gu.size(0) == out.size(0),
              "silu_mul: gu must be [T, 2I] and out [T, I]");
  done(lse_silu_mul(gu.data_ptr(), dtype_code(gu, "gu"), out.data_ptr(), dtype_code(out, "out"),
                    (int)gu.size(0), (int)out.size(1), (int)act, stream()),
       "silu_mul");
}

void gemm_f32(const Tensor& a, const Tensor& w, const OptTensor& bias, Tensor& out) {
  check_f32(a, "a");
  check_f32(w, "w");
  check_f32(out, "out");
  TORCH_CHECK(a.dim() == 2 && w.dim() == 2 && out.dim() == 2 && a.size(1) == w.size(1) &&
                  out.size(0) == a.size(0) && out.size(1) == w.size(0),
              "gemm_f32: need a [T, K], w [N, K], out [T, N]");
  const float* b = nullptr;
  if (bias) {
    check_f32(*bias, "bias");
    TORCH_CHECK(bias->numel() == w.size(0), "gemm_f32: bias length");
    b = bias->data_ptr<float>();
  }
  done(lse_gemm_f32(a.data_ptr<float>(), w.data_ptr<float>(), b, out.data_ptr<float>(),
                    (int)a.size(0), (int)w.size(0), (int)a.size(1), stream()),
       "gemm_f32");
}

// A host-mapped int that kernels set when a bounded wait runs out; the host reads it without a copy.
int* error_flag() {
  static int* flag = nullptr;
  if (!flag) {
    TORCH_CHECK(cudaHostAlloc(&flag, sizeof(int), cudaHostAllocMapped) == cudaSuccess,
                "cannot allocate the kernels' error flag");
    *flag = 0;
  }
  return flag;
}

int64_t kernel_error() { return *error_flag(); }
void clear_kernel_error() { *error_flag() = 0; }

int64_t gemm_bf16_skinny_max_rows() { return lse_gemm_bf16_skinny_max_rows(); }

// out += a w^T (+ bias), out a buffer of fixed-point sums (int64)
void gemm_bf16_skinny(const Tensor& a, const Tensor& w, const OptTensor& bias, Tensor& out) {
  check_cuda(a, "a");
  check_cuda(w, "w");
  check_cuda(out, "out");
  TORCH_CHECK(a.scalar_type() == torch::kBFloat16 && w.scalar_type() == torch::kBFloat16,
              "gemm_bf16_skinny: a and w must be bfloat16");
  TORCH_CHECK(a.dim() == 2 && w.dim() == 2 && out.dim() == 2 && a.size(1) == w.size(1) &&
                  out.size(0) == a.size(0) && out.size(1) == w.size(0),
              "gemm_bf16_skinny: need a [T, K], w [N, K], out [T, N]");
  const void* b = nullptr;
  if (bias) {
    check_cuda(*bias, "bias");
    TORCH_CHECK(bias->scalar_type() == torch::kBFloat16 && bias->numel() == w.size(0),
                "gemm_bf16_skinny: bias must be bfloat16 [N]");
    b = bias->data_ptr();
  }
  TORCH_CHECK(out.scalar_type() == torch::kInt64, "gemm_bf16_skinny: out must be int64 (fixed-point sums)");
  done(lse_gemm_bf16_skinny(a.data_ptr(), w.data_ptr(), b, out.data_ptr(),
                            (int)a.size(0), (int)w.size(0), (int)a.size(1), error_flag(), stream()),
       "gemm_bf16_skinny");
}

// out (+)= value of the fixed-point sums in acc; acc is left zero
void fixed_to_float(Tensor& acc, Tensor& out, bool add) {
  check_cuda(acc, "acc");
  check_cuda(out, "out");
  TORCH_CHECK(acc.scalar_type() == torch::kInt64 && acc.numel() == out.numel(),
              "fixed_to_float: acc must be int64 with as many elements as out");
  const int code = dtype_code(out, "out");
  TORCH_CHECK(code != LSE_FIXED64 && (!add || code == LSE_F32), "fixed_to_float: bad out dtype");
  done(lse_fixed_to_float(acc.data_ptr(), out.data_ptr(), code, add ? 1 : 0, (long long)acc.numel(), stream()),
       "fixed_to_float");
}

// ------------------------------------------------------------------ attention libraries
struct AttnLib {
  void* handle;
  int (*head_dim)(void);
  int (*q_tile)(int);
  size_t (*scratch_floats)(int, int, int);
  int (*decode_blocks_per_sm)(int, int, int);
  int (*decode_takes_sums)(int, int, int);
  int (*prefill)(const LseAttnArgs*, cudaStream_t);
  int (*decode)(const LseAttnArgs*, cudaStream_t);
};
std::map<int, AttnLib>& libs() {
  static std::map<int, AttnLib> m;
  return m;
}

void load_attention_library(const std::string& path, int64_t head_dim) {
  if (libs().count((int)head_dim)) return;
  void* h = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
  TORCH_CHECK(h, "cannot load attention library ", path, ": ", dlerror());
  AttnLib lib;
  lib.handle = h;
  lib.head_dim = (int (*)(void))dlsym(h, "lse_attn_head_dim");
  lib.q_tile = (int (*)(int))dlsym(h, "lse_attn_q_tile");
  lib.scratch_floats = (size_t(*)(int, int, int))dlsym(h, "lse_attn_decode_scratch_floats");
  lib.decode_blocks_per_sm = (int (*)(int, int, int))dlsym(h, "lse_attn_decode_blocks_per_sm");
  lib.decode_takes_sums = (int (*)(int, int, int))dlsym(h, "lse_attn_decode_takes_sums");
  lib.prefill = (int (*)(const LseAttnArgs*, cudaStream_t))dlsym(h, "lse_attn_prefill");
  lib.decode = (int (*)(const LseAttnArgs*, cudaStream_t))dlsym(h, "lse_attn_decode");
  TORCH_CHECK(lib.head_dim && lib.q_tile && lib.scratch_floats && lib.decode_blocks_per_sm &&
                  lib.decode_takes_sums && lib.prefill && lib.decode,
              "attention library ", path, " lacks an entry point");
  TORCH_CHECK(lib.head_dim() == head_dim, "attention library ", path, " was built for head size ",
              num(lib.head_dim()), ", not ", num(head_dim));
  libs()[(int)head_dim] = lib;
}

const AttnLib& attn_lib(int64_t D) {
  auto it = libs().find((int)D);
  TORCH_CHECK(it != libs().end(), "no attention library loaded for head size ", num(D));
  return it->second;
}

int64_t attention_q_tile(int64_t D, bool bf16, int64_t force_kernel) {
  const AttnLib& lib = attn_lib(D);
  return force_kernel == 1 ? lib.q_tile(LSE_F32) : lib.q_tile(bf16 ? LSE_BF16 : LSE_F32);
}

int64_t attention_scratch_floats(int64_t D, int64_t num_decode, int64_t num_heads, int64_t splits) {
  return (int64_t)attn_lib(D).scratch_floats((int)num_decode, (int)num_heads, (int)splits);
}

int64_t attention_decode_blocks_per_sm(int64_t D, bool bf16, int64_t num_heads, int64_t num_kv_heads) {
  return attn_lib(D).decode_blocks_per_sm(bf16 ? LSE_BF16 : LSE_F32, (int)num_heads, (int)num_kv_heads);
}

// q: the fused projection [T, q_width_total] whose first num_heads*D columns are the queries, or
// any [T, >= num_heads*D] tensor with unit column stride.
void paged_attention(const Tensor& q, Tensor& out, const Tensor& k_pages, const Tensor& v_pages,
                     int64_t num_heads, int64_t num_kv_heads, int64_t D, double scale,
                     int64_t window, const Tensor& block_tables, const Tensor& ctx_lens,
                     const Tensor& cu_q, const OptTensor& tiles, int64_t num_tiles,
                     const OptTensor& decode_seqs, int64_t num_decode, int64_t num_splits,
                     const OptTensor& scratch, int64_t force_kernel, const OptTensor& head_scale,
                     const OptTensor& slopes, int64_t chunk, const OptTensor& sinks, int64_t keep_first) {
  const AttnLib& lib = attn_lib(D);
  TORCH_CHECK(q.is_cuda() && q.dim() == 2 && q.stride(1) == 1 && q.size(1) >= num_heads * D,
              "paged_attention: q must be [T, >= heads*head_dim] with unit column stride");
  check_cuda(out, "out");
  check_cuda(k_pages, "k_pages");
  check_cuda(v_pages, "v_pages");
  check_i32(block_tables, "block_tables");
  check_i32(ctx_lens, "ctx_lens");
  check_i32(cu_q, "cu_q");
  TORCH_CHECK(out.dim() == 2 && out.size(0) == q.size(0) && out.size(1) == num_heads * D,
              "paged_attention: out must be [T, heads*head_dim]");
  // a bfloat16 call may ask for its results unrounded, in a float32 out
  const bool out_f32 = q.scalar_type() == torch::kBFloat16 && out.scalar_type() == torch::kFloat32;
  TORCH_CHECK((out.scalar_type() == q.scalar_type() || out_f32) && k_pages.scalar_type() == q.scalar_type() &&
                  v_pages.scalar_type() == q.scalar_type(),
              "paged_attention: q, out and pages must share a dtype (out may be float32 beside bfloat16)");
  TORCH_CHECK(k_pages.dim() == 4 && k_pages.size(1) == num_kv_heads && k_pages.size(3) == D &&
                  v_pages.sizes() == k_pages.sizes(),
              "paged_attention: pages must be [pages, kv_heads, page_tokens, head_dim]");
  TORCH_CHECK(block_tables.dim() == 2 && cu_q.size(0) == ctx_lens.size(0) + 1 &&
                  block_tables.size(0) >= ctx_lens.size(0),
              "paged_attention: per-sequence arrays disagree");
  TORCH_CHECK((reinterpret_cast<uintptr_t>(q.data_ptr()) % 16) == 0 &&
                  (q.stride(0) * q.element_size()) % 16 == 0,
              "paged_attention: q rows must be 16-byte aligned");
  LseAttnArgs a{};
  a.dtype = dtype_code(q, "q");
  a.q = q.data_ptr();
  a.q_row_stride = q.stride(0);
  a.out_f32 = out_f32 ? 1 : 0;
  a.out = out.data_ptr();
  a.out_row_stride = out.stride(0);
  a.k_pages = k_pages.data_ptr();
  a.v_pages = v_pages.data_ptr();
  a.num_heads = (int)num_heads;
  a.num_kv_heads = (int)num_kv_heads;
  a.page_tokens = (int)k_pages.size(2);
  a.window = (int)window;
  a.scale = (float)scale;
  a.block_tables = block_tables.data_ptr<int>();
  a.table_stride = (int)block_tables.size(1);
  a.ctx_lens = ctx_lens.data_ptr<int>();
  a.cu_q = cu_q.data_ptr<int>();
  a.force_simt = (int)force_kernel;
  a.num_rows = q.size(0);
  a.num_pages = k_pages.size(0);
  a.error_flag = error_flag();
  if (head_scale) {
    check_f32(*head_scale, "head_scale");
    TORCH_CHECK(head_scale->numel() == num_heads, "paged_attention: head_scale needs one value per head");
    a.head_scale = head_scale->data_ptr<float>();
  }
  if (slopes) {
    check_f32(*slopes, "slopes");
    TORCH_CHECK(slopes->numel() == num_heads, "paged_attention: slopes needs one value per head");
    a.slopes = slopes->data_ptr<float>();
  }
  TORCH_CHECK(chunk >= 0, "paged_attention: chunk must not be negative");
  a.chunk = (int)chunk;
  TORCH_CHECK(keep_first >= 0 && !(keep_first > 0 && chunk > 0), "paged_attention: keep_first must not be negative, and not with chunks");
  a.keep_first = (int)keep_first;
  if (sinks) {
    check_f32(*sinks, "sinks");
    TORCH_CHECK(sinks->numel() == num_heads, "paged_attention: sinks needs one value per head");
    a.sinks = sinks->data_ptr<float>();
  }
  if (num_tiles > 0) {
    TORCH_CHECK(tiles.has_value(), "paged_attention: num_tiles > 0 without tiles");
    check_i32(*tiles, "tiles");
    TORCH_CHECK(tiles->numel() >= 2 * num_tiles, "paged_attention: tiles too short");
    a.tiles = tiles->data_ptr<int>();
    a.num_tiles = (int)num_tiles;
    done(lib.prefill(&a, stream()), "paged_attention (portions)");
  }
  if (num_decode > 0) {
    TORCH_CHECK(decode_seqs.has_value(), "paged_attention: num_decode > 0 without decode_seqs");
    check_i32(*decode_seqs, "decode_seqs");
    TORCH_CHECK(decode_seqs->numel() >= num_decode, "paged_attention: decode_seqs too short");
    a.decode_seqs = decode_seqs->data_ptr<int>();
    a.num_decode = (int)num_decode;
    a.num_splits = (int)num_splits;
    if (num_splits > 1) {
      TORCH_CHECK(scratch.has_value(), "paged_attention: num_splits > 1 needs scratch");
      check_f32(*scratch, "scratch");
      TORCH_CHECK((size_t)scratch->numel() >=
                      lib.scratch_floats((int)num_decode, (int)num_heads, (int)num_splits),
                  "paged_attention: scratch too small");
      a.scratch = scratch->data_ptr<float>();
    }
    done(lib.decode(&a, stream()), "paged_attention (single tokens)");
  }
}

// ------------------------------------------------------------------ state mixers, branch norms
int out_code(const Tensor& t, const char* what) {
  const int c = dtype_code(t, what);
  TORCH_CHECK(c == LSE_F32 || c == LSE_BF16, what, ": dtype must be float32 or bfloat16");
  return c;
}

// ------------------------------------------------------------------ embeddings, latent attention, experts
void hashed_pair_add(Tensor& x, const Tensor& table, Tensor& state, const Tensor& ids,
                     const Tensor& positions, const Tensor& token_seq, const Tensor& cu_q,
                     const Tensor& slots, int64_t buckets, int64_t mul_prev, int64_t mul_cur) {
  check_f32(x, "x");
  check_cuda(table, "table");
  check_i32(ids, "ids");
  check_i32(positions, "positions");
  check_i32(token_seq, "token_seq");
  check_i32(cu_q, "cu_q");
  check_i32(slots, "slots");
  TORCH_CHECK(state.is_cuda() && state.is_contiguous() && state.scalar_type() == torch::kInt32,
              "hashed_pair_add: state must be a contiguous int32 CUDA tensor");
  const int T = (int)x.size(0), W = (int)x.size(1);
  TORCH_CHECK(x.dim() == 2 && table.dim() == 2 && table.size(1) == W && table.size(0) == buckets + 1,
              "hashed_pair_add: table must be [buckets + 1, width]");
  TORCH_CHECK(ids.numel() == T && positions.numel() == T && token_seq.numel() == T &&
                  cu_q.numel() == slots.numel() + 1 && state.numel() >= 1,
              "hashed_pair_add: lengths differ");
  TORCH_CHECK(buckets > 0 && mul_prev >= 0 && mul_cur >= 0, "hashed_pair_add: bad constants");
  done(lse_hashed_pair_add(x.data_ptr<float>(), table.data_ptr(), out_code(table, "table"),
                           state.data_ptr<int>(), ids.data_ptr<int>(), positions.data_ptr<int>(),
                           token_seq.data_ptr<int>(), cu_q.data_ptr<int>(), slots.data_ptr<int>(), T, (int)slots.numel(), W,
                           (long long)buckets, (long long)mul_prev, (long long)mul_cur, stream()),
       "hashed_pair_add");
}

void sinusoid_add(Tensor& x, const Tensor& positions, const Tensor& freq) {
  check_f32(x, "x");
  check_i32(positions, "positions");
  check_f32(freq, "freq");
  TORCH_CHECK(x.dim() == 2 && positions.numel() == x.size(0) && freq.numel() * 2 >= x.size(1),
              "sinusoid_add: need x [T, W], positions [T] and freq [ceil(W / 2)]");
  done(lse_sinusoid_add(x.data_ptr<float>(), positions.data_ptr<int>(), freq.data_ptr<float>(),
                        (int)x.size(0), (int)x.size(1), stream()),
       "sinusoid_add");
}

void latent_write(const Tensor& proj, int64_t col0, int64_t R, const Tensor& weight, double eps,
                  Tensor& pages, const Tensor& positions, const Tensor& token_seq,
                  const Tensor& block_tables) {
  check_cuda(proj, "proj");
  check_f32(weight, "weight");
  check_cuda(pages, "pages");
  check_i32(positions, "positions");
  check_i32(token_seq, "token_seq");
  check_i32(block_tables, "block_tables");
  TORCH_CHECK(proj.dim() == 2 && col0 >= 0 && R > 0 && col0 + R <= proj.size(1), "latent_write: columns outside proj");
  TORCH_CHECK(pages.dim() == 4 && pages.size(1) == 1 && pages.size(3) >= R,
              "latent_write: pages must be [pages, 1, page_tokens, >= rank]");
  TORCH_CHECK(weight.numel() == R, "latent_write: one weight per latent dim");
  const int T = (int)proj.size(0);
  TORCH_CHECK(positions.numel() == T && token_seq.numel() == T && block_tables.dim() == 2,
              "latent_write: lengths differ");
  done(lse_latent_write(proj.data_ptr(), out_code(proj, "proj"), proj.size(1), (int)col0, (int)R,
                        (int)pages.size(3), weight.data_ptr<float>(), (float)eps, pages.data_ptr(),
                        out_code(pages, "pages"), positions.data_ptr<int>(), token_seq.data_ptr<int>(),
                        block_tables.data_ptr<int>(), (int)block_tables.size(1), (int)pages.size(2), T,
                        stream()),
       "latent_write");
}

// out[t, h, :] = w[h] . a[t, col0 + h*K : col0 + (h+1)*K]     w [H, N, K], out [T, H*N]
const float* opt_f32(const OptTensor& t, int64_t n, const char* what);

// a_head_cols / out_head_cols (0: K / N): columns from one head to the next in a and in out; a head's
// result may be the first N columns of a wider slot of out.
void head_linear(const Tensor& a, int64_t col0, const Tensor& w, Tensor& out, int64_t kind, int64_t a_head_cols,
                 int64_t out_head_cols) {
  check_cuda(a, "a");
  check_cuda(w, "w");
  check_cuda(out, "out");
  TORCH_CHECK(a.dim() == 2 && w.dim() == 3 && out.dim() == 2, "head_linear: need a [T, >= H*K], w [H, N, K], out [T, H*N]");
  const int64_t H = w.size(0), N = w.size(1), K = w.size(2);
  const int64_t ah = a_head_cols > 0 ? a_head_cols : K, oh = out_head_cols > 0 ? out_head_cols : N;
  TORCH_CHECK(ah >= K && oh >= N && col0 >= 0 && col0 + (H - 1) * ah + K <= a.size(1) && out.size(0) == a.size(0) &&
                  out.size(1) == H * oh,
              "head_linear: shapes disagree");
  done(lse_head_linear(a.data_ptr(), out_code(a, "a"), a.size(1), col0, w.data_ptr(), out_code(w, "w"),
                       out.data_ptr(), out_code(out, "out"), (int)a.size(0), (int)H, (int)N, (int)K, (int)kind, stream(),
                       ah, oh, out.size(1)),
       "head_linear");
}

void moe_route(const Tensor& h, const Tensor& router, int64_t E, int64_t top, Tensor& idx, Tensor& wts,
               const OptTensor& gate, const OptTensor& bias, int64_t mode) {
  check_cuda(h, "h");
  check_f32(router, "router");
  check_i32(idx, "idx");
  check_f32(wts, "wts");
  const int64_t T = h.size(0), W = h.size(1);
  const int has_gate = gate.has_value() ? 1 : 0;
  TORCH_CHECK(h.dim() == 2 && router.dim() == 2 && router.size(1) == W && router.size(0) == E + has_gate,
              "moe_route: router must be [experts (+1 with a gate), width]");
  TORCH_CHECK(idx.numel() == T * top && wts.numel() == T * top, "moe_route: idx and wts must be [T, top]");
  float* g = nullptr;
  if (gate) {
    check_f32(*gate, "gate");
    TORCH_CHECK(gate->numel() == T, "moe_route: gate must be [T]");
    g = gate->data_ptr<float>();
  }
  done(lse_moe_route(h.data_ptr(), out_code(h, "h"), router.data_ptr<float>(), (int)T, (int)W, (int)E,
                     has_gate, (int)top, idx.data_ptr<int>(), wts.data_ptr<float>(), g, stream(),
                     opt_f32(bias, E, "router bias"), (int)mode),
       "moe_route");
}

// work: int32 [>= (E + 1) + 2 n + 2 max_tiles + 1] holding offsets | perm | pos_of | tile_batch |
// tile_row0 | num_tiles, max_tiles = n / tile_rows + E.
int64_t moe_max_tiles(int64_t n, int64_t E, int64_t tile_rows) { return n / tile_rows + E; }
int64_t moe_tile_rows(int64_t kind) { return kind == 3 ? lse_expert_linear_tc_tile_rows() : lse_moe_tile_rows(); }

void moe_sort(const Tensor& idx, int64_t E, Tensor& work, int64_t tile_rows) {
  check_i32(idx, "idx");
  check_i32(work, "work");
  TORCH_CHECK(tile_rows > 0, "moe_sort: tile_rows must be positive");
  const int64_t n = idx.numel(), mt = moe_max_tiles(n, E, tile_rows);
  TORCH_CHECK(work.numel() >= E + 1 + 2 * n + 2 * mt + 1, "moe_sort: work too small");
  int* p = work.data_ptr<int>();
  done(lse_moe_sort(idx.data_ptr<int>(), (int)n, (int)E, (int)tile_rows, p, p + E + 1, p + E + 1 + n,
                    p + E + 1 + 2 * n, p + E + 1 + 2 * n + mt, p + E + 1 + 2 * n + 2 * mt, stream()),
       "moe_sort");
}

// out[r] = w[expert of sorted row r] . a-row(r); gather: a-row(r) = a[choice / top] * wts[choice].
// kind 0..2: see lse_expert_linear (tiles of lse_moe_tile_rows() rows); kind 3: tcgen05 tensor cores
// (bfloat16, K a multiple of 8, tiles of lse_expert_linear_tc_tile_rows() rows; with top the rows are
// first gathered into `gathered` [n, K]).
void expert_linear(const Tensor& a, const Tensor& w, Tensor& out, const Tensor& work, int64_t n, int64_t top,
                   const OptTensor& wts, int64_t kind, const OptTensor& gathered) {
  check_cuda(a, "a");
  check_cuda(w, "w");
  check_f32(out, "out");
  check_i32(work, "work");
  TORCH_CHECK(a.dim() == 2 && w.dim() == 3 && out.dim() == 2 && w.size(2) == a.size(1) && out.size(0) == n &&
                  out.size(1) == w.size(1),
              "expert_linear: need a [rows, K], w [E, N, K], out [n, N]");
  const int64_t E = w.size(0), mt = moe_max_tiles(n, E, moe_tile_rows(kind));
  TORCH_CHECK(work.numel() >= E + 1 + 2 * n + 2 * mt + 1, "expert_linear: work too small");
  const bool gather = top > 0;
  TORCH_CHECK(gather ? a.size(0) * top == n : a.size(0) == n, "expert_linear: rows of a disagree with n");
  const float* sc = nullptr;
  if (wts) {
    check_f32(*wts, "wts");
    TORCH_CHECK(gather && wts->numel() == n, "expert_linear: wts must be [n] and needs top");
    sc = wts->data_ptr<float>();
  }
  const int* p = work.data_ptr<int>();
  const int *perm = p + E + 1, *tile_batch = p + E + 1 + 2 * n, *tile_row0 = tile_batch + mt, *num_tiles = tile_row0 + mt;
  if (kind == 3) {
    TORCH_CHECK(a.scalar_type() == torch::kBFloat16 && w.scalar_type() == torch::kBFloat16 && a.size(1) % 8 == 0,
                "expert_linear: the tcgen05 kernel takes bfloat16 rows of a multiple of 8 elements");
    const void* rows = a.data_ptr();
    if (gather) {
      TORCH_CHECK(gathered.has_value(), "expert_linear: the tcgen05 kernel needs room for the gathered rows");
      check_cuda(*gathered, "gathered");
      TORCH_CHECK(gathered->scalar_type() == torch::kBFloat16 && gathered->numel() >= n * a.size(1),
                  "expert_linear: gathered must be bfloat16 [n, K]");
      done(lse_moe_gather_rows(a.data_ptr(), perm, (int)top, gathered->data_ptr(), (int)n, (int)a.size(1), stream()),
           "expert_linear (gather)");
      rows = gathered->data_ptr();
    }
    done(lse_expert_linear_tc(rows, w.data_ptr(), out.data_ptr<float>(), (int)n, (int)E, (int)w.size(1),
                              (int)w.size(2), sc, perm, p, tile_batch, tile_row0, num_tiles, (int)mt, error_flag(),
                              stream()),
         "expert_linear (tcgen05)");
    return;
  }
  done(lse_expert_linear(a.data_ptr(), out_code(a, "a"), a.size(1), gather ? perm : nullptr,
                         gather ? (int)top : 1, sc, w.data_ptr(), out_code(w, "w"), out.data_ptr<float>(),
                         (int)n, (int)w.size(1), (int)w.size(2), p, tile_batch, tile_row0, num_tiles, (int)mt,
                         (int)kind, stream()),
       "expert_linear");
}

void moe_combine(const Tensor& y, const Tensor& work, int64_t E, int64_t top, const OptTensor& shared_out,
                 const OptTensor& gate, Tensor& out, bool accumulate, const OptTensor& wts) {
  check_f32(y, "y");
  check_i32(work, "work");
  check_f32(out, "out");
  const int64_t n = y.size(0), T = out.size(0), W = out.size(1);
  TORCH_CHECK(y.dim() == 2 && out.dim() == 2 && y.size(1) == W && n == T * top, "moe_combine: shapes disagree");
  const float *sp = nullptr, *gp = nullptr;
  if (shared_out) {
    check_f32(*shared_out, "shared_out");
    TORCH_CHECK(shared_out->sizes() == out.sizes(), "moe_combine: shared_out needs out's shape");
    sp = shared_out->data_ptr<float>();
    if (gate) {
      check_f32(*gate, "gate");
      TORCH_CHECK(gate->numel() == T, "moe_combine: gate must be [T]");
      gp = gate->data_ptr<float>();
    }
  }
  done(lse_moe_combine(y.data_ptr<float>(), work.data_ptr<int>() + E + 1 + n, (int)top, sp, gp,
                       out.data_ptr<float>(), accumulate ? 1 : 0, (int)T, (int)W, stream(), opt_f32(wts, n, "experts' weights")),
       "moe_combine");
}

void cast_f32(const Tensor& x, Tensor& out) {
  check_f32(x, "x");
  check_cuda(out, "out");
  TORCH_CHECK(out.numel() == x.numel(), "cast: sizes differ");
  done(lse_cast(x.data_ptr<float>(), out.data_ptr(), out_code(out, "out"), x.numel(), stream()), "cast");
}

void token_shift(const Tensor& x, const Tensor& mix, Tensor& state, Tensor& out, const Tensor& token_seq,
                 const Tensor& cu_q, const Tensor& ctx_lens, const Tensor& slots) {
  check_f32(x, "x");
  check_f32(mix, "mix");
  check_state(state, "state", 1);
  check_cuda(out, "out");
  check_i32(token_seq, "token_seq");
  check_i32(cu_q, "cu_q");
  check_i32(ctx_lens, "ctx_lens");
  check_i32(slots, "slots");
  TORCH_CHECK(x.dim() == 2 && out.sizes() == x.sizes() && state.dim() == 2 && state.size(1) == x.size(1) &&
                  mix.numel() == x.size(1),
              "token_shift: x and out must be [T, W], state [slots, W], mix [W]");
  TORCH_CHECK(token_seq.numel() >= x.size(0) && cu_q.numel() == ctx_lens.numel() + 1 &&
                  slots.numel() >= ctx_lens.numel(),
              "token_shift: the batch arrays disagree");
  done(lse_token_shift(x.data_ptr<float>(), mix.data_ptr<float>(), state.data_ptr<float>(), out.data_ptr(),
                       out_code(out, "out"), token_seq.data_ptr<int>(), cu_q.data_ptr<int>(),
                       ctx_lens.data_ptr<int>(), slots.data_ptr<int>(), (int)x.size(0), (int)x.size(1),
                       stream()),
       "token_shift");
}

const float* opt_f32(const OptTensor& t, int64_t n, const char* what) {
  if (!t) return nullptr;
  check_f32(*t, what);
  TORCH_CHECK(t->numel() == n, what, ": expected ", num(n), " values, got ", num(t->numel()));
  return t->data_ptr<float>();
}

void rmsnorm_add(Tensor& x, const Tensor& a, const OptTensor& b, const OptTensor& wa, const OptTensor& wb,
                 double ca, double cb, double eps_in, const Tensor& w, double eps, const OptTensor& out,
                 const OptTensor& then_w, double then_eps) {
  check_f32(x, "x");
  check_cuda(a, "a");
  check_f32(w, "w");
  TORCH_CHECK(x.dim() == 2 && a.sizes() == x.sizes() && w.numel() == x.size(1), "rmsnorm_add: bad shapes");
  const int branch_code = dtype_code(a, "a");  // float32, or the fixed-point sums of a few-rows product
  TORCH_CHECK(branch_code == LSE_F32 || branch_code == LSE_FIXED64, "rmsnorm_add: a must be float32 or sums");
  const int64_t H = x.size(1);
  const void* bp = nullptr;
  if (b) {
    check_cuda(*b, "b");
    TORCH_CHECK(b->sizes() == x.sizes() && wa && wb, "rmsnorm_add: a second branch needs its shape and both weights");
    TORCH_CHECK(b->scalar_type() == a.scalar_type(), "rmsnorm_add: both branches must be of one kind");
    bp = b->data_ptr();
  }
  TORCH_CHECK(branch_code == LSE_F32 || H * (b ? 2 : 1) * 4 <= 48 * 1024, "rmsnorm_add: rows of sums are too long");
  void* op = nullptr;
  int oc = LSE_F32;
  if (out) {
    check_cuda(*out, "out");
    TORCH_CHECK(out->sizes() == x.sizes(), "rmsnorm_add: out shape differs from x");
    op = out->data_ptr();
    oc = out_code(*out, "out");
  }
  TORCH_CHECK(!then_w || out, "rmsnorm_add: the norm that follows needs an output tensor");
  done(lse_rmsnorm_add(x.data_ptr<float>(), a.data_ptr(), bp, branch_code, opt_f32(wa, H, "wa"), opt_f32(wb, H, "wb"),
                       (float)ca, (float)cb, (float)eps_in, w.data_ptr<float>(), (float)eps, op, oc,
                       opt_f32(then_w, H, "then_w"), (float)then_eps, (int)x.size(0), (int)H, stream()),
       "rmsnorm_add");
}

void mix_normed(const Tensor& a, const OptTensor& b, const Tensor& wa, const OptTensor& wb, double ca, double cb,
                double eps, Tensor& out) {
  check_f32(a, "a");
  check_f32(wa, "wa");
  check_f32(out, "out");
  TORCH_CHECK(a.dim() == 2 && out.sizes() == a.sizes() && wa.numel() == a.size(1), "mix_normed: bad shapes");
  const float* bp = nullptr;
  if (b) {
    check_f32(*b, "b");
    TORCH_CHECK(b->sizes() == a.sizes() && wb, "mix_normed: a second branch needs its shape and weight");
    bp = b->data_ptr<float>();
  }
  done(lse_mix_normed(a.data_ptr<float>(), bp, wa.data_ptr<float>(), opt_f32(wb, a.size(1), "wb"), (float)ca,
                      (float)cb, (float)eps, out.data_ptr<float>(), (int)a.size(0), (int)a.size(1), stream()),
       "mix_normed");
}

void gated_group_norm(const Tensor& o, const Tensor& proj, int64_t gate_offset, int64_t group,
                      const OptTensor& weight, double eps, bool sigmoid, Tensor& out) {
  check_f32(o, "o");
  check_f32(proj, "proj");
  check_cuda(out, "out");
  TORCH_CHECK(o.dim() == 2 && proj.dim() == 2 && proj.size(0) == o.size(0) && out.sizes() == o.sizes(),
              "gated_group_norm: o and out must be [T, N], proj [T, >= gate_offset + N]");
  const int64_t N = o.size(1);
  TORCH_CHECK(gate_offset >= 0 && gate_offset + N <= proj.size(1), "gated_group_norm: the gate lies outside proj");
  TORCH_CHECK(group > 0 && N % group == 0, "gated_group_norm: group must divide the row");
  done(lse_gated_group_norm(o.data_ptr<float>(), proj.data_ptr<float>() + gate_offset, proj.size(1), (int)o.size(0),
                            (int)N, (int)group, opt_f32(weight, N, "weight"), (float)eps, sigmoid ? 1 : 0,
                            out.data_ptr(), out_code(out, "out"), stream()),
       "gated_group_norm");
}

void norm_rope_kv_write(const Tensor& qkv, Tensor& q_out, int64_t nq, int64_t nk, int64_t D, bool v_from_k,
                        const OptTensor& qw, const OptTensor& kw, double eps, const Tensor& positions,
                        const Tensor& token_seq, const OptTensor& cos, const OptTensor& sin,
                        const OptTensor& k_pages, const OptTensor& v_pages, const Tensor& block_tables,
                        int64_t page_tokens, int64_t norm_dim) {
  check_f32(qkv, "qkv");
  TORCH_CHECK(norm_dim > 0 && norm_dim <= D, "norm_rope_kv_write: norm_dim must lie in 1..head_dim");
  check_cuda(q_out, "q_out");
  check_i32(positions, "positions");
  check_i32(token_seq, "token_seq");
  check_i32(block_tables, "block_tables");
  const int64_t heads = nq + nk + (v_from_k ? 0 : nk);
  TORCH_CHECK(qkv.dim() == 2 && qkv.size(1) >= heads * D, "norm_rope_kv_write: qkv width");
  TORCH_CHECK(D > 0 && D <= 256, "norm_rope_kv_write: head size must be at most 256");
  const int64_t T = qkv.size(0);
  TORCH_CHECK(q_out.dim() == 2 && q_out.size(0) == T && q_out.size(1) == nq * D, "norm_rope_kv_write: q_out shape");
  TORCH_CHECK(positions.numel() >= T && token_seq.numel() >= T && block_tables.dim() == 2,
              "norm_rope_kv_write: the batch arrays disagree");
  TORCH_CHECK(qw.has_value() == kw.has_value() && cos.has_value() == sin.has_value() &&
                  k_pages.has_value() == v_pages.has_value(),
              "norm_rope_kv_write: weights, tables and pages come in pairs");
  if (cos) {
    check_f32(*cos, "cos");
    check_f32(*sin, "sin");
    TORCH_CHECK(cos->dim() == 2 && cos->size(1) == D / 2 && sin->sizes() == cos->sizes() && D % 2 == 0,
                "norm_rope_kv_write: cos and sin must be [positions, head_dim / 2]");
  }
  void *kp = nullptr, *vp = nullptr;
  if (k_pages) {
    check_cuda(*k_pages, "k_pages");
    check_cuda(*v_pages, "v_pages");
    TORCH_CHECK(k_pages->scalar_type() == q_out.scalar_type() && v_pages->scalar_type() == q_out.scalar_type() &&
                    k_pages->dim() == 4 && k_pages->size(1) == nk && k_pages->size(2) == page_tokens &&
                    k_pages->size(3) == D && v_pages->sizes() == k_pages->sizes(),
                "norm_rope_kv_write: pages must be [pages, kv_heads, page_tokens, head_dim] of q_out's dtype");
    kp = k_pages->data_ptr();
    vp = v_pages->data_ptr();
  }
  done(lse_norm_rope_kv_write(qkv.data_ptr<float>(), q_out.data_ptr(), out_code(q_out, "q_out"), (int)T, (int)nq,
                              (int)nk, (int)D, v_from_k ? 1 : 0, opt_f32(qw, D, "q weight"), opt_f32(kw, D, "k weight"),
                              (float)eps, positions.data_ptr<int>(), token_seq.data_ptr<int>(),
                              cos ? cos->data_ptr<float>() : nullptr, sin ? sin->data_ptr<float>() : nullptr, kp, vp,
                              block_tables.data_ptr<int>(), (int)block_tables.size(1), (int)page_tokens,
                              (int)norm_dim, stream(), qkv.size(1)),
       "norm_rope_kv_write");
}

void decay_linear_attention(const Tensor& proj, Tensor& out, Tensor& state, const OptTensor& decay, const Tensor& cu_q,
                            const Tensor& ctx_lens, const Tensor& slots, int64_t H, int64_t dk, int64_t dv,
                            const OptTensor& cos, const OptTensor& sin, bool silu, double key_scale,
                            int64_t max_chunks, const OptTensor& chunks, const OptTensor& gate_z,
                            double decay_root, double query_scale) {
  check_f32(proj, "proj");
  check_f32(out, "out");
  check_state(state, "state", dk);
  TORCH_CHECK(decay.has_value() != gate_z.has_value(),
              "decay_linear_attention: give the decays per head or the logits of decays per channel and token");
  if (decay) check_f32(*decay, "decay");
  if (gate_z) {
    check_f32(*gate_z, "gate_z");
    TORCH_CHECK(gate_z->dim() == 2 && gate_z->size(0) == proj.size(0) && gate_z->size(1) >= H * dk && decay_root > 0,
                "decay_linear_attention: the decay logits must be [T, >= heads * key_dim] and the root positive");
  }
  check_i32(cu_q, "cu_q");
  check_i32(ctx_lens, "ctx_lens");
  check_i32(slots, "slots");
  TORCH_CHECK(proj.dim() == 2 && proj.size(1) >= 2 * H * dk + H * dv, "decay_linear_attention: proj is too narrow");
  TORCH_CHECK(out.dim() == 2 && out.size(0) == proj.size(0) && out.size(1) == H * dv,
              "decay_linear_attention: out must be [T, heads * value_dim]");
  TORCH_CHECK(state.dim() == 4 && state.size(1) == H && state.size(2) == dv && state.size(3) == dk,
              "decay_linear_attention: state must be [slots, heads, value_dim, key_dim]");
  TORCH_CHECK((!decay || decay->numel() == H) && cu_q.numel() == ctx_lens.numel() + 1 && slots.numel() >= ctx_lens.numel(),
              "decay_linear_attention: per-head or per-sequence arrays disagree");
  TORCH_CHECK(dk > 0 && dk <= 256 && dv > 0, "decay_linear_attention: key size must be at most 256");
  TORCH_CHECK(cos.has_value() == sin.has_value(), "decay_linear_attention: cos and sin go together");
  int rot = 0;
  if (cos) {
    check_f32(*cos, "cos");
    check_f32(*sin, "sin");
    TORCH_CHECK(cos->dim() == 2 && sin->sizes() == cos->sizes() && 2 * cos->size(1) <= dk,
                "decay_linear_attention: cos and sin must be [positions, rotated dims / 2]");
    rot = 2 * (int)cos->size(1);
  }
  float *chunk_ptr = nullptr, *chunk_decay = nullptr;
  if (max_chunks > 1) {
    TORCH_CHECK(chunks.has_value(), "decay_linear_attention: chunked portions need the scratch");
    check_f32(*chunks, "chunks");
    // every sequence of more than one chunk holds at most tokens / chunk + 1 of them
    const int64_t L = lse_linear_attention_chunk();
    const int64_t most = proj.size(0) / L + ctx_lens.numel();
    TORCH_CHECK(chunks->numel() >= most * H * (dv * dk + (gate_z ? dk : 0)),
                "decay_linear_attention: the scratch is too small");
    chunk_ptr = chunks->data_ptr<float>();
    if (gate_z) chunk_decay = chunk_ptr + most * H * dv * dk;  // behind the chunks' states
  }
  done(lse_decay_linear_attention(proj.data_ptr<float>(), proj.size(1), out.data_ptr<float>(), state.data_ptr<float>(),
                                  decay ? decay->data_ptr<float>() : nullptr, cu_q.data_ptr<int>(), ctx_lens.data_ptr<int>(),
                                  slots.data_ptr<int>(), (int)ctx_lens.numel(), (int)H, (int)dk, (int)dv,
                                  cos ? cos->data_ptr<float>() : nullptr, sin ? sin->data_ptr<float>() : nullptr, rot,
                                  silu ? 1 : 0, (float)key_scale, (int)max_chunks, chunk_ptr, stream(),
                                  gate_z ? gate_z->data_ptr<float>() : nullptr, gate_z ? gate_z->size(1) : 0,
                                  (float)decay_root, (float)query_scale, chunk_decay, (int)proj.size(0)),
       "decay_linear_attention");
}

bool attention_takes_sums(int64_t D, bool bf16, int64_t num_heads, int64_t num_kv_heads) {
  return attn_lib(D).decode_takes_sums(bf16 ? LSE_BF16 : LSE_F32, (int)num_heads, (int)num_kv_heads) != 0;
}

// Single tokens straight from the fixed-point sums of the fused q|k|v projection: rotation, cache
// write and attention in one launch; the sums are left zero. Every row of `sums` is one sequence's
// single token (row i belongs to sequence decode_seqs[i] through cu_q).
void paged_attention_from_sums(Tensor& sums, Tensor& out, Tensor& k_pages, Tensor& v_pages,
                               int64_t num_heads, int64_t num_kv_heads, int64_t D, double scale,
                               int64_t window, const Tensor& block_tables, const Tensor& ctx_lens,
                               const Tensor& cu_q, const Tensor& decode_seqs, int64_t num_splits,
                               const OptTensor& scratch, const OptTensor& cos, const OptTensor& sin) {
  const AttnLib& lib = attn_lib(D);
  check_cuda(sums, "sums");
  check_cuda(out, "out");
  check_cuda(k_pages, "k_pages");
  check_cuda(v_pages, "v_pages");
  check_i32(block_tables, "block_tables");
  check_i32(ctx_lens, "ctx_lens");
  check_i32(cu_q, "cu_q");
  check_i32(decode_seqs, "decode_seqs");
  const int64_t T = sums.size(0);
  TORCH_CHECK(sums.scalar_type() == torch::kInt64 && sums.dim() == 2 &&
                  sums.size(1) == (num_heads + 2 * num_kv_heads) * D,
              "paged_attention_from_sums: sums must be int64 [T, (heads + 2 kv_heads) * head_dim]");
  TORCH_CHECK(out.scalar_type() == torch::kBFloat16 && k_pages.scalar_type() == torch::kBFloat16 &&
                  v_pages.scalar_type() == torch::kBFloat16,
              "paged_attention_from_sums: out and pages must be bfloat16");
  TORCH_CHECK(out.dim() == 2 && out.size(0) == T && out.size(1) == num_heads * D,
              "paged_attention_from_sums: out must be [T, heads*head_dim]");
  TORCH_CHECK(k_pages.dim() == 4 && k_pages.size(1) == num_kv_heads && k_pages.size(3) == D &&
                  v_pages.sizes() == k_pages.sizes(),
              "paged_attention_from_sums: pages must be [pages, kv_heads, page_tokens, head_dim]");
  TORCH_CHECK(block_tables.dim() == 2 && cu_q.size(0) == ctx_lens.size(0) + 1 &&
                  block_tables.size(0) >= ctx_lens.size(0) && decode_seqs.numel() == T,
              "paged_attention_from_sums: per-sequence arrays disagree, or a row is not a single token");
  TORCH_CHECK(lib.decode_takes_sums(LSE_BF16, (int)num_heads, (int)num_kv_heads),
              "paged_attention_from_sums: not served for these head counts");
  TORCH_CHECK(cos.has_value() == sin.has_value(), "paged_attention_from_sums: cos and sin go together");
  LseAttnArgs a{};
  a.dtype = LSE_BF16;
  a.qkv_sums = reinterpret_cast<const long long*>(sums.data_ptr());
  if (cos) {
    check_f32(*cos, "cos");
    check_f32(*sin, "sin");
    TORCH_CHECK(cos->dim() == 2 && cos->size(1) == D / 2 && sin->sizes() == cos->sizes(),
                "paged_attention_from_sums: cos and sin must be [positions, head_dim / 2]");
    a.rope_cos = cos->data_ptr<float>();
    a.rope_sin = sin->data_ptr<float>();
  }
  a.out = out.data_ptr();
  a.out_row_stride = out.stride(0);
  a.k_pages = k_pages.data_ptr();
  a.v_pages = v_pages.data_ptr();
  a.num_heads = (int)num_heads;
  a.num_kv_heads = (int)num_kv_heads;
  a.page_tokens = (int)k_pages.size(2);
  a.window = (int)window;
  a.scale = (float)scale;
  a.block_tables = block_tables.data_ptr<int>();
  a.table_stride = (int)block_tables.size(1);
  a.ctx_lens = ctx_lens.data_ptr<int>();
  a.cu_q = cu_q.data_ptr<int>();
  a.num_rows = T;
  a.num_pages = k_pages.size(0);
  a.error_flag = error_flag();
  a.decode_seqs = decode_seqs.data_ptr<int>();
  a.num_decode = (int)T;
  a.num_splits = (int)num_splits;
  if (num_splits > 1) {
    TORCH_CHECK(scratch.has_value(), "paged_attention_from_sums: num_splits > 1 needs scratch");
    check_f32(*scratch, "scratch");
    TORCH_CHECK((size_t)scratch->numel() >= lib.scratch_floats((int)T, (int)num_heads, (int)num_splits),
                "paged_attention_from_sums: scratch too small");
    a.scratch = scratch->data_ptr<float>();
  }
  if (T > 0) done(lib.decode(&a, stream()), "paged_attention_from_sums");
}

// ------------------------------------------------------------------ sampling
void sample(const Tensor& logits, const Tensor& temperature, const Tensor& top_k,
            const Tensor& top_p, const Tensor& min_p, const Tensor& seed, const Tensor& draw,
            Tensor& out, const OptTensor& scratch, int64_t which) {
  check_f32(logits, "logits");
  check_f32(temperature, "temperature");
  check_i32(top_k, "top_k");
  check_f32(top_p, "top_p");
  check_f32(min_p, "min_p");
  check_cuda(seed, "seed");
  TORCH_CHECK(seed.scalar_type() == torch::kInt64, "seed must be int64");
  check_i32(draw, "draw");
  check_i32(out, "out");
  const int R = (int)logits.size(0);
  TORCH_CHECK(logits.dim() == 2 && temperature.numel() == R && top_k.numel() == R &&
                  top_p.numel() == R && min_p.numel() == R && seed.numel() == R &&
                  draw.numel() == R && out.numel() == R,
              "sample: one parameter per row of logits is needed");
  int* sc = nullptr;
  int sc_rows = 0;
  if (scratch) {  // several blocks per row for rows without a cut, if it was made for R rows or more
    check_i32(*scratch, "scratch");
    sc = scratch->data_ptr<int>();
    sc_rows = (int)(scratch->numel() / (int64_t)lse_sample_scratch_ints(1));
  }
  done(lse_sample(logits.data_ptr<float>(), R, (int)logits.size(1), temperature.data_ptr<float>(),
                  top_k.data_ptr<int>(), top_p.data_ptr<float>(), min_p.data_ptr<float>(),
                  reinterpret_cast<const uint64_t*>(seed.data_ptr<int64_t>()), draw.data_ptr<int>(),
                  out.data_ptr<int>(), sc, sc_rows, (int)which, stream()),
       "sample");
}

void logsumexp(const Tensor& logits, Tensor& out) {
  check_f32(logits, "logits");
  check_f32(out, "out");
  TORCH_CHECK(logits.dim() == 2 && out.numel() == logits.size(0), "logsumexp: shapes");
  done(lse_logsumexp(logits.data_ptr<float>(), (int)logits.size(0), (int)logits.size(1),
                     out.data_ptr<float>(), stream()),
       "logsumexp");
}

void apply_penalties(Tensor& logits, const Tensor& row, const Tensor& token, const Tensor& count,
                     const Tensor& presence, const Tensor& frequency, const Tensor& repetition) {
  check_f32(logits, "logits");
  check_i32(row, "row");
  check_i32(token, "token");
  check_i32(count, "count");
  check_f32(presence, "presence");
  check_f32(frequency, "frequency");
  check_f32(repetition, "repetition");
  const int n = (int)row.numel();
  TORCH_CHECK(token.numel() == n && count.numel() == n && presence.numel() == n &&
                  frequency.numel() == n && repetition.numel() == n,
              "apply_penalties: lengths differ");
  done(lse_apply_penalties(logits.data_ptr<float>(), (int)logits.size(1), row.data_ptr<int>(),
                           token.data_ptr<int>(), count.data_ptr<int>(), presence.data_ptr<float>(),
                           frequency.data_ptr<float>(), repetition.data_ptr<float>(), n, stream()),
       "apply_penalties");
}

void token_state_add(Tensor& state, const Tensor& slot, const Tensor& token, const Tensor& in_prompt) {
  check_i32(state, "state");
  check_i32(slot, "slot");
  check_i32(token, "token");
  check_i32(in_prompt, "in_prompt");
  TORCH_CHECK(state.dim() == 2, "token_state_add: state must be [slots, vocab]");
  const int n = (int)slot.numel();
  TORCH_CHECK(token.numel() == n && in_prompt.numel() == n, "token_state_add: lengths differ");
  done(lse_token_state_add(state.data_ptr<int>(), (int)state.size(1), slot.data_ptr<int>(),
                           token.data_ptr<int>(), in_prompt.data_ptr<int>(), n, stream()),
       "token_state_add");
}

void apply_penalties_dense(Tensor& logits, const Tensor& row, const Tensor& slot, const Tensor& presence,
                           const Tensor& frequency, const Tensor& repetition, const Tensor& state) {
  check_f32(logits, "logits");
  check_i32(row, "row");
  check_i32(slot, "slot");
  check_f32(presence, "presence");
  check_f32(frequency, "frequency");
  check_f32(repetition, "repetition");
  check_i32(state, "state");
  const int n = (int)row.numel();
  TORCH_CHECK(slot.numel() == n && presence.numel() == n && frequency.numel() == n &&
                  repetition.numel() == n,
              "apply_penalties_dense: lengths differ");
  TORCH_CHECK(logits.dim() == 2 && state.dim() == 2 && state.size(1) == logits.size(1),
              "apply_penalties_dense: state must be [slots, vocab]");
  done(lse_apply_penalties_dense(logits.data_ptr<float>(), (int)logits.size(1), row.data_ptr<int>(),
                                 slot.data_ptr<int>(), presence.data_ptr<float>(),
                                 frequency.data_ptr<float>(), repetition.data_ptr<float>(),
                                 state.data_ptr<int>(), n, stream()),
       "apply_penalties_dense");
}

void ban_tokens(Tensor& logits, const Tensor& row, const Tensor& token) {
  check_f32(logits, "logits");
  check_i32(row, "row");
  check_i32(token, "token");
  TORCH_CHECK(row.numel() == token.numel(), "ban_tokens: lengths differ");
  done(lse_ban_tokens(logits.data_ptr<float>(), (int)logits.size(1), row.data_ptr<int>(),
                      token.data_ptr<int>(), (int)row.numel(), stream()),
       "ban_tokens");
}

}  // namespace

// ---- latent attention with a rotated key part, gates, plain activations (rotary_latent.cu) ----
// proj [T, stride]: columns q_col0 .. +Rq are the query latent (Rq = q_weight's size; no q_weight:
// none), columns kv_col0 .. +R the key/value latent and the Dr columns behind them the key part
// that is turned by the position (R = kv_weight's size; no kv_weight: the layer writes no rows).
void latent_rope_write(const Tensor& proj, int64_t q_col0, const OptTensor& q_weight, const OptTensor& cq,
                       int64_t kv_col0, const OptTensor& kv_weight, int64_t Dr, int64_t rot, double eps,
                       const OptTensor& cos, const OptTensor& sin, const OptTensor& pages, const Tensor& positions,
                       const Tensor& token_seq, const Tensor& block_tables) {
  check_cuda(proj, "proj");
  check_i32(positions, "positions");
  check_i32(token_seq, "token_seq");
  check_i32(block_tables, "block_tables");
  TORCH_CHECK(proj.dim() == 2 && block_tables.dim() == 2, "latent_rope_write: proj and block_tables are matrices");
  const int64_t T = proj.size(0);
  TORCH_CHECK(positions.numel() >= T && token_seq.numel() >= T, "latent_rope_write: the batch arrays are too short");
  int64_t Rq = 0, R = 0, Rp = 0, page_tokens = 1;
  int dtype = -1;
  void *cq_ptr = nullptr, *pages_ptr = nullptr;
  if (q_weight) {
    check_f32(*q_weight, "q_weight");
    Rq = q_weight->numel();
    TORCH_CHECK(cq.has_value(), "latent_rope_write: a query latent needs its output");
    check_cuda(*cq, "cq");
    TORCH_CHECK(cq->dim() == 2 && cq->size(0) == T && cq->size(1) == Rq && q_col0 >= 0 && q_col0 + Rq <= proj.size(1),
                "latent_rope_write: cq must be [T, query rank] and its columns lie in proj");
    dtype = out_code(*cq, "cq");
    cq_ptr = cq->data_ptr();
  }
  if (kv_weight) {
    check_f32(*kv_weight, "kv_weight");
    R = kv_weight->numel();
    TORCH_CHECK(pages.has_value(), "latent_rope_write: a key/value latent needs its pages");
    check_cuda(*pages, "pages");
    TORCH_CHECK(pages->dim() == 4 && pages->size(1) == 1 && pages->size(3) >= R + Dr,
                "latent_rope_write: pages must be [pages, 1, page_tokens, >= rank + rotated dims]");
    TORCH_CHECK(kv_col0 >= 0 && Dr >= 0 && kv_col0 + R + Dr <= proj.size(1), "latent_rope_write: columns outside proj");
    TORCH_CHECK(dtype < 0 || dtype == out_code(*pages, "pages"), "latent_rope_write: cq and pages must share a dtype");
    dtype = out_code(*pages, "pages");
    pages_ptr = pages->data_ptr();
    Rp = pages->size(3);
    page_tokens = pages->size(2);
    TORCH_CHECK(rot >= 0 && rot <= Dr && rot % 2 == 0, "latent_rope_write: rot must be even and at most the key part's size");
    if (rot > 0) {
      TORCH_CHECK(cos.has_value() && sin.has_value(), "latent_rope_write: rotation needs its tables");
      check_f32(*cos, "cos");
      check_f32(*sin, "sin");
      TORCH_CHECK(cos->dim() == 2 && cos->size(1) == rot / 2 && sin->sizes() == cos->sizes(),
                  "latent_rope_write: cos and sin must be [positions, rot / 2]");
    }
  }
  TORCH_CHECK(dtype >= 0, "latent_rope_write: nothing to do");
  done(lse_latent_rope_write(proj.data_ptr(), out_code(proj, "proj"), proj.size(1), (int)q_col0, (int)Rq,
                             q_weight ? q_weight->data_ptr<float>() : nullptr, cq_ptr, (int)kv_col0, (int)R, (int)Dr,
                             (int)rot, kv_weight ? kv_weight->data_ptr<float>() : nullptr, (float)eps,
                             cos ? cos->data_ptr<float>() : nullptr, sin ? sin->data_ptr<float>() : nullptr, pages_ptr,
                             (int)Rp, dtype, positions.data_ptr<int>(), token_seq.data_ptr<int>(),
                             block_tables.data_ptr<int>(), (int)block_tables.size(1), (int)page_tokens, (int)T, stream()),
       "latent_rope_write");
}

// q [T, H * (D + Dr)] -> out [T, H * Rp]: dims R .. R + Dr of every head's slot (turned), zeros behind.
void latent_query_rope(const Tensor& q, int64_t H, int64_t D, int64_t Dr, int64_t rot, const OptTensor& cos,
                       const OptTensor& sin, const Tensor& positions, Tensor& out, int64_t R) {
  check_cuda(q, "q");
  check_cuda(out, "out");
  check_i32(positions, "positions");
  TORCH_CHECK(q.dim() == 2 && out.dim() == 2 && H > 0 && q.size(1) == H * (D + Dr) && out.size(0) == q.size(0) &&
                  out.size(1) % H == 0 && out.scalar_type() == q.scalar_type() && positions.numel() >= q.size(0),
              "latent_query_rope: q must be [T, H * (D + Dr)] and out [T, H * slot] of the same dtype");
  const int64_t Rp = out.size(1) / H;
  TORCH_CHECK(R >= 0 && R + Dr <= Rp && rot >= 0 && rot <= Dr && rot % 2 == 0, "latent_query_rope: sizes disagree");
  if (rot > 0) {
    TORCH_CHECK(cos.has_value() && sin.has_value(), "latent_query_rope: rotation needs its tables");
    check_f32(*cos, "cos");
    check_f32(*sin, "sin");
    TORCH_CHECK(cos->dim() == 2 && cos->size(1) == rot / 2 && sin->sizes() == cos->sizes(),
                "latent_query_rope: cos and sin must be [positions, rot / 2]");
  }
  done(lse_latent_query_rope(q.data_ptr(), out_code(q, "q"), (int)q.size(0), (int)H, (int)D, (int)Dr, (int)rot,
                             cos ? cos->data_ptr<float>() : nullptr, sin ? sin->data_ptr<float>() : nullptr,
                             positions.data_ptr<int>(), out.data_ptr(), (int)R, (int)Rp, stream()),
       "latent_query_rope");
}

// o[t, i] *= sigmoid(g[t, col0 + i / group])
void sigmoid_gate_mul(Tensor& o, const Tensor& g, int64_t col0, int64_t group) {
  check_cuda(o, "o");
  check_cuda(g, "g");
  TORCH_CHECK(o.dim() == 2 && g.dim() == 2 && g.size(0) == o.size(0) && group > 0 && col0 >= 0 &&
                  col0 + (o.size(1) + group - 1) / group <= g.size(1),
              "sigmoid_gate_mul: the gate's columns lie outside g");
  done(lse_sigmoid_gate_mul(o.data_ptr(), out_code(o, "o"), g.data_ptr(), out_code(g, "g"), g.size(1), (int)col0,
                            (int)group, (int)o.size(0), (int)o.size(1), stream()),
       "sigmoid_gate_mul");
}

// out = act(in) element by element; in may be fixed-point sums (int64), which are left zero
void act_rows(const Tensor& in, Tensor& out, int64_t act) {
  check_cuda(in, "in");
  check_cuda(out, "out");
  TORCH_CHECK(in.numel() == out.numel(), "act_rows: sizes differ");
  const int in_code = in.scalar_type() == torch::kInt64 ? LSE_FIXED64 : out_code(in, "in");
  done(lse_act_rows(in.data_ptr(), in_code, out.data_ptr(), out_code(out, "out"), in.numel(), (int)act, stream()),
       "act_rows");
}

// ------------------------------------------------------------------ residual streams, rows of q/k/v, differential attention
void streams_spread(const Tensor& x, Tensor& out, int64_t S, double scale) {
  check_f32(x, "x");
  check_f32(out, "out");
  TORCH_CHECK(x.dim() == 2 && out.dim() == 2 && S > 0 && out.size(0) == x.size(0) && out.size(1) == S * x.size(1),
              "streams_spread: out must be [T, streams * width]");
  done(lse_streams_spread(x.data_ptr<float>(), out.data_ptr<float>(), (int)x.size(0), (int)x.size(1), (int)S,
                          (float)scale, stream()),
       "streams_spread");
}

void streams_read_norm(const Tensor& x, const Tensor& read, const Tensor& w, double eps, Tensor& out, int64_t S,
                       const OptTensor& rows) {
  check_f32(x, "x");
  check_f32(read, "read");
  check_f32(w, "weight");
  check_cuda(out, "out");
  TORCH_CHECK(x.dim() == 2 && S > 0 && x.size(1) % S == 0 && read.numel() == S, "streams_read_norm: x must be [T, streams * width]");
  const int64_t W = x.size(1) / S;
  const int* rp = nullptr;
  int64_t n = x.size(0);
  if (rows) {
    check_i32(*rows, "rows");
    rp = rows->data_ptr<int>();
    n = rows->numel();
  }
  TORCH_CHECK(w.numel() == W && out.dim() == 2 && out.size(0) == n && out.size(1) == W, "streams_read_norm: out must be [rows, width]");
  done(lse_streams_read_norm(x.data_ptr<float>(), read.data_ptr<float>(), w.data_ptr<float>(), (float)eps,
                             out.data_ptr(), out_code(out, "out"), rp, (int)n, (int)W, (int)S, stream()),
       "streams_read_norm");
}

void streams_write(Tensor& x, const Tensor& y, const OptTensor& scale, const Tensor& mix, const Tensor& outw,
                   int64_t S, const OptTensor& then_read, const OptTensor& then_w, double then_eps,
                   const OptTensor& out) {
  check_f32(x, "x");
  check_cuda(y, "y");
  check_f32(mix, "mix");
  check_f32(outw, "out weights");
  TORCH_CHECK(x.dim() == 2 && S > 0 && x.size(1) % S == 0 && mix.numel() == S * S && outw.numel() == S,
              "streams_write: x must be [T, streams * width], mix [streams, streams]");
  const int64_t W = x.size(1) / S;
  TORCH_CHECK(y.dim() == 2 && y.size(0) == x.size(0) && y.size(1) == W, "streams_write: y must be [T, width]");
  TORCH_CHECK(then_read.has_value() == then_w.has_value() && then_read.has_value() == out.has_value(),
              "streams_write: the read that follows needs its weights, the norm's weight and an output");
  void* op = nullptr;
  int ocode = LSE_F32;
  if (out) {
    check_cuda(*out, "out");
    TORCH_CHECK(out->dim() == 2 && out->size(0) == x.size(0) && out->size(1) == W, "streams_write: out must be [T, width]");
    op = out->data_ptr();
    ocode = out_code(*out, "out");
  }
  done(lse_streams_write(x.data_ptr<float>(), y.data_ptr(), dtype_code(y, "y"), opt_f32(scale, W, "scale"),
                         mix.data_ptr<float>(), outw.data_ptr<float>(), (int)x.size(0), (int)W, (int)S,
                         opt_f32(then_read, S, "then_read"), opt_f32(then_w, W, "then_weight"), (float)then_eps, op,
                         ocode, stream()),
       "streams_write");
}

void qkv_norm_rope_write(const Tensor& proj, Tensor& q_out, int64_t nq, int64_t nk, int64_t nv, int64_t D, int64_t Dv,
                         int64_t Dp, const OptTensor& qw, const OptTensor& kw, double eps, double temp_coef,
                         int64_t temp_every, const Tensor& positions, const Tensor& token_seq, const OptTensor& cos,
                         const OptTensor& sin, const OptTensor& k_pages, const OptTensor& v_pages,
                         const Tensor& block_tables, int64_t page_tokens) {
  check_f32(proj, "proj");
  check_cuda(q_out, "q_out");
  check_i32(positions, "positions");
  check_i32(token_seq, "token_seq");
  check_i32(block_tables, "block_tables");
  const int64_t T = proj.size(0);
  TORCH_CHECK(proj.dim() == 2 && nq > 0 && nk > 0 && nv >= 0 && D > 0 && Dp >= D && Dp <= 256 &&
                  proj.size(1) >= (nq + nk) * D + nv * Dv,
              "qkv_norm_rope_write: the projection is too narrow for these heads");
  TORCH_CHECK(q_out.dim() == 2 && q_out.size(0) == T && q_out.size(1) == nq * Dp, "qkv_norm_rope_write: q_out shape");
  TORCH_CHECK(positions.numel() >= T && token_seq.numel() >= T && block_tables.dim() == 2,
              "qkv_norm_rope_write: the batch arrays disagree");
  TORCH_CHECK(qw.has_value() == kw.has_value() && cos.has_value() == sin.has_value() &&
                  k_pages.has_value() == v_pages.has_value(),
              "qkv_norm_rope_write: weights, tables and pages come in pairs");
  int rot = 0;
  if (cos) {
    check_f32(*cos, "cos");
    check_f32(*sin, "sin");
    TORCH_CHECK(cos->dim() == 2 && sin->sizes() == cos->sizes() && 2 * cos->size(1) <= D,
                "qkv_norm_rope_write: cos and sin must be [positions, rotated dims / 2]");
    rot = 2 * (int)cos->size(1);
  }
  void *kp = nullptr, *vp = nullptr;
  if (k_pages) {
    check_cuda(*k_pages, "k_pages");
    check_cuda(*v_pages, "v_pages");
    TORCH_CHECK(k_pages->scalar_type() == q_out.scalar_type() && v_pages->scalar_type() == q_out.scalar_type() &&
                    k_pages->dim() == 4 && k_pages->size(1) == nk && k_pages->size(2) == page_tokens &&
                    k_pages->size(3) == Dp && v_pages->sizes() == k_pages->sizes(),
                "qkv_norm_rope_write: pages must be [pages, key heads, page_tokens, out_dim] of q_out's dtype");
    kp = k_pages->data_ptr();
    vp = v_pages->data_ptr();
  }
  done(lse_qkv_norm_rope_write(proj.data_ptr<float>(), proj.size(1), (int)T, (int)nq, (int)nk, (int)nv, (int)D, (int)Dv,
                               (int)Dp, opt_f32(qw, nq * D, "q weight"), opt_f32(kw, nk * D, "k weight"), (float)eps,
                               (float)temp_coef, (int)temp_every, positions.data_ptr<int>(), token_seq.data_ptr<int>(),
                               cos ? cos->data_ptr<float>() : nullptr, sin ? sin->data_ptr<float>() : nullptr, rot,
                               q_out.data_ptr(), kp, vp, out_code(q_out, "q_out"), block_tables.data_ptr<int>(),
                               (int)block_tables.size(1), (int)page_tokens, stream()),
       "qkv_norm_rope_write");
}

void differential_combine(const Tensor& a, const Tensor& gate, int64_t gate_col0, int64_t H, int64_t n, int64_t Dp,
                          int64_t Dv, double lam, double eps, double out_scale, Tensor& out) {
  check_cuda(a, "a");
  check_f32(gate, "gate");
  check_cuda(out, "out");
  TORCH_CHECK(a.dim() == 2 && a.size(1) == 2 * H * Dp && gate.dim() == 2 && gate.size(0) == a.size(0) &&
                  gate_col0 >= 0 && gate_col0 + H <= gate.size(1) && out.dim() == 2 && out.size(0) == a.size(0) &&
                  out.size(1) == H * Dv &&
                  (out.scalar_type() == a.scalar_type() || a.scalar_type() == torch::kFloat32),
              "differential_combine: need a [T, 2*heads*head_dim], gate columns inside gate, out [T, heads*value_dim] of a's dtype (or a in float32)");
  done(lse_differential_combine(a.data_ptr(), out_code(a, "a"), gate.data_ptr<float>() + gate_col0, gate.size(1),
                                (int)a.size(0), (int)H, (int)n, (int)Dp, (int)Dv, (float)lam, (float)eps,
                                (float)out_scale, out.data_ptr(), out_code(out, "out"), stream()),
       "differential_combine");
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("embedding", &embedding);
  m.def("add_rmsnorm", &add_rmsnorm);
  m.def("rope_kv_write", &rope_kv_write);
  m.def("silu_mul", &silu_mul, py::arg("gu"), py::arg("out"), py::arg("act") = 0);
  m.def("gemm_f32", &gemm_f32);
  m.def("gemm_bf16_skinny", &gemm_bf16_skinny);
  m.def("gemm_bf16_skinny_max_rows", &gemm_bf16_skinny_max_rows);
  m.def("fixed_to_float", &fixed_to_float);
  m.def("kernel_error", &kernel_error);
  m.def("clear_kernel_error", &clear_kernel_error);
  m.def("load_attention_library", &load_attention_library);
  m.def("attention_q_tile", &attention_q_tile);
  m.def("attention_scratch_floats", &attention_scratch_floats);
  m.def("attention_decode_blocks_per_sm", &attention_decode_blocks_per_sm);
  m.def("paged_attention", &paged_attention, py::arg("q"), py::arg("out"), py::arg("k_pages"), py::arg("v_pages"),
        py::arg("num_heads"), py::arg("num_kv_heads"), py::arg("head_dim"), py::arg("scale"), py::arg("window"),
        py::arg("block_tables"), py::arg("ctx_lens"), py::arg("cu_q"), py::arg("tiles"), py::arg("num_tiles"),
        py::arg("decode_seqs"), py::arg("num_decode"), py::arg("num_splits"), py::arg("scratch"),
        py::arg("force_kernel"), py::arg("head_scale"), py::arg("slopes"), py::arg("chunk"),
        py::arg("sinks") = py::none(), py::arg("keep_first") = 0);
  m.def("hashed_pair_add", &hashed_pair_add);
  m.def("sinusoid_add", &sinusoid_add);
  m.def("latent_write", &latent_write);
  m.def("head_linear", &head_linear, py::arg("a"), py::arg("col0"), py::arg("w"), py::arg("out"), py::arg("kind"),
        py::arg("a_head_cols") = 0, py::arg("out_head_cols") = 0);
  m.def("moe_route", &moe_route, py::arg("h"), py::arg("router"), py::arg("num_experts"), py::arg("top"),
        py::arg("idx"), py::arg("wts"), py::arg("gate"), py::arg("bias") = py::none(), py::arg("mode") = 0);
  m.def("moe_max_tiles", &moe_max_tiles);
  m.def("moe_tile_rows", &moe_tile_rows);
  m.def("moe_sort", &moe_sort);
  m.def("expert_linear", &expert_linear);
  m.def("moe_combine", &moe_combine, py::arg("y"), py::arg("work"), py::arg("num_experts"), py::arg("top"),
        py::arg("shared_out"), py::arg("gate"), py::arg("out"), py::arg("accumulate"), py::arg("wts") = py::none());
  m.def("latent_rope_write", &latent_rope_write);
  m.def("latent_query_rope", &latent_query_rope);
  m.def("sigmoid_gate_mul", &sigmoid_gate_mul);
  m.def("act_rows", &act_rows);
  m.def("cast_f32", &cast_f32);
  m.def("token_shift", &token_shift);
  m.def("rmsnorm_add", &rmsnorm_add);
  m.def("mix_normed", &mix_normed);
  m.def("gated_group_norm", &gated_group_norm);
  m.def("norm_rope_kv_write", &norm_rope_kv_write);
  m.def("decay_linear_attention", &decay_linear_attention, py::arg("proj"), py::arg("out"), py::arg("state"),
        py::arg("decay"), py::arg("cu_q"), py::arg("ctx_lens"), py::arg("slots"), py::arg("H"), py::arg("dk"),
        py::arg("dv"), py::arg("cos"), py::arg("sin"), py::arg("silu"), py::arg("key_scale"), py::arg("max_chunks"),
        py::arg("chunks"), py::arg("gate_z") = py::none(), py::arg("decay_root") = 1.0, py::arg("query_scale") = 1.0);
  m.def("streams_spread", &streams_spread);
  m.def("streams_read_norm", &streams_read_norm);
  m.def("streams_write", &streams_write);
  m.def("qkv_norm_rope_write", &qkv_norm_rope_write);
  m.def("differential_combine", &differential_combine);
  m.def("linear_attention_chunk", []() { return (int64_t)lse_linear_attention_chunk(); });
  m.def("paged_attention_from_sums", &paged_attention_from_sums);
  m.def("attention_takes_sums", &attention_takes_sums);
  m.def("sample", &sample, py::arg("logits"), py::arg("temperature"), py::arg("top_k"), py::arg("top_p"),
        py::arg("min_p"), py::arg("seed"), py::arg("draw"), py::arg("out"), py::arg("scratch") = py::none(),
        py::arg("which") = 3);
  m.def("sample_scratch_ints", [](int64_t rows) { return (int64_t)lse_sample_scratch_ints((int)rows); });
  m.def("logsumexp", &logsumexp);
  m.def("apply_penalties", &apply_penalties);
  m.def("ban_tokens", &ban_tokens);
  m.def("token_state_add", &token_state_add);
  m.def("apply_penalties_dense", &apply_penalties_dense);
}
