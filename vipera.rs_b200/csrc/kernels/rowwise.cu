// Row-wise kernels: embedding lookup into the 32-bit residual stream, and RMSNorm.
//
// Embedding: a row lookup (crates/vipera-backend-cpu/src/model.rs:956-966; the reference's
// device version dequantises one row, crates/vipera-backend-gpu/src/layer.cu:545-563).  The
// reference's model does not scale the rows; `scale` is for architectures that do, and a
// scale of exactly 1 leaves the values as they are.
// RMSNorm: out = x * rsqrt(mean(x^2) + eps) * w with 32-bit statistics
// (model.rs:4282-4288; device version layer.cu:32-58, one block per row with a tree sum).
#include "common.cuh"

// ---------------------------------------------------------------------------------------
// embedding: out[t, :] = scale * table[tokens[t], :]  (32-bit out, whatever the table's type)
// ---------------------------------------------------------------------------------------
template <typename TW>
__global__ void embed_kernel(const TW* __restrict__ table, const int* __restrict__ tokens,
                             float* __restrict__ out, int hidden, int vocab, float scale) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  int token = tokens[t];
  // The host refuses ids outside the vocabulary before the launch; the clamp only keeps
  // a stale buffer in a replayed graph from reading outside the table.
  token = min(max(token, 0), vocab - 1);
  const TW* row = table + static_cast<size_t>(token) * hidden;
  float* dst = out + static_cast<size_t>(t) * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = scale * to_float<TW>(row[i]);
}

VIPERA_API int vipera_embed(const void* table, int table_dtype, const int* tokens, float* out,
                            int num_tokens, int hidden, int vocab, float scale, void* stream) {
  if (num_tokens <= 0) return VIPERA_OK;
  if (hidden <= 0 || vocab <= 0) return VIPERA_BAD_SHAPE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int threads = hidden >= 1024 ? 256 : 128;
  if (table_dtype == VIPERA_F32)
    return vipera_launch(embed_kernel<float>, num_tokens, threads, 0, s, static_cast<const float*>(table), tokens, out, hidden, vocab, scale);
  if (table_dtype == VIPERA_BF16)
    return vipera_launch(embed_kernel<__nv_bfloat16>, num_tokens, threads, 0, s, static_cast<const __nv_bfloat16*>(table), tokens, out, hidden, vocab, scale);
  return VIPERA_BAD_DTYPE;
}

// ---------------------------------------------------------------------------------------
// RMSNorm over rows of the 32-bit residual stream.  `rows` (optional) picks which rows of
// x are normalised: out[r, :] = norm(x[rows[r], :]).  For few rows, one block per output row;
// the row stays in registers between the two passes when it is short enough, else it is read
// twice.
// ---------------------------------------------------------------------------------------
constexpr int kNormThreads = 256;
constexpr int kNormRegs = 8;  // elements per thread kept in registers: rows up to 2048 wide

template <typename TO>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ weight,
                               const int* __restrict__ rows, TO* __restrict__ out, int hidden, float eps) {
  __shared__ float scratch[32];
  pdl_launch_dependents();
  const int r = blockIdx.x;
  const bool fits = hidden <= kNormThreads * kNormRegs;
  // The norm's weights depend on no kernel ahead of this one: they are in registers before the
  // wait, so that the second pass does not pay a memory round trip for them.
  float gain[kNormRegs];
  if (fits) {
#pragma unroll
    for (int j = 0; j < kNormRegs; ++j) {
      const int i = threadIdx.x + j * kNormThreads;
      gain[j] = i < hidden ? weight[i] : 0.0f;
    }
  }
  pdl_wait();
  const int src_row = rows ? rows[r] : r;
  const float* src = x + static_cast<size_t>(src_row) * hidden;
  TO* dst = out + static_cast<size_t>(r) * hidden;
  float kept[kNormRegs];
  float sum = 0.0f;
  if (fits) {
#pragma unroll
    for (int j = 0; j < kNormRegs; ++j) {
      const int i = threadIdx.x + j * kNormThreads;
      kept[j] = i < hidden ? src[i] : 0.0f;
      sum += kept[j] * kept[j];
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += kNormThreads) {
      const float v = src[i];
      sum += v * v;
    }
  }
  const float total = block_sum(sum, scratch);
  const float inverse = 1.0f / sqrtf(total / static_cast<float>(hidden) + eps);
  if (fits) {
#pragma unroll
    for (int j = 0; j < kNormRegs; ++j) {
      const int i = threadIdx.x + j * kNormThreads;
      if (i < hidden) dst[i] = from_float<TO>(kept[j] * inverse * gain[j]);
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += kNormThreads)
      dst[i] = from_float<TO>(src[i] * inverse * weight[i]);
  }
}

// The same for many rows (prompt portions): a warp per row, the row in registers as 16-byte
// vectors, the sum by shuffles; no block-wide barrier, eight rows to a block.  VECS vectors
// of four values per lane: rows up to 128 * VECS wide, a multiple of four.
constexpr int kRowsPerBlock = 8;
constexpr int kManyRows = 128;  // from this many rows on

__device__ __forceinline__ void store_four(float* dst, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(dst) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void store_four(__nv_bfloat16* dst, float a, float b, float c, float d) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  uint2 packed;
  packed.x = *reinterpret_cast<uint32_t*>(&lo);
  packed.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(dst) = packed;
}

template <typename TO, int VECS>
__global__ void __launch_bounds__(kRowsPerBlock * 32)
rmsnorm_rows_kernel(const float* __restrict__ x, const float* __restrict__ weight, const int* __restrict__ rows,
                    TO* __restrict__ out, int num_rows, int hidden, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x * kRowsPerBlock + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (r >= num_rows) return;
  const int src_row = rows ? rows[r] : r;
  const float4* src = reinterpret_cast<const float4*>(x + static_cast<size_t>(src_row) * hidden);
  const float4* w = reinterpret_cast<const float4*>(weight);
  TO* dst = out + static_cast<size_t>(r) * hidden;
  const int vectors = hidden >> 2;
  float4 kept[VECS];
  float sum = 0.0f;
#pragma unroll
  for (int j = 0; j < VECS; ++j) {
    const int i = lane + j * 32;
    kept[j] = i < vectors ? src[i] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    sum += kept[j].x * kept[j].x + kept[j].y * kept[j].y + kept[j].z * kept[j].z + kept[j].w * kept[j].w;
  }
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, offset);
  const float inverse = 1.0f / sqrtf(sum / static_cast<float>(hidden) + eps);
#pragma unroll
  for (int j = 0; j < VECS; ++j) {
    const int i = lane + j * 32;
    if (i < vectors) {
      const float4 g = w[i];
      store_four(dst + 4 * i, kept[j].x * inverse * g.x, kept[j].y * inverse * g.y, kept[j].z * inverse * g.z,
                 kept[j].w * inverse * g.w);
    }
  }
}

template <typename TO>
static int launch_rmsnorm_rows(const float* x, const float* weight, const int* rows, TO* out, int num_rows, int hidden,
                               float eps, cudaStream_t s) {
  const int blocks = (num_rows + kRowsPerBlock - 1) / kRowsPerBlock;
  if (hidden <= 128 * 8)
    return vipera_launch(rmsnorm_rows_kernel<TO, 8>, blocks, kRowsPerBlock * 32, 0, s, x, weight, rows, out, num_rows, hidden, eps);
  if (hidden <= 128 * 16)
    return vipera_launch(rmsnorm_rows_kernel<TO, 16>, blocks, kRowsPerBlock * 32, 0, s, x, weight, rows, out, num_rows, hidden, eps);
  return vipera_launch(rmsnorm_rows_kernel<TO, 32>, blocks, kRowsPerBlock * 32, 0, s, x, weight, rows, out, num_rows, hidden, eps);
}

VIPERA_API int vipera_rmsnorm(const float* x, const float* weight, const int* rows, void* out,
                              int out_dtype, int num_rows, int hidden, float eps, void* stream) {
  if (num_rows <= 0) return VIPERA_OK;
  if (hidden <= 0) return VIPERA_BAD_SHAPE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  if (num_rows >= kManyRows && hidden % 4 == 0 && hidden <= 128 * 32 && aligned) {
    if (out_dtype == VIPERA_F32) return launch_rmsnorm_rows(x, weight, rows, static_cast<float*>(out), num_rows, hidden, eps, s);
    if (out_dtype == VIPERA_BF16) return launch_rmsnorm_rows(x, weight, rows, static_cast<__nv_bfloat16*>(out), num_rows, hidden, eps, s);
    return VIPERA_BAD_DTYPE;
  }
  if (out_dtype == VIPERA_F32)
    return vipera_launch(rmsnorm_kernel<float>, num_rows, kNormThreads, 0, s, x, weight, rows, static_cast<float*>(out), hidden, eps);
  if (out_dtype == VIPERA_BF16)
    return vipera_launch(rmsnorm_kernel<__nv_bfloat16>, num_rows, kNormThreads, 0, s, x, weight, rows, static_cast<__nv_bfloat16*>(out), hidden, eps);
  return VIPERA_BAD_DTYPE;
}

VIPERA_API const char* vipera_rowwise_status_text(int status) { return vipera_status_text(status); }
