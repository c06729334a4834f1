// Causal grouped-query attention over the paged cache, for any mix of prompt portions and
// single decode tokens, with 32-bit scores, softmax and accumulation.
//
// Definition (crates/vipera-backend-cpu/src/model.rs:1804-1859): query head h reads KV head
// h / group; s_j = (q . k_j) * scale; a query at position p sees keys 0..p (with a window w,
// keys p-w+1..p); weights exp(s_j - max) over their sum; output = weighted sum of v_j.
// Traversal: one warp per (token, query head) folds the keys 32 at a time with a running
// (max, sum, output), the online form of the reference's chunk fold (model.rs:2752-2857) and
// of its device kernels' partials (crates/vipera-backend-gpu/src/layer.cu:307-467).
// Keys are found through the block table: position j lives in page table[j / page], slot
// j % page (model.rs:1507-1542).
//
// This kernel is the attention of the 32-bit path and takes every head size that is a
// multiple of 16 up to 256, any number of heads and groups, any page size.
#include "common.cuh"

constexpr int kWarpsPerBlock = 4;
constexpr int kMaxHeadDim = 256;

template <typename T>
__device__ __forceinline__ float dot_row(const float* __restrict__ q, const T* __restrict__ row, int d);

template <>
__device__ __forceinline__ float dot_row<float>(const float* __restrict__ q, const float* __restrict__ row, int d) {
  float sum = 0.0f;
  const float4* r4 = reinterpret_cast<const float4*>(row);
  for (int i = 0; i < d / 4; ++i) {
    const float4 v = r4[i];
    sum = fmaf(q[4 * i + 0], v.x, sum);
    sum = fmaf(q[4 * i + 1], v.y, sum);
    sum = fmaf(q[4 * i + 2], v.z, sum);
    sum = fmaf(q[4 * i + 3], v.w, sum);
  }
  return sum;
}

template <>
__device__ __forceinline__ float dot_row<__nv_bfloat16>(const float* __restrict__ q, const __nv_bfloat16* __restrict__ row, int d) {
  float sum = 0.0f;
  const uint4* r8 = reinterpret_cast<const uint4*>(row);
  for (int i = 0; i < d / 8; ++i) {
    const uint4 raw = r8[i];
    const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = __bfloat1622float2(pairs[e]);
      sum = fmaf(q[8 * i + 2 * e], f.x, sum);
      sum = fmaf(q[8 * i + 2 * e + 1], f.y, sum);
    }
  }
  return sum;
}

template <typename T>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
attention_kernel(const T* __restrict__ q, T* __restrict__ out, const T* __restrict__ k_pool,
                 const T* __restrict__ v_pool, const int* __restrict__ token_seq,
                 const int* __restrict__ positions, const int* __restrict__ block_table, int table_width,
                 int page_size, int num_heads, int num_kv_heads, int head_dim, float scale, int window) {
  __shared__ float q_shared[kWarpsPerBlock][kMaxHeadDim];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int h = blockIdx.y * kWarpsPerBlock + warp;
  if (h >= num_heads) return;
  const int group = num_heads / num_kv_heads;
  const int kv_head = h / group;
  const int position = positions[t];
  const int* table = block_table + static_cast<size_t>(token_seq[t]) * table_width;
  const int first = window > 0 ? max(0, position - window + 1) : 0;

  const T* q_row = q + (static_cast<size_t>(t) * num_heads + h) * head_dim;
  float* qs = q_shared[warp];
  for (int i = lane; i < head_dim; i += 32) qs[i] = to_float<T>(q_row[i]);
  __syncwarp();

  float acc[kMaxHeadDim / 32];
#pragma unroll
  for (int i = 0; i < kMaxHeadDim / 32; ++i) acc[i] = 0.0f;
  float running_max = -INFINITY, running_sum = 0.0f;
  const size_t row_stride = static_cast<size_t>(num_kv_heads) * head_dim;

  for (int base = first; base <= position; base += 32) {
    const int j = base + lane;
    const bool valid = j <= position;
    float score = -INFINITY;
    if (valid) {
      const int page = table[j / page_size];
      const T* k_row = k_pool + (static_cast<size_t>(page) * page_size + j % page_size) * row_stride +
                       static_cast<size_t>(kv_head) * head_dim;
      score = dot_row<T>(qs, k_row, head_dim) * scale;
    }
    const float new_max = fmaxf(running_max, warp_max(score));
    const float alpha = expf(running_max - new_max);  // 0 on the first tile
    const float weight = valid ? expf(score - new_max) : 0.0f;
    running_sum = running_sum * alpha + warp_sum(weight);
    running_max = new_max;
#pragma unroll
    for (int i = 0; i < kMaxHeadDim / 32; ++i) acc[i] *= alpha;
    const int count = min(32, position - base + 1);
    for (int jj = 0; jj < count; ++jj) {
      const float w = __shfl_sync(0xffffffffu, weight, jj);
      const int key = base + jj;
      const int page = table[key / page_size];
      const T* v_row = v_pool + (static_cast<size_t>(page) * page_size + key % page_size) * row_stride +
                       static_cast<size_t>(kv_head) * head_dim;
#pragma unroll
      for (int i = 0; i < kMaxHeadDim / 32; ++i) {
        const int e = lane + 32 * i;
        if (e < head_dim) acc[i] = fmaf(w, to_float<T>(v_row[e]), acc[i]);
      }
    }
  }
  const float inverse = 1.0f / running_sum;
  T* out_row = out + (static_cast<size_t>(t) * num_heads + h) * head_dim;
#pragma unroll
  for (int i = 0; i < kMaxHeadDim / 32; ++i) {
    const int e = lane + 32 * i;
    if (e < head_dim) out_row[e] = from_float<T>(acc[i] * inverse);
  }
}

// q and out are [tokens, heads, d]; the pools are [pages, page_size, kv_heads, d].
// token_seq[t] is the row of block_table (width table_width) of token t's request and
// positions[t] its position.  The keys and values of this step's tokens must already be
// in the cache.  window = 0 means every earlier key is visible.
VIPERA_API int vipera_attention(const void* q, void* out, int dtype, const void* k_pool, const void* v_pool,
                                const int* token_seq, const int* positions, const int* block_table,
                                int table_width, int page_size, int num_tokens, int num_heads,
                                int num_kv_heads, int head_dim, float scale, int window, void* stream) {
  if (num_tokens <= 0) return VIPERA_OK;
  if (head_dim <= 0 || head_dim % 16 != 0 || head_dim > kMaxHeadDim) return VIPERA_BAD_SHAPE;
  if (num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads != 0) return VIPERA_BAD_SHAPE;
  if (page_size <= 0 || table_width <= 0 || window < 0) return VIPERA_BAD_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  dim3 grid(num_tokens, (num_heads + kWarpsPerBlock - 1) / kWarpsPerBlock);
  if (dtype == VIPERA_F32)
    attention_kernel<float><<<grid, kWarpsPerBlock * 32, 0, s>>>(
        static_cast<const float*>(q), static_cast<float*>(out), static_cast<const float*>(k_pool),
        static_cast<const float*>(v_pool), token_seq, positions, block_table, table_width, page_size,
        num_heads, num_kv_heads, head_dim, scale, window);
  else if (dtype == VIPERA_BF16)
    attention_kernel<__nv_bfloat16><<<grid, kWarpsPerBlock * 32, 0, s>>>(
        static_cast<const __nv_bfloat16*>(q), static_cast<__nv_bfloat16*>(out),
        static_cast<const __nv_bfloat16*>(k_pool), static_cast<const __nv_bfloat16*>(v_pool), token_seq,
        positions, block_table, table_width, page_size, num_heads, num_kv_heads, head_dim, scale, window);
  else
    return VIPERA_BAD_DTYPE;
  return vipera_launch_status();
}

VIPERA_API const char* vipera_attention_status_text(int status) { return vipera_status_text(status); }
