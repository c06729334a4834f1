// Rotary position encoding of q and k, and the write of k and v into the paged cache.
//
// Rotation (NeoX pairing): for each head and i < d/2, with (s, c) the sine and cosine of
// position * base^(-2i/d): out[i] = a*c - b*s, out[i + d/2] = a*s + b*c where a = in[i],
// b = in[i + d/2] (crates/vipera-backend-cpu/src/model.rs:4226-4251; the reference's device
// kernel computes powf and sincosf per element, crates/vipera-backend-gpu/src/layer.cu:61-84;
// here the angles come from a 32-bit table built once on the host).
// Cache write: position p of a request goes to page block_table[p / page], slot p % page
// (model.rs:1507-1542); the reference's device port does this with two device copies per
// layer and token (crates/vipera-backend-gpu/src/device.rs:299-320).
#include "common.cuh"

enum RopeStyle { ROPE_NONE = 0, ROPE_NEOX = 1, ROPE_INTERLEAVED = 2 };

// grid: (tokens, heads + 2*kv_heads); one block handles one head of one token.
// Input: the 32-bit result of the q/k/v product with bias, [tokens, (heads + 2*kv_heads) * d].
// Output: rotated q in the activation type, [tokens, heads * d]; rotated k and plain v in
// the cache's type, written to their page (when write_cache is set).
template <typename T>
__global__ void rope_cache_kernel(const float* __restrict__ qkv, T* __restrict__ q_out, int num_heads,
                                  int num_kv_heads, int head_dim, const int* __restrict__ positions,
                                  const float* __restrict__ cos_table, const float* __restrict__ sin_table,
                                  int style, T* __restrict__ k_pool, T* __restrict__ v_pool,
                                  const int* __restrict__ token_seq, const int* __restrict__ block_table,
                                  int table_width, int page_size, int write_cache) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int h = blockIdx.y;
  const int half = head_dim >> 1;
  const int row_width = (num_heads + 2 * num_kv_heads) * head_dim;
  const float* head = qkv + static_cast<size_t>(t) * row_width + static_cast<size_t>(h) * head_dim;
  const int position = positions[t];
  const bool is_q = h < num_heads;
  const bool is_k = !is_q && h < num_heads + num_kv_heads;
  const bool is_v = !is_q && !is_k;

  T* dst = nullptr;
  if (is_q) {
    dst = q_out + (static_cast<size_t>(t) * num_heads + h) * head_dim;
  } else if (write_cache) {
    const int seq = token_seq[t];
    const int page = block_table[static_cast<size_t>(seq) * table_width + position / page_size];
    if (page >= 0) {
      const int kv_head = is_k ? h - num_heads : h - num_heads - num_kv_heads;
      T* pool = is_k ? k_pool : v_pool;
      dst = pool + ((static_cast<size_t>(page) * page_size + position % page_size) * num_kv_heads + kv_head) * head_dim;
    }
  }
  if (!dst) return;

  if (is_v || style == ROPE_NONE) {
    for (int i = threadIdx.x; i < head_dim; i += blockDim.x) dst[i] = from_float<T>(head[i]);
    return;
  }
  const float* cos_row = cos_table + static_cast<size_t>(position) * half;
  const float* sin_row = sin_table + static_cast<size_t>(position) * half;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const int lo = style == ROPE_NEOX ? i : 2 * i;
    const int hi = style == ROPE_NEOX ? i + half : 2 * i + 1;
    const float a = head[lo];
    const float b = head[hi];
    const float c = cos_row[i], s = sin_row[i];
    dst[lo] = from_float<T>(a * c - b * s);
    dst[hi] = from_float<T>(a * s + b * c);
  }
}

VIPERA_API int vipera_rope_cache(const float* qkv, void* q_out, int dtype, int num_tokens, int num_heads,
                                 int num_kv_heads, int head_dim, const int* positions,
                                 const float* cos_table, const float* sin_table, int style, void* k_pool,
                                 void* v_pool, const int* token_seq, const int* block_table,
                                 int table_width, int page_size, int write_cache, void* stream) {
  if (num_tokens <= 0) return VIPERA_OK;
  if (head_dim <= 0 || (head_dim & 1) || num_heads <= 0 || num_kv_heads <= 0) return VIPERA_BAD_SHAPE;
  if (style != ROPE_NONE && (!cos_table || !sin_table)) return VIPERA_BAD_ARGUMENT;
  if (write_cache && (!k_pool || !v_pool || !token_seq || !block_table || page_size <= 0)) return VIPERA_BAD_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  dim3 grid(num_tokens, num_heads + 2 * num_kv_heads);
  const int threads = head_dim >= 128 ? 64 : 32;
  if (dtype == VIPERA_F32)
    return vipera_launch(rope_cache_kernel<float>, grid, threads, 0, s, qkv, static_cast<float*>(q_out), num_heads, num_kv_heads, head_dim,
        positions, cos_table, sin_table, style, static_cast<float*>(k_pool), static_cast<float*>(v_pool),
        token_seq, block_table, table_width, page_size, write_cache);
  if (dtype == VIPERA_BF16)
    return vipera_launch(rope_cache_kernel<__nv_bfloat16>, grid, threads, 0, s, qkv, static_cast<__nv_bfloat16*>(q_out), num_heads, num_kv_heads, head_dim,
        positions, cos_table, sin_table, style, static_cast<__nv_bfloat16*>(k_pool), static_cast<__nv_bfloat16*>(v_pool),
        token_seq, block_table, table_width, page_size, write_cache);
  return VIPERA_BAD_DTYPE;
}

VIPERA_API const char* vipera_rope_cache_status_text(int status) { return vipera_status_text(status); }
