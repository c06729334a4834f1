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

// One block per token; its threads walk the pairs of all heads, two pairs (four values) at
// a time where the head size allows, so that loads and stores are 8 and 16 bytes wide.
// Input: the 32-bit result of the q/k/v product with bias, [tokens, (heads + 2*kv_heads) * d].
// Output: rotated q in the activation type, [tokens, heads * d]; rotated k and plain v in
// the cache's type, written to their page (when write_cache is set).
template <typename T>
__device__ __forceinline__ void store_pair(T* dst, float a, float b);
template <>
__device__ __forceinline__ void store_pair<float>(float* dst, float a, float b) {
  *reinterpret_cast<float2*>(dst) = make_float2(a, b);
}
template <>
__device__ __forceinline__ void store_pair<__nv_bfloat16>(__nv_bfloat16* dst, float a, float b) {
  *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(a, b);
}

template <typename T>
__global__ void __launch_bounds__(256)
rope_cache_kernel(const float* __restrict__ qkv, T* __restrict__ q_out, int num_heads, int num_kv_heads,
                  int head_dim, const int* __restrict__ positions, const float* __restrict__ cos_table,
                  const float* __restrict__ sin_table, int style, T* __restrict__ k_pool, T* __restrict__ v_pool,
                  const int* __restrict__ token_seq, const int* __restrict__ block_table, int table_width,
                  int page_size, int write_cache) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int half = head_dim >> 1;
  const int all_heads = num_heads + 2 * num_kv_heads;
  const float* row = qkv + static_cast<size_t>(t) * all_heads * head_dim;
  const int position = positions[t];
  T* k_row = nullptr;
  T* v_row = nullptr;
  if (write_cache) {
    const int page = block_table[static_cast<size_t>(token_seq[t]) * table_width + position / page_size];
    if (page >= 0) {
      const size_t at = (static_cast<size_t>(page) * page_size + position % page_size) * num_kv_heads * head_dim;
      k_row = k_pool + at;
      v_row = v_pool + at;
    }
  }
  const float* cos_row = cos_table ? cos_table + static_cast<size_t>(position) * half : nullptr;
  const float* sin_row = sin_table ? sin_table + static_cast<size_t>(position) * half : nullptr;
  // work item: (head, pair of neighbouring pair indices i, i + 1); head sizes are even, and a
  // head size that is a multiple of 4 keeps every access 8 bytes aligned
  const int pairs = half >> 1;  // items per head when two pairs go together
  const bool two = (half & 1) == 0;
  const int per_head = two ? pairs : half;
  for (int item = threadIdx.x; item < all_heads * per_head; item += blockDim.x) {
    const int h = item / per_head;
    const int i = (item % per_head) * (two ? 2 : 1);
    const bool is_q = h < num_heads;
    const bool is_v = h >= num_heads + num_kv_heads;
    const float* head = row + static_cast<size_t>(h) * head_dim;
    T* dst;
    if (is_q) dst = q_out + (static_cast<size_t>(t) * num_heads + h) * head_dim;
    else if (is_v) dst = v_row ? v_row + static_cast<size_t>(h - num_heads - num_kv_heads) * head_dim : nullptr;
    else dst = k_row ? k_row + static_cast<size_t>(h - num_heads) * head_dim : nullptr;
    if (!dst) continue;
    const int count = two ? 2 : 1;
    float lo[2], hi[2];
    int at_lo[2], at_hi[2];
    for (int e = 0; e < count; ++e) {
      at_lo[e] = style == ROPE_INTERLEAVED ? 2 * (i + e) : i + e;
      at_hi[e] = style == ROPE_INTERLEAVED ? 2 * (i + e) + 1 : i + e + half;
      const float a = head[at_lo[e]], b = head[at_hi[e]];
      if (is_v || style == ROPE_NONE) {
        lo[e] = a;
        hi[e] = b;
      } else {
        const float c = cos_row[i + e], s = sin_row[i + e];
        lo[e] = a * c - b * s;
        hi[e] = a * s + b * c;
      }
    }
    if (two && style != ROPE_INTERLEAVED) {
      store_pair<T>(dst + at_lo[0], lo[0], lo[1]);  // i and i + 1 are neighbours in both halves
      store_pair<T>(dst + at_hi[0], hi[0], hi[1]);
    } else {
      for (int e = 0; e < count; ++e) {
        dst[at_lo[e]] = from_float<T>(lo[e]);
        dst[at_hi[e]] = from_float<T>(hi[e]);
      }
    }
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
  dim3 grid(num_tokens);
  const int work = (num_heads + 2 * num_kv_heads) * (head_dim / 4);
  const int threads = work >= 256 ? 256 : (work >= 128 ? 128 : 64);
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
