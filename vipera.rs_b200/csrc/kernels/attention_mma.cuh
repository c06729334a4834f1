// Pieces shared by the bfloat16 attention kernels on the tensor cores (mma.sync m16n8k16):
// swizzled shared-memory tiles, the copies of cache rows into them through the block table,
// and the fold of one block of keys into a warp's running (max, sum, output).
#pragma once

#include "common.cuh"

namespace {

constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// A tile of rows x D bf16 in shared memory; 16-byte chunks are XOR-swizzled by the row so
// that ldmatrix reads eight rows without bank conflicts.
template <int D>
__device__ __forceinline__ uint32_t tile_offset(int row, int chunk) {
  return static_cast<uint32_t>(row * D * 2 + ((chunk ^ (row & 7)) << 4));
}

// Copy `rows` cache rows (keys tile_key0 ..) of one KV head into a tile, through the block
// table.  Only keys in [visible_key, end_key) are read; every other row of the tile is
// filled with zeros: keys before `visible_key` may lie in pages the request has given back
// (a window has passed them), keys from `end_key` on are not written yet, and a masked
// value still enters the value product with weight zero, where 0 * NaN would be NaN.
template <int D, int ROWS, int THREADS>
__device__ __forceinline__ void load_kv_tile(uint32_t tile, const __nv_bfloat16* __restrict__ pool,
                                             const int* __restrict__ table, int page_size, int num_kv_heads,
                                             int kv_head, int tile_key0, int visible_key, int end_key, int thread) {
  constexpr int kChunks = D / 8;
  constexpr int kPasses = ROWS * kChunks / THREADS;
  static_assert(ROWS * kChunks % THREADS == 0, "the tile must divide among the threads");
  // first every source address (the block table reads are independent and overlap), then the copies
  const __nv_bfloat16* src[kPasses];
#pragma unroll
  for (int pass = 0; pass < kPasses; ++pass) {
    const int index = thread + pass * THREADS;
    const int row = index / kChunks, chunk = index % kChunks;
    const int key = tile_key0 + row;
    src[pass] = nullptr;
    if (key >= visible_key && key < end_key) {
      const int page = table[key / page_size];
      if (page >= 0)
        src[pass] = pool + ((static_cast<size_t>(page) * page_size + key % page_size) * num_kv_heads + kv_head) * D + chunk * 8;
    }
  }
#pragma unroll
  for (int pass = 0; pass < kPasses; ++pass) {
    const int index = thread + pass * THREADS;
    const int row = index / kChunks, chunk = index % kChunks;
    cp_async_16(tile + tile_offset<D>(row, chunk), src[pass] ? src[pass] : pool, src[pass] != nullptr);
  }
}

// One warp folds a block of KEYS keys into its running state for its 16 rows.
//   q_frag: the warp's 16 x D queries as A fragments, one per 16 columns of D
//   k_tile, v_tile: shared tiles [KEYS][D]
//   key0: position of the tile's first key; row_limit[2]: the last visible key of the rows
//   this thread owns (lane/4 and lane/4 + 8); row_first[2]: their first visible key.
template <int D, int KEYS>
__device__ __forceinline__ void fold_block(const uint32_t (&q_frag)[D / 16][4], uint32_t k_tile, uint32_t v_tile,
                                           int key0, const int (&row_first)[2], const int (&row_limit)[2],
                                           float scale_log2, float (&row_max)[2], float (&row_sum)[2],
                                           float (&out)[D / 8][4]) {
  const int lane = threadIdx.x & 31;
  float s[KEYS / 8][4];
#pragma unroll
  for (int n = 0; n < KEYS / 8; ++n)
#pragma unroll
    for (int i = 0; i < 4; ++i) s[n][i] = 0.0f;
  // scores = q . k^T
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
    for (int np = 0; np < KEYS / 16; ++np) {
      uint32_t b[4];
      const int row = np * 16 + (lane & 7) + ((lane >> 4) << 3);
      const int chunk = ks * 2 + ((lane >> 3) & 1);
      ldmatrix_x4(b, k_tile + tile_offset<D>(row, chunk));
      mma_16816(s[2 * np], q_frag[ks], b[0], b[1]);
      mma_16816(s[2 * np + 1], q_frag[ks], b[2], b[3]);
    }
  }
  // mask, running max
  float block_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int n = 0; n < KEYS / 8; ++n) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int key = key0 + n * 8 + 2 * (lane & 3) + (i & 1);
      const int r = i >> 1;
      const bool visible = key >= row_first[r] && key <= row_limit[r];
      s[n][i] = visible ? s[n][i] * scale_log2 : -INFINITY;
      block_max[r] = fmaxf(block_max[r], s[n][i]);
    }
  }
  float rescale[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    block_max[r] = fmaxf(block_max[r], __shfl_xor_sync(0xffffffffu, block_max[r], 1));
    block_max[r] = fmaxf(block_max[r], __shfl_xor_sync(0xffffffffu, block_max[r], 2));
    const float new_max = fmaxf(row_max[r], block_max[r]);
    // a row that has seen no visible key yet keeps max = -inf; guard the exponent
    rescale[r] = new_max == -INFINITY ? 1.0f : exp2f(row_max[r] - new_max);
    row_max[r] = new_max;
  }
  float block_sum[2] = {0.0f, 0.0f};
#pragma unroll
  for (int n = 0; n < KEYS / 8; ++n) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = i >> 1;
      const float p = row_max[r] == -INFINITY ? 0.0f : exp2f(s[n][i] - row_max[r]);
      s[n][i] = p;
      block_sum[r] += p;
    }
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) row_sum[r] = row_sum[r] * rescale[r] + block_sum[r];
#pragma unroll
  for (int n = 0; n < D / 8; ++n) {
    out[n][0] *= rescale[0];
    out[n][1] *= rescale[0];
    out[n][2] *= rescale[1];
    out[n][3] *= rescale[1];
  }
  // out += p . v
#pragma unroll
  for (int kk = 0; kk < KEYS / 16; ++kk) {
    uint32_t a[4];
    a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
    a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
    a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
    a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
    for (int np = 0; np < D / 16; ++np) {
      uint32_t b[4];
      const int row = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
      const int chunk = np * 2 + (lane >> 4);
      ldmatrix_x4_trans(b, v_tile + tile_offset<D>(row, chunk));
      mma_16816(out[2 * np], a, b[0], b[1]);
      mma_16816(out[2 * np + 1], a, b[2], b[3]);
    }
  }
}

// One warp's copy of ROWS (16 or 32) cache rows into its tile: in every pass the warp reads
// two whole rows (16 lanes x 16 bytes each), so global reads are contiguous.  Rows whose keys
// lie outside [visible_key, end_key) are filled with zeros, or left as they are when
// ZERO_FILL is false (a second copy that adds rows to a tile filled before).
template <int D, int ROWS, bool ZERO_FILL = true>
__device__ __forceinline__ void load_kv_rows(uint32_t k_tile, uint32_t v_tile, const __nv_bfloat16* __restrict__ k_pool,
                                             const __nv_bfloat16* __restrict__ v_pool, const int* __restrict__ table,
                                             int page_size, int page_shift, int num_kv_heads, int kv_head,
                                             int tile_key0, int visible_key, int end_key, int lane) {
  static_assert(ROWS == 16 || ROWS == 32, "a warp copies 16 or 32 rows");
  constexpr int kChunks = D / 8;            // 16-byte chunks in a row
  constexpr int kRowsPerPass = 32 / kChunks;  // 2 for d = 128, 4 for d = 64
  const int chunk = lane % kChunks;
  // Lane l finds where key tile_key0 + l lives (one block table read per lane, all at once);
  // the rows' offsets then travel by shuffle.  -1 marks a row that is not read.
  long long my_offset = -1;
  {
    const int key = tile_key0 + lane;
    if (lane < ROWS && key >= visible_key && key < end_key) {
      const int page = page_shift >= 0 ? table[key >> page_shift] : table[key / page_size];
      const int slot = page_shift >= 0 ? (key & (page_size - 1)) : key % page_size;
      if (page >= 0)
        my_offset = ((static_cast<long long>(page) * page_size + slot) * num_kv_heads + kv_head) * D;
    }
  }
#pragma unroll
  for (int pass = 0; pass < ROWS / kRowsPerPass; ++pass) {
    const int row = pass * kRowsPerPass + lane / kChunks;
    const long long offset = __shfl_sync(0xffffffffu, my_offset, row);
    const bool valid = offset >= 0;
    const long long at = valid ? offset + chunk * 8 : 0;
    if (ZERO_FILL || valid) {
      cp_async_16(k_tile + tile_offset<D>(row, chunk), k_pool + at, valid);
      cp_async_16(v_tile + tile_offset<D>(row, chunk), v_pool + at, valid);
    }
  }
}

template <int D>
__device__ __forceinline__ void load_kv_rows32(uint32_t k_tile, uint32_t v_tile, const __nv_bfloat16* __restrict__ k_pool,
                                               const __nv_bfloat16* __restrict__ v_pool, const int* __restrict__ table,
                                               int page_size, int page_shift, int num_kv_heads, int kv_head,
                                               int tile_key0, int visible_key, int end_key, int lane) {
  load_kv_rows<D, 32>(k_tile, v_tile, k_pool, v_pool, table, page_size, page_shift, num_kv_heads, kv_head, tile_key0,
                      visible_key, end_key, lane);
}

}  // namespace
