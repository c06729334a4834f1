// bfloat16 attention over the paged cache on the tensor cores (mma.sync m16n8k16), with
// 32-bit scores, softmax and accumulation.  Two kernels share their inner loop:
//
//   * prefill / mixed steps: one block per (64 queries of one entry, one or two query heads
//     of a KV group); four warps per head hold 16 queries each and walk the visible keys 64
//     at a time (every tile loaded once for both heads) with a running
//     (max, sum, output) — the flash form of the reference's online fold
//     (crates/vipera-backend-cpu/src/model.rs:2752-2857);
//   * decode (one query per entry): one block per (entry, KV head, split of the keys); the
//     query heads of the KV head's group are the rows of the tile, so that every key and
//     value is read once for the whole group (the reference's GQA sharing, model.rs:2221-2244,
//     crates/vipera-backend-gpu/src/layer.cu:182-292); each warp folds 32-key blocks of the
//     split, the block's four warps merge into one partial (max, sum, unnormalised output),
//     and a second kernel combines the splits' partials: m = max m_c, l = sum l_c e^(m_c - m), o = sum o_c e^(m_c - m) / l
//     (layer.cu:307-467).
//
// Definition computed: crates/vipera-backend-cpu/src/model.rs:1804-1859 (see attention.cu).
// Head sizes 64 and 128 are built; other sizes use the general kernel in attention.cu.
#include "attention_mma.cuh"

namespace {

// ---------------------------------------------------------------------------------------
// prefill / mixed: block = (tile of 64 queries of one entry, query head)
// ---------------------------------------------------------------------------------------
// HPC: query heads per block (1 or 2).  Two heads of the same KV group share every key and
// value tile the block loads; the block then has eight warps, four per head.
template <int D, int HPC>
__global__ void __launch_bounds__(128 * HPC)
attention_prefill_kernel(const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out,
                         const __nv_bfloat16* __restrict__ k_pool, const __nv_bfloat16* __restrict__ v_pool,
                         const int* __restrict__ entry_starts, const int* __restrict__ entry_pos0,
                         const int* __restrict__ block_table, int table_width, int page_size, int num_entries,
                         int num_heads, int num_kv_heads, float scale, int window, int skip_single) {
  constexpr int kQ = 64, kKeys = 64, kThreads = 128 * HPC;
  extern __shared__ __align__(128) uint8_t smem[];
  pdl_launch_dependents();
  pdl_wait();
  // Which (entry, tile of that entry) is this block?  Blocks are numbered from the back, so
  // that the tiles with the longest history (the last of each entry) start first.
  int entry = -1, tile_in_entry = 0;
  {
    int remaining = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);
    for (int e = 0; e < num_entries; ++e) {
      const int count = entry_starts[e + 1] - entry_starts[e];
      // entries of one token are left to the split-key kernel where the caller says so
      const int tiles = (skip_single && count == 1) ? 0 : (count + kQ - 1) / kQ;
      if (remaining < tiles) { entry = e; tile_in_entry = remaining; break; }
      remaining -= tiles;
    }
  }
  if (entry < 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.y * HPC + (warp >> 2);  // this warp's query head
  const int q_warp = warp & 3;                       // which 16 of the 64 queries
  const int kv_head = (blockIdx.y * HPC) / (num_heads / num_kv_heads);
  const int token0 = entry_starts[entry] + tile_in_entry * kQ;
  const int tokens_here = min(kQ, entry_starts[entry + 1] - token0);
  const int pos0 = entry_pos0[entry] + tile_in_entry * kQ;  // position of the tile's first query
  const int* table = block_table + static_cast<size_t>(entry) * table_width;

  const uint32_t q_tiles = smem_addr(smem);                   // [HPC][64][D]
  const uint32_t k_tiles = q_tiles + HPC * kQ * D * 2;        // two buffers of [64][D]
  const uint32_t v_tiles = k_tiles + 2 * kKeys * D * 2;

  // queries into shared memory (rows beyond the entry's tokens are zero)
  {
    constexpr int kChunks = D / 8;
    for (int index = threadIdx.x; index < HPC * kQ * kChunks; index += kThreads) {
      const int which = index / (kQ * kChunks);
      const int row = (index / kChunks) % kQ, chunk = index % kChunks;
      const bool valid = row < tokens_here;
      const __nv_bfloat16* src = q + (static_cast<size_t>(token0 + (valid ? row : 0)) * num_heads + blockIdx.y * HPC + which) * D + chunk * 8;
      cp_async_16(q_tiles + which * kQ * D * 2 + tile_offset<D>(row, chunk), src, valid);
    }
  }
  const int last_pos = pos0 + tokens_here - 1;
  const int first_key = window > 0 ? max(0, pos0 - window + 1) : 0;
  const int first_block = first_key / kKeys;
  const int end_key = last_pos + 1;
  const int num_blocks = (end_key + kKeys - 1) / kKeys - first_block;

  auto load_block = [&](int block, int buffer) {
    const int key0 = (first_block + block) * kKeys;
    load_kv_tile<D, kKeys, kThreads>(k_tiles + buffer * kKeys * D * 2, k_pool, table, page_size, num_kv_heads, kv_head,
                                     key0, first_key, end_key, threadIdx.x);
    load_kv_tile<D, kKeys, kThreads>(v_tiles + buffer * kKeys * D * 2, v_pool, table, page_size, num_kv_heads, kv_head,
                                     key0, first_key, end_key, threadIdx.x);
  };
  load_block(0, 0);
  cp_async_commit();

  uint32_t q_frag[D / 16][4];
  float acc[D / 8][4];
#pragma unroll
  for (int n = 0; n < D / 8; ++n)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[n][i] = 0.0f;
  float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.0f, 0.0f};
  int row_first[2], row_limit[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = q_warp * 16 + (lane >> 2) + r * 8;
    const int position = pos0 + row;
    row_limit[r] = row < tokens_here ? position : -1;  // rows past the end see nothing
    row_first[r] = window > 0 ? max(0, position - window + 1) : 0;
  }
  const float scale_log2 = scale * kLog2e;

  for (int block = 0; block < num_blocks; ++block) {
    const int buffer = block & 1;
    if (block + 1 < num_blocks) load_block(block + 1, buffer ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    if (block == 0) {
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks)
        ldmatrix_x4(q_frag[ks], q_tiles + (warp >> 2) * kQ * D * 2 +
                                    tile_offset<D>(q_warp * 16 + (lane & 15), ks * 2 + (lane >> 4)));
    }
    const int key0 = (first_block + block) * kKeys;
    // a warp whose 16 queries all stand before this block has nothing to see in it
    if (key0 <= pos0 + q_warp * 16 + 15)
      fold_block<D, kKeys>(q_frag, k_tiles + buffer * kKeys * D * 2, v_tiles + buffer * kKeys * D * 2, key0,
                           row_first, row_limit, scale_log2, row_max, row_sum, acc);
    __syncthreads();
  }
  cp_async_wait<0>();

  // normalise and store
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    float sum = row_sum[r];
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    const int row = q_warp * 16 + (lane >> 2) + r * 8;
    if (row >= tokens_here) continue;
    const float inverse = 1.0f / sum;
    __nv_bfloat16* dst = out + (static_cast<size_t>(token0 + row) * num_heads + head) * D;
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
      const int col = n * 8 + 2 * (lane & 3);
      *reinterpret_cast<__nv_bfloat162*>(dst + col) =
          __floats2bfloat162_rn(acc[n][2 * r] * inverse, acc[n][2 * r + 1] * inverse);
    }
  }
}

// ---------------------------------------------------------------------------------------
// decode: block = (entry, KV head, split); rows of the tile = query heads of the group
// ---------------------------------------------------------------------------------------
// partial layout: [token][head][split]: max (log2 units), sum, and D unnormalised outputs.
template <int D>
__global__ void __launch_bounds__(128, 3)
attention_decode_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pool,
                        const __nv_bfloat16* __restrict__ v_pool, const int* __restrict__ positions,
                        const int* __restrict__ block_table, int table_width, int page_size, int page_shift,
                        int num_heads, int num_kv_heads, float scale, int window, int chunk, int num_splits,
                        float* __restrict__ partial_ml, float* __restrict__ partial_out,
                        const int* __restrict__ entry_starts) {
  constexpr int kKeys = 32;
  constexpr int kWarpTile = 2 * kKeys * D * 2;  // bytes of one warp's key and value tiles
  static_assert(16 * (D + 4) * 4 <= kWarpTile, "a warp's partial must fit in its tiles");
  extern __shared__ __align__(128) uint8_t smem[];
  pdl_launch_dependents();
  // What follows up to pdl_wait() reads only what the host wrote before the step began (the
  // step's description: starts, positions, block tables) and keys and values of earlier steps.
  const int entry = blockIdx.x, kv_head = blockIdx.y, split = blockIdx.z;
  // Token i is entry i in a step of single tokens.  In a step with portions (`entry_starts`
  // given) the entry's token is where its tokens start, and entries that bring more than one
  // token are the flash kernel's.
  int token = entry;
  if (entry_starts) {
    token = entry_starts[entry];
    if (entry_starts[entry + 1] - token != 1) return;
  }
  const int group = num_heads / num_kv_heads;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int position = positions[entry];
  const int* table = block_table + static_cast<size_t>(entry) * table_width;
  const int first_visible = window > 0 ? max(0, position - window + 1) : 0;
  const int begin = max(split * chunk, first_visible / kKeys * kKeys);
  const int end = min((split + 1) * chunk, position + 1);
  if (begin >= end) return;  // a split without visible keys: the combine kernel skips it too

  uint8_t* q_bytes = smem;                                        // [16][D] bf16, shared by the warps
  uint8_t* warp_bytes = smem + 16 * D * 2 + warp * kWarpTile;
  const uint32_t q_tile = smem_addr(q_bytes);
  const uint32_t k_tile = smem_addr(warp_bytes);
  const uint32_t v_tile = k_tile + kKeys * D * 2;

  // The step's own key and value (at `position`) are written by the kernel ahead of this one;
  // every other row is from earlier steps.  A warp whose first block of keys does not hold
  // `position` asks for it now, before the wait: the block table and the cache are then read
  // while the kernel ahead still runs, and only the queries remain to be fetched after it.
  bool asked_early = false;
  {
    const int key0 = begin + warp * kKeys;
    if (key0 < end && !(position >= key0 && position < key0 + kKeys)) {
      load_kv_rows32<D>(k_tile, v_tile, k_pool, v_pool, table, page_size, page_shift, num_kv_heads, kv_head, key0,
                        first_visible, end, lane);
      asked_early = true;
    }
  }
  pdl_wait();

  for (int m_tile = 0; m_tile * 16 < group; ++m_tile) {
    __syncthreads();
    // this warp's first block of keys goes on its way before anything else
    int key0 = begin + warp * kKeys;
    if (key0 < end && !(asked_early && m_tile == 0)) {
      load_kv_rows32<D>(k_tile, v_tile, k_pool, v_pool, table, page_size, page_shift, num_kv_heads, kv_head, key0,
                        first_visible, end, lane);
    }
    {
      constexpr int kChunks = D / 8;
      for (int index = threadIdx.x; index < 16 * kChunks; index += 128) {
        const int row = index / kChunks, c = index % kChunks;
        const int head_in_group = m_tile * 16 + row;
        const bool valid = head_in_group < group;
        const __nv_bfloat16* src = q + (static_cast<size_t>(token) * num_heads + kv_head * group + (valid ? head_in_group : 0)) * D + c * 8;
        cp_async_16(q_tile + tile_offset<D>(row, c), src, valid);
      }
    }
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
    uint32_t q_frag[D / 16][4];
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks)
      ldmatrix_x4(q_frag[ks], q_tile + tile_offset<D>(lane & 15, ks * 2 + (lane >> 4)));

    float acc[D / 8][4];
#pragma unroll
    for (int n = 0; n < D / 8; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[n][i] = 0.0f;
    float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.0f, 0.0f};
    const int row_first[2] = {first_visible, first_visible};
    const int row_limit[2] = {position, position};
    const float scale_log2 = scale * kLog2e;

    for (; key0 < end; key0 += 4 * kKeys) {
      if (key0 != begin + warp * kKeys) {
        load_kv_rows32<D>(k_tile, v_tile, k_pool, v_pool, table, page_size, page_shift, num_kv_heads, kv_head, key0,
                          first_visible, end, lane);
        cp_async_commit();
        cp_async_wait<0>();
        __syncwarp();
      }
      fold_block<D, kKeys>(q_frag, k_tile, v_tile, key0, row_first, row_limit, scale_log2, row_max, row_sum, acc);
      __syncwarp();
    }

    // each warp leaves its partial in its own tiles: [16 rows][D + 4] floats
    float* mine = reinterpret_cast<float*>(warp_bytes);
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float sum = row_sum[r];
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      const int row = (lane >> 2) + r * 8;
      float* dst = mine + row * (D + 4);
      if ((lane & 3) == 0) {
        dst[D] = row_max[r];
        dst[D + 1] = sum;
      }
#pragma unroll
      for (int n = 0; n < D / 8; ++n) {
        const int col = n * 8 + 2 * (lane & 3);
        dst[col] = acc[n][2 * r];
        dst[col + 1] = acc[n][2 * r + 1];
      }
    }
    __syncthreads();
    // merge the four warps' partials: thread = (row, eighth of the columns)
    {
      const int row = threadIdx.x >> 3, part = threadIdx.x & 7;
      const int head_in_group = m_tile * 16 + row;
      if (head_in_group < group) {
        float m[4], best = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          m[w] = reinterpret_cast<const float*>(smem + 16 * D * 2 + w * kWarpTile)[row * (D + 4) + D];
          best = fmaxf(best, m[w]);
        }
        float weight[4], total = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          weight[w] = m[w] == -INFINITY ? 0.0f : exp2f(m[w] - best);
          total += weight[w] * reinterpret_cast<const float*>(smem + 16 * D * 2 + w * kWarpTile)[row * (D + 4) + D + 1];
        }
        const int head = kv_head * group + head_in_group;
        const size_t at = (static_cast<size_t>(entry) * num_heads + head) * num_splits + split;
        if (part == 0) {
          partial_ml[2 * at] = best;
          partial_ml[2 * at + 1] = total;
        }
        float* dst = partial_out + at * D;
#pragma unroll
        for (int c = 0; c < D / 8; c += 4) {
          const int col = part * (D / 8) + c;
          float4 value = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
          for (int w = 0; w < 4; ++w) {
            const float4 v = *reinterpret_cast<const float4*>(
                reinterpret_cast<const float*>(smem + 16 * D * 2 + w * kWarpTile) + row * (D + 4) + col);
            value.x += weight[w] * v.x;
            value.y += weight[w] * v.y;
            value.z += weight[w] * v.z;
            value.w += weight[w] * v.w;
          }
          *reinterpret_cast<float4*>(dst + col) = value;
        }
      }
    }
  }
}

// grid: (tokens, heads); one block of D threads combines the splits of one row.
template <int D>
__global__ void attention_combine_kernel(const float* __restrict__ partial_ml, const float* __restrict__ partial_out,
                                         int slices, __nv_bfloat16* __restrict__ out, int num_heads,
                                         const int* __restrict__ positions, int window, int chunk,
                                         const int* __restrict__ entry_starts) {
  __shared__ float maxima[128];
  __shared__ float sums[128];
  pdl_launch_dependents();
  // the step's description (written by the host before the step) is read before the wait
  const size_t row = static_cast<size_t>(blockIdx.x) * num_heads + blockIdx.y;
  size_t out_row = row;
  if (entry_starts) {   // a step with portions: only entries of one token, written at their token's row
    const int token = entry_starts[blockIdx.x];
    if (entry_starts[blockIdx.x + 1] - token != 1) return;
    out_row = static_cast<size_t>(token) * num_heads + blockIdx.y;
  }
  const float* ml = partial_ml + 2 * row * slices;
  const float* values = partial_out + row * slices * D + threadIdx.x;
  // only the splits that hold visible keys were written by the decode kernel
  const int position = positions[blockIdx.x];
  pdl_wait();
  const int first_visible = window > 0 ? max(0, position - window + 1) : 0;
  const int first = (first_visible / 32 * 32) / chunk;
  const int last = min(slices - 1, position / chunk);
  // Everything is asked for at once: this thread's column of every split's partial output (up to
  // kHeld of them stay in registers) beside all (max, sum) pairs, so that the combine costs one
  // trip to memory and not one per few splits; then the weights of the splits (at most 128 splits).
  constexpr int kHeld = 32;
  const int count = last - first + 1;
  float held[kHeld];
  if (count <= kHeld) {
#pragma unroll
    for (int i = 0; i < kHeld; ++i) held[i] = i < count ? values[static_cast<size_t>(first + i) * D] : 0.0f;
  }
  float mine = -INFINITY;
  for (int s = first + threadIdx.x; s <= last; s += D) {
    maxima[s] = ml[2 * s];
    sums[s] = ml[2 * s + 1];
  }
  __syncthreads();
  for (int s = first; s <= last; ++s) mine = fmaxf(mine, maxima[s]);
  float total = 0.0f, value = 0.0f;
  if (count <= kHeld) {
#pragma unroll
    for (int i = 0; i < kHeld; ++i) {
      if (i < count) {
        const float m = maxima[first + i];
        const float w = m == -INFINITY ? 0.0f : exp2f(m - mine);  // a split that saw no key
        total += sums[first + i] * w;
        value += held[i] * w;
      }
    }
  } else {
#pragma unroll 8
    for (int s = first; s <= last; ++s) {
      const float m = maxima[s];
      const float w = m == -INFINITY ? 0.0f : exp2f(m - mine);
      total += sums[s] * w;
      value += values[static_cast<size_t>(s) * D] * w;
    }
  }
  out[out_row * D + threadIdx.x] = __float2bfloat16_rn(value / total);
}

// ---------------------------------------------------------------------------------------
// Decode attention as one kernel: the splits of an (entry, KV head) form a thread-block
// cluster, keep their partial results in their own shared memory and combine them through
// distributed shared memory, so that no partial goes to global memory and no second kernel
// runs.  A block walks its share of the keys 128 at a time (32 per warp) with the next 128
// already on their way.  The share is cut from the entry's own length, not from the longest
// length the step allows, so the cluster's blocks carry equal loads.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  return rank;
}
// a float at `local` (a shared-memory address of this block) in the block of rank `rank`
__device__ __forceinline__ float cluster_load(uint32_t local, uint32_t rank) {
  uint32_t remote;
  float value;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(value) : "r"(remote) : "memory");
  return value;
}

template <int D, int kClusterBlocks, bool PREFETCH>
__global__ void __launch_bounds__(128, PREFETCH ? 1 : 3)
attention_decode_cluster_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pool,
                                const __nv_bfloat16* __restrict__ v_pool, const int* __restrict__ positions,
                                const int* __restrict__ block_table, int table_width, int page_size, int page_shift,
                                int num_heads, int num_kv_heads, float scale, int window, __nv_bfloat16* __restrict__ out) {
  constexpr int kKeys = 32;
  constexpr int kWarpTile = 2 * kKeys * D * 2;  // bytes of one warp's key and value tiles
  constexpr int kRow = D + 4;                   // floats of a partial row: D outputs, max, sum, padding
  static_assert(16 * kRow * 4 <= kWarpTile, "a warp's partial must fit in its tiles");
  extern __shared__ __align__(128) uint8_t smem[];
  pdl_launch_dependents();
  // up to pdl_wait(): only what the host wrote before the step, and keys and values of earlier steps
  const int entry = blockIdx.x, kv_head = blockIdx.y;
  const int rank = static_cast<int>(cluster_rank());
  const int group = num_heads / num_kv_heads;   // at most 16 (the launcher sees to it)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int position = positions[entry];
  const int* table = block_table + static_cast<size_t>(entry) * table_width;
  const int first_visible = window > 0 ? max(0, position - window + 1) : 0;
  // this block's share of the visible keys, in steps of 128
  const int first = first_visible / kKeys * kKeys;
  const int visible = position + 1 - first;
  const int chunk = ((visible + kClusterBlocks - 1) / kClusterBlocks + 127) / 128 * 128;
  const int begin = first + rank * chunk;
  const int end = min(begin + chunk, position + 1);

  uint8_t* q_bytes = smem;                                              // [16][D] bf16
  constexpr int kBuffers = PREFETCH ? 2 : 1;
  uint8_t* warp_bytes = smem + 16 * D * 2 + warp * kBuffers * kWarpTile;  // one or two buffers of (keys, values)
  float* merged = reinterpret_cast<float*>(smem + 16 * D * 2 + 4 * kBuffers * kWarpTile);  // [16][kRow]
  const uint32_t q_tile = smem_addr(q_bytes);
  const uint32_t tiles = smem_addr(warp_bytes);

  // This warp's first block of keys goes on its way before the wait unless it holds the step's own
  // key (the kernel ahead writes that one); then the queries of the group, which that kernel wrote.
  int key0 = begin + warp * kKeys;
  const bool early = key0 < end && !(position >= key0 && position < key0 + kKeys);
  if (early)
    load_kv_rows32<D>(tiles, tiles + kKeys * D * 2, k_pool, v_pool, table, page_size, page_shift, num_kv_heads, kv_head, key0,
                      first_visible, end, lane);
  pdl_wait();
  {
    constexpr int kChunks = D / 8;
    for (int index = threadIdx.x; index < 16 * kChunks; index += 128) {
      const int row = index / kChunks, c = index % kChunks;
      const bool valid = row < group;
      const __nv_bfloat16* src = q + (static_cast<size_t>(entry) * num_heads + kv_head * group + (valid ? row : 0)) * D + c * 8;
      cp_async_16(q_tile + tile_offset<D>(row, c), src, valid);
    }
  }
  if (key0 < end && !early)
    load_kv_rows32<D>(tiles, tiles + kKeys * D * 2, k_pool, v_pool, table, page_size, page_shift, num_kv_heads, kv_head, key0,
                      first_visible, end, lane);
  cp_async_commit();

  float acc[D / 8][4];
#pragma unroll
  for (int n = 0; n < D / 8; ++n)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[n][i] = 0.0f;
  float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.0f, 0.0f};
  const int row_first[2] = {first_visible, first_visible};
  const int row_limit[2] = {position, position};
  const float scale_log2 = scale * kLog2e;
  uint32_t q_frag[D / 16][4];
  bool have_q = false;
  int buffer = 0;
  for (; key0 < end; key0 += 4 * kKeys, buffer ^= PREFETCH ? 1 : 0) {
    const uint32_t k_tile = tiles + buffer * kWarpTile, v_tile = k_tile + kKeys * D * 2;
    const int next = key0 + 4 * kKeys;
    if (PREFETCH && next < end) {
      const uint32_t k_next = tiles + (buffer ^ 1) * kWarpTile;
      load_kv_rows32<D>(k_next, k_next + kKeys * D * 2, k_pool, v_pool, table, page_size, page_shift, num_kv_heads, kv_head,
                        next, first_visible, end, lane);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      if (!PREFETCH && key0 != begin + warp * kKeys) {
        load_kv_rows32<D>(k_tile, v_tile, k_pool, v_pool, table, page_size, page_shift, num_kv_heads, kv_head, key0,
                          first_visible, end, lane);
        cp_async_commit();
      }
      cp_async_wait<0>();
    }
    if (!have_q) {
      __syncthreads();  // the queries were copied by all threads; every warp with keys comes here once
      have_q = true;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks)
        ldmatrix_x4(q_frag[ks], q_tile + tile_offset<D>(lane & 15, ks * 2 + (lane >> 4)));
    }
    __syncwarp();
    fold_block<D, kKeys>(q_frag, k_tile, v_tile, key0, row_first, row_limit, scale_log2, row_max, row_sum, acc);
    __syncwarp();
  }
  cp_async_wait<0>();
  if (!have_q) __syncthreads();  // warps without keys meet the others at the same barrier

  // each warp leaves its partial in its own first buffer: [16 rows][kRow] floats
  float* mine = reinterpret_cast<float*>(warp_bytes);
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    float sum = row_sum[r];
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    const int row = (lane >> 2) + r * 8;
    float* dst = mine + row * kRow;
    if ((lane & 3) == 0) {
      dst[D] = row_max[r];
      dst[D + 1] = sum;
    }
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
      const int col = n * 8 + 2 * (lane & 3);
      dst[col] = acc[n][2 * r];
      dst[col + 1] = acc[n][2 * r + 1];
    }
  }
  __syncthreads();
  // the block's four partials become one: thread = (row, eighth of the columns)
  {
    const int row = threadIdx.x >> 3, part = threadIdx.x & 7;
    float m[4], best = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      m[w] = reinterpret_cast<const float*>(smem + 16 * D * 2 + w * kBuffers * kWarpTile)[row * kRow + D];
      best = fmaxf(best, m[w]);
    }
    float weight[4], total = 0.0f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      weight[w] = m[w] == -INFINITY ? 0.0f : exp2f(m[w] - best);
      total += weight[w] * reinterpret_cast<const float*>(smem + 16 * D * 2 + w * kBuffers * kWarpTile)[row * kRow + D + 1];
    }
    if (part == 0) {
      merged[row * kRow + D] = best;
      merged[row * kRow + D + 1] = total;
    }
#pragma unroll
    for (int c = 0; c < D / 8; c += 4) {
      const int col = part * (D / 8) + c;
      float4 value = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float4 v = *reinterpret_cast<const float4*>(
            reinterpret_cast<const float*>(smem + 16 * D * 2 + w * kBuffers * kWarpTile) + row * kRow + col);
        value.x += weight[w] * v.x;
        value.y += weight[w] * v.y;
        value.z += weight[w] * v.z;
        value.w += weight[w] * v.w;
      }
      *reinterpret_cast<float4*>(merged + row * kRow + col) = value;
    }
  }
  // every block's partial is in place; the blocks share the heads among them and each reads
  // the eight partials of its heads through distributed shared memory
  cluster_sync_all();
  const uint32_t merged_addr = smem_addr(merged);
  for (int head_in_group = rank; head_in_group < group; head_in_group += kClusterBlocks) {
    const int col = threadIdx.x;
    if (col < D) {
      float maxima[kClusterBlocks], best = -INFINITY;
#pragma unroll
      for (int b = 0; b < kClusterBlocks; ++b) {
        maxima[b] = cluster_load(merged_addr + (head_in_group * kRow + D) * 4, b);
        best = fmaxf(best, maxima[b]);
      }
      float total = 0.0f, value = 0.0f;
#pragma unroll
      for (int b = 0; b < kClusterBlocks; ++b) {
        const float w = maxima[b] == -INFINITY ? 0.0f : exp2f(maxima[b] - best);  // a block that saw no key
        total += w * cluster_load(merged_addr + (head_in_group * kRow + D + 1) * 4, b);
        value += w * cluster_load(merged_addr + (head_in_group * kRow + col) * 4, b);
      }
      const int head = kv_head * group + head_in_group;
      out[(static_cast<size_t>(entry) * num_heads + head) * D + col] = __float2bfloat16_rn(value / total);
    }
  }
  // nobody leaves while its partial may still be read
  cluster_sync_all();
}

template <int D, int HPC>
int launch_prefill_variant(const void* q, void* out, const void* k_pool, const void* v_pool, const int* entry_starts,
                           const int* entry_pos0, const int* block_table, int table_width, int page_size,
                           int num_entries, int num_tokens, int num_heads, int num_kv_heads, float scale, int window,
                           int skip_single, cudaStream_t s) {
  constexpr int kSmem = (HPC * 64 + 4 * 64) * D * 2;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel<D, HPC>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  // at most one partly filled tile per entry beyond the full ones
  dim3 grid((num_tokens + 63) / 64 + num_entries, num_heads / HPC);
  return vipera_launch(attention_prefill_kernel<D, HPC>, grid, dim3(128 * HPC), kSmem, s,
      static_cast<const __nv_bfloat16*>(q), static_cast<__nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(k_pool),
      static_cast<const __nv_bfloat16*>(v_pool), entry_starts, entry_pos0, block_table, table_width, page_size,
      num_entries, num_heads, num_kv_heads, scale, window, skip_single);
}

template <int D>
int launch_prefill(const void* q, void* out, const void* k_pool, const void* v_pool, const int* entry_starts,
                   const int* entry_pos0, const int* block_table, int table_width, int page_size, int num_entries,
                   int num_tokens, int num_heads, int num_kv_heads, float scale, int window, int skip_single,
                   cudaStream_t s) {
  // two heads per block where the heads of a KV group pair up
  if ((num_heads / num_kv_heads) % 2 == 0)
    return launch_prefill_variant<D, 2>(q, out, k_pool, v_pool, entry_starts, entry_pos0, block_table, table_width,
                                        page_size, num_entries, num_tokens, num_heads, num_kv_heads, scale, window,
                                        skip_single, s);
  return launch_prefill_variant<D, 1>(q, out, k_pool, v_pool, entry_starts, entry_pos0, block_table, table_width,
                                      page_size, num_entries, num_tokens, num_heads, num_kv_heads, scale, window,
                                      skip_single, s);
}

// The one-kernel form serves a step of few entries whose groups of heads fit one MMA tile.
// How many blocks a cluster has is chosen by how many clusters the step has (an experiment
// may force a form: VIPERA_ATTENTION_CLUSTER=8p, 8, 16p, 16, where p keeps the next keys on
// their way; "0" means the two-kernel form always).
struct ClusterChoice {
  int blocks;     // 0: the two-kernel form
  bool prefetch;
};
static ClusterChoice cluster_decode_choice(int num_entries, int num_heads, int num_kv_heads, int max_keys) {
  const char* choice = std::getenv("VIPERA_ATTENTION_CLUSTER");
  if ((choice && choice[0] == '0') || num_heads / num_kv_heads > 16) return {0, false};
  if (choice && choice[0] == '8') return {8, choice[1] == 'p'};
  if (choice && choice[0] == '1') return {16, choice[2] == 'p'};
  // Measured on the 1.5B shape at 2,048 keys (ms a step; two-kernel form, 8 blocks, 16 blocks):
  // batch 1: 1.60, 1.52, 1.47; batch 2: 1.60, 1.53, 1.44; batch 4: 1.68, 1.49, 1.56; batch 8: 1.60,
  // 1.64, 1.78; batch 64: 2.42, 3.56, 5.24.  Clusters pay where the step has few blocks and the
  // second kernel is a large part of it; with many clusters their placement costs more than
  // the second kernel did.  A block's share is kept to about 512 keys.
  const long clusters = static_cast<long>(num_entries) * num_kv_heads;
  if (clusters <= 4 && max_keys <= 8192) return {16, true};
  if (clusters <= 8 && max_keys <= 4096) return {8, true};
  return {0, false};
}

template <int D, int BLOCKS, bool PREFETCH>
int launch_decode_cluster(const void* q, void* out, const void* k_pool, const void* v_pool, const int* positions,
                          const int* block_table, int table_width, int page_size, int page_shift, int num_entries,
                          int num_heads, int num_kv_heads, float scale, int window, cudaStream_t s) {
  constexpr int kSmem = 16 * D * 2 + 4 * (PREFETCH ? 2 : 1) * (2 * 32 * D * 2) + 16 * (D + 4) * 4;
  static int configured = 0;  // 1: ready, -1: this cluster size cannot be launched here
  if (configured == 0) {
    cudaError_t e = cudaFuncSetAttribute(attention_decode_cluster_kernel<D, BLOCKS, PREFETCH>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
    if (e == cudaSuccess && BLOCKS > 8)
      e = cudaFuncSetAttribute(attention_decode_cluster_kernel<D, BLOCKS, PREFETCH>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e != cudaSuccess) {
      cudaGetLastError();
      configured = -1;
    } else {
      configured = 1;
    }
  }
  if (configured < 0) return VIPERA_BAD_SHAPE;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(num_entries, num_kv_heads, BLOCKS);
  config.blockDim = dim3(128);
  config.dynamicSmemBytes = kSmem;
  config.stream = s;
  cudaLaunchAttribute attributes[2];
  attributes[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attributes[0].val.programmaticStreamSerializationAllowed = vipera_pdl_enabled() ? 1 : 0;
  attributes[1].id = cudaLaunchAttributeClusterDimension;
  attributes[1].val.clusterDim.x = 1;
  attributes[1].val.clusterDim.y = 1;
  attributes[1].val.clusterDim.z = BLOCKS;
  config.attrs = attributes;
  config.numAttrs = 2;
  cudaError_t error = cudaLaunchKernelEx(&config, attention_decode_cluster_kernel<D, BLOCKS, PREFETCH>,
                                         static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k_pool),
                                         static_cast<const __nv_bfloat16*>(v_pool), positions, block_table, table_width,
                                         page_size, page_shift, num_heads, num_kv_heads, scale, window,
                                         static_cast<__nv_bfloat16*>(out));
  return error == cudaSuccess ? VIPERA_OK : static_cast<int>(error);
}

template <int D>
int launch_decode(const void* q, void* out, const void* k_pool, const void* v_pool, const int* positions,
                  const int* block_table, int table_width, int page_size, int num_entries, int num_heads,
                  int num_kv_heads, float scale, int window, int chunk, int num_splits, float* partial_ml,
                  float* partial_out, const int* entry_starts, cudaStream_t s) {
  constexpr int kSmem = 16 * D * 2 + 4 * 2 * 32 * D * 2;
  int page_shift = -1;
  if ((page_size & (page_size - 1)) == 0) {
    page_shift = 0;
    while ((1 << page_shift) < page_size) ++page_shift;
  }
  // the one-kernel forms serve steps of single tokens only
  const ClusterChoice cluster = entry_starts ? ClusterChoice{0, false}
                                             : cluster_decode_choice(num_entries, num_heads, num_kv_heads, chunk * num_splits);
  if (cluster.blocks == 8 && cluster.prefetch)
    return launch_decode_cluster<D, 8, true>(q, out, k_pool, v_pool, positions, block_table, table_width, page_size,
                                             page_shift, num_entries, num_heads, num_kv_heads, scale, window, s);
  if (cluster.blocks == 8)
    return launch_decode_cluster<D, 8, false>(q, out, k_pool, v_pool, positions, block_table, table_width, page_size,
                                              page_shift, num_entries, num_heads, num_kv_heads, scale, window, s);
  if (cluster.blocks == 16 && cluster.prefetch)
    return launch_decode_cluster<D, 16, true>(q, out, k_pool, v_pool, positions, block_table, table_width, page_size,
                                              page_shift, num_entries, num_heads, num_kv_heads, scale, window, s);
  if (cluster.blocks == 16)
    return launch_decode_cluster<D, 16, false>(q, out, k_pool, v_pool, positions, block_table, table_width, page_size,
                                               page_shift, num_entries, num_heads, num_kv_heads, scale, window, s);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  dim3 grid(num_entries, num_kv_heads, num_splits);
  int status = vipera_launch(attention_decode_kernel<D>, grid, 128, kSmem, s,
      static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k_pool),
      static_cast<const __nv_bfloat16*>(v_pool), positions, block_table, table_width, page_size, page_shift,
      num_heads, num_kv_heads, scale, window, chunk, num_splits, partial_ml, partial_out, entry_starts);
  if (status != VIPERA_OK) return status;
  return vipera_launch(attention_combine_kernel<D>, dim3(num_entries, num_heads), D, 0, s,
      static_cast<const float*>(partial_ml), static_cast<const float*>(partial_out), num_splits,
      static_cast<__nv_bfloat16*>(out), num_heads, positions, window, chunk, entry_starts);
}

}  // namespace

// Attention of a step with portions of any length.  q and out are bfloat16 [tokens, heads, d];
// entry_starts [entries + 1] are cumulative token counts and entry_pos0 [entries] the position
// of each entry's first token.  Head sizes: 64 and 128.  With `skip_single`, entries of one
// token are left out (the caller runs vipera_attention_decode over them).
VIPERA_API int vipera_attention_prefill(const void* q, void* out, const void* k_pool, const void* v_pool,
                                        const int* entry_starts, const int* entry_pos0, const int* block_table,
                                        int table_width, int page_size, int num_entries, int num_tokens,
                                        int num_heads, int num_kv_heads, int head_dim, float scale, int window,
                                        int skip_single, void* stream) {
  if (num_tokens <= 0 || num_entries <= 0) return VIPERA_OK;
  if (num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads) return VIPERA_BAD_SHAPE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (head_dim == 128)
    return launch_prefill<128>(q, out, k_pool, v_pool, entry_starts, entry_pos0, block_table, table_width, page_size,
                               num_entries, num_tokens, num_heads, num_kv_heads, scale, window, skip_single, s);
  if (head_dim == 64)
    return launch_prefill<64>(q, out, k_pool, v_pool, entry_starts, entry_pos0, block_table, table_width, page_size,
                              num_entries, num_tokens, num_heads, num_kv_heads, scale, window, skip_single, s);
  return VIPERA_BAD_SHAPE;
}

// Floats of scratch a decode launch needs: (2 + d) per (entry, head, slice).
VIPERA_API size_t vipera_attention_decode_scratch(int num_entries, int num_heads, int head_dim, int num_splits) {
  // (max, sum) pairs first, padded so that the outputs after them start on 16 bytes
  const size_t rows = static_cast<size_t>(num_entries) * num_heads * num_splits;
  return ((2 * rows + 3) / 4) * 4 + rows * head_dim;
}

// Attention of the entries that bring one token.  With `entry_starts` null every entry does
// (token i belongs to entry i, at positions[i]).  With `entry_starts` [entries + 1] given the step
// has portions too: entry e's token is entry_starts[e], its position positions[e] (the entry's
// first position), and entries of more tokens are skipped (vipera_attention_prefill with
// skip_single runs those); q and out are then [tokens, heads, d] of the whole step.
// The keys of an entry are cut into `num_splits` ranges of `chunk` keys (a multiple of 32).
VIPERA_API int vipera_attention_decode(const void* q, void* out, const void* k_pool, const void* v_pool,
                                       const int* positions, const int* block_table, int table_width, int page_size,
                                       int num_entries, int num_heads, int num_kv_heads, int head_dim, float scale,
                                       int window, int chunk, int num_splits, float* scratch, size_t scratch_floats,
                                       const int* entry_starts, void* stream) {
  if (num_entries <= 0) return VIPERA_OK;
  if (num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads) return VIPERA_BAD_SHAPE;
  if (chunk <= 0 || chunk % 32 || num_splits <= 0 || num_splits > 128) return VIPERA_BAD_ARGUMENT;
  const size_t need = vipera_attention_decode_scratch(num_entries, num_heads, head_dim, num_splits);
  if (!scratch || scratch_floats < need) return VIPERA_BAD_ARGUMENT;
  const size_t rows = static_cast<size_t>(num_entries) * num_heads * num_splits;
  float* partial_ml = scratch;
  float* partial_out = scratch + ((2 * rows + 3) / 4) * 4;
  if (reinterpret_cast<uintptr_t>(scratch) & 15) return VIPERA_BAD_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (head_dim == 128)
    return launch_decode<128>(q, out, k_pool, v_pool, positions, block_table, table_width, page_size, num_entries,
                              num_heads, num_kv_heads, scale, window, chunk, num_splits, partial_ml, partial_out,
                              entry_starts, s);
  if (head_dim == 64)
    return launch_decode<64>(q, out, k_pool, v_pool, positions, block_table, table_width, page_size, num_entries,
                             num_heads, num_kv_heads, scale, window, chunk, num_splits, partial_ml, partial_out,
                             entry_starts, s);
  return VIPERA_BAD_SHAPE;
}

VIPERA_API const char* vipera_attention_mma_status_text(int status) { return vipera_status_text(status); }
