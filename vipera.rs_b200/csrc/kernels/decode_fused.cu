// A whole decode step of a pre-norm decoder (RMSNorm, grouped-query attention with rotary
// pairs over the paged cache, SwiGLU) for up to 16 single-token entries as ONE persistent
// kernel: embedding, every scheduled layer, the final norm and the output matrix.
//
// Why one kernel.  With a handful of tokens each product of the step is a stream of weights
// that takes a few microseconds; launched one by one, every kernel pays its start, the wait
// for its predecessor's last block, and an empty memory pipe until its own first loads come
// back.  Here one block per SM stays resident for the whole step:
//
//   * one warp of every block (the producer) walks the step's weight matrices in the order
//     they are used and copies this block's share of their rows into a ring of shared-memory
//     stages with TMA (boxes of 8 rows x 256 k, completing on mbarriers).  It depends on no
//     activation, so it never stops at a boundary between products: while the other warps
//     wait for the grid or do attention, the ring fills with the weights that come next;
//   * eight warps (the consumers) multiply the staged rows with the step's tokens on the
//     tensor cores (mma.sync m16n8k16, 32-bit accumulation), finish each product with its
//     ending (bias + rotary pairs + cache write; residual addition; SwiGLU; logits) and meet
//     the other blocks at a grid-wide barrier where the next product needs every block's
//     results.
//
// Work is cut into tiles of 16 weight rows with all of K; tile i of the step's tile sequence
// belongs to block i mod gridDim, so the blocks carry equal shares whatever the sizes are.
// The 16 rows of a tile are chosen so that its ending needs no other block: rows i..i+7 and
// i+d/2..i+d/2+7 of one head for q/k/v (the two halves of rotary pairs), 8 gate rows and the
// 8 up rows of the same features for SwiGLU, 16 consecutive rows elsewhere.  The eight warps
// split each stage's 512 k among them and add their partial sums in warp order, so a result
// does not depend on timing.
//
// Attention is the split-key form of attention_mma.cu inside a phase of this kernel: an item
// is (entry, KV head, 128 keys), the query heads of the group are the rows of the tile, each
// warp folds 16 keys, and the block that finishes an (entry, KV head)'s last item combines
// all of its partials (counted with one atomic per item; the sum runs in key order).
//
// The computation is the one of the separate kernels, which follow the reference's decode
// order (crates/vipera-backend-cpu/src/model.rs:977-1252: norm, q/k/v with bias, rotation,
// cache write, attention, output product, norm, gate/up, activation, down, final norm, output
// matrix).  The reference has no such kernel: its device path launches one kernel per
// operation (crates/vipera-backend-gpu/src/layer.cu).
//
// Every wait (ring barriers, grid barrier) is bounded.  A wait that runs out stores an error
// code in the status word and sets a flag that makes every later wait of the block return at
// once; other blocks see the status word at their next grid barrier.  The launcher's caller
// reads the status word after the step.
#include <cuda.h>

#include "attention_mma.cuh"

enum { FUSED_WAIT_EXPIRED = 2 };
enum FusedRope { FUSED_ROPE_NONE = 0, FUSED_ROPE_NEOX = 1 };

struct FusedLayer {
  const __nv_bfloat16* w_qkv;      // [(heads + 2 kv_heads) * d, hidden]
  const float* b_qkv;              // [(heads + 2 kv_heads) * d] or null
  const float* norm1;              // [hidden]
  const __nv_bfloat16* w_o;        // [hidden, heads * d]
  const float* norm2;              // [hidden]
  const __nv_bfloat16* w_gate_up;  // [2 * inter, hidden], gate and up rows alternating in groups of 16
  const __nv_bfloat16* w_down;     // [hidden, inter]
  __nv_bfloat16* k_pool;           // [pages, page_size, kv_heads, d]
  __nv_bfloat16* v_pool;
  const int* block_table;          // [entries, table_width]
  const float* cos_table;          // [positions, d / 2]
  const float* sin_table;
  float eps1, eps2, scale;
  int table_width, page_size, window, writes_cache;
  int num_heads, num_kv_heads, inter, rope_style;
};

struct FusedModel {
  const FusedLayer* layers;        // device array, in execution order
  const CUtensorMap* maps;         // device array [4 * layers + 1]: q/k/v, output, gate/up and down matrix of every
                                   // layer, then the output matrix of the model, as TMA sees them
  const int* tokens;               // [T]
  const int* positions;            // [T]: position of each entry's token
  const __nv_bfloat16* embedding;  // [vocab, hidden]
  float* x;                        // [T, hidden] residual stream
  __nv_bfloat16* q;                // [T, heads * d]
  __nv_bfloat16* attn;             // [T, heads * d]
  __nv_bfloat16* act;              // [T, inter]
  float* partial_ml;               // [T, heads, max_chunks, 2]
  float* partial_out;              // [T, heads, max_chunks, d]
  unsigned int* counters;          // [T * kv_heads], zero between uses
  const float* final_norm;         // [hidden]
  const __nv_bfloat16* head;       // [vocab, hidden]
  float* logits;                   // [T, vocab]
  unsigned int* barrier;           // one word, zero at launch
  int* status;                     // device word: 0, or an error code
  long long* trace;                // null, or [blocks][2 + 10 * layers] timestamps (ns) for profiling
  float final_eps, logit_scale;
  int T, hidden, vocab, num_layers, max_chunks, head_dim;
  // shared-memory plan, made by the launcher
  int ring_stages, union_bytes;
};

namespace {

constexpr int kComputeWarps = 8;
constexpr int kComputeThreads = kComputeWarps * 32;
constexpr int kFusedThreads = kComputeThreads + 32;  // + the producer warp
#ifndef VIPERA_FUSED_STAGE_K
#define VIPERA_FUSED_STAGE_K 512
#endif
constexpr int kStageK = VIPERA_FUSED_STAGE_K;        // k per ring stage, split evenly among the consumer warps
constexpr int kWarpK = kStageK / 8;                  // k per consumer warp and stage
constexpr int kWarpSteps = kWarpK / 32;              // 32 k (two MMAs) per step
constexpr int kBoxK = 256;                           // a TMA box: 256 k of 8 rows
constexpr int kBoxRows = 8;
constexpr int kBoxBytes = kBoxK * kBoxRows * 2;
constexpr int kBoxesK = kStageK / kBoxK;             // boxes along k in a stage
constexpr int kStageBytes = 2 * kBoxesK * kBoxBytes; // [k box][row group][8 rows][256 k]
constexpr int kActPad = 64;
constexpr int kItemKeys = 16;                        // keys one warp folds per attention item
constexpr int kChunkKeys = kComputeWarps * kItemKeys;
constexpr int kMaxTokens = 16;
constexpr int kMaxStages = 12;
constexpr uint32_t kWaitLimit = 1u << 22;
constexpr int kPrefetch = 4;                         // stages ahead for activations read from global

enum TileKind { TILE_PLAIN = 0, TILE_QKV = 1, TILE_GATE_UP = 2 };

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(done) : "r"(smem_addr(bar)), "r"(parity) : "memory");
  return done != 0;
}
__device__ __forceinline__ void tma_load_box(void* dst, const CUtensorMap* map, uint64_t* bar, int k, int row) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_addr(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_addr(bar)), "r"(k), "r"(row) : "memory");
}
// the eight consumer warps meet (the producer warp never takes part)
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kComputeThreads) : "memory"); }
__device__ __forceinline__ unsigned int load_acquire(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Row `r` (0..15) of tile `tile` in a matrix of the given kind.
__device__ __forceinline__ int tile_row(int kind, int tile, int r, int head_dim) {
  if (kind == TILE_QKV) {
    const int per_head = head_dim >> 4;
    return (tile / per_head) * head_dim + (tile % per_head) * 8 + (r & 7) + (r >> 3) * (head_dim >> 1);
  }
  if (kind == TILE_GATE_UP) {
    const int feature = tile * 8 + (r & 7);
    return (feature >> 4) * 32 + (feature & 15) + (r >> 3) * 16;
  }
  return tile * 16 + r;
}

// What every role of a block shares.
struct Shared {
  uint8_t* ring;
  uint8_t* region;        // activations of a product, or the tiles of the attention phase
  float* partial;         // two buffers of [8 warps][NT * 8 tokens][16 rows]
  uint64_t* full;
  uint64_t* empty;
  volatile int* abort_flag;
  volatile int* flag;
  int* positions;         // [16]
  int stages;
};

__device__ __forceinline__ void bounded_wait(uint64_t* bar, uint32_t parity, const Shared& sh, int* status) {
  for (uint32_t spin = 0; spin < kWaitLimit; ++spin) {
    if (mbar_try_wait(bar, parity)) return;
    if ((spin & 1023u) == 1023u && *sh.abort_flag) return;
  }
  *sh.abort_flag = 1;
  atomicExch(status, FUSED_WAIT_EXPIRED);
}

// ---------------------------------------------------------------------------------------
// the producer warp
// ---------------------------------------------------------------------------------------
struct RingCursor {
  int slot = 0;
  uint32_t parity = 0;
  int base = 0;  // block that owns tile 0 of the next matrix
  __device__ __forceinline__ void advance(int stages) {
    if (++slot == stages) { slot = 0; parity ^= 1u; }
  }
};

// A stage holds kStageK k of a tile's two groups of 8 consecutive rows, as boxes
// [k box][row group][8 rows][256 k]; lanes 0 .. 2 * kBoxesK - 1 of the producer warp issue one
// box each.  Rows past the matrix arrive as zeros.
__device__ __forceinline__ void produce_matrix(const Shared& sh, RingCursor& cur, const CUtensorMap* map, int K,
                                               int tiles, int kind, int head_dim, int* status) {
  const int lane = threadIdx.x & 31;
  const int grid = gridDim.x;
  int first = static_cast<int>(blockIdx.x) - cur.base;
  if (first < 0) first += grid;
  const int box_k = lane >> 1, group = lane & 1;  // which box of the stage this lane issues
  for (int tile = first; tile < tiles; tile += grid) {
    const int row = tile_row(kind, tile, group * 8, head_dim);  // first of the group's 8 consecutive rows
    for (int k0 = 0; k0 < K; k0 += kStageK) {
      const int boxes_k = min(kBoxesK, (K - k0 + kBoxK - 1) / kBoxK);
      if (lane == 0) {
        bounded_wait(&sh.empty[cur.slot], cur.parity ^ 1u, sh, status);
        if (!*sh.abort_flag) mbar_expect_tx(&sh.full[cur.slot], static_cast<uint32_t>(2 * boxes_k * kBoxBytes));
      }
      __syncwarp();
      if (*sh.abort_flag) return;
      if (box_k < boxes_k)
        tma_load_box(sh.ring + static_cast<size_t>(cur.slot) * kStageBytes + (box_k * 2 + group) * kBoxBytes, map,
                     &sh.full[cur.slot], k0 + box_k * kBoxK, row);
      cur.advance(sh.stages);
    }
  }
  cur.base = (cur.base + tiles) % grid;
}

template <int D>
__device__ void producer(const FusedModel& m, const Shared& sh) {
  RingCursor cur;
  for (int l = 0; l < m.num_layers; ++l) {
    const FusedLayer& L = m.layers[l];
    const int q_dim = L.num_heads * D;
    const int qkv_tiles = (L.num_heads + (L.writes_cache ? 2 * L.num_kv_heads : 0)) * (D / 16);
    const CUtensorMap* maps = m.maps + 4 * l;
    produce_matrix(sh, cur, maps + 0, m.hidden, qkv_tiles, TILE_QKV, D, m.status);
    produce_matrix(sh, cur, maps + 1, q_dim, (m.hidden + 15) / 16, TILE_PLAIN, D, m.status);
    produce_matrix(sh, cur, maps + 2, m.hidden, L.inter / 8, TILE_GATE_UP, D, m.status);
    produce_matrix(sh, cur, maps + 3, L.inter, (m.hidden + 15) / 16, TILE_PLAIN, D, m.status);
    if (*sh.abort_flag) return;
  }
  produce_matrix(sh, cur, m.maps + 4 * m.num_layers, m.hidden, (m.vocab + 15) / 16, TILE_PLAIN, D, m.status);
}

// ---------------------------------------------------------------------------------------
// the consumers
// ---------------------------------------------------------------------------------------
struct Consumer {
  RingCursor cur;
  unsigned int barrier_target = 0;
  int partial_buffer = 0;
  int mark = 0;
};

__device__ __forceinline__ void trace_mark(const FusedModel& m, Consumer& c) {
  if (m.trace && threadIdx.x == 0) {
    long long now;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
    m.trace[static_cast<size_t>(blockIdx.x) * (2 + 10 * m.num_layers) + c.mark] = now;
  }
  ++c.mark;
}

// All blocks meet.  Writes made before the barrier by any thread of any block are visible to
// every thread after it (reads of such data bypass L1: __ldcg).
__device__ __forceinline__ void grid_barrier(const FusedModel& m, const Shared& sh, Consumer& c) {
  consumer_sync();
  c.barrier_target += gridDim.x;
  if (threadIdx.x == 0 && !*sh.abort_flag) {
    __threadfence();
    atomicAdd(m.barrier, 1u);
    uint32_t spin = 0;
    while (load_acquire(m.barrier) < c.barrier_target) {
      if (++spin >= kWaitLimit) {
        *sh.abort_flag = 1;
        atomicExch(m.status, FUSED_WAIT_EXPIRED);
        break;
      }
      if ((spin & 255u) == 255u && *reinterpret_cast<volatile int*>(m.status) != 0) {
        *sh.abort_flag = 1;  // another block gave up
        break;
      }
    }
    __threadfence();
  }
  consumer_sync();
}

// The normalised residual stream of the step's tokens as bfloat16 rows in shared memory
// (rows past T are zero): x * rsqrt(mean(x^2) + eps) * w, statistics in 32-bit.
template <int NT>
__device__ __forceinline__ void stage_normed(const Shared& sh, const float* x, const float* weight, float eps, int T,
                                             int K) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int stride = K * 2 + kActPad;
  const int chunks = K >> 3;
  const uint4 zero = make_uint4(0, 0, 0, 0);
  for (int t = warp; t < NT * 8; t += kComputeWarps) {
    uint4* dst = reinterpret_cast<uint4*>(sh.region + static_cast<size_t>(t) * stride);
    if (t >= T) {
      for (int c = lane; c < chunks; c += 32) dst[c] = zero;
      continue;
    }
    const float* row = x + static_cast<size_t>(t) * K;
    float squares = 0.0f;
    for (int c = lane; c < chunks; c += 32) {
      const float4 x0 = __ldcg(reinterpret_cast<const float4*>(row + c * 8));
      const float4 x1 = __ldcg(reinterpret_cast<const float4*>(row + c * 8 + 4));
      squares += x0.x * x0.x + x0.y * x0.y + x0.z * x0.z + x0.w * x0.w + x1.x * x1.x + x1.y * x1.y + x1.z * x1.z + x1.w * x1.w;
    }
    squares = warp_sum(squares);
    const float inverse = 1.0f / sqrtf(squares / static_cast<float>(K) + eps);
    for (int c = lane; c < chunks; c += 32) {
      const float4 x0 = __ldcg(reinterpret_cast<const float4*>(row + c * 8));
      const float4 x1 = __ldcg(reinterpret_cast<const float4*>(row + c * 8 + 4));
      const float4 g0 = *reinterpret_cast<const float4*>(weight + c * 8);
      const float4 g1 = *reinterpret_cast<const float4*>(weight + c * 8 + 4);
      uint4 packed;
      __nv_bfloat162* halves = reinterpret_cast<__nv_bfloat162*>(&packed);
      halves[0] = __floats2bfloat162_rn(x0.x * inverse * g0.x, x0.y * inverse * g0.y);
      halves[1] = __floats2bfloat162_rn(x0.z * inverse * g0.z, x0.w * inverse * g0.w);
      halves[2] = __floats2bfloat162_rn(x1.x * inverse * g1.x, x1.y * inverse * g1.y);
      halves[3] = __floats2bfloat162_rn(x1.z * inverse * g1.z, x1.w * inverse * g1.w);
      dst[c] = packed;
    }
  }
  consumer_sync();
}

// This block's tiles of one matrix: out[t, row] = sum_k act[t, k] * W[row, k], finished by
// `finish(row_lo, row_hi, t, v_lo, v_hi)` for every token and every pair of rows (r, r + 8)
// of a tile.  ACT_SHARED: activations are the rows staged in shared memory; otherwise they
// are bfloat16 rows [T, K] in global memory written by other blocks before the last barrier.
template <int NT, bool ACT_SHARED, typename Finish>
__device__ __forceinline__ void consume_matrix(const FusedModel& m, const Shared& sh, Consumer& c, int N, int K, int tiles,
                                               int kind, int head_dim, const __nv_bfloat16* act, Finish finish) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, tq = lane & 3;
  const int grid = gridDim.x;
  const int T = m.T;
  const int act_stride = K * 2 + kActPad;
  const uint4 zero = make_uint4(0, 0, 0, 0);
  const int stages = (K + kStageK - 1) / kStageK;
  int first = static_cast<int>(blockIdx.x) - c.cur.base;
  if (first < 0) first += grid;
  for (int tile = first; tile < tiles; tile += grid) {
    float acc[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[n][i] = 0.0f;

    // activations from global memory: kPrefetch stages ahead, in registers
    uint4 ahead[ACT_SHARED ? 1 : kPrefetch][kWarpSteps][NT];
    auto fetch = [&](int stage, uint4 (&dst)[kWarpSteps][NT]) {
#pragma unroll
      for (int u = 0; u < kWarpSteps; ++u) {
        const int k = stage * kStageK + warp * kWarpK + u * 32 + tq * 8;
#pragma unroll
        for (int n = 0; n < NT; ++n) {
          const int t = n * 8 + g;
          dst[u][n] = (k < K && t < T) ? __ldcg(reinterpret_cast<const uint4*>(act + static_cast<size_t>(t) * K + k)) : zero;
        }
      }
    };
    if (!ACT_SHARED) {
#pragma unroll
      for (int j = 0; j < kPrefetch; ++j) fetch(j, ahead[j]);
    }

    for (int stage0 = 0; stage0 < stages; stage0 += kPrefetch) {
#pragma unroll
      for (int j = 0; j < kPrefetch; ++j) {
        const int stage = stage0 + j;
        if (stage >= stages) break;
        bounded_wait(&sh.full[c.cur.slot], c.cur.parity, sh, m.status);
        const uint8_t* rows = sh.ring + static_cast<size_t>(c.cur.slot) * kStageBytes;
        const int k_warp = stage * kStageK + warp * kWarpK;
#ifdef VIPERA_FUSED_SKIP_MATH
        if (false) {
#else
        if (k_warp < K && !*sh.abort_flag) {
#endif
#pragma unroll
          for (int u = 0; u < kWarpSteps; ++u) {
            if (k_warp + u * 32 >= K) break;
            const int local = warp * kWarpK + u * 32 + tq * 8;  // k inside the stage
            const uint8_t* at = rows + (local / kBoxK) * 2 * kBoxBytes + g * (kBoxK * 2) + (local % kBoxK) * 2;
            const uint4 lo = *reinterpret_cast<const uint4*>(at);
            const uint4 hi = *reinterpret_cast<const uint4*>(at + kBoxBytes);
#pragma unroll
            for (int n = 0; n < NT; ++n) {
              uint4 b;
              if (ACT_SHARED) {
                b = *reinterpret_cast<const uint4*>(sh.region + static_cast<size_t>(n * 8 + g) * act_stride +
                                                    static_cast<size_t>(k_warp + u * 32 + tq * 8) * 2);
              } else {
                b = ahead[ACT_SHARED ? 0 : j][u][n];
              }
              mma_bf16(acc[n], lo.x, hi.x, lo.y, hi.y, b.x, b.y);
              mma_bf16(acc[n], lo.z, hi.z, lo.w, hi.w, b.z, b.w);
            }
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh.empty[c.cur.slot]);
        c.cur.advance(sh.stages);
        if (!ACT_SHARED) fetch(stage + kPrefetch, ahead[ACT_SHARED ? 0 : j]);
      }
    }

    // the warps' partial sums meet in shared memory and are added in warp order
    float* buffer = sh.partial + static_cast<size_t>(c.partial_buffer) * kComputeWarps * NT * 8 * 16;
    c.partial_buffer ^= 1;
    {
      float* mine = buffer + static_cast<size_t>(warp) * NT * 8 * 16;
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        const int t0 = n * 8 + 2 * tq;
        mine[t0 * 16 + g] = acc[n][0];
        mine[(t0 + 1) * 16 + g] = acc[n][1];
        mine[t0 * 16 + g + 8] = acc[n][2];
        mine[(t0 + 1) * 16 + g + 8] = acc[n][3];
      }
    }
    consumer_sync();
    for (int item = threadIdx.x; item < T * 8; item += kComputeThreads) {
      const int t = item >> 3, r = item & 7;
      float v_lo = 0.0f, v_hi = 0.0f;
#pragma unroll
      for (int w = 0; w < kComputeWarps; ++w) {
        const float* src = buffer + (static_cast<size_t>(w) * NT * 8 + t) * 16;
        v_lo += src[r];
        v_hi += src[r + 8];
      }
      const int row_lo = tile_row(kind, tile, r, head_dim);
      const int row_hi = tile_row(kind, tile, r + 8, head_dim);
      if (row_lo < N) finish(row_lo, row_hi, t, v_lo, v_hi);
    }
  }
  c.cur.base = (c.cur.base + tiles) % grid;
}

// ---------------------------------------------------------------------------------------
// attention of the step's tokens over the cache
// ---------------------------------------------------------------------------------------
template <int D>
__device__ void attention_phase(const FusedModel& m, const FusedLayer& L, const Shared& sh) {
  constexpr int kSlab = 16 * (D + 4) * 4;  // a warp's key and value tiles, later its partial
  static_assert(2 * kItemKeys * D * 2 <= kSlab, "a warp's tiles must fit in its slab");
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int T = m.T, kv_heads = L.num_kv_heads, heads = L.num_heads;
  const int group = heads / kv_heads;
  const int window = L.window;
  int page_shift = -1;
  if ((L.page_size & (L.page_size - 1)) == 0) page_shift = 31 - __clz(L.page_size);

  uint8_t* q_bytes = sh.region;
  uint8_t* slabs = sh.region + 16 * D * 2;
  uint8_t* slab = slabs + warp * kSlab;
  const uint32_t q_tile = smem_addr(q_bytes);
  const uint32_t k_tile = smem_addr(slab);
  const uint32_t v_tile = k_tile + kItemKeys * D * 2;
  const float scale_log2 = L.scale * kLog2e;

  int total = 0;
  for (int e = 0; e < T; ++e) {
    const int position = sh.positions[e];
    const int first_visible = window > 0 ? max(0, position - window + 1) : 0;
    total += (position / kChunkKeys - first_visible / kChunkKeys + 1) * kv_heads;
  }

  for (int item = blockIdx.x; item < total; item += gridDim.x) {
    // which (entry, chunk of keys, KV head) is this item?
    int entry = 0, rest = item, position = 0, first_visible = 0, chunk0 = 0, chunks = 0;
    for (int e = 0; e < T; ++e) {
      position = sh.positions[e];
      first_visible = window > 0 ? max(0, position - window + 1) : 0;
      chunk0 = first_visible / kChunkKeys;
      chunks = position / kChunkKeys - chunk0 + 1;
      entry = e;
      if (rest < chunks * kv_heads) break;
      rest -= chunks * kv_heads;
    }
    const int chunk = chunk0 + rest / kv_heads;
    const int kv_head = rest % kv_heads;
    const int* table = L.block_table + static_cast<size_t>(entry) * L.table_width;
    const int end = min((chunk + 1) * kChunkKeys, position + 1);
    const int key0 = chunk * kChunkKeys + warp * kItemKeys;

    consumer_sync();  // the slabs of the item before are read
    if (key0 < end)
      load_kv_rows<D, kItemKeys>(k_tile, v_tile, L.k_pool, L.v_pool, table, L.page_size, page_shift, kv_heads, kv_head,
                                 key0, first_visible, end, lane);
    {
      constexpr int kChunks = D / 8;
      for (int index = threadIdx.x; index < 16 * kChunks; index += kComputeThreads) {
        const int row = index / kChunks, c = index % kChunks;
        const bool valid = row < group;
        const __nv_bfloat16* src = m.q + (static_cast<size_t>(entry) * heads + kv_head * group + (valid ? row : 0)) * D + c * 8;
        cp_async_16(q_tile + tile_offset<D>(row, c), src, valid);
      }
    }
    cp_async_commit();
    cp_async_wait<0>();
    consumer_sync();

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
    if (key0 < end)
      fold_block<D, kItemKeys>(q_frag, k_tile, v_tile, key0, row_first, row_limit, scale_log2, row_max, row_sum, acc);
    __syncwarp();

    // the warp's partial over its tiles: [16 rows][D + 4] floats
    float* mine = reinterpret_cast<float*>(slab);
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
    consumer_sync();
    // merge the eight warps' partials: thread = (row, sixteenth of the columns)
    constexpr int kCols = D / 16;
    const int row = threadIdx.x >> 4, part = threadIdx.x & 15;
    if (row < group) {
      float mx[kComputeWarps], best = -INFINITY;
#pragma unroll
      for (int w = 0; w < kComputeWarps; ++w) {
        mx[w] = reinterpret_cast<const float*>(slabs + w * kSlab)[row * (D + 4) + D];
        best = fmaxf(best, mx[w]);
      }
      float weight[kComputeWarps], sum = 0.0f;
#pragma unroll
      for (int w = 0; w < kComputeWarps; ++w) {
        weight[w] = mx[w] == -INFINITY ? 0.0f : exp2f(mx[w] - best);
        sum += weight[w] * reinterpret_cast<const float*>(slabs + w * kSlab)[row * (D + 4) + D + 1];
      }
      const int head = kv_head * group + row;
      const size_t at = (static_cast<size_t>(entry) * heads + head) * m.max_chunks + chunk;
      if (part == 0) {
        __stcg(m.partial_ml + 2 * at, best);
        __stcg(m.partial_ml + 2 * at + 1, sum);
      }
      float* dst = m.partial_out + at * D;
#pragma unroll
      for (int cc = 0; cc < kCols; cc += 4) {
        const int col = part * kCols + cc;
        float4 value = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
        for (int w = 0; w < kComputeWarps; ++w) {
          const float4 v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(slabs + w * kSlab) + row * (D + 4) + col);
          value.x += weight[w] * v.x;
          value.y += weight[w] * v.y;
          value.z += weight[w] * v.z;
          value.w += weight[w] * v.w;
        }
        __stcg(reinterpret_cast<float4*>(dst + col), value);
      }
    }
    // the block that brings an (entry, KV head)'s last partial combines all of them
    __threadfence();
    consumer_sync();
    if (threadIdx.x == 0) {
      const unsigned int before = atomicAdd(m.counters + entry * kv_heads + kv_head, 1u);
      *sh.flag = before == static_cast<unsigned int>(chunks - 1) ? 1 : 0;
    }
    consumer_sync();
    if (*sh.flag) {
      __threadfence();
      if (row < group) {
        const int head = kv_head * group + row;
        const size_t base = (static_cast<size_t>(entry) * heads + head) * m.max_chunks;
        float best = -INFINITY;
        for (int c = chunk0; c < chunk0 + chunks; ++c) best = fmaxf(best, __ldcg(m.partial_ml + 2 * (base + c)));
        float sum = 0.0f;
        float value[kCols];
#pragma unroll
        for (int i = 0; i < kCols; ++i) value[i] = 0.0f;
        for (int c = chunk0; c < chunk0 + chunks; ++c) {
          const float mc = __ldcg(m.partial_ml + 2 * (base + c));
          const float w = mc == -INFINITY ? 0.0f : exp2f(mc - best);
          sum += w * __ldcg(m.partial_ml + 2 * (base + c) + 1);
          const float* src = m.partial_out + (base + c) * D + part * kCols;
#pragma unroll
          for (int i = 0; i < kCols; i += 4) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(src + i));
            value[i] += w * v.x;
            value[i + 1] += w * v.y;
            value[i + 2] += w * v.z;
            value[i + 3] += w * v.w;
          }
        }
        const float inverse = 1.0f / sum;
        __nv_bfloat16* dst = m.attn + (static_cast<size_t>(entry) * heads + head) * D + part * kCols;
#pragma unroll
        for (int i = 0; i < kCols; i += 2)
          *reinterpret_cast<__nv_bfloat162*>(dst + i) = __floats2bfloat162_rn(value[i] * inverse, value[i + 1] * inverse);
      }
      if (threadIdx.x == 0) m.counters[entry * kv_heads + kv_head] = 0u;
    }
  }
}

// ---------------------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------------------
template <int NT, int D>
__device__ void consumers(const FusedModel& m, const Shared& sh) {
  Consumer c;
  const int T = m.T, H = m.hidden;
  // embedding rows into the 32-bit residual stream
  {
    const int chunks = H >> 3;
    for (int index = blockIdx.x * kComputeThreads + threadIdx.x; index < T * chunks; index += gridDim.x * kComputeThreads) {
      const int t = index / chunks, ch = index % chunks;
      const uint4 packed = *reinterpret_cast<const uint4*>(m.embedding + static_cast<size_t>(m.tokens[t]) * H + ch * 8);
      const __nv_bfloat162* halves = reinterpret_cast<const __nv_bfloat162*>(&packed);
      const float2 a = __bfloat1622float2(halves[0]), b = __bfloat1622float2(halves[1]);
      const float2 cc = __bfloat1622float2(halves[2]), d = __bfloat1622float2(halves[3]);
      float* dst = m.x + static_cast<size_t>(t) * H + ch * 8;
      __stcg(reinterpret_cast<float4*>(dst), make_float4(a.x, a.y, b.x, b.y));
      __stcg(reinterpret_cast<float4*>(dst + 4), make_float4(cc.x, cc.y, d.x, d.y));
    }
  }
  trace_mark(m, c);
  grid_barrier(m, sh, c);
  trace_mark(m, c);

  for (int l = 0; l < m.num_layers; ++l) {
    const FusedLayer& L = m.layers[l];
    const int heads = L.num_heads, kv_heads = L.num_kv_heads;
    const int q_dim = heads * D, inter = L.inter;
    const int qkv_rows = (heads + 2 * kv_heads) * D;
    const int qkv_tiles = (heads + (L.writes_cache ? 2 * kv_heads : 0)) * (D / 16);

    // ---- norm, q/k/v product, bias, rotation, cache write ----
    stage_normed<NT>(sh, m.x, L.norm1, L.eps1, T, H);
    consume_matrix<NT, true>(m, sh, c, qkv_rows, H, qkv_tiles, TILE_QKV, D, nullptr,
        [&](int row_lo, int row_hi, int t, float v_lo, float v_hi) {
          if (L.b_qkv) { v_lo += L.b_qkv[row_lo]; v_hi += L.b_qkv[row_hi]; }
          constexpr int half = D / 2;
          const int head = row_lo / D, i = row_lo % D;
          const int position = sh.positions[t];
          const bool is_q = head < heads;
          const bool is_v = head >= heads + kv_heads;
          if (!is_v && L.rope_style == FUSED_ROPE_NEOX) {
            const float cs = L.cos_table[static_cast<size_t>(position) * half + i];
            const float sn = L.sin_table[static_cast<size_t>(position) * half + i];
            const float lo = v_lo * cs - v_hi * sn, hi = v_lo * sn + v_hi * cs;
            v_lo = lo;
            v_hi = hi;
          }
          __nv_bfloat16* dst = nullptr;
          if (is_q) {
            dst = m.q + (static_cast<size_t>(t) * heads + head) * D;
          } else {
            const int page = L.block_table[static_cast<size_t>(t) * L.table_width + position / L.page_size];
            if (page >= 0) {
              const int kv_head = is_v ? head - heads - kv_heads : head - heads;
              __nv_bfloat16* pool = is_v ? L.v_pool : L.k_pool;
              dst = pool + ((static_cast<size_t>(page) * L.page_size + position % L.page_size) * kv_heads + kv_head) * D;
            }
          }
          if (dst) {
            dst[i] = __float2bfloat16_rn(v_lo);
            dst[i + half] = __float2bfloat16_rn(v_hi);
          }
        });
    trace_mark(m, c);
    grid_barrier(m, sh, c);
    trace_mark(m, c);

    // ---- attention ----
    attention_phase<D>(m, L, sh);
    trace_mark(m, c);
    grid_barrier(m, sh, c);
    trace_mark(m, c);

    // ---- output product into the residual stream ----
    consume_matrix<NT, false>(m, sh, c, H, q_dim, (H + 15) / 16, TILE_PLAIN, D, m.attn,
        [&](int row_lo, int row_hi, int t, float v_lo, float v_hi) {
          float* at = m.x + static_cast<size_t>(t) * H;
          __stcg(at + row_lo, __ldcg(at + row_lo) + v_lo);
          if (row_hi < H) __stcg(at + row_hi, __ldcg(at + row_hi) + v_hi);
        });
    trace_mark(m, c);
    grid_barrier(m, sh, c);
    trace_mark(m, c);

    // ---- norm, gate and up products, activation ----
    stage_normed<NT>(sh, m.x, L.norm2, L.eps2, T, H);
    consume_matrix<NT, true>(m, sh, c, 2 * inter, H, inter / 8, TILE_GATE_UP, D, nullptr,
        [&](int row_lo, int row_hi, int t, float v_lo, float v_hi) {
          const int feature = (row_lo >> 5) * 16 + (row_lo & 15);
          const float value = v_hi * (v_lo / (1.0f + __expf(-v_lo)));
          m.act[static_cast<size_t>(t) * inter + feature] = __float2bfloat16_rn(value);
        });
    trace_mark(m, c);
    grid_barrier(m, sh, c);
    trace_mark(m, c);

    // ---- down product into the residual stream ----
    consume_matrix<NT, false>(m, sh, c, H, inter, (H + 15) / 16, TILE_PLAIN, D, m.act,
        [&](int row_lo, int row_hi, int t, float v_lo, float v_hi) {
          float* at = m.x + static_cast<size_t>(t) * H;
          __stcg(at + row_lo, __ldcg(at + row_lo) + v_lo);
          if (row_hi < H) __stcg(at + row_hi, __ldcg(at + row_hi) + v_hi);
        });
    trace_mark(m, c);
    grid_barrier(m, sh, c);
    trace_mark(m, c);
  }

  // ---- final norm and the output matrix ----
  stage_normed<NT>(sh, m.x, m.final_norm, m.final_eps, T, H);
  const int V = m.vocab;
  consume_matrix<NT, true>(m, sh, c, V, H, (V + 15) / 16, TILE_PLAIN, D, nullptr,
      [&](int row_lo, int row_hi, int t, float v_lo, float v_hi) {
        float* at = m.logits + static_cast<size_t>(t) * V;
        at[row_lo] = v_lo * m.logit_scale;
        if (row_hi < V) at[row_hi] = v_hi * m.logit_scale;
      });
}

template <int NT, int D>
__global__ void __launch_bounds__(kFusedThreads, 1) decode_fused_kernel(const FusedModel m) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  Shared sh;
  sh.stages = m.ring_stages;
  sh.ring = smem;
  sh.region = smem + static_cast<size_t>(sh.stages) * kStageBytes;
  sh.partial = reinterpret_cast<float*>(sh.region + m.union_bytes);
  uint8_t* tail = reinterpret_cast<uint8_t*>(sh.partial) + 2 * kComputeWarps * NT * 8 * 16 * sizeof(float);
  sh.full = reinterpret_cast<uint64_t*>(tail);
  sh.empty = sh.full + kMaxStages;
  sh.positions = reinterpret_cast<int*>(sh.empty + kMaxStages);
  sh.abort_flag = sh.positions + kMaxTokens;
  sh.flag = sh.abort_flag + 1;
  if (threadIdx.x == 0) {
    for (int s = 0; s < sh.stages; ++s) {
      mbar_init(&sh.full[s], 1);
      mbar_init(&sh.empty[s], kComputeWarps);
    }
    *sh.abort_flag = 0;
    *sh.flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (threadIdx.x < kMaxTokens) sh.positions[threadIdx.x] = threadIdx.x < m.T ? m.positions[threadIdx.x] : 0;
  __syncthreads();
  if (threadIdx.x >= kComputeThreads) {
    producer<D>(m, sh);
  } else {
    consumers<NT, D>(m, sh);
  }
}

constexpr int kSharedLimit = 227 * 1024;

struct SharedPlan {
  int stages, union_bytes, total;
};

SharedPlan plan_shared(int tokens, int hidden, int head_dim) {
  const int nt = tokens <= 8 ? 1 : 2;
  const int activations = nt * 8 * (hidden * 2 + kActPad);
  const int attention = 16 * head_dim * 2 + kComputeWarps * 16 * (head_dim + 4) * 4;
  SharedPlan plan{};
  plan.union_bytes = ((activations > attention ? activations : attention) + 127) / 128 * 128;
  const int fixed = plan.union_bytes + 2 * kComputeWarps * nt * 8 * 16 * 4 + 2 * kMaxStages * 8 + (kMaxTokens + 2) * 4 + 128 +
                    1024 /* the ring starts on a multiple of 1024 bytes */;
  plan.stages = (kSharedLimit - fixed) / kStageBytes;
  if (plan.stages > kMaxStages) plan.stages = kMaxStages;
  plan.total = fixed + plan.stages * kStageBytes;
  return plan;
}

template <int NT, int D>
int launch_fused(const FusedModel& m, int shared_bytes, cudaStream_t stream) {
  static bool configured = false;
  static int blocks = 0;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(decode_fused_kernel<NT, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSharedLimit);
    if (e != cudaSuccess) return static_cast<int>(e);
    int device = 0, sms = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    blocks = sms > 0 ? sms : 148;
    configured = true;
  }
  int resident = 0;
  cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, decode_fused_kernel<NT, D>, kFusedThreads, shared_bytes);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (resident < 1) return VIPERA_BAD_SHAPE;
  // every block must be resident at once (they wait for one another): a cooperative launch
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(blocks);
  config.blockDim = dim3(kFusedThreads);
  config.dynamicSmemBytes = shared_bytes;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeCooperative;
  attribute[0].val.cooperative = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  e = cudaMemsetAsync(m.barrier, 0, sizeof(unsigned int), stream);
  if (e != cudaSuccess) return static_cast<int>(e);
  e = cudaLaunchKernelEx(&config, decode_fused_kernel<NT, D>, m);
  return e == cudaSuccess ? VIPERA_OK : static_cast<int>(e);
}

}  // namespace

// A weight matrix [rows, K] (bfloat16, row-major, K a multiple of 8) as the kernel's producer reads
// it: boxes of 8 rows x 256 k, rows and k beyond the matrix filled with zeros.  `map` receives
// the 128 bytes of a CUtensorMap; the caller copies them to the device array of the model.
VIPERA_API int vipera_decode_fused_weight_map(void* map, const void* weight, int rows, int K) {
  typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeTiledFn encode = nullptr;
  if (!encode) {
    void* entry = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &result) != cudaSuccess ||
        result != cudaDriverEntryPointSuccess)
      return VIPERA_NO_DRIVER_ENTRY;
    encode = reinterpret_cast<EncodeTiledFn>(entry);
  }
  if (!map || !weight || rows <= 0 || K <= 0 || K % 8 || (reinterpret_cast<uintptr_t>(weight) & 15)) return VIPERA_BAD_ARGUMENT;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(K) * 2};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(kBoxK), static_cast<cuuint32_t>(kBoxRows)};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = encode(static_cast<CUtensorMap*>(map), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(weight),
                      dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? VIPERA_OK : VIPERA_BAD_ARGUMENT;
}

VIPERA_API int vipera_decode_fused_layer_size() { return static_cast<int>(sizeof(FusedLayer)); }
VIPERA_API int vipera_decode_fused_model_size() { return static_cast<int>(sizeof(FusedModel)); }
VIPERA_API int vipera_decode_fused_chunk_keys() { return kChunkKeys; }

// Whether the fused step takes these sizes: up to 16 tokens, head size 64 or 128, hidden and
// intermediate sizes that are multiples of 64 (the consumers' k steps) and a ring of at least
// four stages beside the activations in shared memory.
VIPERA_API int vipera_decode_fused_takes(int tokens, int hidden, int head_dim, int max_inter, int max_q_dim) {
  if (tokens <= 0 || tokens > kMaxTokens) return 0;
  if (head_dim != 64 && head_dim != 128) return 0;
  if (hidden <= 0 || hidden % 64 || max_inter <= 0 || max_inter % 64 || max_q_dim <= 0 || max_q_dim % 64) return 0;
  return plan_shared(tokens, hidden, head_dim).stages >= 4 ? 1 : 0;
}

// One decode step.  `model` is a host copy of the description; `model->layers` points to a
// device array.  The caller has checked the layers (see vipera_decode_fused_takes) and that
// every position is below max_chunks * 128.
VIPERA_API int vipera_decode_fused(const FusedModel* model, void* stream) {
  FusedModel m = *model;
  if (m.T <= 0) return VIPERA_OK;
  if (m.T > kMaxTokens || m.num_layers < 0 || m.hidden % 64 || m.max_chunks <= 0) return VIPERA_BAD_SHAPE;
  if (!m.layers || !m.maps || !m.tokens || !m.positions || !m.embedding || !m.x || !m.q || !m.attn || !m.act || !m.partial_ml ||
      !m.partial_out || !m.counters || !m.final_norm || !m.head || !m.logits || !m.barrier || !m.status)
    return VIPERA_BAD_ARGUMENT;
  const SharedPlan plan = plan_shared(m.T, m.hidden, m.head_dim);
  if (plan.stages < 4) return VIPERA_BAD_SHAPE;
  m.ring_stages = plan.stages;
  m.union_bytes = plan.union_bytes;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool wide = m.T > 8;
  if (m.head_dim == 128) return wide ? launch_fused<2, 128>(m, plan.total, s) : launch_fused<1, 128>(m, plan.total, s);
  if (m.head_dim == 64) return wide ? launch_fused<2, 64>(m, plan.total, s) : launch_fused<1, 64>(m, plan.total, s);
  return VIPERA_BAD_SHAPE;
}

VIPERA_API const char* vipera_decode_fused_status_text(int status) { return vipera_status_text(status); }
