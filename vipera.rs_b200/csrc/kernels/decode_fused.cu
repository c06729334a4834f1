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
//   * eight warps (the workers) multiply the staged rows with the step's tokens on the
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
// Attention is the split-key form of attention_mma.cu as two phases of this kernel: an item
// is (entry, KV head, 256 keys), the query heads of the group are the rows of the tile and
// each warp folds 32 keys (a block's first item is loaded while the blocks still wait for one
// another after the q/k/v product, all but the key that product writes); then every (entry,
// head) row's partials are combined in key order by one block.
//
// A ninth warp (the finisher) adds the workers' partial sums of a tile and writes its ending
// while the workers are already multiplying the next tile.
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

#include <cstdio>

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
  const float* final_norm;         // [hidden]
  const __nv_bfloat16* head;       // [vocab, hidden]
  float* logits;                   // [T, vocab]
  unsigned int* barrier;           // one word, zero at launch
  int* status;                     // device word: 0, or an error code
  long long* trace;                // null, or [blocks][2 + 12 * layers] timestamps (ns) for profiling
  float final_eps, logit_scale;
  int T, hidden, vocab, num_layers, max_chunks, head_dim;
  // shared-memory plan, made by the launcher
  int ring_stages, union_bytes;
};

namespace {

constexpr int kWorkerWarps = 8;
constexpr int kWorkerThreads = kWorkerWarps * 32;
constexpr int kFinisherWarp = kWorkerWarps;          // finishes tiles: sums the workers' partials, writes the ending
constexpr int kProducerWarp = kWorkerWarps + 1;      // feeds the ring of weight stages
constexpr int kBlockThreads = kWorkerThreads + 32;   // workers + finisher: who meets at the grid barrier
constexpr int kFusedThreads = kWorkerThreads + 64;
#ifndef VIPERA_FUSED_STAGE_K
#define VIPERA_FUSED_STAGE_K 512
#endif
constexpr int kStageK = VIPERA_FUSED_STAGE_K;        // k per ring stage, split evenly among the worker warps
constexpr int kWarpK = kStageK / kWorkerWarps;       // k per worker warp and stage
constexpr int kWarpSteps = kWarpK / 32;              // 32 k (two MMAs) per step
constexpr int kBoxK = 256;                           // a TMA box: 256 k of 8 rows
constexpr int kBoxRows = 8;
constexpr int kBoxBytes = kBoxK * kBoxRows * 2;
constexpr int kBoxesK = kStageK / kBoxK;             // boxes along k in a stage
constexpr int kStageBytes = 2 * kBoxesK * kBoxBytes; // [k box][row group][8 rows][256 k]
constexpr int kActPad = 64;
constexpr int kItemKeys = 32;                        // keys one warp folds per attention item
constexpr int kChunkKeys = kWorkerWarps * kItemKeys;
constexpr int kMaxTokens = 16;
constexpr int kMaxStages = 12;
constexpr int kMaxChunks = 512;                      // (max, sum) pairs of one row that fit the combine's shared memory
constexpr uint32_t kWaitLimit = 1u << 22;

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
// the eight worker warps meet
__device__ __forceinline__ void worker_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kWorkerThreads) : "memory"); }
// workers and finisher meet (the producer warp never takes part)
__device__ __forceinline__ void block_sync() { asm volatile("bar.sync 2, %0;" ::"n"(kBlockThreads) : "memory"); }
__device__ __forceinline__ unsigned int load_acquire(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void add_release(unsigned int* p, unsigned int value) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(value) : "memory");
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
  uint64_t* full;         // ring: a stage's boxes have arrived
  uint64_t* empty;        // ring: the workers have read a stage
  uint64_t* sums_full;    // [2] the workers' partial sums of a tile are written
  uint64_t* sums_empty;   // [2] the finisher has read them
  volatile int* abort_flag;
  int* positions;         // [16]
  int stages;
};

// True when the barrier's phase completed; false when the block has given up (here or elsewhere).
__device__ __forceinline__ bool bounded_wait(uint64_t* bar, uint32_t parity, const Shared& sh, int* status) {
  for (uint32_t spin = 0; spin < kWaitLimit; ++spin) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spin & 1023u) == 1023u && *sh.abort_flag) return false;
  }
  *sh.abort_flag = 1;
  atomicExch(status, FUSED_WAIT_EXPIRED);
  return false;
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
// workers and finisher
// ---------------------------------------------------------------------------------------
// The state both roles keep in step: where the ring stands, which block owns the next
// matrix's first tile, how many tiles this block has handed from workers to finisher.
struct Flow {
  RingCursor cur;
  unsigned int barrier_target = 0;
  int tiles_done = 0;
  int mark = 0;
#ifdef VIPERA_FUSED_TIMING
  long long t_wait = 0, t_math = 0, t_hand = 0, n_stage = 0;
#endif
};
#ifdef VIPERA_FUSED_TIMING
#define FUSED_TICK(var) const long long var = clock64()
#define FUSED_ADD(field, a, b) f.field += (b) - (a)
#else
#define FUSED_TICK(var)
#define FUSED_ADD(field, a, b)
#endif

__device__ __forceinline__ void trace_mark(const FusedModel& m, Flow& f) {
  if (m.trace && threadIdx.x == 0) {
    long long now;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
    m.trace[static_cast<size_t>(blockIdx.x) * (2 + 12 * m.num_layers) + f.mark] = now;
  }
  ++f.mark;
}

// All blocks meet.  Writes made before the barrier by any worker or finisher of any block are
// visible to all of them after it (reads of such data bypass L1: __ldcg, cp.async.cg).  The
// barrier comes in two halves, so that a block can start loads that depend on no other block
// between announcing itself and waiting for the others.
__device__ __forceinline__ void grid_arrive(const FusedModel& m, const Shared& sh, Flow& f) {
  block_sync();
  f.barrier_target += gridDim.x;
  if (threadIdx.x == 0 && !*sh.abort_flag) add_release(m.barrier, 1u);
}
__device__ __forceinline__ void grid_wait(const FusedModel& m, const Shared& sh, Flow& f) {
  if (threadIdx.x == 0 && !*sh.abort_flag) {
    uint32_t spin = 0;
    while (load_acquire(m.barrier) < f.barrier_target) {
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
  }
  block_sync();
}
__device__ __forceinline__ void grid_barrier(const FusedModel& m, const Shared& sh, Flow& f) {
  grid_arrive(m, sh, f);
  grid_wait(m, sh, f);
}

__device__ __forceinline__ uint4 pack_normed(const float4& x0, const float4& x1, const float4& g0, const float4& g1,
                                             float inverse) {
  uint4 packed;
  __nv_bfloat162* halves = reinterpret_cast<__nv_bfloat162*>(&packed);
  halves[0] = __floats2bfloat162_rn(x0.x * inverse * g0.x, x0.y * inverse * g0.y);
  halves[1] = __floats2bfloat162_rn(x0.z * inverse * g0.z, x0.w * inverse * g0.w);
  halves[2] = __floats2bfloat162_rn(x1.x * inverse * g1.x, x1.y * inverse * g1.y);
  halves[3] = __floats2bfloat162_rn(x1.z * inverse * g1.z, x1.w * inverse * g1.w);
  return packed;
}

// The normalised residual stream of the step's tokens as bfloat16 rows in shared memory
// (rows past T are zero): x * rsqrt(mean(x^2) + eps) * w, statistics in 32-bit.  Rows of up to
// 1536 values are read once and kept in registers between the two passes.
template <int NT>
__device__ __forceinline__ void stage_normed(const Shared& sh, const float* x, const float* weight, float eps, int T,
                                             int K) {
  constexpr int kKept = 6;  // chunks of 8 values per lane kept in registers
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int stride = K * 2 + kActPad;
  const int chunks = K >> 3;
  const uint4 zero = make_uint4(0, 0, 0, 0);
  for (int t = warp; t < NT * 8; t += kWorkerWarps) {
    uint4* dst = reinterpret_cast<uint4*>(sh.region + static_cast<size_t>(t) * stride);
    if (t >= T) {
      for (int c = lane; c < chunks; c += 32) dst[c] = zero;
      continue;
    }
    const float* row = x + static_cast<size_t>(t) * K;
    float squares = 0.0f;
    if (chunks <= 32 * kKept) {
      float4 kept[kKept][2];
#pragma unroll
      for (int i = 0; i < kKept; ++i) {
        const int c = lane + 32 * i;
        if (c < chunks) {
          kept[i][0] = __ldcg(reinterpret_cast<const float4*>(row + c * 8));
          kept[i][1] = __ldcg(reinterpret_cast<const float4*>(row + c * 8 + 4));
        }
      }
#pragma unroll
      for (int i = 0; i < kKept; ++i) {
        if (lane + 32 * i < chunks) {
          const float4 x0 = kept[i][0], x1 = kept[i][1];
          squares += x0.x * x0.x + x0.y * x0.y + x0.z * x0.z + x0.w * x0.w + x1.x * x1.x + x1.y * x1.y + x1.z * x1.z + x1.w * x1.w;
        }
      }
      squares = warp_sum(squares);
      const float inverse = 1.0f / sqrtf(squares / static_cast<float>(K) + eps);
#pragma unroll
      for (int i = 0; i < kKept; ++i) {
        const int c = lane + 32 * i;
        if (c < chunks) {
          const float4 g0 = *reinterpret_cast<const float4*>(weight + c * 8);
          const float4 g1 = *reinterpret_cast<const float4*>(weight + c * 8 + 4);
          dst[c] = pack_normed(kept[i][0], kept[i][1], g0, g1, inverse);
        }
      }
      continue;
    }
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
      dst[c] = pack_normed(x0, x1, g0, g1, inverse);
    }
  }
  worker_sync();
}

// Whether this block owns a tile of the next matrix of `tiles` tiles.
__device__ __forceinline__ bool owns_tile(const Flow& f, int tiles) {
  int first = static_cast<int>(blockIdx.x) - f.cur.base;
  if (first < 0) first += gridDim.x;
  return first < tiles;
}

// bfloat16 rows [T, count] of `source` (row pitch `pitch` elements, starting at column
// `begin`) into the shared region as the activations of the next stages; rows past T are zero.
template <int NT>
__device__ __forceinline__ void stage_copy(const Shared& sh, const __nv_bfloat16* source, int pitch, int begin, int count,
                                           int T) {
  const int stride = count * 2 + kActPad;
  const int chunks = count >> 3;
  for (int index = threadIdx.x; index < NT * 8 * chunks; index += kWorkerThreads) {
    const int t = index / chunks, c = index % chunks;
    cp_async_16(smem_addr(sh.region + static_cast<size_t>(t) * stride + c * 16),
                source + static_cast<size_t>(t < T ? t : 0) * pitch + begin + c * 8, t < T);
  }
  cp_async_commit();
  cp_async_wait<0>();
  worker_sync();
}

// The workers' part of a tile: the ring's next stages, which hold k in [k_begin, k_end) of the
// tile's 16 rows, times the activations staged in the shared region (rows [t][k - k_begin]).
template <int NT>
__device__ __forceinline__ void multiply_stages(const FusedModel& m, const Shared& sh, Flow& f, int k_begin, int k_end,
                                             float (&acc)[2][NT][4]) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, tq = lane & 3;
  const int act_stride = (k_end - k_begin) * 2 + kActPad;
#pragma unroll 1
  for (int k0 = k_begin; k0 < k_end; k0 += kStageK) {
    FUSED_TICK(tick0);
    const bool arrived = bounded_wait(&sh.full[f.cur.slot], f.cur.parity, sh, m.status);
    FUSED_TICK(tick1);
    FUSED_ADD(t_wait, tick0, tick1);
    const uint8_t* rows = sh.ring + static_cast<size_t>(f.cur.slot) * kStageBytes;
    const int k_warp = k0 + warp * kWarpK;
#ifdef VIPERA_FUSED_SKIP_MATH
    if (false) {
#else
    if (k_warp < k_end && arrived) {
#endif
#pragma unroll
      for (int u = 0; u < kWarpSteps; ++u) {
        if (k_warp + u * 32 >= k_end) break;
        const int local = warp * kWarpK + u * 32 + tq * 8;  // k inside the stage
        const uint8_t* at = rows + (local / kBoxK) * 2 * kBoxBytes + g * (kBoxK * 2) + (local % kBoxK) * 2;
        const uint4 lo = *reinterpret_cast<const uint4*>(at);
        const uint4 hi = *reinterpret_cast<const uint4*>(at + kBoxBytes);
#pragma unroll
        for (int n = 0; n < NT; ++n) {
          const uint4 b = *reinterpret_cast<const uint4*>(sh.region + static_cast<size_t>(n * 8 + g) * act_stride +
                                                          static_cast<size_t>(k_warp - k_begin + u * 32 + tq * 8) * 2);
          mma_bf16(acc[0][n], lo.x, hi.x, lo.y, hi.y, b.x, b.y);
          mma_bf16(acc[1][n], lo.z, hi.z, lo.w, hi.w, b.z, b.w);
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&sh.empty[f.cur.slot]);
    f.cur.advance(sh.stages);
    FUSED_TICK(tick2);
    FUSED_ADD(t_math, tick1, tick2);
#ifdef VIPERA_FUSED_TIMING
    f.n_stage += 1;
#endif
  }
}

// The workers hand a tile's partial sums (one set per warp) to the finisher.
template <int NT>
__device__ __forceinline__ void hand_over(const FusedModel& m, const Shared& sh, Flow& f, const float (&acc)[2][NT][4]) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, tq = lane & 3;
  FUSED_TICK(tick3);
  const int which = f.tiles_done & 1;
  bounded_wait(&sh.sums_empty[which], (static_cast<uint32_t>(f.tiles_done >> 1) & 1u) ^ 1u, sh, m.status);
  float* mine = sh.partial + (which * kWorkerWarps + warp) * NT * 8 * 16;
#pragma unroll
  for (int n = 0; n < NT; ++n) {
    const int t0 = n * 8 + 2 * tq;
    mine[t0 * 16 + g] = acc[0][n][0] + acc[1][n][0];
    mine[(t0 + 1) * 16 + g] = acc[0][n][1] + acc[1][n][1];
    mine[t0 * 16 + g + 8] = acc[0][n][2] + acc[1][n][2];
    mine[(t0 + 1) * 16 + g + 8] = acc[0][n][3] + acc[1][n][3];
  }
  __syncwarp();
  if (lane == 0) mbar_arrive(&sh.sums_full[which]);
  ++f.tiles_done;
  FUSED_TICK(tick4);
  FUSED_ADD(t_hand, tick3, tick4);
}

// This block's tiles of one matrix: out[t, row] = sum_k act[t, k] * W[row, k].  The workers
// multiply (each warp its share of every stage's k) and leave their partial sums in shared
// memory; the finisher adds them in warp order and calls `finish(row_lo, row_hi, t, v_lo,
// v_hi)` for every token and every pair of rows (r, r + 8) of the tile, while the workers
// are already at the next tile.  Both roles call this function with the same arguments.
// `act` null: the activations are the rows already staged in the shared region (all of K).
// Otherwise they are bfloat16 rows [T, K] in global memory, written by other blocks before
// the last barrier; the workers stage them slice by slice, as much of K as the region holds.
template <int NT, typename Finish>
__device__ __forceinline__ void run_matrix(const FusedModel& m, const Shared& sh, Flow& f, bool finisher, int N, int K,
                                           int tiles, int kind, int head_dim, const __nv_bfloat16* act, Finish finish) {
  const int lane = threadIdx.x & 31;
  const int grid = gridDim.x;
  const int T = m.T;
  int first = static_cast<int>(blockIdx.x) - f.cur.base;
  if (first < 0) first += grid;
  f.cur.base = (f.cur.base + tiles) % grid;
  constexpr int kBufferFloats = kWorkerWarps * NT * 8 * 16;

#ifdef VIPERA_FUSED_SKIP_FINISH
  if (finisher) return;
#endif
  if (finisher) {
    for (int tile = first; tile < tiles; tile += grid, ++f.tiles_done) {
      const int which = f.tiles_done & 1;
      bounded_wait(&sh.sums_full[which], static_cast<uint32_t>(f.tiles_done >> 1) & 1u, sh, m.status);
      const float* buffer = sh.partial + which * kBufferFloats;
      for (int item = lane; item < T * 8; item += 32) {
        const int t = item >> 3, r = item & 7;
        float v_lo = 0.0f, v_hi = 0.0f;
#pragma unroll
        for (int w = 0; w < kWorkerWarps; ++w) {
          const float* src = buffer + (static_cast<size_t>(w) * NT * 8 + t) * 16;
          v_lo += src[r];
          v_hi += src[r + 8];
        }
        const int row_lo = tile_row(kind, tile, r, head_dim);
        const int row_hi = tile_row(kind, tile, r + 8, head_dim);
        if (row_lo < N && !*sh.abort_flag) finish(row_lo, row_hi, t, v_lo, v_hi);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh.sums_empty[which]);
    }
    return;
  }

  // how much of K the region holds for NT * 8 rows, in whole stages
  int slice = K;
  if (act) {
    const int most = ((m.union_bytes / (NT * 8) - kActPad) / 2) / kStageK * kStageK;
    const int slices = (K + most - 1) / most;
    slice = ((K + slices - 1) / slices + kStageK - 1) / kStageK * kStageK;
  }
  for (int tile = first; tile < tiles; tile += grid) {
    float acc[2][NT][4];  // two chains of dependent MMAs instead of one
#pragma unroll
    for (int c = 0; c < 2; ++c)
#pragma unroll
      for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[c][n][i] = 0.0f;
    for (int k_begin = 0; k_begin < K; k_begin += slice) {
      const int k_end = min(K, k_begin + slice);
      if (act) {
        worker_sync();  // the slice before is read
        stage_copy<NT>(sh, act, K, k_begin, k_end - k_begin, T);
      }
      multiply_stages<NT>(m, sh, f, k_begin, k_end, acc);
    }
#ifdef VIPERA_FUSED_SKIP_FINISH
    if (acc[0][0][0] == 12345.678f) sh.partial[threadIdx.x] = acc[0][0][0] + acc[1][NT - 1][3];
    continue;
#endif
    hand_over<NT>(m, sh, f, acc);
  }
#ifdef VIPERA_FUSED_TIMING
  if (m.trace && threadIdx.x == 0) {
    long long* out = m.trace + static_cast<size_t>(gridDim.x) * (2 + 12 * m.num_layers) + (static_cast<size_t>(blockIdx.x) * 32 + (f.mark / 2) % 8) * 4;
    out[0] = f.t_wait; out[1] = f.t_math; out[2] = f.t_hand; out[3] = f.n_stage;
    f.t_wait = f.t_math = f.t_hand = f.n_stage = 0;
  }
#endif
}

// ---------------------------------------------------------------------------------------
// attention of the step's tokens over the cache (workers only)
// ---------------------------------------------------------------------------------------
// An item is (entry, 256 keys, KV head); items are numbered entry by entry, and item i
// belongs to block i mod gridDim.
struct AttentionItem {
  int entry, chunk, kv_head, position, first_visible;
};

__device__ __forceinline__ bool attention_item(const Shared& sh, int T, int kv_heads, int window, int index,
                                               AttentionItem& item) {
  int rest = index;
  for (int e = 0; e < T; ++e) {
    const int position = sh.positions[e];
    const int first_visible = window > 0 ? max(0, position - window + 1) : 0;
    const int chunk0 = first_visible / kChunkKeys;
    const int count = (position / kChunkKeys - chunk0 + 1) * kv_heads;
    if (rest < count) {
      item.entry = e;
      item.chunk = chunk0 + rest / kv_heads;
      item.kv_head = rest % kv_heads;
      item.position = position;
      item.first_visible = first_visible;
      return true;
    }
    rest -= count;
  }
  return false;
}

template <int D>
struct AttentionTiles {
  static constexpr int kSlab = 2 * kItemKeys * D * 2;  // a warp's key and value tiles, later its partial
  static_assert(16 * (D + 4) * 4 <= kSlab, "a warp's partial must fit in its slab");
  uint8_t* slabs;
  uint8_t* slab;
  uint32_t q_tile, k_tile, v_tile;
  __device__ __forceinline__ AttentionTiles(const Shared& sh, int warp) {
    slabs = sh.region + 16 * D * 2;
    slab = slabs + warp * kSlab;
    q_tile = smem_addr(sh.region);
    k_tile = smem_addr(slab);
    v_tile = k_tile + kItemKeys * D * 2;
  }
};

__device__ __forceinline__ int page_shift_of(int page_size) {
  return (page_size & (page_size - 1)) == 0 ? 31 - __clz(page_size) : -1;
}

// Before the barrier that ends the q/k/v product: the keys and values of this block's first
// item are on their way, all but the one this step writes.
template <int D>
__device__ __forceinline__ void attention_prefetch(const FusedModel& m, const FusedLayer& L, const Shared& sh) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  AttentionItem item;
  if (!attention_item(sh, m.T, L.num_kv_heads, L.window, blockIdx.x, item)) return;
  const AttentionTiles<D> tiles(sh, warp);
  const int key0 = item.chunk * kChunkKeys + warp * kItemKeys;
  const int end_early = min((item.chunk + 1) * kChunkKeys, item.position);
  if (key0 < end_early)
    load_kv_rows<D, kItemKeys, true>(tiles.k_tile, tiles.v_tile, L.k_pool, L.v_pool,
                                     L.block_table + static_cast<size_t>(item.entry) * L.table_width, L.page_size,
                                     page_shift_of(L.page_size), L.num_kv_heads, item.kv_head, key0, item.first_visible,
                                     end_early, lane);
  cp_async_commit();
}

template <int D>
__device__ void attention_phase(const FusedModel& m, const FusedLayer& L, const Shared& sh) {
  constexpr int kSlab = AttentionTiles<D>::kSlab;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int T = m.T, kv_heads = L.num_kv_heads, heads = L.num_heads;
  const int group = heads / kv_heads;
  const int page_shift = page_shift_of(L.page_size);
  const AttentionTiles<D> tiles(sh, warp);
  const float scale_log2 = L.scale * kLog2e;

  AttentionItem item;
  bool prefetched = true;
  for (int index = blockIdx.x; attention_item(sh, T, kv_heads, L.window, index, item); index += gridDim.x) {
    const int* table = L.block_table + static_cast<size_t>(item.entry) * L.table_width;
    const int position = item.position, first_visible = item.first_visible;
    const int end = min((item.chunk + 1) * kChunkKeys, position + 1);
    const int key0 = item.chunk * kChunkKeys + warp * kItemKeys;
    if (prefetched) {
      // the rows written before this step are in the tiles (or on their way); add this step's key
      const int end_early = min((item.chunk + 1) * kChunkKeys, position);
      cp_async_wait<0>();
      if (key0 < end) {
        if (key0 >= end_early)
          load_kv_rows<D, kItemKeys, true>(tiles.k_tile, tiles.v_tile, L.k_pool, L.v_pool, table, L.page_size, page_shift,
                                           kv_heads, item.kv_head, key0, first_visible, end, lane);
        else if (position < key0 + kItemKeys && position < end)
          load_kv_rows<D, kItemKeys, false>(tiles.k_tile, tiles.v_tile, L.k_pool, L.v_pool, table, L.page_size,
                                            page_shift, kv_heads, item.kv_head, key0, position, position + 1, lane);
      }
      prefetched = false;
    } else {
      worker_sync();  // the slabs of the item before are read
      if (key0 < end)
        load_kv_rows<D, kItemKeys, true>(tiles.k_tile, tiles.v_tile, L.k_pool, L.v_pool, table, L.page_size, page_shift,
                                         kv_heads, item.kv_head, key0, first_visible, end, lane);
    }
    {
      constexpr int kChunks = D / 8;
      for (int i = threadIdx.x; i < 16 * kChunks; i += kWorkerThreads) {
        const int row = i / kChunks, c = i % kChunks;
        const bool valid = row < group;
        const __nv_bfloat16* src = m.q + (static_cast<size_t>(item.entry) * heads + item.kv_head * group + (valid ? row : 0)) * D + c * 8;
        cp_async_16(tiles.q_tile + tile_offset<D>(row, c), src, valid);
      }
    }
    cp_async_commit();
    cp_async_wait<0>();
    worker_sync();

    uint32_t q_frag[D / 16][4];
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks)
      ldmatrix_x4(q_frag[ks], tiles.q_tile + tile_offset<D>(lane & 15, ks * 2 + (lane >> 4)));
    float acc[D / 8][4];
#pragma unroll
    for (int n = 0; n < D / 8; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[n][i] = 0.0f;
    float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.0f, 0.0f};
    const int row_first[2] = {first_visible, first_visible};
    const int row_limit[2] = {position, position};
    if (key0 < end)
      fold_block<D, kItemKeys>(q_frag, tiles.k_tile, tiles.v_tile, key0, row_first, row_limit, scale_log2, row_max,
                               row_sum, acc);
    __syncwarp();

    // the warp's partial over its tiles: [16 rows][D + 4] floats
    float* mine = reinterpret_cast<float*>(tiles.slab);
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
    worker_sync();
    // merge the eight warps' partials: thread = (row, sixteenth of the columns)
    constexpr int kCols = D / 16;
    const int row = threadIdx.x >> 4, part = threadIdx.x & 15;
    if (row < group) {
      float mx[kWorkerWarps], best = -INFINITY;
#pragma unroll
      for (int w = 0; w < kWorkerWarps; ++w) {
        mx[w] = reinterpret_cast<const float*>(tiles.slabs + w * kSlab)[row * (D + 4) + D];
        best = fmaxf(best, mx[w]);
      }
      float weight[kWorkerWarps], sum = 0.0f;
#pragma unroll
      for (int w = 0; w < kWorkerWarps; ++w) {
        weight[w] = mx[w] == -INFINITY ? 0.0f : exp2f(mx[w] - best);
        sum += weight[w] * reinterpret_cast<const float*>(tiles.slabs + w * kSlab)[row * (D + 4) + D + 1];
      }
      const int head = item.kv_head * group + row;
      const size_t at = (static_cast<size_t>(item.entry) * heads + head) * m.max_chunks + item.chunk;
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
        for (int w = 0; w < kWorkerWarps; ++w) {
          const float4 v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(tiles.slabs + w * kSlab) + row * (D + 4) + col);
          value.x += weight[w] * v.x;
          value.y += weight[w] * v.y;
          value.z += weight[w] * v.z;
          value.w += weight[w] * v.w;
        }
        __stcg(reinterpret_cast<float4*>(dst + col), value);
      }
    }
  }
  cp_async_wait<0>();  // a block without items still has its (empty) prefetch group
}

// The partials of every (entry, head) row become the row's attention output:
// m = max m_c, l = sum l_c e^(m_c - m), out = sum o_c e^(m_c - m) / l, chunks in key order.
// Row i belongs to block i mod gridDim.
template <int D>
__device__ void combine_phase(const FusedModel& m, const FusedLayer& L, const Shared& sh) {
  constexpr int kGroups = D / 4;                       // columns in groups of four
  constexpr int kSlices = kWorkerThreads / kGroups;    // threads that share a group, each taking every kSlices-th chunk
  const int heads = L.num_heads;
  const int group = threadIdx.x % kGroups, slice = threadIdx.x / kGroups;
  float* ml = reinterpret_cast<float*>(sh.region);                                    // [chunks][2]
  float4* sums = reinterpret_cast<float4*>(sh.region + kMaxChunks * 8);               // [kSlices][kGroups]
  float* totals = reinterpret_cast<float*>(sh.region + kMaxChunks * 8 + kSlices * kGroups * 16);  // [kSlices]
  for (int row = blockIdx.x; row < m.T * heads; row += gridDim.x) {
    const int entry = row / heads;
    const int position = sh.positions[entry];
    const int first_visible = L.window > 0 ? max(0, position - L.window + 1) : 0;
    const int chunk0 = first_visible / kChunkKeys;
    const int chunks = position / kChunkKeys - chunk0 + 1;
    const size_t base = static_cast<size_t>(row) * m.max_chunks + chunk0;
    worker_sync();  // the row before is finished with the shared buffers
    for (int c = threadIdx.x; c < chunks; c += kWorkerThreads) {
      const float2 pair = __ldcg(reinterpret_cast<const float2*>(m.partial_ml + 2 * (base + c)));
      ml[2 * c] = pair.x;
      ml[2 * c + 1] = pair.y;
    }
    worker_sync();
    float best = -INFINITY;
    for (int c = 0; c < chunks; ++c) best = fmaxf(best, ml[2 * c]);
    float4 value = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    float total = 0.0f;
    for (int c = slice; c < chunks; c += kSlices) {
      const float w = ml[2 * c] == -INFINITY ? 0.0f : exp2f(ml[2 * c] - best);
      const float4 v = __ldcg(reinterpret_cast<const float4*>(m.partial_out + (base + c) * D + group * 4));
      total += w * ml[2 * c + 1];
      value.x += w * v.x;
      value.y += w * v.y;
      value.z += w * v.z;
      value.w += w * v.w;
    }
    sums[slice * kGroups + group] = value;
    if (group == 0) totals[slice] = total;
    worker_sync();
    if (threadIdx.x < kGroups) {
      float4 out = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      float sum = 0.0f;
#pragma unroll
      for (int s = 0; s < kSlices; ++s) {
        const float4 v = sums[s * kGroups + group];
        out.x += v.x;
        out.y += v.y;
        out.z += v.z;
        out.w += v.w;
        sum += totals[s];
      }
      const float inverse = 1.0f / sum;
      __nv_bfloat16* dst = m.attn + static_cast<size_t>(row) * D + group * 4;
      *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(out.x * inverse, out.y * inverse);
      *reinterpret_cast<__nv_bfloat162*>(dst + 2) = __floats2bfloat162_rn(out.z * inverse, out.w * inverse);
    }
  }
}

// ---------------------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------------------
template <int NT, int D>
__device__ void step(const FusedModel& m, const Shared& sh, const bool finisher) {
  Flow f;
  const int T = m.T, H = m.hidden;
  // embedding rows into the 32-bit residual stream
  if (!finisher) {
    const int chunks = H >> 3;
    for (int index = blockIdx.x * kWorkerThreads + threadIdx.x; index < T * chunks; index += gridDim.x * kWorkerThreads) {
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
  trace_mark(m, f);
  grid_barrier(m, sh, f);
  trace_mark(m, f);

  auto add_to_residual = [&](int row_lo, int row_hi, int t, float v_lo, float v_hi) {
    float* at = m.x + static_cast<size_t>(t) * H;
    __stcg(at + row_lo, __ldcg(at + row_lo) + v_lo);
    if (row_hi < H) __stcg(at + row_hi, __ldcg(at + row_hi) + v_hi);
  };

  for (int l = 0; l < m.num_layers; ++l) {
    const FusedLayer& L = m.layers[l];
    const int heads = L.num_heads, kv_heads = L.num_kv_heads;
    const int q_dim = heads * D, inter = L.inter;
    const int qkv_rows = (heads + 2 * kv_heads) * D;
    const int qkv_tiles = (heads + (L.writes_cache ? 2 * kv_heads : 0)) * (D / 16);

    // ---- norm, q/k/v product, bias, rotation, cache write ----
    if (!finisher && owns_tile(f, qkv_tiles)) stage_normed<NT>(sh, m.x, L.norm1, L.eps1, T, H);
    run_matrix<NT>(m, sh, f, finisher, qkv_rows, H, qkv_tiles, TILE_QKV, D, nullptr,
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
    trace_mark(m, f);
    // between announcing itself and waiting for the other blocks, the block starts loading the
    // keys and values of its first attention item (the staged activations are read by then)
    grid_arrive(m, sh, f);
    if (!finisher) attention_prefetch<D>(m, L, sh);
    grid_wait(m, sh, f);
    trace_mark(m, f);

    // ---- attention: partials per 256 keys, then one output row per (entry, head) ----
    if (!finisher) attention_phase<D>(m, L, sh);
    trace_mark(m, f);
    grid_barrier(m, sh, f);
    trace_mark(m, f);
    if (!finisher) combine_phase<D>(m, L, sh);
    trace_mark(m, f);
    grid_barrier(m, sh, f);
    trace_mark(m, f);

    // ---- output product into the residual stream ----
    run_matrix<NT>(m, sh, f, finisher, H, q_dim, (H + 15) / 16, TILE_PLAIN, D, m.attn, add_to_residual);
    trace_mark(m, f);
    grid_barrier(m, sh, f);
    trace_mark(m, f);

    // ---- norm, gate and up products, activation ----
    if (!finisher && owns_tile(f, inter / 8)) stage_normed<NT>(sh, m.x, L.norm2, L.eps2, T, H);
    run_matrix<NT>(m, sh, f, finisher, 2 * inter, H, inter / 8, TILE_GATE_UP, D, nullptr,
        [&](int row_lo, int row_hi, int t, float v_lo, float v_hi) {
          const int feature = (row_lo >> 5) * 16 + (row_lo & 15);
          const float value = v_hi * (v_lo / (1.0f + __expf(-v_lo)));
          m.act[static_cast<size_t>(t) * inter + feature] = __float2bfloat16_rn(value);
        });
    trace_mark(m, f);
    grid_barrier(m, sh, f);
    trace_mark(m, f);

    // ---- down product into the residual stream ----
    run_matrix<NT>(m, sh, f, finisher, H, inter, (H + 15) / 16, TILE_PLAIN, D, m.act, add_to_residual);
    trace_mark(m, f);
    grid_barrier(m, sh, f);
    trace_mark(m, f);
  }

  // ---- final norm and the output matrix ----
  const int V = m.vocab;
  if (!finisher) stage_normed<NT>(sh, m.x, m.final_norm, m.final_eps, T, H);
  run_matrix<NT>(m, sh, f, finisher, V, H, (V + 15) / 16, TILE_PLAIN, D, nullptr,
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
  uint8_t* tail = reinterpret_cast<uint8_t*>(sh.partial) + 2 * kWorkerWarps * NT * 8 * 16 * sizeof(float);
  sh.full = reinterpret_cast<uint64_t*>(tail);
  sh.empty = sh.full + kMaxStages;
  sh.sums_full = sh.empty + kMaxStages;
  sh.sums_empty = sh.sums_full + 2;
  sh.positions = reinterpret_cast<int*>(sh.sums_empty + 2);
  sh.abort_flag = sh.positions + kMaxTokens;
  if (threadIdx.x == 0) {
    for (int s = 0; s < sh.stages; ++s) {
      mbar_init(&sh.full[s], 1);
      mbar_init(&sh.empty[s], kWorkerWarps);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sh.sums_full[b], kWorkerWarps);
      mbar_init(&sh.sums_empty[b], 1);
    }
    *sh.abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (threadIdx.x < kMaxTokens) sh.positions[threadIdx.x] = threadIdx.x < m.T ? m.positions[threadIdx.x] : 0;
  __syncthreads();
  const int warp = threadIdx.x >> 5;
  if (warp == kProducerWarp) {
    producer<D>(m, sh);
  } else {
    step<NT, D>(m, sh, warp == kFinisherWarp);
  }
  // A block that gave up waiting lets the copies it still has in flight land before it leaves.
  if (*sh.abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
}

constexpr int kSharedLimit = 227 * 1024;

struct SharedPlan {
  int stages, union_bytes, total;
};

SharedPlan plan_shared(int tokens, int hidden, int head_dim) {
  const int nt = tokens <= 8 ? 1 : 2;
  const int activations = nt * 8 * (hidden * 2 + kActPad);
  const int attention = 16 * head_dim * 2 + kWorkerWarps * 2 * kItemKeys * head_dim * 2;
  const int combine = kMaxChunks * 8 + kWorkerThreads * 16 + 64 * 4;
  SharedPlan plan{};
  int most = activations > attention ? activations : attention;
  if (combine > most) most = combine;
  plan.union_bytes = (most + 127) / 128 * 128;
  const int fixed = plan.union_bytes + 2 * kWorkerWarps * nt * 8 * 16 * 4 + (2 * kMaxStages + 4) * 8 + (kMaxTokens + 2) * 4 + 128 +
                    1024 /* the ring starts on a multiple of 1024 bytes */;
  plan.stages = (kSharedLimit - fixed) / kStageBytes;
  if (plan.stages > kMaxStages) plan.stages = kMaxStages;
  if (const char* most_stages = std::getenv("VIPERA_FUSED_MAX_STAGES")) {  // for experiments with the ring's depth
    const int limit = std::atoi(most_stages);
    if (limit >= 2 && limit < plan.stages) plan.stages = limit;
  }
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
  if (resident < 1) {
    cudaFuncAttributes attributes;
    cudaFuncGetAttributes(&attributes, decode_fused_kernel<NT, D>);
    fprintf(stderr, "decode_fused: no block fits an SM (%d threads, %d registers each, %d + %zu bytes of shared memory)\n",
            kFusedThreads, attributes.numRegs, shared_bytes, attributes.sharedSizeBytes);
    return VIPERA_BAD_SHAPE;
  }
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
VIPERA_API int vipera_decode_fused_max_chunks() { return kMaxChunks; }

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
  if (m.T > kMaxTokens || m.num_layers < 0 || m.hidden % 64 || m.max_chunks <= 0 || m.max_chunks > kMaxChunks) return VIPERA_BAD_SHAPE;
  if (!m.layers || !m.maps || !m.tokens || !m.positions || !m.embedding || !m.x || !m.q || !m.attn || !m.act || !m.partial_ml ||
      !m.partial_out || !m.final_norm || !m.head || !m.logits || !m.barrier || !m.status)
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
