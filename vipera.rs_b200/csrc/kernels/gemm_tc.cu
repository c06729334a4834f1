// bfloat16 matrix products on the fifth-generation tensor cores: out[T, N] = A[T, K] . W[N, K]^T
// with 32-bit accumulation in tensor memory, operands brought to shared memory by TMA.
//
// One persistent kernel serves prefill and decode.  Both operands are K-major, so either
// may sit on the 128-row side of the tcgen05 instruction:
//   * many tokens (T >= 128): tokens on the 128-row side, 256 (or 128) weight rows on the
//     other side;
//   * few tokens (decode, short portions): weight rows on the 128-row side and the tokens,
//     padded to 16/32/64/128, on the other side.  Each weight byte is read from HBM once and
//     the K range is cut into splits so that every SM streams a share of the weights; a
//     second small kernel adds the splits' partial sums in a fixed order and writes the ending.
// The reference multiplies every weight matrix by all rows of the batch in one pass over the
// weights (crates/vipera-backend-cpu/src/model.rs:1005-1025, 1154-1198) and has a device
// kernel that shares one weight read between up to 8 activation sets
// (crates/vipera-backend-gpu/src/q4k_matvec_q8_batch.cu:40-116); this kernel is that idea on
// tcgen05.
//
// Roles inside a block: warps 0-3 read accumulators from tensor memory and write the ending; one
// thread of warp 4 issues TMA loads (wide tiles: one thread of warp 6 too, the two taking turns at
// the k-blocks); warp 5 issues tcgen05.mma through an elected lane.  Two accumulators alternate,
// so that the ending of one tile overlaps the products of the next.  What bounds the loop over K
// is instruction latency in these single threads, not bytes: a wait on a barrier and an arrival
// cost about 100 clocks each, a TMA instruction 60 to 90, and a k-block of a 128 x 256 tile is
// only 512 clocks of tensor-core work.  Hence the second loading warp, the look ahead at the next
// stage's barrier while this stage's products are issued, and the uniform operands.
//
// Pairs (many tokens): two blocks of a cluster share tiles of 256 tokens (cta_group::2).  Each
// loads its own 128 tokens and half of the tile's weight rows; the first block's warp issues
// products that read both blocks' shared memory and write both blocks' tensor memory; each block
// writes the ending of its own 128 tokens.  A third fewer bytes per flop pass through each SM's
// shared memory, and six stages fit where four did.  Every wait on an mbarrier is bounded: when it runs out the block
// records an error code, stops waiting anywhere, drains and frees its tensor memory, and
// the launcher's caller finds the code in the status word.
//
// Even shares (tokens on the 128-row side, endings through TMA): where whole tiles would leave
// SMs idle in the last wave, the run of all k-blocks of all tiles is cut into one equal share
// per block instead.  A block whose share starts inside a tile writes that tile's partial sums
// to a slot of its own and raises a flag; the block whose share holds the tile's first k-block
// adds the partial sums of the blocks behind it, in their order, before the ending.  A tile's
// later parts are the first work of their blocks and its first part is the last work of its
// block, so the flags are long up when they are looked at; the wait is bounded all the same.
//
// Endings (as in gemm_simt.cu): STORE (+bias) as float32 or bfloat16, RESIDUAL (add into
// the 32-bit residual stream), SWIGLU over gate and up rows interleaved in groups of 16.
#include <cuda.h>

#include <algorithm>
#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"

enum GemmEpilogue { EPI_STORE = 0, EPI_RESIDUAL = 1, EPI_SWIGLU = 2, EPI_ROPE_CACHE = 4 };
enum { GEMM_ROPE_NONE = 0, GEMM_ROPE_NEOX = 1 };
enum { GEMM_TC_WAIT_EXPIRED = 1 };

constexpr int kBlockK = 64;        // bf16 elements per k-block: one 128-byte swizzle row
constexpr int kTileX = 128;        // rows on the 128-row side of the instruction
constexpr int kThreads = 192;
// Wide tiles have a second loading warp: the two take turns at the k-blocks.  Waiting for a
// stage, announcing its bytes and handing two boxes to TMA are some 600 clocks of instruction
// latency in one thread, more than the 512 the tensor core needs for the stage.
constexpr int kThreadsWide = 224;
template <int BN> constexpr int threads_for() { return BN >= 128 ? kThreadsWide : kThreads; }
constexpr uint32_t kWaitLimit = 1u << 22;

struct GemmParams {
  int tokens;        // T
  int features;      // N (for SWIGLU: interleaved gate+up rows)
  int num_k_blocks;
  int tiles_x, tiles_y, splits, k_blocks_per_split;
  int epilogue;
  int out_dtype;
  const float* bias;
  void* out;
  float* resid;
  int tma_ending;    // 1: the ending goes through shared memory and TMA stores (map_out)
  float* scratch;    // split partials: [item][BN][128] floats; even shares: [block][BN][128]
  int* status;       // device word: 0, or an error code
  int even_shares;   // 1: every block takes an equal share of all k-blocks of all tiles
  int* share_flags;  // even shares: [blocks], 0 between launches
  // EPI_ROPE_CACHE: the columns are the q, k and v heads of a step's tokens; the ending adds the
  // bias, turns the rotary pairs of q and k, and writes q to q_out and k and v into their pages
  int num_heads, num_kv_heads, head_dim, rope_style, write_cache;
  const int* positions;      // [T]
  const int* token_entry;    // [T] row of the block table
  const int* block_table;    // [entries, table_width]
  int table_width, page_size;
  const float* cos_table;    // [positions, d / 2]
  const float* sin_table;
  __nv_bfloat16* q_out;      // [T, heads * d]
  __nv_bfloat16* k_pool;     // [pages, page_size, kv_heads, d]
  __nv_bfloat16* v_pool;
};

// ---------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return done != 0;
}
// whether the phase has completed, without waiting
__device__ __forceinline__ uint32_t mbar_peek(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return done;
}
// Bounded wait.  When the limit runs out, or another thread's wait already did, the caller
// goes on as if the barrier had completed: every role then runs to its end without waiting,
// so the block drains; what it writes is marked invalid by the status word.
__device__ __forceinline__ void mbar_wait_limited(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status,
                                                  uint32_t limit) {
  for (uint32_t spin = 0; spin < limit; ++spin) {
    if (mbar_try_wait(bar, parity)) return;
    if ((spin & 1023u) == 1023u && *abort_flag) return;
  }
  *abort_flag = 1;
  atomicExch(status, GEMM_TC_WAIT_EXPIRED);
}
__device__ __forceinline__ void mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status) {
  mbar_wait_limited(bar, parity, abort_flag, status, kWaitLimit);
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(src)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, const void* src, int c0, int c1) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(src)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// Issued by a whole warp that walks the loop together: every lane holds the same operands (so they
// can live in the warp's uniform registers, which is where the instruction wants them) and one
// elected lane issues.  A single lane in a diverged branch pays for moving each operand there:
// about 77 clocks an instruction, measured, against 35 this way and 96 that the instruction runs.
__device__ __forceinline__ void tcgen05_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tcgen05_mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tcgen05_commit_elect(uint64_t* bar) {
  asm volatile(
      "{\n .reg .pred leader;\n elect.sync _|leader, 0xffffffff;\n"
      " @leader tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n}\n"
      ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tcgen05_mma_bf16_elect(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p, leader;\n elect.sync _|leader, 0xffffffff;\n setp.ne.b32 p, %4, 0;\n"
      " @leader tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// ---- the forms for a pair of blocks (a cluster of two, cta_group::2) ----
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  return rank;
}
// the address, in the cluster's window, of the same shared-memory location in the block of `rank`
__device__ __forceinline__ uint32_t in_block(uint32_t saddr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(saddr), "r"(rank));
  return out;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// a load into this block's shared memory whose bytes count on a barrier of the pair's first block
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tcgen05_commit_pair(uint32_t bar_cluster_addr) {
  asm volatile(
      "{\n .reg .pred leader;\n elect.sync _|leader, 0xffffffff;\n"
      " @leader tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];\n}\n"
      ::"r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void tcgen05_mma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p, leader;\n elect.sync _|leader, 0xffffffff;\n setp.ne.b32 p, %4, 0;\n"
      " @leader tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_load_32(uint32_t taddr, float* v) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_load_32_nowait(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_load_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_load_16(uint32_t taddr, float* v) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor of a K-major tile with 128-byte swizzle: rows of 128
// bytes, 8-row groups 1024 bytes apart (stride byte offset), descriptor version 1.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {
  uint64_t desc = 0;
  desc |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);  // start address
  desc |= static_cast<uint64_t>(1) << 16;                  // leading byte offset (unused with swizzle)
  desc |= static_cast<uint64_t>(1024 >> 4) << 32;          // stride byte offset
  desc |= static_cast<uint64_t>(1) << 46;                  // version
  desc |= static_cast<uint64_t>(2) << 61;                  // SWIZZLE_128B
  return desc;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// up * silu(gate); the quotient with the hardware's reciprocal (the result is rounded to
// bfloat16 by every caller on the tensor-core path, which hides the last bits)
__device__ __forceinline__ float silu_mul(float gate, float up) { return up * __fdividef(gate, 1.0f + __expf(-gate)); }

#ifndef VIPERA_SMALL_BUDGET
#define VIPERA_SMALL_BUDGET 100
#endif
// PAIR: two blocks of a cluster work on one tile of 256 rows (cta_group::2); each holds its own
// 128 rows of the one operand and half of the BN rows of the other.
template <int BN, bool PAIR = false>
struct TileConfig {
  static constexpr int kRowsY = PAIR ? BN / 2 : BN;   // rows of the second operand in this block's stage
  static constexpr int kStageBytes = (kTileX + kRowsY) * kBlockK * 2;
  // Wide tiles take all the shared memory of an SM; narrow ones (few tokens) take less
  // than half, so that two blocks share an SM and the next product's block can set up and
  // prefetch weights while this one finishes.
  static constexpr int kStagingBytes = BN >= 128 ? 4 * 2 * 4096 : 0;  // 2 buffers of 32 rows x 128 B per epilogue warp
  static constexpr int kBudget = BN >= 128 ? 193 * 1024 : VIPERA_SMALL_BUDGET * 1024;   // for the stages
  static constexpr int kStages = kBudget / kStageBytes;
  // two accumulators; tensor memory is handed out in powers of two of at least 32 columns
  static constexpr int kTmemCols = 2 * BN <= 32 ? 32 : 2 * BN <= 64 ? 64 : 2 * BN <= 128 ? 128 : 2 * BN <= 256 ? 256 : 512;
  static constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + 1024 /*alignment*/ + 256 /*barriers*/;
  static_assert(kSmemBytes <= 227 * 1024, "more shared memory than a block can have");
};

// ---------------------------------------------------------------------------------------
// the ending of one tile, by the four epilogue warps
// ---------------------------------------------------------------------------------------
// SWAP = false: accumulator rows are tokens, columns are features.
// SWAP = true : accumulator rows are features, columns are tokens.
template <int BN, bool SWAP>
__device__ __forceinline__ void finish_chunk(const GemmParams& p, const float* v, int width, int row, int col0) {
  // `row`: global index on the 128-row side; `col0`: global index of v[0] on the other side.
  const int N = p.features;
  if (!SWAP) {
    const int t = row;
    if (t >= p.tokens) return;
    if (p.epilogue == EPI_SWIGLU) {
      // columns [col0, col0+16) are gate, [col0+16, col0+32) up, of features col0/2 ..
      const int inter = N >> 1;
      const int f0 = col0 >> 1;
      __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.out) + static_cast<size_t>(t) * inter + f0;
      float* dst32 = static_cast<float*>(p.out) + static_cast<size_t>(t) * inter + f0;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        if (col0 + 16 + i >= N) break;
        const float value = silu_mul(v[i], v[16 + i]);
        if (p.out_dtype == VIPERA_BF16) dst[i] = __float2bfloat16_rn(value); else dst32[i] = value;
      }
      return;
    }
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      if (i >= width) break;
      const int n = col0 + i;
      if (n >= N) break;
      const size_t at = static_cast<size_t>(t) * N + n;
      if (p.epilogue == EPI_RESIDUAL) {
        p.resid[at] += v[i];
      } else {
        const float value = v[i] + (p.bias ? p.bias[n] : 0.0f);
        if (p.out_dtype == VIPERA_BF16) static_cast<__nv_bfloat16*>(p.out)[at] = __float2bfloat16_rn(value);
        else static_cast<float*>(p.out)[at] = value;
      }
    }
  } else {
    const int n = row;
    const int lane = threadIdx.x & 31;
    if (p.epilogue == EPI_SWIGLU) {
      // lanes 0-15 of a warp hold gate rows, lanes 16-31 the up rows of the same features
      const int inter = N >> 1;
      const int f = ((n - lane) >> 1) + (lane & 15);
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        if (i >= width) break;
        const float other = __shfl_xor_sync(0xffffffffu, v[i], 16);
        const int t = col0 + i;
        if (lane < 16 && t < p.tokens && n + 16 < N) {
          const float value = silu_mul(v[i], other);
          const size_t at = static_cast<size_t>(t) * inter + f;
          if (p.out_dtype == VIPERA_BF16) static_cast<__nv_bfloat16*>(p.out)[at] = __float2bfloat16_rn(value);
          else static_cast<float*>(p.out)[at] = value;
        }
      }
      return;
    }
    if (n >= N) return;
    const float bias = (p.epilogue == EPI_STORE && p.bias) ? p.bias[n] : 0.0f;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      if (i >= width) break;
      const int t = col0 + i;
      if (t >= p.tokens) break;
      const size_t at = static_cast<size_t>(t) * N + n;
      if (p.epilogue == EPI_RESIDUAL) {
        p.resid[at] += v[i];
      } else {
        const float value = v[i] + bias;
        if (p.out_dtype == VIPERA_BF16) static_cast<__nv_bfloat16*>(p.out)[at] = __float2bfloat16_rn(value);
        else static_cast<float*>(p.out)[at] = value;
      }
    }
  }
}

// The work of one block, piece by piece: whole tiles or splits of tiles dealt round robin, or
// (even shares) the pieces of its run of k-blocks.  All three roles of a block walk it alike.
constexpr int kShareSnap = 2;   // a share boundary this close to a tile's edge moves onto it
__device__ __forceinline__ long share_begin(const GemmParams& p, int block, int blocks) {
  const long all = static_cast<long>(p.tiles_x) * p.tiles_y * p.num_k_blocks;
  if (block >= blocks) return all;
  long at = all * block / blocks;
  const int inside = static_cast<int>(at % p.num_k_blocks);
  if (inside <= kShareSnap) at -= inside;
  else if (p.num_k_blocks - inside <= kShareSnap) at += p.num_k_blocks - inside;
  return at;
}
struct Piece {
  int tile, kb_begin, kb_end;
  int slot;      // where a partial sum of this piece goes in the scratch
};
// EVEN: whether this form of the kernel can be given even shares at all (the others keep the
// code out: the few-token forms are bound by the latency of their first instructions)
template <bool EVEN>
struct WorkLoop {
  const GemmParams& p;
  int item;
  long at, end;
  int stride;
  // `pair`: the two blocks of a cluster walk the same tiles
  __device__ __forceinline__ explicit WorkLoop(const GemmParams& params, bool pair = false)
      : p(params), item(pair ? blockIdx.x >> 1 : blockIdx.x), at(0), end(0), stride(pair ? gridDim.x >> 1 : gridDim.x) {
    if (EVEN && p.even_shares) {
      at = share_begin(p, blockIdx.x, gridDim.x);
      end = share_begin(p, blockIdx.x + 1, gridDim.x);
    }
  }
  __device__ __forceinline__ bool next(Piece& piece) {
    if (EVEN && p.even_shares) {
      if (at >= end) return false;
      piece.tile = static_cast<int>(at / p.num_k_blocks);
      piece.kb_begin = static_cast<int>(at % p.num_k_blocks);
      const long left = end - at;
      piece.kb_end = left < p.num_k_blocks - piece.kb_begin ? piece.kb_begin + static_cast<int>(left) : p.num_k_blocks;
      piece.slot = blockIdx.x;
      at += piece.kb_end - piece.kb_begin;
      return true;
    }
    if (item >= p.tiles_x * p.tiles_y * p.splits) return false;
    const int split = item % p.splits;
    piece.tile = item / p.splits;
    piece.kb_begin = split * p.k_blocks_per_split;
    piece.kb_end = min(p.num_k_blocks, piece.kb_begin + p.k_blocks_per_split);
    piece.slot = item;
    item += stride;
    return true;
  }
};

template <int BN, bool SWAP, bool PAIR = false, bool EVEN = false>
__global__ void __launch_bounds__(threads_for<BN>(), (BN >= 128 || VIPERA_SMALL_BUDGET > 110 ? 1 : 2))
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_y,
               const __grid_constant__ CUtensorMap map_out, const GemmParams p) {
  static_assert(!PAIR || (!SWAP && BN >= 128), "pairs of blocks: tokens on the 128-row side, wide tiles");
  using Config = TileConfig<BN, PAIR>;
  constexpr int kStages = Config::kStages;
  // a pair's instruction covers 256 rows: 128 in each block's tensor memory
  constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(BN >> 3) << 17) |
                              (static_cast<uint32_t>((PAIR ? 2 * kTileX : kTileX) >> 4) << 24);
  const uint32_t rank = PAIR ? cluster_rank() : 0u;   // 0: the block that issues the pair's products
  constexpr bool kWide = BN >= 128;                   // the forms for many tokens
  constexpr bool kEven = EVEN;                        // the form that runs with even shares, an instance of its own
  static_assert(!EVEN || (!SWAP && BN >= 128 && !PAIR), "even shares: tokens on the 128-row side, wide tiles, blocks alone");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* tiles = smem;
  uint8_t* staging = smem + kStages * Config::kStageBytes;  // 1024-byte aligned: stage sizes are multiples of 1024
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + Config::kStagingBytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + kStages;
  uint64_t* acc_full = bars + 2 * kStages;
  uint64_t* acc_empty = bars + 2 * kStages + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    // a pair's accumulator is free when the epilogue warps of both blocks have read their halves
    for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], PAIR ? 8 : 4); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    if (PAIR) {
      // the same warp of both blocks: the columns are handed out in both blocks' tensor memory
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(Config::kTmemCols));
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(Config::kTmemCols));
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
  }
  tcgen05_fence_before();
  if (PAIR) cluster_sync_all();   // the other block's barriers exist before anything arrives at them
  else __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = __shfl_sync(0xffffffffu, *tmem_slot, 0);   // the same in every lane, and known to be

  constexpr int kProducers = BN >= 128 ? 2 : 1;   // (narrow tiles: a second loading warp was measured and changes nothing)
  if (warp == 4 || (kProducers == 2 && warp == 6)) {
    // ---------------- TMA producers: warp 4, and warp 6 for every other k-block of wide tiles ----------------
    const int mine = warp == 4 ? 0 : 1;
    if (lane == 0) {
      // The weight operand depends on no earlier kernel: its tiles for the first stages are
      // on their way before this kernel waits for the kernels ahead of it.
      // A pair: both blocks load their own rows into their own shared memory; all four loads of
      // a stage count on the first block's barrier, which expects the bytes of both blocks.
      int prefetched = 0;
      const uint32_t pair_full = PAIR ? in_block(smem_u32(&full[0]), 0) : 0u;   // + 8 * stage
      const int y_row = PAIR ? static_cast<int>(rank) * (BN / 2) : 0;           // this block's rows inside the tile's BN
      Piece first;
      if (WorkLoop<kEven>(p, PAIR).next(first)) {
        const int tx = PAIR ? 2 * (first.tile % p.tiles_x) + static_cast<int>(rank) : first.tile % p.tiles_x;
        const int ty = first.tile / p.tiles_x;
        const int kb_begin = first.kb_begin;
        prefetched = min(kStages, first.kb_end - first.kb_begin);
        for (int i = 0; i < prefetched; ++i) {
          if (i % kProducers != mine) continue;
          uint8_t* x_tile = tiles + i * Config::kStageBytes;
          uint8_t* y_tile = x_tile + kTileX * kBlockK * 2;
          if (PAIR) {
            if (rank == 0) mbar_expect_tx(&full[i], 2 * Config::kStageBytes);
            tma_load_2d_pair(y_tile, &map_y, pair_full + 8 * i, (kb_begin + i) * kBlockK, ty * BN + y_row);
            continue;
          }
          mbar_expect_tx(&full[i], Config::kStageBytes);
          if (SWAP) tma_load_2d(x_tile, &map_x, &full[i], (kb_begin + i) * kBlockK, tx * kTileX);
          else tma_load_2d(y_tile, &map_y, &full[i], (kb_begin + i) * kBlockK, ty * BN);
        }
      }
      pdl_wait();
      int stage = 0, issued = 0;
      uint32_t phase = 0;
      WorkLoop<kEven> work(p, PAIR);
      Piece piece;
      while (work.next(piece)) {
        const int tx = PAIR ? 2 * (piece.tile % p.tiles_x) + static_cast<int>(rank) : piece.tile % p.tiles_x;
        const int ty = piece.tile / p.tiles_x;
        for (int kb = piece.kb_begin; kb < piece.kb_end; ++kb, ++issued) {
          if (issued % kProducers != mine) {
            if (++stage == kStages) { stage = 0; phase ^= 1u; }
            continue;
          }
          uint8_t* x_tile = tiles + stage * Config::kStageBytes;
          uint8_t* y_tile = x_tile + kTileX * kBlockK * 2;
          if (PAIR) {
            if (issued < prefetched) {
              tma_load_2d_pair(x_tile, &map_x, pair_full + 8 * stage, kb * kBlockK, tx * kTileX);
            } else {
              mbar_wait(&empty[stage], phase ^ 1u, abort_flag, p.status);
              if (rank == 0) mbar_expect_tx(&full[stage], 2 * Config::kStageBytes);
              tma_load_2d_pair(x_tile, &map_x, pair_full + 8 * stage, kb * kBlockK, tx * kTileX);
              tma_load_2d_pair(y_tile, &map_y, pair_full + 8 * stage, kb * kBlockK, ty * BN + y_row);
            }
          } else if (issued < prefetched) {
            // the weight half of this stage is already in flight: add the activation half
            if (SWAP) tma_load_2d(y_tile, &map_y, &full[stage], kb * kBlockK, ty * BN);
            else tma_load_2d(x_tile, &map_x, &full[stage], kb * kBlockK, tx * kTileX);
          } else {
            mbar_wait(&empty[stage], phase ^ 1u, abort_flag, p.status);
            mbar_expect_tx(&full[stage], Config::kStageBytes);
            tma_load_2d(x_tile, &map_x, &full[stage], kb * kBlockK, tx * kTileX);
            tma_load_2d(y_tile, &map_y, &full[stage], kb * kBlockK, ty * BN);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 5) {
    // ---------------- MMA issuer ----------------
    // Wide tiles: the whole warp walks the loop (see tcgen05_mma_bf16_elect); of a pair, the first
    // block's warp issues for both.  Narrow tiles (few tokens) wait for their weights, not for the
    // issue, and keep the shortest code: one lane.
    if (rank == 0 && (kWide || lane == 0)) {
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool arrived = false;
      uint32_t arrived_next = 0;
      const uint32_t other_empty = PAIR ? in_block(smem_u32(&empty[0]), 1) : 0u;
      const uint32_t other_acc_full = PAIR ? in_block(smem_u32(&acc_full[0]), 1) : 0u;
      WorkLoop<kEven> work(p, PAIR);
      Piece piece;
      for (; work.next(piece); ++local) {
        const int kb_begin = piece.kb_begin, kb_end = piece.kb_end;
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1u;
        if (kWide) {
          if (lane == 0) mbar_wait(&acc_empty[acc], acc_phase ^ 1u, abort_flag, p.status);
          __syncwarp();
        } else {
          mbar_wait(&acc_empty[acc], acc_phase ^ 1u, abort_flag, p.status);
        }
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          // `arrived`: the look ahead of the k-block before already saw this stage full
          if (kWide) {
            if (!arrived && lane == 0) mbar_wait(&full[stage], phase, abort_flag, p.status);   // one lane polls, the warp follows
            __syncwarp();
          } else {
            mbar_wait(&full[stage], phase, abort_flag, p.status);
          }
          if (kWide) {
            // a look at the next stage, asked now and read after this stage's products are issued:
            // the barrier's answer takes about 100 clocks, which the issue then hides
            const int next = stage + 1 == kStages ? 0 : stage + 1;
            arrived_next = mbar_peek(&full[next], next == 0 ? phase ^ 1u : phase);
          }
          tcgen05_fence_after();
          const uint32_t x_addr = smem_u32(tiles + stage * Config::kStageBytes);
          const uint32_t y_addr = x_addr + kTileX * kBlockK * 2;
          const uint64_t x_desc = smem_desc_sw128(x_addr);
          const uint64_t y_desc = smem_desc_sw128(y_addr);
#pragma unroll
          for (int k = 0; k < kBlockK / 16; ++k) {
            // 16 bf16 = 32 bytes further along K inside the swizzled row: +2 in the address field
            if (PAIR)
              tcgen05_mma_bf16_pair(d_tmem, x_desc + static_cast<uint64_t>(2 * k), y_desc + static_cast<uint64_t>(2 * k),
                                    kIdesc, (kb > kb_begin || k > 0) ? 1u : 0u);
            else if (kWide)
              tcgen05_mma_bf16_elect(d_tmem, x_desc + static_cast<uint64_t>(2 * k), y_desc + static_cast<uint64_t>(2 * k),
                                     kIdesc, (kb > kb_begin || k > 0) ? 1u : 0u);
            else
              tcgen05_mma_bf16(d_tmem, x_desc + static_cast<uint64_t>(2 * k), y_desc + static_cast<uint64_t>(2 * k),
                               kIdesc, (kb > kb_begin || k > 0) ? 1u : 0u);
          }
          // the stage is free once these products have read it (in both blocks of a pair)
          if (PAIR) {
            tcgen05_commit_pair(smem_u32(&empty[stage]));
            tcgen05_commit_pair(other_empty + 8 * stage);
          } else if (kWide) {
            tcgen05_commit_elect(&empty[stage]);
          } else {
            tcgen05_commit(&empty[stage]);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
          if (kWide) arrived = __shfl_sync(0xffffffffu, arrived_next, 0) != 0;
        }
        if (PAIR) {
          tcgen05_commit_pair(smem_u32(&acc_full[acc]));
          tcgen05_commit_pair(other_acc_full + 8 * acc);
        } else if (kWide) {
          tcgen05_commit_elect(&acc_full[acc]);
        } else {
          tcgen05_commit(&acc_full[acc]);
        }
      }
    }
  } else {
    // ---------------- epilogue warps 0..3 ----------------
    pdl_wait();  // outputs, the residual stream, and the scratch belong to earlier kernels until now
    int local = 0;
    WorkLoop<kEven> work(p, PAIR);
    Piece piece;
    const uint32_t pair_acc_empty = PAIR ? in_block(smem_u32(&acc_empty[0]), 0) : 0u;
    for (; work.next(piece); ++local) {
      const int tile = piece.tile;
      const int tx = PAIR ? 2 * (tile % p.tiles_x) + static_cast<int>(rank) : tile % p.tiles_x;
      const int ty = tile / p.tiles_x;
      const int acc = local & 1;
      // Even shares: a piece that starts inside a tile is a partial sum for another block; the
      // piece with the tile's first k-block that does not reach its last one waits for the blocks
      // behind this one whose shares start inside the same tile.
      const bool whole = piece.kb_begin == 0 && piece.kb_end == p.num_k_blocks;
      const bool partial = p.splits > 1 || (kEven && p.even_shares && piece.kb_begin > 0);
      int helpers = 0;
      if (kEven && p.even_shares && !whole && !partial) {
        const long tile_end = static_cast<long>(tile + 1) * p.num_k_blocks;
        while (share_begin(p, blockIdx.x + 1 + helpers, gridDim.x) < tile_end) ++helpers;
      }
      const uint32_t acc_phase = (local >> 1) & 1u;
      const int row_in_tile = warp * 32 + lane;
      const int row = tx * kTileX + row_in_tile;
      // The q/k/v ending's inputs that the host wrote before the step (the token's position, its
      // cache page, the biases of the tile's columns) are fetched while the products still run;
      // after them only the rows of the cosine and sine tables are read from memory.
      int rope_position = 0, rope_page = -1;
      float* tile_bias = reinterpret_cast<float*>(staging) + (local & 1) * BN;   // two buffers: a warp may be one tile ahead
      if (!SWAP && BN >= 128 && p.epilogue == EPI_ROPE_CACHE) {
        if (row < p.tokens) {
          rope_position = p.positions[row];
          if (p.write_cache)
            rope_page = p.block_table[static_cast<size_t>(p.token_entry[row]) * p.table_width + rope_position / p.page_size];
        }
        for (int c = row_in_tile; c < BN; c += 128) {
          const int n = ty * BN + c;
          tile_bias[c] = (p.bias && n < p.features) ? p.bias[n] : 0.0f;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
      if (kWide) {
        if (lane == 0) mbar_wait(&acc_full[acc], acc_phase, abort_flag, p.status);   // one lane of a warp polls
        __syncwarp();
      } else {
        mbar_wait(&acc_full[acc], acc_phase, abort_flag, p.status);
      }
      tcgen05_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + static_cast<uint32_t>(acc * BN);
      if (kEven && helpers > 0) {
        if (warp == 0 && lane == 0) {
          for (int h = 0; h < helpers; ++h) {
            int* flag = p.share_flags + blockIdx.x + 1 + h;
            uint32_t spin = 0;
            int up = 0;
            for (; spin < kWaitLimit; ++spin) {
              asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(up) : "l"(flag) : "memory");
              if (up != 0) break;
              if ((spin & 1023u) == 1023u && *abort_flag) break;
              __nanosleep(64);
            }
            if (up == 0 && !*abort_flag) {
              *abort_flag = 1;
              atomicExch(p.status, GEMM_TC_WAIT_EXPIRED);
            }
            *flag = 0;   // down again for the next launch; its slot is not written again in this one
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
      if (!partial) {
        if (!SWAP && BN >= 128 && p.epilogue == EPI_ROPE_CACHE) {
          // The q/k/v product's ending: thread = token; a head's d columns are read as pairs of
          // 32-column chunks (i, i + d/2), the halves of the rotary pairs.  A chunk of the token's
          // cosines and sines serves every head of the tile, and the next chunk is asked for
          // before this one is used.
          const int d = p.head_dim, half = d >> 1;
          const int t = row;
          const bool live = t < p.tokens;
          const int position = rope_position;
          const bool rotate = p.rope_style == GEMM_ROPE_NEOX;
          const float4* cos_row = reinterpret_cast<const float4*>(p.cos_table + static_cast<size_t>(position) * half);
          const float4* sin_row = reinterpret_cast<const float4*>(p.sin_table + static_cast<size_t>(position) * half);
          float4 cs[8], sn[8];
          if (rotate && live) {
#pragma unroll
            for (int i = 0; i < 8; ++i) { cs[i] = cos_row[i]; sn[i] = sin_row[i]; }
          }
#pragma unroll 1
          for (int i0 = 0; i0 < half; i0 += 32) {
            float4 cs_next[8], sn_next[8];
            if (rotate && live && i0 + 32 < half) {
#pragma unroll
              for (int i = 0; i < 8; ++i) { cs_next[i] = cos_row[(i0 + 32) / 4 + i]; sn_next[i] = sin_row[(i0 + 32) / 4 + i]; }
            }
#pragma unroll 1
            for (int hc = 0; hc < BN; hc += d) {
              const int n0 = ty * BN + hc;
              if (n0 >= p.features) break;
              const int head = n0 / d;
              const bool is_q = head < p.num_heads;
              const bool is_v = head >= p.num_heads + p.num_kv_heads;
              __nv_bfloat16* dst = nullptr;
              if (live) {
                if (is_q) {
                  dst = p.q_out + (static_cast<size_t>(t) * p.num_heads + head) * d;
                } else if (rope_page >= 0) {
                  const int kv_head = is_v ? head - p.num_heads - p.num_kv_heads : head - p.num_heads;
                  dst = (is_v ? p.v_pool : p.k_pool) +
                        ((static_cast<size_t>(rope_page) * p.page_size + position % p.page_size) * p.num_kv_heads + kv_head) * d;
                }
              }
              uint32_t lo_bits[32], hi_bits[32];
              tmem_load_32_nowait(taddr + hc + i0, lo_bits);
              tmem_load_32_nowait(taddr + hc + half + i0, hi_bits);
              tmem_load_wait();
              if (dst == nullptr) continue;
              float lo[32], hi[32];
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                lo[i] = __uint_as_float(lo_bits[i]) + tile_bias[hc + i0 + i];
                hi[i] = __uint_as_float(hi_bits[i]) + tile_bias[hc + half + i0 + i];
              }
              if (!is_v && rotate) {
#pragma unroll
                for (int i = 0; i < 32; i += 4) {
                  const float4 c4 = cs[i >> 2], s4 = sn[i >> 2];
                  const float cv[4] = {c4.x, c4.y, c4.z, c4.w}, sv[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
                  for (int u = 0; u < 4; ++u) {
                    const float x = lo[i + u], y = hi[i + u];
                    lo[i + u] = x * cv[u] - y * sv[u];
                    hi[i + u] = x * sv[u] + y * cv[u];
                  }
                }
              }
#pragma unroll
              for (int i = 0; i < 32; i += 8) {
                uint4 packed_lo, packed_hi;
                packed_lo.x = pack_bf16x2(lo[i], lo[i + 1]); packed_lo.y = pack_bf16x2(lo[i + 2], lo[i + 3]);
                packed_lo.z = pack_bf16x2(lo[i + 4], lo[i + 5]); packed_lo.w = pack_bf16x2(lo[i + 6], lo[i + 7]);
                packed_hi.x = pack_bf16x2(hi[i], hi[i + 1]); packed_hi.y = pack_bf16x2(hi[i + 2], hi[i + 3]);
                packed_hi.z = pack_bf16x2(hi[i + 4], hi[i + 5]); packed_hi.w = pack_bf16x2(hi[i + 6], hi[i + 7]);
                *reinterpret_cast<uint4*>(dst + i0 + i) = packed_lo;
                *reinterpret_cast<uint4*>(dst + half + i0 + i) = packed_hi;
              }
            }
            if (rotate && live && i0 + 32 < half) {
#pragma unroll
              for (int i = 0; i < 8; ++i) { cs[i] = cs_next[i]; sn[i] = sn_next[i]; }
            }
          }
        } else if (!SWAP && BN >= 128 && p.tma_ending) {
          // The ending through shared memory: each warp lays 32 rows x 128 bytes into a
          // swizzled buffer (no bank conflicts), and one lane hands the box to TMA, which
          // writes whole lines, clips at the matrix's edges and, for the residual stream,
          // does the addition in memory.  Two buffers per warp: one is filled while the
          // other is read.
          uint8_t* mine = staging + warp * 2 * 4096;
          int use = 0;
          const int row0 = tx * kTileX + warp * 32;
          if (p.epilogue == EPI_SWIGLU) {
            // 128 accumulator columns make 64 outputs = one 128-byte row of bfloat16
#pragma unroll 1
            for (int c = 0; c < BN; c += 128) {
              // a box that lies wholly outside the matrix is skipped altogether (were it only
              // not handed over, the next box would overwrite a buffer TMA may still be reading)
              if (row0 >= p.tokens || ty * BN + c >= p.features) continue;
              uint8_t* buffer = mine + use * 4096;
              if (lane == 0) tma_store_wait_read<1>();
              __syncwarp();
#pragma unroll 1
              for (int q4 = 0; q4 < 4; ++q4) {
                float v[32];
                tmem_load_32(taddr + c + q4 * 32, v);
                uint32_t packed[8];
#pragma unroll
                for (int i = 0; i < 8; ++i)
                  packed[i] = pack_bf16x2(silu_mul(v[2 * i], v[16 + 2 * i]), silu_mul(v[2 * i + 1], v[16 + 2 * i + 1]));
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                  const int chunk = (q4 * 2 + h) ^ (lane & 7);
                  *reinterpret_cast<uint4*>(buffer + lane * 128 + chunk * 16) =
                      make_uint4(packed[4 * h], packed[4 * h + 1], packed[4 * h + 2], packed[4 * h + 3]);
                }
              }
              fence_async_shared();
              __syncwarp();
              if (lane == 0) {
                tma_store_2d(&map_out, buffer, (ty * BN + c) >> 1, row0);
                tma_store_commit();
              }
              use ^= 1;
            }
          } else {
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
              if (row0 >= p.tokens || ty * BN + c >= p.features) continue;
              uint8_t* buffer = mine + use * 4096;
              float v[32];
              tmem_load_32(taddr + c, v);
              for (int h = 0; kEven && h < helpers; ++h) {
                const float* part = p.scratch + (static_cast<size_t>(blockIdx.x + 1 + h) * BN + c) * kTileX + row_in_tile;
                float more[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) more[i] = __ldcg(part + i * kTileX);
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] += more[i];
              }
              if (p.epilogue == EPI_STORE && p.bias) {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                  const int n = ty * BN + c + i;
                  v[i] += n < p.features ? p.bias[n] : 0.0f;
                }
              }
              if (lane == 0) tma_store_wait_read<1>();
              __syncwarp();
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const int chunk = j ^ (lane & 7);
                *reinterpret_cast<float4*>(buffer + lane * 128 + chunk * 16) =
                    make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
              }
              fence_async_shared();
              __syncwarp();
              if (lane == 0) {
                if (p.epilogue == EPI_RESIDUAL) tma_reduce_add_2d(&map_out, buffer, ty * BN + c, row0);
                else tma_store_2d(&map_out, buffer, ty * BN + c, row0);
                tma_store_commit();
              }
              use ^= 1;
            }
          }
        } else if (BN >= 32) {
#pragma unroll 1
          for (int c = 0; c < BN; c += 32) {
            float v[32];
            tmem_load_32(taddr + c, v);
            finish_chunk<BN, SWAP>(p, v, 32, row, ty * BN + c);
          }
        } else {
          float v[32];
          tmem_load_16(taddr, v);
          finish_chunk<BN, SWAP>(p, v, 16, row, ty * BN);
        }
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (PAIR) mbar_arrive_cluster(pair_acc_empty + 8 * acc);
          else mbar_arrive(&acc_empty[acc]);
        }
      } else {
        // partial sums: scratch[slot][column][row_in_tile]
        float* part = p.scratch + static_cast<size_t>(piece.slot) * BN * kTileX;
        if (BN >= 32) {
#pragma unroll 1
          for (int c = 0; c < BN; c += 32) {
            float v[32];
            tmem_load_32(taddr + c, v);
#pragma unroll
            for (int i = 0; i < 32; ++i) __stcg(part + static_cast<size_t>(c + i) * kTileX + row_in_tile, v[i]);
          }
        } else {
          float v[32];
          tmem_load_16(taddr, v);
#pragma unroll
          for (int i = 0; i < 16; ++i) __stcg(part + static_cast<size_t>(i) * kTileX + row_in_tile, v[i]);
        }
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[acc]);
        if (kEven && p.even_shares) {
          // the flag goes up when all four warps' partial sums can be seen by the other blocks
          __threadfence();
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (warp == 0 && lane == 0) {
            int* flag = p.share_flags + piece.slot;
            asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(flag), "r"(1) : "memory");
          }
        }
      }
    }
  }

  // stores handed to TMA must have landed before the block leaves
  if (warp < 4 && lane == 0) tma_store_wait_all();

  // ---------------- teardown ----------------
  tcgen05_fence_before();
  if (PAIR) cluster_sync_all();   // neither block leaves while the other may still read its shared memory
  else __syncthreads();
  if (*abort_flag && threadIdx.x == 0) {
    // Loads this block issued may still be landing in its shared memory: give them time.
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }
  __syncthreads();
  if (warp == 0) {
    tcgen05_fence_after();
    if (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(Config::kTmemCols));
    else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(Config::kTmemCols));
  }
}

// The second kernel of a product that was cut along K (few tokens: rows of the partial tiles
// are features, columns are tokens): one thread per output element adds the splits' partial
// sums, split 0 first, and writes the ending.  Neighbouring threads take neighbouring
// features, so the partial sums and the outputs are both read and written in whole lines.
template <int BN>
__global__ void __launch_bounds__(256)
splitk_finish_kernel(const GemmParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int N = p.features;
  const bool swiglu = p.epilogue == EPI_SWIGLU;
  const int width = swiglu ? N >> 1 : N;            // outputs per token
  const long id = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (id >= static_cast<long>(p.tokens) * width) return;
  const int t = static_cast<int>(id / width), o = static_cast<int>(id % width);
  const int ty = t / BN, col = t % BN;
  // feature rows this output needs: itself, or the gate and up rows of feature o
  const int n0 = swiglu ? (o >> 4) * 32 + (o & 15) : o;
  const int n1 = n0 + 16;
  auto total = [&](int n) {
    const int tx = n / kTileX, row = n % kTileX;
    const size_t tile = static_cast<size_t>(ty) * p.tiles_x + tx;
    const float* src = p.scratch + ((tile * p.splits) * BN + col) * kTileX + row;
    const size_t step = static_cast<size_t>(BN) * kTileX;
    // sixteen loads in flight at a time (a decode step's products have at most about that many
    // splits, so the sum costs one trip to L2, not one per few splits); the additions stay in the
    // order of the splits
    float sum = 0.0f;
    for (int s0 = 0; s0 < p.splits; s0 += 16) {
      float v[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) v[i] = s0 + i < p.splits ? __ldcg(src + (s0 + i) * step) : 0.0f;
#pragma unroll
      for (int i = 0; i < 16; ++i)
        if (s0 + i < p.splits) sum += v[i];
    }
    return sum;
  };
  if (swiglu) {
    const float value = silu_mul(total(n0), total(n1));
    const size_t at = static_cast<size_t>(t) * width + o;
    if (p.out_dtype == VIPERA_BF16) static_cast<__nv_bfloat16*>(p.out)[at] = __float2bfloat16_rn(value);
    else static_cast<float*>(p.out)[at] = value;
    return;
  }
  const float value = total(n0);
  const size_t at = static_cast<size_t>(t) * N + o;
  if (p.epilogue == EPI_RESIDUAL) {
    atomicAdd(p.resid + at, value);   // one addition per element: no need to read the old value back
  } else {
    const float biased = value + (p.bias ? p.bias[o] : 0.0f);
    if (p.out_dtype == VIPERA_BF16) static_cast<__nv_bfloat16*>(p.out)[at] = __float2bfloat16_rn(biased);
    else static_cast<float*>(p.out)[at] = biased;
  }
}

// The same for portions of a few hundred tokens, where the kernel above is several waves of
// blocks that each make one trip to memory: a thread takes four neighbouring outputs of a token
// (16-byte reads of the partial sums, one 16-byte write), a quarter of the threads.  A kernel of
// its own, so that the few-token form stays as short as it is.
template <int BN>
__global__ void __launch_bounds__(256)
splitk_finish4_kernel(const GemmParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int N = p.features;
  const bool swiglu = p.epilogue == EPI_SWIGLU;
  const int width = swiglu ? N >> 1 : N;            // outputs per token, a multiple of 4
  const int quads = width >> 2;
  const long id = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (id >= static_cast<long>(p.tokens) * quads) return;
  const int t = static_cast<int>(id / quads), o = static_cast<int>(id % quads) * 4;
  const int ty = t / BN, col = t % BN;
  const int n0 = swiglu ? (o >> 4) * 32 + (o & 15) : o;   // four neighbouring rows of one tile (o is a multiple of 4)
  auto total = [&](int n) {
    const int tx = n / kTileX, row = n % kTileX;
    const size_t tile = static_cast<size_t>(ty) * p.tiles_x + tx;
    const float4* src = reinterpret_cast<const float4*>(p.scratch + ((tile * p.splits) * BN + col) * kTileX + row);
    const size_t step = static_cast<size_t>(BN) * kTileX / 4;
    float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (int s0 = 0; s0 < p.splits; s0 += 8) {
      float4 v[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = s0 + i < p.splits ? __ldcg(src + (s0 + i) * step) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (s0 + i < p.splits) { sum.x += v[i].x; sum.y += v[i].y; sum.z += v[i].z; sum.w += v[i].w; }
      }
    }
    return sum;
  };
  float4 value = total(n0);
  const size_t at = static_cast<size_t>(t) * width + o;
  if (swiglu) {
    const float4 up = total(n0 + 16);
    value = make_float4(silu_mul(value.x, up.x), silu_mul(value.y, up.y), silu_mul(value.z, up.z), silu_mul(value.w, up.w));
  } else if (p.epilogue == EPI_RESIDUAL) {
    // one addition per element, nothing read back
    float* dst = p.resid + at;
    atomicAdd(dst, value.x);
    atomicAdd(dst + 1, value.y);
    atomicAdd(dst + 2, value.z);
    atomicAdd(dst + 3, value.w);
    return;
  } else if (p.bias) {
    const float4 b = *reinterpret_cast<const float4*>(p.bias + o);
    value = make_float4(value.x + b.x, value.y + b.y, value.z + b.z, value.w + b.w);
  }
  if (p.out_dtype == VIPERA_BF16) {
    uint2 packed;
    packed.x = pack_bf16x2(value.x, value.y);
    packed.y = pack_bf16x2(value.z, value.w);
    *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(p.out) + at) = packed;
  } else {
    *reinterpret_cast<float4*>(static_cast<float*>(p.out) + at) = value;
  }
}

// The split sums of a q/k/v product of a few dozen to a few hundred tokens, with that product's
// ending: a thread adds up, for one token and one head, four neighbouring values of the head's
// first half and the four they are paired with in the second half, adds the biases, turns the
// pairs by the token's position and writes q to its buffer, k and v into their cache pages.  (The
// same sums, formulas and roundings as the split-sum kernel followed by the rotation kernel, in
// one launch instead of two.)
template <int BN>
__global__ void __launch_bounds__(256)
splitk_finish_rope_kernel(const GemmParams p) {
  pdl_launch_dependents();
  const int d = p.head_dim, half = d >> 1;
  const int quads = half >> 2;                          // per head
  const int all_heads = p.num_heads + 2 * p.num_kv_heads;
  const long id = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const bool mine = id < static_cast<long>(p.tokens) * all_heads * quads;
  const int t = mine ? static_cast<int>(id / (all_heads * quads)) : 0;
  const int within = mine ? static_cast<int>(id % (all_heads * quads)) : 0;
  const int head = within / quads, i = (within % quads) * 4;
  // what the host wrote before the step is read before the wait
  const int position = p.positions[t];
  const bool is_q = head < p.num_heads;
  const bool is_v = head >= p.num_heads + p.num_kv_heads;
  __nv_bfloat16* dst = nullptr;
  if (is_q) {
    dst = p.q_out + (static_cast<size_t>(t) * p.num_heads + head) * d;
  } else if (p.write_cache) {
    const int page = p.block_table[static_cast<size_t>(p.token_entry[t]) * p.table_width + position / p.page_size];
    if (page >= 0) {
      const int kv_head = is_v ? head - p.num_heads - p.num_kv_heads : head - p.num_heads;
      dst = (is_v ? p.v_pool : p.k_pool) +
            ((static_cast<size_t>(page) * p.page_size + position % p.page_size) * p.num_kv_heads + kv_head) * d;
    }
  }
  const bool rotate = !is_v && p.rope_style == GEMM_ROPE_NEOX;
  float4 c4 = make_float4(1.0f, 1.0f, 1.0f, 1.0f), s4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  if (rotate) {
    c4 = *reinterpret_cast<const float4*>(p.cos_table + static_cast<size_t>(position) * half + i);
    s4 = *reinterpret_cast<const float4*>(p.sin_table + static_cast<size_t>(position) * half + i);
  }
  const int n_lo = head * d + i, n_hi = n_lo + half;
  float4 b_lo = make_float4(0.0f, 0.0f, 0.0f, 0.0f), b_hi = b_lo;
  if (p.bias) {
    b_lo = *reinterpret_cast<const float4*>(p.bias + n_lo);
    b_hi = *reinterpret_cast<const float4*>(p.bias + n_hi);
  }
  pdl_wait();
  if (!mine || dst == nullptr) return;
  const int ty = t / BN, col = t % BN;
  auto total = [&](int n) {
    const int tx = n / kTileX, row = n % kTileX;
    const size_t tile = static_cast<size_t>(ty) * p.tiles_x + tx;
    const float4* src = reinterpret_cast<const float4*>(p.scratch + ((tile * p.splits) * BN + col) * kTileX + row);
    const size_t step = static_cast<size_t>(BN) * kTileX / 4;
    float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (int s0 = 0; s0 < p.splits; s0 += 8) {
      float4 v[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) v[k] = s0 + k < p.splits ? __ldcg(src + (s0 + k) * step) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        if (s0 + k < p.splits) { sum.x += v[k].x; sum.y += v[k].y; sum.z += v[k].z; sum.w += v[k].w; }
      }
    }
    return sum;
  };
  float4 lo = total(n_lo), hi = total(n_hi);
  lo = make_float4(lo.x + b_lo.x, lo.y + b_lo.y, lo.z + b_lo.z, lo.w + b_lo.w);
  hi = make_float4(hi.x + b_hi.x, hi.y + b_hi.y, hi.z + b_hi.z, hi.w + b_hi.w);
  if (rotate) {
    const float4 a = lo, b = hi;
    lo = make_float4(a.x * c4.x - b.x * s4.x, a.y * c4.y - b.y * s4.y, a.z * c4.z - b.z * s4.z, a.w * c4.w - b.w * s4.w);
    hi = make_float4(a.x * s4.x + b.x * c4.x, a.y * s4.y + b.y * c4.y, a.z * s4.z + b.z * c4.z, a.w * s4.w + b.w * c4.w);
  }
  uint2 packed_lo, packed_hi;
  packed_lo.x = pack_bf16x2(lo.x, lo.y); packed_lo.y = pack_bf16x2(lo.z, lo.w);
  packed_hi.x = pack_bf16x2(hi.x, hi.y); packed_hi.y = pack_bf16x2(hi.z, hi.w);
  *reinterpret_cast<uint2*>(dst + i) = packed_lo;
  *reinterpret_cast<uint2*>(dst + half + i) = packed_hi;
}

// Even shares: one flag per block, up while that block's partial sum waits to be taken.  All
// are 0 between launches (the taker lowers them); products run one after another on a stream.
constexpr int kMostShares = 1024;
__device__ int share_flags_store[kMostShares];

// ---------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool looked = false;
  if (!looked) {
    looked = true;
    void* entry = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &result) == cudaSuccess &&
        result == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(entry);
  }
  return fn;
}

// A [rows, K] bf16 row-major matrix, read in boxes of [box_rows, 64] with 128-byte swizzle;
// rows and K beyond the matrix read as zero.
// Maps already made, by what they describe: the same weights and workspace buffers come
// back step after step, and encoding a map costs about as much as the launch's own
// bookkeeping.  (A map holds an address and sizes only, so it stays valid while that memory
// is what the caller says it is.)
struct MapKey {
  const void* base;
  int rows, cols, box_rows, kind;
  bool operator<(const MapKey& o) const {
    return std::tie(base, rows, cols, box_rows, kind) < std::tie(o.base, o.rows, o.cols, o.box_rows, o.kind);
  }
};
static std::map<MapKey, CUtensorMap>& kept_maps() {
  static std::map<MapKey, CUtensorMap> kept;
  return kept;
}
static std::mutex& kept_maps_guard() {
  static std::mutex guard;
  return guard;
}
static bool find_map(const MapKey& key, CUtensorMap* map) {
  std::lock_guard<std::mutex> lock(kept_maps_guard());
  auto found = kept_maps().find(key);
  if (found == kept_maps().end()) return false;
  *map = found->second;
  return true;
}
static void keep_map(const MapKey& key, const CUtensorMap& map) {
  std::lock_guard<std::mutex> lock(kept_maps_guard());
  if (kept_maps().size() > 8192) kept_maps().clear();
  kept_maps()[key] = map;
}

static int make_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
  const MapKey key{base, rows, K, box_rows, 0};
  if (find_map(key, map)) return VIPERA_OK;
  EncodeTiledFn encode = encode_tiled_fn();
  if (!encode) return VIPERA_NO_DRIVER_ENTRY;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(K) * 2};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(kBlockK), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return VIPERA_BAD_ARGUMENT;
  keep_map(key, *map);
  return VIPERA_OK;
}

// The output as TMA sees it: [rows, cols] of float32 or bfloat16, in boxes of 32 rows x 128 bytes.
static int make_out_map(CUtensorMap* map, void* base, int rows, int cols, bool bf16) {
  const MapKey key{base, rows, cols, 32, bf16 ? 1 : 2};
  if (find_map(key, map)) return VIPERA_OK;
  EncodeTiledFn encode = encode_tiled_fn();
  if (!encode) return VIPERA_NO_DRIVER_ENTRY;
  const int element = bf16 ? 2 : 4;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * element};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(128 / element), 32};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = encode(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, base, dims,
                      strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                      CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return VIPERA_BAD_ARGUMENT;
  keep_map(key, *map);
  return VIPERA_OK;
}

struct GemmPlan {
  bool swap;
  bool pair;          // tiles of 256 tokens by pairs of blocks (clusters of two)
  bool even_shares;   // one equal share of all k-blocks per block instead of whole tiles
  int blocks;         // even shares: the grid
  int bn;
  int tiles_x, tiles_y, splits, k_blocks_per_split, num_k_blocks;
  size_t scratch_floats;
};

static int sm_count() {
  static int count = 0;
  if (count == 0) {
    int device = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device);
    if (count <= 0) count = 148;
  }
  return count;
}

// 0: never; 1: where the estimate favours them; 2: wherever the ending allows them (tests).
// Off unless asked for: blocks with even shares drift apart along K, and tiles read by several
// blocks at different times cost more lookups in L2 than tiles read in step (2,048 tokens through
// a [1536, 8960] matrix: 68 us against 65 with whole tiles of 192 columns; ahead only from about
// 4,096 tokens on: 110 us against 124).
static int& even_shares_mode() {
  static int mode = std::getenv("VIPERA_GEMM_EVEN_SHARES") ? std::atoi(std::getenv("VIPERA_GEMM_EVEN_SHARES")) : 0;
  return mode;
}
// 0: never; 1: where the estimate favours them; 2: wherever the form allows them
static int& pair_mode() {
  static int mode = std::getenv("VIPERA_GEMM_PAIR") ? std::atoi(std::getenv("VIPERA_GEMM_PAIR")) : 1;
  return mode;
}
// How many pairs of blocks of this tile width the device runs at once (0: clusters of two with
// this much shared memory cannot be launched here, and the product stays with blocks alone).
template <int BN>
static int pair_clusters() {
  static int clusters = -1;
  if (clusters < 0) {
    using Config = TileConfig<BN, true>;
    auto kernel = gemm_tc_kernel<BN, false, true>;
    clusters = 0;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Config::kSmemBytes) == cudaSuccess) {
      cudaLaunchConfig_t config = {};
      config.blockDim = dim3(threads_for<BN>());
      config.dynamicSmemBytes = Config::kSmemBytes;
      config.gridDim = dim3(2 * (sm_count() / 2));
      cudaLaunchAttribute attribute[1];
      attribute[0].id = cudaLaunchAttributeClusterDimension;
      attribute[0].val.clusterDim.x = 2;
      attribute[0].val.clusterDim.y = 1;
      attribute[0].val.clusterDim.z = 1;
      config.attrs = attribute;
      config.numAttrs = 1;
      int fit = 0;
      if (cudaOccupancyMaxActiveClusters(&fit, kernel, &config) == cudaSuccess && fit > 0) clusters = std::min(fit, sm_count() / 2);
    }
    cudaGetLastError();   // a refusal above is an answer, not an error of the caller's
  }
  return clusters;
}
static int pair_clusters_for(int bn) { return bn == 256 ? pair_clusters<256>() : bn == 192 ? pair_clusters<192>() : pair_clusters<128>(); }

constexpr int kShareLeast = 8;      // even shares: k-blocks a block must get at least
constexpr double kShareCost = 4.0;  // what a block's partial sum costs (written, read back, added), in k-blocks of its time

// `even_ok`: the ending can take partial sums of other blocks (the TMA ending of STORE and RESIDUAL).
static GemmPlan make_plan(int T, int N, int K, int sms, int epilogue = EPI_STORE, bool even_ok = false) {
  GemmPlan plan{};
  plan.num_k_blocks = (K + kBlockK - 1) / kBlockK;
  // Tokens go on the 128-row side from 192 tokens on.  A matrix wide enough to give half
  // the SMs a tile of 128 features each takes that form from 33 tokens on: its ending
  // leaves through shared memory and TMA in whole rows, where the swapped form writes
  // 32-feature pieces of a row (measured at 64 tokens on a [17920, 1536] matrix with the
  // SwiGLU ending: 14.1 us against 17.4; at 128 tokens 14.4 against 22.8).
  static const int nonswap_from = std::getenv("VIPERA_GEMM_NONSWAP_FROM") ? std::atoi(std::getenv("VIPERA_GEMM_NONSWAP_FROM")) : 33;
  plan.swap = true;
  if (T >= 128 + 64 || (T >= nonswap_from && N >= 64 * sms)) {
    plan.swap = false;
    plan.tiles_x = (T + kTileX - 1) / kTileX;
    // The widest tile that keeps the SMs busy: a tile of 256 columns reads the least per
    // flop, but when the tiles do not fill the last wave a narrower tile wastes less.
    const int candidates[3] = {256, 192, 128};
    double best = -1.0;
    plan.bn = 128;
    for (int bn : candidates) {
      if (bn > 128 && N < bn) continue;
      if (bn == 192 && (epilogue == EPI_SWIGLU || epilogue == EPI_ROPE_CACHE)) continue;  // these endings work in steps of 128 (or of a head)
      const long items = static_cast<long>(plan.tiles_x) * ((N + bn - 1) / bn);
      const long waves = (items + sms - 1) / sms;
      double efficiency = static_cast<double>(plan.tiles_x) * N / (static_cast<double>(waves) * sms * bn);
      efficiency *= bn == 256 ? 1.0 : bn == 192 ? 0.95 : 0.85;  // narrower tiles run below the wide tile's rate
      if (efficiency > best) { best = efficiency; plan.bn = bn; }
    }
    // Against that, even shares of all k-blocks with the widest tile: no idle SMs in a last
    // wave, but every block pays for one partial sum.
    const int even_mode = even_shares_mode();
    if (even_ok && even_mode > 0 && N >= 128) {
      const int bn = N >= 256 ? 256 : 128;
      const long tiles = static_cast<long>(plan.tiles_x) * ((N + bn - 1) / bn);
      const long all = tiles * plan.num_k_blocks;
      const int blocks = static_cast<int>(std::min<long>(sms, all / kShareLeast));
      if (blocks >= 2 && tiles % blocks != 0) {
        double efficiency = static_cast<double>(plan.tiles_x) * N / (static_cast<double>(tiles) * bn);
        efficiency *= static_cast<double>(all) / (static_cast<double>(all) + kShareCost * blocks);
        efficiency *= (bn == 256 ? 1.0 : 0.85) * static_cast<double>(blocks) / sms;
        if (efficiency > best + 0.03 || even_mode > 1) {
          plan.even_shares = true;
          plan.blocks = blocks;
          plan.bn = bn;
        }
      }
    }
    // Pairs of blocks on tiles of 256 tokens: each block reads its own 128 tokens and half of the
    // tile's weight rows, a third less per flop than a block alone, which is what holds the
    // tensor cores up.  Clusters of two fill half as many slots as there are SMs.
    const int pairs_mode = pair_mode();
    if (!plan.even_shares && pairs_mode > 0 && T > kTileX) {
      static const int forced_bn = std::getenv("VIPERA_GEMM_PAIR_BN") ? std::atoi(std::getenv("VIPERA_GEMM_PAIR_BN")) : 0;
      const int rows2 = (T + 2 * kTileX - 1) / (2 * kTileX);
      double best_pair = -1.0;
      int bn_pair = 0;
      for (int bn : candidates) {
        if (N < bn) continue;
        if (bn == 192 && (epilogue == EPI_SWIGLU || epilogue == EPI_ROPE_CACHE)) continue;
        if (forced_bn && bn != forced_bn) continue;
        const int clusters = pair_clusters_for(bn);
        if (clusters <= 0) continue;
        const long items = static_cast<long>(rows2) * ((N + bn - 1) / bn);
        const long waves = (items + clusters - 1) / clusters;
        // one wave over a short K is all set-up and ending, and a pair has more of both
        if (waves < 2 && plan.num_k_blocks < 48 && pairs_mode < 2) continue;
        double efficiency = static_cast<double>(T) * N / (static_cast<double>(waves) * clusters * 2 * kTileX * bn);
        efficiency *= bn == 256 ? 1.15 : bn == 192 ? 1.1 : 0.9;   // measured against blocks alone
        if (efficiency > best_pair) { best_pair = efficiency; bn_pair = bn; }
      }
      // `best` counts whole 128-row tiles; put it on the same footing (tokens, not tiles)
      const double best_alone = best * T / (static_cast<double>(plan.tiles_x) * kTileX);
      if (bn_pair && (best_pair > best_alone || pairs_mode > 1)) {
        plan.pair = true;
        plan.bn = bn_pair;
        plan.tiles_x = rows2;
      }
    }
    plan.tiles_y = (N + plan.bn - 1) / plan.bn;
    plan.splits = 1;
    plan.k_blocks_per_split = plan.num_k_blocks;
    // A narrow matrix under a portion of a few hundred tokens has tiles for a fraction of the
    // SMs only (1,536 columns, 512 tokens: 32 tiles), and this form does not cut K.  The other
    // form does: its tiles of 128 features x 256 tokens are cut along K until every SM has one,
    // at the price of a second kernel that adds the partial sums.  Which is quicker is estimated
    // where this form is a single wave (microseconds: 5 for a block's start and ending, 0.3 for a
    // k-block, 6 for the second kernel and 1 more per 1.5 MB of partial sums; fitted to
    // [1536, 1536], [1536, 8960], [3584, 3584] and [3584, 18944] under 192 to 1,792 tokens).
    // (The q/k/v ending inside the product kernel exists in this form only.)
    static const bool narrow_swaps = std::getenv("VIPERA_GEMM_NARROW_NONSWAP") == nullptr;
    const bool forced = (plan.pair && pair_mode() > 1);   // tests ask for pairs on small sizes too
    const int at_once = plan.pair ? std::max(1, pair_clusters_for(plan.bn)) : sms;
    if (narrow_swaps && !plan.even_shares && !forced && epilogue != EPI_ROPE_CACHE && plan.tiles_x * plan.tiles_y <= at_once) {
      const double this_form = 5.0 + plan.num_k_blocks * 0.3;
      const int bn_other = T <= 16 ? 16 : T <= 32 ? 32 : T <= 64 ? 64 : T <= 128 ? 128 : 256;
      const int tiles_other = ((N + kTileX - 1) / kTileX) * ((T + bn_other - 1) / bn_other);
      const int want = std::max(1, std::min(sms / tiles_other, plan.num_k_blocks));
      const int per_split = (plan.num_k_blocks + want - 1) / want;
      const int splits_other = (plan.num_k_blocks + per_split - 1) / per_split;
      const int waves_other = (tiles_other * splits_other + sms - 1) / sms;
      // the second kernel: its launch and one trip to memory, and the partial sums it has to read
      const double second = splits_other > 1 ? 6.0 + static_cast<double>(T) * N * splits_other * 4.0 / 1.5e6 : 0.0;
      const double other_form = 5.0 + waves_other * per_split * 0.3 + second;
      if (other_form + 5.0 < this_form) {   // (a margin: the estimate is coarse)
        plan.swap = true;
        plan.pair = false;
      }
    }
  }
  if (plan.swap) {
    plan.bn = T <= 16 ? 16 : T <= 32 ? 32 : T <= 64 ? 64 : T <= 128 ? 128 : 256;
    plan.tiles_x = (N + kTileX - 1) / kTileX;
    plan.tiles_y = (T + plan.bn - 1) / plan.bn;
    const int tiles = plan.tiles_x * plan.tiles_y;
    int want = sms / tiles;
    if (want < 1) want = 1;
    if (want > plan.num_k_blocks) want = plan.num_k_blocks;
    plan.k_blocks_per_split = (plan.num_k_blocks + want - 1) / want;
    plan.splits = (plan.num_k_blocks + plan.k_blocks_per_split - 1) / plan.k_blocks_per_split;
  }
  plan.scratch_floats = plan.splits > 1
      ? static_cast<size_t>(plan.tiles_x) * plan.tiles_y * plan.splits * plan.bn * kTileX : 0;
  if (plan.even_shares) plan.scratch_floats = static_cast<size_t>(plan.blocks) * plan.bn * kTileX;
  return plan;
}

// Bytes of scratch a product of these sizes needs for the partial sums of its splits (0 when
// it runs without splits).
VIPERA_API int vipera_gemm_tc_workspace(int T, int N, int K, size_t* scratch_bytes) {
  const GemmPlan plan = make_plan(T, N, K, sm_count());
  const GemmPlan even = make_plan(T, N, K, sm_count(), EPI_RESIDUAL, true);
  *scratch_bytes = std::max(plan.scratch_floats, even.scratch_floats) * sizeof(float);
  return VIPERA_OK;
}

VIPERA_API int vipera_gemm_tc_even_shares(int mode) {
  const int before = even_shares_mode();
  if (mode >= 0) even_shares_mode() = mode;
  return before;
}

VIPERA_API int vipera_gemm_tc_pairs(int mode) {
  const int before = pair_mode();
  if (mode >= 0) pair_mode() = mode;
  return before;
}

// The form a product of these sizes takes: {swapped, tile width, splits, even shares, blocks, pairs}.
VIPERA_API int vipera_gemm_tc_plan(int T, int N, int K, int epilogue, int even_ok, int* form) {
  const GemmPlan plan = make_plan(T, N, K, sm_count(), epilogue, even_ok != 0);
  form[0] = plan.swap ? 1 : 0;
  form[1] = plan.bn;
  form[2] = plan.splits;
  form[3] = plan.even_shares ? 1 : 0;
  form[4] = plan.even_shares ? plan.blocks : std::min(sm_count(), plan.tiles_x * plan.tiles_y * plan.splits);
  if (plan.pair) form[4] = 2 * std::min(pair_clusters_for(plan.bn), plan.tiles_x * plan.tiles_y);
  form[5] = plan.pair ? 1 : 0;
  return VIPERA_OK;
}

template <int BN, bool SWAP, bool EVEN = false>
static int launch_variant(const CUtensorMap& map_x, const CUtensorMap& map_y, const CUtensorMap& map_out,
                          const GemmParams& p, int grid, cudaStream_t s) {
  using Config = TileConfig<BN>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, SWAP, false, EVEN>, cudaFuncAttributeMaxDynamicSharedMemorySize, Config::kSmemBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  int status = vipera_launch(gemm_tc_kernel<BN, SWAP, false, EVEN>, grid, threads_for<BN>(), Config::kSmemBytes, s, map_x, map_y, map_out, p);
  if (status != VIPERA_OK || p.splits == 1) return status;   // (even shares run with splits == 1)
  if (p.epilogue == EPI_ROPE_CACHE) {
    const long threads = static_cast<long>(p.tokens) * (p.num_heads + 2 * p.num_kv_heads) * (p.head_dim / 8);
    return vipera_launch(splitk_finish_rope_kernel<BN>, dim3(static_cast<unsigned>((threads + 255) / 256)), dim3(256), 0, s, p);
  }
  const int width = p.epilogue == EPI_SWIGLU ? p.features / 2 : p.features;
  const long outputs = static_cast<long>(p.tokens) * width;
  // portions: four outputs to a thread where rows and pointers allow 16-byte accesses
  const bool aligned = (reinterpret_cast<uintptr_t>(p.scratch) & 15) == 0 && (reinterpret_cast<uintptr_t>(p.out) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(p.resid) & 15) == 0 && (reinterpret_cast<uintptr_t>(p.bias) & 15) == 0;
  // (from about 600 K outputs on: below that the scalar kernel is one wave of blocks anyway and
  // has four times the loads in flight; measured 1.98 against 2.21 ms for a step of 128 tokens,
  // 2.86 against 2.80 for 512)
  if (outputs >= 600000 && width % 4 == 0 && aligned)
    return vipera_launch(splitk_finish4_kernel<BN>, dim3(static_cast<unsigned>((outputs / 4 + 255) / 256)), dim3(256), 0, s, p);
  return vipera_launch(splitk_finish_kernel<BN>, dim3(static_cast<unsigned>((outputs + 255) / 256)), dim3(256), 0, s, p);
}

// Pairs of blocks: clusters of two, as many as fit on the device at once (a persistent loop).
template <int BN>
static int launch_pairs(const CUtensorMap& map_x, const CUtensorMap& map_y, const CUtensorMap& map_out,
                        const GemmParams& p, int items, cudaStream_t s) {
  using Config = TileConfig<BN, true>;
  auto kernel = gemm_tc_kernel<BN, false, true>;
  cudaLaunchConfig_t config = {};
  config.blockDim = dim3(threads_for<BN>());
  config.dynamicSmemBytes = Config::kSmemBytes;
  config.stream = s;
  cudaLaunchAttribute attributes[2];
  attributes[0].id = cudaLaunchAttributeClusterDimension;
  attributes[0].val.clusterDim.x = 2;
  attributes[0].val.clusterDim.y = 1;
  attributes[0].val.clusterDim.z = 1;
  attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attributes[1].val.programmaticStreamSerializationAllowed = vipera_pdl_enabled() ? 1 : 0;
  config.attrs = attributes;
  const int clusters = pair_clusters<BN>();
  if (clusters <= 0) return VIPERA_BAD_ARGUMENT;   // (the plan does not choose pairs then)
  config.numAttrs = 2;
  config.gridDim = dim3(2 * std::min(items, clusters));
  cudaError_t error = cudaLaunchKernelEx(&config, kernel, map_x, map_y, map_out, p);
  return error == cudaSuccess ? VIPERA_OK : static_cast<int>(error);
}

// A is [T, K] bfloat16, W is [N, K] bfloat16, both row-major and contiguous with K a
// multiple of 8 (TMA needs 16-byte row strides).  `status` is a device word that must be 0
// before the launch; it is non-zero afterwards when a bounded wait inside the kernel ran out.
// `rope`: for EPI_ROPE_CACHE, the fields of that ending (the others are filled in here).
static int run_gemm(const void* A, const void* W, int T, int N, int K, int epilogue, const float* bias, void* out,
                    int out_dtype, float* resid, float* scratch, size_t scratch_bytes, int* status, void* stream,
                    const GemmParams* rope) {
  if (T <= 0) return VIPERA_OK;
  if (N <= 0 || K <= 0 || (K % 8) != 0) return VIPERA_BAD_SHAPE;
  if (epilogue == EPI_SWIGLU && (N % 32) != 0) return VIPERA_BAD_SHAPE;
  if (out_dtype != VIPERA_F32 && out_dtype != VIPERA_BF16) return VIPERA_BAD_DTYPE;
  if ((epilogue == EPI_RESIDUAL && !resid) || (epilogue != EPI_RESIDUAL && epilogue != EPI_ROPE_CACHE && !out) || !status)
    return VIPERA_BAD_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(W) & 15)) return VIPERA_BAD_ARGUMENT;
  const int sms = sm_count();
  // what the TMA ending of STORE and RESIDUAL needs (the only ending that takes other blocks' partial sums)
  const bool direct_store = std::getenv("VIPERA_GEMM_DIRECT_STORE") != nullptr;
  const bool even_ok = !direct_store && N % 4 == 0 && scratch != nullptr &&
      ((epilogue == EPI_STORE && out_dtype == VIPERA_F32 && (reinterpret_cast<uintptr_t>(out) & 15) == 0) ||
       (epilogue == EPI_RESIDUAL && (reinterpret_cast<uintptr_t>(resid) & 15) == 0));
  const GemmPlan plan = make_plan(T, N, K, sms, epilogue, even_ok);
  if (plan.splits > 1 || plan.even_shares) {
    if (!scratch || scratch_bytes < plan.scratch_floats * sizeof(float)) return VIPERA_BAD_ARGUMENT;
  }
  CUtensorMap map_x, map_y;
  int r;
  if (plan.swap) {
    if ((r = make_map(&map_x, W, N, K, kTileX)) != VIPERA_OK) return r;
    if ((r = make_map(&map_y, A, T, K, plan.bn)) != VIPERA_OK) return r;
  } else {
    if ((r = make_map(&map_x, A, T, K, kTileX)) != VIPERA_OK) return r;
    if ((r = make_map(&map_y, W, N, K, plan.pair ? plan.bn / 2 : plan.bn)) != VIPERA_OK) return r;
  }
  GemmParams p{};
  if (rope) p = *rope;
  p.tokens = T;
  p.features = N;
  p.num_k_blocks = plan.num_k_blocks;
  p.tiles_x = plan.tiles_x;
  p.tiles_y = plan.tiles_y;
  p.splits = plan.splits;
  p.k_blocks_per_split = plan.k_blocks_per_split;
  p.epilogue = epilogue;
  p.out_dtype = out_dtype;
  p.bias = bias;
  p.out = out;
  p.resid = resid;
  p.scratch = scratch;
  p.status = status;
  const int items = plan.tiles_x * plan.tiles_y * plan.splits;
  const int grid = plan.even_shares ? plan.blocks : items < sms ? items : sms;
  p.even_shares = plan.even_shares ? 1 : 0;
  if (plan.even_shares) {
    if (plan.blocks > kMostShares) return VIPERA_BAD_ARGUMENT;
    void* flags = nullptr;
    if (cudaGetSymbolAddress(&flags, share_flags_store) != cudaSuccess) return VIPERA_BAD_ARGUMENT;
    p.share_flags = static_cast<int*>(flags);
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // The ending goes through TMA stores where the output's rows are whole multiples of 16
  // bytes: float32 [T, N] for STORE and RESIDUAL, bfloat16 [T, N / 2] for SWIGLU.
  CUtensorMap map_out = map_x;  // a valid map where the ending does not use one
  p.tma_ending = 0;
  if (!plan.swap && !direct_store) {
    if (epilogue == EPI_SWIGLU && out_dtype == VIPERA_BF16 && (N / 2) % 8 == 0 &&
        (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
      if ((r = make_out_map(&map_out, out, T, N / 2, true)) != VIPERA_OK) return r;
      p.tma_ending = 1;
    } else if (epilogue == EPI_STORE && out_dtype == VIPERA_F32 && N % 4 == 0 &&
               (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
      if ((r = make_out_map(&map_out, out, T, N, false)) != VIPERA_OK) return r;
      p.tma_ending = 1;
    } else if (epilogue == EPI_RESIDUAL && N % 4 == 0 && (reinterpret_cast<uintptr_t>(resid) & 15) == 0) {
      if ((r = make_out_map(&map_out, resid, T, N, false)) != VIPERA_OK) return r;
      p.tma_ending = 1;
    }
  }
  if (plan.pair) {
    const int launched = plan.bn == 256 ? launch_pairs<256>(map_x, map_y, map_out, p, items, s)
                       : plan.bn == 192 ? launch_pairs<192>(map_x, map_y, map_out, p, items, s)
                                        : launch_pairs<128>(map_x, map_y, map_out, p, items, s);
    if (launched == VIPERA_OK) return launched;
    // The device refused the clusters (nothing has run): from now on blocks alone, this product too.
    cudaGetLastError();
    pair_mode() = 0;
    return run_gemm(A, W, T, N, K, epilogue, bias, out, out_dtype, resid, scratch, scratch_bytes, status, stream, rope);
  }
  if (plan.even_shares) {
    if (plan.bn == 256) return launch_variant<256, false, true>(map_x, map_y, map_out, p, grid, s);
    return launch_variant<128, false, true>(map_x, map_y, map_out, p, grid, s);
  }
  if (!plan.swap) {
    if (plan.bn == 256) return launch_variant<256, false>(map_x, map_y, map_out, p, grid, s);
    if (plan.bn == 192) return launch_variant<192, false>(map_x, map_y, map_out, p, grid, s);
    return launch_variant<128, false>(map_x, map_y, map_out, p, grid, s);
  }
  switch (plan.bn) {
    case 16: return launch_variant<16, true>(map_x, map_y, map_out, p, grid, s);
    case 32: return launch_variant<32, true>(map_x, map_y, map_out, p, grid, s);
    case 64: return launch_variant<64, true>(map_x, map_y, map_out, p, grid, s);
    case 128: return launch_variant<128, true>(map_x, map_y, map_out, p, grid, s);
    default: return launch_variant<256, true>(map_x, map_y, map_out, p, grid, s);
  }
}

VIPERA_API int vipera_gemm_tc(const void* A, const void* W, int T, int N, int K, int epilogue, const float* bias,
                              void* out, int out_dtype, float* resid, float* scratch, size_t scratch_bytes,
                              int* status, void* stream) {
  if (epilogue == EPI_ROPE_CACHE) return VIPERA_BAD_ARGUMENT;  // that ending has an entry point of its own
  return run_gemm(A, W, T, N, K, epilogue, bias, out, out_dtype, resid, scratch, scratch_bytes, status, stream, nullptr);
}

// What the q/k/v ending needs beside the product itself (mirrored by the caller).
struct GemmRope {
  const int* positions;
  const int* token_entry;
  const int* block_table;
  const float* cos_table;
  const float* sin_table;
  void* q_out;
  void* k_pool;
  void* v_pool;
  int table_width, page_size, num_heads, num_kv_heads, head_dim, rope_style, write_cache;
};

VIPERA_API int vipera_gemm_tc_rope_size() { return static_cast<int>(sizeof(GemmRope)); }

// Whether vipera_gemm_tc_rope takes these sizes: heads of 64 or 128 values, whole heads in every
// 128-column step, and either enough tokens for tiles with the tokens on the 128-row side or a
// product whose K is cut.
VIPERA_API int vipera_gemm_tc_rope_takes(int T, int N, int K, int head_dim) {
  if (T <= 0 || K <= 0 || K % 8 || N <= 0) return 0;
  if (head_dim != 64 && head_dim != 128) return 0;
  if (N % head_dim) return 0;
  if (T >= 128 + 64) return 1;
  // fewer tokens: the form with the tokens on the other side, whose split sums' kernel has this
  // ending; where K is not cut there is no such kernel
  const GemmPlan plan = make_plan(T, N, K, sm_count(), EPI_ROPE_CACHE);
  return plan.swap && plan.splits > 1 ? 1 : 0;
}

// The q/k/v product of a step with its ending: out = A . W^T + bias, rotary pairs of the q and k
// heads turned by the tokens' positions, q written to q_out [T, heads * d] and k, v into their
// cache pages (rope_style 0: no rotation).  N = (heads + 2 * kv_heads) * d.
VIPERA_API int vipera_gemm_tc_rope(const void* A, const void* W, int T, int N, int K, const float* bias,
                                   const GemmRope* rope, float* scratch, size_t scratch_bytes, int* status, void* stream) {
  if (!rope || !vipera_gemm_tc_rope_takes(T, N, K, rope->head_dim)) return VIPERA_BAD_SHAPE;
  if (N != (rope->num_heads + 2 * rope->num_kv_heads) * rope->head_dim) return VIPERA_BAD_SHAPE;
  if (!rope->positions || !rope->q_out) return VIPERA_BAD_ARGUMENT;
  if (rope->rope_style == GEMM_ROPE_NEOX && (!rope->cos_table || !rope->sin_table)) return VIPERA_BAD_ARGUMENT;
  if (rope->rope_style != GEMM_ROPE_NEOX && rope->rope_style != GEMM_ROPE_NONE) return VIPERA_BAD_ARGUMENT;
  if (rope->write_cache && (!rope->k_pool || !rope->v_pool || !rope->token_entry || !rope->block_table || rope->page_size <= 0))
    return VIPERA_BAD_ARGUMENT;
  GemmParams p{};
  p.positions = rope->positions;
  p.token_entry = rope->token_entry;
  p.block_table = rope->block_table;
  p.cos_table = rope->cos_table;
  p.sin_table = rope->sin_table;
  p.q_out = static_cast<__nv_bfloat16*>(rope->q_out);
  p.k_pool = static_cast<__nv_bfloat16*>(rope->k_pool);
  p.v_pool = static_cast<__nv_bfloat16*>(rope->v_pool);
  p.table_width = rope->table_width;
  p.page_size = rope->page_size;
  p.num_heads = rope->num_heads;
  p.num_kv_heads = rope->num_kv_heads;
  p.head_dim = rope->head_dim;
  p.rope_style = rope->rope_style;
  p.write_cache = rope->write_cache;
  return run_gemm(A, W, T, N, K, EPI_ROPE_CACHE, bias, nullptr, VIPERA_BF16, nullptr, scratch, scratch_bytes, status, stream, &p);
}

// ---------------------------------------------------------------------------------------
// A wait that runs out, on purpose and harmlessly, so that the way the kernels report it can be
// tested without a fault: one block waits, with the kernels' own bounded wait and a limit of
// `limit` polls, on a barrier in its shared memory that is initialised, that nothing arrives at
// and that no copy is bound to.  Nothing is in flight when the wait gives up; the code lands in
// the status word as it does from the product kernel, and a second thread that waits on the same
// barrier leaves through the block's abort flag as the product kernel's other roles do.
// ---------------------------------------------------------------------------------------
__global__ void wait_probe_kernel(int* status, uint32_t limit) {
  __shared__ uint64_t barrier;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&barrier, 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (threadIdx.x == 0) mbar_wait_limited(&barrier, 0, &abort_flag, status, limit);
  __syncthreads();
  if (threadIdx.x == 32) mbar_wait_limited(&barrier, 0, &abort_flag, status, 1u << 20);
}

VIPERA_API int vipera_gemm_tc_wait_probe(int* status, int limit, void* stream) {
  if (!status || limit < 1 || limit > (1 << 16)) return VIPERA_BAD_ARGUMENT;
  wait_probe_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(status, static_cast<uint32_t>(limit));
  return vipera_launch_status();
}

// After a kernel reported a wait that ran out, flags of partial sums nobody took may still be
// up: this lowers them all (on the stream, after the work already there).
VIPERA_API int vipera_gemm_tc_reset(void* stream) {
  void* flags = nullptr;
  if (cudaGetSymbolAddress(&flags, share_flags_store) != cudaSuccess) return VIPERA_BAD_ARGUMENT;
  return cudaMemsetAsync(flags, 0, sizeof(int) * kMostShares, static_cast<cudaStream_t>(stream)) == cudaSuccess
      ? VIPERA_OK : VIPERA_BAD_ARGUMENT;
}

VIPERA_API const char* vipera_gemm_tc_status_text(int status) { return vipera_status_text(status); }
