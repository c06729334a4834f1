// bfloat16 attention of prompt portions over the paged cache on the fifth-generation tensor
// cores (tcgen05, accumulators in tensor memory), head sizes 64 and 128.
//
// One block serves 128 queries of one entry and one query head and walks the visible keys
// 128 at a time, in the flash form of the reference's online fold
// (crates/vipera-backend-cpu/src/model.rs:2752-2857; definition model.rs:1804-1859):
//
//   scores  S = Q . K^T        tcgen05.mma, 128 x 128 x d, into tensor memory
//   softmax                    one query row per thread: running max and sum in 32-bit,
//                              p = 2^(s * scale * log2 e - max), rounded to bfloat16 into
//                              shared memory
//   output  O += P . V         tcgen05.mma, 128 x d x 128, accumulated in tensor memory;
//                              when a row's max grows, its accumulator is scaled first
//
// The key tiles are dealt to two softmax groups of four warps, even tiles to one and odd tiles
// to the other.  Each group has a score accumulator, a P tile, an output accumulator and a
// running max and sum of its own, so the two folds never wait for one another: while one
// group's P . V runs, the other group computes its exponentials.  The ending joins the two
// partial results the way two splits of the keys are joined:
// O = (O_a 2^(m_a - m) + O_b 2^(m_b - m)) / (l_a 2^(m_a - m) + l_b 2^(m_b - m)).
//
// Roles: warps 0-3 and 4-7 the two softmax groups (and the ending), warp 8 issues the MMAs,
// warps 9-12 bring keys and values through the block table into shared memory, two tiles in
// flight: with TMA, one box per page and half of the head, or one box per 128 rows where the
// pages follow one another in memory (pages of 8, 16, 32, 64 or multiples of 128 keys; the
// copies of four warps' 16-byte cp.async cannot keep enough bytes in flight), else with
// cp.async.  Keys and values share one shared-memory image, 128-byte rows with 16-byte chunks
// XOR-swizzled by the row: for the scores it is read K-major (the contraction runs along the
// head dimension), for the output MN-major (the contraction runs along the keys), so no
// transposed copy of V is made.
//
// Rows of a tile that hold no visible key (before a window, after the causal limit, past the
// written part of the cache) are zero-filled, never read: they may lie in pages the request
// gave back.  Every wait on an mbarrier is bounded; a wait that runs out records an error
// code in the status word and lets every role run to its end.
#include <cuda.h>

#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"

enum { ATTENTION_TC_WAIT_EXPIRED = 3 };


namespace {

constexpr int kQ = 128;                 // queries per block
constexpr int kKeys = 128;              // keys per tile
constexpr int kTileBytes = 128 * 256;   // a [128][128] bfloat16 tile: two halves of [128 rows][128 bytes]; head size 64 fills one
constexpr int kHalfBytes = 128 * 128;
constexpr int kSoftmaxWarps = 8, kLoaderWarps = 4;   // two softmax groups of four warps
constexpr int kGroupThreads = 128;
constexpr int kMmaWarp = kSoftmaxWarps;           // and the next one: an MMA issuer per softmax group
constexpr int kFirstLoaderWarp = kSoftmaxWarps + 2;
constexpr int kThreads = (kSoftmaxWarps + 2 + kLoaderWarps) * 32;
constexpr int kLoaderThreads = kLoaderWarps * 32;
constexpr uint32_t kWaitLimit = 1u << 22;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kMaxSlack = 8.0f;       // in powers of two
// tensor memory columns: a score accumulator and an output accumulator per softmax group
constexpr uint32_t kColsS0 = 0, kColsS1 = 128, kColsO0 = 256, kColsO1 = 384, kTmemCols = 512;

struct Params {
  const __nv_bfloat16* q;      // [tokens, heads, d]
  __nv_bfloat16* out;          // [tokens, heads, d]
  const __nv_bfloat16* k_pool; // [pages, page_size, kv_heads, d]
  const __nv_bfloat16* v_pool;
  const int* entry_starts;     // [entries + 1]
  const int* entry_pos0;       // [entries]
  const int* block_table;      // [entries, table_width]
  int table_width, page_size, num_entries, num_heads, num_kv_heads, window;
  float scale;
  int skip_single;             // entries of one token are left out (the split-key kernel runs them)
  int* status;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
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
__device__ __forceinline__ void mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status) {
  for (uint32_t spin = 0; spin < kWaitLimit; ++spin) {
    if (mbar_try_wait(bar, parity)) return;
    if (spin > 8) __nanosleep(64);  // a waiting role leaves the issue slots to the working ones
    if ((spin & 1023u) == 1023u && *abort_flag) return;
  }
  *abort_flag = 1;
  atomicExch(status, ATTENTION_TC_WAIT_EXPIRED);
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// one box [1 page][rows][1 KV head][64 values] of a cache pool
__device__ __forceinline__ void tma_load_box(void* dst, const CUtensorMap* map, uint64_t* bar, int d0, int kv_head, int slot, int page) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(d0), "r"(kv_head), "r"(slot), "r"(page)
      : "memory");
}
// one box [128 rows of the pool, whatever pages they lie in][1 KV head][64 values]
__device__ __forceinline__ void tma_load_run(void* dst, const CUtensorMap* map, uint64_t* bar, int d0, int kv_head, int row) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(d0), "r"(kv_head), "r"(row)
      : "memory");
}
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tcgen05_mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_load_32(uint32_t taddr, uint32_t (&r)[32]) {
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
// 2^x with the hardware's approximation (exact enough for weights that are rounded to bfloat16);
// 2^(-inf) = 0.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void tmem_store_32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_store_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// A tile in shared memory: halves (columns 0-63 and, where there are more, 64-127) of
// [128 rows][128 bytes], the 16-byte chunks of a row XOR-swizzled by the row (the 128-byte
// swizzle of the tensor cores).
__device__ __forceinline__ uint32_t tile_offset(int row, int chunk /* 0..15 */) {
  return static_cast<uint32_t>((chunk >> 3) * kHalfBytes + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}

// Descriptor of a tile read K-major: rows are the M or N side, the contraction runs along the
// 128-byte rows.  Groups of 8 rows are 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_k_major(uint32_t saddr) {
  uint64_t desc = 0;
  desc |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
  desc |= static_cast<uint64_t>(1) << 16;                 // leading byte offset: unused with this swizzle
  desc |= static_cast<uint64_t>(1024 >> 4) << 32;         // stride byte offset: between groups of 8 rows
  desc |= static_cast<uint64_t>(1) << 46;                 // descriptor version
  desc |= static_cast<uint64_t>(2) << 61;                 // 128-byte swizzle
  return desc;
}
// Descriptor of the same image read MN-major: the 128-byte rows run along the N side (64
// values each, the second 64 in the other half), the contraction runs down the rows.
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t saddr) {
  uint64_t desc = 0;
  desc |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
  desc |= static_cast<uint64_t>(kHalfBytes >> 4) << 16;   // leading byte offset: between the halves (64 values of N)
  desc |= static_cast<uint64_t>(1024 >> 4) << 32;         // stride byte offset: between groups of 8 rows (of the contraction)
  desc |= static_cast<uint64_t>(1) << 46;
  desc |= static_cast<uint64_t>(2) << 61;
  return desc;
}

// One block's work: a tile of 128 queries of an entry (entry < 0: none).
struct Job {
  int entry, tile;
  int token0, tokens_here, pos0;   // the tile's first token in the step, how many it has, the first one's position
};
// Blocks are numbered from the back, and the heads run along x (the index that changes fastest
// as blocks are handed out), so that the tiles with the longest history, of every head, start
// first.  The step's entries are the host's, written before the step: they may be read before
// the kernel waits for the one ahead.
// A warp looks at 32 entries at a time, a lane each (one trip to memory for all of them).
__device__ __forceinline__ Job find_job(const Params& p, int from_the_back, int lane) {
  Job job{-1, 0, 0, 0, 0};
  int remaining = from_the_back;
  for (int e0 = 0; e0 < p.num_entries; e0 += 32) {
    const int e = e0 + lane;
    int start = 0, next = 0, first_position = 0;
    if (e < p.num_entries) {
      start = p.entry_starts[e];
      next = p.entry_starts[e + 1];
      first_position = p.entry_pos0[e];
    }
    const int count = next - start;
    // entries of one token are left to the split-key kernel where the caller says so
    const int tiles = (count <= 0 || (p.skip_single && count == 1)) ? 0 : (count + kQ - 1) / kQ;
    // tiles of the lanes before this one, and of all 32
    int before = tiles;
#pragma unroll
    for (int step = 1; step < 32; step <<= 1) {
      const int other = __shfl_up_sync(0xffffffffu, before, step);
      if (lane >= step) before += other;
    }
    const int all = __shfl_sync(0xffffffffu, before, 31);
    before -= tiles;
    const bool mine = remaining >= before && remaining < before + tiles;
    const unsigned found = __ballot_sync(0xffffffffu, mine);
    if (found) {
      const int owner = __ffs(found) - 1;
      const int tile = remaining - __shfl_sync(0xffffffffu, before, owner);
      const int owner_start = __shfl_sync(0xffffffffu, start, owner), owner_next = __shfl_sync(0xffffffffu, next, owner);
      job.entry = e0 + owner;
      job.tile = tile;
      job.token0 = owner_start + tile * kQ;
      job.tokens_here = min(kQ, owner_next - job.token0);
      job.pos0 = __shfl_sync(0xffffffffu, first_position, owner) + tile * kQ;
      break;
    }
    remaining -= all;
  }
  return job;
}

struct Barriers {
  uint64_t q_full;
  uint64_t k_full[2], k_empty[2], v_full[2], v_empty[2];
  uint64_t v_landed[2];  // TMA path: the boxes of a value tile have arrived (rows outside the visible keys are zeroed after that)
  uint64_t s_full[2], s_empty[2];  // per softmax group
  uint64_t p_full[2], pv_done[2];  // per softmax group
  uint32_t tmem_base;
  int abort_flag;
  Job job;
};

template <int D, bool TMA_KV>
__global__ void __launch_bounds__(kThreads, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                            const __grid_constant__ CUtensorMap k_run_map, const __grid_constant__ CUtensorMap v_run_map,
                            const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* q_tile = smem;
  uint8_t* k_tiles = smem + kTileBytes;       // two tiles
  uint8_t* v_tiles = smem + 3 * kTileBytes;   // two tiles
  uint8_t* p_tiles = smem + 5 * kTileBytes;   // one per softmax group
  Barriers* bars = reinterpret_cast<Barriers*>(smem + 7 * kTileBytes);
  volatile int* abort_flag = &bars->abort_flag;

  static_assert(D == 64 || D == 128, "whole halves of 64 values");
  constexpr int kHalves = D / 64;      // halves of a query, key or value tile
  constexpr int kChunks = D / 8;       // 16-byte chunks of a row
  constexpr int kHalfCols = D / 2;     // output columns of a row one thread writes in the ending
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_launch_dependents();
  // One thread finds the block's tile and hands it to the others through shared memory (each
  // role reading the entry arrays for itself was three dependent trips to memory after the
  // wait); a block without a tile leaves before it sets anything up.
  if (warp == 0) {
    const Job found = find_job(p, static_cast<int>(gridDim.y) - 1 - static_cast<int>(blockIdx.y), lane);
    if (lane == 0) bars->job = found;
  }
  __syncthreads();
  const Job job = bars->job;
  if (job.entry < 0) return;
  const int entry = job.entry;
  const int head = blockIdx.x;
  const int kv_head = head / (p.num_heads / p.num_kv_heads);
  const int token0 = job.token0, tokens_here = job.tokens_here;
  const int pos0 = job.pos0;                                  // position of the tile's first query
  const int first_key = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
  const int end_key = pos0 + tokens_here;                     // one past the last visible key
  const int first_tile = first_key / kKeys;
  const int num_tiles = (end_key + kKeys - 1) / kKeys - first_tile;

  // The pages of a loading warp's first tile are asked for now (the block table is the host's),
  // so that the answer travels while the barriers and the tensor memory are set up.
  int early_page = -1;
  if (TMA_KV && warp >= kFirstLoaderWarp) {
    const int stream_group = (warp - kFirstLoaderWarp) >> 1;
    const int rows_per_box = min(p.page_size, kKeys);
    const int key = (first_tile + stream_group) * kKeys + lane * rows_per_box;
    if (stream_group < num_tiles && lane < kKeys / rows_per_box && key + rows_per_box > first_key && key < end_key)
      early_page = p.block_table[static_cast<size_t>(entry) * p.table_width + key / p.page_size];
  }
  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, kLoaderThreads);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->k_full[i], TMA_KV ? 1 : kLoaderThreads);
      mbar_init(&bars->v_full[i], TMA_KV ? 32 : kLoaderThreads);
      mbar_init(&bars->v_landed[i], 1);
      mbar_init(&bars->k_empty[i], 1);
      mbar_init(&bars->v_empty[i], 1);
      mbar_init(&bars->s_full[i], 1);
      mbar_init(&bars->s_empty[i], kGroupThreads);
      mbar_init(&bars->p_full[i], kGroupThreads);
      mbar_init(&bars->pv_done[i], 1);
    }
    bars->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kMmaWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)), "r"(kTmemCols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  // (Each role waits for the kernels ahead where it first needs what they wrote: the loaders
  // after they have looked up their first pages, the softmax warps at once; the issuing warps
  // touch shared and tensor memory only.)

  if (warp < kSoftmaxWarps) {
    // ---------------- softmax and ending: thread = query row, group = every other key tile ----------------
    // Warps w and w + 4 share the rows 32 (w % 4) .. + 31 (a warp reaches only its quarter of
    // the tensor memory's lanes); they belong to different groups and so work on different key
    // tiles, independently, and fill each other's waits.
    pdl_wait();   // the output belongs to earlier kernels until now
    const int quarter = warp & 3, group = warp >> 2;
    const int row = quarter * 32 + lane;
    const int position = pos0 + row;
    const int row_limit = row < tokens_here ? position : -1;  // rows past the entry's end see nothing
    const int row_first = p.window > 0 ? max(0, position - p.window + 1) : 0;
    const float scale_log2 = p.scale * kLog2e;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const uint32_t s_addr = lane_base + (group ? kColsS1 : kColsS0);
    const uint32_t o_addr = lane_base + (group ? kColsO1 : kColsO0);
    uint8_t* p_tile = p_tiles + group * kTileBytes;
    const int group_tiles = (num_tiles - group + 1) / 2;  // tiles group, group + 2, ...
    float row_max = -INFINITY, row_sum = 0.0f;
    for (int i = 0; i < group_tiles; ++i) {
      const int j = 2 * i + group;
      const int key0 = (first_tile + j) * kKeys;
      mbar_wait(&bars->s_full[group], static_cast<uint32_t>(i) & 1u, abort_flag, p.status);
      tcgen05_fence_after();
      // does any row of this block need a mask in this tile?
      const bool edge = key0 + kKeys - 1 > pos0 || (p.window > 0 && key0 < pos0 + tokens_here - p.window + 1) || tokens_here < kQ;
      // first pass over the row's 128 scores: the largest visible one
      float tile_max = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < kKeys; c += 64) {
        uint32_t sv[64];
        tmem_load_32_nowait(s_addr + c, *reinterpret_cast<uint32_t(*)[32]>(&sv[0]));
        tmem_load_32_nowait(s_addr + c + 32, *reinterpret_cast<uint32_t(*)[32]>(&sv[32]));
        tmem_load_wait();
        if (edge) {
#pragma unroll
          for (int k = 0; k < 64; ++k) {
            const int key = key0 + c + k;
            if (key < row_first || key > row_limit) sv[k] = __float_as_uint(-INFINITY);
          }
        }
        // four chains, so that the 128 comparisons do not wait for one another
        float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
        for (int k = 0; k < 64; k += 4) {
          m0 = fmaxf(m0, __uint_as_float(sv[k]));
          m1 = fmaxf(m1, __uint_as_float(sv[k + 1]));
          m2 = fmaxf(m2, __uint_as_float(sv[k + 2]));
          m3 = fmaxf(m3, __uint_as_float(sv[k + 3]));
        }
        tile_max = fmaxf(tile_max, fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)));
      }
      tile_max *= scale_log2;
      // The running max only has to keep the exponentials in range: it follows the row's true
      // max when that has grown by more than kMaxSlack (weights then stay below 2^kMaxSlack,
      // and the final division by the sum cancels the common factor).  Most tiles thus leave the
      // output accumulator as it is.
      float new_max = row_max;
      if (tile_max > row_max + kMaxSlack || row_max == -INFINITY) new_max = fmaxf(row_max, tile_max);
      const float alpha = new_max == row_max ? 1.0f : fast_exp2(row_max - new_max);
      row_max = new_max;
      row_sum *= alpha;
      // the group's output accumulator and P tile are free once the product of its tile before is done
      if (i > 0) mbar_wait(&bars->pv_done[group], static_cast<uint32_t>(i - 1) & 1u, abort_flag, p.status);
      tcgen05_fence_after();
      if (i > 0 && __any_sync(0xffffffffu, alpha != 1.0f)) {
#pragma unroll 1
        for (int c = 0; c < D; c += 32) {
          uint32_t v[32];
          tmem_load_32(o_addr + c, v);
#pragma unroll
          for (int k = 0; k < 32; ++k) v[k] = __float_as_uint(__uint_as_float(v[k]) * alpha);
          tmem_store_32(o_addr + c, v);
        }
        tmem_store_wait();
      }
      // second pass: p = 2^(s * scale * log2 e - max), summed in 32-bit, rounded to bfloat16 into the P tile
      float tile_sum = 0.0f, tile_sum_b = 0.0f;
      const float shift = row_max == -INFINITY ? 0.0f : row_max;  // a row without visible keys: 2^(-inf) = 0 everywhere
#pragma unroll 1
      for (int c = 0; c < kKeys; c += 64) {
        uint32_t sv[64];
        tmem_load_32_nowait(s_addr + c, *reinterpret_cast<uint32_t(*)[32]>(&sv[0]));
        tmem_load_32_nowait(s_addr + c + 32, *reinterpret_cast<uint32_t(*)[32]>(&sv[32]));
        tmem_load_wait();
        if (c + 64 == kKeys) {
          // the scores are in registers: the accumulator is free for the group's next tile
          tcgen05_fence_before();
          mbar_arrive(&bars->s_empty[group]);
        }
        if (edge) {
#pragma unroll
          for (int k = 0; k < 64; ++k) {
            const int key = key0 + c + k;
            if (key < row_first || key > row_limit) sv[k] = __float_as_uint(-INFINITY);
          }
        }
#pragma unroll
        for (int k8 = 0; k8 < 64; k8 += 8) {
          uint32_t packed[4];
#pragma unroll
          for (int k = 0; k < 8; k += 2) {
            const float p0 = fast_exp2(fmaf(__uint_as_float(sv[k8 + k]), scale_log2, -shift));
            const float p1 = fast_exp2(fmaf(__uint_as_float(sv[k8 + k + 1]), scale_log2, -shift));
            tile_sum += p0;
            tile_sum_b += p1;
            __nv_bfloat162 pair = __floats2bfloat162_rn(p0, p1);
            packed[k >> 1] = *reinterpret_cast<uint32_t*>(&pair);
          }
          *reinterpret_cast<uint4*>(p_tile + tile_offset(row, (c + k8) >> 3)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        }
      }
      row_sum += tile_sum + tile_sum_b;
      // P is written: hand it over to the MMA warp
      tcgen05_fence_before();
      fence_async_shared();
      mbar_arrive(&bars->p_full[group]);
    }
    // ---------------- ending: join the two groups' folds, out = O / sum ----------------
    if (num_tiles > 0) {
      // A group's last product must be done before its P tile carries the group's max and sum
      // to the other group (and before anyone reads its output accumulator).
      if (group_tiles > 0) mbar_wait(&bars->pv_done[group], static_cast<uint32_t>(group_tiles - 1) & 1u, abort_flag, p.status);
      tcgen05_fence_after();
      float2* told = reinterpret_cast<float2*>(p_tile);
      told[row] = make_float2(row_max, row_sum);
      tcgen05_fence_before();
      asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory");
      const float2 other = reinterpret_cast<const float2*>(p_tiles + (group ^ 1) * kTileBytes)[row];
      tcgen05_fence_after();
      const bool other_has_tiles = group == 1 || num_tiles > 1;  // the other group's accumulator holds numbers
      const float joint_max = fmaxf(row_max, other.x);
      const float own_weight = row_max == -INFINITY ? 0.0f : fast_exp2(row_max - joint_max);
      const float other_weight = other.x == -INFINITY ? 0.0f : fast_exp2(other.x - joint_max);
      const float joint_sum = row_sum * own_weight + other.y * other_weight;
      const float inverse = joint_sum > 0.0f ? 1.0f / joint_sum : 0.0f;
      const float own_factor = own_weight * inverse, other_factor = other_weight * inverse;
      const uint32_t other_o = lane_base + (group ? kColsO0 : kColsO1);
      const bool own_has_tiles = group_tiles > 0;
      // each group writes half of the row's columns
      const int col0 = group * kHalfCols;
      // The tile leaves through shared memory (the query tile's space: every product that read
      // it is done once both groups' last output products are), so that a warp's store covers two
      // whole rows of the output.  A thread writing its own row straight to memory makes 32 lines
      // per store instruction; the block's eight warps then queue for 5,000 clocks.
      uint8_t* staged = q_tile;
#pragma unroll 1
      for (int c = 0; c < kHalfCols; c += 32) {
        uint32_t v[32], w[32];
        if (own_has_tiles) tmem_load_32_nowait(o_addr + col0 + c, v);
        if (other_has_tiles) tmem_load_32_nowait(other_o + col0 + c, w);
        tmem_load_wait();
        float joined[32];
#pragma unroll
        for (int k = 0; k < 32; ++k) {
          joined[k] = own_has_tiles ? __uint_as_float(v[k]) * own_factor : 0.0f;
          if (other_has_tiles) joined[k] = fmaf(__uint_as_float(w[k]), other_factor, joined[k]);
        }
#pragma unroll
        for (int k = 0; k < 32; k += 8) {
          uint4 packed;
          __nv_bfloat162* halves = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
          for (int h = 0; h < 4; ++h) halves[h] = __floats2bfloat162_rn(joined[k + 2 * h], joined[k + 2 * h + 1]);
          *reinterpret_cast<uint4*>(staged + tile_offset(row, (col0 + c + k) >> 3)) = packed;
        }
      }
      asm volatile("bar.sync 6, 256;" ::: "memory");
      if (!*abort_flag) {
        __nv_bfloat16* out_tile = p.out + (static_cast<size_t>(token0) * p.num_heads + head) * D;
        const size_t row_pitch = static_cast<size_t>(p.num_heads) * D;
#pragma unroll
        for (int pass = 0; pass < kQ * kChunks / (kSoftmaxWarps * 32); ++pass) {
          const int id = pass * (kSoftmaxWarps * 32) + static_cast<int>(threadIdx.x);   // neighbours copy one row
          const int r = id / kChunks, chunk = id % kChunks;
          if (r < tokens_here)
            *reinterpret_cast<uint4*>(out_tile + r * row_pitch + chunk * 8) = *reinterpret_cast<const uint4*>(staged + tile_offset(r, chunk));
        }
      }
    }
    tcgen05_fence_before();
  } else if (warp < kFirstLoaderWarp) {
    // ---------------- MMA issuers, one per softmax group ----------------
    const int g = warp - kMmaWarp;
    const int group_tiles = (num_tiles - g + 1) / 2;
    if (lane == 0 && group_tiles > 0) {
      // instruction descriptors: bf16 x bf16 -> f32, M = 128; N = 128 keys and B K-major for the
      // scores, N = d and B MN-major for the output
      constexpr uint32_t kIdescCommon = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(kQ >> 4) << 24);
      constexpr uint32_t kIdescS = kIdescCommon | (static_cast<uint32_t>(kKeys >> 3) << 17);
      constexpr uint32_t kIdescO = kIdescCommon | (static_cast<uint32_t>(D >> 3) << 17) | (1u << 16);
      const uint32_t q_addr = smem_u32(q_tile);
      // Tile j belongs to softmax group j & 1 and is that group's tile number j >> 1; its keys
      // and values lie in buffer j & 1 as well.  The two groups drift against one another, so
      // each has an issuer of its own, which follows its group's order of events: the scores
      // of the next tile as soon as the group has taken the current ones into registers (in the
      // middle of its second pass), then the output product of the current tile when P is written.
      const uint32_t k_addr = smem_u32(k_tiles + g * kTileBytes);
      const uint32_t v_addr = smem_u32(v_tiles + g * kTileBytes);
      const uint32_t p_addr = smem_u32(p_tiles + g * kTileBytes);
      const uint32_t s_tmem = tmem_base + (g ? kColsS1 : kColsS0);
      const uint32_t o_tmem = tmem_base + (g ? kColsO1 : kColsO0);
      auto issue_scores = [&](int i) {   // the group's tile i
        mbar_wait(&bars->k_full[g], static_cast<uint32_t>(i) & 1u, abort_flag, p.status);
        if (i > 0) mbar_wait(&bars->s_empty[g], static_cast<uint32_t>(i - 1) & 1u, abort_flag, p.status);
        tcgen05_fence_after();
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          // 16 values further along the row: 32 bytes inside a half, the other half after 4 steps
          const uint32_t offset = static_cast<uint32_t>((ks >> 2) * kHalfBytes + (ks & 3) * 32);
          tcgen05_mma_bf16(s_tmem, desc_k_major(q_addr + offset), desc_k_major(k_addr + offset), kIdescS, ks > 0 ? 1u : 0u);
        }
        tcgen05_commit(&bars->k_empty[g]);
        tcgen05_commit(&bars->s_full[g]);
      };
      mbar_wait(&bars->q_full, 0, abort_flag, p.status);
      issue_scores(0);
      for (int i = 0; i < group_tiles; ++i) {
        // With TMA the next keys land without a loader thread's doing, so their scores can be
        // asked for first.  The cp.async loaders hand tiles over in one fixed order, in which
        // they wait for this tile's output product before they hand over the next keys: there
        // the output product goes first.
        if (TMA_KV && i + 1 < group_tiles) issue_scores(i + 1);
        const int key0 = (first_tile + 2 * i + g) * kKeys;
        const bool zeroed_rows = key0 < first_key || key0 + kKeys > end_key;  // then a loader warp hands the tile over (as the cp.async path always does)
        mbar_wait(&bars->p_full[g], static_cast<uint32_t>(i) & 1u, abort_flag, p.status);
        mbar_wait((zeroed_rows || !TMA_KV) ? &bars->v_full[g] : &bars->v_landed[g], static_cast<uint32_t>(i) & 1u, abort_flag, p.status);
        tcgen05_fence_after();
#pragma unroll
        for (int ks = 0; ks < kKeys / 16; ++ks) {
          // P: 16 keys further along its rows; V: 16 rows (two groups of 8) further down
          const uint32_t p_offset = static_cast<uint32_t>((ks >> 2) * kHalfBytes + (ks & 3) * 32);
          tcgen05_mma_bf16(o_tmem, desc_k_major(p_addr + p_offset), desc_mn_major(v_addr + ks * 2048), kIdescO,
                           (i > 0 || ks > 0) ? 1u : 0u);
        }
        tcgen05_commit(&bars->v_empty[g]);
        tcgen05_commit(&bars->pv_done[g]);
        if (!TMA_KV && i + 1 < group_tiles) issue_scores(i + 1);
      }
    }
    tcgen05_fence_before();
  } else {
    // ---------------- loaders: queries once, then keys and values tile by tile ----------------
    const int t = threadIdx.x - kFirstLoaderWarp * 32;  // 0..127
    if (num_tiles > 0) {
      const int* table = p.block_table + static_cast<size_t>(entry) * p.table_width;
      auto load_queries = [&]() {
        for (int index = t; index < kQ * kChunks; index += kLoaderThreads) {
          const int row = index / kChunks, chunk = index % kChunks;
          const bool valid = row < tokens_here;
          const __nv_bfloat16* src = p.q + (static_cast<size_t>(token0 + (valid ? row : 0)) * p.num_heads + head) * D + chunk * 8;
          cp_async_16(smem_u32(q_tile) + tile_offset(row, chunk), src, valid);
        }
        cp_async_commit();
      };
      if constexpr (TMA_KV) {
        // ---- keys and values by TMA: the first loader warp issues one box per page and half ----
        const int rows_per_box = min(p.page_size, kKeys);
        const int boxes = kKeys / rows_per_box;
        const int loader_warp = t >> 5;
        // the page a lane's box lies in (-1: no visible key in it, or no such box)
        auto look_up = [&](int j) {
          const int key = (first_tile + j) * kKeys + lane * rows_per_box;
          int page = -1;
          if (lane < boxes && key + rows_per_box > first_key && key < end_key) page = table[key / p.page_size];
          return page;
        };
        auto issue_boxes = [&](int j, int page, const CUtensorMap* map, const CUtensorMap* run_map, uint8_t* tile, uint64_t* landed) {
          const int key = (first_tile + j) * kKeys + lane * rows_per_box;
          // a box is fetched when it holds a visible key; the others stay as they are (keys) or are zeroed (values)
          const unsigned fetched = __ballot_sync(0xffffffffu, page >= 0);
          // Pages that follow one another in memory (what a fresh request gets) are fetched as one
          // run of 128 rows: two boxes instead of two per page.  Rows of the run past the pages
          // wanted are rows of other pages or past the pool; they are masked (keys) or zeroed (values).
          if (boxes > 1) {
            const int page0 = __shfl_sync(0xffffffffu, page, 0);
            const bool in_run = page < 0 || page == page0 + lane;
            const unsigned wanted = fetched;
            // the wanted boxes must be the first ones, one after another
            if (page0 >= 0 && __all_sync(0xffffffffu, in_run) && (wanted & (wanted + 1u)) == 0u) {
              if (lane == 0) {
                mbar_expect_tx(landed, static_cast<uint32_t>(kKeys * D * 2));
#pragma unroll
                for (int h = 0; h < kHalves; ++h) tma_load_run(tile + h * kHalfBytes, run_map, landed, 64 * h, kv_head, page0 * p.page_size);
              }
              return;
            }
          }
          if (lane == 0) mbar_expect_tx(landed, static_cast<uint32_t>(__popc(fetched) * rows_per_box * D * 2));
          __syncwarp();
          if (page >= 0) {
            uint8_t* dst = tile + lane * rows_per_box * 128;
#pragma unroll
            for (int h = 0; h < kHalves; ++h) tma_load_box(dst + h * kHalfBytes, map, landed, 64 * h, kv_head, key % p.page_size, page);
          }
        };
        // Four streams with waits of their own, a loader warp each: the keys and the values of
        // either softmax group's tiles (a key buffer is free once the scores of the group's tile
        // before are computed, a value buffer once that tile's output product is done, which is
        // much later; and the groups drift against one another).  The block table entries of a
        // stream's next tile are read before the wait for this tile's buffer, so that the read
        // adds to no wait.
        const int stream_group = loader_warp >> 1;
        const bool values = (loader_warp & 1) != 0;
        const int stream_tiles = (num_tiles - stream_group + 1) / 2;
        // (the block table is the host's: the first look-up does not wait for the kernels ahead)
        int pages = early_page;   // = look_up(stream_group), asked for before the set-up
        pdl_wait();
        load_queries();
        auto issue_tile = [&](int i) {   // the group's tile i
          const int j = 2 * i + stream_group;
          const int page = pages;
          if (i + 1 < stream_tiles) pages = look_up(j + 2);
          uint64_t* empty = values ? &bars->v_empty[stream_group] : &bars->k_empty[stream_group];
          if (i >= 1) mbar_wait(empty, static_cast<uint32_t>(i - 1) & 1u, abort_flag, p.status);
          if (!*abort_flag) {
            if (values) issue_boxes(j, page, &v_map, &v_run_map, v_tiles + stream_group * kTileBytes, &bars->v_landed[stream_group]);
            else issue_boxes(j, page, &k_map, &k_run_map, k_tiles + stream_group * kTileBytes, &bars->k_full[stream_group]);
          }
        };
        if (stream_tiles > 0) issue_tile(0);
        cp_async_wait<0>();
        fence_async_shared();
        mbar_arrive(&bars->q_full);
        for (int i = 0; i < stream_tiles; ++i) {
          if (i >= 1) issue_tile(i);
          if (!values) continue;
          // A value row that holds no visible key must be zero: its weight is zero, but what lies
          // in the cache there may be anything.  Only the first tiles of a window and the last
          // tile have such rows; the MMA issuer takes every other tile as it lands.
          const int key0 = (first_tile + 2 * i + stream_group) * kKeys;
          if (key0 < first_key || key0 + kKeys > end_key) {
            mbar_wait(&bars->v_landed[stream_group], static_cast<uint32_t>(i) & 1u, abort_flag, p.status);
            uint8_t* tile = v_tiles + stream_group * kTileBytes;
            for (int r = lane; r < kKeys; r += 32) {
              const int key = key0 + r;
              if (key < first_key || key >= end_key) {
#pragma unroll
                for (int chunk = 0; chunk < kChunks; ++chunk) *reinterpret_cast<uint4*>(tile + tile_offset(r, chunk)) = make_uint4(0, 0, 0, 0);
              }
            }
            fence_async_shared();
          }
          mbar_arrive(&bars->v_full[stream_group]);
        }
      } else {
      pdl_wait();
      load_queries();
      // A tile is copied in passes of 8 rows (16 with head size 64): consecutive threads copy the
      // chunks of one cache row, so that global reads are whole rows.  Where a page holds a power
      // of two of keys, page and slot come from a shift and a mask.
      constexpr int kRowsPerPass = kLoaderThreads / kChunks, kPasses = kKeys / kRowsPerPass;
      const int page_shift = (p.page_size & (p.page_size - 1)) == 0 ? 31 - __clz(p.page_size) : -1;
      const long long row_stride = static_cast<long long>(p.num_kv_heads) * D;
      auto copy_tile = [&](int j, const __nv_bfloat16* pool, uint32_t dst) {
        const int key_base = (first_tile + j) * kKeys + t / kChunks;
        const int chunk = t % kChunks;
        const __nv_bfloat16* base = pool + static_cast<long long>(kv_head) * D + chunk * 8;
        // the block table first (independent reads), then the copies
        int pages[kPasses];
#pragma unroll
        for (int pass = 0; pass < kPasses; ++pass) {
          const int key = key_base + pass * kRowsPerPass;
          pages[pass] = -1;
          if (key >= first_key && key < end_key) pages[pass] = table[page_shift >= 0 ? key >> page_shift : key / p.page_size];
        }
#pragma unroll
        for (int pass = 0; pass < kPasses; ++pass) {
          const int key = key_base + pass * kRowsPerPass;
          const int slot = page_shift >= 0 ? key & (p.page_size - 1) : key % p.page_size;
          const bool valid = pages[pass] >= 0;
          const long long at = valid ? (static_cast<long long>(pages[pass]) * p.page_size + slot) * row_stride : 0;
          cp_async_16(dst + tile_offset(pass * kRowsPerPass + t / kChunks, chunk), base + at, valid);
        }
        cp_async_commit();
      };
      auto issue_keys = [&](int j) {    // waits until the scores of tile j - 2 have read the buffer
        const int buffer = j & 1;
        if (j >= 2) mbar_wait(&bars->k_empty[buffer], static_cast<uint32_t>((j >> 1) - 1) & 1u, abort_flag, p.status);
        copy_tile(j, p.k_pool, smem_u32(k_tiles + buffer * kTileBytes));
      };
      auto issue_values = [&](int j) {  // waits until the output product of tile j - 2 has read the buffer
        const int buffer = j & 1;
        if (j >= 2) mbar_wait(&bars->v_empty[buffer], static_cast<uint32_t>((j >> 1) - 1) & 1u, abort_flag, p.status);
        copy_tile(j, p.v_pool, smem_u32(v_tiles + buffer * kTileBytes));
      };
      auto wait_pending = [&](int groups) {  // until at most `groups` of this thread's copy groups are in flight
        if (groups <= 0) cp_async_wait<0>();
        else if (groups == 1) cp_async_wait<1>();
        else if (groups == 2) cp_async_wait<2>();
        else if (groups == 3) cp_async_wait<3>();
        else cp_async_wait<4>();
      };
      // Copy groups are committed in this order: Q, K0, V0, K1, V1, then K(j+2) in pass j and
      // V(j+2) in pass j + 1.  A pass hands over what has landed before it waits for a buffer
      // to be free: the products that free it need the data handed over.
      issue_keys(0);
      issue_values(0);
      if (num_tiles > 1) { issue_keys(1); issue_values(1); }
      wait_pending(num_tiles > 1 ? 4 : 2);
      fence_async_shared();
      mbar_arrive(&bars->q_full);
      for (int j = 0; j < num_tiles; ++j) {
        const int buffer = j & 1;
        // groups committed after K_j so far: V_j, K_j+1 (and V_1 in pass 0)
        const int after_keys = j == 0 ? (num_tiles > 1 ? 3 : 1) : (j + 1 < num_tiles ? 2 : 1);
        wait_pending(after_keys);
        fence_async_shared();
        mbar_arrive(&bars->k_full[buffer]);
        wait_pending(after_keys - 1);
        fence_async_shared();
        mbar_arrive(&bars->v_full[buffer]);
        if (j >= 1 && j + 1 < num_tiles) issue_values(j + 1);
        if (j + 2 < num_tiles) issue_keys(j + 2);
      }
      }
    }
  }
  __syncthreads();
  if (warp == kMmaWarp) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols));
  }
}

constexpr int kSmemBytes = 7 * kTileBytes + 1024 /* alignment */ + static_cast<int>(sizeof(Barriers)) + 64;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
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

// Pages the TMA path takes: boxes of whole pages (or of 128 rows of a longer page) that start
// on a multiple of 8 rows of the tile.
bool tma_takes_page(int page_size) {
  return page_size % 8 == 0 && (kKeys % page_size == 0 || page_size % kKeys == 0);
}

// A cache pool [pages, page_size, kv_heads, d] as TMA reads it: boxes of one page's rows
// (at most 128) of one KV head and 64 values, 128-byte swizzle.  Maps are kept by pool.
// `run`: the same pool as rows that follow one another whatever page they are in,
// [pages * page_size, kv_heads, d], in boxes of 128 rows.
// The map is copied out under the lock: the table may be emptied by a later call.
bool pool_map(const void* pool, int pages, int page_size, int kv_heads, int head_dim, bool run, CUtensorMap* out) {
  static std::map<std::tuple<const void*, int, int, int, int, bool>, CUtensorMap> kept;
  static std::mutex guard;
  std::lock_guard<std::mutex> lock(guard);
  const auto key = std::make_tuple(pool, pages, page_size, kv_heads, head_dim, run);
  const cuuint64_t d = static_cast<cuuint64_t>(head_dim);
  auto found = kept.find(key);
  if (found != kept.end()) {
    *out = found->second;
    return true;
  }
  EncodeTiledFn encode = encode_tiled_fn();
  if (!encode || (reinterpret_cast<uintptr_t>(pool) & 15)) return false;
  CUtensorMap map;
  if (run) {
    cuuint64_t dims[3] = {d, static_cast<cuuint64_t>(kv_heads),
                          static_cast<cuuint64_t>(pages) * page_size};
    cuuint64_t strides[2] = {d * 2, static_cast<cuuint64_t>(kv_heads) * d * 2};
    cuuint32_t box[3] = {64, 1, static_cast<cuuint32_t>(kKeys)};
    cuuint32_t elem[3] = {1, 1, 1};
    CUresult r = encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(pool), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return false;
    if (kept.size() > 4096) kept.clear();
    kept.emplace(key, map);
    *out = map;
    return true;
  }
  cuuint64_t dims[4] = {d, static_cast<cuuint64_t>(kv_heads), static_cast<cuuint64_t>(page_size),
                        static_cast<cuuint64_t>(pages)};
  cuuint64_t strides[3] = {d * 2, static_cast<cuuint64_t>(kv_heads) * d * 2,
                           static_cast<cuuint64_t>(page_size) * kv_heads * d * 2};
  cuuint32_t box[4] = {64, 1, static_cast<cuuint32_t>(page_size < kKeys ? page_size : kKeys), 1};
  cuuint32_t elem[4] = {1, 1, 1, 1};
  CUresult r = encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(pool), dims, strides, box, elem,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  if (kept.size() > 4096) kept.clear();
  kept.emplace(key, map);
  *out = map;
  return true;
}

template <int D, bool TMA_KV>
int launch_attention(const CUtensorMap& k_map, const CUtensorMap& v_map, const CUtensorMap& k_run_map,
                     const CUtensorMap& v_run_map, const Params& p, dim3 grid, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc_kernel<D, TMA_KV>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  return vipera_launch(attention_prefill_tc_kernel<D, TMA_KV>, grid, dim3(kThreads), kSmemBytes, stream, k_map, v_map, k_run_map,
                       v_run_map, p);
}

}  // namespace

// Attention of a step with portions of any length, head size 64 or 128 (see attention_mma.cu for the
// meaning of the arguments; `num_pages` is the pools' first extent).  `status` is a device word
// that must be 0 before the launch; it is non-zero afterwards when a bounded wait inside the
// kernel ran out.
VIPERA_API int vipera_attention_prefill_tc(const void* q, void* out, const void* k_pool, const void* v_pool,
                                           const int* entry_starts, const int* entry_pos0, const int* block_table,
                                           int table_width, int page_size, int num_entries, int num_tokens,
                                           int num_heads, int num_kv_heads, int head_dim, float scale, int window,
                                           int num_pages, int skip_single, int* status, void* stream) {
  if (num_tokens <= 0 || num_entries <= 0) return VIPERA_OK;
  if ((head_dim != 64 && head_dim != 128) || num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads || page_size <= 0 || num_pages <= 0)
    return VIPERA_BAD_SHAPE;
  if (!status) return VIPERA_BAD_ARGUMENT;
  Params p{};
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.k_pool = static_cast<const __nv_bfloat16*>(k_pool);
  p.v_pool = static_cast<const __nv_bfloat16*>(v_pool);
  p.entry_starts = entry_starts;
  p.entry_pos0 = entry_pos0;
  p.block_table = block_table;
  p.table_width = table_width;
  p.page_size = page_size;
  p.num_entries = num_entries;
  p.num_heads = num_heads;
  p.num_kv_heads = num_kv_heads;
  p.window = window;
  p.scale = scale;
  p.skip_single = skip_single;
  p.status = status;
  // at most one partly filled tile per entry beyond the full ones
  dim3 grid(num_heads, (num_tokens + kQ - 1) / kQ + num_entries);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (tma_takes_page(page_size) && std::getenv("VIPERA_ATTENTION_NO_TMA") == nullptr) {
    CUtensorMap k_map, v_map, k_run, v_run;
    if (pool_map(k_pool, num_pages, page_size, num_kv_heads, head_dim, false, &k_map) &&
        pool_map(v_pool, num_pages, page_size, num_kv_heads, head_dim, false, &v_map) &&
        pool_map(k_pool, num_pages, page_size, num_kv_heads, head_dim, true, &k_run) &&
        pool_map(v_pool, num_pages, page_size, num_kv_heads, head_dim, true, &v_run))
      return head_dim == 64 ? launch_attention<64, true>(k_map, v_map, k_run, v_run, p, grid, s)
                            : launch_attention<128, true>(k_map, v_map, k_run, v_run, p, grid, s);
  }
  CUtensorMap none{};
  return head_dim == 64 ? launch_attention<64, false>(none, none, none, none, p, grid, s)
                        : launch_attention<128, false>(none, none, none, none, p, grid, s);
}

VIPERA_API const char* vipera_attention_tc_status_text(int status) { return vipera_status_text(status); }
