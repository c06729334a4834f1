// Products of a bfloat16 weight matrix with the few tokens of a decode step (up to 32):
// out[T, N] = act[T, K] . W[N, K]^T, every weight byte read from HBM once, straight into
// registers, and multiplied on the tensor cores (mma.sync m16n8k16) with 32-bit accumulation.
//
// At these sizes a step is bound by the weight stream and by the number of kernels in the
// chain, so this kernel takes the work of its neighbours with it:
//   * in front: RMSNorm of the 32-bit residual stream.  Every block needs all activations
//     anyway; it normalises the few rows itself while it stages them in shared memory
//     (rounded to bfloat16 there, as the separate norm kernel would store them);
//   * behind: bias, the residual addition, SwiGLU, or (for the q/k/v product) the rotary
//     encoding and the write of keys and values into their cache pages.
// The reference's decode path is likewise one weight read for all rows of the batch
// (crates/vipera-backend-cpu/src/model.rs:1005-1025) with norm and activation fused into
// the activation preparation of the next product (crates/vipera-backend-cpu/src/quant.rs:578-603,
// `Fusion::{Norm,Silu}`).
//
// Layout of the work.  A block owns 16 output rows, chosen so that the ending needs no other
// block: 16 consecutive rows for plain endings; 8 gate rows and the 8 up rows of the same
// features for SwiGLU; rows i..i+7 and i+d/2..i+d/2+7 of one head (the two halves of rotary
// pairs) for the q/k/v product.  Its warps split K; each lane loads 16 bytes (8 consecutive
// k) of two rows per step, which are, word for word, the A operands of two MMAs: the
// instruction's k slots are assigned to memory's k in the order the loads deliver them, and
// the activations in shared memory are read with the same assignment, so no value is ever
// unpacked or shuffled.  The warps' partial sums meet in shared memory and are added in warp
// order, so a result does not depend on timing or on the number of tokens.
#include "common.cuh"

enum GemvEpilogue { GEMV_STORE = 0, GEMV_RESIDUAL = 1, GEMV_SWIGLU = 2, GEMV_ROPE_CACHE = 3 };
enum RopeStyle { ROPE_NONE = 0, ROPE_NEOX = 1 };

struct GemvParams {
  const __nv_bfloat16* weight;  // [N, K]
  int N, K, T;
  // input: either the 32-bit residual stream with a norm in front, or bfloat16 activations
  const float* x32;             // [*, K]
  const float* norm_weight;     // [K]
  float eps;
  const int* rows;              // optional: token t reads x32[rows[t]]
  const __nv_bfloat16* a16;     // [T, K]
  int epilogue;
  const float* bias;            // [N] or null
  void* out;                    // STORE: [T, N]; SWIGLU: [T, N/2]
  int out_dtype;
  float* resid;                 // RESIDUAL: [T, N]
  // ROPE_CACHE
  int num_heads, num_kv_heads, head_dim, rope_style;
  const int* positions;
  const float* cos_table;
  const float* sin_table;
  __nv_bfloat16* q_out;         // [T, heads * d]
  __nv_bfloat16* k_pool;
  __nv_bfloat16* v_pool;
  const int* token_entry;
  const int* block_table;
  int table_width, page_size, write_cache;
};

constexpr int kGemvMaxShared = 200 * 1024;
constexpr int kActPadBytes = 64;  // between token rows in shared memory, against bank conflicts

__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// The two rows a lane's accumulators (c0,c1) and (c2,c3) belong to, for tile `tile`, lane group g.
__device__ __forceinline__ void tile_rows(const GemvParams& p, int tile, int g, int* row_lo, int* row_hi) {
  if (p.epilogue == GEMV_SWIGLU) {
    *row_lo = (tile >> 1) * 32 + (tile & 1) * 8 + g;   // gate row
    *row_hi = *row_lo + 16;                            // up row of the same feature
  } else if (p.epilogue == GEMV_ROPE_CACHE) {
    const int per_head = p.head_dim >> 4;              // tiles per head
    *row_lo = (tile / per_head) * p.head_dim + (tile % per_head) * 8 + g;
    *row_hi = *row_lo + (p.head_dim >> 1);
  } else {
    *row_lo = tile * 16 + g;
    *row_hi = *row_lo + 8;
  }
}

// What the ending of one (row pair, token) result needs besides the two sums, fetched ahead of
// the products: bias values, the rotation's cosine and sine, where the result goes.  Everything
// read here was written before the step began (biases, tables, the step's positions and block
// tables), so it may be fetched before the kernel waits for the kernels ahead of it; the ending
// itself then touches memory only to store (or to add, without reading back).
struct Ending {
  float bias_lo, bias_hi, cosine, sine;
  void* dst;        // STORE, SWIGLU: the output element; RESIDUAL: the stream's element of row_lo; ROPE: the head's row
  int active;       // 0: nothing to write (a value that is not cached)
  int rotate;
};

__device__ __forceinline__ Ending prepare_ending(const GemvParams& p, int row_lo, int row_hi, int t) {
  Ending e;
  e.bias_lo = e.bias_hi = 0.0f;
  e.cosine = 1.0f;
  e.sine = 0.0f;
  e.dst = nullptr;
  e.active = 1;
  e.rotate = 0;
  const bool has_hi = row_hi < p.N;
  if (p.epilogue == GEMV_STORE) {
    if (p.bias) { e.bias_lo = p.bias[row_lo]; if (has_hi) e.bias_hi = p.bias[row_hi]; }
  } else if (p.epilogue == GEMV_ROPE_CACHE) {
    if (p.bias) { e.bias_lo = p.bias[row_lo]; e.bias_hi = p.bias[row_hi]; }
    const int d = p.head_dim, half = d >> 1;
    const int head = row_lo / d, i = row_lo % d;
    const int position = p.positions[t];
    const bool is_q = head < p.num_heads;
    const bool is_v = head >= p.num_heads + p.num_kv_heads;
    if (!is_v && p.rope_style == ROPE_NEOX) {
      e.cosine = p.cos_table[static_cast<size_t>(position) * half + i];
      e.sine = p.sin_table[static_cast<size_t>(position) * half + i];
      e.rotate = 1;
    }
    __nv_bfloat16* dst = nullptr;
    if (is_q) {
      dst = p.q_out + (static_cast<size_t>(t) * p.num_heads + head) * d;
    } else if (p.write_cache) {
      const int page = p.block_table[static_cast<size_t>(p.token_entry[t]) * p.table_width + position / p.page_size];
      if (page >= 0) {
        const int kv_head = is_v ? head - p.num_heads - p.num_kv_heads : head - p.num_heads;
        __nv_bfloat16* pool = is_v ? p.v_pool : p.k_pool;
        dst = pool + ((static_cast<size_t>(page) * p.page_size + position % p.page_size) * p.num_kv_heads + kv_head) * d;
      }
    }
    e.dst = dst ? dst + i : nullptr;
    e.active = dst != nullptr;
  }
  return e;
}

// One (row pair, token) result, finished and stored.
__device__ __forceinline__ void finish(const GemvParams& p, const Ending& e, int row_lo, int row_hi, int t, float v_lo,
                                       float v_hi) {
  const bool has_hi = row_hi < p.N;
  if (p.epilogue == GEMV_RESIDUAL) {
    // every element of the stream gets one addition from one thread: an addition that does not
    // read the old value back gives the same sum and spares the ending a memory round trip
    atomicAdd(p.resid + static_cast<size_t>(t) * p.N + row_lo, v_lo);
    if (has_hi) atomicAdd(p.resid + static_cast<size_t>(t) * p.N + row_hi, v_hi);
  } else if (p.epilogue == GEMV_SWIGLU) {
    const int feature = (row_lo >> 5) * 16 + (row_lo & 15);
    const float value = v_hi * (v_lo / (1.0f + __expf(-v_lo)));
    const size_t at = static_cast<size_t>(t) * (p.N >> 1) + feature;
    if (p.out_dtype == VIPERA_BF16) static_cast<__nv_bfloat16*>(p.out)[at] = __float2bfloat16_rn(value);
    else static_cast<float*>(p.out)[at] = value;
  } else if (p.epilogue == GEMV_STORE) {
    v_lo += e.bias_lo;
    v_hi += e.bias_hi;
    const size_t at = static_cast<size_t>(t) * p.N;
    if (p.out_dtype == VIPERA_BF16) {
      static_cast<__nv_bfloat16*>(p.out)[at + row_lo] = __float2bfloat16_rn(v_lo);
      if (has_hi) static_cast<__nv_bfloat16*>(p.out)[at + row_hi] = __float2bfloat16_rn(v_hi);
    } else {
      static_cast<float*>(p.out)[at + row_lo] = v_lo;
      if (has_hi) static_cast<float*>(p.out)[at + row_hi] = v_hi;
    }
  } else {  // GEMV_ROPE_CACHE
    v_lo += e.bias_lo;
    v_hi += e.bias_hi;
    if (e.rotate) {
      const float lo = v_lo * e.cosine - v_hi * e.sine, hi = v_lo * e.sine + v_hi * e.cosine;
      v_lo = lo;
      v_hi = hi;
    }
    if (e.active) {
      __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(e.dst);
      dst[0] = __float2bfloat16_rn(v_lo);
      dst[p.head_dim >> 1] = __float2bfloat16_rn(v_hi);
    }
  }
}

// NT: token tiles of 8 (tokens padded to NT * 8).  Block: 32 * warps threads; it stages the
// activations once and then takes 16-row tiles blockIdx.x, blockIdx.x + gridDim.x, ...
template <int NT, bool NORM>
__global__ void __launch_bounds__(512)
gemv_small_kernel(const GemvParams p, int num_tiles) {
  extern __shared__ __align__(16) uint8_t shared[];
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int g = lane >> 2, tq = lane & 3;
  int tile = blockIdx.x;
  int row_lo, row_hi;
  tile_rows(p, tile, g, &row_lo, &row_hi);
  bool has_lo = row_lo < p.N, has_hi = row_hi < p.N;
  const __nv_bfloat16* w_lo = p.weight + static_cast<size_t>(has_lo ? row_lo : 0) * p.K;
  const __nv_bfloat16* w_hi = p.weight + static_cast<size_t>(has_hi ? row_hi : 0) * p.K;

  // this warp's share of K, in steps of 32
  const int steps_total = (p.K + 31) >> 5;
  const int steps_per_warp = (steps_total + warps - 1) / warps;
  const int step_begin = warp * steps_per_warp;
  const int step_end = min(steps_total, step_begin + steps_per_warp);

  // The weights do not depend on the kernels ahead of this one: the warp's first kHeld steps of
  // its share of K (all of it where K is small) are asked for before the wait and are in
  // registers when the activations arrive.
  const uint4 zero = make_uint4(0, 0, 0, 0);
  // (six steps are a warp's whole share at an inner size of 1536; eight were measured slower, the
  // kernel then spills, and so were five and four, which leave loads for after the wait)
  constexpr int kHeld = NT <= 2 ? 6 : 4;
  uint4 held_lo[kHeld], held_hi[kHeld];
#pragma unroll
  for (int u = 0; u < kHeld; ++u) {
    const int step = step_begin + u;
    const int k = step * 32 + tq * 8;
    held_lo[u] = zero;
    held_hi[u] = zero;
    if (step < step_end && k < p.K) {
      if (has_lo) held_lo[u] = __ldg(reinterpret_cast<const uint4*>(w_lo + k));
      if (has_hi) held_hi[u] = __ldg(reinterpret_cast<const uint4*>(w_hi + k));
    }
  }
  // A thread's own ending (where the block's threads cover the tile's (token, row pair) items
  // one each) is prepared ahead too.
  const bool one_item = p.T * 8 <= static_cast<int>(blockDim.x);
  const int my_t = threadIdx.x >> 3, my_r = threadIdx.x & 7;
  Ending my_ending;
  my_ending.active = 0;
  if (one_item && my_t < p.T) {
    int out_lo, out_hi;
    tile_rows(p, tile, my_r, &out_lo, &out_hi);
    if (out_lo < p.N) my_ending = prepare_ending(p, out_lo, out_hi, my_t);
  }
  pdl_wait();

  // ---- activations into shared memory: [NT * 8 tokens][K bf16 + pad], rows past T are zero ----
  const int act_stride = p.K * 2 + kActPadBytes;
  const int chunks = p.K >> 3;
  for (int t = warp; t < NT * 8; t += warps) {
    uint4* dst = reinterpret_cast<uint4*>(shared + static_cast<size_t>(t) * act_stride);
    if (t >= p.T) {
      for (int c = lane; c < chunks; c += 32) dst[c] = zero;
    } else if (NORM) {
      const float* x = p.x32 + static_cast<size_t>(p.rows ? p.rows[t] : t) * p.K;
      float squares = 0.0f;
      for (int c = lane; c < chunks; c += 32) {
        const float4 x0 = *reinterpret_cast<const float4*>(x + c * 8);
        const float4 x1 = *reinterpret_cast<const float4*>(x + c * 8 + 4);
        squares += x0.x * x0.x + x0.y * x0.y + x0.z * x0.z + x0.w * x0.w + x1.x * x1.x + x1.y * x1.y + x1.z * x1.z + x1.w * x1.w;
      }
      squares = warp_sum(squares);
      const float inverse = 1.0f / sqrtf(squares / static_cast<float>(p.K) + p.eps);
      for (int c = lane; c < chunks; c += 32) {
        const float4 x0 = *reinterpret_cast<const float4*>(x + c * 8);
        const float4 x1 = *reinterpret_cast<const float4*>(x + c * 8 + 4);
        const float4 g0 = *reinterpret_cast<const float4*>(p.norm_weight + c * 8);
        const float4 g1 = *reinterpret_cast<const float4*>(p.norm_weight + c * 8 + 4);
        uint4 packed;
        __nv_bfloat162* halves = reinterpret_cast<__nv_bfloat162*>(&packed);
        halves[0] = __floats2bfloat162_rn(x0.x * inverse * g0.x, x0.y * inverse * g0.y);
        halves[1] = __floats2bfloat162_rn(x0.z * inverse * g0.z, x0.w * inverse * g0.w);
        halves[2] = __floats2bfloat162_rn(x1.x * inverse * g1.x, x1.y * inverse * g1.y);
        halves[3] = __floats2bfloat162_rn(x1.z * inverse * g1.z, x1.w * inverse * g1.w);
        dst[c] = packed;
      }
    } else {
      const uint4* src = reinterpret_cast<const uint4*>(p.a16 + static_cast<size_t>(t) * p.K);
      for (int c = lane; c < chunks; c += 32) dst[c] = src[c];
    }
  }
  __syncthreads();

  // the warps' partial sums live behind the activations: [warps][NT * 8 tokens][16 rows]
  float* partial = reinterpret_cast<float*>(shared + static_cast<size_t>(NT) * 8 * act_stride);

  for (; tile < num_tiles; tile += gridDim.x) {
  if (tile != static_cast<int>(blockIdx.x)) {
    tile_rows(p, tile, g, &row_lo, &row_hi);
    has_lo = row_lo < p.N;
    has_hi = row_hi < p.N;
    w_lo = p.weight + static_cast<size_t>(has_lo ? row_lo : 0) * p.K;
    w_hi = p.weight + static_cast<size_t>(has_hi ? row_hi : 0) * p.K;
#pragma unroll
    for (int u = 0; u < kHeld; ++u) {
      const int step = step_begin + u;
      const int k = step * 32 + tq * 8;
      held_lo[u] = zero;
      held_hi[u] = zero;
      if (step < step_end && k < p.K) {
        if (has_lo) held_lo[u] = __ldg(reinterpret_cast<const uint4*>(w_lo + k));
        if (has_hi) held_hi[u] = __ldg(reinterpret_cast<const uint4*>(w_hi + k));
      }
    }
    if (one_item && my_t < p.T) {
      int out_lo, out_hi;
      tile_rows(p, tile, my_r, &out_lo, &out_hi);
      if (out_lo < p.N) my_ending = prepare_ending(p, out_lo, out_hi, my_t);
    }
  }
  // ---- the products ----
  float acc[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[n][i] = 0.0f;

  // the held steps first ...
#pragma unroll
  for (int u = 0; u < kHeld; ++u) {
    const int step = step_begin + u;
    const int k = step * 32 + tq * 8;
    if (step >= step_end) continue;   // the same for every lane of the warp
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      // a lane past the end of K (its weights are zeros) must not read past the row either
      const uint4 a = k < p.K
          ? *reinterpret_cast<const uint4*>(shared + static_cast<size_t>(n * 8 + g) * act_stride + k * 2) : zero;
      mma_16816(acc[n], held_lo[u].x, held_hi[u].x, held_lo[u].y, held_hi[u].y, a.x, a.y);
      mma_16816(acc[n], held_lo[u].z, held_hi[u].z, held_lo[u].w, held_hi[u].w, a.z, a.w);
    }
  }
  // ... then the rest of the warp's share, four steps in flight at a time
  constexpr int kUnroll = 4;
  for (int step0 = step_begin + kHeld; step0 < step_end; step0 += kUnroll) {
    uint4 lo[kUnroll], hi[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int step = step0 + u;
      const int k = step * 32 + tq * 8;
      lo[u] = zero;
      hi[u] = zero;
      if (step < step_end && k < p.K) {
        if (has_lo) lo[u] = __ldg(reinterpret_cast<const uint4*>(w_lo + k));
        if (has_hi) hi[u] = __ldg(reinterpret_cast<const uint4*>(w_hi + k));
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int step = step0 + u;
      const int k = step * 32 + tq * 8;
      if (step >= step_end) continue;   // the same for every lane of the warp
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        const uint4 a = k < p.K
            ? *reinterpret_cast<const uint4*>(shared + static_cast<size_t>(n * 8 + g) * act_stride + k * 2) : zero;
        mma_16816(acc[n], lo[u].x, hi[u].x, lo[u].y, hi[u].y, a.x, a.y);
        mma_16816(acc[n], lo[u].z, hi[u].z, lo[u].w, hi[u].w, a.z, a.w);
      }
    }
  }

  // ---- the warps' partial sums meet in shared memory ----
  {
    float* mine = partial + static_cast<size_t>(warp) * NT * 8 * 16;
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      const int t0 = n * 8 + 2 * tq;
      mine[t0 * 16 + g] = acc[n][0];
      mine[(t0 + 1) * 16 + g] = acc[n][1];
      mine[t0 * 16 + g + 8] = acc[n][2];
      mine[(t0 + 1) * 16 + g + 8] = acc[n][3];
    }
  }
  __syncthreads();
  // item = (token, pair of rows r and r + 8): summed over the warps in order, then finished
  for (int item = threadIdx.x; item < p.T * 8; item += blockDim.x) {
    const int t = item >> 3, r = item & 7;
    float v_lo = 0.0f, v_hi = 0.0f;
    for (int w = 0; w < warps; ++w) {
      const float* src = partial + (static_cast<size_t>(w) * NT * 8 + t) * 16;
      v_lo += src[r];
      v_hi += src[r + 8];
    }
    int out_lo, out_hi;
    tile_rows(p, tile, r, &out_lo, &out_hi);
    if (out_lo < p.N) {
      if (one_item) finish(p, my_ending, out_lo, out_hi, t, v_lo, v_hi);
      else finish(p, prepare_ending(p, out_lo, out_hi, t), out_lo, out_hi, t, v_lo, v_hi);
    }
  }
  __syncthreads();  // the partials are read; the next tile may overwrite them
  }
}

template <int NT, bool NORM>
static int launch_gemv(const GemvParams& p, int tiles, int warps, size_t shared, cudaStream_t s) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemv_small_kernel<NT, NORM>, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemvMaxShared);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  static int sms = 0;
  if (sms == 0) {
    int device = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    if (sms <= 0) sms = 148;
  }
  // as many blocks as fit on the device at once (by shared memory), each looping over tiles
  int per_sm = static_cast<int>((220 * 1024) / (shared + 1024));
  if (per_sm < 1) per_sm = 1;
  if (per_sm > 2048 / (warps * 32)) per_sm = 2048 / (warps * 32);
  int blocks = sms * per_sm;
  if (blocks > tiles) blocks = tiles;
  return vipera_launch(gemv_small_kernel<NT, NORM>, dim3(blocks), dim3(warps * 32), shared, s, p, tiles);
}

// Token tiles of 8 the kernel is built for: 1, 2, 4 or 8.
static int gemv_token_tiles(int tokens) {
  const int nt = (tokens + 7) / 8;
  return nt <= 1 ? 1 : nt <= 2 ? 2 : nt <= 4 ? 4 : 8;
}

static size_t gemv_shared_bytes(int tokens, int K, int warps) {
  const int padded = gemv_token_tiles(tokens) * 8;  // the kernel stages (and zero-fills) this many rows
  const size_t activations = static_cast<size_t>(padded) * (static_cast<size_t>(K) * 2 + kActPadBytes);
  const size_t partials = static_cast<size_t>(warps) * padded * 16 * sizeof(float);
  return activations + partials;
}

static int gemv_warps(int K) { return K >= 4096 ? 16 : 8; }

// Whether vipera_gemv_small takes `tokens` tokens against a matrix of N rows and inner size K
// (the activations of the step must fit in one block's shared memory).
VIPERA_API int vipera_gemv_small_takes(int tokens, int K, int N) {
  if (tokens <= 0 || tokens > 32 || K <= 0 || (K % 8) != 0 || N <= 0) return 0;
  return gemv_shared_bytes(tokens, K, gemv_warps(K)) <= kGemvMaxShared ? 1 : 0;
}

// out = act . W^T for at most 32 tokens.  `x32` (with `norm_weight`, `eps` and optional `rows`)
// or `a16` is the input; exactly one of them is given.  K must be a multiple of 8 and all
// row starts 16-byte aligned.  For GEMV_ROPE_CACHE, N = (heads + 2 * kv_heads) * d with d a
// multiple of 16, and the outputs go to q_out and the cache pools; see GemvParams.
VIPERA_API int vipera_gemv_small(const GemvParams* params, void* stream) {
  const GemvParams& p = *params;
  if (p.T <= 0) return VIPERA_OK;
  if (p.N <= 0 || !vipera_gemv_small_takes(p.T, p.K, p.N)) return VIPERA_BAD_SHAPE;
  if ((p.x32 == nullptr) == (p.a16 == nullptr)) return VIPERA_BAD_ARGUMENT;
  if (p.x32 && !p.norm_weight) return VIPERA_BAD_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(p.weight) & 15) return VIPERA_BAD_ARGUMENT;
  int tiles;
  if (p.epilogue == GEMV_SWIGLU) {
    if (p.N % 32 || !p.out) return VIPERA_BAD_SHAPE;
    tiles = p.N / 16;
  } else if (p.epilogue == GEMV_ROPE_CACHE) {
    if (p.head_dim <= 0 || (p.head_dim % 16) || p.N != (p.num_heads + 2 * p.num_kv_heads) * p.head_dim) return VIPERA_BAD_SHAPE;
    if (!p.q_out || !p.positions) return VIPERA_BAD_ARGUMENT;
    if (p.rope_style == ROPE_NEOX && (!p.cos_table || !p.sin_table)) return VIPERA_BAD_ARGUMENT;
    if (p.rope_style != ROPE_NEOX && p.rope_style != ROPE_NONE) return VIPERA_BAD_ARGUMENT;
    if (p.write_cache && (!p.k_pool || !p.v_pool || !p.token_entry || !p.block_table || p.page_size <= 0)) return VIPERA_BAD_ARGUMENT;
    tiles = p.N / 16;
  } else if (p.epilogue == GEMV_STORE) {
    if (!p.out) return VIPERA_BAD_ARGUMENT;
    tiles = (p.N + 15) / 16;
  } else if (p.epilogue == GEMV_RESIDUAL) {
    if (!p.resid) return VIPERA_BAD_ARGUMENT;
    tiles = (p.N + 15) / 16;
  } else {
    return VIPERA_BAD_ARGUMENT;
  }
  const int warps = gemv_warps(p.K);
  const size_t shared = gemv_shared_bytes(p.T, p.K, warps);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int nt = gemv_token_tiles(p.T);
#define VIPERA_GEMV_CASE(NT)                                                               \
  return p.x32 ? launch_gemv<NT, true>(p, tiles, warps, shared, s) : launch_gemv<NT, false>(p, tiles, warps, shared, s)
  if (nt == 1) { VIPERA_GEMV_CASE(1); }
  if (nt == 2) { VIPERA_GEMV_CASE(2); }
  if (nt == 4) { VIPERA_GEMV_CASE(4); }
  VIPERA_GEMV_CASE(8);
#undef VIPERA_GEMV_CASE
}

VIPERA_API int vipera_gemv_params_size() { return static_cast<int>(sizeof(GemvParams)); }
