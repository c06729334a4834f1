// Sampling on the device: penalties, greedy argmax, and temperature sampling with top-k,
// top-p and min-p, one block per row of logits.
//
// Semantics are those of the reference's sampler crate.  Greedy: the best finite logit,
// ties to the lowest id (crates/vipera-sampler/src/lib.rs:135-156).  Temperature: the k best
// candidates, best first with ties by ascending id (lib.rs:440-527); peak = best/T; total =
// sum over every finite logit of exp(x/T - peak); candidate weights exp(x/T - peak); the
// shortest head whose weights reach top_p * total; drop weights below min_p * best weight;
// target = uniform * mass, first candidate whose running sum (64-bit) exceeds it
// (lib.rs:172-247).  Penalties: for ids seen recently, logit > 0 ? logit / f : logit * f,
// minus presence + frequency * count; then the bias of the id (lib.rs:596-616).  The
// uniform number is drawn on the host from the request's own generator.
//
// With top_k = 0 the reference keeps a head of 4096 and sorts the whole vocabulary only if
// top-p reaches past it (lib.rs:437, 206-216); this kernel reports that case in `status`
// (SAMPLE_NEEDS_HOST) and the caller draws that row with the host sampler.
#include "common.cuh"

enum SampleStatus { SAMPLE_OK = 0, SAMPLE_NO_FINITE = 1, SAMPLE_NO_MASS = 2, SAMPLE_NEEDS_HOST = 3 };

constexpr int kSampleThreads = 1024;
constexpr int kMaxCandidates = 4096;

__device__ __forceinline__ uint32_t ordered_key(float v) {
  const uint32_t bits = __float_as_uint(v);
  return (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
}
__device__ __forceinline__ float key_value(uint32_t key) {
  return __uint_as_float((key & 0x80000000u) ? (key & 0x7fffffffu) : ~key);
}
__device__ __forceinline__ bool finite(float v) { return fabsf(v) <= 3.402823466e38f; }

// ---------------------------------------------------------------------------------------
// penalties: one thread per (row, id) entry
// ---------------------------------------------------------------------------------------
__global__ void penalty_kernel(float* __restrict__ logits, int vocab, int entries,
                               const int* __restrict__ entry_row, const int* __restrict__ entry_id,
                               const int* __restrict__ entry_count, const float* __restrict__ entry_bias,
                               const float* __restrict__ repetition, const float* __restrict__ presence,
                               const float* __restrict__ frequency) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= entries) return;
  const int row = entry_row[e], id = entry_id[e];
  if (id < 0 || id >= vocab) return;
  float* cell = logits + static_cast<size_t>(row) * vocab + id;
  float value = *cell;
  if (!finite(value)) return;
  const int count = entry_count[e];
  if (count > 0) {
    const float f = repetition[row];
    if (f != 1.0f) value = value > 0.0f ? value / f : value * f;
    value -= presence[row] + frequency[row] * static_cast<float>(count);
  }
  value += entry_bias[e];
  *cell = value;
}

VIPERA_API int vipera_apply_penalties(float* logits, int vocab, int entries, const int* entry_row,
                                      const int* entry_id, const int* entry_count, const float* entry_bias,
                                      const float* repetition, const float* presence, const float* frequency,
                                      void* stream) {
  if (entries <= 0) return VIPERA_OK;
  penalty_kernel<<<(entries + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      logits, vocab, entries, entry_row, entry_id, entry_count, entry_bias, repetition, presence, frequency);
  return vipera_launch_status();
}

// ---------------------------------------------------------------------------------------
// argmax with ties to the lowest id, over the block
// ---------------------------------------------------------------------------------------
struct Best {
  float value;
  int id;  // -1: nothing finite seen
};
__device__ __forceinline__ Best better_of(Best a, Best b) {
  if (a.id < 0) return b;
  if (b.id < 0) return a;
  if (a.value > b.value) return a;
  if (b.value > a.value) return b;
  return a.id < b.id ? a : b;
}
__device__ Best block_argmax(const float* __restrict__ row, int vocab, Best* scratch /* 32 */) {
  Best best{0.0f, -1};
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = row[i];
    if (finite(v)) best = better_of(best, Best{v, i});
  }
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    Best other;
    other.value = __shfl_xor_sync(0xffffffffu, best.value, offset);
    other.id = __shfl_xor_sync(0xffffffffu, best.id, offset);
    best = better_of(best, other);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) scratch[warp] = best;
  __syncthreads();
  const int warps = (blockDim.x + 31) >> 5;
  best = lane < warps ? scratch[lane] : Best{0.0f, -1};
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    Best other;
    other.value = __shfl_xor_sync(0xffffffffu, best.value, offset);
    other.id = __shfl_xor_sync(0xffffffffu, best.id, offset);
    best = better_of(best, other);
  }
  return best;
}

// Greedy over a wide vocabulary in two stages, so that many blocks read each row at once:
// every block finds the best of its slice of the row (eight independent loads in flight per
// thread), then one warp per row picks the best of the slices.  Ties still go to the lowest id.
constexpr int kArgmaxSlices = 32;
constexpr int kArgmaxThreads = 256;

__global__ void __launch_bounds__(kArgmaxThreads)
argmax_slice_kernel(const float* __restrict__ logits, int vocab, float* __restrict__ slice_value,
                    int* __restrict__ slice_id) {
  __shared__ Best scratch[32];
  const int row = blockIdx.x, slice = blockIdx.y;
  const int per = (vocab + kArgmaxSlices - 1) / kArgmaxSlices;
  const int begin = slice * per, end = min(vocab, begin + per);
  const float* src = logits + static_cast<size_t>(row) * vocab;
  Best best{0.0f, -1};
  for (int base = begin + threadIdx.x; base < end; base += 8 * kArgmaxThreads) {
    float v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = base + u * kArgmaxThreads;
      v[u] = i < end ? src[i] : NAN;
    }
#pragma unroll
    for (int u = 0; u < 8; ++u)
      if (finite(v[u])) best = better_of(best, Best{v[u], base + u * kArgmaxThreads});
  }
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    Best other;
    other.value = __shfl_xor_sync(0xffffffffu, best.value, offset);
    other.id = __shfl_xor_sync(0xffffffffu, best.id, offset);
    best = better_of(best, other);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) scratch[warp] = best;
  __syncthreads();
  if (warp == 0) {
    best = lane < kArgmaxThreads / 32 ? scratch[lane] : Best{0.0f, -1};
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
      Best other;
      other.value = __shfl_xor_sync(0xffffffffu, best.value, offset);
      other.id = __shfl_xor_sync(0xffffffffu, best.id, offset);
      best = better_of(best, other);
    }
    if (lane == 0) {
      slice_value[row * kArgmaxSlices + slice] = best.value;
      slice_id[row * kArgmaxSlices + slice] = best.id;
    }
  }
}

__global__ void argmax_final_kernel(const float* __restrict__ slice_value, const int* __restrict__ slice_id,
                                    int* __restrict__ tokens, int* __restrict__ status) {
  const int row = blockIdx.x, lane = threadIdx.x;
  Best best{slice_value[row * kArgmaxSlices + lane], slice_id[row * kArgmaxSlices + lane]};
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    Best other;
    other.value = __shfl_xor_sync(0xffffffffu, best.value, offset);
    other.id = __shfl_xor_sync(0xffffffffu, best.id, offset);
    best = better_of(best, other);
  }
  if (lane == 0) {
    tokens[row] = best.id < 0 ? 0 : best.id;
    if (status) status[row] = best.id < 0 ? SAMPLE_NO_FINITE : SAMPLE_OK;
  }
}

// `scratch` holds 64 * rows 32-bit words (a value and an id for each of 32 slices of a row).
VIPERA_API int vipera_argmax(const float* logits, int rows, int vocab, int* tokens, int* status, void* scratch,
                             void* stream) {
  if (rows <= 0) return VIPERA_OK;
  if (vocab <= 0) return VIPERA_BAD_SHAPE;
  if (!scratch) return VIPERA_BAD_ARGUMENT;
  static_assert(kArgmaxSlices == 32, "the final stage is one warp");
  float* slice_value = static_cast<float*>(scratch);
  int* slice_id = reinterpret_cast<int*>(slice_value + static_cast<size_t>(rows) * kArgmaxSlices);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  argmax_slice_kernel<<<dim3(rows, kArgmaxSlices), kArgmaxThreads, 0, s>>>(logits, vocab, slice_value, slice_id);
  int launched = vipera_launch_status();
  if (launched != VIPERA_OK) return launched;
  argmax_final_kernel<<<rows, 32, 0, s>>>(slice_value, slice_id, tokens, status);
  return vipera_launch_status();
}

// ---------------------------------------------------------------------------------------
// temperature sampling
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
              const double* __restrict__ uniform, int* __restrict__ tokens, int* __restrict__ status) {
  __shared__ Best best_scratch[32];
  __shared__ float sum_scratch[32];
  __shared__ unsigned int histogram[256];
  __shared__ unsigned long long candidates[kMaxCandidates];
  __shared__ unsigned int shared_prefix, shared_remaining, shared_count, shared_equal_taken;
  __shared__ unsigned int scan_scratch[32];

  const int r = blockIdx.x;
  const float* row = logits + static_cast<size_t>(r) * vocab;
  const int tid = threadIdx.x;

  const Best best = block_argmax(row, vocab, best_scratch);
  if (best.id < 0) {
    if (tid == 0) { tokens[r] = 0; status[r] = SAMPLE_NO_FINITE; }
    return;
  }
  const float temp = temperature[r];
  if (temp == 0.0f) {
    if (tid == 0) { tokens[r] = best.id; status[r] = SAMPLE_OK; }
    return;
  }
  const float scale = 1.0f / temp;
  const float peak = best.value * scale;

  // softmax mass over every finite logit, and how many there are
  float partial = 0.0f;
  unsigned int finite_count = 0;
  for (int i = tid; i < vocab; i += kSampleThreads) {
    const float v = row[i];
    if (finite(v)) { partial += expf(v * scale - peak); ++finite_count; }
  }
  const float total = block_sum(partial, sum_scratch);
  const unsigned int finite_total = __float2uint_rn(block_sum(static_cast<float>(finite_count), sum_scratch));
  if (!(total > 0.0f) || !finite(total)) {
    if (tid == 0) { tokens[r] = 0; status[r] = SAMPLE_NO_MASS; }
    return;
  }

  const int requested = top_k[r];
  const bool uncut = requested == 0;
  if (requested > kMaxCandidates) {
    if (tid == 0) { tokens[r] = 0; status[r] = SAMPLE_NEEDS_HOST; }
    return;
  }
  unsigned int bound = uncut ? kMaxCandidates : static_cast<unsigned int>(requested);
  if (bound > finite_total) bound = finite_total;

  // radix select: the key of the bound-th largest finite logit
  unsigned int prefix = 0, prefix_mask = 0, remaining = bound;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = tid; i < 256; i += kSampleThreads) histogram[i] = 0;
    __syncthreads();
    for (int i = tid; i < vocab; i += kSampleThreads) {
      const float v = row[i];
      if (!finite(v)) continue;
      const uint32_t key = ordered_key(v);
      if ((key & prefix_mask) == prefix) atomicAdd(&histogram[(key >> shift) & 255u], 1u);
    }
    __syncthreads();
    if (tid == 0) {
      unsigned int seen = 0;
      int bin = 255;
      for (; bin > 0; --bin) {
        if (seen + histogram[bin] >= remaining) break;
        seen += histogram[bin];
      }
      shared_prefix = prefix | (static_cast<unsigned int>(bin) << shift);
      shared_remaining = remaining - seen;
    }
    __syncthreads();
    prefix = shared_prefix;
    remaining = shared_remaining;
    prefix_mask |= 255u << shift;
    __syncthreads();
  }
  const uint32_t threshold_key = prefix;    // key of the bound-th largest
  const unsigned int need_equal = remaining; // how many with exactly that key are taken

  // gather: everything above the threshold, then the lowest ids among the equal ones
  if (tid == 0) { shared_count = 0; shared_equal_taken = 0; }
  __syncthreads();
  for (int i = tid; i < vocab; i += kSampleThreads) {
    const float v = row[i];
    if (!finite(v)) continue;
    const uint32_t key = ordered_key(v);
    if (key > threshold_key) {
      const unsigned int slot = atomicAdd(&shared_count, 1u);
      if (slot < kMaxCandidates)
        candidates[slot] = (static_cast<unsigned long long>(key) << 32) | (0xffffffffu - static_cast<unsigned int>(i));
    }
  }
  __syncthreads();
  // equal keys in ascending id order: a block-wide ordered compaction, chunk by chunk
  for (int chunk = 0; chunk < vocab; chunk += kSampleThreads) {
    if (shared_equal_taken >= need_equal) break;
    const int i = chunk + tid;
    bool is_equal = false;
    if (i < vocab) {
      const float v = row[i];
      is_equal = finite(v) && ordered_key(v) == threshold_key;
    }
    const unsigned int ballot = __ballot_sync(0xffffffffu, is_equal);
    const int lane = tid & 31, warp = tid >> 5;
    if (lane == 0) scan_scratch[warp] = __popc(ballot);
    __syncthreads();
    unsigned int before = shared_equal_taken;
    for (int w = 0; w < warp; ++w) before += scan_scratch[w];
    const unsigned int rank = before + __popc(ballot & ((1u << lane) - 1u));
    if (is_equal && rank < need_equal) {
      const unsigned int slot = atomicAdd(&shared_count, 1u);
      if (slot < kMaxCandidates)
        candidates[slot] = (static_cast<unsigned long long>(threshold_key) << 32) | (0xffffffffu - static_cast<unsigned int>(i));
    }
    __syncthreads();
    if (tid == 0) {
      unsigned int all = 0;
      for (int w = 0; w < kSampleThreads / 32; ++w) all += scan_scratch[w];
      shared_equal_taken += all;
    }
    __syncthreads();
  }
  __syncthreads();
  const unsigned int count = min(shared_count, static_cast<unsigned int>(kMaxCandidates));

  // bitonic sort, descending by (value, then lower id first)
  unsigned int padded = 1;
  while (padded < count) padded <<= 1;
  for (unsigned int i = count + tid; i < padded; i += kSampleThreads) candidates[i] = 0ull;
  __syncthreads();
  for (unsigned int size = 2; size <= padded; size <<= 1) {
    for (unsigned int stride = size >> 1; stride > 0; stride >>= 1) {
      for (unsigned int i = tid; i < padded; i += kSampleThreads) {
        const unsigned int partner = i ^ stride;
        if (partner > i) {
          const bool descending = (i & size) == 0;
          const unsigned long long a = candidates[i], b = candidates[partner];
          if (descending ? a < b : a > b) { candidates[i] = b; candidates[partner] = a; }
        }
      }
      __syncthreads();
    }
  }

  if (tid == 0) {
    // weights, top-p cut, min-p filter and the draw, in order, by one thread
    const float target_mass = top_p[r] * total;
    float cumulative = 0.0f;
    int cut = -1;
    for (unsigned int i = 0; i < count; ++i) {
      const float w = expf(key_value(static_cast<uint32_t>(candidates[i] >> 32)) * scale - peak);
      cumulative += w;
      if (cumulative >= target_mass) { cut = static_cast<int>(i) + 1; break; }
    }
    if (uncut && cut < 0 && count < finite_total) {
      tokens[r] = 0;
      status[r] = SAMPLE_NEEDS_HOST;
      return;
    }
    const unsigned int kept_end = cut >= 0 ? static_cast<unsigned int>(cut) : count;
    const float best_weight = expf(key_value(static_cast<uint32_t>(candidates[0] >> 32)) * scale - peak);
    const float floor_weight = min_p[r] * best_weight;
    float mass = 0.0f;
    for (unsigned int i = 0; i < kept_end; ++i) {
      const float w = expf(key_value(static_cast<uint32_t>(candidates[i] >> 32)) * scale - peak);
      if (w >= floor_weight) mass += w;
    }
    const double target = uniform[r] * static_cast<double>(mass);
    double running = 0.0;
    int chosen = -1, last = -1;
    for (unsigned int i = 0; i < kept_end; ++i) {
      const float w = expf(key_value(static_cast<uint32_t>(candidates[i] >> 32)) * scale - peak);
      if (!(w >= floor_weight)) continue;
      last = static_cast<int>(0xffffffffu - static_cast<unsigned int>(candidates[i] & 0xffffffffull));
      running += static_cast<double>(w);
      if (target < running) { chosen = last; break; }
    }
    tokens[r] = chosen >= 0 ? chosen : (last >= 0 ? last : best.id);
    status[r] = SAMPLE_OK;
  }
}

// One row of `logits` per request; rows with temperature 0 are drawn greedily.  `status`
// gets a SampleStatus per row.
VIPERA_API int vipera_sample(const float* logits, int rows, int vocab, const float* temperature,
                             const int* top_k, const float* top_p, const float* min_p,
                             const double* uniform, int* tokens, int* status, void* stream) {
  if (rows <= 0) return VIPERA_OK;
  if (vocab <= 0) return VIPERA_BAD_SHAPE;
  if (!status || !tokens) return VIPERA_BAD_ARGUMENT;
  sample_kernel<<<rows, kSampleThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      logits, vocab, temperature, top_k, top_p, min_p, uniform, tokens, status);
  return vipera_launch_status();
}

// ---------------------------------------------------------------------------------------
// Log-probabilities of drawn tokens (crates/vipera-sampler/src/lib.rs:319-378): over every
// finite logit (penalties already applied), x = logit / temperature (1 where the row is drawn
// greedily), logprob(id) = x_id - max - ln(sum exp(x - max)); the drawn token's, and the top_n
// most likely ids with theirs, best first, ties to the lowest id.  One block per asked row.
// ---------------------------------------------------------------------------------------
constexpr int kLogprobThreads = 256;

__global__ void __launch_bounds__(kLogprobThreads)
logprob_kernel(const float* __restrict__ logits, int vocab, const int* __restrict__ rows, const int* __restrict__ tokens,
               const float* __restrict__ temperature, int top_n, float* __restrict__ chosen, int* __restrict__ top_ids,
               float* __restrict__ top_values) {
  __shared__ float scratch[32];
  __shared__ float best_value[kLogprobThreads];
  __shared__ int best_id[kLogprobThreads];
  const int item = blockIdx.x;
  const float* row = logits + static_cast<size_t>(rows[item]) * vocab;
  const float t = temperature[item] > 0.0f ? temperature[item] : 1.0f;
  float peak = -INFINITY;
  for (int i = threadIdx.x; i < vocab; i += kLogprobThreads) {
    const float v = row[i];
    if (finite(v)) peak = fmaxf(peak, v / t);
  }
  peak = block_max(peak, scratch);
  float mass = 0.0f;
  for (int i = threadIdx.x; i < vocab; i += kLogprobThreads) {
    const float v = row[i];
    if (finite(v)) mass += expf(v / t - peak);
  }
  mass = block_sum(mass, scratch);
  const float log_mass = logf(mass);
  if (threadIdx.x == 0) {
    const float v = row[tokens[item]];
    chosen[item] = finite(peak) && finite(v) ? v / t - peak - log_mass : -INFINITY;
  }
  // the top_n: each round takes the best (value, then lowest id) that comes after the one before
  float last_value = INFINITY;
  int last_id = -1;
  for (int k = 0; k < top_n; ++k) {
    float mine = -INFINITY;
    int mine_id = -1;
    for (int i = threadIdx.x; i < vocab; i += kLogprobThreads) {
      const float v = row[i];
      if (!finite(v)) continue;
      const float x = v / t;
      const bool after = x < last_value || (x == last_value && i > last_id);
      if (after && (x > mine || mine_id < 0)) {   // ids rise within a thread, so the first of equals stays
        mine = x;
        mine_id = i;
      }
    }
    best_value[threadIdx.x] = mine;
    best_id[threadIdx.x] = mine_id;
    __syncthreads();
    for (int stride = kLogprobThreads / 2; stride > 0; stride >>= 1) {
      if (threadIdx.x < stride) {
        const float a = best_value[threadIdx.x], b = best_value[threadIdx.x + stride];
        const int ia = best_id[threadIdx.x], ib = best_id[threadIdx.x + stride];
        const bool take_b = ib >= 0 && (ia < 0 || b > a || (b == a && ib < ia));
        if (take_b) {
          best_value[threadIdx.x] = b;
          best_id[threadIdx.x] = ib;
        }
      }
      __syncthreads();
    }
    last_value = best_value[0];
    last_id = best_id[0];
    __syncthreads();
    if (threadIdx.x == 0) {
      top_ids[static_cast<size_t>(item) * top_n + k] = last_id;
      top_values[static_cast<size_t>(item) * top_n + k] = last_id >= 0 ? last_value - peak - log_mass : -INFINITY;
    }
    if (last_id < 0) last_value = -INFINITY;   // nothing left: the remaining places stay empty
  }
}

// chosen[i] = log-probability of tokens[i] in row rows[i] of `logits` at temperature[i]; with
// top_n > 0 also the top_n most likely ids of that row and their log-probabilities (-1 and
// -inf where the row has fewer finite logits).
VIPERA_API int vipera_logprobs(const float* logits, int vocab, int count, const int* rows, const int* tokens,
                               const float* temperature, int top_n, float* chosen, int* top_ids, float* top_values,
                               void* stream) {
  if (count <= 0) return VIPERA_OK;
  if (vocab <= 0 || top_n < 0) return VIPERA_BAD_SHAPE;
  if (!logits || !rows || !tokens || !temperature || !chosen || (top_n > 0 && (!top_ids || !top_values)))
    return VIPERA_BAD_ARGUMENT;
  logprob_kernel<<<count, kLogprobThreads, 0, static_cast<cudaStream_t>(stream)>>>(logits, vocab, rows, tokens, temperature,
                                                                                   top_n, chosen, top_ids, top_values);
  return vipera_launch_status();
}

VIPERA_API const char* vipera_sampling_status_text(int status) { return vipera_status_text(status); }

// ---------------------------------------------------------------------------------------
// greedy argmax for callers that cannot allocate (see no_alloc.h)
// ---------------------------------------------------------------------------------------
#include "no_alloc.h"

// The scratch of the two argmax stages, inside the library image itself.  In host code this
// name is only a handle for the symbol, not a device address: the address comes from
// cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned int argmax_static_scratch[64 * VIPERA_ARGMAX_STATIC_MAX_ROWS];

// Device address of the array on each device, looked up on the first call there.
static void* argmax_static_address[64] = {nullptr};

extern "C" __attribute__((visibility("default")))
int vipera_argmax_static(const float* logits, int rows, int vocab, int* tokens, int* status, void* stream) {
  if (rows <= 0) return VIPERA_OK;
  if (rows > VIPERA_ARGMAX_STATIC_MAX_ROWS || vocab <= 0) return VIPERA_BAD_SHAPE;
  if (!logits || !tokens) return VIPERA_BAD_ARGUMENT;
  int device = 0;
  cudaError_t error = cudaGetDevice(&device);
  if (error != cudaSuccess) return static_cast<int>(error);
  if (device < 0 || device >= 64) return VIPERA_BAD_ARGUMENT;
  if (argmax_static_address[device] == nullptr) {
    // set-up, once per device, with that device current
    void* address = nullptr;
    error = cudaGetSymbolAddress(&address, argmax_static_scratch);
    if (error != cudaSuccess) return static_cast<int>(error);
    argmax_static_address[device] = address;
  }
  float* slice_value = static_cast<float*>(argmax_static_address[device]);
  int* slice_id = reinterpret_cast<int*>(slice_value + static_cast<size_t>(rows) * kArgmaxSlices);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // Every (row, slice) word is written by the first kernel before the second reads it, so
  // nothing left by an earlier call is ever read and nothing needs clearing.
  argmax_slice_kernel<<<dim3(rows, kArgmaxSlices), kArgmaxThreads, 0, s>>>(logits, vocab, slice_value, slice_id);
  int launched = vipera_launch_status();
  if (launched != VIPERA_OK) return launched;
  argmax_final_kernel<<<rows, 32, 0, s>>>(slice_value, slice_id, tokens, status);
  return vipera_launch_status();
}

// The tokens a step has drawn become the next step's input without a trip to the host:
// dst[i] = src[i] for the step's own entries; the entries a captured graph adds to fill its
// size repeat entry 0, as they do in every other input.
__global__ void feed_tokens_kernel(const int* __restrict__ src, int* __restrict__ dst, int own, int total) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < total) dst[i] = src[i < own ? i : 0];
}

VIPERA_API int vipera_feed_tokens(const int* src, int* dst, int own, int total, void* stream) {
  if (own <= 0 || total < own) return VIPERA_BAD_SHAPE;
  return vipera_launch(feed_tokens_kernel, dim3((total + 255) / 256), dim3(256), 0, static_cast<cudaStream_t>(stream), src, dst,
                       own, total);
}

// Wait until everything queued on `stream` so far has run.
VIPERA_API int vipera_stream_synchronize(void* stream) {
  const cudaError_t error = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  return error == cudaSuccess ? VIPERA_OK : static_cast<int>(error);
}
