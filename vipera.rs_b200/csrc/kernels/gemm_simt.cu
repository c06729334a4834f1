// Matrix products on the CUDA cores with 32-bit accumulation: out[M, N] = A[M, K] . W[N, K]^T.
//
// This is the product kernel of the true 32-bit path (no tensor cores, no reduced-precision
// mode) and the fallback of the bfloat16 path for sizes the tensor-core kernel refuses.
// The reference multiplies one weight matrix by all B activation rows in one pass over the
// weights (crates/vipera-backend-cpu/src/model.rs:1005-1025) and promises that a row's
// result does not depend on its neighbours in the batch (model.rs:881-882); here every output
// element sums over K in the same fixed order whatever M is.
//
// Epilogues:
//   STORE     out[m, n] = acc (+ bias[n]), stored as float or bfloat16
//   RESIDUAL  resid[m, n] += acc            (32-bit residual stream)
//   SWIGLU    W holds gate and up rows interleaved in groups of 16 (16 gate rows, then the
//             16 up rows of the same features); out[m, f] = up * silu(gate), silu(z) = z/(1+exp(-z))
//             (model.rs:4368-4374)
#include "common.cuh"

enum GemmEpilogue { EPI_STORE = 0, EPI_RESIDUAL = 1, EPI_SWIGLU = 2 };

constexpr int BM = 64, BN = 64, BK = 16, PAD = 4;

template <typename TA, typename TW, typename TO, int EPI>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TA* __restrict__ A, const TW* __restrict__ W, int M, int N, int K,
                 const float* __restrict__ bias, TO* __restrict__ out, float* __restrict__ resid) {
  __shared__ float As[BK][BM + PAD];
  __shared__ float Ws[BK][BN + PAD];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int load_row = tid >> 2, load_k = (tid & 3) * 4;

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    {
      const int m = m0 + load_row;
      const TA* src = A + static_cast<size_t>(m) * K + k0 + load_k;
#pragma unroll
      for (int e = 0; e < 4; ++e)
        As[load_k + e][load_row] = (m < M && k0 + load_k + e < K) ? to_float<TA>(src[e]) : 0.0f;
      const int n = n0 + load_row;
      const TW* wsrc = W + static_cast<size_t>(n) * K + k0 + load_k;
#pragma unroll
      for (int e = 0; e < 4; ++e)
        Ws[load_k + e][load_row] = (n < N && k0 + load_k + e < K) ? to_float<TW>(wsrc[e]) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = Ws[k][tx + 16 * j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
    if (EPI == EPI_SWIGLU) {
      // columns tx, tx+16 are gate and up of feature (n0/2 + tx); tx+32, tx+48 of (n0/2 + 16 + tx)
#pragma unroll
      for (int pair = 0; pair < 2; ++pair) {
        const int n_gate = n0 + tx + 32 * pair;
        if (n_gate + 16 >= N) continue;
        const int feature = n0 / 2 + 16 * pair + tx;
        const float gate = acc[i][2 * pair], up = acc[i][2 * pair + 1];
        const float value = up * (gate / (1.0f + expf(-gate)));
        out[static_cast<size_t>(m) * (N / 2) + feature] = from_float<TO>(value);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int n = n0 + tx + 16 * j;
        if (n >= N) continue;
        float value = acc[i][j];
        if (EPI == EPI_STORE) {
          if (bias) value += bias[n];
          out[static_cast<size_t>(m) * N + n] = from_float<TO>(value);
        } else {
          resid[static_cast<size_t>(m) * N + n] += value;
        }
      }
    }
  }
}

template <typename TA, typename TW>
static int launch_typed(const TA* A, const TW* W, int M, int N, int K, int epilogue, const float* bias,
                        void* out, int out_dtype, float* resid, cudaStream_t s) {
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (epilogue == EPI_RESIDUAL) {
    if (!resid) return VIPERA_BAD_ARGUMENT;
    gemm_simt_kernel<TA, TW, float, EPI_RESIDUAL><<<grid, 256, 0, s>>>(A, W, M, N, K, nullptr, nullptr, resid);
  } else if (epilogue == EPI_STORE) {
    if (!out) return VIPERA_BAD_ARGUMENT;
    if (out_dtype == VIPERA_F32)
      gemm_simt_kernel<TA, TW, float, EPI_STORE><<<grid, 256, 0, s>>>(A, W, M, N, K, bias, static_cast<float*>(out), nullptr);
    else if (out_dtype == VIPERA_BF16)
      gemm_simt_kernel<TA, TW, __nv_bfloat16, EPI_STORE><<<grid, 256, 0, s>>>(A, W, M, N, K, bias, static_cast<__nv_bfloat16*>(out), nullptr);
    else
      return VIPERA_BAD_DTYPE;
  } else if (epilogue == EPI_SWIGLU) {
    if (!out) return VIPERA_BAD_ARGUMENT;
    if (N % 32 != 0) return VIPERA_BAD_SHAPE;  // gate/up groups of 16 must pair up
    if (out_dtype == VIPERA_F32)
      gemm_simt_kernel<TA, TW, float, EPI_SWIGLU><<<grid, 256, 0, s>>>(A, W, M, N, K, nullptr, static_cast<float*>(out), nullptr);
    else if (out_dtype == VIPERA_BF16)
      gemm_simt_kernel<TA, TW, __nv_bfloat16, EPI_SWIGLU><<<grid, 256, 0, s>>>(A, W, M, N, K, nullptr, static_cast<__nv_bfloat16*>(out), nullptr);
    else
      return VIPERA_BAD_DTYPE;
  } else {
    return VIPERA_BAD_ARGUMENT;
  }
  return vipera_launch_status();
}

// A is [M, K] and W is [N, K], both row-major and contiguous.  For SWIGLU, N counts the
// interleaved gate and up rows (twice the intermediate size) and out is [M, N/2].
VIPERA_API int vipera_gemm_simt(const void* A, int a_dtype, const void* W, int w_dtype, int M, int N, int K,
                                int epilogue, const float* bias, void* out, int out_dtype, float* resid,
                                void* stream) {
  if (M <= 0) return VIPERA_OK;
  if (N <= 0 || K <= 0) return VIPERA_BAD_SHAPE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (a_dtype == VIPERA_F32 && w_dtype == VIPERA_F32)
    return launch_typed(static_cast<const float*>(A), static_cast<const float*>(W), M, N, K, epilogue, bias, out, out_dtype, resid, s);
  if (a_dtype == VIPERA_BF16 && w_dtype == VIPERA_BF16)
    return launch_typed(static_cast<const __nv_bfloat16*>(A), static_cast<const __nv_bfloat16*>(W), M, N, K, epilogue, bias, out, out_dtype, resid, s);
  if (a_dtype == VIPERA_F32 && w_dtype == VIPERA_BF16)
    return launch_typed(static_cast<const float*>(A), static_cast<const __nv_bfloat16*>(W), M, N, K, epilogue, bias, out, out_dtype, resid, s);
  return VIPERA_BAD_DTYPE;
}

VIPERA_API const char* vipera_gemm_simt_status_text(int status) { return vipera_status_text(status); }
