// Matrix products on the CUDA cores: out[M, N] = x[M, K] . w[N, K]^T (+ bias[N]) (+ residual[M, N]).
//
// This is the product kernel of the true 32-bit path (FFMA with float32 accumulation:
// no tensor cores, no TF32, no bfloat16 staging) and the kernel that takes every size
// and every mix of element types in the bfloat16 path: any M, N, K, no alignment
// needed, bfloat16 or float32 activations, weights and outputs. The bfloat16 path's
// tensor-core kernels serve the shapes they are built for; whatever they refuse runs here.
//
// Weights are [out, in] row-major as the checkpoint stores them, which is what
// x . w^T reads (engine/model.py:303-320 of the reference calls F.linear on the same
// layout). Every output element sums its K products in the same order whatever M is, so
// a token's result does not depend on what else is in the batch.
#include "common.cuh"

using namespace pae;

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;  // 256 threads, 4x4 outputs each

template <typename TA, typename TW, typename TO>
__global__ void __launch_bounds__(256) gemm_simt_kernel(TO* __restrict__ out, const TA* __restrict__ x,
                                                        const TW* __restrict__ w, const float* __restrict__ bias,
                                                        const TO* __restrict__ residual, int M, int N, int K) {
  dependent_launch_prologue();
  __shared__ float xs[BK][BM + 4];
  __shared__ float ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tx = tid % 16, ty = tid / 16;      // outputs rows ty*4.., cols tx*4..
  const int load_row = tid / 4, load_k = (tid % 4) * 4;

  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    {
      const int m = m0 + load_row;
      const TA* src = x + (size_t)m * K + k0 + load_k;
#pragma unroll
      for (int j = 0; j < 4; ++j) xs[load_k + j][load_row] = (m < M && k0 + load_k + j < K) ? to_float(src[j]) : 0.f;
      const int n = n0 + load_row;
      const TW* wsrc = w + (size_t)n * K + k0 + load_k;
#pragma unroll
      for (int j = 0; j < 4; ++j) ws[load_k + j][load_row] = (n < N && k0 + load_k + j < K) ? to_float(wsrc[j]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = xs[k][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = ws[k][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = m0 + ty * TM + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (bias != nullptr) v += bias[n];
      if (residual != nullptr) v += to_float(residual[(size_t)m * N + n]);
      out[(size_t)m * N + n] = from_float<TO>(v);
    }
  }
}

template <typename TA, typename TW, typename TO>
int launch(void* out, const void* x, const void* w, const float* bias, const void* residual, int M, int N, int K,
           cudaStream_t s) {
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  launch_kernel(gemm_simt_kernel<TA, TW, TO>, grid, 256, 0, s, (TO*)out, (const TA*)x, (const TW*)w, bias, (const TO*)residual, M, N, K);
  return check_launch("linear_simt");
}

}  // namespace

// x_dtype, w_dtype, out_dtype: 0 float32, 1 bfloat16. bias (float32) and residual
// (out_dtype, may be `out` itself) may be null.
PAE_EXPORT int pae_linear_simt(void* out, const void* x, const void* w, const float* bias, const void* residual,
                               int M, int N, int K, int x_dtype, int w_dtype, int out_dtype, void* stream) {
  if (M == 0 || N == 0) return 0;
  if ((long long)((M + BM - 1) / BM) > 65535) return fail(3, "linear_simt: %d rows are more than one launch takes", M);
  cudaStream_t s = (cudaStream_t)stream;
  using bf = __nv_bfloat16;
  const int key = x_dtype * 100 + w_dtype * 10 + out_dtype;
  switch (key) {
    case 0: return launch<float, float, float>(out, x, w, bias, residual, M, N, K, s);
    case 111: return launch<bf, bf, bf>(out, x, w, bias, residual, M, N, K, s);
    case 110: return launch<bf, bf, float>(out, x, w, bias, residual, M, N, K, s);
    case 101: return launch<bf, float, bf>(out, x, w, bias, residual, M, N, K, s);
    case 100: return launch<bf, float, float>(out, x, w, bias, residual, M, N, K, s);
    default:
      return fail(1, "linear_simt: element types x=%d w=%d out=%d are not supported", x_dtype, w_dtype, out_dtype);
  }
}

PAE_DEFINE_LAST_ERROR()
