// C = A * B^T on CUDA cores with float32 accumulation: the matrix product of the
// all-32-bit path, and the always-correct form of every product of the bfloat16 path.
//
// One kernel covers the dense linear layers (reference: rocBLAS ``gemm_ex`` with f32
// compute, src/ops/linear.hip:9-59, and the GEMV kernels of src/ops/gemv.hip) and the
// routed experts (reference: a host loop over experts, src/models/model.hip:355-427):
//   * groups: rows [offsets[g], offsets[g+1]) of A use weight matrix g of B;
//   * gather: row r of A is taken from a_rows[r] / a_div (token of a routed pair);
//   * SwiGLU epilogue: B holds [gate rows | up rows]; C = silu(A gate^T) * (A up^T).
// Each output element is one thread's sequential sum over k, so a row's result does not
// depend on how many other rows are in the batch.
#include "common.cuh"

namespace nf {

constexpr int BM = 64, BN = 64, BK = 16;

template <typename TA, typename TC, bool SWIGLU>
__global__ void __launch_bounds__(256)
gemm_nt_kernel(const TA* __restrict__ A, int lda, const TA* __restrict__ B, size_t b_group_stride,
               TC* __restrict__ C, int ldc, int M, int N, int K,
               const int* __restrict__ offsets, const int* __restrict__ a_rows, int a_div) {
  // N is the number of output columns (for SWIGLU: the inner width; B has 2N rows).
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[BK][BN + 4];
  const int g = blockIdx.z;
  int row_begin = 0, row_end = M;
  if (offsets) {
    row_begin = offsets[g];
    row_end = offsets[g + 1];
  }
  const int m0 = row_begin + blockIdx.y * BM;
  if (m0 >= row_end) return;
  constexpr int NCOL = SWIGLU ? BN / 2 : BN;   // output columns per block
  const int n0 = blockIdx.x * NCOL;
  const TA* Bg = B + (size_t)g * b_group_stride;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;

  // loader roles: 256 threads move 64 x 16 elements of A and of B per k-step (4 each)
  const int lrow = threadIdx.x >> 2;        // 0..63
  const int lk = (threadIdx.x & 3) * 4;     // 0,4,8,12
  const int arow = m0 + lrow;
  long a_src = -1;
  if (arow < row_end) a_src = a_rows ? (long)(a_rows[arow] / a_div) : (long)arow;
  // B tile row `lrow`: for SWIGLU rows 0..31 are gate rows n0.., rows 32..63 the matching up rows
  long b_src;
  if (SWIGLU) {
    const int c = n0 + (lrow & 31);
    b_src = c < N ? (long)(lrow < 32 ? c : N + c) : -1;
  } else {
    b_src = n0 + lrow < N ? (long)(n0 + lrow) : -1;
  }

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = k0 + lk + i;
      As[lk + i][lrow] = (a_src >= 0 && k < K) ? to_float(A[a_src * lda + k]) : 0.f;
      Bs[lk + i][lrow] = (b_src >= 0 && k < K) ? to_float(Bg[b_src * (long)K + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[k][tx + 16 * j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = m0 + ty * 4 + i;
    if (r >= row_end) continue;
    if (SWIGLU) {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int c = n0 + tx + 16 * j;
        if (c < N) {
          const float gt = acc[i][j], up = acc[i][j + 2];
          C[(size_t)r * ldc + c] = from_float<TC>(gt / (1.f + expf(-gt)) * up);
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c = n0 + tx + 16 * j;
        if (c < N) C[(size_t)r * ldc + c] = from_float<TC>(acc[i][j]);
      }
    }
  }
}

template <typename TA, typename TC>
static int launch(const void* A, int lda, const void* B, size_t bgs, void* C, int ldc, int M, int N,
                  int K, int groups, int max_rows_per_group, const int* offsets,
                  const int* a_rows, int a_div, bool swiglu, cudaStream_t stream) {
  const int ncol = swiglu ? BN / 2 : BN;
  dim3 grid((N + ncol - 1) / ncol, (max_rows_per_group + BM - 1) / BM, groups);
  NF_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "gemm: too many row tiles (%u) or groups (%u)", grid.y, grid.z);
  if (swiglu)
    gemm_nt_kernel<TA, TC, true><<<grid, 256, 0, stream>>>((const TA*)A, lda, (const TA*)B, bgs, (TC*)C, ldc, M, N, K, offsets, a_rows, a_div);
  else
    gemm_nt_kernel<TA, TC, false><<<grid, 256, 0, stream>>>((const TA*)A, lda, (const TA*)B, bgs, (TC*)C, ldc, M, N, K, offsets, a_rows, a_div);
  return check_launch("gemm_simt");
}

}  // namespace nf

using namespace nf;

// C[M, N] = epilogue(A[M, K] * B[g]^T).  in_dtype: A and B; out_dtype: C (float32 allowed
// with bfloat16 inputs, for logits).  groups == 1 and offsets == null: dense.
// For swiglu, B[g] has 2N rows (gate rows first) and C has N columns.
extern "C" int nf_gemm_simt(const void* A, int lda, const void* B, long long b_group_stride, void* C,
                            int ldc, int M, int N, int K, int groups, int max_rows_per_group,
                            const int* offsets, const int* a_rows, int a_div, int swiglu,
                            int in_dtype, int out_dtype, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  NF_REQUIRE(M > 0 && N > 0 && K > 0 && groups > 0 && a_div > 0, "gemm: bad sizes M=%d N=%d K=%d groups=%d", M, N, K, groups);
  NF_REQUIRE(groups == 1 || offsets, "gemm: grouped product needs row offsets");
  if (in_dtype == kF32 && out_dtype == kF32)
    return launch<float, float>(A, lda, B, (size_t)b_group_stride, C, ldc, M, N, K, groups, max_rows_per_group, offsets, a_rows, a_div, swiglu, stream);
  if (in_dtype == kBF16 && out_dtype == kBF16)
    return launch<__nv_bfloat16, __nv_bfloat16>(A, lda, B, (size_t)b_group_stride, C, ldc, M, N, K, groups, max_rows_per_group, offsets, a_rows, a_div, swiglu, stream);
  if (in_dtype == kBF16 && out_dtype == kF32)
    return launch<__nv_bfloat16, float>(A, lda, B, (size_t)b_group_stride, C, ldc, M, N, K, groups, max_rows_per_group, offsets, a_rows, a_div, swiglu, stream);
  set_error("gemm: unsupported dtype pair in=%d out=%d", in_dtype, out_dtype);
  return 1;
}
