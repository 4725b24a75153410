// Counter-based random weights: element i of a tensor is a function of (key of the tensor, i)
// alone, made of integer arithmetic and two IEEE single-precision operations, so that the host
// (weights/counter_rng.py, in torch integer ops) and this kernel give the same bits, in any order
// and any chunking.  The reference has no random-weights mode.
//
//   s  = mix(mix(lo32(i) ^ k1) ^ hi32(i) ^ k2)
//   w_j = mix(s ^ C_j), j = 0..3                  four 32-bit words
//   n  = sum of the twelve 10-bit fields of w_0..w_3, minus 6138    (mean 0, variance 1048575)
//   z  = float(n) * kInvStd                        approximately N(0, 1), |z| <= 5.995
//   "linear": 0.02 * z      "norm": 1 + 0.05 * z   rounded to bfloat16 (nearest even)
//
// mix is a 32-bit finaliser (xor-shift 16, * 0x7feb352d, xor-shift 15, * 0x846ca68b, xor-shift 16).
#include "common.cuh"

namespace nf {
namespace {

__host__ __device__ __forceinline__ unsigned mix32(unsigned x) {
  x ^= x >> 16;
  x *= 0x7feb352du;
  x ^= x >> 15;
  x *= 0x846ca68bu;
  x ^= x >> 16;
  return x;
}

__device__ __forceinline__ float draw(unsigned long long i, unsigned k1, unsigned k2, int init) {
  const unsigned s = mix32(mix32((unsigned)(i & 0xffffffffull) ^ k1) ^ (unsigned)(i >> 32) ^ k2);
  const unsigned c[4] = {0x9e3779b9u, 0x85ebca6bu, 0xc2b2ae35u, 0x27d4eb2fu};
  int n = -6138;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const unsigned w = mix32(s ^ c[j]);
    n += (int)(w & 1023u) + (int)((w >> 10) & 1023u) + (int)((w >> 20) & 1023u);
  }
  const float z = __fmul_rn((float)n, 9.765629656612873e-4f);      // 1 / sqrt(1048575)
  const float v = init == 1 ? __fadd_rn(1.0f, __fmul_rn(0.05f, z)) : __fmul_rn(0.02f, z);
  return __bfloat162float(__float2bfloat16_rn(v));                   // every value is a bfloat16 number
}

template <typename T>
__global__ void random_fill_kernel(T* __restrict__ out, long long n, long long first, unsigned k1, unsigned k2,
                                   int init) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    out[i] = from_float<T>(draw((unsigned long long)(first + i), k1, k2, init));
}

}  // namespace
}  // namespace nf

using namespace nf;

// out[i] = value of element `first + i` of the tensor with keys (k1, k2), i < n.
// init: 0 "linear" (0.02 z), 1 "norm" (1 + 0.05 z).  dtype: 0 float32 (holding bfloat16 values), 1 bfloat16.
extern "C" int nf_random_fill(void* out, long long n, long long first, unsigned k1, unsigned k2, int init,
                              int dtype, cudaStream_t stream) {
  if (n == 0) return 0;
  NF_REQUIRE(n > 0 && first >= 0 && (init == 0 || init == 1), "random_fill: bad arguments n=%lld first=%lld init=%d", n, first, init);
  const int block = 256;
  long long want = (n + block - 1) / block;
  const int grid = (int)(want < 148 * 16 ? want : 148 * 16);
  if (dtype == kBF16)
    random_fill_kernel<__nv_bfloat16><<<grid, block, 0, stream>>>((__nv_bfloat16*)out, n, first, k1, k2, init);
  else if (dtype == kF32)
    random_fill_kernel<float><<<grid, block, 0, stream>>>((float*)out, n, first, k1, k2, init);
  else {
    set_error("random_fill: dtype %d is neither float32 nor bfloat16", dtype);
    return 1;
  }
  return check_launch("random_fill");
}
