// Row-wise kernels: embedding gather, residual sum + RMS norm, SwiGLU activation, and
// the combination of routed and shared expert outputs.
//
// Formulas follow the reference's kernels (src/ops/kernels.hip): embed_gather 150-159,
// rmsnorm 17-41, fused_residual_rmsnorm 100-129, silu_and_mul 131-140; the weighted
// sum of expert outputs replaces scale_rows (216-223) + scatter_add_rows
// (src/ops/moe.hip:22-31, which races) by one pass with a fixed order and no atomics.
// The residual stream is float32 in both modes.
#define NF_CHAIN_CLASS 2
#include "common.cuh"

namespace nf {

template <typename T>
__global__ void embed_rows_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                  float* __restrict__ out, int hidden, int vocab) {
  const int t = blockIdx.x;
  chain_wait();          // before the first write too: `out` may be memory that the kernel before still reads
  const int id = ids[t];
  float* o = out + (size_t)t * hidden;
  if (id < 0 || id >= vocab) {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = 0.f;
    return;
  }
  const T* row = table + (size_t)id * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = to_float(row[i]);
}

// h[t] += delta[t] (if delta), out[t] = h[t] * rsqrt(mean(h[t]^2) + eps) * w.
// With `rows`, row r reads h[rows[r]] / delta[rows[r]], writes out[r] and leaves h alone.
template <typename T, bool GATHER>
__global__ void add_rmsnorm_kernel(float* __restrict__ h, const T* __restrict__ delta,
                                   const int* __restrict__ rows, const float* __restrict__ w,
                                   float eps, T* __restrict__ out, int hidden) {
  __shared__ float red[33];
  const int r = blockIdx.x;
  const int src = GATHER ? rows[r] : r;
  float* hr = h + (size_t)src * hidden;
  const T* dr = delta ? delta + (size_t)src * hidden : nullptr;
  T* o = out + (size_t)r * hidden;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = hr[i];
    if (dr) {
      v += to_float(dr[i]);
      if (!GATHER) hr[i] = v;
    }
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)hidden + eps);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = hr[i];
    if (GATHER && dr) v += to_float(dr[i]);
    o[i] = from_float<T>(v * inv * w[i]);
  }
}

// Four elements a thread per step (float4 of h, 4 values of delta / out); same sums in the
// same order per thread as the scalar kernel would give with a stride of 4 * blockDim.
template <typename T, bool GATHER>
__global__ void add_rmsnorm_x4_kernel(float* __restrict__ h, const T* __restrict__ delta,
                                      const int* __restrict__ rows, const float* __restrict__ w,
                                      float eps, T* __restrict__ out, int hidden) {
  __shared__ float red[33];
  const int r = blockIdx.x;
  chain_release_if_small();
  chain_wait(h, delta, rows);
  const int src = GATHER ? rows[r] : r;
  float* hr = h + (size_t)src * hidden;
  const T* dr = delta ? delta + (size_t)src * hidden : nullptr;
  T* o = out + (size_t)r * hidden;
  float ss = 0.f;
  for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
    float v[4];
    load4(hr + i, v);
    if (dr) {
      float d[4];
      load4(dr + i, d);
#pragma unroll
      for (int e = 0; e < 4; ++e) v[e] += d[e];
      if (!GATHER) store4(hr + i, v);
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) ss += v[e] * v[e];
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)hidden + eps);
  for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
    float v[4], wv[4];
    load4(hr + i, v);
    if (GATHER && dr) {
      float d[4];
      load4(dr + i, d);
#pragma unroll
      for (int e = 0; e < 4; ++e) v[e] += d[e];
    }
    load4(w + i, wv);
#pragma unroll
    for (int e = 0; e < 4; ++e) v[e] = v[e] * inv * wv[e];
    store4(o + i, v);
  }
}

template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ act, int inner) {
  const int m = blockIdx.x;
  const int i = blockIdx.y * blockDim.x + threadIdx.x;
  if (i >= inner) return;
  const float g = to_float(gu[(size_t)m * 2 * inner + i]);
  const float u = to_float(gu[(size_t)m * 2 * inner + inner + i]);
  act[(size_t)m * inner + i] = from_float<T>(g / (1.f + expf(-g)) * u);
}

// out[t] = sum_j wts[t,j] * y[inv[t*k+j]]  (j ascending)  + sigmoid(gate[t*gate_stride]) * shared[t]
template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ y, const int* __restrict__ inv,
                                   const float* __restrict__ wts, const T* __restrict__ shared,
                                   const float* __restrict__ gate, int gate_stride,
                                   T* __restrict__ out, int hidden, int k) {
  const int t = blockIdx.x;
  const int i = blockIdx.y * blockDim.x + threadIdx.x;
  if (i >= hidden) return;
  float acc = 0.f;
  for (int j = 0; j < k; ++j) {
    const int p = inv[t * k + j];
    acc += wts[t * k + j] * to_float(y[(size_t)p * hidden + i]);
  }
  if (shared) {
    float s = to_float(shared[(size_t)t * hidden + i]);
    if (gate) s *= 1.f / (1.f + expf(-gate[(size_t)t * gate_stride]));
    acc += s;
  }
  out[(size_t)t * hidden + i] = from_float<T>(acc);
}

// out[p] = x[rows[p] / div]: rows of 16-byte pieces
__global__ void gather_rows_kernel(const uint4* __restrict__ x, const int* __restrict__ rows, int div,
                                   uint4* __restrict__ out, int pieces) {
  const int p = blockIdx.x;
  chain_wait(x, rows);
  const uint4* src = x + (size_t)(rows[p] / div) * pieces;
  uint4* dst = out + (size_t)p * pieces;
  for (int i = threadIdx.x; i < pieces; i += blockDim.x) dst[i] = src[i];
}

// 8 bfloat16 at a time: act = silu(gate) * up
__global__ void silu_mul_bf16x8_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ act,
                                       int inner) {
  const int m = blockIdx.x;
  const int i = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  chain_wait(gu);
  if (i >= inner) return;
  float g[8], u[8];
  load8(gu + (size_t)m * 2 * inner + i, g);
  load8(gu + (size_t)m * 2 * inner + inner + i, u);
  __align__(16) __nv_bfloat16 o[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) o[e] = __float2bfloat16_rn(g[e] / (1.f + expf(-g[e])) * u[e]);
  *reinterpret_cast<uint4*>(act + (size_t)m * inner + i) = *reinterpret_cast<const uint4*>(o);
}

// set to 1 + token if a combine met a sorted position outside the step's pairs (read and reset by
// nf_index_status)
__device__ int g_combine_index_error = 0;

__global__ void moe_combine_bf16x8_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ inv,
                                          const float* __restrict__ wts,
                                          const __nv_bfloat16* __restrict__ shared,
                                          const float* __restrict__ gate, int gate_stride,
                                          __nv_bfloat16* __restrict__ out, int hidden, int k) {
  const int t = blockIdx.x;
  const int i = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  chain_release();
  chain_wait(y, inv, wts, shared, gate);
  if (i >= hidden) return;
  float acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.f;
  for (int j = 0; j < k; ++j) {
    const int p = inv[t * k + j];
    if ((unsigned)p >= (unsigned)(gridDim.x * k)) {      // not a sorted position of this step: skip, and say so
      atomicCAS(&g_combine_index_error, 0, 1 + t);
      continue;
    }
    const float w = wts[t * k + j];
    float v[8];
    load8(y + (size_t)p * hidden + i, v);
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = fmaf(w, v[e], acc[e]);
  }
  if (shared) {
    float v[8];
    load8(shared + (size_t)t * hidden + i, v);
    const float gsc = gate ? 1.f / (1.f + expf(-gate[(size_t)t * gate_stride])) : 1.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = fmaf(v[e], gsc, acc[e]);
  }
  __align__(16) __nv_bfloat16 o[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) o[e] = __float2bfloat16_rn(acc[e]);
  *reinterpret_cast<uint4*>(out + (size_t)t * hidden + i) = *reinterpret_cast<const uint4*>(o);
}

// The combine above and add_rmsnorm_x4_kernel in one pass over a row: the weighted sum of the
// row's expert outputs (+ gated shared expert), rounded to bfloat16 as the separate combine
// stores it, is added to the float32 residual row, and the row is normalised.  Same thread-to-
// element map, same order of every sum as the two separate kernels, hence the same bits; one
// launch and one round trip of [T, hidden] less.  A thread keeps its elements in registers:
// rows of up to kFusedIters * 4 * blockDim elements.
constexpr int kFusedIters = 8;
constexpr int kFusedMaxK = 32;     // most experts a token (the row's positions and weights sit in shared memory)

template <bool GATHER>
__global__ void moe_combine_add_rmsnorm_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ inv,
                                               const float* __restrict__ wts,
                                               const __nv_bfloat16* __restrict__ shared,
                                               const float* __restrict__ gate, int gate_stride,
                                               float* __restrict__ h, const int* __restrict__ rows,
                                               const float* __restrict__ w, float eps,
                                               __nv_bfloat16* __restrict__ out, int hidden, int k, int n_pairs) {
  __shared__ float red[33];
  __shared__ int s_pos[kFusedMaxK];
  __shared__ float s_wt[kFusedMaxK];
  const int r = blockIdx.x;
  chain_release_if_small();
  chain_wait(y, inv, wts, shared, gate, h, rows);
  const int t = GATHER ? rows[r] : r;
  float* hr = h + (size_t)t * hidden;
  // the row's k sorted positions and weights first, so that the sums below are nothing but
  // independent loads of expert rows (a position outside the step's pairs is skipped, and said)
  if (threadIdx.x < k) {
    int p = inv[t * k + threadIdx.x];
    if ((unsigned)p >= (unsigned)n_pairs) {
      atomicCAS(&g_combine_index_error, 0, 1 + t);
      p = -1;
    }
    s_pos[threadIdx.x] = p;
    s_wt[threadIdx.x] = wts[t * k + threadIdx.x];
  }
  const float gsc = (shared && gate) ? 1.f / (1.f + expf(-gate[(size_t)t * gate_stride])) : 1.f;
  __syncthreads();
  float keep[kFusedIters][4];
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < kFusedIters; ++it) {
    const int i = (it * blockDim.x + threadIdx.x) * 4;
    if (i < hidden) {
      float hv[4], sv[4] = {0.f, 0.f, 0.f, 0.f};
      load4(hr + i, hv);
      if (shared) load4(shared + (size_t)t * hidden + i, sv);
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
      for (int j = 0; j < k; ++j) {
        const int p = s_pos[j];
        if (p < 0) continue;
        const float wj = s_wt[j];
        float v[4];
        load4(y + (size_t)p * hidden + i, v);
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[e] = fmaf(wj, v[e], acc[e]);
      }
      if (shared) {
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[e] = fmaf(sv[e], gsc, acc[e]);
      }
      float v[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) v[e] = hv[e] + __bfloat162float(__float2bfloat16_rn(acc[e]));
      if (!GATHER) store4(hr + i, v);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        ss += v[e] * v[e];
        keep[it][e] = v[e];
      }
    }
  }
  ss = block_sum(ss, red);
  const float inv_rms = rsqrtf(ss / (float)hidden + eps);
  __nv_bfloat16* o = out + (size_t)r * hidden;
#pragma unroll
  for (int it = 0; it < kFusedIters; ++it) {
    const int i = (it * blockDim.x + threadIdx.x) * 4;
    if (i < hidden) {
      float wv[4], v[4];
      load4(w + i, wv);
#pragma unroll
      for (int e = 0; e < 4; ++e) v[e] = keep[it][e] * inv_rms * wv[e];
      store4(o + i, v);
    }
  }
}

static inline int row_threads(int n) {
  int t = 32;
  while (t < n && t < 256) t <<= 1;
  return t;
}

}  // namespace nf

using namespace nf;

extern "C" int nf_embed_rows(const void* table, const int* ids, float* out, int T, int hidden,
                             int vocab, int dtype, cudaStream_t stream) {
  if (T == 0) return 0;
  NF_REQUIRE(T > 0 && hidden > 0 && vocab > 0, "embed_rows: bad sizes T=%d hidden=%d vocab=%d", T, hidden, vocab);
  if (dtype == kF32)
    launch_chained(embed_rows_kernel<float>, dim3(T), dim3(row_threads(hidden)), 0, stream, (const float*)table, ids, out, hidden, vocab);
  else
    launch_chained(embed_rows_kernel<__nv_bfloat16>, dim3(T), dim3(row_threads(hidden)), 0, stream, (const __nv_bfloat16*)table, ids, out, hidden, vocab);
  return check_launch("embed_rows");
}

extern "C" int nf_add_rmsnorm(float* h, const void* delta, const int* rows, const float* w,
                              float eps, void* out, int R, int hidden, int dtype,
                              cudaStream_t stream) {
  if (R == 0) return 0;
  NF_REQUIRE(R > 0 && hidden > 0, "add_rmsnorm: bad sizes R=%d hidden=%d", R, hidden);
  if (hidden % 4 == 0 && (uintptr_t)h % 16 == 0 && (uintptr_t)out % 16 == 0 && (uintptr_t)w % 16 == 0 &&
      (!delta || (uintptr_t)delta % 16 == 0)) {
    const int t4 = row_threads(hidden / 4);
    if (dtype == kF32) {
      if (rows) launch_chained(add_rmsnorm_x4_kernel<float, true>, dim3(R), dim3(t4), 0, stream, h, (const float*)delta, rows, w, eps, (float*)out, hidden);
      else launch_chained(add_rmsnorm_x4_kernel<float, false>, dim3(R), dim3(t4), 0, stream, h, (const float*)delta, rows, w, eps, (float*)out, hidden);
    } else {
      if (rows) launch_chained(add_rmsnorm_x4_kernel<__nv_bfloat16, true>, dim3(R), dim3(t4), 0, stream, h, (const __nv_bfloat16*)delta, rows, w, eps, (__nv_bfloat16*)out, hidden);
      else launch_chained(add_rmsnorm_x4_kernel<__nv_bfloat16, false>, dim3(R), dim3(t4), 0, stream, h, (const __nv_bfloat16*)delta, rows, w, eps, (__nv_bfloat16*)out, hidden);
    }
    return check_launch("add_rmsnorm");
  }
  const int th = row_threads(hidden);
  if (dtype == kF32) {
    if (rows) add_rmsnorm_kernel<float, true><<<R, th, 0, stream>>>(h, (const float*)delta, rows, w, eps, (float*)out, hidden);
    else add_rmsnorm_kernel<float, false><<<R, th, 0, stream>>>(h, (const float*)delta, rows, w, eps, (float*)out, hidden);
  } else {
    if (rows) add_rmsnorm_kernel<__nv_bfloat16, true><<<R, th, 0, stream>>>(h, (const __nv_bfloat16*)delta, rows, w, eps, (__nv_bfloat16*)out, hidden);
    else add_rmsnorm_kernel<__nv_bfloat16, false><<<R, th, 0, stream>>>(h, (const __nv_bfloat16*)delta, rows, w, eps, (__nv_bfloat16*)out, hidden);
  }
  return check_launch("add_rmsnorm");
}

extern "C" int nf_silu_mul(const void* gu, void* act, int M, int inner, int dtype,
                           cudaStream_t stream) {
  if (M == 0) return 0;
  NF_REQUIRE(M > 0 && inner > 0, "silu_mul: bad sizes M=%d inner=%d", M, inner);
  if (dtype == kBF16 && inner % 8 == 0 && (uintptr_t)gu % 16 == 0 && (uintptr_t)act % 16 == 0) {
    dim3 g8(M, (inner / 8 + 127) / 128);
    launch_chained(silu_mul_bf16x8_kernel, g8, dim3(128), 0, stream, (const __nv_bfloat16*)gu, (__nv_bfloat16*)act, inner);
    return check_launch("silu_mul");
  }
  dim3 grid(M, (inner + 255) / 256);
  if (dtype == kF32) silu_mul_kernel<float><<<grid, 256, 0, stream>>>((const float*)gu, (float*)act, inner);
  else silu_mul_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)act, inner);
  return check_launch("silu_mul");
}

extern "C" int nf_moe_combine(const void* y, const int* inv, const float* wts, const void* shared,
                              const float* gate, int gate_stride, void* out, int T, int hidden,
                              int k, int dtype, cudaStream_t stream) {
  if (T == 0) return 0;
  NF_REQUIRE(T > 0 && hidden > 0 && k > 0, "moe_combine: bad sizes T=%d hidden=%d k=%d", T, hidden, k);
  if (dtype == kBF16 && hidden % 8 == 0 && (uintptr_t)y % 16 == 0 && (uintptr_t)out % 16 == 0 &&
      (!shared || (uintptr_t)shared % 16 == 0)) {
    dim3 g8(T, (hidden / 8 + 127) / 128);
    launch_chained(moe_combine_bf16x8_kernel, g8, dim3(128), 0, stream, (const __nv_bfloat16*)y, inv, wts, (const __nv_bfloat16*)shared, gate, gate_stride, (__nv_bfloat16*)out, hidden, k);
    return check_launch("moe_combine");
  }
  dim3 grid(T, (hidden + 255) / 256);
  if (dtype == kF32)
    moe_combine_kernel<float><<<grid, 256, 0, stream>>>((const float*)y, inv, wts, (const float*)shared, gate, gate_stride, (float*)out, hidden, k);
  else
    moe_combine_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)y, inv, wts, (const __nv_bfloat16*)shared, gate, gate_stride, (__nv_bfloat16*)out, hidden, k);
  return check_launch("moe_combine");
}

// 1 if the fused combine + add + norm kernel takes these sizes (bfloat16 only).
extern "C" int nf_moe_combine_add_rmsnorm_fits(int hidden) {
  if (hidden <= 0 || hidden % 4) return 0;
  return hidden <= kFusedIters * 4 * row_threads(hidden / 4) ? 1 : 0;
}

// h[t] += bfloat16(sum_j wts[t, j] * y[inv[t, j]] + sigmoid(gate[t]) * shared[t]); out[r] = rmsnorm(h[t]) * w
// for t = r (rows null; h is updated) or t = rows[r] (h is left as it is).  T: rows of h's step
// (inv and wts have T * k entries), R: rows written.
extern "C" int nf_moe_combine_add_rmsnorm(const void* y, const int* inv, const float* wts, const void* shared,
                                          const float* gate, int gate_stride, float* h, const int* rows,
                                          const float* w, float eps, void* out, int T, int R, int hidden,
                                          int k, cudaStream_t stream) {
  if (R == 0) return 0;
  NF_REQUIRE(T > 0 && R > 0 && k > 0 && k <= kFusedMaxK && nf_moe_combine_add_rmsnorm_fits(hidden), "moe_combine_add_rmsnorm: bad sizes T=%d R=%d hidden=%d k=%d", T, R, hidden, k);
  NF_REQUIRE((uintptr_t)y % 8 == 0 && (uintptr_t)h % 16 == 0 && (uintptr_t)out % 8 == 0 && (uintptr_t)w % 16 == 0 &&
             (!shared || (uintptr_t)shared % 8 == 0), "moe_combine_add_rmsnorm: operands must be 16-byte aligned");
  const int t4 = row_threads(hidden / 4);
  if (rows)
    launch_chained(moe_combine_add_rmsnorm_kernel<true>, dim3(R), dim3(t4), 0, stream, (const __nv_bfloat16*)y, inv, wts,
                   (const __nv_bfloat16*)shared, gate, gate_stride, h, rows, w, eps, (__nv_bfloat16*)out, hidden, k, T * k);
  else
    launch_chained(moe_combine_add_rmsnorm_kernel<false>, dim3(R), dim3(t4), 0, stream, (const __nv_bfloat16*)y, inv, wts,
                   (const __nv_bfloat16*)shared, gate, gate_stride, h, rows, w, eps, (__nv_bfloat16*)out, hidden, k, T * k);
  return check_launch("moe_combine_add_rmsnorm");
}

// 0, or 1 + the token whose combine met an index outside the step's pairs since the last call.
extern "C" int nf_combine_index_status() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_combine_index_error, sizeof(int)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(g_combine_index_error, &zero, sizeof(int));
  return v;
}

// out[p, :] = x[rows[p] / div, :] for n rows of `row_bytes` bytes (a multiple of 16).
extern "C" int nf_gather_rows(const void* x, const int* rows, int div, void* out, int n, int row_bytes,
                              cudaStream_t stream) {
  if (n == 0) return 0;
  NF_REQUIRE(n > 0 && div > 0 && row_bytes > 0 && row_bytes % 16 == 0, "gather_rows: rows of %d bytes are not whole 16-byte pieces", row_bytes);
  NF_REQUIRE(((uintptr_t)x % 16 == 0) && ((uintptr_t)out % 16 == 0), "gather_rows: operands must be 16-byte aligned");
  launch_chained(gather_rows_kernel, dim3(n), dim3(row_threads(row_bytes / 16)), 0, stream, (const uint4*)x, rows, div, (uint4*)out, row_bytes / 16);
  return check_launch("gather_rows");
}
