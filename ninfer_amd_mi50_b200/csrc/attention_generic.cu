// Causal grouped-query attention over the paged cache, for any mix of rows: the plain,
// always-applicable kernel (one warp per row and query head).
//
// Same mathematics as the reference's two kernels (src/ops/attention.hip:14-94 decode,
// 136-268 prefill): q head h reads kv head h / (Hq / Hkv); score = (q . k) * scale; key j
// is visible to a row at position p iff lo <= j <= p with lo = 0, or p - window + 1 with a
// window; online softmax (running max m, sum l, rescale exp(m_old - m_new)); o = acc / l.
// Scores, max, exp, sums and the accumulator are float32.  Keys are visited in blocks of
// 32 in ascending order from `lo`, so a row's result depends only on its own position,
// never on how the prompt was cut or what else is in the batch.
#include "common.cuh"

namespace nf {

constexpr int kMaxDimsPerLane = 8;   // head_dim <= 256

template <typename T>
__global__ void __launch_bounds__(128)
paged_attention_generic_kernel(const T* __restrict__ qkv, int q_row_stride,
                               const T* __restrict__ pages, const int* __restrict__ block_table,
                               int bt_width, const int* __restrict__ positions,
                               const int* __restrict__ row_seg, T* __restrict__ out, int Hq,
                               int Hkv, int D, int page_size, int num_pages, int window,
                               float scale) {
  extern __shared__ float q_smem[];          // [4 warps][D]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int h = blockIdx.y * 4 + warp;
  if (h >= Hq) return;
  float* q = q_smem + warp * D;
  const T* qrow = qkv + (size_t)t * q_row_stride + (size_t)h * D;
  for (int d = lane; d < D; d += 32) q[d] = to_float(qrow[d]);
  __syncwarp();

  const int kvh = h / (Hq / Hkv);
  const int pos = positions[t];
  const int seg = row_seg[t];
  const int* bt = block_table + (size_t)seg * bt_width;
  int lo = 0;
  if (window > 0 && pos - window + 1 > 0) lo = pos - window + 1;
  const size_t head_stride = (size_t)page_size * D;            // one kv head inside a page
  const size_t page_stride = (size_t)2 * Hkv * head_stride;

  float m = -INFINITY, l = 0.f;
  float acc[kMaxDimsPerLane];
#pragma unroll
  for (int i = 0; i < kMaxDimsPerLane; ++i) acc[i] = 0.f;

  for (int j0 = lo; j0 <= pos; j0 += 32) {
    const int j = j0 + lane;
    float s = -INFINITY;
    const T* vrow = nullptr;
    if (j <= pos) {
      const int lp = j / page_size;
      const int page = lp < bt_width ? bt[lp] : -1;
      if (page >= 0 && page < num_pages) {
        const T* krow = pages + (size_t)page * page_stride + (size_t)kvh * head_stride +
                        (size_t)(j % page_size) * D;
        vrow = krow + (size_t)Hkv * head_stride;
        float dot = 0.f;
        for (int d = 0; d < D; d += 8) {
          float kk[8];
          load8(krow + d, kk);
#pragma unroll
          for (int e = 0; e < 8; ++e) dot = fmaf(q[d + e], kk[e], dot);
        }
        s = dot * scale;
      }
    }
    const float m_new = fmaxf(m, warp_max(s));
    if (m_new == -INFINITY) continue;      // no visible key in this block (cannot happen for j0 <= pos)
    const float p = (s == -INFINITY) ? 0.f : expf(s - m_new);
    const float alpha = (m == -INFINITY) ? 0.f : expf(m - m_new);
    l = l * alpha + warp_sum(p);
    m = m_new;
#pragma unroll
    for (int i = 0; i < kMaxDimsPerLane; ++i) acc[i] *= alpha;
    const int nkeys = min(32, pos - j0 + 1);
    for (int jj = 0; jj < nkeys; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const unsigned long long vp = __shfl_sync(0xffffffffu, (unsigned long long)vrow, jj);
      if (vp == 0ull) continue;
      const T* vr = reinterpret_cast<const T*>(vp);
#pragma unroll
      for (int i = 0; i < kMaxDimsPerLane; ++i) {
        const int d = lane + 32 * i;
        if (d < D) acc[i] = fmaf(pj, to_float(vr[d]), acc[i]);
      }
    }
  }
  const float inv_l = l > 0.f ? 1.f / l : 0.f;
  T* o = out + (size_t)t * Hq * D + (size_t)h * D;
#pragma unroll
  for (int i = 0; i < kMaxDimsPerLane; ++i) {
    const int d = lane + 32 * i;
    if (d < D) o[d] = from_float<T>(acc[i] * inv_l);
  }
}

}  // namespace nf

using namespace nf;

extern "C" int nf_paged_attention_generic(const void* qkv, int q_row_stride, const void* pages,
                                          const int* block_table, int bt_width,
                                          const int* positions, const int* row_seg, void* out,
                                          int T, int Hq, int Hkv, int D, int page_size,
                                          int num_pages, int window, float scale, int dtype,
                                          cudaStream_t stream) {
  if (T == 0) return 0;
  NF_REQUIRE(T > 0 && Hq > 0 && Hkv > 0 && Hq % Hkv == 0, "attention: bad sizes T=%d Hq=%d Hkv=%d", T, Hq, Hkv);
  NF_REQUIRE(D % 16 == 0 && D >= 16 && D <= 256, "attention: head_dim %d must be a multiple of 16 in [16, 256]", D);
  dim3 grid(T, (Hq + 3) / 4);
  const size_t smem = 4 * D * sizeof(float);
  if (dtype == kF32)
    paged_attention_generic_kernel<float><<<grid, 128, smem, stream>>>((const float*)qkv, q_row_stride, (const float*)pages, block_table, bt_width, positions, row_seg, (float*)out, Hq, Hkv, D, page_size, num_pages, window, scale);
  else
    paged_attention_generic_kernel<__nv_bfloat16><<<grid, 128, smem, stream>>>((const __nv_bfloat16*)qkv, q_row_stride, (const __nv_bfloat16*)pages, block_table, bt_width, positions, row_seg, (__nv_bfloat16*)out, Hq, Hkv, D, page_size, num_pages, window, scale);
  return check_launch("paged_attention_generic");
}
