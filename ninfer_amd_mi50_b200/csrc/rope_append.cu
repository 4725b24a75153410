// The stage after the QKV projection: add the bias, rotate queries and keys by their
// positions, write keys and values into the request's cache pages.
//
// Reference: ``post_qkv_kernel`` / ``post_qkv_batch_kernel`` (src/ops/gemv.hip:205-326)
// for single rows, ``rope_kernel`` (src/ops/kernels.hip:73-94) + ``KVCache::append``
// (src/runtime/kv_cache.cpp:27-47) for portions.  One kernel serves both here: a row
// carries its own position and its own segment, so a batch may mix prompt portions and
// decoded tokens.  Half-split pairing over the first `rot` dims of a head:
//   angle = float(pos) * inv_freq[i];  x'[i] = x[i] cos - x[i+rot/2] sin;
//   x'[i+rot/2] = x[i] sin + x[i+rot/2] cos          (angle, cos, sin, products in float32)
// Cache page layout: [2 (k, v)][kv_heads][page_size][head_dim].
#include "common.cuh"

namespace nf {

template <typename T>
__global__ void rope_append_kernel(T* __restrict__ qkv, const float* __restrict__ bias,
                                   const int* __restrict__ positions,
                                   const int* __restrict__ row_seg,
                                   const float* __restrict__ inv_freq, int rot, int Hq, int Hkv,
                                   int D, T* __restrict__ pages, const int* __restrict__ block_table,
                                   int bt_width, int page_size, int num_pages) {
  const int t = blockIdx.x;
  const int head = blockIdx.y;           // [0,Hq) q, [Hq,Hq+Hkv) k, [Hq+Hkv, Hq+2Hkv) v
  const int W = (Hq + 2 * Hkv) * D;
  T* x = qkv + (size_t)t * W + (size_t)head * D;
  const float* b = bias ? bias + (size_t)head * D : nullptr;
  const int pos = positions[t];
  const bool is_q = head < Hq;
  const bool is_v = head >= Hq + Hkv;

  T* dst = nullptr;                       // where the k / v head goes in the cache
  if (!is_q) {
    const int seg = row_seg[t];
    const int lp = pos / page_size;
    int page = (lp >= 0 && lp < bt_width) ? block_table[(size_t)seg * bt_width + lp] : -1;
    if (page < 0 || page >= num_pages) return;   // no page reserved: never write out of bounds
    const int kvh = is_v ? head - Hq - Hkv : head - Hq;
    dst = pages + ((((size_t)page * 2 + (is_v ? 1 : 0)) * Hkv + kvh) * page_size + pos % page_size) * D;
  }
  const int half = rot / 2;
  const float fpos = (float)pos;
  // blockDim.x >= D: one sweep covers the head, so the barrier below is uniform
  const int i = threadIdx.x;
  float v = 0.f;
  if (i < D) {
    v = to_float(x[i]) + (b ? b[i] : 0.f);
    if (!is_v && i < rot) {
      const int j = i < half ? i : i - half;
      const int partner = i < half ? i + half : i - half;
      const float other = to_float(x[partner]) + (b ? b[partner] : 0.f);
      const float angle = fpos * inv_freq[j];
      const float c = cosf(angle), s = sinf(angle);
      v = i < half ? v * c - other * s : other * s + v * c;
    }
  }
  // every thread has read what it needs from x before anyone overwrites it
  __syncthreads();
  if (i < D) {
    if (is_q) x[i] = from_float<T>(v);
    else dst[i] = from_float<T>(v);
  }
}

}  // namespace nf

using namespace nf;

extern "C" int nf_rope_append(void* qkv, const float* bias, const int* positions, const int* row_seg,
                              const float* inv_freq, int rot, int T, int Hq, int Hkv, int D,
                              void* pages, const int* block_table, int bt_width, int page_size,
                              int num_pages, int append, int dtype, cudaStream_t stream) {
  if (T == 0) return 0;
  NF_REQUIRE(T > 0 && Hq > 0 && Hkv > 0 && D > 0, "rope_append: bad sizes T=%d Hq=%d Hkv=%d D=%d", T, Hq, Hkv, D);
  NF_REQUIRE(rot >= 0 && rot <= D && rot % 2 == 0, "rope_append: rotary width %d must be even and <= head_dim %d", rot, D);
  NF_REQUIRE(rot == 0 || inv_freq, "rope_append: rotation asked without a frequency table");
  NF_REQUIRE(Hq + 2 * Hkv <= 65535, "rope_append: too many heads");
  // one block covers a whole head in a single sweep
  int threads = 32;
  while (threads < D) threads <<= 1;
  NF_REQUIRE(threads <= 1024, "rope_append: head_dim %d too large", D);
  dim3 grid(T, append ? Hq + 2 * Hkv : Hq);
  if (dtype == kF32)
    rope_append_kernel<float><<<grid, threads, 0, stream>>>((float*)qkv, bias, positions, row_seg, inv_freq, rot, Hq, Hkv, D, (float*)pages, block_table, bt_width, page_size, num_pages);
  else
    rope_append_kernel<__nv_bfloat16><<<grid, threads, 0, stream>>>((__nv_bfloat16*)qkv, bias, positions, row_seg, inv_freq, rot, Hq, Hkv, D, (__nv_bfloat16*)pages, block_table, bt_width, page_size, num_pages);
  return check_launch("rope_append");
}
