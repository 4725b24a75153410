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
#define NF_CHAIN_CLASS 4
#include "common.cuh"

namespace nf {

// One block per row.  A thread owns pairs of elements: the rotated pair (i, i + rot/2) of a
// q or k head, or two neighbouring elements that are only biased and copied (dims beyond
// `rot`, and every dim of a v head).  Owning both elements of a pair, it can write q back in
// place without a barrier.
template <typename T>
__global__ void __launch_bounds__(256)
rope_append_kernel(T* __restrict__ qkv, const float* __restrict__ bias,
                   const int* __restrict__ positions, const int* __restrict__ row_seg,
                   const float* __restrict__ inv_freq, int rot, int Hq, int Hkv, int D,
                   T* __restrict__ pages, const int* __restrict__ block_table, int bt_width,
                   int page_size, int num_pages, int append) {
  extern __shared__ float cs[];            // [rot/2] cos, [rot/2] sin
  const int t = blockIdx.x;
  const int half = rot / 2;
  const int pos = positions[t];
  const float fpos = (float)pos;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float angle = fpos * inv_freq[i];
    cs[i] = cosf(angle);
    cs[half + i] = sinf(angle);
  }
  __syncthreads();
  const int W = (Hq + 2 * Hkv) * D;
  T* x = qkv + (size_t)t * W;
  // where this row's keys and values go
  T* kdst = nullptr;
  if (append) {
    const int seg = row_seg[t];
    const int lp = pos / page_size;
    const int page = (lp >= 0 && lp < bt_width) ? block_table[(size_t)seg * bt_width + lp] : -1;
    if (page >= 0 && page < num_pages)       // no page reserved: never write out of bounds
      kdst = pages + ((size_t)page * 2 * Hkv * page_size + (size_t)(pos - lp * page_size)) * D;
  }
  const size_t kv_head_stride = (size_t)page_size * D;
  const int slots = D / 2;
  const int heads = append ? Hq + 2 * Hkv : Hq;
  for (int idx = threadIdx.x; idx < heads * slots; idx += blockDim.x) {
    const int head = idx / slots, s = idx - head * slots;
    const bool is_q = head < Hq, is_v = head >= Hq + Hkv;
    int i0, i1;
    bool rotate = false;
    if (!is_v && s < half) { i0 = s; i1 = s + half; rotate = true; }
    else if (!is_v) { i0 = rot + 2 * (s - half); i1 = i0 + 1; }
    else { i0 = 2 * s; i1 = i0 + 1; }
    const size_t base = (size_t)head * D;
    float a = to_float(x[base + i0]), b = to_float(x[base + i1]);
    if (bias) { a += bias[base + i0]; b += bias[base + i1]; }
    if (rotate) {
      const float c = cs[s], sn = cs[half + s];
      const float ra = a * c - b * sn, rb = a * sn + b * c;
      a = ra; b = rb;
    }
    if (is_q) {
      x[base + i0] = from_float<T>(a);
      x[base + i1] = from_float<T>(b);
    } else if (kdst) {
      const int kvh = is_v ? head - Hq - Hkv : head - Hq;
      T* dst = kdst + ((size_t)(is_v ? Hkv : 0) + kvh) * kv_head_stride;
      dst[i0] = from_float<T>(a);
      dst[i1] = from_float<T>(b);
    }
  }
}

// bfloat16, rotation over the whole head (rot == D, D % 16 == 0): a thread owns 8 consecutive
// dims of the low half and the 8 matching dims of the high half of one head, 16 bytes each way.
__global__ void __launch_bounds__(256)
rope_append_bf16x8_kernel(__nv_bfloat16* __restrict__ qkv, const float* __restrict__ bias,
                          const int* __restrict__ positions, const int* __restrict__ row_seg,
                          const float* __restrict__ inv_freq, int Hq, int Hkv, int D,
                          __nv_bfloat16* __restrict__ pages, const int* __restrict__ block_table,
                          int bt_width, int page_size, int num_pages, int append) {
  extern __shared__ __align__(16) float cs[];            // [D/2] cos, [D/2] sin
  const int t = blockIdx.x;
  const int half = D / 2;
  chain_release();
  chain_wait(qkv, positions, row_seg, block_table);
  const int pos = positions[t];
  const int W = (Hq + 2 * Hkv) * D;
  __nv_bfloat16* x = qkv + (size_t)t * W;
  const int groups = half / 8;             // 8-dim groups per half head
  const int heads = append ? Hq + 2 * Hkv : Hq;
  const int n_items = heads * groups;
  bool have_table = false;
  __nv_bfloat16* kdst = nullptr;
  const size_t kv_head_stride = (size_t)page_size * D;
  // Two items a thread and round: the row's values are asked for first, the cosines and sines
  // and the page lookup are worked out while they are on their way.
  for (int idx0 = threadIdx.x; idx0 - (int)threadIdx.x < n_items; idx0 += 2 * blockDim.x) {
    uint4 ra[2], rb[2];
    int head[2], gi[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int idx = idx0 + u * blockDim.x;
      head[u] = idx / groups;
      gi[u] = idx - head[u] * groups;
      if (idx < n_items) {
        const __nv_bfloat16* src = x + (size_t)head[u] * D + gi[u] * 8;
        ra[u] = *reinterpret_cast<const uint4*>(src);
        rb[u] = *reinterpret_cast<const uint4*>(src + half);
      }
    }
    if (!have_table) {
      const float fpos = (float)pos;
      for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float angle = fpos * inv_freq[i];
        cs[i] = cosf(angle);
        cs[half + i] = sinf(angle);
      }
      if (append) {
        const int seg = row_seg[t];
        const int lp = pos / page_size;
        const int page = (lp >= 0 && lp < bt_width) ? block_table[(size_t)seg * bt_width + lp] : -1;
        if (page >= 0 && page < num_pages)
          kdst = pages + ((size_t)page * 2 * Hkv * page_size + (size_t)(pos - lp * page_size)) * D;
      }
      __syncthreads();
      have_table = true;
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (idx0 + u * (int)blockDim.x >= n_items) continue;
      const bool is_q = head[u] < Hq, is_v = head[u] >= Hq + Hkv;
      const size_t base = (size_t)head[u] * D;
      const int i0 = gi[u] * 8, i1 = half + gi[u] * 8;
      float a[8], b[8];
      unpack8(ra[u], a);
      unpack8(rb[u], b);
      if (bias) {
        // 16-byte loads: one float at a time, a warp's loads of a bias touch eight lines each
        float ba[8], bb[8];
        load8(bias + base + i0, ba);
        load8(bias + base + i1, bb);
#pragma unroll
        for (int e = 0; e < 8; ++e) { a[e] += ba[e]; b[e] += bb[e]; }
      }
      if (!is_v) {
        float c[8], sn[8];
        load8(cs + i0, c);
        load8(cs + half + i0, sn);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float xa = a[e] * c[e] - b[e] * sn[e], xb = a[e] * sn[e] + b[e] * c[e];
          a[e] = xa; b[e] = xb;
        }
      }
      __align__(16) __nv_bfloat16 oa[8], ob[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) { oa[e] = __float2bfloat16_rn(a[e]); ob[e] = __float2bfloat16_rn(b[e]); }
      __nv_bfloat16* dst = nullptr;
      if (is_q) dst = x + base;
      else if (kdst) dst = kdst + ((size_t)(is_v ? Hkv : 0) + (is_v ? head[u] - Hq - Hkv : head[u] - Hq)) * kv_head_stride;
      if (dst) {
        *reinterpret_cast<uint4*>(dst + i0) = *reinterpret_cast<const uint4*>(oa);
        *reinterpret_cast<uint4*>(dst + i1) = *reinterpret_cast<const uint4*>(ob);
      }
    }
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
  NF_REQUIRE(D % 2 == 0, "rope_append: head_dim %d must be even", D);
  const size_t smem = (size_t)rot * sizeof(float);
  NF_REQUIRE(smem <= 48 * 1024, "rope_append: rotary width %d too large", rot);
  if (dtype == kBF16 && rot == D && D % 16 == 0 && (uintptr_t)qkv % 16 == 0 && (uintptr_t)pages % 16 == 0 &&
      (uintptr_t)bias % 16 == 0) {
    launch_chained(rope_append_bf16x8_kernel, dim3(T), dim3(256), smem, stream, (__nv_bfloat16*)qkv, bias, positions, row_seg, inv_freq, Hq, Hkv, D, (__nv_bfloat16*)pages, block_table, bt_width, page_size, num_pages, append);
    return check_launch("rope_append");
  }
  if (dtype == kF32)
    rope_append_kernel<float><<<T, 256, smem, stream>>>((float*)qkv, bias, positions, row_seg, inv_freq, rot, Hq, Hkv, D, (float*)pages, block_table, bt_width, page_size, num_pages, append);
  else
    rope_append_kernel<__nv_bfloat16><<<T, 256, smem, stream>>>((__nv_bfloat16*)qkv, bias, positions, row_seg, inv_freq, rot, Hq, Hkv, D, (__nv_bfloat16*)pages, block_table, bt_width, page_size, num_pages, append);
  return check_launch("rope_append");
}
