// Decode attention in bfloat16: every row is one request's newest token and reads that
// request's whole cache.  The work is reading keys and values once, so it is split over
// the keys: one CTA per (row, kv head, block of 128 keys) writes an unnormalised partial
// result with its running maximum and sum, and a second kernel merges the blocks in
// ascending order.
//
// Reference: ``decode_attention_kernel`` (src/ops/attention.hip:14-94) runs one block per
// query head over all keys in tiles of 256, with thread 0 doing the softmax bookkeeping
// serially; at batch 1 that is 16 blocks on the whole device.  Same mathematics here
// (scores * 1/sqrt(D), online softmax in float32, o = acc / l), different decomposition.
// Key blocks are aligned to absolute key indices, so the partition, and with it the
// order of every sum, depends on the row's own position (and window) only.
//
// All query heads of a group share the CTA, so keys and values are read once per kv head.
#include "common.cuh"

namespace nf {

constexpr int kSplit = 128;        // keys per CTA
constexpr int kHeadChunk = 4;      // query heads of a group handled per pass over the keys
constexpr int kU = 4;              // key rows in flight per lane

// Workspace layout per (row, q head, split): D floats of acc, then (m, l) in a separate array.
template <int D>
__global__ void __launch_bounds__(128)
decode_attention_split_kernel(const __nv_bfloat16* __restrict__ qkv, int q_row_stride,
                              const __nv_bfloat16* __restrict__ pages,
                              const int* __restrict__ block_table, int bt_width,
                              const int* __restrict__ positions, const int* __restrict__ row_seg,
                              float* __restrict__ ws_acc, float* __restrict__ ws_ml, int Hq, int Hkv,
                              int page_size, int num_pages, int window, float scale, int nsplit) {
  constexpr int LPR = D / 8;            // lanes that cover one key row with 16-byte loads
  constexpr int RPL = 32 / LPR;         // key rows per warp-wide load
  extern __shared__ float smem[];
  const int G = Hq / Hkv;
  float* qs = smem;                     // [G][D]
  float* sc = qs + G * D;               // [G][kSplit]
  float* red = sc + G * kSplit;         // [4 warps][kHeadChunk][D] partial outputs
  float* ml = red + 4 * kHeadChunk * D; // [G][2]
  const int t = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pos = positions[t];
  int lo = 0;
  if (window > 0 && pos - window + 1 > 0) lo = pos - window + 1;
  const int k_base = split * kSplit;
  const int k_begin = max(lo, k_base);
  const int k_end = min(pos + 1, k_base + kSplit);
  if (k_begin >= k_end) return;
  const int seg = row_seg[t];
  const int* bt = block_table + (size_t)seg * bt_width;
  const size_t head_stride = (size_t)page_size * D;
  const size_t page_stride = (size_t)2 * Hkv * head_stride;

  for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
    const int h = i / D, d = i - h * D;
    qs[i] = __bfloat162float(qkv[(size_t)t * q_row_stride + (size_t)(kvh * G + h) * D + d]);
  }
  __syncthreads();

  const int sub = lane / LPR, li = lane % LPR;

  // ---- scores -------------------------------------------------------------------------
  for (int h0 = 0; h0 < G; h0 += kHeadChunk) {
    const int nh = min(kHeadChunk, G - h0);
    for (int j0 = k_begin + warp * RPL; j0 < k_end; j0 += 4 * RPL * kU) {
      float kk[kU][8];
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const int j = j0 + u * 4 * RPL + sub;
#pragma unroll
        for (int e = 0; e < 8; ++e) kk[u][e] = 0.f;
        if (j < k_end) {
          const int lp = j / page_size;
          const int page = lp < bt_width ? bt[lp] : -1;
          if (page >= 0 && page < num_pages)
            load8(pages + (size_t)page * page_stride + (size_t)kvh * head_stride +
                  (size_t)(j % page_size) * D + li * 8, kk[u]);
        }
      }
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const int j = j0 + u * 4 * RPL + sub;
        const bool valid = j < k_end;
#pragma unroll
        for (int hh = 0; hh < kHeadChunk; ++hh) {
          if (hh < nh) {
            const float* qh = qs + (h0 + hh) * D + li * 8;
            float dot = 0.f;
#pragma unroll
            for (int e = 0; e < 8; ++e) dot = fmaf(qh[e], kk[u][e], dot);
#pragma unroll
            for (int o = LPR / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
            if (valid && li == 0) sc[(h0 + hh) * kSplit + (j - k_base)] = dot * scale;
          }
        }
      }
    }
  }
  __syncthreads();

  // ---- per head: maximum, exponentials, sum (one warp per head) ----------------------------
  const int n0 = k_begin - k_base, n1 = k_end - k_base;
  for (int h = warp; h < G; h += 4) {
    float m = -INFINITY;
    for (int i = n0 + lane; i < n1; i += 32) m = fmaxf(m, sc[h * kSplit + i]);
    m = warp_max(m);
    float l = 0.f;
    for (int i = n0 + lane; i < n1; i += 32) {
      const float p = expf(sc[h * kSplit + i] - m);
      sc[h * kSplit + i] = p;
      l += p;
    }
    l = warp_sum(l);
    if (lane == 0) { ml[2 * h] = m; ml[2 * h + 1] = l; }
  }
  __syncthreads();

  // ---- acc = sum_j p_j v_j ------------------------------------------------------------------
  for (int h0 = 0; h0 < G; h0 += kHeadChunk) {
    const int nh = min(kHeadChunk, G - h0);
    float acc[kHeadChunk][8];
#pragma unroll
    for (int hh = 0; hh < kHeadChunk; ++hh)
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[hh][e] = 0.f;
    for (int j0 = k_begin + warp * RPL; j0 < k_end; j0 += 4 * RPL * kU) {
      float vv[kU][8];
      bool have[kU];
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const int j = j0 + u * 4 * RPL + sub;
        have[u] = false;
        if (j < k_end) {
          const int lp = j / page_size;
          const int page = lp < bt_width ? bt[lp] : -1;
          if (page >= 0 && page < num_pages) {
            load8(pages + (size_t)page * page_stride + (size_t)(Hkv + kvh) * head_stride +
                  (size_t)(j % page_size) * D + li * 8, vv[u]);
            have[u] = true;
          }
        }
      }
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        if (have[u]) {
          const int j = j0 + u * 4 * RPL + sub;
#pragma unroll
          for (int hh = 0; hh < kHeadChunk; ++hh) {
            if (hh < nh) {
              const float p = sc[(h0 + hh) * kSplit + (j - k_base)];
#pragma unroll
              for (int e = 0; e < 8; ++e) acc[hh][e] = fmaf(p, vv[u][e], acc[hh][e]);
            }
          }
        }
      }
    }
    // lanes with the same `li` hold different key rows: add them, then add the warps in order
#pragma unroll
    for (int hh = 0; hh < kHeadChunk; ++hh)
#pragma unroll
      for (int e = 0; e < 8; ++e)
#pragma unroll
        for (int o = LPR; o < 32; o <<= 1) acc[hh][e] += __shfl_xor_sync(0xffffffffu, acc[hh][e], o);
    if (sub == 0) {
#pragma unroll
      for (int hh = 0; hh < kHeadChunk; ++hh)
#pragma unroll
        for (int e = 0; e < 8; ++e) red[(warp * kHeadChunk + hh) * D + li * 8 + e] = acc[hh][e];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < nh * D; i += blockDim.x) {
      const int hh = i / D, d = i - hh * D;
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) s += red[(w * kHeadChunk + hh) * D + d];
      const int hq = kvh * G + h0 + hh;
      ws_acc[(((size_t)t * Hq + hq) * nsplit + split) * D + d] = s;
    }
    __syncthreads();
  }
  for (int h = threadIdx.x; h < G; h += blockDim.x) {
    const int hq = kvh * G + h;
    float* o = ws_ml + (((size_t)t * Hq + hq) * nsplit + split) * 2;
    o[0] = ml[2 * h];
    o[1] = ml[2 * h + 1];
  }
}

// One block per (row, q head): merge the splits of the row's key range in ascending order.
template <typename T>
__global__ void decode_attention_merge_kernel(const float* __restrict__ ws_acc,
                                              const float* __restrict__ ws_ml,
                                              const int* __restrict__ positions, T* __restrict__ out,
                                              int Hq, int D, int window, int nsplit) {
  const int t = blockIdx.x, h = blockIdx.y;
  const int pos = positions[t];
  int lo = 0;
  if (window > 0 && pos - window + 1 > 0) lo = pos - window + 1;
  const int s0 = lo / kSplit, s1 = pos / kSplit;      // first and last split with keys
  const float* ml = ws_ml + ((size_t)t * Hq + h) * nsplit * 2;
  const float* acc = ws_acc + ((size_t)t * Hq + h) * nsplit * D;
  float m = -INFINITY;
  for (int s = s0; s <= s1 && s < nsplit; ++s) m = fmaxf(m, ml[2 * s]);
  float l = 0.f;
  for (int s = s0; s <= s1 && s < nsplit; ++s) l += ml[2 * s + 1] * expf(ml[2 * s] - m);
  const float inv_l = l > 0.f ? 1.f / l : 0.f;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float o = 0.f;
    for (int s = s0; s <= s1 && s < nsplit; ++s) o += acc[(size_t)s * D + d] * expf(ml[2 * s] - m);
    out[((size_t)t * Hq + h) * D + d] = from_float<T>(o * inv_l);
  }
}

template <int D>
static int launch_split(const void* qkv, int q_row_stride, const void* pages, const int* block_table,
                        int bt_width, const int* positions, const int* row_seg, float* ws_acc,
                        float* ws_ml, int T, int Hq, int Hkv, int page_size, int num_pages, int window,
                        float scale, int nsplit, cudaStream_t stream) {
  const int G = Hq / Hkv;
  const size_t smem = ((size_t)G * D + (size_t)G * kSplit + 4 * kHeadChunk * D + 2 * G) * sizeof(float);
  NF_REQUIRE(smem <= 160 * 1024, "decode attention: %d query heads per kv head need too much shared memory", G);
  static size_t allowed = 48 * 1024;
  if (smem > allowed) {
    cudaFuncSetAttribute(decode_attention_split_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    allowed = smem;
  }
  dim3 grid(T, Hkv, nsplit);
  decode_attention_split_kernel<D><<<grid, 128, smem, stream>>>(
      (const __nv_bfloat16*)qkv, q_row_stride, (const __nv_bfloat16*)pages, block_table, bt_width, positions,
      row_seg, ws_acc, ws_ml, Hq, Hkv, page_size, num_pages, window, scale, nsplit);
  return check_launch("decode_attention_split");
}

}  // namespace nf

using namespace nf;

extern "C" int nf_decode_attention_split_size() { return kSplit; }

// bfloat16 only; head_dim in {16, 32, 64, 128, 256}.  `nsplit` >= ceil(max context / 128) of
// the rows in this call.  Workspace: ws_acc float32 [T, Hq, nsplit, D], ws_ml [T, Hq, nsplit, 2].
extern "C" int nf_decode_attention(const void* qkv, int q_row_stride, const void* pages,
                                   const int* block_table, int bt_width, const int* positions,
                                   const int* row_seg, void* out, float* ws_acc, float* ws_ml, int T,
                                   int Hq, int Hkv, int D, int page_size, int num_pages, int window,
                                   float scale, int nsplit, cudaStream_t stream) {
  if (T == 0) return 0;
  NF_REQUIRE(T > 0 && Hq > 0 && Hkv > 0 && Hq % Hkv == 0 && nsplit > 0, "decode attention: bad sizes T=%d Hq=%d Hkv=%d nsplit=%d", T, Hq, Hkv, nsplit);
  NF_REQUIRE(Hkv <= 65535 && nsplit <= 65535, "decode attention: too many kv heads or key blocks");
  int rc;
  switch (D) {
    case 16: rc = launch_split<16>(qkv, q_row_stride, pages, block_table, bt_width, positions, row_seg, ws_acc, ws_ml, T, Hq, Hkv, page_size, num_pages, window, scale, nsplit, stream); break;
    case 32: rc = launch_split<32>(qkv, q_row_stride, pages, block_table, bt_width, positions, row_seg, ws_acc, ws_ml, T, Hq, Hkv, page_size, num_pages, window, scale, nsplit, stream); break;
    case 64: rc = launch_split<64>(qkv, q_row_stride, pages, block_table, bt_width, positions, row_seg, ws_acc, ws_ml, T, Hq, Hkv, page_size, num_pages, window, scale, nsplit, stream); break;
    case 128: rc = launch_split<128>(qkv, q_row_stride, pages, block_table, bt_width, positions, row_seg, ws_acc, ws_ml, T, Hq, Hkv, page_size, num_pages, window, scale, nsplit, stream); break;
    case 256: rc = launch_split<256>(qkv, q_row_stride, pages, block_table, bt_width, positions, row_seg, ws_acc, ws_ml, T, Hq, Hkv, page_size, num_pages, window, scale, nsplit, stream); break;
    default:
      set_error("decode attention: head_dim %d is not one of 16, 32, 64, 128, 256", D);
      return 1;
  }
  if (rc) return rc;
  dim3 grid(T, Hq);
  int threads = 32;
  while (threads < D && threads < 256) threads <<= 1;
  decode_attention_merge_kernel<__nv_bfloat16><<<grid, threads, 0, stream>>>(ws_acc, ws_ml, positions, (__nv_bfloat16*)out, Hq, D, window, nsplit);
  return check_launch("decode_attention_merge");
}
