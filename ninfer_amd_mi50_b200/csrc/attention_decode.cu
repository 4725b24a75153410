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
#define NF_CHAIN_CLASS 8
#include "common.cuh"
#include "decode_range.cuh"

namespace nf {

constexpr int kSplit = 128;        // keys per CTA

// 1 + a row whose position lay beyond the key blocks that a call allowed for (see decode_range.cuh);
// read and reset by nf_decode_attention_status
__device__ int g_decode_split_range_error = 0;

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gmem_src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void mma16816(float* c, unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

// Workspace per (row, q head, split): D floats of unnormalised output, and (m, l) apart.
// The CTA first asks for all of its keys and values (asynchronous copies into shared
// memory, so that all 2 * 128 * D * 2 bytes are in flight at once).  Scores and the
// weighted sum of values are tensor-core products with the keys (values) as the 16-row
// operand and up to 8 query heads of the group as the 8-column operand; softmax stays in
// float32 in between.  Warp w owns keys [32 w, 32 w + 32) of the block.
template <int D>
__global__ void __launch_bounds__(128)
decode_attention_split_kernel(const __nv_bfloat16* __restrict__ qkv, int q_row_stride,
                              const __nv_bfloat16* __restrict__ pages,
                              const int* __restrict__ block_table, int bt_width,
                              const int* __restrict__ positions, const int* __restrict__ row_seg,
                              float* __restrict__ ws_acc, float* __restrict__ ws_ml, int Hq, int Hkv,
                              int page_size, int num_pages, int window, float scale, int nsplit,
                              int* __restrict__ counters, __nv_bfloat16* __restrict__ out,
                              const int* __restrict__ row_list) {
  constexpr int LPR = D / 8;            // 16-byte pieces of one key row
  constexpr int RPL = 32 / LPR;         // key rows a warp copies at once
  constexpr int DS = D + 8;             // shared-memory row stride: 16 bytes of padding keep
                                        // ldmatrix free of bank conflicts
  constexpr int HC = 8;                 // query heads per tensor-core pass
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int G = Hq / Hkv;
  __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // [kSplit][DS]
  __nv_bfloat16* Vs = Ks + kSplit * DS;                             // [kSplit][DS]
  float* sc = reinterpret_cast<float*>(Vs + kSplit * DS);           // [G][kSplit] scores, then p
  const int RH = min(G, HC);                                        // heads kept per pass
  float* red = sc + G * kSplit;                                     // [4 warps][RH][D]
  float* ml = red + 4 * RH * D;                                     // [G][2]
  // wi: the row's place in this launch (workspace, counters); t: the row itself
  const int wi = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tq = lane & 3;
  chain_release_if_small();
  // Positions, row list, segments and block table are the step's inputs, complete before the
  // step's kernels began.  The kernel before this one wrote the queries and, into the pages, the
  // keys and values of each row's own (newest) position - nothing else.  So everything but that
  // one row of keys and values is asked for before the wait, while that kernel still runs.
  const int t = row_list ? row_list[wi] : wi;
  const int newest = positions[t];
  int pos = newest, lo;
  if (decode_key_range(pos, lo, window, nsplit, kSplit) && kvh == 0 && split == 0 && threadIdx.x == 0)
    atomicCAS(&g_decode_split_range_error, 0, 1 + t);
  const int k_base = split * kSplit;
  const int k_begin = max(lo, k_base);
  const int k_end = min(pos + 1, k_base + kSplit);
  if (k_begin >= k_end) return;
  const int seg = row_seg[t];
  const int* bt = block_table + (size_t)seg * bt_width;
  const size_t head_stride = (size_t)page_size * D;
  const size_t page_stride = (size_t)2 * Hkv * head_stride;
  const size_t v_off = (size_t)Hkv * head_stride;
  const int n0 = k_begin - k_base, n1 = k_end - k_base;
  const int sub = lane / LPR, li = lane % LPR;
  const int new_row = (newest >= k_begin && newest < k_end) ? newest - k_base : -1;   // the row written a kernel ago

  // ---- ask for keys, then values; rows outside the key range become zeros --------------------
  // Lane l looks up the page of row 32 w + l once; the copy loop fetches each row's address
  // from the lane that knows it.
  const __nv_bfloat16* new_src = nullptr;
  {
    const int myrow = warp * 32 + lane;
    const __nv_bfloat16* my_src = nullptr;
    if (myrow >= n0 && myrow < n1) {
      const int j = k_base + myrow;
      const int lp = j / page_size;
      const int page = lp < bt_width ? bt[lp] : -1;
      if (page >= 0 && page < num_pages)
        my_src = pages + (size_t)page * page_stride + (size_t)kvh * head_stride + (size_t)(j - lp * page_size) * D;
    }
#pragma unroll
    for (int kv = 0; kv < 2; ++kv) {
      __nv_bfloat16* dst = kv ? Vs : Ks;
#pragma unroll 4
      for (int it = 0; it < 32 / RPL; ++it) {
        const int rl = it * RPL + sub;
        const unsigned long long src = __shfl_sync(0xffffffffu, (unsigned long long)my_src, rl);
        const int r = warp * 32 + rl;
        if (rl < 32) {
          if (r == new_row) new_src = reinterpret_cast<const __nv_bfloat16*>(src);      // after the wait
          else if (src) cp_async16(dst + r * DS + li * 8, reinterpret_cast<const __nv_bfloat16*>(src) + (kv ? v_off : 0) + li * 8);
          else *reinterpret_cast<uint4*>(dst + r * DS + li * 8) = make_uint4(0, 0, 0, 0);
        }
      }
      cp_async_commit();
    }
  }
  for (int i = threadIdx.x; i < G * kSplit; i += blockDim.x) sc[i] = 0.f;
  chain_wait(qkv, pages);
  if (new_row >= 0) {
    // the lanes that met the newest row in the loop above fetch it now (keys and values)
    if (warp == new_row / 32 && sub == (new_row & 31) % RPL) {
      if (new_src) {
        cp_async16(Ks + new_row * DS + li * 8, new_src + li * 8);
        cp_async16(Vs + new_row * DS + li * 8, new_src + v_off + li * 8);
      } else {
        *reinterpret_cast<uint4*>(Ks + new_row * DS + li * 8) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(Vs + new_row * DS + li * 8) = make_uint4(0, 0, 0, 0);
      }
    }
    cp_async_commit();
    cp_async_wait<0>();        // all three groups
  } else {
    cp_async_wait<1>();        // keys have landed (values may still be on their way)
  }
  __syncthreads();

  const __nv_bfloat16* qrow = qkv + (size_t)t * q_row_stride + (size_t)kvh * G * D;

  // ---- scores = K q^T: [32 keys of the warp] x [8 heads] per pass ---------------------------
  for (int h0 = 0; h0 < G; h0 += HC) {
    float c[2][4];
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
      for (int i = 0; i < 4; ++i) c[m][i] = 0.f;
    const bool head_ok = h0 + g < G;
    const __nv_bfloat16* qh = qrow + (size_t)(h0 + g) * D;
#pragma unroll
    for (int k0 = 0; k0 < D; k0 += 16) {
      unsigned b0 = 0, b1 = 0;
      if (head_ok) {
        b0 = *reinterpret_cast<const unsigned*>(qh + k0 + 2 * tq);
        b1 = *reinterpret_cast<const unsigned*>(qh + k0 + 2 * tq + 8);
      }
#pragma unroll
      for (int m = 0; m < 2; ++m) {
        unsigned a0, a1, a2, a3;
        const int row = warp * 32 + m * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        ldmatrix_x4(a0, a1, a2, a3, Ks + row * DS + k0 + (lane >> 4) * 8);
        mma16816(c[m], a0, a1, a2, a3, b0, b1);
      }
    }
    // c[m] = {(key g, head 2tq), (key g, head 2tq+1), (key g+8, head 2tq), (key g+8, head 2tq+1)}
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = warp * 32 + m * 16 + g + (i >> 1) * 8;
        const int h = h0 + 2 * tq + (i & 1);
        if (h < G && r >= n0 && r < n1) sc[h * kSplit + r] = c[m][i] * scale;
      }
  }
  __syncthreads();

  // ---- per head: maximum, exponentials, sum (one warp per head) ----------------------------
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
  cp_async_wait<0>();          // values have landed
  __syncthreads();
  chain_release_late();

  // ---- acc^T = V^T p^T: [D dims] x [8 heads], summed over the warp's 32 keys ------------------
  for (int h0 = 0; h0 < G; h0 += HC) {
    // p of head h0 + g for this lane's key columns, as bfloat16 pairs
    unsigned pb[2][2];
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
      const int j0 = warp * 32 + ks * 16;
      if (h0 + g < G) {
        const float* pr = sc + (h0 + g) * kSplit + j0;
        pb[ks][0] = pack_bf16(pr[2 * tq], pr[2 * tq + 1]);
        pb[ks][1] = pack_bf16(pr[2 * tq + 8], pr[2 * tq + 9]);
      } else {
        pb[ks][0] = pb[ks][1] = 0u;
      }
    }
#pragma unroll
    for (int d0 = 0; d0 < D; d0 += 16) {
      float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int ks = 0; ks < 2; ++ks) {
        unsigned a0, a1, a2, a3;
        const int mi = lane >> 3;
        const int row = warp * 32 + ks * 16 + (lane & 7) + (mi >> 1) * 8;
        ldmatrix_x4_trans(a0, a1, a2, a3, Vs + row * DS + d0 + (mi & 1) * 8);
        mma16816(c, a0, a1, a2, a3, pb[ks][0], pb[ks][1]);
      }
      // c = {(dim g, head 2tq), (dim g, head 2tq+1), (dim g+8, head 2tq), (dim g+8, head 2tq+1)}
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int hh = 2 * tq + (i & 1);
        if (hh < RH) red[(warp * RH + hh) * D + d0 + g + (i >> 1) * 8] = c[i];
      }
    }
    __syncthreads();
    const int nh = min(HC, G - h0);
    for (int i = threadIdx.x; i < nh * D; i += blockDim.x) {
      const int hh = i / D, d = i - hh * D;
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) s += red[(w * RH + hh) * D + d];
      const int hq = kvh * G + h0 + hh;
      ws_acc[(((size_t)wi * Hq + hq) * nsplit + split) * D + d] = s;
    }
    __syncthreads();
  }
  for (int h = threadIdx.x; h < G; h += blockDim.x) {
    const int hq = kvh * G + h;
    float* o = ws_ml + (((size_t)wi * Hq + hq) * nsplit + split) * 2;
    o[0] = ml[2 * h];
    o[1] = ml[2 * h + 1];
  }
  if (!counters) return;
  // ---- the CTA that finishes last for this (row, kv head) merges the key blocks -----------------
  // Which CTA that is does not matter: it reads every block's partial result and adds them in
  // ascending block order.  The counter is left at zero for the next launch.
  __shared__ int s_last;
  __threadfence();
  __syncthreads();
  const int s0 = lo / kSplit, s1 = pos / kSplit;
  if (threadIdx.x == 0) {
    const int prev = atomicAdd(&counters[wi * Hkv + kvh], 1);
    s_last = prev == s1 - s0;
    if (s_last) counters[wi * Hkv + kvh] = 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int h = 0; h < G; ++h) {
    const int hq = kvh * G + h;
    const float* mlp = ws_ml + ((size_t)wi * Hq + hq) * nsplit * 2;
    const float* accp = ws_acc + ((size_t)wi * Hq + hq) * nsplit * D;
    float m = -INFINITY;
    for (int s = s0; s <= s1; ++s) m = fmaxf(m, __ldcg(mlp + 2 * s));
    float l = 0.f;
    for (int s = s0; s <= s1; ++s) l += __ldcg(mlp + 2 * s + 1) * expf(__ldcg(mlp + 2 * s) - m);
    const float inv_l = l > 0.f ? 1.f / l : 0.f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
      float o = 0.f;
      for (int s = s0; s <= s1; ++s) o += __ldcg(accp + (size_t)s * D + d) * expf(__ldcg(mlp + 2 * s) - m);
      out[((size_t)t * Hq + hq) * D + d] = __float2bfloat16_rn(o * inv_l);
    }
  }
}

// One block per (row, q head): merge the splits of the row's key range in ascending order.
// The blocks' (m, l) go to shared memory in one parallel read; then every thread owns a few
// output dims and adds the blocks' partial outputs with weights exp(m_s - m) / l.
constexpr int kMaxMergeSplits = 1024;
constexpr int kMergeRun = 16;        // blocks one thread adds in a row
// dthreads: threads that share the D dims (a power of two); blockDim.x is a multiple of it.
// Dynamic shared memory: ceil(nsplit / kMergeRun) * D floats if nsplit > kMergeRun, else none.
template <typename T>
__global__ void decode_attention_merge_kernel(const float* __restrict__ ws_acc,
                                              const float* __restrict__ ws_ml,
                                              const int* __restrict__ positions, T* __restrict__ out,
                                              int Hq, int D, int window, int nsplit, int dthreads,
                                              const int* __restrict__ row_list) {
  extern __shared__ float runs[];      // [runs of this row][D]
  __shared__ float wgt[kMaxMergeSplits], wl[kMaxMergeSplits];
  __shared__ float s_m, s_inv;
  const int wi = blockIdx.x, h = blockIdx.y;
  chain_release_if_small();
  // positions and the row list are the step's inputs, complete before the kernels of the step
  // began; the partial results are the predecessor's
  const int t = row_list ? row_list[wi] : wi;
  int pos = positions[t], lo;
  decode_key_range(pos, lo, window, nsplit, kSplit);
  chain_wait(ws_acc, ws_ml);
  const int s0 = lo / kSplit, s1 = pos / kSplit;                       // first and last split with keys
  const int n = s1 - s0 + 1;
  const float* ml = ws_ml + (((size_t)wi * Hq + h) * nsplit + s0) * 2;
  const float* acc = ws_acc + (((size_t)wi * Hq + h) * nsplit + s0) * D;
  // every block's (m, l) in one parallel read; the serial parts below then walk shared memory
  for (int s = threadIdx.x; s < n; s += blockDim.x) {
    const float2 v = *reinterpret_cast<const float2*>(ml + 2 * s);
    wgt[s] = v.x;          // m_s for now
    wl[s] = v.y;
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    float m = -INFINITY;
    for (int s = threadIdx.x; s < n; s += 32) m = fmaxf(m, wgt[s]);
    m = warp_max(m);
    if (threadIdx.x == 0) s_m = m;
  }
  __syncthreads();
  for (int s = threadIdx.x; s < n; s += blockDim.x) wgt[s] = expf(wgt[s] - s_m);  // now exp(m_s - m)
  __syncthreads();
  if (threadIdx.x == 0) {
    float l = 0.f;
    for (int s = 0; s < n; ++s) l += wl[s] * wgt[s];                              // ascending order
    s_inv = l > 0.f ? 1.f / l : 0.f;
  }
  __syncthreads();
  // Runs of kMergeRun blocks are added by different thread groups (a long context has hundreds of
  // blocks, and one thread walking them all is a chain of memory latencies); the runs' sums are
  // then added in ascending order.  Which run a block falls in depends on the row's own range
  // only, so the order of the sum does too.
  const int nruns = (n + kMergeRun - 1) / kMergeRun;
  const int groups = blockDim.x / dthreads, group = threadIdx.x / dthreads, dl = threadIdx.x - group * dthreads;
  for (int r = group; r < nruns; r += groups) {
    const int sb = r * kMergeRun, se = min(n, sb + kMergeRun);
    for (int d = dl; d < D; d += dthreads) {
      float o = 0.f;
      int s = sb;
      for (; s + 4 <= se; s += 4) {
        const float a0 = acc[(size_t)s * D + d], a1 = acc[(size_t)(s + 1) * D + d];
        const float a2 = acc[(size_t)(s + 2) * D + d], a3 = acc[(size_t)(s + 3) * D + d];
        o += a0 * wgt[s];
        o += a1 * wgt[s + 1];
        o += a2 * wgt[s + 2];
        o += a3 * wgt[s + 3];
      }
      for (; s < se; ++s) o += acc[(size_t)s * D + d] * wgt[s];
      if (nruns == 1) out[((size_t)t * Hq + h) * D + d] = from_float<T>(o * s_inv);
      else runs[(size_t)r * D + d] = o;
    }
  }
  if (nruns == 1) return;
  __syncthreads();
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float o = 0.f;
    for (int r = 0; r < nruns; ++r) o += runs[(size_t)r * D + d];
    out[((size_t)t * Hq + h) * D + d] = from_float<T>(o * s_inv);
  }
}

template <int D>
static int launch_split(const void* qkv, int q_row_stride, const void* pages, const int* block_table,
                        int bt_width, const int* positions, const int* row_seg, float* ws_acc,
                        float* ws_ml, int T, int Hq, int Hkv, int page_size, int num_pages, int window,
                        float scale, int nsplit, int* counters, void* out, const int* row_list, cudaStream_t stream) {
  const int G = Hq / Hkv;
  const size_t smem = (size_t)2 * kSplit * (D + 8) * sizeof(__nv_bfloat16) +
                      ((size_t)G * kSplit + 4 * (G < 8 ? G : 8) * D + 2 * G) * sizeof(float);
  NF_REQUIRE(smem <= 200 * 1024, "decode attention: %d query heads per kv head need too much shared memory", G);
  static size_t allowed = 48 * 1024;
  if (smem > allowed) {
    cudaFuncSetAttribute(decode_attention_split_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    allowed = smem;
  }
  dim3 grid(T, Hkv, nsplit);
  launch_chained(decode_attention_split_kernel<D>, grid, dim3(128), smem, stream,
                 (const __nv_bfloat16*)qkv, q_row_stride, (const __nv_bfloat16*)pages, block_table, bt_width,
                 positions, row_seg, ws_acc, ws_ml, Hq, Hkv, page_size, num_pages, window, scale, nsplit, counters,
                 (__nv_bfloat16*)out, row_list);
  return check_launch("decode_attention_split");
}

}  // namespace nf

namespace nf {
// attention_decode_stream.cu: the persistent form of the split kernel (same partial results layout)
int decode_attention_stream_fits(int T, int Hq, int Hkv, int D, int page_size);
int decode_attention_stream(const void* qkv, int q_row_stride, const void* pages, const int* block_table,
                            int bt_width, const int* positions, const int* row_seg, float* ws_acc, float* ws_ml,
                            int T, int Hq, int Hkv, int D, int page_size, int num_pages, int window, float scale,
                            int nsplit, const int* row_list, cudaStream_t stream);
int decode_attention_stream_status();
int g_decode_stream = 1;
}  // namespace nf

using namespace nf;

extern "C" int nf_decode_attention_split_size() { return kSplit; }

// 0, or 1 + a row whose position needed more key blocks than `nsplit` gave (its result is then
// the attention over the first nsplit * 128 keys only).  Reads and clears; synchronises.
extern "C" int nf_decode_attention_status() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_decode_split_range_error, sizeof(int)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(g_decode_split_range_error, &zero, sizeof(int));
  const int w = decode_attention_stream_status();
  return v ? v : w;
}

// 0: one CTA per block of keys; 1 (default): the persistent streaming kernel where it fits.
extern "C" int nf_set_decode_stream(int on) {
  g_decode_stream = on ? 1 : 0;
  return 0;
}

// bfloat16 only; head_dim in {16, 32, 64, 128, 256}.  `nsplit` >= ceil(max context / 128) of
// the rows in this call.  Workspace: ws_acc float32 [T, Hq, nsplit, D], ws_ml [T, Hq, nsplit, 2].
static int decode_attention_impl(const void* qkv, int q_row_stride, const void* pages,
                                 const int* block_table, int bt_width, const int* positions,
                                 const int* row_seg, void* out, float* ws_acc, float* ws_ml, int T,
                                 int Hq, int Hkv, int D, int page_size, int num_pages, int window,
                                 float scale, int nsplit, int* counters, const int* row_list,
                                 cudaStream_t stream) {
  if (T == 0) return 0;
  NF_REQUIRE(T > 0 && Hq > 0 && Hkv > 0 && Hq % Hkv == 0 && nsplit > 0, "decode attention: bad sizes T=%d Hq=%d Hkv=%d nsplit=%d", T, Hq, Hkv, nsplit);
  NF_REQUIRE(Hkv <= 65535 && nsplit <= kMaxMergeSplits, "decode attention: too many kv heads or key blocks (context beyond %d keys)", kMaxMergeSplits * kSplit);
  int rc;
  // The persistent kernel pays a start-up (every CTA lists the rows' blocks) that only many
  // blocks repay: measured on B200, it wins from about a thousand blocks on.
  if (g_decode_stream && !counters && (long long)T * Hkv * nsplit >= 1024 &&
      decode_attention_stream_fits(T, Hq, Hkv, D, page_size)) {
    rc = decode_attention_stream(qkv, q_row_stride, pages, block_table, bt_width, positions, row_seg, ws_acc, ws_ml,
                                 T, Hq, Hkv, D, page_size, num_pages, window, scale, nsplit, row_list, stream);
  } else
  switch (D) {
    case 16: rc = launch_split<16>(qkv, q_row_stride, pages, block_table, bt_width, positions, row_seg, ws_acc, ws_ml, T, Hq, Hkv, page_size, num_pages, window, scale, nsplit, counters, out, row_list, stream); break;
    case 32: rc = launch_split<32>(qkv, q_row_stride, pages, block_table, bt_width, positions, row_seg, ws_acc, ws_ml, T, Hq, Hkv, page_size, num_pages, window, scale, nsplit, counters, out, row_list, stream); break;
    case 64: rc = launch_split<64>(qkv, q_row_stride, pages, block_table, bt_width, positions, row_seg, ws_acc, ws_ml, T, Hq, Hkv, page_size, num_pages, window, scale, nsplit, counters, out, row_list, stream); break;
    case 128: rc = launch_split<128>(qkv, q_row_stride, pages, block_table, bt_width, positions, row_seg, ws_acc, ws_ml, T, Hq, Hkv, page_size, num_pages, window, scale, nsplit, counters, out, row_list, stream); break;
    case 256: rc = launch_split<256>(qkv, q_row_stride, pages, block_table, bt_width, positions, row_seg, ws_acc, ws_ml, T, Hq, Hkv, page_size, num_pages, window, scale, nsplit, counters, out, row_list, stream); break;
    default:
      set_error("decode attention: head_dim %d is not one of 16, 32, 64, 128, 256", D);
      return 1;
  }
  if (rc || counters) return rc;      // with counters the split kernel's last CTAs have merged
  dim3 grid(T, Hq);
  int dthreads = 32;
  while (dthreads < D && dthreads < 256) dthreads <<= 1;
  const int max_runs = (nsplit + kMergeRun - 1) / kMergeRun;
  int groups = 1024 / dthreads < max_runs ? 1024 / dthreads : max_runs;
  const size_t smem = max_runs > 1 ? (size_t)max_runs * D * sizeof(float) : 0;
  static size_t allowed = 48 * 1024;
  if (smem > allowed) {
    cudaError_t e = cudaFuncSetAttribute(decode_attention_merge_kernel<__nv_bfloat16>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    NF_REQUIRE(e == cudaSuccess, "decode attention: the merge cannot have %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    allowed = smem;
  }
  launch_chained(decode_attention_merge_kernel<__nv_bfloat16>, grid, dim3(dthreads * groups), smem, stream,
                 (const float*)ws_acc, (const float*)ws_ml, positions, (__nv_bfloat16*)out, Hq, D, window, nsplit,
                 dthreads, row_list);
  return check_launch("decode_attention_merge");
}

extern "C" int nf_decode_attention(const void* qkv, int q_row_stride, const void* pages,
                                   const int* block_table, int bt_width, const int* positions,
                                   const int* row_seg, void* out, float* ws_acc, float* ws_ml, int T,
                                   int Hq, int Hkv, int D, int page_size, int num_pages, int window,
                                   float scale, int nsplit, cudaStream_t stream) {
  return decode_attention_impl(qkv, q_row_stride, pages, block_table, bt_width, positions, row_seg, out, ws_acc,
                               ws_ml, T, Hq, Hkv, D, page_size, num_pages, window, scale, nsplit, nullptr, nullptr,
                               stream);
}

// The same for some rows of a step: `row_list` (int32 [T] on the device) names the rows of qkv,
// positions, row_seg and out that this call serves; the workspace is indexed by the place in
// the list.  A step that mixes prompt portions and single decoded tokens sends the latter here.
extern "C" int nf_decode_attention_rows(const void* qkv, int q_row_stride, const void* pages,
                                        const int* block_table, int bt_width, const int* positions,
                                        const int* row_seg, void* out, float* ws_acc, float* ws_ml,
                                        const int* row_list, int T, int Hq, int Hkv, int D, int page_size,
                                        int num_pages, int window, float scale, int nsplit,
                                        cudaStream_t stream) {
  NF_REQUIRE(row_list, "decode attention: the form for some rows needs its row list");
  return decode_attention_impl(qkv, q_row_stride, pages, block_table, bt_width, positions, row_seg, out, ws_acc,
                               ws_ml, T, Hq, Hkv, D, page_size, num_pages, window, scale, nsplit, nullptr, row_list,
                               stream);
}

// The same in one launch: `counters` are T * Hkv ints that are zero before the call and are left
// zero after it; the CTA that finishes a (row, kv head) last merges its key blocks.
extern "C" int nf_decode_attention_fused(const void* qkv, int q_row_stride, const void* pages,
                                         const int* block_table, int bt_width, const int* positions,
                                         const int* row_seg, void* out, float* ws_acc, float* ws_ml,
                                         int* counters, int T, int Hq, int Hkv, int D, int page_size,
                                         int num_pages, int window, float scale, int nsplit,
                                         cudaStream_t stream) {
  NF_REQUIRE(counters, "decode attention: the one-launch form needs its counters");
  return decode_attention_impl(qkv, q_row_stride, pages, block_table, bt_width, positions, row_seg, out, ws_acc,
                               ws_ml, T, Hq, Hkv, D, page_size, num_pages, window, scale, nsplit, counters, nullptr,
                               stream);
}

// ---- the entry point that allocates nothing ---------------------------------------------------
//
// Some callers cannot call cudaMalloc (see ninfer_ops.h: plug-ins inside a host that owns the
// device's memory, loops that cannot afford an allocation's synchronisation, sandboxes that
// forbid allocations after start-up).  For them the split kernel's scratch lives in this
// fixed array.  In host code the name `g_decode_scratch` is only a stand-in for the symbol,
// not a device address: the address is asked for once per device with cudaGetSymbolAddress
// and then handed to the kernels like any other pointer.

namespace nf {
constexpr long long kStaticScratchBytes = 8ll << 20;     // 8 MiB on every GPU that loads the library
static __device__ __align__(256) unsigned char g_decode_scratch[kStaticScratchBytes];
constexpr int kMaxDevices = 64;
static void* g_scratch_addr[kMaxDevices] = {nullptr};
}  // namespace nf

extern "C" long long nf_decode_attention_static_scratch_bytes() { return nf::kStaticScratchBytes; }

// Decode attention with the library's own scratch.  Same arguments as nf_decode_attention
// without the two workspace pointers.  The first call on a device performs the address
// look-up (make it before any stream capture, with that device current).  Calls share the
// scratch: kernels of two calls must not overlap on the GPU.  Nothing is allocated.
extern "C" int nf_decode_attention_static(const void* qkv, int q_row_stride, const void* pages,
                                          const int* block_table, int bt_width, const int* positions,
                                          const int* row_seg, void* out, int T, int Hq, int Hkv, int D,
                                          int page_size, int num_pages, int window, float scale,
                                          int nsplit, cudaStream_t stream) {
  if (T == 0) return 0;
  NF_REQUIRE(T > 0 && Hq > 0 && nsplit > 0 && D > 0, "decode attention (static scratch): bad sizes T=%d Hq=%d nsplit=%d D=%d", T, Hq, nsplit, D);
  const long long acc_bytes = (long long)T * Hq * nsplit * D * (long long)sizeof(float);
  const long long ml_bytes = (long long)T * Hq * nsplit * 2 * (long long)sizeof(float);
  const long long acc_padded = (acc_bytes + 255) / 256 * 256;
  NF_REQUIRE(acc_padded + ml_bytes <= kStaticScratchBytes,
             "decode attention (static scratch): T=%d rows x %d heads x %d key blocks x head_dim %d needs %lld bytes "
             "of scratch, the fixed array holds %lld; use nf_decode_attention with your own workspace",
             T, Hq, nsplit, D, acc_padded + ml_bytes, kStaticScratchBytes);
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  NF_REQUIRE(e == cudaSuccess && dev >= 0 && dev < kMaxDevices, "decode attention (static scratch): cannot tell the current device (%s)", cudaGetErrorString(e));
  if (!g_scratch_addr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_decode_scratch);
    NF_REQUIRE(e == cudaSuccess && p, "decode attention (static scratch): cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
    g_scratch_addr[dev] = p;
  }
  unsigned char* base = static_cast<unsigned char*>(g_scratch_addr[dev]);
  return nf_decode_attention(qkv, q_row_stride, pages, block_table, bt_width, positions, row_seg, out,
                             reinterpret_cast<float*>(base), reinterpret_cast<float*>(base + acc_padded), T, Hq,
                             Hkv, D, page_size, num_pages, window, scale, nsplit, stream);
}
