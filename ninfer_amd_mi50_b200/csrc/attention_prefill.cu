// Prefill attention in bfloat16: a flash-style kernel over the paged cache for any mix of
// segments (portions of prompts beside single rows).
//
// Reference: ``prefill_attention_kernel<D>`` (src/ops/attention.hip:136-268): tiles of 16
// queries x 32 keys, a software double buffer, causal mask on absolute positions so that a
// later portion sees the keys of earlier ones, online softmax, never a T x T score matrix.
// Same structure here with tensor cores: a tile is up to 64 consecutive rows of one segment
// and one query head, 16 rows per warp; a CTA runs two tiles one after the other, a heavy one
// (late in a long prompt, many keys) and a light one, so that CTAs are about equally long; keys and values come in blocks
// of 64 through ``cp.async`` into a two-stage shared-memory ring (rows padded by 16 bytes so
// that ``ldmatrix`` is free of bank conflicts); S = Q K^T and O += P V are
// ``mma.sync.m16n8k16`` with float32 accumulators; max, exp and sums are float32 (the
// exponential is ``ex2.approx`` on scores pre-multiplied by log2 e: 2^-22 relative, far below
// the bfloat16 rounding of P that follows).
// Key j is visible to a row at position p iff max(0, p - window + 1) <= j <= p.
// Key blocks are aligned to multiples of 64 keys, so the order of a row's sums depends on
// its own position only, not on how the prompt was cut.
#include "common.cuh"

namespace nf {

constexpr int kBQ = 64, kBKeys = 64;      // rows per tile (4 warps x 16), keys per block
constexpr int kThreads = 128;
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ void pf_cp_async16(void* smem_dst, const void* gmem_src) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gmem_src));
}
__device__ __forceinline__ void pf_commit() { asm volatile("cp.async.commit_group;"); }
template <int N> __device__ __forceinline__ void pf_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }
__device__ __forceinline__ void pf_ldm4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void pf_ldm4t(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void pf_mma(float* c, unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pf_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

template <int D>
__global__ void __launch_bounds__(kThreads)
prefill_attention_kernel(const __nv_bfloat16* __restrict__ qkv, int q_row_stride,
                         const __nv_bfloat16* __restrict__ pages, const int* __restrict__ block_table,
                         int bt_width, const int* __restrict__ positions, const int* __restrict__ seg_row0,
                         const int* __restrict__ tiles, __nv_bfloat16* __restrict__ out, int Hq, int Hkv,
                         int page_size, int num_pages, int window, float scale) {
  constexpr int DS = D + 8;             // padded row stride in elements
  constexpr int LPR = D / 8;            // 16-byte pieces per row
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);        // [64][DS]
  __nv_bfloat16* KVs = Qs + kBQ * DS;                                     // [2 stages][K, V][64][DS]
  const int h = blockIdx.y;
  for (int which = 0; which < 2; ++which) {
  const int seg = tiles[4 * blockIdx.x + 2 * which], row0 = tiles[4 * blockIdx.x + 2 * which + 1];
  if (seg < 0) break;
  const int kvh = h / (Hq / Hkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tq = lane & 3;
  const int n_rows = min(kBQ, seg_row0[seg + 1] - row0);
  const int pos_first = positions[row0];
  const int pos_last = pos_first + n_rows - 1;
  const int* bt = block_table + (size_t)seg * bt_width;
  const size_t head_stride = (size_t)page_size * D;
  const size_t page_stride = (size_t)2 * Hkv * head_stride;
  int lo_tile = 0;
  if (window > 0 && pos_first - window + 1 > 0) lo_tile = pos_first - window + 1;
  const int kb_first = (lo_tile / kBKeys) * kBKeys;
  const int n_blocks = (pos_last - kb_first) / kBKeys + 1;

  // ---- Q tile ------------------------------------------------------------------------------
  for (int c = threadIdx.x; c < kBQ * LPR; c += blockDim.x) {
    const int r = c / LPR, piece = c - r * LPR;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < n_rows)
      v = *reinterpret_cast<const uint4*>(qkv + (size_t)(row0 + r) * q_row_stride + (size_t)h * D + piece * 8);
    *reinterpret_cast<uint4*>(Qs + r * DS + piece * 8) = v;
  }

  auto load_block = [&](int blk, int stage) {
    __nv_bfloat16* Ks = KVs + (size_t)stage * 2 * kBKeys * DS;
    __nv_bfloat16* Vs = Ks + kBKeys * DS;
    const int kb = kb_first + blk * kBKeys;
    for (int c = threadIdx.x; c < kBKeys * LPR; c += blockDim.x) {
      const int r = c / LPR, piece = c - r * LPR;
      const int j = kb + r;
      const __nv_bfloat16* src = nullptr;
      if (j <= pos_last) {
        const int lp = j / page_size;
        const int page = lp < bt_width ? bt[lp] : -1;
        if (page >= 0 && page < num_pages)
          src = pages + (size_t)page * page_stride + (size_t)kvh * head_stride + (size_t)(j - lp * page_size) * D + piece * 8;
      }
      if (src) {
        pf_cp_async16(Ks + r * DS + piece * 8, src);
        pf_cp_async16(Vs + r * DS + piece * 8, src + (size_t)Hkv * head_stride);
      } else {
        *reinterpret_cast<uint4*>(Ks + r * DS + piece * 8) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(Vs + r * DS + piece * 8) = make_uint4(0, 0, 0, 0);
      }
    }
  };

  float o[D / 8][4];
#pragma unroll
  for (int n = 0; n < D / 8; ++n)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[n][i] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  // this thread's two query rows and their positions
  const int r_lo = warp * 16 + g, r_hi = r_lo + 8;
  const int p_lo = pos_first + r_lo, p_hi = pos_first + r_hi;
  const int w_lo = window > 0 ? p_lo - window + 1 : 0, w_hi = window > 0 ? p_hi - window + 1 : 0;

  load_block(0, 0);
  pf_commit();
  for (int blk = 0; blk < n_blocks; ++blk) {
    if (blk + 1 < n_blocks) load_block(blk + 1, (blk + 1) & 1);
    pf_commit();
    pf_wait<1>();
    __syncthreads();
    const __nv_bfloat16* Ks = KVs + (size_t)(blk & 1) * 2 * kBKeys * DS;
    const __nv_bfloat16* Vs = Ks + kBKeys * DS;
    const int kb = kb_first + blk * kBKeys;

    // a warp whose 16 rows lie beyond the tile's rows, or wholly before this block's keys,
    // only helps with the copies
    const bool warp_active = warp * 16 < n_rows && kb <= pos_first + warp * 16 + 15;
    if (warp_active) {
    // ---- S = Q K^T for this warp's 16 rows x 64 keys -------------------------------------------
    float s[kBKeys / 8][4];
#pragma unroll
    for (int n = 0; n < kBKeys / 8; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) s[n][i] = 0.f;
#pragma unroll
    for (int k0 = 0; k0 < D; k0 += 16) {
      unsigned a0, a1, a2, a3;
      pf_ldm4(a0, a1, a2, a3, Qs + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * DS + k0 + (lane >> 4) * 8);
#pragma unroll
      for (int n0 = 0; n0 < kBKeys; n0 += 16) {
        unsigned b0, b1, b2, b3;
        const int mi = lane >> 3;
        pf_ldm4(b0, b1, b2, b3, Ks + (n0 + (lane & 7) + (mi >> 1) * 8) * DS + k0 + (mi & 1) * 8);
        pf_mma(s[n0 / 8], a0, a1, a2, a3, b0, b1);
        pf_mma(s[n0 / 8 + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    // ---- scale (to base-2 exponent units), mask, online softmax ------------------------------------
    float mx[2] = {-INFINITY, -INFINITY};
    const float sc2 = scale * kLog2e;
    // every key of the block visible to every row of the warp: no mask to apply
    const bool all_visible = warp * 16 + 15 < n_rows && kb + kBKeys - 1 <= pos_first + warp * 16 &&
                             (window <= 0 || kb >= pos_first + warp * 16 + 15 - window + 1);
    if (all_visible) {
#pragma unroll
      for (int n = 0; n < kBKeys / 8; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          s[n][i] *= sc2;
          mx[i >> 1] = fmaxf(mx[i >> 1], s[n][i]);
        }
    } else {
#pragma unroll
      for (int n = 0; n < kBKeys / 8; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int j = kb + n * 8 + 2 * tq + (i & 1);
          const bool hi_row = i >= 2;
          const int p = hi_row ? p_hi : p_lo;
          const int w = hi_row ? w_hi : w_lo;
          const bool row_ok = (hi_row ? r_hi : r_lo) < n_rows;
          const float v = (row_ok && j <= p && j >= w) ? s[n][i] * sc2 : -INFINITY;
          s[n][i] = v;
          mx[i >> 1] = fmaxf(mx[i >> 1], v);
        }
    }
    float alpha[2], m_use[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float m_new = fmaxf(m_run[r], mx[r]);
      m_use[r] = m_new == -INFINITY ? 0.f : m_new;       // a row with nothing visible yet
      alpha[r] = exp2f(m_run[r] - m_use[r]);
      m_run[r] = m_new;
    }
    float sum[2] = {0.f, 0.f};
#pragma unroll
    for (int n = 0; n < kBKeys / 8; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float p = exp2f(s[n][i] - m_use[i >> 1]);
        s[n][i] = p;
        sum[i >> 1] += p;
      }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 1);
      sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 2);
      l_run[r] = l_run[r] * alpha[r] + sum[r];
    }
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
      o[n][0] *= alpha[0]; o[n][1] *= alpha[0];
      o[n][2] *= alpha[1]; o[n][3] *= alpha[1];
    }
    // ---- O += P V ----------------------------------------------------------------------------------
#pragma unroll
    for (int kk = 0; kk < kBKeys / 16; ++kk) {
      const unsigned a0 = pf_pack(s[2 * kk][0], s[2 * kk][1]);
      const unsigned a1 = pf_pack(s[2 * kk][2], s[2 * kk][3]);
      const unsigned a2 = pf_pack(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      const unsigned a3 = pf_pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int d0 = 0; d0 < D; d0 += 16) {
        unsigned b0, b1, b2, b3;
        const int mi = lane >> 3;
        pf_ldm4t(b0, b1, b2, b3, Vs + (kk * 16 + (lane & 7) + (mi & 1) * 8) * DS + d0 + (mi >> 1) * 8);
        pf_mma(o[d0 / 8], a0, a1, a2, a3, b0, b1);
        pf_mma(o[d0 / 8 + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    }  // warp_active
    __syncthreads();      // everyone is done with this stage before the next prefetch overwrites it
  }

  // ---- write O / l -----------------------------------------------------------------------------------
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = r ? r_hi : r_lo;
    if (row >= n_rows) continue;
    const float inv = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
    __nv_bfloat16* dst = out + (size_t)(row0 + row) * Hq * D + (size_t)h * D;
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
      const unsigned v = pf_pack(o[n][2 * r] * inv, o[n][2 * r + 1] * inv);
      *reinterpret_cast<unsigned*>(dst + n * 8 + 2 * tq) = v;
    }
  }
  __syncthreads();      // the next tile reuses the shared memory
  }  // which
}

template <int D>
static int launch_prefill(const void* qkv, int q_row_stride, const void* pages, const int* block_table,
                          int bt_width, const int* positions, const int* seg_row0, const int* tiles,
                          int n_tiles, void* out, int Hq, int Hkv, int page_size, int num_pages, int window,
                          float scale, cudaStream_t stream) {
  const size_t smem = (size_t)(kBQ + 4 * kBKeys) * (D + 8) * sizeof(__nv_bfloat16);
  static bool set = false;
  if (smem > 48 * 1024 && !set) {
    cudaFuncSetAttribute(prefill_attention_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    set = true;
  }
  dim3 grid(n_tiles, Hq);
  prefill_attention_kernel<D><<<grid, kThreads, smem, stream>>>(
      (const __nv_bfloat16*)qkv, q_row_stride, (const __nv_bfloat16*)pages, block_table, bt_width, positions,
      seg_row0, tiles, (__nv_bfloat16*)out, Hq, Hkv, page_size, num_pages, window, scale);
  return check_launch("prefill_attention");
}

}  // namespace nf

using namespace nf;

extern "C" int nf_prefill_attention_tile_rows() { return kBQ; }

// bfloat16; head_dim a multiple of 16 up to 128.  `tiles` is int32 [n_ctas, 2, 2]: for every CTA two
// tiles as (segment, first row), each at most 64 consecutive rows of one segment; the second may
// be (-1, -1).
extern "C" int nf_prefill_attention(const void* qkv, int q_row_stride, const void* pages,
                                    const int* block_table, int bt_width, const int* positions,
                                    const int* seg_row0, const int* tiles, int n_tiles, void* out, int Hq,
                                    int Hkv, int D, int page_size, int num_pages, int window, float scale,
                                    cudaStream_t stream) {
  if (n_tiles == 0) return 0;
  NF_REQUIRE(n_tiles > 0 && Hq > 0 && Hkv > 0 && Hq % Hkv == 0 && Hq <= 65535, "prefill attention: bad sizes tiles=%d Hq=%d Hkv=%d", n_tiles, Hq, Hkv);
  NF_REQUIRE(q_row_stride % 8 == 0 && (uintptr_t)qkv % 16 == 0, "prefill attention: query rows must be 16-byte aligned");
#define NF_PF(DD) case DD: return launch_prefill<DD>(qkv, q_row_stride, pages, block_table, bt_width, positions, seg_row0, tiles, n_tiles, out, Hq, Hkv, page_size, num_pages, window, scale, stream);
  switch (D) {
    NF_PF(16) NF_PF(32) NF_PF(48) NF_PF(64) NF_PF(80) NF_PF(96) NF_PF(112) NF_PF(128)
    default:
      set_error("prefill attention: head_dim %d is not a multiple of 16 up to 128", D);
      return 1;
  }
#undef NF_PF
}
