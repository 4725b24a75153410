// Y = X W^T for few rows of X: the weight-streaming kernel of skinny_gemm.cu with its weights
// staged through shared memory by asynchronous copies.
//
// Reference counterparts: as for skinny_gemm.cu (``gemv_kernel_vec8`` src/ops/gemv.hip:52-93,
// ``gemv_fused_kernel<SWIGLU>`` gemv.hip:103-166, the per-expert loop src/models/model.hip:355-427).
//
// Why a second form.  skinny_gemm.cu keeps the weights it has asked for in registers, so what a
// lane has in flight is bounded by its registers (4 chunks of 2 x 16 bytes) and its loop runs in
// rounds: ask for four chunks, wait for all, multiply.  Here every lane owns a private ring of
// `kDepth` slots in shared memory and fills it with ``cp.async`` (16 bytes, L1 bypassed): eight
// chunks are in flight from the first instruction on without holding a register, each is
// multiplied as soon as it has landed, and its slot is asked to be refilled at once.  A lane
// copies exactly the 16-byte pieces that it multiplies itself (the fragment trick of
// skinny_gemm.cu needs no exchange between lanes), so the only synchronisation is the lane's own
// ``cp.async.wait_group``: no barrier, no mbarrier, nothing that could wait on another thread.
//
// The arithmetic is that of skinny_gemm.cu bit for bit: the same split of k over the 8 warps
// (interleaved 32-wide chunks), the same order of products within a warp and of the warps'
// partial sums.
#include "common.cuh"

namespace nf {

namespace {

constexpr int kWarps = 8;
constexpr int kDepth = 8;        // chunks in flight per lane (ring slots)
constexpr int kAhead = 4;        // chunks of X held in registers ahead of use

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ uint4 ld_cached(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ void mma_bf16(float* c, unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// N: output columns (SWIGLU: the inner width; W has 2N rows, gate rows first).  PACKED: W in
// the tile layout of `pack_weights` (see skinny_gemm.cu).  early_index != 0: offsets, x_rows and
// group_map were complete before the kernel that precedes this launch in the stream began (the
// router, when this is the experts' second product), so they may be read - and the weights asked
// for - before the dependency wait.  A dense product (no index arrays) always starts early.
template <int NT, bool SWIGLU, bool PACKED, typename TC>
__global__ void __launch_bounds__(kWarps * 32)
skinny_staged_kernel(const __nv_bfloat16* __restrict__ X, int ldx, const __nv_bfloat16* __restrict__ W,
                     size_t w_group_stride, TC* __restrict__ Y, int ldy, int M, int N, int K,
                     const int* __restrict__ offsets, const int* __restrict__ x_rows, int x_div,
                     const int* __restrict__ group_map, int early_index) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint4* ring = reinterpret_cast<uint4*>(smem_raw);                       // [kDepth][2][256]
  float* partial = reinterpret_cast<float*>(ring + kDepth * 2 * kWarps * 32);   // [kWarps][NT * 4 * 32]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const bool early = early_index || (!offsets && !x_rows && !group_map);
  if (!early) chain_wait();
  // row tiles vary fastest, so CTAs that share weight rows run together; with a group map,
  // blockIdx.z counts only the groups that have rows (a decode step uses few of the experts)
  const int group = group_map ? group_map[blockIdx.z] : blockIdx.z;
  if (group < 0) {
    if (early) chain_wait();
    return;
  }
  constexpr int FEAT = SWIGLU ? 8 : 16;
  const int n0 = blockIdx.y * FEAT;
  const __nv_bfloat16* Wg = W + (size_t)group * w_group_stride;

  // weight rows of this lane: tile row g and tile row g + 8
  int wr0, wr1;
  if (SWIGLU) {
    const int f = min(n0 + g, N - 1);
    wr0 = f;            // gate
    wr1 = N + f;        // up
  } else {
    wr0 = min(n0 + g, N - 1);
    wr1 = min(n0 + g + 8, N - 1);
  }
  const __nv_bfloat16* w0 = Wg + (size_t)wr0 * K + 8 * t;
  const __nv_bfloat16* w1 = Wg + (size_t)wr1 * K + 8 * t;
  constexpr int TROWS = SWIGLU ? 256 : 128;
  const int ktiles = (K + 63) >> 6;
  int pr0 = 0, pr1 = 0;
  size_t ptile = 0;
  if (PACKED) {
    const int f = n0 + g;                      // < padded N by construction of the grid
    ptile = (size_t)(f >> 7) * ktiles * (TROWS * 64);
    if (SWIGLU) { pr0 = f & 127; pr1 = 128 + (f & 127); }
    else { pr0 = f & 127; pr1 = (f + 8) & 127; }   // f + 8 stays inside the tile: n0 is a multiple of 16
  }
  const int nchunks = (K + 31) >> 5;
  const int mine = warp < nchunks ? (nchunks - warp + kWarps - 1) / kWarps : 0;   // chunks of this warp
  uint4* slot_a = ring + threadIdx.x;                       // slot s: slot_a[s * 512], slot_b = + 256
  // ask for this lane's pieces of its warp's chunk number i (chunk warp + 8 i) into slot i % kDepth;
  // always commits a group, so that group i is chunk i
  auto fetch = [&](int i) {
    if (i < mine) {
      const int k = (warp + i * kWarps) * 32;
      uint4* sa = slot_a + (i % kDepth) * (2 * kWarps * 32);
      if (PACKED) {
        const int kk = k + 8 * t;                   // < padded K: the padding holds zeros
        const __nv_bfloat16* tile = Wg + ptile + (size_t)(kk >> 6) * (TROWS * 64);
        const int j = (kk >> 3) & 7;
        cp_async16(sa, tile + pr0 * 64 + ((j ^ (pr0 & 7)) << 3));
        cp_async16(sa + kWarps * 32, tile + pr1 * 64 + ((j ^ (pr1 & 7)) << 3));
      } else if (k + 8 * t + 8 <= K) {
        cp_async16(sa, w0 + k);
        cp_async16(sa + kWarps * 32, w1 + k);
      } else {
        *sa = make_uint4(0, 0, 0, 0);
        sa[kWarps * 32] = make_uint4(0, 0, 0, 0);
      }
    }
    cp_commit();
  };
#pragma unroll
  for (int i = 0; i < kDepth; ++i) fetch(i);
  if (early) chain_wait();

  int row_begin = 0, row_end = M;
  if (offsets) { row_begin = offsets[group]; row_end = offsets[group + 1]; }
  const int m0 = row_begin + blockIdx.x * (8 * NT);
  if (m0 >= row_end) {                 // no rows for this CTA: let the copies land, then leave
    cp_wait<0>();
    return;
  }
  const int rows = min(8 * NT, row_end - m0);
  const int ntiles = (rows + 7) >> 3;

  // X rows of this lane: row g of every 8-row tile
  const __nv_bfloat16* xp[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int r = m0 + nt * 8 + g;
    long src = -1;
    if (r < row_end) src = x_rows ? (long)(x_rows[r] / x_div) : (long)r;
    xp[nt] = src >= 0 ? X + src * (long)ldx + 8 * t : nullptr;
  }
  auto load_x = [&](int i, uint4* xv) {
    const int k = (warp + i * kWarps) * 32;
    const bool in = i < mine && k + 8 * t + 8 <= K;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      xv[nt] = make_uint4(0, 0, 0, 0);
      if (in && nt < ntiles && xp[nt]) xv[nt] = ld_cached(xp[nt] + k);
    }
  };

  float acc[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[nt][i] = 0.f;

  uint4 xv[kAhead][NT];
#pragma unroll
  for (int u = 0; u < kAhead; ++u) load_x(u, xv[u]);
  for (int i0 = 0; i0 < mine; i0 += kAhead) {
#pragma unroll
    for (int u = 0; u < kAhead; ++u) {
      const int i = i0 + u;
      // group i is complete once at most kDepth - 1 younger groups are pending (one group is
      // committed per chunk, in order, also past the end)
      cp_wait<kDepth - 1>();
      if (i < mine) {
        const uint4* sa = slot_a + (i % kDepth) * (2 * kWarps * 32);
        const uint4 a = *sa, b = sa[kWarps * 32];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          if (nt < ntiles) {
            mma_bf16(acc[nt], a.x, b.x, a.y, b.y, xv[u][nt].x, xv[u][nt].y);
            mma_bf16(acc[nt], a.z, b.z, a.w, b.w, xv[u][nt].z, xv[u][nt].w);
          }
        }
      }
      fetch(i + kDepth);               // refill the slot just read (or commit an empty group)
      load_x(i + kAhead, xv[u]);
    }
  }
  cp_wait<0>();
  chain_release_late();

  // add the warps' partial sums in warp order
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) partial[warp * (NT * 4 * 32) + (nt * 4 + i) * 32 + lane] = acc[nt][i];
  __syncthreads();
  for (int e = threadIdx.x; e < ntiles * 2 * 32; e += blockDim.x) {
    // e -> (tile nt, column half h of the fragment, lane l); this thread owns fragment
    // entries (c[h], c[h + 2]) = (row g, row g + 8) of token column 2 t + h
    const int l = e & 31, h = (e >> 5) & 1, nt = e >> 6;
    float lo = 0.f, hi = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      lo += partial[w * (NT * 4 * 32) + (nt * 4 + h) * 32 + l];
      hi += partial[w * (NT * 4 * 32) + (nt * 4 + h + 2) * 32 + l];
    }
    const int gg = l >> 2, tt = l & 3;
    const int row = m0 + nt * 8 + 2 * tt + h;          // token (sorted position) of this column
    if (row >= row_end) continue;
    if (SWIGLU) {
      const int f = n0 + gg;
      if (f < N) Y[(size_t)row * ldy + f] = from_float<TC>(lo / (1.f + expf(-lo)) * hi);
    } else {
      const int f0 = n0 + gg, f1 = n0 + gg + 8;
      if (f0 < N) Y[(size_t)row * ldy + f0] = from_float<TC>(lo);
      if (f1 < N) Y[(size_t)row * ldy + f1] = from_float<TC>(hi);
    }
  }
}

template <int NT, bool SWIGLU, bool PACKED, typename TC>
int launch_staged(const void* X, int ldx, const void* W, size_t wgs, void* Y, int ldy, int M, int N, int K,
                  int groups, int max_rows, const int* offsets, const int* x_rows, int x_div,
                  const int* group_map, int n_mapped, int early_index, cudaStream_t stream) {
  const int feat = SWIGLU ? 8 : 16;
  const size_t smem = (size_t)kDepth * 2 * kWarps * 32 * sizeof(uint4) + (size_t)kWarps * NT * 4 * 32 * sizeof(float);
  static bool set = false;
  if (!set) {
    cudaError_t e = cudaFuncSetAttribute(skinny_staged_kernel<NT, SWIGLU, PACKED, TC>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    NF_REQUIRE(e == cudaSuccess, "skinny_staged: cannot have %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    set = true;
  }
  dim3 grid((max_rows + 8 * NT - 1) / (8 * NT), (N + feat - 1) / feat, group_map ? n_mapped : groups);
  NF_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "skinny_staged: too many feature tiles or groups");
  launch_chained(skinny_staged_kernel<NT, SWIGLU, PACKED, TC>, grid, dim3(kWarps * 32), smem, stream,
                 (const __nv_bfloat16*)X, ldx, (const __nv_bfloat16*)W, wgs, (TC*)Y, ldy, M, N, K,
                 offsets, x_rows, x_div, group_map, early_index);
  return check_launch("skinny_staged");
}

template <bool SWIGLU, typename TC>
int launch_pick(int nt, bool packed, const void* X, int ldx, const void* W, size_t wgs, void* Y, int ldy, int M,
                int N, int K, int groups, int max_rows, const int* offsets, const int* x_rows, int x_div,
                const int* group_map, int n_mapped, int early_index, cudaStream_t stream) {
  if (packed) {
    if (nt == 1) return launch_staged<1, SWIGLU, true, TC>(X, ldx, W, wgs, Y, ldy, M, N, K, groups, max_rows, offsets, x_rows, x_div, group_map, n_mapped, early_index, stream);
    return launch_staged<2, SWIGLU, true, TC>(X, ldx, W, wgs, Y, ldy, M, N, K, groups, max_rows, offsets, x_rows, x_div, group_map, n_mapped, early_index, stream);
  }
  if (nt == 1) return launch_staged<1, SWIGLU, false, TC>(X, ldx, W, wgs, Y, ldy, M, N, K, groups, max_rows, offsets, x_rows, x_div, group_map, n_mapped, early_index, stream);
  return launch_staged<2, SWIGLU, false, TC>(X, ldx, W, wgs, Y, ldy, M, N, K, groups, max_rows, offsets, x_rows, x_div, group_map, n_mapped, early_index, stream);
}

}  // namespace
}  // namespace nf

using namespace nf;

// The arguments of nf_skinny_gemm, plus `early_index`: non-zero if offsets, x_rows and group_map
// were complete before the kernel that precedes this launch in the stream began (then the
// weights are asked for without waiting for that kernel).
extern "C" int nf_skinny_staged(const void* X, int ldx, const void* W, long long w_group_stride, void* Y,
                                int ldy, int M, int N, int K, int groups, int max_rows,
                                const int* offsets, const int* x_rows, int x_div, int swiglu,
                                int out_dtype, int packed, const int* group_map, int n_mapped,
                                int early_index, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  NF_REQUIRE(M > 0 && N > 0 && K > 0 && groups > 0 && x_div > 0, "skinny_staged: bad sizes M=%d N=%d K=%d", M, N, K);
  NF_REQUIRE(K % 8 == 0 && ldx % 8 == 0, "skinny_staged: K=%d and the row stride %d must be multiples of 8", K, ldx);
  NF_REQUIRE(((uintptr_t)X % 16 == 0) && ((uintptr_t)W % 16 == 0) && (w_group_stride % 8 == 0),
             "skinny_staged: operands must be 16-byte aligned");
  NF_REQUIRE(groups == 1 || offsets, "skinny_staged: grouped product needs row offsets");
  const int nt = max_rows <= 8 ? 1 : 2;
  const size_t wgs = (size_t)w_group_stride;
  if (swiglu) {
    NF_REQUIRE(out_dtype == kBF16, "skinny_staged: the SwiGLU epilogue writes bfloat16");
    return launch_pick<true, __nv_bfloat16>(nt, packed != 0, X, ldx, W, wgs, Y, ldy, M, N, K, groups, max_rows, offsets, x_rows, x_div, group_map, n_mapped, early_index, stream);
  }
  if (out_dtype == kBF16)
    return launch_pick<false, __nv_bfloat16>(nt, packed != 0, X, ldx, W, wgs, Y, ldy, M, N, K, groups, max_rows, offsets, x_rows, x_div, group_map, n_mapped, early_index, stream);
  return launch_pick<false, float>(nt, packed != 0, X, ldx, W, wgs, Y, ldy, M, N, K, groups, max_rows, offsets, x_rows, x_div, group_map, n_mapped, early_index, stream);
}
