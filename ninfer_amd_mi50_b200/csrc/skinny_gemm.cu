// Y = X W^T for few rows of X (decode batches): a weight-streaming kernel whose time is the
// time to read W once.
//
// Reference counterparts: ``gemv_kernel_vec8`` (one block per output row, 16-byte loads,
// float32 accumulation, src/ops/gemv.hip:52-93), ``gemv_fused_kernel<SWIGLU>`` (gate and up
// rows with the activation in the epilogue, gemv.hip:103-166) and the per-expert GEMV loop of
// the MoE branch (src/models/model.hip:355-427).  Those serve one row; a batch of decode
// tokens would read the weights once per row.  Here the weights are the M operand of
// ``mma.sync.m16n8k16`` (16 output features a tile) and up to 64 rows of X are the N operand,
// so every weight is read once for the whole batch, and one launch serves all experts.
//
// Fragment trick: a lane loads 16 contiguous bytes (8 bf16) of a weight row and 16 bytes of
// an X row at the same k offset and feeds them to two MMAs as if they were the scattered
// k columns the instruction expects.  A dot product does not care in which order k is
// summed as long as both operands agree, so no shuffle or shared-memory staging is needed.
//
// Work split: a CTA owns 16 features (8 gate + 8 up with the SwiGLU epilogue) of one
// group; its 8 warps take interleaved 32-wide chunks of k and their partial sums are added
// in warp order in shared memory.  The order of summation depends on K only, so a row's
// result does not depend on the batch it is in.
//
// A product with few features and a long k (the shared expert's down projection: 2048 features
// make 128 CTAs, each with 180 KB of weights to stream and nothing else on its SM) is launched
// as clusters of 2 or 4 CTAs that share a feature tile and split k between them; the members'
// sums meet in the first member's shared memory (distributed shared memory, the hardware
// cluster barrier) and are added there in member order.  How many members is decided by the
// product's shape alone.
#define NF_CHAIN_CLASS 1
#include "common.cuh"

namespace nf {

constexpr int kWarps = 8;
constexpr int kUnroll = 4;      // chunks of k in flight per warp (8 costs registers and occupancy: measured slower)
constexpr int kMaxSplit = 4;    // most cluster members that split k between them

__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
// Rows of X: written by the kernel before this one, which may still be running when this kernel's
// CTAs arrive (chained launch).  So never the non-coherent path (its contract is "read-only for the
// kernel's lifetime", and this kernel's lifetime begins before X is complete): a load that is
// served from L2, issued after the wait.
__device__ __forceinline__ uint4 ld_cached(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void mma_bf16(float* c, unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// What the rotate-and-append epilogue needs (see rope_append.cu for the separate kernel): the
// product is the q/k/v projection of attention, rows of W laid out [q heads | k heads | v heads]
// x D.  A CTA then owns 8 dims of the low half of one head and the 8 matching dims of the high
// half, so each accumulator pair (row g, row g + 8) is one rotation pair: bias, rotation by
// pos * inv_freq (float32), and the result goes to Y (queries) or straight into the cache page
// of (request, position) (keys, values) - the projection's output never makes a round trip.
// set to a code if a grouped product met a group, a row range or a row index outside its operands
// (1 group, 2 row range, 3 row index); read and reset by nf_skinny_index_status
__device__ int g_skinny_index_error = 0;

struct RopeEpilogue {
  const float* bias;          // [(Hq + 2 Hkv) D] or null
  const int* positions;       // [M]
  const int* row_seg;         // [M] block-table row of each row of X
  const float* inv_freq;      // [D / 2]
  __nv_bfloat16* pages;       // [num_pages, 2, Hkv, page_size, D]
  const int* block_table;     // [segments, bt_width]
  int Hq, Hkv, D, bt_width, page_size, num_pages, append;
};

// NT: number of 8-row tiles of X a CTA covers (rows <= 8 * NT).
// PACKED: W is held as tiles of 128 (SwiGLU: 128 gate + 128 up) rows x 64 k, contiguous per
// (feature tile, k tile) and 128-byte swizzled (16-byte piece j of row r sits at j ^ (r & 7)),
// zero-padded: the layout the tensor-core kernel streams.  A CTA's 16 rows of one k tile are
// then 2 KB of contiguous memory instead of 16 pieces 2 K bytes apart.
// ROPE: the rotate-and-append epilogue (dense, unpacked, bfloat16 out); blockIdx.y then counts
// (head, 8-dim group of the low half) instead of 16-feature tiles.
template <int NT, bool SWIGLU, bool PACKED, typename TC, bool ROPE = false>
__global__ void __launch_bounds__(kWarps * 32, NT == 1 ? 4 : 3)
skinny_gemm_kernel(const __nv_bfloat16* __restrict__ X, int ldx, const __nv_bfloat16* __restrict__ W,
                   size_t w_group_stride, TC* __restrict__ Y, int ldy, int M, int N, int K,
                   const int* __restrict__ offsets, const int* __restrict__ x_rows, int x_div,
                   const int* __restrict__ group_map, int early_index, int n_groups, RopeEpilogue rope, int ksplit) {
  // N: output columns (SWIGLU: the inner width; W has 2N rows, gate rows first)
  // ksplit > 1: blockIdx.x counts (row tile, cluster member); member s takes the s-th part of k
  __shared__ float partial[kWarps][NT * 4 * 32];
  __shared__ float others[kMaxSplit - 1][NT * 2 * 32 * 2];     // members 1.. leave their sums here, in member 0
  const int member = ksplit > 1 ? (int)(blockIdx.x % (unsigned)ksplit) : 0;
  const int row_tile = ksplit > 1 ? (int)(blockIdx.x / (unsigned)ksplit) : (int)blockIdx.x;
  // every member announces itself; a member waits for the others right before its first remote store
  if (ksplit > 1) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  chain_release();
  // A dense product needs nothing from the kernel before it until it reads X: its first round
  // of weights is asked for before the wait.  A grouped one reads offsets and row maps at once,
  // unless the caller vouches (early_index) that those were complete before the kernel that
  // precedes this launch began - the router's plan, when this is the experts' second product.
  const bool dense = (!offsets && !x_rows && !group_map) || early_index;
  bool waited = !dense;
  if (!dense) chain_wait(X, offsets, x_rows, group_map);
  // row tiles vary fastest, so CTAs that share weight rows run together; with a group map,
  // blockIdx.z counts only the groups that have rows (a decode step uses few of the experts)
  // (grouped products are never split over k: the early returns below leave no cluster waiting)
  const int group = group_map ? group_map[blockIdx.z] : blockIdx.z;
  if (group < 0 || group >= n_groups) {
    if (group >= n_groups) atomicCAS(&g_skinny_index_error, 0, 1);
    if (!waited) chain_wait();
    return;
  }
  int row_begin = 0, row_end = M;
  if (offsets) { row_begin = offsets[group]; row_end = offsets[group + 1]; }
  if (row_begin < 0 || row_end > M) {          // not offsets of this step's rows: do nothing, and say so
    atomicCAS(&g_skinny_index_error, 0, 2);
    if (!waited) chain_wait();
    return;
  }
  const int m0 = row_begin + row_tile * (8 * NT);
  if (m0 >= row_end && ksplit <= 1) {
    if (!waited) chain_wait();
    return;
  }
  const int rows = min(8 * NT, row_end - m0);
  const int ntiles = (rows + 7) >> 3;
  constexpr int FEAT = SWIGLU ? 8 : 16;
  const int n0 = blockIdx.y * FEAT;
  const __nv_bfloat16* Wg = W + (size_t)group * w_group_stride;

  // weight rows of this lane: tile row g and tile row g + 8
  int wr0, wr1;
  int rope_f0 = 0;      // ROPE: first of this CTA's 8 low-half features
  if (ROPE) {
    const int groups = rope.D >> 4;                    // 8-dim groups in half a head
    const int head = blockIdx.y / groups, j = blockIdx.y - head * groups;
    rope_f0 = head * rope.D + j * 8;
    wr0 = rope_f0 + g;
    wr1 = wr0 + (rope.D >> 1);
  } else if (SWIGLU) {
    const int f = min(n0 + g, N - 1);
    wr0 = f;            // gate
    wr1 = N + f;        // up
  } else {
    wr0 = min(n0 + g, N - 1);
    wr1 = min(n0 + g + 8, N - 1);
  }
  const __nv_bfloat16* w0 = Wg + (size_t)wr0 * K + 8 * t;
  const __nv_bfloat16* w1 = Wg + (size_t)wr1 * K + 8 * t;
  // packed form: tile row of each of the lane's two rows, and the tile strides
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

  // X rows of this lane: row g of every 8-row tile
  const __nv_bfloat16* xp[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int r = m0 + nt * 8 + g;
    long src = -1;
    if (r < row_end) {
      src = x_rows ? (long)x_rows[r] : (long)r;
      if (src < 0 || src >= M) {               // (x_rows holds pair indices below M)
        atomicCAS(&g_skinny_index_error, 0, 3);
        src = -1;
      } else if (x_rows) {
        src /= x_div;
      }
    }
    xp[nt] = src >= 0 ? X + src * (long)ldx + 8 * t : nullptr;
  }

  float acc[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[nt][i] = 0.f;

  // this member's chunks of k: [chunk_begin, nchunks)
  int chunk_begin = 0, nchunks = (K + 31) >> 5;
  if (ksplit > 1) {
    const int per = (nchunks + ksplit - 1) / ksplit;
    chunk_begin = min(member * per, nchunks);
    nchunks = min(chunk_begin + per, nchunks);
  }
  // (rounds of equal size - 3 + 3 chunks instead of 4 + 2 - were tried: the run-time round size cost
  // 15 % of a decode step)
  for (int c0 = chunk_begin + warp; c0 < nchunks; c0 += kWarps * kUnroll) {
    // a round: ask for the weights and the matching pieces of X of kUnroll chunks at once, so
    // that the (L2) latency of X hides behind the (DRAM) latency of W
    uint4 a[kUnroll], b[kUnroll], xv[kUnroll][NT];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int k = (c0 + u * kWarps) * 32;
      const bool live = c0 + u * kWarps < nchunks;
      if (PACKED && live) {
        const int kk = k + 8 * t;                   // < padded K: the padding holds zeros
        const __nv_bfloat16* tile = Wg + ptile + (size_t)(kk >> 6) * (TROWS * 64);
        const int j = (kk >> 3) & 7;
        a[u] = ld_stream(tile + pr0 * 64 + ((j ^ (pr0 & 7)) << 3));
        b[u] = ld_stream(tile + pr1 * 64 + ((j ^ (pr1 & 7)) << 3));
      } else if (!PACKED && live && k + 8 * t + 8 <= K) {
        a[u] = ld_stream(w0 + k);
        b[u] = ld_stream(w1 + k);
      } else {
        a[u] = make_uint4(0, 0, 0, 0);
        b[u] = make_uint4(0, 0, 0, 0);
      }
    }
    if (!waited) {
      // the rows of X (and, for the rotary epilogue, the step's tables) are read only from here on
      chain_wait(rope.positions, rope.row_seg, rope.block_table);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) chain_fresh(xp[nt]);      // no load of X may be placed above the wait
      waited = true;
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int k = (c0 + u * kWarps) * 32;
      const bool in = c0 + u * kWarps < nchunks && k + 8 * t + 8 <= K;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        xv[u][nt] = make_uint4(0, 0, 0, 0);
        if (in && nt < ntiles && xp[nt]) xv[u][nt] = ld_cached(xp[nt] + k);
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        if (nt < ntiles) {
          mma_bf16(acc[nt], a[u].x, b[u].x, a[u].y, b[u].y, xv[u][nt].x, xv[u][nt].y);
          mma_bf16(acc[nt], a[u].z, b[u].z, a[u].w, b[u].w, xv[u][nt].z, xv[u][nt].w);
        }
      }
    }
  }

  if (!waited) chain_wait(rope.positions, rope.row_seg, rope.block_table);   // a warp without chunks: no write, no table read before the wait
  chain_release_late();
  // add the warps' partial sums in warp order
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) partial[warp][(nt * 4 + i) * 32 + lane] = acc[nt][i];
  __syncthreads();
  if (ksplit > 1) {
    // members 1.. hand their sums to member 0 and are done; member 0 adds them in member order
    if (member > 0) {
      asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");       // member 0 is running
      for (int e = threadIdx.x; e < NT * 2 * 32; e += blockDim.x) {
        const int l = e & 31, h = (e >> 5) & 1, nt = e >> 6;
        float lo = 0.f, hi = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
          lo += partial[w][(nt * 4 + h) * 32 + l];
          hi += partial[w][(nt * 4 + h + 2) * 32 + l];
        }
        const unsigned a = (unsigned)__cvta_generic_to_shared(&others[member - 1][2 * e]);
        unsigned remote;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(a), "r"(0));
        asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};" ::"r"(remote), "f"(lo), "f"(hi) : "memory");
      }
      asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
      asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
      return;
    }
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");         // the others' sums are here
  }
  for (int e = threadIdx.x; e < ntiles * 2 * 32; e += blockDim.x) {
    // e -> (tile nt, column half h of the fragment, lane l); this thread owns fragment
    // entries (c[h], c[h + 2]) = (row g, row g + 8) of token column 2 t + h
    const int l = e & 31, h = (e >> 5) & 1, nt = e >> 6;
    float lo = 0.f, hi = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      lo += partial[w][(nt * 4 + h) * 32 + l];
      hi += partial[w][(nt * 4 + h + 2) * 32 + l];
    }
    for (int s = 1; s < ksplit; ++s) {
      lo += others[s - 1][2 * e];
      hi += others[s - 1][2 * e + 1];
    }
    const int gg = l >> 2, tt = l & 3;
    const int row = m0 + nt * 8 + 2 * tt + h;          // token (sorted position) of this column
    if (row >= row_end) continue;
    if (ROPE) {
      const int half = rope.D >> 1;
      const int f0 = rope_f0 + gg, f1 = f0 + half;
      const int head = f0 / rope.D, d = f0 - head * rope.D;
      if (rope.bias) { lo += rope.bias[f0]; hi += rope.bias[f1]; }
      const int pos = rope.positions[row];
      if (head < rope.Hq + rope.Hkv) {                 // queries and keys turn, values do not
        const float angle = (float)pos * rope.inv_freq[d];
        const float c = cosf(angle), sn = sinf(angle);
        const float ra = lo * c - hi * sn, rb = lo * sn + hi * c;
        lo = ra;
        hi = rb;
      }
      if (head < rope.Hq) {
        Y[(size_t)row * ldy + f0] = from_float<TC>(lo);
        Y[(size_t)row * ldy + f1] = from_float<TC>(hi);
      } else if (rope.append) {
        const int lp = pos / rope.page_size;
        const int page = (lp >= 0 && lp < rope.bt_width) ? rope.block_table[(size_t)rope.row_seg[row] * rope.bt_width + lp] : -1;
        if (page >= 0 && page < rope.num_pages) {
          const bool is_v = head >= rope.Hq + rope.Hkv;
          const int kvh = head - rope.Hq - (is_v ? rope.Hkv : 0);
          __nv_bfloat16* dst = rope.pages + ((((size_t)page * 2 + (is_v ? 1 : 0)) * rope.Hkv + kvh) * rope.page_size +
                                             (size_t)(pos - lp * rope.page_size)) * rope.D;
          dst[d] = __float2bfloat16_rn(lo);
          dst[d + half] = __float2bfloat16_rn(hi);
        }
      }
    } else if (SWIGLU) {
      const int f = n0 + gg;
      if (f < N) Y[(size_t)row * ldy + f] = from_float<TC>(lo / (1.f + expf(-lo)) * hi);
    } else {
      const int f0 = n0 + gg, f1 = n0 + gg + 8;
      if (f0 < N) Y[(size_t)row * ldy + f0] = from_float<TC>(lo);
      if (f1 < N) Y[(size_t)row * ldy + f1] = from_float<TC>(hi);
    }
  }
}

int g_skinny_max_split = kMaxSplit;      // nf_set_skinny_max_split(): 1 turns the split over k off

template <int NT, bool SWIGLU, bool PACKED, typename TC>
static int launch_nt(const void* X, int ldx, const void* W, size_t wgs, void* Y, int ldy, int M, int N,
                     int K, int groups, int max_rows, const int* offsets, const int* x_rows, int x_div,
                     const int* group_map, int n_mapped, int early_index, cudaStream_t stream) {
  const int feat = SWIGLU ? 8 : 16;
  dim3 grid((max_rows + 8 * NT - 1) / (8 * NT), (N + feat - 1) / feat, group_map ? n_mapped : groups);
  NF_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "skinny_gemm: too many feature tiles or groups");
  // A dense product whose CTAs would not even fill the SMs twice over splits k between the
  // members of a cluster, as long as every member's warps still get a chunk each.
  int ksplit = 1;
  if (groups == 1 && !offsets && !x_rows && !group_map) {
    const long long ctas = (long long)grid.x * grid.y;
    const int nchunks = (K + 31) / 32;
    while (ksplit * 2 <= g_skinny_max_split && ctas * ksplit * 2 <= 4 * 148 && nchunks / (ksplit * 2) >= kWarps) ksplit *= 2;
  }
  if (ksplit > 1) {
    grid.x *= ksplit;
    launch_chained_cluster(skinny_gemm_kernel<NT, SWIGLU, PACKED, TC>, grid, dim3(kWarps * 32), 0, stream, ksplit,
                           (const __nv_bfloat16*)X, ldx, (const __nv_bfloat16*)W, wgs, (TC*)Y, ldy, M, N, K, offsets,
                           x_rows, x_div, group_map, early_index, groups, RopeEpilogue{}, ksplit);
  } else {
    launch_chained(skinny_gemm_kernel<NT, SWIGLU, PACKED, TC>, grid, dim3(kWarps * 32), 0, stream,
                   (const __nv_bfloat16*)X, ldx, (const __nv_bfloat16*)W, wgs, (TC*)Y, ldy, M, N, K, offsets, x_rows,
                   x_div, group_map, early_index, groups, RopeEpilogue{}, 1);
  }
  return check_launch("skinny_gemm");
}

template <bool SWIGLU, typename TC>
static int launch_sw(int nt, bool packed, const void* X, int ldx, const void* W, size_t wgs, void* Y, int ldy, int M,
                     int N, int K, int groups, int max_rows, const int* offsets, const int* x_rows,
                     int x_div, const int* group_map, int n_mapped, int early_index, cudaStream_t stream) {
  if (packed) {
    if (nt == 1) return launch_nt<1, SWIGLU, true, TC>(X, ldx, W, wgs, Y, ldy, M, N, K, groups, max_rows, offsets, x_rows, x_div, group_map, n_mapped, early_index, stream);
    return launch_nt<2, SWIGLU, true, TC>(X, ldx, W, wgs, Y, ldy, M, N, K, groups, max_rows, offsets, x_rows, x_div, group_map, n_mapped, early_index, stream);
  }
  if (nt == 1) return launch_nt<1, SWIGLU, false, TC>(X, ldx, W, wgs, Y, ldy, M, N, K, groups, max_rows, offsets, x_rows, x_div, group_map, n_mapped, early_index, stream);
  return launch_nt<2, SWIGLU, false, TC>(X, ldx, W, wgs, Y, ldy, M, N, K, groups, max_rows, offsets, x_rows, x_div, group_map, n_mapped, early_index, stream);
}

}  // namespace nf

using namespace nf;

// Y[M, N] = epilogue(X[M, K] W[g]^T), bfloat16 inputs, float32 accumulation.
// out_dtype: 1 bfloat16, 0 float32.  max_rows: bound on the rows of any one group.
// Needs K % 8 == 0 and 16-byte aligned rows (ldx % 8 == 0, bases aligned).
// packed != 0: W is in the packed tile layout (w_group_stride then counts packed elements).
// group_map / n_mapped: optional list of the groups to run (-1 entries are skipped); the grid
// then has n_mapped groups instead of `groups`.  early_index != 0: offsets, x_rows and group_map
// were complete before the kernel that precedes this launch in the stream began, so they may be
// read - and the first weights asked for - before that kernel has finished.
extern "C" int nf_skinny_gemm(const void* X, int ldx, const void* W, long long w_group_stride, void* Y,
                              int ldy, int M, int N, int K, int groups, int max_rows,
                              const int* offsets, const int* x_rows, int x_div, int swiglu,
                              int out_dtype, int packed, const int* group_map, int n_mapped,
                              int early_index, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  NF_REQUIRE(M > 0 && N > 0 && K > 0 && groups > 0 && x_div > 0, "skinny_gemm: bad sizes M=%d N=%d K=%d", M, N, K);
  NF_REQUIRE(K % 8 == 0 && ldx % 8 == 0, "skinny_gemm: K=%d and the row stride %d must be multiples of 8", K, ldx);
  NF_REQUIRE(((uintptr_t)X % 16 == 0) && ((uintptr_t)W % 16 == 0) && (w_group_stride % 8 == 0),
             "skinny_gemm: operands must be 16-byte aligned");
  NF_REQUIRE(groups == 1 || offsets, "skinny_gemm: grouped product needs row offsets");
  // at most 16 rows a CTA: more rows are further CTAs over the same weight rows, launched
  // next to each other so that the second reading comes from L2
  const int nt = max_rows <= 8 ? 1 : 2;
  const size_t wgs = (size_t)w_group_stride;
  if (swiglu) {
    NF_REQUIRE(out_dtype == kBF16, "skinny_gemm: the SwiGLU epilogue writes bfloat16");
    return launch_sw<true, __nv_bfloat16>(nt, packed != 0, X, ldx, W, wgs, Y, ldy, M, N, K, groups, max_rows, offsets, x_rows, x_div, group_map, n_mapped, early_index, stream);
  }
  if (out_dtype == kBF16)
    return launch_sw<false, __nv_bfloat16>(nt, packed != 0, X, ldx, W, wgs, Y, ldy, M, N, K, groups, max_rows, offsets, x_rows, x_div, group_map, n_mapped, early_index, stream);
  return launch_sw<false, float>(nt, packed != 0, X, ldx, W, wgs, Y, ldy, M, N, K, groups, max_rows, offsets, x_rows, x_div, group_map, n_mapped, early_index, stream);
}

// Most cluster members a dense product may split k between (1, 2 or 4; 1: never split).
extern "C" int nf_set_skinny_max_split(int n) {
  nf::g_skinny_max_split = n < 1 ? 1 : (n > nf::kMaxSplit ? nf::kMaxSplit : n);
  return 0;
}

// qkv = X Wqkv^T with bias, rotation and the append to the cache in the epilogue (see
// RopeEpilogue): queries land rotated in Y [M, (Hq + 2 Hkv) D] (its key and value columns are
// left untouched), keys and values in `pages` at (block_table[row_seg[r]], positions[r]).
// bfloat16; the rotation covers the whole head; D % 16 == 0; M <= 16 rows.
extern "C" int nf_skinny_qkv_rope(const void* X, int ldx, const void* W, void* Y, int ldy, int M, int K,
                                  const float* bias, const int* positions, const int* row_seg,
                                  const float* inv_freq, int Hq, int Hkv, int D, void* pages,
                                  const int* block_table, int bt_width, int page_size, int num_pages,
                                  int append, cudaStream_t stream) {
  if (M == 0) return 0;
  NF_REQUIRE(M > 0 && M <= 16 && K > 0 && Hq > 0 && Hkv > 0, "skinny_qkv_rope: bad sizes M=%d K=%d", M, K);
  NF_REQUIRE(D > 0 && D % 16 == 0, "skinny_qkv_rope: head_dim %d must be a multiple of 16", D);
  NF_REQUIRE(K % 8 == 0 && ldx % 8 == 0, "skinny_qkv_rope: K=%d and the row stride %d must be multiples of 8", K, ldx);
  NF_REQUIRE(((uintptr_t)X % 16 == 0) && ((uintptr_t)W % 16 == 0), "skinny_qkv_rope: operands must be 16-byte aligned");
  NF_REQUIRE(positions && row_seg && inv_freq && pages && block_table, "skinny_qkv_rope: missing tables");
  const int N = (Hq + 2 * Hkv) * D;
  RopeEpilogue r{bias, positions, row_seg, inv_freq, (__nv_bfloat16*)pages, block_table,
                 Hq, Hkv, D, bt_width, page_size, num_pages, append};
  dim3 grid(1, N / 16, 1);
  NF_REQUIRE(grid.y <= 65535, "skinny_qkv_rope: too many heads");
  if (M <= 8)
    launch_chained(skinny_gemm_kernel<1, false, false, __nv_bfloat16, true>, grid, dim3(kWarps * 32), 0, stream,
                   (const __nv_bfloat16*)X, ldx, (const __nv_bfloat16*)W, (size_t)0, (__nv_bfloat16*)Y, ldy, M, N, K,
                   (const int*)nullptr, (const int*)nullptr, 1, (const int*)nullptr, 0, 1, r, 1);
  else
    launch_chained(skinny_gemm_kernel<2, false, false, __nv_bfloat16, true>, grid, dim3(kWarps * 32), 0, stream,
                   (const __nv_bfloat16*)X, ldx, (const __nv_bfloat16*)W, (size_t)0, (__nv_bfloat16*)Y, ldy, M, N, K,
                   (const int*)nullptr, (const int*)nullptr, 1, (const int*)nullptr, 0, 1, r, 1);
  return check_launch("skinny_qkv_rope");
}

// 0, or the code of the first index a grouped product found outside its operands since the last
// call (1 group, 2 row range, 3 row index).  Synchronises.
extern "C" int nf_skinny_index_status() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_skinny_index_error, sizeof(int)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(g_skinny_index_error, &zero, sizeof(int));
  return v;
}
