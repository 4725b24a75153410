// Routed experts at prefill: a grouped GEMM on the 5th-generation tensor cores.
//
//   act[p, :] = silu(x[p] Wgate_e^T) * (x[p] Wup_e^T)      (first product, SwiGLU epilogue)
//   y[p, :]   = act[p] Wdown_e^T                           (second product)
// for every sorted (token, expert) pair p of expert e, rows [offsets[e], offsets[e+1]).
//
// Reference: a host loop over experts with one rocBLAS GEMM each plus gather, activation and
// scale kernels (src/models/model.hip:355-427).  Here one launch covers all experts.
//
// Shape of the work.  With ~137 rows per expert (2,048 tokens, 60 experts, top-4) the
// product does ~137 FLOP per weight byte, below the machine's ridge: the bound is reading
// each expert's weights once from HBM.  So the weights are the 128-row M operand
// (`tcgen05.mma.cta_group::1.kind::f16`, M = 128 features), the expert's tokens are the N
// operand (N = the expert's row count rounded up to 16, at most 256 per pass), and a CTA owns
// (expert, 128 features): it streams its slice of the weight matrix exactly once while the
// expert's rows come from L2.  Ragged row counts cost at most 15 padded columns, not a
// half-empty 128-row tile.
//
// Weights are held *packed* (see kernels/ops.py `pack_weights`): tiles of 128 rows x 64 k,
// stored contiguously in the order a CTA reads them and already in the 128-byte-swizzled
// image the tensor core expects, so a stage's weights are one contiguous `cp.async.bulk`
// copy (32 KB for gate + up) - a stream of whole DRAM pages instead of 128-byte pieces 4 KB
// apart.  The expert's token rows arrive by TMA tensor copies (`cp.async.bulk.tensor.2d`,
// 128-byte swizzle, boxes of 64 rows, as many as the pass has rows).  Both land in a ring of
// shared-memory stages guarded by mbarriers, as deep as shared memory allows for this
// expert's row count; one elected thread issues the MMAs,
// whose float32 accumulators live in tensor memory (gate in columns [0, 256), up in
// [256, 512)); `tcgen05.commit` hands stages back to the producer and the finished
// accumulator to twelve epilogue warps, which read it with `tcgen05.ld`, apply the epilogue
// and store bfloat16.  No TMA multicast, no clusters.
//
// Every wait on an mbarrier is bounded: after a fixed number of polls the kernel records a
// code in `g_tc_error`, tells its other warps to stop, waits (again bounded) for its own
// copies in flight, frees its tensor memory and returns.
#include "tcgen05.cuh"

namespace nf {

constexpr int kBM = 128;          // features per CTA (MMA M)
constexpr int kBK = 64;           // k per stage: 64 bf16 = one 128-byte swizzle row
constexpr int kBNMax = 256;       // tokens per pass (MMA N, columns of one accumulator)
constexpr int kTmemCols = 512;
constexpr int kEpilogueWarps = 12; // three for each quadrant of tensor-memory lanes
constexpr int kTcThreads = 64 + 32 * kEpilogueWarps;
constexpr int kWarpCols = 48;      // accumulator columns a warp holds in registers at a time
constexpr int kRoundCols = kWarpCols * kEpilogueWarps / 4;
constexpr int kXBox = 64;         // token rows per TMA box
constexpr int kMaxStages = 8;
constexpr int kMaxGroupsTc = 1024;   // groups one launch may have (their pass counts live in shared memory)
constexpr int kSmemBudget = 225 * 1024;   // + 1 KB of alignment slack + a few static bytes <= the 227 KB a CTA may have

__device__ int g_tc_error = 0;

// Instruction descriptor: bf16 x bf16 -> f32, both operands K-major, M = 128, N = n.
__device__ __forceinline__ unsigned instr_desc(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(n >> 3) << 17) | ((unsigned)(kBM >> 4) << 24);
}

struct __align__(8) Barriers {
  unsigned long long full[kMaxStages], empty[kMaxStages], acc_full[2], acc_empty[2];
  unsigned tmem_base;
  int stop;
};

// Persistent: one CTA per SM walks the work items (group, pass of 256 rows, feature tile)
// cta, cta + grid, ... with feature tiles varying fastest, so CTAs that run together share an
// expert's token rows in L2, and the passes of a heavily loaded expert - which re-read its
// weights - run next to each other and find them in L2.  Items cost about the same, so the
// static assignment stays balanced however unevenly the router loads the experts.  448 threads: warp 0 producer, warp 1 MMA + tensor memory, warps 2..13 epilogue.  The
// producer is not held back by the epilogue: while the epilogue warps drain an item's
// accumulator, the stages fill with the next item's first k tiles, so the memory pipe never
// goes idle between items.  Wp: packed weights [groups][feature tiles][k tiles][A_ROWS][64].
// PAIR (second product only): an item is two neighbouring feature tiles of one expert, with an
// accumulator each, over the same token rows.  With a hundred and more rows an expert, a tile's
// token rows (rows x K) weigh as much as its weights (128 x K), and every feature tile of the
// expert fetches them again from L2; the CTA's load pipe, not HBM, is then the bound.  Two tiles
// an item halve that traffic.  (The first product has gate and up in one item already.)
template <bool SWIGLU, bool PAIR>
__global__ void __launch_bounds__(kTcThreads, 1)
grouped_gemm_tc_kernel(const __nv_bfloat16* __restrict__ Wp, const __grid_constant__ CUtensorMap map_x,
                       const __grid_constant__ CUtensorMap map_x_half,
                       const int* __restrict__ offsets, __nv_bfloat16* __restrict__ out, int ldo,
                       int n_features, int K, int groups) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  static_assert(!(SWIGLU && PAIR), "the first product already has two weight tiles an item");
  constexpr int TILE_BYTES = kBM * kBK * 2;
  constexpr int A_BYTES = (SWIGLU || PAIR ? 2 : 1) * TILE_BYTES;     // gate (+ up) tile, or two feature tiles
  constexpr int FT_STEP = PAIR ? 2 : 1;                               // feature tiles an item covers
  constexpr int BOX_BYTES = kXBox * kBK * 2;
  __shared__ int s_max_rows;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k_steps = (K + kBK - 1) / kBK;
  const int n_ftiles = (n_features + kBM - 1) / kBM;
  const int n_fitems = (n_ftiles + FT_STEP - 1) / FT_STEP;      // items along the features

  // Barriers and the groups' pass table at the head of shared memory, the stages behind them.
  // Launched chained, the CTA is resident while the kernel before it drains: barriers and
  // tensor memory are set up meanwhile, and everything that reads what that kernel (or the
  // routing before it) wrote comes after the wait.
  Barriers* bars = reinterpret_cast<Barriers*>(smem);
  int* s_pass_start = reinterpret_cast<int*>(bars + 1);     // [groups + 1] first pass index of every group
  const int head_bytes = ((int)sizeof(Barriers) + (groups + 1) * (int)sizeof(int) + 1023) & ~1023;
  unsigned char* stage0 = smem + head_bytes;
  volatile int* stop = &bars->stop;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kMaxStages; ++s) { mbar_init(&bars->full[s], 1); mbar_init(&bars->empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&bars->acc_full[b], 1); mbar_init(&bars->acc_empty[b], kEpilogueWarps); }
    bars->stop = 0;
    s_max_rows = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  chain_wait(offsets);

  // stage geometry, the same for every item: weights + as many 64-row boxes as the largest
  // pass of any group needs.  Thread g counts the passes of group g; warp 0 adds them up.
  __syncthreads();
  {
    int mx = 0;
    for (int g = threadIdx.x; g < groups; g += blockDim.x) {
      const int n = offsets[g + 1] - offsets[g];
      mx = max(mx, n);
      s_pass_start[g + 1] = (n + kBNMax - 1) / kBNMax;
    }
    if (mx) atomicMax(&s_max_rows, mx);
  }
  __syncthreads();
  if (warp == 0) {
    int run = 0;
    if (lane == 0) s_pass_start[0] = 0;
    for (int g0 = 0; g0 < groups; g0 += 32) {
      const int g = g0 + lane;
      int v = g < groups ? s_pass_start[g + 1] : 0;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int o = __shfl_up_sync(0xffffffffu, v, d);
        if (lane >= d) v += o;
      }
      if (g < groups) s_pass_start[g + 1] = run + v;
      run += __shfl_sync(0xffffffffu, v, 31);
    }
  }
  constexpr int kAccBuffers = (SWIGLU || PAIR) ? 1 : 2;      // accumulators of kBNMax columns that fit beside each other
  const int max_boxes = (min(max(s_max_rows, 1), kBNMax) + kXBox - 1) / kXBox;
  const int stage_bytes = A_BYTES + max_boxes * BOX_BYTES;
  const int stages = min(kMaxStages, (kSmemBudget - head_bytes) / stage_bytes);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem = bars->tmem_base;
  const int n_items = s_pass_start[groups] * n_fitems;

  if (warp == 0) {
    // ---- producer ---------------------------------------------------------------------------
    if (lane == 0) {
      int it = 0, issued = 0;
      bool ok = true;
      int group = 0;
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
        const int gp = item / n_fitems, ft = (item - gp * n_fitems) * FT_STEP;      // global pass index, feature tile
        while (s_pass_start[group + 1] <= gp) ++group;
        const int pass = gp - s_pass_start[group];
        const int row_begin = offsets[group], n_rows = offsets[group + 1] - row_begin;
        constexpr int W_TILE_BYTES = SWIGLU ? 2 * TILE_BYTES : TILE_BYTES;    // one feature tile's weights of one k step
        const unsigned char* w_tile = reinterpret_cast<const unsigned char*>(Wp) +
                                      ((size_t)group * n_ftiles + ft) * k_steps * W_TILE_BYTES;
        const bool second = PAIR && ft + 1 < n_ftiles;                    // the pair's second tile exists
        const int a_bytes = PAIR ? (second ? 2 : 1) * TILE_BYTES : A_BYTES;
        {
          const int x_row = row_begin + pass * kBNMax;
          const int rows_here = min(kBNMax, n_rows - pass * kBNMax);
          const int boxes = (rows_here + kXBox - 1) / kXBox;
          // a last box with at most 32 rows is fetched through the map of half the height: the same
          // number of copies, a quarter of a stage's token rows fewer on average
          const bool half_last = rows_here - (boxes - 1) * kXBox <= kXBox / 2;
          const int x_bytes = boxes * BOX_BYTES - (half_last ? BOX_BYTES / 2 : 0);
          for (int ks = 0; ks < k_steps; ++ks, ++it) {
            const int s = it % stages;
            if (!mbar_wait(&bars->empty[s], ((it / stages) & 1) ^ 1, stop, 1, &g_tc_error)) { ok = false; break; }
            unsigned char* st = stage0 + (size_t)s * stage_bytes;
            mbar_expect_tx(&bars->full[s], a_bytes + x_bytes);
            if (PAIR) {
              bulk_load(st, w_tile + (size_t)ks * TILE_BYTES, TILE_BYTES, &bars->full[s]);
              if (second)
                bulk_load(st + TILE_BYTES, w_tile + ((size_t)k_steps + ks) * TILE_BYTES, TILE_BYTES, &bars->full[s]);
            } else {
              bulk_load(st, w_tile + (size_t)ks * A_BYTES, A_BYTES, &bars->full[s]);
            }
            for (int b = 0; b < boxes; ++b)
              tma_load_2d(st + A_BYTES + b * BOX_BYTES, (half_last && b == boxes - 1) ? &map_x_half : &map_x, ks * kBK,
                          x_row + b * kXBox, &bars->full[s]);
            issued = it + 1;
          }
        }
      }
      if (!ok) {
        // copies already asked for still land in this CTA's shared memory: wait for them
        for (int j = max(0, issued - stages); j < issued; ++j) {
          const int s = j % stages;
          for (unsigned i = 0; i < (1u << 20); ++i)
            if (mbar_try(&bars->full[s], (j / stages) & 1)) break;
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer -----------------------------------------------------------------------------
    if (lane == 0) {
      int it = 0, pass_ctr = 0;
      bool ok = true;
      int group = 0;
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++pass_ctr) {
        const int gp = item / n_fitems;
        while (s_pass_start[group + 1] <= gp) ++group;
        const int pass = gp - s_pass_start[group];
        const int n_rows = offsets[group + 1] - offsets[group];
        const bool second = SWIGLU || (PAIR && (item - gp * n_fitems) * FT_STEP + 1 < n_ftiles);
        {
          // without the second (up) accumulator there is room for two: the epilogue of one item
          // runs under the products of the next
          const int ab = pass_ctr % kAccBuffers, aph = (pass_ctr / kAccBuffers) & 1;
          const unsigned acc_tmem = tmem + ab * kBNMax;
          if (!mbar_wait(&bars->acc_empty[ab], aph ^ 1, stop, 2, &g_tc_error)) { ok = false; break; }
          tc_fence_after();
          const int n = min(kBNMax, (n_rows - pass * kBNMax + 15) & ~15);
          const unsigned idesc = instr_desc(n);
          for (int ks = 0; ks < k_steps; ++ks, ++it) {
            const int s = it % stages;
            if (!mbar_wait(&bars->full[s], (it / stages) & 1, stop, 3, &g_tc_error)) { ok = false; break; }
            tc_fence_after();
            unsigned char* st = stage0 + (size_t)s * stage_bytes;
            const unsigned long long a0 = smem_desc(st);
            const unsigned long long a1 = smem_desc(st + kBM * kBK * 2);
            const unsigned long long b = smem_desc(st + A_BYTES);
#pragma unroll
            for (int kk = 0; kk < kBK / 16; ++kk) {
              // 16 k = 32 bytes further along the swizzled row: +2 in the address field
              const unsigned acc = (ks > 0 || kk > 0) ? 1u : 0u;
              tc_mma(acc_tmem, a0 + 2 * kk, b + 2 * kk, idesc, acc);
              if (second) tc_mma(acc_tmem + kBNMax, a1 + 2 * kk, b + 2 * kk, idesc, acc);
            }
            tc_commit(&bars->empty[s]);          // the stage is free once these MMAs have read it
          }
          if (ok) tc_commit(&bars->acc_full[ab]);   // the accumulator is complete once they have all run
        }
      }
    }
  } else {
    // ---- epilogue: warps 2..13 read tensor-memory lanes 32 * (warp % 4) .. + 31 ---------------------
    const int quad = warp & 3, half = (warp - 2) >> 2;     // the warps of a quadrant's lanes take 32 columns in turn
    int pass_ctr = 0;
    bool ok = true;
    int group = 0;
    for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++pass_ctr) {
      const int gp = item / n_fitems, ft0 = (item - gp * n_fitems) * FT_STEP;
      while (s_pass_start[group + 1] <= gp) ++group;
      const int pass = gp - s_pass_start[group];
      const int row_begin = offsets[group], n_rows = offsets[group + 1] - row_begin;
      const int tiles_here = (PAIR && ft0 + 1 < n_ftiles) ? 2 : 1;      // accumulators of this item to drain
      {
        const int ab = pass_ctr % kAccBuffers, aph = (pass_ctr / kAccBuffers) & 1;
        if (!mbar_wait(&bars->acc_full[ab], aph, stop, 4, &g_tc_error)) { ok = false; break; }
        tc_fence_after();
        const int p0 = row_begin + pass * kBNMax;
        const int valid = min(kBNMax, n_rows - pass * kBNMax);
        // Each warp turns kWarpCols columns of every round of kRoundCols into bfloat16 values in
        // registers; after the last round's loads the accumulator goes back to the MMA warp, and
        // the stores run under the next item's products.
        for (int tile = 0; tile < tiles_here; ++tile) {
        const int f = (ft0 + tile) * kBM + quad * 32 + lane;
        const unsigned lane_addr = tmem + (ab + tile) * kBNMax + ((unsigned)(quad * 32) << 16);
        for (int r0 = 0; r0 < valid; r0 += kRoundCols) {
          const int c0 = r0 + half * kWarpCols;
          unsigned pk[kWarpCols / 2];       // two bfloat16 results a register
          if (c0 < valid) {
#pragma unroll
            for (int j = 0; j < kWarpCols / 16; ++j) {
              if (c0 + 16 * j < valid) {
                unsigned g[16], u[16];
                tc_ld16(lane_addr + c0 + 16 * j, g);
                if (SWIGLU) tc_ld16(lane_addr + kBNMax + c0 + 16 * j, u);
                tc_wait_ld();
#pragma unroll
                for (int c = 0; c < 16; c += 2) {
                  float v0 = __uint_as_float(g[c]), v1 = __uint_as_float(g[c + 1]);
                  // the result is rounded to bfloat16 (2^-9): the fast exponential's 2^-21 is far below
                  if (SWIGLU) {
                    v0 = __fdividef(v0, 1.f + __expf(-v0)) * __uint_as_float(u[c]);
                    v1 = __fdividef(v1, 1.f + __expf(-v1)) * __uint_as_float(u[c + 1]);
                  }
                  const __nv_bfloat162 h = __floats2bfloat162_rn(v0, v1);
                  pk[8 * j + c / 2] = *reinterpret_cast<const unsigned*>(&h);
                }
              }
            }
          }
          if (r0 + kRoundCols >= valid && tile + 1 == tiles_here) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->acc_empty[ab]);
          }
          if (c0 < valid && f < n_features) {
#pragma unroll
            for (int c = 0; c < kWarpCols; ++c)
              if (c0 + c < valid)
                out[(size_t)(p0 + c0 + c) * ldo + f] =
                    __ushort_as_bfloat16((unsigned short)((c & 1) ? pk[c / 2] >> 16 : pk[c / 2] & 0xffffu));
          }
        }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
}

// ---- host ---------------------------------------------------------------------------------------

template <bool SWIGLU, bool PAIR>
static int launch_tc(const void* Wp, const CUtensorMap& mx, const CUtensorMap& mx_half, const int* offsets, void* out, int ldo,
                     int n_features, int K, int groups, cudaStream_t stream) {
  const size_t smem = (size_t)kSmemBudget + 1024;
  static bool set = false;
  if (!set) {
    cudaError_t e = cudaFuncSetAttribute(grouped_gemm_tc_kernel<SWIGLU, PAIR>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    NF_REQUIRE(e == cudaSuccess, "grouped_gemm_tc: cannot have %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    set = true;
  }
  static int n_sm = 0;
  if (!n_sm) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
    if (n_sm <= 0) n_sm = 1;
  }
  // at least one pass per non-empty group; the kernel itself counts the exact number of items
  const int grid = n_sm;
  launch_chained(grouped_gemm_tc_kernel<SWIGLU, PAIR>, dim3(grid), dim3(kTcThreads), smem, stream,
                 (const __nv_bfloat16*)Wp, mx, mx_half, offsets, (__nv_bfloat16*)out, ldo, n_features, K, groups);
  return check_launch("grouped_gemm_tc");
}

}  // namespace nf

namespace nf {
int g_tc_pair = 1, g_tc_pair_min_rows = 64;
}

using namespace nf;

// 0: the second product never pairs feature tiles; otherwise it does from `min_rows` rows an
// expert (on average) on.
extern "C" int nf_set_grouped_gemm_pair(int on, int min_rows) {
  g_tc_pair = on ? 1 : 0;
  if (min_rows > 0) g_tc_pair_min_rows = min_rows;
  return 0;
}

// out[p, :n_features] for sorted rows p of every group.  X holds the rows in sorted order
// ([total_rows, K], already gathered).  Wp holds the groups' weights packed as
// [groups][ceil(n_features / 128)][ceil(K / 64)][128 or 256 rows][64], each tile in the
// 128-byte-swizzled image (SwiGLU: 128 gate rows then the 128 matching up rows per tile),
// zero-padded.  Needs K % 8 == 0 and a 16-byte aligned X (TMA).
extern "C" int nf_grouped_gemm_tc(const void* X, long long total_rows, const void* Wp, int groups,
                                  int n_features, int K, const int* offsets, void* out, int ldo,
                                  int swiglu, cudaStream_t stream) {
  if (total_rows == 0) return 0;
  NF_REQUIRE(total_rows > 0 && groups > 0 && n_features > 0 && K > 0, "grouped_gemm_tc: bad sizes");
  NF_REQUIRE(K % 8 == 0, "grouped_gemm_tc: K=%d must be a multiple of 8 (16-byte rows for TMA)", K);
  NF_REQUIRE(((uintptr_t)X % 16 == 0) && ((uintptr_t)Wp % 16 == 0), "grouped_gemm_tc: operands must be 16-byte aligned");
  NF_REQUIRE(groups <= kMaxGroupsTc, "grouped_gemm_tc: %d groups, at most %d", groups, kMaxGroupsTc);
  CUtensorMap mx, mx_half;
  if (int rc = make_map(&mx, X, total_rows, K, kXBox)) return rc;
  if (int rc = make_map(&mx_half, X, total_rows, K, kXBox / 2)) return rc;
  if (swiglu) return launch_tc<true, false>(Wp, mx, mx_half, offsets, out, ldo, n_features, K, groups, stream);
  // two feature tiles an item once an expert's rows weigh about as much as a tile's weights
  // (decided by the counts the host knows: all rows, all groups)
  if (g_tc_pair && total_rows >= (long long)g_tc_pair_min_rows * groups)
    return launch_tc<false, true>(Wp, mx, mx_half, offsets, out, ldo, n_features, K, groups, stream);
  return launch_tc<false, false>(Wp, mx, mx_half, offsets, out, ldo, n_features, K, groups, stream);
}

// A wait that nothing will ever satisfy, given `polls` polls: the bounded wait runs out, records
// code 9 and the kernel returns; the context stays usable.  It shows (to tests) that a wait
// which gives up reaches the host as a status, the way the kernels above report theirs.
__global__ void bounded_wait_selftest_kernel(unsigned polls) {
  __shared__ __align__(8) unsigned long long bar;
  __shared__ int stop;
  if (threadIdx.x == 0) {
    stop = 0;
    mbar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    mbar_wait(&bar, 0, &stop, 9, &g_tc_error, polls);
  }
}

extern "C" int nf_bounded_wait_selftest(int polls, cudaStream_t stream) {
  NF_REQUIRE(polls > 0 && polls <= (1 << 20), "bounded wait self-test: polls=%d must lie in [1, 2^20]", polls);
  bounded_wait_selftest_kernel<<<1, 32, 0, stream>>>((unsigned)polls);
  return check_launch("bounded_wait_selftest");
}

// 0 if no tensor-core kernel has given up on a wait since the last call; else the code of the
// first wait that did (1 producer, 2 accumulator hand-back, 3 operands, 4 epilogue).  Synchronises.
extern "C" int nf_grouped_gemm_tc_status() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_tc_error, sizeof(int)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(g_tc_error, &zero, sizeof(int));
  return v;
}
