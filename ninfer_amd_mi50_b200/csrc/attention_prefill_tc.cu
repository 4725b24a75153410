// Prefill attention in bfloat16 on the 5th-generation tensor cores: the flash decomposition of
// attention_prefill.cu with both products as ``tcgen05.mma`` and the accumulators in tensor
// memory.
//
// Reference: ``prefill_attention_kernel<D>`` (src/ops/attention.hip:136-268): tiles of 16 queries
// x 32 keys on the vector units, causal mask on absolute positions, online softmax.  Same
// mathematics: scores * 1/sqrt(D), key j visible to a row at position p iff
// max(0, p - window + 1) <= j <= p, softmax and its sums in float32.
//
// Shape of the work.  A tile is up to 128 consecutive rows of one segment and one query head;
// a CTA runs the tiles of its entry of `tiles` one after the other (the caller gives one tile a
// CTA, heaviest first, see `StepContext.paired_query_tiles`; a second one is taken if present).
// Keys and values come in blocks of 128 keys, aligned to multiples of 128, so the order of a
// row's sums depends on its own position only.
//
//   warp 0     producer of Q and K, warp 10 producer of V: TMA tensor copies (128-byte swizzle),
//              page by page through the block table, into two-stage rings (a key stage is free
//              as soon as its scores are done, a value stage after the second product)
//   warp 1     MMA issuer: S = Q K^T (M = 128 rows, N = 128 keys, both operands K-major) into
//              one of two S buffers in tensor memory, and O += P V (M = 128, N = D, P K-major
//              from shared memory, V as it lies in the cache: MN-major); QK of block b + 1 is
//              issued before PV of block b, so the tensor core works while the softmax runs
//   warps 2-9  softmax: row r is tensor-memory lane r; two threads share a row (warps w and w + 4
//              may touch the same 32 lanes) and take 64 of its 128 scores each: ``tcgen05.ld``,
//              mask, a reference maximum that is only raised when a score exceeds it by more than
//              2^8 (then O's row is rescaled in tensor memory), P = 2^(s - m) as bfloat16 into
//              shared memory in the swizzled K-major image; at the end of the tile O divided by
//              the row sum is stored
//
// Everything between the roles goes through mbarriers; every wait is bounded: after a fixed
// number of polls the kernel records a code in `g_fa_error`, tells its other warps to stop,
// waits (bounded) for its own copies in flight, frees its tensor memory and returns.
//
// Contract on the cache: rows of a page that lie beyond a request's position are read (whole
// pages are copied) and multiplied by zero, so they must hold finite numbers; the cache manager
// creates its pool zero-filled and only kernels write to it.
#include "tcgen05.cuh"

namespace nf {

namespace {

constexpr int kQ = 128;          // rows per tile (MMA M)
constexpr int kKeys = 128;       // keys per block (MMA N of the first product, K of the second)
constexpr int kFaThreads = 352;  // key producer, MMA issuer, 8 softmax warps, value producer
constexpr int kAtom = 128 * 128; // bytes of a swizzle atom column: 128 rows x 64 bf16
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRaise = 8.f;    // raise the reference maximum only beyond this many powers of two

__device__ int g_fa_error = 0;

struct __align__(8) FaBarriers {
  unsigned long long q_full, q_empty, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], s_empty[2], p_full,
      p_free, o_final, o_read;
  unsigned tmem_base;
  int stop;
};

// Shared-memory descriptor of an MN-major operand tile with 128-byte swizzle: 64 contiguous
// MN elements a row, rows = k, 8-row groups 1024 bytes apart, the next 64 MN elements `lbo`
// bytes further.
__device__ __forceinline__ unsigned long long smem_desc_mn(const void* p, unsigned lbo) {
  unsigned long long d = 0;
  d |= (unsigned long long)((smem_u32(p) & 0x3FFFFu) >> 4);
  d |= (unsigned long long)(lbo >> 4) << 16;
  d |= (unsigned long long)(1024 >> 4) << 32;
  d |= (unsigned long long)1 << 46;
  d |= (unsigned long long)2 << 61;
  return d;
}
// bf16 x bf16 -> f32, M = 128, N = n; b_mn: the B operand is MN-major.
__device__ __forceinline__ unsigned fa_idesc(int n, bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn ? (1u << 16) : 0u) | ((unsigned)(n >> 3) << 17) |
         ((unsigned)(kQ >> 4) << 24);
}

// 2^x by the special-function unit (2^-22 relative; P is rounded to bfloat16 right after);
// -inf gives 0.
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct TileInfo {
  int seg, row0, n_rows, pos_first, pos_last, kb_first, n_blocks;
};
__device__ __forceinline__ TileInfo tile_info(const int* tiles, int which, const int* seg_row0, const int* positions,
                                              int window) {
  TileInfo t;
  t.seg = tiles[4 * blockIdx.y + 2 * which];
  t.row0 = tiles[4 * blockIdx.y + 2 * which + 1];
  if (t.seg < 0) return t;
  t.n_rows = min(kQ, seg_row0[t.seg + 1] - t.row0);
  t.pos_first = positions[t.row0];
  t.pos_last = t.pos_first + t.n_rows - 1;
  int lo = 0;
  if (window > 0 && t.pos_first - window + 1 > 0) lo = t.pos_first - window + 1;
  t.kb_first = (lo / kKeys) * kKeys;
  t.n_blocks = (t.pos_last - t.kb_first) / kKeys + 1;
  return t;
}

template <int D>
__global__ void __launch_bounds__(kFaThreads, 1)
prefill_attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                            const int* __restrict__ block_table, int bt_width, const int* __restrict__ positions,
                            const int* __restrict__ seg_row0, const int* __restrict__ tiles,
                            __nv_bfloat16* __restrict__ out, int Hq, int Hkv, int page_size, int num_pages,
                            int window, float scale) {
  constexpr int ATOMS = D / 64;                   // 64-column swizzle atoms across the head
  constexpr int QB = ATOMS * kAtom;               // bytes of the Q tile, of a K block, of a V block
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* Qs = smem;
  unsigned char* KV = Qs + QB;                    // [2 stages][K block, V block]
  unsigned char* Ps = KV + 4 * QB;                // [2 atoms][128 rows][128 bytes]
  FaBarriers* bars = reinterpret_cast<FaBarriers*>(Ps + 2 * kAtom);
  float* s_rowsum = reinterpret_cast<float*>(bars + 1);      // [2 halves][128 rows]: the two threads of a row add up
  float* s_rowmax = s_rowsum + 2 * kQ;                       // [2 block parities][2 halves][128 rows]
  volatile int* stop = &bars->stop;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.x;        // heads vary fastest: the device starts the heaviest tiles of all heads first
  const int kvh = h / (Hq / Hkv);

  // zeros in both stages: a block's second page may not exist, and what the tensor core then
  // reads in its place (times a zero probability) must be finite
  for (int i = threadIdx.x; i < 4 * QB / 16; i += blockDim.x) reinterpret_cast<uint4*>(KV)[i] = make_uint4(0, 0, 0, 0);
  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    mbar_init(&bars->q_empty, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars->k_full[s], 1);
      mbar_init(&bars->k_empty[s], 1);
      mbar_init(&bars->v_full[s], 1);
      mbar_init(&bars->v_empty[s], 1);
      mbar_init(&bars->s_full[s], 1);
      mbar_init(&bars->s_empty[s], 8);
    }
    mbar_init(&bars->p_full, 8);
    mbar_init(&bars->p_free, 1);
    mbar_init(&bars->o_final, 1);
    mbar_init(&bars->o_read, 8);
    bars->stop = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem = bars->tmem_base;
  const unsigned tmem_o = tmem + 2 * kKeys;       // S buffers at columns 0 and 128, O at 256
  // Launched chained: the zero-fill, the barriers and the tensor-memory allocation above touch
  // nothing outside the SM and ran while the kernel before this one drained; queries, keys and
  // values (and the first write of `out`) come after the wait.
  chain_wait(block_table, positions, seg_row0, tiles);

  if (warp == 0 || warp == 10) {
    // ---- producers: warp 0 brings Q and the keys, warp 10 the values --------------------------------
    // Two threads, because the two rings turn at different times: a key stage is free as soon as
    // the scores of its block are done (long before that block's softmax), a value stage only after
    // the second product; one thread serving both in turn would hold the keys back.
    if (lane == 0) {
      const int kv = warp == 0 ? 0 : 1;
      int gb = 0, issued_stage[2] = {-1, -1};
      bool ok = true, q_pending = false;
      int gq = 0;
      const int per = kKeys / page_size;               // pages a block spans (at most 8)
      for (int which = 0; which < 2 && ok; ++which, ++gq) {
        const TileInfo t = tile_info(tiles, which, seg_row0, positions, window);
        if (t.seg < 0) break;
        const int* bt = block_table + (size_t)t.seg * bt_width;
        // the pages of a block: looked up one block ahead, so that the trip to the block table
        // passes while this thread waits for a free stage
        auto lookup = [&](int blk, int* page_of) {
          const int kb = t.kb_first + blk * kKeys;
          for (int pi = 0; pi < per; ++pi) {
            const int j0 = kb + pi * page_size;
            int page = -1;
            if (blk < t.n_blocks && j0 <= t.pos_last) {
              const int lp = j0 / page_size;
              page = lp < bt_width ? bt[lp] : -1;
              if (page >= num_pages) page = -1;
            }
            page_of[pi] = page;
          }
        };
        int page_now[8], page_next[8];
        lookup(0, page_next);
        if (kv == 0) {
          if (!mbar_wait(&bars->q_empty, (gq & 1) ^ 1, stop, 1, &g_fa_error)) { ok = false; break; }
          mbar_expect_tx(&bars->q_full, QB);
          for (int a = 0; a < ATOMS; ++a) tma_load_2d(Qs + a * kAtom, &map_q, h * D + 64 * a, t.row0, &bars->q_full);
          q_pending = true;
        }
        for (int blk = 0; blk < t.n_blocks; ++blk, ++gb) {
          const int s = gb & 1;
          int n_ok = 0;
          for (int pi = 0; pi < per; ++pi) { page_now[pi] = page_next[pi]; n_ok += page_now[pi] >= 0; }
          lookup(blk + 1, page_next);
          unsigned char* st = KV + (size_t)s * 2 * QB + kv * QB;
          void* full = kv ? &bars->v_full[s] : &bars->k_full[s];
          void* empty = kv ? &bars->v_empty[s] : &bars->k_empty[s];
          if (!mbar_wait(empty, ((gb >> 1) & 1) ^ 1, stop, 2, &g_fa_error)) { ok = false; break; }
          mbar_expect_tx(full, (unsigned)n_ok * page_size * D * 2);
          for (int pi = 0; pi < per; ++pi) {
            if (page_now[pi] < 0) continue;
            const int y = ((page_now[pi] * 2 + kv) * Hkv + kvh) * page_size;
            for (int a = 0; a < ATOMS; ++a)
              tma_load_2d(st + a * kAtom + pi * page_size * 128, &map_kv, 64 * a, y, full);
          }
          issued_stage[s] = gb;
        }
      }
      if (!ok) {
        // copies already asked for still land in this CTA's shared memory: wait for them
        if (q_pending)
          for (unsigned i = 0; i < (1u << 20); ++i)
            if (mbar_try(&bars->q_full, (gq - 1) & 1)) break;
        for (int s = 0; s < 2; ++s) {
          if (issued_stage[s] < 0) continue;
          void* full = kv ? &bars->v_full[s] : &bars->k_full[s];
          for (unsigned i = 0; i < (1u << 20); ++i)
            if (mbar_try(full, (issued_stage[s] >> 1) & 1)) break;
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer ---------------------------------------------------------------------------------
    if (lane == 0) {
      const unsigned idesc_qk = fa_idesc(kKeys, false), idesc_pv = fa_idesc(D, true);
      int gb = 0, gp = 0, gq = 0;
      bool ok = true;
      // O += P V of the block whose keys sit in stage (gp & 1); `first`: the first block of a tile
      auto issue_pv = [&](bool first) -> bool {
        if (!mbar_wait(&bars->v_full[gp & 1], (gp >> 1) & 1, stop, 4, &g_fa_error)) return false;
        if (!mbar_wait(&bars->p_full, gp & 1, stop, 5, &g_fa_error)) return false;
        if (first && gq > 0 && !mbar_wait(&bars->o_read, (gq - 1) & 1, stop, 6, &g_fa_error)) return false;
        tc_fence_after();
        const unsigned char* vst = KV + (size_t)(gp & 1) * 2 * QB + QB;
#pragma unroll
        for (int kk = 0; kk < kKeys / 16; ++kk) {
          const unsigned long long a = smem_desc(Ps + (kk >> 2) * kAtom) + 2 * (kk & 3);
          const unsigned long long b = smem_desc_mn(vst + kk * 16 * 128, kAtom);
          tc_mma(tmem_o, a, b, idesc_pv, (!first || kk > 0) ? 1u : 0u);
        }
        tc_commit(&bars->v_empty[gp & 1]);       // the values of this block are free ...
        tc_commit(&bars->p_free);                // ... and so are P and O, once these have run
        ++gp;
        return true;
      };
      for (int which = 0; which < 2 && ok; ++which, ++gq) {
        const TileInfo t = tile_info(tiles, which, seg_row0, positions, window);
        if (t.seg < 0) break;
        if (!mbar_wait(&bars->q_full, gq & 1, stop, 3, &g_fa_error)) { ok = false; break; }
        for (int blk = 0; blk < t.n_blocks && ok; ++blk, ++gb) {
          const int s = gb & 1;
          if (!mbar_wait(&bars->k_full[s], (gb >> 1) & 1, stop, 4, &g_fa_error)) { ok = false; break; }
          if (!mbar_wait(&bars->s_empty[s], ((gb >> 1) & 1) ^ 1, stop, 7, &g_fa_error)) { ok = false; break; }
          tc_fence_after();
          const unsigned char* kst = KV + (size_t)s * 2 * QB;
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const unsigned long long a = smem_desc(Qs + (kk >> 2) * kAtom) + 2 * (kk & 3);
            const unsigned long long b = smem_desc(kst + (kk >> 2) * kAtom) + 2 * (kk & 3);
            tc_mma(tmem + s * kKeys, a, b, idesc_qk, kk > 0 ? 1u : 0u);
          }
          tc_commit(&bars->s_full[s]);
          tc_commit(&bars->k_empty[s]);                           // the keys are free once the scores are done
          if (blk == t.n_blocks - 1) tc_commit(&bars->q_empty);   // the tile's last use of Q
          if (blk > 0 && !issue_pv(blk == 1)) { ok = false; break; }
        }
        if (!ok) break;
        if (!issue_pv(t.n_blocks == 1)) { ok = false; break; }
        tc_commit(&bars->o_final);
      }
    }
  } else {
    // ---- softmax, correction, epilogue ---------------------------------------------------------------
    // Eight warps: warp w may touch tensor-memory lanes 32 (w % 4) .. + 31, so warps w and w + 4
    // share 32 rows and split their columns in halves.  Two warps a scheduler instead of one hide
    // each other's latencies (tensor-memory loads, the exponential unit, instruction fetch).
    const int quad = warp & 3;                       // the 32 lanes (rows) this warp may touch
    const int half = (warp - 2) >> 2;                // which half of the columns
    const int r = quad * 32 + lane;
    const unsigned lane_addr = (unsigned)(quad * 32) << 16;
    const float sc2 = scale * kLog2e;
    constexpr int HK = kKeys / 2;                    // score columns of this thread
    constexpr int HD = D / 2;                        // output columns of this thread
    int gs = 0, gp = 0, gq = 0;
    bool ok = true;
    // the two threads of a row meet at a named barrier of their 64 (ids 1..4)
    auto pair_sync = [&]() { asm volatile("bar.sync %0, 64;" ::"r"(1 + quad) : "memory"); };
    for (int which = 0; which < 2 && ok; ++which, ++gq) {
      const TileInfo t = tile_info(tiles, which, seg_row0, positions, window);
      if (t.seg < 0) break;
      const bool row_ok = r < t.n_rows;
      const int p_r = t.pos_first + r;
      const int w_r = window > 0 ? max(0, p_r - window + 1) : 0;
      const bool row_sees = row_ok && p_r >= w_r;
      const unsigned j_span = row_sees ? (unsigned)(p_r - w_r) : 0u;
      float m_ref = 0.f, l_run = 0.f;      // l_run: this thread's half of the row sum
      bool have = false;                   // the row has seen a visible key
      for (int blk = 0; blk < t.n_blocks && ok; ++blk, ++gs, ++gp) {
        const int s = gs & 1;
        if (!mbar_wait(&bars->s_full[s], (gs >> 1) & 1, stop, 8, &g_fa_error)) { ok = false; break; }
        tc_fence_after();
        const int kb = t.kb_first + blk * kKeys;
        // every key of the block visible to every row of this warp: no mask to apply
        const bool all_visible = quad * 32 + 31 < t.n_rows && kb + kKeys - 1 <= t.pos_first + quad * 32 &&
                                 (window <= 0 || kb >= t.pos_first + quad * 32 + 31 - window + 1);
        // key j of this block (0..127) is visible to the row iff j - j_lo <= j_span (unsigned)
        const int j_lo = w_r - kb;
        // This thread's 64 scores, read once and kept in registers.
        unsigned u[HK];
        tc_ld32(tmem + lane_addr + s * kKeys + half * HK, u);
        tc_ld32(tmem + lane_addr + s * kKeys + half * HK + 32, u + 32);
        tc_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->s_empty[s]);           // the buffer may take the scores of block + 2
        float mx;
        {
          float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};     // four chains, not one
          if (all_visible) {
#pragma unroll
            for (int i = 0; i < HK; ++i) m4[i & 3] = fmaxf(m4[i & 3], __uint_as_float(u[i]));
          } else {
#pragma unroll
            for (int i = 0; i < HK; ++i) {
              const bool vis = row_sees && (unsigned)(half * HK + i - j_lo) <= j_span;
              u[i] = vis ? u[i] : 0xff800000u;                   // -inf: stays masked below
              m4[i & 3] = fmaxf(m4[i & 3], __uint_as_float(u[i]));
            }
          }
          mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
        }
        // the row's maximum: the larger of the two halves (slots alternate with the block's parity,
        // so a fast thread cannot overwrite what its partner has yet to read)
        float* slot = s_rowmax + (gs & 1) * 2 * kQ;
        slot[half * kQ + r] = mx;
        pair_sync();
        mx = fmaxf(mx, slot[(half ^ 1) * kQ + r]) * sc2;         // sc2 > 0: the maximum of the scaled scores
        // the reference maximum: set by the first block with a visible key, raised only when a
        // score passes it by 2^8 (both threads of a row decide alike)
        float alpha = 1.f;
        bool raise = false;
        if (!have) {                       // nothing visible so far (O's row and l are zero)
          have = mx != -INFINITY;
          m_ref = have ? mx : 0.f;
        } else if (mx > m_ref + kRaise) {
          raise = true;
          alpha = exp2f(m_ref - mx);
          m_ref = mx;
        }
        // P and O are free once the product of the block before has run
        if (gp > 0 && !mbar_wait(&bars->p_free, (gp - 1) & 1, stop, 9, &g_fa_error)) { ok = false; break; }
        if (__any_sync(0xffffffffu, raise)) {                   // the whole warp, each row by its own factor
          tc_fence_after();
#pragma unroll 1
          for (int c = 0; c < HD / 32; ++c) {
            unsigned o[32];
            tc_ld32(tmem_o + lane_addr + half * HD + 32 * c, o);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tc_st32(tmem_o + lane_addr + half * HD + 32 * c, o);
          }
          tc_wait_st();
          l_run *= alpha;
        }
        // P = 2^(s * scale * log2 e - m) as bfloat16 in the swizzled K-major image (this thread's
        // 64 keys are one swizzle atom of its row); the sum in float32.  A masked score is -inf
        // and gives 0.
        float sum = 0.f;
        unsigned char* prow = Ps + half * kAtom + r * 128;
#pragma unroll
        for (int q = 0; q < HK / 8; ++q) {
          float p[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) p[i] = ex2(fmaf(__uint_as_float(u[8 * q + i]), sc2, -m_ref));
          uint4 w;
          __nv_bfloat162 b0 = __floats2bfloat162_rn(p[0], p[1]), b1 = __floats2bfloat162_rn(p[2], p[3]);
          __nv_bfloat162 b2 = __floats2bfloat162_rn(p[4], p[5]), b3 = __floats2bfloat162_rn(p[6], p[7]);
          w.x = *reinterpret_cast<unsigned*>(&b0);
          w.y = *reinterpret_cast<unsigned*>(&b1);
          w.z = *reinterpret_cast<unsigned*>(&b2);
          w.w = *reinterpret_cast<unsigned*>(&b3);
          *reinterpret_cast<uint4*>(prow + ((q ^ (r & 7)) << 4)) = w;   // piece q: keys 8 q .. 8 q + 7 of the atom
          sum += ((p[0] + p[1]) + (p[2] + p[3])) + ((p[4] + p[5]) + (p[6] + p[7]));
        }
        l_run += sum;
        fence_async_smem();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->p_full);
      }
      if (!ok) break;
      // ---- the tile's rows: O / l ---------------------------------------------------------------------
      s_rowsum[half * kQ + r] = l_run;
      pair_sync();
      const float l_row = s_rowsum[r] + s_rowsum[kQ + r];        // same order in both threads
      pair_sync();                                               // both have read: the slots may be reused
      if (!mbar_wait(&bars->o_final, gq & 1, stop, 10, &g_fa_error)) { ok = false; break; }
      tc_fence_after();
      const float inv = l_row > 0.f ? 1.f / l_row : 0.f;
      __nv_bfloat16* dst = out + (size_t)(t.row0 + r) * Hq * D + (size_t)h * D + half * HD;
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        unsigned o[32];
        tc_ld32(tmem_o + lane_addr + half * HD + 32 * c, o);
        tc_wait_ld();
        if (row_ok) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 w;
            __nv_bfloat162 b0 = __floats2bfloat162_rn(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv);
            __nv_bfloat162 b1 = __floats2bfloat162_rn(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
            __nv_bfloat162 b2 = __floats2bfloat162_rn(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv);
            __nv_bfloat162 b3 = __floats2bfloat162_rn(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv);
            w.x = *reinterpret_cast<unsigned*>(&b0);
            w.y = *reinterpret_cast<unsigned*>(&b1);
            w.z = *reinterpret_cast<unsigned*>(&b2);
            w.w = *reinterpret_cast<unsigned*>(&b3);
            *reinterpret_cast<uint4*>(dst + 32 * c + i) = w;
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->o_read);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
  }
}

template <int D>
int launch_prefill_tc(const CUtensorMap& mq, const CUtensorMap& mkv, const int* block_table, int bt_width,
                      const int* positions, const int* seg_row0, const int* tiles, int n_tiles, void* out, int Hq,
                      int Hkv, int page_size, int num_pages, int window, float scale, cudaStream_t stream) {
  constexpr int QB = (D / 64) * kAtom;
  const size_t smem = 1024 + (size_t)5 * QB + 2 * kAtom + sizeof(FaBarriers) + 6 * kQ * sizeof(float);
  static bool set = false;
  if (!set) {
    cudaError_t e = cudaFuncSetAttribute(prefill_attention_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    NF_REQUIRE(e == cudaSuccess, "prefill attention: cannot have %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    set = true;
  }
  dim3 grid(Hq, n_tiles);
  launch_chained(prefill_attention_tc_kernel<D>, grid, dim3(kFaThreads), smem, stream, mq, mkv, block_table, bt_width,
                 positions, seg_row0, tiles, (__nv_bfloat16*)out, Hq, Hkv, page_size, num_pages, window, scale);
  return check_launch("prefill_attention_tc");
}

}  // namespace
}  // namespace nf

using namespace nf;

extern "C" int nf_prefill_attention_tc_tile_rows() { return kQ; }

// 1 if the tensor-core kernel takes these sizes.
extern "C" int nf_prefill_attention_tc_fits(int Hq, int Hkv, int D, int page_size, long long num_pages) {
  const bool page_ok = page_size == 16 || page_size == 32 || page_size == 64 || page_size == 128;
  return (D == 64 || D == 128) && page_ok && Hkv > 0 && Hq % Hkv == 0 &&
         num_pages * 2 * Hkv * page_size < (1ll << 31);
}

// bfloat16; head_dim 64 or 128; page size 16, 32, 64 or 128.  `tiles` is int32 [n_ctas, 2, 2]: for
// every CTA two tiles as (segment, first row), each at most 128 consecutive rows of one segment;
// the second may be (-1, -1).  qkv is [T, q_row_stride] with the queries in its first Hq * D
// columns; out is [T, Hq * D].
extern "C" int nf_prefill_attention_tc(const void* qkv, long long T, int q_row_stride, const void* pages,
                                       const int* block_table, int bt_width, const int* positions,
                                       const int* seg_row0, const int* tiles, int n_tiles, void* out, int Hq,
                                       int Hkv, int D, int page_size, int num_pages, int window, float scale,
                                       cudaStream_t stream) {
  if (n_tiles == 0) return 0;
  NF_REQUIRE(n_tiles > 0 && n_tiles <= 65535 && T > 0, "prefill attention: bad sizes tiles=%d T=%lld", n_tiles, T);
  NF_REQUIRE(nf_prefill_attention_tc_fits(Hq, Hkv, D, page_size, num_pages), "prefill attention: sizes the tensor-core kernel does not take (Hq=%d Hkv=%d D=%d page=%d)", Hq, Hkv, D, page_size);
  NF_REQUIRE(q_row_stride % 8 == 0 && (uintptr_t)qkv % 16 == 0 && (uintptr_t)pages % 16 == 0, "prefill attention: rows must be 16-byte aligned");
  CUtensorMap mq, mkv;
  if (int rc = make_map(&mq, qkv, T, (long long)Hq * D, kQ, q_row_stride)) return rc;
  if (int rc = make_map(&mkv, pages, (long long)num_pages * 2 * Hkv * page_size, D, page_size)) return rc;
  if (D == 64)
    return launch_prefill_tc<64>(mq, mkv, block_table, bt_width, positions, seg_row0, tiles, n_tiles, out, Hq, Hkv,
                                 page_size, num_pages, window, scale, stream);
  return launch_prefill_tc<128>(mq, mkv, block_table, bt_width, positions, seg_row0, tiles, n_tiles, out, Hq, Hkv,
                                page_size, num_pages, window, scale, stream);
}

// 0 if no tensor-core attention kernel has given up on a wait since the last call; else the code
// of the first wait that did (1-2 producer, 3-7 MMA issuer, 8-10 softmax).  Synchronises.
extern "C" int nf_prefill_attention_tc_status() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_fa_error, sizeof(int)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(g_fa_error, &zero, sizeof(int));
  return v;
}
