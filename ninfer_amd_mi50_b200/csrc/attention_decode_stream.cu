// Decode attention in bfloat16 as a persistent streaming kernel: the split-key decomposition
// of attention_decode.cu (one partial result per row, kv head and aligned block of 128 keys,
// merged in ascending order by `decode_attention_merge_kernel`) with the blocks dealt to warps
// that never stop fetching.
//
// Reference: ``decode_attention_kernel`` (src/ops/attention.hip:14-94): one block per query head
// walks all keys in tiles of 256 with the softmax bookkeeping on thread 0.  Same mathematics
// (scores * 1/sqrt(D), online softmax in float32, o = acc / l after the merge).
//
// Why a second form.  In attention_decode.cu a CTA lives for one block of 128 keys: it finds its
// page (two dependent reads), asks for 64 KB, waits, computes, writes, ends; while it computes or
// looks up, nothing of its own is in flight, and the device reaches about 60 % of its memory
// bandwidth.  Here one CTA per SM stays for the whole launch.  Each of its 8 warps is a worker of
// its own: it takes blocks c = w, w + W, ... of the flattened list (row, block, kv head), and
// moves the block's keys and values through a private ring of 16-key tiles in shared memory
// (``cp.async``, 16 bytes a lane, L1 bypassed).  A tile is refilled the moment it has been used,
// so a warp always has two or more tiles on their way while it multiplies a third, whatever the
// other warps do: no CTA-wide barrier in the loop, no wait on another thread beyond the warp.
//
// Mathematics of a tile, the usual flash form with the group's query heads as the 16 rows of
// ``mma.sync.m16n8k16``: S = Q K^T (two 8-key column blocks), online softmax per head in float32
// registers, P rounded to bfloat16 as the A operand of O += P V.  Keys and values sit in shared
// memory with a 16-byte XOR swizzle, so ``ldmatrix`` is conflict-free without padding.
//
// A block's partial result depends on the row's own position and window only (blocks are
// aligned to absolute key indices, tiles run in ascending order), so a row's output does not
// depend on what else is in the batch.
#define NF_CHAIN_CLASS 8
#include "common.cuh"
#include "decode_range.cuh"

namespace nf {

namespace {

constexpr int kBlockKeys = 128;       // keys per partial result (must equal attention_decode.cu's kSplit)
constexpr int kTile = 16;             // keys per ring stage
constexpr int kWorkers = 8;           // warps per CTA
constexpr int kMaxRows = 1024;        // rows one launch may have (their block counts live in shared memory)
constexpr int kRingBytes = 24 * 1024; // per warp

// A row whose position needs more key blocks than the caller's `nsplit` has its blocks beyond
// nsplit - 1 left out (nothing is written outside the workspace) and 1 + row recorded here;
// read and reset by nf_decode_attention_status.
__device__ int g_decode_range_error = 0;

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(unsigned dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr) : "memory");
}
__device__ __forceinline__ void ldsm_x4_trans(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr) : "memory");
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

// D: head size, 64 or 128.  G = Hq / Hkv <= 16 query heads share a kv head.
// ws_acc [T, Hq, nsplit, D], ws_ml [T, Hq, nsplit, 2] as in attention_decode.cu.
template <int D>
__global__ void __launch_bounds__(kWorkers * 32, 1)
decode_attention_stream_kernel(const __nv_bfloat16* __restrict__ qkv, int q_row_stride,
                               const __nv_bfloat16* __restrict__ pages, const int* __restrict__ block_table,
                               int bt_width, const int* __restrict__ positions, const int* __restrict__ row_seg,
                               float* __restrict__ ws_acc, float* __restrict__ ws_ml, int T, int Hq, int Hkv,
                               int page_size, int num_pages, int window, float scale, int nsplit,
                               const int* __restrict__ row_list) {
  constexpr int PIECES = D / 8;                    // 16-byte pieces of a key row
  constexpr int TILE_BYTES = kTile * D * 2;        // keys (or values) of one tile
  constexpr int STAGE_BYTES = 2 * TILE_BYTES;
  constexpr int NS = kRingBytes / STAGE_BYTES < 8 ? kRingBytes / STAGE_BYTES : 8;   // ring stages
  static_assert(NS >= 2, "ring too small for this head size");
  constexpr int TILES = kBlockKeys / kTile;        // tiles of a full block
  constexpr int COPIES = kTile * PIECES / 32;      // cp.async per lane for the keys of a tile
  extern __shared__ __align__(128) unsigned char smem_raw[];
  int* s_first = reinterpret_cast<int*>(smem_raw + (size_t)kWorkers * NS * STAGE_BYTES);   // [T] first block of row t
  int* s_cum = s_first + T;                                                               // [T + 1] blocks before row t
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tq = lane & 3;
  const int G = Hq / Hkv;
  // one CTA an SM with nearly all of its shared memory: the merge kernel's small CTAs fit beside
  // it and are then in place when the last partial result is written
  asm volatile("griddepcontrol.launch_dependents;");

  // ---- every CTA lists the rows' blocks: row t has blocks s_first[t] .. of its key range -------
  // Rows are counted by their place in this launch (0 .. T - 1: shared-memory lists, workspace);
  // `row_of` gives the row itself (queries, positions, segments).
  auto row_of = [&](int i) { return row_list ? row_list[i] : i; };
  for (int t = threadIdx.x; t < T; t += blockDim.x) {
    int pos = positions[row_of(t)], lo;
    if (decode_key_range(pos, lo, window, nsplit, kBlockKeys) && blockIdx.x == 0)
      atomicCAS(&g_decode_range_error, 0, 1 + t);  // the workspace has no slot for the row's last blocks
    s_first[t] = lo / kBlockKeys;
    s_cum[t + 1] = pos / kBlockKeys - lo / kBlockKeys + 1;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    s_cum[0] = 0;
    for (int t = 0; t < T; ++t) { const int n = s_cum[t + 1]; run += n; s_cum[t + 1] = run; }
  }
  __syncthreads();
  // The lists above need only the step's positions (and the row list), which the caller wrote
  // before the kernel that precedes this one began, like the segments and the block table.  What
  // that kernel writes is the queries and, in the pages, each row's keys and values at its own
  // (newest) position: the wait stands before the first tile that holds such a position and
  // before the first use of a query, and the ring is filled up to there meanwhile.
  const int total = s_cum[T] * Hkv;                // blocks of the launch: (row, block) major, kv head minor
  const int W = gridDim.x * kWorkers;
  const int wid = warp * gridDim.x + blockIdx.x;   // workers of one CTA are W / 8 apart: CTAs stay level

  const unsigned ring = smem_u32(smem_raw) + warp * (NS * STAGE_BYTES);
  const size_t head_stride = (size_t)page_size * D;
  const size_t page_stride = (size_t)2 * Hkv * head_stride;
  const size_t v_off = (size_t)Hkv * head_stride;

  // ---- the producer's view: which tile comes next ------------------------------------------------
  // A worker's tiles form one sequence over its blocks; the producer runs NS - 1 tiles ahead of
  // the consumer.  Producer state: block pc (in the flattened list), its row and key range, the
  // next tile index pt inside the block.
  int pc = wid, p_t = 0, p_kvh = 0, p_kbase = 0, p_kb = 0, p_ke = 0, p_tile = 0, p_tile_end = 0, p_new = 0;
  const int* p_bt = nullptr;
  auto producer_open = [&]() {           // set the producer's state for block pc (pc < total)
    const int rc = pc / Hkv;
    p_kvh = pc - rc * Hkv;
    int lo_t = 0, hi_t = T;              // the row whose block range holds rc: s_cum[t] <= rc < s_cum[t + 1]
    while (hi_t - lo_t > 1) {
      const int mid = (lo_t + hi_t) >> 1;
      if (s_cum[mid] <= rc) lo_t = mid; else hi_t = mid;
    }
    p_t = lo_t;
    const int p_row = row_of(p_t);
    int pos = positions[p_row], lo;
    p_new = pos;                         // the position whose keys and values the kernel before this one wrote
    decode_key_range(pos, lo, window, nsplit, kBlockKeys);
    const int split = s_first[p_t] + (rc - s_cum[p_t]);
    p_kbase = split * kBlockKeys;
    p_kb = max(lo, p_kbase);
    p_ke = min(pos + 1, p_kbase + kBlockKeys);
    p_tile = (p_kb - p_kbase) / kTile;
    p_tile_end = (p_ke - 1 - p_kbase) / kTile + 1;
    p_bt = block_table + (size_t)row_seg[p_row] * bt_width;
  };
  int issued = 0;                        // tiles asked for so far (ring position)
  auto produce = [&]() {                 // ask for the next tile, or commit an empty group at the end
    if (pc < total) {
      const int j0 = p_kbase + p_tile * kTile;             // first key of the tile; inside one page
      const int lp = j0 / page_size;
      const int page = lp < bt_width ? p_bt[lp] : -1;
      const unsigned dst = ring + (issued % NS) * STAGE_BYTES;
      const bool page_ok = page >= 0 && page < num_pages;
      const __nv_bfloat16* src = pages + (size_t)(page_ok ? page : 0) * page_stride + (size_t)p_kvh * head_stride +
                                 (size_t)(j0 - lp * page_size) * D;
#pragma unroll
      for (int i = 0; i < COPIES; ++i) {
        const int p = lane + 32 * i;                       // piece p of the tile: row p / PIECES
        const int row = p / PIECES, c = p % PIECES;
        const unsigned d = dst + row * (D * 2) + ((c ^ (row & 7)) << 4);
        const int key = j0 + row;
        if (page_ok && key >= p_kb && key < p_ke) {
          cp_async16(d, src + (size_t)p * 8);
          cp_async16(d + TILE_BYTES, src + v_off + (size_t)p * 8);
        } else {                                           // outside the row's keys: zeros, never garbage
          asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(d), "r"(0) : "memory");
          asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(d + TILE_BYTES), "r"(0) : "memory");
        }
      }
      ++issued;
      if (++p_tile == p_tile_end) {
        pc += W;
        if (pc < total) producer_open();
      }
    }
    cp_commit();
  };

  if (pc < total) producer_open();
  int filled = 0;
#pragma unroll 1
  for (; filled < NS - 1; ++filled) {
    const int j0 = p_kbase + p_tile * kTile;
    if (pc < total && p_new >= j0 && p_new < j0 + kTile) break;      // this tile holds a newest position
    produce();
  }
  chain_wait(qkv, pages);
#pragma unroll 1
  for (; filled < NS - 1; ++filled) produce();

  // ---- the consumer ---------------------------------------------------------------------------------
  int used = 0;                          // tiles multiplied so far
  for (int c = wid; c < total; c += W) {
    const int rc = c / Hkv, kvh = c - rc * Hkv;
    int lo_t = 0, hi_t = T;
    while (hi_t - lo_t > 1) {
      const int mid = (lo_t + hi_t) >> 1;
      if (s_cum[mid] <= rc) lo_t = mid; else hi_t = mid;
    }
    const int t = lo_t, q_row = row_of(lo_t);
    int pos = positions[q_row], lo;
    decode_key_range(pos, lo, window, nsplit, kBlockKeys);
    const int split = s_first[t] + (rc - s_cum[t]);
    const int k_base = split * kBlockKeys;
    const int k_begin = max(lo, k_base), k_end = min(pos + 1, k_base + kBlockKeys);
    const int tile0 = (k_begin - k_base) / kTile, tile1 = (k_end - 1 - k_base) / kTile + 1;

    // query heads of the group as the rows of the A operand: row g and row g + 8
    unsigned qa[D / 16][4];
    {
      const __nv_bfloat16* q0 = qkv + (size_t)q_row * q_row_stride + (size_t)(kvh * G + g) * D;
      const __nv_bfloat16* q1 = q0 + 8 * D;
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        qa[kk][0] = g < G ? *reinterpret_cast<const unsigned*>(q0 + kk * 16 + 2 * tq) : 0u;
        qa[kk][1] = g + 8 < G ? *reinterpret_cast<const unsigned*>(q1 + kk * 16 + 2 * tq) : 0u;
        qa[kk][2] = g < G ? *reinterpret_cast<const unsigned*>(q0 + kk * 16 + 2 * tq + 8) : 0u;
        qa[kk][3] = g + 8 < G ? *reinterpret_cast<const unsigned*>(q1 + kk * 16 + 2 * tq + 8) : 0u;
      }
    }
    float o[D / 8][4];
#pragma unroll
    for (int db = 0; db < D / 8; ++db)
#pragma unroll
      for (int i = 0; i < 4; ++i) o[db][i] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;      // rows g and g + 8; l: this lane's share

    for (int tile = tile0; tile < tile1; ++tile, ++used) {
      produce();                         // tile used + NS - 1 (its stage was released at the end of the last turn)
      cp_wait<NS - 1>();                 // this lane's pieces of tile `used` have landed
      __syncwarp();                      // ... and so have the other lanes'
      const unsigned ks = ring + (used % NS) * STAGE_BYTES, vs = ks + TILE_BYTES;
      // S = Q K^T: columns = the tile's 16 keys in two blocks of 8
      float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      {
        const int row = (lane & 7) + ((lane >> 4) & 1) * 8;
        const int half = (lane >> 3) & 1;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          unsigned b0, b1, b2, b3;
          ldsm_x4(b0, b1, b2, b3, ks + row * (D * 2) + (((kk * 2 + half) ^ (row & 7)) << 4));
          mma16816(s[0], qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], b0, b1);
          mma16816(s[1], qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], b2, b3);
        }
      }
      // s[nb] = {(head g, key 8 nb + 2 tq), (g, +1), (head g + 8, key 8 nb + 2 tq), (g + 8, +1)}
      const int key0 = k_base + tile * kTile;
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int nb = 0; nb < 2; ++nb)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int key = key0 + nb * 8 + 2 * tq + (i & 1);
          const float v = (key >= k_begin && key < k_end) ? s[nb][i] * scale : -INFINITY;
          s[nb][i] = v;
          if (i < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
        }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      // every tile of a block holds at least one key of the row, so the maxima are finite
      const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
      const float a0 = expf(m0 - n0), a1 = expf(m1 - n1);          // exp(-inf) = 0 on the first tile
      m0 = n0;
      m1 = n1;
      float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
      for (int nb = 0; nb < 2; ++nb) {
        s[nb][0] = expf(s[nb][0] - n0);
        s[nb][1] = expf(s[nb][1] - n0);
        s[nb][2] = expf(s[nb][2] - n1);
        s[nb][3] = expf(s[nb][3] - n1);
        ps0 += s[nb][0] + s[nb][1];
        ps1 += s[nb][2] + s[nb][3];
      }
      l0 = l0 * a0 + ps0;
      l1 = l1 * a1 + ps1;
      const unsigned pa0 = pack_bf16(s[0][0], s[0][1]), pa1 = pack_bf16(s[0][2], s[0][3]);
      const unsigned pa2 = pack_bf16(s[1][0], s[1][1]), pa3 = pack_bf16(s[1][2], s[1][3]);
      // O = O * alpha + P V: columns = head dims in blocks of 8, two blocks per ldmatrix
      {
        const int row = (lane & 7) + ((lane >> 3) & 1) * 8;
        const int half = (lane >> 4) & 1;
#pragma unroll
        for (int db = 0; db < D / 8; db += 2) {
          unsigned b0, b1, b2, b3;
          ldsm_x4_trans(b0, b1, b2, b3, vs + row * (D * 2) + (((db + half) ^ (row & 7)) << 4));
          o[db][0] *= a0; o[db][1] *= a0; o[db][2] *= a1; o[db][3] *= a1;
          o[db + 1][0] *= a0; o[db + 1][1] *= a0; o[db + 1][2] *= a1; o[db + 1][3] *= a1;
          mma16816(o[db], pa0, pa1, pa2, pa3, b0, b1);
          mma16816(o[db + 1], pa0, pa1, pa2, pa3, b2, b3);
        }
      }
      __syncwarp();                      // the stage may be refilled once every lane has read it
    }

    // ---- the block's partial result ------------------------------------------------------------------
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int h = g + 8 * r;
      if (h < G) {
        const int hq = kvh * G + h;
        float* acc = ws_acc + (((size_t)t * Hq + hq) * nsplit + split) * D;
#pragma unroll
        for (int db = 0; db < D / 8; ++db)
          *reinterpret_cast<float2*>(acc + db * 8 + 2 * tq) = make_float2(o[db][2 * r], o[db][2 * r + 1]);
        if (tq == 0) {
          float* mlp = ws_ml + (((size_t)t * Hq + hq) * nsplit + split) * 2;
          mlp[0] = r ? m1 : m0;
          mlp[1] = r ? l1 : l0;
        }
      }
    }
  }
  cp_wait<0>();
}

template <int D>
int launch_stream(const void* qkv, int q_row_stride, const void* pages, const int* block_table, int bt_width,
                  const int* positions, const int* row_seg, float* ws_acc, float* ws_ml, int T, int Hq, int Hkv,
                  int page_size, int num_pages, int window, float scale, int nsplit, const int* row_list,
                  cudaStream_t stream) {
  constexpr int STAGE_BYTES = 2 * kTile * D * 2;
  constexpr int NS = kRingBytes / STAGE_BYTES < 8 ? kRingBytes / STAGE_BYTES : 8;
  const size_t smem = (size_t)kWorkers * NS * STAGE_BYTES + (size_t)(2 * T + 1) * sizeof(int);
  static bool set = false;
  if (!set) {
    const size_t most = (size_t)kWorkers * NS * STAGE_BYTES + (size_t)(2 * kMaxRows + 1) * sizeof(int);
    cudaError_t e = cudaFuncSetAttribute(decode_attention_stream_kernel<D>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)most);
    NF_REQUIRE(e == cudaSuccess, "decode attention: cannot have %zu bytes of shared memory: %s", most, cudaGetErrorString(e));
    set = true;
  }
  static int n_sm = 0;
  if (!n_sm) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
    if (n_sm <= 0) n_sm = 1;
  }
  // one CTA per SM, fewer only if there cannot be a block for each (rows x kv heads x blocks of
  // the longest row); workers are numbered CTA-fastest, so few blocks spread over all SMs
  const long long most_blocks = (long long)T * Hkv * nsplit;
  const int grid = (int)(most_blocks < n_sm ? most_blocks : n_sm);
  launch_chained(decode_attention_stream_kernel<D>, dim3(grid), dim3(kWorkers * 32), smem, stream,
                 (const __nv_bfloat16*)qkv, q_row_stride, (const __nv_bfloat16*)pages, block_table, bt_width,
                 positions, row_seg, ws_acc, ws_ml, T, Hq, Hkv, page_size, num_pages, window, scale, nsplit, row_list);
  return check_launch("decode_attention_stream");
}

}  // namespace

// 0, or 1 + the first row whose position lay beyond the key blocks that the call allowed for since
// the last call of this function (synchronises the device).
int decode_attention_stream_status() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_decode_range_error, sizeof(int)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(g_decode_range_error, &zero, sizeof(int));
  return v;
}

// 1 if the streaming kernel takes these sizes (the caller then runs the merge kernel after it).
int decode_attention_stream_fits(int T, int Hq, int Hkv, int D, int page_size) {
  return (D == 64 || D == 128) && Hq / Hkv <= 16 && page_size % kTile == 0 && T <= kMaxRows;
}

int decode_attention_stream(const void* qkv, int q_row_stride, const void* pages, const int* block_table,
                            int bt_width, const int* positions, const int* row_seg, float* ws_acc, float* ws_ml,
                            int T, int Hq, int Hkv, int D, int page_size, int num_pages, int window, float scale,
                            int nsplit, const int* row_list, cudaStream_t stream) {
  if (D == 64)
    return launch_stream<64>(qkv, q_row_stride, pages, block_table, bt_width, positions, row_seg, ws_acc, ws_ml, T,
                             Hq, Hkv, page_size, num_pages, window, scale, nsplit, row_list, stream);
  return launch_stream<128>(qkv, q_row_stride, pages, block_table, bt_width, positions, row_seg, ws_acc, ws_ml, T,
                            Hq, Hkv, page_size, num_pages, window, scale, nsplit, row_list, stream);
}

}  // namespace nf
