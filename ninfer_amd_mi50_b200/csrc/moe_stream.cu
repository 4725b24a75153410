// The routed experts of a decode step in one persistent launch: both products of every
// selected expert, streamed through one ring of shared memory that never runs dry.
//
// Reference counterpart: the per-expert loop of the MoE branch (src/models/model.hip:355-427),
// which launches a fused gate/up GEMV and a down GEMV for each selected expert of one token.
// A decode batch selects a few dozen experts, each with one to a handful of rows; the time of
// the step is the time to read their weights once.  Two launches of a weight-streaming kernel
// (skinny_gemm.cu) leave the memory idle at their start, between them and at their end, and
// their CTAs hold few bytes in flight; this kernel instead keeps one CTA on every SM for the
// whole MoE branch:
//
//   * a producer thread walks the work items - (expert, 16*Q features) of the gate/up product,
//     then of the down product - and copies their weights, block after block (16 Q rows x 64 k,
//     contiguous in the packed tile layout), into a ring of shared memory with bulk copies
//     (`cp.async.bulk`, completion on an mbarrier); it runs ahead of the consumers by the whole
//     ring, across item and product boundaries, so every SM always has about 100 KB in flight;
//   * eight consumer warps read the blocks with `ldmatrix` and multiply with
//     `mma.sync.m16n8k16` (float32 sums) against up to eight rows of X in shared memory; SwiGLU
//     in the epilogue.  An expert with more than eight rows in the step is served as several
//     row groups of eight (its weights then come from L2 the second time);
//   * a loader thread brings each item's rows of X in with bulk copies, one item ahead of the
//     consumers (two buffers): the hidden rows of the group's tokens for the first product, the
//     group's activation rows for the second.  The second product needs every feature of those:
//     the first product counts finished items per row group in global memory, and the loader
//     waits (bounded) for the count;
//   * items are handed out by a ticket counter, so the SMs stay balanced whatever the sizes of
//     the two products.  Tickets are handed out in order and first-product items never wait, so
//     the wait for activations cannot deadlock as long as the grid's CTAs run.
//
// Two optional parts in front of that (see `nf_moe_stream`):
//
//   * the routing: the consumer warps of every CTA first compute router logits (a unit is 8
//     router rows x 1 token, taken by ticket), the CTA whose unit is counted last selects for
//     every token, builds the plan in shared memory and publishes the routed row groups; the
//     producers wait (bounded) for that before their first routed item;
//   * a shared expert, cut into chunks of the experts' width and packed like further experts:
//     its row groups stand first in the table and need no plan, so their weights stream while
//     the routing is still being computed.
//
// The sums of a row are formed in an order that depends on the sizes and on Q only (k tiles in
// order, k groups added in order), never on the batch or on which CTA took the item.  Every
// wait is bounded; the first to give up records a code and the CTA leaves.
#define NF_CHAIN_CLASS 0x20
#include "router_device.cuh"
#include "tcgen05.cuh"

namespace nf {

constexpr int kMsConsumers = 8;                          // consumer warps
constexpr int kMsThreads = 32 * (kMsConsumers + 2);      // + the weight producer's warp + the row loader's
constexpr int kMsMaxStages = 32;
constexpr int kMsSlotBytes = 16 * 1024;                  // a stage: 128 weight rows x 64 k, or 64 x 128, or 32 x 256
constexpr int kMsMinStages = 4;
constexpr int kMsMaxGroups = 512;                        // row groups (an expert's rows, eight at a time) of one step
constexpr int kMsMaxPairs = 1024;                        // rows of X of one step: (token, expert) pairs + the shared expert's
constexpr int kMsRows = 8;                               // rows of a group
constexpr int kMsFifo = 64;                              // item ids between producer, loader and consumers
constexpr unsigned kMsCountPolls = 1u << 20;             // polls of a group's counter (about a second)
// `work`: 0 the item ticket, 1 CTAs that have finished, 2 the routing's unit ticket, 3 its units done,
// 4 "the routed row groups are written"; then the row groups' counters; then, written by the
// routing of a launch and read by its producers, the routed row groups (their number, expert,
// first row and rows of each) and the token of every pair
constexpr int kMsWork = 8;
constexpr int kMsTable = kMsWork + kMsMaxGroups;     // n, expert[], row_begin[], rows[], token[]
constexpr int kMsWorkInts = kMsTable + 1 + 3 * kMsMaxGroups + kMsMaxPairs;

// 1-3 ring waits, 4 the wait for a group's activations, 5-7 a plan that does not fit, 8 the
// consumers' barrier, 9-11 the loader's waits, 12 the consumers' wait for an item's rows, 14 the wait for the router's logits
__device__ int g_moe_stream_error = 0;
__device__ __align__(16) unsigned char g_ms_zeros[128];   // source of the zeros behind a row's last k

struct MsHeader {
  unsigned long long full[kMsMaxStages], empty[kMsMaxStages];
  unsigned long long meet;                 // the consumer warps' own barrier
  unsigned long long xfull[2], xempty[2];  // row buffers: filled by the loader, released by the consumers
  int fifo[kMsFifo];
  int stop, n_routed, published, loaded;   // routed row groups; items the producer has named / the loader has read
  int expert[kMsMaxGroups], row_begin[kMsMaxGroups], rows[kMsMaxGroups];
  int order[kMsMaxPairs];                  // sorted pair -> token
};

struct MsArgs {
  const __nv_bfloat16* X;      // [T, H] hidden rows
  const __nv_bfloat16* W13;    // packed [E][ceil(I/128)][ceil(H/64)][256][64]
  const __nv_bfloat16* W2;     // packed [E][ceil(H/128)][ceil(I/64)][128][64]
  __nv_bfloat16* act;          // [M, I] sorted pairs
  __nv_bfloat16* Y;            // [M, H] sorted pairs
  const int* offsets;          // [E + 1]
  const int* order;            // [M] sorted pair -> pair index (token * k + slot)
  const int* active;           // [n_mapped] experts with rows, ascending, -1 padded
  int* work;                   // [kMsWork + kMsMaxGroups]: counters (see kMsWork) and items done per row group; all zero between launches
  // routing inside the launch (Wr != null): offsets, order and active are then written here too
  const float* Wr;             // [E + extra, H] float32 router rows, then the rows whose raw logits are handed back
  float* logits;               // [T, E + extra] scratch
  int* topk_idx;               // [T, k]
  float* topk_w;               // [T, k]
  float* extra_out;            // [T, extra] or null
  int* inv;                    // [M] pair -> sorted position
  int extra, norm_topk;
  // a shared expert inside the launch (n_shared > 0, with routing only): its intermediate features in
  // n_shared chunks of I, packed like n_shared further experts; chunk c takes rows M + c T .. of act and Y
  const __nv_bfloat16* Ws13;   // packed [n_shared][...] like W13
  const __nv_bfloat16* Ws2;    // packed [n_shared][...] like W2
  long long gss13, gss2;
  float* cw;                   // [T, k + n_shared] weights of the k experts, then sigmoid(gate) (or 1) for every chunk
  int* cinv;                   // [T, k + n_shared] rows of Y that belong to them
  int n_shared;
  long long gs13, gs2;         // group strides in elements
  int ldx, M, T, H, I, E, k, n_mapped;
  int b_stride;                // bytes between rows of X (hidden rows or activations) in shared memory
  int red_bytes, scratch_bytes, smem_bytes;   // the k groups' meeting place; the routing's tables; all of the launch's dynamic shared memory
};

__device__ __forceinline__ void ldsm4(unsigned addr, unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm2(unsigned addr, unsigned& r0, unsigned& r1) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ void ms_mma(float* c, unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ int ld_acquire(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int add_acq_rel(int* p, int v) {
  int old;
  asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
  return old;
}
__device__ __forceinline__ void add_release(int* p, int v) {
  asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// what the kernel before wrote is read from L2, never through a cache that may hold an older line
__device__ __forceinline__ uint4 ld_l2(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ld_l2_int(const int* p) {
  int v;
  asm volatile("ld.global.cg.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// bounded spin on an int in shared memory until it exceeds `than`
__device__ __forceinline__ bool spin_above(volatile int* v, int than, volatile int* stop, int code) {
  for (unsigned i = 0; i < kPollLimit; ++i) {
    if (*v > than) return true;
    if ((i & 255u) == 255u && *stop) return false;
    __nanosleep(32);
  }
  *stop = 1;
  atomicCAS(&g_moe_stream_error, 0, code);
  return false;
}

// A position in the ring: slot and the parity of its current use.
struct MsRing {
  int s, parity, stages;
  __device__ __forceinline__ void next() {
    if (++s == stages) { s = 0; parity ^= 1; }
  }
};

// An item id -> (product, row group, sub-tile of 16 Q features).  Items in ticket order: the
// first product of the shared expert's ns row groups (they need no plan), of the nr routed ones,
// then the second product of the shared and of the routed ones.  n1, n2: items a group.
struct MsItem {
  int second, a, sub;
};
__device__ __forceinline__ MsItem ms_decode(int id, int ns, int nr, int n1, int n2) {
  MsItem it;
  const int first = (ns + nr) * n1;
  it.second = id >= first;
  const int r = it.second ? id - first : id;
  const int per = it.second ? n2 : n1;
  it.a = r / per;                  // shared groups come first in the table as well
  it.sub = r - it.a * per;
  return it;
}

// The k loop of one item for one consumer warp.  Q: the item has 16 Q weight rows, and a stage
// holds them for G = 8 / Q consecutive k tiles (block g of the stage: k tile j G + g); warp
// (row group rg, k group kg) takes block kg.  SECOND: the down product, one set of sums; else
// stages alternate between the gate rows and the up rows of the same k tiles, two sets.
// The item's first stage has been waited for.  False if a wait gave up.
template <int Q, bool SECOND>
__device__ __forceinline__ bool ms_k_loop(MsHeader* hd, unsigned char* ring, MsRing& at, int kt, int kg, int a_row,
                                          int a_hi, unsigned b_lane, float (&acc)[2][4]) {
  constexpr int G = kMsConsumers / Q;
  constexpr int BLOCK_BYTES = Q * 2048;
  volatile int* stop = &hd->stop;
  const int lane = threadIdx.x & 31;
  bool first = true;
  for (int t0 = 0; t0 < kt; t0 += G) {
#pragma unroll
    for (int half = 0; half < (SECOND ? 1 : 2); ++half) {
      if (!first && !mbar_wait(&hd->full[at.s], at.parity, stop, 3, &g_moe_stream_error)) return false;
      first = false;
      if (t0 + kg < kt) {
        const unsigned block = smem_u32(ring + (size_t)at.s * kMsSlotBytes) + kg * BLOCK_BYTES;
        const unsigned b_addr = b_lane + (unsigned)(t0 + kg) * 128;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          unsigned a0, a1, a2, a3, b0, b1;
          ldsm4(block + a_row * 128 + (((2 * ks + a_hi) ^ (a_row & 7)) << 4), a0, a1, a2, a3);
          ldsm2(b_addr + ks * 32, b0, b1);
          ms_mma(acc[half], a0, a1, a2, a3, b0, b1);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&hd->empty[at.s]);
      at.next();
    }
  }
  return true;
}

__device__ __forceinline__ void consumers_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kMsConsumers * 32) : "memory"); }

// The routing, by the consumer warps of every CTA before they turn to the products: logits by
// whoever takes a unit (8 router rows x 1 token, a warp a row, the sums in `lane_dot`'s order as
// in the router's own kernels); the CTA whose unit is counted last selects for every token,
// builds the plan and writes both out, then raises the flag that the producers wait for.
// `scratch`: x as float32, then the selection's and the plan's tables.
__device__ __forceinline__ void ms_route(const MsArgs& p, float* scratch, int* s_unit, int* s_last, int warp, int lane) {
  const int tid = threadIdx.x;                    // consumer threads: 0 .. 255
  const int rows = p.E + p.extra, nblk = (rows + 7) >> 3, n_units = nblk * p.T, n = p.M;
  float* xf = scratch;
  // The first unit needs no ticket; they go to the CTAs from the end of the grid, the first items
  // of the shared expert to those from its start: a CTA then rarely has both.
  int unit = (int)gridDim.x - 1 - (int)blockIdx.x;
  while (unit < n_units) {
    const int t = unit / nblk, e = (unit - t * nblk) * 8 + warp;
    for (int i = tid; i < (p.H >> 3); i += kMsConsumers * 32) {
      const uint4 v = ld_l2(p.X + (size_t)t * p.ldx + i * 8);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        xf[i * 8 + 2 * j] = f.x;
        xf[i * 8 + 2 * j + 1] = f.y;
      }
    }
    consumers_sync();
    if (e < rows) {
      const float v = warp_sum(lane_dot(xf, p.Wr + (size_t)e * p.H, p.H, lane));
      if (lane == 0) p.logits[(size_t)t * rows + e] = v;
    }
    consumers_sync();
    if (tid == 0) {
      // The barrier before this orders the warps' stores of the unit's logits before the count
      // (release), and for the CTA that counts last, the barrier after it orders every unit's
      // logits before its reads (acquire): one thread's atomic does for the CTA what a grid-wide
      // barrier's does.
      *s_unit = n_units > (int)gridDim.x ? (int)gridDim.x + atomicAdd(p.work + 2, 1) : n_units;
      *s_last = add_acq_rel(p.work + 3, 1) == n_units - 1;
    }
    consumers_sync();
    if (*s_last) {
      // everything in shared memory first: what the producers wait for (the routed row groups and
      // the pairs' tokens) goes out before what only the kernels after this launch read
      float* lg = xf;                                                                  // [8 warps][E]
      float* sw = lg + kMsConsumers * p.E;                                             // [n] weight of each pair
      float* sext = sw + n;                                                            // [T, extra] raw logits of the further rows
      int* counts = reinterpret_cast<int*>(sext + p.T * p.extra);                      // [E + 1] rows an expert, then offsets
      unsigned short* chosen = reinterpret_cast<unsigned short*>(counts + p.E + 1);    // [n] expert of each pair
      unsigned short* rank = chosen + n;                                               // [n] its rank inside the expert
      int* table = p.work + kMsTable;
      for (int tt = warp; tt < p.T; tt += kMsConsumers)
        select_token(p.logits + (size_t)tt * rows, 1, lg + warp * p.E, tt, p.E, p.extra, p.k, p.norm_topk, nullptr,
                     sw, p.extra > 0 ? sext : nullptr, lane, chosen);
      consumers_sync();
      // stable counting sort of the pairs by expert
      for (int e2 = warp; e2 < p.E; e2 += kMsConsumers) {
        int running = 0;
        for (int base = 0; base < n; base += 32) {
          const int i = base + lane;
          const bool mine = i < n && (int)chosen[i] == e2;
          const unsigned bits = __ballot_sync(0xffffffffu, mine);
          if (mine) rank[i] = (unsigned short)(running + __popc(bits & ((1u << lane) - 1u)));
          running += __popc(bits);
        }
        if (lane == 0) counts[e2] = running;
      }
      consumers_sync();
      if (warp == 0) {
        // 32 experts a round: offsets (exclusive prefix of the counts), the experts that have pairs,
        // and their rows eight at a time
        int run = 0, na = 0, ng = 0;
        for (int base = 0; base <= p.E; base += 32) {
          const int e2 = base + lane;
          const int c = e2 < p.E ? counts[e2] : 0;
          int incl = c;
#pragma unroll
          for (int o = 1; o < 32; o <<= 1) {
            const int up = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += up;
          }
          const int off = run + incl - c;
          __syncwarp();
          if (e2 <= p.E) counts[e2] = off;
          run += __shfl_sync(0xffffffffu, incl, 31);
          const int gcount = (c + kMsRows - 1) / kMsRows;
          int gi = gcount;
#pragma unroll
          for (int o = 1; o < 32; o <<= 1) {
            const int up = __shfl_up_sync(0xffffffffu, gi, o);
            if (lane >= o) gi += up;
          }
          const int first = ng + gi - gcount;
          for (int j = 0; j < gcount; ++j)
            if (first + j < kMsMaxGroups) {
              table[1 + first + j] = e2;
              table[1 + kMsMaxGroups + first + j] = off + j * kMsRows;
              table[1 + 2 * kMsMaxGroups + first + j] = min(kMsRows, c - j * kMsRows);
            }
          ng += __shfl_sync(0xffffffffu, gi, 31);
          // (for the kernels after this launch)
          if (e2 <= p.E) const_cast<int*>(p.offsets)[e2] = off;
          const unsigned bits = __ballot_sync(0xffffffffu, c > 0);
          const int at = na + __popc(bits & ((1u << lane) - 1u));
          if (c > 0 && at < p.n_mapped) const_cast<int*>(p.active)[at] = e2;
          na += __popc(bits);
        }
        for (int i = min(na, p.n_mapped) + lane; i < p.n_mapped; i += 32) const_cast<int*>(p.active)[i] = -1;
        if (lane == 0) table[0] = min(ng, kMsMaxGroups);
      }
      consumers_sync();
      for (int i = tid; i < n; i += kMsConsumers * 32) {
        const int pos = counts[chosen[i]] + rank[i];
        if (pos < kMsMaxPairs) table[1 + 3 * kMsMaxGroups + pos] = i / p.k;
        rank[i] = (unsigned short)pos;                 // (n <= 1024: a position fits)
      }
      consumers_sync();
      if (tid == 0) add_release(p.work + 4, 1);          // (after the barrier: it covers every thread's stores)
      // ---- the producers are on their way; now what the kernels after this launch read ----------------
      const int kk = p.k + p.n_shared;
      for (int i = tid; i < n; i += kMsConsumers * 32) {
        const int pos = rank[i];
        p.inv[i] = pos;
        const_cast<int*>(p.order)[pos] = i;
        p.topk_idx[i] = chosen[i];
        p.topk_w[i] = sw[i];
        if (p.cinv) {
          const int t = i / p.k, j = i - t * p.k;
          p.cinv[t * kk + j] = pos;
          p.cw[t * kk + j] = sw[i];
        }
      }
      if (p.extra_out)
        for (int i = tid; i < p.T * p.extra; i += kMsConsumers * 32) p.extra_out[i] = sext[i];
      if (p.cinv)
        for (int i = tid; i < p.T * p.n_shared; i += kMsConsumers * 32) {
          const int t = i / p.n_shared, c = i - t * p.n_shared;
          p.cinv[t * kk + p.k + c] = p.M + c * p.T + t;
          p.cw[t * kk + p.k + c] = p.extra > 0 ? 1.f / (1.f + expf(-sext[(size_t)t * p.extra])) : 1.f;
        }
    }
    unit = *s_unit;
  }
}

// Q: an item is 16 Q features (2, 4 or 8 sixteen-row groups); the 8 consumer warps are Q row
// groups x 8 / Q k groups.  (At most 102 registers a thread, so that kernels of another stream
// still find room on the SM.)
template <int Q>
__global__ void __launch_bounds__(kMsThreads, 2) moe_stream_kernel(const MsArgs p) {
  extern __shared__ unsigned char ms_smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)ms_smem_raw + 1023) & ~(uintptr_t)1023);
  static_assert(Q == 2 || Q == 4 || Q == 8, "16 Q features an item");
  constexpr int G = kMsConsumers / Q;                  // k groups = k tiles a stage
  constexpr int BLOCK_BYTES = Q * 2048;
  constexpr int HEADER_BYTES = (sizeof(MsHeader) + 1023) & ~1023;
  MsHeader* hd = reinterpret_cast<MsHeader*>(smem);
  float* red = reinterpret_cast<float*>(smem + HEADER_BYTES);
  float* scratch = reinterpret_cast<float*>(smem + HEADER_BYTES + p.red_bytes);
  unsigned char* xs = smem + HEADER_BYTES + p.red_bytes + p.scratch_bytes;     // [buffers][8 rows][b_stride], then the ring
  unsigned char* smem_end = ms_smem_raw + p.smem_bytes;
  volatile int* stop = &hd->stop;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __shared__ int s_last, s_unit, s_last_unit;
  const int kt1 = (p.H + 63) >> 6, kt2 = (p.I + 63) >> 6;               // k tiles of the two products
  const int n1 = (p.I + 16 * Q - 1) / (16 * Q), n2 = (p.H + 16 * Q - 1) / (16 * Q);     // items a row group
  const int target = n1 * kMsConsumers;                                 // counts that say "this group's activations are complete"
  const int spt = (p.T + kMsRows - 1) / kMsRows;                        // row groups of one chunk of the shared expert
  const int ns = p.n_shared * spt;                                      // the shared expert's row groups: first in the table
  const int items_s1 = ns * n1;                                         // items that need no plan

  // ---- set-up that needs nothing from the kernel before ------------------------------------------
  if (threadIdx.x == 0) {
    for (int s = 0; s < kMsMaxStages; ++s) { mbar_init(&hd->full[s], 1); mbar_init(&hd->empty[s], kMsConsumers); }
    mbar_init(&hd->meet, kMsConsumers);
    for (int b = 0; b < 2; ++b) { mbar_init(&hd->xfull[b], 1); mbar_init(&hd->xempty[b], kMsConsumers); }
    hd->stop = 0;
    hd->n_routed = 0;
    hd->published = 0;
    hd->loaded = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int g = threadIdx.x; g < ns; g += blockDim.x) {
    const int c = g / spt, j = g - c * spt;
    hd->expert[g] = p.E + c;
    hd->row_begin[g] = p.M + c * p.T + j * kMsRows;
    hd->rows[g] = min(kMsRows, p.T - j * kMsRows);
  }
  for (int i = threadIdx.x; i < p.n_shared * p.T; i += blockDim.x) hd->order[p.M + i] = i % p.T;
  if (p.Wr && warp < kMsConsumers) {
    // the router rows of this CTA's first unit are weights: asked into L2 before the dependency wait
    const int rows = p.E + p.extra, nblk = (rows + 7) >> 3;
    const int unit = (int)gridDim.x - 1 - (int)blockIdx.x;
    if (unit < nblk * p.T) {
      const int e = (unit % nblk) * 8 + warp;
      if (e < rows)
        for (int off = lane * 128; off < p.H * 4; off += 32 * 128)
          asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char*>(p.Wr + (size_t)e * p.H) + off));
    }
  }
  const int* offsets = p.offsets;
  const int* active = p.active;
  const int* order = p.order;
  const __nv_bfloat16* X = p.X;
  int* ticket = p.work;
  int* finished = p.work + 1;
  int* done = p.work + kMsWork;
  chain_wait(offsets, active, order, X, ticket);
  __syncthreads();

  // two buffers of eight rows of X if the ring keeps enough stages beside them, else one
  const size_t buf_bytes = (size_t)kMsRows * p.b_stride;
  const size_t room = (size_t)(smem_end - xs);
  const int n_bufs = room >= 2 * buf_bytes + 1024 + (size_t)(kMsMinStages + 1) * kMsSlotBytes ? 2 : 1;
  unsigned char* ring = reinterpret_cast<unsigned char*>(((uintptr_t)(xs + n_bufs * buf_bytes) + 1023) & ~(uintptr_t)1023);
  const int stages = min(kMsMaxStages, (int)((smem_end - ring) / kMsSlotBytes));
  if (smem_end < ring || stages < 2) {             // (the host's check of the sizes rules this out)
    if (threadIdx.x == 0) atomicCAS(&g_moe_stream_error, 0, 7);
  } else if (warp == kMsConsumers) {
    // ---- weight producer -----------------------------------------------------------------------------
    // Lane 0 streams the items; in between, once, the whole warp reads the plan into the table
    // (the routed row groups behind the shared expert's, the tokens of the pairs).
    MsRing at = {0, 1, stages};               // parity of the "empty" wait: a fresh slot counts as released
    int issued = 0, seq = 0, total = 0x7fffffff;
    // items that need no plan go to the CTAs in order, without a ticket; tickets count on from there
    const int untaken = min(items_s1, (int)gridDim.x);
    int pending = (int)blockIdx.x < untaken ? (int)blockIdx.x : -1;
    bool ok = true, ended = false;
    auto stream_items = [&](int nr) {
      // takes tickets and streams their items; returns with `pending` set at the first item that needs the plan
      while (ok && !ended) {
        const int id = pending >= 0 ? pending : untaken + atomicAdd(ticket, 1);
        pending = -1;
        if (nr < 0 && id >= items_s1) { pending = id; return; }
        const bool last = id >= total;
        // name the item for the loader and the consumers (the loader must have read the slot's last tenant)
        if (seq >= kMsFifo && !spin_above(&hd->loaded, seq - kMsFifo, stop, 9)) { ok = false; return; }
        hd->fifo[seq % kMsFifo] = last ? -1 : id;
        __threadfence_block();
        *reinterpret_cast<volatile int*>(&hd->published) = seq + 1;
        ++seq;
        if (last) {
          if (mbar_wait(&hd->empty[at.s], at.parity, stop, 1, &g_moe_stream_error)) mbar_arrive(&hd->full[at.s]);   // an empty stage that carries the end mark
          ended = true;
          return;
        }
        const MsItem item = ms_decode(id, ns, max(nr, 0), n1, n2);
        const int e = hd->expert[item.a];
        const int f0 = item.sub * 16 * Q, ft = f0 >> 7, r0 = f0 & 127;
        // first product: tile (ft, kt) holds 256 rows, gate rows at r0, up rows at 128 + r0; second: 128 rows
        const int kt = item.second ? kt2 : kt1;
        const size_t tile = item.second ? 128 * 64 : 256 * 64;
        const __nv_bfloat16* w = e < p.E ? (item.second ? p.W2 + (size_t)e * p.gs2 : p.W13 + (size_t)e * p.gs13)
                                         : (item.second ? p.Ws2 + (size_t)(e - p.E) * p.gss2 : p.Ws13 + (size_t)(e - p.E) * p.gss13);
        const __nv_bfloat16* src = w + ((size_t)ft * kt * (item.second ? 128 : 256) + r0) * 64;
        for (int t0 = 0; t0 < kt && ok; t0 += G) {
          const int nblk = min(G, kt - t0);
          for (int half = 0; half < (item.second ? 1 : 2); ++half) {
            if (!mbar_wait(&hd->empty[at.s], at.parity, stop, 1, &g_moe_stream_error)) { ok = false; break; }
            unsigned char* dst = ring + (size_t)at.s * kMsSlotBytes;
            mbar_expect_tx(&hd->full[at.s], nblk * BLOCK_BYTES);
            for (int b = 0; b < nblk; ++b)
              bulk_load(dst + b * BLOCK_BYTES, src + (size_t)(t0 + b) * tile + half * (128 * 64), BLOCK_BYTES, &hd->full[at.s]);
            at.next();
            ++issued;
          }
        }
      }
    };
    if (lane == 0) stream_items(-1);          // the shared expert's first product needs no plan
    __syncwarp();
    // ---- the plan: wait for it if this launch routes, then the routed row groups and the pairs' tokens ----
    int have = 1;
    if (lane == 0) {
      have = ok && !*stop;
      if (have && p.Wr) {
        have = 0;
        for (unsigned i = 0; i < kMsCountPolls; ++i)
          if (ld_acquire(p.work + 4) > 0) { have = 1; break; }
        if (!have) {
          *stop = 1;
          atomicCAS(&g_moe_stream_error, 0, 14);
        }
      }
    }
    __syncwarp();                                // lane 0's acquire comes before the other lanes' reads of the table
    have = __shfl_sync(0xffffffffu, have, 0);
    int nr = 0;
    if (have && p.Wr) {
      // the routing of this launch has written the routed row groups and the pairs' tokens as they are needed
      const int* table = p.work + kMsTable;
      // (the first groups are asked for together with their number: one trip to L2 instead of two)
      const int most = min(p.n_mapped + p.M / kMsRows, kMsMaxGroups - ns);      // routed row groups at worst
      int e0 = 0, rb0 = 0, rw0 = 0;
      if (lane < most) {
        e0 = ld_l2_int(table + 1 + lane);
        rb0 = ld_l2_int(table + 1 + kMsMaxGroups + lane);
        rw0 = ld_l2_int(table + 1 + 2 * kMsMaxGroups + lane);
      }
      nr = min(ld_l2_int(table), kMsMaxGroups - ns);
      if (lane < nr) {
        hd->expert[ns + lane] = e0;
        hd->row_begin[ns + lane] = rb0;
        hd->rows[ns + lane] = rw0;
      }
      for (int g0 = 32; g0 < nr; g0 += 32) {
        const int g2 = g0 + lane;
        if (g2 < nr) {
          const int e = ld_l2_int(table + 1 + g2), rb = ld_l2_int(table + 1 + kMsMaxGroups + g2);
          const int rw = ld_l2_int(table + 1 + 2 * kMsMaxGroups + g2);
          hd->expert[ns + g2] = e;
          hd->row_begin[ns + g2] = rb;
          hd->rows[ns + g2] = rw;
        }
      }
      for (int i0 = 0; i0 < p.M; i0 += 4 * 32) {
        int tk[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) tk[u] = i0 + u * 32 + lane < p.M ? ld_l2_int(table + 1 + 3 * kMsMaxGroups + i0 + u * 32 + lane) : 0;
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (i0 + u * 32 + lane < p.M) hd->order[i0 + u * 32 + lane] = tk[u];
      }
      if (lane == 0) *reinterpret_cast<volatile int*>(&hd->n_routed) = nr;
    } else if (have) {
      for (int i0 = 0; i0 < p.n_mapped; i0 += 32) {
        const int i = i0 + lane;
        int e = i < p.n_mapped ? ld_l2_int(active + i) : -1;
        int rb = 0, cnt = 0;
        if (e >= p.E) { atomicCAS(&g_moe_stream_error, 0, 5); e = -1; }
        if (e >= 0) {
          rb = ld_l2_int(offsets + e);
          const int re = ld_l2_int(offsets + e + 1);
          if (rb < 0 || re > p.M) atomicCAS(&g_moe_stream_error, 0, 6);
          else cnt = max(re - rb, 0);
        }
        // an expert's rows, eight at a time
        const int ng = (cnt + kMsRows - 1) / kMsRows;
        int incl = ng;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          const int o = __shfl_up_sync(0xffffffffu, incl, d);
          if (lane >= d) incl += o;
        }
        const int first = ns + nr + incl - ng;
        for (int j = 0; j < ng; ++j)
          if (first + j < kMsMaxGroups) {
            hd->expert[first + j] = e;
            hd->row_begin[first + j] = rb + j * kMsRows;
            hd->rows[first + j] = min(kMsRows, cnt - j * kMsRows);
          }
        nr += __shfl_sync(0xffffffffu, incl, 31);
      }
      if (ns + nr > kMsMaxGroups) {
        if (lane == 0) atomicCAS(&g_moe_stream_error, 0, 7);
        nr = kMsMaxGroups - ns;
      }
      for (int i0 = 0; i0 < p.M; i0 += 4 * 32) {
        int pr[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) pr[u] = i0 + u * 32 + lane < p.M ? ld_l2_int(order + i0 + u * 32 + lane) : 0;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int i = i0 + u * 32 + lane;
          if (i < p.M) {
            int tok = pr[u] / p.k;
            if (pr[u] < 0 || tok >= p.T) { atomicCAS(&g_moe_stream_error, 0, 6); tok = -1; }     // no row is copied for it
            hd->order[i] = tok;
          }
        }
      }
      if (lane == 0) *reinterpret_cast<volatile int*>(&hd->n_routed) = nr;
    }
    __threadfence_block();
    __syncwarp();
    if (lane == 0) {
      if (have) {
        total = (ns + nr) * (n1 + n2);
        stream_items(nr);
      }
      if (!ok || !have) {
        // gave up: let every copy that was started land before the CTA's shared memory goes away
        int s2 = at.s, parity = at.parity ^ 1;       // "full" parity of the slot issued last is the "empty" parity it was waited with, flipped
        for (int j = 0; j < min(issued, stages); ++j) {
          if (--s2 < 0) { s2 = stages - 1; parity ^= 1; }
          for (unsigned i = 0; i < (1u << 20); ++i)
            if (mbar_try(&hd->full[s2], parity)) break;
        }
      }
    }
  } else if (warp == kMsConsumers + 1) {
    // ---- row loader: the rows of X of the next item, as soon as they are complete ---------------------
    if (lane == 0) {
      int seq = 0;                      // items read = items served
      int issued_buf = -1, issued_use = 0;
      const unsigned pad1 = (unsigned)(kt1 * 128 - p.H * 2), pad2 = (unsigned)(kt2 * 128 - p.I * 2);   // bytes behind a row's last k
      while (true) {
        if (!spin_above(&hd->published, seq, stop, 10)) break;
        const int id = reinterpret_cast<volatile int*>(hd->fifo)[seq % kMsFifo];
        const int n = seq;
        ++seq;
        *reinterpret_cast<volatile int*>(&hd->loaded) = seq;
        if (id < 0) break;
        const MsItem item = ms_decode(id, ns, *reinterpret_cast<volatile int*>(&hd->n_routed), n1, n2);
        const int buf = n % n_bufs, use = n / n_bufs;
        if (!mbar_wait(&hd->xempty[buf], (use & 1) ^ 1, stop, 11, &g_moe_stream_error)) break;
        const int rows = hd->rows[item.a], row_begin = hd->row_begin[item.a];
        unsigned char* dst = xs + (size_t)buf * buf_bytes;
        if (item.second) {
          bool there = false;
          for (unsigned i = 0; i < kMsCountPolls; ++i) {
            if (ld_acquire(done + item.a) >= target) { there = true; break; }
            if ((i & 255u) == 255u && *stop) break;
          }
          if (!there) {
            *stop = 1;
            atomicCAS(&g_moe_stream_error, 0, 4);
            break;
          }
          asm volatile("fence.proxy.async;" ::: "memory");      // the rows were written by ordinary stores of other SMs
          const unsigned bytes = (unsigned)p.I * 2;
          mbar_expect_tx(&hd->xfull[buf], rows * (bytes + pad2));
          for (int r = 0; r < rows; ++r) {
            bulk_load(dst + (size_t)r * p.b_stride, p.act + (size_t)(row_begin + r) * p.I, bytes, &hd->xfull[buf]);
            if (pad2) bulk_load(dst + (size_t)r * p.b_stride + bytes, g_ms_zeros, pad2, &hd->xfull[buf]);
          }
        } else {
          const unsigned bytes = (unsigned)p.H * 2;
          int live = 0;
          for (int r = 0; r < rows; ++r) live += hd->order[row_begin + r] >= 0;
          mbar_expect_tx(&hd->xfull[buf], live * bytes + rows * pad1);
          for (int r = 0; r < rows; ++r) {
            const int tok = hd->order[row_begin + r];
            if (tok >= 0) bulk_load(dst + (size_t)r * p.b_stride, X + (size_t)tok * p.ldx, bytes, &hd->xfull[buf]);
            if (pad1) bulk_load(dst + (size_t)r * p.b_stride + bytes, g_ms_zeros, pad1, &hd->xfull[buf]);
          }
        }
        issued_buf = buf;
        issued_use = use;
      }
      if (*stop && issued_buf >= 0) {
        // let the last rows that were asked for land (the consumers may have left without them)
        for (unsigned i = 0; i < (1u << 20); ++i)
          if (mbar_try(&hd->xfull[issued_buf], issued_use & 1)) break;
      }
    }
  } else {
    // ---- consumers: the routing first, if the launch has it --------------------------------------------
    if (p.Wr) ms_route(p, scratch, &s_unit, &s_last_unit, warp, lane);
    const int rg = warp % Q, kg = warp / Q;
    const int g = lane >> 2, t = lane & 3;
    // ldmatrix addresses inside a block of 16 Q rows x 64 k: this lane's row and 16-byte piece parity
    const int a_row = 16 * rg + ((lane >> 3) & 1) * 8 + (lane & 7);
    const int a_hi = lane >> 4;                  // second pair of matrices: k + 8
    // B: matrices (rows 0-7, k..k+7), (rows 0-7, k+8..): this lane's row and k half.  (Rows beyond
    // the group's last hold what an earlier item left: they only reach columns that are not stored.)
    const unsigned b_off = (unsigned)(lane & 7) * p.b_stride + ((lane >> 3) & 1) * 16;
    MsRing at = {0, 0, stages};
    int seq = 0;
    unsigned meets = 0;                          // how often the consumers have met
    while (true) {
      if (!mbar_wait(&hd->full[at.s], at.parity, stop, 2, &g_moe_stream_error)) break;
      const int id = hd->fifo[seq % kMsFifo];
      const int buf = seq % n_bufs, use = seq / n_bufs;
      ++seq;
      if (id < 0) break;
      const MsItem item = ms_decode(id, ns, *reinterpret_cast<volatile int*>(&hd->n_routed), n1, n2);
      const int row_begin = hd->row_begin[item.a], rows = hd->rows[item.a];

      float acc[2][4];
#pragma unroll
      for (int b = 0; b < 2; ++b)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[b][i] = 0.f;
      if (!mbar_wait(&hd->xfull[buf], use & 1, stop, 12, &g_moe_stream_error)) break;
      const unsigned b_lane = smem_u32(xs) + (unsigned)(buf * buf_bytes) + b_off;
      const bool ok = item.second ? ms_k_loop<Q, true>(hd, ring, at, kt2, kg, a_row, a_hi, b_lane, acc)
                                  : ms_k_loop<Q, false>(hd, ring, at, kt1, kg, a_row, a_hi, b_lane, acc);
      __syncwarp();
      if (lane == 0) mbar_arrive(&hd->xempty[buf]);
      if (!ok) break;

      // ---- k groups meet, in order --------------------------------------------------------------
      if (G > 1) {
        // (two meeting places in turn: a warp may write the next item's sums while the sums of
        // this one are still being read, and the meeting after that orders the rest)
        float* red_now = red + (meets & 1) * (kMsConsumers * 2 * 4 * 32);
        if (kg > 0) {
#pragma unroll
          for (int b = 0; b < 2; ++b)
#pragma unroll
            for (int i = 0; i < 4; ++i) red_now[((warp * 2 + b) * 4 + i) * 32 + lane] = acc[b][i];
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&hd->meet);
        const bool met = mbar_wait(&hd->meet, meets & 1, stop, 8, &g_moe_stream_error);
        ++meets;
        if (!met) break;
        if (kg == 0) {
          for (int o = 1; o < G; ++o) {
            const int w = o * Q + rg;
#pragma unroll
            for (int b = 0; b < 2; ++b)
#pragma unroll
              for (int i = 0; i < 4; ++i) acc[b][i] += red_now[((w * 2 + b) * 4 + i) * 32 + lane];
          }
        }
      }

      // ---- epilogue: lane holds features (f, f + 8) of rows (2t, 2t + 1) --------------------------
      if (kg == 0) {
        const int f_lo = item.sub * 16 * Q + 16 * rg + g;
        const int N = item.second ? p.H : p.I;
        __nv_bfloat16* out = item.second ? p.Y : p.act;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int r = 2 * t + (i & 1), f = f_lo + (i >> 1) * 8;
          if (r < rows && f < N) {
            float v = acc[0][i];
            if (!item.second) v = v / (1.f + expf(-v)) * acc[1][i];
            out[(size_t)(row_begin + r) * N + f] = __float2bfloat16_rn(v);
          }
        }
      }
      if (!item.second) {
        // this warp's share of the item is in memory: count it (8 counts an item)
        __syncwarp();
        if (lane == 0) add_release(done + item.a, 1);
      }
    }
  }

  // ---- the last CTA to finish puts the counters back to zero ------------------------------------
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    s_last = atomicAdd(finished, 1) == (int)gridDim.x - 1;
  }
  __syncthreads();
  if (s_last) {
    for (int i = threadIdx.x; i < kMsMaxGroups; i += blockDim.x) done[i] = 0;
    __syncthreads();
    if (threadIdx.x == 0) {
      *ticket = 0;
      p.work[2] = 0;
      p.work[3] = 0;
      p.work[4] = 0;
      __threadfence();
      *finished = 0;
    }
  }
}

template <int Q>
static int launch_ms(const MsArgs& a, int grid, size_t smem, cudaStream_t stream) {
  static size_t set_bytes = 0;
  if (smem > set_bytes) {
    cudaError_t e = cudaFuncSetAttribute(moe_stream_kernel<Q>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    NF_REQUIRE(e == cudaSuccess, "moe_stream: cannot have %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    set_bytes = smem;
  }
  launch_chained(moe_stream_kernel<Q>, dim3(grid), dim3(kMsThreads), smem, stream, a);
  return check_launch("moe_stream");
}

// The row stride, the k groups' meeting place and the routing's tables of a launch, and whether
// they, one buffer of eight rows and a ring of the smallest size fit into `budget` bytes of
// shared memory.
static bool ms_layout(int q, int H, int I, size_t budget, MsArgs* a, int route_experts = 0, int pairs = 0) {
  const int widest = H > I ? H : I;
  const int b_stride = (widest + 63) / 64 * 64 * 2 + 16;      // + 16: rows eight apart do not share a bank
  const int red = q < 8 ? 2 * kMsConsumers * 2 * 4 * 32 * 4 : 0;
  size_t scratch = 0;
  if (route_experts) {
    // x as float32, then: selection tables, the pairs' weights, experts and ranks, further logits, counts
    scratch = (size_t)H * 4;
    const size_t tables = (size_t)kMsConsumers * route_experts * 4 + (size_t)pairs * 16 + 64 + (size_t)(route_experts + 1) * 4;
    if (tables > scratch) scratch = tables;
    scratch = (scratch + 1023) & ~(size_t)1023;
  }
  const size_t worst = 1024 + ((sizeof(MsHeader) + 1023) & ~(size_t)1023) + red + scratch + (size_t)kMsRows * b_stride + 1024 +
                       (size_t)kMsMinStages * kMsSlotBytes;
  if (worst > budget) return false;
  if (a) { a->b_stride = b_stride; a->red_bytes = red; a->scratch_bytes = (int)scratch; a->smem_bytes = (int)budget; }
  return true;
}

}  // namespace nf

using namespace nf;

// How many ints of zeroed device memory a launch needs as `work` (its counters are zero again
// when it has finished; the rest is scratch).
extern "C" int nf_moe_stream_work_ints() { return kMsWorkInts; }
// ... and how many of them, from the first on, are the counters.
extern "C" int nf_moe_stream_counter_ints() { return kMsTable; }

// 1 if the sizes fit the kernel: `pairs` (token, expert) pairs, `n_mapped` listed experts,
// `shared_rows` rows of the shared expert's chunks (chunks x tokens), and room for a row buffer
// and a ring inside `smem_bytes` of shared memory.
// route_experts: 0, or E if the launch also routes (its tables then need room too, and E < 65536).
extern "C" int nf_moe_stream_fits(int H, int I, int pairs, int n_mapped, int q, int smem_bytes, int route_experts,
                                  int shared_rows) {
  if (!(q == 2 || q == 4 || q == 8) || pairs < 1 || shared_rows < 0 || pairs + shared_rows > kMsMaxPairs) return 0;
  if (n_mapped + pairs / kMsRows + shared_rows > kMsMaxGroups) return 0;           // row groups at worst
  if (H % 8 || I % 8 || smem_bytes > 227 * 1024) return 0;
  if (route_experts < 0 || route_experts > 65535 || (shared_rows && !route_experts)) return 0;
  return ms_layout(q, H, I, (size_t)smem_bytes, nullptr, route_experts, pairs) ? 1 : 0;
}

// act[M, I] = silu(x Wgate_e^T) * (x Wup_e^T) and Y[M, H] = act Wdown_e^T for the sorted pairs of
// every expert that has rows, in one persistent launch.  X [T, H] bfloat16 (row stride ldx),
// W13 / W2 packed (strides in elements), offsets / order / active from the routing plan, M = T k
// pairs.  q: an item is 16 q features (2, 4, 8).  `work`: nf_moe_stream_work_ints() ints, zero
// before the first launch; the kernel leaves them zero.  smem_bytes: shared memory the launch
// takes (what is left stays free for kernels of other streams on the same SM).
// Wr != null: the launch routes first - logits[t, e] = x[t] . Wr[e] in float32 for the E router
// rows and `extra` further rows, softmax, the k largest (ties to the lower index), weights
// p_e or p_e / sum(selected) - and writes topk_idx [T, k], topk_w [T, k], extra_out [T, extra]
// (the further rows' raw logits), offsets, order, inv [M] and active itself; `logits`
// [T, E + extra] is scratch.  The values are those of the router kernels (router.cu).
// n_shared > 0 (with routing only): a shared expert as well, its intermediate features cut into
// n_shared chunks of I and packed like n_shared experts (Ws13, Ws2); chunk c writes rows
// M + c T .. M + (c + 1) T of act and Y, which then have M + n_shared T rows.  Its products are
// under way while the routing is still being computed.  cw / cinv [T, k + n_shared]: for every
// token the weights and rows of Y to add up - the k experts', then every chunk's with
// sigmoid(extra_out[t, 0]) (1 without further rows).
extern "C" int nf_moe_stream(const void* X, int ldx, const void* W13, long long gs13, const void* W2, long long gs2,
                             void* act, void* Y, int M, int T, int H, int I, int E, int k, const int* offsets,
                             const int* order, const int* active, int n_mapped, int* work, int q,
                             int smem_bytes, const float* Wr, int extra, int norm_topk, float* logits, int* topk_idx,
                             float* topk_w, float* extra_out, int* inv, const void* Ws13, long long gss13,
                             const void* Ws2, long long gss2, int n_shared, float* cw, int* cinv,
                             cudaStream_t stream) {
  if (M == 0) return 0;
  NF_REQUIRE(M > 0 && T > 0 && k > 0 && E > 0 && ldx % 8 == 0 && n_shared >= 0, "moe_stream: bad sizes");
  NF_REQUIRE(!Wr || (logits && topk_idx && topk_w && inv && extra >= 0 && (extra == 0 || extra_out) && M == T * k && k <= E),
             "moe_stream: routing needs its outputs");
  NF_REQUIRE(n_shared == 0 || (Wr && Ws13 && Ws2 && cw && cinv && gss13 % 8 == 0 && gss2 % 8 == 0 &&
                               (uintptr_t)Ws13 % 16 == 0 && (uintptr_t)Ws2 % 16 == 0),
             "moe_stream: a shared expert needs the routing inside the launch, its packed weights and cw / cinv");
  NF_REQUIRE(nf_moe_stream_fits(H, I, M, n_mapped, q, smem_bytes, Wr ? E : 0, n_shared * T),
             "moe_stream: sizes do not fit (H=%d I=%d pairs=%d experts=%d q=%d smem=%d shared chunks=%d)",
             H, I, M, n_mapped, q, smem_bytes, n_shared);
  NF_REQUIRE(((uintptr_t)X % 16 == 0) && ((uintptr_t)W13 % 16 == 0) && ((uintptr_t)W2 % 16 == 0) && ((uintptr_t)act % 16 == 0) &&
             gs13 % 8 == 0 && gs2 % 8 == 0, "moe_stream: operands must be 16-byte aligned");
  MsArgs a;
  a.X = (const __nv_bfloat16*)X; a.W13 = (const __nv_bfloat16*)W13; a.W2 = (const __nv_bfloat16*)W2;
  a.act = (__nv_bfloat16*)act; a.Y = (__nv_bfloat16*)Y;
  a.offsets = offsets; a.order = order; a.active = active; a.work = work;
  a.gs13 = gs13; a.gs2 = gs2;
  a.Wr = Wr; a.logits = logits; a.topk_idx = topk_idx; a.topk_w = topk_w; a.extra_out = extra_out; a.inv = inv;
  a.extra = Wr ? extra : 0; a.norm_topk = norm_topk;
  a.Ws13 = (const __nv_bfloat16*)Ws13; a.Ws2 = (const __nv_bfloat16*)Ws2; a.gss13 = gss13; a.gss2 = gss2;
  a.n_shared = n_shared; a.cw = n_shared ? cw : nullptr; a.cinv = n_shared ? cinv : nullptr;
  a.ldx = ldx; a.M = M; a.T = T; a.H = H; a.I = I; a.E = E; a.k = k; a.n_mapped = n_mapped;
  ms_layout(q, H, I, (size_t)smem_bytes, &a, Wr ? E : 0, M);
  static int n_sm = 0;
  if (!n_sm) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
    if (n_sm <= 0) n_sm = 1;
  }
  if (q == 2) return launch_ms<2>(a, n_sm, (size_t)smem_bytes, stream);
  if (q == 4) return launch_ms<4>(a, n_sm, (size_t)smem_bytes, stream);
  return launch_ms<8>(a, n_sm, (size_t)smem_bytes, stream);
}

// 0, or the code of the first wait the kernel gave up on / the first bad plan entry since the
// last call (synchronises the device).
extern "C" int nf_moe_stream_status() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_moe_stream_error, sizeof(int)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(g_moe_stream_error, &zero, sizeof(int));
  return v;
}
