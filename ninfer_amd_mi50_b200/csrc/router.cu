// Routing on the device: router logits, softmax, top-k and the execution plan that
// groups (token, expert) pairs by expert.
//
// The reference computes the logits on the GPU in float32 and then routes on the host
// (``moe_route_cpu``, src/ops/moe.hip:49-106: stream sync, copy, softmax with the maximum
// subtracted, ``partial_sort`` of the k largest, renormalisation, counting sort by expert,
// stable in token order).  Here the same steps stay on the device, so a step never waits
// for the host.  Ties go to the lower expert index.  With norm_topk the weights are
// p_e / sum(selected p); without, p_e as they are (the reference always renormalises,
// moe.hip:77-82).
#define NF_CHAIN_CLASS 16
#include "router_device.cuh"

namespace nf {

// Router logits: out[t, e] = x[t] . wr[e] in float32, for the E router rows and `extra`
// further rows (the shared expert's gate).  A block takes TT tokens and 8 rows of wr, one
// warp per row; a lane sums its strided share of the hidden dimension and the warp adds the
// 32 shares in a fixed tree, so the value for (t, e) is the same whatever TT is and
// whatever else is in the batch.
template <typename T, int TT>
__global__ void __launch_bounds__(256)
router_logits_kernel(const T* __restrict__ x, const float* __restrict__ wr, int n_tokens, int hidden,
                     int rows, float* __restrict__ out) {
  extern __shared__ float xs[];        // [TT][hidden]
  const int t0 = blockIdx.y * TT;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nt = min(TT, n_tokens - t0);
  for (int i = threadIdx.x; i < nt * hidden; i += blockDim.x) {
    const int tt = i / hidden, c = i - tt * hidden;
    xs[tt * hidden + c] = to_float(x[(size_t)(t0 + tt) * hidden + c]);
  }
  __syncthreads();
  const int e = blockIdx.x * 8 + warp;
  if (e >= rows) return;
  const float* w = wr + (size_t)e * hidden;
  float acc[TT];
#pragma unroll
  for (int tt = 0; tt < TT; ++tt) acc[tt] = lane_dot(xs + tt * hidden, w, hidden, lane);
#pragma unroll
  for (int tt = 0; tt < TT; ++tt) {
    const float v = warp_sum(acc[tt]);
    if (lane == 0 && tt < nt) out[(size_t)(t0 + tt) * rows + e] = v;
  }
}

__global__ void __launch_bounds__(128)
router_select_kernel(const float* __restrict__ logits, long tok_stride, long exp_stride, int n_tokens,
                     int E, int extra, int k, int norm_topk, int* __restrict__ topk_idx,
                     float* __restrict__ topk_w, float* __restrict__ extra_out) {
  extern __shared__ float smem[];      // [4 warps][E]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + warp;
  chain_wait(logits);
  if (t >= n_tokens) return;
  // logits[t, e] sits at t * tok_stride + e * exp_stride (either may be the unit stride)
  select_token(logits + (size_t)t * tok_stride, exp_stride, smem + warp * E, t, E, extra, k, norm_topk,
               topk_idx, topk_w, extra_out, lane);
}

template <bool STAGED>
__global__ void __launch_bounds__(1024)
moe_plan_kernel(const int* __restrict__ topk_idx, int n, int E, int* __restrict__ offsets,
                int* __restrict__ order, int* __restrict__ inv, int* __restrict__ active,
                int n_active_max) {
  extern __shared__ int counts[];      // [E + 1], then (STAGED) n experts as 16-bit
  plan_block<STAGED>(topk_idx, n, E, offsets, order, inv, counts,
                     reinterpret_cast<unsigned short*>(counts + E + 1), active, n_active_max);
}

// Few tokens (decode steps): logits, selection and plan in one launch.  Blocks (8 router rows,
// 1 token) compute logits as `router_logits_kernel` does; the block that finishes last - which
// one does not matter, it reads what all have written - selects for every token and builds the
// plan.  `ticket` is an int that is zero before the launch and is left zero after it.
template <typename T>
__global__ void __launch_bounds__(256)
router_fused_kernel(const T* __restrict__ x, const float* __restrict__ wr, int n_tokens, int hidden,
                    int E, int extra, int k, int norm_topk, float* __restrict__ logits,
                    int* __restrict__ topk_idx, float* __restrict__ topk_w, float* __restrict__ extra_out,
                    int* __restrict__ offsets, int* __restrict__ order, int* __restrict__ inv,
                    int* __restrict__ active, int n_active_max, int* __restrict__ ticket) {
  extern __shared__ float xs[];        // [hidden]; the last block reuses it
  __shared__ int s_last;
  const int rows = E + extra;
  const int t = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  chain_release();
  // The router's row is a weight: a lane asks for its share (up to 16 pieces of 16 bytes) before
  // it waits for the kernel that writes x.  The sums below run in lane_dot's order exactly.
  const int e = blockIdx.x * 8 + warp;
  const float* w = wr + (size_t)min(e, rows - 1) * hidden;
  constexpr int kPre = 16;
  const bool pre = (hidden & 3) == 0 && ((uintptr_t)wr & 15) == 0 && hidden <= kPre * 128;
  float4 wv[kPre];
  if (pre) {
#pragma unroll
    for (int j = 0; j < kPre; ++j) {
      const int i = lane * 4 + j * 128;
      wv[j] = i < hidden ? *reinterpret_cast<const float4*>(w + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  chain_wait(x);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) xs[i] = to_float(x[(size_t)t * hidden + i]);
  __syncthreads();
  if (e < rows) {
    float v;
    if (pre) {
      float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
      for (int j = 0; j < kPre; ++j) {
        const int i = lane * 4 + j * 128;
        if (i < hidden) {
          const float4 xv = *reinterpret_cast<const float4*>(xs + i);
          s0 = fmaf(xv.x, wv[j].x, s0);
          s1 = fmaf(xv.y, wv[j].y, s1);
          s2 = fmaf(xv.z, wv[j].z, s2);
          s3 = fmaf(xv.w, wv[j].w, s3);
        }
      }
      v = warp_sum((s0 + s1) + (s2 + s3));
    } else {
      v = warp_sum(lane_dot(xs, w, hidden, lane));
    }
    if (lane == 0) logits[(size_t)t * rows + e] = v;
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(ticket, 1) == (int)(gridDim.x * gridDim.y) - 1;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // ---- the last block: selection for every token, then the plan ------------------------------
  float* lg = xs;                                   // [8 warps][E]
  for (int tt = warp; tt < n_tokens; tt += 8)
    select_token(logits + (size_t)tt * rows, 1, lg + warp * E, tt, E, extra, k, norm_topk, topk_idx, topk_w,
                 extra_out, lane);
  __threadfence_block();
  __syncthreads();
  int* counts = reinterpret_cast<int*>(xs);         // [E + 1], then the pairs' experts
  plan_block<true>(topk_idx, n_tokens * k, E, offsets, order, inv, counts,
                   reinterpret_cast<unsigned short*>(counts + E + 1), active, n_active_max);
  if (threadIdx.x == 0) *ticket = 0;
}

// Few tokens, second form: the same work by ONE thread-block cluster of 8 CTAs, with the
// hand-over from "all logits" to "selection and plan" through distributed shared memory and the
// cluster barrier instead of global memory, a fence and a ticket.  Every warp of the cluster
// owns router rows e = 8 cta + warp + 64 j: it asks for its first row's weights before the
// dependency wait, multiplies it with every token of the step (x sits in shared memory as
// float32, the sums run in `lane_dot`'s order, so a logit has the bits the other kernels give
// it) and stores the logits into CTA 0's shared memory.  After the barrier CTA 0 selects (one
// warp per token) and builds the plan without leaving shared memory; the others are done.
constexpr int kRouterCluster = 8;

__device__ __forceinline__ unsigned cluster_ctarank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void st_cluster_f32(float* local_ptr, unsigned cta, float v) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(local_ptr);
  unsigned remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(a), "r"(cta));
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

template <typename T>
__global__ void __launch_bounds__(256)
router_cluster_kernel(const T* __restrict__ x, const float* __restrict__ wr, int n_tokens, int hidden,
                      int E, int extra, int k, int norm_topk, float* __restrict__ logits_out,
                      int* __restrict__ topk_idx, float* __restrict__ topk_w, float* __restrict__ extra_out,
                      int* __restrict__ offsets, int* __restrict__ order, int* __restrict__ inv,
                      int* __restrict__ active, int n_active_max) {
  extern __shared__ __align__(16) float rs[];
  const int rows = E + extra;
  const int n = n_tokens * k;
  float* xs = rs;                                        // [n_tokens][hidden]
  float* lg_all = xs + (size_t)n_tokens * hidden;        // [n_tokens][rows]   (CTA 0's copy is the one used)
  float* sel = lg_all + (size_t)n_tokens * rows;         // [8 warps][E]
  int* counts = reinterpret_cast<int*>(sel + 8 * E);     // [E + 1]
  int* rank = counts + E + 1;                            // [n]
  unsigned short* chosen = reinterpret_cast<unsigned short*>(rank + n);   // [n]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned cta = cluster_ctarank();
  const int e0 = (int)cta * 8 + warp;
  // A CTA's shared memory may only be written from another CTA once that CTA is running: every
  // thread announces itself here, and waits for all the others right before its first remote
  // store (the dot products pass in between, so the meeting costs nothing).
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");

  constexpr int kPre = 16;
  const bool vec = (hidden & 3) == 0 && ((uintptr_t)wr & 15) == 0;
  const bool pre = vec && hidden <= kPre * 128 && e0 < rows;
  float4 wv[kPre];
  if (pre) {
    const float* w = wr + (size_t)e0 * hidden;
#pragma unroll
    for (int j = 0; j < kPre; ++j) {
      const int i = lane * 4 + j * 128;
      wv[j] = i < hidden ? *reinterpret_cast<const float4*>(w + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  chain_wait(x);
  {
    // x -> float32 in shared memory, 16 bytes of x a thread a step where alignment allows
    const int total = n_tokens * hidden;
    constexpr int PER = 16 / (int)sizeof(T);
    if (((uintptr_t)x & 15) == 0 && total % PER == 0) {
      constexpr int U = 8;                       // loads in flight a thread: the rows are one trip to L2, not one each
      const int step = blockDim.x * PER;
      for (int i0 = threadIdx.x * PER; i0 < total; i0 += step * U) {
        uint4 raw[U];
#pragma unroll
        for (int u = 0; u < U; ++u)
          if (i0 + u * step < total) raw[u] = *reinterpret_cast<const uint4*>(x + i0 + u * step);
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (i0 + u * step < total) {
            const T* v = reinterpret_cast<const T*>(&raw[u]);
            // 16-byte stores: scalar ones would put the lanes 8 floats apart, 8 to a bank
#pragma unroll
            for (int j = 0; j < PER; j += 4)
              *reinterpret_cast<float4*>(xs + i0 + u * step + j) =
                  make_float4(to_float(v[j]), to_float(v[j + 1]), to_float(v[j + 2]), to_float(v[j + 3]));
          }
        }
      }
    } else {
      for (int i = threadIdx.x; i < total; i += blockDim.x) xs[i] = to_float(x[i]);
    }
  }
  __syncthreads();
  bool met = false;                      // this thread has seen every CTA of the cluster running
  for (int e = e0; e < rows; e += 8 * kRouterCluster) {
    const float* w = wr + (size_t)e * hidden;
    float mine = 0.f;
    for (int t = 0; t < n_tokens; ++t) {
      const float* xt = xs + (size_t)t * hidden;
      float v;
      if (pre && e == e0) {
        float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
        for (int j = 0; j < kPre; ++j) {
          const int i = lane * 4 + j * 128;
          if (i < hidden) {
            const float4 xv = *reinterpret_cast<const float4*>(xt + i);
            s0 = fmaf(xv.x, wv[j].x, s0);
            s1 = fmaf(xv.y, wv[j].y, s1);
            s2 = fmaf(xv.z, wv[j].z, s2);
            s3 = fmaf(xv.w, wv[j].w, s3);
          }
        }
        v = warp_sum((s0 + s1) + (s2 + s3));
      } else {
        v = warp_sum(lane_dot(xt, w, hidden, lane));
      }
      if (lane == t) mine = v;          // lane t keeps token t's logit (n_tokens <= 32)
    }
    // one remote store a lane, all in flight together: a store into another CTA's shared
    // memory takes long, and one after the other they would add up
    if (!met) {
      asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
      met = true;
    }
    if (lane < n_tokens) {
      st_cluster_f32(lg_all + (size_t)lane * rows + e, 0, mine);
      if (logits_out) logits_out[(size_t)lane * rows + e] = mine;
    }
  }
  if (!met) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");   // a warp without rows
  cluster_sync_all();
  if (cta != 0) return;
  // ---- CTA 0: selection for every token, then the plan, all in shared memory --------------------
  for (int tt = warp; tt < n_tokens; tt += 8)
    select_token<false>(lg_all + (size_t)tt * rows, 1, sel + warp * E, tt, E, extra, k, norm_topk, topk_idx, topk_w,
                        extra_out, lane, chosen);
  __syncthreads();
  for (int e = warp; e < E; e += 8) {
    int running = 0;
    for (int base = 0; base < n; base += 32) {
      const int i = base + lane;
      const bool mine = i < n && (int)chosen[i] == e;
      const unsigned b = __ballot_sync(0xffffffffu, mine);
      if (mine) rank[i] = running + __popc(b & ((1u << lane) - 1u));   // rank inside the expert
      running += __popc(b);
    }
    if (lane == 0) counts[e] = running;
  }
  __syncthreads();
  if (warp == 0) {
    // one warp, 32 experts a round: exclusive prefix of the counts (-> offsets) and the list of
    // the experts that have pairs, ascending, then -1
    int run = 0, na = 0;
    for (int base = 0; base <= E; base += 32) {
      const int e = base + lane;
      const int c = e < E ? counts[e] : 0;
      int incl = c;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
      }
      if (e <= E) {
        counts[e] = run + incl - c;
        offsets[e] = run + incl - c;
      }
      run += __shfl_sync(0xffffffffu, incl, 31);
      const unsigned b = __ballot_sync(0xffffffffu, c > 0);
      if (active) {
        const int at = na + __popc(b & ((1u << lane) - 1u));
        if (c > 0 && at < n_active_max) active[at] = e;
      }
      na += __popc(b);
    }
    if (active)
      for (int i = min(na, n_active_max) + lane; i < n_active_max; i += 32) active[i] = -1;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int p = counts[chosen[i]] + rank[i];
    inv[i] = p;
    order[p] = i;
  }
}

// The same plan for many pairs, spread over the device.  Block e ranks the pairs of expert e
// (in pair order, so token order is kept) and counts them; the second kernel turns counts into
// offsets and scatters.
__global__ void __launch_bounds__(1024)
moe_rank_kernel(const int* __restrict__ topk_idx, int n, int* __restrict__ counts, int* __restrict__ inv) {
  // warp w takes the contiguous chunk w of the pairs: count, prefix over warps, then rank
  __shared__ int warp_tot[32];
  const int e = blockIdx.x;
  chain_release_if_small();
  chain_wait(topk_idx);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
  const int chunk = ((n + nwarp - 1) / nwarp + 31) & ~31;
  const int lo = warp * chunk, hi = min(n, lo + chunk);
  int cnt = 0;
  for (int base = lo; base < hi; base += 32) {
    const int i = base + lane;
    cnt += __popc(__ballot_sync(0xffffffffu, i < hi && topk_idx[i] == e));
  }
  if (lane == 0) warp_tot[warp] = cnt;
  __syncthreads();
  int running = 0;
  for (int w = 0; w < warp; ++w) running += warp_tot[w];
  for (int base = lo; base < hi; base += 32) {
    const int i = base + lane;
    const bool mine = i < hi && topk_idx[i] == e;
    const unsigned b = __ballot_sync(0xffffffffu, mine);
    if (mine) inv[i] = running + __popc(b & ((1u << lane) - 1u));
    running += __popc(b);
  }
  if (threadIdx.x == blockDim.x - 1) counts[e] = running;
}

__global__ void __launch_bounds__(256)
moe_scatter_kernel(const int* __restrict__ topk_idx, int n, int E, const int* __restrict__ counts,
                   int* __restrict__ offsets, int* __restrict__ order, int* __restrict__ inv,
                   int* __restrict__ active, int n_active_max) {
  extern __shared__ int off[];        // [E + 1]
  chain_release_if_small();
  chain_wait(topk_idx, counts);
  if (threadIdx.x == 0) {
    int run = 0, na = 0;
    const bool list = active && blockIdx.x == 0;
    for (int e = 0; e < E; ++e) {
      off[e] = run;
      if (list && counts[e] > 0 && na < n_active_max) active[na++] = e;
      run += counts[e];
    }
    off[E] = run;
    if (list)
      for (; na < n_active_max; ++na) active[na] = -1;
  }
  __syncthreads();
  if (blockIdx.x == 0)
    for (int e = threadIdx.x; e <= E; e += blockDim.x) offsets[e] = off[e];
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int e = topk_idx[i];
  if (e < 0 || e >= E) return;
  const int p = off[e] + inv[i];
  inv[i] = p;
  order[p] = i;
}

}  // namespace nf

using namespace nf;

template <typename T, int TT>
static int launch_logits(const void* x, const float* wr, int T_, int hidden, int rows, float* logits,
                         cudaStream_t stream) {
  const size_t smem = (size_t)TT * hidden * sizeof(float);
  static size_t allowed = 48 * 1024;      // raised once per size, outside any stream capture
  if (smem > allowed) {
    cudaFuncSetAttribute(router_logits_kernel<T, TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    allowed = smem;
  }
  dim3 grid((rows + 7) / 8, (T_ + TT - 1) / TT);
  NF_REQUIRE(grid.y <= 65535, "router: too many tokens in one call (%d)", T_);
  router_logits_kernel<T, TT><<<grid, 256, smem, stream>>>((const T*)x, wr, T_, hidden, rows, logits);
  return check_launch("router_logits");
}

template <typename T>
static int launch_logits_t(const void* x, const float* wr, int T_, int hidden, int rows, float* logits,
                           cudaStream_t stream) {
  // tokens per block: as many as fit shared memory, to read the router matrix fewer times
  if (T_ > 128 && (size_t)8 * hidden * 4 <= 160 * 1024) return launch_logits<T, 8>(x, wr, T_, hidden, rows, logits, stream);
  if (T_ > 8 && (size_t)2 * hidden * 4 <= 160 * 1024) return launch_logits<T, 2>(x, wr, T_, hidden, rows, logits, stream);
  return launch_logits<T, 1>(x, wr, T_, hidden, rows, logits, stream);
}

// logits: float32 scratch [T, E + extra], also an output (the raw router logits).
extern "C" int nf_router_topk(const void* x, const float* wr, int T, int hidden, int E, int extra,
                              int k, int norm_topk, float* logits, int* topk_idx, float* topk_w,
                              float* extra_out, int dtype, cudaStream_t stream) {
  if (T == 0) return 0;
  NF_REQUIRE(T > 0 && hidden > 0 && E > 0 && k > 0 && k <= E && extra >= 0, "router: bad sizes T=%d hidden=%d E=%d k=%d", T, hidden, E, k);
  NF_REQUIRE((size_t)hidden * 4 <= 200 * 1024, "router: hidden=%d needs more shared memory than a block has", hidden);
  NF_REQUIRE((size_t)4 * E * 4 <= 48 * 1024, "router: %d experts are more than the selection kernel holds (3072)", E);
  int rc = dtype == kF32 ? launch_logits_t<float>(x, wr, T, hidden, E + extra, logits, stream)
                         : launch_logits_t<__nv_bfloat16>(x, wr, T, hidden, E + extra, logits, stream);
  if (rc) return rc;
  router_select_kernel<<<(T + 3) / 4, 128, (size_t)4 * E * sizeof(float), stream>>>(logits, E + extra, 1, T, E, extra, k, norm_topk, topk_idx, topk_w, extra_out);
  return check_launch("router_select");
}

// Few tokens: logits + selection + plan in one launch.  Needs max(hidden, 8 * E, E + 1 + T * k / 2 + 1)
// floats of shared memory; `ticket` is a zeroed int that the kernel leaves zeroed.
extern "C" int nf_router_fused(const void* x, const float* wr, int T, int hidden, int E, int extra, int k,
                               int norm_topk, float* logits, int* topk_idx, float* topk_w,
                               float* extra_out, int* offsets, int* order, int* inv, int* active,
                               int n_active_max, int* ticket, int dtype, cudaStream_t stream) {
  if (T == 0) return 0;
  NF_REQUIRE(T > 0 && T <= 65535 && hidden > 0 && E > 0 && k > 0 && k <= E && extra >= 0, "router: bad sizes T=%d hidden=%d E=%d k=%d", T, hidden, E, k);
  size_t words = (size_t)hidden;
  if ((size_t)8 * E > words) words = (size_t)8 * E;
  if ((size_t)E + 2 + (size_t)T * k / 2 > words) words = (size_t)E + 2 + (size_t)T * k / 2;
  const size_t smem = words * sizeof(float);
  NF_REQUIRE(smem <= 160 * 1024 && E < 65536, "router: sizes too large for the fused kernel");
  static size_t allowed_f = 48 * 1024, allowed_b = 48 * 1024;
  dim3 grid((E + extra + 7) / 8, T);
  if (dtype == kF32) {
    if (smem > allowed_f) { cudaFuncSetAttribute(router_fused_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); allowed_f = smem; }
    launch_chained(router_fused_kernel<float>, grid, dim3(256), smem, stream, (const float*)x, wr, T, hidden, E, extra, k, norm_topk, logits, topk_idx, topk_w, extra_out, offsets, order, inv, active, n_active_max, ticket);
  } else {
    if (smem > allowed_b) { cudaFuncSetAttribute(router_fused_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); allowed_b = smem; }
    launch_chained(router_fused_kernel<__nv_bfloat16>, grid, dim3(256), smem, stream, (const __nv_bfloat16*)x, wr, T, hidden, E, extra, k, norm_topk, logits, topk_idx, topk_w, extra_out, offsets, order, inv, active, n_active_max, ticket);
  }
  return check_launch("router_fused");
}

// The same by one cluster of 8 CTAs (see router_cluster_kernel); `logits` may be null.  Takes what
// fits its shared memory: 0 if (T, hidden, E, k) do, so that the caller can fall back.
extern "C" int nf_router_cluster_fits(int T, int hidden, int E, int extra, int k) {
  const size_t words = (size_t)T * hidden + (size_t)T * (E + extra) + (size_t)8 * E + (size_t)E + 1 + (size_t)T * k +
                       ((size_t)T * k + 1) / 2;
  return T > 0 && T <= 32 && E < 65536 && words * sizeof(float) <= 180 * 1024 ? 1 : 0;
}

extern "C" int nf_router_cluster(const void* x, const float* wr, int T, int hidden, int E, int extra, int k,
                                 int norm_topk, float* logits, int* topk_idx, float* topk_w,
                                 float* extra_out, int* offsets, int* order, int* inv, int* active,
                                 int n_active_max, int dtype, cudaStream_t stream) {
  if (T == 0) return 0;
  NF_REQUIRE(T > 0 && hidden > 0 && E > 0 && k > 0 && k <= E && extra >= 0, "router: bad sizes T=%d hidden=%d E=%d k=%d", T, hidden, E, k);
  NF_REQUIRE(nf_router_cluster_fits(T, hidden, E, extra, k), "router: sizes too large for the cluster kernel");
  const size_t words = (size_t)T * hidden + (size_t)T * (E + extra) + (size_t)8 * E + (size_t)E + 1 + (size_t)T * k +
                       ((size_t)T * k + 1) / 2;
  const size_t smem = words * sizeof(float);
  static size_t allowed_f = 48 * 1024, allowed_b = 48 * 1024;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(kRouterCluster);
  cfg.blockDim = dim3(256);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  // The routed experts wait for this small kernel while the shared expert's large one, launched
  // at the same moment on another stream, would fill every SM first: ask for the highest launch
  // priority, so that these 8 CTAs are placed before that kernel's.
  static int top_priority = 1;
  if (top_priority == 1) {
    int least = 0, greatest = 0;
    cudaDeviceGetStreamPriorityRange(&least, &greatest);
    top_priority = greatest;
  }
  cudaLaunchAttribute attrs[3];
  attrs[0].id = cudaLaunchAttributeClusterDimension;
  attrs[0].val.clusterDim.x = kRouterCluster;
  attrs[0].val.clusterDim.y = 1;
  attrs[0].val.clusterDim.z = 1;
  attrs[1].id = cudaLaunchAttributePriority;
  attrs[1].val.priority = top_priority;
  attrs[2].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attrs[2].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attrs;
  cfg.numAttrs = chain_this_launch(NF_CHAIN_CLASS, stream) ? 3 : 2;
  cudaError_t e;
  if (dtype == kF32) {
    if (smem > allowed_f) { cudaFuncSetAttribute(router_cluster_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); allowed_f = smem; }
    e = cudaLaunchKernelEx(&cfg, router_cluster_kernel<float>, (const float*)x, wr, T, hidden, E, extra, k, norm_topk,
                           logits, topk_idx, topk_w, extra_out, offsets, order, inv, active, n_active_max);
  } else {
    if (smem > allowed_b) { cudaFuncSetAttribute(router_cluster_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); allowed_b = smem; }
    e = cudaLaunchKernelEx(&cfg, router_cluster_kernel<__nv_bfloat16>, (const __nv_bfloat16*)x, wr, T, hidden, E, extra, k,
                           norm_topk, logits, topk_idx, topk_w, extra_out, offsets, order, inv, active, n_active_max);
  }
  if (e != cudaSuccess) note_launch_error(e);
  return check_launch("router_cluster");
}

// Selection alone, from float32 logits that something else has produced: logits[t, e] at
// t * tok_stride + e * exp_stride ([T, E + extra] row-major: strides (E + extra, 1); transposed:
// (1, T)).
extern "C" int nf_router_select(const float* logits, long long tok_stride, long long exp_stride, int T,
                                int E, int extra, int k, int norm_topk, int* topk_idx, float* topk_w,
                                float* extra_out, cudaStream_t stream) {
  if (T == 0) return 0;
  NF_REQUIRE(T > 0 && E > 0 && k > 0 && k <= E && extra >= 0, "router: bad sizes T=%d E=%d k=%d", T, E, k);
  NF_REQUIRE((size_t)4 * E * 4 <= 48 * 1024, "router: %d experts are more than the selection kernel holds (3072)", E);
  launch_chained(router_select_kernel, dim3((T + 3) / 4), dim3(128), (size_t)4 * E * sizeof(float), stream, logits, (long)tok_stride, (long)exp_stride, T, E, extra, k, norm_topk, topk_idx, topk_w, extra_out);
  return check_launch("router_select");
}

// counts: int32 scratch [E] (may be null: then one block does everything).
// active / n_active_max: optional list of the experts that have pairs (ascending, -1 padded).
extern "C" int nf_moe_plan(const int* topk_idx, int n, int E, int* offsets, int* order, int* inv,
                           int* counts, int* active, int n_active_max, cudaStream_t stream) {
  NF_REQUIRE(n >= 0 && E > 0 && E <= 8192, "moe_plan: bad sizes n=%d E=%d", n, E);
  if (n > 2048 && counts) {
    launch_chained(moe_rank_kernel, dim3(E), dim3(1024), 0, stream, topk_idx, n, counts, inv);
    if (int rc = check_launch("moe_rank")) return rc;
    launch_chained(moe_scatter_kernel, dim3((n + 255) / 256), dim3(256), (E + 1) * sizeof(int), stream, topk_idx, n, E, (const int*)counts, offsets, order, inv, active, n_active_max);
    return check_launch("moe_scatter");
  }
  const size_t staged = (size_t)(E + 1) * sizeof(int) + (size_t)n * sizeof(unsigned short);
  if (E < 65536 && staged <= 160 * 1024) {
    static size_t allowed = 48 * 1024;
    if (staged > allowed) {
      cudaFuncSetAttribute(moe_plan_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)staged);
      allowed = staged;
    }
    moe_plan_kernel<true><<<1, 1024, staged, stream>>>(topk_idx, n, E, offsets, order, inv, active, n_active_max);
  } else {
    moe_plan_kernel<false><<<1, 1024, (E + 1) * sizeof(int), stream>>>(topk_idx, n, E, offsets, order, inv, active, n_active_max);
  }
  return check_launch("moe_plan");
}
