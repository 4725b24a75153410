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
#include "common.cuh"

namespace nf {

// One block per token.  wr holds `E + extra` rows of `hidden` float32: E router rows and
// `extra` further rows whose logits are returned raw (the shared expert's gate).
template <typename T>
__global__ void __launch_bounds__(128)
router_topk_kernel(const T* __restrict__ x, const float* __restrict__ wr, int hidden, int E,
                   int extra, int k, int norm_topk, int* __restrict__ topk_idx,
                   float* __restrict__ topk_w, float* __restrict__ extra_out) {
  extern __shared__ float smem[];      // [hidden] x, [E + extra] logits -> probabilities
  float* xs = smem;
  float* lg = smem + hidden;
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const T* xr = x + (size_t)t * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) xs[i] = to_float(xr[i]);
  __syncthreads();
  for (int e = warp; e < E + extra; e += 4) {
    const float* w = wr + (size_t)e * hidden;
    float dot = 0.f;
    for (int i = lane; i < hidden; i += 32) dot = fmaf(xs[i], w[i], dot);
    dot = warp_sum(dot);
    if (lane == 0) lg[e] = dot;
  }
  __syncthreads();
  if (warp != 0) return;
  for (int g = lane; g < extra; g += 32) extra_out[(size_t)t * extra + g] = lg[E + g];
  float mx = -INFINITY;
  for (int e = lane; e < E; e += 32) mx = fmaxf(mx, lg[e]);
  mx = warp_max(mx);
  float sum = 0.f;
  for (int e = lane; e < E; e += 32) {
    const float p = expf(lg[e] - mx);
    lg[e] = p;
    sum += p;
  }
  sum = warp_sum(sum);
  __syncwarp();
  float sel_sum = 0.f;
  for (int j = 0; j < k; ++j) {
    float best = -1.f;
    int best_e = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float p = lg[e];
      if (p > best) { best = p; best_e = e; }     // ascending e: first maximum wins
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
    }
    if (lane == 0) {
      topk_idx[(size_t)t * k + j] = best_e;
      topk_w[(size_t)t * k + j] = best / sum;
      lg[best_e] = -2.f;                           // taken
    }
    sel_sum += best / sum;
    __syncwarp();
  }
  if (norm_topk) {
    for (int j = lane; j < k; j += 32) topk_w[(size_t)t * k + j] /= sel_sum;
  }
}

// Plan: stable counting sort of the n = T*k pairs by expert.
//   offsets[e] .. offsets[e+1]  rows of expert e in sorted order
//   order[p] = pair (t*k + j) at sorted position p;   inv[pair] = p
// One block; warp w ranks the pairs of experts w, w + nwarps, ... with ballots, which keeps
// token order inside an expert.
__global__ void __launch_bounds__(1024)
moe_plan_kernel(const int* __restrict__ topk_idx, int n, int E, int* __restrict__ offsets,
                int* __restrict__ order, int* __restrict__ inv) {
  extern __shared__ int counts[];      // [E + 1]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
  for (int e = warp; e < E; e += nwarp) {
    int running = 0;
    for (int base = 0; base < n; base += 32) {
      const int i = base + lane;
      const bool mine = i < n && topk_idx[i] == e;
      const unsigned b = __ballot_sync(0xffffffffu, mine);
      if (mine) inv[i] = running + __popc(b & ((1u << lane) - 1u));   // rank inside the expert
      running += __popc(b);
    }
    if (lane == 0) counts[e] = running;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < E; ++e) {
      const int c = counts[e];
      counts[e] = run;
      offsets[e] = run;
      run += c;
    }
    counts[E] = run;
    offsets[E] = run;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int e = topk_idx[i];
    if (e < 0 || e >= E) continue;
    const int p = counts[e] + inv[i];
    inv[i] = p;
    order[p] = i;
  }
}

}  // namespace nf

using namespace nf;

extern "C" int nf_router_topk(const void* x, const float* wr, int T, int hidden, int E, int extra,
                              int k, int norm_topk, int* topk_idx, float* topk_w,
                              float* extra_out, int dtype, cudaStream_t stream) {
  if (T == 0) return 0;
  NF_REQUIRE(T > 0 && hidden > 0 && E > 0 && k > 0 && k <= E && extra >= 0, "router: bad sizes T=%d hidden=%d E=%d k=%d", T, hidden, E, k);
  const size_t smem = (size_t)(hidden + E + extra) * sizeof(float);
  NF_REQUIRE(smem <= 200 * 1024, "router: hidden=%d with %d experts needs %zu bytes of shared memory (limit 200 KiB)", hidden, E, smem);
  if (dtype == kF32) {
    static size_t allowed = 48 * 1024;      // raised once per size, outside any stream capture
    if (smem > allowed) { cudaFuncSetAttribute(router_topk_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); allowed = smem; }
    router_topk_kernel<float><<<T, 128, smem, stream>>>((const float*)x, wr, hidden, E, extra, k, norm_topk, topk_idx, topk_w, extra_out);
  } else {
    static size_t allowed = 48 * 1024;
    if (smem > allowed) { cudaFuncSetAttribute(router_topk_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); allowed = smem; }
    router_topk_kernel<__nv_bfloat16><<<T, 128, smem, stream>>>((const __nv_bfloat16*)x, wr, hidden, E, extra, k, norm_topk, topk_idx, topk_w, extra_out);
  }
  return check_launch("router_topk");
}

extern "C" int nf_moe_plan(const int* topk_idx, int n, int E, int* offsets, int* order, int* inv,
                           cudaStream_t stream) {
  NF_REQUIRE(n >= 0 && E > 0 && E <= 8192, "moe_plan: bad sizes n=%d E=%d", n, E);
  moe_plan_kernel<<<1, 1024, (E + 1) * sizeof(int), stream>>>(topk_idx, n, E, offsets, order, inv);
  return check_launch("moe_plan");
}
