// Device functions of the routing that more than one kernel file uses: the lane's share of a
// router logit, the selection of a token's experts, and the plan of a step by one block.
// (Reference: ``moe_route_cpu``, src/ops/moe.hip:49-106, does these steps on the host.)
#pragma once

#include "common.cuh"

namespace nf {

// A lane's share of a dot product in four partial sums, added as (s0 + s1) + (s2 + s3): with a
// width that is a multiple of 4, elements 4 lane .. 4 lane + 3 of every 128; else elements lane,
// lane + 32, ...  Every router kernel
// uses this, so a logit's value does not depend on which of them computed it.
__device__ __forceinline__ float lane_dot(const float* __restrict__ xs, const float* __restrict__ w,
                                          int hidden, int lane) {
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  if ((hidden & 3) == 0 && ((uintptr_t)w & 15) == 0) {
    // 16 bytes a lane a step; eight steps asked for before the first is used, so that the
    // whole row is two round trips to memory, not sixteen
#pragma unroll 8
    for (int i = lane * 4; i < hidden; i += 128) {
      const float4 wv = *reinterpret_cast<const float4*>(w + i);
      const float4 xv = *reinterpret_cast<const float4*>(xs + i);
      s0 = fmaf(xv.x, wv.x, s0);
      s1 = fmaf(xv.y, wv.y, s1);
      s2 = fmaf(xv.z, wv.z, s2);
      s3 = fmaf(xv.w, wv.w, s3);
    }
    return (s0 + s1) + (s2 + s3);
  }
  int i = lane;
  for (; i + 96 < hidden; i += 128) {
    const float w0 = w[i], w1 = w[i + 32], w2 = w[i + 64], w3 = w[i + 96];
    s0 = fmaf(xs[i], w0, s0);
    s1 = fmaf(xs[i + 32], w1, s1);
    s2 = fmaf(xs[i + 64], w2, s2);
    s3 = fmaf(xs[i + 96], w3, s3);
  }
  if (i < hidden) s0 = fmaf(xs[i], w[i], s0);
  if (i + 32 < hidden) s1 = fmaf(xs[i + 32], w[i + 32], s1);
  if (i + 64 < hidden) s2 = fmaf(xs[i + 64], w[i + 64], s2);
  return (s0 + s1) + (s2 + s3);
}

// One warp, one token: softmax over the E router logits, the k largest (ties to the lower
// index), weights p_e or p_e / sum(selected).  `lg` is E floats of the warp's shared memory;
// logits[t, e] sits at row[e * exp_stride].
// GLOBAL: the logits are in global memory, written by other blocks of this launch (read past
// L1); otherwise they are in this block's shared memory.  `chosen`, if given, also receives the
// k selected experts of the token as 16-bit ids (shared memory, for a plan in the same block).
// topk_idx / topk_w / extra_out may be null: a block that only needs `chosen`.
template <bool GLOBAL = true>
__device__ __forceinline__ void select_token(const float* row, long exp_stride, float* lg, int t, int E,
                                             int extra, int k, int norm_topk, int* __restrict__ topk_idx,
                                             float* __restrict__ topk_w, float* __restrict__ extra_out,
                                             int lane, unsigned short* chosen = nullptr) {
  // (the further rows' logits are asked for together with the experts', and stored once those are in)
  const bool has_extra = extra_out && lane < extra;
  float extra_v = 0.f;
  if (has_extra) {
    const float* p = row + (size_t)(E + lane) * exp_stride;
    extra_v = GLOBAL ? __ldcg(p) : *p;
  }
  float mx = -INFINITY;
  for (int e = lane; e < E; e += 32) {
    const float* p = row + (size_t)e * exp_stride;
    const float v = GLOBAL ? __ldcg(p) : *p;
    lg[e] = v;
    mx = fmaxf(mx, v);
  }
  mx = warp_max(mx);
  if (has_extra) extra_out[(size_t)t * extra + lane] = extra_v;
  if (extra_out)
    for (int g = lane + 32; g < extra; g += 32) {
      const float* p = row + (size_t)(E + g) * exp_stride;
      extra_out[(size_t)t * extra + g] = GLOBAL ? __ldcg(p) : *p;
    }
  // A logit that is not a number (a broken checkpoint, an overflow upstream) must not become an
  // index: such a probability counts as zero in the selection, so the k experts chosen are
  // always valid ones, and the row's weights are made NaN so that its output shows the fault
  // instead of hiding it.
  bool bad = false;
  float sum = 0.f;
  for (int e = lane; e < E; e += 32) {
    float p = expf(lg[e] - mx);
    if (!(p >= 0.f && p <= 1.f)) { p = 0.f; bad = true; }
    lg[e] = p;
    sum += p;
  }
  sum = warp_sum(sum);
  bad = __any_sync(0xffffffffu, bad) || !(sum > 0.f);
  if (bad) sum = 1.f;
  __syncwarp();
  float sel_sum = 0.f;
  for (int j0 = 0; j0 < k; j0 += 32) {
    // lane j - j0 keeps the weight of choice j until the sum of the selected is known
    float mine = 0.f;
    const int j1 = min(k, j0 + 32);
    for (int j = j0; j < j1; ++j) {
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
      // (k <= E and every probability is >= 0 > -1, and a taken one is -2: best_e is a valid expert)
      if (lane == 0) {
        if (topk_idx) topk_idx[(size_t)t * k + j] = best_e;
        if (chosen) chosen[(size_t)t * k + j] = (unsigned short)best_e;
        lg[best_e] = -2.f;                           // taken
      }
      if (lane == j - j0) mine = bad ? __int_as_float(0x7fc00000) : best / sum;
      sel_sum += best / sum;
      __syncwarp();
    }
    if (topk_w && !norm_topk && j0 + lane < j1) topk_w[(size_t)t * k + j0 + lane] = mine;
    if (norm_topk && k <= 32) {
      if (topk_w && lane < k) topk_w[(size_t)t * k + lane] = mine / sel_sum;
    } else if (topk_w && norm_topk && j0 + lane < j1) {
      topk_w[(size_t)t * k + j0 + lane] = mine;      // more than 32 choices: divided below, once all are known
    }
  }
  if (norm_topk && k > 32 && topk_w) {
    __syncwarp();
    for (int j = lane; j < k; j += 32) topk_w[(size_t)t * k + j] /= sel_sum;
  }
  __syncwarp();
}

// Plan by one block: stable counting sort of the n pairs by expert, and (if `active` is
// given) the list of experts that have pairs, ascending, padded with -1 to n_active_max.  `counts` is E + 1 ints
// of shared memory; with STAGED, `ex` holds n 16-bit expert ids so that the E passes over the
// pairs do not go to global memory.
template <bool STAGED>
__device__ __forceinline__ void plan_block(const int* __restrict__ topk_idx, int n, int E,
                                           int* __restrict__ offsets, int* __restrict__ order,
                                           int* __restrict__ inv, int* counts, unsigned short* ex,
                                           int* __restrict__ active, int n_active_max) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
  if (STAGED) {
    for (int i = threadIdx.x; i < n; i += blockDim.x) ex[i] = (unsigned short)__ldcg(topk_idx + i);
    __syncthreads();
  }
  for (int e = warp; e < E; e += nwarp) {
    int running = 0;
    for (int base = 0; base < n; base += 32) {
      const int i = base + lane;
      const bool mine = i < n && (STAGED ? (int)ex[i] : topk_idx[i]) == e;
      const unsigned b = __ballot_sync(0xffffffffu, mine);
      if (mine) inv[i] = running + __popc(b & ((1u << lane) - 1u));   // rank inside the expert
      running += __popc(b);
    }
    if (lane == 0) counts[e] = running;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0, na = 0;
    for (int e = 0; e < E; ++e) {
      const int c = counts[e];
      if (c > 0 && active && na < n_active_max) active[na++] = e;
      counts[e] = run;
      offsets[e] = run;
      run += c;
    }
    counts[E] = run;
    offsets[E] = run;
    if (active)
      for (; na < n_active_max; ++na) active[na] = -1;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int e = STAGED ? (int)ex[i] : topk_idx[i];
    if (e < 0 || e >= E) continue;
    const int p = counts[e] + inv[i];
    inv[i] = p;
    order[p] = i;
  }
}

}  // namespace nf
