// Sampling on the device: greedy argmax, and temperature / top-k / top-p draws.
//
// Policy of the reference's ``sample_logits`` (src/runtime/engine.cpp:18-82), which runs on
// the host after copying the vocabulary's logits back: repetition penalty (v > 0 ? v / p :
// v * p for every recent id) -> greedy first maximum if temperature <= 0 -> logits /
// temperature -> keep the k largest -> softmax over them -> smallest prefix (in descending
// order) whose mass reaches top_p, renormalised -> the first candidate whose running sum
// reaches a uniform draw r.  Here one block per row does the same without leaving the
// device; the draw r comes from the host, so that a host twin given the same logits and
// the same r picks the same token.
//
// Two forms: `k <= 1024` keeps the candidates in shared memory, sorted (ties: lower id
// first), exactly as above.  With no top-k limit (k >= vocab) and top_p >= 1 the draw walks
// the vocabulary in id order instead of sorted order: the same distribution, without a
// sort of the whole vocabulary.
#include "common.cuh"

namespace nf {

__global__ void __launch_bounds__(1024)
argmax_rows_kernel(const float* __restrict__ logits, int V, int* __restrict__ out) {
  __shared__ float sv[32];
  __shared__ int si[32];
  const float* row = logits + (size_t)blockIdx.x * V;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = row[i];
    if (v > best || (v == best && i < bi)) { best = v; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { sv[warp] = best; si[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    best = lane < nw ? sv[lane] : -INFINITY;
    bi = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) out[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;   // all NaN: token 0
  }
}

// The same over a long row in two steps: the row is cut into `chunks` pieces, a block per piece
// writes its first maximum (value and index), and a warp per row picks the first maximum among
// the pieces.  One block per row reads a 600 KB row of a large vocabulary alone for 40 us; cut
// into pieces the whole device reads it.
__global__ void __launch_bounds__(256)
argmax_partial_kernel(const float* __restrict__ logits, int V, int chunk, float* __restrict__ pv,
                      int* __restrict__ pi) {
  __shared__ float sv[8];
  __shared__ int si[8];
  const int r = blockIdx.y, c = blockIdx.x;
  const float* row = logits + (size_t)r * V;
  const int lo = c * chunk, hi = min(V, lo + chunk);
  float best = -INFINITY;
  int bi = 0x7fffffff;
  // ascending indices per thread, so "greater than" keeps the first of equal values
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const float v = row[i];
    if (v > best) { best = v; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { sv[warp] = best; si[warp] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w)
      if (sv[w] > best || (sv[w] == best && si[w] < bi)) { best = sv[w]; bi = si[w]; }
    pv[(size_t)r * gridDim.x + c] = best;
    pi[(size_t)r * gridDim.x + c] = bi;
  }
}

__global__ void __launch_bounds__(32)
argmax_final_kernel(const float* __restrict__ pv, const int* __restrict__ pi, int chunks, int* __restrict__ out) {
  const int r = blockIdx.x, lane = threadIdx.x;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int c = lane; c < chunks; c += 32) {
    const float v = pv[(size_t)r * chunks + c];
    const int i = pi[(size_t)r * chunks + c];
    if (v > best || (v == best && i < bi)) { best = v; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  if (lane == 0) out[r] = bi == 0x7fffffff ? 0 : bi;   // all NaN: token 0
}

// logits[row, id] = v > 0 ? v / p^count : v * p^count for (id, count) pairs of each row.
__global__ void repetition_penalty_kernel(float* __restrict__ logits, int V,
                                          const int* __restrict__ ids, const int* __restrict__ counts,
                                          const int* __restrict__ row_of, const float* __restrict__ penalty,
                                          int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int id = ids[i], r = row_of[i];
  if (id < 0 || id >= V) return;
  const float p = penalty[r];
  float v = logits[(size_t)r * V + id];
  for (int c = 0; c < counts[i]; ++c) v = v > 0.f ? v / p : v * p;
  logits[(size_t)r * V + id] = v;
}

__device__ __forceinline__ unsigned order_key(float v) {
  // larger float -> larger unsigned; NaN sorts lowest
  if (v != v) return 0u;
  const unsigned u = __float_as_uint(v);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

constexpr int kMaxK = 1024;

// One block of 1024 threads per row.
__global__ void __launch_bounds__(1024)
sample_rows_kernel(const float* __restrict__ logits, int V, const float* __restrict__ temperature,
                   const int* __restrict__ top_k, const float* __restrict__ top_p,
                   const float* __restrict__ draw, int* __restrict__ out) {
  __shared__ unsigned hist[256];
  __shared__ float cand_v[kMaxK];
  __shared__ int cand_i[kMaxK];
  __shared__ float red[33];
  __shared__ unsigned s_prefix, s_remaining;
  __shared__ int s_n_gt, s_n_eq, s_result;
  __shared__ float scan[1024];
  __shared__ int warp_cnt[32];
  const int r = blockIdx.x, tid = threadIdx.x;
  const float* row = logits + (size_t)r * V;
  const float inv_t = 1.f / temperature[r];
  int k = top_k[r];
  k = k < 1 ? 1 : (k > V ? V : k);
  const float tp = top_p[r];
  const float u = draw[r];

  if (k >= V && tp >= 1.f) {
    // ---- whole vocabulary in id order --------------------------------------------------
    float mx = -INFINITY;
    for (int i = tid; i < V; i += blockDim.x) mx = fmaxf(mx, row[i] * inv_t);
    mx = warp_max(mx);
    if ((tid & 31) == 0) red[tid >> 5] = mx;
    __syncthreads();
    if (tid < 32) {
      float t = tid < (blockDim.x >> 5) ? red[tid] : -INFINITY;
      t = warp_max(t);
      if (tid == 0) red[32] = t;
    }
    __syncthreads();
    mx = red[32];
    float sum = 0.f;
    for (int i = tid; i < V; i += blockDim.x) sum += expf(row[i] * inv_t - mx);
    sum = block_sum(sum, red);
    const float target = u * sum;
    // chunks of blockDim.x ids in order; inclusive scan inside a chunk; the pick is the
    // lowest id whose running sum reaches the target
    float base = 0.f;
    if (tid == 0) s_result = 0x7fffffff;
    __syncthreads();
    for (int c0 = 0; c0 < V; c0 += blockDim.x) {
      const int i = c0 + tid;
      const float p = i < V ? expf(row[i] * inv_t - mx) : 0.f;
      scan[tid] = p;
      __syncthreads();
      for (int o = 1; o < blockDim.x; o <<= 1) {
        const float add = tid >= o ? scan[tid - o] : 0.f;
        __syncthreads();
        scan[tid] += add;
        __syncthreads();
      }
      if (i < V && base + scan[tid] >= target) atomicMin(&s_result, i);
      __syncthreads();
      if (s_result != 0x7fffffff) break;
      base += scan[blockDim.x - 1];
      __syncthreads();
    }
    if (tid == 0) out[r] = s_result != 0x7fffffff ? s_result : V - 1;
    return;
  }

  // ---- the k largest: radix select of the k-th key, 8 bits a pass ------------------------
  if (tid == 0) { s_prefix = 0u; s_remaining = (unsigned)k; }
  __syncthreads();
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    if (tid < 256) hist[tid] = 0u;
    __syncthreads();
    const unsigned prefix = s_prefix;
    const unsigned mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
    for (int i = tid; i < V; i += blockDim.x) {
      const unsigned key = order_key(row[i] * inv_t);
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
    }
    __syncthreads();
    if (tid == 0) {
      unsigned rem = s_remaining;
      int d = 255;
      for (; d > 0; --d) {
        if (hist[d] >= rem) break;
        rem -= hist[d];
      }
      s_prefix = prefix | ((unsigned)d << shift);
      s_remaining = rem;
    }
    __syncthreads();
  }
  const unsigned kth = s_prefix;          // key of the k-th largest value
  const int need_eq = (int)s_remaining;   // how many equal to it are kept (lowest ids first)
  if (tid == 0) { s_n_gt = 0; s_n_eq = 0; }
  __syncthreads();
  for (int i = tid; i < V; i += blockDim.x) {
    const float v = row[i] * inv_t;
    if (order_key(v) > kth) {
      const int slot = atomicAdd(&s_n_gt, 1);
      cand_v[slot] = v;
      cand_i[slot] = i;
    }
  }
  __syncthreads();
  const int n_gt = s_n_gt;
  // equals: ids ascending; walked in order so that the lowest ids are the ones kept
  for (int c0 = 0; c0 < V && s_n_eq < need_eq; c0 += blockDim.x) {
    const int i = c0 + tid;
    const bool eq = i < V && order_key(row[i] * inv_t) == kth;
    const unsigned b = __ballot_sync(0xffffffffu, eq);
    if ((tid & 31) == 0) warp_cnt[tid >> 5] = __popc(b);
    __syncthreads();
    int before = s_n_eq;
    for (int w = 0; w < (tid >> 5); ++w) before += warp_cnt[w];
    const int my = before + __popc(b & ((1u << (tid & 31)) - 1u));
    if (eq && my < need_eq) {
      cand_v[n_gt + my] = row[i] * inv_t;
      cand_i[n_gt + my] = i;
    }
    __syncthreads();
    if (tid == 0) {
      int tot = s_n_eq;
      for (int w = 0; w < 32; ++w) tot += warp_cnt[w];
      s_n_eq = tot;
    }
    __syncthreads();
  }
  // pad to 1024 and sort descending by (value, then lower id first): bitonic
  for (int i = tid; i < kMaxK; i += blockDim.x)
    if (i >= k) { cand_v[i] = -INFINITY; cand_i[i] = 0x7fffffff; }
  __syncthreads();
  for (int size = 2; size <= kMaxK; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      const int i = tid, j = i ^ stride;
      if (j > i) {
        const bool desc = (i & size) == 0;
        const float vi = cand_v[i], vj = cand_v[j];
        const int ii = cand_i[i], ij = cand_i[j];
        const bool i_first = vi > vj || (vi == vj && ii < ij);   // i belongs before j in descending order
        if (desc ? !i_first : i_first) {
          cand_v[i] = vj; cand_v[j] = vi;
          cand_i[i] = ij; cand_i[j] = ii;
        }
      }
      __syncthreads();
    }
  }
  // softmax over the k kept, top-p prefix, draw; k <= 1024 so one thread walks them
  if (tid == 0) {
    const float m = cand_v[0];
    float sum = 0.f;
    for (int i = 0; i < k; ++i) sum += expf(cand_v[i] - m);
    int keep = k;
    if (tp < 1.f) {
      float cum = 0.f;
      for (int i = 0; i < k; ++i) {
        cum += expf(cand_v[i] - m) / sum;
        if (cum >= tp) { keep = i + 1; break; }
      }
    }
    float s2 = 0.f;
    for (int i = 0; i < keep; ++i) s2 += expf(cand_v[i] - m) / sum;
    float cum = 0.f;
    int pick = cand_i[keep - 1];
    for (int i = 0; i < keep; ++i) {
      cum += expf(cand_v[i] - m) / sum / s2;
      if (u <= cum) { pick = cand_i[i]; break; }
    }
    out[r] = pick;
  }
}

}  // namespace nf

using namespace nf;

extern "C" int nf_argmax_rows(const float* logits, int R, int V, int* out, cudaStream_t stream) {
  if (R == 0) return 0;
  NF_REQUIRE(R > 0 && V > 0, "argmax: bad sizes R=%d V=%d", R, V);
  argmax_rows_kernel<<<R, 1024, 0, stream>>>(logits, V, out);
  return check_launch("argmax_rows");
}

// Pieces a row is cut into by the two-step form: 1 means "use nf_argmax_rows".
extern "C" int nf_argmax_chunks(int R, int V) {
  if (V < 16384 || R > 4096) return 1;       // short rows, or rows enough to fill the device anyway
  int c = (V + 4095) / 4096;
  return c > 64 ? 64 : c;
}

// scratch_v float32 [R, chunks], scratch_i int32 [R, chunks], chunks = nf_argmax_chunks(R, V) > 1.
extern "C" int nf_argmax_rows_split(const float* logits, int R, int V, int chunks, float* scratch_v,
                                    int* scratch_i, int* out, cudaStream_t stream) {
  if (R == 0) return 0;
  NF_REQUIRE(R > 0 && V > 0 && chunks > 1 && R <= 65535, "argmax: bad sizes R=%d V=%d chunks=%d", R, V, chunks);
  const int chunk = (V + chunks - 1) / chunks;
  argmax_partial_kernel<<<dim3(chunks, R), 256, 0, stream>>>(logits, V, chunk, scratch_v, scratch_i);
  argmax_final_kernel<<<R, 32, 0, stream>>>(scratch_v, scratch_i, chunks, out);
  return check_launch("argmax_rows_split");
}

extern "C" int nf_repetition_penalty(float* logits, int V, const int* ids, const int* counts,
                                     const int* row_of, const float* penalty, int n,
                                     cudaStream_t stream) {
  if (n == 0) return 0;
  repetition_penalty_kernel<<<(n + 255) / 256, 256, 0, stream>>>(logits, V, ids, counts, row_of, penalty, n);
  return check_launch("repetition_penalty");
}

// Host must make sure that every row has temperature > 0 and either top_k <= 1024 or
// (top_k >= V and top_p >= 1).
extern "C" int nf_sample_rows(const float* logits, int R, int V, const float* temperature,
                              const int* top_k, const float* top_p, const float* draw, int* out,
                              cudaStream_t stream) {
  if (R == 0) return 0;
  NF_REQUIRE(R > 0 && V > 0, "sample: bad sizes R=%d V=%d", R, V);
  sample_rows_kernel<<<R, 1024, 0, stream>>>(logits, V, temperature, top_k, top_p, draw, out);
  return check_launch("sample_rows");
}
