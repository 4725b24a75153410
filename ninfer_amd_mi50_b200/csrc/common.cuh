// Shared device helpers and the host-side error convention of the kernel library.
//
// Every exported launcher is `extern "C" int nf_<name>(...)`: 0 on success, non-zero
// after a refused argument or a failed launch, with the reason kept for
// nf_last_error().  The reference reports device errors by throwing from HIP_CHECK
// (src/core/device.h:15-25); a C ABI cannot throw, so it uses codes like the
// reference's C API does (src/api/ninfer_c_api.cpp:78-81).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace nf {

enum DType : int { kF32 = 0, kBF16 = 1 };

void set_error(const char* fmt, ...);
int check_launch(const char* what);
void note_launch_error(cudaError_t e);

// Programmatic dependent launch.  A kernel launched through `launch_chained` may begin while
// the kernel before it in the stream is still draining: its CTAs are scheduled as soon as every
// CTA of the predecessor has started (each calls `chain_release` first thing), do whatever does
// not depend on the predecessor (index arithmetic, fetching weights), and then block in
// `chain_wait` until the predecessor has completed and its writes are visible.  That hides the
// launch and ramp-up of the many short kernels of a decode step.  Kernels launched the ordinary
// way are unaffected; for them both calls do nothing.
// nf_chain_break(): the next launch through `launch_chained` (by this thread) is an ordinary one.
// For the first kernel after a wait on another stream's event: its dependency is then not the
// kernel before it in its own stream, and a programmatic edge does not describe it.
bool take_chain_break();
// Whether a launch of class `cls` on `stream` gets the attribute: the class is switched on and no
// break is pending.  (It used to be given only while the stream was being captured: driven from
// the host, one decode step in some ten thousand came out different.  That was the stale read
// through the non-coherent path that skinny_gemm.cu describes, not the attribute; with it gone,
// 48,000 host-driven steps run twice agree bit for bit, and a prompt of 2,048 tokens, whose
// kernels are launched one by one from the host, is 2 % faster.)
bool chain_this_launch(int cls, cudaStream_t stream);
extern int g_chained_launch;   // nf_set_chained_launch(): a mask over NF_CHAIN_CLASS bits; 0 turns the attribute off
#ifndef NF_CHAIN_CLASS
#define NF_CHAIN_CLASS 0x40     // a source file may name its class before including this header
#endif
#ifdef NF_CHAIN_EARLY_RELEASE
__device__ __forceinline__ void chain_release() { asm volatile("griddepcontrol.launch_dependents;"); }
#else
// Measured on B200: releasing at the top of every kernel made decode steps 20-25 % slower (the
// successors' CTAs sit on the SMs spinning while the predecessor still needs them), so the
// release is left to the implicit one at kernel exit; the attribute then only lets the next
// launch be prepared early.
__device__ __forceinline__ void chain_release() {}
#endif
// A release at the top of a kernel that does not fill the device (a norm over 8 rows, the merge
// of a decode step): its successor's CTAs find free SMs anyway, become resident at once and ask
// for their first weights while this kernel's few CTAs work through their latency chain.
__device__ __forceinline__ void chain_release_if_small() {
  if (gridDim.x * gridDim.y * gridDim.z <= 148u) asm volatile("griddepcontrol.launch_dependents;");
}
// A release late in a kernel, once its CTA has asked for all it will read: the successor's
// CTAs then arrive while this one reduces and writes.
__device__ __forceinline__ void chain_release_late() { asm volatile("griddepcontrol.launch_dependents;"); }
__device__ __forceinline__ void chain_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// The wait, and then every pointer through which the kernel will read what earlier kernels
// wrote is passed through an empty asm statement.  Loads through `const __restrict__` pointers
// are "invariant" to the compiler (ld.global.nc), and a compiler may move invariant loads above
// barriers; a load of the predecessor's output issued before the wait would read it
// half-written.  A pointer that comes out of an asm statement is a new value to the compiler,
// and a load cannot be issued before its address exists.  A precaution: no such move was seen.
template <typename T>
__device__ __forceinline__ void chain_fresh(T& p) {          // T: a pointer type, qualifiers and all
  static_assert(sizeof(T) == 8, "chain_fresh takes pointers");
  asm volatile("" : "+l"(p)::"memory");
}
template <typename... P>
__device__ __forceinline__ void chain_wait(P&... ptrs) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  (chain_fresh(ptrs), ...);
}

template <typename... KArgs, typename... Args>
inline void launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                           Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = chain_this_launch(NF_CHAIN_CLASS, stream) ? 1 : 0;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
  if (e != cudaSuccess) note_launch_error(e);     // check_launch reports it even if the runtime
                                                  // did not keep it as its last error
}

// The same with the CTAs launched as clusters of `cluster_x` consecutive blocks of grid.x.
template <typename... KArgs, typename... Args>
inline void launch_chained_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                   int cluster_x, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  attrs[0].id = cudaLaunchAttributeClusterDimension;
  attrs[0].val.clusterDim.x = cluster_x;
  attrs[0].val.clusterDim.y = 1;
  attrs[0].val.clusterDim.z = 1;
  attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attrs[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attrs;
  cfg.numAttrs = chain_this_launch(NF_CHAIN_CLASS, stream) ? 2 : 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
  if (e != cudaSuccess) note_launch_error(e);
}

#define NF_REQUIRE(cond, ...)            \
  do {                                   \
    if (!(cond)) {                       \
      nf::set_error(__VA_ARGS__);        \
      return 1;                          \
    }                                    \
  } while (0)

template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  `red` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarp = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarp ? red[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

// 4 consecutive elements as floats, and back.
__device__ __forceinline__ void load4(const float* p, float* v) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
}
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float* v) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
  const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
__device__ __forceinline__ void store4(float* p, const float* v) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, const float* v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
  uint2 raw;
  raw.x = *reinterpret_cast<unsigned*>(&a);
  raw.y = *reinterpret_cast<unsigned*>(&b);
  *reinterpret_cast<uint2*>(p) = raw;
}

// 8 consecutive bfloat16 (16 bytes) or 4 consecutive floats (16 bytes) as floats.
__device__ __forceinline__ void unpack8(const uint4& raw, float* out) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __bfloat1622float2(h[i]);
    out[2 * i] = f.x;
    out[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float* out) {
  uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __bfloat1622float2(h[i]);
    out[2 * i] = f.x;
    out[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ void load8(const float* p, float* out) {
  float4 a = *reinterpret_cast<const float4*>(p);
  float4 b = *reinterpret_cast<const float4*>(p + 4);
  out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
  out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
}

}  // namespace nf
