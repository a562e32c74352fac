// Shared helpers of the featgraph_b200 kernels: error reporting, unfused fp32
// arithmetic, cache-hinted loads/stores and cp.async wrappers.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>
#include <string>

#include "../../include/featgraph_b200.h"

namespace fg {

// Where a kernel writes its result: the caller's own buffer and, in a multi-GPU run,
// the same position in the buffers of up to seven peers (peer-mapped pointers, plain
// stores over NVLink) -- the "all-gather" then happens inside the kernel's epilogue.
//
// mcast != 0: p[0] is instead a MULTICAST address (an NVLink-switch multicast object that
// maps the same buffer on every GPU of the group, this one included) and n == 1: one
// multimem.st leaves the GPU once and the switch writes every GPU's copy.
// Kernels take it as a `const __grid_constant__` parameter: the loop over p[] then indexes
// the parameter where it lies (constant bank) instead of a per-thread copy in local memory
// -- that copy cost every thread a 72-byte stack frame, whose lines, written back, were
// two thirds of the SpMM's and half of the SDDMM's DRAM writes.
constexpr int kMaxOutputs = 8;
struct OutPtrs {
  float* p[kMaxOutputs];
  int n = 0;
  int mcast = 0;
  // SpMM over column blocks only (out_fold): 0 store the result; 1 store 0 + result (the
  // first block); 2 store what p[0] holds + result (every later block)
  int accumulate = 0;
};

// The flag arrays of fg_peer_barrier, one per rank (peer-mapped pointers), and how long a
// wait polls by default: about a microsecond per poll, so a few seconds.
struct PeerFlags {
  unsigned* p[kMaxOutputs];
};
constexpr unsigned kPeerBarrierPolls = 1u << 22;

// Expands CALL(MSG, RED) for the operator pair (msg_op, reduce_op), both already range-checked.
#define FG_DISPATCH_OPS(msg_op, reduce_op, CALL)                      \
  switch ((msg_op) * 3 + (reduce_op)) {                               \
    case 0: CALL(0, 0); break;   case 1: CALL(0, 1); break;   case 2: CALL(0, 2); break;   \
    case 3: CALL(1, 0); break;   case 4: CALL(1, 1); break;   case 5: CALL(1, 2); break;   \
    case 6: CALL(2, 0); break;   case 7: CALL(2, 1); break;   case 8: CALL(2, 2); break;   \
    case 9: CALL(3, 0); break;   case 10: CALL(3, 1); break;  case 11: CALL(3, 2); break;  \
    case 12: CALL(4, 0); break;  case 13: CALL(4, 1); break;  case 14: CALL(4, 2); break;  \
    case 15: CALL(5, 0); break;  case 16: CALL(5, 1); break;  default: CALL(5, 2); break;  \
  }

// Options of the next kernel-launching call of the calling host thread (fg_next_launch_options).
struct LaunchOptions {
  int flags = 0;
  int max_ctas = 0;
};
LaunchOptions take_launch_options();  // returns them and resets them to none

// ---- host side: per-thread error message -----------------------------------
std::string& last_error();
int fail(int code, const char* fmt, ...);

#define FG_CUDA_TRY(expr)                                                      \
  do {                                                                         \
    cudaError_t fg_err__ = (expr);                                             \
    if (fg_err__ != cudaSuccess)                                               \
      return ::fg::fail(FG_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,           \
                        cudaGetErrorString(fg_err__), __FILE__, __LINE__);     \
  } while (0)

// Switches the current device for the lifetime of the object.
struct DeviceGuard {
  int prev = -1;
  bool changed = false;
  cudaError_t status = cudaSuccess;
  explicit DeviceGuard(int device) {
    status = cudaGetDevice(&prev);
    if (status == cudaSuccess && prev != device) {
      status = cudaSetDevice(device);
      changed = (status == cudaSuccess);
    }
  }
  ~DeviceGuard() {
    if (changed) cudaSetDevice(prev);
  }
};

// ---- device side -------------------------------------------------------------
#ifdef __CUDACC__

// acc + a * b with the product rounded to fp32 before the sum: the arithmetic
// of a code generator that does not contract into FMA.
__device__ __forceinline__ float mul_then_add(float acc, float a, float b) {
  return __fadd_rn(acc, __fmul_rn(a, b));
}

// The same for two adjacent features: scalar products, one packed fp32x2 add
// (Blackwell's add.f32x2).  The products are deliberately NOT a packed
// mul.f32x2: ptxas 12.9 contracts a single-use packed multiply feeding a packed
// add into a packed FMA even though both carry .rn (measured: 20 % of random
// results differ from the unfused ones), which would break bit-parity.
__device__ __forceinline__ float2 mul_then_add2(float2 acc, float a, float2 b) {
  return __fadd2_rn(acc, make_float2(__fmul_rn(a, b.x), __fmul_rn(a, b.y)));
}

// ---- generalised message / reduce operators ------------------------------------
// msg(lhs, rhs) and acc <- reduce(acc, msg); the operator numbers are those of the C ABI
// (fg_msg_op / fg_reduce_op).  Every operation is a single correctly rounded fp32
// instruction, never contracted; max / min are comparisons that keep the accumulator on a
// tie and never take a NaN, so a walk in order gives the same bits as a sequential loop.
template <int MSG>
__device__ __forceinline__ float msg_apply(float lhs, float rhs) {
  if (MSG == FG_MSG_MUL) return __fmul_rn(lhs, rhs);
  if (MSG == FG_MSG_ADD) return __fadd_rn(lhs, rhs);
  if (MSG == FG_MSG_SUB) return __fsub_rn(lhs, rhs);
  if (MSG == FG_MSG_DIV) return __fdiv_rn(lhs, rhs);
  if (MSG == FG_MSG_COPY_LHS) return lhs;
  return rhs;
}
template <int RED>
__device__ __forceinline__ float red_apply(float acc, float m) {
  if (RED == FG_REDUCE_SUM) return __fadd_rn(acc, m);
  if (RED == FG_REDUCE_MAX) return m > acc ? m : acc;
  return m < acc ? m : acc;
}
template <int RED>
__device__ __forceinline__ float red_identity() {
  if (RED == FG_REDUCE_SUM) return 0.f;
  // the lowest / highest finite fp32 value
  return __int_as_float(RED == FG_REDUCE_MAX ? 0xff7fffff : 0x7f7fffff);
}
template <int MSG, int RED>
__device__ __forceinline__ float combine(float acc, float lhs, float rhs) {
  return red_apply<RED>(acc, msg_apply<MSG>(lhs, rhs));
}

// Streaming (read-once) loads of the adjacency arrays.
__device__ __forceinline__ int ld_stream(const int* p) { return __ldcs(p); }
__device__ __forceinline__ float ld_stream(const float* p) { return __ldcs(p); }

// Read-only gathers of feature rows.
__device__ __forceinline__ float4 ld_gather4(const float* p) {
  return __ldg(reinterpret_cast<const float4*>(p));
}

__device__ __forceinline__ void st_stream4(float* p, float4 v) {
  __stcs(reinterpret_cast<float4*>(p), v);
}

// ---- result stores: every listed buffer, or one multicast store ---------------
// The running sum over column blocks: the value to store for a result `v` at `off`.
__device__ __forceinline__ float out_fold(const OutPtrs& o, size_t off, float v) {
  if (o.accumulate == 0) return v;
  return __fadd_rn(o.accumulate == 2 ? o.p[0][off] : 0.0f, v);
}
__device__ __forceinline__ float2 out_fold(const OutPtrs& o, size_t off, float2 v) {
  if (o.accumulate == 0) return v;
  float2 prev = make_float2(0.f, 0.f);
  if (o.accumulate == 2) prev = *reinterpret_cast<const float2*>(o.p[0] + off);
  return make_float2(__fadd_rn(prev.x, v.x), __fadd_rn(prev.y, v.y));
}
__device__ __forceinline__ float4 out_fold(const OutPtrs& o, size_t off, float4 v) {
  if (o.accumulate == 0) return v;
  float4 prev = make_float4(0.f, 0.f, 0.f, 0.f);
  if (o.accumulate == 2) prev = *reinterpret_cast<const float4*>(o.p[0] + off);
  return make_float4(__fadd_rn(prev.x, v.x), __fadd_rn(prev.y, v.y), __fadd_rn(prev.z, v.z),
                     __fadd_rn(prev.w, v.w));
}
__device__ __forceinline__ void out_store(const OutPtrs& o, size_t off, float v) {
  if (o.mcast) {
    asm volatile("multimem.st.relaxed.sys.global.f32 [%0], %1;" ::"l"(o.p[0] + off), "f"(v)
                 : "memory");
    return;
  }
  for (int q = 0; q < o.n; ++q) __stcs(o.p[q] + off, v);
}
__device__ __forceinline__ void out_store(const OutPtrs& o, size_t off, float2 v) {
  if (o.mcast) {
    asm volatile("multimem.st.relaxed.sys.global.v2.f32 [%0], {%1,%2};" ::"l"(o.p[0] + off),
                 "f"(v.x), "f"(v.y)
                 : "memory");
    return;
  }
  for (int q = 0; q < o.n; ++q) __stcs(reinterpret_cast<float2*>(o.p[q] + off), v);
}
__device__ __forceinline__ void out_store(const OutPtrs& o, size_t off, float4 v) {
  if (o.mcast) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(o.p[0] + off),
                 "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
                 : "memory");
    return;
  }
  for (int q = 0; q < o.n; ++q) st_stream4(o.p[q] + off, v);
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// 16-byte asynchronous copy global -> shared that bypasses L1.
__device__ __forceinline__ void cp_async16_cg(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_u32(smem_dst)),
               "l"(gmem_src)
               : "memory");
}
// 16-byte asynchronous copy that allocates in L1 (reused rows hit there).
__device__ __forceinline__ void cp_async16_ca(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16;\n" ::"r"(smem_u32(smem_dst)),
               "l"(gmem_src)
               : "memory");
}
// 4-byte asynchronous copy (no alignment beyond the element's own).
__device__ __forceinline__ void cp_async4(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(smem_u32(smem_dst)),
               "l"(gmem_src)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() {
  asm volatile("cp.async.commit_group;\n" ::: "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.wait_all;\n" ::: "memory");
}
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

// Programmatic dependent launch: lets a kernel that was launched behind this one in the
// same stream WITH the programmatic-serialization attribute be dispatched as soon as every
// CTA of this grid has executed this (or exited), instead of when the grid has completed.
// Without such a dependent it does nothing.
__device__ __forceinline__ void launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
// Waits until the grids this one was programmatically launched behind have COMPLETED and
// their stores are visible; returns at once for a normally launched grid.  A dependent that
// never waits may complete before its predecessor; where something later in the stream
// relies on both, ONE CTA of the dependent calls this at its end.
__device__ __forceinline__ void wait_for_prior_grids() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

// ---- flag words in shared memory (release / acquire at CTA scope) -------------
// A load's result sits in a register like any other load's: the warp only waits
// where the value is used, so a flag can be read long before it is checked (an
// mbarrier test hands its verdict over in a predicate, which stalls the warp at
// once; measured 180 cycles for a warp-wide test, 50 to 100 for one lane).
__device__ __forceinline__ unsigned ld_acquire_shared(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.cta.shared::cta.u32 %0, [%1];\n" : "=r"(v) : "r"(smem_u32(p)) : "memory");
  return v;
}
__device__ __forceinline__ unsigned ld_relaxed_shared(const unsigned* p) {
  unsigned v;
  asm volatile("ld.relaxed.cta.shared::cta.u32 %0, [%1];\n" : "=r"(v) : "r"(smem_u32(p)) : "memory");
  return v;
}
__device__ __forceinline__ void fence_acquire_cta() {
  asm volatile("fence.acq_rel.cta;\n" ::: "memory");
}
__device__ __forceinline__ void st_release_shared(unsigned* p, unsigned v) {
  asm volatile("st.release.cta.shared::cta.u32 [%0], %1;\n" ::"r"(smem_u32(p)), "r"(v) : "memory");
}

#endif  // __CUDACC__

}  // namespace fg
