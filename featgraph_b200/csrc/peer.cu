// Multi-GPU plumbing that is not a kernel of the hot path itself: a device-side barrier
// between the GPUs of one box whose waits are bounded, and the measurement of the
// L2-resident gather rate that the SpMM / SDDMM kernels are compared with.
#include "common.cuh"

namespace fg {

// Rank `rank` announces `epoch` in slot `rank` of every rank's flag array (its own
// included) and then waits until every slot of its own array has reached `epoch`.
// One thread per rank.  Flags only ever grow; the signed difference keeps the
// comparison right when the 32-bit counter wraps.
//
// Everything a rank's earlier kernels stored -- into its own memory, into a peer's
// through a peer-mapped pointer or a multicast address -- is ordered before the
// announcement (kernel boundary, system-scope fence, release store), and the loads of
// later kernels come after the acquire loads that saw every announcement.
//
// Every wait is bounded: after max_polls polls a thread records 1 + the rank it waited
// for in *status (the first code sticks) and returns.  The host reads the word when it
// next synchronises; a barrier that gave up means a peer never arrived, and what was
// computed around it must not be trusted.
__global__ void peer_barrier_kernel(const __grid_constant__ PeerFlags flags, int rank, int world,
                                    unsigned epoch, int* __restrict__ status,
                                    unsigned max_polls) {
  const int t = threadIdx.x;
  if (t >= world) return;
  __threadfence_system();
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flags.p[t] + rank), "r"(epoch) : "memory");
  const unsigned* mine = flags.p[rank] + t;
  bool got = false;
  for (unsigned i = 0; i < max_polls && !got; ++i) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    got = (int)(v - epoch) >= 0;
    if (!got) __nanosleep(200);
  }
  if (!got) atomicCAS(status, 0, 1 + t);
}

// One warp-wide 16-byte gather per (lane group, row): groups of `row_floats / 4` lanes
// read whole rows of a table at pseudo-random row indices, eight rows in flight per lane,
// and fold them into a checksum.  The access pattern of the SpMM light kernel without its
// arithmetic or its index stream: what the L2 -> SM path delivers for gathers of rows of
// this length out of a table that fits L2.
template <int G>
__global__ void __launch_bounds__(256)
gather_probe_kernel(const float* __restrict__ table, int n_rows, int rows_per_group,
                    float* __restrict__ sink) {
  const int gl = threadIdx.x % G;
  const unsigned group = (blockIdx.x * 256u + threadIdx.x) / G;
  unsigned state = group * 2654435761u + 12345u;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int i = 0; i < rows_per_group; i += 8) {
    float4 x[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      state = state * 1664525u + 1013904223u;
      const unsigned r = (unsigned)(((unsigned long long)state * (unsigned)n_rows) >> 32);
      x[u] = ld_gather4(table + (size_t)r * (4 * G) + 4 * gl);
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      acc.x += x[u].x;
      acc.y += x[u].y;
      acc.z += x[u].z;
      acc.w += x[u].w;
    }
  }
  const float s = acc.x + acc.y + acc.z + acc.w;
  if (s == 123456.789f) sink[0] = s;  // keeps the loads alive; practically never true
}

}  // namespace fg

extern "C" int fg_peer_barrier(uint32_t* const* flag_arrays, int32_t rank, int32_t world,
                               uint32_t epoch, int32_t* status_dev, int64_t max_polls,
                               int32_t device, void* stream) {
  using namespace fg;
  if (world < 1 || world > kMaxOutputs || rank < 0 || rank >= world)
    return fail(FG_ERR_INVALID_ARGUMENT, "bad rank %d / world %d (at most %d ranks)", (int)rank,
                (int)world, kMaxOutputs);
  if (!flag_arrays || !status_dev) return fail(FG_ERR_INVALID_ARGUMENT, "null flag array or status");
  PeerFlags flags;
  for (int q = 0; q < kMaxOutputs; ++q) {
    flags.p[q] = q < world ? flag_arrays[q] : nullptr;
    if (q < world && !flag_arrays[q])
      return fail(FG_ERR_INVALID_ARGUMENT, "flag array %d is null", q);
  }
  const unsigned polls =
      max_polls < 0 ? kPeerBarrierPolls : (unsigned)(max_polls > 0xffffffffLL ? 0xffffffffLL : max_polls);
  DeviceGuard guard(device);
  if (guard.status != cudaSuccess)
    return fail(FG_ERR_CUDA, "cannot select device %d: %s", device,
                cudaGetErrorString(guard.status));
  peer_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(flags, rank, world, epoch,
                                                                      status_dev, polls);
  FG_CUDA_TRY(cudaGetLastError());
  return FG_OK;
}

extern "C" int fg_gather_probe(const float* table_dev, int64_t n_rows, int32_t row_floats,
                               int64_t rows_per_group, int32_t n_blocks, float* sink_dev,
                               int32_t device, void* stream) {
  using namespace fg;
  if (!table_dev || !sink_dev || n_rows <= 0 || n_rows >= INT32_MAX || rows_per_group <= 0 ||
      rows_per_group >= INT32_MAX || n_blocks <= 0)
    return fail(FG_ERR_INVALID_ARGUMENT, "bad probe arguments");
  if (reinterpret_cast<uintptr_t>(table_dev) % 16 != 0)
    return fail(FG_ERR_INVALID_ARGUMENT, "the table must be 16-byte aligned");
  DeviceGuard guard(device);
  if (guard.status != cudaSuccess)
    return fail(FG_ERR_CUDA, "cannot select device %d: %s", device,
                cudaGetErrorString(guard.status));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int rpg = (int)((rows_per_group + 7) / 8 * 8);
  switch (row_floats) {
    case 32: gather_probe_kernel<8><<<n_blocks, 256, 0, st>>>(table_dev, (int)n_rows, rpg, sink_dev); break;
    case 64: gather_probe_kernel<16><<<n_blocks, 256, 0, st>>>(table_dev, (int)n_rows, rpg, sink_dev); break;
    case 128: gather_probe_kernel<32><<<n_blocks, 256, 0, st>>>(table_dev, (int)n_rows, rpg, sink_dev); break;
    default: return fail(FG_ERR_UNSUPPORTED, "row_floats must be 32, 64 or 128");
  }
  FG_CUDA_TRY(cudaGetLastError());
  return FG_OK;
}
