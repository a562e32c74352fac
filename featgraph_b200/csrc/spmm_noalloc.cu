// Allocation-free CSR SpMM entry point.
//
// fg_spmm_csr_f32 needs a plan, and making a plan calls cudaMalloc for the
// degree-ordered row lists.  Some hosts cannot do that: a plug-in loaded into
// an inference server whose device memory is handed out entirely by the
// server's own pool, a latency-critical loop in which cudaMalloc / cudaFree
// (which synchronise the whole device) are banned after start-up, or a process
// running under a hard memory budget that was spent before this library was
// loaded.  For those callers fg_spmm_csr_f32_noalloc keeps the row list in a
// fixed array that is part of the library image, builds it on the device on
// every call, and calls no allocator of any kind.
//
// The price: the array is sized for FG_NOALLOC_MAX_ROWS rows and exists on
// every GPU that loads the library until the process exits; every call
// re-derives the row order (four small kernels); all rows, long ones included,
// go through the group-per-row kernel, so graphs with very long rows run
// slower than through a plan; and because all calls share the one array, two
// calls that overlap on the same GPU race with each other.
#include <mutex>

#include "common.cuh"

namespace fg {

constexpr int kNoAllocMaxRows = 1 << 20;   // 1 048 576 rows -> 4 MiB of row ids
constexpr int kNaBuckets = 33;             // bucket = bit length of the row's degree
constexpr int kNaHeaderInts = 128;         // [0,33) counts, [64,97) cursors

// Row order scratch.  In HOST code this name is only a handle for
// cudaGetSymbolAddress; it is not a device address.
static __device__ __align__(256) int g_noalloc_scratch[kNaHeaderInts + kNoAllocMaxRows];

__device__ __forceinline__ int degree_bucket(int deg) { return 32 - __clz(deg); }

__global__ void noalloc_clear_kernel(int* scratch) {
  if (threadIdx.x < kNaHeaderInts) scratch[threadIdx.x] = 0;
}

__global__ void __launch_bounds__(256)
noalloc_count_kernel(const int* __restrict__ indptr, int n_rows, int* scratch) {
  __shared__ int hist[kNaBuckets];
  if (threadIdx.x < kNaBuckets) hist[threadIdx.x] = 0;
  __syncthreads();
  const int r = blockIdx.x * 256 + threadIdx.x;
  if (r < n_rows) atomicAdd(&hist[degree_bucket(indptr[r + 1] - indptr[r])], 1);
  __syncthreads();
  if (threadIdx.x < kNaBuckets && hist[threadIdx.x]) atomicAdd(&scratch[threadIdx.x], hist[threadIdx.x]);
}

// cursor[b] <- number of rows in longer buckets: long rows come first.
__global__ void noalloc_offsets_kernel(int* scratch) {
  if (threadIdx.x == 0) {
    int running = 0;
    for (int b = kNaBuckets - 1; b >= 0; --b) {
      scratch[64 + b] = running;
      running += scratch[b];
    }
  }
}

__global__ void __launch_bounds__(256)
noalloc_scatter_kernel(const int* __restrict__ indptr, int n_rows, int* scratch) {
  __shared__ int hist[kNaBuckets];
  __shared__ int base[kNaBuckets];
  if (threadIdx.x < kNaBuckets) hist[threadIdx.x] = 0;
  __syncthreads();
  const int r = blockIdx.x * 256 + threadIdx.x;
  int b = 0, local = 0;
  if (r < n_rows) {
    b = degree_bucket(indptr[r + 1] - indptr[r]);
    local = atomicAdd(&hist[b], 1);
  }
  __syncthreads();
  if (threadIdx.x < kNaBuckets && hist[threadIdx.x])
    base[threadIdx.x] = atomicAdd(&scratch[64 + threadIdx.x], hist[threadIdx.x]);
  __syncthreads();
  if (r < n_rows) scratch[kNaHeaderInts + base[b] + local] = r;
}

// Group-per-row SpMM over the row order held in the scratch array: G lanes own
// one (row, 4*G-float slab); nonzeros are walked in CSR order with product and
// sum rounded separately, exactly as in the plan-based kernels, so the two
// entry points agree bit for bit.
template <int G>
__global__ void __launch_bounds__(256)
spmm_noalloc_rows_kernel(const int* __restrict__ indptr, const int* __restrict__ indices,
                         const float* __restrict__ vals, const float* __restrict__ X,
                         float* __restrict__ Y, const int* __restrict__ order, int n_rows,
                         long long n_items, int F) {
  constexpr unsigned kFull = 0xffffffffu;
  const int gl = threadIdx.x % G;
  const long long item = (long long)blockIdx.x * (256 / G) + threadIdx.x / G;
  const bool valid = item < n_items;
  int row = 0, slab = 0, e = 0, end = 0;
  if (valid) {
    slab = (int)(item / n_rows);
    row = order[item - (long long)slab * n_rows];
    e = indptr[row];
    end = indptr[row + 1];
  }
  const size_t col_off = (size_t)slab * (4 * G) + (size_t)gl * 4;
  const float* xcol = X + col_off;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  while (__any_sync(kFull, e < end)) {
    const int cnt = end - e;
    int idx = 0;
    float v = 0.f;
    if (gl < cnt) {
      idx = ld_stream(indices + e + gl);
      v = ld_stream(vals + e + gl);
    }
#pragma unroll
    for (int j0 = 0; j0 < G; j0 += 8) {
      if (j0 > 0 && !__any_sync(kFull, j0 < cnt)) break;
      float4 x[8];
      float vv[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int c = __shfl_sync(kFull, idx, j0 + u, G);
        vv[u] = __shfl_sync(kFull, v, j0 + u, G);
        if (j0 + u < cnt) x[u] = ld_gather4(xcol + (size_t)c * F);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (j0 + u < cnt) {
          acc.x = mul_then_add(acc.x, vv[u], x[u].x);
          acc.y = mul_then_add(acc.y, vv[u], x[u].y);
          acc.z = mul_then_add(acc.z, vv[u], x[u].z);
          acc.w = mul_then_add(acc.w, vv[u], x[u].w);
        }
      }
    }
    if (cnt > 0) e += (cnt < G ? cnt : G);
  }
  if (valid) st_stream4(Y + (size_t)row * F + col_off, acc);
}

constexpr int kNaMaxDevices = 64;
static std::mutex g_na_mutex;
static int* g_na_scratch_ptr[kNaMaxDevices] = {nullptr};

// Device address of the scratch array on `device` (which must be current).
// Resolved once per device; cudaGetSymbolAddress allocates nothing.
static int noalloc_scratch(int device, int** out) {
  if (device < 0 || device >= kNaMaxDevices)
    return fail(FG_ERR_INVALID_ARGUMENT, "device index %d out of range", device);
  std::lock_guard<std::mutex> lock(g_na_mutex);
  if (!g_na_scratch_ptr[device]) {
    int* ptr = nullptr;
    FG_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_scratch));
    g_na_scratch_ptr[device] = ptr;
  }
  *out = g_na_scratch_ptr[device];
  return FG_OK;
}

}  // namespace fg

extern "C" int fg_spmm_noalloc_max_rows(void) { return fg::kNoAllocMaxRows; }

extern "C" int fg_spmm_csr_f32_noalloc(const int32_t* indptr, const int32_t* indices,
                                       const float* vals, const float* x, float* y,
                                       int64_t n_rows, int64_t n_cols, int32_t feat_len,
                                       int32_t device, void* stream) {
  using namespace fg;
  if (n_rows < 0 || n_cols < 0 || feat_len <= 0)
    return fail(FG_ERR_INVALID_ARGUMENT, "bad shape: n_rows=%lld n_cols=%lld feat_len=%d",
                (long long)n_rows, (long long)n_cols, (int)feat_len);
  if (n_rows > kNoAllocMaxRows)
    return fail(FG_ERR_UNSUPPORTED,
                "fg_spmm_csr_f32_noalloc handles at most %d rows (its scratch array is fixed "
                "at build time), got %lld; use a plan and fg_spmm_csr_f32 instead",
                kNoAllocMaxRows, (long long)n_rows);
  if (feat_len % 32 != 0)
    return fail(FG_ERR_UNSUPPORTED,
                "fg_spmm_csr_f32_noalloc needs feat_len to be a multiple of 32, got %d",
                (int)feat_len);
  if (n_rows == 0) return FG_OK;
  if (!indptr || !indices || !vals || !x || !y)
    return fail(FG_ERR_INVALID_ARGUMENT, "null device pointer");
  if (reinterpret_cast<uintptr_t>(x) % 16 != 0 || reinterpret_cast<uintptr_t>(y) % 16 != 0)
    return fail(FG_ERR_UNSUPPORTED, "x_dev and y_dev must be 16-byte aligned");

  DeviceGuard guard(device);
  if (guard.status != cudaSuccess)
    return fail(FG_ERR_CUDA, "cannot select device %d: %s", device,
                cudaGetErrorString(guard.status));
  int* scratch = nullptr;
  const int rc = noalloc_scratch(device, &scratch);
  if (rc != FG_OK) return rc;

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int rows = (int)n_rows;
  const unsigned row_blocks = (unsigned)((rows + 255) / 256);
  // The header (bucket counts and cursors) keeps the previous call's values: clear it.
  noalloc_clear_kernel<<<1, kNaHeaderInts, 0, st>>>(scratch);
  noalloc_count_kernel<<<row_blocks, 256, 0, st>>>(indptr, rows, scratch);
  noalloc_offsets_kernel<<<1, 32, 0, st>>>(scratch);
  noalloc_scatter_kernel<<<row_blocks, 256, 0, st>>>(indptr, rows, scratch);
  const int* order = scratch + kNaHeaderInts;
  if (feat_len % 64 == 0) {
    const long long items = (long long)rows * (feat_len / 64);
    const long long grid = (items + 15) / 16;
    if (grid >= INT32_MAX) return fail(FG_ERR_UNSUPPORTED, "too many (row, slab) items");
    spmm_noalloc_rows_kernel<16><<<(unsigned)grid, 256, 0, st>>>(indptr, indices, vals, x, y,
                                                                   order, rows, items, feat_len);
  } else {
    const long long items = (long long)rows * (feat_len / 32);
    const long long grid = (items + 31) / 32;
    if (grid >= INT32_MAX) return fail(FG_ERR_UNSUPPORTED, "too many (row, slab) items");
    spmm_noalloc_rows_kernel<8><<<(unsigned)grid, 256, 0, st>>>(indptr, indices, vals, x, y,
                                                                  order, rows, items, feat_len);
  }
  FG_CUDA_TRY(cudaGetLastError());
  return FG_OK;
}
