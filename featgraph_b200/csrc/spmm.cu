// CSR SpMM for sm_100a:  Y[r,:] = sum_e vals[e] * X[indices[e],:]
//
// Every (row, feature) accumulator walks the row's nonzeros in CSR order with
// the product and the sum rounded separately, so the result equals, bit for
// bit, a sequential fp32 loop over the row (the loop nest the reference's x86
// schedule produces, python/featgraph/op/vanilla_spmm.py:46-56, 73).  All
// parallelism is across rows and across features, never across one row's
// nonzeros.
//
// Rows are binned by degree on the host (plan):
//   * light rows  -> spmm_light_kernel: a group of G = W/4 lanes owns one
//                    (row, W-float feature slab); float4 gathers, 8 in flight
//                    per lane; rows are served in descending degree so the
//                    groups of a warp finish together.
//   * heavy rows  -> spmm_heavy_kernel: one warp owns one (row, 32-float
//                    slab); indices/values and the gathered X segments are
//                    staged through shared memory with cp.async rings, which
//                    decouples the sequential add chain from the gather
//                    latency.  Launched on an auxiliary stream so the long
//                    rows overlap the light kernel.
//   * anything the vector paths cannot take (feat_len not a multiple of 32,
//     unaligned pointers) -> spmm_generic_kernel, one warp per row.
#include <algorithm>
#include <cstring>
#include <vector>

#include "common.cuh"

namespace fg {

// ------------------------------------------------------------------ kernels --

// One group of G lanes per (row, slab) item; W = 4 * G floats per slab.
template <int G>
__global__ void __launch_bounds__(256)
spmm_light_kernel(const int* __restrict__ indptr, const int* __restrict__ indices,
                  const float* __restrict__ vals, const float* __restrict__ X,
                  float* __restrict__ Y, const int* __restrict__ rows, int n_listed,
                  long long n_items, int F) {
  constexpr unsigned kFull = 0xffffffffu;
  const int gl = threadIdx.x % G;  // lane within the group
  const long long item = (long long)blockIdx.x * (256 / G) + threadIdx.x / G;
  const bool valid = item < n_items;
  int row = 0, slab = 0, e = 0, end = 0;
  if (valid) {
    slab = (int)(item / n_listed);
    row = __ldg(rows + (item - (long long)slab * n_listed));
    e = __ldg(indptr + row);
    end = __ldg(indptr + row + 1);
  }
  const size_t col_off = (size_t)slab * (4 * G) + (size_t)gl * 4;
  const float* xcol = X + col_off;
  float2 acc_lo = make_float2(0.f, 0.f), acc_hi = make_float2(0.f, 0.f);

  // Index/value tile of the NEXT iteration, fetched one iteration ahead so that
  // its DRAM latency overlaps the gathers of the current one.
  int idx_next = 0;
  float v_next = 0.f;
  if (gl < end - e) {
    idx_next = ld_stream(indices + e + gl);
    v_next = ld_stream(vals + e + gl);
  }

  // The loop is warp-uniform: groups whose row is exhausted idle (cnt <= 0).
  while (__any_sync(kFull, e < end)) {
    const int cnt = end - e;
    const int idx = idx_next;
    const float v = v_next;
    idx_next = 0;
    v_next = 0.f;
    if (gl < cnt - G) {
      idx_next = ld_stream(indices + e + G + gl);
      v_next = ld_stream(vals + e + G + gl);
    }
#pragma unroll
    for (int j0 = 0; j0 < G; j0 += 8) {
      float4 x[8];
      if (__all_sync(kFull, cnt >= j0 + 8)) {
        // every group of the warp has a full batch: no predicates
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int c = __shfl_sync(kFull, idx, j0 + u, G);
          x[u] = ld_gather4(xcol + (size_t)c * F);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const float vu = __shfl_sync(kFull, v, j0 + u, G);
          acc_lo = mul_then_add2(acc_lo, vu, make_float2(x[u].x, x[u].y));
          acc_hi = mul_then_add2(acc_hi, vu, make_float2(x[u].z, x[u].w));
        }
      } else {
        if (!__any_sync(kFull, j0 < cnt)) break;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int c = __shfl_sync(kFull, idx, j0 + u, G);
          if (j0 + u < cnt) x[u] = ld_gather4(xcol + (size_t)c * F);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const float vu = __shfl_sync(kFull, v, j0 + u, G);
          if (j0 + u < cnt) {
            acc_lo = mul_then_add2(acc_lo, vu, make_float2(x[u].x, x[u].y));
            acc_hi = mul_then_add2(acc_hi, vu, make_float2(x[u].z, x[u].w));
          }
        }
      }
    }
    if (cnt > 0) e += (cnt < G ? cnt : G);
  }
  if (valid)
    st_stream4(Y + (size_t)row * F + col_off, make_float4(acc_lo.x, acc_lo.y, acc_hi.x, acc_hi.y));
}

constexpr int kHvEdges = 32;    // nonzeros per stage
constexpr int kHvXSlots = 8;    // ring of gathered X segments (power of two)
constexpr int kHvDist = kHvXSlots - 1;  // stages of gathers in flight
constexpr int kHvISlots = 16;   // ring of index/value tiles, >= 2 * kHvDist + 1

template <int VEC>
constexpr int heavy_smem_bytes() {
  return kHvXSlots * kHvEdges * 32 * VEC * 4 + kHvISlots * kHvEdges * 8;
}

// One warp per (heavy row, 32*VEC-float slab); VEC = floats per lane (1 or 2).
template <int VEC>
__global__ void __launch_bounds__(32)
spmm_heavy_kernel(const int* __restrict__ indptr, const int* __restrict__ indices,
                  const float* __restrict__ vals, const float* __restrict__ X,
                  float* __restrict__ Y, const int* __restrict__ rows, int n_listed,
                  int subs_per_slab, int F) {
  constexpr int kSlab = 32 * VEC;                 // floats per gathered segment
  constexpr int kLanesPerRow = kSlab / 4;         // 16-byte copies per segment
  constexpr int kRowsPerCopy = 32 / kLanesPerRow; // segments covered by one warp-wide copy
  extern __shared__ __align__(16) unsigned char heavy_smem[];
  float(*xs)[kHvEdges][kSlab] = reinterpret_cast<float(*)[kHvEdges][kSlab]>(heavy_smem);
  int(*idx_s)[kHvEdges] =
      reinterpret_cast<int(*)[kHvEdges]>(heavy_smem + kHvXSlots * kHvEdges * kSlab * 4);
  float(*val_s)[kHvEdges] = reinterpret_cast<float(*)[kHvEdges]>(
      heavy_smem + kHvXSlots * kHvEdges * kSlab * 4 + kHvISlots * kHvEdges * 4);

  const int lane = threadIdx.x;
  // Item order: (residency slab, row, sub-slab) so that the sub-slabs of one
  // row run side by side and share their index stream in L2.
  const long long item = blockIdx.x;
  const long long per_slab = (long long)n_listed * subs_per_slab;
  const int ss = (int)(item / per_slab);
  const long long rem = item - ss * per_slab;
  const int row = __ldg(rows + rem / subs_per_slab);
  const int sub = ss * subs_per_slab + (int)(rem % subs_per_slab);

  const int beg = __ldg(indptr + row);
  const int deg = __ldg(indptr + row + 1) - beg;
  const int n_stages = (deg + kHvEdges - 1) / kHvEdges;
  const int* ind = indices + beg;
  const float* val = vals + beg;
  const float* xbase = X + (size_t)sub * kSlab;

  auto issue_idx = [&](int s) {
    if (s < n_stages) {
      const int e = s * kHvEdges + lane;
      if (e < deg) {
        cp_async4(&idx_s[s & (kHvISlots - 1)][lane], ind + e);
        cp_async4(&val_s[s & (kHvISlots - 1)][lane], val + e);
      }
    }
  };
  auto issue_gather = [&](int s) {
    if (s < n_stages) {
      constexpr int kCopies = kHvEdges / kRowsPerCopy;
      const int cnt = min(kHvEdges, deg - s * kHvEdges);
      const int part = (lane % kLanesPerRow) * 4;
      const int* it = idx_s[s & (kHvISlots - 1)];
      float(*xt)[kSlab] = xs[s & (kHvXSlots - 1)];
      // All column indices are read before the first copy is issued: the copies
      // are ordered against shared-memory reads, so a read placed between two of
      // them would serialise the whole sequence on its latency.
      int c[kCopies];
#pragma unroll
      for (int k = 0; k < kCopies; ++k) c[k] = it[lane / kLanesPerRow + kRowsPerCopy * k];
#pragma unroll
      for (int k = 0; k < kCopies; ++k) {
        const int e = lane / kLanesPerRow + kRowsPerCopy * k;
        if (e < cnt) cp_async16_cg(&xt[e][part], xbase + (size_t)c[k] * F + part);
      }
    }
  };

  for (int s = 0; s < kHvDist; ++s) {
    issue_idx(s);
    cp_async_commit();
  }
  cp_async_wait<0>();
  __syncwarp();
  for (int s = 0; s < kHvDist; ++s) {
    issue_gather(s);
    issue_idx(s + kHvDist);
    cp_async_commit();
  }

  float acc1 = 0.f;
  float2 acc2 = make_float2(0.f, 0.f);
  for (int i = 0; i < n_stages; ++i) {
    cp_async_wait<kHvDist - 1>();  // stage i's gathers and stage i+D's indices landed
    __syncwarp();                  // ... for every lane; stage i-1 is fully consumed
    issue_gather(i + kHvDist);
    issue_idx(i + 2 * kHvDist);
    cp_async_commit();

    const float(*xt)[kSlab] = xs[i & (kHvXSlots - 1)];
    const float* vt = val_s[i & (kHvISlots - 1)];
    const int cnt = min(kHvEdges, deg - i * kHvEdges);
    if (cnt == kHvEdges) {
#pragma unroll
      for (int e4 = 0; e4 < kHvEdges; e4 += 4) {
        const float4 v4 = *reinterpret_cast<const float4*>(vt + e4);
        const float vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          if (VEC == 2)
            acc2 = mul_then_add2(acc2, vv[q],
                                 *reinterpret_cast<const float2*>(&xt[e4 + q][lane * VEC]));
          else
            acc1 = mul_then_add(acc1, vv[q], xt[e4 + q][lane * VEC]);
        }
      }
    } else {
      for (int e = 0; e < cnt; ++e) {
        if (VEC == 2)
          acc2 = mul_then_add2(acc2, vt[e], *reinterpret_cast<const float2*>(&xt[e][lane * VEC]));
        else
          acc1 = mul_then_add(acc1, vt[e], xt[e][lane * VEC]);
      }
    }
  }
  cp_async_wait<0>();
  float* yout = Y + (size_t)row * F + (size_t)sub * kSlab + lane * VEC;
  if (VEC == 2)
    __stcs(reinterpret_cast<float2*>(yout), acc2);
  else
    __stcs(yout, acc1);
}

// Fallback for any feat_len / alignment: one warp per row, lanes over features.
__global__ void __launch_bounds__(256)
spmm_generic_kernel(const int* __restrict__ indptr, const int* __restrict__ indices,
                    const float* __restrict__ vals, const float* __restrict__ X,
                    float* __restrict__ Y, long long n_rows, int F) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  const int beg = indptr[row], end = indptr[row + 1];
  for (int f0 = 0; f0 < F; f0 += 32) {
    const int f = f0 + lane;
    float acc = 0.f;
    if (f < F) {
      for (int e = beg; e < end; ++e)
        acc = mul_then_add(acc, vals[e], X[(size_t)indices[e] * F + f]);
      Y[(size_t)row * F + f] = acc;
    }
  }
}

}  // namespace fg

// --------------------------------------------------------------------- plan --

struct fg_spmm_plan {
  int device = 0;
  int64_t n_rows = 0, n_cols = 0, nnz = 0;
  int feat_len = 0;
  bool vector_ok = false;  // feat_len % 32 == 0
  int slab_w = 0;          // floats per light item (32, 64 or 128)
  int heavy_vec = 1;       // floats per lane of the heavy kernel (1 or 2)
  int heavy_threshold = 0;
  int n_light = 0, n_heavy = 0;
  int64_t max_deg = 0, heavy_nnz = 0;
  int* light_rows_dev = nullptr;
  int* heavy_rows_dev = nullptr;
  cudaStream_t aux = nullptr;
  cudaEvent_t fork_ev = nullptr, join_ev = nullptr;
  int l2_bytes = 0;
};

namespace fg {

constexpr int kDefaultHeavyThreshold = 2048;

static void plan_release(fg_spmm_plan* p) {
  if (!p) return;
  DeviceGuard g(p->device);
  if (p->light_rows_dev) cudaFree(p->light_rows_dev);
  if (p->heavy_rows_dev) cudaFree(p->heavy_rows_dev);
  if (p->fork_ev) cudaEventDestroy(p->fork_ev);
  if (p->join_ev) cudaEventDestroy(p->join_ev);
  if (p->aux) cudaStreamDestroy(p->aux);
  delete p;
}

// Largest slab width in {128, 64, 32} that divides F and keeps one slab of X
// (n_cols x W floats) within half of L2; if no width fits, the widest divisor
// (fewest passes over the adjacency).
static int choose_slab_width(int F, int64_t n_cols, int l2_bytes) {
  const int cand[3] = {128, 64, 32};
  for (int w : cand)
    if (F % w == 0 && n_cols * (int64_t)w * 4 <= (int64_t)l2_bytes / 2) return w;
  for (int w : cand)
    if (F % w == 0) return w;
  return 32;
}

}  // namespace fg

extern "C" int fg_spmm_plan_create(const int32_t* indptr, int64_t n_rows, int64_t n_cols,
                                   int32_t feat_len, int32_t device, int32_t heavy_threshold,
                                   fg_spmm_plan** out_plan) {
  using namespace fg;
  if (!out_plan) return fail(FG_ERR_INVALID_ARGUMENT, "out_plan is null");
  *out_plan = nullptr;
  if (n_rows < 0 || n_cols < 0 || feat_len <= 0)
    return fail(FG_ERR_INVALID_ARGUMENT, "bad shape: n_rows=%lld n_cols=%lld feat_len=%d",
                (long long)n_rows, (long long)n_cols, (int)feat_len);
  if (n_rows >= INT32_MAX || n_cols >= INT32_MAX)
    return fail(FG_ERR_UNSUPPORTED, "row/column counts must fit int32");
  if (!indptr) return fail(FG_ERR_INVALID_ARGUMENT, "indptr_host is null");
  if (indptr[0] != 0) return fail(FG_ERR_INVALID_ARGUMENT, "indptr[0] must be 0");
  int64_t max_deg = 0;
  for (int64_t r = 0; r < n_rows; ++r) {
    const int64_t d = (int64_t)indptr[r + 1] - indptr[r];
    if (d < 0) return fail(FG_ERR_INVALID_ARGUMENT, "indptr decreases at row %lld", (long long)r);
    max_deg = std::max(max_deg, d);
  }

  fg_spmm_plan* p = new (std::nothrow) fg_spmm_plan();
  if (!p) return fail(FG_ERR_OUT_OF_MEMORY, "plan allocation failed");
  p->device = device;
  p->n_rows = n_rows;
  p->n_cols = n_cols;
  p->nnz = indptr[n_rows];
  p->feat_len = feat_len;
  p->max_deg = max_deg;
  p->heavy_threshold = heavy_threshold > 0 ? heavy_threshold : kDefaultHeavyThreshold;
  p->vector_ok = (feat_len % 32 == 0);

  DeviceGuard guard(device);
  if (guard.status != cudaSuccess) {
    delete p;
    return fail(FG_ERR_CUDA, "cannot select device %d: %s", device,
                cudaGetErrorString(guard.status));
  }
#define FG_PLAN_TRY(expr)                                                            \
  do {                                                                               \
    cudaError_t e__ = (expr);                                                        \
    if (e__ != cudaSuccess) {                                                        \
      plan_release(p);                                                               \
      return fail(e__ == cudaErrorMemoryAllocation ? FG_ERR_OUT_OF_MEMORY : FG_ERR_CUDA, \
                  "%s failed: %s", #expr, cudaGetErrorString(e__));                  \
    }                                                                                \
  } while (0)

  FG_PLAN_TRY(cudaDeviceGetAttribute(&p->l2_bytes, cudaDevAttrL2CacheSize, device));
  p->slab_w = choose_slab_width(feat_len, n_cols, p->l2_bytes);
  p->heavy_vec = (p->slab_w % 64 == 0) ? 2 : 1;

  if (p->vector_ok && n_rows > 0) {
    // Stable counting sort of the rows by degree, descending: the hardware
    // block scheduler then hands out the longest rows first, and the groups
    // that share a warp get rows of (nearly) equal length.
    std::vector<int32_t> start((size_t)max_deg + 2, 0);
    for (int64_t r = 0; r < n_rows; ++r) start[(size_t)(indptr[r + 1] - indptr[r])]++;
    // start[d] <- number of rows with degree > d
    int64_t running = 0;
    for (int64_t d = max_deg; d >= 0; --d) {
      const int32_t c = start[(size_t)d];
      start[(size_t)d] = (int32_t)running;
      running += c;
    }
    std::vector<int32_t> order((size_t)n_rows);
    for (int64_t r = 0; r < n_rows; ++r)
      order[(size_t)start[(size_t)(indptr[r + 1] - indptr[r])]++] = (int32_t)r;
    int64_t n_heavy = 0, heavy_nnz = 0;
    while (n_heavy < n_rows) {
      const int64_t d = indptr[order[(size_t)n_heavy] + 1] - indptr[order[(size_t)n_heavy]];
      if (d <= p->heavy_threshold) break;
      heavy_nnz += d;
      ++n_heavy;
    }
    p->n_heavy = (int)n_heavy;
    p->n_light = (int)(n_rows - n_heavy);
    p->heavy_nnz = heavy_nnz;
    if (p->n_heavy > 0) {
      FG_PLAN_TRY(cudaMalloc(&p->heavy_rows_dev, sizeof(int32_t) * (size_t)p->n_heavy));
      FG_PLAN_TRY(cudaMemcpy(p->heavy_rows_dev, order.data(), sizeof(int32_t) * (size_t)p->n_heavy,
                             cudaMemcpyHostToDevice));
      FG_PLAN_TRY(cudaFuncSetAttribute(spmm_heavy_kernel<1>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       heavy_smem_bytes<1>()));
      FG_PLAN_TRY(cudaFuncSetAttribute(spmm_heavy_kernel<2>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       heavy_smem_bytes<2>()));
      int lo = 0, hi = 0;
      FG_PLAN_TRY(cudaDeviceGetStreamPriorityRange(&lo, &hi));
      FG_PLAN_TRY(cudaStreamCreateWithPriority(&p->aux, cudaStreamNonBlocking, hi));
      FG_PLAN_TRY(cudaEventCreateWithFlags(&p->fork_ev, cudaEventDisableTiming));
      FG_PLAN_TRY(cudaEventCreateWithFlags(&p->join_ev, cudaEventDisableTiming));
    }
    if (p->n_light > 0) {
      FG_PLAN_TRY(cudaMalloc(&p->light_rows_dev, sizeof(int32_t) * (size_t)p->n_light));
      FG_PLAN_TRY(cudaMemcpy(p->light_rows_dev, order.data() + n_heavy,
                             sizeof(int32_t) * (size_t)p->n_light, cudaMemcpyHostToDevice));
    }
  }
#undef FG_PLAN_TRY
  *out_plan = p;
  return FG_OK;
}

extern "C" int fg_spmm_plan_destroy(fg_spmm_plan* plan) {
  fg::plan_release(plan);
  return FG_OK;
}

extern "C" int fg_spmm_plan_num_launches(const fg_spmm_plan* p) {
  if (!p || p->n_rows == 0) return 0;
  if (!p->vector_ok) return 1;
  return (p->n_heavy > 0 ? 1 : 0) + (p->n_light > 0 ? 1 : 0);
}

extern "C" int fg_spmm_plan_describe(const fg_spmm_plan* p, char* buf, int64_t buf_len) {
  using namespace fg;
  if (!p || !buf || buf_len <= 0) return fail(FG_ERR_INVALID_ARGUMENT, "null plan or buffer");
  if (p->vector_ok) {
    const int G = p->slab_w / 4;
    const long long light_items = (long long)p->n_light * (p->feat_len / p->slab_w);
    const long long heavy_items = (long long)p->n_heavy * (p->feat_len / (32 * p->heavy_vec));
    snprintf(buf, (size_t)buf_len,
             "spmm_csr_f32 rows=%lld cols=%lld nnz=%lld feat_len=%d | L2=%d B slab_w=%d | "
             "light: %d rows (deg<=%d) -> spmm_light_kernel<G=%d> grid=%lld x 256 thr | "
             "heavy: %d rows, %lld nnz, max_deg=%lld -> spmm_heavy_kernel<VEC=%d> grid=%lld x 32 thr, "
             "%d-stage cp.async ring, aux stream",
             (long long)p->n_rows, (long long)p->n_cols, (long long)p->nnz, p->feat_len,
             p->l2_bytes, p->slab_w, p->n_light, p->heavy_threshold, G,
             (light_items + 256 / G - 1) / (256 / G), p->n_heavy, (long long)p->heavy_nnz,
             (long long)p->max_deg, p->heavy_vec, heavy_items, kHvDist);
  } else {
    snprintf(buf, (size_t)buf_len,
             "spmm_csr_f32 rows=%lld cols=%lld nnz=%lld feat_len=%d | spmm_generic_kernel "
             "(feat_len %% 32 != 0) grid=%lld x 256 thr",
             (long long)p->n_rows, (long long)p->n_cols, (long long)p->nnz, p->feat_len,
             (long long)((p->n_rows + 7) / 8));
  }
  return FG_OK;
}

// ------------------------------------------------------------------- launch --

namespace fg {

template <int G>
static void launch_light(const fg_spmm_plan* p, const int32_t* indptr, const int32_t* indices,
                         const float* vals, const float* x, float* y, cudaStream_t st) {
  const long long items = (long long)p->n_light * (p->feat_len / (4 * G));
  const long long grid = (items + 256 / G - 1) / (256 / G);
  spmm_light_kernel<G><<<(unsigned)grid, 256, 0, st>>>(indptr, indices, vals, x, y,
                                                        p->light_rows_dev, p->n_light, items,
                                                        p->feat_len);
}

}  // namespace fg

extern "C" int fg_spmm_csr_f32(const fg_spmm_plan* p, const int32_t* indptr,
                               const int32_t* indices, const float* vals, const float* x,
                               float* y, void* stream) {
  using namespace fg;
  if (!p) return fail(FG_ERR_INVALID_ARGUMENT, "plan is null");
  if (p->n_rows == 0) return FG_OK;
  if (!indptr || !y) return fail(FG_ERR_INVALID_ARGUMENT, "indptr_dev or y_dev is null");
  if (p->nnz > 0 && (!indices || !vals || !x))
    return fail(FG_ERR_INVALID_ARGUMENT, "indices_dev, vals_dev or x_dev is null");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  DeviceGuard guard(p->device);
  if (guard.status != cudaSuccess)
    return fail(FG_ERR_CUDA, "cannot select device %d: %s", p->device,
                cudaGetErrorString(guard.status));

  const bool aligned = (reinterpret_cast<uintptr_t>(x) % 16 == 0) &&
                       (reinterpret_cast<uintptr_t>(y) % 16 == 0);
  if (!p->vector_ok || !aligned) {
    const long long grid = (p->n_rows + 7) / 8;
    spmm_generic_kernel<<<(unsigned)grid, 256, 0, st>>>(indptr, indices, vals, x, y, p->n_rows,
                                                        p->feat_len);
    FG_CUDA_TRY(cudaGetLastError());
    return FG_OK;
  }

  if (p->n_heavy > 0) {
    // Fork: the heavy rows run on the plan's high-priority stream while the
    // light kernel fills the rest of the machine; join before returning.
    FG_CUDA_TRY(cudaEventRecord(p->fork_ev, st));
    FG_CUDA_TRY(cudaStreamWaitEvent(p->aux, p->fork_ev, 0));
    const int slab = 32 * p->heavy_vec;
    const long long items = (long long)p->n_heavy * (p->feat_len / slab);
    if (items >= INT32_MAX) return fail(FG_ERR_UNSUPPORTED, "too many heavy items");
    if (p->heavy_vec == 2)
      spmm_heavy_kernel<2><<<(unsigned)items, 32, heavy_smem_bytes<2>(), p->aux>>>(
          indptr, indices, vals, x, y, p->heavy_rows_dev, p->n_heavy, p->slab_w / slab,
          p->feat_len);
    else
      spmm_heavy_kernel<1><<<(unsigned)items, 32, heavy_smem_bytes<1>(), p->aux>>>(
          indptr, indices, vals, x, y, p->heavy_rows_dev, p->n_heavy, p->slab_w / slab,
          p->feat_len);
    FG_CUDA_TRY(cudaGetLastError());
    FG_CUDA_TRY(cudaEventRecord(p->join_ev, p->aux));
  }
  if (p->n_light > 0) {
    switch (p->slab_w) {
      case 128: launch_light<32>(p, indptr, indices, vals, x, y, st); break;
      case 64: launch_light<16>(p, indptr, indices, vals, x, y, st); break;
      default: launch_light<8>(p, indptr, indices, vals, x, y, st); break;
    }
    FG_CUDA_TRY(cudaGetLastError());
  }
  if (p->n_heavy > 0) FG_CUDA_TRY(cudaStreamWaitEvent(st, p->join_ev, 0));
  return FG_OK;
}

extern "C" int fg_spmm_csr_f32_host(const fg_spmm_plan* p, const int32_t* indptr,
                                    const int32_t* indices, const float* vals,
                                    const float* x_host, float* y_host, float* x_stage,
                                    float* y_stage, void* stream) {
  using namespace fg;
  if (!p) return fail(FG_ERR_INVALID_ARGUMENT, "plan is null");
  if (!x_host || !y_host || !x_stage || !y_stage)
    return fail(FG_ERR_INVALID_ARGUMENT, "null host or staging buffer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  DeviceGuard guard(p->device);
  if (guard.status != cudaSuccess)
    return fail(FG_ERR_CUDA, "cannot select device %d: %s", p->device,
                cudaGetErrorString(guard.status));
  const size_t xb = sizeof(float) * (size_t)p->n_cols * p->feat_len;
  const size_t yb = sizeof(float) * (size_t)p->n_rows * p->feat_len;
  if (xb) FG_CUDA_TRY(cudaMemcpyAsync(x_stage, x_host, xb, cudaMemcpyHostToDevice, st));
  const int rc = fg_spmm_csr_f32(p, indptr, indices, vals, x_stage, y_stage, stream);
  if (rc != FG_OK) return rc;
  if (yb) FG_CUDA_TRY(cudaMemcpyAsync(y_host, y_stage, yb, cudaMemcpyDeviceToHost, st));
  FG_CUDA_TRY(cudaStreamSynchronize(st));
  return FG_OK;
}
