// CSR SpMM for sm_100a:  Y[r,:] = sum_e vals[e] * X[indices[e],:]
//
// Every (row, feature) accumulator walks the row's nonzeros in CSR order with
// the product and the sum rounded separately, so the result equals, bit for
// bit, a sequential fp32 loop over the row (the loop nest the reference's x86
// schedule produces, python/featgraph/op/vanilla_spmm.py:46-56, 73).  All
// parallelism is across rows and across features, never across one row's
// nonzeros.
//
// Rows are sorted by degree on the host (plan) and split into three classes,
// each with its own kernel, launched on three streams so that they overlap:
//   * light rows (deg <= 2048) -> spmm_light_kernel: a group of G = W/4 lanes
//       owns one (row, W-float feature slab); float4 gathers straight into
//       registers, 8 in flight per lane, index/value tile fetched one iteration
//       ahead; rows are served in descending degree so that the groups of a
//       warp finish together.
//   * heavy rows -> spmm_heavy_kernel: one warp owns one (row, 32- or 64-float
//       slab); indices/values and the gathered X segments are staged through
//       shared memory with cp.async rings, which takes the gather latency off
//       the sequential add chain.
//   * giant rows (deg > 32768, at most one CTA per SM) -> spmm_giant_kernel: a
//       consumer warp adds in order while nine producer warps gather, handing
//       stages over through mbarriers.  The longest row bounds the whole call
//       (its sum is one dependent chain) and a single warp cannot keep enough
//       copies in flight to feed that chain.
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
                  OutPtrs Y, const int* __restrict__ rows, int n_listed,
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
    for (int q = 0; q < Y.n; ++q)
      st_stream4(Y.p[q] + (size_t)row * F + col_off,
                 make_float4(acc_lo.x, acc_lo.y, acc_hi.x, acc_hi.y));
}

constexpr int kHvEdges = 32;    // nonzeros per stage
constexpr int kHvXSlots = 2;    // ring of gathered X segments (power of two)
constexpr int kHvDist = kHvXSlots - 1;  // stages of gathers in flight
constexpr int kHvISlots = 4;    // ring of index/value tiles, >= 2 * kHvDist + 1

template <int VEC>
constexpr int heavy_smem_bytes() {
  return kHvXSlots * kHvEdges * 32 * VEC * 4 + kHvISlots * kHvEdges * 8;
}

// Adds one stage (cnt <= 32 gathered segments, in CSR order) to a lane's
// accumulators; xt[e] is the segment of nonzero e, vt[e] its value.
template <int VEC>
__device__ __forceinline__ void heavy_consume_stage(const float (*xt)[32 * VEC], const float* vt,
                                                    int cnt, int lane, float& acc_a,
                                                    float& acc_b) {
  if (cnt == kHvEdges) {
#pragma unroll
    for (int e4 = 0; e4 < kHvEdges; e4 += 4) {
      const float4 v4 = *reinterpret_cast<const float4*>(vt + e4);
      const float vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        if (VEC == 2) {
          const float2 xv = *reinterpret_cast<const float2*>(&xt[e4 + q][lane * 2]);
          acc_a = mul_then_add(acc_a, vv[q], xv.x);
          acc_b = mul_then_add(acc_b, vv[q], xv.y);
        } else {
          acc_a = mul_then_add(acc_a, vv[q], xt[e4 + q][lane]);
        }
      }
    }
  } else {
    for (int e = 0; e < cnt; ++e) {
      if (VEC == 2) {
        const float2 xv = *reinterpret_cast<const float2*>(&xt[e][lane * 2]);
        acc_a = mul_then_add(acc_a, vt[e], xv.x);
        acc_b = mul_then_add(acc_b, vt[e], xv.y);
      } else {
        acc_a = mul_then_add(acc_a, vt[e], xt[e][lane]);
      }
    }
  }
}

template <int VEC>
__device__ __forceinline__ void heavy_store_row(const OutPtrs& Y, size_t slab_off, int lane,
                                                float acc_a, float acc_b) {
  for (int q = 0; q < Y.n; ++q) {
    float* yslab = Y.p[q] + slab_off;
    if (VEC == 2)
      __stcs(reinterpret_cast<float2*>(yslab + lane * 2), make_float2(acc_a, acc_b));
    else
      __stcs(yslab + lane, acc_a);
  }
}

// Decodes blockIdx.x of the heavy / giant kernels: items are ordered
// (residency slab, row, sub-slab) so that the sub-slabs of one row run side by
// side and share their index stream in L2.
__device__ __forceinline__ void heavy_decode_item(const int* __restrict__ rows, int n_listed,
                                                  int subs_per_slab, int& row, int& sub) {
  const long long item = blockIdx.x;
  const long long per_slab = (long long)n_listed * subs_per_slab;
  const int ss = (int)(item / per_slab);
  const long long rem = item - ss * per_slab;
  row = __ldg(rows + rem / subs_per_slab);
  sub = ss * subs_per_slab + (int)(rem % subs_per_slab);
}

// One warp per (heavy row, 32*VEC-float slab); VEC = floats per lane (1 or 2).
template <int VEC>
__global__ void __launch_bounds__(32)
spmm_heavy_kernel(const int* __restrict__ indptr, const int* __restrict__ indices,
                  const float* __restrict__ vals, const float* __restrict__ X,
                  OutPtrs Y, const int* __restrict__ rows, int n_listed,
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
  int row, sub;
  heavy_decode_item(rows, n_listed, subs_per_slab, row, sub);

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

  // Two scalar chains per lane (VEC == 2) rather than one packed add: on this
  // latency-bound path the packed fp32x2 add is the slower dependency.
  float acc_a = 0.f, acc_b = 0.f;
  for (int i = 0; i < n_stages; ++i) {
    cp_async_wait<kHvDist - 1>();  // stage i's gathers and stage i+D's indices landed
    __syncwarp();                  // ... for every lane; stage i-1 is fully consumed
    issue_gather(i + kHvDist);
    issue_idx(i + 2 * kHvDist);
    cp_async_commit();
    heavy_consume_stage<VEC>(xs[i & (kHvXSlots - 1)], val_s[i & (kHvISlots - 1)],
                             min(kHvEdges, deg - i * kHvEdges), lane, acc_a, acc_b);
  }
  cp_async_wait<0>();
  heavy_store_row<VEC>(Y, (size_t)row * F + (size_t)sub * kSlab, lane, acc_a, acc_b);
}

constexpr int kGtWarps = 12;      // warps per CTA; warp 0 consumes, warps 4 and 8 retire
constexpr int kGtProducers = 9;   // producer warps per CTA (the warps with id % 4 != 0)
constexpr int kGtSlots = 16;      // ring of stages (power of two)
constexpr int kGtQueue = 4;       // stages of column indices a producer holds in registers
constexpr unsigned kGtMaxPolls = 1u << 20;  // bound of every barrier wait
// A parity wait tells the current phase from the previous one only.  A producer's
// consecutive stages are kGtProducers apart; were that more than the ring size it
// would skip a round of a slot and its wait would pass one phase too early.
static_assert(kGtProducers <= kGtSlots, "a producer may not skip a round of a slot");
constexpr int kGtErrProducerTimeout = 1, kGtErrConsumerTimeout = 2;

template <int VEC>
constexpr int giant_smem_bytes() {
  return kGtSlots * kHvEdges * 32 * VEC * 4   // gathered X segments
         + kGtSlots * kHvEdges * 4            // values
         + 2 * kGtSlots * 8;                  // full / empty barriers
}

// One CTA of 1 consumer + kGtProducers producer warps per (giant row, slab).
// Warps are dealt to the SM's four schedulers round-robin by id, so warps 4 and
// 8 -- which would share the consumer's scheduler -- retire at once: the add
// chain keeps a scheduler's issue slots to itself.
//
// The sum of one row is a dependent chain (CSR order, one accumulator per
// feature), so the longest row bounds the whole SpMM.  A single warp cannot feed
// that chain: it can keep only a few cp.async copies outstanding (measured: 85
// cycles per 512-byte copy instruction for a lone warp, i.e. 47 cycles per
// nonzero at 64 features, while the chain itself needs 4 to 6).  Here producer
// warp w gathers stages w, w+P, w+2P, ... (column indices through a register
// queue, 16-byte cp.async copies that signal the stage's "full" mbarrier when
// they land) and the consumer warp adds the stages in order and hands slots
// back through "empty" mbarriers.  Every barrier wait is a bounded poll; a wait
// that gives up records a code in *status and the warp leaves.
template <int VEC>
__global__ void __launch_bounds__(32 * kGtWarps)
spmm_giant_kernel(const int* __restrict__ indptr, const int* __restrict__ indices,
                  const float* __restrict__ vals, const float* __restrict__ X,
                  OutPtrs Y, const int* __restrict__ rows, int n_listed,
                  int subs_per_slab, int F, int* __restrict__ status) {
  constexpr unsigned kFull = 0xffffffffu;
  constexpr int kSlab = 32 * VEC;
  constexpr int kLanesPerRow = kSlab / 4;
  constexpr int kRowsPerCopy = 32 / kLanesPerRow;
  constexpr int kCopies = kHvEdges / kRowsPerCopy;
  extern __shared__ __align__(16) unsigned char giant_smem[];
  float(*xs)[kHvEdges][kSlab] = reinterpret_cast<float(*)[kHvEdges][kSlab]>(giant_smem);
  float(*val_s)[kHvEdges] =
      reinterpret_cast<float(*)[kHvEdges]>(giant_smem + kGtSlots * kHvEdges * kSlab * 4);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(giant_smem + kGtSlots * kHvEdges * kSlab * 4 +
                                                   kGtSlots * kHvEdges * 4);
  uint64_t* empty_bar = full_bar + kGtSlots;

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  int row, sub;
  heavy_decode_item(rows, n_listed, subs_per_slab, row, sub);
  const int beg = __ldg(indptr + row);
  const int deg = __ldg(indptr + row + 1) - beg;
  const int n_stages = (deg + kHvEdges - 1) / kHvEdges;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kGtSlots; ++i) {
      mbar_init(&full_bar[i], 32);  // one arrival per lane of the producing warp
      mbar_init(&empty_bar[i], 1);  // one arrival by the consumer
    }
  }
  __syncthreads();

  if (warp > 0 && (warp & 3) == 0) return;  // leave the consumer's scheduler alone
  if (warp > 0) {
    // ------------------------------------------------------------ producer --
    const int* ind = indices + beg;
    const float* val = vals + beg;
    const int part = (lane % kLanesPerRow) * 4;
    const int first = lane / kLanesPerRow;
    const float* xbase = X + (size_t)sub * kSlab + part;
    const int s_first = warp - 1 - (warp >> 2);  // producer index 0 .. kGtProducers-1
    int idxq[kGtQueue];
#pragma unroll
    for (int u = 0; u < kGtQueue; ++u) {
      const long long e = (long long)(s_first + u * kGtProducers) * kHvEdges + lane;
      idxq[u] = e < deg ? ld_stream(ind + e) : 0;
    }
    bool ok = true;
    for (int s0 = s_first; s0 < n_stages && ok; s0 += kGtQueue * kGtProducers) {
#pragma unroll
      for (int u = 0; u < kGtQueue; ++u) {
        const int s = s0 + u * kGtProducers;
        if (s < n_stages && ok) {
          const int slot = s & (kGtSlots - 1);
          const unsigned round = (unsigned)(s / kGtSlots);
          // slot handed back by the consumer?  (passes at once in round 0)
          ok = mbar_wait_park(&empty_bar[slot], (round & 1u) ^ 1u, kGtMaxPolls);
          if (ok) {
            const int cnt = min(kHvEdges, deg - s * kHvEdges);
            const int my_idx = idxq[u];
            const long long e_ahead =
                (long long)(s + kGtQueue * kGtProducers) * kHvEdges + lane;
            idxq[u] = e_ahead < deg ? ld_stream(ind + e_ahead) : 0;
            if (lane < cnt) cp_async4(&val_s[slot][lane], val + s * kHvEdges + lane);
#pragma unroll
            for (int k = 0; k < kCopies; ++k) {
              const int e = first + kRowsPerCopy * k;
              const int c = __shfl_sync(kFull, my_idx, e);
              if (e < cnt) cp_async16_cg(&xs[slot][e][part], xbase + (size_t)c * F);
            }
            cp_async_arrive_on(&full_bar[slot]);
          }
        }
      }
    }
    if (!ok && lane == 0) atomicExch(status, kGtErrProducerTimeout);
    cp_async_wait_all();
    return;
  }

  // -------------------------------------------------------------- consumer --
  // Software pipeline over the full stages: while the products of stage i are
  // being added (the dependent chain), the segments of stage i+1 are read from
  // shared memory and multiplied into a second register set.  A stage's slot is
  // handed back as soon as its products sit in registers.
  float acc_a = 0.f, acc_b = 0.f;
  float pa[kHvEdges], pb[kHvEdges], qa[kHvEdges], qb[kHvEdges];
  const int n_full = deg / kHvEdges;
  bool ok = true;
  auto wait_stage = [&](int i) {
    return mbar_wait_spin(&full_bar[i & (kGtSlots - 1)], (unsigned)(i / kGtSlots) & 1u,
                          kGtMaxPolls);
  };
  auto release_stage = [&](int i) {
    __syncwarp();  // every lane has read the slot
    if (lane == 0) mbar_arrive(&empty_bar[i & (kGtSlots - 1)]);
  };
#define FG_GIANT_PRODUCTS(i, A, B)                                                        \
  do {                                                                                    \
    const float(*xt)[kSlab] = xs[(i) & (kGtSlots - 1)];                                   \
    const float* vt = val_s[(i) & (kGtSlots - 1)];                                        \
    _Pragma("unroll") for (int e4 = 0; e4 < kHvEdges; e4 += 4) {                          \
      const float4 v4 = *reinterpret_cast<const float4*>(vt + e4);                        \
      const float vv[4] = {v4.x, v4.y, v4.z, v4.w};                                       \
      _Pragma("unroll") for (int q = 0; q < 4; ++q) {                                     \
        if (VEC == 2) {                                                                   \
          const float2 xv = *reinterpret_cast<const float2*>(&xt[e4 + q][lane * 2]);      \
          A[e4 + q] = __fmul_rn(vv[q], xv.x);                                             \
          B[e4 + q] = __fmul_rn(vv[q], xv.y);                                             \
        } else {                                                                          \
          A[e4 + q] = __fmul_rn(vv[q], xt[e4 + q][lane]);                                 \
          B[e4 + q] = 0.f;                                                                \
        }                                                                                 \
      }                                                                                   \
    }                                                                                     \
  } while (0)
#define FG_GIANT_CHAIN(A, B)                                                              \
  do {                                                                                    \
    _Pragma("unroll") for (int e = 0; e < kHvEdges; ++e) {                                \
      acc_a = __fadd_rn(acc_a, A[e]);                                                     \
      if (VEC == 2) acc_b = __fadd_rn(acc_b, B[e]);                                       \
    }                                                                                     \
  } while (0)

  // products(i+1) and chain(i) share one basic block so that the compiler
  // interleaves the shared-memory reads and multiplies with the add chain.
  if (n_full > 0) {
    ok = wait_stage(0);
    if (ok) {
      FG_GIANT_PRODUCTS(0, pa, pb);
      release_stage(0);
    }
    int i = 0;
    while (ok && i + 2 < n_full) {
      ok = wait_stage(i + 1);
      if (!ok) break;
      FG_GIANT_PRODUCTS(i + 1, qa, qb);
      FG_GIANT_CHAIN(pa, pb);
      release_stage(i + 1);
      ok = wait_stage(i + 2);
      if (!ok) break;
      FG_GIANT_PRODUCTS(i + 2, pa, pb);
      FG_GIANT_CHAIN(qa, qb);
      release_stage(i + 2);
      i += 2;
    }
    // stage i is in (pa, pb); at most one more full stage follows
    if (ok && i + 1 < n_full) {
      ok = wait_stage(i + 1);
      if (ok) {
        FG_GIANT_PRODUCTS(i + 1, qa, qb);
        FG_GIANT_CHAIN(pa, pb);
        release_stage(i + 1);
        FG_GIANT_CHAIN(qa, qb);
      }
    } else if (ok) {
      FG_GIANT_CHAIN(pa, pb);
    }
  }
#undef FG_GIANT_PRODUCTS
#undef FG_GIANT_CHAIN
  if (ok && n_full < n_stages) {  // the ragged last stage
    ok = wait_stage(n_full);
    if (ok) {
      heavy_consume_stage<VEC>(xs[n_full & (kGtSlots - 1)], val_s[n_full & (kGtSlots - 1)],
                               deg - n_full * kHvEdges, lane, acc_a, acc_b);
      release_stage(n_full);
    }
  }
  if (!ok) {
    if (lane == 0) atomicExch(status, kGtErrConsumerTimeout);
    return;  // the row is not written; the host sees the status
  }
  heavy_store_row<VEC>(Y, (size_t)row * F + (size_t)sub * kSlab, lane, acc_a, acc_b);
}

// Fallback for any feat_len / alignment: one warp per row, lanes over features.
__global__ void __launch_bounds__(256)
spmm_generic_kernel(const int* __restrict__ indptr, const int* __restrict__ indices,
                    const float* __restrict__ vals, const float* __restrict__ X,
                    OutPtrs Y, long long n_rows, int F) {
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
      for (int q = 0; q < Y.n; ++q) Y.p[q][(size_t)row * F + f] = acc;
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
  int heavy_vec = 1;       // floats per lane of the heavy / giant kernels (1 or 2)
  int heavy_threshold = 0, giant_threshold = 0;
  // rows sorted by degree, descending: [0, n_giant) giant, then n_heavy heavy, then light
  int n_giant = 0, n_heavy = 0, n_light = 0;
  int64_t max_deg = 0, giant_nnz = 0, heavy_nnz = 0;
  int* rows_dev = nullptr;    // the whole sorted list
  int* status_dev = nullptr;  // set by a giant-kernel barrier wait that gave up
  cudaStream_t aux_giant = nullptr, aux_heavy = nullptr;
  cudaEvent_t fork_ev = nullptr, join_giant = nullptr, join_heavy = nullptr;
  int l2_bytes = 0, n_sms = 0;
};

namespace fg {

constexpr int kDefaultHeavyThreshold = 2048;
constexpr int kDefaultGiantThreshold = 32768;

static void plan_release(fg_spmm_plan* p) {
  if (!p) return;
  DeviceGuard g(p->device);
  if (p->rows_dev) cudaFree(p->rows_dev);
  if (p->status_dev) cudaFree(p->status_dev);
  if (p->fork_ev) cudaEventDestroy(p->fork_ev);
  if (p->join_giant) cudaEventDestroy(p->join_giant);
  if (p->join_heavy) cudaEventDestroy(p->join_heavy);
  if (p->aux_giant) cudaStreamDestroy(p->aux_giant);
  if (p->aux_heavy) cudaStreamDestroy(p->aux_heavy);
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
  // An explicit threshold (tests use tiny ones) also scales the giant class down.
  p->giant_threshold =
      heavy_threshold > 0 ? std::min(kDefaultGiantThreshold, 16 * heavy_threshold)
                          : kDefaultGiantThreshold;
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
  FG_PLAN_TRY(cudaDeviceGetAttribute(&p->n_sms, cudaDevAttrMultiProcessorCount, device));
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
    auto degree_at = [&](int64_t k) {
      return (int64_t)indptr[order[(size_t)k] + 1] - indptr[order[(size_t)k]];
    };
    // Giant class: rows over the giant threshold, but no more (row, slab) CTAs
    // than SMs -- a giant CTA wants an SM's worth of copy bandwidth to itself.
    const int64_t giant_cap = std::max<int64_t>(1, p->n_sms / (feat_len / (32 * p->heavy_vec)));
    int64_t k = 0;
    while (k < n_rows && k < giant_cap && degree_at(k) > p->giant_threshold) p->giant_nnz += degree_at(k++);
    p->n_giant = (int)k;
    while (k < n_rows && degree_at(k) > p->heavy_threshold) p->heavy_nnz += degree_at(k++);
    p->n_heavy = (int)(k - p->n_giant);
    p->n_light = (int)(n_rows - k);

    FG_PLAN_TRY(cudaMalloc(&p->rows_dev, sizeof(int32_t) * (size_t)n_rows));
    FG_PLAN_TRY(cudaMemcpy(p->rows_dev, order.data(), sizeof(int32_t) * (size_t)n_rows,
                           cudaMemcpyHostToDevice));
    if (p->n_giant + p->n_heavy > 0) {
      int lo = 0, hi = 0;
      FG_PLAN_TRY(cudaDeviceGetStreamPriorityRange(&lo, &hi));
      FG_PLAN_TRY(cudaEventCreateWithFlags(&p->fork_ev, cudaEventDisableTiming));
      if (p->n_giant > 0) {
        FG_PLAN_TRY(cudaFuncSetAttribute(spmm_giant_kernel<1>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         giant_smem_bytes<1>()));
        FG_PLAN_TRY(cudaFuncSetAttribute(spmm_giant_kernel<2>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         giant_smem_bytes<2>()));
        FG_PLAN_TRY(cudaStreamCreateWithPriority(&p->aux_giant, cudaStreamNonBlocking, hi));
        FG_PLAN_TRY(cudaEventCreateWithFlags(&p->join_giant, cudaEventDisableTiming));
        FG_PLAN_TRY(cudaMalloc(&p->status_dev, sizeof(int)));
        FG_PLAN_TRY(cudaMemset(p->status_dev, 0, sizeof(int)));
      }
      if (p->n_heavy > 0) {
        FG_PLAN_TRY(cudaFuncSetAttribute(spmm_heavy_kernel<1>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         heavy_smem_bytes<1>()));
        FG_PLAN_TRY(cudaFuncSetAttribute(spmm_heavy_kernel<2>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         heavy_smem_bytes<2>()));
        FG_PLAN_TRY(cudaStreamCreateWithPriority(&p->aux_heavy, cudaStreamNonBlocking, hi));
        FG_PLAN_TRY(cudaEventCreateWithFlags(&p->join_heavy, cudaEventDisableTiming));
      }
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

extern "C" int fg_spmm_plan_status(const fg_spmm_plan* p, int32_t* device_status) {
  using namespace fg;
  if (!p || !device_status) return fail(FG_ERR_INVALID_ARGUMENT, "null plan or output");
  *device_status = 0;
  if (!p->status_dev) return FG_OK;
  DeviceGuard guard(p->device);
  FG_CUDA_TRY(cudaDeviceSynchronize());
  int v = 0;
  FG_CUDA_TRY(cudaMemcpy(&v, p->status_dev, sizeof(int), cudaMemcpyDeviceToHost));
  *device_status = v;
  if (v != 0)
    return fail(FG_ERR_CUDA, "spmm_giant_kernel: a bounded barrier wait gave up (code %d: %s warp)",
                v, v == kGtErrProducerTimeout ? "producer" : "consumer");
  return FG_OK;
}

extern "C" int fg_spmm_plan_num_launches(const fg_spmm_plan* p) {
  if (!p || p->n_rows == 0) return 0;
  if (!p->vector_ok) return 1;
  return (p->n_giant > 0 ? 1 : 0) + (p->n_heavy > 0 ? 1 : 0) + (p->n_light > 0 ? 1 : 0);
}

extern "C" int fg_spmm_plan_describe(const fg_spmm_plan* p, char* buf, int64_t buf_len) {
  using namespace fg;
  if (!p || !buf || buf_len <= 0) return fail(FG_ERR_INVALID_ARGUMENT, "null plan or buffer");
  if (p->vector_ok) {
    const int G = p->slab_w / 4;
    const int hv_slabs = p->feat_len / (32 * p->heavy_vec);
    const long long light_items = (long long)p->n_light * (p->feat_len / p->slab_w);
    snprintf(buf, (size_t)buf_len,
             "spmm_csr_f32 rows=%lld cols=%lld nnz=%lld feat_len=%d max_deg=%lld | L2=%d B "
             "slab_w=%d | light: %d rows (deg<=%d) -> spmm_light_kernel<G=%d> grid=%lld x 256 thr | "
             "heavy: %d rows (deg<=%d), %lld nnz -> spmm_heavy_kernel<VEC=%d> grid=%lld x 32 thr, "
             "%d-stage cp.async ring, own stream | giant: %d rows, %lld nnz -> "
             "spmm_giant_kernel<VEC=%d> grid=%lld x %d thr (%d producer warps + 1 consumer, "
             "%d-slot ring, mbarriers), own stream",
             (long long)p->n_rows, (long long)p->n_cols, (long long)p->nnz, p->feat_len,
             (long long)p->max_deg, p->l2_bytes, p->slab_w, p->n_light, p->heavy_threshold, G,
             (light_items + 256 / G - 1) / (256 / G), p->n_heavy, p->giant_threshold,
             (long long)p->heavy_nnz, p->heavy_vec, (long long)p->n_heavy * hv_slabs, kHvXSlots,
             p->n_giant, (long long)p->giant_nnz, p->heavy_vec, (long long)p->n_giant * hv_slabs,
             32 * kGtWarps, kGtProducers, kGtSlots);
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
                         const float* vals, const float* x, const OutPtrs& y, cudaStream_t st) {
  const long long items = (long long)p->n_light * (p->feat_len / (4 * G));
  const long long grid = (items + 256 / G - 1) / (256 / G);
  spmm_light_kernel<G><<<(unsigned)grid, 256, 0, st>>>(
      indptr, indices, vals, x, y, p->rows_dev + p->n_giant + p->n_heavy, p->n_light, items,
      p->feat_len);
}

}  // namespace fg

extern "C" int fg_spmm_csr_f32_multi(const fg_spmm_plan* p, const int32_t* indptr,
                                     const int32_t* indices, const float* vals, const float* x,
                                     float* const* ys, int32_t n_ys, void* stream) {
  using namespace fg;
  if (!p) return fail(FG_ERR_INVALID_ARGUMENT, "plan is null");
  if (!ys || n_ys < 1 || n_ys > kMaxOutputs)
    return fail(FG_ERR_INVALID_ARGUMENT, "need 1 to %d output pointers, got %d", kMaxOutputs,
                (int)n_ys);
  if (p->n_rows == 0) return FG_OK;
  OutPtrs y;
  y.n = n_ys;
  bool aligned = reinterpret_cast<uintptr_t>(x) % 16 == 0;
  for (int q = 0; q < kMaxOutputs; ++q) {
    y.p[q] = q < n_ys ? ys[q] : nullptr;
    if (q < n_ys && !ys[q]) return fail(FG_ERR_INVALID_ARGUMENT, "output pointer %d is null", q);
    if (q < n_ys && reinterpret_cast<uintptr_t>(ys[q]) % 16 != 0) aligned = false;
  }
  if (!indptr) return fail(FG_ERR_INVALID_ARGUMENT, "indptr_dev is null");
  if (p->nnz > 0 && (!indices || !vals || !x))
    return fail(FG_ERR_INVALID_ARGUMENT, "indices_dev, vals_dev or x_dev is null");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  DeviceGuard guard(p->device);
  if (guard.status != cudaSuccess)
    return fail(FG_ERR_CUDA, "cannot select device %d: %s", p->device,
                cudaGetErrorString(guard.status));

  if (!p->vector_ok || !aligned) {
    const long long grid = (p->n_rows + 7) / 8;
    spmm_generic_kernel<<<(unsigned)grid, 256, 0, st>>>(indptr, indices, vals, x, y, p->n_rows,
                                                        p->feat_len);
    FG_CUDA_TRY(cudaGetLastError());
    return FG_OK;
  }

  // Fork: giant and heavy rows run on the plan's own high-priority streams, the
  // longest first, while the light kernel fills the rest of the machine; the
  // caller's stream joins both before the call returns control to it.
  const int slab = 32 * p->heavy_vec;
  const int hv_slabs = p->feat_len / slab;
  if (p->fork_ev) FG_CUDA_TRY(cudaEventRecord(p->fork_ev, st));
  if (p->n_giant > 0) {
    FG_CUDA_TRY(cudaStreamWaitEvent(p->aux_giant, p->fork_ev, 0));
    const unsigned grid = (unsigned)(p->n_giant * hv_slabs);
    const unsigned threads = 32 * kGtWarps;
    if (p->heavy_vec == 2)
      spmm_giant_kernel<2><<<grid, threads, giant_smem_bytes<2>(), p->aux_giant>>>(
          indptr, indices, vals, x, y, p->rows_dev, p->n_giant, p->slab_w / slab, p->feat_len,
          p->status_dev);
    else
      spmm_giant_kernel<1><<<grid, threads, giant_smem_bytes<1>(), p->aux_giant>>>(
          indptr, indices, vals, x, y, p->rows_dev, p->n_giant, p->slab_w / slab, p->feat_len,
          p->status_dev);
    FG_CUDA_TRY(cudaGetLastError());
    FG_CUDA_TRY(cudaEventRecord(p->join_giant, p->aux_giant));
  }
  if (p->n_heavy > 0) {
    FG_CUDA_TRY(cudaStreamWaitEvent(p->aux_heavy, p->fork_ev, 0));
    const long long items = (long long)p->n_heavy * hv_slabs;
    if (items >= INT32_MAX) return fail(FG_ERR_UNSUPPORTED, "too many heavy items");
    if (p->heavy_vec == 2)
      spmm_heavy_kernel<2><<<(unsigned)items, 32, heavy_smem_bytes<2>(), p->aux_heavy>>>(
          indptr, indices, vals, x, y, p->rows_dev + p->n_giant, p->n_heavy, p->slab_w / slab,
          p->feat_len);
    else
      spmm_heavy_kernel<1><<<(unsigned)items, 32, heavy_smem_bytes<1>(), p->aux_heavy>>>(
          indptr, indices, vals, x, y, p->rows_dev + p->n_giant, p->n_heavy, p->slab_w / slab,
          p->feat_len);
    FG_CUDA_TRY(cudaGetLastError());
    FG_CUDA_TRY(cudaEventRecord(p->join_heavy, p->aux_heavy));
  }
  if (p->n_light > 0) {
    switch (p->slab_w) {
      case 128: launch_light<32>(p, indptr, indices, vals, x, y, st); break;
      case 64: launch_light<16>(p, indptr, indices, vals, x, y, st); break;
      default: launch_light<8>(p, indptr, indices, vals, x, y, st); break;
    }
    FG_CUDA_TRY(cudaGetLastError());
  }
  if (p->n_giant > 0) FG_CUDA_TRY(cudaStreamWaitEvent(st, p->join_giant, 0));
  if (p->n_heavy > 0) FG_CUDA_TRY(cudaStreamWaitEvent(st, p->join_heavy, 0));
  return FG_OK;
}

extern "C" int fg_spmm_csr_f32(const fg_spmm_plan* p, const int32_t* indptr,
                               const int32_t* indices, const float* vals, const float* x,
                               float* y, void* stream) {
  if (p && p->n_rows > 0 && !y)
    return fg::fail(FG_ERR_INVALID_ARGUMENT, "indptr_dev or y_dev is null");
  float* ys[1] = {y};
  return fg_spmm_csr_f32_multi(p, indptr, indices, vals, x, ys, 1, stream);
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
