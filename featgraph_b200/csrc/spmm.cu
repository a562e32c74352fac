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
// each with its own kernel; the three are launched back to back in one stream, giant rows
// first, each dispatched behind the one before it without waiting for it to complete
// (programmatic dependent launch), so that they overlap:
//   * light rows (deg <= max(2048, call estimate / 400 cycles)) -> spmm_light_kernel: a
//       group of G = W/4 lanes owns one (row, W-float feature slab); float4 gathers
//       straight into registers, 8 in flight per lane, index/value tile fetched one
//       iteration ahead; rows are served in descending degree so that the groups of a
//       warp finish together.  The cheapest path per nonzero: nothing crosses shared
//       memory.
//   * heavy rows -> spmm_heavy_kernel: one warp owns one (row, 32- or 64-float
//       slab); indices/values and the gathered X segments are staged through
//       shared memory with cp.async rings, which takes the gather latency off
//       the sequential add chain.
//   * giant rows (the few whose chain would outlast its share of the call) ->
//       spmm_chain_kernel<GiantShape>: one CTA per (row, 32-float slab); nine producer
//       warps gather, multiply and store transposed products into a shared-memory
//       ring, one consumer warp only adds, in order, at 5.5 cycles per nonzero
//       (the dependent fp32 add alone takes 4.2).  The longest row bounds the
//       whole call -- its sum is one dependent chain.
//   * anything the vector paths cannot take (feat_len not a multiple of 32,
//     unaligned pointers) -> spmm_generic_kernel, one warp per row.
// With feat_len wider than the slab of X that stays in L2, that trio runs once per slab,
// one trio after the other.
// Every kernel is a template over a message operator and a reducer (common.cuh); multiply
// with sum is the reference's SpMM, the other pairs are the generalised form.
// At the end of the file: SpMM over the reference's column-blocked (DDS) form, as one CSR
// call per column block whose stores add to the output.
#include <algorithm>
#include <cstring>
#include <vector>

#include "common.cuh"

namespace fg {

// ------------------------------------------------------------------ kernels --

// One group of G lanes per (row, slab) item; W = 4 * G floats per slab; U gathers of 16
// bytes in flight per lane (a row advances U nonzeros per gather latency).
// MSG / RED: message and reduce operators (FG_MSG_MUL with FG_REDUCE_SUM is the reference's
// SpMM; lhs = the gathered X element, rhs = the edge value).
template <int G, int U, int MSG, int RED>
__global__ void __launch_bounds__(256, U <= 8 ? 4 : 2)
spmm_light_kernel(const int* __restrict__ indptr, const int* __restrict__ indices,
                  const float* __restrict__ vals, const float* __restrict__ X,
                  const __grid_constant__ OutPtrs Y, const int* __restrict__ rows, int n_listed,
                  long long n_items, int F) {
  constexpr unsigned kFull = 0xffffffffu;
  launch_dependents();  // a kernel launched programmatically behind this one may be dispatched
  constexpr int T = G > U ? G : U;  // nonzeros per index / value tile: one per lane, or two
  constexpr int PER = T / G;        // index words per lane and tile
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
  float2 acc_lo = make_float2(red_identity<RED>(), red_identity<RED>()), acc_hi = acc_lo;
  // acc <- reduce(acc, msg(x, v)) on the lane's four features; the reference's pair takes
  // the packed-add form
  auto fold = [&](float vu, const float4& xv) {
    if (MSG == FG_MSG_MUL && RED == FG_REDUCE_SUM) {
      acc_lo = mul_then_add2(acc_lo, vu, make_float2(xv.x, xv.y));
      acc_hi = mul_then_add2(acc_hi, vu, make_float2(xv.z, xv.w));
    } else {
      acc_lo.x = combine<MSG, RED>(acc_lo.x, xv.x, vu);
      acc_lo.y = combine<MSG, RED>(acc_lo.y, xv.y, vu);
      acc_hi.x = combine<MSG, RED>(acc_hi.x, xv.z, vu);
      acc_hi.y = combine<MSG, RED>(acc_hi.y, xv.w, vu);
    }
  };

  // Index/value tile of the NEXT iteration, fetched one iteration ahead so that
  // its DRAM latency overlaps the gathers of the current one.
  int idx_next[PER];
  float v_next[PER];
#pragma unroll
  for (int p = 0; p < PER; ++p) {
    idx_next[p] = 0;
    v_next[p] = 0.f;
    if (p * G + gl < end - e) {
      idx_next[p] = ld_stream(indices + e + p * G + gl);
      v_next[p] = ld_stream(vals + e + p * G + gl);
    }
  }

  // The loop is warp-uniform: groups whose row is exhausted idle (cnt <= 0).
  while (__any_sync(kFull, e < end)) {
    const int cnt = end - e;
    int idx[PER];
    float v[PER];
#pragma unroll
    for (int p = 0; p < PER; ++p) {
      idx[p] = idx_next[p];
      v[p] = v_next[p];
      idx_next[p] = 0;
      v_next[p] = 0.f;
      if (p * G + gl < cnt - T) {
        idx_next[p] = ld_stream(indices + e + T + p * G + gl);
        v_next[p] = ld_stream(vals + e + T + p * G + gl);
      }
    }
#pragma unroll
    for (int j0 = 0; j0 < T; j0 += U) {
      float4 x[U];
      if (__all_sync(kFull, cnt >= j0 + U)) {
        // every group of the warp has a full batch: no predicates
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int c = __shfl_sync(kFull, idx[(j0 + u) / G], (j0 + u) % G, G);
          x[u] = ld_gather4(xcol + (size_t)c * F);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const float vu = __shfl_sync(kFull, v[(j0 + u) / G], (j0 + u) % G, G);
          fold(vu, x[u]);
        }
      } else {
        if (!__any_sync(kFull, j0 < cnt)) break;
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int c = __shfl_sync(kFull, idx[(j0 + u) / G], (j0 + u) % G, G);
          if (j0 + u < cnt) x[u] = ld_gather4(xcol + (size_t)c * F);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const float vu = __shfl_sync(kFull, v[(j0 + u) / G], (j0 + u) % G, G);
          if (j0 + u < cnt) fold(vu, x[u]);
        }
      }
    }
    if (cnt > 0) e += (cnt < T ? cnt : T);
  }
  if (valid) {
    const size_t off = (size_t)row * F + col_off;
    out_store(Y, off, out_fold(Y, off, make_float4(acc_lo.x, acc_lo.y, acc_hi.x, acc_hi.y)));
  }
  // This grid may have been dispatched behind the heavy / giant kernels of the same call
  // without waiting for them; its last CTA stays until they have completed, so that "this
  // grid is complete" means "the whole SpMM is complete" to whatever follows in the stream.
  if (blockIdx.x == gridDim.x - 1) wait_for_prior_grids();
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
template <int VEC, int MSG, int RED>
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
          acc_a = combine<MSG, RED>(acc_a, xv.x, vv[q]);
          acc_b = combine<MSG, RED>(acc_b, xv.y, vv[q]);
        } else {
          acc_a = combine<MSG, RED>(acc_a, xt[e4 + q][lane], vv[q]);
        }
      }
    }
  } else {
    for (int e = 0; e < cnt; ++e) {
      if (VEC == 2) {
        const float2 xv = *reinterpret_cast<const float2*>(&xt[e][lane * 2]);
        acc_a = combine<MSG, RED>(acc_a, xv.x, vt[e]);
        acc_b = combine<MSG, RED>(acc_b, xv.y, vt[e]);
      } else {
        acc_a = combine<MSG, RED>(acc_a, xt[e][lane], vt[e]);
      }
    }
  }
}

template <int VEC>
__device__ __forceinline__ void heavy_store_row(const OutPtrs& Y, size_t slab_off, int lane,
                                                float acc_a, float acc_b) {
  if (VEC == 2)
    out_store(Y, slab_off + lane * 2, out_fold(Y, slab_off + lane * 2, make_float2(acc_a, acc_b)));
  else
    out_store(Y, slab_off + lane, out_fold(Y, slab_off + lane, acc_a));
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
template <int VEC, int MSG, int RED>
__global__ void __launch_bounds__(32)
spmm_heavy_kernel(const int* __restrict__ indptr, const int* __restrict__ indices,
                  const float* __restrict__ vals, const float* __restrict__ X,
                  const __grid_constant__ OutPtrs Y, const int* __restrict__ rows, int n_listed,
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

  launch_dependents();  // the next kernel of the call may be dispatched behind this CTA
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
  float acc_a = red_identity<RED>(), acc_b = red_identity<RED>();
  for (int i = 0; i < n_stages; ++i) {
    cp_async_wait<kHvDist - 1>();  // stage i's gathers and stage i+D's indices landed
    __syncwarp();                  // ... for every lane; stage i-1 is fully consumed
    issue_gather(i + kHvDist);
    issue_idx(i + 2 * kHvDist);
    cp_async_commit();
    heavy_consume_stage<VEC, MSG, RED>(xs[i & (kHvXSlots - 1)], val_s[i & (kHvISlots - 1)],
                             min(kHvEdges, deg - i * kHvEdges), lane, acc_a, acc_b);
  }
  cp_async_wait<0>();
  heavy_store_row<VEC>(Y, (size_t)row * F + (size_t)sub * kSlab, lane, acc_a, acc_b);
  if (blockIdx.x == gridDim.x - 1) wait_for_prior_grids();  // as in spmm_light_kernel
}

// Shape of a chain CTA (spmm_chain_kernel): warp 0 consumes, the others produce.
//   WARPS      warps per CTA
//   PRODUCERS  producer warps
//   GROUP      32-nonzero blocks per group: one hand-over per group
//   GROUPS     groups in the ring of products
//   RETIRE     the warps that would share the consumer's scheduler (ids 4, 8, ...) retire
//   MIN_CTAS   CTAs per SM the register allocation must allow
template <int WARPS_, int PRODUCERS_, int GROUP_, int GROUPS_, bool RETIRE_, int MIN_CTAS_>
struct ChainShape {
  static constexpr int WARPS = WARPS_, PRODUCERS = PRODUCERS_, GROUP = GROUP_, GROUPS = GROUPS_;
  static constexpr bool RETIRE = RETIRE_;
  static constexpr int MIN_CTAS = MIN_CTAS_;
  static constexpr int RING = GROUP * GROUPS;  // blocks in the ring
  static constexpr int SMEM_BYTES = RING * kHvEdges * 32 * 4  // products, [block][feature][nonzero]
                                    + (RING + 4) * 4;         // one flag per ring block, group counter
  // producers prefetch their index / value blocks into L2 about 200 row blocks ahead
  static constexpr int AHEAD = (216 / PRODUCERS + 2) / 3 * 3;
  static_assert(RING < 32 * WARPS && GROUP % 4 == 0 && GROUP >= 8 && GROUPS >= 2, "ring / group shape");
  static_assert(PRODUCERS == (RETIRE ? WARPS - 1 - (WARPS - 1) / 4 : WARPS - 1), "producer count");
};
// The giant rows: a whole SM per (row, 32-float slab), nine producers, a 48-block ring.
using GiantShape = ChainShape<12, 9, 16, 3, true, 1>;
// Smaller shapes (4 to 6 warps, rings of 16 to 32 blocks, two or three CTAs per SM) were
// built and measured as the kernel of the heavy class: one 30 000-nonzero row alone walks
// at 7.5 to 9.4 cycles per nonzero (the single-warp cp.async kernel: 24 alone, 45 beside
// others), but every product crosses shared memory twice, the L1/shared pipe saturates
// (75 %) at 0.17 (nonzero, 32-float slab) pairs per SM-cycle against 0.27 for the cp.async
// kernel and 0.5 for the group kernel, and the whole SpMM was slower with them (2.04 ms at
// best against 1.91).  So this kernel serves only the rows that need its speed.
constexpr unsigned kGtMaxPolls = 1u << 20;     // bound of every wait for a flag
constexpr int kGtErrProducerTimeout = 1, kGtErrConsumerTimeout = 2;

// Quad position of giant_kernel's product layout.  With it both the producers'
// 16-byte stores (8 lanes = 8 feature quads, one nonzero quad) and the consumer's
// 16-byte loads (8 lanes = 8 consecutive features, one nonzero quad) spread over
// all 32 banks.
__device__ __forceinline__ int giant_swizzle(int f) { return ((f >> 2) ^ f) & 7; }

// One CTA per (giant row, 32-float slab): a consumer warp and nine producer warps.
//
// The sum of one row is a dependent chain (CSR order, one accumulator per
// feature), so the longest row bounds the whole SpMM -- on several GPUs even more
// so, because the chain does not shrink with the shard -- and everything but the
// add itself has to stay off that chain: 4.2 cycles per nonzero is the dependent
// fp32 add alone.  What the measurements said, in cycles per block of 32 nonzeros
// (the chain bound is 135):
//   * a lone warp gathering by cp.async: 1500 (it keeps only a few copies
//     outstanding), so the gathers need several warps;
//   * a consumer that reads X segments from shared memory, multiplies and adds:
//     290 alone, 450 beside busy producers -- 32 four-byte loads, 32 multiplies
//     and the adds do not fit the chain's issue gaps; 8 sixteen-byte loads of
//     ready products do (139), hence products stored TRANSPOSED;
//   * an mbarrier test: 180 by a whole warp (32 lanes on one word), 50 to 100 by
//     one lane, and the instruction that takes the verdict out of the predicate
//     stalls the warp at once; a flag word read with a plain load can be read a
//     step before it is looked at.  Hence flag words (release / acquire), and a
//     hand-over only once per group of 16 blocks;
//   * a warp has six scoreboards for all its loads and shuffles in flight, so a
//     wait for a quick result (a shuffle) also waits for whatever slow load shares
//     its scoreboard: software pipelines across batches of gathers ran at one
//     memory latency per step whatever their depth.  Hence batches.
// Producer w takes blocks w, w+9, w+18, ... of the row, three per batch: all the
// batch's shuffles (each lane's 8 columns and values out of the warp's coalesced
// copy), then its 24 gathers of 16 bytes and the next batch's columns / values, then,
// per block, the multiplies, the lane's 8x4 tile transposed in registers, 8
// sixteen-byte stores into the ring block and the block's flag.  The consumer (lane =
// feature) holds the next three blocks in registers while it adds the current one,
// loads alternating with adds in one basic block; it checks a whole group's flags at
// once and hands a group back when its last block sits in registers.  Result: 5.5
// cycles per nonzero (14.3 with row-major segments and per-block mbarriers).
// Every wait is a bounded poll (max_polls); a wait that gives up is recorded in *status
// (the first code sticks) and the row's slab is then filled with NaN.
template <class S_, int MSG, int RED>
__global__ void __launch_bounds__(32 * S_::WARPS, S_::MIN_CTAS)
spmm_chain_kernel(const int* __restrict__ indptr, const int* __restrict__ indices,
                  const float* __restrict__ vals, const float* __restrict__ X,
                  const __grid_constant__ OutPtrs Y, const int* __restrict__ rows, int n_listed,
                  int subs_per_slab, int F, int* __restrict__ status, unsigned max_polls) {
  constexpr unsigned kFull = 0xffffffffu;
  launch_dependents();  // the next kernel of the call may be dispatched behind this CTA
  constexpr int kGtProducers = S_::PRODUCERS, kGtGroup = S_::GROUP, kGtGroups = S_::GROUPS;
  constexpr int kGtRing = S_::RING;
  extern __shared__ __align__(16) unsigned char giant_smem[];
  // prod[block][feature][nonzero]: a feature's 32 products of a block are 8 quads of 4
  // consecutive nonzeros, stored at quad position q ^ giant_swizzle(feature)
  float(*prod)[32][kHvEdges] = reinterpret_cast<float(*)[32][kHvEdges]>(giant_smem);
  // ready[s] = 1 + the number of the block whose products sit in ring block s (written
  // by its producer); *consumed = groups the consumer has handed back
  unsigned* ready = reinterpret_cast<unsigned*>(giant_smem + kGtRing * kHvEdges * 32 * 4);
  unsigned* consumed = ready + kGtRing;

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  int row, sub;
  heavy_decode_item(rows, n_listed, subs_per_slab, row, sub);
  const int beg = __ldg(indptr + row);
  const int deg = __ldg(indptr + row + 1) - beg;
  const int n_blocks = (deg + kHvEdges - 1) / kHvEdges;  // incl. a ragged last one

  if (threadIdx.x <= kGtRing) ready[threadIdx.x] = 0;  // the last one is *consumed
  __syncthreads();

  // Warps are dealt to the SM's four schedulers round-robin by id: warps 4 and 8 would
  // share the consumer's and retire at once (measured: 5.5 cycles per nonzero this way,
  // 6.3 with producers on the consumer's scheduler).
  if (S_::RETIRE && warp > 0 && (warp & 3) == 0) return;
  if (warp > 0) {
    // ------------------------------------------------------------ producer --
    const int* ind = indices + beg;
    const float* val = vals + beg;
    const int pw = S_::RETIRE ? warp - 1 - (warp >> 2) : warp - 1;  // producer index 0 .. P-1
    const int m = lane & 7;                 // this lane's feature quad: 4m .. 4m+3
    const int g8 = (lane >> 3) * 8;         // and its nonzeros within a block: g8 .. g8+7
    const float* xbase = X + (size_t)sub * 32 + 4 * m;
    // the producer's own sequence of blocks u = 0, 1, 2, ...: block pw + u * P of the row
    int my_blocks = 0;
    if (pw < n_blocks) my_blocks = (n_blocks - pw + kGtProducers - 1) / kGtProducers;
    auto load_iv = [&](int u, int& c, float& v) {
      const long long e = (long long)(pw + u * kGtProducers) * kHvEdges + lane;
      c = e < deg ? ld_stream(ind + e) : 0;
      v = e < deg ? ld_stream(val + e) : 0.f;
    };
    auto prefetch_iv = [&](int u) {
      const long long e = (long long)(pw + u * kGtProducers) * kHvEdges + lane;
      if (e < deg && (lane & 7) == 0) {  // one request per 32-byte sector
        asm volatile("prefetch.global.L2 [%0];" ::"l"(ind + e));
        asm volatile("prefetch.global.L2 [%0];" ::"l"(val + e));
      }
    };
    // this lane's eight columns / values of a block, out of the warp's coalesced copy
    auto spread = [&](int c, float v, int (&col)[8], float (&vs)[8]) {
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        col[k] = __shfl_sync(kFull, c, g8 + k);
        vs[k] = __shfl_sync(kFull, v, g8 + k);
      }
    };
    auto gather = [&](int u, const int (&col)[8], float4 (&x)[8]) {
      const long long left = (long long)deg - (long long)(pw + u * kGtProducers) * kHvEdges;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        x[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (g8 + k < left) x[k] = ld_gather4(xbase + (size_t)col[k] * F);
      }
    };
    bool ok = true;
    int entered = -1;  // last group this warp has found handed back
    auto emit = [&](int u, const float (&vs)[8], const float4 (&x)[8]) {
      const int b = pw + u * kGtProducers;
      const int grp = b / kGtGroup;
      float4 pr[8];
#pragma unroll
      for (int k = 0; k < 8; ++k)
        pr[k] = make_float4(msg_apply<MSG>(x[k].x, vs[k]), msg_apply<MSG>(x[k].y, vs[k]),
                            msg_apply<MSG>(x[k].z, vs[k]), msg_apply<MSG>(x[k].w, vs[k]));
      if (grp != entered) {
        if (grp >= kGtGroups) {  // the ring block has held group grp - kGtGroups: handed back?
          int got = 0;
          if (lane == 0) {
            const unsigned need = (unsigned)(grp - kGtGroups + 1);
            for (unsigned i = 0; i < max_polls && !got; ++i) {
              got = ld_acquire_shared(consumed) >= need;
              if (!got) __nanosleep(64);
            }
          }
          __syncwarp();  // lane 0's acquire covers the warp
          ok = __shfl_sync(kFull, got, 0) != 0;
          if (!ok) return;
        }
        entered = grp;
      }
      // the lane holds an 8-nonzero x 4-feature tile: transposed in registers, it
      // leaves as 8 quads (one feature, 4 consecutive nonzeros each)
      float(*pt)[kHvEdges] = prod[b % kGtRing];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int q = (g8 >> 2) + h;  // quad of nonzeros g8 + 4h .. g8 + 4h + 3
        *reinterpret_cast<float4*>(&pt[4 * m + 0][(q ^ giant_swizzle(4 * m + 0)) << 2]) =
            make_float4(pr[4 * h].x, pr[4 * h + 1].x, pr[4 * h + 2].x, pr[4 * h + 3].x);
        *reinterpret_cast<float4*>(&pt[4 * m + 1][(q ^ giant_swizzle(4 * m + 1)) << 2]) =
            make_float4(pr[4 * h].y, pr[4 * h + 1].y, pr[4 * h + 2].y, pr[4 * h + 3].y);
        *reinterpret_cast<float4*>(&pt[4 * m + 2][(q ^ giant_swizzle(4 * m + 2)) << 2]) =
            make_float4(pr[4 * h].z, pr[4 * h + 1].z, pr[4 * h + 2].z, pr[4 * h + 3].z);
        *reinterpret_cast<float4*>(&pt[4 * m + 3][(q ^ giant_swizzle(4 * m + 3)) << 2]) =
            make_float4(pr[4 * h].w, pr[4 * h + 1].w, pr[4 * h + 2].w, pr[4 * h + 3].w);
      }
      __syncwarp();  // every lane's stores are ordered before lane 0's release
      if (lane == 0) st_release_shared(&ready[b % kGtRing], (unsigned)b + 1u);
    };
    // Batches of three blocks.  A warp has six scoreboards for all its loads and
    // shuffles in flight, so a wait for any one result tends to wait for the newest
    // load as well; the batch is therefore ordered to have nothing slow in flight
    // when something quick is waited for: (1) all shuffles of the batch (columns and
    // values per lane), (2) all 24 gathers, the next batch's columns / values (they
    // stream from DRAM, behind an L2 prefetch eight batches ahead) -- one exposed
    // latency for the lot -- (3) multiply, wait for the ring block, store, three times.
    float4 xa[8], xb[8], xc[8];
    float vsa[8], vsb[8], vsc[8];
    int ca, cb, cc;
    float va, vb, vc;
    load_iv(0, ca, va);
    load_iv(1, cb, vb);
    load_iv(2, cc, vc);
    for (int u = 0; u < my_blocks && ok; u += 3) {
      {
        int cola[8], colb[8], colc[8];
        spread(ca, va, cola, vsa);
        spread(cb, vb, colb, vsb);
        spread(cc, vc, colc, vsc);
        gather(u, cola, xa);
        gather(u + 1, colb, xb);
        gather(u + 2, colc, xc);
      }
      load_iv(u + 3, ca, va);
      load_iv(u + 4, cb, vb);
      load_iv(u + 5, cc, vc);
      prefetch_iv(u + S_::AHEAD);
      prefetch_iv(u + S_::AHEAD + 1);
      prefetch_iv(u + S_::AHEAD + 2);
      emit(u, vsa, xa);
      if (u + 1 < my_blocks && ok) emit(u + 1, vsb, xb);
      if (u + 2 < my_blocks && ok) emit(u + 2, vsc, xc);
    }
    if (!ok && lane == 0) atomicCAS(status, 0, kGtErrProducerTimeout);
    return;
  }

  // -------------------------------------------------------------- consumer --
  // lane = feature.  Block j lives in register set j % 4; blocks j+1 .. j+3 are
  // on their way from shared memory while block j is added.
  float acc = red_identity<RED>();
  const int n_full = deg / kHvEdges;
  // Every lane reads the flag itself (a broadcast): a relaxed load long before the
  // check, so that the check costs a compare; the fence behind a successful check
  // turns it into an acquire (every lane's loads of the block come after it).  A lane
  // whose bounded wait gives up only notes it; the warp looks at the notes at the end.
  auto peek = [&](int j) { return ld_relaxed_shared(&ready[j % kGtRing]); };
  bool gave_up = false;
  auto await = [&](int j, unsigned seen) {
    const unsigned want = (unsigned)j + 1u;
    if (seen != want && !gave_up) {  // rare: the producers are behind (once given up, no more waits)
      bool got = false;
      for (unsigned i = 0; i < max_polls && !got; ++i) got = peek(j) == want;
      gave_up |= !got;
    }
    fence_acquire_cta();
  };
  auto release_after = [&](int j) {  // after the reads of block j: its group, if j closes it
    if (j % kGtGroup == kGtGroup - 1) {
      __syncwarp();  // every lane's reads are ordered before lane 0's release
      if (lane == 0) st_release_shared(consumed, (unsigned)(j / kGtGroup) + 1u);
    }
  };
  const int swz = giant_swizzle(lane);
  auto fetch = [&](int j, float4 (&s)[8]) {  // prologue only
    if (j >= n_full) return;
    const float* src = prod[j % kGtRing][lane];
#pragma unroll
    for (int q = 0; q < 8; ++q) s[q] = *reinterpret_cast<const float4*>(src + ((q ^ swz) << 2));
    release_after(j);
  };
  // Adds the block in sa and reads block jf into sf.  The reads and the adds sit in ONE
  // basic block, alternating, so that the loads issue in the gaps of the dependent add
  // chain instead of ahead of it.
  auto core = [&](const float4 (&sa)[8], float4 (&sf)[8], int jf) {
    const float* src = prod[jf % kGtRing][lane];
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      sf[q] = *reinterpret_cast<const float4*>(src + ((q ^ swz) << 2));
      acc = red_apply<RED>(acc, sa[q].x);
      acc = red_apply<RED>(acc, sa[q].y);
      acc = red_apply<RED>(acc, sa[q].z);
      acc = red_apply<RED>(acc, sa[q].w);
    }
  };
  auto chain = [&](const float4 (&sa)[8]) {
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      acc = red_apply<RED>(acc, sa[q].x);
      acc = red_apply<RED>(acc, sa[q].y);
      acc = red_apply<RED>(acc, sa[q].z);
      acc = red_apply<RED>(acc, sa[q].w);
    }
  };
  // One block with its own flag check: the row's tail.
  unsigned seen = 0;  // flag of the block the next step reads, as of one step ago
  auto step = [&](int jc, const float4 (&sa)[8], float4 (&sf)[8]) {
    if (jc >= n_full) return;
    const int jf = jc + 3;
    if (jf < n_full) {
      await(jf, seen);
      core(sa, sf, jf);
      seen = peek(jf + 1);
      release_after(jf);
    } else {
      chain(sa);
    }
  };

  float4 S[4][8];  // indexed by constants only (the loops below unroll fully): registers
  for (int i = 0; i < kGtGroup && i < n_full; ++i) await(i, 0u);  // group 0, block by block
  fetch(0, S[0]);
  fetch(1, S[1]);
  fetch(2, S[2]);
  // Whole groups: blocks j (a multiple of the group size) .. j+2 sit in S[0] .. S[2] and
  // group j / kGtGroup has been checked.  Step s adds block j+s and reads block j+s+3.
  // The next group's flags are read two per step in the first steps, folded into one
  // word a step after they were read, and checked -- all at once, with the fence that
  // makes the check an acquire -- before the step that reads the next group's first
  // block; this group is handed back after the step that reads its last block.
  int j = 0;
  for (; j + 2 * kGtGroup <= n_full; j += kGtGroup) {
    const int nx = j + kGtGroup;
    const unsigned w = (unsigned)nx + 1u;
    unsigned mism = 0, pk0 = 0, pk1 = 0;
#pragma unroll
    for (int s = 0; s < kGtGroup; ++s) {
      if (s >= 1 && s <= kGtGroup / 2)
        mism |= (pk0 ^ (w + 2 * (s - 1))) | (pk1 ^ (w + 2 * (s - 1) + 1));
      if (s < kGtGroup / 2) {
        pk0 = peek(nx + 2 * s);
        pk1 = peek(nx + 2 * s + 1);
      }
      if (s == kGtGroup - 3) {
        if (mism != 0) {  // rare: the producers are behind; block by block then
          for (int i = 0; i < kGtGroup; ++i) await(nx + i, 0u);
        } else {
          fence_acquire_cta();
        }
      }
      core(S[s & 3], S[(s + 3) & 3], j + 3 + s);
      if (s == kGtGroup - 4) {
        __syncwarp();  // every lane's reads of the group are ordered before lane 0's release
        if (lane == 0) st_release_shared(consumed, (unsigned)(j / kGtGroup) + 1u);
      }
    }
  }
  // the tail: fewer than two groups of full blocks are left
  seen = peek(j + 3);
  for (; j < n_full; j += 4) {
    step(j, S[0], S[3]);
    step(j + 1, S[1], S[0]);
    step(j + 2, S[2], S[1]);
    step(j + 3, S[3], S[2]);
  }
  if (n_full < n_blocks) {  // the ragged last block, straight from shared memory
    await(n_full, 0u);
    const float* src = prod[n_full % kGtRing][lane];
    const int cnt = deg - n_full * kHvEdges;
    for (int e = 0; e < cnt; ++e) acc = red_apply<RED>(acc, src[(((e >> 2) ^ swz) << 2) | (e & 3)]);
  }
  if (__any_sync(kFull, gave_up)) {
    // No sum to report: the slab is filled with NaN so that a stale value of an earlier
    // call cannot pass for a result, and the host finds the code in the status word.
    if (lane == 0) atomicCAS(status, 0, kGtErrConsumerTimeout);
    heavy_store_row<1>(Y, (size_t)row * F + (size_t)sub * 32, lane, __int_as_float(0x7fc00000), 0.f);
    return;
  }
  heavy_store_row<1>(Y, (size_t)row * F + (size_t)sub * 32, lane, acc, 0.f);
  if (blockIdx.x == gridDim.x - 1) wait_for_prior_grids();  // as in spmm_light_kernel
}

// Fallback for any feat_len / alignment: one warp per row, lanes over features.
template <int MSG, int RED>
__global__ void __launch_bounds__(256)
spmm_generic_kernel(const int* __restrict__ indptr, const int* __restrict__ indices,
                    const float* __restrict__ vals, const float* __restrict__ X,
                    const __grid_constant__ OutPtrs Y, long long n_rows, int F) {
  launch_dependents();
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  const int beg = indptr[row], end = indptr[row + 1];
  for (int f0 = 0; f0 < F; f0 += 32) {
    const int f = f0 + lane;
    float acc = red_identity<RED>();
    if (f < F) {
      for (int e = beg; e < end; ++e)
        acc = combine<MSG, RED>(acc, X[(size_t)indices[e] * F + f], vals[e]);
      out_store(Y, (size_t)row * F + f, out_fold(Y, (size_t)row * F + f, acc));
    }
  }
  if (blockIdx.x == gridDim.x - 1) wait_for_prior_grids();  // as in spmm_light_kernel
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
  int heavy_threshold = 0, giant_threshold = 0;
  // rows sorted by degree, descending: [0, n_giant) giant, then n_heavy heavy, then light
  int n_giant = 0, n_heavy = 0, n_light = 0;
  int64_t max_deg = 0, giant_nnz = 0, heavy_nnz = 0;
  int* rows_dev = nullptr;    // the whole sorted list
  int* status_dev = nullptr;  // set by a giant-kernel wait that gave up
  unsigned poll_limit = 0;    // polls a chain-kernel wait makes before it gives up
  int l2_bytes = 0, n_sms = 0;
};

namespace fg {

constexpr int kDefaultHeavyThreshold = 2048;
constexpr int kMinGiantThreshold = 4096;
// Measured on B200 (1965 MHz, feat_len 64, the 114.6 M-edge power-law graph): the whole
// SpMM moves 50 (nonzero, 32-float slab) pairs per cycle on 148 SMs; the heavy kernel
// walks one row at 47 cycles per nonzero, the giant kernel at 5.6.
constexpr double kCyclesPerNnzSlab = 0.0197, kHeavyCyclesPerNnz = 47.0, kGiantCyclesPerNnz = 5.6;
// light/heavy boundary = estimated time of one residency-slab pass in cycles / this (11 289
// nonzeros for the 4.5 M-cycle estimate of the full graph at feat_len 64)
constexpr double kLightCyclesPerNnzOfPass = 400.0;
// heavy/giant boundary: rows whose chain in the heavy kernel would outlast this share of the call
constexpr double kGiantShareOfCall = 0.45;

static void plan_release(fg_spmm_plan* p) {
  if (!p) return;
  DeviceGuard g(p->device);
  if (p->rows_dev) cudaFree(p->rows_dev);
  if (p->status_dev) cudaFree(p->status_dev);
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

namespace fg {

// Rows by degree, descending, ties in row order (a stable sort): the hardware block
// scheduler then hands out the longest rows first, and the groups that share a warp get
// rows of (nearly) equal length.  A counting sort over the degrees below kSortCap (the
// table stays at 16 MiB whatever the longest row is); the few rows at or over the cap are
// sorted by comparison.
constexpr int64_t kSortCap = 1 << 22;
static void rows_by_degree(const int32_t* indptr, int64_t n_rows, int64_t max_deg,
                           std::vector<int32_t>& order) {
  auto deg = [&](int64_t r) { return (int64_t)indptr[r + 1] - indptr[r]; };
  order.resize((size_t)n_rows);
  const int64_t buckets = std::min<int64_t>(max_deg, kSortCap - 1) + 1;  // degrees 0 .. buckets-1
  std::vector<int32_t> longest;
  std::vector<int64_t> start((size_t)buckets + 1, 0);
  for (int64_t r = 0; r < n_rows; ++r) {
    const int64_t d = deg(r);
    if (d >= buckets) longest.push_back((int32_t)r);
    else start[(size_t)d]++;
  }
  std::stable_sort(longest.begin(), longest.end(),
                   [&](int32_t a, int32_t b) { return deg(a) > deg(b); });
  std::copy(longest.begin(), longest.end(), order.begin());
  // start[d] <- position of the first row of degree d
  int64_t running = (int64_t)longest.size();
  for (int64_t d = buckets - 1; d >= 0; --d) {
    const int64_t c = start[(size_t)d];
    start[(size_t)d] = running;
    running += c;
  }
  for (int64_t r = 0; r < n_rows; ++r) {
    const int64_t d = deg(r);
    if (d < buckets) order[(size_t)start[(size_t)d]++] = (int32_t)r;
  }
}

static int plan_create(const int32_t* indptr, int64_t n_rows, int64_t n_cols, int32_t feat_len,
                       int32_t device, int32_t heavy_threshold, fg_spmm_plan** out_plan) {
  if (!out_plan) return fail(FG_ERR_INVALID_ARGUMENT, "out_plan is null");
  *out_plan = nullptr;
  if (n_rows < 0 || n_cols < 0 || feat_len <= 0)
    return fail(FG_ERR_INVALID_ARGUMENT, "bad shape: n_rows=%lld n_cols=%lld feat_len=%d",
                (long long)n_rows, (long long)n_cols, (int)feat_len);
  if (n_rows >= INT32_MAX || n_cols >= INT32_MAX)
    return fail(FG_ERR_UNSUPPORTED, "row/column counts must fit int32");
  if (!indptr) return fail(FG_ERR_INVALID_ARGUMENT, "indptr_host is null");
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
  p->nnz = (int64_t)indptr[n_rows] - indptr[0];
  p->feat_len = feat_len;
  p->max_deg = max_deg;
  p->heavy_threshold = heavy_threshold > 0 ? heavy_threshold : kDefaultHeavyThreshold;
  p->vector_ok = (feat_len % 32 == 0);
  p->poll_limit = kGtMaxPolls;

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
  {
    // Giant class: the rows whose add chain, walked by the heavy kernel's single warp,
    // would last more than kGiantShareOfCall of a trio (the three kernels' pass over one
    // residency slab).  The trio is estimated as the longer of
    // its throughput time and the longest row's chain in the giant kernel; a shard of
    // a multi-GPU run has less of the former, so more of its rows turn giant.  The
    // giant kernel gives an SM to 32 floats of one row, so it is kept for such rows.
    // (one giant / heavy / light trio covers one residency slab of every row: slab_w floats)
    const double t_throughput = (double)p->nnz * (p->slab_w / 32.0) * kCyclesPerNnzSlab * 148.0 /
                                std::max(1, p->n_sms);
    const double t_call = std::max(t_throughput, (double)max_deg * kGiantCyclesPerNnz);
    // Heavy class: the light kernel moves about twice the nonzeros per SM-cycle of the heavy
    // one (its gathers go straight to registers; the heavy and giant kernels pass every
    // gathered byte through shared memory) but walks a row at about one gather latency per 8
    // nonzeros, so it keeps every row whose walk fits inside the call.  Measured on the full
    // graph at feat_len 64 with an SDDMM between the calls, as in a GNN layer (ms per call;
    // light boundary / giant boundary in nonzeros): 4105 / 57648: 2.18, 8210 / 57648: 2.11,
    // 8210 / 38432: 2.01, 11289 / 43236: 1.91, 11289 / 38432: 1.92, 12204 / 43236: 1.92,
    // 11289 / 28824: 1.98, 15052 / 38432: 2.12, 22579 / 57648: 2.56.
    if (heavy_threshold <= 0)
      p->heavy_threshold = (int)std::min<double>(
          1 << 20, std::max<double>(kDefaultHeavyThreshold, t_call / kLightCyclesPerNnzOfPass));
    const double by_time = kGiantShareOfCall * t_call / kHeavyCyclesPerNnz;
    int64_t thr = (int64_t)std::min(by_time, 1e9);
    thr = std::max<int64_t>(thr, kMinGiantThreshold);
    // an explicit heavy threshold (tests use tiny ones) scales the giant class down with it
    if (heavy_threshold > 0) thr = std::min<int64_t>(thr, 16 * (int64_t)heavy_threshold);
    p->giant_threshold = (int)std::max<int64_t>(thr, p->heavy_threshold);
  }

  if (p->vector_ok && n_rows > 0) {
    std::vector<int32_t> order;
    try {
      rows_by_degree(indptr, n_rows, max_deg, order);
    } catch (const std::bad_alloc&) {
      plan_release(p);
      return fail(FG_ERR_OUT_OF_MEMORY, "fg_spmm_plan_create: host allocation failed");
    }
    auto degree_at = [&](int64_t k) {
      return (int64_t)indptr[order[(size_t)k] + 1] - indptr[order[(size_t)k]];
    };
    // Giant class: the rows over the giant threshold, as long as their (row, 32-float
    // slab) CTAs fit a 32-bit grid; likewise the heavy class and the light items.
    const int64_t grid_cap = (int64_t)INT32_MAX / std::max(1, feat_len / 32);
    int64_t k = 0;
    while (k < n_rows && k < grid_cap && degree_at(k) > p->giant_threshold) p->giant_nnz += degree_at(k++);
    p->n_giant = (int)k;
    while (k < n_rows && degree_at(k) > p->heavy_threshold) p->heavy_nnz += degree_at(k++);
    p->n_heavy = (int)(k - p->n_giant);
    p->n_light = (int)(n_rows - k);
    if ((int64_t)p->n_heavy * (feat_len / 32) >= INT32_MAX ||
        (int64_t)p->n_light * (feat_len / 32) >= INT32_MAX) {
      plan_release(p);
      return fail(FG_ERR_UNSUPPORTED, "too many (row, slab) items for one launch");
    }

    FG_PLAN_TRY(cudaMalloc(&p->rows_dev, sizeof(int32_t) * (size_t)n_rows));
    FG_PLAN_TRY(cudaMemcpy(p->rows_dev, order.data(), sizeof(int32_t) * (size_t)n_rows,
                           cudaMemcpyHostToDevice));
    if (p->n_giant > 0) {
      FG_PLAN_TRY(cudaMalloc(&p->status_dev, sizeof(int)));
      FG_PLAN_TRY(cudaMemset(p->status_dev, 0, sizeof(int)));
    }
  }
#undef FG_PLAN_TRY
  *out_plan = p;
  return FG_OK;
}

}  // namespace fg

extern "C" int fg_spmm_plan_create(const int32_t* indptr, int64_t n_rows, int64_t n_cols,
                                   int32_t feat_len, int32_t device, int32_t heavy_threshold,
                                   fg_spmm_plan** out_plan) {
  if (indptr && indptr[0] != 0) return fg::fail(FG_ERR_INVALID_ARGUMENT, "indptr[0] must be 0");
  // the host-side containers may throw; the C ABI never does
  try {
    return fg::plan_create(indptr, n_rows, n_cols, feat_len, device, heavy_threshold, out_plan);
  } catch (const std::bad_alloc&) {
    return fg::fail(FG_ERR_OUT_OF_MEMORY, "fg_spmm_plan_create: host allocation failed");
  } catch (...) {
    return fg::fail(FG_ERR_CUDA, "fg_spmm_plan_create: unexpected exception");
  }
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
  if (v != 0) {
    // reported once: the word is cleared so that later calls are judged on their own
    FG_CUDA_TRY(cudaMemset(p->status_dev, 0, sizeof(int)));
    return fail(FG_ERR_CUDA, "spmm_chain_kernel: a bounded wait gave up (code %d: %s warp); "
                "the rows it was summing hold NaN", v,
                v == kGtErrProducerTimeout ? "producer" : "consumer");
  }
  return FG_OK;
}

extern "C" int fg_spmm_plan_set_poll_limit(fg_spmm_plan* p, int64_t polls) {
  using namespace fg;
  if (!p) return fail(FG_ERR_INVALID_ARGUMENT, "plan is null");
  p->poll_limit = polls < 0 ? kGtMaxPolls : (unsigned)std::min<int64_t>(polls, kGtMaxPolls);
  return FG_OK;
}

extern "C" int fg_spmm_plan_num_launches(const fg_spmm_plan* p) {
  if (!p || p->n_rows == 0) return 0;
  if (!p->vector_ok) return 1;
  const int trios = p->feat_len / p->slab_w;
  return trios * ((p->n_giant > 0 ? 1 : 0) + (p->n_heavy > 0 ? 1 : 0) + (p->n_light > 0 ? 1 : 0));
}

extern "C" int fg_spmm_plan_describe(const fg_spmm_plan* p, char* buf, int64_t buf_len) {
  using namespace fg;
  if (!p || !buf || buf_len <= 0) return fail(FG_ERR_INVALID_ARGUMENT, "null plan or buffer");
  if (p->vector_ok) {
    const int G = p->slab_w / 4;
    // grids of ONE trio: the kernels run once per residency slab of the features
    const int width = p->slab_w;
    const int hv_slabs = width / (32 * p->heavy_vec);
    const long long light_items = (long long)p->n_light * (width / p->slab_w);
    snprintf(buf, (size_t)buf_len,
             "spmm_csr_f32 rows=%lld cols=%lld nnz=%lld feat_len=%d max_deg=%lld | L2=%d B "
             "slab_w=%d | light: %d rows (deg<=%d) -> spmm_light_kernel<G=%d> grid=%lld x 256 thr | "
             "heavy: %d rows (deg<=%d), %lld nnz -> spmm_heavy_kernel<VEC=%d> grid=%lld x 32 thr, "
             "%d-stage cp.async ring | giant: %d rows, %lld nnz -> "
             "spmm_chain_kernel grid=%lld x %d thr (%d producer warps + 1 consumer, "
             "%d-block ring of products, flag words); %d slab(s) one after the other, each: "
             "giant, heavy, light, chained by programmatic dependent launches",
             (long long)p->n_rows, (long long)p->n_cols, (long long)p->nnz, p->feat_len,
             (long long)p->max_deg, p->l2_bytes, p->slab_w, p->n_light, p->heavy_threshold, G,
             (light_items + 256 / G - 1) / (256 / G), p->n_heavy, p->giant_threshold,
             (long long)p->heavy_nnz, p->heavy_vec, (long long)p->n_heavy * hv_slabs, kHvXSlots,
             p->n_giant, (long long)p->giant_nnz, (long long)p->n_giant * (width / 32),
             32 * GiantShape::WARPS, GiantShape::PRODUCERS, GiantShape::RING, p->feat_len / width);
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

// Raises the dynamic shared-memory limit of one kernel instantiation, once per device
// (and host thread).
template <auto Kernel>
static cudaError_t ensure_smem(int bytes, int device) {
  static thread_local int configured_dev = -1;
  if (configured_dev == device) return cudaSuccess;
  const cudaError_t e =
      cudaFuncSetAttribute(Kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess) configured_dev = device;
  return e;
}

// One kernel launch; `programmatic`: the kernel may be dispatched as soon as every CTA of
// the kernel before it in the stream has let its dependents go (launch_dependents()),
// instead of when that kernel has completed.
template <typename... Params, typename... Args>
static cudaError_t launch_kernel(void (*kernel)(Params...), unsigned grid, unsigned block,
                                 size_t smem, cudaStream_t st, bool programmatic, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = programmatic ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<Params>(args)...);
}

// Launches the group-per-row kernel over `n_listed` rows of the plan's list from `first`.
template <int G, int U, int MSG, int RED>
static cudaError_t launch_light(const fg_spmm_plan* p, const int32_t* indptr,
                                const int32_t* indices, const float* vals, const float* x,
                                const OutPtrs& y, int first, int n_listed, int width,
                                cudaStream_t st, bool programmatic) {
  const long long items = (long long)n_listed * (width / (4 * G));
  const long long grid = (items + 256 / G - 1) / (256 / G);
  return launch_kernel(spmm_light_kernel<G, U, MSG, RED>, (unsigned)grid, 256, 0, st, programmatic,
                       indptr, indices, vals, x, y, p->rows_dev + first, n_listed, items,
                       p->feat_len);
}

template <class Shape, int MSG, int RED>
static cudaError_t launch_chain(const fg_spmm_plan* p, const int32_t* indptr,
                                const int32_t* indices, const float* vals, const float* x,
                                const OutPtrs& y, int first, int n_listed, int width,
                                cudaStream_t st, bool programmatic) {
  const cudaError_t e =
      ensure_smem<spmm_chain_kernel<Shape, MSG, RED>>(Shape::SMEM_BYTES, p->device);
  if (e != cudaSuccess) return e;
  // one CTA per (row, 32-float slab)
  const unsigned grid = (unsigned)(n_listed * (width / 32));
  return launch_kernel(spmm_chain_kernel<Shape, MSG, RED>, grid, 32 * Shape::WARPS,
                       Shape::SMEM_BYTES, st, programmatic, indptr, indices, vals, x, y,
                       p->rows_dev + first, n_listed, p->slab_w / 32, p->feat_len, p->status_dev,
                       p->poll_limit);
}

template <int VEC, int MSG, int RED>
static cudaError_t launch_heavy(const fg_spmm_plan* p, const int32_t* indptr,
                                const int32_t* indices, const float* vals, const float* x,
                                const OutPtrs& y, int width, cudaStream_t st,
                                bool programmatic) {
  const cudaError_t e =
      ensure_smem<spmm_heavy_kernel<VEC, MSG, RED>>(heavy_smem_bytes<VEC>(), p->device);
  if (e != cudaSuccess) return e;
  const int slab = 32 * VEC;
  const long long items = (long long)p->n_heavy * (width / slab);  // < INT32_MAX (plan)
  return launch_kernel(spmm_heavy_kernel<VEC, MSG, RED>, (unsigned)items, 32,
                       heavy_smem_bytes<VEC>(), st, programmatic, indptr, indices, vals, x, y,
                       p->rows_dev + p->n_giant, p->n_heavy, p->slab_w / slab, p->feat_len);
}

// All kernels of one call for one operator pair.
template <int MSG, int RED>
static int spmm_launch_ops(const fg_spmm_plan* p, const int32_t* indptr, const int32_t* indices,
                           const float* vals, const float* x, const OutPtrs& y, bool aligned,
                           cudaStream_t st, const LaunchOptions& opt) {
  // `any`: the next launch of this call may be programmatic -- because the call itself is
  // (the caller's assertion), or because a kernel of this call is already in the stream
  bool any = (opt.flags & FG_LAUNCH_PROGRAMMATIC) != 0;
  // which row classes this call serves (the cuts of fg_launch_flags)
  const bool giants = (opt.flags & (FG_SPMM_SKIP_GIANT_ROWS | FG_SPMM_SKIP_LONG_ROWS)) == 0;
  const bool heavies = (opt.flags & (FG_SPMM_GIANT_ROWS_ONLY | FG_SPMM_SKIP_LONG_ROWS)) == 0;
  const bool rest = (opt.flags & (FG_SPMM_GIANT_ROWS_ONLY | FG_SPMM_LONG_ROWS_ONLY)) == 0;
  if (!p->vector_ok || !aligned) {  // no row classes here: the whole SpMM is "the rest"
    if (!rest) return FG_OK;
    const long long grid = (p->n_rows + 7) / 8;
    FG_CUDA_TRY(launch_kernel(spmm_generic_kernel<MSG, RED>, (unsigned)grid, 256, 0, st, any, indptr,
                              indices, vals, x, y, (long long)p->n_rows, p->feat_len));
    return FG_OK;
  }

  // One stream, longest rows first: giant kernel, heavy kernel, light kernel, each
  // dispatched as soon as every CTA of the one before it is resident (programmatic
  // dependent launch) -- not when it has completed; the three write disjoint rows.  A
  // giant CTA needs a whole SM, so it must get there before the light kernel's CTAs do:
  // once they are on an SM the block scheduler keeps backfilling it with them and the
  // giant rows, the call's critical path, start when the light kernel is nearly done.
  // (Measured with the three kernels on three streams and fork / join events instead:
  // 2.02 or 2.45 ms per call, depending on which launch reached the GPU first; this
  // way 1.875 ms, every time.)  The last CTA of every kernel waits for the grids before
  // it, so whatever follows in the stream sees the whole SpMM complete.
  //
  // One such trio per residency slab, one after the other: the three kernels of a trio then
  // gather from the SAME slab of X.  In one launch over all slabs each kernel walks the
  // slabs at its own pace, two or three slabs are live at a time, and together they no
  // longer fit L2.
  const int width = p->slab_w;
  for (int f0 = 0; f0 < p->feat_len; f0 += width) {
    // a trio starts when the one before it has COMPLETED (an ordinary launch): dispatched
    // behind it programmatically, its giant CTAs trickle onto the SMs that the light
    // kernel's tail frees while its other kernels wait for them -- 17.4 against 15.3 ms at
    // feat_len 512
    if (f0 > 0) any = false;
    const float* xs = x + f0;
    OutPtrs ys = y;
    for (int q = 0; q < ys.n; ++q) ys.p[q] += f0;
    if (giants && p->n_giant > 0) {
      FG_CUDA_TRY((launch_chain<GiantShape, MSG, RED>(p, indptr, indices, vals, xs, ys, 0,
                                                      p->n_giant, width, st, any)));
      any = true;
    }
    if (heavies && p->n_heavy > 0) {
      FG_CUDA_TRY((p->heavy_vec == 2
                       ? launch_heavy<2, MSG, RED>(p, indptr, indices, vals, xs, ys, width, st, any)
                       : launch_heavy<1, MSG, RED>(p, indptr, indices, vals, xs, ys, width, st, any)));
      any = true;
    }
    if (rest && p->n_light > 0) {
      const int first = p->n_giant + p->n_heavy;
      cudaError_t e;
      switch (p->slab_w) {
        case 128: e = launch_light<32, 8, MSG, RED>(p, indptr, indices, vals, xs, ys, first, p->n_light, width, st, any); break;
        case 64: e = launch_light<16, 8, MSG, RED>(p, indptr, indices, vals, xs, ys, first, p->n_light, width, st, any); break;
        default: e = launch_light<8, 8, MSG, RED>(p, indptr, indices, vals, xs, ys, first, p->n_light, width, st, any); break;
      }
      FG_CUDA_TRY(e);
      any = true;
    }
  }
  return FG_OK;
}

}  // namespace fg

static int spmm_launch(const fg_spmm_plan* p, const int32_t* indptr, const int32_t* indices,
                       const float* vals, const float* x, float* const* ys, int32_t n_ys,
                       int mcast, void* stream, int32_t msg_op = FG_MSG_MUL,
                       int32_t reduce_op = FG_REDUCE_SUM, int accumulate = 0) {
  using namespace fg;
  const LaunchOptions opt = take_launch_options();
  if (!p) return fail(FG_ERR_INVALID_ARGUMENT, "plan is null");
  if (!ys || n_ys < 1 || n_ys > kMaxOutputs)
    return fail(FG_ERR_INVALID_ARGUMENT, "need 1 to %d output pointers, got %d", kMaxOutputs,
                (int)n_ys);
  if (msg_op < FG_MSG_MUL || msg_op > FG_MSG_COPY_RHS || reduce_op < FG_REDUCE_SUM ||
      reduce_op > FG_REDUCE_MIN)
    return fail(FG_ERR_INVALID_ARGUMENT, "unknown msg_op %d or reduce_op %d", (int)msg_op,
                (int)reduce_op);
  if (p->n_rows == 0) return FG_OK;
  OutPtrs y;
  y.n = n_ys;
  y.mcast = mcast;
  y.accumulate = accumulate;
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
  int rc = FG_OK;
#define FG_SPMM_OPS(M, R) \
  rc = spmm_launch_ops<M, R>(p, indptr, indices, vals, x, y, aligned, st, opt)
  FG_DISPATCH_OPS(msg_op, reduce_op, FG_SPMM_OPS);
#undef FG_SPMM_OPS
  return rc;
}

extern "C" int fg_spmm_csr_f32_general(const fg_spmm_plan* p, const int32_t* indptr,
                                       const int32_t* indices, const float* vals,
                                       const float* x, float* y, int32_t msg_op,
                                       int32_t reduce_op, void* stream) {
  if (p && p->n_rows > 0 && !y) return fg::fail(FG_ERR_INVALID_ARGUMENT, "y_dev is null");
  float* ys[1] = {y};
  return spmm_launch(p, indptr, indices, vals, x, ys, 1, 0, stream, msg_op, reduce_op);
}

extern "C" int fg_spmm_csr_f32_multi(const fg_spmm_plan* p, const int32_t* indptr,
                                     const int32_t* indices, const float* vals, const float* x,
                                     float* const* ys, int32_t n_ys, void* stream) {
  return spmm_launch(p, indptr, indices, vals, x, ys, n_ys, 0, stream);
}

extern "C" int fg_spmm_csr_f32_mcast(const fg_spmm_plan* p, const int32_t* indptr,
                                     const int32_t* indices, const float* vals, const float* x,
                                     float* y_mcast, void* stream) {
  if (p && p->n_rows > 0 && !y_mcast)
    return fg::fail(FG_ERR_INVALID_ARGUMENT, "y_mcast_dev is null");
  float* ys[1] = {y_mcast};
  return spmm_launch(p, indptr, indices, vals, x, ys, 1, 1, stream);
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

// ------------------------------------------------- SpMM over column blocks (DDS) --
//
// The reference's 1-D source-vertex partitioning (vanilla_spmm_dds_x86,
// python/featgraph/op/vanilla_spmm.py:149-246): the columns are cut into P blocks, block p
// is a CSR matrix of its own over block-local column indices, and
//   Out[row] = ((0 + S_0[row]) + S_1[row]) + ... ,   S_p[row] = the block's sum in stored order.
// Here block p IS a CSR SpMM -- the same kernels, row pointers s1_pos + p * (n_rows + 1),
// features X + p * width * feat_len -- whose stores add to the output instead of replacing
// it (OutPtrs::accumulate).  The P calls follow each other in the stream, so block p + 1
// gathers only from its own width * feat_len * 4 bytes of X: the partitioning's purpose,
// features that stay in cache, with the 126 MB L2 in the role of the CPU's LLC.

struct fg_spmm_dds_plan {
  int device = 0, feat_len = 0, parts = 0;
  int64_t n_rows = 0, n_cols = 0, width = 0;
  std::vector<fg_spmm_plan*> blocks;
};

extern "C" int fg_spmm_dds_plan_destroy(fg_spmm_dds_plan* plan) {
  if (!plan) return FG_OK;
  for (fg_spmm_plan* b : plan->blocks) fg::plan_release(b);
  delete plan;
  return FG_OK;
}

extern "C" int fg_spmm_dds_plan_create(const int32_t* s1_pos, int64_t n_rows, int64_t n_cols,
                                       int32_t feat_len, int32_t num_col_partitions,
                                       int32_t device, fg_spmm_dds_plan** out_plan) {
  using namespace fg;
  if (!out_plan) return fail(FG_ERR_INVALID_ARGUMENT, "out_plan is null");
  *out_plan = nullptr;
  if (num_col_partitions < 1)
    return fail(FG_ERR_INVALID_ARGUMENT, "num_col_partitions must be at least 1, got %d",
                (int)num_col_partitions);
  if (!s1_pos) return fail(FG_ERR_INVALID_ARGUMENT, "s1_pos_host is null");
  if (n_rows < 0 || n_cols < 0) return fail(FG_ERR_INVALID_ARGUMENT, "bad shape");
  if (s1_pos[0] != 0) return fail(FG_ERR_INVALID_ARGUMENT, "s1_pos[0] must be 0");
  for (int64_t p = 1; p < num_col_partitions; ++p)
    if (s1_pos[p * (n_rows + 1)] != s1_pos[p * (n_rows + 1) - 1])
      return fail(FG_ERR_INVALID_ARGUMENT, "block %lld does not start where block %lld ends",
                  (long long)p, (long long)p - 1);
  try {
    fg_spmm_dds_plan* d = new fg_spmm_dds_plan();
    d->device = device;
    d->feat_len = feat_len;
    d->parts = num_col_partitions;
    d->n_rows = n_rows;
    d->n_cols = n_cols;
    d->width = std::max<int64_t>((n_cols + num_col_partitions - 1) / num_col_partitions, 1);
    for (int64_t p = 0; p < num_col_partitions; ++p) {
      fg_spmm_plan* b = nullptr;
      const int64_t cols = std::max<int64_t>(0, std::min(d->width, n_cols - p * d->width));
      const int rc = plan_create(s1_pos + p * (n_rows + 1), n_rows, cols, feat_len, device, 0, &b);
      if (rc != FG_OK) {
        fg_spmm_dds_plan_destroy(d);
        return rc;
      }
      d->blocks.push_back(b);
    }
    *out_plan = d;
    return FG_OK;
  } catch (const std::bad_alloc&) {
    return fail(FG_ERR_OUT_OF_MEMORY, "fg_spmm_dds_plan_create: host allocation failed");
  } catch (...) {
    return fail(FG_ERR_CUDA, "fg_spmm_dds_plan_create: unexpected exception");
  }
}

extern "C" int fg_spmm_dds_f32(const fg_spmm_dds_plan* d, const int32_t* s1_pos,
                               const int32_t* s1_idx, const float* vals, const float* x,
                               float* y, void* stream) {
  using namespace fg;
  take_launch_options();  // per-call options address the phases of one CSR call; none apply here
  if (!d) return fail(FG_ERR_INVALID_ARGUMENT, "plan is null");
  if (d->n_rows == 0) return FG_OK;
  if (!s1_pos || !y) return fail(FG_ERR_INVALID_ARGUMENT, "s1_pos_dev or y_dev is null");
  float* ys[1] = {y};
  for (int64_t p = 0; p < d->parts; ++p) {
    const int rc = spmm_launch(d->blocks[(size_t)p], s1_pos + p * (d->n_rows + 1), s1_idx, vals,
                               x ? x + (size_t)p * d->width * d->feat_len : x, ys, 1, 0, stream,
                               FG_MSG_MUL, FG_REDUCE_SUM, p == 0 ? 1 : 2);
    if (rc != FG_OK) return rc;
  }
  return FG_OK;
}

extern "C" int fg_spmm_dds_plan_status(const fg_spmm_dds_plan* d, int32_t* device_status) {
  using namespace fg;
  if (!d || !device_status) return fail(FG_ERR_INVALID_ARGUMENT, "plan or device_status is null");
  *device_status = 0;
  for (const fg_spmm_plan* b : d->blocks) {
    const int rc = fg_spmm_plan_status(b, device_status);
    if (rc != FG_OK) return rc;
  }
  return FG_OK;
}

extern "C" int fg_spmm_dds_plan_num_launches(const fg_spmm_dds_plan* d) {
  int n = 0;
  if (d)
    for (const fg_spmm_plan* b : d->blocks) n += fg_spmm_plan_num_launches(b);
  return n;
}
